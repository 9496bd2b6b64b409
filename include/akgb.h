/*
 * akgb.h — C ABI of the B200 fused-operator library.
 *
 * The library takes the MindSpore graph-kernel fused-op description (the
 * ".info" JSON that AKG-MLIR's `mindspore-translate` reads) and runs it on an
 * sm_100a device.  Every entry point below replaces one step of the
 * reference's GPU lowering + launch path; the reference interface it stands in
 * for is cited as <file within akg-mlir>:<line>.
 *
 * Conventions
 *   - plain C types only; tensors are bare pointers, dense row-major, offset 0
 *     (python/akg_mlir/mlir_driver.py:211-216, lib/Pipelines/GPUPipelines/GPUCodegen.cpp:50)
 *   - argument order of every tensor list: `input_desc` order, then
 *     `output_desc` order (lib/Target/MindsporeDialect/TranslateToMindsporeDialect.cpp:581-611)
 *   - every call returns an akgb_status; nothing here exits the process
 *     (the reference launcher calls exit(1) on a CUDA error,
 *     python/akg_mlir/utils/code_template.py:47-56)
 *   - there is no CPU fallback: a fused region the matcher cannot place on a
 *     kernel template yields AKGB_UNSUPPORTED.
 */
#ifndef AKGB_H_
#define AKGB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum akgb_status {
  AKGB_OK = 0,
  AKGB_INVALID_JSON = 1,   /* malformed text or a key the schema requires is missing */
  AKGB_UNSUPPORTED = 2,    /* valid description, but no kernel template covers it */
  AKGB_INVALID_ARG = 3,    /* null pointer, short buffer, bad option */
  AKGB_CUDA_ERROR = 4,     /* a CUDA runtime/driver call failed; see akgb_last_error() */
  AKGB_MISALIGNED = 5,     /* a tensor pointer is not 16-byte aligned */
  AKGB_DEVICE_TIMEOUT = 6, /* a bounded device-side wait gave up (error word set) */
  AKGB_TOO_LARGE = 7,      /* size beyond a fixed-capacity entry point's limit */
  AKGB_OUT_OF_RANGE = 8    /* a checked launch (AKGB_FLAG_CHECKED) reported an access outside its tensors */
} akgb_status;

/* Element types of the .info schema (TranslateToMindsporeDialect.cpp:488-502). */
typedef enum akgb_dtype {
  AKGB_BOOL = 0, AKGB_INT8 = 1, AKGB_INT16 = 2, AKGB_INT32 = 3, AKGB_INT64 = 4,
  AKGB_FLOAT16 = 5, AKGB_FLOAT32 = 6, AKGB_FLOAT64 = 7, AKGB_BFLOAT16 = 8
} akgb_dtype;

/* How a tensor argument relates to the leading-axis shard this kernel was
 * compiled for (see akgb_options.shard_world). */
typedef enum akgb_shard_kind {
  AKGB_REPLICATED = 0,   /* every rank passes the whole tensor */
  AKGB_SPLIT_AXIS0 = 1,  /* each rank passes its contiguous slice of axis 0 */
  AKGB_PARTIAL_SUM = 2,  /* output holds a per-rank partial: all-reduce(sum) it */
  AKGB_PARTIAL_MAX = 3,  /* all-reduce(max) */
  AKGB_PARTIAL_MIN = 4,  /* all-reduce(min) */
  AKGB_PARTIAL_PROD = 5  /* all-reduce(prod) */
} akgb_shard_kind;

#define AKGB_MAX_RANK 8

typedef struct akgb_tensor_desc {
  char name[64];
  int32_t dtype;                 /* akgb_dtype */
  int32_t rank;
  int64_t shape[AKGB_MAX_RANK];  /* the LOCAL shape (after sharding) */
  int64_t nbytes;                /* local size in bytes */
  int32_t is_output;
  int32_t shard_kind;            /* akgb_shard_kind */
  int32_t written_in_place;      /* an INPUT that an Assign/InplaceAssign of the region stores into; the reference
                                    harness treats such inputs as extra outputs
                                    (python/akg_mlir/utils/composite_op_helper.py:791-805) */
  int32_t reserved;
} akgb_tensor_desc;

typedef struct akgb_options {
  int32_t struct_size;  /* sizeof(akgb_options); lets the struct grow */
  int32_t device;       /* CUDA device ordinal; -1 = current device */
  int32_t shard_rank;   /* this rank's index in the leading-axis split */
  int32_t shard_world;  /* number of ranks the leading axis is split over; 0/1 = no split */
  int32_t flags;        /* bit set of AKGB_FLAG_* */
} akgb_options;

/* Run generic elementwise groups with the interpreting kernel only, never the run-time instantiated
 * (NVRTC-compiled) variant of the same template.  Results are identical; this is for hosts without NVRTC
 * and for tests. */
#define AKGB_FLAG_NO_JIT 1
/* Fold the per-CTA partials of column / all-element reductions by the last CTA of the launch that produced them
 * instead of in a second, small launch.  Results are identical bit for bit.  Measured on B200 the second launch is the
 * faster of the two (the in-launch fold ends the kernel with a chain of dependent global-memory round trips: store
 * acknowledged, arrival counter, partials read back -- about 6 us, against about 2 us for a dependent launch inside a
 * CUDA graph), so this is off by default; a sharded reduction that completes its exchange in its own launch
 * (akgb_launch_sharded) folds in-launch regardless. */
#define AKGB_FLAG_FOLD_IN_LAUNCH 2
/* Reduce-X regions whose rows do not fit the register file (above about 16 384 elements) walk the row once per
 * reduction.  By default the passes after the first re-read the row through L2 (evict-last hints, alternating walk
 * direction).  With this flag the first pass keeps the row in shared memory instead -- across a thread-block cluster
 * of 2, 4 or 8 CTAs when it exceeds one CTA's share, the per-row reductions then completed through distributed shared
 * memory -- so the row crosses HBM/L2 once.  Identical results.  Measured on B200 the L2 schedule is the faster one
 * (log-softmax float32 [8192,32000]: 415 us against 523 us staged), which is why this is opt-in. */
#define AKGB_FLAG_STAGE_LONG_ROWS 4
/* Checked launches (memory-safety evidence where compute-sanitizer is not available): kernels generated at run time
 * are built with every access to global memory tested against the address ranges of the launch's tensors and
 * workspace.  An access outside all of them sets bit 9 (512) of the device error word (akgb_check_device_error) and is
 * skipped -- a load gives zeros; nothing asserts or traps.  The kernel templates built into the library are not
 * instrumented (their tests run with guard zones around every buffer instead).  Slower; for tests. */
#define AKGB_FLAG_CHECKED 8

typedef struct akgb_kernel akgb_kernel;

/* Parse + classify + match + plan.  Replaces `mindspore-translate`,
 * `akg-opt --gpu-opt`, `--gpu-codegen`, `akg-translate -gen-ptx` and
 * `akg-ptx-replace` (python/akg_mlir/mlir_driver.py:337-374).  Needs no GPU. */
akgb_status akgb_compile(const char* info_json, size_t len, const akgb_options* opt,
                         akgb_kernel** out);

/* Frees the plan and any staging memory the library allocated for it. */
void akgb_release(akgb_kernel* k);

/* Number of tensor arguments (inputs then outputs) and their descriptions. */
int32_t akgb_num_tensors(const akgb_kernel* k);
int32_t akgb_num_inputs(const akgb_kernel* k);
akgb_status akgb_tensor_info(const akgb_kernel* k, int32_t index, akgb_tensor_desc* out);

/* Bytes of device scratch a launch needs (partials of split reductions, values that cross launches).  For a region that
 * runs as a kernel generated at run time this is what that kernel needs; should the kernel fail to compile on the
 * host, akgb_launch returns AKGB_UNSUPPORTED with the larger size the separate launches would need, and the region can
 * be compiled with AKGB_FLAG_NO_JIT instead. */
size_t akgb_workspace_size(const akgb_kernel* k);

/* Number of device kernels one akgb_launch enqueues. */
int32_t akgb_launch_count(const akgb_kernel* k);

/* Enqueue the fused op on `stream` (a cudaStream_t, may be NULL).  `tensors`
 * are DEVICE pointers, inputs then outputs.  `workspace` must hold at least
 * akgb_workspace_size() bytes (may be NULL when that is 0).  Asynchronous.
 * Replaces cuLaunchKernel of the generated kernel
 * (python/akg_mlir/utils/code_template.py:204).
 * The calling thread's current CUDA device must be the one the kernel was compiled for (akgb_options.device):
 * otherwise AKGB_INVALID_ARG, nothing is launched.  The same holds for akgb_launch_dynamic, akgb_launch_sharded and
 * akgb_allreduce_partials; akgb_run_host, akgb_profile_host and akgb_prepare select the kernel's device themselves
 * and leave it current.  Launches of ONE kernel object must be ordered on the device (one stream, or events between
 * streams): the object owns small device-side arrival counters that its reductions share. */
akgb_status akgb_launch(akgb_kernel* k, void* const* tensors, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Does ahead of time what the first akgb_launch would do lazily on the kernel's device: uploads the library's device
 * tables and compiles (or loads from the on-disk cache) the kernels generated for this region.  Call it before
 * capturing launches into a CUDA graph -- compilation and module loading are not allowed during capture.  The
 * reference does all of this in compile_gpu (python/akg_mlir/mlir_driver.py:337-374), which needs no device. */
akgb_status akgb_prepare(akgb_kernel* k);

/* Dynamic-shape regions: descriptions whose extents contain -1 (the form MindSpore emits for unknown
 * dims; the reference handles them with its --gpu-dyn-opt pipeline and passes sizes and strides of every
 * tensor to the launcher, lib/Pipelines/GPUPipelines/GPUDynOpt.cpp:47-143,
 * python/akg_mlir/utils/gen_runtime_code.py:39-58).  akgb_compile parses and classifies them; the kernel
 * templates are chosen when the extents are known.  `shapes` lists, for every argument in order (inputs
 * then outputs), all of its extents; `count` is their total number.  Plans are cached per set of extents.
 * akgb_bind_shapes reports the workspace a launch with these extents needs. */
akgb_status akgb_bind_shapes(akgb_kernel* k, const int64_t* shapes, size_t count, size_t* workspace_bytes);
akgb_status akgb_launch_dynamic(akgb_kernel* k, void* const* tensors, const int64_t* shapes, size_t count,
                                void* workspace, size_t workspace_bytes, void* stream);

/* Same contract as the generated launcher's `cuda_runtime_exec`
 * (python/akg_mlir/utils/code_template.py:160-211): `host_tensors` are HOST
 * pointers, inputs then outputs; inputs are copied to the device, the fused op
 * runs, outputs are copied back; synchronous.  Device staging buffers are kept
 * in the kernel object between calls instead of being re-allocated. */
akgb_status akgb_run_host(akgb_kernel* k, void* const* host_tensors);

/* Same contract as `cuda_runtime_profiling`
 * (python/akg_mlir/utils/code_template.py:68-157): one warm-up, then
 * `number * repeat` launches; writes the average device time of one launch in
 * microseconds (CUDA events, not the reference's host clock). */
akgb_status akgb_profile_host(akgb_kernel* k, void* const* host_tensors, int32_t number,
                              int32_t repeat, double* avg_us);

/* The launch metadata the reference writes to <kernel>.json
 * (lib/Dialect/GPU/Transforms/GPUMapping.cpp:645-703,
 * python/akg_mlir/mlir_driver.py:776-815): blockIdx.{x,y,z}, threadIdx.{x,y,z},
 * kernelName, is_dynamic, sha256 — plus class, template, bytes, flops, smem,
 * workspace, launches and "steps" (the kernel family of every step of the
 * plan, in launch order).  Writes a NUL-terminated JSON text; `*needed` receives the size including the NUL. */
akgb_status akgb_kernel_meta(const akgb_kernel* k, char* buf, size_t cap, size_t* needed);

/* Writes <dir>/<kernel>.cubin and <dir>/<kernel>.json for a region that runs as ONE kernel generated at run time
 * (elementwise / broadcast chains, reduce-X regions without sums over all rows): the artefact pair the reference
 * leaves under KERNEL_META_DIR for the framework's own runtime (<kernel>.ptx + <kernel>.json,
 * python/akg_mlir/mlir_driver.py:47-53, 776-815).  The image's entry point "<kernel>_kernel" takes the device pointers
 * of the inputs, then of the outputs, and nothing else (extents are compiled in); the JSON carries kernelName,
 * blockIdx.{x,y,z}, threadIdx.{x,y,z}, is_dynamic, the sha256 of the image, and the pointer alignment the image
 * assumes.  Needs the run-time compiler but no device.  Regions that run on the templates built into the library, in
 * several launches, or with dynamic shapes have no such binary: AKGB_UNSUPPORTED. */
akgb_status akgb_export_kernel(const akgb_kernel* k, const char* dir);

/* The CUDA C++ text that is compiled at run time for the first generic elementwise group of the region
 * (`vectorised` != 0: the 16-byte-vector variant, else the scalar one); an empty text means the region has
 * no such group or it runs on the interpreting kernel.  The counterpart of the reference's IR/PTX dumps
 * (AKG_DUMP_IR, python/akg_mlir/mlir_driver.py:711-721). */
akgb_status akgb_dump_jit_source(const akgb_kernel* k, int32_t vectorised, char* buf, size_t cap, size_t* needed);

/* ---- multi-GPU: the exchange step of a sharded kernel --------------------------------------------------------
 * A kernel compiled with akgb_options.shard_world > 1 computes on its rank's slice of the leading axis; outputs whose
 * shard_kind is AKGB_PARTIAL_* hold per-rank partials that one all-reduce completes.  The reference runs a fused
 * operator on one device only (python/akg_mlir/utils/code_template.py:181); these entry points have no counterpart
 * there.  NCCL is loaded at run time (the copy already in the process, else the system's libnccl.so.2). */
typedef struct akgb_comm akgb_comm;
#define AKGB_COMM_ID_BYTES 128

/* Rank 0 creates the rendezvous id and hands its AKGB_COMM_ID_BYTES bytes to the other ranks by any means. */
akgb_status akgb_comm_unique_id(void* id, size_t cap);
/* Collective over all `world` ranks (one process per GPU); `device` < 0 keeps the current device. */
akgb_status akgb_comm_create(const void* id, int32_t rank, int32_t world, int32_t device, akgb_comm** out);
/* Uses a communicator the caller already has (an ncclComm_t); it is not destroyed by akgb_comm_destroy. */
akgb_status akgb_comm_wrap(void* nccl_comm, int32_t rank, int32_t world, akgb_comm** out);
void akgb_comm_destroy(akgb_comm* c);
/* Optional faster exchange for small float32 partials (up to 16 384 elements, up to 8 ranks on one box): every rank
 * exports a handle of its exchange buffer, the caller gathers the handles of all ranks (rank order) and hands them to
 * every rank; from then on akgb_allreduce_partials uses one kernel over the mapped buffers (peer stores over NVLink, a
 * flag per rank, a fold in rank order) instead of NCCL for such tensors.  The wait for the other ranks is bounded
 * (akgb_comm_set_timeout_ms, default 1000): on expiry bit 8 of the device error word is set (akgb_check_device_error),
 * the output is left as it was and the context stays usable.  `handles` == NULL attaches the rank's own buffer for every
 * rank (single-rank use).  If a peer's buffer cannot be mapped the call fails and NCCL keeps carrying the exchange. */
#define AKGB_COMM_HANDLE_BYTES 64
/* A communicator without NCCL (1..8 ranks of one box): only the peer-memory exchange below is available; a partial it
 * cannot carry makes akgb_allreduce_partials return AKGB_UNSUPPORTED. */
akgb_status akgb_comm_create_local(int32_t rank, int32_t world, int32_t device, akgb_comm** out);
/* Turns the peer-memory exchange off (or on again once all buffers are attached): every rank must use the same path, so
 * a caller whose attach failed on some rank turns it off on all of them. */
akgb_status akgb_comm_set_peer_exchange(akgb_comm* c, int32_t enabled);
akgb_status akgb_comm_exchange_handle(akgb_comm* c, void* handle, size_t cap);
akgb_status akgb_comm_attach_peers(akgb_comm* c, const void* handles, size_t bytes);
akgb_status akgb_comm_set_timeout_ms(akgb_comm* c, double ms);
/* Whether a reduction that produces all partial outputs of a kernel completes the exchange inside its fold step
 * (see akgb_launch_sharded; the default) or leaves it to the exchange kernel / NCCL after the launch.  Every rank must choose the
 * same. */
akgb_status akgb_comm_set_exchange_in_reduction(akgb_comm* c, int32_t enabled);

/* All-reduces, in place and on `stream`, every tensor of `tensors` (inputs then outputs, device pointers) whose
 * shard_kind is a partial; one NCCL group for all of them.  No-op for kernels without partial outputs. */
akgb_status akgb_allreduce_partials(const akgb_kernel* k, akgb_comm* c, void* const* tensors, void* stream);
/* The kernel and the exchange of its partial outputs on one stream.  Where ONE reduction (column, all-elements, or both
 * in one pass) produces all partial outputs and the peers' buffers are attached, the reduction's fold step completes
 * the exchange (results of up to 8192 float32 elements): the CTA that folds a tile of the per-CTA partials stores each
 * value, tagged with the call number, into every rank's buffer as one 8-byte word, polls (bounded) the other ranks'
 * words and folds them in rank order -- two launches per rank and step (the reduction and its fold; one with
 * AKGB_FLAG_FOLD_IN_LAUNCH) instead of reduction, fold and exchange kernel.  Otherwise:
 * akgb_launch followed by akgb_allreduce_partials.  After a sharded step every rank should read akgb_check_device_error: once a bounded wait has
 * run out on a device (AKGB_DEVICE_TIMEOUT, bit 8), further peer-memory exchanges there are refused with
 * AKGB_DEVICE_TIMEOUT until akgb_comm_set_peer_exchange has been called on ALL ranks (1: restart the path, 0: continue
 * over NCCL) and the ranks have synchronised. */
akgb_status akgb_launch_sharded(akgb_kernel* k, akgb_comm* c, void* const* tensors, void* workspace,
                                size_t workspace_bytes, void* stream);
/* A region in which a reduction over the split axis feeds later ops (batch-norm statistics over a batch that is split
 * across the ranks) compiles, with shard_world > 1, into STAGES cut at those reductions (class "sharded_stages"):
 * akgb_launch_sharded runs stage, exchange, stage, ... on the one stream; results of such reductions are reported as
 * AKGB_REPLICATED because the caller receives them completed.  akgb_launch and akgb_run_host refuse such a kernel
 * (AKGB_INVALID_ARG): its stages cannot run without the exchange between them.
 *
 * Which way the partial outputs of `k` travel with communicator `c` as it is set up now (for a kernel made of stages:
 * the least direct way among its stages). */
#define AKGB_EXCHANGE_NONE 0          /* no partial outputs, or a single rank */
#define AKGB_EXCHANGE_NCCL 1          /* ncclAllReduce after the kernel */
#define AKGB_EXCHANGE_PEER_KERNEL 2   /* one exchange kernel over the ranks' mapped buffers after the kernel */
#define AKGB_EXCHANGE_IN_REDUCTION 3  /* inside the reduction's fold step (see akgb_launch_sharded) */
int32_t akgb_sharded_exchange_kind(const akgb_kernel* k, const akgb_comm* c);

/* Directory of the on-disk cache of run-time compiled kernels.  The reference keeps its compiled kernels
 * (<kernel>.ptx / .json) under KERNEL_META_DIR and reuses them by name (python/akg_mlir/mlir_driver.py:47-53,
 * 337-374); here every generated elementwise kernel is stored as
 * `<dir>/akgb_ew_<sha256 of the generated text and options>.sm_100a.cubin` and loaded from there by later
 * processes instead of being compiled again.  Without this call the directory is $AKGB_JIT_CACHE_DIR, else
 * $KERNEL_META_DIR, else there is no disk cache.  NULL returns to the environment's choice, "" disables. */
akgb_status akgb_set_cache_dir(const char* dir);

/* How many generated kernels this process compiled, and how many it loaded from the on-disk cache. */
akgb_status akgb_jit_cache_stats(uint64_t* compiled, uint64_t* loaded_from_disk);

/* Operator class the matcher assigned, as a static string
 * ("elementwise", "broadcast", "reduce_x", "reduce_y", "reduce_all",
 * "layernorm", "softmax", "transpose", "matmul", "generic"). */
const char* akgb_kernel_class(const akgb_kernel* k);

/* Algorithmic bytes (every input read once, every output written once) and
 * floating-point operations (2*M*N*K for matmul, else 0) of one launch. */
int64_t akgb_kernel_bytes(const akgb_kernel* k);
int64_t akgb_kernel_flops(const akgb_kernel* k);

/* For tests of the checker itself: take `bytes` off the end of every tensor range of subsequent checked launches of
 * this process (0 restores).  The accesses then reported and skipped lie inside the real tensors. */
void akgb_checked_shrink_for_test(int bytes);

/* Reads and clears the device-side error word of the last launches of `k`
 * (bounded waits that gave up).  0 = none. */
akgb_status akgb_check_device_error(akgb_kernel* k, uint32_t* word);

/* Column sum x[rows, cols] -> out[cols] (float32, device pointers, asynchronous on `stream`) that
 * allocates nothing: no cudaMalloc/cudaFree, no workspace argument.  It has no counterpart in the
 * reference; it exists for callers that cannot allocate device memory where they need the reduction
 * (inside a memory-planned region of a framework, while an allocator is exhausted or shutting down,
 * in a loop that cannot afford cudaMalloc's implicit synchronisation).  The partial sums live in a
 * 1 MiB array built into the library (resident on every GPU that loads it, until the process exits).
 *   - Limit: cols <= 65536 (any row count); wider inputs, or a device with so many SMs that the
 *     partials would not fit the 1 MiB, return AKGB_TOO_LARGE: use akgb_launch with a workspace.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call outside any stream capture.  The current device must be the one holding x/out.
 *   - All calls on a device share the array: issue them so that their kernels do not overlap on the
 *     GPU (same stream, or ordered by events).  No clearing is needed between calls.
 *   - The address found by the first call is kept per device ordinal for the life of the process; it
 *     does not survive cudaDeviceReset (do not call this entry point again after one).
 * Results are bit-identical to akgb_launch of the same ReduceSum(axis 0) description. */
akgb_status akgb_reduce_sum_axis0_f32_noalloc(const float* x, float* out, int64_t rows, int64_t cols, void* stream);

/* Text of the last error on the calling thread. */
const char* akgb_last_error(void);

/* Library version string. */
const char* akgb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* AKGB_H_ */
