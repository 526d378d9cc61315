/*
 * trifast_b200 — C ABI of the B200 (sm_100a) triangle self-attention kernels.
 *
 * This is the boundary a host binding attaches to: plain pointers, sizes and
 * element strides, no C++ or torch types.  It replaces the launch layer of the
 * reference (latkins/trifast), where Python code in src/trifast/torch.py
 * allocates the outputs and launches four Triton kernels; each entry point
 * below names the reference code it stands in for.
 *
 * Tensors (layout of src/trifast/torch.py:220-226 of the reference):
 *   q, k, v, o, dO, dq, dk, dv : (batch, heads, n_rows, n, d), innermost d contiguous
 *   bias, db                   : (batch, heads, n, n) = (b, h, j, k), innermost contiguous
 *   mask                       : (batch, n_rows, n) = (b, i, k), one byte per key,
 *                                non-zero = key k is masked OUT for pair row i
 *   lse, delta                 : (batch, heads, n_rows, n) fp32, contiguous
 * n_rows is the number of pair rows i held by this call: n for the whole
 * problem, fewer for a row shard (rows are independent except for db, which is
 * then a partial sum over the local rows).
 *
 * Ownership: the caller owns every buffer, including the workspace.  No entry
 * point allocates, frees or synchronises device memory unless its comment says
 * otherwise.  Outputs are fully overwritten.  All work is enqueued on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *
 * Errors: every function returns TRIFAST_OK (0) or a negative trifast_status;
 * nothing throws across this boundary.  trifast_status_str() names a code.
 */
#ifndef TRIFAST_B200_H_
#define TRIFAST_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum trifast_status {
  TRIFAST_OK = 0,
  TRIFAST_ERR_NULL = -1,          /* a required pointer is NULL */
  TRIFAST_ERR_SHAPE = -2,         /* non-positive extent, n_rows > n, ... */
  TRIFAST_ERR_HEAD_DIM = -3,      /* d is not one of 16, 32, 64, 128 */
  TRIFAST_ERR_DTYPE = -4,         /* unknown trifast_dtype */
  TRIFAST_ERR_STRIDE = -5,        /* negative stride / stride breaks 16-byte rule */
  TRIFAST_ERR_ALIGN = -6,         /* a base pointer is not 16-byte aligned */
  TRIFAST_ERR_WORKSPACE = -7,     /* workspace missing or too small */
  TRIFAST_ERR_ARCH = -8,          /* device is not compute capability 10.x */
  TRIFAST_ERR_LAUNCH = -9,        /* CUDA reported an error at launch */
  TRIFAST_ERR_KERNEL_CHOICE = -10,/* forced kernel cannot run this problem */
  TRIFAST_ERR_DEVICE_TIMEOUT = -11,/* a bounded wait inside a kernel gave up */
  TRIFAST_ERR_TOO_LARGE = -12     /* size beyond a stated maximum */
} trifast_status;

typedef enum trifast_dtype {
  TRIFAST_F32 = 0,
  TRIFAST_BF16 = 1,
  TRIFAST_F16 = 2
} trifast_dtype;

/* Which kernel family runs.  AUTO applies the fixed heuristic keyed on
 * (n, h, d, dtype) that replaces the reference's benchmark-and-cache autotuner
 * (src/trifast/autotune.py:28-156, config lists autotune_helpers.py:58-211). */
typedef enum trifast_kernel {
  TRIFAST_KERNEL_AUTO = 0,
  TRIFAST_KERNEL_SIMT = 1,   /* fp32-accumulate CUDA-core kernels: any dtype, any n */
  TRIFAST_KERNEL_TCGEN05 = 2 /* tcgen05 / TMEM / TMA kernels: bf16 and fp16 */
} trifast_kernel;

/* Debug overrides of the heuristic (trifast_shape.flags).  They stand in for the
 * reference's TRIFAST_FORCE_TUNE switch (src/trifast/autotune_helpers.py:12-14):
 * a way to make a non-default kernel run, for A/B measurements and tests. */
typedef enum trifast_flags {
  TRIFAST_FLAG_SPLIT_BWD = 1, /* dq and dk/dv as two kernels even where the one-pass kernel fits */
  /* Not a debug switch: set by row-sharded callers.  trifast_backward_dqkv then leaves 8 SMs
   * free, so that the all-reduce of db launched beside it (another stream) finds room to run
   * at once instead of after it.  (No reference counterpart: the reference is single-GPU.) */
  TRIFAST_FLAG_SHARE_GPU = 2
} trifast_flags;
/* With TRIFAST_FLAG_SHARE_GPU, bits 8-15 of `flags` hold the number of SMs to leave free
 * (0 = 8): as many as the collective beside the kernel has CTAs that must run at once. */
#define TRIFAST_FLAG_SHARE_SMS(sms) (((sms) & 0xff) << 8)

/* Problem extents, shared by every call. */
typedef struct trifast_shape {
  int32_t batch;
  int32_t heads;
  int32_t n;       /* keys per row = queries per row */
  int32_t n_rows;  /* pair rows i in this call (<= n) */
  int32_t d;       /* head dim: 16, 32, 64 or 128 */
  int32_t dtype;   /* trifast_dtype of q, k, v, bias, o and the gradients */
  int32_t kernel;  /* trifast_kernel; 0 = heuristic */
  int32_t flags;   /* OR of trifast_flags; 0 = the heuristic decides everything */
} trifast_shape;

/* (b, h, i, j, d) tensor: strides in elements for b, h, i, j; d has stride 1. */
typedef struct trifast_t5 {
  void* data;
  int64_t stride[4];
} trifast_t5;

/* (b, h, j, k) tensor: strides in elements for b, h, j; k has stride 1. */
typedef struct trifast_t4 {
  void* data;
  int64_t stride[3];
} trifast_t4;

/* (b, i, k) byte mask: strides in bytes for b, i; k has stride 1. */
typedef struct trifast_mask {
  const uint8_t* data;
  int64_t stride[2];
} trifast_mask;

/* Tile plan chosen by the heuristic (host only; no device needed). */
typedef struct trifast_plan {
  int32_t kernel;        /* trifast_kernel actually used (by the backward, when the two differ) */
  int32_t block_j;       /* query tile */
  int32_t block_k;       /* key tile */
  int32_t rows_per_cta;  /* pair rows sharing one bias tile in the forward */
  int32_t stages;        /* K/V/bias pipeline depth */
  int32_t db_row_splits; /* row groups whose db partials are summed in fixed order */
  int32_t bwd_fused;     /* 1: dq, dk, dv come from one kernel (one exponential per score) */
  int32_t bwd_chunks;    /* query chunks a row is walked in by that kernel (1: dQ of a row fits TMEM) */
  int32_t fwd_kernel;    /* trifast_kernel of the forward: differs from `kernel` for head dim 128,
                            whose forward has tensor-core tiles and whose backward has not */
} trifast_plan;

/* Library version as major*10000 + minor*100 + patch. */
int trifast_version(void);

/* Text for a status code (static storage). */
const char* trifast_status_str(int status);

/* Name of the CUDA error behind the calling thread's most recent TRIFAST_ERR_LAUNCH
 * ("cudaSuccess" if there was none).  No reference counterpart: the reference raises
 * the CUDA error through PyTorch. */
const char* trifast_last_cuda_error(void);

/* Fixed tile heuristic.  Stands in for Autotuner.run of the reference
 * (src/trifast/autotune.py:110-156): same key (n, h, d, dtype), but a table
 * instead of benchmarking and an on-disk cache.  Pure host code. */
int trifast_pick_plan(const trifast_shape* shape, trifast_plan* plan);

/* Bytes of caller-provided workspace the backward needs (delta, packed masks, fp32
 * db and its row-split partials, bias copies).  Returns 0 on an invalid shape. */
size_t trifast_backward_workspace_bytes(const trifast_shape* shape);

/* Bytes of workspace the forward needs: 0 on the CUDA-core plan.  On the tensor-core
 * plan: one word per pair row (the range of 128-key tiles that hold an open key; tiles
 * outside it are not walked), and for n % 8 != 0 also a copy of the bias with a 16-byte
 * row pitch and the key mask as packed words (all made inside trifast_forward). */
size_t trifast_forward_workspace_bytes(const trifast_shape* shape);

/* Forward: o = softmax_k(q.k^T * d^-0.5 + bias + mask) v and lse (natural log).
 * Stands in for _triangle_attention + the _fwd kernel of the reference
 * (src/trifast/torch.py:17-65, src/trifast/triton.py:14-132).
 * Rows whose keys are all masked get uniform weights 1/n over all n keys, as
 * the reference's PyTorch path does (src/trifast/equiv.py:42-69); their lse is
 * stored as finfo(dtype).min.  `workspace` holds at least
 * trifast_forward_workspace_bytes() bytes (NULL is fine when that is 0). */
int trifast_forward(const trifast_shape* shape,
                    const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
                    const trifast_t4* bias, const trifast_mask* mask,
                    const trifast_t5* o, float* lse,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Whole backward on one device: dq, dk, dv and db (db in the input dtype).
 * Stands in for triangle_attention_bwd and its three kernels
 * (src/trifast/torch.py:68-182; triton.py:268-383 _bwd_q, :137-263 _bwd_kv,
 * :388-501 _bwd_b).  `workspace` holds at least
 * trifast_backward_workspace_bytes() bytes.  db is reduced over rows in a fixed
 * order (deterministic, no atomics). */
int trifast_backward(const trifast_shape* shape,
                     const trifast_t5* d_o,
                     const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
                     const trifast_t4* bias, const trifast_mask* mask,
                     const trifast_t5* o, const float* lse,
                     const trifast_t5* dq, const trifast_t5* dk, const trifast_t5* dv,
                     const trifast_t4* db,
                     void* workspace, size_t workspace_bytes, void* stream);

/* The backward in three steps, for row-sharded runs that overlap the
 * all-reduce of db with the rest of the backward.  The reference has no
 * multi-device path; these split triangle_attention_bwd
 * (src/trifast/torch.py:68-182) at the points where the exchange happens.
 *
 * 1. trifast_backward_db: delta = sum_d o*dO (kept fp32 inside the workspace)
 *    and the partial bias gradient over the local rows, written as fp32
 *    (batch, heads, n, n) contiguous into db_f32.
 * 2. (caller) all-reduce db_f32 across row shards on another stream.
 * 3. trifast_backward_dqkv: dq, dk, dv; reads the delta step 1 left in the
 *    same workspace.
 * 4. trifast_db_finalize: round the summed fp32 db to the input dtype. */
int trifast_backward_db(const trifast_shape* shape,
                        const trifast_t5* d_o,
                        const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
                        const trifast_t4* bias, const trifast_mask* mask,
                        const trifast_t5* o, const float* lse,
                        float* db_f32,
                        void* workspace, size_t workspace_bytes, void* stream);

int trifast_backward_dqkv(const trifast_shape* shape,
                          const trifast_t5* d_o,
                          const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
                          const trifast_t4* bias, const trifast_mask* mask,
                          const float* lse,
                          const trifast_t5* dq, const trifast_t5* dk, const trifast_t5* dv,
                          void* workspace, size_t workspace_bytes, void* stream);

int trifast_db_finalize(const trifast_shape* shape, const float* db_f32,
                        const trifast_t4* db, void* stream);

/* Sum of the fp32 db partials of the row shards of one box by plain stores to peer-mapped
 * memory, in place of the all-reduce of step 2 above (no collective library in the path,
 * cross-rank summation order fixed = rank order).  Every rank calls it once per step with
 * the same `epoch` (1, 2, 3, ...), at about the same time; rank r pushes slice s of its
 * partial into rank s's staging area, rank s adds the `world` staged slices in rank order
 * and pushes the reduced slice into every rank's result buffer.  When the kernel ends,
 * `result[rank]` holds the full sum.  The staging, result and flag areas of ALL ranks must be
 * mapped into this process (CUDA IPC / symmetric memory; peer access enabled) and are passed
 * as device pointers valid here; flags (16 words per rank) and counters (2 words, local) start
 * at zero and are never reset by the caller.  The ranks wait for each other inside the kernel
 * with a bounded wait (about 2 s): a rank that misses its peers sets the device status word
 * (trifast_check_device_status) and returns.  No reference counterpart: the reference is
 * single-GPU and holds no distributed code. */
typedef struct trifast_push_reduce {
  int32_t rank, world;      /* world <= 8 */
  int32_t ctas;             /* CTAs of 1024 threads to launch; 0 = 4.  They meet through a counter,
                               so all of them must find a free SM at once: pass no more than the
                               dq/dk/dv kernel beside them leaves free (TRIFAST_FLAG_SHARE_SMS) */
  uint32_t epoch;           /* same on every rank, +1 per call, never 0 */
  int64_t count;            /* fp32 elements of db */
  const float* partial;     /* this rank's partial sum (any local memory, 16-byte aligned) */
  uint32_t* counters;       /* this rank's 2 counter words (local) */
  float* staging[8];        /* rank r's staging area: trifast_db_push_reduce_staging_floats() floats */
  float* result[8];         /* rank r's result buffer: count floats */
  uint32_t* flags[8];       /* rank r's 16 flag words */
} trifast_push_reduce;

size_t trifast_db_push_reduce_staging_floats(int64_t count, int32_t world);

int trifast_db_push_reduce(const trifast_push_reduce* args, void* stream);

/* Copy of `blocks` equally spaced blocks of `block_bytes` bytes each between pinned host
 * memory and the device in one asynchronous 2-D transfer on `stream` (to_host != 0:
 * device -> host): block i is read at src + i * src_pitch and written at dst + i *
 * dst_pitch.  The host-resident pipeline moves the same pair rows of every (batch, head)
 * of a tensor with one such call instead of one copy per (batch, head), whose fixed
 * cost per transfer showed (4 MiB host-to-device copies reached 40 GB/s where 64 MiB ones
 * reach 55).  No reference counterpart: the reference takes device tensors only. */
int trifast_copy_blocks(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                        size_t block_bytes, size_t blocks, int to_host, void* stream);

/* Reads and clears the per-device status word that kernels set when one of
 * their bounded waits gives up.  Synchronises `stream` first.  Returns
 * TRIFAST_OK or TRIFAST_ERR_DEVICE_TIMEOUT.  (No reference counterpart: Triton
 * kernels have no such waits.) */
int trifast_check_device_status(void* stream);

/* Enqueues, on `stream`, a copy of the same status word into *host_word without
 * synchronising or clearing anything.  With host_word in pinned host memory a
 * binding can call this after each launch and look at the word at the start of its
 * next call: a non-zero value means some earlier kernel gave up on a wait (its
 * outputs are not valid), and trifast_check_device_status() then reads and clears
 * it.  This is how the Python operators turn a device-side timeout into an
 * exception without a synchronisation per call.  (No reference counterpart.) */
int trifast_snapshot_device_status(uint32_t* host_word, void* stream);

/* Test support for that path: launches one warp that waits, with the same bounded
 * wait the kernels use, on a barrier nobody arrives on; after limit_us
 * microseconds (1 .. 100000) the wait gives up, the kernel sets the status word
 * and exits normally.  Nothing traps, faults or spins beyond the limit.  (No
 * reference counterpart.) */
int trifast_debug_wait_probe(uint32_t limit_us, void* stream);

/* The whole backward (same results as trifast_backward) for callers that cannot
 * allocate device memory: a runtime that gave the whole GPU to its own pool at
 * start-up, a plugin whose enqueue hook may not allocate, a latency-critical
 * loop that cannot take cudaMalloc's implicit synchronisation.  The workspace
 * is a fixed array inside the library instead of a caller buffer; the call
 * allocates and frees nothing.  (No counterpart in the reference, whose host
 * code always allocates through PyTorch.)
 *
 * Limit: trifast_backward_workspace_bytes(shape) must not exceed
 * TRIFAST_STATIC_SCRATCH_BYTES (16 MiB, reserved on every GPU that loads the
 * library until the process exits); larger problems return
 * TRIFAST_ERR_TOO_LARGE and nothing is launched.  At h = 4 that covers n up to 224
 * for bf16 / fp16 with d = 16, 32 or 64 (where the fp32 row-split partials of db take most
 * of the workspace) and n up to 576 for fp32 or d = 128; with h = 1, n up to 448.
 *
 * The first call on each device resolves the array's device address (that
 * device must be current); make that first call outside any stream capture.
 * All calls on a device share the one array, which keeps whatever the last
 * call left in it: this call overwrites every region before reading it, so no
 * clearing is needed, but two calls whose GPU work overlaps (different streams,
 * or threads) race on it -- serialise them. */
#define TRIFAST_STATIC_SCRATCH_BYTES ((size_t)16 << 20)
int trifast_backward_static_scratch(const trifast_shape* shape,
                                    const trifast_t5* d_o,
                                    const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
                                    const trifast_t4* bias, const trifast_mask* mask,
                                    const trifast_t5* o, const float* lse,
                                    const trifast_t5* dq, const trifast_t5* dk, const trifast_t5* dv,
                                    const trifast_t4* db, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TRIFAST_B200_H_ */
