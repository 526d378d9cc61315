// C ABI of the library: argument validation, the fixed tile heuristic, workspace
// carving and dispatch to the kernel launchers.  Entry points are declared and
// documented in include/trifast_b200.h.

#include <float.h>
#include <math.h>

#include <mutex>

#include "kernels.h"

namespace trifast {
namespace {

__device__ unsigned int g_device_status;  // OR of DeviceStatusBits

constexpr int kMaxDevices = 64;
// SMs the persistent dq / dk / dv kernels leave free under TRIFAST_FLAG_SHARE_GPU: their
// CTAs take a whole SM each (registers, shared memory), so a collective kernel launched
// beside them would otherwise only start when they end.
constexpr int kSharedGpuSms = 8;
unsigned int* g_status_ptr[kMaxDevices];
int g_arch_major[kMaxDevices];
std::once_flag g_once[kMaxDevices];

// Per-device set-up, once: address of the status word and the compute capability.
int device_setup(int* dev_out, unsigned int** status) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return TRIFAST_ERR_LAUNCH;
  std::call_once(g_once[dev], [dev] {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess) g_status_ptr[dev] = (unsigned int*)p;
    int major = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    g_arch_major[dev] = major;
  });
  if (!g_status_ptr[dev]) return TRIFAST_ERR_LAUNCH;
  if (g_arch_major[dev] != 10) return TRIFAST_ERR_ARCH;
  *dev_out = dev;
  *status = g_status_ptr[dev];
  return TRIFAST_OK;
}

int elem_bytes(int dtype) { return dtype == TRIFAST_F32 ? 4 : 2; }

float dtype_sentinel(int dtype) {
  switch (dtype) {
    case TRIFAST_F32: return -FLT_MAX;
    case TRIFAST_BF16: return -3.3895313892515355e38f;  // finfo(bfloat16).min
    default: return -65504.f;                           // finfo(float16).min
  }
}

int check_shape(const trifast_shape* s) {
  if (!s) return TRIFAST_ERR_NULL;
  if (s->batch <= 0 || s->heads <= 0 || s->n <= 0 || s->n_rows <= 0 || s->n_rows > s->n)
    return TRIFAST_ERR_SHAPE;
  if ((int64_t)s->batch * s->heads > 65535 || s->n_rows > 65535) return TRIFAST_ERR_SHAPE;
  if (s->d != 16 && s->d != 32 && s->d != 64 && s->d != 128) return TRIFAST_ERR_HEAD_DIM;
  if (s->dtype < TRIFAST_F32 || s->dtype > TRIFAST_F16) return TRIFAST_ERR_DTYPE;
  if (s->kernel < TRIFAST_KERNEL_AUTO || s->kernel > TRIFAST_KERNEL_TCGEN05)
    return TRIFAST_ERR_KERNEL_CHOICE;
  if (s->flags & ~(TRIFAST_FLAG_SPLIT_BWD | TRIFAST_FLAG_SHARE_GPU | 0xff00)) return TRIFAST_ERR_KERNEL_CHOICE;
  if ((s->flags & 0xff00) && !(s->flags & TRIFAST_FLAG_SHARE_GPU)) return TRIFAST_ERR_KERNEL_CHOICE;
  return TRIFAST_OK;
}

// Row-vector tensors are read with 16-byte vector / TMA accesses by the
// tensor-core kernels, so bases are 16-byte aligned and every stride is a
// whole number of 16-byte units for all kernels alike.
int check_t5(const trifast_t5* t, const trifast_shape* s) {
  if (!t || !t->data) return TRIFAST_ERR_NULL;
  if (((uintptr_t)t->data) & 15) return TRIFAST_ERR_ALIGN;
  const int eb = elem_bytes(s->dtype);
  for (int a = 0; a < 4; ++a) {
    if (t->stride[a] < 0) return TRIFAST_ERR_STRIDE;
    if ((t->stride[a] * eb) & 15) return TRIFAST_ERR_STRIDE;
  }
  if (t->stride[3] < s->d) return TRIFAST_ERR_STRIDE;
  // A stride of 0 (an expanded dimension) cannot be described to TMA; callers
  // materialise such views first.  Dimensions of extent 1 may carry any stride.
  const int ext[3] = {s->batch, s->heads, s->n_rows};
  for (int a = 0; a < 3; ++a)
    if (ext[a] > 1 && t->stride[a] == 0) return TRIFAST_ERR_STRIDE;
  return TRIFAST_OK;
}

int check_t4(const trifast_t4* t, const trifast_shape* s) {
  if (!t || !t->data) return TRIFAST_ERR_NULL;
  const int eb = elem_bytes(s->dtype);
  if (((uintptr_t)t->data) & (eb - 1)) return TRIFAST_ERR_ALIGN;
  for (int a = 0; a < 3; ++a)
    if (t->stride[a] < 0) return TRIFAST_ERR_STRIDE;
  if (t->stride[2] < s->n) return TRIFAST_ERR_STRIDE;
  return TRIFAST_OK;
}

int check_mask(const trifast_mask* m, const trifast_shape* s) {
  if (!m || !m->data) return TRIFAST_ERR_NULL;
  if (m->stride[0] < 0 || m->stride[1] < s->n) return TRIFAST_ERR_STRIDE;
  return TRIFAST_OK;
}

Dims make_dims(const trifast_shape* s) {
  Dims dm;
  dm.batch = s->batch;
  dm.heads = s->heads;
  dm.n = s->n;
  dm.n_rows = s->n_rows;
  dm.d = s->d;
  dm.n_pad = (s->n + 7) / 8 * 8;
  dm.scale = 1.0f / sqrtf((float)s->d);
  dm.sentinel = dtype_sentinel(s->dtype);
  return dm;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Carve-up of the backward workspace.
struct Workspace {
  size_t delta_off, nlse_off, rowfull_off, rowrange_off, maskbits_off, db_off, bias_t_off,
      bias_pad_off, partial_off, kv_scratch_off, kv_scratch_bytes, total;
  int mask_words;
  bool has_bias_t, has_bias_pad;
};

// Forward workspace of the tensor-core path: the live key-tile range of every row, and for
// n % 8 != 0 a copy of the bias with a 16-byte row pitch, the packed key masks and the row
// flags.  The CUDA-core path needs none.
struct FwdWorkspace {
  size_t rowrange_off, rowfull_off, maskbits_off, bias_pad_off, total;
  int mask_words;
  bool masks, bias_pad;   // the packed masks and row flags / the padded bias copy are present
};

FwdWorkspace carve_fwd(const trifast_shape* s, const trifast_plan& plan) {
  FwdWorkspace w{};
  w.mask_words = ((s->n + 127) / 128) * 4;
  if (plan.fwd_kernel != TRIFAST_KERNEL_TCGEN05) return w;
  size_t off = 0;
  w.rowrange_off = off;
  off = (off + (size_t)s->batch * s->n_rows * sizeof(uint32_t) + 255) / 256 * 256;
  w.total = off;
  w.bias_pad = s->n % 8 != 0;
  w.masks = w.bias_pad || s->d == 128;   // the head-dim-128 forward always reads prepared masks
  if (!w.masks) return w;
  const size_t n_pad = (size_t)(s->n + 7) / 8 * 8;
  w.rowfull_off = off;
  off = (off + (size_t)s->batch * s->n_rows + 255) / 256 * 256;
  w.maskbits_off = off;
  off = (off + (size_t)s->batch * s->n_rows * w.mask_words * sizeof(uint32_t) + 255) / 256 * 256;
  w.bias_pad_off = off;
  if (w.bias_pad) off = (off + (size_t)s->batch * s->heads * s->n * n_pad * 2 + 255) / 256 * 256;
  w.total = off;
  return w;
}

Workspace carve(const trifast_shape* s, const trifast_plan& plan) {
  Workspace w;
  const size_t n_pad = (size_t)(s->n + 7) / 8 * 8;  // row pitch of the vectors and bias copies
  const size_t stat = (size_t)s->batch * s->heads * s->n_rows * n_pad * sizeof(float);
  const size_t dbb = (size_t)s->batch * s->heads * s->n * s->n * sizeof(float);
  const size_t bias_copy = (size_t)s->batch * s->heads * s->n * n_pad * 2;
  size_t off = 0;
  w.delta_off = off;
  off = align_up(off + stat, 256);
  w.nlse_off = off;
  off = align_up(off + stat, 256);
  w.rowfull_off = off;
  off = align_up(off + (size_t)s->batch * s->n_rows, 256);
  w.rowrange_off = off;
  off = align_up(off + (size_t)s->batch * s->n_rows * sizeof(uint32_t), 256);
  w.mask_words = ((s->n + 127) / 128) * 4;
  w.maskbits_off = off;
  // two layouts of the packed key masks, one after the other (see BwdArgs)
  off = align_up(off + 2 * (size_t)s->batch * s->n_rows * w.mask_words * sizeof(uint32_t), 256);
  w.db_off = off;
  off = align_up(off + dbb, 256);
  // transposed bias copy for the tensor-core dk/dv kernel (16-bit dtypes only)
  w.has_bias_t = plan.kernel == TRIFAST_KERNEL_TCGEN05;
  w.bias_t_off = off;
  if (w.has_bias_t) off = align_up(off + bias_copy, 256);
  // bias copy with a 16-byte row pitch, when the bias rows themselves are not
  w.has_bias_pad = w.has_bias_t && s->n % 8 != 0;
  w.bias_pad_off = off;
  if (w.has_bias_pad) off = align_up(off + bias_copy, 256);
  w.partial_off = off;
  if (plan.db_row_splits > 1) off = align_up(off + dbb * plan.db_row_splits, 256);
  // dK / dV partials of the one-pass backward for rows walked in several query chunks
  w.kv_scratch_off = off;
  w.kv_scratch_bytes = plan.bwd_fused ? tc_bwd_fused_scratch_bytes(s->n, s->d) : 0;
  off = align_up(off + w.kv_scratch_bytes, 256);
  w.total = off;
  return w;
}

int pick_plan(const trifast_shape* s, trifast_plan* p) {
  int rc = check_shape(s);
  if (rc) return rc;
  *p = trifast_plan{};
  const bool half = s->dtype != TRIFAST_F32;
  // tcgen05 path: 16-bit inputs, d in {16, 32, 64}; problems smaller than one 128-wide
  // tile gain nothing from it.  (n % 8 != 0 runs on it through a padded bias copy in
  // the workspace: TMA needs a 16-byte row pitch.)  The two-kernel backward has no
  // d = 16 tiles.
  const bool tc_ok = half && (s->d == 16 || s->d == 32 || s->d == 64) && s->n >= kMinTensorCoreN &&
                     !(s->d == 16 && (s->flags & TRIFAST_FLAG_SPLIT_BWD));
  // Head dim 128 has tensor-core tiles in the forward only: its backward stays on the CUDA
  // cores (`kernel`), and asking for the tensor-core family fails in the backward entry points.
  const bool tc_fwd_only = half && s->d == 128 && s->n >= kMinTensorCoreN;
  int kernel = s->kernel;
  if (kernel == TRIFAST_KERNEL_AUTO) kernel = tc_ok ? TRIFAST_KERNEL_TCGEN05 : TRIFAST_KERNEL_SIMT;
  if (kernel == TRIFAST_KERNEL_TCGEN05 && !tc_ok && !tc_fwd_only) return TRIFAST_ERR_KERNEL_CHOICE;
  if (tc_fwd_only) kernel = TRIFAST_KERNEL_SIMT;
  p->kernel = kernel;
  p->fwd_kernel = (tc_fwd_only && s->kernel != TRIFAST_KERNEL_SIMT) ? TRIFAST_KERNEL_TCGEN05 : kernel;
  if (kernel == TRIFAST_KERNEL_TCGEN05) {
    p->block_j = 128;
    p->block_k = 128;
    p->rows_per_cta = 2;
    p->stages = (s->d <= 32) ? 3 : 2;
  } else {
    p->block_j = 64;
    p->block_k = (s->d <= 32) ? 32 : 16;
    p->rows_per_cta = 1;
    p->stages = 1;
  }
  // db: CTAs = tiles * splits.  Split the local rows until the grid covers the
  // 148 SMs twice (CUDA-core kernel, 32 x 32 tiles, several CTAs per SM) or four
  // times (tensor-core kernel, 128 x 128 tiles, one CTA per SM), but never below
  // 8 rows per split and at most 16 splits.
  const bool tc_db = kernel == TRIFAST_KERNEL_TCGEN05;
  const int tile = tc_db ? 128 : 32;
  const int64_t want = tc_db ? 592 : 296;
  const int64_t t = (s->n + tile - 1) / tile;
  const int64_t tiles = t * t * s->batch * s->heads;
  int splits = 1;
  while (splits < 16 && tiles * splits < want && s->n_rows / (splits * 2) >= 8) splits *= 2;
  p->db_row_splits = splits;
  // dq, dk, dv from one kernel on the tensor-core path; a row whose dQ (D fp32 columns
  // per 128 queries) does not fit in TMEM beside the other accumulators (192 + 2 D
  // columns) is walked in bwd_chunks query chunks
  p->bwd_fused = (tc_db && !(s->flags & TRIFAST_FLAG_SPLIT_BWD)) ? 1 : 0;
  p->bwd_chunks = p->bwd_fused ? tc_bwd_fused_chunks(s->n, s->d) : 0;
  return TRIFAST_OK;
}

struct Common {
  Dims dm;
  trifast_plan plan;
  unsigned int* status;
};

int common_setup(const trifast_shape* s, Common* c) {
  int rc = pick_plan(s, &c->plan);
  if (rc) return rc;
  int dev;
  rc = device_setup(&dev, &c->status);
  if (rc) return rc;
  c->dm = make_dims(s);
  return TRIFAST_OK;
}

int fill_bwd(const trifast_shape* shape, const Common& c, const trifast_t5* d_o,
             const trifast_t5* q, const trifast_t5* k, const trifast_t5* v,
             const trifast_t4* bias, const trifast_mask* mask, const trifast_t5* o,
             const float* lse, void* workspace, size_t workspace_bytes, BwdArgs* a) {
  int rc;
  if ((rc = check_t5(d_o, shape)) || (rc = check_t5(q, shape)) || (rc = check_t5(k, shape)) ||
      (rc = check_t5(v, shape)) || (rc = check_t4(bias, shape)) || (rc = check_mask(mask, shape)))
    return rc;
  if (o && (rc = check_t5(o, shape))) return rc;
  if (!lse) return TRIFAST_ERR_NULL;
  // (head dim 128: tensor-core tiles exist for the forward only)
  if (shape->kernel == TRIFAST_KERNEL_TCGEN05 && c.plan.kernel != TRIFAST_KERNEL_TCGEN05)
    return TRIFAST_ERR_KERNEL_CHOICE;
  const Workspace w = carve(shape, c.plan);
  if (!workspace || workspace_bytes < w.total) return TRIFAST_ERR_WORKSPACE;
  if (((uintptr_t)workspace) & 255) return TRIFAST_ERR_ALIGN;
  *a = BwdArgs{};
  a->d_o = make_view(d_o);
  a->q = make_view(q);
  a->k = make_view(k);
  a->v = make_view(v);
  if (o) a->o = make_view(o);
  a->bias = make_view(bias);
  a->mask = make_view(mask);
  a->lse = lse;
  char* base = (char*)workspace;
  a->delta = (float*)(base + w.delta_off);
  a->neg_lse2 = (float*)(base + w.nlse_off);
  a->bias_t = w.has_bias_t ? (void*)(base + w.bias_t_off) : nullptr;
  a->bias_pad = w.has_bias_pad ? (void*)(base + w.bias_pad_off) : nullptr;
  a->rowfull = (uint8_t*)(base + w.rowfull_off);
  a->rowrange = (uint32_t*)(base + w.rowrange_off);
  a->maskbits = (uint32_t*)(base + w.maskbits_off);
  a->maskbits_lin = a->maskbits + (size_t)shape->batch * shape->n_rows * w.mask_words;
  a->mask_words = w.mask_words;
  a->db_f32 = (float*)(base + w.db_off);
  a->db_partials = (float*)(base + w.partial_off);
  a->kv_scratch = w.kv_scratch_bytes ? (float*)(base + w.kv_scratch_off) : nullptr;
  a->splits = c.plan.db_row_splits;
  a->dm = c.dm;
  a->dtype = shape->dtype;
  a->reserve_sms = (shape->flags & TRIFAST_FLAG_SHARE_GPU)
                       ? (((shape->flags >> 8) & 0xff) ? ((shape->flags >> 8) & 0xff) : kSharedGpuSms)
                       : 0;
  a->status = c.status;
  return TRIFAST_OK;
}

// The CUDA error behind the last TRIFAST_ERR_LAUNCH of the calling thread.
thread_local cudaError_t g_last_cuda_error = cudaSuccess;

int cuda_rc(cudaError_t e) {
  if (e == cudaSuccess) return TRIFAST_OK;
  g_last_cuda_error = e;
  return TRIFAST_ERR_LAUNCH;
}

}  // namespace
}  // namespace trifast

using namespace trifast;

extern "C" {

int trifast_version(void) { return 100; }

int trifast_copy_blocks(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                        size_t block_bytes, size_t blocks, int to_host, void* stream) {
  if (!dst || !src) return TRIFAST_ERR_NULL;
  if (block_bytes == 0 || blocks == 0) return TRIFAST_OK;
  if (dst_pitch < block_bytes || src_pitch < block_bytes) return TRIFAST_ERR_STRIDE;
  return cuda_rc(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, block_bytes, blocks,
                                   to_host ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice,
                                   (cudaStream_t)stream));
}

const char* trifast_last_cuda_error(void) { return cudaGetErrorName(g_last_cuda_error); }

const char* trifast_status_str(int status) {
  switch (status) {
    case TRIFAST_OK: return "ok";
    case TRIFAST_ERR_NULL: return "a required pointer is NULL";
    case TRIFAST_ERR_SHAPE: return "invalid shape (extents must be positive, n_rows <= n, batch*heads and n_rows <= 65535)";
    case TRIFAST_ERR_HEAD_DIM: return "head dim must be 16, 32, 64 or 128";
    case TRIFAST_ERR_DTYPE: return "dtype must be fp32, bf16 or fp16";
    case TRIFAST_ERR_STRIDE: return "invalid stride (negative, overlapping, or not a multiple of 16 bytes)";
    case TRIFAST_ERR_ALIGN: return "pointer is not sufficiently aligned (16 bytes for q/k/v/o and gradients, 256 for the workspace)";
    case TRIFAST_ERR_WORKSPACE: return "workspace is NULL or smaller than trifast_backward_workspace_bytes()";
    case TRIFAST_ERR_ARCH: return "device is not compute capability 10.x (B200)";
    case TRIFAST_ERR_LAUNCH: return "CUDA reported an error at launch";
    case TRIFAST_ERR_KERNEL_CHOICE: return "the requested kernel family cannot run this problem";
    case TRIFAST_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    case TRIFAST_ERR_TOO_LARGE: return "problem is larger than this entry point's stated maximum";
    default: return "unknown status";
  }
}

int trifast_pick_plan(const trifast_shape* shape, trifast_plan* plan) {
  if (!plan) return TRIFAST_ERR_NULL;
  return pick_plan(shape, plan);
}

size_t trifast_backward_workspace_bytes(const trifast_shape* shape) {
  trifast_plan plan;
  if (pick_plan(shape, &plan)) return 0;
  return carve(shape, plan).total;
}

size_t trifast_forward_workspace_bytes(const trifast_shape* shape) {
  trifast_plan plan;
  if (pick_plan(shape, &plan)) return 0;
  return carve_fwd(shape, plan).total;
}

int trifast_forward(const trifast_shape* shape, const trifast_t5* q, const trifast_t5* k,
                    const trifast_t5* v, const trifast_t4* bias, const trifast_mask* mask,
                    const trifast_t5* o, float* lse, void* workspace, size_t workspace_bytes,
                    void* stream) {
  int rc = check_shape(shape);
  if (rc) return rc;
  if ((rc = check_t5(q, shape)) || (rc = check_t5(k, shape)) || (rc = check_t5(v, shape)) ||
      (rc = check_t5(o, shape)) || (rc = check_t4(bias, shape)) || (rc = check_mask(mask, shape)))
    return rc;
  if (!lse) return TRIFAST_ERR_NULL;
  Common c;
  if ((rc = common_setup(shape, &c))) return rc;
  const FwdWorkspace w = carve_fwd(shape, c.plan);
  if (w.total && (!workspace || workspace_bytes < w.total)) return TRIFAST_ERR_WORKSPACE;
  if (w.total && (((uintptr_t)workspace) & 255)) return TRIFAST_ERR_ALIGN;
  FwdArgs a{};
  a.q = make_view(q);
  a.k = make_view(k);
  a.v = make_view(v);
  a.o = make_view(o);
  a.bias = make_view(bias);
  a.mask = make_view(mask);
  a.lse = lse;
  a.dm = c.dm;
  a.dtype = shape->dtype;
  a.status = c.status;
  a.mask_words = w.mask_words;
  if (w.total) {
    char* base = (char*)workspace;
    a.rowrange = (uint32_t*)(base + w.rowrange_off);
    if (w.masks) {
      a.rowfull = (uint8_t*)(base + w.rowfull_off);
      a.maskbits = (uint32_t*)(base + w.maskbits_off);
    }
    if (w.bias_pad) a.bias_pad = (void*)(base + w.bias_pad_off);
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (c.plan.fwd_kernel == TRIFAST_KERNEL_TCGEN05) {
    const bool d128 = c.dm.d == 128;
    if (!(d128 ? tc_forward_d128_supported(c.dm, shape->dtype, &a)
               : tc_forward_supported(c.dm, shape->dtype, &a))) {
      if (shape->kernel == TRIFAST_KERNEL_TCGEN05) return TRIFAST_ERR_KERNEL_CHOICE;
      return cuda_rc(simt_forward(a, s));
    }
    if (w.total && (rc = cuda_rc(fwd_prepare(a, s)))) return rc;
    return cuda_rc(d128 ? tc_forward_d128(a, s) : tc_forward(a, c.plan, s));
  }
  return cuda_rc(simt_forward(a, s));
}

int trifast_backward_db(const trifast_shape* shape, const trifast_t5* d_o, const trifast_t5* q,
                        const trifast_t5* k, const trifast_t5* v, const trifast_t4* bias,
                        const trifast_mask* mask, const trifast_t5* o, const float* lse,
                        float* db_f32, void* workspace, size_t workspace_bytes, void* stream) {
  Common c;
  int rc = common_setup(shape, &c);
  if (rc) return rc;
  if (!o || !db_f32) return TRIFAST_ERR_NULL;
  BwdArgs a;
  if ((rc = fill_bwd(shape, c, d_o, q, k, v, bias, mask, o, lse, workspace, workspace_bytes, &a)))
    return rc;
  a.db_f32 = db_f32;
  cudaStream_t s = (cudaStream_t)stream;
  if ((rc = cuda_rc(bwd_prepare(a, s)))) return rc;
  bool tc = c.plan.kernel == TRIFAST_KERNEL_TCGEN05;
  if (tc && !tc_backward_supported(a)) {
    if (shape->kernel == TRIFAST_KERNEL_TCGEN05) return TRIFAST_ERR_KERNEL_CHOICE;
    tc = false;
  }
  if ((rc = cuda_rc(tc ? tc_bwd_db(a, s) : simt_bwd_db(a, s)))) return rc;
  return cuda_rc(db_reduce_splits(a, s));
}

int trifast_backward_dqkv(const trifast_shape* shape, const trifast_t5* d_o, const trifast_t5* q,
                          const trifast_t5* k, const trifast_t5* v, const trifast_t4* bias,
                          const trifast_mask* mask, const float* lse, const trifast_t5* dq,
                          const trifast_t5* dk, const trifast_t5* dv, void* workspace,
                          size_t workspace_bytes, void* stream) {
  Common c;
  int rc = common_setup(shape, &c);
  if (rc) return rc;
  if ((rc = check_t5(dq, shape)) || (rc = check_t5(dk, shape)) || (rc = check_t5(dv, shape)))
    return rc;
  BwdArgs a;
  if ((rc = fill_bwd(shape, c, d_o, q, k, v, bias, mask, nullptr, lse, workspace,
                     workspace_bytes, &a)))
    return rc;
  a.dq = make_view(dq);
  a.dk = make_view(dk);
  a.dv = make_view(dv);
  cudaStream_t s = (cudaStream_t)stream;
  bool tc = c.plan.kernel == TRIFAST_KERNEL_TCGEN05;
  if (tc && !tc_backward_supported(a)) {
    if (shape->kernel == TRIFAST_KERNEL_TCGEN05) return TRIFAST_ERR_KERNEL_CHOICE;
    tc = false;
  }
  if (tc && c.plan.bwd_fused && tc_bwd_fused_supported(a)) return cuda_rc(tc_bwd_dqkv_fused(a, s));
  if ((rc = cuda_rc(tc ? tc_bwd_dq(a, s) : simt_bwd_dq(a, s)))) return rc;
  return cuda_rc(tc ? tc_bwd_dkv(a, s) : simt_bwd_dkv(a, s));
}

int trifast_db_finalize(const trifast_shape* shape, const float* db_f32, const trifast_t4* db,
                        void* stream) {
  int rc = check_shape(shape);
  if (rc) return rc;
  if (!db_f32) return TRIFAST_ERR_NULL;
  if ((rc = check_t4(db, shape))) return rc;
  return cuda_rc(db_cast(db_f32, make_view(db), shape->dtype, shape->batch, shape->heads,
                         shape->n, (cudaStream_t)stream));
}

int trifast_backward(const trifast_shape* shape, const trifast_t5* d_o, const trifast_t5* q,
                     const trifast_t5* k, const trifast_t5* v, const trifast_t4* bias,
                     const trifast_mask* mask, const trifast_t5* o, const float* lse,
                     const trifast_t5* dq, const trifast_t5* dk, const trifast_t5* dv,
                     const trifast_t4* db, void* workspace, size_t workspace_bytes,
                     void* stream) {
  int rc = check_shape(shape);
  if (rc) return rc;
  // every argument is checked before the first launch, so that a bad descriptor
  // never leaves part of the backward enqueued
  if ((rc = check_t5(dq, shape)) || (rc = check_t5(dk, shape)) || (rc = check_t5(dv, shape)) ||
      (rc = check_t4(db, shape)))
    return rc;
  trifast_plan plan;
  if ((rc = pick_plan(shape, &plan))) return rc;
  const Workspace w = carve(shape, plan);
  if (!workspace || workspace_bytes < w.total) return TRIFAST_ERR_WORKSPACE;
  float* db_f32 = (float*)((char*)workspace + w.db_off);
  if ((rc = trifast_backward_db(shape, d_o, q, k, v, bias, mask, o, lse, db_f32, workspace,
                                workspace_bytes, stream)))
    return rc;
  if ((rc = trifast_backward_dqkv(shape, d_o, q, k, v, bias, mask, lse, dq, dk, dv, workspace,
                                  workspace_bytes, stream)))
    return rc;
  return trifast_db_finalize(shape, db_f32, db, stream);
}

int trifast_check_device_status(void* stream) {
  int dev;
  unsigned int* status;
  int rc = device_setup(&dev, &status);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  unsigned int host = 0;
  if (cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return TRIFAST_ERR_LAUNCH;
  if (cudaStreamSynchronize(s) != cudaSuccess) return TRIFAST_ERR_LAUNCH;
  if (host == 0) return TRIFAST_OK;
  cudaMemsetAsync(status, 0, sizeof(host), s);
  cudaStreamSynchronize(s);
  return TRIFAST_ERR_DEVICE_TIMEOUT;
}

size_t trifast_db_push_reduce_staging_floats(int64_t count, int32_t world) {
  if (count <= 0 || world < 1 || world > 8) return 0;
  const int64_t slice = ((count + world - 1) / world + 3) / 4 * 4;
  return (size_t)slice * world;
}

int trifast_db_push_reduce(const trifast_push_reduce* a, void* stream) {
  if (!a) return TRIFAST_ERR_NULL;
  if (a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world || a->count <= 0 ||
      a->epoch == 0 || a->ctas < 0 || a->ctas > 64)
    return TRIFAST_ERR_SHAPE;
  if (!a->partial || !a->counters) return TRIFAST_ERR_NULL;
  if (((uintptr_t)a->partial) & 15) return TRIFAST_ERR_ALIGN;
  for (int r = 0; r < a->world; ++r) {
    if (!a->staging[r] || !a->result[r] || !a->flags[r]) return TRIFAST_ERR_NULL;
    if ((((uintptr_t)a->staging[r]) & 15) || (((uintptr_t)a->result[r]) & 15)) return TRIFAST_ERR_ALIGN;
  }
  int dev;
  unsigned int* status;
  int rc = device_setup(&dev, &status);
  if (rc) return rc;
  return cuda_rc(db_push_reduce(a, status, (cudaStream_t)stream));
}

int trifast_snapshot_device_status(uint32_t* host_word, void* stream) {
  if (!host_word) return TRIFAST_ERR_NULL;
  int dev;
  unsigned int* status;
  int rc = device_setup(&dev, &status);
  if (rc) return rc;
  return cuda_rc(cudaMemcpyAsync(host_word, status, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                 (cudaStream_t)stream));
}

int trifast_debug_wait_probe(uint32_t limit_us, void* stream) {
  if (limit_us == 0 || limit_us > 100000u) return TRIFAST_ERR_TOO_LARGE;
  int dev;
  unsigned int* status;
  int rc = device_setup(&dev, &status);
  if (rc) return rc;
  // about 2000 clock cycles per microsecond at the B200's 1.97 GHz
  return cuda_rc(wait_probe((long long)limit_us * 2000LL, status, (cudaStream_t)stream));
}

}  // extern "C"
