// Shared device/host helpers of the triangle-attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/trifast_b200.h"

namespace trifast {

// Smallest n the tensor-core kernels take: one 128 x 128 tile at least a quarter full.
constexpr int kMinTensorCoreN = 64;


// (b, h, i, j, d) view with element strides; d contiguous.
struct View5 {
  char* p;
  int64_t sb, sh, si, sj;
};
// (b, h, j, k) view with element strides; k contiguous.
struct View4 {
  char* p;
  int64_t sb, sh, sj;
};
// (b, i, k) byte mask.
struct MaskView {
  const uint8_t* p;
  int64_t sb, si;
};

struct Dims {
  int batch, heads, n, n_rows, d;
  int n_pad;       // n rounded up to 8: row pitch (elements) of workspace vectors and bias copies
  float scale;     // d^-0.5
  float sentinel;  // finfo(dtype).min as float: stored as lse of fully masked rows
};

inline View5 make_view(const trifast_t5* t) {
  return View5{(char*)t->data, t->stride[0], t->stride[1], t->stride[2], t->stride[3]};
}
inline View4 make_view(const trifast_t4* t) {
  return View4{(char*)t->data, t->stride[0], t->stride[1], t->stride[2]};
}
inline MaskView make_view(const trifast_mask* t) {
  return MaskView{t->data, t->stride[0], t->stride[1]};
}

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}
template <> __device__ __forceinline__ __half from_f32<__half>(float x) {
  return __float2half_rn(x);
}

// Kernels whose bounded waits give up OR a non-zero code into a device status
// word (they never trap); its address is handed to them as a kernel argument.
enum DeviceStatusBits : unsigned int {
  kStatusTimeoutFwd = 1u,
  kStatusTimeoutBwdDb = 2u,
  kStatusTimeoutBwdDq = 4u,
  kStatusTimeoutBwdDkv = 8u,
  kStatusTimeoutBwdFused = 16u,
  kStatusTimeoutProbe = 32u,
  kStatusTimeoutPushReduce = 64u,
};

}  // namespace trifast
