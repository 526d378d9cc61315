// Host-side launcher interface between the C ABI (api.cu) and the kernel files.
#pragma once

#include "common.cuh"

namespace trifast {

struct FwdArgs {
  View5 q, k, v, o;
  View4 bias;
  MaskView mask;
  float* lse;
  Dims dm;
  int dtype;
  unsigned int* status;  // device status word
};

struct BwdArgs {
  View5 d_o, q, k, v, o, dq, dk, dv;
  View4 bias;
  MaskView mask;
  const float* lse;
  float* delta;          // (b, h, n_rows, n) fp32, in the workspace
  float* neg_lse2;       // (b, h, n_rows, n) fp32: -lse * log2(e), in the workspace
  void* bias_t;          // (b, h, k, j) transposed bias copy in the input dtype, or null
  uint8_t* rowfull;      // (b, n_rows): 1 = every key of the row is masked
  uint32_t* maskbits;    // (b, n_rows, mask_words): bit set = key dropped or beyond n
  int mask_words;        // 4 * ceil(n / 128)
  float* db_f32;         // (b, h, n, n) fp32 result of the row reduction
  float* db_partials;    // (splits, b, h, n, n) fp32, used when splits > 1
  int splits;
  Dims dm;
  int dtype;
  unsigned int* status;
};

// CUDA-core kernels (simt_kernels.cu): any dtype, any n, d in {16, 32, 64, 128}.
cudaError_t simt_forward(const FwdArgs& a, cudaStream_t s);
cudaError_t bwd_prepare(const BwdArgs& a, cudaStream_t s);   // delta + rowfull (all paths)
cudaError_t simt_bwd_db(const BwdArgs& a, cudaStream_t s);
cudaError_t simt_bwd_dq(const BwdArgs& a, cudaStream_t s);
cudaError_t simt_bwd_dkv(const BwdArgs& a, cudaStream_t s);
cudaError_t db_reduce_splits(const BwdArgs& a, cudaStream_t s);
cudaError_t db_cast(const float* db_f32, View4 db, int dtype, int batch, int heads, int n,
                    cudaStream_t s);

// tcgen05 kernels (tc_*.cu): bf16 / fp16.
bool tc_forward_supported(const Dims& dm, int dtype, const FwdArgs* a);
cudaError_t tc_forward(const FwdArgs& a, const trifast_plan& plan, cudaStream_t s);
bool tc_backward_supported(const BwdArgs& a);
cudaError_t tc_bwd_dq(const BwdArgs& a, cudaStream_t s);
cudaError_t tc_bwd_dkv(const BwdArgs& a, cudaStream_t s);
cudaError_t tc_bwd_db(const BwdArgs& a, cudaStream_t s);

}  // namespace trifast
