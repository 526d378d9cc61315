// Host-side launcher interface between the C ABI (api.cu) and the kernel files.
#pragma once

#include "common.cuh"

namespace trifast {

struct FwdArgs {
  View5 q, k, v, o;
  View4 bias;
  MaskView mask;
  float* lse;
  // forward workspace (tensor-core path with n % 8 != 0 only; null otherwise)
  void* bias_pad;        // (b, h, j, n_pad) copy of the bias with a 16-byte row pitch
  uint8_t* rowfull;      // (b, n_rows)
  uint32_t* maskbits;    // (b, n_rows, mask_words)
  int mask_words;
  // (b, n_rows): live key tiles [lo, hi) of each row as lo | hi << 16 (tensor-core path,
  // every n; null otherwise)
  uint32_t* rowrange;
  Dims dm;
  int dtype;
  unsigned int* status;  // device status word
};

struct BwdArgs {
  View5 d_o, q, k, v, o, dq, dk, dv;
  View4 bias;
  MaskView mask;
  const float* lse;
  float* delta;          // (b, h, n_rows, n_pad) fp32, in the workspace
  float* neg_lse2;       // (b, h, n_rows, n_pad) fp32: -lse * log2(e), in the workspace
  void* bias_t;          // (b, h, k, n_pad) transposed bias copy in the input dtype, or null
  void* bias_pad;        // (b, h, j, n_pad) bias copy with a 16-byte row pitch (n % 8 != 0), or null
  uint8_t* rowfull;      // (b, n_rows): 1 = every key of the row is masked
  // (b, n_rows, mask_words): bit set = key dropped or beyond n.  Per 128-key chunk c
  // four words: word c*4 + jb holds, at bit l, key c*128 + 4*l + jb.
  uint32_t* maskbits;
  // same bits in key order: word w holds, at bit l, key 32 * w + l
  uint32_t* maskbits_lin;
  int mask_words;        // 4 * ceil(n / 128)
  uint32_t* rowrange;    // (b, n_rows): live key tiles [lo, hi) of the row as lo | hi << 16
  float* db_f32;         // (b, h, n, n) fp32 result of the row reduction
  float* db_partials;    // (splits, b, h, n, n) fp32, used when splits > 1
  int splits;
  Dims dm;
  int dtype;
  float* kv_scratch;     // per-CTA fp32 dK / dV partials of rows walked in several query chunks, or null
  int reserve_sms;       // SMs the persistent dq / dk / dv kernels leave free (a collective running beside them)
  unsigned int* status;
};

// CUDA-core kernels (simt_kernels.cu): any dtype, any n, d in {16, 32, 64, 128}.
cudaError_t simt_forward(const FwdArgs& a, cudaStream_t s);
cudaError_t bwd_prepare(const BwdArgs& a, cudaStream_t s);   // delta, row flags, masks, bias copies
cudaError_t fwd_prepare(const FwdArgs& a, cudaStream_t s);   // row flags, masks, padded bias
cudaError_t simt_bwd_db(const BwdArgs& a, cudaStream_t s);
cudaError_t simt_bwd_dq(const BwdArgs& a, cudaStream_t s);
cudaError_t simt_bwd_dkv(const BwdArgs& a, cudaStream_t s);
cudaError_t db_reduce_splits(const BwdArgs& a, cudaStream_t s);
cudaError_t db_cast(const float* db_f32, View4 db, int dtype, int batch, int heads, int n,
                    cudaStream_t s);

// tcgen05 kernels (tc_*.cu): bf16 / fp16.
bool tc_forward_d128_supported(const Dims& dm, int dtype, const FwdArgs* a);
cudaError_t tc_forward_d128(const FwdArgs& a, cudaStream_t s);
bool tc_forward_supported(const Dims& dm, int dtype, const FwdArgs* a);
cudaError_t tc_forward(const FwdArgs& a, const trifast_plan& plan, cudaStream_t s);
bool tc_backward_supported(const BwdArgs& a);
cudaError_t tc_bwd_dq(const BwdArgs& a, cudaStream_t s);
cudaError_t tc_bwd_dkv(const BwdArgs& a, cudaStream_t s);
cudaError_t tc_bwd_db(const BwdArgs& a, cudaStream_t s);
// dq, dk and dv in one pass over the scores
bool tc_bwd_fused_supported(const BwdArgs& a);
int tc_bwd_fused_chunks(int n, int d);             // query chunks per row (1: dQ of a row fits TMEM)
size_t tc_bwd_fused_scratch_bytes(int n, int d);   // 0 when one chunk
cudaError_t tc_bwd_dqkv_fused(const BwdArgs& a, cudaStream_t s);

// Sum of the row shards' fp32 db partials by peer stores (db_push_reduce.cu).
cudaError_t db_push_reduce(const trifast_push_reduce* a, unsigned int* status, cudaStream_t s);

// One warp whose bounded wait runs out after limit_cycles (test support).
cudaError_t wait_probe(long long limit_cycles, unsigned int* status, cudaStream_t s);

}  // namespace trifast
