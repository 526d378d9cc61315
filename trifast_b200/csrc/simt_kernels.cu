// CUDA-core (fp32 accumulate, fp32 softmax) triangle-attention kernels.
//
// They serve every dtype, every n (ragged included) and d in {16, 32, 64, 128}:
// the fp32 contract (1e-4 relative to the fp32 reference cannot be met through
// tensor cores without operand splitting) and the shapes the tcgen05 kernels do
// not take.  Structure per kernel:
//   forward : one thread per query j of a (b, h, i, j-tile); K/V tiles staged in
//             shared memory and read as broadcasts; online softmax per key tile.
//   dq      : same mapping; recomputes P from lse, dS = P * (dP - delta).
//   dk/dv   : one thread per key k of a (b, h, i, k-tile); Q/dO tiles broadcast.
//   db      : one CTA per (b, h, 32x32 (j,k) tile, row split); loops over its rows
//             and sums dS in registers -> fixed-order reduction, no atomics.
// Semantics follow the reference's PyTorch path (src/trifast/equiv.py:42-69):
// masked keys weigh exactly 0; a row whose keys are all masked gets uniform
// weights 1/n in the forward and in the backward.

#include <math.h>

#include <type_traits>

#include "kernels.h"

namespace trifast {
namespace {

constexpr float kMinusInf = -INFINITY;
constexpr float kMaxInit = -1e30f;  // finite start of the running max: exp(-inf - m) stays 0, never NaN

template <typename T>
__device__ __forceinline__ const T* row5(const View5& t, int b, int h, int i, int j) {
  return (const T*)t.p + b * t.sb + h * t.sh + (int64_t)i * t.si + (int64_t)j * t.sj;
}
template <typename T>
__device__ __forceinline__ T* row5w(const View5& t, int b, int h, int i, int j) {
  return (T*)t.p + b * t.sb + h * t.sh + (int64_t)i * t.si + (int64_t)j * t.sj;
}
template <typename T>
__device__ __forceinline__ const T* row4(const View4& t, int b, int h, int j) {
  return (const T*)t.p + b * t.sb + h * t.sh + (int64_t)j * t.sj;
}

// Stage `rows` x D elements (row r at src(r)) into shared memory as fp32; rows
// beyond `valid` are zero.  Consecutive threads read consecutive elements.
template <typename T, int D, int ROWS, int NT, typename RowFn>
__device__ __forceinline__ void stage_tile(float (*dst)[D], int valid, RowFn src) {
  for (int idx = threadIdx.x; idx < ROWS * D; idx += NT) {
    const int r = idx / D, c = idx % D;
    dst[r][c] = (r < valid) ? to_f32<T>(src(r)[c]) : 0.f;
  }
}

template <int D>
__device__ __forceinline__ float dot_smem(const float* reg, const float* sm) {
  float acc = 0.f;
  const float4* s4 = reinterpret_cast<const float4*>(sm);
#pragma unroll
  for (int c = 0; c < D / 4; ++c) {
    const float4 x = s4[c];
    acc = fmaf(reg[4 * c + 0], x.x, acc);
    acc = fmaf(reg[4 * c + 1], x.y, acc);
    acc = fmaf(reg[4 * c + 2], x.z, acc);
    acc = fmaf(reg[4 * c + 3], x.w, acc);
  }
  return acc;
}

template <int D>
__device__ __forceinline__ void axpy_smem(float a, const float* sm, float* reg) {
  const float4* s4 = reinterpret_cast<const float4*>(sm);
#pragma unroll
  for (int c = 0; c < D / 4; ++c) {
    const float4 x = s4[c];
    reg[4 * c + 0] = fmaf(a, x.x, reg[4 * c + 0]);
    reg[4 * c + 1] = fmaf(a, x.y, reg[4 * c + 1]);
    reg[4 * c + 2] = fmaf(a, x.z, reg[4 * c + 2]);
    reg[4 * c + 3] = fmaf(a, x.w, reg[4 * c + 3]);
  }
}

// ---------------------------------------------------------------------------
// rowfull[b, i] = 1 when every key of pair row i is masked.
// ---------------------------------------------------------------------------
__global__ void rowfull_kernel(MaskView mask, int n, int n_rows, uint8_t* rowfull,
                               uint32_t* maskbits, uint32_t* maskbits_lin, int mask_words,
                               uint32_t* rowrange) {
  const int bi = blockIdx.x;
  const int b = bi / n_rows, i = bi % n_rows;
  const uint8_t* row = mask.p + b * mask.sb + (int64_t)i * mask.si;
  __shared__ int first_open, last_open;
  if (threadIdx.x == 0) {
    first_open = n;
    last_open = -1;
  }
  __syncthreads();
  int lo = n, hi = -1;
  for (int k = threadIdx.x; k < n; k += blockDim.x) {
    if (row[k] == 0) {
      lo = min(lo, k);
      hi = max(hi, k);
    }
  }
  if (hi >= 0) {
    atomicMin(&first_open, lo);
    atomicMax(&last_open, hi);
  }
  __syncthreads();
  const int open = last_open >= 0;
  if (threadIdx.x == 0) {
    if (rowfull) rowfull[bi] = open ? 0 : 1;
    // 128-key tiles [first, last + 1) that hold an open key: the tensor-core kernels walk
    // only those.  A fully masked row weighs all n keys: every tile.
    if (rowrange) {
      const uint32_t t0 = open ? (uint32_t)(first_open >> 7) : 0u;
      const uint32_t t1 = open ? (uint32_t)(last_open >> 7) + 1u : (uint32_t)((n + 127) >> 7);
      rowrange[bi] = t0 | (t1 << 16);
    }
  }
  if (!maskbits) return;
  // Packed key mask (bit set = key dropped or beyond n).  A fully masked row keeps
  // all n keys with uniform weight, so only the keys beyond n stay set.  Layout per
  // 128-key chunk c: word c*4 + jb holds, at bit l, key c*128 + 4*l + jb (the order
  // in which a warp reading four mask bytes per lane produces the words).
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = warp; c < mask_words / 4; c += blockDim.x >> 5) {
#pragma unroll
    for (int jb = 0; jb < 4; ++jb) {
      const int k = c * 128 + 4 * lane + jb;
      const int dropped = (k < n) ? (open ? (row[k] != 0) : 0) : 1;
      const unsigned bits = __ballot_sync(0xffffffffu, dropped);
      if (lane == 0) maskbits[(int64_t)bi * mask_words + c * 4 + jb] = bits;
    }
  }
  // The same bits in key order (word w, bit l: key 32 * w + l), when asked for.
  if (maskbits_lin) {
    for (int w = warp; w < mask_words; w += blockDim.x >> 5) {
      const int k = w * 32 + lane;
      const int dropped = (k < n) ? (open ? (row[k] != 0) : 0) : 1;
      const unsigned bits = __ballot_sync(0xffffffffu, dropped);
      if (lane == 0) maskbits_lin[(int64_t)bi * mask_words + w] = bits;
    }
  }
}

// bias_pad[b, h, j, 0..n_pad) = bias[b, h, j, 0..n) (pad = 0): a copy whose row pitch
// is a multiple of 16 bytes, as TMA needs, for n % 8 != 0.
__global__ void bias_pad_kernel(View4 bias, uint16_t* out, int heads, int n, int n_pad) {
  const int bh = blockIdx.z, b = bh / heads, h = bh % heads;
  const int j = blockIdx.y;
  const uint16_t* src = (const uint16_t*)bias.p + b * bias.sb + h * bias.sh + (int64_t)j * bias.sj;
  uint16_t* dst = out + ((int64_t)bh * n + j) * n_pad;
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < n_pad; k += gridDim.x * blockDim.x)
    dst[k] = (k < n) ? src[k] : (uint16_t)0;
}

// ---------------------------------------------------------------------------
// delta[b, h, i, j] = sum_d o * dO   (fp32; never rounded to the input dtype)
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void delta_kernel(View5 o, View5 d_o, const float* lse, float* delta, float* neg_lse2,
                             Dims dm) {
  // A group of G threads owns one (b, h, i, j) row of D elements, 16 bytes per thread
  // and step, so that a warp reads whole 128-byte lines of o and dO.
  constexpr int kVec = 16 / sizeof(T);   // elements per 16-byte load
  constexpr int G = (D / kVec) < 4 ? (D / kVec) : 4;
  constexpr int kSteps = D / (kVec * G);
  const int64_t total = (int64_t)dm.batch * dm.heads * dm.n_rows * dm.n;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t idx = gid / G;
  const int part = (int)(gid % G);
  const bool valid = idx < total;
  float acc = 0.f;
  if (valid) {
    const int j = idx % dm.n;
    int64_t r = idx / dm.n;
    const int i = r % dm.n_rows;
    r /= dm.n_rows;
    const int h = r % dm.heads, b = r / dm.heads;
    const T* po = row5<T>(o, b, h, i, j);
    const T* pd = row5<T>(d_o, b, h, i, j);
#pragma unroll
    for (int st = 0; st < kSteps; ++st) {
      const int off = (st * G + part) * kVec;
      const uint4 uo = *reinterpret_cast<const uint4*>(po + off);
      const uint4 ud = *reinterpret_cast<const uint4*>(pd + off);
      const T* eo = reinterpret_cast<const T*>(&uo);
      const T* ed = reinterpret_cast<const T*>(&ud);
#pragma unroll
      for (int c = 0; c < kVec; ++c) acc = fmaf(to_f32<T>(eo[c]), to_f32<T>(ed[c]), acc);
    }
  }
#pragma unroll
  for (int m = G / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (valid && part == 0) {
    const int64_t out = (idx / dm.n) * dm.n_pad + idx % dm.n;  // row pitch n_pad
    delta[out] = acc;
    neg_lse2[out] = -lse[idx] * 1.4426950408889634f;
  }
}

// bias_t[b, h, k, j] = bias[b, h, j, k] (row pitch n_pad) for 2-byte elements (the dk/dv kernel reads
// the bias with keys on the rows).  64 x 64 tiles; 4-byte accesses on both sides when the rows allow it.
__global__ void __launch_bounds__(256)
bias_transpose_kernel(View4 bias, uint16_t* out, int heads, int n, int n_pad) {
  __shared__ uint16_t tile[64][66];
  const int bh = blockIdx.z, b = bh / heads, h = bh % heads;
  const uint16_t* src = (const uint16_t*)bias.p + b * bias.sb + h * bias.sh;
  uint16_t* dst = out + (int64_t)bh * n * n_pad;
  const int j0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const bool pairs_in = (bias.sj % 2 == 0) && (bias.sh % 2 == 0) && (bias.sb % 2 == 0) &&
                        ((reinterpret_cast<uintptr_t>(bias.p) & 3) == 0);
  for (int r = ty; r < 64; r += 8) {
    const int j = j0 + r, k = k0 + 2 * tx;
    if (j < n) {
      if (pairs_in && k + 1 < n) {
        const uint32_t u = *reinterpret_cast<const uint32_t*>(src + (int64_t)j * bias.sj + k);
        tile[r][2 * tx] = (uint16_t)(u & 0xffffu);
        tile[r][2 * tx + 1] = (uint16_t)(u >> 16);
      } else {
        if (k < n) tile[r][2 * tx] = src[(int64_t)j * bias.sj + k];
        if (k + 1 < n) tile[r][2 * tx + 1] = src[(int64_t)j * bias.sj + k + 1];
      }
    }
  }
  __syncthreads();
  for (int r = ty; r < 64; r += 8) {  // output row k0 + r holds queries j0 .. j0 + 63
    const int k = k0 + r, j = j0 + 2 * tx;
    if (k < n) {
      if (j + 1 < n) {  // n_pad is even and dst 4-byte aligned: a pair never straddles
        const uint32_t u = (uint32_t)tile[2 * tx][r] | ((uint32_t)tile[2 * tx + 1][r] << 16);
        *reinterpret_cast<uint32_t*>(dst + (int64_t)k * n_pad + j) = u;
      } else if (j < n) {
        dst[(int64_t)k * n_pad + j] = tile[2 * tx][r];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename T, int D, int BJ, int BK>
__global__ void __launch_bounds__(BJ) simt_fwd_kernel(View5 q, View5 k, View5 v, View4 bias,
                                                      MaskView mask, View5 o, float* lse,
                                                      Dims dm) {
  __shared__ __align__(16) float Ks[BK][D];
  __shared__ __align__(16) float Vs[BK][D];
  __shared__ uint8_t Ms[BK];
  const int n = dm.n;
  const int i = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  const int tid = threadIdx.x;
  const int j = blockIdx.x * BJ + tid;
  const bool jvalid = j < n;

  const uint8_t* mrow = mask.p + b * mask.sb + (int64_t)i * mask.si;
  int open = 0;
  for (int kk = tid; kk < n; kk += BJ) open |= (mrow[kk] == 0);
  const bool row_full = !__syncthreads_or(open);

  float qr[D], acc[D];
#pragma unroll
  for (int c = 0; c < D; ++c) acc[c] = 0.f;
  {
    const T* pq = row5<T>(q, b, h, i, jvalid ? j : 0);
#pragma unroll
    for (int c = 0; c < D; ++c) qr[c] = jvalid ? to_f32<T>(pq[c]) : 0.f;
  }
  const T* brow = row4<T>(bias, b, h, jvalid ? j : 0);
  float m = kMaxInit, l = 0.f;

  for (int k0 = 0; k0 < n; k0 += BK) {
    __syncthreads();
    const int valid = min(BK, n - k0);
    stage_tile<T, D, BK, BJ>(Ks, valid, [&](int r) { return row5<T>(k, b, h, i, k0 + r); });
    stage_tile<T, D, BK, BJ>(Vs, valid, [&](int r) { return row5<T>(v, b, h, i, k0 + r); });
    for (int t = tid; t < BK; t += BJ) Ms[t] = (t < valid) ? (row_full ? 0 : mrow[k0 + t]) : 1;
    __syncthreads();

    float sc[BK];
    float mt = kMinusInf;
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float x = dot_smem<D>(qr, Ks[kk]);
      const float bv = (kk < valid && jvalid) ? to_f32<T>(brow[k0 + kk]) : 0.f;
      x = row_full ? 0.f : fmaf(x, dm.scale, bv);
      if (Ms[kk]) x = kMinusInf;
      sc[kk] = x;
      mt = fmaxf(mt, x);
    }
    const float m_new = fmaxf(m, mt);
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int c = 0; c < D; ++c) acc[c] *= alpha;
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float p = expf(sc[kk] - m_new);
      l += p;
      axpy_smem<D>(p, Vs[kk], acc);
    }
    m = m_new;
  }
  if (jvalid) {
    const float inv = 1.f / l;
    T* po = row5w<T>(o, b, h, i, j);
#pragma unroll
    for (int c = 0; c < D; ++c) po[c] = from_f32<T>(acc[c] * inv);
    lse[(((int64_t)b * dm.heads + h) * dm.n_rows + i) * n + j] =
        row_full ? dm.sentinel : m + logf(l);
  }
}

// ---------------------------------------------------------------------------
// dq: thread per query j.
// ---------------------------------------------------------------------------
template <typename T, int D, int BJ, int BK>
__global__ void __launch_bounds__(BJ) simt_dq_kernel(View5 q, View5 k, View5 v, View4 bias,
                                                     MaskView mask, View5 d_o, View5 dq,
                                                     const float* lse, const float* delta,
                                                     const uint8_t* rowfull, Dims dm) {
  __shared__ __align__(16) float Ks[BK][D];
  __shared__ __align__(16) float Vs[BK][D];
  __shared__ uint8_t Ms[BK];
  const int n = dm.n;
  const int i = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  const int tid = threadIdx.x;
  const int j = blockIdx.x * BJ + tid;
  const bool jvalid = j < n;
  const bool row_full = rowfull[b * dm.n_rows + i] != 0;
  const float uniform = 1.f / (float)n;
  const uint8_t* mrow = mask.p + b * mask.sb + (int64_t)i * mask.si;

  float qr[D], gr[D], acc[D];
  {
    const T* pq = row5<T>(q, b, h, i, jvalid ? j : 0);
    const T* pg = row5<T>(d_o, b, h, i, jvalid ? j : 0);
#pragma unroll
    for (int c = 0; c < D; ++c) {
      qr[c] = jvalid ? to_f32<T>(pq[c]) : 0.f;
      gr[c] = jvalid ? to_f32<T>(pg[c]) : 0.f;
      acc[c] = 0.f;
    }
  }
  const int64_t stat = (((int64_t)b * dm.heads + h) * dm.n_rows + i) * n + (jvalid ? j : 0);
  const float my_lse = lse[stat];
  const float my_delta =
      delta[(((int64_t)b * dm.heads + h) * dm.n_rows + i) * dm.n_pad + (jvalid ? j : 0)];
  const T* brow = row4<T>(bias, b, h, jvalid ? j : 0);

  for (int k0 = 0; k0 < n; k0 += BK) {
    __syncthreads();
    const int valid = min(BK, n - k0);
    stage_tile<T, D, BK, BJ>(Ks, valid, [&](int r) { return row5<T>(k, b, h, i, k0 + r); });
    stage_tile<T, D, BK, BJ>(Vs, valid, [&](int r) { return row5<T>(v, b, h, i, k0 + r); });
    for (int t = tid; t < BK; t += BJ) Ms[t] = (t < valid) ? (row_full ? 0 : mrow[k0 + t]) : 1;
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < BK; ++kk) {
      float p;
      if (Ms[kk]) {
        p = 0.f;
      } else if (row_full) {
        p = uniform;
      } else {
        const float s = dot_smem<D>(qr, Ks[kk]);
        const float bv = jvalid ? to_f32<T>(brow[k0 + kk]) : 0.f;
        p = expf(fmaf(s, dm.scale, bv) - my_lse);
      }
      const float dp = dot_smem<D>(gr, Vs[kk]);
      const float ds = p * (dp - my_delta);
      axpy_smem<D>(ds, Ks[kk], acc);
    }
  }
  if (jvalid) {
    T* pdq = row5w<T>(dq, b, h, i, j);
#pragma unroll
    for (int c = 0; c < D; ++c) pdq[c] = from_f32<T>(acc[c] * dm.scale);
  }
}

// ---------------------------------------------------------------------------
// dk, dv: thread per key k.
// ---------------------------------------------------------------------------
template <typename T, int D, int BKT, int BJT>
__global__ void __launch_bounds__(BKT) simt_dkv_kernel(View5 q, View5 k, View5 v, View4 bias,
                                                       MaskView mask, View5 d_o, View5 dk,
                                                       View5 dv, const float* lse,
                                                       const float* delta,
                                                       const uint8_t* rowfull, Dims dm) {
  __shared__ __align__(16) float Qs[BJT][D];
  __shared__ __align__(16) float Gs[BJT][D];
  __shared__ float Ls[BJT], Ds[BJT];
  const int n = dm.n;
  const int i = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  const int tid = threadIdx.x;
  const int key = blockIdx.x * BKT + tid;
  const bool kvalid = key < n;
  const bool row_full = rowfull[b * dm.n_rows + i] != 0;
  const float uniform = 1.f / (float)n;
  const bool masked =
      !kvalid || (!row_full && mask.p[b * mask.sb + (int64_t)i * mask.si + key] != 0);

  float kr[D], vr[D], acck[D], accv[D];
  {
    const T* pk = row5<T>(k, b, h, i, kvalid ? key : 0);
    const T* pv = row5<T>(v, b, h, i, kvalid ? key : 0);
#pragma unroll
    for (int c = 0; c < D; ++c) {
      kr[c] = kvalid ? to_f32<T>(pk[c]) : 0.f;
      vr[c] = kvalid ? to_f32<T>(pv[c]) : 0.f;
      acck[c] = 0.f;
      accv[c] = 0.f;
    }
  }
  const int64_t stat0 = (((int64_t)b * dm.heads + h) * dm.n_rows + i) * n;

  for (int j0 = 0; j0 < n; j0 += BJT) {
    __syncthreads();
    const int valid = min(BJT, n - j0);
    stage_tile<T, D, BJT, BKT>(Qs, valid, [&](int r) { return row5<T>(q, b, h, i, j0 + r); });
    stage_tile<T, D, BJT, BKT>(Gs, valid, [&](int r) { return row5<T>(d_o, b, h, i, j0 + r); });
    for (int t = tid; t < BJT; t += BKT) {
      Ls[t] = (t < valid) ? lse[stat0 + j0 + t] : 0.f;
      Ds[t] = (t < valid) ? delta[stat0 / n * dm.n_pad + j0 + t] : 0.f;
    }
    __syncthreads();
    if (masked) continue;  // exactly zero weight: no contribution to dk, dv
    for (int jj = 0; jj < valid; ++jj) {
      float p;
      if (row_full) {
        p = uniform;
      } else {
        const float s = dot_smem<D>(kr, Qs[jj]);
        const float bv = to_f32<T>(row4<T>(bias, b, h, j0 + jj)[key]);
        p = expf(fmaf(s, dm.scale, bv) - Ls[jj]);
      }
      const float dp = dot_smem<D>(vr, Gs[jj]);
      const float ds = p * (dp - Ds[jj]);
      axpy_smem<D>(p, Gs[jj], accv);
      axpy_smem<D>(ds, Qs[jj], acck);
    }
  }
  if (kvalid) {
    T* pdk = row5w<T>(dk, b, h, i, key);
    T* pdv = row5w<T>(dv, b, h, i, key);
#pragma unroll
    for (int c = 0; c < D; ++c) {
      pdk[c] = from_f32<T>(acck[c] * dm.scale);
      pdv[c] = from_f32<T>(accv[c]);
    }
  }
}

// ---------------------------------------------------------------------------
// dq and dk / dv for head dim 128: a row of 128 floats per operand and accumulator does not
// fit the registers of one thread (the kernels above spill 8-10 KB per thread there), so G = 4
// neighbouring lanes share a query (a key): lane p of the group owns the 16-byte chunks
// p, p + 4, p + 8, ... of every row (neighbouring lanes read neighbouring chunks of a
// shared-memory row: no bank conflicts), the partial dot products are summed over the group
// with two shuffles, and every lane then holds the score.
// ---------------------------------------------------------------------------
template <int D, int G>
struct GroupCols {
  static constexpr int kChunks = D / (4 * G);   // 16-byte chunks per lane
  static constexpr int kFloats = 4 * kChunks;
};

template <typename T, int D, int G>
__device__ __forceinline__ void load_part(const T* row, int part, bool valid, float* reg) {
#pragma unroll
  for (int ci = 0; ci < GroupCols<D, G>::kChunks; ++ci) {
    const int c0 = (ci * G + part) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) reg[4 * ci + e] = valid ? to_f32<T>(row[c0 + e]) : 0.f;
  }
}

template <int D, int G>
__device__ __forceinline__ float dot_part(const float* reg, const float* sm, int part) {
  float acc = 0.f;
  const float4* s4 = reinterpret_cast<const float4*>(sm);
#pragma unroll
  for (int ci = 0; ci < GroupCols<D, G>::kChunks; ++ci) {
    const float4 x = s4[ci * G + part];
    acc = fmaf(reg[4 * ci + 0], x.x, acc);
    acc = fmaf(reg[4 * ci + 1], x.y, acc);
    acc = fmaf(reg[4 * ci + 2], x.z, acc);
    acc = fmaf(reg[4 * ci + 3], x.w, acc);
  }
  return acc;
}

template <int D, int G>
__device__ __forceinline__ void axpy_part(float a, const float* sm, int part, float* reg) {
  const float4* s4 = reinterpret_cast<const float4*>(sm);
#pragma unroll
  for (int ci = 0; ci < GroupCols<D, G>::kChunks; ++ci) {
    const float4 x = s4[ci * G + part];
    reg[4 * ci + 0] = fmaf(a, x.x, reg[4 * ci + 0]);
    reg[4 * ci + 1] = fmaf(a, x.y, reg[4 * ci + 1]);
    reg[4 * ci + 2] = fmaf(a, x.z, reg[4 * ci + 2]);
    reg[4 * ci + 3] = fmaf(a, x.w, reg[4 * ci + 3]);
  }
}

template <int G>
__device__ __forceinline__ float group_sum(float x, unsigned gmask) {
#pragma unroll
  for (int o = 1; o < G; o <<= 1) x += __shfl_xor_sync(gmask, x, o);
  return x;
}

template <typename T, int D, int G, int BJ, int BK>
__global__ void __launch_bounds__(BJ * G) simt_dq_group_kernel(View5 q, View5 k, View5 v, View4 bias,
                                                               MaskView mask, View5 d_o, View5 dq,
                                                               const float* lse, const float* delta,
                                                               const uint8_t* rowfull, Dims dm) {
  constexpr int NT = BJ * G, W = GroupCols<D, G>::kFloats;
  __shared__ __align__(16) float Ks[BK][D];
  __shared__ __align__(16) float Vs[BK][D];
  __shared__ uint8_t Ms[BK];
  const int n = dm.n;
  const int i = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  const int tid = threadIdx.x, part = tid % G;
  const unsigned gmask = ((1u << G) - 1u) << ((tid & 31) & ~(G - 1));
  const int j = blockIdx.x * BJ + tid / G;
  const bool jvalid = j < n;
  const bool row_full = rowfull[b * dm.n_rows + i] != 0;
  const float uniform = 1.f / (float)n;
  const uint8_t* mrow = mask.p + b * mask.sb + (int64_t)i * mask.si;

  float qr[W], gr[W], acc[W];
  load_part<T, D, G>(row5<T>(q, b, h, i, jvalid ? j : 0), part, jvalid, qr);
  load_part<T, D, G>(row5<T>(d_o, b, h, i, jvalid ? j : 0), part, jvalid, gr);
#pragma unroll
  for (int c = 0; c < W; ++c) acc[c] = 0.f;
  const int64_t stat = (((int64_t)b * dm.heads + h) * dm.n_rows + i) * n + (jvalid ? j : 0);
  const float my_lse = lse[stat];
  const float my_delta =
      delta[(((int64_t)b * dm.heads + h) * dm.n_rows + i) * dm.n_pad + (jvalid ? j : 0)];
  const T* brow = row4<T>(bias, b, h, jvalid ? j : 0);

  for (int k0 = 0; k0 < n; k0 += BK) {
    __syncthreads();
    const int valid = min(BK, n - k0);
    stage_tile<T, D, BK, NT>(Ks, valid, [&](int r) { return row5<T>(k, b, h, i, k0 + r); });
    stage_tile<T, D, BK, NT>(Vs, valid, [&](int r) { return row5<T>(v, b, h, i, k0 + r); });
    for (int t = tid; t < BK; t += NT) Ms[t] = (t < valid) ? (row_full ? 0 : mrow[k0 + t]) : 1;
    __syncthreads();
#pragma unroll 2
    for (int kk = 0; kk < BK; ++kk) {
      const float s = group_sum<G>(dot_part<D, G>(qr, Ks[kk], part), gmask);
      const float dp = group_sum<G>(dot_part<D, G>(gr, Vs[kk], part), gmask);
      float p;
      if (Ms[kk]) {
        p = 0.f;
      } else if (row_full) {
        p = uniform;
      } else {
        const float bv = jvalid ? to_f32<T>(brow[k0 + kk]) : 0.f;
        p = expf(fmaf(s, dm.scale, bv) - my_lse);
      }
      axpy_part<D, G>(p * (dp - my_delta), Ks[kk], part, acc);
    }
  }
  if (jvalid) {
    T* pdq = row5w<T>(dq, b, h, i, j);
#pragma unroll
    for (int ci = 0; ci < GroupCols<D, G>::kChunks; ++ci)
#pragma unroll
      for (int e = 0; e < 4; ++e) pdq[(ci * G + part) * 4 + e] = from_f32<T>(acc[4 * ci + e] * dm.scale);
  }
}

template <typename T, int D, int G, int BKT, int BJT>
__global__ void __launch_bounds__(BKT * G) simt_dkv_group_kernel(View5 q, View5 k, View5 v, View4 bias,
                                                                 MaskView mask, View5 d_o, View5 dk,
                                                                 View5 dv, const float* lse,
                                                                 const float* delta,
                                                                 const uint8_t* rowfull, Dims dm) {
  constexpr int NT = BKT * G, W = GroupCols<D, G>::kFloats;
  __shared__ __align__(16) float Qs[BJT][D];
  __shared__ __align__(16) float Gs[BJT][D];
  __shared__ float Ls[BJT], Ds[BJT];
  const int n = dm.n;
  const int i = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  const int tid = threadIdx.x, part = tid % G;
  const unsigned gmask = ((1u << G) - 1u) << ((tid & 31) & ~(G - 1));
  const int key = blockIdx.x * BKT + tid / G;
  const bool kvalid = key < n;
  const bool row_full = rowfull[b * dm.n_rows + i] != 0;
  const float uniform = 1.f / (float)n;
  const bool masked =
      !kvalid || (!row_full && mask.p[b * mask.sb + (int64_t)i * mask.si + key] != 0);

  float kr[W], vr[W], acck[W], accv[W];
  load_part<T, D, G>(row5<T>(k, b, h, i, kvalid ? key : 0), part, kvalid, kr);
  load_part<T, D, G>(row5<T>(v, b, h, i, kvalid ? key : 0), part, kvalid, vr);
#pragma unroll
  for (int c = 0; c < W; ++c) {
    acck[c] = 0.f;
    accv[c] = 0.f;
  }
  const int64_t stat0 = (((int64_t)b * dm.heads + h) * dm.n_rows + i) * n;

  for (int j0 = 0; j0 < n; j0 += BJT) {
    __syncthreads();
    const int valid = min(BJT, n - j0);
    stage_tile<T, D, BJT, NT>(Qs, valid, [&](int r) { return row5<T>(q, b, h, i, j0 + r); });
    stage_tile<T, D, BJT, NT>(Gs, valid, [&](int r) { return row5<T>(d_o, b, h, i, j0 + r); });
    for (int t = tid; t < BJT; t += NT) {
      Ls[t] = (t < valid) ? lse[stat0 + j0 + t] : 0.f;
      Ds[t] = (t < valid) ? delta[stat0 / n * dm.n_pad + j0 + t] : 0.f;
    }
    __syncthreads();
    if (masked) continue;  // exactly zero weight (the whole group: its lanes share the key)
    for (int jj = 0; jj < valid; ++jj) {
      const float s = group_sum<G>(dot_part<D, G>(kr, Qs[jj], part), gmask);
      const float dp = group_sum<G>(dot_part<D, G>(vr, Gs[jj], part), gmask);
      float p;
      if (row_full) {
        p = uniform;
      } else {
        const float bv = to_f32<T>(row4<T>(bias, b, h, j0 + jj)[key]);
        p = expf(fmaf(s, dm.scale, bv) - Ls[jj]);
      }
      axpy_part<D, G>(p, Gs[jj], part, accv);
      axpy_part<D, G>(p * (dp - Ds[jj]), Qs[jj], part, acck);
    }
  }
  if (kvalid) {
    T* pdk = row5w<T>(dk, b, h, i, key);
    T* pdv = row5w<T>(dv, b, h, i, key);
#pragma unroll
    for (int ci = 0; ci < GroupCols<D, G>::kChunks; ++ci)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pdk[(ci * G + part) * 4 + e] = from_f32<T>(acck[4 * ci + e] * dm.scale);
        pdv[(ci * G + part) * 4 + e] = from_f32<T>(accv[4 * ci + e]);
      }
  }
}

// ---------------------------------------------------------------------------
// db partials: CTA = (32 x 32 (j, k) tile, row split); 256 threads, 2 x 2 each.
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256) simt_db_kernel(View5 q, View5 k, View5 v, View4 bias,
                                                      MaskView mask, View5 d_o,
                                                      const float* lse, const float* delta,
                                                      const uint8_t* rowfull, float* out,
                                                      int splits, Dims dm) {
  // The head dim is staged in chunks of DC so the four tiles fit static shared memory.
  constexpr int TJ = 32, TK = 32, DC = (D > 64) ? 64 : D, P = DC + 1;  // +1: conflict-free row reads
  __shared__ float Qs[TJ][P], Gs[TJ][P], Ks[TK][P], Vs[TK][P];
  __shared__ float Ls[TJ], Ds[TJ];
  __shared__ uint8_t Ms[TK];
  const int n = dm.n;
  const int tiles_k = (n + TK - 1) / TK;
  const int jt = blockIdx.x / tiles_k, kt = blockIdx.x % tiles_k;
  const int split = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  const int tid = threadIdx.x;
  const int tj = (tid / 16) * 2, tk = (tid % 16) * 2;  // my 2 x 2 corner
  const int j0 = jt * TJ, k0 = kt * TK;
  const int vj = min(TJ, n - j0), vk = min(TK, n - k0);
  const float uniform = 1.f / (float)n;

  float bv[2][2], acc[2][2];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int j = j0 + tj + a, key = k0 + tk + c;
      bv[a][c] = (j < n && key < n) ? to_f32<T>(row4<T>(bias, b, h, j)[key]) : 0.f;
      acc[a][c] = 0.f;
    }

  // Rows of this split: a contiguous block, the same partition for every tile.
  const int per = (dm.n_rows + splits - 1) / splits;
  const int i_begin = split * per, i_end = min(dm.n_rows, i_begin + per);

  for (int i = i_begin; i < i_end; ++i) {
    const bool row_full = rowfull[b * dm.n_rows + i] != 0;
    const int64_t stat0 = (((int64_t)b * dm.heads + h) * dm.n_rows + i) * n;
    float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, dp[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int c0 = 0; c0 < D; c0 += DC) {
      __syncthreads();
      for (int idx = tid; idx < TJ * DC; idx += 256) {
        const int r = idx / DC, c = idx % DC;
        const bool ok = r < vj;
        Qs[r][c] = ok ? to_f32<T>(row5<T>(q, b, h, i, j0 + r)[c0 + c]) : 0.f;
        Gs[r][c] = ok ? to_f32<T>(row5<T>(d_o, b, h, i, j0 + r)[c0 + c]) : 0.f;
      }
      for (int idx = tid; idx < TK * DC; idx += 256) {
        const int r = idx / DC, c = idx % DC;
        const bool ok = r < vk;
        Ks[r][c] = ok ? to_f32<T>(row5<T>(k, b, h, i, k0 + r)[c0 + c]) : 0.f;
        Vs[r][c] = ok ? to_f32<T>(row5<T>(v, b, h, i, k0 + r)[c0 + c]) : 0.f;
      }
      if (c0 == 0) {
        if (tid < TJ) {
          Ls[tid] = (tid < vj) ? lse[stat0 + j0 + tid] : 0.f;
          Ds[tid] = (tid < vj) ? delta[stat0 / n * dm.n_pad + j0 + tid] : 0.f;
        } else if (tid < TJ + TK) {
          const int t = tid - TJ;
          Ms[t] = (t < vk) ? (row_full ? 0 : mask.p[b * mask.sb + (int64_t)i * mask.si + k0 + t]) : 1;
        }
      }
      __syncthreads();
#pragma unroll 8
      for (int c = 0; c < DC; ++c) {
        const float q0 = Qs[tj][c], q1 = Qs[tj + 1][c], g0 = Gs[tj][c], g1 = Gs[tj + 1][c];
        const float x0 = Ks[tk][c], x1 = Ks[tk + 1][c], y0 = Vs[tk][c], y1 = Vs[tk + 1][c];
        s[0][0] = fmaf(q0, x0, s[0][0]);
        s[0][1] = fmaf(q0, x1, s[0][1]);
        s[1][0] = fmaf(q1, x0, s[1][0]);
        s[1][1] = fmaf(q1, x1, s[1][1]);
        dp[0][0] = fmaf(g0, y0, dp[0][0]);
        dp[0][1] = fmaf(g0, y1, dp[0][1]);
        dp[1][0] = fmaf(g1, y0, dp[1][0]);
        dp[1][1] = fmaf(g1, y1, dp[1][1]);
      }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float p;
        if (Ms[tk + c] || tj + a >= vj) {
          p = 0.f;
        } else if (row_full) {
          p = uniform;
        } else {
          p = expf(fmaf(s[a][c], dm.scale, bv[a][c]) - Ls[tj + a]);
        }
        acc[a][c] += p * (dp[a][c] - Ds[tj + a]);
      }
  }
  float* dst = out + ((int64_t)split * dm.batch * dm.heads + bh) * n * n;
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int j = j0 + tj + a, key = k0 + tk + c;
      if (j < n && key < n) dst[(int64_t)j * n + key] = acc[a][c];
    }
}

// Sum the row-split partials in split order (fixed order => deterministic).
__global__ void db_reduce_kernel(const float* partials, float* out, int splits, int64_t count) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  float acc = partials[idx];
  for (int s = 1; s < splits; ++s) acc += partials[(int64_t)s * count + idx];
  out[idx] = acc;
}

// four elements per thread (count % 4 == 0)
__global__ void db_reduce4_kernel(const float4* partials, float4* out, int splits, int64_t count4) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count4) return;
  float4 acc = __ldg(partials + idx);
  for (int s = 1; s < splits; ++s) {  // fixed split order: deterministic
    const float4 v = __ldg(partials + (int64_t)s * count4 + idx);
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  out[idx] = acc;
}

// four keys of one row per thread (n % 4 == 0, destination rows 8-byte aligned; T is 16 bits)
template <typename T>
__global__ void db_cast4_kernel(const float4* src, View4 db, int heads, int n, int64_t count4) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count4) return;
  const int n4 = n >> 2;
  const int key = (int)(idx % n4) * 4;
  int64_t r = idx / n4;
  const int j = (int)(r % n);
  r /= n;
  const int h = (int)(r % heads), b = (int)(r / heads);
  const float4 v = __ldg(src + idx);
  T* dst = (T*)db.p + b * db.sb + h * db.sh + (int64_t)j * db.sj + key;
  const T o4[4] = {from_f32<T>(v.x), from_f32<T>(v.y), from_f32<T>(v.z), from_f32<T>(v.w)};
  *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o4);
}

template <typename T>
__global__ void db_cast_kernel(const float* src, View4 db, int heads, int n, int64_t count) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  const int key = idx % n;
  int64_t r = idx / n;
  const int j = r % n;
  r /= n;
  const int h = r % heads, b = r / heads;
  T* dst = (T*)db.p + b * db.sb + h * db.sh + (int64_t)j * db.sj;
  dst[key] = from_f32<T>(src[idx]);
}

// ---------------------------------------------------------------------------
// dispatch on (dtype, d)
// ---------------------------------------------------------------------------
template <typename F>
cudaError_t dispatch(int dtype, int d, F&& f) {
#define TRIFAST_D_CASES(T)                                 \
  switch (d) {                                             \
    case 16: f((T*)nullptr, std::integral_constant<int, 16>{}); break;   \
    case 32: f((T*)nullptr, std::integral_constant<int, 32>{}); break;   \
    case 64: f((T*)nullptr, std::integral_constant<int, 64>{}); break;   \
    case 128: f((T*)nullptr, std::integral_constant<int, 128>{}); break; \
    default: return cudaErrorInvalidValue;                 \
  }
  switch (dtype) {
    case TRIFAST_F32: TRIFAST_D_CASES(float) break;
    case TRIFAST_BF16: TRIFAST_D_CASES(__nv_bfloat16) break;
    case TRIFAST_F16: TRIFAST_D_CASES(__half) break;
    default: return cudaErrorInvalidValue;
  }
#undef TRIFAST_D_CASES
  return cudaGetLastError();
}

}  // namespace

cudaError_t simt_forward(const FwdArgs& a, cudaStream_t s) {
  const Dims& dm = a.dm;
  return dispatch(a.dtype, dm.d, [&](auto* tp, auto dc) {
    using T = std::remove_pointer_t<decltype(tp)>;
    constexpr int D = decltype(dc)::value;
    constexpr int BJ = 64, BK = (D <= 32) ? 32 : 16;
    dim3 grid((dm.n + BJ - 1) / BJ, dm.n_rows, dm.batch * dm.heads);
    simt_fwd_kernel<T, D, BJ, BK><<<grid, BJ, 0, s>>>(a.q, a.k, a.v, a.bias, a.mask, a.o, a.lse, dm);
  });
}

cudaError_t bwd_prepare(const BwdArgs& a, cudaStream_t s) {
  const Dims& dm = a.dm;
  rowfull_kernel<<<dm.batch * dm.n_rows, 128, 0, s>>>(a.mask, dm.n, dm.n_rows, a.rowfull, a.maskbits,
                                                      a.maskbits_lin, a.mask_words, a.rowrange);
  if (a.bias_t) {
    dim3 grid((dm.n + 63) / 64, (dm.n + 63) / 64, dm.batch * dm.heads);
    bias_transpose_kernel<<<grid, 256, 0, s>>>(a.bias, (uint16_t*)a.bias_t, dm.heads, dm.n,
                                                       dm.n_pad);
  }
  if (a.bias_pad) {
    dim3 grid(1, dm.n, dm.batch * dm.heads);
    bias_pad_kernel<<<grid, 256, 0, s>>>(a.bias, (uint16_t*)a.bias_pad, dm.heads, dm.n, dm.n_pad);
  }
  return dispatch(a.dtype, dm.d, [&](auto* tp, auto dc) {
    using T = std::remove_pointer_t<decltype(tp)>;
    constexpr int D = decltype(dc)::value;
    constexpr int kVec = 16 / sizeof(T);
    constexpr int G = (D / kVec) < 4 ? (D / kVec) : 4;
    const int64_t threads = (int64_t)dm.batch * dm.heads * dm.n_rows * dm.n * G;
    delta_kernel<T, D><<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(a.o, a.d_o, a.lse, a.delta,
                                                                       a.neg_lse2, dm);
  });
}

cudaError_t fwd_prepare(const FwdArgs& a, cudaStream_t s) {
  const Dims& dm = a.dm;
  // the live key-tile range of every row always; the packed masks, row flags and the padded
  // bias copy only where the workspace holds them (n % 8 != 0)
  rowfull_kernel<<<dm.batch * dm.n_rows, 128, 0, s>>>(a.mask, dm.n, dm.n_rows, a.rowfull, a.maskbits,
                                                      nullptr, a.mask_words, a.rowrange);
  if (a.bias_pad) {
    dim3 grid(1, dm.n, dm.batch * dm.heads);
    bias_pad_kernel<<<grid, 256, 0, s>>>(a.bias, (uint16_t*)a.bias_pad, dm.heads, dm.n, dm.n_pad);
  }
  return cudaGetLastError();
}

cudaError_t simt_bwd_db(const BwdArgs& a, cudaStream_t s) {
  const Dims& dm = a.dm;
  return dispatch(a.dtype, dm.d, [&](auto* tp, auto dc) {
    using T = std::remove_pointer_t<decltype(tp)>;
    constexpr int D = decltype(dc)::value;
    const int t = (dm.n + 31) / 32;
    dim3 grid(t * t, a.splits, dm.batch * dm.heads);
    float* out = a.splits > 1 ? a.db_partials : a.db_f32;
    simt_db_kernel<T, D><<<grid, 256, 0, s>>>(a.q, a.k, a.v, a.bias, a.mask, a.d_o, a.lse,
                                              a.delta, a.rowfull, out, a.splits, dm);
  });
}

cudaError_t db_reduce_splits(const BwdArgs& a, cudaStream_t s) {
  if (a.splits <= 1) return cudaSuccess;
  const int64_t count = (int64_t)a.dm.batch * a.dm.heads * a.dm.n * a.dm.n;
  if (count % 4 == 0) {  // the partials and db_f32 sit on 256-byte boundaries of the workspace
    const int64_t c4 = count / 4;
    db_reduce4_kernel<<<(unsigned)((c4 + 255) / 256), 256, 0, s>>>(
        reinterpret_cast<const float4*>(a.db_partials), reinterpret_cast<float4*>(a.db_f32), a.splits,
        c4);
    return cudaGetLastError();
  }
  db_reduce_kernel<<<(unsigned)((count + 255) / 256), 256, 0, s>>>(a.db_partials, a.db_f32,
                                                                 a.splits, count);
  return cudaGetLastError();
}

cudaError_t simt_bwd_dq(const BwdArgs& a, cudaStream_t s) {
  const Dims& dm = a.dm;
  return dispatch(a.dtype, dm.d, [&](auto* tp, auto dc) {
    using T = std::remove_pointer_t<decltype(tp)>;
    constexpr int D = decltype(dc)::value;
    constexpr int BJ = 64, BK = (D <= 32) ? 32 : 16;
    dim3 gq((dm.n + BJ - 1) / BJ, dm.n_rows, dm.batch * dm.heads);
    if constexpr (D == 128) {  // four lanes per query: a thread's rows stay in registers
      simt_dq_group_kernel<T, D, 4, BJ, BK><<<gq, BJ * 4, 0, s>>>(a.q, a.k, a.v, a.bias, a.mask, a.d_o,
                                                                  a.dq, a.lse, a.delta, a.rowfull, dm);
    } else {
      simt_dq_kernel<T, D, BJ, BK><<<gq, BJ, 0, s>>>(a.q, a.k, a.v, a.bias, a.mask, a.d_o, a.dq,
                                                     a.lse, a.delta, a.rowfull, dm);
    }
  });
}

cudaError_t simt_bwd_dkv(const BwdArgs& a, cudaStream_t s) {
  const Dims& dm = a.dm;
  return dispatch(a.dtype, dm.d, [&](auto* tp, auto dc) {
    using T = std::remove_pointer_t<decltype(tp)>;
    constexpr int D = decltype(dc)::value;
    constexpr int BKT = 64, BJT = (D <= 32) ? 32 : 16;
    dim3 gk((dm.n + BKT - 1) / BKT, dm.n_rows, dm.batch * dm.heads);
    if constexpr (D == 128) {
      simt_dkv_group_kernel<T, D, 4, BKT, BJT><<<gk, BKT * 4, 0, s>>>(
          a.q, a.k, a.v, a.bias, a.mask, a.d_o, a.dk, a.dv, a.lse, a.delta, a.rowfull, dm);
    } else {
      simt_dkv_kernel<T, D, BKT, BJT><<<gk, BKT, 0, s>>>(a.q, a.k, a.v, a.bias, a.mask, a.d_o,
                                                         a.dk, a.dv, a.lse, a.delta, a.rowfull, dm);
    }
  });
}

cudaError_t db_cast(const float* db_f32, View4 db, int dtype, int batch, int heads, int n,
                    cudaStream_t s) {
  const int64_t count = (int64_t)batch * heads * n * n;
  const bool wide = dtype != TRIFAST_F32 && n % 4 == 0 && db.sj % 4 == 0 && db.sh % 4 == 0 &&
                    db.sb % 4 == 0 && (reinterpret_cast<uintptr_t>(db.p) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(db_f32) & 15) == 0;
  if (wide) {
    const int64_t c4 = count / 4;
    const unsigned blocks4 = (unsigned)((c4 + 255) / 256);
    const float4* src = reinterpret_cast<const float4*>(db_f32);
    if (dtype == TRIFAST_BF16)
      db_cast4_kernel<__nv_bfloat16><<<blocks4, 256, 0, s>>>(src, db, heads, n, c4);
    else
      db_cast4_kernel<__half><<<blocks4, 256, 0, s>>>(src, db, heads, n, c4);
    return cudaGetLastError();
  }
  const unsigned blocks = (unsigned)((count + 255) / 256);
  switch (dtype) {
    case TRIFAST_F32: db_cast_kernel<float><<<blocks, 256, 0, s>>>(db_f32, db, heads, n, count); break;
    case TRIFAST_BF16: db_cast_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(db_f32, db, heads, n, count); break;
    case TRIFAST_F16: db_cast_kernel<__half><<<blocks, 256, 0, s>>>(db_f32, db, heads, n, count); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace trifast
