// Bias gradient db[j, k] = sum over pair rows i of dS[i, j, k] on the tensor cores.
//
// One CTA owns a 128 x 128 (j, k) tile of one (b, h) and one block of pair rows
// (a "row split"); it walks its rows, recomputing per row
//     S  = Q_i K_i^T,   dP = dO_i V_i^T        (two SS MMAs, 128 x 128 each)
//     P  = exp2(S * c + bias * log2e - lse_i * log2e),   dS = P * (dP - delta_i)
// and sums dS in fp32 registers: thread = (query row j, 64-key half), 64
// accumulators.  The partial of every row split is written as fp32 and the splits
// are added in split order afterwards, so the result is deterministic: no atomics.
//
// Warps 0-3 and 4-7: elementwise warpgroups (key halves 0 and 1); warp 8 TMA
// producer (Q, dO, K, V tiles and the -lse*log2e / delta vectors per row, NS-deep
// ring); warp 9 MMA issuer; warps 10-11 idle.  TMEM: two buffers of S [0,128) and
// dP [128,256), so the MMAs of row i+1 overlap the elementwise work of row i.
//
// Stands in for `_bwd_b` of the reference (src/trifast/triton.py:388-501), which
// loops over all rows with 16-32 wide tiles.

#include <math.h>

#include <type_traits>

#include "kernels.h"
#include "tc_common.cuh"

namespace trifast {
namespace {
using namespace tc;

constexpr float kLog2e = 1.4426950408889634f;
// Register hand-over (setmaxnreg): 384 threads launch with 168 registers each; what
// the math warpgroups gain must not exceed what the issue warpgroup releases, or
// the request blocks forever.
constexpr int kRegsIssue = 56, kRegsMath = 224;
static_assert(256 * kRegsMath + 128 * kRegsIssue <= 384 * 168, "setmaxnreg pool");

template <int D, int NS>
struct DbCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = 128 * kRowBytes;
  static constexpr int kVecBytes = 128 * 4;
  static constexpr int kStageBytes = 4 * kTileBytes + 2 * kVecBytes;   // multiple of 1024
  static constexpr int kThreads = 384;
  static constexpr uint64_t kSwz = (D == 32) ? kSwizzle64 : kSwizzle128;
  static constexpr int kSbo = 8 * kRowBytes;
  static int smem_bytes() { return 1024 + 1024 + NS * kStageBytes; }
};

template <typename T, int D, int NS>
__global__ void __launch_bounds__(384, 1)
tc_db_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
             const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
             const __grid_constant__ CUtensorMap map_nlse, const __grid_constant__ CUtensorMap map_delta,
             View4 bias, const uint8_t* __restrict__ rowfull, const uint32_t* __restrict__ maskbits,
             int mask_words, float* __restrict__ out, int splits, Dims dm, unsigned int* status) {
  using Cfg = DbCfg<D, NS>;
  constexpr int FULL = 0, EMPTY = FULL + NS, S_FULL = EMPTY + NS, S_FREE = S_FULL + 2,
                NBARS = S_FREE + 2;
  static_assert(NBARS * 8 <= 256, "barrier area");
  static_assert(Cfg::kStageBytes % 1024 == 0, "stage alignment");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 260);

  const int n = dm.n;
  constexpr uint32_t tiles_off = 1024;
  auto bar = [&](int i) -> uint32_t { return base + 8u * i; };
  auto stage_off = [&](int s) -> uint32_t { return tiles_off + s * Cfg::kStageBytes; };
  auto q_tile = [&](int s) -> uint32_t { return base + stage_off(s); };
  auto do_tile = [&](int s) -> uint32_t { return base + stage_off(s) + Cfg::kTileBytes; };
  auto k_tile = [&](int s) -> uint32_t { return base + stage_off(s) + 2 * Cfg::kTileBytes; };
  auto v_tile = [&](int s) -> uint32_t { return base + stage_off(s) + 3 * Cfg::kTileBytes; };
  auto nlse_off = [&](int s) -> uint32_t { return stage_off(s) + 4 * Cfg::kTileBytes; };
  auto delta_off = [&](int s) -> uint32_t { return nlse_off(s) + Cfg::kVecBytes; };

  if (*reinterpret_cast<volatile unsigned int*>(status) != 0u) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_k = (n + 127) / 128;
  const int jt = blockIdx.x / tiles_k, kt = blockIdx.x % tiles_k;
  const int split = blockIdx.y, bh = blockIdx.z;
  const int b = bh / dm.heads, h = bh % dm.heads;
  // Rows of this split: a contiguous block, the same partition for every tile.
  const int per = (dm.n_rows + splits - 1) / splits;
  const int i_begin = split * per;
  const int nrows = max(0, min(dm.n_rows, i_begin + per) - i_begin);

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), 1 + 8);  // MMA commit + 8 elementwise warps (vectors read)
    }
    for (int u = 0; u < 2; ++u) {
      mbar_init(bar(S_FULL + u), 1);
      mbar_init(bar(S_FREE + u), 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_do);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_nlse);
    tma_prefetch_desc(&map_delta);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
    if (warp == 8) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0) {
        for (int it = 0; it < nrows; ++it) {
          const int s = it % NS, i = i_begin + it;
          if (it >= NS && !mbar_wait(bar(EMPTY + s), ((it / NS) - 1) & 1, abort_flag)) break;
          mbar_arrive_expect_tx(bar(FULL + s), Cfg::kStageBytes);
          tma_load_5d(q_tile(s), &map_q, bar(FULL + s), 0, jt * 128, i, h, b);
          tma_load_5d(do_tile(s), &map_do, bar(FULL + s), 0, jt * 128, i, h, b);
          tma_load_5d(k_tile(s), &map_k, bar(FULL + s), 0, kt * 128, i, h, b);
          tma_load_5d(v_tile(s), &map_v, bar(FULL + s), 0, kt * 128, i, h, b);
          tma_load_4d(base + nlse_off(s), &map_nlse, bar(FULL + s), jt * 128, i, h, b);
          tma_load_4d(base + delta_off(s), &map_delta, bar(FULL + s), jt * 128, i, h, b);
        }
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t idesc = make_idesc(128, 128, kBf16, false, false);
        bool ok = true;
        for (int it = 0; it < nrows && ok; ++it) {
          const int s = it % NS, u = it & 1;
          ok = mbar_wait(bar(FULL + s), (it / NS) & 1, abort_flag);
          if (ok && it >= 2) ok = mbar_wait(bar(S_FREE + u), ((it >> 1) - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t aq = make_smem_desc(q_tile(s) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bk = make_smem_desc(k_tile(s) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            umma_ss(tmem_base + u * 256, aq, bk, idesc, kk > 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t ag = make_smem_desc(do_tile(s) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bv = make_smem_desc(v_tile(s) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            umma_ss(tmem_base + u * 256 + 128, ag, bv, idesc, kk > 0);
          }
          umma_commit(bar(S_FULL + u));
          umma_commit(bar(EMPTY + s));
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMath));
    // ------------------------------------------------------------ elementwise warpgroups
    const int half = warp >> 2, wq = warp & 3, row = tid & 127;
    const int j = jt * 128 + row;
    const int key0 = kt * 128 + half * 64;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const float c1 = dm.scale * kLog2e;
    const float uniform = 1.f / (float)n;

    float acc[64], bl[64];
    {
      const T* brow = reinterpret_cast<const T*>(bias.p) + b * bias.sb + h * bias.sh +
                      (int64_t)min(j, n - 1) * bias.sj;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        acc[c] = 0.f;
        bl[c] = (key0 + c < n) ? to_f32<T>(brow[key0 + c]) * kLog2e : 0.f;
      }
    }
    bool ok = true;
    for (int it = 0; it < nrows; ++it) {
      const int s = it % NS, u = it & 1, i = i_begin + it;
      // per-row inputs that do not come through shared memory
      const uint32_t* mrow = maskbits + ((int64_t)b * dm.n_rows + i) * mask_words + kt * 4 + half * 2;
      const uint32_t mw0 = __ldg(mrow), mw1 = __ldg(mrow + 1);
      const bool row_full = rowfull[b * dm.n_rows + i] != 0;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(FULL + s), (it / NS) & 1, abort_flag));
      if (!ok) break;
      const float nl = reinterpret_cast<const float*>(gbase + nlse_off(s))[row];
      const float dl = reinterpret_cast<const float*>(gbase + delta_off(s))[row];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(EMPTY + s));
      ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + u), (it >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tS = tmem_base + lane_base + u * 256 + half * 64;
      const uint32_t tDP = tS + 128;
#pragma unroll
      for (int hc = 0; hc < 2; ++hc) {
        float x[32], g[32];
        tmem_ld32(tS + hc * 32, reinterpret_cast<uint32_t*>(x));
        tmem_ld32(tDP + hc * 32, reinterpret_cast<uint32_t*>(g));
        tmem_wait_ld();
        const uint32_t mw = hc ? mw1 : mw0;
        if (row_full) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float p = ((mw >> c) & 1u) ? 0.f : uniform;
            acc[hc * 32 + c] = fmaf(p, g[c] - dl, acc[hc * 32 + c]);
          }
        } else if (mw == 0u) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float p = ex2(fmaf(x[c], c1, bl[hc * 32 + c]) + nl);
            acc[hc * 32 + c] = fmaf(p, g[c] - dl, acc[hc * 32 + c]);
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float p = ex2(fmaf(x[c], c1, bl[hc * 32 + c]) + nl);
            if ((mw >> c) & 1u) p = 0.f;
            acc[hc * 32 + c] = fmaf(p, g[c] - dl, acc[hc * 32 + c]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(S_FREE + u));
    }
    if (ok && j < n) {
      float* dst = out + (((int64_t)split * dm.batch * dm.heads + bh) * n + j) * n + key0;
      if (key0 + 64 <= n) {
#pragma unroll
        for (int c = 0; c < 64; c += 4)
          *reinterpret_cast<float4*>(dst + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (key0 + c < n) dst[c] = acc[c];
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (tid == 0) atomicOr(status, (unsigned int)kStatusTimeoutBwdDb);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int D, int NS>
cudaError_t launch_db(const BwdArgs& a, cudaStream_t stream) {
  using Cfg = DbCfg<D, NS>;
  const Dims& dm = a.dm;
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const uint64_t eb = 2;
  CUtensorMap mq, mdo, mk, mv, mnl, mdl;
  const uint64_t dims5[5] = {(uint64_t)D, (uint64_t)dm.n, (uint64_t)dm.n_rows, (uint64_t)dm.heads,
                             (uint64_t)dm.batch};
  const uint32_t box[5] = {(uint32_t)D, 128, 1, 1, 1};
  const CUtensorMapSwizzle swz = (D == 32) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  auto map5 = [&](CUtensorMap* m, const View5& v) {
    const uint64_t st[4] = {(uint64_t)v.sj * eb, (uint64_t)v.si * eb, (uint64_t)v.sh * eb,
                            (uint64_t)v.sb * eb};
    return make_tensor_map(m, bf16, 5, v.p, dims5, st, box, swz);
  };
  if (!map5(&mq, a.q) || !map5(&mdo, a.d_o) || !map5(&mk, a.k) || !map5(&mv, a.v))
    return cudaErrorInvalidValue;
  {
    const uint64_t n = dm.n, rows = dm.n_rows;
    const uint64_t dims4[4] = {n, rows, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st[3] = {n * 4, n * rows * 4, n * rows * dm.heads * 4};
    const uint32_t box4[4] = {128, 1, 1, 1};
    if (!make_tensor_map_f32(&mnl, 4, a.neg_lse2, dims4, st, box4) ||
        !make_tensor_map_f32(&mdl, 4, a.delta, dims4, st, box4))
      return cudaErrorInvalidValue;
  }
  const int smem = Cfg::smem_bytes();
  auto kern = tc_db_kernel<T, D, NS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  const int t = (dm.n + 127) / 128;
  dim3 grid(t * t, a.splits, dm.batch * dm.heads);
  float* out = a.splits > 1 ? a.db_partials : a.db_f32;
  kern<<<grid, Cfg::kThreads, smem, stream>>>(mq, mdo, mk, mv, mnl, mdl, a.bias, a.rowfull,
                                              a.maskbits, a.mask_words, out, a.splits, dm, a.status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_bwd_db(const BwdArgs& a, cudaStream_t s) {
  const bool bf16 = a.dtype == TRIFAST_BF16;
  if (!a.neg_lse2 || !a.maskbits) return cudaErrorInvalidValue;
  if (a.dm.d == 32)
    return bf16 ? launch_db<__nv_bfloat16, 32, 4>(a, s) : launch_db<__half, 32, 4>(a, s);
  return bf16 ? launch_db<__nv_bfloat16, 64, 3>(a, s) : launch_db<__half, 64, 3>(a, s);
}

}  // namespace trifast
