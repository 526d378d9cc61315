// Bias gradient db[j, k] = sum over pair rows i of dS[i, j, k] on the tensor cores.
//
// A work item is a 128 x 128 (j, k) tile of one (b, h) and one block of pair rows
// (a "row split"); every CTA works on exactly one item (blockIdx.x).  Per row of its item the CTA
// recomputes
//     S  = Q_i K_i^T,   dP = dO_i V_i^T        (two SS MMAs, 128 x 128 each)
//     P  = exp2(S * c + bias * log2e - lse_i * log2e),   dS = P * (dP - delta_i)
// and sums dS in fp32 registers: thread = (query row j, 32-key quarter), 32
// accumulators.  The partial of every row split is written as fp32 and the splits
// are added in split order afterwards, so the result is deterministic: no atomics.
//
// Warps 0-15: four elementwise warpgroups, one per 32-key quarter of the tile, so
// that four warps per scheduler cover each other's barrier, TMEM-load and MUFU
// latencies; warp 16 TMA producer (Q, dO, K, V tiles and the -lse*log2e / delta
// vectors per row, NS-deep ring); warp 17 MMA issuer; warps 18-19 idle.  TMEM: two buffers of S [0,128) and
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
// Register hand-over (setmaxnreg): 640 threads launch with 96 registers each; what
// the math warpgroups gain must not exceed what the issue warpgroup releases (the
// registers a CTA did not get at launch are not part of the pool), or the request
// blocks forever.
constexpr int kRegsLaunch = 96, kRegsIssue = 32, kRegsMath = 112;
static_assert(512 * kRegsMath + 128 * kRegsIssue <= 640 * kRegsLaunch, "setmaxnreg pool");
constexpr int kTmaWarp = 16, kMmaWarp = 17;

template <int D, int NS>
struct DbCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = 128 * kRowBytes;
  static constexpr int kVecBytes = 128 * 4;
  static constexpr int kStageBytes = 4 * kTileBytes + 2 * kVecBytes;   // multiple of 1024
  static constexpr int kThreads = 640;
  static constexpr uint64_t kSwz = RowSwizzle<D>::kDesc;
  static constexpr int kSbo = 8 * kRowBytes;
  static constexpr int kLiveBytes = 8192;   // one bit per row of the split (n_rows <= 65535)
  static int smem_bytes() { return 1024 + 1024 + NS * kStageBytes + kLiveBytes; }
};

template <typename T, int D, int NS>
__global__ void __launch_bounds__(640, 1)
tc_db_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
             const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
             const __grid_constant__ CUtensorMap map_nlse, const __grid_constant__ CUtensorMap map_delta,
             View4 bias, const uint8_t* __restrict__ rowfull, const uint32_t* __restrict__ maskbits,
             int mask_words, const uint32_t* __restrict__ rowrange, float* __restrict__ out,
             int splits, Dims dm, unsigned int* status) {
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
  const int tiles = tiles_k * tiles_k;
  // Rows of a split: a contiguous block, the same partition for every tile.
  const int per = (dm.n_rows + splits - 1) / splits;
  struct Item {
    int jt, kt, split, bh, b, h, i_begin, nrows;
  };
  // item order: tile fastest, then split, then (b, h): the CTAs running together work
  // on the same rows of the same (b, h), so the Q/dO/K/V row tiles are shared in L2
  auto decode = [&](int w) {
    Item im;
    const int tile = w % tiles;
    const int rest = w / tiles;
    im.jt = tile / tiles_k;
    im.kt = tile % tiles_k;
    im.split = rest % splits;
    im.bh = rest / splits;
    im.b = im.bh / dm.heads;
    im.h = im.bh % dm.heads;
    im.i_begin = im.split * per;
    im.nrows = max(0, min(dm.n_rows, im.i_begin + per) - im.i_begin);
    return im;
  };

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), 1 + 16);  // MMA commit + 16 elementwise warps (vectors read)
    }
    for (int u = 0; u < 2; ++u) {
      mbar_init(bar(S_FULL + u), 1);
      mbar_init(bar(S_FREE + u), 16);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  // Rows of this split whose live key-tile range holds this item's key tile, one bit per
  // row: the others weigh all 128 keys of the tile zero and add nothing to db, so no role
  // touches them.  (A fully masked row's range is every tile.)
  uint32_t* live = reinterpret_cast<uint32_t*>(gbase + tiles_off + NS * Cfg::kStageBytes);
  {
    const Item im = decode(blockIdx.x);
    for (int w0 = warp * 32; w0 < im.nrows; w0 += 32 * (Cfg::kThreads / 32)) {
      const int g = w0 + lane;
      bool on = false;
      if (g < im.nrows) {
        const uint32_t v = rowrange ? __ldg(rowrange + im.b * dm.n_rows + im.i_begin + g) : 0xffff0000u;
        on = (uint32_t)im.kt >= (v & 0xffffu) && (uint32_t)im.kt < (v >> 16);
      }
      const uint32_t bits = __ballot_sync(0xffffffffu, on);
      if (lane == 0) live[w0 >> 5] = bits;
    }
  }
  // (the roles walk the set bits word by word: one shared-memory read per 32 rows, nothing
  // per row)
  if (warp == kTmaWarp && lane == 0) {
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

  if (warp >= kTmaWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
    if (warp == kTmaWarp) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0) {
        const Item im = decode(blockIdx.x);
        int g = 0;
        bool stop = false;
        for (int r0 = 0; r0 < im.nrows && !stop; r0 += 32) {
        for (uint32_t bits = live[r0 >> 5]; bits != 0u; bits &= bits - 1u) {
          {
            const int s = g % NS, i = im.i_begin + r0 + __ffs(bits) - 1;
            if (g >= NS && !mbar_wait(bar(EMPTY + s), ((g / NS) - 1) & 1, abort_flag)) {
              stop = true;
              break;
            }
            mbar_arrive_expect_tx(bar(FULL + s), Cfg::kStageBytes);
            tma_load_5d(q_tile(s), &map_q, bar(FULL + s), 0, im.jt * 128, i, im.h, im.b);
            tma_load_5d(do_tile(s), &map_do, bar(FULL + s), 0, im.jt * 128, i, im.h, im.b);
            tma_load_5d(k_tile(s), &map_k, bar(FULL + s), 0, im.kt * 128, i, im.h, im.b);
            tma_load_5d(v_tile(s), &map_v, bar(FULL + s), 0, im.kt * 128, i, im.h, im.b);
            tma_load_4d(base + nlse_off(s), &map_nlse, bar(FULL + s), im.jt * 128, i, im.h, im.b);
            tma_load_4d(base + delta_off(s), &map_delta, bar(FULL + s), im.jt * 128, i, im.h, im.b);
          }
          ++g;
        }
        }
      }
    } else if (warp == kMmaWarp) {
      // ---------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t idesc = make_idesc(128, 128, kBf16, false, false);
        bool ok = true;
        {
          const int nrows = decode(blockIdx.x).nrows;
          int g = 0;
          for (int r0 = 0; r0 < nrows && ok; r0 += 32) {
          for (uint32_t bits = live[r0 >> 5]; bits != 0u && ok; bits &= bits - 1u) {
            const int s = g % NS, u = g & 1;
            ok = mbar_wait(bar(FULL + s), (g / NS) & 1, abort_flag);
            if (ok && g >= 2) ok = mbar_wait(bar(S_FREE + u), ((g >> 1) - 1) & 1, abort_flag);
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
            ++g;
          }
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMath));
    // ------------------------------------------------------------ elementwise warpgroups
    const int quarter = warp >> 2, wq = warp & 3, row = tid & 127;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const float c1 = dm.scale * kLog2e;
    const float uniform = 1.f / (float)n;

    bool ok = true;
    {
      const Item im = decode(blockIdx.x);
      const int b = im.b, h = im.h, kt = im.kt;
      const int j = im.jt * 128 + row;
      const int key0 = kt * 128 + quarter * 32;

      // where this thread's 32 sums go, settled now so that the item's indices need not
      // stay live through the row loop
      float* const dst =
          out + (((int64_t)im.split * dm.batch * dm.heads + im.bh) * n + min(j, n - 1)) * n + key0;
      const int n_store = (j < n) ? min(32, n - key0) : 0;  // <= 0: nothing to store

      float acc[32];
      uint32_t bp[16];  // this thread's 32 bias values, kept as 16-bit pairs
      {
        const T* brow = reinterpret_cast<const T*>(bias.p) + b * bias.sb + h * bias.sh +
                        (int64_t)min(j, n - 1) * bias.sj + key0;
#pragma unroll
        for (int c = 0; c < 32; ++c) acc[c] = 0.f;
        if (key0 + 32 <= n && (reinterpret_cast<uintptr_t>(brow) & 15) == 0) {
          // four 16-byte loads: a lane reads its own row, so every load instruction
          // touches 32 lines; 2-byte loads would take 32 such instructions
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 u = __ldg(reinterpret_cast<const uint4*>(brow) + c);
            bp[4 * c + 0] = u.x;
            bp[4 * c + 1] = u.y;
            bp[4 * c + 2] = u.z;
            bp[4 * c + 3] = u.w;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float b0 = (key0 + c < n) ? to_f32<T>(brow[c]) : 0.f;
            const float b1 = (key0 + c + 1 < n) ? to_f32<T>(brow[c + 1]) : 0.f;
            bp[c >> 1] = pack2<T>(b0, b1);  // exact: the values are 16-bit already
          }
        }
      }
      int g = 0;
      for (int r0 = 0; r0 < im.nrows && ok; r0 += 32) {
      for (uint32_t bits = live[r0 >> 5]; bits != 0u; bits &= bits - 1u) {
        const int s = g % NS, u = g & 1, i = im.i_begin + r0 + __ffs(bits) - 1;
        // per-row inputs that do not come through shared memory (consumed after the
        // barrier waits below, which hide their latency)
        const uint32_t mw =
            __ldg(maskbits + ((int64_t)b * dm.n_rows + i) * mask_words + kt * 4 + quarter);
        const bool row_full = rowfull[b * dm.n_rows + i] != 0;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(FULL + s), (g / NS) & 1, abort_flag));
        if (!ok) break;
        const float nl = reinterpret_cast<const float*>(gbase + nlse_off(s))[row];
        const float dl = reinterpret_cast<const float*>(gbase + delta_off(s))[row];
        const float ndl = -dl;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(EMPTY + s));
        ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + u), (g >> 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t tS = tmem_base + lane_base + u * 256 + quarter * 32;
        const uint32_t tDP = tS + 128;
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          float x[16], gd[16];
          tmem_ld16(tS + hc * 16, reinterpret_cast<uint32_t*>(x));
          tmem_ld16(tDP + hc * 16, reinterpret_cast<uint32_t*>(gd));
          tmem_wait_ld();
          if (hc == 1) {  // everything this warp needs from the buffer is in registers
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(S_FREE + u));
          }
          const uint32_t mh = (mw >> (hc * 16)) & 0xffffu;
          if (row_full) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const float p = ((mh >> c) & 1u) ? 0.f : uniform;
              acc[hc * 16 + c] = fmaf(p, gd[c] - dl, acc[hc * 16 + c]);
            }
          } else if (mh == 0u) {  // no dropped key: a straight block the compiler can overlap
#pragma unroll
            for (int c = 0; c < 16; c += 2) {  // packed fp32 pairs: two scores per FMA instruction
              float b0, b1, t0, t1, a0, a1, s0, s1;
              unpack2<T>(bp[(hc * 16 + c) >> 1], b0, b1);
              ffma2(t0, t1, b0, b1, kLog2e, kLog2e, nl, nl);
              ffma2(a0, a1, x[c], x[c + 1], c1, c1, t0, t1);
              const float p0 = ex2(a0), p1 = ex2(a1);
              fadd2(s0, s1, gd[c], gd[c + 1], ndl, ndl);
              ffma2(acc[hc * 16 + c], acc[hc * 16 + c + 1], p0, p1, s0, s1, acc[hc * 16 + c],
                    acc[hc * 16 + c + 1]);
            }
          } else {
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
              float b0, b1, t0, t1, a0, a1, s0, s1;
              unpack2<T>(bp[(hc * 16 + c) >> 1], b0, b1);
              ffma2(t0, t1, b0, b1, kLog2e, kLog2e, nl, nl);
              ffma2(a0, a1, x[c], x[c + 1], c1, c1, t0, t1);
              float p0 = ex2(a0), p1 = ex2(a1);
              p0 = ((mh >> c) & 1u) ? 0.f : p0;
              p1 = ((mh >> (c + 1)) & 1u) ? 0.f : p1;
              fadd2(s0, s1, gd[c], gd[c + 1], ndl, ndl);
              ffma2(acc[hc * 16 + c], acc[hc * 16 + c + 1], p0, p1, s0, s1, acc[hc * 16 + c],
                    acc[hc * 16 + c + 1]);
            }
          }
        }
        ++g;
      }
      }
      if (ok && n_store > 0) {
        if (n_store == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(dst + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (c < n_store) dst[c] = acc[c];
        }
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
  if (warp == kMmaWarp) {
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
  const CUtensorMapSwizzle swz = (CUtensorMapSwizzle)RowSwizzle<D>::kTma;
  auto map5 = [&](CUtensorMap* m, const View5& v) {
    const uint64_t st[4] = {(uint64_t)v.sj * eb, (uint64_t)v.si * eb, (uint64_t)v.sh * eb,
                            (uint64_t)v.sb * eb};
    return make_tensor_map(m, bf16, 5, v.p, dims5, st, box, swz);
  };
  if (!map5(&mq, a.q) || !map5(&mdo, a.d_o) || !map5(&mk, a.k) || !map5(&mv, a.v))
    return cudaErrorInvalidValue;
  {
    const uint64_t n = dm.n, np = dm.n_pad, rows = dm.n_rows;
    const uint64_t dims4[4] = {n, rows, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st[3] = {np * 4, np * rows * 4, np * rows * dm.heads * 4};
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
  const int total = t * t * a.splits * dm.batch * dm.heads;
  const int grid = total;  // one item per CTA
  float* out = a.splits > 1 ? a.db_partials : a.db_f32;
  View4 bias = a.bias;
  if (a.bias_pad) {  // the copy with a 16-byte row pitch: its rows can be read 16 bytes at a time
    bias.p = (char*)a.bias_pad;
    bias.sj = dm.n_pad;
    bias.sh = (int64_t)dm.n * dm.n_pad;
    bias.sb = bias.sh * dm.heads;
  }
  kern<<<grid, Cfg::kThreads, smem, stream>>>(mq, mdo, mk, mv, mnl, mdl, bias, a.rowfull,
                                              a.maskbits_lin, a.mask_words, a.rowrange, out, a.splits,
                                              dm, a.status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_bwd_db(const BwdArgs& a, cudaStream_t s) {
  const bool bf16 = a.dtype == TRIFAST_BF16;
  if (!a.neg_lse2 || !a.maskbits_lin) return cudaErrorInvalidValue;
  if (a.dm.d == 16)
    return bf16 ? launch_db<__nv_bfloat16, 16, 4>(a, s) : launch_db<__half, 16, 4>(a, s);
  if (a.dm.d == 32)
    return bf16 ? launch_db<__nv_bfloat16, 32, 4>(a, s) : launch_db<__half, 32, 4>(a, s);
  return bf16 ? launch_db<__nv_bfloat16, 64, 3>(a, s) : launch_db<__half, 64, 3>(a, s);
}

}  // namespace trifast
