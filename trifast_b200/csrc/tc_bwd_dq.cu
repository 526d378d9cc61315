// dq of triangle attention on the tensor cores (bf16 / fp16).
//
// Same decomposition as the forward: a work item is a 128-query tile of two
// consecutive pair rows ("slots", sharing the bias tiles) walked over the keys in
// tiles of 64; CTAs are persistent (one per SM, looping over items) so the loads of
// the next item overlap the tail of the current one.  Per slot and key tile:
//     S  = Q K^T          (SS MMA, 128 x 64)      dP = dO V^T        (SS MMA, 128 x 64)
//     P  = exp2(S * c + bias * log2e - lse * log2e)   (recomputed from the saved lse)
//     dS = P * (dP - delta)  -> 16-bit -> TMEM
//     dQ += dS K          (A = dS from TMEM, B = K as an MN-major tile)
// and at the end dq = dQ * d^-0.5.
//
// Warps: 0-7 two elementwise warpgroups (thread = query row), 8 TMA producer,
// 9-10 MMA issuers (one per slot, so a slot never queues behind the other's waits),
// 11 idle (it completes the warpgroup whose registers are handed over with setmaxnreg).  TMEM columns per slot r (base r * 256):
// S [0,64), dP [64,128), dS [128,160) as 16-bit pairs, dQ [160, 160 + D).
//
// Stands in for `_bwd_q` of the reference (src/trifast/triton.py:268-383); delta
// comes from the fp32 workspace instead of being computed here and stored in the
// input dtype.  Masked keys get exactly zero weight; rows whose keys are all
// masked use P = 1/n (the PyTorch semantics, src/trifast/equiv.py:42-69).

#include <math.h>

#include <type_traits>

#include "kernels.h"
#include "tc_common.cuh"

namespace trifast {
namespace {
using namespace tc;

constexpr int kBJ = 128, kBK = 64;
#ifndef TRIFAST_DQ_TOKEN
#define TRIFAST_DQ_TOKEN 0
#endif
constexpr bool kSlotToken = TRIFAST_DQ_TOKEN != 0;
constexpr float kLog2e = 1.4426950408889634f;
// Register hand-over (setmaxnreg): 384 threads launch with 168 registers each; what
// the math warpgroups gain must not exceed what the issue warpgroup releases, or
// the request blocks forever.
constexpr int kRegsIssue = 56, kRegsMath = 224;
static_assert(256 * kRegsMath + 128 * kRegsIssue <= 384 * 168, "setmaxnreg pool");

template <int D, int NS>
struct DqCfg {
  static constexpr int R = 2;
  static constexpr int kRowBytes = D * 2;
  static constexpr int kQBytes = 128 * kRowBytes;         // Q or dO tile
  static constexpr int kKBytes = kBK * kRowBytes;         // K or V tile
  static constexpr int kBiasBytes = 128 * kBK * 2;        // [128 x 64] box, 128-byte rows
  static constexpr int kStageBytes = 2 * R * kKBytes + kBiasBytes;
  static constexpr int kTilesBytes = 2 * R * kQBytes + NS * kStageBytes;
  static constexpr int kThreads = R * 128 + 128;
  static constexpr uint64_t kSwz = (D == 32) ? kSwizzle64 : kSwizzle128;
  static constexpr int kSbo = 8 * kRowBytes;
  static int mask_words(int n) { return ((n + 127) / 128) * 4; }
  static int smem_bytes(int n) {
    (void)n;
    return 1024 + 1024 + kTilesBytes;
  }
};

struct ItemGrid {
  int njt, nrp, total;
};

template <typename T, int D, int NS>
__global__ void __launch_bounds__(384, 1)
tc_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
             const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
             const __grid_constant__ CUtensorMap map_b, View5 dq, const float* __restrict__ lse,
             const float* __restrict__ delta, const uint8_t* __restrict__ rowfull,
             const uint32_t* __restrict__ maskbits, int mask_words, Dims dm, ItemGrid items,
             unsigned int* status) {
  using Cfg = DqCfg<D, NS>;
  constexpr int R = Cfg::R;
  constexpr int IN_FULL = 0, IN_EMPTY = 1, FULL = 2, EMPTY = FULL + NS, S_FULL = EMPTY + NS,
                S_FREE = S_FULL + R, DS_READY = S_FREE + R, DQ_DONE = DS_READY + R,
                DQ_FREE = DQ_DONE + R, TOKEN = DQ_FREE + R, NBARS = TOKEN + R;
  static_assert(NBARS * 8 <= 256, "barrier area");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 260);

  const int n = dm.n;
  const int nkt = (n + kBK - 1) / kBK;
  constexpr uint32_t tiles_off = 1024;
  const uint32_t tiles = base + tiles_off;
  auto bar = [&](int i) -> uint32_t { return base + 8u * i; };
  auto q_tile = [&](int r) -> uint32_t { return tiles + r * Cfg::kQBytes; };
  auto do_tile = [&](int r) -> uint32_t { return tiles + (R + r) * Cfg::kQBytes; };
  auto stage_off = [&](int s) -> uint32_t {
    return tiles_off + 2 * R * Cfg::kQBytes + s * Cfg::kStageBytes;
  };
  auto k_tile = [&](int s, int r) -> uint32_t { return base + stage_off(s) + r * Cfg::kKBytes; };
  auto v_tile = [&](int s, int r) -> uint32_t {
    return base + stage_off(s) + (R + r) * Cfg::kKBytes;
  };
  auto bias_off = [&](int s) -> uint32_t { return stage_off(s) + 2 * R * Cfg::kKBytes; };
  // item -> (j tile, first row, head, batch); a slot beyond the last row re-does the
  // last row (its loads stay in range, its results are not stored)
  struct Item {
    int jt, i0, h, b;
  };
  auto decode = [&](int w) -> Item {
    Item it;
    it.jt = w % items.njt;
    const int rest = w / items.njt;
    it.i0 = (rest % items.nrp) * R;
    const int bh = rest / items.nrp;
    it.h = bh % dm.heads;
    it.b = bh / dm.heads;
    return it;
  };
  auto slot_row = [&](const Item& it, int r) -> int { return min(it.i0 + r, dm.n_rows - 1); };

  if (*reinterpret_cast<volatile unsigned int*>(status) != 0u) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(bar(IN_FULL), 1);
    mbar_init(bar(IN_EMPTY), R);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), R * 5);
    }
    for (int r = 0; r < R; ++r) {
      mbar_init(bar(S_FULL + r), 1);
      mbar_init(bar(S_FREE + r), 4);
      mbar_init(bar(DS_READY + r), 4);
      mbar_init(bar(DQ_DONE + r), 1);
      mbar_init(bar(DQ_FREE + r), 4);
      mbar_init(bar(TOKEN + r), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 * R + 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (warp == 4 * R && lane == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_do);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 4 * R) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
    if (warp == 4 * R) {
      // ---------------------------------------------------------- TMA producer
      if (lane == 0) {
        int g = 0, it = 0;  // running key-tile and item counters (barrier phases)
        bool ok = true;
        for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
          const Item im = decode(w);
          if (it > 0) ok = mbar_wait(bar(IN_EMPTY), (it - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar(IN_FULL), R * 2 * Cfg::kQBytes);
          for (int r = 0; r < R; ++r) {
            tma_load_5d(q_tile(r), &map_q, bar(IN_FULL), 0, im.jt * kBJ, slot_row(im, r), im.h, im.b);
            tma_load_5d(do_tile(r), &map_do, bar(IN_FULL), 0, im.jt * kBJ, slot_row(im, r), im.h, im.b);
          }
          for (int kt = 0; kt < nkt; ++kt, ++g) {
            const int s = g % NS;
            if (g >= NS) ok = mbar_wait(bar(EMPTY + s), ((g / NS) - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(bar(FULL + s), R * 2 * Cfg::kKBytes + Cfg::kBiasBytes);
            for (int r = 0; r < R; ++r) {
              tma_load_5d(k_tile(s, r), &map_k, bar(FULL + s), 0, kt * kBK, slot_row(im, r), im.h, im.b);
              tma_load_5d(v_tile(s, r), &map_v, bar(FULL + s), 0, kt * kBK, slot_row(im, r), im.h, im.b);
            }
            tma_load_4d(base + bias_off(s), &map_b, bar(FULL + s), kt * kBK, im.jt * kBJ, im.h, im.b);
          }
        }
      }
    } else if (warp - (4 * R + 1) < R) {
      // ---------------------------------------------------------- MMA issuers (one per slot)
      const int r = warp - (4 * R + 1);
      if (lane == 0) {
        constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t idesc_s = make_idesc(128, kBK, kBf16, false, false);
        constexpr uint32_t idesc_dq = make_idesc(128, D, kBf16, false, true);
        auto issue_s_dp = [&](int s) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t aq = make_smem_desc(q_tile(r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bk = make_smem_desc(k_tile(s, r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            umma_ss(tmem_base + r * 256, aq, bk, idesc_s, kk > 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t ag = make_smem_desc(do_tile(r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bv = make_smem_desc(v_tile(s, r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            umma_ss(tmem_base + r * 256 + 64, ag, bv, idesc_s, kk > 0);
          }
          umma_commit(bar(S_FULL + r));
        };
        int g = 0, it = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
          ok = mbar_wait(bar(IN_FULL), it & 1, abort_flag) &&
               mbar_wait(bar(FULL + g % NS), (g / NS) & 1, abort_flag) &&
               (g == 0 || mbar_wait(bar(S_FREE + r), (g - 1) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after();
          issue_s_dp(g % NS);
          if (nkt == 1) umma_commit(bar(IN_EMPTY));
          for (int kt = 0; kt < nkt && ok; ++kt, ++g) {
            const int s = g % NS;
            if (kt + 1 < nkt) {
              const int ns = (g + 1) % NS;
              ok = mbar_wait(bar(FULL + ns), ((g + 1) / NS) & 1, abort_flag) &&
                   mbar_wait(bar(S_FREE + r), g & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
              issue_s_dp(ns);
              if (kt + 2 == nkt) umma_commit(bar(IN_EMPTY));  // last read of this item's Q, dO
            }
            ok = mbar_wait(bar(DS_READY + r), g & 1, abort_flag);
            // the first dQ MMA of an item overwrites dQ: the previous epilogue must have read it
            if (ok && kt == 0 && it > 0) ok = mbar_wait(bar(DQ_FREE + r), (it - 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < kBK / 16; ++ks) {
              const uint64_t bd = make_smem_desc(k_tile(s, r) + ks * 16 * Cfg::kRowBytes, Cfg::kSbo,
                                                 Cfg::kSbo, Cfg::kSwz);
              umma_ts(tmem_base + r * 256 + 160, tmem_base + r * 256 + 128 + ks * 8, bd, idesc_dq,
                      (kt > 0 || ks > 0) ? 1u : 0u);
            }
            umma_commit(bar(DQ_DONE + r));
            umma_commit(bar(EMPTY + s));
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMath));
    {
      // ---------------------------------------------------------- elementwise warpgroups
      const int r = warp / 4, wq = warp & 3, t = tid & 127;
      const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
      const uint32_t tS = tmem_base + lane_base + r * 256;
      const uint32_t tDP = tS + 64, tDS = tS + 128, tDQ = tS + 160;
      const float c1 = dm.scale * kLog2e;
      const float uniform = 1.f / (float)n;

      int g = 0, it = 0;
      bool ok = true;
      // What an item needs from global memory before its first tile (row flag, this
      // thread's lse and delta, the first mask words) is loaded one item ahead, before
      // the wait of the previous epilogue, and only used (compared, scaled) at the top
      // of its own item: a load that is used where it is issued stalls the warp for
      // the whole memory latency.
      struct ItemLoads {
        uint32_t flag;
        float lse, delta;
        uint32_t nx[4];
      };
      auto item_loads = [&](int w) -> ItemLoads {
        const Item im = decode(w);
        const int i = slot_row(im, r);
        const int64_t row = ((int64_t)im.b * dm.heads + im.h) * dm.n_rows + i;
        const int jc = min(im.jt * kBJ + t, n - 1);
        ItemLoads ld;
        ld.flag = rowfull[im.b * dm.n_rows + i];
        ld.lse = __ldg(lse + row * n + jc);
        ld.delta = __ldg(delta + row * dm.n_pad + jc);
        const uint32_t* mrow = maskbits + ((int64_t)im.b * dm.n_rows + i) * mask_words;
#pragma unroll
        for (int jb = 0; jb < 4; ++jb) ld.nx[jb] = __ldg(mrow + jb);
        return ld;
      };
      ItemLoads next_loads{};
      if ((int)blockIdx.x < items.total) next_loads = item_loads(blockIdx.x);
      for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
        const Item im = decode(w);
        const int i = slot_row(im, r);
        const bool do_store = im.i0 + r < dm.n_rows;
        const int b = im.b, h = im.h;
        const int j = im.jt * kBJ + t;
        const bool row_full = next_loads.flag != 0u;

        // Key mask of row i as packed words made by the prepare step (bit set = key
        // dropped or beyond n; none dropped inside n on a fully masked row).  Per 128-key
        // chunk c: word c*4 + jb holds, at bit l, key c*128 + 4*l + jb.
        const uint32_t* mb = maskbits + ((int64_t)b * dm.n_rows + i) * mask_words;
        const float neg_lse2 = -next_loads.lse * kLog2e;
        const float my_delta = next_loads.delta;

        // mask words are fetched one key tile ahead: a global load consumed in the same
        // tile would stall the pass for its whole latency
        uint32_t nx[4];
#pragma unroll
        for (int jb = 0; jb < 4; ++jb) nx[jb] = next_loads.nx[jb];

        auto key_loop = [&](auto row_full_tag) {
          constexpr bool kRowFull = decltype(row_full_tag)::value;
          for (int kt = 0; kt < nkt; ++kt, ++g) {
            const int s = g % NS;
            // S/dP of this tile and its bias stage: S_FULL implies FULL (the MMA that made
            // S read K from the same stage), so both tests succeed together and their
            // latencies overlap instead of adding up.
            {
              const bool a = mbar_wait(bar(S_FULL + r), g & 1, abort_flag);
              const bool c = mbar_wait(bar(FULL + s), (g / NS) & 1, abort_flag);
              ok = __all_sync(0xffffffffu, a && c);
            }
            if (!ok) break;
            tc_fence_after();
            float x[64], gd[64];
            {
              uint32_t* xr = reinterpret_cast<uint32_t*>(x);
              uint32_t* gr = reinterpret_cast<uint32_t*>(gd);
              tmem_ld32(tS + 0, xr + 0);
              tmem_ld32(tS + 32, xr + 32);
              tmem_ld32(tDP + 0, gr + 0);
              tmem_ld32(tDP + 32, gr + 32);
            }
            // while the TMEM loads are in flight: mask words of this 64-key tile (the
            // tile is half (kt & 1) of chunk kt >> 1; column c is position
            // pos = (kt & 1) * 64 + c: bit (pos >> 2) of word (pos & 3)) and the test that
            // the dQ MMA of the previous key tile no longer reads the dS columns
            uint32_t mw[4];
#pragma unroll
            for (int jb = 0; jb < 4; ++jb) mw[jb] = (nx[jb] >> ((kt & 1) * 16)) & 0xffffu;
            if (kt + 1 < nkt) {
#pragma unroll
              for (int jb = 0; jb < 4; ++jb) nx[jb] = __ldg(mb + ((kt + 1) >> 1) * 4 + jb);
            }
            const bool clean = (mw[0] | mw[1] | mw[2] | mw[3]) == 0u;
            // (a non-blocking look now; if it is not done yet the wait happens after the pass)
            const bool dq_done =
                __all_sync(0xffffffffu, (kt == 0) || mbar_test_wait(bar(DQ_DONE + r), (g - 1) & 1));
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(S_FREE + r));

            // One fused pass per 8 keys: bias load and unpack (LSU, ALU), two FMAs, the
            // exponential (MUFU), dS and the 16-bit pack.  Two copies, chosen per tile:
            // the copy for tiles without dropped keys has no branch in it, so the
            // compiler can overlap the eight groups.
            uint32_t pk[32];
            const uint8_t* brow = gbase + bias_off(s) + t * 128;
            auto pass = [&](auto clean_tag) {
              constexpr bool kClean = decltype(clean_tag)::value;
#pragma unroll
              for (int q8 = 0; q8 < 8; ++q8) {
                float p[8];
                if (kRowFull) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) p[e] = uniform;
                } else {
                  const uint4 u = *reinterpret_cast<const uint4*>(brow + ((q8 ^ (t & 7)) << 4));
                  float bv[8];
                  unpack2<T>(u.x, bv[0], bv[1]);
                  unpack2<T>(u.y, bv[2], bv[3]);
                  unpack2<T>(u.z, bv[4], bv[5]);
                  unpack2<T>(u.w, bv[6], bv[7]);
#pragma unroll
                  for (int e = 0; e < 8; ++e)
                    p[e] = ex2(fmaf(x[q8 * 8 + e], c1, fmaf(bv[e], kLog2e, neg_lse2)));
                }
                if (!kClean) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const int c = q8 * 8 + e;
                    p[e] = ((mw[c & 3] >> (c >> 2)) & 1u) ? 0.f : p[e];
                  }
                }
#pragma unroll
                for (int e = 0; e < 8; e += 2)
                  pk[(q8 * 8 + e) >> 1] = pack2<T>(p[e] * (gd[q8 * 8 + e] - my_delta),
                                                   p[e + 1] * (gd[q8 * 8 + e + 1] - my_delta));
              }
            };
            if (clean) pass(std::true_type{}); else pass(std::false_type{});
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(bar(EMPTY + s));  // bias tile consumed by this warp
              if (kSlotToken) mbar_arrive(bar(TOKEN + (r ^ 1)));
            }

            if (!dq_done) {
              ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_DONE + r), (g - 1) & 1, abort_flag));
              if (!ok) break;
            }
            tmem_st32(tDS, pk);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(DS_READY + r));
          }
        };
        if (row_full) key_loop(std::true_type{}); else key_loop(std::false_type{});
        if (!ok) break;
        if (w + (int)gridDim.x < items.total) next_loads = item_loads(w + gridDim.x);

        ok = __all_sync(0xffffffffu, mbar_wait(bar(DQ_DONE + r), (g - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        uint32_t acc[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld32(tDQ + 32 * c, acc + 32 * c);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(DQ_FREE + r));  // the next item's first dQ MMA may overwrite dQ
        if (do_store && j < n) {
          T* dst = reinterpret_cast<T*>(dq.p) + b * dq.sb + h * dq.sh + (int64_t)i * dq.si +
                   (int64_t)j * dq.sj;
#pragma unroll
          for (int e = 0; e < D; e += 8) {
            uint4 u;
            u.x = pack2<T>(__uint_as_float(acc[e + 0]) * dm.scale, __uint_as_float(acc[e + 1]) * dm.scale);
            u.y = pack2<T>(__uint_as_float(acc[e + 2]) * dm.scale, __uint_as_float(acc[e + 3]) * dm.scale);
            u.z = pack2<T>(__uint_as_float(acc[e + 4]) * dm.scale, __uint_as_float(acc[e + 5]) * dm.scale);
            u.w = pack2<T>(__uint_as_float(acc[e + 6]) * dm.scale, __uint_as_float(acc[e + 7]) * dm.scale);
            *reinterpret_cast<uint4*>(dst + e) = u;
          }
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
    if (tid == 0) atomicOr(status, (unsigned int)kStatusTimeoutBwdDq);
    __syncthreads();
  }
  if (warp == 4 * R + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int sm_count_dq() {
  int dev = 0, c = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev);
  return c > 0 ? c : 148;
}

template <typename T, int D, int NS>
cudaError_t launch_dq(const BwdArgs& a, cudaStream_t stream) {
  using Cfg = DqCfg<D, NS>;
  const Dims& dm = a.dm;
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const uint64_t eb = 2;
  CUtensorMap mq, mdo, mk, mv, mbias;
  const uint64_t dims5[5] = {(uint64_t)D, (uint64_t)dm.n, (uint64_t)dm.n_rows, (uint64_t)dm.heads,
                             (uint64_t)dm.batch};
  const uint32_t box_q[5] = {(uint32_t)D, 128, 1, 1, 1};
  const uint32_t box_k[5] = {(uint32_t)D, (uint32_t)kBK, 1, 1, 1};
  const CUtensorMapSwizzle swz = (D == 32) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  auto map5 = [&](CUtensorMap* m, const View5& v, const uint32_t* box) {
    const uint64_t st[4] = {(uint64_t)v.sj * eb, (uint64_t)v.si * eb, (uint64_t)v.sh * eb,
                            (uint64_t)v.sb * eb};
    return make_tensor_map(m, bf16, 5, v.p, dims5, st, box, swz);
  };
  if (!map5(&mq, a.q, box_q) || !map5(&mdo, a.d_o, box_q) || !map5(&mk, a.k, box_k) ||
      !map5(&mv, a.v, box_k))
    return cudaErrorInvalidValue;
  {
    // the bias itself when its rows are 16-byte pitched, else the padded copy
    const uint64_t n = dm.n, np = dm.n_pad;
    const uint64_t dims4[4] = {n, n, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st_user[3] = {(uint64_t)a.bias.sj * eb, (uint64_t)a.bias.sh * eb, (uint64_t)a.bias.sb * eb};
    const uint64_t st_pad[3] = {np * eb, n * np * eb, n * np * dm.heads * eb};
    const uint32_t box4[4] = {(uint32_t)kBK, 128, 1, 1};
    if (!make_tensor_map(&mbias, bf16, 4, a.bias_pad ? a.bias_pad : (void*)a.bias.p, dims4,
                         a.bias_pad ? st_pad : st_user, box4, CU_TENSOR_MAP_SWIZZLE_128B))
      return cudaErrorInvalidValue;
  }
  const int smem = Cfg::smem_bytes(dm.n);
  auto kern = tc_dq_kernel<T, D, NS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  ItemGrid items;
  items.njt = (dm.n + kBJ - 1) / kBJ;
  items.nrp = (dm.n_rows + 1) / 2;
  items.total = items.njt * items.nrp * dm.batch * dm.heads;
  const int sms = sm_count_dq() - a.reserve_sms > 0 ? sm_count_dq() - a.reserve_sms : 1;
  const int grid = items.total < sms ? items.total : sms;
  kern<<<grid, Cfg::kThreads, smem, stream>>>(mq, mdo, mk, mv, mbias, a.dq, a.lse, a.delta,
                                              a.rowfull, a.maskbits, a.mask_words, dm, items, a.status);
  return cudaGetLastError();
}

}  // namespace

bool tc_backward_supported(const BwdArgs& a) {
  const Dims& dm = a.dm;
  if (a.dtype != TRIFAST_BF16 && a.dtype != TRIFAST_F16) return false;
  if (dm.d != 16 && dm.d != 32 && dm.d != 64) return false;  // (d = 16: one-pass kernel only)
  if (dm.n < kMinTensorCoreN) return false;
  if (!a.maskbits || !a.rowfull || !a.delta || !a.neg_lse2) return false;
  // the bias goes through TMA: 16-byte row pitch, or the padded copy from the workspace
  const bool bias_tma_ok = !(((uintptr_t)a.bias.p) & 15) && (a.bias.sj * 2) % 16 == 0 &&
                           (a.bias.sh * 2) % 16 == 0 && (a.bias.sb * 2) % 16 == 0;
  if (!bias_tma_ok && !a.bias_pad) return false;
  return tc::get_encode_tiled() != nullptr;
}

cudaError_t tc_bwd_dq(const BwdArgs& a, cudaStream_t s) {
  const bool bf16 = a.dtype == TRIFAST_BF16;
  if (a.dm.d != 32 && a.dm.d != 64) return cudaErrorInvalidValue;
  if (a.dm.d == 32)
    return bf16 ? launch_dq<__nv_bfloat16, 32, 4>(a, s) : launch_dq<__half, 32, 4>(a, s);
  return bf16 ? launch_dq<__nv_bfloat16, 64, 3>(a, s) : launch_dq<__half, 64, 3>(a, s);
}

}  // namespace trifast
