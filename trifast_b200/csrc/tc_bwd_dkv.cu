// dk and dv of triangle attention on the tensor cores (bf16 / fp16).
//
// A work item is a 128-key tile of R consecutive pair rows ("slots"), walked over
// the queries in tiles of 64; CTAs are persistent (one per SM, looping over items)
// so the loads of the next item overlap the tail of the current one.  Everything is computed transposed, keys on the TMEM
// lanes, so that P^T and dS^T feed the second pair of MMAs straight from TMEM:
//     S^T  = K Q^T            (SS MMA, 128 keys x 64 queries)
//     dP^T = V dO^T           (SS MMA)
//     P^T  = exp2(S^T * c + bias^T * log2e - lse_j * log2e),  dS^T = P^T * (dP^T - delta_j)
//            (the vector -lse * log2e is made once by the prepare step)
//     dV  += P^T dO           (A = P^T from TMEM, B = dO tile as MN-major)
//     dK  += dS^T Q           (A = dS^T from TMEM, B = Q tile as MN-major)
// and at the end dk = dK * d^-0.5.  A thread owns one key, so the key mask is a
// per-thread flag; lse and delta are per-column vectors read from shared memory;
// the bias is read from a transposed copy (k-major) made by the prepare step, so
// that a thread reads its row contiguously.
//
// Warps: 0 .. 4R-1 elementwise warpgroups, 4R TMA producer, 4R+1 .. 4R+R MMA issuers
// (one per slot, so a slot never queues behind the other's waits), the rest idle.  TMEM columns per slot r (base r * 256): S^T [0,64),
// dP^T [64,128), P^T [128,160), dS^T [160,192), dK [192, 192+D), dV [192+D, 192+2D)
// (d = 64 runs one slot per CTA).
//
// Stands in for `_bwd_kv` of the reference (src/trifast/triton.py:137-263).

#include <math.h>

#include <type_traits>

#include "kernels.h"
#include "tc_common.cuh"

namespace trifast {
namespace {
using namespace tc;

constexpr int kBKeys = 128, kBJ = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kSmemLimit = 232448;
// Register hand-over (setmaxnreg): 384 threads launch with 168 registers each; what
// the math warpgroups gain must not exceed what the issue warpgroup releases, or
// the request blocks forever.
constexpr int kRegsIssue = 56, kRegsMath = 224;
static_assert(256 * kRegsMath + 128 * kRegsIssue <= 384 * 168, "setmaxnreg pool");

template <int D, int R, int NS>
struct DkvCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kKVBytes = 128 * kRowBytes;       // resident K or V tile
  static constexpr int kQBytes = kBJ * kRowBytes;        // streamed Q or dO tile
  static constexpr int kBiasBytes = 128 * kBJ * 2;       // bias^T tile: 128 keys x 64 queries
  static constexpr int kVecBytes = kBJ * 4;              // lse or delta of 64 queries
  static constexpr int kStageData = 2 * R * kQBytes + kBiasBytes + 2 * R * kVecBytes;
  static constexpr int kStageBytes = (kStageData + 1023) / 1024 * 1024;
  static constexpr int kTilesBytes = 2 * R * kKVBytes + NS * kStageBytes;
  static constexpr int kThreads = R * 128 + 128;
  static constexpr uint64_t kSwz = (D == 32) ? kSwizzle64 : kSwizzle128;
  static constexpr int kSbo = 8 * kRowBytes;
  static constexpr int kSlotCols = (R == 1) ? 512 : 256;
  static int smem_bytes() { return 1024 + 1024 + kTilesBytes; }
};

struct ItemGrid {
  int nkt, nrp, total;
};

template <typename T, int D, int R, int NS>
__global__ void __launch_bounds__(R * 128 + 128, 1)
tc_dkv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
              const __grid_constant__ CUtensorMap map_bt, const __grid_constant__ CUtensorMap map_lse,
              const __grid_constant__ CUtensorMap map_delta, View5 dk, View5 dv,
              const uint8_t* __restrict__ rowfull, MaskView mask, Dims dm, ItemGrid items,
              unsigned int* status) {
  using Cfg = DkvCfg<D, R, NS>;
  constexpr int IN_FULL = 0, IN_EMPTY = 1, FULL = 2, EMPTY = FULL + NS, S_FULL = EMPTY + NS,
                S_FREE = S_FULL + R, P_READY = S_FREE + R, ACC_DONE = P_READY + R,
                ACC_FREE = ACC_DONE + R, NBARS = ACC_FREE + R;
  static_assert(NBARS * 8 <= 256, "barrier area");
  constexpr int kSlot = Cfg::kSlotCols;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 260);

  const int n = dm.n;
  const int njt = (n + kBJ - 1) / kBJ;
  constexpr uint32_t tiles_off = 1024;
  auto bar = [&](int i) -> uint32_t { return base + 8u * i; };
  auto k_tile = [&](int r) -> uint32_t { return base + tiles_off + r * Cfg::kKVBytes; };
  auto v_tile = [&](int r) -> uint32_t { return base + tiles_off + (R + r) * Cfg::kKVBytes; };
  auto stage_off = [&](int s) -> uint32_t {
    return tiles_off + 2 * R * Cfg::kKVBytes + s * Cfg::kStageBytes;
  };
  auto q_tile = [&](int s, int r) -> uint32_t { return base + stage_off(s) + r * Cfg::kQBytes; };
  auto do_tile = [&](int s, int r) -> uint32_t {
    return base + stage_off(s) + (R + r) * Cfg::kQBytes;
  };
  auto bias_off = [&](int s) -> uint32_t { return stage_off(s) + 2 * R * Cfg::kQBytes; };
  auto lse_off = [&](int s, int r) -> uint32_t {
    return bias_off(s) + Cfg::kBiasBytes + r * Cfg::kVecBytes;
  };
  auto delta_off = [&](int s, int r) -> uint32_t {
    return bias_off(s) + Cfg::kBiasBytes + (R + r) * Cfg::kVecBytes;
  };
  // item -> (key tile, first row, head, batch); a slot beyond the last row re-does the
  // last row (its loads stay in range, its results are not stored)
  struct Item {
    int kt, i0, h, b;
  };
  auto decode = [&](int w) -> Item {
    Item it;
    it.kt = w % items.nkt;
    const int rest = w / items.nkt;
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
      mbar_init(bar(P_READY + r), 4);
      mbar_init(bar(ACC_DONE + r), 1);
      mbar_init(bar(ACC_FREE + r), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 4 * R + 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (warp == 4 * R && lane == 0) {
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_do);
    tma_prefetch_desc(&map_bt);
    tma_prefetch_desc(&map_lse);
    tma_prefetch_desc(&map_delta);
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
        int g = 0, it = 0;  // running query-tile and item counters (barrier phases)
        bool ok = true;
        for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
          const Item im = decode(w);
          if (it > 0) ok = mbar_wait(bar(IN_EMPTY), (it - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar(IN_FULL), R * 2 * Cfg::kKVBytes);
          for (int r = 0; r < R; ++r) {
            tma_load_5d(k_tile(r), &map_k, bar(IN_FULL), 0, im.kt * kBKeys, slot_row(im, r), im.h, im.b);
            tma_load_5d(v_tile(r), &map_v, bar(IN_FULL), 0, im.kt * kBKeys, slot_row(im, r), im.h, im.b);
          }
          for (int jt = 0; jt < njt; ++jt, ++g) {
            const int s = g % NS;
            if (g >= NS) ok = mbar_wait(bar(EMPTY + s), ((g / NS) - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(bar(FULL + s),
                                  R * (2 * Cfg::kQBytes + 2 * Cfg::kVecBytes) + Cfg::kBiasBytes);
            for (int r = 0; r < R; ++r) {
              const int i = slot_row(im, r);
              tma_load_5d(q_tile(s, r), &map_q, bar(FULL + s), 0, jt * kBJ, i, im.h, im.b);
              tma_load_5d(do_tile(s, r), &map_do, bar(FULL + s), 0, jt * kBJ, i, im.h, im.b);
              tma_load_4d(base + lse_off(s, r), &map_lse, bar(FULL + s), jt * kBJ, i, im.h, im.b);
              tma_load_4d(base + delta_off(s, r), &map_delta, bar(FULL + s), jt * kBJ, i, im.h, im.b);
            }
            tma_load_4d(base + bias_off(s), &map_bt, bar(FULL + s), jt * kBJ, im.kt * kBKeys, im.h, im.b);
          }
        }
      }
    } else if (warp - (4 * R + 1) < R) {
      // ---------------------------------------------------------- MMA issuers (one per slot)
      const int r = warp - (4 * R + 1);
      if (lane == 0) {
        constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t idesc_s = make_idesc(128, kBJ, kBf16, false, false);
        constexpr uint32_t idesc_acc = make_idesc(128, D, kBf16, false, true);
        auto issue_s_dp = [&](int s) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t ak = make_smem_desc(k_tile(r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bq = make_smem_desc(q_tile(s, r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            umma_ss(tmem_base + r * kSlot, ak, bq, idesc_s, kk > 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t av = make_smem_desc(v_tile(r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bg = make_smem_desc(do_tile(s, r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
            umma_ss(tmem_base + r * kSlot + 64, av, bg, idesc_s, kk > 0);
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
          if (njt == 1) umma_commit(bar(IN_EMPTY));
          for (int jt = 0; jt < njt && ok; ++jt, ++g) {
            const int s = g % NS;
            if (jt + 1 < njt) {
              const int ns = (g + 1) % NS;
              ok = mbar_wait(bar(FULL + ns), ((g + 1) / NS) & 1, abort_flag) &&
                   mbar_wait(bar(S_FREE + r), g & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
              issue_s_dp(ns);
              if (jt + 2 == njt) umma_commit(bar(IN_EMPTY));  // last read of this item's K, V
            }
            ok = mbar_wait(bar(P_READY + r), g & 1, abort_flag);
            // the first accumulating MMAs of an item overwrite dK, dV: the previous
            // epilogue must have read them
            if (ok && jt == 0 && it > 0) ok = mbar_wait(bar(ACC_FREE + r), (it - 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = (jt > 0) ? 1u : 0u;
#pragma unroll
            for (int ks = 0; ks < kBJ / 16; ++ks) {  // dV += P^T dO
              const uint64_t bd = make_smem_desc(do_tile(s, r) + ks * 16 * Cfg::kRowBytes, Cfg::kSbo,
                                                 Cfg::kSbo, Cfg::kSwz);
              umma_ts(tmem_base + r * kSlot + 192 + D, tmem_base + r * kSlot + 128 + ks * 8, bd,
                      idesc_acc, (ks > 0) ? 1u : acc);
            }
#pragma unroll
            for (int ks = 0; ks < kBJ / 16; ++ks) {  // dK += dS^T Q
              const uint64_t bd = make_smem_desc(q_tile(s, r) + ks * 16 * Cfg::kRowBytes, Cfg::kSbo,
                                                 Cfg::kSbo, Cfg::kSwz);
              umma_ts(tmem_base + r * kSlot + 192, tmem_base + r * kSlot + 160 + ks * 8, bd,
                      idesc_acc, (ks > 0) ? 1u : acc);
            }
            umma_commit(bar(ACC_DONE + r));
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
      const uint32_t tS = tmem_base + lane_base + r * kSlot;
      const uint32_t tDP = tS + 64, tP = tS + 128, tDS = tS + 160, tDK = tS + 192, tDV = tS + 192 + D;
      const float c1 = dm.scale * kLog2e;
      const float uniform = 1.f / (float)n;

      int g = 0, it = 0;
      bool ok = true;
      // Row flag and this thread's mask byte pick the loop copy at the top of an item, so
      // their loads would be paid in full there: they are fetched one item ahead, under
      // the previous epilogue.
      struct KeyState {  // raw bytes: compared at the top of their own item, not where they are loaded
        uint32_t row_full, masked;
      };
      auto key_state = [&](int w) -> KeyState {
        const Item im = decode(w);
        const int i = slot_row(im, r);
        const int key = min(im.kt * kBKeys + t, n - 1);
        KeyState ks;
        ks.row_full = rowfull[im.b * dm.n_rows + i];
        ks.masked = mask.p[im.b * mask.sb + (int64_t)i * mask.si + key];
        return ks;
      };
      KeyState next_state{0u, 0u};
      if ((int)blockIdx.x < items.total) next_state = key_state(blockIdx.x);
      for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
        const Item im = decode(w);
        const int i = slot_row(im, r);
        const bool do_store = im.i0 + r < dm.n_rows;
        const int b = im.b, h = im.h;
        const int key = im.kt * kBKeys + t;
        const bool row_full = next_state.row_full != 0u;
        // weight of this thread's key: 0 when dropped (or beyond n); on a fully masked
        // row every key inside n weighs 1/n
        const bool dropped = key >= n || (!row_full && next_state.masked != 0u);
        // The key weight pattern is fixed for the whole query loop, so the loop is
        // instantiated per pattern of this warp: 0 = every key kept (no selects),
        // 1 = mixed, 2 = every key dropped (no exponentials), 3 = fully masked row.
        const int mode = row_full ? 3
                         : __all_sync(0xffffffffu, !dropped) ? 0
                         : __all_sync(0xffffffffu, dropped)  ? 2
                                                             : 1;
        auto query_loop = [&](auto mode_tag) {
        constexpr int kMode = decltype(mode_tag)::value;
        for (int jt = 0; jt < njt; ++jt, ++g) {
          const int s = g % NS;
          ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + r), g & 1, abort_flag));
          if (!ok) break;
          tc_fence_after();
          float x[64], g_[64];
          {
            uint32_t* xr = reinterpret_cast<uint32_t*>(x);
            uint32_t* gr = reinterpret_cast<uint32_t*>(g_);
            tmem_ld32(tS + 0, xr + 0);
            tmem_ld32(tS + 32, xr + 32);
            tmem_ld32(tDP + 0, gr + 0);
            tmem_ld32(tDP + 32, gr + 32);
            tmem_wait_ld();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(S_FREE + r));

          ok = __all_sync(0xffffffffu, mbar_wait(bar(FULL + s), (g / NS) & 1, abort_flag));
          if (!ok) break;
        // One fused pass per 8 queries: bias^T / lse / delta loads, unpack, FMAs, the
        // exponential, dS and both 16-bit packs, so that the LSU, ALU, FMA and MUFU
        // pipes overlap inside one warp.
        uint32_t pp[32], pd[32];
        {
          const uint8_t* brow = gbase + bias_off(s) + t * 128;
          const float4* lse4 = reinterpret_cast<const float4*>(gbase + lse_off(s, r));
          const float4* del4 = reinterpret_cast<const float4*>(gbase + delta_off(s, r));
#pragma unroll
          for (int q8 = 0; q8 < 8; ++q8) {
            const float4 da = del4[q8 * 2], db = del4[q8 * 2 + 1];
            const float dl[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
            float p[8];
            if (kMode == 2) {
#pragma unroll
              for (int e = 0; e < 8; ++e) p[e] = 0.f;
            } else if (kMode == 3) {
#pragma unroll
              for (int e = 0; e < 8; ++e) p[e] = uniform;
            } else {
              const uint4 u = *reinterpret_cast<const uint4*>(brow + ((q8 ^ (t & 7)) << 4));
              const float4 la = lse4[q8 * 2], lb = lse4[q8 * 2 + 1];
              const float nl[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
              float bv[8];
              unpack2<T>(u.x, bv[0], bv[1]);
              unpack2<T>(u.y, bv[2], bv[3]);
              unpack2<T>(u.z, bv[4], bv[5]);
              unpack2<T>(u.w, bv[6], bv[7]);
#pragma unroll
              for (int e = 0; e < 8; ++e)
                p[e] = ex2(fmaf(x[q8 * 8 + e], c1, fmaf(bv[e], kLog2e, nl[e])));
            }
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              const int c = q8 * 8 + e;
              uint32_t wp = pack2<T>(p[e], p[e + 1]);
              uint32_t wd = pack2<T>(p[e] * (g_[c] - dl[e]), p[e + 1] * (g_[c + 1] - dl[e + 1]));
              if (kMode == 1 || kMode == 3) {  // dropped keys weigh exactly zero
                wp = dropped ? 0u : wp;
                wd = dropped ? 0u : wd;
              }
              pp[c >> 1] = wp;
              pd[c >> 1] = wd;
            }
          }
        }
        __syncwarp();
          if (lane == 0) mbar_arrive(bar(EMPTY + s));  // bias^T, lse, delta consumed by this warp

          if (jt > 0) {  // the accumulating MMAs of the previous query tile still read P^T, dS^T
            ok = __all_sync(0xffffffffu, mbar_wait(bar(ACC_DONE + r), (g - 1) & 1, abort_flag));
            if (!ok) break;
          }
          tmem_st32(tP, pp);
          tmem_st32(tDS, pd);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(P_READY + r));
        }
        };
        switch (mode) {
          case 0: query_loop(std::integral_constant<int, 0>{}); break;
          case 1: query_loop(std::integral_constant<int, 1>{}); break;
          case 2: query_loop(std::integral_constant<int, 2>{}); break;
          default: query_loop(std::integral_constant<int, 3>{}); break;
        }
        if (!ok) break;
        if (w + (int)gridDim.x < items.total) next_state = key_state(w + gridDim.x);

        ok = __all_sync(0xffffffffu, mbar_wait(bar(ACC_DONE + r), (g - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        uint32_t acck[D], accv[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          tmem_ld32(tDK + 32 * c, acck + 32 * c);
          tmem_ld32(tDV + 32 * c, accv + 32 * c);
        }
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(ACC_FREE + r));  // the next item may overwrite dK, dV
        if (do_store && key < n) {
          T* dst_k = reinterpret_cast<T*>(dk.p) + b * dk.sb + h * dk.sh + (int64_t)i * dk.si +
                     (int64_t)key * dk.sj;
          T* dst_v = reinterpret_cast<T*>(dv.p) + b * dv.sb + h * dv.sh + (int64_t)i * dv.si +
                     (int64_t)key * dv.sj;
#pragma unroll
          for (int e = 0; e < D; e += 8) {
            uint4 u;
            u.x = pack2<T>(__uint_as_float(acck[e + 0]) * dm.scale, __uint_as_float(acck[e + 1]) * dm.scale);
            u.y = pack2<T>(__uint_as_float(acck[e + 2]) * dm.scale, __uint_as_float(acck[e + 3]) * dm.scale);
            u.z = pack2<T>(__uint_as_float(acck[e + 4]) * dm.scale, __uint_as_float(acck[e + 5]) * dm.scale);
            u.w = pack2<T>(__uint_as_float(acck[e + 6]) * dm.scale, __uint_as_float(acck[e + 7]) * dm.scale);
            *reinterpret_cast<uint4*>(dst_k + e) = u;
            u.x = pack2<T>(__uint_as_float(accv[e + 0]), __uint_as_float(accv[e + 1]));
            u.y = pack2<T>(__uint_as_float(accv[e + 2]), __uint_as_float(accv[e + 3]));
            u.z = pack2<T>(__uint_as_float(accv[e + 4]), __uint_as_float(accv[e + 5]));
            u.w = pack2<T>(__uint_as_float(accv[e + 6]), __uint_as_float(accv[e + 7]));
            *reinterpret_cast<uint4*>(dst_v + e) = u;
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
    if (tid == 0) atomicOr(status, (unsigned int)kStatusTimeoutBwdDkv);
    __syncthreads();
  }
  if (warp == 4 * R + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int D, int R, int NS>
cudaError_t launch_dkv(const BwdArgs& a, cudaStream_t stream) {
  using Cfg = DkvCfg<D, R, NS>;
  const Dims& dm = a.dm;
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const uint64_t eb = 2;
  CUtensorMap mk, mv, mq, mdo, mbt, mlse, mdelta;
  const uint64_t dims5[5] = {(uint64_t)D, (uint64_t)dm.n, (uint64_t)dm.n_rows, (uint64_t)dm.heads,
                             (uint64_t)dm.batch};
  const uint32_t box_kv[5] = {(uint32_t)D, 128, 1, 1, 1};
  const uint32_t box_q[5] = {(uint32_t)D, (uint32_t)kBJ, 1, 1, 1};
  const CUtensorMapSwizzle swz = (D == 32) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  auto map5 = [&](CUtensorMap* m, const View5& v, const uint32_t* box) {
    const uint64_t st[4] = {(uint64_t)v.sj * eb, (uint64_t)v.si * eb, (uint64_t)v.sh * eb,
                            (uint64_t)v.sb * eb};
    return make_tensor_map(m, bf16, 5, v.p, dims5, st, box, swz);
  };
  if (!map5(&mk, a.k, box_kv) || !map5(&mv, a.v, box_kv) || !map5(&mq, a.q, box_q) ||
      !map5(&mdo, a.d_o, box_q))
    return cudaErrorInvalidValue;
  {  // transposed bias copy: (b, h, k, j) with row pitch n_pad
    const uint64_t n = dm.n, np = dm.n_pad;
    const uint64_t dims4[4] = {n, n, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st[3] = {np * eb, n * np * eb, n * np * dm.heads * eb};
    const uint32_t box4[4] = {(uint32_t)kBJ, 128, 1, 1};
    if (!make_tensor_map(&mbt, bf16, 4, a.bias_t, dims4, st, box4, CU_TENSOR_MAP_SWIZZLE_128B))
      return cudaErrorInvalidValue;
  }
  {  // -lse * log2(e) and delta: (b, h, rows, n_pad) fp32, made by the prepare step
    const uint64_t n = dm.n, np = dm.n_pad, rows = dm.n_rows;
    const uint64_t dims4[4] = {n, rows, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st[3] = {np * 4, np * rows * 4, np * rows * dm.heads * 4};
    const uint32_t box4[4] = {(uint32_t)kBJ, 1, 1, 1};
    if (!make_tensor_map_f32(&mlse, 4, a.neg_lse2, dims4, st, box4) ||
        !make_tensor_map_f32(&mdelta, 4, a.delta, dims4, st, box4))
      return cudaErrorInvalidValue;
  }
  const int smem = Cfg::smem_bytes();
  auto kern = tc_dkv_kernel<T, D, R, NS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  ItemGrid items;
  items.nkt = (dm.n + kBKeys - 1) / kBKeys;
  items.nrp = (dm.n_rows + R - 1) / R;
  items.total = items.nkt * items.nrp * dm.batch * dm.heads;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  sms = sms - a.reserve_sms > 0 ? sms - a.reserve_sms : 1;
  const int grid = items.total < sms ? items.total : sms;
  kern<<<grid, Cfg::kThreads, smem, stream>>>(mk, mv, mq, mdo, mbt, mlse, mdelta, a.dk, a.dv,
                                              a.rowfull, a.mask, dm, items, a.status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_bwd_dkv(const BwdArgs& a, cudaStream_t s) {
  const bool bf16 = a.dtype == TRIFAST_BF16;
  if (a.dm.d != 32 && a.dm.d != 64) return cudaErrorInvalidValue;
  static_assert(DkvCfg<32, 2, 4>::kTilesBytes + 2048 <= kSmemLimit, "smem");
  static_assert(DkvCfg<64, 1, 4>::kTilesBytes + 2048 <= kSmemLimit, "smem");
  if (!a.bias_t || !a.neg_lse2) return cudaErrorInvalidValue;
  if (a.dm.d == 32)
    return bf16 ? launch_dkv<__nv_bfloat16, 32, 2, 4>(a, s) : launch_dkv<__half, 32, 2, 4>(a, s);
  return bf16 ? launch_dkv<__nv_bfloat16, 64, 1, 4>(a, s) : launch_dkv<__half, 64, 1, 4>(a, s);
}

}  // namespace trifast
