// Forward triangle attention for head dim 128 on the 5th-generation tensor cores
// (bf16 / fp16).  At d = 128 a 128 x 128 score tile costs four times the contraction of
// d = 32 for the same exponentials, so the tensor pipe and the softmax are about evenly
// loaded; the tile sizes, not the arithmetic, are what sets this kernel apart from the
// d <= 64 forward:
//
//   * a 128 x 128 operand tile is 32 KiB: a row is two 128-byte swizzle spans, so every
//     tile is two [128 rows x 64 elements] halves 16 KiB apart (two TMA boxes; the
//     K-major operands take their K slices from one half or the other, the MN-major V
//     gets the halves as its two N atoms, leading offset 16 KiB);
//   * S (128 columns) + P (64) + O (128) of two slots do not fit the 512 TMEM columns:
//     P is written over the first half of S once S is in registers, so a slot's next
//     S = Q K^T can only be issued behind its O += P V.  MMAs of one issuing thread
//     execute in issue order, which gives exactly that order without a barrier;
//   * the two slots are the two 128-query tiles of a pair of tiles of ONE pair row: they
//     share K and V (and the key mask), which are single-buffered, as are the two bias
//     tiles: a softmax phase is long enough to hide the reload of each buffer.
//
//   warps 0-3 / 4-7 : softmax warpgroups of slot 0 / 1; thread t owns query row t
//   warp 8          : TMA producer (one lane): Q of both slots per item; K, bias x 2, V
//                     per key tile
//   warp 9          : MMA issuer (one lane) for both slots, and TMEM allocation
//   warps 10, 11    : idle; they complete the warpgroup whose registers are handed over
//
// TMEM columns of slot r (base r * 256): S [0,128) fp32, overwritten in [0,64) by P as
// 16-bit pairs; O [128,256) fp32.
//
// Semantics as in the d <= 64 forward: the PyTorch path of the reference
// (src/trifast/equiv.py:42-69); stands in for `_fwd` (src/trifast/triton.py:14-132).

#include <math.h>

#include "kernels.h"
#include "tc_common.cuh"

namespace trifast {
namespace {
using namespace tc;

constexpr int kD = 128;
constexpr int kRegDec = 56, kRegInc = 224;
static_assert(256 * kRegInc + 128 * kRegDec <= 384 * 168, "setmaxnreg pool");
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMaxInit = -1e30f;
// A key tile moves a row's running maximum only when it exceeds it by more than kLazyTau
// (natural-log units): weights then reach e^kLazyTau instead of 1, which 16-bit P holds with
// the same relative precision, and the 128-column rescale of O (a TMEM round trip of the
// whole accumulator) runs for the first tiles of a row only instead of nearly every tile.
#ifndef TRIFAST_D128_LAZY_TAU
#define TRIFAST_D128_LAZY_TAU 5.5f
#endif
constexpr float kLazyTau = TRIFAST_D128_LAZY_TAU;
constexpr int kTileBytes = 128 * kD * 2;     // Q, K or V tile: two halves of 16 KiB
constexpr int kHalfBytes = 16384;
constexpr int kBiasBytes = 128 * 128 * 2;    // two [128 queries x 64 keys] boxes
constexpr int kHeader = 1024;
constexpr int kSmemBytes = 1024 + kHeader + 4 * kTileBytes + 2 * kBiasBytes;
static_assert(kSmemBytes <= 232448, "shared memory");

struct Grid128 {
  int njt, njp, total;   // 128-query tiles of a row, pairs of them, work items
};

template <typename T>
__global__ void __launch_bounds__(384, 1)
tc_fwd_d128_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_b,
                   View5 o, float* __restrict__ lse, const uint8_t* __restrict__ rowfull,
                   const uint32_t* __restrict__ maskbits, int mask_words,
                   const uint32_t* __restrict__ rowrange, Dims dm, Grid128 items,
                   unsigned int* status) {
  constexpr int Q_FULL = 0, Q_EMPTY = 1, K_FULL = 2, K_EMPTY = 3, V_FULL = 4, V_EMPTY = 5,
                B_FULL = 6, B_EMPTY = 8, S_FULL = 10, P_READY = 12, O_DONE = 14, O_FREE = 16,
                NBARS = 18;
  static_assert(NBARS * 8 <= 256, "barrier area");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 260);
  // the item's live key-tile range, lo | hi << 16, per item parity: written by the producer
  // before its arrive on Q_FULL, read by the issuer after its wait on Q_FULL and by the
  // softmax warps after the item's first S_FULL
  volatile uint32_t* rng_word = reinterpret_cast<volatile uint32_t*>(gbase + 264);

  const int n = dm.n;
  const int nkt = (n + 127) / 128;
  auto bar = [&](int i) -> uint32_t { return base + 8u * i; };
  auto q_tile = [&](int r) -> uint32_t { return base + kHeader + r * kTileBytes; };
  const uint32_t k_tile = base + kHeader + 2 * kTileBytes;
  const uint32_t v_tile = base + kHeader + 3 * kTileBytes;
  auto bias_off = [&](int r) -> uint32_t { return kHeader + 4 * kTileBytes + r * kBiasBytes; };

  struct Item {
    int jp, i, h, b;
  };
  // item order: tile pair fastest, then row, then (b, h)
  auto decode = [&](int w) -> Item {
    Item it;
    it.jp = w % items.njp;
    const int rest = w / items.njp;
    it.i = rest % dm.n_rows;
    const int bh = rest / dm.n_rows;
    it.h = bh % dm.heads;
    it.b = bh / dm.heads;
    return it;
  };
  // slot r works on query tile 2 jp + r; an odd tile count leaves the last item's slot 1
  // without one: it repeats slot 0's tile (its loads stay in range) and stores nothing
  auto slot_tile = [&](const Item& it, int r) -> int { return min(2 * it.jp + r, items.njt - 1); };

  if (*reinterpret_cast<volatile unsigned int*>(status) != 0u) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(Q_EMPTY), 1);
    mbar_init(bar(K_FULL), 1);
    mbar_init(bar(K_EMPTY), 1);
    mbar_init(bar(V_FULL), 1);
    mbar_init(bar(V_EMPTY), 1);
    for (int r = 0; r < 2; ++r) {
      mbar_init(bar(B_FULL + r), 1);
      mbar_init(bar(B_EMPTY + r), 4);
      mbar_init(bar(S_FULL + r), 1);
      mbar_init(bar(P_READY + r), 4);
      mbar_init(bar(O_DONE + r), 1);
      mbar_init(bar(O_FREE + r), 4);
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
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegDec));
    if (warp == 8) {
      // ---------------------------------------------------------------- TMA producer
      if (lane == 0) {
        auto item_range = [&](int w) -> uint32_t {
          if (rowrange == nullptr || w >= items.total) return (uint32_t)nkt << 16;
          const Item it = decode(w);
          return __ldg(rowrange + it.b * dm.n_rows + it.i);
        };
        int g = 0, it = 0;   // running key-tile and item counters (barrier phases)
        bool ok = true;
        uint32_t rng_next = item_range(blockIdx.x);
        for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
          const Item im = decode(w);
          const uint32_t rng = rng_next;
          const int kt_lo = rng & 0xffffu, kt_hi = rng >> 16;
          rng_next = item_range(w + gridDim.x);
          if (it > 0) ok = mbar_wait(bar(Q_EMPTY), (it - 1) & 1, abort_flag);
          if (!ok) break;
          rng_word[it & 1] = rng;
          mbar_arrive_expect_tx(bar(Q_FULL), 2 * kTileBytes);
          for (int r = 0; r < 2; ++r) {
            const int j0 = slot_tile(im, r) * 128;
            tma_load_5d(q_tile(r), &map_q, bar(Q_FULL), 0, j0, im.i, im.h, im.b);
            tma_load_5d(q_tile(r) + kHalfBytes, &map_q, bar(Q_FULL), 64, j0, im.i, im.h, im.b);
          }
          for (int kt = kt_lo; kt < kt_hi; ++kt, ++g) {
            if (g > 0) ok = mbar_wait(bar(K_EMPTY), (g - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(bar(K_FULL), kTileBytes);
            tma_load_5d(k_tile, &map_k, bar(K_FULL), 0, kt * 128, im.i, im.h, im.b);
            tma_load_5d(k_tile + kHalfBytes, &map_k, bar(K_FULL), 64, kt * 128, im.i, im.h, im.b);
            for (int r = 0; r < 2 && ok; ++r) {
              if (g > 0) ok = mbar_wait(bar(B_EMPTY + r), (g - 1) & 1, abort_flag);
              if (!ok) break;
              const uint32_t dst = base + bias_off(r);
              const int j0 = slot_tile(im, r) * 128;
              mbar_arrive_expect_tx(bar(B_FULL + r), kBiasBytes);
              tma_load_4d(dst, &map_b, bar(B_FULL + r), kt * 128, j0, im.h, im.b);
              tma_load_4d(dst + 16384, &map_b, bar(B_FULL + r), kt * 128 + 64, j0, im.h, im.b);
            }
            if (!ok) break;
            if (g > 0) ok = mbar_wait(bar(V_EMPTY), (g - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_arrive_expect_tx(bar(V_FULL), kTileBytes);
            tma_load_5d(v_tile, &map_v, bar(V_FULL), 0, kt * 128, im.i, im.h, im.b);
            tma_load_5d(v_tile + kHalfBytes, &map_v, bar(V_FULL), 64, kt * 128, im.i, im.h, im.b);
          }
        }
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t idesc_qk = make_idesc(128, 128, kBf16, false, false);
        constexpr uint32_t idesc_pv = make_idesc(128, 128, kBf16, false, true);
        // S_r = Q_r K^T: eight K slices of 16 elements, four in each half of the tiles
        auto issue_qk = [&](int r) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
            const uint64_t ad = make_smem_desc(q_tile(r) + off, 16, 1024, kSwizzle128);
            const uint64_t bd = make_smem_desc(k_tile + off, 16, 1024, kSwizzle128);
            umma_ss(tmem_base + r * 256, ad, bd, idesc_qk, kk > 0);
          }
          umma_commit(bar(S_FULL + r));
        };
        // O_r (+)= P_r V: eight slices of 16 keys; V is MN-major, its two 64-element halves
        // are the two N atoms (leading offset 16 KiB), 8-key groups 1 KiB apart
        auto issue_pv = [&](int r, bool first) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t bd = make_smem_desc(v_tile + ks * 2048, kHalfBytes, 1024, kSwizzle128);
            umma_ts(tmem_base + r * 256 + 128, tmem_base + r * 256 + ks * 8, bd, idesc_pv,
                    (!first || ks > 0) ? 1u : 0u);
          }
          umma_commit(bar(O_DONE + r));
        };
        int g = 0, it = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
          ok = mbar_wait_spin(bar(Q_FULL), it & 1, abort_flag) &&
               mbar_wait_spin(bar(K_FULL), g & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t rng = rng_word[it & 1];
          const int kt_lo = rng & 0xffffu, kt_hi = rng >> 16;
          // (these S overwrite the S / P columns of the previous item's last tile: its
          // O += P V were issued before them by this thread and so execute before them)
          issue_qk(0);
          issue_qk(1);
          umma_commit(bar(K_EMPTY));
          if (kt_hi - kt_lo == 1) umma_commit(bar(Q_EMPTY));
          for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++g) {
            const bool more = kt + 1 < kt_hi;
            for (int r = 0; r < 2; ++r) {
              ok = mbar_wait_spin2(bar(P_READY + r), g & 1, r == 0, bar(V_FULL), g & 1, abort_flag);
              // the first O += P V of an item overwrites O: the previous item's epilogue must
              // have read it
              if (ok && kt == kt_lo && it > 0) ok = mbar_wait_spin(bar(O_FREE + r), (it - 1) & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
              issue_pv(r, kt == kt_lo);
              if (r == 1) umma_commit(bar(V_EMPTY));
              if (more) {
                // the slot's next S goes behind its O += P V (P lies over S)
                if (r == 0) {
                  ok = mbar_wait_spin(bar(K_FULL), (g + 1) & 1, abort_flag);
                  if (!ok) break;
                  tc_fence_after();
                }
                issue_qk(r);
                if (r == 1) {
                  umma_commit(bar(K_EMPTY));
                  if (kt + 2 == kt_hi) umma_commit(bar(Q_EMPTY));   // last read of the item's Q
                }
              }
            }
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegInc));
    // ------------------------------------------------------------------ softmax warpgroups
    const int r = warp >> 2, wq = warp & 3, t = tid & 127;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + r * 256;
    const uint32_t tP = tS, tO = tS + 128;

    int g = 0, it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
      const Item im = decode(w);
      const int i = im.i, b = im.b, h = im.h;
      const int jt = slot_tile(im, r);
      const bool do_store = 2 * im.jp + r < items.njt;
      const bool row_full = rowfull[b * dm.n_rows + i] != 0;
      const uint32_t* mbr = maskbits + ((int64_t)b * dm.n_rows + i) * mask_words;

      float m_run = kMaxInit, l_run = 0.f;
      // two copies of the key loop, chosen once per row (a merged loop would keep both
      // variants of the 128 scores live)
      auto key_loop = [&](auto row_full_tag) {
        constexpr bool kRowFull = decltype(row_full_tag)::value;
        int kt_lo = -1, kt_hi = 1;   // settled after the item's first S_FULL
        for (int kt = 0; kt < kt_hi; ++kt, ++g) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + r), g & 1, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (kt_lo < 0) {
            const uint32_t rng = rng_word[it & 1];
            kt_lo = kt = rng & 0xffffu;
            kt_hi = rng >> 16;
          }
          float x[128];
          {
            uint32_t* xr = reinterpret_cast<uint32_t*>(x);
            tmem_ld32(tS + 0, xr + 0);
            tmem_ld32(tS + 32, xr + 32);
            tmem_ld32(tS + 64, xr + 64);
            tmem_ld32(tS + 96, xr + 96);
            tmem_wait_ld();
          }
          // mask words of this key tile (uniform over the warp); column c of the tile is
          // bit (c >> 2) of word (c & 3)
          uint32_t mw[4];
#pragma unroll
          for (int jb = 0; jb < 4; ++jb) {
            if (kRowFull) {   // only keys beyond n stay dropped
              const int rem = n - kt * 128 - jb;
              const int groups = rem <= 0 ? 0 : (rem + 3) / 4;
              mw[jb] = groups >= 32 ? 0u : ~((1u << groups) - 1u);
            } else {
              mw[jb] = __ldg(mbr + kt * 4 + jb);
            }
          }
          const bool clean = (mw[0] | mw[1] | mw[2] | mw[3]) == 0u;

          ok = __all_sync(0xffffffffu, mbar_wait(bar(B_FULL + r), g & 1, abort_flag));
          if (!ok) break;
          if (kRowFull) {
#pragma unroll
            for (int c = 0; c < 128; ++c) x[c] = 0.f;
          } else {
            const uint8_t* brow = gbase + bias_off(r) + t * 128;
#pragma unroll
            for (int gq = 0; gq < 16; ++gq) {
              const uint4 u = *reinterpret_cast<const uint4*>(brow + (gq >> 3) * 16384 +
                                                              (((gq & 7) ^ (t & 7)) << 4));
              float b0, b1;
              unpack2<T>(u.x, b0, b1);
              ffma2(x[gq * 8 + 0], x[gq * 8 + 1], x[gq * 8 + 0], x[gq * 8 + 1], dm.scale, dm.scale, b0, b1);
              unpack2<T>(u.y, b0, b1);
              ffma2(x[gq * 8 + 2], x[gq * 8 + 3], x[gq * 8 + 2], x[gq * 8 + 3], dm.scale, dm.scale, b0, b1);
              unpack2<T>(u.z, b0, b1);
              ffma2(x[gq * 8 + 4], x[gq * 8 + 5], x[gq * 8 + 4], x[gq * 8 + 5], dm.scale, dm.scale, b0, b1);
              unpack2<T>(u.w, b0, b1);
              ffma2(x[gq * 8 + 6], x[gq * 8 + 7], x[gq * 8 + 6], x[gq * 8 + 7], dm.scale, dm.scale, b0, b1);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_EMPTY + r));   // bias tile consumed by this warp

          if (!clean) {
#pragma unroll
            for (int c = 0; c < 128; ++c)
              if ((mw[c & 3] >> (c >> 2)) & 1u) x[c] = -INFINITY;
          }
          float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
          for (int c = 4; c < 124; c += 8) {
            mx[0] = fmax3(mx[0], x[c + 0], x[c + 1]);
            mx[1] = fmax3(mx[1], x[c + 2], x[c + 3]);
            mx[2] = fmax3(mx[2], x[c + 4], x[c + 5]);
            mx[3] = fmax3(mx[3], x[c + 6], x[c + 7]);
          }
          mx[0] = fmax3(mx[0], x[124], x[125]);
          mx[1] = fmax3(mx[1], x[126], x[127]);
          const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
          const float m_new = (mt > m_run + kLazyTau) ? mt : m_run;
          const float neg = -m_new * kLog2e;
          // (difference first: exactly 1 when the maximum stays, also at its initial value)
          const float alpha = ex2((m_run - m_new) * kLog2e);
          m_run = m_new;

          if (kt > kt_lo) {
            // the previous tile's O += P V must be done before O is rescaled
            ok = __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + r), (g - 1) & 1, abort_flag));
            if (!ok) break;
            tc_fence_after();
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
              for (int c = 0; c < kD / 32; ++c) {
                uint32_t acc[32];
                tmem_ld32(tO + 32 * c, acc);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
                tmem_st32(tO + 32 * c, acc);
              }
            }
          }
          // exponentials and the P store in chunks of 32 keys; P overwrites columns [0, 64)
          // of S, which this thread has in registers (a thread only ever touches its own lane)
          float sm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 4) {
              const int c = ch * 32 + e;
              float a0, a1, a2, a3;
              ffma2(a0, a1, x[c + 0], x[c + 1], kLog2e, kLog2e, neg, neg);
              ffma2(a2, a3, x[c + 2], x[c + 3], kLog2e, kLog2e, neg, neg);
              const float p0 = ex2(a0), p1 = ex2(a1), p2 = ex2(a2), p3 = ex2(a3);
              fadd2(sm[0], sm[1], sm[0], sm[1], p0, p1);
              fadd2(sm[2], sm[3], sm[2], sm[3], p2, p3);
              pk[(e >> 1) + 0] = pack2<T>(p0, p1);
              pk[(e >> 1) + 1] = pack2<T>(p2, p3);
            }
            tmem_st16(tP + ch * 16, pk);
          }
          l_run = fmaf(l_run, alpha, (sm[0] + sm[1]) + (sm[2] + sm[3]));
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(P_READY + r));
        }
      };
      if (row_full) key_loop(std::true_type{}); else key_loop(std::false_type{});
      if (!ok) break;

      // epilogue of the item: O / l and lse
      ok = __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + r), (g - 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const int j = jt * 128 + t;
      const float inv = 1.f / l_run;
      T* dst = reinterpret_cast<T*>(o.p) + b * o.sb + h * o.sh + (int64_t)i * o.si + (int64_t)j * o.sj;
      uint32_t acc[kD];
      tmem_ld_cols<kD>(tO, acc);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(O_FREE + r));   // the next item's first O += P V may overwrite O
      if (do_store && j < n) {
#pragma unroll
        for (int e = 0; e < kD; e += 8) {
          uint4 u;
          u.x = pack2<T>(__uint_as_float(acc[e + 0]) * inv, __uint_as_float(acc[e + 1]) * inv);
          u.y = pack2<T>(__uint_as_float(acc[e + 2]) * inv, __uint_as_float(acc[e + 3]) * inv);
          u.z = pack2<T>(__uint_as_float(acc[e + 4]) * inv, __uint_as_float(acc[e + 5]) * inv);
          u.w = pack2<T>(__uint_as_float(acc[e + 6]) * inv, __uint_as_float(acc[e + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + e) = u;
        }
        lse[(((int64_t)b * dm.heads + h) * dm.n_rows + i) * n + j] =
            row_full ? dm.sentinel : fmaf(lg2(l_run), kLn2, m_run);
      }
    }
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let copies and MMAs in flight land before TMEM and shared memory are
    // released, then report through the status word
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (tid == 0) atomicOr(status, (unsigned int)kStatusTimeoutFwd);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T>
cudaError_t launch128(const FwdArgs& a, cudaStream_t stream) {
  const Dims& dm = a.dm;
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const uint64_t eb = 2;
  CUtensorMap mq, mk, mv, mbias;
  const uint64_t dims5[5] = {(uint64_t)kD, (uint64_t)dm.n, (uint64_t)dm.n_rows, (uint64_t)dm.heads,
                             (uint64_t)dm.batch};
  const uint32_t box5[5] = {64, 128, 1, 1, 1};
  auto map5 = [&](CUtensorMap* m, const View5& v) {
    const uint64_t st[4] = {(uint64_t)v.sj * eb, (uint64_t)v.si * eb, (uint64_t)v.sh * eb,
                            (uint64_t)v.sb * eb};
    return tc::make_tensor_map(m, bf16, 5, v.p, dims5, st, box5, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  if (!map5(&mq, a.q) || !map5(&mk, a.k) || !map5(&mv, a.v)) return cudaErrorInvalidValue;
  {
    // the bias itself when its rows are 16-byte pitched, else the padded copy
    const uint64_t n = dm.n, np = dm.n_pad;
    const uint64_t dims4[4] = {n, n, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st_user[3] = {(uint64_t)a.bias.sj * eb, (uint64_t)a.bias.sh * eb, (uint64_t)a.bias.sb * eb};
    const uint64_t st_pad[3] = {np * eb, n * np * eb, n * np * dm.heads * eb};
    const uint32_t box4[4] = {64, 128, 1, 1};
    if (!tc::make_tensor_map(&mbias, bf16, 4, a.bias_pad ? a.bias_pad : (void*)a.bias.p, dims4,
                             a.bias_pad ? st_pad : st_user, box4, CU_TENSOR_MAP_SWIZZLE_128B))
      return cudaErrorInvalidValue;
  }
  auto kern = tc_fwd_d128_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  Grid128 items;
  items.njt = (dm.n + 127) / 128;
  items.njp = (items.njt + 1) / 2;
  items.total = items.njp * dm.n_rows * dm.batch * dm.heads;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int grid = items.total < sms ? items.total : sms;
  kern<<<grid, 384, kSmemBytes, stream>>>(mq, mk, mv, mbias, a.o, a.lse, a.rowfull, a.maskbits,
                                          a.mask_words, a.rowrange, dm, items, a.status);
  return cudaGetLastError();
}

}  // namespace

// Needs the prepared row flags and packed key masks (and the padded bias copy when the
// bias rows are not 16-byte pitched): the forward workspace of head dim 128 always holds them.
bool tc_forward_d128_supported(const Dims& dm, int dtype, const FwdArgs* a) {
  if (dtype != TRIFAST_BF16 && dtype != TRIFAST_F16) return false;
  if (dm.d != kD || dm.n < kMinTensorCoreN) return false;
  if (a) {
    if (((uintptr_t)a->o.p) & 15 || (a->o.sj * 2) % 16) return false;
    if (!a->maskbits || !a->rowfull || !a->rowrange) return false;
    if (!a->bias_pad) {
      if (dm.n % 8 != 0) return false;
      if ((a->bias.sj * 2) % 16 || (a->bias.sh * 2) % 16 || (a->bias.sb * 2) % 16) return false;
      if (((uintptr_t)a->bias.p) & 15) return false;
    }
  }
  return tc::get_encode_tiled() != nullptr;
}

cudaError_t tc_forward_d128(const FwdArgs& a, cudaStream_t s) {
  return a.dtype == TRIFAST_BF16 ? launch128<__nv_bfloat16>(a, s) : launch128<__half>(a, s);
}

}  // namespace trifast
