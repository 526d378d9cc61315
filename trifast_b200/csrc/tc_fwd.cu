// Forward triangle attention on the 5th-generation tensor cores (bf16 / fp16).
//
// Work item = one 128-query tile (h, j-tile) of R = 2 consecutive pair rows i
// ("slots"), walked over the keys in tiles of 128.  The slots share every bias
// tile, which is the dominant shared-memory stream (32 KiB per step against
// 8-16 KiB of K+V per slot), and give the tensor pipe independent work while the
// softmax of the other slot runs.  CTAs are persistent: one per SM, each looping
// over work items, so that the loads and the first MMA of the next item overlap
// the tail of the current one instead of paying a pipeline fill per item.
//
//   warps 0 .. 4R-1 : softmax warpgroups, one per slot; thread t owns query row t:
//                     S (TMEM) -> registers, + bias (shared memory), mask, online
//                     softmax in fp32, P -> TMEM as 16-bit pairs, O rescale when
//                     the row maximum moves, final O / l and lse
//   warp 4R         : TMA producer (one lane): Q per item, then K, V (per slot)
//                     and the bias tile per key step through an NS-deep ring
//   warps 4R+1, 4R+2: MMA issuers, one per slot (one lane each): S = Q K^T (SS,
//                     both operands K-major) and O += P V (A = P from TMEM, B = V as
//                     an MN-major tile); a slot's MMAs never wait behind the other's
//   warp 4R + 3     : idle; it completes the warpgroup whose registers are handed
//                     to the softmax warpgroups (setmaxnreg)
//
// TMEM columns per slot r (base r * 256): S [0,128) fp32, P [128,192) packed
// 16-bit pairs, O [192, 192 + D) fp32.
//
// Semantics follow the PyTorch path of the reference (src/trifast/equiv.py:42-69):
// masked keys weigh exactly zero; rows whose keys are all masked get uniform
// weights over all n keys and lse = finfo(dtype).min.  The kernel stands in for
// `_fwd` of the reference (src/trifast/triton.py:14-132); unlike it, the scale
// d^-0.5 is applied to the fp32 accumulator, not to Q in 16 bits.

#include <math.h>

#include <mutex>

#include "kernels.h"
#include "tc_common.cuh"

namespace trifast {
namespace {
using namespace tc;

// Registers per thread after the warpgroups rebalance (setmaxnreg): the last
// warpgroup drops to TRIFAST_REG_DEC, the softmax warpgroups rise to
// TRIFAST_REG_INC.  The hand-over must balance: 384 threads launch with 168
// registers each, and a request beyond what the issue warpgroup released would
// block forever.
#ifndef TRIFAST_REG_DEC
#define TRIFAST_REG_DEC 56
#endif
#ifndef TRIFAST_REG_INC
#define TRIFAST_REG_INC 224
#endif
static_assert(256 * TRIFAST_REG_INC + 128 * TRIFAST_REG_DEC <= 384 * 168, "setmaxnreg pool");

constexpr int kBJ = 128, kBK = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMaxInit = -1e30f;
// A tile moves the running maximum only when it exceeds it by more than the lazy threshold
// (natural-log units).  0 = always track the exact maximum: the largest weight of a
// row is then exactly 1 before rounding to 16 bits, which keeps the error of peaked
// rows lowest; a positive value (FlashAttention-style lazy rescale) trades that for
// fewer rescales of O.  Measured at n = 1024: 2.7 % of the forward at d = 64 (64 columns of
// O per rescale), 1.5 % at d = 32, 1 % at d = 16, for a maximum error against the fp64 oracle
// about a third larger: taken at d = 64 only.
template <int D> constexpr float lazy_tau() { return D >= 64 ? 5.5f : 0.f; }
constexpr int kSmemLimit = 232448;  // 227 KiB opt-in limit per CTA
constexpr int kHeaderBytes = 512;

template <int D, int R, int NS>
struct FwdCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = 128 * kRowBytes;      // one Q / K / V tile
  static constexpr int kBiasBytes = 128 * 128 * 2;        // two [128 x 64] boxes
  static constexpr int kStageBytes = 2 * R * kTileBytes + kBiasBytes;
  static constexpr int kTilesBytes = R * kTileBytes + NS * kStageBytes;
  static constexpr int kThreads = R * 128 + 128;
  static constexpr uint64_t kSwz = RowSwizzle<D>::kDesc;
  static constexpr int kSbo = 8 * kRowBytes;              // pitch of 8-row groups
  // per slot: 4 mask words per 128-key chunk, one or two buffers (this item's and the next's)
  static int mask_bytes(int n, int bufs) { return bufs * R * ((n + kBK - 1) / kBK) * 16; }
  static int smem_with(int n, int bufs) {
    const int head = (kHeaderBytes + mask_bytes(n, bufs) + 1023) / 1024 * 1024;
    return 1024 + head + kTilesBytes;                     // 1024: manual base alignment
  }
  // two mask buffers (the next item's words are made ahead) when they fit, else one
  static int mask_bufs(int n) { return smem_with(n, 2) <= kSmemLimit ? 2 : 1; }
  static int smem_bytes(int n) {
    const int head = (kHeaderBytes + mask_bytes(n, mask_bufs(n)) + 1023) / 1024 * 1024;
    return 1024 + head + kTilesBytes;                     // 1024: manual base alignment
  }
};

// Work items in launch order: j-tile fastest, then row pair, then (b, h): the CTAs
// running at one time share bias strips and K/V rows in L2.
struct ItemGrid {
  int njt, nrp, total;
};

// MB: mask buffers per softmax warp (2: the next item's words are made ahead).
template <typename T, int D, int R, int NS, int MB>
__global__ void __launch_bounds__(R * 128 + 128, 1)
tc_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_b,
              View5 o, float* __restrict__ lse, MaskView mask, const uint8_t* __restrict__ ws_rowfull,
              const uint32_t* __restrict__ ws_maskbits, int ws_mask_words,
              const uint32_t* __restrict__ ws_rowrange, Dims dm, ItemGrid items,
              unsigned int* status) {
  using Cfg = FwdCfg<D, R, NS>;
  static_assert(R == 2, "two slots: the exp phases alternate between them");
  constexpr int Q_FULL = 0, Q_EMPTY = 1, FULL = 2, EMPTY = FULL + NS, S_FULL = EMPTY + NS,
                S_FREE = S_FULL + R, P_READY = S_FREE + R, O_DONE = P_READY + R,
                O_FREE = O_DONE + R, TOKEN = O_FREE + R, NBARS = TOKEN + R;
  static_assert(NBARS * 8 <= 256, "barrier area");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 260);
  uint32_t* maskbits = reinterpret_cast<uint32_t*>(gbase + kHeaderBytes);  // [R slots][MB][nkt][4]

  const int n = dm.n;
  const int nkt = (n + kBK - 1) / kBK;
  const uint32_t tiles_off = (kHeaderBytes + MB * R * nkt * 16 + 1023u) & ~1023u;
  const uint32_t tiles = base + tiles_off;
  auto bar = [&](int i) -> uint32_t { return base + 8u * i; };
  auto q_tile = [&](int r) -> uint32_t { return tiles + r * Cfg::kTileBytes; };
  auto stage_base = [&](int s) -> uint32_t {
    return tiles + R * Cfg::kTileBytes + s * Cfg::kStageBytes;
  };
  auto k_tile = [&](int s, int r) -> uint32_t { return stage_base(s) + r * Cfg::kTileBytes; };
  auto v_tile = [&](int s, int r) -> uint32_t {
    return stage_base(s) + (R + r) * Cfg::kTileBytes;
  };
  auto bias_off = [&](int s) -> uint32_t {  // byte offset from gbase
    return tiles_off + R * Cfg::kTileBytes + s * Cfg::kStageBytes + 2 * R * Cfg::kTileBytes;
  };
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
  // Key tiles [lo, hi) an item walks, as lo | hi << 16: the union of the live ranges of its
  // rows (tiles outside it hold no open key of either row and weigh exactly zero).  Only the
  // producer computes it (one item ahead; it alone is off the critical path) and hands it to
  // the other roles through a shared-memory word per item parity, written before its arrive
  // on Q_FULL: the issuers read it after their wait on Q_FULL, the softmax warps after the
  // item's first S_FULL, which the issuers' MMAs complete.  The producer is never more than
  // one item ahead of the issuers (Q_EMPTY) nor the issuers of the softmax warps (S_FREE),
  // so a word is rewritten only after every reader of its previous value has moved on.
  volatile uint32_t* rng_word = reinterpret_cast<volatile uint32_t*>(gbase + 264);   // [2]
  auto item_range = [&](int w) -> uint32_t {
    if (ws_rowrange == nullptr || w >= items.total) return (uint32_t)nkt << 16;
    const Item it = decode(w);
    uint32_t lo = 0xffffu, hi = 0u;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t v = __ldg(ws_rowrange + it.b * dm.n_rows + slot_row(it, r));
      lo = min(lo, v & 0xffffu);
      hi = max(hi, v >> 16);
    }
    return lo | (hi << 16);
  };

  // A wait that gave up in an earlier CTA or launch leaves the status word set:
  // stop doing work until the host has read and cleared it.
  if (*reinterpret_cast<volatile unsigned int*>(status) != 0u) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(Q_EMPTY), R);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), R * 5);  // per slot: 1 MMA commit + 4 softmax warps
    }
    for (int r = 0; r < R; ++r) {
      mbar_init(bar(S_FULL + r), 1);
      mbar_init(bar(S_FREE + r), 4);
      mbar_init(bar(P_READY + r), 4);
      mbar_init(bar(O_DONE + r), 1);
      mbar_init(bar(O_FREE + r), 4);
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
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 4 * R) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TRIFAST_REG_DEC));
  if (warp == 4 * R) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int g = 0, it = 0;  // running key-tile and item counters (barrier phases)
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
        mbar_arrive_expect_tx(bar(Q_FULL), R * Cfg::kTileBytes);
        for (int r = 0; r < R; ++r)
          tma_load_5d(q_tile(r), &map_q, bar(Q_FULL), 0, im.jt * kBJ, slot_row(im, r), im.h, im.b);
        for (int kt = kt_lo; kt < kt_hi; ++kt, ++g) {
          const int s = g % NS;
          if (g >= NS) ok = mbar_wait(bar(EMPTY + s), ((g / NS) - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(bar(FULL + s), R * 2 * Cfg::kTileBytes + Cfg::kBiasBytes);
          for (int r = 0; r < R; ++r) {
            tma_load_5d(k_tile(s, r), &map_k, bar(FULL + s), 0, kt * kBK, slot_row(im, r), im.h, im.b);
            tma_load_5d(v_tile(s, r), &map_v, bar(FULL + s), 0, kt * kBK, slot_row(im, r), im.h, im.b);
          }
          const uint32_t bias_s = base + bias_off(s);
          tma_load_4d(bias_s, &map_b, bar(FULL + s), kt * kBK, im.jt * kBJ, im.h, im.b);
          tma_load_4d(bias_s + 16384, &map_b, bar(FULL + s), kt * kBK + 64, im.jt * kBJ, im.h, im.b);
        }
      }
    }
  } else if (warp - (4 * R + 1) < R) {
    // ------------------------------------------------------------ MMA issuers (one per slot)
    const int r = warp - (4 * R + 1);
    if (lane == 0) {
      constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
      constexpr uint32_t idesc_qk = make_idesc(128, 128, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc(128, D, kBf16, false, true);
      auto issue_qk = [&](int s) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t ad = make_smem_desc(q_tile(r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
          const uint64_t bd = make_smem_desc(k_tile(s, r) + kk * 32, 16, Cfg::kSbo, Cfg::kSwz);
          umma_ss(tmem_base + r * 256, ad, bd, idesc_qk, kk > 0);
        }
        umma_commit(bar(S_FULL + r));
      };
      int g = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
        // S of the item's first key tile: needs Q, the first stage, and the S columns
        // released by the softmax of the previous item's last tile
        ok = mbar_wait(bar(Q_FULL), it & 1, abort_flag) &&
             mbar_wait(bar(FULL + g % NS), (g / NS) & 1, abort_flag) &&
             (g == 0 || mbar_wait(bar(S_FREE + r), (g - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t rng = rng_word[it & 1];
        const int kt_lo = rng & 0xffffu, kt_hi = rng >> 16;
        issue_qk(g % NS);
        if (kt_hi - kt_lo == 1) umma_commit(bar(Q_EMPTY));
        for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++g) {
          const int s = g % NS;
          if (kt + 1 < kt_hi) {
            const int ns = (g + 1) % NS;
            ok = mbar_wait(bar(FULL + ns), ((g + 1) / NS) & 1, abort_flag) &&
                 mbar_wait(bar(S_FREE + r), g & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_qk(ns);
            if (kt + 2 == kt_hi) umma_commit(bar(Q_EMPTY));  // last read of this item's Q tile
          }
          ok = mbar_wait(bar(P_READY + r), g & 1, abort_flag);
          // the first PV of an item overwrites O: the previous item's epilogue must have read it
          if (ok && kt == kt_lo && it > 0) ok = mbar_wait(bar(O_FREE + r), (it - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks) {
            const uint64_t bd = make_smem_desc(v_tile(s, r) + ks * 16 * Cfg::kRowBytes, Cfg::kSbo,
                                               Cfg::kSbo, Cfg::kSwz);
            umma_ts(tmem_base + r * 256 + 192, tmem_base + r * 256 + 128 + ks * 8, bd, idesc_pv,
                    (kt > kt_lo || ks > 0) ? 1u : 0u);
          }
          umma_commit(bar(O_DONE + r));
          umma_commit(bar(EMPTY + s));
        }
      }
    }
  }
  } else {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TRIFAST_REG_INC));
  {
    // ------------------------------------------------------------ softmax warpgroups
    const int r = warp / 4, wq = warp & 3, t = tid & 127;
    const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + r * 256;
    const uint32_t tP = tS + 128, tO = tS + 192;
    // One copy per slot: the four warps of a slot work on the same row, each makes the
    // same words and writes them to the same place, and reads them back after its own
    // writes: whatever the interleaving, every read sees the one value all warps write.
    uint32_t* mb = maskbits + r * MB * nkt * 4;

    // Key mask of a row as bit words (bit set = key dropped or beyond n), made one item
    // ahead so that the loads run under the last PV of the current item.  Lane l reads
    // keys 4l .. 4l+3 of a 128-key chunk as one word; word j of the chunk then holds,
    // at bit l, key 4l + j.
    struct RowMask {
      const uint32_t* words;
      bool full;
    };
    auto row_mask = [&](int w, uint32_t* dst) -> RowMask {
      const Item im = decode(w);
      const int i = slot_row(im, r), b = im.b;
      RowMask rm;
      if (ws_maskbits != nullptr) {
        // made by the prepare step (n % 8 != 0: the mask rows are not word-aligned)
        rm.words = ws_maskbits + ((int64_t)b * dm.n_rows + i) * ws_mask_words;
        rm.full = ws_rowfull[b * dm.n_rows + i] != 0;
        return rm;
      }
      const uint8_t* mrow = mask.p + b * mask.sb + (int64_t)i * mask.si;
      uint32_t open = 0;
      // four chunks at a time: the loads go out together, so a batch costs one
      // memory latency instead of four
      for (int c0 = 0; c0 < nkt; c0 += 4) {
        uint32_t u[4];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int key4 = (c0 + cc) * kBK + 4 * lane;
          u[cc] = (c0 + cc < nkt && key4 < n) ? __ldg(reinterpret_cast<const uint32_t*>(mrow + key4))
                                              : 0x01010101u;
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int c = c0 + cc;
          if (c < nkt) {
            const uint32_t vm = __ballot_sync(0xffffffffu, c * kBK + 4 * lane < n);
#pragma unroll
            for (int jb = 0; jb < 4; ++jb) {
              const uint32_t bits = __ballot_sync(0xffffffffu, ((u[cc] >> (8 * jb)) & 0xffu) != 0u);
              if (lane == 0) dst[c * 4 + jb] = bits;
              open |= ~bits & vm;
            }
          }
        }
      }
      __syncwarp();
      rm.words = dst;
      rm.full = open == 0u;
      return rm;
    };

    int g = 0, it = 0;
    bool ok = true;
    constexpr bool ahead = MB == 2;
    RowMask next_mask{mb, false};
    if (ahead && (int)blockIdx.x < items.total) next_mask = row_mask(blockIdx.x, mb);
    for (int w = blockIdx.x; w < items.total && ok; w += gridDim.x, ++it) {
      const Item im = decode(w);
      const int i = slot_row(im, r);
      const bool do_store = im.i0 + r < dm.n_rows;
      const int b = im.b, h = im.h, jt = im.jt;
      if (!ahead) next_mask = row_mask(w, mb);  // one buffer: made at the top of the item
      const bool row_full = next_mask.full;
      const uint32_t* mbr = next_mask.words;

      float m_run = kMaxInit, l_run = 0.f;
      // The key loop exists in two copies, chosen once per row: the fully-masked-row
      // case (every score is 0) must not merge with the regular case inside the
      // loop, or the 128 live scores get duplicated and spill.
      auto key_loop = [&](auto row_full_tag) {
      constexpr bool kRowFull = decltype(row_full_tag)::value;
      // (the item's tile range is read after its first S_FULL: see rng_word)
      int kt_lo = -1, kt_hi = 1;
      for (int kt = 0; kt < kt_hi; ++kt, ++g) {
        const int s = g % NS;
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
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(S_FREE + r));

        // mask words of this key tile (uniform over the warp); column c of the tile
        // is bit (c >> 2) of word (c & 3)
        uint32_t mw[4];
#pragma unroll
        for (int jb = 0; jb < 4; ++jb) {
          if (kRowFull) {  // only keys beyond n stay dropped: key 4l + jb of the chunk
            const int rem = n - kt * kBK - jb;             // keys 4l + jb < n  <=>  l < ceil(rem / 4)
            const int groups = rem <= 0 ? 0 : (rem + 3) / 4;
            mw[jb] = groups >= 32 ? 0u : ~((1u << groups) - 1u);
          } else {
            mw[jb] = mbr[kt * 4 + jb];
          }
        }
        const bool clean = (mw[0] | mw[1] | mw[2] | mw[3]) == 0u;

        ok = __all_sync(0xffffffffu, mbar_wait(bar(FULL + s), (g / NS) & 1, abort_flag));
        if (!ok) break;
        if (kRowFull) {
#pragma unroll
          for (int c = 0; c < 128; ++c) x[c] = 0.f;
        } else {
          const uint8_t* brow = gbase + bias_off(s) + t * 128;
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
        if (lane == 0) mbar_arrive(bar(EMPTY + s));  // bias tile consumed by this warp

        if (!clean) {
#pragma unroll
          for (int c = 0; c < 128; ++c)
            if ((mw[c & 3] >> (c >> 2)) & 1u) x[c] = -INFINITY;
        }
        // Four independent chains for the row maximum and the row sum: with two
        // warps per scheduler a single dependent chain of 128 would be latency-bound.
        float mx[4] = {x[0], x[1], x[2], x[3]};
#pragma unroll
        for (int c = 4; c < 124; c += 8) {  // 3-input max: two scores per instruction
          mx[0] = fmax3(mx[0], x[c + 0], x[c + 1]);
          mx[1] = fmax3(mx[1], x[c + 2], x[c + 3]);
          mx[2] = fmax3(mx[2], x[c + 4], x[c + 5]);
          mx[3] = fmax3(mx[3], x[c + 6], x[c + 7]);
        }
        mx[0] = fmax3(mx[0], x[124], x[125]);
        mx[1] = fmax3(mx[1], x[126], x[127]);
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        // running maximum (see lazy_tau)
        const float m_new = (mt > m_run + lazy_tau<D>()) ? mt : m_run;
        const float neg = -m_new * kLog2e;
        // (difference first: exactly 1 when the maximum stays, also at the initial value,
        // where a fused m_run * log2e + neg would leave the rounding residue of 1e30 * log2e
        // in the exponent and turn a key tile with no open key into inf * 0)
        const float alpha = ex2((m_run - m_new) * kLog2e);
        m_run = m_new;

        if (kt > kt_lo) {
          // PV of the previous key tile must be done before O is rescaled and P reused.
          ok = __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + r), (g - 1) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            if constexpr (D == 16) {
              uint32_t acc[16];
              tmem_ld16(tO, acc);
              tmem_wait_ld();
#pragma unroll
              for (int e = 0; e < 16; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
              tmem_st16(tO, acc);
            } else {
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
                uint32_t acc[32];
                tmem_ld32(tO + 32 * c, acc);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
                tmem_st32(tO + 32 * c, acc);
              }
            }
          }
        }
        // The two slots take turns in the exp phase, so that one slot's loads, bias
        // FMAs and maximum overlap the other's exponentials instead of both phases
        // running in lockstep.  Slot 0 goes first; each slot passes the turn on
        // after issuing its exponentials.
        ok = __all_sync(0xffffffffu,
                        mbar_wait(bar(TOKEN + r), (r == 0) ? ((g & 1) ^ 1) : (g & 1), abort_flag));
        if (!ok) break;
        // exp and P store in chunks of 32 keys, so a packed chunk leaves the
        // registers as soon as it is made; four independent partial sums.
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
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(TOKEN + (r ^ 1)));
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY + r));
      }
      };
      if (row_full) key_loop(std::true_type{}); else key_loop(std::false_type{});
      if (!ok) break;

      // the next item's mask words, while the last PV of this item runs
      if (ahead && w + (int)gridDim.x < items.total)
        next_mask = row_mask(w + gridDim.x, mb + ((it + 1) & 1) * nkt * 4);

      // epilogue of the item: O / l and lse
      ok = __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + r), (g - 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const int j = jt * kBJ + t;
      const float inv = 1.f / l_run;
      T* dst = reinterpret_cast<T*>(o.p) + b * o.sb + h * o.sh + (int64_t)i * o.si + (int64_t)j * o.sj;
      uint32_t acc[D];
      tmem_ld_cols<D>(tO, acc);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(O_FREE + r));  // the next item's first PV may overwrite O
      if (do_store && j < n) {
#pragma unroll
        for (int e = 0; e < D; e += 8) {
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
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: let copies and MMAs in flight land before TMEM and shared
    // memory are released, then report through the status word.
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000LL) {
    }
    if (tid == 0) atomicOr(status, (unsigned int)kStatusTimeoutFwd);
    __syncthreads();
  }
  if (warp == 4 * R + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int sm_count() {
  static int count[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (count[dev] == 0) {
    int c = 0;
    cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev);
    count[dev] = c > 0 ? c : 148;
  }
  return count[dev];
}

template <typename T, int D, int R, int NS>
cudaError_t launch(const FwdArgs& a, cudaStream_t stream) {
  using Cfg = FwdCfg<D, R, NS>;
  const Dims& dm = a.dm;
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const uint64_t eb = 2;
  CUtensorMap mq, mk, mv, mbias;
  const uint64_t dims5[5] = {(uint64_t)D, (uint64_t)dm.n, (uint64_t)dm.n_rows, (uint64_t)dm.heads,
                             (uint64_t)dm.batch};
  const uint32_t box5[5] = {(uint32_t)D, 128, 1, 1, 1};
  const CUtensorMapSwizzle swz = (CUtensorMapSwizzle)RowSwizzle<D>::kTma;
  auto map5 = [&](CUtensorMap* m, const View5& v) {
    const uint64_t st[4] = {(uint64_t)v.sj * eb, (uint64_t)v.si * eb, (uint64_t)v.sh * eb,
                            (uint64_t)v.sb * eb};
    return make_tensor_map(m, bf16, 5, v.p, dims5, st, box5, swz);
  };
  if (!map5(&mq, a.q) || !map5(&mk, a.k) || !map5(&mv, a.v)) return cudaErrorInvalidValue;
  {
    // the bias itself when its rows are 16-byte pitched, else the padded copy
    const uint64_t n = dm.n, np = dm.n_pad;
    const uint64_t dims4[4] = {n, n, (uint64_t)dm.heads, (uint64_t)dm.batch};
    const uint64_t st_user[3] = {(uint64_t)a.bias.sj * eb, (uint64_t)a.bias.sh * eb, (uint64_t)a.bias.sb * eb};
    const uint64_t st_pad[3] = {np * eb, n * np * eb, n * np * dm.heads * eb};
    const uint32_t box4[4] = {64, 128, 1, 1};
    if (!make_tensor_map(&mbias, bf16, 4, a.bias_pad ? a.bias_pad : (void*)a.bias.p, dims4,
                         a.bias_pad ? st_pad : st_user, box4, CU_TENSOR_MAP_SWIZZLE_128B))
      return cudaErrorInvalidValue;
  }
  const int smem = Cfg::smem_bytes(dm.n);
  const bool two = Cfg::mask_bufs(dm.n) == 2;
  auto kern = two ? tc_fwd_kernel<T, D, R, NS, 2> : tc_fwd_kernel<T, D, R, NS, 1>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  ItemGrid items;
  items.njt = (dm.n + kBJ - 1) / kBJ;
  items.nrp = (dm.n_rows + R - 1) / R;
  items.total = items.njt * items.nrp * dm.batch * dm.heads;
  const int grid = items.total < sm_count() ? items.total : sm_count();
  kern<<<grid, Cfg::kThreads, smem, stream>>>(mq, mk, mv, mbias, a.o, a.lse, a.mask, a.rowfull,
                                              a.maskbits, a.mask_words, a.rowrange, dm, items,
                                              a.status);
  return cudaGetLastError();
}

}  // namespace

namespace tc {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static bool encode(CUtensorMap* map, CUtensorMapDataType dt, uint64_t elem_bytes, int rank,
                   void* base, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, CUtensorMapSwizzle swz) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return false;
  cuuint64_t gdim[5], gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    uint64_t s = strides_bytes[i];
    // extent-1 dimensions may come with arbitrary strides: give them the dense pitch
    // (rounded up to the 16 bytes a stride must be a multiple of; it is never stepped)
    if (dims[i + 1] == 1)
      s = (i == 0) ? ((dims[0] * elem_bytes + 15) & ~(uint64_t)15) : gstr[i - 1] * dims[i];
    if (s == 0 || (s & 15)) return false;
    gstr[i] = s;
  }
  const CUresult r = enc(map, dt, (cuuint32_t)rank, base, gdim, gstr, bx, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_tensor_map(CUtensorMap* map, bool bf16, int rank, void* base, const uint64_t* dims,
                     const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz) {
  return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                rank, base, dims, strides_bytes, box, swz);
}

bool make_tensor_map_f32(CUtensorMap* map, int rank, void* base, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, rank, base, dims, strides_bytes, box,
                CU_TENSOR_MAP_SWIZZLE_NONE);
}

}  // namespace tc

bool tc_forward_supported(const Dims& dm, int dtype, const FwdArgs* a) {
  if (dtype != TRIFAST_BF16 && dtype != TRIFAST_F16) return false;
  if (dm.d != 16 && dm.d != 32 && dm.d != 64) return false;
  if (dm.n < kMinTensorCoreN) return false;
  const int smem = (dm.d == 16)   ? FwdCfg<16, 2, 3>::smem_bytes(dm.n)
                   : (dm.d == 32) ? FwdCfg<32, 2, 3>::smem_bytes(dm.n)
                                  : FwdCfg<64, 2, 2>::smem_bytes(dm.n);
  if (smem > kSmemLimit) return false;
  if (a) {
    if (((uintptr_t)a->o.p) & 15 || (a->o.sj * 2) % 16) return false;
    const bool have_ws = a->bias_pad && a->maskbits && a->rowfull;
    if (!have_ws) {
      // without the prepared copies the bias goes through TMA as it is (16-byte row
      // pitch) and the key mask is read four bytes at a time
      if (dm.n % 8 != 0) return false;
      if ((a->bias.sj * 2) % 16 || (a->bias.sh * 2) % 16 || (a->bias.sb * 2) % 16) return false;
      if (((uintptr_t)a->bias.p) & 15) return false;
      if (((uintptr_t)a->mask.p) & 3 || a->mask.sb % 4 || a->mask.si % 4) return false;
    }
  }
  return tc::get_encode_tiled() != nullptr;
}

cudaError_t tc_forward(const FwdArgs& a, const trifast_plan&, cudaStream_t s) {
  const bool bf16 = a.dtype == TRIFAST_BF16;
  if (a.dm.d == 16)
    return bf16 ? launch<__nv_bfloat16, 16, 2, 3>(a, s) : launch<__half, 16, 2, 3>(a, s);
  if (a.dm.d == 32)
    return bf16 ? launch<__nv_bfloat16, 32, 2, 3>(a, s) : launch<__half, 32, 2, 3>(a, s);
  return bf16 ? launch<__nv_bfloat16, 64, 2, 2>(a, s) : launch<__half, 64, 2, 2>(a, s);
}

}  // namespace trifast
