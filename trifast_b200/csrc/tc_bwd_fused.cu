// dq, dk and dv of triangle attention in ONE pass over the scores (bf16 / fp16).
//
// A work item is one pair row i of one (b, h): the CTA walks the row's key tiles
// (128 keys, outer loop) and, per key tile, its queries in steps of 64 (inner loop),
// and evaluates every score exactly once.  Everything is computed transposed, keys
// on the TMEM lanes:
//     S^T  = K Q^T,  dP^T = V dO^T                      (SS MMAs, 128 keys x 64 queries)
//     P^T  = exp2(S^T * c + bias^T * log2e - lse_j * log2e),  dS^T = P^T * (dP^T - delta_j)
//     dV  += P^T dO,  dK += dS^T Q                      (A = P^T / dS^T from TMEM)
//     dQ  += dS K                                       (A = dS from shared memory)
// dK and dV of the current key tile and dQ of the WHOLE row stay in TMEM: dK / dV
// are written out after each key tile, dQ once per row.  dS is needed in both
// orientations; the elementwise threads (one key each) write their dS^T rows to TMEM
// for dK and, as 16-bit, to a shared-memory tile whose rows are keys and whose columns
// are queries; read as an MN-major A operand that tile is dS.  One dQ MMA (128 queries
// x D, K = 128 keys) is issued per pair of steps.
//
// The reference computes dq and dk/dv in two kernels that each recompute S, P and
// dS (src/trifast/triton.py:268-383 _bwd_q, :137-263 _bwd_kv); this kernel replaces
// both with one exponential per score.
//
// Warps 0-7: elementwise (thread = key; warps w and w + 4 share the TMEM lanes and
// take 32 of the step's 64 queries each); warp 8 TMA producer; warp 9 issues the S / dP MMAs (and owns the TMEM allocation), warp 10 the dV / dK
// MMAs, warp 11 the dQ MMAs: one thread can issue an MMA only every ~60 cycles
// whatever its size, and no kind queues behind a wait of another.  TMEM columns: S^T [0,64), dP^T [64,128), P^T [128,160),
// dS^T [160,192) (16-bit pairs), dK [192,192+D), dV [192+D,192+2D), dQ from 192+2D,
// D columns per 128-query tile: a row fits when ceil(n/128) * D <= 320 - 2D
// (d = 32: n <= 1024; d = 64: n <= 384).  A longer row is walked in query chunks of as
// many tiles as fit: per chunk all key tiles are swept again (S, P, dS of a chunk's
// queries are still evaluated once), dQ of the chunk leaves at its end, and dK / dV of
// a key tile are completed over the chunks: the partial of the earlier chunks waits as
// fp32 in a per-CTA scratch (written and read by the same thread, L2-resident).
//
// Masked keys weigh exactly zero; rows whose keys are all masked use P = 1/n over
// the n keys (the PyTorch semantics, src/trifast/equiv.py:42-69).

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
constexpr int kFusedMaxCtas = 160;  // grid cap: the per-CTA dK / dV scratch is sized by it
// Register hand-over (setmaxnreg): 384 threads launch with 168 registers each; what
// the math warpgroups gain must not exceed what the issue warpgroup releases, or
// the request blocks forever.
constexpr int kRegsIssue = 56, kRegsMath = 224;
static_assert(256 * kRegsMath + 128 * kRegsIssue <= 384 * 168, "setmaxnreg pool");

template <int D, int NS, int SB>
struct FusedCfg {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kKVBytes = 128 * kRowBytes;       // resident K or V tile
  static constexpr int kQBytes = kBJ * kRowBytes;        // streamed Q or dO tile
  static constexpr int kBiasBytes = 128 * kBJ * 2;       // bias^T tile: 128 keys x 64 queries
  static constexpr int kVecBytes = kBJ * 4;              // -lse*log2e or delta of 64 queries
  static constexpr int kStageData = 2 * kQBytes + kBiasBytes + 2 * kVecBytes;
  static constexpr int kStageBytes = (kStageData + 1023) / 1024 * 1024;
  static constexpr int kHalfBytes = 128 * kBJ * 2;       // dS of one step: 128 keys x 64 queries
  static constexpr int kPairBytes = 2 * kHalfBytes;      // dS of a pair of steps: 128 x 128
  static constexpr int kTilesBytes = 4 * kKVBytes + NS * kStageBytes + 2 * kPairBytes;
  static constexpr int kThreads = 384;
  static constexpr uint64_t kSwz = RowSwizzle<D>::kDesc;
  static constexpr int kSbo = 8 * kRowBytes;
  // TMEM columns: SB buffers of S^T [0,64) + dP^T [64,128); then P^T, dS^T (32 each, 16-bit
  // pairs), dK, dV (D each) and dQ, D columns per 128-query tile
  // (an accumulator of D = 16 columns still starts on a multiple of 32 columns)
  static constexpr int kAcc = D < 32 ? 32 : D;
  static constexpr int kPCol = SB * 128, kDsCol = kPCol + 32, kDkCol = kPCol + 64,
                       kDvCol = kDkCol + kAcc;
  static constexpr int kDqCol = kDvCol + kAcc;              // first dQ column
  static constexpr int kMaxJTiles = (512 - kDqCol) / kAcc;  // 128-query tiles whose dQ fits
  static constexpr int kTilesPerGroup = (kMaxJTiles + 1) / 2;
  static int smem_bytes() { return 1024 + 1024 + kTilesBytes; }
};

struct FusedGrid {
  int total;     // work items = batch * heads * n_rows
  int nkt;       // key tiles of 128
  int njs;       // query steps of 64
  int njt;       // query tiles of 128 (dQ tiles)
  int nch;       // query chunks: a row whose dQ does not fit TMEM is walked chunk by chunk
  int jsc;       // query steps per full chunk (even)
};

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

template <typename T, int D, int NS, int SB>
__global__ void __launch_bounds__(384, 1)
tc_dqkv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
               const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
               const __grid_constant__ CUtensorMap map_bt, const __grid_constant__ CUtensorMap map_lse,
               const __grid_constant__ CUtensorMap map_delta, View5 dq, View5 dk, View5 dv,
               const uint8_t* __restrict__ rowfull, const uint32_t* __restrict__ maskbits_lin,
               int mask_words, const uint32_t* __restrict__ rowrange, Dims dm, FusedGrid grid,
               float* __restrict__ kv_scratch, unsigned int* status) {
  using Cfg = FusedCfg<D, NS, SB>;
  // Barriers.  The per-step ones exist once per step parity (index g & 1, phase
  // (g >> 1) & 1), which leaves every waiter a whole step of slack before a parity
  // could be mistaken for the one two steps earlier.
  constexpr int KV_FULL = 0, KV_EMPTY = 2, FULL = 4, EMPTY = FULL + NS, S_FULL = EMPTY + NS,
                S_FREE = S_FULL + 2, P_READY = S_FREE + 2, ACC_DONE = P_READY + 2,
                ACC_FREE = ACC_DONE + 2, DQ_FREE = ACC_FREE + 1, NBARS = DQ_FREE + 1;
  static_assert(NBARS * 8 <= 256, "barrier area");
  static_assert(Cfg::kDqCol + Cfg::kMaxJTiles * Cfg::kAcc <= 512, "TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gbase + 260);

  const int n = dm.n;
  const int nkt = grid.nkt, njs = grid.njs, njt = grid.njt, nch = grid.nch, jsc = grid.jsc;
  constexpr uint32_t tiles_off = 1024;
  constexpr uint32_t stages_off = tiles_off + 4 * Cfg::kKVBytes;
  constexpr uint32_t pairs_off = stages_off + NS * Cfg::kStageBytes;
  auto bar = [&](int i) -> uint32_t { return base + 8u * i; };
  auto k_tile = [&](int kvb) -> uint32_t { return base + tiles_off + (2 * kvb) * Cfg::kKVBytes; };
  auto v_tile = [&](int kvb) -> uint32_t { return base + tiles_off + (2 * kvb + 1) * Cfg::kKVBytes; };
  auto stage_off = [&](int s) -> uint32_t { return stages_off + s * Cfg::kStageBytes; };
  auto q_tile = [&](int s) -> uint32_t { return base + stage_off(s); };
  auto do_tile = [&](int s) -> uint32_t { return base + stage_off(s) + Cfg::kQBytes; };
  auto bias_off = [&](int s) -> uint32_t { return stage_off(s) + 2 * Cfg::kQBytes; };
  auto lse_off = [&](int s) -> uint32_t { return bias_off(s) + Cfg::kBiasBytes; };
  auto delta_off = [&](int s) -> uint32_t { return lse_off(s) + Cfg::kVecBytes; };
  auto pair_off = [&](int pb) -> uint32_t { return pairs_off + pb * Cfg::kPairBytes; };
  // item -> (row, head, batch): consecutive CTAs work on neighbouring rows of one
  // (b, h) and sweep the same bias tiles at about the same time (L2 hits)
  struct Item {
    int i, h, b;
  };
  auto decode = [&](int w) -> Item {
    Item it;
    it.i = w % dm.n_rows;
    const int bh = w / dm.n_rows;
    it.h = bh % dm.heads;
    it.b = bh / dm.heads;
    return it;
  };
  // Key tiles [lo, hi) of the item's row that hold an open key, as lo | hi << 16: the roles
  // walk only those (dK, dV of the others are zero-filled, dQ gets nothing from them).
  // Fetched one item ahead.
  auto item_range = [&](int w) -> uint32_t {
    if (rowrange == nullptr || w >= grid.total) return (uint32_t)nkt << 16;
    const Item it = decode(w);
    return __ldg(rowrange + it.b * dm.n_rows + it.i);
  };

  if (*reinterpret_cast<volatile unsigned int*>(status) != 0u) return;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int u = 0; u < 2; ++u) {
      mbar_init(bar(KV_FULL + u), 1);
      mbar_init(bar(KV_EMPTY + u), 1);
      mbar_init(bar(S_FULL + u), 1);
      mbar_init(bar(S_FREE + u), 8);
      mbar_init(bar(P_READY + u), 8);
      mbar_init(bar(ACC_DONE + u), 2);  // one commit from each accumulating issuer
    }
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), 9);  // the dV / dK commit + the 8 elementwise warps
    }
    mbar_init(bar(ACC_FREE), 8);
    mbar_init(bar(DQ_FREE), 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
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

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));
    if (warp == 8) {
      // ------------------------------------------------------------ TMA producer
      // (Every lane of an issuing warp runs the loop, so that addresses, coordinates
      // and descriptors are warp-uniform values; one lane issues.)
      const bool leader = lane == 0;
      int g = 0, ktg = 0;  // running step and key-tile counters (barrier phases)
      bool ok = true;
      uint32_t rng_next = item_range(blockIdx.x);
      for (int w = blockIdx.x; w < grid.total && ok; w += gridDim.x) {
        const Item im = decode(w);
        const int kt_lo = rng_next & 0xffffu, kt_hi = rng_next >> 16;
        rng_next = item_range(w + gridDim.x);
        for (int c = 0; c < nch && ok; ++c) {
        const int js0 = c * jsc, js1 = min(njs, js0 + jsc);
        for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++ktg) {
          const int kvb = ktg & 1;
          if (ktg >= 2)
            ok = __all_sync(0xffffffffu,
                            mbar_wait_spin(bar(KV_EMPTY + kvb), ((ktg >> 1) - 1) & 1, abort_flag));
          if (!ok) break;
          if (leader) {
            mbar_arrive_expect_tx(bar(KV_FULL + kvb), 2 * Cfg::kKVBytes);
            tma_load_5d(k_tile(kvb), &map_k, bar(KV_FULL + kvb), 0, kt * kBKeys, im.i, im.h, im.b);
            tma_load_5d(v_tile(kvb), &map_v, bar(KV_FULL + kvb), 0, kt * kBKeys, im.i, im.h, im.b);
          }
          for (int js = js0; js < js1; ++js, ++g) {
            const int s = g % NS;
            if (g >= NS)
              ok = __all_sync(0xffffffffu,
                              mbar_wait_spin(bar(EMPTY + s), ((g / NS) - 1) & 1, abort_flag));
            if (!ok) break;
            if (leader) {
              mbar_arrive_expect_tx(bar(FULL + s),
                                    2 * Cfg::kQBytes + Cfg::kBiasBytes + 2 * Cfg::kVecBytes);
              tma_load_5d(q_tile(s), &map_q, bar(FULL + s), 0, js * kBJ, im.i, im.h, im.b);
              tma_load_5d(do_tile(s), &map_do, bar(FULL + s), 0, js * kBJ, im.i, im.h, im.b);
              tma_load_4d(base + bias_off(s), &map_bt, bar(FULL + s), js * kBJ, kt * kBKeys, im.h, im.b);
              tma_load_4d(base + lse_off(s), &map_lse, bar(FULL + s), js * kBJ, im.i, im.h, im.b);
              tma_load_4d(base + delta_off(s), &map_delta, bar(FULL + s), js * kBJ, im.i, im.h, im.b);
            }
            __syncwarp();
          }
        }
        }
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------ S^T / dP^T issuer
      const bool leader = lane == 0;
      constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
      constexpr uint32_t idesc_s = make_idesc(128, kBJ, kBf16, false, false);
      int g = 0, ktg = 0;
      bool ok = true;
      uint32_t rng_next = item_range(blockIdx.x);
      for (int w = blockIdx.x; w < grid.total && ok; w += gridDim.x) {
        const int kt_lo = rng_next & 0xffffu, kt_hi = rng_next >> 16;
        rng_next = item_range(w + gridDim.x);
        for (int c = 0; c < nch && ok; ++c) {
        const int js0 = c * jsc, js1 = min(njs, js0 + jsc);
        for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++ktg) {
          const int kvb = ktg & 1;
          for (int js = js0; js < js1; ++js, ++g) {
            const int s = g % NS;
            // the S / dP buffer of this step was last read at step g - SB
            const int gp = g - SB;
            ok = (js > js0 || mbar_wait_spin(bar(KV_FULL + kvb), (ktg >> 1) & 1, abort_flag)) &&
                 mbar_wait_spin2(bar(FULL + s), (g / NS) & 1, gp >= 0, bar(S_FREE + (gp & 1)),
                                 (gp >> 1) & 1, abort_flag);
            const uint32_t t_s = tmem_base + (g % SB) * 128;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint64_t ak = make_smem_desc(k_tile(kvb), 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bq = make_smem_desc(q_tile(s), 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t av = make_smem_desc(v_tile(kvb), 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t bg = make_smem_desc(do_tile(s), 16, Cfg::kSbo, Cfg::kSwz);
            if (leader) {
              // a K slice of 16 elements is 32 bytes further along the row: + 2 in the
              // descriptor's address field (16-byte units)
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk)
                umma_ss(t_s, ak + 2 * kk, bq + 2 * kk, idesc_s, kk > 0);
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk)
                umma_ss(t_s + 64, av + 2 * kk, bg + 2 * kk, idesc_s, kk > 0);
              umma_commit(bar(S_FULL + (g & 1)));
            }
            __syncwarp();
          }
        }
        }
      }
    } else if (warp == 10) {
      // ------------------------------------------------------------ dV / dK issuer
      const bool leader = lane == 0;
      constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
      constexpr uint32_t idesc_acc = make_idesc(128, D, kBf16, false, true);
      // 16 rows of an MN-major tile are this many 16-byte units further on
      constexpr uint32_t kStep16Rows = (16 * Cfg::kRowBytes) >> 4;
      int g = 0, ktg = 0;
      bool ok = true;
      uint32_t rng_next = item_range(blockIdx.x);
      for (int w = blockIdx.x; w < grid.total && ok; w += gridDim.x) {
        const int kt_lo = rng_next & 0xffffu, kt_hi = rng_next >> 16;
        rng_next = item_range(w + gridDim.x);
        for (int c = 0; c < nch && ok; ++c) {
        const int js0 = c * jsc, js1 = min(njs, js0 + jsc);
        for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++ktg) {
          for (int js = js0; js < js1; ++js, ++g) {
            const int s = g % NS;
            // the first accumulating MMAs of a key tile overwrite dK, dV: the epilogue
            // of the previous key tile must have read them (tested together with
            // P_READY: each test costs a shared-memory round trip)
            const bool first = js == js0 && ktg > 0;
            ok = mbar_wait_spin2(bar(P_READY + (g & 1)), (g >> 1) & 1, first, bar(ACC_FREE),
                                 (ktg - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = (js > js0) ? 1u : 0u;
            const uint64_t b_do = make_smem_desc(do_tile(s), Cfg::kSbo, Cfg::kSbo, Cfg::kSwz);
            const uint64_t b_q = make_smem_desc(q_tile(s), Cfg::kSbo, Cfg::kSbo, Cfg::kSwz);
            if (leader) {
#pragma unroll
              for (int ks = 0; ks < kBJ / 16; ++ks) {  // dV += P^T dO, dK += dS^T Q, interleaved
                umma_ts(tmem_base + Cfg::kDvCol, tmem_base + Cfg::kPCol + ks * 8,
                        b_do + ks * kStep16Rows, idesc_acc, (ks > 0) ? 1u : acc);
                umma_ts(tmem_base + Cfg::kDkCol, tmem_base + Cfg::kDsCol + ks * 8,
                        b_q + ks * kStep16Rows, idesc_acc, (ks > 0) ? 1u : acc);
              }
              umma_commit(bar(ACC_DONE + (g & 1)));
              umma_commit(bar(EMPTY + s));
            }
            __syncwarp();
          }
        }
        }
      }
    } else {
      // ------------------------------------------------------------ dQ issuer
      const bool leader = lane == 0;
      constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
      constexpr uint32_t idesc_dq = make_idesc(128, D, kBf16, true, true);
      constexpr uint32_t kStep16Rows = (16 * Cfg::kRowBytes) >> 4;
      int g = 0, ktg = 0, pgc = 0, chg = 0;  // chg: running chunk counter (DQ_FREE phases)
      bool ok = true;
      uint32_t rng_next = item_range(blockIdx.x);
      for (int w = blockIdx.x; w < grid.total && ok; w += gridDim.x) {
        const int kt_lo = rng_next & 0xffffu, kt_hi = rng_next >> 16;
        rng_next = item_range(w + gridDim.x);
        for (int c = 0; c < nch && ok; ++c, ++chg) {
        const int js0 = c * jsc, js1 = min(njs, js0 + jsc);
        for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++ktg) {
          const int kvb = ktg & 1;
          for (int js = js0; js < js1; ++js, ++g) {
            const bool with_dq = ((js - js0) & 1) || js == js1 - 1;
            const int pr = (js - js0) >> 1, pb = (pgc + pr) & 1;
            // the first dQ MMA of a chunk overwrites dQ: the previous chunk's epilogue must
            // have read it
            const bool first = with_dq && kt == kt_lo && pr == 0 && chg > 0;
            ok = mbar_wait_spin2(bar(P_READY + (g & 1)), (g >> 1) & 1, first, bar(DQ_FREE),
                                 (chg - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            // dS tile of the pair (rows = keys, 128-byte rows of 64 queries, two halves):
            // read as an MN-major A operand it is dS (queries x keys)
            const uint64_t a_ds = make_smem_desc(base + pair_off(pb), Cfg::kHalfBytes, 1024, kSwizzle128);
            const uint64_t b_k = make_smem_desc(k_tile(kvb), Cfg::kSbo, Cfg::kSbo, Cfg::kSwz);
            if (leader) {
              if (with_dq) {
                // dQ of the 128-query tile js / 2: both halves of its dS tile are written
                // (an odd last step leaves the second half stale: those queries lie
                // beyond n and their dQ rows are never stored)
#pragma unroll
                for (int ks = 0; ks < kBKeys / 16; ++ks)
                  umma_ss(tmem_base + Cfg::kDqCol + pr * Cfg::kAcc, a_ds + ks * ((16 * 128) >> 4),
                          b_k + ks * kStep16Rows, idesc_dq, (kt > kt_lo || ks > 0) ? 1u : 0u);
              }
              umma_commit(bar(ACC_DONE + (g & 1)));
              if (js == js1 - 1) umma_commit(bar(KV_EMPTY + kvb));  // last read of this K, V
            }
            __syncwarp();
          }
          pgc += (js1 - js0 + 1) >> 1;
        }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMath));
    {
      // ------------------------------------------------------------ elementwise warps
      // Thread = one key (TMEM lane); warps w and w + 4 share the lanes and take one half
      // of the step's 64 queries each.
      const int half = warp >> 2, wq = warp & 3, t = tid & 127;
      const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
      const uint32_t tS0 = tmem_base + lane_base + half * 32;
      const uint32_t tP = tmem_base + lane_base + Cfg::kPCol + half * 16, tDS = tP + 32;
      const uint32_t tAcc = tmem_base + lane_base + Cfg::kDkCol + half * Cfg::kAcc;  // dK (half 0) or dV (half 1)
      const uint32_t tDQ = tmem_base + lane_base + Cfg::kDqCol;
      const float c1 = dm.scale * kLog2e;
      const float uniform = 1.f / (float)n;

      int g = 0, ktg = 0, pgc = 0;
      bool ok = true;
      uint32_t rng_next = item_range(blockIdx.x);
      for (int w = blockIdx.x; w < grid.total && ok; w += gridDim.x) {
        const Item im = decode(w);
        const int i = im.i, b = im.b, h = im.h;
        const int kt_lo = rng_next & 0xffffu, kt_hi = rng_next >> 16;
        rng_next = item_range(w + gridDim.x);
        // dK (warps 0-3) and dV (warps 4-7) of the key tiles nobody walks: zero
        for (int kt = 0; kt < nkt; ++kt) {
          const int key = kt * kBKeys + t;
          if ((kt < kt_lo || kt >= kt_hi) && key < n) {
            const View5& out = half ? dv : dk;
            T* dst = reinterpret_cast<T*>(out.p) + b * out.sb + h * out.sh + (int64_t)i * out.si +
                     (int64_t)key * out.sj;
#pragma unroll
            for (int e = 0; e < D; e += 8) *reinterpret_cast<uint4*>(dst + e) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        const bool row_full = rowfull[b * dm.n_rows + i] != 0;
        // key mask of the row in key order (bit set = key dropped or beyond n; on a
        // fully masked row only the keys beyond n): word kt * 4 + wq covers this warp's
        // 32 keys of key tile kt, fetched one key tile ahead
        const uint32_t* mrow = maskbits_lin + ((int64_t)b * dm.n_rows + i) * mask_words;
        for (int c = 0; c < nch && ok; ++c) {
        const int js0 = c * jsc, js1 = min(njs, js0 + jsc);
        uint32_t mword_next = __ldg(mrow + kt_lo * 4 + wq);

        for (int kt = kt_lo; kt < kt_hi && ok; ++kt, ++ktg) {
          const uint32_t mword = mword_next;
          if (kt + 1 < kt_hi) mword_next = __ldg(mrow + (kt + 1) * 4 + wq);
          const int key = kt * kBKeys + t;
          const bool dropped = ((mword >> lane) & 1u) != 0u;
          // The key weight pattern is fixed for the whole query loop of a key tile, so
          // the loop is instantiated per pattern of this warp: 0 = every key kept (no
          // selects), 1 = mixed, 2 = every key dropped (no exponentials), 3 = fully
          // masked row.
          const int mode = row_full ? 3
                           : __all_sync(0xffffffffu, !dropped) ? 0
                           : __all_sync(0xffffffffu, dropped)  ? 2
                                                               : 1;
          const int g0 = g;
          auto query_loop = [&](auto mode_tag) {
            constexpr int kMode = decltype(mode_tag)::value;
            for (int js = js0; js < js1; ++js) {
              const int gg = g0 + (js - js0);
              const int s = gg % NS;
              // S^T / dP^T of this step and its bias / lse / delta stage (implied by
              // S_FULL, whose MMAs read Q from the same stage): tested together, each
              // test being a shared-memory round trip.  The waits poll instead of
              // parking: a parked thread resumes hundreds of cycles after the phase
              // completes.
              ok = __all_sync(0xffffffffu,
                              mbar_wait_spin2(bar(S_FULL + (gg & 1)), (gg >> 1) & 1, true,
                                              bar(FULL + s), (gg / NS) & 1, abort_flag));
              if (!ok) break;
              tc_fence_after();
              float x[32], g_[32];
              const uint32_t tS = tS0 + (gg % SB) * 128;
              tmem_ld32(tS, reinterpret_cast<uint32_t*>(x));
              tmem_ld32(tS + 64, reinterpret_cast<uint32_t*>(g_));
              tmem_wait_ld();
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(S_FREE + (gg & 1)));

              // One fused pass per 8 queries: bias^T / lse / delta loads, unpack, FMAs, the
              // exponential, dS and both 16-bit packs; the dS chunk also goes to the
              // shared-memory tile (row = key, 128-byte rows, 16-byte chunks swizzled by
              // the row as the 128B TMA / UMMA swizzle does).  That tile's last reader (a
              // dQ MMA) was issued no later than the accumulating MMAs of step gg - 2,
              // which this warp waited for before its previous store.
              uint32_t pp[16], pd[16];
              {
                const uint8_t* brow = gbase + bias_off(s) + t * 128;
                const float4* lse4 = reinterpret_cast<const float4*>(gbase + lse_off(s)) + half * 8;
                const float4* del4 = reinterpret_cast<const float4*>(gbase + delta_off(s)) + half * 8;
                uint8_t* srow = gbase + pair_off((pgc + ((js - js0) >> 1)) & 1) +
                                ((js - js0) & 1) * Cfg::kHalfBytes + t * 128;
#pragma unroll
                for (int q8 = 0; q8 < 4; ++q8) {
                  const int chunk = (((half * 4 + q8) ^ (t & 7)) << 4);
                  const float4 da = del4[q8 * 2];
                  const float4 db = del4[q8 * 2 + 1];
                  const float dl[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
                  float p[8];
                  if (kMode == 2) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) p[e] = 0.f;
                  } else if (kMode == 3) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) p[e] = uniform;
                  } else {
                    const uint4 u = *reinterpret_cast<const uint4*>(brow + chunk);
                    const float4 la = lse4[q8 * 2];
                    const float4 lb = lse4[q8 * 2 + 1];
                    const float nl[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
                    float bv[8];
                    unpack2<T>(u.x, bv[0], bv[1]);
                    unpack2<T>(u.y, bv[2], bv[3]);
                    unpack2<T>(u.z, bv[4], bv[5]);
                    unpack2<T>(u.w, bv[6], bv[7]);
                    // packed fp32 pairs: two scores per FMA instruction
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                      float t0, t1, a0, a1;
                      ffma2(t0, t1, bv[e], bv[e + 1], kLog2e, kLog2e, nl[e], nl[e + 1]);
                      ffma2(a0, a1, x[q8 * 8 + e], x[q8 * 8 + e + 1], c1, c1, t0, t1);
                      p[e] = ex2(a0);
                      p[e + 1] = ex2(a1);
                    }
                  }
#pragma unroll
                  for (int e = 0; e < 8; e += 2) {
                    const int col = q8 * 8 + e;
                    float s0, s1, d0, d1;
                    ffma2(s0, s1, dl[e], dl[e + 1], -1.f, -1.f, g_[col], g_[col + 1]);   // dP - delta
                    fmul2(d0, d1, p[e], p[e + 1], s0, s1);
                    uint32_t wp = pack2<T>(p[e], p[e + 1]);
                    uint32_t wd = pack2<T>(d0, d1);
                    if (kMode == 1 || kMode == 3) {  // dropped keys weigh exactly zero
                      wp = dropped ? 0u : wp;
                      wd = dropped ? 0u : wd;
                    }
                    pp[col >> 1] = wp;
                    pd[col >> 1] = wd;
                  }
                  *reinterpret_cast<uint4*>(srow + chunk) =
                      make_uint4(pd[q8 * 4 + 0], pd[q8 * 4 + 1], pd[q8 * 4 + 2], pd[q8 * 4 + 3]);
                }
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(EMPTY + s));  // bias^T, lse, delta consumed by this warp

              if (gg >= 1) {  // the accumulating MMAs of the previous step still read P^T, dS^T
                ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(ACC_DONE + ((gg - 1) & 1)),
                                                            ((gg - 1) >> 1) & 1, abort_flag));
                if (!ok) break;
              }
              tmem_st16(tP, pp);
              tmem_st16(tDS, pd);
              tmem_wait_st();
              tc_fence_before();
              fence_proxy_async_smem();  // the dS rows in shared memory are read by an MMA
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(P_READY + (gg & 1)));
            }
          };
          switch (mode) {
            case 0: query_loop(std::integral_constant<int, 0>{}); break;
            case 1: query_loop(std::integral_constant<int, 1>{}); break;
            case 2: query_loop(std::integral_constant<int, 2>{}); break;
            default: query_loop(std::integral_constant<int, 3>{}); break;
          }
          if (!ok) break;
          g = g0 + (js1 - js0);
          pgc += (js1 - js0 + 1) >> 1;

          // dK (warps 0-3) and dV (warps 4-7) of this key tile
          {
            const int g_last = g - 1;
            ok = __all_sync(0xffffffffu, mbar_wait_spin(bar(ACC_DONE + (g_last & 1)), (g_last >> 1) & 1,
                                                        abort_flag));
            if (!ok) break;
            tc_fence_after();
            uint32_t acc[D];
            tmem_ld_cols<D>(tAcc, acc);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ACC_FREE));  // the next key tile may overwrite dK, dV
            // A row walked in several query chunks: dK / dV of a key tile are sums over the
            // chunks.  The partial of the earlier chunks waits, as fp32, in this CTA's own
            // scratch (the same thread writes and reads a given element; it stays in L2).
            if (nch > 1) {
              float4* part = reinterpret_cast<float4*>(
                  kv_scratch + ((size_t)blockIdx.x * nkt * kBKeys + (size_t)key) * (2 * D) + half * D);
              if (c > 0) {
#pragma unroll
                for (int e = 0; e < D; e += 4) {
                  const float4 pv = __ldcg(part + (e >> 2));
                  acc[e + 0] = __float_as_uint(__uint_as_float(acc[e + 0]) + pv.x);
                  acc[e + 1] = __float_as_uint(__uint_as_float(acc[e + 1]) + pv.y);
                  acc[e + 2] = __float_as_uint(__uint_as_float(acc[e + 2]) + pv.z);
                  acc[e + 3] = __float_as_uint(__uint_as_float(acc[e + 3]) + pv.w);
                }
              }
              if (c + 1 < nch) {
#pragma unroll
                for (int e = 0; e < D; e += 4)
                  __stcg(part + (e >> 2),
                         make_float4(__uint_as_float(acc[e + 0]), __uint_as_float(acc[e + 1]),
                                     __uint_as_float(acc[e + 2]), __uint_as_float(acc[e + 3])));
              }
            }
            if (key < n && c + 1 == nch) {
              const View5& out = half ? dv : dk;
              const float sc = half ? 1.f : dm.scale;
              T* dst = reinterpret_cast<T*>(out.p) + b * out.sb + h * out.sh + (int64_t)i * out.si +
                       (int64_t)key * out.sj;
#pragma unroll
              for (int e = 0; e < D; e += 8) {
                uint4 u;
                u.x = pack2<T>(__uint_as_float(acc[e + 0]) * sc, __uint_as_float(acc[e + 1]) * sc);
                u.y = pack2<T>(__uint_as_float(acc[e + 2]) * sc, __uint_as_float(acc[e + 3]) * sc);
                u.z = pack2<T>(__uint_as_float(acc[e + 4]) * sc, __uint_as_float(acc[e + 5]) * sc);
                u.w = pack2<T>(__uint_as_float(acc[e + 6]) * sc, __uint_as_float(acc[e + 7]) * sc);
                *reinterpret_cast<uint4*>(dst + e) = u;
              }
            }
          }
        }
        if (!ok) break;

        // dQ of the chunk's queries (complete with the last key tile's MMAs, waited for
        // above): warps 0-3 take the even 128-query tiles, warps 4-7 the odd ones
        // (lane = query)
        {
          tc_fence_after();
          const int jt0 = c * Cfg::kMaxJTiles;
          const int tiles = min(njt - jt0, (js1 - js0 + 1) >> 1);
          for (int jl = half; jl < tiles; jl += 2) {
            uint32_t acc[D];
            tmem_ld_cols<D>(tDQ + jl * Cfg::kAcc, acc);
            tmem_wait_ld();
            const int j = (jt0 + jl) * 128 + t;
            if (j < n) {
              T* dst = reinterpret_cast<T*>(dq.p) + b * dq.sb + h * dq.sh + (int64_t)i * dq.si +
                       (int64_t)j * dq.sj;
#pragma unroll
              for (int e = 0; e < D; e += 8) {
                uint4 v4;
                v4.x = pack2<T>(__uint_as_float(acc[e + 0]) * dm.scale, __uint_as_float(acc[e + 1]) * dm.scale);
                v4.y = pack2<T>(__uint_as_float(acc[e + 2]) * dm.scale, __uint_as_float(acc[e + 3]) * dm.scale);
                v4.z = pack2<T>(__uint_as_float(acc[e + 4]) * dm.scale, __uint_as_float(acc[e + 5]) * dm.scale);
                v4.w = pack2<T>(__uint_as_float(acc[e + 6]) * dm.scale, __uint_as_float(acc[e + 7]) * dm.scale);
                *reinterpret_cast<uint4*>(dst + e) = v4;
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(DQ_FREE));  // the next chunk's first dQ MMA may overwrite dQ
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
    if (tid == 0) atomicOr(status, (unsigned int)kStatusTimeoutBwdFused);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int D, int NS, int SB>
cudaError_t launch_fused(const BwdArgs& a, cudaStream_t stream) {
  using Cfg = FusedCfg<D, NS, SB>;
  static_assert(Cfg::kTilesBytes + 2048 <= kSmemLimit, "shared memory");
  const Dims& dm = a.dm;
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const uint64_t eb = 2;
  CUtensorMap mk, mv, mq, mdo, mbt, mlse, mdelta;
  const uint64_t dims5[5] = {(uint64_t)D, (uint64_t)dm.n, (uint64_t)dm.n_rows, (uint64_t)dm.heads,
                             (uint64_t)dm.batch};
  const uint32_t box_kv[5] = {(uint32_t)D, 128, 1, 1, 1};
  const uint32_t box_q[5] = {(uint32_t)D, (uint32_t)kBJ, 1, 1, 1};
  const CUtensorMapSwizzle swz = (CUtensorMapSwizzle)RowSwizzle<D>::kTma;
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
  auto kern = tc_dqkv_kernel<T, D, NS, SB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  FusedGrid grid;
  grid.total = dm.batch * dm.heads * dm.n_rows;
  grid.nkt = (dm.n + kBKeys - 1) / kBKeys;
  grid.njs = (dm.n + kBJ - 1) / kBJ;
  grid.njt = (dm.n + 127) / 128;
  grid.jsc = 2 * Cfg::kMaxJTiles;
  grid.nch = (grid.njt + Cfg::kMaxJTiles - 1) / Cfg::kMaxJTiles;
  if (grid.nch > 1 && !a.kv_scratch) return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  if (sms > kFusedMaxCtas) sms = kFusedMaxCtas;  // the dK / dV scratch is sized for this many CTAs
  int ctas = grid.total < sms ? grid.total : sms;
  if (a.reserve_sms > 0) {
    // A collective runs beside this kernel: leave it SMs.  Every CTA walks its items one
    // after the other, so the kernel lasts ceil(items / CTAs) items: keep at least
    // `reserve_sms` SMs free, then drop every further CTA that does not shorten that.
    // (Measured on 4 GPUs, n = 1024: with 8 SMs free the kernel takes 8 rounds instead of 7,
    // +0.11 ms, and the all-reduce stays hidden; with 1 SM free it keeps 7 rounds but the
    // all-reduce crawls and 0.20 ms of it show after the kernel.)
    const int keep = sms - a.reserve_sms > 0 ? sms - a.reserve_sms : 1;
    const int waves = (grid.total + keep - 1) / keep;
    ctas = (grid.total + waves - 1) / waves;
  }
  kern<<<ctas, Cfg::kThreads, smem, stream>>>(mk, mv, mq, mdo, mbt, mlse, mdelta, a.dq, a.dk, a.dv,
                                              a.rowfull, a.maskbits_lin, a.mask_words, a.rowrange, dm,
                                              grid, a.kv_scratch, a.status);
  return cudaGetLastError();
}

}  // namespace

// Rows whose dQ fits in TMEM next to the other accumulators are walked once; when that
// leaves 128 columns free, S^T / dP^T get a second buffer.  Longer rows are walked in
// query chunks of as many 128-query tiles as fit (8 at d = 32, 3 at d = 64), dK / dV
// being completed over the chunks through the scratch.
bool tc_bwd_fused_supported(const BwdArgs& a) {
  const int d = a.dm.d;
  if (d != 16 && d != 32 && d != 64) return false;
  if (!a.bias_t || !a.neg_lse2 || !a.maskbits_lin) return false;
  return tc_bwd_fused_chunks(a.dm.n, d) == 1 || a.kv_scratch != nullptr;
}

int tc_bwd_fused_chunks(int n, int d) {
  const int njt = (n + 127) / 128;
  const int max_tiles = (d == 16)   ? FusedCfg<16, 4, 1>::kMaxJTiles
                        : (d == 32) ? FusedCfg<32, 4, 1>::kMaxJTiles
                                    : FusedCfg<64, 2, 1>::kMaxJTiles;
  return (njt + max_tiles - 1) / max_tiles;
}

size_t tc_bwd_fused_scratch_bytes(int n, int d) {
  if (tc_bwd_fused_chunks(n, d) <= 1) return 0;
  const size_t nkt = (n + kBKeys - 1) / kBKeys;
  return (size_t)kFusedMaxCtas * nkt * kBKeys * 2 * d * sizeof(float);
}

cudaError_t tc_bwd_dqkv_fused(const BwdArgs& a, cudaStream_t s) {
  const bool bf16 = a.dtype == TRIFAST_BF16;
  if (!tc_bwd_fused_supported(a)) return cudaErrorInvalidValue;
  const int njt = (a.dm.n + 127) / 128;
  if (a.dm.d == 16) {
    if (njt <= FusedCfg<16, 4, 2>::kMaxJTiles)
      return bf16 ? launch_fused<__nv_bfloat16, 16, 4, 2>(a, s) : launch_fused<__half, 16, 4, 2>(a, s);
    return bf16 ? launch_fused<__nv_bfloat16, 16, 4, 1>(a, s) : launch_fused<__half, 16, 4, 1>(a, s);
  }
  if (a.dm.d == 32) {
    if (njt <= FusedCfg<32, 4, 2>::kMaxJTiles)
      return bf16 ? launch_fused<__nv_bfloat16, 32, 4, 2>(a, s) : launch_fused<__half, 32, 4, 2>(a, s);
    return bf16 ? launch_fused<__nv_bfloat16, 32, 4, 1>(a, s) : launch_fused<__half, 32, 4, 1>(a, s);
  }
  if (njt <= FusedCfg<64, 2, 2>::kMaxJTiles)
    return bf16 ? launch_fused<__nv_bfloat16, 64, 2, 2>(a, s) : launch_fused<__half, 64, 2, 2>(a, s);
  return bf16 ? launch_fused<__nv_bfloat16, 64, 2, 1>(a, s) : launch_fused<__half, 64, 2, 1>(a, s);
}

}  // namespace trifast
