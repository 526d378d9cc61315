// Sum of the fp32 bias-gradient partials of the row shards of one box, without a
// collective library: every rank pushes slice s of its partial into rank s's staging
// area with plain stores to peer-mapped memory, rank s adds the G staged slices in
// rank order (a fixed order: the result does not depend on timing) and pushes the
// reduced slice into every rank's result buffer.  Consumers only ever read local
// memory; nothing loads from a peer, and no multicast is used.
//
// One launch per rank and step, all ranks at about the same time (right after their db
// kernels), one to a few CTAs of 1024 threads each, so that it runs beside the dq / dk / dv kernel on the SMs
// that kernel leaves free.  Ranks meet twice through flag words in each other's memory
// (epoch-valued, so they never need resetting): "my pushes into your staging area have
// landed" and "my reduced slice has landed in your result".  Every wait is bounded: a
// rank that does not see its peers within the limit sets the device status word and
// returns; nothing traps.
//
// The reference is single-GPU and has no counterpart; this replaces the NCCL
// all-reduce of the row-sharded backward (trifast_b200/dist.py) on request.

#include "kernels.h"

namespace trifast {
namespace {

constexpr int kMaxWorld = 8;
constexpr long long kPeerWaitCycles = 4000000000LL;  // about two seconds

struct PushReduceParams {
  float* staging[kMaxWorld];      // staging[r]: rank r's staging area, world * slice floats (peer-mapped)
  float* result[kMaxWorld];       // result[r]: rank r's result buffer, count floats (peer-mapped)
  unsigned int* flags[kMaxWorld]; // flags[r]: rank r's 2 * kMaxWorld flag words (peer-mapped)
  const float* partial;           // this rank's partial sum (local)
  unsigned int* counters;         // this rank's two CTA counters (local, start at 0)
  long long count;                // fp32 elements
  long long slice;                // elements per rank slice (multiple of 4)
  int rank, world;
  unsigned int epoch;             // same on every rank, +1 per call, never 0
};

__device__ __forceinline__ void store_flag_system(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int load_flag_system(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs of this launch have finished (and fenced) their stores when the last one
// arrives: that CTA's thread 0 then tells every peer by writing `epoch` into word
// `base + rank` of the peer's flag array, and resets the counter for the next call.
__device__ void announce(const PushReduceParams& p, unsigned int* counter, int base) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int arrived = atomicAdd(counter, 1u);
    if (arrived == gridDim.x - 1) {
      *counter = 0u;
      __threadfence();
      for (int r = 0; r < p.world; ++r) store_flag_system(p.flags[r] + base + p.rank, p.epoch);
    }
  }
}

// Every thread waits until every peer's word (this rank's own array, local memory) shows
// the epoch; bounded.
__device__ bool await(const PushReduceParams& p, int base, int* gave_up) {
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    bool ok = true;
    for (int r = 0; r < p.world && ok; ++r) {
      while (load_flag_system(p.flags[p.rank] + base + r) != p.epoch) {
        if (clock64() - t0 > kPeerWaitCycles) {
          ok = false;
          break;
        }
        __nanosleep(200);
      }
    }
    *gave_up = ok ? 0 : 1;
  }
  __syncthreads();
  return *gave_up == 0;
}

__global__ void __launch_bounds__(1024) db_push_reduce_kernel(PushReduceParams p, unsigned int* status) {
  __shared__ int gave_up;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long slice4 = p.slice >> 2;

  // 1. scatter: slice s of the local partial -> row `rank` of rank s's staging area
  for (int s = 0; s < p.world; ++s) {
    const long long first = (long long)s * p.slice;
    float4* dst = reinterpret_cast<float4*>(p.staging[s] + (long long)p.rank * p.slice);
    const float4* src = reinterpret_cast<const float4*>(p.partial + first);
    for (long long i = tid; i < slice4; i += nthreads) {
      const long long e = first + 4 * i;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (e + 3 < p.count) {
        v = src[i];
      } else {  // ragged end of the last slice
        if (e + 0 < p.count) v.x = p.partial[e + 0];
        if (e + 1 < p.count) v.y = p.partial[e + 1];
        if (e + 2 < p.count) v.z = p.partial[e + 2];
      }
      dst[i] = v;
    }
  }
  announce(p, p.counters + 0, 0);
  if (!await(p, 0, &gave_up)) {
    if (threadIdx.x == 0) atomicOr(status, (unsigned int)kStatusTimeoutPushReduce);
    return;
  }

  // 2. reduce this rank's slice in rank order (local reads), push it to every result
  {
    const float4* st = reinterpret_cast<const float4*>(p.staging[p.rank]);
    const long long first = (long long)p.rank * p.slice;
    for (long long i = tid; i < slice4; i += nthreads) {
      // (L2 loads: the staged data arrived from the peers' stores; an L1 line from an
      // earlier call would be stale)
      float4 acc = __ldcg(st + i);
      for (int r = 1; r < p.world; ++r) {
        const float4 v = __ldcg(st + (long long)r * slice4 + i);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      const long long e = first + 4 * i;
      for (int s = 0; s < p.world; ++s) {
        float* out = p.result[s] + e;
        if (e + 3 < p.count) {
          *reinterpret_cast<float4*>(out) = acc;
        } else {
          if (e + 0 < p.count) out[0] = acc.x;
          if (e + 1 < p.count) out[1] = acc.y;
          if (e + 2 < p.count) out[2] = acc.z;
        }
      }
    }
  }
  announce(p, p.counters + 1, kMaxWorld);
  if (!await(p, kMaxWorld, &gave_up)) {
    if (threadIdx.x == 0) atomicOr(status, (unsigned int)kStatusTimeoutPushReduce);
  }
}

}  // namespace

cudaError_t db_push_reduce(const trifast_push_reduce* a, unsigned int* status, cudaStream_t s) {
  PushReduceParams p{};
  for (int r = 0; r < a->world; ++r) {
    p.staging[r] = a->staging[r];
    p.result[r] = a->result[r];
    p.flags[r] = a->flags[r];
  }
  p.partial = a->partial;
  p.counters = a->counters;
  p.count = a->count;
  p.slice = ((a->count + a->world - 1) / a->world + 3) / 4 * 4;
  p.rank = a->rank;
  p.world = a->world;
  p.epoch = a->epoch;
  // CTAs of 1024 threads: each needs an SM of its own, and all of them must run at once
  // (they meet through a counter), so the caller passes no more than it keeps SMs free
  const int ctas = a->ctas > 0 ? a->ctas : 4;
  db_push_reduce_kernel<<<ctas, 1024, 0, s>>>(p, status);
  return cudaGetLastError();
}

}  // namespace trifast
