// Dispatch planning, token dispatch over NVLink peer memory, and the final weighted
// reduction of the benchmark MoE layer (sm_100a).  The reference has no MoE layer; these
// kernels consume the planner's redirected indices for the end-to-end measurement.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "moe_gemm.cuh"

namespace lplb {
namespace moe {

constexpr int kSupportThreads = 256;
constexpr int kCombineMaxTopk = 64;
// The layer's status block: words 0-7 its own (word 0 = first error), 8-15 the counting
// kernel's, 16-31 the record of the bounds-checking build (same layout as the planner's block).
constexpr int kMoeStatusWords = 32;
constexpr int kMoeBoundsBase = 16;

__device__ __forceinline__ unsigned long long ldv_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stv_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

struct PlanArgs {
  unsigned long long* cnt_words[kMaxRanks];  // per rank: uint64 [2][n_ranks][P]
  const int* local_counts;                   // [P] pairs this rank sends to each physical expert
  int* plan;                                 // see plan_words() in moe_api.h
  int* status;
  int n_ranks, my_rank, n_local, capacity;
  int fused;  // the launch uses the fused dispatch: advance the cumulative arrival targets
  uint32_t epoch;
  unsigned long long timeout_ns;
};

// One CTA.  All-gathers the per-expert pair counts with the packed (epoch, value) words
// used by the planner's exchange, then derives for this launch:
//   rows[le], row_start[le]      rows each local expert receives and where they start
//   dst_row_start[p]             first row, on the target rank, of this rank's pairs for
//                                physical expert p
//   all_counts[src][p]
__global__ void __launch_bounds__(kSupportThreads) plan_kernel(const PlanArgs a) {
  const int P = a.n_ranks * a.n_local;
  int* rows = a.plan;
  int* row_start = rows + a.n_local;
  int* dst_row_start = row_start + a.n_local;
  int* all_counts = dst_row_start + P;
  int* tail = all_counts + a.n_ranks * P;
  const int parity = a.epoch & 1;
  const unsigned long long tag = (unsigned long long)a.epoch << 32;
  __shared__ int s_missing;
  if (threadIdx.x == 0) s_missing = 0;
  __syncthreads();
  for (int r = 0; r < a.n_ranks; ++r) {
    unsigned long long* slot = a.cnt_words[r] + ((size_t)parity * a.n_ranks + a.my_rank) * P;
    for (int i = threadIdx.x; i < P; i += kSupportThreads) stv_u64(&slot[i], tag | (uint32_t)a.local_counts[i]);
  }
  const unsigned long long* base = a.cnt_words[a.my_rank] + (size_t)parity * a.n_ranks * P;
  const uint64_t t0 = global_timer_ns();
  for (int i = threadIdx.x; i < a.n_ranks * P; i += kSupportThreads) {
    unsigned long long w = ldv_u64(&base[i]);
    uint32_t spins = 0;
    while ((uint32_t)(w >> 32) != a.epoch) {
      if ((++spins & 63u) == 0) {
        if (global_timer_ns() - t0 > a.timeout_ns) {
          s_missing = 1;
          break;
        }
        __nanosleep(100);
      }
      w = ldv_u64(&base[i]);
    }
    all_counts[i] = (uint32_t)(w >> 32) == a.epoch ? (int)(uint32_t)w : 0;
  }
  __syncthreads();
  if (s_missing && threadIdx.x == 0) atomicCAS(a.status, 0, kMoeFlagTimeout);
  // rows per expert on every rank: n[p] = sum_src all_counts[src][p]; prefix within each rank
  extern __shared__ int sm[];
  int* n_all = sm;          // [P]
  int* start_all = sm + P;  // [P] row start of expert p on its own rank
  for (int p = threadIdx.x; p < P; p += kSupportThreads) {
    int n = 0;
    for (int s = 0; s < a.n_ranks; ++s) n += all_counts[s * P + p];
    n_all[p] = n;
  }
  __syncthreads();
  if (threadIdx.x < a.n_ranks) {
    int run = 0;
    for (int le = 0; le < a.n_local; ++le) {
      start_all[threadIdx.x * a.n_local + le] = run;
      run += n_all[threadIdx.x * a.n_local + le];
    }
    if (threadIdx.x == a.my_rank) {
      tail[0] = run;
      tail[1] = run > a.capacity;
      if (run > a.capacity) atomicCAS(a.status, 0, kMoeOverflow);
    }
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += kSupportThreads) {
    int before = 0;
    for (int s = 0; s < a.my_rank; ++s) before += all_counts[s * P + p];
    dst_row_start[p] = start_all[p] + before;
  }
  int* order_base = tail + 8;
  int* send_base = order_base + P;
  int* arrive_target = send_base + P;
  int* arrive_cum = arrive_target + a.n_local;
  for (int le = threadIdx.x; le < a.n_local; le += kSupportThreads) {
    // rows past the receive buffer's capacity are dropped by the senders; clamp to match
    const int st = start_all[a.my_rank * a.n_local + le];
    const int n = n_all[a.my_rank * a.n_local + le];
    const int kept = max(0, min(n, a.capacity - st));
    rows[le] = kept;
    row_start[le] = min(st, a.capacity);
    // the fused dispatch counts landed rows cumulatively over launches
    const int cum = arrive_cum[le] + (a.fused ? kept : 0);
    arrive_cum[le] = cum;
    arrive_target[le] = cum;
  }
  if (threadIdx.x == 0) {
    // Send order of this rank's pairs: local expert index first, then target rank starting
    // with this rank and rotating, so that at any moment the eight senders aim at eight
    // different receivers while every rank's expert 0 completes first, then expert 1, ...
    int pos = 0;
    for (int le = 0; le < a.n_local; ++le)
      for (int step = 0; step < a.n_ranks; ++step) {
        const int p = ((a.my_rank + step) % a.n_ranks) * a.n_local + le;
        order_base[p] = pos;
        pos += a.local_counts[p];
      }
    tail[2] = pos;
    int slot = 0;  // return slots: physical expert order
    for (int p = 0; p < P; ++p) {
      send_base[p] = slot;
      slot += a.local_counts[p];
    }
  }
}

struct ScheduleArgs {
  const void* idx;           // [n_pairs] physical expert ids
  const int* by_cta;         // [n_cta, P] inclusive prefix rows
  const int* dst_row_start;  // [P]
  const int* order_base;     // [P]
  const int* send_base;      // [P]
  int* pair_slot;            // [n_pairs] out
  int* send_pair;            // [n_send] out
  int* send_target;          // [n_send] out
  int* status;
  long long n_pairs;
  int idx_is64, n_local, n_ranks, capacity;
};

// Same slicing as the counting kernel.  For the k-th pair this rank sends to physical expert e:
// target row dst_row_start[e] + k, return slot send_base[e] + k, send position order_base[e] + k.
__global__ void __launch_bounds__(kSupportThreads) schedule_kernel(const ScheduleArgs a) {
  extern __shared__ int sm[];
  const int P = a.n_ranks * a.n_local;
  int* cur = sm;
  const int p = blockIdx.x, n_cta = gridDim.x;
  for (int i = threadIdx.x; i < P; i += kSupportThreads) cur[i] = p == 0 ? 0 : a.by_cta[(size_t)(p - 1) * P + i];
  __syncthreads();
  const long long begin = slice_begin(a.n_pairs, p, n_cta, kSupportThreads);
  const long long end = slice_begin(a.n_pairs, p + 1, n_cta, kSupportThreads);
  for (long long i = begin + threadIdx.x; i < end; i += kSupportThreads) {
    const long long e = a.idx_is64 ? ((const long long*)a.idx)[i] : (long long)((const int*)a.idx)[i];
    int slot = -1;
    if (e >= 0 && e < P) {
      const int k = atomicAdd(&cur[e], 1);
      const int row = a.dst_row_start[e] + k;
      const int pos = a.order_base[e] + k;
      if (!LPLB_CHECKED(pos, a.n_pairs, a.status + kMoeBoundsBase, kPhRedirect)) continue;
      a.send_pair[pos] = (((int)e % a.n_local) << 20) | (int)i;  // local expert index rides along
      if (row < a.capacity) {
        slot = a.send_base[e] + k;
        a.send_target[pos] = (((int)e / a.n_local) << 24) | row;
      } else {
        a.send_target[pos] = -1;
      }
    }
    a.pair_slot[i] = slot;
  }
}

struct DispatchArgs {
  __nv_bfloat16* recv_x[kMaxRanks];  // per rank: [capacity, hidden]
  int* recv_meta[kMaxRanks];         // per rank: [capacity]
  uint32_t* flags[kMaxRanks];        // per rank: uint32 [2][n_ranks]
  const __nv_bfloat16* x;            // [tokens, hidden] local hidden states
  const void* idx;                   // [tokens * topk] physical expert ids, -1 = skip
  const int* dst_row_start;          // [P]
  const int* by_cta;                 // [n_cta, P] inclusive prefix rows from the counting kernel
  int* pair_slot;                    // [tokens * topk] out: return slot of every pair, -1 = dropped
  int* status;
  unsigned* ticket;
  long long n_pairs;
  int idx_is64, topk, hidden, n_local, n_ranks, my_rank, capacity;
  uint32_t epoch;
};

constexpr int kDispatchChunk = 1024;

// Push dispatch: CTA p owns the same slice of (token, k) pairs as CTA p of the counting
// kernel, so by_cta[p-1] is where its ordinals start.  Rows go straight into the target
// rank's receive buffer with 16-byte stores over NVLink; the last CTA to finish raises this
// rank's "dispatch done" flag on every peer.
//
// Return path: the k-th pair this rank sends to physical expert e gets return slot
// send_base[e] + k, where send_base is the exclusive prefix of this rank's own counts.  The
// slot travels with the row (meta), and the expert's rank writes the result row to that slot
// of this rank's return buffer.  Consecutive rows of an expert therefore come back to
// consecutive slots: the stores that cross NVLink walk through memory sequentially, the same
// way the dispatch stores do, instead of hitting a random page per row.
__global__ void __launch_bounds__(kSupportThreads) dispatch_kernel(const DispatchArgs a) {
  extern __shared__ int sm[];
  const int P = a.n_ranks * a.n_local;
  int* cur = sm;            // [P] next ordinal per physical expert
  int* dst_start = sm + P;  // [P]
  int* target = sm + 2 * P; // [kDispatchChunk] (rank << 24) | row, or -1
  int* send_base = target + kDispatchChunk;  // [P]
  const int p = blockIdx.x, n_cta = gridDim.x;
  for (int i = threadIdx.x; i < P; i += kSupportThreads) {
    cur[i] = p == 0 ? 0 : a.by_cta[(size_t)(p - 1) * P + i];
    dst_start[i] = a.dst_row_start[i];
  }
  if (threadIdx.x < 32) {  // exclusive prefix of this rank's totals, one warp
    int carry = 0;
    for (int i0 = 0; i0 < P; i0 += 32) {
      const int i = i0 + threadIdx.x;
      const int v = i < P ? a.by_cta[(size_t)(n_cta - 1) * P + i] : 0;
      int inc = v;
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, inc, o);
        if ((int)threadIdx.x >= o) inc += up;
      }
      if (i < P) send_base[i] = carry + inc - v;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
  }
  __syncthreads();
  const long long begin = slice_begin(a.n_pairs, p, n_cta, kSupportThreads);
  const long long end = slice_begin(a.n_pairs, p + 1, n_cta, kSupportThreads);
  const int vec_per_row = a.hidden / 8;  // 16-byte vectors per row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (long long c0 = begin; c0 < end; c0 += kDispatchChunk) {
    const int n = (int)min((long long)kDispatchChunk, end - c0);
    for (int j = threadIdx.x; j < n; j += kSupportThreads) {
      const long long i = c0 + j;
      const long long e = a.idx_is64 ? ((const long long*)a.idx)[i] : (long long)((const int*)a.idx)[i];
      int t = -1, slot = -1;
      if (e >= 0 && e < P) {
        const int k = atomicAdd(&cur[e], 1);
        const int row = dst_start[e] + k;
        if (row >= 0 && row < a.capacity) {
          const int dr = (int)e / a.n_local;
          slot = send_base[e] + k;
          if (LPLB_CHECKED(dr, a.n_ranks, a.status + kMoeBoundsBase, kPhRedirect) &&
              LPLB_CHECKED(slot, a.n_pairs, a.status + kMoeBoundsBase, kPhRedirect)) {
            t = (dr << 24) | row;
            a.recv_meta[dr][row] = (a.my_rank << 20) | slot;
          } else {
            slot = -1;
          }
        }
      }
      a.pair_slot[i] = slot;
      target[j] = t;
    }
    __syncthreads();
    for (int j = warp; j < n; j += kSupportThreads / 32) {
      const int t = target[j];
      if (t < 0) continue;
      const long long i = c0 + j;
      const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)(i / a.topk) * a.hidden);
      uint4* dst = reinterpret_cast<uint4*>(a.recv_x[t >> 24] + (size_t)(t & 0xFFFFFF) * a.hidden);
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = __ldg(&src[v]);
    }
    __syncthreads();
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(a.ticket, 1u) == (unsigned)n_cta - 1) {
      *a.ticket = 0;
      __threadfence_system();
      for (int r = 0; r < a.n_ranks; ++r) st_release_sys(a.flags[r] + a.my_rank, a.epoch);
    }
  }
}

struct CombineArgs {
  const __nv_bfloat16* comb;  // [tokens * topk, hidden] rows written by the experts' ranks
  const float* weights;       // [tokens, topk]
  const int* pair_slot;       // [tokens * topk] row of `comb` that holds each pair's result, -1 = none
  __nv_bfloat16* out;         // [tokens, hidden]
  const uint32_t* wait_flags; // this rank's "combine done" flags [n_ranks]
  int* status;
  int n_tokens, topk, hidden, n_ranks;
  uint32_t epoch;
  unsigned long long timeout_ns;
};

// out[t] = sum_k weights[t, k] * comb[pair_slot[t * topk + k]], fp32 accumulation, after every rank has
// signalled that its expert outputs for this launch are in place.
__global__ void __launch_bounds__(kSupportThreads) combine_kernel(const CombineArgs a) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint64_t t0 = global_timer_ns();
    for (int r = 0; r < a.n_ranks && ok; ++r) {
      while ((int32_t)(ld_acquire_sys(a.wait_flags + r) - a.epoch) < 0) {
        if (global_timer_ns() - t0 > a.timeout_ns) {
          ok = 0;
          atomicCAS(a.status, 0, kMoeFlagTimeout);
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
  if (!ok) return;
  const int vec_per_row = a.hidden / 8;
  // Per token: the slots and weights of its pairs go through shared memory once, then every
  // thread has the rows of up to eight pairs in flight before it starts to accumulate.
  __shared__ int s_slot[kCombineMaxTopk];
  __shared__ float s_w[kCombineMaxTopk];
  for (int t = blockIdx.x; t < a.n_tokens; t += gridDim.x) {
    __syncthreads();
    for (int k = threadIdx.x; k < a.topk; k += kSupportThreads) {
      const long long pair = (long long)t * a.topk + k;
      s_slot[k] = a.pair_slot[pair];
      s_w[k] = a.weights[pair];
    }
    __syncthreads();
    for (int v = threadIdx.x; v < vec_per_row; v += kSupportThreads) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k0 = 0; k0 < a.topk; k0 += 8) {
        uint4 raw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int slot = k0 + j < a.topk ? s_slot[k0 + j] : -1;
          raw[j] = make_uint4(0, 0, 0, 0);
          if (slot >= 0 && LPLB_CHECKED(slot, (long long)a.n_tokens * a.topk, a.status + kMoeBoundsBase, kPhRedirect))
            raw[j] = __ldcg(reinterpret_cast<const uint4*>(a.comb + (size_t)slot * a.hidden) + v);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float w = (k0 + j < a.topk && s_slot[k0 + j] >= 0) ? s_w[k0 + j] : 0.f;  // dropped pair: no term
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(h[q]);
            acc[2 * q] += w * f.x;
            acc[2 * q + 1] += w * f.y;
          }
        }
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]);
      o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]);
      o.w = pack_bf16(acc[6], acc[7]);
      reinterpret_cast<uint4*>(a.out + (size_t)t * a.hidden)[v] = o;
    }
  }
}

}  // namespace moe
}  // namespace lplb
