// Planner kernels for sm_100a: token histogram, statistics exchange over NVLink peer
// memory, per-group LP solve, index redirect, and the single-launch fusion of all four.
//
// Reference counterparts (lplb/resources/csrc-tmpl/minilp.cu): kernel_count_idx :410-443,
// the communication phase of kernel_solve :109-197, its LP phase :199-401 and
// kernel_map_idx :445-515.  None of the code below is derived from them; the contracts
// that are kept are the tensor shapes of the Python API.
#pragma once

#include "common.cuh"
#include "lp_solver.cuh"

namespace lplb {

constexpr int kBlock = 256;          // threads per CTA for every planner kernel
constexpr int kWarps = kBlock / 32;
constexpr int kMaxExperts = 8192;    // logical experts supported by the shared-memory tables

// Static description of one placement (device pointers, uploaded once per mapping).
struct Topo {
  const int* r2o;       // [G, D]   source rank of replica slot d
  const int* o2r;       // [G, D]   holder rank of own bundle d
  const int* phy2log;   // [NG*G*Pl]
  const int* log2phy;   // [E, 2]   (original, replica or -1)
  const int* log2edge;  // [E]      index into probs[NG*G*D] or -1
  int n_group, g, d, ll, c, pl, e;
};

// Peer-memory exchange state.  recv[r] points at rank r's receive buffer
// uint64[2 parities][2 levels][n_ranks][E]; every word is (epoch << 32) | count.
struct Exchange {
  unsigned long long* const* recv;
  int n_ranks;
  int my_rank;
  int node_size;  // ranks per node for the two-level schedule; 0 or n_ranks = one level
  unsigned long long timeout_ns;
};

// Per-engine scratch in this GPU's memory; zero-initialised by the host once.
struct Workspace {
  uint32_t epoch;     // launches completed
  uint32_t arrive;    // CTAs of the running launch that published their counts
  uint32_t lp_done;   // epoch whose shares are ready
  uint32_t exit_cnt;  // CTAs of the running launch that finished
  uint32_t count_ticket;  // used by the stand-alone counting kernel
  uint32_t pad[3];
  // followed by: int total[2][E]; int global_cnt[E];
};
__host__ __device__ inline size_t workspace_bytes(int e) { return sizeof(Workspace) + sizeof(int) * 3 * (size_t)e; }
__device__ __forceinline__ int* ws_total(Workspace* ws, int parity, int e) {
  return reinterpret_cast<int*>(ws + 1) + (size_t)parity * e;
}
__device__ __forceinline__ int* ws_global(Workspace* ws, int e) { return reinterpret_cast<int*>(ws + 1) + 2 * (size_t)e; }

// ---------------------------------------------------------------------------------------
// Histogram of one CTA's token slice into shared memory.  Indices outside [-1, E) are
// ignored and counted in the status block.
template <typename IdxT>
__device__ __forceinline__ void histogram_slice(const IdxT* __restrict__ idx, long long begin, long long end, int e,
                                                int* __restrict__ hist, int* status, int tid = threadIdx.x,
                                                int stride = kBlock) {
  int bad = 0;
  for (long long i = begin + tid; i < end; i += stride) {
    const long long v = (long long)idx[i];
    if (v >= 0 && v < e) atomicAdd(&hist[v], 1);
    else if (v != -1) ++bad;
  }
  if (bad) {
    atomicAdd(&status[kStBadIdx], bad);
    raise_status(status, kErrBadIndex, kPhCount, bad);
  }
}

// Spread `quota` picks evenly over `total` ordinals: ordinal k is a pick iff
// floor((k+1)*quota/total) > floor(k*quota/total), i.e. (k*quota mod total) + quota >= total.
// Exactly `quota` of the ordinals 0..total-1 are picks for any 0 <= quota <= total, which
// the reference's multiplicative hash only guarantees when 499 does not divide total
// (reference minilp.cu:505).
__device__ __forceinline__ bool even_pick(unsigned k, unsigned quota, unsigned total) {
  if (quota >= total) return true;
  if (quota == 0) return false;
  unsigned rem;
  if (total <= 65536u) rem = (k * quota) % total;  // k < total, quota < total: fits in 32 bits
  else rem = (unsigned)(((unsigned long long)k * quota) % total);
  return rem + quota >= total;
}

// Quota of expert e's local tokens that stay on the original.
__device__ __forceinline__ int quota_of(int total, int edge, const float* __restrict__ probs) {
  if (edge < 0) return total;
  float p = __ldcg(&probs[edge]);  // may have been written by another CTA of this launch
  p = p != p ? 0.5f : fminf(fmaxf(p, 0.f), 1.f);
  int q = __float2int_rn(p * (float)total);
  return q < 0 ? 0 : (q > total ? total : q);
}

template <typename IdxT>
__device__ __forceinline__ void redirect_slice(const IdxT* __restrict__ idx, long long begin, long long end, int e,
                                               int* __restrict__ cur, const int* __restrict__ total,
                                               const int* __restrict__ quota, const int2* __restrict__ phys,
                                               IdxT* __restrict__ out) {
  for (long long i = begin + threadIdx.x; i < end; i += kBlock) {
    const long long v = (long long)idx[i];
    long long o = -1;
    if (v >= 0 && v < e) {
      const int2 ph = phys[v];
      const int k = atomicAdd(&cur[v], 1);
      const bool keep = ph.y < 0 || even_pick((unsigned)k, (unsigned)quota[v], (unsigned)total[v]);
      o = keep ? ph.x : ph.y;
    }
    out[i] = (IdxT)o;
  }
}

// The fused kernel touches every index twice (count, then rewrite).  Each thread keeps its
// first kKeep indices in registers between the two phases, so the index array is read from
// memory once; that matters most when the array lives in pinned host memory and every read
// crosses PCIe.  Loads are cache-volatile so a host buffer that is refilled between launches
// is never served stale.
constexpr int kKeep = 4;

template <typename IdxT>
__device__ __forceinline__ long long load_index(const IdxT* p) {
  return (long long)__ldcv(p);
}

template <typename IdxT>
__device__ __forceinline__ void histogram_keep(const IdxT* __restrict__ idx, long long begin, long long end, int e,
                                               int* __restrict__ hist, int* status, long long (&keep)[kKeep]) {
  int bad = 0;
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const long long i = begin + threadIdx.x + (long long)j * kBlock;
    keep[j] = -1;
    if (i < end) {
      const long long v = load_index(idx + i);
      keep[j] = v;
      if (v >= 0 && v < e) atomicAdd(&hist[v], 1);
      else if (v != -1) ++bad;
    }
  }
  for (long long i = begin + threadIdx.x + (long long)kKeep * kBlock; i < end; i += kBlock) {
    const long long v = load_index(idx + i);
    if (v >= 0 && v < e) atomicAdd(&hist[v], 1);
    else if (v != -1) ++bad;
  }
  if (bad) {
    atomicAdd(&status[kStBadIdx], bad);
    raise_status(status, kErrBadIndex, kPhCount, bad);
  }
}

template <typename IdxT>
__device__ __forceinline__ void redirect_keep(const IdxT* __restrict__ idx, long long begin, long long end, int e,
                                              int* __restrict__ cur, const int* __restrict__ total,
                                              const int* __restrict__ quota, const int2* __restrict__ phys,
                                              IdxT* __restrict__ out, const long long (&keep)[kKeep]) {
  auto place = [&](long long i, long long v) {
    long long o = -1;
    if (v >= 0 && v < e) {
      const int2 ph = phys[v];
      const int k = atomicAdd(&cur[v], 1);
      const bool stay = ph.y < 0 || even_pick((unsigned)k, (unsigned)quota[v], (unsigned)total[v]);
      o = stay ? ph.x : ph.y;
    }
    out[i] = (IdxT)o;
  };
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const long long i = begin + threadIdx.x + (long long)j * kBlock;
    if (i < end) place(i, keep[j]);
  }
  for (long long i = begin + threadIdx.x + (long long)kKeep * kBlock; i < end; i += kBlock) place(i, load_index(idx + i));
}

// ---------------------------------------------------------------------------------------
// Stand-alone counting kernel.  Row p of `by_cta` receives CTA p's counts; the CTA that
// finishes last turns the rows into inclusive prefixes over CTAs, so row n_cta-1 is the
// rank-local total.  No cooperative launch and no spinning: the last arriver is found
// with a ticket.
template <typename IdxT>
__global__ void __launch_bounds__(kBlock) count_kernel(const IdxT* __restrict__ idx, long long n, int e,
                                                       int* __restrict__ by_cta, Workspace* ws, int* status) {
  extern __shared__ int smem[];
  int* hist = smem;
  __shared__ bool last;
  const int p = blockIdx.x, n_cta = gridDim.x;
  for (int i = threadIdx.x; i < e; i += kBlock) hist[i] = 0;
  __syncthreads();
  histogram_slice(idx, slice_begin(n, p, n_cta, kBlock), slice_begin(n, p + 1, n_cta, kBlock), e, hist, status);
  __syncthreads();
  for (int i = threadIdx.x; i < e; i += kBlock) by_cta[(size_t)p * e + i] = hist[i];
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&ws->count_ticket, 1u) == (unsigned)n_cta - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  // Column-wise inclusive scan over the CTA rows.  Eight rows are loaded before any of them is
  // stored back, so the loads of a batch overlap instead of queueing behind the stores.
  for (int i = threadIdx.x; i < e; i += kBlock) {
    int run = 0;
    for (int r0 = 0; r0 < n_cta; r0 += 8) {
      int v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = r0 + j < n_cta ? __ldcg(&by_cta[(size_t)(r0 + j) * e + i]) : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        run += v[j];
        if (r0 + j < n_cta) by_cta[(size_t)(r0 + j) * e + i] = run;
      }
    }
  }
  if (threadIdx.x == 0) ws->count_ticket = 0;
}

// ---------------------------------------------------------------------------------------
// LP phase shared by the stand-alone solve kernel and the fused kernel.  `bundle` holds the
// per-rank bundle and fixed loads made by bundle_sums from the group-wide (already summed
// over ranks) counts.  Each warp carries 32/GP groups; a CTA covers `kWarps * 32/GP` groups
// per round.
// The success counter may be an int32 or an int64 tensor (the reference's README shows
// int64, its launcher demands int32: reference README.md:32, csrc/plugin.cpp:528-529).
struct Counter {
  void* ptr;
  int is64;
};
__device__ __forceinline__ void bump(Counter c) {
  if (c.is64) atomicAdd(reinterpret_cast<unsigned long long*>(c.ptr), 1ull);
  else atomicAdd(reinterpret_cast<int*>(c.ptr), 1);
}

// Whole-CTA prologue of the LP: fold the per-expert counts into per-rank bundle loads with one
// load per (rank, slot) spread over all threads, instead of a serial walk by the few lanes that
// solve.  bundle[rank * (D + 1) + d] = load of the rank's bundle d, [.. + D] = its fixed load.
// Integer sums, so the result does not depend on the order of the atomics.
// Only ranks [rank_begin, rank_end) are filled (a CTA of the stand-alone kernel needs its own
// groups only); `bundle` is indexed by absolute rank.
template <int D>
__device__ __forceinline__ void bundle_sums(const int* __restrict__ cnt, const Topo& tp, int* __restrict__ bundle,
                                            int rank_begin, int rank_end) {
  const int n_rep = tp.c * D;
  for (int i = rank_begin * (D + 1) + threadIdx.x; i < rank_end * (D + 1); i += kBlock) bundle[i] = 0;
  __syncthreads();
  for (int i = rank_begin * tp.ll + threadIdx.x; i < rank_end * tp.ll; i += kBlock) {
    const int rank = i / tp.ll, sl = i - rank * tp.ll;
    const int c = cnt[tp.phy2log[(size_t)rank * tp.pl + sl]];
    if (c) atomicAdd(&bundle[rank * (D + 1) + (sl < n_rep ? sl % D : D)], c);
  }
  __syncthreads();
}

template <int GP, int D>
__device__ void solve_groups(const int* __restrict__ bundle, const Topo& tp, int first_group, int group_stride,
                             IpmParams prm, float* __restrict__ probs, Counter avail, int* status) {
  constexpr int kSeg = 32 / GP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = lane / GP, li = lane % GP;
  for (int g0 = first_group + warp * kSeg; g0 < tp.n_group; g0 += group_stride) {
    const int grp = g0 + seg;
    const bool live = grp < tp.n_group && li < tp.g;
    double w[D], fixed = 0.0, f[D];
    int src[D], dst[D];
#pragma unroll
    for (int d = 0; d < D; ++d) {
      w[d] = 0.0;
      src[d] = dst[d] = li;
    }
    if (live) {
      const int* mine = bundle + ((size_t)grp * tp.g + li) * (D + 1);
      fixed = (double)mine[D];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        w[d] = (double)mine[d];
        src[d] = tp.r2o[li * D + d];
        dst[d] = tp.o2r[li * D + d];
      }
    }
    double* anchor = nullptr;
    int* anchor_valid = nullptr;
    if (live && prm.anchor != nullptr) {
      anchor = prm.anchor + ((size_t)grp * tp.g + li) * (4 * D + 3);
      anchor_valid = prm.anchor_valid + grp;
    }
    IpmOutcome res;
    if constexpr (GP == 32) res = ipm_solve_segment_ool<GP, D>(li, w, fixed, src, dst, prm, f, anchor, anchor_valid);
    else res = ipm_solve_segment<GP, D>(li, w, fixed, src, dst, prm, f, anchor, anchor_valid);
    if (live) {
#pragma unroll
      for (int d = 0; d < D; ++d) probs[((size_t)grp * tp.g + li) * D + d] = (float)f[d];
      if (li == 0) {
        if (res.converged) bump(avail);
        else {
          atomicAdd(&status[kStLpFail], 1);
          raise_status(status, kErrLpNotConverged, kPhSolve, grp);
        }
        atomicMax(&status[kStLpIters], res.iters);
      }
    }
  }
}

// Stand-alone solve kernel: one CTA per `kWarps * 32/GP` groups.  `workload` is int32[E],
// already summed over ranks by the caller.  Also writes the counts divided by their
// maximum, which the Python API returns next to the shares
// (reference csrc/plugin.cpp:504-506, :577).
template <int GP, int D>
__global__ void __launch_bounds__(kBlock) solve_kernel(const int* __restrict__ workload, Topo tp, IpmParams prm,
                                                       float* __restrict__ probs, float* __restrict__ normalised,
                                                       Counter avail, int* status) {
  __shared__ int wmax[kWarps];
  if (blockIdx.x == 0) {
    int m = 0;
    for (int i = threadIdx.x; i < tp.e; i += kBlock) m = max(m, workload[i]);
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    m = 0;
    for (int i = 0; i < kWarps; ++i) m = max(m, wmax[i]);
    const float inv = m > 0 ? 1.f / (float)m : 0.f;
    for (int i = threadIdx.x; i < tp.e; i += kBlock) normalised[i] = (float)workload[i] * inv;
    if (threadIdx.x == 0) status[kStLpIters] = 0;
    __syncthreads();
  }
  extern __shared__ int bundle[];
  constexpr int kPerCta = kWarps * (32 / GP);
  bundle_sums<D>(workload, tp, bundle, min(tp.n_group, (int)blockIdx.x * kPerCta) * tp.g,
                 min(tp.n_group, ((int)blockIdx.x + 1) * kPerCta) * tp.g);
  solve_groups<GP, D>(bundle, tp, blockIdx.x * kPerCta, gridDim.x * kPerCta, prm, probs, avail, status);
}

// ---------------------------------------------------------------------------------------
// Stand-alone redirect kernel.  Must run with the grid of the counting kernel that made
// `by_cta` (the same coupling exists in the reference, minilp.cu:468-470 and :498-499).
template <typename IdxT>
__global__ void __launch_bounds__(kBlock) redirect_kernel(const IdxT* __restrict__ idx, long long n,
                                                          const float* __restrict__ probs,
                                                          const int* __restrict__ by_cta, Topo tp,
                                                          IdxT* __restrict__ out) {
  extern __shared__ int smem[];
  const int e = tp.e, p = blockIdx.x, n_cta = gridDim.x;
  int* total = smem;
  int* cur = total + e;
  int* quota = cur + e;
  int2* phys = reinterpret_cast<int2*>(quota + e);
  for (int i = threadIdx.x; i < e; i += kBlock) {
    const int tot = by_cta[(size_t)(n_cta - 1) * e + i];
    total[i] = tot;
    cur[i] = p == 0 ? 0 : by_cta[(size_t)(p - 1) * e + i];
    quota[i] = quota_of(tot, tp.log2edge[i], probs);
    phys[i] = reinterpret_cast<const int2*>(tp.log2phy)[i];
  }
  __syncthreads();
  redirect_slice(idx, slice_begin(n, p, n_cta, kBlock), slice_begin(n, p + 1, n_cta, kBlock), e, cur, total, quota,
                 phys, out);
}

// ---------------------------------------------------------------------------------------
// All-reduce of int32[E] counts over the ranks of one NVLink domain, called by one CTA.
// Push model with the flag packed next to the data: every rank stores each count together
// with the epoch as one aligned 8-byte word into slot `my_rank` of every peer's receive
// buffer (plain st over NVLink).  An aligned 8-byte store is single-copy atomic, so a
// reader that sees the epoch in the upper half also sees the count in the lower half; no
// fence, no separate flag and no second NVLink round trip are needed.  Each thread then
// polls the words of its own elements in this GPU's memory and sums them.
// Two receive buffers alternate by epoch parity: a rank can only be one launch ahead of the
// slowest peer (it needs that peer's words of the current epoch to finish), so the buffer
// it overwrites is never still being read.  `mine` and `sum` are shared-memory arrays of E
// ints.  Returns a bit mask of peers that never arrived; their share of the sum is replaced
// by this rank's own counts.
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// One level of the exchange among the peers first_peer, first_peer + stride, ... (n_peers of
// them, this rank included): push `mine` into slot [parity][level][my_rank] of each, wait for
// their words in this rank's buffer, sum.  Adds the ranks that never arrived to `missing`.
// Counts use 31 bits.  Bit 31 of a vector's first word is the sender's `degraded` mark ("this
// vector already contains a substituted share"); a vector that arrives with it is summed as
// it is and its sender is added to `missing` too, so the report reaches every rank that used it.
__device__ __forceinline__ void exchange_level(const Exchange& ex, uint32_t epoch, int e, int level, int first_peer,
                                               int stride, int n_peers, const int* mine, int* sum,
                                               unsigned* missing, bool degraded) {
  const int parity = epoch & 1;
  const size_t level_base = ((size_t)parity * 2 + level) * ex.n_ranks;
  const unsigned long long tag = (unsigned long long)epoch << 32;
  for (int j = 0; j < n_peers; ++j) {
    const int r = first_peer + j * stride;
    unsigned long long* slot = ex.recv[r] + (level_base + ex.my_rank) * e;
    for (int i = threadIdx.x; i < e; i += kBlock) {
      const uint32_t mark = (degraded && i == 0) ? 0x80000000u : 0u;
      st_volatile_u64(&slot[i], tag | ((uint32_t)mine[i] & 0x7FFFFFFFu) | mark);
    }
  }
  const unsigned long long* base = ex.recv[ex.my_rank] + level_base * e;
  // pass 1: wait until every word of this thread's elements carries the epoch
  unsigned late = 0;
  const uint64_t t0 = global_timer_ns();
  for (int i = threadIdx.x; i < e; i += kBlock) {
    for (int j = 0; j < n_peers; ++j) {
      const int r = first_peer + j * stride;
      if ((late >> (r & 31)) & 1u) continue;
      const unsigned long long* word = &base[(size_t)r * e + i];
      uint32_t spins = 0;
      while ((uint32_t)(ld_volatile_u64(word) >> 32) != epoch) {
        if ((++spins & 63u) == 0) {
          if (global_timer_ns() - t0 > ex.timeout_ns) {
            late |= 1u << (r & 31);
            break;
          }
          __nanosleep(100);
        }
      }
    }
  }
  if (late) atomicOr(missing, late);
  __syncthreads();
  const unsigned miss = *missing;
  // pass 2: sum; an absent peer contributes this rank's own vector instead of stale data
  for (int i = threadIdx.x; i < e; i += kBlock) {
    int acc = 0;
    for (int j = 0; j < n_peers; ++j) {
      const int r = first_peer + j * stride;
      const bool absent = (miss >> (r & 31)) & 1u;
      const uint32_t word = (uint32_t)ld_volatile_u64(&base[(size_t)r * e + i]);
      if (i == 0 && !absent && (word >> 31)) atomicOr(missing, 1u << (r & 31));
      acc += absent ? mine[i] : (int)(word & 0x7FFFFFFFu);
    }
    sum[i] = acc;
  }
  __syncthreads();
}

// All-reduce over all ranks.  With ex.node_size < n_ranks it runs in two levels, the schedule
// of a machine whose ranks form nodes of node_size (the reference reduces inside a node over
// NVLink and between nodes over the network, reference minilp.cu:111-163): first among the
// ranks of this rank's node, then the node sums among the ranks with the same position in
// every node; (node_size - 1) + (n_nodes - 1) partners instead of n_ranks - 1.  `mine` is
// overwritten with the node sum in that case.
__device__ __forceinline__ unsigned exchange_counts(const Exchange& ex, uint32_t epoch, int e, int* mine, int* sum) {
  __shared__ unsigned missing;
  if (threadIdx.x == 0) missing = 0;
  __syncthreads();
  const int s = ex.node_size;
  if (s <= 0 || s >= ex.n_ranks) {
    exchange_level(ex, epoch, e, 0, 0, 1, ex.n_ranks, mine, sum, &missing, false);
  } else {
    const int node = ex.my_rank / s, local = ex.my_rank - node * s;
    exchange_level(ex, epoch, e, 0, node * s, 1, s, mine, sum, &missing, false);
    const bool degraded = missing != 0;  // every thread reads it after the level's closing barrier
    for (int i = threadIdx.x; i < e; i += kBlock) mine[i] = sum[i];
    __syncthreads();
    exchange_level(ex, epoch, e, 1, local, s, ex.n_ranks / s, mine, sum, &missing, degraded);
  }
  return missing;
}

// ---------------------------------------------------------------------------------------
// Stand-alone all-reduce of int32[E] counts over the peers (one CTA), for callers that
// feed their own statistics to the solver.  Shares the epoch with the fused kernel, so it
// keeps that kernel's invariant: the totals of the other parity are zero when it ends.
__global__ void __launch_bounds__(kBlock) exchange_kernel(const int* __restrict__ in, int e, Exchange ex,
                                                          Workspace* ws, int* __restrict__ out, int* status) {
  extern __shared__ int smem[];
  int* mine = smem;
  int* summed = smem + e;
  const uint32_t epoch = ld_acquire_gpu(&ws->epoch) + 1;
  int* other = ws_total(ws, (epoch & 1) ^ 1, e);
  for (int i = threadIdx.x; i < e; i += kBlock) {
    mine[i] = in[i];
    other[i] = 0;
  }
  __syncthreads();
  const unsigned miss = exchange_counts(ex, epoch, e, mine, summed);
  if (miss && threadIdx.x == 0) {
    atomicAdd(&status[kStTimeouts], 1);
    raise_status(status, kErrPeerTimeout, kPhExchange, (int)miss);
  }
  for (int i = threadIdx.x; i < e; i += kBlock) out[i] = summed[i];
  __syncthreads();
  if (threadIdx.x == 0) st_release_gpu(&ws->epoch, epoch);
}

// ---------------------------------------------------------------------------------------
// Single-launch planner step.  Launched cooperatively so that all CTAs are co-resident.
//
//   every CTA : histogram its slice; reserve an ordinal range per expert with one
//               returning atomicAdd on the rank-local totals; arrive.
//   CTA 0     : wait for all arrivals; exchange totals with the peers; solve the LPs
//               (one warp segment per group); publish the shares; raise lp_done.
//   every CTA : wait for lp_done; turn shares into integer quotas; rewrite its slice.
//
// The ordinal ranges come from atomics, so which CTA gets which range differs from run
// to run; quotas are exact regardless.  Shared memory: 5 int arrays of E entries plus the
// (D + 1) bundle sums per rank.
template <int GP, int D, typename IdxT>
__global__ void __launch_bounds__(kBlock) fused_run_kernel(const IdxT* __restrict__ idx, long long n, Topo tp,
                                                           Exchange ex, IpmParams prm, Workspace* ws,
                                                           float* __restrict__ probs, Counter avail, int* status,
                                                           IdxT* __restrict__ out, unsigned long long grid_timeout_ns,
                                                           unsigned long long* __restrict__ trace) {
  extern __shared__ int smem[];
  const int e = tp.e, p = blockIdx.x, n_cta = gridDim.x;
  // Optional phase stamps (globaltimer, ns) written by thread 0 of CTA 0 and by the CTA
  // that leaves last: 0 start, 1 own slice counted, 2 all CTAs arrived, 3 statistics
  // exchanged, 4 LPs solved, 5 CTA 0 redirected its slice, 6 last CTA left.
  const bool tracing = trace != nullptr && threadIdx.x == 0;
  if (tracing && p == 0) trace[0] = global_timer_ns();
  int* hist = smem;        // this CTA's counts, later the rank-local totals
  int* cur = hist + e;     // next ordinal to hand out per expert
  int* quota = cur + e;
  int2* phys = reinterpret_cast<int2*>(quota + e);
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;

  if (threadIdx.x == 0) s_epoch = ld_acquire_gpu(&ws->epoch) + 1;
  for (int i = threadIdx.x; i < e; i += kBlock) hist[i] = 0;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int parity = epoch & 1;
  int* total_g = ws_total(ws, parity, e);

  const long long begin = slice_begin(n, p, n_cta, kBlock), end = slice_begin(n, p + 1, n_cta, kBlock);
  long long keep[kKeep];
  if (p == 0) {
    // CTA 0 will run the LP: start fetching the tables it gathers from, in the shadow of the
    // counting phase (they were evicted if anything ran since the last step).
    const int n_slots = tp.n_group * tp.g * tp.pl;
    for (int i = threadIdx.x * 32; i < n_slots; i += kBlock * 32)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(tp.phy2log + i));
    if (threadIdx.x == 0) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(tp.r2o));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(tp.o2r));
    }
    if (prm.anchor != nullptr) {  // warm-start state: (4 D + 3) doubles per rank
      const int n_bytes = tp.n_group * tp.g * (4 * D + 3) * 8;
      for (int b = threadIdx.x * 128; b < n_bytes; b += kBlock * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(prm.anchor) + b));
      if (threadIdx.x == 1) asm volatile("prefetch.global.L2 [%0];" ::"l"(prm.anchor_valid));
    }
    histogram_keep(idx, begin, end, e, hist, status, keep);
  } else {
    histogram_keep(idx, begin, end, e, hist, status, keep);
    // static lookup tables, fetched while CTA 0 works (quota[] holds the edge ids for now)
    for (int i = threadIdx.x; i < e; i += kBlock) {
      quota[i] = tp.log2edge[i];
      phys[i] = reinterpret_cast<const int2*>(tp.log2phy)[i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < e; i += kBlock) {
    const int c = hist[i];
    cur[i] = c ? atomicAdd(&total_g[i], c) : 0;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) atomicAdd(&ws->arrive, 1u);

  if (p == 0) {
    if (tracing) trace[1] = global_timer_ns();
    if (threadIdx.x == 0) {
      s_ok = bounded_wait_ge<false>(&ws->arrive, (uint32_t)n_cta, grid_timeout_ns);
      if (tracing) trace[2] = global_timer_ns();
      if (!s_ok) {
        atomicAdd(&status[kStTimeouts], 1);
        raise_status(status, kErrGridTimeout, kPhCount, (int)ld_acquire_gpu(&ws->arrive));
      }
      status[kStLpIters] = 0;
    }
    __syncthreads();
    int* mine = quota;                           // reuse: local totals
    int* summed = reinterpret_cast<int*>(phys);  // reuse: group-wide totals (needs E ints of the 2E)
    int* other = ws_total(ws, parity ^ 1, e);
    for (int i = threadIdx.x; i < e; i += kBlock) {
      mine[i] = __ldcg(&total_g[i]);
      other[i] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (ex.n_ranks > 1) {
      const unsigned miss = exchange_counts(ex, epoch, e, mine, summed);
      if (miss && threadIdx.x == 0) {
        atomicAdd(&status[kStTimeouts], 1);
        raise_status(status, kErrPeerTimeout, kPhExchange, (int)miss);
      }
    } else {
      for (int i = threadIdx.x; i < e; i += kBlock) summed[i] = mine[i];
      __syncthreads();
    }
    int* glob = ws_global(ws, e);
    for (int i = threadIdx.x; i < e; i += kBlock) glob[i] = summed[i];
    if (tracing) trace[3] = global_timer_ns();
    int* bundle = reinterpret_cast<int*>(phys + e);  // past the five E-sized tables
    bundle_sums<D>(summed, tp, bundle, 0, tp.n_group * tp.g);
    solve_groups<GP, D>(bundle, tp, 0, kWarps * (32 / GP), prm, probs, avail, status);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(&ws->lp_done, epoch);
    if (tracing) trace[4] = global_timer_ns();
  }

  if (threadIdx.x == 0) {
    s_ok = bounded_wait_ge<false>(&ws->lp_done, epoch, grid_timeout_ns);
    if (!s_ok) {
      atomicAdd(&status[kStTimeouts], 1);
      raise_status(status, kErrLpTimeout, kPhRedirect, p);
    }
  }
  __syncthreads();
  const bool have_probs = s_ok;
  for (int i = threadIdx.x; i < e; i += kBlock) {
    const int tot = __ldcg(&total_g[i]);
    hist[i] = tot;
    const int edge = p == 0 ? tp.log2edge[i] : quota[i];
    quota[i] = have_probs ? quota_of(tot, edge, probs) : (edge < 0 ? tot : tot / 2);
    if (p == 0) phys[i] = reinterpret_cast<const int2*>(tp.log2phy)[i];
  }
  __syncthreads();
  redirect_keep(idx, begin, end, e, cur, hist, quota, phys, out, keep);

  __syncthreads();
  if (tracing && p == 0) trace[5] = global_timer_ns();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&ws->exit_cnt, 1u) == (unsigned)n_cta - 1) {
      ws->arrive = 0;
      ws->exit_cnt = 0;
      atomicAdd(&status[kStCalls], 1);
      st_release_gpu(&ws->epoch, epoch);
      if (trace != nullptr) trace[6] = global_timer_ns();
    }
  }
}

}  // namespace lplb
