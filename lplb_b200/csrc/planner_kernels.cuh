// Planner kernels for sm_100a: token histogram, statistics exchange over NVLink peer
// memory, per-group LP solve, index redirect, and the single-launch fusion of all four.
//
// Reference counterparts (lplb/resources/csrc-tmpl/minilp.cu): kernel_count_idx :410-443,
// the communication phase of kernel_solve :109-197, its LP phase :199-401 and
// kernel_map_idx :445-515.  None of the code below is derived from them; the contracts
// that are kept are the tensor shapes of the Python API.
#pragma once

#include "common.cuh"
#include "lp_block_solver.cuh"
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
  const int* log2slot;  // [E]      rank * (D + 1) + bundle (D = the rank's non-replicated experts)
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
  uint32_t epoch;      // launches completed
  uint32_t arrive[2];  // by launch parity: CTAs of that launch that published their counts
  uint32_t lp_done;    // epoch whose shares are ready
  uint32_t count_ticket;  // used by the stand-alone counting kernel
  uint32_t exit_cnt;   // tracing only: CTAs of the running launch that finished
  uint32_t pad[2];
  // followed by: int total[2][E]; int global_cnt[E];
};
static_assert(sizeof(Workspace) == 32, "the tables that follow the header start at byte 32");
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

// Shared-memory tables of the redirect phase.  The int2 table comes first so that it is 8-byte
// aligned for every number of experts, odd ones included.
struct RedirectTables {
  int2* phys;  // [E] (original, replica or -1)
  int* total;  // [E] rank-local tokens per expert (during counting: this CTA's counts)
  int* cur;    // [E] next ordinal to hand out
  int* quota;  // [E] ordinals that stay on the original (before the LP: the edge ids)
  int* rest;   // whatever follows the five E-sized int tables
};
__device__ __forceinline__ RedirectTables redirect_tables(int* smem, int e) {
  RedirectTables t;
  t.phys = reinterpret_cast<int2*>(smem);
  t.total = smem + 2 * (size_t)e;
  t.cur = t.total + e;
  t.quota = t.cur + e;
  t.rest = t.quota + e;
  return t;
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

// Issue the loads of the thread's first kKeep indices (slots past the slice read as -1).
template <typename IdxT>
__device__ __forceinline__ void load_keep(const IdxT* __restrict__ idx, long long begin, long long end,
                                          long long (&keep)[kKeep]) {
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const long long i = begin + threadIdx.x + (long long)j * kBlock;
    keep[j] = i < end ? load_index(idx + i) : -1;
  }
}

// Count the kept indices and whatever the slice holds beyond them.
template <typename IdxT>
__device__ __forceinline__ void histogram_keep(const IdxT* __restrict__ idx, long long begin, long long end, int e,
                                               int* __restrict__ hist, int* status, const long long (&keep)[kKeep]) {
  int bad = 0;
#pragma unroll
  for (int j = 0; j < kKeep; ++j) {
    const long long v = keep[j];
    if (v >= 0 && v < e) atomicAdd(&hist[v], 1);
    else if (v != -1) ++bad;
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
constexpr int kScanBatch = 32;  // rows of a column loaded before any is stored back

template <typename IdxT>
__global__ void __launch_bounds__(kBlock) count_kernel(const IdxT* __restrict__ idx, long long n, int e,
                                                       int* __restrict__ by_cta, Workspace* ws, int* status) {
  extern __shared__ __align__(16) int smem[];
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
  // Column-wise inclusive scan over the CTA rows.  The walk down a column is serial, so its
  // cost is the number of memory round trips: kScanBatch rows are loaded before any of them is
  // stored back, and every thread owns its own column, which keeps all of those loads in flight.
  for (int i = threadIdx.x; i < e; i += kBlock) {
    int run = 0;
    for (int r0 = 0; r0 < n_cta; r0 += kScanBatch) {
      int v[kScanBatch];
#pragma unroll
      for (int j = 0; j < kScanBatch; ++j) v[j] = r0 + j < n_cta ? __ldcg(&by_cta[(size_t)(r0 + j) * e + i]) : 0;
#pragma unroll
      for (int j = 0; j < kScanBatch; ++j) {
        run += v[j];
        if (r0 + j < n_cta) by_cta[(size_t)(r0 + j) * e + i] = run;
      }
    }
  }
  if (threadIdx.x == 0) ws->count_ticket = 0;
}

// ---------------------------------------------------------------------------------------
// LP phase shared by the stand-alone solve kernels and the fused kernel.  `bundle` holds the
// per-rank bundle and fixed loads made from the group-wide (already summed over ranks) counts.
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
// solve.  bundle[rank * (D + 1) + d] = load of the rank's bundle d, [.. + D] = its fixed load
// (D = tp.d).  Integer sums, so the result does not depend on the order of the atomics.
// Only ranks [rank_begin, rank_end) are filled (a CTA of the stand-alone kernel needs its own
// groups only); `bundle` is indexed by absolute rank.
__device__ __forceinline__ void bundle_sums(const int* __restrict__ cnt, const Topo& tp, int* __restrict__ bundle,
                                            int rank_begin, int rank_end, int* status) {
  const int dd = tp.d, n_rep = tp.c * dd;
  for (int i = rank_begin * (dd + 1) + threadIdx.x; i < rank_end * (dd + 1); i += kBlock) bundle[i] = 0;
  __syncthreads();
  for (int i = rank_begin * tp.ll + threadIdx.x; i < rank_end * tp.ll; i += kBlock) {
    const int rank = i / tp.ll, sl = i - rank * tp.ll;
    const int log = tp.phy2log[(size_t)rank * tp.pl + sl];
    if (!LPLB_CHECKED(log, tp.e, status, kPhSolve)) continue;
    const int c = cnt[log];
    if (c) atomicAdd(&bundle[rank * (dd + 1) + (sl < n_rep ? sl % dd : dd)], c);
  }
  __syncthreads();
}

__device__ __forceinline__ void report_group(const IpmOutcome& res, int grp, Counter avail, int* status) {
  if (res.converged) bump(avail);
  else {
    atomicAdd(&status[kStLpFail], 1);
    raise_status(status, kErrLpNotConverged, kPhSolve, grp);
  }
  atomicMax(&status[kStLpIters], res.iters);
  const double ppb = fmin(fmax(res.gap, 0.0) * 1e9, 2.0e9);
  atomicMax(&status[kStGapPpb], ppb == ppb ? (int)ppb : 2000000000);
}

// Warp solver: each warp carries 32/GP groups; a CTA covers `kWarps * 32/GP` groups per round.
// With SKIP_IDLE, segments past the last group do not execute the solve at all, and the lanes
// of the others are the mask of every warp-level operation in it; without it they run along on
// zeros.  Which is faster was measured per kernel: inside the fused kernel skipping saves about
// 1 us per step (one group in a warp of four segments), in the stand-alone solve kernel it
// costs 1.5-2 us per call.
template <int GP, int D, bool SKIP_IDLE = false>
__device__ __forceinline__ void solve_groups(const int* __restrict__ bundle, const Topo& tp, int first_group, int group_stride,
                             IpmParams prm, float* __restrict__ probs, Counter avail, int* status) {
  constexpr int kSeg = 32 / GP;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = lane / GP, li = lane % GP;
  for (int g0 = first_group + warp * kSeg; g0 < tp.n_group; g0 += group_stride) {
    const int live_segs = SKIP_IDLE ? min(kSeg, tp.n_group - g0) : kSeg;
    const unsigned lanes = first_lanes(live_segs * GP);
    if (seg >= live_segs) break;  // g0 + stride is past the last group for these lanes too
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
        const int s = tp.r2o[li * D + d], t = tp.o2r[li * D + d];
        if (LPLB_CHECKED(s, tp.g, status, kPhSolve) && LPLB_CHECKED(t, tp.g, status, kPhSolve)) {
          src[d] = s;
          dst[d] = t;
        }
      }
    }
    double* anchor = nullptr;
    int* anchor_valid = nullptr;
    if (live && prm.anchor != nullptr) {
      anchor = prm.anchor + ((size_t)grp * tp.g + li) * (4 * D + 3);
      anchor_valid = prm.anchor_valid + grp;
    }
    IpmOutcome res;
    if constexpr (GP == 32) res = ipm_solve_segment_ool<GP, D>(li, w, fixed, src, dst, prm, f, anchor, anchor_valid, lanes);
    else res = ipm_solve_segment<GP, D>(li, w, fixed, src, dst, prm, f, anchor, anchor_valid, lanes);
    if (live) {
#pragma unroll
      for (int d = 0; d < D; ++d) probs[((size_t)grp * tp.g + li) * D + d] = (float)f[d];
      if (li == 0) report_group(res, grp, avail, status);
    }
  }
}

// Thread-block solver: the whole CTA solves one group at a time.  DP >= tp.d is the
// instantiated replica count; slots tp.d..DP-1 are self edges of weight zero.  `scratch` is
// block_solver_smem_bytes(tp.g, DP) of shared memory, 8-byte aligned.
template <int DP>
__device__ __forceinline__ void solve_groups_block(const int* __restrict__ bundle, const Topo& tp, int first_group, int group_stride,
                                   IpmParams prm, float* __restrict__ probs, Counter avail, int* status,
                                   double* scratch) {
  const int tid = threadIdx.x, dd = tp.d;
  for (int grp = first_group; grp < tp.n_group; grp += group_stride) {
    const bool live = tid < tp.g;
    double w[DP], fixed = 0.0, f[DP];
    int src[DP], dst[DP];
#pragma unroll
    for (int d = 0; d < DP; ++d) {
      w[d] = 0.0;
      src[d] = dst[d] = tid;
    }
    if (live) {
      const int* mine = bundle + ((size_t)grp * tp.g + tid) * (dd + 1);
      fixed = (double)mine[dd];
#pragma unroll
      for (int d = 0; d < DP; ++d) {
        if (d < dd) {
          w[d] = (double)mine[d];
          const int s = tp.r2o[tid * dd + d], t = tp.o2r[tid * dd + d];
          if (LPLB_CHECKED(s, tp.g, status, kPhSolve) && LPLB_CHECKED(t, tp.g, status, kPhSolve)) {
            src[d] = s;
            dst[d] = t;
          }
        }
      }
    }
    double* anchor = nullptr;
    int* anchor_valid = nullptr;
    if (live && prm.anchor != nullptr) {
      anchor = prm.anchor + ((size_t)grp * tp.g + tid) * (4 * DP + 3);
      anchor_valid = prm.anchor_valid + grp;
    }
    const IpmOutcome res = ipm_solve_block<DP>(tid, tp.g, w, fixed, src, dst, prm, f, anchor, anchor_valid, scratch);
    if (live) {
#pragma unroll
      for (int d = 0; d < DP; ++d)
        if (d < dd) probs[((size_t)grp * tp.g + tid) * dd + d] = (float)f[d];
      if (tid == 0) report_group(res, grp, avail, status);
    }
    __syncthreads();  // the scratch area is reused by the next group
  }
}

// Counts divided by their maximum, which the Python API returns next to the shares
// (reference csrc/plugin.cpp:504-506, :577).  Called by one CTA.
__device__ __forceinline__ void normalise_counts(const int* __restrict__ workload, int e, float* __restrict__ normalised) {
  __shared__ int wmax[kWarps];
  int m = 0;
  for (int i = threadIdx.x; i < e; i += kBlock) m = max(m, workload[i]);
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  m = 0;
  for (int i = 0; i < kWarps; ++i) m = max(m, wmax[i]);
  const float inv = m > 0 ? 1.f / (float)m : 0.f;
  for (int i = threadIdx.x; i < e; i += kBlock) normalised[i] = (float)workload[i] * inv;
  __syncthreads();
}

// Stand-alone solve kernel, warp solver: one CTA per `solver_warps * 32/GP` groups.  `workload` is
// int32[E], already summed over ranks by the caller.
template <int GP, int D>
__global__ void __launch_bounds__(kBlock) solve_kernel(const int* __restrict__ workload, Topo tp, IpmParams prm,
                                                       float* __restrict__ probs, float* __restrict__ normalised,
                                                       Counter avail, int* status, int solver_warps) {
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) status[kStLpIters] = status[kStGapPpb] = 0;
    normalise_counts(workload, tp.e, normalised);
  }
  extern __shared__ __align__(16) int smem[];
  int* bundle = smem;
  // Only the first `solver_warps` warps solve (the host spreads the groups over as many SMs as
  // it can: a warp that has an SM's double-precision pipes to itself is the fastest); all
  // warps help with the bundle sums.
  const int per_cta = solver_warps * (32 / GP);
  bundle_sums(workload, tp, bundle, min(tp.n_group, (int)blockIdx.x * per_cta) * tp.g,
              min(tp.n_group, ((int)blockIdx.x + 1) * per_cta) * tp.g, status);
  if ((int)(threadIdx.x >> 5) < solver_warps)
    solve_groups<GP, D>(bundle, tp, blockIdx.x * per_cta, gridDim.x * per_cta, prm, probs, avail, status);
}

// Stand-alone solve kernel, thread-block solver: one CTA per group (the reference launches
// one block per group too, reference csrc/plugin.cpp:559-565).
// Shared memory for the bundle sums plus the slack that lets the solver's scratch area start on
// a 16-byte boundary whatever precedes the sums.
__host__ __device__ inline size_t bundle_bytes_aligned(int n_ranks, int d) {
  return ((sizeof(int) * (size_t)n_ranks * (d + 1)) + 15 + 16) & ~(size_t)15;
}
__device__ __forceinline__ double* scratch_after(int* bundle, int n_ranks, int d) {
  const uintptr_t end = reinterpret_cast<uintptr_t>(bundle + (size_t)n_ranks * (d + 1));
  return reinterpret_cast<double*>((end + 15) & ~(uintptr_t)15);
}
template <int DP>
__global__ void __launch_bounds__(kBlock) solve_block_kernel(const int* __restrict__ workload, Topo tp, IpmParams prm,
                                                             float* __restrict__ probs,
                                                             float* __restrict__ normalised, Counter avail,
                                                             int* status) {
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) status[kStLpIters] = status[kStGapPpb] = 0;
    normalise_counts(workload, tp.e, normalised);
  }
  extern __shared__ __align__(16) int smem[];
  int* bundle = smem;
  double* scratch = scratch_after(bundle, tp.n_group * tp.g, tp.d);
  const int grp = blockIdx.x;
  bundle_sums(workload, tp, bundle, grp * tp.g, (grp + 1) * tp.g, status);
  solve_groups_block<DP>(bundle, tp, grp, gridDim.x, prm, probs, avail, status, scratch);
}

// ---------------------------------------------------------------------------------------
// Stand-alone redirect kernel.  Must run with the grid of the counting kernel that made
// `by_cta` (the same coupling exists in the reference, minilp.cu:468-470 and :498-499).
template <typename IdxT>
__global__ void __launch_bounds__(kBlock) redirect_kernel(const IdxT* __restrict__ idx, long long n,
                                                          const float* __restrict__ probs,
                                                          const int* __restrict__ by_cta, Topo tp,
                                                          IdxT* __restrict__ out) {
  extern __shared__ __align__(16) int smem[];
  const int e = tp.e, p = blockIdx.x, n_cta = gridDim.x;
  const RedirectTables tb = redirect_tables(smem, e);
  for (int i = threadIdx.x; i < e; i += kBlock) {
    const int tot = by_cta[(size_t)(n_cta - 1) * e + i];
    tb.total[i] = tot;
    tb.cur[i] = p == 0 ? 0 : by_cta[(size_t)(p - 1) * e + i];
    tb.quota[i] = quota_of(tot, tp.log2edge[i], probs);
    tb.phys[i] = reinterpret_cast<const int2*>(tp.log2phy)[i];
  }
  __syncthreads();
  redirect_slice(idx, slice_begin(n, p, n_cta, kBlock), slice_begin(n, p + 1, n_cta, kBlock), e, tb.cur, tb.total,
                 tb.quota, tb.phys, out);
}

// ---------------------------------------------------------------------------------------
// All-reduce of int32[E] counts over the ranks of one NVLink domain, called by one CTA.
// Push model with the flag packed next to the data: every rank stores each count together
// with the epoch as one aligned 8-byte word into slot `my_rank` of every peer's receive
// buffer (plain st over NVLink).  An aligned 8-byte store is single-copy atomic, so a
// reader that sees the epoch in the upper half also sees the count in the lower half; no
// fence, no separate flag and no second NVLink round trip are needed.  Each thread then
// polls the words of its own elements in this GPU's memory and sums them as they arrive.
// Two receive buffers alternate by epoch parity: a rank can only be one launch ahead of the
// slowest peer (it needs that peer's words of the current epoch to finish), so the buffer
// it overwrites is never still being read.
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Two adjacent words in one 16-byte store.  Each 8-byte half carries its own epoch, so it does
// not matter whether the two halves become visible together.
__device__ __forceinline__ void st_volatile_u64x2(unsigned long long* p, unsigned long long a, unsigned long long b) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

constexpr int kMaxRanks = 32;     // peers of one exchange (bit masks are 32 bits wide)
constexpr int kPollChunk = 8;     // peers whose words one thread keeps in flight per polling pass
constexpr int kSpinsBeforeSleep = 512;

// Shared state of one exchange call.  `recv` is a copy of the peers' buffer addresses in shared
// memory (filled by exchange_prepare in the shadow of other work), so the exchange itself
// starts without a dependent global load.
struct ExchangeShared {
  unsigned long long* recv[kMaxRanks];
  unsigned missing;  // peers that never arrived
  unsigned marked;   // peers whose vector carried the sender's `degraded` mark
};
// Barrier among the first NT threads of the CTA (all of them: the ordinary block barrier).
template <int NT>
__device__ __forceinline__ void team_sync() {
  if constexpr (NT == kBlock) __syncthreads();
  else asm volatile("bar.sync 2, %0;" ::"n"(NT) : "memory");
}

__device__ __forceinline__ void exchange_prepare(const Exchange& ex, ExchangeShared* xs) {
  if (threadIdx.x < kMaxRanks) xs->recv[threadIdx.x] = (int)threadIdx.x < ex.n_ranks && ex.recv != nullptr ? ex.recv[threadIdx.x] : nullptr;
  if (threadIdx.x == 0) xs->missing = xs->marked = 0;
}

// One level of the exchange among the peers first_peer, first_peer + stride, ... (n_peers of
// them, this rank included): push `vec` into slot [parity][level][my_rank] of each, wait for
// their words in this rank's buffer, and replace `vec` by the sum.  Ranks that never arrived go
// to xs->missing; their share of the sum is this rank's own vector instead.  Counts use 31
// bits.  Bit 31 of a vector's first word is the sender's `degraded` mark ("this vector already
// contains a substituted share"); such a vector is summed as it is and its sender goes to
// xs->marked, which the caller folds into the report once the level has ended.
// `xtrace` (thread 0 only, may be null) receives four stamps: own pushes issued, first and
// last word of another peer seen (for element 0), and that last peer's rank.
// Called by the first NT threads of the CTA.
template <int NT>
__device__ __forceinline__ void exchange_level(const Exchange& ex, ExchangeShared* xs, uint32_t epoch, int e, int level,
                                               int first_peer, int stride, int n_peers, int* vec, bool degraded,
                                               int* status, unsigned long long* xtrace) {
  const int parity = epoch & 1;
  const size_t level_base = ((size_t)parity * 2 + level) * ex.n_ranks;
  const unsigned long long tag = (unsigned long long)epoch << 32;
  const size_t my_slot = (level_base + ex.my_rank) * e;
  // ---- push: all peers' stores are issued back to back, nothing waits in between -----------
  if ((e & 1) == 0) {
    const int half = e >> 1, items = n_peers * half;
    for (int it = threadIdx.x; it < items; it += NT) {
      const int j = it / half, pr = it - j * half, r = first_peer + j * stride;
      if (!LPLB_CHECKED(r, ex.n_ranks, status, kPhExchange)) continue;
      const uint32_t mark = (degraded && pr == 0) ? 0x80000000u : 0u;
      st_volatile_u64x2(xs->recv[r] + my_slot + 2 * pr, tag | ((uint32_t)vec[2 * pr] & 0x7FFFFFFFu) | mark,
                        tag | ((uint32_t)vec[2 * pr + 1] & 0x7FFFFFFFu));
    }
  } else {
    const int items = n_peers * e;
    for (int it = threadIdx.x; it < items; it += NT) {
      const int j = it / e, i = it - j * e, r = first_peer + j * stride;
      if (!LPLB_CHECKED(r, ex.n_ranks, status, kPhExchange)) continue;
      const uint32_t mark = (degraded && i == 0) ? 0x80000000u : 0u;
      st_volatile_u64(xs->recv[r] + my_slot + i, tag | ((uint32_t)vec[i] & 0x7FFFFFFFu) | mark);
    }
  }
  const bool stamping = xtrace != nullptr && threadIdx.x == 0;
  if (stamping) xtrace[0] = global_timer_ns();
  team_sync<NT>();  // every thread has read the `vec` entries it pushes; they may be overwritten now
  // ---- poll and sum: one pass over all peers per element, kPollChunk loads in flight --------
  const unsigned long long* base = xs->recv[ex.my_rank] + level_base * e;
  unsigned late = 0;
  bool seen_any = false;
  const uint64_t t0 = global_timer_ns();
  for (int i = threadIdx.x; i < e; i += NT) {
    int acc = 0;
    for (int j0 = 0; j0 < n_peers; j0 += kPollChunk) {
      const int nj = min(kPollChunk, n_peers - j0);
      unsigned pend = (1u << nj) - 1u;
#pragma unroll
      for (int b = 0; b < kPollChunk; ++b)
        if (b < nj && ((late >> ((first_peer + (j0 + b) * stride) & 31)) & 1u)) pend &= ~(1u << b);
      uint32_t spins = 0;
      while (pend) {
        unsigned long long v[kPollChunk];
#pragma unroll
        for (int b = 0; b < kPollChunk; ++b)
          if ((pend >> b) & 1u) v[b] = ld_volatile_u64(&base[(size_t)(first_peer + (j0 + b) * stride) * e + i]);
#pragma unroll
        for (int b = 0; b < kPollChunk; ++b) {
          if (((pend >> b) & 1u) && (uint32_t)(v[b] >> 32) == epoch) {
            const uint32_t word = (uint32_t)v[b];
            const int r = first_peer + (j0 + b) * stride;
            acc += (int)(word & 0x7FFFFFFFu);
            if (i == 0 && (word >> 31)) atomicOr(&xs->marked, 1u << (r & 31));
            pend &= ~(1u << b);
            if (stamping && i == 0 && r != ex.my_rank) {
              const unsigned long long now = global_timer_ns();
              if (!seen_any) xtrace[1] = now;
              seen_any = true;
              xtrace[2] = now;
              xtrace[3] = (unsigned long long)r;
            }
          }
        }
        if (pend && (++spins & 63u) == 0) {
          if (global_timer_ns() - t0 > ex.timeout_ns) {
#pragma unroll
            for (int b = 0; b < kPollChunk; ++b)
              if ((pend >> b) & 1u) late |= 1u << ((first_peer + (j0 + b) * stride) & 31);
            break;
          }
          if (spins > kSpinsBeforeSleep) __nanosleep(100);
        }
      }
    }
    vec[i] = acc;
  }
  if (late) atomicOr(&xs->missing, late);
  team_sync<NT>();
  const unsigned miss = xs->missing;
  if (miss) {
    // Rare path: a peer is absent for at least one element, so it is absent for all of them.
    // This rank's own vector is still in its own slot of the receive buffer.
    for (int i = threadIdx.x; i < e; i += NT) {
      const int own = (int)((uint32_t)ld_volatile_u64(&base[(size_t)ex.my_rank * e + i]) & 0x7FFFFFFFu);
      int acc = 0;
      for (int j = 0; j < n_peers; ++j) {
        const int r = first_peer + j * stride;
        const bool absent = (miss >> (r & 31)) & 1u;
        const uint32_t word = (uint32_t)ld_volatile_u64(&base[(size_t)r * e + i]);
        acc += absent ? own : (int)(word & 0x7FFFFFFFu);
      }
      vec[i] = acc;
    }
    team_sync<NT>();
  }
}

// All-reduce over all ranks, in place in `vec` (shared memory, E ints).  With ex.node_size <
// n_ranks it runs in two levels, the schedule of a machine whose ranks form nodes of node_size
// (the reference reduces inside a node over NVLink and between nodes over the network,
// reference minilp.cu:111-163): first among the ranks of this rank's node, then the node sums
// among the ranks with the same position in every node; (node_size - 1) + (n_nodes - 1)
// partners instead of n_ranks - 1.  Returns a bit mask of the peers that never arrived or sent
// a marked vector.  exchange_prepare must have run, followed by a block barrier.
template <int NT>
__device__ __forceinline__ unsigned exchange_counts(const Exchange& ex, ExchangeShared* xs, uint32_t epoch, int e,
                                                    int* vec, int* status, unsigned long long* xtrace) {
  const int s = ex.node_size;
  if (s <= 0 || s >= ex.n_ranks) {
    exchange_level<NT>(ex, xs, epoch, e, 0, 0, 1, ex.n_ranks, vec, false, status, xtrace);
  } else {
    const int node = ex.my_rank / s, local = ex.my_rank - node * s;
    exchange_level<NT>(ex, xs, epoch, e, 0, node * s, 1, s, vec, false, status, xtrace);
    const bool degraded = xs->missing != 0;  // every thread reads it after the level's closing barrier
    exchange_level<NT>(ex, xs, epoch, e, 1, local, s, ex.n_ranks / s, vec, degraded, status,
                       xtrace != nullptr ? xtrace + 4 : nullptr);
  }
  return xs->missing | xs->marked;  // both final: the last level ended with a block barrier
}

// ---------------------------------------------------------------------------------------
// Stand-alone all-reduce of int32[E] counts over the peers (one CTA), for callers that
// feed their own statistics to the solver.  Shares the epoch with the fused kernel, so it
// keeps that kernel's invariant: the totals of the other parity are zero when it ends.
__global__ void __launch_bounds__(kBlock) exchange_kernel(const int* __restrict__ in, int e, Exchange ex,
                                                          Workspace* ws, int* __restrict__ out, int* status) {
  extern __shared__ __align__(16) int smem[];
  __shared__ ExchangeShared xs;
  int* vec = smem;
  const uint32_t epoch = ld_acquire_gpu(&ws->epoch) + 1;
  int* other = ws_total(ws, (epoch & 1) ^ 1, e);
  exchange_prepare(ex, &xs);
  for (int i = threadIdx.x; i < e; i += kBlock) {
    vec[i] = in[i];
    other[i] = 0;
  }
  __syncthreads();
  const unsigned miss = exchange_counts<kBlock>(ex, &xs, epoch, e, vec, status, nullptr);
  if (miss && threadIdx.x == 0) {
    atomicAdd(&status[kStTimeouts], 1);
    raise_status(status, kErrPeerTimeout, kPhExchange, (int)miss);
  }
  for (int i = threadIdx.x; i < e; i += kBlock) out[i] = vec[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    ws->arrive[(epoch & 1) ^ 1] = 0;  // every launch leaves the next one's arrival counter at zero
    st_release_gpu(&ws->epoch, epoch);
  }
}

// ---------------------------------------------------------------------------------------
// Single-launch planner step.  Launched cooperatively so that all CTAs are co-resident.
//
//   CTAs 1..n  ("workers"): histogram their slice of the indices; reserve an ordinal range per
//                expert with one returning atomicAdd on the rank-local totals; arrive.
//   CTA 0      ("solver"):  meanwhile pulls the solver's inputs into its caches; waits for the
//                arrivals; exchanges the totals with the peers; solves the LPs; publishes the
//                shares; raises lp_done.
//   workers:     wait for lp_done; turn shares into integer quotas; rewrite their slice.
//
// The solver CTA touches no indices.  Its code path shares no registers with the workers' (the
// workers keep indices and table pointers live across their wait; inlined into one path with
// the solver they cost it the registers it needs for its own instruction-level parallelism),
// and because it is always CTA 0 the solver's code, some two thousand straight-line
// instructions per iteration, stays in one SM's instruction cache from launch to launch.  Both
// were measured: with the CTA that delivers the last counts doing the solve instead, on
// whichever SM that is, the step's 90th percentile went from 27 to 41 us.
//
// The ordinal ranges come from atomics, so which worker gets which range differs from run
// to run; quotas are exact regardless.  Shared memory: the five E-sized redirect tables
// (workers) or the statistics vector (solver), the (D + 1) bundle sums per rank, and for
// GP == 0 the scratch area of the thread-block solver.  GP = 8, 16, 32 selects the warp solver
// for groups of up to GP ranks, GP = 0 the thread-block solver for any group size; D is the
// instantiated replica count (>= tp.d when GP == 0).
constexpr int kTraceWords = 16;

// Optional phase stamps (globaltimer, ns): 0 solver CTA started, 1 first worker arrived, 2 all
// counts in, 3 statistics exchanged, 4 LPs solved, 5 first worker redirected its slice, 6 last
// worker left; 8-11 and 12-15 the stamps of the two exchange levels (see exchange_level).
template <int GP, int D>
__device__ __forceinline__ void solver_cta(Topo tp, const Exchange& ex, IpmParams prm, Workspace* ws,
                                           float* __restrict__ probs, Counter avail, int* status, int n_workers,
                                           unsigned long long grid_timeout_ns, unsigned long long* __restrict__ trace,
                                           int* smem) {
  const int e = tp.e;
  const bool tracing = trace != nullptr && threadIdx.x == 0;
  if (tracing) trace[0] = global_timer_ns();
  __shared__ uint32_t s_epoch;
  __shared__ ExchangeShared xs;
  if (threadIdx.x == 0) s_epoch = ld_acquire_gpu(&ws->epoch) + 1;
  // The solver's inputs go to L2 and to this SM's L1 while the workers count (they were
  // evicted if anything ran since the last step).
  {
    const int ranks = tp.n_group * tp.g;
    for (int b = threadIdx.x * 128; b < e * 4; b += kBlock * 128)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const char*>(tp.log2slot) + b));
    for (int b = threadIdx.x * 128; b < tp.g * tp.d * 4; b += kBlock * 128) {
      asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const char*>(tp.r2o) + b));
      asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const char*>(tp.o2r) + b));
    }
    if (prm.anchor != nullptr) {  // warm-start state: (4 D + 3) doubles per rank
      for (int b = threadIdx.x * 128; b < ranks * (4 * D + 3) * 8; b += kBlock * 128)
        asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const char*>(prm.anchor) + b));
      if (threadIdx.x == 0) asm volatile("prefetch.global.L1 [%0];" ::"l"(prm.anchor_valid));
    }
  }
  exchange_prepare(ex, &xs);
  __shared__ int s_stop;
  if (threadIdx.x == 0) s_stop = 0;
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int parity = epoch & 1;
  int* total_g = ws_total(ws, parity, e);
  int* vec = smem;  // rank-local, then group-wide totals
  int* bundle = smem + e;
  constexpr int NT = kBlock;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 1) {
    if (lane == 0) {
      if (!bounded_wait_ge<false>(&ws->arrive[parity], (uint32_t)n_workers, grid_timeout_ns)) {
        atomicAdd(&status[kStTimeouts], 1);
        raise_status(status, kErrGridTimeout, kPhCount, (int)ld_acquire_gpu(&ws->arrive[parity]));
      }
      *reinterpret_cast<volatile int*>(&s_stop) = 1;  // ends the rehearsal
      if (trace != nullptr) trace[2] = global_timer_ns();
      status[kStLpIters] = 0;
      status[kStGapPpb] = 0;
      // Every worker of this launch has read the launch number, so the bookkeeping for the next
      // launch can be done here: its arrival counter starts at zero and it will see this launch
      // as completed (launches of one engine are stream-ordered).
      ws->arrive[parity ^ 1] = 0;
      ws->epoch = epoch;
      atomicAdd(&status[kStCalls], 1);
    }
  } else if (warp == 0) {
    if constexpr (GP != 0) {
      // Rehearsal while the workers count: the warp that will solve runs the solver on made-up
      // loads until the counts are in.  Whatever ran since the last step has evicted the
      // solver's code from the caches, the instruction caches included, and one warp running
      // two thousand straight-line instructions per iteration waits for every line of it; here
      // it takes the first of those waits while it has nothing else to do.  Nothing it
      // computes is kept.
      const int li = lane, g = tp.g;
      if (lane < GP) {
      double w[D], f[D];
      int src[D], dst[D];
#pragma unroll
      for (int d = 0; d < D; ++d) {
        const bool real = li < g && (d + 1) % g != 0;
        w[d] = real ? 1.0 + 0.37 * li + 0.11 * d : 0.0;
        src[d] = real ? (li + d + 1) % g : li;
        dst[d] = real ? (li + g - (d + 1) % g) % g : li;
      }
      IpmParams rehearsal{3, 0.0};
      rehearsal.stop = &s_stop;
      ipm_solve_segment<GP, D>(li, w, li < g ? 3.0 + 0.2 * li : 0.0, src, dst, rehearsal, f, nullptr, nullptr,
                               first_lanes(GP));
      }
    }
  }
  team_sync<NT>();
  // the workers' counts are in total_g: their atomics precede their arrivals
  int* other = ws_total(ws, parity ^ 1, e);
  const int first = threadIdx.x;
  const int first_slot = first < e ? tp.log2slot[first] : 0;  // in flight while the exchange runs
  for (int i = threadIdx.x; i < e; i += NT) {
    vec[i] = __ldcg(&total_g[i]);
    other[i] = 0;  // ready for the next launch
  }
  team_sync<NT>();
  if (ex.n_ranks > 1) {
    const unsigned miss = exchange_counts<NT>(ex, &xs, epoch, e, vec, status, trace != nullptr ? trace + 8 : nullptr);
    if (miss) {
      // Shares made from substituted statistics must not become the next warm start, and the
      // saved iterate may no longer match the peers': this solve and the next one start cold.
      if (prm.anchor_valid != nullptr)
        for (int g = threadIdx.x; g < tp.n_group; g += NT) prm.anchor_valid[g] = 0;
      prm.anchor = nullptr;
      prm.anchor_valid = nullptr;
      if (threadIdx.x == 0) {
        atomicAdd(&status[kStTimeouts], 1);
        raise_status(status, kErrPeerTimeout, kPhExchange, (int)miss);
      }
    }
  }
  if (tracing) trace[3] = global_timer_ns();
  // group-wide counts -> per-rank bundle loads, and a copy for the host
  int* glob = ws_global(ws, e);
  const int n_bundle = tp.n_group * tp.g * (tp.d + 1);
  for (int i = threadIdx.x; i < n_bundle; i += NT) bundle[i] = 0;
  team_sync<NT>();
  for (int i = threadIdx.x; i < e; i += NT) {
    const int c = vec[i];
    glob[i] = c;
    const int slot = i == first ? first_slot : tp.log2slot[i];
    if (c && LPLB_CHECKED(slot, n_bundle, status, kPhSolve)) atomicAdd(&bundle[slot], c);
  }
  team_sync<NT>();
  if constexpr (GP == 0) {
    solve_groups_block<D>(bundle, tp, 0, 1, prm, probs, avail, status, scratch_after(bundle, tp.n_group * tp.g, tp.d));
  } else {
    solve_groups<GP, D, true>(bundle, tp, 0, (NT / 32) * (32 / GP), prm, probs, avail, status);
  }
  __threadfence();
  team_sync<NT>();
  if (threadIdx.x == 0) st_release_gpu(&ws->lp_done, epoch);
  if (tracing) trace[4] = global_timer_ns();
}

template <typename IdxT>
__device__ __forceinline__ void worker_cta(const IdxT* __restrict__ idx, long long n, const Topo& tp, Workspace* ws,
                                           const float* __restrict__ probs, int* status, IdxT* __restrict__ out,
                                           int q, int n_workers, unsigned long long grid_timeout_ns,
                                           unsigned long long* __restrict__ trace, int* smem) {
  const int e = tp.e;
  const bool tracing = trace != nullptr && threadIdx.x == 0 && q == 0;
  const RedirectTables tb = redirect_tables(smem, e);
  int* hist = tb.total;  // this CTA's counts, later the rank-local totals
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  // Everything that does not depend on the launch number is issued before the first barrier:
  // the launch number itself, this thread's indices, the static lookup tables.
  if (threadIdx.x == 0) s_epoch = ld_acquire_gpu(&ws->epoch) + 1;
  const long long begin = slice_begin(n, q, n_workers, kBlock), end = slice_begin(n, q + 1, n_workers, kBlock);
  long long keep[kKeep];
  load_keep(idx, begin, end, keep);
  for (int i = threadIdx.x; i < e; i += kBlock) {
    hist[i] = 0;
    tb.quota[i] = tp.log2edge[i];  // the edge ids, until the shares are known
    tb.phys[i] = reinterpret_cast<const int2*>(tp.log2phy)[i];
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  int* total_g = ws_total(ws, epoch & 1, e);
  histogram_keep(idx, begin, end, e, hist, status, keep);
  __syncthreads();
  for (int i = threadIdx.x; i < e; i += kBlock) {
    const int c = hist[i];
    tb.cur[i] = c ? atomicAdd(&total_g[i], c) : 0;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(&ws->arrive[epoch & 1], 1u);
    if (tracing) trace[1] = global_timer_ns();
    s_ok = bounded_wait_ge<false>(&ws->lp_done, epoch, grid_timeout_ns);
    if (!s_ok) {
      atomicAdd(&status[kStTimeouts], 1);
      raise_status(status, kErrLpTimeout, kPhRedirect, q);
    }
  }
  __syncthreads();
  const bool have_probs = s_ok;
  for (int i = threadIdx.x; i < e; i += kBlock) {
    const int tot = __ldcg(&total_g[i]);
    tb.total[i] = tot;
    const int edge = tb.quota[i];
    tb.quota[i] = have_probs ? quota_of(tot, edge, probs) : (edge < 0 ? tot : tot / 2);
  }
  __syncthreads();
  redirect_keep(idx, begin, end, e, tb.cur, tb.total, tb.quota, tb.phys, out, keep);
  if (trace != nullptr) {  // tracing only: find the worker that leaves last
    __syncthreads();
    if (tracing) trace[5] = global_timer_ns();
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(&ws->exit_cnt, 1u) == (unsigned)n_workers - 1) {
        ws->exit_cnt = 0;
        trace[6] = global_timer_ns();
      }
    }
  }
}

// Grid = 1 solver CTA + (gridDim.x - 1) worker CTAs.
template <int GP, int D, typename IdxT>
__global__ void __launch_bounds__(kBlock) fused_run_kernel(const IdxT* __restrict__ idx, long long n, Topo tp,
                                                           Exchange ex, IpmParams prm, Workspace* ws,
                                                           float* __restrict__ probs, Counter avail, int* status,
                                                           IdxT* __restrict__ out, unsigned long long grid_timeout_ns,
                                                           unsigned long long* __restrict__ trace) {
  extern __shared__ __align__(16) int smem[];
  const int n_workers = (int)gridDim.x - 1;
  if (blockIdx.x == 0) solver_cta<GP, D>(tp, ex, prm, ws, probs, avail, status, n_workers, grid_timeout_ns, trace, smem);
  else worker_cta<IdxT>(idx, n, tp, ws, probs, status, out, (int)blockIdx.x - 1, n_workers, grid_timeout_ns, trace, smem);
}

}  // namespace lplb
