// Host-side launch interface of the benchmark MoE layer kernels (dispatch, grouped GEMMs,
// combine).  Plain C++ so that the CUDA translation unit needs no torch headers.
// The reference contains no MoE layer; these kernels consume the planner's redirected
// indices for the end-to-end measurement.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lplb {
namespace moe {

constexpr int kApiMaxRanks = 8;

struct LayerShape {
  int hidden;        // H
  int inter;         // I (SwiGLU width); w13 is [experts, 2*I, H], w2 is [experts, H, I]
  int n_local;       // physical experts on this rank
  int n_ranks, my_rank;
  int topk;
  int max_tokens;    // tokens per rank (upper bound)
  int capacity;      // rows of the receive buffer
};

// Pointers into this rank's own and its peers' buffers (peer entries alias the local ones
// when n_ranks == 1).
struct LayerBuffers {
  // peer-visible
  void* recv_x[kApiMaxRanks];          // bf16 [capacity, H]
  int* recv_meta[kApiMaxRanks];        // int32 [capacity]
  void* comb[kApiMaxRanks];            // bf16 [max_tokens * topk, H]
  unsigned long long* cnt_words[kApiMaxRanks];  // uint64 [2][n_ranks][n_ranks * n_local]
  uint32_t* flags[kApiMaxRanks];       // uint32 [2][n_ranks]: dispatch done, combine done
  // local
  void* act;                           // bf16 [capacity, I]
  int* plan;                           // int32 plan block, see plan_words()
  int* by_cta;                         // int32 [n_cta, n_ranks * n_local] prefix rows of the pair histogram
  int* pair_slot;                      // int32 [max_tokens * topk] return slot of every pair
  int* send_pair;                      // int32 [max_tokens * topk] pair index at every send position
  int* send_target;                    // int32 [max_tokens * topk] (rank << 24) | row, or -1
  uint32_t* arrived[kApiMaxRanks];     // per rank: uint32 [n_local] rows that have landed, cumulative
  unsigned long long* debug;           // optional uint64 [n_cta * 4] timing of the fused kernel, may be null
  void* planner_workspace;             // counting kernel workspace (ticket)
  unsigned* tickets;                   // uint32 [4], zero
  int* status;                         // int32 [16]
};

// Layout of the plan block (ints), P = n_ranks * n_local:
//   rows[n_local], row_start[n_local], dst_row_start[P], all_counts[n_ranks * P],
//   tail[8] = {total_rows, overflow, n_send, ...},
//   order_base[P]      first send position of this rank's pairs for physical expert p,
//   send_base[P]       first return slot of this rank's pairs for physical expert p,
//   arrive_target[n_local], arrive_cum[n_local]   cumulative rows expected per local expert
//                      (arrive_cum persists across launches, it is never zeroed by a launch).
inline int plan_words(int n_ranks, int n_local) {
  const int p = n_ranks * n_local;
  return 2 * n_local + p + n_ranks * p + 8 + 2 * p + 2 * n_local;
}

size_t gemm_smem_bytes();

// Encodes a 2-D bf16 row-major tensor map with 128-byte swizzle and a box of
// `box_rows` x 64 elements.  Returns 0 on success.
int make_tensor_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// Step 1: all-gather the per-expert pair counts of this launch and derive row offsets.
cudaError_t launch_plan(const LayerShape& sh, const LayerBuffers& b, int n_cta, uint32_t epoch,
                        unsigned long long timeout_ns, int fused, cudaStream_t stream);
// Step 2: copy every (token, k) pair's hidden state into its expert's rows on the target rank.
cudaError_t launch_dispatch(const LayerShape& sh, const LayerBuffers& b, const void* x, const void* phys_idx,
                            int idx_is64, int n_tokens, int n_cta, uint32_t epoch, cudaStream_t stream);
// Step 2a (fused path only): decide the send order and every pair's target row and return slot.
cudaError_t launch_schedule(const LayerShape& sh, const LayerBuffers& b, const void* phys_idx, int idx_is64,
                            int n_tokens, int n_cta, cudaStream_t stream);
// Step 2b+3 fused: the first grouped GEMM, which also streams this rank's rows to their targets
// while the tensor cores work on the experts whose rows have landed.  send_ctas == 0: four
// extra warps in every CTA send.  send_ctas > 0: that many of the n_cta CTAs only send and the
// other n_cta - send_ctas only run tiles.
cudaError_t launch_dispatch_gemm(const LayerShape& sh, const LayerBuffers& b, const CUtensorMap& tmap_a,
                                 const CUtensorMap& tmap_b, const void* x, uint32_t epoch,
                                 unsigned long long timeout_ns, int n_cta, int send_ctas, cudaStream_t stream);
// Step 3/4: grouped GEMMs.  which = 0: recv_x x w13 -> SwiGLU -> act.  which = 1: act x w2 -> peers' comb.
cudaError_t launch_gemm(const LayerShape& sh, const LayerBuffers& b, const CUtensorMap& tmap_a,
                        const CUtensorMap& tmap_b, int which, uint32_t epoch, unsigned long long timeout_ns,
                        int n_cta, cudaStream_t stream);
// Step 5: out[t] = sum_k weight[t, k] * comb[pair_slot[t * topk + k]].
cudaError_t launch_combine(const LayerShape& sh, const LayerBuffers& b, const float* weights, void* out, int n_tokens,
                           uint32_t epoch, unsigned long long timeout_ns, int n_cta, cudaStream_t stream);

}  // namespace moe
}  // namespace lplb
