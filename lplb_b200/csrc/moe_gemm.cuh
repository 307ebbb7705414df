// Grouped expert GEMM for the benchmark MoE layer on sm_100a: bf16 x bf16 -> fp32 on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory), operands staged
// by TMA into 128-byte-swizzled shared memory, persistent warp-specialised CTAs.
//
//   C_e[rows_e, N] = A_e[rows_e, K] * B_e[N, K]^T        for every local expert e
//
// A is the row-major receive buffer (all experts' rows back to back, expert e starts at
// row_start[e]); B is the weight tensor [experts * N, K].  Rows per expert are only known
// on the device, so the tile list is derived in-kernel from `rows`.
//
// Roles inside a CTA (192 threads):
//   warp 0      TMA producer: A tile 128 x 64 and B tile 256 x 64 per stage, 4 stages
//   warp 1      allocates 512 TMEM columns, issues tcgen05.mma (one elected lane)
//   warps 2-5   epilogue: tcgen05.ld their 32-lane quarter, apply the epilogue, store
// Two 128 x 256 fp32 accumulators (2 x 256 TMEM columns) let the epilogue of tile i overlap
// the main loop of tile i+1.
//
// Epilogues:
//   kSwiGLU   columns [0,128) of a tile are gate, [128,256) the matching up projections
//             (the weight rows are stored in that order); writes silu(gate)*up as bf16
//             into act[row, n_tile*128 + c].
//   kScatter  converts to bf16 and stores each row to the buffer of the GPU the token came
//             from (peer memory over NVLink), at the return slot meta[row] & 0xFFFFF: this is the
//             combine step of the MoE layer fused into the last GEMM.
//
// The reference has no MoE layer; this kernel exists for the end-to-end benchmark.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include "tcgen05.cuh"

namespace lplb {
namespace moe {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4, kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;
constexpr uint32_t kStageBytesA = kBM * kBK * 2, kStageBytesB = kBN * kBK * 2;
// per epilogue warp: 32 rows x 128 bf16 columns, staged so that rows leave as 256-byte segments
constexpr uint32_t kStageOutBytes = 32 * 128 * 2;
constexpr size_t kGemmSmem = 1024 + (size_t)kStages * (kStageBytesA + kStageBytesB) + 256 + 4 * kStageOutBytes;
constexpr int kMaxLocalExperts = 128;
constexpr int kMaxRanks = 8;

enum Epilogue : int { kSwiGLU = 0, kScatter = 1 };

enum MoeErr : int { kMoeOk = 0, kMoeGemmTimeout = 11, kMoeFlagTimeout = 12, kMoeOverflow = 13 };

struct GemmArgs {
  const int* rows;        // [n_experts] rows received per local expert
  const int* row_start;   // [n_experts] first row of each expert in the A buffer
  int n_experts;
  int n_tiles_n;          // N / 256
  int k_blocks;           // K / 64
  int n_per_expert;       // N (rows of B per expert)
  // kSwiGLU
  __nv_bfloat16* act;     // [capacity, act_ld]
  int act_ld;             // N / 2
  // kScatter
  const int* meta;        // [capacity] (src_rank << 20) | return slot on the source rank
  __nv_bfloat16* comb[kMaxRanks];  // per source rank: [tokens * topk, out_ld]
  int out_ld;             // N
  // cross-GPU flags (epoch valued).  wait_flags: this rank's array [n_ranks], all must reach
  // `epoch` before the first tile is loaded.  done_flags[r]: rank r's array, slot my_rank is
  // raised by the last CTA of this launch.
  const uint32_t* wait_flags;
  uint32_t* done_flags[kMaxRanks];
  int n_ranks, my_rank;
  uint32_t epoch;
  unsigned* ticket;       // zero before launch; left at zero
  int* status;            // first error code
  unsigned long long timeout_ns;
  // fused dispatch (FUSED kernels only): this rank's rows are sent while the tensor cores
  // work; an expert's tiles start once `arrived[e]` reached `arrive_target[e]`.  With
  // send_ctas == 0 warps 6-9 of every CTA send; with send_ctas > 0 the last `send_ctas`
  // CTAs of the grid do nothing but send (all their warps) and the others only run tiles.
  const __nv_bfloat16* x;        // [tokens, hidden] local hidden states
  const int* send_pair;          // [n_send] (local expert << 20) | pair index, in send order
  const int* send_target;        // [n_send] (rank << 24) | row, or -1
  const int* pair_slot;          // [pairs] return slot of every pair
  const int* n_send;             // number of send positions
  const int* arrive_target;      // [n_experts] cumulative rows expected per local expert
  __nv_bfloat16* recv_x[kMaxRanks];
  int* recv_meta[kMaxRanks];
  uint32_t* arrived[kMaxRanks];  // per rank: [n_experts] cumulative rows landed
  int topk, hidden;
  int send_ctas;
  unsigned long long* debug;     // optional [gridDim.x * 4] ns: kernel start, senders done, producer wait, end
};

constexpr int kSendWarps = 4;        // sender warps per CTA when every CTA also runs tiles
constexpr int kFusedThreads = 512;   // a dedicated sender CTA uses all 16 warps
constexpr int kFusedWarps = kFusedThreads / 32;

// One warp copies a row of `n_vec` 16-byte words with U independent loads in flight per lane.
template <int U>
__device__ __forceinline__ void copy_row(const uint4* __restrict__ src, uint4* __restrict__ dst, int n_vec, int lane) {
  int v = lane;
  for (; v + 32 * (U - 1) < n_vec; v += 32 * U) {
    uint4 q[U];
#pragma unroll
    for (int i = 0; i < U; ++i) q[i] = __ldg(&src[v + 32 * i]);
#pragma unroll
    for (int i = 0; i < U; ++i) dst[v + 32 * i] = q[i];
  }
  for (; v < n_vec; v += 32) dst[v] = __ldg(&src[v]);
}

// Sender role of the fused kernel: warp `gw` of `n_gw` streams blocks of eight consecutive
// send positions.  After a block, every lane fences its stores at system scope, the warp
// re-converges, and one lane per row bumps the target expert's arrival counter on the
// receiving GPU, which is what the receiver's TMA producer polls.
template <int U>
__device__ __forceinline__ void send_rows(const GemmArgs& a, int gw, int n_gw, int lane) {
  const int n_send = *a.n_send;
  const int vec_per_row = a.hidden / 8;
  for (int blk = gw; blk * 8 < n_send; blk += n_gw) {
    const int pos0 = blk * 8, cnt = min(8, n_send - pos0);
    int my_pair = -1, my_tgt = -1;
    if (lane < cnt) {
      my_pair = a.send_pair[pos0 + lane];
      my_tgt = a.send_target[pos0 + lane];
    }
    for (int j = 0; j < cnt; ++j) {
      const int pr = __shfl_sync(0xffffffffu, my_pair, j), tg = __shfl_sync(0xffffffffu, my_tgt, j);
      if (tg < 0) continue;
      const int pair = pr & 0xFFFFF, dr = tg >> 24, row = tg & 0xFFFFFF;
      const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)(pair / a.topk) * a.hidden);
      uint4* dst = reinterpret_cast<uint4*>(a.recv_x[dr] + (size_t)row * a.hidden);
      copy_row<U>(src, dst, vec_per_row, lane);
      if (lane == 0) a.recv_meta[dr][row] = (a.my_rank << 20) | a.pair_slot[pair];
    }
    __threadfence_system();
    __syncwarp();
    if (lane < cnt && my_tgt >= 0) {
      uint32_t* ctr = a.arrived[my_tgt >> 24] + (my_pair >> 20);
      asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
    }
  }
}

struct TileCursor {
  int expert = 0, first_tile = 0;  // first tile id of `expert`
  int tiles_m = 0;
  // Advance to the expert that owns tile `t`; returns false when t is past the last tile.
  __device__ __forceinline__ bool seek(int t, const GemmArgs& a) {
    for (;;) {
      if (expert >= a.n_experts) return false;
      tiles_m = (a.rows[expert] + kBM - 1) / kBM;
      const int n = tiles_m * a.n_tiles_n;
      if (t < first_tile + n) return true;
      first_tile += n;
      ++expert;
    }
  }
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ void st_global_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int EPI, bool FUSED = false>
__global__ void __launch_bounds__(FUSED ? kFusedThreads : kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmArgs args) {
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kStageBytesA;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_b + kStages * kStageBytesB);
  uint8_t* smem_out = smem_b + kStages * kStageBytesB + 256;  // 4 x kStageOutBytes, 256-byte aligned
  // bars: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + kStages);
  const uint32_t bar_tfull = smem_u32(bars + 2 * kStages), bar_tempty = smem_u32(bars + 2 * kStages + 2);
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int s_flags_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTAs [0, n_gemm) run tiles; in the fused kernel the rest (if any) only send rows
  const int n_gemm = FUSED ? (int)gridDim.x - args.send_ctas : (int)gridDim.x;
  const bool sender_cta = FUSED && (int)blockIdx.x >= n_gemm;
  unsigned long long* dbg = FUSED && args.debug ? args.debug + 4 * blockIdx.x : nullptr;

  if (threadIdx.x == 0) {
    if (dbg) dbg[0] = timer_ns();
    abort_flag = 0;
    s_flags_ok = 1;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    // every source rank must have finished writing this launch's A rows
    if (args.wait_flags != nullptr) {
      const uint64_t t0 = timer_ns();
      for (int r = 0; r < args.n_ranks; ++r) {
        for (;;) {
          uint32_t v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(args.wait_flags + r) : "memory");
          if ((int32_t)(v - args.epoch) >= 0) break;
          if (timer_ns() - t0 > args.timeout_ns) {
            s_flags_ok = 0;
            atomicCAS(args.status, 0, kMoeFlagTimeout);
            break;
          }
          __nanosleep(200);
        }
      }
    }
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort = &abort_flag;
  const uint64_t budget = args.timeout_ns;
  const bool go = s_flags_ok != 0;

  if (sender_cta) {
    // ---------------- dedicated sender CTA (never waits on anything) ----------------
    send_rows<7>(args, ((int)blockIdx.x - n_gemm) * kFusedWarps + warp, args.send_ctas * kFusedWarps, lane);
    if (dbg && lane == 0) atomicMax(&dbg[1], (unsigned long long)timer_ns());
  } else if (go && warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      TileCursor cur;
      uint32_t it = 0;  // running k-block counter over all tiles of this CTA
      int ready_expert = -1;
      for (int t = blockIdx.x; cur.seek(t, args) && !*abort; t += n_gemm) {
        if (FUSED && cur.expert != ready_expert) {
          // all rows of this expert must have landed (senders on every GPU count them in)
          const uint32_t* ctr = args.arrived[args.my_rank] + cur.expert;
          const uint32_t want = (uint32_t)args.arrive_target[cur.expert];
          const uint64_t t0 = timer_ns();
          for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
            if ((int32_t)(v - want) >= 0) break;
            if (*abort || timer_ns() - t0 > budget) {
              *abort = 1;
              atomicCAS(args.status, 0, kMoeFlagTimeout);
              break;
            }
            __nanosleep(100);
          }
          if (dbg) dbg[2] += timer_ns() - t0;
          if (*abort) break;
          fence_proxy_async_global();
          ready_expert = cur.expert;
        }
        const int local = t - cur.first_tile;
        const int m = local % cur.tiles_m, n = local / cur.tiles_m;
        const int row_a = args.row_start[cur.expert] + m * kBM;
        const int row_b = cur.expert * args.n_per_expert + n * kBN;
        for (int kb = 0; kb < args.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort, budget)) break;
          mbar_expect_tx(bar_full + 8 * s, kStageBytesA + kStageBytesB);
          tma_load_2d(smem_u32(smem_a + s * kStageBytesA), &tmap_a, bar_full + 8 * s, kb * kBK, row_a);
          tma_load_2d(smem_u32(smem_b + s * kStageBytesB), &tmap_b, bar_full + 8 * s, kb * kBK, row_b);
        }
      }
    }
  } else if (go && warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(kBM, kBN);
      TileCursor cur;
      uint32_t it = 0, tile_n = 0;
      for (int t = blockIdx.x; cur.seek(t, args) && !*abort; t += n_gemm, ++tile_n) {
        const uint32_t acc = tile_n & 1, acc_ph = (tile_n >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_ph ^ 1, abort, budget)) break;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * kBN;
        bool ok = true;
        for (int kb = 0; kb < args.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort, budget)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t da = umma_desc_sw128(smem_u32(smem_a + s * kStageBytesA));
          const uint64_t db = umma_desc_sw128(smem_u32(smem_b + s * kStageBytesB));
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzled 128-byte row
            umma_bf16(tmem_d, da + (uint64_t)(k * kUmmaK * 2 >> 4), db + (uint64_t)(k * kUmmaK * 2 >> 4), idesc,
                      (kb | k) != 0);
          }
          umma_commit(bar_empty + 8 * s);  // stage reusable once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);  // accumulator complete
      }
    }
  } else if (FUSED && warp >= 6) {
    // ---------------- sender warps beside the tile roles (never wait on anything) ----------------
    if (args.send_ctas == 0 && warp < 6 + kSendWarps) {
      send_rows<4>(args, blockIdx.x * kSendWarps + (warp - 6), gridDim.x * kSendWarps, lane);
      if (dbg && lane == 0) atomicMax(&dbg[1], (unsigned long long)timer_ns());
    }
  } else if (go && warp >= 2) {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    TileCursor cur;
    uint32_t tile_n = 0;
    for (int t = blockIdx.x; cur.seek(t, args) && !*abort; t += n_gemm, ++tile_n) {
      const uint32_t acc = tile_n & 1, acc_ph = (tile_n >> 1) & 1;
      const int local = t - cur.first_tile;
      const int m = local % cur.tiles_m, n = local / cur.tiles_m;
      const int row_in_expert = m * kBM + quarter * 32 + lane;
      const bool valid = row_in_expert < args.rows[cur.expert];
      const size_t row = (size_t)args.row_start[cur.expert] + row_in_expert;
      // tcgen05.ld is a whole-warp instruction: leave the loop only if every lane agrees
      if (!__all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * acc, acc_ph, abort, budget))) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBN;
      if constexpr (EPI == kSwiGLU) {
        __nv_bfloat16* dst = args.act + row * args.act_ld + (size_t)n * (kBN / 2);
#pragma unroll 1
        for (int c0 = 0; c0 < kBN / 2; c0 += 32) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c0, g);
          tmem_ld32(taddr + kBN / 2 + c0, u);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint32_t o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float a0 = silu(__uint_as_float(g[j + 2 * q])) * __uint_as_float(u[j + 2 * q]);
                const float a1 = silu(__uint_as_float(g[j + 2 * q + 1])) * __uint_as_float(u[j + 2 * q + 1]);
                o[q] = pack_bf16(a0, a1);
              }
              st_global_v4(dst + c0 + j, o[0], o[1], o[2], o[3]);
            }
          }
        }
      } else {
        // Each lane owns one output row in TMEM, but a row's 512 bytes should leave the SM
        // as long contiguous stores (they cross NVLink).  Stage 32 rows x 128 columns in
        // shared memory (16-byte chunks XOR-swizzled by row against bank conflicts), then
        // let 16 lanes write one row's 256 bytes: two rows per store instruction.
        unsigned long long dst_addr = 0;
        if (valid) {
          const int mt = args.meta[row];
          dst_addr = reinterpret_cast<unsigned long long>(args.comb[(mt >> 20) & (kMaxRanks - 1)] +
                                                          (size_t)(mt & 0xFFFFF) * args.out_ld + (size_t)n * kBN);
        }
        uint8_t* stage = smem_out + (warp - 2) * kStageOutBytes;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(taddr + half * 128 + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int chunk = (c0 + j) >> 3;  // 16-byte chunk index within the 256-byte row
              uint4 o;
              o.x = pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
              o.y = pack_bf16(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              o.z = pack_bf16(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
              o.w = pack_bf16(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
              *reinterpret_cast<uint4*>(stage + lane * 256 + ((chunk ^ (lane & 15)) << 4)) = o;
            }
          }
          __syncwarp();
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int r = 2 * i + (lane >> 4), chunk = lane & 15;
            const unsigned long long base = __shfl_sync(0xffffffffu, dst_addr, r);
            const uint4 o = *reinterpret_cast<const uint4*>(stage + r * 256 + ((chunk ^ (r & 15)) << 4));
            if (base != 0)
              st_global_v4(reinterpret_cast<void*>(base + (size_t)half * 256 + (size_t)chunk * 16), o.x, o.y, o.z, o.w);
          }
          __syncwarp();
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  // ---------------- teardown ----------------
  if (*abort) {
    // A role gave up.  Give copies that may still be in flight a bounded time to land before
    // shared memory and TMEM are released.
    const uint64_t t0 = timer_ns();
    while (timer_ns() - t0 < 200000) __nanosleep(1000);
    if (threadIdx.x == 0) atomicCAS(args.status, 0, kMoeGemmTimeout);
  }
  if constexpr (EPI == kScatter) __threadfence_system();  // rows stored to peers are visible before the flag
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if (dbg && threadIdx.x == 0) dbg[3] = timer_ns();
  if (threadIdx.x == 0 && args.ticket != nullptr) {
    __threadfence();
    if (atomicAdd(args.ticket, 1u) == gridDim.x - 1) {
      *args.ticket = 0;
      if constexpr (EPI == kScatter) {
        __threadfence_system();
        for (int r = 0; r < args.n_ranks; ++r)
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(args.done_flags[r] + args.my_rank), "r"(args.epoch)
                       : "memory");
      }
    }
  }
}

}  // namespace moe
}  // namespace lplb
