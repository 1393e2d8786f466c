// Backward of the fused causal cosine attention in ONE pass over the sequence: dQ, dK, dV and the gradient of
// the length-norm parameter from a single read of q, k, v, dO (tcgen05 + TMEM + TMA).
//
// The reference's backward is three scans (Cuda_Kernel/Custom_Kernel.py:106-108): dQ needs the state of
// everything BEFORE a position, dK and dV the state of everything AFTER it, which is why two kernels walking in
// opposite directions each had to read all four tensors.  Here the forward pass leaves its 16-bit state operand
// of every chunk in HBM (8 KB per 128 positions: half a tensor pass, `saved`), so the prefix state is a TMA load
// away and one reverse walk does everything (the reference's own unused sketch of a merged backward,
// Cuda_Kernel/backwardv2_comb.cu:58-149, carries three states in one loop instead).
//
// Per chunk of 128 positions, walking from the end of the sequence, with
//   Qw = q^ (rows scaled in place)        Vw = diag(a_s / |k_s|) V (in place; a_s = length-norm factor)
//   S  = state before the chunk  sum_{s < chunk} k_s (x) Vw_s   (saved by the forward, rows d_k)
//   R  = state after the chunk   sum_{t > chunk} Qw_t (x) dO_t  (fp32 in TMEM, 16-bit copy in smem)
// the products are
//   E = mask_{t>=s}(Vw dO^T)   F = mask_{t>=s}(K Qw^T)                        tcgen05 128x128x64 each
//   AccQ = E^T K + dO S^T      AccK = E Qw + Vw R^T      AccV = F dO + K R    128x64x128 + 128x64x64 each
//   R += Qw^T dO                                                              64x64x128 (M = 64)
// E leaves TMEM as a 16-bit [128 x 128] shared-memory tile: read K-major it is the A operand of AccK, read
// MN-major (the same bytes) it is E^T, the A operand of AccQ -- the transposed score tile costs no second MMA
// and no second mask pass.  F is converted in place in TMEM and used as the A operand from TMEM.
//   dq_t = (AccQ_t - Qw_t (Qw_t . AccQ_t)) / |q_t|
//   dv_s = w_s AccV_s,  eps_s = Vw_s . AccV_s,  dk_s = AccK_s - k_s eps_s / |k_s|^2
//   d norm_const[h] += -sigma (1 - sigma) sum_s ln(n_s) eps_s
// Output rows go to a staging area of their own and leave by TMA, so the q, K, V tiles of a stage are refilled as
// soon as the output groups have read their rows (with two stages, waiting for the stores to drain first put the
// store latency on the path that feeds the next score MMAs).  Shared memory: two stages of (q, K, V, dO) = 128 KB,
// the E tile 32 KB, output staging 48 KB, one S tile and one 16-bit R operand of 8 KB each = 224 KB.
// TMEM: E 128 | F 128 | AccQ 64 | AccK 64 | AccV 64 | R 64 = 512 columns.
//
// Where it stands (B = 8, H = 16, N = 4096, bf16, one B200): 7.5 tensor passes of HBM traffic instead of 11, but
// about the run time of the two-kernel backward (142-156 us against 146-148 us), because the walk is bound on the
// SM, not by HBM: a chunk costs ~6300 cycles on the fastest CTA and ~7700 on the median one, against ~3900 cycles
// of tensor-pipe time (36 of its 52 MMAs are 128 x 64 x 16, which run at ~70 cycles each because their A operand
// comes from shared memory), ~5000 cycles of shared-memory traffic (~640 KB per chunk: MMA operands 280 KB, TMA in
// and out 170 KB, the row passes 190 KB) and a serial chain score MMA -> mask -> accumulator MMA -> output rows of
// ~5000 cycles that a single CTA per SM cannot overlap with a second sequence (TMEM and shared memory are both full).
// Two stages are all that fit, so the refill latency of the slower L2 partitions is exposed as well.
#pragma once

#include "causal_tc.cuh"

namespace cott {

constexpr int kBwThreads = 608;  // 2 issuing warps, 4 groups of 4 warps, 1 TMA warp
constexpr int kBwStages = 2;
constexpr int kStateTileBytes = kTcD * 128;              // one 16-bit [64 x 64] state operand
constexpr int kBwStageBytes = 4 * kTileBytes;

// Mask + convert a 128-column fp32 score row held in this thread's TMEM lane (row s of E; column t survives iff
// t >= s) and write it as 16 bits into the two [128 x 64] swizzled panels of `sE` (panel p = columns 64p ..).
template <typename T>
__device__ __forceinline__ void mask_pack_to_smem(uint32_t taddr_lane, unsigned char* sE, int row, int lane, int wq) {
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t packed[16];
    if (blk < wq) {  // warp-uniform: columns below the warp's first row
#pragma unroll
      for (int j = 0; j < 16; ++j) packed[j] = 0u;
    } else {
      uint32_t r[32];
      ptx::tmem_ld_x32(taddr_lane + 32 * blk, r);
      ptx::tmem_ld_wait();
      if (blk == wq) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          packed[j] = Pack2<T>::pack(2 * j >= lane ? __uint_as_float(r[2 * j]) : 0.f,
                                     2 * j + 1 >= lane ? __uint_as_float(r[2 * j + 1]) : 0.f);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) packed[j] = Pack2<T>::pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
      }
    }
    unsigned char* panel = sE + (blk >> 1) * kTileBytes;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *tile_piece(panel, row, 4 * (blk & 1) + j) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
  }
}

enum { kWaitOut = 9, kWaitRFull = 10, kWaitStaging = 11, kWaitSTile = 12, kWaitEps = 13, kWaitAlign = 14 };

template <typename T, bool EXT>
__global__ void __launch_bounds__(kBwThreads, 1)
causal_bwd_fused_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                        const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                        const __grid_constant__ CUtensorMap mapS, const __grid_constant__ CUtensorMap mapDQ,
                        const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV,
                        float* __restrict__ dnorm, const float* __restrict__ norm_const, int H, int N,
                        const float* __restrict__ init_state_arg, int chunks_per_seg_arg,
                        const unsigned char* __restrict__ keep_arg, const int* __restrict__ count_arg) {
  using namespace ptx;
  constexpr int NS = kBwStages;
  constexpr int STAGE = kBwStageBytes;
  constexpr bool BF = Pack2<T>::kBf16;

  // All of the CTA's shared memory is the dynamic array (no static __shared__ at all, so that the array starts at
  // the beginning of the CTA's window and its 1024-byte alignment -- required by the 128-byte swizzle atoms -- costs
  // no padding): tiles first, then the per-row scalars, then the barriers.  224 KB + 2.7 KB of the 227 KB.
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* sE = smem + NS * STAGE;       // [128 x 128] 16-bit E: two swizzled [128 x 64] panels
  unsigned char* sO = sE + 2 * kTileBytes;     // output staging: dQ, dK, dV rows of one item
  unsigned char* sS = sO + 3 * kTileBytes;     // [64 x 64] 16-bit S of the current item (rows d_k)
  unsigned char* sR = sS + kStateTileBytes;    // [64 x 64] 16-bit R operand (rows d_k)
  float* s_rq = reinterpret_cast<float*>(sR + kStateTileBytes);  // [NS][128]  1 / |q_t| (the q tile itself becomes Qw)
  float* s_rk = s_rq + NS * kTcChunk;                            // [NS][128]  1 / |k_s|
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_rk + NS * kTcChunk);
  uint64_t *bar_full = bars, *bar_free_in = bars + NS, *bar_out = bars + 2 * NS, *bar_prep = bars + 3 * NS;
  uint64_t* bar1 = bars + 4 * NS;
  uint64_t &bar_p_full = bar1[0], &bar_p_ready = bar1[1], &bar_acc_full = bar1[2], &bar_acc_free = bar1[3], &bar_state = bar1[4],
           &bar_state2 = bar1[5], &bar_r_full = bar1[6], &bar_init = bar1[7], &bar_s_full = bar1[8], &bar_st_done = bar1[9],
           &bar_stg_free = bar1[10], &bar_pe_full = bar1[11];
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bar1 + 14);
  int& abort_flag_s = *(reinterpret_cast<int*>(bar1 + 14) + 1);
  int& s_tile_loads = *reinterpret_cast<int*>(bar1 + 15);  // S tiles requested so far (for the drain on an aborted run)
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int bh = blockIdx.x;
  const int h = bh % H, bb = bh / H;
  // Segment-parallel launches (gridDim.y > 1): this CTA owns `chunks_per_seg` consecutive chunks, walks them
  // backwards and starts from the R of everything after them (`init_state[bh][seg]`, fp32 [64 x 64], rows d_k).
  // Item ci is chunk `last_chunk - ci` of the sequence.
  const int total_chunks = (N + kTcChunk - 1) / kTcChunk;
  const float* init_state = EXT ? init_state_arg : nullptr;
  const int chunks_per_seg = EXT ? chunks_per_seg_arg : total_chunks;
  const int seg = EXT ? static_cast<int>(blockIdx.y) : 0;
  const int chunk0 = seg * chunks_per_seg;
  const int nchunks = EXT ? min(chunks_per_seg, total_chunks - chunk0) : total_chunks;
  const int last_chunk = chunk0 + nchunks - 1;
  const bool has_init = EXT && init_state != nullptr && seg + 1 < static_cast<int>(gridDim.y);
  const unsigned char* keep_b = (EXT && keep_arg) ? keep_arg + static_cast<size_t>(bh / H) * N : nullptr;
  const int* count_b = (EXT && count_arg) ? count_arg + static_cast<size_t>(bh / H) * N : nullptr;

  if (smem_u32(smem) & 1023u) {  // never seen; the tiles would be read with the wrong swizzle phase
    if (tid == 0) atomicCAS(&g_cott_status, 0, (kWaitAlign << 16));
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_free_in[s], 8);  // dK/dV group (accumulator MMAs done) + operand group (state MMAs done)
      mbar_init(&bar_out[s], 8);      // dK/dV and dQ groups
      mbar_init(&bar_prep[s], 8);     // Vw (score group) + Qw (operand group)
    }
    mbar_init(&bar_p_full, 1);
    mbar_init(&bar_p_ready, 8);  // score group (E) + operand group (F)
    mbar_init(&bar_acc_full, 1);
    mbar_init(&bar_acc_free, 8);  // accumulators read out: dK/dV and dQ groups
    mbar_init(&bar_pe_full, 1);   // E complete (F follows on bar_p_full)
    mbar_init(&bar_state, 4);
    mbar_init(&bar_state2, 4);
    mbar_init(&bar_r_full, 1);
    mbar_init(&bar_init, 4);
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_st_done, 1);
    mbar_init(&bar_stg_free, 1);
    s_tile_loads = 0;
    mbar_fence_init();
    abort_flag_s = 0;
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapDO);
    tma_prefetch_desc(&mapS);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tE = tmem, tF = tmem + 128, tQ = tmem + 256, tK = tmem + 320, tV = tmem + 384, tR = tmem + 448;

  // tile addresses inside a stage
  auto st_q = [&](int ci) { return smem + (ci % NS) * STAGE; };
  auto st_k = [&](int ci) { return smem + (ci % NS) * STAGE + kTileBytes; };
  auto st_v = [&](int ci) { return smem + (ci % NS) * STAGE + 2 * kTileBytes; };
  auto st_d = [&](int ci) { return smem + (ci % NS) * STAGE + 3 * kTileBytes; };
  // chunk 0 of the sequence has nothing before it: no S tile is loaded and the S term is skipped
  auto has_s = [&](int ci) { return last_chunk - ci > 0; };

  // Roles:
  //   warp 0, lane 0:   score tiles E, F of item ci+1; state R += Qw^T dO (ci)
  //   warp 1, lane 0:   accumulators AccQ, AccK, AccV of item ci
  //   warps 2-5:        score group: mask + convert E into shared memory; Vw of the next item
  //   warps 6-9:        dK/dV group: output rows of dV and dK, the norm_const gradient
  //   warps 10-13:      operand group: mask + convert F in TMEM; fp32 R -> 16-bit operand; Qw of the next item
  //   warp 14, lane 0:  TMA loads and stores
  //   warps 15-18:      dQ group: output rows of dQ
  constexpr uint32_t kIdescP = make_idesc(128, 128, BF, false, false);
  constexpr uint32_t kIdescKK = make_idesc(128, 64, BF, false, false);  // A K-major, B K-major
  constexpr uint32_t kIdescKM = make_idesc(128, 64, BF, false, true);   // A K-major (or TMEM), B MN-major
  constexpr uint32_t kIdescMM = make_idesc(128, 64, BF, true, true);    // A MN-major, B MN-major
  constexpr uint32_t kIdescR = make_idesc(64, 64, BF, true, true);
  if (warp == 14) {
    if (lane == 0) {
      // dO of a stage is free as soon as every MMA of its item has completed; q, K, V as soon as the output
      // groups have read their rows.  All four land on the same `full` barrier; the single S tile has its own.
      auto load_early = [&](int ci) {
        const int s = ci % NS;
        mbar_expect_tx(&bar_full[s], STAGE);
        tma_load_tile(st_d(ci), &mapDO, &bar_full[s], (last_chunk - ci) * kTcChunk, h, bb);
      };
      auto load_rest = [&](int ci) {
        const int s = ci % NS;
        const int y = (last_chunk - ci) * kTcChunk;
        tma_load_tile(st_q(ci), &mapQ, &bar_full[s], y, h, bb);
        tma_load_tile(st_k(ci), &mapK, &bar_full[s], y, h, bb);
        tma_load_tile(st_v(ci), &mapV, &bar_full[s], y, h, bb);
      };
      auto load_s = [&](int ci) {
        if (!has_s(ci)) return;
        mbar_expect_tx(&bar_s_full, kStateTileBytes);
        tma_load_tile(sS, &mapS, &bar_s_full, (last_chunk - ci) * kTcD, h, bb);
        s_tile_loads = ci + 1;
      };
      // Items further ahead are pulled into L2 while the ring is busy, so that a refill costs an L2 hit.  (Issued
      // behind the item's own loads and stores: the copy engine takes its requests in order.)
      auto prefetch = [&](int ci) {
        if (ci >= nchunks) return;
        const int gc = last_chunk - ci;
        tma_prefetch_tile(&mapQ, gc * kTcChunk, h, bb);
        tma_prefetch_tile(&mapK, gc * kTcChunk, h, bb);
        tma_prefetch_tile(&mapV, gc * kTcChunk, h, bb);
        tma_prefetch_tile(&mapDO, gc * kTcChunk, h, bb);
        if (has_s(ci)) tma_prefetch_tile(&mapS, gc * kTcD, h, bb);
      };
      load_s(0);
      for (int ci = 0; ci < NS && ci < nchunks; ++ci) {
        load_early(ci);
        load_rest(ci);
      }
      prefetch(NS);
      for (int ci = 0; ci < nchunks; ++ci) {
        const int s = ci % NS;
        const int y = (last_chunk - ci) * kTcChunk;
        const bool refill = ci + NS < nchunks;
        if (ci + 1 < nchunks) {
          // every MMA of item ci has completed: its dO tile and the S tile can be overwritten
          if (!wait_bar(&bar_free_in[s], (ci / NS) & 1, abort_flag, kWaitStageFree, ci)) break;
          load_s(ci + 1);
          if (refill) load_early(ci + NS);
        }
        if (!wait_bar(&bar_out[s], (ci / NS) & 1, abort_flag, kWaitOut, ci)) break;
        if (refill) load_rest(ci + NS);
        tma_store_tile(&mapDV, sO + 2 * kTileBytes, y, h, bb);
        tma_store_tile(&mapDK, sO + kTileBytes, y, h, bb);
        tma_store_tile(&mapDQ, sO, y, h, bb);
        tma_store_commit();
        prefetch(ci + NS + 1);
        tma_store_wait_read<0>();
        mbar_arrive(&bar_stg_free);
      }
      tma_store_wait<0>();
    }
  } else if (warp == 0) {
    if (lane == 0) {
      auto issue_scores = [&](int ci) {  // caller has waited for Qw(ci), Vw(ci) (hence the TMA) and for tE, tF, sE
        const uint64_t dQ = kdesc(smem_u32(st_q(ci))), dK = kdesc(smem_u32(st_k(ci))), dV = kdesc(smem_u32(st_v(ci))),
                       dD = kdesc(smem_u32(st_d(ci)));
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tE, dV + 2 * k, dD + 2 * k, kIdescP, k > 0);
        mma_commit(&bar_pe_full);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tF, dK + 2 * k, dQ + 2 * k, kIdescP, k > 0);
        mma_commit(&bar_p_full);
      };
      bool ok = wait_bar1(&bar_prep[0], 0, abort_flag, kWaitPrepped, 0);
      if (ok) {
        tc_fence_after_sync();
        issue_scores(0);
      }
      for (int ci = 0; ok && ci + 1 < nchunks; ++ci) {
        // state of item ci (Qw(ci) was waited for before its score tiles were issued); the 16-bit conversion
        // after item ci-1 must have finished reading the TMEM state
        if (ci > 0 && !(ok = wait_bar1(&bar_state2, (ci - 1) & 1, abort_flag, kWaitState, ci))) break;
        if (ci == 0 && has_init && !(ok = wait_bar1(&bar_init, 0, abort_flag, kWaitState, ci))) break;
        tc_fence_after_sync();
        const uint64_t dQm = mdesc(smem_u32(st_q(ci))), dDm = mdesc(smem_u32(st_d(ci)));
        mma_ss(tR, dQm, dDm, kIdescR, (ci > 0 || has_init) ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ss(tR, dQm + 128 * k, dDm + 128 * k, kIdescR, 1u);
        mma_commit(&bar_r_full);
        // score tiles of item ci+1: tF is read by the accumulator MMAs of item ci and sE is rewritten by the
        // mask pass that follows these MMAs, so those accumulator MMAs must be complete
        const int s1 = (ci + 1) % NS;
        ok = wait_bar2(&bar_prep[s1], ((ci + 1) / NS) & 1, &bar_acc_full, ci & 1, abort_flag, kWaitPrepped, ci);
        if (!ok) break;
        tc_fence_after_sync();
        issue_scores(ci + 1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t r0 = smem_u32(sR), e0 = smem_u32(sE);
      const uint64_t dEk0 = kdesc(e0), dEk1 = kdesc(e0 + kTileBytes);        // E as a K-major A operand (two panels)
      const uint64_t dEm = make_smem_desc(e0, kTileBytes, 1024)   ;     // E^T: MN-major A, M blocks one panel apart
      for (int ci = 0; ci < nchunks; ++ci) {
        const int s = ci % NS;
        const uint64_t dKk = kdesc(smem_u32(st_k(ci))), dVk = kdesc(smem_u32(st_v(ci))), dDk = kdesc(smem_u32(st_d(ci)));
        const uint64_t dQm = mdesc(smem_u32(st_q(ci))), dKm = mdesc(smem_u32(st_k(ci))), dDm = mdesc(smem_u32(st_d(ci)));
        const bool with_r = ci > 0 || has_init, with_s = has_s(ci);
        // The state terms need Vw(ci) (hence the TMA of the item), the 16-bit R after item ci-1, the S tile and the
        // accumulators read out -- not the masked scores: they are issued while the score tiles are being masked.
        if (!wait_bar4(&bar_prep[s], (ci / NS) & 1, ci > 0 ? &bar_state : (has_init ? &bar_init : nullptr),
                       ci > 0 ? ((ci - 1) & 1) : 0, ci > 0 ? &bar_acc_free : nullptr, (ci - 1) & 1,
                       with_s ? &bar_s_full : nullptr, ci & 1, abort_flag, kWaitState, ci))
          break;
        tc_fence_after_sync();
        if (with_r) {
          const uint64_t dRk = kdesc(r0), dRm = mdesc(r0);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // AccK = Vw R^T : B[n = d_k][k = d_v] = R, K-major
            mma_ss(tK, dVk + 2 * k, dRk + 2 * k, kIdescKK, k > 0);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // AccV = K R : B[n = d_v][k = d_k] = R, MN-major
            mma_ss(tV, dKk + 2 * k, dRm + 128 * k, kIdescKM, k > 0);
        }
        if (with_s) {
          const uint64_t dSk = kdesc(smem_u32(sS));
#pragma unroll
          for (int k = 0; k < 4; ++k)  // AccQ = dO S^T : B[n = d_k][k = d_v] = S, K-major
            mma_ss(tQ, dDk + 2 * k, dSk + 2 * k, kIdescKK, k > 0);
        }
        mma_commit(&bar_st_done);  // the single R operand and S tile may be rewritten once these have completed
        // masked scores of item ci: E in shared memory, F in TMEM
        if (!wait_bar1(&bar_p_ready, ci & 1, abort_flag, kWaitScoreReady, ci)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k)  // AccK += E Qw : A = E K-major (k-steps 0-3 panel 0, 4-7 panel 1), B = Qw MN-major
          mma_ss(tK, (k < 4 ? dEk0 + 2 * k : dEk1 + 2 * (k - 4)), dQm + 128 * k, kIdescKM, (with_r || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // AccQ += E^T K : A = the same tile MN-major, B = K MN-major
          mma_ss(tQ, dEm + 128 * k, dKm + 128 * k, kIdescMM, (with_s || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)  // AccV += F dO : A from TMEM, B = dO MN-major
          mma_ts(tV, tF + 8 * k, dDm + 128 * k, kIdescKM, (with_r || k > 0) ? 1u : 0u);
        mma_commit(&bar_acc_full);
      }
    }
  } else if (warp < 6) {
    // score group: mask + convert E into shared memory, then Vw of the next item in place
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
    auto prepare = [&](int ci) -> bool {
      const int s = ci % NS;
      if (!wait_bar_warp(&bar_full[s], (ci / NS) & 1, abort_flag, kWaitTma, ci)) return false;
      const RowMask m = row_mask(keep_b, count_b, (last_chunk - ci) * kTcChunk + row, N);
      const float rk = m.kp ? inv_norm(row_sumsq_rolled<T>(st_k(ci), row)) : 0.f;
      s_rk[s * kTcChunk + row] = rk;
      scale_row_rolled<T>(st_v(ci), row, rk * length_factor(m.n, sigma));
      fence_proxy_async_smem();
      warp_arrive(&bar_prep[s], lane);
      return true;
    };
    bool ok = prepare(0);
    for (int ci = 0; ok && ci < nchunks; ++ci) {
      if (!(ok = wait_bar_warp(&bar_pe_full, ci & 1, abort_flag, kWaitScore, ci))) break;
      tc_fence_after_sync();
      mask_pack_to_smem<T>(tE + lane_base, sE, row, lane, wq);
      tc_fence_before_sync();
      fence_proxy_async_smem();
      warp_arrive(&bar_p_ready, lane);
      if (ci + 1 < nchunks && !(ok = prepare(ci + 1))) break;
    }
  } else if (warp >= 10 && warp < 14) {
    // operand group: Qw of the next item in place; mask + convert F in TMEM; the fp32 R after this item -> 16-bit operand
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    auto prepare = [&](int ci) -> bool {
      const int s = ci % NS;
      if (!wait_bar_warp(&bar_full[s], (ci / NS) & 1, abort_flag, kWaitTma, ci)) return false;
      unsigned char* sQ = st_q(ci);
      const float rq = row_mask(keep_b, count_b, (last_chunk - ci) * kTcChunk + row, N).kp ? inv_norm(row_sumsq_rolled<T>(sQ, row)) : 0.f;
      s_rq[s * kTcChunk + row] = rq;
      scale_row_rolled<T>(sQ, row, rq);
      fence_proxy_async_smem();
      warp_arrive(&bar_prep[s], lane);
      return true;
    };
    if (has_init) {
      load_init_state<T>(init_state + (static_cast<size_t>(bh) * gridDim.y + seg) * (kTcD * kTcD), tR + lane_base, sR, wq, lane);
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&bar_init, lane);
    }
    bool ok = prepare(0);
    for (int ci = 0; ok && ci < nchunks; ++ci) {
      if (!wait_bar_warp(&bar_p_full, ci & 1, abort_flag, kWaitScore, ci)) break;
      tc_fence_after_sync();
      mask_pack_inplace<T, false>(tF + lane_base, lane, wq);
      tc_fence_before_sync();
      warp_arrive(&bar_p_ready, lane);
      if (ci + 1 < nchunks) {  // R after item ci -> 16-bit operand of item ci+1, then Qw of that item
        if (!wait_bar_warp(&bar_r_full, ci & 1, abort_flag, kWaitRFull, ci)) break;
        tc_fence_after_sync();
        if (lane == 0) mbar_arrive(&bar_free_in[ci % NS]);  // the state MMAs of item ci have read its tiles
        // the 16-bit R operand is single-buffered: the state terms of item ci must have read it
        if (!wait_bar_warp(&bar_st_done, ci & 1, abort_flag, kWaitState, ci)) break;
        state_to_smem_rolled<T>(tR + lane_base, sR, wq, lane);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        warp_arrive(&bar_state, lane);
        if (lane == 0) mbar_arrive(&bar_state2);
        if (!(ok = prepare(ci + 1))) break;
      }
    }
  } else if (warp >= 6 && warp < 10) {
    // dK/dV group: dv rows and eps, then the dk rows; the norm_const gradient
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
    float gsum = 0.f;  // sum_s ln(n_s) eps_s over this thread's rows
    for (int ci = 0; ci < nchunks; ++ci) {
      const int s = ci % NS;
      const int pos = (last_chunk - ci) * kTcChunk + row;
      // (every phase of `prep` is observed; also orders the reads of s_rk after the score group's writes)
      if (!wait_bar_warp(&bar_prep[s], (ci / NS) & 1, abort_flag, kWaitPrepped, ci)) break;
      const RowMask m = row_mask(keep_b, count_b, pos, N);
      const float rk = s_rk[s * kTcChunk + row];
      const float w = rk * length_factor(m.n, sigma);
      // the staging area is free once the stores of the item before have read it
      if (ci > 0 && !wait_bar_warp(&bar_stg_free, (ci - 1) & 1, abort_flag, kWaitStaging, ci)) break;
      if (!wait_bar_warp(&bar_acc_full, ci & 1, abort_flag, kWaitAcc, ci)) break;
      tc_fence_after_sync();
      // Every MMA that reads the tiles of this item completed before acc_full.  (dO and S are free once the
      // state MMAs are done too: the operand group reports those.)
      if (lane == 0) mbar_arrive(&bar_free_in[s]);
      // dv = w AccV;  eps = v' . dv' = Vw . AccV  (the V tile holds Vw = w v)
      const float eps = row_from_acc_dot<T>(st_v(ci), row, tV + lane_base, w, sO + 2 * kTileBytes);
      // dk = (dk^ - k^ (k^ . dk^)) / |k| with dk^ / |k| = AccK (Vw carries a_s / |k_s|) and k^ . dk^ = eps
      row_from_acc<T, true>(st_k(ci), row, tK + lane_base, 1.0f, -rk * rk * eps, sO + kTileBytes);
      tc_fence_before_sync();
      warp_arrive(&bar_acc_free, lane);
      fence_proxy_async_smem();
      warp_arrive(&bar_out[s], lane);
      if (m.n > 1.0f && pos < N) gsum += logf(m.n) * eps;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) gsum += __shfl_down_sync(0xffffffffu, gsum, off);
    if (lane == 0) atomicAdd(dnorm + h, -sigma * (1.0f - sigma) * gsum);
  } else {
    // dQ group (warps 15-18): dq = (dq^ - q^ (q^ . dq^)) / |q| with dq^ = AccQ and the q tile holding q^ = Qw
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    for (int ci = 0; ci < nchunks; ++ci) {
      const int s = ci % NS;
      if (!wait_bar_warp(&bar_prep[s], (ci / NS) & 1, abort_flag, kWaitPrepped, ci)) break;
      const float rq = s_rq[s * kTcChunk + row];
      if (ci > 0 && !wait_bar_warp(&bar_stg_free, (ci - 1) & 1, abort_flag, kWaitStaging, ci)) break;
      if (!wait_bar_warp(&bar_acc_full, ci & 1, abort_flag, kWaitAcc, ci)) break;
      tc_fence_after_sync();
      const float delta = row_dot_acc<T>(st_q(ci), row, tQ + lane_base);
      row_from_acc<T, true>(st_q(ci), row, tQ + lane_base, rq, -rq * delta, sO);
      tc_fence_before_sync();
      warp_arrive(&bar_acc_free, lane);
      fence_proxy_async_smem();
      warp_arrive(&bar_out[s], lane);
    }
  }

  // ---- leave: make sure no TMA of this CTA is still in flight (bounded), release TMEM ------------
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    for (int ci = (nchunks > NS ? nchunks - NS : 0); ci < nchunks; ++ci)
      mbar_wait(&bar_full[ci % NS], (ci / NS) & 1, 64);
    if (s_tile_loads > 0) mbar_wait(&bar_s_full, (s_tile_loads - 1) & 1, 64);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

inline size_t causal_bwd_fused_smem_bytes() {
  return static_cast<size_t>(kBwStages * kBwStageBytes + 2 * kTileBytes + 3 * kTileBytes + 2 * kStateTileBytes +
                             2 * kBwStages * kTcChunk * sizeof(float) + (4 * kBwStages + 16) * sizeof(uint64_t));
}

}  // namespace cott
