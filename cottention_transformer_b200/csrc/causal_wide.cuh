// Causal scan with head dim 128 on the 5th-generation tensor cores (tcgen05 + TMEM + TMA): the kernel behind
// cott_scan and the fused cosine attention for D_attn = 128.
//
// The reference runs kernel_mod_4<T, 32> for D_attn >= 128 (Cuda_Kernel/combined_kernel_general.cu:173-251, selected at
// :281-284): one warp per output column, four state elements per lane, N serial steps.  Here a CTA owns one
// (batch, head) sequence and one 64-column slice of the value / output dimension, walks the sequence in chunks of
// 128 positions, and the whole head dimension of Q and K goes into the SAME score and state accumulators:
//   P   = mask(X Y^T)            128 x 128, contraction over 128 = two 64-column panels, 8 k-steps   (tcgen05, TMEM)
//   Acc = P Zs + X S             128 x 64                                                            (A = P from TMEM)
//   S  += Y^T Zs                 128 x 64 with M = 128: the natural tcgen05 shape, every TMEM lane holds a state row
// X, Y are [128 x 128] tiles (two swizzled 64-column panels each), Zs the [128 x 64] slice of Z with its rows scaled.
// Nothing goes through a scratch buffer and the products are rounded to 16 bits once.
//
// The module math around the scan (GPT_Trainer/GPTCosAttention.py:229-248 and its backward) is row scalings, which
// enter through hooks rather than through extra passes over the tensors:
//   NORMS   (forward): 1/|x_t|, 1/|y_s| from the tiles themselves, Zs = diag(keep a_s / |y_s|) Z, out rows / |x_t|;
//           the three row vectors are also written out for the backward
//   yscale, zscale, oscale: per-position fp32 vectors that scale the rows of Y (in shared memory), of Z (likewise)
//           and of the output
//   C, ccoef: out_row += ccoef[pos] * C_row for a fourth tile C (the normalisation terms of the backward: -q (q^.dq^) / |q|^2 ...)
//   eps:    eps[pos] += oscale[pos] * (C_row . Acc_row)   (v'_s . dv'_s, summed over the two column slices by atomics)
// REV walks the sequence backwards with the mask flipped (the reversed scans of Custom_Kernel.py:107-108).
// STATE_ONLY keeps only the state chain and writes the segment's own S to global memory (segment-parallel launches).
//
// Shared memory (all dynamic): two stages of (X 32 KB, Y 32 KB, Z 16 KB), the double-buffered 16-bit state operand
// 2 x 16 KB and a two-slot output staging ring 2 x 16 KB = 224 KB, then the row scalars and the barriers.  A stage is
// refilled as soon as the MMAs of its chunk have completed: output rows are staged in the ring (C rows are copied
// there straight from global memory by the thread that owns the row), so no store has to drain first.
// TMEM: P 2 x 128 | Acc 2 x 64 | S 64.
#pragma once

#include "causal_tc.cuh"

namespace cott {

constexpr int kWdThreads = 640;  // 3 issuing warps, 1 TMA warp, 4 groups of 4 warps
constexpr int kWdStages = 2;
constexpr int kWdStageBytes = 5 * kTileBytes;
constexpr int kWdStateBytes = kTcChunk * 128;  // one 16-bit [128 x 64] state operand

struct WideArgs {
  const float* yscale;  // [B*H*N] or null
  const float* zscale;
  const float* oscale;
  const float* ccoef;
  float* eps;           // [B*H*N], accumulated by atomics (zero it first), or null
  const float* norm_const;  // NORMS only: [H]
  float* rq_out;        // NORMS only (may be null): 1/|x_t|, 1/|y_s|, keep a_s/|y_s|
  float* rk_out;
  float* w_out;
  const float* init_state;  // [B*H][slices][nseg][128 x 64] fp32, the state before each segment in scan order, or null
  float* state_out;         // STATE_ONLY: [B*H][slices][nseg][128 x 64]
  const unsigned char* keep;  // NORMS only: padding ([B, N], with its inclusive running count) or both null
  const int* count;
  const void* c;        // the C tensor [B,H,N,dz] (dense), or null
  int dz;               // row length of Z / C / out in elements
  int chunks_per_seg;
  int H, N;
};

// a 128-column row of a two-panel tile.  (Rolled two-piece routines on purpose: versions with eight pieces in flight
// are faster in isolation and slowed the whole kernel down -- every role runs on every scheduler and competes for
// one instruction cache.)
template <typename T>
__device__ __forceinline__ float row_sumsq2(unsigned char* tile, int row) {
  return row_sumsq_rolled<T>(tile, row) + row_sumsq_rolled<T>(tile + kTileBytes, row);
}

template <typename T, bool REV, bool NORMS, bool STATE_ONLY>
__global__ void __launch_bounds__(kWdThreads, 1)
wide_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
            const __grid_constant__ CUtensorMap mapZ, const __grid_constant__ CUtensorMap mapOut, const WideArgs a) {
  using namespace ptx;
  constexpr int NS = kWdStages;
  constexpr bool BF = Pack2<T>::kBf16;

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* sS = smem + NS * kWdStageBytes;  // 2 x [128 x 64] 16-bit state operand (rows = columns of Y)
  unsigned char* sO = sS + 2 * kWdStateBytes;     // 2 x [128 x 64] output staging ring
  float* s_rq = reinterpret_cast<float*>(sO + 2 * kTileBytes);  // [NS][128] output row scale of a stage (NORMS)
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_rq + NS * kTcChunk);
  uint64_t *bar_full = bars, *bar_free_in = bars + 2, *bar_out = bars + 4, *bar_prep = bars + 6, *bar_p_full = bars + 8,
           *bar_p_ready = bars + 10, *bar_acc_full = bars + 12, *bar_acc_free = bars + 14, *bar_state = bars + 16;
  uint64_t &bar_s_full = bars[18], &bar_state2 = bars[19], &bar_init = bars[20];
  uint64_t* bar_stg_free = bars + 21;  // [2]: the store of the chunk that used the slot has read it
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 23);
  int& abort_flag_s = *(reinterpret_cast<int*>(bars + 23) + 1);
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int bh = blockIdx.x, slice = blockIdx.y, seg = blockIdx.z;
  const int h = bh % a.H, bb = bh / a.H;
  const int N = a.N;
  const int total_chunks = (N + kTcChunk - 1) / kTcChunk;
  const int chunk0 = seg * a.chunks_per_seg;
  const int nchunks = min(a.chunks_per_seg, total_chunks - chunk0);
  const bool has_init = !STATE_ONLY && a.init_state != nullptr && seg > 0;
  const size_t state_index = (static_cast<size_t>(bh) * gridDim.y + slice) * gridDim.z + seg;
  const size_t row_base = static_cast<size_t>(bh) * N;  // the per-position vectors are [B*H, N]
  const unsigned char* keep_b = (NORMS && a.keep) ? a.keep + static_cast<size_t>(bb) * N : nullptr;
  const int* count_b = (NORMS && a.count) ? a.count + static_cast<size_t>(bb) * N : nullptr;
  // first row of local chunk c (the reversed scan numbers chunks and segments from the end of the sequence)
  auto row0_of = [&](int c) { return (REV ? total_chunks - 1 - (chunk0 + c) : chunk0 + c) * kTcChunk; };
  auto st_x = [&](int c) { return smem + (c % NS) * kWdStageBytes; };
  auto st_y = [&](int c) { return smem + (c % NS) * kWdStageBytes + 2 * kTileBytes; };
  auto st_z = [&](int c) { return smem + (c % NS) * kWdStageBytes + 4 * kTileBytes; };
  auto st_o = [&](int c) { return sO + (c & 1) * kTileBytes; };

  if (smem_u32(smem) & 1023u) {  // the swizzle atoms need the 1024-byte alignment the declaration asks for
    if (tid == 0) atomicCAS(&g_cott_status, 0, (15 << 16));
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bar_full[s], 1);
      // state group (state MMAs done) + in NORMS mode the output group (it reads the X tile for the row norm);
      // the TMA thread itself waits for the accumulator MMAs
      mbar_init(&bar_free_in[s], (NORMS && !STATE_ONLY) ? 8 : 4);
      mbar_init(&bar_out[s], 4);
      mbar_init(&bar_prep[s], 4);
      mbar_init(&bar_p_full[s], 1);
      mbar_init(&bar_p_ready[s], 4);
      mbar_init(&bar_acc_full[s], 1);
      mbar_init(&bar_acc_free[s], 4);
      mbar_init(&bar_state[s], 4);
      mbar_init(&bar_stg_free[s], 1);
    }
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_state2, 4);
    mbar_init(&bar_init, 4);
    mbar_fence_init();
    abort_flag_s = 0;
    tma_prefetch_desc(&mapX);
    tma_prefetch_desc(&mapY);
    tma_prefetch_desc(&mapZ);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tP0 = tmem, tAcc0 = tmem + 256, tS = tmem + 384;  // P 2 x 128 | Acc 2 x 64 | S 64

  // Roles:
  //   warp 0, lane 0:   scores P(c+1) = X Y^T
  //   warp 1, lane 0:   accumulators Acc(c) = X S + P Zs
  //   warp 19, lane 0:  state S += Y^T Zs (c)
  //   warps 2-5:        mask group: mask + convert P in TMEM
  //   warps 6-9:        output group: accumulator -> output rows
  //   warps 10-13:      state group: fp32 state -> 16-bit operand
  //   warp 14, lane 0:  TMA loads and stores
  //   warps 15-18:      operand group: row norms / row scalings of Y and Z in place
  constexpr uint32_t kIdescP = make_idesc(128, 128, BF, false, false);
  constexpr uint32_t kIdescAcc = make_idesc(128, 64, BF, false, true);
  constexpr uint32_t kIdescS = make_idesc(128, 64, BF, true, true);
  if (warp == 14) {
    // ---------------------------------------------------------------- TMA loads and stores
    if (lane == 0) {
      const int xz = 64 * slice;  // column offset of the Z / C / output slice
      auto issue_loads = [&](int c) {
        const int s = c % NS, y = row0_of(c);
        mbar_expect_tx(&bar_full[s], (STATE_ONLY ? 3 : 5) * kTileBytes);
        if (!STATE_ONLY) {
          tma_load_tile_x(st_x(c), &mapX, &bar_full[s], 0, y, h, bb);
          tma_load_tile_x(st_x(c) + kTileBytes, &mapX, &bar_full[s], 64, y, h, bb);
        }
        tma_load_tile_x(st_y(c), &mapY, &bar_full[s], 0, y, h, bb);
        tma_load_tile_x(st_y(c) + kTileBytes, &mapY, &bar_full[s], 64, y, h, bb);
        tma_load_tile_x(st_z(c), &mapZ, &bar_full[s], xz, y, h, bb);
      };
      auto prefetch = [&](int c) {  // pull a chunk further ahead into L2: with two stages a refill should be an L2 hit
        if (c >= nchunks) return;
        const int y = row0_of(c);
        if (!STATE_ONLY) {
          tma_prefetch_tile_x(&mapX, 0, y, h, bb);
          tma_prefetch_tile_x(&mapX, 64, y, h, bb);
        }
        tma_prefetch_tile_x(&mapY, 0, y, h, bb);
        tma_prefetch_tile_x(&mapY, 64, y, h, bb);
        tma_prefetch_tile_x(&mapZ, xz, y, h, bb);
      };
      for (int c = 0; c < NS && c < nchunks; ++c) issue_loads(c);
      prefetch(NS);
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % NS;
        if (c + NS < nchunks) {
          // every MMA of chunk c has completed and nothing else reads its tiles: refill the stage.  (The output
          // group may be running late -- its rows of the previous chunk, a C row still on its way from HBM -- so the
          // accumulator MMAs are waited for here, not reported by it.)
          if (!STATE_ONLY && !wait_bar(&bar_acc_full[c & 1], (c >> 1) & 1, abort_flag, kWaitAcc, c)) break;
          if (!wait_bar(&bar_free_in[s], (c / NS) & 1, abort_flag, kWaitStageFree, c)) break;
          issue_loads(c + NS);
          prefetch(c + NS + 1);
        }
        if (STATE_ONLY) continue;
        if (!wait_bar(&bar_out[s], (c / NS) & 1, abort_flag, kWaitStageFree, c)) break;
        tma_store_tile_x(&mapOut, st_o(c), xz, row0_of(c), h, bb);
        tma_store_commit();
        if (c >= 1) {  // the store of chunk c-1 has read its staging slot
          tma_store_wait_read<1>();
          mbar_arrive(&bar_stg_free[(c - 1) & 1]);
        }
      }
      tma_store_wait<0>();
    }
  } else if (warp == 0) {
    // ---------------------------------------------------------------- scores
    if (lane == 0 && !STATE_ONLY) {
      auto issue_scores = [&](int c) {  // caller has waited for the prepared tiles of chunk c and for the buffer
        const uint64_t dX = kdesc(smem_u32(st_x(c))), dY = kdesc(smem_u32(st_y(c)));
        const uint32_t tP = tP0 + 128 * (c & 1);
        constexpr uint64_t kPanel = kTileBytes >> 4;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ss(tP, dX + (k >> 2) * kPanel + 2 * (k & 3), dY + (k >> 2) * kPanel + 2 * (k & 3), kIdescP, k > 0);
        mma_commit(&bar_p_full[c & 1]);
      };
      // The scores read X and Y only: they can go as soon as the TMA has landed, without waiting for the row pass
      // of the operand group -- unless that pass rewrites Y (yscale).
      uint64_t* gate = a.yscale ? bar_prep : bar_full;
      bool ok = wait_bar1(&gate[0], 0, abort_flag, kWaitPrepped, 0);
      if (ok) {
        tc_fence_after_sync();
        issue_scores(0);
      }
      for (int c = 0; ok && c + 1 < nchunks; ++c) {
        // scores of chunk c+1: its tiles, and (buffer reuse) the accumulator MMAs of chunk c-1 done
        const int s1 = (c + 1) % NS;
        ok = wait_bar2(&gate[s1], ((c + 1) / NS) & 1, c >= 1 ? &bar_acc_full[(c + 1) & 1] : &gate[s1],
                       c >= 1 ? (((c - 1) >> 1) & 1) : (((c + 1) / NS) & 1), abort_flag, kWaitTma, c);
        if (!ok) break;
        tc_fence_after_sync();
        issue_scores(c + 1);
      }
    }
  } else if (warp == 19) {
    // ---------------------------------------------------------------- state
    if (lane == 0) {
      const int last = STATE_ONLY ? nchunks : nchunks - 1;  // the state after the last chunk is only needed by STATE_ONLY
      for (int c = 0; c < last; ++c) {
        // state update of chunk c: its prepared tiles, and the conversion of S after chunk c-1 (it reads the fp32 state)
        if (!wait_bar4(&bar_prep[c % NS], (c / NS) & 1, (!STATE_ONLY && c > 0) ? &bar_state2 : (has_init ? &bar_init : nullptr),
                       c > 0 ? ((c - 1) & 1) : 0, nullptr, 0, nullptr, 0, abort_flag, kWaitPrepped, c))
          break;
        tc_fence_after_sync();
        // A = Y^T: MN-major, M = 128 = the two panels of Y (one panel apart), K = the 128 positions
        const uint64_t dYm = make_smem_desc(smem_u32(st_y(c)), kTileBytes, 1024), dZm = mdesc(smem_u32(st_z(c)));
        mma_ss(tS, dYm, dZm, kIdescS, (c > 0 || has_init) ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ss(tS, dYm + 128 * k, dZm + 128 * k, kIdescS, 1u);
        mma_commit(&bar_s_full);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- accumulators
    if (lane == 0 && !STATE_ONLY) {
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % NS, b = c & 1;
        const uint64_t dX = kdesc(smem_u32(st_x(c))), dZm = mdesc(smem_u32(st_z(c)));
        const uint32_t tP = tP0 + 128 * b, tAcc = tAcc0 + 64 * b;
        // masked scores of chunk c, the 16-bit state after chunk c-1, the accumulator buffer read out, the prepared Z
        if (!wait_bar4(&bar_p_ready[b], (c >> 1) & 1, c > 0 ? &bar_state[(c - 1) & 1] : (has_init ? &bar_init : nullptr),
                       c > 0 ? (((c - 1) >> 1) & 1) : 0, c >= 2 ? &bar_acc_free[b] : nullptr, ((c >> 1) - 1) & 1, &bar_prep[s],
                       (c / NS) & 1, abort_flag, kWaitScoreReady, c))
          break;
        tc_fence_after_sync();
        const bool with_s = c > 0 || has_init;
        if (with_s) {
          // Acc = X S: A = X K-major over both panels, B = the 16-bit state [K = 128 rows, N = 64], MN-major
          const uint64_t dS = mdesc(smem_u32(sS + b * kWdStateBytes));
          constexpr uint64_t kPanel = kTileBytes >> 4;
#pragma unroll
          for (int k = 0; k < 8; ++k) mma_ss(tAcc, dX + (k >> 2) * kPanel + 2 * (k & 3), dS + 128 * k, kIdescAcc, k > 0);
        }
        mma_ts(tAcc, tP, dZm, kIdescAcc, with_s ? 1u : 0u);  // Acc += P Zs   (P from TMEM, Zs MN-major)
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ts(tAcc, tP + 8 * k, dZm + 128 * k, kIdescAcc, 1u);
        mma_commit(&bar_acc_full[b]);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- mask group
    if (!STATE_ONLY) {
      const int wq = warp & 3;
      const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
      for (int c = 0; c < nchunks; ++c) {
        const int b = c & 1;
        if (!wait_bar_warp(&bar_p_full[b], (c >> 1) & 1, abort_flag, kWaitScore, c)) break;
        tc_fence_after_sync();
        mask_pack_inplace<T, !REV>(tP0 + 128 * b + lane_base, lane, wq);
        tc_fence_before_sync();
        warp_arrive(&bar_p_ready[b], lane);
      }
    }
  } else if (warp >= 10 && warp < 14) {
    // ---------------------------------------------------------------- state group (thread = state row = TMEM lane)
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    if (has_init) {
      // the state before this segment: fp32 into TMEM, 16-bit into the operand buffer of chunk 0
      const float* src = a.init_state + state_index * (kTcChunk * kTcD) + row * kTcD;
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 f = *reinterpret_cast<const float4*>(src + 32 * half + 4 * j);
          r[4 * j] = __float_as_uint(f.x), r[4 * j + 1] = __float_as_uint(f.y);
          r[4 * j + 2] = __float_as_uint(f.z), r[4 * j + 3] = __float_as_uint(f.w);
        }
        tmem_st_x32(tS + lane_base + 32 * half, r);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *tile_piece(sS, row, 4 * half + j) =
              make_uint4(Pack2<T>::pack(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1])),
                         Pack2<T>::pack(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                         Pack2<T>::pack(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                         Pack2<T>::pack(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&bar_init, lane);
    }
    if (STATE_ONLY) {
      // every state MMA frees its stage; after the last one the segment's own state goes to global memory
      bool ok = true;
      for (int c = 0; ok && c < nchunks; ++c) {
        if (!(ok = wait_bar_warp(&bar_s_full, c & 1, abort_flag, kWaitState, c))) break;
        if (lane == 0) mbar_arrive(&bar_free_in[c % NS]);
      }
      if (ok) {
        tc_fence_after_sync();
        float* dst = a.state_out + state_index * (kTcChunk * kTcD) + row * kTcD;
#pragma unroll 1
        for (int blk = 0; blk < 4; ++blk) {
          uint32_t r[16];
          tmem_ld_x16(tS + lane_base + 16 * blk, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(dst + 16 * blk + 4 * j) =
                make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                            __uint_as_float(r[4 * j + 3]));
        }
      }
    } else {
      for (int c = 0; c + 1 < nchunks; ++c) {
        // S after chunk c -> 16-bit operand for chunk c+1 (buffer (c+1)&1)
        if (!wait_bar_warp(&bar_s_full, c & 1, abort_flag, kWaitState, c)) break;
        tc_fence_after_sync();
        if (lane == 0) mbar_arrive(&bar_free_in[c % NS]);  // the state MMAs of chunk c have read its tiles
        uint32_t r[32], pk[32];
        tmem_ld_x32(tS + lane_base, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = Pack2<T>::pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        tmem_ld_x32(tS + lane_base + 32, r);
        tmem_ld_wait();
        tc_fence_before_sync();
        warp_arrive(&bar_state2, lane);  // the fp32 state has been read: the next state MMAs may run
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[16 + j] = Pack2<T>::pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        // the 16-bit buffer written now was last read by the accumulator MMAs of chunk c-1
        if (c > 0 && !wait_bar_warp(&bar_acc_full[(c - 1) & 1], ((c - 1) >> 1) & 1, abort_flag, kWaitAccFree, c)) break;
        unsigned char* dst = sS + ((c + 1) & 1) * kWdStateBytes;
#pragma unroll
        for (int j = 0; j < 8; ++j) *tile_piece(dst, row, j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        fence_proxy_async_smem();
        warp_arrive(&bar_state[c & 1], lane);
      }
    }
  } else if (warp >= 15 && warp < 19) {
    // ---------------------------------------------------------------- operand group: rows of Y and Z in place
    const int row = 32 * (warp & 3) + lane;
    const float sigma = NORMS ? 1.0f / (1.0f + __expf(-a.norm_const[h])) : 0.f;
    for (int c = 0; c < nchunks; ++c) {
      const int s = c % NS;
      if (!wait_bar_warp(&bar_full[s], (c / NS) & 1, abort_flag, kWaitTma, c)) break;
      const int pos = row0_of(c) + row;
      if constexpr (NORMS) {
        const RowMask m = row_mask(keep_b, count_b, pos, N);
        const float rk = m.kp ? inv_norm(row_sumsq2<T>(st_y(c), row)) : 0.f;
        const float w = rk * length_factor(m.n, sigma);
        scale_row_rolled<T>(st_z(c), row, w);
        if (!STATE_ONLY && slice == 0 && pos < N && a.rk_out) {
          a.rk_out[row_base + pos] = rk;
          a.w_out[row_base + pos] = w;
        }
      } else {
        if (a.yscale) {
          const float f = pos < N ? a.yscale[row_base + pos] : 0.f;
          scale_row_rolled<T>(st_y(c), row, f);
          scale_row_rolled<T>(st_y(c) + kTileBytes, row, f);
        }
        if (a.zscale) scale_row_rolled<T>(st_z(c), row, pos < N ? a.zscale[row_base + pos] : 0.f);
      }
      fence_proxy_async_smem();
      warp_arrive(&bar_prep[s], lane);
    }
  } else if (warp >= 6 && warp < 10) {
    // ---------------------------------------------------------------- output group
    if (!STATE_ONLY) {
      const int wq = warp & 3, row = 32 * wq + lane;
      const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
      const bool has_c = a.c != nullptr;
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % NS, b = c & 1;
        const int pos = row0_of(c) + row;
        unsigned char* dst = st_o(c);
        // (every phase of `full` is observed)
        if (!wait_bar_warp(&bar_full[s], (c / NS) & 1, abort_flag, kWaitTma, c)) break;
        float beta = 1.f, alpha = 0.f;
        if constexpr (NORMS) {
          // the row norm of x only needs the TMA data: taken while the MMAs run (the stage cannot be refilled before
          // this group reports the accumulator MMAs)
          beta = row_mask(keep_b, count_b, pos, N).kp ? inv_norm(row_sumsq2<T>(st_x(c), row)) : 0.f;
          if (slice == 0 && pos < N && a.rq_out) a.rq_out[row_base + pos] = beta;
          if (lane == 0) mbar_arrive(&bar_free_in[s]);  // (warp-converged) this warp is done with the X tile
        } else {
          if (a.oscale) beta = pos < N ? a.oscale[row_base + pos] : 0.f;
          if (has_c && a.ccoef) alpha = pos < N ? a.ccoef[row_base + pos] : 0.f;
        }
        // this thread's C row, straight from global memory: issued now, so that the loads have the waits below to land
        uint4 u[8];
        if (has_c) {
          const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(a.c) + (row_base + min(pos, N - 1)) * a.dz + 64 * slice);
#pragma unroll
          for (int j = 0; j < 8; ++j) u[j] = pos < N ? src[j] : make_uint4(0, 0, 0, 0);
        }
        // the staging slot was last stored from two chunks ago
        if (c >= 2 && !wait_bar_warp(&bar_stg_free[b], ((c - 2) >> 1) & 1, abort_flag, kWaitStageFree, c)) break;
        if (has_c) {
#pragma unroll
          for (int j = 0; j < 8; ++j) *tile_piece(dst, row, j) = u[j];
        }
        if (!wait_bar_warp(&bar_acc_full[b], (c >> 1) & 1, abort_flag, kWaitAcc, c)) break;
        tc_fence_after_sync();
        const uint32_t tAcc = tAcc0 + 64 * b + lane_base;
        if (has_c) {
          if (a.eps) {  // eps += beta (C_row . Acc_row), then the row itself
            const float e = beta * row_from_acc_dot<T>(dst, row, tAcc, beta);
            if (pos < N) atomicAdd(a.eps + row_base + pos, e);
          } else {
            row_from_acc<T, true>(dst, row, tAcc, beta, alpha);
          }
        } else {
          row_from_acc<T, false>(dst, row, tAcc, beta, 0.f);
        }
        tc_fence_before_sync();
        warp_arrive(&bar_acc_free[b], lane);
        fence_proxy_async_smem();
        warp_arrive(&bar_out[s], lane);
      }
    }
  }

  // ---- leave: make sure no TMA of this CTA is still in flight (bounded), release TMEM ------------
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    for (int c = (nchunks > NS ? nchunks - NS : 0); c < nchunks; ++c) mbar_wait(&bar_full[c % NS], (c / NS) & 1, 64);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// Decode state of a whole prompt from the segment states of a head-dim-128 state pass:
// state[bh][j][i] (+)= sum_seg seg_state[bh][j / 64][seg][i][j % 64]   (the decode kernel keeps the value index first,
// GPTCosAttention.py:264).  grid = (B*H, 2 slices), any block size.
__global__ void wide_seg_to_decode_state_kernel(const float* __restrict__ seg_state, float* __restrict__ state, int nseg,
                                                int accumulate) {
  const int slice = blockIdx.y;
  const size_t base = (static_cast<size_t>(blockIdx.x) * gridDim.y + slice) * nseg * (kTcChunk * kTcD);
  float* dst = state + static_cast<size_t>(blockIdx.x) * (128 * 128);
  for (int e = threadIdx.x; e < 64 * 128; e += blockDim.x) {
    const int jj = e / 128, i = e % 128;  // output element [64 slice + jj][i] = input element [i][jj]
    float sum = accumulate ? dst[(64 * slice + jj) * 128 + i] : 0.f;
    for (int s = 0; s < nseg; ++s) sum += seg_state[base + static_cast<size_t>(s) * (kTcChunk * kTcD) + i * kTcD + jj];
    dst[(64 * slice + jj) * 128 + i] = sum;
  }
}

inline size_t wide_smem_bytes() {
  return static_cast<size_t>(kWdStages * kWdStageBytes + 2 * kWdStateBytes + 2 * kTileBytes + kWdStages * kTcChunk * sizeof(float) +
                             32 * sizeof(uint64_t));
}

// Exclusive prefix over the segments of each (b, h, slice), in scan order: prefix[u][seg] = sum_{s' < seg} state[u][s'].
// grid = (B*H*slices, any), any block size; `elems` floats per matrix (the elements are split over gridDim.y blocks).
__global__ void seg_prefix_kernel(const float* __restrict__ state, float* __restrict__ prefix, int nseg, int elems) {
  const size_t base = static_cast<size_t>(blockIdx.x) * nseg * elems;
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < elems; e += gridDim.y * blockDim.x) {
    float run = 0.f;
    for (int s = 0; s < nseg; ++s) {
      prefix[base + static_cast<size_t>(s) * elems + e] = run;
      run += state[base + static_cast<size_t>(s) * elems + e];
    }
  }
}

// The segment states of a pass whose roles of Y and Z are swapped are the transposes of these: with the full state
// M[r][c] (128 x 128, r over the columns of Y, c over the columns of Z) stored as two [128 x 64] column slices,
//   dst[u][I][seg][r][c] = src[u][r / 64][seg][64 I + c][r % 64]          (u = batch * heads + head, I = 0, 1)
// (dq's prefix states from the forward's, dk's from dv's: two state-only launches less per backward).
// grid = (B*H, nseg, any), any block size.
__global__ void seg_transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int nseg) {
  const int u = blockIdx.x, seg = blockIdx.y;
  constexpr int E = kTcChunk * kTcD;  // 128 x 64
  for (int e = blockIdx.z * blockDim.x + threadIdx.x; e < 2 * E; e += gridDim.z * blockDim.x) {
    const int I = e / E, r = (e % E) / kTcD, c = e % kTcD;
    dst[((static_cast<size_t>(u) * 2 + I) * nseg + seg) * E + r * kTcD + c] =
        src[((static_cast<size_t>(u) * 2 + r / 64) * nseg + seg) * E + (64 * I + c) * kTcD + r % 64];
  }
}

// coef[r] = -scale[r]^2 * (a[r, :] . b[r, :]) for rows of 128 16-bit elements: sixteen threads per row, one 16-byte piece
// each.  (-q^.dq^ / |q|^2 of the normalisation backward, from q^_t . dq^_t = dO_t . O_t.)
template <typename T>
__global__ void rowdot_coef_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ scale,
                                   float* __restrict__ coef, long rows) {
  const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long r = i >> 4;
  float s = 0.f;
  if (r < rows) {
    const uint4 u = *reinterpret_cast<const uint4*>(a + r * 128 + (i & 15) * 8);
    const uint4 w = *reinterpret_cast<const uint4*>(b + r * 128 + (i & 15) * 8);
    const uint32_t* x = reinterpret_cast<const uint32_t*>(&u);
    const uint32_t* y = reinterpret_cast<const uint32_t*>(&w);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = Pack2<T>::unpack(x[e]), g = Pack2<T>::unpack(y[e]);
      s = fmaf(f.x, g.x, fmaf(f.y, g.y, s));
    }
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off, 16);
  if (r < rows && (i & 15) == 0) {
    const float q = scale[r];
    coef[r] = -q * q * s;
  }
}

// After the dV pass: ck[r] = -rk[r]^2 eps[r], and d norm_const[h] += -sigma (1 - sigma) sum_s ln(n_s) eps_s
// (GPTCosAttention.py:241 by the chain rule; n_s = the running count of kept positions, s + 1 without padding).
// grid = (B*H, ceil(N / 1024)), block = 256.
__global__ void eps_coef_kernel(const float* __restrict__ eps, const float* __restrict__ rk, float* __restrict__ ck,
                                const float* __restrict__ norm_const, float* __restrict__ dnorm, const int* __restrict__ count,
                                int H, int N) {
  const int bh = blockIdx.x, h = bh % H, b = bh / H;
  const size_t base = static_cast<size_t>(bh) * N;
  float g = 0.f;
  for (int s = blockIdx.y * 1024 + threadIdx.x; s < min(N, (static_cast<int>(blockIdx.y) + 1) * 1024); s += blockDim.x) {
    const float e = eps[base + s], r = rk[base + s];
    ck[base + s] = -r * r * e;
    const float n = count ? fmaxf(static_cast<float>(count[static_cast<size_t>(b) * N + s]), 1.f) : static_cast<float>(s + 1);
    if (n > 1.f) g += logf(n) * e;
  }
  __shared__ float red[8];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) g += __shfl_down_sync(0xffffffffu, g, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = g;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) t += red[w];
    const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
    atomicAdd(dnorm + h, -sigma * (1.0f - sigma) * t);
  }
}

}  // namespace cott
