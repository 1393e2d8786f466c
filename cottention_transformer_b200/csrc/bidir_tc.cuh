// Bidirectional (encoder) cosine attention on the tensor cores (tcgen05 + TMEM + TMA), head dim 64,
// 16-bit inputs, fp32 accumulation.
//
// Math (BERT_Trainer/BertCosAttention.py:162-178,197-249 of the reference), per (batch, head):
//   keep_s = un-masked position, L = their count, a = 1 / max(L^sigmoid(c_h), 1)
//   q^ = keep q/|q|,  k^ = keep k/|k|,  v' = keep a v
//   S = sum_s k^_s (x) v'_s  [64 x 64],   out_t = q^_t S
// backward (autograd of the einsum; the reference's hand-written `Multiply.backward` is not used):
//   D = sum_t q^_t (x) dO_t,   dq^ = dO S^T,   dk^ = v' D^T,   dv' = k^ D
//   dq = keep/|q| (dq^ - q^ (q^.dq^)),  dk = 1/|k| (dk^ - k^ (k^.dk^)),  dv = keep a dv'
//   dc_h = -sigma (1 - sigma) ln(L) [L^sigma > 1] sum_s v'_s . dv'_s
//
// One CTA per (batch, head) walks the sequence twice in chunks of 128 positions: the first pass
// accumulates the state(s) in TMEM (M = 64 MMAs, one row-scaled operand per product), the second applies
// them.  With w_s = keep_s a / |k_s| and Zw = diag(w) V, Qw = diag(keep/|q|) Q:
//   S = K^T Zw,  D = Qw^T dO;   out = (Q S) keep/|q|;
//   AccQ = dO S^T,  AccK = Zw D^T = dk^/|k|,  AccV = K D = |k| dv'
//   dq = keep/|q| (AccQ - q^ (q^.AccQ)),  dk = AccK - k^ (k^.AccK),  dv = w AccV,  v'.dv' = w (v . AccV)
// Roles: warp 0 lane 0 = TMA loads and stores, warp 1 lane 0 = MMA issue, warps 2-5 = the per-row work
// (row norms, operand scaling in place, state conversion, output rows staged in place over an input
// tile and stored by TMA).  Every wait is bounded (see causal_tc.cuh).
#pragma once

#include "causal_tc.cuh"

namespace cott {

constexpr int kBtcThreads = 192;

// number of un-masked positions of one batch entry, computed redundantly by every warp that asks
__device__ __forceinline__ float btc_count_keep(const unsigned char* keep_b, int N, int lane) {
  if (!keep_b) return static_cast<float>(N);
  int cnt = 0;
  for (int s = lane; s < N; s += 32) cnt += keep_b[s] ? 1 : 0;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
  return static_cast<float>(cnt);
}

// -------------------------------------------------------------------------------------------------
// forward
// shared memory: kBtcKv x (K, V) tiles | 2 x Q tile (also the output staging buffer) | 16-bit state
// TMEM (128 columns): state 64 | accumulator 64
// Sized for three CTAs per SM (73 KB of shared memory, 128 TMEM columns each): the 384 (b,h) sequences of a
// BERT-base batch are then resident in one wave, and the CTAs of an SM cover each other's load and hand-off
// latency, which a deeper ring inside one CTA would otherwise have to.
constexpr int kBtcKv = 1;   // (K, V) stages
constexpr int kBtcAcc = 1;  // accumulator buffers
template <typename T>
__global__ void __launch_bounds__(kBtcThreads, 3)
bidir_fwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                    const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapOut,
                    const unsigned char* __restrict__ keep, const float* __restrict__ norm_const, int H, int N) {
  using namespace ptx;
  constexpr bool BF = Pack2<T>::kBf16;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sKV = smem;                                 // [kBtcKv][K tile, V tile]
  unsigned char* sQ = smem + 2 * kBtcKv * kTileBytes;        // [2]
  unsigned char* sS = smem + (2 * kBtcKv + 2) * kTileBytes;  // [64 x 64] 16-bit
  __shared__ uint64_t bar_full1[2], bar_prep1[2], bar_free1[2], bar_s_full, bar_state, bar_fullq[2], bar_acc_full[2],
      bar_acc_free[2], bar_out[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int bh = blockIdx.x, h = bh % H, b = bh / H, bb = b;
  const int nchunks = (N + kTcChunk - 1) / kTcChunk;
  const unsigned char* keep_b = keep ? keep + static_cast<size_t>(b) * N : nullptr;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_full1[s], 1);
      mbar_init(&bar_prep1[s], 4);
      mbar_init(&bar_free1[s], 1);
      mbar_init(&bar_fullq[s], 1);
      mbar_init(&bar_acc_full[s], 1);
      mbar_init(&bar_acc_free[s], 4);
      mbar_init(&bar_out[s], 4);
    }
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_state, 4);
    mbar_fence_init();
    abort_flag_s = 0;
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapOut);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem, tAcc0 = tmem + 64;
  constexpr uint32_t kIdescS = make_idesc(64, 64, BF, true, true);
  constexpr uint32_t kIdescAcc = make_idesc(128, 64, BF, false, true);

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      for (int c = 0; c < 2 && c < nchunks; ++c) {  // the first two Q tiles travel while the state is built
        mbar_expect_tx(&bar_fullq[c], kTileBytes);
        tma_load_tile(sQ + c * kTileBytes, &mapQ, &bar_fullq[c], c * kTcChunk, h, bb);
      }
      for (int c = 0; ok && c < nchunks; ++c) {
        const int s = c % kBtcKv;
        if (c >= kBtcKv && !(ok = wait_bar(&bar_free1[s], (c / kBtcKv - 1) & 1, abort_flag, kWaitStageFree, c))) break;
        unsigned char* st = sKV + s * 2 * kTileBytes;
        mbar_expect_tx(&bar_full1[s], 2 * kTileBytes);
        tma_load_tile(st, &mapK, &bar_full1[s], c * kTcChunk, h, bb);
        tma_load_tile(st + kTileBytes, &mapV, &bar_full1[s], c * kTcChunk, h, bb);
      }
      for (int c = 0; ok && c < nchunks; ++c) {
        const int s = c & 1;
        if (!(ok = wait_bar(&bar_out[s], (c >> 1) & 1, abort_flag, kWaitStageFree, c))) break;
        tma_store_tile(&mapOut, sQ + s * kTileBytes, c * kTcChunk, h, bb);
        tma_store_commit();
        if (c + 2 < nchunks) {
          tma_store_wait_read<0>();
          mbar_expect_tx(&bar_fullq[s], kTileBytes);
          tma_load_tile(sQ + s * kTileBytes, &mapQ, &bar_fullq[s], (c + 2) * kTcChunk, h, bb);
        }
      }
      tma_store_wait<0>();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int c = 0; ok && c < nchunks; ++c) {  // S += K^T Zw
        const int s = c % kBtcKv;
        if (!(ok = wait_bar1(&bar_prep1[s], (c / kBtcKv) & 1, abort_flag, kWaitPrepped, c))) break;
        tc_fence_after_sync();
        const uint32_t k0 = smem_u32(sKV + s * 2 * kTileBytes);
        const uint64_t dKm = mdesc(k0), dZm = mdesc(k0 + kTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ss(tS, dKm + 128 * k, dZm + 128 * k, kIdescS, (c > 0 || k > 0) ? 1u : 0u);
        mma_commit(&bar_free1[s]);  // the stage may be refilled once these MMAs have read it
      }
      if (ok) mma_commit(&bar_s_full);
      ok = ok && wait_bar1(&bar_state, 0, abort_flag, kWaitState, 0);
      const uint64_t dS = mdesc(smem_u32(sS));
      for (int c = 0; ok && c < nchunks; ++c) {  // Acc = Q S
        const int s = c & 1, ab = c % kBtcAcc;
        if (!(ok = wait_bar4(&bar_fullq[s], (c >> 1) & 1, c >= kBtcAcc ? &bar_acc_free[ab] : nullptr,
                             (c / kBtcAcc - 1) & 1, nullptr, 0, nullptr, 0, abort_flag, kWaitTma, c)))
          break;
        tc_fence_after_sync();
        const uint64_t dX = kdesc(smem_u32(sQ + s * kTileBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tAcc0 + 64 * ab, dX + 2 * k, dS + 128 * k, kIdescAcc, k > 0);
        mma_commit(&bar_acc_full[ab]);
      }
    }
  } else {
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    const float L = btc_count_keep(keep_b, N, lane);
    const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
    const float a = length_factor(fmaxf(L, 1.0f), sigma);
    bool ok = true;
    for (int c = 0; ok && c < nchunks; ++c) {  // Zw = diag(keep a / |k|) V, in place
      const int s = c % kBtcKv, pos = c * kTcChunk + row;
      if (!(ok = wait_bar_warp(&bar_full1[s], (c / kBtcKv) & 1, abort_flag, kWaitTma, c))) break;
      unsigned char* sK = sKV + s * 2 * kTileBytes;
      const bool kp = pos < N && (!keep_b || keep_b[pos]);
      const float w = kp ? inv_norm(row_sumsq_rolled<T>(sK, row)) * a : 0.f;
      scale_row_rolled<T>(sK + kTileBytes, row, w);
      fence_proxy_async_smem();
      warp_arrive(&bar_prep1[s], lane);
    }
    if (ok && (ok = wait_bar_warp(&bar_s_full, 0, abort_flag, kWaitState, 0))) {
      tc_fence_after_sync();
      state_to_smem_rolled<T>(tS + lane_base, sS, wq, lane);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&bar_state, lane);
    }
    for (int c = 0; ok && c < nchunks; ++c) {  // out = keep / |q| (Q S), staged over the Q tile
      const int s = c & 1, pos = c * kTcChunk + row;
      unsigned char* q = sQ + s * kTileBytes;
      if (!(ok = wait_bar_warp(&bar_fullq[s], (c >> 1) & 1, abort_flag, kWaitTma, c))) break;
      const bool kp = pos < N && (!keep_b || keep_b[pos]);
      const float rq = kp ? inv_norm(row_sumsq_rolled<T>(q, row)) : 0.f;
      const int ab = c % kBtcAcc;
      if (!(ok = wait_bar_warp(&bar_acc_full[ab], (c / kBtcAcc) & 1, abort_flag, kWaitAcc, c))) break;
      tc_fence_after_sync();
      row_from_acc<T, false>(q, row, tAcc0 + 64 * ab + lane_base, rq, 0.f);
      tc_fence_before_sync();
      warp_arrive(&bar_acc_free[ab], lane);
      fence_proxy_async_smem();
      warp_arrive(&bar_out[s], lane);
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {  // bounded drain of loads that may still be in flight
    for (int s = 0; s < 2; ++s) {
      mbar_wait(&bar_full1[s], 0, 64);
      mbar_wait(&bar_fullq[s], 0, 64);
    }
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
}

// -------------------------------------------------------------------------------------------------
// backward
// A persistent kernel: CTA x takes the sequences x, x + gridDim.x, ... (one CTA per SM), and the tiles of all its
// sequences go through ONE ring of three stages (q, K, V, dO tiles of a chunk).  A sequence is walked twice: the
// first pass builds the two states, the second applies them; dq, dk, dv rows are staged in place over the q, K, V
// tiles and leave by TMA.
// The kernel is bound by the bytes an SM can move (a traced CTA sustains ~40 GB/s: 64 KB loads that take 2-3 us,
// 48 KB stores), so the second pass does not load again what is still in shared memory: the last three chunks of
// the first pass stay in their stages ("resident") and are the first three chunks of the second pass; only the
// chunks before them are loaded a second time.  At BERT sizes (four chunks) a sequence is 5 loads instead of 8.
//   slots of a sequence (a slot = one load into the next stage of the ring):  first pass chunks 0 .. n-1, then the
//   reloads of chunks 0 .. n-R-1 (R = min(n, stages) resident chunks);
//   second pass order: the resident chunks n-R .. n-1, then the reloaded ones -- the order in which their stages
//   are needed again, so stages retire in slot order.
// A resident chunk arrives in the second pass as the first pass left it: the q tile holds Qw = q^, the V tile
// Zw = w v, and its row factors are in shared memory; a reloaded chunk is raw (its factors are computed again and
// the factor of Zw is applied to the dk rows instead, so nothing is rewritten before its MMAs).
// Why persistent: a sequence of four chunks cost 9 us of fixed latency (launch wave, TMEM allocation, first load,
// final stores), and 384 sequences on 148 SMs ran as three waves; here the ring carries on across sequences.
// Barrier phases: `full` completes once per slot, so its parity follows the slot number; the other per-stage barriers
// complete for some slots only, and each of their waiters waits for every completion, so each waiter keeps a phase
// bit per stage.
// TMEM (512 columns): S 64 | D 64 | 2 x (AccQ 64 | AccK 64 | AccV 64) -- the accumulators are double-buffered, so the
// MMAs of the next chunk run while the rows of this one are written (the second pass is a chain MMAs -> rows otherwise)
// Warps: 0 = TMA (lane 0), 1 = MMA issue (lane 0), three groups of four (each warp works on the tile rows /
// TMEM lanes 32 (w % 4) ..).  First pass: group 0 (warps 2-5) builds Qw, group 1 (6-9) Zw, in place, and both leave
// their row factors.  Second pass: group 0 writes the dv rows (and, for a reloaded chunk, the row factors first),
// group 1 the dq rows, group 2 (10-13) the dk rows.
constexpr int kBtcBwdThreads = 448;
constexpr int kBtcBwdStages = 3;

template <typename T>
__global__ void __launch_bounds__(kBtcBwdThreads, 1)
bidir_bwd_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                    const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                    const __grid_constant__ CUtensorMap mapDQ, const __grid_constant__ CUtensorMap mapDK,
                    const __grid_constant__ CUtensorMap mapDV, const unsigned char* __restrict__ keep,
                    const float* __restrict__ norm_const, float* __restrict__ dnorm, int H, int N, int BH) {
  using namespace ptx;
  constexpr bool BF = Pack2<T>::kBf16;
  constexpr int STAGE = 4 * kTileBytes;
  constexpr int NS = kBtcBwdStages;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sS = smem + NS * STAGE;     // [64 x 64] 16-bit, rows d_k
  unsigned char* sD = sS + kTcD * 128;       // [64 x 64] 16-bit, rows d_k
  __shared__ uint64_t bar_full[NS], bar_prep1[NS], bar_prep2[NS], bar_free1[NS], bar_out[NS], bar_st_full, bar_state, bar_acc_full[2],
      bar_acc_free[2];
  __shared__ float s_rq[NS][kTcChunk], s_rk[NS][kTcChunk], s_w[NS][kTcChunk];  // row factors of the second pass
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int n = (N + kTcChunk - 1) / kTcChunk;  // chunks of a sequence
  const int R = n < NS ? n : NS;                // chunks that stay in their stages between the two passes
  const int SL = 2 * n - R;                     // slots (loads) of a sequence: n first-pass chunks + n - R reloads
  const int nseq = (BH - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int total = nseq * SL;                  // slots of this CTA; slot t * SL + i of its t-th sequence, stage = slot % NS
  // second-pass item m of a sequence: its chunk and the slot that holds it
  auto p2_chunk = [&](int m) { return m < R ? n - R + m : m - R; };
  auto p2_slot = [&](int m) { return m < R ? n - R + m : n + (m - R); };
  auto seq_of = [&](int t) { return static_cast<int>(blockIdx.x) + t * static_cast<int>(gridDim.x); };

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_prep1[s], 8);  // groups 0 and 1
      mbar_init(&bar_prep2[s], 4);  // group 0
      mbar_init(&bar_free1[s], 1);
      mbar_init(&bar_out[s], 12);   // all three groups
    }
    mbar_init(&bar_st_full, 1);
    mbar_init(&bar_state, 8);       // groups 1 and 2
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_acc_full[i], 1);
      mbar_init(&bar_acc_free[i], 12);  // all three groups
    }
    mbar_fence_init();
    abort_flag_s = 0;
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapDO);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem, tD = tmem + 64, tAcc = tmem + 128;  // accumulator set i: AccQ, AccK, AccV at tAcc + 192 i + 0 / 64 / 128
  constexpr uint32_t kIdescS = make_idesc(64, 64, BF, true, true);
  constexpr uint32_t kIdescKK = make_idesc(128, 64, BF, false, false);  // B K-major
  constexpr uint32_t kIdescMN = make_idesc(128, 64, BF, false, true);   // B MN-major

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t ph_free1 = 0, ph_out = 0;  // phase bit per stage
      // hand back the stage of slot g: a first-pass chunk that does not stay is released by its MMAs, every other
      // slot once the three output tiles of its chunk have been stored from it
      auto retire = [&](int g) -> bool {
        const int t = g / SL, i = g - t * SL, s = g % NS;
        if (i < n - R) {
          const bool r = wait_bar(&bar_free1[s], (ph_free1 >> s) & 1, abort_flag, kWaitStageFree, g);
          ph_free1 ^= 1u << s;
          return r;
        }
        if (!wait_bar(&bar_out[s], (ph_out >> s) & 1, abort_flag, kWaitStageFree, g)) return false;
        ph_out ^= 1u << s;
        const int bh = seq_of(t), h = bh % H, bb = bh / H;
        unsigned char* st = smem + s * STAGE;
        const int y = (i < n ? i : i - n) * kTcChunk;
        tma_store_tile(&mapDQ, st, y, h, bb);
        tma_store_tile(&mapDK, st + kTileBytes, y, h, bb);
        tma_store_tile(&mapDV, st + 2 * kTileBytes, y, h, bb);
        tma_store_commit();
        tma_store_wait_read<0>();
        return true;
      };
      for (int g = 0; ok && g < total; ++g) {
        const int t = g / SL, i = g - t * SL, s = g % NS;
        const int bh = seq_of(t), h = bh % H, bb = bh / H;
        const int y = (i < n ? i : i - n) * kTcChunk;
        if (g >= NS && !(ok = retire(g - NS))) break;
        unsigned char* st = smem + s * STAGE;
        mbar_expect_tx(&bar_full[s], STAGE);
        tma_load_tile(st, &mapQ, &bar_full[s], y, h, bb);
        tma_load_tile(st + kTileBytes, &mapK, &bar_full[s], y, h, bb);
        tma_load_tile(st + 2 * kTileBytes, &mapV, &bar_full[s], y, h, bb);
        tma_load_tile(st + 3 * kTileBytes, &mapDO, &bar_full[s], y, h, bb);
      }
      for (int g = (total >= NS ? total - NS : 0); ok && g < total; ++g) ok = retire(g);
      tma_store_wait<0>();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      uint32_t ph_prep1 = 0;
      int p2 = 0;  // second-pass items issued so far (they take the two accumulator sets in turn, across sequences too)
      const uint64_t dSk = kdesc(smem_u32(sS)), dDk = kdesc(smem_u32(sD)), dDmn = mdesc(smem_u32(sD));
      for (int t = 0; ok && t < nseq; ++t) {
        const int g0 = t * SL;
        for (int j = 0; ok && j < n; ++j) {  // S += K^T Zw,  D += Qw^T dO
          const int s = (g0 + j) % NS;
          if (!(ok = wait_bar1(&bar_prep1[s], (ph_prep1 >> s) & 1, abort_flag, kWaitPrepped, g0 + j))) break;
          ph_prep1 ^= 1u << s;
          tc_fence_after_sync();
          const uint32_t q0 = smem_u32(smem + s * STAGE);
          const uint64_t dQm = mdesc(q0), dKm = mdesc(q0 + kTileBytes), dZm = mdesc(q0 + 2 * kTileBytes),
                         dDm = mdesc(q0 + 3 * kTileBytes);
#pragma unroll
          for (int k = 0; k < 8; ++k) mma_ss(tS, dKm + 128 * k, dZm + 128 * k, kIdescS, (j > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 8; ++k) mma_ss(tD, dQm + 128 * k, dDm + 128 * k, kIdescS, (j > 0 || k > 0) ? 1u : 0u);
          if (j < n - R) mma_commit(&bar_free1[s]);  // (a chunk that stays is not handed back here)
        }
        if (!ok) break;
        // (the commit also covers the second-pass MMAs of the previous sequence, which read the 16-bit states that
        // the conversion triggered by this barrier overwrites)
        mma_commit(&bar_st_full);
        if (!(ok = wait_bar1(&bar_state, t & 1, abort_flag, kWaitState, t))) break;
        for (int m = 0; ok && m < n; ++m, ++p2) {
          const int g = g0 + p2_slot(m), s = g % NS;
          // a reloaded chunk: its tiles as they arrive (nothing is rewritten before the MMAs); a resident one is
          // there already.  And the accumulators read out.
          const int ab = p2 & 1;
          const uint32_t tAQ = tAcc + 192 * ab, tAK = tAQ + 64, tAV = tAQ + 128;
          if (!(ok = wait_bar4(m >= R ? &bar_full[s] : nullptr, (g / NS) & 1, p2 >= 2 ? &bar_acc_free[ab] : nullptr,
                               ((p2 >> 1) - 1) & 1, nullptr, 0, nullptr, 0, abort_flag, kWaitPrepped, g)))
            break;
          tc_fence_after_sync();
          const uint32_t q0 = smem_u32(smem + s * STAGE);
          const uint64_t dK = kdesc(q0 + kTileBytes), dZ = kdesc(q0 + 2 * kTileBytes), dDO = kdesc(q0 + 3 * kTileBytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tAQ, dDO + 2 * k, dSk + 2 * k, kIdescKK, k > 0);   // AccQ = dO S^T
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tAK, dZ + 2 * k, dDk + 2 * k, kIdescKK, k > 0);    // AccK = (Zw or V) D^T
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tAV, dK + 2 * k, dDmn + 128 * k, kIdescMN, k > 0);  // AccV = K D
          mma_commit(&bar_acc_full[ab]);
        }
      }
    }
  } else {
    const int group = (warp - 2) >> 2;  // 0, 1, 2
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    uint32_t ph_prep2 = 0;
    int p2 = 0;  // second-pass items seen so far
    bool ok = true;
    for (int t = 0; ok && t < nseq; ++t) {
      const int g0 = t * SL;
      const int bh = seq_of(t), h = bh % H, b = bh / H;
      const unsigned char* keep_b = keep ? keep + static_cast<size_t>(b) * N : nullptr;
      const float L = btc_count_keep(keep_b, N, lane);
      const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
      const float a = length_factor(fmaxf(L, 1.0f), sigma);
      float gsum = 0.f;
      // ---- first pass: Qw = diag(keep / |q|) q (group 0),  Zw = diag(keep a / |k|) V (group 1), in place; the row
      // factors stay in shared memory for the chunks that stay
      if (group < 2) {
        for (int j = 0; ok && j < n; ++j) {
          const int g = g0 + j, s = g % NS, pos = j * kTcChunk + row;
          if (!(ok = wait_bar_warp(&bar_full[s], (g / NS) & 1, abort_flag, kWaitTma, g))) break;
          unsigned char* st = smem + s * STAGE;
          const bool kp = pos < N && (!keep_b || keep_b[pos]);
          if (group == 0) {
            const float rq = kp ? inv_norm(row_sumsq_rolled<T>(st, row)) : 0.f;
            s_rq[s][row] = rq;
            scale_row_rolled<T>(st, row, rq);
          } else {
            const float rk = kp ? inv_norm(row_sumsq_rolled<T>(st + kTileBytes, row)) : 0.f;
            s_rk[s][row] = rk;
            s_w[s][row] = rk * a;
            scale_row_rolled<T>(st + 2 * kTileBytes, row, rk * a);
          }
          fence_proxy_async_smem();
          warp_arrive(&bar_prep1[s], lane);
        }
      }
      // ---- the two states -> 16-bit operands (group 1: S, group 2: D)
      if (group >= 1 && ok && (ok = wait_bar_warp(&bar_st_full, t & 1, abort_flag, kWaitState, t))) {
        tc_fence_after_sync();
        if (group == 1)
          state_to_smem_rolled<T>(tS + lane_base, sS, wq, lane);
        else
          state_to_smem_rolled<T>(tD + lane_base, sD, wq, lane);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        warp_arrive(&bar_state, lane);
      }
      // ---- second pass
      for (int m = 0; ok && m < n; ++m, ++p2) {
        const int g = g0 + p2_slot(m), s = g % NS, pos = p2_chunk(m) * kTcChunk + row;
        const bool resident = m < R;  // the q tile holds Qw and the V tile Zw; the row factors are in shared memory
        const int ab = p2 & 1;
        const uint32_t tAQ = tAcc + 192 * ab, tAK = tAQ + 64, tAV = tAQ + 128;
        unsigned char* sQ = smem + s * STAGE;
        unsigned char* sK = sQ + kTileBytes;
        unsigned char* sV = sQ + 2 * kTileBytes;
        if (group == 0) {
          if (!resident) {  // the row factors of a reloaded chunk, for the other two groups
            if (!(ok = wait_bar_warp(&bar_full[s], (g / NS) & 1, abort_flag, kWaitTma, g))) break;
            const bool kp = pos < N && (!keep_b || keep_b[pos]);
            const float rk = kp ? inv_norm(row_sumsq_rolled<T>(sK, row)) : 0.f;
            s_rq[s][row] = kp ? inv_norm(row_sumsq_rolled<T>(sQ, row)) : 0.f;
            s_rk[s][row] = rk;
            s_w[s][row] = rk * a;
            warp_arrive(&bar_prep2[s], lane);
          }
          if (!(ok = wait_bar_warp(&bar_acc_full[ab], (p2 >> 1) & 1, abort_flag, kWaitAcc, g))) break;
          tc_fence_after_sync();
          // dv = w AccV;  v' . dv' = (w v) . AccV: the tile holds w v (resident) or v (reloaded)
          const float w = s_w[s][row];
          const float d = row_from_acc_dot<T>(sV, row, tAV + lane_base, w);
          gsum += resident ? d : w * d;
        } else {
          // groups 1 and 2: the row factors (prep2, for a reloaded chunk) and the accumulators
          if (!resident) {
            if (!(ok = wait_bar_warp(&bar_prep2[s], (ph_prep2 >> s) & 1, abort_flag, kWaitPrepped, g))) break;
            ph_prep2 ^= 1u << s;
          }
          if (!(ok = wait_bar_warp(&bar_acc_full[ab], (p2 >> 1) & 1, abort_flag, kWaitAcc, g))) break;
          tc_fence_after_sync();
          if (group == 1) {
            // dq = keep/|q| (dq^ - q^ (q^ . dq^)),  dq^ = AccQ; the tile holds q^ (resident) or q (reloaded: q^ = rq q)
            const float rq = s_rq[s][row];
            const float dotq = row_dot_acc<T>(sQ, row, tAQ + lane_base);
            row_from_acc<T, true>(sQ, row, tAQ + lane_base, rq, resident ? -rq * dotq : -rq * rq * rq * dotq);
          } else {
            // dk = dk^' - k^ (k^ . dk^') with dk^' = dk^ / |k| = AccK (resident: Zw D^T) or w AccK (reloaded: V D^T)
            const float rk = s_rk[s][row], w = resident ? 1.0f : s_w[s][row];
            const float dotk = row_dot_acc<T>(sK, row, tAK + lane_base);
            row_from_acc<T, true>(sK, row, tAK + lane_base, w, -rk * rk * w * dotk);
          }
        }
        tc_fence_before_sync();
        warp_arrive(&bar_acc_free[ab], lane);
        fence_proxy_async_smem();
        warp_arrive(&bar_out[s], lane);
      }
      if (group == 0 && ok) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) gsum += __shfl_down_sync(0xffffffffu, gsum, off);
        if (lane == 0 && L > 1.0f) atomicAdd(dnorm + h, -sigma * (1.0f - sigma) * __logf(L) * gsum);
      }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    for (int s = 0; s < NS; ++s) mbar_wait(&bar_full[s], 0, 64);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

inline size_t bidir_bwd_tc_smem_bytes() { return static_cast<size_t>(kBtcBwdStages * 4 * kTileBytes + 2 * kTcD * 128 + 1024); }

inline size_t bidir_fwd_tc_smem_bytes() { return static_cast<size_t>((2 * kBtcKv + 2) * kTileBytes + kTcD * 128 + 1024); }

}  // namespace cott
