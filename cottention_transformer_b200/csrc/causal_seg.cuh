// Segment-parallel causal cosine attention: the pieces that let one (batch, head) sequence be walked by
// several CTAs at once (long sequences with few (batch, head) pairs, e.g. B = 1, H = 16, N = 256k).
//
// The sequence is cut into segments of `chunks_per_seg` chunks.  A causal kernel that starts at a segment
// boundary only needs the state accumulated over everything before it (forward, dQ) or after it (dK/dV):
//   1. seg_state_kernel   one CTA per (b, h, segment): the segment's own contribution  sum_s y_s (x) z_s
//                         (forward state: y = k^, z = v';  reverse state: y = q^, z = dO), tcgen05 M = 64 MMAs
//   2. seg_scan_kernel    exclusive prefix (or suffix) sums over the segments of each (b, h), fp32
//   3. causal_tc_kernel / causal_bwd_kv_kernel with gridDim.y = number of segments and `init_state`
// Step 1 re-reads two of the tensors, i.e. the forward moves 6 instead of 4 tensor passes.
#pragma once

#include "causal_tc.cuh"

namespace cott {

constexpr int kSegThreads = 192;
// kSegRawState / kSegRawStateRev: plain Y^T Z for the bare scan; Rev numbers the segments from the end of the sequence
enum { kSegFwdState = 0, kSegRevState = 1, kSegRawState = 2, kSegRawStateRev = 3 };

// state[bh][seg] = sum over the chunks of the segment of Y^T Z with one operand row-scaled in place:
//   kSegFwdState: Y = K,  Z = diag(a_s / |k_s|) V      kSegRevState: Y = diag(1 / |q_t|) Q,  Z = dO
//   kSegRawState / kSegRawStateRev: Y, Z as they are
// shared memory: 2 x (Y, Z) tiles.  TMEM: 64 columns.
template <typename T, int MODE>
__global__ void __launch_bounds__(kSegThreads, 2)
seg_state_kernel(const __grid_constant__ CUtensorMap mapY, const __grid_constant__ CUtensorMap mapZ,
                 const float* __restrict__ norm_const, float* __restrict__ state, int H, int N, int chunks_per_seg,
                 const unsigned char* __restrict__ keep, const int* __restrict__ count) {
  using namespace ptx;
  constexpr bool BF = Pack2<T>::kBf16;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar_full[2], bar_prep[2], bar_free[2], bar_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int bh = blockIdx.x, h = bh % H, bb = bh / H, seg = blockIdx.y;
  const int total_chunks = (N + kTcChunk - 1) / kTcChunk;
  const int chunk0 = seg * chunks_per_seg;
  const int nchunks = min(chunks_per_seg, total_chunks - chunk0);
  const unsigned char* keep_b = keep ? keep + static_cast<size_t>(bh / H) * N : nullptr;
  const int* count_b = count ? count + static_cast<size_t>(bh / H) * N : nullptr;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_prep[s], 4);
      mbar_init(&bar_free[s], 1);
    }
    mbar_init(&bar_done, 1);
    mbar_fence_init();
    abort_flag_s = 0;
    tma_prefetch_desc(&mapY);
    tma_prefetch_desc(&mapZ);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tS = tmem_slot;
  constexpr uint32_t kIdescS = make_idesc(64, 64, BF, true, true);

  if (warp == 0) {
    if (lane == 0) {
      for (int c = 0; c < nchunks; ++c) {
        const int s = c & 1;
        if (c >= 2 && !wait_bar(&bar_free[s], ((c >> 1) - 1) & 1, abort_flag, kWaitStageFree, c)) break;
        unsigned char* st = smem + s * 2 * kTileBytes;
        mbar_expect_tx(&bar_full[s], 2 * kTileBytes);
        const int y = (MODE == kSegRawStateRev ? total_chunks - 1 - (chunk0 + c) : chunk0 + c) * kTcChunk;
        tma_load_tile(st, &mapY, &bar_full[s], y, h, bb);
        tma_load_tile(st + kTileBytes, &mapZ, &bar_full[s], y, h, bb);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int c = 0; ok && c < nchunks; ++c) {
        const int s = c & 1;
        if (!(ok = wait_bar1(&bar_prep[s], (c >> 1) & 1, abort_flag, kWaitPrepped, c))) break;
        tc_fence_after_sync();
        const uint32_t y0 = smem_u32(smem + s * 2 * kTileBytes);
        const uint64_t dYm = mdesc(y0), dZm = mdesc(y0 + kTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ss(tS, dYm + 128 * k, dZm + 128 * k, kIdescS, (c > 0 || k > 0) ? 1u : 0u);
        mma_commit(&bar_free[s]);
      }
      if (ok) mma_commit(&bar_done);
    }
  } else {
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    const float sigma = MODE >= kSegRawState ? 0.f : 1.0f / (1.0f + __expf(-norm_const[h]));
    bool ok = true;
    for (int c = 0; ok && c < nchunks; ++c) {
      const int s = c & 1;
      if (!(ok = wait_bar_warp(&bar_full[s], (c >> 1) & 1, abort_flag, kWaitTma, c))) break;
      unsigned char* sY = smem + s * 2 * kTileBytes;
      if constexpr (MODE < kSegRawState) {
        const RowMask m = row_mask(keep_b, count_b, (chunk0 + c) * kTcChunk + row, N);
        const float r = m.kp ? inv_norm(row_sumsq_rolled<T>(sY, row)) : 0.f;
        if (MODE == kSegFwdState)
          scale_row_rolled<T>(sY + kTileBytes, row, r * length_factor(m.n, sigma));
        else
          scale_row_rolled<T>(sY, row, r);
      }
      fence_proxy_async_smem();
      warp_arrive(&bar_prep[s], lane);
    }
    if (ok && wait_bar_warp(&bar_done, 0, abort_flag, kWaitState, 0)) {
      tc_fence_after_sync();
      // M=64 accumulator layout: lanes 0-15 of the warp that owns sub-partition q hold rows 16q .. 16q+15
      float* dst = state + ((static_cast<size_t>(bh) * gridDim.y + seg) * kTcD + 16 * wq + (lane & 15)) * kTcD;
#pragma unroll 1
      for (int blk = 0; blk < 4; ++blk) {
        uint32_t r[16];
        tmem_ld_x16(tS + lane_base + 16 * blk, r);
        tmem_ld_wait();
        if (lane < 16) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(dst + 16 * blk + 4 * j) =
                make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                            __uint_as_float(r[4 * j + 3]));
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    mbar_wait(&bar_full[0], 0, 64);
    mbar_wait(&bar_full[1], 0, 64);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tS, 64);
}

inline size_t seg_state_smem_bytes() { return static_cast<size_t>(4 * kTileBytes + 1024); }

// Exclusive scans over the segments of each (b, h):  grid = B*H, any block size.
//   prefix[seg]   = sum_{s' < seg} state[s']          (forward state before the segment)
//   prefix_t[seg] = prefix[seg] transposed            (the dQ pass uses the state with rows d_v)
//   suffix[seg]   = sum_{s' > seg} state[s']          (reverse state after the segment)
// Null outputs are skipped.
__global__ void seg_scan_kernel(const float* __restrict__ state, float* __restrict__ prefix, float* __restrict__ prefix_t,
                                float* __restrict__ suffix, int nseg) {
  const size_t base = static_cast<size_t>(blockIdx.x) * nseg * (kTcD * kTcD);
  for (int e = threadIdx.x; e < kTcD * kTcD; e += blockDim.x) {
    const int et = (e % kTcD) * kTcD + e / kTcD;
    if (prefix || prefix_t) {
      float run = 0.f;
      for (int s = 0; s < nseg; ++s) {
        if (prefix) prefix[base + static_cast<size_t>(s) * (kTcD * kTcD) + e] = run;
        if (prefix_t) prefix_t[base + static_cast<size_t>(s) * (kTcD * kTcD) + et] = run;
        run += state[base + static_cast<size_t>(s) * (kTcD * kTcD) + e];
      }
    }
    if (suffix) {
      float run = 0.f;
      for (int s = nseg - 1; s >= 0; --s) {
        suffix[base + static_cast<size_t>(s) * (kTcD * kTcD) + e] = run;
        run += state[base + static_cast<size_t>(s) * (kTcD * kTcD) + e];
      }
    }
  }
}

// Decode state of a whole prompt from its segment states: state[bh][j][i] (+)= sum_seg seg_state[bh][seg][i][j]
// (the decode kernel keeps the value index first, GPTCosAttention.py:264).  grid = B*H, any block size.
__global__ void seg_to_decode_state_kernel(const float* __restrict__ seg_state, float* __restrict__ state, int nseg,
                                           int accumulate) {
  const size_t base = static_cast<size_t>(blockIdx.x) * nseg * (kTcD * kTcD);
  float* dst = state + static_cast<size_t>(blockIdx.x) * (kTcD * kTcD);
  for (int e = threadIdx.x; e < kTcD * kTcD; e += blockDim.x) {
    const int j = e / kTcD, i = e % kTcD;  // output element [j][i] = input element [i][j]
    float sum = accumulate ? dst[e] : 0.f;
    for (int s = 0; s < nseg; ++s) sum += seg_state[base + static_cast<size_t>(s) * (kTcD * kTcD) + i * kTcD + j];
    dst[e] = sum;
  }
}

// count[b][s] = number of kept positions among 0 .. s of batch entry b (inclusive).  grid = B, block = 256.
__global__ void keep_count_kernel(const unsigned char* __restrict__ keep, int* __restrict__ count, int N) {
  __shared__ int part[256];
  const unsigned char* kb = keep + static_cast<size_t>(blockIdx.x) * N;
  int* cb = count + static_cast<size_t>(blockIdx.x) * N;
  const int per = (N + blockDim.x - 1) / blockDim.x;
  const int lo = min(static_cast<int>(threadIdx.x) * per, N), hi = min(lo + per, N);
  int sum = 0;
  for (int s = lo; s < hi; ++s) sum += kb[s] ? 1 : 0;
  part[threadIdx.x] = sum;
  __syncthreads();
  int run = 0;
  for (int t = 0; t < static_cast<int>(threadIdx.x); ++t) run += part[t];
  for (int s = lo; s < hi; ++s) {
    run += kb[s] ? 1 : 0;
    cb[s] = run;
  }
}

}  // namespace cott
