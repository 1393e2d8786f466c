// Fused causal cosine attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Math (GPT_Trainer/GPTCosAttention.py:229-248,282 of the reference):
//   q^ = q/|q|, k^ = k/|k|, v' = v / max(n_s^sigma(c_h), 1),  O_t = sum_{s<=t} (q^_t . k^_s) v'_s
// and its gradients.  Head dim 64, 16-bit inputs, fp32 accumulation.
//
// Chunked form, chunk = 128 positions, one CTA walks one (batch, head) sequence:
//   w_s  = a_s / |k_s|                      (a_s = length-norm factor, folded with the key norm)
//   Zw   = diag(w) Z                        (one row-scaled operand per chunk, rewritten in smem)
//   P    = mask(X Y^T)                      tcgen05 128x128x64, masked in registers, written back
//                                           to TMEM as 16-bit and used as the A operand from TMEM
//   Acc  = P Zw + X S                       tcgen05 128x64x128 + 128x64x64
//   S   += Y^T Zw                           tcgen05 64x64x128 (M=64), S lives in TMEM in fp32 and is
//                                           re-materialised in smem as a 16-bit operand per chunk
// forward:  (X, Y, Z) = (Q, K, V)   out_t = Acc_t / |q_t|
// dQ:       (X, Y, Z) = (dO, V, K)  dq^_t = Acc_t,  dq_t = (dq^_t - q^_t (q^_t . dq^_t)) / |q_t|
// dK, dV:   reverse direction, see causal_bwd_kv_kernel.
//
// HBM tiles arrive by TMA (128-byte swizzle, no multicast) into a 2-stage ring.  Every wait is
// bounded; on a time-out the CTA records a code in g_cott_status and leaves cleanly.
#pragma once

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace cott {

__device__ int g_cott_status;  // 0 = ok; else (code << 16 | chunk) of the first wait that gave up

constexpr int kTcChunk = 128;
constexpr int kTcD = 64;
constexpr int kTileBytes = kTcChunk * kTcD * 2;  // 16 KB: one [128 x 64] 16-bit tile

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
  static constexpr bool kBf16 = true;
};
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static constexpr bool kBf16 = false;
};

// Row `row` of a [128 x 64] 16-bit tile stored with the 128-byte swizzle: 16-byte piece j of the
// row sits at piece (j ^ (row & 7)).  Reads by 32 consecutive rows are bank-conflict free.
__device__ __forceinline__ uint4* tile_piece(unsigned char* tile, int row, int j) {
  return reinterpret_cast<uint4*>(tile + row * 128 + ((j ^ (row & 7)) << 4));
}

template <typename T>
__device__ __forceinline__ void load_row(unsigned char* tile, int row, float* x /*64*/) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 u = *tile_piece(tile, row, j);
    float2 a = Pack2<T>::unpack(u.x), b = Pack2<T>::unpack(u.y), c = Pack2<T>::unpack(u.z),
           d = Pack2<T>::unpack(u.w);
    x[8 * j + 0] = a.x; x[8 * j + 1] = a.y; x[8 * j + 2] = b.x; x[8 * j + 3] = b.y;
    x[8 * j + 4] = c.x; x[8 * j + 5] = c.y; x[8 * j + 6] = d.x; x[8 * j + 7] = d.y;
  }
}

template <typename T>
__device__ __forceinline__ float row_sumsq(unsigned char* tile, int row) {
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 u = *tile_piece(tile, row, j);
    float2 a = Pack2<T>::unpack(u.x), b = Pack2<T>::unpack(u.y), c = Pack2<T>::unpack(u.z),
           d = Pack2<T>::unpack(u.w);
    s += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
  }
  return s;
}

// tile[row] *= w (in place)
template <typename T>
__device__ __forceinline__ void scale_row(unsigned char* tile, int row, float w) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4* p = tile_piece(tile, row, j);
    uint4 u = *p;
    float2 a = Pack2<T>::unpack(u.x), b = Pack2<T>::unpack(u.y), c = Pack2<T>::unpack(u.z),
           d = Pack2<T>::unpack(u.w);
    u.x = Pack2<T>::pack(a.x * w, a.y * w);
    u.y = Pack2<T>::pack(b.x * w, b.y * w);
    u.z = Pack2<T>::pack(c.x * w, c.y * w);
    u.w = Pack2<T>::pack(d.x * w, d.y * w);
    *p = u;
  }
}

// 1 / max(|x|, 1e-12): torch.nn.functional.normalize's denominator (GPTCosAttention.py:229-230)
__device__ __forceinline__ float inv_norm(float sumsq) { return 1.0f / fmaxf(sqrtf(sumsq), 1e-12f); }

// a = 1 / max(n ** sigma, 1)  (GPTCosAttention.py:241), n >= 1
__device__ __forceinline__ float length_factor(float n, float sigma) {
  return 1.0f / fmaxf(exp2f(sigma * log2f(n)), 1.0f);
}

// Read `NB` blocks of 32 fp32 columns of this thread's TMEM lane, keep column s iff keep(s, row),
// convert to 16 bit and write the packed pairs back to TMEM starting at the same column base
// (packed column j holds elements 2j, 2j+1), for use as a tcgen05 A operand from TMEM.
// `lo` / `hi`: causal bounds -- element (row, s) survives iff lo <= s <= hi.
template <typename T>
__device__ __forceinline__ void mask_pack_inplace(uint32_t taddr_lane, int lo, int hi, int warp_lo_block,
                                                  int warp_hi_block) {
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    uint32_t packed[16];
    if (b < warp_lo_block || b > warp_hi_block) {  // warp-uniform: whole block masked out
#pragma unroll
      for (int j = 0; j < 16; ++j) packed[j] = 0u;
    } else {
      uint32_t r[32];
      ptx::tmem_ld_x32(taddr_lane + 32 * b, r);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int s0 = 32 * b + 2 * j;
        const float x0 = (s0 >= lo && s0 <= hi) ? __uint_as_float(r[2 * j]) : 0.f;
        const float x1 = (s0 + 1 >= lo && s0 + 1 <= hi) ? __uint_as_float(r[2 * j + 1]) : 0.f;
        packed[j] = Pack2<T>::pack(x0, x1);
      }
    }
    ptx::tmem_st_x8(taddr_lane + 16 * b, packed);
    ptx::tmem_st_x8(taddr_lane + 16 * b + 8, packed + 8);
  }
  ptx::tmem_st_wait();
}

enum { kModeFwd = 0, kModeDq = 1 };

// status codes recorded in g_cott_status
enum { kWaitTma = 1, kWaitP = 2, kWaitAcc = 3 };

template <typename T, int MODE>
__global__ void __launch_bounds__(128, 1)
causal_tc_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
                 const __grid_constant__ CUtensorMap mapZ, const __grid_constant__ CUtensorMap mapQ,
                 T* __restrict__ out, const float* __restrict__ norm_const, int H, int N) {
  using namespace ptx;
  constexpr int NT = (MODE == kModeFwd) ? 3 : 4;  // tiles per stage
  constexpr int STAGE = NT * kTileBytes;
  constexpr bool BF = Pack2<T>::kBf16;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  unsigned char* sStage[2] = {smem, smem + STAGE};
  unsigned char* sS = smem + 2 * STAGE;  // [64 x 64] 16-bit state operand, 8 KB
  __shared__ uint64_t bar_full[2], bar_p, bar_acc;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x;
  const int h = bh % H;
  const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
  const int nchunks = (N + kTcChunk - 1) / kTcChunk;

  if (tid == 0) {
    mbar_init(&bar_full[0], 1);
    mbar_init(&bar_full[1], 1);
    mbar_init(&bar_p, 1);
    mbar_init(&bar_acc, 1);
    mbar_fence_init();
    abort_flag = 0;
    tma_prefetch_desc(&mapX);
    tma_prefetch_desc(&mapY);
    tma_prefetch_desc(&mapZ);
    if (MODE == kModeDq) tma_prefetch_desc(&mapQ);
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tP = tmem, tAcc = tmem + 128, tS = tmem + 192;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;

  auto issue_loads = [&](int c) {
    unsigned char* st = sStage[c & 1];
    uint64_t* bar = &bar_full[c & 1];
    mbar_expect_tx(bar, STAGE);
    tma_load_3d(st, &mapX, bar, 0, c * kTcChunk, bh);
    tma_load_3d(st + kTileBytes, &mapY, bar, 0, c * kTcChunk, bh);
    tma_load_3d(st + 2 * kTileBytes, &mapZ, bar, 0, c * kTcChunk, bh);
    if (MODE == kModeDq) tma_load_3d(st + 3 * kTileBytes, &mapQ, bar, 0, c * kTcChunk, bh);
  };
  int pending[2] = {-1, -1};  // thread 0 only: chunk whose load into stage s has not been waited for
  if (tid == 0) {
    issue_loads(0);
    pending[0] = 0;
  }

  constexpr uint32_t kIdescP = make_idesc(128, 128, BF, false, false);
  constexpr uint32_t kIdescAcc = make_idesc(128, 64, BF, false, true);
  constexpr uint32_t kIdescS = make_idesc(64, 64, BF, true, true);

  int c = 0;
  for (; c < nchunks; ++c) {
    unsigned char* sX = sStage[c & 1];
    unsigned char* sY = sX + kTileBytes;
    unsigned char* sZ = sX + 2 * kTileBytes;
    unsigned char* sQ = (MODE == kModeDq) ? sX + 3 * kTileBytes : sX;
    unsigned char* sK = (MODE == kModeDq) ? sZ : sY;
    if (tid == 0 && c + 1 < nchunks) {
      issue_loads(c + 1);
      pending[(c + 1) & 1] = c + 1;
    }
    if (!mbar_wait(&bar_full[c & 1], (c >> 1) & 1)) {
      abort_flag = 1;
      atomicCAS(&g_cott_status, 0, (kWaitTma << 16) | c);
    } else if (tid == 0) {
      pending[c & 1] = -1;
    }

    // ---- prepare: row norms, length factor, Zw = diag(w) Z --------------------------------------
    const int row = tid;
    const int pos = c * kTcChunk + row;
    const float rq = inv_norm(row_sumsq<T>(sQ, row));
    const float rk = inv_norm(row_sumsq<T>(sK, row));
    const float a = length_factor(static_cast<float>(pos + 1), sigma);
    scale_row<T>(sZ, row, rk * a);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag) break;

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t x0 = smem_u32(sX), y0 = smem_u32(sY);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_ss(tP, make_smem_desc(x0 + 32 * k, 16, 1024), make_smem_desc(y0 + 32 * k, 16, 1024), kIdescP, k > 0);
      mma_commit(&bar_p);
      if (c > 0) {
        const uint32_t s0 = smem_u32(sS);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          mma_ss(tAcc, make_smem_desc(x0 + 32 * k, 16, 1024), make_smem_desc(s0 + 2048 * k, 8192, 1024),
                 kIdescAcc, k > 0);
      }
    }

    // ---- P: mask (s <= t), convert, back to TMEM as the A operand --------------------------------
    if (!mbar_wait(&bar_p, c & 1)) {
      abort_flag = 1;
      atomicCAS(&g_cott_status, 0, (kWaitP << 16) | c);
    }
    tc_fence_after_sync();
    mask_pack_inplace<T>(tP + lane_base, 0, row, 0, warp);
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag) break;

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t y0 = smem_u32(sY), z0 = smem_u32(sZ);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ts(tAcc, tP + 8 * k, make_smem_desc(z0 + 2048 * k, 8192, 1024), kIdescAcc, (c > 0 || k > 0));
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ss(tS, make_smem_desc(y0 + 2048 * k, 8192, 1024), make_smem_desc(z0 + 2048 * k, 8192, 1024), kIdescS,
               (c > 0 || k > 0));
      mma_commit(&bar_acc);
    }

    if (!mbar_wait(&bar_acc, c & 1)) {
      abort_flag = 1;
      atomicCAS(&g_cott_status, 0, (kWaitAcc << 16) | c);
    }
    tc_fence_after_sync();

    // ---- output rows -------------------------------------------------------------------------------
    {
      float acc[64];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint32_t r[32];
        tmem_ld_x32(tAcc + lane_base + 32 * b, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 * b + j] = __uint_as_float(r[j]);
      }
      if (MODE == kModeFwd) {
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] *= rq;
      } else {
        float qv[64];
        load_row<T>(sQ, row, qv);
        float delta = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          qv[j] *= rq;
          delta += qv[j] * acc[j];
        }
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] = rq * (acc[j] - qv[j] * delta);
      }
      if (pos < N) {
        uint4* dst = reinterpret_cast<uint4*>(out + (static_cast<size_t>(bh) * N + pos) * kTcD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 u;
          u.x = Pack2<T>::pack(acc[8 * j + 0], acc[8 * j + 1]);
          u.y = Pack2<T>::pack(acc[8 * j + 2], acc[8 * j + 3]);
          u.z = Pack2<T>::pack(acc[8 * j + 4], acc[8 * j + 5]);
          u.w = Pack2<T>::pack(acc[8 * j + 6], acc[8 * j + 7]);
          dst[j] = u;
        }
      }
    }

    // ---- state -> 16-bit operand for the next chunk (M=64 accumulator: row i sits in TMEM lane
    //      32*(i/16) + i%16, so lanes 0-15 of each warp hold rows 16*warp .. 16*warp+15) -----------
    if (c + 1 < nchunks) {
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint32_t r[32];
        tmem_ld_x32(tS + lane_base + 32 * b, r);
        tmem_ld_wait();
        if (lane < 16) {
          const int i = 16 * warp + lane;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 u;
            u.x = Pack2<T>::pack(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            u.y = Pack2<T>::pack(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            u.z = Pack2<T>::pack(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            u.w = Pack2<T>::pack(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *tile_piece(sS, i, 4 * b + j) = u;
          }
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag) break;
  }

  // ---- leave: drain any TMA still in flight (bounded), release TMEM ------------------------------
  if (tid == 0) {
    for (int s = 0; s < 2; ++s)
      if (pending[s] >= 0) mbar_wait(&bar_full[s], (pending[s] >> 1) & 1, 1u << 16);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// -------------------------------------------------------------------------------------------------
// dK, dV and the gradient of the length-norm parameter: one reverse-direction pass.
//
// With q^ = q/|q| (written back to smem as the 16-bit operand Qw), R = sum_{t > chunk} q^_t (x) dO_t:
//   E = mask_{t>=s}(V dO^T)        F = mask_{t>=s}(K Qw^T)            tcgen05 128x128x64 each
//   AccK = E Qw + V R^T            AccV = F dO + K R                  tcgen05 128x64x128 + 128x64x64
//   R   += Qw^T dO                                                    tcgen05 64x64x128 (M=64)
//   dv'_s = AccV_s / |k_s|         (gradient w.r.t. v' = a_s v)       dv_s = a_s dv'_s
//   eps_s = v'_s . dv'_s           (= k^_s . dk^_s)
//   dk^_s = a_s AccK_s             dk_s = (dk^_s - k^_s eps_s) / |k_s|
//   d norm_const[h] += -sigma (1 - sigma) sum_s ln(n_s) eps_s         (GPTCosAttention.py:241 by the chain rule)
template <typename T>
__global__ void __launch_bounds__(128, 1)
causal_bwd_kv_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                     const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                     T* __restrict__ dk, T* __restrict__ dv, float* __restrict__ dnorm,
                     const float* __restrict__ norm_const, int H, int N) {
  using namespace ptx;
  constexpr int STAGE = 4 * kTileBytes;
  constexpr bool BF = Pack2<T>::kBf16;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  unsigned char* sStage[2] = {smem, smem + STAGE};
  unsigned char* sR = smem + 2 * STAGE;  // [64 x 64] 16-bit state operand (rows = d_k, cols = d_v)
  __shared__ uint64_t bar_full[2], bar_p, bar_acc;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float red[4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x;
  const int h = bh % H;
  const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
  const int nchunks = (N + kTcChunk - 1) / kTcChunk;

  if (tid == 0) {
    mbar_init(&bar_full[0], 1);
    mbar_init(&bar_full[1], 1);
    mbar_init(&bar_p, 1);
    mbar_init(&bar_acc, 1);
    mbar_fence_init();
    abort_flag = 0;
    tma_prefetch_desc(&mapQ);
    tma_prefetch_desc(&mapK);
    tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapDO);
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t tE = tmem, tF = tmem + 128, tK = tmem + 256, tV = tmem + 320, tR = tmem + 384;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;

  // iteration ci handles chunk nchunks-1-ci
  auto issue_loads = [&](int ci) {
    const int y = (nchunks - 1 - ci) * kTcChunk;
    unsigned char* st = sStage[ci & 1];
    uint64_t* bar = &bar_full[ci & 1];
    mbar_expect_tx(bar, STAGE);
    tma_load_3d(st, &mapQ, bar, 0, y, bh);
    tma_load_3d(st + kTileBytes, &mapK, bar, 0, y, bh);
    tma_load_3d(st + 2 * kTileBytes, &mapV, bar, 0, y, bh);
    tma_load_3d(st + 3 * kTileBytes, &mapDO, bar, 0, y, bh);
  };
  int pending[2] = {-1, -1};
  if (tid == 0) {
    issue_loads(0);
    pending[0] = 0;
  }

  constexpr uint32_t kIdescP = make_idesc(128, 128, BF, false, false);
  constexpr uint32_t kIdescAccKK = make_idesc(128, 64, BF, false, false);  // B K-major (V R^T)
  constexpr uint32_t kIdescAccMN = make_idesc(128, 64, BF, false, true);   // B MN-major
  constexpr uint32_t kIdescR = make_idesc(64, 64, BF, true, true);

  float gsum = 0.f;  // sum_s ln(n_s) eps_s over this thread's rows

  for (int ci = 0; ci < nchunks; ++ci) {
    unsigned char* sQ = sStage[ci & 1];
    unsigned char* sK = sQ + kTileBytes;
    unsigned char* sV = sQ + 2 * kTileBytes;
    unsigned char* sDO = sQ + 3 * kTileBytes;
    if (tid == 0 && ci + 1 < nchunks) {
      issue_loads(ci + 1);
      pending[(ci + 1) & 1] = ci + 1;
    }
    if (!mbar_wait(&bar_full[ci & 1], (ci >> 1) & 1)) {
      abort_flag = 1;
      atomicCAS(&g_cott_status, 0, (kWaitTma << 16) | ci);
    } else if (tid == 0) {
      pending[ci & 1] = -1;
    }

    const int row = tid;
    const int pos = (nchunks - 1 - ci) * kTcChunk + row;
    const float rq = inv_norm(row_sumsq<T>(sQ, row));
    const float rk = inv_norm(row_sumsq<T>(sK, row));
    const float a = length_factor(static_cast<float>(pos + 1), sigma);
    scale_row<T>(sQ, row, rq);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag) break;

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t q0 = smem_u32(sQ), k0 = smem_u32(sK), v0 = smem_u32(sV), d0 = smem_u32(sDO);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_ss(tE, make_smem_desc(v0 + 32 * k, 16, 1024), make_smem_desc(d0 + 32 * k, 16, 1024), kIdescP, k > 0);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        mma_ss(tF, make_smem_desc(k0 + 32 * k, 16, 1024), make_smem_desc(q0 + 32 * k, 16, 1024), kIdescP, k > 0);
      mma_commit(&bar_p);
      if (ci > 0) {
        const uint32_t r0 = smem_u32(sR);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // AccK = V R^T : B[n = d_k][k = d_v] = R, K-major
          mma_ss(tK, make_smem_desc(v0 + 32 * k, 16, 1024), make_smem_desc(r0 + 32 * k, 16, 1024), kIdescAccKK,
                 k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // AccV = K R : B[n = d_v][k = d_k] = R, MN-major
          mma_ss(tV, make_smem_desc(k0 + 32 * k, 16, 1024), make_smem_desc(r0 + 2048 * k, 8192, 1024),
                 kIdescAccMN, k > 0);
      }
    }

    if (!mbar_wait(&bar_p, ci & 1)) {
      abort_flag = 1;
      atomicCAS(&g_cott_status, 0, (kWaitP << 16) | ci);
    }
    tc_fence_after_sync();
    mask_pack_inplace<T>(tE + lane_base, row, 127, warp, 3);
    mask_pack_inplace<T>(tF + lane_base, row, 127, warp, 3);
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag) break;

    if (tid == 0) {
      tc_fence_after_sync();
      const uint32_t q0 = smem_u32(sQ), d0 = smem_u32(sDO);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ts(tK, tE + 8 * k, make_smem_desc(q0 + 2048 * k, 8192, 1024), kIdescAccMN, (ci > 0 || k > 0));
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ts(tV, tF + 8 * k, make_smem_desc(d0 + 2048 * k, 8192, 1024), kIdescAccMN, (ci > 0 || k > 0));
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ss(tR, make_smem_desc(q0 + 2048 * k, 8192, 1024), make_smem_desc(d0 + 2048 * k, 8192, 1024), kIdescR,
               (ci > 0 || k > 0));
      mma_commit(&bar_acc);
    }

    if (!mbar_wait(&bar_acc, ci & 1)) {
      abort_flag = 1;
      atomicCAS(&g_cott_status, 0, (kWaitAcc << 16) | ci);
    }
    tc_fence_after_sync();

    float eps = 0.f;
    {  // dV
      float acc[64];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint32_t r[32];
        tmem_ld_x32(tV + lane_base + 32 * b, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 * b + j] = __uint_as_float(r[j]) * rk;  // dv'
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 u = *tile_piece(sV, row, j);
        float2 p0 = Pack2<T>::unpack(u.x), p1 = Pack2<T>::unpack(u.y), p2 = Pack2<T>::unpack(u.z),
               p3 = Pack2<T>::unpack(u.w);
        eps += p0.x * acc[8 * j] + p0.y * acc[8 * j + 1] + p1.x * acc[8 * j + 2] + p1.y * acc[8 * j + 3] +
               p2.x * acc[8 * j + 4] + p2.y * acc[8 * j + 5] + p3.x * acc[8 * j + 6] + p3.y * acc[8 * j + 7];
      }
      eps *= a;  // v' . dv'
      if (pos < N) {
        uint4* dst = reinterpret_cast<uint4*>(dv + (static_cast<size_t>(bh) * N + pos) * kTcD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 u;
          u.x = Pack2<T>::pack(a * acc[8 * j + 0], a * acc[8 * j + 1]);
          u.y = Pack2<T>::pack(a * acc[8 * j + 2], a * acc[8 * j + 3]);
          u.z = Pack2<T>::pack(a * acc[8 * j + 4], a * acc[8 * j + 5]);
          u.w = Pack2<T>::pack(a * acc[8 * j + 6], a * acc[8 * j + 7]);
          dst[j] = u;
        }
        if (pos > 0) gsum += logf(static_cast<float>(pos + 1)) * eps;
      }
    }
    {  // dK
      float acc[64];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint32_t r[32];
        tmem_ld_x32(tK + lane_base + 32 * b, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 * b + j] = __uint_as_float(r[j]) * a;  // dk^
      }
      const float ke = rk * eps;
      if (pos < N) {
        uint4* dst = reinterpret_cast<uint4*>(dk + (static_cast<size_t>(bh) * N + pos) * kTcD);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 kk = *tile_piece(sK, row, j);
          float2 p0 = Pack2<T>::unpack(kk.x), p1 = Pack2<T>::unpack(kk.y), p2 = Pack2<T>::unpack(kk.z),
                 p3 = Pack2<T>::unpack(kk.w);
          uint4 u;
          u.x = Pack2<T>::pack(rk * (acc[8 * j + 0] - p0.x * ke), rk * (acc[8 * j + 1] - p0.y * ke));
          u.y = Pack2<T>::pack(rk * (acc[8 * j + 2] - p1.x * ke), rk * (acc[8 * j + 3] - p1.y * ke));
          u.z = Pack2<T>::pack(rk * (acc[8 * j + 4] - p2.x * ke), rk * (acc[8 * j + 5] - p2.y * ke));
          u.w = Pack2<T>::pack(rk * (acc[8 * j + 6] - p3.x * ke), rk * (acc[8 * j + 7] - p3.y * ke));
          dst[j] = u;
        }
      }
    }

    if (ci + 1 < nchunks) {
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        uint32_t r[32];
        tmem_ld_x32(tR + lane_base + 32 * b, r);
        tmem_ld_wait();
        if (lane < 16) {
          const int i = 16 * warp + lane;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 u;
            u.x = Pack2<T>::pack(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            u.y = Pack2<T>::pack(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            u.z = Pack2<T>::pack(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            u.w = Pack2<T>::pack(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            *tile_piece(sR, i, 4 * b + j) = u;
          }
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (abort_flag) break;
  }

  // d norm_const: warp shuffle, then one atomic per CTA
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) gsum += __shfl_down_sync(0xffffffffu, gsum, off);
  if (lane == 0) red[warp] = gsum;
  if (tid == 0) {
    for (int s = 0; s < 2; ++s)
      if (pending[s] >= 0) mbar_wait(&bar_full[s], (pending[s] >> 1) & 1, 1u << 16);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0) atomicAdd(dnorm + h, -sigma * (1.0f - sigma) * (red[0] + red[1] + red[2] + red[3]));
  if (warp == 0) tmem_dealloc(tmem, 512);
}

inline size_t causal_bwd_kv_smem_bytes() { return static_cast<size_t>(2 * 4 * kTileBytes + kTcD * 128 + 1024); }

inline size_t causal_tc_smem_bytes(int mode) {
  const int nt = mode == kModeFwd ? 3 : 4;
  return static_cast<size_t>(2 * nt * kTileBytes + kTcD * 128 + 1024);
}

}  // namespace cott
