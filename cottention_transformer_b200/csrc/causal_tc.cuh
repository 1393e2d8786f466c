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
// Warp roles (listed at each kernel): single threads issue the MMAs and the TMA traffic; groups of four
// warps (one warp per TMEM sub-partition) do the per-row work -- mask + convert of P, row norms, Zw, the
// state conversion, output rows -- and hand work to each other through mbarriers, so the TMA of chunk
// c+3, the score MMA of chunk c+1, the mask pass of chunk c and the output pass of chunk c-1 overlap.
// HBM tiles arrive by TMA (128-byte swizzle, no multicast) into a 3-stage ring and outputs leave by TMA
// from a tile they are staged over.  Every wait is bounded; on a time-out the CTA records a code in
// g_cott_status and leaves cleanly.
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

// tile[row] *= w (in place), in packed 16-bit arithmetic.  w is split into a 16-bit head and a
// 16-bit tail, and x*w = fma(x, w_hi, x*w_lo): the tail product is tiny, so the result carries one
// 16-bit rounding, the same as converting the fp32 product -- at 2 instructions per element pair.
template <typename T> struct Vec2;
template <> struct Vec2<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ type bcast(float x) { return __float2bfloat162_rn(x); }
  static __device__ __forceinline__ float head(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Vec2<__half> {
  using type = __half2;
  static __device__ __forceinline__ type bcast(float x) { return __float2half2_rn(x); }
  static __device__ __forceinline__ float head(float x) { return __half2float(__float2half_rn(x)); }
};
// One MUFU.RSQ.  A non-zero 16-bit row has |x| >= 6e-8 > 1e-12, so the epsilon only ever matters for
// an all-zero row, whose normalised value is zero whatever the factor: return 0 there (a huge factor
// would overflow the 16-bit operand it is folded into).
__device__ __forceinline__ float inv_norm(float sumsq) { return sumsq > 0.f ? rsqrtf(sumsq) : 0.f; }

// a = 1 / max(n ** sigma, 1)  (GPTCosAttention.py:241), n >= 1
__device__ __forceinline__ float length_factor(float n, float sigma) {
  // 1 / max(n^sigma, 1) = min(2^(-sigma log2 n), 1); lg2.approx / ex2.approx, relative error ~1e-6
  return fminf(exp2f(-sigma * __log2f(n)), 1.0f);
}

// Padding: `keep` ([B, N] bytes, non-zero = un-masked) and `count` ([B, N] int32, inclusive running count of
// keep along the sequence) are both null (no padding: n_s = s + 1) or both set (GPTCosAttention.py:232-248:
// masked rows of q^, k^, v' are zero and n_s counts the un-masked positions up to s).
struct RowMask {
  bool kp;   // row takes part
  float n;   // n_s >= 1
};
__device__ __forceinline__ RowMask row_mask(const unsigned char* keep_b, const int* count_b, int pos, int N) {
  RowMask m;
  m.kp = pos < N && (!keep_b || keep_b[pos]);
  m.n = (count_b && pos < N) ? fmaxf(static_cast<float>(count_b[pos]), 1.0f) : static_cast<float>(pos + 1);
  return m;
}

// Bounded wait that also gives up when another role of the CTA has raised `abort_flag`.
// On its own time-out it raises the flag and records (code << 16 | chunk) in g_cott_status.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code,
                                         int chunk, uint32_t max_polls = ptx::kMaxPolls) {
  for (uint32_t i = 0; i < max_polls; ++i) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_cott_status, 0, (code << 16) | (chunk & 0xffff));
  return false;
}
// The same for a role that is a single thread: plain polling (no suspend hint), bounded by kMaxSpins.
__device__ __forceinline__ bool wait_bar1(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code,
                                          int chunk) {
  for (uint32_t i = 0; i < ptx::kMaxSpins; ++i) {
    if (ptx::mbar_test_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_cott_status, 0, (code << 16) | (chunk & 0xffff));
  return false;
}
// Two barriers at once: both try_waits are in flight together, so the pair costs one mbarrier
// round trip (about 200 cycles even for a completed phase) instead of two.
__device__ __forceinline__ bool wait_bar2(uint64_t* bar_a, uint32_t parity_a, uint64_t* bar_b, uint32_t parity_b,
                                          volatile int* abort_flag, int code, int chunk) {
  bool a = false, b = false;
  for (uint32_t i = 0; i < ptx::kMaxSpins; ++i) {
    const bool ta = a || ptx::mbar_test_wait(bar_a, parity_a);
    const bool tb = b || ptx::mbar_test_wait(bar_b, parity_b);
    a = ta;
    b = tb;
    if (a && b) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_cott_status, 0, (code << 16) | (chunk & 0xffff));
  return false;
}
// Up to four barriers at once (null entries are skipped).
__device__ __forceinline__ bool wait_bar4(uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1, uint64_t* b2, uint32_t p2,
                                          uint64_t* b3, uint32_t p3, volatile int* abort_flag, int code, int chunk) {
  bool d0 = b0 == nullptr, d1 = b1 == nullptr, d2 = b2 == nullptr, d3 = b3 == nullptr;
  for (uint32_t i = 0; i < ptx::kMaxSpins; ++i) {
    const bool t0 = d0 || ptx::mbar_test_wait(b0, p0);
    const bool t1 = d1 || ptx::mbar_test_wait(b1, p1);
    const bool t2 = d2 || ptx::mbar_test_wait(b2, p2);
    const bool t3 = d3 || ptx::mbar_test_wait(b3, p3);
    d0 = t0; d1 = t1; d2 = t2; d3 = t3;
    if (d0 && d1 && d2 && d3) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_cott_status, 0, (code << 16) | (chunk & 0xffff));
  return false;
}
// Whole-warp wait: every lane waits on the barrier itself (each thread must observe the completion
// to see TMA-written data) -- one warp-wide try_wait with a suspend hint, so a waiting warp sleeps in
// hardware instead of spinning; the outcome is made warp-uniform.
__device__ __forceinline__ bool wait_bar_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code,
                                              int chunk, uint32_t max_polls = ptx::kMaxPolls) {
  return __all_sync(0xffffffffu, wait_bar(bar, parity, abort_flag, code, chunk, max_polls) ? 1 : 0) != 0;
}
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive(bar);
}

// Mask + convert a 128-column fp32 score row held in this thread's TMEM lane and write it back to the
// same columns as packed 16-bit pairs (packed column j = elements 2j, 2j+1), for use as a tcgen05
// A operand from TMEM.  LOWER: element (row, s) survives iff s <= row (forward, dQ); else iff s >= row (dK/dV).
template <typename T, bool LOWER>
__device__ __forceinline__ void mask_pack_inplace(uint32_t taddr_lane, int lane, int wq) {
  // One 32-column block per iteration of a loop that is NOT unrolled: the fully unrolled form is four
  // times the code, and the roles of this kernel already overflow the instruction cache.  Packed block
  // b lands on fp32 columns 16b .. 16b+15, which belong to block b/2 <= b: already read.
  // The warp owns rows 32 wq .. 32 wq + 31 (row = 32 wq + lane): of the four column blocks, those on one
  // side of block wq are kept whole, those on the other side are zero, and only block wq needs the
  // per-element test (LOWER: column e of it survives iff e <= lane; else iff e >= lane).
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t packed[16];
    if (LOWER ? blk > wq : blk < wq) {  // warp-uniform: nothing of this block survives for any row
#pragma unroll
      for (int j = 0; j < 16; ++j) packed[j] = 0u;
    } else {
      uint32_t r[32];
      ptx::tmem_ld_x32(taddr_lane + 32 * blk, r);
      ptx::tmem_ld_wait();
      if (blk == wq) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const bool k0 = LOWER ? (2 * j <= lane) : (2 * j >= lane);
          const bool k1 = LOWER ? (2 * j + 1 <= lane) : (2 * j + 1 >= lane);
          packed[j] = Pack2<T>::pack(k0 ? __uint_as_float(r[2 * j]) : 0.f, k1 ? __uint_as_float(r[2 * j + 1]) : 0.f);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) packed[j] = Pack2<T>::pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
      }
    }
    ptx::tmem_st_x16(taddr_lane + 16 * blk, packed);
  }
  ptx::tmem_st_wait();
}

// fp32 state (M=64 accumulator: row i sits in TMEM lane 32*(i/16) + i%16, so lanes 0-15 of the warp
// that owns sub-partition q hold rows 16q .. 16q+15) -> 16-bit [64 x 64] swizzled smem operand.
// ---- rolled row routines ---------------------------------------------------------------------------
// The per-row work below is written as loops that are NOT unrolled (16 columns = two 16-byte pieces per
// trip).  Every role of these kernels runs on every scheduler, so the roles' code competes for one
// instruction cache; straight-line versions of these routines (4-8 times the code) measurably slowed
// all roles down.

// sum of squares of a tile row
template <typename T>
__device__ __forceinline__ float row_sumsq_rolled(unsigned char* tile, int row) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 1
  for (int j = 0; j < 8; j += 2) {
    const uint4 u = *tile_piece(tile, row, j), w = *tile_piece(tile, row, j + 1);
    float2 a = Pack2<T>::unpack(u.x), b = Pack2<T>::unpack(u.y), c = Pack2<T>::unpack(u.z), d = Pack2<T>::unpack(u.w);
    s0 = fmaf(a.x, a.x, fmaf(b.x, b.x, fmaf(c.x, c.x, fmaf(d.x, d.x, s0))));
    s1 = fmaf(a.y, a.y, fmaf(b.y, b.y, fmaf(c.y, c.y, fmaf(d.y, d.y, s1))));
    a = Pack2<T>::unpack(w.x), b = Pack2<T>::unpack(w.y), c = Pack2<T>::unpack(w.z), d = Pack2<T>::unpack(w.w);
    s2 = fmaf(a.x, a.x, fmaf(b.x, b.x, fmaf(c.x, c.x, fmaf(d.x, d.x, s2))));
    s3 = fmaf(a.y, a.y, fmaf(b.y, b.y, fmaf(c.y, c.y, fmaf(d.y, d.y, s3))));
  }
  return (s0 + s1) + (s2 + s3);
}

// 16 fp32 accumulator columns (this thread's TMEM lane, columns 16 blk ..) times the matching two pieces
// of a packed 16-bit row
template <typename T>
__device__ __forceinline__ float dot16(const uint32_t* r, const uint4& u, const uint4& w) {
  float2 a = Pack2<T>::unpack(u.x), b = Pack2<T>::unpack(u.y), c = Pack2<T>::unpack(u.z), d = Pack2<T>::unpack(u.w);
  float s0 = fmaf(a.x, __uint_as_float(r[0]), fmaf(b.x, __uint_as_float(r[2]),
                  fmaf(c.x, __uint_as_float(r[4]), d.x * __uint_as_float(r[6]))));
  float s1 = fmaf(a.y, __uint_as_float(r[1]), fmaf(b.y, __uint_as_float(r[3]),
                  fmaf(c.y, __uint_as_float(r[5]), d.y * __uint_as_float(r[7]))));
  a = Pack2<T>::unpack(w.x), b = Pack2<T>::unpack(w.y), c = Pack2<T>::unpack(w.z), d = Pack2<T>::unpack(w.w);
  s0 = fmaf(a.x, __uint_as_float(r[8]), fmaf(b.x, __uint_as_float(r[10]),
            fmaf(c.x, __uint_as_float(r[12]), fmaf(d.x, __uint_as_float(r[14]), s0))));
  s1 = fmaf(a.y, __uint_as_float(r[9]), fmaf(b.y, __uint_as_float(r[11]),
            fmaf(c.y, __uint_as_float(r[13]), fmaf(d.y, __uint_as_float(r[15]), s1))));
  return s0 + s1;
}
// (tile row) . (64 fp32 accumulator columns at taddr_lane)
template <typename T>
__device__ __forceinline__ float row_dot_acc(unsigned char* tile, int row, uint32_t taddr_lane) {
  float s = 0.f;
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t r[16];
    ptx::tmem_ld_x16(taddr_lane + 16 * blk, r);
    const uint4 u = *tile_piece(tile, row, 2 * blk), w = *tile_piece(tile, row, 2 * blk + 1);
    ptx::tmem_ld_wait();
    s += dot16<T>(r, u, w);
  }
  return s;
}
// tile row <- beta * (64 fp32 accumulator columns) + alpha * (tile row), in place (16-bit, swizzled)
// (`dst` = the tile that receives the row; by default the row is replaced in place)
template <typename T, bool kWithRow>
__device__ __forceinline__ void row_from_acc(unsigned char* tile, int row, uint32_t taddr_lane, float beta, float alpha,
                                             unsigned char* dst = nullptr) {
  if (dst == nullptr) dst = tile;
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t r[16];
    ptx::tmem_ld_x16(taddr_lane + 16 * blk, r);
    uint4* p0 = tile_piece(dst, row, 2 * blk);
    uint4* p1 = tile_piece(dst, row, 2 * blk + 1);
    uint4 u = make_uint4(0, 0, 0, 0), w = make_uint4(0, 0, 0, 0);
    if (kWithRow) {
      u = *tile_piece(tile, row, 2 * blk);
      w = *tile_piece(tile, row, 2 * blk + 1);
    }
    ptx::tmem_ld_wait();
    float x[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) x[j] = beta * __uint_as_float(r[j]);
    if (kWithRow) {
      const uint32_t q[8] = {u.x, u.y, u.z, u.w, w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = Pack2<T>::unpack(q[j]);
        x[2 * j] = fmaf(alpha, f.x, x[2 * j]);
        x[2 * j + 1] = fmaf(alpha, f.y, x[2 * j + 1]);
      }
    }
    u.x = Pack2<T>::pack(x[0], x[1]);   u.y = Pack2<T>::pack(x[2], x[3]);
    u.z = Pack2<T>::pack(x[4], x[5]);   u.w = Pack2<T>::pack(x[6], x[7]);
    w.x = Pack2<T>::pack(x[8], x[9]);   w.y = Pack2<T>::pack(x[10], x[11]);
    w.z = Pack2<T>::pack(x[12], x[13]); w.w = Pack2<T>::pack(x[14], x[15]);
    *p0 = u;
    *p1 = w;
  }
}
// One pass that does both: returns (tile row) . (64 fp32 accumulator columns) and replaces the tile row by
// beta * (those columns).  The accumulator is read once, so it can be handed back sooner.
template <typename T>
__device__ __forceinline__ float row_from_acc_dot(unsigned char* tile, int row, uint32_t taddr_lane, float beta,
                                                  unsigned char* dst = nullptr) {
  if (dst == nullptr) dst = tile;
  float s = 0.f;
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t r[16];
    ptx::tmem_ld_x16(taddr_lane + 16 * blk, r);
    uint4* p0 = tile_piece(dst, row, 2 * blk);
    uint4* p1 = tile_piece(dst, row, 2 * blk + 1);
    uint4 u = *tile_piece(tile, row, 2 * blk), w = *tile_piece(tile, row, 2 * blk + 1);
    ptx::tmem_ld_wait();
    s += dot16<T>(r, u, w);
    u.x = Pack2<T>::pack(beta * __uint_as_float(r[0]), beta * __uint_as_float(r[1]));
    u.y = Pack2<T>::pack(beta * __uint_as_float(r[2]), beta * __uint_as_float(r[3]));
    u.z = Pack2<T>::pack(beta * __uint_as_float(r[4]), beta * __uint_as_float(r[5]));
    u.w = Pack2<T>::pack(beta * __uint_as_float(r[6]), beta * __uint_as_float(r[7]));
    w.x = Pack2<T>::pack(beta * __uint_as_float(r[8]), beta * __uint_as_float(r[9]));
    w.y = Pack2<T>::pack(beta * __uint_as_float(r[10]), beta * __uint_as_float(r[11]));
    w.z = Pack2<T>::pack(beta * __uint_as_float(r[12]), beta * __uint_as_float(r[13]));
    w.w = Pack2<T>::pack(beta * __uint_as_float(r[14]), beta * __uint_as_float(r[15]));
    *p0 = u;
    *p1 = w;
  }
  return s;
}
// tile row *= w, in place (see scale_row for the arithmetic)
template <typename T>
__device__ __forceinline__ void scale_row_rolled(unsigned char* tile, int row, float w) {
  using V = typename Vec2<T>::type;
  const float wh = Vec2<T>::head(w);
  const V whi = Vec2<T>::bcast(wh), wlo = Vec2<T>::bcast(w - wh);
#pragma unroll 1
  for (int j = 0; j < 8; j += 2) {
    uint4* p0 = tile_piece(tile, row, j);
    uint4* p1 = tile_piece(tile, row, j + 1);
    uint4 u = *p0, v = *p1;
    if constexpr (Pack2<T>::kBf16) {
      V* x = reinterpret_cast<V*>(&u);
      V* y = reinterpret_cast<V*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x[e] = __hfma2(x[e], whi, __hmul2(x[e], wlo));
        y[e] = __hfma2(y[e], whi, __hmul2(y[e], wlo));
      }
    } else {  // float16 has too little range to hold the factor itself: multiply in fp32
      uint32_t* x = reinterpret_cast<uint32_t*>(&u);
      uint32_t* y = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = Pack2<T>::unpack(x[e]), g = Pack2<T>::unpack(y[e]);
        x[e] = Pack2<T>::pack(f.x * w, f.y * w);
        y[e] = Pack2<T>::pack(g.x * w, g.y * w);
      }
    }
    *p0 = u;
    *p1 = v;
  }
}
// Rotary position embedding inside the kernels (GPTCosAttention.py:458-476, "rotate every two"): the tables are
// fp32 [N, 4 * pieces] (sin and cos of the `4 * pieces` rotated pairs of a position; one table per batch entry when
// batch_stride != 0), `pieces` = rotary dim / 8 = the 16-byte pieces of a row that are rotated (a multiple of 2).
struct RotArgs {
  const float* sin;
  const float* cos;
  int pieces;
  long long batch_stride;
};
// A warp rotates its own 32 rows of a tile (rows 32 (warp % 4) ..): lane l takes piece l % 8 of the rows 4 i + l / 8,
// i = 0 .. 7, so that one load instruction of the warp covers four whole table rows (row-per-thread loads touch 32
// different lines per instruction and are bound by the load pipe).  A batch = the table values of four of a lane's
// eight rows, in registers; the loads of the first batch are issued before the wait that precedes the rotation (the position
// is known in advance), so their latency -- an L2 round trip -- hides behind it.
struct RotRegs {
  float4 sn[4], cs[4];
};
// `sin_tab`, `cos_tab`: the table rows of the warp's first row; `nrows`: how many of the warp's rows exist (<= 32)
__device__ __forceinline__ void rot_load(RotRegs& t, const float* __restrict__ sin_tab, const float* __restrict__ cos_tab, int lane,
                                         int batch, int pieces, int nrows) {
  const int pj = lane & 7;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 16 * batch + 4 * i + (lane >> 3);
    if (pj < pieces && r < nrows) {
      t.sn[i] = __ldg(reinterpret_cast<const float4*>(sin_tab + static_cast<size_t>(r) * (4 * pieces)) + pj);
      t.cs[i] = __ldg(reinterpret_cast<const float4*>(cos_tab + static_cast<size_t>(r) * (4 * pieces)) + pj);
    }
  }
}
// Rotates (INV: by the transposed rotation) the first 8 * pieces elements of the warp's rows `row_base` .. of one or
// two tiles that hold the same positions, in place; `t` holds the first batch.  Ends with a __syncwarp: the rows are then
// read row-per-thread.
template <typename T, bool INV, int NT>
__device__ __forceinline__ void rotate_rows(RotRegs& t, unsigned char* t0, unsigned char* t1, int row_base, int lane,
                                            const float* __restrict__ sin_tab, const float* __restrict__ cos_tab, int pieces,
                                            int nrows) {
  const int pj = lane & 7;
#pragma unroll 1
  for (int batch = 0; batch < 2; ++batch) {
    if (batch) rot_load(t, sin_tab, cos_tab, lane, 1, pieces, nrows);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 16 * batch + 4 * i + (lane >> 3);
      if (pj < pieces && r < nrows) {
        const float s4[4] = {t.sn[i].x, t.sn[i].y, t.sn[i].z, t.sn[i].w}, c4[4] = {t.cs[i].x, t.cs[i].y, t.cs[i].z, t.cs[i].w};
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
          uint4* p = tile_piece(tt ? t1 : t0, row_base + r, pj);
          uint4 u = *p;
          uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = Pack2<T>::unpack(w[e]);
            float xo, yo;
            rot_pair(f.x, f.y, c4[e], INV ? -s4[e] : s4[e], xo, yo);
            w[e] = Pack2<T>::pack(xo, yo);
          }
          *p = u;
        }
      }
    }
  }
  __syncwarp();
}
// fp32 state (M=64 accumulator layout, see state_to_smem) -> 16-bit swizzled smem operand
template <typename T>
__device__ __forceinline__ void state_to_smem_rolled(uint32_t tS_lane, unsigned char* sS, int wq, int lane) {
  const int i = 16 * wq + (lane & 15);
#pragma unroll 1
  for (int blk = 0; blk < 4; ++blk) {
    uint32_t r[16];
    ptx::tmem_ld_x16(tS_lane + 16 * blk, r);
    ptx::tmem_ld_wait();
    if (lane < 16) {
      uint4 u, w;
      u.x = Pack2<T>::pack(__uint_as_float(r[0]), __uint_as_float(r[1]));
      u.y = Pack2<T>::pack(__uint_as_float(r[2]), __uint_as_float(r[3]));
      u.z = Pack2<T>::pack(__uint_as_float(r[4]), __uint_as_float(r[5]));
      u.w = Pack2<T>::pack(__uint_as_float(r[6]), __uint_as_float(r[7]));
      w.x = Pack2<T>::pack(__uint_as_float(r[8]), __uint_as_float(r[9]));
      w.y = Pack2<T>::pack(__uint_as_float(r[10]), __uint_as_float(r[11]));
      w.z = Pack2<T>::pack(__uint_as_float(r[12]), __uint_as_float(r[13]));
      w.w = Pack2<T>::pack(__uint_as_float(r[14]), __uint_as_float(r[15]));
      *tile_piece(sS, i, 2 * blk) = u;
      *tile_piece(sS, i, 2 * blk + 1) = w;
    }
  }
}

// A segment's starting state (fp32 [64 x 64], row-major) -> TMEM in the M=64 accumulator layout (lanes 16-31
// of the warp belong to no row of that layout and receive a copy of lanes 0-15) and, as 16 bits, into the
// swizzled smem operand.  The caller waits for the TMEM stores (tcgen05.wait::st) and fences.
template <typename T>
__device__ __noinline__ void load_init_state(const float* state, uint32_t tS_lane, unsigned char* sS, int wq, int lane) {
  const float* src = state + (16 * wq + (lane & 15)) * kTcD;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 f = *reinterpret_cast<const float4*>(src + 32 * half + 4 * j);
      r[4 * j] = __float_as_uint(f.x), r[4 * j + 1] = __float_as_uint(f.y);
      r[4 * j + 2] = __float_as_uint(f.z), r[4 * j + 3] = __float_as_uint(f.w);
    }
    ptx::tmem_st_x32(tS_lane + 32 * half, r);
    if (lane < 16) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u;
        u.x = Pack2<T>::pack(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        u.y = Pack2<T>::pack(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        u.z = Pack2<T>::pack(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        u.w = Pack2<T>::pack(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        *tile_piece(sS, 16 * wq + lane, 4 * half + j) = u;
      }
    }
  }
}

// Descriptors of a [rows x 64] 16-bit tile with the 128-byte swizzle (see sm100_ptx.cuh).
// K-major: advance K by 16 elements = +32 B = +2 in descriptor units; MN-major: +2048 B = +128.
__device__ __forceinline__ uint64_t kdesc(uint32_t saddr) { return ptx::make_smem_desc(saddr, 16, 1024); }
__device__ __forceinline__ uint64_t mdesc(uint32_t saddr) { return ptx::make_smem_desc(saddr, 8192, 1024); }

// kModeScan / kModeScanRev: the bare scan out_t = sum_{s<=t} (x_t . y_s) z_s (s >= t when reversed, walking the
// sequence backwards) with no normalisation: the forward kernel minus its row scalings.
enum { kModeFwd = 0, kModeDq = 1, kModeScan = 2, kModeScanRev = 3 };

// which wait gave up (recorded in g_cott_status)
enum {
  kWaitTma = 1, kWaitStageFree = 2, kWaitScore = 3, kWaitScoreReady = 4, kWaitPrepped = 5, kWaitAcc = 6,
  kWaitAccFree = 7, kWaitState = 8
};

constexpr int kTcThreads = 896;  // forward / dQ: 3 issuing warps, 6 groups of 4 warps, 1 TMA warp
constexpr int kKvThreads = 480;  // dK/dV: 2 issuing warps, 3 groups of 4 warps, 1 TMA warp
constexpr int kKvThreadsRot = 608;  // + a group that rotates the Q and K tiles (rotary embedding inside the kernel)
constexpr int kTcStages = 3;
constexpr int kTcStagesFwd = 4;  // the forward kernel has the shared memory for a deeper ring (2 tiles per stage)

// EXT = false compiles the segment / padding arguments away (they must be null / one segment): these kernels are
// sensitive to every instruction added to their loops, and the common case needs neither.
// SAVE (forward only): the 16-bit state operand of every chunk -- the state BEFORE the chunk, [64 x 64], rows d_k --
// is also written to `saved` ([B*H][chunks of the sequence][64][64], row-major), for the one-pass backward.
// ROT (forward and dQ, EXT only, one segment): q and k are rotated by the rotary embedding inside the kernel -- the
// Q and K tiles are rewritten in shared memory before any MMA reads them, and the dQ rows are rotated back before
// they are stored -- so the tensors in HBM stay un-rotated and no separate pass over q, k, dq, dk is needed.
template <typename T, int MODE, bool EXT, bool SAVE = false, bool ROT = false>
__global__ void __launch_bounds__(kTcThreads, 1)
causal_tc_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
                 const __grid_constant__ CUtensorMap mapZ, const __grid_constant__ CUtensorMap mapQ,
                 const __grid_constant__ CUtensorMap mapOut, const float* __restrict__ norm_const, int H, int N,
                 const float* __restrict__ init_state_arg, int chunks_per_seg_arg,
                 const unsigned char* __restrict__ keep_arg, const int* __restrict__ count_arg,
                 uint4* __restrict__ saved, const RotArgs rot) {
  using namespace ptx;
  static_assert(!ROT || (EXT && !SAVE && (MODE == kModeFwd || MODE == kModeDq)), "rotary: forward / dQ, EXT, no saved states");
  // Shared memory: NS stages of the tiles that are only read (forward: Y, Z; dQ: X, Y, Z), a ring of
  // NS + 1 tiles for the tile that doubles as the output staging buffer (forward: X; dQ: q), the 16-bit
  // state operand (2 x 8 KB).  The ring is one slot longer than the stage count, so the tile of chunk c+NS
  // is loaded into the slot chunk c-1 left, while chunk c's output is still being written and stored.
  constexpr bool kScan = MODE >= kModeScan, kRev = MODE == kModeScanRev;
  constexpr int NIN = (MODE == kModeDq) ? 3 : 2;  // read-only tiles per stage
  constexpr int STAGE = NIN * kTileBytes;
  constexpr int NS = (MODE == kModeDq) ? kTcStages : kTcStagesFwd;
  constexpr int RING = NS + 1;
  constexpr int kIdxY = (MODE == kModeDq) ? 1 : 0, kIdxZ = kIdxY + 1;  // tile index inside a stage (dQ: X = 0)
  constexpr bool BF = Pack2<T>::kBf16;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms
  // (offset arithmetic on the __shared__ array keeps the pointer's address space known to the
  // compiler, so tile accesses compile to LDS/STS rather than generic loads and stores)
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* ring = smem + NS * STAGE;
  unsigned char* sS = ring + RING * kTileBytes;  // 2 x [64 x 64] 16-bit state operand (double-buffered)
  auto stage_of = [&](int c) { return smem + (c % NS) * STAGE; };
  auto ring_of = [&](int c) { return ring + (c % RING) * kTileBytes; };
  auto tile_x = [&](int c) { return MODE == kModeDq ? stage_of(c) : ring_of(c); };
  __shared__ uint64_t bar_full[NS], bar_free_in[NS], bar_out[NS], bar_prep[NS], bar_p_full[2], bar_p_ready[2], bar_acc_full[2],
      bar_acc_free[2], bar_s_full, bar_state[2], bar_state2, bar_init;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // broadcast: provably warp-uniform
  const int bh = blockIdx.x;
  const int h = bh % H, bb = bh / H;
  pdl_allow_next();  // the next kernel of the stream may set itself up on the SMs this one leaves free
  // Segment-parallel launches (gridDim.y > 1) give each CTA `chunks_per_seg` consecutive chunks of the
  // sequence and the state before its first chunk (`init_state[bh][seg]`, fp32 [64 x 64] in this kernel's
  // own state layout, rows = columns of Y); chunk numbers below are local, `chunk0 + c` is the position.
  const int total_chunks = (N + kTcChunk - 1) / kTcChunk;
  const float* init_state = EXT ? init_state_arg : nullptr;
  const int chunks_per_seg = EXT ? chunks_per_seg_arg : total_chunks;
  const int seg = EXT ? static_cast<int>(blockIdx.y) : 0;
  const int chunk0 = seg * chunks_per_seg;
  const int nchunks = EXT ? min(chunks_per_seg, total_chunks - chunk0) : total_chunks;
  const bool has_init = EXT && init_state != nullptr && seg > 0;
  const unsigned char* keep_b = (EXT && keep_arg) ? keep_arg + static_cast<size_t>(bh / H) * N : nullptr;
  const int* count_b = (EXT && count_arg) ? count_arg + static_cast<size_t>(bh / H) * N : nullptr;
  // first row of local chunk c (the reversed scan numbers chunks and segments from the end of the sequence)
  auto row0_of = [&](int c) { return (kRev ? total_chunks - 1 - (chunk0 + c) : chunk0 + c) * kTcChunk; };
  // table rows of position `pos` of this CTA's batch entry
  const long long rot_base = ROT ? static_cast<long long>(bb) * rot.batch_stride : 0;
  auto rot_sin = [&](int pos) { return rot.sin + rot_base + static_cast<long long>(pos) * (4 * rot.pieces); };
  auto rot_cos = [&](int pos) { return rot.cos + rot_base + static_cast<long long>(pos) * (4 * rot.pieces); };

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_free_in[s], 8);  // output group (accumulator MMAs done) + operand group (state MMAs done)
      mbar_init(&bar_out[s], 4);
      mbar_init(&bar_prep[s], 4);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bar_p_full[b], 1);
      mbar_init(&bar_p_ready[b], 4);
      mbar_init(&bar_acc_full[b], 1);
      mbar_init(&bar_acc_free[b], 4);
    }
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_state[0], 4);
    mbar_init(&bar_state[1], 4);
    mbar_init(&bar_state2, 4);
    mbar_init(&bar_init, 4);
    mbar_fence_init();
    abort_flag_s = 0;
    tma_prefetch_desc(&mapX);
    tma_prefetch_desc(&mapY);
    tma_prefetch_desc(&mapZ);
    if (MODE == kModeDq) tma_prefetch_desc(&mapQ);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  pdl_wait_prior();  // nothing another kernel may have written has been read so far
  const uint32_t tmem = tmem_slot;
  // TMEM columns: scores 2 x 128 | accumulators 2 x 64 | state 64
  const uint32_t tP0 = tmem, tAcc0 = tmem + 256, tS = tmem + 384;

  // Roles.  Two issuing threads on two different schedulers share the tensor-core issue work (a single
  // one was busy for the whole chunk period and so was the critical path); their MMAs are ordered only
  // through the mbarriers.  The per-row work is spread over six groups of four warps (warp w of a group
  // owns TMEM lanes / tile rows 32 (w % 4) ..): each group's work per chunk is serial and latency-bound,
  // so the chunk period is set by the busiest group.
  //   warp 0, lane 0:   scores P(c+1) = X Y^T
  //   warp 19, lane 0:  state S += Y^T Zw (c)
  //   warp 1, lane 0:   accumulators Acc(c) = X S + P Zw
  //   warps 2-5:        score group: mask + convert P
  //   warps 6-9, 20-23: output groups (even / odd chunks): row norm of q, accumulator -> output rows
  //   warps 10-13:      state group: fp32 state -> 16-bit operand
  //   warp 14, lane 0:  TMA loads and stores
  //   warps 15-18, 24-27: operand groups (even / odd chunks): Zw in place
  constexpr uint32_t kIdescP = make_idesc(128, 128, BF, false, false);
  constexpr uint32_t kIdescAcc = make_idesc(128, 64, BF, false, true);
  constexpr uint32_t kIdescS = make_idesc(64, 64, BF, true, true);
  if (warp == 0) {
    // ---------------------------------------------------------------- scores
    if (lane == 0) {
      auto issue_scores = [&](int c) {  // caller has waited for the TMA of chunk c and for the buffer
        const uint64_t dX = kdesc(smem_u32(tile_x(c))), dY = kdesc(smem_u32(stage_of(c) + kIdxY * kTileBytes));
        const uint32_t tP = tP0 + 128 * (c & 1);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tP, dX + 2 * k, dY + 2 * k, kIdescP, k > 0);
        mma_commit(&bar_p_full[c & 1]);
      };
      // (with the rotary embedding in the kernel the scores read the rotated Q and K tiles: wait for the operand group)
      constexpr bool kRotScores = ROT && MODE == kModeFwd;
      bool ok = kRotScores ? wait_bar2(&bar_full[0], 0, &bar_prep[0], 0, abort_flag, kWaitTma, 0)
                           : wait_bar1(&bar_full[0], 0, abort_flag, kWaitTma, 0);
      if (ok) {
        tc_fence_after_sync();
        issue_scores(0);
      }
      for (int c = 0; ok && c + 1 < nchunks; ++c) {
        {
          // scores of chunk c+1: its TMA, and (buffer reuse) the accumulator MMAs of chunk c-1 done
          const int s1 = (c + 1) % NS;
          ok = wait_bar4(&bar_full[s1], ((c + 1) / NS) & 1, c >= 1 ? &bar_acc_full[(c + 1) & 1] : nullptr,
                         ((c - 1) >> 1) & 1, kRotScores ? &bar_prep[s1] : nullptr, ((c + 1) / NS) & 1, nullptr, 0, abort_flag,
                         kWaitTma, c);
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores(c + 1);
        }
      }
    }
  } else if (warp == 19) {
    // ---------------------------------------------------------------- state
    // state MMA -> conversion -> next state MMA is the loop that sets the chunk period: its issuing thread
    // does nothing else
    if (lane == 0) {
      for (int c = 0; c + 1 < nchunks; ++c) {
        {
          // state update of chunk c: Zw(c), and the conversion of S after chunk c-1
          if (!wait_bar4(&bar_prep[c % NS], (c / NS) & 1, c > 0 ? &bar_state2 : (has_init ? &bar_init : nullptr),
                         c > 0 ? ((c - 1) & 1) : 0, nullptr, 0, nullptr, 0, abort_flag, kWaitPrepped, c))
            break;
          tc_fence_after_sync();
          const uint32_t y0 = smem_u32(stage_of(c) + kIdxY * kTileBytes);
          const uint64_t dYm = mdesc(y0), dZm = mdesc(y0 + kTileBytes);
          mma_ss(tS, dYm, dZm, kIdescS, (c > 0 || has_init) ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k) mma_ss(tS, dYm + 128 * k, dZm + 128 * k, kIdescS, 1u);
          mma_commit(&bar_s_full);
        }
      }
    }
  } else if (warp == 14) {
    // ---------------------------------------------------------------- TMA loads and stores
    // A thread of its own.  The output rows of a chunk are staged over the ring tile of the chunk (forward:
    // the X tile, dQ: the q tile -- the tile whose rows the output group reads last) and stored from there.
    if (lane == 0) {
      auto issue_loads = [&](int c) {
        const int s = c % NS;
        unsigned char* st = stage_of(c);
        mbar_expect_tx(&bar_full[s], STAGE + kTileBytes);
        if (MODE == kModeDq) tma_load_tile(st, &mapX, &bar_full[s], row0_of(c), h, bb);
        tma_load_tile(st + kIdxY * kTileBytes, &mapY, &bar_full[s], row0_of(c), h, bb);
        tma_load_tile(st + kIdxZ * kTileBytes, &mapZ, &bar_full[s], row0_of(c), h, bb);
        tma_load_tile(ring_of(c), MODE == kModeDq ? &mapQ : &mapX, &bar_full[s], row0_of(c), h, bb);
      };
      for (int c = 0; c < NS && c < nchunks; ++c) issue_loads(c);
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % NS;
        if (c + NS < nchunks) {
          // every MMA of chunk c has completed; the ring slot of chunk c+NS is the one chunk c-1 was stored
          // from (group committed one iteration ago): make sure the TMA engine has read it
          if (!wait_bar(&bar_free_in[s], (c / NS) & 1, abort_flag, kWaitStageFree, c)) break;
          tma_store_wait_read<0>();
          issue_loads(c + NS);
        }
        if (!wait_bar(&bar_out[s], (c / NS) & 1, abort_flag, kWaitStageFree, c)) break;
        tma_store_tile(&mapOut, ring_of(c), row0_of(c), h, bb);
        tma_store_commit();
      }
      tma_store_wait<0>();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- accumulators
    if (lane == 0) {
      const uint64_t dS0 = mdesc(smem_u32(sS));
      for (int c = 0; c < nchunks; ++c) {
        const int s = c % NS, b = c & 1;
        const uint64_t dX = kdesc(smem_u32(tile_x(c))), dZm = mdesc(smem_u32(stage_of(c) + kIdxZ * kTileBytes));
        const uint32_t tP = tP0 + 128 * b, tAcc = tAcc0 + 64 * b;
        // masked scores of chunk c, the 16-bit state after chunk c-1, the accumulator buffer read out, Zw(c)
        if (!wait_bar4(&bar_p_ready[b], (c >> 1) & 1, c > 0 ? &bar_state[(c - 1) & 1] : (has_init ? &bar_init : nullptr),
                       c > 0 ? (((c - 1) >> 1) & 1) : 0,
                       c >= 2 ? &bar_acc_free[b] : nullptr, ((c >> 1) - 1) & 1, &bar_prep[s], (c / NS) & 1, abort_flag,
                       kWaitScoreReady, c))
          break;
        tc_fence_after_sync();
        if (c > 0 || has_init) {
          const uint64_t dS = dS0 + static_cast<uint64_t>(b * ((kTcD * 128) >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k)  // Acc = X S   (S as MN-major B operand)
            mma_ss(tAcc, dX + 2 * k, dS + 128 * k, kIdescAcc, k > 0);
        }
        mma_ts(tAcc, tP, dZm, kIdescAcc, (c > 0 || has_init) ? 1u : 0u);  // Acc += P Zw   (P from TMEM, Zw MN-major)
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ts(tAcc, tP + 8 * k, dZm + 128 * k, kIdescAcc, 1u);
        mma_commit(&bar_acc_full[b]);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- score group
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    for (int c = 0; c < nchunks; ++c) {
      const int b = c & 1;
      if (!wait_bar_warp(&bar_p_full[b], (c >> 1) & 1, abort_flag, kWaitScore, c)) break;
      tc_fence_after_sync();
      mask_pack_inplace<T, !kRev>(tP0 + 128 * b + lane_base, lane, wq);
      tc_fence_before_sync();
      warp_arrive(&bar_p_ready[b], lane);
    }
  } else if (warp >= 10 && warp < 14) {
    // ---------------------------------------------------------------- state group
    const int wq = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    if (has_init) {
      // the state before this segment: fp32 into TMEM, 16-bit into the operand buffer of chunk 0
      load_init_state<T>(init_state + (static_cast<size_t>(bh) * gridDim.y + seg) * (kTcD * kTcD), tS + lane_base, sS, wq, lane);
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&bar_init, lane);
      if (SAVE && lane < 16) {  // the state before the segment's first chunk, as the operand buffer holds it
        uint4* dst = saved + ((static_cast<size_t>(bh) * total_chunks + chunk0) * kTcD + 16 * wq + lane) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = *tile_piece(sS, 16 * wq + lane, j);
      }
    }
    for (int c = 0; c + 1 < nchunks; ++c) {
      // S after chunk c -> 16-bit operand for chunk c+1 (buffer (c+1)&1)
      if (!wait_bar_warp(&bar_s_full, c & 1, abort_flag, kWaitState, c)) break;
      tc_fence_after_sync();
      if (lane == 0) mbar_arrive(&bar_free_in[c % NS]);  // the state MMAs of chunk c have read its tiles
      // The state MMA of chunk c+1 waits for this read of the fp32 state (and the accumulator MMAs of
      // chunk c+1 for the 16-bit copy): that loop sets the chunk period.  So the read is reported as soon
      // as the second half of the row has arrived, before its conversion and the shared-memory writes.
      {
        uint32_t r[32], pk[32];
        tmem_ld_x32(tS + lane_base, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = Pack2<T>::pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        tmem_ld_x32(tS + lane_base + 32, r);
        tmem_ld_wait();
        tc_fence_before_sync();
        warp_arrive(&bar_state2, lane);
#pragma unroll
        for (int j = 0; j < 16; ++j)
          pk[16 + j] = Pack2<T>::pack(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        // The 16-bit buffer written now was last read by the accumulator MMAs of chunk c-1.  (The state
        // thread runs ahead of the accumulator thread, so nothing else orders the two.)
        if (c > 0 && !wait_bar_warp(&bar_acc_full[(c - 1) & 1], ((c - 1) >> 1) & 1, abort_flag, kWaitAccFree, c)) break;
        if (lane < 16) {
          unsigned char* dst = sS + ((c + 1) & 1) * (kTcD * 128);
          const int i = 16 * wq + lane;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *tile_piece(dst, i, j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
        }
      }
      fence_proxy_async_smem();
      warp_arrive(&bar_state[c & 1], lane);
      if (SAVE && lane < 16) {  // after the hand-off: the stores are off the loop that sets the chunk period
        uint4* dst = saved + ((static_cast<size_t>(bh) * total_chunks + chunk0 + c + 1) * kTcD + 16 * wq + lane) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = *tile_piece(sS + ((c + 1) & 1) * (kTcD * 128), 16 * wq + lane, j);
      }
    }
  } else if ((warp >= 15 && warp < 19) || warp >= 24) {
    // ---------------------------------------------------------------- operand groups (even / odd chunks)
    const int row = 32 * (warp & 3) + lane;
    const float sigma = kScan ? 0.f : 1.0f / (1.0f + __expf(-norm_const[h]));
    const int mine = (warp >= 24) ? 1 : 0;
    for (int c = 0; c < nchunks; ++c) {  // Zw = diag(a_s / |k_s|) Z, in place
      const int s = c % NS;
      // Every phase of a barrier has to be observed, also for the chunks of the other group: a parity
      // wait cannot tell phase n from phase n+2, and with 3 stages a group that only looked at its own
      // chunks would skip every other phase of each `full` barrier.
      RotRegs rt;
      const int wrow0 = row0_of(c) + 32 * (warp & 3);  // position of the warp's first row
      if (ROT && (c & 1) == mine) rot_load(rt, rot_sin(wrow0), rot_cos(wrow0), lane, 0, rot.pieces, N - wrow0);
      if (!wait_bar_warp(&bar_full[s], (c / NS) & 1, abort_flag, kWaitTma, c)) break;
      if ((c & 1) != mine) continue;
      unsigned char* sZ = stage_of(c) + kIdxZ * kTileBytes;
      unsigned char* sK = (MODE == kModeDq) ? sZ : stage_of(c) + kIdxY * kTileBytes;
      // (rotary: the K rows and the Q / q rows of these positions, with the same table values.  This group runs ahead
      // of the MMAs -- it waits for nothing but the loads -- so the rotation is off the chain that sets the chunk period.)
      if constexpr (ROT)
        rotate_rows<T, false, 2>(rt, ring_of(c), sK, 32 * (warp & 3), lane, rot_sin(wrow0), rot_cos(wrow0), rot.pieces, N - wrow0);
      if constexpr (!kScan) {
        const RowMask m = row_mask(keep_b, count_b, row0_of(c) + row, N);
        const float rk = m.kp ? inv_norm(row_sumsq_rolled<T>(sK, row)) : 0.f;
        scale_row_rolled<T>(sZ, row, rk * length_factor(m.n, sigma));
      }
      fence_proxy_async_smem();
      warp_arrive(&bar_prep[s], lane);
    }
  } else {
    // ---------------------------------------------------------------- output groups (even / odd chunks)
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    const int mine = (warp >= 20) ? 1 : 0;
    for (int c = 0; c < nchunks; ++c) {
      const int s = c % NS, b = c & 1;
      unsigned char* sQ = ring_of(c);  // forward: X; dQ: q
      // the row norm of q only needs the TMA data: do it while the MMAs run
      // (every phase of `full` is observed, also for the other group's chunks: see the operand groups)
      const int wrow0 = row0_of(c) + 32 * wq;  // position of the warp's first row
      if (!wait_bar_warp(&bar_full[s], (c / NS) & 1, abort_flag, kWaitTma, c)) break;
      if ((c & 1) != mine) continue;
      // (rotary in the kernel: the tile is rotated by the operand group, so its norm is taken once the MMAs, which
      // wait for that group, have completed -- the value read never depends on which of the two groups was faster)
      float rq = 1.f;
      if (!kScan && !ROT) rq = row_mask(keep_b, count_b, row0_of(c) + row, N).kp ? inv_norm(row_sumsq_rolled<T>(sQ, row)) : 0.f;
      if (!wait_bar_warp(&bar_acc_full[b], (c >> 1) & 1, abort_flag, kWaitAcc, c)) break;
      tc_fence_after_sync();
      if (ROT) rq = row_mask(keep_b, count_b, row0_of(c) + row, N).kp ? inv_norm(row_sumsq_rolled<T>(sQ, row)) : 0.f;
      // The score and accumulator MMAs of this chunk have completed (the operand group reports the state
      // MMAs): the stage can be refilled.
      if (lane == 0) mbar_arrive(&bar_free_in[s]);
      // The staging tile has no MMA reader left (forward: X, whose row norm this thread has taken; dQ: the
      // q tile, which no MMA reads).  Its rows are replaced in place, in the swizzled layout, by the
      // output rows; the TMA thread stores the tile and refills it.
      const uint32_t tAcc = tAcc0 + 64 * b + lane_base;
      if (MODE != kModeDq) {
        row_from_acc<T, false>(sQ, row, tAcc, rq, 0.f);  // o = acc / |q|  (the bare scan: o = acc)
      } else {
        // dq = (dq^ - q^ (q^ . dq^)) / |q| with dq^ = acc and q^ = rq q
        const float delta = row_dot_acc<T>(sQ, row, tAcc) * (rq * rq * rq);
        row_from_acc<T, true>(sQ, row, tAcc, rq, -delta);
      }
      tc_fence_before_sync();
      warp_arrive(&bar_acc_free[b], lane);
      if (ROT && MODE == kModeDq) {  // the rows are the gradient of the rotated q: back through the rotation
        RotRegs rt;
        __syncwarp();  // the rows are now rotated piece-per-lane
        rot_load(rt, rot_sin(wrow0), rot_cos(wrow0), lane, 0, rot.pieces, N - wrow0);
        rotate_rows<T, true, 1>(rt, sQ, sQ, 32 * wq, lane, rot_sin(wrow0), rot_cos(wrow0), rot.pieces, N - wrow0);
      }
      fence_proxy_async_smem();
      warp_arrive(&bar_out[s], lane);
    }
  }

  // ---- leave: make sure no TMA of this CTA is still in flight (bounded), release TMEM ------------
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    for (int c = (nchunks > NS ? nchunks - NS : 0); c < nchunks; ++c)
      mbar_wait(&bar_full[c % NS], (c / NS) & 1, 64);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
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
// Same warp roles as causal_tc_kernel; the two score tiles fill TMEM, so they are single-buffered:
// the score MMAs of chunk c+1 are queued right behind the accumulator MMAs of chunk c.
// ROT: as in causal_tc_kernel -- the Q and K tiles are rotated in shared memory, by a warp group of their own that
// works as soon as a stage has arrived (two chunks ahead of its use: the rotation is off the chain that sets the chunk
// period), and the dK rows are rotated back before they are stored.
template <typename T, bool EXT, bool ROT = false>
__global__ void __launch_bounds__(ROT ? kKvThreadsRot : kKvThreads, 1)
causal_bwd_kv_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                     const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapDO,
                     const __grid_constant__ CUtensorMap mapDK, const __grid_constant__ CUtensorMap mapDV, float* __restrict__ dnorm,
                     const float* __restrict__ norm_const, int H, int N, const float* __restrict__ init_state_arg,
                     int chunks_per_seg_arg, const unsigned char* __restrict__ keep_arg,
                     const int* __restrict__ count_arg, const RotArgs rot) {
  using namespace ptx;
  static_assert(!ROT || EXT, "rotary: EXT only");
  constexpr int STAGE = 4 * kTileBytes;
  constexpr int NS = kTcStages;
  constexpr bool BF = Pack2<T>::kBf16;

  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // (offset arithmetic on the __shared__ array keeps the pointer's address space known to the
  // compiler, so tile accesses compile to LDS/STS rather than generic loads and stores)
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sR = smem + NS * STAGE;  // 2 x [64 x 64] 16-bit state operand (rows = d_k, cols = d_v), double-buffered
  __shared__ uint64_t bar_full[NS], bar_free_in[NS], bar_out[NS], bar_prep[NS], bar_rot[NS], bar_p_full, bar_p_ready, bar_acc_full,
      bar_acc_free, bar_state, bar_state2, bar_r_full, bar_init;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // broadcast: provably warp-uniform
  const int bh = blockIdx.x;
  const int h = bh % H, bb = bh / H;
  pdl_allow_next();
  // Segment-parallel launches (gridDim.y > 1): this CTA owns `chunks_per_seg` consecutive chunks, walks them
  // backwards, and starts from the state of everything after them (`init_state[bh][seg]`, fp32 [64 x 64],
  // rows d_k).  `ci` is local; the position of item ci is chunk `last_chunk - ci`.
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
  const long long rot_base = ROT ? static_cast<long long>(bb) * rot.batch_stride : 0;
  auto rot_sin = [&](int pos) { return rot.sin + rot_base + static_cast<long long>(pos) * (4 * rot.pieces); };
  auto rot_cos = [&](int pos) { return rot.cos + rot_base + static_cast<long long>(pos) * (4 * rot.pieces); };

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_free_in[s], 8);  // output group (accumulator MMAs done) + operand group (state MMAs done)
      mbar_init(&bar_out[s], 4);
      mbar_init(&bar_prep[s], 4);
      mbar_init(&bar_rot[s], 4);
    }
    mbar_init(&bar_p_full, 1);
    mbar_init(&bar_p_ready, 8);  // score group (E) + operand group (F)
    mbar_init(&bar_acc_full, 1);
    mbar_init(&bar_acc_free, 4);
    mbar_init(&bar_state, 4);
    mbar_init(&bar_state2, 4);
    mbar_init(&bar_r_full, 1);
    mbar_init(&bar_init, 4);
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
  pdl_wait_prior();
  const uint32_t tmem = tmem_slot;
  const uint32_t tE = tmem, tF = tmem + 128, tK = tmem + 256, tV = tmem + 320, tR = tmem + 384;

  // iteration ci handles chunk nchunks-1-ci (the sequence is walked backwards)
  // Two issuing threads (see causal_tc_kernel):
  //   warp 0, lane 0:  TMA loads, score tiles E, F of chunk ci+1, state R += Qw^T dO (ci)
  //   warp 1, lane 0:  accumulators AccK, AccV of chunk ci
  constexpr uint32_t kIdescP = make_idesc(128, 128, BF, false, false);
  constexpr uint32_t kIdescAccKK = make_idesc(128, 64, BF, false, false);  // B K-major (V R^T)
  constexpr uint32_t kIdescAccMN = make_idesc(128, 64, BF, false, true);   // B MN-major
  constexpr uint32_t kIdescR = make_idesc(64, 64, BF, true, true);
  if (warp == 14) {
    // TMA loads and stores (a thread of its own, see causal_tc_kernel).  dK and dV are staged in the K and
    // V tiles of the chunk's own stage: q and dO are refilled as soon as every MMA of the chunk has
    // completed, K and V once the output stores have read them.
    if (lane == 0) {
      auto load_inputs = [&](int ci) {
        const int s = ci % NS;
        const int y = (last_chunk - ci) * kTcChunk;
        unsigned char* st = smem + s * STAGE;
        mbar_expect_tx(&bar_full[s], STAGE);
        tma_load_tile(st, &mapQ, &bar_full[s], y, h, bb);
        tma_load_tile(st + 3 * kTileBytes, &mapDO, &bar_full[s], y, h, bb);
      };
      auto load_staging = [&](int ci) {
        const int s = ci % NS;
        const int y = (last_chunk - ci) * kTcChunk;
        unsigned char* st = smem + s * STAGE;
        tma_load_tile(st + kTileBytes, &mapK, &bar_full[s], y, h, bb);
        tma_load_tile(st + 2 * kTileBytes, &mapV, &bar_full[s], y, h, bb);
      };
      for (int ci = 0; ci < NS && ci < nchunks; ++ci) {
        load_inputs(ci);
        load_staging(ci);
      }
      for (int ci = 0; ci < nchunks; ++ci) {
        const int s = ci % NS;
        const int y = (last_chunk - ci) * kTcChunk;
        const bool refill = ci + NS < nchunks;
        if (refill) {
          if (!wait_bar(&bar_free_in[s], (ci / NS) & 1, abort_flag, kWaitStageFree, ci)) break;
          load_inputs(ci + NS);
        }
        if (!wait_bar(&bar_out[s], (ci / NS) & 1, abort_flag, kWaitStageFree, ci)) break;
        tma_store_tile(&mapDV, smem + s * STAGE + 2 * kTileBytes, y, h, bb);
        tma_store_tile(&mapDK, smem + s * STAGE + kTileBytes, y, h, bb);
        tma_store_commit();
        if (refill) {
          tma_store_wait_read<0>();
          load_staging(ci + NS);
        }
      }
      tma_store_wait<0>();
    }
  } else if (warp == 0) {
    if (lane == 0) {
      auto issue_scores = [&](int ci) {  // caller has waited for TMA(ci), Qw(ci) and for the tiles to be free
        const uint32_t q0 = smem_u32(smem + (ci % NS) * STAGE);
        const uint64_t dQ = kdesc(q0), dK = kdesc(q0 + kTileBytes), dV = kdesc(q0 + 2 * kTileBytes),
                       dD = kdesc(q0 + 3 * kTileBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tE, dV + 2 * k, dD + 2 * k, kIdescP, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(tF, dK + 2 * k, dQ + 2 * k, kIdescP, k > 0);
        mma_commit(&bar_p_full);
      };
      bool ok = wait_bar2(&bar_full[0], 0, &bar_prep[0], 0, abort_flag, kWaitTma, 0);
      if (ok) {
        tc_fence_after_sync();
        issue_scores(0);
      }
      for (int ci = 0; ok && ci + 1 < nchunks; ++ci) {
        {
          // state of chunk ci (Qw(ci) was waited for before its score tiles were issued); the 16-bit
          // conversion after chunk ci-1 must have finished reading the TMEM state
          if (ci > 0 && !(ok = wait_bar1(&bar_state2, (ci - 1) & 1, abort_flag, kWaitState, ci))) break;
          if (ci == 0 && has_init && !(ok = wait_bar1(&bar_init, 0, abort_flag, kWaitState, ci))) break;
          tc_fence_after_sync();
          const uint32_t q0 = smem_u32(smem + (ci % NS) * STAGE);
          const uint64_t dQm = mdesc(q0), dDm = mdesc(q0 + 3 * kTileBytes);
          mma_ss(tR, dQm, dDm, kIdescR, (ci > 0 || has_init) ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k) mma_ss(tR, dQm + 128 * k, dDm + 128 * k, kIdescR, 1u);
          mma_commit(&bar_r_full);
          // score tiles of chunk ci+1: single-buffered, so the accumulator MMAs of chunk ci (which read the
          // 16-bit scores from TMEM) must be complete
          const int s1 = (ci + 1) % NS;
          ok = wait_bar4(&bar_full[s1], ((ci + 1) / NS) & 1, &bar_prep[s1], ((ci + 1) / NS) & 1, &bar_acc_full, ci & 1,
                         nullptr, 0, abort_flag, kWaitTma, ci);
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores(ci + 1);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t r0 = smem_u32(sR);
      for (int ci = 0; ci < nchunks; ++ci) {
        const int s = ci % NS;
        const uint32_t q0 = smem_u32(smem + s * STAGE);
        const uint64_t dK = kdesc(q0 + kTileBytes), dV = kdesc(q0 + 2 * kTileBytes), dQm = mdesc(q0),
                       dDm = mdesc(q0 + 3 * kTileBytes);
        const uint32_t acc0 = (ci > 0 || has_init) ? 1u : 0u;
        if (ci > 0 || has_init) {
          // the state terms need the 16-bit state after chunk ci-1 and the accumulators read out, not the
          // masked scores: they are issued while the score tiles are still being masked
          // (rotary in the kernel: they read the rotated K tile, which the score group reports with Qw)
          if (ci > 0 ? !wait_bar4(&bar_state, (ci - 1) & 1, &bar_acc_free, (ci - 1) & 1, ROT ? &bar_prep[s] : nullptr,
                                  (ci / NS) & 1, nullptr, 0, abort_flag, kWaitState, ci)
                     : !wait_bar1(&bar_init, 0, abort_flag, kWaitState, ci))
            break;
          tc_fence_after_sync();
          const uint32_t rb = r0 + (ci & 1) * (kTcD * 128);
          const uint64_t dRk = kdesc(rb), dRm = mdesc(rb);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // AccK = V R^T : B[n = d_k][k = d_v] = R, K-major
            mma_ss(tK, dV + 2 * k, dRk + 2 * k, kIdescAccKK, k > 0);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // AccV = K R : B[n = d_v][k = d_k] = R, MN-major
            mma_ss(tV, dK + 2 * k, dRm + 128 * k, kIdescAccMN, k > 0);
        }
        // masked scores of chunk ci (which implies Qw(ci))
        if (!wait_bar1(&bar_p_ready, ci & 1, abort_flag, kWaitScoreReady, ci)) break;
        tc_fence_after_sync();
        mma_ts(tK, tE, dQm, kIdescAccMN, acc0);
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ts(tK, tE + 8 * k, dQm + 128 * k, kIdescAccMN, 1u);
        mma_ts(tV, tF, dDm, kIdescAccMN, acc0);
#pragma unroll
        for (int k = 1; k < 8; ++k) mma_ts(tV, tF + 8 * k, dDm + 128 * k, kIdescAccMN, 1u);
        mma_commit(&bar_acc_full);
      }
    }
  } else if (warp < 6) {
    // score group: mask + convert E, then Qw = q^ of the next chunk in place
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    auto prepare = [&](int ci) -> bool {
      const int s = ci % NS;
      if (!wait_bar_warp(&bar_full[s], (ci / NS) & 1, abort_flag, kWaitTma, ci)) return false;
      // (rotary in the kernel: the rotated Q tile)
      if (ROT && !wait_bar_warp(&bar_rot[s], (ci / NS) & 1, abort_flag, kWaitTma, ci)) return false;
      unsigned char* sQ = smem + s * STAGE;
      scale_row_rolled<T>(sQ, row, row_mask(keep_b, count_b, (last_chunk - ci) * kTcChunk + row, N).kp
                                       ? inv_norm(row_sumsq_rolled<T>(sQ, row))
                                       : 0.f);
      fence_proxy_async_smem();
      warp_arrive(&bar_prep[s], lane);
      return true;
    };
    bool ok = prepare(0);
    for (int ci = 0; ok && ci < nchunks; ++ci) {
      if (!(ok = wait_bar_warp(&bar_p_full, ci & 1, abort_flag, kWaitScore, ci))) break;
      tc_fence_after_sync();
      mask_pack_inplace<T, false>(tE + lane_base, lane, wq);
      tc_fence_before_sync();
      warp_arrive(&bar_p_ready, lane);
      // Qw of the next chunk, while the accumulator MMAs of this one run
      if (ci + 1 < nchunks && !(ok = prepare(ci + 1))) break;
    }
  } else if (ROT && warp >= 15) {
    // rotary group: the Q and K tiles of every stage, as soon as it has arrived
    const int wq = warp & 3;
    for (int ci = 0; ci < nchunks; ++ci) {
      const int s = ci % NS;
      const int wrow0 = (last_chunk - ci) * kTcChunk + 32 * wq;
      RotRegs rt;
      rot_load(rt, rot_sin(wrow0), rot_cos(wrow0), lane, 0, rot.pieces, N - wrow0);
      if (!wait_bar_warp(&bar_full[s], (ci / NS) & 1, abort_flag, kWaitTma, ci)) break;
      unsigned char* sQ = smem + s * STAGE;
      rotate_rows<T, false, 2>(rt, sQ, sQ + kTileBytes, 32 * wq, lane, rot_sin(wrow0), rot_cos(wrow0), rot.pieces, N - wrow0);
      fence_proxy_async_smem();
      warp_arrive(&bar_rot[s], lane);
    }
  } else if (warp >= 10) {
    // operand group: mask + convert F, then the fp32 state after this chunk -> 16-bit operand
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    if (has_init) {  // the state after this segment: fp32 into TMEM, 16-bit into the operand buffer of item 0
      load_init_state<T>(init_state + (static_cast<size_t>(bh) * gridDim.y + seg) * (kTcD * kTcD), tR + lane_base, sR, wq, lane);
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      warp_arrive(&bar_init, lane);
    }
    for (int ci = 0; ci < nchunks; ++ci) {
      if (!wait_bar_warp(&bar_p_full, ci & 1, abort_flag, kWaitScore, ci)) break;
      tc_fence_after_sync();
      mask_pack_inplace<T, false>(tF + lane_base, lane, wq);
      tc_fence_before_sync();
      warp_arrive(&bar_p_ready, lane);
      if (ci + 1 < nchunks) {  // R after chunk ci -> 16-bit operand of chunk ci+1 (buffer (ci+1)&1)
        if (!wait_bar_warp(&bar_r_full, ci & 1, abort_flag, kWaitState, ci)) break;
        tc_fence_after_sync();
        if (lane == 0) mbar_arrive(&bar_free_in[ci % NS]);  // the state MMAs of chunk ci have read its tiles
        state_to_smem_rolled<T>(tR + lane_base, sR + ((ci + 1) & 1) * (kTcD * 128), wq, lane);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        warp_arrive(&bar_state, lane);
        if (lane == 0) mbar_arrive(&bar_state2);
      }
    }
  } else {
    // output group
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
    const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
    float gsum = 0.f;  // sum_s ln(n_s) eps_s over this thread's rows
    for (int ci = 0; ci < nchunks; ++ci) {
      const int s = ci % NS;
      unsigned char* sK = smem + s * STAGE + kTileBytes;
      unsigned char* sV = smem + s * STAGE + 2 * kTileBytes;
      const int pos = (last_chunk - ci) * kTcChunk + row;
      if (!wait_bar_warp(&bar_full[s], (ci / NS) & 1, abort_flag, kWaitTma, ci)) break;
      const RowMask m = row_mask(keep_b, count_b, pos, N);
      // (rotary in the kernel: the K tile is rotated by the score group, so the norm is taken once the MMAs, which
      // wait for that group, have completed -- the value never depends on which group was faster)
      float rk = 0.f;
      if (!ROT) rk = m.kp ? inv_norm(row_sumsq_rolled<T>(sK, row)) : 0.f;
      const float a = length_factor(m.n, sigma);
      if (!wait_bar_warp(&bar_acc_full, ci & 1, abort_flag, kWaitAcc, ci)) break;
      tc_fence_after_sync();
      if (ROT) rk = m.kp ? inv_norm(row_sumsq_rolled<T>(sK, row)) : 0.f;
      RotRegs rt;  // (rotary: the table values for the way back, loaded while the accumulator rows are written)
      if (ROT) rot_load(rt, rot_sin(pos - lane), rot_cos(pos - lane), lane, 0, rot.pieces, N - (pos - lane));
      // dV first (its row product with v gives eps), then dK; each is staged as soon as it is ready, in
      // the V / K tile of this stage: every MMA that reads them completed before acc_full and this thread
      // is done with its own rows, so they have no reader left.  The TMA thread stores and refills them.
      if (lane == 0) mbar_arrive(&bar_free_in[s]);  // (warp-converged: follows wait_bar_warp) q, dO tiles are free
      const float c1 = rk * a;
      // dv = a dv' = c1 raw;  eps = v' . dv' = c1 (v . raw)
      const float eps = c1 * row_from_acc_dot<T>(sV, row, tV + lane_base, c1);
      // dk = rk (dk^ - k^ (k^ . dk^)) with dk^ = a raw, k^ . dk^ = v' . dv' = eps and k^ = rk k
      row_from_acc<T, true>(sK, row, tK + lane_base, c1, -rk * rk * eps);
      tc_fence_before_sync();
      warp_arrive(&bar_acc_free, lane);
      // the row is the gradient of the rotated k: back through the rotation
      if (ROT) {
        const int wrow0 = pos - lane;  // position of the warp's first row
        __syncwarp();  // the rows are now rotated piece-per-lane
        rotate_rows<T, true, 1>(rt, sK, sK, 32 * wq, lane, rot_sin(wrow0), rot_cos(wrow0), rot.pieces, N - wrow0);
      }
      ptx::fence_proxy_async_smem();
      warp_arrive(&bar_out[s], lane);
      if (m.n > 1.0f && pos < N) gsum += logf(m.n) * eps;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) gsum += __shfl_down_sync(0xffffffffu, gsum, off);
    if (lane == 0) atomicAdd(dnorm + h, -sigma * (1.0f - sigma) * gsum);
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag) {
    for (int ci = (nchunks > NS ? nchunks - NS : 0); ci < nchunks; ++ci)
      mbar_wait(&bar_full[ci % NS], (ci / NS) & 1, 64);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

inline size_t causal_bwd_kv_smem_bytes() {
  return static_cast<size_t>(kTcStages * 4 * kTileBytes + 2 * kTcD * 128 + 1024);
}

inline size_t causal_tc_smem_bytes(int mode) {
  const int nin = mode == kModeDq ? 3 : 2;
  const int ns = mode == kModeDq ? kTcStages : kTcStagesFwd;
  return static_cast<size_t>((ns * nin + ns + 1) * kTileBytes + 2 * kTcD * 128 + 1024);
}

}  // namespace cott
