// Recurrent decode step of cosine attention (HBM-bound, CUDA cores).
//
// Per (batch, head) the reference keeps a d_v x d_k state and, per generated token
// (GPT_Trainer/GPTCosAttention.py:229-230,236,253-272):
//     q^ = q/|q|,  k^ = k/|k|,  v' = v / max(pos^sigmoid(c_h), 1)          pos = 1-based position
//     state[j][i] += v'[j] * k^[i]                                          (:264, layout [d_v, d_k])
//     out[j]       = sum_i q^[i] * state[j][i]                              (:267)
// The reference runs this on the CPU in float64 for batch 1; here the state is fp32 in HBM,
// [B, H, d_v, d_k], updated in place.  One CTA per (b,h); a row of the state is spread over
// d_k/4 lanes that each own one float4, so every state access is a coalesced 128-bit access and
// the row dot product is a shuffle reduction.
//
// cott_decode_steps runs T consecutive positions in one launch with the state held in registers
// between steps (it is read from and written to HBM once), which is also how a prompt is absorbed.
#pragma once

#include "common.cuh"

namespace cott {

// Threads per CTA: 128 for d <= 64 (8 CTAs per SM: the 1024 (b,h) states of a batch-64, 16-head step are then
// resident in one wave of 148 x 8 CTAs, and twice the bytes are in flight per SM), 256 for d = 128.
template <int DK> struct DecodeCfg { static constexpr int kThreads = DK <= 64 ? 128 : 256, kCtasPerSm = DK <= 64 ? 8 : 2; };

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p) { return to_acc(*p); }

// q, k: [B,H,T,Dk]  v, out: [B,H,T,Dv] (T = 1 for a single step); state: [B,H,Dv,Dk] fp32.
// positions: optional [B] int64 array of the 1-based position of the FIRST token of this call for
// each batch entry; if null, `pos0` is used for all.  LPR = lanes per state row = Dk/4.
// (the kernel is latency-bound on its state loads, so resident CTAs are what hides the HBM latency)
template <typename T, int DK, int MAX_DV>
__global__ void __launch_bounds__(DecodeCfg<DK>::kThreads, DecodeCfg<DK>::kCtasPerSm)
decode_kernel(float* __restrict__ state, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
              const float* __restrict__ norm_const, T* __restrict__ out, int H, int Dv, int Tsteps, long long pos0,
              const long long* __restrict__ positions) {
  constexpr int kDecodeThreads = DecodeCfg<DK>::kThreads;
  constexpr int LPR = DK / 4;                    // lanes per row (4, 8, 16 or 32)
  constexpr int ROWS_PER_PASS = kDecodeThreads / LPR;
  constexpr int MAXR = (MAX_DV + ROWS_PER_PASS - 1) / ROWS_PER_PASS;  // state rows held per thread
  __shared__ float sq[DK], sk[DK], sv[MAX_DV];
  __shared__ float red[2][kDecodeThreads / 32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long bh = blockIdx.x;
  const int b = static_cast<int>(bh / H), h = static_cast<int>(bh % H);
  // Programmatic dependent launch: a token-by-token loop is a chain of these launches, each waiting for the state the
  // one before wrote.  The launch is allowed to begin while its predecessor in the stream is still draining (its CTAs
  // are placed as slots free up, instead of after the whole grid has retired and a launch gap has passed); nothing
  // that another kernel may have produced -- state, q, k, v, norm_const -- is read before the wait below.
  pdl_allow_next();
  pdl_wait_prior();
  const float sigma = 1.0f / (1.0f + __expf(-norm_const[h]));
  const long long p0 = positions ? positions[b] : pos0;
  const int piece = tid % LPR;        // which float4 of the row
  const int row0 = tid / LPR;         // first row of this thread; then += ROWS_PER_PASS

  float* st = state + bh * static_cast<long>(Dv) * DK;
  float4 s[MAXR];
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int j = row0 + r * ROWS_PER_PASS;
    s[r] = (j < Dv) ? *reinterpret_cast<const float4*>(st + static_cast<long>(j) * DK + 4 * piece)
                    : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  for (int t = 0; t < Tsteps; ++t) {
    const T* qt = q + (bh * Tsteps + t) * static_cast<long>(DK);
    const T* kt = k + (bh * Tsteps + t) * static_cast<long>(DK);
    const T* vt = v + (bh * Tsteps + t) * static_cast<long>(Dv);
    // stage q, k, v and their norms
    float x = 0.f, y = 0.f;
    if (tid < DK) {
      x = ld_as_float(qt + tid);
      y = ld_as_float(kt + tid);
      sq[tid] = x;
      sk[tid] = y;
    }
    if (tid < Dv) sv[tid] = ld_as_float(vt + tid);
    float xx = x * x, yy = y * y;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      xx += __shfl_xor_sync(0xffffffffu, xx, off);
      yy += __shfl_xor_sync(0xffffffffu, yy, off);
    }
    if (lane == 0) {
      red[0][warp] = xx;
      red[1][warp] = yy;
    }
    __syncthreads();
    float nq = 0.f, nk = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeThreads / 32; ++w) {
      nq += red[0][w];
      nk += red[1][w];
    }
    const float rq = 1.0f / fmaxf(sqrtf(nq), 1e-12f);
    const float rk = 1.0f / fmaxf(sqrtf(nk), 1e-12f);
    const float a = 1.0f / fmaxf(exp2f(sigma * log2f(static_cast<float>(p0 + t))), 1.0f);
    const float4 k4 = *reinterpret_cast<const float4*>(sk + 4 * piece);
    const float4 q4 = *reinterpret_cast<const float4*>(sq + 4 * piece);
    const float ws = rk * a;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      const int j = row0 + r * ROWS_PER_PASS;
      const bool valid = j < Dv;  // the same for all LPR lanes of a row; rows of one warp may differ
      const float vj = valid ? sv[j] * ws : 0.f;
      s[r].x += vj * k4.x;
      s[r].y += vj * k4.y;
      s[r].z += vj * k4.z;
      s[r].w += vj * k4.w;
      float dot = q4.x * s[r].x + q4.y * s[r].y + q4.z * s[r].z + q4.w * s[r].w;
#pragma unroll
      for (int off = LPR / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off, LPR);
      if (valid && piece == 0) out[(bh * Tsteps + t) * static_cast<long>(Dv) + j] = from_acc<T>(dot * rq);
    }
    __syncthreads();  // sq/sk/sv/red are rewritten by the next step
  }

#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int j = row0 + r * ROWS_PER_PASS;
    if (j < Dv) *reinterpret_cast<float4*>(st + static_cast<long>(j) * DK + 4 * piece) = s[r];
  }
}

template <typename T>
int launch_decode(float* state, const void* q, const void* k, const void* v, const float* nc, void* out, int B, int H,
                  int Dk, int Dv, int T_steps, long long pos0, const long long* positions, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>(static_cast<long>(B) * H);
#define COTT_DECODE_CASE(DK)                                                                                     \
  case DK:                                                                                                       \
    if (Dv <= 64)                                                                                                \
      COTT_CUDA_TRY(launch_pdl(decode_kernel<T, DK, 64>, dim3(grid), DecodeCfg<DK>::kThreads, 0, stream, state,           \
                               static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), nc, \
                               static_cast<T*>(out), H, Dv, T_steps, pos0, positions));                          \
    else                                                                                                         \
      COTT_CUDA_TRY(launch_pdl(decode_kernel<T, DK, 128>, dim3(grid), DecodeCfg<DK>::kThreads, 0, stream, state,          \
                               static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), nc, \
                               static_cast<T*>(out), H, Dv, T_steps, pos0, positions));                          \
    break;
  switch (Dk) {
    COTT_DECODE_CASE(16)
    COTT_DECODE_CASE(32)
    COTT_DECODE_CASE(64)
    COTT_DECODE_CASE(128)
    default: return fail(COTT_ERR_SHAPE, "decode supports D_attn in {16, 32, 64, 128} (got %d)", Dk);
  }
#undef COTT_DECODE_CASE
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

}  // namespace cott
