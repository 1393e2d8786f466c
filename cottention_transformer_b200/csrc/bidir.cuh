// Bidirectional (encoder) cosine attention: out = q^ (k^T v'), BERT_Trainer/BertCosAttention.py:162-178,249.
//
//   keep_s = un-masked position, L_b = number of un-masked positions of batch entry b      (:162-166,178)
//   q^ = keep q/|q|,  k^ = keep k/|k|,  v' = keep v / max(L_b^sigmoid(c_h), 1)             (:170-178)
//   S  = sum_s k^_s (x) v'_s      [Dk x Dv] per (b,h)                                       (:249, inner einsum)
//   out_t = q^_t S                                                                          (:249, outer einsum)
// The reference runs two torch.einsum (cuBLAS) calls plus elementwise kernels; here it is two
// kernels with everything elementwise fused:
//   1. bidir_state_kernel: S partials per (b,h,split) -> SCRATCH [B*H, nsplit, Dk, Dv] (accumulator type)
//   2. bidir_apply_kernel: sums the partials, out_t = q^_t S
// and for the backward
//   3. bidir_state_kernel again with (x, y) = (q, dO): dS = sum_t q^_t (x) dO_t -> SCRATCH
//   4. bidir_bwd_kernel:  dq^_t = dO_t S^T,  dk^_s = v'_s dS^T,  dv'_s = k^_s dS, then the
//      gradients of the normalisations and of the length-norm parameter.
// CUDA-core kernels with fp32 (fp64 for double) accumulation; sizes are small (BERT: N=512, d=64).
#pragma once

#include "common.cuh"

namespace cott {

constexpr int kBidirThreads = 256;
constexpr int kBidirTile = 32;  // tokens staged per iteration

template <typename A>
__device__ __forceinline__ A block_sum(A x, A* red /* [8] */) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  A s = 0;
#pragma unroll
  for (int w = 0; w < kBidirThreads / 32; ++w) s += red[w];
  return s;
}

// L_b and the length factor a = 1 / max(L^sigma, 1); also returns ln(L) gate for the gradient.
template <typename A>
__device__ __forceinline__ A bidir_length_factor(const unsigned char* keep_b, int N, float nc_h, A* red, A* logL) {
  A cnt = 0;
  if (keep_b) {
    for (int s = threadIdx.x; s < N; s += kBidirThreads) cnt += keep_b[s] ? A(1) : A(0);
    cnt = block_sum<A>(cnt, red);
  } else {
    cnt = A(N);
  }
  const A sigma = A(1) / (A(1) + exp(-A(nc_h)));
  const A p = pow(cnt, sigma);  // pow(0, sigma) = 0 -> clamped to 1
  *logL = (p > A(1)) ? log(cnt) : A(0);
  return A(1) / (p > A(1) ? p : A(1));
}

// S_partial[bh][split] = sum_{s in split} wx_s x_s (x) y_s with wx_s = keep_s / |x_s| * (scale_by_length ? a : 1).
// Thread (ty, tx) of a 16x16 grid owns S[i][j] for i = ty + 16 a, j = tx + 16 b.
template <typename T>
__global__ void __launch_bounds__(kBidirThreads)
bidir_state_kernel(const T* __restrict__ X, const T* __restrict__ Y, const unsigned char* __restrict__ keep,
                   const float* __restrict__ norm_const, typename AccOf<T>::type* __restrict__ scratch, int H, int N,
                   int Dk, int Dv, int nsplit, int scale_by_length) {
  using A = typename AccOf<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* sx = reinterpret_cast<A*>(smem_raw);       // [32][Dk+1]
  A* sy = sx + kBidirTile * (Dk + 1);           // [32][Dv+1]
  __shared__ A red[kBidirThreads / 32];
  __shared__ A sw[kBidirTile];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16, lane = tid & 31, warp = tid >> 5;
  const long bh = blockIdx.x;
  const int b = static_cast<int>(bh / H), h = static_cast<int>(bh % H), split = blockIdx.y;
  const unsigned char* keep_b = keep ? keep + static_cast<long>(b) * N : nullptr;
  A logL;
  const A a = scale_by_length ? bidir_length_factor<A>(keep_b, N, norm_const[h], red, &logL) : A(1);
  const int per = (N + nsplit - 1) / nsplit;
  const int s_begin = split * per, s_end = min(N, s_begin + per);
  const T* x = X + bh * static_cast<long>(N) * Dk;
  const T* y = Y + bh * static_cast<long>(N) * Dv;
  const int ti = Dk / 16, tj = Dv / 16;
  A acc[8][8];
#pragma unroll
  for (int p = 0; p < 8; ++p)
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[p][r] = A(0);

  for (int s0 = s_begin; s0 < s_end; s0 += kBidirTile) {
    __syncthreads();
    for (int idx = tid; idx < kBidirTile * Dk; idx += kBidirThreads) {
      const int r = idx / Dk, i = idx - r * Dk, s = s0 + r;
      sx[r * (Dk + 1) + i] = (s < s_end) ? to_acc(x[static_cast<long>(s) * Dk + i]) : A(0);
    }
    for (int idx = tid; idx < kBidirTile * Dv; idx += kBidirThreads) {
      const int r = idx / Dv, j = idx - r * Dv, s = s0 + r;
      sy[r * (Dv + 1) + j] = (s < s_end) ? to_acc(y[static_cast<long>(s) * Dv + j]) : A(0);
    }
    __syncthreads();
    // row weights: each warp handles 4 rows
    for (int r = warp; r < kBidirTile; r += kBidirThreads / 32) {
      A ss = 0;
      for (int i = lane; i < Dk; i += 32) ss += sx[r * (Dk + 1) + i] * sx[r * (Dk + 1) + i];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      if (lane == 0) {
        const int s = s0 + r;
        const bool kp = s < s_end && (!keep_b || keep_b[s]);
        const A nrm = sqrt(ss);
        sw[r] = kp ? a / (nrm > A(1e-12) ? nrm : A(1e-12)) : A(0);
      }
    }
    __syncthreads();
    for (int r = 0; r < kBidirTile; ++r) {
      const A w = sw[r];
      A xv[8], yv[8];
#pragma unroll
      for (int p = 0; p < 8; ++p) xv[p] = (p < ti) ? w * sx[r * (Dk + 1) + ty + 16 * p] : A(0);
#pragma unroll
      for (int q = 0; q < 8; ++q) yv[q] = (q < tj) ? sy[r * (Dv + 1) + tx + 16 * q] : A(0);
#pragma unroll
      for (int p = 0; p < 8; ++p)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[p][q] += xv[p] * yv[q];
    }
  }
  A* out = scratch + (bh * nsplit + split) * static_cast<long>(Dk) * Dv;
#pragma unroll
  for (int p = 0; p < 8; ++p)
#pragma unroll
    for (int q = 0; q < 8; ++q)
      if (p < ti && q < tj) out[static_cast<long>(ty + 16 * p) * Dv + tx + 16 * q] = acc[p][q];
}

// Loads sum over splits of a [Dk x Dv] state into shared memory (row stride Dv+1).
template <typename A>
__device__ __forceinline__ void load_state_sum(A* dst, const A* scratch_bh, int nsplit, int Dk, int Dv) {
  for (int idx = threadIdx.x; idx < Dk * Dv; idx += kBidirThreads) {
    A s = 0;
    for (int p = 0; p < nsplit; ++p) s += scratch_bh[static_cast<long>(p) * Dk * Dv + idx];
    dst[(idx / Dv) * (Dv + 1) + idx % Dv] = s;
  }
}

// out_t = keep_t / |q_t| * (q_t S).  Grid (B*H, ceil(N/32)); thread (ty, tx): rows ty + 16 a (a<2), columns tx + 16 b.
template <typename T>
__global__ void __launch_bounds__(kBidirThreads)
bidir_apply_kernel(const T* __restrict__ Q, const unsigned char* __restrict__ keep,
                   const typename AccOf<T>::type* __restrict__ scratch, T* __restrict__ O, int H, int N, int Dk,
                   int Dv, int nsplit) {
  using A = typename AccOf<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* sS = reinterpret_cast<A*>(smem_raw);       // [Dk][Dv+1]
  A* sq = sS + Dk * (Dv + 1);                   // [32][Dk+1]
  __shared__ A sw[kBidirTile];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16, lane = tid & 31, warp = tid >> 5;
  const long bh = blockIdx.x;
  const int b = static_cast<int>(bh / H);
  const int t0 = blockIdx.y * kBidirTile;
  const unsigned char* keep_b = keep ? keep + static_cast<long>(b) * N : nullptr;
  load_state_sum<A>(sS, scratch + bh * nsplit * static_cast<long>(Dk) * Dv, nsplit, Dk, Dv);
  const T* q = Q + bh * static_cast<long>(N) * Dk;
  for (int idx = tid; idx < kBidirTile * Dk; idx += kBidirThreads) {
    const int r = idx / Dk, i = idx - r * Dk, t = t0 + r;
    sq[r * (Dk + 1) + i] = (t < N) ? to_acc(q[static_cast<long>(t) * Dk + i]) : A(0);
  }
  __syncthreads();
  for (int r = warp; r < kBidirTile; r += kBidirThreads / 32) {
    A ss = 0;
    for (int i = lane; i < Dk; i += 32) ss += sq[r * (Dk + 1) + i] * sq[r * (Dk + 1) + i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) {
      const int t = t0 + r;
      const bool kp = t < N && (!keep_b || keep_b[t]);
      const A nrm = sqrt(ss);
      sw[r] = kp ? A(1) / (nrm > A(1e-12) ? nrm : A(1e-12)) : A(0);
    }
  }
  __syncthreads();
  const int tj = Dv / 16;
  A acc[2][8];
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[p][r] = A(0);
  for (int i = 0; i < Dk; ++i) {
    const A q0 = sq[ty * (Dk + 1) + i], q1 = sq[(ty + 16) * (Dk + 1) + i];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < tj) {
        const A sv = sS[i * (Dv + 1) + tx + 16 * r];
        acc[0][r] += q0 * sv;
        acc[1][r] += q1 * sv;
      }
    }
  }
  T* o = O + bh * static_cast<long>(N) * Dv;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int t = t0 + ty + 16 * p;
    if (t < N) {
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < tj) o[static_cast<long>(t) * Dv + tx + 16 * r] = from_acc<T>(acc[p][r] * sw[ty + 16 * p]);
    }
  }
}

// Backward per token tile (32 tokens): with S (forward state) and dS = sum q^ (x) dO:
//   dq^ = dO S^T           dq = keep/|q| (dq^ - q^ (q^.dq^))
//   dk^ = a keep (v dS^T)  dk = 1/|k| (dk^ - k^ (k^.dk^))
//   dv' = k^ dS            dv = a keep dv'
//   dnorm_const[h] += -sigma(1-sigma) ln(L) sum_s v'_s . dv'_s      (only when L^sigma > 1)
// One warp per token row at a time (8 warps, 4 rows each); lanes stride over the feature dims.
template <typename T>
__global__ void __launch_bounds__(kBidirThreads)
bidir_bwd_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V, const T* __restrict__ dO,
                 const unsigned char* __restrict__ keep, const float* __restrict__ norm_const,
                 const typename AccOf<T>::type* __restrict__ scratch_S,
                 const typename AccOf<T>::type* __restrict__ scratch_dS, T* __restrict__ dQ, T* __restrict__ dK,
                 T* __restrict__ dV, float* __restrict__ dnorm, int H, int N, int Dk, int Dv, int nsplit) {
  using A = typename AccOf<T>::type;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  A* sS = reinterpret_cast<A*>(smem_raw);    // [Dk][Dv+1]
  A* sdS = sS + Dk * (Dv + 1);               // [Dk][Dv+1]
  A* srow = sdS + Dk * (Dv + 1);             // per warp: q[Dk] k[Dk] v[Dv] do[Dv] dk^[Dk]
  __shared__ A red[kBidirThreads / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long bh = blockIdx.x;
  const int b = static_cast<int>(bh / H), h = static_cast<int>(bh % H);
  const int t0 = blockIdx.y * kBidirTile;
  const unsigned char* keep_b = keep ? keep + static_cast<long>(b) * N : nullptr;
  A logL;
  const A a = bidir_length_factor<A>(keep_b, N, norm_const[h], red, &logL);
  load_state_sum<A>(sS, scratch_S + bh * nsplit * static_cast<long>(Dk) * Dv, nsplit, Dk, Dv);
  load_state_sum<A>(sdS, scratch_dS + bh * nsplit * static_cast<long>(Dk) * Dv, nsplit, Dk, Dv);
  __syncthreads();
  const int rowlen = 3 * Dk + 2 * Dv;
  A* wq = srow + warp * rowlen;
  A* wk = wq + Dk;
  A* wv = wk + Dk;
  A* wdo = wv + Dv;
  A* wdk = wdo + Dv;
  A gsum = 0;
  for (int r = warp; r < kBidirTile; r += kBidirThreads / 32) {
    const int t = t0 + r;
    if (t >= N) break;  // warp-uniform
    const bool kp = !keep_b || keep_b[t];
    const long base_k = (bh * N + t) * static_cast<long>(Dk), base_v = (bh * N + t) * static_cast<long>(Dv);
    A ssq = 0, ssk = 0;
    for (int i = lane; i < Dk; i += 32) {
      const A qv = to_acc(Q[base_k + i]), kv = to_acc(K[base_k + i]);
      wq[i] = qv;
      wk[i] = kv;
      ssq += qv * qv;
      ssk += kv * kv;
    }
    for (int j = lane; j < Dv; j += 32) {
      wv[j] = to_acc(V[base_v + j]);
      wdo[j] = to_acc(dO[base_v + j]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      ssq += __shfl_xor_sync(0xffffffffu, ssq, off);
      ssk += __shfl_xor_sync(0xffffffffu, ssk, off);
    }
    __syncwarp();
    const A nq = sqrt(ssq), nk = sqrt(ssk);
    const A rq = kp ? A(1) / (nq > A(1e-12) ? nq : A(1e-12)) : A(0);
    const A rk = kp ? A(1) / (nk > A(1e-12) ? nk : A(1e-12)) : A(0);
    const A av = kp ? a : A(0);
    // dq^[i] = sum_j dO[j] S[i][j];  dk^[i] = a sum_j v[j] dS[i][j]
    A dotq = 0, dotk = 0;
    for (int i = lane; i < Dk; i += 32) {
      A dqh = 0, dkh = 0;
      for (int j = 0; j < Dv; ++j) {
        dqh += wdo[j] * sS[i * (Dv + 1) + j];
        dkh += wv[j] * sdS[i * (Dv + 1) + j];
      }
      dkh *= av;
      wdk[i] = dkh;
      dotq += (rq * wq[i]) * dqh;
      dotk += (rk * wk[i]) * dkh;
      // stash dq^ in registers is impossible across the loop: recompute after the reduction instead
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      dotq += __shfl_xor_sync(0xffffffffu, dotq, off);
      dotk += __shfl_xor_sync(0xffffffffu, dotk, off);
    }
    __syncwarp();
    for (int i = lane; i < Dk; i += 32) {
      A dqh = 0;
      for (int j = 0; j < Dv; ++j) dqh += wdo[j] * sS[i * (Dv + 1) + j];
      const A qh = rq * wq[i], kh = rk * wk[i];
      dQ[base_k + i] = from_acc<T>(rq * (dqh - qh * dotq));
      dK[base_k + i] = from_acc<T>(rk * (wdk[i] - kh * dotk));
    }
    // dv'[j] = sum_i k^[i] dS[i][j];  dv = a keep dv';  eps = v' . dv'
    A eps = 0;
    for (int j = lane; j < Dv; j += 32) {
      A dvp = 0;
      for (int i = 0; i < Dk; ++i) dvp += (rk * wk[i]) * sdS[i * (Dv + 1) + j];
      dV[base_v + j] = from_acc<T>(av * dvp);
      eps += (av * wv[j]) * dvp;
    }
    gsum += eps;
    __syncwarp();
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) gsum += __shfl_xor_sync(0xffffffffu, gsum, off);
  if (lane == 0 && gsum != A(0)) {
    const A sigma = A(1) / (A(1) + exp(-A(norm_const[h])));
    atomicAdd(dnorm + h, static_cast<float>(-sigma * (A(1) - sigma) * logL * gsum));
  }
}

template <typename A>
inline size_t bidir_state_smem(int Dk, int Dv) { return sizeof(A) * kBidirTile * (size_t)(Dk + 1 + Dv + 1); }
template <typename A>
inline size_t bidir_apply_smem(int Dk, int Dv) { return sizeof(A) * ((size_t)Dk * (Dv + 1) + kBidirTile * (Dk + 1)); }
template <typename A>
inline size_t bidir_bwd_smem(int Dk, int Dv) {
  return sizeof(A) * (2 * (size_t)Dk * (Dv + 1) + (kBidirThreads / 32) * (size_t)(3 * Dk + 2 * Dv));
}

// number of sequence splits of the state kernels: enough CTAs to fill the GPU, at most 8
inline int bidir_nsplit(long BH, int N) {
  int ns = static_cast<int>((2 * 148 + BH - 1) / (BH > 0 ? BH : 1));
  const int max_by_len = (N + 4 * kBidirTile - 1) / (4 * kBidirTile);
  if (ns > max_by_len) ns = max_by_len;
  if (ns > 8) ns = 8;
  if (ns < 1) ns = 1;
  return ns;
}

}  // namespace cott
