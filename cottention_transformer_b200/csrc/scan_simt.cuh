// Exact-mode scan: chunked cosine-linear-attention scan on CUDA cores.
//
// Computes what the reference's kernel_mod_2/kernel_mod_4
// (Cuda_Kernel/combined_kernel_general.cu:96-251) compute,
//   out[s, j] = sum_i Q[s, i] * sum_{t<=s} K[t, i] V[t, j]        (t >= s when reversed)
// but in chunked form: the sequence is cut into chunks of C positions; inside a chunk the
// masked product (Q K^T) V is formed directly, everything older is carried in a
// Dk x 16 slice of the state S = sum K (x) V that lives in shared memory.  Sums are kept
// in fp32 (fp64 for double inputs) whatever the storage type -- the reference keeps them
// in the storage type (:121,133).
//
// One CTA per (batch*head, 16-column slice of Dv); the slices of the state are independent,
// exactly as the reference's one-block-per-output-column decomposition (:104-106).
// This is the fp32/fp64 correctness path; the bf16/fp16 fast path is the tcgen05 kernel.
#pragma once

#include "common.cuh"

namespace cott {

constexpr int kSimtThreads = 256;
constexpr int kSimtDvTile = 16;

template <typename A>
inline size_t scan_simt_smem_bytes(int C, int Dk) {
  return sizeof(A) * ((size_t)2 * C * (Dk + 1) + (size_t)C * (C + 1) + (size_t)C * kSimtDvTile +
                      (size_t)Dk * kSimtDvTile);
}

template <typename T, int C>
__global__ void __launch_bounds__(kSimtThreads)
scan_simt_kernel(const T* Q, const T* K, const T* V, T* O, int N, int Dk, int Dv, int reversed) {
  using A = typename AccOf<T>::type;
  constexpr int DVT = kSimtDvTile;
  constexpr int R = C / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ldk = Dk + 1;
  A* sQ = reinterpret_cast<A*>(smem_raw);  // [C][Dk+1]
  A* sK = sQ + (size_t)C * ldk;            // [C][Dk+1]
  A* sP = sK + (size_t)C * ldk;            // [C][C+1]
  A* sV = sP + (size_t)C * (C + 1);        // [C][16]
  A* sS = sV + (size_t)C * DVT;            // [Dk][16]

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const long bh = blockIdx.x;
  const int j0 = blockIdx.y * DVT;
  const T* q = Q + bh * (long)N * Dk;
  const T* k = K + bh * (long)N * Dk;
  const T* v = V + bh * (long)N * Dv;
  T* o = O + bh * (long)N * Dv;

  for (int idx = tid; idx < Dk * DVT; idx += kSimtThreads) sS[idx] = A(0);

  for (int c0 = 0; c0 < N; c0 += C) {
    // Stage the chunk.  Row r holds logical position p = c0 + r of the scan order;
    // physical row s = p (forward) or N-1-p (reversed).  Rows past the end are zero.
    for (int idx = tid; idx < C * Dk; idx += kSimtThreads) {
      const int r = idx / Dk, i = idx - r * Dk;
      const int p = c0 + r;
      A qv = A(0), kv = A(0);
      if (p < N) {
        const long s = reversed ? (long)(N - 1 - p) : (long)p;
        qv = to_acc(q[s * Dk + i]);
        kv = to_acc(k[s * Dk + i]);
      }
      sQ[r * ldk + i] = qv;
      sK[r * ldk + i] = kv;
    }
    for (int idx = tid; idx < C * DVT; idx += kSimtThreads) {
      const int r = idx / DVT, j = idx - r * DVT;
      const int p = c0 + r;
      A vv = A(0);
      if (p < N && j0 + j < Dv) {
        const long s = reversed ? (long)(N - 1 - p) : (long)p;
        vv = to_acc(v[s * Dv + j0 + j]);
      }
      sV[idx] = vv;
    }
    __syncthreads();

    // P[t][s] = Q_t . K_s for s <= t (scan order), else 0.  Thread (ty,tx) owns rows
    // ty+16a and columns tx+16b.
    {
      A acc[R][R];
#pragma unroll
      for (int a = 0; a < R; ++a)
#pragma unroll
        for (int b = 0; b < R; ++b) acc[a][b] = A(0);
      for (int i = 0; i < Dk; ++i) {
        A qa[R], kb[R];
#pragma unroll
        for (int a = 0; a < R; ++a) qa[a] = sQ[(ty + 16 * a) * ldk + i];
#pragma unroll
        for (int b = 0; b < R; ++b) kb[b] = sK[(tx + 16 * b) * ldk + i];
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
          for (int b = 0; b < R; ++b) acc[a][b] += qa[a] * kb[b];
      }
#pragma unroll
      for (int a = 0; a < R; ++a)
#pragma unroll
        for (int b = 0; b < R; ++b) {
          const int t = ty + 16 * a, s = tx + 16 * b;
          sP[t * (C + 1) + s] = (s <= t) ? acc[a][b] : A(0);
        }
    }
    __syncthreads();

    // out[t][j] = sum_{s<=t} P[t][s] V[s][j] + sum_i Q[t][i] S[i][j]   (S = state before this chunk)
#pragma unroll
    for (int a = 0; a < R; ++a) {
      const int t = ty + 16 * a;
      A acc = A(0);
      for (int s = 0; s <= t; ++s) acc += sP[t * (C + 1) + s] * sV[s * DVT + tx];
      for (int i = 0; i < Dk; ++i) acc += sQ[t * ldk + i] * sS[i * DVT + tx];
      const int p = c0 + t;
      if (p < N && j0 + tx < Dv) {
        const long s = reversed ? (long)(N - 1 - p) : (long)p;
        o[s * Dv + j0 + tx] = from_acc<T>(acc);
      }
    }
    __syncthreads();

    // S[i][j] += sum_s K[s][i] V[s][j]
    for (int i = ty; i < Dk; i += 16) {
      A acc = sS[i * DVT + tx];
      for (int s = 0; s < C; ++s) acc += sK[s * ldk + i] * sV[s * DVT + tx];
      sS[i * DVT + tx] = acc;
    }
    __syncthreads();
  }
}

template <typename T>
int launch_scan_simt(const void* q, const void* k, const void* v, void* out, int B, int H, int N,
                     int Dk, int Dv, int reversed, cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  constexpr int C = sizeof(A) == 8 ? 32 : 64;
  const size_t smem = scan_simt_smem_bytes<A>(C, Dk);
  auto kern = scan_simt_kernel<T, C>;
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((long)B * H), (unsigned)((Dv + kSimtDvTile - 1) / kSimtDvTile));
  kern<<<grid, kSimtThreads, smem, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k),
                                             static_cast<const T*>(v), static_cast<T*>(out), N, Dk,
                                             Dv, reversed);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

}  // namespace cott
