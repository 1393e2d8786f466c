// Exact-mode scan: chunked cosine-linear-attention scan on CUDA cores.
//
// Computes what the reference's kernel_mod_2/kernel_mod_4
// (Cuda_Kernel/combined_kernel_general.cu:96-251) compute,
//   out[s, j] = sum_i Q[s, i] * sum_{t<=s} K[t, i] V[t, j]        (t >= s when reversed)
// but in chunked form: the sequence is cut into chunks of C positions; inside a chunk the
// masked product (Q K^T) V is formed directly, everything older is carried in a
// Dk x 16 (or Dk x 64) slice of the state S = sum K (x) V that lives in shared memory.  Sums are kept
// in fp32 (fp64 for double inputs) whatever the storage type -- the reference keeps them
// in the storage type (:121,133).
//
// One CTA per (batch*head, 16- or 64-column slice of Dv); the slices of the state are independent,
// exactly as the reference's one-block-per-output-column decomposition (:104-106).
// This is the fp32/fp64 correctness path; the bf16/fp16 fast path is the tcgen05 kernel.
#pragma once

#include "common.cuh"

namespace cott {

constexpr int kSimtThreads = 256;

template <typename A>
inline size_t scan_simt_smem_bytes(int C, int Dk, int dvt) {
  return sizeof(A) * ((size_t)2 * C * (Dk + 1) + (size_t)C * (C + 1) + (size_t)C * dvt + (size_t)Dk * dvt);
}

// C = chunk length, DVT = columns of V (and of the state) one CTA owns.  Thread (ty, tx) of the 16 x 16 thread
// grid owns rows ty + 16 a and columns tx + 16 b of every product, so each step of an inner loop is
// (C/16 + DVT/16) shared-memory loads for (C/16) x (DVT/16) multiply-adds.
template <typename T, int C, int DVT, int PRE>
__global__ void __launch_bounds__(kSimtThreads)
scan_simt_kernel(const T* Q, const T* K, const T* V, T* O, int N, int Dk, int Dv, int reversed) {
  using A = typename AccOf<T>::type;
  constexpr int R = C / 16, NB = DVT / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ldk = Dk + 1;
  A* sQ = reinterpret_cast<A*>(smem_raw);  // [C][Dk+1]
  A* sK = sQ + (size_t)C * ldk;            // [C][Dk+1]
  A* sP = sK + (size_t)C * ldk;            // [C][C+1]
  A* sV = sP + (size_t)C * (C + 1);        // [C][DVT]
  A* sS = sV + (size_t)C * DVT;            // [Dk][DVT]

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const long bh = blockIdx.x;
  const int j0 = blockIdx.y * DVT;
  const T* q = Q + bh * (long)N * Dk;
  const T* k = K + bh * (long)N * Dk;
  const T* v = V + bh * (long)N * Dv;
  T* o = O + bh * (long)N * Dv;

  for (int idx = tid; idx < Dk * DVT; idx += kSimtThreads) sS[idx] = A(0);

  // The rows of the next chunk are fetched into registers while the current one is worked on (their latency
  // was the largest stall of the kernel when the staging was synchronous).  Element m of a thread is flat index
  // tid + 256 m of the [C][Dk] tile; PRE elements per tensor fit the register budget (Dk <= 128), wider tiles
  // are staged synchronously.
  constexpr int NV = C * DVT / kSimtThreads;
  const int nqk = C * Dk / kSimtThreads;
  const bool pre = nqk <= PRE;
  const int r_first = tid / Dk, i_first = tid % Dk, r_step = kSimtThreads / Dk, i_step = kSimtThreads % Dk;
  const T zero = from_acc<T>(A(0));
  T pq[PRE], pk[PRE], pv[NV];
  auto fetch = [&](int c0) {
    int r = r_first, i = i_first;
#pragma unroll
    for (int m = 0; m < PRE; ++m) {
      if (m < nqk) {
        const int p = c0 + r;
        pq[m] = zero, pk[m] = zero;
        if (p < N) {
          const long s = reversed ? (long)(N - 1 - p) : (long)p;
          pq[m] = q[s * Dk + i];
          pk[m] = k[s * Dk + i];
        }
        i += i_step, r += r_step;
        if (i >= Dk) i -= Dk, ++r;
      }
    }
#pragma unroll
    for (int m = 0; m < NV; ++m) {
      const int idx = tid + kSimtThreads * m, rr = idx / DVT, j = idx % DVT, p = c0 + rr;
      pv[m] = zero;
      if (p < N && j0 + j < Dv) {
        const long s = reversed ? (long)(N - 1 - p) : (long)p;
        pv[m] = v[s * Dv + j0 + j];
      }
    }
  };
  auto stash = [&]() {
    int r = r_first, i = i_first;
#pragma unroll
    for (int m = 0; m < PRE; ++m) {
      if (m < nqk) {
        sQ[r * ldk + i] = to_acc(pq[m]);
        sK[r * ldk + i] = to_acc(pk[m]);
        i += i_step, r += r_step;
        if (i >= Dk) i -= Dk, ++r;
      }
    }
#pragma unroll
    for (int m = 0; m < NV; ++m) sV[tid + kSimtThreads * m] = to_acc(pv[m]);
  };
  if (pre) fetch(0);

  for (int c0 = 0; c0 < N; c0 += C) {
    // Stage the chunk.  Row r holds logical position p = c0 + r of the scan order;
    // physical row s = p (forward) or N-1-p (reversed).  Rows past the end are zero.
    if (pre) {
      stash();
    } else {
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
    }
    __syncthreads();
    if (pre && c0 + C < N) fetch(c0 + C);

    // P[t][s] = Q_t . K_s for s <= t (scan order), else 0.
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

    // out[t][j] = sum_s P[t][s] V[s][j] + sum_i Q[t][i] S[i][j]   (S = state before this chunk; P is zero
    // above the diagonal, so the first sum stops at the thread's last row)
    {
      A acc[R][NB];
#pragma unroll
      for (int a = 0; a < R; ++a)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[a][b] = A(0);
      const int s_end = ty + 16 * (R - 1);
      for (int s = 0; s <= s_end; ++s) {
        A pa[R], vb[NB];
#pragma unroll
        for (int a = 0; a < R; ++a) pa[a] = sP[(ty + 16 * a) * (C + 1) + s];
#pragma unroll
        for (int b = 0; b < NB; ++b) vb[b] = sV[s * DVT + tx + 16 * b];
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
          for (int b = 0; b < NB; ++b) acc[a][b] += pa[a] * vb[b];
      }
      for (int i = 0; i < Dk; ++i) {
        A qa[R], sb[NB];
#pragma unroll
        for (int a = 0; a < R; ++a) qa[a] = sQ[(ty + 16 * a) * ldk + i];
#pragma unroll
        for (int b = 0; b < NB; ++b) sb[b] = sS[i * DVT + tx + 16 * b];
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
          for (int b = 0; b < NB; ++b) acc[a][b] += qa[a] * sb[b];
      }
#pragma unroll
      for (int a = 0; a < R; ++a) {
        const int p = c0 + ty + 16 * a;
        if (p < N) {
          const long s = reversed ? (long)(N - 1 - p) : (long)p;
#pragma unroll
          for (int b = 0; b < NB; ++b)
            if (j0 + tx + 16 * b < Dv) o[s * Dv + j0 + tx + 16 * b] = from_acc<T>(acc[a][b]);
        }
      }
    }
    __syncthreads();

    // S[i][j] += sum_s K[s][i] V[s][j], 64 rows of the state at a time
    for (int i0 = 0; i0 < Dk; i0 += 64) {
      A acc[4][NB];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[a][b] = A(0);
      for (int s = 0; s < C; ++s) {
        A ka[4], vb[NB];
#pragma unroll
        for (int a = 0; a < 4; ++a) ka[a] = (i0 + ty + 16 * a < Dk) ? sK[s * ldk + i0 + ty + 16 * a] : A(0);
#pragma unroll
        for (int b = 0; b < NB; ++b) vb[b] = sV[s * DVT + tx + 16 * b];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < NB; ++b) acc[a][b] += ka[a] * vb[b];
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
        if (i0 + ty + 16 * a < Dk) {
#pragma unroll
          for (int b = 0; b < NB; ++b) sS[(i0 + ty + 16 * a) * DVT + tx + 16 * b] += acc[a][b];
        }
    }
    __syncthreads();
  }
}

template <typename T, int C, int DVT, int PRE>
int launch_scan_simt_p(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk, int Dv,
                       int reversed, cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  const size_t smem = scan_simt_smem_bytes<A>(C, Dk, DVT);
  auto kern = scan_simt_kernel<T, C, DVT, PRE>;
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)((long)B * H), (unsigned)((Dv + DVT - 1) / DVT));
  kern<<<grid, kSimtThreads, smem, stream>>>(static_cast<const T*>(q), static_cast<const T*>(k),
                                             static_cast<const T*>(v), static_cast<T*>(out), N, Dk,
                                             Dv, reversed);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

// PRE = prefetch registers per tensor: 16 covers Dk <= 64 (Dk <= 128 in fp64), 32 covers Dk <= 128 in the 4-byte types
template <typename T, int C, int DVT>
int launch_scan_simt_t(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk, int Dv,
                       int reversed, cudaStream_t stream) {
  if (sizeof(typename AccOf<T>::type) <= 4 && C * Dk / kSimtThreads > 16)
    return launch_scan_simt_p<T, C, DVT, 32>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
  return launch_scan_simt_p<T, C, DVT, 16>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
}

// A CTA owns 64 columns of V when V has more than 16 and the tiles fit in 200 KB of shared memory, otherwise 16: the masked product Q K^T is the largest term and every column slice recomputes it.
template <typename T>
int launch_scan_simt(const void* q, const void* k, const void* v, void* out, int B, int H, int N,
                     int Dk, int Dv, int reversed, cudaStream_t stream) {
  using A = typename AccOf<T>::type;
  constexpr int C = sizeof(A) == 8 ? 32 : 64;
  if (Dv > 16 && scan_simt_smem_bytes<A>(C, Dk, 64) <= 200 * 1024)
    return launch_scan_simt_t<T, C, 64>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
  return launch_scan_simt_t<T, C, 16>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
}

}  // namespace cott
