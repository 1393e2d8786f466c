/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's cosine linear
 * attention scan.  Nothing in the product links, loads or calls this file; only
 * the tests, the smoke check and the benchmark's CPU-baseline leg do, and only
 * as the checker or the timed baseline.
 *
 * Parity status: pinned.  The restatement is checked in tests against (i)
 * fixtures produced by executing the reference's own Python modules
 * (tests/golden/make_golden.py) and (ii) fixtures produced by running the
 * reference's compiled CUDA kernel on a B200 (tests/golden/make_golden_gpu.py).
 *
 * Each function cites the reference lines it follows (paths inside the
 * reference project).
 *
 * Build: gcc -O3 -fopenmp -fPIC -shared -o oracle/libcott_oracle.so oracle/cott_oracle.c -lm
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/*
 * The scan of Cuda_Kernel/combined_kernel_general.cu:96-170 (kernel_mod_2) and
 * :173-251 (kernel_mod_4), which differ only in loop unrolling:
 *
 *   for every (n, h, d_out):   state[0..D_attn) = 0                      (:121-123)
 *     for s in 0..S-1 (or S-1..0 when reversed)                          (:126-130)
 *       state[i] += V[n,h,s,d_out] * K[n,h,s,i]                          (:143-144)
 *       out[n,h,s,d_out] = sum_i state[i] * Q[n,h,s,i]                   (:148-165)
 *
 * All tensors are contiguous [B,H,N,D] row-major (:136,143,165).  The reference
 * keeps `state` and the sum in the storage type T; this restatement is written
 * once per accumulator type (double, float).
 */
#define DEFINE_SCAN(NAME, T)                                                          \
  void NAME(const T* q, const T* k, const T* v, T* out, int B, int H, int N, int Dk,  \
            int Dv, int reversed) {                                                   \
    const long BH = (long)B * H;                                                      \
    _Pragma("omp parallel for collapse(2) schedule(static)")                          \
    for (long bh = 0; bh < BH; ++bh) {                                                \
      for (int j = 0; j < Dv; ++j) {                                                  \
        T* state = (T*)calloc((size_t)Dk, sizeof(T));                                 \
        const T* qb = q + bh * (long)N * Dk;                                          \
        const T* kb = k + bh * (long)N * Dk;                                          \
        const T* vb = v + bh * (long)N * Dv;                                          \
        T* ob = out + bh * (long)N * Dv;                                              \
        for (int s_ = 0; s_ < N; ++s_) {                                              \
          const int s = reversed ? N - 1 - s_ : s_;                                   \
          const T vv = vb[(long)s * Dv + j];                                          \
          T sum = 0;                                                                  \
          for (int i = 0; i < Dk; ++i) {                                              \
            state[i] += vv * kb[(long)s * Dk + i];                                    \
            sum += state[i] * qb[(long)s * Dk + i];                                   \
          }                                                                           \
          ob[(long)s * Dv + j] = sum;                                                 \
        }                                                                             \
        free(state);                                                                  \
      }                                                                               \
    }                                                                                 \
  }

DEFINE_SCAN(cott_oracle_scan_f64, double)
DEFINE_SCAN(cott_oracle_scan_f32, float)

/*
 * Round-to-nearest-even float -> bfloat16 -> float, used to restate the
 * reference's bf16 mode, where state, products and sums are all held in bf16
 * (combined_kernel_general.cu:121,133,143-149 with T = at::BFloat16).
 */
static inline float bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return x; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&x, &u, 4);
  return x;
}

/*
 * The same scan with every intermediate rounded to bf16, following the order of
 * operations of kernel_mod_2 for D_attn < 128 with 32 lanes
 * (combined_kernel_general.cu:109-165): lane l owns the contiguous slice
 * [l*D/32, (l+1)*D/32) (:109-113), accumulates its partial sum in pairs
 * (:140-149), and the lanes are combined by a shfl_down tree (:155-158).
 * Inputs and outputs are float arrays holding bf16-representable values.
 */
void cott_oracle_scan_bf16_emul(const float* q, const float* k, const float* v, float* out, int B,
                                int H, int N, int Dk, int Dv, int reversed) {
  const long BH = (long)B * H;
  const int lanes = (Dk == 32) ? 16 : 32; /* :273-277 */
  const int per = Dk / lanes;
#pragma omp parallel for collapse(2) schedule(static)
  for (long bh = 0; bh < BH; ++bh) {
    for (int j = 0; j < Dv; ++j) {
      float* state = (float*)calloc((size_t)Dk, sizeof(float));
      float part[32];
      const float* qb = q + bh * (long)N * Dk;
      const float* kb = k + bh * (long)N * Dk;
      const float* vb = v + bh * (long)N * Dv;
      float* ob = out + bh * (long)N * Dv;
      for (int s_ = 0; s_ < N; ++s_) {
        const int s = reversed ? N - 1 - s_ : s_;
        const float vv = vb[(long)s * Dv + j];
        for (int l = 0; l < lanes; ++l) {
          float sum = 0.f;
          for (int i = l * per; i < (l + 1) * per; i += 2) {
            state[i] = bf16_round(state[i] + bf16_round(vv * kb[(long)s * Dk + i]));
            state[i + 1] = bf16_round(state[i + 1] + bf16_round(vv * kb[(long)s * Dk + i + 1]));
            float a = bf16_round(state[i] * qb[(long)s * Dk + i]);
            float b = bf16_round(state[i + 1] * qb[(long)s * Dk + i + 1]);
            sum = bf16_round(sum + bf16_round(a + b));
          }
          part[l] = sum;
        }
        for (int off = lanes / 2; off > 0; off /= 2)
          for (int l = 0; l < off; ++l) part[l] = bf16_round(part[l] + part[l + off]);
        ob[(long)s * Dv + j] = part[0];
      }
      free(state);
    }
  }
}

/*
 * Recurrent decode step of GPT_Trainer/GPTCosAttention.py:236,253-272 for a
 * batch of independent (b,h) states (the reference runs batch 1):
 *   v' = v / max(cur_s ** sigmoid(c_h), 1)                         (:236)
 *   state[b,h,j,i] += v'[j] * k_hat[i]     (float64, [d_v, d_k])   (:264)
 *   o[j] = sum_i q_hat[i] * state[b,h,j,i]                         (:267)
 * q_hat, k_hat are the L2-normalised rows (:229-230, eps 1e-12).  cur_s is the
 * 1-based position counter (:82, :269).
 */
void cott_oracle_decode_step_f64(double* state, const double* q, const double* k, const double* v,
                                 const double* norm_const, double* out, int B, int H, int Dk,
                                 int Dv, long cur_s) {
#pragma omp parallel for schedule(static)
  for (long bh = 0; bh < (long)B * H; ++bh) {
    const int h = (int)(bh % H);
    const double* qq = q + bh * Dk;
    const double* kk = k + bh * Dk;
    const double* vv = v + bh * Dv;
    double* st = state + bh * (long)Dk * Dv;
    double nq = 0, nk = 0;
    for (int i = 0; i < Dk; ++i) {
      nq += qq[i] * qq[i];
      nk += kk[i] * kk[i];
    }
    nq = fmax(sqrt(nq), 1e-12);
    nk = fmax(sqrt(nk), 1e-12);
    const double sig = 1.0 / (1.0 + exp(-norm_const[h]));
    const double scale = fmax(pow((double)cur_s, sig), 1.0);
    for (int j = 0; j < Dv; ++j) {
      const double vj = vv[j] / scale;
      double o = 0;
      for (int i = 0; i < Dk; ++i) {
        st[(long)j * Dk + i] += vj * (kk[i] / nk);
        o += (qq[i] / nq) * st[(long)j * Dk + i];
      }
      out[bh * Dv + j] = o;
    }
  }
}
