// Rotary position embedding of the reference's GPT module (GPT_Trainer/GPTCosAttention.py:458-476, the GPT-J
// "rotate every two" form of transformers' apply_rotary_pos_emb), applied in place to q and k wherever they
// lie -- e.g. the q and k slices of a packed [B, N, 3, H, d] projection output -- in one pass:
//   x'[2i]   = x[2i] cos_i - x[2i+1] sin_i
//   x'[2i+1] = x[2i+1] cos_i + x[2i] sin_i          i < rot_dim / 2, the other elements pass through
// `inverse` applies the transposed rotation (sin -> -sin), which is the backward of the op.
// HBM-bound elementwise work: one 16-byte piece (four pairs) per thread, fp32 arithmetic, one read and one write
// of q and k; the tables are [N, rot_dim/2] fp32 (per batch entry when `table_batch_stride` is not 0).
#include "common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

using namespace cott;

namespace {

template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Pair16<__half> {
  static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// one thread per 16-byte piece of a row, for q and k both (same sin / cos)
template <typename T>
__global__ void rotary_kernel(T* __restrict__ q, T* __restrict__ k, const float* __restrict__ sin_t,
                              const float* __restrict__ cos_t, long long sb, long long sh, long long sn, int H, int N,
                              int pieces, long long table_batch_stride, float sign, long long total, int h_inner) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int p = static_cast<int>(idx % pieces);
  const long long row = idx / pieces;
  // consecutive threads walk the dimension with the smaller stride (heads in a packed [B, N, 3, H, d] tensor)
  const int n = static_cast<int>(h_inner ? (row / H) % N : row % N);
  const int h = static_cast<int>(h_inner ? row % H : (row / N) % H);
  const long long b = row / (static_cast<long long>(H) * N);
  const long long off = b * sb + h * sh + n * sn + p * 8;
  const long long t = b * table_batch_stride + static_cast<long long>(n) * (pieces * 4) + p * 4;
  const float4 s4 = *reinterpret_cast<const float4*>(sin_t + t), c4 = *reinterpret_cast<const float4*>(cos_t + t);
  const float s[4] = {sign * s4.x, sign * s4.y, sign * s4.z, sign * s4.w}, c[4] = {c4.x, c4.y, c4.z, c4.w};
  uint4 u[2] = {*reinterpret_cast<uint4*>(q + off), *reinterpret_cast<uint4*>(k + off)};
#pragma unroll
  for (int t2 = 0; t2 < 2; ++t2) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&u[t2]);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = Pair16<T>::unpack(w[e]);
      float xo, yo;
      rot_pair(f.x, f.y, c[e], s[e], xo, yo);
      w[e] = Pair16<T>::pack(xo, yo);
    }
  }
  *reinterpret_cast<uint4*>(q + off) = u[0];
  *reinterpret_cast<uint4*>(k + off) = u[1];
}

}  // namespace

extern "C" int cott_rotary(void* q, void* k, const float* sin_table, const float* cos_table, const cott_layout* layout, int B,
                           int H, int N, int D, int rot_dim, long long table_batch_stride, int inverse, int dtype,
                           void* stream) {
  if (dtype != COTT_BF16 && dtype != COTT_F16)
    return fail(COTT_ERR_DTYPE, "cott_rotary takes float16 / bfloat16 (dtype code %d)", dtype);
  if (B < 0 || H < 0 || N < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d N=%d", B, H, N);
  if (D < 8 || D % 8 || rot_dim < 8 || rot_dim % 8 || rot_dim > D)
    return fail(COTT_ERR_SHAPE, "head dim and rotary dim must be multiples of 8 with rot_dim <= D (got %d, %d)", D, rot_dim);
  if ((long)B * H * N == 0) return COTT_OK;
  if (!q || !k || !sin_table || !cos_table) return fail(COTT_ERR_NULL, "null pointer");
  const long long sb = layout ? layout->in_b : (long long)H * N * D, sh = layout ? layout->in_h : (long long)N * D,
                  sn = layout ? layout->in_n : D;
  if ((sb | sh | sn) & 7 || table_batch_stride & 3) return fail(COTT_ERR_ALIGN, "strides must be multiples of 8 elements");
  for (const void* p : {(const void*)q, (const void*)k, (const void*)sin_table, (const void*)cos_table})
    if (reinterpret_cast<uintptr_t>(p) & 15) return fail(COTT_ERR_ALIGN, "tensors must be 16-byte aligned");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  const int pieces = rot_dim / 8;
  const long long total = (long long)B * H * N * pieces;
  const dim3 grid((unsigned)((total + 255) / 256), 1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sign = inverse ? -1.f : 1.f;
  if (dtype == COTT_BF16)
    rotary_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), sin_table,
                                                     cos_table, sb, sh, sn, H, N, pieces, table_batch_stride, sign, total, sh < sn);
  else
    rotary_kernel<__half><<<grid, 256, 0, s>>>(static_cast<__half*>(q), static_cast<__half*>(k), sin_table, cos_table, sb, sh,
                                              sn, H, N, pieces, table_batch_stride, sign, total, sh < sn);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}
