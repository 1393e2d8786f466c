// C ABI of the bidirectional (encoder) cosine attention.
#include "bidir.cuh"
#include "common.cuh"

using namespace cott;

namespace {

constexpr size_t kMaxSmem = 227 * 1024;

int check_bidir(int B, int H, int N, int Dk, int Dv, int dtype) {
  if (dtype_size(dtype) == 0) return fail(COTT_ERR_DTYPE, "unknown dtype code %d", dtype);
  if (B < 0 || H < 0 || N < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d N=%d", B, H, N);
  if (Dk < 16 || Dk > 128 || Dk % 16 || Dv < 16 || Dv > 128 || Dv % 16)
    return fail(COTT_ERR_SHAPE, "bidirectional attention needs head dims divisible by 16 in [16, 128] (got %d, %d)", Dk, Dv);
  if ((long)B * H > 0x7fffffffL) return fail(COTT_ERR_SHAPE, "B*H too large");
  return COTT_OK;
}

template <typename T>
int run_state(const void* x, const void* y, const unsigned char* keep, const float* nc, void* scratch, int B, int H,
              int N, int Dk, int Dv, int scale_by_length, cudaStream_t s) {
  using A = typename AccOf<T>::type;
  const long BH = (long)B * H;
  const int ns = bidir_nsplit(BH, N);
  const size_t smem = bidir_state_smem<A>(Dk, Dv);
  auto kern = bidir_state_kernel<T>;
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)BH, ns), kBidirThreads, smem, s>>>(static_cast<const T*>(x), static_cast<const T*>(y), keep, nc,
                                                          static_cast<A*>(scratch), H, N, Dk, Dv, ns, scale_by_length);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

template <typename T>
int run_fwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, void* out,
            void* scratch, int B, int H, int N, int Dk, int Dv, cudaStream_t s) {
  using A = typename AccOf<T>::type;
  const long BH = (long)B * H;
  const int ns = bidir_nsplit(BH, N);
  const size_t smem = bidir_apply_smem<A>(Dk, Dv);
  if (smem > kMaxSmem) return fail(COTT_ERR_SHAPE, "head dims %d x %d need %zu bytes of shared memory for this dtype", Dk, Dv, smem);
  int st = run_state<T>(k, v, keep, nc, scratch, B, H, N, Dk, Dv, 1, s);
  if (st) return st;
  auto kern = bidir_apply_kernel<T>;
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)BH, (N + kBidirTile - 1) / kBidirTile), kBidirThreads, smem, s>>>(
      static_cast<const T*>(q), keep, static_cast<const A*>(scratch), static_cast<T*>(out), H, N, Dk, Dv, ns);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

template <typename T>
int run_bwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, const void* dout,
            const void* scratch_s, void* scratch_ds, void* dq, void* dk, void* dv, float* dnorm, int B, int H, int N,
            int Dk, int Dv, cudaStream_t s) {
  using A = typename AccOf<T>::type;
  const long BH = (long)B * H;
  const int ns = bidir_nsplit(BH, N);
  const size_t smem = bidir_bwd_smem<A>(Dk, Dv);
  if (smem > kMaxSmem) return fail(COTT_ERR_SHAPE, "head dims %d x %d need %zu bytes of shared memory for this dtype", Dk, Dv, smem);
  COTT_CUDA_TRY(cudaMemsetAsync(dnorm, 0, sizeof(float) * H, s));
  int st = run_state<T>(q, dout, keep, nc, scratch_ds, B, H, N, Dk, Dv, 0, s);
  if (st) return st;
  auto kern = bidir_bwd_kernel<T>;
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)BH, (N + kBidirTile - 1) / kBidirTile), kBidirThreads, smem, s>>>(
      static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<const T*>(dout), keep,
      nc, static_cast<const A*>(scratch_s), static_cast<const A*>(scratch_ds), static_cast<T*>(dq), static_cast<T*>(dk),
      static_cast<T*>(dv), dnorm, H, N, Dk, Dv, ns);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

}  // namespace

extern "C" {

size_t cott_bidir_scratch_bytes(int B, int H, int N, int Dk, int Dv, int dtype) {
  if (check_bidir(B, H, N, Dk, Dv, dtype)) return 0;
  const long BH = (long)B * H;
  const size_t acc = dtype == COTT_F64 ? 8 : 4;
  return (size_t)BH * bidir_nsplit(BH, N) * Dk * Dv * acc;
}

int cott_bidir_fwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* norm_const,
                   void* out, void* scratch, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_bidir(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if (!q || !k || !v || !norm_const || !out || !scratch) return fail(COTT_ERR_NULL, "null pointer");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // head dim 64 in a 16-bit dtype: tensor-core kernel (it keeps the state on chip and ignores `scratch`)
  if (bidir_tc_usable(Dk, Dv, dtype, {q, k, v, out})) return launch_bidir_fwd_tc(q, k, v, keep, norm_const, out, B, H, N, dtype, s);
  switch (dtype) {
    case COTT_F32: return run_fwd<float>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
    case COTT_F64: return run_fwd<double>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
    case COTT_F16: return run_fwd<__half>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
    default: return run_fwd<__nv_bfloat16>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
  }
}

int cott_bidir_bwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* norm_const,
                   const void* dout, const void* scratch_state, void* scratch_dstate, void* dq, void* dk, void* dv,
                   float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_bidir(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if (H == 0) return COTT_OK;
  DeviceScope scope(dnorm_const);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((long)B * H * N == 0) {
    COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, s));
    return COTT_OK;
  }
  if (!q || !k || !v || !norm_const || !dout || !scratch_state || !scratch_dstate || !dq || !dk || !dv)
    return fail(COTT_ERR_NULL, "null pointer");
  // tensor-core kernel: recomputes the forward state on chip, so neither scratch buffer is touched
  if (bidir_tc_usable(Dk, Dv, dtype, {q, k, v, dout, dq, dk, dv}))
    return launch_bidir_bwd_tc(q, k, v, keep, norm_const, dout, dq, dk, dv, dnorm_const, B, H, N, dtype, s);
  switch (dtype) {
    case COTT_F32:
      return run_bwd<float>(q, k, v, keep, norm_const, dout, scratch_state, scratch_dstate, dq, dk, dv, dnorm_const, B, H, N, Dk, Dv, s);
    case COTT_F64:
      return run_bwd<double>(q, k, v, keep, norm_const, dout, scratch_state, scratch_dstate, dq, dk, dv, dnorm_const, B, H, N, Dk, Dv, s);
    case COTT_F16:
      return run_bwd<__half>(q, k, v, keep, norm_const, dout, scratch_state, scratch_dstate, dq, dk, dv, dnorm_const, B, H, N, Dk, Dv, s);
    default:
      return run_bwd<__nv_bfloat16>(q, k, v, keep, norm_const, dout, scratch_state, scratch_dstate, dq, dk, dv, dnorm_const, B, H, N, Dk, Dv, s);
  }
}

int cott_bidir_fwd_strided(const void* q, const void* k, const void* v, const unsigned char* keep,
                           const float* norm_const, void* out, const cott_layout* layout, int B, int H, int N, int Dk,
                           int Dv, int dtype, void* stream) {
  int st = check_bidir(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if (!q || !k || !v || !norm_const || !out) return fail(COTT_ERR_NULL, "null pointer");
  if (!bidir_tc_usable(Dk, Dv, dtype, {q, k, v, out}))
    return fail(COTT_ERR_UNSUPPORTED, "strided bidirectional attention needs head dim 64, a 16-bit dtype and 16-byte aligned tensors");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  return launch_bidir_fwd_tc(q, k, v, keep, norm_const, out, B, H, N, dtype, static_cast<cudaStream_t>(stream), layout);
}

int cott_bidir_bwd_strided(const void* q, const void* k, const void* v, const unsigned char* keep,
                           const float* norm_const, const void* dout, const cott_layout* layout, void* dq, void* dk,
                           void* dv, float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_bidir(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if (H == 0) return COTT_OK;
  DeviceScope scope(dnorm_const);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if ((long)B * H * N == 0) {
    COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, s));
    return COTT_OK;
  }
  if (!q || !k || !v || !norm_const || !dout || !dq || !dk || !dv) return fail(COTT_ERR_NULL, "null pointer");
  if (!bidir_tc_usable(Dk, Dv, dtype, {q, k, v, dout, dq, dk, dv}))
    return fail(COTT_ERR_UNSUPPORTED, "strided bidirectional attention needs head dim 64, a 16-bit dtype and 16-byte aligned tensors");
  return launch_bidir_bwd_tc(q, k, v, keep, norm_const, dout, dq, dk, dv, dnorm_const, B, H, N, dtype, s, layout);
}

}  // extern "C"
