// C ABI of cottention_b200: argument validation and dispatch.  No torch types here;
// the Python host (ctypes) and any other FFI bind these symbols directly.
#include "common.cuh"
#include "decode.cuh"
#include "scan_simt.cuh"

using namespace cott;

namespace {

int check_scan_args(const void* q, const void* k, const void* v, const void* out, int B, int H,
                    int N, int Dk, int Dv, int dtype) {
  if (dtype_size(dtype) == 0) return fail(COTT_ERR_DTYPE, "unknown dtype code %d", dtype);
  if (B < 0 || H < 0 || N < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d N=%d", B, H, N);
  if (Dk < 16 || Dk > 256 || Dk % 16 != 0)
    return fail(COTT_ERR_SHAPE, "D_attn must be divisible by 16 and in [16, 256] (got %d)", Dk);
  if (Dv < 1) return fail(COTT_ERR_SHAPE, "D_value must be >= 1 (got %d)", Dv);
  if ((long)B * H > 0x7fffffffL) return fail(COTT_ERR_SHAPE, "B*H too large");
  if ((long)B * H * N > 0 && (!q || !k || !v || !out)) return fail(COTT_ERR_NULL, "null tensor pointer");
  return COTT_OK;
}

int scan_dispatch(const void* q, const void* k, const void* v, void* out, int B, int H, int N,
                  int Dk, int Dv, int dtype, int reversed, cudaStream_t stream) {
  if ((long)B * H * N == 0) return COTT_OK;
  // head dims 64, 128, 192, 256 in a 16-bit dtype: tensor cores (products rounded to the storage type between the two GEMMs of a
  // chunk, fp32 accumulation); everything else: the exact CUDA-core kernel
  if (scan_tc_usable(Dk, Dv, dtype, q, k, v, out)) return launch_scan_tc(q, k, v, out, B, H, N, Dk, Dv, dtype, reversed, stream);
  switch (dtype) {
    case COTT_F32: return launch_scan_simt<float>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
    case COTT_F64: return launch_scan_simt<double>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
    case COTT_F16: return launch_scan_simt<__half>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
    case COTT_BF16:
      return launch_scan_simt<__nv_bfloat16>(q, k, v, out, B, H, N, Dk, Dv, reversed, stream);
  }
  return fail(COTT_ERR_DTYPE, "unknown dtype code %d", dtype);
}

}  // namespace

extern "C" {

const char* cott_version(void) { return "cottention_b200 0.1.0 sm_100a"; }

const char* cott_last_error(void) { return err_buf(); }

const char* cott_status_string(int status) {
  switch (status) {
    case COTT_OK: return "ok";
    case COTT_ERR_NULL: return "null pointer";
    case COTT_ERR_SHAPE: return "unsupported shape";
    case COTT_ERR_DTYPE: return "unsupported dtype";
    case COTT_ERR_CUDA: return "CUDA error";
    case COTT_ERR_ALIGN: return "misaligned pointer";
    case COTT_ERR_DEVICE_WAIT: return "device-side wait gave up";
    case COTT_ERR_UNSUPPORTED: return "unsupported request";
    default: return "unknown status";
  }
}

int cott_scan(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk,
              int Dv, int dtype, int reversed, void* stream) {
  int st = check_scan_args(q, k, v, out, B, H, N, Dk, Dv, dtype);
  if (st != COTT_OK) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  return scan_dispatch(q, k, v, out, B, H, N, Dk, Dv, dtype, reversed != 0,
                       static_cast<cudaStream_t>(stream));
}

int cott_scan_bwd(const void* q, const void* k, const void* v, const void* dout, void* dq, void* dk,
                  void* dv, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_scan_args(q, k, v, dout, B, H, N, Dk, Dv, dtype);
  if (st != COTT_OK) return st;
  if (Dv < 16 || Dv > 256 || Dv % 16 != 0)
    return fail(COTT_ERR_SHAPE, "backward needs D_value divisible by 16 and in [16, 256] (got %d)", Dv);
  if ((long)B * H * N > 0 && (!dq || !dk || !dv)) return fail(COTT_ERR_NULL, "null gradient pointer");
  if ((long)B * H * N == 0) return COTT_OK;
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // dq = scan(dout, v, k): "Q"=dout [Dv], "K"=v [Dv], "V"=k [Dk]
  st = scan_dispatch(dout, v, k, dq, B, H, N, Dv, Dk, dtype, 0, s);
  if (st != COTT_OK) return st;
  // dk = scan(v, dout, q, reversed)
  st = scan_dispatch(v, dout, q, dk, B, H, N, Dv, Dk, dtype, 1, s);
  if (st != COTT_OK) return st;
  // dv = scan(k, q, dout, reversed)
  return scan_dispatch(k, q, dout, dv, B, H, N, Dk, Dv, dtype, 1, s);
}


int cott_decode_steps(float* state, const void* q, const void* k, const void* v, const float* norm_const, void* out,
                      int B, int H, int T, int Dk, int Dv, int dtype, long long pos, const long long* positions,
                      void* stream) {
  if (dtype != COTT_F32 && dtype != COTT_F16 && dtype != COTT_BF16)
    return fail(COTT_ERR_DTYPE, "decode takes float32/float16/bfloat16 tokens and a float32 state (dtype code %d)", dtype);
  if (B < 0 || H < 0 || T < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d T=%d", B, H, T);
  if (Dk != 16 && Dk != 32 && Dk != 64 && Dk != 128)
    return fail(COTT_ERR_SHAPE, "decode supports D_attn in {16, 32, 64, 128} (got %d)", Dk);
  if (Dv < 1 || Dv > 128) return fail(COTT_ERR_SHAPE, "decode supports D_value in [1, 128] (got %d)", Dv);
  if (!positions && pos < 1) return fail(COTT_ERR_SHAPE, "positions are 1-based (got %lld)", pos);
  if ((long)B * H * T == 0) return COTT_OK;
  if (!state || !q || !k || !v || !norm_const || !out) return fail(COTT_ERR_NULL, "null pointer");
  if (reinterpret_cast<uintptr_t>(state) & 15) return fail(COTT_ERR_ALIGN, "state must be 16-byte aligned");
  DeviceScope scope(state);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case COTT_F32: return launch_decode<float>(state, q, k, v, norm_const, out, B, H, Dk, Dv, T, pos, positions, s);
    case COTT_F16: return launch_decode<__half>(state, q, k, v, norm_const, out, B, H, Dk, Dv, T, pos, positions, s);
    default: return launch_decode<__nv_bfloat16>(state, q, k, v, norm_const, out, B, H, Dk, Dv, T, pos, positions, s);
  }
}

int cott_decode_step(float* state, const void* q, const void* k, const void* v, const float* norm_const, void* out,
                     int B, int H, int Dk, int Dv, int dtype, long long pos, const long long* positions,
                     void* stream) {
  return cott_decode_steps(state, q, k, v, norm_const, out, B, H, 1, Dk, Dv, dtype, pos, positions, stream);
}

}  // extern "C"
