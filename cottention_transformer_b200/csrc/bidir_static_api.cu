// cott_bidir_fwd_static: the bidirectional forward for callers that must not allocate.
//
// Who this is for: hosts that hand out all device memory once at start-up and then run a steady
// state in which a call into the CUDA allocator is off limits -- a serving process whose memory
// pool is frozen and shared with other tenants, or a latency-critical loop where cudaMalloc's
// implicit device synchronisation would stall every stream.  cott_bidir_fwd needs a scratch buffer
// from its caller; a caller of this kind has nowhere to get one.  Here the scratch is a fixed
// array that is part of the library image itself.
#include "bidir.cuh"
#include "common.cuh"

using namespace cott;

namespace {

// The scratch.  It occupies COTT_BIDIR_STATIC_SCRATCH_BYTES on every GPU that loads this library,
// from load until the process exits, whether or not the entry point is ever called.
constexpr size_t kStaticScratchBytes = COTT_BIDIR_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_bidir_static_scratch[kStaticScratchBytes];

// In host code `g_bidir_static_scratch` is only a handle for the symbol, not a device address;
// the address is looked up once per device (with that device current) and remembered.
constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

int static_scratch(void** ptr) {
  int dev = 0;
  COTT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(COTT_ERR_UNSUPPORTED, "device index %d out of range", dev);
  void* p = __atomic_load_n(&g_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    COTT_CUDA_TRY(cudaGetSymbolAddress(&p, g_bidir_static_scratch));
    __atomic_store_n(&g_scratch_ptr[dev], p, __ATOMIC_RELEASE);  // racing threads store the same value
  }
  *ptr = p;
  return COTT_OK;
}

template <typename T>
int run(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, void* out,
        void* scratch, int B, int H, int N, int Dk, int Dv, cudaStream_t s) {
  using A = typename AccOf<T>::type;
  const long BH = (long)B * H;
  const int ns = bidir_nsplit(BH, N);
  const size_t smem_state = bidir_state_smem<A>(Dk, Dv), smem_apply = bidir_apply_smem<A>(Dk, Dv);
  if (smem_apply > 227 * 1024)
    return fail(COTT_ERR_SHAPE, "head dims %d x %d need %zu bytes of shared memory for this dtype", Dk, Dv, smem_apply);
  auto state_kern = bidir_state_kernel<T>;
  auto apply_kern = bidir_apply_kernel<T>;
  COTT_CUDA_TRY(cudaFuncSetAttribute(state_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_state));
  COTT_CUDA_TRY(cudaFuncSetAttribute(apply_kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_apply));
  // Every (b,h,split) slot that the second kernel reads is written in full by the first one, so
  // nothing in the shared array has to be cleared between calls.
  state_kern<<<dim3((unsigned)BH, ns), kBidirThreads, smem_state, s>>>(
      static_cast<const T*>(k), static_cast<const T*>(v), keep, nc, static_cast<A*>(scratch), H, N, Dk, Dv, ns, 1);
  COTT_CUDA_TRY(cudaGetLastError());
  apply_kern<<<dim3((unsigned)BH, (N + kBidirTile - 1) / kBidirTile), kBidirThreads, smem_apply, s>>>(
      static_cast<const T*>(q), keep, static_cast<const A*>(scratch), static_cast<T*>(out), H, N, Dk, Dv, ns);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

}  // namespace

extern "C" int cott_bidir_fwd_static(const void* q, const void* k, const void* v, const unsigned char* keep,
                                     const float* norm_const, void* out, int B, int H, int N, int Dk, int Dv,
                                     int dtype, void* stream) {
  if (dtype_size(dtype) == 0) return fail(COTT_ERR_DTYPE, "unknown dtype code %d", dtype);
  if (B < 0 || H < 0 || N < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d N=%d", B, H, N);
  if (Dk < 16 || Dk > 128 || Dk % 16 || Dv < 16 || Dv > 128 || Dv % 16)
    return fail(COTT_ERR_SHAPE, "bidirectional attention needs head dims divisible by 16 in [16, 128] (got %d, %d)", Dk, Dv);
  const long BH = (long)B * H;
  if (BH > 0x7fffffffL) return fail(COTT_ERR_SHAPE, "B*H too large");
  // 16-bit tensors with head dim 64 run on the tensor-core kernel, which keeps the state on chip: it needs no
  // scratch at all (so no size limit applies) and allocates nothing either (tensor maps are built on the host stack)
  const bool on_chip = bidir_tc_usable(Dk, Dv, dtype, {q, k, v, out});
  const size_t need = (size_t)BH * bidir_nsplit(BH, N) * Dk * Dv * (dtype == COTT_F64 ? 8 : 4);
  if (!on_chip && need > kStaticScratchBytes)
    return fail(COTT_ERR_SHAPE,
                "this problem needs %zu bytes of scratch but the built-in scratch of cott_bidir_fwd_static holds %zu "
                "(COTT_BIDIR_STATIC_SCRATCH_BYTES); use cott_bidir_fwd with a caller-provided buffer",
                need, kStaticScratchBytes);
  if (BH * N == 0) return COTT_OK;
  if (!q || !k || !v || !norm_const || !out) return fail(COTT_ERR_NULL, "null pointer");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  if (on_chip)
    return launch_bidir_fwd_tc(q, k, v, keep, norm_const, out, B, H, N, dtype, static_cast<cudaStream_t>(stream));
  void* scratch = nullptr;
  int st = static_scratch(&scratch);
  if (st) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case COTT_F32: return run<float>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
    case COTT_F64: return run<double>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
    case COTT_F16: return run<__half>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
    default: return run<__nv_bfloat16>(q, k, v, keep, norm_const, out, scratch, B, H, N, Dk, Dv, s);
  }
}
