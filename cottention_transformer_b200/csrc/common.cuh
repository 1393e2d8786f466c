// Shared host/device helpers for the cottention_b200 kernels.
#pragma once
#include <initializer_list>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/cottention_b200.h"

namespace cott {

// ---- per-thread error text -----------------------------------------------------------------
inline char* err_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
inline int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return status;
}
inline int cuda_fail(cudaError_t e, const char* what) {
  return fail(COTT_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}
#define COTT_CUDA_TRY(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return ::cott::cuda_fail(_e, #expr); \
  } while (0)

// Makes the device that owns `ptr` current on the calling thread for the lifetime of the object
// (like the reference's at::cuda::CUDAGuard, combined_kernel_general.cu:412) and thereby binds
// that device's primary context to the thread -- needed before any driver-API call on threads
// that have made no CUDA call yet, e.g. autograd worker threads.
class DeviceScope {
 public:
  explicit DeviceScope(const void* ptr) {
    cudaPointerAttributes attr;
    if (ptr && cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeDevice) {
      dev_ = attr.device;
    } else {
      cudaGetLastError();
      if (cudaGetDevice(&dev_) != cudaSuccess) dev_ = 0;
    }
    if (cudaGetDevice(&prev_) != cudaSuccess) prev_ = dev_;
    status_ = cudaSetDevice(dev_);
  }
  ~DeviceScope() {
    if (prev_ != dev_) cudaSetDevice(prev_);
  }
  cudaError_t status() const { return status_; }
  int device() const { return dev_; }

 private:
  int dev_ = 0, prev_ = 0;
  cudaError_t status_ = cudaSuccess;
};

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case COTT_F32: return 4;
    case COTT_F64: return 8;
    case COTT_F16: return 2;
    case COTT_BF16: return 2;
    default: return 0;
  }
}

// ---- element <-> accumulator conversions ------------------------------------------------------
template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };

__device__ __forceinline__ float to_acc(float x) { return x; }
__device__ __forceinline__ double to_acc(double x) { return x; }
__device__ __forceinline__ float to_acc(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_acc(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_acc(typename AccOf<T>::type x);
template <> __device__ __forceinline__ float from_acc<float>(float x) { return x; }
template <> __device__ __forceinline__ double from_acc<double>(double x) { return x; }
template <> __device__ __forceinline__ __half from_acc<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

// Programmatic dependent launch.  A kernel that begins with pdl_allow_next() lets the next kernel in the stream be
// scheduled while it is still running -- that kernel's CTAs take the SMs this one leaves idle or frees, and run their
// set-up (barriers, TMEM allocation, descriptor prefetch) -- and a kernel launched with launch_pdl() must call
// pdl_wait_prior() before it touches anything another kernel may have produced: the wait returns once every kernel
// before it in the stream has completed and its writes are visible, so the results are those of plain stream order.
// (Measured: 10.3 -> 8.9 us per token for eagerly launched decode steps; no difference for the 50-90 us causal kernels,
// whose launch gaps were ~1 us already.)
__device__ __forceinline__ void pdl_allow_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
template <typename K, typename... Args>
cudaError_t launch_pdl(K kernel, dim3 grid, unsigned threads, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// One pair of the rotary embedding ("rotate every two"): (x, y) -> (x c - y s, y c + x s).  Spelled with explicit
// roundings so that every kernel that rotates -- the stand-alone pass and the causal kernels that rotate their tiles
// in shared memory -- produces the same bits.
__device__ __forceinline__ void rot_pair(float x, float y, float c, float s, float& xo, float& yo) {
  xo = __fmaf_rn(x, c, -__fmul_rn(y, s));
  yo = __fmaf_rn(y, c, __fmul_rn(x, s));
}

// Tensor-core path of the bidirectional form (defined next to the other tcgen05 kernels, which share the
// device status word): head dim 64, 16-bit dtypes, 16-byte aligned tensors.  `*_usable` says whether a
// problem qualifies; the launchers assume it does.
bool bidir_tc_usable(int Dk, int Dv, int dtype, std::initializer_list<const void*> tensors);
// cott_scan on the tensor cores: 16-bit dtypes, head dims that are multiples of 64 (up to 256), 16-byte aligned
// tensors, in place only at head dim 64.
bool scan_tc_usable(int Dk, int Dv, int dtype, const void* q, const void* k, const void* v, const void* out);
int launch_scan_tc(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk, int Dv, int dtype,
                   int reversed, cudaStream_t stream);
int launch_bidir_fwd_tc(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc,
                        void* out, int B, int H, int N, int dtype, cudaStream_t stream, const cott_layout* layout = nullptr);
int launch_bidir_bwd_tc(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc,
                        const void* dout, void* dq, void* dk, void* dv, float* dnorm, int B, int H, int N, int dtype,
                        cudaStream_t stream, const cott_layout* layout = nullptr);

}  // namespace cott
