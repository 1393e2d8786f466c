/*
 * cottention_b200 -- C ABI of the B200 (sm_100a) cosine linear attention kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t / CUstream passed as void*; NULL = the legacy default stream),
 * launches asynchronously on that stream, and returns 0 (COTT_OK) or a COTT_ERR_*
 * code.  Nothing throws, nothing takes or returns a torch type.  After a non-zero
 * return, cott_last_error() gives a message for the calling thread.
 *
 * All tensors are dense row-major [B, H, N, D] (batch, heads, sequence, head dim;
 * the reference's C++ names the same axes N, H, S, D).  Q and K have head dim Dk
 * ("D_attn"), V and the output have Dv ("D_value").
 *
 * "Reference" in the comments below is gmongaras/Cottention_Transformer; paths are
 * relative to that project.
 */
#ifndef COTTENTION_B200_H_
#define COTTENTION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types; the numbering is part of the ABI */
enum { COTT_F32 = 0, COTT_F64 = 1, COTT_F16 = 2, COTT_BF16 = 3 };

/* status codes */
enum {
  COTT_OK = 0,
  COTT_ERR_NULL = 1,        /* a required pointer is NULL                                   */
  COTT_ERR_SHAPE = 2,       /* a size is out of the supported range                         */
  COTT_ERR_DTYPE = 3,       /* unknown or unsupported element type for this entry point     */
  COTT_ERR_CUDA = 4,        /* a CUDA runtime/driver call failed (message has the CUDA text) */
  COTT_ERR_ALIGN = 5,       /* a pointer is not 16-byte aligned                             */
  COTT_ERR_DEVICE_WAIT = 6, /* a bounded device-side wait gave up (reported by cott_check_status) */
  COTT_ERR_UNSUPPORTED = 7  /* valid request that this build has no kernel for              */
};

/* Library / build identification: "cottention_b200 <version> sm_100a". */
const char* cott_version(void);
/* Message for the last non-zero status returned to the calling thread ("" if none). */
const char* cott_last_error(void);
/* Text for a status code. */
const char* cott_status_string(int status);

/*
 * The scan.  out[b,h,s,:] = sum_{t<=s} (Q[b,h,s,:] . K[b,h,t,:]) V[b,h,t,:]   (t>=s when reversed)
 *
 * Replaces forward_<T> -> kernel_call<T> -> kernel_mod_2/4<T,32> of
 * Cuda_Kernel/combined_kernel_general.cu:96-289,352-429, i.e. what the pybind entry
 * points FastAttention2.kernel.{float32,float64,float16,bfloat16} (:444-454) run.
 * Unlike the reference (which accumulates in the storage type, :121,133) sums are
 * kept in fp32 (fp64 for COTT_F64).  Constraints: Dk % 16 == 0, 16 <= Dk <= 256
 * (the reference: D_attn % 16 == 0, D_attn >= 32, :372-374), Dv >= 1, N >= 0.
 * `out` may alias `v` (the reference's inplace=true, :403-404) only if Dv <= 16.
 */
int cott_scan(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk,
              int Dv, int dtype, int reversed, void* stream);

/*
 * Gradients of the scan: the three permuted scans of CustomAttention.backward,
 * Cuda_Kernel/Custom_Kernel.py:106-108
 *   dq = scan(dout, v, k, fwd)   dk = scan(v, dout, q, rev)   dv = scan(k, q, dout, rev)
 * issued on `stream` in that order.  Dv must satisfy the Dk constraints too (V and
 * dout take the Q/K role in two of the scans).
 */
int cott_scan_bwd(const void* q, const void* k, const void* v, const void* dout, void* dq, void* dk,
                  void* dv, int B, int H, int N, int Dk, int Dv, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* COTTENTION_B200_H_ */
