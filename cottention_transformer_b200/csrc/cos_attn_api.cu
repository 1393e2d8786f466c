// C ABI of the fused cosine-attention operators (tensor-core path).
#include "bidir_tc.cuh"
#include "causal_bwd_fused.cuh"
#include "causal_seg.cuh"
#include "causal_tc.cuh"
#include "causal_wide.cuh"
#include "common.cuh"

#include <initializer_list>
#include <mutex>
#include <utility>

using namespace cott;

namespace {

int check_fused_args(int B, int H, int N, int Dk, int Dv, int dtype) {
  if (dtype != COTT_BF16 && dtype != COTT_F16)
    return fail(COTT_ERR_DTYPE,
                "the fused tensor-core path takes float16/bfloat16 (dtype code %d given); float32/float64 go "
                "through cott_scan", dtype);
  if (B < 0 || H < 0 || N < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d N=%d", B, H, N);
  if (Dk != kTcD || Dv != kTcD)
    return fail(COTT_ERR_UNSUPPORTED, "the fused tensor-core path is built for head dim 64 (got Dk=%d Dv=%d)", Dk, Dv);
  if ((long)B * H > 0x7fffffffL) return fail(COTT_ERR_SHAPE, "B*H too large");
  return COTT_OK;
}

int aligned16(const void* p, const char* name) {
  if (reinterpret_cast<uintptr_t>(p) & 15) return fail(COTT_ERR_ALIGN, "%s must be 16-byte aligned", name);
  return COTT_OK;
}

int tmap(CUtensorMap* m, const void* p, int dtype, long B, long H, long N, TileStrides st) {
  if ((st.b | st.h | st.n) & 7 || st.b <= 0 || st.h <= 0 || st.n <= 0)
    return fail(COTT_ERR_ALIGN, "tensor strides must be positive multiples of 8 elements (got %lld, %lld, %lld)", st.b, st.h, st.n);
  int r = make_tmap_rows64(m, p, dtype == COTT_BF16, B, H, N, st, kTcChunk);
  if (r == 1) return fail(COTT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (r) return fail(COTT_ERR_CUDA, "cuTensorMapEncodeTiled failed: CUresult %d (ptr %p, B %ld, H %ld, N %ld)", r - 100, p, B, H, N);
  return COTT_OK;
}

// One segment (`nseg` = 1, `init` = nullptr) or segment-parallel: gridDim.y = nseg CTAs per (b, h), each starting
// from init[bh][seg].
struct SegPlan {
  int nseg = 1;  // segments actually launched
  int cps = 0;   // chunks per segment
  const unsigned char* keep = nullptr;  // padding: [B, N] keep flags and their inclusive running count, or both null
  const int* count = nullptr;
  TileStrides in{0, 0, 0}, out{0, 0, 0};  // strides of q, k, v, dq, dk, dv / of out, dout; all zero = contiguous [B,H,N,64]
  RotArgs rot{nullptr, nullptr, 0, 0};    // rotary embedding of q, k inside the kernels (one segment only), or sin = null
  // The caller has already zeroed the norm_const gradient on the stream, before the dQ launch: a memset between the dQ
  // and the dK/dV launch would end the chain of programmatic dependent launches (the dK/dV kernel could not set itself
  // up while the dQ kernel drains).
  bool dnorm_zeroed = false;
};
TileStrides in_strides(const SegPlan& p, long H, long N) { return p.in.n ? p.in : contiguous_bhnd(H, N); }
TileStrides out_strides(const SegPlan& p, long H, long N) { return p.out.n ? p.out : contiguous_bhnd(H, N); }
SegPlan plan_segments(int N, int nseg_requested) {
  const int total = (N + kTcChunk - 1) / kTcChunk;
  SegPlan p;
  const int want = nseg_requested < 1 ? 1 : (nseg_requested > total ? total : nseg_requested);
  p.cps = (total + want - 1) / want;
  p.nseg = (total + p.cps - 1) / p.cps;
  return p;
}

template <typename T>
int launch_fwd(const void* q, const void* k, const void* v, const float* nc, void* out, int B, int H, int N,
               int dtype, cudaStream_t stream, const float* init = nullptr, SegPlan plan = SegPlan(), void* saved = nullptr) {
  const long BH = (long)B * H;
  CUtensorMap mq, mk, mv, mo;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mk, k, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mv, v, dtype, B, H, N, in_strides(plan, H, N))) ||
      (st = tmap(&mo, out, dtype, B, H, N, out_strides(plan, H, N))))
    return st;
  const bool ext = plan.nseg > 1 || init || plan.keep;
  auto kern = plan.rot.sin ? causal_tc_kernel<T, kModeFwd, true, false, true>
              : saved      ? (ext ? causal_tc_kernel<T, kModeFwd, true, true> : causal_tc_kernel<T, kModeFwd, false, true>)
                           : (ext ? causal_tc_kernel<T, kModeFwd, true, false> : causal_tc_kernel<T, kModeFwd, false, false>);
  const size_t smem = causal_tc_smem_bytes(kModeFwd);
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (plan.cps == 0) plan.cps = plan_segments(N, 1).cps;
  COTT_CUDA_TRY(launch_pdl(kern, dim3((unsigned)BH, plan.nseg), kTcThreads, smem, stream, mq, mk, mv, mq, mo, nc, H, N, init, plan.cps,
                           plan.keep, plan.count, static_cast<uint4*>(saved), plan.rot));
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

template <typename T>
int launch_bwd_dq(const void* q, const void* k, const void* v, const float* nc, const void* dout, void* dq, int B,
                  int H, int N, int dtype, cudaStream_t stream, const float* init = nullptr, SegPlan plan = SegPlan()) {
  const long BH = (long)B * H;
  CUtensorMap mq, mk, mv, md, mo;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mk, k, dtype, B, H, N, in_strides(plan, H, N))) ||
      (st = tmap(&mv, v, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&md, dout, dtype, B, H, N, out_strides(plan, H, N))) ||
      (st = tmap(&mo, dq, dtype, B, H, N, in_strides(plan, H, N))))
    return st;
  const bool ext = plan.nseg > 1 || init || plan.keep;
  auto kern = plan.rot.sin ? causal_tc_kernel<T, kModeDq, true, false, true>
                           : (ext ? causal_tc_kernel<T, kModeDq, true> : causal_tc_kernel<T, kModeDq, false>);
  const size_t smem = causal_tc_smem_bytes(kModeDq);
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (plan.cps == 0) plan.cps = plan_segments(N, 1).cps;
  COTT_CUDA_TRY(launch_pdl(kern, dim3((unsigned)BH, plan.nseg), kTcThreads, smem, stream, md, mv, mk, mq, mo, nc, H, N, init, plan.cps,
                           plan.keep, plan.count, static_cast<uint4*>(nullptr), plan.rot));
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

template <typename T>
int launch_bwd_dkdv(const void* q, const void* k, const void* v, const float* nc, const void* dout, void* dk,
                    void* dv, float* dnorm, int B, int H, int N, int dtype, cudaStream_t stream,
                    const float* init = nullptr, SegPlan plan = SegPlan()) {
  const long BH = (long)B * H;
  CUtensorMap mq, mk, mv, md, mdk, mdv;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mk, k, dtype, B, H, N, in_strides(plan, H, N))) ||
      (st = tmap(&mv, v, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&md, dout, dtype, B, H, N, out_strides(plan, H, N))) ||
      (st = tmap(&mdk, dk, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mdv, dv, dtype, B, H, N, in_strides(plan, H, N))))
    return st;
  if (!plan.dnorm_zeroed) COTT_CUDA_TRY(cudaMemsetAsync(dnorm, 0, sizeof(float) * H, stream));
  const bool ext = plan.nseg > 1 || init || plan.keep;
  auto kern = plan.rot.sin ? causal_bwd_kv_kernel<T, true, true>
                           : (ext ? causal_bwd_kv_kernel<T, true> : causal_bwd_kv_kernel<T, false>);
  const size_t smem = causal_bwd_kv_smem_bytes();
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (plan.cps == 0) plan.cps = plan_segments(N, 1).cps;
  COTT_CUDA_TRY(launch_pdl(kern, dim3((unsigned)BH, plan.nseg), plan.rot.sin ? kKvThreadsRot : kKvThreads, smem, stream, mq, mk, mv, md, mdk,
                           mdv, dnorm, nc, H, N, init, plan.cps, plan.keep, plan.count, plan.rot));
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

// The one-pass backward: `saved` holds the forward's 16-bit state before every chunk ([B*H][chunks][64][64]).
template <typename T>
int launch_bwd_fused(const void* q, const void* k, const void* v, const float* nc, const void* dout, const void* saved,
                     void* dq, void* dk, void* dv, float* dnorm, int B, int H, int N, int dtype, cudaStream_t stream,
                     const float* init = nullptr, SegPlan plan = SegPlan()) {
  const long BH = (long)B * H;
  const long rows = (long)((N + kTcChunk - 1) / kTcChunk) * kTcD;  // state rows per (b, h)
  CUtensorMap mq, mk, mv, md, ms, mdq, mdk, mdv;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mk, k, dtype, B, H, N, in_strides(plan, H, N))) ||
      (st = tmap(&mv, v, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&md, dout, dtype, B, H, N, out_strides(plan, H, N))) ||
      (st = tmap(&mdq, dq, dtype, B, H, N, in_strides(plan, H, N))) || (st = tmap(&mdk, dk, dtype, B, H, N, in_strides(plan, H, N))) ||
      (st = tmap(&mdv, dv, dtype, B, H, N, in_strides(plan, H, N))))
    return st;
  int r = make_tmap_rows64(&ms, saved, dtype == COTT_BF16, B, H, rows, contiguous_bhnd(H, rows), kTcD);
  if (r) return fail(COTT_ERR_CUDA, "cuTensorMapEncodeTiled failed for the saved states: %d", r);
  COTT_CUDA_TRY(cudaMemsetAsync(dnorm, 0, sizeof(float) * H, stream));
  const bool ext = plan.nseg > 1 || init || plan.keep;
  auto kern = ext ? causal_bwd_fused_kernel<T, true> : causal_bwd_fused_kernel<T, false>;
  const size_t smem = causal_bwd_fused_smem_bytes();
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if (plan.cps == 0) plan.cps = plan_segments(N, 1).cps;
  kern<<<dim3((unsigned)BH, plan.nseg), kBwThreads, smem, stream>>>(mq, mk, mv, md, ms, mdq, mdk, mdv, dnorm, nc, H, N, init, plan.cps,
                                                                   plan.keep, plan.count);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

// state[bh][seg] of every segment: Y^T Z with one operand row-scaled (see seg_state_kernel)
template <typename T, int MODE>
int launch_seg_state(const void* y, const void* z, TileStrides sy, TileStrides sz, const float* nc, float* state, int B,
                     int H, int N, int dtype, SegPlan plan, cudaStream_t stream) {
  const long BH = (long)B * H;
  CUtensorMap my, mz;
  int st;
  if ((st = tmap(&my, y, dtype, B, H, N, sy)) || (st = tmap(&mz, z, dtype, B, H, N, sz))) return st;
  auto kern = seg_state_kernel<T, MODE>;
  const size_t smem = seg_state_smem_bytes();
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)BH, plan.nseg), kSegThreads, smem, stream>>>(my, mz, nc, state, H, N, plan.cps, plan.keep, plan.count);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

// workspace of the segment-parallel path: five arrays of B*H*nseg fp32 [64 x 64] matrices
//   0 forward segment states | 1 their exclusive prefix | 2 the prefix transposed | 3 reverse segment states |
//   4 their exclusive suffix
size_t seg_array_floats(int B, int H, int nseg) { return (size_t)B * H * nseg * kTcD * kTcD; }

void apply_layout(SegPlan& plan, const cott_layout* l) {
  if (!l) return;
  plan.in = TileStrides{l->in_b, l->in_h, l->in_n};
  plan.out = TileStrides{l->out_b, l->out_h, l->out_n};
}

template <typename T>
int run_fwd_seg(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, void* out,
                float* ws, int nseg, const cott_layout* layout, int B, int H, int N, int dtype, cudaStream_t stream,
                void* saved = nullptr, RotArgs rot = RotArgs{nullptr, nullptr, 0, 0}) {
  SegPlan plan = plan_segments(N, nseg);
  apply_layout(plan, layout);
  plan.rot = rot;
  const size_t A = seg_array_floats(B, H, plan.nseg);
  if (keep) {  // running count of the kept positions, behind the five state arrays
    int* count = reinterpret_cast<int*>(ws + 5 * A);
    keep_count_kernel<<<(unsigned)B, 256, 0, stream>>>(keep, count, N);
    COTT_CUDA_TRY(cudaGetLastError());
    plan.keep = keep;
    plan.count = count;
  }
  if (plan.nseg == 1) return launch_fwd<T>(q, k, v, nc, out, B, H, N, dtype, stream, nullptr, plan, saved);
  int st = launch_seg_state<T, kSegFwdState>(k, v, in_strides(plan, H, N), in_strides(plan, H, N), nc, ws, B, H, N, dtype, plan, stream);
  if (st) return st;
  seg_scan_kernel<<<(unsigned)((long)B * H), 256, 0, stream>>>(ws, ws + A, ws + 2 * A, nullptr, plan.nseg);
  COTT_CUDA_TRY(cudaGetLastError());
  return launch_fwd<T>(q, k, v, nc, out, B, H, N, dtype, stream, ws + A, plan, saved);
}

template <typename T>
int run_bwd_seg(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, const void* dout,
                float* ws, int nseg, const cott_layout* layout, void* dq, void* dk, void* dv, float* dnorm, int B, int H,
                int N, int dtype, cudaStream_t stream, RotArgs rot = RotArgs{nullptr, nullptr, 0, 0}) {
  SegPlan plan = plan_segments(N, nseg);
  apply_layout(plan, layout);
  plan.rot = rot;
  const size_t A = seg_array_floats(B, H, plan.nseg);
  if (keep) {  // the forward call left the running count in the workspace
    plan.keep = keep;
    plan.count = reinterpret_cast<const int*>(ws + 5 * A);
  }
  if (plan.nseg == 1) {
    COTT_CUDA_TRY(cudaMemsetAsync(dnorm, 0, sizeof(float) * H, stream));
    plan.dnorm_zeroed = true;
    int st = launch_bwd_dq<T>(q, k, v, nc, dout, dq, B, H, N, dtype, stream, nullptr, plan);
    return st ? st : launch_bwd_dkdv<T>(q, k, v, nc, dout, dk, dv, dnorm, B, H, N, dtype, stream, nullptr, plan);
  }
  // dQ: the forward prefix states, transposed (written by the forward call into the same workspace)
  int st = launch_bwd_dq<T>(q, k, v, nc, dout, dq, B, H, N, dtype, stream, ws + 2 * A, plan);
  if (st) return st;
  // dK, dV: reverse states of the segments, their exclusive suffix
  if ((st = launch_seg_state<T, kSegRevState>(q, dout, in_strides(plan, H, N), out_strides(plan, H, N), nc, ws + 3 * A, B, H, N, dtype, plan,
                                              stream))) return st;
  seg_scan_kernel<<<(unsigned)((long)B * H), 256, 0, stream>>>(ws + 3 * A, nullptr, nullptr, ws + 4 * A, plan.nseg);
  COTT_CUDA_TRY(cudaGetLastError());
  return launch_bwd_dkdv<T>(q, k, v, nc, dout, dk, dv, dnorm, B, H, N, dtype, stream, ws + 4 * A, plan);
}

// The time-out path of the tensor-core kernels on its own: one CTA sets up what those kernels set up (an
// mbarrier, a TMEM allocation), three of its warps wait -- with the same bounded wait, a few polls long -- on a
// barrier phase that nothing ever completes, and the CTA then leaves the way the kernels leave after a time-out:
// status word written once, every role out of its loop, TMEM handed back.  Nothing faults and nothing spins
// without a limit; the launch ends after about `polls` x 0.2 ms.
__global__ void __launch_bounds__(128, 1) wait_selftest_kernel(int polls, int code, int chunk) {
  using namespace ptx;
  __shared__ uint64_t bar_never, bar_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar_never, 1);
    mbar_init(&bar_done, 1);
    mbar_fence_init();
    abort_flag_s = 0;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (warp == 0) {
    // the role whose wait runs out: it raises the abort flag and records (code << 16 | chunk)
    wait_bar_warp(&bar_never, 0, abort_flag, code, chunk, static_cast<uint32_t>(polls));
  } else if (warp >= 2) {
    // roles waiting for something else (with the full limit) must notice the abort flag and leave too
    wait_bar_warp(&bar_done, 0, abort_flag, code + 1, chunk);
  }
  (void)lane;
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 32);
}

// ---- head dim 128: causal_wide.cuh ----------------------------------------------------------------------------
struct WideTensors {  // X, Y: [B,H,N,128]; Z, C, out: [B,H,N,dz] (dz a multiple of 64), all dense
  const void *x, *y, *z, *c;
  void* out;
  int dz;
};
inline TileStrides dense_rows(long H, long N, long D) { return TileStrides{H * N * D, N * D, D}; }

template <typename T, bool REV, bool NORMS, bool STATE_ONLY>
int launch_wide_t(const WideTensors& t, WideArgs a, int B, int H, int N, int dtype, int nseg, cudaStream_t stream) {
  CUtensorMap mx, my, mz, mo;
  const int bf = dtype == COTT_BF16;
  int r;
  const void* xs = t.x ? t.x : t.y;  // STATE_ONLY launches have no X
  if ((r = make_tmap_rows64(&mx, xs, bf, B, H, N, dense_rows(H, N, 128), kTcChunk, 128)) ||
      (r = make_tmap_rows64(&my, t.y, bf, B, H, N, dense_rows(H, N, 128), kTcChunk, 128)) ||
      (r = make_tmap_rows64(&mz, t.z, bf, B, H, N, dense_rows(H, N, t.dz), kTcChunk, t.dz)) ||
      (r = make_tmap_rows64(&mo, t.out ? t.out : t.z, bf, B, H, N, dense_rows(H, N, t.dz), kTcChunk, t.dz)))
    return fail(COTT_ERR_CUDA, "cuTensorMapEncodeTiled failed for a head-dim-128 tensor: %d", r);
  a.c = t.c;
  a.dz = t.dz;
  a.H = H;
  a.N = N;
  auto kern = wide_kernel<T, REV, NORMS, STATE_ONLY>;
  const size_t smem = wide_smem_bytes();
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)((long)B * H), t.dz / 64, nseg), kWdThreads, smem, stream>>>(mx, my, mz, mo, a);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

// One scan-type pass over head-dim-128 tensors, cut into `nseg` segments per sequence when nseg > 1: the segments'
// own states (STATE_ONLY launch), their exclusive prefix in scan order, then the pass itself.  `ws`: 2 x B*H*(dz/64)*nseg
// fp32 [128 x 64] matrices (only touched when nseg > 1).
// `given_prefix`: the prefix states are already there (a transposed copy of another pass's), skip the state-only launch.
// After the call ws + A holds the prefix states this pass ran with (A = units * nseg matrices).
template <typename T, bool REV, bool NORMS>
int run_wide(const WideTensors& t, WideArgs a, int B, int H, int N, int dtype, int nseg_requested, float* ws, cudaStream_t stream,
             const float* given_prefix = nullptr) {
  const SegPlan plan = plan_segments(N, nseg_requested);
  a.chunks_per_seg = plan.cps;
  a.init_state = nullptr;
  a.state_out = nullptr;
  if (plan.nseg > 1 && given_prefix) {
    a.init_state = given_prefix;
  } else if (plan.nseg > 1) {
    const size_t units = (size_t)B * H * (t.dz / 64);
    const size_t A = units * plan.nseg * (size_t)(kTcChunk * kTcD);
    WideArgs sa = a;
    sa.state_out = ws;
    sa.eps = nullptr;
    sa.rq_out = sa.rk_out = sa.w_out = nullptr;
    WideTensors st = t;
    st.x = nullptr, st.c = nullptr, st.out = nullptr;
    int r = launch_wide_t<T, REV, NORMS, true>(st, sa, B, H, N, dtype, plan.nseg, stream);
    if (r) return r;
    seg_prefix_kernel<<<dim3((unsigned)units, 8), 256, 0, stream>>>(ws, ws + A, plan.nseg, kTcChunk * kTcD);
    COTT_CUDA_TRY(cudaGetLastError());
    a.init_state = ws + A;
  }
  return launch_wide_t<T, REV, NORMS, false>(t, a, B, H, N, dtype, plan.nseg, stream);
}

size_t wide_ws_floats(int B, int H, int N, int dz, int nseg) {
  return 2 * (size_t)B * H * (dz / 64) * plan_segments(N, nseg).nseg * (size_t)(kTcChunk * kTcD);
}

int wide_seg_count(int B, int H, int N, int dz) {
  const long units = (long)B * H * (dz / 64);
  const int total = (N + kTcChunk - 1) / kTcChunk;
  if (units <= 0 || total < 4) return 1;
  int sm = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  long nseg = sm / units;
  if (nseg > total / 2) nseg = total / 2;
  return nseg < 2 ? 1 : (int)nseg;
}

// workspace of the fused head-dim-128 pair: six fp32 vectors [B*H*N] (1/|q|, 1/|k|, keep a/|k|, -q^.dq^/|q|^2, eps,
// -eps/|k|^2), the running keep count [B*N], then the segment states
struct WideWs {
  float *rq, *rk, *w, *cq, *eps, *ck;
  int* count;
  float* seg;      // 2 x A floats: the segments' own states and their prefix, of the pass that is running
  float* seg_fwd;  // A floats: the forward's prefix states (the backward transposes them for dq)
  float* seg_t;    // A floats: a transposed prefix for the pass that is running
};
WideWs wide_ws(void* workspace, int B, int H, int N) {
  const size_t V = (size_t)B * H * N;
  float* f = static_cast<float*>(workspace);
  WideWs s{f, f + V, f + 2 * V, f + 3 * V, f + 4 * V, f + 5 * V, reinterpret_cast<int*>(f + 6 * V), nullptr, nullptr, nullptr};
  const size_t cnt = ((size_t)B * N + 3) & ~(size_t)3;
  const size_t A = wide_ws_floats(B, H, N, 128, wide_seg_count(B, H, N, 128)) / 2;
  s.seg = f + 6 * V + cnt;
  s.seg_fwd = s.seg + 2 * A;
  s.seg_t = s.seg_fwd + A;
  return s;
}

template <typename T>
int run_wide_fwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, void* out, void* workspace,
                 int B, int H, int N, int dtype, cudaStream_t stream) {
  WideWs ws = wide_ws(workspace, B, H, N);
  WideArgs a = {};
  a.norm_const = nc;
  a.rq_out = ws.rq, a.rk_out = ws.rk, a.w_out = ws.w;
  if (keep) {
    keep_count_kernel<<<(unsigned)B, 256, 0, stream>>>(keep, ws.count, N);
    COTT_CUDA_TRY(cudaGetLastError());
    a.keep = keep, a.count = ws.count;
  }
  WideTensors t{q, k, v, nullptr, out, 128};
  const int nseg = plan_segments(N, wide_seg_count(B, H, N, 128)).nseg;
  int st = run_wide<T, false, true>(t, a, B, H, N, dtype, nseg, ws.seg, stream);
  if (st == COTT_OK && nseg > 1) {  // the backward's dq pass starts its segments from the transposes of these
    const size_t A = wide_ws_floats(B, H, N, 128, nseg) / 2;
    COTT_CUDA_TRY(cudaMemcpyAsync(ws.seg_fwd, ws.seg + A, A * sizeof(float), cudaMemcpyDeviceToDevice, stream));
  }
  return st;
}

template <typename T>
int run_wide_bwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, const void* out, const void* dout,
                 void* workspace, void* dq, void* dk, void* dv, float* dnorm, int B, int H, int N, int dtype, cudaStream_t stream) {
  WideWs ws = wide_ws(workspace, B, H, N);
  const long rows = (long)B * H * N;
  const int nseg = plan_segments(N, wide_seg_count(B, H, N, 128)).nseg;
  const size_t A = wide_ws_floats(B, H, N, 128, nseg) / 2;
  const dim3 tgrid((unsigned)((long)B * H), (unsigned)nseg, 8);
  // -q^.dq^ / |q|^2 from q^_t . dq^_t = dO_t . O_t
  rowdot_coef_kernel<T><<<(unsigned)((rows * 16 + 255) / 256), 256, 0, stream>>>(static_cast<const T*>(dout), static_cast<const T*>(out), ws.rq,
                                                                                ws.cq, rows);
  COTT_CUDA_TRY(cudaGetLastError());
  int st;
  {  // dq = rq scan(dO, V, diag(w) K) + cq q                      (Custom_Kernel.py:106 with the module math around it)
    WideArgs a = {};
    a.zscale = ws.w, a.oscale = ws.rq, a.ccoef = ws.cq;
    WideTensors t{dout, v, k, q, dq, 128};
    if (nseg > 1) {  // sum_s v_s (x) w_s k_s is the transpose of the forward's sum_s k_s (x) w_s v_s
      seg_transpose_kernel<<<tgrid, 256, 0, stream>>>(ws.seg_fwd, ws.seg_t, nseg);
      COTT_CUDA_TRY(cudaGetLastError());
    }
    if ((st = run_wide<T, false, false>(t, a, B, H, N, dtype, nseg, ws.seg, stream, nseg > 1 ? ws.seg_t : nullptr))) return st;
  }
  COTT_CUDA_TRY(cudaMemsetAsync(ws.eps, 0, sizeof(float) * rows, stream));
  COTT_CUDA_TRY(cudaMemsetAsync(dnorm, 0, sizeof(float) * H, stream));
  {  // dv = w scan_rev(K, diag(rq) Q, dO);  eps = v' . dv'          (:108)
    WideArgs a = {};
    a.yscale = ws.rq, a.oscale = ws.w, a.eps = ws.eps;
    WideTensors t{k, q, dout, v, dv, 128};
    if ((st = run_wide<T, true, false>(t, a, B, H, N, dtype, nseg, ws.seg, stream))) return st;
  }
  eps_coef_kernel<<<dim3((unsigned)((long)B * H), (unsigned)((N + 1023) / 1024)), 256, 0, stream>>>(ws.eps, ws.rk, ws.ck, nc, dnorm,
                                                                                                 keep ? ws.count : nullptr, H, N);
  COTT_CUDA_TRY(cudaGetLastError());
  {  // dk = w scan_rev(V, dO, diag(rq) Q) + ck k                    (:107)
    WideArgs a = {};
    a.zscale = ws.rq, a.oscale = ws.w, a.ccoef = ws.ck;
    WideTensors t{v, dout, q, k, dk, 128};
    if (nseg > 1) {  // sum_t dO_t (x) q^_t is the transpose of the dv pass's sum_t q^_t (x) dO_t (its prefix is still in ws.seg + A)
      seg_transpose_kernel<<<tgrid, 256, 0, stream>>>(ws.seg + A, ws.seg_t, nseg);
      COTT_CUDA_TRY(cudaGetLastError());
    }
    if ((st = run_wide<T, true, false>(t, a, B, H, N, dtype, nseg, ws.seg, stream, nseg > 1 ? ws.seg_t : nullptr))) return st;
  }
  return COTT_OK;
}

template <typename T>
int run_bwd_train(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc, const void* dout,
                  const void* saved, float* ws, int nseg, const cott_layout* layout, void* dq, void* dk, void* dv, float* dnorm,
                  int B, int H, int N, int dtype, cudaStream_t stream) {
  SegPlan plan = plan_segments(N, nseg);
  apply_layout(plan, layout);
  const size_t A = seg_array_floats(B, H, plan.nseg);
  if (keep) {  // the forward call left the running count in the workspace
    plan.keep = keep;
    plan.count = reinterpret_cast<const int*>(ws + 5 * A);
  }
  if (plan.nseg == 1) return launch_bwd_fused<T>(q, k, v, nc, dout, saved, dq, dk, dv, dnorm, B, H, N, dtype, stream, nullptr, plan);
  // reverse states of the segments and their exclusive suffix; the prefix states come from `saved`
  int st = launch_seg_state<T, kSegRevState>(q, dout, in_strides(plan, H, N), out_strides(plan, H, N), nc, ws + 3 * A, B, H, N, dtype, plan,
                                             stream);
  if (st) return st;
  seg_scan_kernel<<<(unsigned)((long)B * H), 256, 0, stream>>>(ws + 3 * A, nullptr, nullptr, ws + 4 * A, plan.nseg);
  COTT_CUDA_TRY(cudaGetLastError());
  return launch_bwd_fused<T>(q, k, v, nc, dout, saved, dq, dk, dv, dnorm, B, H, N, dtype, stream, ws + 4 * A, plan);
}

int check_ptrs16(std::initializer_list<std::pair<const void*, const char*>> ps) {
  for (auto& p : ps) {
    if (!p.first) return fail(COTT_ERR_NULL, "null pointer: %s", p.second);
    int st = aligned16(p.first, p.second);
    if (st) return st;
  }
  return COTT_OK;
}

template <typename T>
int launch_bidir_fwd_tc_t(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc,
                          void* out, int B, int H, int N, int dtype, cudaStream_t stream, TileStrides si, TileStrides so) {
  const long BH = (long)B * H;
  CUtensorMap mq, mk, mv, mo;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, si)) || (st = tmap(&mk, k, dtype, B, H, N, si)) || (st = tmap(&mv, v, dtype, B, H, N, si)) ||
      (st = tmap(&mo, out, dtype, B, H, N, so)))
    return st;
  auto kern = bidir_fwd_tc_kernel<T>;
  const size_t smem = bidir_fwd_tc_smem_bytes();
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)BH, kBtcThreads, smem, stream>>>(mq, mk, mv, mo, keep, nc, H, N);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

template <typename T>
int launch_bidir_bwd_tc_t(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc,
                          const void* dout, void* dq, void* dk, void* dv, float* dnorm, int B, int H, int N, int dtype,
                          cudaStream_t stream, TileStrides si, TileStrides so) {
  const long BH = (long)B * H;
  CUtensorMap mq, mk, mv, md, mdq, mdk, mdv;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, si)) || (st = tmap(&mk, k, dtype, B, H, N, si)) || (st = tmap(&mv, v, dtype, B, H, N, si)) ||
      (st = tmap(&md, dout, dtype, B, H, N, so)) || (st = tmap(&mdq, dq, dtype, B, H, N, si)) || (st = tmap(&mdk, dk, dtype, B, H, N, si)) ||
      (st = tmap(&mdv, dv, dtype, B, H, N, si)))
    return st;
  COTT_CUDA_TRY(cudaMemsetAsync(dnorm, 0, sizeof(float) * H, stream));
  auto kern = bidir_bwd_tc_kernel<T>;
  const size_t smem = bidir_bwd_tc_smem_bytes();
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // persistent: one CTA per SM, each takes every gridDim.x-th sequence
  int dev = 0, sm = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  const unsigned grid = (unsigned)(BH < sm ? BH : sm);
  kern<<<grid, kBtcBwdThreads, smem, stream>>>(mq, mk, mv, md, mdq, mdk, mdv, keep, nc, dnorm, H, N, (int)BH);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

}  // namespace

namespace cott {

int launch_bidir_bwd_tc(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc,
                        const void* dout, void* dq, void* dk, void* dv, float* dnorm, int B, int H, int N, int dtype,
                        cudaStream_t stream, const cott_layout* l) {
  const TileStrides si = l ? TileStrides{l->in_b, l->in_h, l->in_n} : contiguous_bhnd(H, N);
  const TileStrides so = l ? TileStrides{l->out_b, l->out_h, l->out_n} : contiguous_bhnd(H, N);
  return dtype == COTT_BF16
             ? launch_bidir_bwd_tc_t<__nv_bfloat16>(q, k, v, keep, nc, dout, dq, dk, dv, dnorm, B, H, N, dtype, stream, si, so)
             : launch_bidir_bwd_tc_t<__half>(q, k, v, keep, nc, dout, dq, dk, dv, dnorm, B, H, N, dtype, stream, si, so);
}

// The bare scan of cott_scan on the tensor cores (head dim 64, 16-bit dtypes): the forward kernel without its row
// scalings, walking the sequence backwards when `reversed`.  `out` may be one of the inputs: a chunk's rows are
// stored after every load of that chunk has completed, and no other chunk reads them.
// `ws` (2 x B*H*nseg fp32 [64 x 64] matrices) is only used when plan.nseg > 1: the segments' own states and their
// exclusive prefix in scan order.
template <typename T>
int launch_scan_tc_t(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int dtype, int reversed,
                     cudaStream_t stream, TileStrides sqk, TileStrides sv, TileStrides so, SegPlan plan, float* ws) {
  CUtensorMap mq, mk, mv, mo;
  int st;
  if ((st = tmap(&mq, q, dtype, B, H, N, sqk)) || (st = tmap(&mk, k, dtype, B, H, N, sqk)) || (st = tmap(&mv, v, dtype, B, H, N, sv)) ||
      (st = tmap(&mo, out, dtype, B, H, N, so)))
    return st;
  const float* init = nullptr;
  if (plan.nseg > 1) {
    const size_t A = seg_array_floats(B, H, plan.nseg);
    st = reversed ? launch_seg_state<T, kSegRawStateRev>(k, v, sqk, sv, nullptr, ws, B, H, N, dtype, plan, stream)
                  : launch_seg_state<T, kSegRawState>(k, v, sqk, sv, nullptr, ws, B, H, N, dtype, plan, stream);
    if (st) return st;
    seg_scan_kernel<<<(unsigned)((long)B * H), 256, 0, stream>>>(ws, ws + A, nullptr, nullptr, plan.nseg);
    COTT_CUDA_TRY(cudaGetLastError());
    init = ws + A;
  }
  auto kern = plan.nseg > 1 ? (reversed ? causal_tc_kernel<T, kModeScanRev, true> : causal_tc_kernel<T, kModeScan, true>)
                            : (reversed ? causal_tc_kernel<T, kModeScanRev, false> : causal_tc_kernel<T, kModeScan, false>);
  const size_t smem = causal_tc_smem_bytes(kModeScan);
  COTT_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  COTT_CUDA_TRY(launch_pdl(kern, dim3((unsigned)((long)B * H), plan.nseg), kTcThreads, smem, stream, mq, mk, mv, mq, mo,
                           static_cast<const float*>(nullptr), H, N, init, plan.cps, static_cast<const unsigned char*>(nullptr),
                           static_cast<const int*>(nullptr), static_cast<uint4*>(nullptr), RotArgs{nullptr, nullptr, 0, 0}));
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

// dst[r][0..63] += src[r][0..63] for `rows` rows; dst rows are `dst_stride` elements apart, src is dense.
template <typename T>
__global__ void add_rows64_kernel(T* __restrict__ dst, long dst_stride, const T* __restrict__ src, long rows) {
  const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;  // one 8-element piece per thread
  if (i >= rows * 8) return;
  uint4* d = reinterpret_cast<uint4*>(dst + (i >> 3) * dst_stride + (i & 7) * 8);
  uint4 a = *d;
  const uint4 b = *reinterpret_cast<const uint4*>(src + i * 8);
  uint32_t* x = reinterpret_cast<uint32_t*>(&a);
  const uint32_t* y = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = Pack2<T>::unpack(x[e]), g = Pack2<T>::unpack(y[e]);
    x[e] = Pack2<T>::pack(f.x + g.x, f.y + g.y);
  }
  *d = a;
}

// Head dims that are multiples of 64: the scan is linear in 64-wide slices of the head dimension,
//   scan(q, k, v)[:, J] = sum_I scan(q[:, I], k[:, I], v[:, J]),
// so every (I, J) pair is one launch of the 64-wide kernel on strided views of the tensors; partial results of
// I > 0 go through a stream-ordered scratch buffer and are added in.
// Stream-ordered scratch of the scan comes from a pool of the library's own that keeps what it has been given
// (release threshold = max): the default pool hands memory back at every synchronisation, which turned each
// long-sequence scan into a fresh device allocation.
cudaError_t scratch_pool(cudaMemPool_t* pool) {
  static cudaMemPool_t pools[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    if ((e = cudaMemPoolCreate(&pools[dev], &props)) != cudaSuccess) return e;
    unsigned long long keep = ~0ull;
    if ((e = cudaMemPoolSetAttribute(pools[dev], cudaMemPoolAttrReleaseThreshold, &keep)) != cudaSuccess) return e;
  }
  *pool = pools[dev];
  return cudaSuccess;
}

// Head dim 128 for Q and K: the native kernel (both halves of q, k go into the same score and state accumulators);
// scratch only for the segment states of long sequences with few (batch, head) pairs.
template <typename T>
int launch_scan_tc_128(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dv, int dtype,
                       int reversed, cudaStream_t stream) {
  const int nseg = wide_seg_count(B, H, N, Dv);
  const size_t ws_bytes = nseg > 1 ? wide_ws_floats(B, H, N, Dv, nseg) * sizeof(float) : 0;
  float* ws = nullptr;
  if (ws_bytes) {
    cudaMemPool_t pool;
    COTT_CUDA_TRY(scratch_pool(&pool));
    COTT_CUDA_TRY(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&ws), ws_bytes, pool, stream));
  }
  WideTensors t{q, k, v, nullptr, out, Dv};
  WideArgs a = {};
  const int st = reversed ? run_wide<T, true, false>(t, a, B, H, N, dtype, nseg, ws, stream)
                          : run_wide<T, false, false>(t, a, B, H, N, dtype, nseg, ws, stream);
  if (ws) COTT_CUDA_TRY(cudaFreeAsync(ws, stream));
  return st;
}

template <typename T>
int launch_scan_tc_wide(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk, int Dv, int dtype,
                        int reversed, cudaStream_t stream) {
  if (Dk == 128) return launch_scan_tc_128<T>(q, k, v, out, B, H, N, Dv, dtype, reversed, stream);
  const TileStrides sqk{(long long)H * N * Dk, (long long)N * Dk, Dk}, sv{(long long)H * N * Dv, (long long)N * Dv, Dv};
  const TileStrides dense = contiguous_bhnd(H, N);
  const long rows = (long)B * H * N;
  const T *qq = static_cast<const T*>(q), *kk = static_cast<const T*>(k), *vv = static_cast<const T*>(v);
  T* oo = static_cast<T*>(out);
  // few (batch, head) pairs and a long sequence: several CTAs per sequence, as in the fused path
  const SegPlan plan = plan_segments(N, cott_cos_attn_seg_count(B, H, N));
  const size_t ws_bytes = plan.nseg > 1 ? 2 * seg_array_floats(B, H, plan.nseg) * sizeof(float) : 0;
  const size_t tmp_bytes = Dk > kTcD ? sizeof(T) * rows * kTcD : 0;
  char* scratch = nullptr;  // stream-ordered: segment states, then the partial result of the slices I > 0
  if (ws_bytes + tmp_bytes) {
    cudaMemPool_t pool;
    COTT_CUDA_TRY(scratch_pool(&pool));
    COTT_CUDA_TRY(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&scratch), ws_bytes + tmp_bytes, pool, stream));
  }
  float* ws = reinterpret_cast<float*>(scratch);
  T* tmp = reinterpret_cast<T*>(scratch + ws_bytes);
  int st = COTT_OK;
  for (int j = 0; st == COTT_OK && j < Dv; j += kTcD)
    for (int i = 0; st == COTT_OK && i < Dk; i += kTcD) {
      st = i == 0 ? launch_scan_tc_t<T>(qq, kk, vv + j, oo + j, B, H, N, dtype, reversed, stream, sqk, sv, sv, plan, ws)
                  : launch_scan_tc_t<T>(qq + i, kk + i, vv + j, tmp, B, H, N, dtype, reversed, stream, sqk, sv, dense, plan, ws);
      if (st == COTT_OK && i > 0) {
        add_rows64_kernel<T><<<(unsigned)((rows * 8 + 255) / 256), 256, 0, stream>>>(oo + j, Dv, tmp, rows);
        if (cudaGetLastError() != cudaSuccess) st = fail(COTT_ERR_CUDA, "add_rows64_kernel launch failed");
      }
    }
  if (scratch) COTT_CUDA_TRY(cudaFreeAsync(scratch, stream));
  return st;
}

bool scan_tc_usable(int Dk, int Dv, int dtype, const void* q, const void* k, const void* v, const void* out) {
  if (dtype != COTT_BF16 && dtype != COTT_F16) return false;
  if (Dk % kTcD || Dv % kTcD || Dk > 256 || Dv > 256) return false;
  for (const void* p : {q, k, v, out})
    if (reinterpret_cast<uintptr_t>(p) & 15) return false;
  // in place (out over an input) only for the single 64-wide launch: a wider head re-reads v after writing out
  if ((Dk > kTcD || Dv > kTcD) && (out == q || out == k || out == v)) return false;
  return true;
}

int launch_scan_tc(const void* q, const void* k, const void* v, void* out, int B, int H, int N, int Dk, int Dv, int dtype,
                   int reversed, cudaStream_t stream) {
  return dtype == COTT_BF16 ? launch_scan_tc_wide<__nv_bfloat16>(q, k, v, out, B, H, N, Dk, Dv, dtype, reversed, stream)
                            : launch_scan_tc_wide<__half>(q, k, v, out, B, H, N, Dk, Dv, dtype, reversed, stream);
}

bool bidir_tc_usable(int Dk, int Dv, int dtype, std::initializer_list<const void*> tensors) {
  if (Dk != kTcD || Dv != kTcD || (dtype != COTT_BF16 && dtype != COTT_F16)) return false;
  for (const void* p : tensors)
    if (reinterpret_cast<uintptr_t>(p) & 15) return false;
  return true;
}

int launch_bidir_fwd_tc(const void* q, const void* k, const void* v, const unsigned char* keep, const float* nc,
                        void* out, int B, int H, int N, int dtype, cudaStream_t stream, const cott_layout* l) {
  const TileStrides si = l ? TileStrides{l->in_b, l->in_h, l->in_n} : contiguous_bhnd(H, N);
  const TileStrides so = l ? TileStrides{l->out_b, l->out_h, l->out_n} : contiguous_bhnd(H, N);
  return dtype == COTT_BF16 ? launch_bidir_fwd_tc_t<__nv_bfloat16>(q, k, v, keep, nc, out, B, H, N, dtype, stream, si, so)
                            : launch_bidir_fwd_tc_t<__half>(q, k, v, keep, nc, out, B, H, N, dtype, stream, si, so);
}

}  // namespace cott

extern "C" {

int cott_cos_attn_fwd(const void* q, const void* k, const void* v, const float* norm_const, void* out, int B,
                      int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if (!q || !k || !v || !out || !norm_const) return fail(COTT_ERR_NULL, "null tensor pointer");
  if ((st = aligned16(q, "q")) || (st = aligned16(k, "k")) || (st = aligned16(v, "v")) || (st = aligned16(out, "out")))
    return st;
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == COTT_BF16 ? launch_fwd<__nv_bfloat16>(q, k, v, norm_const, out, B, H, N, dtype, s)
                            : launch_fwd<__half>(q, k, v, norm_const, out, B, H, N, dtype, s);
}

int cott_cos_attn_bwd_dq(const void* q, const void* k, const void* v, const float* norm_const, const void* dout,
                         void* dq, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}, {dq, "dq"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == COTT_BF16 ? launch_bwd_dq<__nv_bfloat16>(q, k, v, norm_const, dout, dq, B, H, N, dtype, s)
                            : launch_bwd_dq<__half>(q, k, v, norm_const, dout, dq, B, H, N, dtype, s);
}

int cott_cos_attn_bwd_dkdv(const void* q, const void* k, const void* v, const float* norm_const, const void* dout,
                           void* dk, void* dv, float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype,
                           void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
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
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}, {dk, "dk"}, {dv, "dv"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  return dtype == COTT_BF16
             ? launch_bwd_dkdv<__nv_bfloat16>(q, k, v, norm_const, dout, dk, dv, dnorm_const, B, H, N, dtype, s)
             : launch_bwd_dkdv<__half>(q, k, v, norm_const, dout, dk, dv, dnorm_const, B, H, N, dtype, s);
}

int cott_cos_attn_bwd(const void* q, const void* k, const void* v, const float* norm_const, const void* dout,
                      void* dq, void* dk, void* dv, float* dnorm_const, int B, int H, int N, int Dk, int Dv,
                      int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if ((long)B * H * N == 0 || !norm_const) {  // nothing to launch, or an argument error: the two calls report it
    st = cott_cos_attn_bwd_dq(q, k, v, norm_const, dout, dq, B, H, N, Dk, Dv, dtype, stream);
    return st ? st : cott_cos_attn_bwd_dkdv(q, k, v, norm_const, dout, dk, dv, dnorm_const, B, H, N, Dk, Dv, dtype, stream);
  }
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}, {dq, "dq"}, {dk, "dk"}, {dv, "dv"}}))) return st;
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the gradient of norm_const is zeroed before the dQ launch, so that the two kernels follow each other directly
  COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, s));
  SegPlan plan;
  plan.dnorm_zeroed = true;
  if (dtype == COTT_BF16) {
    st = launch_bwd_dq<__nv_bfloat16>(q, k, v, norm_const, dout, dq, B, H, N, dtype, s, nullptr, plan);
    return st ? st : launch_bwd_dkdv<__nv_bfloat16>(q, k, v, norm_const, dout, dk, dv, dnorm_const, B, H, N, dtype, s, nullptr, plan);
  }
  st = launch_bwd_dq<__half>(q, k, v, norm_const, dout, dq, B, H, N, dtype, s, nullptr, plan);
  return st ? st : launch_bwd_dkdv<__half>(q, k, v, norm_const, dout, dk, dv, dnorm_const, B, H, N, dtype, s, nullptr, plan);
}

int cott_cos_attn_seg_count(int B, int H, int N) {
  const long BH = (long)B * H;
  const int total = (N + kTcChunk - 1) / kTcChunk;
  if (BH <= 0 || total < 4) return 1;
  int sm = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
  long nseg = sm / BH;              // one CTA per SM; more sequences than half the SMs: no gain
  if (nseg > total / 2) nseg = total / 2;  // at least two chunks per segment
  return nseg < 2 ? 1 : (int)nseg;
}

size_t cott_cos_attn_seg_workspace_bytes(int B, int H, int N, int nseg) {
  if (B <= 0 || H <= 0 || N <= 0) return 0;
  return 5 * seg_array_floats(B, H, plan_segments(N, nseg).nseg) * sizeof(float) + (size_t)B * N * sizeof(int);
}

int cott_cos_attn_fwd_seg(const void* q, const void* k, const void* v, const unsigned char* keep,
                          const float* norm_const, void* out, void* workspace, int nseg, const cott_layout* layout,
                          int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {out, "out"}, {workspace, "workspace"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  return dtype == COTT_BF16 ? run_fwd_seg<__nv_bfloat16>(q, k, v, keep, norm_const, out, ws, nseg, layout, B, H, N, dtype, s)
                            : run_fwd_seg<__half>(q, k, v, keep, norm_const, out, ws, nseg, layout, B, H, N, dtype, s);
}

int cott_cos_attn_bwd_seg(const void* q, const void* k, const void* v, const unsigned char* keep,
                          const float* norm_const, const void* dout, void* workspace, int nseg,
                          const cott_layout* layout, void* dq, void* dk, void* dv, float* dnorm_const, int B, int H,
                          int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if ((long)B * H * N == 0) {
    if (H > 0) COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, static_cast<cudaStream_t>(stream)));
    return COTT_OK;
  }
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}, {dq, "dq"}, {dk, "dk"}, {dv, "dv"},
                          {workspace, "workspace"}})))
    return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  return dtype == COTT_BF16
             ? run_bwd_seg<__nv_bfloat16>(q, k, v, keep, norm_const, dout, ws, nseg, layout, dq, dk, dv, dnorm_const, B, H, N, dtype, s)
             : run_bwd_seg<__half>(q, k, v, keep, norm_const, dout, ws, nseg, layout, dq, dk, dv, dnorm_const, B, H, N, dtype, s);
}

namespace {
// checks of the rotary argument shared by the two calls below
int check_rotary(const cott_rotary_tables* r, RotArgs* out) {
  if (!r || !r->sin_table || !r->cos_table) return fail(COTT_ERR_NULL, "null pointer: rotary tables");
  if (r->rot_dim < 16 || r->rot_dim % 16 || r->rot_dim > kTcD)
    return fail(COTT_ERR_SHAPE, "rotary dim must be a multiple of 16 between 16 and 64 (got %d)", r->rot_dim);
  if (r->table_batch_stride & 3 || r->table_batch_stride < 0) return fail(COTT_ERR_ALIGN, "table_batch_stride must be a non-negative multiple of 4");
  if ((reinterpret_cast<uintptr_t>(r->sin_table) | reinterpret_cast<uintptr_t>(r->cos_table)) & 15)
    return fail(COTT_ERR_ALIGN, "rotary tables must be 16-byte aligned");
  *out = RotArgs{r->sin_table, r->cos_table, r->rot_dim / 8, r->table_batch_stride};
  return COTT_OK;
}
}  // namespace

int cott_cos_attn_fwd_rotary(const void* q, const void* k, const void* v, const unsigned char* keep,
                             const float* norm_const, void* out, void* workspace, const cott_layout* layout,
                             const cott_rotary_tables* rotary, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  RotArgs rot;
  if ((st = check_rotary(rotary, &rot))) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {out, "out"}, {workspace, "workspace"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  return dtype == COTT_BF16 ? run_fwd_seg<__nv_bfloat16>(q, k, v, keep, norm_const, out, ws, 1, layout, B, H, N, dtype, s, nullptr, rot)
                            : run_fwd_seg<__half>(q, k, v, keep, norm_const, out, ws, 1, layout, B, H, N, dtype, s, nullptr, rot);
}

int cott_cos_attn_bwd_rotary(const void* q, const void* k, const void* v, const unsigned char* keep,
                             const float* norm_const, const void* dout, void* workspace, const cott_layout* layout,
                             const cott_rotary_tables* rotary, void* dq, void* dk, void* dv, float* dnorm_const, int B,
                             int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  RotArgs rot;
  if ((st = check_rotary(rotary, &rot))) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if ((long)B * H * N == 0) {
    if (H > 0) COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, static_cast<cudaStream_t>(stream)));
    return COTT_OK;
  }
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}, {dq, "dq"}, {dk, "dk"}, {dv, "dv"},
                          {workspace, "workspace"}})))
    return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  return dtype == COTT_BF16
             ? run_bwd_seg<__nv_bfloat16>(q, k, v, keep, norm_const, dout, ws, 1, layout, dq, dk, dv, dnorm_const, B, H, N, dtype, s, rot)
             : run_bwd_seg<__half>(q, k, v, keep, norm_const, dout, ws, 1, layout, dq, dk, dv, dnorm_const, B, H, N, dtype, s, rot);
}

size_t cott_cos_attn_saved_bytes(int B, int H, int N) {
  if (B <= 0 || H <= 0 || N <= 0) return 0;
  return (size_t)B * H * ((N + kTcChunk - 1) / kTcChunk) * kStateTileBytes;
}

int cott_cos_attn_fwd_train(const void* q, const void* k, const void* v, const unsigned char* keep,
                            const float* norm_const, void* out, void* saved, void* workspace, int nseg,
                            const cott_layout* layout, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {out, "out"}, {saved, "saved"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  if ((nseg > 1 || keep) && (st = check_ptrs16({{workspace, "workspace"}}))) return st;
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  return dtype == COTT_BF16 ? run_fwd_seg<__nv_bfloat16>(q, k, v, keep, norm_const, out, ws, nseg, layout, B, H, N, dtype, s, saved)
                            : run_fwd_seg<__half>(q, k, v, keep, norm_const, out, ws, nseg, layout, B, H, N, dtype, s, saved);
}

int cott_cos_attn_bwd_train(const void* q, const void* k, const void* v, const unsigned char* keep,
                            const float* norm_const, const void* dout, const void* saved, void* workspace, int nseg,
                            const cott_layout* layout, void* dq, void* dk, void* dv, float* dnorm_const, int B, int H,
                            int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if ((long)B * H * N == 0) {
    if (H > 0) COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, static_cast<cudaStream_t>(stream)));
    return COTT_OK;
  }
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {dout, "dout"}, {dq, "dq"}, {dk, "dk"}, {dv, "dv"}, {saved, "saved"}})))
    return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  if ((nseg > 1 || keep) && (st = check_ptrs16({{workspace, "workspace"}}))) return st;
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  return dtype == COTT_BF16 ? run_bwd_train<__nv_bfloat16>(q, k, v, keep, norm_const, dout, saved, ws, nseg, layout, dq, dk, dv,
                                                           dnorm_const, B, H, N, dtype, s)
                            : run_bwd_train<__half>(q, k, v, keep, norm_const, dout, saved, ws, nseg, layout, dq, dk, dv, dnorm_const,
                                                    B, H, N, dtype, s);
}

size_t cott_cos_attn_wide_workspace_bytes(int B, int H, int N) {
  if (B <= 0 || H <= 0 || N <= 0) return 0;
  const size_t V = (size_t)B * H * N, cnt = ((size_t)B * N + 3) & ~(size_t)3;
  return (6 * V + cnt + 2 * wide_ws_floats(B, H, N, 128, wide_seg_count(B, H, N, 128))) * sizeof(float);
}

static int check_wide_args(int B, int H, int N, int Dk, int Dv, int dtype) {
  if (dtype != COTT_BF16 && dtype != COTT_F16)
    return fail(COTT_ERR_DTYPE, "the fused head-dim-128 path takes float16/bfloat16 (dtype code %d given)", dtype);
  if (B < 0 || H < 0 || N < 0) return fail(COTT_ERR_SHAPE, "negative size B=%d H=%d N=%d", B, H, N);
  if (Dk != 128 || Dv != 128) return fail(COTT_ERR_UNSUPPORTED, "this entry point is built for head dim 128 (got Dk=%d Dv=%d)", Dk, Dv);
  if ((long)B * H > 0x7fffffffL) return fail(COTT_ERR_SHAPE, "B*H too large");
  return COTT_OK;
}

int cott_cos_attn_wide_fwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* norm_const,
                           void* out, void* workspace, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_wide_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H * N == 0) return COTT_OK;
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {out, "out"}, {workspace, "workspace"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == COTT_BF16 ? run_wide_fwd<__nv_bfloat16>(q, k, v, keep, norm_const, out, workspace, B, H, N, dtype, s)
                            : run_wide_fwd<__half>(q, k, v, keep, norm_const, out, workspace, B, H, N, dtype, s);
}

int cott_cos_attn_wide_bwd(const void* q, const void* k, const void* v, const unsigned char* keep, const float* norm_const,
                           const void* out, const void* dout, void* workspace, void* dq, void* dk, void* dv,
                           float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  int st = check_wide_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if (!dnorm_const && H > 0) return fail(COTT_ERR_NULL, "null pointer: dnorm_const");
  if ((long)B * H * N == 0) {
    if (H > 0) COTT_CUDA_TRY(cudaMemsetAsync(dnorm_const, 0, sizeof(float) * H, static_cast<cudaStream_t>(stream)));
    return COTT_OK;
  }
  if ((st = check_ptrs16({{q, "q"}, {k, "k"}, {v, "v"}, {out, "out"}, {dout, "dout"}, {dq, "dq"}, {dk, "dk"}, {dv, "dv"},
                          {workspace, "workspace"}})))
    return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  DeviceScope scope(q);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return dtype == COTT_BF16
             ? run_wide_bwd<__nv_bfloat16>(q, k, v, keep, norm_const, out, dout, workspace, dq, dk, dv, dnorm_const, B, H, N, dtype, s)
             : run_wide_bwd<__half>(q, k, v, keep, norm_const, out, dout, workspace, dq, dk, dv, dnorm_const, B, H, N, dtype, s);
}

}  // extern "C"

namespace {
// head dim 128: a state-only pass of the wide kernel (row norms and the length factor from the tiles), then the sum
// over the segments, transposed into the decode layout.  `workspace`: cott_cos_attn_wide_workspace_bytes(B, H, N).
template <typename T>
int run_wide_prefill_state(const void* k, const void* v, const float* nc, float* state, void* workspace, int accumulate, int B,
                           int H, int N, int dtype, cudaStream_t stream) {
  WideWs ws = wide_ws(workspace, B, H, N);
  const SegPlan plan = plan_segments(N, wide_seg_count(B, H, N, 128));
  WideArgs a = {};
  a.norm_const = nc;
  a.chunks_per_seg = plan.cps;
  a.state_out = ws.seg;
  WideTensors t{nullptr, k, v, nullptr, nullptr, 128};
  int st = launch_wide_t<T, false, true, true>(t, a, B, H, N, dtype, plan.nseg, stream);
  if (st) return st;
  wide_seg_to_decode_state_kernel<<<dim3((unsigned)((long)B * H), 2), 256, 0, stream>>>(ws.seg, state, plan.nseg, accumulate != 0);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}
}  // namespace

extern "C" {

int cott_cos_attn_prefill_state(const void* k, const void* v, const float* norm_const, float* state, void* workspace,
                                int nseg, int accumulate, int B, int H, int N, int Dk, int Dv, int dtype, void* stream) {
  if (Dk == 128 && Dv == 128 && (dtype == COTT_BF16 || dtype == COTT_F16) && B > 0 && H > 0 && N > 0) {
    int stw = check_ptrs16({{k, "k"}, {v, "v"}, {workspace, "workspace"}, {state, "state"}});
    if (stw) return stw;
    if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
    DeviceScope scope(state);
    COTT_CUDA_TRY(scope.status());
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == COTT_BF16 ? run_wide_prefill_state<__nv_bfloat16>(k, v, norm_const, state, workspace, accumulate, B, H, N, dtype, s)
                              : run_wide_prefill_state<__half>(k, v, norm_const, state, workspace, accumulate, B, H, N, dtype, s);
  }
  int st = check_fused_args(B, H, N, Dk, Dv, dtype);
  if (st) return st;
  if ((long)B * H == 0) return COTT_OK;
  if (!state) return fail(COTT_ERR_NULL, "null pointer: state");
  DeviceScope scope(state);
  COTT_CUDA_TRY(scope.status());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N == 0) {
    if (!accumulate) COTT_CUDA_TRY(cudaMemsetAsync(state, 0, sizeof(float) * (size_t)B * H * kTcD * kTcD, s));
    return COTT_OK;
  }
  if ((st = check_ptrs16({{k, "k"}, {v, "v"}, {workspace, "workspace"}, {state, "state"}}))) return st;
  if (!norm_const) return fail(COTT_ERR_NULL, "null pointer: norm_const");
  const SegPlan plan = plan_segments(N, nseg);
  float* ws = static_cast<float*>(workspace);
  st = dtype == COTT_BF16 ? launch_seg_state<__nv_bfloat16, kSegFwdState>(k, v, contiguous_bhnd(H, N), contiguous_bhnd(H, N), norm_const, ws, B, H, N,
                                                                        dtype, plan, s)
                          : launch_seg_state<__half, kSegFwdState>(k, v, contiguous_bhnd(H, N), contiguous_bhnd(H, N), norm_const, ws, B, H, N, dtype,
                                                                 plan, s);
  if (st) return st;
  seg_to_decode_state_kernel<<<(unsigned)((long)B * H), 256, 0, s>>>(ws, state, plan.nseg, accumulate != 0);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

int cott_selftest_device_wait(int polls, int code, int chunk, void* stream) {
  if (polls < 1 || polls > 64) return fail(COTT_ERR_SHAPE, "polls must be in [1, 64] (got %d)", polls);
  if (code < 1 || code > 0x7fff || chunk < 0 || chunk > 0xffff)
    return fail(COTT_ERR_SHAPE, "code must be in [1, 32767] and chunk in [0, 65535] (got %d, %d)", code, chunk);
  wait_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(polls, code, chunk);
  COTT_CUDA_TRY(cudaGetLastError());
  return COTT_OK;
}

int cott_check_status(int* detail) {
  int v = 0;
  COTT_CUDA_TRY(cudaDeviceSynchronize());
  COTT_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_cott_status, sizeof(int)));
  if (detail) *detail = v;
  if (v != 0) {
    int zero = 0;
    COTT_CUDA_TRY(cudaMemcpyToSymbol(g_cott_status, &zero, sizeof(int)));
    return fail(COTT_ERR_DEVICE_WAIT, "a device-side wait gave up: stage %d (1=TMA, 2=score MMA, 3=accumulator MMA) at chunk %d",
                v >> 16, v & 0xffff);
  }
  return COTT_OK;
}

}  // extern "C"
