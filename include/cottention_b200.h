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
 * `out` may be the same buffer as `v` (the reference's inplace=true, :403-404).
 *
 * Kernels: 16-bit dtypes with D_attn = 64 or 128 and D_value a multiple of 64 run on the tensor cores (tcgen05; at 128
 * both halves of q and k go into the same score and state accumulators, the counterpart of the reference's
 * kernel_mod_4<T, 32>, :173-251); D_attn = 192 / 256 as 64-wide tensor-core launches on strided slices, whose partial
 * results (one per 64-wide slice of D_attn, each an fp32 sum rounded once to the storage type) are added in the storage
 * type -- up to four roundings per output at D_attn = 256, 1e-2 relative against the exact kernel; everything else on the
 * exact CUDA-core kernel.
 * Memory: unlike the reference's kernel call, which needs no workspace, the tensor-core paths take stream-ordered
 * scratch from a memory pool that the LIBRARY owns and keeps for the life of the process (cudaMallocFromPoolAsync /
 * cudaFreeAsync on `stream`, release threshold = unlimited) in two cases: few (batch, head) pairs with a long sequence
 * (fp32 segment states, 2 x B*H*ceil(Dv/64)*nseg*32 KB) and D_attn = 192 / 256 (one [B,H,N,64] partial result).  The
 * allocation is visible under stream capture.  Callers that must control every byte use the fused entry points below,
 * which take their workspace from the caller.
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

/*
 * Fused causal cosine attention, forward (tensor-core path: tcgen05 / TMEM / TMA).
 *
 *   q^ = q/max(|q|,1e-12)   k^ = k/max(|k|,1e-12)   v'_s = v_s / max((s+1)^sigmoid(norm_const[h]), 1)
 *   out[b,h,t,:] = sum_{s<=t} (q^_t . k^_s) v'_s
 *
 * Replaces, in one launch, the non-decode branch of GPTCosAttention._cos_attn,
 * GPT_Trainer/GPTCosAttention.py:229-248 (normalize, length-norm of V by key position) followed by
 * CustomAttention.apply (:282 -> Cuda_Kernel/Custom_Kernel.py:9-30 -> combined_kernel_general.cu),
 * for an all-keep attention mask.  `norm_const` is H floats in device memory (the module's
 * [1,H,1,1] parameter, :89).  dtype: COTT_BF16 or COTT_F16; Dk = Dv = 64; pointers 16-byte aligned.
 * fp32 accumulation throughout.
 */
int cott_cos_attn_fwd(const void* q, const void* k, const void* v, const float* norm_const, void* out,
                      int B, int H, int N, int Dk, int Dv, int dtype, void* stream);

/*
 * Fused backward of cott_cos_attn_fwd: dq, dk, dv (same layout and dtype as the inputs) and
 * dnorm_const (H floats, overwritten).  Two launches: a forward-direction pass for dq and a
 * reverse-direction pass for dk, dv and dnorm_const.
 *
 * Replaces CustomAttention.backward (Cuda_Kernel/Custom_Kernel.py:35-141, three kernel calls) plus
 * the autograd of GPTCosAttention.py:229-230 (normalize) and :241 (length-norm; this is where the
 * gradient of norm_const comes from in the reference).
 */
int cott_cos_attn_bwd(const void* q, const void* k, const void* v, const float* norm_const,
                      const void* dout, void* dq, void* dk, void* dv, float* dnorm_const, int B, int H,
                      int N, int Dk, int Dv, int dtype, void* stream);

/*
 * The two launches of cott_cos_attn_bwd as separate calls (same arguments, same results), so
 * that a caller can time or schedule them individually:
 *   _dq    forward-direction pass: dq     (role of Custom_Kernel.py:106 + autograd of the q normalize)
 *   _dkdv  reverse-direction pass: dk, dv, dnorm_const   (Custom_Kernel.py:107-108 + autograd of the
 *          k normalize and of the length-norm, GPTCosAttention.py:230,241)
 */
int cott_cos_attn_bwd_dq(const void* q, const void* k, const void* v, const float* norm_const,
                         const void* dout, void* dq, int B, int H, int N, int Dk, int Dv, int dtype,
                         void* stream);
int cott_cos_attn_bwd_dkdv(const void* q, const void* k, const void* v, const float* norm_const,
                           const void* dout, void* dk, void* dv, float* dnorm_const, int B, int H, int N,
                           int Dk, int Dv, int dtype, void* stream);

/*
 * Segment-parallel form of the three calls above, for long sequences with few (batch, head) pairs
 * (B = 1, H = 16, N = 16k .. 256k): every sequence is cut into `nseg` segments that run on different
 * SMs.  The results are those of cott_cos_attn_fwd / cott_cos_attn_bwd (the state is carried across
 * segment boundaries in fp32; summation order differs).  No counterpart in the reference, whose kernel
 * (combined_kernel_general.cu:96-251) is sequential in N with one block per (batch, head, output column).
 *   cott_cos_attn_seg_count            suggested nseg for this device (1 = use the plain calls)
 *   cott_cos_attn_seg_workspace_bytes  size of `workspace` (device memory, 16-byte aligned) for that nseg
 *   _fwd_seg writes the segment states into `workspace`; pass the same buffer and nseg, untouched, to _bwd_seg.
 * These two calls also take the padding mask of GPTCosAttention.py:232-248: `keep` ([B, N] bytes, non-zero =
 * un-masked, NULL = no padding) zeroes the masked rows of q^, k^, v' and makes n_s the running count of
 * un-masked positions; nseg = 1 is allowed (one CTA per sequence, workspace still needed for the count).
 * They also take strided tensors: `layout` (NULL = contiguous [B,H,N,64]) gives the element strides of the batch,
 * head and position dimensions, one triple for q, k, v, dq, dk, dv and one for out, dout (multiples of 8
 * elements; base pointers 16-byte aligned).  q, k, v may so be slices of the packed [B, N, 3, H, 64] output of a
 * QKV projection and out the [B, N, H*64] input of the output projection: the head split / merge permutes of
 * GPTCosAttention.py:447-449,478-479,500 cost no copy.
 */
typedef struct cott_layout { /* element strides of [B, H, N, 64] views whose innermost dimension is contiguous */
  long long in_b, in_h, in_n;    /* q, k, v and dq, dk, dv */
  long long out_b, out_h, out_n; /* out and dout */
} cott_layout;
int cott_cos_attn_seg_count(int B, int H, int N);
size_t cott_cos_attn_seg_workspace_bytes(int B, int H, int N, int nseg);
int cott_cos_attn_fwd_seg(const void* q, const void* k, const void* v, const unsigned char* keep,
                          const float* norm_const, void* out, void* workspace, int nseg,
                          const cott_layout* layout, int B, int H, int N, int Dk, int Dv, int dtype,
                          void* stream);
int cott_cos_attn_bwd_seg(const void* q, const void* k, const void* v, const unsigned char* keep,
                          const float* norm_const, const void* dout, void* workspace, int nseg,
                          const cott_layout* layout, void* dq, void* dk, void* dv, float* dnorm_const, int B,
                          int H, int N, int Dk, int Dv, int dtype, void* stream);

/*
 * Training pair: forward that keeps what a ONE-pass backward needs, and that backward.
 *
 * cott_cos_attn_fwd_train is cott_cos_attn_fwd_seg (same arguments, same `out`) that also writes `saved`: the
 * 16-bit state operand of every 128-position chunk, i.e. sum_{s < chunk} k_s (x) v'_s / |k_s| as the forward's
 * tensor-core products consume it ([B*H][ceil(N/128)][64][64] elements of `dtype`, cott_cos_attn_saved_bytes(B, H, N)
 * bytes = half the size of q; device memory, 16-byte aligned).  cott_cos_attn_bwd_train takes q, k, v, dout and
 * `saved`, untouched, and produces dq, dk, dv, dnorm_const in a single reverse walk over the sequence: every input
 * tensor is read once (7.5 tensor passes against the 11 of cott_cos_attn_bwd, whose two kernels walk in opposite
 * directions and each read q, k, v, dout).  Same results as cott_cos_attn_bwd up to rounding.
 * `workspace` is only needed (and only touched) when nseg > 1 or keep != NULL; pass the same buffer to both calls.
 *
 * Replaces CustomAttention.forward / .backward (Cuda_Kernel/Custom_Kernel.py:9-30,35-141) with the module math of
 * GPTCosAttention.py:229-248 around them, as cott_cos_attn_fwd / _bwd do.  The reference's own sketch of a merged
 * backward (Cuda_Kernel/backwardv2_comb.cu:58-149, not built by its setup.py) is the closest counterpart.
 */
size_t cott_cos_attn_saved_bytes(int B, int H, int N);
int cott_cos_attn_fwd_train(const void* q, const void* k, const void* v, const unsigned char* keep,
                            const float* norm_const, void* out, void* saved, void* workspace, int nseg,
                            const cott_layout* layout, int B, int H, int N, int Dk, int Dv, int dtype,
                            void* stream);
int cott_cos_attn_bwd_train(const void* q, const void* k, const void* v, const unsigned char* keep,
                            const float* norm_const, const void* dout, const void* saved, void* workspace,
                            int nseg, const cott_layout* layout, void* dq, void* dk, void* dv,
                            float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype, void* stream);

/*
 * Fused causal cosine attention for head dim 128 (Dk = Dv = 128, bf16 / fp16): the math of cott_cos_attn_fwd / _bwd,
 * padding mask included (`keep`, see cott_cos_attn_fwd_seg).  In the reference this head dim runs kernel_mod_4<T, 32>
 * (Cuda_Kernel/combined_kernel_general.cu:173-251, chosen at :281-284) inside the same module math
 * (GPT_Trainer/GPTCosAttention.py:229-248,282) and the three scans of CustomAttention.backward (Custom_Kernel.py:106-108).
 * Forward: one tensor-core pass (two CTAs per sequence, one per 64-column half of V; both halves of q and k go into the
 * same score and state accumulators).  Backward: a row-dot pass over (dout, out), then three tensor-core passes (dq
 * forward; dv and dk reversed) with the normalisation terms applied in their epilogues.  Few (batch, head) pairs with a
 * long sequence are cut into segments inside the call.
 * `workspace`: cott_cos_attn_wide_workspace_bytes(B, H, N) bytes of device memory, 16-byte aligned; the forward leaves
 * its row factors there, so pass the same buffer, untouched, to the backward together with the forward's `out`.
 */
size_t cott_cos_attn_wide_workspace_bytes(int B, int H, int N);
int cott_cos_attn_wide_fwd(const void* q, const void* k, const void* v, const unsigned char* keep,
                           const float* norm_const, void* out, void* workspace, int B, int H, int N, int Dk, int Dv,
                           int dtype, void* stream);
int cott_cos_attn_wide_bwd(const void* q, const void* k, const void* v, const unsigned char* keep,
                           const float* norm_const, const void* out, const void* dout, void* workspace, void* dq,
                           void* dk, void* dv, float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype,
                           void* stream);

/*
 * Prefill -> decode hand-off: the decode state (cott_decode_step layout, float32 [B,H,Dv,Dk]) that a prompt of N
 * tokens at positions 1..N leaves behind, state[b,h,j,i] = sum_s v'_s[j] k^_s[i], computed with the segment-state
 * kernels instead of N recurrent steps (the reference absorbs a prompt token by token, GPTCosAttention.py:253-272).
 * `accumulate` != 0 adds to `state` instead of overwriting it -- only meaningful for a state that is still at
 * position 0, since the length factor uses positions 1..N.  `workspace`: cott_cos_attn_seg_workspace_bytes(B, H, N,
 * nseg) bytes.  bf16 / fp16 prompts, head dim 64 (the prompt's outputs come from cott_cos_attn_fwd(_seg)) or head dim
 * 128 (a state-only pass of the 128-wide kernel; `nseg` is ignored, `workspace` is
 * cott_cos_attn_wide_workspace_bytes(B, H, N) bytes, the outputs come from cott_cos_attn_wide_fwd).
 */
int cott_cos_attn_prefill_state(const void* k, const void* v, const float* norm_const, float* state,
                                void* workspace, int nseg, int accumulate, int B, int H, int N, int Dk, int Dv,
                                int dtype, void* stream);

/*
 * Recurrent decode.  Per (batch, head) a float32 state[b,h,j,i] ([B,H,Dv,Dk], updated in place) is
 * advanced by one token:
 *   q^ = q/|q|, k^ = k/|k|, v' = v / max(pos^sigmoid(norm_const[h]), 1)
 *   state[j][i] += v'[j] k^[i]        out[j] = sum_i q^[i] state[j][i]
 * q, k are [B,H,Dk], v and out [B,H,Dv] of `dtype` (COTT_F32, COTT_F16 or COTT_BF16).  `pos` is the
 * 1-based position of the token (the reference's cur_s); if `positions` is not NULL it is an array
 * of B int64 positions in device memory, one per batch entry, and `pos` is ignored.
 *
 * Replaces the fast_inference branch of GPTCosAttention._cos_attn for one token,
 * GPT_Trainer/GPTCosAttention.py:229-230,236,253-272 (state init :76-85; driven token by token by
 * GPT_Trainer/fast_infer.py:111-139).  The reference keeps a float64 [1,H,d,d] state on the CPU;
 * this one is float32, batched, in HBM.  Dk in {16,32,64,128}, 1 <= Dv <= 128.
 */
int cott_decode_step(float* state, const void* q, const void* k, const void* v, const float* norm_const,
                     void* out, int B, int H, int Dk, int Dv, int dtype, long long pos,
                     const long long* positions, void* stream);

/*
 * T consecutive decode steps in one launch: q, k [B,H,T,Dk], v, out [B,H,T,Dv]; token t of batch
 * entry b sits at position (positions ? positions[b] : pos) + t.  The state is read once, kept in
 * registers for the T steps and written back once.  This is the reference's loop over the tokens
 * of a prompt in the same branch (GPTCosAttention.py:262-269).
 */
int cott_decode_steps(float* state, const void* q, const void* k, const void* v, const float* norm_const,
                      void* out, int B, int H, int T, int Dk, int Dv, int dtype, long long pos,
                      const long long* positions, void* stream);

/*
 * Bidirectional (encoder) cosine attention, forward:
 *   keep_s: un-masked positions ([B,N] bytes, non-zero = keep; NULL = keep all), L_b = their count
 *   q^ = keep q/|q|, k^ = keep k/|k|, v' = keep v / max(L_b^sigmoid(norm_const[h]), 1)
 *   out[b,h,t,:] = q^_t (sum_s k^_s (x) v'_s)
 * Replaces the cosine section of BertCosAttention.forward, BERT_Trainer/BertCosAttention.py:162-178
 * (mask, normalize, length-norm) and :197-249 (the two einsum orders, which are the same function).
 * All four dtypes; Dk, Dv divisible by 16 and <= 128; fp32 accumulation (fp64 for COTT_F64).
 *
 * `scratch` is caller-provided device memory of cott_bidir_scratch_bytes(...) bytes that receives
 * the per-(b,h) state partials; pass the same buffer, untouched, to cott_bidir_bwd as `scratch_state`.
 */
size_t cott_bidir_scratch_bytes(int B, int H, int N, int Dk, int Dv, int dtype);
int cott_bidir_fwd(const void* q, const void* k, const void* v, const unsigned char* keep,
                   const float* norm_const, void* out, void* scratch, int B, int H, int N, int Dk, int Dv,
                   int dtype, void* stream);

/*
 * Backward of cott_bidir_fwd: dq, dk, dv and dnorm_const (H floats, overwritten).  The reference
 * obtains these by autograd through the einsums (its hand-written non-causal Function `Multiply`,
 * GPT_Trainer/GPTCosAttention.py:22-37, is unused and its grad_V line is wrong).
 * `scratch_state` is the forward's scratch; `scratch_dstate` is a second buffer of the same size.
 */
int cott_bidir_bwd(const void* q, const void* k, const void* v, const unsigned char* keep,
                   const float* norm_const, const void* dout, const void* scratch_state, void* scratch_dstate,
                   void* dq, void* dk, void* dv, float* dnorm_const, int B, int H, int N, int Dk, int Dv,
                   int dtype, void* stream);

/*
 * The bidirectional pair on strided tensors (`cott_layout`, see cott_cos_attn_fwd_seg; NULL = contiguous): head dim
 * 64, bf16 / fp16 only (the tensor-core kernels, which keep the state on chip and need no scratch).  Lets
 * BertCosAttention read q, k, v straight out of its projections' [B, N, H*64] outputs and write the context layer in
 * the layout its output projection reads (BERT_Trainer/BertCosAttention.py:148-156,252-254: transpose_for_scores and
 * the permute back cost no copy).
 */
int cott_bidir_fwd_strided(const void* q, const void* k, const void* v, const unsigned char* keep,
                           const float* norm_const, void* out, const cott_layout* layout, int B, int H, int N,
                           int Dk, int Dv, int dtype, void* stream);
int cott_bidir_bwd_strided(const void* q, const void* k, const void* v, const unsigned char* keep,
                           const float* norm_const, const void* dout, const cott_layout* layout, void* dq,
                           void* dk, void* dv, float* dnorm_const, int B, int H, int N, int Dk, int Dv, int dtype,
                           void* stream);

/*
 * cott_bidir_fwd for callers that cannot allocate.  (No counterpart in the reference, whose
 * bidirectional path lets PyTorch allocate its einsum intermediates.)
 *
 * Same inputs, outputs and results as cott_bidir_fwd, but there is no `scratch` argument: the state
 * partials go to a fixed array of COTT_BIDIR_STATIC_SCRATCH_BYTES that is linked into the library
 * and therefore sits on every GPU that loads it until the process exits.  Meant for hosts that
 * give away all device memory at start-up and must never enter the CUDA allocator afterwards (a
 * serving process with a frozen pool, a loop that cannot afford cudaMalloc's device-wide
 * synchronisation).  The call makes no cudaMalloc/cudaFree and uses no allocating library routine.
 *
 * Limits and rules:
 *  - B*H*nsplit*Dk*Dv accumulator elements (4 bytes, 8 for COTT_F64; nsplit <= 8 is chosen from
 *    B*H and N) must fit in COTT_BIDIR_STATIC_SCRATCH_BYTES; larger problems are rejected with
 *    COTT_ERR_SHAPE and a message that names both sizes.  BERT-base at batch 32 (B*H = 384,
 *    N = 512, d = 64) needs 6 MiB.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and caches it; make that first call before any stream capture begins.
 *  - All calls on a device share the one array, and it keeps whatever the last call left in it.
 *    Nothing needs clearing (every slot that is read is first written in full by the same call),
 *    but two calls that overlap on the GPU -- different streams, or the same array reached from two
 *    host threads -- race on it.  Serialise them.
 *  - There is no matching backward: the backward needs the forward's scratch kept alive, which a
 *    shared array cannot promise.
 */
#define COTT_BIDIR_STATIC_SCRATCH_BYTES (8u << 20)
int cott_bidir_fwd_static(const void* q, const void* k, const void* v, const unsigned char* keep,
                          const float* norm_const, void* out, int B, int H, int N, int Dk, int Dv,
                          int dtype, void* stream);

/*
 * Device-side health check.  The tensor-core kernels bound every wait (TMA arrival, MMA
 * completion); a wait that gives up records a code and the kernel returns without hanging.
 * This call synchronises the current device, returns COTT_ERR_DEVICE_WAIT if a code was
 * recorded since the last check (clearing it), else COTT_OK.  `detail` (may be NULL) receives
 * the raw code: (stage << 16) | chunk.  No counterpart in the reference, which checks no errors.
 */
int cott_check_status(int* detail);

/*
 * Exercises that time-out path without a fault: launches one small CTA that sets up an mbarrier and a TMEM
 * allocation like the tensor-core kernels, lets one warp wait (same bounded wait, `polls` tries of about 0.2 ms
 * each, 1 <= polls <= 64) on a barrier phase that nothing completes while the other warps wait elsewhere with
 * the normal limit, and leaves the way those kernels leave after a time-out.  Afterwards cott_check_status
 * returns COTT_ERR_DEVICE_WAIT with detail == (code << 16) | chunk, and the device is usable as before.
 * For tests of a host's handling of that status.  No counterpart in the reference.
 */
int cott_selftest_device_wait(int polls, int code, int chunk, void* stream);

/* Rotary position embedding of the reference's GPT module (GPT_Trainer/GPTCosAttention.py:458-476; transformers'
 * apply_rotary_pos_emb / rotate_every_two), in place on q and k: x'[2i] = x[2i] cos_i - x[2i+1] sin_i,
 * x'[2i+1] = x[2i+1] cos_i + x[2i] sin_i for i < rot_dim/2; elements from rot_dim on pass through.
 * q, k: [B, H, N, D] views (float16 / bfloat16) with the element strides layout->in_b, in_h, in_n (NULL = dense), so
 * the q and k slices of a packed [B, N, 3, H, D] projection output can be rotated where they lie.
 * sin_table, cos_table: fp32 [N, rot_dim/2] (table_batch_stride = 0) or one table per batch entry
 * (table_batch_stride = N * rot_dim/2).  inverse != 0 applies the transposed rotation (the backward of the op). */
int cott_rotary(void* q, void* k, const float* sin_table, const float* cos_table, const cott_layout* layout, int B,
                int H, int N, int D, int rot_dim, long long table_batch_stride, int inverse, int dtype, void* stream);

/*
 * The fused causal forward / backward with the rotary position embedding of the reference's GPT module folded in
 * (GPT_Trainer/GPTCosAttention.py:458-476 followed by :229-248,282): q and k are rotated inside the kernels -- their
 * tiles are rewritten in shared memory before any product reads them, and the dq and dk rows are rotated back before
 * they are stored -- so q, k in device memory stay as the projection wrote them and the separate passes over q, k
 * (forward) and dq, dk (backward) of cott_rotary are not needed.  Results are those of cott_rotary followed by
 * cott_cos_attn_fwd_seg / _bwd_seg with nseg = 1 (bit for bit: the same fp32 arithmetic and the same roundings).
 * Arguments as for those calls (keep, layout and workspace included; workspace of
 * cott_cos_attn_seg_workspace_bytes(B, H, N, 1) bytes, passed untouched from the forward to the backward call),
 * one segment per sequence; `rotary` as for cott_rotary, with rot_dim a multiple of 16, 16 <= rot_dim <= 64.
 */
typedef struct cott_rotary_tables {
  const float* sin_table;         /* fp32 [N, rot_dim/2], or [B, N, rot_dim/2] with table_batch_stride = N * rot_dim/2 */
  const float* cos_table;
  int rot_dim;                    /* the first rot_dim elements of every head are rotated */
  long long table_batch_stride;   /* 0 = one table for every batch entry */
} cott_rotary_tables;
int cott_cos_attn_fwd_rotary(const void* q, const void* k, const void* v, const unsigned char* keep,
                             const float* norm_const, void* out, void* workspace, const cott_layout* layout,
                             const cott_rotary_tables* rotary, int B, int H, int N, int Dk, int Dv, int dtype,
                             void* stream);
int cott_cos_attn_bwd_rotary(const void* q, const void* k, const void* v, const unsigned char* keep,
                             const float* norm_const, const void* dout, void* workspace, const cott_layout* layout,
                             const cott_rotary_tables* rotary, void* dq, void* dk, void* dv, float* dnorm_const,
                             int B, int H, int N, int Dk, int Dv, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* COTTENTION_B200_H_ */
