/* vrwkv_b200 -- C ABI of the B200 (sm_100a) token-mixing kernels of Vision-RWKV.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA
 * stream it is given (a cudaStream_t passed as void*; NULL is the legacy default
 * stream), never synchronises, never allocates, and returns a status code
 * (VRWKV_OK == 0).  The caller owns every buffer, including the scratch
 * "workspace" (256-byte aligned), whose size the matching *_workspace_bytes function
 * reports.
 * Outputs need no initialisation: every element is written.
 *
 * Layouts: k, v, y, gy, gk, gv, r, gr, w_raw, gw_raw are (B, T, C) row-major,
 * channel fastest (the backbones' token-major layout).  All data are fp32, as in
 * the reference, whose Python wrappers cast to fp32 before calling the kernels.
 *
 * Each declaration names the reference interface it stands in for, by path inside
 * the OpenGVLab/Vision-RWKV tree ("CLS/" = classification/mmcls_custom/models/
 * backbones/, "MAE/" = classification/mae/).
 */
#ifndef VRWKV_B200_H_
#define VRWKV_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum vrwkv_status {
    VRWKV_OK = 0,
    VRWKV_ERR_SHAPE = 1,       /* a dimension is <= 0 or beyond what a launch can index   */
    VRWKV_ERR_NULL = 2,        /* a required pointer is NULL                               */
    VRWKV_ERR_WORKSPACE = 3,   /* workspace_bytes is smaller than *_workspace_bytes says   */
    VRWKV_ERR_ALIGNMENT = 4,   /* data pointer not 4-byte / workspace not 256-byte aligned */
    VRWKV_ERR_LAUNCH = 5,      /* cudaGetLastError() reported a failure after a launch     */
    VRWKV_ERR_DEVICE = 6,      /* driver entry point or device attribute unavailable       */
    VRWKV_ERR_HEAD_SIZE = 7,   /* WKV6: C != 64 * H                                        */
    VRWKV_ERR_UNSUPPORTED = 8  /* bf16 and saved-result entry points: shape or alignment outside
                                  what their kernels cover; nothing ran, use the plain f32
                                  entry points                                               */
};

/* Library version, major*10000 + minor*100 + patch. */
int vrwkv_version(void);
/* Human-readable text for a status code (static storage). */
const char* vrwkv_status_string(int status);
/* One line about the most recent non-zero status of the calling thread (for instance the name
 * of the CUDA error behind VRWKV_ERR_LAUNCH).  Thread-local storage.  Diagnostic. */
const char* vrwkv_last_error_detail(void);
/* Number of kernels this library has launched in the calling process so far. */
unsigned long long vrwkv_launch_count(void);

/* Kernel path selection, for tests and measurements: 0 = automatic (default: Bi-WKV takes the
 * cluster-resident single-pass kernels when T <= 32768, C % 4 == 0 (bfloat16: C % 8 == 0) and the
 * tensors are 16-byte aligned - one cluster per sequence strip up to T = 4096, several above -,
 * else the persistent tile kernels, else the generic multi-launch path), 1 = the
 * first-generation kernels (Bi-WKV: the generic multi-launch path; WKV6 tensor-core forward:
 * the serial-phase kernel instead of the warp-specialised one), 2 = Bi-WKV skips the
 * cluster-resident kernels (persistent tile kernels where eligible), 3 = test of the bounded
 * device-side waits: as 0, but one CTA of every cluster withholds what it owes the others and
 * the waits give up after about a thousand polls, so the call returns promptly with bit 0 of the
 * status word set and meaningless results (nothing hangs, nothing faults).  Process-wide.
 * No reference counterpart. */
int vrwkv_set_path(int path);
/* Copies the device status word kept in the first 4 bytes of a workspace to *status_out
 * after synchronising `stream`.  0 means no bounded device-side wait ran out; bit 0 = a
 * hand-over between CTAs (tile-exchange flag, cluster mbarrier) never arrived, bit 1 = a TMA load never
 * completed, bit 2 = a record of another segment of a long sequence never arrived.  Diagnostic only;
 * no reference counterpart (the reference never checks its launches). */
int vrwkv_workspace_status(const void* workspace, void* stream, unsigned* status_out);

/* ---- Bi-WKV --------------------------------------------------------------------
 * y[b,t,c] = sum_j p_tj v[b,j,c] / sum_j p_tj,  log p_tj = k[b,j,c] - w[c]|t-j| for
 * j != t and u[c] + k[b,t,c] for j == t.  w, u: (C,).
 *
 * vrwkv_biwkv_forward_f32 replaces
 *   cuda_forward(int B,int T,int C,float*w,float*u,float*k,float*v,float*y)
 *       MAE/vrwkv/cuda/wkv_op.cpp:3,6-8  (kernel MAE/vrwkv/cuda/wkv_cuda.cu:332-338)
 *   bi_wkv_cuda_forward(w,u,k,v) -> y
 *       CLS/cuda_new/bi_wkv.cpp:11-15,23-33 (kernel CLS/cuda_new/bi_wkv_kernel.cu:370-399)
 * without their T <= T_MAX, C >= 32 and B*C % 32 == 0 restrictions.
 */
size_t vrwkv_biwkv_forward_workspace_bytes(int B, int T, int C);
int vrwkv_biwkv_forward_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                            const float* v, float* y, void* workspace, size_t workspace_bytes,
                            void* stream);

/* vrwkv_biwkv_backward_f32 replaces
 *   cuda_backward(int B,int T,int C,float*w,float*u,float*k,float*v,float*gy,
 *                 float*gw,float*gu,float*gk,float*gv)
 *       MAE/vrwkv/cuda/wkv_op.cpp:4,9-11 (kernel MAE/vrwkv/cuda/wkv_cuda.cu:340-345)
 *   bi_wkv_cuda_backward(w,u,k,v,gy) -> {gw,gu,gk,gv}
 *       CLS/cuda_new/bi_wkv.cpp:17-21,35-47 (kernel CLS/cuda_new/bi_wkv_kernel.cu:401-443)
 * gwgu is (2, C): row 0 = gw, row 1 = gu, already summed over batch and tokens in
 * a fixed order (no atomics), contiguous so one all-reduce covers both.  Nothing
 * per-token is kept from the forward: the backward recomputes from k, v, gy.
 */
size_t vrwkv_biwkv_backward_workspace_bytes(int B, int T, int C);
int vrwkv_biwkv_backward_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                             const float* v, const float* gy, float* gwgu, float* gk, float* gv,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Forward that keeps what the backward needs, and the backward that uses it.  The reference's
 * backward rebuilds y, 1/Den and the shift per token inside its kernel and holds them in three
 * scratch tensors (bi_wkv_kernel.cu:259-302, 415-417).  Here the forward can write log Den_t next
 * to y (one extra float per element), and vrwkv_biwkv_backward_saved_f32 takes k, v, gy and the
 * saved y, log Den: it needs one cross-tile exchange instead of two, at the price of keeping logden
 * (B*T*C floats) from forward to backward.  The pair runs on the tile kernels; for T <= 4096 the
 * cluster-resident vrwkv_biwkv_forward_f32 + vrwkv_biwkv_backward_f32, which keep nothing, are
 * about twice as fast.  Results agree with the recomputing pair to float32 rounding.  Same workspace sizes.  Both are
 * served by the single-pass TMA kernels only (C % 4 == 0, 16-byte aligned tensors, T below about
 * 37 000); otherwise they return VRWKV_ERR_UNSUPPORTED and nothing ran. */
int vrwkv_biwkv_forward_save_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                                 const float* v, float* y, float* logden, void* workspace,
                                 size_t workspace_bytes, void* stream);
int vrwkv_biwkv_backward_saved_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                                   const float* v, const float* gy, const float* y, const float* logden,
                                   float* gwgu, float* gk, float* gv, void* workspace,
                                   size_t workspace_bytes, void* stream);

/* bfloat16 activations: k, v, y, gy, gk, gv are bfloat16 bit patterns (uint16_t), w, u and
 * gwgu stay float, arithmetic is the f32 kernels' (inputs widened in shared memory, results
 * rounded to nearest-even on the way out).  They replace the float casts around the extension
 * calls in WKV.forward / WKV.backward (CLS/vrwkv.py:34-37, 51-55: `k.float().contiguous()` ...)
 * together with the calls themselves.  Workspace sizes are those of the f32 entry points.
 * Served by the single-pass TMA kernels only: C % 8 == 0, 16-byte aligned tensors and
 * ceil(T / 128) below the number of resident thread blocks (about T < 37 000); anything else
 * returns VRWKV_ERR_UNSUPPORTED before launching, and the caller casts and uses the f32 calls.
 */
int vrwkv_biwkv_forward_bf16(int B, int T, int C, const float* w, const float* u, const uint16_t* k,
                             const uint16_t* v, uint16_t* y, void* workspace, size_t workspace_bytes,
                             void* stream);
int vrwkv_biwkv_backward_bf16(int B, int T, int C, const float* w, const float* u, const uint16_t* k,
                              const uint16_t* v, const uint16_t* gy, float* gwgu, uint16_t* gk,
                              uint16_t* gv, void* workspace, size_t workspace_bytes, void* stream);

/* vrwkv_biwkv_forward_f32_noalloc has no counterpart in the reference.  It is
 * vrwkv_biwkv_forward_f32 for callers that cannot allocate device memory and so have no
 * workspace to pass (a host that owns all device memory and lends only inputs and outputs,
 * a loop running under a frozen memory plan, code inside a region where allocation is
 * forbidden).  Its scratch is a 16 MiB array built into the library's device image, present
 * once on every GPU that loads the library until the process exits.
 *   - A shape is accepted when B * ceil(T / 16) * 24 * C bytes fit in 16 MiB (for example
 *     B=2, T=196, C=192, or B=4, T=1024, C=768); larger shapes return VRWKV_ERR_WORKSPACE.
 *   - The first call on a device also looks up the array's device address; make that call
 *     before starting any stream capture.  No call allocates or frees.
 *   - All calls on a device share the array: two calls that can overlap on the GPU (different
 *     streams with no ordering between them) race; calls on one stream do not.
 * Results equal vrwkv_biwkv_forward_f32's generic path bit for bit. */
int vrwkv_biwkv_forward_f32_noalloc(int B, int T, int C, const float* w, const float* u,
                                    const float* k, const float* v, float* y, void* stream);

/* ---- WKV6 (bidirectional, head size 64) ---------------------------------------------
 * Per (batch, head), state S in R^{64x64} [key][value], d_t = exp(-exp(w_raw_t)):
 *   S>_{t+1} = diag(d_t) S>_t + k_t v_t^T,  S<_{t-1} = diag(d_t) S<_t + k_t v_t^T
 *   y_t = r_t^T (S>_t + diag(u) k_t v_t^T) + r_t^T S<_t
 * r, k, v, w_raw, y, gy and the gradients are (B, T, C) with C = 64 H; u and gu are (H, 64).
 * Inputs must be 16-byte aligned.
 *
 * vrwkv_wkv6_forward_f32 replaces
 *   cuda_forward(int B,int T,int C,int H,float*r,float*k,float*v,float*w,float*u,float*y)
 *       CLS/cuda_v6/wkv6_op.cpp:4,7-9 (kernel CLS/cuda_v6/wkv6_cuda.cu:6-97,348-353)
 * It takes the raw decay input and forms -exp(w_raw) itself, where the reference's Python
 * wrapper does that in a separate pass (CLS/vrwkv6.py:48).
 */
int vrwkv_wkv6_forward_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                           const float* w_raw, const float* u, float* y, void* stream);

/* vrwkv_wkv6_forward_tc_f32: the same forward on the tensor cores (tcgen05, state in tensor
 * memory): r, k, v and the state copy enter the matrix products rounded to bfloat16, sums are
 * fp32.  Results agree with vrwkv_wkv6_forward_f32 to about 1e-2 of max|y|: meant for callers
 * whose r, k, v are bfloat16 already.  `workspace`: 256 bytes, 256-byte aligned; its first word is
 * a status word as in vrwkv_workspace_status.  Stands in for the same reference entry point as
 * vrwkv_wkv6_forward_f32. */
int vrwkv_wkv6_forward_tc_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                              const float* w_raw, const float* u, float* y, void* workspace,
                              size_t workspace_bytes, void* stream);
/* The same kernel for callers whose r, k, v are bfloat16 (uint16_t bit patterns; the usual case
 * under autocast): the tiles are read as bfloat16, so the `.float()` passes in front of the
 * reference's call (CLS/vrwkv6.py:220 hands whatever dtype the projections produced to a kernel
 * that reads float) disappear.  w_raw, u and y stay float32. */
int vrwkv_wkv6_forward_tc_bf16(int B, int T, int C, int H, const uint16_t* r, const uint16_t* k,
                               const uint16_t* v, const float* w_raw, const float* u, float* y,
                               void* workspace, size_t workspace_bytes, void* stream);

/* vrwkv_wkv6_backward_f32 replaces
 *   cuda_backward(int B,int T,int C,int H,float*r,...,float*gy,float*gr,float*gk,float*gv,
 *                 float*gw,float*gu)
 *       CLS/cuda_v6/wkv6_op.cpp:5,10-12 (kernels CLS/cuda_v6/wkv6_cuda.cu:99-346,355-362)
 * without its T <= 256 limit.  gw is the gradient w.r.t. w_raw (as in the reference, whose
 * kernels multiply by -exp(w_raw)); gu is already summed over batch (the reference returns
 * (B, C) and sums in Python, CLS/vrwkv6.py:69).  gv may be NULL: the value gradient is then left
 * out (a third of the work); by the symmetry of the operator it equals the forward applied to
 * (r, k, v) := (k, r, gy), which a half-precision caller can take from vrwkv_wkv6_forward_tc_*.
 */
size_t vrwkv_wkv6_backward_workspace_bytes(int B, int T, int C, int H);
int vrwkv_wkv6_backward_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                            const float* w_raw, const float* u, const float* gy, float* gr, float* gk,
                            float* gv, float* gw, float* gu, void* workspace, size_t workspace_bytes,
                            void* stream);

/* The same gradients on the tensor cores (tcgen05, states in tensor memory), for callers whose
 * activations are half precision anyway: r, k, v, gy enter the matrix products rounded to bfloat16,
 * sums are fp32; results agree with vrwkv_wkv6_backward_f32 to about 1e-2 of each tensor's maximum.
 * gv is the forward kernel applied to (k, r, gy); gr and gk come from a second kernel of the same
 * block structure; gw and gu from their one-sided sums.  vrwkv_wkv6_backward_tc_bf16 reads r, k, v,
 * gy as bfloat16 bit patterns directly (the reference hands whatever dtype the projections produced
 * to kernels that read float, CLS/vrwkv6.py:60-70, so a half-precision caller pays widening passes
 * there).  All gradients are float32; gw is w.r.t. w_raw; gu is summed over batch.  They stand in for
 * the same reference entry point as vrwkv_wkv6_backward_f32 (CLS/cuda_v6/wkv6_op.cpp:5,10-12). */
size_t vrwkv_wkv6_backward_tc_workspace_bytes(int B, int T, int C, int H);
int vrwkv_wkv6_backward_tc_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                               const float* w_raw, const float* u, const float* gy, float* gr, float* gk, float* gv,
                               float* gw, float* gu, void* workspace, size_t workspace_bytes, void* stream);
int vrwkv_wkv6_backward_tc_bf16(int B, int T, int C, int H, const uint16_t* r, const uint16_t* k, const uint16_t* v,
                                const float* w_raw, const float* u, const uint16_t* gy, float* gr, float* gk, float* gv,
                                float* gw, float* gu, void* workspace, size_t workspace_bytes, void* stream);

/* ---- Q-Shift + token-mix interpolation (the step in front of the K/V/R projections) ----
 * x is (B, H*W, C), tokens in raster order.  xx = x with channel group g (`group` channels
 * each, group = int(C * channel_gamma)) moved by `shift` pixels: g=0 right, g=1 left, g=2 down,
 * g=3 up, zero fill at the image border, channels beyond 4*group copied.  Outputs
 * out[m] = x * mix[m] + xx * (1 - mix[m]), m < n_out (1..3), mix[m] of shape (C,).
 * `mix`, `out`, `gout`, `gmix` are host arrays of n_out device pointers.
 *
 * Replaces the tensor-op sequence q_shift(...) followed by the n_out lerps of
 *   VRWKV_SpatialMix.jit_func   CLS/vrwkv.py:156-164  (n_out = 3: xk, xv, xr)
 *   VRWKV_ChannelMix.forward    CLS/vrwkv.py:247-250  (n_out = 2: xk, xr)
 *   q_shift                     CLS/vrwkv.py:68-79
 * The backward returns gx and gmix[m] (C,), the latter summed over batch and tokens in a
 * fixed order. */
int vrwkv_qshift_mix_forward_f32(int B, int H, int W, int C, int group, int shift, int n_out,
                                 const float* x, const float* const* mix, float* const* out,
                                 void* stream);
size_t vrwkv_qshift_mix_backward_workspace_bytes(int B, int H, int W, int C, int n_out);
int vrwkv_qshift_mix_backward_f32(int B, int H, int W, int C, int group, int shift, int n_out,
                                  const float* x, const float* const* mix, const float* const* gout,
                                  float* gx, float* const* gmix, void* workspace, size_t workspace_bytes,
                                  void* stream);

/* The per-head shift of VRWKV6 (q_shift_multihead, CLS/vrwkv6.py:75-101) fused with the same
 * interpolations (VRWKV_ChannelMix of vrwkv6.py: xk, xr): within every head of head_dim channels
 * the four quarters take the left, right, upper and lower neighbour.  head_dim is a multiple of 4
 * that divides C.  Workspace of the backward: vrwkv_qshift_mix_backward_workspace_bytes. */
int vrwkv_qshift_multihead_mix_forward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out,
                                           const float* x, const float* const* mix, float* const* out,
                                           void* stream);
int vrwkv_qshift_multihead_mix_backward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out,
                                            const float* x, const float* const* mix,
                                            const float* const* gout, float* gx, float* const* gmix,
                                            void* workspace, size_t workspace_bytes, void* stream);

/* The per-head shift fused with the data-dependent interpolations of the VRWKV6 spatial mix
 * (CLS/vrwkv6.py:75-100, 180-193):  out_j = x + (q_shift_multihead(x) - x) * (maa_j[c] + m_j[b,t,c]),
 * j < n_out <= 5.  maa: n_out device pointers to (C,) float vectors; m: n_out device pointers to
 * (B, H*W, C) per-token offsets, float32 or (m_is_bf16 != 0) bfloat16 bit patterns, any of them NULL
 * for "no offset" (n_out = 1 with m[0] = NULL is xxx = x + xx * time_maa_x; n_out = 5 gives the inputs
 * of the w, k, v, r, g branches).  head_dim: a multiple of 16 that divides C.  The backward returns gx,
 * the offset gradients gm_j (dtype of m; NULL exactly where m_j is NULL) and the (C,) gradients gmaa_j,
 * summed in a fixed order.  All tensors 16-byte aligned (bfloat16 ones 8). */
int vrwkv_qshift_ddlerp_forward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out, const float* x,
                                    const float* const* maa, const void* const* m, int m_is_bf16, float* const* out,
                                    void* stream);
size_t vrwkv_qshift_ddlerp_backward_workspace_bytes(int B, int H, int W, int C, int n_out);
int vrwkv_qshift_ddlerp_backward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out, const float* x,
                                     const float* const* maa, const void* const* m, int m_is_bf16,
                                     const float* const* gout, float* gx, void* const* gm, float* const* gmaa,
                                     void* workspace, size_t workspace_bytes, void* stream);

/* Normalise-and-gate epilogue behind the two operators, one pass forward and one backward:
 *   out = (normalise(x) * gamma + beta) * gate
 * over rows of C channels; group == C is the LayerNorm + sigmoid gate behind Bi-WKV in the large
 * backbone (key_norm, then sr * x: CLS/vrwkv.py:184-186), group == 64 the per-head GroupNorm + SiLU
 * gate behind WKV6 (ln_x, then x * g: CLS/vrwkv6.py:133, 205-212).  The reference runs them as a
 * normalisation pass and a multiply pass (and an activation pass before them).  `gate` holds, float32 or
 * (gate_is_bf16 != 0) bfloat16 bit patterns, the gate itself (gate_act 0), or the projection whose sigmoid
 * (gate_act 1) or SiLU (gate_act 2) is the gate - the backward then returns the gradient of that projection; x, out, gamma, beta float32; mean and rstd receive
 * rows * C / group floats each for the backward.  group must be a multiple of 64, at most 1024, and
 * divide C (else VRWKV_ERR_UNSUPPORTED); pointers 8-byte aligned.  Biased variance, eps inside the
 * square root, as torch.nn.LayerNorm / GroupNorm.  The backward returns gx, ggate (dtype of gate) and
 * ggamma | gbeta as one (2, C) float buffer, summed in a fixed order. */
int vrwkv_normgate_forward_f32(int rows, int C, int group, float eps, const float* x, const void* gate,
                               int gate_is_bf16, int gate_act, const float* gamma, const float* beta, float* out,
                               float* mean, float* rstd, void* stream);
size_t vrwkv_normgate_backward_workspace_bytes(int rows, int C, int group);
int vrwkv_normgate_backward_f32(int rows, int C, int group, const float* gout, const float* x, const void* gate,
                                int gate_is_bf16, int gate_act, const float* gamma, const float* beta, const float* mean,
                                const float* rstd, float* gx, void* ggate, float* ggamma_gbeta, void* workspace,
                                size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VRWKV_B200_H_ */
