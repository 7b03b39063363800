// Declarations shared between the C-ABI translation unit and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <initializer_list>

// Remember a one-line explanation of the most recent failure (read by vrwkv_last_error_detail).
void set_error_detail(const char* text);
// Add `launched` kernels to the process-wide count and turn the CUDA error state into a status.
int record_launches(int launched);

namespace biwkv {
// Each launcher returns the number of kernels it enqueued.
size_t generic_forward_workspace(int B, int T, int C);
size_t generic_backward_workspace(int B, int T, int C);
int generic_forward(int B, int T, int C, const float* w, const float* u, const float* k,
                    const float* v, float* y, void* workspace, cudaStream_t stream);
int generic_backward(int B, int T, int C, const float* w, const float* u, const float* k,
                     const float* v, const float* gy, float* gwgu, float* gk, float* gv,
                     void* workspace, cudaStream_t stream);
namespace resident {
// Cluster-resident single-pass path (biwkv_resident.cu): float32 (C % 4 == 0) or bfloat16 (C % 8 == 0)
// tensors, 16-byte aligned, T <= 4096.  True when it can serve this call on the current device.
bool eligible(int B, int T, int C, std::initializer_list<const void*> ptrs, bool bwd, bool bf16 = false);
void set_withhold_test(bool on);   // test only: one rank per cluster sends nothing, waits give up early
size_t workspace_bytes(int B, int T, int C, bool bwd);
// Sequences longer than one cluster holds (T > 4096) run as several clusters per sequence.  Inputs outside the
// plain-float range then leave workspace word 1 non-zero instead of results: the caller follows up with the
// chunked kernels switched on by that word.
bool multi_segment(int T);
int forward(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
            float* y, void* workspace, cudaStream_t stream);
int backward(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
             const float* gy, float* gwgu, float* gk, float* gv, void* workspace,
             cudaStream_t stream);
// k, v, y, gy, gk, gv hold bfloat16; w, u, gwgu stay float; arithmetic and shared-memory state are the float kernels'.
int forward_bf16(int B, int T, int C, const float* w, const float* u, const void* k, const void* v, void* y,
                 void* workspace, cudaStream_t stream);
int backward_bf16(int B, int T, int C, const float* w, const float* u, const void* k, const void* v,
                  const void* gy, float* gwgu, void* gk, void* gv, void* workspace, cudaStream_t stream);
}  // namespace resident
namespace fused {
// True when the fused TMA path can serve this call on the current device.
bool eligible(int B, int T, int C, std::initializer_list<const void*> ptrs, bool bf16 = false);
size_t workspace_bytes(int B, int T, int C, bool bwd);
// run_if: when set, every kernel of the launch returns at once while that device word is zero.
int forward(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
            float* y, void* workspace, cudaStream_t stream, const unsigned* run_if = nullptr);
int backward(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
             const float* gy, float* gwgu, float* gk, float* gv, void* workspace,
             cudaStream_t stream, const unsigned* run_if = nullptr);
// Forward that also writes log Den (one float per element), and the backward that starts from the
// saved y and log Den: one exchange level instead of two.
bool eligible_saved(int B, int T, int C, std::initializer_list<const void*> ptrs);
int forward_save(int B, int T, int C, const float* w, const float* u, const float* k, const float* v, float* y,
                 float* logden, void* workspace, cudaStream_t stream);
int backward_saved(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
                   const float* gy, const float* y, const float* logden, float* gwgu, float* gk, float* gv,
                   void* workspace, cudaStream_t stream);
// k, v, y, gy, gk, gv hold bfloat16; w, u, gwgu stay float; arithmetic is the float kernels'.
int forward_bf16(int B, int T, int C, const float* w, const float* u, const void* k, const void* v, void* y,
                 void* workspace, cudaStream_t stream, const unsigned* run_if = nullptr);
int backward_bf16(int B, int T, int C, const float* w, const float* u, const void* k, const void* v,
                  const void* gy, float* gwgu, void* gk, void* gv, void* workspace, cudaStream_t stream,
                  const unsigned* run_if = nullptr);
}  // namespace fused
}  // namespace biwkv

namespace wkv6 {
size_t backward_workspace(int B, int T, int H);
int forward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw,
            const float* u, float* y, cudaStream_t stream);
int backward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw,
             const float* u, const float* gy, float* gr, float* gk, float* gv, float* gw, float* gu,
             void* workspace, cudaStream_t stream);
}  // namespace wkv6

namespace wkv6tc {
// Tensor-core forward (bf16 operands, fp32 state).  `status` points at 4 writable device bytes.
// pipelined = false runs the first-generation kernel (all warps do every phase in turn).
int forward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw,
            const float* u, float* y, unsigned* status, bool pipelined, cudaStream_t stream);
// r, k, v in bfloat16 (read as such by the kernel: no widening pass), w_raw, u, y float32.
int forward_bf16in(int B, int T, int H, const void* r, const void* k, const void* v, const float* w_raw,
                   const float* u, float* y, unsigned* status, cudaStream_t stream);
// Tensor-core backward: gv through the forward kernel with permuted operands, gr and gk through a
// token-mixing kernel of the same structure, gw and gu from their one-sided sums.  half_in: r, k, v, gy
// point at bfloat16 (read as such).  Gradients are float32.
size_t backward_workspace(int B, int T, int H);
int backward(int B, int T, int H, const void* r, const void* k, const void* v, const float* w_raw, const float* u,
             const void* gy, float* gr, float* gk, float* gv, float* gw, float* gu, void* workspace, bool half_in,
             cudaStream_t stream);
}  // namespace wkv6tc
