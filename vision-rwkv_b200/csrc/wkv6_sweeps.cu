// WKV6 (head size 64, bidirectional) as exact sequential state sweeps, fp32, any T.
//
// Per (batch, head) the operator carries a 64 x 64 state S[key i][value j]
//   rightward  S>_{t+1} = diag(d_t) S>_t + k_t v_t^T      y_t  = r_t^T (S>_t + diag(u) k_t v_t^T)
//   leftward   S<_{t-1} = diag(d_t) S<_t + k_t v_t^T      y_t += r_t^T S<_t
// with d_t = exp(-exp(w_raw_t)).  The gradients need the states S and their adjoints
// A = dL/dS (rightward adjoint runs backwards in time, A>_t = r_t gy_t^T + diag(d_t) A>_{t+1},
// and mirrored for the leftward direction):
//   gr_t = S_t gy_t (+ bonus)   gk_t = A_{t+1} v_t (+ bonus)   gv_t = A_{t+1}^T k_t (+ bonus)
// Every one of these is "read out a 64-vector product of the state, then update the state
// by a decayed rank-1 term", so one sweep engine serves them all.  A block of 64 threads
// owns either the rows (thread = key channel) or the columns (thread = value channel) of
// one state, whichever makes the read-out a sum inside the thread, and keeps its 64 state
// values in registers.  Tokens arrive in shared memory 16 at a time through cp.async,
// double-buffered.  One block runs the rightward pass and then the leftward one of its
// kind and adds the second result to the first itself, so outputs are written without
// atomics and are bit-reproducible.
//
// Decay gradient.  With p_t = r_t * (S_t gy_t) and q_t = k_t * (A_{t+1} v_t) (state parts
// only, elementwise over key channels),
//   d_t * dL/dd_t = sum_{tau>t} p>_tau - sum_{tau>=t} q>_tau + sum_{tau<t} p<_tau - sum_{tau<=t} q<_tau
// (every (source, reader) token pair whose decay product contains d_t, counted from the
// reader side minus the pairs that do not straddle t).  The sweeps write running sums of
// p and q (accumulated in double) to scratch; a last elementwise kernel combines them and
// applies d(d_t)/d(w_raw) = d_t * (-exp(w_raw)), which cancels the division by d_t.
//
// Reference being replaced: classification/mmcls_custom/models/backbones/cuda_v6/
// wkv6_cuda.cu:6-97 (forward), :99-346 (backward; its T <= 256 limit does not apply here).
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include "vrwkv_internal.h"

namespace wkv6 {

constexpr int N = 64;          // head size
constexpr int kBatch = 8;      // tokens per shared-memory batch (two batches of 10 KB per block: 11 blocks per SM)
constexpr int kParts = N / kBatch;   // threads that share one token's dot products
constexpr int kVecs = 5;       // r, k, v, gy, decay
enum Kind { KIND_Y = 0, KIND_GR = 1, KIND_GK = 2, KIND_GV = 3 };
enum Vec { V_R = 0, V_K = 1, V_V = 2, V_G = 3, V_D = 4 };

struct Args {
    int B, T, H;
    const float* src[kVecs];   // r, k, v, gy (null in the forward), w_raw  -- (B, T, 64 H)
    const float* u;            // (H, 64)
    float* out[4];             // by kind: y, gr, gk, gv
    float* cum[4];             // running sums: p> (prefix), q> (suffix), p< (suffix), q< (prefix)
    float* gu_part;            // (B, 64 H)
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

struct Batch {
    float vec[kVecs][kBatch][N];
    float vg[kBatch];    // v_t . gy_t
    float ruk[kBatch];   // sum_i r_t[i] u[i] k_t[i]
};

// One pass of one kind over the whole sequence.  kRow: thread owns a row (key channel) of
// the state, else a column (value channel).  kForward: direction of time.  kOut: how the result
// meets the other direction's: OUT_WRITE (first pass of a block), OUT_ADD (second pass of the same
// block), OUT_ATOMIC (the two directions run in two blocks and add into a zeroed output: exactly
// two addends per element, so the sum does not depend on their order).  kFirst: first
// pass of the block (writes its output; the second pass adds to it).
enum OutMode { OUT_WRITE = 0, OUT_ADD = 1, OUT_ATOMIC = 2 };
template <int kKind, bool kForward, int kOut>
__device__ __forceinline__ void sweep(const Args& a, Batch* buf, int b, int h, float u_self, const float* u_smem,
                                      float& gu_acc) {
    constexpr bool kRow = (kKind == KIND_GR || kKind == KIND_GK);
    constexpr int kA = (kKind == KIND_Y || kKind == KIND_GR) ? V_K : V_R;   // rank-1 update: alpha beta^T
    constexpr int kB_ = (kKind == KIND_Y || kKind == KIND_GR) ? V_V : V_G;
    constexpr int kC = kKind == KIND_Y ? V_R : kKind == KIND_GR ? V_G : kKind == KIND_GK ? V_V : V_K;   // read-out
    // the rightward state S> runs forward in time, its adjoint A> backward; mirrored for "<"
    constexpr bool kRightward = (kKind == KIND_Y || kKind == KIND_GR) ? kForward : !kForward;
    const int tid = threadIdx.x;
    const int T = a.T, C = a.H * N;
    const size_t base = (static_cast<size_t>(b) * T) * C + static_cast<size_t>(h) * N;
    const int n_batches = (T + kBatch - 1) / kBatch;

    auto issue = [&](int bi, Batch* dst) {
        const int bt0 = (kForward ? bi : n_batches - 1 - bi) * kBatch;
#pragma unroll
        for (int vsel = 0; vsel < kVecs; ++vsel) {
            const float* src = a.src[vsel];
            if (src == nullptr) continue;
#pragma unroll
            for (int q = 0; q < (kBatch * N / 4) / N; ++q) {          // 256 chunks of 16 B, 64 threads
                const int chunk = q * N + tid;
                const int row = chunk >> 4, col4 = (chunk & 15) * 4;      // 16 chunks of 16 bytes per token row
                const int t = bt0 + row;
                if (t < T) cp_async16(&dst->vec[vsel][row][col4], src + base + static_cast<size_t>(t) * C + col4);
            }
        }
        cp_async_commit();
    };

    float X[N];
#pragma unroll
    for (int n = 0; n < N; ++n) X[n] = 0.f;
    double run = 0.0;

    issue(0, &buf[0]);
    for (int bi = 0; bi < n_batches; ++bi) {
        Batch* cur = &buf[bi & 1];
        if (bi + 1 < n_batches) {
            issue(bi + 1, &buf[(bi + 1) & 1]);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int bt0 = (kForward ? bi : n_batches - 1 - bi) * kBatch;
        const int rows = min(kBatch, T - bt0);
        // decay in place, per-token scalars
        for (int row = 0; row < rows; ++row) cur->vec[V_D][row][tid] = expf(-expf(cur->vec[V_D][row][tid]));
        {
            const int row = tid / kParts, part = tid % kParts;
            float s1 = 0.f, s2 = 0.f;
            if (row < rows) {
#pragma unroll
                for (int n = part * kBatch; n < part * kBatch + kBatch; ++n) {
                    if (a.src[V_G] != nullptr) s1 += cur->vec[V_V][row][n] * cur->vec[V_G][row][n];
                    s2 += cur->vec[V_R][row][n] * u_smem[n] * cur->vec[V_K][row][n];
                }
            }
#pragma unroll
            for (int m = 1; m < kParts; m <<= 1) {
                s1 += __shfl_xor_sync(0xffffffffu, s1, m);
                s2 += __shfl_xor_sync(0xffffffffu, s2, m);
            }
            if (part == 0 && row < kBatch) { cur->vg[row] = s1; cur->ruk[row] = s2; }
        }
        __syncthreads();
        for (int step = 0; step < rows; ++step) {
            const int row = kForward ? step : rows - 1 - step;
            const int t = bt0 + row;
            const float4* cv = reinterpret_cast<const float4*>(cur->vec[kC][row]);
            float out = 0.f;
            if (kRow) {
                const float di = cur->vec[V_D][row][tid];
                const float ai = cur->vec[kA][row][tid];
                const float4* bv = reinterpret_cast<const float4*>(cur->vec[kB_][row]);
#pragma unroll
                for (int n4 = 0; n4 < N / 4; ++n4) {
                    const float4 c4 = cv[n4], b4 = bv[n4];
                    out += c4.x * X[4 * n4 + 0]; X[4 * n4 + 0] = fmaf(di, X[4 * n4 + 0], ai * b4.x);
                    out += c4.y * X[4 * n4 + 1]; X[4 * n4 + 1] = fmaf(di, X[4 * n4 + 1], ai * b4.y);
                    out += c4.z * X[4 * n4 + 2]; X[4 * n4 + 2] = fmaf(di, X[4 * n4 + 2], ai * b4.z);
                    out += c4.w * X[4 * n4 + 3]; X[4 * n4 + 3] = fmaf(di, X[4 * n4 + 3], ai * b4.w);
                }
            } else {
                const float bj = cur->vec[kB_][row][tid];
                const float4* av = reinterpret_cast<const float4*>(cur->vec[kA][row]);
                const float4* dv = reinterpret_cast<const float4*>(cur->vec[V_D][row]);
#pragma unroll
                for (int n4 = 0; n4 < N / 4; ++n4) {
                    const float4 c4 = cv[n4], a4 = av[n4], d4 = dv[n4];
                    out += c4.x * X[4 * n4 + 0]; X[4 * n4 + 0] = fmaf(d4.x, X[4 * n4 + 0], a4.x * bj);
                    out += c4.y * X[4 * n4 + 1]; X[4 * n4 + 1] = fmaf(d4.y, X[4 * n4 + 1], a4.y * bj);
                    out += c4.z * X[4 * n4 + 2]; X[4 * n4 + 2] = fmaf(d4.z, X[4 * n4 + 2], a4.z * bj);
                    out += c4.w * X[4 * n4 + 3]; X[4 * n4 + 3] = fmaf(d4.w, X[4 * n4 + 3], a4.w * bj);
                }
            }
            const size_t idx = base + static_cast<size_t>(t) * C + tid;
            // running sums for the decay gradient (state part only)
            if (kKind == KIND_GR) {
                run += static_cast<double>(cur->vec[V_R][row][tid] * out);
                a.cum[kRightward ? 0 : 2][idx] = static_cast<float>(run);
            }
            if (kKind == KIND_GK) {
                run += static_cast<double>(cur->vec[V_K][row][tid] * out);
                a.cum[kRightward ? 1 : 3][idx] = static_cast<float>(run);
            }
            // the bonus term lives in the rightward direction only
            if (kRightward) {
                if (kKind == KIND_Y) out += cur->ruk[row] * cur->vec[V_V][row][tid];
                if (kKind == KIND_GV) out += cur->ruk[row] * cur->vec[V_G][row][tid];
                if (kKind == KIND_GR) {
                    const float kvg = cur->vec[V_K][row][tid] * cur->vg[row];
                    out += u_self * kvg;
                    gu_acc += cur->vec[V_R][row][tid] * kvg;
                }
                if (kKind == KIND_GK) out += u_self * cur->vec[V_R][row][tid] * cur->vg[row];
            }
            float* dst = a.out[kKind] + idx;
            if (kOut == OUT_WRITE) *dst = out;
            else if (kOut == OUT_ADD) *dst += out;
            else atomicAdd(dst, out);
        }
        __syncthreads();   // the batch buffer is refilled two iterations later
    }
}

// kSplit: blockIdx.z picks the direction and the two blocks of a (batch, head, kind) add into a zeroed
// output; otherwise one block runs both directions in turn.
template <bool kBackward, bool kSplit>
__global__ void __launch_bounds__(N, 9) wkv6_sweep_kernel(const Args a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Batch* buf = reinterpret_cast<Batch*>(smem_raw);
    __shared__ float u_smem[N];
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int kind = kBackward ? 1 + static_cast<int>(blockIdx.y) : 0;
    const int tid = threadIdx.x;
    u_smem[tid] = a.u[h * N + tid];
    __syncthreads();
    const float u_self = u_smem[tid];
    float gu = 0.f;
    constexpr int kOut1 = kSplit ? OUT_ATOMIC : OUT_WRITE, kOut2 = kSplit ? OUT_ATOMIC : OUT_ADD;
    const bool first = !kSplit || blockIdx.z == 0, second = !kSplit || blockIdx.z == 1;
    if (!kBackward) {
        if (first) sweep<KIND_Y, false, kOut1>(a, buf, b, h, u_self, u_smem, gu);   // leftward state first
        if (second) sweep<KIND_Y, true, kOut2>(a, buf, b, h, u_self, u_smem, gu);
    } else if (kind == KIND_GR) {
        if (first) {
            sweep<KIND_GR, true, kOut1>(a, buf, b, h, u_self, u_smem, gu);
            a.gu_part[static_cast<size_t>(b) * a.H * N + h * N + tid] = gu;            // the bonus lives in this direction
        }
        if (second) sweep<KIND_GR, false, kOut2>(a, buf, b, h, u_self, u_smem, gu);
    } else if (kind == KIND_GK) {
        if (first) sweep<KIND_GK, false, kOut1>(a, buf, b, h, u_self, u_smem, gu);  // rightward adjoint: back in time
        if (second) sweep<KIND_GK, true, kOut2>(a, buf, b, h, u_self, u_smem, gu);
    } else {
        if (first) sweep<KIND_GV, false, kOut1>(a, buf, b, h, u_self, u_smem, gu);
        if (second) sweep<KIND_GV, true, kOut2>(a, buf, b, h, u_self, u_smem, gu);
    }
}

// gw_raw = -exp(w_raw) * [ (P>_last - P>_t - Q>_t) + (P<_first - P<_t - Q<_t) ]
__global__ void wkv6_decay_grad_kernel(int B, int T, int C, const float* __restrict__ w_raw,
                                       const float* __restrict__ cp, const float* __restrict__ cq,
                                       const float* __restrict__ cp2, const float* __restrict__ cq2,
                                       float* __restrict__ gw) {
    const size_t total = static_cast<size_t>(B) * T * C;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t c = i % C;
        const size_t b = i / (static_cast<size_t>(T) * C);
        const size_t first = b * T * C + c, last = first + static_cast<size_t>(T - 1) * C;
        const float right = (cp[last] - cp[i]) - cq[i];
        const float left = (cp2[first] - cp2[i]) - cq2[i];
        gw[i] = -expf(w_raw[i]) * (right + left);
    }
}

// gu[c] = sum over batch of gu_part[b][c], fixed order
__global__ void wkv6_bonus_grad_kernel(int B, int C, const float* __restrict__ part, float* __restrict__ gu) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float acc = 0.f;
    for (int b = 0; b < B; ++b) acc += part[static_cast<size_t>(b) * C + c];
    gu[c] = acc;
}

// Blocks of the sweep kernel that fit the device at once (0 if the kernel cannot be configured).
static int resident_blocks() {
    static int cached[64];
    static bool known[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    if (!known[dev]) {
        const int smem = static_cast<int>(2 * sizeof(Batch));
        bool ok = cudaFuncSetAttribute(wkv6_sweep_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                  cudaFuncSetAttribute(wkv6_sweep_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                  cudaFuncSetAttribute(wkv6_sweep_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
                  cudaFuncSetAttribute(wkv6_sweep_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess;
        int per_sm = 0, sms = 0;
        ok = ok && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, wkv6_sweep_kernel<true, false>, N, smem) == cudaSuccess;
        ok = ok && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
        if (!ok) cudaGetLastError();
        cached[dev] = ok ? per_sm * sms : 0;
        known[dev] = true;
    }
    return cached[dev];
}
static bool configure() { return resident_blocks() > 0; }

// The two directions of a (batch, head, kind) go to two blocks when that still fits the device in
// one wave: the walks are latency-bound, so twice the blocks is close to twice the speed then.
static bool split_directions(int blocks) { return 2 * blocks <= resident_blocks(); }

size_t backward_workspace(int B, int T, int H) {
    const size_t E = static_cast<size_t>(B) * T * H * N;
    return (4 * E + static_cast<size_t>(B) * H * N) * sizeof(float);
}

int forward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw,
            const float* u, float* y, cudaStream_t stream) {
    if (!configure()) return -1;
    Args a{};
    a.B = B; a.T = T; a.H = H;
    a.src[V_R] = r; a.src[V_K] = k; a.src[V_V] = v; a.src[V_G] = nullptr; a.src[V_D] = w_raw;
    a.u = u;
    a.out[KIND_Y] = y;
    if (split_directions(B * H)) {
        cudaMemsetAsync(y, 0, static_cast<size_t>(B) * T * H * N * sizeof(float), stream);
        wkv6_sweep_kernel<false, true><<<dim3(B * H, 1, 2), N, 2 * sizeof(Batch), stream>>>(a);
    } else {
        wkv6_sweep_kernel<false, false><<<dim3(B * H), N, 2 * sizeof(Batch), stream>>>(a);
    }
    return 1;
}

int backward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw,
             const float* u, const float* gy, float* gr, float* gk, float* gv, float* gw, float* gu,
             void* workspace, cudaStream_t stream) {
    if (!configure()) return -1;
    const int C = H * N;
    const size_t E = static_cast<size_t>(B) * T * C;
    float* ws = static_cast<float*>(workspace);
    Args a{};
    a.B = B; a.T = T; a.H = H;
    a.src[V_R] = r; a.src[V_K] = k; a.src[V_V] = v; a.src[V_G] = gy; a.src[V_D] = w_raw;
    a.u = u;
    a.out[KIND_GR] = gr; a.out[KIND_GK] = gk; a.out[KIND_GV] = gv;
    for (int i = 0; i < 4; ++i) a.cum[i] = ws + i * E;
    a.gu_part = ws + 4 * E;
    const int kinds = gv ? 3 : 2;      // gv == nullptr: the caller gets gv elsewhere (the kinds are gr, gk, gv in this order)
    if (split_directions(kinds * B * H)) {
        cudaMemsetAsync(gr, 0, E * sizeof(float), stream);
        cudaMemsetAsync(gk, 0, E * sizeof(float), stream);
        if (gv) cudaMemsetAsync(gv, 0, E * sizeof(float), stream);
        wkv6_sweep_kernel<true, true><<<dim3(B * H, kinds, 2), N, 2 * sizeof(Batch), stream>>>(a);
    } else {
        wkv6_sweep_kernel<true, false><<<dim3(B * H, kinds), N, 2 * sizeof(Batch), stream>>>(a);
    }
    const int blocks = static_cast<int>(std::min<size_t>((E + 255) / 256, 148 * 16));
    wkv6_decay_grad_kernel<<<blocks, 256, 0, stream>>>(B, T, C, w_raw, a.cum[0], a.cum[1], a.cum[2], a.cum[3], gw);
    wkv6_bonus_grad_kernel<<<(C + 127) / 128, 128, 0, stream>>>(B, C, a.gu_part, gu);
    return 3;
}

}  // namespace wkv6
