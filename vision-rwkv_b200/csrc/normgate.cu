// Normalise-and-gate epilogue of the token-mixing operators, forward and backward, one pass each.
//
// Behind Bi-WKV the large backbone applies a LayerNorm over the channels to the operator's output
// and multiplies by the sigmoid gate before the output projection
// (classification/mmcls_custom/models/backbones/vrwkv.py:184-186: key_norm, then sr * x); behind
// WKV6 a GroupNorm with one group per 64-channel head is followed by the SiLU gate
// (classification/mmcls_custom/models/backbones/vrwkv6.py:133, 205-212: ln_x, then x * g).  With
// tensor ops that is a normalisation pass (read, write) and a multiply pass (two reads, a write);
// here out = (normalise(x) * gamma + beta) * gate is one pass that reads x and gate once and writes
// out, and the backward reads gout, x, gate once and writes gx and ggate; the affine parameters'
// gradients are accumulated per warp in registers and summed in a fixed order (no atomics).
//
// group = C is LayerNorm, group = 64 is the per-head GroupNorm.  One warp per (row, group); a lane
// holds the channel pairs (64 i + 2 lane, +1) of the group, so a warp reads 256 contiguous bytes per
// step.  Biased variance in two passes over registers, eps inside the square root, as
// torch.nn.LayerNorm / GroupNorm compute it.  `gate` may hold the gate itself or the projection it is the
// sigmoid / SiLU of (then the activation and its derivative are applied here too, one more pass saved), in
// float32 or bfloat16; x, out and the statistics are float32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "vrwkv_b200.h"
#include "vrwkv_internal.h"

namespace normgate {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxPairs = 16;          // channel pairs per lane: groups of up to 1024 channels
constexpr int kMaxGroup = kMaxPairs * 64;

struct Args {
    int rows, C, G, n_groups, pairs;   // pairs = G / 64
    int act;                           // what `gate` holds: 0 the gate itself, 1 the input of a sigmoid, 2 the input of a SiLU
    float eps;
    const float* x;
    const void* gate;
    const float* gamma;
    const float* beta;
    float* out;
    float* mean;      // (rows, n_groups)
    float* rstd;
    // backward
    const float* gout;
    float* gx;
    void* ggate;
    float* partial;   // [gridDim.x][2][C]
};

template <bool kHalfGate>
__device__ __forceinline__ float2 load_gate(const void* gate, size_t at) {
    if (kHalfGate) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(static_cast<const __nv_bfloat16*>(gate) + at));
    return *reinterpret_cast<const float2*>(static_cast<const float*>(gate) + at);
}
template <bool kHalfGate>
__device__ __forceinline__ void store_gate(void* gate, size_t at, float2 v) {
    if (kHalfGate) *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(gate) + at) = __float22bfloat162_rn(v);
    else *reinterpret_cast<float2*>(static_cast<float*>(gate) + at) = v;
}
// the gate from what was loaded (act as in Args), and its derivative with respect to what was loaded
__device__ __forceinline__ float gate_value(float x, int act) {
    if (act == 0) return x;
    const float s = 1.f / (1.f + __expf(-x));
    return act == 1 ? s : x * s;
}
__device__ __forceinline__ float gate_slope(float x, int act) {
    if (act == 0) return 1.f;
    const float s = 1.f / (1.f + __expf(-x));
    return act == 1 ? s * (1.f - s) : s * (1.f + x * (1.f - s));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// kPairs: channel pairs a lane can hold (>= a.pairs); the kernels are instantiated for 1, 2, 4, 8 and 16 so that a
// small group does not pay the registers of a large one
template <bool kHalfGate, int kPairs>
__global__ void __launch_bounds__(kThreads) normgate_forward_kernel(const Args a) {
    // items a warp takes per step (more than one was measured slower for 64-channel groups: 0.45 against 0.54 of the
    // HBM peak; the code keeps the general form)
    constexpr int kB = 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long items = static_cast<long long>(a.rows) * a.n_groups;
    const float inv = 1.f / static_cast<float>(a.G);
    for (long long first = (static_cast<long long>(blockIdx.x) * kWarps + warp) * kB; first < items;
         first += static_cast<long long>(gridDim.x) * kWarps * kB) {
        float2 v[kB][kPairs];
        size_t base[kB];
        int c0[kB];
        float mu[kB], rs[kB];
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            const long long item = first + j < items ? first + j : items - 1;      // a repeated last item is harmless
            const long long row = item / a.n_groups;
            c0[j] = static_cast<int>(item - row * a.n_groups) * a.G + 2 * lane;
            base[j] = static_cast<size_t>(row) * a.C + c0[j];
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < kPairs; ++i) {
                v[j][i] = make_float2(0.f, 0.f);
                if (i < a.pairs) {
                    v[j][i] = *reinterpret_cast<const float2*>(a.x + base[j] + 64 * i);
                    s += v[j][i].x + v[j][i].y;
                }
            }
            mu[j] = s;
        }
#pragma unroll
        for (int j = 0; j < kB; ++j) mu[j] = warp_sum(mu[j]) * inv;
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            float q = 0.f;
#pragma unroll
            for (int i = 0; i < kPairs; ++i)
                if (i < a.pairs) {
                    const float dx = v[j][i].x - mu[j], dy = v[j][i].y - mu[j];
                    q += dx * dx + dy * dy;
                }
            rs[j] = q;
        }
#pragma unroll
        for (int j = 0; j < kB; ++j) rs[j] = rsqrtf(warp_sum(rs[j]) * inv + a.eps);
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            if (first + j >= items) break;
            if (lane == 0) {
                a.mean[first + j] = mu[j];
                a.rstd[first + j] = rs[j];
            }
#pragma unroll
            for (int i = 0; i < kPairs; ++i)
                if (i < a.pairs) {
                    const int c = c0[j] + 64 * i;
                    const float2 ga = *reinterpret_cast<const float2*>(a.gamma + c), be = *reinterpret_cast<const float2*>(a.beta + c);
                    const float2 raw = load_gate<kHalfGate>(a.gate, base[j] + 64 * i);
                    float2 o;
                    o.x = ((v[j][i].x - mu[j]) * rs[j] * ga.x + be.x) * gate_value(raw.x, a.act);
                    o.y = ((v[j][i].y - mu[j]) * rs[j] * ga.y + be.y) * gate_value(raw.y, a.act);
                    *reinterpret_cast<float2*>(a.out + base[j] + 64 * i) = o;
                }
        }
    }
}

// grid (blocks, n_groups): a warp stays with one group, so that its lanes own the same channels in every
// row it visits and can keep the parameter gradients in registers
template <bool kHalfGate, int kPairs>
__global__ void __launch_bounds__(kThreads) normgate_backward_kernel(const Args a) {
    __shared__ float red[kWarps][kPairs * 64 + 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = blockIdx.y;
    const int c0 = g * a.G + 2 * lane;
    const float inv = 1.f / static_cast<float>(a.G);
    // per lane only the two running parameter gradients live in registers across rows; gamma and beta are re-read
    // (cache hits), and the second sweep over a row reloads what the first one read instead of holding it
    float2 ag[kPairs], ab[kPairs];
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
        ag[i] = make_float2(0.f, 0.f);
        ab[i] = make_float2(0.f, 0.f);
    }
    constexpr int kB = 1;     // rows per step, as in the forward
    for (long long first = (static_cast<long long>(blockIdx.x) * kWarps + warp) * kB; first < a.rows;
         first += static_cast<long long>(gridDim.x) * kWarps * kB) {
        float mu[kB], rs[kB], s1[kB], s2[kB];
        size_t base[kB];
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            const bool live = first + j < a.rows;
            const long long row = live ? first + j : first;
            base[j] = static_cast<size_t>(row) * a.C + c0;
            mu[j] = a.mean[row * a.n_groups + g];
            rs[j] = a.rstd[row * a.n_groups + g];
            s1[j] = 0.f; s2[j] = 0.f;
            if (!live) continue;
#pragma unroll
            for (int i = 0; i < kPairs; ++i)
                if (i < a.pairs) {
                    const float2 xv = *reinterpret_cast<const float2*>(a.x + base[j] + 64 * i);
                    const float2 go = *reinterpret_cast<const float2*>(a.gout + base[j] + 64 * i);
                    const float2 raw = load_gate<kHalfGate>(a.gate, base[j] + 64 * i);
                    const float2 gt = make_float2(gate_value(raw.x, a.act), gate_value(raw.y, a.act));
                    const float2 ga = *reinterpret_cast<const float2*>(a.gamma + c0 + 64 * i), be = *reinterpret_cast<const float2*>(a.beta + c0 + 64 * i);
                    const float nx = (xv.x - mu[j]) * rs[j], ny = (xv.y - mu[j]) * rs[j];
                    store_gate<kHalfGate>(a.ggate, base[j] + 64 * i, make_float2(go.x * (nx * ga.x + be.x) * gate_slope(raw.x, a.act),
                                                                                  go.y * (ny * ga.y + be.y) * gate_slope(raw.y, a.act)));
                    const float gzx = go.x * gt.x, gzy = go.y * gt.y;
                    ag[i].x += gzx * nx; ag[i].y += gzy * ny;
                    ab[i].x += gzx; ab[i].y += gzy;
                    const float gnx = gzx * ga.x, gny = gzy * ga.y;
                    s1[j] += gnx + gny;
                    s2[j] += gnx * nx + gny * ny;
                }
        }
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            s1[j] = warp_sum(s1[j]) * inv;
            s2[j] = warp_sum(s2[j]) * inv;
        }
#pragma unroll
        for (int j = 0; j < kB; ++j) {
            if (first + j >= a.rows) break;
#pragma unroll
            for (int i = 0; i < kPairs; ++i)
                if (i < a.pairs) {
                    const float2 xv = *reinterpret_cast<const float2*>(a.x + base[j] + 64 * i);
                    const float2 go = *reinterpret_cast<const float2*>(a.gout + base[j] + 64 * i);
                    const float2 raw = load_gate<kHalfGate>(a.gate, base[j] + 64 * i);
                    const float2 gt = make_float2(gate_value(raw.x, a.act), gate_value(raw.y, a.act));
                    const float2 ga = *reinterpret_cast<const float2*>(a.gamma + c0 + 64 * i);
                    const float nx = (xv.x - mu[j]) * rs[j], ny = (xv.y - mu[j]) * rs[j];
                    float2 o;
                    o.x = rs[j] * (go.x * gt.x * ga.x - s1[j] - nx * s2[j]);
                    o.y = rs[j] * (go.y * gt.y * ga.y - s1[j] - ny * s2[j]);
                    *reinterpret_cast<float2*>(a.gx + base[j] + 64 * i) = o;
                }
        }
    }
    // the CTA's sums of the two parameter gradients, warps added in index order
    for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int i = 0; i < kPairs; ++i)
            if (i < a.pairs) *reinterpret_cast<float2*>(&red[warp][64 * i + 2 * lane]) = which ? ab[i] : ag[i];
        __syncthreads();
        for (int c = threadIdx.x; c < a.G; c += kThreads) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) t += red[w][c];
            a.partial[(static_cast<size_t>(blockIdx.x) * 2 + which) * a.C + g * a.G + c] = t;
        }
        __syncthreads();
    }
}

// out[which][c] = sum over the CTAs of partial[cta][which][c], in index order
__global__ void __launch_bounds__(256) normgate_reduce_kernel(const float* __restrict__ partial, int blocks, int C, float* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int which = blockIdx.y;
    if (c >= C) return;
    float t = 0.f;
    for (int b = 0; b < blocks; ++b) t += partial[(static_cast<size_t>(b) * 2 + which) * C + c];
    out[static_cast<size_t>(which) * C + c] = t;
}

static int check(int rows, int C, int group) {
    if (rows <= 0 || C <= 0 || group <= 0) return VRWKV_ERR_SHAPE;
    if (group % 64 != 0 || group > kMaxGroup || C % group != 0) return VRWKV_ERR_UNSUPPORTED;
    return VRWKV_OK;
}
static int sm_count() {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}
static int backward_blocks(int rows) {
    const int sms = sm_count();
    const long long want = (static_cast<long long>(rows) + kWarps - 1) / kWarps;
    return static_cast<int>(want < 4LL * sms ? (want < 1 ? 1 : want) : 4LL * sms);
}

}  // namespace normgate

static inline bool ng_misaligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

extern "C" int vrwkv_normgate_forward_f32(int rows, int C, int group, float eps, const float* x, const void* gate,
                                          int gate_is_bf16, int gate_act, const float* gamma, const float* beta, float* out,
                                          float* mean, float* rstd, void* stream) {
    using namespace normgate;
    if (int st = check(rows, C, group)) return st;
    if (!x || !gate || !gamma || !beta || !out || !mean || !rstd) return VRWKV_ERR_NULL;
    if (gate_act < 0 || gate_act > 2) return VRWKV_ERR_SHAPE;
    if (ng_misaligned(x, 8) || ng_misaligned(gate, gate_is_bf16 ? 4 : 8) || ng_misaligned(gamma, 8) || ng_misaligned(beta, 8) ||
        ng_misaligned(out, 8) || ng_misaligned(mean, 4) || ng_misaligned(rstd, 4))
        return VRWKV_ERR_ALIGNMENT;
    Args a{};
    a.rows = rows; a.C = C; a.G = group; a.n_groups = C / group; a.pairs = group / 64; a.eps = eps; a.act = gate_act;
    a.x = x; a.gate = gate; a.gamma = gamma; a.beta = beta; a.out = out; a.mean = mean; a.rstd = rstd;
    const long long items = static_cast<long long>(rows) * a.n_groups;
    const long long want = (items + kWarps - 1) / kWarps;
    const long long cap = 8LL * sm_count();                    // grid-stride loop: a few CTAs per SM, not one per eight items
    const unsigned grid = static_cast<unsigned>(want < cap ? want : cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define NG_FWD(P)                                                                     \
    do {                                                                              \
        if (gate_is_bf16) normgate_forward_kernel<true, P><<<grid, kThreads, 0, s>>>(a);  \
        else normgate_forward_kernel<false, P><<<grid, kThreads, 0, s>>>(a);              \
    } while (0)
    if (a.pairs <= 1) NG_FWD(1);
    else if (a.pairs <= 2) NG_FWD(2);
    else if (a.pairs <= 4) NG_FWD(4);
    else if (a.pairs <= 8) NG_FWD(8);
    else NG_FWD(16);
#undef NG_FWD
    return record_launches(1);
}

extern "C" size_t vrwkv_normgate_backward_workspace_bytes(int rows, int C, int group) {
    if (normgate::check(rows, C, group) != VRWKV_OK) return 0;
    return static_cast<size_t>(normgate::backward_blocks(rows)) * 2 * C * sizeof(float) + 256;
}

extern "C" int vrwkv_normgate_backward_f32(int rows, int C, int group, const float* gout, const float* x, const void* gate,
                                           int gate_is_bf16, int gate_act, const float* gamma, const float* beta, const float* mean,
                                           const float* rstd, float* gx, void* ggate, float* ggamma_gbeta, void* workspace,
                                           size_t workspace_bytes, void* stream) {
    using namespace normgate;
    if (int st = check(rows, C, group)) return st;
    if (!gout || !x || !gate || !gamma || !beta || !mean || !rstd || !gx || !ggate || !ggamma_gbeta || !workspace) return VRWKV_ERR_NULL;
    if (ng_misaligned(gout, 8) || ng_misaligned(x, 8) || ng_misaligned(gate, gate_is_bf16 ? 4 : 8) || ng_misaligned(gamma, 8) ||
        ng_misaligned(beta, 8) || ng_misaligned(gx, 8) || ng_misaligned(ggate, gate_is_bf16 ? 4 : 8) || ng_misaligned(workspace, 256))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_normgate_backward_workspace_bytes(rows, C, group)) return VRWKV_ERR_WORKSPACE;
    if (gate_act < 0 || gate_act > 2) return VRWKV_ERR_SHAPE;
    Args a{};
    a.rows = rows; a.C = C; a.G = group; a.n_groups = C / group; a.pairs = group / 64; a.act = gate_act;
    a.x = x; a.gate = gate; a.gamma = gamma; a.beta = beta; a.mean = const_cast<float*>(mean); a.rstd = const_cast<float*>(rstd);
    a.gout = gout; a.gx = gx; a.ggate = ggate; a.partial = static_cast<float*>(workspace);
    const int blocks = backward_blocks(rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(blocks, a.n_groups);
#define NG_BWD(P)                                                                      \
    do {                                                                               \
        if (gate_is_bf16) normgate_backward_kernel<true, P><<<grid, kThreads, 0, s>>>(a);  \
        else normgate_backward_kernel<false, P><<<grid, kThreads, 0, s>>>(a);              \
    } while (0)
    if (a.pairs <= 1) NG_BWD(1);
    else if (a.pairs <= 2) NG_BWD(2);
    else if (a.pairs <= 4) NG_BWD(4);
    else if (a.pairs <= 8) NG_BWD(8);
    else NG_BWD(16);
#undef NG_BWD
    normgate_reduce_kernel<<<dim3((C + 255) / 256, 2), 256, 0, s>>>(a.partial, blocks, C, ggamma_gbeta);
    return record_launches(2);
}
