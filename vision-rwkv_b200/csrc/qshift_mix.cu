// Fused Q-Shift + token-mix interpolation, forward and backward.
//
// In the backbones every mixing block first builds a shifted copy xx of its input x
// (tokens laid out as an H x W grid, channel quarters moved by `s` pixels right / left /
// down / up with zero fill at the border, the remaining channels copied) and then forms
// n interpolations  out_m = x * mix_m + xx * (1 - mix_m)  (n = 3 in the spatial mix: k, v, r;
// n = 2 in the channel mix: k, r) that feed the linear layers
// (classification/mmcls_custom/models/backbones/vrwkv.py:68-79, 156-164, 247-250).  Done
// with tensor ops that is a transpose, a zero fill, five strided copies, a transpose back and
// 3 n elementwise passes.  Here: one pass that reads x once (the shifted read is a second,
// cache-resident read of a neighbouring token row) and writes the n outputs; the backward
// reads the n output gradients and x once, writes gx, and reduces the n mix gradients in a
// fixed order.  Pure bandwidth work: 4 (1 + n) bytes per element forward, 4 (n + 2) backward.
#include <cuda_runtime.h>
#include <cstdint>
#include "vrwkv_internal.h"

namespace qshift {

constexpr int kMaxOut = 3;
constexpr int kThreads = 128;
constexpr int kTokensPerBlock = 32;

struct Args {
    int B, H, W, C;
    int group;     // channels per shifted group = int(C * gamma), or head_dim / 4 for the per-head variant
    int period;    // 0: the four groups are channels [0, 4 * group); n: they repeat every n channels (n = head_dim)
    int shift;     // pixels
    int n_out;
    const float* x;
    const float* mix[kMaxOut];     // (C,)
    float* out[kMaxOut];           // forward outputs (B, T, C)
    const float* gout[kMaxOut];    // backward: output gradients
    float* gx;
    float* partial;                // backward: [blocks_y][n_out][C]
};

// Token that channel c of token (h, w) reads its shifted value from; -1 = zero fill.
__device__ __forceinline__ int source_token(const Args& a, int h, int w, int c) {
    const int g = (a.period ? c % a.period : c) / a.group;
    int hs = h, ws = w;
    if (g == 0) ws = w - a.shift;
    else if (g == 1) ws = w + a.shift;
    else if (g == 2) hs = h - a.shift;
    else if (g == 3) hs = h + a.shift;
    if (hs < 0 || hs >= a.H || ws < 0 || ws >= a.W) return -1;
    return hs * a.W + ws;
}
// Token whose shifted value is read *from* (h, w) for channel c (the transpose); -1 = none.
__device__ __forceinline__ int reader_token(const Args& a, int h, int w, int c) {
    const int g = (a.period ? c % a.period : c) / a.group;
    int hd = h, wd = w;
    if (g == 0) wd = w + a.shift;
    else if (g == 1) wd = w - a.shift;
    else if (g == 2) hd = h + a.shift;
    else if (g == 3) hd = h - a.shift;
    if (hd < 0 || hd >= a.H || wd < 0 || wd >= a.W) return -1;
    return hd * a.W + wd;
}

// kVec: 4 channels per thread (needs C % 4 == 0, group % 4 == 0 and 16-byte aligned tensors)
template <int kVec>
__global__ void __launch_bounds__(kThreads) qshift_mix_forward(const Args a) {
    const int cv = (blockIdx.x * kThreads + threadIdx.x) * kVec;
    if (cv >= a.C) return;
    const int T = a.H * a.W;
    float mixv[kMaxOut][kVec];
#pragma unroll
    for (int m = 0; m < kMaxOut; ++m)
        if (m < a.n_out)
#pragma unroll
            for (int j = 0; j < kVec; ++j) mixv[m][j] = a.mix[m][cv + j];
    const long long tok0 = static_cast<long long>(blockIdx.y) * kTokensPerBlock;
    const long long ntok = static_cast<long long>(a.B) * T;
    for (int i = 0; i < kTokensPerBlock; ++i) {
        const long long tok = tok0 + i;
        if (tok >= ntok) break;
        const int b = static_cast<int>(tok / T), t = static_cast<int>(tok % T);
        const int h = t / a.W, w = t % a.W;
        const size_t base = static_cast<size_t>(tok) * a.C + cv;
        float xv[kVec], sv[kVec];
        const int src = source_token(a, h, w, cv);          // one group per vector (group % kVec == 0)
        if (kVec == 4) {
            const float4 x4 = *reinterpret_cast<const float4*>(a.x + base);
            xv[0] = x4.x; xv[1] = x4.y; xv[2] = x4.z; xv[3] = x4.w;
            float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (src >= 0) s4 = *reinterpret_cast<const float4*>(a.x + (static_cast<size_t>(b) * T + src) * a.C + cv);
            sv[0] = s4.x; sv[1] = s4.y; sv[2] = s4.z; sv[3] = s4.w;
        } else {
            xv[0] = a.x[base];
            sv[0] = src >= 0 ? a.x[(static_cast<size_t>(b) * T + src) * a.C + cv] : 0.f;
        }
#pragma unroll
        for (int m = 0; m < kMaxOut; ++m) {
            if (m < a.n_out) {
                float o[kVec];
#pragma unroll
                for (int j = 0; j < kVec; ++j) o[j] = fmaf(mixv[m][j], xv[j] - sv[j], sv[j]);
                if (kVec == 4) *reinterpret_cast<float4*>(a.out[m] + base) = make_float4(o[0], o[1], o[2], o[3]);
                else a.out[m][base] = o[0];
            }
        }
    }
}

template <int kVec>
__global__ void __launch_bounds__(kThreads) qshift_mix_backward(const Args a) {
    const int cv = (blockIdx.x * kThreads + threadIdx.x) * kVec;
    if (cv >= a.C) return;
    const int T = a.H * a.W;
    float mixv[kMaxOut][kVec], gmix[kMaxOut][kVec];
#pragma unroll
    for (int m = 0; m < kMaxOut; ++m)
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            mixv[m][j] = m < a.n_out ? a.mix[m][cv + j] : 0.f;
            gmix[m][j] = 0.f;
        }
    const long long tok0 = static_cast<long long>(blockIdx.y) * kTokensPerBlock;
    const long long ntok = static_cast<long long>(a.B) * T;
    for (int i = 0; i < kTokensPerBlock; ++i) {
        const long long tok = tok0 + i;
        if (tok >= ntok) break;
        const int b = static_cast<int>(tok / T), t = static_cast<int>(tok % T);
        const int h = t / a.W, w = t % a.W;
        const size_t base = static_cast<size_t>(tok) * a.C + cv;
        const int src = source_token(a, h, w, cv);
        const int rdr = reader_token(a, h, w, cv);
        const size_t sbase = (static_cast<size_t>(b) * T + (src >= 0 ? src : 0)) * a.C + cv;
        const size_t rbase = (static_cast<size_t>(b) * T + (rdr >= 0 ? rdr : 0)) * a.C + cv;
        float xv[kVec], sv[kVec], gxv[kVec];
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            xv[j] = a.x[base + j];
            sv[j] = src >= 0 ? a.x[sbase + j] : 0.f;
            gxv[j] = 0.f;
        }
#pragma unroll
        for (int m = 0; m < kMaxOut; ++m) {
            if (m < a.n_out) {
#pragma unroll
                for (int j = 0; j < kVec; ++j) {
                    const float g = a.gout[m][base + j];
                    gxv[j] = fmaf(g, mixv[m][j], gxv[j]);
                    gmix[m][j] = fmaf(g, xv[j] - sv[j], gmix[m][j]);
                    if (rdr >= 0) gxv[j] = fmaf(a.gout[m][rbase + j], 1.f - mixv[m][j], gxv[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < kVec; ++j) a.gx[base + j] = gxv[j];
    }
#pragma unroll
    for (int m = 0; m < kMaxOut; ++m)
        if (m < a.n_out)
#pragma unroll
            for (int j = 0; j < kVec; ++j)
                a.partial[(static_cast<size_t>(blockIdx.y) * a.n_out + m) * a.C + cv + j] = gmix[m][j];
}

// gmix[m][c] = sum over row blocks of partial[block][m][c], fixed order
__global__ void __launch_bounds__(1024) qshift_reduce(const float* __restrict__ partial, int blocks, int n_out, int C,
                                                      float* __restrict__ gmix0, float* __restrict__ gmix1,
                                                      float* __restrict__ gmix2) {
    __shared__ float red[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x, m = blockIdx.y;
    float acc = 0.f;
    if (c < C)
        for (int r = threadIdx.y; r < blocks; r += 32) acc += partial[(static_cast<size_t>(r) * n_out + m) * C + c];
    red[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) total += red[r][threadIdx.x];
        (m == 0 ? gmix0 : m == 1 ? gmix1 : gmix2)[c] = total;
    }
}

static bool vector_ok(const Args& a, bool bwd) {
    if (a.C % 4 || a.group % 4) return false;
    uintptr_t bits = reinterpret_cast<uintptr_t>(a.x);
    for (int m = 0; m < a.n_out; ++m) {
        bits |= reinterpret_cast<uintptr_t>(a.mix[m]);
        bits |= reinterpret_cast<uintptr_t>(bwd ? static_cast<const void*>(a.gout[m]) : static_cast<const void*>(a.out[m]));
    }
    if (bwd) bits |= reinterpret_cast<uintptr_t>(a.gx);
    return (bits & 15u) == 0;
}

static int row_blocks(const Args& a) {
    const long long ntok = static_cast<long long>(a.B) * a.H * a.W;
    return static_cast<int>((ntok + kTokensPerBlock - 1) / kTokensPerBlock);
}

size_t backward_workspace(int B, int H, int W, int C, int n_out) {
    Args a{};
    a.B = B; a.H = H; a.W = W;
    return static_cast<size_t>(row_blocks(a)) * n_out * C * sizeof(float);
}

int forward(const Args& a, cudaStream_t stream) {
    const int by = row_blocks(a);
    if (vector_ok(a, false)) {
        qshift_mix_forward<4><<<dim3((a.C / 4 + kThreads - 1) / kThreads, by), kThreads, 0, stream>>>(a);
    } else {
        qshift_mix_forward<1><<<dim3((a.C + kThreads - 1) / kThreads, by), kThreads, 0, stream>>>(a);
    }
    return 1;
}

int backward(const Args& a, float* const gmix[kMaxOut], cudaStream_t stream) {
    const int by = row_blocks(a);
    // the vector path of the backward only needs the group boundary rule (scalar loads inside)
    if (a.C % 4 == 0 && a.group % 4 == 0) {
        qshift_mix_backward<4><<<dim3((a.C / 4 + kThreads - 1) / kThreads, by), kThreads, 0, stream>>>(a);
    } else {
        qshift_mix_backward<1><<<dim3((a.C + kThreads - 1) / kThreads, by), kThreads, 0, stream>>>(a);
    }
    qshift_reduce<<<dim3((a.C + 31) / 32, a.n_out), dim3(32, 32), 0, stream>>>(a.partial, by, a.n_out, a.C, gmix[0],
                                                                              gmix[1], gmix[2]);
    return 2;
}

}  // namespace qshift

// ---- C ABI --------------------------------------------------------------------------------------
#include "vrwkv_b200.h"

static int qshift_check(int B, int H, int W, int C, int group, int shift, int n_out) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || group <= 0 || shift < 0 || n_out < 1 || n_out > 3) return VRWKV_ERR_SHAPE;
    if (4LL * group > C + 0LL && group * 4 > C) return VRWKV_ERR_SHAPE;      // at most four shifted groups fit
    if ((static_cast<long long>(B) * H * W + 31) / 32 > 65535LL * 32768) return VRWKV_ERR_SHAPE;
    return VRWKV_OK;
}

static int qshift_forward_any(int B, int H, int W, int C, int group, int period, int shift, int n_out, const float* x,
                              const float* const* mix, float* const* out, void* stream) {
    if (int st = qshift_check(B, H, W, C, group, shift, n_out)) return st;
    if (!x || !mix || !out) return VRWKV_ERR_NULL;
    qshift::Args a{};
    a.B = B; a.H = H; a.W = W; a.C = C; a.group = group; a.period = period; a.shift = shift; a.n_out = n_out; a.x = x;
    for (int m = 0; m < n_out; ++m) {
        if (!mix[m] || !out[m]) return VRWKV_ERR_NULL;
        a.mix[m] = mix[m];
        a.out[m] = out[m];
    }
    return record_launches(qshift::forward(a, static_cast<cudaStream_t>(stream)));
}

static int qshift_backward_any(int B, int H, int W, int C, int group, int period, int shift, int n_out, const float* x,
                               const float* const* mix, const float* const* gout, float* gx, float* const* gmix,
                               void* workspace, size_t workspace_bytes, void* stream) {
    if (int st = qshift_check(B, H, W, C, group, shift, n_out)) return st;
    if (!x || !mix || !gout || !gx || !gmix || !workspace) return VRWKV_ERR_NULL;
    if (workspace_bytes < qshift::backward_workspace(B, H, W, C, n_out)) return VRWKV_ERR_WORKSPACE;
    qshift::Args a{};
    a.B = B; a.H = H; a.W = W; a.C = C; a.group = group; a.period = period; a.shift = shift; a.n_out = n_out; a.x = x;
    a.gx = gx;
    a.partial = static_cast<float*>(workspace);
    float* gm[qshift::kMaxOut] = {nullptr, nullptr, nullptr};
    for (int m = 0; m < n_out; ++m) {
        if (!mix[m] || !gout[m] || !gmix[m]) return VRWKV_ERR_NULL;
        a.mix[m] = mix[m];
        a.gout[m] = gout[m];
        gm[m] = gmix[m];
    }
    return record_launches(qshift::backward(a, gm, static_cast<cudaStream_t>(stream)));
}

// head_dim channels per head, a multiple of 4 that divides C; the groups are its quarters
static int multihead_check(int C, int head_dim) {
    return (head_dim < 4 || head_dim % 4 != 0 || C % head_dim != 0) ? VRWKV_ERR_SHAPE : VRWKV_OK;
}

extern "C" int vrwkv_qshift_mix_forward_f32(int B, int H, int W, int C, int group, int shift, int n_out,
                                            const float* x, const float* const* mix, float* const* out,
                                            void* stream) {
    return qshift_forward_any(B, H, W, C, group, 0, shift, n_out, x, mix, out, stream);
}

extern "C" int vrwkv_qshift_multihead_mix_forward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out,
                                                      const float* x, const float* const* mix, float* const* out,
                                                      void* stream) {
    if (int st = multihead_check(C, head_dim)) return st;
    return qshift_forward_any(B, H, W, C, head_dim / 4, head_dim, shift, n_out, x, mix, out, stream);
}

extern "C" size_t vrwkv_qshift_mix_backward_workspace_bytes(int B, int H, int W, int C, int n_out) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || n_out < 1 || n_out > 3) return 0;
    return qshift::backward_workspace(B, H, W, C, n_out);
}

extern "C" int vrwkv_qshift_mix_backward_f32(int B, int H, int W, int C, int group, int shift, int n_out,
                                             const float* x, const float* const* mix, const float* const* gout,
                                             float* gx, float* const* gmix, void* workspace, size_t workspace_bytes,
                                             void* stream) {
    return qshift_backward_any(B, H, W, C, group, 0, shift, n_out, x, mix, gout, gx, gmix, workspace, workspace_bytes, stream);
}

extern "C" int vrwkv_qshift_multihead_mix_backward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out,
                                                       const float* x, const float* const* mix,
                                                       const float* const* gout, float* gx, float* const* gmix,
                                                       void* workspace, size_t workspace_bytes, void* stream) {
    if (int st = multihead_check(C, head_dim)) return st;
    return qshift_backward_any(B, H, W, C, head_dim / 4, head_dim, shift, n_out, x, mix, gout, gx, gmix, workspace,
                               workspace_bytes, stream);
}
