// Per-head token shift fused with the data-dependent interpolations of the VRWKV6 spatial mix,
// forward and backward.
//
// The block first forms xx = q_shift_multihead(x) - x, then xxx = x + xx * maa_x for the low-rank
// branch, and from that branch's five per-token offsets m_j the five inputs of its projections,
// x + xx * (maa_j + m_j)  (classification/mmcls_custom/models/backbones/vrwkv6.py:75-100,
// 180-193).  With tensor ops that is the shift (a transpose, five strided copies, a transpose
// back), a subtraction and three elementwise passes per output.  Here one pass reads x once (the
// shifted read is a second, cache-resident read of a neighbouring token row) and the n offsets and
// writes the n outputs:  out_j = x + (shift(x) - x) * (maa_j[c] + m_j[b,t,c]),  m_j optional, so
// the same kernel serves xxx (n = 1, no offset) and the five projections' inputs (n = 5).  The
// backward reads the n output gradients (twice: at the token and at the token that reads it
// through the shift), x and the offsets, and writes gx, the n offset gradients and the per-channel
// gradients of maa_j, reduced in a fixed order.  Pure bandwidth work.  The offsets may be float32
// or bfloat16 (they come out of a half-precision matrix product); everything else is float32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "vrwkv_b200.h"
#include "vrwkv_internal.h"

namespace ddlerp {

constexpr int kMaxOut = 5;
constexpr int kThreads = 128;
constexpr int kTokensPerBlock = 32;
constexpr int kVec = 4;

struct Args {
    int B, H, W, C;
    int head_dim;   // the four shifted groups are the quarters of every head
    int shift;
    int n_out;
    const float* x;
    const float* maa[kMaxOut];   // (C,)
    const void* m[kMaxOut];      // (B, T, C) or null
    float* out[kMaxOut];
    const float* gout[kMaxOut];
    float* gx;
    void* gm[kMaxOut];           // null where m is null
    float* partial;              // [row blocks][n_out][C]
};

// token whose value channel c of token (h, w) takes through the shift (-1: zero), and the token that takes
// the value of (h, w) (-1: none); group = quarter of the head: left, right, upper, lower neighbour
__device__ __forceinline__ int source_token(const Args& a, int h, int w, int c) {
    const int g = (c % a.head_dim) / (a.head_dim / 4);
    int hs = h, ws = w;
    if (g == 0) ws = w - a.shift;
    else if (g == 1) ws = w + a.shift;
    else if (g == 2) hs = h - a.shift;
    else hs = h + a.shift;
    if (hs < 0 || hs >= a.H || ws < 0 || ws >= a.W) return -1;
    return hs * a.W + ws;
}
__device__ __forceinline__ int reader_token(const Args& a, int h, int w, int c) {
    const int g = (c % a.head_dim) / (a.head_dim / 4);
    int hd = h, wd = w;
    if (g == 0) wd = w + a.shift;
    else if (g == 1) wd = w - a.shift;
    else if (g == 2) hd = h + a.shift;
    else hd = h - a.shift;
    if (hd < 0 || hd >= a.H || wd < 0 || wd >= a.W) return -1;
    return hd * a.W + wd;
}

template <bool kHalfM>
__device__ __forceinline__ float4 load_m(const void* m, size_t at) {
    if (m == nullptr) return make_float4(0.f, 0.f, 0.f, 0.f);
    if (kHalfM) {
        const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(m) + at);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    }
    return *reinterpret_cast<const float4*>(static_cast<const float*>(m) + at);
}
template <bool kHalfM>
__device__ __forceinline__ void store_m(void* m, size_t at, float4 v) {
    if (kHalfM) {
        uint2 raw;
        *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(m) + at) = raw;
    } else {
        *reinterpret_cast<float4*>(static_cast<float*>(m) + at) = v;
    }
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// thread = 4 consecutive channels (one quarter of a head never splits them: head_dim % 16 == 0); a block walks
// kTokensPerBlock tokens
template <bool kHalfM>
__global__ void __launch_bounds__(kThreads) ddlerp_forward(const Args a) {
    const int cv = (blockIdx.x * kThreads + threadIdx.x) * kVec;
    if (cv >= a.C) return;
    const int T = a.H * a.W;
    float4 maa[kMaxOut];
#pragma unroll
    for (int j = 0; j < kMaxOut; ++j)
        maa[j] = j < a.n_out ? *reinterpret_cast<const float4*>(a.maa[j] + cv) : make_float4(0.f, 0.f, 0.f, 0.f);
    const long long tok0 = static_cast<long long>(blockIdx.y) * kTokensPerBlock;
    const long long ntok = static_cast<long long>(a.B) * T;
    for (int i = 0; i < kTokensPerBlock; ++i) {
        const long long tok = tok0 + i;
        if (tok >= ntok) break;
        const int b = static_cast<int>(tok / T), t = static_cast<int>(tok % T);
        const int h = t / a.W, w = t % a.W;
        const size_t base = static_cast<size_t>(tok) * a.C + cv;
        const int src = source_token(a, h, w, cv);
        const float4 x4 = *reinterpret_cast<const float4*>(a.x + base);
        float4 d4 = make_float4(-x4.x, -x4.y, -x4.z, -x4.w);      // shift(x) - x
        if (src >= 0) {
            const float4 s4 = *reinterpret_cast<const float4*>(a.x + (static_cast<size_t>(b) * T + src) * a.C + cv);
            d4 = make_float4(s4.x - x4.x, s4.y - x4.y, s4.z - x4.z, s4.w - x4.w);
        }
#pragma unroll
        for (int j = 0; j < kMaxOut; ++j)
            if (j < a.n_out) {
                const float4 mu = add4(maa[j], load_m<kHalfM>(a.m[j], base));
                *reinterpret_cast<float4*>(a.out[j] + base) =
                    make_float4(fmaf(d4.x, mu.x, x4.x), fmaf(d4.y, mu.y, x4.y), fmaf(d4.z, mu.z, x4.z), fmaf(d4.w, mu.w, x4.w));
            }
    }
}

template <bool kHalfM>
__global__ void __launch_bounds__(kThreads) ddlerp_backward(const Args a) {
    const int cv = (blockIdx.x * kThreads + threadIdx.x) * kVec;
    if (cv >= a.C) return;
    const int T = a.H * a.W;
    float4 maa[kMaxOut], gmaa[kMaxOut];
#pragma unroll
    for (int j = 0; j < kMaxOut; ++j) {
        maa[j] = j < a.n_out ? *reinterpret_cast<const float4*>(a.maa[j] + cv) : make_float4(0.f, 0.f, 0.f, 0.f);
        gmaa[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const long long tok0 = static_cast<long long>(blockIdx.y) * kTokensPerBlock;
    const long long ntok = static_cast<long long>(a.B) * T;
    for (int i = 0; i < kTokensPerBlock; ++i) {
        const long long tok = tok0 + i;
        if (tok >= ntok) break;
        const int b = static_cast<int>(tok / T), t = static_cast<int>(tok % T);
        const int h = t / a.W, w = t % a.W;
        const size_t base = static_cast<size_t>(tok) * a.C + cv;
        const int src = source_token(a, h, w, cv), rdr = reader_token(a, h, w, cv);
        const size_t rbase = (static_cast<size_t>(b) * T + (rdr >= 0 ? rdr : 0)) * a.C + cv;
        const float4 x4 = *reinterpret_cast<const float4*>(a.x + base);
        float4 d4 = make_float4(-x4.x, -x4.y, -x4.z, -x4.w);
        if (src >= 0) {
            const float4 s4 = *reinterpret_cast<const float4*>(a.x + (static_cast<size_t>(b) * T + src) * a.C + cv);
            d4 = make_float4(s4.x - x4.x, s4.y - x4.y, s4.z - x4.z, s4.w - x4.w);
        }
        float4 gx = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kMaxOut; ++j)
            if (j < a.n_out) {
                const float4 g = *reinterpret_cast<const float4*>(a.gout[j] + base);
                const float4 mu = add4(maa[j], load_m<kHalfM>(a.m[j], base));
                // out = x (1 - mu) + shift(x) mu: the token's own share, and its offset gradient
                gx.x = fmaf(g.x, 1.f - mu.x, gx.x); gx.y = fmaf(g.y, 1.f - mu.y, gx.y);
                gx.z = fmaf(g.z, 1.f - mu.z, gx.z); gx.w = fmaf(g.w, 1.f - mu.w, gx.w);
                const float4 gm = make_float4(g.x * d4.x, g.y * d4.y, g.z * d4.z, g.w * d4.w);
                gmaa[j] = add4(gmaa[j], gm);
                if (a.gm[j] != nullptr) store_m<kHalfM>(a.gm[j], base, gm);
                if (rdr >= 0) {
                    // the token that reads this one through the shift hands back its gradient times its own weight
                    const float4 gr = *reinterpret_cast<const float4*>(a.gout[j] + rbase);
                    const float4 mr = add4(maa[j], load_m<kHalfM>(a.m[j], rbase));
                    gx.x = fmaf(gr.x, mr.x, gx.x); gx.y = fmaf(gr.y, mr.y, gx.y);
                    gx.z = fmaf(gr.z, mr.z, gx.z); gx.w = fmaf(gr.w, mr.w, gx.w);
                }
            }
        *reinterpret_cast<float4*>(a.gx + base) = gx;
    }
#pragma unroll
    for (int j = 0; j < kMaxOut; ++j)
        if (j < a.n_out)
            *reinterpret_cast<float4*>(a.partial + (static_cast<size_t>(blockIdx.y) * a.n_out + j) * a.C + cv) = gmaa[j];
}

// gmaa[j][c] = sum over row blocks of partial[block][j][c], fixed order
struct ReduceArgs {
    const float* partial;
    int blocks, n_out, C;
    float* gmaa[kMaxOut];
};
__global__ void __launch_bounds__(1024) ddlerp_reduce(const ReduceArgs r) {
    __shared__ float red[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x, j = blockIdx.y;
    float acc = 0.f;
    if (c < r.C)
        for (int q = threadIdx.y; q < r.blocks; q += 32) acc += r.partial[(static_cast<size_t>(q) * r.n_out + j) * r.C + c];
    red[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < r.C) {
        float total = 0.f;
#pragma unroll
        for (int q = 0; q < 32; ++q) total += red[q][threadIdx.x];
        r.gmaa[j][c] = total;
    }
}

static int row_blocks(int B, int H, int W) {
    const long long ntok = static_cast<long long>(B) * H * W;
    return static_cast<int>((ntok + kTokensPerBlock - 1) / kTokensPerBlock);
}
static int check(int B, int H, int W, int C, int head_dim, int shift, int n_out) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || head_dim <= 0 || shift < 0 || n_out < 1 || n_out > kMaxOut) return VRWKV_ERR_SHAPE;
    if (static_cast<long long>(B) * H * W > 2000000000LL) return VRWKV_ERR_SHAPE;
    if (head_dim % 16 != 0 || C % head_dim != 0) return VRWKV_ERR_UNSUPPORTED;      // a quarter of a head holds whole 4-channel vectors
    return VRWKV_OK;
}
static bool misaligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

}  // namespace ddlerp

extern "C" int vrwkv_qshift_ddlerp_forward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out, const float* x,
                                               const float* const* maa, const void* const* m, int m_is_bf16, float* const* out,
                                               void* stream) {
    using namespace ddlerp;
    if (int st = check(B, H, W, C, head_dim, shift, n_out)) return st;
    if (!x || !maa || !m || !out) return VRWKV_ERR_NULL;
    Args a{};
    a.B = B; a.H = H; a.W = W; a.C = C; a.head_dim = head_dim; a.shift = shift; a.n_out = n_out; a.x = x;
    if (misaligned(x, 16)) return VRWKV_ERR_ALIGNMENT;
    for (int j = 0; j < n_out; ++j) {
        if (!maa[j] || !out[j]) return VRWKV_ERR_NULL;
        if (misaligned(maa[j], 16) || misaligned(out[j], 16) || (m[j] && misaligned(m[j], m_is_bf16 ? 8 : 16))) return VRWKV_ERR_ALIGNMENT;
        a.maa[j] = maa[j]; a.m[j] = m[j]; a.out[j] = out[j];
    }
    const dim3 grid((C / kVec + kThreads - 1) / kThreads, row_blocks(B, H, W));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m_is_bf16) ddlerp_forward<true><<<grid, kThreads, 0, s>>>(a);
    else ddlerp_forward<false><<<grid, kThreads, 0, s>>>(a);
    return record_launches(1);
}

extern "C" size_t vrwkv_qshift_ddlerp_backward_workspace_bytes(int B, int H, int W, int C, int n_out) {
    if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || n_out < 1 || n_out > ddlerp::kMaxOut) return 0;
    return static_cast<size_t>(ddlerp::row_blocks(B, H, W)) * n_out * C * sizeof(float) + 256;
}

extern "C" int vrwkv_qshift_ddlerp_backward_f32(int B, int H, int W, int C, int head_dim, int shift, int n_out, const float* x,
                                                const float* const* maa, const void* const* m, int m_is_bf16,
                                                const float* const* gout, float* gx, void* const* gm, float* const* gmaa,
                                                void* workspace, size_t workspace_bytes, void* stream) {
    using namespace ddlerp;
    if (int st = check(B, H, W, C, head_dim, shift, n_out)) return st;
    if (!x || !maa || !m || !gout || !gx || !gm || !gmaa || !workspace) return VRWKV_ERR_NULL;
    if (workspace_bytes < vrwkv_qshift_ddlerp_backward_workspace_bytes(B, H, W, C, n_out)) return VRWKV_ERR_WORKSPACE;
    if (misaligned(x, 16) || misaligned(gx, 16) || misaligned(workspace, 256)) return VRWKV_ERR_ALIGNMENT;
    Args a{};
    a.B = B; a.H = H; a.W = W; a.C = C; a.head_dim = head_dim; a.shift = shift; a.n_out = n_out; a.x = x; a.gx = gx;
    a.partial = static_cast<float*>(workspace);
    ReduceArgs r{};
    r.partial = a.partial; r.blocks = row_blocks(B, H, W); r.n_out = n_out; r.C = C;
    for (int j = 0; j < n_out; ++j) {
        if (!maa[j] || !gout[j] || !gmaa[j] || (m[j] != nullptr) != (gm[j] != nullptr)) return VRWKV_ERR_NULL;
        if (misaligned(maa[j], 16) || misaligned(gout[j], 16) || misaligned(gmaa[j], 4) ||
            (m[j] && (misaligned(m[j], m_is_bf16 ? 8 : 16) || misaligned(gm[j], m_is_bf16 ? 8 : 16))))
            return VRWKV_ERR_ALIGNMENT;
        a.maa[j] = maa[j]; a.m[j] = m[j]; a.gout[j] = gout[j]; a.gm[j] = gm[j];
        r.gmaa[j] = gmaa[j];
    }
    const dim3 grid((C / kVec + kThreads - 1) / kThreads, r.blocks);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (m_is_bf16) ddlerp_backward<true><<<grid, kThreads, 0, s>>>(a);
    else ddlerp_backward<false><<<grid, kThreads, 0, s>>>(a);
    ddlerp_reduce<<<dim3((C + 31) / 32, n_out), dim3(32, 32), 0, s>>>(r);
    return record_launches(2);
}
