// Launchers of the generic Bi-WKV path (see biwkv_generic.cuh for the algorithm).
#include <cuda_runtime.h>
#include "biwkv_generic.cuh"
#include "vrwkv_internal.h"

namespace biwkv {

constexpr int kLanes = 32;     // channels per warp
constexpr int kRows = 8;       // sub-chunks per CTA
constexpr int kFwdL = 16;
constexpr int kBwdL = 8;

template <int L>
__global__ void __launch_bounds__(kLanes * kRows)
generic_fwd_aggregate(GenericShape s, const float* __restrict__ w, const float* __restrict__ k,
                      const float* __restrict__ v, float* __restrict__ carry) {
    const int c = blockIdx.x * kLanes + threadIdx.x;
    const int sc = blockIdx.y * kRows + threadIdx.y;
    const int b = blockIdx.z;
    if (c < s.C && sc < s.NS) fwd_aggregate_thread<L>(s, w, k, v, carry, b, sc, c);
}

__global__ void generic_fwd_carry(GenericShape s, const float* __restrict__ w,
                                  float* __restrict__ carry) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c < s.C) fwd_carry_thread(s, w, carry, b, c);
}

template <int L>
__global__ void __launch_bounds__(kLanes * kRows)
generic_fwd_emit(GenericShape s, const float* __restrict__ w, const float* __restrict__ u,
                 const float* __restrict__ k, const float* __restrict__ v,
                 const float* __restrict__ carry, float* __restrict__ y) {
    const int c = blockIdx.x * kLanes + threadIdx.x;
    const int sc = blockIdx.y * kRows + threadIdx.y;
    const int b = blockIdx.z;
    if (c < s.C && sc < s.NS) fwd_emit_thread<L>(s, w, u, k, v, carry, y, b, sc, c);
}

template <int L>
__global__ void __launch_bounds__(kLanes * kRows)
generic_bwd_aggregate(GenericShape s, const float* __restrict__ w, const float* __restrict__ u,
                      const float* __restrict__ k, const float* __restrict__ v,
                      const float* __restrict__ gy, const float* __restrict__ carry,
                      float* __restrict__ adj) {
    const int c = blockIdx.x * kLanes + threadIdx.x;
    const int sc = blockIdx.y * kRows + threadIdx.y;
    const int b = blockIdx.z;
    if (c < s.C && sc < s.NS) bwd_aggregate_thread<L>(s, w, u, k, v, gy, carry, adj, b, sc, c);
}

__global__ void generic_bwd_carry(GenericShape s, const float* __restrict__ w,
                                  float* __restrict__ adj) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c < s.C) bwd_carry_thread(s, w, adj, b, c);
}

// partial rows: [B * gridDim.y][2][C], one row per CTA-row of sub-chunks
template <int L>
__global__ void __launch_bounds__(kLanes * kRows)
generic_bwd_emit(GenericShape s, const float* __restrict__ w, const float* __restrict__ u,
                 const float* __restrict__ k, const float* __restrict__ v,
                 const float* __restrict__ gy, const float* __restrict__ carry,
                 const float* __restrict__ adj, float* __restrict__ gk, float* __restrict__ gv,
                 float* __restrict__ partial) {
    __shared__ float red[2][kRows][kLanes];
    const int c = blockIdx.x * kLanes + threadIdx.x;
    const int sc = blockIdx.y * kRows + threadIdx.y;
    const int b = blockIdx.z;
    float gw = 0.f, gu = 0.f;
    if (c < s.C && sc < s.NS)
        bwd_emit_thread<L>(s, w, u, k, v, gy, carry, adj, gk, gv, gw, gu, b, sc, c);
    red[0][threadIdx.y][threadIdx.x] = gw;
    red[1][threadIdx.y][threadIdx.x] = gu;
    __syncthreads();
    if (threadIdx.y < 2 && c < s.C) {
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc += red[threadIdx.y][r][threadIdx.x];
        const size_t row = static_cast<size_t>(b) * gridDim.y + blockIdx.y;
        partial[(row * 2 + threadIdx.y) * s.C + c] = acc;
    }
}

// out[j][c] = sum over rows of partial[row][j][c], fixed order
__global__ void __launch_bounds__(1024)
reduce_partials(const float* __restrict__ partial, int rows, int C, float* __restrict__ out) {
    __shared__ float red[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    const int j = blockIdx.y;
    float acc = 0.f;
    if (c < C)
        for (int r = threadIdx.y; r < rows; r += 32)
            acc += partial[(static_cast<size_t>(r) * 2 + j) * C + c];
    red[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) total += red[r][threadIdx.x];
        out[static_cast<size_t>(j) * C + c] = total;
    }
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

size_t generic_forward_workspace(int B, int T, int C) {
    const size_t NS = ceil_div(T, kFwdL);
    return static_cast<size_t>(B) * NS * kFwdRows * C * sizeof(float);
}

size_t generic_backward_workspace(int B, int T, int C) {
    const size_t NS = ceil_div(T, kBwdL);
    const size_t rows = static_cast<size_t>(B) * ceil_div(static_cast<int>(NS), kRows);
    return (static_cast<size_t>(B) * NS * (kFwdRows + kAdjRows) * C + rows * 2 * C) * sizeof(float);
}

int generic_forward(int B, int T, int C, const float* w, const float* u, const float* k,
                    const float* v, float* y, void* workspace, cudaStream_t stream) {
    GenericShape s{B, T, C, kFwdL, ceil_div(T, kFwdL)};
    float* carry = static_cast<float*>(workspace);
    const dim3 block(kLanes, kRows);
    const dim3 grid(ceil_div(C, kLanes), ceil_div(s.NS, kRows), B);
    generic_fwd_aggregate<kFwdL><<<grid, block, 0, stream>>>(s, w, k, v, carry);
    generic_fwd_carry<<<dim3(ceil_div(C, 128), B), 128, 0, stream>>>(s, w, carry);
    generic_fwd_emit<kFwdL><<<grid, block, 0, stream>>>(s, w, u, k, v, carry, y);
    return 3;
}

int generic_backward(int B, int T, int C, const float* w, const float* u, const float* k,
                     const float* v, const float* gy, float* gwgu, float* gk, float* gv,
                     void* workspace, cudaStream_t stream) {
    GenericShape s{B, T, C, kBwdL, ceil_div(T, kBwdL)};
    float* carry = static_cast<float*>(workspace);
    float* adj = carry + static_cast<size_t>(B) * s.NS * kFwdRows * C;
    float* partial = adj + static_cast<size_t>(B) * s.NS * kAdjRows * C;
    const dim3 block(kLanes, kRows);
    const dim3 grid(ceil_div(C, kLanes), ceil_div(s.NS, kRows), B);
    generic_fwd_aggregate<kBwdL><<<grid, block, 0, stream>>>(s, w, k, v, carry);
    generic_fwd_carry<<<dim3(ceil_div(C, 128), B), 128, 0, stream>>>(s, w, carry);
    generic_bwd_aggregate<kBwdL><<<grid, block, 0, stream>>>(s, w, u, k, v, gy, carry, adj);
    generic_bwd_carry<<<dim3(ceil_div(C, 128), B), 128, 0, stream>>>(s, w, adj);
    generic_bwd_emit<kBwdL><<<grid, block, 0, stream>>>(s, w, u, k, v, gy, carry, adj, gk, gv,
                                                        partial);
    const int rows = B * static_cast<int>(grid.y);
    reduce_partials<<<dim3(ceil_div(C, 32), 2), dim3(32, 32), 0, stream>>>(partial, rows, C, gwgu);
    return 6;
}

}  // namespace biwkv
