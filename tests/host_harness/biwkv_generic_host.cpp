// Host-compiled driver for the per-thread bodies of the generic Bi-WKV kernels.
// TEST INFRASTRUCTURE: it lets the CPU test-suite check the arithmetic and the
// index maps of the CUDA kernels (same header, host compiler) against the oracle
// on machines without a GPU.  The product never builds or loads this file.
#include <cstddef>
#include <vector>
#include "biwkv_generic.cuh"

using namespace biwkv;

template <int L>
static void run_forward(int B, int T, int C, const float* w, const float* u, const float* k,
                        const float* v, float* y) {
    GenericShape s{B, T, C, L, (T + L - 1) / L};
    std::vector<float> carry(static_cast<size_t>(B) * s.NS * kFwdRows * C);
    for (int b = 0; b < B; ++b)
        for (int sc = 0; sc < s.NS; ++sc)
            for (int c = 0; c < C; ++c) fwd_aggregate_thread<L>(s, w, k, v, carry.data(), b, sc, c);
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < C; ++c) fwd_carry_thread(s, w, carry.data(), b, c);
    for (int b = 0; b < B; ++b)
        for (int sc = 0; sc < s.NS; ++sc)
            for (int c = 0; c < C; ++c)
                fwd_emit_thread<L>(s, w, u, k, v, carry.data(), y, b, sc, c);
}

template <int L>
static void run_backward(int B, int T, int C, const float* w, const float* u, const float* k,
                         const float* v, const float* gy, float* gwgu, float* gk, float* gv) {
    GenericShape s{B, T, C, L, (T + L - 1) / L};
    std::vector<float> carry(static_cast<size_t>(B) * s.NS * kFwdRows * C);
    std::vector<float> adj(static_cast<size_t>(B) * s.NS * kAdjRows * C);
    for (int b = 0; b < B; ++b)
        for (int sc = 0; sc < s.NS; ++sc)
            for (int c = 0; c < C; ++c) fwd_aggregate_thread<L>(s, w, k, v, carry.data(), b, sc, c);
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < C; ++c) fwd_carry_thread(s, w, carry.data(), b, c);
    for (int b = 0; b < B; ++b)
        for (int sc = 0; sc < s.NS; ++sc)
            for (int c = 0; c < C; ++c)
                bwd_aggregate_thread<L>(s, w, u, k, v, gy, carry.data(), adj.data(), b, sc, c);
    for (int b = 0; b < B; ++b)
        for (int c = 0; c < C; ++c) bwd_carry_thread(s, w, adj.data(), b, c);
    for (int c = 0; c < 2 * C; ++c) gwgu[c] = 0.f;
    for (int b = 0; b < B; ++b)
        for (int sc = 0; sc < s.NS; ++sc)
            for (int c = 0; c < C; ++c) {
                float gw, gu;
                bwd_emit_thread<L>(s, w, u, k, v, gy, carry.data(), adj.data(), gk, gv, gw, gu, b,
                                   sc, c);
                gwgu[c] += gw;
                gwgu[C + c] += gu;
            }
}

extern "C" {
void host_biwkv_forward(int L, int B, int T, int C, const float* w, const float* u,
                        const float* k, const float* v, float* y) {
    if (L == 16) run_forward<16>(B, T, C, w, u, k, v, y);
    else run_forward<8>(B, T, C, w, u, k, v, y);
}
void host_biwkv_backward(int L, int B, int T, int C, const float* w, const float* u,
                         const float* k, const float* v, const float* gy, float* gwgu, float* gk,
                         float* gv) {
    if (L == 16) run_backward<16>(B, T, C, w, u, k, v, gy, gwgu, gk, gv);
    else run_backward<8>(B, T, C, w, u, k, v, gy, gwgu, gk, gv);
}
}
