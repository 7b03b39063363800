// Per-thread arithmetic of the bidirectional WKV scan, shared by every Bi-WKV kernel.
//
// Everything here is a pure function of its arguments (no thread indices, no
// memory side effects beyond the pointers it is given), marked host+device so
// the test-suite can compile the same code with a host compiler and drive it
// thread by thread.
//
// A decayed sum  sum_j e^{x_j - w * dist_j} [p_j, q_j]  is carried as a value
// pair and one exponent, [a, b] * e^{o}, with o tracking the running maximum of
// the terms' exponents, so neither e^{k} nor 1/Den is ever formed on its own
// (the reference does the same with MIN_VALUE = -1e38 as "minus infinity",
// classification/mmcls_custom/models/backbones/cuda_new/bi_wkv_kernel.cu:14,48-67).
#pragma once

#if defined(__CUDACC__)
#define WKV_HD __host__ __device__ __forceinline__
#else
#include <cmath>
#include <algorithm>
#define WKV_HD inline
#endif

namespace biwkv {

constexpr float kMinExp = -1e38f;

// Full-accuracy exponential: this header serves the paths that must hold 1e-5 over
// thousands of tokens for any exponent range; the packed fast path has its own ex2.
WKV_HD float wkv_exp(float x) {
#if defined(__CUDA_ARCH__)
    return expf(x);
#else
    return std::exp(x);
#endif
}
WKV_HD float wkv_max(float a, float b) { return a > b ? a : b; }

// [a, b] * e^{o}
struct Acc2 {
    float a, b, o;
};
WKV_HD Acc2 acc2_zero() { return Acc2{0.f, 0.f, kMinExp}; }

// s += e^{x} [p, q]   (no decay)
WKV_HD void acc2_add(Acc2& s, float x, float p, float q) {
    const float no = wkv_max(s.o, x);
    const float e1 = wkv_exp(s.o - no);
    const float e2 = wkv_exp(x - no);
    s.a = e1 * s.a + e2 * p;
    s.b = e1 * s.b + e2 * q;
    s.o = no;
}
// every term moves n tokens further away
WKV_HD void acc2_decay(Acc2& s, float w, float n) { s.o -= w * n; }
WKV_HD Acc2 acc2_merge(const Acc2& x, const Acc2& y) {
    const float no = wkv_max(x.o, y.o);
    const float e1 = wkv_exp(x.o - no);
    const float e2 = wkv_exp(y.o - no);
    return Acc2{e1 * x.a + e2 * y.a, e1 * x.b + e2 * y.b, no};
}

// value pair [a, b] and its first moment in distance [ma, mb], one exponent:
//   [a, b]   = sum_t e^{-w d_t} X_t,   [ma, mb] = sum_t d_t e^{-w d_t} X_t
struct Acc4 {
    float a, b, ma, mb, o;
};
WKV_HD Acc4 acc4_zero() { return Acc4{0.f, 0.f, 0.f, 0.f, kMinExp}; }
// absorb X = e^{x}[p, q] at distance 0, then move everything one token away
WKV_HD void acc4_step(Acc4& s, float x, float p, float q, float w) {
    const float no = wkv_max(s.o, x);
    const float e1 = wkv_exp(s.o - no);
    const float e2 = wkv_exp(x - no);
    s.a = e1 * s.a + e2 * p;
    s.b = e1 * s.b + e2 * q;
    s.ma = e1 * s.ma + s.a;
    s.mb = e1 * s.mb + s.b;
    s.o = no - w;
}
// absorb X = e^{x}[p, q] and count one more unit of distance for everything held so far,
// without moving the exponent: for sweeps that fold the position into x (see below)
WKV_HD void acc4_absorb(Acc4& s, float x, float p, float q) {
    const float no = wkv_max(s.o, x);
    const float e1 = wkv_exp(s.o - no);
    const float e2 = wkv_exp(x - no);
    s.a = e1 * s.a + e2 * p;
    s.b = e1 * s.b + e2 * q;
    s.ma = e1 * s.ma + s.a;
    s.mb = e1 * s.mb + s.b;
    s.o = no;
}
// every term moves n tokens further away
WKV_HD void acc4_decay(Acc4& s, float w, float n) {
    s.ma += n * s.a;
    s.mb += n * s.b;
    s.o -= w * n;
}
WKV_HD Acc4 acc4_merge(const Acc4& x, const Acc4& y) {
    const float no = wkv_max(x.o, y.o);
    const float e1 = wkv_exp(x.o - no);
    const float e2 = wkv_exp(y.o - no);
    return Acc4{e1 * x.a + e2 * y.a, e1 * x.b + e2 * y.b, e1 * x.ma + e2 * y.ma,
                e1 * x.mb + e2 * y.mb, no};
}

// Position-anchored sweeps.  Subtracting w from the exponent once per token would add one
// rounding of the exponent per token, a random walk that reaches 1e-5 after a few
// thousand tokens.  The per-token loops therefore keep the state's exponent relative to a
// fixed anchor position: a term of token i enters with exponent x_i + w * (its distance
// from the anchor, counted against the sweep direction), and the state seen at distance d
// from the anchor is [a, b] e^{o - w d}.  Only the hand-over between sub-chunks moves an
// exponent, once per sub-chunk.
WKV_HD Acc2 acc2_at(const Acc2& s, float w, float d) { return Acc2{s.a, s.b, s.o - w * d}; }

// One token's output from its prefix state P, suffix state S and own term:
//   y = (P + S + e^{u+k}[v,1]) ratio.  Also returns 1/den' and the shift m with
//   Den = den' * e^{m}  (what the backward needs).
struct TokenOut {
    float y, inv_den, m;
};
WKV_HD TokenOut token_out(const Acc2& P, const Acc2& S, float k, float v, float u) {
    const float own = u + k;
    const float m = wkv_max(wkv_max(P.o, S.o), own);
    const float e1 = wkv_exp(P.o - m);
    const float e2 = wkv_exp(S.o - m);
    const float e3 = wkv_exp(own - m);
    const float num = P.a * e1 + S.a * e2 + e3 * v;
    const float den = P.b * e1 + S.b * e2 + e3;
    const float inv = 1.0f / den;
    return TokenOut{num * inv, inv, m};
}

}  // namespace biwkv
