// Bi-WKV "generic" path: any B, T, C, any alignment, exponent-safe for any w, u, k.
//
// The sequence of every (batch, channel) pair is cut into sub-chunks of L tokens;
// one thread owns one (batch, sub-chunk, channel), lanes run along channels so a
// warp reads 128 contiguous bytes of a token row.  Three launches make a forward,
// six a backward:
//
//   aggregate : per sub-chunk, the decayed sums it contributes to its right and to
//               its left neighbour                         (reads k, v)
//   carry     : per (batch, channel), a serial walk over the sub-chunk aggregates
//               turning them, in place, into the prefix state entering each
//               sub-chunk from the left and the suffix state entering it from the
//               right
//   emit      : per sub-chunk, suffix sweep (kept in registers), prefix sweep, output
//
// and for the backward the same three steps once more on the adjoint pairs
// [G, H] = [gy/Den, gy*y/Den] (with their first moments in distance, which give gw),
// followed by a fixed-order reduction of the per-sub-chunk gw/gu partials.  Nothing
// per-token is stored between launches: every launch recomputes what it needs from
// k, v, gy and the O(T/L) carries.
//
// The functions below are the per-thread bodies; they compile for host and device.
// Math being restated: the recurrence of
// classification/mmcls_custom/models/backbones/cuda_new/bi_wkv_kernel.cu:21-116 (y)
// and the gradients it returns at :119-367 (gw, gu, gk, gv).
#pragma once
#include "biwkv_math.cuh"

namespace biwkv {

struct GenericShape {
    int B, T, C;
    int L;    // tokens per sub-chunk
    int NS;   // sub-chunks per sequence = ceil(T / L)
};

// scratch rows: [B][NS][ROWS][C]
WKV_HD size_t scratch_index(const GenericShape& s, int rows, int b, int sc, int row, int c) {
    return ((static_cast<size_t>(b) * s.NS + sc) * rows + row) * s.C + c;
}
WKV_HD size_t token_index(const GenericShape& s, int b, int t, int c) {
    return (static_cast<size_t>(b) * s.T + t) * s.C + c;
}

constexpr int kFwdRows = 6;    // prefix a,b,o | suffix a,b,o
constexpr int kAdjRows = 10;   // towards-later a,b,ma,mb,o | towards-earlier a,b,ma,mb,o

WKV_HD void store_acc2(float* base, size_t stride, const Acc2& s) {
    base[0] = s.a; base[stride] = s.b; base[2 * stride] = s.o;
}
WKV_HD Acc2 load_acc2(const float* base, size_t stride) {
    return Acc2{base[0], base[stride], base[2 * stride]};
}
WKV_HD void store_acc4(float* base, size_t stride, const Acc4& s) {
    base[0] = s.a; base[stride] = s.b; base[2 * stride] = s.ma; base[3 * stride] = s.mb;
    base[4 * stride] = s.o;
}
WKV_HD Acc4 load_acc4(const float* base, size_t stride) {
    return Acc4{base[0], base[stride], base[2 * stride], base[3 * stride], base[4 * stride]};
}

// ---- step 1: sub-chunk aggregates of e^{k}[v,1] ----------------------------------
template <int L>
WKV_HD void fwd_aggregate_thread(const GenericShape& s, const float* w_, const float* k_,
                                 const float* v_, float* carry, int b, int sc, int c) {
    const float w = w_[c];
    const int t0 = sc * L;
    const int n = (s.T - t0 < L) ? (s.T - t0) : L;
    float kk[L], vv[L];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (i < n) {
            const size_t idx = token_index(s, b, t0 + i, c);
            kk[i] = k_[idx];
            vv[i] = v_[idx];
        } else {
            kk[i] = 0.f; vv[i] = 0.f;
        }
    }
    Acc2 right = acc2_zero();   // what this sub-chunk adds to the prefix state of the token after it
#pragma unroll
    for (int i = 0; i < L; ++i)
        if (i < n) acc2_add(right, kk[i] + w * static_cast<float>(i), vv[i], 1.f);     // anchor: token 0
    acc2_decay(right, w, static_cast<float>(n));
    Acc2 left = acc2_zero();    // what it adds to the suffix state of the token before it
#pragma unroll
    for (int i = L - 1; i >= 0; --i)
        if (i < n) acc2_add(left, kk[i] - w * static_cast<float>(i), vv[i], 1.f);      // anchor: token 0, leftwards
    acc2_decay(left, w, 1.f);
    float* base = carry + scratch_index(s, kFwdRows, b, sc, 0, c);
    store_acc2(base, s.C, right);
    store_acc2(base + 3 * static_cast<size_t>(s.C), s.C, left);
}

// ---- step 2: aggregates -> entering states, in place -------------------------------
// The running exponent of the walk is kept in double: it is decremented once per sub-chunk,
// hundreds of times along a long sequence, and in float those roundings add up to ~1e-5.
WKV_HD void fwd_carry_thread(const GenericShape& s, const float* w_, float* carry, int b, int c) {
    const double w = w_[c];
    for (int dir = 0; dir < 2; ++dir) {
        float a = 0.f, bb = 0.f;
        double o = kMinExp;
        for (int q = 0; q < s.NS; ++q) {
            const int sc = dir == 0 ? q : s.NS - 1 - q;
            float* base = carry + scratch_index(s, kFwdRows, b, sc, dir * 3, c);
            const Acc2 agg = load_acc2(base, s.C);
            store_acc2(base, s.C, Acc2{a, bb, static_cast<float>(o)});
            const int t0 = sc * s.L;
            const int n = (s.T - t0 < s.L) ? (s.T - t0) : s.L;
            o -= w * n;
            const double no = o > agg.o ? o : static_cast<double>(agg.o);
            const float e1 = wkv_exp(static_cast<float>(o - no));
            const float e2 = wkv_exp(static_cast<float>(agg.o - no));
            a = e1 * a + e2 * agg.a;
            bb = e1 * bb + e2 * agg.b;
            o = no;
        }
    }
}

// Recompute the forward of one sub-chunk from its entering states.  Calls
// sink(i, k_i, v_i, TokenOut) for every valid token, in ascending order.
template <int L, typename Sink>
WKV_HD void fwd_recompute(const float (&kk)[L], const float (&vv)[L], int n, float w, float u,
                          Acc2 P, Acc2 S, Sink&& sink) {
    // S enters at the last valid token, P at token 0; both sweeps are anchored there.
    Acc2 stash[L];
    const float last = static_cast<float>(n - 1);
#pragma unroll
    for (int i = L - 1; i >= 0; --i) {
        if (i < n) {
            const float d = last - static_cast<float>(i);
            stash[i] = acc2_at(S, w, d);
            acc2_add(S, kk[i] + w * d, vv[i], 1.f);
        }
    }
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (i < n) {
            const float d = static_cast<float>(i);
            sink(i, token_out(acc2_at(P, w, d), stash[i], kk[i], vv[i], u));
            acc2_add(P, kk[i] + w * d, vv[i], 1.f);
        }
    }
}

// ---- step 3: y ---------------------------------------------------------------------
template <int L>
WKV_HD void fwd_emit_thread(const GenericShape& s, const float* w_, const float* u_,
                            const float* k_, const float* v_, const float* carry, float* y_,
                            int b, int sc, int c) {
    const float w = w_[c], u = u_[c];
    const int t0 = sc * L;
    const int n = (s.T - t0 < L) ? (s.T - t0) : L;
    float kk[L], vv[L];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (i < n) {
            const size_t idx = token_index(s, b, t0 + i, c);
            kk[i] = k_[idx];
            vv[i] = v_[idx];
        } else {
            kk[i] = 0.f; vv[i] = 0.f;
        }
    }
    const float* base = carry + scratch_index(s, kFwdRows, b, sc, 0, c);
    const Acc2 P = load_acc2(base, s.C);
    const Acc2 S = load_acc2(base + 3 * static_cast<size_t>(s.C), s.C);
    float* y = y_ + token_index(s, b, t0, c);
    const size_t C = s.C;
    fwd_recompute<L>(kk, vv, n, w, u, P, S,
                     [&](int i, const TokenOut& o) { y[i * C] = o.y; });
}

// ---- backward step 3': sub-chunk aggregates of the adjoint pairs --------------------
template <int L>
WKV_HD void bwd_aggregate_thread(const GenericShape& s, const float* w_, const float* u_,
                                 const float* k_, const float* v_, const float* gy_,
                                 const float* carry, float* adj, int b, int sc, int c) {
    const float w = w_[c], u = u_[c];
    const int t0 = sc * L;
    const int n = (s.T - t0 < L) ? (s.T - t0) : L;
    float kk[L], vv[L], gg[L];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (i < n) {
            const size_t idx = token_index(s, b, t0 + i, c);
            kk[i] = k_[idx];
            vv[i] = v_[idx];
            gg[i] = gy_[idx];
        } else {
            kk[i] = 0.f; vv[i] = 0.f; gg[i] = 0.f;
        }
    }
    const float* base = carry + scratch_index(s, kFwdRows, b, sc, 0, c);
    const Acc2 P = load_acc2(base, s.C);
    const Acc2 S = load_acc2(base + 3 * static_cast<size_t>(s.C), s.C);
    float hh[L], xo[L];
    fwd_recompute<L>(kk, vv, n, w, u, P, S, [&](int i, const TokenOut& o) {
        gg[i] = gg[i] * o.inv_den;   // G_i e^{m_i}
        hh[i] = gg[i] * o.y;         // H_i e^{m_i}
        xo[i] = -o.m;
    });
    Acc4 later = acc4_zero();     // what the outputs of this sub-chunk send to later inputs
#pragma unroll
    for (int i = 0; i < L; ++i)
        if (i < n) acc4_absorb(later, xo[i] + w * static_cast<float>(i), gg[i], hh[i]);
    later.o -= w * static_cast<float>(n);
    Acc4 earlier = acc4_zero();   // ... and to earlier inputs
#pragma unroll
    for (int i = L - 1; i >= 0; --i)
        if (i < n) acc4_absorb(earlier, xo[i] - w * static_cast<float>(i), gg[i], hh[i]);
    earlier.o -= w;
    float* out = adj + scratch_index(s, kAdjRows, b, sc, 0, c);
    store_acc4(out, s.C, later);
    store_acc4(out + 5 * static_cast<size_t>(s.C), s.C, earlier);
}

WKV_HD void bwd_carry_thread(const GenericShape& s, const float* w_, float* adj, int b, int c) {
    const double w = w_[c];
    for (int dir = 0; dir < 2; ++dir) {
        float a = 0.f, bb = 0.f, ma = 0.f, mb = 0.f;
        double o = kMinExp;
        for (int q = 0; q < s.NS; ++q) {
            const int sc = dir == 0 ? q : s.NS - 1 - q;
            float* base = adj + scratch_index(s, kAdjRows, b, sc, dir * 5, c);
            const Acc4 agg = load_acc4(base, s.C);
            store_acc4(base, s.C, Acc4{a, bb, ma, mb, static_cast<float>(o)});
            const int t0 = sc * s.L;
            const int n = (s.T - t0 < s.L) ? (s.T - t0) : s.L;
            ma += n * a;
            mb += n * bb;
            o -= w * n;
            const double no = o > agg.o ? o : static_cast<double>(agg.o);
            const float e1 = wkv_exp(static_cast<float>(o - no));
            const float e2 = wkv_exp(static_cast<float>(agg.o - no));
            a = e1 * a + e2 * agg.a;
            bb = e1 * bb + e2 * agg.b;
            ma = e1 * ma + e2 * agg.ma;
            mb = e1 * mb + e2 * agg.mb;
            o = no;
        }
    }
}

// ---- backward step 5: gk, gv and this sub-chunk's share of gw, gu --------------------
template <int L>
WKV_HD void bwd_emit_thread(const GenericShape& s, const float* w_, const float* u_,
                            const float* k_, const float* v_, const float* gy_,
                            const float* carry, const float* adj, float* gk_, float* gv_,
                            float& gw_out, float& gu_out, int b, int sc, int c) {
    const float w = w_[c], u = u_[c];
    const int t0 = sc * L;
    const int n = (s.T - t0 < L) ? (s.T - t0) : L;
    float kk[L], vv[L], gg[L];
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (i < n) {
            const size_t idx = token_index(s, b, t0 + i, c);
            kk[i] = k_[idx];
            vv[i] = v_[idx];
            gg[i] = gy_[idx];
        } else {
            kk[i] = 0.f; vv[i] = 0.f; gg[i] = 0.f;
        }
    }
    const float* base = carry + scratch_index(s, kFwdRows, b, sc, 0, c);
    const Acc2 P = load_acc2(base, s.C);
    const Acc2 S = load_acc2(base + 3 * static_cast<size_t>(s.C), s.C);
    float hh[L], xo[L];
    fwd_recompute<L>(kk, vv, n, w, u, P, S, [&](int i, const TokenOut& o) {
        gg[i] = gg[i] * o.inv_den;
        hh[i] = gg[i] * o.y;
        xo[i] = -o.m;
    });
    const float* abase = adj + scratch_index(s, kAdjRows, b, sc, 0, c);
    Acc4 R = load_acc4(abase, s.C);                                      // from outputs before t0
    Acc4 Q = load_acc4(abase + 5 * static_cast<size_t>(s.C), s.C);       // from outputs after the sub-chunk
    float gw = 0.f, gu = 0.f;
    float pk[L], pv[L];
    const float last = static_cast<float>(n - 1);
#pragma unroll
    for (int i = L - 1; i >= 0; --i) {
        if (i < n) {
            const float d = last - static_cast<float>(i);     // Q is anchored at the last valid token
            const float e = wkv_exp(kk[i] + Q.o - w * d);
            pv[i] = e * Q.a;
            pk[i] = e * (Q.a * vv[i] - Q.b);
            gw -= e * (Q.ma * vv[i] - Q.mb);
            acc4_absorb(Q, xo[i] + w * d, gg[i], hh[i]);
        }
    }
    float* gk = gk_ + token_index(s, b, t0, c);
    float* gv = gv_ + token_index(s, b, t0, c);
    const size_t C = s.C;
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (i < n) {
            const float d = static_cast<float>(i);            // R is anchored at token 0
            const float e = wkv_exp(kk[i] + R.o - w * d);
            const float es = wkv_exp(u + kk[i] + xo[i]);
            const float self = es * (vv[i] * gg[i] - hh[i]);   // e^{u+k}(v - y) G
            gv[i * C] = pv[i] + e * R.a + es * gg[i];
            gk[i * C] = pk[i] + e * (R.a * vv[i] - R.b) + self;
            gu += self;
            gw -= e * (R.ma * vv[i] - R.mb);
            acc4_absorb(R, xo[i] + w * d, gg[i], hh[i]);
        }
    }
    gw_out = gw;
    gu_out = gu;
}

}  // namespace biwkv
