// Bi-WKV "fused" path: one persistent kernel per forward (biwkv_forward_pipelined_kernel), one
// per backward (biwkv_fused_kernel<true>), each element of k, v (and gy) crossing HBM once in
// and each output once out.
//
// Work unit ("tile"): kTc = 128 consecutive tokens x kCs = 32 consecutive channels of
// one sequence.  A CTA is 8 warps; warp s owns the sub-chunk of kL = 16 tokens
// [16 s, 16 s + 16) of the tile, its lane c the channel; a thread walks its 16 tokens
// sequentially out of shared memory.  Thread 0 moves tiles with TMA (tiled 3-D tensor maps
// over (C, T, B): zero fill past T and C on load, clipping on store), double-buffered.
//
// The scan needs, at every token, the decayed sum over all earlier tokens of the
// sequence and over all later ones.  Per scan level every warp
//   1. posts its sub-chunk aggregate (both directions) to shared memory;
//   2. sums the aggregates of the other sub-chunks of its tile that lie before / after it;
//      warp 7 (resp. 0) thereby holds the whole tile's rightward (leftward) aggregate,
//      writes it to the tile's global exchange record and bumps the tile's flag;
//   3. waits (bounded spin) for the flags of the tiles j = s, s + 8, ... of the same
//      (sequence, channel strip), reads their records back through L2 and posts the partial
//      sum to shared memory;
//   4. adds the eight partials and its own inside sum: the state entering its sub-chunk.
// No tile waits for another tile's *result*, only for its aggregate, which depends on that
// tile's own data alone, so one exchange round suffices per level (one level in the
// forward: e^{k}[v,1]; a second in the backward: the adjoint pairs [gy/Den, gy y/Den]).
// All sums over several (value, exponent) records take the maximum exponent first and then
// add the rescaled values, so the exponentials are independent and pipeline.
//
// The kernel is launched cooperatively with one CTA per resident slot and walks the tile
// list round-robin; consecutive tile ids are the chunks of one (sequence, strip), so the
// peers of a tile are in flight at the same time on neighbouring CTAs.  A tile only waits for
// tiles whose ids differ by less than the grid size, all started by resident CTAs, so the
// wait cannot deadlock; it is bounded anyway and sets bit 0 of the workspace status word
// instead of hanging.
//
// Numerics.  All hand-overs are (value, exponent) pairs as in biwkv_math.cuh.  Inside a
// sub-chunk a thread shifts by one reference exponent (the maximum over its 16 k values
// and the states entering it) and then runs plain decayed recurrences with lambda =
// e^{-w}, packed two floats per instruction (numerator|denominator).  That is exact
// enough whenever (max k - min k) + 16 |w| + |u| <= 60 inside the sub-chunk; a warp that
// sees otherwise takes the per-token max-shifted path of biwkv_math.cuh for that tile.
//
// Recurrence restated: classification/mmcls_custom/models/backbones/cuda_new/
// bi_wkv_kernel.cu:21-116 (forward), :119-367 (gradients).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdint>
#include <initializer_list>
#include <mutex>
#include <type_traits>
#include "biwkv_math.cuh"
#include "sm100_async.cuh"
#include "tensor_map.h"
#include "vrwkv_internal.h"

namespace biwkv {
namespace fused {

constexpr int kL = 16;                 // tokens per thread
constexpr int kWarps = 8;              // warps = sub-chunks per tile
constexpr int kTc = kL * kWarps;       // tokens per tile
constexpr int kCs = 32;                // channels per tile
constexpr int kThreads = kWarps * 32;
constexpr int kSlotFloats = kTc * kCs;
constexpr int kRows = 8;               // exchange rows per channel: a,b,ma,mb,o | a,b,o
constexpr int kRecFloats = kRows * kCs;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kFastRange = 60.f;
constexpr uint32_t kSpinLimit = 1u << 20;   // ~0.1 s of polling

// Division of a non-negative 31-bit number by a launch constant: q = (n * mul) >> shift with
// mul = ceil(2^shift / d), shift = 31 + ceil(log2 d) (exact for every n < 2^31).  The tile loops
// decode their tile id several times per tile; three hardware divisions each were a tenth of the
// forward's instructions.
struct FastDiv {
    uint32_t mul, shift;
};
static inline FastDiv make_fastdiv(uint32_t d) {
    uint32_t s = 0;
    while ((1u << s) < d) ++s;
    FastDiv f;
    f.mul = static_cast<uint32_t>(((1ull << (31 + s)) + d - 1) / d);
    f.shift = 31 + s;
    return f;
}
__device__ __forceinline__ int fast_div(int n, FastDiv f) {
    return static_cast<int>((static_cast<uint64_t>(static_cast<uint32_t>(n)) * f.mul) >> f.shift);
}

struct Params {
    int B, T, C;
    int n_chunks;      // tiles along T
    int n_strips;      // tiles along C
    int interleave;    // strips whose tiles alternate in the id order (divides n_strips)
    int n_tiles;
    FastDiv by_span, by_interleave, by_strips;
    const float* w;
    const float* u;
    float* exch;       // [n_tiles][levels][kRows][kCs]
    unsigned* flags;   // [n_tiles][levels], zero before launch, 2 when both halves are written
    unsigned* status;  // device status word
    float* partial;    // backward: [n_tiles][2][kCs]
    const unsigned* run_if;   // when set: every kernel of the launch returns at once while this word is zero
};
__device__ __forceinline__ bool switched_off(const Params& p) {
    return p.run_if != nullptr && *reinterpret_cast<const volatile unsigned*>(p.run_if) == 0u;
}

struct TileCoord {
    int b, strip, chunk;
};
__device__ __forceinline__ TileCoord decode_tile(const Params& p, int id) {
    const int span = p.interleave * p.n_chunks;
    const int block = fast_div(id, p.by_span);
    const int r = id - block * span;
    const int chunk = fast_div(r, p.by_interleave);
    const int gs = block * p.interleave + (r - chunk * p.interleave);   // strip index over all sequences
    TileCoord t;
    t.b = fast_div(gs, p.by_strips);
    t.strip = gs - t.b * p.n_strips;
    t.chunk = chunk;
    return t;
}

__device__ __forceinline__ float fast_exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * kLog2e));
    return y;
}
__device__ __forceinline__ float2 f2(float a, float b) { return make_float2(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// One thread's column of a tile in shared memory: element i = token i of the warp's sub-chunk,
// channel = lane.  float tiles are read and written in place.  bfloat16 tiles are read as the
// 32-bit word that holds a lane pair and written by the even lane after a shuffle, because 2-byte
// shared accesses are slow on this part; st() must therefore be reached by all 32 lanes together.
template <typename E>
struct Col;
template <>
struct Col<float> {
    float* p;
    __device__ __forceinline__ Col(void* slot, int warp, int lane)
        : p(static_cast<float*>(slot) + (warp * kL) * kCs + lane) {}
    __device__ __forceinline__ float ld(int i) const { return p[i * kCs]; }
    __device__ __forceinline__ void st(int i, float x) const { p[i * kCs] = x; }
};
template <>
struct Col<__nv_bfloat16> {
    uint32_t* p;
    bool hi;
    __device__ __forceinline__ Col(void* slot, int warp, int lane)
        : p(static_cast<uint32_t*>(slot) + (warp * kL) * (kCs / 2) + (lane >> 1)), hi(lane & 1) {}
    __device__ __forceinline__ float ld(int i) const {
        const uint32_t word = p[i * (kCs / 2)];
        return __uint_as_float(hi ? (word & 0xffff0000u) : (word << 16));
    }
    __device__ __forceinline__ void st(int i, float x) const {
        const float other = __shfl_xor_sync(0xffffffffu, x, 1);
        if (!hi) {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(x, other);
            p[i * (kCs / 2)] = *reinterpret_cast<const uint32_t*>(&pair);
        }
    }
};
template <typename E>
constexpr uint32_t kSlotBytes = kTc * kCs * sizeof(E);

// ---- exchange records: rec[row * kCs], rec already offset by the lane -------------------------
__device__ __forceinline__ void post_acc4(float* rec, const Acc4& s) {
    rec[0 * kCs] = s.a; rec[1 * kCs] = s.b; rec[2 * kCs] = s.ma; rec[3 * kCs] = s.mb; rec[4 * kCs] = s.o;
}
__device__ __forceinline__ void post_acc2(float* rec, const Acc2& s) {
    rec[5 * kCs] = s.a; rec[6 * kCs] = s.b; rec[7 * kCs] = s.o;
}
__device__ __forceinline__ Acc4 merge4(const Acc4& x, const Acc4& y) {
    const float no = wkv_max(x.o, y.o);
    const float e1 = fast_exp(x.o - no), e2 = fast_exp(y.o - no);
    return Acc4{e1 * x.a + e2 * y.a, e1 * x.b + e2 * y.b, e1 * x.ma + e2 * y.ma, e1 * x.mb + e2 * y.mb, no};
}
__device__ __forceinline__ Acc2 merge2(const Acc2& x, const Acc2& y) {
    const float no = wkv_max(x.o, y.o);
    const float e1 = fast_exp(x.o - no), e2 = fast_exp(y.o - no);
    return Acc2{e1 * x.a + e2 * y.a, e1 * x.b + e2 * y.b, no};
}

struct Entering {
    Acc4 left;    // state entering the sub-chunk at its first token (with first moments)
    Acc2 right;   // state entering it at its last position
};

struct Inside {
    Acc4 inP;     // what the earlier sub-chunks of the same tile send to this one
    Acc2 inS;     // ... and the later ones
};

// First half of an exchange level for one warp (steps 1-2 of the file header): post, sum the
// rest of the tile, publish the tile aggregate.  own_right / own_left: this sub-chunk's
// aggregates, relative to the position after its 16-token span / before it.
__device__ __forceinline__ Inside exchange_publish(const Params& p, float* sub, int lane, int warp, float w,
                                                   int tile, int level, int levels, const Acc4& own_right,
                                                   const Acc2& own_left) {
    post_acc4(sub + warp * kRecFloats + lane, own_right);
    post_acc2(sub + warp * kRecFloats + lane, own_left);
    __syncthreads();
    // (2) the other sub-chunks of this tile
    Acc4 inP;
    Acc2 inS;
    {
        float x4[kWarps], x2[kWarps];
        float m4 = kMinExp, m2 = kMinExp;
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            const float* r = sub + s * kRecFloats + lane;
            x4[s] = (s < warp) ? r[4 * kCs] - w * static_cast<float>((warp - 1 - s) * kL) : kMinExp;
            x2[s] = (s > warp) ? r[7 * kCs] - w * static_cast<float>((s - warp - 1) * kL) : kMinExp;
            m4 = wkv_max(m4, x4[s]);
            m2 = wkv_max(m2, x2[s]);
        }
        inP = Acc4{0.f, 0.f, 0.f, 0.f, m4};
        inS = Acc2{0.f, 0.f, m2};
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            const float* r = sub + s * kRecFloats + lane;
            if (s < warp) {
                const float f = fast_exp(x4[s] - m4);
                const float d = static_cast<float>((warp - 1 - s) * kL);
                const float a = r[0], b = r[kCs];
                inP.a += f * a;
                inP.b += f * b;
                inP.ma += f * (r[2 * kCs] + d * a);
                inP.mb += f * (r[3 * kCs] + d * b);
            }
            if (s > warp) {
                const float f = fast_exp(x2[s] - m2);
                inS.a += f * r[5 * kCs];
                inS.b += f * r[6 * kCs];
            }
        }
    }
    // publish the tile's aggregate: rightward half by the last warp, leftward by the first
    if (warp == kWarps - 1 || warp == 0) {
        float* mine = p.exch + (static_cast<size_t>(tile) * levels + level) * kRecFloats + lane;
        if (warp == kWarps - 1) {
            Acc4 t = inP;
            acc4_decay(t, w, static_cast<float>(kL));
            post_acc4(mine, merge4(t, own_right));
        }
        if (warp == 0) {
            Acc2 t = inS;
            acc2_decay(t, w, static_cast<float>(kL));
            post_acc2(mine, merge2(t, own_left));
        }
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            atomicAdd(p.flags + static_cast<size_t>(tile) * levels + level, 1u);
        }
    }
    return Inside{inP, inS};
}

// Second half (steps 3-4): collect the other tiles' aggregates and form the entering states.
__device__ __forceinline__ Entering exchange_collect(const Params& p, float* ext, int lane, int warp, float w,
                                                     int tile, int chunk, int level, int levels,
                                                     const Inside& in) {
    const Acc4 inP = in.inP;
    const Acc2 inS = in.inS;
    // (3) the records of the tiles j = warp, warp + 8, ... of this (sequence, strip)
    {
        const int first = tile - chunk * p.interleave;
        Acc4 P = acc4_zero();
        Acc2 S = acc2_zero();
        for (int j0 = warp; j0 < p.n_chunks; j0 += 4 * kWarps) {
            // Poll the (up to four) flags of the batch together: independent relaxed loads, one
            // round trip through L2 for all of them; once all are set, one acquire load per flag
            // (again together) orders the record loads behind the publishers' writes.  The
            // publisher put a fence between its record and its flag.
            bool ok = true;
            const unsigned* fl[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                fl[q] = (j < p.n_chunks && j != chunk)
                            ? p.flags + static_cast<size_t>(first + j * p.interleave) * levels + level
                            : nullptr;
            }
            unsigned seen[4] = {0u, 0u, 0u, 0u};
            for (uint32_t spins = 0;; ++spins) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (seen[q] < 2u) seen[q] = fl[q] ? sm100::flag_relaxed(fl[q]) : 2u;   // only what is still missing
                if (seen[0] >= 2u && seen[1] >= 2u && seen[2] >= 2u && seen[3] >= 2u) break;
                // give up after ~0.1 s, or at once if any wait of this launch already did
                if (spins > kSpinLimit ||
                    ((spins & 1023u) == 1023u && *reinterpret_cast<volatile unsigned*>(p.status) != 0u)) {
                    ok = false;
                    break;
                }
                __nanosleep(spins < 8 ? 32 : 128);
            }
            // the polls above are relaxed; one acquire load per flag, issued together, is what orders
            // the record loads below after the publishers' writes (the address dependency through
            // `dep` alone is not an ordering the PTX memory model gives)
            if (ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (fl[q]) seen[q] |= sm100::flag_acquire(fl[q]);
            }
            const unsigned seen_all = seen[0] | seen[1] | seen[2] | seen[3];
            const size_t dep = seen_all >> 31;
            if (!ok && lane == 0) atomicOr(p.status, 1u);
            // all loads of the batch first, then the arithmetic
            float r0[4], r1[4], r2[4], r3[4], x[4];
            float mP = kMinExp, mS = kMinExp;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                r0[q] = r1[q] = r2[q] = r3[q] = 0.f;
                x[q] = kMinExp;
                if (j < p.n_chunks && j != chunk) {
                    const float* rec = p.exch + (static_cast<size_t>(first + j * p.interleave) * levels + level) * kRecFloats + lane + dep;
                    if (j < chunk) {
                        r0[q] = sm100::ld_cg(rec); r1[q] = sm100::ld_cg(rec + kCs);
                        r2[q] = sm100::ld_cg(rec + 2 * kCs); r3[q] = sm100::ld_cg(rec + 3 * kCs);
                        x[q] = sm100::ld_cg(rec + 4 * kCs);
                    } else {
                        r0[q] = sm100::ld_cg(rec + 5 * kCs); r1[q] = sm100::ld_cg(rec + 6 * kCs);
                        x[q] = sm100::ld_cg(rec + 7 * kCs);
                    }
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                if (j < p.n_chunks && j != chunk) {
                    const float d = static_cast<float>((j < chunk ? chunk - 1 - j : j - chunk - 1) * kTc);
                    x[q] -= w * d;
                    if (j < chunk) { r2[q] += d * r0[q]; r3[q] += d * r1[q]; mP = wkv_max(mP, x[q]); }
                    else mS = wkv_max(mS, x[q]);
                }
            }
            Acc4 bp{0.f, 0.f, 0.f, 0.f, mP};
            Acc2 bs{0.f, 0.f, mS};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                if (j < p.n_chunks && j != chunk) {
                    if (j < chunk) {
                        const float f = fast_exp(x[q] - mP);
                        bp.a += f * r0[q]; bp.b += f * r1[q]; bp.ma += f * r2[q]; bp.mb += f * r3[q];
                    } else {
                        const float f = fast_exp(x[q] - mS);
                        bs.a += f * r0[q]; bs.b += f * r1[q];
                    }
                }
            }
            P = merge4(P, bp);
            S = merge2(S, bs);
        }
        post_acc4(ext + warp * kRecFloats + lane, P);
        post_acc2(ext + warp * kRecFloats + lane, S);
    }
    __syncthreads();
    // (4) everything outside the tile, moved to this sub-chunk's edges, plus the inside sums
    Entering out;
    {
        float m4 = kMinExp, m2 = kMinExp;
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            m4 = wkv_max(m4, ext[s * kRecFloats + 4 * kCs + lane]);
            m2 = wkv_max(m2, ext[s * kRecFloats + 7 * kCs + lane]);
        }
        Acc4 P{0.f, 0.f, 0.f, 0.f, m4};
        Acc2 S{0.f, 0.f, m2};
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            const float* r = ext + s * kRecFloats + lane;
            const float f4 = fast_exp(r[4 * kCs] - m4), f2_ = fast_exp(r[7 * kCs] - m2);
            P.a += f4 * r[0]; P.b += f4 * r[kCs]; P.ma += f4 * r[2 * kCs]; P.mb += f4 * r[3 * kCs];
            S.a += f2_ * r[5 * kCs]; S.b += f2_ * r[6 * kCs];
        }
        acc4_decay(P, w, static_cast<float>(warp * kL));
        acc2_decay(S, w, static_cast<float>((kWarps - 1 - warp) * kL));
        out.left = merge4(P, inP);
        out.right = merge2(S, inS);
    }
    return out;
}

// A whole exchange level, for kernels that hold the tile while the peers publish.
__device__ __forceinline__ Entering exchange(const Params& p, float* sub, float* ext, int lane, int warp,
                                             float w, int tile, int chunk, int level, int levels,
                                             const Acc4& own_right, const Acc2& own_left) {
    const Inside in = exchange_publish(p, sub, lane, warp, w, tile, level, levels, own_right, own_left);
    return exchange_collect(p, ext, lane, warp, w, tile, chunk, level, levels, in);
}

// ---- per-token max-shifted path (any exponent range) -------------------------------------------
// Handles one tile for one thread, both exchange levels, out of line so that its register
// needs do not weigh on the packed path.  Sweeps are position-anchored (biwkv_math.cuh).
struct ExchangeCtx {
    float* sub;
    float* ext;
    int lane, warp, tile, chunk;
};

template <bool kBwd, typename E>
__device__ __noinline__ void rigorous_tile(const Params& p, const ExchangeCtx& x, const Col<E> ks, const Col<E> vs,
                                           const Col<E> gs, int n, float w, float u, float& gw_out, float& gu_out) {
    constexpr int kLevels = kBwd ? 2 : 1;
    const float last = static_cast<float>(n - 1);
    Acc4 right = acc4_zero();
    Acc2 left = acc2_zero();
    for (int i = 0; i < n; ++i) acc4_absorb(right, ks.ld(i) + w * static_cast<float>(i), vs.ld(i), 1.f);
    for (int i = n - 1; i >= 0; --i) acc2_add(left, ks.ld(i) - w * static_cast<float>(i), vs.ld(i), 1.f);
    // a short sub-chunk still spans kL positions for its right-hand neighbours
    right.o -= w * static_cast<float>(n);
    acc4_decay(right, w, static_cast<float>(kL - n));
    left.o -= w;
    const Entering e1 = exchange(p, x.sub, x.ext, x.lane, x.warp, w, x.tile, x.chunk, 0, kLevels, right, left);
    const Acc4 P4 = e1.left;                         // anchored at token 0
    Acc2 S = e1.right;
    acc2_decay(S, w, static_cast<float>(kL - n));   // given at position kL-1; anchor it at token n-1
    Acc2 stash[kL];
    for (int i = n - 1; i >= 0; --i) {
        const float d = last - static_cast<float>(i);
        stash[i] = acc2_at(S, w, d);
        acc2_add(S, ks.ld(i) + w * d, vs.ld(i), 1.f);
    }
    if (!kBwd) {
        Acc2 P{P4.a, P4.b, P4.o};
        for (int i = 0; i < n; ++i) {
            const float k = ks.ld(i), v = vs.ld(i), d = static_cast<float>(i);
            const TokenOut o = token_out(acc2_at(P, w, d), stash[i], k, v, u);
            ks.st(i, o.y);
            acc2_add(P, k + w * d, v, 1.f);
        }
        return;
    }
    // backward: G e^{m}, H e^{m}, -m per token; gw from pairs (output later than input)
    float gg[kL], hh[kL], xo[kL];
    float gw = 0.f, gu = 0.f;
    Acc4 PM = P4;   // prefix state with first moments
    for (int i = 0; i < n; ++i) {
        const float k = ks.ld(i), v = vs.ld(i), d = static_cast<float>(i);
        const Acc2 Pi{PM.a, PM.b, PM.o - w * d};
        const TokenOut o = token_out(Pi, stash[i], k, v, u);
        gg[i] = gs.ld(i) * o.inv_den;
        hh[i] = gg[i] * o.y;
        xo[i] = -o.m;
        gw -= wkv_exp(Pi.o + xo[i]) * (gg[i] * PM.ma - hh[i] * PM.mb);
        acc4_absorb(PM, k + w * d, v, 1.f);
    }
    Acc4 later = acc4_zero();
    Acc2 earlier = acc2_zero();
    for (int i = 0; i < n; ++i) acc4_absorb(later, xo[i] + w * static_cast<float>(i), gg[i], hh[i]);
    for (int i = n - 1; i >= 0; --i) acc2_add(earlier, xo[i] - w * static_cast<float>(i), gg[i], hh[i]);
    later.o -= w * static_cast<float>(n);
    acc4_decay(later, w, static_cast<float>(kL - n));
    earlier.o -= w;
    const Entering e2 = exchange(p, x.sub, x.ext, x.lane, x.warp, w, x.tile, x.chunk, 1, kLevels, later, earlier);
    Acc4 R = e2.left;                                // anchored at token 0
    Acc2 Q = e2.right;
    acc2_decay(Q, w, static_cast<float>(kL - n));   // anchored at token n-1
    float pk[kL], pv[kL];
    for (int i = n - 1; i >= 0; --i) {
        const float d = last - static_cast<float>(i);
        const float e = wkv_exp(ks.ld(i) + Q.o - w * d);
        pv[i] = e * Q.a;
        pk[i] = e * (Q.a * vs.ld(i) - Q.b);
        acc2_add(Q, xo[i] + w * d, gg[i], hh[i]);
    }
    for (int i = 0; i < n; ++i) {
        const float k = ks.ld(i), v = vs.ld(i), d = static_cast<float>(i);
        const float e = wkv_exp(k + R.o - w * d);
        const float es = wkv_exp(u + k + xo[i]);
        const float self = es * (v * gg[i] - hh[i]);
        vs.st(i, pv[i] + e * R.a + es * gg[i]);
        ks.st(i, pk[i] + e * (R.a * v - R.b) + self);
        gu += self;
        gw -= e * (R.ma * v - R.mb);
        acc4_absorb(R, xo[i] + w * d, gg[i], hh[i]);
    }
    gw_out = gw;
    gu_out = gu;
}

// ---- the kernel -----------------------------------------------------------------------------
template <bool kBwd, typename E>
__global__ void __launch_bounds__(kThreads, 2)
biwkv_fused_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __grid_constant__ CUtensorMap map_g,     // backward: gy
                   const __grid_constant__ CUtensorMap map_o0,    // forward: y ; backward: gk
                   const __grid_constant__ CUtensorMap map_o1,    // backward: gv
                   const Params p) {
    constexpr int kSlots = kBwd ? 3 : 2;
    constexpr int kLevels = kBwd ? 2 : 1;
    constexpr bool kHalf = !std::is_same<E, float>::value;
    constexpr uint32_t kStageBytes = kSlots * kSlotBytes<E>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if (switched_off(p)) return;
    unsigned char* stage_base = smem_raw;                                           // [2][kSlots][kTc][kCs] of E
    // bfloat16 tiles: the scaled output gradients of the tile in flight stay in fp32 in a region of their own
    float* gscratch = reinterpret_cast<float*>(stage_base + 2 * kStageBytes);       // [kTc][kCs], kBwd && kHalf only
    float* sub = gscratch + ((kBwd && kHalf) ? kSlotFloats : 0);                    // [kWarps][kRows][kCs]
    float* ext = sub + kWarps * kRecFloats;                                         // [kWarps][kRows][kCs]
    float* red = sub;                 // [kWarps][2][kCs]: gw/gu of a tile, between two barriers at its end
    uint64_t* full = reinterpret_cast<uint64_t*>(ext + kWarps * kRecFloats);        // [2]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        sm100::mbar_init(&full[0], 1);
        sm100::mbar_init(&full[1], 1);
        sm100::mbar_init_fence();
    }
    __syncthreads();

    auto issue_loads = [&](int tile, int stage) {
        const TileCoord tc = decode_tile(p, tile);
        unsigned char* dst = stage_base + stage * kStageBytes;
        sm100::mbar_expect_tx(&full[stage], kStageBytes);
        sm100::tma_load_3d(dst, &map_k, &full[stage], tc.strip * kCs, tc.chunk * kTc, tc.b);
        sm100::tma_load_3d(dst + kSlotBytes<E>, &map_v, &full[stage], tc.strip * kCs, tc.chunk * kTc, tc.b);
        if (kBwd)
            sm100::tma_load_3d(dst + 2 * kSlotBytes<E>, &map_g, &full[stage], tc.strip * kCs, tc.chunk * kTc, tc.b);
    };

    if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < p.n_tiles) issue_loads(blockIdx.x, 0);

    int it = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
        const int stage = it & 1;
        const TileCoord tc = decode_tile(p, tile);
        unsigned char* slot_k = stage_base + stage * kStageBytes;
        unsigned char* slot_v = slot_k + kSlotBytes<E>;
        unsigned char* slot_g = slot_v + kSlotBytes<E>;
        const int c = tc.strip * kCs + lane;
        const float w = (c < p.C) ? p.w[c] : 0.f;
        const float u = (c < p.C) ? p.u[c] : 0.f;

        if (threadIdx.x == 0) {
            sm100::tma_store_wait_read();            // the other stage's outputs have left shared memory
            const int next = tile + gridDim.x;
            if (next < p.n_tiles) issue_loads(next, stage ^ 1);
        }
        if (!sm100::mbar_wait(&full[stage], (it >> 1) & 1, kSpinLimit)) atomicOr(p.status, 2u);
        const int t0 = tc.chunk * kTc + warp * kL;               // first token of this sub-chunk
        const int n = max(0, min(kL, p.T - t0));
        const Col<E> ks(slot_k, warp, lane), vs(slot_v, warp, lane), gs(slot_g, warp, lane);
        // where the scaled output gradient is parked between the two backward levels (fp32 either way)
        const Col<float> gpark((kBwd && kHalf) ? static_cast<void*>(gscratch) : static_cast<void*>(slot_g), warp, lane);
        float gw = 0.f, gu = 0.f;

        float kk[kL], vv[kL];
        float m = kMinExp, mn = 1e38f;
#pragma unroll
        for (int i = 0; i < kL; ++i) {
            kk[i] = ks.ld(i);
            vv[i] = vs.ld(i);
            if (i < n) { m = wkv_max(m, kk[i]); mn = fminf(mn, kk[i]); }
        }
        const bool safe = (n == 0) || ((m - mn) + fabsf(w) * kL + fabsf(u) <= kFastRange);
        if (!__all_sync(0xffffffffu, safe)) {
            const ExchangeCtx xc{sub, ext, lane, warp, tile, tc.chunk};
            rigorous_tile<kBwd, E>(p, xc, ks, vs, gs, n, w, u, gw, gu);
        } else {
            const float lam = fast_exp(-w);
            const float2 lam2 = f2(lam, lam);
            // ---- level 1: aggregates in scale e^{m} ----
            Acc4 own_right;
            Acc2 own_left;
            {
                float2 a = f2(0.f, 0.f), ma = f2(0.f, 0.f), a2 = f2(0.f, 0.f);
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    const float e = (i < n) ? fast_exp(kk[i] - m) : 0.f;
                    a = mul2(add2(a, f2(e * vv[i], e)), lam2);
                    if (kBwd) ma = fma2(ma, lam2, a);
                }
#pragma unroll
                for (int i = kL - 1; i >= 0; --i) {
                    const float e = (i < n) ? fast_exp(kk[i] - m) : 0.f;
                    a2 = mul2(add2(a2, f2(e * vv[i], e)), lam2);
                }
                own_right = Acc4{a.x, a.y, ma.x, ma.y, m};
                own_left = Acc2{a2.x, a2.y, m};
            }
            const Entering e1 = exchange(p, sub, ext, lane, warp, w, tile, tc.chunk, 0, kLevels, own_right, own_left);
            const Acc4 cp = e1.left;
            const Acc2 cs = e1.right;
            const float M = wkv_max(m, wkv_max(cp.o, cs.o));
            const float fp = fast_exp(cp.o - M), fs = fast_exp(cs.o - M);
            const float eu = fast_exp(u);
            float2 pr = f2(cp.a * fp, cp.b * fp);
            float2 sf = f2(cs.a * fs, cs.b * fs);
            float2 stash[kL];
#pragma unroll
            for (int i = kL - 1; i >= 0; --i) {
                stash[i] = sf;
                const float e = (i < n) ? fast_exp(kk[i] - M) : 0.f;
                sf = mul2(add2(sf, f2(e * vv[i], e)), lam2);
            }
            if (!kBwd) {
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    const float e = (i < n) ? fast_exp(kk[i] - M) : 0.f;
                    const float2 x = f2(e * vv[i], e);
                    const float2 nd = fma2(x, f2(eu, eu), add2(pr, stash[i]));
                    ks.st(i, __fdividef(nd.x, nd.y));
                    pr = mul2(add2(pr, x), lam2);
                }
            } else {
                // ---- level 1 emit: G' = gy/Den', H' = G' y (scale e^{-M}); gu; gw from pairs t > j ----
                float2 pm = f2(cp.ma * fp, cp.mb * fp);
                float hh[kL];
                float2 r = f2(0.f, 0.f), mr = f2(0.f, 0.f), q = f2(0.f, 0.f);
                float mu = lam;
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    const float e = (i < n) ? fast_exp(kk[i] - M) : 0.f;
                    const float2 x = f2(e * vv[i], e);
                    const float2 nd = fma2(x, f2(eu, eu), add2(pr, stash[i]));
                    const float inv = (i < n) ? __frcp_rn(nd.y) : 0.f;
                    const float y = nd.x * inv;
                    const float g = gs.ld(i) * inv;
                    const float h = g * y;
                    gpark.st(i, g);
                    hh[i] = h;
                    gu += eu * (x.x * g - x.y * h);
                    gw -= g * pm.x - h * pm.y;
                    pr = mul2(add2(pr, x), lam2);
                    pm = fma2(pm, lam2, pr);
                    const float2 gh = f2(g, h);
                    r = mul2(add2(r, gh), lam2);
                    mr = fma2(mr, lam2, r);
                    q = fma2(gh, f2(mu, mu), q);
                    mu *= lam;
                }
                const Entering e2 = exchange(p, sub, ext, lane, warp, w, tile, tc.chunk, 1, kLevels,
                                             Acc4{r.x, r.y, mr.x, mr.y, -M}, Acc2{q.x, q.y, -M});
                const Acc4 cr = e2.left;
                const Acc2 cq = e2.right;
                // adjoint values live in scale e^{N}; inputs re-enter as e^{k + N}
                const float N = wkv_max(-M, wkv_max(cr.o, cq.o));
                const float fl = fast_exp(-M - N), fr = fast_exp(cr.o - N), fq = fast_exp(cq.o - N);
                float2 qq = f2(cq.a * fq, cq.b * fq);
                float2 rr = f2(cr.a * fr, cr.b * fr);
                float2 mrr = f2(cr.ma * fr, cr.mb * fr);
                const float2 fl2 = f2(fl, fl);
                float2 part[kL];
#pragma unroll
                for (int i = kL - 1; i >= 0; --i) {
                    const float e = (i < n) ? fast_exp(kk[i] + N) : 0.f;
                    part[i] = f2(e * (qq.x * vv[i] - qq.y), e * qq.x);          // (gk, gv) from later outputs
                    qq = mul2(fma2(f2(gpark.ld(i), hh[i]), fl2, qq), lam2);
                }
                const float euf = eu * fl;
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    const float e = (i < n) ? fast_exp(kk[i] + N) : 0.f;
                    const float g = gpark.ld(i), h = hh[i];
                    const float ev = e * vv[i];
                    const float self = euf * (ev * g - e * h);
                    ks.st(i, part[i].x + (ev * rr.x - e * rr.y) + self);
                    vs.st(i, part[i].y + e * rr.x + euf * e * g);
                    gw -= ev * mrr.x - e * mrr.y;
                    rr = mul2(fma2(f2(g, h), fl2, rr), lam2);
                    mrr = fma2(mrr, lam2, rr);
                }
            }
        }
        if (kBwd) {
            red[(warp * 2 + 0) * kCs + lane] = gw;
            red[(warp * 2 + 1) * kCs + lane] = gu;
            __syncthreads();
            if (warp < 2) {
                float acc = 0.f;
#pragma unroll
                for (int s = 0; s < kWarps; ++s) acc += red[(s * 2 + warp) * kCs + lane];
                p.partial[(static_cast<size_t>(tile) * 2 + warp) * kCs + lane] = acc;
            }
        }
        sm100::fence_proxy_async_smem();
        __syncthreads();
        if (threadIdx.x == 0) {
            sm100::tma_store_3d(&map_o0, slot_k, tc.strip * kCs, tc.chunk * kTc, tc.b);
            if (kBwd) sm100::tma_store_3d(&map_o1, slot_v, tc.strip * kCs, tc.chunk * kTc, tc.b);
            sm100::tma_store_commit();
        }
    }
    if (threadIdx.x == 0) sm100::tma_store_wait_all();
}

// ---- forward, pipelined ---------------------------------------------------------------------------
// The forward needs one exchange level only, and its tile is small enough (32 KB) to keep three
// of them per CTA.  That allows the two halves of the exchange to be pulled apart in time: in
// iteration n a CTA first *publishes* tile n (aggregates, inside sums, tile record + flag), then
// *finishes* tile n-1 (collect the peers' records, emit y, store), and the third stage receives
// tile n+1 meanwhile.  The peers of tile n-1 published a whole iteration ago, so the collect step
// finds their flags set instead of waiting for the slowest of them.  Between the two halves a
// thread carries only its eight inside sums in registers.  Deadlock freedom is unchanged: a
// CTA publishes tile n before it may wait for anything belonging to tile n-1.
constexpr int kFwdStages = 3;

// per-token max-shifted path, split in the same two halves (forward only)
template <typename E>
__device__ __noinline__ void rigorous_aggregates(const Col<E> ks, const Col<E> vs, int n, float w, Acc4& right,
                                                 Acc2& left) {
    right = acc4_zero();
    left = acc2_zero();
    for (int i = 0; i < n; ++i) acc4_absorb(right, ks.ld(i) + w * static_cast<float>(i), vs.ld(i), 1.f);
    for (int i = n - 1; i >= 0; --i) acc2_add(left, ks.ld(i) - w * static_cast<float>(i), vs.ld(i), 1.f);
    right.o -= w * static_cast<float>(n);
    acc4_decay(right, w, static_cast<float>(kL - n));
    left.o -= w;
}
template <typename E, bool kSave>
__device__ __noinline__ void rigorous_emit_forward(const Col<E> ks, const Col<E> vs, int n, float w, float u,
                                                   const Entering& e) {
    const float last = static_cast<float>(n - 1);
    Acc2 S = e.right;
    acc2_decay(S, w, static_cast<float>(kL - n));
    Acc2 stash[kL];
    for (int i = n - 1; i >= 0; --i) {
        const float d = last - static_cast<float>(i);
        stash[i] = acc2_at(S, w, d);
        acc2_add(S, ks.ld(i) + w * d, vs.ld(i), 1.f);
    }
    Acc2 P{e.left.a, e.left.b, e.left.o};
    for (int i = 0; i < n; ++i) {
        const float k = ks.ld(i), v = vs.ld(i), d = static_cast<float>(i);
        const TokenOut o = token_out(acc2_at(P, w, d), stash[i], k, v, u);
        ks.st(i, o.y);
        if (kSave) vs.st(i, o.m - logf(o.inv_den));          // log Den_t
        acc2_add(P, k + w * d, v, 1.f);
    }
}

// kSave: also write log Den_t (one float per element, into the v slot and out through map_l) for
// the backward that starts from the saved y and log Den instead of recomputing them.
template <typename E, bool kSave>
__global__ void __launch_bounds__(kThreads, 2)
biwkv_forward_pipelined_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                               const __grid_constant__ CUtensorMap map_y, const __grid_constant__ CUtensorMap map_l,
                               const Params p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if (switched_off(p)) return;
    constexpr uint32_t kStageBytes = 2 * kSlotBytes<E>;
    unsigned char* stage_base = smem_raw;                                           // [3][2][kTc][kCs] of E
    float* sub = reinterpret_cast<float*>(stage_base + kFwdStages * kStageBytes);   // [kWarps][kRows][kCs]
    float* ext = sub + kWarps * kRecFloats;                                         // [kWarps][kRows][kCs]
    uint64_t* full = reinterpret_cast<uint64_t*>(ext + kWarps * kRecFloats);        // [3]
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kFwdStages; ++s) sm100::mbar_init(&full[s], 1);
        sm100::mbar_init_fence();
    }
    __syncthreads();

    const int G = static_cast<int>(gridDim.x);
    const int first = static_cast<int>(blockIdx.x);
    const int mine = first < p.n_tiles ? (p.n_tiles - first + G - 1) / G : 0;      // tiles of this CTA
    auto issue_loads = [&](int n) {
        const int stage = n % kFwdStages;
        const TileCoord tc = decode_tile(p, first + n * G);
        unsigned char* dst = stage_base + stage * kStageBytes;
        sm100::mbar_expect_tx(&full[stage], kStageBytes);
        sm100::tma_load_3d(dst, &map_k, &full[stage], tc.strip * kCs, tc.chunk * kTc, tc.b);
        sm100::tma_load_3d(dst + kSlotBytes<E>, &map_v, &full[stage], tc.strip * kCs, tc.chunk * kTc, tc.b);
    };
    if (threadIdx.x == 0)
        for (int n = 0; n < kFwdStages && n < mine; ++n) issue_loads(n);

    Inside prev_in{acc4_zero(), acc2_zero()};
    bool prev_safe = true;
    for (int n = 0; n <= mine; ++n) {
        Inside cur_in{acc4_zero(), acc2_zero()};
        bool cur_safe = true;
        if (n < mine) {
            // ---- publish tile n ----
            const int tile = first + n * G;
            const int stage = n % kFwdStages;
            const TileCoord tc = decode_tile(p, tile);
            const int c = tc.strip * kCs + lane;
            const float w = (c < p.C) ? p.w[c] : 0.f;
            const float u = (c < p.C) ? p.u[c] : 0.f;
            if (!sm100::mbar_wait(&full[stage], (n / kFwdStages) & 1, kSpinLimit)) atomicOr(p.status, 2u);
            const int nv = max(0, min(kL, p.T - (tc.chunk * kTc + warp * kL)));
            const Col<E> ks(stage_base + stage * kStageBytes, warp, lane);
            const Col<E> vs(stage_base + stage * kStageBytes + kSlotBytes<E>, warp, lane);
            float kk[kL], vv[kL];
            float m = kMinExp, mn = 1e38f;
#pragma unroll
            for (int i = 0; i < kL; ++i) {
                kk[i] = ks.ld(i);
                vv[i] = vs.ld(i);
                if (i < nv) { m = wkv_max(m, kk[i]); mn = fminf(mn, kk[i]); }
            }
            const bool safe = (nv == 0) || ((m - mn) + fabsf(w) * kL + fabsf(u) <= kFastRange);
            cur_safe = __all_sync(0xffffffffu, safe);
            Acc4 own_right;
            Acc2 own_left;
            if (!cur_safe) {
                rigorous_aggregates(ks, vs, nv, w, own_right, own_left);
            } else {
                const float lam = fast_exp(-w);
                const float2 lam2 = f2(lam, lam);
                float2 a = f2(0.f, 0.f), a2 = f2(0.f, 0.f);
                float mu = lam;
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    const float e = (i < nv) ? fast_exp(kk[i] - m) : 0.f;
                    const float2 x = f2(e * vv[i], e);
                    a = mul2(add2(a, x), lam2);                 // rightward: relative to the span's end
                    a2 = fma2(x, f2(mu, mu), a2);               // leftward: weight lambda^{i+1}
                    mu *= lam;
                }
                own_right = Acc4{a.x, a.y, 0.f, 0.f, m};
                own_left = Acc2{a2.x, a2.y, m};
            }
            cur_in = exchange_publish(p, sub, lane, warp, w, tile, 0, 1, own_right, own_left);
            // the stage that tile n-2 left gets tile n+1 (its store was issued an iteration ago)
            if (threadIdx.x == 0 && n >= 2 && n + 1 < mine) {
                sm100::tma_store_wait_read();
                issue_loads(n + 1);
            }
        }
        if (n >= 1) {
            // ---- finish tile n-1 ----
            const int tile = first + (n - 1) * G;
            const int stage = (n - 1) % kFwdStages;
            const TileCoord tc = decode_tile(p, tile);
            const int c = tc.strip * kCs + lane;
            const float w = (c < p.C) ? p.w[c] : 0.f;
            const float u = (c < p.C) ? p.u[c] : 0.f;
            const int nv = max(0, min(kL, p.T - (tc.chunk * kTc + warp * kL)));
            unsigned char* slot_k = stage_base + stage * kStageBytes;
            const Col<E> ks(slot_k, warp, lane), vs(slot_k + kSlotBytes<E>, warp, lane);
            const Entering e1 = exchange_collect(p, ext, lane, warp, w, tile, tc.chunk, 0, 1, prev_in);
            if (!prev_safe) {
                rigorous_emit_forward<E, kSave>(ks, vs, nv, w, u, e1);
            } else {
                float kk[kL], vv[kL];
                float m = kMinExp;
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    kk[i] = ks.ld(i);
                    vv[i] = vs.ld(i);
                    if (i < nv) m = wkv_max(m, kk[i]);
                }
                const float lam = fast_exp(-w);
                const float2 lam2 = f2(lam, lam);
                const Acc4 cp = e1.left;
                const Acc2 cs = e1.right;
                const float M = wkv_max(m, wkv_max(cp.o, cs.o));
                const float fp = fast_exp(cp.o - M), fs = fast_exp(cs.o - M);
                const float eu = fast_exp(u);
                float2 pr = f2(cp.a * fp, cp.b * fp);
                float2 sf = f2(cs.a * fs, cs.b * fs);
                float2 stash[kL];
#pragma unroll
                for (int i = kL - 1; i >= 0; --i) {
                    stash[i] = sf;
                    const float e = (i < nv) ? fast_exp(kk[i] - M) : 0.f;
                    kk[i] = e;                                   // reused by the emit sweep
                    sf = mul2(add2(sf, f2(e * vv[i], e)), lam2);
                }
#pragma unroll
                for (int i = 0; i < kL; ++i) {
                    const float2 x = f2(kk[i] * vv[i], kk[i]);
                    const float2 nd = fma2(x, f2(eu, eu), add2(pr, stash[i]));
                    ks.st(i, __fdividef(nd.x, nd.y));
                    if (kSave) vs.st(i, M + __logf(nd.y));   // log Den_t; v of this token is in a register
                    pr = mul2(add2(pr, x), lam2);
                }
            }
            sm100::fence_proxy_async_smem();
            __syncthreads();
            if (threadIdx.x == 0) {
                sm100::tma_store_3d(&map_y, slot_k, tc.strip * kCs, tc.chunk * kTc, tc.b);
                if (kSave) sm100::tma_store_3d(&map_l, slot_k + kSlotBytes<E>, tc.strip * kCs, tc.chunk * kTc, tc.b);
                sm100::tma_store_commit();
            }
        }
        prev_in = cur_in;
        prev_safe = cur_safe;
    }
    if (threadIdx.x == 0) sm100::tma_store_wait_all();
}

// ---- backward from the saved forward results ----------------------------------------------------
// When the forward has kept y and log Den (biwkv_forward_pipelined_kernel<float, true>), the
// backward does not need the first exchange level at all: G_t = gy_t / Den_t and H_t = G_t y_t are
// local.  What remains is one level for the adjoint pairs [G, H], with first moments in distance in
// *both* directions, because gw is then taken entirely from the adjoint side:
//   gw = - sum_j e^{k_j} ((MQ^G_j + MR^G_j) v_j - (MQ^H_j + MR^H_j)).
// Records therefore have ten rows (a, b, ma, mb, o for each direction).
constexpr int kRows2 = 10;
constexpr int kRecFloats2 = kRows2 * kCs;

__device__ __forceinline__ void post_left4(float* rec, const Acc4& s) {
    rec[5 * kCs] = s.a; rec[6 * kCs] = s.b; rec[7 * kCs] = s.ma; rec[8 * kCs] = s.mb; rec[9 * kCs] = s.o;
}
struct Entering4 {
    Acc4 left;    // adjoint state entering the sub-chunk at its first token (from earlier outputs)
    Acc4 right;   // ... at its last position (from later outputs)
};
struct Inside4 {
    Acc4 inP, inS;
};

__device__ __forceinline__ Inside4 exchange_publish4(const Params& p, float* sub, int lane, int warp, float w, int tile,
                                                     const Acc4& own_right, const Acc4& own_left) {
    post_acc4(sub + warp * kRecFloats2 + lane, own_right);
    post_left4(sub + warp * kRecFloats2 + lane, own_left);
    __syncthreads();
    Acc4 inP, inS;
    {
        float x4[kWarps], x2[kWarps];
        float m4 = kMinExp, m2 = kMinExp;
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            const float* r = sub + s * kRecFloats2 + lane;
            x4[s] = (s < warp) ? r[4 * kCs] - w * static_cast<float>((warp - 1 - s) * kL) : kMinExp;
            x2[s] = (s > warp) ? r[9 * kCs] - w * static_cast<float>((s - warp - 1) * kL) : kMinExp;
            m4 = wkv_max(m4, x4[s]);
            m2 = wkv_max(m2, x2[s]);
        }
        inP = Acc4{0.f, 0.f, 0.f, 0.f, m4};
        inS = Acc4{0.f, 0.f, 0.f, 0.f, m2};
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            const float* r = sub + s * kRecFloats2 + lane;
            if (s < warp) {
                const float f = fast_exp(x4[s] - m4);
                const float d = static_cast<float>((warp - 1 - s) * kL);
                const float a = r[0], b = r[kCs];
                inP.a += f * a;
                inP.b += f * b;
                inP.ma += f * (r[2 * kCs] + d * a);
                inP.mb += f * (r[3 * kCs] + d * b);
            }
            if (s > warp) {
                const float f = fast_exp(x2[s] - m2);
                const float d = static_cast<float>((s - warp - 1) * kL);
                const float a = r[5 * kCs], b = r[6 * kCs];
                inS.a += f * a;
                inS.b += f * b;
                inS.ma += f * (r[7 * kCs] + d * a);
                inS.mb += f * (r[8 * kCs] + d * b);
            }
        }
    }
    if (warp == kWarps - 1 || warp == 0) {
        float* mine = p.exch + static_cast<size_t>(tile) * kRecFloats2 + lane;
        if (warp == kWarps - 1) {
            Acc4 t = inP;
            acc4_decay(t, w, static_cast<float>(kL));
            post_acc4(mine, merge4(t, own_right));
        }
        if (warp == 0) {
            Acc4 t = inS;
            acc4_decay(t, w, static_cast<float>(kL));
            post_left4(mine, merge4(t, own_left));
        }
        __syncwarp();
        if (lane == 0) {
            __threadfence();
            atomicAdd(p.flags + tile, 1u);
        }
    }
    return Inside4{inP, inS};
}

__device__ __forceinline__ Entering4 exchange_collect4(const Params& p, float* ext, int lane, int warp, float w, int tile,
                                                       int chunk, const Inside4& in) {
    {
        const int first = tile - chunk * p.interleave;
        Acc4 P = acc4_zero(), S = acc4_zero();
        for (int j0 = warp; j0 < p.n_chunks; j0 += 4 * kWarps) {
            // flags polled four at a time with relaxed loads; the record loads take their address from the
            // polled values, which orders them after the flags (see exchange_collect)
            bool ok = true;
            const unsigned* fl[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                fl[q] = (j < p.n_chunks && j != chunk) ? p.flags + (first + j * p.interleave) : nullptr;
            }
            unsigned seen[4] = {0u, 0u, 0u, 0u};
            for (uint32_t spins = 0;; ++spins) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (seen[q] < 2u) seen[q] = fl[q] ? sm100::flag_relaxed(fl[q]) : 2u;
                if (seen[0] >= 2u && seen[1] >= 2u && seen[2] >= 2u && seen[3] >= 2u) break;
                if (spins > kSpinLimit ||
                    ((spins & 1023u) == 1023u && *reinterpret_cast<volatile unsigned*>(p.status) != 0u)) {
                    ok = false;
                    break;
                }
                __nanosleep(spins < 8 ? 32 : 128);
            }
            // the polls above are relaxed; one acquire load per flag, issued together, is what orders
            // the record loads below after the publishers' writes (the address dependency through
            // `dep` alone is not an ordering the PTX memory model gives)
            if (ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (fl[q]) seen[q] |= sm100::flag_acquire(fl[q]);
            }
            const unsigned seen_all = seen[0] | seen[1] | seen[2] | seen[3];
            const size_t dep = seen_all >> 31;
            if (!ok && lane == 0) atomicOr(p.status, 1u);
            float r0[4], r1[4], r2[4], r3[4], x[4];
            float mP = kMinExp, mS = kMinExp;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                r0[q] = r1[q] = r2[q] = r3[q] = 0.f;
                x[q] = kMinExp;
                if (j < p.n_chunks && j != chunk) {
                    const float* rec = p.exch + static_cast<size_t>(first + j * p.interleave) * kRecFloats2 + lane + dep +
                                       (j < chunk ? 0 : 5 * kCs);
                    r0[q] = sm100::ld_cg(rec); r1[q] = sm100::ld_cg(rec + kCs);
                    r2[q] = sm100::ld_cg(rec + 2 * kCs); r3[q] = sm100::ld_cg(rec + 3 * kCs);
                    x[q] = sm100::ld_cg(rec + 4 * kCs);
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                if (j < p.n_chunks && j != chunk) {
                    const float d = static_cast<float>((j < chunk ? chunk - 1 - j : j - chunk - 1) * kTc);
                    x[q] -= w * d;
                    r2[q] += d * r0[q];
                    r3[q] += d * r1[q];
                    if (j < chunk) mP = wkv_max(mP, x[q]);
                    else mS = wkv_max(mS, x[q]);
                }
            }
            Acc4 bp{0.f, 0.f, 0.f, 0.f, mP}, bs{0.f, 0.f, 0.f, 0.f, mS};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = j0 + q * kWarps;
                if (j < p.n_chunks && j != chunk) {
                    if (j < chunk) {
                        const float f = fast_exp(x[q] - mP);
                        bp.a += f * r0[q]; bp.b += f * r1[q]; bp.ma += f * r2[q]; bp.mb += f * r3[q];
                    } else {
                        const float f = fast_exp(x[q] - mS);
                        bs.a += f * r0[q]; bs.b += f * r1[q]; bs.ma += f * r2[q]; bs.mb += f * r3[q];
                    }
                }
            }
            P = merge4(P, bp);
            S = merge4(S, bs);
        }
        post_acc4(ext + warp * kRecFloats2 + lane, P);
        post_left4(ext + warp * kRecFloats2 + lane, S);
    }
    __syncthreads();
    Entering4 out;
    {
        float m4 = kMinExp, m2 = kMinExp;
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            m4 = wkv_max(m4, ext[s * kRecFloats2 + 4 * kCs + lane]);
            m2 = wkv_max(m2, ext[s * kRecFloats2 + 9 * kCs + lane]);
        }
        Acc4 P{0.f, 0.f, 0.f, 0.f, m4}, S{0.f, 0.f, 0.f, 0.f, m2};
#pragma unroll
        for (int s = 0; s < kWarps; ++s) {
            const float* r = ext + s * kRecFloats2 + lane;
            const float f4 = fast_exp(r[4 * kCs] - m4), f2_ = fast_exp(r[9 * kCs] - m2);
            P.a += f4 * r[0]; P.b += f4 * r[kCs]; P.ma += f4 * r[2 * kCs]; P.mb += f4 * r[3 * kCs];
            S.a += f2_ * r[5 * kCs]; S.b += f2_ * r[6 * kCs]; S.ma += f2_ * r[7 * kCs]; S.mb += f2_ * r[8 * kCs];
        }
        acc4_decay(P, w, static_cast<float>(warp * kL));
        acc4_decay(S, w, static_cast<float>((kWarps - 1 - warp) * kL));
        out.left = merge4(P, in.inP);
        out.right = merge4(S, in.inS);
    }
    return out;
}

// per-token max-shifted path of the saved-result backward (any exponent range)
__device__ __noinline__ void rigorous_tile_saved(const Params& p, float* sub, float* ext, int lane, int warp, int tile,
                                                 int chunk, const Col<float> ks, const Col<float> vs, const Col<float> gs,
                                                 const Col<float> ys, const Col<float> ls, int n, float w, float u,
                                                 float& gw_out, float& gu_out) {
    const float last = static_cast<float>(n - 1);
    float gg[kL], hh[kL], xo[kL];
    Acc4 later = acc4_zero(), earlier = acc4_zero();
    for (int i = 0; i < n; ++i) {
        gg[i] = gs.ld(i);
        hh[i] = gg[i] * ys.ld(i);
        xo[i] = -ls.ld(i);
    }
    for (int i = 0; i < n; ++i) acc4_absorb(later, xo[i] + w * static_cast<float>(i), gg[i], hh[i]);
    for (int i = n - 1; i >= 0; --i) acc4_absorb(earlier, xo[i] - w * static_cast<float>(i), gg[i], hh[i]);
    later.o -= w * static_cast<float>(n);
    acc4_decay(later, w, static_cast<float>(kL - n));
    earlier.o -= w;
    const Inside4 in = exchange_publish4(p, sub, lane, warp, w, tile, later, earlier);
    const Entering4 e = exchange_collect4(p, ext, lane, warp, w, tile, chunk, in);
    Acc4 R = e.left;                                 // anchored at token 0
    Acc4 Q = e.right;
    acc4_decay(Q, w, static_cast<float>(kL - n));   // anchored at token n-1
    float gw = 0.f, gu = 0.f;
    float pk[kL], pv[kL];
    for (int i = n - 1; i >= 0; --i) {
        const float d = last - static_cast<float>(i);
        const float k = ks.ld(i), v = vs.ld(i);
        const float ex = wkv_exp(k + Q.o - w * d);
        pv[i] = ex * Q.a;
        pk[i] = ex * (Q.a * v - Q.b);
        gw -= ex * (Q.ma * v - Q.mb);
        acc4_absorb(Q, xo[i] + w * d, gg[i], hh[i]);
    }
    for (int i = 0; i < n; ++i) {
        const float k = ks.ld(i), v = vs.ld(i), d = static_cast<float>(i);
        const float ex = wkv_exp(k + R.o - w * d);
        const float es = wkv_exp(u + k + xo[i]);
        const float self = es * (v * gg[i] - hh[i]);
        vs.st(i, pv[i] + ex * R.a + es * gg[i]);
        ks.st(i, pk[i] + ex * (R.a * v - R.b) + self);
        gu += self;
        gw -= ex * (R.ma * v - R.mb);
        acc4_absorb(R, xo[i] + w * d, gg[i], hh[i]);
    }
    gw_out = gw;
    gu_out = gu;
}

constexpr int kSavedSlots = 5;     // k, v, gy, y, log Den
__global__ void __launch_bounds__(kThreads, 2)
biwkv_backward_saved_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_y,
                            const __grid_constant__ CUtensorMap map_l, const __grid_constant__ CUtensorMap map_gk,
                            const __grid_constant__ CUtensorMap map_gv, const Params p) {
    constexpr uint32_t kSlot = kSlotBytes<float>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* slots = smem_raw;                                                // [5][kTc][kCs] floats, one stage
    float* sub = reinterpret_cast<float*>(slots + kSavedSlots * kSlot);            // [kWarps][kRows2][kCs]
    float* ext = sub + kWarps * kRecFloats2;
    float* red = sub;
    uint64_t* full = reinterpret_cast<uint64_t*>(ext + kWarps * kRecFloats2);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        sm100::mbar_init(full, 1);
        sm100::mbar_init_fence();
    }
    __syncthreads();
    auto issue_loads = [&](int tile) {
        const TileCoord tc = decode_tile(p, tile);
        const int x = tc.strip * kCs, y = tc.chunk * kTc;
        sm100::mbar_expect_tx(full, kSavedSlots * kSlot);
        sm100::tma_load_3d(slots + 0 * kSlot, &map_k, full, x, y, tc.b);
        sm100::tma_load_3d(slots + 1 * kSlot, &map_v, full, x, y, tc.b);
        sm100::tma_load_3d(slots + 2 * kSlot, &map_g, full, x, y, tc.b);
        sm100::tma_load_3d(slots + 3 * kSlot, &map_y, full, x, y, tc.b);
        sm100::tma_load_3d(slots + 4 * kSlot, &map_l, full, x, y, tc.b);
    };
    if (threadIdx.x == 0 && static_cast<int>(blockIdx.x) < p.n_tiles) issue_loads(blockIdx.x);

    int it = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
        const TileCoord tc = decode_tile(p, tile);
        const int c = tc.strip * kCs + lane;
        const float w = (c < p.C) ? p.w[c] : 0.f;
        const float u = (c < p.C) ? p.u[c] : 0.f;
        if (!sm100::mbar_wait(full, it & 1, kSpinLimit)) atomicOr(p.status, 2u);
        const int t0 = tc.chunk * kTc + warp * kL;
        const int n = max(0, min(kL, p.T - t0));
        const Col<float> ks(slots, warp, lane), vs(slots + kSlot, warp, lane), gs(slots + 2 * kSlot, warp, lane);
        const Col<float> ys(slots + 3 * kSlot, warp, lane), ls(slots + 4 * kSlot, warp, lane);
        float gw = 0.f, gu = 0.f;

        float kk[kL], vv[kL];
        float mk = kMinExp, mnk = 1e38f, X = kMinExp, mnx = 1e38f;
#pragma unroll
        for (int i = 0; i < kL; ++i) {
            kk[i] = ks.ld(i);
            vv[i] = vs.ld(i);
            const float xl = -ls.ld(i);
            if (i < n) {
                mk = wkv_max(mk, kk[i]); mnk = fminf(mnk, kk[i]);
                X = wkv_max(X, xl); mnx = fminf(mnx, xl);
            }
        }
        const bool safe = (n == 0) || ((mk - mnk) + (X - mnx) + fabsf(w) * kL + fabsf(u) <= kFastRange);
        if (!__all_sync(0xffffffffu, safe)) {
            rigorous_tile_saved(p, sub, ext, lane, warp, tile, tc.chunk, ks, vs, gs, ys, ls, n, w, u, gw, gu);
        } else {
            const float lam = fast_exp(-w);
            const float2 lam2 = f2(lam, lam);
            const float eu = fast_exp(u);
            // ---- G' = gy e^{-log Den - X}, H' = G' y (scale e^{X}); aggregates with first moments both ways ----
            float hh[kL];
            float2 r = f2(0.f, 0.f), mr = f2(0.f, 0.f), q = f2(0.f, 0.f), mq = f2(0.f, 0.f);
            float mu = lam;
#pragma unroll
            for (int i = 0; i < kL; ++i) {
                const float g = (i < n) ? gs.ld(i) * fast_exp(-ls.ld(i) - X) : 0.f;
                const float h = g * ys.ld(i);
                gs.st(i, g);
                hh[i] = (i < n) ? h : 0.f;
                const float2 gh = f2(g, hh[i]);
                r = mul2(add2(r, gh), lam2);
                mr = fma2(mr, lam2, r);
                q = fma2(gh, f2(mu, mu), q);
                const float mw = mu * static_cast<float>(i + 1);
                mq = fma2(gh, f2(mw, mw), mq);
                mu *= lam;
            }
            const Inside4 in = exchange_publish4(p, sub, lane, warp, w, tile, Acc4{r.x, r.y, mr.x, mr.y, X},
                                                 Acc4{q.x, q.y, mq.x, mq.y, X});
            const Entering4 e = exchange_collect4(p, ext, lane, warp, w, tile, tc.chunk, in);
            const Acc4 cr = e.left, cq = e.right;
            // adjoint values live in scale e^{N}; inputs re-enter as e^{k + N}
            const float N = wkv_max(X, wkv_max(cr.o, cq.o));
            const float fl = fast_exp(X - N), fr = fast_exp(cr.o - N), fq = fast_exp(cq.o - N);
            float2 qq = f2(cq.a * fq, cq.b * fq), mqq = f2(cq.ma * fq, cq.mb * fq);
            float2 rr = f2(cr.a * fr, cr.b * fr), mrr = f2(cr.ma * fr, cr.mb * fr);
            const float2 fl2 = f2(fl, fl);
            float2 part[kL];
#pragma unroll
            for (int i = kL - 1; i >= 0; --i) {
                const float ex = (i < n) ? fast_exp(kk[i] + N) : 0.f;
                part[i] = f2(ex * (qq.x * vv[i] - qq.y), ex * qq.x);          // (gk, gv) from later outputs
                gw -= ex * (mqq.x * vv[i] - mqq.y);
                qq = mul2(fma2(f2(gs.ld(i), hh[i]), fl2, qq), lam2);
                mqq = fma2(mqq, lam2, qq);
            }
            const float euf = eu * fl;
#pragma unroll
            for (int i = 0; i < kL; ++i) {
                const float ex = (i < n) ? fast_exp(kk[i] + N) : 0.f;
                const float g = gs.ld(i), h = hh[i];
                const float ev = ex * vv[i];
                const float self = euf * (ev * g - ex * h);
                ks.st(i, part[i].x + (ev * rr.x - ex * rr.y) + self);
                vs.st(i, part[i].y + ex * rr.x + euf * ex * g);
                gu += self;
                gw -= ev * mrr.x - ex * mrr.y;
                rr = mul2(fma2(f2(g, h), fl2, rr), lam2);
                mrr = fma2(mrr, lam2, rr);
            }
        }
        red[(warp * 2 + 0) * kCs + lane] = gw;
        red[(warp * 2 + 1) * kCs + lane] = gu;
        __syncthreads();
        if (warp < 2) {
            float acc = 0.f;
#pragma unroll
            for (int s = 0; s < kWarps; ++s) acc += red[(s * 2 + warp) * kCs + lane];
            p.partial[(static_cast<size_t>(tile) * 2 + warp) * kCs + lane] = acc;
        }
        sm100::fence_proxy_async_smem();
        __syncthreads();
        if (threadIdx.x == 0) {
            sm100::tma_store_3d(&map_gk, slots, tc.strip * kCs, tc.chunk * kTc, tc.b);
            sm100::tma_store_3d(&map_gv, slots + kSlot, tc.strip * kCs, tc.chunk * kTc, tc.b);
            sm100::tma_store_commit();
            const int next = tile + gridDim.x;
            if (next < p.n_tiles) {
                sm100::tma_store_wait_read();        // one stage: the outputs must have left before the next tile lands
                issue_loads(next);
            }
        }
    }
    if (threadIdx.x == 0) sm100::tma_store_wait_all();
}

// out[j][c] = sum over the tiles of channel c's strip of partial[tile][j][c % 32]
__global__ void __launch_bounds__(1024)
reduce_tile_partials(Params p, float* __restrict__ out) {
    __shared__ float red[32][33];
    const int strip = blockIdx.x, j = blockIdx.y, lane = threadIdx.x;
    const int c = strip * kCs + lane;
    if (switched_off(p)) return;
    const int rows = p.B * p.n_chunks;
    float acc = 0.f;
    for (int r = threadIdx.y; r < rows; r += 32) {
        const int b = r / p.n_chunks, chunk = r - b * p.n_chunks;
        const int gs = b * p.n_strips + strip;
        const int block = gs / p.interleave, si = gs - block * p.interleave;
        const int tile = block * p.interleave * p.n_chunks + chunk * p.interleave + si;
        acc += p.partial[(static_cast<size_t>(tile) * 2 + j) * kCs + lane];
    }
    red[threadIdx.y][lane] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < p.C) {
        float total = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) total += red[r][lane];
        out[static_cast<size_t>(j) * p.C + c] = total;
    }
}

// ---- host side ----------------------------------------------------------------------------------
template <typename E>
static bool make_map(CUtensorMap* map, const void* base, int B, int T, int C) {
    return tensor_map::make_btc(map, base, B, T, C, kCs, kTc, !std::is_same<E, float>::value);
}

template <typename E>
static constexpr size_t fwd_pipelined_smem_bytes() {
    return kFwdStages * 2 * kSlotBytes<E> + 2 * kWarps * kRecFloats * sizeof(float) + 64;
}

template <bool kBwd, typename E>
static constexpr size_t smem_bytes() {
    return 2 * (kBwd ? 3 : 2) * kSlotBytes<E> + ((kBwd && !std::is_same<E, float>::value) ? kSlotFloats * sizeof(float) : 0) +
           2 * kWarps * kRecFloats * sizeof(float) + 64;
}

struct DeviceInfo {
    int sms = 0;
    int resident[2][2] = {{0, 0}, {0, 0}};   // CTAs per SM: [float | bfloat16 tiles][forward | backward]
    bool ok = false;
};

template <typename E>
static bool configure_kernels(int (&resident)[2]) {
    bool good = cudaFuncSetAttribute(biwkv_fused_kernel<true, E>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem_bytes<true, E>())) == cudaSuccess;
    good = good && cudaFuncSetAttribute(biwkv_forward_pipelined_kernel<E, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(fwd_pipelined_smem_bytes<E>())) == cudaSuccess;
    good = good && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident[0], biwkv_forward_pipelined_kernel<E, false>,
                                                                 kThreads, fwd_pipelined_smem_bytes<E>()) == cudaSuccess;
    good = good && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident[1], biwkv_fused_kernel<true, E>, kThreads,
                                                                 smem_bytes<true, E>()) == cudaSuccess;
    return good && resident[0] > 0 && resident[1] > 0;
}

static std::mutex g_config_lock;

static const DeviceInfo& device_info() {
    static DeviceInfo infos[64];
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> guard(g_config_lock);
    DeviceInfo& d = infos[dev & 63];
    if (d.ok) return d;
    cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    bool good = tensor_map::encode_fn() != nullptr;
    good = good && configure_kernels<float>(d.resident[0]) && configure_kernels<__nv_bfloat16>(d.resident[1]);
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    d.ok = good && coop && d.sms > 0;
    if (!d.ok) cudaGetLastError();
    return d;
}

// Strips whose tiles alternate in the id order.  Measured on B200 (B=64, T=4096, C=768):
// 1 -> 1.21 / 2.74 ms (forward / backward), 2 -> 1.43 / 3.28, 4 -> 1.39 / 3.29, 8 -> 1.58 / 3.45:
// keeping the peers of a tile on adjacent CTAs matters more than sharing DRAM pages.
static int pick_interleave(int /*n_strips*/) { return 1; }

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct Layout {
    Params p;
    size_t off_status, off_flags, off_exch, off_partial, total;
};

static Layout make_layout(int B, int T, int C, bool bwd) {
    Layout l{};
    Params& p = l.p;
    p.B = B; p.T = T; p.C = C;
    p.n_chunks = (T + kTc - 1) / kTc;
    p.n_strips = (C + kCs - 1) / kCs;
    p.interleave = pick_interleave(p.n_strips);
    p.n_tiles = B * p.n_strips * p.n_chunks;
    p.by_span = make_fastdiv(static_cast<uint32_t>(p.interleave * p.n_chunks));
    p.by_interleave = make_fastdiv(static_cast<uint32_t>(p.interleave));
    p.by_strips = make_fastdiv(static_cast<uint32_t>(p.n_strips));
    const int levels = bwd ? 2 : 1;
    l.off_status = 0;
    l.off_flags = 256;
    l.off_exch = align_up(l.off_flags + static_cast<size_t>(p.n_tiles) * levels * 4, 256);
    l.off_partial = align_up(l.off_exch + static_cast<size_t>(p.n_tiles) * levels * kRows * kCs * 4, 256);
    l.total = l.off_partial + (bwd ? static_cast<size_t>(p.n_tiles) * 2 * kCs * 4 : 0);
    return l;
}

bool eligible(int B, int T, int C, std::initializer_list<const void*> ptrs, bool bf16) {
    if (C % (bf16 ? 8 : 4) != 0) return false;                     // TMA row pitch must be 16-byte
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) & 15u) return false;    // TMA base alignment
    const DeviceInfo& d = device_info();
    if (!d.ok) return false;
    const long long tiles = static_cast<long long>(B) * ((C + kCs - 1) / kCs) * ((T + kTc - 1) / kTc);
    if (tiles > (1LL << 30)) return false;
    // every peer of a tile must be reachable inside one sweep of the resident grid
    const int n_chunks = (T + kTc - 1) / kTc;
    const int (&res)[2] = d.resident[bf16 ? 1 : 0];
    const int grid = d.sms * std::min(res[0], res[1]);
    return static_cast<long long>(n_chunks) * pick_interleave((C + kCs - 1) / kCs) < grid;
}

size_t workspace_bytes(int B, int T, int C, bool bwd) { return make_layout(B, T, C, bwd).total; }

template <bool kBwd, typename E>
static int launch(Layout& l, const float* w, const float* u, const E* k, const E* v, const E* gy, E* o0, E* o1,
                  float* gwgu, void* workspace, cudaStream_t stream, const unsigned* run_if = nullptr) {
    Params& p = l.p;
    p.run_if = run_if;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    p.w = w; p.u = u;
    p.status = reinterpret_cast<unsigned*>(ws + l.off_status);
    p.flags = reinterpret_cast<unsigned*>(ws + l.off_flags);
    p.exch = reinterpret_cast<float*>(ws + l.off_exch);
    p.partial = reinterpret_cast<float*>(ws + l.off_partial);
    tensor_map::bind_primary_context();   // the tensor-map encoder is a driver call
    CUtensorMap mk, mv, mg, m0, m1;
    bool ok = make_map<E>(&mk, k, p.B, p.T, p.C) && make_map<E>(&mv, v, p.B, p.T, p.C) &&
              make_map<E>(&m0, o0, p.B, p.T, p.C);
    ok = ok && make_map<E>(&mg, kBwd ? gy : k, p.B, p.T, p.C) &&
         make_map<E>(&m1, (kBwd || o1 != nullptr) ? o1 : o0, p.B, p.T, p.C);
    if (!ok) {
        set_error_detail("cuTensorMapEncodeTiled rejected a (C, T, B) tensor map");
        return -1;
    }
    // status word + flags start at zero
    cudaMemsetAsync(ws, 0, l.off_exch, stream);
    const DeviceInfo& d = device_info();
    const int grid = std::min(p.n_tiles, d.sms * d.resident[std::is_same<E, float>::value ? 0 : 1][kBwd ? 1 : 0]);
    void* args[] = {&mk, &mv, &mg, &m0, &m1, &p};
    void* fwd_args[] = {&mk, &mv, &m0, &m1, &p};
    void* fwd_kernel = reinterpret_cast<void*>(biwkv_forward_pipelined_kernel<E, false>);
    if constexpr (std::is_same<E, float>::value) {
        if (!kBwd && o1 != nullptr) {                 // forward that also writes log Den into o1
            // the attribute is per device: one flag per device, under the lock of device_info()
            static bool configured[64] = {};
            int dev = 0;
            cudaGetDevice(&dev);
            std::lock_guard<std::mutex> guard(g_config_lock);
            if (!configured[dev & 63]) {
                cudaFuncSetAttribute(biwkv_forward_pipelined_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(fwd_pipelined_smem_bytes<float>()));
                configured[dev & 63] = true;
            }
            fwd_kernel = reinterpret_cast<void*>(biwkv_forward_pipelined_kernel<float, true>);
        }
    }
    const cudaError_t err =
        kBwd ? cudaLaunchCooperativeKernel(reinterpret_cast<void*>(biwkv_fused_kernel<true, E>), dim3(grid),
                                           dim3(kThreads), args, smem_bytes<true, E>(), stream)
             : cudaLaunchCooperativeKernel(fwd_kernel, dim3(grid), dim3(kThreads), fwd_args,
                                           fwd_pipelined_smem_bytes<E>(), stream);
    if (err != cudaSuccess) {
        set_error_detail(cudaGetErrorName(err));
        return -1;
    }
    int launched = 1;
    if (kBwd) {
        reduce_tile_partials<<<dim3(p.n_strips, 2), dim3(32, 32), 0, stream>>>(p, gwgu);
        ++launched;
    }
    return launched;
}

int forward(int B, int T, int C, const float* w, const float* u, const float* k, const float* v, float* y,
            void* workspace, cudaStream_t stream, const unsigned* run_if) {
    Layout l = make_layout(B, T, C, false);
    return launch<false, float>(l, w, u, k, v, nullptr, y, nullptr, nullptr, workspace, stream, run_if);
}

int backward(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
             const float* gy, float* gwgu, float* gk, float* gv, void* workspace, cudaStream_t stream,
             const unsigned* run_if) {
    Layout l = make_layout(B, T, C, true);
    return launch<true, float>(l, w, u, k, v, gy, gk, gv, gwgu, workspace, stream, run_if);
}

static constexpr size_t saved_smem_bytes() {
    return kSavedSlots * kSlotBytes<float> + 2 * kWarps * kRecFloats2 * sizeof(float) + 64;
}

// CTAs of the saved-result backward that fit one SM (0: the kernel cannot run here)
static int saved_resident() {
    static int cached[64];
    static bool known[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev &= 63;
    std::lock_guard<std::mutex> guard(g_config_lock);
    if (!known[dev]) {
        int n = 0;
        if (cudaFuncSetAttribute(biwkv_backward_saved_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(saved_smem_bytes())) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, biwkv_backward_saved_kernel, kThreads,
                                                          saved_smem_bytes()) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        cached[dev] = n;
        known[dev] = true;
    }
    return cached[dev];
}

bool eligible_saved(int B, int T, int C, std::initializer_list<const void*> ptrs) {
    if (!eligible(B, T, C, ptrs, false)) return false;
    const int res = saved_resident();
    if (res <= 0) return false;
    const int n_chunks = (T + kTc - 1) / kTc;
    return static_cast<long long>(n_chunks) * pick_interleave((C + kCs - 1) / kCs) < static_cast<long long>(device_info().sms) * res;
}

int backward_saved(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
                   const float* gy, const float* y, const float* logden, float* gwgu, float* gk, float* gv,
                   void* workspace, cudaStream_t stream) {
    Layout l = make_layout(B, T, C, true);       // sized for two 8-row levels: more than one 10-row level needs
    Params& p = l.p;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    p.w = w; p.u = u;
    p.status = reinterpret_cast<unsigned*>(ws + l.off_status);
    p.flags = reinterpret_cast<unsigned*>(ws + l.off_flags);
    p.exch = reinterpret_cast<float*>(ws + l.off_exch);
    p.partial = reinterpret_cast<float*>(ws + l.off_partial);
    tensor_map::bind_primary_context();   // the tensor-map encoder is a driver call
    CUtensorMap mk, mv, mg, my, ml, m0, m1;
    const bool ok = make_map<float>(&mk, k, B, T, C) && make_map<float>(&mv, v, B, T, C) && make_map<float>(&mg, gy, B, T, C) &&
                    make_map<float>(&my, y, B, T, C) && make_map<float>(&ml, logden, B, T, C) &&
                    make_map<float>(&m0, gk, B, T, C) && make_map<float>(&m1, gv, B, T, C);
    if (!ok) {
        set_error_detail("cuTensorMapEncodeTiled rejected a (C, T, B) tensor map");
        return -1;
    }
    cudaMemsetAsync(ws, 0, l.off_exch, stream);
    const int grid = std::min(p.n_tiles, device_info().sms * saved_resident());
    void* args[] = {&mk, &mv, &mg, &my, &ml, &m0, &m1, &p};
    const cudaError_t err = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(biwkv_backward_saved_kernel), dim3(grid),
                                                        dim3(kThreads), args, saved_smem_bytes(), stream);
    if (err != cudaSuccess) {
        set_error_detail(cudaGetErrorName(err));
        return -1;
    }
    reduce_tile_partials<<<dim3(p.n_strips, 2), dim3(32, 32), 0, stream>>>(p, gwgu);
    return 2;
}

int forward_save(int B, int T, int C, const float* w, const float* u, const float* k, const float* v, float* y,
                 float* logden, void* workspace, cudaStream_t stream) {
    Layout l = make_layout(B, T, C, false);
    return launch<false, float>(l, w, u, k, v, nullptr, y, logden, nullptr, workspace, stream);
}

int forward_bf16(int B, int T, int C, const float* w, const float* u, const void* k, const void* v, void* y,
                 void* workspace, cudaStream_t stream, const unsigned* run_if) {
    using E = __nv_bfloat16;
    Layout l = make_layout(B, T, C, false);
    return launch<false, E>(l, w, u, static_cast<const E*>(k), static_cast<const E*>(v), nullptr, static_cast<E*>(y),
                            nullptr, nullptr, workspace, stream, run_if);
}

int backward_bf16(int B, int T, int C, const float* w, const float* u, const void* k, const void* v, const void* gy,
                  float* gwgu, void* gk, void* gv, void* workspace, cudaStream_t stream, const unsigned* run_if) {
    using E = __nv_bfloat16;
    Layout l = make_layout(B, T, C, true);
    return launch<true, E>(l, w, u, static_cast<const E*>(k), static_cast<const E*>(v), static_cast<const E*>(gy),
                           static_cast<E*>(gk), static_cast<E*>(gv), gwgu, workspace, stream, run_if);
}

}  // namespace fused
}  // namespace biwkv

