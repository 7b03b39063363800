// WKV6 forward on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 operands, fp32 state.
//
// Per (batch, head) the 64 x 64 state S[key][value] lives in tensor memory as its transpose
// (TMEM lane = value channel, column = key channel, fp32).  The sequence is walked 16 tokens
// at a time; for every 16-token block, with a_t = sum of log-decays of the block's tokens
// before t and A = a_16, all matrix work runs as UMMA instructions (M = 128, fp32 accumulate):
//
//   P (16 x 16)    = Rs (16 x 64) . Kb^T        Rs[t][i] = r_t[i] e^{a_t[i]},  Kb[s][i] = k_s[i] e^{-a_{s+1}[i]}
//                    masked to s < t, the diagonal replaced by the bonus  sum_i r_t[i] u[i] k_t[i]
//   y^T (64 x 16)  = S^T (64 x 64, bf16 copy) . Rs^T  +  V^T (64 x 16) . P^T
//   S^T (64 x 64) += V^T (64 x 16) . Ks         Ks[t][i] = k_t[i] e^{A[i] - a_{t+1}[i]}
//                    after S^T was scaled by e^{A[i]} per key column on its way through registers
//
// The rows of Rs also sit in rows 64..79 of the state operand, so the score product is the same
// instruction shape as the read-out and lands in TMEM lanes 64..79, which an otherwise idle warp
// owns.  e^{-a_{s+1}} grows with the decay; a block whose accumulated log-decay exceeds 80 in any
// channel evaluates its 16 x 16 scores pairwise on the CUDA cores instead (every exponent <= 0
// there), so nothing overflows however strong the decay is.  The leftward direction is the same
// walk over the reversed sequence without the bonus; one CTA runs both and adds the second into
// the first.  The state never leaves the SM: per block it makes one round trip TMEM -> registers
// -> TMEM (decay) and leaves a bf16 copy in shared memory as the next A operand.
//
// Data movement: r, k, v, w tiles (16 tokens x 64 channels) arrive by TMA, the next block's while
// the current one is on the tensor core; y tiles leave by TMA store (rightward) and TMA reduce-add
// (leftward).  All bf16 operand writes are 16-byte shared stores (2-byte shared stores measured
// two orders of magnitude slower here), which fixes the thread-to-element maps of the operand phase.
//
// Accuracy is that of bf16 operands with fp32 accumulation (about 1e-2 of max|y|); the exact fp32
// sweeps of wkv6_sweeps.cu remain the default for float32 callers.
//
// Reference being replaced: classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu:6-97.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "sm100_async.cuh"
#include "tensor_map.h"
#include "vrwkv_internal.h"

namespace wkv6tc {

constexpr int N = 64;            // head size
constexpr int SC = 16;           // tokens per block
constexpr int kThreads = 128;
constexpr int kIssuer = 96;      // the thread that issues the tensor-core instructions (warp 3)
constexpr uint32_t kWaitLimit = 1u << 20;
constexpr uint32_t kTmemCols = 128;   // S^T: columns 0..63, y^T: 64..79, P^T: 80..95
constexpr float kMaxLogDecay = 80.f;  // per block and channel, for the tensor-core score product

struct Args {
    int B, T, H;
    const float* r;
    const float* k;
    const float* v;
    const float* w;      // raw decay input
    const float* u;      // (H, 64)
    float* y;
    unsigned* status;    // set to 1 if a bounded wait ran out
};

struct __align__(1024) Smem {
    __nv_bfloat16 opS[128 * 64];      // A: rows 0..63 = S^T (value x key), rows 64..79 = Rs (token x key)
    __nv_bfloat16 opV[128 * 16];      // A of the update and of the in-block part: V^T, rows = value, K = token
    __nv_bfloat16 opR[16 * 64];       // B of the read-out and of the scores: rows = token, K = key
    __nv_bfloat16 opK[64 * 16];       // B of the update: rows = key, K = token
    __nv_bfloat16 opP[16 * 16];       // B of the in-block part: rows = token t, K = token s
    __nv_bfloat16 opKb[16 * 64];      // B of the scores: rows = token s, K = key
    float raw[4][SC][N];              // r, k, v, w of the block as the copy engine delivers them (memory order)
    float ytile[SC][N];               // this block's output on its way to global memory (memory order)
    float acum[SC + 1][N];            // running log-decay sums: rows 0..8 from the block start, rows 9..16 from token 8
    float diag[SC];                   // bonus terms  sum_i r_t[i] u[i] k_t[i]
    float dtot[N];
    float u[N];
    uint64_t bar_main;
    uint64_t bar_score;
    uint64_t bar_load;
    uint32_t tmem_base;
};

using sm100::smem_u32;


// canonical K-major, no swizzle: element (row, k) of a [rows x K] bf16 operand
__device__ __forceinline__ int op_index(int rows, int row, int k) { return (k >> 3) * (rows * 8) + row * 8 + (k & 7); }

__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;        // descriptor version of this architecture
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ constexpr uint32_t instr_desc(int m, int n) {
    // fp32 accumulator, bf16 A and B, both K-major
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&x)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]), "=r"(x[8]),
          "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// y tile += shared tile (fp32), through the copy engine
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::
                     "l"(reinterpret_cast<uint64_t>(map)),
                 "r"(smem_u32(src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

__global__ void __launch_bounds__(kThreads, 4)
wkv6_tc_forward_kernel(const Args a, const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_w,
                       const __grid_constant__ CUtensorMap map_y) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int T = a.T, C = a.H * N;
    const size_t base = static_cast<size_t>(b) * T * C + static_cast<size_t>(h) * N;
    const int n_blocks = (T + SC - 1) / SC;
    const int n_steps = 2 * n_blocks;

    // first token (memory order) of the 16-row tile that holds block `step`; negative for a ragged last leftward block
    auto tile_start = [&](int step) { return step < n_blocks ? step * SC : T - SC * (step - n_blocks + 1); };
    auto issue_loads = [&](int step) {
        const int y0 = tile_start(step);
        sm100::mbar_expect_tx(&s.bar_load, 4 * SC * N * sizeof(float));
        sm100::tma_load_3d(&s.raw[0][0][0], &map_r, &s.bar_load, h * N, y0, b);
        sm100::tma_load_3d(&s.raw[1][0][0], &map_k, &s.bar_load, h * N, y0, b);
        sm100::tma_load_3d(&s.raw[2][0][0], &map_v, &s.bar_load, h * N, y0, b);
        sm100::tma_load_3d(&s.raw[3][0][0], &map_w, &s.bar_load, h * N, y0, b);
    };

    if (tid == kIssuer) {
        sm100::mbar_init(&s.bar_main, 1);
        sm100::mbar_init(&s.bar_score, 1);
        sm100::mbar_init(&s.bar_load, 1);
        sm100::mbar_init_fence();
        issue_loads(0);
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                     "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid < N) s.u[tid] = a.u[h * N + tid];
    // rows of the A operands that carry no data are still read by the tensor core: keep them finite
    for (int i = tid; i < 128 * 64; i += kThreads) s.opS[i] = __float2bfloat16(0.f);
    for (int i = tid; i < 128 * 16; i += kThreads) s.opV[i] = __float2bfloat16(0.f);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's 32 TMEM lanes

    uint32_t phase_main = 0, phase_score = 0, phase_load = 0;
    bool failed = false;
    auto wait_on = [&](uint64_t* bar, uint32_t parity) {
        if (!failed && !sm100::mbar_wait(bar, parity, kWaitLimit)) { failed = true; atomicExch(a.status, 1u); }
    };

    for (int step = 0; step < n_steps; ++step) {
        const bool rightward = step < n_blocks;
        const int blk = rightward ? step : step - n_blocks;
        auto row_of = [&](int t) { return rightward ? t : SC - 1 - t; };   // block order -> tile row

        wait_on(&s.bar_load, phase_load);
        phase_load ^= 1u;
        if (tid == 0) sm100::tma_store_wait_read();        // the previous y tile has left shared memory

        // ---- phase A: log-decays and their running sums; thread = (key channel, half of the block) ----
        {
            const int c = tid & 63, half = tid >> 6;
            float wv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = s.raw[3][row_of(half * 8 + j)][c];    // all loads before the first store
            float run = 0.f;
            if (half == 0) s.acum[0][c] = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = half * 8 + j;
                run += (blk * SC + t < T) ? -__expf(wv[j]) : 0.f;
                s.acum[t + 1][c] = run;
            }
        }
        __syncthreads();
        // a_t[c] = acum[t][c] (+ acum[8][c] for t > 8);  A[c] = a_16[c]
        // ---- phase B, job 1: thread = (token t, 8 key channels): Rs (twice), Kb, bonus; 16-byte stores only ----
        {
            const int t = tid >> 3, c0 = (tid & 7) * 8, row = row_of(t);
            float rv[8], kv[8], at[8], at1[8], a8[8], a16[8];
            *reinterpret_cast<float4*>(&rv[0]) = *reinterpret_cast<const float4*>(&s.raw[0][row][c0]);
            *reinterpret_cast<float4*>(&rv[4]) = *reinterpret_cast<const float4*>(&s.raw[0][row][c0 + 4]);
            *reinterpret_cast<float4*>(&kv[0]) = *reinterpret_cast<const float4*>(&s.raw[1][row][c0]);
            *reinterpret_cast<float4*>(&kv[4]) = *reinterpret_cast<const float4*>(&s.raw[1][row][c0 + 4]);
            *reinterpret_cast<float4*>(&at[0]) = *reinterpret_cast<const float4*>(&s.acum[t][c0]);
            *reinterpret_cast<float4*>(&at[4]) = *reinterpret_cast<const float4*>(&s.acum[t][c0 + 4]);
            *reinterpret_cast<float4*>(&at1[0]) = *reinterpret_cast<const float4*>(&s.acum[t + 1][c0]);
            *reinterpret_cast<float4*>(&at1[4]) = *reinterpret_cast<const float4*>(&s.acum[t + 1][c0 + 4]);
            *reinterpret_cast<float4*>(&a8[0]) = *reinterpret_cast<const float4*>(&s.acum[8][c0]);
            *reinterpret_cast<float4*>(&a8[4]) = *reinterpret_cast<const float4*>(&s.acum[8][c0 + 4]);
            *reinterpret_cast<float4*>(&a16[0]) = *reinterpret_cast<const float4*>(&s.acum[16][c0]);
            *reinterpret_cast<float4*>(&a16[4]) = *reinterpret_cast<const float4*>(&s.acum[16][c0 + 4]);
            float rs[8], kb[8], bonus = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a_t = at[i] + (t > 8 ? a8[i] : 0.f);
                const float a_t1 = at1[i] + (t + 1 > 8 ? a8[i] : 0.f);
                rs[i] = rv[i] * __expf(a_t);
                kb[i] = (a16[i] + a8[i] < -kMaxLogDecay) ? 0.f : kv[i] * __expf(-a_t1);
                bonus += rv[i] * s.u[c0 + i] * kv[i];
            }
            const uint4 rs_packed = make_uint4(pack_bf16(rs[0], rs[1]), pack_bf16(rs[2], rs[3]), pack_bf16(rs[4], rs[5]),
                                               pack_bf16(rs[6], rs[7]));
            *reinterpret_cast<uint4*>(&s.opR[op_index(16, t, c0)]) = rs_packed;
            *reinterpret_cast<uint4*>(&s.opS[op_index(128, 64 + t, c0)]) = rs_packed;
            *reinterpret_cast<uint4*>(&s.opKb[op_index(16, t, c0)]) =
                make_uint4(pack_bf16(kb[0], kb[1]), pack_bf16(kb[2], kb[3]), pack_bf16(kb[4], kb[5]), pack_bf16(kb[6], kb[7]));
            bonus += __shfl_xor_sync(0xffffffffu, bonus, 1);
            bonus += __shfl_xor_sync(0xffffffffu, bonus, 2);
            bonus += __shfl_xor_sync(0xffffffffu, bonus, 4);
            if ((tid & 7) == 0) s.diag[t] = rightward ? bonus : 0.f;
        }
        // ---- phase B, job 2: thread = (key channel, half of the block): Ks, V^T, e^A ----
        bool big;
        {
            const int c = tid & 63, half = tid >> 6;
            const float a8 = s.acum[8][c];
            const float A = s.acum[16][c] + a8;
            big = A < -kMaxLogDecay;
            float kh[8], vv[8], a1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = half * 8 + j, row = row_of(t);
                a1[j] = s.acum[t + 1][c];
                kh[j] = s.raw[1][row][c];
                vv[j] = s.raw[2][row][c];
            }
            if (half == 0) s.dtot[c] = __expf(A);
#pragma unroll
            for (int j = 0; j < 8; ++j) kh[j] *= __expf(A - (a1[j] + (half * 8 + j + 1 > 8 ? a8 : 0.f)));
            *reinterpret_cast<uint4*>(&s.opK[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(kh[0], kh[1]), pack_bf16(kh[2], kh[3]), pack_bf16(kh[4], kh[5]), pack_bf16(kh[6], kh[7]));
            *reinterpret_cast<uint4*>(&s.opV[op_index(128, c, half * 8)]) =
                make_uint4(pack_bf16(vv[0], vv[1]), pack_bf16(vv[2], vv[3]), pack_bf16(vv[4], vv[5]), pack_bf16(vv[6], vv[7]));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        const bool pairwise = __syncthreads_or(big) != 0;      // CTA-uniform
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- scores on the tensor core: rows 64..79 of (opS . opKb^T), lane 64 + t <- score[t][.] ----
        if (!pairwise && tid == kIssuer) {
#pragma unroll
            for (int ks = 0; ks < N / 16; ++ks) {
                const uint64_t da = make_desc(smem_u32(s.opS) + ks * 2 * (128 * 16), 128 * 16, 128);
                const uint64_t db = make_desc(smem_u32(s.opKb) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 80, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
            }
            tc_commit(&s.bar_score);
            if (step + 1 < n_steps) issue_loads(step + 1);     // the staging arrays were last read before the barrier
        }
        // ---- state round trip (warps 0, 1): bf16 copy for the read-out, decay in place ----
        if (tid < N) {
            uint32_t x[4][16];
            if (blk > 0) {
#pragma unroll
                for (int g = 0; g < 4; ++g) tmem_ld16_issue(lane_addr + g * 16, x[g]);
                tmem_ld_wait();
            } else {
#pragma unroll
                for (int g = 0; g < 4; ++g)
#pragma unroll
                    for (int i = 0; i < 16; ++i) x[g][i] = 0u;                   // a direction starts from the zero state
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float f[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(x[g][i]);
                *reinterpret_cast<uint4*>(&s.opS[op_index(128, tid, g * 16)]) =
                    make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
                *reinterpret_cast<uint4*>(&s.opS[op_index(128, tid, g * 16 + 8)]) =
                    make_uint4(pack_bf16(f[8], f[9]), pack_bf16(f[10], f[11]), pack_bf16(f[12], f[13]), pack_bf16(f[14], f[15]));
#pragma unroll
                for (int i = 0; i < 16; ++i) x[g][i] = __float_as_uint(f[i] * s.dtot[g * 16 + i]);
                tmem_st16(lane_addr + g * 16, x[g]);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        if (!pairwise) {
            if (warp == 2) {
                // ---- warp 2 owns TMEM lanes 64..79: row t of the scores, masked to s < t, bonus on the diagonal ----
                wait_on(&s.bar_score, phase_score);
                phase_score ^= 1u;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t x[16];
                tmem_ld16_issue(lane_addr + 80, x);
                tmem_ld_wait();
                if (lane < 16) {
                    float pr[16];
                    const float dg = s.diag[lane];
#pragma unroll
                    for (int q = 0; q < SC; ++q) pr[q] = q < lane ? __uint_as_float(x[q]) : (q == lane ? dg : 0.f);
                    *reinterpret_cast<uint4*>(&s.opP[op_index(16, lane, 0)]) =
                        make_uint4(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
                    *reinterpret_cast<uint4*>(&s.opP[op_index(16, lane, 8)]) =
                        make_uint4(pack_bf16(pr[8], pr[9]), pack_bf16(pr[10], pr[11]), pack_bf16(pr[12], pr[13]), pack_bf16(pr[14], pr[15]));
                }
            }
        } else {
            // ---- strong decay: the 16 x 16 scores pairwise in fp32, every exponent <= 0 ----
            for (int idx = tid; idx < SC * SC; idx += kThreads) {
                const int t = idx >> 4, sidx = idx & 15;
                const float* rt = s.raw[0][row_of(t)];
                const float* ks = s.raw[1][row_of(sidx)];
                float acc = 0.f;
                if (sidx < t) {
                    const bool t_hi = t > 8, s_hi = sidx + 1 > 8;     // running sums restart at token 8
#pragma unroll 8
                    for (int i = 0; i < N; ++i) {
                        const float a8 = s.acum[8][i];
                        const float e = (s.acum[t][i] + (t_hi ? a8 : 0.f)) - (s.acum[sidx + 1][i] + (s_hi ? a8 : 0.f));
                        acc += rt[i] * ks[i] * __expf(e);
                    }
                } else if (sidx == t) {
                    acc = s.diag[t];
                }
                s.opP[op_index(16, t, sidx)] = __float2bfloat16(acc);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        // ---- tensor core: read-out against the old state, in-block part, state update; then the next block's loads ----
        if (tid == kIssuer) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < N / 16; ++ks) {
                const uint64_t da = make_desc(smem_u32(s.opS) + ks * 2 * (128 * 16), 128 * 16, 128);
                const uint64_t db = make_desc(smem_u32(s.opR) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 64, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
            }
            const uint64_t dv = make_desc(smem_u32(s.opV), 128 * 16, 128);
            umma_bf16(tmem + 64, dv, make_desc(smem_u32(s.opP), 16 * 16, 128), instr_desc(128, 16), 1u);
            umma_bf16(tmem, dv, make_desc(smem_u32(s.opK), 64 * 16, 128), instr_desc(128, 64), 1u);
            tc_commit(&s.bar_main);
            if (pairwise && step + 1 < n_steps) issue_loads(step + 1);   // the pairwise scores read the staging arrays too
        }
        // ---- everyone waits for the tensor core (the operands are rewritten next); warps 0, 1 send this block's y ----
        wait_on(&s.bar_main, phase_main);
        phase_main ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tid < N) {
            uint32_t yt[16];
            tmem_ld16_issue(lane_addr + 64, yt);
            tmem_ld_wait();
            const int y0 = tile_start(step);
            if (y0 >= 0) {
#pragma unroll
                for (int t = 0; t < SC; ++t) s.ytile[row_of(t)][tid] = __uint_as_float(yt[t]);
                sm100::fence_proxy_async_smem();
                sm100::named_bar_sync(1, N);
                if (tid == 0) {
                    if (rightward) {
                        sm100::tma_store_3d(&map_y, &s.ytile[0][0], h * N, y0, b);        // rows past T are clipped
                    } else {
                        if (blk == 0) sm100::tma_store_wait_all();                        // every rightward store has landed
                        tma_reduce_add_3d(&map_y, &s.ytile[0][0], h * N, y0, b);
                    }
                    sm100::tma_store_commit();
                }
            } else {
                // ragged last block of the leftward walk: its tile would start before token 0
                if (tid == 0) sm100::tma_store_wait_all();
                sm100::named_bar_sync(1, N);
#pragma unroll
                for (int t = 0; t < SC; ++t) {
                    const int t_seq = blk * SC + t;
                    if (t_seq < T) atomicAdd(a.y + base + static_cast<size_t>(T - 1 - t_seq) * C + tid, __uint_as_float(yt[t]));
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (tid == 0) sm100::tma_store_wait_all();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}

int forward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw, const float* u,
            float* y, unsigned* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(wkv6_tc_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(Smem))) != cudaSuccess)
            return -1;
        configured = true;
    }
    cudaFree(nullptr);   // descriptors are encoded against the current context; a fresh thread may not have one bound
    const int C = H * N;
    CUtensorMap mr, mk, mv, mw, my;
    if (!(tensor_map::make_btc_f32(&mr, r, B, T, C, N, SC) && tensor_map::make_btc_f32(&mk, k, B, T, C, N, SC) &&
          tensor_map::make_btc_f32(&mv, v, B, T, C, N, SC) && tensor_map::make_btc_f32(&mw, w_raw, B, T, C, N, SC) &&
          tensor_map::make_btc_f32(&my, y, B, T, C, N, SC))) {
        set_error_detail("cuTensorMapEncodeTiled rejected a (C, T, B) fp32 tensor map");
        return -1;
    }
    Args a{B, T, H, r, k, v, w_raw, u, y, status};
    cudaMemsetAsync(status, 0, sizeof(unsigned), stream);
    wkv6_tc_forward_kernel<<<B * H, kThreads, sizeof(Smem), stream>>>(a, mr, mk, mv, mw, my);
    return 1;
}

}  // namespace wkv6tc
