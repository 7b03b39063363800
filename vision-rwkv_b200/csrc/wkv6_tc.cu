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
// Two kernels share this arithmetic.  wkv6_tc_forward_kernel, described above, does every phase of
// a block with all of its four warps in turn.  wkv6_tc_pipelined_kernel, further down and the one
// used by default, splits the phases over warp roles so that only the state's round trip and the
// products remain serial.
//
// Reference being replaced: classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu:6-97.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <mutex>
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
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }
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

// ---- the pipelined kernel ---------------------------------------------------------------------------
// Same arithmetic, different schedule.  The serial kernel above does every phase of a block with all
// of its warps, one phase after the other; what must be serial, though, is only
//     state round trip (block n)  ->  read-out / update products (block n)  ->  round trip (n + 1).
// Here one CTA walks one direction of one (batch, head) with nine warps in three roles:
//   producers (warps 3, 6..12, two groups of four): group g prepares the operands of the blocks g, g+2, ...
//       (log-decay sums, scalings, bf16 rounding, the pairwise scores of a strongly decaying block)
//       into operand set g, two block periods ahead of their use;
//   loader (warp 13): the TMA loads of block n+2 as soon as the producers have read block n (issuing
//       the four copies costs several hundred cycles, too many for a thread the others wait for);
//   control (warp 2, owner of TMEM lanes 64..95): issues all tensor-core work; between the score
//       product and the main products it masks the 16 x 16 scores into the P operand;
//   state (warps 0, 1, 4, 5; each owns 32 TMEM lanes x 32 state columns): the round trip, and, while
//       the main products of block n run, the output tile of block n-1 (TMEM -> shared -> TMA
//       reduce-add into y, which the host zeroed; the two directions of a head are two CTAs).
// Hand-overs are mbarriers (operands ready / operand set free / products done) and two named
// barriers; every wait is bounded.
constexpr int kPThreads = 448;    // 4 state warps, 1 control warp, 8 producer warps, 1 loader warp
constexpr int kBarRound = 1;     // named barrier: state + control, 160 threads
constexpr int kBarYTile = 2;     // state, 128 threads
constexpr int kBarProd = 3;      // producer group 0 (128 threads); group 1 uses the next id

struct OpSet {
    __nv_bfloat16 opR[16 * 64];       // B of the read-out; through a base 1 KB lower also the A of the scores (rows 64..79)
    __nv_bfloat16 opKb[16 * 64];      // B of the scores: rows = token s, K = key
    __nv_bfloat16 opK[64 * 16];       // B of the update: rows = key, K = token
    __nv_bfloat16 opV[64 * 16];       // A of the update and of the in-block part (rows 64..127 of the instruction: whatever follows)
    __nv_bfloat16 opP[16 * 16];       // B of the in-block part: rows = token t, K = token s
    float dtot[N];
    float diag[SC];
    uint32_t pairwise;                // the producers wrote opP themselves (strong decay)
    uint32_t pad[15];
};

struct __align__(1024) SmemP {
    __nv_bfloat16 opS[64 * 64];       // A of the read-out: S^T, rows = value, K = key (rows 64..127: the bytes that follow)
    OpSet sets[2];
    float raw[2][4][SC][N];           // r, k, v, w of two blocks in flight
    float ytile[2][SC][N];
    float acum[2][SC + 1][N];         // a_0 .. a_16 per key channel, one array per producer group
    float u[N];
    uint64_t raw_full[2];
    uint64_t raw_free[2];
    uint64_t ops_ready[2];
    uint64_t ops_free[2];
    uint64_t bar_main;
    uint64_t bar_score;
    uint32_t tmem_base;
};

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool named_bar_or(int id, int threads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(pred)), "r"(id), "r"(threads)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&x)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7])
                 : "r"(taddr));
}

// r, k, v staging tiles hold float32 or, for callers whose activations are bfloat16, bfloat16 in the
// first half of the same space (w stays float32).  bfloat16 elements are read as the 32-bit word
// of a channel pair, never as 2-byte accesses.
template <bool kHalfIn>
__device__ __forceinline__ float4 raw_ld4(const float* tile, int row, int c0) {
    if (!kHalfIn) return *reinterpret_cast<const float4*>(tile + row * N + c0);
    const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(tile) + row * N + c0);
    return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                       __uint_as_float(w.y & 0xffff0000u));
}
template <bool kHalfIn>
__device__ __forceinline__ float raw_ld1(const float* tile, int row, int c) {
    if (!kHalfIn) return tile[row * N + c];
    const uint32_t word = reinterpret_cast<const uint32_t*>(tile)[(row * N + c) >> 1];
    return __uint_as_float((c & 1) ? (word & 0xffff0000u) : (word << 16));
}

template <bool kHalfIn>
__global__ void __launch_bounds__(kPThreads, 2)
wkv6_tc_pipelined_kernel(const Args a, const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_y) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    SmemP& s = *reinterpret_cast<SmemP*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.x >> 1;
    const bool rightward = (blockIdx.x & 1) == 0;
    const int b = bh / a.H, h = bh % a.H;
    const int T = a.T, C = a.H * N;
    const size_t base = static_cast<size_t>(b) * T * C + static_cast<size_t>(h) * N;
    const int n_steps = (T + SC - 1) / SC;

    const bool is_state = (warp & 3) < 2 && warp < 8;          // warps 0, 1, 4, 5
    const bool is_control = warp == 2;
    const bool is_loader = warp == 13;
    const bool is_producer = !is_state && !is_control && !is_loader;   // warps 3, 6..12
    const int pid = ((warp == 3) ? 0 : warp - 5) * 32 + lane;   // producers: 0..255

    auto tile_start = [&](int step) { return rightward ? step * SC : T - SC * (step + 1); };
    auto row_of = [&](int t) { return rightward ? t : SC - 1 - t; };

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            sm100::mbar_init(&s.raw_full[i], 1);
            sm100::mbar_init(&s.raw_free[i], 1);
            sm100::mbar_init(&s.ops_ready[i], 1);
            sm100::mbar_init(&s.ops_free[i], 1);
        }
        sm100::mbar_init(&s.bar_main, 1);
        sm100::mbar_init(&s.bar_score, 1);
        sm100::mbar_init_fence();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                     "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid < N) s.u[tid] = a.u[h * N + tid];
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);   // this warp's 32 TMEM lanes

    bool failed = false;
    auto wait_on = [&](uint64_t* bar, uint32_t parity) {
        if (!failed && !sm100::mbar_wait(bar, parity, kWaitLimit)) { failed = true; atomicExch(a.status, 1u); }
    };

    if (is_producer) {
        // =================================== producers ===================================
        // two groups of four warps; group g prepares the blocks q = g, g + 2, ... into operand set g from staging
        // slot g, with its own running-sum array and named barrier, so that a block has two block periods to get ready
        const int group = pid >> 7, gid = pid & 127;
        const int bar_id = kBarProd + group;
        float(&acum)[SC + 1][N] = s.acum[group];
        OpSet& set = s.sets[group];
        float(&raw)[4][SC][N] = s.raw[group];
        for (int q = group; q < n_steps; q += 2) {
            const uint32_t use_parity = (q >> 1) & 1;
            wait_on(&s.raw_full[group], use_parity);
            // ---- phase A: running sums of the log-decays, a_t[c] for t = 0..16; thread = (key channel, half of the
            //      block), the two halves of a channel in one warp so that the first half's total travels by shuffle ----
            {
                const int c = (gid >> 5) * 16 + (lane & 15), half = lane >> 4;
                float wv[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) wv[j] = raw[3][row_of(half * 8 + j)][c];
                float pre[8], run = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    run += (q * SC + half * 8 + j < T) ? -__expf(wv[j]) : 0.f;
                    pre[j] = run;
                }
                const float up = __shfl_up_sync(0xffffffffu, run, 16);
                const float before = half ? up : 0.f;
                if (half == 0) acum[0][c] = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) acum[half * 8 + j + 1][c] = pre[j] + before;
            }
            if (q >= 2) wait_on(&s.ops_free[group], use_parity ^ 1u);   // the products of block q-2 are done with this set
            sm100::named_bar_sync(bar_id, 128);
            // ---- job 1: work item = (token t, 4 key channels): Rs, Kb, bonus; two items per thread ----
#pragma unroll
            for (int rep = 0; rep < 2; ++rep) {
                const int it = gid + 128 * rep;
                const int t = it >> 4, c0 = (it & 15) * 4, row = row_of(t);
                const float4 rv = raw_ld4<kHalfIn>(&raw[0][0][0], row, c0);
                const float4 kv = raw_ld4<kHalfIn>(&raw[1][0][0], row, c0);
                const float4 at = *reinterpret_cast<const float4*>(&acum[t][c0]);
                const float4 at1 = *reinterpret_cast<const float4*>(&acum[t + 1][c0]);
                const float4 aA = *reinterpret_cast<const float4*>(&acum[SC][c0]);
                const float rvv[4] = {rv.x, rv.y, rv.z, rv.w}, kvv[4] = {kv.x, kv.y, kv.z, kv.w};
                const float a0[4] = {at.x, at.y, at.z, at.w}, a1[4] = {at1.x, at1.y, at1.z, at1.w};
                const float aa[4] = {aA.x, aA.y, aA.z, aA.w};
                float rs[4], kb[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    rs[i] = rvv[i] * __expf(a0[i]);
                    kb[i] = (aa[i] < -kMaxLogDecay) ? 0.f : kvv[i] * __expf(-a1[i]);
                }
                *reinterpret_cast<uint2*>(&set.opR[op_index(16, t, c0)]) = make_uint2(pack_bf16(rs[0], rs[1]), pack_bf16(rs[2], rs[3]));
                *reinterpret_cast<uint2*>(&set.opKb[op_index(16, t, c0)]) = make_uint2(pack_bf16(kb[0], kb[1]), pack_bf16(kb[2], kb[3]));
                if (rightward) {       // the bonus exists in this direction only
                    const float4 uu = *reinterpret_cast<const float4*>(&s.u[c0]);
                    float bonus = (rv.x * uu.x * kv.x + rv.y * uu.y * kv.y) + (rv.z * uu.z * kv.z + rv.w * uu.w * kv.w);
                    bonus += __shfl_xor_sync(0xffffffffu, bonus, 1);
                    bonus += __shfl_xor_sync(0xffffffffu, bonus, 2);
                    bonus += __shfl_xor_sync(0xffffffffu, bonus, 4);
                    bonus += __shfl_xor_sync(0xffffffffu, bonus, 8);
                    if ((it & 15) == 0) set.diag[t] = bonus;
                } else if ((it & 15) == 0) {
                    set.diag[t] = 0.f;
                }
            }
            // ---- job 2: work item = (key channel, quarter of the block): Ks, V^T, e^A; two items per thread ----
            bool big = false;
#pragma unroll
            for (int rep = 0; rep < 2; ++rep) {
                const int it = gid + 128 * rep;
                const int c = it & 63, quarter = it >> 6;
                const float A = acum[SC][c];
                big = big || (A < -kMaxLogDecay);
                float kh[4], vv[4], a1[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int t = quarter * 4 + j, row = row_of(t);
                    a1[j] = acum[t + 1][c];
                    kh[j] = raw_ld1<kHalfIn>(&raw[1][0][0], row, c);
                    vv[j] = raw_ld1<kHalfIn>(&raw[2][0][0], row, c);
                }
                if (quarter == 0) set.dtot[c] = __expf(A);
#pragma unroll
                for (int j = 0; j < 4; ++j) kh[j] *= __expf(A - a1[j]);
                *reinterpret_cast<uint2*>(&set.opK[op_index(64, c, quarter * 4)]) = make_uint2(pack_bf16(kh[0], kh[1]), pack_bf16(kh[2], kh[3]));
                *reinterpret_cast<uint2*>(&set.opV[op_index(64, c, quarter * 4)]) = make_uint2(pack_bf16(vv[0], vv[1]), pack_bf16(vv[2], vv[3]));
            }
            const bool pairwise = named_bar_or(bar_id, 128, big);   // also orders diag before the loop below
            if (pairwise) {
                // ---- strong decay: the 16 x 16 scores pairwise in fp32, every exponent <= 0 ----
                for (int rep = 0; rep < 2; ++rep) {
                    const int it = gid + 128 * rep;
                    const int t = it >> 4, sidx = it & 15;
                    const int row_t = row_of(t), row_s = row_of(sidx);
                    float acc = 0.f;
                    if (sidx < t) {
#pragma unroll 8
                        for (int i = 0; i < N; ++i)
                            acc += raw_ld1<kHalfIn>(&raw[0][0][0], row_t, i) * raw_ld1<kHalfIn>(&raw[1][0][0], row_s, i) *
                                   __expf(acum[t][i] - acum[sidx + 1][i]);
                    } else if (sidx == t) {
                        acc = set.diag[t];
                    }
                    // one 4-byte store per lane pair: 2-byte shared stores are slow
                    const float other = __shfl_xor_sync(0xffffffffu, acc, 1);
                    if ((sidx & 1) == 0) *reinterpret_cast<uint32_t*>(&set.opP[op_index(16, t, sidx)]) = pack_bf16(acc, other);
                }
            }
            if (gid == 0) set.pairwise = pairwise ? 1u : 0u;
            sm100::fence_proxy_async_smem();
            sm100::named_bar_sync(bar_id, 128);
            if (gid == 0) {
                mbar_arrive(&s.ops_ready[group]);
                mbar_arrive(&s.raw_free[group]);              // every producer of the group is done reading this staging slot
            }
        }
    } else if (is_loader) {
        // =================================== loader ===================================
        if (lane == 0) {
            sm100::prefetch_tensormap(&map_r);
            sm100::prefetch_tensormap(&map_k);
            sm100::prefetch_tensormap(&map_v);
            sm100::prefetch_tensormap(&map_w);
            for (int step = 0; step < n_steps; ++step) {
                const int slot = step & 1, y0 = tile_start(step);
                if (step >= 2) wait_on(&s.raw_free[slot], ((step >> 1) & 1) ^ 1u);
                sm100::mbar_expect_tx(&s.raw_full[slot], (kHalfIn ? 3 * 2 + 4 : 4 * 4) * SC * N);
                sm100::tma_load_3d(&s.raw[slot][0][0][0], &map_r, &s.raw_full[slot], h * N, y0, b);
                sm100::tma_load_3d(&s.raw[slot][1][0][0], &map_k, &s.raw_full[slot], h * N, y0, b);
                sm100::tma_load_3d(&s.raw[slot][2][0][0], &map_v, &s.raw_full[slot], h * N, y0, b);
                sm100::tma_load_3d(&s.raw[slot][3][0][0], &map_w, &s.raw_full[slot], h * N, y0, b);
            }
        }
    } else if (is_control) {
        // =================================== control ===================================
        uint32_t score_parity = 0;
        // descriptors are formed by the whole warp (warp-uniform values), one elected lane issues
        const uint64_t d_state = make_desc(smem_u32(s.opS), 1024, 128);
        for (int m = 0; m < n_steps; ++m) {
            const int slot = m & 1;
            OpSet& set = s.sets[slot];
            const uint64_t d_r = make_desc(smem_u32(set.opR), 256, 128);
            const uint64_t d_ra = make_desc(smem_u32(set.opR) - 1024, 256, 128);      // rows 64..79 = Rs
            const uint64_t d_kb = make_desc(smem_u32(set.opKb), 256, 128);
            const uint64_t d_v = make_desc(smem_u32(set.opV), 1024, 128);
            const uint64_t d_p = make_desc(smem_u32(set.opP), 256, 128);
            const uint64_t d_k = make_desc(smem_u32(set.opK), 1024, 128);
            wait_on(&s.ops_ready[slot], (m >> 1) & 1);
            const bool pairwise = set.pairwise != 0;
            if (!pairwise) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < N / 16; ++ks)      // a K step of 16 = 512 bytes = 32 descriptor units
                        umma_bf16(tmem + 80, d_ra + 32 * ks, d_kb + 32 * ks, instr_desc(128, 16), ks > 0 ? 1u : 0u);
                    tc_commit(&s.bar_score);
                }
                __syncwarp();
                wait_on(&s.bar_score, score_parity);
                score_parity ^= 1u;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t x[16];
                tmem_ld16_issue(lane_addr + 80, x);
                tmem_ld_wait();
                if (lane < 16) {
                    float pr[16];
                    const float dg = set.diag[lane];
#pragma unroll
                    for (int qq = 0; qq < SC; ++qq) pr[qq] = qq < lane ? __uint_as_float(x[qq]) : (qq == lane ? dg : 0.f);
                    *reinterpret_cast<uint4*>(&set.opP[op_index(16, lane, 0)]) =
                        make_uint4(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
                    *reinterpret_cast<uint4*>(&set.opP[op_index(16, lane, 8)]) =
                        make_uint4(pack_bf16(pr[8], pr[9]), pack_bf16(pr[10], pr[11]), pack_bf16(pr[12], pr[13]), pack_bf16(pr[14], pr[15]));
                }
                sm100::fence_proxy_async_smem();
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            sm100::named_bar_sync(kBarRound, 160);            // the state warps have finished the round trip of block m
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t ycol = tmem + 64 + 32 * slot;      // y^T of even blocks at columns 64..79, odd at 96..111
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < N / 16; ++ks)          // state operand: a K step of 16 = 2048 bytes = 128 units
                    umma_bf16(ycol, d_state + 128 * ks, d_r + 32 * ks, instr_desc(128, 16), ks > 0 ? 1u : 0u);
                umma_bf16(ycol, d_v, d_p, instr_desc(128, 16), 1u);
                umma_bf16(tmem, d_v, d_k, instr_desc(128, 64), 1u);
                tc_commit(&s.bar_main);
                tc_commit(&s.ops_free[slot]);
            }
            __syncwarp();
        }
    } else {
        // =================================== state ===================================
        const int lg = warp & 1, ch = warp >> 2;               // 32 TMEM lanes x 32 state columns per warp
        const int j = lg * 32 + lane;                          // value channel = TMEM lane
        const int sid = ch * 64 + j;                           // 0..127 within the role
        for (int m = 0; m <= n_steps; ++m) {
            if (m >= 1) wait_on(&s.bar_main, (m - 1) & 1);     // products of block m-1 are complete
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (m < n_steps) {
                const OpSet& set = s.sets[m & 1];
                wait_on(&s.ops_ready[m & 1], (m >> 1) & 1);    // dtot of block m
                // ---- round trip of this warp's 32 x 32 piece: bf16 copy for the read-out, decay in place ----
                uint32_t x[2][16];
                if (m > 0) {
                    tmem_ld16_issue(lane_addr + ch * 32, x[0]);
                    tmem_ld16_issue(lane_addr + ch * 32 + 16, x[1]);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) x[0][i] = x[1][i] = 0u;   // the walk starts from the zero state
                }
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    const int c0 = ch * 32 + g * 16;
                    float f[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(x[g][i]);
                    *reinterpret_cast<uint4*>(&s.opS[op_index(64, j, c0)]) =
                        make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
                    *reinterpret_cast<uint4*>(&s.opS[op_index(64, j, c0 + 8)]) =
                        make_uint4(pack_bf16(f[8], f[9]), pack_bf16(f[10], f[11]), pack_bf16(f[12], f[13]), pack_bf16(f[14], f[15]));
#pragma unroll
                    for (int i = 0; i < 16; ++i) x[g][i] = __float_as_uint(f[i] * set.dtot[c0 + i]);
                    tmem_st16(lane_addr + c0, x[g]);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                sm100::fence_proxy_async_smem();
                if (sid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // the y tile of block m-3 has left
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                sm100::named_bar_sync(kBarRound, 160);
            }
            if (m == n_steps) {
                // last pass: no round trip above, so the y slot is released here
                if (sid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                sm100::named_bar_sync(kBarYTile, 128);
            }
            if (m >= 1) {
                // ---- y of block m-1, while the products of block m run: this warp takes 8 of the 16 tokens ----
                const int step = m - 1, ys = step & 1;
                uint32_t yt[8];
                tmem_ld8_issue(lane_addr + 64 + 32 * ys + ch * 8, yt);
                tmem_ld_wait();
                const int y0 = tile_start(step);
                if (y0 >= 0) {
#pragma unroll
                    for (int t = 0; t < 8; ++t) s.ytile[ys][row_of(ch * 8 + t)][j] = __uint_as_float(yt[t]);
                    sm100::fence_proxy_async_smem();
                    sm100::named_bar_sync(kBarYTile, 128);
                    if (sid == 0) {
                        tma_reduce_add_3d(&map_y, &s.ytile[ys][0][0], h * N, y0, b);      // rows past T are clipped
                        sm100::tma_store_commit();
                    }
                } else {
                    // ragged last block of the leftward walk: its tile would start before token 0
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const int t_seq = step * SC + ch * 8 + t;
                        if (t_seq < T) atomicAdd(a.y + base + static_cast<size_t>(T - 1 - t_seq) * C + j, __uint_as_float(yt[t]));
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
        }
        if (sid == 0) sm100::tma_store_wait_all();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}


// ---- backward building block ----------------------------------------------------------------------
// With D_i(t, s) = product of the decays of channel i over the tokens strictly between s and t, the
// gradients of the bidirectional WKV6 are three applications of two token-mixing forms:
//   gv   = forward(k, r, gy)                            (the forward itself, operands permuted)
//   gr_t = sum_{s != t} D(t, s) (.) k_s (v_s . gy_t)   + u (.) k_t (v_t . gy_t)
//   gk_t = sum_{s != t} D(t, s) (.) r_s (gy_s . v_t)   + u (.) r_t (gy_t . v_t)
// The last two are  G(a, p, q)_t[i] = sum_{s != t} D_i(t, s) a_s[i] (p_s . q_t): the decay sits on the
// OUTPUT channel, the contraction runs over the value index.  wkv6_tc_mix_kernel evaluates G without
// its diagonal term, one CTA per (batch, head, direction), the rightward sum (s < t) and the
// leftward sum (s > t) into separate tensors, because the decay gradient needs them apart:
//   g log w_m = sum_{s<m} k_s (.) gk>_s - sum_{t<=m} r_t (.) gr>_t + sum_{s>m} k_s (.) gk<_s - sum_{t>=m} r_t (.) gr<_t
// (">": pairs whose output token is the later one).  Per 16-token block, state Z[i][j] = key x value in
// tensor memory (lane = key channel), a_t = log-decay accumulated over the block's tokens before t:
//   B (16 x 16)      = Q (16 x 64) . P^T                      no decay inside: plain bf16 tiles
//   out'^T (64 x 16) = Z (64 x 64, bf16 copy) . Q^T  +  At^T (64 x 16) . Bm^T     At[s][i] = a_s[i] e^{-a_{s+1}[i]}, Bm = B masked to s < t
//   out_t[i]         = e^{a_t[i]} out'_t[i]                    scaled in fp32 on the way out
//   Z (64 x 64)      = e^{A[i]} Z  +  Ah^T (64 x 16) . P      Ah[s][i] = a_s[i] e^{A[i] - a_{s+1}[i]}
// A block whose accumulated log-decay exceeds 80 in any channel (e^{-a} would overflow) takes its
// in-block part on the CUDA cores with non-positive exponents instead.
struct MixArgs {
    int B, T, H;
    const void* a;       // the tensor that carries the decay's channel index (k for gr, r for gk)
    const void* p;       // paired with a at the source token (v for gr, gy for gk)
    const void* q;       // taken at the output token (gy for gr, v for gk)
    const float* w;      // raw decay input
    float* out_right;    // sums over earlier source tokens
    float* out_left;     // sums over later source tokens
    float* dots;         // (B, T, H): p_t . q_t, written by the rightward CTAs when not null
    unsigned* status;
};

struct __align__(1024) SmemMix {
    __nv_bfloat16 opS[128 * 64];      // A: rows 0..63 = Z (key x value), rows 64..79 = Q (token x value)
    // 64-row A operands of M = 128 products: the tensor core also reads "rows 64..127", which with this k-group
    // stride are the next k-group's rows (or the next array): finite values whose products land in TMEM lanes
    // 64..127, which nobody reads in these columns
    __nv_bfloat16 opAt[64 * 16];      // A of the in-block part: At^T, rows = key channel, K = token
    __nv_bfloat16 opAh[64 * 16];      // A of the update: Ah^T
    __nv_bfloat16 opQ[16 * 64];       // B of the read-out: rows = token, K = value
    __nv_bfloat16 opPb[16 * 64];      // B of the scores: rows = token s, K = value
    __nv_bfloat16 opPt[64 * 16];      // B of the update: rows = value, K = token
    __nv_bfloat16 opBm[16 * 16];      // B of the in-block part: rows = token t, K = token s
    // low halves: every operand that is not a bfloat16 input is carried as hi + lo (lo = x - bf16(x)), and a
    // product of two such operands as hi.hi + hi.lo + lo.hi, which brings the sums to float32 accuracy
    __nv_bfloat16 opSlo[64 * 64];     // Z - bf16(Z)
    __nv_bfloat16 opAtlo[64 * 16];
    __nv_bfloat16 opAhlo[64 * 16];
    __nv_bfloat16 opBmlo[16 * 16];
    __nv_bfloat16 tail_pad[64 * 8];   // what the last k-group of the array before it runs into: zeros
    float raw[4][SC][N];              // a, p, q, w of the block as the copy engine delivers them
    float otile[SC][N];
    float acum[SC + 1][N];
    float scores[SC][SC + 1];         // fp32 copy of B for the strong-decay path
    float dots[SC];
    float dtot[N];
    uint64_t bar_main;
    uint64_t bar_score;
    uint64_t bar_load;
    uint32_t tmem_base;
};

template <bool kHalfIn>
__global__ void __launch_bounds__(kThreads, 4)
wkv6_tc_mix_kernel(const MixArgs a, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_or, const __grid_constant__ CUtensorMap map_ol) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    SmemMix& s = *reinterpret_cast<SmemMix*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit = blockIdx.x >> 1;
    const bool rightward = (blockIdx.x & 1) == 0;
    const int b = unit / a.H, h = unit % a.H;
    const int T = a.T, C = a.H * N;
    const size_t base = static_cast<size_t>(b) * T * C + static_cast<size_t>(h) * N;
    const int n_blocks = (T + SC - 1) / SC;
    float* out = rightward ? a.out_right : a.out_left;
    const CUtensorMap* map_o = rightward ? &map_or : &map_ol;

    // first token (memory order) of the 16-row tile that holds block `blk`; negative for a ragged last leftward block
    auto tile_start = [&](int blk) { return rightward ? blk * SC : T - SC * (blk + 1); };
    auto issue_loads = [&](int blk) {
        const int y0 = tile_start(blk);
        constexpr uint32_t kIn = SC * N * (kHalfIn ? 2 : 4);
        sm100::mbar_expect_tx(&s.bar_load, 3 * kIn + SC * N * 4);
        sm100::tma_load_3d(&s.raw[0][0][0], &map_a, &s.bar_load, h * N, y0, b);
        sm100::tma_load_3d(&s.raw[1][0][0], &map_p, &s.bar_load, h * N, y0, b);
        sm100::tma_load_3d(&s.raw[2][0][0], &map_q, &s.bar_load, h * N, y0, b);
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
    // rows of the A operands that carry no data are still read by the tensor core: keep them finite
    for (int i = tid; i < 128 * 64; i += kThreads) s.opS[i] = __float2bfloat16(0.f);
    for (int i = tid; i < 64 * 64; i += kThreads) s.opSlo[i] = __float2bfloat16(0.f);
    for (int i = tid; i < 64 * 16; i += kThreads) {
        s.opAt[i] = __float2bfloat16(0.f); s.opAh[i] = __float2bfloat16(0.f);
        s.opAtlo[i] = __float2bfloat16(0.f); s.opAhlo[i] = __float2bfloat16(0.f);
    }
    for (int i = tid; i < 16 * 16; i += kThreads) { s.opBm[i] = __float2bfloat16(0.f); s.opBmlo[i] = __float2bfloat16(0.f); }
    for (int i = tid; i < 64 * 8; i += kThreads) s.tail_pad[i] = __float2bfloat16(0.f);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);

    uint32_t phase_main = 0, phase_score = 0, phase_load = 0;
    bool failed = false;
    auto wait_on = [&](uint64_t* bar, uint32_t parity) {
        if (!failed && !sm100::mbar_wait(bar, parity, kWaitLimit)) { failed = true; atomicExch(a.status, 1u); }
    };

    for (int blk = 0; blk < n_blocks; ++blk) {
        auto row_of = [&](int t) { return rightward ? t : SC - 1 - t; };   // block order -> tile row

        wait_on(&s.bar_load, phase_load);
        phase_load ^= 1u;
        if (tid == 0) sm100::tma_store_wait_read();        // the previous output tile has left shared memory

        // ---- phase A: log-decays and their running sums; thread = (key channel, half of the block) ----
        {
            const int c = tid & 63, half = tid >> 6;
            float wv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = s.raw[3][row_of(half * 8 + j)][c];
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
        // ---- phase B, job 1: thread = (token t, 8 value channels): Q (twice), P as the scores' B operand, p . q ----
        {
            const int t = tid >> 3, c0 = (tid & 7) * 8, row = row_of(t);
            float qv[8], pv[8];
            *reinterpret_cast<float4*>(&qv[0]) = raw_ld4<kHalfIn>(&s.raw[2][0][0], row, c0);
            *reinterpret_cast<float4*>(&qv[4]) = raw_ld4<kHalfIn>(&s.raw[2][0][0], row, c0 + 4);
            *reinterpret_cast<float4*>(&pv[0]) = raw_ld4<kHalfIn>(&s.raw[1][0][0], row, c0);
            *reinterpret_cast<float4*>(&pv[4]) = raw_ld4<kHalfIn>(&s.raw[1][0][0], row, c0 + 4);
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) dot += qv[i] * pv[i];
            const uint4 q_packed = make_uint4(pack_bf16(qv[0], qv[1]), pack_bf16(qv[2], qv[3]), pack_bf16(qv[4], qv[5]),
                                              pack_bf16(qv[6], qv[7]));
            *reinterpret_cast<uint4*>(&s.opQ[op_index(16, t, c0)]) = q_packed;
            *reinterpret_cast<uint4*>(&s.opS[op_index(128, 64 + t, c0)]) = q_packed;
            *reinterpret_cast<uint4*>(&s.opPb[op_index(16, t, c0)]) =
                make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]), pack_bf16(pv[6], pv[7]));
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            dot += __shfl_xor_sync(0xffffffffu, dot, 4);
            if ((tid & 7) == 0) s.dots[t] = dot;
        }
        // ---- phase B, job 2: thread = (channel, half of the block): At, Ah (key channel), P^T (value channel), e^A ----
        bool big;
        {
            const int c = tid & 63, half = tid >> 6;
            const float a8 = s.acum[8][c];
            const float A = s.acum[16][c] + a8;
            big = A < -kMaxLogDecay;
            float av[8], pv[8], a1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = half * 8 + j, row = row_of(t);
                a1[j] = s.acum[t + 1][c] + (t + 1 > 8 ? a8 : 0.f);      // a_{t+1}
                av[j] = raw_ld1<kHalfIn>(&s.raw[0][0][0], row, c);
                pv[j] = raw_ld1<kHalfIn>(&s.raw[1][0][0], row, c);
            }
            if (half == 0) s.dtot[c] = __expf(A);
            float at[8], ah[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                at[j] = big ? 0.f : av[j] * __expf(-a1[j]);
                ah[j] = av[j] * __expf(A - a1[j]);
            }
            *reinterpret_cast<uint4*>(&s.opAt[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(at[0], at[1]), pack_bf16(at[2], at[3]), pack_bf16(at[4], at[5]), pack_bf16(at[6], at[7]));
            *reinterpret_cast<uint4*>(&s.opAh[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(ah[0], ah[1]), pack_bf16(ah[2], ah[3]), pack_bf16(ah[4], ah[5]), pack_bf16(ah[6], ah[7]));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                at[j] -= bf16_round(at[j]);
                ah[j] -= bf16_round(ah[j]);
            }
            *reinterpret_cast<uint4*>(&s.opAtlo[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(at[0], at[1]), pack_bf16(at[2], at[3]), pack_bf16(at[4], at[5]), pack_bf16(at[6], at[7]));
            *reinterpret_cast<uint4*>(&s.opAhlo[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(ah[0], ah[1]), pack_bf16(ah[2], ah[3]), pack_bf16(ah[4], ah[5]), pack_bf16(ah[6], ah[7]));
            *reinterpret_cast<uint4*>(&s.opPt[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]), pack_bf16(pv[6], pv[7]));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        const bool pairwise = __syncthreads_or(big) != 0;      // CTA-uniform
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- scores on the tensor core: rows 64..79 of (opS . opPb^T), lane 64 + t <- B[t][.] ----
        if (tid == kIssuer) {
#pragma unroll
            for (int ks = 0; ks < N / 16; ++ks) {
                const uint64_t da = make_desc(smem_u32(s.opS) + ks * 2 * (128 * 16), 128 * 16, 128);
                const uint64_t db = make_desc(smem_u32(s.opPb) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 80, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
            }
            tc_commit(&s.bar_score);
        }
        // ---- state round trip (warps 0, 1; lane = key channel): bf16 copy for the read-out, decay in place ----
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
                    for (int i = 0; i < 16; ++i) x[g][i] = 0u;
            }
            const float decay = s.dtot[tid];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float f[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(x[g][i]);
                *reinterpret_cast<uint4*>(&s.opS[op_index(128, tid, g * 16)]) =
                    make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
                *reinterpret_cast<uint4*>(&s.opS[op_index(128, tid, g * 16 + 8)]) =
                    make_uint4(pack_bf16(f[8], f[9]), pack_bf16(f[10], f[11]), pack_bf16(f[12], f[13]), pack_bf16(f[14], f[15]));
                float lo[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) lo[i] = f[i] - bf16_round(f[i]);
                *reinterpret_cast<uint4*>(&s.opSlo[op_index(64, tid, g * 16)]) =
                    make_uint4(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]), pack_bf16(lo[4], lo[5]), pack_bf16(lo[6], lo[7]));
                *reinterpret_cast<uint4*>(&s.opSlo[op_index(64, tid, g * 16 + 8)]) =
                    make_uint4(pack_bf16(lo[8], lo[9]), pack_bf16(lo[10], lo[11]), pack_bf16(lo[12], lo[13]), pack_bf16(lo[14], lo[15]));
#pragma unroll
                for (int i = 0; i < 16; ++i) x[g][i] = __float_as_uint(f[i] * decay);
                tmem_st16(lane_addr + g * 16, x[g]);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        if (warp == 2) {
            // ---- warp 2 owns TMEM lanes 64..79: row t of the scores, masked to s < t ----
            wait_on(&s.bar_score, phase_score);
            phase_score ^= 1u;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t x[16];
            tmem_ld16_issue(lane_addr + 80, x);
            tmem_ld_wait();
            if (lane < 16) {
                float pr[16];
#pragma unroll
                for (int q = 0; q < SC; ++q) {
                    pr[q] = q < lane ? __uint_as_float(x[q]) : 0.f;
                    s.scores[lane][q] = pr[q];
                }
                *reinterpret_cast<uint4*>(&s.opBm[op_index(16, lane, 0)]) =
                    make_uint4(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
                *reinterpret_cast<uint4*>(&s.opBm[op_index(16, lane, 8)]) =
                    make_uint4(pack_bf16(pr[8], pr[9]), pack_bf16(pr[10], pr[11]), pack_bf16(pr[12], pr[13]), pack_bf16(pr[14], pr[15]));
#pragma unroll
                for (int q = 0; q < SC; ++q) pr[q] -= bf16_round(pr[q]);
                *reinterpret_cast<uint4*>(&s.opBmlo[op_index(16, lane, 0)]) =
                    make_uint4(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[6], pr[7]));
                *reinterpret_cast<uint4*>(&s.opBmlo[op_index(16, lane, 8)]) =
                    make_uint4(pack_bf16(pr[8], pr[9]), pack_bf16(pr[10], pr[11]), pack_bf16(pr[12], pr[13]), pack_bf16(pr[14], pr[15]));
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        // ---- tensor core: read-out against the old state, in-block part, state update ----
        if (tid == kIssuer) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int ks = 0; ks < N / 16; ++ks) {
                const uint64_t da = make_desc(smem_u32(s.opS) + ks * 2 * (128 * 16), 128 * 16, 128);
                const uint64_t db = make_desc(smem_u32(s.opQ) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 64, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
            }
#pragma unroll
            for (int ks = 0; ks < N / 16; ++ks) {                 // the state's low half against the same Q
                const uint64_t da = make_desc(smem_u32(s.opSlo) + ks * 2 * (64 * 16), 64 * 16, 128);
                const uint64_t db = make_desc(smem_u32(s.opQ) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 64, da, db, instr_desc(128, 16), 1u);
            }
            if (!pairwise) {
                const uint64_t at_hi = make_desc(smem_u32(s.opAt), 64 * 16, 128), at_lo = make_desc(smem_u32(s.opAtlo), 64 * 16, 128);
                const uint64_t bm_hi = make_desc(smem_u32(s.opBm), 16 * 16, 128), bm_lo = make_desc(smem_u32(s.opBmlo), 16 * 16, 128);
                umma_bf16(tmem + 64, at_hi, bm_hi, instr_desc(128, 16), 1u);
                umma_bf16(tmem + 64, at_hi, bm_lo, instr_desc(128, 16), 1u);
                umma_bf16(tmem + 64, at_lo, bm_hi, instr_desc(128, 16), 1u);
            }
            umma_bf16(tmem, make_desc(smem_u32(s.opAh), 64 * 16, 128), make_desc(smem_u32(s.opPt), 64 * 16, 128),
                      instr_desc(128, 64), 1u);
            umma_bf16(tmem, make_desc(smem_u32(s.opAhlo), 64 * 16, 128), make_desc(smem_u32(s.opPt), 64 * 16, 128),
                      instr_desc(128, 64), 1u);
            tc_commit(&s.bar_main);
        }
        // ---- strong decay: in-block part per channel in fp32, every exponent <= 0 (added on the way out) ----
        float extra[SC];
#pragma unroll
        for (int t = 0; t < SC; ++t) extra[t] = 0.f;
        if (pairwise && tid < N) {
            const float a8 = s.acum[8][tid];
            for (int t = 1; t < SC; ++t) {
                const float a_t = s.acum[t][tid] + (t > 8 ? a8 : 0.f);
                float acc = 0.f;
                for (int q = 0; q < t; ++q) {
                    const float a_q1 = s.acum[q + 1][tid] + (q + 1 > 8 ? a8 : 0.f);
                    acc += s.scores[t][q] * raw_ld1<kHalfIn>(&s.raw[0][0][0], row_of(q), tid) * __expf(a_t - a_q1);
                }
                extra[t] = acc;
            }
        }
        float scale[SC];
        if (tid < N) {
            const float a8 = s.acum[8][tid];
#pragma unroll
            for (int t = 0; t < SC; ++t) scale[t] = __expf(s.acum[t][tid] + (t > 8 ? a8 : 0.f));
        }
        const int y0 = tile_start(blk);
        if (tid < SC && rightward && a.dots != nullptr && blk * SC + tid < T)
            a.dots[(static_cast<size_t>(b) * T + blk * SC + tid) * a.H + h] = s.dots[tid];
        // ---- everyone waits for the tensor core (the operands are rewritten next); warps 0, 1 send this block's output ----
        wait_on(&s.bar_main, phase_main);
        phase_main ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // the strong-decay path reads the staging tiles until just now: everyone must be past them before they are refilled
        if (pairwise) __syncthreads();
        if (tid == kIssuer && blk + 1 < n_blocks) issue_loads(blk + 1);
        if (tid < N) {
            uint32_t ot[16];
            tmem_ld16_issue(lane_addr + 64, ot);
            tmem_ld_wait();
            if (y0 >= 0) {
#pragma unroll
                for (int t = 0; t < SC; ++t)
                    s.otile[row_of(t)][tid] = pairwise ? scale[t] * __uint_as_float(ot[t]) + extra[t] : scale[t] * __uint_as_float(ot[t]);
                sm100::fence_proxy_async_smem();
                sm100::named_bar_sync(1, N);
                if (tid == 0) {
                    sm100::tma_store_3d(map_o, &s.otile[0][0], h * N, y0, b);        // rows past T are clipped
                    sm100::tma_store_commit();
                }
            } else {
                // ragged last block of the leftward walk: its tile would start before token 0
#pragma unroll
                for (int t = 0; t < SC; ++t) {
                    const int t_seq = blk * SC + t;
                    if (t_seq < T)
                        out[base + static_cast<size_t>(T - 1 - t_seq) * C + tid] =
                            pairwise ? scale[t] * __uint_as_float(ot[t]) + extra[t] : scale[t] * __uint_as_float(ot[t]);
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    if (tid == 0) sm100::tma_store_wait_all();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
}


// ---- backward: combining the four one-sided sums --------------------------------------------------
// gr> = G(k, v, gy) over earlier tokens, gr< over later ones; gk< = G(r, gy, v) over earlier tokens,
// gk> over later ones (">" = pairs whose output token is the later one); dots_t = v_t . gy_t per head.
//   gr = gr> + gr< + u k dots        gk = gk> + gk< + u r dots        gu = sum_{b,t} r k dots
//   x>_t = k_t gk>_t - r_t gr>_t     g log w_m = (sum_{t<m} x>_t) - r_m gr>_m + (sum_{t>m} x<_t) - r_m gr<_m
//   gw_raw = g log w * (-exp(w_raw))
// The sums along T are taken per segment of kSeg tokens: totals (first kernel), their exclusive
// prefix / suffix over the segments (second), the walk inside each segment (third).
constexpr int kSeg = 128;

template <bool kHalfIn>
__device__ __forceinline__ float in_ld(const void* base, size_t idx) {
    if (kHalfIn) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    return static_cast<const float*>(base)[idx];
}

struct FinArgs {
    int B, T, H, n_seg;
    const void* r;
    const void* k;
    const float* w;
    const float* u;
    const float* gr_right;   // gr>
    const float* gr_left;    // gr<
    const float* gk_right;   // G(r, gy, v) over earlier tokens = gk<
    const float* gk_left;    // = gk>
    const float* dots;       // (B, T, H)
    float* gr;
    float* gk;
    float* gw;
    float* gu;               // (H, 64)
    float* tot;              // [3][B][n_seg][C]: x> totals, x< totals, gu parts
};

// grid (n_seg, H, B), 64 threads: thread = channel of the head
template <bool kHalfIn>
__global__ void __launch_bounds__(N) wkv6_bwd_combine_kernel(const FinArgs a) {
    const int seg = blockIdx.x, h = blockIdx.y, b = blockIdx.z, c = h * N + threadIdx.x;
    const int C = a.H * N;
    const int t0 = seg * kSeg, t1 = min(a.T, t0 + kSeg);
    const float u = a.u[c];
    float sx_r = 0.f, sx_l = 0.f, sgu = 0.f;
    for (int t = t0; t < t1; ++t) {
        const size_t i = (static_cast<size_t>(b) * a.T + t) * C + c;
        const float r = in_ld<kHalfIn>(a.r, i), k = in_ld<kHalfIn>(a.k, i);
        const float grr = a.gr_right[i], grl = a.gr_left[i], gkl = a.gk_right[i], gkr = a.gk_left[i];
        const float d = a.dots[(static_cast<size_t>(b) * a.T + t) * a.H + h];
        a.gr[i] = grr + grl + u * k * d;
        a.gk[i] = gkr + gkl + u * r * d;
        sx_r += k * gkr - r * grr;
        sx_l += k * gkl - r * grl;
        sgu += r * k * d;
    }
    const size_t j = (static_cast<size_t>(b) * a.n_seg + seg) * C + c;
    const size_t plane = static_cast<size_t>(a.B) * a.n_seg * C;
    a.tot[j] = sx_r;
    a.tot[plane + j] = sx_l;
    a.tot[2 * plane + j] = sgu;
}

// grid (ceil(C / 128), B + 1): rows b < B turn the totals of batch entry b into exclusive prefix (x>) /
// suffix (x<) sums over its segments; the last row sums the gu parts over batch and segments, fixed order
__global__ void __launch_bounds__(128) wkv6_bwd_carry_kernel(const FinArgs a) {
    const int C = a.H * N;
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c >= C) return;
    const size_t plane = static_cast<size_t>(a.B) * a.n_seg * C;
    if (static_cast<int>(blockIdx.y) < a.B) {
        const int b = blockIdx.y;
        float run = 0.f;
        for (int s = 0; s < a.n_seg; ++s) {
            float* q = a.tot + (static_cast<size_t>(b) * a.n_seg + s) * C + c;
            const float x = *q;
            *q = run;
            run += x;
        }
        run = 0.f;
        for (int s = a.n_seg - 1; s >= 0; --s) {
            float* q = a.tot + plane + (static_cast<size_t>(b) * a.n_seg + s) * C + c;
            const float x = *q;
            *q = run;
            run += x;
        }
    } else {
        float acc = 0.f;
        for (int i = 0; i < a.B * a.n_seg; ++i) acc += a.tot[2 * plane + static_cast<size_t>(i) * C + c];
        a.gu[c] = acc;
    }
}

// grid (n_seg, H, B), 64 threads: the walk inside a segment; the rightward part is parked in gw itself and read back
// by the leftward walk (32 KB per block, still in L2), which leaves the block without shared memory and the SM
// with four times the warps
template <bool kHalfIn>
__global__ void __launch_bounds__(N) wkv6_bwd_decay_kernel(const FinArgs a) {
    const int seg = blockIdx.x, h = blockIdx.y, b = blockIdx.z, lane = threadIdx.x, c = h * N + lane;
    const int C = a.H * N;
    const int t0 = seg * kSeg, t1 = min(a.T, t0 + kSeg);
    const size_t plane = static_cast<size_t>(a.B) * a.n_seg * C;
    const size_t j = (static_cast<size_t>(b) * a.n_seg + seg) * C + c;
    // eight tokens' loads are issued before the running sums consume them: the sums are a serial chain, the loads are not
    constexpr int kU = 8;
    const size_t i0 = (static_cast<size_t>(b) * a.T + t0) * C + c;
    const int n = t1 - t0;
    float run = a.tot[j];
    for (int s0 = 0; s0 < n; s0 += kU) {
        float p[kU], q[kU];
#pragma unroll
        for (int e = 0; e < kU; ++e) {
            p[e] = 0.f; q[e] = 0.f;
            if (s0 + e < n) {
                const size_t i = i0 + static_cast<size_t>(s0 + e) * C;
                p[e] = in_ld<kHalfIn>(a.r, i) * a.gr_right[i];
                q[e] = in_ld<kHalfIn>(a.k, i) * a.gk_left[i];
            }
        }
#pragma unroll
        for (int e = 0; e < kU; ++e)
            if (s0 + e < n) {
                a.gw[i0 + static_cast<size_t>(s0 + e) * C] = run - p[e];
                run += q[e] - p[e];
            }
    }
    run = a.tot[plane + j];
    for (int s1 = n; s1 > 0; s1 -= kU) {
        float p[kU], q[kU], ew[kU], part[kU];
#pragma unroll
        for (int e = 0; e < kU; ++e) {
            p[e] = 0.f; q[e] = 0.f; ew[e] = 0.f; part[e] = 0.f;
            const int s = s1 - 1 - e;
            if (s >= 0) {
                const size_t i = i0 + static_cast<size_t>(s) * C;
                p[e] = in_ld<kHalfIn>(a.r, i) * a.gr_left[i];
                q[e] = in_ld<kHalfIn>(a.k, i) * a.gk_right[i];
                ew[e] = -__expf(a.w[i]);
                part[e] = a.gw[i];
            }
        }
#pragma unroll
        for (int e = 0; e < kU; ++e) {
            const int s = s1 - 1 - e;
            if (s >= 0) {
                a.gw[i0 + static_cast<size_t>(s) * C] = (part[e] + run - p[e]) * ew[e];
                run += q[e] - p[e];
            }
        }
    }
}

// cudaFuncSetAttribute applies to the current device only: one flag per device, under a lock
static bool configure_once() {
    static std::mutex lock;
    static bool done[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    std::lock_guard<std::mutex> guard(lock);
    bool& configured = done[dev & 63];
    if (!configured) {
        if (cudaFuncSetAttribute(wkv6_tc_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(Smem))) != cudaSuccess ||
            cudaFuncSetAttribute(wkv6_tc_pipelined_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(SmemP))) != cudaSuccess ||
            cudaFuncSetAttribute(wkv6_tc_pipelined_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(SmemP))) != cudaSuccess ||
            cudaFuncSetAttribute(wkv6_tc_mix_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(SmemMix))) != cudaSuccess ||
            cudaFuncSetAttribute(wkv6_tc_mix_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(sizeof(SmemMix))) != cudaSuccess)
            return false;
        configured = true;
    }
    return true;
}

// half_in: r, k, v point at bfloat16; w_raw, u, y are float32 either way
static int launch(int B, int T, int H, const void* r, const void* k, const void* v, const float* w_raw, const float* u,
                  float* y, unsigned* status, bool half_in, bool pipelined, cudaStream_t stream, bool clear_status = true) {
    if (!configure_once()) return -1;
    tensor_map::bind_primary_context();   // the tensor-map encoder is a driver call
    const int C = H * N;
    CUtensorMap mr, mk, mv, mw, my;
    if (!(tensor_map::make_btc(&mr, r, B, T, C, N, SC, half_in) && tensor_map::make_btc(&mk, k, B, T, C, N, SC, half_in) &&
          tensor_map::make_btc(&mv, v, B, T, C, N, SC, half_in) && tensor_map::make_btc_f32(&mw, w_raw, B, T, C, N, SC) &&
          tensor_map::make_btc_f32(&my, y, B, T, C, N, SC))) {
        set_error_detail("cuTensorMapEncodeTiled rejected a (C, T, B) tensor map");
        return -1;
    }
    Args a{B, T, H, static_cast<const float*>(r), static_cast<const float*>(k), static_cast<const float*>(v), w_raw, u, y,
           status};
    if (clear_status) cudaMemsetAsync(status, 0, sizeof(unsigned), stream);
    if (pipelined || half_in) {
        // both directions add into y
        cudaMemsetAsync(y, 0, static_cast<size_t>(B) * T * C * sizeof(float), stream);
        if (half_in) wkv6_tc_pipelined_kernel<true><<<2 * B * H, kPThreads, sizeof(SmemP), stream>>>(a, mr, mk, mv, mw, my);
        else wkv6_tc_pipelined_kernel<false><<<2 * B * H, kPThreads, sizeof(SmemP), stream>>>(a, mr, mk, mv, mw, my);
        return 1;
    }
    wkv6_tc_forward_kernel<<<B * H, kThreads, sizeof(Smem), stream>>>(a, mr, mk, mv, mw, my);
    return 1;
}

int forward(int B, int T, int H, const float* r, const float* k, const float* v, const float* w_raw, const float* u,
            float* y, unsigned* status, bool pipelined, cudaStream_t stream) {
    return launch(B, T, H, r, k, v, w_raw, u, y, status, false, pipelined, stream);
}

int forward_bf16in(int B, int T, int H, const void* r, const void* k, const void* v, const float* w_raw, const float* u,
                   float* y, unsigned* status, cudaStream_t stream) {
    return launch(B, T, H, r, k, v, w_raw, u, y, status, true, true, stream);
}

// G(a, p, q) without its diagonal, the two one-sided sums into out_right / out_left (see wkv6_tc_mix_kernel)
static int launch_mix(int B, int T, int H, const void* a_, const void* p_, const void* q_, const float* w_raw, float* out_right,
                      float* out_left, float* dots, unsigned* status, bool half_in, cudaStream_t stream) {
    const int C = H * N;
    CUtensorMap ma, mp, mq, mw, mor, mol;
    if (!(tensor_map::make_btc(&ma, a_, B, T, C, N, SC, half_in) && tensor_map::make_btc(&mp, p_, B, T, C, N, SC, half_in) &&
          tensor_map::make_btc(&mq, q_, B, T, C, N, SC, half_in) && tensor_map::make_btc_f32(&mw, w_raw, B, T, C, N, SC) &&
          tensor_map::make_btc_f32(&mor, out_right, B, T, C, N, SC) && tensor_map::make_btc_f32(&mol, out_left, B, T, C, N, SC))) {
        set_error_detail("cuTensorMapEncodeTiled rejected a (C, T, B) tensor map");
        return -1;
    }
    MixArgs m{B, T, H, a_, p_, q_, w_raw, out_right, out_left, dots, status};
    if (half_in) wkv6_tc_mix_kernel<true><<<2 * B * H, kThreads, sizeof(SmemMix), stream>>>(m, ma, mp, mq, mw, mor, mol);
    else wkv6_tc_mix_kernel<false><<<2 * B * H, kThreads, sizeof(SmemMix), stream>>>(m, ma, mp, mq, mw, mor, mol);
    return 1;
}

size_t backward_workspace(int B, int T, int H) {
    const size_t C = static_cast<size_t>(H) * N, E = static_cast<size_t>(B) * T * C;
    const size_t n_seg = (static_cast<size_t>(T) + kSeg - 1) / kSeg;
    return 256 + (4 * E + static_cast<size_t>(B) * T * H + 3 * static_cast<size_t>(B) * n_seg * C) * sizeof(float);
}

// gv through the forward kernel with permuted operands, gr and gk through the mixing kernel, the
// decay and bonus gradients from their one-sided sums.  half_in: r, k, v, gy point at bfloat16.
int backward(int B, int T, int H, const void* r, const void* k, const void* v, const float* w_raw, const float* u,
             const void* gy, float* gr, float* gk, float* gv, float* gw, float* gu, void* workspace, bool half_in,
             cudaStream_t stream) {
    if (!configure_once()) return -1;
    tensor_map::bind_primary_context();   // the tensor-map encoder is a driver call
    const size_t C = static_cast<size_t>(H) * N, E = static_cast<size_t>(B) * T * C;
    unsigned* status = static_cast<unsigned*>(workspace);
    float* ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + 256);
    float* gr_right = ws;
    float* gr_left = ws + E;
    float* gk_right = ws + 2 * E;
    float* gk_left = ws + 3 * E;
    float* dots = ws + 4 * E;
    float* tot = dots + static_cast<size_t>(B) * T * H;
    int launched = 0;
    // The value gradient and the two mixing launches are independent: the former runs on a side stream (forked from and
    // joined back into the caller's stream by events) and fills the tails of the latter (measured -2.4 % at T = 4096,
    // -5 % at T = 196; moving one mixing launch over as well was measured slower).
    struct Side {
        cudaStream_t stream = nullptr;
        cudaEvent_t fork = nullptr, join = nullptr;
    };
    thread_local Side sides[64];
    int dev = 0;
    cudaGetDevice(&dev);
    Side& side = sides[dev & 63];
    if (side.stream == nullptr) {
        if (cudaStreamCreateWithFlags(&side.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&side.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&side.join, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
    }
    cudaMemsetAsync(status, 0, sizeof(unsigned), stream);
    cudaEventRecord(side.fork, stream);
    cudaStreamWaitEvent(side.stream, side.fork, 0);
    // gv_s = sum_t A(t, s) gy_t with A symmetric under r <-> k: the forward with (r, k, v) := (k, r, gy)
    int n = launch(B, T, H, k, r, gy, w_raw, u, gv, status, half_in, true, side.stream, false);
    cudaEventRecord(side.join, side.stream);
    int n2 = launch_mix(B, T, H, k, v, gy, w_raw, gr_right, gr_left, dots, status, half_in, stream);
    int n3 = launch_mix(B, T, H, r, gy, v, w_raw, gk_right, gk_left, nullptr, status, half_in, stream);
    cudaStreamWaitEvent(stream, side.join, 0);
    if (n < 0 || n2 < 0 || n3 < 0) return -1;
    launched += n + n2 + n3;
    FinArgs f{};
    f.B = B; f.T = T; f.H = H; f.n_seg = (T + kSeg - 1) / kSeg;
    f.r = r; f.k = k; f.w = w_raw; f.u = u;
    f.gr_right = gr_right; f.gr_left = gr_left; f.gk_right = gk_right; f.gk_left = gk_left; f.dots = dots;
    f.gr = gr; f.gk = gk; f.gw = gw; f.gu = gu; f.tot = tot;
    const dim3 grid(f.n_seg, H, B);
    if (half_in) wkv6_bwd_combine_kernel<true><<<grid, N, 0, stream>>>(f);
    else wkv6_bwd_combine_kernel<false><<<grid, N, 0, stream>>>(f);
    wkv6_bwd_carry_kernel<<<dim3((static_cast<unsigned>(C) + 127) / 128, B + 1), 128, 0, stream>>>(f);
    if (half_in) wkv6_bwd_decay_kernel<true><<<grid, N, 0, stream>>>(f);
    else wkv6_bwd_decay_kernel<false><<<grid, N, 0, stream>>>(f);
    return launched + 3;
}

}  // namespace wkv6tc
