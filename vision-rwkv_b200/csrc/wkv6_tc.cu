// WKV6 forward on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 operands, fp32 state.
//
// Per (batch, head) the 64 x 64 state S[key][value] lives in tensor memory as its transpose
// (TMEM lane = value channel, column = key channel, fp32).  The sequence is walked 16 tokens
// at a time; for every 16-token block, with a_t = sum of log-decays of the block's tokens
// before t and A = a_16, all matrix work runs as UMMA instructions (M = 128, fp32 accumulate):
//
//   P^T (16 x 16)  = Kb (16 x 64) . Rs^T        Kb[s][i] = k_s[i] e^{-a_{s+1}[i]},  Rs[t][i] = r_t[i] e^{a_t[i]}
//                    masked to s < t, the diagonal replaced by the bonus  sum_i r_t[i] u[i] k_t[i]
//   y^T (64 x 16)  = S^T (64 x 64, bf16 copy) . Rs^T  +  V^T (64 x 16) . P^T
//   S^T (64 x 64) += V^T (64 x 16) . Ks         Ks[t][i] = k_t[i] e^{A[i] - a_{t+1}[i]}
//                    after S^T was scaled by e^{A[i]} per key column on its way through registers
//
// The rows of Kb sit in rows 64..79 of the state operand, so the score product is the same
// instruction shape as the read-out and lands in TMEM lanes 64..79, which an otherwise idle warp
// owns.  e^{-a_{s+1}} grows with the decay; a block whose accumulated log-decay exceeds 80 in any
// channel evaluates its 16 x 16 scores pairwise on the CUDA cores instead (every exponent <= 0
// there), so nothing overflows however strong the decay is.  The leftward direction is the same
// walk over the reversed sequence without the bonus; one CTA runs both and adds the second into
// the first.  The state never leaves the SM: per block it makes one round trip TMEM -> registers
// -> TMEM (decay) and leaves a bf16 copy in shared memory as the next A operand.  The next
// block's r, k, v, w are fetched into registers while the current block is processed.
//
// Accuracy is that of bf16 operands with fp32 accumulation (about 1e-2 of max|y|); the exact fp32
// sweeps of wkv6_sweeps.cu remain the default for float32 callers.
//
// Reference being replaced: classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu:6-97.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
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
    __nv_bfloat16 opS[128 * 64];      // A: rows 0..63 = S^T (value x key), rows 64..79 = Kb (token x key)
    __nv_bfloat16 opV[128 * 16];      // A of the update and of the in-block part: V^T, rows = value, K = token
    __nv_bfloat16 opR[16 * 64];       // B of the read-out and of the scores: rows = token, K = key
    __nv_bfloat16 opK[64 * 16];       // B of the update: rows = key, K = token
    __nv_bfloat16 opP[16 * 16];       // B of the in-block part: rows = token t, K = token s
    float raw[4][SC][N];              // r, k, v, w of the block (fp32)
    float acum[SC + 1][N];            // a_0 .. a_16 per key channel (pairwise score path only)
    float dtot[N];
    float u[N];
    uint64_t bar_main;
    uint64_t bar_score;
    uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

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
// Bounded wait on an mbarrier phase; false if it ran out.
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0,1,0,p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
        if (i > 64) __nanosleep(32);
    }
    return false;
}

// The 8 float4 of one 16-token block that a thread stages: 4 arrays x 16 tokens x 16 float4.
struct Prefetch {
    float4 q[8];
};
__device__ __forceinline__ void fetch_block(Prefetch& p, const Args& a, size_t base, int C, int T, int step,
                                            int n_blocks, int tid) {
    const bool rightward = step < n_blocks;
    const int blk = rightward ? step : step - n_blocks;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = tid + j * kThreads;
        const int which = i >> 8, row = (i >> 4) & 15, c4 = (i & 15) * 4;
        const int t_seq = blk * SC + row;
        const int tg = rightward ? t_seq : T - 1 - t_seq;
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t_seq < T) {
            const float* src = which == 0 ? a.r : which == 1 ? a.k : which == 2 ? a.v : a.w;
            val = __ldg(reinterpret_cast<const float4*>(src + base + static_cast<size_t>(tg) * C + c4));
        }
        p.q[j] = val;
    }
}
__device__ __forceinline__ void stage_block(Smem& s, const Prefetch& p, int tid) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = tid + j * kThreads;
        const int which = i >> 8, row = (i >> 4) & 15, c4 = (i & 15) * 4;
        *reinterpret_cast<float4*>(&s.raw[which][row][c4]) = p.q[j];
    }
}

__global__ void __launch_bounds__(kThreads, 4) wkv6_tc_forward_kernel(const Args a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int T = a.T, C = a.H * N;
    const size_t base = static_cast<size_t>(b) * T * C + static_cast<size_t>(h) * N;
    const int n_blocks = (T + SC - 1) / SC;
    const int n_steps = 2 * n_blocks;

    Prefetch pre;
    fetch_block(pre, a, base, C, T, 0, n_blocks, tid);

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s.bar_main)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s.bar_score)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
    stage_block(s, pre, tid);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's 32 TMEM lanes

    uint32_t phase_main = 0, phase_score = 0;
    bool failed = false;
    for (int step = 0; step < n_steps; ++step) {
        const bool rightward = step < n_blocks;
        const int blk = rightward ? step : step - n_blocks;
        if (step + 1 < n_steps) fetch_block(pre, a, base, C, T, step + 1, n_blocks, tid);   // lands during this block

        // ---- per key channel: cumulative log-decays and the scaled bf16 operands (two threads per channel) ----
        bool big;
        {
            const int c = tid & 63, half = tid >> 6;
            float ld[SC];
            float A = 0.f, a_half = 0.f;
#pragma unroll
            for (int t = 0; t < SC; ++t) {
                ld[t] = (blk * SC + t < T) ? -__expf(s.raw[3][t][c]) : 0.f;
                if (t == SC / 2) a_half = A;
                A += ld[t];
            }
            big = A < -kMaxLogDecay;
            const float dt = __expf(A);
            if (half == 0) { s.dtot[c] = dt; s.acum[0][c] = 0.f; }
            float at = half ? a_half : 0.f;
            float kh[8], vv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = half * 8 + j;
                const float ldt = half ? ld[8 + j] : ld[j];
                const float rs = s.raw[0][t][c] * __expf(at);
                at += ldt;                                                      // a_{t+1}
                s.acum[t + 1][c] = at;
                const float kv = s.raw[1][t][c];
                float kb;
                if (!big) { kb = kv * __expf(-at); kh[j] = kb * dt; }
                else      { kb = 0.f;              kh[j] = kv * __expf(A - at); }
                vv[j] = s.raw[2][t][c];
                s.opR[op_index(16, t, c)] = __float2bfloat16(rs);
                s.opS[op_index(128, 64 + t, c)] = __float2bfloat16(kb);
            }
            *reinterpret_cast<uint4*>(&s.opK[op_index(64, c, half * 8)]) =
                make_uint4(pack_bf16(kh[0], kh[1]), pack_bf16(kh[2], kh[3]), pack_bf16(kh[4], kh[5]), pack_bf16(kh[6], kh[7]));
            *reinterpret_cast<uint4*>(&s.opV[op_index(128, c, half * 8)]) =
                make_uint4(pack_bf16(vv[0], vv[1]), pack_bf16(vv[2], vv[3]), pack_bf16(vv[4], vv[5]), pack_bf16(vv[6], vv[7]));
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        const bool pairwise = __syncthreads_or(big) != 0;      // CTA-uniform
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- scores on the tensor core: rows 64..79 of (opS . opR^T) ----
        if (!pairwise && tid == kIssuer) {
#pragma unroll
            for (int ks = 0; ks < N / 16; ++ks) {
                const uint64_t da = make_desc(smem_u32(s.opS) + ks * 2 * (128 * 16), 128 * 16, 128);
                const uint64_t db = make_desc(smem_u32(s.opR) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 80, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
            }
            tc_commit(&s.bar_score);
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
            // ---- warp 2 owns TMEM lanes 64..79: mask the scores, put the bonus on the diagonal ----
            if (warp == 2) {
                float diag = 0.f;
                if (rightward) {
                    const int t = lane & 15, i0 = (lane >> 4) * 32;
#pragma unroll 8
                    for (int ii = 0; ii < 32; ++ii) {
                        const int i = i0 + ((ii + t) & 31);                     // rotate: lanes of one half hit distinct banks
                        diag += s.raw[0][t][i] * s.u[i] * s.raw[1][t][i];
                    }
                    diag += __shfl_xor_sync(0xffffffffu, diag, 16);
                }
                if (!failed && !bar_wait(&s.bar_score, phase_score)) { failed = true; atomicExch(a.status, 1u); }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t x[16];
                tmem_ld16_issue(lane_addr + 80, x);
                tmem_ld_wait();
                if (lane < 16) {
#pragma unroll
                    for (int t = 0; t < SC; ++t) {
                        const float val = t > lane ? __uint_as_float(x[t]) : (t == lane ? diag : 0.f);
                        s.opP[op_index(16, t, lane)] = __float2bfloat16(val);
                    }
                }
            }
            phase_score ^= 1u;
        } else {
            // ---- strong decay: the 16 x 16 scores pairwise in fp32, every exponent <= 0 ----
            for (int idx = tid; idx < SC * SC; idx += kThreads) {
                const int t = idx >> 4, sidx = idx & 15;
                float acc = 0.f;
                if (sidx < t) {
#pragma unroll 8
                    for (int i = 0; i < N; ++i)
                        acc += s.raw[0][t][i] * s.raw[1][sidx][i] * __expf(s.acum[t][i] - s.acum[sidx + 1][i]);
                } else if (sidx == t && rightward) {
#pragma unroll 8
                    for (int i = 0; i < N; ++i) acc += s.raw[0][t][i] * s.u[i] * s.raw[1][t][i];
                }
                s.opP[op_index(16, t, sidx)] = __float2bfloat16(acc);
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
                const uint64_t db = make_desc(smem_u32(s.opR) + ks * 2 * (16 * 16), 16 * 16, 128);
                umma_bf16(tmem + 64, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
            }
            const uint64_t dv = make_desc(smem_u32(s.opV), 128 * 16, 128);
            umma_bf16(tmem + 64, dv, make_desc(smem_u32(s.opP), 16 * 16, 128), instr_desc(128, 16), 1u);
            umma_bf16(tmem, dv, make_desc(smem_u32(s.opK), 64 * 16, 128), instr_desc(128, 64), 1u);
            tc_commit(&s.bar_main);
        }
        // the staging arrays are free now: park the next block
        if (step + 1 < n_steps) stage_block(s, pre, tid);
        // ---- warps 0, 1: wait for the tensor core (bounded), write this block's y ----
        if (tid < N) {
            if (!failed && !bar_wait(&s.bar_main, phase_main)) { failed = true; if (lane == 0) atomicExch(a.status, 1u); }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t yt[16];
            tmem_ld16_issue(lane_addr + 64, yt);
            tmem_ld_wait();
#pragma unroll
            for (int t = 0; t < SC; ++t) {
                const int t_seq = blk * SC + t;
                if (t_seq < T) {
                    const int tg = rightward ? t_seq : T - 1 - t_seq;
                    float* dst = a.y + base + static_cast<size_t>(tg) * C + tid;
                    if (rightward) *dst = __uint_as_float(yt[t]);
                    else atomicAdd(dst, __uint_as_float(yt[t]));      // second of exactly two addends: order-free
                }
            }
        }
        phase_main ^= 1u;
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
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
    Args a{B, T, H, r, k, v, w_raw, u, y, status};
    cudaMemsetAsync(status, 0, sizeof(unsigned), stream);
    wkv6_tc_forward_kernel<<<B * H, kThreads, sizeof(Smem), stream>>>(a);
    return 1;
}

}  // namespace wkv6tc
