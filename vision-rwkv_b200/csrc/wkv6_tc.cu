// WKV6 forward on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 operands, fp32 state.
//
// Per (batch, head) the 64 x 64 state S[key][value] lives in tensor memory as its transpose
// (TMEM lane = value channel, column = key channel, fp32).  The sequence is walked 16 tokens
// at a time; for every 16-token block, with a_t = sum of log-decays of the block's tokens
// before t and A = a_16:
//
//   y^T (64 x 16)  = S^T (64 x 64, bf16 copy) . Rs^T      Rs[t][i] = r_t[i] e^{a_t[i]}          (UMMA, K = 64)
//   S^T (64 x 64) += V^T (64 x 16) . Ks                   Ks[t][i] = k_t[i] e^{A[i] - a_{t+1}[i]} (UMMA, K = 16)
//                    after S^T was scaled by e^{A[i]} per key column on its way through registers
//   y_t           += sum_{s<t} (sum_i r_t[i] k_s[i] e^{a_t[i] - a_{s+1}[i]}) v_s  (+ bonus)      (CUDA cores, exact)
//
// Every exponent that is formed is <= 0, so nothing overflows however strong the decay is; the
// 16 x 16 in-block scores are evaluated pairwise in fp32 for that reason.  The leftward
// direction is the same walk over the reversed sequence without the bonus term; one CTA runs
// both and adds the second into the first.  The state never leaves the SM: per block it makes
// one round trip TMEM -> registers -> TMEM (decay) and leaves a bf16 copy in shared memory as the
// next A operand.  M = 128 instructions are used with rows 64..127 idle.
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
constexpr int NP = N + 4;        // padded row length of the fp32 staging arrays
constexpr int kThreads = 128;
constexpr uint32_t kWaitLimit = 1u << 20;
constexpr uint32_t kTmemCols = 128;   // S^T: columns 0..63, y^T: columns 64..79

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
    __nv_bfloat16 opS[128 * 64];      // A of the read-out: S^T, rows = value (64 used), K = key
    __nv_bfloat16 opV[128 * 16];      // A of the update:   V^T, rows = value, K = token
    __nv_bfloat16 opR[16 * 64];       // B of the read-out: rows = token, K = key
    __nv_bfloat16 opK[64 * 16];       // B of the update:   rows = key,   K = token
    float raw[4][SC][NP];             // r, k, v, w of the block (fp32); rows padded against bank conflicts
    float acum[SC + 1][NP];           // a_0 .. a_16 per key channel
    float score[SC][SC + 1];
    float dtot[N];
    float u[N];
    uint64_t bar;
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t x[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]), "=r"(x[8]),
          "=r"(x[9]), "=r"(x[10]), "=r"(x[11]), "=r"(x[12]), "=r"(x[13]), "=r"(x[14]), "=r"(x[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(x[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
        : "memory");
}

__global__ void __launch_bounds__(kThreads) wkv6_tc_forward_kernel(const Args a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int T = a.T, C = a.H * N;
    const size_t base = static_cast<size_t>(b) * T * C + static_cast<size_t>(h) * N;

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s.bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)),
                     "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    if (tid < N) s.u[tid] = a.u[h * N + tid];
    // rows 64..127 of the A operands are never meaningful but are read by the tensor core: keep them finite
    for (int i = tid; i < 128 * 64; i += kThreads) s.opS[i] = __float2bfloat16(0.f);
    for (int i = tid; i < 128 * 16; i += kThreads) s.opV[i] = __float2bfloat16(0.f);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s.tmem_base;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);   // this warp's 32 TMEM lanes

    const int n_blocks = (T + SC - 1) / SC;
    uint32_t phase = 0;
    bool failed = false;
    for (int dir = 0; dir < 2; ++dir) {
        const bool rightward = (dir == 0);
        // state <- 0
        if (tid < N) {
            float z[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) z[i] = 0.f;
#pragma unroll
            for (int c0 = 0; c0 < N; c0 += 16) tmem_st16(lane_addr + c0, z);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        for (int blk = 0; blk < n_blocks; ++blk) {
            // ---- load the block (token order of this direction), zero rows past the sequence ----
            for (int i = tid; i < 4 * SC * (N / 4); i += kThreads) {
                const int which = i / (SC * (N / 4));
                const int rem = i - which * (SC * (N / 4));
                const int row = rem / (N / 4), c4 = (rem % (N / 4)) * 4;
                const int t_seq = blk * SC + row;
                const int tg = rightward ? t_seq : T - 1 - t_seq;
                float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t_seq < T) {
                    const float* src = which == 0 ? a.r : which == 1 ? a.k : which == 2 ? a.v : a.w;
                    val = *reinterpret_cast<const float4*>(src + base + static_cast<size_t>(tg) * C + c4);
                } else if (which == 3) {
                    val = make_float4(-1e30f, -1e30f, -1e30f, -1e30f);   // exp(w) = 0: log-decay 0 for padding
                }
                *reinterpret_cast<float4*>(&s.raw[which][row][c4]) = val;
            }
            __syncthreads();
            // ---- per key channel: cumulative log-decays, scaled operands ----
            if (tid < N) {
                const int c = tid;
                float acc = 0.f;
                s.acum[0][c] = 0.f;
                float ld[SC];
#pragma unroll
                for (int t = 0; t < SC; ++t) {
                    ld[t] = -__expf(s.raw[3][t][c]);
                    acc += ld[t];
                    s.acum[t + 1][c] = acc;
                }
                const float A = acc;
                s.dtot[c] = __expf(A);
                float at = 0.f;
#pragma unroll
                for (int t = 0; t < SC; ++t) {
                    s.opR[op_index(16, t, c)] = __float2bfloat16(s.raw[0][t][c] * __expf(at));
                    at += ld[t];                                            // a_{t+1}
                    s.opK[op_index(64, c, t)] = __float2bfloat16(s.raw[1][t][c] * __expf(A - at));
                    s.opV[op_index(128, c, t)] = __float2bfloat16(s.raw[2][t][c]);
                }
            }
            __syncthreads();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // ---- state round trip: bf16 copy for the read-out, decay in place ----
            if (tid < N) {
#pragma unroll
                for (int c0 = 0; c0 < N; c0 += 16) {
                    float x[16];
                    tmem_ld16(lane_addr + c0, x);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        s.opS[op_index(128, tid, c0 + i)] = __float2bfloat16(x[i]);
                        x[i] *= s.dtot[c0 + i];
                    }
                    tmem_st16(lane_addr + c0, x);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            // ---- in-block scores, exact: all 128 threads share the 136 (t, s <= t) pairs ----
            for (int pidx = tid; pidx < SC * (SC + 1) / 2; pidx += kThreads) {
                int t = 0, rem = pidx;
                while (rem > t) { rem -= t + 1; ++t; }      // pidx -> (t, s = rem), s <= t
                const int sidx = rem;
                float acc = 0.f;
                if (sidx < t) {
#pragma unroll 8
                    for (int i = 0; i < N; ++i)
                        acc += s.raw[0][t][i] * s.raw[1][sidx][i] * __expf(s.acum[t][i] - s.acum[sidx + 1][i]);
                } else if (rightward) {
#pragma unroll 8
                    for (int i = 0; i < N; ++i) acc += s.raw[0][t][i] * s.u[i] * s.raw[1][t][i];   // bonus
                }
                s.score[t][sidx] = acc;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            // ---- tensor core: read-out against the old state, then the update ----
            if (tid == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < N / 16; ++ks) {
                    const uint64_t da = make_desc(smem_u32(s.opS) + ks * 2 * (128 * 16), 128 * 16, 128);
                    const uint64_t db = make_desc(smem_u32(s.opR) + ks * 2 * (16 * 16), 16 * 16, 128);
                    umma_bf16(tmem + 64, da, db, instr_desc(128, 16), ks > 0 ? 1u : 0u);
                }
                {
                    const uint64_t da = make_desc(smem_u32(s.opV), 128 * 16, 128);
                    const uint64_t db = make_desc(smem_u32(s.opK), 64 * 16, 128);
                    umma_bf16(tmem, da, db, instr_desc(128, 64), 1u);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&s.bar))
                             : "memory");
            }
            // ---- meanwhile: in-block part of y for this thread's value channel ----
            float yin[SC];
            if (tid < N) {
#pragma unroll
                for (int t = 0; t < SC; ++t) {
                    float acc = 0.f;
#pragma unroll
                    for (int q = 0; q <= t; ++q) acc += s.score[t][q] * s.raw[2][q][tid];
                    yin[t] = acc;
                }
            }
            // ---- wait for the tensor core (bounded) ----
            if (!failed) {
                bool done = false;
                for (uint32_t i = 0; i < kWaitLimit; ++i) {
                    uint32_t ok;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0,1,0,p;\n\t}"
                        : "=r"(ok)
                        : "r"(smem_u32(&s.bar)), "r"(phase)
                        : "memory");
                    if (ok) { done = true; break; }
                    if (i > 32) __nanosleep(32);
                }
                if (!done) { failed = true; if (tid == 0) atomicExch(a.status, 1u); }
            }
            phase ^= 1u;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (tid < N) {
                float yt[16];
                tmem_ld16(lane_addr + 64, yt);
#pragma unroll
                for (int t = 0; t < SC; ++t) {
                    const int t_seq = blk * SC + t;
                    if (t_seq < T) {
                        const int tg = rightward ? t_seq : T - 1 - t_seq;
                        float* dst = a.y + base + static_cast<size_t>(tg) * C + tid;
                        const float val = yt[t] + yin[t];
                        if (rightward) *dst = val; else *dst += val;
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
        }
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
