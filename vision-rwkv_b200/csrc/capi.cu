// C ABI of the library: argument validation, path selection, launch accounting.
// The contract of every function is stated in include/vrwkv_b200.h.
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include "vrwkv_b200.h"
#include "vrwkv_internal.h"

namespace {
std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_path{0};   // 0 auto (resident, else fused, else generic), 1 generic only, 2 skip the resident path

thread_local char g_detail[256] = "";   // per calling thread: no lock needed

inline bool misaligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) != 0; }

int check_shape(int B, int T, int C) {
    if (B <= 0 || T <= 0 || C <= 0) return VRWKV_ERR_SHAPE;
    if (B > 65535) return VRWKV_ERR_SHAPE;                       // gridDim.z
    if (static_cast<long long>(T) > 4000000LL) return VRWKV_ERR_SHAPE;
    return VRWKV_OK;
}

int finish(int launched) {
    if (launched < 0) { cudaGetLastError(); return VRWKV_ERR_DEVICE; }
    g_launches.fetch_add(static_cast<unsigned long long>(launched), std::memory_order_relaxed);
    const cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return VRWKV_OK;
    set_error_detail(cudaGetErrorName(err));
    return VRWKV_ERR_LAUNCH;
}
}  // namespace

void set_error_detail(const char* text) {
    std::strncpy(g_detail, text ? text : "", sizeof(g_detail) - 1);
    g_detail[sizeof(g_detail) - 1] = 0;
}

int record_launches(int launched) { return finish(launched); }

extern "C" {

int vrwkv_version(void) { return 100; }

const char* vrwkv_last_error_detail(void) { return g_detail; }

const char* vrwkv_status_string(int status) {
    switch (status) {
        case VRWKV_OK: return "ok";
        case VRWKV_ERR_SHAPE: return "bad shape: B, T, C must be positive, B <= 65535, T <= 4000000";
        case VRWKV_ERR_NULL: return "null pointer argument";
        case VRWKV_ERR_WORKSPACE: return "workspace smaller than the *_workspace_bytes value";
        case VRWKV_ERR_ALIGNMENT: return "pointer alignment: data 4 bytes (WKV6 inputs 16 bytes), workspace 256 bytes";
        case VRWKV_ERR_LAUNCH: return "CUDA reported an error after a kernel launch";
        case VRWKV_ERR_DEVICE: return "required driver entry point or device attribute unavailable";
        case VRWKV_ERR_HEAD_SIZE: return "WKV6 requires C == 64 * H";
        case VRWKV_ERR_UNSUPPORTED: return "shape or alignment not covered by this entry point's kernels; use the plain f32 entry points";
        default: return "unknown status";
    }
}

unsigned long long vrwkv_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int vrwkv_set_path(int path) {
    if (path < 0 || path > 3) return VRWKV_ERR_SHAPE;
    biwkv::resident::set_withhold_test(path == 3);
    g_path.store(path == 3 ? 0 : path);
    return VRWKV_OK;
}

int vrwkv_workspace_status(const void* workspace, void* stream, unsigned* status_out) {
    if (!workspace || !status_out) return VRWKV_ERR_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(status_out, workspace, sizeof(unsigned), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        cudaGetLastError();
        return VRWKV_ERR_LAUNCH;
    }
    return VRWKV_OK;
}

// The resident kernels' workspace; for sequences of several segments the chunked kernels' workspace follows it
// (they stand by for inputs outside the plain-float range and run only when the resident launch says so).
static size_t resident_offset(int B, int T, int C, bool bwd) {
    return (biwkv::resident::workspace_bytes(B, T, C, bwd) + 255) / 256 * 256;
}
static size_t resident_total(int B, int T, int C, bool bwd) {
    return resident_offset(B, T, C, bwd) + (biwkv::resident::multi_segment(T) ? biwkv::fused::workspace_bytes(B, T, C, bwd) : 0);
}

size_t vrwkv_biwkv_forward_workspace_bytes(int B, int T, int C) {
    if (check_shape(B, T, C) != VRWKV_OK) return 0;
    return std::max({biwkv::generic_forward_workspace(B, T, C) + 256, biwkv::fused::workspace_bytes(B, T, C, false),
                     resident_total(B, T, C, false)});
}

int vrwkv_biwkv_forward_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                            const float* v, float* y, void* workspace, size_t workspace_bytes,
                            void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !y || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || misaligned4(k) || misaligned4(v) || misaligned4(y) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_forward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool multi = biwkv::resident::multi_segment(T);
    if (g_path.load() == 0 && biwkv::resident::eligible(B, T, C, {k, v, y}, false) &&
        (!multi || biwkv::fused::eligible(B, T, C, {k, v, y}))) {
        int n = biwkv::resident::forward(B, T, C, w, u, k, v, y, workspace, s);
        if (n >= 0 && multi) {
            const int m = biwkv::fused::forward(B, T, C, w, u, k, v, y, static_cast<char*>(workspace) + resident_offset(B, T, C, false), s,
                                                static_cast<const unsigned*>(workspace) + 1);
            n = m < 0 ? m : n + m;
        }
        return finish(n);
    }
    if (g_path.load() != 1 && biwkv::fused::eligible(B, T, C, {k, v, y}))
        return finish(biwkv::fused::forward(B, T, C, w, u, k, v, y, workspace, s));
    // generic path: status word (first 256 bytes) is cleared, scratch follows
    cudaMemsetAsync(workspace, 0, 256, s);
    return finish(biwkv::generic_forward(B, T, C, w, u, k, v, y, static_cast<char*>(workspace) + 256, s));
}

size_t vrwkv_biwkv_backward_workspace_bytes(int B, int T, int C) {
    if (check_shape(B, T, C) != VRWKV_OK) return 0;
    return std::max({biwkv::generic_backward_workspace(B, T, C) + 256, biwkv::fused::workspace_bytes(B, T, C, true),
                     resident_total(B, T, C, true)});
}

int vrwkv_biwkv_backward_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                             const float* v, const float* gy, float* gwgu, float* gk, float* gv,
                             void* workspace, size_t workspace_bytes, void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !gy || !gwgu || !gk || !gv || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || misaligned4(k) || misaligned4(v) || misaligned4(gy) ||
        misaligned4(gwgu) || misaligned4(gk) || misaligned4(gv) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_backward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool multi = biwkv::resident::multi_segment(T);
    if (g_path.load() == 0 && biwkv::resident::eligible(B, T, C, {k, v, gy, gk, gv}, true) &&
        (!multi || biwkv::fused::eligible(B, T, C, {k, v, gy, gk, gv}))) {
        int n = biwkv::resident::backward(B, T, C, w, u, k, v, gy, gwgu, gk, gv, workspace, s);
        if (n >= 0 && multi) {
            const int m = biwkv::fused::backward(B, T, C, w, u, k, v, gy, gwgu, gk, gv,
                                                 static_cast<char*>(workspace) + resident_offset(B, T, C, true), s,
                                                 static_cast<const unsigned*>(workspace) + 1);
            n = m < 0 ? m : n + m;
        }
        return finish(n);
    }
    if (g_path.load() != 1 && biwkv::fused::eligible(B, T, C, {k, v, gy, gk, gv}))
        return finish(biwkv::fused::backward(B, T, C, w, u, k, v, gy, gwgu, gk, gv, workspace, s));
    cudaMemsetAsync(workspace, 0, 256, s);
    return finish(biwkv::generic_backward(B, T, C, w, u, k, v, gy, gwgu, gk, gv,
                                          static_cast<char*>(workspace) + 256, s));
}

int vrwkv_biwkv_forward_save_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                                 const float* v, float* y, float* logden, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !y || !logden || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_forward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    if (!biwkv::fused::eligible(B, T, C, {k, v, y, logden})) return VRWKV_ERR_UNSUPPORTED;
    return finish(biwkv::fused::forward_save(B, T, C, w, u, k, v, y, logden, workspace, static_cast<cudaStream_t>(stream)));
}

int vrwkv_biwkv_backward_saved_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                                   const float* v, const float* gy, const float* y, const float* logden,
                                   float* gwgu, float* gk, float* gv, void* workspace,
                                   size_t workspace_bytes, void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !gy || !y || !logden || !gwgu || !gk || !gv || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || misaligned4(gwgu) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_backward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    if (!biwkv::fused::eligible_saved(B, T, C, {k, v, gy, y, logden, gk, gv})) return VRWKV_ERR_UNSUPPORTED;
    return finish(biwkv::fused::backward_saved(B, T, C, w, u, k, v, gy, y, logden, gwgu, gk, gv, workspace,
                                               static_cast<cudaStream_t>(stream)));
}

int vrwkv_biwkv_forward_bf16(int B, int T, int C, const float* w, const float* u, const uint16_t* k,
                             const uint16_t* v, uint16_t* y, void* workspace, size_t workspace_bytes,
                             void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !y || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_forward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    const bool multi = biwkv::resident::multi_segment(T);
    if (g_path.load() == 0 && biwkv::resident::eligible(B, T, C, {k, v, y}, false, true) &&
        (!multi || biwkv::fused::eligible(B, T, C, {k, v, y}, true))) {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        int n = biwkv::resident::forward_bf16(B, T, C, w, u, k, v, y, workspace, s);
        if (n >= 0 && multi) {
            const int m = biwkv::fused::forward_bf16(B, T, C, w, u, k, v, y, static_cast<char*>(workspace) + resident_offset(B, T, C, false), s,
                                                     static_cast<const unsigned*>(workspace) + 1);
            n = m < 0 ? m : n + m;
        }
        return finish(n);
    }
    if (!biwkv::fused::eligible(B, T, C, {k, v, y}, true)) return VRWKV_ERR_UNSUPPORTED;
    return finish(biwkv::fused::forward_bf16(B, T, C, w, u, k, v, y, workspace, static_cast<cudaStream_t>(stream)));
}

int vrwkv_biwkv_backward_bf16(int B, int T, int C, const float* w, const float* u, const uint16_t* k,
                              const uint16_t* v, const uint16_t* gy, float* gwgu, uint16_t* gk,
                              uint16_t* gv, void* workspace, size_t workspace_bytes, void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !gy || !gwgu || !gk || !gv || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || misaligned4(gwgu) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_backward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    const bool multi = biwkv::resident::multi_segment(T);
    if (g_path.load() == 0 && biwkv::resident::eligible(B, T, C, {k, v, gy, gk, gv}, true, true) &&
        (!multi || biwkv::fused::eligible(B, T, C, {k, v, gy, gk, gv}, true))) {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        int n = biwkv::resident::backward_bf16(B, T, C, w, u, k, v, gy, gwgu, gk, gv, workspace, s);
        if (n >= 0 && multi) {
            const int m = biwkv::fused::backward_bf16(B, T, C, w, u, k, v, gy, gwgu, gk, gv,
                                                      static_cast<char*>(workspace) + resident_offset(B, T, C, true), s,
                                                      static_cast<const unsigned*>(workspace) + 1);
            n = m < 0 ? m : n + m;
        }
        return finish(n);
    }
    if (!biwkv::fused::eligible(B, T, C, {k, v, gy, gk, gv}, true)) return VRWKV_ERR_UNSUPPORTED;
    return finish(biwkv::fused::backward_bf16(B, T, C, w, u, k, v, gy, gwgu, gk, gv, workspace,
                                              static_cast<cudaStream_t>(stream)));
}

// ---- WKV6 ---------------------------------------------------------------------------------------
static int check_wkv6(int B, int T, int C, int H) {
    if (B <= 0 || T <= 0 || C <= 0 || H <= 0) return VRWKV_ERR_SHAPE;
    if (C != 64 * H) return VRWKV_ERR_HEAD_SIZE;
    if (static_cast<long long>(B) * H > 1000000000LL || T > 4000000) return VRWKV_ERR_SHAPE;   // 2*B*H is a grid dimension
    return VRWKV_OK;
}
static inline bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

size_t vrwkv_wkv6_backward_workspace_bytes(int B, int T, int C, int H) {
    if (check_wkv6(B, T, C, H) != VRWKV_OK) return 0;
    return wkv6::backward_workspace(B, T, H);
}

int vrwkv_wkv6_forward_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                           const float* w_raw, const float* u, float* y, void* stream) {
    if (int st = check_wkv6(B, T, C, H)) return st;
    if (!r || !k || !v || !w_raw || !u || !y) return VRWKV_ERR_NULL;
    if (misaligned16(r) || misaligned16(k) || misaligned16(v) || misaligned16(w_raw) || misaligned4(u) ||
        misaligned4(y))
        return VRWKV_ERR_ALIGNMENT;
    return finish(wkv6::forward(B, T, H, r, k, v, w_raw, u, y, static_cast<cudaStream_t>(stream)));
}

int vrwkv_wkv6_forward_tc_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                              const float* w_raw, const float* u, float* y, void* workspace,
                              size_t workspace_bytes, void* stream) {
    if (int st = check_wkv6(B, T, C, H)) return st;
    if (!r || !k || !v || !w_raw || !u || !y || !workspace) return VRWKV_ERR_NULL;
    if (misaligned16(r) || misaligned16(k) || misaligned16(v) || misaligned16(w_raw) || misaligned4(u) ||
        misaligned16(y) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < 256) return VRWKV_ERR_WORKSPACE;
    return finish(wkv6tc::forward(B, T, H, r, k, v, w_raw, u, y, static_cast<unsigned*>(workspace),
                                  g_path.load() != 1, static_cast<cudaStream_t>(stream)));
}

int vrwkv_wkv6_forward_tc_bf16(int B, int T, int C, int H, const uint16_t* r, const uint16_t* k,
                               const uint16_t* v, const float* w_raw, const float* u, float* y,
                               void* workspace, size_t workspace_bytes, void* stream) {
    if (int st = check_wkv6(B, T, C, H)) return st;
    if (!r || !k || !v || !w_raw || !u || !y || !workspace) return VRWKV_ERR_NULL;
    if (misaligned16(r) || misaligned16(k) || misaligned16(v) || misaligned16(w_raw) || misaligned4(u) ||
        misaligned16(y) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < 256) return VRWKV_ERR_WORKSPACE;
    return finish(wkv6tc::forward_bf16in(B, T, H, r, k, v, w_raw, u, y, static_cast<unsigned*>(workspace),
                                         static_cast<cudaStream_t>(stream)));
}

int vrwkv_wkv6_backward_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                            const float* w_raw, const float* u, const float* gy, float* gr, float* gk,
                            float* gv, float* gw, float* gu, void* workspace, size_t workspace_bytes,
                            void* stream) {
    if (int st = check_wkv6(B, T, C, H)) return st;
    if (!r || !k || !v || !w_raw || !u || !gy || !gr || !gk || !gw || !gu || !workspace)      // gv may be NULL
        return VRWKV_ERR_NULL;
    if (misaligned16(r) || misaligned16(k) || misaligned16(v) || misaligned16(w_raw) || misaligned16(gy) ||
        misaligned4(u) || misaligned4(gr) || misaligned4(gk) || misaligned4(gv) || misaligned4(gw) ||
        misaligned4(gu) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < wkv6::backward_workspace(B, T, H)) return VRWKV_ERR_WORKSPACE;
    return finish(wkv6::backward(B, T, H, r, k, v, w_raw, u, gy, gr, gk, gv, gw, gu, workspace,
                                 static_cast<cudaStream_t>(stream)));
}

size_t vrwkv_wkv6_backward_tc_workspace_bytes(int B, int T, int C, int H) {
    if (check_wkv6(B, T, C, H) != VRWKV_OK) return 0;
    return wkv6tc::backward_workspace(B, T, H);
}

static int wkv6_backward_tc(int B, int T, int C, int H, const void* r, const void* k, const void* v, const float* w_raw,
                            const float* u, const void* gy, float* gr, float* gk, float* gv, float* gw, float* gu,
                            void* workspace, size_t workspace_bytes, void* stream, bool half_in) {
    if (int st = check_wkv6(B, T, C, H)) return st;
    if (!r || !k || !v || !w_raw || !u || !gy || !gr || !gk || !gv || !gw || !gu || !workspace) return VRWKV_ERR_NULL;
    if (misaligned16(r) || misaligned16(k) || misaligned16(v) || misaligned16(w_raw) || misaligned16(gy) || misaligned4(u) ||
        misaligned16(gr) || misaligned16(gk) || misaligned16(gv) || misaligned4(gw) || misaligned4(gu) ||
        (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < wkv6tc::backward_workspace(B, T, H)) return VRWKV_ERR_WORKSPACE;
    return finish(wkv6tc::backward(B, T, H, r, k, v, w_raw, u, gy, gr, gk, gv, gw, gu, workspace, half_in,
                                   static_cast<cudaStream_t>(stream)));
}

int vrwkv_wkv6_backward_tc_f32(int B, int T, int C, int H, const float* r, const float* k, const float* v,
                               const float* w_raw, const float* u, const float* gy, float* gr, float* gk, float* gv,
                               float* gw, float* gu, void* workspace, size_t workspace_bytes, void* stream) {
    return wkv6_backward_tc(B, T, C, H, r, k, v, w_raw, u, gy, gr, gk, gv, gw, gu, workspace, workspace_bytes, stream, false);
}

int vrwkv_wkv6_backward_tc_bf16(int B, int T, int C, int H, const uint16_t* r, const uint16_t* k, const uint16_t* v,
                                const float* w_raw, const float* u, const uint16_t* gy, float* gr, float* gk, float* gv,
                                float* gw, float* gu, void* workspace, size_t workspace_bytes, void* stream) {
    return wkv6_backward_tc(B, T, C, H, r, k, v, w_raw, u, gy, gr, gk, gv, gw, gu, workspace, workspace_bytes, stream, true);
}

}  // extern "C"
