// C ABI of the library: argument validation, path selection, launch accounting.
// The contract of every function is stated in include/vrwkv_b200.h.
#include <atomic>
#include <cstdint>
#include "vrwkv_b200.h"
#include "vrwkv_internal.h"

namespace {
std::atomic<unsigned long long> g_launches{0};

inline bool misaligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) != 0; }

int check_shape(int B, int T, int C) {
    if (B <= 0 || T <= 0 || C <= 0) return VRWKV_ERR_SHAPE;
    if (B > 65535) return VRWKV_ERR_SHAPE;                       // gridDim.z
    if (static_cast<long long>(T) > 4000000LL) return VRWKV_ERR_SHAPE;
    return VRWKV_OK;
}

int finish(int launched) {
    g_launches.fetch_add(static_cast<unsigned long long>(launched), std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? VRWKV_OK : VRWKV_ERR_LAUNCH;
}
}  // namespace

extern "C" {

int vrwkv_version(void) { return 100; }

const char* vrwkv_status_string(int status) {
    switch (status) {
        case VRWKV_OK: return "ok";
        case VRWKV_ERR_SHAPE: return "bad shape: B, T, C must be positive, B <= 65535, T <= 4000000";
        case VRWKV_ERR_NULL: return "null pointer argument";
        case VRWKV_ERR_WORKSPACE: return "workspace smaller than the *_workspace_bytes value";
        case VRWKV_ERR_ALIGNMENT: return "pointer not aligned to 4 bytes";
        case VRWKV_ERR_LAUNCH: return "CUDA reported an error after a kernel launch";
        case VRWKV_ERR_DEVICE: return "required driver entry point or device attribute unavailable";
        case VRWKV_ERR_HEAD_SIZE: return "WKV6 requires C == 64 * H";
        default: return "unknown status";
    }
}

unsigned long long vrwkv_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t vrwkv_biwkv_forward_workspace_bytes(int B, int T, int C) {
    if (check_shape(B, T, C) != VRWKV_OK) return 0;
    return biwkv::generic_forward_workspace(B, T, C);
}

int vrwkv_biwkv_forward_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                            const float* v, float* y, void* workspace, size_t workspace_bytes,
                            void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !y || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || misaligned4(k) || misaligned4(v) || misaligned4(y) ||
        misaligned4(workspace))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_forward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    return finish(biwkv::generic_forward(B, T, C, w, u, k, v, y, workspace,
                                         static_cast<cudaStream_t>(stream)));
}

size_t vrwkv_biwkv_backward_workspace_bytes(int B, int T, int C) {
    if (check_shape(B, T, C) != VRWKV_OK) return 0;
    return biwkv::generic_backward_workspace(B, T, C);
}

int vrwkv_biwkv_backward_f32(int B, int T, int C, const float* w, const float* u, const float* k,
                             const float* v, const float* gy, float* gwgu, float* gk, float* gv,
                             void* workspace, size_t workspace_bytes, void* stream) {
    if (int st = check_shape(B, T, C)) return st;
    if (!w || !u || !k || !v || !gy || !gwgu || !gk || !gv || !workspace) return VRWKV_ERR_NULL;
    if (misaligned4(w) || misaligned4(u) || misaligned4(k) || misaligned4(v) || misaligned4(gy) ||
        misaligned4(gwgu) || misaligned4(gk) || misaligned4(gv) || misaligned4(workspace))
        return VRWKV_ERR_ALIGNMENT;
    if (workspace_bytes < vrwkv_biwkv_backward_workspace_bytes(B, T, C)) return VRWKV_ERR_WORKSPACE;
    return finish(biwkv::generic_backward(B, T, C, w, u, k, v, gy, gwgu, gk, gv, workspace,
                                          static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
