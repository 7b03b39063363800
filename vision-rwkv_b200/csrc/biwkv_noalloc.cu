// Bi-WKV forward for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or torch's allocator) around a
// launch: code running inside a region where allocation is forbidden or would deadlock
// (a CUDA-graph capture in progress on another stream of the process, a real-time
// inference loop with a frozen memory plan, a plugin whose host application owns all
// device memory and hands out only the input and output buffers).  The regular entry
// points ask such a caller for a workspace it cannot provide.  This one brings its own:
// the scratch of the generic forward kernels lives in a fixed array in the library's
// device image, below.  The array exists once per GPU that loads the library, for the
// life of the process, which is why it is kept to a modest 16 MiB and why larger problems
// are refused rather than served.
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include "vrwkv_b200.h"
#include "vrwkv_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;

// Scratch shared by every call on this device.  In host code this name is only a handle
// for cudaGetSymbolAddress; the kernels get the device address resolved from it below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};

// Resolve the device address of the scratch array for the current device, once.
int scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        set_error_detail("no-alloc forward: cannot identify the current CUDA device");
        return VRWKV_ERR_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[dev] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (err != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            set_error_detail(err != cudaSuccess ? cudaGetErrorName(err)
                                                : "cudaGetSymbolAddress returned a null address");
            return VRWKV_ERR_DEVICE;
        }
        g_scratch_address[dev] = ptr;
    }
    *out = g_scratch_address[dev];
    return VRWKV_OK;
}

}  // namespace

extern "C" int vrwkv_biwkv_forward_f32_noalloc(int B, int T, int C, const float* w, const float* u,
                                               const float* k, const float* v, float* y, void* stream) {
    if (B <= 0 || T <= 0 || C <= 0 || B > 65535 || T > 4000000) return VRWKV_ERR_SHAPE;
    if (!w || !u || !k || !v || !y) return VRWKV_ERR_NULL;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(u) |
                           reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                           reinterpret_cast<uintptr_t>(y);
    if (bits & 3u) return VRWKV_ERR_ALIGNMENT;
    const size_t need = biwkv::generic_forward_workspace(B, T, C);
    if (need > kStaticScratchBytes) {
        char msg[200];
        std::snprintf(msg, sizeof(msg),
                      "no-alloc forward: this shape needs %zu bytes of scratch, the built-in array holds %zu",
                      need, kStaticScratchBytes);
        set_error_detail(msg);
        return VRWKV_ERR_WORKSPACE;
    }
    void* scratch = nullptr;
    if (int st = scratch_for_current_device(&scratch)) return st;
    // Every scratch element the kernels read is written earlier in the same call, so nothing
    // left over from the previous call needs clearing.
    const int launched = biwkv::generic_forward(B, T, C, w, u, k, v, y, scratch, static_cast<cudaStream_t>(stream));
    return record_launches(launched);
}
