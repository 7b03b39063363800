// Host-side construction of tiled TMA descriptors for (B, T, C) fp32 tensors, seen by the copy
// engine as a 3-D array with C innermost.  The driver entry point is looked up through the
// runtime, so nothing links against libcuda directly.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace tensor_map {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// cuTensorMapEncodeTiled needs a current context; a host thread that has made no runtime call that creates one
// (a fresh worker thread) binds the primary context here, once per thread.  Not repeated per call: an allocator
// call is not allowed while a stream is being captured into a graph.
inline void bind_primary_context() {
    thread_local bool bound = false;
    if (!bound) {
        cudaFree(nullptr);
        bound = true;
    }
}

// Box of box_c channels x box_t tokens of one batch entry; out-of-range elements load as zero and
// are clipped on store.  `base` must be 16-byte aligned and the row pitch C * elem_bytes a multiple
// of 16 (C % 4 == 0 for float, C % 8 == 0 for bfloat16).
inline bool make_btc(CUtensorMap* map, const void* base, int B, int T, int C, int box_c, int box_t, bool bf16) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t eb = bf16 ? 2 : 4;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(C) * eb, static_cast<cuuint64_t>(T) * C * eb};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_c), static_cast<cuuint32_t>(box_t), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base),
              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
inline bool make_btc_f32(CUtensorMap* map, const float* base, int B, int T, int C, int box_c, int box_t) {
    return make_btc(map, base, B, T, C, box_c, box_t, false);
}

}  // namespace tensor_map
