// C-callable doorway to the Bi-WKV kernels the four live backbones of the reference load
// (classification/mmcls_custom/models/backbones/cuda_new/bi_wkv_kernel.cu), for the oracle only.
// REF_SOURCE is that file inside the reference checkout; it is compiled where it lies, against the
// stand-in headers under ref_stubs/ (see build_ref.py); nothing of it is copied here.
#include REF_SOURCE

// Only the gradient kernel is exported.  The file's forward kernel combines its token segments with
// __shfl_sync(0xffffffff, ...) inside loops whose trip count differs per lane (:71-77, :82-88), which CUDA leaves
// undefined; it is not run from here.
extern "C" void ref_biwkv_live_backward(int B, int T, int C, float* w, float* u, float* k, float* v, float* gy,
                                        float* gw, float* gu, float* gk, float* gv) {
    std::vector<torch::Tensor> g = bi_wkv_cuda_backward(torch::wrap(w, C), torch::wrap(u, C), torch::wrap(k, B, T, C),
                                                        torch::wrap(v, B, T, C), torch::wrap(gy, B, T, C));
    const size_t n = sizeof(float) * static_cast<size_t>(B) * T * C;
    cudaMemcpy(gw, g[0].ptr, sizeof(float) * C, cudaMemcpyDeviceToDevice);
    cudaMemcpy(gu, g[1].ptr, sizeof(float) * C, cudaMemcpyDeviceToDevice);
    cudaMemcpy(gk, g[2].ptr, n, cudaMemcpyDeviceToDevice);
    cudaMemcpy(gv, g[3].ptr, n, cudaMemcpyDeviceToDevice);
}
