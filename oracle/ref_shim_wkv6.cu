// C-callable doorway to the reference's own WKV6 kernels, for the oracle only.
// REF_SOURCE is the path of classification/mmcls_custom/models/backbones/cuda_v6/wkv6_cuda.cu
// inside the reference checkout; compiled where it lies, nothing of it is copied here.
#include REF_SOURCE

extern "C" void ref_wkv6_forward(int B, int T, int C, int H, float* r, float* k, float* v, float* ew, float* u,
                                 float* y) {
    cuda_forward(B, T, C, H, r, k, v, ew, u, y);
}
extern "C" void ref_wkv6_backward(int B, int T, int C, int H, float* r, float* k, float* v, float* ew, float* u,
                                  float* gy, float* gr, float* gk, float* gv, float* gw, float* gu) {
    cuda_backward(B, T, C, H, r, k, v, ew, u, gy, gr, gk, gv, gw, gu);
}
extern "C" int ref_wkv6_tmax(void) { return _T_; }
