// C-callable doorway to the reference's own Bi-WKV kernels, for the oracle only.
// REF_SOURCE is the path of classification/mae/vrwkv/cuda/wkv_cuda.cu inside the reference
// checkout; it is compiled where it lies (see build_ref.py), nothing of it is copied here.
#include REF_SOURCE

extern "C" void ref_biwkv_forward(int B, int T, int C, float* w, float* u, float* k, float* v, float* y) {
    cuda_forward(B, T, C, w, u, k, v, y);
}
extern "C" void ref_biwkv_backward(int B, int T, int C, float* w, float* u, float* k, float* v, float* gy,
                                   float* gw, float* gu, float* gk, float* gv) {
    cuda_backward(B, T, C, w, u, k, v, gy, gw, gu, gk, gv);
}
extern "C" int ref_biwkv_tmax(void) { return Tmax; }
