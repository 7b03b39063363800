// Empty stand-in: the reference's wkv6_cuda.cu includes "ATen/ATen.h" but uses nothing from
// it, so the kernels can be compiled for the oracle without pulling in torch headers.
