// Stand-in for <THC/THCAtomics.cuh>, for the oracle only: the reference's bi_wkv_kernel.cu uses
// atomicAdd on float, which the device provides natively.
#pragma once
