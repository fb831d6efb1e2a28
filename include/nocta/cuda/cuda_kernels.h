/* Forwarding header: the kernel ABI that replaces the reference's nocta/cuda/cuda_kernels.h. */
#ifndef NOCTA_FWD_CUDA_CUDA_KERNELS_H
#define NOCTA_FWD_CUDA_CUDA_KERNELS_H
#include "../../nocta_cuda.h"
#endif
