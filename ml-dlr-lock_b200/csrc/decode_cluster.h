// Internal interface between the C-ABI layer and the cluster small-batch kernel.
#pragma once

#include <cuda_runtime.h>

#include "../../include/dlr_b200.h"

namespace dlr {

bool decode_cluster_supported(int d, int r);
int decode_cluster_plan(int M, int d, int r, int L, int smem_optin, dlrb200_plan* plan);
int decode_cluster_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d,
                           int r, int L, float eps, int* status_dev, cudaStream_t stream, int smem_optin,
                           unsigned int spin_limit, unsigned long long* prof);

}  // namespace dlr
