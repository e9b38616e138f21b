// Large-batch DLR-Net forward, streamed path on CTA pairs (see stream_pair.cu).
#pragma once
#include <cuda_runtime.h>

#include "cluster.h"

namespace dlr {

bool stream_pair_supported(int d, int r);
int stream_pair_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan);
int stream_pair_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                        int L, float eps, int* status_dev, cudaStream_t stream, int num_sms, int smem_optin,
                        unsigned int spin_limit, unsigned long long* prof);

}  // namespace dlr
