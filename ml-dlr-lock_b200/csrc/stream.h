// Large-batch DLR-Net forward, streamed path (see stream.cu).
#pragma once
#include <cuda_runtime.h>

#include "cluster.h"

namespace dlr {

bool stream_supported(int d, int r);
bool stream_aligned(const void* x, const void* y);
int stream_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan);
size_t stream_workspace_bytes(int M, int d, int r);
int stream_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                   int L, float eps, void* workspace, int* status_dev, cudaStream_t stream, int num_sms, int smem_optin,
                   unsigned int spin_limit, unsigned long long* prof);

}  // namespace dlr
