// Internal interface between the C-ABI layer and the large-batch kernel.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/dlr_b200.h"

namespace dlr {

// Encode a 2-D bf16 tensor map (inner = contiguous dimension).  `encode_fn_ptr`
// is the driver's cuTensorMapEncodeTiled entry point.
bool encode_2d_bf16(void* encode_fn_ptr, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                    int box_inner, int box_outer, int swizzle_bytes);

bool cluster_supported(int d, int r, int L);
size_t cluster_workspace_bytes(int M, int d, int r, int L);
int cluster_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan);
int cluster_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d,
                    int r, int L, float eps, void* workspace, int* status_dev, cudaStream_t stream, int num_sms,
                    int smem_optin, unsigned int spin_limit);

}  // namespace dlr
