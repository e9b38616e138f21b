// Internal interface between the C-ABI layer and the small-batch kernel with the two-level exchange
// (see decode_tl.cu).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/dlr_b200.h"

namespace dlr {

struct DecodeTLParams {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int M;                        // rows, 1..64
    int d;
    int L;
    float eps;
    float inv_d;
    unsigned long long* words;    // [L][padded rows][r + 4] accumulator words, zero on entry
    float* pre;                   // [CTAs][64] sums of squares of the input per CTA
    unsigned int* counter;        // zero on entry
    int* status;                  // device status word, untouched unless a wait gives up
    unsigned int spin_limit;
    int stages;                   // filled by the launcher
};

struct DecodeTLLaunch {
    DecodeTLParams p;
    CUtensorMap tmV;              // over V' viewed as (L*r, d)
    CUtensorMap tmU;              // over U' viewed as (L*d, r)
    int d, r, L, dc;
    int num_sms;
    int smem_optin;
    cudaStream_t stream;
};

bool decode_tl_supported(int d, int r, int dc);
size_t decode_tl_workspace_bytes(int M, int r, int L);
size_t decode_tl_clear_bytes(int M, int r, int L);
// plan_only: fill the plan and launch nothing
int decode_tl_launch(const DecodeTLLaunch& a, dlrb200_plan* plan_only);

}  // namespace dlr
