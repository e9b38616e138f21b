// Internal interface between the C-ABI layer and the small-batch kernel.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/dlr_b200.h"

namespace dlr {

struct DecodeParams {
    const __nv_bfloat16* x;   // first row of this pass, row stride d
    __nv_bfloat16* y;
    int M;                    // rows in this pass, 1..64
    int d;
    int L;
    float eps;
    float inv_d;
    float* zacc;              // 3 slots x 64 rows x (r+4) floats, zero on entry
    unsigned int* counter;    // zero on entry
    int* status;              // device status word, untouched unless a wait gives up
    unsigned int spin_limit;
    int stages;               // filled by the launcher
};

struct DecodeLaunch {
    DecodeParams p;
    CUtensorMap tmV;          // over V' viewed as (L*r, d)
    CUtensorMap tmU;          // over U' viewed as (L*d, r)
    int d, r, L, dc;
    int num_sms;
    int smem_optin;           // cudaDevAttrMaxSharedMemoryPerBlockOptin
    int max_stages;           // 0 = as many as fit
    cudaStream_t stream;
};

size_t decode_zacc_floats(int r);
bool decode_box_dims(int r, int dc, int* v_box_cols, int* v_box_rows, int* u_box_cols, int* u_box_rows,
                     int* v_swizzle_bytes, int* u_swizzle_bytes);
int decode_launch(const DecodeLaunch& a);

}  // namespace dlr
