/* Plain-C restatement of the DLR-Net forward.  TEST INFRASTRUCTURE ONLY: it is
 * built by oracle/build_oracle.py and called from the tests to cross-check the
 * torch oracle (oracle/dlrnet_oracle.py) with code that shares nothing with
 * torch.  Nothing in the shipped package links or calls it.
 *
 * Follows the reference layer loop, dlr_lock/model.py:93-101:
 *   ms  = mean(h^2)                       (:96)
 *   inp = h * w_i * rsqrt(ms + eps)       (:97)
 *   z   = inp . V_i^T                     (:98)   V_i is (r, d)
 *   dh  = silu(z) . U_i^T                 (:99)   U_i is (d, r)
 *   h   = h + alpha_i * dh                (:100)
 * All inputs are fp32 arrays; sums are carried in double so that the result
 * does not depend on summation order to fp32 precision.
 * Parity pin: compared in tests/test_oracle_golden.py against the fp32 outputs
 * of the real reference stored under tests/golden/.
 */
#include <math.h>
#include <stdlib.h>

int dlrnet_forward_f32(const float* x, float* y, const float* V, const float* U, const float* w,
                       const float* alpha, int M, int d, int r, int L, float eps) {
    double* h = (double*)malloc(sizeof(double) * (size_t)d);
    double* inp = (double*)malloc(sizeof(double) * (size_t)d);
    double* s = (double*)malloc(sizeof(double) * (size_t)r);
    if (!h || !inp || !s) {
        free(h); free(inp); free(s);
        return 1;
    }
    for (int m = 0; m < M; ++m) {
        for (int j = 0; j < d; ++j) h[j] = x[(size_t)m * d + j];
        for (int i = 0; i < L; ++i) {
            const float* Vi = V + (size_t)i * r * d;
            const float* Ui = U + (size_t)i * d * r;
            const float* wi = w + (size_t)i * d;
            double ms = 0.0;
            for (int j = 0; j < d; ++j) ms += h[j] * h[j];
            const double rstd = 1.0 / sqrt(ms / d + (double)eps);
            for (int j = 0; j < d; ++j) inp[j] = h[j] * wi[j] * rstd;
            for (int k = 0; k < r; ++k) {
                double z = 0.0;
                for (int j = 0; j < d; ++j) z += inp[j] * Vi[(size_t)k * d + j];
                s[k] = z / (1.0 + exp(-z));
            }
            for (int j = 0; j < d; ++j) {
                double dh = 0.0;
                for (int k = 0; k < r; ++k) dh += s[k] * Ui[(size_t)j * r + k];
                h[j] += (double)alpha[i] * dh;
            }
        }
        for (int j = 0; j < d; ++j) y[(size_t)m * d + j] = (float)h[j];
    }
    free(h); free(inp); free(s);
    return 0;
}
