#include "cluster.h"
namespace dlr {
bool cluster_supported(int, int, int) { return false; }
size_t cluster_workspace_bytes(int, int, int, int) { return 0; }
int cluster_plan(int, int, int, int, int, int, dlrb200_plan*) { return DLRB200_ERR_UNSUPPORTED_SHAPE; }
int cluster_forward(void*, const void*, void*, const void*, const void*, int, int, int, int, float, void*, int*,
                    cudaStream_t, int, int, unsigned int) { return DLRB200_ERR_UNSUPPORTED_SHAPE; }
}
