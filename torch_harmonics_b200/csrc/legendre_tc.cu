// Legendre contraction on the tcgen05 tensor cores (placeholder until the kernel lands).
#include "common.cuh"

namespace shtb200 {

bool gemm_tc_supported(const Plan &, const GemmParams &) { return false; }

int launch_gemm_tc(const Plan &, const GemmParams &, cudaStream_t) { return fail(SHTB200_EINVAL, "tcgen05 engine not available in this build"); }

}  // namespace shtb200
