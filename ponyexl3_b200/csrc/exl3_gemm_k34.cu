// Prefill GEMM kernels for K = 3 and K = 4 bits per weight (all codebooks).
#include "exl3_gemm2.cuh"

namespace exl3 {
template int launch_gemm_k<3>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
template int launch_gemm_k<4>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
}
