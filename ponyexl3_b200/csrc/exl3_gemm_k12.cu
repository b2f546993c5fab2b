// Prefill GEMM kernels for K = 1 and K = 2 bits per weight (all codebooks).
#include "exl3_gemm2.cuh"

namespace exl3 {
template int launch_gemm_k<1>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
template int launch_gemm_k<2>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
}
