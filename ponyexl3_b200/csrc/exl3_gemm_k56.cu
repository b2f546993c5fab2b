// Prefill GEMM kernels for K = 5 and K = 6 bits per weight (all codebooks).
#include "exl3_gemm2.cuh"

namespace exl3 {
template int launch_gemm_k<5>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
template int launch_gemm_k<6>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
}
