// Prefill GEMM kernels for K = 7 and K = 8 bits per weight (all codebooks).
#include "exl3_gemm2.cuh"

namespace exl3 {
template int launch_gemm_k<7>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
template int launch_gemm_k<8>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
}
