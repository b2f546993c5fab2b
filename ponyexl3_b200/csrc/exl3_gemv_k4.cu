// Streamed GEMV kernels for K = 4 bits per weight (all codebooks, row groups and modes).
#include "exl3_gemv.cuh"

namespace exl3 {
template int launch_gemv_k<4>(const GemvArgs&, int, bool, cudaStream_t);
}
