// Host-side dispatch of the prefill GEMM over K; the kernel template (exl3_gemm.cuh) is
// instantiated in exl3_gemm_k12.cu .. exl3_gemm_k78.cu.
#include "exl3_internal.h"

namespace exl3 {

int g_gemm_one_acc_rows = 128;
int g_gemm_split_last_wave = 1;
void gemm_set_tuning(int one_acc_rows)
{
    g_gemm_one_acc_rows = (one_acc_rows & 255) == 0 ? 0 : 128;
    g_gemm_split_last_wave = (one_acc_rows & 256) ? 0 : 1;     // + 256: whole tiles only
}
// Off: measured on 8192 x 5120 x 5120 the pair kernel is at 0.43 ms against 0.40 ms (see exl3_gemm2.cuh).
int g_gemm_pairs = 0;
void gemm_set_pairs(int on) { g_gemm_pairs = on ? 1 : 0; }

template <int K>
int launch_gemm_k(const GemmArgs& a, int cb, const __half* xh, const uint32_t* trellis, cudaStream_t s);
#define EXL3_DECL(K) \
    extern template int launch_gemm_k<K>(const GemmArgs&, int, const __half*, const uint32_t*, cudaStream_t);
EXL3_DECL(1) EXL3_DECL(2) EXL3_DECL(3) EXL3_DECL(4) EXL3_DECL(5) EXL3_DECL(6) EXL3_DECL(7) EXL3_DECL(8)
#undef EXL3_DECL

int launch_gemm(const GemmArgs& a, int k, int cb, const __half* xh, const uint32_t* trellis,
                cudaStream_t s)
{
    switch (k) {
        case 1: return launch_gemm_k<1>(a, cb, xh, trellis, s);
        case 2: return launch_gemm_k<2>(a, cb, xh, trellis, s);
        case 3: return launch_gemm_k<3>(a, cb, xh, trellis, s);
        case 4: return launch_gemm_k<4>(a, cb, xh, trellis, s);
        case 5: return launch_gemm_k<5>(a, cb, xh, trellis, s);
        case 6: return launch_gemm_k<6>(a, cb, xh, trellis, s);
        case 7: return launch_gemm_k<7>(a, cb, xh, trellis, s);
        case 8: return launch_gemm_k<8>(a, cb, xh, trellis, s);
        default: return EXL3_E_K;
    }
}

}  // namespace exl3
