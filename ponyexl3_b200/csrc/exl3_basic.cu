// Codec kernels outside the matmul: tile unpack, full decode to fp16 (the
// bit-exact test target), the codebook table, and the stand-alone Hadamard-128
// rotation.  All are HBM-trivial; the matmul kernels reuse the same device
// functions, so a bit-exact decode here proves the arithmetic they run.
#include "exl3_internal.h"

namespace exl3 {

// ---- unpack: one warp per tile ------------------------------------------------------------
template <int K>
__global__ void __launch_bounds__(256) unpack_kernel(const uint32_t* __restrict__ trellis,
                                                     int64_t n_tiles, uint16_t* __restrict__ out)
{
    const int lane = threadIdx.x & 31;
    LaneWords<K> lw;
    lw.init(lane);
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t tile = warp0; tile < n_tiles; tile += nwarps) {
        const uint32_t* w = trellis + tile * (8 * K);
        uint32_t cw[8];
        lane_codewords<K>(w[lw.i0], w[lw.i1], LaneWords<K>::kThree ? w[lw.i2] : 0u, lw.sh, cw);
        uint4 v;
        v.x = cw[0] | (cw[1] << 16);
        v.y = cw[2] | (cw[3] << 16);
        v.z = cw[4] | (cw[5] << 16);
        v.w = cw[6] | (cw[7] << 16);
        reinterpret_cast<uint4*>(out + tile * 256)[lane] = v;
    }
}

// ---- decode: one warp per tile, fp16 W written at its matrix position ------------------------
template <int K, int CB>
__global__ void __launch_bounds__(256)
    decode_kernel(const uint32_t* __restrict__ trellis, int64_t t_in, int64_t t_out, int64_t tn0,
                  int64_t tn_count, __half* __restrict__ w, int64_t ld)
{
    const int lane = threadIdx.x & 31;
    LaneWords<K> lw;
    lw.init(lane);
    const int64_t warp0 = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t n_tiles = t_in * tn_count;
    for (int64_t i = warp0; i < n_tiles; i += nwarps) {
        const int64_t tk = i / tn_count, tl = i % tn_count;
        const uint32_t* p = trellis + (tk * t_out + tn0 + tl) * (8 * K);
        uint32_t cw[8];
        lane_codewords<K>(p[lw.i0], p[lw.i1], LaneWords<K>::kThree ? p[lw.i2] : 0u, lw.sh, cw);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            const __half2 v = u32_as_h2(decode_pair<CB>(cw[j], cw[j + 1]));
            __half* dst = w + (tk * 16) * ld + tl * 16;
            dst[(int64_t)frag_row(lane, j) * ld + frag_col(lane, j)] = __low2half(v);
            dst[(int64_t)frag_row(lane, j + 1) * ld + frag_col(lane, j + 1)] = __high2half(v);
        }
    }
}

template <int CB> __global__ void table_kernel(__half* __restrict__ table)
{
    const uint32_t w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w < 65536u) table[w] = decode_one<CB>(w);
}

// ---- Hadamard-128: one warp per (row, block) ----------------------------------------------
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4])
{
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(u32_as_h2(u.x)), b = __half22float2(u32_as_h2(u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4])
{
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xFFFF0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4])
{
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}

// Rows of x may be gathered (row_src) and the scale vectors chosen per output row
// (pre_row / post_row give the row of the pre / post matrix to use), which is what the
// sibling-group and MoE paths need; the plain rotation passes NULL for all three.
template <typename T>
__global__ void __launch_bounds__(256)
    hadamard_kernel(const T* __restrict__ x, int64_t rows, int64_t n, int64_t x_row_stride,
                    const __half* __restrict__ pre, const __half* __restrict__ post,
                    __half* __restrict__ out, const int32_t* __restrict__ row_src,
                    const int32_t* __restrict__ pre_row, const int32_t* __restrict__ post_row,
                    int wait_dependency, int out_mode, int glu)
{
    // Let the next kernel of the stream (the GEMV that consumes `out`) start streaming its
    // weights right away; it waits for this grid before it reads any activation.
    griddep_launch_dependents();
    if (wait_dependency) griddep_wait();
    // 32-bit block arithmetic (the launcher refuses more than 2^31 blocks): the 64-bit divisions
    // that split a block index into (row, block of the row) cost more than the butterfly itself
    const int lane = threadIdx.x & 31;
    const uint32_t nblk = (uint32_t)(n >> 7);
    const uint32_t total = (uint32_t)rows * nblk;
    const uint32_t warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t nwarps = gridDim.x * (blockDim.x >> 5);
    // Four 128-blocks per warp and turn: the loads of all four are in flight before the first
    // butterfly starts (one 256-byte load per warp at a time left the kernel latency-bound).
    constexpr int U = 4;
    for (uint32_t i0 = warp0; i0 < total; i0 += nwarps * U) {
        float v[U][4], sp[U][4];
        int64_t rr[U], cc[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t i = i0 + u * nwarps;      // strided: small problems still use every warp
            const bool ok = i < total && i >= i0;    // (i >= i0: no wrap-around)
            const uint32_t rq = ok ? i / nblk : 0u;
            const int64_t r = rq, b = ok ? i - rq * nblk : 0u;
            rr[u] = ok ? r : -1;
            cc[u] = b * 128 + lane * 4;
            const int64_t rs = row_src ? row_src[r] : r;
            load4<T>(x + rs * x_row_stride + cc[u], v[u]);
            if (glu && ok) {
                // the row holds [gate (n) | up (n)]: the input is fp16(act(gate) * up)
                float up[4];
                load4<T>(x + rs * x_row_stride + n + cc[u], up);
#pragma unroll
                for (int q = 0; q < 4; q++) v[u][q] = glu_value(v[u][q], up[q], glu);
            }
            if (pre) load4<__half>(pre + (pre_row ? (int64_t)pre_row[r] * n : 0) + cc[u], sp[u]);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            // the reference rounds x to fp16 first (ponyexl3/ref/forward.py:26)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                v[u][q] = __half2float(__float2half_rn(v[u][q]));
                if (pre) v[u][q] *= sp[u][q];
            }
            had128_warp(v[u], lane);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (rr[u] < 0) continue;
            const int64_t r = rr[u], col = cc[u];
#pragma unroll
            for (int q = 0; q < 4; q++) v[u][q] *= EXL3_HAD_SCALE;
            if (post) {
                float s[4];
                load4<__half>(post + (post_row ? (int64_t)post_row[r] * n : 0) + col, s);
#pragma unroll
                for (int q = 0; q < 4; q++) v[u][q] *= s[q];
            }
            uint2 o;
            o.x = h2_as_u32(__floats2half2_rn(v[u][0], v[u][1]));
            o.y = h2_as_u32(__floats2half2_rn(v[u][2], v[u][3]));
            if (out_mode == HAD_OUT_F16) {
                *reinterpret_cast<uint2*>(out + r * n + col) = o;
            } else {
                // one 32-bit word per element for the GEMV's two-slot fragments:
                // (x, 0) keeps exactly-decoded weights, (x, x) lets the MMA add the two
                // codebook halves itself
                uint4 e;
                const uint32_t m = (out_mode == HAD_OUT_PAIR_X0) ? 0u : 0x00010000u;
                e.x = (o.x & 0xFFFFu) * (1u + m);
                e.y = (o.x >> 16) * (1u + m);
                e.z = (o.y & 0xFFFFu) * (1u + m);
                e.w = (o.y >> 16) * (1u + m);
                *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(out) + r * n + col) = e;
            }
        }
    }
}

// ---- launchers ------------------------------------------------------------------------------

static int grid_for(int64_t warps_needed, int warps_per_block)
{
    int64_t blocks = (warps_needed + warps_per_block - 1) / warps_per_block;
    const int64_t cap = (int64_t)device_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <int K> static void launch_unpack_k(const uint32_t* t, int64_t n, uint16_t* o, cudaStream_t s)
{
    unpack_kernel<K><<<grid_for(n, 8), 256, 0, s>>>(t, n, o);
}

int launch_unpack(const uint32_t* trellis, int64_t n_tiles, int k, uint16_t* out, cudaStream_t s)
{
    switch (k) {
        case 1: launch_unpack_k<1>(trellis, n_tiles, out, s); break;
        case 2: launch_unpack_k<2>(trellis, n_tiles, out, s); break;
        case 3: launch_unpack_k<3>(trellis, n_tiles, out, s); break;
        case 4: launch_unpack_k<4>(trellis, n_tiles, out, s); break;
        case 5: launch_unpack_k<5>(trellis, n_tiles, out, s); break;
        case 6: launch_unpack_k<6>(trellis, n_tiles, out, s); break;
        case 7: launch_unpack_k<7>(trellis, n_tiles, out, s); break;
        case 8: launch_unpack_k<8>(trellis, n_tiles, out, s); break;
        default: return EXL3_E_K;
    }
    return check_launch();
}

template <int K>
static int launch_decode_k(const uint32_t* t, int64_t t_in, int64_t t_out, int cb, int64_t tn0,
                           int64_t tnc, __half* w, int64_t ld, cudaStream_t s)
{
    const int g = grid_for(t_in * tnc, 8);
    switch (cb) {
        case CB_3INST: decode_kernel<K, CB_3INST><<<g, 256, 0, s>>>(t, t_in, t_out, tn0, tnc, w, ld); break;
        case CB_MCG: decode_kernel<K, CB_MCG><<<g, 256, 0, s>>>(t, t_in, t_out, tn0, tnc, w, ld); break;
        case CB_MUL1: decode_kernel<K, CB_MUL1><<<g, 256, 0, s>>>(t, t_in, t_out, tn0, tnc, w, ld); break;
        default: return EXL3_E_CODEBOOK;
    }
    return check_launch();
}

int launch_decode(const uint32_t* trellis, int64_t t_in, int64_t t_out, int k, int cb, int64_t tn0,
                  int64_t tn_count, __half* w, int64_t ld, cudaStream_t s)
{
    switch (k) {
        case 1: return launch_decode_k<1>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 2: return launch_decode_k<2>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 3: return launch_decode_k<3>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 4: return launch_decode_k<4>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 5: return launch_decode_k<5>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 6: return launch_decode_k<6>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 7: return launch_decode_k<7>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        case 8: return launch_decode_k<8>(trellis, t_in, t_out, cb, tn0, tn_count, w, ld, s);
        default: return EXL3_E_K;
    }
}

int launch_table(int cb, __half* table, cudaStream_t s)
{
    switch (cb) {
        case CB_3INST: table_kernel<CB_3INST><<<256, 256, 0, s>>>(table); break;
        case CB_MCG: table_kernel<CB_MCG><<<256, 256, 0, s>>>(table); break;
        case CB_MUL1: table_kernel<CB_MUL1><<<256, 256, 0, s>>>(table); break;
        default: return EXL3_E_CODEBOOK;
    }
    return check_launch();
}

int launch_hadamard(const void* x, int x_dtype, int64_t rows, int64_t n, int64_t x_row_stride,
                    const __half* pre, const __half* post, __half* out, const int32_t* row_src,
                    const int32_t* pre_row, const int32_t* post_row, bool pdl, int out_mode,
                    cudaStream_t s, int glu)
{
    if (rows * (n >> 7) >= ((int64_t)1 << 31)) return EXL3_E_RANGE;   // the kernel counts blocks in 32 bits
    const int g = grid_for(rows * (n >> 7), 8);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(g);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    const int wait = pdl ? 1 : 0;
    cudaError_t e;
    switch (x_dtype) {
        case EXL3_DT_F16:
            e = cudaLaunchKernelEx(&cfg, hadamard_kernel<__half>, (const __half*)x, rows, n,
                                   x_row_stride, pre, post, out, row_src, pre_row, post_row, wait, out_mode, glu);
            break;
        case EXL3_DT_BF16:
            e = cudaLaunchKernelEx(&cfg, hadamard_kernel<__nv_bfloat16>, (const __nv_bfloat16*)x,
                                   rows, n, x_row_stride, pre, post, out, row_src, pre_row, post_row,
                                   wait, out_mode, glu);
            break;
        case EXL3_DT_F32:
            e = cudaLaunchKernelEx(&cfg, hadamard_kernel<float>, (const float*)x, rows, n,
                                   x_row_stride, pre, post, out, row_src, pre_row, post_row, wait, out_mode, glu);
            break;
        default: return EXL3_E_DTYPE;
    }
    return note_cuda(e);
}

}  // namespace exl3
