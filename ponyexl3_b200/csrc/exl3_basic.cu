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

// ---- the rotation of many rows, on the tensor cores ---------------------------------------------
// had128(x * suh) for blocks of 16 rows x 128 columns as mma.sync m16n8k16 products with the
// +-1 Sylvester matrix H[k][n] = (-1)^popcount(k & n): the warp-shuffle butterfly above costs
// about 130 instructions per row and 128-block and made the prefill GEMM's input rotation
// instruction-bound at a quarter of the memory bandwidth; here a row and block costs about 40.
// fp16 inputs times +-1 are exact and the sums are fp32, as in the butterfly; only the order of
// the fp32 additions differs.
//
// A lane loads 16 contiguous bytes (8 columns) of rows g and g + 8 per quarter of the block.
// The MMA's k index is a free bijection as long as A and B agree: k-step (q, s) takes columns
// 32 q + 8 t + 4 s + {0, 1} and + {2, 3} of lane t as its k = 2t, 2t+1 and 2t+8, 2t+9.  The
// matching B fragment is H at those columns against output column n = 8 nt + g: its sign splits
// into a part that depends on the column's low three bits and g, a part parity(t & nt) that
// depends on the lane and the low two bits of nt (together sixteen constant registers per lane),
// and a part parity(q & (nt >> 2)) that is known at compile time and picks one of two
// accumulators, subtracted at the end: no sign arithmetic is left inside the loop.
constexpr int kHadTileRow = 272;                 // 256 bytes of a row + 16: the fragment stores hit 32 banks
constexpr int kHadTileBytes = 16 * kHadTileRow;
template <typename T> struct Load8;
template <> struct Load8<__half> {
    static __device__ __forceinline__ uint4 at(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
};
template <> struct Load8<__nv_bfloat16> {
    static __device__ __forceinline__ uint4 at(const __nv_bfloat16* p)
    {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++)
            o[i] = h2_as_u32(__floats2half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u)));
        return make_uint4(o[0], o[1], o[2], o[3]);
    }
};
template <> struct Load8<float> {
    static __device__ __forceinline__ uint4 at(const float* p)
    {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        return make_uint4(h2_as_u32(__floats2half2_rn(a.x, a.y)), h2_as_u32(__floats2half2_rn(a.z, a.w)),
                          h2_as_u32(__floats2half2_rn(b.x, b.y)), h2_as_u32(__floats2half2_rn(b.z, b.w)));
    }
};

__device__ __forceinline__ uint32_t glu_pair(uint32_t gate, uint32_t up, int glu)
{
    const float2 gf = __half22float2(u32_as_h2(gate)), uf = __half22float2(u32_as_h2(up));
    return h2_as_u32(__floats2half2_rn(glu_value(gf.x, uf.x, glu), glu_value(gf.y, uf.y, glu)));
}

template <typename T>
__global__ void __launch_bounds__(256, 2)
    hadamard_mma_kernel(const T* __restrict__ x, int64_t rows, int64_t n, int64_t x_row_stride,
                        const __half* __restrict__ pre, __half* __restrict__ out,
                        const int32_t* __restrict__ row_src, const int32_t* __restrict__ pre_row,
                        const int32_t* __restrict__ rows_dev, int wait_dependency, int glu)
{
    griddep_launch_dependents();
    if (wait_dependency || rows_dev) griddep_wait();
    if (rows_dev) {           // the number of rows in use was left on the device by an earlier kernel
        const int64_t r = *rows_dev;
        rows = r < 0 ? 0 : (r < rows ? r : rows);
    }
    __shared__ __align__(16) uint8_t stile[8 * kHadTileBytes];
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // B fragments, constant per lane: pt[nl][s][j] holds H at columns 4 s + 2 j + {0, 1} of the
    // lane's 8-column group against output column 8 (4 nh + nl) + g, without the sign of the
    // quarter (see the loop): the column's low bits meet g, the lane's t meets nl.
    uint32_t pt[4][2][2];
#pragma unroll
    for (int nl = 0; nl < 4; nl++) {
        const uint32_t flip = (__popc(t & nl) & 1) ? 0x80008000u : 0u;
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const uint32_t lo = (__popc((4 * s + 2 * j) & g) & 1) ? 0xBC00u : 0x3C00u;
                const uint32_t hi = (__popc((4 * s + 2 * j + 1) & g) & 1) ? 0xBC00u : 0x3C00u;
                pt[nl][s][j] = (lo | (hi << 16)) ^ flip;
            }
    }
    const uint32_t nblk = (uint32_t)(n >> 7);
    const uint32_t total = (uint32_t)((rows + 15) >> 4) * nblk;
    const uint32_t warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t nwarps = gridDim.x * (blockDim.x >> 5);
    for (uint32_t blk = warp0; blk < total; blk += nwarps) {
        const uint32_t rb = blk / nblk, cb = blk - rb * nblk;
        const int64_t r0 = (int64_t)rb * 16 + g, r1 = r0 + 8;
        const bool ok0 = r0 < rows, ok1 = r1 < rows;
        const int64_t col = (int64_t)cb * 128 + 8 * t;
        uint4 xa[4], xb[4];
        {
            const int64_t s0 = ok0 ? (row_src ? row_src[r0] : r0) : 0, s1 = ok1 ? (row_src ? row_src[r1] : r1) : 0;
            const T* p0 = x + s0 * x_row_stride + col;
            const T* p1 = x + s1 * x_row_stride + col;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                xa[q] = ok0 ? Load8<T>::at(p0 + 32 * q) : make_uint4(0u, 0u, 0u, 0u);
                xb[q] = ok1 ? Load8<T>::at(p1 + 32 * q) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (glu) {
                // the row holds [gate (n) | up (n)]: the input is fp16(act(gate) * up)
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    if (ok0) {
                        const uint4 u = Load8<T>::at(p0 + n + 32 * q);
                        xa[q] = make_uint4(glu_pair(xa[q].x, u.x, glu), glu_pair(xa[q].y, u.y, glu),
                                           glu_pair(xa[q].z, u.z, glu), glu_pair(xa[q].w, u.w, glu));
                    }
                    if (ok1) {
                        const uint4 u = Load8<T>::at(p1 + n + 32 * q);
                        xb[q] = make_uint4(glu_pair(xb[q].x, u.x, glu), glu_pair(xb[q].y, u.y, glu),
                                           glu_pair(xb[q].z, u.z, glu), glu_pair(xb[q].w, u.w, glu));
                    }
                }
            }
        }
        if (pre) {
            const __half* q0 = pre + (ok0 && pre_row ? (int64_t)pre_row[r0] * n : 0) + col;
            const __half* q1 = pre + (ok1 && pre_row ? (int64_t)pre_row[r1] * n : 0) + col;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint4 a = *reinterpret_cast<const uint4*>(q0 + 32 * q);
                const uint4 b = *reinterpret_cast<const uint4*>(q1 + 32 * q);
                xa[q].x = h2_as_u32(__hmul2(u32_as_h2(xa[q].x), u32_as_h2(a.x)));
                xa[q].y = h2_as_u32(__hmul2(u32_as_h2(xa[q].y), u32_as_h2(a.y)));
                xa[q].z = h2_as_u32(__hmul2(u32_as_h2(xa[q].z), u32_as_h2(a.z)));
                xa[q].w = h2_as_u32(__hmul2(u32_as_h2(xa[q].w), u32_as_h2(a.w)));
                xb[q].x = h2_as_u32(__hmul2(u32_as_h2(xb[q].x), u32_as_h2(b.x)));
                xb[q].y = h2_as_u32(__hmul2(u32_as_h2(xb[q].y), u32_as_h2(b.y)));
                xb[q].z = h2_as_u32(__hmul2(u32_as_h2(xb[q].z), u32_as_h2(b.z)));
                xb[q].w = h2_as_u32(__hmul2(u32_as_h2(xb[q].w), u32_as_h2(b.w)));
            }
        }
        // The accumulator fragments (4 bytes per lane, row and 8-column group) go through a padded
        // tile in shared memory so that every lane stores 16 contiguous bytes: 8 instead of 32
        // stores, and whole 32-byte sectors.
        uint8_t* tile = stile + (threadIdx.x >> 5) * kHadTileBytes;
#pragma unroll
        for (int nh = 0; nh < 4; nh++)
#pragma unroll
            for (int nl = 0; nl < 4; nl++) {
                // output columns 8 nt + g, nt = 4 nh + nl: quarter q enters with the sign
                // parity(q & nh), known at compile time, so it picks one of two accumulators
                float cp[4] = {0.f, 0.f, 0.f, 0.f}, cm[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t a0[4] = {xa[q].x, xb[q].x, xa[q].y, xb[q].y};
                    const uint32_t a1[4] = {xa[q].z, xb[q].z, xa[q].w, xb[q].w};
                    if (((q & nh) == 1) || ((q & nh) == 2)) {       // odd number of common bits
                        mma_16816(cm, a0, pt[nl][0][0], pt[nl][0][1]);
                        mma_16816(cm, a1, pt[nl][1][0], pt[nl][1][1]);
                    } else {
                        mma_16816(cp, a0, pt[nl][0][0], pt[nl][0][1]);
                        mma_16816(cp, a1, pt[nl][1][0], pt[nl][1][1]);
                    }
                }
                const int nt = 4 * nh + nl;
                *reinterpret_cast<__half2*>(tile + g * kHadTileRow + 16 * nt + 4 * t) =
                    __floats2half2_rn((cp[0] - cm[0]) * EXL3_HAD_SCALE, (cp[1] - cm[1]) * EXL3_HAD_SCALE);
                *reinterpret_cast<__half2*>(tile + (g + 8) * kHadTileRow + 16 * nt + 4 * t) =
                    __floats2half2_rn((cp[2] - cm[2]) * EXL3_HAD_SCALE, (cp[3] - cm[3]) * EXL3_HAD_SCALE);
            }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; i++) {          // 16 rows x 16 chunks of 16 bytes, two rows per turn
            const int rr = 2 * i + (lane >> 4), ch = lane & 15;
            const int64_t r = (int64_t)rb * 16 + rr;
            const uint4 v = *reinterpret_cast<const uint4*>(tile + rr * kHadTileRow + 16 * ch);
            if (r < rows) *reinterpret_cast<uint4*>(out + r * n + (int64_t)cb * 128 + 8 * ch) = v;
        }
        __syncwarp();
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
                    cudaStream_t s, int glu, const int32_t* rows_dev)
{
    if (rows * (n >> 7) >= ((int64_t)1 << 31)) return EXL3_E_RANGE;   // the kernel counts blocks in 32 bits
    // Many rows into a plain fp16 matrix (the prefill GEMM's operand): 16-row blocks on the tensor cores.
    // (a GLU over bf16 / fp32 rows stays on the butterfly kernel, which applies it before the fp16 rounding)
    // (a row count read from the device always takes this kernel, however few rows there may be)
    const bool mma = out_mode == HAD_OUT_F16 && !post && !post_row && (rows >= kHadamardMmaMinRows || rows_dev) &&
                     (!glu || x_dtype == EXL3_DT_F16) &&
                     x_row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                     (!pre || (reinterpret_cast<uintptr_t>(pre) & 15) == 0) && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (rows_dev && !mma) return EXL3_E_UNSUPPORTED;
    const int g = mma ? grid_for(((rows + 15) >> 4) * (n >> 7), 8) : grid_for(rows * (n >> 7), 8);
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
    if (mma) {
        switch (x_dtype) {
            case EXL3_DT_F16:
                e = cudaLaunchKernelEx(&cfg, hadamard_mma_kernel<__half>, (const __half*)x, rows, n, x_row_stride, pre,
                                       out, row_src, pre_row, rows_dev, wait, glu);
                break;
            case EXL3_DT_BF16:
                e = cudaLaunchKernelEx(&cfg, hadamard_mma_kernel<__nv_bfloat16>, (const __nv_bfloat16*)x, rows, n,
                                       x_row_stride, pre, out, row_src, pre_row, rows_dev, wait, glu);
                break;
            case EXL3_DT_F32:
                e = cudaLaunchKernelEx(&cfg, hadamard_mma_kernel<float>, (const float*)x, rows, n, x_row_stride, pre,
                                       out, row_src, pre_row, rows_dev, wait, glu);
                break;
            default: return EXL3_E_DTYPE;
        }
        return note_cuda(e);
    }
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
