// The pieces of a decode step that sit between the EXL3 linears: residual add + RMSNorm,
// rotary embedding + KV-cache append, grouped-query attention over the cache for 1..16 new
// positions (split over the context, then combined), and SwiGLU.  They are the caller's side
// of the path — the reference leaves them to its array framework (mlx.fast.rms_norm / rope /
// scaled_dot_product_attention in the model graphs it patches, ponyexl3/mlx/model.py:628-634)
// — and exist here so that a whole step can be measured without a framework's launch and
// element-wise overheads between the linears.  All tensors are fp16, accumulation is fp32.
#include <cuda_fp16.h>

#include <algorithm>

#include "exl3_internal.h"

namespace exl3 {

// ------------------------------------------------------------------ residual + RMSNorm ----
// x <- fp16(x + delta) (delta may be NULL), h <- fp16(x * rsqrt(mean(x^2) + eps) * w).
// One CTA per row, eight elements per thread and turn.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(__half* x, const __half* delta, const __half* w,
                                                          __half* h, int n, int64_t x_stride,
                                                          int64_t d_stride, int64_t h_stride, float eps)
{
    griddep_launch_dependents();
    griddep_wait();
    __shared__ float red[8];
    __half* xr = x + (int64_t)blockIdx.x * x_stride;
    const __half* dr = delta ? delta + (int64_t)blockIdx.x * d_stride : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < n; i += 256 * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(xr + i);
        __half2* hv = reinterpret_cast<__half2*>(&v);
        if (dr) {
            const uint4 d = *reinterpret_cast<const uint4*>(dr + i);
            const __half2* hd = reinterpret_cast<const __half2*>(&d);
#pragma unroll
            for (int q = 0; q < 4; q++) hv[q] = __hadd2(hv[q], hd[q]);
            *reinterpret_cast<uint4*>(xr + i) = v;
        }
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float2 f = __half22float2(hv[q]);
            ss += f.x * f.x + f.y * f.y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int q = 0; q < 8; q++) tot += red[q];
    const float rstd = rsqrtf(tot / (float)n + eps);
    __half* hr = h + (int64_t)blockIdx.x * h_stride;
    for (int i = threadIdx.x * 8; i < n; i += 256 * 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(xr + i);   // own writes: same thread, same address
        const uint4 g = *reinterpret_cast<const uint4*>(w + i);
        const __half2* hv = reinterpret_cast<const __half2*>(&v);
        const __half2* hg = reinterpret_cast<const __half2*>(&g);
        uint4 o;
        __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float2 f = __half22float2(hv[q]), gg = __half22float2(hg[q]);
            ho[q] = __floats2half2_rn(f.x * rstd * gg.x, f.y * rstd * gg.y);
        }
        *reinterpret_cast<uint4*>(hr + i) = o;
    }
}

// ------------------------------------------------------------- RoPE + KV-cache append ----
// qkv row r holds [q heads | k heads | v heads], head_dim 128.  q and k get the rotate-half
// rotary embedding of position pos0 + r (cos/sin rows r of the tables); q goes to q_out
// (rows, hq, 128), k and v to row pos0 + r of their head's cache (hkv, cache_len, 128).
__global__ void __launch_bounds__(64) rope_append_kernel(const __half* qkv, int64_t qkv_stride, const __half* cos_t,
                                                         const __half* sin_t, __half* q_out, __half* k_cache,
                                                         __half* v_cache, int hq, int hkv, int64_t cache_len,
                                                         int pos0)
{
    griddep_launch_dependents();
    griddep_wait();
    const int r = blockIdx.x, head = blockIdx.y, d = threadIdx.x;   // d and d + 64
    const __half* src = qkv + (int64_t)r * qkv_stride + (int64_t)head * 128;
    const float lo = __half2float(src[d]), hi = __half2float(src[d + 64]);
    if (head >= hq + hkv) {   // v: plain copy
        __half* dst = v_cache + ((int64_t)(head - hq - hkv) * cache_len + pos0 + r) * 128;
        dst[d] = src[d];
        dst[d + 64] = src[d + 64];
        return;
    }
    const float c0 = __half2float(cos_t[r * 128 + d]), s0 = __half2float(sin_t[r * 128 + d]);
    const float c1 = __half2float(cos_t[r * 128 + d + 64]), s1 = __half2float(sin_t[r * 128 + d + 64]);
    const __half o0 = __float2half_rn(lo * c0 - hi * s0);
    const __half o1 = __float2half_rn(hi * c1 + lo * s1);
    __half* dst = head < hq ? q_out + ((int64_t)r * hq + head) * 128
                            : k_cache + ((int64_t)(head - hq) * cache_len + pos0 + r) * 128;
    dst[d] = o0;
    dst[d + 64] = o1;
}

// ------------------------------------------------------------------------------ SwiGLU ----
// gu row = [gate (h) | up (h)]: out = fp16(silu(gate) * up).
__global__ void __launch_bounds__(256) swiglu_kernel(const __half* gu, int64_t gu_stride, __half* out,
                                                     int64_t out_stride, int h)
{
    griddep_launch_dependents();
    griddep_wait();
    const int r = blockIdx.y;
    const int i = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (i >= h) return;
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (int64_t)r * gu_stride + i);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + (int64_t)r * gu_stride + h + i);
    const __half2* hg = reinterpret_cast<const __half2*>(&gv);
    const __half2* hu = reinterpret_cast<const __half2*>(&uv);
    uint4 o;
    __half2* ho = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const float2 g = __half22float2(hg[q]), u = __half22float2(hu[q]);
        ho[q] = __floats2half2_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (int64_t)r * out_stride + i) = o;
}

// --------------------------------------------------- grouped-query decode attention ----
// One launch covers all query heads of all new positions: the M = group * rows query rows
// that share a KV head (row m = g * rows + r: query head kvh * group + g, new position r)
// form the M side of tensor-core tiles, so the cache is read once per KV head whatever the
// group size and row count.  The context is cut into chunks; CTA (chunk, kv head) runs an
// online-softmax pass over its chunk in 64-key tiles (cp.async double buffer) and writes an
// un-normalised partial output with its running maximum and sum; a second kernel combines
// the chunks.  Position r sees keys 0 .. ctx + r (the new keys have been appended already).
constexpr int kAttnTile = 64;               // keys per shared-memory tile
constexpr int kAttnLd = 136;                // halves per shared row: 128 + 8 (bank spread, 16 B aligned)
constexpr int kAttnTileBytes = kAttnTile * kAttnLd * 2;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid)
{
    const int sz = valid ? 16 : 0;          // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4])
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) { return h2_as_u32(__floats2half2_rn(a, b)); }

struct AttnArgs {
    const __half* q;          // (rows, hq, 128)
    const __half* k_cache;    // (hkv, cache_len, 128)
    const __half* v_cache;
    float* part_o;            // (hkv, nsplit, M, 128) un-normalised partial outputs
    float* part_ml;           // (hkv, nsplit, M, 2): running max (log2 domain), running sum
    __half* out;              // (rows, hq * 128)
    int64_t cache_len;
    int rows, hq, hkv, group, ctx, chunk, nsplit;
    int nbuf;                 // shared-memory tile buffers per tensor: 2 (double buffer) or 1 (one-tile chunks)
    float scale_log2;         // log2(e) / sqrt(128)
};

template <int NW>   // warps = 16-row query tiles
__global__ void __launch_bounds__(NW * 32) attn_partial_kernel(const AttnArgs a)
{
    extern __shared__ __align__(128) uint8_t smem[];
    griddep_launch_dependents();
    griddep_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int M = a.group * a.rows;
    const int total = a.ctx + a.rows;                   // keys in the cache now
    const int p0 = split * a.chunk;
    const int p1 = min(total, p0 + a.chunk);
    const int ntiles = (p1 - p0 + kAttnTile - 1) / kAttnTile;
    const __half* kbase = a.k_cache + (int64_t)kvh * a.cache_len * 128;
    const __half* vbase = a.v_cache + (int64_t)kvh * a.cache_len * 128;
    const uint32_t s_k = smem_u32(smem), s_v = s_k + a.nbuf * kAttnTileBytes;   // K tile buffers, then V tile buffers

    auto load_tile = [&](int ti, int buf) {
        const int key0 = p0 + ti * kAttnTile;
        for (int c = tid; c < kAttnTile * 16; c += NW * 32) {        // 16-byte pieces: 16 per row
            const int row = c >> 4, piece = c & 15;
            const int key = key0 + row;
            const bool ok = key < p1;
            const int64_t off = (int64_t)(ok ? key : p1 - 1) * 128 + piece * 8;
            const uint32_t d = (uint32_t)(buf * kAttnTileBytes + (row * kAttnLd + piece * 8) * 2);
            cp_async16(s_k + d, kbase + off, ok);
            cp_async16(s_v + d, vbase + off, ok);
        }
        cp_async_commit();
    };
    if (ntiles > 0) load_tile(0, 0);

    // query fragments of this warp's 16 rows (rows m0 + g and m0 + g + 8), all 8 k-steps
    const int m0 = warp * 16;
    uint32_t qf[8][4];
    int lim[2];                                          // last visible key of the two rows
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int m = m0 + g + 8 * h;
        const bool ok = m < M;
        const int gq = ok ? m / a.rows : 0, r = ok ? m - gq * a.rows : 0;
        lim[h] = ok ? a.ctx + r : -1;
        const __half* qr = a.q + ((int64_t)r * a.hq + kvh * a.group + gq) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            qf[ks][h] = ok ? *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 2 * t) : 0u;
            qf[ks][h + 2] = ok ? *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 2 * t + 8) : 0u;
        }
    }
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++)
#pragma unroll
        for (int q = 0; q < 4; q++) o[i][q] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    for (int ti = 0; ti < ntiles; ti++) {
        const int buf = ti & (a.nbuf - 1);
        if (ti + 1 < ntiles) {
            load_tile(ti + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __half* ks_ = reinterpret_cast<const __half*>(smem + buf * kAttnTileBytes);
        const int key0 = p0 + ti * kAttnTile;

        // S = Q K^T for 64 keys: 8 key tiles x 8 k-steps
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int q = 0; q < 4; q++) s[nt][q] = 0.f;
            const __half* kr = ks_ + (nt * 8 + g) * kAttnLd + 2 * t;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr + ks * 16);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + ks * 16 + 8);
                mma_16816(s[nt], qf[ks], b0, b1);
            }
        }
        // scale, mask (keys past a row's own position, and the zero-filled tail), running max
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int key = key0 + nt * 8 + 2 * t + (q & 1);
                const int h = q >> 1;
                const float v = (key <= lim[h] && key < p1) ? s[nt][q] * a.scale_log2 : -INFINITY;
                s[nt][q] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        float alpha[2], msafe[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float mnew = fmaxf(mrow[h], mx[h]);
            msafe[h] = mnew == -INFINITY ? 0.f : mnew;
            alpha[h] = exp2f(mrow[h] - msafe[h]);          // 0 when nothing was seen before
            mrow[h] = mnew;
            lrow[h] *= alpha[h];
        }
#pragma unroll
        for (int i = 0; i < 16; i++) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }
        // P = exp2(S - m), as A fragments of the 4 k-steps of P V
        uint32_t pa[4][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            float p[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                p[q] = exp2f(s[nt][q] - msafe[q >> 1]);
                lrow[q >> 1] += p[q];
            }
            pa[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(p[0], p[1]);
            pa[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(p[2], p[3]);
        }
        // O += P V: 16 feature tiles x 4 k-steps, V fragments through transposing ldmatrix
        const uint32_t vs_ = s_v + buf * kAttnTileBytes;
        const int lrow_ = (lane & 7) + ((lane >> 3) & 1) * 8, lcol = (lane >> 4) * 8;
#pragma unroll
        for (int k2 = 0; k2 < 4; k2++)
#pragma unroll
            for (int dp = 0; dp < 8; dp++) {          // two feature tiles per ldmatrix.x4
                uint32_t b[4];
                ldmatrix_x4_trans(vs_ + (uint32_t)(((k2 * 16 + lrow_) * kAttnLd + dp * 16 + lcol) * 2), b);
                mma_16816(o[2 * dp], pa[k2], b[0], b[1]);
                mma_16816(o[2 * dp + 1], pa[k2], b[2], b[3]);
            }
        __syncthreads();                               // the buffer is refilled two turns later
    }

    // partial results of this chunk
#pragma unroll
    for (int h = 0; h < 2; h++) {
        lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 1);
        lrow[h] += __shfl_xor_sync(0xffffffffu, lrow[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int m = m0 + g + 8 * h;
        if (m >= M) continue;
        const int64_t row = ((int64_t)kvh * a.nsplit + split) * M + m;
        float* po = a.part_o + row * 128 + 2 * t;
#pragma unroll
        for (int i = 0; i < 16; i++)
            *reinterpret_cast<float2*>(po + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
        if (t == 0) {
            a.part_ml[row * 2] = mrow[h];
            a.part_ml[row * 2 + 1] = lrow[h];
        }
    }
}

// out[r, head, :] = sum_i 2^(m_i - m*) O_i / sum_i 2^(m_i - m*) l_i over the chunks i.
// One CTA per query row: L chunk lanes (about a quarter of the chunk count, 4..32) x 32 threads of
// four features.  Lane j folds chunks j, j + L, ... into a running (max, sum, output) in ONE pass — the loads of a lane do not depend on
// its running state, so they are all in flight together — and the lanes are merged through shared
// memory by the same rule.  (A two-pass version with a thread per feature took as long as the
// partial kernel at 16 rows.)
constexpr int kCombineMaxLanes = 32;
__global__ void __launch_bounds__(32 * kCombineMaxLanes) attn_combine_kernel(const AttnArgs a)
{
    griddep_launch_dependents();
    griddep_wait();
    __shared__ float4 s_acc[kCombineMaxLanes][32];
    __shared__ float s_l[kCombineMaxLanes], s_m[kCombineMaxLanes];
    const int m = blockIdx.x, kvh = blockIdx.y, d4 = threadIdx.x & 31, j = threadIdx.x >> 5;
    const int lanes = blockDim.x >> 5;
    const int M = a.group * a.rows;
    const int64_t base = (int64_t)kvh * a.nsplit * M + m;
    float mrun = -INFINITY, lrun = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int i = j; i < a.nsplit; i += lanes) {
        const int64_t row = base + (int64_t)i * M;
        const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + row * 2);
        const float4 o = *reinterpret_cast<const float4*>(a.part_o + row * 128 + 4 * d4);
        if (ml.x == -INFINITY) continue;                    // a chunk this row does not see at all
        const float mnew = fmaxf(mrun, ml.x);
        const float so = exp2f(mrun - mnew), sn = exp2f(ml.x - mnew);   // so = 0 on the first chunk
        acc.x = acc.x * so + o.x * sn; acc.y = acc.y * so + o.y * sn;
        acc.z = acc.z * so + o.z * sn; acc.w = acc.w * so + o.w * sn;
        lrun = lrun * so + ml.y * sn;
        mrun = mnew;
    }
    s_acc[j][d4] = acc;
    if (d4 == 0) { s_l[j] = lrun; s_m[j] = mrun; }
    __syncthreads();
    if (j == 0) {
        float mmax = s_m[0];
        for (int q = 1; q < lanes; q++) mmax = fmaxf(mmax, s_m[q]);
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        float den = 0.f;
        for (int q = 0; q < lanes; q++) {
            const float w = s_m[q] == -INFINITY ? 0.f : exp2f(s_m[q] - mmax);
            const float4 v = s_acc[q][d4];
            num.x += w * v.x; num.y += w * v.y; num.z += w * v.z; num.w += w * v.w;
            den += w * s_l[q];
        }
        const float inv = 1.f / den;
        const int gq = m / a.rows, r = m - gq * a.rows;
        uint2 ov;
        ov.x = pack_h2(num.x * inv, num.y * inv);
        ov.y = pack_h2(num.z * inv, num.w * inv);
        *reinterpret_cast<uint2*>(a.out + ((int64_t)r * a.hq + kvh * a.group + gq) * 128 + 4 * d4) = ov;
    }
}

template <int NW> static int launch_attn_partial(const AttnArgs& a, cudaStream_t s, bool pdl)
{
    const size_t smem = 2 * (size_t)a.nbuf * kAttnTileBytes;
    static bool set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return EXL3_E_UNSUPPORTED;
    if (!set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_partial_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             4 * kAttnTileBytes);
        if (e != cudaSuccess) return note_cuda(e);
        set[dev] = true;
    }
    return launch_kernel(attn_partial_kernel<NW>, dim3((unsigned)a.nsplit, (unsigned)a.hkv), dim3(NW * 32), smem, s,
                         pdl, a);
}

// Chunking: about two CTAs per SM (a CTA of the verify shape, 5 warps at 170 registers, fits twice),
// chunks a multiple of the 64-key tile.  One CTA per SM was tried for many query rows and left the
// kernel bound by the latency of a single CTA's MMA chain (41 us at 16 rows); single-tile chunks
// were tried for one row and only moved time into the combine kernel.
static void attn_plan(int total_keys, int hkv, int m_rows, int* chunk, int* nsplit, int* nbuf)
{
    (void)m_rows;
    const int want = std::max(1, 2 * device_sm_count() / std::max(1, hkv));
    int c = (total_keys + want - 1) / want;
    c = (c + kAttnTile - 1) / kAttnTile * kAttnTile;
    *chunk = c;
    *nsplit = (total_keys + c - 1) / c;
    *nbuf = c > kAttnTile ? 2 : 1;
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_add_rmsnorm(uint16_t* x, const uint16_t* delta, const uint16_t* weight, uint16_t* h,
                                int rows, int64_t n, int64_t x_row_stride, int64_t delta_row_stride,
                                int64_t h_row_stride, float eps, unsigned flags, exl3_stream_t stream)
{
    if (!x || !weight || !h) return EXL3_E_NULL;
    if (rows < 1 || n < 8 || n % 8) return EXL3_E_SHAPE;
    if (x_row_stride % 8 || h_row_stride % 8 || (delta && delta_row_stride % 8)) return EXL3_E_ALIGN;
    if (((uintptr_t)x | (uintptr_t)weight | (uintptr_t)h | (uintptr_t)delta) & 15) return EXL3_E_ALIGN;
    return launch_kernel(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream,
                         (flags & EXL3_FLAG_PDL) != 0, reinterpret_cast<__half*>(x),
                         reinterpret_cast<const __half*>(delta), reinterpret_cast<const __half*>(weight),
                         reinterpret_cast<__half*>(h), (int)n, x_row_stride, delta_row_stride, h_row_stride, eps);
}

extern "C" int exl3_rope_append(const uint16_t* qkv, int64_t qkv_row_stride, const uint16_t* cos_table,
                                const uint16_t* sin_table, uint16_t* q_out, uint16_t* k_cache,
                                uint16_t* v_cache, int rows, int q_heads, int kv_heads, int64_t cache_len,
                                int pos0, unsigned flags, exl3_stream_t stream)
{
    if (!qkv || !cos_table || !sin_table || !q_out || !k_cache || !v_cache) return EXL3_E_NULL;
    if (rows < 1 || q_heads < 1 || kv_heads < 1) return EXL3_E_SHAPE;
    if (pos0 < 0 || (int64_t)pos0 + rows > cache_len) return EXL3_E_RANGE;
    return launch_kernel(rope_append_kernel, dim3((unsigned)rows, (unsigned)(q_heads + 2 * kv_heads)), dim3(64), 0,
                         (cudaStream_t)stream, (flags & EXL3_FLAG_PDL) != 0, reinterpret_cast<const __half*>(qkv),
                         qkv_row_stride, reinterpret_cast<const __half*>(cos_table),
                         reinterpret_cast<const __half*>(sin_table), reinterpret_cast<__half*>(q_out),
                         reinterpret_cast<__half*>(k_cache), reinterpret_cast<__half*>(v_cache), q_heads, kv_heads,
                         cache_len, pos0);
}

extern "C" int exl3_swiglu(const uint16_t* gate_up, int64_t gu_row_stride, uint16_t* out, int64_t out_row_stride,
                           int rows, int64_t h, unsigned flags, exl3_stream_t stream)
{
    if (!gate_up || !out) return EXL3_E_NULL;
    if (rows < 1 || h < 8 || h % 8) return EXL3_E_SHAPE;
    if (gu_row_stride % 8 || out_row_stride % 8 || (((uintptr_t)gate_up | (uintptr_t)out) & 15)) return EXL3_E_ALIGN;
    return launch_kernel(swiglu_kernel, dim3((unsigned)((h / 8 + 255) / 256), (unsigned)rows), dim3(256), 0,
                         (cudaStream_t)stream, (flags & EXL3_FLAG_PDL) != 0, reinterpret_cast<const __half*>(gate_up),
                         gu_row_stride, reinterpret_cast<__half*>(out), out_row_stride, (int)h);
}

extern "C" size_t exl3_attn_workspace_bytes(int rows, int q_heads, int kv_heads, int64_t total_keys)
{
    if (rows < 1 || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads || total_keys < 1) return 0;
    // The number of context chunks depends on the context length through the rounding of the
    // chunk size, but never exceeds the CTA count the plan aims at: the bound over all contexts,
    // so that a workspace sized once for the longest context serves every shorter one.
    const int m = q_heads / kv_heads * rows;
    const int want = std::max(1, 2 * device_sm_count() / std::max(1, kv_heads));
    return (size_t)kv_heads * want * m * (128 + 2) * sizeof(float) + 256;
}

extern "C" int exl3_attn_decode(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                uint16_t* out, int rows, int q_heads, int kv_heads, int64_t cache_len, int ctx,
                                void* workspace, size_t workspace_bytes, unsigned flags, exl3_stream_t stream)
{
    if (!q || !k_cache || !v_cache || !out || !workspace) return EXL3_E_NULL;
    if (rows < 1 || rows > 16) return EXL3_E_ROWS;
    if (q_heads < 1 || kv_heads < 1 || q_heads % kv_heads) return EXL3_E_SHAPE;
    const int group = q_heads / kv_heads, m = group * rows;
    if (m > 128) return EXL3_E_UNSUPPORTED;
    if (ctx < 0 || (int64_t)ctx + rows > cache_len) return EXL3_E_RANGE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out | (uintptr_t)workspace) & 15)
        return EXL3_E_ALIGN;
    AttnArgs a;
    a.q = reinterpret_cast<const __half*>(q);
    a.k_cache = reinterpret_cast<const __half*>(k_cache);
    a.v_cache = reinterpret_cast<const __half*>(v_cache);
    a.out = reinterpret_cast<__half*>(out);
    a.cache_len = cache_len;
    a.rows = rows; a.hq = q_heads; a.hkv = kv_heads; a.group = group; a.ctx = ctx;
    attn_plan(ctx + rows, kv_heads, m, &a.chunk, &a.nsplit, &a.nbuf);
    const size_t need = (size_t)kv_heads * a.nsplit * m * (128 + 2) * sizeof(float);
    if (workspace_bytes < need) return EXL3_E_WORKSPACE;
    a.part_o = static_cast<float*>(workspace);
    a.part_ml = a.part_o + (size_t)kv_heads * a.nsplit * m * 128;
    a.scale_log2 = 1.4426950408889634f * 0.08838834764831845f;   // log2(e) / sqrt(128)
    cudaStream_t s = (cudaStream_t)stream;
    const bool pdl = (flags & EXL3_FLAG_PDL) != 0;
    int rc;
    switch ((m + 15) / 16) {
        case 1: rc = launch_attn_partial<1>(a, s, pdl); break;
        case 2: rc = launch_attn_partial<2>(a, s, pdl); break;
        case 3: rc = launch_attn_partial<3>(a, s, pdl); break;
        case 4: rc = launch_attn_partial<4>(a, s, pdl); break;
        case 5: rc = launch_attn_partial<5>(a, s, pdl); break;
        case 6: rc = launch_attn_partial<6>(a, s, pdl); break;
        case 7: rc = launch_attn_partial<7>(a, s, pdl); break;
        default: rc = launch_attn_partial<8>(a, s, pdl); break;
    }
    if (rc) return rc;
    const int lanes = std::min(kCombineMaxLanes, std::max(4, (a.nsplit + 3) / 4));
    return launch_kernel(attn_combine_kernel, dim3((unsigned)m, (unsigned)kv_heads), dim3(32 * lanes), 0, s, pdl, a);
}
