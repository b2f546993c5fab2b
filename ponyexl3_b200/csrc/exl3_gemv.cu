// Streamed EXL3 GEMV for 1..16 activation rows (decode and speculative verify).
//
// Work decomposition ("stream-K"): the layer is cut into items of 8x8 tiles —
// one 128-row k-block of one 128-column output block, 2*K KiB of packed trellis —
// numbered column-block-major.  The grid is persistent (a fixed number of CTAs per
// SM) and CTA i takes the contiguous item range [N*i/G, N*(i+1)/G), so every CTA
// streams the same number of bytes whatever the layer shape.
//
// Inside a CTA one producer lane feeds a shared-memory ring with the bulk-copy
// engine (cp.async.bulk, completion counted on mbarriers): eight contiguous
// 256*K-byte tile rows plus the item's 128 rotated activations per row.  Weight
// copies of the first ring fill are issued BEFORE the programmatic-launch wait, so
// under EXL3_FLAG_PDL a layer's weights stream while the previous kernel drains.
// Eight consumer warps each own one 16-column tile column of the block: a lane
// reads the 2-3 words holding its eight codewords, cuts the 16-bit windows, runs
// the codebook in registers and feeds mma.sync m16n8k16 (the packed tile order is
// the A-fragment order of W^T), accumulating in fp32.
//
// A column block whose k-range is split over several CTAs is finished by the last
// CTA to arrive (partial sums in the workspace, one atomic counter per block, no
// spinning): it adds the partials in CTA order, rounds to fp16 as the reference
// does, applies the output Hadamard-128, svh and bias, and re-arms the counter.
#include <algorithm>

#include "exl3_internal.h"

namespace exl3 {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kGemvThreads = kConsumerThreads + 32;
constexpr int kXRowBytes = 272;      // 128 halves + 16 bytes so the 8 rows of a fragment hit 8 banks
constexpr int kYStride = 132;
constexpr int kMaxStages = 16;
constexpr int kHeaderBytes = 512;

template <int K, int NMMA> struct GemvLayout {
    static constexpr int kTileWords = 8 * K;
    static constexpr int kRowBytes = 8 * kTileWords * 4;          // one tile row of the item
    static constexpr int kWeightBytes = 8 * kRowBytes;            // 2048 * K
    static constexpr int kXBytes = NMMA * 8 * kXRowBytes;
    static constexpr int kStageBytes = kWeightBytes + kXBytes;
    static constexpr int kYBytes = NMMA * 8 * kYStride * 4;
    static constexpr int kStage0 = kHeaderBytes + kYBytes;
    static_assert(kStage0 % 128 == 0 && kStageBytes % 16 == 0, "bulk copies need 16-byte alignment");
};

__device__ __forceinline__ int64_t item_begin(int64_t n_items, int cta, int grid)
{
    return n_items * cta / grid;
}
// CTA whose item range holds item i (every CTA owns at least one item).
__device__ __forceinline__ int item_owner(int64_t n_items, int64_t i, int grid)
{
    return (int)(((i + 1) * grid - 1) / n_items);
}

template <int K, int CB, int NMMA>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_kernel(const GemvArgs a)
{
    using L = GemvLayout<K, NMMA>;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    volatile int* s_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
    float* ybuf = reinterpret_cast<float*>(smem + kHeaderBytes);
    uint8_t* stage0 = smem + L::kStage0;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = a.t_in >> 3;
    const int64_t n_items = (int64_t)a.ncb * nkb;
    const int grid = gridDim.x, cta = blockIdx.x;
    const int64_t it_begin = item_begin(n_items, cta, grid);
    const int nitems = (int)(item_begin(n_items, cta + 1, grid) - it_begin);
    const int ns = a.stages;
    const int in_features = a.t_in * 16;

    if (tid == 0) {
        for (int s = 0; s < ns; s++) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), kConsumerWarps);
        }
        s_flag[0] = 0;
        mbar_fence_init();
    }
    __syncthreads();
    griddep_launch_dependents();

    // ------------------------------------------------------------------ producer ----
    if (warp == kConsumerWarps) {
        if (lane != 0) return;
        const uint32_t tx = L::kWeightBytes + (uint32_t)a.rows * 256u;
        auto issue_weights = [&](int li) {
            const int64_t it = it_begin + li;
            const int cb = (int)(it / nkb), kb = (int)(it % nkb);
            const int phys = a.blocks ? a.blocks[cb].phys : cb;
            const int s = li % ns;
            const uint32_t bar = smem_u32(&full[s]);
            const uint32_t dst = smem_u32(stage0 + (size_t)s * L::kStageBytes);
            const uint32_t* src =
                a.trellis + ((int64_t)(8 * kb) * a.t_out_total + 8 * (int64_t)phys) * L::kTileWords;
#pragma unroll
            for (int r = 0; r < 8; r++)
                bulk_g2s(dst + r * L::kRowBytes, src + (int64_t)r * a.t_out_total * L::kTileWords,
                         L::kRowBytes, bar);
        };
        auto issue_x = [&](int li) {
            const int64_t it = it_begin + li;
            const int cb = (int)(it / nkb), kb = (int)(it % nkb);
            const int xrow = a.blocks ? a.blocks[cb].xrow : 0;
            const int s = li % ns;
            const uint32_t bar = smem_u32(&full[s]);
            const uint32_t dst = smem_u32(stage0 + (size_t)s * L::kStageBytes + L::kWeightBytes);
            const __half* src = a.xh + (int64_t)xrow * in_features + 128 * kb;
            for (int n = 0; n < a.rows; n++)
                bulk_g2s(dst + n * kXRowBytes, src + (int64_t)n * in_features, 256u, bar);
        };
        // A block table is written by an earlier kernel of the stream: read it only
        // after the dependency wait.  Plain layers prefetch their weights first.
        if (a.blocks) griddep_wait();
        const int pre = nitems < ns ? nitems : ns;
        for (int li = 0; li < pre; li++) {
            mbar_arrive_expect_tx(smem_u32(&full[li]), tx);
            issue_weights(li);
        }
        if (!a.blocks) griddep_wait();
        for (int li = 0; li < pre; li++) issue_x(li);
        for (int li = pre; li < nitems; li++) {
            const int s = li % ns;
            if (!mbar_wait(smem_u32(&empty[s]), (uint32_t)((li / ns) - 1) & 1u)) {
                atomicOr(a.status, ST_WAIT_EMPTY_TIMEOUT);
                return;  // consumers run into their own bounded waits and finish
            }
            mbar_arrive_expect_tx(smem_u32(&full[s]), tx);
            issue_weights(li);
            issue_x(li);
        }
        return;
    }

    // ----------------------------------------------------------------- consumers ----
    // Partial sums and counters of the workspace belong to the previous kernel until it
    // has finished.
    griddep_wait();

    LaneWords<K> lw;
    lw.init(lane);
    const int g = lane >> 2, tig = lane & 3;
    float acc[NMMA][4];
#pragma unroll
    for (int m = 0; m < NMMA; m++)
#pragma unroll
        for (int q = 0; q < 4; q++) acc[m][q] = 0.f;

    bool failed = false;
    const int first_cb = (int)(it_begin / nkb);
    int seg_kb0 = (int)(it_begin % nkb);

    for (int li = 0; li < nitems; li++) {
        const int64_t it = it_begin + li;
        const int cb = (int)(it / nkb), kb = (int)(it % nkb);
        const int s = li % ns;
        if (!failed && !mbar_wait(smem_u32(&full[s]), (uint32_t)(li / ns) & 1u)) {
            failed = true;
            if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
        }
        if (!failed) {
            const uint8_t* st = stage0 + (size_t)s * L::kStageBytes;
            const uint32_t* wst = reinterpret_cast<const uint32_t*>(st) + warp * L::kTileWords;
            const uint8_t* xst = st + L::kWeightBytes;
#pragma unroll
            for (int tk = 0; tk < 8; tk++) {
                const uint32_t* tw = wst + tk * 8 * L::kTileWords;
                const uint32_t wa = tw[lw.i0], wb = tw[lw.i1];
                const uint32_t wc = LaneWords<K>::kThree ? tw[lw.i2] : 0u;
                uint32_t cw[8];
                lane_codewords<K>(wa, wb, wc, lw.sh, cw);
                uint32_t fa[4];
                fa[0] = decode_pair<CB>(cw[0], cw[1]);
                fa[1] = decode_pair<CB>(cw[4], cw[5]);
                fa[2] = decode_pair<CB>(cw[2], cw[3]);
                fa[3] = decode_pair<CB>(cw[6], cw[7]);
#pragma unroll
                for (int m = 0; m < NMMA; m++) {
                    const int n = g + 8 * m;
                    const uint32_t* xr =
                        reinterpret_cast<const uint32_t*>(xst + n * kXRowBytes) + tk * 8 + tig;
                    const uint32_t b0 = n < a.rows ? xr[0] : 0u;
                    const uint32_t b1 = n < a.rows ? xr[4] : 0u;
                    mma_16816(acc[m], fa, b0, b1);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[s]));

        if (kb != nkb - 1 && li != nitems - 1) continue;

        // ---- end of this CTA's share of column block cb -------------------------------
#pragma unroll
        for (int m = 0; m < NMMA; m++) {
            float* y0 = ybuf + (2 * tig + 8 * m) * kYStride + 16 * warp + g;
            y0[0] = acc[m][0];
            y0[kYStride] = acc[m][1];
            y0[8] = acc[m][2];
            y0[kYStride + 8] = acc[m][3];
            acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
        }
        named_bar_sync(1, kConsumerThreads);
        bool finish = (seg_kb0 == 0 && kb == nkb - 1);
        if (!finish) {
            const int which = (cb == first_cb) ? 0 : 1;
            float* slot = a.partials + ((size_t)(cta * 2 + which) * a.rows) * 128;
            for (int i = tid; i < a.rows * 128; i += kConsumerThreads)
                slot[i] = ybuf[(i >> 7) * kYStride + (i & 127)];
            __threadfence();
            named_bar_sync(1, kConsumerThreads);
            const int c_first = item_owner(n_items, (int64_t)cb * nkb, grid);
            const int c_last = item_owner(n_items, (int64_t)(cb + 1) * nkb - 1, grid);
            if (tid == 0) {
                const unsigned old = atomicAdd(&a.counters[cb], 1u);
                s_flag[0] = (old == (unsigned)(c_last - c_first)) ? 1 : 0;
            }
            named_bar_sync(1, kConsumerThreads);
            finish = s_flag[0] != 0;
            if (finish) {
                __threadfence();
                for (int i = tid; i < a.rows * 128; i += kConsumerThreads) {
                    float sum = 0.f;
                    for (int c = c_first; c <= c_last; c++) {
                        const int wh = ((int)(item_begin(n_items, c, grid) / nkb) == cb) ? 0 : 1;
                        sum += ld_cg_f32(a.partials + ((size_t)(c * 2 + wh) * a.rows) * 128 + i);
                    }
                    ybuf[(i >> 7) * kYStride + (i & 127)] = sum;
                }
                if (tid == 0) a.counters[cb] = 0u;
                named_bar_sync(1, kConsumerThreads);
            }
        }
        if (finish) {
            const int sv_off = a.blocks ? a.blocks[cb].sv_off : cb * 128;
            const int y_off = a.blocks ? a.blocks[cb].y_off : cb * 128;
            for (int n = warp; n < a.rows; n += kConsumerWarps) {
                float v[4];
#pragma unroll
                for (int q = 0; q < 4; q++)
                    v[q] = __half2float(__float2half_rn(ybuf[n * kYStride + 4 * lane + q]));
                if (!a.raw_out) {
                    had128_warp(v, lane);
#pragma unroll
                    for (int q = 0; q < 4; q++) v[q] *= EXL3_HAD_SCALE;
                    if (a.svh && sv_off >= 0) {
                        const uint2 sv = *reinterpret_cast<const uint2*>(a.svh + sv_off + 4 * lane);
                        const float2 s0 = __half22float2(u32_as_h2(sv.x));
                        const float2 s1 = __half22float2(u32_as_h2(sv.y));
                        v[0] *= s0.x; v[1] *= s0.y; v[2] *= s1.x; v[3] *= s1.y;
                    }
                }
                __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                if (a.bias && sv_off >= 0 && !a.raw_out) {
                    const uint2 bv = *reinterpret_cast<const uint2*>(a.bias + sv_off + 4 * lane);
                    h0 = __hadd2(h0, u32_as_h2(bv.x));
                    h1 = __hadd2(h1, u32_as_h2(bv.y));
                }
                uint2 o;
                o.x = h2_as_u32(h0);
                o.y = h2_as_u32(h1);
                *reinterpret_cast<uint2*>(a.y + (int64_t)n * a.y_row_stride + y_off + 4 * lane) = o;
            }
        }
        named_bar_sync(1, kConsumerThreads);  // ybuf and s_flag are reused by the next block
        seg_kb0 = 0;
    }
}

// ---- host side ----------------------------------------------------------------------------------

static int g_ctas_per_sm = 2;
static int g_smem_budget = 110 * 1024;

void gemv_set_tuning(int ctas_per_sm, int smem_budget_bytes)
{
    if (ctas_per_sm >= 1 && ctas_per_sm <= 2) g_ctas_per_sm = ctas_per_sm;
    if (smem_budget_bytes >= 32 * 1024 && smem_budget_bytes <= 226 * 1024)
        g_smem_budget = smem_budget_bytes;
}

template <int K, int CB, int NMMA>
static int launch_gemv_t(GemvArgs a, bool pdl, cudaStream_t s)
{
    using L = GemvLayout<K, NMMA>;
    int budget = g_smem_budget;
    if (g_ctas_per_sm == 1) budget = std::max(budget, 200 * 1024);
    int stages = (budget - L::kStage0) / L::kStageBytes;
    stages = std::min(stages, kMaxStages);
    if (stages < 2) return EXL3_E_UNSUPPORTED;
    a.stages = stages;
    const size_t smem = (size_t)L::kStage0 + (size_t)stages * L::kStageBytes;

    static bool attr_set[16] = {};  // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<K, CB, NMMA>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return note_cuda(e);
        attr_set[dev] = true;
    }
    const int64_t n_items = (int64_t)a.ncb * (a.t_in >> 3);
    int64_t grid = (int64_t)device_sm_count() * g_ctas_per_sm;
    grid = std::min<int64_t>(grid, std::min<int64_t>(n_items, kMaxCtas));

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return note_cuda(cudaLaunchKernelEx(&cfg, gemv_kernel<K, CB, NMMA>, a));
}

template <int K> static int launch_gemv_k(const GemvArgs& a, int cb, bool pdl, cudaStream_t s)
{
    const bool two = a.rows > 8;
    switch (cb) {
        case CB_3INST:
            return two ? launch_gemv_t<K, CB_3INST, 2>(a, pdl, s) : launch_gemv_t<K, CB_3INST, 1>(a, pdl, s);
        case CB_MCG:
            return two ? launch_gemv_t<K, CB_MCG, 2>(a, pdl, s) : launch_gemv_t<K, CB_MCG, 1>(a, pdl, s);
        case CB_MUL1:
            return two ? launch_gemv_t<K, CB_MUL1, 2>(a, pdl, s) : launch_gemv_t<K, CB_MUL1, 1>(a, pdl, s);
        default: return EXL3_E_CODEBOOK;
    }
}

int launch_gemv(const GemvArgs& a, int k, int cb, bool pdl, cudaStream_t s)
{
    switch (k) {
        case 1: return launch_gemv_k<1>(a, cb, pdl, s);
        case 2: return launch_gemv_k<2>(a, cb, pdl, s);
        case 3: return launch_gemv_k<3>(a, cb, pdl, s);
        case 4: return launch_gemv_k<4>(a, cb, pdl, s);
        case 5: return launch_gemv_k<5>(a, cb, pdl, s);
        case 6: return launch_gemv_k<6>(a, cb, pdl, s);
        case 7: return launch_gemv_k<7>(a, cb, pdl, s);
        case 8: return launch_gemv_k<8>(a, cb, pdl, s);
        default: return EXL3_E_K;
    }
}

}  // namespace exl3
