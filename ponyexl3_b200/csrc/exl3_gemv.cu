// Streamed EXL3 GEMV for 1..16 activation rows (decode and speculative verify).
//
// Work decomposition ("stream-K"): the layer is cut into items of 8x8 tiles —
// one 128-row k-block of one 128-column output block, 2*K KiB of packed trellis —
// numbered column-block-major.  The grid is persistent (a fixed number of CTAs per
// SM) and CTA i takes the contiguous item range [N*i/G, N*(i+1)/G), so every CTA
// streams the same number of bytes whatever the layer shape.
//
// Inside a CTA one producer lane feeds a shared-memory ring with TMA tensor copies
// (completion counted on mbarriers): ONE 3-D box per item for the 8x8 packed tiles
// and ONE 128B-swizzled 3-D box for the item's 128 rotated activations of every row.
// (Issuing the eight tile rows as separate bulk copies made the single producer lane
// the bottleneck: a copy instruction costs tens of cycles to issue.)  Weight copies
// of the first ring fill are issued BEFORE the programmatic-launch wait, so under
// EXL3_FLAG_PDL a layer's weights stream while the previous kernel drains.
//
// Sixteen consumer warps (the decode chains need ~32 resident warps per SM to hide
// their latency; two CTAs per SM give that); warp w owns tile columns 2*(w&3),
// 2*(w&3)+1 of the block and the k-quarter (w>>2) of the item, so one activation
// fragment load serves two tiles.
// The decode is bound by the half-rate logic pipe of the SM (64 lanes/clk: LOP3, PRMT;
// shifts run at a quarter), so the inner loop is written to spend exactly two logic
// operations per weight at K = 4 — one byte-permute to cut the codeword window, one
// LOP3 for the codebook mask — and pushes everything else to other pipes: shifts
// become wide integer multiplies, and the two fp16 halves of a 3INST value are added
// by HADD2 with broadcast operands straight into a (w, w) register.  Each weight thus
// occupies both k-slots of a 32-bit A-fragment register of mma.sync m16n8k16 and the
// activations arrive as (x, 0) words, which costs a second MMA per tile on the
// otherwise idle tensor pipe instead of byte-permutes on the saturated one.
// With EXL3_FLAG_FAST_ACCUM the HADD2 is skipped: the register keeps the two halves
// (lo, hi), the activations arrive as (x, x), and the MMA adds lo*x + hi*x in fp32
// (weights then differ from the reference's fp16-rounded sum by under 2^-11 relative).
//
// A column block whose k-range is split over several CTAs is finished by the last
// CTA to arrive (partial sums in the workspace, one atomic counter per block, no
// spinning): it adds the partials in CTA order, rounds to fp16 as the reference
// does, applies the output Hadamard-128, svh and bias, and re-arms the counter.
#include <algorithm>

#include "exl3_internal.h"
#include "exl3_tma.h"

namespace exl3 {

constexpr int kConsumerWarps = 16;
constexpr int kKGroups = kConsumerWarps / 4;        // warps that split the item's 8 tile rows
constexpr int kTileRowsPerWarp = 8 / kKGroups;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kGemvThreads = kConsumerThreads + 32;
constexpr int kYStride = 132;
constexpr int kMaxStages = 16;
constexpr int kHeaderBytes = 512;

template <int K, int NMMA> struct GemvLayout {
    static constexpr int kTileWords = 8 * K;
    static constexpr int kWeightBytes = 64 * kTileWords * 4;      // 8x8 tiles: 2048 * K
    static constexpr int kYBytes = kKGroups * NMMA * 8 * kYStride * 4;   // one copy per k-group
    static constexpr int kStage0 = (kHeaderBytes + kYBytes + 1023) / 1024 * 1024;
};

// Activations of one item in shared memory: 4 quarters of 32 k-values, each `rows`
// lines of 128 bytes (32 words of (x, 0) or (x, x)); the TMA engine XOR-swizzles the
// 16-byte chunk index with the 128-byte line index (128B swizzle).
__host__ __device__ inline int x_stage_bytes(int rows) { return (4 * rows * 128 + 1023) / 1024 * 1024; }

__device__ __forceinline__ int64_t item_begin(int64_t n_items, int cta, int grid)
{
    return n_items * cta / grid;
}
// CTA whose item range holds item i (every CTA owns at least one item).
__device__ __forceinline__ int item_owner(int64_t n_items, int64_t i, int grid)
{
    return (int)(((i + 1) * grid - 1) / n_items);
}

// (w, w) from the two-halves word of 3INST / MCG, or from the MUL1 pattern.
template <int CB, bool FAST> __device__ __forceinline__ uint32_t weight_slot_pair(uint32_t cw)
{
    const uint32_t r = codebook_word<CB>(cw);
    if (CB == CB_MUL1) {
        const __half2 h = u32_as_h2(r * 0x00010001u);
        return h2_as_u32(__hfma2(h, u32_as_h2(0x1EEE1EEEu), u32_as_h2(0xC931C931u)));
    }
    if (FAST) return r;
    const __half2 h = u32_as_h2(r);
    return h2_as_u32(__hadd2(__low2half2(h), __high2half2(h)));
}

template <int K, int CB, int NMMA, bool FAST>
__global__ void __launch_bounds__(kGemvThreads, 2)
    gemv_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_x)
{
    using L = GemvLayout<K, NMMA>;
    extern __shared__ __align__(1024) uint8_t smem[];
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
    const int xbytes = x_stage_bytes(a.rows);
    const int stage_bytes = xbytes + L::kWeightBytes;

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
        const uint32_t tx = L::kWeightBytes + (uint32_t)a.rows * 512u;
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
        // (cb, kb) of the next item to fetch, advanced without divisions: the producer is one
        // lane sharing its scheduler with busy consumer warps, so its per-item instruction
        // chain must stay short or it becomes the bottleneck of the whole CTA.
        int w_cb = (int)(it_begin / nkb), w_kb = (int)(it_begin % nkb);
        int x_cb = w_cb, x_kb = w_kb;
        auto issue_weights = [&](int s) {
            const int phys = a.blocks ? a.blocks[w_cb].phys : w_cb;
            tma_load_3d(smem_u32(stage0 + (size_t)s * stage_bytes + xbytes), &tm_w, 0, 8 * phys,
                        8 * w_kb, smem_u32(&full[s]));
            if (++w_kb == nkb) { w_kb = 0; ++w_cb; }
        };
        auto issue_x = [&](int s) {
            const int xrow = a.blocks ? a.blocks[x_cb].xrow : 0;
            tma_load_3d(smem_u32(stage0 + (size_t)s * stage_bytes), &tm_x, 0, xrow, 4 * x_kb,
                        smem_u32(&full[s]));
            if (++x_kb == nkb) { x_kb = 0; ++x_cb; }
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
        int s = 0;
        uint32_t parity = 0;
#ifdef EXL3_PROFILE
        long long pprof_wait = 0, pprof_start = clock64();
#endif
        for (int li = pre; li < nitems; li++) {
#ifdef EXL3_PROFILE
            long long tq0 = clock64();
#endif
            if (!mbar_wait(smem_u32(&empty[s]), parity)) {
                atomicOr(a.status, ST_WAIT_EMPTY_TIMEOUT);
                return;  // consumers run into their own bounded waits and finish
            }
#ifdef EXL3_PROFILE
            pprof_wait += clock64() - tq0;
            if (li == nitems - 1 && a.prof) {
                a.prof[(cta * 17 + 16) * 4 + 0] = pprof_wait;
                a.prof[(cta * 17 + 16) * 4 + 2] = clock64() - pprof_start;
            }
#endif
            mbar_arrive_expect_tx(smem_u32(&full[s]), tx);
            issue_weights(s);
            issue_x(s);
            if (++s == ns) { s = 0; parity ^= 1u; }
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
    const int tnp = warp & 3, kg = warp >> 2;
    const int prev_word = (lane + 31) & 31;

    // Byte offsets of this lane's activation words for the tile rows of its k-group:
    // element e = 16*tk + 2*tig (+8 for the second MMA) of the 128-value block sits in
    // quarter e/32, line `row`, chunk ((e%32)/4) ^ (line & 7), byte 8*(tig&1).
    int xoff[kTileRowsPerWarp][2];
#pragma unroll
    for (int tl = 0; tl < kTileRowsPerWarp; tl++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int tk = kTileRowsPerWarp * kg + tl;
            const int q = tk >> 1;
            const int chunk = 4 * (tk & 1) + (tig >> 1) + 2 * h;
            const int line = q * a.rows + g;  // rows of the second MMA group add 8 lines
            xoff[tl][h] = line * 128 + ((chunk ^ (line & 7)) << 4) + 8 * (tig & 1);
        }

    float acc[2][NMMA][4];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int m = 0; m < NMMA; m++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[t][m][q] = 0.f;

#ifdef EXL3_PROFILE
    long long prof_wait = 0, prof_comp = 0, prof_start = clock64();
#endif
    bool failed = false;
    const int first_cb = (int)(it_begin / nkb);
    int seg_kb0 = (int)(it_begin % nkb);

    int cb = first_cb, kb = seg_kb0 - 1, s = -1;
    uint32_t parity = 0;
    for (int li = 0; li < nitems; li++) {
        if (++kb == nkb) { kb = 0; ++cb; }
        if (++s == ns) { s = 0; parity ^= 1u; }
#ifdef EXL3_PROFILE
        long long tp0 = clock64();
#endif
        if (!failed && !mbar_wait(smem_u32(&full[s]), parity)) {
            failed = true;
            if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
        }
#ifdef EXL3_PROFILE
        long long tp1 = clock64();
        prof_wait += tp1 - tp0;
#endif
        if (!failed) {
            const uint8_t* xst = stage0 + (size_t)s * stage_bytes;
            const uint32_t* wst = reinterpret_cast<const uint32_t*>(xst + xbytes) +
                                  (kTileRowsPerWarp * kg * 8 + 2 * tnp) * L::kTileWords;
#pragma unroll
            for (int tl = 0; tl < kTileRowsPerWarp; tl++) {
                // activation fragments: rows g (+8), k-slots of this lane
                uint2 xb[NMMA][2];
#pragma unroll
                for (int m = 0; m < NMMA; m++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        xb[m][h] = make_uint2(0u, 0u);
                        if (g + 8 * m < a.rows) {
                            // line index grows by 8 for the second row group: the swizzle
                            // term (line & 7) is unchanged
                            xb[m][h] = *reinterpret_cast<const uint2*>(xst + xoff[tl][h] + m * 1024);
                        }
                    }
#pragma unroll
                for (int t = 0; t < 2; t++) {
                    const uint32_t* tw = wst + (tl * 8 + t) * L::kTileWords;
                    uint32_t cw[8];
                    if (K == 4) {
                        lane_codewords_k4(tw[lane], tw[prev_word], cw);
                    } else {
                        const uint32_t wa = tw[lw.i0], wb = tw[lw.i1];
                        const uint32_t wc = LaneWords<K>::kThree ? tw[lw.i2] : 0u;
                        lane_codewords<K>(wa, wb, wc, lw.sh, cw);
                    }
                    uint32_t d[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) d[j] = weight_slot_pair<CB, FAST>(cw[j]);
                    // tile rows 2*tig, 2*tig+1 (codewords 0,4 | 1,5), then rows +8 (2,6 | 3,7)
                    const uint32_t a1[4] = {d[0], d[4], d[1], d[5]};
                    const uint32_t a2[4] = {d[2], d[6], d[3], d[7]};
#pragma unroll
                    for (int m = 0; m < NMMA; m++) {
                        mma_16816(acc[t][m], a1, xb[m][0].x, xb[m][0].y);
                        mma_16816(acc[t][m], a2, xb[m][1].x, xb[m][1].y);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[s]));
#ifdef EXL3_PROFILE
        long long tp2 = clock64();
        prof_comp += tp2 - tp1;
        if (li == nitems - 1 && lane == 0 && a.prof) {
            a.prof[(cta * 17 + warp) * 4 + 0] = prof_wait;
            a.prof[(cta * 17 + warp) * 4 + 1] = prof_comp;
            a.prof[(cta * 17 + warp) * 4 + 2] = tp2 - prof_start;
            a.prof[(cta * 17 + warp) * 4 + 3] = nitems;
        }
#endif

        if (kb != nkb - 1 && li != nitems - 1) continue;

        // ---- end of this CTA's share of column block cb -------------------------------
        constexpr int kYCopy = NMMA * 8 * kYStride;  // floats per k-group copy
        float* yk = ybuf + kg * kYCopy;
#pragma unroll
        for (int t = 0; t < 2; t++)
#pragma unroll
            for (int m = 0; m < NMMA; m++) {
                float* y0 = yk + (2 * tig + 8 * m) * kYStride + 16 * (2 * tnp + t) + g;
                y0[0] = acc[t][m][0];
                y0[kYStride] = acc[t][m][1];
                y0[8] = acc[t][m][2];
                y0[kYStride + 8] = acc[t][m][3];
#pragma unroll
                for (int q = 0; q < 4; q++) acc[t][m][q] = 0.f;
            }
        named_bar_sync(1, kConsumerThreads);
        auto ysum = [&](int o) {  // the k-groups' copies, added in a fixed order
            float f = ybuf[o];
#pragma unroll
            for (int c = 1; c < kKGroups; c++) f += ybuf[o + c * kYCopy];
            return f;
        };
        bool finish = (seg_kb0 == 0 && kb == nkb - 1);
        if (!finish) {
            const int which = (cb == first_cb) ? 0 : 1;
            float* slot = a.partials + ((size_t)(cta * 2 + which) * a.rows) * 128;
            for (int i = tid; i < a.rows * 128; i += kConsumerThreads) {
                const int o = (i >> 7) * kYStride + (i & 127);
                slot[i] = ysum(o);
            }
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
            const bool direct = (seg_kb0 == 0 && kb == nkb - 1);  // k-group copies still apart
            const int sv_off = a.blocks ? a.blocks[cb].sv_off : cb * 128;
            const int y_off = a.blocks ? a.blocks[cb].y_off : cb * 128;
            for (int n = warp; n < a.rows; n += kConsumerWarps) {
                float v[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int o = n * kYStride + 4 * lane + q;
                    const float f = direct ? ysum(o) : ybuf[o];
                    v[q] = __half2float(__float2half_rn(f));
                }
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

template <int K, int CB, int NMMA, bool FAST>
static int launch_gemv_t(GemvArgs a, bool pdl, cudaStream_t s)
{
    using L = GemvLayout<K, NMMA>;
    int budget = g_smem_budget;
    if (g_ctas_per_sm == 1) budget = std::max(budget, 200 * 1024);
    const int stage_bytes = x_stage_bytes(a.rows) + L::kWeightBytes;
    int stages = (budget - L::kStage0) / stage_bytes;
    stages = std::min(stages, kMaxStages);
    if (stages < 2) return EXL3_E_UNSUPPORTED;
    a.stages = stages;
    const size_t smem = (size_t)L::kStage0 + (size_t)stages * stage_bytes;

    static bool attr_set[16] = {};  // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<K, CB, NMMA, FAST>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return note_cuda(e);
        attr_set[dev] = true;
    }
    CUtensorMap tm_w, tm_x;
    {
        const uint64_t dims[3] = {(uint64_t)L::kTileWords, (uint64_t)a.t_out_total, (uint64_t)a.t_in};
        const uint64_t strides[2] = {(uint64_t)L::kTileWords * 4,
                                     (uint64_t)a.t_out_total * L::kTileWords * 4};
        const uint32_t box[3] = {(uint32_t)L::kTileWords, 8u, 8u};
        int rc = make_tensor_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.trellis, dims, strides,
                                 box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        // xh viewed as (32 words, rows, in/32): one box brings the four quarters of a k-block
        const uint64_t in = (uint64_t)a.t_in * 16;
        const uint64_t xdims[3] = {32u, (uint64_t)a.x_rows_total, in / 32};
        const uint64_t xstrides[2] = {in * 4, 128u};
        const uint32_t xbox[3] = {32u, (uint32_t)a.rows, 4u};
        rc = make_tensor_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.xh, xdims, xstrides, xbox,
                             CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
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
    return note_cuda(cudaLaunchKernelEx(&cfg, gemv_kernel<K, CB, NMMA, FAST>, a, tm_w, tm_x));
}

template <int K, int CB> static int launch_gemv_kc(const GemvArgs& a, bool pdl, cudaStream_t s)
{
    const bool two = a.rows > 8;
    // MUL1 has no two-halves form: its fast mode is the exact one
    const bool fast = a.fast_accum && CB != CB_MUL1;
    if (fast)
        return two ? launch_gemv_t<K, CB, 2, (CB != CB_MUL1)>(a, pdl, s)
                   : launch_gemv_t<K, CB, 1, (CB != CB_MUL1)>(a, pdl, s);
    return two ? launch_gemv_t<K, CB, 2, false>(a, pdl, s) : launch_gemv_t<K, CB, 1, false>(a, pdl, s);
}

template <int K> static int launch_gemv_k(const GemvArgs& a, int cb, bool pdl, cudaStream_t s)
{
    switch (cb) {
        case CB_3INST: return launch_gemv_kc<K, CB_3INST>(a, pdl, s);
        case CB_MCG: return launch_gemv_kc<K, CB_MCG>(a, pdl, s);
        case CB_MUL1: return launch_gemv_kc<K, CB_MUL1>(a, pdl, s);
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
