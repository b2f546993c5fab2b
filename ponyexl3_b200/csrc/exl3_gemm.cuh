// Prefill GEMM on the 5th-generation tensor cores: y = had( fp16( xh @ W ) ) * svh + bias
// for many rows (tokens), W decoded on the fly from the packed trellis — never materialised
// in global memory.
//
// One persistent CTA per SM walks output tiles of 256 tokens x 256 columns.  Per 64-wide
// k-step and ring stage:
//   * warp 0 (one lane) issues TMA loads: two 128-token x 64-k boxes of the rotated fp16
//     activations (128B-swizzled, the canonical K-major operand layout) and one 3-D box with
//     the 16 x 4 packed tiles of the step (2*K KiB);
//   * warps 2..9 decode those tiles in registers (the same window / codebook code as the
//     GEMV, bit-exact) and store fp16 pairs into the 128B-swizzled K-major B operand tile
//     (conflict-free 4-byte stores: the packed tile order puts 8 rows x 4 k-pairs in a warp);
//   * warp 1 (one lane) issues tcgen05.mma (M = 128 tokens, N = 256 columns, K = 16) for BOTH
//     token halves against the same decoded B tile, accumulating in two 128 x 256 fp32
//     accumulators that fill the SM's 512 tensor-memory columns; tcgen05.commit frees the
//     stage.  Sharing B between two accumulators halves the decode work per FLOP.
// When a tile's k-loop is done the decode warps become the epilogue: each thread owns one
// token (tensor-memory lane) and 128 columns, loads them with tcgen05.ld, rounds to fp16 as
// the reference does, runs the 128-point Hadamard entirely in registers, applies svh and
// bias, and writes 256 contiguous bytes (32 bytes per store when the rows are 32-byte aligned).
// A grouped launch may spread its output rows over several GPUs: the epilogue then stores each
// row into the buffer of the GPU that owns it and the last CTA announces the grid to every peer.
//
// Measured on 8192 x 5120 x 5120 (K = 4) by switching parts off with all barriers and copies
// intact: the kernel is bound by shared-memory bandwidth and by the latency of a ring turn, not
// by the tensor pipe (about half active) nor by the number of decode warps — per k-step an SM
// reads 96 KiB of MMA operands (B once per accumulator), takes 40 KiB of TMA data and moves
// about 48 KiB of decode loads and stores.  Sixteen decode warps (with the epilogue's first
// Hadamard half parked in tensor memory to fit the registers) and rings of separate depth for
// packed tiles, activations and B were measured equal and slower respectively, and are not kept.
//
// fp16 operands are exact for the decoded weights (|w| < 4) and equal to the reference's
// fp16 rounding of the rotated activations; accumulation is fp32.
// Every mbarrier wait is bounded; a wait that gives up sets ST_TC_TIMEOUT in the status
// word, every role leaves its loop, and the tensor memory is freed before the CTA exits.
#pragma once
#include <algorithm>

#include "exl3_internal.h"
#include "exl3_tc.cuh"
#include "exl3_tma.h"

namespace exl3 {

constexpr int kGemmThreads = 320;          // TMA warp, MMA warp, 8 decode / epilogue warps
constexpr int kGemmDecodeWarps = 8;
constexpr int kTileM = 256, kTileN = 256, kStepK = 64;
constexpr int kABytes = 128 * kStepK * 2;  // one 128-token activation box
constexpr int kBBytes = kTileN * kStepK * 2;
constexpr int kGemmCtrlBytes = 1024;

template <int K> struct GemmLayout {
    static constexpr int kTileWords = 8 * K;
    static constexpr int kWBytes = 64 * kTileWords * 4;                  // 16 x 4 packed tiles
    static constexpr int kStageBytes = 2 * kABytes + kBBytes + kWBytes;  // 64 KiB + 2K KiB
    static constexpr int kStages = (227 * 1024 - kGemmCtrlBytes) / kStageBytes >= 3 ? 3 : 2;
    static constexpr int kSmemBytes = kGemmCtrlBytes + kStages * kStageBytes;
};

// Two codewords -> (w_a, w_b) fp16, with the XOR constant as a run-time value (one LOP3).
template <int CB> __device__ __forceinline__ uint32_t decode_pair_rt(uint32_t cw_a, uint32_t cw_b, uint32_t xc)
{
    const uint32_t xa = codebook_word_rt<CB>(cw_a, xc);
    const uint32_t xb = codebook_word_rt<CB>(cw_b, xc);
    if (CB == CB_MUL1) {
        const uint32_t s = xa | (xb << 16);
        return h2_as_u32(__hfma2(u32_as_h2(s), u32_as_h2(0x1EEE1EEEu), u32_as_h2(0xC931C931u)));
    }
    const uint32_t lo = __byte_perm(xa, xb, 0x5410);
    const uint32_t hi = __byte_perm(xa, xb, 0x7632);
    return h2_as_u32(__hadd2(u32_as_h2(lo), u32_as_h2(hi)));
}

// One 32-byte store (sm_100: 256-bit vector stores); p must be 32-byte aligned.
__device__ __forceinline__ void st_global_256(void* p, const uint4& a, const uint4& b)
{
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

// In-register 128-point Sylvester Hadamard (un-normalised).
__device__ __forceinline__ void had128_regs(float (&v)[128])
{
#pragma unroll
    for (int h = 1; h < 128; h <<= 1)
#pragma unroll
        for (int i = 0; i < 128; i += 2 * h)
#pragma unroll
            for (int j = i; j < i + h; j++) {
                const float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
}

// One output tile: rows [m0, m_end) of the rotated activations against 256 trellis columns
// starting at tile column tn0; outputs go to y rows (row + y_row_delta), columns y_col.. ;
// svh / bias are read at sv_off.  Dense layers derive it from the tile index; grouped (MoE)
// launches read it from a device table of 8 ints per tile, where m0 >= m_end marks an unused
// slot that every role skips.
struct GemmTile {
    int m0, m_end, tn0, sv_off, y_col, ncols, y_row_delta;
    int half;      // -1: all 256 columns; 0 / 1: only the first / second 128 columns of the packed box
};
// Dense layers: the first a.n_full_tiles work items are whole tiles; the tiles that would make up
// a short last wave are cut into two 128-column halves each (half the decode, half the MMAs), so
// that the last wave keeps more SMs busy for half as long.
__device__ __forceinline__ GemmTile gemm_tile(const GemmArgs& a, int item)
{
    GemmTile t;
    if (a.tile_tab) {
        const int4 u = reinterpret_cast<const int4*>(a.tile_tab)[2 * item];
        const int4 v = reinterpret_cast<const int4*>(a.tile_tab)[2 * item + 1];
        t.m0 = u.x; t.m_end = u.y; t.tn0 = u.z; t.sv_off = u.w;
        t.y_col = v.x; t.ncols = v.y; t.y_row_delta = v.z;
        t.half = -1;
    } else {
        int tile = item, h = -1;
        if (item >= a.n_full_tiles) {
            const int j = item - a.n_full_tiles;
            tile = a.n_full_tiles + (j >> 1);
            h = j & 1;
        }
        const int n0 = (tile % a.tiles_n) * kTileN;
        t.m0 = (tile / a.tiles_n) * kTileM;
        t.m_end = a.m;
        t.tn0 = n0 / 16;
        t.half = h;
        const int c0 = n0 + (h > 0 ? 128 : 0);
        t.sv_off = c0;
        t.y_col = c0;
        t.ncols = h < 0 ? a.t_out * 16 - n0 : min(128, a.t_out * 16 - c0);
        t.y_row_delta = 0;
        if (t.ncols <= 0) t.m_end = t.m0;      // a second half beyond the last column: nothing to do
    }
    return t;
}

template <int K, int CB>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tm_x,
                const __grid_constant__ CUtensorMap tm_w)
{
    using L = GemmLayout<K>;
    constexpr int NS = L::kStages;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* a_full = reinterpret_cast<uint64_t*>(smem);      // activations + packed tiles landed
    uint64_t* b_full = a_full + 4;                             // decoded B tile written
    uint64_t* empty = b_full + 4;                              // MMAs that read the stage are done
    uint64_t* tmem_full = empty + 4;                           // accumulators complete
    uint64_t* tmem_empty = tmem_full + 1;                      // accumulators drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    uint8_t* stage0 = smem + kGemmCtrlBytes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nks = a.t_in / 4;                                // 64-wide k-steps
    const int n_tiles = a.n_items;                             // work items: tiles, or tiles and half tiles

    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(smem_u32(&a_full[s]), 1);
            mbar_init(smem_u32(&b_full[s]), kGemmDecodeWarps);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        mbar_init(smem_u32(tmem_full), 1);
        mbar_init(smem_u32(tmem_empty), kGemmDecodeWarps);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_w);
            int s = 0;
            uint32_t parity = 0;
            bool first_pass = true;
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const GemmTile ti = gemm_tile(a, tile);
                if (ti.m0 >= ti.m_end) continue;
                const int m0 = ti.m0, tn0 = ti.tn0;
                const bool two = ti.m_end - ti.m0 > a.one_acc_rows;   // tiles of up to 128 rows use one accumulator
                for (int ks = 0; ks < nks; ks++) {
                    if (!first_pass && !mbar_wait(smem_u32(&empty[s]), parity ^ 1u)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                    uint8_t* st = stage0 + (size_t)s * L::kStageBytes;
                    const uint32_t bar = smem_u32(&a_full[s]);
                    mbar_arrive_expect_tx(bar, (two ? 2 : 1) * kABytes + L::kWBytes);
                    tma_load_2d(smem_u32(st), &tm_x, ks * kStepK, m0, bar);
                    if (two) tma_load_2d(smem_u32(st + kABytes), &tm_x, ks * kStepK, m0 + 128, bar);
                    tma_load_3d(smem_u32(st + 2 * kABytes + kBBytes), &tm_w, 0, tn0, 4 * ks, bar);
                    if (++s == NS) { s = 0; parity ^= 1u; first_pass = false; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------- MMA issuer ----
        if (lane == 0) {
            int s = 0;
            uint32_t parity = 0, tile_parity = 0;
            bool first_tile = true;
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                bool two;
                uint32_t idesc;
                {
                    const GemmTile ti = gemm_tile(a, tile);
                    if (ti.m0 >= ti.m_end) continue;
                    two = ti.m_end - ti.m0 > a.one_acc_rows;
                    idesc = ti.half < 0 ? mma_idesc_f16(128, kTileN) : mma_idesc_f16(128, 128);
                }
                if (!first_tile) {   // the epilogue of the previous tile must have drained D
                    if (!mbar_wait(smem_u32(tmem_empty), tile_parity ^ 1u)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                }
                tc_fence_after_sync();
                for (int ks = 0; ks < nks; ks++) {
                    if (!mbar_wait(smem_u32(&a_full[s]), parity) ||
                        !mbar_wait(smem_u32(&b_full[s]), parity)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(stage0 + (size_t)s * L::kStageBytes);
#pragma unroll
                    for (int kk = 0; kk < kStepK / 16; kk++) {
                        const uint64_t da0 = smem_desc_sw128(sa + kk * 32);
                        const uint64_t da1 = smem_desc_sw128(sa + kABytes + kk * 32);
                        const uint64_t db = smem_desc_sw128(sa + 2 * kABytes + kk * 32);
                        const uint32_t accum = (ks | kk) != 0 ? 1u : 0u;
                        tc_mma_f16(tmem_base, da0, db, idesc, accum);
                        if (two) tc_mma_f16(tmem_base + kTileN, da1, db, idesc, accum);
                    }
                    tc_commit(smem_u32(&empty[s]));
                    if (++s == NS) { s = 0; parity ^= 1u; }
                }
                tc_commit(smem_u32(tmem_full));
                first_tile = false;
                tile_parity ^= 1u;
            }
        }
    } else {
        // ------------------------------------------------------- decode, then epilogue ----
        const int dw = warp - 2;
        const int g = lane >> 2, q = lane & 3;
        const int prev_word = (lane + 31) & 31;
        const uint32_t xc = a.cb_xor;
        LaneWords<K> lw;
        lw.init(lane);
        int s = 0;
        uint32_t parity = 0, tile_parity = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const GemmTile ti = gemm_tile(a, tile);
            if (ti.m0 >= ti.m_end) continue;
            const int m0 = ti.m0;
            for (int ks = 0; ks < nks; ks++) {
                // all lanes take the same decision: the tensor-memory loads below are warp-wide
                if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&a_full[s]), parity))) {
                    if (lane == 0) atomicOr(a.status, ST_TC_TIMEOUT);
                    goto done;
                }
                uint8_t* st = stage0 + (size_t)s * L::kStageBytes;
                uint8_t* bt = st + 2 * kABytes;
                const uint32_t* wt = reinterpret_cast<const uint32_t*>(bt + kBBytes);
                // All packed words of the warp's eight tiles are fetched before the first store: the
                // stores into the B tile could alias the packed words as far as the compiler knows,
                // so loads written after them would wait for them, tile after tile.
                // Whole tile: this warp decodes tile columns 2 dw, 2 dw + 1 of all four tile rows; half
                // tile: column 8 half + dw of the box, stored as column dw of a 128-column B tile.
                const int n_mine = ti.half < 0 ? 8 : 4;
                uint32_t pw[8][3];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (i < n_mine) {
                        const int tk = ti.half < 0 ? i >> 1 : i;
                        const int tn = ti.half < 0 ? 2 * dw + (i & 1) : 8 * ti.half + dw;
                        const uint32_t* tw = wt + (tk * 16 + tn) * L::kTileWords;
                        if (K == 4) {
                            pw[i][0] = tw[lane];
                            pw[i][1] = tw[prev_word];
                            pw[i][2] = 0u;
                        } else {
                            pw[i][0] = tw[lw.i0];
                            pw[i][1] = tw[lw.i1];
                            pw[i][2] = LaneWords<K>::kThree ? tw[lw.i2] : 0u;
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (i < n_mine) {
                        const int tk = ti.half < 0 ? i >> 1 : i;
                        const int tn = ti.half < 0 ? 2 * dw + (i & 1) : dw;
                        uint32_t cw[8];
                        if (K == 4) lane_codewords_k4(pw[i][0], pw[i][1], cw);
                        else lane_codewords<K>(pw[i][0], pw[i][1], pw[i][2], lw.sh, cw);
                        // B[n][k] K-major, 128B swizzle: n = 16 tn + g (+8), k = 16 tk + 2q (+8)
                        uint8_t* row = bt + (2 * tn) * 1024 + g * 128 + 4 * q;
                        const int c0 = ((2 * tk) ^ g) << 4, c1 = ((2 * tk + 1) ^ g) << 4;
                        *reinterpret_cast<uint32_t*>(row + c0) = decode_pair_rt<CB>(cw[0], cw[1], xc);
                        *reinterpret_cast<uint32_t*>(row + 1024 + c0) = decode_pair_rt<CB>(cw[4], cw[5], xc);
                        *reinterpret_cast<uint32_t*>(row + c1) = decode_pair_rt<CB>(cw[2], cw[3], xc);
                        *reinterpret_cast<uint32_t*>(row + 1024 + c1) = decode_pair_rt<CB>(cw[6], cw[7], xc);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&b_full[s]));
                if (++s == NS) { s = 0; parity ^= 1u; }
            }

            // ---- epilogue of this tile ----
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(tmem_full), tile_parity))) {
                if (lane == 0) atomicOr(a.status, ST_TC_TIMEOUT);
                goto done;
            }
            tile_parity ^= 1u;
            tc_fence_after_sync();
            const int quarter = warp & 3, chalf = dw >> 2;
            const int col0 = ti.y_col + 128 * chalf, sv0 = ti.sv_off + 128 * chalf;
            if (128 * chalf < ti.ncols) {
#pragma unroll 1
                for (int acc = 0; acc < (ti.m_end - m0 > a.one_acc_rows ? 2 : 1); acc++) {
                    const int row = m0 + 128 * acc + 32 * quarter + lane;
                    const uint32_t taddr =
                        tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(kTileN * acc + 128 * chalf);
                    float v[128];
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        float t32[32];
                        tmem_ld_32cols(taddr + 32 * c, t32);
#pragma unroll
                        for (int i = 0; i < 32; i++) v[32 * c + i] = __half2float(__float2half_rn(t32[i]));
                    }
                    had128_regs(v);
                    if (row < ti.m_end) {
                        const int orow = a.y_row_map ? a.y_row_map[row + ti.y_row_delta] : row + ti.y_row_delta;
                        __half* yp;
                        if (a.n_peer > 0) {      // the row belongs to the GPU that holds its token
                            const int pr = orow / a.rows_per_peer;
                            yp = a.y_peer[pr] + (int64_t)(orow - pr * a.rows_per_peer) * a.y_row_stride + col0;
                        } else {
                            yp = a.y + (int64_t)orow * a.y_row_stride + col0;
                        }
                        uint4 held = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                        for (int c = 0; c < 16; c++) {
                            float o[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) o[i] = v[8 * c + i] * EXL3_HAD_SCALE;
                            if (a.svh) {
                                const uint4 sv = *reinterpret_cast<const uint4*>(a.svh + sv0 + 8 * c);
                                const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const float2 f = __half22float2(u32_as_h2(sw[i]));
                                    o[2 * i] *= f.x;
                                    o[2 * i + 1] *= f.y;
                                }
                            }
                            __half2 h[4];
#pragma unroll
                            for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
                            if (a.bias) {
                                const uint4 bv = *reinterpret_cast<const uint4*>(a.bias + sv0 + 8 * c);
                                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                                for (int i = 0; i < 4; i++) h[i] = __hadd2(h[i], u32_as_h2(bw[i]));
                            }
                            uint4 ov;
                            ov.x = h2_as_u32(h[0]); ov.y = h2_as_u32(h[1]);
                            ov.z = h2_as_u32(h[2]); ov.w = h2_as_u32(h[3]);
                            if (!a.y_wide) {
                                *reinterpret_cast<uint4*>(yp + 8 * c) = ov;
                            } else if (c & 1) {
                                // 32-byte stores (whole sectors): what a row stored into another GPU's
                                // memory travels as
                                st_global_256(yp + 8 * (c - 1), held, ov);
                            } else {
                                held = ov;
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(tmem_empty));
        }
    }
done:
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
    if (a.n_peer > 0 && tid == 0) {
        // Rows were stored into other GPUs' memory: every CTA is counted on a local counter (the
        // barrier above orders the CTA's stores before this thread's fence), and the CTA that
        // completes the count announces this GPU's rows to every peer — one system-scope fence
        // and one arrival per peer for the whole grid.
        __threadfence();
        const unsigned done = atomicAdd(a.done_ctr, 1u) + 1u;
        if (done == gridDim.x) {
            atomicExch(a.done_ctr, 0u);           // re-armed for the next launch on this workspace
            __threadfence_system();
            for (int p = 0; p < a.n_peer; p++)
                asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.ctr_peer[p]) : "memory");
        }
    }
}

// ---- host side ----------------------------------------------------------------------------------

extern int g_gemm_one_acc_rows;   // exl3_gemm.cu: 128, or 0 from the benchmark hook (always two accumulators)
extern int g_gemm_split_last_wave;   // exl3_gemm.cu: 1, or 0 from the benchmark hook

template <int K, int CB>
static int launch_gemm_t(GemmArgs a, const __half* xh, const uint32_t* trellis, cudaStream_t s)
{
    using L = GemmLayout<K>;
    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return EXL3_E_UNSUPPORTED;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<K, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             L::kSmemBytes);
        if (e != cudaSuccess) return note_cuda(e);
        attr_set[dev] = true;
    }
    CUtensorMap tm_x, tm_w;
    {
        const uint64_t in = (uint64_t)a.t_in * 16;
        const uint64_t xdims[2] = {in, (uint64_t)a.xh_rows};
        const uint64_t xstrides[1] = {in * 2};
        const uint32_t xbox[2] = {(uint32_t)kStepK, 128u};
        int rc = make_tensor_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, xh, xdims, xstrides, xbox,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        const uint64_t dims[3] = {(uint64_t)L::kTileWords, (uint64_t)a.t_out, (uint64_t)a.t_in};
        const uint64_t strides[2] = {(uint64_t)L::kTileWords * 4, (uint64_t)a.t_out * L::kTileWords * 4};
        const uint32_t box[3] = {(uint32_t)L::kTileWords, 16u, 4u};
        rc = make_tensor_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, trellis, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
    }
    a.tiles_m = (a.m + kTileM - 1) / kTileM;
    a.tiles_n = (a.t_out * 16 + kTileN - 1) / kTileN;
    a.cb_xor = 0x3B603B60u;
    a.one_acc_rows = g_gemm_one_acc_rows;
    const int sms = device_sm_count();
    if (a.tile_tab) {
        a.n_full_tiles = a.n_items = a.n_tiles_tab;
    } else {
        // a last wave that would fill at most half of the SMs is run as half tiles
        const int n = a.tiles_m * a.tiles_n, rest = n % sms;
        a.n_full_tiles = (n > sms && rest > 0 && 2 * rest <= sms && g_gemm_split_last_wave) ? n - rest : n;
        a.n_items = a.n_full_tiles + 2 * (n - a.n_full_tiles);
    }
    const int grid = std::min(a.n_items, sms);
    gemm_kernel<K, CB><<<grid, kGemmThreads, L::kSmemBytes, s>>>(a, tm_x, tm_w);
    return check_launch();
}

}  // namespace exl3
