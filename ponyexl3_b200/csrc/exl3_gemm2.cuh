// Prefill GEMM for dense layers with many rows, on PAIRS of SMs (tcgen05.mma.cta_group::2).
//
// The one-CTA kernel (exl3_gemm.cuh) is bound by shared-memory bandwidth, not by the tensor
// core: per 64-wide k-step an SM moves 96 KiB of MMA operands out of shared memory (the decoded
// B tile is read once per accumulator), 40 KiB of TMA data and 48 KiB of decode traffic into
// it — about 1,470 cycles at 128 bytes per cycle against 1,024 cycles of MMA.  A pair of CTAs
// that shares one 256-column B tile halves the B traffic AND the decode work of each SM:
//
//   cluster of 2 CTAs, output tile 512 tokens x 256 columns;
//   CTA r holds tokens [256 r, 256 r + 256) of the tile as two 128-row accumulators
//   (all 512 tensor-memory columns) and decodes columns [128 r, 128 r + 128) of the B tile;
//   every tcgen05.mma is M = 256 (128 rows from each CTA) x N = 256 (128 columns from each
//   CTA's shared memory) x K = 16, issued by one thread of CTA 0 for both SMs.
//
// Per CTA and k-step: 64 KiB of MMA operands, 36 KiB of TMA data, 24 KiB of decode traffic
// (~990 cycles), and 32 instead of 64 packed tiles to decode.
//
// Rings (every CTA has the same shared-memory layout, so one offset names a barrier or a tile
// in both CTAs):
//   packed tiles   kWStages deep, local: TMA (warp 2) -> decode warps -> w_empty -> TMA
//   A + B stages   kStages deep: activations by TMA (warp 0 of each CTA, its own a_full), B
//                  written by the CTA's decode warps (its own b_full).  Warp 1 of CTA 1 waits for
//                  both and sends ONE arrival per stage to peer_ready of CTA 0, where the MMA
//                  issuer waits for its own a_full and b_full and for peer_ready.  A multicast
//                  tcgen05.commit (`empty`) frees the stage in both CTAs when its MMAs are done.
// tmem_full is committed to both CTAs; tmem_empty of CTA 0 counts the epilogue warps of both.
// Every wait is bounded; a wait that gives up sets ST_TC_TIMEOUT, all roles leave their loops,
// the pair meets at a cluster barrier and frees the tensor memory.
//
// Measured (8192 x 5120 x 5120, K = 4): results bit-identical to the one-CTA kernel, 0.43 ms
// against its 0.40 ms, so it is NOT the default (exl3_tune_gemm_pairs(1) selects it).  With the
// MMAs and the decode arithmetic both switched off (all barriers and copies intact) it still
// takes 0.40 ms: a stage's turn through the pair — TMA, the arrival forwarded from CTA 1, the
// multicast commit back — lasts about 4 us, three times the one-CTA ring's, and four 48 KiB
// stages do not cover it.  A first version in which CTA 1's TMA and its eight decode warps
// signalled CTA 0's barriers directly (nine messages across the pair per stage) took 0.60 ms.
#pragma once
#include <algorithm>

#include "exl3_gemm.cuh"

namespace exl3 {

constexpr int kPairThreads = 352;          // A-TMA warp, MMA warp, W-TMA warp, 8 decode / epilogue warps
constexpr int kPairDecodeWarps = 8;
constexpr int kPairFirstDecodeWarp = 3;
constexpr int kPairTileM = 512;            // tokens per pair tile (256 per CTA)
constexpr int kPairStages = 4;
constexpr int kPairMaxWStages = 8;
constexpr int kPairBBytes = 128 * kStepK * 2;   // this CTA's half of the decoded B tile

template <int K> struct PairLayout {
    static constexpr int kTileWords = 8 * K;
    static constexpr int kWBytes = 32 * kTileWords * 4;                  // 8 x 4 packed tiles: K KiB
    static constexpr int kStageBytes = 2 * kABytes + kPairBBytes;        // 48 KiB
    static constexpr int kWOff = kGemmCtrlBytes + kPairStages * kStageBytes;
    static constexpr int kWRoom = (226 * 1024 - kWOff) / kWBytes;
    static constexpr int kWStages = kWRoom > kPairMaxWStages ? kPairMaxWStages : kWRoom;
    static constexpr int kSmemBytes = kWOff + kWStages * kWBytes;
    static_assert(kWStages >= 3, "packed-tile ring too short");
};

// ---- cluster-scope helpers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kWaitSpins; i++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
// ---- tensor memory and MMAs of a CTA pair ------------------------------------------------------
// Executed by the same warp index in BOTH CTAs, with the same destination offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate)
{
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs when every MMA issued so far is done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(bar),
        "h"((uint16_t)3)
        : "memory");
}

template <int K, int CB>
__global__ void __launch_bounds__(kPairThreads, 1)
    gemm_pair_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tm_x,
                     const __grid_constant__ CUtensorMap tm_w)
{
    using L = PairLayout<K>;
    constexpr int NS = kPairStages, NW = L::kWStages;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint64_t* w_full = bars;                                   // packed tiles landed (local)            [NW]
    uint64_t* w_empty = w_full + kPairMaxWStages;              // ... read by the local decode warps      [NW]
    uint64_t* a_full = w_empty + kPairMaxWStages;              // local: this CTA's activation boxes landed  [NS]
    uint64_t* b_full = a_full + kPairStages;                   // local: this CTA's half of B written       [NS]
    uint64_t* empty = b_full + kPairStages;                    // local: the MMAs that read the stage are done [NS]
    uint64_t* peer_ready = empty + kPairStages;                // CTA 0: CTA 1's stage is complete          [NS]
    uint64_t* tmem_full = peer_ready + kPairStages;            // local: accumulators complete
    uint64_t* tmem_empty = tmem_full + 1;                      // CTA 0: accumulators of both CTAs drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
    uint8_t* stage0 = smem + kGemmCtrlBytes;
    uint8_t* w_ring = smem + L::kWOff;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_cta_rank();
    const bool leader = rank == 0;
    const int nks = a.t_in / 4;                                // 64-wide k-steps
    const int n_tiles = a.tiles_m * a.tiles_n;                 // pair tiles
    const int first_tile = (int)(blockIdx.x >> 1), tile_step = (int)(gridDim.x >> 1);

    if (tid == 0) {
        for (int s = 0; s < NW; s++) {
            mbar_init(smem_u32(&w_full[s]), 1);
            mbar_init(smem_u32(&w_empty[s]), kPairDecodeWarps);
        }
        for (int s = 0; s < NS; s++) {
            mbar_init(smem_u32(&a_full[s]), 1);
            mbar_init(smem_u32(&b_full[s]), kPairDecodeWarps);
            mbar_init(smem_u32(&empty[s]), 1);
            mbar_init(smem_u32(&peer_ready[s]), 1);
        }
        mbar_init(smem_u32(tmem_full), 1);
        mbar_init(smem_u32(tmem_empty), 2 * kPairDecodeWarps);
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();            // both CTAs' barriers exist before anything is signalled across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------- TMA producer: activations ----
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            int s = 0;
            uint32_t parity = 0;
            bool first_pass = true;
            for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
                const int m0 = (tile / a.tiles_n) * kPairTileM + 256 * (int)rank;
                for (int ks = 0; ks < nks; ks++) {
                    if (!first_pass && !mbar_wait_cluster(smem_u32(&empty[s]), parity ^ 1u)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                    uint8_t* st = stage0 + (size_t)s * L::kStageBytes;
                    const uint32_t bar = smem_u32(&a_full[s]);
                    mbar_arrive_expect_tx(bar, 2 * kABytes);
                    tma_load_2d(smem_u32(st), &tm_x, ks * kStepK, m0, bar);
                    tma_load_2d(smem_u32(st + kABytes), &tm_x, ks * kStepK, m0 + 128, bar);
                    if (++s == NS) { s = 0; parity ^= 1u; first_pass = false; }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------- TMA producer: packed tiles ----
        if (lane == 0) {
            tma_prefetch_desc(&tm_w);
            int s = 0;
            uint32_t parity = 0;
            bool first_pass = true;
            for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
                const int tn0 = (tile % a.tiles_n) * (kTileN / 16) + 8 * (int)rank;   // this CTA's 8 tile columns
                for (int ks = 0; ks < nks; ks++) {
                    if (!first_pass && !mbar_wait(smem_u32(&w_empty[s]), parity ^ 1u)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                    const uint32_t bar = smem_u32(&w_full[s]);
                    mbar_arrive_expect_tx(bar, L::kWBytes);
                    tma_load_3d(smem_u32(w_ring + (size_t)s * L::kWBytes), &tm_w, 0, tn0, 4 * ks, bar);
                    if (++s == NW) { s = 0; parity ^= 1u; first_pass = false; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------- MMA issuer (CTA 0, for both SMs) ----
        if (leader && lane == 0) {
            constexpr uint32_t idesc = mma_idesc_f16(256, kTileN);
            int s = 0;
            uint32_t parity = 0, tile_parity = 0;
            bool first = true;
            for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
                if (!first) {   // the epilogues of both CTAs must have drained the accumulators
                    if (!mbar_wait_cluster(smem_u32(tmem_empty), tile_parity ^ 1u)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                }
                tc_fence_after_sync();
                for (int ks = 0; ks < nks; ks++) {
                    if (!mbar_wait(smem_u32(&a_full[s]), parity) || !mbar_wait(smem_u32(&b_full[s]), parity) ||
                        !mbar_wait_cluster(smem_u32(&peer_ready[s]), parity)) {
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
                        tc_mma_f16_pair(tmem_base, da0, db, idesc, accum);
                        tc_mma_f16_pair(tmem_base + kTileN, da1, db, idesc, accum);
                    }
                    tc_commit_pair(smem_u32(&empty[s]));
                    if (++s == NS) { s = 0; parity ^= 1u; }
                }
                tc_commit_pair(smem_u32(tmem_full));
                first = false;
                tile_parity ^= 1u;
            }
        } else if (!leader && lane == 0) {
            // CTA 1: when this CTA's activations have landed and its half of B is written, one
            // arrival tells the MMA issuer in CTA 0 (one message across the pair per stage).
            int s = 0;
            uint32_t parity = 0;
            for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
                for (int ks = 0; ks < nks; ks++) {
                    if (!mbar_wait(smem_u32(&a_full[s]), parity) || !mbar_wait(smem_u32(&b_full[s]), parity)) {
                        atomicOr(a.status, ST_TC_TIMEOUT);
                        goto done;
                    }
                    mbar_arrive_cluster(map_to_cta(smem_u32(&peer_ready[s]), 0));
                    if (++s == NS) { s = 0; parity ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------------------------------- decode, then epilogue ----
        const int dw = warp - kPairFirstDecodeWarp;
        const int g = lane >> 2, q = lane & 3;
        const int prev_word = (lane + 31) & 31;
        const uint32_t xc = a.cb_xor;
        LaneWords<K> lw;
        lw.init(lane);
        int s = 0, sw = 0;
        uint32_t parity = 0, w_parity = 0, tile_parity = 0;
        bool first_pass = true;
        for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
            const int m0 = (tile / a.tiles_n) * kPairTileM + 256 * (int)rank;
            const int n0 = (tile % a.tiles_n) * kTileN;
            for (int ks = 0; ks < nks; ks++) {
                // all lanes take the same decision: the tensor-memory loads below are warp-wide
                bool ok = mbar_wait(smem_u32(&w_full[sw]), w_parity);
                if (ok && !first_pass) ok = mbar_wait_cluster(smem_u32(&empty[s]), parity ^ 1u);
                if (!__all_sync(0xFFFFFFFFu, ok)) {
                    if (lane == 0) atomicOr(a.status, ST_TC_TIMEOUT);
                    goto done;
                }
                tc_fence_after_sync();
                uint8_t* bt = stage0 + (size_t)s * L::kStageBytes + 2 * kABytes;
                const uint32_t* wt = reinterpret_cast<const uint32_t*>(w_ring + (size_t)sw * L::kWBytes);
                uint32_t pw[4][3];
#pragma unroll
                for (int tk = 0; tk < 4; tk++) {
                    const uint32_t* tw = wt + (tk * 8 + dw) * L::kTileWords;
                    if (K == 4) {
                        pw[tk][0] = tw[lane];
                        pw[tk][1] = tw[prev_word];
                        pw[tk][2] = 0u;
                    } else {
                        pw[tk][0] = tw[lw.i0];
                        pw[tk][1] = tw[lw.i1];
                        pw[tk][2] = LaneWords<K>::kThree ? tw[lw.i2] : 0u;
                    }
                }
                // the packed words are in registers: their slot can be refilled while they are decoded
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&w_empty[sw]));
#pragma unroll
                for (int tk = 0; tk < 4; tk++) {
                    uint32_t cw[8];
                    if (K == 4) lane_codewords_k4(pw[tk][0], pw[tk][1], cw);
                    else lane_codewords<K>(pw[tk][0], pw[tk][1], pw[tk][2], lw.sh, cw);
                    // B[n][k] K-major, 128B swizzle: n = 16 dw + g (+8) of this CTA's 128 columns, k = 16 tk + 2q (+8)
                    uint8_t* row = bt + (2 * dw) * 1024 + g * 128 + 4 * q;
                    const int c0 = ((2 * tk) ^ g) << 4, c1 = ((2 * tk + 1) ^ g) << 4;
                    *reinterpret_cast<uint32_t*>(row + c0) = decode_pair_rt<CB>(cw[0], cw[1], xc);
                    *reinterpret_cast<uint32_t*>(row + 1024 + c0) = decode_pair_rt<CB>(cw[4], cw[5], xc);
                    *reinterpret_cast<uint32_t*>(row + c1) = decode_pair_rt<CB>(cw[2], cw[3], xc);
                    *reinterpret_cast<uint32_t*>(row + 1024 + c1) = decode_pair_rt<CB>(cw[6], cw[7], xc);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&b_full[s]));
                if (++sw == NW) { sw = 0; w_parity ^= 1u; }
                if (++s == NS) { s = 0; parity ^= 1u; first_pass = false; }
            }

            // ---- epilogue of this tile: this CTA's 256 tokens x 256 columns ----
            if (!__all_sync(0xFFFFFFFFu, mbar_wait_cluster(smem_u32(tmem_full), tile_parity))) {
                if (lane == 0) atomicOr(a.status, ST_TC_TIMEOUT);
                goto done;
            }
            tile_parity ^= 1u;
            tc_fence_after_sync();
            const int quarter = warp & 3, chalf = dw >> 2;
            const int col0 = n0 + 128 * chalf;
            if (col0 < a.t_out * 16) {
#pragma unroll 1
                for (int acc = 0; acc < 2; acc++) {
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
                    if (row < a.m) {
                        __half* yp = a.y + (int64_t)row * a.y_row_stride + col0;
#pragma unroll
                        for (int c = 0; c < 16; c++) {
                            float o[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) o[i] = v[8 * c + i] * EXL3_HAD_SCALE;
                            if (a.svh) {
                                const uint4 sv = *reinterpret_cast<const uint4*>(a.svh + col0 + 8 * c);
                                const uint32_t sw4[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const float2 f = __half22float2(u32_as_h2(sw4[i]));
                                    o[2 * i] *= f.x;
                                    o[2 * i + 1] *= f.y;
                                }
                            }
                            __half2 h[4];
#pragma unroll
                            for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
                            if (a.bias) {
                                const uint4 bv = *reinterpret_cast<const uint4*>(a.bias + col0 + 8 * c);
                                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                                for (int i = 0; i < 4; i++) h[i] = __hadd2(h[i], u32_as_h2(bw[i]));
                            }
                            uint4 ov;
                            ov.x = h2_as_u32(h[0]); ov.y = h2_as_u32(h[1]);
                            ov.z = h2_as_u32(h[2]); ov.w = h2_as_u32(h[3]);
                            *reinterpret_cast<uint4*>(yp + 8 * c) = ov;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(smem_u32(tmem_empty));
                else mbar_arrive_cluster(map_to_cta(smem_u32(tmem_empty), 0));
            }
        }
    }
done:
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();            // nothing of the pair is in flight any more
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---- host side ----------------------------------------------------------------------------------

extern int g_gemm_pairs;          // exl3_gemm.cu: 0, or 1 from the benchmark hook exl3_tune_gemm_pairs

// Dense layers with at least this many rows run on CTA pairs (a pair tile is 512 rows).
constexpr int kPairMinRows = 1024;

template <int K, int CB>
static int launch_gemm_pair_t(GemmArgs a, const __half* xh, const uint32_t* trellis, cudaStream_t s)
{
    using L = PairLayout<K>;
    static bool attr_set[kMaxDevices] = {};
    static int max_clusters[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return EXL3_E_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = L::kSmemBytes;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<K, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             L::kSmemBytes);
        if (e != cudaSuccess) return note_cuda(e);
        cfg.gridDim = dim3(2 * device_sm_count());
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<K, CB>, &cfg);
        if (e != cudaSuccess) return note_cuda(e);
        max_clusters[dev] = n;
        attr_set[dev] = true;
    }
    if (max_clusters[dev] < 1) return EXL3_E_UNSUPPORTED;
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
        const uint32_t box[3] = {(uint32_t)L::kTileWords, 8u, 4u};
        rc = make_tensor_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, trellis, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
    }
    a.tiles_m = (a.m + kPairTileM - 1) / kPairTileM;
    a.tiles_n = (a.t_out * 16 + kTileN - 1) / kTileN;
    a.cb_xor = 0x3B603B60u;
    const int clusters = std::min(a.tiles_m * a.tiles_n, max_clusters[dev]);
    cfg.gridDim = dim3(2 * clusters);
    return note_cuda(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<K, CB>, a, tm_x, tm_w));
}

// Dense layers with many rows run on CTA pairs; few rows and tile-table (grouped) launches on
// the one-CTA kernel.
template <int K, int CB>
static int launch_gemm_any_t(const GemmArgs& a, const __half* xh, const uint32_t* trellis, cudaStream_t s)
{
    if (!a.tile_tab && a.m >= kPairMinRows && g_gemm_pairs) return launch_gemm_pair_t<K, CB>(a, xh, trellis, s);
    return launch_gemm_t<K, CB>(a, xh, trellis, s);
}

template <int K>
int launch_gemm_k(const GemmArgs& a, int cb, const __half* xh, const uint32_t* trellis, cudaStream_t s)
{
    switch (cb) {
        case CB_3INST: return launch_gemm_any_t<K, CB_3INST>(a, xh, trellis, s);
        case CB_MCG: return launch_gemm_any_t<K, CB_MCG>(a, xh, trellis, s);
        case CB_MUL1: return launch_gemm_any_t<K, CB_MUL1>(a, xh, trellis, s);
        default: return EXL3_E_CODEBOOK;
    }
}

}  // namespace exl3
