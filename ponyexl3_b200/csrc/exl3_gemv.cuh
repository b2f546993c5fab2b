// Streamed EXL3 GEMV for 1..16 activation rows (decode and speculative verify).
//
// Decomposition.  The output is cut into 128-column blocks (the width of the output
// Hadamard rotation).  A thread-block CLUSTER of S CTAs computes one block at a time: CTA
// r of the cluster owns the k-slice [nkb*r/S, nkb*(r+1)/S) of the layer's 128-row k-blocks,
// so every CTA streams "items" of 8x8 packed tiles (one k-block of one column block,
// 2*K KiB) and keeps its slice of the rotated activations for its whole life.  S is chosen
// on the host so that (column blocks x S) fills the two CTA slots of every SM.  When a
// block is finished the other CTAs PUSH their fp32 partial sums into landing slots in the
// leader's shared memory (st.shared::cluster, then one remote mbarrier arrive) and, after
// their last block, leave at once; the leader adds the slots in rank order, rounds to fp16
// as the reference does, applies the output Hadamard-128, svh and bias, and stores the
// block.  Nothing goes through global memory and nobody reads a remote CTA's memory.
//
// Inside a CTA one producer lane feeds a shared-memory ring with TMA tensor copies
// (completion counted on mbarriers): ONE 3-D box per item.  Weight copies of the first
// ring fill are issued BEFORE the programmatic-launch wait, so under EXL3_FLAG_PDL a
// layer's weights stream while the previous kernel drains.
//
// Activations.  For few rows the input rotation is fused: after the dependency wait the
// consumer warps read x, multiply by suh, run the 128-point Hadamard butterfly with warp
// shuffles and park fp16 (x, 0) words of the CTA's k-slice in shared memory (kernel
// template XFUSED).  For more rows a small rotation kernel writes the words to the
// workspace and they ride the ring as a second, 128B-swizzled TMA box per item.
//
// Sixteen consumer warps in four groups; group q takes items q, q+4, ... of the CTA, and
// inside an item warp t of the group owns tile columns 2t, 2t+1 for all eight tile rows,
// so one activation fragment load serves two tiles and the per-item overhead (barrier
// wait, pointer set-up) is spread over sixteen tiles.  The decode is bound by the
// half-rate logic pipe of the SM (64 lanes/clk for LOP3 and PRMT; shifts run at a
// quarter), so the inner loop spends two logic operations per weight at K = 4 — one
// byte-permute to cut the codeword window, one LOP3 for the codebook mask — and pushes
// the rest to other pipes: shifts become wide integer multiplies and the two fp16 halves
// of a 3INST value are added by HADD2 with broadcast operands straight into a (w, w)
// register.  Each weight thus fills both k-slots of a 32-bit A-fragment register of
// mma.sync m16n8k16 and the activations are (x, 0) words: a second MMA per tile on the
// otherwise idle tensor pipe instead of byte-permutes on the saturated one.
// With EXL3_FLAG_FAST_ACCUM the HADD2 is skipped: the register keeps the two halves
// (lo, hi), the activations are (x, x), and the MMA adds lo*x + hi*x in fp32.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets a bit in the workspace
// status word and the kernel runs to its end without touching the data it missed.
#pragma once
#include <algorithm>

#include "exl3_internal.h"
#include "exl3_tma.h"

namespace exl3 {

constexpr int kGroups = 4;                          // consumer warp groups
constexpr int kConsumerWarps = 4 * kGroups;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kGemvThreads = kConsumerThreads + 32;
constexpr int kYStride = 132;
constexpr int kMaxStages = 16;
constexpr int kHeaderBytes = 512;
constexpr int kXsRowBytes = 544;                    // fused activations: 128 words + 8 of padding
constexpr int kMaxCluster = 16;

template <int K, int NMMA> struct GemvLayout {
    static constexpr int kTileWords = 8 * K;
    static constexpr int kWeightBytes = 64 * kTileWords * 4;             // 8x8 tiles: 2048 * K
    static constexpr int kYCopy = NMMA * 8 * kYStride;                   // floats per group copy
    static constexpr int kYBytes = kGroups * kYCopy * 4;
    static constexpr int kXBoxRows = 8 * NMMA;                           // rows of the TMA activation box
    static constexpr int kXBoxBytes = 4 * kXBoxRows * 128;
};

// ---- small cluster helpers ----------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctaid_x()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t dynamic_smem_bytes()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(r));
    return r;
}
#ifdef EXL3_PROFILE
__device__ __forceinline__ long long global_ns()
{
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#endif
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void fence_cluster()
{
    asm volatile("fence.acq_rel.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v)
{
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kWaitSpins; i++)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    return false;
}

// (w, w) from the two-halves word of 3INST / MCG, or from the MUL1 pattern.
template <int CB, bool FAST>
__device__ __forceinline__ uint32_t weight_slot_pair(uint32_t cw, uint32_t xor_const)
{
    const uint32_t r = codebook_word_rt<CB>(cw, xor_const);
    if (CB == CB_MUL1) {
        const __half2 h = u32_as_h2(r * 0x00010001u);
        return h2_as_u32(__hfma2(h, u32_as_h2(0x1EEE1EEEu), u32_as_h2(0xC931C931u)));
    }
    if (FAST) return r;
    const __half2 h = u32_as_h2(r);
    return h2_as_u32(__hadd2(__low2half2(h), __high2half2(h)));
}

template <typename T> __device__ __forceinline__ void load4_any(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4_any<__half>(const __half* p, float (&v)[4])
{
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(u32_as_h2(u.x)), b = __half22float2(u32_as_h2(u.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <> __device__ __forceinline__ void load4_any<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4])
{
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xFFFF0000u);
    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void load4_any<float>(const float* p, float (&v)[4])
{
    const float4 f = *reinterpret_cast<const float4*>(p);
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
}

template <int K, int CB, int NMMA, bool FAST, bool XFUSED>
__global__ void __launch_bounds__(kGemvThreads, 2)
    gemv_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_x)
{
    using L = GemvLayout<K, NMMA>;
    static_assert(!XFUSED || NMMA == 1, "fused activations are for few rows");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    uint64_t* red_full = empty + kMaxStages;      // leader: the other CTAs' partial sums have landed
    uint64_t* red_done = red_full + 1;            // non-leader: the leader has emptied the landing slots
    float* slots = reinterpret_cast<float*>(smem + a.slot_off);   // leader: (S-1) x rows x 128 floats
    float* ybuf = reinterpret_cast<float*>(smem + kHeaderBytes);
    uint8_t* xs = smem + kHeaderBytes + L::kYBytes;           // fused activations (XFUSED)
    uint8_t* stage0 = smem + a.stage0_off;

#ifdef EXL3_PROFILE
    const long long gt_entry = global_ns();
#endif
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = a.ksplit;
    const int rank = S > 1 ? (int)cluster_ctarank() : 0;
    const int cluster_id = blockIdx.x / S, n_clusters = gridDim.x / S;
    const int nkb = a.t_in >> 3;
    const int kb0 = nkb * rank / S, klen = nkb * (rank + 1) / S - kb0;
    const int n_cb = (a.ncb - cluster_id + n_clusters - 1) / n_clusters;   // blocks of this cluster
    const int nitems = n_cb * klen;
    const int ns = a.stages;
    const int xbox = XFUSED ? 0 : L::kXBoxBytes;
    const int stage_bytes = xbox + L::kWeightBytes;

    // The launch must match the plan the host made: every thread of every CTA takes the same
    // branch here, so a mismatch ends the grid before any barrier or remote access.
    if (dynamic_smem_bytes() < (uint32_t)(a.stage0_off + ns * stage_bytes) || ns < kGroups || ns > kMaxStages ||
        (S > 1 && cluster_nctaid_x() != (uint32_t)S) || (gridDim.x % (unsigned)S) != 0) {
        if (tid == 0) atomicOr(a.status, ST_BAD_LAUNCH);
        return;
    }

    if (tid < ns) {
        mbar_init(smem_u32(&full[tid]), 1);
        mbar_init(smem_u32(&empty[tid]), 4);
        if (tid == 0) {
            mbar_init(smem_u32(red_full), (uint32_t)(S > 1 ? S - 1 : 1));
            mbar_init(smem_u32(red_done), 1);
        }
        mbar_fence_init();
    }
    __syncthreads();
    // Every CTA's barriers must exist before a partner arrives on them, which happens only at
    // the end of a block: arrive here, wait just before the first remote access.
    if (S > 1) cluster_arrive();
    griddep_launch_dependents();

    // ------------------------------------------------------------------ producer ----
    if (warp == kConsumerWarps) {
        if (lane != 0) return;
        const uint32_t tx = L::kWeightBytes + (uint32_t)xbox;
        tma_prefetch_desc(&tm_w);
        if (!XFUSED) tma_prefetch_desc(&tm_x);
        // (block, k-block) of the next item, advanced without divisions: this lane shares a
        // scheduler with busy consumer warps, so its per-item instruction chain stays short.
        int w_cb = cluster_id, w_kb = 0, x_cb = cluster_id, x_kb = 0;
        auto issue_weights = [&](int s) {
            const int phys = a.blocks ? a.blocks[w_cb].phys : w_cb;
            tma_load_3d(smem_u32(stage0 + (size_t)s * stage_bytes + xbox), &tm_w, 0, 8 * phys,
                        8 * (kb0 + w_kb), smem_u32(&full[s]));
            if (++w_kb == klen) { w_kb = 0; w_cb += n_clusters; }
        };
        auto issue_x = [&](int s) {
            if (XFUSED) return;
            const int xrow = a.blocks ? a.blocks[x_cb].xrow : 0;
            tma_load_3d(smem_u32(stage0 + (size_t)s * stage_bytes), &tm_x, 0, xrow, 4 * (kb0 + x_kb),
                        smem_u32(&full[s]));
            if (++x_kb == klen) { x_kb = 0; x_cb += n_clusters; }
        };
        // A block table is written by an earlier kernel of the stream: read it only after
        // the dependency wait.  Plain layers prefetch their weights first.
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
        for (int li = pre; li < nitems; li++) {
            if (!mbar_wait(smem_u32(&empty[s]), parity)) {
                atomicOr(a.status, ST_WAIT_EMPTY_TIMEOUT);
                return;  // consumers run into their own bounded waits and finish
            }
            mbar_arrive_expect_tx(smem_u32(&full[s]), tx);
            issue_weights(s);
            issue_x(s);
            if (++s == ns) { s = 0; parity ^= 1u; }
        }
        return;
    }

    // ----------------------------------------------------------------- consumers ----
#ifdef EXL3_PROFILE
    long long pt_start = clock64(), pt_wait = 0, pt_comp = 0, pt_flush = 0;
    const long long gt_init = global_ns();
    long long gt_dep = 0;
#endif
    const int g = lane >> 2, tig = lane & 3;
    const int grp = warp >> 2, tnp = warp & 3;
    const int prev_word = (lane + 31) & 31;
    // A literal 16: handing it in as a run-time value (so that the nibble shift becomes a wide
    // multiply) was measured slower, twice — the multiplier pipe is as busy as the logic pipe.
    const uint32_t sixteen = 16u;
    const uint32_t xor_const = a.cb_xor;   // 0x3B603B60, kept opaque on purpose (see exl3_bits.cuh)
    LaneWords<K> lw;
    lw.init(lane);

    // ---- activations ----
    uint32_t xlane = 0;     // XFUSED: byte offset of this lane's row inside one k-block of xs
    uint32_t xkb_step = 0;  // XFUSED: bytes between k-blocks for this lane (0 on the zero line)
    int xo[4] = {0, 0, 0, 0};  // TMA box: swizzled chunk offsets of the (tile-row parity, half) cases
    if (XFUSED) {
        const int rows = a.rows;
        const int ntask = rows * klen;               // one (row, k-block) per warp and turn
        const int zero_off = klen * rows * kXsRowBytes;
        // Block-table launches (one block per cluster here): rotated row xrow0 + r of the table's
        // numbering is x[row_src[..]] with the sign vector suh[suh_row[..]]; the table belongs to an
        // earlier kernel of the stream, so nothing of it is read before the dependency wait.
        int xrow0 = 0;
        auto task_col = [&](int task) {
            const int r = task / klen;
            return (int64_t)(kb0 + task - r * klen) * 128 + lane * 4;
        };
        auto load_scale = [&](int task, float (&sc)[4]) {
            if (a.suh && task < ntask) {
                const int r = task / klen;
                const int64_t srow = a.suh_row ? a.suh_row[xrow0 + r] : 0;
                load4_any<__half>(a.suh + srow * ((int64_t)a.t_in * 16) + task_col(task), sc);
            } else {
                sc[0] = sc[1] = sc[2] = sc[3] = 1.f;
            }
        };
        auto load_x = [&](int task, float (&v)[4]) {
            if (task >= ntask) return;
            const int r0 = task / klen;
            const int64_t r = a.row_src ? a.row_src[xrow0 + r0] : xrow0 + r0;
            const int64_t off = r * a.x_row_stride + task_col(task);
            if (a.x_dtype == EXL3_DT_F16) load4_any<__half>(reinterpret_cast<const __half*>(a.x) + off, v);
            else if (a.x_dtype == EXL3_DT_BF16)
                load4_any<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(a.x) + off, v);
            else load4_any<float>(reinterpret_cast<const float*>(a.x) + off, v);
        };
        auto rotate_store = [&](int task, float (&v)[4], const float (&sc)[4]) {
            if (task >= ntask) return;
            const int r = task / klen, kbl = task - r * klen;
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = __half2float(__float2half_rn(v[q])) * sc[q];
            had128_warp(v, lane);
            const uint32_t dupm = FAST ? 0x00010001u : 1u;
            uint4 e;
            e.x = (uint32_t)__half_as_ushort(__float2half_rn(v[0] * EXL3_HAD_SCALE)) * dupm;
            e.y = (uint32_t)__half_as_ushort(__float2half_rn(v[1] * EXL3_HAD_SCALE)) * dupm;
            e.z = (uint32_t)__half_as_ushort(__float2half_rn(v[2] * EXL3_HAD_SCALE)) * dupm;
            e.w = (uint32_t)__half_as_ushort(__float2half_rn(v[3] * EXL3_HAD_SCALE)) * dupm;
            *reinterpret_cast<uint4*>(xs + (kbl * rows + r) * kXsRowBytes + lane * 16) = e;
        };
        // suh is a weight: the first two turns' scales are fetched while the previous kernel
        // of the stream may still be running; x belongs to it until the dependency wait.
        float sc0[4], sc1[4], v0[4] = {0.f, 0.f, 0.f, 0.f}, v1[4] = {0.f, 0.f, 0.f, 0.f};
        if (!a.blocks) {
            load_scale(warp, sc0);
            load_scale(warp + kConsumerWarps, sc1);
        }
        griddep_wait();
#ifdef EXL3_PROFILE
        gt_dep = global_ns();
#endif
        if (a.blocks) xrow0 = a.blocks[cluster_id < a.ncb ? cluster_id : 0].xrow;
        for (int task = warp; task < ntask; task += 2 * kConsumerWarps) {
            if (task != warp || a.blocks) {
                load_scale(task, sc0);
                load_scale(task + kConsumerWarps, sc1);
            }
            load_x(task, v0);                       // both loads in flight before either is used
            load_x(task + kConsumerWarps, v1);
            rotate_store(task, v0, sc0);
            rotate_store(task + kConsumerWarps, v1, sc1);
        }
        if (tid < kXsRowBytes / 4) reinterpret_cast<uint32_t*>(xs + zero_off)[tid] = 0u;
        // lanes whose batch row does not exist read the zero line
        xlane = (uint32_t)((g < rows ? g * kXsRowBytes : zero_off) + 8 * tig);
        xkb_step = g < rows ? (uint32_t)(rows * kXsRowBytes) : 0u;
        named_bar_sync(1, kConsumerThreads);
    } else {
        const int v = (tig >> 1) ^ g;
#pragma unroll
        for (int c = 0; c < 4; c++) xo[c] = (((2 * c) ^ v) << 4) + g * 128 + 8 * (tig & 1);
        griddep_wait();   // y belongs to earlier kernels of the stream until they end
#ifdef EXL3_PROFILE
        gt_dep = global_ns();
#endif
    }

    float acc[2][NMMA][4];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int m = 0; m < NMMA; m++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[t][m][q] = 0.f;
#ifdef EXL3_PROFILE
    long long pt_pro = clock64();
    const long long gt_loop = global_ns();
#endif

    bool failed = false;
    int li = grp;                         // this group's next item
    int s = grp;                          // its ring stage (ns >= kGroups)
    uint32_t parity = 0;
    uint32_t red_parity = 0;              // phase of red_full (leader) / red_done (others)

    for (int cbi = 0; cbi < n_cb; cbi++) {
        const int cb = cluster_id + cbi * n_clusters;
        const int li_end = (cbi + 1) * klen;
        for (; li < li_end; li += kGroups) {
#ifdef EXL3_PROFILE
            long long q0 = clock64();
#endif
            if (!failed && !mbar_wait(smem_u32(&full[s]), parity)) {
                failed = true;
                if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
            }
#ifdef EXL3_PROFILE
            long long q1 = clock64();
            pt_wait += q1 - q0;
#endif
            if (!failed) {
                const uint8_t* st = stage0 + (size_t)s * stage_bytes;
                const uint32_t* wst =
                    reinterpret_cast<const uint32_t*>(st + xbox) + 2 * tnp * L::kTileWords;
                const uint8_t* xk =
                    XFUSED ? xs + (uint32_t)(li - cbi * klen) * xkb_step + xlane : st;
#pragma unroll
                for (int tk = 0; tk < 8; tk++) {
                    uint2 xb[NMMA][2];
#pragma unroll
                    for (int m = 0; m < NMMA; m++)
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (XFUSED)
                                xb[m][h] = *reinterpret_cast<const uint2*>(xk + 64 * tk + 32 * h);
                            else
                                xb[m][h] = *reinterpret_cast<const uint2*>(
                                    xk + (tk >> 1) * (L::kXBoxRows * 128) + m * 1024 +
                                    xo[2 * (tk & 1) + h]);
                        }
#pragma unroll
                    for (int t = 0; t < 2; t++) {
                        const uint32_t* tw = wst + (tk * 8 + t) * L::kTileWords;
                        uint32_t cw[8];
                        if (K == 4) {
                            lane_codewords_k4(tw[lane], tw[prev_word], cw, sixteen);
                        } else {
                            const uint32_t wa = tw[lw.i0], wb = tw[lw.i1];
                            const uint32_t wc = LaneWords<K>::kThree ? tw[lw.i2] : 0u;
                            lane_codewords<K>(wa, wb, wc, lw.sh, cw);
                        }
                        uint32_t d[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) d[j] = weight_slot_pair<CB, FAST>(cw[j], xor_const);
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
            s += kGroups;
            if (s >= ns) { s -= ns; parity ^= 1u; }
#ifdef EXL3_PROFILE
            pt_comp += clock64() - q1;
#endif
        }
#ifdef EXL3_PROFILE
        long long f0 = clock64();
#endif

        // ---- block cb is done in this CTA: gather the partial sums ------------------------
        float* yg = ybuf + grp * L::kYCopy;
#pragma unroll
        for (int t = 0; t < 2; t++)
#pragma unroll
            for (int m = 0; m < NMMA; m++) {
                float* y0 = yg + (2 * tig + 8 * m) * kYStride + 16 * (2 * tnp + t) + g;
                y0[0] = acc[t][m][0];
                y0[kYStride] = acc[t][m][1];
                y0[8] = acc[t][m][2];
                y0[kYStride + 8] = acc[t][m][3];
#pragma unroll
                for (int q = 0; q < 4; q++) acc[t][m][q] = 0.f;
            }
        named_bar_sync(1, kConsumerThreads);
        if (S > 1 && cbi == 0) cluster_wait();   // all CTAs of the cluster have set up their barriers
        if (rank != 0) {
            // The landing slots still hold the previous block until the leader says otherwise.
            if (cbi > 0) {
                if (!failed && !mbar_wait_cluster(smem_u32(red_done), red_parity)) {
                    failed = true;
                    if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
                }
                red_parity ^= 1u;
            }
            // the groups' copies, added in a fixed order, go straight into this CTA's slot
            const uint32_t slot = map_to_cta(smem_u32(slots + (rank - 1) * a.rows * 128), 0);
            if (!failed)
                for (int i = tid; i < a.rows * 128; i += kConsumerThreads) {
                    const int o = (i >> 7) * kYStride + (i & 127);
                    float f = ybuf[o];
#pragma unroll
                    for (int c = 1; c < kGroups; c++) f += ybuf[o + c * L::kYCopy];
                    st_cluster_f32(slot + 4u * (uint32_t)i, f);
                }
            fence_cluster();                       // my stores, before the arrive below, cluster-wide
            named_bar_sync(1, kConsumerThreads);   // everybody's stores are issued; ybuf is free again
            if (tid == 0 && !failed) mbar_arrive_remote(map_to_cta(smem_u32(red_full), 0));
#ifdef EXL3_PROFILE
            pt_flush += clock64() - f0;
#endif
            continue;
        }
        for (int i = tid; i < a.rows * 128; i += kConsumerThreads) {
            const int o = (i >> 7) * kYStride + (i & 127);
            float f = ybuf[o];
#pragma unroll
            for (int c = 1; c < kGroups; c++) f += ybuf[o + c * L::kYCopy];
            ybuf[o] = f;
        }
        if (S > 1) {
            if (!failed && !mbar_wait_cluster(smem_u32(red_full), red_parity)) {
                failed = true;
                if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
            }
            red_parity ^= 1u;
        }
        named_bar_sync(1, kConsumerThreads);
        const int sv_off = a.blocks ? a.blocks[cb].sv_off : cb * 128;
        const int y_off = a.blocks ? a.blocks[cb].y_off : cb * 128;
        for (int n = warp; n < a.rows; n += kConsumerWarps) {
            float v[4];
            const int o = n * kYStride + 4 * lane;
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = ybuf[o + q];
            if (!failed)
                for (int r = 1; r < S; r++) {   // the other CTAs' sums, in rank order
                    const float4 p = *reinterpret_cast<const float4*>(slots + ((r - 1) * a.rows + n) * 128 + 4 * lane);
                    v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
                }
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = __half2float(__float2half_rn(v[q]));
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
            uint2 ov;
            ov.x = h2_as_u32(h0);
            ov.y = h2_as_u32(h1);
            if (a.n_peer == 0) {
                *reinterpret_cast<uint2*>(a.y + (int64_t)n * a.y_row_stride + y_off + 4 * lane) = ov;
            } else {
                // all-gather fused into the epilogue: the block lands in every rank's full row
                const int64_t off = (int64_t)n * a.y_row_stride + a.y_col0 + y_off + 4 * lane;
                for (int p = 0; p < a.n_peer; p++) *reinterpret_cast<uint2*>(a.y_peer[p] + off) = ov;
            }
        }
        if (a.n_peer > 0) {
            // System-scope fences are expensive and queue up behind one another, so only ONE thread of
            // the whole grid pays for them: every block is counted on a local counter (GPU scope),
            // and the CTA that finishes the last block of this rank announces the rank to all peers.
            named_bar_sync(1, kConsumerThreads);          // every row of the block has been sent
            if (tid == 0) {
                __threadfence();
                const unsigned done = atomicAdd(a.done_ctr, 1u) + 1u;
                if (done == (unsigned)a.ncb) {
                    atomicExch(a.done_ctr, 0u);           // re-armed for the next launch on this workspace
                    __threadfence_system();               // one fence orders all blocks before all arrivals
                    for (int p = 0; p < a.n_peer; p++)
                        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.ctr_peer[p]) : "memory");
                }
            }
        }
        if (cbi + 1 < n_cb) {
            // more blocks follow: tell the others that the landing slots are free again
            named_bar_sync(1, kConsumerThreads);   // all reads of ybuf and of the slots are done
            if (S > 1 && tid == 0)
                for (int r = 1; r < S; r++) mbar_arrive_remote(map_to_cta(smem_u32(red_done), (uint32_t)r));
        }
#ifdef EXL3_PROFILE
        pt_flush += clock64() - f0;
#endif
    }
#ifdef EXL3_PROFILE
    long long pt_main = clock64();
    const long long gt_main = global_ns();
#endif
    // The leader's shared memory is the target of the other CTAs' stores and arrives, so it
    // leaves last: every CTA arrives at the cluster barrier, only the leader waits on it —
    // also when a bounded wait above gave up.  (Threads that have exited count as arrived.)
    if (S > 1) {
        cluster_arrive();
        if (rank == 0) cluster_wait();
    }
#ifdef EXL3_PROFILE
    if (a.prof && lane == 0) {
        long long* p = a.prof + ((size_t)blockIdx.x * kConsumerWarps + warp) * 16;
        p[8] = gt_entry;               // wall clock (ns): kernel entry of this CTA
        p[9] = gt_init;                // barriers set up, cluster synchronised
        p[10] = gt_dep;                // previous kernel complete
        p[11] = gt_loop;               // activations ready, main loop starts
        p[12] = gt_main;               // main loop + gathers done
        p[13] = global_ns();           // end
        {
            uint32_t smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            p[14] = smid;
        }
        p[0] = pt_pro - pt_start;      // dependency wait + activation prologue
        p[1] = pt_wait;                // waiting for ring stages
        p[2] = pt_comp;                // decode + MMA
        p[3] = pt_flush;               // gather / epilogue
        p[4] = clock64() - pt_main;    // final wait for the leader
        p[5] = clock64() - pt_start;   // total
        p[6] = rank;
        p[7] = nitems;
    }
#endif
}

// ---- host side ----------------------------------------------------------------------------------

// tuning state and shape decisions live in exl3_gemv.cu
extern int g_gemv_ctas_per_sm;
extern int g_gemv_smem_budget;
void gemv_choose_split(int ncb, int nkb, int rows, int* ksplit, int* grid);

template <int K, int CB, int NMMA, bool FAST, bool XFUSED>
static int launch_gemv_t(GemvArgs a, bool pdl, cudaStream_t s)
{
    using L = GemvLayout<K, NMMA>;
    const int nkb = a.t_in >> 3;
    int ksplit, grid;
    gemv_choose_split(a.ncb, nkb, a.rows, &ksplit, &grid);
    a.ksplit = ksplit;
    a.cb_xor = 0x3B603B60u;
    a.sixteen = 16u;
    const int klen_max = (nkb + ksplit - 1) / ksplit;
    const int xs_bytes = XFUSED ? (klen_max * a.rows + 1) * kXsRowBytes : 0;
    const int slot_bytes = (ksplit - 1) * a.rows * 512;
    a.slot_off = kHeaderBytes + L::kYBytes + xs_bytes;
    const int stage0 = (a.slot_off + slot_bytes + 1023) / 1024 * 1024;
    const int stage_bytes = (XFUSED ? 0 : L::kXBoxBytes) + L::kWeightBytes;
    int budget = g_gemv_smem_budget;
    int stages = (budget - stage0) / stage_bytes;
    if (stages < kGroups) stages = (200 * 1024 - stage0) / stage_bytes;   // one CTA per SM
    stages = std::min(stages, kMaxStages);
    if (stages < kGroups) return EXL3_E_UNSUPPORTED;
    a.stages = stages;
    a.stage0_off = stage0;
    const size_t smem = (size_t)stage0 + (size_t)stages * stage_bytes;

    static bool attr_set[16] = {};  // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 16 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<K, CB, NMMA, FAST, XFUSED>,
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
        tm_x = tm_w;
        if (!XFUSED) {
            // xh viewed as (32 words, rows, in/32): one box brings the four quarters of a
            // k-block for 8 or 16 rows; rows past the end of xh read as zero
            const uint64_t in = (uint64_t)a.t_in * 16;
            const uint64_t xdims[3] = {32u, (uint64_t)a.x_rows_total, in / 32};
            const uint64_t xstrides[2] = {in * 4, 128u};
            const uint32_t xbox[3] = {32u, (uint32_t)L::kXBoxRows, 4u};
            rc = make_tensor_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.xh, xdims, xstrides,
                                 xbox, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (ksplit > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)ksplit;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return note_cuda(cudaLaunchKernelEx(&cfg, gemv_kernel<K, CB, NMMA, FAST, XFUSED>, a, tm_w, tm_x));
}

// Co-resident clusters of `cluster` CTAs the device can hold for this kernel family
// (same block size and register count for every instantiation).
template <int K> int gemv_query_active_clusters(int cluster, int smem_bytes)
{
    auto kern = gemv_kernel<K, CB_3INST, 1, false, true>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(cluster * 64));
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

template <int K, int CB> static int launch_gemv_kc(const GemvArgs& a, bool pdl, cudaStream_t s)
{
    constexpr bool kCanFast = (CB != CB_MUL1);   // MUL1 has no two-halves form
    const bool fast = a.fast_accum && kCanFast;
    if (a.x_fused) {
        return fast ? launch_gemv_t<K, CB, 1, kCanFast, true>(a, pdl, s)
                    : launch_gemv_t<K, CB, 1, false, true>(a, pdl, s);
    }
    if (a.rows > 8)
        return fast ? launch_gemv_t<K, CB, 2, kCanFast, false>(a, pdl, s)
                    : launch_gemv_t<K, CB, 2, false, false>(a, pdl, s);
    return fast ? launch_gemv_t<K, CB, 1, kCanFast, false>(a, pdl, s)
                : launch_gemv_t<K, CB, 1, false, false>(a, pdl, s);
}

template <int K> int launch_gemv_k(const GemvArgs& a, int cb, bool pdl, cudaStream_t s)
{
    switch (cb) {
        case CB_3INST: return launch_gemv_kc<K, CB_3INST>(a, pdl, s);
        case CB_MCG: return launch_gemv_kc<K, CB_MCG>(a, pdl, s);
        case CB_MUL1: return launch_gemv_kc<K, CB_MUL1>(a, pdl, s);
        default: return EXL3_E_CODEBOOK;
    }
}

}  // namespace exl3
