// Streamed EXL3 GEMV for 1..16 activation rows (decode and speculative verify).
//
// Decomposition.  The output is cut into 128-column blocks (the width of the output
// Hadamard rotation) and the input into 128-row k-blocks (the width of the input one); an
// ITEM is one k-block of one column block: 8x8 packed tiles, 2*K KiB.  The items of a layer,
// numbered column block by column block, are dealt out EVENLY to 2 x SMs "virtual CTAs",
// however many column blocks the layer has: virtual CTA c streams the contiguous item range
// [I*c/G, I*(c+1)/G).  A range is a sequence of SEGMENTS, each the part of one column block
// that falls inside it.  A segment that covers its whole block is finished by its virtual CTA
// alone.  A block that straddles virtual CTAs is finished by whichever of them ends its segment
// last: every contributor writes its fp32 partial sums to its own slot of the workspace and
// counts itself on the block's counter; the one that completes the count adds the slots in
// order (so the result does not depend on who came last), rounds to fp16 as the reference
// does, applies the output Hadamard-128, svh and bias, and stores the block.
//
// One real CTA of 1024 threads per SM carries TWO virtual CTAs, its halves of 16 warps: each
// half has its own range, ring, barriers and partial sums and never synchronises with the
// other.  While one half is in a latency-bound phase (rotating its activations, handing over a
// segment's sums) the other keeps the SM's issue slots busy; two separate 16-warp CTAs per SM
// would do that too, but the hardware favours the older CTA, which then runs ahead and leaves
// the SM half empty for the last third of the launch.
//
// Inside a half a shared-memory ring is fed by TMA tensor copies (completion counted on
// mbarriers): ONE 3-D box per item.  Sixteen warps in four groups; group q takes items q,
// q+4, ... of the range, and inside an item warp t of the group owns tile columns 2t, 2t+1
// for all eight tile rows, so one activation fragment load serves two tiles and the per-item
// overhead (barrier wait, pointer set-up) is spread over sixteen tiles.  There is no producer
// warp and nobody waits for a free stage: the warp that is last to finish with a stage refills
// it on the spot.  Weight copies of the first ring fill are issued BEFORE the
// programmatic-launch wait, so under EXL3_FLAG_PDL a layer's weights stream while the previous
// kernel drains.
// (Measured alternatives, all slower: one undivided 32-warp CTA — every flush and the input
// rotation stall the whole SM; an issuer lane per group that waits for its group every turn,
// or that refills a turn late; the last items of a segment shared by all groups, a few tile
// rows each; per-warp
// cp.async rings without any shared ring or barrier — the loop is bound by instruction issue,
// and the per-row copy bookkeeping costs more than the ring's per-item bookkeeping.)
//
// Activations.  For few rows the input rotation is fused: after the dependency wait the
// warps read x, multiply by suh, run the 128-point Hadamard butterfly with warp shuffles and
// park fp16 (x, 0) words of the k-blocks of the CTA's range in shared memory (kernel template
// XFUSED).  For more rows a small rotation kernel writes the words to the workspace and they
// ride the ring as a second, 128B-swizzled TMA box per item.
//
// The decode is bound by the half-rate logic pipe of the SM (64 lanes/clk for LOP3 and PRMT;
// shifts run at a quarter), so the inner loop spends two logic operations per weight at
// K = 4 — one byte-permute to cut the codeword window (the two 16-bit aligned windows of a
// word come from 16-bit shared-memory loads instead), one LOP3 for the codebook mask — and
// pushes the rest to other pipes: shifts become wide integer multiplies and the two fp16
// halves of a 3INST value are added by HADD2 with broadcast operands straight into a (w, w)
// register.  Each weight thus fills both k-slots of a 32-bit A-fragment register of mma.sync
// m16n8k16 and the activations are (x, 0) words: a second MMA per tile on the otherwise idle
// tensor pipe instead of byte-permutes on the saturated one.  With EXL3_FLAG_FAST_ACCUM the
// HADD2 is skipped: the register keeps the two halves (lo, hi), the activations are (x, x),
// and the MMA adds lo*x + hi*x in fp32.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets a bit in the workspace
// status word and the kernel runs to its end without touching the data it missed.  No CTA
// waits for another one.
#pragma once
#include <algorithm>

#include "exl3_internal.h"
#include "exl3_tma.h"

namespace exl3 {

constexpr int kGroups = 4;                          // warp groups of four warps per half
constexpr int kHalfWarps = 4 * kGroups;
constexpr int kHalfThreads = kHalfWarps * 32;
constexpr int kGemvThreads = 2 * kHalfThreads;      // one CTA of 1024 threads per SM: two halves
constexpr int kYStride = 132;
constexpr int kMaxStages = 16;                      // per half
constexpr int kHeaderBytes = 512;                   // per half: 16 mbarriers, counters, hand-off words, table cache
constexpr int kDoneCntOff = 128;
constexpr int kIssuedOff = 192;
constexpr int kHandoffOff = 256;
constexpr int kIssuerOff = 288;                     // 4 groups x 4 ints
constexpr int kXsRowBytes = 544;                    // fused activations: 128 words + 8 of padding
constexpr int kGemvSmemBytes = 226 * 1024;          // dynamic shared memory of the one CTA per SM

template <int K, int NMMA> struct GemvLayout {
    static constexpr int kTileWords = 8 * K;
    static constexpr int kYCopy = NMMA * 8 * kYStride;                   // floats per group copy
    static constexpr int kCopies = NMMA == 1 ? 4 : 2;                    // copies of the partial sums per half
    static constexpr int kYBytes = kCopies * kYCopy * 4;
    static constexpr int kWeightBytes = 64 * kTileWords * 4;             // 8x8 tiles: 2048 * K
    static constexpr int kXBoxRows = 8 * NMMA;                           // rows of the TMA activation box
    static constexpr int kXBoxBytes = 4 * kXBoxRows * 128;
};

__device__ __forceinline__ uint32_t dynamic_smem_bytes()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(r));
    return r;
}

#ifdef EXL3_PROFILE
// Timeline builds (python -m ponyexl3_b200.build --profile): wall-clock stamps per CTA.
__device__ __forceinline__ long long global_ns()
{
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define EXL3_STAMP(var) const long long var = global_ns()
#else
#define EXL3_STAMP(var)
#endif

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

// Compile-time loop: f(integral_constant<int, 0>) ... f(integral_constant<int, N-1>).  The tile
// loops of the GEMV are written with it because `#pragma unroll` left them rolled (a branch, a
// compare and two address computations per tile on the pipe that bounds the kernel).
template <int V> struct IntC { static constexpr int value = V; };
template <int N, int I0 = 0, typename F> __device__ __forceinline__ void static_for(F&& f)
{
    if constexpr (I0 < N) {
        f(IntC<I0>{});
        static_for<N, I0 + 1>(f);
    }
}

// CTA that streams item i when I items are dealt to G CTAs as [I*c/G, I*(c+1)/G).
__device__ __forceinline__ int cta_of_item(int64_t i, int64_t I, int G)
{
    return (int)(((i + 1) * G - 1) / I);
}

// atomicInc with release + acquire semantics at GPU scope: one instruction where a fence, the
// count and a second fence would each cost a round trip.
__device__ __forceinline__ unsigned atom_inc_acq_rel(unsigned* p, unsigned bound)
{
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.inc.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(bound) : "memory");
    return old;
}

template <int K, int CB, int NMMA, bool FAST, bool XFUSED>
__global__ void __launch_bounds__(kGemvThreads, 1)
    gemv_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap tm_w,
                const __grid_constant__ CUtensorMap tm_x)
{
    using L = GemvLayout<K, NMMA>;
    static_assert(!XFUSED || NMMA == 1, "fused activations are for few rows");
    extern __shared__ __align__(1024) uint8_t smem[];

    EXL3_STAMP(gt_entry);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // The CTA is two independent halves of 16 warps; each is one "virtual CTA" of the partition.
    const int half = warp >> 4, wl = warp & 15, tidh = tid & (kHalfThreads - 1);
    const int hbar = 1 + half;                         // the half's named barrier
    const int c = 2 * (int)blockIdx.x + half;
    const int nkb = a.t_in >> 3;
    // The number of column blocks may be a count that an earlier kernel of the stream has left on
    // the device (a table of which only the first entries are in use): every thread reads the same
    // word, so the partition below is the same in every CTA.  The plan was made for a.ncb blocks.
    int ncb = a.ncb;
    if (a.ncb_dev) {
        griddep_wait();
        const int v = *a.ncb_dev;
        ncb = v < 0 ? 0 : (v < a.ncb ? v : a.ncb);
    }
    const int64_t I = (int64_t)ncb * nkb;
    // Every virtual CTA of the partition holds at least one item (the hand-over of a split block
    // counts on it: all CTAs between a block's first and last contribute), so a count that leaves
    // fewer items than planned CTAs uses fewer of them.
    const int G = (int)(I < (int64_t)a.grid_virtual ? (I > 0 ? I : 1) : (int64_t)a.grid_virtual);
    const int64_t i0 = c < G ? I * c / G : 0;
    const int nitems = c < G ? (int)(I * (c + 1) / G - i0) : 0;
    const int cb0 = (int)(i0 / nkb), kb0 = (int)(i0 - (int64_t)cb0 * nkb);
    const int ns = a.stages;                           // per half
    const int xbox = XFUSED ? 0 : L::kXBoxBytes;
    const int stage_bytes = xbox + L::kWeightBytes;
    // fused activations: one slot per k-block of the range; a plain layer multiplies every
    // column block by the same rows, so its slots wrap after a full turn over the k-blocks
    const bool xs_wrap = !a.blocks && nitems > nkb;
    const int n_slots = xs_wrap ? nkb : nitems;

    // The launch must match the plan the host made: every thread of every CTA takes the same
    // branch here, so a mismatch ends the grid before any barrier is touched.
    if (dynamic_smem_bytes() < (uint32_t)(a.stage0_off + 2 * ns * stage_bytes) || ns < kGroups || ns > kMaxStages ||
        (int)gridDim.x * 2 < G || G < 1 ||
        (XFUSED && (a.blocks ? (I + G - 1) / G : min((I + G - 1) / G, (int64_t)nkb)) > a.n_slots)) {
        if (tid == 0) atomicOr(a.status, ST_BAD_LAUNCH);
        return;
    }

    uint8_t* hdr = smem + half * kHeaderBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(hdr);
    int* done_cnt = reinterpret_cast<int*>(hdr + kDoneCntOff);       // warps that have finished with each stage
    volatile int* issued = reinterpret_cast<volatile int*>(hdr + kIssuedOff);   // item each stage was last filled with
    volatile int* handoff = reinterpret_cast<volatile int*>(hdr + kHandoffOff);
    float* ybuf = reinterpret_cast<float*>(smem + 2 * kHeaderBytes + half * L::kYBytes);
    uint8_t* xs = smem + 2 * kHeaderBytes + 2 * L::kYBytes + half * a.xs_bytes;   // fused activations (XFUSED)
    uint8_t* stage0 = smem + a.stage0_off + half * ns * stage_bytes;

    if (tidh < ns) {
        mbar_init(smem_u32(&full[tidh]), 1);
        done_cnt[tidh] = 0;
        issued[tidh] = -1;
        mbar_fence_init();
    }
    __syncthreads();
    griddep_launch_dependents();
    if (nitems == 0) return;                           // an odd number of virtual CTAs: the last half idles

    const int g = lane >> 2, tig = lane & 3;
    const int grp = wl >> 2, tnp = wl & 3;

    // ---- the ring: item p of the range lives in stage p % ns ----------------------------------
    // There is no producer warp and nobody waits for a free stage.  The first ring fill is
    // issued at once, one lane per warp group taking its share.  After that every warp counts
    // itself on the stage it has finished with (a shared-memory atomic), and the warp that
    // completes the count — the last of the item's four — refills the stage on the spot with
    // the item ns places further on.  `issued[stage]` names the item a stage was last filled
    // with: a warp looks at a stage's barrier only once its item has been issued there, so a
    // parity test can never be taken for a phase that has not begun.
    const uint32_t tx = L::kWeightBytes + (uint32_t)xbox;
    // per group: [0] block seen last, [1] its physical block, [2] its first activation row
    volatile int* iq = reinterpret_cast<volatile int*>(hdr + kIssuerOff) + 4 * grp;
    auto issue_item = [&](int p, int st, bool weights, bool acts) {
        const int kq = kb0 + p;
        const int d = kq / nkb;
        const int cb = cb0 + d, kb = kq - d * nkb;
        if (st < 0 || st >= ns || p < 0 || p >= nitems || cb >= ncb) {   // never true for a launch as planned
            atomicOr(a.status, ST_BAD_LAUNCH);
            return;
        }
        int phys = cb, xrow = 0;
        if (a.blocks) {
            // the table entry of the block seen last is kept (a race between the group's warps
            // only writes the same values twice)
            if (cb != iq[0]) {
                iq[1] = a.blocks[cb].phys;
                iq[2] = a.blocks[cb].xrow;
                __threadfence_block();
                iq[0] = cb;
            }
            phys = iq[1];
            xrow = iq[2];
            if (iq[0] != cb) { phys = a.blocks[cb].phys; xrow = a.blocks[cb].xrow; }
        }
        if (weights) {
            mbar_arrive_expect_tx(smem_u32(&full[st]), tx);
            tma_load_3d(smem_u32(stage0 + (size_t)st * stage_bytes + xbox), &tm_w, 0, 8 * phys, 8 * kb,
                        smem_u32(&full[st]));
            issued[st] = p;
        }
        if (!XFUSED && acts)
            tma_load_3d(smem_u32(stage0 + (size_t)st * stage_bytes), &tm_x, 0, xrow, 4 * kb,
                        smem_u32(&full[st]));
    };
    // This warp is done with stage st, which held item p.
    auto release_stage = [&](int p, int st) {
        __syncwarp();
        if (lane == 0 && atomicAdd(&done_cnt[st], 1) == 3) {
            done_cnt[st] = 0;
            if (p + ns < nitems) issue_item(p + ns, st, true, true);
        }
    };
    if (tnp == 0 && lane == 0) {
        const int pre = nitems < ns ? nitems : ns;   // first ring fill: item p goes to stage p
        iq[0] = -1;
        tma_prefetch_desc(&tm_w);
        if (!XFUSED) tma_prefetch_desc(&tm_x);
        // A block table is written by an earlier kernel of the stream: read it only after the
        // dependency wait.  Plain layers prefetch their weights first; the rotated activations
        // (when they ride the ring) belong to the previous kernel until the wait.
        if (a.blocks) griddep_wait();
        for (int p = grp; p < pre; p += kGroups) issue_item(p, p, true, false);
        if (!XFUSED) {
            if (!a.blocks) griddep_wait();
            for (int p = grp; p < pre; p += kGroups) issue_item(p, p, false, true);
        }
    }

    EXL3_STAMP(gt_init);
#ifdef EXL3_PROFILE
    long long gt_dep = 0, gt_last_item = 0, ck_wait = 0, ck_loop = 0;
#endif
    const int prev_word = (lane + 31) & 31;
    // A literal 16 (the nibble shift becomes two shift-adds on the logic pipe): handing it in as a
    // run-time value, so that it becomes one wide multiply, was measured slower three times.
    const uint32_t sixteen = 16u;
    const uint32_t xor_const = a.cb_xor;   // 0x3B603B60, kept opaque on purpose (see exl3_bits.cuh)
    LaneWords<K> lw;
    lw.init(lane);

    // ---- activations ----
    uint32_t xlane = 0;     // XFUSED: byte offset of this lane's row inside one slot of xs
    uint32_t xkb_step = 0;  // XFUSED: bytes between slots for this lane (0 on the zero line)
    int xo[4] = {0, 0, 0, 0};  // TMA box: swizzled chunk offsets of the (tile-row parity, half) cases
    if (XFUSED) {
        const int rows = a.rows;
        const int ntask = rows * n_slots;            // one (row, slot) per warp and turn
        const int zero_off = n_slots * rows * kXsRowBytes;
        // Task -> (row r, slot sl); slot sl holds the k-block of range item sl.  With a block
        // table, row r of the item's block is x[row_src[xrow + r]] with the sign vector
        // suh[suh_row[xrow + r]]; the table belongs to an earlier kernel of the stream, so
        // nothing of it is read before the dependency wait.
        struct Task { int64_t xoff, soff; int dst; };
        auto make_task = [&](int task, Task& t) {
            if (task >= ntask) { t.dst = -1; return; }
            const int r = task / n_slots, sl = task - r * n_slots;
            const int kq = kb0 + sl;
            const int dcb = kq / nkb;
            const int kb = kq - dcb * nkb;
            int64_t xr = r, sr = 0;
            if (a.blocks) {
                const int xrow = a.blocks[cb0 + dcb].xrow + r;
                xr = a.row_src ? a.row_src[xrow] : xrow;
                sr = a.suh_row ? a.suh_row[xrow] : 0;
            }
            const int64_t col = (int64_t)kb * 128 + lane * 4;
            t.xoff = xr * a.x_row_stride + col;
            t.soff = sr * ((int64_t)a.t_in * 16) + col;
            t.dst = (sl * rows + r) * kXsRowBytes + lane * 16;
        };
        auto load_scale = [&](const Task& t, float (&sc)[4]) {
            if (a.suh && t.dst >= 0) load4_any<__half>(a.suh + t.soff, sc);
            else sc[0] = sc[1] = sc[2] = sc[3] = 1.f;
        };
        auto load_at = [&](int64_t off, float (&v)[4]) {
            if (a.x_dtype == EXL3_DT_F16) load4_any<__half>(reinterpret_cast<const __half*>(a.x) + off, v);
            else if (a.x_dtype == EXL3_DT_BF16)
                load4_any<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(a.x) + off, v);
            else load4_any<float>(reinterpret_cast<const float*>(a.x) + off, v);
        };
        auto load_x = [&](const Task& t, float (&v)[4]) {
            if (t.dst < 0) return;
            load_at(t.xoff, v);
            if (a.x_glu) {
                // the row holds [gate (in) | up (in)]: the input is fp16(act(gate) * up), the
                // rounding being the one rotate_store applies to every input
                float up[4];
                load_at(t.xoff + (int64_t)a.t_in * 16, up);
#pragma unroll
                for (int q = 0; q < 4; q++) v[q] = glu_value(v[q], up[q], a.x_glu);
            }
        };
        auto rotate_store = [&](const Task& t, float (&v)[4], const float (&sc)[4]) {
            if (t.dst < 0) return;
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = __half2float(__float2half_rn(v[q])) * sc[q];
            had128_warp(v, lane);
            const uint32_t dupm = FAST ? 0x00010001u : 1u;
            uint4 e;
            e.x = (uint32_t)__half_as_ushort(__float2half_rn(v[0] * EXL3_HAD_SCALE)) * dupm;
            e.y = (uint32_t)__half_as_ushort(__float2half_rn(v[1] * EXL3_HAD_SCALE)) * dupm;
            e.z = (uint32_t)__half_as_ushort(__float2half_rn(v[2] * EXL3_HAD_SCALE)) * dupm;
            e.w = (uint32_t)__half_as_ushort(__float2half_rn(v[3] * EXL3_HAD_SCALE)) * dupm;
            *reinterpret_cast<uint4*>(xs + t.dst) = e;
        };
        // suh is a weight: the first two turns' scales are fetched while the previous kernel
        // of the stream may still be running; x belongs to it until the dependency wait.
        Task t0, t1;
        float sc0[4], sc1[4], v0[4] = {0.f, 0.f, 0.f, 0.f}, v1[4] = {0.f, 0.f, 0.f, 0.f};
        if (!a.blocks) {
            make_task(wl, t0);
            make_task(wl + kHalfWarps, t1);
            load_scale(t0, sc0);
            load_scale(t1, sc1);
        }
        griddep_wait();
#ifdef EXL3_PROFILE
        gt_dep = global_ns();
#endif
        // x may be a row that the other GPUs are still completing over peer memory: wait (bounded)
        // until the expected number of ranks have announced their blocks on this rank's counter.
        // The virtual CTA that is last to get past re-arms the counter by taking the arrivals off
        // again, so an arrival that belongs to a later exchange is kept.
        if (a.wait_ctr) {
            if (tidh == 0) {
                bool ok = false;
                for (unsigned i = 0; i < kPeerPolls && !ok; i++) {
                    unsigned v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.wait_ctr) : "memory");
                    ok = v >= a.wait_target;
                    if (!ok) __nanosleep(200);
                }
                if (!ok) atomicOr(a.status, ST_PEER_TIMEOUT);
                const unsigned passed = atomicInc(a.pass_ctr, (unsigned)(G - 1));
                if (ok && passed == (unsigned)(G - 1))
                    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(a.wait_ctr), "r"(0u - a.wait_target)
                                 : "memory");
            }
            named_bar_sync(hbar, kHalfThreads);
        }
        for (int task = wl; task < ntask; task += 2 * kHalfWarps) {
            if (task != wl || a.blocks) {
                make_task(task, t0);
                make_task(task + kHalfWarps, t1);
                load_scale(t0, sc0);
                load_scale(t1, sc1);
            }
            load_x(t0, v0);                         // both loads in flight before either is used
            load_x(t1, v1);
            rotate_store(t0, v0, sc0);
            rotate_store(t1, v1, sc1);
        }
        if (tidh < kXsRowBytes / 4) reinterpret_cast<uint32_t*>(xs + zero_off)[tidh] = 0u;
        // lanes whose batch row does not exist read the zero line
        xlane = (uint32_t)((g < rows ? g * kXsRowBytes : zero_off) + 8 * tig);
        xkb_step = g < rows ? (uint32_t)(rows * kXsRowBytes) : 0u;
        named_bar_sync(hbar, kHalfThreads);
    } else {
        const int v = (tig >> 1) ^ g;
#pragma unroll
        for (int cc = 0; cc < 4; cc++) xo[cc] = (((2 * cc) ^ v) << 4) + g * 128 + 8 * (tig & 1);
        griddep_wait();   // y belongs to earlier kernels of the stream until they end
#ifdef EXL3_PROFILE
        gt_dep = global_ns();
#endif
    }
    EXL3_STAMP(gt_loop);

    float acc[2][NMMA][4];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int m = 0; m < NMMA; m++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[t][m][q] = 0.f;

    // Both tiles (columns 2*tnp, 2*tnp + 1 of the item) of tile row TK: decode, multiply.
    auto tile_row = [&](const uint8_t* xk, const uint32_t* wst, auto tkc) {
        constexpr int tk = decltype(tkc)::value;
        uint2 xb[NMMA][2];
#pragma unroll
        for (int m = 0; m < NMMA; m++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (XFUSED)
                    xb[m][h] = *reinterpret_cast<const uint2*>(xk + 64 * tk + 32 * h);
                else
                    xb[m][h] = *reinterpret_cast<const uint2*>(xk + (tk >> 1) * (L::kXBoxRows * 128) + m * 1024 +
                                                               xo[2 * (tk & 1) + h]);
            }
        static_for<2>([&](auto tc) {
            constexpr int t = decltype(tc)::value;
            const uint32_t* tw = wst + (tk * 8 + t) * L::kTileWords;
            uint32_t cw[8];
            if (K == 4) {
                // the two 16-bit aligned windows come straight from shared memory
                const uint16_t* th = reinterpret_cast<const uint16_t*>(tw) + 2 * lane;
                lane_codewords_k4_halves(tw[lane], tw[prev_word], th[0], th[1], cw, sixteen);
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
        });
    };

    // Ring position of the item this thread looks at next; items are visited in rising order.
    int cur_p = 0, s = 0, slot = 0;
    uint32_t parity = 0;
    auto seek = [&](int p) {
        const int d = p - cur_p;
        cur_p = p;
        s += d;
        while (s >= ns) { s -= ns; parity ^= 1u; }
        if (XFUSED) {
            if (xs_wrap) {
                slot += d;
                while (slot >= n_slots) slot -= n_slots;
            } else {
                slot = p;
            }
        }
    };
    bool failed = false;
    auto wait_item = [&]() {
        if (failed) return;
        // the item must have been issued into the stage before its barrier means anything
        uint32_t spins = 0;
        while (issued[s] != cur_p && ++spins < kWaitSpins) {}
        if (spins >= kWaitSpins || !mbar_wait(smem_u32(&full[s]), parity)) {
            failed = true;
            if (lane == 0) atomicOr(a.status, ST_WAIT_FULL_TIMEOUT);
        }
    };
    const int nv = a.rows * 128;

    int seg0 = 0;                         // first item of the current segment
    int li = grp;                         // this group's next item of the range
    for (int cbl = cb0; seg0 < nitems; cbl++) {
        const int seg_len = min(nitems - seg0, seg0 == 0 ? nkb - kb0 : nkb);
        const int seg_end = seg0 + seg_len;
        for (; li < seg_end; li += kGroups) {
#ifdef EXL3_PROFILE
            const long long q0 = clock64();
#endif
            seek(li);
            wait_item();
#ifdef EXL3_PROFILE
            const long long q1 = clock64();
            ck_wait += q1 - q0;
#endif
            if (!failed) {
                const uint8_t* st = stage0 + (size_t)s * stage_bytes;
                const uint8_t* xk = XFUSED ? xs + (uint32_t)slot * xkb_step + xlane : st;
                const uint32_t* wst = reinterpret_cast<const uint32_t*>(st + xbox) + 2 * tnp * L::kTileWords;
                static_for<8>([&](auto tkc) { tile_row(xk, wst, tkc); });
            }
            release_stage(cur_p, s);
#ifdef EXL3_PROFILE
            ck_loop += clock64() - q1;
#endif
        }

#ifdef EXL3_PROFILE
        gt_last_item = global_ns();
#endif
        // ---- the segment is done in this half: gather the groups' sums ------------------------
        // one copy per group; with two MMA row groups two copies, filled in two rounds
        float* yg = ybuf + (grp % L::kCopies) * L::kYCopy;
#pragma unroll
        for (int round = 0; round < kGroups / L::kCopies; round++) {
            if (grp / L::kCopies == round) {
#pragma unroll
                for (int t = 0; t < 2; t++)
#pragma unroll
                    for (int m = 0; m < NMMA; m++) {
                        float* y0 = yg + (2 * tig + 8 * m) * kYStride + 16 * (2 * tnp + t) + g;
                        if (round == 0) {
                            y0[0] = acc[t][m][0];
                            y0[kYStride] = acc[t][m][1];
                            y0[8] = acc[t][m][2];
                            y0[kYStride + 8] = acc[t][m][3];
                        } else {
                            y0[0] += acc[t][m][0];
                            y0[kYStride] += acc[t][m][1];
                            y0[8] += acc[t][m][2];
                            y0[kYStride + 8] += acc[t][m][3];
                        }
#pragma unroll
                        for (int q = 0; q < 4; q++) acc[t][m][q] = 0.f;
                    }
            }
            named_bar_sync(hbar, kHalfThreads);
        }

        // A segment shorter than the block's k-range is one of several contributions: it goes to
        // this virtual CTA's slot of the workspace (first segment of the range: slot 0, else slot 1)
        // and the contributor that completes the count finishes the block.
        bool finish = true;
        int c_first = 0, n_contrib = 0, slot_first = 0;
        if (seg_len == nkb) {
            for (int i = tidh; i < nv; i += kHalfThreads) {
                const int o = (i >> 7) * kYStride + (i & 127);
                float f = ybuf[o];
#pragma unroll
                for (int cc = 1; cc < L::kCopies; cc++) f += ybuf[o + cc * L::kYCopy];
                ybuf[o] = f;
            }
            named_bar_sync(hbar, kHalfThreads);
        } else {
            if ((size_t)(2 * c + 2) * nv * sizeof(float) > a.partial_bytes) {   // never true for a launch as planned
                if (tidh == 0) atomicOr(a.status, ST_BAD_LAUNCH);
                return;
            }
            float* part = a.partials + (size_t)(2 * c + (seg0 == 0 ? 0 : 1)) * nv;
            for (int i = tidh; i < nv; i += kHalfThreads) {
                const int o = (i >> 7) * kYStride + (i & 127);
                float f = ybuf[o];
#pragma unroll
                for (int cc = 1; cc < L::kCopies; cc++) f += ybuf[o + cc * L::kYCopy];
                __stcg(part + i, f);
            }
            named_bar_sync(hbar, kHalfThreads);
            if (tidh == 0) {
                // The barrier orders the half's stores before this release; the count wraps to 0
                // with the last arrival (re-armed for the next launch) and, being an acquire too,
                // orders the other contributors' stores before the reads below.
                const int64_t first_item = (int64_t)cbl * nkb;
                const int cf = cta_of_item(first_item, I, G);
                const int cl = cta_of_item(first_item + nkb - 1, I, G);
                const unsigned old = atom_inc_acq_rel(a.split_ctr + cf, (unsigned)(cl - cf));
                handoff[0] = old == (unsigned)(cl - cf) ? 1 : 0;
                handoff[1] = cf;
                handoff[2] = cl - cf + 1;
                handoff[3] = (I * cf / G == first_item) ? 0 : 1;   // the first contributor's slot
            }
            named_bar_sync(hbar, kHalfThreads);
            finish = handoff[0] != 0;
            c_first = handoff[1];
            n_contrib = handoff[2];
            slot_first = handoff[3];
        }

        if (finish) {
            const int sv_off = a.blocks ? a.blocks[cbl].sv_off : cbl * 128;
            const int y_off = a.blocks ? a.blocks[cbl].y_off : cbl * 128;
            for (int n = wl; n < a.rows; n += kHalfWarps) {
                float v[4];
                uint2 sv = make_uint2(0x3C003C00u, 0x3C003C00u), bv = make_uint2(0u, 0u);
                const bool scaled = a.svh && sv_off >= 0 && !a.raw_out;
                const bool biased = a.bias && sv_off >= 0 && !a.raw_out;
                if (scaled) sv = *reinterpret_cast<const uint2*>(a.svh + sv_off + 4 * lane);
                if (biased) bv = *reinterpret_cast<const uint2*>(a.bias + sv_off + 4 * lane);
                if (seg_len == nkb) {
                    const int o = n * kYStride + 4 * lane;
#pragma unroll
                    for (int q = 0; q < 4; q++) v[q] = ybuf[o + q];
                } else {
                    // the contributors' sums, in virtual-CTA order
                    v[0] = v[1] = v[2] = v[3] = 0.f;
                    const float* p0 = a.partials + (size_t)n * 128 + 4 * lane;
#pragma unroll 4
                    for (int j = 0; j < n_contrib; j++) {
                        const int sl = 2 * (c_first + j) + (j == 0 ? slot_first : 0);
                        const float4 p = __ldcg(reinterpret_cast<const float4*>(p0 + (size_t)sl * nv));
                        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) v[q] = __half2float(__float2half_rn(v[q]));
                if (!a.raw_out) {
                    had128_warp(v, lane);
                    const float2 s0 = __half22float2(u32_as_h2(sv.x));
                    const float2 s1 = __half22float2(u32_as_h2(sv.y));
                    v[0] *= EXL3_HAD_SCALE; v[1] *= EXL3_HAD_SCALE; v[2] *= EXL3_HAD_SCALE; v[3] *= EXL3_HAD_SCALE;
                    if (scaled) { v[0] *= s0.x; v[1] *= s0.y; v[2] *= s1.x; v[3] *= s1.y; }
                }
                __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                if (biased) {
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
                // and the one that finishes the last block of this rank announces the rank to all peers.
                named_bar_sync(hbar, kHalfThreads);           // every row of the block has been sent
                if (tidh == 0) {
                    __threadfence();
                    const unsigned done = atomicAdd(a.done_ctr, 1u) + 1u;
                    if (done == (unsigned)ncb) {
                        atomicExch(a.done_ctr, 0u);           // re-armed for the next launch on this workspace
                        __threadfence_system();               // one fence orders all blocks before all arrivals
                        for (int p = 0; p < a.n_peer; p++)
                            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.ctr_peer[p]) : "memory");
                    }
                }
            }
        }
        seg0 = seg_end;
        // more segments follow: all reads of ybuf and of the hand-off words are done
        if (seg0 < nitems) named_bar_sync(hbar, kHalfThreads);
    }
#ifdef EXL3_PROFILE
    if (a.prof && tidh == 0) {
        long long* p = a.prof + (size_t)c * 16;
        p[0] = gt_entry;        // kernel entry of this CTA (ns, GPU wall clock)
        p[1] = gt_init;         // barriers set up, first ring fill issued
        p[2] = gt_dep;          // previous kernel of the stream complete
        p[3] = gt_loop;         // activations ready, main loop starts
        p[4] = gt_last_item;    // last item of the range consumed by this warp
        p[5] = global_ns();     // last segment flushed / finished
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        p[6] = smid;
        p[7] = nitems;
        p[8] = ck_wait;         // clocks warp 0 of the half waited for staged items
        p[9] = ck_loop;         // clocks it spent decoding and multiplying
    }
#endif
}

// ---- host side ----------------------------------------------------------------------------------

template <int K, int CB, int NMMA, bool FAST, bool XFUSED>
static int launch_gemv_t(GemvArgs a, bool pdl, cudaStream_t s)
{
    using L = GemvLayout<K, NMMA>;
    const int nkb = a.t_in >> 3;
    const GemvPlan plan = gemv_plan(a.ncb, nkb, a.rows, a.blocks != nullptr, a.partial_bytes);
    if (plan.grid < 1) return EXL3_E_WORKSPACE;
    if (plan.x_fused != XFUSED) return EXL3_E_UNSUPPORTED;
    a.grid_virtual = plan.grid;
    a.n_slots = plan.n_slots;
    a.cb_xor = 0x3B603B60u;
    a.sixteen = 16u;
    a.xs_bytes = XFUSED ? (plan.n_slots * a.rows + 1) * kXsRowBytes : 0;
    const int stage0 = (2 * kHeaderBytes + 2 * L::kYBytes + 2 * a.xs_bytes + 1023) / 1024 * 1024;
    const int stage_bytes = (XFUSED ? 0 : L::kXBoxBytes) + L::kWeightBytes;
    int stages = (kGemvSmemBytes - stage0) / (2 * stage_bytes);
    stages = std::min(stages, kMaxStages);
    if (stages < kGroups) return EXL3_E_UNSUPPORTED;
    a.stages = stages;
    a.stage0_off = stage0;
    const size_t smem = (size_t)stage0 + 2 * (size_t)stages * stage_bytes;

    static bool attr_set[kMaxDevices] = {};  // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= kMaxDevices) return EXL3_E_UNSUPPORTED;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<K, CB, NMMA, FAST, XFUSED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmemBytes);
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
    cfg.gridDim = dim3((unsigned)((plan.grid + 1) / 2));
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return note_cuda(cudaLaunchKernelEx(&cfg, gemv_kernel<K, CB, NMMA, FAST, XFUSED>, a, tm_w, tm_x));
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
