// Launch tables of the stacked-expert SwitchGLU for decode-class calls (few tokens): every
// (token, slot) pair is a one-row problem against its expert's column range of the stacked
// trellises (the reference maps pairs to experts the same way for its mapped GEMV,
// ponyexl3/mlx/exl3_moe.py:634-683).  One kernel turns the routing indices into the block
// tables and row maps that exl3_gemv_blocks takes for the gate/up launch and the down launch,
// so a call is a handful of launches with no host round trip.
#include <algorithm>

#include "exl3_internal.h"

namespace exl3 {

struct MoeTableArgs {
    const void* indices;   // (n,) expert of every (token, slot) pair, int32 or int64
    int idx64;
    int n, kk, E, D, H;
    int e_lo, e_hi;        // experts held here (the stacked tensors hold e_hi - e_lo experts)
    int32_t* blocks_gu;    // (n * 2 * H/128, 4): phys, xrow, sv_off, y_off
    int32_t* row_src_gu;   // (2n,): token of rotated row 2s + p
    int32_t* suh_row_gu;   // (2n,): row of gu_suh (E*2, D) for rotated row 2s + p
    int32_t* blocks_dn;    // (n * D/128, 4)
    int32_t* suh_row_dn;   // (n,): expert of pair s
    int32_t* counts;       // NULL, or {blocks in use of blocks_gu, of blocks_dn}
};

constexpr int kMoeOwnedMaxPairs = 2048;

// With an expert range (counts != NULL) only the pairs whose expert is held here get blocks;
// their blocks are packed to the front of the tables in pair order and the number in use is left
// on the device for exl3_gemv_blocks_counted.  Rows and outputs keep the numbering of all pairs,
// so the rows of pairs that are computed elsewhere are simply never touched.
__global__ void __launch_bounds__(256) moe_decode_tables_kernel(const MoeTableArgs a)
{
    griddep_launch_dependents();
    griddep_wait();
    __shared__ short before[kMoeOwnedMaxPairs];   // held pairs in front of pair s
    __shared__ unsigned char held[kMoeOwnedMaxPairs];
    const int gb = a.H / 128, db = a.D / 128;
    const int n_gu = a.n * 2 * gb, n_dn = a.n * db;
    const int E_here = a.e_hi - a.e_lo;
    auto expert = [&](int s) -> int {
        const long long e = a.idx64 ? static_cast<const long long*>(a.indices)[s]
                                    : (long long)static_cast<const int*>(a.indices)[s];
        return (int)(e < 0 ? 0 : (e >= a.E ? a.E - 1 : e));       // a bad index must not leave the tensors
    };
    const bool ranged = a.counts != nullptr;
    if (ranged) {
        for (int s = threadIdx.x; s < a.n; s += blockDim.x) {
            const int e = expert(s);
            held[s] = e >= a.e_lo && e < a.e_hi;
        }
        __syncthreads();
        for (int s = threadIdx.x; s < a.n; s += blockDim.x) {
            int q = 0;
            for (int t = 0; t < s; t++) q += held[t];
            before[s] = (short)q;
        }
        __syncthreads();
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            const int total = before[a.n - 1] + held[a.n - 1];
            a.counts[0] = total * 2 * gb;
            a.counts[1] = total * db;
        }
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_gu + n_dn; i += gridDim.x * blockDim.x) {
        if (i < n_gu) {
            const int j = i % gb, sp = i / gb, p = sp & 1, s = sp >> 1;
            const int e = expert(s);
            const bool mine = !ranged || held[s];
            const int el = mine ? e - a.e_lo : 0;
            if (j == 0) {
                a.row_src_gu[sp] = s / a.kk;
                a.suh_row_gu[sp] = 2 * el + p;
            }
            if (!mine) continue;
            const int q = ranged ? before[s] : s;
            int4 b;
            b.x = (p * E_here + el) * gb + j;               // all gates, then all ups
            b.y = 2 * s + p;
            b.z = el * 2 * a.H + p * a.H + 128 * j;
            b.w = s * 2 * a.H + p * a.H + 128 * j;
            reinterpret_cast<int4*>(a.blocks_gu)[(2 * q + p) * gb + j] = b;
        } else {
            const int t = i - n_gu, j = t % db, s = t / db;
            const int e = expert(s);
            const bool mine = !ranged || held[s];
            const int el = mine ? e - a.e_lo : 0;
            if (j == 0) a.suh_row_dn[s] = el;
            if (!mine) continue;
            const int q = ranged ? before[s] : s;
            int4 b;
            b.x = el * db + j;
            b.y = s;
            b.z = el * a.D + 128 * j;
            b.w = s * a.D + 128 * j;
            reinterpret_cast<int4*>(a.blocks_dn)[q * db + j] = b;
        }
    }
}


// ---- prefill-class calls: group the pairs by expert, cut row tiles, write the tile tables ----
struct MoePrefillArgs {
    const void* indices;
    int idx64;
    int n, kk, E, D, H, slots;
    int e_lo, e_hi;        // experts held here; pairs of other experts get no rows
    int32_t* order;        // (n,): sorted position -> pair
    int32_t* row_src_gu;   // (2n,)
    int32_t* suh_row_gu;   // (2n,)
    int32_t* suh_row_dn;   // (n,)
    int32_t* tiles_gu;     // (2 * slots * ceil(H/256), 8)
    int32_t* tiles_dn;     // (slots * ceil(D/256), 8)
    int32_t* counts;       // NULL, or {rotated gate/up rows in use, sorted positions in use}
};

constexpr int kMoeMaxExperts = 1024;

// One CTA: shared-memory histogram, scan, scatter.  32 K pairs take a few microseconds; the
// tables are tiny next to the GEMMs they drive.
//
// Row layout.  The held pairs are sorted by expert; expert e owns sorted positions
// [seg, seg + cnt).  The rotated rows of the gate/up launch keep an expert's rows together —
// gate rows [2 seg, 2 seg + cnt), then up rows [2 seg + cnt, 2 seg + 2 cnt) — so the rows in use
// are the first 2 x (held pairs) and a launch that reads their number from the device skips the
// rest.  Gate and up tiles store to the [gate | up] row of the sorted position.
__global__ void __launch_bounds__(1024) moe_prefill_tables_kernel(const MoePrefillArgs a)
{
    griddep_launch_dependents();
    griddep_wait();
    __shared__ int count[kMoeMaxExperts], seg[kMoeMaxExperts], blk0[kMoeMaxExperts], cursor[kMoeMaxExperts];
    __shared__ int total_blocks;
    const int tid = threadIdx.x;
    const int E_here = a.e_hi - a.e_lo;
    auto expert = [&](int s) -> int {       // local index of the pair's expert, -1: not held here
        const long long e = a.idx64 ? static_cast<const long long*>(a.indices)[s]
                                    : (long long)static_cast<const int*>(a.indices)[s];
        const int ec = (int)(e < 0 ? 0 : (e >= a.E ? a.E - 1 : e));      // a bad index must not leave the tensors
        return ec >= a.e_lo && ec < a.e_hi ? ec - a.e_lo : -1;
    };
    for (int e = tid; e < E_here; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int s = tid; s < a.n; s += blockDim.x) {
        const int e = expert(s);
        if (e >= 0) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (tid == 0) {                       // E <= 1024: a serial scan is a microsecond
        int rows = 0, blocks = 0;
        for (int e = 0; e < E_here; e++) {
            seg[e] = rows;
            blk0[e] = blocks;
            rows += count[e];
            blocks += (count[e] + 255) >> 8;
        }
        total_blocks = blocks;
        if (a.counts) {
            a.counts[0] = 2 * rows;
            a.counts[1] = rows;
        }
    }
    __syncthreads();
    for (int s = tid; s < a.n; s += blockDim.x) {
        const int e = expert(s);
        if (e < 0) continue;
        const int i = atomicAdd(&cursor[e], 1);
        const int pos = seg[e] + i;
        a.order[pos] = s;
        const int tok = s / a.kk;
        const int rg = 2 * seg[e] + i, ru = rg + count[e];
        a.row_src_gu[rg] = tok;
        a.row_src_gu[ru] = tok;
        a.suh_row_gu[rg] = 2 * e;
        a.suh_row_gu[ru] = 2 * e + 1;
        a.suh_row_dn[pos] = e;
    }
    // tile tables: slot = row tile of one expert; every slot x every 256-column tile of the projection
    const int ct_h = (a.H + 255) / 256, ct_d = (a.D + 255) / 256;
    auto put = [&](int32_t* tab, int idx, int row0, int row_end, int tn0, int sv, int ycol, int ncols, int shift) {
        int4 u, v;
        u.x = row0 < row_end ? row0 + shift : 0;
        u.y = row0 < row_end ? row_end + shift : 0;
        u.z = tn0; u.w = sv;
        v.x = ycol; v.y = ncols; v.z = -shift; v.w = 0;
        reinterpret_cast<int4*>(tab)[2 * idx] = u;
        reinterpret_cast<int4*>(tab)[2 * idx + 1] = v;
    };
    auto emit = [&](int slot, int e, int row0, int row_end, int gate_shift, int up_shift) {
        for (int j = 0; j < ct_h; j++) {
            const int nc = min(a.H - 256 * j, 256);
            put(a.tiles_gu, slot * ct_h + j, row0, row_end, e * (a.H / 16) + 16 * j, e * 2 * a.H + 256 * j, 256 * j, nc,
                gate_shift);
            put(a.tiles_gu, (a.slots + slot) * ct_h + j, row0, row_end, (E_here + e) * (a.H / 16) + 16 * j,
                e * 2 * a.H + a.H + 256 * j, a.H + 256 * j, nc, up_shift);
        }
        for (int j = 0; j < ct_d; j++)
            put(a.tiles_dn, slot * ct_d + j, row0, row_end, e * (a.D / 16) + 16 * j, e * a.D + 256 * j, 256 * j,
                min(a.D - 256 * j, 256), 0);
    };
    for (int e = tid; e < E_here; e += blockDim.x) {
        const int nb = (count[e] + 255) >> 8;
        for (int b = 0; b < nb; b++) {
            const int row0 = seg[e] + 256 * b;
            emit(blk0[e] + b, e, row0, min(row0 + 256, seg[e] + count[e]), seg[e], seg[e] + count[e]);
        }
    }
    for (int slot = total_blocks + tid; slot < a.slots; slot += blockDim.x) emit(slot, 0, 0, 0, 0, 0);   // unused
}

}  // namespace exl3

using namespace exl3;

static int moe_decode_tables_impl(const void* indices, int index_bytes, int n_pairs, int top_k, int num_experts,
                                  int e_lo, int e_hi, int64_t d, int64_t h, int32_t* blocks_gu,
                                  int32_t* row_src_gu, int32_t* suh_row_gu, int32_t* blocks_dn,
                                  int32_t* suh_row_dn, int32_t* counts, unsigned flags, exl3_stream_t stream)
{
    if (!indices || !blocks_gu || !row_src_gu || !suh_row_gu || !blocks_dn || !suh_row_dn) return EXL3_E_NULL;
    if (index_bytes != 4 && index_bytes != 8) return EXL3_E_DTYPE;
    if (n_pairs < 1 || top_k < 1 || num_experts < 1 || d < 128 || h < 128 || d % 128 || h % 128)
        return EXL3_E_SHAPE;
    if ((int64_t)n_pairs * (2 * h / 128 + d / 128) > (1 << 28)) return EXL3_E_RANGE;
    if (e_lo < 0 || e_hi <= e_lo || e_hi > num_experts) return EXL3_E_RANGE;
    if (counts && n_pairs > kMoeOwnedMaxPairs) return EXL3_E_RANGE;
    if (((uintptr_t)blocks_gu | (uintptr_t)blocks_dn) & 15) return EXL3_E_ALIGN;
    MoeTableArgs a;
    a.indices = indices;
    a.idx64 = index_bytes == 8;
    a.n = n_pairs; a.kk = top_k; a.E = num_experts; a.D = (int)d; a.H = (int)h;
    a.e_lo = e_lo; a.e_hi = e_hi;
    a.blocks_gu = blocks_gu; a.row_src_gu = row_src_gu; a.suh_row_gu = suh_row_gu;
    a.blocks_dn = blocks_dn; a.suh_row_dn = suh_row_dn;
    a.counts = counts;
    const int total = n_pairs * (int)(2 * h / 128 + d / 128);
    return launch_kernel(moe_decode_tables_kernel, dim3((unsigned)std::min(1024, (total + 255) / 256)), dim3(256), 0,
                         (cudaStream_t)stream, (flags & EXL3_FLAG_PDL) != 0, a);
}

extern "C" int exl3_moe_decode_tables(const void* indices, int index_bytes, int n_pairs, int top_k,
                                      int num_experts, int64_t d, int64_t h, int32_t* blocks_gu,
                                      int32_t* row_src_gu, int32_t* suh_row_gu, int32_t* blocks_dn,
                                      int32_t* suh_row_dn, unsigned flags, exl3_stream_t stream)
{
    return moe_decode_tables_impl(indices, index_bytes, n_pairs, top_k, num_experts, 0, num_experts, d, h,
                                  blocks_gu, row_src_gu, suh_row_gu, blocks_dn, suh_row_dn, nullptr, flags, stream);
}

extern "C" int exl3_moe_decode_tables_range(const void* indices, int index_bytes, int n_pairs, int top_k,
                                            int num_experts, int expert_lo, int expert_hi, int64_t d, int64_t h,
                                            int32_t* blocks_gu, int32_t* row_src_gu, int32_t* suh_row_gu,
                                            int32_t* blocks_dn, int32_t* suh_row_dn, int32_t* counts,
                                            unsigned flags, exl3_stream_t stream)
{
    if (!counts) return EXL3_E_NULL;
    return moe_decode_tables_impl(indices, index_bytes, n_pairs, top_k, num_experts, expert_lo, expert_hi, d, h,
                                  blocks_gu, row_src_gu, suh_row_gu, blocks_dn, suh_row_dn, counts, flags, stream);
}

static int moe_prefill_tables_impl(const void* indices, int index_bytes, int n_pairs, int top_k, int num_experts,
                                   int e_lo, int e_hi, int64_t d, int64_t h, int32_t* order, int32_t* row_src_gu,
                                   int32_t* suh_row_gu, int32_t* suh_row_dn, int32_t* tiles_gu, int32_t* tiles_dn,
                                   int32_t* counts, unsigned flags, exl3_stream_t stream)
{
    if (!indices || !order || !row_src_gu || !suh_row_gu || !suh_row_dn || !tiles_gu || !tiles_dn)
        return EXL3_E_NULL;
    if (index_bytes != 4 && index_bytes != 8) return EXL3_E_DTYPE;
    if (n_pairs < 1 || n_pairs > (1 << 20) || top_k < 1 || num_experts < 1) return EXL3_E_RANGE;
    if (e_lo < 0 || e_hi <= e_lo || e_hi > num_experts || e_hi - e_lo > kMoeMaxExperts) return EXL3_E_RANGE;
    if (d < 128 || h < 128 || d % 128 || h % 128) return EXL3_E_SHAPE;
    if (((uintptr_t)tiles_gu | (uintptr_t)tiles_dn) & 15) return EXL3_E_ALIGN;
    MoePrefillArgs a;
    a.indices = indices;
    a.idx64 = index_bytes == 8;
    a.n = n_pairs; a.kk = top_k; a.E = num_experts; a.D = (int)d; a.H = (int)h;
    a.e_lo = e_lo; a.e_hi = e_hi;
    a.slots = n_pairs / 256 + (e_hi - e_lo);
    a.order = order; a.row_src_gu = row_src_gu; a.suh_row_gu = suh_row_gu; a.suh_row_dn = suh_row_dn;
    a.tiles_gu = tiles_gu; a.tiles_dn = tiles_dn;
    a.counts = counts;
    return launch_kernel(moe_prefill_tables_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream,
                         (flags & EXL3_FLAG_PDL) != 0, a);
}

extern "C" int exl3_moe_prefill_tables(const void* indices, int index_bytes, int n_pairs, int top_k,
                                       int num_experts, int64_t d, int64_t h, int32_t* order,
                                       int32_t* row_src_gu, int32_t* suh_row_gu, int32_t* suh_row_dn,
                                       int32_t* tiles_gu, int32_t* tiles_dn, unsigned flags,
                                       exl3_stream_t stream)
{
    if (num_experts > kMoeMaxExperts) return EXL3_E_RANGE;
    return moe_prefill_tables_impl(indices, index_bytes, n_pairs, top_k, num_experts, 0, num_experts, d, h, order,
                                   row_src_gu, suh_row_gu, suh_row_dn, tiles_gu, tiles_dn, nullptr, flags, stream);
}

extern "C" int exl3_moe_prefill_tables_range(const void* indices, int index_bytes, int n_pairs, int top_k,
                                             int num_experts, int expert_lo, int expert_hi, int64_t d, int64_t h,
                                             int32_t* order, int32_t* row_src_gu, int32_t* suh_row_gu,
                                             int32_t* suh_row_dn, int32_t* tiles_gu, int32_t* tiles_dn,
                                             int32_t* counts, unsigned flags, exl3_stream_t stream)
{
    if (!counts) return EXL3_E_NULL;
    return moe_prefill_tables_impl(indices, index_bytes, n_pairs, top_k, num_experts, expert_lo, expert_hi, d, h,
                                   order, row_src_gu, suh_row_gu, suh_row_dn, tiles_gu, tiles_dn, counts, flags,
                                   stream);
}
