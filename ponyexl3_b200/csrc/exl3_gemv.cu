// Host-side dispatch of the streamed GEMV: the launch plan (grid, fused rotation or not) and the
// switch over K.  The kernel template lives in exl3_gemv.cuh and is instantiated once per K in
// exl3_gemv_k{1..8}.cu so the eight translation units compile in parallel.
#include <algorithm>

#include "exl3_internal.h"

namespace exl3 {

constexpr int kCtasPerSm = 2;           // virtual CTAs: the two halves of the one real CTA per SM
static int g_fuse_x_bytes = 28 * 1024;   // fuse the input rotation when a half's words fit in this
constexpr int kXsRowBytesHost = 544;

static int g_gemv_max_grid = 0;          // 0: two virtual CTAs per SM
static bool g_gemv_search_grid = true;

// Benchmark hook (exl3_b200_tuning.h): cap the grid and the size of the fused-rotation buffer.
void gemv_set_tuning(int max_grid, int fuse_x_bytes)
{
    g_gemv_max_grid = max_grid > 0 ? std::min(max_grid, kGemvMaxGrid) : 0;
    g_gemv_search_grid = max_grid == 0;      // a forced count is taken as it is
    if (fuse_x_bytes >= 0 && fuse_x_bytes <= 28 * 1024) g_fuse_x_bytes = fuse_x_bytes;
}

size_t gemv_partial_bytes(int rows)
{
    return (size_t)kGemvMaxGrid * (size_t)rows * kGemvPartialBytesPerCtaRow;
}

// Cost of dealing the items to g virtual CTAs, in item times of one warp group: the slowest
// virtual CTA sets the launch time; each of its segments costs its rounds (four groups, one item
// each per round) plus a hand-over of the partial sums, which stalls the half for most of an item
// time.
static double plan_cost(int64_t ncb, int nkb, int g)
{
    const int64_t items = ncb * nkb;
    double worst = 0;
    for (int c = 0; c < g; c++) {
        int64_t i0 = items * c / g;
        const int64_t i1 = items * (c + 1) / g;
        double t = 0;
        while (i0 < i1) {
            const int64_t end = std::min(i1, (i0 / nkb + 1) * nkb);
            t += (double)((end - i0 + 3) / 4) + 0.8;
            i0 = end;
        }
        worst = std::max(worst, t);
    }
    return worst;
}

// The items (column blocks x k-blocks) are dealt out evenly to `grid` virtual CTAs (two per SM:
// the halves of the real CTA), fewer when the layer has fewer items or the caller's partial-sum
// area holds fewer.  Among the counts down to half of the largest one the cheapest by
// plan_cost is taken: a count that lets ranges end on block boundaries (136 column blocks on 272
// of 296 halves) saves more by avoiding second segments than it loses in idle SMs.  The choice
// is remembered per shape.
GemvPlan gemv_plan(int64_t ncb, int nkb, int rows, bool table, size_t partial_bytes)
{
    GemvPlan p = {};
    const int64_t items = ncb * nkb;
    int64_t grid = std::min<int64_t>(kGemvMaxGrid, (int64_t)device_sm_count() * kCtasPerSm);
    if (g_gemv_max_grid > 0) grid = std::min<int64_t>(grid, g_gemv_max_grid);
    grid = std::min<int64_t>(grid, (int64_t)(partial_bytes / ((size_t)rows * kGemvPartialBytesPerCtaRow)));
    grid = std::min(grid, items);
    p.grid = (int)std::max<int64_t>(grid, 0);
    if (p.grid < 1) return p;
    if (g_gemv_search_grid && p.grid >= 16 && ncb <= (1 << 16)) {
        struct Memo { int64_t ncb; int nkb, gmax, best; };
        static thread_local Memo memo[16] = {};
        static thread_local int memo_next = 0;
        int best = 0;
        for (const Memo& m : memo)
            if (m.ncb == ncb && m.nkb == nkb && m.gmax == p.grid) best = m.best;
        if (!best) {
            double best_cost = 0;
            for (int g = p.grid; g >= p.grid - p.grid / 2; g--) {
                const double cst = plan_cost(ncb, nkb, g);
                if (!best || cst < best_cost - 1e-9) { best = g; best_cost = cst; }
            }
            memo[memo_next] = Memo{ncb, nkb, p.grid, best};
            memo_next = (memo_next + 1) % 16;
        }
        p.grid = best;
    }
    const int64_t range = (items + p.grid - 1) / p.grid;         // longest item range of a virtual CTA
    const int64_t slots = table ? range : std::min<int64_t>(range, nkb);
    p.n_slots = (int)std::min<int64_t>(slots, 1 << 20);
    p.x_fused = rows <= 8 && (slots * rows + 1) * kXsRowBytesHost <= g_fuse_x_bytes;
    return p;
}

bool gemv_x_is_fused(int rows, int t_in, int64_t ncb, bool table, size_t partial_bytes)
{
    return gemv_plan(ncb, t_in >> 3, rows, table, partial_bytes).x_fused;
}

template <int K> int launch_gemv_k(const GemvArgs& a, int cb, bool pdl, cudaStream_t s);
extern template int launch_gemv_k<1>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<2>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<3>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<4>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<5>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<6>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<7>(const GemvArgs&, int, bool, cudaStream_t);
extern template int launch_gemv_k<8>(const GemvArgs&, int, bool, cudaStream_t);

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
