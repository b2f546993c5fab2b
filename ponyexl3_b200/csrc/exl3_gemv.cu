// Host-side dispatch of the streamed GEMV: tuning knobs, the k-split choice, and the switch
// over K.  The kernel template lives in exl3_gemv.cuh and is instantiated once per K in
// exl3_gemv_k{1..8}.cu so the eight translation units compile in parallel.
#include <algorithm>

#include "exl3_internal.h"

namespace exl3 {

int g_gemv_ctas_per_sm = 2;
int g_gemv_smem_budget = 110 * 1024;
static int g_fuse_x_bytes = 40 * 1024;   // fuse the input rotation when its words fit in this
constexpr int kXsRowBytesHost = 544;

static int g_cluster_cache[16][9] = {};

void gemv_set_tuning(int ctas_per_sm, int smem_budget_bytes)
{
    if (ctas_per_sm >= 1 && ctas_per_sm <= 2) g_gemv_ctas_per_sm = ctas_per_sm;
    if (smem_budget_bytes >= 32 * 1024 && smem_budget_bytes <= 226 * 1024)
        g_gemv_smem_budget = smem_budget_bytes;
    for (auto& row : g_cluster_cache)
        for (int& v : row) v = 0;
}

static int g_force_split = 0;
void gemv_force_split(int ksplit) { g_force_split = (ksplit >= 1 && ksplit <= 8) ? ksplit : 0; }

int gemv_active_clusters_probe(int cluster, int smem_bytes);   // exl3_gemv_k4.cu

// Clusters of s CTAs that are resident at once (a cluster must fit inside one GPC, so this
// is not slots / s: e.g. clusters of 7 leave a remainder in every GPC).  Cached per device.
static int active_clusters(int s)
{
    int (&cache)[16][9] = g_cluster_cache;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) dev = 0;
    if (cache[dev][s] == 0) {
        int n = s == 1 ? device_sm_count() * g_gemv_ctas_per_sm
                       : gemv_active_clusters_probe(s, g_gemv_smem_budget);
        if (n <= 0) n = std::max(1, device_sm_count() * g_gemv_ctas_per_sm / s / 2);
        n = std::min(n, std::max(1, device_sm_count() * g_gemv_ctas_per_sm / s));
        cache[dev][s] = n;
    }
    return cache[dev][s];
}

// k-split S and grid for a layer.  Time is proportional to (waves of clusters) x (k-blocks
// per CTA); pick the S that minimises it, preferring the smaller S on ties.
// The leader keeps (S - 1) x rows x 128 floats of landing slots for the others' partial sums;
// S is capped so that they stay under 24 KiB.
void gemv_choose_split(int ncb, int nkb, int rows, int* ksplit, int* grid)
{
    int best_s = 1, best_clusters = 1;
    long best_t = -1;
    const int s_max = std::min(std::min(8, nkb), 1 + 24576 / (rows * 512));
    const int s_lo = g_force_split ? std::min(g_force_split, s_max) : 1;
    const int s_hi = g_force_split ? s_lo : s_max;
    for (int s = s_lo; s <= s_hi; s++) {
        const int clusters = std::min(ncb, active_clusters(s));
        const long waves = (ncb + clusters - 1) / clusters;
        const long t = waves * ((nkb + s - 1) / s) * 16 + s;   // + s: cost of gathering s partial sums
        if (best_t < 0 || t < best_t) {
            best_t = t;
            best_s = s;
            best_clusters = clusters;
        }
    }
    *ksplit = best_s;
    *grid = best_clusters * best_s;
}

bool gemv_x_is_fused(int rows, int t_in, int ncb)
{
    if (rows > 8) return false;
    int s, grid;
    gemv_choose_split(ncb, t_in >> 3, rows, &s, &grid);
    const int nkb = t_in >> 3;
    const int klen = (nkb + s - 1) / s;
    return (klen * rows + 1) * kXsRowBytesHost <= g_fuse_x_bytes;
}

// A block-table launch can rotate its activations in the kernel when every cluster computes a
// single block: the CTA then needs one (rotated row, sign vector) pair for its whole life.
bool gemv_blocks_x_is_fused(int rows, int t_in, int ncb)
{
    if (!gemv_x_is_fused(rows, t_in, ncb)) return false;
    int s, grid;
    gemv_choose_split(ncb, t_in >> 3, rows, &s, &grid);
    return ncb <= grid / s;
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
