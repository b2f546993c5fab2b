// extern "C" surface of libexl3b200.so: argument validation on the host, then the
// kernel launchers.  No allocation; the only process-wide state is per-device caches of
// immutable facts (SM count, function attributes) and the two benchmark knobs of
// exl3_b200_tuning.h, which no product path sets.
#include <stdio.h>
#include <string.h>

#include "exl3_internal.h"
#include "../../include/exl3_b200_tuning.h"
#include "exl3_tma.h"

namespace exl3 {

char* g_cuda_err_buf();

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return EXL3_E_CUDA;
    cuuint64_t gdim[5], gstr[5];
    cuuint32_t bdim[5], estr[5];
    for (int i = 0; i < rank; i++) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUresult r = fn(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bdim, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_cuda_err_buf(), 256, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return EXL3_E_CUDA;
    }
    return EXL3_OK;
}

static thread_local char g_cuda_err[256] = "";
char* g_cuda_err_buf() { return g_cuda_err; }

int note_cuda(cudaError_t e)
{
    if (e == cudaSuccess) return EXL3_OK;
    strncpy(g_cuda_err, cudaGetErrorString(e), sizeof(g_cuda_err) - 1);
    g_cuda_err[sizeof(g_cuda_err) - 1] = 0;
    return EXL3_E_CUDA;
}

int check_launch() { return note_cuda(cudaGetLastError()); }

int device_sm_count()
{
    static int cached[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

#ifdef EXL3_PROFILE
// Timeline builds only: a caller-owned device buffer that consecutive GEMV launches fill with
// per-CTA time stamps, kGemvMaxGrid x 16 x 8 bytes per launch, until it is full.
static long long* g_prof_buf = nullptr;
static size_t g_prof_launches = 0, g_prof_next = 0;
static long long* next_prof_slot()
{
    if (!g_prof_buf || g_prof_next >= g_prof_launches) return nullptr;
    return g_prof_buf + (g_prof_next++) * (size_t)kGemvMaxGrid * 16;
}
#endif

static int glu_mode(unsigned flags)
{
    return (flags & EXL3_FLAG_GLU_GELU) ? GLU_GELU : (flags & EXL3_FLAG_GLU_SILU) ? GLU_SILU : GLU_NONE;
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace exl3

using namespace exl3;

extern "C" {

int exl3_version(void) { return EXL3_B200_VERSION; }

const char* exl3_error_string(int code)
{
    switch (code) {
        case EXL3_OK: return "ok";
        case EXL3_E_NULL: return "a required pointer is NULL";
        case EXL3_E_K: return "K must be in [1, 8]";
        case EXL3_E_CODEBOOK: return "unknown codebook mode (0 = 3INST, 1 = MCG, 2 = MUL1)";
        case EXL3_E_SHAPE: return "bad shape: features must be positive multiples of 128 (tiles of 16)";
        case EXL3_E_ROWS: return "row count outside the supported range of this entry point";
        case EXL3_E_ALIGN: return "pointer or stride not aligned as required";
        case EXL3_E_WORKSPACE: return "workspace missing or too small";
        case EXL3_E_DTYPE: return "unknown activation dtype";
        case EXL3_E_CUDA: return "CUDA runtime error";
        case EXL3_E_RANGE: return "index or slice out of range";
        case EXL3_E_UNSUPPORTED: return "configuration not supported";
        default: return "unknown error code";
    }
}

const char* exl3_last_cuda_error(void) { return g_cuda_err; }

int exl3_unpack(const uint16_t* trellis, int64_t n_tiles, int k, uint16_t* codewords,
                exl3_stream_t stream)
{
    if (!trellis || !codewords) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (n_tiles < 0) return EXL3_E_SHAPE;
    if (!aligned(trellis, 4) || !aligned(codewords, 16)) return EXL3_E_ALIGN;
    if (n_tiles == 0) return EXL3_OK;
    return launch_unpack(reinterpret_cast<const uint32_t*>(trellis), n_tiles, k, codewords,
                         (cudaStream_t)stream);
}

int exl3_decode(const uint16_t* trellis, int64_t t_in, int64_t t_out, int k, int cb, int64_t tn0,
                int64_t tn_count, uint16_t* w, int64_t ld, exl3_stream_t stream)
{
    if (!trellis || !w) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    if (t_in < 0 || t_out < 0 || tn_count < 0) return EXL3_E_SHAPE;
    if (tn0 < 0 || tn0 + tn_count > t_out || ld < 16 * tn_count) return EXL3_E_RANGE;
    if (!aligned(trellis, 4)) return EXL3_E_ALIGN;
    if (t_in == 0 || tn_count == 0) return EXL3_OK;
    return launch_decode(reinterpret_cast<const uint32_t*>(trellis), t_in, t_out, k, cb, tn0,
                         tn_count, reinterpret_cast<__half*>(w), ld, (cudaStream_t)stream);
}

int exl3_codebook_table(int cb, uint16_t* table65536, exl3_stream_t stream)
{
    if (!table65536) return EXL3_E_NULL;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    return launch_table(cb, reinterpret_cast<__half*>(table65536), (cudaStream_t)stream);
}

static int check_dtype_align(const void* x, int x_dtype, int64_t stride)
{
    switch (x_dtype) {
        case EXL3_DT_F16:
        case EXL3_DT_BF16:
            if (!aligned(x, 8) || stride % 4) return EXL3_E_ALIGN;
            return EXL3_OK;
        case EXL3_DT_F32:
            if (!aligned(x, 16) || stride % 4) return EXL3_E_ALIGN;
            return EXL3_OK;
        default: return EXL3_E_DTYPE;
    }
}

int exl3_hadamard128(const void* x, int x_dtype, int64_t rows, int64_t n, int64_t x_row_stride,
                     const uint16_t* pre, const uint16_t* post, uint16_t* out, exl3_stream_t stream)
{
    if (!x || !out) return EXL3_E_NULL;
    if (rows < 0 || n <= 0 || n % 128) return EXL3_E_SHAPE;
    if (x_row_stride < n) return EXL3_E_SHAPE;
    int rc = check_dtype_align(x, x_dtype, x_row_stride);
    if (rc) return rc;
    if (!aligned(out, 8) || (pre && !aligned(pre, 8)) || (post && !aligned(post, 8))) return EXL3_E_ALIGN;
    if (rows == 0) return EXL3_OK;
    return launch_hadamard(x, x_dtype, rows, n, x_row_stride, reinterpret_cast<const __half*>(pre),
                           reinterpret_cast<const __half*>(post), reinterpret_cast<__half*>(out),
                           nullptr, nullptr, nullptr, false, HAD_OUT_F16, (cudaStream_t)stream);
}

// Where the partial sums of split column blocks start: after the rotated activations (one word
// per element), on a 256-byte boundary.
static size_t gemv_partial_offset(int64_t xh_rows, int64_t in)
{
    return (kWsScratch + (size_t)xh_rows * (size_t)in * 4 + 255) & ~(size_t)255;
}

size_t exl3_workspace_bytes(int64_t max_rows, int64_t max_in)
{
    if (max_rows < 1) max_rows = 1;
    if (max_in < 128) max_in = 128;
    return gemv_partial_offset(max_rows, max_in) + gemv_partial_bytes((int)(max_rows < 16 ? max_rows : 16));
}

int exl3_workspace_init(void* workspace, size_t bytes, exl3_stream_t stream)
{
    if (!workspace) return EXL3_E_NULL;
    if (bytes < kWsScratch) return EXL3_E_WORKSPACE;
    if (!aligned(workspace, 256)) return EXL3_E_ALIGN;
    return note_cuda(cudaMemsetAsync(workspace, 0, kWsScratch, (cudaStream_t)stream));
}

int exl3_workspace_status(const void* workspace, int* status_out, exl3_stream_t stream)
{
    if (!workspace || !status_out) return EXL3_E_NULL;
    cudaError_t e = cudaMemcpyAsync(status_out, workspace, sizeof(int), cudaMemcpyDeviceToHost,
                                    (cudaStream_t)stream);
    if (e != cudaSuccess) return note_cuda(e);
    return note_cuda(cudaStreamSynchronize((cudaStream_t)stream));
}

// Peer description of the fused output all-gather (n == 0: plain local output).
struct PeerOut {
    int n = 0;
    int64_t col0 = 0;
    const uint64_t* y = nullptr;      // host arrays of device pointers
    const uint64_t* ctr = nullptr;
    uint32_t* wait_ctr = nullptr;     // the input row is complete after wait_target arrivals here
    uint32_t wait_target = 0;
};

static int gemv_common(const void* x, int x_dtype, int rows, int64_t x_row_stride, const uint16_t* trellis,
                       int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
                       const uint16_t* bias, uint16_t* y, int64_t y_row_stride, void* workspace,
                       size_t workspace_bytes, unsigned flags, exl3_stream_t stream, const PeerOut& peer)
{
    if (!x || !trellis || !y) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    if (t_in <= 0 || t_out <= 0 || t_in % 8 || t_out % 8) return EXL3_E_SHAPE;
    if (t_in > (1 << 24) || t_out > (1 << 24)) return EXL3_E_SHAPE;
    if (rows < 1 || rows > 16) return EXL3_E_ROWS;
    const int64_t in = 16 * t_in, out = 16 * t_out;
    const int glu = glu_mode(flags);
    if (x_row_stride < (glu ? 2 * in : in) || y_row_stride < out) return EXL3_E_SHAPE;
    int rc = check_dtype_align(x, x_dtype, x_row_stride);
    if (rc) return rc;
    if (!aligned(trellis, 16) || !aligned(y, 8) || y_row_stride % 4) return EXL3_E_ALIGN;
    if ((suh && !aligned(suh, 8)) || (svh && !aligned(svh, 8)) || (bias && !aligned(bias, 8)))
        return EXL3_E_ALIGN;
    if (!workspace) return EXL3_E_WORKSPACE;
    if (!aligned(workspace, 256)) return EXL3_E_ALIGN;
    const size_t part_off = gemv_partial_offset(rows, in);
    if (workspace_bytes < part_off + (size_t)rows * kGemvPartialBytesPerCtaRow) return EXL3_E_WORKSPACE;
    const size_t part_bytes = workspace_bytes - part_off;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint32_t* xh = reinterpret_cast<uint32_t*>(ws + kWsScratch);
    const bool pdl = (flags & EXL3_FLAG_PDL) != 0;
    const bool fast = (flags & EXL3_FLAG_FAST_ACCUM) != 0 && cb != CB_MUL1;
    cudaStream_t s = (cudaStream_t)stream;

    const bool x_fused = gemv_x_is_fused(rows, (int)t_in, t_out / 8, false, part_bytes);
    // only the kernel that reads x can wait for it: with the separate rotation kernel the caller
    // has to run exl3_peer_wait first
    if (peer.wait_ctr && !x_fused) return EXL3_E_UNSUPPORTED;
    if (!x_fused) {
        rc = launch_hadamard(x, x_dtype, rows, in, x_row_stride, reinterpret_cast<const __half*>(suh),
                             nullptr, reinterpret_cast<__half*>(xh), nullptr, nullptr, nullptr, pdl,
                             fast ? HAD_OUT_PAIR_XX : HAD_OUT_PAIR_X0, s, glu);
        if (rc) return rc;
    }

    GemvArgs a = {};
    a.x_glu = glu;
    a.trellis = reinterpret_cast<const uint32_t*>(trellis);
    a.xh = xh;
    a.svh = reinterpret_cast<const __half*>(svh);
    a.bias = reinterpret_cast<const __half*>(bias);
    a.y = reinterpret_cast<__half*>(y);
    a.blocks = nullptr;
    a.status = reinterpret_cast<int*>(ws + kWsStatus);
    a.y_row_stride = y_row_stride;
    a.t_in = (int)t_in;
    a.t_out_total = (int)t_out;
    a.ncb = (int)(t_out / 8);
    a.rows = rows;
    a.x_rows_total = rows;
    a.raw_out = 0;
    a.fast_accum = fast ? 1 : 0;
    a.x = x;
    a.suh = reinterpret_cast<const __half*>(suh);
    a.x_row_stride = x_row_stride;
    a.x_dtype = x_dtype;
    a.x_fused = x_fused ? 1 : 0;
    a.partials = reinterpret_cast<float*>(ws + part_off);
    a.partial_bytes = part_bytes;
    a.split_ctr = reinterpret_cast<unsigned*>(ws + kWsSplitCtr);
#ifdef EXL3_PROFILE
    a.prof = next_prof_slot();
#endif
    a.n_peer = peer.n;
    a.y_col0 = peer.col0;
    a.done_ctr = reinterpret_cast<unsigned*>(ws + kWsDoneCtr);
    a.wait_ctr = reinterpret_cast<unsigned*>(peer.wait_ctr);
    a.wait_target = peer.wait_target;
    a.pass_ctr = reinterpret_cast<unsigned*>(ws + kWsPassCtr);
    for (int p = 0; p < peer.n; p++) {
        a.y_peer[p] = reinterpret_cast<__half*>(peer.y[p]);
        a.ctr_peer[p] = reinterpret_cast<unsigned*>(peer.ctr[p]);
    }
    return launch_gemv(a, k, cb, pdl, s);
}

int exl3_gemv(const void* x, int x_dtype, int rows, int64_t x_row_stride, const uint16_t* trellis,
              int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
              const uint16_t* bias, uint16_t* y, int64_t y_row_stride, void* workspace,
              size_t workspace_bytes, unsigned flags, exl3_stream_t stream)
{
    return gemv_common(x, x_dtype, rows, x_row_stride, trellis, t_in, t_out, k, cb, suh, svh, bias, y,
                       y_row_stride, workspace, workspace_bytes, flags, stream, PeerOut{});
}

int exl3_gemv_peers(const void* x, int x_dtype, int rows, int64_t x_row_stride, const uint16_t* trellis,
                    int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
                    const uint16_t* bias, const uint64_t* y_peers, const uint64_t* counter_peers, int n_peers,
                    int64_t full_row_stride, int64_t col0, void* workspace, size_t workspace_bytes,
                    unsigned flags, exl3_stream_t stream)
{
    if (!y_peers || !counter_peers) return EXL3_E_NULL;
    if (n_peers < 1 || n_peers > kMaxPeers) return EXL3_E_RANGE;
    if (col0 < 0 || col0 % 128 || col0 + 16 * t_out > full_row_stride) return EXL3_E_SHAPE;
    for (int p = 0; p < n_peers; p++) {
        if (!y_peers[p] || !counter_peers[p]) return EXL3_E_NULL;
        if (y_peers[p] % 8 || counter_peers[p] % 4) return EXL3_E_ALIGN;
    }
    PeerOut peer;
    peer.n = n_peers;
    peer.col0 = col0;
    peer.y = y_peers;
    peer.ctr = counter_peers;
    // the local y of the plain entry point is unused; hand in rank 0's buffer for the checks
    return gemv_common(x, x_dtype, rows, x_row_stride, trellis, t_in, t_out, k, cb, suh, svh, bias,
                       reinterpret_cast<uint16_t*>(y_peers[0]), full_row_stride, workspace, workspace_bytes,
                       flags, stream, peer);
}

int exl3_gemv_peers_after(const void* x, int x_dtype, int rows, int64_t x_row_stride, const uint16_t* trellis,
                          int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
                          const uint16_t* bias, const uint64_t* y_peers, const uint64_t* counter_peers, int n_peers,
                          int64_t full_row_stride, int64_t col0, uint32_t* wait_counter, uint32_t wait_target,
                          void* workspace, size_t workspace_bytes, unsigned flags, exl3_stream_t stream)
{
    if (!y_peers || !counter_peers || !wait_counter) return EXL3_E_NULL;
    if (n_peers < 1 || n_peers > kMaxPeers || wait_target == 0) return EXL3_E_RANGE;
    if (col0 < 0 || col0 % 128 || col0 + 16 * t_out > full_row_stride) return EXL3_E_SHAPE;
    if (reinterpret_cast<uintptr_t>(wait_counter) % 4) return EXL3_E_ALIGN;
    for (int p = 0; p < n_peers; p++) {
        if (!y_peers[p] || !counter_peers[p]) return EXL3_E_NULL;
        if (y_peers[p] % 8 || counter_peers[p] % 4) return EXL3_E_ALIGN;
    }
    PeerOut peer;
    peer.n = n_peers;
    peer.col0 = col0;
    peer.y = y_peers;
    peer.ctr = counter_peers;
    peer.wait_ctr = wait_counter;
    peer.wait_target = wait_target;
    return gemv_common(x, x_dtype, rows, x_row_stride, trellis, t_in, t_out, k, cb, suh, svh, bias,
                       reinterpret_cast<uint16_t*>(y_peers[0]), full_row_stride, workspace, workspace_bytes,
                       flags, stream, peer);
}

static int gemv_blocks_impl(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                            const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                            const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                            const int32_t* blocks, int64_t n_blocks, const int32_t* n_blocks_dev, int rows,
                            const uint16_t* svh, const uint16_t* bias, uint16_t* y, int64_t y_row_stride,
                            int raw_out, void* workspace, size_t workspace_bytes, unsigned flags,
                            exl3_stream_t stream)
{
    if (!x || !trellis || !y || !blocks) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    if (t_in <= 0 || t_out_total <= 0 || t_in % 8 || t_out_total % 8) return EXL3_E_SHAPE;
    if (t_in > (1 << 24) || t_out_total > (1 << 24)) return EXL3_E_SHAPE;
    if (rows < 1 || rows > 16 || xh_rows < rows || xh_rows > (1 << 24)) return EXL3_E_ROWS;
    if (n_blocks < 0 || n_blocks > (1 << 24)) return EXL3_E_SHAPE;
    const int64_t in = 16 * t_in;
    const int glu = glu_mode(flags);
    if (x_row_stride < (glu ? 2 * in : in)) return EXL3_E_SHAPE;
    int rc = check_dtype_align(x, x_dtype, x_row_stride);
    if (rc) return rc;
    if (!aligned(trellis, 16) || !aligned(y, 8) || y_row_stride % 4 || !aligned(blocks, 16))
        return EXL3_E_ALIGN;
    if ((suh && !aligned(suh, 8)) || (svh && !aligned(svh, 8)) || (bias && !aligned(bias, 8)))
        return EXL3_E_ALIGN;
    if (!workspace) return EXL3_E_WORKSPACE;
    if (!aligned(workspace, 256)) return EXL3_E_ALIGN;
    const size_t part_off = gemv_partial_offset(xh_rows, in);
    if (workspace_bytes < part_off + (size_t)rows * kGemvPartialBytesPerCtaRow) return EXL3_E_WORKSPACE;
    const size_t part_bytes = workspace_bytes - part_off;
    if (n_blocks == 0) return EXL3_OK;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint32_t* xh = reinterpret_cast<uint32_t*>(ws + kWsScratch);
    const bool pdl = (flags & EXL3_FLAG_PDL) != 0;
    const bool fast = (flags & EXL3_FLAG_FAST_ACCUM) != 0 && cb != CB_MUL1;
    cudaStream_t s = (cudaStream_t)stream;
    // Few rows and short item ranges: the kernel rotates the rows of its own blocks; else a
    // rotation kernel fills the workspace first.
    const bool x_fused = gemv_x_is_fused(rows, (int)t_in, n_blocks, true, part_bytes);
    if (!x_fused) {
        rc = launch_hadamard(x, x_dtype, xh_rows, in, x_row_stride, reinterpret_cast<const __half*>(suh),
                             nullptr, reinterpret_cast<__half*>(xh), row_src, suh_row, nullptr, pdl,
                             fast ? HAD_OUT_PAIR_XX : HAD_OUT_PAIR_X0, s, glu);
        if (rc) return rc;
    }
    GemvArgs a = {};
    a.x_glu = glu;
    a.trellis = reinterpret_cast<const uint32_t*>(trellis);
    a.xh = xh;
    a.svh = reinterpret_cast<const __half*>(svh);
    a.bias = reinterpret_cast<const __half*>(bias);
    a.y = reinterpret_cast<__half*>(y);
    a.blocks = reinterpret_cast<const ColBlock*>(blocks);
    a.status = reinterpret_cast<int*>(ws + kWsStatus);
    a.y_row_stride = y_row_stride;
    a.t_in = (int)t_in;
    a.t_out_total = (int)t_out_total;
    a.ncb = (int)n_blocks;
    a.ncb_dev = n_blocks_dev;
    a.rows = rows;
    a.x_rows_total = (int)xh_rows;
    a.raw_out = raw_out ? 1 : 0;
    a.fast_accum = fast ? 1 : 0;
    a.x = x;
    a.suh = reinterpret_cast<const __half*>(suh);
    a.x_row_stride = x_row_stride;
    a.x_dtype = x_dtype;
    a.x_fused = x_fused ? 1 : 0;
    a.row_src = row_src;
    a.suh_row = suh_row;
    a.partials = reinterpret_cast<float*>(ws + part_off);
    a.partial_bytes = part_bytes;
    a.split_ctr = reinterpret_cast<unsigned*>(ws + kWsSplitCtr);
    a.done_ctr = reinterpret_cast<unsigned*>(ws + kWsDoneCtr);
    return launch_gemv(a, k, cb, pdl, s);
}

int exl3_gemv_blocks(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                     const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                     const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                     const int32_t* blocks, int64_t n_blocks, int rows, const uint16_t* svh,
                     const uint16_t* bias, uint16_t* y, int64_t y_row_stride, int raw_out,
                     void* workspace, size_t workspace_bytes, unsigned flags, exl3_stream_t stream)
{
    return gemv_blocks_impl(x, x_dtype, x_row_stride, xh_rows, row_src, suh, suh_row, trellis, t_in, t_out_total,
                            k, cb, blocks, n_blocks, nullptr, rows, svh, bias, y, y_row_stride, raw_out,
                            workspace, workspace_bytes, flags, stream);
}

int exl3_gemv_blocks_counted(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                             const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                             const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                             const int32_t* blocks, int64_t max_blocks, const int32_t* n_blocks_dev, int rows,
                             const uint16_t* svh, const uint16_t* bias, uint16_t* y, int64_t y_row_stride,
                             int raw_out, void* workspace, size_t workspace_bytes, unsigned flags,
                             exl3_stream_t stream)
{
    if (!n_blocks_dev) return EXL3_E_NULL;
    if (reinterpret_cast<uintptr_t>(n_blocks_dev) % 4) return EXL3_E_ALIGN;
    return gemv_blocks_impl(x, x_dtype, x_row_stride, xh_rows, row_src, suh, suh_row, trellis, t_in, t_out_total,
                            k, cb, blocks, max_blocks, n_blocks_dev, rows, svh, bias, y, y_row_stride, raw_out,
                            workspace, workspace_bytes, flags, stream);
}

size_t exl3_gemm_workspace_bytes(int64_t rows, int64_t in)
{
    if (rows < 1) rows = 1;
    if (in < 128) in = 128;
    return ((size_t)kWsScratch + (size_t)rows * (size_t)in * 2 + 255) & ~(size_t)255;
}

int exl3_gemm(const void* x, int x_dtype, int64_t rows, int64_t x_row_stride, const uint16_t* trellis,
              int64_t t_in, int64_t t_out, int k, int cb, const uint16_t* suh, const uint16_t* svh,
              const uint16_t* bias, uint16_t* y, int64_t y_row_stride, void* workspace,
              size_t workspace_bytes, unsigned flags, exl3_stream_t stream)
{
    (void)flags;
    if (!x || !trellis || !y) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    if (t_in <= 0 || t_out <= 0 || t_in % 8 || t_out % 8) return EXL3_E_SHAPE;
    if (t_in > (1 << 24) || t_out > (1 << 24)) return EXL3_E_SHAPE;
    if (rows < 1 || rows > (1 << 30)) return EXL3_E_ROWS;
    const int64_t in = 16 * t_in, out = 16 * t_out;
    if (x_row_stride < in || y_row_stride < out) return EXL3_E_SHAPE;
    int rc = check_dtype_align(x, x_dtype, x_row_stride);
    if (rc) return rc;
    if (!aligned(trellis, 16) || !aligned(y, 16) || y_row_stride % 8) return EXL3_E_ALIGN;
    if ((suh && !aligned(suh, 8)) || (svh && !aligned(svh, 16)) || (bias && !aligned(bias, 16)))
        return EXL3_E_ALIGN;
    if (!workspace) return EXL3_E_WORKSPACE;
    if (!aligned(workspace, 256)) return EXL3_E_ALIGN;
    if (workspace_bytes < exl3_gemm_workspace_bytes(rows, in)) return EXL3_E_WORKSPACE;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    __half* xh = reinterpret_cast<__half*>(ws + kWsScratch);
    cudaStream_t s = (cudaStream_t)stream;
    rc = launch_hadamard(x, x_dtype, rows, in, x_row_stride, reinterpret_cast<const __half*>(suh), nullptr,
                         xh, nullptr, nullptr, nullptr, false, HAD_OUT_F16, s);
    if (rc) return rc;
    GemmArgs a = {};
    a.svh = reinterpret_cast<const __half*>(svh);
    a.bias = reinterpret_cast<const __half*>(bias);
    a.y = reinterpret_cast<__half*>(y);
    a.status = reinterpret_cast<int*>(ws + kWsStatus);
    a.y_row_stride = y_row_stride;
    a.m = (int)rows;
    a.xh_rows = (int)rows;
    a.t_in = (int)t_in;
    a.t_out = (int)t_out;
    a.y_wide = (y_row_stride % 16 == 0 && aligned(y, 32)) ? 1 : 0;   // 32-byte stores in the epilogue
    return launch_gemm(a, k, cb, xh, reinterpret_cast<const uint32_t*>(trellis), s);
}

struct TilePeers {
    const int32_t* xh_rows_dev = nullptr;   // rotated rows in use, on the device (NULL: all xh_rows)
    int n = 0;                              // GPUs the output rows are spread over (0: plain local y)
    int64_t rows_per_peer = 0;
    const uint64_t* y = nullptr;            // host arrays of device pointers
    const uint64_t* ctr = nullptr;
};

static int gemm_tiles_impl(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                           const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                           const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                           const int32_t* tiles, int64_t n_tiles, const uint16_t* svh, uint16_t* y,
                           int64_t y_row_stride, const int32_t* y_row_map, void* workspace, size_t workspace_bytes,
                           unsigned flags, exl3_stream_t stream, const TilePeers& peers)
{
    if (!x || !trellis || !y || !tiles) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    if (t_in <= 0 || t_out_total <= 0 || t_in % 8 || t_out_total % 8) return EXL3_E_SHAPE;
    if (t_in > (1 << 24) || t_out_total > (1 << 24)) return EXL3_E_SHAPE;
    if (xh_rows < 1 || xh_rows > (1 << 30)) return EXL3_E_ROWS;
    if (n_tiles < 0 || n_tiles > (1 << 24)) return EXL3_E_SHAPE;
    const int64_t in = 16 * t_in;
    const int glu = glu_mode(flags);
    if (x_row_stride < (glu ? 2 * in : in)) return EXL3_E_SHAPE;
    int rc = check_dtype_align(x, x_dtype, x_row_stride);
    if (rc) return rc;
    if (!aligned(trellis, 16) || !aligned(y, 16) || y_row_stride % 8 || !aligned(tiles, 16))
        return EXL3_E_ALIGN;
    if ((suh && !aligned(suh, 8)) || (svh && !aligned(svh, 16))) return EXL3_E_ALIGN;
    if (!workspace) return EXL3_E_WORKSPACE;
    if (!aligned(workspace, 256)) return EXL3_E_ALIGN;
    if (workspace_bytes < exl3_gemm_workspace_bytes(xh_rows, in)) return EXL3_E_WORKSPACE;
    if (peers.n < 0 || peers.n > kMaxPeers) return EXL3_E_RANGE;
    if (peers.n > 0 && (!peers.y || !peers.ctr || peers.rows_per_peer < 1 || peers.rows_per_peer > (1 << 30) || !y_row_map))
        return EXL3_E_NULL;
    if (n_tiles == 0) return EXL3_OK;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    __half* xh = reinterpret_cast<__half*>(ws + kWsScratch);
    cudaStream_t s = (cudaStream_t)stream;
    rc = launch_hadamard(x, x_dtype, xh_rows, in, x_row_stride, reinterpret_cast<const __half*>(suh),
                         nullptr, xh, row_src, suh_row, nullptr, false, HAD_OUT_F16, s, glu, peers.xh_rows_dev);
    if (rc) return rc;
    GemmArgs a = {};
    a.svh = reinterpret_cast<const __half*>(svh);
    a.bias = nullptr;
    a.y = reinterpret_cast<__half*>(y);
    a.status = reinterpret_cast<int*>(ws + kWsStatus);
    a.y_row_stride = y_row_stride;
    a.tile_tab = tiles;
    a.y_row_map = y_row_map;
    a.n_tiles_tab = (int)n_tiles;
    a.xh_rows = (int)xh_rows;
    a.m = (int)xh_rows;
    a.t_in = (int)t_in;
    a.t_out = (int)t_out_total;
    a.n_peer = peers.n;
    a.rows_per_peer = (int)peers.rows_per_peer;
    a.done_ctr = reinterpret_cast<unsigned*>(ws + kWsDoneCtr);
    bool wide = y_row_stride % 16 == 0 && (peers.n > 0 || aligned(y, 32));
    for (int p = 0; p < peers.n; p++) {
        if (!peers.y[p] || !peers.ctr[p]) return EXL3_E_NULL;
        if (peers.y[p] % 16 || peers.ctr[p] % 4) return EXL3_E_ALIGN;
        wide = wide && peers.y[p] % 32 == 0;
        a.y_peer[p] = reinterpret_cast<__half*>(peers.y[p]);
        a.ctr_peer[p] = reinterpret_cast<unsigned*>(peers.ctr[p]);
    }
    // tile tables place outputs at multiples of 128 columns, so a 32-byte aligned base and row
    // stride make every 16-column piece 32-byte aligned
    a.y_wide = wide ? 1 : 0;
    return launch_gemm(a, k, cb, xh, reinterpret_cast<const uint32_t*>(trellis), s);
}

int exl3_gemm_tiles(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                    const int32_t* row_src, const uint16_t* suh, const int32_t* suh_row,
                    const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k, int cb,
                    const int32_t* tiles, int64_t n_tiles, const uint16_t* svh, uint16_t* y,
                    int64_t y_row_stride, const int32_t* y_row_map, void* workspace, size_t workspace_bytes,
                    unsigned flags, exl3_stream_t stream)
{
    return gemm_tiles_impl(x, x_dtype, x_row_stride, xh_rows, row_src, suh, suh_row, trellis, t_in, t_out_total, k,
                           cb, tiles, n_tiles, svh, y, y_row_stride, y_row_map, workspace, workspace_bytes, flags,
                           stream, TilePeers{});
}

int exl3_gemm_tiles_peers(const void* x, int x_dtype, int64_t x_row_stride, int64_t xh_rows,
                          const int32_t* xh_rows_dev, const int32_t* row_src, const uint16_t* suh,
                          const int32_t* suh_row, const uint16_t* trellis, int64_t t_in, int64_t t_out_total, int k,
                          int cb, const int32_t* tiles, int64_t n_tiles, const uint16_t* svh, uint16_t* y,
                          int64_t y_row_stride, const int32_t* y_row_map, const uint64_t* y_peers,
                          const uint64_t* counter_peers, int n_peers, int64_t rows_per_peer, void* workspace,
                          size_t workspace_bytes, unsigned flags, exl3_stream_t stream)
{
    TilePeers p;
    p.xh_rows_dev = xh_rows_dev;
    p.n = n_peers;
    p.rows_per_peer = rows_per_peer;
    p.y = y_peers;
    p.ctr = counter_peers;
    if (n_peers > 0 && !y) y = reinterpret_cast<uint16_t*>(y_peers ? y_peers[0] : 0);
    return gemm_tiles_impl(x, x_dtype, x_row_stride, xh_rows, row_src, suh, suh_row, trellis, t_in, t_out_total, k,
                           cb, tiles, n_tiles, svh, y, y_row_stride, y_row_map, workspace, workspace_bytes, flags,
                           stream, p);
}

#ifdef EXL3_PROFILE
/* Timeline builds only (python -m ponyexl3_b200.build --profile): hand in a zeroed device buffer of
 * launches x 512 x 128 bytes; the next `launches` exl3_gemv calls each fill one slot with 16 words
 * per CTA (see the end of gemv_kernel). */
EXL3_API void exl3_profile_buffer(void* buf, size_t launches)
{
    g_prof_buf = static_cast<long long*>(buf);
    g_prof_launches = launches;
    g_prof_next = 0;
}
#endif

void exl3_tune_gemv(int max_grid, int fuse_x_bytes)
{
    gemv_set_tuning(max_grid, fuse_x_bytes);
}

void exl3_tune_gemm(int one_acc_rows)
{
    gemm_set_tuning(one_acc_rows);
}

void exl3_tune_gemm_pairs(int on)
{
    gemm_set_pairs(on);
}

}  // extern "C"
