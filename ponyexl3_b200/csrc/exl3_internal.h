// Internal C++ interface between the translation units of libexl3b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/exl3_b200.h"
#include "exl3_device.cuh"

namespace exl3 {

// ---- host helpers (exl3_capi.cu) -------------------------------------------------------------
int device_sm_count();              // SM count of the current device (cached per device)
int note_cuda(cudaError_t e);       // records the error text; returns EXL3_OK or EXL3_E_CUDA
int check_launch();                 // note_cuda(cudaGetLastError())

// Launch with or without the programmatic-dependent-launch attribute (EXL3_FLAG_PDL): the kernel
// may then start while its predecessor in the stream drains; it orders itself with griddep_wait.
template <typename... KArgs, typename... Args>
inline int launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl,
                         Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return note_cuda(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
}

// Per-device caches of immutable facts (function attributes, SM count) are arrays of this size;
// a device index beyond it is refused with EXL3_E_UNSUPPORTED.
constexpr int kMaxDevices = 64;

// ---- workspace layout ------------------------------------------------------------------------
// [0, 256)        status word + padding (zero = no bounded wait ever gave up)
// [256, 2304)     arrival counters of the streamed GEMV's split column blocks (one per CTA of the
//                 largest grid); zero between launches: the CTA that completes a count resets it
// [2304, ...)     scratch: the rotated activations xh of the current call — one 32-bit word per
//                 element for the GEMV when the rotation is not fused, fp16 for the GEMM
// after xh        GEMV only: fp32 partial sums of split column blocks, two slots of rows x 128
//                 floats per CTA (exl3_workspace_bytes reserves kGemvMaxGrid CTAs; a smaller
//                 area only shrinks the grid)
constexpr size_t kWsStatus = 0;
constexpr size_t kWsDoneCtr = 64;   // finished-block counter of a launch with peer outputs (inside the status area)
constexpr size_t kWsPassCtr = 68;   // virtual CTAs that got past the wait for a peer-completed input
constexpr unsigned kPeerPolls = 1u << 22;      // x ~250 ns sleep: about a second
constexpr size_t kWsSplitCtr = 256;
constexpr int kGemvMaxGrid = 512;
constexpr size_t kWsScratch = kWsSplitCtr + 4 * (size_t)kGemvMaxGrid;
constexpr size_t kGemvPartialBytesPerCtaRow = 2 * 128 * 4;   // two slots of 128 floats

// ---- launchers -------------------------------------------------------------------------------
int launch_unpack(const uint32_t* trellis, int64_t n_tiles, int k, uint16_t* out, cudaStream_t s);
int launch_decode(const uint32_t* trellis, int64_t t_in, int64_t t_out, int k, int cb, int64_t tn0,
                  int64_t tn_count, __half* w, int64_t ld, cudaStream_t s);
int launch_table(int cb, __half* table, cudaStream_t s);
// Output forms of the rotation kernel: plain fp16, or one 32-bit word per element holding
// (x, 0) / (x, x) for the GEMV's two-slot activation fragments.
enum : int { HAD_OUT_F16 = 0, HAD_OUT_PAIR_X0 = 1, HAD_OUT_PAIR_XX = 2 };
constexpr int kHadamardMmaMinRows = 64;   // from here on the rotation runs on the tensor cores (16-row blocks)
int launch_hadamard(const void* x, int x_dtype, int64_t rows, int64_t n, int64_t x_row_stride,
                    const __half* pre, const __half* post, __half* out, const int32_t* row_src,
                    const int32_t* pre_row, const int32_t* post_row, bool pdl, int out_mode,
                    cudaStream_t s, int glu = 0, const int32_t* rows_dev = nullptr);   // glu: x rows are [gate (n) | up (n)], see glu_value

// One logical 128-column output block of a streamed GEMV: where its weights, activations,
// output scales and results live.  NULL descriptor table = the identity mapping of a plain
// linear layer.
struct ColBlock {
    int32_t phys;      // column-block index inside the trellis (tile column = 8 * phys)
    int32_t xrow;      // first row of xh this block multiplies
    int32_t sv_off;    // element offset into svh / bias (multiple of 128), -1 = none
    int32_t y_off;     // element offset of the block's 128 outputs inside a y row
};

struct GemvArgs {
    const uint32_t* trellis;   // (t_in, t_out_total, 8K) words
    const uint32_t* xh;        // rotated activations, one 32-bit word per element (see HAD_OUT_*)
    const __half* svh;         // may be NULL
    const __half* bias;        // may be NULL
    __half* y;
    const ColBlock* blocks;    // may be NULL
    int* status;
    int64_t y_row_stride;
    int t_in;                  // input tiles (multiple of 8)
    int t_out_total;           // tile columns of the trellis tensor
    int ncb;                   // logical 128-column blocks to compute
    const int32_t* ncb_dev;    // optional: the count lives on the device (at most ncb, which the plan is made for)
    int rows;                  // activation rows per block (1..16)
    int x_rows_total;          // rows of the xh matrix (>= xrow + rows of every block)
    int raw_out;               // 1: write fp16(y_inner) without rotation (MoE gate/up)
    int fast_accum;
    // fused input rotation (few rows): the kernel reads x itself
    const void* x;             // raw activations
    const __half* suh;         // may be NULL
    int64_t x_row_stride;
    int x_dtype;
    int x_fused;               // 1: rotate x in the kernel; 0: xh was written by the rotation kernel
    int x_glu;                 // GLU_*: x rows are [gate (in) | up (in)] and the input is fp16(act(gate) * up)
    const int32_t* row_src;    // fused rotation of a block-table launch: x row of rotated row i (NULL: i)
    const int32_t* suh_row;    // ... and its row of the stacked suh matrix (NULL: row 0)
    // split column blocks: partial sums and arrival counters in the workspace
    float* partials;           // two slots of rows x 128 floats per CTA
    size_t partial_bytes;      // size of that area (bounds the grid)
    unsigned* split_ctr;       // kGemvMaxGrid counters, zero between launches
    long long* prof;           // timeline builds: 8 stamps per CTA of this launch; NULL otherwise
    // filled in by the launcher
    uint32_t sixteen;          // the number 16 as a run-time value (keeps shifts on the multiplier)
    uint32_t cb_xor;           // XOR constant of the 3INST / MCG codebooks, as a run-time value
    int grid_virtual;          // virtual CTAs (halves of real CTAs) the items are dealt to
    int xs_bytes;              // fused rotation: bytes of rotated activations per half
    int n_slots;               // fused rotation: k-block slots of rotated activations per CTA
    int stages;                // depth of the shared-memory ring
    int stage0_off;            // byte offset of the ring inside dynamic shared memory
    // output all-gather over peer memory (tensor parallel by output tile): when n_peer > 0 every
    // finished block is stored into each rank's full-width row buffer and announced on its counter
    int n_peer;
    int64_t y_col0;            // this rank's first column inside the full row
    __half* y_peer[8];         // full-width (rows, y_row_stride) buffers of all ranks, this one included
    unsigned* ctr_peer[8];     // arrival counters of all ranks (one increment per rank and launch)
    unsigned* done_ctr;        // local: finished blocks of this launch (the last one announces the rank)
    // input completed by the other ranks (fused rotation only): wait for wait_target arrivals on
    // wait_ctr before x is read; pass_ctr counts the virtual CTAs that got past (the last re-arms)
    unsigned* wait_ctr;        // NULL: x is ready when the previous kernel of the stream has ended
    unsigned wait_target;
    unsigned* pass_ctr;
};
constexpr int kMaxPeers = 8;

int launch_gemv(const GemvArgs& a, int k, int cb, bool pdl, cudaStream_t s);
// Does the GEMV rotate its activations itself (few rows, short item ranges), or does a rotation
// kernel have to fill xh first?  `table`: the launch goes through a block table.
bool gemv_x_is_fused(int rows, int t_in, int64_t ncb, bool table, size_t partial_bytes);
// Bytes of the partial-sum area that let a launch with `rows` rows use the largest grid.
size_t gemv_partial_bytes(int rows);
// The launch plan of a streamed GEMV: the items (column blocks x k-blocks) are dealt out evenly
// to `grid` CTAs.
struct GemvPlan {
    int grid;       // CTAs (0: the partial-sum area holds not even one)
    int n_slots;    // fused rotation: k-block slots of rotated activations per CTA
    bool x_fused;
};
GemvPlan gemv_plan(int64_t ncb, int nkb, int rows, bool table, size_t partial_bytes);
void gemv_set_tuning(int max_grid, int fuse_x_bytes);
void gemm_set_tuning(int one_acc_rows);                      // benchmark hook, see exl3_b200_tuning.h
void gemm_set_pairs(int on);                                 // benchmark hook, see exl3_b200_tuning.h

// ---- prefill GEMM (exl3_gemm.cuh) ---------------------------------------------------------
struct GemmArgs {
    const __half* svh;        // may be NULL
    const __half* bias;       // may be NULL
    __half* y;
    int* status;
    int64_t y_row_stride;
    const int32_t* tile_tab;  // grouped launches: device table of 8 ints per tile, else NULL
    const int32_t* y_row_map; // grouped launches: output row of every computed row, or NULL (identity)
    int n_tiles_tab;          // slots in tile_tab
    int xh_rows;              // rows of the rotated-activation matrix
    int m;                    // rows (tokens)
    int t_in, t_out;          // tiles
    int tiles_m, tiles_n;
    int n_full_tiles, n_items; // dense: whole tiles, then two half tiles per remaining tile (see gemm_tile)
    int stages;
    int one_acc_rows;         // tiles with at most this many rows use only the first accumulator
    uint32_t cb_xor;
    // grouped launches whose output rows live on several GPUs (expert parallelism): output row r
    // (after y_row_map) is row r % rows_per_peer of y_peer[r / rows_per_peer]; when the whole grid
    // is done, every peer's counter gets one arrival
    int n_peer;
    int rows_per_peer;
    __half* y_peer[kMaxPeers];
    unsigned* ctr_peer[kMaxPeers];
    unsigned* done_ctr;       // local: CTAs that have stored all their tiles
    int y_wide;               // every output row piece is 32-byte aligned: store 32 bytes at a time
};

int launch_gemm(const GemmArgs& a, int k, int cb, const __half* xh, const uint32_t* trellis,
                cudaStream_t s);

}  // namespace exl3
