// exl3_gemv_noalloc: the 1..16-row linear forward for callers that cannot allocate device
// memory themselves and therefore cannot hand the library a workspace.  Two kinds of
// callers are in that position: plug-in hosts that receive input and output buffers from a
// framework but have no allocator of their own (an inference server's operator slot, a
// language binding that only passes tensors through), and code running where cudaMalloc is
// forbidden or too costly — inside a latency-critical decode loop, or after the process has
// handed all free device memory to a pool it does not control.
//
// The scratch that exl3_gemv takes from the caller's workspace (the status word, the arrival
// counters and partial sums of column blocks split over several CTAs, and the rotated
// activations of the current call) lives here in a file-scope device array of fixed size
// instead.  Every GPU that loads the library holds that array until the process exits.
#include "exl3_internal.h"

namespace exl3 {

// rows x in_features may not exceed this (16 rows of 16,384 features, 8 of 32,768, ...).
constexpr size_t kNoAllocMaxElems = 262144;
// Partial sums of split column blocks: room for 304 CTAs (two per SM of a 152-SM part) at 16 rows.
constexpr size_t kNoAllocPartialBytes = 304 * 16 * kGemvPartialBytesPerCtaRow;
constexpr size_t kNoAllocBytes = kWsScratch + kNoAllocMaxElems * 4 + kNoAllocPartialBytes;   // 5.75 MiB + 2304 B

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// Device address of the array, per device.  In host code the array's name is only a
// stand-in symbol; the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device with that device current.
static void* g_noalloc_ptr[64] = {};

static int noalloc_scratch(void** out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return note_cuda(e);
    if (dev < 0 || dev >= 64) return EXL3_E_UNSUPPORTED;
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return note_cuda(e);
        if (!p) return EXL3_E_CUDA;
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return EXL3_OK;
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_gemv_noalloc(const void* x, int x_dtype, int rows, int64_t x_row_stride,
                                 const uint16_t* trellis, int64_t t_in, int64_t t_out, int k, int cb,
                                 const uint16_t* suh, const uint16_t* svh, const uint16_t* bias,
                                 uint16_t* y, int64_t y_row_stride, unsigned flags,
                                 exl3_stream_t stream)
{
    // Size limit first, with its own code, so the caller can tell "too big for the built-in
    // scratch" from a malformed call.
    if (rows < 1 || rows > 16) return EXL3_E_ROWS;
    if (t_in <= 0 || t_out <= 0) return EXL3_E_SHAPE;
    if ((uint64_t)rows * (uint64_t)t_in * 16u > kNoAllocMaxElems) return EXL3_E_RANGE;
    void* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    // The array keeps whatever the previous call left: the rotated activations and the partial
    // sums are rewritten in full by every call that reads them, the arrival counters start at
    // zero (zero-initialised device memory) and every launch leaves them at zero, and the
    // status word is sticky on purpose (as in a caller-owned workspace), so nothing needs
    // clearing here.
    return exl3_gemv(x, x_dtype, rows, x_row_stride, trellis, t_in, t_out, k, cb, suh, svh, bias, y,
                     y_row_stride, scratch, kNoAllocBytes, flags, stream);
}

// The sticky status word of the built-in scratch (0 = no bounded wait ever gave up), copied to
// *status_out after synchronising the stream; the caller of exl3_gemv_noalloc never sees the
// array and so cannot use exl3_workspace_status.
extern "C" int exl3_gemv_noalloc_status(int* status_out, exl3_stream_t stream)
{
    if (!status_out) return EXL3_E_NULL;
    void* scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    return exl3_workspace_status(scratch, status_out, stream);
}
