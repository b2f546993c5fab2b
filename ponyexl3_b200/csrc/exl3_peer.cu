// Output exchange of the tensor-parallel path over peer memory (one process per GPU, every
// rank's buffers mapped into every other rank: NVLink / NVSwitch loads and stores).
//
// A rank's kernels write their slice of a row straight into the full-width row buffer of
// EVERY rank and then add one to an arrival counter on every rank (release at system scope).
// Before a rank reads its full row it runs exl3_peer_wait on its own counter: one thread
// polls (acquire at system scope) until the expected number of arrivals is there, subtracts
// them again and ends; the kernels after it in the stream see the complete row.
//
// The poll is bounded: after about a second it gives up, records ST_PEER_TIMEOUT in the
// status word and ends, so a rank whose peer has stopped does not hang its GPU.
// A rank that is ahead may already send the NEXT exchange while a slower rank still reads the
// current one, so the same (buffer, counter) pair must not serve two consecutive exchanges:
// callers rotate over a small ring of pairs.
#include <cuda_fp16.h>

#include "exl3_internal.h"

namespace exl3 {

__global__ void peer_wait_kernel(unsigned* counter, unsigned target, int* status)
{
    griddep_launch_dependents();
    griddep_wait();
    for (unsigned i = 0; i < kPeerPolls; i++) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= target) {
            // re-arm by subtracting, so an arrival that belongs to a later exchange is kept
            asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(counter), "r"(0u - target) : "memory");
            return;
        }
        __nanosleep(200);
    }
    atomicOr(status, ST_PEER_TIMEOUT);
}

struct PeerCopyArgs {
    const __half* src;
    int64_t src_stride, dst_stride, col0;
    int rows, cols, n_peer;
    __half* dst[kMaxPeers];
    unsigned* ctr[kMaxPeers];
};

// One CTA: (rows, cols) from src into columns col0.. of every rank's full row, then one arrival
// on every rank's counter.  cols is a multiple of 8, everything 16-byte aligned.
__global__ void __launch_bounds__(512) peer_allgather_kernel(const PeerCopyArgs a)
{
    griddep_launch_dependents();
    griddep_wait();
    const int per_row = a.cols / 8;
    for (int i = threadIdx.x; i < a.rows * per_row; i += blockDim.x) {
        const int r = i / per_row, c = (i - r * per_row) * 8;
        const uint4 v = *reinterpret_cast<const uint4*>(a.src + (int64_t)r * a.src_stride + c);
        for (int p = 0; p < a.n_peer; p++)
            *reinterpret_cast<uint4*>(a.dst[p] + (int64_t)r * a.dst_stride + a.col0 + c) = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();                   // the CTA's stores (ordered by the barrier), then the arrivals
        for (int p = 0; p < a.n_peer; p++)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(a.ctr[p]) : "memory");
    }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_peer_wait(uint32_t* counter, uint32_t target, void* workspace, unsigned flags,
                              exl3_stream_t stream)
{
    if (!counter || !workspace) return EXL3_E_NULL;
    if (target == 0) return EXL3_E_RANGE;
    // With EXL3_FLAG_PDL the poll is resident while the producing kernel of this rank still runs,
    // and ends the moment the last block (local or remote) has arrived.
    return launch_kernel(peer_wait_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, (flags & EXL3_FLAG_PDL) != 0,
                         reinterpret_cast<unsigned*>(counter), (unsigned)target,
                         reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + kWsStatus));
}

extern "C" int exl3_peer_allgather(const uint16_t* src, int rows, int64_t cols, int64_t src_row_stride,
                                   const uint64_t* dst_peers, const uint64_t* counter_peers, int n_peers,
                                   int64_t dst_row_stride, int64_t col0, unsigned flags, exl3_stream_t stream)
{
    if (!src || !dst_peers || !counter_peers) return EXL3_E_NULL;
    if (n_peers < 1 || n_peers > kMaxPeers) return EXL3_E_RANGE;
    if (rows < 1 || cols < 8 || cols % 8 || col0 < 0 || col0 % 8 || col0 + cols > dst_row_stride)
        return EXL3_E_SHAPE;
    if (src_row_stride % 8 || dst_row_stride % 8 || ((uintptr_t)src & 15)) return EXL3_E_ALIGN;
    PeerCopyArgs a;
    a.src = reinterpret_cast<const __half*>(src);
    a.src_stride = src_row_stride;
    a.dst_stride = dst_row_stride;
    a.col0 = col0;
    a.rows = rows;
    a.cols = (int)cols;
    a.n_peer = n_peers;
    for (int p = 0; p < n_peers; p++) {
        if (!dst_peers[p] || !counter_peers[p]) return EXL3_E_NULL;
        if (dst_peers[p] % 16 || counter_peers[p] % 4) return EXL3_E_ALIGN;
        a.dst[p] = reinterpret_cast<__half*>(dst_peers[p]);
        a.ctr[p] = reinterpret_cast<unsigned*>(counter_peers[p]);
    }
    return launch_kernel(peer_allgather_kernel, dim3(1), dim3(512), 0, (cudaStream_t)stream,
                         (flags & EXL3_FLAG_PDL) != 0, a);
}
