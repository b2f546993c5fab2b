// Trellis encoder: exact Viterbi search of 16x16 tiles over the bitshift trellis, the
// converter's side of the EXL3 format (reference: quantize_tile_reference,
// ponyexl3/convert/reference_search.py:30-87, itself the parity oracle of the reference's
// search kernel).
//
// A tile is 256 weights in codeword order.  The trellis has 65,536 states (the 16-bit windows);
// a step appends K bits, s' = ((s << K) | j) & 0xFFFF, so the predecessors of s' are
// (s' >> K) | (j << (16 - K)), j = 0 .. 2^K - 1.  Path cost = sum of (codebook(s_t) - w[t])^2 in
// float64 with the product and the sum rounded separately, the FIRST minimum winning among
// predecessors and among final states, exactly as the reference's numpy code, so the chosen
// states are bit-identical.  The bitstream is tail-biting (codeword 0's window reaches back into
// codeword 255's): a free pass proposes the closing state, pinned passes start from it until
// the path's pre-state of step 0 and its last state both equal the pin (at most max_pins passes).
//
// One CTA of 1024 threads per tile: a thread owns the bases (s' >> K) i + 1024 m and writes the
// 2^K successor states of each.  The two cost arrays
// (2 x 512 KiB of float64) and the back-pointers (one byte per base and step, in a 16 MiB area) live in
// a workspace slot of the CTA and stay in L2; the cost arrays are read and written with
// cache-global accesses because every step reads what other threads of the CTA wrote in the
// step before.  The only synchronisation is the CTA barrier: nothing waits on another CTA.
#include <cuda_fp16.h>

#include <algorithm>

#include "exl3_bits.cuh"
#include "exl3_device.cuh"
#include "exl3_internal.h"

namespace exl3 {

constexpr int kEncStates = 65536;
constexpr size_t kEncSlotBytes = 2 * (size_t)kEncStates * sizeof(double) + 256 * (size_t)kEncStates;

struct EncodeArgs {
    const float* w;        // (n_tiles, 256) codeword order
    int64_t n_tiles;
    int k, max_pins;
    uint16_t* states;      // (n_tiles, 256) the 16-bit window of every codeword
    uint32_t* packed;      // NULL or (n_tiles, 8K) packed tile words
    uint8_t* slots;        // gridDim.x workspace slots
};

template <int CB>
__global__ void __launch_bounds__(1024) encode_kernel(const EncodeArgs a)
{
    __shared__ float sh_w[256];
    __shared__ uint16_t sh_states[256];
    __shared__ double red_c[32];
    __shared__ int red_s[32];
    __shared__ uint32_t sh_words[64];
    __shared__ int sh_fin, sh_pin, sh_done;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = a.k, kk = 1 << k;
    uint8_t* slot = a.slots + (size_t)blockIdx.x * kEncSlotBytes;
    double* cost0 = reinterpret_cast<double*>(slot);
    double* cost1 = cost0 + kEncStates;
    uint8_t* back = slot + 2 * (size_t)kEncStates * sizeof(double);

    for (int64_t tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
        if (tid < 256) sh_w[tid] = a.w[tile * 256 + tid];
        if (tid == 0) { sh_pin = -1; sh_done = 0; }
        __syncthreads();
        for (int pass = 0; pass <= a.max_pins; pass++) {
            const int pin = sh_pin;
            for (int s = tid; s < kEncStates; s += 1024) __stcg(cost0 + s, (pin < 0 || s == pin) ? 0.0 : 1e30);
            __syncthreads();
            double* cur = cost0;
            double* nxt = cost1;
            for (int t = 0; t < 256; t++) {
                const double wt = (double)sh_w[t];
                uint8_t* bt = back + (size_t)t * kEncStates;
                // The 2^K successors of one base (s' >> K) share their predecessor set, hence its
                // cheapest member: every cost of the step before is read exactly once.
                for (uint32_t base = tid; base < (uint32_t)(kEncStates >> k); base += 1024) {
                    double cb = __ldcg(cur + base);
                    int best = 0;
                    for (int j = 1; j < kk; j++) {
                        const double c = __ldcg(cur + (base | ((uint32_t)j << (16 - k))));
                        if (c < cb) { cb = c; best = j; }
                    }
                    __stcg(bt + base, (uint8_t)best);          // one back-pointer for all 2^K successors
                    for (int low = 0; low < kk; low += 2) {
                        const uint32_t s = (base << k) | (uint32_t)low;
                        const double d0 = (double)__half2float(decode_one<CB>(s)) - wt;
                        const double d1 = (double)__half2float(decode_one<CB>(s + 1)) - wt;
                        __stcg(reinterpret_cast<double2*>(nxt + s),
                               make_double2(__dadd_rn(cb, __dmul_rn(d0, d0)), __dadd_rn(cb, __dmul_rn(d1, d1))));
                    }
                }
                __syncthreads();
                double* tmp = cur; cur = nxt; nxt = tmp;
            }
            // the cheapest final state, the lowest index among equals
            double bc = __ldcg(cur + tid);
            int bs = tid;
            for (int s = tid + 1024; s < kEncStates; s += 1024) {
                const double c = __ldcg(cur + s);
                if (c < bc) { bc = c; bs = s; }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const double oc = __shfl_down_sync(0xFFFFFFFFu, bc, off);
                const int os = __shfl_down_sync(0xFFFFFFFFu, bs, off);
                if (oc < bc || (oc == bc && os < bs)) { bc = oc; bs = os; }
            }
            if (lane == 0) { red_c[warp] = bc; red_s[warp] = bs; }
            __syncthreads();
            if (warp == 0) {
                bc = red_c[lane];
                bs = red_s[lane];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const double oc = __shfl_down_sync(0xFFFFFFFFu, bc, off);
                    const int os = __shfl_down_sync(0xFFFFFFFFu, bs, off);
                    if (oc < bc || (oc == bc && os < bs)) { bc = oc; bs = os; }
                }
                if (lane == 0) sh_fin = bs;
            }
            __syncthreads();
            if (tid == 0) {
                // walk the back-pointers (the stores of this CTA are visible after the barriers)
                uint32_t s = (uint32_t)sh_fin;
                for (int t = 255; t >= 0; t--) {
                    sh_states[t] = (uint16_t)s;
                    const uint32_t j = __ldcg(back + (size_t)t * kEncStates + (s >> k));
                    s = (s >> k) | (j << (16 - k));
                }
                const int last = sh_states[255];
                if (pass > 0 && (int)s == pin && last == pin) sh_done = 1;
                sh_pin = last;
            }
            __syncthreads();
            if (sh_done) break;
        }
        if (tid < 256) a.states[tile * 256 + tid] = sh_states[tid];
        if (a.packed) {
            // the low K bits of every codeword, MSB first in codeword order, as little-endian
            // 32-bit words (ponyexl3/ref/trellis.py:12-50)
            if (tid < 64) sh_words[tid] = 0u;
            __syncthreads();
            if (tid < 256) {
                const uint32_t v = sh_states[tid] & (uint32_t)(kk - 1);
                for (int b = 0; b < k; b++)
                    if ((v >> (k - 1 - b)) & 1u) {
                        const int pos = tid * k + b;
                        atomicOr(&sh_words[pos >> 5], 1u << (31 - (pos & 31)));
                    }
            }
            __syncthreads();
            if (tid < 8 * k) a.packed[tile * 8 * k + tid] = sh_words[tid];
        }
        __syncthreads();
    }
}

}  // namespace exl3

using namespace exl3;

extern "C" size_t exl3_encode_workspace_bytes(int64_t n_tiles)
{
    if (n_tiles < 1) n_tiles = 1;
    int64_t slots = device_sm_count();
    if (slots < 1) slots = 1;
    if (n_tiles < slots) slots = n_tiles;
    return (size_t)slots * kEncSlotBytes;
}

extern "C" int exl3_encode_tiles(const float* w, int64_t n_tiles, int k, int cb, int max_pins, uint16_t* states,
                                 uint16_t* packed, void* workspace, size_t workspace_bytes, exl3_stream_t stream)
{
    if (!w || !states) return EXL3_E_NULL;
    if (k < 1 || k > 8) return EXL3_E_K;
    if (cb < 0 || cb > 2) return EXL3_E_CODEBOOK;
    if (n_tiles < 0 || n_tiles > ((int64_t)1 << 32) || max_pins < 0 || max_pins > 64) return EXL3_E_RANGE;
    if ((reinterpret_cast<uintptr_t>(w) & 3) || (reinterpret_cast<uintptr_t>(states) & 1) ||
        (packed && (reinterpret_cast<uintptr_t>(packed) & 3)))
        return EXL3_E_ALIGN;
    if (!workspace || workspace_bytes < kEncSlotBytes) return EXL3_E_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 255) return EXL3_E_ALIGN;
    if (n_tiles == 0) return EXL3_OK;
    int64_t slots = (int64_t)(workspace_bytes / kEncSlotBytes);
    slots = std::min<int64_t>(slots, std::min<int64_t>(n_tiles, 4 * (int64_t)device_sm_count()));
    EncodeArgs a;
    a.w = w;
    a.n_tiles = n_tiles;
    a.k = k;
    a.max_pins = max_pins;
    a.states = states;
    a.packed = reinterpret_cast<uint32_t*>(packed);
    a.slots = static_cast<uint8_t*>(workspace);
    cudaStream_t s = (cudaStream_t)stream;
    switch (cb) {
        case CB_3INST: encode_kernel<CB_3INST><<<(unsigned)slots, 1024, 0, s>>>(a); break;
        case CB_MCG: encode_kernel<CB_MCG><<<(unsigned)slots, 1024, 0, s>>>(a); break;
        default: encode_kernel<CB_MUL1><<<(unsigned)slots, 1024, 0, s>>>(a); break;
    }
    return check_launch();
}
