// Tensor-parallel all-reduce of a short vector (the partial hidden state of a row-parallel
// projection) over NVLink peer memory, without NCCL.
//
// Every rank owns an exchange buffer (cudaMalloc, exported with CUDA IPC) holding, for each of two
// parities, one slot per source rank.  A slot element is an 8-byte pair {fp32 value, epoch}: the
// arrival flag travels in the same store as the data (an aligned 8-byte store is delivered whole),
// so there is no separate fence-then-flag round trip over the link.  One launch does:
//   push   every rank stores its {value, epoch} pairs into its slot of EVERY rank's buffer (plain
//          peer stores; the data lands in the consumer's local memory before it is consumed),
//   wait + reduce   every thread spins -- bounded -- on its own elements of its LOCAL slots until
//          each carries this call's epoch, adds them in rank order (the same fixed order on every
//          rank: bitwise identical results everywhere) and writes y in place.
// Epochs live in device memory (one counter per CTA), so a captured CUDA graph can be replayed.
// Two parities suffice: a rank can only start call k+2 after every rank contributed to k+1, i.e.
// after every rank finished reading the slots of call k.  A slot never holds the epoch being waited
// for from an earlier call (same parity => epoch - 2, - 4, ...).
// No multicast, no loads from peer memory: peers are only written to.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qgemv.h"
#include "ptx.cuh"

namespace qg {

constexpr int kTpMaxWorld = 8;
constexpr int kTpCtas = 8;
constexpr int kTpThreads = 256;

struct TpParams {
    uint8_t* buf[kTpMaxWorld];  // exchange buffer of every rank as mapped in this process
    int32_t rank, world;
    int64_t max_elems;          // slot capacity in fp32 elements
    void* y;                    // local vector, reduced in place
    int32_t y_dtype;
    int64_t n;
    uint32_t* epochs;           // local device counters [kTpCtas]
    int32_t* status;
    int64_t spin_limit;
};

// layout of one exchange buffer: [parity][source rank][max_elems] pairs {value bits, epoch}
__host__ __device__ inline size_t tp_buffer_bytes(int world, int64_t max_elems) {
    return size_t(2) * world * size_t(max_elems) * 8;
}

__device__ __forceinline__ void st_pair_sys(uint2* p, uint32_t a, uint32_t b) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_pair_sys(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kTpThreads) tp_allreduce_kernel(const TpParams P) {
    __shared__ uint32_t s_epoch;
    pdl_launch_dependents();
    pdl_wait();  // y is produced by the preceding kernel
    const int cta = blockIdx.x;
    if (threadIdx.x == 0) s_epoch = ++P.epochs[cta];
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const size_t par_off = size_t(epoch & 1u) * P.world * size_t(P.max_elems);
    // this CTA's slice of the vector
    const int64_t e0 = (P.n * cta) / kTpCtas, e1 = (P.n * (cta + 1)) / kTpCtas;

    // ---- push {value, epoch} into my slot of every rank's buffer ----
    for (int64_t e = e0 + threadIdx.x; e < e1; e += kTpThreads) {
        const float v = P.y_dtype == QGEMV_OUT_F32 ? static_cast<const float*>(P.y)[e]
                                                   : __bfloat162float(static_cast<const __nv_bfloat16*>(P.y)[e]);
        for (int d = 0; d < P.world; ++d) {
            const int peer = (P.rank + d) % P.world;  // start with myself, spread the link load
            uint2* slot = reinterpret_cast<uint2*>(P.buf[peer]) + par_off + size_t(P.rank) * size_t(P.max_elems);
            st_pair_sys(slot + e, __float_as_uint(v), epoch);
        }
    }
    // ---- wait (bounded) for every source's pair of this epoch in MY buffer, add in rank order ----
    const uint2* slots = reinterpret_cast<const uint2*>(P.buf[P.rank]) + par_off;
    const uint64_t t0 = globaltimer_ns();
    for (int64_t e = e0 + threadIdx.x; e < e1; e += kTpThreads) {
        float acc = 0.f;
        for (int r = 0; r < P.world; ++r) {
            const uint2* src = slots + size_t(r) * size_t(P.max_elems) + e;
            uint2 v = ld_pair_sys(src);
            for (int64_t it = 0; v.y != epoch; ++it) {
                if (it >= P.spin_limit || ((it & 255) == 255 && globaltimer_ns() - t0 > 2000000000ull)) {
                    if (atomicCAS(P.status, 0, QGEMV_ERR_TIMEOUT) == 0) {
                        P.status[1] = 30;
                        P.status[2] = cta;
                        P.status[3] = r;
                    }
                    return;  // a peer never arrived: y keeps what it had, the status word says why
                }
                v = ld_pair_sys(src);
            }
            const float x = __uint_as_float(v.x);
            acc = r == 0 ? x : acc + x;
        }
        if (P.y_dtype == QGEMV_OUT_F32) {
            static_cast<float*>(P.y)[e] = acc;
        } else {
            static_cast<__nv_bfloat16*>(P.y)[e] = __float2bfloat16_rn(acc);
        }
    }
}

}  // namespace qg
