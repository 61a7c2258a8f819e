// Tensor-parallel all-reduce of a short vector (the partial hidden state of a row-parallel
// projection) over NVLink peer memory, without NCCL.
//
// Every rank owns an exchange buffer (cudaMalloc, exported with CUDA IPC) holding, for each of two
// parities, one slot per source rank plus arrival flags.  One launch does:
//   push   every rank stores its fp32 partial into its slot of EVERY rank's buffer (plain
//          peer stores; the data lands in the consumer's local memory before it is consumed),
//   flag   then releases a per-(source, CTA) flag carrying the call's epoch in every buffer,
//   wait   spins -- bounded -- on its OWN local flags until all sources of this epoch arrived,
//   reduce sums the slots in rank order (the same fixed order on every rank: bitwise identical
//          results everywhere) and writes y in place.
// Epochs live in device memory (one counter per CTA), so a captured CUDA graph can be replayed.
// Two parities suffice: a rank can only start call k+2 after every rank contributed to k+1, i.e.
// after every rank finished reading the slots of call k.
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

// layout of one exchange buffer
__host__ __device__ inline size_t tp_flags_offset(int world, int64_t max_elems) {
    return size_t(2) * world * size_t(max_elems) * 4;
}
__host__ __device__ inline size_t tp_buffer_bytes(int world, int64_t max_elems) {
    return tp_flags_offset(world, max_elems) + size_t(2) * kTpMaxWorld * kTpCtas * 4;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(kTpThreads) tp_allreduce_kernel(const TpParams P) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_fail;
    pdl_launch_dependents();
    pdl_wait();  // y is produced by the preceding kernel
    const int cta = blockIdx.x;
    if (threadIdx.x == 0) {
        s_epoch = ++P.epochs[cta];
        s_fail = 0;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int par = int(epoch & 1u);
    // this CTA's slice of the vector, in units of four elements
    const int64_t quads = (P.n + 3) / 4;
    const int64_t q0 = (quads * cta) / kTpCtas, q1 = (quads * (cta + 1)) / kTpCtas;

    // ---- push my partial into my slot of every rank's buffer ----
    for (int64_t q = q0 + threadIdx.x; q < q1; q += kTpThreads) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const int64_t i = 4 * q;
        if (P.y_dtype == QGEMV_OUT_F32) {
            const float* y = static_cast<const float*>(P.y);
            v.x = y[i];
            if (i + 1 < P.n) v.y = y[i + 1];
            if (i + 2 < P.n) v.z = y[i + 2];
            if (i + 3 < P.n) v.w = y[i + 3];
        } else {
            const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(P.y);
            v.x = __bfloat162float(y[i]);
            if (i + 1 < P.n) v.y = __bfloat162float(y[i + 1]);
            if (i + 2 < P.n) v.z = __bfloat162float(y[i + 2]);
            if (i + 3 < P.n) v.w = __bfloat162float(y[i + 3]);
        }
        for (int d = 0; d < P.world; ++d) {
            const int peer = (P.rank + d) % P.world;  // start with myself, spread the link load
            float4* slot = reinterpret_cast<float4*>(P.buf[peer]) +
                           (size_t(par) * P.world + P.rank) * size_t(P.max_elems / 4);
            slot[q] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < P.world) {
        const int peer = threadIdx.x;
        uint32_t* flags = reinterpret_cast<uint32_t*>(P.buf[peer] + tp_flags_offset(P.world, P.max_elems));
        st_release_sys(flags + (size_t(par) * kTpMaxWorld + P.rank) * kTpCtas + cta, epoch);
    }
    // ---- wait (bounded) for every source rank's flag of this epoch in MY buffer ----
    if (threadIdx.x < P.world) {
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(P.buf[P.rank] + tp_flags_offset(P.world, P.max_elems)) +
                               (size_t(par) * kTpMaxWorld + threadIdx.x) * kTpCtas + cta;
        const uint64_t t0 = globaltimer_ns();
        bool ok = false;
        for (int64_t it = 0; it < P.spin_limit; ++it) {
            if (ld_acquire_sys(mine) == epoch) {
                ok = true;
                break;
            }
            if ((it & 255) == 255 && globaltimer_ns() - t0 > 2000000000ull) break;
        }
        if (!ok) {
            s_fail = 1;
            if (atomicCAS(P.status, 0, QGEMV_ERR_TIMEOUT) == 0) {
                P.status[1] = 30;
                P.status[2] = cta;
                P.status[3] = int(threadIdx.x);
            }
        }
    }
    __syncthreads();
    if (s_fail) return;  // a peer never arrived: leave y as it was, the status word says why
    // ---- reduce the slots in rank order, write back ----
    const float4* slots = reinterpret_cast<const float4*>(P.buf[P.rank]) + size_t(par) * P.world * size_t(P.max_elems / 4);
    for (int64_t q = q0 + threadIdx.x; q < q1; q += kTpThreads) {
        float4 acc = __ldcg(slots + q);
        for (int r = 1; r < P.world; ++r) {
            const float4 v = __ldcg(slots + size_t(r) * size_t(P.max_elems / 4) + q);
            acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
        }
        const int64_t i = 4 * q;
        const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
        for (int k = 0; k < 4; ++k) {
            if (i + k < P.n) {
                if (P.y_dtype == QGEMV_OUT_F32) {
                    static_cast<float*>(P.y)[i + k] = vals[k];
                } else {
                    static_cast<__nv_bfloat16*>(P.y)[i + k] = __float2bfloat16_rn(vals[k]);
                }
            }
        }
    }
}

}  // namespace qg
