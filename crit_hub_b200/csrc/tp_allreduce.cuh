// Tensor-parallel exchange of short vectors (the partial hidden state of a row-parallel projection,
// the shards of a column-parallel one) over NVLink peer memory, without NCCL.
//
// Every rank owns an exchange buffer (cudaMalloc, exported with CUDA IPC) holding, for each of two
// parities, one slot per source rank.  A slot element is an 8-byte pair {fp32 value, tag}: the
// arrival flag travels in the same store as the data (an aligned 8-byte store is delivered whole),
// so there is no separate fence-then-flag round trip over the link.  One exchange is:
//   push   every rank stores its {value, tag} pairs into its slot of EVERY rank's buffer (plain
//          peer stores; the data lands in the consumer's local memory before it is consumed),
//   wait   every thread loads the pairs of all source ranks for its element at once, re-polls
//          -- bounded -- only the ones that do not carry this exchange's tag yet,
//   reduce adds them in rank order (the same fixed order on every rank: bitwise identical results
//          everywhere), or, for the all-gather, writes them side by side.
// The tag is a count of exchanges kept in device memory, so a captured CUDA graph can be replayed.
// Two parities suffice: a rank can only start exchange k+2 after every rank contributed to k+1,
// i.e. after every rank finished reading the slots of exchange k.  A slot never holds the tag being
// waited for from an earlier exchange (same parity => tag - 2, - 4, ...).
// No multicast, no loads from peer memory: peers are only written to.
//
// The same slots are used from inside the GEMV-sequence kernel (gemv_seq.cuh), which pushes the
// partial sums of a row-parallel projection straight from the thread that finished adding them up.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qgemv.h"
#include "ptx.cuh"

namespace qg {

constexpr int kTpMaxWorld = 8;
constexpr int kTpThreads = 256;

struct TpParams {
    uint8_t* buf[kTpMaxWorld];  // exchange buffer of every rank as mapped in this process
    int32_t rank, world;
    int64_t max_elems;          // slot capacity in elements
    const void* in;             // all-reduce: the local vector (== y); all-gather: this rank's shard
    void* y;                    // result
    int32_t y_dtype;
    int32_t gather;             // 0: y[e] = sum over ranks; 1: y[r * n + e] = rank r's in[e]
    int64_t n;                  // elements per rank
    uint32_t* epoch;            // [0] exchanges completed by this handle, [1] CTAs of this launch that are through
    int32_t* status;
    int64_t spin_limit;
};

// layout of one exchange buffer: [parity][source rank][max_elems] pairs {value bits, tag}
__host__ __device__ inline size_t tp_buffer_bytes(int world, int64_t max_elems) {
    return size_t(2) * world * size_t(max_elems) * 8;
}

__device__ __forceinline__ void st_pair_sys(unsigned long long* p, uint32_t value, uint32_t tag) {
    const unsigned long long v = (static_cast<unsigned long long>(tag) << 32) | value;
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_pair_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// Pushes `value` for element `elem` of this rank's slot into every rank's buffer (myself first: the
// link load spreads over the peers), then gathers the pairs of all ranks for that element from
// the local buffer.  Returns false when a peer's pair did not arrive within the bounds; `missing`
// then names the first rank that is missing.
struct TpExchange {
    uint8_t* const* buf;
    int rank, world;
    int64_t max_elems;
    size_t par_off;  // pairs before this parity's slots
    uint32_t tag;

    __device__ __forceinline__ void push(int64_t elem, float value) const {
        for (int d = 0; d < world; ++d) {
            const int peer = rank + d < world ? rank + d : rank + d - world;
            unsigned long long* slot = reinterpret_cast<unsigned long long*>(buf[peer]) + par_off + size_t(rank) * size_t(max_elems);
            st_pair_sys(slot + elem, __float_as_uint(value), tag);
        }
    }
    // (not inlined: the GEMV-sequence kernel keeps its code small, and calls this only when ranks exchange)
    __device__ __noinline__ bool gather(int64_t elem, float* out, int64_t spin_limit, int& missing) const {
        const unsigned long long* slots = reinterpret_cast<const unsigned long long*>(buf[rank]) + par_off + elem;
        unsigned long long w[kTpMaxWorld];
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r) w[r] = r < world ? ld_pair_sys(slots + size_t(r) * size_t(max_elems)) : 0ull;
        uint64_t t0 = 0;
        for (int64_t it = 0;; ++it) {
            int first = -1;
#pragma unroll
            for (int r = kTpMaxWorld - 1; r >= 0; --r)
                if (r < world && uint32_t(w[r] >> 32) != tag) first = r;
            if (first < 0) break;
            if (it == 0) t0 = globaltimer_ns();
            if (it >= spin_limit || ((it & 63) == 63 && globaltimer_ns() - t0 > 2000000000ull)) {
                missing = first;
                return false;
            }
#pragma unroll
            for (int r = 0; r < kTpMaxWorld; ++r)
                if (r < world && uint32_t(w[r] >> 32) != tag) w[r] = ld_pair_sys(slots + size_t(r) * size_t(max_elems));
        }
#pragma unroll
        for (int r = 0; r < kTpMaxWorld; ++r)
            if (r < world) out[r] = __uint_as_float(uint32_t(w[r]));
        return true;
    }
};

// One element per thread.  All-reduce: in place on y (fp32 or bf16; the pairs carry fp32).
// All-gather: y[r * n + e] = rank r's in[e].
__global__ void __launch_bounds__(kTpThreads) tp_exchange_kernel(const TpParams P) {
    pdl_launch_dependents();
    pdl_wait();  // the input is produced by the preceding kernel; the exchange count by the preceding exchange
    const uint32_t done = *reinterpret_cast<volatile uint32_t*>(P.epoch);
    TpExchange X;
    X.buf = P.buf, X.rank = P.rank, X.world = P.world, X.max_elems = P.max_elems;
    X.tag = done + 1u;
    X.par_off = size_t(X.tag & 1u) * size_t(P.world) * size_t(P.max_elems);
    const int64_t e = int64_t(blockIdx.x) * kTpThreads + threadIdx.x;
    if (e < P.n) {
        const float v = P.y_dtype == QGEMV_OUT_F32 ? static_cast<const float*>(P.in)[e]
                                                   : __bfloat162float(static_cast<const __nv_bfloat16*>(P.in)[e]);
        X.push(e, v);
        float part[kTpMaxWorld];
        int missing = 0;
        if (!X.gather(e, part, P.spin_limit, missing)) {
            // a peer never arrived: y keeps what it had, the status word says why
            if (atomicCAS(P.status, 0, QGEMV_ERR_TIMEOUT) == 0) {
                P.status[1] = 30;
                P.status[2] = int(blockIdx.x);
                P.status[3] = missing;
            }
        } else if (P.gather) {
            for (int r = 0; r < P.world; ++r) {
                const int64_t idx = int64_t(r) * P.n + e;
                if (P.y_dtype == QGEMV_OUT_F32) {
                    static_cast<float*>(P.y)[idx] = part[r];
                } else {
                    static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(part[r]);
                }
            }
        } else {
            float acc = part[0];
            for (int r = 1; r < P.world; ++r) acc += part[r];
            if (P.y_dtype == QGEMV_OUT_F32) {
                static_cast<float*>(P.y)[e] = acc;
            } else {
                static_cast<__nv_bfloat16*>(P.y)[e] = __float2bfloat16_rn(acc);
            }
        }
    }
    // the last CTA through counts the exchange (also after a time-out: the ranks stay in step)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(P.epoch + 1, 1u) == gridDim.x - 1u) {
            P.epoch[1] = 0u;
            *reinterpret_cast<volatile uint32_t*>(P.epoch) = done + 1u;
        }
    }
}

}  // namespace qg
