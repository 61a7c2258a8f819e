// Small kernels around the GEMV: the dequantisation parity hook, the MoE router walk that
// builds the grouped-GEMV problem table, and the weighted combine of expert outputs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemv_kernel.cuh"

namespace qg {

__device__ __forceinline__ float h_lo(uint32_t v) { return __half2float(__ushort_as_half(uint16_t(v & 0xFFFFu))); }
__device__ __forceinline__ float h_hi(uint32_t v) { return __half2float(__ushort_as_half(uint16_t(v >> 16))); }

// One warp per (panel, unit): decodes the unit with the conversion instructions of the GEMV and
// writes fp32( f16(code * scale) * tensor_scale ) -- the f16 product is exact.
template <int FMT>
__global__ void dequant_kernel(const uint8_t* payload, const float* chan, float tensor_scale,
                               int32_t N, int32_t K, int32_t units, float* out) {
    constexpr int kUnitBytes = FmtTraits<FMT>::kUnitBytes;
    const int lane = threadIdx.x & 31;
    const int64_t wid = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int64_t panel = wid / units;
    const int u = int(wid - panel * units);
    if (panel * 16 >= N) return;
    const uint8_t* unit = payload + uint64_t(wid) * kUnitBytes;
    const int g = lane >> 2, t = lane & 3;
    uint32_t a[4][4];  // [tile][reg]
    if (FMT == QGEMV_FMT_NVFP4) {
        const uint4 cw = *reinterpret_cast<const uint4*>(unit + lane * 16);
        const uint2 sw = *reinterpret_cast<const uint2*>(unit + 512 + g * 8);
        uint32_t sg[2], sh[2];
        cvt_e4m3x4(sw.x, sg[0], sg[1]);
        cvt_e4m3x4(sw.y, sh[0], sh[1]);
        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int T = 0; T < 4; ++T) {
            cvt_e2m1x8(w[T], a[T][0], a[T][1], a[T][2], a[T][3]);
            a[T][0] = hmul2(a[T][0], sg[T >> 1]);
            a[T][2] = hmul2(a[T][2], sg[T >> 1]);
            a[T][1] = hmul2(a[T][1], sh[T >> 1]);
            a[T][3] = hmul2(a[T][3], sh[T >> 1]);
        }
    } else {
        const uint4 v0 = *reinterpret_cast<const uint4*>(unit + lane * 16);
        const uint4 v1 = *reinterpret_cast<const uint4*>(unit + 512 + lane * 16);
        cvt_e4m3x4(v0.x, a[0][0], a[0][1]);
        cvt_e4m3x4(v0.y, a[0][2], a[0][3]);
        cvt_e4m3x4(v0.z, a[1][0], a[1][1]);
        cvt_e4m3x4(v0.w, a[1][2], a[1][3]);
        cvt_e4m3x4(v1.x, a[2][0], a[2][1]);
        cvt_e4m3x4(v1.y, a[2][2], a[2][3]);
        cvt_e4m3x4(v1.z, a[3][0], a[3][1]);
        cvt_e4m3x4(v1.w, a[3][2], a[3][3]);
    }
#pragma unroll
    for (int T = 0; T < 4; ++T) {
#pragma unroll
        for (int jb = 0; jb < 4; ++jb) {
            const int row = g + 8 * (jb & 1), r = jb >> 1;
            const int pr = T >> 1, sub = T & 1;
            const int e = 4 * t + 2 * sub + r;
            const int64_t n = panel * 16 + row;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t k = int64_t(u) * 64 + (2 * pr + h) * 16 + e;
                if (n < N && k < K) {
                    const float v = h ? h_hi(a[T][jb]) : h_lo(a[T][jb]);
                    const float s = (FMT == QGEMV_FMT_NVFP4) ? tensor_scale : chan[n];
                    out[n * K + k] = __fmul_rn(v, s);
                }
            }
        }
    }
}

// Router walk: groups the (token, slot) pairs of expert_ids [T][topk] by expert, in ascending
// (t, j) order, and cuts each group into problems of at most eight activation rows.
// prob[0] = problem count; problem i = {expert, nrows, xrow[8], orow[8], 0, 0}.
// One CTA: counts by a shared-memory histogram, a warp prefix scan, then one warp walks the list in
// order, so the order inside every problem is the list order and the table is deterministic.
__global__ void moe_prep_kernel(const int32_t* expert_ids, int T, int topk, int n_experts,
                                int per_slot_input, int max_prob, int32_t* prob, int32_t* status) {
    extern __shared__ int sh[];  // ids[T*topk], counts[n_experts], base[n_experts], seen[n_experts], flags[2]
    const int total = T * topk;
    int* ids = sh;
    int* counts = sh + total;
    int* base = counts + n_experts;
    int* seen = base + n_experts;
    int* flags = seen + n_experts;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) flags[0] = 0, flags[1] = 0;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0, seen[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < total; i += blockDim.x) {  // one coalesced read of the router output
        const int e = __ldcg(expert_ids + i);
        ids[i] = e;
        if (e < 0 || e >= n_experts) flags[0] = 1;
    }
    __syncthreads();
    // per-expert entry counts: a shared-memory histogram (order does not matter for a count)
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int e = ids[i];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive prefix of the per-expert problem counts
        int carry = 0;
        for (int e0 = 0; e0 < n_experts; e0 += 32) {
            const int e = e0 + lane;
            const int np = e < n_experts ? (counts[e] + 7) / 8 : 0;
            int incl = np;
            for (int d = 1; d < 32; d <<= 1) {
                const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                if (lane >= d) incl += v;
            }
            if (e < n_experts) base[e] = carry + incl - np;
            carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
        if (lane == 0) {
            int acc = carry;
            if (flags[0]) {
                report(status, QGEMV_ERR_BOUNDS, 21, 0);
                acc = 0;
            } else if (acc > max_prob) {
                report(status, QGEMV_ERR_BOUNDS, 20, acc);
                acc = 0;
            }
            prob[0] = acc;
            flags[1] = acc;
        }
    }
    __syncthreads();
    if (flags[1] == 0) return;
    // Fill the table in list order: one warp walks the list 32 entries at a time; entries of a tile
    // that name the same expert find each other with match_any, their rank in the expert's list is
    // the running count `seen[e]` plus their position among the tile's matches.
    if (warp == 0) {
        for (int i0 = 0; i0 < total; i0 += 32) {
            const int i = i0 + lane;
            const bool valid = i < total;
            const int e = valid ? ids[i] : -1 - lane;  // invalid lanes match nobody
            const unsigned m = __match_any_sync(0xFFFFFFFFu, e);
            int k = 0, cnt = 0;
            if (valid) {
                k = seen[e] + __popc(m & ((1u << lane) - 1u));  // rank of this entry in the expert's list
                cnt = counts[e];
            }
            __syncwarp();
            if (valid) {
                int32_t* p = prob + 1 + (base[e] + (k >> 3)) * kProbInts;
                const int r = k & 7;
                if (r == 0) {
                    p[0] = e;
                    const int left = cnt - k;
                    p[1] = left < 8 ? left : 8;
                    p[18] = p[19] = 0;
                }
                p[2 + r] = per_slot_input ? i : i / topk;
                p[10 + r] = i;
                if (k == cnt - 1) {  // last entry of the expert: clear the unused row slots of its last problem
                    for (int z = r + 1; z < 8; ++z) p[2 + z] = 0, p[10 + z] = 0;
                }
                if ((m & ((1u << lane) - 1u)) == 0) seen[e] += __popc(m);  // the tile's first match updates the count
            }
            __syncwarp();
        }
    }
}

// y[t][n] = sum_j w[t][j] * slot_out[t*topk + j][n], j ascending, fp32.
__global__ void moe_combine_kernel(const void* slot_out, int slot_dtype, const float* w, int T,
                                   int topk, int64_t N, void* y, int y_dtype) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= int64_t(T) * N) return;
    const int64_t t = idx / N, n = idx - t * N;
    float acc = 0.f;
    for (int j = 0; j < topk; ++j) {
        const int64_t src = (t * topk + j) * N + n;
        const float v = slot_dtype == QGEMV_OUT_F32
                            ? static_cast<const float*>(slot_out)[src]
                            : __bfloat162float(static_cast<const __nv_bfloat16*>(slot_out)[src]);
        acc = fmaf(w[t * topk + j], v, acc);
    }
    if (y_dtype == QGEMV_OUT_F32) {
        static_cast<float*>(y)[idx] = acc;
    } else {
        static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(acc);
    }
}

// K-chunked GEMV: y = sum over chunks (in chunk order) of the fp32 partial results, rounded once.
__global__ void chunk_sum_kernel(const float* parts, int n_chunks, int64_t n, void* y, int y_dtype) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = __ldcg(parts + i);
    for (int c = 1; c < n_chunks; ++c) v += __ldcg(parts + int64_t(c) * n + i);
    if (y_dtype == QGEMV_OUT_F32) {
        static_cast<float*>(y)[i] = v;
    } else {
        static_cast<__nv_bfloat16*>(y)[i] = __float2bfloat16_rn(v);
    }
}

// ---- device-side packer of the tensor-core layout ------------------------------------------------
// Canonical NVFP4 (codes u8 [N][K/2], scales u8 [N][K/16], row-major, in device memory) -> the item
// order of QGEMV_FMT_NVFP4_TC, the same bytes qgemv_pack_host writes.  The layout is a permutation of
// 8-byte code groups and single scale bytes, so one thread builds one 16-byte chunk of the payload
// and stores it whole; rows and K blocks beyond the window are zero.
struct PackTcParams {
    const uint8_t* codes;
    const uint8_t* scales;
    uint8_t* payload;
    int64_t N, K;      // the canonical matrix
    int64_t n0, k0;    // origin of the window that is packed
    int64_t n, k;      // its extent
    int64_t tiles, kt; // ceil(n / 128), ceil(k / 64)
};

__global__ void __launch_bounds__(256) pack_tc_kernel(const PackTcParams P) {
    constexpr int kChunks = QG_TC_ITEM_BYTES / 16;  // 288: 256 of codes, 32 of scales
    const int64_t total = P.tiles * P.kt * kChunks;
    for (int64_t c = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; c < total; c += int64_t(gridDim.x) * blockDim.x) {
        const int64_t it = c / kChunks;
        const int within = int(c - it * kChunks);
        const int64_t tile = it / P.kt, item = it - tile * P.kt;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (within < 256) {
            // chunk (r / 8) * 16 + (k / 32) * 8 + r % 8: codes of row r, 32 elements from k
            const int r = (within >> 4) * 8 + (within & 7);
            const int64_t n = tile * QG_TC_TILE_ROWS + r, kk = item * 64 + ((within >> 3) & 1) * 32;
            if (n < P.n) {
                const uint8_t* src = P.codes + (P.n0 + n) * (P.K / 2) + (P.k0 + kk) / 2;
                if (kk < P.k) {
                    const uint2 v = *reinterpret_cast<const uint2*>(src);
                    out.x = v.x, out.y = v.y;
                }
                if (kk + 16 < P.k) {
                    const uint2 v = *reinterpret_cast<const uint2*>(src + 8);
                    out.z = v.x, out.w = v.y;
                }
            }
        } else {
            // chunk r % 32: block scales of rows r % 32 + 32 q, q = 0..3, four K blocks each
            const int r32 = within - 256;
            uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int64_t n = tile * QG_TC_TILE_ROWS + r32 + 32 * q;
                if (n < P.n) {
                    const uint8_t* src = P.scales + (P.n0 + n) * (P.K / 16) + (P.k0 + item * 64) / 16;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb)
                        if (item * 64 + kb * 16 < P.k) w[q] |= uint32_t(src[kb]) << (8 * kb);
                }
            }
            out = make_uint4(w[0], w[1], w[2], w[3]);
        }
        *reinterpret_cast<uint4*>(P.payload + it * QG_TC_ITEM_BYTES + (within < 256 ? within * 16 : 4096 + (within - 256) * 16)) = out;
    }
}

}  // namespace qg
