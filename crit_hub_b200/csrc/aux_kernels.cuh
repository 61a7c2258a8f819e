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
// One CTA, one thread per expert (strided), so the table is deterministic.
__global__ void moe_prep_kernel(const int32_t* expert_ids, int T, int topk, int n_experts,
                                int per_slot_input, int max_prob, int32_t* prob, int32_t* status) {
    extern __shared__ int sh[];  // counts[n_experts], base[n_experts]
    int* counts = sh;
    int* base = sh + n_experts;
    pdl_launch_dependents();
    pdl_wait();
    const int total = T * topk;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        int c = 0;
        for (int i = 0; i < total; ++i) c += (__ldcg(expert_ids + i) == e);
        counts[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < n_experts; ++e) {
            base[e] = acc;
            acc += (counts[e] + 7) / 8;
        }
        if (acc > max_prob) {
            report(status, QGEMV_ERR_BOUNDS, 20, acc);
            acc = 0;
        }
        prob[0] = acc;
        int bad = 0;
        for (int i = 0; i < total; ++i) {
            const int e = __ldcg(expert_ids + i);
            bad |= (e < 0 || e >= n_experts);
        }
        if (bad) {
            report(status, QGEMV_ERR_BOUNDS, 21, 0);
            prob[0] = 0;
        }
    }
    __syncthreads();
    if (prob[0] == 0) return;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        if (counts[e] == 0) continue;
        int seen = 0;
        for (int i = 0; i < total; ++i) {
            if (__ldcg(expert_ids + i) != e) continue;
            int32_t* p = prob + 1 + (base[e] + seen / 8) * kProbInts;
            const int r = seen & 7;
            if (r == 0) {
                p[0] = e;
                const int left = counts[e] - seen;
                p[1] = left < 8 ? left : 8;
                for (int z = 0; z < 8; ++z) p[2 + z] = 0, p[10 + z] = 0;
                p[18] = p[19] = 0;
            }
            p[2 + r] = per_slot_input ? i : i / topk;
            p[10 + r] = i;
            ++seen;
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

}  // namespace qg
