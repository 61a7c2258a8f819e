// Persistent, warp-specialised weight-streaming GEMV for sm_100a.
//
// One CTA per SM walks a contiguous range of (panel, unit) blocks of the packed weight
// (qgemv_layout.h).  Warp roles:
//   warps 0..7   consumers: each owns two of the sixteen 64-wide K units of the current
//                1024-wide K phase, for every panel of the current item, so the activation
//                fragments are loaded once per phase and reused across panels; weights are
//                converted E2M1/E4M3 -> f16 in registers (hardware cvt), multiplied by their
//                block scales in f16x2 (exact) and fed to mma.m16n8k16 with fp32 accumulators.
//   warp  8      producer: one thread streams weight blocks with bulk (TMA) copies through a
//                ring of shared-memory stages guarded by mbarriers.
//   warps 9..11  converters: turn the bf16 activations of the next phase into f16 MMA
//                fragments, scaled per batch row by a power of two so the row maximum lands in
//                [2^14, 2^15): the scaling is exact, and undone in fp32 when a phase ends.
// The K split between CTAs and warps depends only on (N, K, CTA count), never on the batch or
// on timing; partial panels are written to per-CTA workspace slots and summed in a fixed order
// by whichever CTA arrives last.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qgemv.h"
#include "ptx.cuh"
#include "qgemv_layout.h"

namespace qg {

constexpr int kConsumerWarps = 8;
constexpr int kProducerWarp = 8;
constexpr int kFirstConverterWarp = 9;
constexpr int kConverterWarps = 3;
constexpr int kThreads = 32 * (kConsumerWarps + 1 + kConverterWarps);  // 384
constexpr int kPMax = 8;        // panels per item (accumulators held in registers)
constexpr int kXBufBytes = QG_PHASE_UNITS * 1024;  // f16 fragments of one phase, 8 columns
constexpr int kRedBytes = 2 * kConsumerWarps * 512;
constexpr int kProbInts = 20;   // expert, nrows, xrow[8], orow[8], pad[2]

template <int FMT>
struct FmtTraits;
template <>
struct FmtTraits<QGEMV_FMT_NVFP4> {
    static constexpr int kUnitBytes = QG_NVFP4_UNIT_BYTES;
    static constexpr int kStages = 7;
};
template <>
struct FmtTraits<QGEMV_FMT_FP8> {
    static constexpr int kUnitBytes = QG_FP8_UNIT_BYTES;
    static constexpr int kStages = 4;
};

struct GemvParams {
    const uint8_t* payload;     // payload of stacked weight 0
    uint64_t stack_stride;      // bytes between stacked weights
    const float* chan_scale;    // FP8: fp32 [n_panels*16] of stacked weight 0
    uint64_t chan_stride;       // bytes between stacked channel-scale arrays
    const float* tensor_scale;  // device fp32 [n_stack]
    const uint16_t* x;          // bf16 activations
    void* y;
    float* ws;                  // partial slots: [2 * grid][32 lanes] float4
    int32_t* counters;          // one per virtual panel, zero between launches
    int32_t* status;            // qgemv_dev_status
    const int32_t* prob;        // [0] = problem count, then kProbInts ints per problem; or null
    int64_t spin_limit;
    int32_t N, K;
    int32_t n_panels, units;
    int32_t B;                  // dense batch (prob == null)
    int32_t y_dtype;
    int32_t debug;
    uint64_t payload_bytes;     // per stacked weight, for debug bounds checks
};

struct Smem {
    // offsets from the 128-byte aligned dynamic shared memory base
    static constexpr int kBarFull = 0;                  // kStages * 8
    static constexpr int kBarEmpty = 64;                // kStages * 8
    static constexpr int kBarXFull = 128;               // 2 * 8
    static constexpr int kBarXEmpty = 144;              // 2 * 8
    static constexpr int kXExp = 160;                   // 2 * 8 ints
    static constexpr int kAbort = 224;                  // int
    static constexpr int kXBuf = 256;                   // 2 * kXBufBytes
    static constexpr int kRed = kXBuf + 2 * kXBufBytes; // kRedBytes
    static constexpr int kStage0 = kRed + kRedBytes;
    template <int FMT>
    static constexpr int total() {
        return kStage0 + FmtTraits<FMT>::kStages * QG_PHASE_UNITS * FmtTraits<FMT>::kUnitBytes;
    }
};

__device__ __forceinline__ void report(int32_t* status, int code, int where, int extra) {
    if (atomicCAS(status, 0, code) == 0) {
        status[1] = where;
        status[2] = (int)blockIdx.x;
        status[3] = extra;
    }
}

// ---- work decomposition --------------------------------------------------------------------
// The linear work space is (virtual panel, unit), virtual panel = problem * n_panels + panel.
// CTA c owns [c*total/G, (c+1)*total/G).  Its range is cut into items: a partial panel (one
// panel, part of K) or up to kPMax whole panels of one problem.
struct Item {
    int64_t vp;       // first virtual panel
    int32_t np;       // panels
    int32_t u0, u1;   // unit range
    int32_t partial;  // 1: contributes a partial sum
    int64_t start;    // linear position of the item's first block
};

struct ItemWalker {
    int64_t pos, end, total;
    int32_t units, n_panels;
    __device__ __forceinline__ void init(int64_t total_, int32_t units_, int32_t n_panels_, int cta,
                                         int grid) {
        total = total_;
        units = units_;
        n_panels = n_panels_;
        pos = (int64_t(cta) * total) / grid;
        end = (int64_t(cta + 1) * total) / grid;
    }
    __device__ __forceinline__ bool next(Item& it) {
        if (pos >= end) return false;
        it.start = pos;
        it.vp = pos / units;
        it.u0 = int32_t(pos - it.vp * units);
        const int64_t left = end - pos;
        if (it.u0 != 0 || left < units) {
            it.np = 1;
            const int64_t u1 = it.u0 + left;
            it.u1 = u1 < units ? int32_t(u1) : units;
            it.partial = 1;
            pos += it.u1 - it.u0;
        } else {
            int64_t np = left / units;
            const int64_t in_problem = n_panels - (it.vp % n_panels);
            if (np > in_problem) np = in_problem;
            if (np > kPMax) np = kPMax;
            it.np = int32_t(np);
            it.u1 = units;
            it.partial = 0;
            pos += np * units;
        }
        return true;
    }
};

__device__ __forceinline__ int64_t cta_of(int64_t idx, int64_t total, int grid) {
    return ((idx + 1) * grid - 1) / total;
}
// Workspace slot of the part of a split panel that CTA `c` computes.
__device__ __forceinline__ int64_t part_slot(int64_t c, int64_t vp, int32_t units, int64_t total,
                                             int grid) {
    const int64_t a = (c * total) / grid;
    const int64_t ov = a > vp * units ? a : vp * units;
    return 2 * c + (ov == a ? 0 : 1);
}

// ---- weight tile consumption -------------------------------------------------------------------
template <int FMT>
__device__ __forceinline__ void consume_unit(float (&c)[4], uint32_t unit, int lane,
                                             const uint32_t (&bf)[8]);

template <>
__device__ __forceinline__ void consume_unit<QGEMV_FMT_NVFP4>(float (&c)[4], uint32_t unit, int lane,
                                                              const uint32_t (&bf)[8]) {
    const uint4 cw = lds128(unit + lane * 16);
    const uint2 sw = lds64(unit + 512 + (lane >> 2) * 8);
    uint32_t sg0, sg1, sh0, sh1;
    cvt_e4m3x4(sw.x, sg0, sg1);  // row g:     (blk0,blk1), (blk2,blk3)
    cvt_e4m3x4(sw.y, sh0, sh1);  // row g + 8
    uint32_t a0, a1, a2, a3;
    cvt_e2m1x8(cw.x, a0, a1, a2, a3);
    mma_16816(c, hmul2(a0, sg0), hmul2(a1, sh0), hmul2(a2, sg0), hmul2(a3, sh0), bf[0], bf[1]);
    cvt_e2m1x8(cw.y, a0, a1, a2, a3);
    mma_16816(c, hmul2(a0, sg0), hmul2(a1, sh0), hmul2(a2, sg0), hmul2(a3, sh0), bf[2], bf[3]);
    cvt_e2m1x8(cw.z, a0, a1, a2, a3);
    mma_16816(c, hmul2(a0, sg1), hmul2(a1, sh1), hmul2(a2, sg1), hmul2(a3, sh1), bf[4], bf[5]);
    cvt_e2m1x8(cw.w, a0, a1, a2, a3);
    mma_16816(c, hmul2(a0, sg1), hmul2(a1, sh1), hmul2(a2, sg1), hmul2(a3, sh1), bf[6], bf[7]);
}

template <>
__device__ __forceinline__ void consume_unit<QGEMV_FMT_FP8>(float (&c)[4], uint32_t unit, int lane,
                                                            const uint32_t (&bf)[8]) {
    const uint4 v0 = lds128(unit + lane * 16);        // tiles 0, 1
    const uint4 v1 = lds128(unit + 512 + lane * 16);  // tiles 2, 3
    uint32_t a0, a1, a2, a3;
    cvt_e4m3x4(v0.x, a0, a1);
    cvt_e4m3x4(v0.y, a2, a3);
    mma_16816(c, a0, a1, a2, a3, bf[0], bf[1]);
    cvt_e4m3x4(v0.z, a0, a1);
    cvt_e4m3x4(v0.w, a2, a3);
    mma_16816(c, a0, a1, a2, a3, bf[2], bf[3]);
    cvt_e4m3x4(v1.x, a0, a1);
    cvt_e4m3x4(v1.y, a2, a3);
    mma_16816(c, a0, a1, a2, a3, bf[4], bf[5]);
    cvt_e4m3x4(v1.z, a0, a1);
    cvt_e4m3x4(v1.w, a2, a3);
    mma_16816(c, a0, a1, a2, a3, bf[6], bf[7]);
}

__device__ __forceinline__ float pow2i(int e) {  // 2^e for e in [-126, 127]
    e = e < -126 ? -126 : (e > 127 ? 127 : e);
    return __int_as_float((e + 127) << 23);
}

// Final store of one panel's 16 x 8 results held as one float4 per lane
// (v.x: row g col 2t, v.y: row g col 2t+1, v.z: row g+8 col 2t, v.w: row g+8 col 2t+1).
template <int FMT>
__device__ __forceinline__ void store_panel(const GemvParams& P, float4 v, int lane, int32_t panel,
                                            int nrows, const int32_t* pr, const float* chan) {
    const int g = lane >> 2, t = lane & 3;
    const int n0 = panel * 16 + g, n1 = n0 + 8;
    if (FMT == QGEMV_FMT_FP8) {
        const float s0 = chan[n0], s1 = chan[n1];  // padded to 16 rows per panel
        v.x *= s0, v.y *= s0, v.z *= s1, v.w *= s1;
    }
    const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int col = 2 * t + (i & 1);
        const int n = (i & 2) ? n1 : n0;
        if (col < nrows && n < P.N) {
            const int64_t idx = int64_t(pr ? __ldcg(pr + 10 + col) : col) * P.N + n;
            if (P.y_dtype == QGEMV_OUT_F32) {
                static_cast<float*>(P.y)[idx] = vals[i];
            } else {
                static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(vals[i]);
            }
        }
    }
}

template <int FMT>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const GemvParams P) {
    using Tr = FmtTraits<FMT>;
    constexpr int kUnitBytes = Tr::kUnitBytes;
    constexpr int kStages = Tr::kStages;
    constexpr int kStageBytes = QG_PHASE_UNITS * kUnitBytes;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const bool dense = (P.prob == nullptr);

    // ---- set-up -------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(sbase + Smem::kBarFull + 8 * s, 1);
            mbar_init(sbase + Smem::kBarEmpty + 8 * s, kConsumerWarps);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(sbase + Smem::kBarXFull + 8 * b, kConverterWarps);
            mbar_init(sbase + Smem::kBarXEmpty + 8 * b, kConsumerWarps);
        }
        *reinterpret_cast<volatile int*>(smem_raw + Smem::kAbort) = 0;
        mbar_fence_init();
    }
    // zero both activation fragment buffers: columns >= B are never written afterwards
    for (int i = threadIdx.x; i < 2 * kXBufBytes / 16; i += kThreads)
        sts128(sbase + Smem::kXBuf + 16 * i, make_uint4(0, 0, 0, 0));
    __syncthreads();
    pdl_launch_dependents();

    // problem count: 1 for a dense GEMV, read from the router prep output for MoE
    int nprob = 1;
    if (!dense) {
        pdl_wait();  // the problem table is produced by the preceding kernel
        nprob = __ldcg(P.prob);
    }
    const int64_t total = int64_t(nprob) * P.n_panels * P.units;
    // every participating CTA owns at least one block, so the parts of a split panel are
    // exactly the CTAs between the owners of its first and last block
    const int grid = total < int64_t(gridDim.x) ? int(total) : int(gridDim.x);
    if (cta >= grid) return;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + Smem::kAbort);

    if (warp == kProducerWarp) {
        // ================= producer: stream weight blocks =================
        // debug bit 1 is a host-set fault injection: the producer issues no copy at all, so the
        // consumers' first wait must run out and report instead of hanging
        if (lane == 0 && !(P.debug & 2)) {
            const uint64_t pol = policy_evict_first();
            ItemWalker wk;
            wk.init(total, P.units, P.n_panels, cta, grid);
            Item it;
            uint32_t cnt = 0;
            bool ok = true;
            while (ok && wk.next(it)) {
                const int f0 = it.u0 / QG_PHASE_UNITS, f1 = (it.u1 - 1) / QG_PHASE_UNITS;
                for (int f = f0; ok && f <= f1; ++f) {
                    const int ua = max(it.u0, f * QG_PHASE_UNITS);
                    const int ub = min(it.u1, (f + 1) * QG_PHASE_UNITS);
                    const uint32_t bytes = uint32_t(ub - ua) * kUnitBytes;
                    for (int pl = 0; pl < it.np; ++pl) {
                        const int s = cnt % kStages;
                        const uint32_t use = cnt / kStages;
                        if (use > 0 &&
                            !mbar_wait(sbase + Smem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                            report(P.status, QGEMV_ERR_TIMEOUT, 1, int(cnt));
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        const int64_t vp = it.vp + pl;
                        const int64_t prob = vp / P.n_panels;
                        const int64_t panel = vp - prob * P.n_panels;
                        const int expert = dense ? 0 : __ldcg(P.prob + 1 + prob * kProbInts);
                        const uint64_t off = (uint64_t(panel) * P.units + ua) * kUnitBytes;
                        if ((P.debug & 1) && off + bytes > P.payload_bytes) {
                            report(P.status, QGEMV_ERR_BOUNDS, 2, int(cnt));
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        const uint8_t* src = P.payload + uint64_t(expert) * P.stack_stride + off;
                        const uint32_t bar = sbase + Smem::kBarFull + 8 * s;
                        mbar_arrive_expect_tx(bar, bytes);
                        bulk_g2s(sbase + Smem::kStage0 + s * kStageBytes, src, bytes, bar, pol);
                        ++cnt;
                    }
                }
            }
            // never leave with copies in flight: wait (bounded) for the last use of every stage
            const uint32_t first = cnt > uint32_t(kStages) ? cnt - kStages : 0;
            for (uint32_t i = first; i < cnt; ++i)
                (void)mbar_wait(sbase + Smem::kBarFull + 8 * (i % kStages), (i / kStages) & 1,
                                int64_t(1) << 26);
        }
    } else if (warp >= kFirstConverterWarp) {
        // ================= converters: bf16 activations -> scaled f16 fragments =================
        const int role = warp - kFirstConverterWarp;
        pdl_wait();  // activations come from the preceding kernel
        ItemWalker wk;
        wk.init(total, P.units, P.n_panels, cta, grid);
        Item it;
        uint32_t xcnt = 0;
        bool ok = true;
        while (ok && wk.next(it)) {
            const int64_t prob = it.vp / P.n_panels;
            const int32_t* pr = dense ? nullptr : P.prob + 1 + prob * kProbInts;
            const int nrows = dense ? P.B : __ldcg(pr + 1);
            const int f0 = it.u0 / QG_PHASE_UNITS, f1 = (it.u1 - 1) / QG_PHASE_UNITS;
            for (int f = f0; ok && f <= f1; ++f) {
                const int ua = max(it.u0, f * QG_PHASE_UNITS);
                const int ub = min(it.u1, (f + 1) * QG_PHASE_UNITS);
                const int xb = xcnt & 1;
                const uint32_t use = xcnt >> 1;
                if (use > 0 && !mbar_wait(sbase + Smem::kBarXEmpty + 8 * xb, (use - 1) & 1, P.spin_limit)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 3, int(xcnt));
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint32_t xbuf = sbase + Smem::kXBuf + xb * kXBufBytes;
                int* xexp = reinterpret_cast<int*>(smem_raw + Smem::kXExp) + xb * 8;
                for (int b = role; b < 8; b += kConverterWarps) {
                    if (b >= nrows) {
                        if (lane == 0) xexp[b] = 0;
                        continue;
                    }
                    const int64_t row = dense ? b : __ldcg(pr + 2 + b);
                    const uint16_t* xr = P.x + row * int64_t(P.K);
                    uint2 va[4], vb[4];
                    uint32_t m = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i = lane + 32 * j;
                        const int q = i >> 3, pp = (i >> 2) & 1, t = i & 3;
                        const int u = f * QG_PHASE_UNITS + q;
                        const int k = u * 64 + pp * 32 + 4 * t;
                        va[j] = make_uint2(0, 0);
                        vb[j] = make_uint2(0, 0);
                        if (u >= ua && u < ub) {
                            if (k < P.K) va[j] = __ldcg(reinterpret_cast<const uint2*>(xr + k));
                            if (k + 16 < P.K) vb[j] = __ldcg(reinterpret_cast<const uint2*>(xr + k + 16));
                        }
                        // |bf16| bit patterns order like magnitudes; a pair lives in one 32-bit word
                        const uint32_t w[4] = {va[j].x, va[j].y, vb[j].x, vb[j].y};
#pragma unroll
                        for (int z = 0; z < 4; ++z) {
                            m = max(m, w[z] & 0x7FFFu);
                            m = max(m, (w[z] >> 16) & 0x7FFFu);
                        }
                    }
                    m = __reduce_max_sync(0xFFFFFFFFu, m);
                    // exponent E with row max * 2^-E in [2^14, 2^15)
                    int E = 0;
                    if (m != 0) {
                        const int ef = int(m >> 7);
                        E = (ef == 0 ? -126 : ef - 127) - 14;
                        E = E < -100 ? -100 : (E > 113 ? 113 : E);
                    }
                    const float sf = pow2i(-E);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int i = lane + 32 * j;
                        const int q = i >> 3, pp = (i >> 2) & 1, t = i & 3;
                        const int u = f * QG_PHASE_UNITS + q;
                        if (u >= ua && u < ub) {
                            const float a0 = __uint_as_float(va[j].x << 16) * sf;
                            const float a1 = __uint_as_float(va[j].x & 0xFFFF0000u) * sf;
                            const float a2 = __uint_as_float(va[j].y << 16) * sf;
                            const float a3 = __uint_as_float(va[j].y & 0xFFFF0000u) * sf;
                            const float b0 = __uint_as_float(vb[j].x << 16) * sf;
                            const float b1 = __uint_as_float(vb[j].x & 0xFFFF0000u) * sf;
                            const float b2 = __uint_as_float(vb[j].y << 16) * sf;
                            const float b3 = __uint_as_float(vb[j].y & 0xFFFF0000u) * sf;
                            uint4 o;
                            o.x = pack_f16x2(a0, b0);
                            o.y = pack_f16x2(a1, b1);
                            o.z = pack_f16x2(a2, b2);
                            o.w = pack_f16x2(a3, b3);
                            sts128(xbuf + q * 1024 + pp * 512 + (4 * b + t) * 16, o);
                        }
                    }
                    if (lane == 0) xexp[b] = E;
                }
                __threadfence_block();
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + Smem::kBarXFull + 8 * xb);
                ++xcnt;
            }
        }
    } else {
        // ================= consumers =================
        const int w = warp;
        const int g = lane >> 2, t = lane & 3;
        pdl_wait();  // outputs and workspace may still be in use by the preceding kernel
        ItemWalker wk;
        wk.init(total, P.units, P.n_panels, cta, grid);
        Item it;
        uint32_t cnt = 0, xcnt = 0;
        bool ok = true;
        const int* xexp_base = reinterpret_cast<const int*>(smem_raw + Smem::kXExp);
        while (ok && wk.next(it)) {
            float c[kPMax][4];
#pragma unroll
            for (int p = 0; p < kPMax; ++p) c[p][0] = c[p][1] = c[p][2] = c[p][3] = 0.f;
            int e0 = 0, e1 = 0;
            const int f0 = it.u0 / QG_PHASE_UNITS, f1 = (it.u1 - 1) / QG_PHASE_UNITS;
            for (int f = f0; ok && f <= f1; ++f) {
                const int ua = max(it.u0, f * QG_PHASE_UNITS);
                const int ub = min(it.u1, (f + 1) * QG_PHASE_UNITS);
                const int xb = xcnt & 1;
                if (!mbar_wait(sbase + Smem::kBarXFull + 8 * xb, (xcnt >> 1) & 1, P.spin_limit)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 4, int(xcnt));
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                // activation fragments of this warp's two units
                const uint32_t xbuf = sbase + Smem::kXBuf + xb * kXBufBytes;
                const int ua_q = 2 * w, ub_q = 2 * w + 1;
                const int uA = f * QG_PHASE_UNITS + ua_q, uB = f * QG_PHASE_UNITS + ub_q;
                const bool haveA = uA >= ua && uA < ub, haveB = uB >= ua && uB < ub;
                uint32_t bfA[8], bfB[8];
                {
                    const uint4 x0 = lds128(xbuf + ua_q * 1024 + lane * 16);
                    const uint4 x1 = lds128(xbuf + ua_q * 1024 + 512 + lane * 16);
                    const uint4 x2 = lds128(xbuf + ub_q * 1024 + lane * 16);
                    const uint4 x3 = lds128(xbuf + ub_q * 1024 + 512 + lane * 16);
                    bfA[0] = x0.x, bfA[1] = x0.y, bfA[2] = x0.z, bfA[3] = x0.w;
                    bfA[4] = x1.x, bfA[5] = x1.y, bfA[6] = x1.z, bfA[7] = x1.w;
                    bfB[0] = x2.x, bfB[1] = x2.y, bfB[2] = x2.z, bfB[3] = x2.w;
                    bfB[4] = x3.x, bfB[5] = x3.y, bfB[6] = x3.z, bfB[7] = x3.w;
                }
                const int n0 = xexp_base[xb * 8 + 2 * t], n1 = xexp_base[xb * 8 + 2 * t + 1];
                if (f != f0) {
                    const int d0 = e0 - n0, d1 = e1 - n1;
                    if (__any_sync(0xFFFFFFFFu, (d0 | d1) != 0)) {
                        const float s0 = pow2i(d0), s1 = pow2i(d1);
#pragma unroll
                        for (int p = 0; p < kPMax; ++p) {
                            c[p][0] *= s0, c[p][2] *= s0;
                            c[p][1] *= s1, c[p][3] *= s1;
                        }
                    }
                }
                e0 = n0, e1 = n1;
#pragma unroll
                for (int pl = 0; pl < kPMax; ++pl) {
                    if (pl < it.np && ok) {
                        const int s = cnt % kStages;
                        if (!mbar_wait(sbase + Smem::kBarFull + 8 * s, (cnt / kStages) & 1, P.spin_limit)) {
                            if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 5, int(cnt));
                            *abort_flag = 1;
                            ok = false;
                        } else {
                            const uint32_t st = sbase + Smem::kStage0 + s * kStageBytes;
                            if (haveA) consume_unit<FMT>(c[pl], st + (uA - ua) * kUnitBytes, lane, bfA);
                            if (haveB) consume_unit<FMT>(c[pl], st + (uB - ua) * kUnitBytes, lane, bfB);
                            __syncwarp();
                            if (lane == 0) mbar_arrive(sbase + Smem::kBarEmpty + 8 * s);
                            ++cnt;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + Smem::kBarXEmpty + 8 * xb);
                ++xcnt;
            }
            // a consumer that gave up must not enter the named barriers of the flush; every
            // consumer sees the same abort flag only eventually, so the flush is skipped by
            // all of them through the shared flag checked after one barrier
            named_bar_sync(1, 32 * kConsumerWarps);
            if (*abort_flag) break;

            // ---- flush: reduce the eight K slices of each panel, then store ----
            const int64_t prob = it.vp / P.n_panels;
            const int32_t panel0 = int32_t(it.vp - prob * P.n_panels);
            const int32_t* pr = dense ? nullptr : P.prob + 1 + prob * kProbInts;
            const int expert = dense ? 0 : __ldcg(pr);
            const int nrows = dense ? P.B : __ldcg(pr + 1);
            const float ts = (FMT == QGEMV_FMT_NVFP4) ? P.tensor_scale[expert] : 1.0f;
            const float* chan = (FMT == QGEMV_FMT_FP8)
                                    ? reinterpret_cast<const float*>(
                                          reinterpret_cast<const uint8_t*>(P.chan_scale) +
                                          uint64_t(expert) * P.chan_stride)
                                    : nullptr;
            const float fs0 = pow2i(e0) * ts, fs1 = pow2i(e1) * ts;
            const uint32_t red = sbase + Smem::kRed;
#pragma unroll
            for (int r = 0; r < kPMax / 2; ++r) {
                if (2 * r < it.np) {  // uniform across the CTA
#pragma unroll
                    for (int pp = 0; pp < 2; ++pp) {
                        const int pl = 2 * r + pp;
                        if (pl < it.np)
                            sts128f(red + (pp * kConsumerWarps + w) * 512 + lane * 16, c[pl][0], c[pl][1],
                                    c[pl][2], c[pl][3]);
                    }
                    named_bar_sync(1, 32 * kConsumerWarps);
                    if (w < 2 && 2 * r + w < it.np) {
                        float4 v = lds128f(red + (w * kConsumerWarps) * 512 + lane * 16);
#pragma unroll
                        for (int ww = 1; ww < kConsumerWarps; ++ww) {
                            const float4 q = lds128f(red + (w * kConsumerWarps + ww) * 512 + lane * 16);
                            v.x += q.x, v.y += q.y, v.z += q.z, v.w += q.w;
                        }
                        v.x *= fs0, v.z *= fs0, v.y *= fs1, v.w *= fs1;
                        const int pl = 2 * r + w;
                        if (!it.partial) {
                            store_panel<FMT>(P, v, lane, panel0 + pl, nrows, pr, chan);
                        } else {
                            // split panel: park the part, last arriver sums all parts in CTA order
                            const int64_t vp = it.vp;
                            const int64_t c_lo = cta_of(vp * P.units, total, grid);
                            const int64_t c_hi = cta_of((vp + 1) * P.units - 1, total, grid);
                            const int nparts = int(c_hi - c_lo + 1);
                            const int64_t slot = part_slot(cta, vp, P.units, total, grid);
                            float4* wsv = reinterpret_cast<float4*>(P.ws);
                            __stcg(wsv + slot * 32 + lane, v);
                            __threadfence();
                            __syncwarp();
                            int old = 0;
                            if (lane == 0) old = atomicAdd(P.counters + vp, 1);
                            old = __shfl_sync(0xFFFFFFFFu, old, 0);
                            if (old == nparts - 1) {
                                __threadfence();
                                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                                for (int64_t cc = c_lo; cc <= c_hi; ++cc) {
                                    const float4 q =
                                        __ldcg(wsv + part_slot(cc, vp, P.units, total, grid) * 32 + lane);
                                    if (cc == c_lo) {
                                        acc = q;
                                    } else {
                                        acc.x += q.x, acc.y += q.y, acc.z += q.z, acc.w += q.w;
                                    }
                                }
                                store_panel<FMT>(P, acc, lane, panel0, nrows, pr, chan);
                                __syncwarp();
                                if (lane == 0) P.counters[vp] = 0;
                            }
                        }
                    }
                    named_bar_sync(1, 32 * kConsumerWarps);
                }
            }
        }
    }
}

}  // namespace qg
