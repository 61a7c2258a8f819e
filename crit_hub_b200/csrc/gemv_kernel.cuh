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
//   warps 9..11  converters: turn the bf16 activations of a phase into f16 MMA fragments, scaled
//                per batch row by a power of two so the row maximum lands in [2^14, 2^15): the
//                scaling is exact, and undone in fp32 when a phase ends.
//   warp  9      doubles as epilogue on the resident path: sums the eight K slices of a finished
//                panel in a fixed order and stores it, so consumers never meet a CTA-wide barrier.
// Two schedules share the kernel.  When the f16 fragments of the whole K extent fit their buffer
// (batch * ceil(K / 1024) <= 16) they are converted once by all warps and stay resident; the
// consumers then walk their blocks panel by panel with one accumulator pair.  Otherwise the
// buffer is a ring of phases refilled by the converters and the consumers walk phase by phase
// over up to eight panels held in registers.
// The K split between CTAs and warps depends only on (N, K, CTA count), never on the batch or
// on timing; partial panels are written to per-CTA workspace slots and summed in a fixed order
// by whichever CTA arrives last.
#pragma once
#include <cuda_bf16.h>
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
constexpr int kEpilogueWarp = kFirstConverterWarp;  // resident path: converter 0 turns epilogue
constexpr int kThreads = 32 * (kFirstConverterWarp + kConverterWarps);  // 384
constexpr int kRedSlots = 2;    // reduction slots of the resident path (one panel each)
constexpr int kPMax = 8;        // panels per item (accumulators held in registers)
constexpr int kXBufBytes = 32768;  // f16 activation fragments, QG_PHASE_UNITS * 128 bytes per (phase, row)
constexpr int kXSlotsMax = 16;     // phases resident at once at batch 1
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
    // K-chunked calls (dense, activations too large to stage at once): the launch covers `units`
    // units of every panel starting at `payload`; panels are `unit_stride` units apart and
    // activation rows `x_stride` elements apart
    int32_t unit_stride, x_stride;
    uint64_t payload_bytes;     // per stacked weight, for debug bounds checks
    const uint8_t* pf_base;     // optional: payload of the weight the caller will use next
    uint64_t pf_bytes;          // bytes of it to pull into L2 while this GEMV runs (0 = none)
};

struct Smem {
    // offsets from the 128-byte aligned dynamic shared memory base
    static constexpr int kBarFull = 0;                  // kStages * 8
    static constexpr int kBarEmpty = 64;                // kStages * 8
    static constexpr int kBarXFull = 128;               // kXSlotsMax * 8
    static constexpr int kBarXEmpty = 256;              // kXSlotsMax * 8
    static constexpr int kXExp = 384;                   // kXSlotsMax * 8 ints
    static constexpr int kAbort = 896;                  // int
    static constexpr int kBarRedFull = 904;             // kRedSlots * 8
    static constexpr int kBarRedEmpty = 936;            // kRedSlots * 8
    static constexpr int kXBuf = 1024;                  // kXBufBytes
    static constexpr int kRed = kXBuf + kXBufBytes;     // kRedBytes
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

// Host-side twin of the kernel's schedule choice: the resident path needs every phase of K to
// fit the fragment buffer at this batch.
inline bool use_resident_path(bool dense, int batch, int64_t units) {
    const int64_t n_phases = (units + QG_PHASE_UNITS - 1) / QG_PHASE_UNITS;
    return dense && batch >= 1 && n_phases <= kXSlotsMax / batch;
}

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

// Two units at once into two independent accumulators: all shared-memory loads are issued
// first and the tiles of the two units alternate, so two MMA dependency chains are in flight.
template <int FMT>
__device__ __forceinline__ void consume_two(float (&cA)[4], float (&cB)[4], uint32_t unitA,
                                            uint32_t unitB, int lane, const uint32_t (&bfA)[8],
                                            const uint32_t (&bfB)[8]);

template <>
__device__ __forceinline__ void consume_two<QGEMV_FMT_NVFP4>(float (&cA)[4], float (&cB)[4],
                                                             uint32_t unitA, uint32_t unitB, int lane,
                                                             const uint32_t (&bfA)[8],
                                                             const uint32_t (&bfB)[8]) {
    const uint4 wA = lds128(unitA + lane * 16);
    const uint4 wB = lds128(unitB + lane * 16);
    const uint2 sA = lds64(unitA + 512 + (lane >> 2) * 8);
    const uint2 sB = lds64(unitB + 512 + (lane >> 2) * 8);
    uint32_t gA0, gA1, hA0, hA1, gB0, gB1, hB0, hB1;
    cvt_e4m3x4(sA.x, gA0, gA1);
    cvt_e4m3x4(sA.y, hA0, hA1);
    cvt_e4m3x4(sB.x, gB0, gB1);
    cvt_e4m3x4(sB.y, hB0, hB1);
    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
    cvt_e2m1x8(wA.x, a0, a1, a2, a3);
    cvt_e2m1x8(wB.x, b0, b1, b2, b3);
    mma_16816(cA, hmul2(a0, gA0), hmul2(a1, hA0), hmul2(a2, gA0), hmul2(a3, hA0), bfA[0], bfA[1]);
    mma_16816(cB, hmul2(b0, gB0), hmul2(b1, hB0), hmul2(b2, gB0), hmul2(b3, hB0), bfB[0], bfB[1]);
    cvt_e2m1x8(wA.y, a0, a1, a2, a3);
    cvt_e2m1x8(wB.y, b0, b1, b2, b3);
    mma_16816(cA, hmul2(a0, gA0), hmul2(a1, hA0), hmul2(a2, gA0), hmul2(a3, hA0), bfA[2], bfA[3]);
    mma_16816(cB, hmul2(b0, gB0), hmul2(b1, hB0), hmul2(b2, gB0), hmul2(b3, hB0), bfB[2], bfB[3]);
    cvt_e2m1x8(wA.z, a0, a1, a2, a3);
    cvt_e2m1x8(wB.z, b0, b1, b2, b3);
    mma_16816(cA, hmul2(a0, gA1), hmul2(a1, hA1), hmul2(a2, gA1), hmul2(a3, hA1), bfA[4], bfA[5]);
    mma_16816(cB, hmul2(b0, gB1), hmul2(b1, hB1), hmul2(b2, gB1), hmul2(b3, hB1), bfB[4], bfB[5]);
    cvt_e2m1x8(wA.w, a0, a1, a2, a3);
    cvt_e2m1x8(wB.w, b0, b1, b2, b3);
    mma_16816(cA, hmul2(a0, gA1), hmul2(a1, hA1), hmul2(a2, gA1), hmul2(a3, hA1), bfA[6], bfA[7]);
    mma_16816(cB, hmul2(b0, gB1), hmul2(b1, hB1), hmul2(b2, gB1), hmul2(b3, hB1), bfB[6], bfB[7]);
}

template <>
__device__ __forceinline__ void consume_two<QGEMV_FMT_FP8>(float (&cA)[4], float (&cB)[4],
                                                           uint32_t unitA, uint32_t unitB, int lane,
                                                           const uint32_t (&bfA)[8],
                                                           const uint32_t (&bfB)[8]) {
    const uint4 vA0 = lds128(unitA + lane * 16);
    const uint4 vB0 = lds128(unitB + lane * 16);
    const uint4 vA1 = lds128(unitA + 512 + lane * 16);
    const uint4 vB1 = lds128(unitB + 512 + lane * 16);
    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
    cvt_e4m3x4(vA0.x, a0, a1);
    cvt_e4m3x4(vA0.y, a2, a3);
    cvt_e4m3x4(vB0.x, b0, b1);
    cvt_e4m3x4(vB0.y, b2, b3);
    mma_16816(cA, a0, a1, a2, a3, bfA[0], bfA[1]);
    mma_16816(cB, b0, b1, b2, b3, bfB[0], bfB[1]);
    cvt_e4m3x4(vA0.z, a0, a1);
    cvt_e4m3x4(vA0.w, a2, a3);
    cvt_e4m3x4(vB0.z, b0, b1);
    cvt_e4m3x4(vB0.w, b2, b3);
    mma_16816(cA, a0, a1, a2, a3, bfA[2], bfA[3]);
    mma_16816(cB, b0, b1, b2, b3, bfB[2], bfB[3]);
    cvt_e4m3x4(vA1.x, a0, a1);
    cvt_e4m3x4(vA1.y, a2, a3);
    cvt_e4m3x4(vB1.x, b0, b1);
    cvt_e4m3x4(vB1.y, b2, b3);
    mma_16816(cA, a0, a1, a2, a3, bfA[4], bfA[5]);
    mma_16816(cB, b0, b1, b2, b3, bfB[4], bfB[5]);
    cvt_e4m3x4(vA1.z, a0, a1);
    cvt_e4m3x4(vA1.w, a2, a3);
    cvt_e4m3x4(vB1.z, b0, b1);
    cvt_e4m3x4(vB1.w, b2, b3);
    mma_16816(cA, a0, a1, a2, a3, bfA[6], bfA[7]);
    mma_16816(cB, b0, b1, b2, b3, bfB[6], bfB[7]);
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
            const float val = vals[i];
            if (P.y_dtype == QGEMV_OUT_F32) {
                static_cast<float*>(P.y)[idx] = val;
            } else {
                static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(val);
            }
        }
    }
}

// Activation staging.  One (phase, row) pair = 1024 K elements of one bf16 activation row; a warp
// handles it as 4 x 32 lanes x (8 + 8) bytes: lane i + 32*j reads elements 4t..4t+3 of blocks
// 2pp and 2pp+1 of unit q, with q = i >> 3, pp = (i >> 2) & 1, t = i & 3.
struct RowRegs {
    uint2 va[4], vb[4];
};
// Loads units [ua, ub) of phase f; returns the largest |bf16| bit pattern seen by the warp.
__device__ __forceinline__ uint32_t load_row(RowRegs& r, const uint16_t* xr, int K, int f, int ua, int ub,
                                             int lane) {
    uint32_t m = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        const int q = i >> 3, pp = (i >> 2) & 1, t = i & 3;
        const int u = f * QG_PHASE_UNITS + q;
        const int k = u * 64 + pp * 32 + 4 * t;
        r.va[j] = make_uint2(0, 0);
        r.vb[j] = make_uint2(0, 0);
        if (u >= ua && u < ub) {
            if (k < K) r.va[j] = __ldcg(reinterpret_cast<const uint2*>(xr + k));
            if (k + 16 < K) r.vb[j] = __ldcg(reinterpret_cast<const uint2*>(xr + k + 16));
        }
        // |bf16| bit patterns order like magnitudes; two of them live in one 32-bit word
        const uint32_t w[4] = {r.va[j].x, r.va[j].y, r.vb[j].x, r.vb[j].y};
#pragma unroll
        for (int z = 0; z < 4; ++z) {
            m = max(m, w[z] & 0x7FFFu);
            m = max(m, (w[z] >> 16) & 0x7FFFu);
        }
    }
    return __reduce_max_sync(0xFFFFFFFFu, m);
}
// Exponent E such that max * 2^-E lies in [2^14, 2^15), from the largest |bf16| bit pattern.
__device__ __forceinline__ int row_exponent(uint32_t m) {
    if (m == 0) return 0;
    const int ef = int(m >> 7);
    const int E = (ef == 0 ? -126 : ef - 127) - 14;
    return E < -100 ? -100 : (E > 113 ? 113 : E);
}
// Writes the f16 fragments scaled by 2^-E.  Fragment of (unit q, block pair pp, row b, lane
// column t): 16 bytes at slot + ((q*2 + pp)*Bl + b)*64 + t*16, words 2*sub + r =
// f16x2(x[blk 2pp][4t + 2sub + r], x[blk 2pp+1][4t + 2sub + r]).
__device__ __forceinline__ void store_row(const RowRegs& r, int E, int f, int ua, int ub, uint32_t slot,
                                          int Bl, int b, int lane) {
    const float sf = pow2i(-E);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        const int q = i >> 3, pp = (i >> 2) & 1, t = i & 3;
        const int u = f * QG_PHASE_UNITS + q;
        if (u >= ua && u < ub) {
            uint4 o;
            o.x = pack_f16x2(__uint_as_float(r.va[j].x << 16) * sf, __uint_as_float(r.vb[j].x << 16) * sf);
            o.y = pack_f16x2(__uint_as_float(r.va[j].x & 0xFFFF0000u) * sf,
                             __uint_as_float(r.vb[j].x & 0xFFFF0000u) * sf);
            o.z = pack_f16x2(__uint_as_float(r.va[j].y << 16) * sf, __uint_as_float(r.vb[j].y << 16) * sf);
            o.w = pack_f16x2(__uint_as_float(r.va[j].y & 0xFFFF0000u) * sf,
                             __uint_as_float(r.vb[j].y & 0xFFFF0000u) * sf);
            sts128(slot + ((q * 2 + pp) * Bl + b) * 64 + t * 16, o);
        }
    }
}
// Ring path: one (phase, row) pair with its own exponent.  Returns E.
__device__ __forceinline__ int convert_row(const uint16_t* xr, int K, int f, int ua, int ub,
                                           uint32_t slot, int Bl, int b, int lane) {
    RowRegs r;
    const int E = row_exponent(load_row(r, xr, K, f, ua, ub, lane));
    store_row(r, E, f, ua, ub, slot, Bl, b, lane);
    return E;
}

// Split panel: park this CTA's part in its workspace slot; whichever CTA arrives last sums all
// parts in ascending CTA order (a fixed order, whatever the arrival order) and stores the panel.
template <int FMT>
__device__ __forceinline__ void finish_partial(const GemvParams& P, float4 v, int lane, int64_t vp,
                                               int32_t panel, int cta, int grid, int64_t total,
                                               int nrows, const int32_t* pr, const float* chan) {
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
            const float4 q = __ldcg(wsv + part_slot(cc, vp, P.units, total, grid) * 32 + lane);
            if (cc == c_lo) {
                acc = q;
            } else {
                acc.x += q.x, acc.y += q.y, acc.z += q.z, acc.w += q.w;
            }
        }
        store_panel<FMT>(P, acc, lane, panel, nrows, pr, chan);
        __syncwarp();
        if (lane == 0) P.counters[vp] = 0;
    }
}

template <int FMT, bool RESIDENT>
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
    // Activation fragments: Bl rows are laid out per phase (Bl * 2 KB).  When every phase of K
    // fits the buffer they are converted once and stay resident for all items of the CTA;
    // otherwise the buffer is a ring of phase slots refilled per (item, phase).
    const int Bl = dense ? P.B : 8;
    const int n_phases = (P.units + QG_PHASE_UNITS - 1) / QG_PHASE_UNITS;
    const int n_slots = kXSlotsMax / Bl;
    constexpr bool resident = RESIDENT;  // host guarantees: dense and n_phases <= n_slots
    const uint32_t slot_bytes = uint32_t(Bl) * 2048u;

    // ---- set-up -------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(sbase + Smem::kBarFull + 8 * s, 1);
            mbar_init(sbase + Smem::kBarEmpty + 8 * s, kConsumerWarps);
        }
        for (int b = 0; b < kXSlotsMax; ++b) {
            // resident mode: one arrival per activation row of the phase; ring mode: one per
            // converter warp
            mbar_init(sbase + Smem::kBarXFull + 8 * b, resident ? uint32_t(Bl) : uint32_t(kConverterWarps));
            mbar_init(sbase + Smem::kBarXEmpty + 8 * b, kConsumerWarps);
        }
        for (int b = 0; b < kRedSlots; ++b) {
            mbar_init(sbase + Smem::kBarRedFull + 8 * b, kConsumerWarps);
            mbar_init(sbase + Smem::kBarRedEmpty + 8 * b, 1);
        }
        *reinterpret_cast<volatile int*>(smem_raw + Smem::kAbort) = 0;
        for (int b = 0; b < 8; ++b) reinterpret_cast<volatile unsigned int*>(smem_raw + Smem::kXExp)[64 + b] = 0u;
        mbar_fence_init();
    }
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
    // Resident path: consumers and converters (11 warps) share the (phase, row) pairs.  Each warp
    // loads its (at most two) pairs, the row maxima meet in shared memory, and every pair is
    // written with the exponent of its whole row -- so no rescaling is needed while consuming.
    auto convert_resident = [&](int wid) {
        constexpr int kWarps = kConsumerWarps + kConverterWarps;
        unsigned int* rowmax = reinterpret_cast<unsigned int*>(smem_raw + Smem::kXExp) + 64;  // 8 words
        int* rowexp = reinterpret_cast<int*>(smem_raw + Smem::kXExp);                           // 8 words
        RowRegs r0, r1;
        const int n_pairs = n_phases * Bl;
        const int i0 = wid, i1 = wid + kWarps;
        const int f_0 = i0 / Bl, b_0 = i0 - f_0 * Bl, f_1 = i1 / Bl, b_1 = i1 - f_1 * Bl;
        if (i0 < n_pairs) {
            const uint32_t m = load_row(r0, P.x + int64_t(b_0) * P.K, P.K, f_0, f_0 * QG_PHASE_UNITS,
                                        min(P.units, (f_0 + 1) * QG_PHASE_UNITS), lane);
            if (lane == 0) atomicMax(rowmax + b_0, m);
        }
        if (i1 < n_pairs) {
            const uint32_t m = load_row(r1, P.x + int64_t(b_1) * P.K, P.K, f_1, f_1 * QG_PHASE_UNITS,
                                        min(P.units, (f_1 + 1) * QG_PHASE_UNITS), lane);
            if (lane == 0) atomicMax(rowmax + b_1, m);
        }
        named_bar_sync(2, 32 * kWarps);
        if (i0 < n_pairs)
            store_row(r0, row_exponent(rowmax[b_0]), f_0, f_0 * QG_PHASE_UNITS,
                      min(P.units, (f_0 + 1) * QG_PHASE_UNITS), sbase + Smem::kXBuf + f_0 * slot_bytes, Bl, b_0, lane);
        if (i1 < n_pairs)
            store_row(r1, row_exponent(rowmax[b_1]), f_1, f_1 * QG_PHASE_UNITS,
                      min(P.units, (f_1 + 1) * QG_PHASE_UNITS), sbase + Smem::kXBuf + f_1 * slot_bytes, Bl, b_1, lane);
        if (wid < 8 && lane == 0) rowexp[wid] = wid < Bl ? row_exponent(rowmax[wid]) : 0;
        named_bar_sync(2, 32 * kWarps);
    };

    // Epilogue of the resident path (runs on converter warp 0 once the activations are converted):
    // reduce the eight K slices of each finished panel in warp order, scale, store.
    auto run_epilogue = [&]() {
        ItemWalker wk;
        wk.init(total, P.units, P.n_panels, cta, grid);
        Item it;
        uint32_t rcnt = 0;
        const float ts = (FMT == QGEMV_FMT_NVFP4) ? P.tensor_scale[0] : 1.0f;
        const uint32_t red = sbase + Smem::kRed;
        while (wk.next(it)) {
            for (int pl = 0; pl < it.np; ++pl) {
                const int rs = rcnt % kRedSlots;
                if (!mbar_wait(sbase + Smem::kBarRedFull + 8 * rs, (rcnt / kRedSlots) & 1, P.spin_limit)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 6, int(rcnt));
                    *abort_flag = 1;
                    return;
                }
                float4 v = lds128f(red + (rs * kConsumerWarps) * 512 + lane * 16);
#pragma unroll
                for (int ww = 1; ww < kConsumerWarps; ++ww) {
                    const float4 q = lds128f(red + (rs * kConsumerWarps + ww) * 512 + lane * 16);
                    v.x += q.x, v.y += q.y, v.z += q.z, v.w += q.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + Smem::kBarRedEmpty + 8 * rs);
                ++rcnt;
                v.x *= ts, v.y *= ts, v.z *= ts, v.w *= ts;
                const int32_t panel = int32_t(it.vp + pl);  // dense: virtual panel == panel
                if (!it.partial) {
                    store_panel<FMT>(P, v, lane, panel, P.B, nullptr, P.chan_scale);
                } else {
                    finish_partial<FMT>(P, v, lane, it.vp, panel, cta, grid, total, P.B, nullptr, P.chan_scale);
                }
            }
        }
    };

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
            // one stage = the units of one (panel, phase) that the item covers; the per-stage path
            // is additions only (stage index, parity and source address are carried along)
            int s = 0;
            uint32_t use = 0;
            auto issue = [&](const uint8_t* panel_base, int64_t panel_off, int u0, int u1, int f) -> bool {
                const int ua = max(u0, f * QG_PHASE_UNITS);
                const int ub = min(u1, (f + 1) * QG_PHASE_UNITS);
                const uint32_t bytes = uint32_t(ub - ua) * kUnitBytes;
                if (use > 0 && !mbar_wait(sbase + Smem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 1, int(cnt));
                    *abort_flag = 1;
                    return false;
                }
                const uint64_t off = uint64_t(panel_off) + uint64_t(ua) * kUnitBytes;
                if ((P.debug & 1) && off + bytes > P.payload_bytes) {
                    report(P.status, QGEMV_ERR_BOUNDS, 2, int(cnt));
                    *abort_flag = 1;
                    return false;
                }
                const uint32_t bar = sbase + Smem::kBarFull + 8 * s;
                mbar_arrive_expect_tx(bar, bytes);
                bulk_g2s(sbase + Smem::kStage0 + s * kStageBytes, panel_base + off, bytes, bar, pol);
                ++cnt;
                if (++s == kStages) {
                    s = 0;
                    ++use;
                }
                return true;
            };
            const int64_t panel_bytes = int64_t(P.units) * kUnitBytes;
            while (ok && wk.next(it)) {
                const int f0 = it.u0 / QG_PHASE_UNITS, f1 = (it.u1 - 1) / QG_PHASE_UNITS;
                const int64_t prob = dense ? 0 : it.vp / P.n_panels;
                const int64_t panel0 = it.vp - prob * P.n_panels;
                const int expert = dense ? 0 : __ldcg(P.prob + 1 + prob * kProbInts);
                const uint8_t* base = P.payload + uint64_t(expert) * P.stack_stride;
                if (resident) {  // panel by panel
                    for (int pl = 0; ok && pl < it.np; ++pl)
                        for (int f = f0; ok && f <= f1; ++f)
                            ok = issue(base, (panel0 + pl) * panel_bytes, it.u0, it.u1, f);
                } else {         // phase by phase over the panels of the item
                    for (int f = f0; ok && f <= f1; ++f)
                        for (int pl = 0; ok && pl < it.np; ++pl)
                            ok = issue(base, (panel0 + pl) * panel_bytes, it.u0, it.u1, f);
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
        int* xexp_all = reinterpret_cast<int*>(smem_raw + Smem::kXExp);
        if (resident) {
            convert_resident(kConsumerWarps + role);
            if (warp == kEpilogueWarp) run_epilogue();
        } else {
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
                    const int xs = int(xcnt % uint32_t(n_slots));
                    const uint32_t use = xcnt / uint32_t(n_slots);
                    if (use > 0 &&
                        !mbar_wait(sbase + Smem::kBarXEmpty + 8 * xs, (use - 1) & 1, P.spin_limit)) {
                        if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 3, int(xcnt));
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    for (int b = role; b < Bl; b += kConverterWarps) {
                        int E = 0;
                        if (b < nrows) {
                            const int64_t row = dense ? b : __ldcg(pr + 2 + b);
                            E = convert_row(P.x + row * int64_t(P.K), P.K, f, ua, ub,
                                            sbase + Smem::kXBuf + xs * slot_bytes, Bl, b, lane);
                        }
                        if (lane == 0) xexp_all[xs * 8 + b] = E;
                    }
                    __threadfence_block();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + Smem::kBarXFull + 8 * xs);
                    ++xcnt;
                }
            }
        }
    } else if (resident) {
        // ================= consumers, resident path: panel by panel =================
        const int w = warp;
        const int g = lane >> 2, t = lane & 3;
        pdl_wait();  // activations come from the preceding kernel
        convert_resident(w);
        ItemWalker wk;
        wk.init(total, P.units, P.n_panels, cta, grid);
        Item it;
        uint32_t rcnt = 0;
        int s = 0;
        uint32_t par = 0;
        const int* rowexp = reinterpret_cast<const int*>(smem_raw + Smem::kXExp);
        const float fs0 = pow2i(rowexp[2 * t]), fs1 = pow2i(rowexp[2 * t + 1]);
        const uint32_t red = sbase + Smem::kRed + w * 512 + lane * 16;
        const int qA = 2 * w;
        // this lane's activation fragments of unit qA, pair 0, inside a phase slot
        const bool xlane = g < Bl;
        const uint32_t xlane_off = sbase + Smem::kXBuf + (qA * 2 * Bl + g) * 64 + t * 16;
        const uint32_t xpair = uint32_t(Bl) * 64u;
        while (wk.next(it)) {
            const int f0 = it.u0 / QG_PHASE_UNITS, f1 = (it.u1 - 1) / QG_PHASE_UNITS;
            for (int pl = 0; pl < it.np; ++pl) {
                float cA[4] = {0.f, 0.f, 0.f, 0.f}, cB[4] = {0.f, 0.f, 0.f, 0.f};
                for (int f = f0; f <= f1; ++f) {
                    const int ua = max(it.u0, f * QG_PHASE_UNITS);
                    const int ub = min(it.u1, (f + 1) * QG_PHASE_UNITS);
                    const int uA = f * QG_PHASE_UNITS + qA, uB = uA + 1;
                    const bool haveA = uA >= ua && uA < ub, haveB = uB >= ua && uB < ub;
                    uint32_t bfA[8], bfB[8];
#pragma unroll
                    for (int z = 0; z < 8; ++z) bfA[z] = bfB[z] = 0u;
                    if (xlane) {
                        const uint32_t xl = xlane_off + f * slot_bytes;
                        const uint4 x0 = lds128(xl);
                        const uint4 x1 = lds128(xl + xpair);
                        const uint4 x2 = lds128(xl + 2 * xpair);
                        const uint4 x3 = lds128(xl + 3 * xpair);
                        bfA[0] = x0.x, bfA[1] = x0.y, bfA[2] = x0.z, bfA[3] = x0.w;
                        bfA[4] = x1.x, bfA[5] = x1.y, bfA[6] = x1.z, bfA[7] = x1.w;
                        bfB[0] = x2.x, bfB[1] = x2.y, bfB[2] = x2.z, bfB[3] = x2.w;
                        bfB[4] = x3.x, bfB[5] = x3.y, bfB[6] = x3.z, bfB[7] = x3.w;
                    }
                    if (!mbar_wait(sbase + Smem::kBarFull + 8 * s, par, P.spin_limit)) {
                        if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 5, s);
                        *abort_flag = 1;
                        return;
                    }
                    const uint32_t st = sbase + Smem::kStage0 + s * kStageBytes + (uA - ua) * kUnitBytes;
                    if (haveA && haveB) {
                        consume_two<FMT>(cA, cB, st, st + kUnitBytes, lane, bfA, bfB);
                    } else if (haveA) {
                        consume_unit<FMT>(cA, st, lane, bfA);
                    } else if (haveB) {
                        consume_unit<FMT>(cB, st + kUnitBytes, lane, bfB);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + Smem::kBarEmpty + 8 * s);
                    if (++s == kStages) {
                        s = 0;
                        par ^= 1u;
                    }
                }
                // hand this warp's K slice of the panel to the epilogue warp
                const int rs = rcnt % kRedSlots;
                const uint32_t ruse = rcnt / kRedSlots;
                if (ruse > 0 && !mbar_wait(sbase + Smem::kBarRedEmpty + 8 * rs, (ruse - 1) & 1, P.spin_limit)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 7, int(rcnt));
                    *abort_flag = 1;
                    return;
                }
                sts128f(red + rs * kConsumerWarps * 512, (cA[0] + cB[0]) * fs0, (cA[1] + cB[1]) * fs1,
                        (cA[2] + cB[2]) * fs0, (cA[3] + cB[3]) * fs1);
                __threadfence_block();
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + Smem::kBarRedFull + 8 * rs);
                ++rcnt;
            }
        }
    } else {
        // ================= consumers, ring path: phase by phase over up to kPMax panels =================
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
                const int xb = resident ? f : int(xcnt % uint32_t(n_slots));
                const uint32_t xpar = resident ? 0u : ((xcnt / uint32_t(n_slots)) & 1u);
                if (!mbar_wait(sbase + Smem::kBarXFull + 8 * xb, xpar, P.spin_limit)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 4, int(xcnt));
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                // activation fragments of this warp's two units (lanes of columns >= Bl hold zeros)
                const uint32_t xbuf = sbase + Smem::kXBuf + xb * slot_bytes;
                const int ua_q = 2 * w, ub_q = 2 * w + 1;
                const int uA = f * QG_PHASE_UNITS + ua_q, uB = f * QG_PHASE_UNITS + ub_q;
                const bool haveA = uA >= ua && uA < ub, haveB = uB >= ua && uB < ub;
                uint32_t bfA[8], bfB[8];
#pragma unroll
                for (int z = 0; z < 8; ++z) bfA[z] = bfB[z] = 0u;
                if (g < Bl) {
                    const uint32_t xl = xbuf + g * 64 + t * 16;
                    const uint4 x0 = lds128(xl + (ua_q * 2 + 0) * Bl * 64);
                    const uint4 x1 = lds128(xl + (ua_q * 2 + 1) * Bl * 64);
                    const uint4 x2 = lds128(xl + (ub_q * 2 + 0) * Bl * 64);
                    const uint4 x3 = lds128(xl + (ub_q * 2 + 1) * Bl * 64);
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
                if (!resident && lane == 0) mbar_arrive(sbase + Smem::kBarXEmpty + 8 * xb);
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
                            finish_partial<FMT>(P, v, lane, it.vp, panel0, cta, grid, total, nrows, pr, chan);
                        }
                    }
                    named_bar_sync(1, 32 * kConsumerWarps);
                }
            }
        }
    }
}

}  // namespace qg
