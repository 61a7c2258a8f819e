// Skinny GEMM / short prefill on the 5th-generation tensor cores (tcgen05, TMEM):
//     Y[M][N] = X[M][K] * dequant(W)^T,   M = 16 .. 256 tokens (multiple of 16).
//
// "W4A16-exact" variant: the packed NVFP4 / FP8 weights are dequantised to f16 (the f16 value of
// code * block scale is exact) and multiplied with f16 activations by tcgen05.mma kind::f16 with
// fp32 accumulators in tensor memory.  Activations are converted bf16 -> f16 once per call by
// x_prep_kernel, scaled per token row by a power of two exactly as in the GEMV kernels.  (The
// block-scaled kinds, mxf4nvf4 / f8f6f4, need FP4 / FP8 activations and cannot meet a 2e-3 bound
// against unquantised activations; they are a different operator.)
//
// MMA shape: M = 128 weight rows (8 panels) x N = M_tokens x K = 16; a unit (64 K) is four MMAs.
//   A operand (weights)  lives in TENSOR MEMORY: the packed unit is ordered as mma.m16n8k16
//       fragments, and the register quadruple of one fragment is exactly what
//       tcgen05.st.16x256b wants for a 16-row x 16-k slab, so a dequantising warp converts
//       (cvt + one f16x2 multiply per register) and stores a whole unit with one tcgen05.st.x4:
//       no shuffles, no shared-memory round trip.  The slab's k order is the packed layout's
//       permutation (slot s = 4t + 2r + h); x_prep_kernel writes the activations in the same order.
//   B operand (activations) is read from shared memory through a K-major no-swizzle descriptor
//       (core matrix = 8 token rows x 16 bytes); x_prep_kernel lays the tiles out in that order
//       so one bulk copy brings a whole [M x 64] tile.
//   D (fp32) occupies TMEM columns [0, M); the A ring (two or three stages of one run = up to four
//       units, 32 columns per unit) sits at the end of the allocation.
//
// Pipeline grain: a RUN = up to four consecutive units of one row tile.  One bulk copy per panel
// fetches a run of packed weights; the MMA issuer waits once per run for the dequantised weights and
// once per activation stage (1, 2 or 4 units, whatever leaves >= 3-4 stages in shared memory), so
// its per-unit path is four tcgen05.mma and nothing else -- measured here, a wait + fence + commit
// per unit costs ~300 cycles of the issuing thread, more than the MMAs of a narrow tile.
//
// Work split: the linear space (row tile, run) is cut evenly over the CTAs (one per SM); a CTA's
// range is a sequence of segments, each a K range of one row tile.  A segment that covers its
// whole tile stores Y directly; otherwise the fp32 partial goes to a workspace slot and the last
// contributor of the tile (atomic counter) adds all parts in CTA order -- deterministic.
//
// Warp roles (15 warps):
//   0-11 three dequantising warpgroups; group q = warp / 4 takes the CTA's runs r = q (mod 3), so the
//        latency of one run's conversion, tcgen05.st and barrier round trips overlaps the other
//        groups' runs.  Warp w handles panels 2(w%4), 2(w%4)+1 = TMEM lanes 32(w%4)..+31 (the lane
//        quarter a warp may access), and in the epilogue the same lanes of every third 16-column chunk
//   12   one thread issues the bulk copies of packed weights (ring of 3-4 runs)
//   13   allocates TMEM; one elected lane walks the runs, issues tcgen05.mma and the commits that free
//        ring stages
//   14   one thread issues the bulk copies of activation tiles (L2 evict-last: every CTA re-reads them)
// Every wait is bounded; TMEM is always released before the CTA exits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemv_kernel.cuh"

namespace qg {

constexpr int kGsGroups = 3;     // dequantising warpgroups; group q takes the CTA's runs r = q (mod 3)
constexpr int kGsDqWarps = 4 * kGsGroups;
constexpr int kGsWarpP = kGsDqWarps, kGsWarpMma = kGsDqWarps + 1, kGsWarpX = kGsDqWarps + 2;
constexpr int kGsThreads = 32 * (kGsDqWarps + 3);
constexpr int kGsMaxM = 256;
constexpr int kGsRunMax = 4;     // units of one panel fetched by one bulk copy (a run); also the pipeline's grain
constexpr int kGsPStagesMax = 10; // packed-weight ring: stages of 8 panels x one run
constexpr int kGsAStagesMax = 3; // dequantised-weight ring in TMEM: stages of one run (32 columns per unit)
constexpr int kGsXStagesMax = 16;
constexpr int kGsSmemBudget = 227 * 1024;

struct GsParams {
    const uint8_t* payload;   // packed weight
    const float* chan_scale;  // FP8 channel scales
    float tensor_scale;
    const uint8_t* xt;        // f16 activation tiles: [units][M/8][8 chunks][8 rows][8 slots]
    const int32_t* xexp;      // per token row: exponent E (x was scaled by 2^-E)
    unsigned int* rowmax;     // x_rowmax_kernel's scratch; cleared here for the next call
    void* y;                  // [M][N]
    float* ws;                // partial tiles: slot (2*cta + which) of [M][128] fp32
    int32_t* counters;        // per row tile, zero between launches
    int32_t y_dtype;
    int32_t N, K, M;
    int32_t units;            // K / 64
    int32_t tiles;            // N / 128
    int32_t x_stages;
    int32_t p_stages;
    int32_t run_log2;         // log2(units per run): 2, 1 or 0, the largest that divides K / 64
    int32_t xg_log2;          // log2(units per activation-ring stage), <= run_log2
    int32_t* status;
    int64_t spin_limit;
    int32_t debug;
};

struct GsSmem {
    static constexpr int kBarPFull = 0;      // kGsPStagesMax
    static constexpr int kBarPEmpty = 80;    // kGsPStagesMax
    static constexpr int kBarXFull = 160;    // kGsXStagesMax
    static constexpr int kBarXEmpty = 288;   // kGsXStagesMax
    static constexpr int kBarAReady = 416;   // kGsAStagesMax
    static constexpr int kBarAEmpty = 440;   // kGsAStagesMax
    static constexpr int kBarDone = 464;
    static constexpr int kBarDFree = 472;
    static constexpr int kTmemPtr = 480;
    static constexpr int kAbort = 484;
    static constexpr int kBarDrain = 488;
    static constexpr int kRing0 = 1024;
    // Layout: [barriers][activation ring: x_stages x (M*128 << xg_log2)][packed ring: p_stages x
    // packed_stage].  Both rings sit between a producer and the MMAs with a memory latency of a few
    // thousand cycles in the loop, so what matters is how many RUNS each holds: the budget is split
    // so that the two depths (in runs) are about equal.
    __host__ __device__ static constexpr int packed_stage(int unit_bytes) { return 8 * kGsRunMax * unit_bytes; }
    // activation stage grain: the largest (<= the run) whose stage is at most 32 KB
    __host__ __device__ static int xg_log2(int M, int run_log2) {
        int g = run_log2;
        while (g > 0 && ((M * 128) << g) > 32768) --g;
        return g;
    }
    __host__ __device__ static int x_stages(int unit_bytes, int M, int xg_log2) {
        const int budget = kGsSmemBudget - kRing0;
        const int per_run = M * 128 * kGsRunMax + packed_stage(unit_bytes);
        int n = (budget / per_run) * kGsRunMax + ((budget % per_run) * kGsRunMax) / per_run;  // depth in units
        n >>= xg_log2;                                                                       // in stages
        const int keep_p = (budget - 3 * packed_stage(unit_bytes)) / ((M * 128) << xg_log2);  // leave >= 3 packed stages
        n = n > keep_p ? keep_p : n;
        return n > kGsXStagesMax ? kGsXStagesMax : (n < 2 ? 2 : n);
    }
    __host__ __device__ static int p_off(int unit_bytes, int M, int xg_log2) {
        return kRing0 + x_stages(unit_bytes, M, xg_log2) * ((M * 128) << xg_log2);
    }
    __host__ __device__ static int p_stages(int unit_bytes, int M, int xg_log2) {
        const int n = (kGsSmemBudget - p_off(unit_bytes, M, xg_log2)) / packed_stage(unit_bytes);
        return n > kGsPStagesMax ? kGsPStagesMax : n;
    }
    __host__ __device__ static int total(int unit_bytes, int M, int xg_log2) {
        return p_off(unit_bytes, M, xg_log2) + p_stages(unit_bytes, M, xg_log2) * packed_stage(unit_bytes);
    }
    // Tensor memory: D in columns [0, M); behind it the A ring, three stages of one run (32 columns
    // per unit) when they fit 512 columns, else two; the allocation is the next power of two.
    __host__ __device__ static int a_stages(int M, int run_log2) { return M + 3 * (32 << run_log2) <= 512 ? 3 : 2; }
    __host__ __device__ static int tmem_columns(int M, int run_log2) {
        int n = 32;
        while (n < M + a_stages(M, run_log2) * (32 << run_log2)) n <<= 1;
        return n;
    }
};

// ---- tcgen05 wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 16 lanes x 32 columns: slab j (columns 8j..8j+7) takes registers 4j..4j+3 of every thread;
// thread (g, t) supplies lane g: columns 2t, 2t+1 (registers 0, 1) and lane g+8 (registers 2, 3).
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n .reg .pred P;\n elect.sync _|P, 0xFFFFFFFF;\n selp.u32 %0, 1, 0, P;\n}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// K-major, no swizzle: core matrix = 8 rows x 16 bytes (128 contiguous bytes); the next 16-byte K
// chunk is LBO bytes away, the next 8-row group SBO bytes away.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return uint64_t((addr >> 4) & 0x3FFFu) | (uint64_t((lbo >> 4) & 0x3FFFu) << 16) |
           (uint64_t((sbo >> 4) & 0x3FFFu) << 32) | (uint64_t(1) << 46);
}

// Position (0..63) inside a unit's MMA k order of logical element k (0..63): slab j = tile T of
// the packed layout, slot s = 4t + 2r + h inside the slab.
__host__ __device__ __forceinline__ int gs_kslot(int k) {
    const int kb = k >> 4, e = k & 15;
    const int pr = kb >> 1, h = kb & 1, t = e >> 2, sub = (e >> 1) & 1, r = e & 1;
    return 16 * (2 * pr + sub) + 4 * t + 2 * r + h;
}

// Activation preparation, two small kernels over a grid of (2048-element segment, token row):
// x_rowmax_kernel finds every row's largest |bf16| bit pattern (atomicMax into rowmax[], which is
// zero between calls: the GEMM kernel clears it once it no longer needs it); x_prep_kernel
// converts bf16 -> f16 scaled by 2^-E (row maximum into [2^14, 2^15)) and writes tile order:
// element (m, k), unit u = k / 64, position p = gs_kslot(k % 64) goes to
//   xt + u * (M*128) + (m/8)*1024 + (p/8)*128 + (m%8)*16 + (p%8)*2.
constexpr int kXPrepThreads = 256;
__global__ void __launch_bounds__(kXPrepThreads) x_rowmax_kernel(const uint16_t* x, int K, unsigned int* rowmax) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.y;
    const int k = (blockIdx.x * kXPrepThreads + threadIdx.x) * 8;
    unsigned int mx = 0;
    if (k < K) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + int64_t(m) * K + k));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int z = 0; z < 4; ++z) {
            mx = max(mx, w[z] & 0x7FFFu);
            mx = max(mx, (w[z] >> 16) & 0x7FFFu);
        }
    }
    mx = __reduce_max_sync(0xFFFFFFFFu, mx);
    __shared__ unsigned int smax;
    if (threadIdx.x == 0) smax = 0u;
    __syncthreads();
    if ((threadIdx.x & 31) == 0 && mx != 0) atomicMax(&smax, mx);
    __syncthreads();
    if (threadIdx.x == 0 && smax != 0) atomicMax(rowmax + m, smax);
}
__global__ void __launch_bounds__(kXPrepThreads) x_prep_kernel(const uint16_t* x, int M, int K, const unsigned int* rowmax,
                                                               uint8_t* xt, int32_t* xexp) {
    __shared__ __align__(16) uint16_t seg[kXPrepThreads * 8];  // 2048 elements = 32 units
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.y;
    const int E = row_exponent(__ldcg(rowmax + m));
    if (blockIdx.x == 0 && threadIdx.x == 0) xexp[m] = E;
    const float sf = pow2i(-E);
    const int k = (blockIdx.x * kXPrepThreads + threadIdx.x) * 8;
    if (k < K) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + int64_t(m) * K + k));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        const int ubase = (threadIdx.x >> 3) * 64, kin = (threadIdx.x & 7) * 8;
#pragma unroll
        for (int z = 0; z < 4; ++z) {
            const uint32_t f = pack_f16x2(__uint_as_float(w[z] << 16) * sf, __uint_as_float(w[z] & 0xFFFF0000u) * sf);
            seg[ubase + gs_kslot(kin + 2 * z)] = uint16_t(f & 0xFFFFu);
            seg[ubase + gs_kslot(kin + 2 * z + 1)] = uint16_t(f >> 16);
        }
    }
    __syncthreads();
    if (k < K) {
        const uint4 o = *reinterpret_cast<const uint4*>(seg + threadIdx.x * 8);
        const int u = k >> 6, chunk = (k & 63) >> 3;
        *reinterpret_cast<uint4*>(xt + size_t(u) * (size_t(M) * 128) + size_t(m >> 3) * 1024 + (m & 7) * 16 + chunk * 128) = o;
    }
}

// Dequantises one packed unit (lane-ordered MMA-fragment layout) and stores it as four 16x16
// slabs into 16 TMEM lanes x 32 columns at `taddr`.
template <int FMT>
__device__ __forceinline__ void dequant_unit_to_tmem(uint32_t unit, uint32_t taddr, int lane) {
    uint32_t a[16];  // [slab T][register]: order (row g, r=0), (row g, r=1), (row g+8, r=0), (row g+8, r=1)
    if (FMT == QGEMV_FMT_NVFP4) {
        const uint4 cw = lds128(unit + lane * 16);
        const uint2 sw = lds64(unit + 512 + (lane >> 2) * 8);
        uint32_t sg[2], sh[2];
        cvt_e4m3x4(sw.x, sg[0], sg[1]);  // row g:   (blk0, blk1), (blk2, blk3)
        cvt_e4m3x4(sw.y, sh[0], sh[1]);  // row g+8
        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int T = 0; T < 4; ++T) {
            uint32_t b0, b1, b2, b3;  // bytes jb = rowhi + 2r
            cvt_e2m1x8(w[T], b0, b1, b2, b3);
            a[4 * T + 0] = hmul2(b0, sg[T >> 1]);
            a[4 * T + 1] = hmul2(b2, sg[T >> 1]);
            a[4 * T + 2] = hmul2(b1, sh[T >> 1]);
            a[4 * T + 3] = hmul2(b3, sh[T >> 1]);
        }
    } else {
        const uint4 v0 = lds128(unit + lane * 16);
        const uint4 v1 = lds128(unit + 512 + lane * 16);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int T = 0; T < 4; ++T) {
            uint32_t b0, b1, b2, b3;
            cvt_e4m3x4(w[2 * T], b0, b1);
            cvt_e4m3x4(w[2 * T + 1], b2, b3);
            a[4 * T + 0] = b0, a[4 * T + 1] = b2, a[4 * T + 2] = b1, a[4 * T + 3] = b3;
        }
    }
    tmem_st_16x256b_x4(taddr, a);
}

// One segment of a CTA's range: units [u0, u1) of row tile `tile`.
struct GsSeg {
    int32_t tile, u0, u1;
};
struct GsWalker {
    int32_t pos, end, units;
    __device__ __forceinline__ void init(int32_t total, int32_t units_, int cta, int grid) {
        units = units_;
        pos = int32_t((int64_t(cta) * total) / grid);
        end = int32_t((int64_t(cta + 1) * total) / grid);
    }
    __device__ __forceinline__ bool next(GsSeg& s) {
        if (pos >= end) return false;
        s.tile = pos / units;
        s.u0 = pos - s.tile * units;
        const int32_t left = end - pos;
        s.u1 = s.u0 + left < units ? s.u0 + left : units;
        pos += s.u1 - s.u0;
        return true;
    }
};
// Workspace slot of the part of row tile `tile` that CTA c computes: its first segment uses slot
// 2c, its last one slot 2c + 1 (segments in between are whole tiles and need none).
__device__ __forceinline__ int32_t gs_slot(int32_t c, int32_t tile, int32_t units, int32_t total, int grid) {
    const int32_t a = int32_t((int64_t(c) * total) / grid);
    return 2 * c + (a / units == tile ? 0 : 1);
}

template <int FMT>
__global__ void __launch_bounds__(kGsThreads, 1) gemm_skinny_kernel(const GsParams P) {
    constexpr int kUnitBytes = FmtTraits<FMT>::kUnitBytes;
    constexpr int kPStage = GsSmem::packed_stage(kUnitBytes);
    extern __shared__ __align__(128) unsigned char gs_smem[];
    const uint32_t sbase = smem_u32(gs_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int M = P.M;
    const int grid = gridDim.x, cta = blockIdx.x;
    // the work space is counted in runs (1 << rl units of one row tile): `runs` per tile, `total` runs
    const int rl = P.run_log2, run = 1 << rl;
    const int xgl = P.xg_log2, xg = 1 << xgl;
    const int runs = P.units >> rl;
    const int32_t total = P.tiles * runs;
    const int32_t r_begin = int32_t((int64_t(cta) * total) / grid);
    const int32_t r_end = int32_t((int64_t(cta + 1) * total) / grid);
    const uint32_t x_bytes = uint32_t(M) * 128u;       // one unit of activations
    const uint32_t xs_bytes = x_bytes << xgl;          // one stage of the activation ring
    const uint32_t xring = sbase + GsSmem::kRing0;
    const int x_stages = P.x_stages, kPStages = P.p_stages;
    const uint32_t pring = xring + uint32_t(x_stages) * xs_bytes;
    // TMEM: D in columns [0, M); behind it the A ring, kA stages of one run (32 columns per unit)
    const uint32_t a_cols = 32u << rl;
    const int kA = GsSmem::a_stages(M, rl);
    const uint32_t ncols = uint32_t(GsSmem::tmem_columns(M, rl));
    const uint32_t acol0 = ncols - kA * a_cols;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gs_smem + GsSmem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gs_smem + GsSmem::kTmemPtr);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGsPStagesMax; ++s) {
            mbar_init(sbase + GsSmem::kBarPFull + 8 * s, 1);
            mbar_init(sbase + GsSmem::kBarPEmpty + 8 * s, 4);  // the four warps of the group that converts the run
        }
        for (int s = 0; s < kGsXStagesMax; ++s) {
            mbar_init(sbase + GsSmem::kBarXFull + 8 * s, 1);
            mbar_init(sbase + GsSmem::kBarXEmpty + 8 * s, 1);
        }
        for (int s = 0; s < kGsAStagesMax; ++s) {
            mbar_init(sbase + GsSmem::kBarAReady + 8 * s, 4);
            mbar_init(sbase + GsSmem::kBarAEmpty + 8 * s, 1);
        }
        mbar_init(sbase + GsSmem::kBarDone, 1);
        mbar_init(sbase + GsSmem::kBarDFree, kGsDqWarps);
        mbar_init(sbase + GsSmem::kBarDrain, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kGsWarpMma) {
        __syncwarp();
        tmem_alloc(sbase + GsSmem::kTmemPtr, ncols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    pdl_launch_dependents();

    if (warp == kGsWarpP) {
        // ================= packed-weight producer: one stage = 8 panels x one run =================
        // Eight lanes issue the eight panels' copies with one instruction each turn (a single thread
        // issuing them back to back spends longer per run than the copies take to arrive).
        if (lane < 8 && !(P.debug & 2)) {
            const uint64_t pol = policy_evict_first();
            int32_t tile = r_begin / runs, u = r_begin - tile * runs;
            const uint32_t run_bytes = uint32_t(kUnitBytes) << rl;
            int s = 0;
            uint32_t use = 0;
            for (int32_t pos = r_begin; pos < r_end; ++pos) {
                bool ok = use == 0 || mbar_wait_probe(sbase + GsSmem::kBarPEmpty + 8 * s, (use - 1) & 1, P.spin_limit);
                if (!__all_sync(0xFFu, ok)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 41, pos);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t bar = sbase + GsSmem::kBarPFull + 8 * s;
                const uint32_t st = pring + s * kPStage;
                if (lane == 0) mbar_arrive_expect_tx(bar, 8u * run_bytes);
                __syncwarp(0xFFu);
                const uint8_t* src = P.payload + (uint64_t(tile) * 8 * P.units + (uint64_t(u) << rl)) * kUnitBytes;
                bulk_g2s(st + lane * run_bytes, src + uint64_t(lane) * P.units * kUnitBytes, run_bytes, bar, pol);
                if (++u == runs) u = 0, ++tile;
                if (++s == kPStages) s = 0, ++use;
            }
        }
    } else if (warp == kGsWarpX) {
        // ================= activation-tile producer: one stage = xg units, one bulk copy =================
        if (lane == 0) {
            pdl_wait();  // the tiles come from x_prep_kernel
            if (cta == 0)
                for (int m = 0; m < M; ++m) P.rowmax[m] = 0u;  // x_prep_kernel has finished with it
            const uint64_t keep = policy_evict_last();  // every CTA re-reads the tiles: hold them in L2
            const int32_t c_begin = r_begin << (rl - xgl), c_end = r_end << (rl - xgl);  // in stages
            const int32_t cpt = P.units >> xgl;                                         // stages per tile
            int32_t c = c_begin % cpt;
            int s = 0;
            uint32_t use = 0;
            for (int32_t pos = c_begin; pos < c_end; ++pos) {
                if (use > 0 && !mbar_wait_probe(sbase + GsSmem::kBarXEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 46, pos);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t bar = sbase + GsSmem::kBarXFull + 8 * s;
                mbar_arrive_expect_tx(bar, xs_bytes);
                bulk_g2s(xring + s * xs_bytes, P.xt + uint64_t(c) * xs_bytes, xs_bytes, bar, keep);
                if (++c == cpt) c = 0;
                if (++s == x_stages) s = 0, ++use;
            }
        }
    } else if (warp == kGsWarpMma) {
        // ===== MMA issuer: one elected lane runs the whole loop (entering a one-lane region per unit
        // costs more than the four MMAs of a narrow tile).  Barriers are waited once per run (A) and
        // once per activation stage, so the per-unit path is four tcgen05.mma =====
        if (elect_one()) {
            const uint32_t idesc = (1u << 4) | (uint32_t(M >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            GsWalker wk;
            wk.init(total, runs, cta, grid);
            GsSeg sg;
            int sa = 0, sx = 0;
            uint32_t usea = 0, usex = 0, nseg = 0;
            int32_t istep = 0;  // unit index inside the CTA's range
            bool ok = true;
            while (ok && wk.next(sg)) {
                // the accumulator is free once the epilogue of the previous segment has read it
                if (nseg > 0 && !mbar_wait_probe(sbase + GsSmem::kBarDFree, (nseg - 1) & 1, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 47, int(nseg));
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                uint32_t acc = 0;  // the segment's first MMA overwrites D
                for (int32_t rr = sg.u0; rr < sg.u1 && ok; ++rr) {
                    if (!mbar_wait_probe(sbase + GsSmem::kBarAReady + 8 * sa, usea & 1, P.spin_limit)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 42, rr);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t ta_run = tmem_base + acol0 + sa * a_cols;
                    for (int s = 0; s < run; ++s, ++istep) {
                        const int xi = istep & (xg - 1);
                        if (xi == 0 && !mbar_wait_probe(sbase + GsSmem::kBarXFull + 8 * sx, usex & 1, P.spin_limit)) {
                            report(P.status, QGEMV_ERR_TIMEOUT, 48, rr);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        const uint64_t db = smem_desc(xring + sx * xs_bytes + xi * x_bytes, 128, 1024);
                        const uint32_t ta = ta_run + 32 * s;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {  // four K=16 slabs: 8 TMEM columns / two 16-byte chunks (+16 in the descriptor) each
                            tc_mma_f16_ts(tmem_base, ta + 8 * j, db + uint64_t(16 * j), idesc, acc);
                            acc = 1;
                        }
                        if (xi == xg - 1) {
                            tc_commit(sbase + GsSmem::kBarXEmpty + 8 * sx);  // stage reusable once these retire
                            if (++sx == x_stages) sx = 0, ++usex;
                        }
                    }
                    if (ok) tc_commit(sbase + GsSmem::kBarAEmpty + 8 * sa);
                    if (++sa == kA) sa = 0, ++usea;
                }
                tc_commit(sbase + GsSmem::kBarDone);
                ++nseg;
            }
        }
        __syncwarp();
    } else {
        // ================= dequantisation warps; epilogue of each segment =================
        const int q = warp >> 2, wq = warp & 3;  // group, TMEM lane quarter
        GsWalker wk;
        wk.init(total, runs, cta, grid);
        GsSeg sg;
        // Each TMEM stage must always be refilled by the same group (a parity wait may not run more than
        // one phase ahead of the barrier), so with two stages only two groups convert; all three
        // share the epilogue.
        const int ng = kA < kGsGroups ? kA : kGsGroups;
        int32_t rnext = q < ng ? q : 0x7FFFFFF0;  // this group's next run, as an index into the CTA's range
        int32_t seg_r0 = 0;  // index of the segment's first run
        uint32_t nseg = 0;
        bool ok = true;
        bool waited_x = false;
        const uint32_t lane_base = uint32_t(32 * wq) << 16;
        const int32_t n_local = r_end - r_begin;  // runs of this CTA
        // converts run r of the CTA's range into its TMEM stage; false when a wait ran out
        auto convert_run = [&](int32_t r) -> bool {
            const int sp = r % kPStages, sa = r % kA;
            const uint32_t usep = uint32_t(r / kPStages), usea = uint32_t(r / kA);
            // the TMEM stage is free once the MMAs of the run that used it last retired
            bool w_ok = usea == 0 || mbar_wait_probe(sbase + GsSmem::kBarAEmpty + 8 * sa, (usea - 1) & 1, P.spin_limit);
            w_ok = w_ok && mbar_wait_probe(sbase + GsSmem::kBarPFull + 8 * sp, usep & 1, P.spin_limit);
            if (!__all_sync(0xFFFFFFFFu, w_ok)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 44, r);
                *abort_flag = 1;
                return false;
            }
            tc_fence_after();
            // packed stage layout: [panel][unit of the run]; this warp: panels 2wq, 2wq+1
            const uint32_t st = pring + sp * kPStage + uint32_t((2 * wq) << rl) * kUnitBytes;
            const uint32_t ta = tmem_base + lane_base + acol0 + sa * a_cols;
            for (int ui = 0; ui < run; ++ui) {
                dequant_unit_to_tmem<FMT>(st + ui * kUnitBytes, ta + 32 * ui, lane);
                dequant_unit_to_tmem<FMT>(st + (uint32_t(kUnitBytes) << rl) + ui * kUnitBytes, ta + 32 * ui + (16u << 16), lane);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(sbase + GsSmem::kBarAReady + 8 * sa);
                mbar_arrive(sbase + GsSmem::kBarPEmpty + 8 * sp);
            }
            return true;
        };
        while (ok && wk.next(sg)) {
            const int32_t seg_r1 = seg_r0 + (sg.u1 - sg.u0);
            for (; rnext < seg_r1 && ok; rnext += ng) ok = convert_run(rnext);
            // While this segment's last MMAs drain, convert this group's first run of the NEXT segment:
            // its TMEM stage was last used by a run of this segment or earlier (rnext - kA < seg_r1), so
            // the wait above needs nothing that comes after the epilogue below.
            if (ok && rnext < n_local && rnext - kA < seg_r1) {
                ok = convert_run(rnext);
                rnext += ng;
            }
            seg_r0 = seg_r1;
            if (!ok) break;
            // ---- epilogue: this warp owns TMEM lanes [32wq, 32wq+32) and every third 16-column chunk ----
            if (!__all_sync(0xFFFFFFFFu, mbar_wait_probe(sbase + GsSmem::kBarDone, nseg & 1, P.spin_limit))) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 45, int(nseg));
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            if (!waited_x) {
                pdl_wait();  // the row exponents come from x_prep_kernel
                waited_x = true;
            }
            const int row = 32 * wq + lane;
            const int n = sg.tile * 128 + row;
            const float rs = (FMT == QGEMV_FMT_NVFP4) ? P.tensor_scale : __ldg(P.chan_scale + n);
            auto store_cols = [&](int c, const float (&v)[16]) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int m = c + i;
                    const float val = v[i] * rs * pow2i(__ldg(P.xexp + m));
                    const int64_t idx = int64_t(m) * P.N + n;
                    if (P.y_dtype == QGEMV_OUT_F32) {
                        static_cast<float*>(P.y)[idx] = val;
                    } else {
                        static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(val);
                    }
                }
            };
            if (sg.u0 == 0 && sg.u1 == runs) {  // the segment is the whole tile
                for (int c = 16 * q; c < M; c += 16 * kGsGroups) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + lane_base + uint32_t(c), r);
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
                    store_cols(c, v);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + GsSmem::kBarDFree);
            } else {
                // partial: park the fp32 sums, then the last contributor of (tile, warp) adds all
                // parts in CTA order
                float* slot = P.ws + size_t(gs_slot(cta, sg.tile, runs, total, grid)) * size_t(M) * 128;
                for (int c = 16 * q; c < M; c += 16 * kGsGroups) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + lane_base + uint32_t(c), r);
#pragma unroll
                    for (int i = 0; i < 16; ++i) __stcg(slot + (c + i) * 128 + row, __uint_as_float(r[i]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + GsSmem::kBarDFree);  // the next segment may start
                __threadfence();
                __syncwarp();
                const int32_t c_lo = int32_t(cta_of(int64_t(sg.tile) * runs, total, grid));
                const int32_t c_hi = int32_t(cta_of(int64_t(sg.tile + 1) * runs - 1, total, grid));
                int old = 0;
                if (lane == 0) old = atomicAdd(P.counters + sg.tile * 16 + warp, 1);
                old = __shfl_sync(0xFFFFFFFFu, old, 0);
                if (old == c_hi - c_lo) {
                    __threadfence();
                    for (int c = 16 * q; c < M; c += 16 * kGsGroups) {
                        float v[16];
                        for (int32_t cc = c_lo; cc <= c_hi; ++cc) {
                            const float* sl = P.ws + size_t(gs_slot(cc, sg.tile, runs, total, grid)) * size_t(M) * 128;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float qv = __ldcg(sl + (c + i) * 128 + row);
                                v[i] = cc == c_lo ? qv : v[i] + qv;
                            }
                        }
                        store_cols(c, v);
                    }
                    __syncwarp();
                    if (lane == 0) P.counters[sg.tile * 16 + warp] = 0;
                }
            }
            ++nseg;
        }
    }
    // ---- release TMEM (always), after every role is done with it ----
    tc_fence_before();
    __syncthreads();
    if (warp == kGsWarpMma) {
        __syncwarp();
        if (*abort_flag) {
            // let whatever MMAs were issued retire before the columns are handed back (bounded)
            if (lane == 0) {
                tc_commit(sbase + GsSmem::kBarDrain);
                (void)mbar_wait_probe(sbase + GsSmem::kBarDrain, 0, int64_t(1) << 16);
            }
            __syncwarp();
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, ncols);
    }
}

}  // namespace qg
