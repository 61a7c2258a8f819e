// Block-scaled prefill GEMM, activations quantised to NVFP4 ("A4"): Y[M][N] = Xq[M][K] Wq[N][K]^T for
// 16..256 tokens on tcgen05.mma kind::mxf4nvf4 with BOTH operands consumed as stored -- the weights
// in the tensor-core tile order (QGEMV_FMT_NVFP4_TC), the activations as E2M1 codes with one E4M3
// scale per 16 K elements and one fp32 scale per token row, produced by the quantiser below.  No SM
// instruction touches a weight or an activation element; the MMA's N extent is the token count, so
// a 64-K item of a 128-row tile is ONE instruction for up to 128 tokens (two for up to 256).
//
// The quantiser is specified bit for bit (the host-side checker restates it): per token row, fp32 with
// round-to-nearest-even throughout,
//   amax = max |x|;  g = amax == 0 ? 1 : amax / 2688          (2688 = 6 * 448)
//   per 16-element block:  a = max |x| in the block;  s = E4M3(a / (6 * g)), saturating
//                          t = decode(s) * g;  code = t == 0 ? 0 : E2M1(x / t), saturating
// so an activation is decode(code) * decode(s) * g.  The result is
//   y[m][n] = tensor_scale * g[m] * sum_k (wcode * wscale)(n, k) * (code * s)(m, k),
// products and sums in the tensor core's fp32.
//
// Layout of the quantised activations in device memory (internal): one ITEM per 64 K elements,
//   [0, 32 M)            codes as the MMA's K-major no-swizzle B operand: token m, element k at
//                        (m / 8) * 256 + (k / 32) * 128 + (m % 8) * 16 + (k % 32) / 2
//   then one 512-byte block per 128 tokens: scales of token r = m % 128, block kb at (r % 32) * 16 + (r / 32) * 4 + kb
// i.e. the order tcgen05.cp.32x128b.warpx4 copies into tensor memory, like the weights' scales.
//
// Work: (row tile, K chunk) units dealt round-robin to one CTA per SM; with at least as many row
// tiles as SMs a unit is a whole tile and stores y, otherwise K is cut into chunks whose fp32
// results are added in chunk order by chunk_sum_kernel (deterministic).
// Warps: 0 producer (bulk copies of a weight item and an activation item per stage), 1 MMA issuer,
// 2-5 epilogue (tcgen05.ld, scale, store).  Every wait is bounded.
#pragma once
#include "gemv_tc.cuh"

namespace qg {

constexpr int kA4Threads = 32 * 6;
constexpr int kA4MaxRing = 16;
constexpr int kA4StageItems = 4;   // items of each operand per pipeline stage: one wait and one commit per stage
constexpr int kA4TmemCols = 512;

// the stage of its K range at which the unit of row tile `tile` starts (the order is part of the result's bits)
__host__ __device__ inline int a4_first_stage(int tile, int n_stages) { return int((uint32_t(tile) * 7u) % uint32_t(n_stages)); }
__host__ __device__ inline int a4_item_bytes(int M) { return M * 32 + ((M + 127) / 128) * 512; }

// fp32 pair -> two E4M3 bytes (a in the low byte), four fp32 -> four E2M1 codes (a in the low nibble)
__device__ __forceinline__ uint32_t a4_cvt_e4m3(float a) {
    uint32_t r;
    asm volatile("{\n .reg .b16 t;\n cvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\n cvt.u32.u16 %0, t;\n}" : "=r"(r) : "f"(0.f), "f"(a));
    return r & 0xFFu;
}
__device__ __forceinline__ uint32_t a4_cvt_e2m1x8(const float (&q)[8]) {
    uint32_t r;
    asm volatile(
        "{\n .reg .b8 b0, b1, b2, b3;\n"
        " cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        " cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        " mov.b32 %0, {b0, b1, b2, b3};\n}"
        : "=r"(r)
        : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
    return r;
}

struct A4QuantParams {
    const uint16_t* x;   // bf16 [M][K]
    int32_t M, K;
    uint8_t* items;      // internal layout (see above), or null
    float* g;            // [M] row scales
    uint8_t* codes;      // canonical parity outputs u8 [M][K/2], u8 [M][K/16], or null
    uint8_t* scales;
};

// One CTA per token row: row maximum, then one thread per 16-element block.
__global__ void __launch_bounds__(256) a4_quant_kernel(const A4QuantParams P) {
    __shared__ float s_max[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    const uint16_t* xr = P.x + int64_t(m) * P.K;
    const int nblk = P.K / 16;
    float amax = 0.f;
    for (int kb = threadIdx.x; kb < nblk; kb += blockDim.x) {
        const uint4 v0 = *reinterpret_cast<const uint4*>(xr + kb * 16), v1 = *reinterpret_cast<const uint4*>(xr + kb * 16 + 8);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int z = 0; z < 8; ++z) {
            amax = fmaxf(amax, fabsf(__uint_as_float(w[z] << 16)));
            amax = fmaxf(amax, fabsf(__uint_as_float(w[z] & 0xFFFF0000u)));
        }
    }
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
    if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.f;
    for (int w = 0; w < int(blockDim.x >> 5); ++w) amax = fmaxf(amax, s_max[w]);
    const float g = amax == 0.f ? 1.0f : __fdiv_rn(amax, 2688.0f);
    if (threadIdx.x == 0) P.g[m] = g;
    const float d6 = __fmul_rn(6.0f, g);
    const int item_bytes = a4_item_bytes(P.M);
    for (int kb = threadIdx.x; kb < nblk; kb += blockDim.x) {
        const uint4 v0 = *reinterpret_cast<const uint4*>(xr + kb * 16), v1 = *reinterpret_cast<const uint4*>(xr + kb * 16 + 8);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        float xv[16];
        float a = 0.f;
#pragma unroll
        for (int z = 0; z < 8; ++z) {
            xv[2 * z] = __uint_as_float(w[z] << 16), xv[2 * z + 1] = __uint_as_float(w[z] & 0xFFFF0000u);
            a = fmaxf(a, fmaxf(fabsf(xv[2 * z]), fabsf(xv[2 * z + 1])));
        }
        const uint32_t sb = a4_cvt_e4m3(__fdiv_rn(a, d6));
        // decode(s): E4M3 -> fp32 (exact), through the hardware conversion to f16
        uint32_t h2;
        asm volatile("{\n .reg .b16 t;\n cvt.u16.u32 t, %1;\n cvt.rn.f16x2.e4m3x2 %0, t;\n}" : "=r"(h2) : "r"(sb));
        const float sd = __half2float(__ushort_as_half(uint16_t(h2 & 0xFFFFu)));
        const float t = __fmul_rn(sd, g);
        uint32_t c0 = 0, c1 = 0;
        if (t != 0.f) {
            float q[8];
#pragma unroll
            for (int z = 0; z < 8; ++z) q[z] = __fdiv_rn(xv[z], t);
            c0 = a4_cvt_e2m1x8(q);
#pragma unroll
            for (int z = 0; z < 8; ++z) q[z] = __fdiv_rn(xv[8 + z], t);
            c1 = a4_cvt_e2m1x8(q);
        }
        if (P.codes) {
            *reinterpret_cast<uint2*>(P.codes + int64_t(m) * (P.K / 2) + kb * 8) = make_uint2(c0, c1);
            P.scales[int64_t(m) * nblk + kb] = uint8_t(sb);
        }
        if (P.items) {
            uint8_t* item = P.items + int64_t(kb >> 2) * item_bytes;
            const int k = (kb & 3) * 16;
            *reinterpret_cast<uint2*>(item + (m >> 3) * 256 + (k >> 5) * 128 + (m & 7) * 16 + ((k & 31) >> 1)) = make_uint2(c0, c1);
            const int r = m & 127;
            item[P.M * 32 + (m >> 7) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = uint8_t(sb);
        }
    }
}

struct A4Params {
    const uint8_t* payload;   // weight items: (tile * kt + item) * 4608
    const uint8_t* xq;        // activation items: item * xq_item_bytes
    const float* g;           // [M] row scales of the activations
    void* y;                  // [M][N] in y_dtype when n_chunk == 1, else fp32 partial results [chunk][M][N]
    int32_t* status;
    int64_t spin_limit;
    float tensor_scale;
    int32_t N, M;
    int32_t tiles, kt;        // ceil(N / 128), ceil(K / 64)
    int32_t n_chunk, chunk_items;
    int32_t xq_item_bytes;
    int32_t ring;
    int32_t y_dtype;
    int32_t debug;
};

struct A4Smem {
    static constexpr int kBarFull = 0;      // kA4MaxRing
    static constexpr int kBarEmpty = 128;   // kA4MaxRing
    static constexpr int kBarDFull = 256;
    static constexpr int kBarDFree = 264;
    static constexpr int kBarDrain = 272;
    static constexpr int kTmemPtr = 280;
    static constexpr int kAbort = 284;
    static constexpr int kIssued = 288;
    static constexpr int kConsumed = 292;
    static constexpr int kRing = 384;
    __host__ __device__ static constexpr int stage_bytes(int M) { return kA4StageItems * (kTcItemBytes + M * 32 + ((M + 127) / 128) * 512); }
    __host__ __device__ static constexpr int total(int M, int ring) { return kRing + ring * stage_bytes(M); }
    // tensor memory: accumulators in columns [0, 256), then per ring stage 4 columns of weight scales and
    // 4 per 128 tokens of activation scales
    __host__ __device__ static constexpr int max_ring(int M) { return (kA4TmemCols - 256) / (kA4StageItems * (4 + 4 * ((M + 127) / 128))); }
};

__global__ void __launch_bounds__(kA4Threads, 1) gemm_a4_kernel(const A4Params P) {
    extern __shared__ __align__(128) unsigned char a4_smem[];
    const uint32_t sbase = smem_u32(a4_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grid = gridDim.x, cta = blockIdx.x;
    const int M = P.M, R = P.ring;
    const int n_half = (M + 127) / 128;                 // MMAs per item: one per 128 tokens
    const uint32_t stage_bytes = uint32_t(A4Smem::stage_bytes(M));   // of a whole stage (kA4StageItems items of each operand)
    const uint32_t ring0 = sbase + A4Smem::kRing;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(a4_smem + A4Smem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(a4_smem + A4Smem::kTmemPtr);
    volatile int* n_issued = reinterpret_cast<volatile int*>(a4_smem + A4Smem::kIssued);
    volatile int* n_consumed = reinterpret_cast<volatile int*>(a4_smem + A4Smem::kConsumed);
    const int total_units = P.tiles * P.n_chunk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kA4MaxRing; ++s) {
            mbar_init(sbase + A4Smem::kBarFull + 8 * s, 1);
            mbar_init(sbase + A4Smem::kBarEmpty + 8 * s, 1);
        }
        mbar_init(sbase + A4Smem::kBarDFull, 1);
        mbar_init(sbase + A4Smem::kBarDFree, 4);
        mbar_init(sbase + A4Smem::kBarDrain, 1);
        *abort_flag = 0, *n_issued = 0, *n_consumed = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        __syncwarp();
        tmem_alloc(sbase + A4Smem::kTmemPtr, kA4TmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    pdl_launch_dependents();

    if (warp == 0) {
        // ---- producer: a weight item and the matching activation item per stage ----
        if (lane == 0) {
            const uint64_t pol_w = policy_evict_first();
            const uint32_t xib = uint32_t(P.xq_item_bytes);
            const bool drop = (P.debug & 2) != 0;   // host-set injection: never issue a copy
            int s = 0, issued = 0;
            uint32_t use = 0;
            bool ok = true;
            // the weights do not depend on what ran before; the activation items do
            bool waited = false;
            for (int u = cta; u < total_units && ok; u += grid) {
                const int tile = u / P.n_chunk, chunk = u - tile * P.n_chunk;
                const int i0 = chunk * P.chunk_items, i1 = min(P.kt, i0 + P.chunk_items);
                const uint8_t* wbase = P.payload + uint64_t(tile) * P.kt * kTcItemBytes;
                // The CTAs walk K in the same direction but start at different stages (by tile): at any
                // moment they ask L2 for different activation items instead of all for the same one.
                const int nst = (i1 - i0 + kA4StageItems - 1) / kA4StageItems;
                int sidx = a4_first_stage(tile, nst);
                for (int j = 0; j < nst && ok; ++j, sidx = sidx + 1 == nst ? 0 : sidx + 1) {
                    const int i = i0 + sidx * kA4StageItems;
                    const uint8_t* wsrc = wbase + uint64_t(i) * kTcItemBytes;
                    if (use > 0 && !mbar_wait_probe(sbase + A4Smem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 91, i);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    if (!drop) {
                        const uint32_t bar = sbase + A4Smem::kBarFull + 8 * s;
                        const uint32_t dst = ring0 + uint32_t(s) * stage_bytes;
                        const uint32_t n = uint32_t(min(kA4StageItems, i1 - i));
                        mbar_arrive_expect_tx(bar, n * (uint32_t(kTcItemBytes) + xib));
                        bulk_g2s(dst, wsrc, n * kTcItemBytes, bar, pol_w);
                        if (!waited) pdl_wait(), waited = true;   // the quantiser's output
                        bulk_g2s_plain(dst + kA4StageItems * kTcItemBytes, P.xq + uint64_t(i) * xib, n * xib, bar);
                        ++issued;
                    }
                    if (++s == R) s = 0, ++use;
                    if (*abort_flag) ok = false;
                }
            }
            *n_issued = issued;
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        // One thread, and a dependent instruction on one thread costs about five cycles: everything per stage
        // is additions on 32-bit descriptor halves (addresses in 16-byte units), unrolled over the stage's items.
        if (elect_one()) {
            const uint64_t d_ab = smem_desc(0, 128, 256), d_sf = smem_desc(0, 0, 128);
            const uint32_t ab_hi = uint32_t(d_ab >> 32), ab_lo = uint32_t(d_ab), sf_hi = uint32_t(d_sf >> 32), sf_lo = uint32_t(d_sf);
            const uint32_t n0 = uint32_t(M < 128 ? M : 128), n1 = uint32_t(M > 128 ? M - 128 : 0);
            const uint32_t idesc0 = (1u << 7) | (1u << 10) | ((n0 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            const uint32_t idesc1 = (1u << 7) | (1u << 10) | ((n1 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            const uint32_t sf_cols = 4u + 4u * uint32_t(n_half);
            const uint32_t xib16 = uint32_t(P.xq_item_bytes) >> 4, m2_16 = (uint32_t(M) * 32u) >> 4;
            constexpr uint32_t kItem16 = kTcItemBytes >> 4, kCode16 = kTcCodeBytes >> 4, kW16 = (kA4StageItems * kTcItemBytes) >> 4;
            const uint32_t stage16 = stage_bytes >> 4, ring16 = (ring0 >> 4) & 0x3FFFu, ring_end16 = ring16 + uint32_t(R) * stage16;
            const uint32_t sf_stage = sf_cols * kA4StageItems, sf_first = tmem_base + 256u;
            uint32_t w16 = ring16, sf0 = sf_first, bar_full = sbase + A4Smem::kBarFull, bar_empty = sbase + A4Smem::kBarEmpty;
            int mi = 0;
            uint32_t full_par = 0, nunit = 0;
            bool ok = true;
            for (int u = cta; u < total_units && ok; u += grid, ++nunit) {
                const int tile = u / P.n_chunk, chunk = u - tile * P.n_chunk;
                const int i0 = chunk * P.chunk_items, i1 = min(P.kt, i0 + P.chunk_items);
                // one accumulator: the epilogue of the unit before must have read it
                if (nunit > 0 && !mbar_wait(sbase + A4Smem::kBarDFree, (nunit - 1) & 1, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 92, u);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                uint32_t acc = 0;
                const int nst = (i1 - i0 + kA4StageItems - 1) / kA4StageItems;
                int sidx = a4_first_stage(tile, nst);
                const int n_last = i1 - i0 - (nst - 1) * kA4StageItems;   // items of the K range's last stage
                for (int j = 0; j < nst; ++j, sidx = sidx + 1 == nst ? 0 : sidx + 1) {
                    if (!mbar_wait_probe(bar_full, full_par, P.spin_limit)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 93, mi);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t x16 = w16 + kW16;     // the stage: S weight items, then S activation items
                    if (sidx + 1 < nst || n_last == kA4StageItems) {
                        // the scales of all the stage's items first, then its MMAs
#pragma unroll
                        for (int z = 0; z < kA4StageItems; ++z) {
                            const uint32_t sfa = sf0 + uint32_t(z) * sf_cols;
                            tc_cp_sf2(sfa, sf_lo | (w16 + kCode16 + kItem16 * z), sf_hi);
                            tc_cp_sf2(sfa + 4u, sf_lo | (x16 + m2_16 + xib16 * z), sf_hi);
                            if (n_half > 1) tc_cp_sf2(sfa + 8u, sf_lo | (x16 + m2_16 + 32u + xib16 * z), sf_hi);
                        }
#pragma unroll
                        for (int z = 0; z < kA4StageItems; ++z) {
                            const uint32_t sfa = sf0 + uint32_t(z) * sf_cols;
                            tc_mma_nvf4_2(tmem_base, ab_lo | (w16 + kItem16 * z), ab_lo | (x16 + xib16 * z), ab_hi, idesc0, sfa, sfa + 4u,
                                          z == 0 ? acc : 1u);
                            if (n_half > 1)
                                tc_mma_nvf4_2(tmem_base + 128u, ab_lo | (w16 + kItem16 * z), ab_lo | (x16 + 256u + xib16 * z), ab_hi, idesc1, sfa,
                                              sfa + 8u, z == 0 ? acc : 1u);
                        }
                    } else {
                        for (int z = 0; z < n_last; ++z) {
                            const uint32_t sfa = sf0 + uint32_t(z) * sf_cols;
                            tc_cp_sf2(sfa, sf_lo | (w16 + kCode16 + kItem16 * z), sf_hi);
                            tc_cp_sf2(sfa + 4u, sf_lo | (x16 + m2_16 + xib16 * z), sf_hi);
                            if (n_half > 1) tc_cp_sf2(sfa + 8u, sf_lo | (x16 + m2_16 + 32u + xib16 * z), sf_hi);
                        }
                        for (int z = 0; z < n_last; ++z) {
                            const uint32_t sfa = sf0 + uint32_t(z) * sf_cols;
                            tc_mma_nvf4_2(tmem_base, ab_lo | (w16 + kItem16 * z), ab_lo | (x16 + xib16 * z), ab_hi, idesc0, sfa, sfa + 4u,
                                          z == 0 ? acc : 1u);
                            if (n_half > 1)
                                tc_mma_nvf4_2(tmem_base + 128u, ab_lo | (w16 + kItem16 * z), ab_lo | (x16 + 256u + xib16 * z), ab_hi, idesc1, sfa,
                                              sfa + 8u, z == 0 ? acc : 1u);
                        }
                    }
                    acc = 1;
                    tc_commit(bar_empty);
                    ++mi;
                    w16 += stage16, sf0 += sf_stage, bar_full += 8, bar_empty += 8;
                    if (w16 == ring_end16) w16 = ring16, sf0 = sf_first, full_par ^= 1u, bar_full = sbase + A4Smem::kBarFull, bar_empty = sbase + A4Smem::kBarEmpty;
                }
                if (!ok) break;
                tc_commit(sbase + A4Smem::kBarDFull);
            }
            *n_consumed = mi;
        }
        __syncwarp();
    } else {
        // ---- epilogue: accumulator -> scaled rows of y (token-major: 32 lanes store 32 consecutive n) ----
        const int q = warp & 3;
        const uint32_t lane_base = uint32_t(32 * q) << 16;
        uint32_t nunit = 0;
        bool ok = true;
        for (int u = cta; u < total_units; u += grid, ++nunit) {
            const int tile = u / P.n_chunk, chunk = u - tile * P.n_chunk;
            if (!ok) continue;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(sbase + A4Smem::kBarDFull, nunit & 1, P.spin_limit))) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 94, u);
                *abort_flag = 1;
                ok = false;
                continue;
            }
            tc_fence_after();
            const int n = tile * 128 + 32 * q + lane;
            float* part = static_cast<float*>(P.y) + size_t(chunk) * size_t(M) * size_t(P.N);
#pragma unroll 1
            for (int m0 = 0; m0 < M; m0 += 8) {
                uint32_t r[8];
                tmem_ld8(tmem_base + lane_base + uint32_t(m0), r);
                if (n < P.N) {
#pragma unroll
                    for (int z = 0; z < 8; ++z) {
                        const float v = __uint_as_float(r[z]) * (__ldg(P.g + m0 + z) * P.tensor_scale);
                        const size_t idx = size_t(m0 + z) * size_t(P.N) + size_t(n);
                        if (P.n_chunk > 1) {
                            part[idx] = v;
                        } else if (P.y_dtype == QGEMV_OUT_F32) {
                            static_cast<float*>(P.y)[idx] = v;
                        } else {
                            static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + A4Smem::kBarDFree);
        }
    }
    // ---- release tensor memory (always), after every role is done with it ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        if (*abort_flag) {
            if (lane == 0) {
                tc_commit(sbase + A4Smem::kBarDrain);
                (void)mbar_wait_probe(sbase + A4Smem::kBarDrain, 0, int64_t(1) << 16);
            }
            __syncwarp();
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, kA4TmemCols);
    } else if (threadIdx.x == 0 && *abort_flag) {
        // never leave with copies in flight: wait (bounded) for every copy that nothing consumed
        const int issued = *n_issued;
        for (int i = *n_consumed; i < issued; ++i)
            (void)mbar_wait(sbase + A4Smem::kBarFull + 8 * (i % R), uint32_t(i / R) & 1u, int64_t(1) << 20);
    }
}

}  // namespace qg
