// Skinny GEMM / short prefill on the 5th-generation tensor cores (tcgen05, TMEM accumulators):
//     Y[M][N] = X[M][K] * dequant(W)^T,   M = 16 .. 256 tokens (multiple of 16).
//
// "W4A16-exact" variant: the packed NVFP4 / FP8 weights are dequantised to f16 tiles in shared
// memory (the f16 value of code * block scale is exact) and multiplied with f16 activations by
// tcgen05.mma kind::f16 with fp32 accumulators in tensor memory.  Activations are converted
// bf16 -> f16 once per call by x_prep_kernel, scaled per token row by a power of two exactly as
// in the GEMV kernels, and laid out in the MMA's canonical K-major tile order so that one bulk
// copy brings a whole [M x 64] tile.  (The block-scaled kinds, mxf4nvf4 / f8f6f4, need FP4 / FP8
// activations and cannot meet a 2e-3 bound against unquantised activations; they are a different
// operator and are not what this kernel computes.)
//
// One CTA per 128 weight rows (8 panels); MMA shape M=128 (weight rows) x N=M_tokens x K=16, four
// MMAs per 64-wide K step.  Warp roles:
//   warps 0-3  dequantise the 8 panels of a stage into the canonical A tile (no swizzle: core
//              matrices of 8 rows x 16 bytes), then fence the async proxy and signal; at the end
//              they read the accumulator from TMEM (each warp its 32 lanes) and store Y
//   warp 4     one thread issues the bulk (TMA) copies: 8 x 576 (or 1024) bytes of packed weights
//              and one activation tile per stage
//   warp 5     allocates TMEM; one thread issues tcgen05.mma and commits to the stage's mbarrier
// Every wait is bounded; TMEM is always released before the CTA exits.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemv_kernel.cuh"

namespace qg {

constexpr int kGsStages = 3;
constexpr int kGsThreads = 192;          // 6 warps
constexpr int kGsATileBytes = 128 * 128; // 128 rows x 64 f16
constexpr int kGsMaxM = 256;

struct GsParams {
    const uint8_t* payload;   // packed weight
    const float* chan_scale;  // FP8 channel scales
    float tensor_scale;
    const uint8_t* xt;        // f16 activation tiles: [units][M/8][8 k-chunks][8 rows][8 elems]
    const int32_t* xexp;      // per token row: exponent E (x was scaled by 2^-E)
    void* y;                  // [M][N]
    int32_t y_dtype;
    int32_t N, K, M;
    int32_t units;            // K / 64
    int32_t* status;
    int64_t spin_limit;
    int32_t debug;
};

struct GsSmem {
    static constexpr int kBarFull = 0;     // kGsStages
    static constexpr int kBarAReady = 32;  // kGsStages
    static constexpr int kBarEmpty = 64;   // kGsStages
    static constexpr int kBarDone = 96;
    static constexpr int kTmemPtr = 104;
    static constexpr int kAbort = 108;
    static constexpr int kStage0 = 1024;
    // stage: [packed weights 8 panels][activation tile M*128][A tile 16 KB]
    __host__ __device__ static constexpr int packed_bytes(int unit_bytes) { return 8 * unit_bytes; }
    __host__ __device__ static constexpr int stage_bytes(int unit_bytes, int M) {
        return ((packed_bytes(unit_bytes) + 1023) / 1024) * 1024 + M * 128 + kGsATileBytes;
    }
    __host__ __device__ static constexpr int total(int unit_bytes, int M) {
        return kStage0 + kGsStages * stage_bytes(unit_bytes, M);
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
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// K-major, no swizzle: core matrix = 8 rows x 16 bytes (128 contiguous bytes); the next 16-byte K
// chunk is LBO bytes away, the next 8-row group SBO bytes away.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return uint64_t((addr >> 4) & 0x3FFFu) | (uint64_t((lbo >> 4) & 0x3FFFu) << 16) |
           (uint64_t((sbo >> 4) & 0x3FFFu) << 32) | (uint64_t(1) << 46);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Activation preparation: one CTA per token row.  bf16 -> f16 scaled by 2^-E (row maximum into
// [2^14, 2^15)), written in tile order: element (m, k) of unit u = k / 64 goes to
//   xt + u * (M*128) + (m/8)*1024 + ((k%64)/8)*128 + (m%8)*16 + (k%8)*2.
__global__ void x_prep_kernel(const uint16_t* x, int M, int K, uint8_t* xt, int32_t* xexp) {
    __shared__ unsigned int smax;
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    if (threadIdx.x == 0) smax = 0u;
    __syncthreads();
    const uint16_t* xr = x + int64_t(m) * K;
    unsigned int mx = 0;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(xr + k));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int z = 0; z < 4; ++z) {
            mx = max(mx, w[z] & 0x7FFFu);
            mx = max(mx, (w[z] >> 16) & 0x7FFFu);
        }
    }
    mx = __reduce_max_sync(0xFFFFFFFFu, mx);
    if ((threadIdx.x & 31) == 0) atomicMax(&smax, mx);
    __syncthreads();
    const int E = row_exponent(smax);
    if (threadIdx.x == 0) xexp[m] = E;
    const float sf = pow2i(-E);
    const size_t tile_bytes = size_t(M) * 128;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(xr + k));
        uint4 o;
        o.x = pack_f16x2(__uint_as_float(v.x << 16) * sf, __uint_as_float(v.x & 0xFFFF0000u) * sf);
        o.y = pack_f16x2(__uint_as_float(v.y << 16) * sf, __uint_as_float(v.y & 0xFFFF0000u) * sf);
        o.z = pack_f16x2(__uint_as_float(v.z << 16) * sf, __uint_as_float(v.z & 0xFFFF0000u) * sf);
        o.w = pack_f16x2(__uint_as_float(v.w << 16) * sf, __uint_as_float(v.w & 0xFFFF0000u) * sf);
        const int u = k >> 6, kc = (k & 63) >> 3;
        *reinterpret_cast<uint4*>(xt + size_t(u) * tile_bytes + size_t(m >> 3) * 1024 + kc * 128 + (m & 7) * 16) = o;
    }
}

// Dequantises one packed unit of one panel (lane-ordered MMA-fragment layout) into the canonical
// A tile: this lane's rows g and g+8 of the panel, four 4-element runs per row.
template <int FMT>
__device__ __forceinline__ void dequant_unit_to_tile(uint32_t unit, uint32_t a_tile, int panel, int lane) {
    const int g = lane >> 2, t = lane & 3;
    uint32_t a[4][4];  // [tile T][register jb]: f16x2 = (block 2*pr, block 2*pr+1)
    if (FMT == QGEMV_FMT_NVFP4) {
        const uint4 cw = lds128(unit + lane * 16);
        const uint2 sw = lds64(unit + 512 + g * 8);
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
        const uint4 v0 = lds128(unit + lane * 16);
        const uint4 v1 = lds128(unit + 512 + lane * 16);
        cvt_e4m3x4(v0.x, a[0][0], a[0][1]);
        cvt_e4m3x4(v0.y, a[0][2], a[0][3]);
        cvt_e4m3x4(v0.z, a[1][0], a[1][1]);
        cvt_e4m3x4(v0.w, a[1][2], a[1][3]);
        cvt_e4m3x4(v1.x, a[2][0], a[2][1]);
        cvt_e4m3x4(v1.y, a[2][2], a[2][3]);
        cvt_e4m3x4(v1.z, a[3][0], a[3][1]);
        cvt_e4m3x4(v1.w, a[3][2], a[3][3]);
    }
    // element (row = g + 8*rowhi, block kb = 2*pr + h, e = 4*t + 2*sub + r) is half h of a[2*pr+sub][rowhi + 2*r]
#pragma unroll
    for (int rowhi = 0; rowhi < 2; ++rowhi) {
        const uint32_t row_base = a_tile + uint32_t(2 * panel + rowhi) * 1024u + uint32_t(g) * 16u + uint32_t(t & 1) * 8u;
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t sel = h ? 0x7632u : 0x5410u;
                const uint32_t lo = prmt(a[2 * pr][rowhi], a[2 * pr][rowhi + 2], sel);          // e = 4t, 4t+1
                const uint32_t hi = prmt(a[2 * pr + 1][rowhi], a[2 * pr + 1][rowhi + 2], sel);  // e = 4t+2, 4t+3
                const int kc = 2 * (2 * pr + h) + (t >> 1);  // 16-byte K chunk inside the 64-wide step
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(row_base + uint32_t(kc) * 128u), "r"(lo), "r"(hi)
                             : "memory");
            }
        }
    }
}

template <int FMT>
__global__ void __launch_bounds__(kGsThreads, 1) gemm_skinny_kernel(const GsParams P) {
    constexpr int kUnitBytes = FmtTraits<FMT>::kUnitBytes;
    extern __shared__ __align__(128) unsigned char gs_smem[];
    const uint32_t sbase = smem_u32(gs_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int M = P.M;
    const int stage_bytes = GsSmem::stage_bytes(kUnitBytes, M);
    const int x_off = ((GsSmem::packed_bytes(kUnitBytes) + 1023) / 1024) * 1024;
    const int a_off = x_off + M * 128;
    uint32_t ncols = 32;
    while (int(ncols) < M) ncols <<= 1;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gs_smem + GsSmem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(gs_smem + GsSmem::kTmemPtr);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGsStages; ++s) {
            mbar_init(sbase + GsSmem::kBarFull + 8 * s, 1);
            mbar_init(sbase + GsSmem::kBarAReady + 8 * s, 4);
            mbar_init(sbase + GsSmem::kBarEmpty + 8 * s, 1);
        }
        mbar_init(sbase + GsSmem::kBarDone, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) tmem_alloc(sbase + GsSmem::kTmemPtr, ncols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    pdl_launch_dependents();
    const int n0 = blockIdx.x * 128;  // first weight row of this CTA
    const int panel0 = n0 / 16;
    const int units = P.units;

    if (warp == 4) {
        // ================= producer =================
        if (lane == 0 && !(P.debug & 2)) {
            const uint64_t pol = policy_evict_first();
            pdl_wait();  // the activation tiles come from x_prep_kernel
            const uint32_t x_bytes = uint32_t(M) * 128u;
            for (int u = 0; u < units; ++u) {
                const int s = u % kGsStages;
                const uint32_t use = uint32_t(u / kGsStages);
                if (use > 0 && !mbar_wait(sbase + GsSmem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 41, u);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t bar = sbase + GsSmem::kBarFull + 8 * s;
                const uint32_t st = sbase + GsSmem::kStage0 + s * stage_bytes;
                mbar_arrive_expect_tx(bar, 8u * kUnitBytes + x_bytes);
                for (int p = 0; p < 8; ++p)
                    bulk_g2s(st + p * kUnitBytes,
                             P.payload + (uint64_t(panel0 + p) * units + u) * kUnitBytes, kUnitBytes, bar, pol);
                bulk_g2s(st + x_off, P.xt + uint64_t(u) * x_bytes, x_bytes, bar, pol);
            }
        }
    } else if (warp == 5) {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (uint32_t(M >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            bool ok = true;
            for (int u = 0; u < units && ok; ++u) {
                const int s = u % kGsStages;
                if (!mbar_wait(sbase + GsSmem::kBarAReady + 8 * s, uint32_t(u / kGsStages) & 1, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 42, u);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t st = sbase + GsSmem::kStage0 + s * stage_bytes;
#pragma unroll
                for (int j = 0; j < 4; ++j) {  // four K=16 steps: two 16-byte chunks each
                    const uint64_t da = smem_desc(st + a_off + j * 256, 128, 1024);
                    const uint64_t db = smem_desc(st + x_off + j * 256, 128, 1024);
                    tc_mma_f16(tmem_base, da, db, idesc, (u > 0 || j > 0) ? 1u : 0u);
                }
                tc_commit(sbase + GsSmem::kBarEmpty + 8 * s);  // stage reusable once these MMAs retire
            }
            tc_commit(sbase + GsSmem::kBarDone);
        }
    } else {
        // ================= dequantisation warps, then epilogue =================
        bool ok = true;
        for (int u = 0; u < units && ok; ++u) {
            const int s = u % kGsStages;
            const uint32_t use = uint32_t(u / kGsStages);
            // the A tile of this stage is free once the MMAs of its previous use retired
            if (use > 0 && !mbar_wait(sbase + GsSmem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 43, u);
                *abort_flag = 1;
                ok = false;
                break;
            }
            if (!mbar_wait(sbase + GsSmem::kBarFull + 8 * s, use & 1, P.spin_limit)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 44, u);
                *abort_flag = 1;
                ok = false;
                break;
            }
            const uint32_t st = sbase + GsSmem::kStage0 + s * stage_bytes;
            dequant_unit_to_tile<FMT>(st + (2 * warp) * kUnitBytes, st + a_off, 2 * warp, lane);
            dequant_unit_to_tile<FMT>(st + (2 * warp + 1) * kUnitBytes, st + a_off, 2 * warp + 1, lane);
            fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + GsSmem::kBarAReady + 8 * s);
        }
        // ---- epilogue: warp w reads TMEM lanes [32w, 32w+32) = weight rows n0 + 32w + lane ----
        ok = __all_sync(0xFFFFFFFFu, ok);
        const bool done = ok && __all_sync(0xFFFFFFFFu, mbar_wait(sbase + GsSmem::kBarDone, 0, P.spin_limit));
        if (done) {
            tc_fence_after();
            const int n = n0 + 32 * warp + lane;
            float rs = (FMT == QGEMV_FMT_NVFP4) ? P.tensor_scale : P.chan_scale[n];
            for (int c = 0; c < M; c += 8) {
                uint32_t v[8];
                tmem_ld8(tmem_base + (uint32_t(32 * warp) << 16) + uint32_t(c), v);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int m = c + i;
                    const float val = __uint_as_float(v[i]) * rs * pow2i(__ldg(P.xexp + m));
                    const int64_t idx = int64_t(m) * P.N + n;
                    if (P.y_dtype == QGEMV_OUT_F32) {
                        static_cast<float*>(P.y)[idx] = val;
                    } else {
                        static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(val);
                    }
                }
            }
            tc_fence_before();
        } else if (ok) {
            if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 45, 0);
            *abort_flag = 1;
        }
    }
    // ---- release TMEM (always), after every role is done with it ----
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        if (*abort_flag) (void)mbar_wait(sbase + GsSmem::kBarDone, 0, int64_t(1) << 16);  // let issued MMAs retire
        tc_fence_after();
        tmem_dealloc(tmem_base, ncols);
    }
}

}  // namespace qg
