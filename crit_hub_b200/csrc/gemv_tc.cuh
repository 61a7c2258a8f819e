// NVFP4 GEMV, batch 1..8, on the block-scaled tensor-core path: the packed weights are consumed
// exactly as stored.
//
// The CUDA-core GEMV (gemv_stream.cuh) converts every E2M1 code to f16 and multiplies it by its
// block scale in registers; measured, that instruction stream -- not HBM -- bounds it.  Here no SM
// instruction touches a weight byte: tcgen05.mma kind::mxf4nvf4 with scale_vec::4X takes E2M1
// operands with one E4M3 scale per 16 K elements, which is NVFP4 itself.  The packer
// (QGEMV_FMT_NVFP4_TC) stores a 128-row x 64-K ITEM as 4096 bytes of codes in the K-major no-swizzle
// core-matrix order of the MMA's A operand followed by 512 bytes of scales in the order
// tcgen05.cp.32x128b.warpx4 copies into tensor memory; items of one row tile are contiguous along
// K, so a bulk copy of any run of items is one contiguous range.  The kernel is then a pure
// stream: bulk copies into a shared-memory ring, one tcgen05.cp + one tcgen05.mma per item issued
// by a single thread, accumulators in tensor memory.
//
// Activations are bf16 and must stay (nearly) exact, but the B operand of this MMA kind is E2M1
// too.  Each activation row is therefore written as EIGHT E2M1 digit planes: the part of the row that
// a CTA multiplies is scaled by a power of two so that its largest magnitude lies in [2^15, 2^16)
// (the scale belongs to one accumulation, so every CTA may take it from its own K range; it depends
// on the shape and the CTA count only, never on the batch), rounded to a 16-bit integer
// magnitude n, and plane j holds the base-4 digit d_j = (n >> 2j) & 3 as the E2M1 code of d_j / 2
// (codes 0..3 are 0, 0.5, 1, 1.5) with the element's sign; the plane's block scale is the constant
// 2^(2j-6), a power of two that E4M3 holds exactly.  The eight planes of a row are eight columns of
// the MMA's N extent; their accumulators are added in plane order in the epilogue and the power of
// two is undone in fp32.  An element is exact when it lies within 2^-8 of that maximum (bf16 has 8
// significant bits) and otherwise rounded to 2^-16 of it.
//
// Work split: the linear space (row tile, item) is cut evenly over the CTAs; a CTA's range is a
// sequence of segments, each a K range of one row tile.  A segment that covers its whole tile
// stores y; otherwise the tile's first contributor collects the other CTAs' fp32 partial sums
// (flagged 8-byte hand-over slots, bounded wait) and adds them in CTA order -- a deterministic
// split along K that depends only on the shape and the CTA count.
//
// Warp roles (10 warps):
//   0     one thread issues the bulk copies of packed items (ring of stages)
//   1     allocates tensor memory; one elected lane issues tcgen05.cp / tcgen05.mma and the commits
//   2-9   convert the activations into digit planes (after the dependency wait), then run the
//         epilogues: warps 2-5 take the CTA's even segments, 6-9 the odd ones (two accumulators)
// Every wait is bounded; tensor memory is always released before the CTA exits.
#pragma once
#include "aux_kernels.cuh"
#include "gemm_skinny.cuh"
#include "gemv_stream.cuh"

namespace qg {

constexpr int kTcItemBytes = QG_TC_ITEM_BYTES;  // 4608
constexpr int kTcCodeBytes = 4096;
constexpr int kTcPlanes = 8;
constexpr int kTcConvWarps = 8;
constexpr int kTcWarpProd = 0, kTcWarpMma = 1, kTcWarpConv0 = 2;
constexpr int kTcConvThreads = 32 * kTcConvWarps;
constexpr int kTcThreads = 32 * (2 + kTcConvWarps);  // 320
constexpr int kTcMaxRing = 16;
constexpr int kTcTmemCols = 256;  // two such CTAs fit the SM's 512 columns

struct TcParams {
    const uint8_t* payload;  // items: (tile * kt_total + kt) * 4608
    const uint16_t* x;       // bf16 activations, first element of the K window
    void* y;                 // [B][N]
    float* ws;               // hand-over slots: (2 * cta) of [8][128] pairs {fp32, flag}, all zero between launches
    int32_t* status;
    int64_t spin_limit;
    float tensor_scale;
    int32_t N;               // rows of the matrix
    int32_t K;               // valid activation elements in the window
    int32_t tiles;           // ceil(N / 128)
    int32_t kt_total;        // items per row tile in the blob
    int32_t kt0, kt_len;     // the window of items this launch covers
    int32_t x_stride;        // elements between activation rows
    int32_t B, y_dtype, debug;
    int32_t npad;            // MMA N extent: 8 * B rounded up to 16
    int32_t ring, stage_items;
    int32_t x_slots;         // item slots of digit planes in shared memory
    int32_t cluster;         // CTAs per thread-block cluster (1: none).  Above 1 the launch has tiles * cluster
                             // CTAs, a cluster owns one row tile and hands partial sums over in shared memory
    unsigned long long* trace;  // optional: 16 globaltimer stamps per CTA (diagnostics), or null
    // optional L2 prefetch of the weight the caller multiplies by next (same kind of blob): CTA c pulls
    // what CTA c of that launch will stream, minus the head its own ring prefetches
    const uint8_t* pf_base;     // payload of the next weight, or null
    int32_t pf_total;           // its items (tiles * items per tile)
    int32_t pf_grid;            // CTAs of its launch
    uint32_t pf_skip;           // bytes at the head of every CTA's share to leave out
};

struct TcSmem {
    static constexpr int kBarFull = 0;      // kTcMaxRing
    static constexpr int kBarEmpty = 128;   // kTcMaxRing
    static constexpr int kBarDFull = 256;   // 2
    static constexpr int kBarDFree = 272;   // 2
    static constexpr int kBarXReady = 288;
    static constexpr int kBarDrain = 296;
    static constexpr int kTmemPtr = 304;
    static constexpr int kAbort = 308;
    static constexpr int kIssued = 312;
    static constexpr int kConsumed = 316;
    static constexpr int kRowMax = 320;     // 8 words: largest |bf16| pattern per activation row
    static constexpr int kWarpMax = 384;    // kTcConvWarps x 8 words: the same per converting warp
    static constexpr int kBarParts = 640;   // cluster mode: arrivals of the other ranks' partial sums
    static constexpr int kSfb = 1024;       // 512 bytes: block scales of the digit planes
    static constexpr int kParts = 1536;     // cluster mode: (cluster - 1) x B x 128 fp32 partial sums, rank 0 only
    __host__ __device__ static constexpr int parts_bytes(int cluster, int B) { return cluster > 1 ? (cluster - 1) * B * 512 : 0; }
    __host__ __device__ static constexpr int x_off(int cluster, int B) { return kParts + parts_bytes(cluster, B); }
    __host__ __device__ static constexpr int x_bytes(int x_slots, int npad) { return x_slots * npad * 32; }
    __host__ __device__ static constexpr int ring_off(int x_slots, int npad, int cluster, int B) {
        return (x_off(cluster, B) + x_bytes(x_slots, npad) + 127) / 128 * 128;
    }
    __host__ __device__ static constexpr int total(int x_slots, int npad, int ring, int stage_items, int cluster, int B) {
        return ring_off(x_slots, npad, cluster, B) + ring * stage_items * kTcItemBytes;
    }
    // tensor memory: two accumulators of npad columns, 4 columns of plane scales, then one 4-column
    // slot of weight block scales per ring item
    __host__ __device__ static constexpr int max_ring_items(int npad) { return (kTcTmemCols - 2 * npad - 4) / 4; }
};

// ---- tcgen05 wrappers for the block-scaled kind ---------------------------------------------------
// 32 rows x 16 bytes of shared memory -> 32 lanes x 4 columns of tensor memory, replicated into all
// four lane quarters: the scale factors of 128 rows x 4 blocks, row r at lane r % 32, column r / 32.
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// The same with the descriptor given as two 32-bit halves: the issuing thread's address arithmetic
// stays 32-bit (only the low half, which holds the address field, changes from item to item).
__device__ __forceinline__ void tc_cp_sf2(uint32_t taddr, uint32_t desc_lo, uint32_t desc_hi) {
    asm volatile("{\n .reg .b64 d;\n mov.b64 d, {%1, %2};\n tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n}" ::"r"(taddr),
                 "r"(desc_lo), "r"(desc_hi)
                 : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_2(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t ab_hi, uint32_t idesc,
                                              uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %4, [%5], [%6], p;\n}" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(ab_hi), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= (A[smem] * SFA[tmem]) * (B[smem] * SFB[tmem]), E2M1 operands, E4M3 scales per 16 K
__device__ __forceinline__ void tc_mma_nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %6, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}

// ---- thread-block cluster helpers (distributed shared memory) --------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared-memory address of `local` in the CTA of rank `rank` of this cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// bounded wait with cluster-scope acquire: the data it guards was written by other CTAs of the cluster
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int64_t spin_limit) {
    uint64_t t0 = 0;
    for (int64_t i = 0; i <= spin_limit; ++i) {
        if (i == 1) t0 = globaltimer_ns();
        if ((i & 63) == 63 && globaltimer_ns() - t0 > 2000000000ull) return false;
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
            " selp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(20000u)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// Split-K hand-over: an aligned 8-byte element {fp32 value, flag 1} written and read as one access.
__device__ __forceinline__ void st_flagged(unsigned long long* p, float v) {
    const unsigned long long w = (1ull << 32) | __float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ld_flagged(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// ---- activation digit planes ------------------------------------------------------------------------
// Exponent E such that max * 2^-E lies in [2^15, 2^16), from the largest |bf16| bit pattern.
__device__ __forceinline__ int tc_row_exponent(uint32_t m) {
    if (m == 0) return 0;
    const int ef = int(m >> 7);
    const int E = (ef == 0 ? -126 : ef - 127) - 15;
    return E < -126 ? -126 : (E > 112 ? 112 : E);  // 2^-E and 2^(E+7) both stay normal fp32 numbers
}
// 16-bit magnitude -> its eight base-4 digits, one per nibble
__device__ __forceinline__ uint32_t tc_spread(uint32_t n) {
    n = (n | (n << 8)) & 0x00FF00FFu;
    n = (n | (n << 4)) & 0x0F0F0F0Fu;
    n = (n | (n << 2)) & 0x33333333u;
    return n;
}
__device__ __forceinline__ uint32_t tc_digits(uint32_t bf, float sf) {
    const uint32_t n = min(__float2uint_rn(__uint_as_float((bf & 0x7FFFu) << 16) * sf), 65535u);
    return tc_spread(n) | (0u - ((bf >> 15) & 1u)) & 0x88888888u;
}
// Eight consecutive bf16 elements -> out[j] = the eight E2M1 codes of plane j (element i in nibble i).
__device__ __forceinline__ void tc_digits8(uint4 v, float sf, uint32_t (&out)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t a[4], b[4];  // byte q of a[p]: plane 2q of elements (2p, 2p+1); b[p]: plane 2q+1
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const uint32_t s0 = tc_digits(w[p] & 0xFFFFu, sf), s1 = tc_digits(w[p] >> 16, sf);
        a[p] = (s0 & 0x0F0F0F0Fu) | ((s1 & 0x0F0F0F0Fu) << 4);
        b[p] = ((s0 >> 4) & 0x0F0F0F0Fu) | (s1 & 0xF0F0F0F0u);
    }
    uint32_t t0 = __byte_perm(a[0], a[1], 0x5140), t1 = __byte_perm(a[2], a[3], 0x5140);
    uint32_t t2 = __byte_perm(a[0], a[1], 0x7362), t3 = __byte_perm(a[2], a[3], 0x7362);
    out[0] = __byte_perm(t0, t1, 0x5410), out[2] = __byte_perm(t0, t1, 0x7632);
    out[4] = __byte_perm(t2, t3, 0x5410), out[6] = __byte_perm(t2, t3, 0x7632);
    t0 = __byte_perm(b[0], b[1], 0x5140), t1 = __byte_perm(b[2], b[3], 0x5140);
    t2 = __byte_perm(b[0], b[1], 0x7362), t3 = __byte_perm(b[2], b[3], 0x7362);
    out[1] = __byte_perm(t0, t1, 0x5410), out[3] = __byte_perm(t0, t1, 0x7632);
    out[5] = __byte_perm(t2, t3, 0x5410), out[7] = __byte_perm(t2, t3, 0x7632);
}

// The tile's first contributor gathers the parts of CTAs c_lo + 1 .. c_hi, two activation rows at a
// time with the loads of up to eight parts in flight together, re-polling -- bounded -- what is
// missing, then adds them to `val` in CTA order and clears the slots it has read.
template <class PT>
__device__ __forceinline__ bool tc_collect(const PT& P, float (&val)[8], int Bl, int32_t c_lo, int32_t c_hi, int row,
                                           volatile int* abort_flag) {
    constexpr int KP = 8;
    uint64_t t_wait = 0;  // read on the first miss only: %globaltimer is a slow register
    unsigned long long* ws = reinterpret_cast<unsigned long long*>(P.ws) + row;
#pragma unroll
    for (int b0 = 0; b0 < 8; b0 += 2) {
        if (b0 >= Bl) break;
        const bool two = b0 + 1 < Bl;
        for (int32_t cc = c_lo + 1; cc <= c_hi; cc += KP) {
            uint32_t w0[KP], w1[KP];
            uint32_t missing = (1u << min(KP, c_hi - cc + 1)) - 1u;
            for (int64_t it = 0; missing != 0; ++it) {
#pragma unroll
                for (int z = 0; z < KP; ++z) {
                    if (!(missing >> z & 1)) continue;
                    const unsigned long long* pz = ws + size_t(2 * (cc + z)) * 1024 + b0 * 128;
                    const unsigned long long e0 = ld_flagged(pz);
                    const unsigned long long e1 = two ? ld_flagged(pz + 128) : (1ull << 32);
                    w0[z] = uint32_t(e0), w1[z] = uint32_t(e1);
                    if ((e0 >> 32) != 0 && (e1 >> 32) != 0) missing &= ~(1u << z);
                }
                if (missing != 0 && t_wait == 0) t_wait = globaltimer_ns();
                if (missing != 0 && (it >= P.spin_limit || ((it & 63) == 63 && globaltimer_ns() - t_wait > 2000000000ull))) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 66, cc);
                    *abort_flag = 1;
                    return false;
                }
            }
#pragma unroll
            for (int z = 0; z < KP; ++z) {
                if (cc + z <= c_hi) {
                    unsigned long long* pz = ws + size_t(2 * (cc + z)) * 1024 + b0 * 128;
                    val[b0] += __uint_as_float(w0[z]);
                    pz[0] = 0ull;
                    if (two) {
                        val[b0 + 1] += __uint_as_float(w1[z]);
                        pz[128] = 0ull;
                    }
                }
            }
        }
    }
    return true;
}

// S: items per ring stage (one bulk copy, one release); a stage never crosses a row-tile boundary.
template <int S>
__global__ void __launch_bounds__(kTcThreads, 2) gemv_tc_kernel(const TcParams P) {
    extern __shared__ __align__(128) unsigned char tc_smem[];
    const uint32_t sbase = smem_u32(tc_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grid = gridDim.x, cta = blockIdx.x;
    const int kt_len = P.kt_len, npad = P.npad, R = P.ring;
    const int32_t total = P.tiles * kt_len;
    const int32_t r_begin = int32_t((int64_t(cta) * total) / grid);
    const int32_t r_end = int32_t((int64_t(cta + 1) * total) / grid);
    // digit planes: slot of item u (window-relative) = (u - xs0) mod kt_len
    const int32_t n_items = r_end - r_begin;
    const int32_t xs0 = n_items >= kt_len ? 0 : r_begin % kt_len;
    const int32_t n_slots = n_items >= kt_len ? kt_len : n_items;
    const uint32_t xslot_bytes = uint32_t(npad) * 32u;
    const uint32_t xbase = sbase + uint32_t(TcSmem::x_off(P.cluster, P.B));
    const uint32_t stage_bytes = uint32_t(S) * kTcItemBytes;
    const uint32_t ring0 = sbase + uint32_t(TcSmem::ring_off(P.x_slots, npad, P.cluster, P.B));
    const uint32_t ncols = kTcTmemCols;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tc_smem + TcSmem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(tc_smem + TcSmem::kTmemPtr);
    volatile int* n_issued = reinterpret_cast<volatile int*>(tc_smem + TcSmem::kIssued);
    volatile int* n_consumed = reinterpret_cast<volatile int*>(tc_smem + TcSmem::kConsumed);
    unsigned int* rowmax = reinterpret_cast<unsigned int*>(tc_smem + TcSmem::kRowMax);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcMaxRing; ++s) {
            mbar_init(sbase + TcSmem::kBarFull + 8 * s, 1);
            mbar_init(sbase + TcSmem::kBarEmpty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(sbase + TcSmem::kBarDFull + 8 * b, 1);
            mbar_init(sbase + TcSmem::kBarDFree + 8 * b, 4);
        }
        mbar_init(sbase + TcSmem::kBarXReady, 1);
        mbar_init(sbase + TcSmem::kBarDrain, 1);
        mbar_init(sbase + TcSmem::kBarParts, P.cluster > 1 ? uint32_t(128 * (P.cluster - 1)) : 1u);
        *abort_flag = 0;
        *n_issued = 0;
        *n_consumed = 0;
        for (int b = 0; b < 16 + 8 * kTcConvWarps; ++b) reinterpret_cast<volatile unsigned int*>(rowmax)[b] = 0u;
        mbar_fence_init();
    }
    if (warp == kTcWarpMma) {
        __syncwarp();
        tmem_alloc(sbase + TcSmem::kTmemPtr, ncols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    // cluster mode: rank 0's hand-over barrier must exist before any other rank can arrive on it
    if (P.cluster > 1) cluster_sync_all();
    pdl_launch_dependents();
    if (P.trace && threadIdx.x == 0) { P.trace[cta * 16 + 0] = globaltimer_ns(); P.trace[cta * 16 + 9] = clock64(); }
    // tensor-memory columns: two accumulators, the planes' block scales, a ring of weight block scales
    const uint32_t tmem_sfb = tmem_base + 2u * uint32_t(npad);
    const uint32_t tmem_sfa0 = tmem_sfb + 4u;

    if (warp == kTcWarpProd) {
        // ================= packed-weight producer (weights never depend on the preceding kernel) =================
        // One thread runs this loop, so its dependent-instruction count per stage bounds the stream:
        // the divisions and 64-bit address arithmetic happen once per segment, a stage is a handful
        // of adds around the wait and the copy.
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            const bool drop = (P.debug & 2) != 0;  // host-set fault injection: never issue a copy
            GsWalker wk;
            wk.init(total, kt_len, cta, grid);
            GsSeg sg;
            int s = 0, issued = 0;
            uint32_t use = 0;
            bool ok = true;
            while (ok && wk.next(sg)) {
                const uint8_t* src = P.payload + (uint64_t(sg.tile) * P.kt_total + uint64_t(P.kt0 + sg.u0)) * kTcItemBytes;
                for (int32_t left = sg.u1 - sg.u0; left > 0; left -= S) {
                    if (use > 0 && !mbar_wait_probe(sbase + TcSmem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 61, sg.tile);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    const uint32_t bytes = uint32_t(min(S, left)) * kTcItemBytes;
                    if (!drop) {
                        const uint32_t bar = sbase + TcSmem::kBarFull + 8 * s;
                        mbar_arrive_expect_tx(bar, bytes);
                        bulk_g2s(ring0 + s * stage_bytes, src, bytes, bar, pol);
                        ++issued;
                    }
                    src += bytes;
                    if (++s == R) s = 0, ++use;
                }
                if (*abort_flag) break;
            }
            *n_issued = issued;
            // This launch's last copy is on its way: from here on HBM would idle through the epilogue,
            // the launch boundary and the next launch's activation conversion.  Pull the next weight
            // towards L2 meanwhile (weights are immutable, so an early prefetch is always safe).
            if (P.pf_base != nullptr && ok) {
                for (int c2 = cta; c2 < P.pf_grid; c2 += grid) {
                    uint64_t lo = (uint64_t(c2) * uint64_t(P.pf_total)) / uint64_t(P.pf_grid) * kTcItemBytes + P.pf_skip;
                    const uint64_t hi = (uint64_t(c2 + 1) * uint64_t(P.pf_total)) / uint64_t(P.pf_grid) * kTcItemBytes;
                    for (; lo < hi; lo += 32768) bulk_prefetch_l2(P.pf_base + lo, uint32_t(min(uint64_t(32768), hi - lo)));
                }
            }
        }
    } else if (warp == kTcWarpMma) {
        // ================= MMA issuer: one elected lane =================
        // A single thread: what bounds it is the length of its dependent instruction chain per stage,
        // so the loops are nested (segment, stage, item) with all divisions in the segment level.
        // Phase A copies the block scales of the prefetched stages into tensor memory (one 4-column
        // slot per ring item) while the digit planes are still being made: that needs no activations.
        // Phase B waits for the planes and issues the MMAs; from the second ring revolution on it also
        // copies each landed stage's scales first.  tcgen05.cp and tcgen05.mma of one thread execute
        // in issue order, and a ring slot's scales are rewritten only after the slot was refilled,
        // i.e. after the MMAs that read them have retired.
        if (elect_one()) {
            // E2M1 x E2M1, E4M3 scales, K-major operands, M = 128, N = npad
            const uint32_t idesc = (1u << 7) | (1u << 10) | (uint32_t(npad >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            // descriptors differ in their 14-bit address field only (shared memory is below 256 KB)
            const uint64_t d_ab = smem_desc(0, 128, 256), d_sf = smem_desc(0, 0, 128);
            const uint32_t ab_hi = uint32_t(d_ab >> 32), ab_lo = uint32_t(d_ab), sf_hi = uint32_t(d_sf >> 32), sf_lo = uint32_t(d_sf);
            // In a cluster launch a CTA's shared-memory addresses carry its window's base above bit 18;
            // the descriptors take the 14-bit field (address within the CTA's window, in 16-byte units).
            const uint32_t x_lo0 = ab_lo | ((xbase >> 4) & 0x3FFFu);
            const uint32_t xslot16 = xslot_bytes >> 4, stage16 = stage_bytes >> 4, ring16 = (ring0 >> 4) & 0x3FFFu;
            constexpr uint32_t kItem16 = kTcItemBytes >> 4, kCode16 = kTcCodeBytes >> 4;
            // block scales of the items of ring slot `slot` -> its tensor-memory columns
            auto copy_scales = [&](uint32_t item16, uint32_t sfa, int cnt) {
                if (cnt == S) {
#pragma unroll
                    for (int i = 0; i < S; ++i) tc_cp_sf2(sfa + 4u * i, sf_lo | (item16 + kCode16 + kItem16 * i), sf_hi);
                } else {
                    for (int i = 0; i < cnt; ++i) tc_cp_sf2(sfa + 4u * i, sf_lo | (item16 + kCode16 + kItem16 * i), sf_hi);
                }
            };
            bool ok = true;
            int a_done = 0;  // stages whose scales phase A has copied
            {
                GsWalker wk;
                wk.init(total, kt_len, cta, grid);
                GsSeg sg;
                while (ok && a_done < R && wk.next(sg)) {
                    for (int32_t left = sg.u1 - sg.u0; left > 0 && a_done < R; left -= S) {
                        if (!mbar_wait_probe(sbase + TcSmem::kBarFull + 8 * a_done, 0, P.spin_limit)) {
                            report(P.status, QGEMV_ERR_TIMEOUT, 64, a_done);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        if (P.trace && a_done == 0) P.trace[cta * 16 + 4] = clock64();
                        copy_scales(ring16 + uint32_t(a_done) * stage16, tmem_sfa0 + uint32_t(a_done) * (4u * S), min(S, left));
                        ++a_done;
                    }
                }
            }
            // everything the first segment needs is computed before the wait for the planes
            GsWalker wk;
            wk.init(total, kt_len, cta, grid);
            GsSeg sg;
            bool have = wk.next(sg);
            uint32_t nseg = 0, full_par = 0;
            uint32_t item16 = ring16, sfa = tmem_sfa0, bar_full = sbase + TcSmem::kBarFull, bar_empty = sbase + TcSmem::kBarEmpty;
            const uint32_t ring_end16 = ring16 + uint32_t(R) * stage16;
            if (ok && !mbar_wait(sbase + TcSmem::kBarXReady, 0, P.spin_limit)) {
                report(P.status, QGEMV_ERR_TIMEOUT, 62, 0);
                *abort_flag = 1;
                ok = false;
            }
            int mi = 0;  // stages issued
            if (ok) {
                tc_fence_after();
                if (P.trace) P.trace[cta * 16 + 3] = clock64();
                tc_cp_sf2(tmem_sfb, sf_lo | (((sbase + TcSmem::kSfb) >> 4) & 0x3FFFu), sf_hi);
                for (; ok && have; have = wk.next(sg)) {
                    // the accumulator is free once the epilogue of the segment before last has read it
                    if (nseg >= 2 &&
                        !mbar_wait_probe(sbase + TcSmem::kBarDFree + 8 * (nseg & 1), ((nseg >> 1) - 1) & 1, P.spin_limit)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 63, int(nseg));
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (nseg & 1) * uint32_t(npad);
                    uint32_t acc = 0;  // the segment's first MMA overwrites D
                    int32_t slot = sg.u0 - xs0;
                    if (slot < 0) slot += kt_len;
                    uint32_t x_lo = x_lo0 + uint32_t(slot) * xslot16;
                    for (int32_t left = sg.u1 - sg.u0; left > 0; left -= S) {
                        if (mi >= a_done) {
                            if (!mbar_wait_probe(bar_full, full_par, P.spin_limit)) {
                                report(P.status, QGEMV_ERR_TIMEOUT, 64, mi);
                                *abort_flag = 1;
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            copy_scales(item16, sfa, min(S, left));
                        }
                        if (left >= S) {
#pragma unroll
                            for (int i = 0; i < S; ++i)
                                tc_mma_nvf4_2(tmem_d, ab_lo | (item16 + kItem16 * i), x_lo + xslot16 * i, ab_hi, idesc, sfa + 4u * i,
                                              tmem_sfb, i == 0 ? acc : 1u);
                        } else {
                            for (int i = 0; i < left; ++i)
                                tc_mma_nvf4_2(tmem_d, ab_lo | (item16 + kItem16 * i), x_lo + xslot16 * i, ab_hi, idesc, sfa + 4u * i,
                                              tmem_sfb, i == 0 ? acc : 1u);
                        }
                        acc = 1;
                        x_lo += xslot16 * S;
                        tc_commit(bar_empty);  // the stage is reusable once these retire
                        ++mi;
                        item16 += stage16, sfa += 4u * S, bar_full += 8, bar_empty += 8;
                        if (item16 == ring_end16) {
                            item16 = ring16, sfa = tmem_sfa0, full_par ^= 1u;
                            bar_full = sbase + TcSmem::kBarFull, bar_empty = sbase + TcSmem::kBarEmpty;
                        }
                    }
                    if (!ok) break;
                    tc_commit(sbase + TcSmem::kBarDFull + 8 * (nseg & 1));
                    ++nseg;
                }
                if (P.trace) P.trace[cta * 16 + 5] = clock64();
            }
            *n_consumed = mi;
        }
        __syncwarp();
    } else {
        // ================= activation digit planes, then the epilogues =================
        const int ct = threadIdx.x - 32 * kTcWarpConv0;  // 0..255
        const int Bl = P.B;
        unsigned int* wmax = reinterpret_cast<unsigned int*>(tc_smem + TcSmem::kWarpMax) + (warp - kTcWarpConv0) * 8;
        // block scales of the planes: column n = 8 b + j carries 2^(2j - 6) in all four K blocks
        if (ct < 128) {
            const int n = ct, j = n & 7;
            const uint32_t byte = n < 8 * Bl ? uint32_t(2 * j + 1) << 3 : 0u;
            *reinterpret_cast<volatile uint32_t*>(tc_smem + TcSmem::kSfb + (n & 31) * 16 + (n >> 5) * 4) = byte * 0x01010101u;
        }
        pdl_wait();  // activations come from the preceding kernel; y and the hand-over slots may still be in use by it
        if (P.trace && ct == 0) { P.trace[cta * 16 + 1] = clock64(); P.trace[cta * 16 + 10] = globaltimer_ns(); }
        // ---- digit planes of the items this CTA multiplies.  Work unit w = ((row b) * n_slots + slot) * 8
        // + octet: eight consecutive elements, one 16-byte load.  One pass loads and finds the row maxima
        // (the first four units of a thread stay in registers), a second one converts. ----
        const int n_work = n_slots * Bl * 8;
        constexpr int kKeep = 4;
        auto unit_src = [&](int wu, int& b, uint32_t& dst) -> uint4 {
            const int o = wu & 7, sb = wu >> 3;
            b = sb / n_slots;
            const int slot = sb - b * n_slots;
            int32_t u = slot + xs0;
            if (u >= kt_len) u -= kt_len;
            const int k0 = u * 64 + o * 8;
            // plane j of (slot, row b): 16 bytes per 32 elements at + (o / 4) * 128 + j * 16; this octet's word (o % 4)
            dst = xbase + uint32_t(slot) * xslot_bytes + uint32_t(b) * 256u + uint32_t(o >> 2) * 128u + uint32_t(o & 3) * 4u;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (k0 + 8 <= P.K) v = *reinterpret_cast<const uint4*>(P.x + int64_t(b) * P.x_stride + k0);
            return v;
        };
        auto unit_max = [&](const uint4& v) {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t m = 0;
#pragma unroll
            for (int z = 0; z < 4; ++z) {
                m = max(m, w[z] & 0x7FFFu);
                m = max(m, (w[z] >> 16) & 0x7FFFu);
            }
            return m;
        };
        auto row_max = [&](int b) {
            const unsigned int* all = reinterpret_cast<const unsigned int*>(tc_smem + TcSmem::kWarpMax);
            uint32_t m = 0;
#pragma unroll
            for (int w = 0; w < kTcConvWarps; ++w) m = max(m, all[w * 8 + b]);
            return m;
        };
        auto store_unit = [&](int b, uint32_t dst, const uint4& v) {
            const float sf = pow2i(-tc_row_exponent(row_max(b)));
            uint32_t pl[8];
            tc_digits8(v, sf, pl);
#pragma unroll
            for (int j = 0; j < 8; ++j) asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + j * 16), "r"(pl[j]) : "memory");
        };
        uint4 keep[kKeep];
        int kb[kKeep];
        uint32_t kdst[kKeep];
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int wu = ct + i * kTcConvThreads;
            kb[i] = 0, kdst[i] = 0;
            keep[i] = make_uint4(0, 0, 0, 0);
            if (wu < n_work) keep[i] = unit_src(wu, kb[i], kdst[i]);
        }
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const uint32_t m = unit_max(keep[i]);
            if (m) atomicMax(wmax + kb[i], m);
        }
        for (int wu = ct + kKeep * kTcConvThreads; wu < n_work; wu += kTcConvThreads) {
            int b;
            uint32_t dst;
            const uint32_t m = unit_max(unit_src(wu, b, dst));
            if (m) atomicMax(wmax + b, m);
        }
        named_bar_sync(1, kTcConvThreads);
        if (ct < 8) rowmax[ct] = row_max(ct);
#pragma unroll
        for (int i = 0; i < kKeep; ++i)
            if (ct + i * kTcConvThreads < n_work) store_unit(kb[i], kdst[i], keep[i]);
        for (int wu = ct + kKeep * kTcConvThreads; wu < n_work; wu += kTcConvThreads) {
            int b;
            uint32_t dst;
            const uint4 v = unit_src(wu, b, dst);
            store_unit(b, dst, v);
        }
        fence_proxy_async_smem();  // the planes are read by the tensor core (async proxy)
        named_bar_sync(1, kTcConvThreads);
        if (ct == 0) mbar_arrive(sbase + TcSmem::kBarXReady);
        if (P.trace && ct == 0) P.trace[cta * 16 + 2] = clock64();

        // ---- epilogues: group g takes the segments with nseg % 2 == g; this warp owns lane quarter q ----
        const int g = (warp - kTcWarpConv0) >> 2, q = warp & 3;
        const uint32_t lane_base = uint32_t(32 * q) << 16;
        const int row = 32 * q + lane;
        GsWalker wk;
        wk.init(total, kt_len, cta, grid);
        GsSeg sg;
        uint32_t nseg = 0;
        float scale[8];
#pragma unroll
        for (int b = 0; b < 8; ++b) scale[b] = b < Bl ? P.tensor_scale * pow2i(tc_row_exponent(rowmax[b]) + 7) : 0.f;
        while (wk.next(sg)) {
            if (int(nseg & 1) != g) {
                ++nseg;
                continue;
            }
            // a partial segment's bookkeeping does not need the accumulator: do it while the MMAs run
            const bool whole = sg.u0 == 0 && sg.u1 == kt_len;
            int32_t c_lo = 0, c_hi = 0;
            if (!whole) {
                c_lo = int32_t(cta_of(int64_t(sg.tile) * kt_len, total, grid));
                c_hi = int32_t(cta_of(int64_t(sg.tile + 1) * kt_len - 1, total, grid));
            }
            if (!__all_sync(0xFFFFFFFFu, mbar_wait_probe(sbase + TcSmem::kBarDFull + 8 * g, (nseg >> 1) & 1, P.spin_limit))) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 65, int(nseg));
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            if (P.trace && lane == 0 && q == 0) P.trace[cta * 16 + 6] = clock64();  // the last one stays
            float val[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                val[b] = 0.f;
                if (b < Bl) {
                    uint32_t r[8];
                    tmem_ld8(tmem_base + lane_base + uint32_t(g * npad + 8 * b), r);
                    float a = __uint_as_float(r[0]);
#pragma unroll
                    for (int j = 1; j < 8; ++j) a += __uint_as_float(r[j]);
                    val[b] = a * scale[b];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + TcSmem::kBarDFree + 8 * g);  // the accumulator may be overwritten
            const int n = sg.tile * 128 + row;
            auto store_row = [&](const float (&v)[8]) {
                if (n < P.N) {
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        if (b < Bl) {
                            const int64_t idx = int64_t(b) * P.N + n;
                            if (P.y_dtype == QGEMV_OUT_F32) {
                                static_cast<float*>(P.y)[idx] = v[b];
                            } else {
                                static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(v[b]);
                            }
                        }
                    }
                }
            };
            if (whole) {
                store_row(val);
            } else if (P.cluster > 1) {
                // The cluster owns this row tile and every CTA of it has exactly this one segment: the
                // partial sums travel through rank 0's shared memory and arrive on its barrier; rank 0
                // adds them in rank order and stores.  No global-memory round trip.  Every thread
                // releases its own stores with its own arrival (one arrival per warp after a warp
                // barrier left some rows unwritten when rank 0 read them, and rank 0 gone when they
                // landed).
                const uint32_t rank = cluster_ctarank();
                if (rank != uint32_t(cta % P.cluster)) {
                    // not launched as the clusters the host planned: touch nobody's shared memory
                    if (lane == 0) report(P.status, QGEMV_ERR_BOUNDS, 68, int(rank));
                    *abort_flag = 1;
                    break;
                }
                if (rank != 0) {
                    const uint32_t dst = cluster_map(sbase + TcSmem::kParts, 0) + ((rank - 1) * uint32_t(Bl) * 128u + uint32_t(row)) * 4u;
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (b < Bl) st_cluster_f32(dst + b * 512, val[b]);
                    mbar_arrive_cluster(cluster_map(sbase + TcSmem::kBarParts, 0));
                } else {
                    if (!__all_sync(0xFFFFFFFFu, mbar_wait_cluster(sbase + TcSmem::kBarParts, 0, P.spin_limit))) {
                        if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 67, sg.tile);
                        *abort_flag = 1;
                        break;
                    }
                    const float* parts = reinterpret_cast<const float*>(tc_smem + TcSmem::kParts) + row;
                    for (int r = 1; r < P.cluster; ++r) {
#pragma unroll
                        for (int b = 0; b < 8; ++b)
                            if (b < Bl) val[b] += parts[((r - 1) * Bl + b) * 128];
                    }
                    store_row(val);
                }
            } else if (cta != c_lo) {
                // Partial, and not the tile's first contributor: hand the fp32 sums to it.  Every later
                // contributor starts its range inside this tile, so the tile is its first segment and
                // the part goes to its slot 0.  A slot element is the 8-byte pair {value, 1}: the
                // arrival flag travels in the same store as the data, so there is no fence, no counter
                // and no round trip on this side.
                unsigned long long* slot = reinterpret_cast<unsigned long long*>(P.ws) + size_t(2 * cta) * 1024 + row;
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    if (b < Bl) st_flagged(slot + b * 128, val[b]);
            } else {
                // The first contributor (for which the tile is the last segment of its range) adds the
                // parts in CTA order -- a fixed order, whatever the arrival order -- as they arrive,
                // clears every slot it has read (the next launch finds them empty) and stores the rows.
                // The loads of up to eight parts are in flight together; the wait is bounded.
                const bool ok = tc_collect(P, val, Bl, c_lo, c_hi, row, abort_flag);
                if (ok) store_row(val);
            }
            ++nseg;
        }
        if (P.trace && lane == 0 && g == 0 && q == 0) { P.trace[cta * 16 + 8] = clock64(); P.trace[cta * 16 + 11] = globaltimer_ns(); }
    }
    // ---- release tensor memory (always), after every role is done with it ----
    tc_fence_before();
    __syncthreads();
    if (P.trace && threadIdx.x == 0) P.trace[cta * 16 + 7] = globaltimer_ns();
    if (warp == kTcWarpMma) {
        __syncwarp();
        if (*abort_flag) {
            // let whatever MMAs were issued retire before the columns are handed back (bounded)
            if (lane == 0) {
                tc_commit(sbase + TcSmem::kBarDrain);
                (void)mbar_wait_probe(sbase + TcSmem::kBarDrain, 0, int64_t(1) << 16);
            }
            __syncwarp();
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, ncols);
    } else if (threadIdx.x == 0 && *abort_flag) {
        // never leave with copies in flight: wait (bounded) for every copy that nothing consumed
        const int issued = *n_issued;
        for (int i = *n_consumed; i < issued; ++i)
            (void)mbar_wait(sbase + TcSmem::kBarFull + 8 * (i % R), uint32_t(i / R) & 1u, int64_t(1) << 20);
    }
}

// Parity hook for the tensor-core layout: one thread per (row, 16-element block), the conversion
// instructions of the CUDA-core kernels (cvt.e2m1x2, cvt.e4m3x2, one f16x2 multiply: exact), then
// fp32 times the tensor scale.
__global__ void dequant_tc_kernel(const uint8_t* payload, float tensor_scale, int32_t N, int32_t K, int32_t kt_total,
                                  float* out) {
    const int64_t id = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t blocks_per_row = K / 16;
    const int64_t n = id / blocks_per_row;
    if (n >= N) return;
    const int kbg = int(id - n * blocks_per_row);  // block index along K
    const int tile = int(n >> 7), row = int(n & 127), kt = kbg >> 2, kb = kbg & 3;
    const uint8_t* item = payload + (uint64_t(tile) * kt_total + kt) * kTcItemBytes;
    int hi;
    const uint2 cw = *reinterpret_cast<const uint2*>(item + qg_tc_code_offset(row, kb * 16, &hi));
    const uint32_t sbyte = item[qg_tc_scale_offset(row, kb)];
    uint32_t s2, unused;
    cvt_e4m3x4(sbyte | (sbyte << 8), s2, unused);  // (scale, scale) as f16x2
    const uint32_t w[2] = {cw.x, cw.y};
#pragma unroll
    for (int z = 0; z < 2; ++z) {
        uint32_t a[4];
        cvt_e2m1x8(w[z], a[0], a[1], a[2], a[3]);  // byte i -> elements 2i (low half), 2i+1 (high half)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t pr = hmul2(a[i], s2);
            const int64_t k = int64_t(kbg) * 16 + 8 * z + 2 * i;
            out[n * K + k] = __fmul_rn(h_lo(pr), tensor_scale);
            out[n * K + k + 1] = __fmul_rn(h_hi(pr), tensor_scale);
        }
    }
}

}  // namespace qg
