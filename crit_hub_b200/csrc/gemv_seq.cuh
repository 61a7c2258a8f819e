// A SEQUENCE of NVFP4 GEMVs (tensor-core layout) as ONE persistent launch: the projections of a
// decode step, executed in order, each allowed to read what the one before it wrote.
//
// Launched one by one, each GEMV of a decode layer pays a serial chain that no weight byte overlaps:
// the previous grid's last partial sums, the launch boundary, the activation conversion, the first
// MMAs -- about 5 us, four times per layer, against 19 us of HBM time.  A launch can only prefetch
// what its own ring holds while it waits.  Here one grid of one CTA per SM walks the whole job
// list.  The producer thread never stops at a job boundary: while the CTA's other warps finish job
// j (epilogue, grid-wide barrier, digit planes of job j+1), it already streams the items of job
// j+1, j+2, ... into a ring that takes most of the SM's shared memory, so HBM stays busy across the
// boundary and the MMAs of the next job find their first ~190 KB per SM waiting.
//
// Per job the arithmetic is gemv_tc.cuh's: weights consumed as stored by tcgen05.mma
// kind::mxf4nvf4, activations as eight E2M1 digit planes scaled per CTA range, split along K over
// the CTAs with a deterministic hand-over to each row tile's first contributor.
//
// Between jobs: every CTA, once its own results of job j are stored, bumps a global counter with
// release semantics; before converting the activations of job j+1 one thread per CTA polls --
// bounded -- until all CTAs have arrived (acquire), then the CTA's converting warps synchronise.
// The CTAs wait on one another, so the launch is cooperative (all CTAs co-resident).
//
// Split along K without a wait: a CTA that holds only part of a row tile stores its fp32 partial
// sums in its own slot of a parts buffer (double-buffered by job parity) and moves on.  The tile's
// first contributor adds the parts in CTA order -- a fixed order -- and stores the rows AFTER the
// barrier, when every part is known to be there, and after it has handed the next job's digit
// planes to the tensor core: the sum is off the critical path and polls nothing.  Only when the
// next job reads or overwrites this job's output (the host compares the address ranges) is the sum
// done first, followed by one more barrier.
//
// Warp roles as in gemv_tc.cuh: 0 producer, 1 MMA issuer, 2-9 digit planes + epilogues.
#pragma once
#include "gemv_tc.cuh"

namespace qg {

struct SeqJob {               // 64 bytes, device memory
    const uint8_t* payload;   // items of the weight: (tile * kt + item) * 4608
    const uint16_t* x;        // bf16 [B][K]
    void* y;                  // [B][N]
    float tensor_scale;
    int32_t N, K;
    int32_t tiles, kt;        // ceil(N / 128), ceil(K / 64)
    int32_t x_stride;         // elements between activation rows
    int32_t y_dtype;
    int32_t flags;            // bit 0: this job's x or y overlaps the previous job's y -- finish that one first
    int32_t pad;
};
static_assert(sizeof(SeqJob) == 64, "SeqJob layout");

struct SeqParams {
    const SeqJob* jobs;
    float* ws;                  // parts buffer: [job parity][2 * cta + which][8][128] fp32 partial sums
    unsigned int* barrier;      // [0] grid-wide arrival counter, [1] CTAs that have left; both zero between launches
    int32_t* status;
    int64_t spin_limit;
    int32_t n_jobs;
    int32_t B, npad;
    int32_t ring;
    int32_t x_slots;            // item slots of digit planes in shared memory (the largest any job needs)
    int32_t debug;
    unsigned long long* trace;  // optional diagnostics: per CTA, per job 8 stamps (see qgemv_set_trace), or null
};

struct SeqSmem {
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
    static constexpr int kRowMax = 320;     // 8 words
    static constexpr int kDecision = 352;   // the converting warps' common verdict on the abort flag, per job
    static constexpr int kWarpMax = 384;    // kTcConvWarps x 8 words
    static constexpr int kSfb = 1024;       // 512 bytes
    static constexpr int kX = 1536;
    __host__ __device__ static constexpr int ring_off(int x_slots, int npad) { return (kX + x_slots * npad * 32 + 127) / 128 * 128; }
    __host__ __device__ static constexpr int total(int x_slots, int npad, int ring, int stage_items) {
        return ring_off(x_slots, npad) + ring * stage_items * kTcItemBytes;
    }
    static constexpr int kTmemCols = 512;   // one CTA per SM owns all of it
    __host__ __device__ static constexpr int max_ring_items(int npad) { return (kTmemCols - 2 * npad - 4) / 4; }
};

__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int atom_release_add(unsigned int* p, unsigned int v) {
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ SeqJob seq_load_job(const SeqJob* j) {
    const uint4* p = reinterpret_cast<const uint4*>(j);
    union {
        uint4 q[4];
        SeqJob job;
    } u;
    u.q[0] = __ldg(p), u.q[1] = __ldg(p + 1), u.q[2] = __ldg(p + 2), u.q[3] = __ldg(p + 3);
    return u.job;
}
// A job is split over min(grid, items) CTAs, exactly as a launch of its own would be; the other CTAs
// only take part in the job's barriers.  Range [begin, end) of CTA `cta` in the job's linear
// (tile, item) space; empty for a CTA beyond the job's share.
__device__ __forceinline__ int seq_job_grid(int32_t total, int grid) { return total < grid ? total : grid; }
__device__ __forceinline__ void seq_range(int32_t total, int cta, int gj, int32_t& begin, int32_t& end) {
    begin = end = 0;
    if (cta < gj) {
        begin = int32_t((int64_t(cta) * total) / gj);
        end = int32_t((int64_t(cta + 1) * total) / gj);
    }
}
// segment walker of CTA `cta` for a job (no segments for a CTA beyond the job's share)
__device__ __forceinline__ void seq_walker(GsWalker& wk, int32_t total, int32_t kt, int cta, int gj) {
    wk.units = kt;
    seq_range(total, cta, gj, wk.pos, wk.end);
}

template <int S>
__global__ void __launch_bounds__(kTcThreads, 1) gemv_seq_kernel(const SeqParams P) {
    extern __shared__ __align__(128) unsigned char sq_smem[];
    const uint32_t sbase = smem_u32(sq_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grid = gridDim.x, cta = blockIdx.x;
    const int npad = P.npad, R = P.ring;
    const uint32_t xslot_bytes = uint32_t(npad) * 32u;
    const uint32_t xbase = sbase + SeqSmem::kX;
    constexpr uint32_t stage_bytes = uint32_t(S) * kTcItemBytes;
    const uint32_t ring0 = sbase + uint32_t(SeqSmem::ring_off(P.x_slots, npad));
    constexpr uint32_t ncols = SeqSmem::kTmemCols;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(sq_smem + SeqSmem::kTmemPtr);
    volatile int* n_issued = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kIssued);
    volatile int* n_consumed = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kConsumed);
    unsigned int* rowmax = reinterpret_cast<unsigned int*>(sq_smem + SeqSmem::kRowMax);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcMaxRing; ++s) {
            mbar_init(sbase + SeqSmem::kBarFull + 8 * s, 1);
            mbar_init(sbase + SeqSmem::kBarEmpty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(sbase + SeqSmem::kBarDFull + 8 * b, 1);
            mbar_init(sbase + SeqSmem::kBarDFree + 8 * b, 4);
        }
        mbar_init(sbase + SeqSmem::kBarXReady, 1);
        mbar_init(sbase + SeqSmem::kBarDrain, 1);
        *abort_flag = 0;
        *n_issued = 0;
        *n_consumed = 0;
        mbar_fence_init();
    }
    if (warp == kTcWarpMma) {
        __syncwarp();
        tmem_alloc(sbase + SeqSmem::kTmemPtr, ncols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    pdl_launch_dependents();
    const uint32_t tmem_sfb = tmem_base + 2u * uint32_t(npad);
    const uint32_t tmem_sfa0 = tmem_sfb + 4u;

    if (warp == kTcWarpProd) {
        // ================= packed-weight producer: runs through the whole job list =================
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            const bool drop = (P.debug & 2) != 0;  // host-set fault injection: never issue a copy
            int s = 0, issued = 0;
            uint32_t use = 0;
            bool ok = true;
            SeqJob job = seq_load_job(P.jobs);
            for (int j = 0; j < P.n_jobs && ok; ++j) {
                SeqJob next = job;
                if (j + 1 < P.n_jobs) next = seq_load_job(P.jobs + j + 1);  // in flight while this job streams
                GsWalker wk;
                seq_walker(wk, job.tiles * job.kt, job.kt, cta, seq_job_grid(job.tiles * job.kt, grid));
                GsSeg sg;
                while (ok && wk.next(sg)) {
                    const uint8_t* src = job.payload + (uint64_t(sg.tile) * job.kt + uint64_t(sg.u0)) * kTcItemBytes;
                    for (int32_t left = sg.u1 - sg.u0; left > 0; left -= S) {
                        if (use > 0 && !mbar_wait_probe(sbase + SeqSmem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                            report(P.status, QGEMV_ERR_TIMEOUT, 71, j);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        const uint32_t bytes = uint32_t(min(S, left)) * kTcItemBytes;
                        if (!drop) {
                            const uint32_t bar = sbase + SeqSmem::kBarFull + 8 * s;
                            mbar_arrive_expect_tx(bar, bytes);
                            bulk_g2s(ring0 + s * stage_bytes, src, bytes, bar, pol);
                            ++issued;
                        }
                        src += bytes;
                        if (++s == R) s = 0, ++use;
                    }
                    if (*abort_flag) ok = false;
                }
                job = next;
            }
            *n_issued = issued;
        }
    } else if (warp == kTcWarpMma) {
        // ================= MMA issuer: one elected lane, all jobs =================
        if (elect_one()) {
            const uint32_t idesc = (1u << 7) | (1u << 10) | (uint32_t(npad >> 3) << 17) | (uint32_t(128 >> 4) << 24);
            const uint64_t d_ab = smem_desc(0, 128, 256), d_sf = smem_desc(0, 0, 128);
            const uint32_t ab_hi = uint32_t(d_ab >> 32), ab_lo = uint32_t(d_ab), sf_hi = uint32_t(d_sf >> 32), sf_lo = uint32_t(d_sf);
            const uint32_t x_lo0 = ab_lo | ((xbase >> 4) & 0x3FFFu);
            const uint32_t xslot16 = xslot_bytes >> 4, ring16 = (ring0 >> 4) & 0x3FFFu;
            constexpr uint32_t kItem16 = kTcItemBytes >> 4, kCode16 = kTcCodeBytes >> 4, stage16 = stage_bytes >> 4;
            uint32_t nseg = 0, full_par = 0;
            uint32_t item16 = ring16, sfa = tmem_sfa0, bar_full = sbase + SeqSmem::kBarFull, bar_empty = sbase + SeqSmem::kBarEmpty;
            const uint32_t ring_end16 = ring16 + uint32_t(R) * stage16;
            bool ok = true;
            int mi = 0;  // stages issued
            SeqJob job = seq_load_job(P.jobs);
            for (int j = 0; j < P.n_jobs && ok; ++j) {
                SeqJob next = job;
                if (j + 1 < P.n_jobs) next = seq_load_job(P.jobs + j + 1);
                const int32_t kt_len = job.kt;
                const int gj = seq_job_grid(job.tiles * kt_len, grid);
                int32_t r_begin, r_end;
                seq_range(job.tiles * kt_len, cta, gj, r_begin, r_end);
                const int32_t n_items = r_end - r_begin;
                const int32_t xs0 = n_items >= kt_len ? 0 : r_begin % kt_len;
                GsWalker wk;
                seq_walker(wk, job.tiles * kt_len, kt_len, cta, gj);
                GsSeg sg;
                bool have = wk.next(sg);
                // the digit planes of this job (every CTA signals, also one without items)
                if (!mbar_wait(sbase + SeqSmem::kBarXReady, uint32_t(j) & 1u, P.spin_limit)) {
                    report(P.status, QGEMV_ERR_TIMEOUT, 72, j);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (P.trace) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 3] = globaltimer_ns();
                if (j == 0) tc_cp_sf2(tmem_sfb, sf_lo | (((sbase + SeqSmem::kSfb) >> 4) & 0x3FFFu), sf_hi);
                for (; ok && have; have = wk.next(sg)) {
                    // the accumulator is free once the epilogue of the segment before last has read it
                    if (nseg >= 2 &&
                        !mbar_wait_probe(sbase + SeqSmem::kBarDFree + 8 * (nseg & 1), ((nseg >> 1) - 1) & 1, P.spin_limit)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 73, int(nseg));
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (nseg & 1) * uint32_t(npad);
                    uint32_t acc = 0;
                    int32_t slot = sg.u0 - xs0;
                    if (slot < 0) slot += kt_len;
                    uint32_t x_lo = x_lo0 + uint32_t(slot) * xslot16;
                    for (int32_t left = sg.u1 - sg.u0; left > 0; left -= S) {
                        // (the stage was written through the async proxy and is read through it: the
                        // barrier's acquire is all the ordering the MMAs need -- no tcgen05 fence here,
                        // which costs this thread a few hundred cycles per stage)
                        if (!mbar_wait_probe(bar_full, full_par, P.spin_limit)) {
                            report(P.status, QGEMV_ERR_TIMEOUT, 74, mi);
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        if (left >= S) {
#pragma unroll
                            for (int i = 0; i < S; ++i) tc_cp_sf2(sfa + 4u * i, sf_lo | (item16 + kCode16 + kItem16 * i), sf_hi);
#pragma unroll
                            for (int i = 0; i < S; ++i)
                                tc_mma_nvf4_2(tmem_d, ab_lo | (item16 + kItem16 * i), x_lo + xslot16 * i, ab_hi, idesc, sfa + 4u * i,
                                              tmem_sfb, i == 0 ? acc : 1u);
                        } else {
                            for (int i = 0; i < left; ++i) tc_cp_sf2(sfa + 4u * i, sf_lo | (item16 + kCode16 + kItem16 * i), sf_hi);
                            for (int i = 0; i < left; ++i)
                                tc_mma_nvf4_2(tmem_d, ab_lo | (item16 + kItem16 * i), x_lo + xslot16 * i, ab_hi, idesc, sfa + 4u * i,
                                              tmem_sfb, i == 0 ? acc : 1u);
                        }
                        acc = 1;
                        x_lo += xslot16 * S;
                        tc_commit(bar_empty);  // the stage is reusable once these retire
                        if (P.trace && P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 7] == 0) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 7] = globaltimer_ns();
                        ++mi;
                        item16 += stage16, sfa += 4u * S, bar_full += 8, bar_empty += 8;
                        if (item16 == ring_end16) {
                            item16 = ring16, sfa = tmem_sfa0, full_par ^= 1u;
                            bar_full = sbase + SeqSmem::kBarFull, bar_empty = sbase + SeqSmem::kBarEmpty;
                        }
                    }
                    if (!ok) break;
                    tc_commit(sbase + SeqSmem::kBarDFull + 8 * (nseg & 1));
                    ++nseg;
                }
                if (P.trace) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 4] = globaltimer_ns();
                job = next;
            }
            *n_consumed = mi;
        }
        __syncwarp();
    } else {
        // ================= digit planes and epilogues, job after job =================
        const int ct = threadIdx.x - 32 * kTcWarpConv0;  // 0..255
        const int Bl = P.B;
        const int g = (warp - kTcWarpConv0) >> 2, q = warp & 3;
        const uint32_t lane_base = uint32_t(32 * q) << 16;
        const int row = 32 * q + lane;
        unsigned int* all_max = reinterpret_cast<unsigned int*>(sq_smem + SeqSmem::kWarpMax);
        unsigned int* wmax = all_max + (warp - kTcWarpConv0) * 8;
        // block scales of the planes: column n = 8 b + j carries 2^(2j - 6) in all four K blocks
        if (ct < 128) {
            const int n = ct, j = n & 7;
            const uint32_t byte = n < 8 * Bl ? uint32_t(2 * j + 1) << 3 : 0u;
            *reinterpret_cast<volatile uint32_t*>(sq_smem + SeqSmem::kSfb + (n & 31) * 16 + (n >> 5) * 4) = byte * 0x01010101u;
        }
        pdl_wait();  // whatever ran before this launch has finished with x, y and the hand-over slots
        uint32_t nseg = 0;
        bool ok = true;  // this warp's own view; leaving the job loop is decided for all eight warps together
        unsigned int n_bar = 0;  // grid-wide barriers so far: the same number on every CTA
        auto grid_arrive = [&]() {  // after a barrier of the eight warps: this CTA's stores are ordered before it
            if (ct == 0) red_release_add(P.barrier, 1u);
            ++n_bar;
        };
        auto grid_wait = [&](int j) {
            if (ct == 0) {
                const unsigned int target = n_bar * unsigned(grid);
                uint64_t t0 = 0;
                for (int64_t it = 0; ld_acquire(P.barrier) < target; ++it) {
                    if (it == 0) t0 = globaltimer_ns();
                    if (it >= P.spin_limit || ((it & 63) == 63 && globaltimer_ns() - t0 > 2000000000ull)) {
                        report(P.status, QGEMV_ERR_TIMEOUT, 75, j);
                        *abort_flag = 1;
                        break;
                    }
                }
            }
        };
        // The row tile of the job before, if this CTA is its first contributor and the tile was split:
        // its rows are the sum of the parts, added here in CTA order once all of them are known to be stored.
        struct {
            bool valid;
            int32_t tile, c_lo, c_hi, lo_slot, N, y_dtype, parity;
            void* y;
        } pend;
        pend.valid = false;
        auto finalize_pending = [&]() {
            if (pend.valid && ct < 128) {
                const int n = pend.tile * 128 + ct;
                const float* parts = P.ws + size_t(pend.parity) * size_t(2 * grid) * 1024 + ct;
                if (n < pend.N) {
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        if (b < Bl) {
                            // eight parts' loads in flight together; the additions stay in CTA order
                            float v = __ldcg(parts + size_t(pend.lo_slot) * 1024 + b * 128);
                            for (int32_t cc = pend.c_lo + 1; cc <= pend.c_hi; cc += 8) {
                                float t[8];
#pragma unroll
                                for (int z = 0; z < 8; ++z) t[z] = __ldcg(parts + size_t(2 * min(cc + z, pend.c_hi)) * 1024 + b * 128);
#pragma unroll
                                for (int z = 0; z < 8; ++z)
                                    if (cc + z <= pend.c_hi) v += t[z];
                            }
                            const int64_t idx = int64_t(b) * pend.N + n;
                            if (pend.y_dtype == QGEMV_OUT_F32) {
                                static_cast<float*>(pend.y)[idx] = v;
                            } else {
                                static_cast<__nv_bfloat16*>(pend.y)[idx] = __float2bfloat16_rn(v);
                            }
                        }
                    }
                }
            }
            pend.valid = false;
        };
        volatile int* decision = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kDecision);
        SeqJob job = seq_load_job(P.jobs);
        for (int j = 0; j < P.n_jobs; ++j) {
            SeqJob next = job;
            if (j + 1 < P.n_jobs) next = seq_load_job(P.jobs + j + 1);
            const int32_t kt_len = job.kt;
            const int32_t total = job.tiles * kt_len;
            const int gj = seq_job_grid(total, grid);
            int32_t r_begin, r_end;
            seq_range(total, cta, gj, r_begin, r_end);
            const int32_t n_items = r_end - r_begin;
            const int32_t xs0 = n_items >= kt_len ? 0 : r_begin % kt_len;
            const int32_t n_slots = n_items >= kt_len ? kt_len : n_items;
            // ---- grid-wide barrier: every CTA has stored its results (or parts) of job j - 1 ----
            if (ct < 8 * kTcConvWarps) all_max[ct] = 0u;  // per-warp row maxima of the last job
            if (j > 0) grid_wait(j);
            // Named barriers have no time-out, so all eight warps must leave the job loop at the same
            // place: one thread samples the abort flag, everybody reads that sample after the barrier.
            if (ct == 0) *decision = *abort_flag;
            named_bar_sync(1, kTcConvThreads);
            if (*decision) break;
            if (j > 0 && (job.flags & 1)) {
                // this job reads or overwrites what the previous one produced: finish that first
                finalize_pending();
                named_bar_sync(1, kTcConvThreads);
                grid_arrive();
                grid_wait(j);
                if (ct == 0) *decision = *abort_flag;
                named_bar_sync(1, kTcConvThreads);
                if (*decision) break;
            }
            if (P.trace && ct == 0) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 0] = globaltimer_ns();
            // ---- digit planes of the items this CTA multiplies in job j (see gemv_tc.cuh) ----
            const int n_work = n_slots * Bl * 8;
            constexpr int kKeep = 4;
            auto unit_src = [&](int wu, int& b, uint32_t& dst) -> uint4 {
                const int o = wu & 7, sb = wu >> 3;
                b = sb / n_slots;
                const int slot = sb - b * n_slots;
                int32_t u = slot + xs0;
                if (u >= kt_len) u -= kt_len;
                const int k0 = u * 64 + o * 8;
                dst = xbase + uint32_t(slot) * xslot_bytes + uint32_t(b) * 256u + uint32_t(o >> 2) * 128u + uint32_t(o & 3) * 4u;
                uint4 v = make_uint4(0, 0, 0, 0);
                // written by other SMs during the previous job: read through L2, never a stale L1 line
                if (k0 + 8 <= job.K) v = __ldcg(reinterpret_cast<const uint4*>(job.x + int64_t(b) * job.x_stride + k0));
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
                uint32_t m = 0;
#pragma unroll
                for (int w = 0; w < kTcConvWarps; ++w) m = max(m, all_max[w * 8 + b]);
                return m;
            };
            auto store_unit = [&](int b, uint32_t dst, const uint4& v) {
                const float sf = pow2i(-tc_row_exponent(row_max(b)));
                uint32_t pl[8];
                tc_digits8(v, sf, pl);
#pragma unroll
                for (int z = 0; z < 8; ++z) asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + z * 16), "r"(pl[z]) : "memory");
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
            if (ct == 0) mbar_arrive(sbase + SeqSmem::kBarXReady);
            if (P.trace && ct == 0) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 1] = globaltimer_ns();
            // the tensor core is busy with this job now: add up the split tile of the job before
            finalize_pending();
            if (P.trace && ct == 0) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 6] = globaltimer_ns();

            // ---- epilogues of job j: group g takes the segments with (global) nseg % 2 == g ----
            float scale[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) scale[b] = b < Bl ? job.tensor_scale * pow2i(tc_row_exponent(rowmax[b]) + 7) : 0.f;
            GsWalker wk;
            seq_walker(wk, total, kt_len, cta, gj);
            GsSeg sg;
            while (ok && wk.next(sg)) {
                const bool whole = sg.u0 == 0 && sg.u1 == kt_len;
                int32_t c_lo = 0, c_hi = 0, my_slot = 0;
                if (!whole) {
                    c_lo = int32_t(cta_of(int64_t(sg.tile) * kt_len, total, gj));
                    c_hi = int32_t(cta_of(int64_t(sg.tile + 1) * kt_len - 1, total, gj));
                    // every contributor after the first starts its range inside this tile (slot 0 of its
                    // pair); the first one's range may have started in an earlier tile
                    my_slot = cta == c_lo ? gs_slot(c_lo, sg.tile, kt_len, total, gj) : 2 * cta;
                    if (cta == c_lo) {  // all eight warps note it, whichever group runs the segment
                        pend.valid = true;
                        pend.tile = sg.tile, pend.c_lo = c_lo, pend.c_hi = c_hi, pend.lo_slot = my_slot;
                        pend.N = job.N, pend.y_dtype = job.y_dtype, pend.parity = j & 1, pend.y = job.y;
                    }
                }
                if (int(nseg & 1) != g) {
                    ++nseg;
                    continue;
                }
                if (!__all_sync(0xFFFFFFFFu, mbar_wait_probe(sbase + SeqSmem::kBarDFull + 8 * g, (nseg >> 1) & 1, P.spin_limit))) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 76, int(nseg));
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                tc_fence_after();
                if (P.trace && lane == 0 && q == 0) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 5] = globaltimer_ns();  // the last one stays
                float val[8];
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    val[b] = 0.f;
                    if (b < Bl) {
                        uint32_t r[8];
                        tmem_ld8(tmem_base + lane_base + uint32_t(g * npad + 8 * b), r);
                        float a = __uint_as_float(r[0]);
#pragma unroll
                        for (int z = 1; z < 8; ++z) a += __uint_as_float(r[z]);
                        val[b] = a * scale[b];
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sbase + SeqSmem::kBarDFree + 8 * g);  // the accumulator may be overwritten
                const int n = sg.tile * 128 + row;
                auto store_row = [&](const float (&v)[8]) {
                    if (n < job.N) {
#pragma unroll
                        for (int b = 0; b < 8; ++b) {
                            if (b < Bl) {
                                const int64_t idx = int64_t(b) * job.N + n;
                                if (job.y_dtype == QGEMV_OUT_F32) {
                                    static_cast<float*>(job.y)[idx] = v[b];
                                } else {
                                    static_cast<__nv_bfloat16*>(job.y)[idx] = __float2bfloat16_rn(v[b]);
                                }
                            }
                        }
                    }
                };
                if (whole) {
                    store_row(val);
                } else {
                    float* slot = P.ws + (size_t(j & 1) * size_t(2 * grid) + size_t(my_slot)) * 1024 + row;
#pragma unroll
                    for (int b = 0; b < 8; ++b)
                        if (b < Bl) __stcg(slot + b * 128, val[b]);
                }
                ++nseg;
            }
            if (P.trace && ct == 0) P.trace[(size_t(cta) * P.n_jobs + j) * 8 + 2] = globaltimer_ns();
            // ---- this CTA's results and parts of job j are stored: arrive ----
            named_bar_sync(1, kTcConvThreads);
            grid_arrive();
            job = next;
        }
        // ---- the last job's split tile, once every CTA has arrived; then leave the counters at zero ----
        if (!*decision) {
            grid_wait(P.n_jobs);
            if (ct == 0) *decision = *abort_flag;
            named_bar_sync(1, kTcConvThreads);
            if (!*decision) {
                finalize_pending();
                named_bar_sync(1, kTcConvThreads);
                if (ct == 0 && atom_release_add(P.barrier + 1, 1u) == unsigned(grid) - 1u) {
                    P.barrier[0] = 0u;  // the last CTA to leave: nobody polls any more
                    P.barrier[1] = 0u;
                }
            }
        }
    }
    // ---- release tensor memory (always), after every role is done with it ----
    tc_fence_before();
    __syncthreads();
    if (warp == kTcWarpMma) {
        __syncwarp();
        if (*abort_flag) {
            if (lane == 0) {
                tc_commit(sbase + SeqSmem::kBarDrain);
                (void)mbar_wait_probe(sbase + SeqSmem::kBarDrain, 0, int64_t(1) << 16);
            }
            __syncwarp();
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, ncols);
    } else if (threadIdx.x == 0 && *abort_flag) {
        // never leave with copies in flight: wait (bounded) for every copy that nothing consumed
        const int issued = *n_issued;
        for (int i = *n_consumed; i < issued; ++i)
            (void)mbar_wait(sbase + SeqSmem::kBarFull + 8 * (i % R), uint32_t(i / R) & 1u, int64_t(1) << 20);
    }
}

}  // namespace qg
