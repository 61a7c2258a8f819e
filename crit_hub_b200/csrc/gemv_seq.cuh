// A SEQUENCE of NVFP4 GEMVs (tensor-core layout) as ONE persistent launch: the projections of a
// decode step, executed in order, each allowed to read what the ones before it wrote.
//
// Launched one by one, each GEMV of a decode layer pays a serial chain that no weight byte overlaps:
// the previous grid's last partial sums, the launch boundary, the activation conversion, the first
// MMAs -- about 5 us, four times per layer, against 19 us of HBM time.  Here one grid of one CTA per
// SM walks the whole job list.  The producer thread never stops at a job boundary: while the CTA's
// other warps finish job j and convert the activations of job j+1, it already streams the items of
// job j+1, j+2, ... into a ring that takes most of the SM's shared memory, so HBM stays busy across
// the boundary and the MMAs of the next job find their first 130-190 KB per SM waiting.
//
// Per job the arithmetic is gemv_tc.cuh's: weights consumed as stored by tcgen05.mma
// kind::mxf4nvf4, activations as eight E2M1 digit planes scaled per CTA range, split along K over
// the CTAs with a deterministic hand-over to each row tile's first contributor.
//
// Warps: 0 producer, 1 MMA issuer, then three groups of four warps that run side by side and meet
// only through mbarriers in shared memory and two counters per job in global memory:
//   PLANES    digit planes of job j into one of up to three buffers (so it may be that many jobs
//             ahead of the epilogues).  A job that must not overtake an earlier one -- the host
//             compares the address ranges of every job's x and y with those of the jobs before it,
//             or the caller says so -- first waits until fin[that job] has been bumped by every CTA.
//   EPILOGUE  accumulators -> y rows (a CTA that holds a whole row tile) or fp32 partial sums in the
//             CTA's slot of a parts buffer (sixteen buffers, taken in turn by the jobs); then bumps
//             done[j] with release semantics.
//   FINISH    once done[j] shows every CTA: the first contributor of a split row tile adds the parts
//             in CTA order -- a fixed order -- and stores the rows; then bumps fin[j].  Nothing here
//             is on the MMA issuer's critical path.
// The CTAs wait on one another, so the launch is cooperative (all CTAs co-resident).
//
// Tensor parallel: a row-parallel projection's output is the sum over the ranks.  For such a job
// (xoff >= 0) the FINISH thread that has added up a row pushes the fp32 partial sum, tagged with
// the count of launches, into its rank's slot of every rank's exchange buffer over NVLink, then
// gathers the ranks' pairs for that row from its own buffer (all loads in flight, bounded
// re-polling), adds them in rank order and stores the row: the all-reduce costs no launch and no
// grid-wide wait (tp_allreduce.cuh describes the slots).  Every rank runs the same job list on the
// same grid, so the same CTA holds a row on every rank.
#pragma once
#include "gemv_tc.cuh"
#include "tp_allreduce.cuh"

namespace qg {

constexpr int kSeqPartBufs = 16;     // parts buffers: jobs a CTA may run ahead of the slowest CTA's split-tile sums
constexpr int kSeqPlaneBufsMax = 3;  // buffers of digit planes (1..3, as many as leave room for a ring): the PLANES group
                                     // may be that many jobs ahead of the epilogues

struct SeqJob {               // 80 bytes, device memory
    const uint8_t* payload;   // items of the weight: (tile * kt + item) * 4608
    const uint16_t* x;        // bf16 [B][K]
    void* y;                  // [B][N]
    float tensor_scale;
    int32_t N, K;
    int32_t tiles, kt;        // ceil(N / 128), ceil(K / 64)
    int32_t x_stride;         // elements between activation rows
    int32_t y_dtype;
    int32_t dep;              // latest earlier job that must be complete on every CTA before this job's activations
                              // are read (an address-range hazard found by the host, or the caller's order); -1: none
    int32_t xoff;             // >= 0: a row-parallel projection, y = sum over the ranks; element offset of this job's
                              // [B][N] block inside every slot of the exchange buffers.  -1: local job
    int32_t pub_off;          // >= 0: a later job reads this job's bf16 output as its activations: every row is also
                              // published as a word {tag, bf16} at pub[pub_off + b * N + n].  -1: not published
    int32_t src_off;          // >= 0: the activations are read from pub[src_off + b * x_stride + k], published by job
                              // src_job, word by word as they appear (no grid-wide wait).  -1: from x
    int32_t src_job;
    int32_t act;              // 1: the activations are silu(x[k]) * x[K + k] of rows that hold 2 K values (rounded to bf16)
    float norm_eps;
    const uint16_t* norm_w;   // bf16 [K] or null: x'[k] = bf16(x[k] * norm_w[k]); y is scaled by rsqrt(mean(x^2) + eps)
    const void* residual;     // [B][N] in y's dtype or null: added to the result before it is rounded
    const int32_t* rowmap;    // expert list only: [16] row of x for each of the job's activation rows, then row of y (shared memory)
    int32_t rows;             // expert list only: activation rows of this job (<= B)
    int32_t fin_release;      // 1: a later job waits for this one's counter (dep), so the counter is bumped with release
                              // semantics; 0: nobody reads what this job wrote on the strength of its counter
};
static_assert(sizeof(SeqJob) == 112, "SeqJob layout");

struct SeqParams {
    const SeqJob* jobs;
    unsigned long long* ws;     // parts buffers: [job % kSeqPartBufs][2 * cta + which][8][128] pairs {fp32 partial sum, tag}
    unsigned int* barrier;      // [0] CTAs that have left the launch (zero between launches), [1] launches of this
                                // handle that exchanged between ranks, [2] sequence launches of this handle
    unsigned int* fin;          // [n_jobs] CTAs that are through with the job (rows stored, split tile added up); zero
                                // between launches.  [n_jobs]: launches of this job list
    uint32_t* pub;              // published outputs of this job list, words {16-bit tag, bf16}
    int32_t* status;
    int64_t spin_limit;
    int32_t n_jobs;
    int32_t B, npad;
    int32_t ring;
    int32_t x_slots;            // item slots of digit planes in one buffer (the largest any job needs)
    int32_t nbuf;               // buffers of digit planes, 1..kSeqPlaneBufsMax
    int32_t debug;
    unsigned long long* trace;  // optional diagnostics: per CTA, per job 8 stamps (see qgemv_set_trace), or null
    int32_t trace_jobs;         // jobs per CTA in the trace (a list: n_jobs; an expert list: kMoeLocalJobs, the CTA's own problems)
    // tensor-parallel exchange (world == 1: none)
    uint8_t* xbuf[kTpMaxWorld];
    int64_t x_max_elems;
    int32_t rank, world;
    // expert list (kSeqMoe): the jobs are the problems of the router's table -- for every expert that the top-k lists
    // [slots / topk][topk] name, its (token, choice) entries in list order, cut into problems of at most B
    // activation rows.  Every CTA works the table out for itself at the start of the launch (the part of it that
    // its range touches); every job is moe_job with the expert's payload and tensor scale.
    const int32_t* ids;
    const float* expert_ts;
    uint64_t expert_stride;
    int32_t slots, topk, n_experts, per_slot;  // per_slot: activation row = the entry's index (else its token)
    int32_t moe_smem;                          // offset of the CTA's problem table in shared memory (behind the ring)
    SeqJob moe_job;
    // Two stages in one launch (n_phases == 2; an expert MLP): moe_job is the gate/up stage, which writes its
    // bf16 rows [slots][N] to moe_job.y, and moe_job2 the down stage, which reads them (with its activation
    // function) as soon as the problem's gate/up tiles are counted complete in moe_cnt.  Each stage's items are
    // a split space of their own, dealt evenly to all CTAs; a CTA works through its share of the first, then
    // of the second.
    int32_t n_phases;
    const float* expert_ts2;
    uint64_t expert_stride2;
    SeqJob moe_job2;
    unsigned int* moe_cnt;                     // [problems] warps that have stored rows of a gate/up problem; zero between launches
};
constexpr int kMoeMaxExperts = 512;   // experts of a stacked weight that the expert-list mode takes
constexpr int kMoeLocalJobs = 32;     // problems that one CTA's range may touch
constexpr int kMoeMaxSlots = 4096;    // (token, choice) entries of the lists
constexpr int kMoeSmemBytes = (kMoeLocalJobs * kProbInts + 32) * 4;            // the table, kept for the whole launch
constexpr int kMoeWalkBytes = (2 * kMoeMaxExperts + kMoeMaxSlots) * 4;          // the walk's scratch: lies in the (still empty) ring

struct SeqSmem {
    static constexpr int kBarFull = 0;      // kTcMaxRing
    static constexpr int kBarEmpty = 128;   // kTcMaxRing
    static constexpr int kBarDFull = 256;   // 2
    static constexpr int kBarDFree = 272;   // 2
    static constexpr int kBarXReady = 704;  // kSeqPlaneBufsMax: the digit planes in a buffer are ready
    static constexpr int kBarEDone = 736;   // kSeqPlaneBufsMax: the epilogues of the job that used a plane buffer are through
    static constexpr int kBarMDone = 768;   // kSeqPlaneBufsMax: the MMA issuer is through with the job that used a plane buffer
    static constexpr int kRange = 800;      // [kSeqPlaneBufsMax][2] ints: this CTA's item range of the job in a plane buffer
    static constexpr int kRowMax = 832;     // [kSeqPlaneBufsMax][8] words: largest |bf16| pattern per activation row
    static constexpr int kBarDrain = 304;
    static constexpr int kTmemPtr = 312;
    static constexpr int kAbort = 316;
    static constexpr int kWarpMax = 384;    // kTcConvWarps x 8 words: the same per converting warp
    static constexpr int kIssued = 640;
    static constexpr int kConsumed = 644;
    static constexpr int kDecision = 928;   // [2][4] every warp group's common samples of the abort flag
    static constexpr int kFinAll = 688;     // jobs up to this index are added up on every CTA (-1: none)
    static constexpr int kRowScale = 512;   // [kSeqPlaneBufsMax][8] floats: rsqrt(mean(x^2) + eps) per activation row of a job with a norm
    static constexpr int kEpiDone = 692;    // jobs whose epilogues this CTA has been through (release / acquire at CTA scope)
    static constexpr int kSfb = 1024;       // 512 bytes
    static constexpr int kX = 1536;
    // nbuf buffers of digit planes (jobs take them in turn), then the ring
    __host__ __device__ static constexpr int ring_off(int x_slots, int npad, int nbuf) { return (kX + nbuf * x_slots * npad * 32 + 127) / 128 * 128; }
    __host__ __device__ static constexpr int total(int x_slots, int npad, int nbuf, int ring, int stage_items) {
        return ring_off(x_slots, npad, nbuf) + ring * stage_items * kTcItemBytes;
    }
    static constexpr int kTmemCols = 512;   // one CTA per SM owns all of it
    __host__ __device__ static constexpr int max_ring_items(int npad) { return (kTmemCols - 2 * npad - 4) / 4; }
};

__device__ __forceinline__ void red_release_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_relaxed_add(unsigned int* p, unsigned int v) {
    asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
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
__device__ __forceinline__ void st_release_cta_shared(uint32_t addr, int v) {
    asm volatile("st.release.cta.shared.b32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cta_shared(uint32_t addr) {
    int v;
    asm volatile("ld.acquire.cta.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_tagged(unsigned long long* p, float v, uint32_t tag) {
    const unsigned long long w = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void st_pub(uint32_t* p, uint32_t w) {
    asm volatile("st.relaxed.gpu.global.b32 [%0], %1;" ::"l"(p), "r"(w) : "memory");
}
__device__ __forceinline__ uint4 ld_pub4(const uint32_t* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// tag of a partial sum: the handle's launch count and the job; of a published word: the job list's
// launch count (low bits) and the job.  A slot is rewritten by every launch that reads it, so what
// is left from before carries another launch's tag.
__device__ __forceinline__ uint32_t seq_part_tag(uint32_t launch, int j) { return launch * 4099u + uint32_t(j) + 1u; }
__device__ __forceinline__ uint32_t seq_pub_tag(uint32_t run, int j) { return ((run & 15u) << 12) | (uint32_t(j + 1) & 0xFFFu); }

__device__ __forceinline__ SeqJob seq_load_job(const SeqJob* j) {
    const uint4* p = reinterpret_cast<const uint4*>(j);
    union {
        uint4 q[7];
        SeqJob job;
    } u;
    u.q[0] = __ldg(p), u.q[1] = __ldg(p + 1), u.q[2] = __ldg(p + 2), u.q[3] = __ldg(p + 3), u.q[4] = __ldg(p + 4);
    u.q[5] = __ldg(p + 5), u.q[6] = __ldg(p + 6);
    return u.job;
}
// MODE of the kernel: a plain job list; one with fused activation transforms; the experts of a router table.
constexpr int kSeqPlain = 0, kSeqFuse = 1, kSeqMoe = 2;
// A job is split over min(grid, items) CTAs, exactly as a launch of its own would be; the other CTAs
// only take part in the job's barriers.  Range [begin, end) of CTA `cta` in the job's linear
// (tile, item) space; empty for a CTA beyond the job's share.
__device__ __forceinline__ int seq_job_grid(int32_t total, int grid) { return total < grid ? total : grid; }
// (32-bit arithmetic: the host refuses job lists with (items + 1) * grid >= 2^32, and 64-bit divisions are
// long instruction sequences that this kernel, whose roles share an instruction cache, can do without)
__device__ __forceinline__ void seq_range(int32_t total, int cta, int gj, int32_t& begin, int32_t& end) {
    begin = end = 0;
    if (cta < gj) {
        begin = int32_t((uint32_t(cta) * uint32_t(total)) / uint32_t(gj));
        end = int32_t((uint32_t(cta + 1) * uint32_t(total)) / uint32_t(gj));
    }
}
// the CTA whose range holds item idx; the parts slot of CTA c for row tile `tile` (first segment 2c, last 2c + 1):
// the values of cta_of() and gs_slot()
__device__ __forceinline__ int32_t seq_cta_of(int32_t idx, int32_t total, int gj) {
    return int32_t((uint32_t(idx + 1) * uint32_t(gj) - 1u) / uint32_t(total));
}
__device__ __forceinline__ int32_t seq_slot(int32_t c, int32_t tile, int32_t units, int32_t total, int gj) {
    const uint32_t a = (uint32_t(c) * uint32_t(total)) / uint32_t(gj);
    return 2 * c + (int32_t(a / uint32_t(units)) == tile ? 0 : 1);
}

// The waits' slow paths out of line as well: a wait that finds its barrier complete costs a probe.
__device__ __noinline__ bool seq_mbar_spin(uint32_t bar, uint32_t parity, int64_t spin_limit) { return mbar_wait(bar, parity, spin_limit); }
__device__ __forceinline__ bool seq_mbar_wait(uint32_t bar, uint32_t parity, int64_t spin_limit) {
    return mbar_try_wait(bar, parity) || seq_mbar_spin(bar, parity, spin_limit);
}
__device__ __forceinline__ bool seq_mbar_probe(uint32_t bar, uint32_t parity, int64_t spin_limit) {
    return mbar_test_wait(bar, parity) || seq_mbar_spin(bar, parity, spin_limit);
}
__device__ __noinline__ void seq_report(int32_t* status, int where, int extra) { report(status, QGEMV_ERR_TIMEOUT, where, extra); }

// Eight activations of one row -> their eight digit planes in shared memory.  Not inlined: the kernel's five
// roles run different code on an SM at once and share its instruction cache, so the code is kept small.
// The 32 lanes of a warp work on units whose addresses differ by multiples of 128 bytes except for the word
// inside a 16-byte plane row (unit mod 4): stored plane by plane they would hit four banks eight deep.  Each
// lane therefore starts with another plane -- (lane / 4) mod 8, the part of its unit number that the bank
// does not see -- so that one store instruction covers all 32 banks.
__device__ __noinline__ void seq_store_unit(uint32_t dst, uint4 v, float sf) {
    uint32_t pl[8];
    tc_digits8(v, sf, pl);
    const int rot = (threadIdx.x >> 2) & 7;
#pragma unroll
    for (int sft = 1; sft < 8; sft <<= 1) {   // pl[z] <- pl[(z + rot) mod 8], one bit of rot at a time
        const bool on = (rot & sft) != 0;
        uint32_t q[8];
#pragma unroll
        for (int z = 0; z < 8; ++z) q[z] = on ? pl[(z + sft) & 7] : pl[z];
#pragma unroll
        for (int z = 0; z < 8; ++z) pl[z] = q[z];
    }
#pragma unroll
    for (int z = 0; z < 8; ++z) asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + uint32_t((z + rot) & 7) * 16u), "r"(pl[z]) : "memory");
}

// ---- fused activation transforms (FUSE instantiation only) ----------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t bf16_pack(float lo, float hi) {
    return uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) | (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
}
__device__ __forceinline__ float silu_f32(float g) { return __fdividef(g, 1.0f + __expf(-g)); }
// eight gate values and eight up values -> bf16(silu(gate) * up)
__device__ __noinline__ uint4 seq_silu_mul(uint4 g, uint4 u) {
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int z = 0; z < 4; ++z) o[z] = bf16_pack(silu_f32(bf16_lo(gw[z])) * bf16_lo(uw[z]), silu_f32(bf16_hi(gw[z])) * bf16_hi(uw[z]));
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// eight activations times eight norm weights -> bf16
__device__ __noinline__ uint4 seq_mul_w(uint4 x, uint4 w) {
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, ww[4] = {w.x, w.y, w.z, w.w};
    uint32_t o[4];
#pragma unroll
    for (int z = 0; z < 4; ++z) o[z] = bf16_pack(bf16_lo(xw[z]) * bf16_lo(ww[z]), bf16_hi(xw[z]) * bf16_hi(ww[z]));
    return make_uint4(o[0], o[1], o[2], o[3]);
}
__device__ __forceinline__ float seq_sumsq(uint4 x) {
    const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
    float a = 0.f;
#pragma unroll
    for (int z = 0; z < 4; ++z) a = fmaf(bf16_lo(xw[z]), bf16_lo(xw[z]), fmaf(bf16_hi(xw[z]), bf16_hi(xw[z]), a));
    return a;
}

#ifdef QGEMV_SEQ_PROFILE   // diagnostics build only: where the MMA issuer's time goes (cycles per CTA, summed over the launch)
#define SEQ_PROF_T0() const long long prof_t0 = clock64()
#define SEQ_PROF_ADD(slot) prof[slot] += clock64() - prof_t0
#define SEQ_STAMPS false
#else
#define SEQ_STAMPS true
#define SEQ_PROF_T0()
#define SEQ_PROF_ADD(slot)
#endif

constexpr int kSeqThreads = 32 * (2 + 12);  // producer, MMA issuer, three groups of four warps

// MODE kSeqFuse: the job list holds jobs with an activation function, a norm or a residual; the plain
// instantiation carries none of that code.  MODE kSeqMoe: the jobs are the problems of a router table (one
// expert's matrix times up to eight gathered activation rows, results scattered to the slots' rows).
template <int S, int MODE>
__global__ void __launch_bounds__(kSeqThreads, 1) gemv_seq_kernel(const SeqParams P) {
    constexpr bool FUSE = MODE == kSeqFuse, MOE = MODE == kSeqMoe;
    constexpr bool ACT = FUSE || MOE;  // jobs may apply an activation function to what they read (the experts' down stage)
    extern __shared__ __align__(128) unsigned char sq_smem[];
    const uint32_t sbase = smem_u32(sq_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grid = gridDim.x, cta = blockIdx.x;
    const int npad = P.npad, R = P.ring;
    const uint32_t xslot_bytes = uint32_t(npad) * 32u;
    const uint32_t xbase = sbase + SeqSmem::kX;
    const uint32_t xbuf_bytes = uint32_t(P.x_slots) * xslot_bytes;  // one buffer of digit planes
    constexpr uint32_t stage_bytes = uint32_t(S) * kTcItemBytes;
    const int nb = P.nbuf;
    const uint32_t ring0 = sbase + uint32_t(SeqSmem::ring_off(P.x_slots, npad, nb));
    constexpr uint32_t ncols = SeqSmem::kTmemCols;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kAbort);
    volatile uint32_t* tmem_ptr = reinterpret_cast<volatile uint32_t*>(sq_smem + SeqSmem::kTmemPtr);
    volatile int* n_issued = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kIssued);
    volatile int* n_consumed = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kConsumed);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcMaxRing; ++s) {
            mbar_init(sbase + SeqSmem::kBarFull + 8 * s, 1);
            mbar_init(sbase + SeqSmem::kBarEmpty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(sbase + SeqSmem::kBarDFull + 8 * b, 1);
            mbar_init(sbase + SeqSmem::kBarDFree + 8 * b, 4);
        }
        mbar_init(sbase + SeqSmem::kBarDrain, 1);
        for (int b = 0; b < kSeqPlaneBufsMax; ++b) {
            mbar_init(sbase + SeqSmem::kBarXReady + 8 * b, 1);
            mbar_init(sbase + SeqSmem::kBarEDone + 8 * b, 1);
            mbar_init(sbase + SeqSmem::kBarMDone + 8 * b, 1);
        }
        *reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kFinAll) = -1;
        *reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kEpiDone) = 0;
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

    // How a job's items are dealt to the CTAs.  A job of a list is split over min(grid, items) CTAs, as a launch
    // of its own would be, and every CTA goes through every job.  The experts of a router table are ONE split
    // space instead -- the problems' items laid end to end and dealt evenly -- so a CTA works on the one to three
    // experts its range touches, goes through those jobs only, and hands over at most two split row tiles.
    int j_lo = 0, j_hi = P.n_jobs;
    const int* m_tab = nullptr;  // expert list: the problems this CTA's range touches, kProbInts ints each
    const volatile int* m_ph = nullptr;  // expert list: the stages' split spaces, five ints each
    int m_nprob = 0;             // expert list: problems of the router's table
    uint32_t m_launch_no = 0, m_run_no = 0;  // expert list: the launch counts, fetched while the lists are walked
    if constexpr (MOE) {
        // ---- the router walk: entries per expert (shared-memory histogram), problems per expert and their prefix
        // (one warp), then one warp per problem of this CTA's range collects the problem's rows in list order ----
        // (counts, prefix and a copy of the lists live where the weight ring will be: no copy is issued before
        // the walk is over and its accesses are fenced off against the asynchronous proxy)
        int* m_counts = reinterpret_cast<int*>(sq_smem + SeqSmem::ring_off(P.x_slots, npad, nb));  // [n_experts] entries
        int* m_base = m_counts + kMoeMaxExperts;                       // [n_experts] first problem
        int* m_ids = m_base + kMoeMaxExperts;                          // [slots] the lists
        int* tab = reinterpret_cast<int*>(sq_smem + P.moe_smem);       // [kMoeLocalJobs][kProbInts]
        volatile int* m_misc = tab + kMoeLocalJobs * kProbInts;        // [0] problems, [1] an id out of range, [2..11] the stages
        m_tab = tab;
        m_ph = m_misc + 2;
        const int E = P.n_experts, slots = P.slots, cap = P.B;
        if (P.trace && threadIdx.x == 0) P.trace[size_t(grid) * P.trace_jobs * 8 + size_t(cta) * 4 + 0] = globaltimer_ns();
        pdl_wait();  // the lists are the work of whatever ran before this launch
        m_launch_no = __ldcg(P.barrier + 2), m_run_no = __ldcg(P.fin + P.n_jobs);
        for (int e = threadIdx.x; e < E; e += kSeqThreads) m_counts[e] = 0;
        if (threadIdx.x == 0) m_misc[0] = 0, m_misc[1] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < slots; i += kSeqThreads) {
            const int e = __ldcg(P.ids + i);
            m_ids[i] = e;
            if (unsigned(e) >= unsigned(E)) {
                m_misc[1] = 1;
            } else {
                atomicAdd(&m_counts[e], 1);
            }
        }
        __syncthreads();
        if (warp == 0) {
            int carry = 0;
            for (int e0 = 0; e0 < E; e0 += 32) {
                const int e = e0 + lane;
                const int np = e < E ? (m_counts[e] + cap - 1) / cap : 0;
                int incl = np;
                for (int d = 1; d < 32; d <<= 1) {
                    const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                    if (lane >= d) incl += v;
                }
                if (e < E) m_base[e] = carry + incl - np;
                carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
            }
            if (lane == 0) {
                if (m_misc[1]) {
                    if (cta == 0) report(P.status, QGEMV_ERR_BOUNDS, 21, 0);
                    carry = 0;  // every CTA sees the same lists and leaves without work
                }
                m_misc[0] = carry;
            }
        }
        __syncthreads();
        // Per stage (one, or two for an expert MLP): its split space and this CTA's share.  m_misc[2 + 5 q ..]:
        // items, first and last + 1 item of this CTA, items per problem, CTAs that share the space.
        m_nprob = m_misc[0];
        int lo[2] = {0, 0}, hi[2] = {0, 0};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            if (q < P.n_phases) {
                const SeqJob& tj = q ? P.moe_job2 : P.moe_job;
                const int32_t per = tj.tiles * tj.kt, total = m_nprob * per;
                const int gjq = seq_job_grid(total, grid);
                int32_t bg, en;
                seq_range(total, cta, gjq, bg, en);
                lo[q] = bg / per;
                hi[q] = en > bg ? (en - 1) / per + 1 : lo[q];
                if (threadIdx.x == 0) {
                    volatile int* z = m_misc + 2 + 5 * q;
                    z[0] = total, z[1] = bg, z[2] = en, z[3] = per, z[4] = gjq;
                }
            }
        }
        const int n_first = hi[0] - lo[0];
        j_lo = 0;
        j_hi = n_first + (hi[1] - lo[1]);   // from here on a job is named by its place in this CTA's list
        if (j_hi > kMoeLocalJobs) {  // (the host refuses shapes that could come here)
            if (threadIdx.x == 0) {
                report(P.status, QGEMV_ERR_BOUNDS, 20, j_hi);
                *abort_flag = 1;
            }
            j_hi = 0;
        }
        for (int e = threadIdx.x; e < E; e += kSeqThreads) {
            const int cnt = m_counts[e];
            const int b0 = m_base[e], np = (cnt + cap - 1) / cap;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                if (j_hi == 0) break;
                for (int j = max(lo[q], b0); j < min(hi[q], b0 + np); ++j) {
                    int* t = tab + ((q ? n_first : 0) + j - lo[q]) * kProbInts;
                    const int qi = j - b0;
                    t[0] = e, t[1] = min(cap, cnt - qi * cap), t[18] = qi, t[19] = j | (q << 16);
                }
            }
        }
        __syncthreads();
        for (int jl = warp; jl < j_hi; jl += kSeqThreads / 32) {
            int* t = tab + jl * kProbInts;
            const int e = t[0], rows = t[1], r0 = t[18] * cap;
            // activation rows: the entry's token, or the entry itself (the second stage of an MLP reads the first one's rows)
            const bool own_row = P.n_phases == 2 ? (t[19] >> 16) != 0 : P.per_slot != 0;
            int seen = 0;
            for (int i0 = 0; i0 < slots && seen < r0 + rows; i0 += 32) {
                const int i = i0 + lane;
                const int id = i < slots ? m_ids[i] : -1;
                const unsigned m = __ballot_sync(0xFFFFFFFFu, id == e);
                const int r = seen + __popc(m & ((1u << lane) - 1u)) - r0;
                if (id == e && r >= 0 && r < rows) {
                    t[2 + r] = own_row ? i : i / P.topk;
                    t[10 + r] = i;
                }
                seen += __popc(m);
            }
        }
        fence_proxy_async_smem();  // the scratch becomes the ring: written next by bulk copies
        __syncthreads();
    }
    if constexpr (MOE) {
        if (P.trace && threadIdx.x == 0) P.trace[size_t(grid) * P.trace_jobs * 8 + size_t(cta) * 4 + 1] = globaltimer_ns();
    }
    // expert list: stage and problem of job j of this CTA's list; the stage's split space
    auto moe_info = [&](int j, int& ph, int& prob) {
        const int v = m_tab[j * kProbInts + 19];
        ph = v >> 16, prob = v & 0xFFFF;
    };
    auto job_at = [&](int j) -> SeqJob {
        if constexpr (MOE) {
            const int* t = m_tab + j * kProbInts;
            const int e = t[0], ph = t[19] >> 16;
            SeqJob job = ph ? P.moe_job2 : P.moe_job;
            job.payload += uint64_t(e) * (ph ? P.expert_stride2 : P.expert_stride);
            job.tensor_scale = __ldg((ph ? P.expert_ts2 : P.expert_ts) + e);
            job.rows = t[1];
            job.rowmap = t + 2;
            return job;
        } else {
            return seq_load_job(P.jobs + j);
        }
    };
    // this CTA's range [rb, re) of job j, in the job's own (tile, item) space
    auto job_range = [&](const SeqJob& job, int j, int32_t& rb, int32_t& re) {
        if constexpr (MOE) {
            int ph, prob;
            moe_info(j, ph, prob);
            const volatile int* z = m_ph + 5 * ph;
            const int32_t per = z[3], base = prob * per;
            rb = min(max(z[1] - base, 0), per), re = min(max(z[2] - base, 0), per);
        } else {
            const int32_t total = job.tiles * job.kt;
            seq_range(total, cta, seq_job_grid(total, grid), rb, re);
        }
    };
    // the CTA that holds item idx of job j; the parts slot of CTA c for row tile `tile` of job j
    auto job_cta_of = [&](const SeqJob& job, int j, int32_t idx) -> int32_t {
        if constexpr (MOE) {
            int ph, prob;
            moe_info(j, ph, prob);
            const volatile int* z = m_ph + 5 * ph;
            return seq_cta_of(prob * z[3] + idx, z[0], z[4]);
        } else {
            const int32_t total = job.tiles * job.kt;
            return seq_cta_of(idx, total, seq_job_grid(total, grid));
        }
    };
    auto job_slot = [&](const SeqJob& job, int j, int32_t c, int32_t tile) -> int32_t {
        if constexpr (MOE) {
            int ph, prob;
            moe_info(j, ph, prob);
            const volatile int* z = m_ph + 5 * ph;
            return seq_slot(c, prob * job.tiles + tile, job.kt, z[0], z[4]);
        } else {
            const int32_t total = job.tiles * job.kt;
            return seq_slot(c, tile, job.kt, total, seq_job_grid(total, grid));
        }
    };
    // what tells a job's tagged partial sums from another job's: the job's index in a list; stage and problem of an
    // expert list (the same on every CTA)
    auto job_tag = [&](int j) -> int {
        if constexpr (MOE) {
            int ph, prob;
            moe_info(j, ph, prob);
            return ph * 2048 + prob;
        } else {
            return j;
        }
    };
    // the parts buffer of job j: the jobs of a list take sixteen in turn; a router table's CTAs each hand over at
    // most two split tiles per stage, so one buffer per stage serves
    auto job_parts = [&](int j) -> size_t { return MOE ? size_t(m_tab[j * kProbInts + 19] >> 16) : size_t(j & (kSeqPartBufs - 1)); };

    if (warp == kTcWarpProd) {
        // ================= packed-weight producer: runs through the whole job list =================
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            const bool drop = (P.debug & 2) != 0;  // host-set fault injection: never issue a copy
            int s = 0, issued = 0;
            uint32_t use = 0;
            bool ok = true;
            SeqJob job = P.moe_job;
            if (j_lo < j_hi) job = job_at(j_lo);
            for (int j = j_lo; j < j_hi && ok; ++j) {
                SeqJob next = job;
                if (j + 1 < j_hi) next = job_at(j + 1);  // in flight while this job streams
                GsWalker wk;
                wk.units = job.kt;
                job_range(job, j, wk.pos, wk.end);
                GsSeg sg;
                while (ok && wk.next(sg)) {
                    const uint8_t* src = job.payload + (uint64_t(sg.tile) * job.kt + uint64_t(sg.u0)) * kTcItemBytes;
                    for (int32_t left = sg.u1 - sg.u0; left > 0; left -= S) {
                        if (use > 0 && !seq_mbar_probe(sbase + SeqSmem::kBarEmpty + 8 * s, (use - 1) & 1, P.spin_limit)) {
                            seq_report(P.status, 71, j);
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
#ifdef QGEMV_SEQ_PROFILE
            long long prof[4] = {0, 0, 0, 0};
            const long long prof_start = clock64();
#endif
            SeqJob job = P.moe_job;
            if (j_lo < j_hi) job = job_at(j_lo);
            int pb = 0;        // plane buffer of job j: j % nbuf, kept as a counter (no division in this thread)
            uint32_t pph = 0;  // parity of that buffer's use: (j / nbuf) & 1
            for (int j = j_lo; j < j_hi && ok; ++j, pph ^= (pb + 1 == nb) ? 1u : 0u, pb = (pb + 1 == nb) ? 0 : pb + 1) {
                SeqJob next = job;
                if (j + 1 < j_hi) next = job_at(j + 1);
                const int32_t kt_len = job.kt;
                // the digit planes of this job (every CTA signals, also one without items)
                SEQ_PROF_T0();
                if (!seq_mbar_wait(sbase + SeqSmem::kBarXReady + 8 * pb, pph, P.spin_limit)) {
                    seq_report(P.status, 72, j);
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                SEQ_PROF_ADD(0);
                tc_fence_after();
                if (SEQ_STAMPS && P.trace) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 3] = globaltimer_ns();
                // this CTA's item range of the job, computed by the PLANES group
                const volatile int* rg = reinterpret_cast<const volatile int*>(sq_smem + SeqSmem::kRange) + pb * 2;
                const int32_t r_begin = rg[0], r_end = rg[1];
                const int32_t n_items = r_end - r_begin;
                const int32_t xs0 = n_items >= kt_len ? 0 : r_begin % kt_len;
                GsWalker wk;
                wk.units = kt_len, wk.pos = r_begin, wk.end = r_end;
                GsSeg sg;
                bool have = wk.next(sg);
                if (j == j_lo) tc_cp_sf2(tmem_sfb, sf_lo | (((sbase + SeqSmem::kSfb) >> 4) & 0x3FFFu), sf_hi);
                for (; ok && have; have = wk.next(sg)) {
                    // the accumulator is free once the epilogue of the segment before last has read it
                    {
                        SEQ_PROF_T0();
                        if (nseg >= 2 &&
                            !seq_mbar_probe(sbase + SeqSmem::kBarDFree + 8 * (nseg & 1), ((nseg >> 1) - 1) & 1, P.spin_limit)) {
                            seq_report(P.status, 73, int(nseg));
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                        SEQ_PROF_ADD(1);
                    }
                    tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (nseg & 1) * uint32_t(npad);
                    uint32_t acc = 0;
                    int32_t slot = sg.u0 - xs0;
                    if (slot < 0) slot += kt_len;
                    uint32_t x_lo = x_lo0 + uint32_t(pb) * (xbuf_bytes >> 4) + uint32_t(slot) * xslot16;
                    for (int32_t left = sg.u1 - sg.u0; left > 0; left -= S) {
                        // (the stage was written through the async proxy and is read through it: the
                        // barrier's acquire is all the ordering the MMAs need -- no tcgen05 fence here,
                        // which costs this thread a few hundred cycles per stage)
                        {
                            SEQ_PROF_T0();
                            if (!seq_mbar_probe(bar_full, full_par, P.spin_limit)) {
                                seq_report(P.status, 74, mi);
                                *abort_flag = 1;
                                ok = false;
                                break;
                            }
                            SEQ_PROF_ADD(2);
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
                        if (SEQ_STAMPS && P.trace && P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 7] == 0) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 7] = globaltimer_ns();
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
                if (SEQ_STAMPS && P.trace) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 4] = globaltimer_ns();
                // Barrier phases are told apart by one parity bit, so nobody may complete a barrier twice
                // before every waiter has seen the first completion: the planes of job j + 2 are only made
                // once this thread (here) and the epilogue group are through with job j.
                if (ok) mbar_arrive(sbase + SeqSmem::kBarMDone + 8 * pb);
                job = next;
            }
#ifdef QGEMV_SEQ_PROFILE
            if (P.trace) {   // per CTA: cycles waiting for planes, accumulators, weight stages; total
                prof[3] = clock64() - prof_start;
                for (int z = 0; z < 4; ++z) P.trace[size_t(gridDim.x) * P.trace_jobs * 8 + size_t(cta) * 4 + z] = (unsigned long long)prof[z];
            }
#endif
            *n_consumed = mi;
        }
        __syncwarp();
    } else {
        // ================= three independent warp groups, job after job =================
        // The chores of a job are round trips to global memory (activations in, results out, other
        // CTAs' partial sums), each most of a microsecond.  Run one after the other by the same warps
        // they cost 6-7 us per job; so they are dealt to three groups of four warps that only meet
        // through barriers in shared memory and tagged words in global memory:
        //   PLANES   (warps 2-5)   digit planes of job j into one of nbuf buffers, that many jobs ahead of
        //                          the epilogues.  Activations that an earlier job of the list produced are
        //                          taken word by word from that job's published output as the tags appear;
        //                          any other hazard the host found waits for fin[dep] on every CTA
        //   EPILOGUE (warps 6-9)   accumulators of job j's segments -> y rows (+ published words), or tagged
        //                          parts of a split tile
        //   FINISH   (warps 10-13) adds up the split tile this CTA is the first contributor of, in CTA order,
        //                          as the contributors' tagged parts appear; exchanges it between ranks where
        //                          the job says so; stores (and publishes) its rows; counts the job in fin[j]
        const int grp = (warp - kTcWarpConv0) >> 2;        // 0 PLANES, 1 EPILOGUE, 2 FINISH
        const int gt = threadIdx.x - 32 * (kTcWarpConv0 + 4 * grp);  // 0..127 inside the group
        const int bar_id = 1 + grp;                         // the group's named barrier
        const int Bl = P.B;
        unsigned int* all_max = reinterpret_cast<unsigned int*>(sq_smem + SeqSmem::kWarpMax);
        unsigned int* rowmax2 = reinterpret_cast<unsigned int*>(sq_smem + SeqSmem::kRowMax);  // [plane buffer][8]
        volatile int* decision = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kDecision) + grp;
        volatile int* fin_all = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kFinAll);
        // Named barriers have no time-out, so a group leaves its job loop at one place for all its
        // warps: one thread samples the abort flag, everybody reads that sample.
        int sample_no = 0;  // two sample slots in turn: the next sample cannot overwrite one that is still being read
        auto group_alive = [&]() -> bool {
            volatile int* slot = decision + 4 * (sample_no & 1);
            ++sample_no;
            if (gt == 0) *slot = *abort_flag;
            named_bar_sync(bar_id, 128);
            return *slot == 0;
        };
        // a bounded spin's budget: iterations, and two seconds of wall clock
        auto out_of_time = [&](int64_t it, uint64_t& t0) -> bool {
            if (it == 0) t0 = globaltimer_ns();
            return it >= P.spin_limit || ((it & 63) == 63 && globaltimer_ns() - t0 > 2000000000ull);
        };
        // bounded poll by the group's first thread until *counter == grid (every CTA has passed that point)
        auto poll_all = [&](const unsigned int* counter, int site, int j) {
            if (gt == 0) {
                uint64_t t0 = 0;
                for (int64_t it = 0; ld_acquire(counter) < unsigned(grid); ++it) {
                    if (*abort_flag) break;
                    if (out_of_time(it, t0)) {
                        seq_report(P.status, site, j);
                        *abort_flag = 1;
                        break;
                    }
                }
            }
        };
        pdl_wait();  // whatever ran before this launch has finished with x, y and the scratch, and has counted itself
        const uint32_t launch_no = MOE ? m_launch_no : __ldcg(P.barrier + 2), run_no = MOE ? m_run_no : __ldcg(P.fin + P.n_jobs);

        if (grp == 0) {
            // ---------------- PLANES ----------------
            const int wq = warp - kTcWarpConv0;  // 0..3
            unsigned int* wmax = all_max + wq * 8;
            if (gt < 128) {  // block scales of the planes: column n = 8 b + j carries 2^(2j - 6) in all four K blocks
                const int n = gt, jj = n & 7;
                const uint32_t byte = n < 8 * Bl ? uint32_t(2 * jj + 1) << 3 : 0u;
                *reinterpret_cast<volatile uint32_t*>(sq_smem + SeqSmem::kSfb + (n & 31) * 16 + (n >> 5) * 4) = byte * 0x01010101u;
            }
            SeqJob job = P.moe_job;
            if (j_lo < j_hi) job = job_at(j_lo);
            int pb = 0;        // plane buffer of job j (j % nbuf) and the parity of its use ((j / nbuf) & 1), as counters
            uint32_t pph = 0;
#ifdef QGEMV_SEQ_PROFILE
            long long pprof[4] = {0, 0, 0, 0};  // cycles of this group: waiting to start a job, fetching, row maxima, writing planes
            long long pt = clock64();
#define SEQ_PPROF(slot) { const long long now_ = clock64(); pprof[slot] += now_ - pt; pt = now_; }
#else
#define SEQ_PPROF(slot)
#endif
            for (int j = j_lo; j < j_hi; ++j, pph ^= (pb + 1 == nb) ? 1u : 0u, pb = (pb + 1 == nb) ? 0 : pb + 1) {
                SeqJob next = job;
                if (j + 1 < j_hi) next = job_at(j + 1);
                // the plane buffer and its row maxima were last used by job j - nbuf: its epilogues must be through
                if (j - j_lo >= nb && gt == 0 &&
                    !seq_mbar_wait(sbase + SeqSmem::kBarEDone + 8 * pb, (pph ^ 1u), P.spin_limit)) {
                    seq_report(P.status, 78, j);
                    *abort_flag = 1;
                }
                if (job.dep >= 0) poll_all(P.fin + job.dep, 80, j);  // an earlier job's buffers are involved
                if constexpr (MOE) {
                    // the second stage of an expert MLP reads the rows its problem's first stage wrote: all of that
                    // problem's row tiles must be counted (four warps each, on whichever CTAs held them)
                    if (P.n_phases == 2 && gt == 0) {
                        int ph, prob;
                        moe_info(j, ph, prob);
                        if (ph == 1) {
                            const unsigned want_warps = 4u * unsigned(P.moe_job.tiles);
                            uint64_t t0 = 0;
                            for (int64_t it = 0; ld_acquire(P.moe_cnt + prob) < want_warps; ++it) {
                                if (*abort_flag) break;
                                if (out_of_time(it, t0)) {
                                    seq_report(P.status, 86, prob);
                                    *abort_flag = 1;
                                    break;
                                }
                            }
                        }
                    }
                }
                const int32_t kt_len = job.kt;
                const int Bj = MOE ? job.rows : Bl;  // activation rows of this job
                int32_t r_begin, r_end;
                job_range(job, j, r_begin, r_end);
                const int32_t n_items = r_end - r_begin;
                const int32_t xs0 = n_items >= kt_len ? 0 : r_begin % kt_len;
                const int32_t n_slots = n_items >= kt_len ? kt_len : n_items;
                const uint32_t xb = xbase + uint32_t(pb) * xbuf_bytes;
                if (gt == 0) {  // for the MMA issuer: one thread there, and 64-bit divisions are slow
                    volatile int* rg = reinterpret_cast<volatile int*>(sq_smem + SeqSmem::kRange) + pb * 2;
                    rg[0] = r_begin, rg[1] = r_end;
                }
                if (gt < 32) all_max[gt] = 0u;
                if (!group_alive()) break;   // (its barrier also publishes the cleared maxima)
                SEQ_PPROF(0);
                if (P.trace && gt == 0) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 0] = globaltimer_ns();
                const int n_work = n_slots * Bj * 8;
                constexpr int kKeep = 4;
                const bool from_pub = job.src_off >= 0;
                const uint32_t want = seq_pub_tag(run_no, job.src_job) << 16;
                bool alive = true;
                // unit wu of this CTA's share: eight consecutive activations of row b; where they go in the planes
                auto unit_at = [&](int wu, int& b, uint32_t& dst) -> int {
                    const int o = wu & 7;
                    int slot = wu >> 3;
                    for (b = 0; slot >= n_slots; ++b) slot -= n_slots;  // b < 8: cheaper and smaller than a division
                    int32_t u = slot + xs0;
                    if (u >= kt_len) u -= kt_len;
                    dst = xb + uint32_t(slot) * xslot_bytes + uint32_t(b) * 256u + uint32_t(o >> 2) * 128u + uint32_t(o & 3) * 4u;
                    const int k0 = u * 64 + o * 8;
                    return k0 + 8 <= job.K ? k0 : -1;
                };
                auto pub_ok = [&](const uint4& a, const uint4& c) -> bool {
                    const uint32_t m = (a.x ^ want) | (a.y ^ want) | (a.z ^ want) | (a.w ^ want) | (c.x ^ want) | (c.y ^ want) | (c.z ^ want) | (c.w ^ want);
                    return (m >> 16) == 0u;
                };
                auto pub_pack = [&](const uint4& a, const uint4& c) -> uint4 {
                    return make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410), __byte_perm(c.x, c.y, 0x5410),
                                      __byte_perm(c.z, c.w, 0x5410));
                };
                // published words of a unit, re-read -- bounded -- until all eight carry the producing job's tag
                auto pub_wait = [&](const uint32_t* p, uint4 a, uint4 c) -> uint4 {
                    uint64_t t0 = 0;
                    for (int64_t it = 0; !pub_ok(a, c); ++it) {
                        if (*abort_flag || out_of_time(it, t0)) {
                            if (!*abort_flag) seq_report(P.status, 84, j);
                            *abort_flag = 1;
                            alive = false;
                            break;
                        }
                        a = ld_pub4(p), c = ld_pub4(p + 4);
                    }
                    return pub_pack(a, c);
                };
                // eight raw activations of row b from column k0 (of the row as it is stored)
                auto fetch8 = [&](int b, int k0) -> uint4 {
                    if (from_pub) {
                        const uint32_t* p = P.pub + size_t(job.src_off) + size_t(b) * size_t(job.x_stride) + size_t(k0);
                        return pub_wait(p, ld_pub4(p), ld_pub4(p + 4));
                    }
                    // possibly written by other SMs during an earlier job: read through L2, never a stale L1 line
                    const int64_t xr = MOE ? int64_t(job.rowmap[b]) : int64_t(b);  // gathered rows
                    return __ldcg(reinterpret_cast<const uint4*>(job.x + xr * job.x_stride + k0));
                };
                // ... and what the GEMV multiplies: the activation function and the norm weight applied (FUSE)
                auto shaped8 = [&](int b, int k0, uint4 v) -> uint4 {
                    if constexpr (ACT) {
                        if (job.act == 1) v = seq_silu_mul(v, fetch8(b, k0 + job.K));
                    }
                    if constexpr (FUSE) {
                        if (job.norm_w) v = seq_mul_w(v, __ldg(reinterpret_cast<const uint4*>(job.norm_w + k0)));
                    }
                    return v;
                };
                auto unit_src = [&](int wu, int& b, uint32_t& dst) -> uint4 {
                    const int k0 = unit_at(wu, b, dst);
                    if (k0 < 0) return make_uint4(0, 0, 0, 0);
                    return shaped8(b, k0, fetch8(b, k0));
                };
                if constexpr (FUSE) {
                    // RMS norm: every CTA needs the whole row's mean square (its own K range is only a part of the
                    // row): one more pass over the row, summed in a fixed order so that every CTA gets the same bits
                    if (job.norm_w) {
                        float* red = reinterpret_cast<float*>(all_max);        // 32 words, free until the maxima are taken
                        float* rowscale = reinterpret_cast<float*>(sq_smem + SeqSmem::kRowScale) + pb * 8;
                        for (int b = 0; b < Bl; ++b) {
                            float a = 0.f;
                            for (int k0 = gt * 8; k0 + 8 <= job.K; k0 += 128 * 8) {
                                uint4 v = fetch8(b, k0);
                                if (job.act == 1) v = seq_silu_mul(v, fetch8(b, k0 + job.K));
                                a += seq_sumsq(v);
                            }
                            for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, d);
                            if (lane == 0) red[wq] = a;
                            named_bar_sync(bar_id, 128);
                            if (gt == 0) rowscale[b] = rsqrtf((red[0] + red[1] + red[2] + red[3]) / float(job.K) + job.norm_eps);
                            named_bar_sync(bar_id, 128);
                        }
                        if (gt < 32) all_max[gt] = 0u;
                        named_bar_sync(bar_id, 128);
                    }
                }
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
                    for (int w = 0; w < 4; ++w) m = max(m, all_max[w * 8 + b]);
                    return m;
                };
                auto store_unit = [&](int b, uint32_t dst, const uint4& v) { seq_store_unit(dst, v, pow2i(-tc_row_exponent(row_max(b)))); };
                // More units than a thread keeps in registers (batches of several rows), read from memory as it is:
                // all of them are fetched at once by 16-byte asynchronous copies into the TOP of the job's plane
                // buffer (the raw values take half the room of their planes), the row maxima are taken from there,
                // and the planes are written from the bottom up in waves of four units per thread -- registers
                // first, a barrier, then the stores.  Groups of eight units (64 activations of one row, 128 bytes raw,
                // 256 bytes of planes) are numbered in address order; the planes of group g end at or below byte
                // 256 (g + 1) and the raw values of group g' start at (end of buffer) - 128 (G - g'), so a wave only
                // overwrites raw values of its own groups (already in registers) and of earlier waves.
                bool staged = !from_pub && n_work > kKeep * 128;
                if constexpr (ACT) staged = staged && job.act == 0;   // (gate and up values together are as large as their planes)
                if constexpr (FUSE) staged = staged && !job.norm_w;
                if (staged) {
                    const uint32_t raw0 = xb + uint32_t(n_slots) * xslot_bytes - uint32_t(n_slots * Bj) * 128u;
                    // a thread's units are 128 apart, i.e. 16 groups: (slot, row) of the next one without a division
                    const int g0 = gt >> 3, slot_first = g0 / Bj, b_first = g0 - slot_first * Bj;
                    const int q16 = 16 / Bj, r16 = 16 - q16 * Bj;
                    auto step = [&](int& slot, int& b) {
                        slot += q16, b += r16;
                        if (b >= Bj) b -= Bj, ++slot;
                    };
                    {
                        int slot = slot_first, b = b_first;
#pragma unroll 1
                        for (int wu = gt; wu < n_work; wu += 128, step(slot, b)) {
                            int32_t u = slot + xs0;
                            if (u >= kt_len) u -= kt_len;
                            const int64_t xr = MOE ? int64_t(job.rowmap[b]) : int64_t(b);
                            cp_async16(raw0 + uint32_t(wu) * 16u, job.x + xr * job.x_stride + u * 64 + (wu & 7) * 8);
                        }
                    }
                    cp_async_wait_all();
                    named_bar_sync(bar_id, 128);
                    SEQ_PPROF(1);
                    {   // row maxima: kept in a register while the row stays the same (it does when B divides 16)
                        int slot = slot_first, b = b_first, bm = b_first;
                        uint32_t m = 0;
#pragma unroll 1
                        for (int wu = gt; wu < n_work; wu += 256) {   // two units a round, their loads together
                            const bool two = wu + 128 < n_work;
                            const uint4 v0 = lds128(raw0 + uint32_t(wu) * 16u);
                            const uint4 v1 = two ? lds128(raw0 + uint32_t(wu + 128) * 16u) : make_uint4(0, 0, 0, 0);
                            const uint32_t m0 = unit_max(v0), m1 = unit_max(v1);
                            if (b != bm) {
                                if (m) atomicMax(wmax + bm, m);
                                bm = b, m = 0;
                            }
                            m = max(m, m0);
                            step(slot, b);
                            if (two) {
                                if (b != bm) {
                                    if (m) atomicMax(wmax + bm, m);
                                    bm = b, m = 0;
                                }
                                m = max(m, m1);
                                step(slot, b);
                            }
                        }
                        if (m) atomicMax(wmax + bm, m);
                    }
                    named_bar_sync(bar_id, 128);
                    SEQ_PPROF(2);
                    if (gt < 8) rowmax2[pb * 8 + gt] = row_max(gt);
                    {
                        int slot = slot_first, b = b_first;
#pragma unroll 1
                        for (int w0 = gt; w0 < n_work + gt; w0 += 4 * 128) {   // (the same number of rounds for every thread)
                            uint4 v[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                v[i] = make_uint4(0, 0, 0, 0);
                                if (w0 + i * 128 < n_work) v[i] = lds128(raw0 + uint32_t(w0 + i * 128) * 16u);
                            }
                            named_bar_sync(bar_id, 128);
                            const uint32_t in_group = uint32_t((gt & 7) >> 2) * 128u + uint32_t(gt & 3) * 4u;   // (unit mod 8 = gt mod 8)
#pragma unroll 1
                            for (int i = 0; i < 4; i += 2) {
                                const int b0 = b;
                                const uint32_t d0 = xb + uint32_t(slot) * xslot_bytes + uint32_t(b) * 256u + in_group;
                                step(slot, b);
                                const int b1 = b;
                                const uint32_t d1 = xb + uint32_t(slot) * xslot_bytes + uint32_t(b) * 256u + in_group;
                                step(slot, b);
                                if (w0 + i * 128 < n_work) store_unit(b0, d0, v[i]);
                                if (w0 + (i + 1) * 128 < n_work) store_unit(b1, d1, v[i + 1]);
                            }
                        }
                    }
                } else {
                uint4 keep[kKeep];
                int kb[kKeep];
                uint32_t kdst[kKeep];
                if (from_pub) {
                    // the loads of all kept units first, then the waits: one round trip when the words are there
                    uint4 ka[kKeep], kc[kKeep];
                    const uint32_t* kp[kKeep];
#pragma unroll
                    for (int i = 0; i < kKeep; ++i) {
                        const int wu = gt + i * 128;
                        kb[i] = 0, kdst[i] = 0, kp[i] = nullptr;
                        ka[i] = kc[i] = make_uint4(0, 0, 0, 0);
                        if (wu < n_work) {
                            const int k0 = unit_at(wu, kb[i], kdst[i]);
                            if (k0 >= 0) {
                                kp[i] = P.pub + size_t(job.src_off) + size_t(kb[i]) * size_t(job.x_stride) + size_t(k0);
                                ka[i] = ld_pub4(kp[i]), kc[i] = ld_pub4(kp[i] + 4);
                            }
                        }
                    }
                    {
                        uint64_t t0 = 0;
                        for (int64_t it = 0;; ++it) {
                            unsigned miss = 0;
#pragma unroll
                            for (int i = 0; i < kKeep; ++i)
                                if (kp[i] && !pub_ok(ka[i], kc[i])) miss |= 1u << i;
                            if (miss == 0) break;
                            if (*abort_flag || out_of_time(it, t0)) {
                                if (!*abort_flag) seq_report(P.status, 84, j);
                                *abort_flag = 1;
                                alive = false;
                                break;
                            }
#pragma unroll
                            for (int i = 0; i < kKeep; ++i)
                                if (miss & (1u << i)) ka[i] = ld_pub4(kp[i]), kc[i] = ld_pub4(kp[i] + 4);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < kKeep; ++i) keep[i] = kp[i] ? pub_pack(ka[i], kc[i]) : make_uint4(0, 0, 0, 0);
                    if constexpr (FUSE) {
                        if (job.act == 1 || job.norm_w) {
#pragma unroll 1
                            for (int i = 0; i < kKeep; ++i)
                                if (kp[i]) keep[i] = shaped8(kb[i], int(kp[i] - (P.pub + size_t(job.src_off) + size_t(kb[i]) * size_t(job.x_stride))), keep[i]);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < kKeep; ++i) {
                        const int wu = gt + i * 128;
                        kb[i] = 0, kdst[i] = 0;
                        keep[i] = make_uint4(0, 0, 0, 0);
                        if (wu < n_work) keep[i] = unit_src(wu, kb[i], kdst[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < kKeep; ++i) {
                    const uint32_t m = unit_max(keep[i]);
                    if (m) atomicMax(wmax + kb[i], m);
                }
                // The units beyond the kept ones (batches of several rows) are read twice, for the row maxima and
                // for the planes, four loads in flight at a time; both passes run the same code.
#pragma unroll 1
                for (int pass = 0; pass < 2; ++pass) {
                    if (pass == 1) {
                        named_bar_sync(bar_id, 128);
                        if (gt < 8) rowmax2[pb * 8 + gt] = row_max(gt);
#pragma unroll
                        for (int i = 0; i < kKeep; ++i)
                            if (gt + i * 128 < n_work) store_unit(kb[i], kdst[i], keep[i]);
                    }
#pragma unroll 1
                    for (int wu0 = gt + kKeep * 128; wu0 < n_work; wu0 += 4 * 128) {
                        uint4 v[4];
                        int vb[4];
                        uint32_t vdst[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            vb[i] = 0, vdst[i] = 0;
                            v[i] = make_uint4(0, 0, 0, 0);
                            if (wu0 + i * 128 < n_work) v[i] = unit_src(wu0 + i * 128, vb[i], vdst[i]);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (pass == 0) {
                                const uint32_t m = unit_max(v[i]);
                                if (m) atomicMax(wmax + vb[i], m);
                            } else if (wu0 + i * 128 < n_work) {
                                store_unit(vb[i], vdst[i], v[i]);
                            }
                        }
                    }
                }
                }
                fence_proxy_async_smem();  // the planes are read by the tensor core (async proxy)
                named_bar_sync(bar_id, 128);
                SEQ_PPROF(3);
                if (gt == 0) mbar_arrive(sbase + SeqSmem::kBarXReady + 8 * pb);
                if (P.trace && gt == 0) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 1] = globaltimer_ns();
                (void)alive;
                job = next;
            }
#ifdef QGEMV_SEQ_PROFILE
            if (P.trace && gt == 0)
                for (int z = 0; z < 4; ++z) P.trace[size_t(gridDim.x) * P.trace_jobs * 8 + size_t(gridDim.x) * 4 + size_t(cta) * 4 + z] = (unsigned long long)pprof[z];
#endif
        } else if (grp == 1) {
            // ---------------- EPILOGUE ----------------
            const int q = warp & 3;
            const uint32_t lane_base = uint32_t(32 * q) << 16;
            const int row = 32 * q + lane;
            uint32_t nseg = 0;
            int seen_all = -1;  // this thread's own knowledge of how far all CTAs have added their tiles up
            SeqJob job = P.moe_job;
            if (j_lo < j_hi) job = job_at(j_lo);
            int pb = 0;
            uint32_t pph = 0;
            for (int j = j_lo; j < j_hi; ++j, pph ^= (pb + 1 == nb) ? 1u : 0u, pb = (pb + 1 == nb) ? 0 : pb + 1) {
                SeqJob next = job;
                if (j + 1 < j_hi) next = job_at(j + 1);
                const int32_t kt_len = job.kt;
                const int Bj = MOE ? job.rows : Bl;
                // the planes of this job are ready, and with them this CTA's item range (a CTA without items
                // in a run of jobs would otherwise race ahead of the PLANES group and complete its barrier
                // twice before that group has looked)
                if (!*abort_flag && !seq_mbar_wait(sbase + SeqSmem::kBarXReady + 8 * pb, pph, P.spin_limit)) {
                    if (gt == 0) seq_report(P.status, 81, j);
                    *abort_flag = 1;
                }
                const volatile int* rg = reinterpret_cast<const volatile int*>(sq_smem + SeqSmem::kRange) + pb * 2;
                const int32_t rb = rg[0], re = rg[1];
                // A split tile's parts go to buffer j % kSeqPartBufs, last used by job j - kSeqPartBufs: every
                // CTA must have added that job's tiles up.  The FINISH group publishes how far that has come while
                // it waits; when its word is old this thread asks global memory itself -- first about a job half a
                // round of buffers later, so that one look serves the next eight jobs (a look per job would sit in
                // the MMA issuer's way: it waits for the accumulator this group has not read yet).
                if (!MOE && re > rb && (rb % kt_len != 0 || re % kt_len != 0) && j >= kSeqPartBufs && gt == 0 &&
                    max(int(*fin_all), seen_all) < j - kSeqPartBufs) {
                    if (ld_acquire(P.fin + (j - kSeqPartBufs / 2)) >= unsigned(grid)) {
                        seen_all = j - kSeqPartBufs / 2;
                    } else {
                        uint64_t t0 = 0;
                        for (int64_t it = 0;; ++it) {
                            // (asked directly: this CTA's FINISH group may itself be waiting for the part written below)
                            if (*abort_flag) break;
                            if (ld_acquire(P.fin + (j - kSeqPartBufs)) >= unsigned(grid)) {
                                seen_all = j - kSeqPartBufs;
                                break;
                            }
                            if (out_of_time(it, t0)) {
                                seq_report(P.status, 79, j);
                                *abort_flag = 1;
                                break;
                            }
                        }
                    }
                }
                if (!group_alive()) break;
                const uint32_t part_tag = seq_part_tag(launch_no, job_tag(j)), pub_tag = seq_pub_tag(run_no, j) << 16;
                GsWalker wk;
                wk.units = kt_len, wk.pos = rb, wk.end = re;
                GsSeg sg;
                bool ok = true;
                while (wk.next(sg)) {
                    if (!ok) continue;  // this warp gave up: it still reaches the group's barriers below
                    const bool whole = sg.u0 == 0 && sg.u1 == kt_len;
                    const uint32_t acc = nseg & 1;
                    if (!__all_sync(0xFFFFFFFFu, seq_mbar_probe(sbase + SeqSmem::kBarDFull + 8 * acc, (nseg >> 1) & 1, P.spin_limit))) {
                        if (lane == 0) seq_report(P.status, 76, int(nseg));
                        *abort_flag = 1;
                        ok = false;
                        continue;
                    }
                    tc_fence_after();
                    if (P.trace && gt == 0) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 5] = globaltimer_ns();  // the last one stays
                    const int n = sg.tile * 128 + row;
                    // every contributor after the first starts its range inside this tile (slot 0 of its
                    // pair); the first one's range may have started in an earlier tile
                    unsigned long long* slot = nullptr;
                    if (!whole) {
                        const int32_t c_lo = job_cta_of(job, j, sg.tile * kt_len);
                        const int32_t my_slot = cta == c_lo ? job_slot(job, j, c_lo, sg.tile) : 2 * cta;
                        slot = P.ws + (job_parts(j) * size_t(2 * grid) + size_t(my_slot)) * 1024 + row;
                    }
                    // (one row of the batch after the other, not unrolled: the code of this group has to stay small)
#pragma unroll 1
                    for (int b = 0; b < Bj; ++b) {
                        uint32_t r[8];
                        tmem_ld8(tmem_base + lane_base + acc * uint32_t(npad) + uint32_t(8 * b), r);
                        float a = __uint_as_float(r[0]);
#pragma unroll
                        for (int z = 1; z < 8; ++z) a += __uint_as_float(r[z]);
                        // (the MMAs of this job have run, so its planes and row maxima are there)
                        a *= job.tensor_scale * pow2i(tc_row_exponent(rowmax2[pb * 8 + b]) + 7);
                        if constexpr (FUSE) {
                            if (job.norm_w) a *= reinterpret_cast<const float*>(sq_smem + SeqSmem::kRowScale)[pb * 8 + b];
                        }
                        if (!whole) {
                            st_tagged(slot + b * 128, a, part_tag);
                        } else if (n < job.N) {
                            const int64_t idx = (MOE ? int64_t(job.rowmap[8 + b]) : int64_t(b)) * job.N + n;  // scattered rows
                            if constexpr (FUSE) {
                                if (job.residual)
                                    a += job.y_dtype == QGEMV_OUT_F32 ? __ldcg(static_cast<const float*>(job.residual) + idx)
                                                                      : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(job.residual) + idx));
                            }
                            if (job.y_dtype == QGEMV_OUT_F32) {
                                static_cast<float*>(job.y)[idx] = a;
                            } else {
                                const __nv_bfloat16 hv = __float2bfloat16_rn(a);
                                static_cast<__nv_bfloat16*>(job.y)[idx] = hv;
                                if (job.pub_off >= 0) st_pub(P.pub + size_t(job.pub_off) + size_t(idx), pub_tag | uint32_t(__bfloat16_as_ushort(hv)));
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(sbase + SeqSmem::kBarDFree + 8 * acc);  // the accumulator may be overwritten
                    if constexpr (MOE) {
                        if (P.n_phases == 2 && whole && lane == 0) {   // this warp's rows of a first-stage tile are stored
                            int ph, prob;
                            moe_info(j, ph, prob);
                            if (ph == 0) red_release_add(P.moe_cnt + prob, 1u);
                        }
                    }
                    ++nseg;
                }
                if (P.trace && gt == 0) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 2] = globaltimer_ns();
                // this CTA's rows and parts of job j are stored; its plane buffer may be reused
                named_bar_sync(bar_id, 128);
                if (gt == 0) {
                    if (!*abort_flag && !seq_mbar_wait(sbase + SeqSmem::kBarMDone + 8 * pb, pph, P.spin_limit)) {
                        seq_report(P.status, 82, j);
                        *abort_flag = 1;
                    }
                    mbar_arrive(sbase + SeqSmem::kBarEDone + 8 * pb);  // first: the PLANES group may be waiting
                    st_release_cta_shared(sbase + SeqSmem::kEpiDone, j - j_lo + 1);  // for the FINISH group's count of the job
                }
                job = next;
            }
        } else {
            // ---------------- FINISH ----------------
            int known = -1;  // jobs up to here are added up on every CTA (published in fin_all)
#ifdef QGEMV_SEQ_PROFILE
            long long fprof[4] = {0, 0, 0, 0};  // cycles of this group's first thread: waiting for the epilogues, partial sums, push, gather
            long long ft = clock64();
#define SEQ_FPROF(slot) if (gt == 0) { const long long now_ = clock64(); fprof[slot] += now_ - ft; ft = now_; }
#define SEQ_FPROF_MARK() if (gt == 0) ft = clock64()
#else
#define SEQ_FPROF(slot)
#define SEQ_FPROF_MARK()
#endif
            SeqJob job = P.moe_job;
            if (j_lo < j_hi) job = job_at(j_lo);
            TpExchange X;
            X.buf = P.xbuf, X.rank = P.rank, X.world = P.world, X.max_elems = P.x_max_elems;
            X.tag = 0u, X.par_off = 0;
            if (P.world > 1) {
                X.tag = __ldcg(P.barrier + 1) + 1u;
                X.par_off = size_t(X.tag & 1u) * size_t(P.world) * size_t(P.x_max_elems);
            }
            for (int j = j_lo; j < j_hi; ++j) {
                SeqJob next = job;
                if (j + 1 < j_hi) next = job_at(j + 1);
                // is this CTA the first contributor of a split tile of job j?  (only its last segment can be)
                const int32_t kt_len = job.kt;
                const int Bj = MOE ? job.rows : Bl;
                int32_t rb, re;
                job_range(job, j, rb, re);
                bool pending = false;
                int32_t tile = 0, c_lo = 0, c_hi = 0, lo_slot = 0;
                if (re > rb && re % kt_len != 0) {
                    tile = (re - 1) / kt_len;
                    c_lo = job_cta_of(job, j, tile * kt_len);
                    c_hi = job_cta_of(job, j, (tile + 1) * kt_len - 1);
                    pending = c_lo == cta;
                    lo_slot = job_slot(job, j, c_lo, tile);
                }
                // (how far ALL CTAs have come -- fin_all, which lets the epilogues reuse a parts buffer without asking
                // global memory themselves -- is looked up below while this group waits anyway: a probe here would put
                // a round trip to L2 into every job of a group whose time per job bounds the small jobs)
                if (!group_alive()) break;
                SEQ_FPROF_MARK();
                // this CTA's own part of the tile comes first, and the other contributors finish at about the same
                // time: nothing is asked of global memory before this CTA's epilogues are through with the job
                if (gt == 0) {
                    uint64_t t0 = 0;
                    for (int64_t it = 0; ld_acquire_cta_shared(sbase + SeqSmem::kEpiDone) <= j - j_lo; ++it) {
                        if (*abort_flag) break;
                        // (the epilogue may itself be waiting for fin_all to move before it reuses a parts buffer)
                        if (!MOE && known + 1 < j && ld_acquire(P.fin + known + 1) >= unsigned(grid)) {
                            *fin_all = ++known;
                        } else {
                            __nanosleep(100);
                        }
                        if (out_of_time(it, t0)) {
                            seq_report(P.status, 85, j);
                            *abort_flag = 1;
                            break;
                        }
                    }
                }
                named_bar_sync(bar_id, 128);
                SEQ_FPROF(0);
                if (pending) {
                    const int n = tile * 128 + gt;
                    const unsigned long long* parts = P.ws + job_parts(j) * size_t(2 * grid) * 1024 + gt;
                    const uint32_t part_tag = seq_part_tag(launch_no, job_tag(j)), pub_tag = seq_pub_tag(run_no, j) << 16;
                    if (n < job.N && !*abort_flag) {
                        bool have = true;
                        uint64_t t0 = 0;
                        int64_t spins = 0;
                        // (one row of the batch after the other, not unrolled: this group's code has to stay small --
                        // five roles run different code on the SM at once and share its instruction cache)
#pragma unroll 1
                        for (int b = 0; b < Bj && have; ++b) {
                            // the first contributor's own part, then the others eight at a time: the loads of a group
                            // are in flight together, the ones whose tag is not there yet are re-read together
                            // -- bounded --, and the additions stay in CTA order
                            float a = 0.f;
#pragma unroll 1
                            for (int32_t cc = c_lo; cc <= c_hi && have; cc += 8) {
                                const unsigned long long* pz[8];
                                unsigned long long t[8];
#pragma unroll
                                for (int z = 0; z < 8; ++z) {
                                    const int32_t c = min(cc + z, c_hi);
                                    pz[z] = parts + size_t(c == c_lo ? lo_slot : 2 * c) * 1024 + b * 128;
                                    t[z] = ld_flagged(pz[z]);
                                }
                                for (;;) {
                                    unsigned miss = 0;
#pragma unroll
                                    for (int z = 0; z < 8; ++z)
                                        if (uint32_t(t[z] >> 32) != part_tag) miss |= 1u << z;
                                    if (miss == 0) break;
                                    if (*abort_flag || out_of_time(spins++, t0)) {
                                        if (!*abort_flag) seq_report(P.status, 77, cc + __ffs(int(miss)) - 1);
                                        *abort_flag = 1;
                                        have = false;
                                        break;
                                    }
#pragma unroll
                                    for (int z = 0; z < 8; ++z)
                                        if (miss & (1u << z)) t[z] = ld_flagged(pz[z]);
                                }
#pragma unroll
                                for (int z = 0; z < 8; ++z)
                                    if (cc + z <= c_hi) a = (cc + z == c_lo) ? __uint_as_float(uint32_t(t[z])) : a + __uint_as_float(uint32_t(t[z]));
                            }
                            if (!have) break;
                            const int64_t idx = (MOE ? int64_t(job.rowmap[8 + b]) : int64_t(b)) * job.N + n;
                            SEQ_FPROF(1);
                            if (job.xoff >= 0) {
                                // this rank's partial sum out to every rank, then the ranks' sums for this row, added in rank order
                                X.push(int64_t(job.xoff) + idx, a);
                                SEQ_FPROF(2);
                                float part[kTpMaxWorld];
                                int missing = 0;
                                if (X.gather(int64_t(job.xoff) + idx, part, P.spin_limit, missing)) {
                                    SEQ_FPROF(3);
                                    a = part[0];
                                    for (int r = 1; r < P.world; ++r) a += part[r];
                                } else {
                                    seq_report(P.status, 83, missing);
                                    *abort_flag = 1;
                                    have = false;
                                    break;
                                }
                            }
                            if constexpr (FUSE) {
                                if (job.residual)
                                    a += job.y_dtype == QGEMV_OUT_F32 ? __ldcg(static_cast<const float*>(job.residual) + idx)
                                                                      : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(job.residual) + idx));
                            }
                            if (job.y_dtype == QGEMV_OUT_F32) {
                                static_cast<float*>(job.y)[idx] = a;
                            } else {
                                const __nv_bfloat16 hv = __float2bfloat16_rn(a);
                                static_cast<__nv_bfloat16*>(job.y)[idx] = hv;
                                if (job.pub_off >= 0) st_pub(P.pub + size_t(job.pub_off) + size_t(idx), pub_tag | uint32_t(__bfloat16_as_ushort(hv)));
                            }
                        }
                    }
                }
                if constexpr (MOE) {
                    if (P.n_phases == 2 && pending) {   // (uniform over the group)
                        __syncwarp();
                        if (lane == 0 && !*abort_flag) {
                            int ph, prob;
                            moe_info(j, ph, prob);
                            if (ph == 0) red_release_add(P.moe_cnt + prob, 1u);
                        }
                    }
                }
                if (P.trace && gt == 0) P.trace[(size_t(cta) * P.trace_jobs + (j - j_lo)) * 8 + 6] = globaltimer_ns();
                // (the epilogues of the job are through, see above: fin[j] == grid means that all of y is there)
                named_bar_sync(bar_id, 128);
                // The counter is what a later job with a `dep` on this one waits for before it reads this job's rows, and
                // what the epilogues ask before they reuse a parts buffer.  Only the first needs release semantics: the
                // partial sums this group read have arrived (their values are in the rows) whatever the order of the
                // bump.  A release here would also wait for the exchange's stores to the other ranks to be
                // acknowledged over the link -- microseconds, in the group whose time per job bounds small jobs.
                if (!MOE && gt == 0) {
                    if (job.fin_release) {
                        red_release_add(P.fin + j, 1u);
                    } else {
                        red_relaxed_add(P.fin + j, 1u);
                    }
                }
                job = next;
            }
#ifdef QGEMV_SEQ_PROFILE
            if (P.trace && gt == 0)
                for (int z = 0; z < 4; ++z) P.trace[size_t(gridDim.x) * P.trace_jobs * 8 + size_t(gridDim.x) * 8 + size_t(cta) * 4 + z] = (unsigned long long)fprof[z];
#endif
        }
    }
    // ---- every role is through (or has given up): the last CTA to leave puts the counters back to zero ----
    __syncthreads();
    if constexpr (MOE) {
        if (P.trace && threadIdx.x == 0) P.trace[size_t(grid) * P.trace_jobs * 8 + size_t(cta) * 4 + 2] = globaltimer_ns();
    }
    if (threadIdx.x == 0 && !*abort_flag && atom_release_add(P.barrier, 1u) == unsigned(grid) - 1u) {
        for (int i = 0; i < P.n_jobs; ++i) P.fin[i] = 0u;  // nobody polls any more
        if constexpr (MOE) {
            if (P.n_phases == 2)
                for (int i = 0; i < m_nprob; ++i) P.moe_cnt[i] = 0u;
        }
        P.barrier[0] = 0u;
        if (P.world > 1) P.barrier[1] = P.barrier[1] + 1u;  // the tag of the next launch's exchange
        P.barrier[2] = P.barrier[2] + 1u;                   // of the next launch's partial sums
        P.fin[P.n_jobs] = P.fin[P.n_jobs] + 1u;             // of this job list's next published words
    }
    // ---- release tensor memory (always), after every role is done with it ----
    tc_fence_before();
    __syncthreads();
    if (warp == kTcWarpMma) {
        __syncwarp();
        if (*abort_flag) {
            if (lane == 0) {
                tc_commit(sbase + SeqSmem::kBarDrain);
                (void)seq_mbar_probe(sbase + SeqSmem::kBarDrain, 0, int64_t(1) << 16);
            }
            __syncwarp();
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, ncols);
    } else if (threadIdx.x == 0 && *abort_flag) {
        // never leave with copies in flight: wait (bounded) for every copy that nothing consumed
        const int issued = *n_issued;
        for (int i = *n_consumed; i < issued; ++i)
            (void)seq_mbar_wait(sbase + SeqSmem::kBarFull + 8 * (i % R), uint32_t(i / R) & 1u, int64_t(1) << 20);
    }
}

}  // namespace qg
