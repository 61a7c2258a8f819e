// Dense weight-streaming GEMV, "warp-stream" schedule: the fast path whenever the f16 activation
// fragments of the whole K extent fit in shared memory (units * batch <= 512).
//
// One CTA per SM owns a contiguous range of (panel, unit) blocks.  Inside the CTA each of the
// sixteen consumer warps owns a fixed K slice of every panel (units [w*S, (w+1)*S), S =
// ceil(units / 16)) and runs its own private pipeline: lane 0 issues bulk (TMA) copies of up to
// four consecutive units of that slice into the warp's own ring of shared-memory slots, each slot
// with its own mbarrier, and the same warp consumes them.  No barrier is shared between consumer
// warps while streaming: a warp only waits for its own copies.  When a warp has finished its slice
// of a panel it hands its 16 x 8 partial tile to the epilogue warp through a two-slot exchange;
// the epilogue warp sums the sixteen slices in warp order, scales and stores (or parks a partial
// sum for the last CTA of a split panel).
//
// Activations are converted once per kernel by the consumer warps: every bf16 row is scaled by a
// power of two so that its largest magnitude lands in [2^14, 2^15) and written as f16 MMA
// fragments; the scaling is exact and is undone in fp32 when a panel is handed over.
#pragma once
#include "gemv_kernel.cuh"

namespace qg {

constexpr int kSWarps = 16;                        // consumer warps
constexpr int kSEpilogueWarp = kSWarps;            // warp 16
constexpr int kSThreads = 32 * (kSWarps + 1);      // 544
constexpr int kSXBufBytes = 65536;                 // resident f16 activation fragments
constexpr int kSMaxUnitsTimesBatch = kSXBufBytes / 128;  // 512
constexpr int kSRedSlots = 2;

template <int FMT>
struct StreamTraits;
template <>
struct StreamTraits<QGEMV_FMT_NVFP4> {
    static constexpr int kChunkUnits = 4;  // 2304 bytes per copy
    static constexpr int kRing = 3;
};
template <>
struct StreamTraits<QGEMV_FMT_FP8> {
    static constexpr int kChunkUnits = 2;  // 2048 bytes per copy
    static constexpr int kRing = 4;
};

struct SSmem {
    static constexpr int kBarFull = 0;        // kSWarps * 4 * 8 = 512 bytes
    static constexpr int kBarRedFull = 512;   // 4 groups * kSRedSlots * 8
    static constexpr int kBarRedEmpty = 576;  // 4 groups * kSRedSlots * 8
    static constexpr int kRowMax = 640;       // 8 words
    static constexpr int kRowExp = 672;       // 8 words
    static constexpr int kAbort = 704;
    static constexpr int kZero = 720;         // 16 zero bytes
    static constexpr int kXBuf = 1024;
    static constexpr int kRed = kXBuf + kSXBufBytes;                   // kSRedSlots * kSWarps * 512
    static constexpr int kRing0 = kRed + kSRedSlots * kSWarps * 512;
    template <int FMT>
    __host__ __device__ static constexpr int total() {
        constexpr int split_ring = StreamTraits<FMT>::kRing;
        constexpr int ring_slots = split_ring > 4 ? split_ring : 4;  // whole-panel kernel: 4 chunk slots
        return kRing0 + kSWarps * ring_slots * StreamTraits<FMT>::kChunkUnits * FmtTraits<FMT>::kUnitBytes;
    }
};

// The activation staging (stream_convert_x) converts at most two (phase, row) pairs per consumer
// warp, a phase being 16 units, and lays a phase out as batch * 2048 bytes: the gate therefore
// counts whole phases.  units * batch <= 512 alone would admit ragged K with 33..35 pairs
// (e.g. 72 units at batch 7), more than the warps convert and than the buffer holds.
inline bool use_stream_path(bool dense, int batch, int64_t units) {
    const int64_t n_phases = (units + QG_PHASE_UNITS - 1) / QG_PHASE_UNITS;
    return dense && batch >= 1 && n_phases * batch <= 2 * kSWarps &&
           n_phases * batch * (QG_PHASE_UNITS * 128) <= kSXBufBytes;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// The units of panel p that belong to this CTA's range [a, b) of the linear (panel, unit) space.
struct PanelRange {
    int lo, hi;
};
__device__ __forceinline__ PanelRange cta_panel_range(int p, int p_first, int p_last, int u_first,
                                                      int u_last_end, int units) {
    PanelRange r;
    r.lo = (p == p_first) ? u_first : 0;
    r.hi = (p == p_last) ? u_last_end : units;
    return r;
}

// Cursor over the chunks of one warp: panels in order, inside a panel the warp's slice in steps
// of kChunkUnits.
template <int CH>
struct ChunkCursor {
    int p, c0, hi;  // current panel, first unit of the chunk, end of the warp's units in the panel
    int p_first, p_last, u_first, u_last_end, units, s_lo, s_hi;
    __device__ __forceinline__ void settle() {
        while (p <= p_last) {
            const PanelRange r = cta_panel_range(p, p_first, p_last, u_first, u_last_end, units);
            const int lo = max(r.lo, s_lo);
            hi = min(r.hi, s_hi);
            if (c0 < lo) c0 = lo;
            if (c0 < hi) return;
            ++p;
            c0 = 0;
        }
    }
    __device__ __forceinline__ void init(int p_first_, int p_last_, int u_first_, int u_last_end_, int units_,
                                         int s_lo_, int s_hi_) {
        p_first = p_first_, p_last = p_last_, u_first = u_first_, u_last_end = u_last_end_;
        units = units_, s_lo = s_lo_, s_hi = s_hi_;
        p = p_first;
        c0 = 0;
        hi = 0;
        settle();
    }
    __device__ __forceinline__ bool valid() const { return p <= p_last; }
    __device__ __forceinline__ int count() const { return min(CH, hi - c0); }
    __device__ __forceinline__ void advance() {
        c0 += CH;
        if (c0 >= hi) {
            ++p;
            c0 = 0;
        }
        settle();
    }
};

// Loads this lane's activation fragments of one unit (two block pairs) or zeros for lanes whose
// batch column does not exist.
__device__ __forceinline__ void load_bfrag(uint32_t (&bf)[8], bool xlane, uint32_t xunit, uint32_t xpair) {
    if (xlane) {
        const uint4 x0 = lds128(xunit);
        const uint4 x1 = lds128(xunit + xpair);
        bf[0] = x0.x, bf[1] = x0.y, bf[2] = x0.z, bf[3] = x0.w;
        bf[4] = x1.x, bf[5] = x1.y, bf[6] = x1.z, bf[7] = x1.w;
    } else {
#pragma unroll
        for (int z = 0; z < 8; ++z) bf[z] = 0u;
    }
}

// Activations: bf16 rows -> f16 MMA fragments with one power-of-two scale per row.  Runs on the
// sixteen consumer warps; at most two (phase, row) pairs per warp.  Ends with every fragment and
// the row exponents visible to all consumer warps.
__device__ __forceinline__ void stream_convert_x(const GemvParams& P, unsigned char* smem_raw, uint32_t sbase,
                                                 int w, int lane) {
    const int Bl = P.B, units = P.units;
    unsigned int* rowmax = reinterpret_cast<unsigned int*>(smem_raw + SSmem::kRowMax);
    int* rowexp = reinterpret_cast<int*>(smem_raw + SSmem::kRowExp);
    const int n_phases = (units + QG_PHASE_UNITS - 1) / QG_PHASE_UNITS;
    const int n_pairs = n_phases * Bl;  // <= 32
    const uint32_t phase_bytes = uint32_t(Bl) * 2048u;
    RowRegs r0, r1;
    const int i0 = w, i1 = w + kSWarps;
    const int f_0 = i0 / Bl, b_0 = i0 - f_0 * Bl, f_1 = i1 / Bl, b_1 = i1 - f_1 * Bl;
    const int e_0 = min(units, (f_0 + 1) * QG_PHASE_UNITS), e_1 = min(units, (f_1 + 1) * QG_PHASE_UNITS);
    if (i0 < n_pairs) {
        const uint32_t m = load_row(r0, P.x + int64_t(b_0) * P.x_stride, P.K, f_0, f_0 * QG_PHASE_UNITS, e_0, lane);
        if (lane == 0) atomicMax(rowmax + b_0, m);
    }
    if (i1 < n_pairs) {
        const uint32_t m = load_row(r1, P.x + int64_t(b_1) * P.x_stride, P.K, f_1, f_1 * QG_PHASE_UNITS, e_1, lane);
        if (lane == 0) atomicMax(rowmax + b_1, m);
    }
    named_bar_sync(1, 32 * kSWarps);
    if (i0 < n_pairs)
        store_row(r0, row_exponent(rowmax[b_0]), f_0, f_0 * QG_PHASE_UNITS, e_0,
                  sbase + SSmem::kXBuf + f_0 * phase_bytes, Bl, b_0, lane);
    if (i1 < n_pairs)
        store_row(r1, row_exponent(rowmax[b_1]), f_1, f_1 * QG_PHASE_UNITS, e_1,
                  sbase + SSmem::kXBuf + f_1 * phase_bytes, Bl, b_1, lane);
    if (w == 0 && lane < 8) rowexp[lane] = lane < Bl ? row_exponent(rowmax[lane]) : 0;
    named_bar_sync(1, 32 * kSWarps);
}

template <int FMT>
__global__ void __launch_bounds__(kSThreads, 1) gemv_stream_kernel(const GemvParams P) {
    using ST = StreamTraits<FMT>;
    constexpr int kUnitBytes = FmtTraits<FMT>::kUnitBytes;
    constexpr int CH = ST::kChunkUnits;
    constexpr int kRing = ST::kRing;
    constexpr int kSlotBytes = CH * kUnitBytes;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Bl = P.B;
    const int units = P.units;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kSWarps * kRing; ++i) mbar_init(sbase + SSmem::kBarFull + 8 * i, 1);
        for (int i = 0; i < kSRedSlots; ++i) {
            mbar_init(sbase + SSmem::kBarRedFull + 8 * i, kSWarps);
            mbar_init(sbase + SSmem::kBarRedEmpty + 8 * i, 1);
        }
        for (int b = 0; b < 8; ++b) reinterpret_cast<volatile unsigned int*>(smem_raw + SSmem::kRowMax)[b] = 0u;
        *reinterpret_cast<volatile int*>(smem_raw + SSmem::kAbort) = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    const int64_t total = int64_t(P.n_panels) * units;
    const int grid = total < int64_t(gridDim.x) ? int(total) : int(gridDim.x);
    const int cta = blockIdx.x;
    if (cta >= grid) return;
    // this CTA's range [a, b) of the linear (panel, unit) space, as panels and unit offsets
    const int64_t a = (int64_t(cta) * total) / grid, b = (int64_t(cta + 1) * total) / grid;
    const int p_first = int(a / units), u_first = int(a - int64_t(p_first) * units);
    const int p_last = int((b - 1) / units), u_last_end = int(b - int64_t(p_last) * units);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + SSmem::kAbort);

    if (warp == kSEpilogueWarp) {
        // ================= epilogue: reduce the sixteen K slices of each panel, scale, store =================
        pdl_wait();  // outputs and workspace may still be in use by the preceding kernel
        const float ts = (FMT == QGEMV_FMT_NVFP4) ? P.tensor_scale[0] : 1.0f;
        const uint32_t red = sbase + SSmem::kRed + lane * 16;
        uint32_t rcnt = 0;
        for (int p = p_first; p <= p_last; ++p, ++rcnt) {
            const int rs = rcnt % kSRedSlots;
            if (!mbar_wait(sbase + SSmem::kBarRedFull + 8 * rs, (rcnt / kSRedSlots) & 1, P.spin_limit, 200u)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 6, int(rcnt));
                *abort_flag = 1;
                return;
            }
            float4 v = lds128f(red + (rs * kSWarps) * 512);
#pragma unroll
            for (int ww = 1; ww < kSWarps; ++ww) {
                const float4 q = lds128f(red + (rs * kSWarps + ww) * 512);
                v.x += q.x, v.y += q.y, v.z += q.z, v.w += q.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + SSmem::kBarRedEmpty + 8 * rs);
            v.x *= ts, v.y *= ts, v.z *= ts, v.w *= ts;
            const PanelRange r = cta_panel_range(p, p_first, p_last, u_first, u_last_end, units);
            if (r.lo == 0 && r.hi == units) {
                store_panel<FMT>(P, v, lane, p, Bl, nullptr, P.chan_scale);
            } else {
                finish_partial<FMT>(P, v, lane, p, p, cta, grid, total, Bl, nullptr, P.chan_scale);
            }
        }
        return;
    }

    // ================= consumer warps =================
    const int w = warp;
    const int g = lane >> 2, t = lane & 3;
    // ---- this warp's K slice and its private copy ring ----
    const int S = (units + kSWarps - 1) / kSWarps;
    const int s_lo = min(units, w * S), s_hi = min(units, (w + 1) * S);
    const uint32_t ring = sbase + SSmem::kRing0 + w * (kRing * kSlotBytes);
    const uint32_t bars = sbase + SSmem::kBarFull + 8 * (w * kRing);
    const uint64_t pol = policy_evict_first();
    const bool drop = (P.debug & 2) != 0;  // host-set fault injection: never issue a copy
    ChunkCursor<CH> issue_cur, cons_cur;
    issue_cur.init(p_first, p_last, u_first, u_last_end, units, s_lo, s_hi);
    cons_cur = issue_cur;
    int issued = 0, consumed = 0;

    auto issue_one = [&]() {  // lane 0 only
        const int slot = issued % kRing;
        const uint32_t bytes = uint32_t(issue_cur.count()) * kUnitBytes;
        const uint64_t off = (uint64_t(issue_cur.p) * units + issue_cur.c0) * kUnitBytes;
        if ((P.debug & 1) && off + bytes > P.payload_bytes) {
            report(P.status, QGEMV_ERR_BOUNDS, 2, issue_cur.p);
            return;
        }
        if (!drop) {
            mbar_arrive_expect_tx(bars + 8 * slot, bytes);
            bulk_g2s(ring + slot * kSlotBytes, P.payload + off, bytes, bars + 8 * slot, pol);
        }
    };
    // prologue: fill the ring
    for (int i = 0; i < kRing && issue_cur.valid(); ++i) {
        if (lane == 0) issue_one();
        ++issued;
        issue_cur.advance();
    }
    // weights never depend on the preceding kernel; activations do
    pdl_wait();
    stream_convert_x(P, smem_raw, sbase, w, lane);
    const int* rowexp = reinterpret_cast<const int*>(smem_raw + SSmem::kRowExp);
    const float fs0 = pow2i(rowexp[2 * t]), fs1 = pow2i(rowexp[2 * t + 1]);

    // activation fragment addressing: unit u, pair pp, row g, column slice t
    const bool xlane = g < Bl;
    const uint32_t xpair = uint32_t(Bl) * 64u;
    const uint32_t xlane_base = sbase + SSmem::kXBuf + g * 64 + t * 16;
    const uint32_t red = sbase + SSmem::kRed + w * 512 + lane * 16;
    uint32_t rcnt = 0;
    bool ok = true;

    for (int p = p_first; p <= p_last && ok; ++p, ++rcnt) {
        float cA[4] = {0.f, 0.f, 0.f, 0.f}, cB[4] = {0.f, 0.f, 0.f, 0.f};
        while (cons_cur.valid() && cons_cur.p == p) {
            const int slot = consumed % kRing;
            if (!mbar_wait(bars + 8 * slot, (consumed / kRing) & 1, P.spin_limit)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 5, consumed);
                *abort_flag = 1;
                ok = false;
                break;
            }
            const int n = cons_cur.count();
            const uint32_t st = ring + slot * kSlotBytes;
            const uint32_t xu = xlane_base + uint32_t(cons_cur.c0) * 2u * xpair;
            uint32_t bfA[8], bfB[8];
#pragma unroll
            for (int j = 0; j < CH; j += 2) {
                if (j + 1 < n) {
                    load_bfrag(bfA, xlane, xu + j * 2 * xpair, xpair);
                    load_bfrag(bfB, xlane, xu + (j + 1) * 2 * xpair, xpair);
                    consume_two<FMT>(cA, cB, st + j * kUnitBytes, st + (j + 1) * kUnitBytes, lane, bfA, bfB);
                } else if (j < n) {
                    load_bfrag(bfA, xlane, xu + j * 2 * xpair, xpair);
                    consume_unit<FMT>(cA, st + j * kUnitBytes, lane, bfA);
                }
            }
            ++consumed;
            cons_cur.advance();
            // the slot is free again: all loads of this chunk have delivered their data (see the
            // whole-panel kernel), so the next asynchronous write needs no cross-proxy fence
            __syncwarp();
            if (issue_cur.valid()) {
                if (lane == 0) issue_one();
                ++issued;
                issue_cur.advance();
            }
        }
        if (!ok) break;
        // hand this warp's K slice of the panel to the epilogue warp (zeros if it had no units)
        const int rs = rcnt % kSRedSlots;
        const uint32_t ruse = rcnt / kSRedSlots;
        if (ruse > 0 && !mbar_wait(sbase + SSmem::kBarRedEmpty + 8 * rs, (ruse - 1) & 1, P.spin_limit)) {
            if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 7, int(rcnt));
            *abort_flag = 1;
            ok = false;
            break;
        }
        sts128f(red + rs * kSWarps * 512, (cA[0] + cB[0]) * fs0, (cA[1] + cB[1]) * fs1, (cA[2] + cB[2]) * fs0,
                (cA[3] + cB[3]) * fs1);
        __syncwarp();  // orders the lanes' stores before lane 0's releasing arrive
        if (lane == 0) mbar_arrive(sbase + SSmem::kBarRedFull + 8 * rs);
    }
    // never leave with copies in flight: wait (bounded) for every copy this warp still owns
    if (!drop) {
        for (int i = consumed; i < issued; ++i)
            (void)mbar_wait(bars + 8 * (i % kRing), (i / kRing) & 1, int64_t(1) << 20);
    }
}

// Whole-panel variant: every CTA owns whole panels (no panel is split between CTAs, so there is
// no cross-CTA fix-up).  The K extent is cut into chunks of kChunkUnits units and warp w owns
// chunks [w*NC/16, (w+1)*NC/16) of every panel, so every warp sees the same chunk sequence in every
// panel and the loop bookkeeping is a handful of running counters.  Chosen by the host when there
// is at least one panel per CTA.  FULL: units is a multiple of kChunkUnits (no ragged last chunk).
__device__ __forceinline__ int wp_short_group(int npc, int n_chunks) {
    int gs = npc >= 8 ? 4 : (npc >= 4 ? 8 : 16);
    while (gs > 4 && gs > n_chunks) gs >>= 1;
    return gs;
}

template <int FMT, bool FULL, int PPI, bool SHORTK = false>
__global__ void __launch_bounds__(kSThreads, 1) gemv_stream_wp_kernel(const GemvParams P) {
    using ST = StreamTraits<FMT>;
    constexpr int kUnitBytes = FmtTraits<FMT>::kUnitBytes;
    constexpr int CH = ST::kChunkUnits;
    constexpr int kRing = ST::kRing;
    constexpr int kSlotBytes = CH * kUnitBytes;
    constexpr int kWpRing = 4 / PPI;  // ring slots per warp; a slot holds one chunk of PPI panels

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Bl = P.B;
    const int units = P.units;
    const int grid = P.n_panels < int(gridDim.x) ? P.n_panels : int(gridDim.x);
    const int cta = blockIdx.x;
    const int p0 = cta < grid ? int((int64_t(cta) * P.n_panels) / grid) : 0;
    const int p1 = cta < grid ? int((int64_t(cta + 1) * P.n_panels) / grid) : 0;
    // Warp groups: the sixteen consumer warps form G groups of GS warps; a group works on every
    // G-th panel of the CTA and splits K between its GS warps.  Many panels per CTA -> small groups
    // (a warp stays longer on one panel, fewer hand-overs); few panels -> all sixteen warps split K.
    const int npc = p1 - p0;
    // SHORTK (a panel has fewer chunks than sixteen): groups no larger than the chunk count, so that
    // no warp idles and more panels are in flight.  A separate instantiation: the common one keeps its code.
    const int GS = SHORTK ? wp_short_group(npc, (units + CH - 1) / CH) : (npc >= 8 ? 4 : (npc >= 4 ? 8 : 16));
    const int G = kSWarps / GS;

    // Set-up is spread over the warps and the CTA-wide barrier comes late: a consumer warp's ring
    // barriers are private to it, so it initialises them itself and starts its first weight copies
    // before the CTA has synchronised at all.
    if (warp == kSEpilogueWarp) {
        if (lane < 4 * kSRedSlots) {  // up to four warp groups, two hand-over slots each
            mbar_init(sbase + SSmem::kBarRedFull + 8 * lane, uint32_t(GS));
            mbar_init(sbase + SSmem::kBarRedEmpty + 8 * lane, 1);
        }
        if (lane < 8) reinterpret_cast<volatile unsigned int*>(smem_raw + SSmem::kRowMax)[lane] = 0u;
        // 16 zero bytes: the activation "fragment" of lanes whose batch column does not exist
        if (lane < 4) reinterpret_cast<volatile unsigned int*>(smem_raw + SSmem::kZero)[lane] = 0u;
        if (lane == 0) *reinterpret_cast<volatile int*>(smem_raw + SSmem::kAbort) = 0;
        mbar_fence_init();
    } else {
        if (lane < kWpRing) mbar_init(sbase + SSmem::kBarFull + 8 * (warp * kWpRing + lane), 1);
        mbar_fence_init();
        __syncwarp();
    }
    pdl_launch_dependents();

    if (cta >= grid) return;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + SSmem::kAbort);

    if (warp == kSEpilogueWarp) {
        // ================= epilogue: reduce the sixteen K slices of each panel, scale, store =================
        __syncthreads();  // the CTA's one barrier: shared set-up is visible to everyone
        pdl_wait();       // the output buffer may still be in use by the preceding kernel
        const float ts = (FMT == QGEMV_FMT_NVFP4) ? P.tensor_scale[0] : 1.0f;
        const uint32_t red = sbase + SSmem::kRed + lane * 16;
        // Optional L2 prefetch of the weight the caller uses next: this CTA's share, issued in
        // pieces as its own panels complete, so it trails this GEMV's demand loads instead of
        // competing with them.  Weights are immutable, so prefetching them early is always safe.
        uint64_t pf_pos = 0, pf_end = 0, pf_step = 0;
        if (P.pf_bytes != 0) {
            pf_pos = ((uint64_t(cta) * P.pf_bytes) / grid) & ~uint64_t(127);
            pf_end = cta + 1 == grid ? (P.pf_bytes & ~uint64_t(15)) : (((uint64_t(cta + 1) * P.pf_bytes) / grid) & ~uint64_t(127));
            pf_step = ((pf_end - pf_pos) / uint64_t(npc) + 127) & ~uint64_t(127);
        }
        for (int i = 0; i < npc; ++i) {
            const int p = p0 + i;
            const int gidx = i % G, use = i / G;
            const int rs = use % kSRedSlots;
            const uint32_t rpar = uint32_t(use / kSRedSlots) & 1u;
            const int bi = gidx * kSRedSlots + rs;
            // FP8: fetch the panel's two channel scales before the wait, so their latency hides in it
            float cs0 = 1.0f, cs1 = 1.0f;
            if (FMT == QGEMV_FMT_FP8) {
                cs0 = __ldg(P.chan_scale + p * 16 + (lane >> 2));  // padded to 16 rows per panel
                cs1 = __ldg(P.chan_scale + p * 16 + (lane >> 2) + 8);
            }
            if (!mbar_wait(sbase + SSmem::kBarRedFull + 8 * bi, rpar, P.spin_limit, 200u)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 6, p);
                *abort_flag = 1;
                return;
            }
            const uint32_t slot = red + uint32_t(bi * GS) * 512u;
            float4 v = lds128f(slot);
            for (int ww = 1; ww < GS; ++ww) {
                const float4 q = lds128f(slot + ww * 512);
                v.x += q.x, v.y += q.y, v.z += q.z, v.w += q.w;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + SSmem::kBarRedEmpty + 8 * bi);
            if (FMT == QGEMV_FMT_FP8) {
                v.x *= cs0, v.y *= cs0, v.z *= cs1, v.w *= cs1;
                store_panel<QGEMV_FMT_NVFP4>(P, v, lane, p, Bl, nullptr, nullptr);  // scaled already
            } else {
                v.x *= ts, v.y *= ts, v.z *= ts, v.w *= ts;
                store_panel<FMT>(P, v, lane, p, Bl, nullptr, P.chan_scale);
            }
            if (pf_pos < pf_end && lane == 0) {
                const uint64_t stop = (i + 1 == npc || pf_pos + pf_step > pf_end) ? pf_end : pf_pos + pf_step;
                while (pf_pos < stop) {
                    const uint32_t n = uint32_t(stop - pf_pos < 32768 ? stop - pf_pos : 32768);
                    bulk_prefetch_l2(P.pf_base + pf_pos, n);
                    pf_pos += n;
                }
            }
        }
        return;
    }

    // ================= consumer warps =================
    // Each iteration handles one chunk of this warp's K slice for TWO consecutive panels: the
    // activation fragments and the loop bookkeeping are shared by both, and four independent
    // accumulator chains are in flight.
    const int w = warp;
    const int g = lane >> 2, t = lane & 3;
    const int n_chunks = (units + CH - 1) / CH;
    const int gidx = w / GS, ws = w - gidx * GS;  // group and K-slice index inside the group
    const int ck_lo = (ws * n_chunks) / GS, ck_hi = ((ws + 1) * n_chunks) / GS;
    const int nck = ck_hi - ck_lo;  // chunks of this warp in every panel
    constexpr int kPairBytes = PPI * kSlotBytes;
    const uint32_t ring = sbase + SSmem::kRing0 + w * (kWpRing * kPairBytes);
    const uint32_t bars = sbase + SSmem::kBarFull + 8 * (w * kWpRing);
    const uint64_t pol = policy_evict_first();
    const bool drop = (P.debug & 2) != 0;  // host-set fault injection: never issue a copy

    // issue cursor: running byte offset of panel a's chunk, chunk counter, ring slot
    const uint32_t panel_bytes = uint32_t(P.unit_stride) * kUnitBytes;  // a packed matrix is below 4 GB
    const int np_g = npc > gidx ? (npc - gidx + G - 1) / G : 0;  // panels of this group
    const int n_pairs = (np_g + PPI - 1) / PPI;
    uint32_t ioff = uint32_t(p0 + gidx) * panel_bytes + uint32_t(ck_lo) * kSlotBytes;
    const uint32_t ioff_next_pair = uint32_t(PPI * G) * panel_bytes - uint32_t(nck) * kSlotBytes;
    int ic = 0, islot = 0, ipair = 0;
    int to_issue = nck * n_pairs, in_flight = 0;
    auto issue_one = [&]() {
        if (lane == 0 && !drop) {
            uint32_t bytes = kSlotBytes;
            if (!FULL) bytes = uint32_t(min(CH, units - (ck_lo + ic) * CH)) * kUnitBytes;
            const bool two = PPI == 2 && 2 * ipair + 1 < np_g;
            if ((P.debug & 1) && uint64_t(ioff) + (two ? uint64_t(G) * panel_bytes : 0u) + bytes > P.payload_bytes) {
                report(P.status, QGEMV_ERR_BOUNDS, 2, ipair);
            } else {
                const uint32_t bar = bars + 8 * islot;
                const uint32_t dst = ring + islot * kPairBytes;
                mbar_arrive_expect_tx(bar, two ? 2u * bytes : bytes);
                bulk_g2s(dst, P.payload + ioff, bytes, bar, pol);
                if (two) bulk_g2s(dst + kSlotBytes, P.payload + ioff + uint32_t(G) * panel_bytes, bytes, bar, pol);
            }
        }
        ioff += kSlotBytes;
        if (++ic == nck) {
            ic = 0;
            ++ipair;
            ioff += ioff_next_pair;
        }
        if (++islot == kWpRing) islot = 0;
        --to_issue;
        ++in_flight;
    };
    for (int i = 0; i < kWpRing && to_issue > 0; ++i) issue_one();

    __syncthreads();  // the CTA's one barrier (the epilogue warp's set-up; see the top of the kernel)
    // weights never depend on the preceding kernel; activations do
    pdl_wait();
    stream_convert_x(P, smem_raw, sbase, w, lane);
    const int* rowexp = reinterpret_cast<const int*>(smem_raw + SSmem::kRowExp);
    const float fs0 = pow2i(rowexp[2 * t]), fs1 = pow2i(rowexp[2 * t + 1]);

    // Activation fragments of (unit u, block pair pp): 16 bytes at xbase + u*xunit + pp*xpair.  Lanes
    // whose batch column does not exist read sixteen zero bytes with zero strides: no branches.
    const bool xlane = g < Bl;
    const uint32_t xpair = xlane ? uint32_t(Bl) * 64u : 0u;
    const uint32_t xunit = 2u * xpair;
    const uint32_t xbase = xlane ? sbase + SSmem::kXBuf + g * 64 + t * 16 : sbase + SSmem::kZero;
    // one chunk per panel: the activation fragments of the slice never change -- keep them in registers
    const bool bf_fixed = (nck == 1) && FULL;
    uint32_t bfr[CH][8];
#pragma unroll
    for (int j = 0; j < CH; ++j) {
        const uint32_t xa = xbase + uint32_t(ck_lo * CH + j) * xunit;
        const uint4 x0 = lds128(bf_fixed ? xa : sbase + SSmem::kZero);
        const uint4 x1 = lds128(bf_fixed ? xa + xpair : sbase + SSmem::kZero);
        bfr[j][0] = x0.x, bfr[j][1] = x0.y, bfr[j][2] = x0.z, bfr[j][3] = x0.w;
        bfr[j][4] = x1.x, bfr[j][5] = x1.y, bfr[j][6] = x1.z, bfr[j][7] = x1.w;
    }
    const uint32_t red = sbase + SSmem::kRed + uint32_t(gidx * kSRedSlots * GS + ws) * 512u + lane * 16;
    const uint32_t red_bars = 8u * uint32_t(gidx * kSRedSlots);
    uint32_t rs = 0, ruse = 0;
    int cslot = 0;
    uint32_t cpar = 0;
    // hands one panel's K slice of this warp to the epilogue warp; false when the wait ran out
    auto hand_over = [&](const float (&cA)[4], const float (&cB)[4], int p) -> bool {
        if (ruse > 0 &&
            !mbar_wait(sbase + SSmem::kBarRedEmpty + red_bars + 8 * rs, (ruse - 1) & 1, P.spin_limit)) {
            if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 7, p);
            *abort_flag = 1;
            return false;
        }
        sts128f(red + rs * uint32_t(GS) * 512u, (cA[0] + cB[0]) * fs0, (cA[1] + cB[1]) * fs1, (cA[2] + cB[2]) * fs0,
                (cA[3] + cB[3]) * fs1);
        __syncwarp();  // orders the lanes' stores before lane 0's releasing arrive
        if (lane == 0) mbar_arrive(sbase + SSmem::kBarRedFull + red_bars + 8 * rs);
        if (++rs == kSRedSlots) {
            rs = 0;
            ++ruse;
        }
        return true;
    };

    for (int pr = 0; pr < n_pairs; ++pr) {
        const int pa = p0 + gidx + PPI * pr * G;
        const bool two = PPI == 2 && PPI * pr + 1 < np_g;
        float cA0[4] = {0.f, 0.f, 0.f, 0.f}, cB0[4] = {0.f, 0.f, 0.f, 0.f};
        float cA1[4] = {0.f, 0.f, 0.f, 0.f}, cB1[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c = 0; c < nck; ++c) {
            if (!mbar_wait(bars + 8 * cslot, cpar, P.spin_limit)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 5, pa);
                *abort_flag = 1;
                goto drain;
            }
            {
                const uint32_t st = ring + cslot * kPairBytes;
                if (bf_fixed && two) {
#pragma unroll
                    for (int j = 0; j < CH; j += 2) {
                        consume_two<FMT>(cA0, cB0, st + j * kUnitBytes, st + (j + 1) * kUnitBytes, lane, bfr[j],
                                         bfr[j + 1]);
                        consume_two<FMT>(cA1, cB1, st + kSlotBytes + j * kUnitBytes,
                                         st + kSlotBytes + (j + 1) * kUnitBytes, lane, bfr[j], bfr[j + 1]);
                    }
                } else {
                    const uint32_t xu = xbase + uint32_t((ck_lo + c) * CH) * xunit;
                    const int n = FULL ? CH : min(CH, units - (ck_lo + c) * CH);
#pragma unroll
                    for (int j = 0; j < CH; j += 2) {
                        uint32_t bfA[8], bfB[8];
                        if (FULL || j + 1 < n) {
                            load_bfrag(bfA, true, xu + j * xunit, xpair);
                            load_bfrag(bfB, true, xu + (j + 1) * xunit, xpair);
                            consume_two<FMT>(cA0, cB0, st + j * kUnitBytes, st + (j + 1) * kUnitBytes, lane, bfA, bfB);
                            if (two)
                                consume_two<FMT>(cA1, cB1, st + kSlotBytes + j * kUnitBytes,
                                                 st + kSlotBytes + (j + 1) * kUnitBytes, lane, bfA, bfB);
                        } else if (j < n) {
                            load_bfrag(bfA, true, xu + j * xunit, xpair);
                            consume_unit<FMT>(cA0, st + j * kUnitBytes, lane, bfA);
                            if (two) consume_unit<FMT>(cA1, st + kSlotBytes + j * kUnitBytes, lane, bfA);
                        }
                    }
                }
            }
            --in_flight;
            if (++cslot == kWpRing) {
                cslot = 0;
                cpar ^= 1u;
            }
            // The slot is free again.  Every shared-memory load of this chunk has already delivered
            // its data (the MMAs above consumed it), so once the warp has converged the next
            // asynchronous write cannot pass a pending read: no cross-proxy fence is needed for this
            // read-then-overwrite order.
            __syncwarp();
            if (to_issue > 0) issue_one();
        }
        // hand this warp's K slice of the panels to the epilogue warp (zeros if it has no chunks)
        if (!hand_over(cA0, cB0, pa)) goto drain;
        if (two && !hand_over(cA1, cB1, pa + G)) goto drain;
    }
drain:
    // never leave with copies in flight: wait (bounded) for every copy this warp still owns
    if (!drop) {
        while (in_flight > 0) {
            (void)mbar_wait(bars + 8 * cslot, cpar, int64_t(1) << 20);
            if (++cslot == kWpRing) {
                cslot = 0;
                cpar ^= 1u;
            }
            --in_flight;
        }
    }
}

}  // namespace qg
