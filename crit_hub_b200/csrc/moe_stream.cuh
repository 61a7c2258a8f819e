// MoE grouped GEMV on the warp-stream schedule.
//
// The router walk (moe_prep_kernel) leaves a problem table: problem q = (expert, <= 8 activation
// rows, their output rows).  The linear work space is (problem, panel) -- every expert matrix read
// once per problem.  It is cut into R = max(CTAs, problems) equal ranges, so a range never spans
// more than two problems; CTA c handles ranges c, c + CTAs, ...  For each range the sixteen consumer
// warps convert the activations of its (at most two) problems into f16 fragments (one power-of-two
// scale per row, as in the dense kernels), then stream the range's panels exactly like the dense
// whole-panel kernel: warp groups split K, private bulk-copy rings per warp, an epilogue warp that
// sums the K slices in warp order and scatters the rows to out[orow].
// Needs units <= 32 (K <= 2048) per launch so that two problems' fragments (8 rows each) fit 64 KB;
// longer K is served as several launches over K chunks whose results are added afterwards.
#pragma once
#include "gemv_stream.cuh"

namespace qg {

struct MSmem {  // extra words inside the 1 KB header region of SSmem
    static constexpr int kRowMax16 = 768;  // 16 words
    static constexpr int kRowExp16 = 832;  // 16 words
    // hand-over barriers of up to sixteen warp groups (two slots each) sit behind the rings
    template <int FMT>
    __host__ __device__ static constexpr int bar_red_full() { return SSmem::total<FMT>(); }
    template <int FMT>
    __host__ __device__ static constexpr int bar_red_empty() { return SSmem::total<FMT>() + 256; }
    template <int FMT>
    __host__ __device__ static constexpr int total() { return SSmem::total<FMT>() + 512; }
};

inline bool use_moe_stream_path(int64_t units) { return units <= 32; }

template <int FMT>
__global__ void __launch_bounds__(kSThreads, 1) moe_stream_kernel(const GemvParams P) {
    using ST = StreamTraits<FMT>;
    constexpr int kUnitBytes = FmtTraits<FMT>::kUnitBytes;
    constexpr int CH = ST::kChunkUnits;
    constexpr int kSlotBytes = CH * kUnitBytes;
    constexpr int kWpRing = 4;
    constexpr int kProbXBytes = 32768;  // f16 fragments of one problem: 32 units x 8 rows x 128 B
    constexpr int kBarRedFull = MSmem::bar_red_full<FMT>(), kBarRedEmpty = MSmem::bar_red_empty<FMT>();

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = P.units;
    // ring barriers do not depend on the problem table: set them up (spread over the warps) while the
    // preceding kernel may still be running
    if (warp < kSWarps && lane < kWpRing) mbar_init(sbase + SSmem::kBarFull + 8 * (warp * kWpRing + lane), 1);
    pdl_launch_dependents();
    pdl_wait();  // the problem table and the activations come from preceding kernels
    const int nprob = __ldcg(P.prob);
    const int64_t VP = int64_t(nprob) * P.n_panels;
    if (VP <= 0) return;
    const int grid = VP < int64_t(gridDim.x) ? int(VP) : int(gridDim.x);
    const int cta = blockIdx.x;
    if (cta >= grid) return;
    const int R = nprob > grid ? nprob : grid;        // ranges; each spans at most two problems
    const int npr = int((VP + R - 1) / R);            // panels per range (upper bound)
    const int n_chunks = (units + CH - 1) / CH;
    // Warps per panel: experts have short K (2048 and less), so a panel is only a few chunks; a warp
    // should keep about four of them per panel (hand-overs to the epilogue warp cost as much as a
    // chunk), which means one or two warps per panel and up to sixteen panels in flight per CTA --
    // unless the range has too few panels to occupy that many groups.
    int GS = 1;
    while (GS < 16 && n_chunks / (2 * GS) >= 4) GS <<= 1;
    while (GS < 16 && kSWarps / GS > npr) GS <<= 1;
    const int G = kSWarps / GS;

    if (warp == kSEpilogueWarp) {
        static_assert(kSWarps * kSRedSlots <= 32, "one hand-over barrier pair per lane");
        if (lane < kSWarps * kSRedSlots) {
            mbar_init(sbase + kBarRedFull + 8 * lane, uint32_t(GS));
            mbar_init(sbase + kBarRedEmpty + 8 * lane, 1);
        }
        if (lane == 0) *reinterpret_cast<volatile int*>(smem_raw + SSmem::kAbort) = 0;
    }
    mbar_fence_init();
    __syncthreads();
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + SSmem::kAbort);

    if (warp == kSEpilogueWarp) {
        // ================= epilogue =================
        const uint32_t red = sbase + SSmem::kRed + lane * 16;
        int hand[kSWarps];  // hand-overs seen so far, per group
#pragma unroll
        for (int i = 0; i < kSWarps; ++i) hand[i] = 0;
        for (int r = cta; r < R; r += grid) {
            const int64_t p0 = (int64_t(r) * VP) / R, p1 = (int64_t(r + 1) * VP) / R;
            const int64_t q0 = p0 / P.n_panels;
            // the (at most two) problems of the range: expert, row count, table pointer
            const int32_t* pr0 = P.prob + 1 + q0 * kProbInts;
            const int32_t* pr1 = (q0 + 1 < nprob) ? pr0 + kProbInts : pr0;
            const int ex0 = __ldcg(pr0), nr0 = __ldcg(pr0 + 1), ex1 = __ldcg(pr1), nr1 = __ldcg(pr1 + 1);
            // everything the per-panel path needs from global memory, fetched once per range: this
            // lane's two output rows of either problem, the experts' tensor scales
            const int tq = lane & 3, gq = lane >> 2;
            const int c0 = 2 * tq, c1 = c0 + 1;
            const int orow00 = c0 < nr0 ? __ldcg(pr0 + 10 + c0) : 0, orow01 = c1 < nr0 ? __ldcg(pr0 + 10 + c1) : 0;
            const int orow10 = c0 < nr1 ? __ldcg(pr1 + 10 + c0) : 0, orow11 = c1 < nr1 ? __ldcg(pr1 + 10 + c1) : 0;
            const float ts0 = (FMT == QGEMV_FMT_NVFP4) ? __ldg(P.tensor_scale + ex0) : 1.0f;
            const float ts1 = (FMT == QGEMV_FMT_NVFP4) ? __ldg(P.tensor_scale + ex1) : 1.0f;
            int sel = 0;
            int32_t panel = int32_t(p0 - q0 * P.n_panels);
            for (int64_t p = p0; p < p1; ++p) {
                const int gidx = int((p - p0) % G);
                const int use = hand[gidx]++;
                const int rs = use % kSRedSlots;
                const uint32_t rpar = uint32_t(use / kSRedSlots) & 1u;
                const int bi = gidx * kSRedSlots + rs;
                if (!mbar_wait(sbase + kBarRedFull + 8 * bi, rpar, P.spin_limit, 200u)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 6, int(p));
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
                if (lane == 0) mbar_arrive(sbase + kBarRedEmpty + 8 * bi);
                const float ts = sel ? ts1 : ts0;
                v.x *= ts, v.y *= ts, v.z *= ts, v.w *= ts;
                const int n0 = panel * 16 + gq, n1 = n0 + 8;
                if (FMT == QGEMV_FMT_FP8) {
                    const float* chan = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(P.chan_scale) +
                                                                       uint64_t(sel ? ex1 : ex0) * P.chan_stride);
                    const float s0 = __ldg(chan + n0), s1 = __ldg(chan + n1);  // padded to 16 rows per panel
                    v.x *= s0, v.y *= s0, v.z *= s1, v.w *= s1;
                }
                const int nrows = sel ? nr1 : nr0;
                const int64_t ra = int64_t(sel ? orow10 : orow00) * P.N, rb = int64_t(sel ? orow11 : orow01) * P.N;
                const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = (i & 2) ? n1 : n0;
                    if (((i & 1) ? c1 : c0) < nrows && n < P.N) {
                        const int64_t idx = ((i & 1) ? rb : ra) + n;
                        if (P.y_dtype == QGEMV_OUT_F32) {
                            static_cast<float*>(P.y)[idx] = vals[i];
                        } else {
                            static_cast<__nv_bfloat16*>(P.y)[idx] = __float2bfloat16_rn(vals[i]);
                        }
                    }
                }
                if (++panel == P.n_panels) {
                    panel = 0;
                    ++sel;
                }
            }
        }
        return;
    }

    // ================= consumer warps =================
    const int w = warp;
    const int g = lane >> 2, t = lane & 3;
    const int gidx = w / GS, ws = w - gidx * GS;
    const int ck_lo = (ws * n_chunks) / GS, ck_hi = ((ws + 1) * n_chunks) / GS;
    const int nck = ck_hi - ck_lo;
    const uint32_t ring = sbase + SSmem::kRing0 + w * (kWpRing * kSlotBytes);
    const uint32_t bars = sbase + SSmem::kBarFull + 8 * (w * kWpRing);
    const uint64_t pol = policy_evict_first();
    const bool drop = (P.debug & 2) != 0;
    const uint64_t panel_bytes = uint64_t(P.unit_stride) * kUnitBytes;  // a K-chunked call covers `units` of them
    const int n_phases = (units + QG_PHASE_UNITS - 1) / QG_PHASE_UNITS;  // 1 or 2
    unsigned int* rowmax = reinterpret_cast<unsigned int*>(smem_raw + MSmem::kRowMax16);
    int* rowexp = reinterpret_cast<int*>(smem_raw + MSmem::kRowExp16);
    const uint32_t xlane_base = sbase + SSmem::kXBuf + g * 64 + t * 16;
    const uint32_t xpair = 8u * 64u, xunit = 2u * xpair;
    const uint32_t red = sbase + SSmem::kRed + uint32_t(gidx * kSRedSlots * GS + ws) * 512u + lane * 16;
    const uint32_t red_bars = 8u * uint32_t(gidx * kSRedSlots);
    uint32_t rs = 0, ruse = 0;
    int islot = 0, cslot = 0, in_flight = 0;
    uint32_t cpar = 0;
    bool ok = true;

    for (int r = cta; r < R; r += grid) {
        if (!ok) {
            // a wait ran out earlier: keep meeting the other warps at the range barriers (a named
            // barrier has no timeout) but do no more work
            for (int z = 0; z < 4; ++z) named_bar_sync(1, 32 * kSWarps);
            continue;
        }
        const int64_t p0 = (int64_t(r) * VP) / R, p1 = (int64_t(r + 1) * VP) / R;
        const int npc = int(p1 - p0);
        const int64_t q0 = p0 / P.n_panels;
        // ---- this group's panels: p0 + gidx, p0 + gidx + G, ... ; issue cursor ----
        const int np_g = npc > gidx ? (npc - gidx + G - 1) / G : 0;
        // the (at most two) problems of the range
        const int ex0 = __ldcg(P.prob + 1 + q0 * kProbInts);
        const int ex1 = (q0 + 1 < nprob) ? __ldcg(P.prob + 1 + (q0 + 1) * kProbInts) : ex0;
        const int panel_first = int(p0 - q0 * P.n_panels) + gidx;  // may already be in the second problem
        // issue cursor: (problem selector, panel inside it, chunk)
        int isel = panel_first >= P.n_panels ? 1 : 0;
        int ipan = panel_first - isel * P.n_panels;
        int ic = 0;
        int to_issue = nck * np_g;
        auto issue_one = [&]() {
            if (lane == 0 && !drop) {
                const int c0 = (ck_lo + ic) * CH;
                const uint32_t bytes = uint32_t(min(CH, units - c0)) * kUnitBytes;
                const uint64_t off = uint64_t(ipan) * panel_bytes + uint64_t(c0) * kUnitBytes;
                if ((P.debug & 1) && off + bytes > P.payload_bytes) {
                    report(P.status, QGEMV_ERR_BOUNDS, 2, ipan);
                } else {
                    mbar_arrive_expect_tx(bars + 8 * islot, bytes);
                    bulk_g2s(ring + islot * kSlotBytes,
                             P.payload + uint64_t(isel ? ex1 : ex0) * P.stack_stride + off, bytes, bars + 8 * islot,
                             pol);
                }
            }
            if (++ic == nck) {
                ic = 0;
                ipan += G;
                if (ipan >= P.n_panels) {
                    ipan -= P.n_panels;
                    isel = 1;
                }
            }
            if (++islot == kWpRing) islot = 0;
            --to_issue;
            ++in_flight;
        };
        for (int i = 0; i < kWpRing && to_issue > 0; ++i) issue_one();

        // ---- activations of the (at most two) problems of this range ----
        named_bar_sync(1, 32 * kSWarps);  // every warp is done with the previous range's fragments
        for (int i = threadIdx.x; i < 2 * kProbXBytes / 16; i += 32 * kSWarps)
            sts128(sbase + SSmem::kXBuf + 16 * i, make_uint4(0, 0, 0, 0));
        if (w == 0 && lane < 16) rowmax[lane] = 0u;
        named_bar_sync(1, 32 * kSWarps);
        {
            RowRegs rr[2];
            int sel_[2], f_[2], b_[2];
            bool act[2];
#pragma unroll
            for (int z = 0; z < 2; ++z) {
                const int i = w + z * kSWarps;  // pair index: (problem sel, phase f, row b)
                sel_[z] = i / (n_phases * 8);
                const int rem = i - sel_[z] * (n_phases * 8);
                f_[z] = rem >> 3;
                b_[z] = rem & 7;
                act[z] = false;
                if (sel_[z] < 2 && q0 + sel_[z] < nprob && (q0 + sel_[z]) * P.n_panels < p1) {
                    const int32_t* pr = P.prob + 1 + (q0 + sel_[z]) * kProbInts;
                    if (b_[z] < __ldcg(pr + 1)) {
                        act[z] = true;
                        const int64_t row = __ldcg(pr + 2 + b_[z]);
                        const uint32_t m = load_row(rr[z], P.x + row * int64_t(P.x_stride), P.K, f_[z], f_[z] * QG_PHASE_UNITS,
                                                    min(units, (f_[z] + 1) * QG_PHASE_UNITS), lane);
                        if (lane == 0) atomicMax(rowmax + sel_[z] * 8 + b_[z], m);
                    }
                }
            }
            named_bar_sync(1, 32 * kSWarps);
#pragma unroll
            for (int z = 0; z < 2; ++z) {
                if (act[z])
                    store_row(rr[z], row_exponent(rowmax[sel_[z] * 8 + b_[z]]), f_[z], f_[z] * QG_PHASE_UNITS,
                              min(units, (f_[z] + 1) * QG_PHASE_UNITS),
                              sbase + SSmem::kXBuf + sel_[z] * kProbXBytes + f_[z] * 16384u, 8, b_[z], lane);
            }
            if (w == 0 && lane < 16) rowexp[lane] = row_exponent(rowmax[lane]);
            named_bar_sync(1, 32 * kSWarps);
        }

        // ---- stream this group's panels ----
        int csel = panel_first >= P.n_panels ? 1 : 0;
        int cpan = panel_first - csel * P.n_panels;
        for (int pi = 0; pi < np_g && ok; ++pi, cpan += G) {
            if (cpan >= P.n_panels) {
                cpan -= P.n_panels;
                csel = 1;
            }
            const int64_t p = p0 + gidx + int64_t(pi) * G;
            const int sel = csel;
            const float fs0 = pow2i(rowexp[sel * 8 + 2 * t]), fs1 = pow2i(rowexp[sel * 8 + 2 * t + 1]);
            const uint32_t xb = xlane_base + sel * kProbXBytes;
            float cA[4] = {0.f, 0.f, 0.f, 0.f}, cB[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = 0; c < nck; ++c) {
                if (!mbar_wait(bars + 8 * cslot, cpar, P.spin_limit)) {
                    if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 5, int(p));
                    *abort_flag = 1;
                    ok = false;
                    break;
                }
                const uint32_t st = ring + cslot * kSlotBytes;
                const int c0 = (ck_lo + c) * CH;
                const int n = min(CH, units - c0);
                const uint32_t xu = xb + uint32_t(c0) * xunit;
#pragma unroll
                for (int j = 0; j < CH; j += 2) {
                    uint32_t bfA[8], bfB[8];
                    if (j + 1 < n) {
                        load_bfrag(bfA, true, xu + j * xunit, xpair);
                        load_bfrag(bfB, true, xu + (j + 1) * xunit, xpair);
                        consume_two<FMT>(cA, cB, st + j * kUnitBytes, st + (j + 1) * kUnitBytes, lane, bfA, bfB);
                    } else if (j < n) {
                        load_bfrag(bfA, true, xu + j * xunit, xpair);
                        consume_unit<FMT>(cA, st + j * kUnitBytes, lane, bfA);
                    }
                }
                --in_flight;
                if (++cslot == kWpRing) {
                    cslot = 0;
                    cpar ^= 1u;
                }
                __syncwarp();  // all loads of the slot have delivered their data: it may be refilled
                if (to_issue > 0) issue_one();
            }
            if (!ok) break;
            if (ruse > 0 &&
                !mbar_wait(sbase + kBarRedEmpty + red_bars + 8 * rs, (ruse - 1) & 1, P.spin_limit)) {
                if (lane == 0) report(P.status, QGEMV_ERR_TIMEOUT, 7, int(p));
                *abort_flag = 1;
                ok = false;
                break;
            }
            sts128f(red + rs * uint32_t(GS) * 512u, (cA[0] + cB[0]) * fs0, (cA[1] + cB[1]) * fs1,
                    (cA[2] + cB[2]) * fs0, (cA[3] + cB[3]) * fs1);
            __syncwarp();
            if (lane == 0) mbar_arrive(sbase + kBarRedFull + red_bars + 8 * rs);
            if (++rs == kSRedSlots) {
                rs = 0;
                ++ruse;
            }
        }
    }
    if (!drop) {  // never leave with copies in flight
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
