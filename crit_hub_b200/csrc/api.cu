// C ABI of the quantized GEMV library (include/qgemv.h): handle and weight lifetime, launches.
// Host code only decides shapes and launch attributes; there is no CPU compute path.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/qgemv.h"
#include "aux_kernels.cuh"
#include "gemv_kernel.cuh"
#include "gemv_stream.cuh"
#include "gemm_skinny.cuh"
#include "gemv_tc.cuh"
#include "gemv_seq.cuh"
#include "moe_stream.cuh"
#include "tp_allreduce.cuh"
#include "gemm_tc_a4.cuh"
#include "qgemv_layout.h"

extern "C" int qgemv_blob_verify(const void* blob, size_t bytes);

struct qgemv_handle {
    qgemv_config cfg;
    int sm_count;
    int32_t* status_dev;
    // tensor-parallel exchange (qgemv_tp_*)
    int tp_rank, tp_world;
    int64_t tp_max_elems;
    uint8_t* tp_local;                     // this rank's exchange buffer
    uint8_t* tp_peer[qg::kTpMaxWorld];     // every rank's buffer as mapped here (tp_peer[rank] == tp_local)
    uint32_t* tp_epochs;                   // [0] exchanges completed by qgemv_tp_allreduce / _allgather, [1] their arrival counter
    bool tp_ipc_opened[qg::kTpMaxWorld];   // mapped by qgemv_tp_connect (closed on destroy), not handed in as a pointer
    int64_t tp_seq_cursor;                 // elements [tp_seq_cursor, tp_max_elems) of every slot belong to job lists
    int64_t tp_call_high;                  // the longest vector a stand-alone exchange has used so far
    // skinny GEMM: f16 activation tiles + per-row exponents, grown on demand
    uint8_t* gs_ws;
    size_t gs_ws_bytes;
    // K-chunked GEMV: fp32 partial results [chunk][B][N], fixed size, allocated with the handle
    float* chunk_ws;
    // tensor-core GEMV: split-K hand-over slots (two per CTA, [8][128] pairs {fp32, flag}), all zero between launches
    float* tc_ws;
    unsigned long long* tc_trace;  // caller's device buffer for phase timestamps, or null
    unsigned int* seq_barrier;     // CTAs that have left a GEMV-sequence launch, zero between launches
    unsigned long long* seq_parts; // its parts buffers: [kSeqPartBufs][2 * grid][8][128] pairs {fp32, tag}
    unsigned int* moe_cnt;         // expert MLP in one launch: per problem, warps that have stored first-stage rows (zero between launches)
    size_t tc_ws_bytes;
    uint8_t* a4_ws;        // block-scaled prefill: quantised activation items, then the row scales
    size_t a4_ws_bytes;
    std::vector<qgemv_sequence*>* sequences;  // live job lists: their counters are cleared after a reported error
};

struct qgemv_sequence {
    qg::SeqJob* dev_jobs;
    unsigned int* dev_counters;  // fin[n_jobs]: zero between launches; [n_jobs]: launches of this list
    uint32_t* dev_pub;           // outputs that later jobs of the list read as their activations, as tagged words
    int n_jobs, B;
    int grid, npad, x_slots, nbuf, ring, stage_items;
    size_t smem;
    int64_t xchg_elems;  // elements of every exchange slot held by this list's all-reduce jobs (0: none)
    int64_t xchg_first;  // where they start
    bool fused;          // some job has an activation function, a norm or a residual: the kernel instantiation with that code
};

struct qgemv_weight {
    int fmt;
    int64_t N, K;
    int64_t n_panels, units;
    int n_stack;
    uint64_t blob_bytes;     // bytes of one stacked blob (header + aux + payload)
    uint64_t aux_bytes;
    uint64_t payload_bytes;
    uint8_t* dev_blob;       // n_stack blobs back to back
    float* dev_tensor_scale; // [n_stack]
    float* ws;               // partial slots
    int32_t* counters;       // per virtual panel
    int32_t* prob;           // MoE problem table (stacked weights only)
    int max_prob;
    float* host_tensor_scale; // [n_stack], host copy
};

namespace {

thread_local cudaError_t g_last_cuda_error = cudaSuccess;

#define QG_CUDA(expr)                                   \
    do {                                                \
        cudaError_t err__ = (expr);                     \
        if (err__ != cudaSuccess) {                      \
            g_last_cuda_error = err__;                   \
            return QGEMV_ERR_CUDA;                       \
        }                                                \
    } while (0)

constexpr int kMaxMoeSlots = 4096;
constexpr size_t kChunkWsBytes = size_t(64) << 20;  // partial results of a K-chunked GEMV / MoE GEMV
constexpr int kGsMaxTiles = 4096;  // skinny GEMM: 128-row tiles a handle keeps counters for

int64_t default_spin(const qgemv_handle* h) {
    return h->cfg.spin_limit > 0 ? h->cfg.spin_limit : (int64_t(1) << 26);
}

thread_local int g_launch_cluster = 1;  // thread-block cluster size of the next launch() (1: none)
thread_local bool g_launch_cooperative = false;  // the next launch()'s CTAs wait on one another: all co-resident

template <typename... KArgs, typename... Args>
cudaError_t launch(const qgemv_handle* h, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                   size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[3];
    int n_attr = 0;
    if (g_launch_cooperative) {
        attr[n_attr].id = cudaLaunchAttributeCooperative;
        attr[n_attr].val.cooperative = 1;
        ++n_attr;
        g_launch_cooperative = false;
    }
    if (h->cfg.use_pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (g_launch_cluster > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = unsigned(g_launch_cluster);
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
        g_launch_cluster = 1;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    if (err != cudaSuccess) g_last_cuda_error = err;
    return err;
}

int gemv_grid(const qgemv_handle* h) {
    return h->cfg.grid_override > 0 ? h->cfg.grid_override : h->sm_count;
}

qg::GemvParams base_params(const qgemv_handle* h, const qgemv_weight* w) {
    qg::GemvParams P;
    std::memset(&P, 0, sizeof P);
    P.payload = w->dev_blob + QG_HEADER_BYTES + w->aux_bytes;
    P.stack_stride = w->blob_bytes;
    P.chan_scale = reinterpret_cast<const float*>(w->dev_blob + QG_HEADER_BYTES);
    P.chan_stride = w->blob_bytes;
    P.tensor_scale = w->dev_tensor_scale;
    P.ws = w->ws;
    P.counters = w->counters;
    P.status = h->status_dev;
    P.spin_limit = default_spin(h);
    P.N = int32_t(w->N);
    P.K = int32_t(w->K);
    P.n_panels = int32_t(w->n_panels);
    P.units = int32_t(w->units);
    P.debug = h->cfg.debug;
    P.unit_stride = int32_t(w->units);
    P.x_stride = int32_t(w->K);
    P.payload_bytes = w->payload_bytes;
    return P;
}

// Whole panels per CTA as soon as a fair share of the SMs gets one: with fewer panels than CTAs
// the idle SMs cost less than the K split's fix-up does (1280 x 8192, 80 panels: 4.9 us on 80 CTAs
// against 8.9 us split over 148).  Below that the split kernel spreads the few panels over all SMs.
bool wp_has_enough_panels(const qgemv_handle* h, const qgemv_weight* w) {
    const int64_t g = gemv_grid(h);
    return w->n_panels >= g || w->n_panels >= std::max<int64_t>(32, g / 4);
}

int launch_gemv(const qgemv_handle* h, const qgemv_weight* w, const qg::GemvParams& P,
                cudaStream_t stream) {
    const dim3 grid(gemv_grid(h)), block(qg::kThreads);
    cudaError_t err;
    if (qg::use_stream_path(P.prob == nullptr, P.B, P.units) && !(h->cfg.debug & 256)) {
        const dim3 sblock(qg::kSThreads);
        // whole panels per CTA (no cross-CTA fix-up)
        // (the whole-panel kernel keeps weight offsets in 32 bits: matrices of 4 GiB and more take the split kernel,
        // whose offsets are 64-bit)
        const bool whole = wp_has_enough_panels(h, w) && !(h->cfg.debug & 512) && w->payload_bytes < (uint64_t(1) << 32);
        if (w->fmt == QGEMV_FMT_NVFP4) {
            const size_t smem = qg::SSmem::total<QGEMV_FMT_NVFP4>();
            const bool full = P.units % qg::StreamTraits<QGEMV_FMT_NVFP4>::kChunkUnits == 0;
            const bool shortk = P.units < 16 * qg::StreamTraits<QGEMV_FMT_NVFP4>::kChunkUnits;
            err = !whole ? launch(h, qg::gemv_stream_kernel<QGEMV_FMT_NVFP4>, grid, sblock, smem, stream, P)
                  : shortk ? (full ? launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, true, 1, true>, grid, sblock, smem, stream, P)
                                   : launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, false, 1, true>, grid, sblock, smem, stream, P))
                  : full ? launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, true, 1>, grid, sblock, smem, stream, P)
                         : launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, false, 1>, grid, sblock, smem, stream, P);
        } else {
            const size_t smem = qg::SSmem::total<QGEMV_FMT_FP8>();
            const bool full = P.units % qg::StreamTraits<QGEMV_FMT_FP8>::kChunkUnits == 0;
            const bool shortk = P.units < 16 * qg::StreamTraits<QGEMV_FMT_FP8>::kChunkUnits;
            err = !whole ? launch(h, qg::gemv_stream_kernel<QGEMV_FMT_FP8>, grid, sblock, smem, stream, P)
                  : shortk ? (full ? launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, true, 1, true>, grid, sblock, smem, stream, P)
                                   : launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, false, 1, true>, grid, sblock, smem, stream, P))
                  : full ? launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, true, 1>, grid, sblock, smem, stream, P)
                         : launch(h, qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, false, 1>, grid, sblock, smem, stream, P);
        }
        return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
    }
    const bool res = qg::use_resident_path(P.prob == nullptr, P.B, w->units);
    if (w->fmt == QGEMV_FMT_NVFP4) {
        const size_t smem = qg::Smem::total<QGEMV_FMT_NVFP4>();
        err = res ? launch(h, qg::gemv_kernel<QGEMV_FMT_NVFP4, true>, grid, block, smem, stream, P)
                  : launch(h, qg::gemv_kernel<QGEMV_FMT_NVFP4, false>, grid, block, smem, stream, P);
    } else {
        const size_t smem = qg::Smem::total<QGEMV_FMT_FP8>();
        err = res ? launch(h, qg::gemv_kernel<QGEMV_FMT_FP8, true>, grid, block, smem, stream, P)
                  : launch(h, qg::gemv_kernel<QGEMV_FMT_FP8, false>, grid, block, smem, stream, P);
    }
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}

// ---- tensor-core GEMV (QGEMV_FMT_NVFP4_TC) -------------------------------------------------------
// Shared-memory plan of one launch over `kt_len` items per tile: digit-plane slots for the items a
// CTA can own, then as many ring stages as the cap allows.
struct TcPlan {
    int grid, npad, x_slots, ring, stage_items, cluster;
    size_t smem;
};
bool tc_plan(const qgemv_handle* h, int64_t tiles, int64_t kt_len, int B, TcPlan* pl) {
    const int64_t total = tiles * kt_len;
    pl->grid = int(std::min<int64_t>(gemv_grid(h), total));
    // Optional (debug bit 5), for matrices with few row tiles: a thread-block cluster per tile, the
    // tile's K range cut evenly over its CTAs, partial sums handed over in distributed shared memory.
    // Measured on the 8B stack it shortens the hand-over (1.5 against 2.3 us after the last MMA) but
    // some clusters are scheduled late behind the previous launch's, and the layer gets slower
    // (40.7 against 38.4 us): off by default.
    pl->cluster = 1;
    if (h->cfg.grid_override == 0 && (h->cfg.debug & 32) && tiles * 2 <= h->sm_count && kt_len >= 2) {
        const int64_t c = std::min<int64_t>({8, h->sm_count / tiles, kt_len});
        if (c >= 2) {
            pl->cluster = int(c);
            pl->grid = int(tiles * c);
        }
    }
    pl->npad = (8 * B + 15) / 16 * 16;  // M = 128 wants N in multiples of 16 (N = 8 gave wrong sums and a memory fault)
    const int64_t per_cta = (total + pl->grid - 1) / pl->grid;
    pl->x_slots = int(std::min<int64_t>(kt_len, per_cta));
    const int si = h->cfg.tc_stage_items;
    pl->stage_items = si >= 8 ? 8 : (si >= 4 ? 4 : (si >= 2 ? 2 : (si == 1 ? 1 : 4)));  // 1, 2, 4 or 8; default 4
    const int stage_bytes = pl->stage_items * qg::kTcItemBytes;
    const int base = qg::TcSmem::ring_off(pl->x_slots, pl->npad, pl->cluster, B);
    // Prefer a footprint of about half an SM: the CTA of the next kernel in the stream is then
    // resident beside this one and fills its ring while this one still streams.
    const int want_cap = (h->cfg.tc_smem_kb > 0 ? std::min(h->cfg.tc_smem_kb, 227) : 112) * 1024;
    int ring = (want_cap - base) / stage_bytes;
    if (ring < 4) ring = (qg::kGsSmemBudget - base) / stage_bytes;  // large activations: the whole SM
    if (ring > qg::kTcMaxRing) ring = qg::kTcMaxRing;
    // every ring item owns a 4-column slot of block scales in tensor memory
    ring = std::min(ring, qg::TcSmem::max_ring_items(pl->npad) / pl->stage_items);
    if (ring < 2) return false;
    pl->ring = ring;
    pl->smem = size_t(qg::TcSmem::total(pl->x_slots, pl->npad, ring, pl->stage_items, pl->cluster, B));
    return pl->smem <= size_t(qg::kGsSmemBudget);
}

int gemv_tc(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int B, void* y, int y_dtype,
            const qgemv_weight* next, cudaStream_t stream) {
    const int64_t tiles = w->n_panels / 8, kt_total = w->units;
    // K window per launch: the whole K when the digit planes of a CTA's items fit beside a ring,
    // otherwise chunks of items whose fp32 results are added in chunk order (as the K-chunked
    // CUDA-core path does; the chunk length depends on B).
    int64_t kt_chunk = kt_total;
    TcPlan pl;
    while (!tc_plan(h, tiles, kt_chunk, B, &pl)) {
        if (kt_chunk <= 4) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        kt_chunk = ((kt_chunk + 1) / 2 + 3) / 4 * 4;
    }
    const int64_t n_chunks = (kt_total + kt_chunk - 1) / kt_chunk;
    const int64_t slice = int64_t(B) * w->N;
    if (n_chunks > 1 && size_t(n_chunks * slice) * sizeof(float) > kChunkWsBytes) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    for (int64_t c = 0; c < n_chunks; ++c) {
        const int64_t k0 = c * kt_chunk, k1 = std::min(kt_total, k0 + kt_chunk);
        if (k1 - k0 != kt_chunk && !tc_plan(h, tiles, k1 - k0, B, &pl)) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        qg::TcParams P;
        std::memset(&P, 0, sizeof P);
        P.payload = w->dev_blob + QG_HEADER_BYTES + w->aux_bytes;
        P.x = static_cast<const uint16_t*>(x_bf16) + k0 * 64;
        P.y = n_chunks == 1 ? y : static_cast<void*>(h->chunk_ws + c * slice);
        P.ws = h->tc_ws;
        P.status = h->status_dev;
        P.spin_limit = default_spin(h);
        P.tensor_scale = w->host_tensor_scale[0];
        P.N = int32_t(w->N);
        P.K = int32_t(std::min<int64_t>(w->K - k0 * 64, (k1 - k0) * 64));
        P.tiles = int32_t(tiles);
        P.kt_total = int32_t(kt_total);
        P.kt0 = int32_t(k0);
        P.kt_len = int32_t(k1 - k0);
        P.x_stride = int32_t(w->K);
        P.B = B;
        P.y_dtype = n_chunks == 1 ? y_dtype : QGEMV_OUT_F32;
        P.debug = h->cfg.debug;
        P.npad = pl.npad;
        P.ring = pl.ring;
        P.stage_items = pl.stage_items;
        P.x_slots = pl.x_slots;
        P.cluster = pl.cluster;
        P.trace = h->tc_trace;
        if (next && next->fmt == QGEMV_FMT_NVFP4_TC && next->n_stack == 1 && c + 1 == n_chunks) {
            // the last launch of this call pulls the next weight towards L2, split as its own launch
            // (same batch assumed) will split it
            TcPlan np;
            if (tc_plan(h, next->n_panels / 8, next->units, B, &np)) {
                P.pf_base = next->dev_blob + QG_HEADER_BYTES + next->aux_bytes;
                P.pf_total = int32_t(next->n_panels / 8 * next->units);
                P.pf_grid = np.grid;
                P.pf_skip = uint32_t(np.ring) * uint32_t(np.stage_items) * qg::kTcItemBytes;
            }
        }
        const dim3 g(unsigned(pl.grid)), blk(qg::kTcThreads);
        g_launch_cluster = pl.cluster;
        const cudaError_t err = pl.stage_items == 1   ? launch(h, qg::gemv_tc_kernel<1>, g, blk, pl.smem, stream, P)
                                : pl.stage_items == 2 ? launch(h, qg::gemv_tc_kernel<2>, g, blk, pl.smem, stream, P)
                                : pl.stage_items == 4 ? launch(h, qg::gemv_tc_kernel<4>, g, blk, pl.smem, stream, P)
                                                      : launch(h, qg::gemv_tc_kernel<8>, g, blk, pl.smem, stream, P);
        if (err != cudaSuccess) return QGEMV_ERR_CUDA;
    }
    if (n_chunks > 1) {
        const cudaError_t err = launch(h, qg::chunk_sum_kernel, dim3(unsigned((slice + 255) / 256)), dim3(256), 0, stream,
                                       static_cast<const float*>(h->chunk_ws), int(n_chunks), slice, y, y_dtype);
        return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
    }
    return QGEMV_OK;
}

}  // namespace

extern "C" {

const char* qgemv_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda_error); }

const char* qgemv_status_string(int status) {
    switch (status) {
        case QGEMV_OK: return "ok";
        case QGEMV_ERR_INVALID_ARG: return "invalid argument";
        case QGEMV_ERR_BAD_BLOB: return "bad packed-weight blob";
        case QGEMV_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
        case QGEMV_ERR_CUDA: return "CUDA error";
        case QGEMV_ERR_NCCL: return "NCCL error";
        case QGEMV_ERR_TIMEOUT: return "device wait timed out";
        case QGEMV_ERR_BOUNDS: return "device bounds check failed";
        case QGEMV_ERR_NO_DEVICE: return "no CUDA device";
        default: return "unknown status";
    }
}

int qgemv_init(const qgemv_config* cfg, qgemv_handle** out) {
    if (!cfg || !out) return QGEMV_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        return QGEMV_ERR_NO_DEVICE;
    }
    if (cfg->device < 0 || cfg->device >= count) return QGEMV_ERR_INVALID_ARG;
    QG_CUDA(cudaSetDevice(cfg->device));
    cudaDeviceProp prop;
    QG_CUDA(cudaGetDeviceProperties(&prop, cfg->device));
    if (prop.major != 10) return QGEMV_ERR_NO_DEVICE;  // built for sm_100a only
    qgemv_handle* h = new (std::nothrow) qgemv_handle;
    if (!h) return QGEMV_ERR_INVALID_ARG;
    h->cfg = *cfg;
    h->sm_count = prop.multiProcessorCount;
    h->status_dev = nullptr;
    h->tp_rank = 0, h->tp_world = 0, h->tp_max_elems = 0;
    h->tp_local = nullptr, h->tp_epochs = nullptr;
    for (int i = 0; i < qg::kTpMaxWorld; ++i) h->tp_peer[i] = nullptr, h->tp_ipc_opened[i] = false;
    h->tp_seq_cursor = 0, h->tp_call_high = 0;
    h->gs_ws = nullptr, h->gs_ws_bytes = 0;
    h->chunk_ws = nullptr;
    h->tc_ws = nullptr, h->tc_trace = nullptr, h->seq_barrier = nullptr, h->seq_parts = nullptr, h->moe_cnt = nullptr;
    h->a4_ws = nullptr, h->a4_ws_bytes = 0;
    h->sequences = new (std::nothrow) std::vector<qgemv_sequence*>();
    const size_t tc_ws_bytes = size_t(2) * size_t(std::max(h->sm_count, cfg->grid_override)) * 1024 * 8;
    h->tc_ws_bytes = tc_ws_bytes;
    if (cudaMalloc(&h->tc_ws, tc_ws_bytes) != cudaSuccess || cudaMemset(h->tc_ws, 0, tc_ws_bytes) != cudaSuccess ||
        cudaMalloc(&h->seq_barrier, 256) != cudaSuccess || cudaMemset(h->seq_barrier, 0, 256) != cudaSuccess ||
        cudaMalloc(&h->moe_cnt, 2048 * 4) != cudaSuccess || cudaMemset(h->moe_cnt, 0, 2048 * 4) != cudaSuccess ||
        cudaMalloc(&h->seq_parts, size_t(qg::kSeqPartBufs) * size_t(2) * size_t(std::max(h->sm_count, cfg->grid_override)) * 8192) != cudaSuccess ||
        cudaMalloc(&h->chunk_ws, kChunkWsBytes) != cudaSuccess ||
        cudaMalloc(&h->status_dev, 4 * sizeof(int32_t)) != cudaSuccess ||
        cudaMemset(h->status_dev, 0, 4 * sizeof(int32_t)) != cudaSuccess) {
        g_last_cuda_error = cudaGetLastError();
        qgemv_destroy(h);  // frees whatever was allocated
        return QGEMV_ERR_CUDA;
    }
    const cudaFuncAttribute dyn = cudaFuncAttributeMaxDynamicSharedMemorySize;
    if (cudaFuncSetAttribute(qg::gemv_kernel<QGEMV_FMT_NVFP4, true>, dyn, qg::Smem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_kernel<QGEMV_FMT_NVFP4, false>, dyn, qg::Smem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_kernel<QGEMV_FMT_FP8, true>, dyn, qg::Smem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_kernel<QGEMV_FMT_FP8, false>, dyn, qg::Smem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_kernel<QGEMV_FMT_NVFP4>, dyn, qg::SSmem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_kernel<QGEMV_FMT_FP8>, dyn, qg::SSmem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::moe_stream_kernel<QGEMV_FMT_NVFP4>, dyn, qg::MSmem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::moe_stream_kernel<QGEMV_FMT_FP8>, dyn, qg::MSmem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, true, 1>, dyn, qg::SSmem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, false, 1>, dyn, qg::SSmem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, true, 1>, dyn, qg::SSmem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, false, 1>, dyn, qg::SSmem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, true, 1, true>, dyn, qg::SSmem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_NVFP4, false, 1, true>, dyn, qg::SSmem::total<QGEMV_FMT_NVFP4>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, true, 1, true>, dyn, qg::SSmem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_stream_wp_kernel<QGEMV_FMT_FP8, false, 1, true>, dyn, qg::SSmem::total<QGEMV_FMT_FP8>()) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<2, qg::kSeqPlain>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<4, qg::kSeqPlain>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<8, qg::kSeqPlain>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<2, qg::kSeqFuse>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<4, qg::kSeqFuse>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<8, qg::kSeqFuse>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_seq_kernel<4, qg::kSeqMoe>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_tc_kernel<1>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_tc_kernel<2>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_tc_kernel<4>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemv_tc_kernel<8>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemm_skinny_kernel<QGEMV_FMT_NVFP4>, dyn, qg::kGsSmemBudget) != cudaSuccess ||
        cudaFuncSetAttribute(qg::gemm_skinny_kernel<QGEMV_FMT_FP8>, dyn, qg::kGsSmemBudget) != cudaSuccess) {
        g_last_cuda_error = cudaGetLastError();
        qgemv_destroy(h);
        return QGEMV_ERR_CUDA;
    }
    *out = h;
    return QGEMV_OK;
}

int qgemv_destroy(qgemv_handle* h) {
    if (!h) return QGEMV_ERR_INVALID_ARG;
    cudaSetDevice(h->cfg.device);
    for (int i = 0; i < h->tp_world; ++i)
        if (i != h->tp_rank && h->tp_peer[i] && h->tp_ipc_opened[i]) cudaIpcCloseMemHandle(h->tp_peer[i]);
    cudaFree(h->tp_local);
    cudaFree(h->tp_epochs);
    cudaFree(h->gs_ws);
    cudaFree(h->chunk_ws);
    cudaFree(h->tc_ws);
    cudaFree(h->seq_barrier);
    cudaFree(h->seq_parts);
    cudaFree(h->moe_cnt);
    cudaFree(h->a4_ws);
    delete h->sequences;
    cudaFree(h->status_dev);
    delete h;
    return QGEMV_OK;
}

int qgemv_sm_count(const qgemv_handle* h) { return h ? h->sm_count : QGEMV_ERR_INVALID_ARG; }

int qgemv_set_trace(qgemv_handle* h, void* dev_buf) {
    if (!h) return QGEMV_ERR_INVALID_ARG;
    h->tc_trace = static_cast<unsigned long long*>(dev_buf);
    return QGEMV_OK;
}

namespace {
// Allocates a weight object and its device buffers for n_stacked blobs with header `h0`; the blob
// bytes themselves are put there by the caller.
int new_weight(qgemv_handle* h, const qg_blob_header* h0, int n_stacked, size_t bytes_each, const float* ts,
               qgemv_weight** out) {
    if (h0->N > INT32_MAX || h0->K > INT32_MAX || h0->n_panels * h0->units_per_panel > (int64_t(1) << 40))
        return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (h0->fmt == QGEMV_FMT_NVFP4_TC && h0->n_panels / 8 * h0->units_per_panel > INT32_MAX)
        return QGEMV_ERR_UNSUPPORTED_SHAPE;
    QG_CUDA(cudaSetDevice(h->cfg.device));
    qgemv_weight* w = new (std::nothrow) qgemv_weight;
    if (!w) return QGEMV_ERR_INVALID_ARG;
    std::memset(w, 0, sizeof *w);
    w->fmt = int(h0->fmt);
    w->N = h0->N;
    w->K = h0->K;
    w->n_panels = h0->n_panels;
    w->units = h0->units_per_panel;
    w->n_stack = n_stacked;
    w->blob_bytes = bytes_each;
    w->aux_bytes = h0->aux_bytes;
    w->payload_bytes = h0->payload_bytes;
    w->host_tensor_scale = new (std::nothrow) float[size_t(n_stacked)];
    if (!w->host_tensor_scale) {
        delete w;
        return QGEMV_ERR_INVALID_ARG;
    }
    std::memcpy(w->host_tensor_scale, ts, size_t(n_stacked) * 4);
    w->max_prob = n_stacked > 1 ? n_stacked + kMaxMoeSlots / 8 : 1;
    const size_t n_counters = size_t(w->max_prob) * size_t(w->n_panels);
    const size_t ws_bytes = size_t(2) * size_t(gemv_grid(h) > h->sm_count ? gemv_grid(h) : h->sm_count) * 512;
    bool ok = cudaMalloc(&w->dev_blob, size_t(n_stacked) * bytes_each) == cudaSuccess &&
              cudaMalloc(&w->dev_tensor_scale, size_t(n_stacked) * 4) == cudaSuccess &&
              cudaMalloc(&w->ws, ws_bytes) == cudaSuccess &&
              cudaMalloc(&w->counters, n_counters * 4) == cudaSuccess;
    if (ok && n_stacked > 1)
        ok = cudaMalloc(&w->prob, (size_t(w->max_prob) * qg::kProbInts + 1) * 4) == cudaSuccess;
    ok = ok && cudaMemcpy(w->dev_tensor_scale, ts, size_t(n_stacked) * 4, cudaMemcpyHostToDevice) == cudaSuccess &&
         cudaMemset(w->counters, 0, n_counters * 4) == cudaSuccess &&
         cudaMemset(w->ws, 0, ws_bytes) == cudaSuccess;
    if (ok && w->prob) ok = cudaMemset(w->prob, 0, (size_t(w->max_prob) * qg::kProbInts + 1) * 4) == cudaSuccess;
    if (!ok) {
        g_last_cuda_error = cudaGetLastError();
        qgemv_unload(h, w);
        return QGEMV_ERR_CUDA;
    }
    *out = w;
    return QGEMV_OK;
}
}  // namespace

int qgemv_load_stacked(qgemv_handle* h, const void* host_blobs, size_t bytes_each, int n_stacked,
                       qgemv_weight** out) {
    if (!h || !host_blobs || !out || n_stacked <= 0) return QGEMV_ERR_INVALID_ARG;
    *out = nullptr;
    const uint8_t* src = static_cast<const uint8_t*>(host_blobs);
    const qg_blob_header* h0 = reinterpret_cast<const qg_blob_header*>(src);
    std::vector<float> ts(size_t(n_stacked), 1.0f);
    for (int i = 0; i < n_stacked; ++i) {
        const uint8_t* b = src + size_t(i) * bytes_each;
        if (qgemv_blob_verify(b, bytes_each) != QGEMV_OK) return QGEMV_ERR_BAD_BLOB;
        const qg_blob_header* hi = reinterpret_cast<const qg_blob_header*>(b);
        if (hi->fmt != h0->fmt || hi->N != h0->N || hi->K != h0->K) return QGEMV_ERR_BAD_BLOB;
        ts[size_t(i)] = hi->tensor_scale;
    }
    qgemv_weight* w = nullptr;
    const int rc = new_weight(h, h0, n_stacked, bytes_each, ts.data(), &w);
    if (rc != QGEMV_OK) return rc;
    if (cudaMemcpy(w->dev_blob, src, size_t(n_stacked) * bytes_each, cudaMemcpyHostToDevice) != cudaSuccess) {
        g_last_cuda_error = cudaGetLastError();
        qgemv_unload(h, w);
        return QGEMV_ERR_CUDA;
    }
    *out = w;
    return QGEMV_OK;
}

namespace {
// Packs one canonical NVFP4 matrix (device memory) into blob `which` of a tensor-core-layout weight: header by a
// copy, payload by the packing kernel.  `hd` must stay alive until the stream has been synchronised.
bool pack_tc_into(qgemv_handle* h, qgemv_weight* w, int which, const void* codes_dev, const void* scales_dev,
                  const qg_blob_header* hd, int64_t N, int64_t K, const qgemv_shard* shard, cudaStream_t st) {
    uint8_t* blob = w->dev_blob + uint64_t(which) * w->blob_bytes;
    qg::PackTcParams P;
    P.codes = static_cast<const uint8_t*>(codes_dev);
    P.scales = static_cast<const uint8_t*>(scales_dev);
    P.payload = blob + QG_HEADER_BYTES + hd->aux_bytes;
    P.N = N, P.K = K;
    P.n0 = shard ? shard->n0 : 0, P.k0 = shard ? shard->k0 : 0;
    P.n = hd->N, P.k = hd->K;
    P.tiles = hd->n_panels / 8, P.kt = hd->units_per_panel;
    const int64_t chunks = P.tiles * P.kt * (QG_TC_ITEM_BYTES / 16);
    const unsigned blocks = unsigned(std::min<int64_t>((chunks + 255) / 256, int64_t(h->sm_count) * 16));
    if (cudaMemcpyAsync(blob, hd, sizeof *hd, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    qg::pack_tc_kernel<<<blocks, 256, 0, st>>>(P);
    return cudaGetLastError() == cudaSuccess;
}
}  // namespace

int qgemv_load_device(qgemv_handle* h, int fmt, const void* codes_dev, const void* scales_dev, float tensor_scale,
                      int64_t N, int64_t K, const qgemv_shard* shard, void* stream, qgemv_weight** out) {
    const void* c[1] = {codes_dev};
    const void* sc[1] = {scales_dev};
    return qgemv_load_stacked_device(h, fmt, c, sc, &tensor_scale, 1, N, K, shard, stream, out);
}

int qgemv_load_stacked_device(qgemv_handle* h, int fmt, const void* const* codes_dev, const void* const* scales_dev,
                              const float* tensor_scales, int n_stacked, int64_t N, int64_t K, const qgemv_shard* shard,
                              void* stream, qgemv_weight** out) {
    if (!h || !codes_dev || !scales_dev || !tensor_scales || !out || n_stacked < 1) return QGEMV_ERR_INVALID_ARG;
    *out = nullptr;
    if (fmt != QGEMV_FMT_NVFP4_TC) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    for (int e = 0; e < n_stacked; ++e) {
        if (!codes_dev[e] || !scales_dev[e]) return QGEMV_ERR_INVALID_ARG;
        if ((reinterpret_cast<uintptr_t>(codes_dev[e]) & 7u) != 0) return QGEMV_ERR_INVALID_ARG;  // read in 8-byte groups
    }
    std::vector<qg_blob_header> hd(static_cast<size_t>(n_stacked));
    for (int e = 0; e < n_stacked; ++e) {
        const int rc0 = qgemv_pack_header(fmt, tensor_scales[e], N, K, shard, &hd[size_t(e)]);
        if (rc0 != QGEMV_OK) return rc0;
    }
    qgemv_weight* w = nullptr;
    const int rc = new_weight(h, &hd[0], n_stacked, size_t(QG_HEADER_BYTES + hd[0].aux_bytes + hd[0].payload_bytes), tensor_scales, &w);
    if (rc != QGEMV_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool ok = true;
    for (int e = 0; e < n_stacked && ok; ++e) ok = pack_tc_into(h, w, e, codes_dev[e], scales_dev[e], &hd[size_t(e)], N, K, shard, st);
    ok = cudaStreamSynchronize(st) == cudaSuccess && ok;  // (the headers live in this frame)
    if (!ok) {
        g_last_cuda_error = cudaGetLastError();
        qgemv_unload(h, w);
        return QGEMV_ERR_CUDA;
    }
    *out = w;
    return QGEMV_OK;
}

int qgemv_load(qgemv_handle* h, const void* host_blob, size_t bytes, qgemv_weight** out) {
    return qgemv_load_stacked(h, host_blob, bytes, 1, out);
}

int qgemv_unload(qgemv_handle* h, qgemv_weight* w) {
    if (!h || !w) return QGEMV_ERR_INVALID_ARG;
    cudaSetDevice(h->cfg.device);
    cudaFree(w->dev_blob);
    cudaFree(w->dev_tensor_scale);
    cudaFree(w->ws);
    cudaFree(w->counters);
    cudaFree(w->prob);
    delete[] w->host_tensor_scale;
    delete w;
    return QGEMV_OK;
}

int qgemv_weight_read(qgemv_handle* h, const qgemv_weight* w, void* host_out, size_t bytes) {
    if (!h || !w || !host_out) return QGEMV_ERR_INVALID_ARG;
    if (bytes != size_t(w->n_stack) * w->blob_bytes) return QGEMV_ERR_INVALID_ARG;
    QG_CUDA(cudaSetDevice(h->cfg.device));
    QG_CUDA(cudaMemcpy(host_out, w->dev_blob, bytes, cudaMemcpyDeviceToHost));
    return QGEMV_OK;
}

int64_t qgemv_weight_bytes(const qgemv_weight* w) {
    if (!w) return QGEMV_ERR_INVALID_ARG;
    if (w->fmt != QGEMV_FMT_FP8) return w->N * w->K / 2 + w->N * w->K / 16 + 4;
    return w->N * w->K + 4 * w->N;
}

int qgemv_sequence_create(qgemv_handle* h, const qgemv_job* jobs, int n_jobs, int B, qgemv_sequence** out) {
    if (!h || !jobs || !out || n_jobs < 1) return QGEMV_ERR_INVALID_ARG;
    *out = nullptr;
    if (B < 1 || B > QGEMV_MAX_BATCH) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    const int grid = gemv_grid(h);
    if (grid > h->sm_count) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // the CTAs wait on one another: one per SM at most
    std::vector<qg::SeqJob> tab(static_cast<size_t>(n_jobs));
    int64_t x_slots = 1, xchg_elems = 0;
    bool fused = false;
    for (int i = 0; i < n_jobs; ++i) {
        const qgemv_job& jb = jobs[i];
        if (!jb.w || !jb.x || !jb.y) return QGEMV_ERR_INVALID_ARG;
        if (jb.w->fmt != QGEMV_FMT_NVFP4_TC || jb.w->n_stack != 1) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        if (jb.y_dtype != QGEMV_OUT_BF16 && jb.y_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
        if ((reinterpret_cast<uintptr_t>(jb.x) & 15u) != 0) return QGEMV_ERR_INVALID_ARG;
        qg::SeqJob& sj = tab[size_t(i)];
        std::memset(&sj, 0, sizeof sj);
        sj.payload = jb.w->dev_blob + QG_HEADER_BYTES + jb.w->aux_bytes;
        sj.x = static_cast<const uint16_t*>(jb.x);
        sj.y = jb.y;
        sj.tensor_scale = jb.w->host_tensor_scale[0];
        sj.N = int32_t(jb.w->N), sj.K = int32_t(jb.w->K);
        sj.tiles = int32_t(jb.w->n_panels / 8), sj.kt = int32_t(jb.w->units);
        sj.y_dtype = jb.y_dtype;
        // Ordering against the earlier jobs, from the address ranges.  RAW: x inside an earlier y.  WAW /
        // WAR: y over an earlier y or x.  The common chain -- x is (a column range of) the bf16 output of
        // ONE earlier job, every row, same row stride -- takes the fast way: the producer publishes its
        // rows as tagged words and this job's conversion picks them up as they appear (src_job).  Every
        // other hazard waits until the job in question is complete on every CTA (dep).
        sj.dep = -1, sj.xoff = -1, sj.pub_off = -1, sj.src_off = -1, sj.src_job = -1;
        if ((jb.flags & ~(QGEMV_JOB_AFTER_PREVIOUS | QGEMV_JOB_ALLREDUCE | QGEMV_JOB_X_SILU_MUL)) != 0 || jb.reserved != 0) return QGEMV_ERR_INVALID_ARG;
        const int64_t x_cols = (jb.flags & QGEMV_JOB_X_SILU_MUL) != 0 ? 2 * jb.w->K : jb.w->K;   // values per stored row of x
        if (jb.x_stride != 0 && (jb.x_stride < x_cols || jb.x_stride > INT32_MAX || (jb.x_stride % 8) != 0)) return QGEMV_ERR_INVALID_ARG;
        if ((jb.flags & QGEMV_JOB_X_SILU_MUL) != 0 && jb.w->K % 8 != 0) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        if (jb.norm_weight && ((reinterpret_cast<uintptr_t>(jb.norm_weight) & 15u) != 0 || !(jb.norm_eps >= 0.f))) return QGEMV_ERR_INVALID_ARG;
        sj.x_stride = int32_t(jb.x_stride != 0 ? jb.x_stride : x_cols);
        sj.act = (jb.flags & QGEMV_JOB_X_SILU_MUL) != 0 ? 1 : 0;
        sj.norm_w = static_cast<const uint16_t*>(jb.norm_weight);
        sj.norm_eps = jb.norm_eps;
        sj.residual = jb.residual;
        if (sj.act || sj.norm_w || sj.residual) fused = true;
        {
            const auto lo = [](const void* p) { return reinterpret_cast<uintptr_t>(p); };
            const auto ysize = [&](const qgemv_job& q) { return size_t(B) * size_t(q.w->N) * (q.y_dtype == QGEMV_OUT_F32 ? 4 : 2); };
            const auto xsize = [&](const qgemv_job& q) {
                const size_t cols = (q.flags & QGEMV_JOB_X_SILU_MUL) != 0 ? size_t(2 * q.w->K) : size_t(q.w->K);
                const size_t st = q.x_stride != 0 ? size_t(q.x_stride) : cols;
                return (size_t(B - 1) * st + cols) * 2;
            };
            const uintptr_t x0 = lo(jb.x), x1 = x0 + xsize(jb), y0 = lo(jb.y), y1 = y0 + ysize(jb);
            int raw = -1, n_raw = 0, other = -1;
            for (int e = i - 1; e >= 0; --e) {
                const qgemv_job& pj = jobs[e];
                const uintptr_t py0 = lo(pj.y), py1 = py0 + ysize(pj), px0 = lo(pj.x), px1 = px0 + xsize(pj);
                const uintptr_t r0 = lo(jb.residual), r1 = jb.residual ? r0 + ysize(jb) : r0;   // the residual is read as well
                const bool r = x0 < py1 && py0 < x1, o = (y0 < py1 && py0 < y1) || (y0 < px1 && px0 < y1) || (r0 < py1 && py0 < r1);
                if (r && n_raw++ == 0) raw = e;
                if (o && other < 0) other = e;
            }
            bool fast = false;
            if (n_raw == 1 && raw > other && (jb.flags & QGEMV_JOB_AFTER_PREVIOUS) == 0) {
                const qgemv_job& pj = jobs[raw];
                const uintptr_t py0 = lo(pj.y);
                const int64_t c0 = (int64_t(x0) - int64_t(py0)) / 2;
                if (pj.y_dtype == QGEMV_OUT_BF16 && x0 >= py0 && c0 + x_cols <= pj.w->N && (B == 1 || sj.x_stride == pj.w->N) &&
                    (pj.w->N % 4) == 0 && (c0 % 4) == 0) {
                    fast = true;
                    sj.src_job = raw;
                    sj.src_off = int32_t(c0);        // + the producer's pub_off, below
                    sj.x_stride = int32_t(pj.w->N);
                }
            }
            sj.dep = fast ? other : std::max(raw, other);
            if ((jb.flags & QGEMV_JOB_AFTER_PREVIOUS) != 0 && i > 0) sj.dep = i - 1;
        }
        if ((jb.flags & QGEMV_JOB_ALLREDUCE) != 0 && h->tp_world > 1) {
            // the sum over the ranks is formed by the thread that adds up a split row tile: every
            // tile must be split, i.e. no CTA's share of the job may hold a whole tile
            const int64_t tot = int64_t(sj.tiles) * sj.kt;
            const int64_t gj = std::min<int64_t>(grid, tot);
            if ((tot + gj - 1) / gj >= sj.kt) return QGEMV_ERR_UNSUPPORTED_SHAPE;
            for (int r = 0; r < h->tp_world; ++r)
                if (!h->tp_peer[r]) return QGEMV_ERR_INVALID_ARG;  // qgemv_tp_connect has not run
            xchg_elems += int64_t(B) * sj.N;
            sj.xoff = 0;  // placed below, once the total is known
        }
        const int64_t total = int64_t(sj.tiles) * sj.kt;
        if ((total + 1) * grid >= (int64_t(1) << 32)) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // the kernel splits in 32-bit arithmetic
        x_slots = std::max(x_slots, std::min<int64_t>(sj.kt, (total + grid - 1) / grid));
    }
    if (n_jobs > 4094) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // the job index is part of a 12-bit tag
    // a job whose counter a later job waits for (dep) bumps it with release semantics
    for (int i = 0; i < n_jobs; ++i)
        if (tab[size_t(i)].dep >= 0) tab[size_t(tab[size_t(i)].dep)].fin_release = 1;
    // published outputs: one block of B * N words for every job that a later job reads the fast way
    int64_t pub_words = 0;
    for (int i = 0; i < n_jobs; ++i) {
        qg::SeqJob& sj = tab[size_t(i)];
        if (sj.src_job < 0) continue;
        qg::SeqJob& pj = tab[size_t(sj.src_job)];
        if (pj.pub_off < 0) {
            pj.pub_off = int32_t(pub_words);
            pub_words += (int64_t(B) * pj.N + 3) / 4 * 4;
            if (pub_words > INT32_MAX / 2) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        }
        sj.src_off += pj.pub_off;
    }
    // the all-reduce jobs take their blocks from the top of the exchange slots downwards
    if (xchg_elems > 0 && h->tp_seq_cursor - xchg_elems < h->tp_call_high) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    {
        int64_t off = h->tp_seq_cursor - xchg_elems;
        for (qg::SeqJob& sj : tab)
            if (sj.xoff >= 0) sj.xoff = int32_t(off), off += int64_t(B) * sj.N;
    }
    qgemv_sequence* q = new (std::nothrow) qgemv_sequence;
    if (!q) return QGEMV_ERR_INVALID_ARG;
    q->dev_jobs = nullptr, q->dev_counters = nullptr, q->dev_pub = nullptr;
    q->xchg_elems = xchg_elems, q->xchg_first = h->tp_seq_cursor - xchg_elems;
    q->fused = fused;
    q->n_jobs = n_jobs, q->B = B, q->grid = grid;
    q->npad = (8 * B + 15) / 16 * 16;
    q->x_slots = int(x_slots);
    const int si = h->cfg.tc_stage_items;
    q->stage_items = si >= 8 ? 8 : (si >= 4 ? 4 : (si >= 2 ? 2 : 4));
    const int cap = (h->cfg.tc_smem_kb > 0 ? std::min(h->cfg.tc_smem_kb, 227) : 227) * 1024;
    // As many plane buffers (jobs the conversion may run ahead) as still leave a ring of four stages.  A list in
    // which most jobs wait for the one before them cannot run ahead: there one buffer is enough and the shared
    // memory goes to the weight ring, which keeps HBM busy while a job waits for its input.
    int n_chain = 0;
    for (int i = 1; i < n_jobs; ++i)
        if (tab[size_t(i)].src_job == i - 1 || tab[size_t(i)].dep == i - 1) ++n_chain;
    const int nbuf_max = 2 * n_chain > n_jobs ? 1 : qg::kSeqPlaneBufsMax;
    int ring = 0;
    for (q->nbuf = nbuf_max; q->nbuf >= 1; --q->nbuf) {
        const int base = qg::SeqSmem::ring_off(q->x_slots, q->npad, q->nbuf);
        ring = (cap - base) / (q->stage_items * qg::kTcItemBytes);
        ring = std::min({ring, qg::kTcMaxRing, qg::SeqSmem::max_ring_items(q->npad) / q->stage_items});
        if (ring >= 4 || q->nbuf == 1) break;
    }
    if (ring < 2) {
        delete q;
        return QGEMV_ERR_UNSUPPORTED_SHAPE;  // the digit planes of one job leave no room for a ring: call qgemv_gemv per job
    }
    q->ring = ring;
    q->smem = size_t(qg::SeqSmem::total(q->x_slots, q->npad, q->nbuf, ring, q->stage_items));
    if (cudaSetDevice(h->cfg.device) != cudaSuccess || cudaMalloc(&q->dev_jobs, size_t(n_jobs) * sizeof(qg::SeqJob)) != cudaSuccess ||
        cudaMemcpy(q->dev_jobs, tab.data(), size_t(n_jobs) * sizeof(qg::SeqJob), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMalloc(&q->dev_counters, size_t(n_jobs + 1) * 4) != cudaSuccess ||
        cudaMemset(q->dev_counters, 0, size_t(n_jobs + 1) * 4) != cudaSuccess ||
        cudaMalloc(&q->dev_pub, size_t(std::max<int64_t>(pub_words, 4)) * 4) != cudaSuccess ||
        cudaMemset(q->dev_pub, 0, size_t(std::max<int64_t>(pub_words, 4)) * 4) != cudaSuccess) {
        g_last_cuda_error = cudaGetLastError();
        cudaFree(q->dev_jobs);
        cudaFree(q->dev_counters);
        cudaFree(q->dev_pub);
        delete q;
        return QGEMV_ERR_CUDA;
    }
    if (h->sequences) h->sequences->push_back(q);
    h->tp_seq_cursor -= xchg_elems;
    *out = q;
    return QGEMV_OK;
}

int qgemv_sequence_destroy(qgemv_handle* h, qgemv_sequence* q) {
    if (!h || !q) return QGEMV_ERR_INVALID_ARG;
    cudaSetDevice(h->cfg.device);
    if (h->sequences) h->sequences->erase(std::remove(h->sequences->begin(), h->sequences->end(), q), h->sequences->end());
    if (q->xchg_elems > 0 && q->xchg_first == h->tp_seq_cursor) h->tp_seq_cursor += q->xchg_elems;  // the latest list: its blocks are free again
    cudaFree(q->dev_jobs);
    cudaFree(q->dev_counters);
    cudaFree(q->dev_pub);
    delete q;
    return QGEMV_OK;
}

int qgemv_sequence_run(qgemv_handle* h, const qgemv_sequence* q, void* stream) {
    if (!h || !q) return QGEMV_ERR_INVALID_ARG;
    qg::SeqParams P;
    std::memset(&P, 0, sizeof P);
    P.jobs = q->dev_jobs;
    P.ws = h->seq_parts;
    P.barrier = h->seq_barrier;
    P.fin = q->dev_counters;
    P.pub = q->dev_pub;
    P.status = h->status_dev;
    P.spin_limit = default_spin(h);
    P.n_jobs = q->n_jobs;
    P.B = q->B;
    P.npad = q->npad;
    P.ring = q->ring;
    P.x_slots = q->x_slots;
    P.nbuf = q->nbuf;
    P.debug = h->cfg.debug;
    P.trace = h->tc_trace;
    P.trace_jobs = q->n_jobs;
    P.world = 1;
    if (q->xchg_elems > 0) {
        for (int r = 0; r < h->tp_world; ++r) P.xbuf[r] = h->tp_peer[r];
        P.x_max_elems = h->tp_max_elems;
        P.rank = h->tp_rank, P.world = h->tp_world;
    }
    const dim3 g(unsigned(q->grid)), blk(qg::kSeqThreads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    g_launch_cooperative = true;
    cudaError_t err;
    if (q->fused) {
        err = q->stage_items == 2   ? launch(h, qg::gemv_seq_kernel<2, qg::kSeqFuse>, g, blk, q->smem, st, P)
              : q->stage_items == 4 ? launch(h, qg::gemv_seq_kernel<4, qg::kSeqFuse>, g, blk, q->smem, st, P)
                                    : launch(h, qg::gemv_seq_kernel<8, qg::kSeqFuse>, g, blk, q->smem, st, P);
    } else {
        err = q->stage_items == 2   ? launch(h, qg::gemv_seq_kernel<2, qg::kSeqPlain>, g, blk, q->smem, st, P)
              : q->stage_items == 4 ? launch(h, qg::gemv_seq_kernel<4, qg::kSeqPlain>, g, blk, q->smem, st, P)
                                    : launch(h, qg::gemv_seq_kernel<8, qg::kSeqPlain>, g, blk, q->smem, st, P);
    }
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}

int qgemv_gemv(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int B, void* y,
               int y_dtype, void* stream) {
    return qgemv_gemv_prefetch(h, w, x_bf16, B, y, y_dtype, nullptr, stream);
}

int qgemv_gemv_prefetch(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int B, void* y,
                        int y_dtype, const qgemv_weight* next, void* stream) {
    if (!h || !w || !x_bf16 || !y) return QGEMV_ERR_INVALID_ARG;
    if (B < 1 || B > QGEMV_MAX_ROWS) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (y_dtype != QGEMV_OUT_BF16 && y_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0) return QGEMV_ERR_INVALID_ARG;
    if (w->fmt == QGEMV_FMT_NVFP4_TC && B <= QGEMV_MAX_BATCH)
        return gemv_tc(h, w, x_bf16, B, y, y_dtype, next, static_cast<cudaStream_t>(stream));
    if (B > QGEMV_MAX_BATCH) {
        // two launches: rows 0..7, then the rest (the second one names the next matrix)
        if ((w->K * 2 * QGEMV_MAX_BATCH) % 16 != 0) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        const int rc = qgemv_gemv_prefetch(h, w, x_bf16, QGEMV_MAX_BATCH, y, y_dtype, nullptr, stream);
        if (rc != QGEMV_OK) return rc;
        const size_t ye = y_dtype == QGEMV_OUT_F32 ? 4 : 2;
        return qgemv_gemv_prefetch(h, w, static_cast<const uint16_t*>(x_bf16) + int64_t(QGEMV_MAX_BATCH) * w->K,
                                   B - QGEMV_MAX_BATCH, static_cast<uint8_t*>(y) + size_t(QGEMV_MAX_BATCH) * w->N * ye,
                                   y_dtype, next, stream);
    }
    qg::GemvParams P = base_params(h, w);
    P.x = static_cast<const uint16_t*>(x_bf16);
    P.y = y;
    P.B = B;
    P.y_dtype = y_dtype;
    P.prob = nullptr;
    const uint8_t* pf_base = next ? next->dev_blob + QG_HEADER_BYTES + next->aux_bytes : nullptr;
    const uint64_t pf_bytes = next ? next->payload_bytes : 0;
    // Activations too large to stage at once (units * B > 512) on a matrix with at least a panel per
    // CTA: multiply in K chunks, one launch of the whole-panel streaming kernel each into its own
    // fp32 slice of the handle's scratch, then add the slices in chunk order and round once.  The
    // chunk length depends on B, so here a row's result matches other batch sizes to fp32 rounding,
    // not bit for bit.  Calls that share a handle share the scratch: keep them on one stream.
    const int unit_bytes = w->fmt == QGEMV_FMT_NVFP4 ? QG_NVFP4_UNIT_BYTES : QG_FP8_UNIT_BYTES;
    if (!qg::use_stream_path(true, B, w->units) && w->n_stack == 1 && wp_has_enough_panels(h, w) &&
        !(h->cfg.debug & (256 | 512))) {
        const int64_t cu = (qg::kSMaxUnitsTimesBatch / B) / QG_PHASE_UNITS * QG_PHASE_UNITS;  // units per chunk
        const int64_t n_chunks = (w->units + cu - 1) / cu;
        const int64_t slice = int64_t(B) * w->N;
        if (size_t(n_chunks * slice) * sizeof(float) <= kChunkWsBytes) {
            cudaStream_t st = static_cast<cudaStream_t>(stream);
            for (int64_t c = 0; c < n_chunks; ++c) {
                qg::GemvParams Pc = P;
                const int64_t u0 = c * cu, u1 = std::min<int64_t>(w->units, u0 + cu);
                Pc.payload = P.payload + uint64_t(u0) * unit_bytes;
                Pc.payload_bytes = w->payload_bytes - uint64_t(u0) * unit_bytes;
                Pc.x = P.x + u0 * QG_UNIT_K;
                Pc.units = int32_t(u1 - u0);
                Pc.K = int32_t(std::min<int64_t>(w->K - u0 * QG_UNIT_K, (u1 - u0) * QG_UNIT_K));
                Pc.y = h->chunk_ws + c * slice;
                Pc.y_dtype = QGEMV_OUT_F32;
                if (c + 1 == n_chunks) Pc.pf_base = pf_base, Pc.pf_bytes = pf_bytes;
                const int rc = launch_gemv(h, w, Pc, st);
                if (rc != QGEMV_OK) return rc;
            }
            const cudaError_t err = launch(h, qg::chunk_sum_kernel, dim3(unsigned((slice + 255) / 256)), dim3(256), 0, st,
                                           static_cast<const float*>(h->chunk_ws), int(n_chunks), slice, y, y_dtype);
            return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
        }
    }
    P.pf_base = pf_base;
    P.pf_bytes = pf_bytes;
    return launch_gemv(h, w, P, static_cast<cudaStream_t>(stream));
}

// CTAs of a skinny GEMM.  With fewer row tiles than SMs every tile is cut into the same number of
// K parts (tiles * floor(SMs / tiles) CTAs): each CTA then has one segment and at most one
// partial tile.  Measured on the 70B shapes this beats spreading the runs evenly over all SMs
// (two or three segment boundaries per CTA, each draining the MMA pipeline and running the fp32
// fix-up): o 8192x8192 at 256 tokens 52.6 us on 128 CTAs against 66.2 us on 148.  Applied from 96
// tokens up.
static int gs_grid(int64_t sms, int64_t tiles, int64_t total_runs, int M) {
    // below ~100 tokens the GEMM is bound by the weight stream and wants every SM pulling
    int64_t g = (tiles <= sms && M >= 96) ? tiles * (sms / tiles) : sms;
    return int(std::min<int64_t>(g, total_runs));
}

int qgemv_gemm_skinny_plan(int fmt, int64_t N, int64_t K, int M, int sm_count, qgemv_skinny_plan* out) {
    if (!out || (fmt != QGEMV_FMT_NVFP4 && fmt != QGEMV_FMT_FP8) || sm_count < 1) return QGEMV_ERR_INVALID_ARG;
    if (M < 16 || M > qg::kGsMaxM || M % 16 != 0 || N < 128 || N % 128 != 0 || K < 64 || K % 64 != 0 ||
        N / 128 > kGsMaxTiles)
        return QGEMV_ERR_UNSUPPORTED_SHAPE;
    const int unit_bytes = fmt == QGEMV_FMT_NVFP4 ? QG_NVFP4_UNIT_BYTES : QG_FP8_UNIT_BYTES;
    const int64_t units = K / 64, tiles = N / 128;
    const int rl = units % 4 == 0 ? 2 : (units % 2 == 0 ? 1 : 0);
    const int xgl = qg::GsSmem::xg_log2(M, rl);
    const int64_t total = tiles * (units >> rl);
    out->run_units = 1 << rl;
    out->x_stage_units = 1 << xgl;
    out->x_stages = qg::GsSmem::x_stages(unit_bytes, M, xgl);
    out->p_stages = qg::GsSmem::p_stages(unit_bytes, M, xgl);
    out->a_stages = qg::GsSmem::a_stages(M, rl);
    out->tmem_columns = qg::GsSmem::tmem_columns(M, rl);
    out->smem_bytes = qg::GsSmem::total(unit_bytes, M, xgl);
    out->ctas = gs_grid(sm_count, tiles, total, M);
    out->scratch_bytes = int64_t(kGsMaxTiles) * 16 * 4 + int64_t(qg::kGsMaxM) * 8 + ((int64_t(M) * K * 2 + 255) / 256) * 256 +
                         int64_t(2) * out->ctas * M * 128 * 4;
    return QGEMV_OK;
}

namespace {
// scratch of the block-scaled prefill: activation items [kt][a4_item_bytes(M)] then fp32 row scales [256]
int a4_scratch(qgemv_handle* h, int M, int64_t kt, uint8_t** items, float** g) {
    const size_t items_bytes = (size_t(kt) * size_t(qg::a4_item_bytes(M)) + 255) / 256 * 256;
    const size_t need = items_bytes + 256 * sizeof(float);
    if (need > h->a4_ws_bytes) {
        // growing the scratch synchronises; it happens on the first call of a new largest shape
        // only and must not fall inside a stream capture
        QG_CUDA(cudaDeviceSynchronize());
        cudaFree(h->a4_ws);
        h->a4_ws = nullptr, h->a4_ws_bytes = 0;
        QG_CUDA(cudaMalloc(&h->a4_ws, need));
        h->a4_ws_bytes = need;
    }
    *items = h->a4_ws;
    *g = reinterpret_cast<float*>(h->a4_ws + h->a4_ws_bytes - 256 * sizeof(float));
    return QGEMV_OK;
}

// Y = Xq Wq^T with the activations quantised to NVFP4 by the stated quantiser (gemm_tc_a4.cuh).
int gemm_a4(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int M, void* y, int y_dtype, cudaStream_t st) {
    if (w->fmt != QGEMV_FMT_NVFP4_TC || w->n_stack != 1) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // weights consumed as stored
    if (w->K % 16 != 0) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    QG_CUDA(cudaSetDevice(h->cfg.device));
    const int64_t kt = w->units, tiles = w->n_panels / 8;
    uint8_t* items = nullptr;
    float* g = nullptr;
    const int rc = a4_scratch(h, M, kt, &items, &g);
    if (rc != QGEMV_OK) return rc;
    const int grid = std::min(gemv_grid(h), h->sm_count);
    // fewer row tiles than CTAs: cut K into chunks (fp32 partial results, added in chunk order)
    int n_chunk = 1;
    if (tiles < grid) {
        n_chunk = int(std::min<int64_t>({int64_t(grid) / tiles, 8, kt, int64_t(kChunkWsBytes / (size_t(M) * size_t(w->N) * 4))}));
        if (n_chunk < 1) n_chunk = 1;
    }
    const int chunk_items = int((kt + n_chunk - 1) / n_chunk);
    n_chunk = int((kt + chunk_items - 1) / chunk_items);
    // K blocks beyond the data must be zero codes with zero scales; with K a multiple of 64 the quantiser writes
    // every byte the MMAs read (scale rows of tokens beyond M are copied to tensor memory but never used)
    if (w->K % 64 != 0) QG_CUDA(cudaMemsetAsync(items, 0, size_t(kt) * size_t(qg::a4_item_bytes(M)), st));
    qg::A4QuantParams Q;
    Q.x = static_cast<const uint16_t*>(x_bf16);
    Q.M = M, Q.K = int32_t(w->K);
    Q.items = items, Q.g = g, Q.codes = nullptr, Q.scales = nullptr;
    if (launch(h, qg::a4_quant_kernel, dim3(unsigned(M)), dim3(256), 0, st, Q) != cudaSuccess) return QGEMV_ERR_CUDA;
    qg::A4Params P;
    std::memset(&P, 0, sizeof P);
    P.payload = w->dev_blob + QG_HEADER_BYTES + w->aux_bytes;
    P.xq = items;
    P.g = g;
    P.y = n_chunk == 1 ? y : static_cast<void*>(h->chunk_ws);
    P.status = h->status_dev;
    P.spin_limit = default_spin(h);
    P.tensor_scale = w->host_tensor_scale[0];
    P.N = int32_t(w->N), P.M = M;
    P.tiles = int32_t(tiles), P.kt = int32_t(kt);
    P.n_chunk = n_chunk, P.chunk_items = chunk_items;
    P.xq_item_bytes = qg::a4_item_bytes(M);
    const int cap = 227 * 1024;
    P.ring = std::min({qg::kA4MaxRing, (cap - qg::A4Smem::kRing) / qg::A4Smem::stage_bytes(M), qg::A4Smem::max_ring(M)});
    P.y_dtype = y_dtype;
    P.debug = h->cfg.debug;
    const size_t smem = size_t(qg::A4Smem::total(M, P.ring));
    static bool attr_set[64] = {};
    if (!attr_set[h->cfg.device & 63]) {
        QG_CUDA(cudaFuncSetAttribute(qg::gemm_a4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, cap));
        attr_set[h->cfg.device & 63] = true;
    }
    const int ctas = int(std::min<int64_t>(grid, tiles * n_chunk));
    if (launch(h, qg::gemm_a4_kernel, dim3(unsigned(ctas)), dim3(qg::kA4Threads), smem, st, P) != cudaSuccess) return QGEMV_ERR_CUDA;
    if (n_chunk > 1) {
        const int64_t slice = int64_t(M) * w->N;
        if (launch(h, qg::chunk_sum_kernel, dim3(unsigned((slice + 255) / 256)), dim3(256), 0, st,
                   static_cast<const float*>(h->chunk_ws), n_chunk, slice, y, y_dtype) != cudaSuccess)
            return QGEMV_ERR_CUDA;
    }
    return QGEMV_OK;
}
}  // namespace

int qgemv_quantize_a4(qgemv_handle* h, const void* x_bf16, int M, int64_t K, void* codes_dev, void* scales_dev,
                      float* row_scales_dev, void* stream) {
    if (!h || !x_bf16 || !codes_dev || !scales_dev || !row_scales_dev) return QGEMV_ERR_INVALID_ARG;
    if (M < 1 || K < 16 || K % 16 != 0 || K > INT32_MAX) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0 || (reinterpret_cast<uintptr_t>(codes_dev) & 7u) != 0) return QGEMV_ERR_INVALID_ARG;
    QG_CUDA(cudaSetDevice(h->cfg.device));
    qg::A4QuantParams Q;
    Q.x = static_cast<const uint16_t*>(x_bf16);
    Q.M = M, Q.K = int32_t(K);
    Q.items = nullptr, Q.g = row_scales_dev;
    Q.codes = static_cast<uint8_t*>(codes_dev), Q.scales = static_cast<uint8_t*>(scales_dev);
    return launch(h, qg::a4_quant_kernel, dim3(unsigned(M)), dim3(256), 0, static_cast<cudaStream_t>(stream), Q) == cudaSuccess
               ? QGEMV_OK
               : QGEMV_ERR_CUDA;
}

int qgemv_gemm_skinny(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int M, void* y,
                      int y_dtype, int act_mode, void* stream) {
    if (!h || !w || !x_bf16 || !y) return QGEMV_ERR_INVALID_ARG;
    if (act_mode == QGEMV_ACT_A4_BLOCKSCALED) {
        if (y_dtype != QGEMV_OUT_BF16 && y_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
        if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0) return QGEMV_ERR_INVALID_ARG;
        if (M < 16 || M > 256 || M % 16 != 0) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        return gemm_a4(h, w, x_bf16, M, y, y_dtype, static_cast<cudaStream_t>(stream));
    }
    if (act_mode != QGEMV_ACT_A16_EXACT) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (y_dtype != QGEMV_OUT_BF16 && y_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0) return QGEMV_ERR_INVALID_ARG;
    if (M < 16 || M > qg::kGsMaxM || M % 16 != 0) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (w->n_stack != 1 || w->N % 128 != 0 || w->K % 64 != 0) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (w->fmt == QGEMV_FMT_NVFP4_TC) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // wants the lane-ordered layout
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QG_CUDA(cudaSetDevice(h->cfg.device));
    const int tiles = int(w->N / 128);
    if (tiles > kGsMaxTiles) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    const int run_log2 = w->units % 4 == 0 ? 2 : (w->units % 2 == 0 ? 1 : 0);
    const int64_t total = int64_t(tiles) * (w->units >> run_log2);  // work items: runs of units
    const int grid = gs_grid(gemv_grid(h), tiles, total, M);
    // scratch: [tile counters, fixed place][row exponents][f16 activation tiles][partial tiles]
    const size_t cnt_bytes = size_t(kGsMaxTiles) * 16 * sizeof(int32_t);
    const size_t exp_bytes = size_t(qg::kGsMaxM) * 8;  // row exponents, then row maxima (zero between calls)
    const size_t xt_bytes = ((size_t(M) * size_t(w->K) * 2 + 255) / 256) * 256;
    const size_t ws_bytes = size_t(2) * grid * size_t(M) * 128 * sizeof(float);
    const size_t need = cnt_bytes + exp_bytes + xt_bytes + ws_bytes;
    if (need > h->gs_ws_bytes) {
        // growing the scratch synchronises; it happens on the first call of a new largest shape
        // only and must not fall inside a stream capture
        QG_CUDA(cudaDeviceSynchronize());
        cudaFree(h->gs_ws);
        h->gs_ws = nullptr, h->gs_ws_bytes = 0;
        QG_CUDA(cudaMalloc(&h->gs_ws, need));
        QG_CUDA(cudaMemset(h->gs_ws, 0, cnt_bytes + exp_bytes));
        h->gs_ws_bytes = need;
    }
    int32_t* counters = reinterpret_cast<int32_t*>(h->gs_ws);
    int32_t* xexp = reinterpret_cast<int32_t*>(h->gs_ws + cnt_bytes);
    uint8_t* xt = h->gs_ws + cnt_bytes + exp_bytes;
    float* ws = reinterpret_cast<float*>(xt + xt_bytes);
    unsigned int* rowmax = reinterpret_cast<unsigned int*>(xexp + qg::kGsMaxM);
    const dim3 pgrid(unsigned((w->K + qg::kXPrepThreads * 8 - 1) / (qg::kXPrepThreads * 8)), unsigned(M));
    if (launch(h, qg::x_rowmax_kernel, pgrid, dim3(qg::kXPrepThreads), 0, st, static_cast<const uint16_t*>(x_bf16),
               int(w->K), rowmax) != cudaSuccess ||
        launch(h, qg::x_prep_kernel, pgrid, dim3(qg::kXPrepThreads), 0, st, static_cast<const uint16_t*>(x_bf16), M,
               int(w->K), static_cast<const unsigned int*>(rowmax), xt, xexp) != cudaSuccess)
        return QGEMV_ERR_CUDA;
    const int unit_bytes = w->fmt == QGEMV_FMT_NVFP4 ? QG_NVFP4_UNIT_BYTES : QG_FP8_UNIT_BYTES;
    qg::GsParams P;
    std::memset(&P, 0, sizeof P);
    P.payload = w->dev_blob + QG_HEADER_BYTES + w->aux_bytes;
    P.chan_scale = reinterpret_cast<const float*>(w->dev_blob + QG_HEADER_BYTES);
    P.tensor_scale = w->host_tensor_scale[0];
    P.xt = xt;
    P.xexp = xexp;
    P.rowmax = rowmax;
    P.y = y;
    P.ws = ws;
    P.counters = counters;
    P.y_dtype = y_dtype;
    P.N = int32_t(w->N), P.K = int32_t(w->K), P.M = M;
    P.units = int32_t(w->units);
    P.tiles = tiles;
    P.run_log2 = run_log2;
    P.xg_log2 = qg::GsSmem::xg_log2(M, run_log2);
    P.x_stages = qg::GsSmem::x_stages(unit_bytes, M, P.xg_log2);
    P.p_stages = qg::GsSmem::p_stages(unit_bytes, M, P.xg_log2);
    P.status = h->status_dev;
    P.spin_limit = default_spin(h);
    P.debug = h->cfg.debug;
    const size_t smem = size_t(qg::GsSmem::total(unit_bytes, M, P.xg_log2));
    const dim3 g(static_cast<unsigned>(grid)), block(qg::kGsThreads);
    const cudaError_t err = w->fmt == QGEMV_FMT_NVFP4
                                ? launch(h, qg::gemm_skinny_kernel<QGEMV_FMT_NVFP4>, g, block, smem, st, P)
                                : launch(h, qg::gemm_skinny_kernel<QGEMV_FMT_FP8>, g, block, smem, st, P);
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}

int qgemv_moe_plan(int64_t K, int64_t K2, int n_experts, int T, int topk, int ctas, int smem_kb, qgemv_moe_plan_t* out) {
    if (!out || K < 64 || K % 64 != 0 || K2 < 0 || K2 % 64 != 0 || n_experts < 1 || T < 1 || topk < 1 || ctas < 1)
        return QGEMV_ERR_INVALID_ARG;
    const int64_t slots = int64_t(T) * topk;
    if (n_experts > qg::kMoeMaxExperts || slots > qg::kMoeMaxSlots) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    // Rows per problem (B): no more than there are tokens, and as many of eight as leave a weight ring of three
    // stages beside the digit planes of B rows x K (halved until they do: a long K gets problems of fewer
    // rows, and an expert with more entries is then read once per problem).
    constexpr int kStage = 4;
    constexpr int kWalk = (qg::kMoeSmemBytes + 127) / 128 * 128;   // the CTA's problem table, behind the ring
    const int cap = (smem_kb > 0 ? std::min(smem_kb, 227) : 227) * 1024 - kWalk;
    const int x_slots = int(std::max(K, K2) / 64);   // a CTA's share of an expert may span a whole row tile
    int B = std::min(QGEMV_MAX_BATCH, T), npad = 0, nbuf = 1, ring = 0;
    for (;; B = (B + 1) / 2) {
        npad = (8 * B + 15) / 16 * 16;
        // two plane buffers (a CTA's range mostly touches two experts) when that leaves a ring of four stages
        for (nbuf = 2; nbuf >= 1; --nbuf) {
            const int base = qg::SeqSmem::ring_off(x_slots, npad, nbuf);
            ring = (cap - base) / (kStage * qg::kTcItemBytes);
            ring = std::min({ring, qg::kTcMaxRing, qg::SeqSmem::max_ring_items(npad) / kStage});
            if (ring >= 4 || nbuf == 1) break;
        }
        if (ring >= 3 || B == 1) break;
    }
    if (ring < 2 || ring * kStage * qg::kTcItemBytes < qg::kMoeWalkBytes)
        return QGEMV_ERR_UNSUPPORTED_SHAPE;  // K too long for the digit planes of one row beside a ring
    const int64_t most_prob = std::min<int64_t>(n_experts, slots) + slots / B;   // problems the lists can make
    if (((most_prob + ctas - 1) / ctas + 1) * (K2 > 0 ? 2 : 1) > qg::kMoeLocalJobs || most_prob >= 2048) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    out->rows_per_problem = B;
    out->plane_buffers = nbuf;
    out->plane_slots = x_slots;
    out->ring_stages = ring;
    out->stage_items = kStage;
    out->max_problems = int32_t(most_prob);
    out->table_offset = (qg::SeqSmem::total(x_slots, npad, nbuf, ring, kStage) + 127) / 128 * 128;
    out->smem_bytes = out->table_offset + kWalk;
    return QGEMV_OK;
}

namespace {
// The experts of a router table on the tensor-core layout: the sequence kernel in its expert-list mode, ONE
// cooperative launch (every CTA walks the top-k lists for itself).  Problems hold at most B activation rows.
// `w2` (nullable): the experts' second stage in the same launch -- w is then the gate/up stage, writing its bf16
// rows to `mid` [T * topk][w->N], and w2 the down stage, which reads them through silu(gate) * up.
int moe_tc(qgemv_handle* h, const qgemv_weight* w, const qgemv_weight* w2, const int32_t* expert_ids, const void* x_bf16,
           int T, int topk, int per_slot_input, int x_act, void* mid, void* out, int out_dtype, cudaStream_t s) {
    const int grid = gemv_grid(h);
    if (grid > h->sm_count) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // the CTAs wait on one another: one per SM at most
    const int slots = T * topk;
    qgemv_moe_plan_t pl;
    const int rcp = qgemv_moe_plan(w->K, w2 ? w2->K : 0, w->n_stack, T, topk, grid, h->cfg.tc_smem_kb, &pl);
    if (rcp != QGEMV_OK) return rcp;
    const int B = pl.rows_per_problem, npad = (8 * B + 15) / 16 * 16, nbuf = pl.plane_buffers, ring = pl.ring_stages;
    const int x_slots = pl.plane_slots;
    const int64_t most_prob = pl.max_problems;
    constexpr int kStage = 4;
    qg::SeqParams P;
    std::memset(&P, 0, sizeof P);
    qg::SeqJob& mj = P.moe_job;
    mj.payload = w->dev_blob + QG_HEADER_BYTES + w->aux_bytes;
    mj.x = static_cast<const uint16_t*>(x_bf16);
    mj.y = out;
    mj.tensor_scale = 1.0f;
    mj.N = int32_t(w->N), mj.K = int32_t(w->K);
    mj.tiles = int32_t(w->n_panels / 8), mj.kt = int32_t(w->units);
    mj.x_stride = int32_t(x_act == QGEMV_MOE_X_SILU_MUL ? 2 * w->K : w->K);
    mj.act = x_act == QGEMV_MOE_X_SILU_MUL ? 1 : 0;
    mj.y_dtype = out_dtype;
    mj.dep = -1, mj.xoff = -1, mj.pub_off = -1, mj.src_off = -1, mj.src_job = -1;
    const int64_t per = int64_t(mj.tiles) * mj.kt;
    if ((most_prob * per + 1) * grid >= (int64_t(1) << 32)) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // 32-bit split arithmetic
    P.n_phases = 1;
    if (w2) {
        mj.y = mid, mj.y_dtype = QGEMV_OUT_BF16;
        qg::SeqJob& m2 = P.moe_job2;
        m2 = mj;
        m2.payload = w2->dev_blob + QG_HEADER_BYTES + w2->aux_bytes;
        m2.x = static_cast<const uint16_t*>(mid);
        m2.y = out, m2.y_dtype = out_dtype;
        m2.N = int32_t(w2->N), m2.K = int32_t(w2->K);
        m2.tiles = int32_t(w2->n_panels / 8), m2.kt = int32_t(w2->units);
        m2.x_stride = int32_t(w->N);
        m2.act = 1;
        const int64_t per2 = int64_t(m2.tiles) * m2.kt;
        if ((most_prob * per2 + 1) * grid >= (int64_t(1) << 32)) return QGEMV_ERR_UNSUPPORTED_SHAPE;
        P.n_phases = 2;
        P.expert_ts2 = w2->dev_tensor_scale;
        P.expert_stride2 = w2->blob_bytes;
        P.moe_cnt = h->moe_cnt;
    }
    P.ws = h->seq_parts;
    P.barrier = h->seq_barrier;
    P.fin = reinterpret_cast<unsigned int*>(w->counters);  // [0]: launches with this weight (nothing else of a job list's counters is used)
    P.status = h->status_dev;
    P.spin_limit = default_spin(h);
    P.n_jobs = 0;
    P.B = B;
    P.npad = npad;
    P.x_slots = x_slots;
    P.nbuf = nbuf;
    P.debug = h->cfg.debug;
    P.trace = h->tc_trace;
    P.trace_jobs = qg::kMoeLocalJobs;
    P.world = 1;
    P.ids = expert_ids;
    P.slots = slots, P.topk = topk, P.n_experts = w->n_stack, P.per_slot = per_slot_input ? 1 : 0;
    P.expert_ts = w->dev_tensor_scale;
    P.expert_stride = w->blob_bytes;
    P.ring = ring;
    P.moe_smem = pl.table_offset;
    const size_t smem = size_t(pl.smem_bytes);
    g_launch_cooperative = (h->cfg.debug & 2048) != 0;
    const cudaError_t err = launch(h, qg::gemv_seq_kernel<kStage, qg::kSeqMoe>, dim3(unsigned(grid)), dim3(qg::kSeqThreads), smem, s, P);
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}
}  // namespace

int qgemv_moe_gemv(qgemv_handle* h, const qgemv_weight* experts, const int32_t* expert_ids,
                   const void* x_bf16, int T, int topk, int per_slot_input, void* out,
                   int out_dtype, void* stream) {
    return qgemv_moe_gemv_act(h, experts, expert_ids, x_bf16, T, topk, per_slot_input, 0, out, out_dtype, stream);
}

int qgemv_moe_gemv_act(qgemv_handle* h, const qgemv_weight* experts, const int32_t* expert_ids,
                       const void* x_bf16, int T, int topk, int per_slot_input, int x_act, void* out,
                       int out_dtype, void* stream) {
    if (!h || !experts || !expert_ids || !x_bf16 || !out) return QGEMV_ERR_INVALID_ARG;
    if (x_act != 0 && x_act != QGEMV_MOE_X_SILU_MUL) return QGEMV_ERR_INVALID_ARG;
    if (x_act != 0 && experts->fmt != QGEMV_FMT_NVFP4_TC) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // the expert-list launch only
    if (!experts->prob) return QGEMV_ERR_INVALID_ARG;  // not a stacked weight
    if (T < 1 || topk < 1 || int64_t(T) * topk > kMaxMoeSlots) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (out_dtype != QGEMV_OUT_BF16 && out_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0) return QGEMV_ERR_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (experts->fmt == QGEMV_FMT_NVFP4_TC) return moe_tc(h, experts, nullptr, expert_ids, x_bf16, T, topk, per_slot_input, x_act, nullptr, out, out_dtype, s);
    const int threads = 1024;
    cudaError_t err = launch(h, qg::moe_prep_kernel, dim3(1), dim3(threads),
                             size_t(experts->n_stack) * 12 + size_t(T) * topk * 4 + 16, s, expert_ids, T, topk, experts->n_stack,
                             per_slot_input, experts->max_prob, experts->prob, h->status_dev);
    if (err != cudaSuccess) return QGEMV_ERR_CUDA;
    qg::GemvParams P = base_params(h, experts);
    P.x = static_cast<const uint16_t*>(x_bf16);
    P.y = out;
    P.B = 0;
    P.y_dtype = out_dtype;
    P.prob = experts->prob;
    const dim3 grid(gemv_grid(h)), block(qg::kSThreads);
    auto launch_stream = [&](const qg::GemvParams& Q) {
        return experts->fmt == QGEMV_FMT_NVFP4
                   ? launch(h, qg::moe_stream_kernel<QGEMV_FMT_NVFP4>, grid, block, qg::MSmem::total<QGEMV_FMT_NVFP4>(), s, Q)
                   : launch(h, qg::moe_stream_kernel<QGEMV_FMT_FP8>, grid, block, qg::MSmem::total<QGEMV_FMT_FP8>(), s, Q);
    };
    if (h->cfg.debug & 256) return launch_gemv(h, experts, P, s);
    if (qg::use_moe_stream_path(experts->units)) return launch_stream(P) == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
    // Experts with K > 2048: one launch of the streaming kernel per K chunk of 32 units, each into its
    // own fp32 slice [T*topk][N] of the handle's scratch, then the slices are added in chunk order.
    const int unit_bytes = experts->fmt == QGEMV_FMT_NVFP4 ? QG_NVFP4_UNIT_BYTES : QG_FP8_UNIT_BYTES;
    const int64_t cu = 32, n_chunks = (experts->units + cu - 1) / cu;
    const int64_t slice = int64_t(T) * topk * experts->N;
    if (size_t(n_chunks * slice) * sizeof(float) > kChunkWsBytes) return launch_gemv(h, experts, P, s);
    for (int64_t c = 0; c < n_chunks; ++c) {
        qg::GemvParams Pc = P;
        const int64_t u0 = c * cu, u1 = std::min<int64_t>(experts->units, u0 + cu);
        Pc.payload = P.payload + uint64_t(u0) * unit_bytes;
        Pc.payload_bytes = experts->payload_bytes - uint64_t(u0) * unit_bytes;
        Pc.x = P.x + u0 * QG_UNIT_K;
        Pc.units = int32_t(u1 - u0);
        Pc.K = int32_t(std::min<int64_t>(experts->K - u0 * QG_UNIT_K, (u1 - u0) * QG_UNIT_K));
        Pc.y = h->chunk_ws + c * slice;
        Pc.y_dtype = QGEMV_OUT_F32;
        if (launch_stream(Pc) != cudaSuccess) return QGEMV_ERR_CUDA;
    }
    err = launch(h, qg::chunk_sum_kernel, dim3(unsigned((slice + 255) / 256)), dim3(256), 0, s,
                 static_cast<const float*>(h->chunk_ws), int(n_chunks), slice, out, out_dtype);
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}

int qgemv_moe_mlp(qgemv_handle* h, const qgemv_weight* gate_up, const qgemv_weight* down, const int32_t* expert_ids,
                  const void* x_bf16, int T, int topk, void* gate_up_rows, void* out, int out_dtype, void* stream) {
    if (!h || !gate_up || !down || !expert_ids || !x_bf16 || !gate_up_rows || !out) return QGEMV_ERR_INVALID_ARG;
    if (T < 1 || topk < 1 || int64_t(T) * topk > kMaxMoeSlots) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (out_dtype != QGEMV_OUT_BF16 && out_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
    if (((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(gate_up_rows)) & 15u) != 0) return QGEMV_ERR_INVALID_ARG;
    if (gate_up->fmt != QGEMV_FMT_NVFP4_TC || down->fmt != QGEMV_FMT_NVFP4_TC) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (gate_up->n_stack != down->n_stack || gate_up->N != 2 * down->K) return QGEMV_ERR_INVALID_ARG;
    return moe_tc(h, gate_up, down, expert_ids, x_bf16, T, topk, 0, 0, gate_up_rows, out, out_dtype, static_cast<cudaStream_t>(stream));
}

int qgemv_moe_combine(qgemv_handle* h, const void* slot_out, int slot_dtype, const float* expert_w,
                      int T, int topk, int64_t N, void* y, int y_dtype, void* stream) {
    if (!h || !slot_out || !expert_w || !y || T < 1 || topk < 1 || N < 1) return QGEMV_ERR_INVALID_ARG;
    const int64_t total = int64_t(T) * N;
    const int threads = 256;
    const unsigned blocks = unsigned((total + threads - 1) / threads);
    cudaError_t err = launch(h, qg::moe_combine_kernel, dim3(blocks), dim3(threads), 0,
                             static_cast<cudaStream_t>(stream), slot_out, slot_dtype, expert_w, T,
                             topk, N, y, y_dtype);
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}

int qgemv_dequant_f32(qgemv_handle* h, const qgemv_weight* w, int which, float* out_dev,
                      void* stream) {
    if (!h || !w || !out_dev || which < 0 || which >= w->n_stack) return QGEMV_ERR_INVALID_ARG;
    const uint8_t* blob = w->dev_blob + uint64_t(which) * w->blob_bytes;
    const uint8_t* payload = blob + QG_HEADER_BYTES + w->aux_bytes;
    const float* chan = reinterpret_cast<const float*>(blob + QG_HEADER_BYTES);
    const float ts = w->fmt == QGEMV_FMT_NVFP4 ? w->host_tensor_scale[which] : 1.0f;
    const int64_t warps = w->n_panels * w->units;
    const int threads = 128;
    const unsigned blocks = unsigned((warps * 32 + threads - 1) / threads);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (w->fmt == QGEMV_FMT_NVFP4_TC) {
        const int64_t n_threads = w->N * (w->K / 16);
        qg::dequant_tc_kernel<<<unsigned((n_threads + 255) / 256), 256, 0, s>>>(payload, w->host_tensor_scale[which], int32_t(w->N),
                                                                                int32_t(w->K), int32_t(w->units), out_dev);
        return cudaGetLastError() == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
    }
    if (w->fmt == QGEMV_FMT_NVFP4) {
        qg::dequant_kernel<QGEMV_FMT_NVFP4><<<blocks, threads, 0, s>>>(payload, chan, ts, int32_t(w->N),
                                                                      int32_t(w->K), int32_t(w->units), out_dev);
    } else {
        qg::dequant_kernel<QGEMV_FMT_FP8><<<blocks, threads, 0, s>>>(payload, chan, ts, int32_t(w->N),
                                                                    int32_t(w->K), int32_t(w->units), out_dev);
    }
    return cudaGetLastError() == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}

int qgemv_last_device_status(qgemv_handle* h, void* stream, qgemv_dev_status* out) {
    if (!h || !out) return QGEMV_ERR_INVALID_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    QG_CUDA(cudaStreamSynchronize(s));
    int32_t v[4];
    QG_CUDA(cudaMemcpy(v, h->status_dev, sizeof v, cudaMemcpyDeviceToHost));
    out->code = v[0];
    out->where = v[1];
    out->block = v[2];
    out->extra = v[3];
    if (v[0] != 0) {
        QG_CUDA(cudaMemset(h->status_dev, 0, sizeof v));
        // a kernel that gave up may have left hand-over flags and the arrival counter behind
        QG_CUDA(cudaMemset(h->tc_ws, 0, h->tc_ws_bytes));
        QG_CUDA(cudaMemset(h->moe_cnt, 0, 2048 * 4));
        // ... and tagged words under the tags of a launch that never counted itself: count it here
        unsigned int cnt[3];
        QG_CUDA(cudaMemcpy(cnt, h->seq_barrier, sizeof cnt, cudaMemcpyDeviceToHost));
        cnt[0] = 0u, cnt[2] += 1u;
        QG_CUDA(cudaMemcpy(h->seq_barrier, cnt, sizeof cnt, cudaMemcpyHostToDevice));
        if (h->sequences) {
            for (qgemv_sequence* q : *h->sequences) {
                unsigned int run = 0;
                QG_CUDA(cudaMemcpy(&run, q->dev_counters + q->n_jobs, 4, cudaMemcpyDeviceToHost));
                run += 1u;
                QG_CUDA(cudaMemset(q->dev_counters, 0, size_t(q->n_jobs) * 4));
                QG_CUDA(cudaMemcpy(q->dev_counters + q->n_jobs, &run, 4, cudaMemcpyHostToDevice));
            }
        }
    }
    return QGEMV_OK;
}


// ---- tensor-parallel exchange over peer memory ------------------------------------------------
int qgemv_tp_create(qgemv_handle* h, int rank, int world, int64_t max_elems, void* ipc_handle_out) {
    if (!h || !ipc_handle_out || world < 1 || world > qg::kTpMaxWorld || rank < 0 || rank >= world)
        return QGEMV_ERR_INVALID_ARG;
    if (max_elems < 4 || max_elems > (int64_t(1) << 30) || h->tp_local) return QGEMV_ERR_INVALID_ARG;
    QG_CUDA(cudaSetDevice(h->cfg.device));
    max_elems = (max_elems + 3) / 4 * 4;
    const size_t bytes = qg::tp_buffer_bytes(world, max_elems);
    cudaIpcMemHandle_t mh;
    const bool ok = cudaMalloc(&h->tp_local, bytes) == cudaSuccess && cudaMemset(h->tp_local, 0, bytes) == cudaSuccess &&
                    cudaMalloc(&h->tp_epochs, 2 * 4) == cudaSuccess && cudaMemset(h->tp_epochs, 0, 2 * 4) == cudaSuccess &&
                    cudaDeviceSynchronize() == cudaSuccess && cudaIpcGetMemHandle(&mh, h->tp_local) == cudaSuccess;
    if (!ok) {
        // leave the handle as it was, so that the call can be retried
        g_last_cuda_error = cudaGetLastError();
        cudaFree(h->tp_local);
        cudaFree(h->tp_epochs);
        h->tp_local = nullptr, h->tp_epochs = nullptr;
        return QGEMV_ERR_CUDA;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == QGEMV_IPC_HANDLE_BYTES, "IPC handle size");
    std::memcpy(ipc_handle_out, &mh, sizeof mh);
    h->tp_rank = rank;
    h->tp_world = world;
    h->tp_max_elems = max_elems;
    h->tp_seq_cursor = max_elems;
    h->tp_call_high = 0;
    h->tp_peer[rank] = h->tp_local;
    return QGEMV_OK;
}

int qgemv_tp_connect(qgemv_handle* h, const void* all_handles) {
    if (!h || !all_handles || !h->tp_local) return QGEMV_ERR_INVALID_ARG;
    QG_CUDA(cudaSetDevice(h->cfg.device));
    const uint8_t* src = static_cast<const uint8_t*>(all_handles);
    for (int r = 0; r < h->tp_world; ++r) {
        if (r == h->tp_rank || h->tp_peer[r]) continue;
        cudaIpcMemHandle_t mh;
        std::memcpy(&mh, src + size_t(r) * QGEMV_IPC_HANDLE_BYTES, sizeof mh);
        void* p = nullptr;
        QG_CUDA(cudaIpcOpenMemHandle(&p, mh, cudaIpcMemLazyEnablePeerAccess));
        h->tp_peer[r] = static_cast<uint8_t*>(p);
        h->tp_ipc_opened[r] = true;
    }
    return QGEMV_OK;
}

int qgemv_tp_connect_ptrs(qgemv_handle* h, void* const* peer_buffers) {
    if (!h || !peer_buffers || !h->tp_local) return QGEMV_ERR_INVALID_ARG;
    for (int r = 0; r < h->tp_world; ++r) {
        if (r == h->tp_rank) continue;
        if (!peer_buffers[r] || h->tp_peer[r] || (reinterpret_cast<uintptr_t>(peer_buffers[r]) & 7u) != 0) return QGEMV_ERR_INVALID_ARG;
    }
    for (int r = 0; r < h->tp_world; ++r)
        if (r != h->tp_rank) h->tp_peer[r] = static_cast<uint8_t*>(peer_buffers[r]);
    return QGEMV_OK;
}

int qgemv_tp_buffer(qgemv_handle* h, void** dev_ptr, size_t* bytes) {
    if (!h || !dev_ptr || !bytes || !h->tp_local) return QGEMV_ERR_INVALID_ARG;
    *dev_ptr = h->tp_local;
    *bytes = qg::tp_buffer_bytes(h->tp_world, h->tp_max_elems);
    return QGEMV_OK;
}

namespace {
int tp_exchange(qgemv_handle* h, const void* in, void* y, int y_dtype, int64_t n, int gather, void* stream) {
    if (!h || !in || !y || n < 1) return QGEMV_ERR_INVALID_ARG;
    if (!h->tp_local) return QGEMV_ERR_INVALID_ARG;
    if (n > h->tp_seq_cursor) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // beyond the buffer, or into the part that job lists hold
    if (y_dtype != QGEMV_OUT_BF16 && y_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
    for (int r = 0; r < h->tp_world; ++r)
        if (!h->tp_peer[r]) return QGEMV_ERR_INVALID_ARG;  // qgemv_tp_connect has not run
    h->tp_call_high = std::max(h->tp_call_high, n);
    qg::TpParams P;
    std::memset(&P, 0, sizeof P);
    for (int r = 0; r < h->tp_world; ++r) P.buf[r] = h->tp_peer[r];
    P.rank = h->tp_rank;
    P.world = h->tp_world;
    P.max_elems = h->tp_max_elems;
    P.in = in;
    P.y = y;
    P.y_dtype = y_dtype;
    P.gather = gather;
    P.n = n;
    P.epoch = h->tp_epochs;
    P.status = h->status_dev;
    P.spin_limit = default_spin(h);
    const unsigned ctas = unsigned((n + qg::kTpThreads - 1) / qg::kTpThreads);
    const cudaError_t err = launch(h, qg::tp_exchange_kernel, dim3(ctas), dim3(qg::kTpThreads), 0,
                                   static_cast<cudaStream_t>(stream), P);
    return err == cudaSuccess ? QGEMV_OK : QGEMV_ERR_CUDA;
}
}  // namespace

int qgemv_tp_allreduce(qgemv_handle* h, void* y, int y_dtype, int64_t n, void* stream) {
    return tp_exchange(h, y, y, y_dtype, n, 0, stream);
}

int qgemv_tp_allgather(qgemv_handle* h, const void* shard, void* y, int y_dtype, int64_t n_shard, void* stream) {
    if (shard == y) return QGEMV_ERR_INVALID_ARG;
    return tp_exchange(h, shard, y, y_dtype, n_shard, 1, stream);
}

// ---- allocation-free GEMV ----------------------------------------------------------------------
// Some callers may not allocate device memory at the moment they need a projection: code running
// inside a memory pool that owns the whole device, a plugin that was handed its buffers by a host
// framework and must not touch the allocator, or a latency-critical path where a cudaMalloc would
// synchronise the device.  qgemv_gemv_noalloc serves them: weights, activations and outputs are the
// caller's buffers, and the kernel's own scratch (the partial-sum slots and arrival counters of
// panels that are split between CTAs, the device status word and the tensor scale) lives in the
// file-scope array below, which every GPU that loads this library holds until the process exits.
namespace {
constexpr int kNoAllocMaxCtas = 256;        // CTAs the scratch has partial-sum slots for
constexpr int kNoAllocMaxPanels = 16384;    // 16-row panels (N <= 262144) it has counters for
constexpr size_t kNoAllocWsBytes = size_t(2) * kNoAllocMaxCtas * 512;       // 256 KiB
constexpr size_t kNoAllocCounterBytes = size_t(kNoAllocMaxPanels) * 4;      // 64 KiB
constexpr size_t kNoAllocMiscBytes = 256;                                   // status word, tensor scale
constexpr size_t kNoAllocBytes = kNoAllocWsBytes + kNoAllocCounterBytes + kNoAllocMiscBytes;
constexpr int kNoAllocMaxDevices = 64;

struct NoAllocDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on that device
    int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
std::mutex g_noalloc_mutex;
}  // namespace

// Clears the arrival counters and the status word and stores the tensor scale ([16, 20) of `misc`).
static __global__ void noalloc_prepare_kernel(int32_t* counters, int32_t n_counters, int32_t* misc, float tensor_scale) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_counters) counters[i] = 0;
    if (i < 4) misc[i] = 0;
    if (i == 4) reinterpret_cast<float*>(misc)[4] = tensor_scale;
}

// In host code this name is only a stand-in for the symbol: the device address comes from
// cudaGetSymbolAddress, once per device, below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

int qgemv_gemv_noalloc(const void* dev_blob, const void* host_header, const void* x_bf16, int B, void* y,
                       int y_dtype, void* stream) {
    if (!dev_blob || !host_header || !x_bf16 || !y) return QGEMV_ERR_INVALID_ARG;
    if (B < 1 || B > QGEMV_MAX_BATCH) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    if (y_dtype != QGEMV_OUT_BF16 && y_dtype != QGEMV_OUT_F32) return QGEMV_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15u) != 0 || (reinterpret_cast<uintptr_t>(dev_blob) & 15u) != 0)
        return QGEMV_ERR_INVALID_ARG;
    qg_blob_header hd;
    std::memcpy(&hd, host_header, sizeof hd);
    if (hd.magic != QG_BLOB_MAGIC || hd.version != QG_BLOB_VERSION || hd.header_bytes != QG_HEADER_BYTES)
        return QGEMV_ERR_BAD_BLOB;
    if (hd.fmt != QGEMV_FMT_NVFP4 && hd.fmt != QGEMV_FMT_FP8) return QGEMV_ERR_BAD_BLOB;
    if (hd.N <= 0 || hd.K <= 0 || hd.K % 16 != 0 || hd.n_panels != (hd.N + 15) / 16 ||
        hd.units_per_panel != (hd.K + 63) / 64)
        return QGEMV_ERR_BAD_BLOB;
    // limits of the static scratch and of the schedule that uses it
    if (hd.n_panels > kNoAllocMaxPanels) return QGEMV_ERR_UNSUPPORTED_SHAPE;  // N above 262144 rows
    // ceil(K / 1024) * B above 32: the activations cannot be staged at once
    if (!qg::use_stream_path(true, B, hd.units_per_panel)) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    // aux_bytes, payload_bytes and unit_bytes are functions of (fmt, N, K): a header that disagrees is
    // stale or damaged, and its values would move the payload pointer
    const uint32_t unit_bytes = hd.fmt == QGEMV_FMT_NVFP4 ? QG_NVFP4_UNIT_BYTES : QG_FP8_UNIT_BYTES;
    const uint64_t aux_bytes = hd.fmt == QGEMV_FMT_FP8 ? (uint64_t(hd.n_panels) * 16 * 4 + 255) / 256 * 256 : 0;
    const uint64_t payload_bytes = uint64_t(hd.n_panels) * uint64_t(hd.units_per_panel) * unit_bytes;
    if (hd.unit_bytes != unit_bytes || hd.aux_bytes != aux_bytes || hd.payload_bytes != payload_bytes)
        return QGEMV_ERR_BAD_BLOB;

    int dev = 0;
    QG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kNoAllocMaxDevices) return QGEMV_ERR_INVALID_ARG;
    NoAllocDevice& nd = g_noalloc_dev[dev];
    {
        // First call on this device: resolve the scratch symbol and opt the kernels into their
        // shared-memory size.  This is set-up work, so it should happen before any stream capture.
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!nd.ready) {
            cudaDeviceProp prop;
            QG_CUDA(cudaGetDeviceProperties(&prop, dev));
            if (prop.major != 10) return QGEMV_ERR_NO_DEVICE;
            void* ptr = nullptr;
            QG_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
            const cudaFuncAttribute dyn = cudaFuncAttributeMaxDynamicSharedMemorySize;
            QG_CUDA(cudaFuncSetAttribute(qg::gemv_stream_kernel<QGEMV_FMT_NVFP4>, dyn, qg::SSmem::total<QGEMV_FMT_NVFP4>()));
            QG_CUDA(cudaFuncSetAttribute(qg::gemv_stream_kernel<QGEMV_FMT_FP8>, dyn, qg::SSmem::total<QGEMV_FMT_FP8>()));
            nd.scratch = static_cast<unsigned char*>(ptr);
            nd.sm_count = prop.multiProcessorCount;
            nd.ready = true;
        }
    }
    if (nd.sm_count > kNoAllocMaxCtas) return QGEMV_ERR_UNSUPPORTED_SHAPE;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char* ws = nd.scratch;
    unsigned char* counters = ws + kNoAllocWsBytes;
    unsigned char* misc = counters + kNoAllocCounterBytes;  // [0,16): status, [16,20): tensor scale
    // The array keeps the previous call's contents: counters and status must start at zero.  One small
    // kernel clears them and stores the tensor scale (passed by value: no host pointer outlives the call).
    noalloc_prepare_kernel<<<dim3(unsigned((hd.n_panels + 255) / 256)), dim3(256), 0, s>>>(
        reinterpret_cast<int32_t*>(counters), int32_t(hd.n_panels), reinterpret_cast<int32_t*>(misc), hd.tensor_scale);
    QG_CUDA(cudaGetLastError());

    qg::GemvParams P;
    std::memset(&P, 0, sizeof P);
    const uint8_t* blob = static_cast<const uint8_t*>(dev_blob);
    P.payload = blob + QG_HEADER_BYTES + aux_bytes;
    P.stack_stride = 0;
    P.chan_scale = reinterpret_cast<const float*>(blob + QG_HEADER_BYTES);
    P.chan_stride = 0;
    P.tensor_scale = reinterpret_cast<const float*>(misc + 16);
    P.x = static_cast<const uint16_t*>(x_bf16);
    P.y = y;
    P.ws = reinterpret_cast<float*>(ws);
    P.counters = reinterpret_cast<int32_t*>(counters);
    P.status = reinterpret_cast<int32_t*>(misc);
    P.prob = nullptr;
    P.spin_limit = int64_t(1) << 26;
    P.N = int32_t(hd.N);
    P.K = int32_t(hd.K);
    P.n_panels = int32_t(hd.n_panels);
    P.units = int32_t(hd.units_per_panel);
    P.unit_stride = P.units;
    P.x_stride = P.K;
    P.B = B;
    P.y_dtype = y_dtype;
    P.debug = 0;
    P.payload_bytes = payload_bytes;
    const dim3 grid(nd.sm_count), block(qg::kSThreads);
    if (hd.fmt == QGEMV_FMT_NVFP4) {
        qg::gemv_stream_kernel<QGEMV_FMT_NVFP4><<<grid, block, qg::SSmem::total<QGEMV_FMT_NVFP4>(), s>>>(P);
    } else {
        qg::gemv_stream_kernel<QGEMV_FMT_FP8><<<grid, block, qg::SSmem::total<QGEMV_FMT_FP8>(), s>>>(P);
    }
    QG_CUDA(cudaGetLastError());
    return QGEMV_OK;
}

int qgemv_noalloc_last_status(void* stream, qgemv_dev_status* out) {
    if (!out) return QGEMV_ERR_INVALID_ARG;
    int dev = 0;
    QG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kNoAllocMaxDevices) return QGEMV_ERR_INVALID_ARG;
    out->code = out->where = out->block = out->extra = 0;
    const NoAllocDevice& nd = g_noalloc_dev[dev];
    if (!nd.ready) return QGEMV_OK;  // no call has run on this device yet
    QG_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int32_t v[4];
    QG_CUDA(cudaMemcpy(v, nd.scratch + kNoAllocWsBytes + kNoAllocCounterBytes, sizeof v, cudaMemcpyDeviceToHost));
    out->code = v[0], out->where = v[1], out->block = v[2], out->extra = v[3];
    return QGEMV_OK;
}

}  // extern "C"
