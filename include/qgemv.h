/*
 * qgemv.h -- C ABI of the B200 (sm_100a) weight-only quantized GEMV library.
 *
 * The crit-hub registry holds no operator interface for this path: its engine
 * cards describe the projection kernels in prose and point at external
 * sources.  Each entry point below therefore cites the card text whose
 * described behaviour it provides.  Listed engines ship native code as an
 * nvcc-built shared object "behind a small C ABI"
 * (tools/fixtures/engines/crit-labs/mtp-adaptive-width/card.yaml:76,103); this
 * header is that boundary for the quantized projections.
 *
 * Conventions
 *   - Every call returns an int status (QGEMV_OK == 0, errors negative); nothing
 *     throws, aborts or exits across the boundary.
 *   - Plain pointers and sizes only.  `stream` is a cudaStream_t passed as void*.
 *   - The caller owns host blobs and all activation / output device buffers; the
 *     library owns handles, loaded weights and their device workspaces.
 *   - One handle per device.  Calls on one handle are serialised by the caller.
 *     gemv / moe / dequant calls are asynchronous on `stream`, allocate nothing,
 *     never synchronise the host, and may be captured into a CUDA graph.
 *   - There is no CPU fallback: compute entry points need a CUDA device.
 */
#ifndef QGEMV_H_
#define QGEMV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
enum {
    QGEMV_OK = 0,
    QGEMV_ERR_INVALID_ARG = -1,
    QGEMV_ERR_BAD_BLOB = -2,
    QGEMV_ERR_UNSUPPORTED_SHAPE = -3,
    QGEMV_ERR_CUDA = -4,
    QGEMV_ERR_NCCL = -5,
    QGEMV_ERR_TIMEOUT = -6,
    QGEMV_ERR_BOUNDS = -7,
    QGEMV_ERR_NO_DEVICE = -8
};

/* ---- weight formats ---------------------------------------------------------------------- */
enum {
    /* E2M1 codes, one E4M3 scale per 16 consecutive K elements, one fp32 per-tensor scale
     * ("NVFP4 E2M1 with E4M3 group scales",
     *  tools/fixtures/engines/crit-labs/mtp-adaptive-width/card.yaml:74). */
    QGEMV_FMT_NVFP4 = 1,
    /* E4M3 codes with one fp32 scale per output channel ("FP8 per-channel ... output head",
     *  tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:74). */
    QGEMV_FMT_FP8 = 2,
    /* The same values as QGEMV_FMT_NVFP4 (same canonical inputs, same dequantisation rule), stored
     * in the tile order that the block-scaled tensor-core instruction consumes as it is (E2M1
     * operands, one E4M3 scale per 16 K elements): the GEMV streams such a weight without
     * executing a single conversion instruction.  The engines' decode rows read "the stored NVFP4
     * ... matrices" (engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:77); this is the stored form for
     * the B200's native FP4 path.  Served by qgemv_gemv / qgemv_gemv_prefetch (all batch sizes)
     * and qgemv_dequant_f32; not by the MoE and skinny-GEMM entry points, which want
     * QGEMV_FMT_NVFP4. */
    QGEMV_FMT_NVFP4_TC = 3
};

enum { QGEMV_OUT_BF16 = 0, QGEMV_OUT_F32 = 1 };

#define QGEMV_MAX_BATCH 8 /* activation rows per kernel launch (decode batch / draft width) */
#define QGEMV_MAX_ROWS 16 /* activation rows per gemv call: 9..16 run as two launches (LM head at batch 16) */

typedef struct qgemv_handle qgemv_handle;
typedef struct qgemv_weight qgemv_weight;

typedef struct qgemv_config {
    int32_t device;        /* CUDA device ordinal */
    int32_t use_pdl;       /* 1: launch kernels with programmatic dependent launch so that a
                              kernel's weight prefetch overlaps the previous kernel's tail */
    int32_t grid_override; /* 0: one CTA per SM; >0: fixed CTA count (testing the K split) */
    int32_t debug;         /* bit 0: kernels bounds-check every staged address and report through
                              the device status word instead of touching memory;
                              bit 1: fault injection for tests -- the weight copies are never
                              issued, so the bounded waits must run out and report;
                              bit 8: schedule override for tests -- dense GEMV and MoE use the
                              general CTA-wide ring kernel instead of the per-warp streaming one;
                              bit 9: schedule override for tests -- the streaming kernel always
                              splits K across CTAs (partial sums + fixed-order fix-up);
                              bit 5: schedule override -- the tensor-core GEMV launches a
                              thread-block cluster per row tile for matrices with few tiles
                              (partial sums handed over in distributed shared memory instead of
                              global-memory slots) */
    int64_t spin_limit;    /* poll budget of every in-kernel wait; 0 = default */
    int32_t tc_stage_items; /* QGEMV_FMT_NVFP4_TC GEMV: 4608-byte items per bulk copy: 1, 2, 4 or 8; 0 = default (4) */
    int32_t tc_smem_kb;     /* ... shared memory per CTA the ring may grow to, in KiB; 0 = default
                               (about half an SM, so that the next kernel's CTA is resident and
                               prefetches its weights while this one streams) */
} qgemv_config;

/* Rows [n0,n1) and columns [k0,k1) of the canonical matrix: a tensor-parallel shard.
 * Column-parallel shards split N, row-parallel shards split K (k0, k1 multiples of 16). */
typedef struct qgemv_shard {
    int64_t n0, n1, k0, k1;
} qgemv_shard;

/* Last error a kernel reported (bounded wait ran out, debug bounds check failed). */
typedef struct qgemv_dev_status {
    int32_t code;  /* 0 or a QGEMV_ERR_* value */
    int32_t where; /* kernel-internal site id */
    int32_t block; /* CTA that reported */
    int32_t extra; /* site-specific detail (stage, item, index) */
} qgemv_dev_status;

/* ---- lifetime ---------------------------------------------------------------------------- */
int qgemv_init(const qgemv_config* cfg, qgemv_handle** out);
int qgemv_destroy(qgemv_handle* h);
const char* qgemv_status_string(int status);
/* Text of the last CUDA runtime error seen by the calling thread (after a QGEMV_ERR_CUDA). */
const char* qgemv_last_cuda_error(void);
/* Number of SMs of the handle's device (the CTA count the kernels are scheduled over). */
int qgemv_sm_count(const qgemv_handle* h);

/* ---- weight packer (pure host code, no GPU needed) ------------------------------------------
 * Canonical inputs ("weights as stored", engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:69,77):
 *   NVFP4: codes u8 [N][K/2] (low nibble = even k), scales u8 [N][K/16] (E4M3), tensor_scale.
 *   FP8:   codes u8 [N][K] (E4M3), scales = const float[N] per-output-channel scales;
 *          tensor_scale is ignored.
 * The blob interleaves codes and scales so that every lane of a warp issues one aligned
 * 128-bit load per 32 codes and a bulk copy of whole K ranges of a 16-row panel is contiguous.
 * K must be a multiple of 16; rows and K are zero-padded to the panel / unit size. */
size_t qgemv_packed_size(int fmt, int64_t N, int64_t K, const qgemv_shard* shard /* nullable */);
int qgemv_pack_host(int fmt, const void* codes, const void* scales, float tensor_scale, int64_t N,
                    int64_t K, const qgemv_shard* shard /* nullable */, void* blob_out);
/* The 256-byte header alone (checksum zero), for callers that lay the payload out themselves. */
int qgemv_pack_header(int fmt, float tensor_scale, int64_t N, int64_t K, const qgemv_shard* shard /* nullable */,
                      void* header_out);
/* Threads of the host packer's loops (launchers of one process per GPU often export
 * OMP_NUM_THREADS=1). */
int qgemv_set_host_threads(int n);
/* Inverse of qgemv_pack_host for the (possibly sharded) sub-matrix held by the blob.
 * scales_out is u8 [n][k/16] (NVFP4) or float [n] (FP8). */
int qgemv_unpack_host(const void* blob, size_t bytes, void* codes_out, void* scales_out,
                      float* tensor_scale_out);
/* QGEMV_OK when the header is consistent and the checksum over scales and codes matches. */
int qgemv_blob_verify(const void* blob, size_t bytes);
/* Shape of the matrix a blob holds. Any out pointer may be NULL. */
int qgemv_blob_info(const void* blob, size_t bytes, int* fmt, int64_t* N, int64_t* K);

/* ---- load / unload ---------------------------------------------------------------------------
 * Copies a packed blob to the device.  `n_stacked` > 1 loads that many equally shaped blobs laid
 * back to back in host memory as one stacked weight (the experts of an MoE layer). */
int qgemv_load(qgemv_handle* h, const void* host_blob, size_t bytes, qgemv_weight** out);
/* The same weight from CANONICAL NVFP4 arrays that are already in device memory (codes u8
 * [N][K/2], 8-byte aligned, and scales u8 [N][K/16], row-major): the layout is produced by a
 * kernel, byte for byte what qgemv_pack_host writes, so a checkpoint that was read straight into
 * device memory needs no host pass.  fmt: QGEMV_FMT_NVFP4_TC only (others:
 * QGEMV_ERR_UNSUPPORTED_SHAPE).  shard as in qgemv_pack_host.  Returns after the kernel has run on
 * `stream`; the inputs may be freed then.  No counterpart in the registry (its engines load
 * pre-quantised files through their own loaders, engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:69). */
int qgemv_load_device(qgemv_handle* h, int fmt, const void* codes_dev, const void* scales_dev, float tensor_scale,
                      int64_t N, int64_t K, const qgemv_shard* shard /* nullable */, void* stream, qgemv_weight** out);
int qgemv_load_stacked(qgemv_handle* h, const void* host_blobs, size_t bytes_each, int n_stacked,
                       qgemv_weight** out);
/* The experts of an MoE layer from canonical NVFP4 arrays in device memory: qgemv_load_device for
 * `n_stacked` equally shaped matrices into one stacked weight.  codes_dev / scales_dev: HOST arrays of
 * n_stacked device pointers (a checkpoint stores every expert as a tensor of its own); tensor_scales:
 * host fp32 [n_stacked].  The result is byte for byte what qgemv_load_stacked makes of the host-packed
 * blobs (zero checksums). */
int qgemv_load_stacked_device(qgemv_handle* h, int fmt, const void* const* codes_dev, const void* const* scales_dev,
                              const float* tensor_scales, int n_stacked, int64_t N, int64_t K,
                              const qgemv_shard* shard /* nullable */, void* stream, qgemv_weight** out);
int qgemv_unload(qgemv_handle* h, qgemv_weight* w);
/* Algorithmic weight bytes of one matrix: N*K*0.5625 + 4 (NVFP4) or N*K + 4*N (FP8). */
int64_t qgemv_weight_bytes(const qgemv_weight* w);
/* Copies the packed blob(s) of a loaded weight back to host memory; bytes must be n_stacked *
 * qgemv_packed_size(...).  (A weight made by qgemv_load_device carries a zero checksum.) */
int qgemv_weight_read(qgemv_handle* h, const qgemv_weight* w, void* host_out, size_t bytes);

/* ---- decode GEMV, batch 1..8 (up to 16 rows per call as two launches) -------------------------
 * y[b][n] = sum_k dequant(W)[n][k] * x[b][k], fp32 accumulation, output bf16 or fp32.
 * x: device bf16 [B][K] row-major; y: device [B][N] row-major.
 * The decode rows / decode-gemv of engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:77 and the
 * tensor-core NVFP4 GEMV of tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:76
 * ("hardware E2M1 conversion into mma.m16n8k16 ... one instruction stream for every column
 * count").  As there, row b of the result does not depend on B, and the split along K is fixed
 * by the shape and the CTA count, never by timing ("column invariant with a deterministic split
 * along K", tools/fixtures/engines/crit-labs/mtp-adaptive-width/card.yaml:77).  Exception: where
 * ceil(K / 1024) * B exceeds 32 (lane-ordered weights) or the digit planes of B * K activations leave no
 * room for a weight ring in shared memory (tensor-core layout), the call is split along K in chunks whose
 * length depends on B, and a row then matches other batch sizes to fp32 rounding only.  B = 9..16 (the output head at batch
 * 16, engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:77) streams the matrix twice: rows 0..7, then
 * the rest. */
int qgemv_gemv(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int B, void* y,
               int y_dtype, void* stream);
/* Same GEMV; additionally pulls the packed weight `next` (nullable) into L2 while this GEMV runs.
 * An engine knows the order of its projections ("one CUDA graph per round",
 * tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:75): naming the next matrix keeps HBM
 * busy across the launch boundary.  Weights are immutable, so the hint never changes a result. */
int qgemv_gemv_prefetch(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int B, void* y,
                        int y_dtype, const qgemv_weight* next, void* stream);

/* ---- a sequence of GEMVs as one launch --------------------------------------------------------
 * The projections of a decode step, in order, as ONE persistent kernel ("one CUDA graph per round",
 * tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:75, taken one step further: one launch).
 * Job i computes y_i = W_i x_i exactly as qgemv_gemv would (same split along K, same bits).
 * Ordering follows the data.  When the sequence is created the address ranges of every job's x and y
 * are compared with those of the jobs before it:
 *   - x_i is the bf16 output of ONE earlier job, or a column range of it (x_i points into that y,
 *     x_stride = that job's N when B > 1), and nothing else touches those buffers in between: the
 *     producer publishes its rows as it finishes them and job i converts them as they appear -- no
 *     grid-wide wait between the two jobs;
 *   - any other overlap (x_i over several outputs or an fp32 output, y_i over an earlier x or y):
 *     job i waits until the latest such job is complete on every CTA;
 *   - no overlap: job i may run alongside the tail of the jobs before it.
 * A caller whose dependency is not visible in the addresses sets QGEMV_JOB_AFTER_PREVIOUS on the job:
 * it then waits for the job before it in any case.  While the CTAs finish one job and convert the next
 * one's activations, the weights of the following jobs keep streaming into shared memory, so HBM
 * does not idle at the boundaries the way it does between separate launches.
 * Weights: QGEMV_FMT_NVFP4_TC only.  All jobs share the batch size B (1..8).  At most 4094 jobs, each
 * of fewer than 2^32 / SMs (128-row tile, 64-column item) pairs.  The job list is copied to the device by
 * qgemv_sequence_create (which allocates); qgemv_sequence_run launches, allocates nothing and may be
 * captured into a CUDA graph.  The kernel's CTAs wait on one another: the launch is cooperative and takes
 * every SM (grid_override above the SM count is refused).  QGEMV_ERR_UNSUPPORTED_SHAPE when the
 * activations of one job (B * K digit planes) leave no room for a weight ring in shared memory: call
 * qgemv_gemv per job then.  After a run that reported QGEMV_ERR_TIMEOUT, read the status
 * (qgemv_last_device_status) before the handle's next sequence run: that call puts the kernel's counters
 * and tags back in order. */
#define QGEMV_JOB_AFTER_PREVIOUS 1 /* start only when the job before this one is complete */
#define QGEMV_JOB_ALLREDUCE 2      /* row-parallel projection: y = sum over the ranks of W_r x_r (see the exchange below) */
#define QGEMV_JOB_X_SILU_MUL 4     /* the rows of x hold 2 K values (gate, then up): the GEMV multiplies bf16(silu(gate[k]) * up[k]) */
typedef struct qgemv_job {
    const qgemv_weight* w;
    const void* x;   /* device bf16 [B][K], 16-byte aligned */
    void* y;         /* device [B][N] */
    int32_t y_dtype; /* QGEMV_OUT_BF16 or QGEMV_OUT_F32 */
    int32_t flags;   /* 0, or an OR of QGEMV_JOB_AFTER_PREVIOUS, QGEMV_JOB_ALLREDUCE, QGEMV_JOB_X_SILU_MUL */
    int64_t x_stride; /* elements between the rows of x; 0 = K (2 K with QGEMV_JOB_X_SILU_MUL).  A multiple of 8 */
    /* Element-wise work of a decoder layer folded into the job ("fused norm / activation", the engines'
     * decode-gemv slot, engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:81).  All optional (NULL / 0): */
    const void* norm_weight; /* device bf16 [K], 16-byte aligned: RMS norm of the activations.  The GEMV multiplies
                              * x'[k] = bf16(x[k] * norm_weight[k]) and its result is scaled by
                              * rsqrt(mean_k x[k]^2 + norm_eps) in fp32 (the mean over the activations as the GEMV
                              * sees them, i.e. after QGEMV_JOB_X_SILU_MUL when both are set) */
    const void* residual;    /* device [B][N] in y's dtype: added to the result in fp32 before it is rounded; may be y */
    float norm_eps;
    int32_t reserved;        /* 0 */
} qgemv_job;
typedef struct qgemv_sequence qgemv_sequence;
int qgemv_sequence_create(qgemv_handle* h, const qgemv_job* jobs, int n_jobs, int B, qgemv_sequence** out);
int qgemv_sequence_run(qgemv_handle* h, const qgemv_sequence* seq, void* stream);
int qgemv_sequence_destroy(qgemv_handle* h, qgemv_sequence* seq);

/* ---- tensor-parallel exchange -------------------------------------------------------------------
 * Not in the registry (every listed engine runs on one GPU, engines/crit-labs/mtp5-nvfp4-drafts/
 * card.yaml:100); needed for the projections of a model sharded over the GPUs of one node:
 * column-parallel QKV and gate/up (shards from qgemv_pack_host / qgemv_load_device with a row
 * range), row-parallel o and down (a column range) whose outputs are partial sums.
 * One process per GPU: qgemv_tp_create allocates this rank's exchange buffer and returns its CUDA
 * IPC handle (QGEMV_IPC_HANDLE_BYTES); the caller gathers the handles of all ranks (any transport)
 * and passes the concatenation, rank order, to qgemv_tp_connect.  One process driving several
 * GPUs (peer access enabled by the caller) hands the other ranks' buffers over as pointers instead:
 * qgemv_tp_buffer of each handle, then qgemv_tp_connect_ptrs (peer_buffers[own rank] is ignored).
 *
 * The buffer: two parities x `world` slots x max_elems pairs {fp32 value, 32-bit tag}, 8 bytes
 * each, all zero at first: slot s of parity p starts at ((p * world + s) * max_elems) * 8.  A rank
 * pushes its values, tagged with the count of exchanges, into its slot of EVERY rank's buffer over
 * NVLink (plain peer stores), then reads the pairs of all ranks from its own buffer, re-polling --
 * bounded -- the ones whose tag is not there yet.  Sums are formed in fp32 in rank order, so every
 * rank gets the same bits.  No multicast; peers are only written to.
 *
 * qgemv_tp_allreduce: y (bf16 or fp32, n elements) becomes the sum over the ranks, in place.
 * qgemv_tp_allgather: y[r * n_shard + e] = rank r's shard[e] (column-parallel outputs, the logits
 * of a vocabulary-parallel output head); shard and y must not overlap.
 * Both are asynchronous on `stream` and may be captured into a CUDA graph; all ranks must issue
 * the same sequence of calls.  They use elements [0, n) of the slots.
 * Inside a job list (qgemv_sequence_create) a job flagged QGEMV_JOB_ALLREDUCE is reduced over the
 * ranks by the sequence kernel itself: the thread that has added up a row of the partial output
 * pushes it and gathers the other ranks' -- no launch, no grid-wide wait.  Such jobs take B * N
 * elements each from the TOP of the slots for as long as the list lives, so max_elems must cover
 * them plus the longest stand-alone exchange; QGEMV_ERR_UNSUPPORTED_SHAPE when it does not, or when
 * one CTA's share of the job would hold a whole 128-row tile (N above about 128 rows per SM).  Every
 * rank must create and run the same lists in the same order.  With world == 1 the flag is ignored.
 * After QGEMV_ERR_TIMEOUT from an exchange the ranks' counts may differ: destroy the handles. */
#define QGEMV_IPC_HANDLE_BYTES 64
int qgemv_tp_create(qgemv_handle* h, int rank, int world, int64_t max_elems, void* ipc_handle_out);
int qgemv_tp_connect(qgemv_handle* h, const void* all_handles);
int qgemv_tp_buffer(qgemv_handle* h, void** dev_ptr, size_t* bytes);
int qgemv_tp_connect_ptrs(qgemv_handle* h, void* const* peer_buffers /* [world] */);
int qgemv_tp_allreduce(qgemv_handle* h, void* y, int y_dtype, int64_t n, void* stream);
int qgemv_tp_allgather(qgemv_handle* h, const void* shard, void* y, int y_dtype, int64_t n_shard, void* stream);

/* ---- allocation-free GEMV --------------------------------------------------------------------
 * No counterpart in the crit-hub registry; added for callers that cannot allocate device memory
 * when they need a projection: code living inside a memory pool that owns the whole GPU, plugins
 * that must only use the buffers their host framework hands them, and latency-critical paths
 * where a cudaMalloc would stall the device.  This call allocates nothing (no cudaMalloc, no
 * cudaFree, no handle): the weights are a packed blob the CALLER copied to device memory
 * (`dev_blob`, 16-byte aligned, laid out by qgemv_pack_host), `host_header` is the first 256 bytes
 * of that blob in host memory, x and y are the caller's device buffers as for qgemv_gemv.
 * The kernel's scratch (partial sums and arrival counters of panels split between CTAs, a status
 * word, the tensor scale) is a 320 KiB array compiled into the library; every GPU that loads
 * the library holds it until the process exits.
 * Limits (QGEMV_ERR_UNSUPPORTED_SHAPE beyond them): N <= 262144 rows, ceil(K / 1024) * B <= 32
 * (e.g. K <= 32768 at B = 1, K <= 4096 at B = 8), B <= 8, at most 256 SMs.  The header is checked
 * against the sizes that follow from its format and shape (QGEMV_ERR_BAD_BLOB when they disagree).
 * The first call on a device resolves the array's device address and sets kernel attributes;
 * make that first call before any stream capture.  All calls share the one array, and it keeps
 * the previous call's contents: the call clears what must start at zero on `stream`, so calls
 * that overlap on the GPU (different streams, or concurrent threads) race -- serialise them.
 * Results equal qgemv_gemv's up to the summation order of the K split.
 * A bounded in-kernel wait that runs out leaves y unwritten and records itself in the array's status
 * word, which qgemv_gemv_noalloc never reads back (it does not synchronise):
 * qgemv_noalloc_last_status synchronises `stream` and copies out the status of the last call on the
 * current device (all zero when none has run).  It allocates nothing either. */
int qgemv_gemv_noalloc(const void* dev_blob, const void* host_header, const void* x_bf16, int B, void* y,
                       int y_dtype, void* stream);
int qgemv_noalloc_last_status(void* stream, qgemv_dev_status* out);

/* ---- skinny GEMM / short prefill -------------------------------------------------------------------
 * Y[M][N] = X[M][K] . dequant(W)^T for M = 16 .. 256 tokens (a multiple of 16) on the tcgen05
 * tensor cores with fp32 accumulators in tensor memory.  Replaces the engines' prompt GEMM
 * ("pinned-gemm ... about 40% of the GPU's FP4 rate",
 * engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:77,95; cuBLASLt NVFP4 / torch._scaled_mm FP8
 * prefill GEMMs, tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:77).
 * x: device bf16 [M][K], 16-byte aligned; y: device [M][N] bf16 or fp32.
 * act_mode QGEMV_ACT_A16_EXACT: weights are dequantised exactly to f16 tiles, activations stay
 * 16-bit (bf16 -> f16 with an exact per-row power-of-two scale), kind::f16 MMA: same 2e-3 bound
 * as the GEMV.  Weights in the lane order (QGEMV_FMT_NVFP4 / QGEMV_FMT_FP8).
 * act_mode QGEMV_ACT_A4_BLOCKSCALED: a different operator -- the activations are quantised to NVFP4
 * (E2M1 codes, one E4M3 scale per 16 K elements, one fp32 scale per token) and both operands go
 * through tcgen05.mma kind::mxf4nvf4 as stored ("NVFP4 ... prefill GEMMs",
 * tools/fixtures/engines/crit-labs/mtp4-nvfp4-mma/card.yaml:77).  Weights: QGEMV_FMT_NVFP4_TC, any N,
 * K a multiple of 16.  The quantiser is fixed bit for bit: per token row, fp32 round-to-nearest-even,
 *   g = max|x| / 2688 (1 if the row is zero);  per block  s = E4M3(max|x_block| / (6 g)), saturating;
 *   t = decode(s) g;  code = t == 0 ? 0 : E2M1(x / t), saturating;   x_q = decode(code) decode(s) g
 * and y[m][n] = tensor_scale * g[m] * sum_k w(n, k) x_q-without-g(m, k), fp32 in the tensor core.
 * Against an fp64 GEMM on the SAME quantised activations the result is within 2e-3 (far inside);
 * against unquantised activations it carries FP4's quantisation error (about 9 % relative L2 on N(0,1)
 * rows).  qgemv_quantize_a4 exposes the quantiser for parity checks.
 * QGEMV_ACT_A8 (FP8 activations) is not built: QGEMV_ERR_UNSUPPORTED_SHAPE.
 * Shapes of the A16 mode: single (unstacked) weight, N a multiple of 128, K a multiple of 64.
 * The call keeps an internal f16 copy of the activations (M*K*2 bytes); the first call with a
 * new largest M*K grows it with cudaMalloc after a device synchronise -- make that call outside
 * stream capture.  Three launches per call (activation row maxima, activation conversion, GEMM). */
#define QGEMV_ACT_A16_EXACT 0
#define QGEMV_ACT_A4_BLOCKSCALED 1
#define QGEMV_ACT_A8 2
int qgemv_gemm_skinny(qgemv_handle* h, const qgemv_weight* w, const void* x_bf16, int M, void* y,
                      int y_dtype, int act_mode, void* stream);
/* The A4 mode's activation quantiser alone (parity hook; no counterpart in the registry): x bf16 [M][K]
 * -> canonical codes u8 [M][K/2] (low nibble = even k, 8-byte aligned), block scales u8 [M][K/16] and
 * row scales fp32 [M], all in device memory. */
int qgemv_quantize_a4(qgemv_handle* h, const void* x_bf16, int M, int64_t K, void* codes_dev, void* scales_dev,
                      float* row_scales_dev, void* stream);
/* How qgemv_gemm_skinny would run a shape: pipeline grain, ring depths, tensor-memory and shared-
 * memory use, CTA count and scratch bytes.  Pure host arithmetic (no device needed); returns
 * QGEMV_ERR_UNSUPPORTED_SHAPE for shapes the GEMM refuses.  No counterpart in the reference. */
typedef struct qgemv_skinny_plan {
    int32_t run_units;      /* K units (of 64) per pipeline run: 4, 2 or 1 */
    int32_t x_stage_units;  /* K units per activation-ring stage */
    int32_t x_stages;       /* activation-ring stages in shared memory */
    int32_t p_stages;       /* packed-weight ring stages (8 panels x one run each) */
    int32_t a_stages;       /* dequantised-weight stages in tensor memory */
    int32_t tmem_columns;   /* tensor-memory columns allocated per CTA (power of two <= 512) */
    int32_t smem_bytes;     /* dynamic shared memory per CTA */
    int32_t ctas;           /* CTAs launched */
    int64_t scratch_bytes;  /* internal scratch the call needs (activation tiles, partial tiles, counters) */
} qgemv_skinny_plan;
int qgemv_gemm_skinny_plan(int fmt, int64_t N, int64_t K, int M, int sm_count, qgemv_skinny_plan* out);

/* ---- MoE grouped GEMV ---------------------------------------------------------------------------
 * One launch walks the router's top-k lists.  For every token t and slot j:
 *   out[t*topk + j][:] = W[expert_ids[t][j]] . x[row][:],
 *   row = t (per_slot_input == 0, gate/up stage) or t*topk + j (per_slot_input == 1, down stage).
 * experts: a stacked weight from qgemv_load_stacked; expert_ids: device int32 [T][topk];
 * x: device bf16; out: device [T*topk][N] bf16 or fp32.  T*topk <= 4096.  An id outside the stacked
 * weight is reported in the status word (QGEMV_ERR_BOUNDS, where 21) and nothing is computed.
 * Experts in the tensor-core layout (QGEMV_FMT_NVFP4_TC, the faster choice from a few tokens on) run as
 * ONE launch that also walks the lists: at most 512 experts; an expert's entries are worked on up to
 * min(8, T) rows at a time, fewer when the digit planes of that many rows x K would not fit beside a weight
 * ring in shared memory (from K > 4096 on), down to one; QGEMV_ERR_UNSUPPORTED_SHAPE beyond that (K > 23000).
 * The split-tile scratch belongs to the handle: keep calls that share a handle on one stream.
 * Lane-order experts (QGEMV_FMT_NVFP4, QGEMV_FMT_FP8) run as a router-walk kernel plus a streaming
 * kernel; with K > 2048 as several launches over K chunks plus a sum (fp32 partial results in a scratch
 * of the handle).
 * No listed engine publishes an MoE kernel; the shape is the registry's `host_expert_gbs`
 * probe slot (engines/crit-labs/mtp5-nvfp4-drafts/evidence/crit-eval.json:124). */
int qgemv_moe_gemv(qgemv_handle* h, const qgemv_weight* experts, const int32_t* expert_ids,
                   const void* x_bf16, int T, int topk, int per_slot_input, void* out,
                   int out_dtype, void* stream);
/* The same with an activation function applied to what is read (the experts' down stage without an element-wise
 * kernel before it; "fused norm / activation", engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:81):
 * x_act = QGEMV_MOE_X_SILU_MUL: the rows of x hold 2 K values, gate then up -- the output rows of the gate/up
 * stage as qgemv_moe_gemv leaves them -- and the GEMV multiplies bf16(silu(gate[k]) * up[k]).  x_act = 0:
 * qgemv_moe_gemv.  Tensor-core-layout experts only (QGEMV_ERR_UNSUPPORTED_SHAPE otherwise). */
#define QGEMV_MOE_X_SILU_MUL 1
int qgemv_moe_gemv_act(qgemv_handle* h, const qgemv_weight* experts, const int32_t* expert_ids,
                       const void* x_bf16, int T, int topk, int per_slot_input, int x_act, void* out,
                       int out_dtype, void* stream);
/* Both stages of the experts' MLP as ONE launch: out[t*topk + j][:] = W_down[e] . bf16(silu(g) * u) with
 * (g, u) = W_gate_up[e] . x[t][:], e = expert_ids[t][j] -- what qgemv_moe_gemv (gate/up, bf16 rows) followed by
 * qgemv_moe_gemv_act (down, QGEMV_MOE_X_SILU_MUL) computes, bit for bit, without the second launch: every CTA
 * works through its share of the gate/up items and then of the down items, and a down problem starts as soon as
 * its expert's gate/up rows are there.  gate_up: stacked [2 I][H], down: stacked [N][I], both in the tensor-core
 * layout with the same number of experts.  gate_up_rows: device bf16 [T*topk][2 I], 16-byte aligned, written by
 * the first stage and read by the second (the caller's scratch).  Limits as for qgemv_moe_gemv. */
int qgemv_moe_mlp(qgemv_handle* h, const qgemv_weight* gate_up, const qgemv_weight* down, const int32_t* expert_ids,
                  const void* x_bf16, int T, int topk, void* gate_up_rows, void* out, int out_dtype, void* stream);
/* How an expert-list launch would be laid out (host arithmetic only, no device needed): K of the experts, K2 of
 * a second stage in the same launch (0: none), experts, tokens, top-k, CTAs (one per SM), shared memory per CTA
 * in KB (0: 227).  QGEMV_ERR_UNSUPPORTED_SHAPE when qgemv_moe_gemv / qgemv_moe_mlp would refuse the shape. */
typedef struct qgemv_moe_plan_t {
    int32_t rows_per_problem; /* an expert's entries are worked on this many activation rows at a time */
    int32_t plane_buffers;    /* buffers of digit planes (problems the conversion may run ahead) */
    int32_t plane_slots;      /* 64-K items of planes per buffer */
    int32_t ring_stages;      /* stages of the weight ring */
    int32_t stage_items;      /* items per stage (4608 bytes each) */
    int32_t max_problems;     /* most problems the lists can make */
    int32_t table_offset;     /* offset of the CTA's problem table in shared memory */
    int32_t smem_bytes;       /* dynamic shared memory per CTA */
} qgemv_moe_plan_t;
int qgemv_moe_plan(int64_t K, int64_t K2, int n_experts, int T, int topk, int ctas, int smem_kb, qgemv_moe_plan_t* out);
/* y[t][:] = sum_j expert_w[t][j] * slot_out[t*topk + j][:]  (fixed j order, fp32 accumulate). */
int qgemv_moe_combine(qgemv_handle* h, const void* slot_out, int slot_dtype, const float* expert_w,
                      int T, int topk, int64_t N, void* y, int y_dtype, void* stream);

/* ---- parity hook ----------------------------------------------------------------------------
 * Writes dequant(W) as fp32 [N][K] (index `which` of a stacked weight) using the same in-kernel
 * conversion instructions as the GEMV; compared bit for bit with the host definition. */
int qgemv_dequant_f32(qgemv_handle* h, const qgemv_weight* w, int which, float* out_dev,
                      void* stream);

/* ---- diagnostics ------------------------------------------------------------------------------ */
/* Phase timestamps of the tensor-core GEMV (diagnostics; no counterpart in the registry).  `dev_buf`:
 * device memory of 16 x 8 bytes per CTA (one CTA per SM unless grid_override says otherwise), or NULL
 * to switch it off again.  Every later QGEMV_FMT_NVFP4_TC launch on the handle makes each CTA store
 * %globaltimer (ns) at [0] set-up done and [7] CTA done, and the SM's cycle counter (cheap to read;
 * comparable inside one CTA only) at: [9] set-up done, [1] dependency wait over, [2] activation
 * digit planes written, [3] MMA issuer released, [4] its first weight stage landed, [5] its last MMA
 * issued, [6] last accumulator complete, [8] last epilogue warp done.  A sequence launch
 * (qgemv_sequence_run) instead stores 8 x 8 bytes per (CTA, job) at [(cta * n_jobs + job) * 8 + k],
 * all %globaltimer: [0] conversion of the job's activations begins (its dependencies are met), [1] digit
 * planes ready, [3] MMA issuer sees them, [7] its first stage of the job issued, [4] its last, [5] last
 * accumulator seen by the epilogue, [2] rows / parts stored, [6] split tile added up and stored.  An
 * expert-list launch (qgemv_moe_gemv on the tensor-core layout) stores the same eight stamps per (CTA, problem
 * of the CTA's own range) at [(cta * 32 + local problem) * 8 + k], then per CTA at [(ctas * 32) * 8 + cta * 4 +
 * k]: [0] kernel entered, [1] router lists walked, [2] all roles through.  The caller zeroes and reads the
 * buffer; the stamps cost time, so a traced run is slower. */
int qgemv_set_trace(qgemv_handle* h, void* dev_buf);
/* Synchronises `stream`, reads and clears the device status word. */
int qgemv_last_device_status(qgemv_handle* h, void* stream, qgemv_dev_status* out);

#ifdef __cplusplus
}
#endif
#endif /* QGEMV_H_ */
