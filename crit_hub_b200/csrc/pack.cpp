// Host weight packer: canonical codes / scales -> the lane-ordered blob described in
// qgemv_layout.h, and its inverse.  Pure byte shuffling, no GPU.
//
// Provides the "weights as stored" side of the quantized projections
// (engines/crit-labs/mtp5-nvfp4-drafts/card.yaml:69,77): the stored NVFP4 / FP8 matrices are
// re-laid once at load time; no value is re-encoded.
#include <cstdint>
#include <cstring>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../../include/qgemv.h"
#include "qgemv_layout.h"

namespace {

struct Dims {
    int64_t n0, n1, k0, k1;  // window of the canonical matrix
    int64_t n, k;            // window extent
    int64_t panels, units;
    uint32_t unit_bytes;
    uint64_t aux_bytes, payload_bytes;
};

bool make_dims(int fmt, int64_t N, int64_t K, const qgemv_shard* sh, Dims* d) {
    if (fmt != QGEMV_FMT_NVFP4 && fmt != QGEMV_FMT_FP8 && fmt != QGEMV_FMT_NVFP4_TC) return false;
    if (N <= 0 || K <= 0 || (K % 16) != 0) return false;
    d->n0 = 0, d->n1 = N, d->k0 = 0, d->k1 = K;
    if (sh) {
        d->n0 = sh->n0, d->n1 = sh->n1, d->k0 = sh->k0, d->k1 = sh->k1;
        if (d->n0 < 0 || d->n1 > N || d->n0 >= d->n1) return false;
        if (d->k0 < 0 || d->k1 > K || d->k0 >= d->k1) return false;
        if ((d->k0 % 16) != 0 || (d->k1 % 16) != 0) return false;
    }
    d->n = d->n1 - d->n0;
    d->k = d->k1 - d->k0;
    d->panels = (d->n + QG_PANEL_ROWS - 1) / QG_PANEL_ROWS;
    if (fmt == QGEMV_FMT_NVFP4_TC) d->panels = (d->n + QG_TC_TILE_ROWS - 1) / QG_TC_TILE_ROWS * 8;  // whole 128-row tiles
    d->units = (d->k + QG_UNIT_K - 1) / QG_UNIT_K;
    d->unit_bytes = fmt == QGEMV_FMT_FP8 ? QG_FP8_UNIT_BYTES : QG_NVFP4_UNIT_BYTES;
    d->aux_bytes = 0;
    if (fmt == QGEMV_FMT_FP8) d->aux_bytes = (uint64_t(d->panels) * 16 * 4 + 255) / 256 * 256;
    d->payload_bytes = uint64_t(d->panels) * uint64_t(d->units) * d->unit_bytes;
    return true;
}

uint64_t checksum64(const uint8_t* p, uint64_t bytes) {
    // word-wise multiply-rotate hash; bytes is always a multiple of 8 here
    uint64_t h = 0x243F6A8885A308D3ull;
    const uint64_t n = bytes / 8;
    for (uint64_t i = 0; i < n; ++i) {
        uint64_t w;
        std::memcpy(&w, p + 8 * i, 8);
        h = (h ^ w) * 0x9E3779B97F4A7C15ull;
        h = (h << 29) | (h >> 35);
    }
    return h ^ bytes;
}

void fill_header(qg_blob_header* hd, int fmt, const Dims& d, float tensor_scale) {
    std::memset(hd, 0, sizeof *hd);
    hd->magic = QG_BLOB_MAGIC;
    hd->version = QG_BLOB_VERSION;
    hd->fmt = uint32_t(fmt);
    hd->header_bytes = QG_HEADER_BYTES;
    hd->N = d.n;
    hd->K = d.k;
    hd->n_panels = d.panels;
    hd->units_per_panel = d.units;
    hd->unit_bytes = d.unit_bytes;
    hd->tensor_scale = fmt == QGEMV_FMT_FP8 ? 1.0f : tensor_scale;
    hd->aux_bytes = d.aux_bytes;
    hd->payload_bytes = d.payload_bytes;
}

const qg_blob_header* check_header(const void* blob, size_t bytes) {
    if (!blob || bytes < QG_HEADER_BYTES) return nullptr;
    const qg_blob_header* hd = static_cast<const qg_blob_header*>(blob);
    if (hd->magic != QG_BLOB_MAGIC || hd->version != QG_BLOB_VERSION) return nullptr;
    if (hd->header_bytes != QG_HEADER_BYTES) return nullptr;
    if (hd->fmt != QGEMV_FMT_NVFP4 && hd->fmt != QGEMV_FMT_FP8 && hd->fmt != QGEMV_FMT_NVFP4_TC) return nullptr;
    if (hd->N <= 0 || hd->K <= 0 || hd->K % 16 != 0) return nullptr;
    const int64_t want_panels = hd->fmt == QGEMV_FMT_NVFP4_TC ? (hd->N + 127) / 128 * 8 : (hd->N + 15) / 16;
    if (hd->n_panels != want_panels || hd->units_per_panel != (hd->K + 63) / 64) return nullptr;
    const uint32_t ub = hd->fmt == QGEMV_FMT_FP8 ? QG_FP8_UNIT_BYTES : QG_NVFP4_UNIT_BYTES;
    if (hd->unit_bytes != ub) return nullptr;
    if (hd->payload_bytes != uint64_t(hd->n_panels) * uint64_t(hd->units_per_panel) * ub) return nullptr;
    if (uint64_t(bytes) != QG_HEADER_BYTES + hd->aux_bytes + hd->payload_bytes) return nullptr;
    return hd;
}

}  // namespace

extern "C" {

size_t qgemv_packed_size(int fmt, int64_t N, int64_t K, const qgemv_shard* shard) {
    Dims d;
    if (!make_dims(fmt, N, K, shard, &d)) return 0;
    return size_t(QG_HEADER_BYTES + d.aux_bytes + d.payload_bytes);
}

// Threads of the packer's OpenMP loops.  Launchers of one process per GPU often export
// OMP_NUM_THREADS=1; a process that packs many matrices sets its share of the cores here.
int qgemv_set_host_threads(int n) {
    if (n < 1) return QGEMV_ERR_INVALID_ARG;
#ifdef _OPENMP
    omp_set_num_threads(n);
#endif
    return QGEMV_OK;
}

// The 256-byte header qgemv_pack_host would write for this matrix (checksum left zero): for
// callers that lay the payload out themselves, on the device.
int qgemv_pack_header(int fmt, float tensor_scale, int64_t N, int64_t K, const qgemv_shard* shard, void* header_out) {
    Dims d;
    if (!header_out) return QGEMV_ERR_INVALID_ARG;
    if (!make_dims(fmt, N, K, shard, &d)) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    fill_header(static_cast<qg_blob_header*>(header_out), fmt, d, tensor_scale);
    return QGEMV_OK;
}

int qgemv_pack_host(int fmt, const void* codes_v, const void* scales_v, float tensor_scale,
                    int64_t N, int64_t K, const qgemv_shard* shard, void* blob_out) {
    Dims d;
    if (!codes_v || !scales_v || !blob_out) return QGEMV_ERR_INVALID_ARG;
    if (!make_dims(fmt, N, K, shard, &d)) return QGEMV_ERR_UNSUPPORTED_SHAPE;
    uint8_t* blob = static_cast<uint8_t*>(blob_out);
    qg_blob_header hd;
    fill_header(&hd, fmt, d, tensor_scale);

    uint8_t* aux = blob + QG_HEADER_BYTES;
    uint8_t* payload = aux + d.aux_bytes;
    const uint8_t* codes = static_cast<const uint8_t*>(codes_v);

    if (fmt == QGEMV_FMT_FP8) {
        std::memset(aux, 0, d.aux_bytes);
        const float* cs = static_cast<const float*>(scales_v);
        std::memcpy(aux, cs + d.n0, size_t(d.n) * 4);
    }

    if (fmt == QGEMV_FMT_NVFP4_TC) {
        const uint8_t* sc = static_cast<const uint8_t*>(scales_v);
        const int64_t tiles = d.panels / 8;
#pragma omp parallel for schedule(static)
        for (int64_t q = 0; q < tiles; ++q) {
            for (int64_t kt = 0; kt < d.units; ++kt) {
                uint8_t* item = payload + (uint64_t(q) * d.units + kt) * QG_TC_ITEM_BYTES;
                std::memset(item, 0, QG_TC_ITEM_BYTES);
                for (int row = 0; row < QG_TC_TILE_ROWS; ++row) {
                    const int64_t n = q * QG_TC_TILE_ROWS + row;
                    if (n >= d.n) break;
                    const int64_t gn = d.n0 + n;
                    for (int kb = 0; kb < 4; ++kb) {
                        const int64_t kk = kt * 64 + kb * 16;  // window-relative k of the block
                        if (kk >= d.k) break;
                        const int64_t gk = d.k0 + kk;
                        int hi;
                        // 16 codes = 8 bytes, already in the item's nibble order (low nibble = even k)
                        std::memcpy(item + qg_tc_code_offset(row, kb * 16, &hi), codes + gn * (K / 2) + gk / 2, 8);
                        item[qg_tc_scale_offset(row, kb)] = sc[gn * (K / 16) + gk / 16];
                    }
                }
            }
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < (fmt == QGEMV_FMT_NVFP4_TC ? 0 : d.panels); ++p) {
        for (int64_t u = 0; u < d.units; ++u) {
            uint8_t* unit = payload + (uint64_t(p) * d.units + u) * d.unit_bytes;
            std::memset(unit, 0, d.unit_bytes);
            for (int row = 0; row < 16; ++row) {
                const int64_t n = p * 16 + row;
                if (n >= d.n) break;
                const int64_t gn = d.n0 + n;
                for (int kb = 0; kb < 4; ++kb) {
                    const int64_t kk = u * 64 + kb * 16;  // window-relative k of the block
                    if (kk >= d.k) break;
                    const int64_t gk = d.k0 + kk;
                    if (fmt == QGEMV_FMT_NVFP4) {
                        const uint8_t* src = codes + gn * (K / 2) + gk / 2;  // 8 bytes, 16 codes
                        for (int e = 0; e < 16; ++e) {
                            const uint8_t byte = src[e >> 1];
                            const uint8_t code = (e & 1) ? uint8_t(byte >> 4) : uint8_t(byte & 15);
                            int hi;
                            const uint32_t off = qg_nvfp4_code_offset(row, kb, e, &hi);
                            unit[off] = uint8_t(unit[off] | (hi ? (code << 4) : code));
                        }
                        const uint8_t* sc = static_cast<const uint8_t*>(scales_v);
                        unit[qg_nvfp4_scale_offset(row, kb)] = sc[gn * (K / 16) + gk / 16];
                    } else {
                        const uint8_t* src = codes + gn * K + gk;
                        for (int e = 0; e < 16; ++e) unit[qg_fp8_code_offset(row, kb, e)] = src[e];
                    }
                }
            }
        }
    }
    hd.checksum = checksum64(aux, d.aux_bytes + d.payload_bytes);
    std::memcpy(blob, &hd, sizeof hd);
    return QGEMV_OK;
}

int qgemv_blob_info(const void* blob, size_t bytes, int* fmt, int64_t* N, int64_t* K) {
    const qg_blob_header* hd = check_header(blob, bytes);
    if (!hd) return QGEMV_ERR_BAD_BLOB;
    if (fmt) *fmt = int(hd->fmt);
    if (N) *N = hd->N;
    if (K) *K = hd->K;
    return QGEMV_OK;
}

// Returns QGEMV_OK when the header is consistent and the checksum matches.
int qgemv_blob_verify(const void* blob, size_t bytes) {
    const qg_blob_header* hd = check_header(blob, bytes);
    if (!hd) return QGEMV_ERR_BAD_BLOB;
    const uint8_t* aux = static_cast<const uint8_t*>(blob) + QG_HEADER_BYTES;
    if (checksum64(aux, hd->aux_bytes + hd->payload_bytes) != hd->checksum) return QGEMV_ERR_BAD_BLOB;
    return QGEMV_OK;
}

int qgemv_unpack_host(const void* blob, size_t bytes, void* codes_out, void* scales_out,
                      float* tensor_scale_out) {
    if (!codes_out || !scales_out) return QGEMV_ERR_INVALID_ARG;
    if (qgemv_blob_verify(blob, bytes) != QGEMV_OK) return QGEMV_ERR_BAD_BLOB;
    const qg_blob_header* hd = static_cast<const qg_blob_header*>(blob);
    const uint8_t* aux = static_cast<const uint8_t*>(blob) + QG_HEADER_BYTES;
    const uint8_t* payload = aux + hd->aux_bytes;
    const int64_t N = hd->N, K = hd->K, units = hd->units_per_panel;
    uint8_t* codes = static_cast<uint8_t*>(codes_out);
    if (tensor_scale_out) *tensor_scale_out = hd->tensor_scale;
    if (hd->fmt == QGEMV_FMT_FP8) {
        std::memcpy(scales_out, aux, size_t(N) * 4);
    } else {
        std::memset(codes, 0, size_t(N) * size_t(K / 2));
    }
    if (hd->fmt == QGEMV_FMT_NVFP4_TC) {
#pragma omp parallel for schedule(static)
        for (int64_t n = 0; n < N; ++n) {
            const int64_t q = n / QG_TC_TILE_ROWS;
            const int row = int(n % QG_TC_TILE_ROWS);
            for (int64_t kk = 0; kk < K; kk += 16) {
                const uint8_t* item = payload + (uint64_t(q) * units + kk / 64) * QG_TC_ITEM_BYTES;
                const int kb = int((kk % 64) / 16);
                int hi;
                std::memcpy(codes + n * (K / 2) + kk / 2, item + qg_tc_code_offset(row, kb * 16, &hi), 8);
                static_cast<uint8_t*>(scales_out)[n * (K / 16) + kk / 16] = item[qg_tc_scale_offset(row, kb)];
            }
        }
        return QGEMV_OK;
    }
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t p = n / 16;
        const int row = int(n % 16);
        for (int64_t kk = 0; kk < K; kk += 16) {
            const int64_t u = kk / 64;
            const int kb = int((kk % 64) / 16);
            const uint8_t* unit = payload + (uint64_t(p) * units + u) * hd->unit_bytes;
            if (hd->fmt == QGEMV_FMT_NVFP4) {
                uint8_t* dst = codes + n * (K / 2) + kk / 2;
                for (int e = 0; e < 16; ++e) {
                    int hi;
                    const uint32_t off = qg_nvfp4_code_offset(row, kb, e, &hi);
                    const uint8_t code = hi ? uint8_t(unit[off] >> 4) : uint8_t(unit[off] & 15);
                    dst[e >> 1] = uint8_t(dst[e >> 1] | ((e & 1) ? (code << 4) : code));
                }
                static_cast<uint8_t*>(scales_out)[n * (K / 16) + kk / 16] =
                    unit[qg_nvfp4_scale_offset(row, kb)];
            } else {
                uint8_t* dst = codes + n * K + kk;
                for (int e = 0; e < 16; ++e) dst[e] = unit[qg_fp8_code_offset(row, kb, e)];
            }
        }
    }
    return QGEMV_OK;
}

}  // extern "C"
