// Packed weight layout shared by the host packer and the sm_100a kernels.
//
// The matrix is cut into PANELS of 16 output rows (the M extent of one
// mma.m16n8k16 tile) and UNITS of 64 consecutive K elements (four E4M3 scale
// blocks of 16).  The blob stores units panel-major:
//
//     payload offset of (panel p, unit u) = (p * units_per_panel + u) * unit_bytes
//
// so any K range of one panel is one contiguous byte range, which a single
// bulk (TMA) copy moves into shared memory, and a shard of whole panels or of
// whole units is a sub-range of the same layout.
//
// Inside a unit the bytes are ordered by the lane that consumes them.  Lane
// l = 4*g + t of a warp (g = l >> 2, t = l & 3) owns rows g and g + 8 of the
// panel.  One unit feeds four MMA tiles T = 0..3.  Tile T = 2*pr + sub covers
// the scale-block pair (2*pr, 2*pr + 1); the k index j of the MMA maps to
//     block  kb = 2*pr + (j & 1)              (even j: first block, odd j: second)
//     elem   e  = 4*((j & 7) >> 1) + 2*sub + (j >> 3)
// i.e. each f16x2 register of the A fragment holds one element of each block
// of the pair, so that one f16x2 (scale[kb], scale[kb+1]) multiplies it, and
// the activation fragment uses the same permutation.  With t = (j & 7) >> 1,
// r = j >> 3 and h = j & 1:  e = 4*t + 2*sub + r,  kb = 2*pr + h.
//
// NVFP4 unit (576 bytes):
//   [0, 512)   lane l: 16 bytes at l*16; 32-bit word T; byte jb = rowhi + 2*r of the word holds
//              row g + 8*rowhi; low nibble = block 2*pr (h = 0), high nibble = block 2*pr + 1.
//   [512, 576) 8 bytes at 512 + g*8: E4M3 scales of row g, blocks 0..3, then row g + 8, blocks 0..3.
// FP8 unit (1024 bytes):
//   half hf = T >> 1 at hf*512; lane l: 16 bytes at hf*512 + l*16; tile T & 1 at +8*(T & 1);
//   16-bit slot jb = rowhi + 2*r at +2*jb; low byte = block 2*pr (h = 0), high byte = h = 1.
//
// Tensor-core layout (QGEMV_FMT_NVFP4_TC): the same NVFP4 values in the order the block-scaled
// tcgen05.mma (kind::mxf4nvf4, one E4M3 scale per 16 K elements) consumes without any conversion.
// The matrix is cut into row TILES of 128 rows and ITEMS of 64 K elements; the blob stores items
// tile-major:
//     payload offset of (tile q, item kt) = (q * items_per_tile + kt) * 4608
// ITEM (4608 bytes):
//   [0, 4096)     E2M1 codes as the MMA's K-major, no-swizzle A operand: core matrices of 8 rows x
//                 16 bytes (32 codes, low nibble = even k); row r, element k at
//                 (r / 8) * 256 + (k / 32) * 128 + (r % 8) * 16 + (k % 32) / 2.
//   [4096, 4608)  E4M3 block scales in the order tcgen05.cp.32x128b.warpx4 copies into tensor
//                 memory: row r, block kb at (r % 32) * 16 + (r / 32) * 4 + kb.
// In the blob header such a matrix reports n_panels = 8 * tiles and unit_bytes = 576 (an item is
// eight panels' worth of units), so payload_bytes = n_panels * units_per_panel * unit_bytes holds.
#ifndef QGEMV_LAYOUT_H_
#define QGEMV_LAYOUT_H_

#include <stdint.h>

#if defined(__CUDACC__)
#define QG_HD __host__ __device__ __forceinline__
#else
#define QG_HD inline
#endif

#define QG_PANEL_ROWS 16
#define QG_UNIT_K 64
#define QG_NVFP4_UNIT_BYTES 576
#define QG_FP8_UNIT_BYTES 1024
#define QG_TC_TILE_ROWS 128
#define QG_TC_ITEM_BYTES 4608
#define QG_PHASE_UNITS 16 /* activation staging window: 1024 K elements */
#define QG_BLOB_MAGIC 0x564D4751u /* "QGMV" */
#define QG_BLOB_VERSION 3u
#define QG_HEADER_BYTES 256

typedef struct qg_blob_header {
    uint32_t magic;
    uint32_t version;
    uint32_t fmt;
    uint32_t header_bytes;
    int64_t N;               /* rows held by this blob */
    int64_t K;               /* columns held by this blob */
    int64_t n_panels;        /* ceil(N / 16) */
    int64_t units_per_panel; /* ceil(K / 64) */
    uint32_t unit_bytes;
    uint32_t reserved0;
    float tensor_scale;
    uint32_t reserved1;
    uint64_t aux_bytes;     /* FP8: fp32 channel scales [n_panels*16], padded to 256 bytes */
    uint64_t payload_bytes; /* n_panels * units_per_panel * unit_bytes */
    uint64_t checksum;      /* over aux + payload */
    uint8_t pad[QG_HEADER_BYTES - 88];
} qg_blob_header;

/* Byte offset inside an NVFP4 unit of the code of (row 0..15, block kb 0..3, element e 0..15);
 * *nibble_hi tells which nibble. */
QG_HD uint32_t qg_nvfp4_code_offset(int row, int kb, int e, int* nibble_hi) {
    const int g = row & 7, rowhi = row >> 3;
    const int pr = kb >> 1, h = kb & 1;
    const int t = e >> 2, sub = (e >> 1) & 1, r = e & 1;
    *nibble_hi = h;
    return (uint32_t)((4 * g + t) * 16 + (2 * pr + sub) * 4 + (rowhi + 2 * r));
}
QG_HD uint32_t qg_nvfp4_scale_offset(int row, int kb) {
    return (uint32_t)(512 + (row & 7) * 8 + (row >> 3) * 4 + kb);
}
QG_HD uint32_t qg_fp8_code_offset(int row, int kb, int e) {
    const int g = row & 7, rowhi = row >> 3;
    const int pr = kb >> 1, h = kb & 1;
    const int t = e >> 2, sub = (e >> 1) & 1, r = e & 1;
    return (uint32_t)(pr * 512 + (4 * g + t) * 16 + sub * 8 + (rowhi + 2 * r) * 2 + h);
}
/* Activation fragment buffer of one phase (16 units): byte offset of the f16 holding
 * (unit q in phase, block kb, element e) of batch column b. */
QG_HD uint32_t qg_xfrag_offset(int q, int kb, int e, int b) {
    const int pr = kb >> 1, h = kb & 1;
    const int t = e >> 2, sub = (e >> 1) & 1, r = e & 1;
    return (uint32_t)(q * 1024 + pr * 512 + (4 * b + t) * 16 + (2 * sub + r) * 4 + h * 2);
}

/* Tensor-core layout: byte offset inside an item of the code of (row 0..127, element k 0..63). */
QG_HD uint32_t qg_tc_code_offset(int row, int k, int* nibble_hi) {
    *nibble_hi = k & 1;
    return (uint32_t)((row >> 3) * 256 + (k >> 5) * 128 + (row & 7) * 16 + ((k & 31) >> 1));
}
QG_HD uint32_t qg_tc_scale_offset(int row, int kb) {
    return (uint32_t)(4096 + (row & 31) * 16 + (row >> 5) * 4 + kb);
}

#endif /* QGEMV_LAYOUT_H_ */
