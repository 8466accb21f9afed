// tstream_format.h -- the library's own on-device weight format ("tile stream"), shared by the host
// packer and the kernels.
//
// The reference stores W as per-column index lists per K-tile (merged tiled CSC,
// ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:156-315).  This format keeps that idea -- 16-bit tile-local row
// ids, one +1 list and one -1 list per (column, tile) -- and lays the lists out for the way a B200
// streams and consumes them:
//
//   * The product is split over `num_ctas` thread blocks.  Block (b, j) owns column block b
//     (`cols_per_block` consecutive columns) and K-split j (`tiles_per_cta` consecutive tiles).  Everything a
//     block reads is ONE contiguous byte range of `stream`, so a single thread can pull it through a
//     shared-memory ring with bulk async copies, independent of list boundaries.
//   * Inside a block's range the order is: tile, column, sign (+ list then - list).  Every list is padded
//     to a multiple of 8 ids (one 16-byte vector) with the id `tile_rows`, which addresses an all-zero
//     row of the activation table, so padding needs no masking.
//   * `vstart` holds, per block and tile, the block-relative vector offset of every list plus an end
//     sentinel: 2*cols+1 uint32 per tile.  List l = 2*c + s (s = 0 for +1, 1 for -1).
//   * Lists are consumed by groups of `lanes_per_list` lanes; 32/lanes_per_list consecutive lists form one
//     warp work unit.  A unit never exceeds TS_RING_VECS - TS_STAGE_VECS vectors (the packer checks), so it
//     always fits in the ring.
//
// Split-K partial sums go to a scratch buffer [k_splits][rows][columns] fp32 (int32 for int8
// activations); the last block to finish a column block adds them in split order, applies the scale and
// writes Y, so the result does not depend on scheduling.
#pragma once
#include <cstdint>
#include <vector>

#define TS_MAX_CTAS 160          // per-block descriptors travel in kernel parameters
#define TS_MAX_TILE_ROWS 1024    // (tile_rows+1) rows * 128 B = 128.1 KiB activation table
#define TS_STAGE_VECS 512        // 16-byte vectors per ring stage (8 KiB)
#define TS_MAX_STAGES 8
#define TS_RING_VECS (TS_STAGE_VECS * TS_MAX_STAGES)   // power of two
#define TS_MAX_META_BYTES (20 * 1024)
#define TS_IDS_PER_VEC 8

struct TsCtaDesc {
    uint32_t stream_off;   // first vector of this block's range (units of 16 B)
    uint32_t nvec;         // vectors in the range
    uint32_t meta_off;     // first uint32 of this block's vstart table (multiple of 4)
    uint32_t meta_words;   // uint32 in the table, padded to a multiple of 4
};

struct TsLayout {
    int inners = 0, columns = 0;
    int tile_rows = 0, tiles = 0;
    int col_blocks = 0, cols_per_block = 0;
    int k_splits = 0, tiles_per_cta = 0;
    int num_ctas = 0;          // col_blocks * k_splits ; block id = j * col_blocks + b
    int lanes_per_list = 0;    // power of two, 1..16
    int64_t nnz = 0;
    int64_t total_vecs = 0;
    TsCtaDesc cta[TS_MAX_CTAS];
};

struct TsHostImage {
    TsLayout lay;
    std::vector<uint16_t> stream;   // total_vecs * 8 ids
    std::vector<uint32_t> vstart;   // concatenated per-block tables
};

struct tllm_pack_opts;

// Builds the image from a dense ternary matrix (int8 [inners][columns]); returns "" or an error message.
const char* ts_pack_dense(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                          TsHostImage* out);

// Inverse, for tests of the packer alone: rebuild the dense matrix from an image.
void ts_unpack_dense(const TsHostImage& img, int8_t* w);

// Checks the invariants the kernel relies on; returns nullptr or a message.
const char* ts_validate(const TsHostImage& img);
