// tstream_format.h -- the library's own on-device weight format ("tile stream"), shared by the host
// packer and the kernels.
//
// The reference stores W as per-column index lists per K-tile (merged tiled CSC,
// ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:156-315).  This format keeps that idea -- 16-bit tile-local row
// ids, one +1 list and one -1 list per (column, tile) -- and lays the lists out for the way a B200 warp
// streams them with 128-bit loads:
//
//   * The product is split over `num_ctas` thread blocks.  Block (b, j) owns column block b
//     (`cols_per_block` consecutive columns, processed in sub-blocks of `sub_cols` columns whose sums fit in
//     shared memory) and K-split j (`tiles_per_cta` consecutive tiles of `tile_rows` rows).
//   * Inside a (block, tile, sub-block) -- a "section" -- the 2*cols lists are sorted by length, longest
//     first, and stored as jagged diagonals: diagonal i holds vector i of every list that has one, in sorted
//     order, so the lists present in a diagonal are always a prefix of the sorted order and nothing but the
//     last vector of a list is ever padded.  Lane l of the section (32 consecutive lanes = one warp's group)
//     owns sorted list l; at step i a warp reads 32 consecutive 16-byte vectors of diagonal i: one coalesced
//     512-byte access, and all warps of the block together sweep a contiguous window of the stream, which is
//     what HBM serves best.  With lanes_per_list = L > 1 (narrow column blocks) a list's vectors are dealt
//     round-robin to L adjacent lanes and its length is rounded up to a multiple of L vectors.
//   * A vector holds 8 row ids; the tail of a list is padded with the id `tile_rows`, which addresses an
//     all-zero row of the activation table, so padding needs no masking.  Diagonals start on 128 bytes.
//   * Per block a table of 32-bit words, copied to shared memory by one bulk async copy, describes its
//     sections in processing order (tile, sub-block):
//        word 0  block-relative vector offset of the section        word 1  number of diagonals D
//        word 2  lists in the section (2 * columns of the sub-block) word 3  reserved
//        D+1 words  section-relative vector offset of every diagonal (last = section length)
//        one word per sorted list: bits 0..14 column within the sub-block, bit 15 sign (1 = the -1 list),
//                                  bits 16..31 steps (vectors per owning lane)
//
// Split-K partial sums go to a scratch buffer [k_splits][rows][columns] fp32 (int32 for int8
// activations); the last block to finish a column block adds them in split order, applies the scale and
// writes Y, so the result does not depend on scheduling.
#pragma once
#include <cstdint>
#include <vector>

#define TS_MAX_CTAS 160          // resident blocks the schedule is sized for (one per SM); the first TS_MAX_CTAS
                                 // per-block descriptors travel in kernel parameters, the rest are read from memory
#define TS_MAX_BLOCKS 4096       // blocks of one launch (wide matrices run as several waves of blocks)
#define TS_MAX_TILE_ROWS 1024    // (tile_rows+1) rows * 128 B = 128.1 KiB activation table
#define TS_MAX_SUB_COLS 512      // column sums of a sub-block live in shared memory: 16 rows * 512 * 4 B = 32 KiB
#define TS_STAGE_BYTES (32 * 1024)   // raw activation tile staged by TMA before it is expanded into the table
#define TS_MAX_META_BYTES (24 * 1024)
#define TS_IDS_PER_VEC 8
#define TS_SEC_HEADER 4          // uint32 words in front of a section's diagonal offsets

struct TsCtaDesc {
    uint32_t stream_off;   // first vector of this block's range (units of 16 B), multiple of 32
    uint32_t nvec;         // vectors in the range, multiple of 32
    uint32_t meta_off;     // first uint32 of this block's section table (multiple of 4)
    uint32_t meta_words;   // uint32 in the table, padded to a multiple of 4
};

struct TsLayout {
    int inners = 0, columns = 0;
    int tile_rows = 0, tiles = 0;
    int col_blocks = 0, cols_per_block = 0, sub_cols = 0;
    int k_splits = 0, tiles_per_cta = 0;
    int num_ctas = 0;          // blocks of a launch: col_blocks * k_splits ; block id = j * col_blocks + b
    int lanes_per_list = 0;    // power of two, 1..16
    int64_t nnz = 0;
    int64_t total_vecs = 0;
    std::vector<TsCtaDesc> cta;   // num_ctas descriptors
};

// number of sub-blocks of a column block of `ncols` columns
inline int ts_num_subs(int ncols, int sub_cols) { return (ncols + sub_cols - 1) / sub_cols; }

struct TsHostImage {
    TsLayout lay;
    std::vector<uint16_t> stream;   // total_vecs * 8 ids
    std::vector<uint32_t> meta;     // concatenated per-block section tables
};

struct tllm_pack_opts;

// Dense two-bit copy of W for the tensor-core kernel ("bit tiles"): for output-column tile nt (128 columns) and
// K-slice kb (64 rows), 128 consecutive 16-byte records, one per column, each holding 64 codes
// (0: zero, 1: +1, 2: -1).  Row k_local of the slice sits in 32-bit word k_local/16 at bit mm_code_bit(k_local%16).
inline int mm_code_bit(int kk) {            // kk = 0..15
    const int j = kk >> 1, h = kk & 1;       // output word (two values) and half within it
    return (j < 4 ? 2 * j : 16 + 2 * (j - 4)) + 8 * h;
}
void mm_pack_bits(const int8_t* w, int inners, int columns, std::vector<uint32_t>* bits, int* n_tiles, int* kb);
void mm_unpack_bits(const std::vector<uint32_t>& bits, int inners, int columns, int8_t* w);

// Builds the image from a dense ternary matrix (int8 [inners][columns]); returns nullptr or an error message.
const char* ts_pack_dense(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                          TsHostImage* out);

// Inverse, for tests of the packer alone: rebuild the dense matrix from an image.
void ts_unpack_dense(const TsHostImage& img, int8_t* w);

// Checks the invariants the kernel relies on; returns nullptr or a message.
const char* ts_validate(const TsHostImage& img);
