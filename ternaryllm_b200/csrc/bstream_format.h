// bstream_format.h -- the compact on-device weight format ("bank stream"), shared by the host packer and
// the decode kernel.
//
// The reference stores W as per-column lists of 16-bit tile-local row ids, one +1 list and one -1 list per
// (column, K-tile) (merged tiled CSC, ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:156-315); its FPGA design already
// uses 8-bit ids inside 128-row slices (ternaryLLM_FPGA/hw/spinal/gemmacc/src/Config.scala:32,52).  This format
// keeps the lists and the tile, but cuts every list by the shared-memory bank its rows fall into:
//
//   * Row k of a K-tile of 4096 rows (BS_TILE_ROWS; a packing option allows fewer) belongs to lane k % 32 and row group (k % 4096) / 32.  The activation table
//     of a tile in shared memory is [129 row groups][32 lanes] entries (group 128 is all zero), so entry
//     (group g, lane l) sits in bank l: a warp in which lane l only ever reads groups of its own lane gathers
//     without bank conflicts whatever the ids are, from a table that is not replicated (16.1 KiB per tile and
//     activation row instead of 128 KiB per 1024 rows).
//   * Because the lane is implied, an id is one byte: the row group 0..127, or 128 = "nothing" (reads zero).
//   * Lane l's stream for a *unit* -- one warp's share of the product: K-tile t, columns [c0, c0+n) -- is the
//     concatenation over those columns of its +1 list and its -1 list, every list padded with id 128 to a whole
//     number of 32-bit words (an empty list is one word of padding).  The words are laid into 16-byte vectors:
//     words 0..2 hold four ids, word 3 holds three ids and, in its top byte, four flags: bit j set = a list ends
//     with word j of this vector.  So a vector carries 15 ids and the list structure travels with them.
//   * The 32 lane streams of a unit differ in length.  Vectors 0 .. min-1 (min = shortest lane) are interleaved,
//     vector i of lane l at (i*32 + l): a warp reads 512 contiguous bytes per step.  The remaining vectors follow
//     lane by lane.  Nothing is padded to the longest lane.
//   * A lane adds what it gathers into one accumulator and, at every flagged word, stores it into its cell of the
//     next slot of a 16-slot ring in shared memory (slot s of a unit = list s: column c0 + s/2, sign s & 1).  The
//     lanes drift apart by a few slots; the packer simulates the walk and records the vector indices ("reduce
//     points") after which the next eight slots are complete in all 32 lanes, and it ends a unit early wherever
//     a lane would otherwise run more than 16 slots ahead of the reduced ones.  At a reduce point the warp adds
//     the 32 lane cells of each of the eight slots and combines (+ list) - (- list) into four column sums.
//   * A thread block owns a contiguous column range and a contiguous range of K-tiles; the ranges are chosen by
//     non-zero count, not by width.  Its warps own contiguous column sub-ranges (again by non-zero count) across
//     all of the block's tiles, one or more units per (warp, tile).  Per block one table of 32-bit words describes
//     that (below); it is copied to shared memory with one bulk async copy.
//
// Block table (uint32 words, offsets relative to the table):
//     0 first column   1 columns   2 first tile   3 tiles   4 K-split index   5 column-block index   6 units   7 0
//     8 .. 8+BS_WARPS   word offset of warp w's first unit descriptor; entry BS_WARPS = end of the last one
//   unit descriptor:
//     0 first vector of the unit (16-byte units, relative to the block's first vector; multiple of 8)
//     1 first column relative to the block | columns << 16
//     2 tile relative to the block | number of reduce points << 8
//     3 shortest lane (vectors) | longest lane << 16
//     4..19  vectors per lane, 16 bits each, lane 0 in the low half of word 4
//     20..   reduce points, 16 bits each: vector index after which eight more slots are reduced
//
// Split-K partial sums go to a scratch buffer [k_splits][rows][columns] fp32 (int32 for int8 activations); the
// last block to finish a column block adds them in split order, applies the scale and writes Y.
#pragma once
#include <cstdint>
#include <vector>

#include "bittile_format.h"

#define BS_TILE_ROWS 4096
#define BS_GROUPS 128             // row groups of 32 rows in a tile
#define BS_NULL_ID 128            // the id that reads the all-zero row group
#define BS_TABLE_GROUPS 129       // row groups of a tile's activation table
#define BS_IDS_PER_VEC 15
#define BS_WARPS 8                // warps of a thread block
#define BS_RING_SLOTS 16          // slots of a warp's ring of lane cells
#define BS_BATCH_SLOTS 8          // slots reduced at one reduce point (four columns)
#define BS_MAX_UNIT_COLS 2048      // columns of one unit (a lane's vector count must fit 16 bits)
#define BS_MAX_META_BYTES (16 * 1024)
#define BS_MAX_CELLS 2048         // (tiles of a block) * (columns of a block): per-(tile, column) sums in shared memory
#define BS_MAX_BLOCKS 8192        // blocks of one launch
#define BS_MAX_PARAM_BLOCKS 160   // block descriptors that travel in kernel parameters; the rest are read from memory
#define BS_BLOCK_HEADER 8
#define BS_UNIT_HEADER 20

struct TsCtaDesc {
    uint32_t stream_off;   // first vector of this block's range (units of 16 B), multiple of 32
    uint32_t nvec;         // vectors in the range, multiple of 32
    uint32_t meta_off;     // first uint32 of this block's table (multiple of 4)
    uint32_t meta_words;   // uint32 in the table, padded to a multiple of 4
};

struct BsLayout {
    int inners = 0, columns = 0;
    int tile_rows = 0;           // rows of a K-tile: a multiple of 32, at most BS_TILE_ROWS (smaller tiles exist for tests)
    int tiles = 0;               // ceil(inners / tile_rows)
    int col_blocks = 0;          // column ranges; block id = j * col_blocks + b
    int k_splits = 0;            // tile ranges
    int tiles_per_cta = 0;
    int num_ctas = 0;
    int max_cols_per_block = 0;
    int64_t nnz = 0;
    int64_t total_vecs = 0;
    int64_t units = 0;
    std::vector<int32_t> col_start;   // col_blocks + 1 : first column of every column block
    std::vector<TsCtaDesc> cta;       // num_ctas descriptors
};

struct BsHostImage {
    BsLayout lay;
    std::vector<uint8_t> stream;    // total_vecs * 16 bytes
    std::vector<uint32_t> meta;     // concatenated block tables
};

struct tllm_pack_opts;

// Builds the image from a dense ternary matrix (int8 [inners][columns]); returns nullptr or an error message.
const char* bs_pack_dense(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms, BsHostImage* out);
// Inverse, for tests of the packer alone.  The image must have passed bs_validate.
void bs_unpack_dense(const BsHostImage& img, int8_t* w);
// Checks every invariant the kernel relies on (ranges, alignments, list counts, ring bound, reduce points);
// returns nullptr or a message.  Safe on arbitrary input: nothing is dereferenced before it is bounded.
const char* bs_validate(const BsHostImage& img);
