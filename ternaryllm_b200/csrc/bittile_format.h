// bittile_format.h -- the dense two-bit copy of W that the tensor-core kernel reads ("bit tiles"), shared by
// the host packer and mma_kernel.cuh.
//
// For output-column tile nt (128 columns) and K-slice kb (64 rows): 128 consecutive 16-byte records, one per
// column, each holding 64 codes (0: zero, 1: +1, 2: -1).  Row k_local of the slice sits in 32-bit word
// k_local/16 at bit mm_code_bit(k_local%16); the positions are chosen so that one shift, one mask and one byte
// permute turn two codes into two fp16 / bf16 values.  The tiles of one column tile are contiguous along K.
#pragma once
#include <cstdint>
#include <vector>

inline int mm_code_bit(int kk) {            // kk = 0..15
    const int j = kk >> 1, h = kk & 1;       // output word (two values) and half within it
    return (j < 4 ? 2 * j : 16 + 2 * (j - 4)) + 8 * h;
}
void mm_pack_bits(const int8_t* w, int inners, int columns, std::vector<uint32_t>* bits, int* n_tiles, int* kb);
void mm_unpack_bits(const std::vector<uint32_t>& bits, int inners, int columns, int8_t* w);
