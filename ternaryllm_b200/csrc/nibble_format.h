// nibble_format.h -- "nibble planes": the transpose of W at four bits per entry, the copy of the weight that
// nibble_kernel.cuh streams straight into the tensor cores.
//
// Row n of the image is column n of W: k_pad / 2 bytes, entry k in nibble (k & 1) of byte k / 2 (low nibble first).
// A code is the fp4 (e2m1) bit pattern of the entry: 0x0 = 0, 0x2 = +1.0, 0xA = -1.0.  k_pad and n_pad are K and N
// rounded up to multiples of 128 (one tensor-map box is 128 x 128 entries); the padding holds zeros.  Size: half a
// byte per entry whatever the sparsity -- less than the reference's two bytes per non-zero
// (ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:156-315) wherever fewer than three entries in four are zero.
#pragma once
#include <cstdint>
#include <vector>

#define NB_CODE_POS 0x2u
#define NB_CODE_NEG 0xAu

struct NbHostImage {
    int inners = 0, columns = 0;
    int k_pad = 0, n_pad = 0;
    std::vector<uint8_t> codes;   // n_pad * k_pad / 2 bytes
};

void nb_pack_dense(const int8_t* w, int inners, int columns, NbHostImage* out);
// inverse, for tests of the packer alone; returns false on a code that is none of the three
bool nb_unpack_dense(const NbHostImage& img, int8_t* w);

// How the grid of nibble_spmm_kernel shares the work.  The K blocks (128 rows of W each) are cut into `splits` ranges
// of up to `kbs` blocks (a block of threads keeps the activation pieces of one range in shared memory); a unit is `uk`
// consecutive K blocks of one column tile; the units of a range, tile-major, are dealt out in equal contiguous runs to
// `gj` thread blocks (block c of a range owns units [total * c / gj, total * (c + 1) / gj)), never more blocks than the
// shortest range has units.  A column tile whose units lie in several thread blocks is added up by the last of them
// to arrive, which has to know who the others are:
//   words[t]                    how many thread blocks (all ranges) hold a part of column tile t
//   words[(1 + j) * tiles + t]  first | last << 16: the run of blocks of range j that hold a part of tile t
#define NB_FMT_TILE 128
#define NB_FMT_MAX_KBS 32
#define NB_FMT_UK 2
struct NbSchedule {
    int kb = 0, tiles = 0, kbs = 0, splits = 0, gj = 0, uk = NB_FMT_UK;
    std::vector<uint32_t> words;
};
void nb_make_schedule(int k_pad, int n_pad, int sms, NbSchedule* out);
