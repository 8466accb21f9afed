// packer.cpp -- host-side format work: the reference's three packers behind the C ABI, decoders for every
// reference weight format, the ternarizer and the bit-tile packer (the bank-stream packer is bstream_pack.cpp).
//
// Replaces ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:9-315 (convert_to_ter_csc, convert_to_ter_tiled_csc,
// convert_to_ter_tiled_mcsc, inter_tile_swizzle) and consumes what ternaryLLM_CPU/src/TCSC.hpp:6-409
// (SparseFormat, MergedTCSC, MergedTCSC_Group) produce.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <string>
#include <thread>
#include <vector>

#include "../../include/tllm.h"
#include "column_lists.h"
#include "bstream_format.h"
#include "nibble_format.h"
#include "util.h"

namespace {

using tllm::ColumnLists;

inline int tiles_of(int inners, int tile) { return (inners + tile - 1) / tile; }

bool ternary_only(const int32_t* w, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (w[i] < -1 || w[i] > 1) return false;
    return true;
}

}  // namespace

extern "C" {

int tllm_count_nnz(const int32_t* w, int columns, int inners, int64_t* cnt_pos, int64_t* cnt_neg) {
    if (!w || columns <= 0 || inners <= 0 || !cnt_pos || !cnt_neg) return tllm::fail(TLLM_ERR_ARG, "tllm_count_nnz: bad argument");
    int64_t p = 0, q = 0;
    const size_t total = (size_t)columns * inners;
    for (size_t i = 0; i < total; ++i) {
        p += w[i] == 1;
        q += w[i] == -1;
    }
    *cnt_pos = p;
    *cnt_neg = q;
    return TLLM_OK;
}

int tllm_convert_to_ter_csc(const int32_t* w, int columns, int inners, int32_t* neg_idx, int32_t* neg_off,
                            int32_t* pos_idx, int32_t* pos_off) {
    if (!w || columns <= 0 || inners <= 0 || !neg_off || !pos_off)
        return tllm::fail(TLLM_ERR_ARG, "tllm_convert_to_ter_csc: bad argument");
    ColumnLists<int32_t> cl(w, inners, columns);
    for (int n = 0; n <= columns; ++n) {
        neg_off[n] = (int32_t)cl.neg_ptr[n];
        pos_off[n] = (int32_t)cl.pos_ptr[n];
    }
    if (!cl.neg_row.empty()) std::memcpy(neg_idx, cl.neg_row.data(), cl.neg_row.size() * sizeof(int32_t));
    if (!cl.pos_row.empty()) std::memcpy(pos_idx, cl.pos_row.data(), cl.pos_row.size() * sizeof(int32_t));
    return TLLM_OK;
}

int tllm_convert_to_ter_tiled_csc(const int32_t* w, int columns, int inners, int tile_k, int32_t* neg_idx,
                                  int32_t* neg_off, int32_t* pos_idx, int32_t* pos_off) {
    if (!w || columns <= 0 || inners <= 0 || tile_k <= 0 || !neg_off || !pos_off)
        return tllm::fail(TLLM_ERR_ARG, "tllm_convert_to_ter_tiled_csc: bad argument");
    ColumnLists<int32_t> cl(w, inners, columns);
    const int tiles = tiles_of(inners, tile_k);
    auto emit = [&](const std::vector<int64_t>& ptr, const std::vector<int32_t>& rows, int32_t* idx, int32_t* off) {
        for (int n = 0; n < columns; ++n) {
            int64_t cur = ptr[n];
            for (int t = 0; t < tiles; ++t) {
                const int hi = (t + 1) * tile_k;
                off[((size_t)n * tiles + t) * 2] = (int32_t)cur;
                while (cur < ptr[n + 1] && rows[cur] < hi) {
                    idx[cur] = rows[cur] - t * tile_k;
                    ++cur;
                }
                off[((size_t)n * tiles + t) * 2 + 1] = (int32_t)cur;
            }
        }
    };
    emit(cl.neg_ptr, cl.neg_row, neg_idx, neg_off);
    emit(cl.pos_ptr, cl.pos_row, pos_idx, pos_off);
    return TLLM_OK;
}

}  // extern "C"

namespace {

// Shared walk for the merged tiled CSC: calls f(column, tile, pos ids, npos, neg ids, nneg) with
// tile-local ids.
template <typename F>
void for_each_tile_list(const ColumnLists<int32_t>& cl, int columns, int inners, int tile_k, F&& f) {
    const int tiles = tiles_of(inners, tile_k);
    std::vector<int32_t> p, q;
    for (int n = 0; n < columns; ++n) {
        int64_t pc = cl.pos_ptr[n], nc = cl.neg_ptr[n];
        for (int t = 0; t < tiles; ++t) {
            const int lo = t * tile_k, hi = lo + tile_k;
            p.clear();
            q.clear();
            while (pc < cl.pos_ptr[n + 1] && cl.pos_row[pc] < hi) p.push_back(cl.pos_row[pc++] - lo);
            while (nc < cl.neg_ptr[n + 1] && cl.neg_row[nc] < hi) q.push_back(cl.neg_row[nc++] - lo);
            f(n, t, p, q);
        }
    }
}

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

// Lengths (pair region, remainder region, both as stored) of one (column, tile) list.
struct McscLen {
    int pair_stored, rem_stored, pair_off, rem_off;   // *_off: what the offsets advertise
};
McscLen mcsc_len(int npos, int nneg, int padding, int padding_size, int mode) {
    const int mn = std::min(npos, nneg), mx = std::max(npos, nneg);
    McscLen L;
    int pair = 2 * mn, rem = mx - mn;
    if (mode == 0) {
        L.pair_stored = L.pair_off = padding ? round_up(pair, padding_size) : pair;
        L.rem_stored = L.rem_off = rem;
        return L;
    }
    // reference-compatible: storage is padded, advertised lengths are cut to multiples of four
    const int pair_pad = padding ? round_up(pair, padding_size) : pair;
    const int rem_pad = padding ? round_up(rem, padding_size) : rem;
    if (rem & 1) --rem;
    if (pair % 4) pair -= 2;
    if (rem % 4) rem -= 2;
    L.pair_stored = pair_pad;
    L.rem_stored = rem_pad;
    L.pair_off = padding ? pair_pad : pair;
    L.rem_off = rem;
    if (!padding) {   // without padding the next list starts right behind the advertised end
        L.pair_stored = pair;
        L.rem_stored = rem;
    }
    return L;
}

}  // namespace

extern "C" {

int64_t tllm_ter_tiled_mcsc_len(const int32_t* w, int columns, int inners, int tile_k, int padding,
                                int padding_size, int mode) {
    if (!w || columns <= 0 || inners <= 0 || tile_k <= 0 || (padding && padding_size <= 0) || mode < 0 || mode > 1)
        return tllm::fail(TLLM_ERR_ARG, "tllm_ter_tiled_mcsc_len: bad argument");
    ColumnLists<int32_t> cl(w, inners, columns);
    int64_t total = 0, true_nnz = cl.pos_row.size() + cl.neg_row.size();
    for_each_tile_list(cl, columns, inners, tile_k, [&](int, int, const std::vector<int32_t>& p, const std::vector<int32_t>& q) {
        const McscLen L = mcsc_len((int)p.size(), (int)q.size(), padding, padding_size, mode);
        total += L.pair_stored + L.rem_stored;
    });
    // the reference's vector is cnt_pos+cnt_neg long without padding even though truncation makes the
    // advertised lists shorter; keep that length so that buffers have the reference's shape
    if (mode == 1 && !padding) total = true_nnz;
    return total;
}

int tllm_convert_to_ter_tiled_mcsc(const int32_t* w, int columns, int inners, int tile_k, int padding,
                                   int padding_size, int mode, int32_t* row_idx, int64_t row_idx_cap,
                                   int32_t* off, int32_t* tile_idx) {
    if (!w || columns <= 0 || inners <= 0 || tile_k <= 0 || !row_idx || !off || (padding && padding_size <= 0) ||
        mode < 0 || mode > 1)
        return tllm::fail(TLLM_ERR_ARG, "tllm_convert_to_ter_tiled_mcsc: bad argument");
    ColumnLists<int32_t> cl(w, inners, columns);
    const int tiles = tiles_of(inners, tile_k);
    std::fill(row_idx, row_idx + row_idx_cap, 0);
    int64_t cursor = 0;
    bool overflow = false;
    // mode 1 needs "the first positive id at or after this tile in the flattened positive list" for its
    // padding value, which may belong to a later tile or column when this tile has no positive entry
    std::vector<int32_t> flat_pos_local;
    std::vector<int64_t> flat_pos_start;
    if (mode == 1 && padding) {
        flat_pos_start.reserve((size_t)columns * tiles);
        for_each_tile_list(cl, columns, inners, tile_k, [&](int, int, const std::vector<int32_t>& p, const std::vector<int32_t>&) {
            flat_pos_start.push_back((int64_t)flat_pos_local.size());
            flat_pos_local.insert(flat_pos_local.end(), p.begin(), p.end());
        });
    }
    size_t list_no = 0;
    for_each_tile_list(cl, columns, inners, tile_k, [&](int n, int t, const std::vector<int32_t>& p, const std::vector<int32_t>& q) {
        const int npos = (int)p.size(), nneg = (int)q.size();
        const int mn = std::min(npos, nneg), mx = std::max(npos, nneg);
        const bool pos_left = nneg <= npos;
        const McscLen L = mcsc_len(npos, nneg, padding, padding_size, mode);
        auto put = [&](int64_t at, int32_t v) {
            if (at >= 0 && at < row_idx_cap) row_idx[at] = v;
            else overflow = overflow || mode == 0;
        };
        for (int i = 0; i < mn; ++i) {
            put(cursor + 2 * i, p[i]);
            put(cursor + 2 * i + 1, q[i]);
        }
        int32_t pad_id = 0;
        if (mode == 0) pad_id = npos ? p[0] : (nneg ? q[0] : 0);
        else if (padding) {
            const int64_t at = flat_pos_start[list_no];
            pad_id = at < (int64_t)flat_pos_local.size() ? flat_pos_local[at] : 0;
        }
        const int pair_pad_end = padding ? round_up(2 * mn, padding_size) : 2 * mn;
        for (int i = 2 * mn; i < pair_pad_end; ++i) put(cursor + i, pad_id);
        // remainder: mode 0 stores it behind the padded pair region; the reference stores it behind the
        // UNPADDED pair region (so it lands inside the padding) while its offsets point past the padding
        const int64_t rem_at = cursor + (mode == 0 ? pair_pad_end : 2 * mn);
        const std::vector<int32_t>& src = pos_left ? p : q;
        for (int i = mn; i < mx; ++i) put(rem_at + (i - mn), src[i]);
        int32_t* o = off + ((size_t)n * tiles + t) * 4;
        o[0] = (int32_t)cursor;
        o[1] = (int32_t)(cursor + L.pair_off);
        o[2] = (int32_t)(cursor + L.pair_off + L.rem_off);
        o[3] = pos_left ? 1 : -1;
        cursor += L.pair_stored + L.rem_stored;
        ++list_no;
    });
    if (overflow) return tllm::fail(TLLM_ERR_ARG, "tllm_convert_to_ter_tiled_mcsc: row_idx_cap too small");
    if (tile_idx) {
        // per column: tile ids ordered by advertised list length, shortest first
        std::vector<int> order(tiles);
        for (int n = 0; n < columns; ++n) {
            std::iota(order.begin(), order.end(), 0);
            const int32_t* o = off + (size_t)n * tiles * 4;
            std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return o[a * 4 + 2] - o[a * 4] < o[b * 4 + 2] - o[b * 4]; });
            for (int t = 0; t < tiles; ++t) tile_idx[(size_t)n * tiles + t] = order[t];
        }
    }
    return TLLM_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------------
// Decoders: any reference format -> dense int8 [inners][columns].  References to the same (row, column)
// with opposite signs cancel, which is how the reference's kernels treat its (a,a) padding pairs.
// ------------------------------------------------------------------------------------------------------
namespace tllm {

static inline bool bump(std::vector<int8_t>& w, int64_t row, int col, int sign, int inners, int columns) {
    if (row < 0 || row >= inners || col < 0 || col >= columns) return false;
    int8_t& e = w[(size_t)row * columns + col];
    e = (int8_t)(e + sign);
    return true;
}

const char* decode_mcsc(const int32_t* row_idx, const int32_t* off, int columns, int inners, int tile_k,
                        std::vector<int8_t>* out) {
    const int tiles = tiles_of(inners, tile_k);
    out->assign((size_t)inners * columns, 0);
    for (int n = 0; n < columns; ++n)
        for (int t = 0; t < tiles; ++t) {
            const int32_t* o = off + ((size_t)n * tiles + t) * 4;
            if (o[0] < 0 || o[1] < o[0] || o[2] < o[1] || (o[3] != 1 && o[3] != -1)) return "merged tiled CSC: malformed offsets";
            const int base = t * tile_k;
            for (int i = o[0]; i + 1 < o[1]; i += 2) {
                if (row_idx[i] < 0 || row_idx[i] >= tile_k || row_idx[i + 1] < 0 || row_idx[i + 1] >= tile_k)
                    return "merged tiled CSC: row id outside its tile";
                if (!bump(*out, base + row_idx[i], n, +1, inners, columns)) return "merged tiled CSC: row id past K";
                if (!bump(*out, base + row_idx[i + 1], n, -1, inners, columns)) return "merged tiled CSC: row id past K";
            }
            for (int i = o[1]; i < o[2]; ++i) {
                if (row_idx[i] < 0 || row_idx[i] >= tile_k) return "merged tiled CSC: row id outside its tile";
                if (!bump(*out, base + row_idx[i], n, o[3], inners, columns)) return "merged tiled CSC: row id past K";
            }
        }
    for (int8_t v : *out)
        if (v < -1 || v > 1) return "merged tiled CSC: an entry is referenced more than once with the same sign";
    return nullptr;
}

const char* decode_cpu_format(int kind, int group, int chunk, const int32_t* meta, const void* ri, int ri32,
                              int64_t aux, int columns, int inners, std::vector<int8_t>* out) {
    out->assign((size_t)inners * columns, 0);
    auto id = [&](int64_t i) -> int64_t { return ri32 ? ((const int32_t*)ri)[i] : ((const int16_t*)ri)[i]; };
    auto add = [&](int64_t i, int col, int sign) { return bump(*out, id(i), col, sign, inners, columns); };
    const char* bad = "CPU format: row id out of range";
    if (kind == 0) {   // SparseFormat: two offset arrays, two id arrays
        const int32_t* cneg = meta;
        const int32_t* cpos = meta + columns + 1;
        for (int n = 0; n < columns; ++n) {
            for (int64_t i = cneg[n]; i < cneg[n + 1]; ++i)
                if (!add(i, n, -1)) return bad;
            for (int64_t i = cpos[n]; i < cpos[n + 1]; ++i)
                if (!add(aux + i, n, +1)) return bad;
        }
    } else if (kind == 1) {   // MergedTCSC: {pair_start, pair_end, rem_end, rem_sign} per column
        for (int n = 0; n < columns; ++n) {
            const int32_t* m = meta + (size_t)n * 4;
            for (int64_t i = m[0]; i + 1 < m[1]; i += 2)
                if (!add(i, n, +1) || !add(i + 1, n, -1)) return bad;
            for (int64_t i = m[1]; i < m[2]; ++i)
                if (m[3] && !add(i, n, m[3])) return bad;
        }
    } else if (kind >= 2 && kind <= 5) {
        if (group <= 0 || columns % group) return "CPU format: columns must be a multiple of the group size";
        if (chunk < 0 || (chunk && group % chunk)) return "CPU format: chunk must divide the group size";
        const int per_group = kind == 4 ? 2 : (kind == 5 ? 0 : 2 + 2 * group);
        for (int g = 0; g < columns / group; ++g) {
            const int32_t* m = meta + (size_t)g * per_group;
            int64_t beg, end;
            if (kind == 5) {
                beg = (int64_t)g * group * meta[0];
                end = beg + (int64_t)group * meta[0];
            } else {
                beg = m[0];
                end = m[1];
            }
            const int col0 = g * group;
            for (int64_t k = beg; k < end; k += 2 * group) {
                if (chunk == 0) {
                    for (int i = 0; i < group; ++i)
                        if (!add(k + 2 * i, col0 + i, +1) || !add(k + 2 * i + 1, col0 + i, -1)) return bad;
                } else {
                    for (int c = 0; c < group; c += chunk)
                        for (int i = 0; i < chunk; ++i)
                            if (!add(k + 2 * c + i, col0 + c + i, +1) || !add(k + 2 * c + chunk + i, col0 + c + i, -1)) return bad;
                }
            }
            if (kind == 2) {          // per column: rest of the +1 ids, then rest of the -1 ids
                int64_t prev = m[1];
                for (int i = 0; i < group; ++i) {
                    for (int64_t k = prev; k < m[2 + 2 * i]; ++k)
                        if (!add(k, col0 + i, +1)) return bad;
                    for (int64_t k = m[2 + 2 * i]; k < m[3 + 2 * i]; ++k)
                        if (!add(k, col0 + i, -1)) return bad;
                    prev = m[3 + 2 * i];
                }
            } else if (kind == 3) {   // per column: one remainder list with its sign
                int64_t prev = m[1];
                for (int i = 0; i < group; ++i) {
                    for (int64_t k = prev; k < m[2 + 2 * i]; ++k)
                        if (!add(k, col0 + i, m[3 + 2 * i])) return bad;
                    prev = m[2 + 2 * i];
                }
            }
        }
    } else {
        return "CPU format: unknown kind";
    }
    for (int8_t v : *out)
        if (v < -1 || v > 1) return "CPU format: an entry is referenced more than once with the same sign";
    return nullptr;
}

}  // namespace tllm

// ---------------------------------------------------------------------------------------------------
// float weights -> ternary weights + per-tensor scale (the reference's ternarize_weights is a stub that raises,
// ternaryLLM_GPU/TernaryLLM/TernaryLinear.py:19-20; this is the threshold rule of ternary weight networks)
// ---------------------------------------------------------------------------------------------------
extern "C" int tllm_ternarize(const float* w, int inners, int columns, float threshold_factor, float target_sparsity, int8_t* out,
                              float* scale) {
    if (!w || !out || inners <= 0 || columns <= 0) return tllm::fail(TLLM_ERR_ARG, "tllm_ternarize: bad argument");
    if (target_sparsity >= 1.f) return tllm::fail(TLLM_ERR_ARG, "tllm_ternarize: target_sparsity must be below 1");
    const size_t n = (size_t)inners * columns;
    double thr;
    if (target_sparsity > 0.f) {
        // zero the k smallest magnitudes: the threshold is the k-th smallest |w| (ties at the threshold are zeroed too)
        const size_t k = (size_t)std::llround((double)target_sparsity * (double)n);
        if (k == 0) thr = -1.0;
        else {
            std::vector<float> mag(n);
            for (size_t i = 0; i < n; ++i) mag[i] = std::fabs(w[i]);
            std::nth_element(mag.begin(), mag.begin() + (k - 1), mag.end());
            thr = mag[k - 1];
        }
    } else {
        double sum = 0.0;
        for (size_t i = 0; i < n; ++i) sum += std::fabs((double)w[i]);
        thr = (double)(threshold_factor > 0.f ? threshold_factor : 0.7f) * (sum / (double)n);
    }
    double kept = 0.0;
    size_t cnt = 0;
    for (size_t i = 0; i < n; ++i) {
        const double a = std::fabs((double)w[i]);
        if (a > thr) {
            out[i] = w[i] > 0.f ? 1 : -1;
            kept += a;
            ++cnt;
        } else out[i] = 0;
    }
    if (scale) *scale = cnt ? (float)(kept / (double)cnt) : 0.f;     // least-squares scale for the kept entries
    return TLLM_OK;
}

// ---------------------------------------------------------------------------------------------------
// bit tiles: the dense two-bit copy the tensor-core kernel reads (layout: tstream_format.h)
// ---------------------------------------------------------------------------------------------------
void mm_pack_bits(const int8_t* w, int inners, int columns, std::vector<uint32_t>* bits, int* n_tiles, int* kb_out) {
    const int NT = (columns + 127) / 128, KB = (inners + 63) / 64;
    bits->assign((size_t)NT * KB * 128 * 4, 0u);
    for (int kb = 0; kb < KB; ++kb) {
        const int k1 = std::min(inners, (kb + 1) * 64);
        for (int k = kb * 64; k < k1; ++k) {
            const int kl = k - kb * 64, word = kl >> 4, bit = mm_code_bit(kl & 15);
            const int8_t* row = w + (size_t)k * columns;
            for (int n = 0; n < columns; ++n) {
                const int8_t v = row[n];
                if (!v) continue;
                const size_t rec = ((size_t)(n >> 7) * KB + kb) * 128 + (n & 127);
                (*bits)[rec * 4 + word] |= (v > 0 ? 1u : 2u) << bit;
            }
        }
    }
    *n_tiles = NT;
    *kb_out = KB;
}

void mm_unpack_bits(const std::vector<uint32_t>& bits, int inners, int columns, int8_t* w) {
    const int KB = (inners + 63) / 64;
    for (int k = 0; k < inners; ++k) {
        const int kb = k >> 6, kl = k & 63, word = kl >> 4, bit = mm_code_bit(kl & 15);
        for (int n = 0; n < columns; ++n) {
            const size_t rec = ((size_t)(n >> 7) * KB + kb) * 128 + (n & 127);
            const uint32_t c = (bits[rec * 4 + word] >> bit) & 3u;
            w[(size_t)k * columns + n] = c == 1 ? 1 : c == 2 ? -1 : 0;
        }
    }
}

namespace tllm {
void bs_fill_info(const BsLayout& L, tllm_weight_info* info);
}

extern "C" int tllm_pack_roundtrip(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                                   int8_t* w_out, tllm_weight_info* info) {
    if (!w || !w_out || inners <= 0 || columns <= 0 || num_sms <= 0) return tllm::fail(TLLM_ERR_ARG, "tllm_pack_roundtrip: bad argument");
    BsHostImage img;
    const char* msg = bs_pack_dense(w, inners, columns, opts, num_sms, &img);
    if (!msg) msg = bs_validate(img);
    if (msg) return tllm::fail(TLLM_ERR_ARG, "%s", msg);
    bs_unpack_dense(img, w_out);
    int64_t bit_bytes = 0;
    {   // the second representation must describe the same matrix
        std::vector<uint32_t> bits;
        int nt = 0, kb = 0;
        mm_pack_bits(w, inners, columns, &bits, &nt, &kb);
        std::vector<int8_t> back((size_t)inners * columns);
        mm_unpack_bits(bits, inners, columns, back.data());
        if (std::memcmp(back.data(), w, back.size()) != 0) return tllm::fail(TLLM_ERR_ARG, "bit tiles do not reproduce the matrix");
        bit_bytes = (int64_t)bits.size() * 4;
    }
    int64_t nibble_bytes = 0;
    {   // and so must the third
        NbHostImage nb;
        nb_pack_dense(w, inners, columns, &nb);
        std::vector<int8_t> back((size_t)inners * columns);
        if (!nb_unpack_dense(nb, back.data()) || std::memcmp(back.data(), w, back.size()) != 0)
            return tllm::fail(TLLM_ERR_ARG, "nibble planes do not reproduce the matrix");
        nibble_bytes = (int64_t)nb.codes.size();
    }
    if (info) {
        std::memset(info, 0, sizeof *info);
        tllm::bs_fill_info(img.lay, info);
        info->bit_tile_bytes = bit_bytes;
        info->nibble_bytes = nibble_bytes;
        info->stream_bytes = (int64_t)img.stream.size();
        info->meta_bytes = (int64_t)img.meta.size() * 4;
    }
    return TLLM_OK;
}

// Host-side check of a packed image given as raw arrays (what a packed-weight file holds): used by tests to show
// that damaged images are refused before anything is uploaded.
extern "C" int tllm_pack_corrupt_check(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms, int what, int64_t where,
                                       uint32_t value) {
    if (!w || inners <= 0 || columns <= 0 || num_sms <= 0) return tllm::fail(TLLM_ERR_ARG, "tllm_pack_corrupt_check: bad argument");
    BsHostImage img;
    const char* msg = bs_pack_dense(w, inners, columns, opts, num_sms, &img);
    if (!msg) msg = bs_validate(img);
    if (msg) return tllm::fail(TLLM_ERR_ARG, "%s", msg);
    BsLayout& L = img.lay;
    switch (what) {
        case 0: break;   // untouched: must validate
        case 1: if (where >= 0 && (size_t)where < img.meta.size()) img.meta[(size_t)where] = value; break;
        case 2: if (where >= 0 && (size_t)where < img.stream.size()) img.stream[(size_t)where] = (uint8_t)value; break;
        case 3: L.tile_rows = (int)value; break;
        case 4: L.tiles = (int)value; break;
        case 5: L.col_blocks = (int)value; break;
        case 6: L.k_splits = (int)value; break;
        case 7: L.tiles_per_cta = (int)value; break;
        case 8: if (where >= 0 && (size_t)where < L.cta.size()) L.cta[(size_t)where].meta_words = value; break;
        case 9: if (where >= 0 && (size_t)where < L.cta.size()) L.cta[(size_t)where].stream_off = value; break;
        case 10: if (where >= 0 && (size_t)where < L.col_start.size()) L.col_start[(size_t)where] = (int32_t)value; break;
        case 11: L.inners = (int)value; break;
        case 12: if (where >= 0 && (size_t)where < L.cta.size()) L.cta[(size_t)where].meta_off = value; break;
        case 13: if (where >= 0 && (size_t)where < L.cta.size()) L.cta[(size_t)where].nvec = value; break;
        default: return tllm::fail(TLLM_ERR_ARG, "tllm_pack_corrupt_check: unknown field");
    }
    msg = bs_validate(img);
    if (msg) return tllm::fail(TLLM_ERR_ARG, "%s", msg);
    return TLLM_OK;
}

// ---------------------------------------------------------------------------------------------------
// nibble planes: the transposed four-bit copy the decode tensor-core kernel reads (layout: nibble_format.h)
// ---------------------------------------------------------------------------------------------------
void nb_pack_dense(const int8_t* w, int inners, int columns, NbHostImage* out) {
    out->inners = inners, out->columns = columns;
    out->k_pad = (inners + 127) / 128 * 128, out->n_pad = (columns + 127) / 128 * 128;
    const size_t pitch = (size_t)out->k_pad / 2;
    out->codes.assign((size_t)out->n_pad * pitch, 0);
    const int tiles = out->n_pad / 128;
    std::atomic<int> next{0};
    // one column tile at a time: its 128 rows of the image are private to the thread that builds it
    auto work = [&]() {
        for (;;) {
            const int t = next.fetch_add(1);
            if (t >= tiles) return;
            const int n0 = t * 128, n1 = std::min(columns, n0 + 128);
            uint8_t* base = out->codes.data() + (size_t)n0 * pitch;
            for (int k = 0; k < inners; ++k) {
                const int8_t* row = w + (size_t)k * columns;
                const int shift = (k & 1) * 4;
                uint8_t* dst = base + (k >> 1);
                for (int n = n0; n < n1; ++n) {
                    const int8_t v = row[n];
                    if (v) dst[(size_t)(n - n0) * pitch] |= (uint8_t)((v > 0 ? NB_CODE_POS : NB_CODE_NEG) << shift);
                }
            }
        }
    };
    unsigned nthreads = std::max(1u, std::min(std::thread::hardware_concurrency(), 32u));
    nthreads = std::min<unsigned>(nthreads, (unsigned)tiles);
    std::vector<std::thread> pool;
    for (unsigned i = 1; i < nthreads; ++i) pool.emplace_back(work);
    work();
    for (std::thread& th : pool) th.join();
}

bool nb_unpack_dense(const NbHostImage& img, int8_t* w) {
    const size_t pitch = (size_t)img.k_pad / 2;
    for (int n = 0; n < img.n_pad; ++n)
        for (int k = 0; k < img.k_pad; ++k) {
            const uint32_t c = (img.codes[(size_t)n * pitch + (k >> 1)] >> ((k & 1) * 4)) & 0xFu;
            if (c != 0 && c != NB_CODE_POS && c != NB_CODE_NEG) return false;
            if (n >= img.columns || k >= img.inners) {
                if (c) return false;
                continue;
            }
            w[(size_t)k * img.columns + n] = c == 0 ? 0 : (c == NB_CODE_POS ? 1 : -1);
        }
    return true;
}

void nb_make_schedule(int k_pad, int n_pad, int sms, NbSchedule* out) {
    NbSchedule& s = *out;
    s.uk = NB_FMT_UK;
    s.kb = k_pad / NB_FMT_TILE;
    s.tiles = n_pad / NB_FMT_TILE;
    // ranges of at most NB_FMT_MAX_KBS blocks, as even as they come
    s.splits = (s.kb + NB_FMT_MAX_KBS - 1) / NB_FMT_MAX_KBS;
    s.kbs = (s.kb + s.splits - 1) / s.splits;
    s.splits = (s.kb + s.kbs - 1) / s.kbs;
    // every range the same number of thread blocks, one thread block per SM in all, never more than the last (shortest) range has units
    const int last_ku = (s.kb - (s.splits - 1) * s.kbs + s.uk - 1) / s.uk;
    long long gj = (long long)sms / s.splits;
    if (gj < 1) gj = 1;
    if (gj > (long long)s.tiles * last_ku) gj = (long long)s.tiles * last_ku;
    if (gj > 0xFFFF) gj = 0xFFFF;                            // a run's ends are 16-bit fields
    s.gj = (int)gj;
    s.words.assign((size_t)(1 + s.splits) * s.tiles, 0u);
    for (int jj = 0; jj < s.splits; ++jj) {
        const long long kbn = std::min(s.kbs, s.kb - jj * s.kbs), kun = (kbn + s.uk - 1) / s.uk, tot = (long long)s.tiles * kun;
        for (int t = 0; t < s.tiles; ++t) {
            // the block that owns unit u is the largest c with tot * c / gj <= u, that is ceil((u + 1) * gj / tot) - 1
            const long long fu = (long long)t * kun, lu = fu + kun - 1;
            const long long cf = ((fu + 1) * gj + tot - 1) / tot - 1, cl = ((lu + 1) * gj + tot - 1) / tot - 1;
            s.words[(size_t)t] += (uint32_t)(cl - cf + 1);
            s.words[(size_t)(1 + jj) * s.tiles + t] = (uint32_t)cf | ((uint32_t)cl << 16);
        }
    }
}

extern "C" int tllm_nibble_schedule(int inners, int columns, int num_sms, int* dims, uint32_t* words, size_t capacity_words) {
    if (inners <= 0 || columns <= 0 || num_sms <= 0 || !dims) return tllm::fail(TLLM_ERR_ARG, "tllm_nibble_schedule: bad argument");
    NbSchedule s;
    nb_make_schedule((inners + NB_FMT_TILE - 1) / NB_FMT_TILE * NB_FMT_TILE, (columns + NB_FMT_TILE - 1) / NB_FMT_TILE * NB_FMT_TILE, num_sms, &s);
    dims[0] = s.kb, dims[1] = s.tiles, dims[2] = s.kbs, dims[3] = s.splits, dims[4] = s.gj, dims[5] = s.uk;
    if (!words) return TLLM_OK;
    if (capacity_words < s.words.size()) return tllm::fail(TLLM_ERR_ARG, "tllm_nibble_schedule: %zu words needed, %zu given", s.words.size(), capacity_words);
    std::memcpy(words, s.words.data(), s.words.size() * sizeof(uint32_t));
    return TLLM_OK;
}
