// packer.cpp -- host-side format work: the reference's three packers behind the C ABI, decoders for every
// reference weight format, and the packer of the library's own tile-stream format.
//
// Replaces ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:9-315 (convert_to_ter_csc, convert_to_ter_tiled_csc,
// convert_to_ter_tiled_mcsc, inter_tile_swizzle) and consumes what ternaryLLM_CPU/src/TCSC.hpp:6-409
// (SparseFormat, MergedTCSC, MergedTCSC_Group) produce.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <numeric>
#include <string>
#include <vector>

#include "../../include/tllm.h"
#include "tstream_format.h"
#include "util.h"

namespace {

inline int tiles_of(int inners, int tile) { return (inners + tile - 1) / tile; }

// Column-major view of a row-major ternary matrix: for every column the ascending row ids of the +1 and
// of the -1 entries.  Built with a counting pass and a scatter pass so that the matrix is read row by row.
template <typename WT>
struct ColumnLists {
    std::vector<int64_t> pos_ptr, neg_ptr;   // columns+1
    std::vector<int32_t> pos_row, neg_row;
    ColumnLists(const WT* w, int inners, int columns) : pos_ptr(columns + 1, 0), neg_ptr(columns + 1, 0) {
        for (int k = 0; k < inners; ++k) {
            const WT* row = w + (size_t)k * columns;
            for (int n = 0; n < columns; ++n) {
                pos_ptr[n + 1] += row[n] > 0;
                neg_ptr[n + 1] += row[n] < 0;
            }
        }
        for (int n = 0; n < columns; ++n) {
            pos_ptr[n + 1] += pos_ptr[n];
            neg_ptr[n + 1] += neg_ptr[n];
        }
        pos_row.resize(pos_ptr[columns]);
        neg_row.resize(neg_ptr[columns]);
        std::vector<int64_t> pc(pos_ptr.begin(), pos_ptr.end() - 1), nc(neg_ptr.begin(), neg_ptr.end() - 1);
        for (int k = 0; k < inners; ++k) {
            const WT* row = w + (size_t)k * columns;
            for (int n = 0; n < columns; ++n) {
                if (row[n] > 0) pos_row[pc[n]++] = k;
                else if (row[n] < 0) neg_row[nc[n]++] = k;
            }
        }
    }
};

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

// ------------------------------------------------------------------------------------------------------
// Tile-stream packer
// ------------------------------------------------------------------------------------------------------
namespace {

int pow2_ceil(int v) {
    int p = 1;
    while (p < v) p *= 2;
    return p;
}

struct ListRef {
    int col;        // column within the sub-block
    int sign;       // 0: +1 list, 1: -1 list
    const int32_t* first;
    int n;          // ids
    int nvec() const { return (n + TS_IDS_PER_VEC - 1) / TS_IDS_PER_VEC; }
};

// upper bound of the table words of one block (a list has at most tile_rows/8 + 1 vectors)
size_t meta_words_of(int ncols, int sub_cols, int T, int ntiles) {
    size_t words = 0;
    for (int c = 0; c < ncols; c += sub_cols) words += TS_SEC_HEADER + (size_t)(T / TS_IDS_PER_VEC + 2) + 2 * (size_t)std::min(sub_cols, ncols - c);
    return words * (size_t)ntiles;
}

}  // namespace

const char* ts_pack_dense(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                          TsHostImage* out) {
    if (!w || inners <= 0 || columns <= 0) return "pack: bad matrix shape";
    if ((int64_t)inners * columns > ((int64_t)1 << 40)) return "pack: matrix too large";
    tllm_pack_opts o{};
    if (opts) o = *opts;
    int T = o.tile_rows > 0 ? o.tile_rows : TS_MAX_TILE_ROWS;
    if (T > TS_MAX_TILE_ROWS || T % 8) return "pack: tile_rows must be a multiple of 8 and at most 1024";
    if (T > inners) T = (inners + 7) / 8 * 8;
    int ctas = o.num_ctas > 0 ? o.num_ctas : num_sms;
    if (ctas <= 0 || ctas > TS_MAX_CTAS) return "pack: num_ctas out of range";
    int lpl = o.lanes_per_list > 0 ? o.lanes_per_list : 1;   // 0: chosen below, once the column blocks are known
    if (lpl < 1 || lpl > 16 || (lpl & (lpl - 1))) return "pack: lanes_per_list must be 1, 2, 4, 8 or 16";
    const int tiles = tiles_of(inners, T);

    // ---- schedule: k_splits x col_blocks blocks, each block owns tiles_per_cta tiles of one column block
    int best_tpc = 0, best_nb = 1;
    double best_cost = 1e300;
    for (int tpc = 1; tpc <= tiles; ++tpc) {
        const int splits = (tiles + tpc - 1) / tpc;
        if (o.k_splits > 0 && tpc != (tiles + o.k_splits - 1) / o.k_splits) continue;
        // column blocks hold an even number of columns, so that (gate, up) column pairs never straddle one
        // (and, when wide enough, a multiple of 16 columns = 32 lists, so that no unit is left with idle lanes)
        auto cols_for = [&](int blocks) {
            const int c = (columns + blocks - 1) / blocks;
            return c >= 64 ? (c + 15) & ~15 : (c + 1) & ~1;
        };
        // one wave of blocks when the per-block section table fits its shared-memory budget; wide matrices
        // take several full waves instead
        for (int wv = 1; wv <= 64; ++wv) {
            int nb = std::min(ctas * wv / splits, (columns + 1) / 2);
            if (nb < 1) nb = 1;
            const int bc = cols_for(nb);
            if (meta_words_of(bc, std::min(bc, TS_MAX_SUB_COLS), T, tpc) * 4 + 16 > TS_MAX_META_BYTES && bc > 2) continue;
            nb = (columns + bc - 1) / bc;
            if ((int64_t)nb * splits > TS_MAX_BLOCKS) break;
            // time ~ waves * (work of the busiest block + one activation-table fill per tile it owns)
            // (a fill takes about as long as streaming the lists of 32 Ki matrix entries at 75 % sparsity)
            const double waves = (nb * splits + ctas - 1) / ctas;
            const double work = (double)tpc * bc * T;
            const double fill = (double)tpc * 32768.0;
            const double cost = waves * (work + fill);
            if (cost < best_cost) {
                best_cost = cost;
                best_tpc = tpc;
                best_nb = nb;
            }
            break;   // more waves of smaller blocks only add fills
        }
    }
    if (best_tpc == 0) return "pack: no schedule fits (matrix too wide for the block budget)";
    TsLayout& L = out->lay;
    L = TsLayout{};
    L.inners = inners;
    L.columns = columns;
    L.tile_rows = T;
    L.tiles = tiles;
    L.tiles_per_cta = best_tpc;
    L.k_splits = (tiles + best_tpc - 1) / best_tpc;
    {
        const int c = (columns + best_nb - 1) / best_nb;
        L.cols_per_block = c >= 64 ? (c + 15) & ~15 : (c + 1) & ~1;
    }
    L.col_blocks = (columns + L.cols_per_block - 1) / L.cols_per_block;
    L.num_ctas = L.col_blocks * L.k_splits;
    L.cta.assign((size_t)L.num_ctas, TsCtaDesc{});
    L.sub_cols = std::min(L.cols_per_block, TS_MAX_SUB_COLS);
    if (o.lanes_per_list <= 0) {
        // One lane per list keeps padding and shuffles lowest.  Narrow column blocks have too few lists to
        // fill the lanes of a unit or to give every warp a unit: there several lanes share a list.
        const int nlists = 2 * L.sub_cols;
        lpl = std::min(16, std::max(1, pow2_ceil((12 * 32 + nlists - 1) / nlists)));
    }
    L.lanes_per_list = lpl;

    ColumnLists<int8_t> cl(w, inners, columns);
    L.nnz = (int64_t)cl.pos_row.size() + (int64_t)cl.neg_row.size();

    out->stream.clear();
    out->meta.clear();
    std::vector<ListRef> lists;
    auto pad_vectors_to = [&](size_t mult) {
        while ((out->stream.size() / TS_IDS_PER_VEC) % mult) out->stream.insert(out->stream.end(), TS_IDS_PER_VEC, (uint16_t)T);
    };
    for (int j = 0; j < L.k_splits; ++j) {
        for (int b = 0; b < L.col_blocks; ++b) {
            const int cta = j * L.col_blocks + b;
            const int c0 = b * L.cols_per_block, c1 = std::min(columns, c0 + L.cols_per_block);
            const int t0 = j * L.tiles_per_cta, t1 = std::min(tiles, t0 + L.tiles_per_cta);
            while (out->meta.size() % 4) out->meta.push_back(0);
            pad_vectors_to(32);
            TsCtaDesc& d = L.cta[cta];
            d.stream_off = (uint32_t)(out->stream.size() / TS_IDS_PER_VEC);
            d.meta_off = (uint32_t)out->meta.size();
            const size_t base = out->stream.size();
            for (int t = t0; t < t1; ++t) {
                const int lo = t * T, hi = lo + T;
                for (int s0 = c0; s0 < c1; s0 += L.sub_cols) {
                    const int s1 = std::min(c1, s0 + L.sub_cols);
                    lists.clear();
                    for (int c = s0; c < s1; ++c)
                        for (int sg = 0; sg < 2; ++sg) {
                            const std::vector<int64_t>& ptr = sg ? cl.neg_ptr : cl.pos_ptr;
                            const std::vector<int32_t>& rows = sg ? cl.neg_row : cl.pos_row;
                            const int32_t* first = std::lower_bound(rows.data() + ptr[c], rows.data() + ptr[c + 1], lo);
                            const int32_t* last = std::lower_bound(first, rows.data() + ptr[c + 1], hi);
                            lists.push_back(ListRef{c - s0, sg, first, (int)(last - first)});
                        }
                    // longest first; ties keep column order, so the layout is a pure function of W
                    auto steps_of = [&](const ListRef& l) { return (l.nvec() + lpl - 1) / lpl; };
                    std::stable_sort(lists.begin(), lists.end(), [&](const ListRef& a, const ListRef& b2) { return steps_of(a) > steps_of(b2); });
                    const int nl = (int)lists.size();
                    const int ndiag = nl ? steps_of(lists[0]) : 0;
                    pad_vectors_to(32);
                    const size_t sec_base = out->stream.size();
                    out->meta.push_back((uint32_t)((sec_base - base) / TS_IDS_PER_VEC));
                    out->meta.push_back((uint32_t)ndiag);
                    out->meta.push_back((uint32_t)nl);
                    out->meta.push_back(0);
                    const size_t diag_words = out->meta.size();
                    out->meta.resize(diag_words + ndiag + 1);
                    int live = nl;   // lists that still have a vector in this diagonal: a prefix of the sorted order
                    for (int i = 0; i < ndiag; ++i) {
                        while (live > 0 && steps_of(lists[live - 1]) <= i) --live;
                        pad_vectors_to(8);
                        out->meta[diag_words + i] = (uint32_t)((out->stream.size() - sec_base) / TS_IDS_PER_VEC);
                        for (int l = 0; l < live; ++l)
                            for (int jj = 0; jj < lpl; ++jj) {
                                const int v = i * lpl + jj;
                                for (int e = 0; e < TS_IDS_PER_VEC; ++e) {
                                    const int at = v * TS_IDS_PER_VEC + e;
                                    out->stream.push_back(at < lists[l].n ? (uint16_t)(lists[l].first[at] - lo) : (uint16_t)T);
                                }
                            }
                    }
                    pad_vectors_to(8);
                    out->meta[diag_words + ndiag] = (uint32_t)((out->stream.size() - sec_base) / TS_IDS_PER_VEC);
                    for (const ListRef& l : lists)
                        out->meta.push_back((uint32_t)(l.col | (l.sign << 15)) | ((uint32_t)steps_of(l) << 16));
                }
            }
            pad_vectors_to(32);
            d.nvec = (uint32_t)((out->stream.size() - base) / TS_IDS_PER_VEC);
            while (out->meta.size() % 4) out->meta.push_back(0);
            d.meta_words = (uint32_t)(out->meta.size() - d.meta_off);
            if ((size_t)d.meta_words * 4 > TS_MAX_META_BYTES) return "pack: section table exceeds its shared-memory budget";
        }
    }
    L.total_vecs = (int64_t)(out->stream.size() / TS_IDS_PER_VEC);
    if (L.total_vecs >= ((int64_t)1 << 32)) return "pack: stream exceeds 64 GiB";
    return nullptr;
}

namespace {

// Walks every section of an image: f(block descriptor, tile, first column of the sub-block, columns in it, section words)
template <typename F>
void for_each_section(const TsHostImage& img, F&& f) {
    const TsLayout& L = img.lay;
    for (int j = 0; j < L.k_splits; ++j)
        for (int b = 0; b < L.col_blocks; ++b) {
            const TsCtaDesc& d = L.cta[j * L.col_blocks + b];
            const int c0 = b * L.cols_per_block, c1 = std::min(L.columns, c0 + L.cols_per_block);
            const int t0 = j * L.tiles_per_cta, t1 = std::min(L.tiles, t0 + L.tiles_per_cta);
            const uint32_t* sec = img.meta.data() + d.meta_off;
            for (int t = t0; t < t1; ++t)
                for (int s0 = c0; s0 < c1; s0 += L.sub_cols) {
                    const int ns = std::min(L.sub_cols, c1 - s0);
                    f(d, t, s0, ns, sec);
                    sec += TS_SEC_HEADER + sec[1] + 1 + sec[2];
                }
        }
}

}  // namespace

void ts_unpack_dense(const TsHostImage& img, int8_t* w) {
    const TsLayout& L = img.lay;
    std::memset(w, 0, (size_t)L.inners * L.columns);
    const int lpl = L.lanes_per_list;
    for_each_section(img, [&](const TsCtaDesc& d, int t, int s0, int, const uint32_t* sec) {
        const uint32_t ndiag = sec[1], nl = sec[2];
        const uint32_t* diag = sec + TS_SEC_HEADER;
        const uint32_t* lists = diag + ndiag + 1;
        for (uint32_t l = 0; l < nl; ++l) {
            const uint32_t tag = lists[l] & 0xffffu, steps = lists[l] >> 16;
            for (uint32_t i = 0; i < steps; ++i)
                for (int jj = 0; jj < lpl; ++jj) {
                    const size_t vec = (size_t)d.stream_off + sec[0] + diag[i] + (size_t)l * lpl + jj;
                    for (int e = 0; e < TS_IDS_PER_VEC; ++e) {
                        const int id = img.stream[vec * TS_IDS_PER_VEC + e];
                        if (id < L.tile_rows && t * L.tile_rows + id < L.inners)
                            w[(size_t)(t * L.tile_rows + id) * L.columns + s0 + (tag & 0x7fff)] += (tag >> 15) ? -1 : 1;
                    }
                }
        }
    });
}

const char* ts_validate(const TsHostImage& img) {
    const TsLayout& L = img.lay;
    if (L.num_ctas != L.col_blocks * L.k_splits || L.num_ctas > TS_MAX_BLOCKS || L.cta.size() != (size_t)L.num_ctas) return "validate: block count";
    if ((L.cols_per_block & 1) || L.sub_cols > TS_MAX_SUB_COLS || L.sub_cols <= 0) return "validate: column block / sub-block size";
    if (L.sub_cols < L.cols_per_block && (L.sub_cols & 1)) return "validate: odd sub-block";
    const int lpl = L.lanes_per_list;
    if (lpl < 1 || lpl > 16 || (lpl & (lpl - 1))) return "validate: lanes per list";
    for (int i = 0; i < L.num_ctas; ++i) {
        const TsCtaDesc& d = L.cta[i];
        if (d.stream_off % 32 || d.nvec % 32 || d.meta_off % 4 || d.meta_words % 4) return "validate: alignment";
        if ((size_t)(d.stream_off + d.nvec) * TS_IDS_PER_VEC > img.stream.size()) return "validate: stream range";
        if ((size_t)d.meta_off + d.meta_words > img.meta.size()) return "validate: table range";
        if ((size_t)d.meta_words * 4 > TS_MAX_META_BYTES) return "validate: table size";
    }
    const char* err = nullptr;
    std::vector<int> seen;
    for_each_section(img, [&](const TsCtaDesc& d, int, int, int ns, const uint32_t* sec) {
        if (err) return;
        const uint32_t ndiag = sec[1], nl = sec[2];
        if ((size_t)(sec - (img.meta.data() + d.meta_off)) + TS_SEC_HEADER + ndiag + 1 + nl > d.meta_words) { err = "validate: section table overruns the block's table"; return; }
        if (nl != (uint32_t)(2 * ns)) { err = "validate: list count"; return; }
        if (sec[0] % 32) err = "validate: section alignment";
        const uint32_t* diag = sec + TS_SEC_HEADER;
        const uint32_t* lists = diag + ndiag + 1;
        if (sec[0] + diag[ndiag] > d.nvec) err = "validate: section data out of the block's range";
        seen.assign((size_t)2 * ns, 0);
        uint32_t prev_steps = 0xffffffffu;
        for (uint32_t l = 0; l < nl; ++l) {
            const uint32_t tag = lists[l] & 0xffffu, steps = lists[l] >> 16;
            if (steps > prev_steps) err = "validate: lists not sorted by length";
            prev_steps = steps;
            if (steps > ndiag) err = "validate: list longer than the diagonal count";
            if ((int)(tag & 0x7fff) >= ns) { err = "validate: column tag out of range"; return; }
            seen[(size_t)2 * (tag & 0x7fff) + (tag >> 15)]++;
        }
        for (int v : seen)
            if (v != 1) err = "validate: a list is missing or duplicated";
        // every diagonal holds exactly the lists that reach it, starts on 128 bytes and fits before the next one
        for (uint32_t i = 0; i < ndiag; ++i) {
            uint32_t live = 0;
            for (uint32_t l = 0; l < nl; ++l) live += (lists[l] >> 16) > i;
            if (diag[i] % 8) err = "validate: diagonal alignment";
            if (diag[i] + live * (uint32_t)lpl > diag[i + 1]) err = "validate: diagonals overlap";
        }
        if (nl && ndiag != (lists[0] >> 16)) err = "validate: diagonal count";
    });
    if (err) return err;
    for (uint16_t id : img.stream)
        if (id > (uint16_t)L.tile_rows) return "validate: row id beyond the zero row";
    return nullptr;
}

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

extern "C" int tllm_pack_roundtrip(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                                   int8_t* w_out, tllm_weight_info* info) {
    if (!w || !w_out || inners <= 0 || columns <= 0 || num_sms <= 0) return tllm::fail(TLLM_ERR_ARG, "tllm_pack_roundtrip: bad argument");
    TsHostImage img;
    const char* msg = ts_pack_dense(w, inners, columns, opts, num_sms, &img);
    if (!msg) msg = ts_validate(img);
    if (msg) return tllm::fail(TLLM_ERR_ARG, "%s", msg);
    ts_unpack_dense(img, w_out);
    {   // the second representation must describe the same matrix
        std::vector<uint32_t> bits;
        int nt = 0, kb = 0;
        mm_pack_bits(w, inners, columns, &bits, &nt, &kb);
        std::vector<int8_t> back((size_t)inners * columns);
        mm_unpack_bits(bits, inners, columns, back.data());
        if (std::memcmp(back.data(), w, back.size()) != 0) return tllm::fail(TLLM_ERR_ARG, "bit tiles do not reproduce the matrix");
        if (info) info->bit_tile_bytes = (int64_t)bits.size() * 4;
    }
    if (info) {
        const int64_t keep_bits = info->bit_tile_bytes;
        const TsLayout& L = img.lay;
        std::memset(info, 0, sizeof *info);
        info->bit_tile_bytes = keep_bits;
        info->inners = L.inners;
        info->columns = L.columns;
        info->tile_rows = L.tile_rows;
        info->tiles = L.tiles;
        info->col_blocks = L.col_blocks;
        info->k_splits = L.k_splits;
        info->tiles_per_cta = L.tiles_per_cta;
        info->num_ctas = L.num_ctas;
        info->lanes_per_list = L.lanes_per_list;
        info->nnz = L.nnz;
        info->stream_bytes = (int64_t)img.stream.size() * 2;
        info->meta_bytes = (int64_t)img.meta.size() * 4;
        info->algorithmic_bytes = 2 * L.nnz + 16 * (int64_t)L.columns * ((L.inners + 511) / 512);
    }
    return TLLM_OK;
}
