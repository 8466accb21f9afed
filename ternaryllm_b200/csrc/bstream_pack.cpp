// bstream_pack.cpp -- host packer, unpacker and validator of the bank-stream format (bstream_format.h).
//
// Takes the place of convert_to_ter_tiled_mcsc + inter_tile_swizzle on the way to the GPU
// (ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:9-27, :156-315): same information -- per (column, K-tile) the rows of
// the +1 and of the -1 entries -- as one-byte ids cut by shared-memory bank, with thread-block and warp ranges
// balanced by non-zero count (the reference's tile reordering by list length is computed and never used by its
// kernels, ter_spmm_kernel.cuh:159-160).
#include <algorithm>
#include <atomic>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/tllm.h"
#include "bstream_format.h"
#include "column_lists.h"

namespace {

using tllm::ColumnLists;

// one lane's stream of a unit under construction
struct LaneStream {
    std::vector<uint8_t> bytes;       // 16 per vector
    std::vector<uint32_t> end_vec;    // per list: the vector that holds its last word
    int word = 4;                     // next free word of the last vector (4: start a new vector)
    void clear() {
        bytes.clear();
        end_vec.clear();
        word = 4;
    }
    // appends one list: n row groups, padded with BS_NULL_ID to whole words; an empty list is one word of padding
    void add_list(const uint8_t* groups, int n) {
        int i = 0;
        do {
            if (word == 4) {
                bytes.insert(bytes.end(), 15, (uint8_t)BS_NULL_ID);
                bytes.push_back(0);
                word = 0;
            }
            uint8_t* v = bytes.data() + bytes.size() - 16;
            const int cap = word < 3 ? 4 : 3;
            for (int e = 0; e < cap && i < n; ++e, ++i) v[4 * word + e] = groups[i];
            if (i >= n) v[15] |= (uint8_t)(1u << word);
            ++word;
        } while (i < n);
        end_vec.push_back((uint32_t)(bytes.size() / 16 - 1));
    }
    uint32_t nvec() const { return (uint32_t)(bytes.size() / 16); }
};

// Walks the 32 lane streams of a unit in lockstep, the way the kernel's warp does, and returns the reduce points;
// false if some lane would run more than a ring ahead of the reduced slots.
bool simulate_unit(const LaneStream (&ls)[32], uint32_t lists, std::vector<uint16_t>* rp) {
    rp->clear();
    uint32_t p[32] = {}, max_nv = 0;
    for (int l = 0; l < 32; ++l) max_nv = std::max(max_nv, ls[l].nvec());
    uint32_t done = 0;
    for (uint32_t i = 0; i < max_nv; ++i) {
        uint32_t lo = lists, hi = 0;
        for (int l = 0; l < 32; ++l) {
            while (p[l] < lists && ls[l].end_vec[p[l]] == i) ++p[l];
            lo = std::min(lo, p[l]);
            hi = std::max(hi, p[l]);
        }
        if (hi > done + BS_RING_SLOTS) return false;
        while (done + BS_BATCH_SLOTS <= lo) {
            rp->push_back((uint16_t)i);
            done += BS_BATCH_SLOTS;
        }
    }
    return true;
}

struct Builder {
    const ColumnLists<int8_t>& cl;
    std::vector<uint8_t>* stream;   // the current block's stream (starts at byte 0)
    int T;                          // rows of a K-tile
    LaneStream ls[32];
    std::vector<uint16_t> rp;
    std::vector<uint8_t> bucket[32];

    // appends to `meta` the descriptor(s) of (tile t, columns [a, b)) and to the stream their vectors
    void emit_units(int t, int a, int b, int c_block0, int t_block0, std::vector<uint32_t>* meta, int* units) {
        if (a >= b) return;
        if (b - a > BS_MAX_UNIT_COLS) {
            const int mid = a + (((b - a) / 2 + 1) & ~1);
            emit_units(t, a, mid, c_block0, t_block0, meta, units);
            emit_units(t, mid, b, c_block0, t_block0, meta, units);
            return;
        }
        const int lo = t * T, hi = lo + T;
        for (int l = 0; l < 32; ++l) ls[l].clear();
        for (int c = a; c < b; ++c)
            for (int sg = 0; sg < 2; ++sg) {
                const std::vector<int64_t>& ptr = sg ? cl.neg_ptr : cl.pos_ptr;
                const std::vector<int32_t>& rows = sg ? cl.neg_row : cl.pos_row;
                const int32_t* first = std::lower_bound(rows.data() + ptr[c], rows.data() + ptr[c + 1], lo);
                const int32_t* last = std::lower_bound(first, rows.data() + ptr[c + 1], hi);
                for (int l = 0; l < 32; ++l) bucket[l].clear();
                for (const int32_t* r = first; r < last; ++r) bucket[(*r) & 31].push_back((uint8_t)((*r - lo) >> 5));
                for (int l = 0; l < 32; ++l) ls[l].add_list(bucket[l].data(), (int)bucket[l].size());
            }
        const uint32_t lists = 2u * (uint32_t)(b - a);
        if (!simulate_unit(ls, lists, &rp) && b - a > BS_BATCH_SLOTS) {
            // some lane runs too far ahead of the slowest one: end the unit earlier (two units of half the columns)
            const int mid = a + (((b - a) / 2 + 1) & ~1);
            emit_units(t, a, mid, c_block0, t_block0, meta, units);
            emit_units(t, mid, b, c_block0, t_block0, meta, units);
            return;
        }
        uint32_t min_nv = 0xffffffffu, max_nv = 0;
        for (int l = 0; l < 32; ++l) {
            min_nv = std::min(min_nv, ls[l].nvec());
            max_nv = std::max(max_nv, ls[l].nvec());
        }
        std::vector<uint8_t>& s = *stream;
        while (s.size() % 128) s.push_back(0);
        const size_t unit_base = s.size();
        for (uint32_t i = 0; i < min_nv; ++i)
            for (int l = 0; l < 32; ++l) s.insert(s.end(), ls[l].bytes.begin() + (size_t)i * 16, ls[l].bytes.begin() + (size_t)(i + 1) * 16);
        for (int l = 0; l < 32; ++l) s.insert(s.end(), ls[l].bytes.begin() + (size_t)min_nv * 16, ls[l].bytes.end());
        meta->push_back((uint32_t)(unit_base / 16));
        meta->push_back((uint32_t)(a - c_block0) | ((uint32_t)(b - a) << 16));
        meta->push_back((uint32_t)(t - t_block0) | ((uint32_t)rp.size() << 8));
        meta->push_back(min_nv | (max_nv << 16));
        for (int l = 0; l < 32; l += 2) meta->push_back(ls[l].nvec() | (ls[l + 1].nvec() << 16));
        for (size_t i = 0; i < rp.size(); i += 2) meta->push_back((uint32_t)rp[i] | ((i + 1 < rp.size() ? (uint32_t)rp[i + 1] : 0u) << 16));
        ++*units;
    }
};

// cuts [0, n) into `parts` contiguous ranges of about equal weight with even boundaries; start has parts+1 entries
void balanced_even_cuts(const std::vector<int64_t>& prefix, int n, int parts, std::vector<int32_t>* start) {
    start->assign((size_t)parts + 1, 0);
    const int64_t total = prefix[n];
    int c = 0;
    for (int p = 1; p < parts; ++p) {
        const int64_t want = total * p / parts;
        while (c < n && prefix[c] < want) ++c;
        // the even boundary nearest to the ideal cut
        int e = c & ~1;
        if (e + 2 <= n && c > e && prefix[std::min(e + 2, n)] - want < want - prefix[e]) e += 2;
        e = std::max(e, (int)(*start)[p - 1]);
        (*start)[p] = std::min(e, n);
    }
    (*start)[parts] = n;
}

}  // namespace

const char* bs_pack_dense(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms, BsHostImage* out) {
    if (!w || inners <= 0 || columns <= 0) return "pack: bad matrix shape";
    if ((int64_t)inners * columns > ((int64_t)1 << 40)) return "pack: matrix too large";
    tllm_pack_opts o{};
    if (opts) o = *opts;
    if (o.num_ctas < 0 || o.num_ctas > BS_MAX_BLOCKS || num_sms <= 0 || num_sms > BS_MAX_BLOCKS / 4) return "pack: num_ctas out of range";
    int T = o.tile_rows > 0 ? o.tile_rows : BS_TILE_ROWS;
    if (T > BS_TILE_ROWS || T % 32) return "pack: tile_rows must be a multiple of 32 and at most 4096";
    const int tiles = (inners + T - 1) / T;
    if (tiles > 255) return "pack: more than 255 K-tiles";

    ColumnLists<int8_t> cl(w, inners, columns);
    BsLayout& L = out->lay;
    L = BsLayout{};
    L.inners = inners;
    L.columns = columns;
    L.tile_rows = T;
    L.tiles = tiles;
    L.nnz = (int64_t)cl.pos_row.size() + (int64_t)cl.neg_row.size();

    // Blocks per SM: a block is eight warps, and the walk is bound by instruction issue and latency, not by bytes, so an
    // SM wants 16 warps of a small product (two more blocks of the next product in the stream wait beside them with
    // their tables and first index vectors already fetched) and 32 warps of a large one.
    int ctas = o.num_ctas;
    if (ctas <= 0) {
        int per_sm = L.nnz / num_sms > 300000 ? 4 : 2;
        while (per_sm > 1 && columns / (per_sm * num_sms) < 16) per_sm /= 2;
        ctas = per_sm * num_sms;
    }

    // K-splits: blocks share a column range along K only where the columns alone would leave a warp with less than
    // four columns of a tile (short units waste lanes at their ragged ends); then every block takes one tile
    int ks = 1;
    if (o.k_splits > 0) ks = std::min(o.k_splits, tiles);
    else if (tiles > 1 && columns / ctas < 4 * BS_WARPS) ks = tiles;
    int tpc = (tiles + ks - 1) / ks;
    ks = (tiles + tpc - 1) / tpc;

    // column weights: non-zeros plus what a column costs whatever it holds (two lists per lane and tile)
    std::vector<int64_t> prefix((size_t)columns + 1, 0);
    for (int c = 0; c < columns; ++c)
        prefix[c + 1] = prefix[c] + (cl.pos_ptr[c + 1] - cl.pos_ptr[c]) + (cl.neg_ptr[c + 1] - cl.neg_ptr[c]) + 96 * (int64_t)tiles;

    int col_blocks = std::max(1, std::min(ctas / ks, (columns + 1) / 2));
    for (int attempt = 0;; ++attempt) {
        if (attempt > 40 || (int64_t)col_blocks * ks > BS_MAX_BLOCKS) return "pack: no schedule fits (matrix too wide for the block budget)";
        balanced_even_cuts(prefix, columns, col_blocks, &L.col_start);
        int widest = 0;
        for (int b = 0; b < col_blocks; ++b) widest = std::max(widest, L.col_start[b + 1] - L.col_start[b]);
        if ((int64_t)widest * tpc > BS_MAX_CELLS) {
            col_blocks = std::min((columns + 1) / 2, std::max(col_blocks + 1, (int)((int64_t)col_blocks * 3 / 2)));
            continue;
        }
        L.col_blocks = col_blocks;
        L.k_splits = ks;
        L.tiles_per_cta = tpc;
        L.num_ctas = col_blocks * ks;
        L.max_cols_per_block = widest;
        L.cta.assign((size_t)L.num_ctas, TsCtaDesc{});
        struct BlockImage {
            std::vector<uint8_t> stream;
            std::vector<uint32_t> meta;
            int units = 0;
        };
        std::vector<BlockImage> blocks((size_t)L.num_ctas);
        std::atomic<int> next{0};
        std::atomic<bool> too_big{false};
        // blocks are independent: they are packed by as many threads as the host offers, then laid end to end
        auto work = [&]() {
            Builder bld{cl, nullptr, T};
            std::vector<int64_t> wprefix;
            std::vector<int32_t> wstart;
            for (;;) {
                const int id = next.fetch_add(1);
                if (id >= L.num_ctas || too_big.load()) return;
                const int j = id / col_blocks, b = id % col_blocks;
                BlockImage& B = blocks[(size_t)id];
                bld.stream = &B.stream;
                const int c0 = L.col_start[b], c1 = L.col_start[b + 1];
                const int t0 = j * tpc, t1 = std::min(tiles, t0 + tpc);
                // warp ranges by the non-zeros inside this block's tiles
                wprefix.assign((size_t)(c1 - c0) + 1, 0);
                for (int c = c0; c < c1; ++c) {
                    int64_t n = 96 * (int64_t)(t1 - t0);
                    for (int sg = 0; sg < 2; ++sg) {
                        const std::vector<int64_t>& ptr = sg ? cl.neg_ptr : cl.pos_ptr;
                        const std::vector<int32_t>& rows = sg ? cl.neg_row : cl.pos_row;
                        const int32_t* first = std::lower_bound(rows.data() + ptr[c], rows.data() + ptr[c + 1], t0 * T);
                        const int32_t* last = std::lower_bound(first, rows.data() + ptr[c + 1], t1 * T);
                        n += last - first;
                    }
                    wprefix[(size_t)(c - c0) + 1] = wprefix[(size_t)(c - c0)] + n;
                }
                balanced_even_cuts(wprefix, c1 - c0, BS_WARPS, &wstart);
                std::vector<uint32_t>& meta = B.meta;
                meta.assign(BS_BLOCK_HEADER + BS_WARPS + 1, 0u);
                meta[0] = (uint32_t)c0, meta[1] = (uint32_t)(c1 - c0), meta[2] = (uint32_t)t0, meta[3] = (uint32_t)(t1 - t0);
                meta[4] = (uint32_t)j, meta[5] = (uint32_t)b;
                for (int wi = 0; wi < BS_WARPS; ++wi) {
                    meta[BS_BLOCK_HEADER + wi] = (uint32_t)meta.size();
                    for (int t = t0; t < t1; ++t) bld.emit_units(t, c0 + wstart[wi], c0 + wstart[wi + 1], c0, t0, &meta, &B.units);
                }
                meta[BS_BLOCK_HEADER + BS_WARPS] = (uint32_t)meta.size();
                meta[6] = (uint32_t)B.units;
                while (meta.size() % 4) meta.push_back(0);
                if (meta.size() * 4 > BS_MAX_META_BYTES) too_big.store(true);
                while (B.stream.size() % 512) B.stream.push_back(0);
            }
        };
        unsigned nthreads = std::thread::hardware_concurrency();
        nthreads = std::max(1u, std::min(nthreads, 32u));
        nthreads = std::min<unsigned>(nthreads, (unsigned)L.num_ctas);
        std::vector<std::thread> pool;
        for (unsigned i = 1; i < nthreads; ++i) pool.emplace_back(work);
        work();
        for (std::thread& th : pool) th.join();
        if (too_big.load()) {
            col_blocks = std::min((columns + 1) / 2, std::max(col_blocks + 1, (int)((int64_t)col_blocks * 3 / 2)));
            continue;
        }
        out->stream.clear();
        out->meta.clear();
        L.units = 0;
        size_t total_stream = 0, total_meta = 0;
        for (const BlockImage& B : blocks) total_stream += B.stream.size(), total_meta += B.meta.size();
        out->stream.reserve(total_stream);
        out->meta.reserve(total_meta);
        for (int id = 0; id < L.num_ctas; ++id) {
            const BlockImage& B = blocks[(size_t)id];
            TsCtaDesc& d = L.cta[(size_t)id];
            d.stream_off = (uint32_t)(out->stream.size() / 16);
            d.nvec = (uint32_t)(B.stream.size() / 16);
            d.meta_off = (uint32_t)out->meta.size();
            d.meta_words = (uint32_t)B.meta.size();
            out->stream.insert(out->stream.end(), B.stream.begin(), B.stream.end());
            out->meta.insert(out->meta.end(), B.meta.begin(), B.meta.end());
            L.units += B.units;
        }
        break;
    }
    L.total_vecs = (int64_t)(out->stream.size() / 16);
    if (L.total_vecs >= ((int64_t)1 << 32)) return "pack: stream exceeds 64 GiB";
    return nullptr;
}

namespace {

struct UnitView {
    uint32_t off, col0, ncols, tile, n_rp, min_nv, max_nv;
    uint32_t nv[32];
    const uint32_t* rp;
    uint32_t words;
};

// Reads the unit descriptor at meta[at] of a block table of `total` words; false if it does not fit.
bool read_unit(const uint32_t* meta, uint32_t at, uint32_t total, UnitView* u) {
    if (at > total || total - at < BS_UNIT_HEADER) return false;
    const uint32_t* d = meta + at;
    u->off = d[0];
    u->col0 = d[1] & 0xffffu, u->ncols = d[1] >> 16;
    u->tile = d[2] & 0xffu, u->n_rp = d[2] >> 8;
    u->min_nv = d[3] & 0xffffu, u->max_nv = d[3] >> 16;
    for (int l = 0; l < 32; ++l) u->nv[l] = (d[4 + l / 2] >> (16 * (l & 1))) & 0xffffu;
    u->words = BS_UNIT_HEADER + (u->n_rp + 1) / 2;
    if (total - at < u->words) return false;
    u->rp = d + BS_UNIT_HEADER;
    return true;
}

// address (in vectors, relative to the unit) of vector i of lane l
inline size_t unit_vec(const UnitView& u, const uint32_t (&tail_off)[32], int l, uint32_t i) {
    return i < u.min_nv ? (size_t)i * 32 + l : (size_t)u.min_nv * 32 + tail_off[l] + (i - u.min_nv);
}

}  // namespace

const char* bs_validate(const BsHostImage& img) {
    const BsLayout& L = img.lay;
    if (L.inners <= 0 || L.columns <= 0) return "validate: matrix shape";
    if (L.tile_rows <= 0 || L.tile_rows > BS_TILE_ROWS || L.tile_rows % 32) return "validate: tile rows";
    if (L.tiles != (L.inners + L.tile_rows - 1) / L.tile_rows || L.tiles > 255) return "validate: tile count";
    if (L.k_splits < 1 || L.tiles_per_cta < 1 || L.col_blocks < 1) return "validate: schedule";
    if ((int64_t)L.k_splits * L.tiles_per_cta < L.tiles || (int64_t)(L.k_splits - 1) * L.tiles_per_cta >= L.tiles) return "validate: K-splits do not tile the tiles";
    if ((int64_t)L.col_blocks * L.k_splits != L.num_ctas || L.num_ctas > BS_MAX_BLOCKS || L.cta.size() != (size_t)L.num_ctas) return "validate: block count";
    if (L.col_start.size() != (size_t)L.col_blocks + 1 || L.col_start[0] != 0 || L.col_start[L.col_blocks] != L.columns) return "validate: column ranges";
    for (int b = 0; b < L.col_blocks; ++b) {
        const int n = L.col_start[b + 1] - L.col_start[b];
        if (n < 0 || (int64_t)n * L.tiles_per_cta > BS_MAX_CELLS || n > L.max_cols_per_block) return "validate: column block too wide";
        if ((L.col_start[b] & 1) && b > 0) return "validate: odd column-block boundary";
    }
    if (img.stream.size() % 16 || (int64_t)(img.stream.size() / 16) != L.total_vecs) return "validate: stream size";
    std::vector<uint8_t> seen;
    std::vector<uint32_t> p(32);
    for (int j = 0; j < L.k_splits; ++j)
        for (int b = 0; b < L.col_blocks; ++b) {
            const TsCtaDesc& d = L.cta[(size_t)j * L.col_blocks + b];
            if (d.stream_off % 32 || d.nvec % 32 || d.meta_off % 4 || d.meta_words % 4) return "validate: alignment";
            if ((uint64_t)d.stream_off + d.nvec > (uint64_t)L.total_vecs) return "validate: stream range";
            if ((uint64_t)d.meta_off + d.meta_words > img.meta.size()) return "validate: table range";
            if ((size_t)d.meta_words * 4 > BS_MAX_META_BYTES || d.meta_words < BS_BLOCK_HEADER + BS_WARPS + 1) return "validate: table size";
            const uint32_t* m = img.meta.data() + d.meta_off;
            const int c0 = L.col_start[b], nc = L.col_start[b + 1] - c0;
            const int t0 = j * L.tiles_per_cta, nt = std::min(L.tiles, t0 + L.tiles_per_cta) - t0;
            if (m[0] != (uint32_t)c0 || m[1] != (uint32_t)nc || m[2] != (uint32_t)t0 || m[3] != (uint32_t)nt || m[4] != (uint32_t)j || m[5] != (uint32_t)b)
                return "validate: block header";
            // every (tile, column) of the block must be covered by exactly one unit
            seen.assign((size_t)nt * nc, 0);
            uint32_t at = BS_BLOCK_HEADER + BS_WARPS + 1, block_units = 0;
            for (int wi = 0; wi < BS_WARPS; ++wi) {
                if (m[BS_BLOCK_HEADER + wi] != at) return "validate: warp table";
                const uint32_t end = m[BS_BLOCK_HEADER + wi + 1];
                if (end < at || end > d.meta_words) return "validate: warp table";
                uint32_t prev_tile = 0;
                while (at < end) {
                    UnitView u;
                    if (!read_unit(m, at, end, &u)) return "validate: unit descriptor overruns its table";
                    if (u.ncols == 0 || u.ncols > BS_MAX_UNIT_COLS || u.col0 + u.ncols > (uint32_t)nc || (u.col0 & 1)) return "validate: unit columns";
                    if (u.tile >= (uint32_t)nt || u.tile < prev_tile) return "validate: unit tile";
                    prev_tile = u.tile;
                    if (u.off % 8) return "validate: unit alignment";
                    uint64_t total = 0;
                    uint32_t lo = 0xffffffffu, hi = 0;
                    for (int l = 0; l < 32; ++l) {
                        total += u.nv[l];
                        lo = std::min(lo, u.nv[l]);
                        hi = std::max(hi, u.nv[l]);
                    }
                    if (lo != u.min_nv || hi != u.max_nv || lo == 0) return "validate: lane lengths";
                    if ((uint64_t)u.off + total > d.nvec) return "validate: unit data out of the block's range";
                    for (uint32_t c = 0; c < u.ncols; ++c) {
                        uint8_t& s = seen[(size_t)u.tile * nc + u.col0 + c];
                        if (s) return "validate: a column of a tile is covered twice";
                        s = 1;
                    }
                    // replay the walk: ids in range, list counts, ring bound, reduce points
                    uint32_t tail_off[32], acc = 0;
                    for (int l = 0; l < 32; ++l) {
                        tail_off[l] = acc;
                        acc += u.nv[l] - u.min_nv;
                    }
                    const uint8_t* base = img.stream.data() + ((size_t)d.stream_off + u.off) * 16;
                    const uint32_t lists = 2 * u.ncols;
                    const int rows_here = std::min(L.tile_rows, L.inners - (t0 + (int)u.tile) * L.tile_rows);
                    const uint32_t groups_here = (uint32_t)(rows_here + 31) / 32;
                    std::fill(p.begin(), p.end(), 0u);
                    uint32_t done = 0, k = 0;
                    for (uint32_t i = 0; i < u.max_nv; ++i) {
                        uint32_t mn = lists, mx = 0;
                        for (int l = 0; l < 32; ++l) {
                            if (i < u.nv[l]) {
                                const uint8_t* v = base + unit_vec(u, tail_off, l, i) * 16;
                                for (int e = 0; e < 15; ++e) {
                                    if (v[e] == BS_NULL_ID) continue;
                                    if (v[e] >= groups_here) return "validate: row group beyond the tile";
                                    if ((uint32_t)v[e] * 32 + l >= (uint32_t)rows_here) return "validate: row beyond the matrix";
                                }
                                if (v[15] & 0xf0) return "validate: flag byte";
                                p[l] += (uint32_t)__builtin_popcount(v[15]);
                            }
                            mn = std::min(mn, p[l]);
                            mx = std::max(mx, p[l]);
                        }
                        if (mx > done + BS_RING_SLOTS || mx > lists) return "validate: a lane runs ahead of the slot ring";
                        while (k < u.n_rp && ((u.rp[k / 2] >> (16 * (k & 1))) & 0xffffu) == i) {
                            if (done + BS_BATCH_SLOTS > mn) return "validate: reduce point before its slots are complete";
                            done += BS_BATCH_SLOTS;
                            ++k;
                        }
                    }
                    if (k != u.n_rp) return "validate: reduce point beyond the unit";
                    for (int l = 0; l < 32; ++l)
                        if (p[l] != lists) return "validate: list count of a lane";
                    if (lists - done > BS_RING_SLOTS) return "validate: too many slots left for the final reduction";
                    at += u.words;
                    ++block_units;
                }
                if (at != end) return "validate: warp table";
            }
            if (m[BS_BLOCK_HEADER + BS_WARPS] != at) return "validate: warp table";
            if (m[6] != block_units || m[7] != 0) return "validate: block header";
            for (uint8_t s : seen)
                if (!s) return "validate: a column of a tile is not covered";
        }
    return nullptr;
}

void bs_unpack_dense(const BsHostImage& img, int8_t* w) {
    const BsLayout& L = img.lay;
    std::memset(w, 0, (size_t)L.inners * L.columns);
    for (int j = 0; j < L.k_splits; ++j)
        for (int b = 0; b < L.col_blocks; ++b) {
            const TsCtaDesc& d = L.cta[(size_t)j * L.col_blocks + b];
            const uint32_t* m = img.meta.data() + d.meta_off;
            const int c0 = (int)m[0], t0 = (int)m[2];
            uint32_t at = m[BS_BLOCK_HEADER];
            const uint32_t end = m[BS_BLOCK_HEADER + BS_WARPS];
            while (at < end) {
                UnitView u;
                if (!read_unit(m, at, end, &u)) return;
                uint32_t tail_off[32], acc = 0;
                for (int l = 0; l < 32; ++l) {
                    tail_off[l] = acc;
                    acc += u.nv[l] - u.min_nv;
                }
                const uint8_t* base = img.stream.data() + ((size_t)d.stream_off + u.off) * 16;
                const int krow0 = (t0 + (int)u.tile) * L.tile_rows;
                for (int l = 0; l < 32; ++l) {
                    uint32_t slot = 0;
                    for (uint32_t i = 0; i < u.nv[l]; ++i) {
                        const uint8_t* v = base + unit_vec(u, tail_off, l, i) * 16;
                        for (int wd = 0; wd < 4; ++wd) {
                            for (int e = 0; e < (wd < 3 ? 4 : 3); ++e) {
                                const int g = v[4 * wd + e];
                                if (g == BS_NULL_ID || slot >= 2 * u.ncols) continue;
                                const int k = krow0 + g * 32 + l;
                                if (k < L.inners) w[(size_t)k * L.columns + c0 + u.col0 + slot / 2] += (slot & 1) ? -1 : 1;
                            }
                            if (v[15] & (1u << wd)) ++slot;
                        }
                    }
                }
                at += u.words;
            }
        }
}
