// bstream_kernel.cuh -- the decode product (1..4 activation rows per launch) on the bank-stream format
// (bstream_format.h): what ter_tiled_mcsc_spmv / ter_tiled_mcsc_spmm compute
// (ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:24-78, :106-308), by gathering, adding and subtracting only.
//
// One block of eight warps per column range.  The activation table of a K-tile is 16.1 KiB per activation row
// and is not replicated: lane l of a warp owns the rows k with k % 32 == l, which are exactly the entries of
// shared-memory bank l, so a warp-wide gather never conflicts.  Each lane streams its own one-byte ids with
// 128-bit loads held in register batches, adds what it gathers into one accumulator and drops it into a ring of
// lane cells at the end of every list; at the reduce points the packer recorded, the warp adds the 32 cells of
// eight lists and combines them into four column sums.  Nothing here waits on another block except the split-K
// hand-over through an arrival counter (no spinning: the last block to arrive does the sum).
//
// HBM-bound byte work: no tensor cores here by design.
#pragma once
#include "bstream_format.h"
#include "kernels.cuh"

namespace tllm {

struct BsParams {
    const uint4* stream;
    const uint32_t* meta;
    const void* X;
    void* Y;
    void* partial;            // [k_splits][M][columns] fp32 / int32 (only read or written when k_splits > 1)
    unsigned int* counters;   // [col_blocks], zero between launches
    int* status;              // 0, or an error code written by a block whose bounded wait ran out
    int x_dtype, x_layout, y_dtype;
    int M;                    // rows in this launch (<= MP)
    int K, N;
    int T;                    // rows of a K-tile
    int col_blocks, k_splits, tiles_per_cta, max_cols;
    int resident;             // K-tiles whose activation tables are in shared memory at the same time
    int epilogue;             // 0: Y = acc*scale ; 1: columns are (gate,up) pairs, Y[c/2] = silu(g*scale)*(u*scale2)
    int y_ld;                 // row stride of Y in elements
    int x_ld;                 // row-major X: elements between rows; column-major X: elements between k
    int x_vec;                // 1: X is row-major, rows start on 16 bytes and K is a multiple of 16: 128-bit loads
    uint32_t l2_prefetch_bytes;
    uint32_t off_table, off_cells, off_meta, off_bars, off_stage;   // shared-memory carve-up behind the rings
    float scale, scale2;
    const TsCtaDesc* cta_ext;   // all block descriptors in device memory; blocks past BS_MAX_PARAM_BLOCKS read theirs here
    TsCtaDesc cta[BS_MAX_PARAM_BLOCKS];
};

#define BS_ERR_META_WAIT 105

// Diagnostic builds (-DBS_TRACE, never the shipped library): every block records the GPU global timer at a few
// points of its life into a buffer of 8 values per block.
#ifdef BS_TRACE
__device__ long long* g_bs_trace = nullptr;
#define BS_STAMP(slot)                                                                                   \
    do {                                                                                                 \
        if (g_bs_trace && threadIdx.x == 0) {                                                            \
            long long t_;                                                                                \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));                                        \
            g_bs_trace[(size_t)blockIdx.x * 8 + (slot)] = t_;                                            \
        }                                                                                                \
    } while (0)
#else
#define BS_STAMP(slot) \
    do {               \
    } while (0)
#endif

// shared-memory bytes of one launch (host and device agree through the offsets in BsParams)
struct BsSmem {
    uint32_t off_table, off_cells, off_meta, off_bars, off_stage, total;
};
inline BsSmem bs_smem_layout(int mp, int resident, int tiles_per_cta, int max_cols, uint32_t max_meta_words, uint32_t stage_bytes) {
    BsSmem s;
    const uint32_t ring = (uint32_t)BS_RING_SLOTS * 128u * (uint32_t)mp;
    s.off_table = (uint32_t)BS_WARPS * ring;
    s.off_cells = s.off_table + (uint32_t)resident * BS_TABLE_GROUPS * 128u * (uint32_t)mp;
    s.off_meta = (s.off_cells + (uint32_t)tiles_per_cta * (uint32_t)max_cols * 4u * (uint32_t)mp + 15u) & ~15u;
    s.off_bars = (s.off_meta + max_meta_words * 4u + 15u) & ~15u;
    s.off_stage = s.off_bars + 64u;
    s.total = s.off_stage + stage_bytes + ring;   // + ring: the base is aligned up to a ring inside the allocation
    return s;
}

template <typename ACC, int MP>
struct BsCell;   // MP accumulators as one shared-memory access
template <typename ACC>
struct BsCell<ACC, 1> {
    static __device__ __forceinline__ void gather_add(uint32_t a, ACC (&v)[1]) {
        uint32_t x;
        asm("ld.shared.b32 %0, [%1];" : "=r"(x) : "r"(a));
        v[0] += bits_as<ACC>(x);
    }
    static __device__ __forceinline__ void load(uint32_t a, ACC (&v)[1]) {
        uint32_t x;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(x) : "r"(a) : "memory");
        v[0] = bits_as<ACC>(x);
    }
    static __device__ __forceinline__ void store(uint32_t a, const ACC (&v)[1]) {
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(*(const uint32_t*)&v[0]) : "memory");
    }
};
template <typename ACC>
struct BsCell<ACC, 2> {
    static __device__ __forceinline__ void gather_add(uint32_t a, ACC (&v)[2]) {
        uint32_t x, y;
        asm("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a));
        v[0] += bits_as<ACC>(x);
        v[1] += bits_as<ACC>(y);
    }
    static __device__ __forceinline__ void load(uint32_t a, ACC (&v)[2]) {
        uint32_t x, y;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a) : "memory");
        v[0] = bits_as<ACC>(x);
        v[1] = bits_as<ACC>(y);
    }
    static __device__ __forceinline__ void store(uint32_t a, const ACC (&v)[2]) {
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(*(const uint32_t*)&v[0]), "r"(*(const uint32_t*)&v[1]) : "memory");
    }
};
template <typename ACC>
struct BsCell<ACC, 4> {
    static __device__ __forceinline__ void gather_add(uint32_t a, ACC (&v)[4]) {
        uint32_t x, y, z, w;
        asm("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "r"(a));
        v[0] += bits_as<ACC>(x);
        v[1] += bits_as<ACC>(y);
        v[2] += bits_as<ACC>(z);
        v[3] += bits_as<ACC>(w);
    }
    static __device__ __forceinline__ void load(uint32_t a, ACC (&v)[4]) {
        uint32_t x, y, z, w;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "r"(a) : "memory");
        v[0] = bits_as<ACC>(x);
        v[1] = bits_as<ACC>(y);
        v[2] = bits_as<ACC>(z);
        v[3] = bits_as<ACC>(w);
    }
    static __device__ __forceinline__ void store(uint32_t a, const ACC (&v)[4]) {
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(*(const uint32_t*)&v[0]), "r"(*(const uint32_t*)&v[1]),
                     "r"(*(const uint32_t*)&v[2]), "r"(*(const uint32_t*)&v[3])
                     : "memory");
    }
};

// One index vector of a lane with a single activation row, hand-scheduled: fifteen address computations (a byte
// permute that isolates the id, a multiply-add that scales it by the 128-byte row pitch and adds the lane's table
// base), fifteen gathers, then per word a small add tree into the accumulator and a predicated flush -- store the
// accumulator into the lane's cell of the current ring slot, advance the slot pointer with wrap-around, clear the
// accumulator -- where the flag byte says a list ends.  No branches.
#define BS_ADDR(n, src, sel) "prmt.b32 t, " src ", 0, " sel ";\n\t mad.lo.u32 a" n ", t, 128, %6;\n\t"
#define BS_FLUSH(bit, ST, ZERO)                                                                                     \
    "and.b32 t, fl, " bit ";\n\t setp.ne.u32 p, t, 0;\n\t"                                                          \
    "@p " ST " [%1], %0;\n\t @p add.u32 t, %1, 128;\n\t @p lop3.b32 %1, t, 2047, %7, 0xEA;\n\t @p " ZERO "\n\t"
#define BS_VEC_ASM(LD, ADD, ZERO, ST)                                                                               \
    "{\n\t"                                                                                                         \
    ".reg .b32 a<15>, fl, t;\n\t"                                                                                   \
    ".reg .b32 v<15>, s<2>;\n\t"                                                                                    \
    ".reg .pred p;\n\t"                                                                                             \
    BS_ADDR("0", "%2", "0x4440") BS_ADDR("1", "%2", "0x4441") BS_ADDR("2", "%2", "0x4442") BS_ADDR("3", "%2", "0x4443")    \
    BS_ADDR("4", "%3", "0x4440") BS_ADDR("5", "%3", "0x4441") BS_ADDR("6", "%3", "0x4442") BS_ADDR("7", "%3", "0x4443")    \
    BS_ADDR("8", "%4", "0x4440") BS_ADDR("9", "%4", "0x4441") BS_ADDR("10", "%4", "0x4442") BS_ADDR("11", "%4", "0x4443")  \
    BS_ADDR("12", "%5", "0x4440") BS_ADDR("13", "%5", "0x4441") BS_ADDR("14", "%5", "0x4442")                              \
    "shr.u32 fl, %5, 24;\n\t"                                                                                       \
    LD " v0, [a0];\n\t" LD " v1, [a1];\n\t" LD " v2, [a2];\n\t" LD " v3, [a3];\n\t"                                 \
    LD " v4, [a4];\n\t" LD " v5, [a5];\n\t" LD " v6, [a6];\n\t" LD " v7, [a7];\n\t"                                 \
    LD " v8, [a8];\n\t" LD " v9, [a9];\n\t" LD " v10, [a10];\n\t" LD " v11, [a11];\n\t"                             \
    LD " v12, [a12];\n\t" LD " v13, [a13];\n\t" LD " v14, [a14];\n\t"                                               \
    ADD " s0, v0, v1;\n\t" ADD " s1, v2, v3;\n\t" ADD " s0, s0, s1;\n\t" ADD " %0, %0, s0;\n\t"                     \
    BS_FLUSH("1", ST, ZERO)                                                                                         \
    ADD " s0, v4, v5;\n\t" ADD " s1, v6, v7;\n\t" ADD " s0, s0, s1;\n\t" ADD " %0, %0, s0;\n\t"                     \
    BS_FLUSH("2", ST, ZERO)                                                                                         \
    ADD " s0, v8, v9;\n\t" ADD " s1, v10, v11;\n\t" ADD " s0, s0, s1;\n\t" ADD " %0, %0, s0;\n\t"                   \
    BS_FLUSH("4", ST, ZERO)                                                                                         \
    ADD " s0, v12, v13;\n\t" ADD " s0, s0, v14;\n\t" ADD " %0, %0, s0;\n\t"                                         \
    BS_FLUSH("8", ST, ZERO)                                                                                         \
    "}"

__device__ __forceinline__ void bs_consume_vec(const uint4& q, uint32_t tb, float& acc, uint32_t& ptr, uint32_t ring_lane) {
    uint32_t a = __float_as_uint(acc);
    asm volatile(BS_VEC_ASM("ld.shared.b32", "add.f32", "mov.b32 %0, 0;", "st.shared.b32")
                 : "+r"(a), "+r"(ptr)
                 : "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w), "r"(tb), "r"(ring_lane)
                 : "memory");
    acc = __uint_as_float(a);
}
__device__ __forceinline__ void bs_consume_vec(const uint4& q, uint32_t tb, int& acc, uint32_t& ptr, uint32_t ring_lane) {
    uint32_t a = (uint32_t)acc;
    asm volatile(BS_VEC_ASM("ld.shared.b32", "add.s32", "mov.b32 %0, 0;", "st.shared.b32")
                 : "+r"(a), "+r"(ptr)
                 : "r"(q.x), "r"(q.y), "r"(q.z), "r"(q.w), "r"(tb), "r"(ring_lane)
                 : "memory");
    acc = (int)a;
}

// Adds the 32 lane cells of each of the slots [done, done + 8) of a warp's ring (slot s = list s of the unit) and
// combines (+ list) - (- list) into column sums.  cell_row == nullptr: the sums are final and go to Y (columns from
// `col_first`, the unit's first column in the matrix); otherwise they go to the block's per-(tile, column) cells.
// Lane 4*s + q adds cells 8q .. 8q+7 of slot done + s, starting at a position rotated by s so that the 32 lanes of a
// step read 32 different banks; the order of every sum is fixed by the layout alone.
template <typename ACC, int MP>
__device__ __noinline__ void bs_reduce_batch(const BsParams& p, uint32_t ring, uint32_t done, uint32_t lists, ACC* cell_row, int col_first, int lane) {
    constexpr uint32_t EB = 4u * MP, ROWB = 128u * MP;
    using Cell = BsCell<ACC, MP>;
    __syncwarp();
    const uint32_t s = (uint32_t)lane >> 2, q = (uint32_t)lane & 3u;
    const uint32_t slot = done + s;
    const bool valid = slot < lists;
    ACC sum[MP];
#pragma unroll
    for (int m = 0; m < MP; ++m) sum[m] = 0;
    if (valid) {
        const uint32_t row = ring + (slot & (BS_RING_SLOTS - 1u)) * ROWB + q * 8u * EB;
#pragma unroll
        for (uint32_t jj = 0; jj < 8; ++jj) {
            ACC v[MP];
            Cell::load(row + ((jj + s) & 7u) * EB, v);
#pragma unroll
            for (int m = 0; m < MP; ++m) sum[m] += v[m];
        }
    }
#pragma unroll
    for (int m = 0; m < MP; ++m) {
        sum[m] += __shfl_xor_sync(0xffffffffu, sum[m], 1);
        sum[m] += __shfl_xor_sync(0xffffffffu, sum[m], 2);
        sum[m] -= __shfl_xor_sync(0xffffffffu, sum[m], 4);   // even slots now hold (+) - (-); odd ones are not used
    }
    const uint32_t col = slot >> 1;   // column within the unit
    if (cell_row == nullptr) {
        if (p.epilogue == 0) {
            if ((lane & 7) == 0 && valid) {
#pragma unroll
                for (int m = 0; m < MP; ++m)
                    if (m < p.M) {
                        const size_t o = (size_t)m * p.y_ld + col_first + col;
                        if (p.y_dtype == TLLM_I32) ((int*)p.Y)[o] = (int)sum[m];
                        else store_out(p.Y, p.y_dtype, o, (float)sum[m] * p.scale);
                    }
            }
        } else {
            // columns are (gate, up) pairs: the up column's sum sits eight lanes further on
#pragma unroll
            for (int m = 0; m < MP; ++m) {
                const ACC up = __shfl_down_sync(0xffffffffu, sum[m], 8);
                if ((lane & 15) == 0 && valid && m < p.M)
                    store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + ((col_first + col) >> 1), silu_mul((float)sum[m] * p.scale, (float)up * p.scale2));
            }
        }
    } else if ((lane & 7) == 0 && valid) {
#pragma unroll
        for (int m = 0; m < MP; ++m) cell_row[(size_t)col * MP + m] = sum[m];
    }
    __syncwarp();
}

// A lane's index vectors travel global -> shared memory with per-lane asynchronous copies: BS_DEPTH slots of 512
// bytes per warp, BS_AHEAD copies in flight while the oldest is consumed.  The walk itself is one rolled loop (its
// code stays in the instruction cache) and holds no index data in registers.
#ifndef BS_DEPTH
#define BS_DEPTH 4          // a power of two
#endif
#ifndef BS_AHEAD
#define BS_AHEAD 3          // < BS_DEPTH: the slot being read is never the one being refilled
#endif
#ifndef BS_MIN_BLOCKS
#define BS_MIN_BLOCKS 4     // blocks per SM the one-row kernel's registers leave room for (two and four rows: 2 and 1,
#endif                      // their shared memory allows no more)
#define BS_STAGE_BYTES ((uint32_t)BS_WARPS * BS_DEPTH * 512u)

template <typename ACC, int MP>
__global__ void __launch_bounds__(BS_WARPS * 32, MP == 1 ? BS_MIN_BLOCKS : (MP == 2 ? 2 : 1)) bstream_spmm_kernel(const __grid_constant__ BsParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr uint32_t EB = 4u * MP;                        // bytes of one table entry / lane cell
    constexpr uint32_t ROWB = 128u * MP;                    // one row group of the table, one slot of a ring
    constexpr uint32_t RINGB = BS_RING_SLOTS * ROWB;        // one warp's ring
    constexpr uint32_t TILEB = BS_TABLE_GROUPS * ROWB;      // one tile's table
    constexpr int SH = MP == 1 ? 7 : (MP == 2 ? 8 : 9);     // log2(ROWB)
    constexpr int NT = BS_WARPS * 32;
    using Cell = BsCell<ACC, MP>;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const TsCtaDesc d = cta < BS_MAX_PARAM_BLOCKS ? p.cta[cta] : p.cta_ext[cta];

    // the rings want their base on a multiple of their size (the slot pointer wraps with one mask)
    const uint32_t s0 = smem_u32(smem_raw), base = (s0 + RINGB - 1u) & ~(RINGB - 1u);
    unsigned char* sm = smem_raw + (base - s0);
    const uint32_t ring = base + (uint32_t)warp * RINGB;
    const uint32_t table = base + p.off_table;
    ACC* cells = (ACC*)(sm + p.off_cells);
    const uint32_t* meta = (const uint32_t*)(sm + p.off_meta);
    uint64_t* bars = (uint64_t*)(sm + p.off_bars);
    volatile int* flags = (volatile int*)(bars + 2);   // [0] abort, [1] last-block flag
    const uint32_t bar_meta = smem_u32(bars);
    const uint32_t stage = base + p.off_stage + (uint32_t)warp * (BS_DEPTH * 512u) + (uint32_t)lane * 16u;

    if (tid == 0) {
        mbar_init(bar_meta, 1);
        flags[0] = 0;
        flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    BS_STAMP(0);
    // The next kernel in the stream may start now: what it does before its own griddepcontrol.wait (fetching its
    // tables and its first index vectors) touches nothing this kernel writes.
    pdl_launch_dependents();
    const char* gbytes = (const char*)(p.stream + d.stream_off);
    if (tid == 0) {
        mbar_expect_tx(bar_meta, d.meta_words * 4u);
        bulk_g2s(smem_u32(meta), p.meta + d.meta_off, d.meta_words * 4u, bar_meta);
    } else if (tid == 32) {
        // weights do not depend on the previous kernel: pull the block's index range towards L2 while that one runs
        const size_t bytes = min((size_t)d.nvec * 16u, (size_t)p.l2_prefetch_bytes);
        for (size_t o = 0; o < bytes; o += 16384) l2_prefetch(gbytes + o, (uint32_t)min((size_t)16384, bytes - o));
    }
    // one warp polls the barrier, the others sleep in the hardware barrier; the result travels in the abort flag
    if (warp == 0) {
        const bool ok = __all_sync(0xffffffffu, bounded_wait(bar_meta, 0, flags));
        if (!ok && lane == 0) {
            flags[0] = 1;
            atomicExch(p.status, BS_ERR_META_WAIT);
        }
    }
    __syncthreads();
    BS_STAMP(1);
    if (flags[0] != 0) return;   // the block's table never arrived (reported through the status word): nothing below can run

    const int c0 = (int)meta[0], ncols = (int)meta[1], t0 = (int)meta[2], ntiles = (int)meta[3], j = (int)meta[4], b = (int)meta[5];
    const bool direct = ntiles == 1 && p.k_splits == 1;   // a column's sum is complete inside one unit: no cells, no final pass
    uint32_t at = meta[BS_BLOCK_HEADER + warp];
    const uint32_t at_end = meta[BS_BLOCK_HEADER + warp + 1];
    const uint4* gstream = p.stream + d.stream_off;

    // ---- per-unit state (set by open_unit) ----
    const uint4 *mainp = nullptr, *tailp = nullptr;
    uint32_t nv = 0, min_nv = 0, max_nv = 0;
    // copy of this lane's vector i into its slot (nothing for a lane past its last vector); always one commit group
    auto issue = [&](uint32_t i) {
        if (i < nv) {
            const uint4* gp = i < min_nv ? mainp + (size_t)i * 32u : tailp + i;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stage + (i & (BS_DEPTH - 1u)) * 512u), "l"(gp) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    auto open_unit = [&](const uint32_t* u) {
        min_nv = u[3] & 0xffffu;
        max_nv = u[3] >> 16;
        nv = (u[4 + (lane >> 1)] >> (16 * (lane & 1))) & 0xffffu;
        // this lane's vectors past the shortest lane follow the interleaved part, lane by lane
        const uint32_t extra = nv - min_nv;
        uint32_t incl = extra;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        const uint4* first = gstream + u[0];
        mainp = first + lane;
        tailp = first + (size_t)min_nv * 32u + (incl - extra) - min_nv;
#pragma unroll
        for (uint32_t i = 0; i < BS_AHEAD; ++i) issue(i);
    };
    bool pre = false;
    if (at < at_end) {
        open_unit(meta + at);
        pre = true;
    }

    // everything below reads X or writes scratch / Y: order it behind the previous kernel in the stream
    BS_STAMP(2);
    pdl_wait();
    BS_STAMP(3);

    for (int g0 = 0; g0 < ntiles; g0 += p.resident) {
        const int g1 = min(ntiles, g0 + p.resident);
        if (g0 > 0) __syncthreads();   // every warp is done with the tables of the previous tiles
        // ---- activation tables of tiles [g0, g1): entry k of a tile at k * EB (row group k / 32, lane k % 32).
        // A thread produces 16 bytes of table at a time, so that a warp's stores are conflict-free. ----
        for (int r = 0; r < g1 - g0; ++r) {
            const int kbase = (t0 + g0 + r) * p.T;
            const int rows_here = min(p.T, p.K - kbase);
            const int fill = (rows_here + 31) & ~31;
            unsigned char* tab = sm + p.off_table + (size_t)r * TILEB;
            constexpr int KPC = 4 / MP;   // rows of W per 16-byte chunk: 4, 2 or 1
            constexpr int UF = 4;         // chunks per thread and pass: their loads are all issued before the first store
            struct alignas(16) Q {
                ACC a, b, c, d;
            };
            const int nchunks = fill / KPC;
            // Several activation rows that 128-bit loads can reach: the raw rows are first copied into the (still unused)
            // ring area, row m at m * rows_here elements, with every load of a thread issued before its first store; the
            // table entries are then put together from shared memory.
            const bool staged = MP > 1 && p.x_vec;
            if (staged) {
                if (r > 0) __syncthreads();   // the previous tile's raw rows have been consumed
                const uint32_t eb = act_bytes(p.x_dtype);
                const int vec_per_row = rows_here * (int)eb / 16, total = p.M * vec_per_row;
                for (int v0 = tid; v0 < total; v0 += NT * UF) {
                    uint4 raw[UF];
#pragma unroll
                    for (int u = 0; u < UF; ++u) {
                        const int vi = v0 + u * NT;
                        if (vi < total) {
                            const int m = vi / vec_per_row, o = vi - m * vec_per_row;
                            raw[u] = __ldcg((const uint4*)((const char*)p.X + ((size_t)m * p.x_ld + kbase) * eb) + o);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UF; ++u) {
                        const int vi = v0 + u * NT;
                        if (vi < total) *(uint4*)(sm + (size_t)vi * 16u) = raw[u];
                    }
                }
                __syncthreads();
            }
            for (int c0f = tid; c0f < nchunks; c0f += NT * UF) {
                ACC v[UF][4];
                if (staged) {
#pragma unroll
                    for (int u = 0; u < UF; ++u) {
                        const int k = (c0f + u * NT) * KPC;
#pragma unroll
                        for (int kk = 0; kk < KPC; ++kk)
#pragma unroll
                            for (int m = 0; m < MP; ++m)
                                v[u][kk * MP + m] = (m < p.M && k + kk < rows_here) ? staged_act<ACC>(sm, p.x_dtype, (uint32_t)(m * rows_here + k + kk)) : (ACC)0;
                    }
                } else if (MP == 1 && p.x_vec) {
                    // four consecutive activations of the one row per load (rows_here is a multiple of 16 here)
                    const uint32_t eb = act_bytes(p.x_dtype);
                    uint4 raw[UF];
#pragma unroll
                    for (int u = 0; u < UF; ++u) {
                        const int k = (c0f + u * NT) * KPC;
                        raw[u] = make_uint4(0, 0, 0, 0);
                        if (k < rows_here) {
                            const char* src = (const char*)p.X + (size_t)(kbase + k) * eb;
                            if (eb == 4) raw[u] = __ldcg((const uint4*)src);
                            else if (eb == 2) {
                                const uint2 a = __ldcg((const uint2*)src);
                                raw[u].x = a.x, raw[u].y = a.y;
                            } else raw[u].x = __ldcg((const uint32_t*)src);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UF; ++u) {
                        const uint4 a = raw[u];
                        if (p.x_dtype == TLLM_F32) {
                            v[u][0] = (ACC)__uint_as_float(a.x), v[u][1] = (ACC)__uint_as_float(a.y), v[u][2] = (ACC)__uint_as_float(a.z),
                            v[u][3] = (ACC)__uint_as_float(a.w);
                        } else if (p.x_dtype == TLLM_F16) {
                            const float2 lo = __half22float2(*(const __half2*)&a.x), hi = __half22float2(*(const __half2*)&a.y);
                            v[u][0] = (ACC)lo.x, v[u][1] = (ACC)lo.y, v[u][2] = (ACC)hi.x, v[u][3] = (ACC)hi.y;
                        } else if (p.x_dtype == TLLM_BF16) {
                            const float2 lo = __bfloat1622float2(*(const __nv_bfloat162*)&a.x), hi = __bfloat1622float2(*(const __nv_bfloat162*)&a.y);
                            v[u][0] = (ACC)lo.x, v[u][1] = (ACC)lo.y, v[u][2] = (ACC)hi.x, v[u][3] = (ACC)hi.y;
                        } else {
                            v[u][0] = (ACC)(signed char)(a.x & 0xff), v[u][1] = (ACC)(signed char)((a.x >> 8) & 0xff),
                            v[u][2] = (ACC)(signed char)((a.x >> 16) & 0xff), v[u][3] = (ACC)(signed char)(a.x >> 24);
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < UF; ++u) {
                        const int k = (c0f + u * NT) * KPC;
#pragma unroll
                        for (int kk = 0; kk < KPC; ++kk)
#pragma unroll
                            for (int m = 0; m < MP; ++m)
                                v[u][kk * MP + m] = (m < p.M && k + kk < rows_here)
                                                        ? load_act_cg<ACC>(p.X, p.x_dtype,
                                                                           p.x_layout ? (size_t)(kbase + k + kk) * p.x_ld + m : (size_t)m * p.x_ld + kbase + k + kk)
                                                        : (ACC)0;
                    }
                }
#pragma unroll
                for (int u = 0; u < UF; ++u) {
                    const int c = c0f + u * NT;
                    if (c < nchunks) *(Q*)(tab + (size_t)c * 16u) = Q{v[u][0], v[u][1], v[u][2], v[u][3]};
                }
            }
            // the all-zero row group that padding ids read
            for (int i = tid; i < 32 * MP; i += NT) ((ACC*)(tab + (size_t)BS_NULL_ID * ROWB))[i] = (ACC)0;
        }
        __syncthreads();
        BS_STAMP(4);

        // ---- this warp's units of these tiles ----
        while (at < at_end) {
            const uint32_t* u = meta + at;
            const uint32_t utile = u[2] & 0xffu;
            if ((int)utile >= g1) break;
            const uint32_t col0 = u[1] & 0xffffu, ucols = u[1] >> 16, n_rp = u[2] >> 8;
            const uint32_t lists = 2u * ucols;
            if (!pre) open_unit(u);
            pre = false;
            const uint32_t tb = table + (utile - (uint32_t)g0) * TILEB + (uint32_t)lane * EB;
            const uint32_t ring_lane = ring + (uint32_t)lane * EB;
            uint32_t ptr = ring_lane;   // slot 0: every slot of the previous unit has been reduced
            ACC acc[MP];
#pragma unroll
            for (int m = 0; m < MP; ++m) acc[m] = 0;
            const uint16_t* rps = (const uint16_t*)(u + BS_UNIT_HEADER);
            uint32_t rk = 0, done = 0;
            uint32_t next_rp = n_rp ? rps[0] : 0xffffffffu;
            ACC* const cell_row = direct ? nullptr : cells + ((size_t)utile * ncols + col0) * MP;

#pragma unroll 1
            for (uint32_t i = 0; i < max_nv; ++i) {
                // vector i has landed (the BS_AHEAD - 1 copies issued after it may still be in flight)
                asm volatile("cp.async.wait_group %0;" ::"n"(BS_AHEAD - 1) : "memory");
                uint4 q;
                asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(stage + (i & (BS_DEPTH - 1u)) * 512u) : "memory");
                issue(i + BS_AHEAD);
                if (MP == 1) {
                    if (i < nv) bs_consume_vec(q, tb, acc[0], ptr, ring_lane);
                } else if (i < nv) {
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                    const uint32_t fl = q.w >> 24;
#pragma unroll
                    for (int wd = 0; wd < 4; ++wd) {
                        // ids of one word: gathered into fresh accumulators (a tree, not a chain through acc)
                        ACC part[MP];
#pragma unroll
                        for (int m = 0; m < MP; ++m) part[m] = 0;
#pragma unroll
                        for (int bb = 0; bb < (wd < 3 ? 4 : 3); ++bb) {
                            const uint32_t off = ((w[wd] >> (8 * bb)) & 0xffu) << SH;
                            Cell::gather_add(tb + off, bb & 1 ? part : acc);
                        }
#pragma unroll
                        for (int m = 0; m < MP; ++m) acc[m] += part[m];
                        if (fl & (1u << wd)) {   // a list ends with this word
                            Cell::store(ptr, acc);
                            ptr = ((ptr + ROWB) & (RINGB - 1u)) | ring_lane;
#pragma unroll
                            for (int m = 0; m < MP; ++m) acc[m] = 0;
                        }
                    }
                }
                while (i == next_rp) {   // eight more slots are complete in all 32 lanes
                    bs_reduce_batch<ACC, MP>(p, ring, done, lists, cell_row, c0 + (int)col0, lane);
                    done += BS_BATCH_SLOTS;
                    ++rk;
                    next_rp = rk < n_rp ? rps[rk] : 0xffffffffu;
                }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");   // only empty groups are left: the next unit starts from a clean count
            while (done < lists) {
                bs_reduce_batch<ACC, MP>(p, ring, done, lists, cell_row, c0 + (int)col0, lane);
                done += BS_BATCH_SLOTS;
            }
            at += BS_UNIT_HEADER + ((n_rp + 1u) >> 1);
        }
    }
#ifdef BS_TRACE
    if (g_bs_trace && lane == 0) {
        long long t_;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));
        atomicMax((unsigned long long*)&g_bs_trace[(size_t)blockIdx.x * 8 + 5], (unsigned long long)t_);
        if (warp == 0) g_bs_trace[(size_t)blockIdx.x * 8 + 6] = t_;
    }
#endif
    if (direct) return;

    // ---- sums over the block's tiles, then Y or the split-K hand-over ----
    __syncthreads();
    ACC* partial = (ACC*)p.partial;
    auto tile_sum = [&](int m, int c) -> ACC {
        ACC s = 0;
        for (int t = 0; t < ntiles; ++t) s += cells[((size_t)t * ncols + c) * MP + m];
        return s;
    };
    if (p.k_splits == 1) {
        if (p.epilogue == 0) {
            for (int i = tid; i < p.M * ncols; i += NT) {
                const int m = i / ncols, c = i - m * ncols;
                const ACC s = tile_sum(m, c);
                if (p.y_dtype == TLLM_I32) ((int*)p.Y)[(size_t)m * p.y_ld + c0 + c] = (int)s;
                else store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + c0 + c, (float)s * p.scale);
            }
        } else {
            const int np = ncols >> 1;
            for (int i = tid; i < p.M * np; i += NT) {
                const int m = i / np, c = i - m * np;
                store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (c0 >> 1) + c,
                          silu_mul((float)tile_sum(m, 2 * c) * p.scale, (float)tile_sum(m, 2 * c + 1) * p.scale2));
            }
        }
        return;
    }
    for (int i = tid; i < p.M * ncols; i += NT) {
        const int m = i / ncols, c = i - m * ncols;
        partial[((size_t)j * p.M + m) * p.N + c0 + c] = tile_sum(m, c);
    }
    // the last block of this column range to arrive adds the partial sums in split order
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicAdd(p.counters + b, 1u);
        flags[1] = (prev == (unsigned int)p.k_splits - 1u) ? 1 : 0;
    }
    __syncthreads();
    if (flags[1] == 0) return;
    __threadfence();
    auto total = [&](int m, int c) -> ACC {
        ACC s = 0;
        for (int js = 0; js < p.k_splits; ++js) s += __ldcg(partial + ((size_t)js * p.M + m) * p.N + c0 + c);
        return s;
    };
    if (p.epilogue == 0) {
        for (int i = tid; i < p.M * ncols; i += NT) {
            const int m = i / ncols, c = i - m * ncols;
            const ACC s = total(m, c);
            if (p.y_dtype == TLLM_I32) ((int*)p.Y)[(size_t)m * p.y_ld + c0 + c] = (int)s;
            else store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + c0 + c, (float)s * p.scale);
        }
    } else {
        const int np = ncols >> 1;
        for (int i = tid; i < p.M * np; i += NT) {
            const int m = i / np, c = i - m * np;
            store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (c0 >> 1) + c, silu_mul((float)total(m, 2 * c) * p.scale, (float)total(m, 2 * c + 1) * p.scale2));
        }
    }
    if (tid == 0) p.counters[b] = 0u;
}

}  // namespace tllm
