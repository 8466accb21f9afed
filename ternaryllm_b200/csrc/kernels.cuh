// kernels.cuh -- sm_100a device code of libtllm.
//
//   tstream_spmm_kernel   the decode product (M = 1..16 rows) on the tile-stream format: one thread block
//                         per SM; the activation tile is staged by TMA bulk copies and expanded into a
//                         bank-replicated shared-memory table, so that a warp-wide gather is free of bank
//                         conflicts; each lane streams one sorted index list with 128-bit loads held in
//                         register batches, gathers, and adds / subtracts only.
//   mcsc_spmm_kernel      the same product directly on the reference's merged tiled CSC arrays
//                         (what ter_tiled_mcsc_spmv / ter_tiled_mcsc_spmm compute,
//                         ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:24-78, :106-308), for callers that hold
//                         those arrays.
//   silu_mul_kernel       SiLU(g)*u (ternaryLLM_CPU/src/initData.hpp:204-210).
//   add_rmsnorm_kernel    residual add + RMSNorm between two products of a decoder layer (the reference leaves
//                         this to stock Hugging Face modules).
//
// HBM-bound integer/byte work: no tensor cores here by design.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tllm.h"
#include "tstream_format.h"

namespace tllm {

// ---------------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(n) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// global -> shared bulk async copy (TMA, untiled): 16-byte aligned addresses, size a multiple of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// hint: bring [p, p+bytes) into L2 (16-byte aligned, size a multiple of 16); nothing waits on it
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void named_bar(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Every spin in this file is bounded: about a second of SM clocks, after which the waiter raises the
// block's abort flag (all other waiters see it and give up too) and the kernel reports through `status`.
#define TLLM_WAIT_LIMIT_CLOCKS (2000000000LL)

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > TLLM_WAIT_LIMIT_CLOCKS) {
            *abort_flag = 1;
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ float load_act_f32(const void* X, int dtype, size_t i) {
    switch (dtype) {
        case TLLM_F32: return __ldg((const float*)X + i);
        case TLLM_F16: return __half2float(__ldg((const __half*)X + i));
        case TLLM_BF16: return __bfloat162float(__ldg((const __nv_bfloat16*)X + i));
        default: return (float)__ldg((const int8_t*)X + i);
    }
}
__device__ __forceinline__ int load_act_i32(const void* X, int dtype, size_t i) { return (int)__ldg((const int8_t*)X + i); }
// Same through L2 only (ld.global.cg): used where the activations may have been written by the kernel that
// precedes this one in the stream while this one was already resident (programmatic dependent launch), so
// that no line cached in an SM's L1 before griddepcontrol.wait can be served.
__device__ __forceinline__ float load_act_f32_cg(const void* X, int dtype, size_t i) {
    switch (dtype) {
        case TLLM_F32: return __ldcg((const float*)X + i);
        case TLLM_F16: return __half2float(__ushort_as_half(__ldcg((const unsigned short*)X + i)));
        case TLLM_BF16: return __bfloat162float(__ushort_as_bfloat16(__ldcg((const unsigned short*)X + i)));
        default: return (float)__ldcg((const signed char*)X + i);
    }
}
__device__ __forceinline__ int load_act_i32_cg(const void* X, int dtype, size_t i) { return (int)__ldcg((const signed char*)X + i); }

__device__ __forceinline__ void store_out(void* Y, int dtype, size_t i, float v) {
    switch (dtype) {
        case TLLM_F32: ((float*)Y)[i] = v; break;
        case TLLM_F16: ((__half*)Y)[i] = __float2half_rn(v); break;
        case TLLM_BF16: ((__nv_bfloat16*)Y)[i] = __float2bfloat16_rn(v); break;
        default: break;
    }
}

// x / (1 + exp(-x)) * y in fp32 with the accurate expf (not the fast-math intrinsic)
__device__ __forceinline__ float silu_mul(float g, float u) { return g * u / (1.0f + expf(-g)); }

// ---------------------------------------------------------------------------------------------------
// tile-stream decode kernel
// ---------------------------------------------------------------------------------------------------
struct TsParams {
    const uint4* stream;
    const uint32_t* meta;
    const void* X;
    void* Y;
    void* partial;            // [k_splits][M][columns] fp32 / int32
    unsigned int* counters;   // [col_blocks], zero between launches
    int* status;              // 0, or an error code written by a block whose bounded wait ran out
    long long* trace;         // optional: 8 globaltimer stamps per block (diagnostics), or nullptr
    int x_dtype, x_layout, y_dtype;
    int M;                    // rows in this launch (<= MP)
    int K, N, T, tiles;
    int col_blocks, cols_per_block, sub_cols, k_splits, tiles_per_cta;
    int lpl_log2;
    int epilogue;             // 0: Y = acc*scale ; 1: columns are (gate,up) pairs, Y[c/2] = silu(g*scale)*(u*scale2)
    int y_ld;                 // row stride of Y in elements
    int x_ld;                 // row-major X: elements between rows (K); column-major X: elements between k (total rows)
    int l2_mode;              // 0: no L2 prefetch of the index range, 1: bulk prefetch by one thread, 2: per-line prefetch by all threads
    int x_tma;                // 1: X is row-major and 16-byte aligned row by row, so tiles of it can be staged by bulk copies
    float scale, scale2;
    const TsCtaDesc* cta_ext;   // all descriptors in device memory; blocks past TS_MAX_CTAS read theirs from here
    TsCtaDesc cta[TS_MAX_CTAS];
};

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TS_STAMP(slot)                                                                       \
    do {                                                                                     \
        if (p.trace && tid == 0) p.trace[(size_t)cta * 8 + (slot)] = global_ns();            \
    } while (0)

#define TS_L2_PREFETCH_BYTES (512u * 1024u)   // per block, at kernel start
#define TS_ERR_META_WAIT 103
#define TS_ERR_X_WAIT 104

// shared-memory carve-up (bytes from a 128-byte aligned base); the same for every launch
#define TS_SMEM_TABLE 0u
#define TS_SMEM_ACC (((TS_MAX_TILE_ROWS + 1) * 128u + 127u) & ~127u)
#define TS_SMEM_STAGE (TS_SMEM_ACC + 16u * TS_MAX_SUB_COLS * 4u)
#define TS_SMEM_META (TS_SMEM_STAGE + TS_STAGE_BYTES)
#define TS_SMEM_BARS (TS_SMEM_META + TS_MAX_META_BYTES)
#define TS_SMEM_TOTAL (TS_SMEM_BARS + 128u)

template <typename T>
__device__ __forceinline__ T bits_as(uint32_t v);
template <>
__device__ __forceinline__ float bits_as<float>(uint32_t v) { return __uint_as_float(v); }
template <>
__device__ __forceinline__ int bits_as<int>(uint32_t v) { return (int)v; }

// One gather of the lane's slice of table row `id`: EB bytes = MP accumulators' worth of activations.
// The table row is 128 bytes = 8 chunks of 16 bytes holding 128/EB copies of the entry; each lane reads
// the copy (and, for entries wider than 16 bytes, the chunk rotation) that makes the 8 lanes of every
// quarter-warp hit 8 different 16-byte bank groups, whatever rows they ask for.  All address arithmetic is
// 32-bit element indexing from a lane-specific shared-memory base: one multiply-add per row id.
template <typename ACC, int MP>
struct Gatherer {
    static constexpr int EB = 4 * MP;
    static constexpr int NCH = EB >= 16 ? EB / 16 : 1;
    struct alignas(8) P2 {
        ACC a, b;
    };
    struct alignas(16) P4 {
        ACC a, b, c, d;
    };
    uint32_t a1;         // shared-memory byte address of this lane's copy (EB == 4: 4-byte entries, 32 copies)
    uint32_t a2;         // EB == 8 : 8-byte entries, 16 copies
    uint32_t a4[NCH];    // EB >= 16: this lane's copy, chunks in rotated order
    int rot;

    __device__ __forceinline__ void init(const unsigned char* table, int lane) {
        const uint32_t t = smem_u32(table);
        a1 = t + (uint32_t)(lane & 31) * 4u;
        a2 = t + (uint32_t)(lane & 15) * 8u;
        const int l8 = lane & 7;
        const int copy = l8 / NCH;
        rot = EB >= 16 ? l8 % NCH : 0;
#pragma unroll
        for (int j = 0; j < NCH; ++j) a4[j] = t + (uint32_t)(EB >= 16 ? copy * NCH + ((rot + j) % NCH) : 0) * 16u;
    }
    // explicit 32-bit shared-memory loads: one multiply-add per row id, no generic-pointer arithmetic
    static __device__ __forceinline__ ACC lds1(uint32_t a) {
        uint32_t v;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
        return bits_as<ACC>(v);
    }
    // both row ids of one 32-bit word of the stream: the address of each is one 16-bit multiply-add
    // (id * 128 + lane base) straight from the packed halves, then one load
    static __device__ __forceinline__ void lds1x2(uint32_t word, uint32_t base, ACC& lo, ACC& hi) {
        uint32_t x, y;
        asm volatile(
            "{\n\t.reg .b16 l, h;\n\t.reg .b32 al, ah;\n\t"
            "mov.b32 {l, h}, %2;\n\t"
            "mad.wide.u16 al, l, 128, %3;\n\t"
            "mad.wide.u16 ah, h, 128, %3;\n\t"
            "ld.shared.b32 %0, [al];\n\t"
            "ld.shared.b32 %1, [ah];\n\t}"
            : "=r"(x), "=r"(y)
            : "r"(word), "r"(base));
        lo = bits_as<ACC>(x);
        hi = bits_as<ACC>(y);
    }
    static __device__ __forceinline__ P2 lds2(uint32_t a) {
        uint32_t x, y;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a));
        P2 r;
        r.a = bits_as<ACC>(x);
        r.b = bits_as<ACC>(y);
        return r;
    }
    static __device__ __forceinline__ P4 lds4(uint32_t a) {
        uint32_t x, y, z, w;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "r"(a));
        P4 r;
        r.a = bits_as<ACC>(x);
        r.b = bits_as<ACC>(y);
        r.c = bits_as<ACC>(z);
        r.d = bits_as<ACC>(w);
        return r;
    }
    // acc += table[id]; accumulators stay in "rotated" chunk order until unrotate()
    __device__ __forceinline__ void add(uint32_t id, ACC (&acc)[MP]) const {
        if (EB == 4) {
            acc[0] += lds1(a1 + id * 128u);
        } else if (EB == 8) {
            const P2 v = lds2(a2 + id * 128u);
            acc[0] += v.a;
            acc[1 % MP] += v.b;
        } else {
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                const P4 v = lds4(a4[j] + id * 128u);
                acc[(4 * j + 0) % MP] += v.a;
                acc[(4 * j + 1) % MP] += v.b;
                acc[(4 * j + 2) % MP] += v.c;
                acc[(4 * j + 3) % MP] += v.d;
            }
        }
    }
    __device__ __forceinline__ void add8(const uint4& q, ACC (&acc)[MP]) const {
        if (EB == 4) {
            // one accumulator: add the eight gathered values as a tree (depth 4) instead of a chain of 8
            ACC v0, v1, v2, v3, v4, v5, v6, v7;
            lds1x2(q.x, a1, v0, v1);
            lds1x2(q.y, a1, v2, v3);
            lds1x2(q.z, a1, v4, v5);
            lds1x2(q.w, a1, v6, v7);
            acc[0] += ((v0 + v1) + (v2 + v3)) + ((v4 + v5) + (v6 + v7));
            return;
        }
        add(q.x & 0xffffu, acc);
        add(q.x >> 16, acc);
        add(q.y & 0xffffu, acc);
        add(q.y >> 16, acc);
        add(q.z & 0xffffu, acc);
        add(q.z >> 16, acc);
        add(q.w & 0xffffu, acc);
        add(q.w >> 16, acc);
    }
    // bring the accumulators back to row order: slot j holds chunk (rot + j) % NCH
    __device__ __forceinline__ void unrotate(ACC (&acc)[MP]) const {
        if (NCH == 2) {
            if (rot) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const ACC t = acc[i];
                    acc[i] = acc[(4 + i) % MP];
                    acc[(4 + i) % MP] = t;
                }
            }
        } else if (NCH == 4) {
            ACC t[MP];
#pragma unroll
            for (int i = 0; i < MP; ++i) t[i] = acc[i];
            if (rot & 1) {   // out[(j+1)%4] = in[j]
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[(4 * ((j + 1) % 4) + i) % MP] = t[(4 * j + i) % MP];
#pragma unroll
                for (int i = 0; i < MP; ++i) t[i] = acc[i];
            }
            if (rot & 2) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[(4 * ((j + 2) % 4) + i) % MP] = t[(4 * j + i) % MP];
            }
        }
    }
};

template <typename ACC>
__device__ __forceinline__ ACC load_act(const void* X, int dtype, size_t i);
template <>
__device__ __forceinline__ float load_act<float>(const void* X, int dtype, size_t i) { return load_act_f32(X, dtype, i); }
template <>
__device__ __forceinline__ int load_act<int>(const void* X, int dtype, size_t i) { return load_act_i32(X, dtype, i); }
template <typename ACC>
__device__ __forceinline__ ACC load_act_cg(const void* X, int dtype, size_t i);
template <>
__device__ __forceinline__ float load_act_cg<float>(const void* X, int dtype, size_t i) { return load_act_f32_cg(X, dtype, i); }
template <>
__device__ __forceinline__ int load_act_cg<int>(const void* X, int dtype, size_t i) { return load_act_i32_cg(X, dtype, i); }

// activation element i of a staged (shared-memory) tile
template <typename ACC>
__device__ __forceinline__ ACC staged_act(const unsigned char* st, int dtype, uint32_t i);
template <>
__device__ __forceinline__ float staged_act<float>(const unsigned char* st, int dtype, uint32_t i) {
    switch (dtype) {
        case TLLM_F32: return ((const float*)st)[i];
        case TLLM_F16: return __half2float(((const __half*)st)[i]);
        case TLLM_BF16: return __bfloat162float(((const __nv_bfloat16*)st)[i]);
        default: return (float)((const signed char*)st)[i];
    }
}
template <>
__device__ __forceinline__ int staged_act<int>(const unsigned char* st, int dtype, uint32_t i) { return (int)((const signed char*)st)[i]; }

__device__ __forceinline__ uint32_t act_bytes(int dtype) { return dtype == TLLM_F32 ? 4u : (dtype == TLLM_I8 ? 1u : 2u); }

// Writes table row k (128 bytes: 128/EB copies of the MP activations of matrix row k) from val[0..MP).
template <typename ACC, int MP>
__device__ __forceinline__ void fill_row(unsigned char* table, int k, int lane, const ACC (&val)[MP]) {
    constexpr int EB = 4 * MP;
    constexpr int NCH = EB >= 16 ? EB / 16 : 1;
    struct alignas(16) P4 {
        ACC a, b, c, d;
    };
    P4* row = (P4*)(table + (size_t)k * 128u);
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
        const int c = (jj + lane) & 7;   // chunk written in this round
        P4 v;
        if (EB == 4) {
            v.a = v.b = v.c = v.d = val[0];
        } else if (EB == 8) {
            v.a = v.c = val[0];
            v.b = v.d = val[1 % MP];
        } else {
            // chunk c holds rows 4*(c % NCH) .. +3
            const int h = c % NCH;
            v.a = val[0];
            v.b = val[1 % MP];
            v.c = val[2 % MP];
            v.d = val[3 % MP];
#pragma unroll
            for (int t = 1; t < NCH; ++t)
                if (h == t) {
                    v.a = val[(4 * t + 0) % MP];
                    v.b = val[(4 * t + 1) % MP];
                    v.c = val[(4 * t + 2) % MP];
                    v.d = val[(4 * t + 3) % MP];
                }
        }
        row[c] = v;
    }
}

// NW warps; NB register batches of D index vectors per lane (NB-1 batches in flight while one is consumed).
template <typename ACC, int MP, int NW, int D, int NB>
__global__ void __launch_bounds__(NW * 32, 1) tstream_spmm_kernel(const __grid_constant__ TsParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int EB = 4 * MP;
    constexpr int NCH = EB >= 16 ? EB / 16 : 1;
    constexpr int NT = NW * 32;
    constexpr int NV = EB == 4 ? 1 : (EB == 8 ? 2 : 4);   // activations per 16-byte table slot

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int b = cta % p.col_blocks, j = cta / p.col_blocks;
    const TsCtaDesc d = cta < TS_MAX_CTAS ? p.cta[cta] : p.cta_ext[cta];

    unsigned char* table = smem + TS_SMEM_TABLE;
    ACC* acc_s = (ACC*)(smem + TS_SMEM_ACC);                   // [MP][sub_cols]
    unsigned char* stage = smem + TS_SMEM_STAGE;
    const uint32_t* meta = (const uint32_t*)(smem + TS_SMEM_META);
    uint64_t* bars = (uint64_t*)(smem + TS_SMEM_BARS);         // [0] unit table arrived, [1] activation chunk arrived
    volatile int* flags = (volatile int*)(bars + 4);           // [0] abort, [1] last-block flag, [2] next group of the wave
    const uint32_t bar_meta = smem_u32(bars), bar_x = smem_u32(bars + 1);

    if (tid == 0) {
        mbar_init(bar_meta, 1);
        mbar_init(bar_x, 1);
        flags[0] = 0;
        flags[1] = 0;
        flags[2] = NW;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    TS_STAMP(0);
    // Let the next kernel in the stream start as SMs drain; nothing it does before its own
    // griddepcontrol.wait touches what this kernel writes.
    pdl_launch_dependents();
    if (tid == 0) {
        mbar_expect_tx(bar_meta, d.meta_words * 4u);
        bulk_g2s(smem_u32(smem + TS_SMEM_META), p.meta + d.meta_off, d.meta_words * 4u, bar_meta);
    }

    const int c0 = b * p.cols_per_block;
    const int ncols = min(p.cols_per_block, p.N - c0);
    const int t0 = j * p.tiles_per_cta;
    const int ntiles = min(p.tiles_per_cta, p.tiles - t0);
    const int nsubs = (ncols + p.sub_cols - 1) / p.sub_cols;
    const int lpl = 1 << p.lpl_log2;
    const bool direct = p.k_splits == 1 && p.tiles_per_cta == 1;   // the block's sums are final: no scratch at all

    // sub-blocks whose sums fit in the accumulator area at once (the area holds 16 * TS_MAX_SUB_COLS cells)
    const int subs_per_wave = max(1, (16 * TS_MAX_SUB_COLS) / (MP * p.sub_cols));
    for (int i = tid; i < 16 * TS_MAX_SUB_COLS; i += NT) acc_s[i] = 0;

    Gatherer<ACC, MP> gat;
    gat.init(table, lane);

    // One warp polls the mbarrier; the others sleep in the hardware barrier instead of spending issue slots
    // on a polling loop.  The result is published through the abort flag.
    if (warp == 0) {
        const bool ok = __all_sync(0xffffffffu, bounded_wait(bar_meta, 0, flags));
        if (!ok && lane == 0) {
            flags[0] = 1;
            atomicExch(p.status, TS_ERR_META_WAIT);
        }
    }
    __syncthreads();
    bool alive = flags[0] == 0;
    TS_STAMP(2);

    // Weights do not depend on the previous kernel.  Pull the block's whole index range towards L2 now (a
    // bounded amount: long ranges are picked up by the loads themselves), and start this warp's first index
    // loads, before waiting for that kernel.
    {
        const char* g = (const char*)(p.stream + d.stream_off);
        const size_t bytes = min((size_t)d.nvec * 16u, (size_t)TS_L2_PREFETCH_BYTES);
        if (p.l2_mode == 1) {
            if (tid == 0)
                for (size_t o = 0; o < bytes; o += 16384) l2_prefetch(g + o, (uint32_t)min((size_t)16384, bytes - o));
        } else if (p.l2_mode == 2) {
            for (size_t o = (size_t)tid * 128u; o < bytes; o += (size_t)NT * 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(g + o));
        }
    }
    const uint4* gstream = p.stream + d.stream_off;
    uint4 buf[NB][D];
    bool pre = false;
    if (alive) {
        // first section of the block, group `warp`
        const uint32_t* sec = meta;
        const uint32_t ndiag = sec[1], nl = sec[2];
        const uint32_t* diag = sec + TS_SEC_HEADER;
        const uint32_t pos = (uint32_t)warp * 32u + lane;
        if ((uint32_t)warp * 32u < (nl << p.lpl_log2)) {
            const uint32_t li = pos >> p.lpl_log2;
            const int len = li < nl ? (int)(diag[ndiag + 1 + li] >> 16) : 0;
            const uint4* ptr = gstream + sec[0] + pos;
#pragma unroll
            for (int dd = 0; dd < D; ++dd)
                if (dd < len) buf[0][dd] = __ldcs(ptr + diag[dd]);
            pre = true;
        }
    }
    TS_STAMP(7);

    // everything below reads X or writes scratch / Y: order it behind the previous kernel in the stream
    pdl_wait();
    TS_STAMP(1);

    ACC* partial = (ACC*)p.partial;
    uint32_t x_phase = 0;
    const uint32_t* sec = meta;   // walks the block's section tables in processing order

    for (int ti = 0; ti < ntiles; ++ti) {
        if (ti > 0) __syncthreads();   // all gathers of the previous tile are done
        // ---- fill the activation table for rows [kbase, kbase+T) plus the zero row T ----
        {
            const int kbase = (t0 + ti) * p.T;
            const int rows_here = min(p.T, p.K - kbase);
            const int slots = (p.T + 1) * 8;
            if (p.x_tma) {
                // raw rows come in by bulk async copies (TMA) and are expanded from shared memory
                const uint32_t e = act_bytes(p.x_dtype);
                const int kc = min(p.T, (int)((TS_STAGE_BYTES / (p.M * e)) / 64u * 64u));
                for (int k0 = 0; k0 < rows_here; k0 += kc) {
                    const int n = min(kc, rows_here - k0);
                    if (tid == 0) {
                        mbar_expect_tx(bar_x, (uint32_t)p.M * n * e);
                        for (int m = 0; m < p.M; ++m)
                            bulk_g2s(smem_u32(stage) + (uint32_t)m * kc * e, (const char*)p.X + ((size_t)m * p.x_ld + kbase + k0) * e, n * e, bar_x);
                    }
                    if (warp == 0 && alive) {
                        const bool ok = __all_sync(0xffffffffu, bounded_wait(bar_x, x_phase, flags));
                        if (!ok && lane == 0) {
                            flags[0] = 1;
                            atomicExch(p.status, TS_ERR_X_WAIT);
                        }
                    }
                    __syncthreads();
                    alive = flags[0] == 0;
                    x_phase ^= 1u;
                    // one table row (128 bytes) per lane: its 8 chunks are written in an order rotated by the
                    // lane number, so that the 8 lanes of a quarter-warp always write 8 different bank groups
                    for (int k = k0 + tid; k < k0 + n; k += NT) {
                        ACC val[MP];
#pragma unroll
                        for (int m = 0; m < MP; ++m) val[m] = m < p.M ? staged_act<ACC>(stage, p.x_dtype, (uint32_t)(m * kc + (k - k0))) : (ACC)0;
                        fill_row<ACC, MP>(table, k, lane, val);
                    }
                    if (k0 + kc < rows_here) __syncthreads();   // the staging buffer is reused by the next chunk
                }
                for (int k = rows_here + tid; k <= p.T; k += NT) {
                    ACC val[MP];
#pragma unroll
                    for (int m = 0; m < MP; ++m) val[m] = 0;
                    fill_row<ACC, MP>(table, k, lane, val);
                }
            } else {
                // generic path (column-major or unaligned activations): loads straight from global memory
                for (int k = tid; k <= p.T; k += NT) {
                    const int kg = kbase + k;
                    const bool live = k < p.T && kg < p.K;
                    ACC val[MP];
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        val[m] = (live && m < p.M) ? load_act_cg<ACC>(p.X, p.x_dtype, p.x_layout ? (size_t)kg * p.x_ld + m : (size_t)m * p.x_ld + kg)
                                                   : (ACC)0;
                    fill_row<ACC, MP>(table, k, lane, val);
                }
            }
        }
        __syncthreads();
        if (ti == 0) TS_STAMP(3);

        // ---- the tile's sections, in waves of as many sub-blocks as have room for their sums in shared memory;
        // inside a wave every warp takes the next group of 32 lanes from a shared counter, so no warp idles
        // while another works through a second group ----
        for (int sub0 = 0; sub0 < nsubs; sub0 += subs_per_wave) {
            const int nsw = min(subs_per_wave, nsubs - sub0);
            const uint32_t* wave_sec = sec;
            // groups in this wave, and the first section after it
            uint32_t wave_groups = 0;
            {
                const uint32_t* q = sec;
                for (int k = 0; k < nsw; ++k) {
                    wave_groups += ((q[2] << p.lpl_log2) + 31u) >> 5;
                    q += TS_SEC_HEADER + q[1] + 1 + q[2];
                }
                sec = q;
            }
            uint32_t f = (uint32_t)warp;   // first group: static, so that it could be prefetched; then the counter
            while (f < wave_groups && alive) {
                // locate section and group of flat index f
                const uint32_t* sc = wave_sec;
                uint32_t g = f;
                int slot = 0;
                for (;; ++slot) {
                    const uint32_t ng = ((sc[2] << p.lpl_log2) + 31u) >> 5;
                    if (g < ng) break;
                    g -= ng;
                    sc += TS_SEC_HEADER + sc[1] + 1 + sc[2];
                }
                const uint32_t ndiag = sc[1], nl = sc[2];
                const uint32_t* diag = sc + TS_SEC_HEADER;
                const uint32_t* lists = diag + ndiag + 1;
                const uint32_t pos = g * 32u + lane;             // lane position in the section's sorted order
                const uint32_t li = pos >> p.lpl_log2;           // sorted list this lane works for
                const uint32_t word = li < nl ? lists[li] : 0u;
                const int len = (int)(word >> 16);               // vectors this lane owns
                const int steps = __shfl_sync(0xffffffffu, len, 0);   // lane 0 has the longest list of the group
                const uint4* ptr = gstream + sc[0] + pos;
                ACC acc[MP];
#pragma unroll
                for (int i = 0; i < MP; ++i) acc[i] = 0;
                // NB register batches of D vectors each.  All loads of a batch are issued back to back, and NB-1
                // batches are in flight while the gathers of the remaining one run.  (A load issued conditionally
                // inside the loop that consumes its neighbours does not overlap with them: measured at about
                // half the bandwidth.)
                auto load_batch = [&](uint4 (&bf)[D], int base) {
#pragma unroll
                    for (int dd = 0; dd < D; ++dd)
                        if (base + dd < len) bf[dd] = __ldcs(ptr + diag[base + dd]);
                };
                auto use_batch = [&](const uint4 (&bf)[D], int base) {
#pragma unroll
                    for (int dd = 0; dd < D; ++dd)
                        if (base + dd < len) gat.add8(bf[dd], acc);
                };
                if (!pre) load_batch(buf[0], 0);
                pre = false;
#pragma unroll
                for (int bb = 1; bb < NB - 1; ++bb) load_batch(buf[bb], bb * D);
                for (int i0 = 0; i0 < steps; i0 += NB * D) {
#pragma unroll
                    for (int bb = 0; bb < NB; ++bb) {
                        load_batch(buf[(bb + NB - 1) % NB], i0 + (bb + NB - 1) * D);
                        use_batch(buf[bb], i0 + bb * D);
                    }
                }
                gat.unrotate(acc);
                for (int o = 1; o < lpl; o <<= 1) {   // lanes that share a list
#pragma unroll
                    for (int i = 0; i < MP; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
                }
                if ((lane & (lpl - 1)) == 0 && li < nl) {
                    // a column's + list and - list are the only two contributions to its cell between two
                    // flushes, so the order in which they arrive cannot change the sum
                    ACC* cell = acc_s + slot * (MP * p.sub_cols) + (word & 0x7fffu);
                    const bool neg = (word & 0x8000u) != 0;
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < p.M) atomicAdd(cell + m * p.sub_cols, neg ? -acc[m] : acc[m]);
                }
                // next group
                uint32_t nf = 0;
                if (lane == 0) nf = (uint32_t)atomicAdd((int*)&flags[2], 1);
                f = __shfl_sync(0xffffffffu, nf, 0);
            }
            __syncthreads();
            // ---- flush the wave's sums ----
            for (int k = 0; k < nsw; ++k) {
                const int sub = sub0 + k;
                const int ns = min(p.sub_cols, ncols - sub * p.sub_cols);
                const int gcol0 = c0 + sub * p.sub_cols;
                ACC* as = acc_s + k * (MP * p.sub_cols);
                if (direct) {
                    if (p.epilogue == 0) {
                        for (int i = tid; i < p.M * ns; i += NT) {
                            const int m = i / ns, c = i - m * ns;
                            const ACC sv = as[m * p.sub_cols + c];
                            as[m * p.sub_cols + c] = 0;
                            if (p.y_dtype == TLLM_I32) ((int*)p.Y)[(size_t)m * p.y_ld + gcol0 + c] = (int)sv;
                            else store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + gcol0 + c, (float)sv * p.scale);
                        }
                    } else {
                        const int np = ns >> 1;
                        for (int i = tid; i < p.M * np; i += NT) {
                            const int m = i / np, c = i - m * np;
                            const float g = (float)as[m * p.sub_cols + 2 * c], up = (float)as[m * p.sub_cols + 2 * c + 1];
                            as[m * p.sub_cols + 2 * c] = 0;
                            as[m * p.sub_cols + 2 * c + 1] = 0;
                            store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (gcol0 >> 1) + c, silu_mul(g * p.scale, up * p.scale2));
                        }
                    }
                } else {
                    for (int i = tid; i < p.M * ns; i += NT) {
                        const int m = i / ns, c = i - m * ns;
                        const ACC sv = as[m * p.sub_cols + c];
                        as[m * p.sub_cols + c] = 0;
                        // the same thread owns this cell of the block's scratch slice in every tile
                        ACC* dst = partial + ((size_t)j * p.M + m) * p.N + gcol0 + c;
                        *dst = ti > 0 ? *dst + sv : sv;
                    }
                }
            }
            if (tid == 0) flags[2] = NW;   // the counter hands out groups NW, NW+1, ... of the next wave
            __syncthreads();
        }
    }
    TS_STAMP(4);

    if (!direct) {
        bool finish = true;
        if (p.k_splits > 1) {
            // split-K: the last block of this column block to arrive adds the partial sums in split order
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int prev = atomicAdd(p.counters + b, 1u);
                flags[1] = (prev == (unsigned int)p.k_splits - 1u) ? 1 : 0;
            }
            __syncthreads();
            finish = flags[1] != 0;
            if (finish) __threadfence();
        }
        TS_STAMP(5);
        if (finish) {
            const int first = p.k_splits > 1 ? 0 : j, count = p.k_splits > 1 ? p.k_splits : 1;
            auto total = [&](int m, int c) -> ACC {
                ACC s = 0;
                for (int js = 0; js < count; ++js) s += __ldcg(partial + ((size_t)(first + js) * p.M + m) * p.N + c0 + c);
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
                const int npairs = ncols >> 1;
                for (int i = tid; i < p.M * npairs; i += NT) {
                    const int m = i / npairs, c = i - m * npairs;
                    const float g = (float)total(m, 2 * c), up = (float)total(m, 2 * c + 1);
                    store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (c0 >> 1) + c, silu_mul(g * p.scale, up * p.scale2));
                }
            }
            if (p.k_splits > 1 && tid == 0) p.counters[b] = 0u;
        }
    }
    TS_STAMP(6);
}

// ---------------------------------------------------------------------------------------------------
// product on the reference's merged tiled CSC arrays: one warp per column, MC rows per pass
// ---------------------------------------------------------------------------------------------------
template <typename ACC, int MC>
__global__ void __launch_bounds__(256) mcsc_spmm_kernel(const void* __restrict__ X, int x_dtype, int x_layout,
                                                         const int16_t* __restrict__ idx, const int32_t* __restrict__ off,
                                                         void* __restrict__ Y, int y_dtype, int M, int N, int K, int T, float scale) {
    const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp_in_block;
    const int m0 = blockIdx.y * MC;
    const size_t batch = blockIdx.z;
    if (n >= N) return;
    const int tiles = (K + T - 1) / T;
    const size_t xb = batch * (size_t)M * K;
    auto xat = [&](int m, int k) -> ACC {
        return load_act<ACC>(X, x_dtype, xb + (x_layout ? (size_t)k * M + m : (size_t)m * K + k));
    };
    ACC acc[MC];
#pragma unroll
    for (int i = 0; i < MC; ++i) acc[i] = 0;
    const int rows = min(MC, M - m0);
    for (int t = 0; t < tiles; ++t) {
        const int4 o = __ldg((const int4*)off + (size_t)n * tiles + t);
        const int base = t * T;
        for (int i = o.x + 2 * lane; i + 1 < o.y; i += 64) {
            const int pr = base + idx[i], qr = base + idx[i + 1];
#pragma unroll
            for (int r = 0; r < MC; ++r)
                if (r < rows) acc[r] += xat(m0 + r, pr) - xat(m0 + r, qr);
        }
        ACC part[MC];
#pragma unroll
        for (int i = 0; i < MC; ++i) part[i] = 0;
        for (int i = o.y + lane; i < o.z; i += 32) {
            const int rr = base + idx[i];
#pragma unroll
            for (int r = 0; r < MC; ++r)
                if (r < rows) part[r] += xat(m0 + r, rr);
        }
#pragma unroll
        for (int r = 0; r < MC; ++r) acc[r] += (ACC)o.w * part[r];
    }
#pragma unroll
    for (int r = 0; r < MC; ++r) {
        ACC v = acc[r];
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0 && r < rows) {
            const size_t at = batch * (size_t)M * N + (size_t)(m0 + r) * N + n;
            if (y_dtype == TLLM_I32) ((int*)Y)[at] = (int)v;
            else store_out(Y, y_dtype, at, (float)v * scale);
        }
    }
}

// g[i] = silu(g[i]) * u[i]
__global__ void silu_mul_kernel(void* g, const void* u, int dtype, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = load_act_f32(g, dtype, (size_t)i), bq = load_act_f32(u, dtype, (size_t)i);
    store_out(g, dtype, (size_t)i, silu_mul(a, bq));
}

// Residual add and RMS normalisation of one row per block, the glue between two ternary products of a decoder
// layer:  x[r] += delta[r] (when delta is given, rounded once to x's type);  h[r] = x[r] * rsqrt(mean(x[r]^2) + eps)
// * weight (weight = 1 when absent).  Sums in fp32; x, delta, h and weight share one 16-bit or 32-bit float type.
// A thread keeps up to four 16-byte vectors of its row in registers between the two passes (rows of up to
// 8192 16-bit or 4096 32-bit values are read once); longer rows re-read the remainder.
template <typename T>
struct RmsVec;   // 16 bytes of T as floats
template <>
struct RmsVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = __ldcg((const float4*)p);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) { *(float4*)p = make_float4(v[0], v[1], v[2], v[3]); }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <>
struct RmsVec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
        const uint4 a = __ldcg((const uint4*)p);
        const __half2* h = (const __half2*)&a;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
        uint4 a;
        __half2* h = (__half2*)&a;
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *(uint4*)p = a;
    }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <>
struct RmsVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 a = __ldcg((const uint4*)p);
        const __nv_bfloat162* h = (const __nv_bfloat162*)&a;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x, v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 a;
        __nv_bfloat162* h = (__nv_bfloat162*)&a;
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *(uint4*)p = a;
    }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// hidden must be a multiple of the vector width and all pointers 16-byte aligned (checked by the caller)
template <typename T>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(T* x, const T* delta, const T* weight, T* h, int hidden, float eps) {
    constexpr int N = RmsVec<T>::N, KEEP = 4;
    __shared__ float red[8];
    const size_t row = (size_t)blockIdx.x * hidden;
    const int nvec = hidden / N;
    float keep[KEEP][8];
    float ss = 0.f;
    auto first_pass = [&](int vi, float (&v)[8]) {
        RmsVec<T>::load(x + row + (size_t)vi * N, v);
        if (delta) {
            float d[8];
            RmsVec<T>::load(delta + row + (size_t)vi * N, d);
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = RmsVec<T>::round(v[i] + d[i]);
            RmsVec<T>::store(x + row + (size_t)vi * N, v);
        }
#pragma unroll
        for (int i = 0; i < N; ++i) ss += v[i] * v[i];
    };
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int vi = threadIdx.x + k * 256;
        if (vi < nvec) first_pass(vi, keep[k]);
    }
    for (int vi = threadIdx.x + KEEP * 256; vi < nvec; vi += 256) {
        float v[8];
        first_pass(vi, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float inv = rsqrtf(tot / (float)hidden + eps);
    auto second_pass = [&](int vi, float (&v)[8]) {
        if (weight) {
            float g[8];
            RmsVec<T>::load(weight + (size_t)vi * N, g);
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = v[i] * inv * g[i];
        } else {
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = v[i] * inv;
        }
        RmsVec<T>::store(h + row + (size_t)vi * N, v);
    };
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int vi = threadIdx.x + k * 256;
        if (vi < nvec) second_pass(vi, keep[k]);
    }
    for (int vi = threadIdx.x + KEEP * 256; vi < nvec; vi += 256) {
        float v[8];
        RmsVec<T>::load(x + row + (size_t)vi * N, v);     // written by this thread in the first pass, or untouched
        second_pass(vi, v);
    }
}

}  // namespace tllm
