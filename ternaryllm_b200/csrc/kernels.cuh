// kernels.cuh -- sm_100a device code of libtllm.
//
//   tstream_spmm_kernel   the decode product (M = 1..16 rows) on the tile-stream format: one persistent
//                         thread block per SM; a producer warp pulls the block's contiguous index stream
//                         through a shared-memory ring with bulk async copies (TMA, mbarrier completion);
//                         consumer warps gather activations from a bank-replicated shared-memory table,
//                         so that a warp-wide gather is free of bank conflicts, and add / subtract only.
//   mcsc_spmm_kernel      the same product directly on the reference's merged tiled CSC arrays
//                         (what ter_tiled_mcsc_spmv / ter_tiled_mcsc_spmm compute,
//                         ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:24-78, :106-308), for callers that hold
//                         those arrays.
//   silu_mul_kernel       SiLU(g)*u (ternaryLLM_CPU/src/initData.hpp:204-210).
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
    const uint32_t* vstart;
    const void* X;
    void* Y;
    void* partial;            // [k_splits][M][columns] fp32 / int32
    unsigned int* counters;   // [col_blocks], zero between launches
    int* status;              // 0, or an error code written by a block whose bounded wait ran out
    int x_dtype, x_layout, y_dtype;
    int M;                    // rows in this launch (<= MP)
    int K, N, T, tiles;
    int col_blocks, cols_per_block, k_splits, tiles_per_cta;
    int lpl_log2, nstages;
    int epilogue;             // 0: Y = acc*scale ; 1: columns are (gate,up) pairs, Y[c/2] = silu(g*scale)*(u*scale2)
    int y_ld;                 // row stride of Y in elements
    int x_ld;                 // row-major X: elements between rows (K); column-major X: elements between k (total rows)
    float scale, scale2;
    TsCtaDesc cta[TS_MAX_CTAS];
};

#define TS_ERR_FULL_WAIT 101
#define TS_ERR_EMPTY_WAIT 102
#define TS_ERR_META_WAIT 103

// shared-memory carve-up (bytes from a 128-byte aligned base)
struct TsSmem {
    uint32_t table, ring, meta, bars, total;
};
__host__ __device__ inline TsSmem ts_smem_layout(int T, int nstages, int meta_bytes) {
    TsSmem s;
    s.table = 0;
    s.ring = (uint32_t)(T + 1) * 128u;
    s.meta = s.ring + (uint32_t)nstages * TS_STAGE_VECS * 16u;
    s.bars = s.meta + (((uint32_t)meta_bytes + 127u) & ~127u);
    s.total = s.bars + 256u;
    return s;
}

// One gather of the lane's slice of table row `id`: EB bytes = MP accumulators' worth of activations.
// The table row is 128 bytes = 8 chunks of 16 bytes holding 128/EB copies of the entry; each lane reads
// the copy (and, for entries wider than 16 bytes, the chunk rotation) that makes the 8 lanes of every
// quarter-warp hit 8 different 16-byte bank groups.
template <typename ACC, int MP>
struct Gatherer {
    static constexpr int EB = 4 * MP;
    static constexpr int NCH = EB >= 16 ? EB / 16 : 1;
    uint32_t off[NCH];   // byte offset inside the 128-byte row for each of the NCH loads
    int rot;

    __device__ __forceinline__ void init(int lane) {
        if (EB == 4) {
            off[0] = (lane & 31) * 4;
            rot = 0;
        } else if (EB == 8) {
            off[0] = (lane & 15) * 8;
            rot = 0;
        } else {
            const int l8 = lane & 7;
            const int copy = l8 / NCH;
            rot = l8 % NCH;
#pragma unroll
            for (int j = 0; j < NCH; ++j) off[j] = (uint32_t)((copy * NCH + ((rot + j) % NCH)) * 16);
        }
    }
    // acc += sign-free table[id]; accumulators stay in "rotated" chunk order until unrotate()
    __device__ __forceinline__ void add(const unsigned char* table, uint32_t id, ACC (&acc)[MP]) const {
        const unsigned char* row = table + (size_t)id * 128u;
        if (EB == 4) {
            acc[0] += *(const ACC*)(row + off[0]);
        } else if (EB == 8) {
            struct alignas(8) P2 {
                ACC a, b;
            };
            const P2 v = *(const P2*)(row + off[0]);
            acc[0] += v.a;
            acc[1] += v.b;
        } else {
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                struct alignas(16) P4 {
                    ACC a, b, c, d;
                };
                const P4 v = *(const P4*)(row + off[j]);
                acc[4 * j + 0] += v.a;
                acc[4 * j + 1] += v.b;
                acc[4 * j + 2] += v.c;
                acc[4 * j + 3] += v.d;
            }
        }
    }
    // bring the accumulators back to row order: slot j holds chunk (rot + j) % NCH
    __device__ __forceinline__ void unrotate(ACC (&acc)[MP]) const {
        if (NCH == 2) {
            if (rot) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const ACC t = acc[i];
                    acc[i] = acc[4 + i];
                    acc[4 + i] = t;
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
                    for (int i = 0; i < 4; ++i) acc[4 * ((j + 1) % 4) + i] = t[4 * j + i];
#pragma unroll
                for (int i = 0; i < MP; ++i) t[i] = acc[i];
            }
            if (rot & 2) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[4 * ((j + 2) % 4) + i] = t[4 * j + i];
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

// NW consumer warps + 1 producer warp.
template <typename ACC, int MP, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, 1) tstream_spmm_kernel(const __grid_constant__ TsParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int EB = 4 * MP;
    constexpr int NCH = EB >= 16 ? EB / 16 : 1;
    constexpr int CT = NW * 32;   // consumer threads

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int b = cta % p.col_blocks, j = cta / p.col_blocks;
    const TsCtaDesc d = p.cta[cta];
    const TsSmem sm = ts_smem_layout(p.T, p.nstages, TS_MAX_META_BYTES);

    unsigned char* table = smem + sm.table;
    const uint4* ring = (const uint4*)(smem + sm.ring);
    const uint32_t* meta = (const uint32_t*)(smem + sm.meta);
    uint64_t* bars = (uint64_t*)(smem + sm.bars);           // [0..7] full, [8..15] empty, [16] meta
    volatile int* flags = (volatile int*)(bars + 20);       // [0] abort, [1] last-block flag
    const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + 8), bar_meta = smem_u32(bars + 16);

    if (tid == 0) {
        for (int s = 0; s < p.nstages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, TS_STAGE_VECS);
        }
        mbar_init(bar_meta, 1);
        flags[0] = 0;
        flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // Let the next kernel in the stream start as SMs drain; it will not touch anything this kernel writes
    // before its own griddepcontrol.wait.
    pdl_launch_dependents();

    const uint32_t nchunks = (d.nvec + TS_STAGE_VECS - 1) / TS_STAGE_VECS;

    if (warp == NW) {
        // ------------------------------ producer: weights only, no dependence on earlier kernels ------
        if (lane == 0) {
            mbar_expect_tx(bar_meta, d.meta_words * 4u);
            bulk_g2s(smem_u32(smem + sm.meta), p.vstart + d.meta_off, d.meta_words * 4u, bar_meta);
            uint32_t issued = 0;
            bool ok = true;
            for (uint32_t i = 0; i < nchunks && ok; ++i) {
                const uint32_t s = i % (uint32_t)p.nstages, g = i / (uint32_t)p.nstages;
                if (g >= 1) ok = bounded_wait(bar_empty + 8 * s, (g - 1) & 1, flags);
                if (!ok) break;
                const uint32_t vecs = min((uint32_t)TS_STAGE_VECS, d.nvec - i * TS_STAGE_VECS);
                mbar_expect_tx(bar_full + 8 * s, vecs * 16u);
                bulk_g2s(smem_u32(smem + sm.ring) + s * (TS_STAGE_VECS * 16u), p.stream + (size_t)d.stream_off + (size_t)i * TS_STAGE_VECS,
                         vecs * 16u, bar_full + 8 * s);
                issued = i + 1;
            }
            if (!ok) {
                atomicExch(p.status, TS_ERR_EMPTY_WAIT);
                // do not leave the block while copies that were issued may still land in its shared memory
                const uint32_t first = issued > (uint32_t)p.nstages ? issued - (uint32_t)p.nstages : 0;
                for (uint32_t i = first; i < issued; ++i) {
                    const uint32_t s = i % (uint32_t)p.nstages, g = i / (uint32_t)p.nstages;
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar_full + 8 * s, g & 1) && clock64() - t0 < TLLM_WAIT_LIMIT_CLOCKS) {
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------- consumers ------------------------------------------------------
    const int c0 = b * p.cols_per_block;
    const int ncols = min(p.cols_per_block, p.N - c0);
    const int t0 = j * p.tiles_per_cta;
    const int ntiles = min(p.tiles_per_cta, p.tiles - t0);
    const int nlists = 2 * ncols;
    const int lpl = 1 << p.lpl_log2;
    const int lists_per_unit = 32 >> p.lpl_log2;
    const int nunits = (nlists + lists_per_unit - 1) / lists_per_unit;
    const uint32_t ring_mask = (uint32_t)p.nstages * TS_STAGE_VECS - 1u;   // nstages is a power of two

    Gatherer<ACC, MP> gat;
    gat.init(lane);

    // everything below reads X or writes scratch / Y: order it behind the previous kernel in the stream
    pdl_wait();

    bool alive = bounded_wait(bar_meta, 0, flags);
    alive = __all_sync(0xffffffffu, alive);
    if (!alive && lane == 0) atomicExch(p.status, TS_ERR_META_WAIT);

    ACC* partial = (ACC*)p.partial;

    for (int ti = 0; ti < ntiles; ++ti) {
        if (ti > 0) named_bar(1, CT);   // all gathers of the previous tile are done
        // ---- fill the activation table for rows [kbase, kbase+T) plus the zero row T ----
        {
            const int kbase = (t0 + ti) * p.T;
            const int slots = (p.T + 1) * 8;
            for (int s = tid; s < slots; s += CT) {
                const int k = s >> 3, q = s & 7;
                const int kg = kbase + k;
                const bool live = (k < p.T) && (kg < p.K);
                struct alignas(16) P4 {
                    ACC a, b, c, d;
                } v;
                v.a = v.b = v.c = v.d = 0;
                if (live) {
                    if (EB == 4) {
                        v.a = load_act<ACC>(p.X, p.x_dtype, p.x_layout ? (size_t)kg * p.x_ld : (size_t)kg);
                        v.b = v.c = v.d = v.a;
                    } else if (EB == 8) {
                        v.a = load_act<ACC>(p.X, p.x_dtype, p.x_layout ? (size_t)kg * p.x_ld : (size_t)kg);
                        if (p.M > 1) v.b = load_act<ACC>(p.X, p.x_dtype, p.x_layout ? (size_t)kg * p.x_ld + 1 : (size_t)p.x_ld + kg);
                        v.c = v.a;
                        v.d = v.b;
                    } else {
                        const int m0 = 4 * (q % NCH);
                        ACC t[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int m = m0 + i;
                            t[i] = m < p.M ? load_act<ACC>(p.X, p.x_dtype, p.x_layout ? (size_t)kg * p.x_ld + m : (size_t)m * p.x_ld + kg) : (ACC)0;
                        }
                        v.a = t[0];
                        v.b = t[1];
                        v.c = t[2];
                        v.d = t[3];
                    }
                }
                *(P4*)(table + (size_t)s * 16) = v;
            }
        }
        named_bar(1, CT);

        const uint32_t* vs = meta + (size_t)ti * (nlists + 1);
        for (int u = warp; u < nunits && alive; u += NW) {
            const int l0 = u * lists_per_unit;
            const int l1 = min(nlists, l0 + lists_per_unit);
            const uint32_t ubeg = vs[l0], uend = vs[l1];
            if (uend > ubeg) {
                for (uint32_t c = ubeg / TS_STAGE_VECS; c <= (uend - 1) / TS_STAGE_VECS && alive; ++c)
                    alive = bounded_wait(bar_full + 8 * (c % (uint32_t)p.nstages), (c / (uint32_t)p.nstages) & 1, flags);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) {
                    if (lane == 0) atomicExch(p.status, TS_ERR_FULL_WAIT);
                    break;
                }
            }
            ACC acc[MP];
#pragma unroll
            for (int i = 0; i < MP; ++i) acc[i] = 0;
            const int mylist = l0 + (lane >> p.lpl_log2);
            if (mylist < l1) {
                const uint32_t vend = vs[mylist + 1];
                for (uint32_t v = vs[mylist] + (uint32_t)(lane & (lpl - 1)); v < vend; v += (uint32_t)lpl) {
                    const uint4 qv = ring[v & ring_mask];
                    gat.add(table, qv.x & 0xffffu, acc);
                    gat.add(table, qv.x >> 16, acc);
                    gat.add(table, qv.y & 0xffffu, acc);
                    gat.add(table, qv.y >> 16, acc);
                    gat.add(table, qv.z & 0xffffu, acc);
                    gat.add(table, qv.z >> 16, acc);
                    gat.add(table, qv.w & 0xffffu, acc);
                    gat.add(table, qv.w >> 16, acc);
                }
            }
            gat.unrotate(acc);
            if (mylist & 1) {
#pragma unroll
                for (int i = 0; i < MP; ++i) acc[i] = -acc[i];
            }
            // sum over the 2*lpl lanes of a column: its + list lanes and its - list lanes
            for (int o = 1; o < 2 * lpl; o <<= 1) {
#pragma unroll
                for (int i = 0; i < MP; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
            }
            if ((lane & (2 * lpl - 1)) == 0 && mylist < l1) {
                const int col = c0 + (mylist >> 1);
#pragma unroll
                for (int m = 0; m < MP; ++m) {
                    if (m < p.M) {
                        ACC* dst = partial + ((size_t)j * p.M + m) * p.N + col;
                        *dst = ti > 0 ? *dst + acc[m] : acc[m];
                    }
                }
            }
            // hand the consumed vectors back to the producer, stage by stage
            __syncwarp();
            if (lane == 0 && uend > ubeg) {
                for (uint32_t c = ubeg / TS_STAGE_VECS; c <= (uend - 1) / TS_STAGE_VECS; ++c) {
                    const uint32_t lo = max(ubeg, c * TS_STAGE_VECS), hi = min(uend, (c + 1) * TS_STAGE_VECS);
                    mbar_arrive_n(bar_empty + 8 * (c % (uint32_t)p.nstages), hi - lo);
                }
            }
        }
    }

    // ---- split-K: the last block of this column block to arrive adds the partial sums in split order ----
    __threadfence();
    named_bar(1, CT);
    if (tid == 0) {
        const unsigned int prev = atomicAdd(p.counters + b, 1u);
        flags[1] = (prev == (unsigned int)p.k_splits - 1u) ? 1 : 0;
    }
    named_bar(1, CT);
    if (flags[1]) {
        __threadfence();
        if (p.epilogue == 0) {
            for (int i = tid; i < p.M * ncols; i += CT) {
                const int m = i / ncols, c = i - m * ncols;
                ACC s = 0;
                for (int js = 0; js < p.k_splits; ++js) s += __ldcg(partial + ((size_t)js * p.M + m) * p.N + c0 + c);
                if (p.y_dtype == TLLM_I32) ((int*)p.Y)[(size_t)m * p.y_ld + c0 + c] = (int)s;
                else store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + c0 + c, (float)s * p.scale);
            }
        } else {
            const int npairs = ncols >> 1;
            for (int i = tid; i < p.M * npairs; i += CT) {
                const int m = i / npairs, c = i - m * npairs;
                float g = 0.f, up = 0.f;
                for (int js = 0; js < p.k_splits; ++js) {
                    const ACC* row = partial + ((size_t)js * p.M + m) * p.N + c0 + 2 * c;
                    g += (float)__ldcg(row);
                    up += (float)__ldcg(row + 1);
                }
                store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (c0 >> 1) + c, silu_mul(g * p.scale, up * p.scale2));
            }
        }
        if (tid == 0) p.counters[b] = 0u;
    }
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

}  // namespace tllm
