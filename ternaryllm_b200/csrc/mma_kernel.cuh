// mma_kernel.cuh -- the batched product on the tcgen05 tensor cores of sm_100a.
//
// Above a measured number of activation rows the gather/add kernel of kernels.cuh is issue-bound (its work grows
// with M * nnz).  This kernel instead keeps a second, dense copy of W at two bits per entry ("bit tiles"),
// expands one 128-column x 64-row tile at a time into fp16 / bf16 values in shared memory and multiplies on
// the tensor cores:  D[n, m] = sum_k Wt[n, k] * X[m, k],  A = Wt tile (K-major, 128-byte swizzle, written by
// decoder warps), B = X tile (K-major, the same swizzle, written by TMA from the row-major activations),
// D in tensor memory (fp32).  The ternary values are exact in both formats and products are exact; sums are
// accumulated in fp32.
//
// One persistent block per SM, fifteen warps:
//   warp 0        streams this block's contiguous range of bit tiles into a shared-memory ring (bulk copies)
//   warp 1        owns tensor memory and issues tcgen05.mma (one lane)
//   warps 2..5    epilogue: tensor memory -> registers -> Y (or split-K partial sums)
//   warps 6..13   decoders: bit tile -> swizzled fp16 / bf16 tile (two groups of four warps, alternate tiles)
//   warp 14       loads the activation tiles by TMA
// Work is the flattened list of (output tile, unit) pairs, a unit being 1, 2 or 4 consecutive 64-row slices of K
// (more slices per unit for narrow activation tiles, so that the fixed cost of one hand-over between the roles
// is spread over more bytes).  Up to 64 activation rows the list is
// cut into equal contiguous ranges, one per block (so every SM streams the same number of bytes); tiles that
// straddle two or more blocks are summed in block order by the last block to arrive, which makes the result
// independent of scheduling.  Above 64 rows whole tiles are dealt out and nothing is shared.
//
// Every wait is bounded (see bounded_wait); on a time-out the block raises its abort flag, every role leaves
// its loop, tensor memory is released and the status word reports the failure.
#pragma once
#include <cuda.h>

#include "kernels.cuh"

namespace tllm {

#define MM_TILE_N 128                 // output columns per tile  (the MMA's M)
#define MM_TILE_K 64                  // rows of W per slice      (four MMAs of K = 16); a unit is 1, 2 or 4 slices
#define MM_CHUNK_BYTES 2048           // one bit tile: 128 columns x 16 bytes
#define MM_A_STAGE_BYTES (MM_TILE_N * MM_TILE_K * 2)
#define MM_MAX_STAGES 8
#define MM_MAX_RAW 8
#define MM_THREADS (15 * 32)
#define MM_SPLIT_MAX_NT 64            // widest activation tile that may use the equal-range split
#define MM_ERR_WAIT 3                 // status word: a bounded wait of the tensor-core kernel ran out

struct MmParams {
    const uint4* bits;        // [n_tiles * KB][128]: for tile (nt, kb) and column c, 64 two-bit codes
    void* Y;
    float* partial;           // [2 * gridDim.x][Nt][128] fp32, used by the equal-range split only
    unsigned int* counters;   // [n_tiles][4], zero between launches
    int* status;
    int M, K, N;
    int KB;                   // ceil(K / 64): slices
    int UK;                   // slices per unit: 1, 2 or 4 (the kernel's template argument)
    int KBU;                  // ceil(KB / UK): units per tile
    int n_tiles, m_tiles;
    int Nt;                   // activation rows per tile (the MMA's N): 16, 32, 64, 128 or 256
    int y_dtype, epilogue, y_ld;
    int S;                    // operand stages, one unit each
    int R;                    // bit-tile ring stages, one unit each
    int split;                // 1: equal contiguous unit ranges, 0: whole tiles
    uint32_t idesc;           // tcgen05 instruction descriptor
    uint32_t tmem_cols;       // power of two >= 2 * Nt
    uint32_t pool;            // byte pool of the decoder: byte 1 = high byte of +w, byte 2 = high byte of -w
    float scale, scale2;
};

// ---- tcgen05 / TMA wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], issued by one thread
__device__ __forceinline__ void umma_f16(uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the barrier receives one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 2-D tiled TMA load into this block's own shared memory: coordinates are (element along K, activation row)
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, groups of
// eight rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Sixteen two-bit codes -> eight words of two 16-bit values each.  Code positions inside the word are chosen
// by the packer (see mm_code_bit in packer.cpp) so that one shift and one mask leave the two codes of an output
// word in selector nibbles 1 and 3 of a byte permute; nibbles 0 and 2 select the pool's zero byte, which is the
// low byte of every value (0, +-1.0 in fp16 and +-2.0 in bf16 all have a zero low byte).
__device__ __forceinline__ void mm_decode_word(uint32_t x, uint32_t pool, uint32_t (&o)[8]) {
    o[0] = __byte_perm(pool, 0u, (x << 4) & 0x3030u);
    o[1] = __byte_perm(pool, 0u, (x << 2) & 0x3030u);
    o[2] = __byte_perm(pool, 0u, x & 0x3030u);
    o[3] = __byte_perm(pool, 0u, (x >> 2) & 0x3030u);
    o[4] = __byte_perm(pool, 0u, (x >> 12) & 0x3030u);
    o[5] = __byte_perm(pool, 0u, (x >> 14) & 0x3030u);
    o[6] = __byte_perm(pool, 0u, (x >> 16) & 0x3030u);
    o[7] = __byte_perm(pool, 0u, (x >> 18) & 0x3030u);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// Non-blocking probe of a barrier phase: unlike try_wait it never suspends the thread, so a spinning waiter
// sees the completion within one loop iteration.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ bool bounded_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((it & 63u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > TLLM_WAIT_LIMIT_CLOCKS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// single-lane roles (producers, MMA issuer) spin on the non-blocking probe; warps that wait with all their
// lanes use the blocking try_wait of bounded_wait, which parks them instead of spending issue slots
#define MM_WAIT(bar, par)                                   \
    do {                                                    \
        if (!bounded_spin((bar), (par), abort_flag)) goto done; \
    } while (0)
#define MM_WAIT_BLOCK(bar, par)                             \
    do {                                                    \
        if (!bounded_wait((bar), (par), abort_flag)) goto done; \
    } while (0)
// ring position and the parity of its current round
#define MM_ADVANCE(idx, ph, n) \
    do {                       \
        if (++(idx) == (n)) {  \
            (idx) = 0;         \
            (ph) ^= 1u;        \
        }                      \
    } while (0)

template <int UK>
__global__ void __launch_bounds__(MM_THREADS, 1) mma_spmm_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ MmParams p) {
    extern __shared__ unsigned char mm_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- this block's unit range -----------------------------------------------------------------------
    const long long G = gridDim.x, cta = blockIdx.x, KBU = p.KBU;
    const long long tiles = (long long)p.n_tiles * p.m_tiles, total = tiles * KBU;
    const long long u0 = p.split ? total * cta / G : (tiles * cta / G) * KBU;
    const long long u1 = p.split ? total * (cta + 1) / G : (tiles * (cta + 1) / G) * KBU;
    if (u0 >= u1) return;

    // ---- shared memory ---------------------------------------------------------------------------------
    const uint32_t raw0 = smem_u32(mm_smem);
    const uint32_t base = (raw0 + 1023u) & ~1023u;                 // swizzled tiles need 1024-byte alignment
    const uint32_t S = (uint32_t)p.S, R = (uint32_t)p.R;
    const int Nt = p.Nt, KB = p.KB;
    const uint32_t b_slice = (uint32_t)Nt * 128u;
    const uint32_t a_stage = (uint32_t)UK * MM_A_STAGE_BYTES, b_stage = (uint32_t)UK * b_slice, r_stage = (uint32_t)UK * MM_CHUNK_BYTES;
    const uint32_t a_base = base, b_base = a_base + S * a_stage, r_base = b_base + S * b_stage;
    const uint32_t bar_base = r_base + R * r_stage;
    volatile int* flags = (volatile int*)(mm_smem + (bar_base - raw0) + 8 * 36);   // [0] tensor-memory address, [1] abort
    volatile int* abort_flag = flags + 1;
#define AB_FULL(s) (bar_base + 8u * (uint32_t)(s))
#define AB_EMPTY(s) (bar_base + 8u * (8u + (uint32_t)(s)))
#define RAW_FULL(r) (bar_base + 8u * (16u + (uint32_t)(r)))
#define RAW_EMPTY(r) (bar_base + 8u * (24u + (uint32_t)(r)))
#define ACC_FULL(a) (bar_base + 8u * (32u + (uint32_t)(a)))
#define ACC_EMPTY(a) (bar_base + 8u * (34u + (uint32_t)(a)))

    if (tid == 0) {
        for (int s = 0; s < MM_MAX_STAGES; ++s) {
            mbar_init(AB_FULL(s), 5);      // four decoder warps + the TMA thread's expect_tx arrival
            mbar_init(AB_EMPTY(s), 1);     // tcgen05.commit
        }
        for (int r = 0; r < MM_MAX_RAW; ++r) {
            mbar_init(RAW_FULL(r), 1);
            mbar_init(RAW_EMPTY(r), 4);    // the four decoder warps of the group that took the unit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(ACC_FULL(a), 1);
            mbar_init(ACC_EMPTY(a), 4);    // the four epilogue warps
        }
        flags[0] = 0;
        flags[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) tmem_alloc(smem_u32((const void*)flags), p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = (uint32_t)flags[0];
    pdl_launch_dependents();

    // Every role walks the same list: segments (tile, units [kbu0, kbu1)) of this block's range.
    if (warp == 0) {
        // ---- bit-tile producer: the weights do not depend on the preceding kernel, so this starts at once
        if (lane == 0) {
            uint32_t r = 0, rph = 0;
            for (long long u = u0; u < u1;) {
                const long long tile = u / KBU;
                const int nt = (int)(tile / p.m_tiles);
                const int kbu0 = (int)(u - tile * KBU);
                const int kbu1 = (int)min(KBU, kbu0 + (u1 - u));
                const uint4* src = p.bits + ((size_t)nt * KB + (size_t)kbu0 * UK) * MM_TILE_N;
                for (int kbu = kbu0; kbu < kbu1; ++kbu, src += (size_t)UK * MM_TILE_N) {
                    MM_WAIT(RAW_EMPTY(r), rph ^ 1u);
                    const uint32_t bytes = (uint32_t)min(UK, KB - kbu * UK) * MM_CHUNK_BYTES;
                    mbar_expect_tx(RAW_FULL(r), bytes);
                    bulk_g2s(r_base + r * r_stage, src, bytes, RAW_FULL(r));
                    MM_ADVANCE(r, rph, R);
                }
                u += kbu1 - kbu0;
            }
        }
    } else if (warp == 14) {
        // ---- activation-tile producer: one TMA box per slice, all slices of a unit on one barrier
        if (lane == 0) {
            pdl_wait();
            uint32_t s = 0, sph = 0;
            for (long long u = u0; u < u1;) {
                const long long tile = u / KBU;
                const int row0 = (int)(tile % p.m_tiles) * Nt;
                const int kbu0 = (int)(u - tile * KBU);
                const int kbu1 = (int)min(KBU, kbu0 + (u1 - u));
                for (int kbu = kbu0; kbu < kbu1; ++kbu) {
                    const int nk = min(UK, KB - kbu * UK);
                    MM_WAIT(AB_EMPTY(s), sph ^ 1u);
                    mbar_expect_tx(AB_FULL(s), (uint32_t)nk * b_slice);
                    for (int q = 0; q < nk; ++q)
                        tma_load_2d(b_base + s * b_stage + (uint32_t)q * b_slice, &tmap, (kbu * UK + q) * MM_TILE_K, row0, AB_FULL(s));
                    MM_ADVANCE(s, sph, S);
                }
                u += kbu1 - kbu0;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = p.idesc;
            const uint64_t ad0 = umma_desc_sw128(a_base), bd0 = umma_desc_sw128(b_base);
            const uint32_t a_step = a_stage >> 4, b_step = b_stage >> 4, bq_step = b_slice >> 4;
            uint32_t s = 0, sph = 0, a = 0, aph = 0;
            for (long long u = u0; u < u1;) {
                const long long tile = u / KBU;
                const int kbu0 = (int)(u - tile * KBU);
                const int kbu1 = (int)min(KBU, kbu0 + (u1 - u));
                MM_WAIT(ACC_EMPTY(a), aph ^ 1u);
                tc_fence_after();
                const uint32_t d = tmem + a * (uint32_t)Nt;
                uint32_t acc = 0;
                for (int kbu = kbu0; kbu < kbu1; ++kbu) {
                    const int nk = min(UK, KB - kbu * UK);
                    MM_WAIT(AB_FULL(s), sph);
                    uint64_t ad = ad0 + s * a_step, bd = bd0 + s * b_step;
#pragma unroll
                    for (int q = 0; q < UK; ++q, ad += MM_A_STAGE_BYTES >> 4, bd += bq_step) {
                        if (q < nk) {
#pragma unroll
                            for (int k4 = 0; k4 < MM_TILE_K / 16; ++k4) {     // 16 values = 32 bytes = 2 descriptor address units
                                umma_f16(d, ad + 2u * k4, bd + 2u * k4, idesc, acc);
                                acc = 1;
                            }
                        }
                    }
                    umma_commit(AB_EMPTY(s));
                    MM_ADVANCE(s, sph, S);
                }
                umma_commit(ACC_FULL(a));
                a ^= 1u;
                aph ^= (a == 0);
                u += kbu1 - kbu0;
            }
        }
    } else if (warp >= 6) {
        // ---- decoders: group 0 (warps 6..9) takes even units, group 1 (warps 10..13) odd units
        const int dw = warp - 6, group = dw >> 2, row = (dw & 3) * 32 + lane;
        const uint32_t sw = (uint32_t)(row & 7), pool = p.pool;
        uint32_t s = 0, sph = 0, r = 0, rph = 0, i = 0;
        for (long long u = u0; u < u1;) {
            const long long tile = u / KBU;
            const int kbu0 = (int)(u - tile * KBU);
            const int kbu1 = (int)min(KBU, kbu0 + (u1 - u));
            for (int kbu = kbu0; kbu < kbu1; ++kbu, ++i) {
                if ((int)(i & 1u) == group) {
                    const int nk = min(UK, KB - kbu * UK);
                    MM_WAIT_BLOCK(RAW_FULL(r), rph);
                    uint4 rw[UK];
#pragma unroll
                    for (int q = 0; q < UK; ++q)
                        if (q < nk) rw[q] = ld_shared_v4(r_base + r * r_stage + (uint32_t)q * MM_CHUNK_BYTES + (uint32_t)row * 16u);
                    MM_WAIT_BLOCK(AB_EMPTY(s), sph ^ 1u);
#pragma unroll
                    for (int q = 0; q < UK; ++q) {
                        if (q < nk) {
                            const uint32_t arow = a_base + s * a_stage + (uint32_t)q * MM_A_STAGE_BYTES + (uint32_t)row * 128u;
                            const uint32_t xs[4] = {rw[q].x, rw[q].y, rw[q].z, rw[q].w};
#pragma unroll
                            for (int w4 = 0; w4 < 4; ++w4) {
                                uint32_t o[8];
                                mm_decode_word(xs[w4], pool, o);
                                st_shared_v4(arow + (((uint32_t)(2 * w4) ^ sw) << 4), o[0], o[1], o[2], o[3]);
                                st_shared_v4(arow + (((uint32_t)(2 * w4 + 1) ^ sw) << 4), o[4], o[5], o[6], o[7]);
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make the tiles visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(AB_FULL(s));
                        mbar_arrive(RAW_EMPTY(r));      // the ring stage was read into registers before the decode
                    }
                }
                MM_ADVANCE(s, sph, S);
                MM_ADVANCE(r, rph, R);
            }
            u += kbu1 - kbu0;
        }
    } else {
        // ---- epilogue (warps 2..5): a warp may read the 32 tensor-memory lanes selected by warp % 4
        const int q = warp & 3, nl = q * 32 + lane;
        pdl_wait();
        uint32_t a = 0, aph = 0;
        for (long long u = u0; u < u1;) {
            const long long tile = u / KBU;
            const int nt = (int)(tile / p.m_tiles), mt = (int)(tile % p.m_tiles);
            const int kbu0 = (int)(u - tile * KBU);
            const int kbu1 = (int)min(KBU, kbu0 + (u1 - u));
            MM_WAIT_BLOCK(ACC_FULL(a), aph);
            tc_fence_after();
            const bool full = kbu0 == 0 && kbu1 == p.KBU;
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + a * (uint32_t)Nt;
            float* slot = p.partial + (size_t)(2 * cta + (u == u0 ? 0 : 1)) * (size_t)(MM_TILE_N * Nt);
            const int n = nt * MM_TILE_N + nl;
            auto emit = [&](float v, int m) {      // called by all lanes of the warp with the same m
                if (p.epilogue == 0) {
                    if (m < p.M && n < p.N) store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + n, v * p.scale);
                } else {
                    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                    if (m < p.M && !(nl & 1) && n + 1 < p.N) store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (n >> 1), silu_mul(v * p.scale, other * p.scale2));
                }
            };
            for (int c16 = 0; c16 < Nt; c16 += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + (uint32_t)c16, v);
                if (full && p.epilogue == 0 && p.y_dtype != TLLM_F32 && !(p.y_ld & 1) && ((uintptr_t)p.Y & 3u) == 0 && nt * MM_TILE_N + MM_TILE_N <= p.N) {
                    // 16-bit outputs: neighbouring lanes trade one value per pair of rows, so that every lane
                    // writes two adjacent columns of one row with a single 4-byte store
#pragma unroll
                    for (int t = 0; t < 16; t += 2) {
                        const float e0 = __uint_as_float(v[t]) * p.scale, e1 = __uint_as_float(v[t + 1]) * p.scale;
                        const float mine = (lane & 1) ? e1 : e0, send = (lane & 1) ? e0 : e1;
                        const float got = __shfl_xor_sync(0xffffffffu, send, 1);
                        const int m = mt * Nt + c16 + t + (lane & 1);
                        const float lo = (lane & 1) ? got : mine, hi = (lane & 1) ? mine : got;
                        if (m < p.M) {
                            uint32_t w;
                            if (p.y_dtype == TLLM_F16) w = (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
                            else w = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
                            *(uint32_t*)((char*)p.Y + ((size_t)m * p.y_ld + (n & ~1)) * 2) = w;
                        }
                    }
                } else if (full) {
#pragma unroll
                    for (int t = 0; t < 16; ++t) emit(__uint_as_float(v[t]), mt * Nt + c16 + t);
                } else {
#pragma unroll
                    for (int t = 0; t < 16; ++t) slot[(size_t)(c16 + t) * MM_TILE_N + nl] = __uint_as_float(v[t]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ACC_EMPTY(a));
            if (!full) {
                // The last of the blocks that share this tile adds their partial sums in block order.  Each
                // epilogue warp owns 32 output columns of the tile and runs the hand-over for them by itself.
                const long long first_unit = tile * KBU, last_unit = first_unit + KBU - 1;
                const long long cf = ((first_unit + 1) * G + total - 1) / total - 1, cl = ((last_unit + 1) * G + total - 1) / total - 1;
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    unsigned int* ctr = p.counters + (size_t)tile * 4 + q;
                    last = atomicAdd(ctr, 1u) == (unsigned int)(cl - cf);
                    if (last) *ctr = 0;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    for (int c16 = 0; c16 < Nt; c16 += 16) {
                        float acc[16];
#pragma unroll
                        for (int t = 0; t < 16; ++t) acc[t] = 0.f;
                        for (long long cc = cf; cc <= cl; ++cc) {
                            const long long cu0 = total * cc / G;
                            const float* sl = p.partial + (size_t)(2 * cc + (cu0 >= first_unit ? 0 : 1)) * (size_t)(MM_TILE_N * Nt);
#pragma unroll
                            for (int t = 0; t < 16; ++t) acc[t] += __ldcg(sl + (size_t)(c16 + t) * MM_TILE_N + nl);
                        }
#pragma unroll
                        for (int t = 0; t < 16; ++t) emit(acc[t], mt * Nt + c16 + t);
                    }
                }
            }
            a ^= 1u;
            aph ^= (a == 0);
            u += kbu1 - kbu0;
        }
    }
done:
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, p.tmem_cols);
    }
    if (tid == 0 && flags[1]) atomicExch(p.status, MM_ERR_WAIT);
#undef AB_FULL
#undef AB_EMPTY
#undef RAW_FULL
#undef RAW_EMPTY
#undef ACC_FULL
#undef ACC_EMPTY
}
#undef MM_WAIT
#undef MM_WAIT_BLOCK
#undef MM_ADVANCE

}  // namespace tllm
