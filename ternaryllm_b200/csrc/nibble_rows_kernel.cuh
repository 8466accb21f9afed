// nibble_rows_kernel.cuh -- the decode tensor-core product for 5 to 64 activation rows: the same four-bit planes of W
// streamed by TMA into tcgen05.mma.kind::f8f6f4 as in nibble_kernel.cuh, but with the activation pieces prepared once
// per call by a small kernel and streamed as the B operand by TMA as well.
//
// With up to four rows, every block of nibble_spmm_kernel builds the B operand for its K range in shared memory.  With
// more rows that would not fit and would be repeated by every block.  Here
//   nibble_pieces_kernel   one block per activation row: largest magnitude of the row, power-of-two scaling, split into
//                          e5m2 pieces (see nibble_kernel.cuh), written as rows of a byte matrix P [piece row][K] in global
//                          memory (it stays in L2), plus the power of two that undoes the scaling;
//   nibble_rows_kernel     one persistent block per SM.  Warp 0 streams (A tile, B tile) pairs: A = 128 columns x 128
//                          rows of W as e2m1 codes (tensor map 16U4_ALIGN16B), B = NB piece rows x 128 K as bytes
//                          (plain 8-bit tensor map, 128-byte swizzle); warp 1 issues MMAs of 128 x NB x 32; warps 2..5
//                          add the pieces of a row, undo the scaling and write Y or hand partial sums over.
// The (tile, unit) list is cut into equal contiguous runs, one per block; column tiles shared by two or more blocks are
// added in block order by the last block to arrive, so the result does not depend on scheduling.  Every wait is
// bounded (status word NB_ERR_WAIT).  NB = 32, 64, 128 or 256 piece rows = 8 .. 64 fp16 / bf16 rows, 4 .. 32 fp32 rows.
#pragma once
#include "nibble_kernel.cuh"

namespace tllm {

#define NR_UK 2                       // tiles per unit
#define NR_MAX_NB 256                 // piece rows of one launch
#define NR_MAX_ROWS 64                // activation rows of one launch (fp16 / bf16; half of it for fp32)
#define NR_THREADS 192

struct NpParams {
    const void* X;
    uint8_t* pieces;          // [NR_MAX_NB][k_pad] e5m2 bytes, row m * P + i = piece i of activation row m
    float* row_pow;           // [NR_MAX_ROWS] power of two that undoes a row's scaling
    int M, K, k_pad, x_dtype, x_ld, P;
};

struct NrParams {
    const float* row_pow;
    void* Y;
    float* partial;           // [2 * gridDim.x][M][128] fp32: a block's first and last (partial) column tile
    unsigned int* counters;   // [n_tiles][4], zero between launches
    int* status;
    int M, N;
    int y_dtype, y_ld, epilogue;
    int P;                    // pieces per activation row: 4 or 8
    int NB;                   // piece rows of B (the MMA's N): 32, 64, 128, 256
    int KB;                   // K blocks of 128 rows
    int n_tiles;
    int S;                    // ring stages of one unit each
    uint32_t idesc, tmem_cols;
    float scale, scale2;
};

// one block per activation row
__global__ void __launch_bounds__(256) nibble_pieces_kernel(const __grid_constant__ NpParams p) {
    __shared__ uint32_t red[8];
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool f32 = p.x_dtype == TLLM_F32, bf16 = p.x_dtype == TLLM_BF16;
    const size_t esz = f32 ? 4 : 2;
    const bool vec_ok = ((uintptr_t)p.X % 16 == 0) && (((size_t)p.x_ld * esz) % 16 == 0);
    const size_t row_off = (size_t)m * p.x_ld;
    const int nchunk = p.k_pad / 16;
    pdl_wait();                       // the activations come from the preceding kernel
    pdl_launch_dependents();          // the product may start streaming its weights now
    // ---- largest magnitude of the row (as a bit pattern: for one sign the order of floats is the order of their bits)
    uint32_t mag = 0;
    for (int c = tid; c < nchunk; c += 256) {
        if (f32) {
            uint4 v[4];
            nb_load_raw<4>(p.X, row_off, c * 16, p.K, vec_ok, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) mag = max(mag, max(max(v[i].x & 0x7FFFFFFFu, v[i].y & 0x7FFFFFFFu), max(v[i].z & 0x7FFFFFFFu, v[i].w & 0x7FFFFFFFu)));
        } else {
            uint4 v[2];
            nb_load_raw<2>(p.X, row_off, c * 16, p.K, vec_ok, v);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                for (int t = 0; t < 4; ++t) mag = max(mag, max(w[t] & 0x7FFFu, (w[t] >> 16) & 0x7FFFu));
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mag = max(mag, __shfl_xor_sync(0xffffffffu, mag, o));
    if (lane == 0) red[warp] = mag;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) mag = max(mag, red[i]);
    const float amax = f32 ? __uint_as_float(mag) : (bf16 ? __uint_as_float(mag << 16) : __half2float(__ushort_as_half((unsigned short)mag)));
    int e = amax > 0.f && amax <= 3.0e38f ? ilogbf(amax) - 14 : 0;      // amax * 2^-e in [2^14, 2^15)
    e = max(-126, min(112, e));
    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
    if (tid == 0) p.row_pow[m] = __uint_as_float((uint32_t)(127 + e) << 23);
    // ---- pieces
    uint8_t* out = p.pieces + (size_t)m * p.P * p.k_pad;
    for (int c = tid; c < nchunk; c += 256) {
        float r[16];
        if (f32) {
            uint4 v[4];
            nb_load_raw<4>(p.X, row_off, c * 16, p.K, vec_ok, v);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                r[4 * i] = __uint_as_float(v[i].x) * down, r[4 * i + 1] = __uint_as_float(v[i].y) * down;
                r[4 * i + 2] = __uint_as_float(v[i].z) * down, r[4 * i + 3] = __uint_as_float(v[i].w) * down;
            }
        } else {
            uint4 v[2];
            nb_load_raw<2>(p.X, row_off, c * 16, p.K, vec_ok, v);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    if (bf16) {
                        r[8 * i + 2 * t] = __uint_as_float(w[t] << 16) * down;
                        r[8 * i + 2 * t + 1] = __uint_as_float(w[t] & 0xFFFF0000u) * down;
                    } else {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
                        r[8 * i + 2 * t] = f.x * down, r[8 * i + 2 * t + 1] = f.y * down;
                    }
                }
            }
        }
        int row0 = 0;
        auto emit = [&](uint32_t (&hw)[8], int n) {
            for (int pc = 0; pc < n; ++pc) {
                uint32_t top[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    top[i] = hw[i] & 0xFF00FF00u;
                    const __half2 rest = __hsub2(*reinterpret_cast<const __half2*>(&hw[i]), *reinterpret_cast<const __half2*>(&top[i]));
                    hw[i] = *reinterpret_cast<const uint32_t*>(&rest);
                }
                *(uint4*)(out + (size_t)(row0 + pc) * p.k_pad + (size_t)c * 16) =
                    make_uint4(__byte_perm(top[0], top[1], 0x7531), __byte_perm(top[2], top[3], 0x7531), __byte_perm(top[4], top[5], 0x7531),
                               __byte_perm(top[6], top[7], 0x7531));
            }
            row0 += n;
        };
        uint32_t hw[8];
        if (!f32) {
#pragma unroll
            for (int t = 0; t < 8; ++t) hw[t] = pack_half2_rz(r[2 * t], r[2 * t + 1]);
            emit(hw, 4);
        } else {
#pragma unroll
            for (int round = 0; round < 3; ++round) {
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    hw[t] = pack_half2_rz(r[2 * t], r[2 * t + 1]);
                    if (round < 2) {
                        hw[t] &= 0xFFFCFFFCu;
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[t]));
                        r[2 * t] -= f.x, r[2 * t + 1] -= f.y;
                    }
                }
                emit(hw, round < 2 ? 3 : 2);
            }
        }
    }
}

#define NR_WAIT(bar, par)                                      \
    do {                                                       \
        if (!bounded_spin((bar), (par), abort_flag)) goto done; \
    } while (0)
#define NR_WAIT_BLOCK(bar, par)                                \
    do {                                                       \
        if (!bounded_wait((bar), (par), abort_flag)) goto done; \
    } while (0)
#define NR_ADVANCE(idx, ph, n) \
    do {                       \
        if (++(idx) == (n)) {  \
            (idx) = 0;         \
            (ph) ^= 1u;        \
        }                      \
    } while (0)

__global__ void __launch_bounds__(NR_THREADS, 1) nibble_rows_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap bmap,
                                                                    const __grid_constant__ NrParams p) {
    extern __shared__ unsigned char nr_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KU = (p.KB + NR_UK - 1) / NR_UK;                      // units per column tile
    const long long G = gridDim.x, cta = blockIdx.x;
    const long long total = (long long)p.n_tiles * KU;
    const int u0 = (int)(total * cta / G), u1 = (int)(total * (cta + 1) / G);
    if (u0 >= u1) return;

    const uint32_t raw0 = smem_u32(nr_smem);
    const uint32_t base = (raw0 + 1023u) & ~1023u;
    const uint32_t S = (uint32_t)p.S, NB = (uint32_t)p.NB;
    const uint32_t a_stage = NR_UK * NB_A_STAGE_BYTES, b_tile = NB * 128u, b_stage = NR_UK * b_tile;
    const uint32_t a_base = base, b_base = a_base + S * a_stage;
    const uint32_t bar_base = b_base + S * b_stage;
    unsigned char* tail = nr_smem + (bar_base - raw0);
    volatile int* flags = (volatile int*)(tail + 8 * 24);          // [0] tensor-memory address, [1] abort
    volatile int* abort_flag = flags + 1;
    float* row_pow = (float*)(tail + 8 * 24 + 16);                 // [NR_MAX_ROWS]
#define A_FULL(s) (bar_base + 8u * (uint32_t)(s))
#define A_EMPTY(s) (bar_base + 8u * (8u + (uint32_t)(s)))
#define ACC_FULL(a) (bar_base + 8u * (16u + (uint32_t)(a)))
#define ACC_EMPTY(a) (bar_base + 8u * (18u + (uint32_t)(a)))

    if (tid == 0) {
        for (int s = 0; s < NB_MAX_STAGES; ++s) {
            mbar_init(A_FULL(s), 1);
            mbar_init(A_EMPTY(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(ACC_FULL(a), 1);
            mbar_init(ACC_EMPTY(a), 4);
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

    if (warp == 0) {
        // ---- producer.  The weights do not depend on the preceding kernel: the first ring of A tiles goes out before the
        // dependency wait, the B tiles (the pieces kernel's output) after it; each stage's barrier counts both.
        uint32_t s = 0, sph = 0;
        int tile = u0 / KU, ku = u0 - tile * KU;
        const int pre = min((int)S, u1 - u0);
        auto unit_bytes = [&](int k) { return (uint32_t)min(NR_UK, p.KB - k * NR_UK) * (NB_A_TILE_BYTES + b_tile); };
        auto load_a = [&](uint32_t st, int tl, int k) {
            const int nk = min(NR_UK, p.KB - k * NR_UK);
#pragma unroll
            for (int t = 0; t < NR_UK; ++t)
                if (t < nk) tma_load_2d(a_base + st * a_stage + (uint32_t)t * NB_A_STAGE_BYTES, &wmap, (k * NR_UK + t) * NB_TILE_K, tl * NB_TILE_N, A_FULL(st));
        };
        auto load_b = [&](uint32_t st, int k) {
            const int nk = min(NR_UK, p.KB - k * NR_UK);
#pragma unroll
            for (int t = 0; t < NR_UK; ++t)
                if (t < nk) tma_load_2d(b_base + st * b_stage + (uint32_t)t * b_tile, &bmap, (k * NR_UK + t) * NB_TILE_K, 0, A_FULL(st));
        };
        {
            int tl = tile, k = ku;
            for (int i = 0; i < pre; ++i) {
                if (elect_one()) {
                    mbar_expect_tx(A_FULL((uint32_t)i), unit_bytes(k));
                    load_a((uint32_t)i, tl, k);
                }
                __syncwarp();
                if (++k == KU) k = 0, ++tl;
            }
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
            if (elect_one()) load_b((uint32_t)i, ku);
            __syncwarp();
            NR_ADVANCE(s, sph, S);
            if (++ku == KU) ku = 0, ++tile;
        }
        for (int u = u0 + pre; u < u1; ++u) {
            NR_WAIT_BLOCK(A_EMPTY(s), sph ^ 1u);
            if (elect_one()) {
                mbar_expect_tx(A_FULL(s), unit_bytes(ku));
                load_a(s, tile, ku);
                load_b(s, ku);
            }
            __syncwarp();
            NR_ADVANCE(s, sph, S);
            if (++ku == KU) ku = 0, ++tile;
        }
    } else if (warp == 1) {
        // ---- MMA issuer (whole warp converged, one elected lane per instruction)
        const uint32_t idesc = p.idesc;
        const uint32_t a_lo0 = (a_base >> 4) & 0x3FFFu, b_lo0 = (b_base >> 4) & 0x3FFFu;
        uint32_t s = 0, sph = 0, a = 0, aph = 0;
        int ku0 = u0 % KU;
        for (int u = u0; u < u1;) {
            const int ku1 = min(KU, ku0 + (u1 - u));
            NR_WAIT(ACC_EMPTY(a), aph ^ 1u);
            tc_fence_after();
            const uint32_t d = tmem + a * NB;
            uint32_t acc = 0;
            for (int ku = ku0; ku < ku1; ++ku) {
                NR_WAIT(A_FULL(s), sph);
                const int nk = min(NR_UK, p.KB - ku * NR_UK);
                const uint32_t a_lo = a_lo0 + s * (a_stage >> 4), b_lo = b_lo0 + s * (b_stage >> 4);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t t = 0; t < NR_UK; ++t)
                        if ((int)t < nk) {
#pragma unroll
                            for (uint32_t k4 = 0; k4 < NB_TILE_K / 32; ++k4)
                                umma_f8f6f4_lo(d, a_lo + t * (NB_A_STAGE_BYTES >> 4) + 2u * k4, b_lo + t * (b_tile >> 4) + 2u * k4, idesc, (t | k4) == 0 ? acc : 1u);
                        }
                    umma_commit(A_EMPTY(s));
                }
                __syncwarp();
                acc = 1;
                NR_ADVANCE(s, sph, S);
            }
            if (elect_one()) umma_commit(ACC_FULL(a));
            __syncwarp();
            a ^= 1u;
            aph ^= (a == 0);
            u += ku1 - ku0;
            ku0 = 0;
        }
    } else {
        // ---- epilogue (warps 2..5): a warp may read the 32 tensor-memory lanes selected by warp % 4
        const int ct = tid - 64, q = warp & 3, nl = q * 32 + lane;
        const int P = p.P;
        pdl_wait();
        if (ct < p.M) row_pow[ct] = __ldcg(p.row_pow + ct);
        named_bar(1, 128);
        uint32_t a = 0, aph = 0;
        int tile = u0 / KU, ku0 = u0 - tile * KU;
        for (int u = u0; u < u1;) {
            const int ku1 = min(KU, ku0 + (u1 - u));
            NR_WAIT_BLOCK(ACC_FULL(a), aph);
            tc_fence_after();
            const bool full = ku0 == 0 && ku1 == KU;
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + a * NB;
            const int n = tile * NB_TILE_N + nl;
            float* slot = p.partial + (size_t)(2 * cta + (u == u0 ? 0 : 1)) * (size_t)(NB_TILE_N * NR_MAX_ROWS);
            auto emit = [&](float v, int m) {      // called by all lanes of the warp with the same m
                if (p.epilogue == 0) {
                    if (n < p.N) store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + n, v * p.scale);
                } else {
                    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                    if (!(nl & 1) && n + 1 < p.N) store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (n >> 1), silu_mul(v * p.scale, other * p.scale2));
                }
            };
            const int cols = p.M * P;
            for (int c16 = 0; c16 < cols; c16 += 16) {
                uint32_t v[16];
                tmem_ld16(taddr + (uint32_t)c16, v);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // four consecutive columns are the four pieces of one 16-bit row; eight are the pieces of one fp32 row
                    const float s4 = ((__uint_as_float(v[4 * j + 3]) + __uint_as_float(v[4 * j + 2])) + __uint_as_float(v[4 * j + 1])) + __uint_as_float(v[4 * j]);
                    if (P == 4) {
                        const int m = c16 / 4 + j;
                        if (m < p.M) {
                            const float y = s4 * row_pow[m];
                            if (full) emit(y, m);
                            else slot[(size_t)m * NB_TILE_N + nl] = y;
                        }
                    } else if (j & 1) {
                        const float lo4 = ((__uint_as_float(v[4 * j + 3]) + __uint_as_float(v[4 * j + 2])) + __uint_as_float(v[4 * j + 1])) + __uint_as_float(v[4 * j]);
                        const float hi4 = ((__uint_as_float(v[4 * j - 1]) + __uint_as_float(v[4 * j - 2])) + __uint_as_float(v[4 * j - 3])) + __uint_as_float(v[4 * j - 4]);
                        const int m = c16 / 8 + (j >> 1);
                        if (m < p.M) {
                            const float y = (lo4 + hi4) * row_pow[m];     // the later pieces are the smaller ones
                            if (full) emit(y, m);
                            else slot[(size_t)m * NB_TILE_N + nl] = y;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ACC_EMPTY(a));
            if (!full) {
                // the last of the blocks that share this column tile adds their parts in block order
                const long long first_unit = (long long)tile * KU, last_unit = first_unit + KU - 1;
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
                    // eight rows at a time: their loads are independent, so a step costs one round trip to L2, not eight
                    // (wider batches cost registers and measured slower up to 16 rows, where this kernel is used most)
                    for (int m0 = 0; m0 < p.M; m0 += 8) {
                        float acc[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
                        for (long long c2 = cf; c2 <= cl; ++c2) {
                            const long long cu0 = total * c2 / G;
                            const float* sl = p.partial + (size_t)(2 * c2 + (cu0 >= first_unit ? 0 : 1)) * (size_t)(NB_TILE_N * NR_MAX_ROWS) + nl;
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (m0 + i < p.M) acc[i] += __ldcg(sl + (size_t)(m0 + i) * NB_TILE_N);
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (m0 + i < p.M) emit(acc[i], m0 + i);
                    }
                }
            }
            a ^= 1u;
            aph ^= (a == 0);
            u += ku1 - ku0;
            ku0 = 0;
            ++tile;
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
    if (tid == 0 && flags[1]) atomicExch(p.status, NB_ERR_WAIT);
#undef A_FULL
#undef A_EMPTY
#undef ACC_FULL
#undef ACC_EMPTY
}
#undef NR_WAIT
#undef NR_WAIT_BLOCK
#undef NR_ADVANCE

}  // namespace tllm
