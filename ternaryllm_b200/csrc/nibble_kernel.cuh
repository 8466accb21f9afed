// nibble_kernel.cuh -- the decode product (one to a few activation rows) on the tcgen05 tensor cores, with W streamed
// from HBM by TMA in a form the tensor core reads as it is.
//
// The gather kernel of bstream_kernel.cuh spends one shared-memory load per non-zero and is bound by the load/store
// pipe of the SM, not by HBM.  This kernel keeps a third copy of W: the transpose, one 4-bit code per entry (the fp4
// format e2m1: 0x0 = 0, 0x2 = +1.0, 0xA = -1.0), K contiguous ("nibble planes", nibble_format.h).  A tensor map of
// type 16U4_ALIGN16B copies a 128-column x 128-row tile of it into shared memory in the padded layout that
// tcgen05.mma.kind::f8f6f4 takes for 4-bit operands, so no thread ever touches a weight: HBM -> TMA -> tensor core.
// Half a byte per entry whatever the sparsity; below about 90 % zeros that is less than the two bytes per non-zero of
// the reference's lists, and the kernel runs at the speed the bytes arrive.
//
//   D[n, r] = sum_k Wt[n, k] * B[r, k]        A = Wt tile (M = 128 columns of W, K-major, 128-byte swizzle, e2m1)
//                                             B = activation pieces (N = 16 rows, K-major, the same swizzle, e5m2)
//                                             D in tensor memory, fp32
//
// Activations as e5m2 without losing bits: the row x (fp16 / bf16 / fp32) is scaled by a power of two so that its
// largest magnitude inside the block's K range lies in [2^14, 2^15), and split into pieces x' = p0 + p1 + ... with
// p_i = e5m2(the remainder rounded toward zero).  Each piece takes three significant bits, the remainder is exact in
// fp32, so four pieces carry fp16 and bf16 values exactly and eight carry fp32 (bits more than 31 binary places below
// the range's largest magnitude are dropped: below the rounding of the fp32 sum itself).  The pieces are rows of B;
// products with 0 / +-1 are exact, sums are fp32 in the tensor core, and the epilogue adds the pieces of a row and
// undoes the power of two.  Integer-valued activations therefore give bit-exact results, like the gather kernel.
//
// One persistent block per SM, six warps:
//   warp 0        TMA producer: this block's contiguous range of weight tiles into a ring of 16 KiB stages
//   warp 1        owns tensor memory, issues tcgen05.mma (one lane)
//   warps 2..5    first build B for the block's K range in shared memory (the weights are already streaming), then
//                 run the epilogue: tensor memory -> registers -> Y, or partial sums for the hand-over below
// K is cut into `k_splits` ranges of at most 4096 rows (so that B fits in shared memory); every range has the same
// number of blocks, and the (tile, K block) list of a range is cut into equal contiguous runs, one per block.  Column
// tiles that receive sums from several blocks are added in a fixed order by the last block to arrive.
//
// Every wait is bounded; on a time-out the block raises its abort flag, all roles leave, tensor memory is released
// and the status word reports NB_ERR_WAIT.
#pragma once
#include "mma_kernel.cuh"

namespace tllm {

#define NB_TILE_N 128                 // columns of W per tile (the MMA's M)
#define NB_TILE_K 128                 // rows of W per tile (four MMAs of K = 32)
#define NB_A_STAGE_BYTES 16384        // shared-memory footprint of a tile: 8 bytes of codes, 8 bytes of gap, ...
#define NB_A_TILE_BYTES 8192          // bytes of a tile in global memory = bytes the copy reports to the barrier
#define NB_ROWS 16                    // piece rows of B (the MMA's N)
#define NB_MAX_STAGES 4               // ring stages of one unit each (a unit is UK tiles: one barrier round and one tcgen05.commit)
#define NB_MAX_KBS 32                 // K blocks of one range: B = 32 * 16 * 128 bytes = 64 KiB
#define NB_THREADS 192
#define NB_ERR_WAIT 4                 // status word: a bounded wait of this kernel ran out

struct NbParams {
    const void* X;
    void* Y;
    float* partial;           // [k_splits][n_tiles + blocks_per_split][M][128] fp32
    unsigned int* counters;   // [n_tiles][4], zero between launches
    const uint32_t* sched;    // [n_tiles] blocks that hold a part of the tile, then [k_splits][n_tiles] first | last << 16 of them per range
    int* status;
    int M, K, N;
    int x_dtype, x_ld;        // row-major activations, leading dimension in elements
    int y_dtype, y_ld, epilogue;
    int P;                    // pieces per activation row: 4 (fp16, bf16) or 8 (fp32); M * P <= NB_ROWS
    int KB;                   // K blocks of 128 rows (K rounded up)
    int KBS;                  // K blocks per range (the last range may hold fewer)
    int k_splits, n_tiles;
    int Gj;                   // blocks per range; gridDim.x = k_splits * Gj
    int S;                    // ring stages
    uint32_t idesc, tmem_cols, tx_bytes;
    float scale, scale2;
    int debug;                // diagnostic builds: 1 = issue no MMA, 2 = copy no tile
};

__device__ __forceinline__ void umma_f8f6f4(uint32_t d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the same with the shared-memory descriptors given by their low words (start address >> 4; the upper word -- stride
// between eight-row groups 1024 bytes, version 1, 128-byte swizzle -- is a constant)
__device__ __forceinline__ void umma_f8f6f4_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\t"
        "mov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t}" ::"r"(d),
        "r"(a_lo | (1u << 16)), "r"(b_lo | (1u << 16)), "r"(idesc), "r"(accumulate), "r"(0x40004040u)
        : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float (&v)[8]) {
    uint32_t r[4];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
#pragma unroll
    for (int i = 4; i < 8; ++i) v[i] = 0.f;
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// two floats -> two fp16 values in one word (low half first), rounded toward zero
__device__ __forceinline__ uint32_t pack_half2_rz(float lo, float hi) {
    uint32_t d;
    asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
// Sixteen fp16 values (eight words) -> `n` rows of sixteen e5m2 pieces.  e5m2 is the upper byte of fp16: a piece is the
// value with its low byte cut off (three significant bits, rounded toward zero), and value - piece is exact in fp16.
// `dst(pc)` gives the shared-memory address of the 16-byte chunk of piece row pc.
template <typename F>
__device__ __forceinline__ void nb_emit_pieces(uint32_t (&hw)[8], int n, F dst) {
    for (int pc = 0; pc < n; ++pc) {
        uint32_t top[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            top[i] = hw[i] & 0xFF00FF00u;
            const __half2 rest = __hsub2(*reinterpret_cast<const __half2*>(&hw[i]), *reinterpret_cast<const __half2*>(&top[i]));
            hw[i] = *reinterpret_cast<const uint32_t*>(&rest);
        }
        // bytes 1 and 3 of two words = the pieces of four consecutive values
        st_shared_v4(dst(pc), __byte_perm(top[0], top[1], 0x7531), __byte_perm(top[2], top[3], 0x7531), __byte_perm(top[4], top[5], 0x7531),
                     __byte_perm(top[6], top[7], 0x7531));
    }
}

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

#ifdef NB_DEBUG
__device__ long long* g_nb_trace = nullptr;
#define NB_STAMP(slot)                                               \
    do {                                                             \
        if (g_nb_trace) {                                            \
            long long t_;                                            \
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t_));    \
            g_nb_trace[(size_t)blockIdx.x * 16 + (slot)] = t_;        \
        }                                                            \
    } while (0)
#define NB_CLK(var) const long long var = clock64()
#define NB_ACC(slot, val) (nb_acc[(slot) - 8] += (val))
#define NB_ACC_DECL long long nb_acc[5] = {0, 0, 0, 0, 0}
#define NB_ACC_FLUSH(slot)                                                                          \
    do {                                                                                            \
        if (g_nb_trace && lane == 0) g_nb_trace[(size_t)blockIdx.x * 16 + (slot)] = nb_acc[(slot) - 8]; \
    } while (0)
#else
#define NB_STAMP(slot) \
    do {               \
    } while (0)
#define NB_CLK(var) \
    do {            \
    } while (0)
#define NB_ACC(slot, val) \
    do {                  \
    } while (0)
#define NB_ACC_DECL \
    do {            \
    } while (0)
#define NB_ACC_FLUSH(slot) \
    do {                   \
    } while (0)
#endif

// Sixteen consecutive activations x[k .. k+16) of one row as they lie in memory (W = 2 vectors of eight 16-bit values, or
// W = 4 vectors of four floats), zero beyond K; through L2 only (the row may have been written by the preceding kernel
// while this one was already resident).
template <int W>
__device__ __forceinline__ void nb_load_raw(const void* X, size_t row_off, int k, int K, bool vec_ok, uint4 (&v)[W]) {
    if (vec_ok && k + 16 <= K) {
        const uint4* s = W == 4 ? (const uint4*)((const float*)X + row_off + k) : (const uint4*)((const unsigned short*)X + row_off + k);
#pragma unroll
        for (int i = 0; i < W; ++i) v[i] = __ldcg(s + i);
    } else {
        uint32_t w[4 * W];
#pragma unroll
        for (int i = 0; i < 4 * W; ++i) {
            if (W == 4) {
                w[i] = k + i < K ? __ldcg((const unsigned int*)X + row_off + k + i) : 0u;
            } else {
                const uint32_t lo = k + 2 * i < K ? (uint32_t)__ldcg((const unsigned short*)X + row_off + k + 2 * i) : 0u;
                const uint32_t hi = k + 2 * i + 1 < K ? (uint32_t)__ldcg((const unsigned short*)X + row_off + k + 2 * i + 1) : 0u;
                w[i] = lo | (hi << 16);
            }
        }
#pragma unroll
        for (int i = 0; i < W; ++i) v[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
}

// B for the K range [k_begin, k_begin + nchunk * 16) of up to MR activation rows, built by 128 threads (ct = 0..127, in
// four warps q = 0..3): all rows are loaded first, their largest magnitudes are found with one exchange through shared
// memory, then every thread turns its chunks into pieces.  row_pow[m] receives the power of two that undoes row m's
// scaling; red is scratch for 16 floats.
template <bool F32>
__device__ __forceinline__ void nb_build_b(const NbParams& p, int ct, int lane, int q, int k_begin, int nchunk, uint32_t b_base, float* row_pow,
                                           float* red) {
    constexpr int W = F32 ? 4 : 2, MR = F32 ? 2 : 4, P = F32 ? 8 : 4;
    constexpr uint32_t b_tile = NB_ROWS * 128u;
    const size_t esz = F32 ? 4 : 2;
    const bool vec_ok = ((uintptr_t)p.X % 16 == 0) && (((size_t)p.x_ld * esz) % 16 == 0);
    const bool bf16 = p.x_dtype == TLLM_BF16;
    uint4 raw[MR][2][W];
    uint32_t mag[MR];        // largest magnitude as a bit pattern: for one sign the order of floats is the order of their bits
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        mag[m] = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int c = ct + i * 128;
            if (m < p.M && c < nchunk) {
                nb_load_raw<W>(p.X, (size_t)m * p.x_ld, k_begin + c * 16, p.K, vec_ok, raw[m][i]);
            } else {
#pragma unroll
                for (int v = 0; v < W; ++v) raw[m][i][v] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int v = 0; v < W; ++v) {
                const uint32_t w[4] = {raw[m][i][v].x, raw[m][i][v].y, raw[m][i][v].z, raw[m][i][v].w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    if (F32) mag[m] = max(mag[m], w[t] & 0x7FFFFFFFu);
                    else mag[m] = max(mag[m], max(w[t] & 0x7FFFu, (w[t] >> 16) & 0x7FFFu));
                }
            }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mag[m] = max(mag[m], __shfl_xor_sync(0xffffffffu, mag[m], o));
        if (lane == 0) red[q * 4 + m] = __uint_as_float(mag[m]);
    }
    if (ct == 0) NB_STAMP(13);
    named_bar(1, 128);
    if (ct == 0) NB_STAMP(14);
    float down[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        const uint32_t bits = max(max(__float_as_uint(red[m]), __float_as_uint(red[4 + m])), max(__float_as_uint(red[8 + m]), __float_as_uint(red[12 + m])));
        const float amax = F32 ? __uint_as_float(bits) : (bf16 ? __uint_as_float(bits << 16) : __half2float(__ushort_as_half((unsigned short)bits)));
        // 2^e with amax * 2^-e in [2^14, 2^15); e kept where both 2^e and 2^-e are normal floats
        int e = amax > 0.f && amax <= 3.0e38f ? ilogbf(amax) - 14 : 0;
        e = max(-126, min(112, e));
        down[m] = __uint_as_float((uint32_t)(127 - e) << 23);
        if (ct == 0 && m < p.M) row_pow[m] = __uint_as_float((uint32_t)(127 + e) << 23);
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        if (m >= p.M) break;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int c = ct + i * 128;
            if (c >= nchunk) continue;
            const int kb = c >> 3, ch = c & 7;
            float r[16];
#pragma unroll
            for (int v = 0; v < W; ++v) {
                const uint32_t w[4] = {raw[m][i][v].x, raw[m][i][v].y, raw[m][i][v].z, raw[m][i][v].w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    if (F32) {
                        r[4 * v + t] = __uint_as_float(w[t]) * down[m];
                    } else if (bf16) {
                        r[8 * v + 2 * t] = __uint_as_float(w[t] << 16) * down[m];
                        r[8 * v + 2 * t + 1] = __uint_as_float(w[t] & 0xFFFF0000u) * down[m];
                    } else {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[t]));
                        r[8 * v + 2 * t] = f.x * down[m];
                        r[8 * v + 2 * t + 1] = f.y * down[m];
                    }
                }
            }
            const uint32_t tile_addr = b_base + (uint32_t)kb * b_tile;
            int row0 = m * P;
            auto dst = [&](int pc) {
                const uint32_t row = (uint32_t)(row0 + pc);
                return tile_addr + (row >> 3) * 1024u + (row & 7u) * 128u + ((((uint32_t)ch) ^ (row & 7u)) << 4);
            };
            uint32_t hw[8];
            if (!F32) {
                // fp16 / bf16 values fit fp16 after the scaling: four pieces take all eleven bits
#pragma unroll
                for (int t = 0; t < 8; ++t) hw[t] = pack_half2_rz(r[2 * t], r[2 * t + 1]);
                nb_emit_pieces(hw, 4, dst);
            } else {
                // fp32: nine bits at a time (three pieces), twice, then the last six bits (two pieces)
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
                    nb_emit_pieces(hw, round < 2 ? 3 : 2, dst);
                    row0 += 3;
                }
            }
        }
    }
}

#define NB_WAIT(bar, par)                                      \
    do {                                                       \
        if (!bounded_spin((bar), (par), abort_flag)) goto done; \
    } while (0)
#define NB_WAIT_BLOCK(bar, par)                                \
    do {                                                       \
        if (!bounded_wait((bar), (par), abort_flag)) goto done; \
    } while (0)
#define NB_ADVANCE(idx, ph, n) \
    do {                       \
        if (++(idx) == (n)) {  \
            (idx) = 0;         \
            (ph) ^= 1u;        \
        }                      \
    } while (0)

template <int UK>
__global__ void __launch_bounds__(NB_THREADS, UK == 1 ? 2 : 1) nibble_spmm_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ NbParams p) {
    extern __shared__ unsigned char nb_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- this block's run of (tile, K block) units inside its K range ------------------------------------
    const int j = blockIdx.x / p.Gj, cc = blockIdx.x % p.Gj, G = p.Gj;
    const int kbj0 = j * p.KBS;
    const int KBj = min(p.KBS, p.KB - kbj0);
    const int KUj = (KBj + UK - 1) / UK;                    // units per column tile in this range
    const long long total = (long long)p.n_tiles * KUj;
    const int u0 = (int)(total * cc / G), u1 = (int)(total * (cc + 1) / G);
    if (u0 >= u1) return;
    if (tid == 0) NB_STAMP(0);

    // ---- shared memory ---------------------------------------------------------------------------------
    const uint32_t raw0 = smem_u32(nb_smem);
    const uint32_t base = (raw0 + 1023u) & ~1023u;                 // swizzled tiles need 1024-byte alignment
    const uint32_t S = (uint32_t)p.S;
    const uint32_t a_stage = UK * NB_A_STAGE_BYTES;
    const uint32_t a_base = base, b_base = a_base + S * a_stage;
    const uint32_t b_tile = NB_ROWS * 128u;                        // bytes of B per K block
    const uint32_t bar_base = b_base + (uint32_t)p.KBS * b_tile;
    unsigned char* tail = nb_smem + (bar_base - raw0);
    volatile int* flags = (volatile int*)(tail + 8 * 24);          // [0] tensor-memory address, [1] abort
    volatile int* abort_flag = flags + 1;
    float* row_pow = (float*)(tail + 8 * 24 + 16);                 // [NB_ROWS] power of two that undoes a row's scaling
    float* red = row_pow + NB_ROWS;                                // [16] per-warp maxima of up to four rows
#define A_FULL(s) (bar_base + 8u * (uint32_t)(s))
#define A_EMPTY(s) (bar_base + 8u * (8u + (uint32_t)(s)))
#define ACC_FULL(a) (bar_base + 8u * (16u + (uint32_t)(a)))
#define ACC_EMPTY(a) (bar_base + 8u * (18u + (uint32_t)(a)))
#define B_READY (bar_base + 8u * 20u)

    if (tid == 0) {
        for (int s = 0; s < NB_MAX_STAGES; ++s) {
            mbar_init(A_FULL(s), 1);       // the producer's expect_tx arrival
            mbar_init(A_EMPTY(s), 1);      // tcgen05.commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(ACC_FULL(a), 1);
            mbar_init(ACC_EMPTY(a), 4);    // the four epilogue warps
        }
        mbar_init(B_READY, 4);             // the four warps that build B
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
    if (tid == 0) NB_STAMP(1);

    // The two single-issuer roles run their loops with the whole warp converged and elect one lane only for the
    // instruction itself: addresses and descriptors then are warp-uniform values.
    if (warp == 0) {
        // ---- weight producer: nothing here depends on the preceding kernel, so the stream starts at once
        uint32_t s = 0, sph = 0;
        int tile = u0 / KUj, ku = u0 - tile * KUj;
        NB_ACC_DECL;
        for (int u = u0; u < u1; ++u) {
            NB_CLK(c0);
            NB_WAIT_BLOCK(A_EMPTY(s), sph ^ 1u);      // parked, not spinning: this wait is long while B is not ready
            NB_CLK(c1);
            NB_ACC(8, c1 - c0);
            if (elect_one()) {
                const int nk = min(UK, KBj - ku * UK);
#ifdef NB_DEBUG
                if (p.debug & 2) mbar_arrive(A_FULL(s));
                else
#endif
                {
                    mbar_expect_tx(A_FULL(s), (uint32_t)nk * p.tx_bytes);
#pragma unroll
                    for (int t = 0; t < UK; ++t)
                        if (t < nk)
                            tma_load_2d(a_base + s * a_stage + (uint32_t)t * NB_A_STAGE_BYTES, &wmap, (kbj0 + ku * UK + t) * NB_TILE_K, tile * NB_TILE_N,
                                        A_FULL(s));
                }
            }
            __syncwarp();
            NB_ADVANCE(s, sph, S);
            if (++ku == KUj) ku = 0, ++tile;
            NB_CLK(c2);
            NB_ACC(9, c2 - c1);
        }
        if (lane == 0) NB_STAMP(7);
        NB_ACC_FLUSH(8);
        NB_ACC_FLUSH(9);
    } else if (warp == 1) {
        // ---- MMA issuer
        const uint32_t idesc = p.idesc;
        const uint32_t a_lo0 = (a_base >> 4) & 0x3FFFu, b_lo0 = (b_base >> 4) & 0x3FFFu;
        uint32_t s = 0, sph = 0, a = 0, aph = 0;
        NB_ACC_DECL;
        NB_WAIT_BLOCK(B_READY, 0u);                   // parked: B waits for the preceding kernel, whose blocks may share this SM
        tc_fence_after();
        int ku0 = u0 % KUj;
        for (int u = u0; u < u1;) {
            const int ku1 = min(KUj, ku0 + (u1 - u));
            NB_CLK(c3);
            NB_WAIT(ACC_EMPTY(a), aph ^ 1u);
            tc_fence_after();
            NB_CLK(c4);
            NB_ACC(12, c4 - c3);
            const uint32_t d = tmem + a * NB_ROWS;
            uint32_t acc = 0;
            for (int ku = ku0; ku < ku1; ++ku) {
                NB_CLK(c0);
                NB_WAIT(A_FULL(s), sph);
                NB_CLK(c1);
                NB_ACC(10, c1 - c0);
#ifdef NB_DEBUG
                if (lane == 0 && u == u0 && ku == ku0) NB_STAMP(4);
#endif
                const int nk = min(UK, KBj - ku * UK);
                const uint32_t a_lo = a_lo0 + s * (a_stage >> 4), b_lo = b_lo0 + (uint32_t)(ku * UK) * (b_tile >> 4);
                if (elect_one()) {
#ifdef NB_DEBUG
                    if (!(p.debug & 1))
#endif
                    {
#pragma unroll
                        for (uint32_t t = 0; t < UK; ++t)
                            if ((int)t < nk) {
#pragma unroll
                                for (uint32_t k4 = 0; k4 < NB_TILE_K / 32; ++k4)       // 32 values = 32 bytes = 2 descriptor address units
                                    umma_f8f6f4_lo(d, a_lo + t * (NB_A_STAGE_BYTES >> 4) + 2u * k4, b_lo + t * (b_tile >> 4) + 2u * k4, idesc,
                                                   (t | k4) == 0 ? acc : 1u);
                            }
                    }
                    umma_commit(A_EMPTY(s));
                }
                __syncwarp();
                acc = 1;
                NB_ADVANCE(s, sph, S);
                NB_CLK(c2);
                NB_ACC(11, c2 - c1);
            }
            if (elect_one()) umma_commit(ACC_FULL(a));
            __syncwarp();
            a ^= 1u;
            aph ^= (a == 0);
            u += ku1 - ku0;
            ku0 = 0;
        }
        if (lane == 0) NB_STAMP(5);
        NB_ACC_FLUSH(10);
        NB_ACC_FLUSH(11);
        NB_ACC_FLUSH(12);
    } else {
        const int ct = tid - 64, q = warp & 3, nl = q * 32 + lane;
        const int P = p.P;
        // rows of B past M * P hold zeros: written while the preceding kernel may still be running
        for (int i = ct; i < KBj * (NB_ROWS * 8); i += 128) {
            const int kb = i / (NB_ROWS * 8), rem = i - kb * (NB_ROWS * 8), row = rem >> 3;
            if (row >= p.M * P) st_shared_v4(b_base + (uint32_t)kb * b_tile + (uint32_t)rem * 16u, 0u, 0u, 0u, 0u);
        }
        pdl_wait();
        if (ct == 0) NB_STAMP(2);
        // ---- B: the activation rows of this block's K range as e5m2 pieces -----------------------------------
        {
            const int k_begin = kbj0 * NB_TILE_K;
            if (ct == 0) NB_STAMP(15);
            if (p.x_dtype == TLLM_F32) nb_build_b<true>(p, ct, lane, q, k_begin, KBj * 8, b_base, row_pow, red);
            else nb_build_b<false>(p, ct, lane, q, k_begin, KBj * 8, b_base, row_pow, red);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make B visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(B_READY);
            named_bar(1, 128);                                             // row_pow is complete
            if (ct == 0) NB_STAMP(3);
        }
        // ---- epilogue: a warp may read the 32 tensor-memory lanes selected by warp % 4 ----------------------
        uint32_t a = 0, aph = 0;
        const long long slots_per_split = (long long)p.n_tiles + G;
        int tile = u0 / KUj, ku0 = u0 - tile * KUj;
        for (int u = u0; u < u1;) {
            const int ku1 = min(KUj, ku0 + (u1 - u));
            const bool full = p.k_splits == 1 && ku0 == 0 && ku1 == KUj;
            // read before the wait, so that the latency hides behind the MMAs: how many blocks hold a part of this tile,
            // and (lane jj) the run of blocks of K range jj that do
            const uint32_t parts = full ? 1u : __ldg(p.sched + tile);
            const uint32_t my_run = (!full && lane < p.k_splits) ? __ldg(p.sched + (size_t)(1 + lane) * p.n_tiles + tile) : 1u;   // 1: an empty run
            NB_WAIT_BLOCK(ACC_FULL(a), aph);
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + a * NB_ROWS;
            const int n = tile * NB_TILE_N + nl;
            auto emit = [&](float v, int m) {      // called by all lanes of the warp with the same m
                if (p.epilogue == 0) {
                    if (n < p.N) store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + n, v * p.scale);
                } else {
                    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                    if (!(nl & 1) && n + 1 < p.N) store_out(p.Y, p.y_dtype, (size_t)m * p.y_ld + (n >> 1), silu_mul(v * p.scale, other * p.scale2));
                }
            };
            float* slot = p.partial + ((size_t)(j * slots_per_split + tile + cc) * (size_t)p.M) * NB_TILE_N;
            for (int m = 0; m < p.M; ++m) {
                float v[8];
                if (P == 4) tmem_ld4(taddr + (uint32_t)(m * 4), v);
                else tmem_ld8(taddr + (uint32_t)(m * 8), v);
                // smallest pieces first
                const float sum = ((((((v[7] + v[6]) + v[5]) + v[4]) + v[3]) + v[2]) + v[1]) + v[0];
                const float y = sum * row_pow[m];
                if (full) emit(y, m);
                else slot[(size_t)m * NB_TILE_N + nl] = y;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ACC_EMPTY(a));
            if (!full) {
                // The last of the blocks that hold a part of this column tile adds the parts: ranges in order, blocks
                // of a range in order.  Each epilogue warp owns 32 columns of the tile and runs the hand-over by itself.
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    unsigned int* ctr = p.counters + (size_t)tile * 4 + q;
                    last = atomicAdd(ctr, 1u) == parts - 1u;
                    if (last) *ctr = 0;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence();
                    // The parts of a tile: for every K range a run of slots (first and last block of the range that
                    // hold some of the tile).  Lane jj keeps the run of range jj; the loads go out sixteen at a time --
                    // one after the other they cost an L2 round trip each, and the block that adds a tile's parts is the
                    // last one of the launch to finish.  The order of the additions stays: ranges, then blocks.
                    constexpr int MAX_M = NB_ROWS / 4;     // rows of one launch: four pieces or more each
                    float acc[MAX_M];
#pragma unroll
                    for (int m = 0; m < MAX_M; ++m) acc[m] = 0.f;
                    int jj = 0, got;
                    uint32_t run = __shfl_sync(0xffffffffu, my_run, 0);
                    uint32_t c2 = run & 0xFFFFu, hi = run >> 16;
                    // (both unrolled loops leave at the first slot that is not used: the instructions of the unused
                    // ones cost this warp, which the whole launch waits for, about a microsecond)
                    do {
                        float v[16][MAX_M];
                        got = 0;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            while (c2 > hi && ++jj < p.k_splits) {       // on to the next range that has blocks on this tile
                                run = jj < 32 ? __shfl_sync(0xffffffffu, my_run, jj) : __ldg(p.sched + (size_t)(1 + jj) * p.n_tiles + tile);
                                c2 = run & 0xFFFFu, hi = run >> 16;
                            }
                            if (c2 > hi) break;                          // no range left
                            const float* part = p.partial + ((size_t)(jj * slots_per_split + tile + c2) * (size_t)p.M) * NB_TILE_N + nl;
                            v[i][0] = __ldcg(part);
#pragma unroll
                            for (int m = 1; m < MAX_M; ++m)
                                if (m < p.M) v[i][m] = __ldcg(part + (size_t)m * NB_TILE_N);
                            ++c2;
                            got = i + 1;
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            if (i >= got) break;
                            acc[0] += v[i][0];
#pragma unroll
                            for (int m = 1; m < MAX_M; ++m)
                                if (m < p.M) acc[m] += v[i][m];
                        }
                    } while (got == 16);
#pragma unroll
                    for (int m = 0; m < MAX_M; ++m)
                        if (m < p.M) emit(acc[m], m);
                }
            }
            a ^= 1u;
            aph ^= (a == 0);
            u += ku1 - ku0;
            ku0 = 0;
            ++tile;
        }
        if (ct == 0) NB_STAMP(6);
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
#undef B_READY
}
#undef NB_WAIT
#undef NB_WAIT_BLOCK
#undef NB_ADVANCE

}  // namespace tllm
