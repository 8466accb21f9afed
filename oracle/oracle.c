/*
 * oracle.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C, single-threaded CPU restatement of the algorithms of fpgasystems/ternaryLLM on the
 * ternary sparse product path  Y = X . W . s  (W in {-1,0,+1}).  It exists so that the CUDA path can
 * be checked against something that follows the reference step by step; it is never linked into,
 * imported by, or called from the shipped library.  Only tests, the smoke check and the CPU-baseline
 * leg of the benchmark may use it.
 *
 * Pinning: every function below is checked (tests/test_oracle_golden.py) against fixtures produced by
 * the reference itself -- its pure-Python packers (ternaryLLM_GPU/TernaryLLM/TernaryCSC.py) and its CPU
 * kernels/format builders (ternaryLLM_CPU/src/TCSC.hpp, GEMM_CPU_FP32.cpp, GEMM_CPU_INT8.cpp) compiled
 * in place.  Capabilities the reference does not have (per-tensor scale, fp16/bf16 inputs, int32
 * accumulation) are pinned only by the fp64/int64 dense product, which is the mathematical definition.
 *
 * Conventions: W is row-major [K][N]; "reference file:line" citations are relative to the reference
 * repository root.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------------ */
/* Ground truth: dense product.                                                                      */
/* Follows GEMM_CPU_FP32_rowMajor_Direct_OpenMP (ternaryLLM_CPU/src/GEMM_CPU_FP32.cpp:16839-16851)   */
/* and GEMM<T> (ternaryLLM_CPU/src/GEMM_CPU_FP32.hpp:27-38), in fp64 with a trailing scale.          */
/* X [M][K] row-major, W [K][N] row-major, Y [M][N] row-major.                                       */
/* ------------------------------------------------------------------------------------------------ */
void orc_dense_f64(const double* X, const int8_t* W, double scale, double* Y, int M, int N, int K) {
    for (int m = 0; m < M; m++) {
        double* y = Y + (size_t)m * N;
        for (int n = 0; n < N; n++) y[n] = 0.0;
        for (int k = 0; k < K; k++) {
            const double x = X[(size_t)m * K + k];
            const int8_t* w = W + (size_t)k * N;
            for (int n = 0; n < N; n++) {
                if (w[n] > 0) y[n] += x;
                else if (w[n] < 0) y[n] -= x;
            }
        }
        for (int n = 0; n < N; n++) y[n] *= scale;
    }
}

/* Integer ground truth (GEMM_CPU_colMajor_Direct_OpenMP<T>, GEMM_CPU_FP32.hpp:14-25, widened to
 * int64 so that both the int32-accumulate path and the reference's int8 wrap-around result can be
 * derived from it by truncation).  X [M][K] row-major int8. */
void orc_dense_i64(const int8_t* X, const int8_t* W, int64_t* Y, int M, int N, int K) {
    for (int m = 0; m < M; m++) {
        int64_t* y = Y + (size_t)m * N;
        for (int n = 0; n < N; n++) y[n] = 0;
        for (int k = 0; k < K; k++) {
            const int64_t x = X[(size_t)m * K + k];
            const int8_t* w = W + (size_t)k * N;
            for (int n = 0; n < N; n++) {
                if (w[n] > 0) y[n] += x;
                else if (w[n] < 0) y[n] -= x;
            }
        }
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* GPU-side formats (ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu, twins in TernaryLLM/TernaryCSC.py).     */
/* w is int32 [K][N] row-major with entries in {-1,0,1}.                                             */
/* ------------------------------------------------------------------------------------------------ */

/* cnt_pos / cnt_neg as TernaryLinear.py:104-105 computes them. */
void orc_count_nnz(const int32_t* w, int N, int K, int64_t* pos, int64_t* neg) {
    int64_t p = 0, q = 0;
    for (size_t i = 0; i < (size_t)N * K; i++) { p += (w[i] == 1); q += (w[i] == -1); }
    *pos = p; *neg = q;
}

/* convert_to_ter_csc (ter_spmm_wrapper.cu:39-78; TernaryCSC.py:17-48): split CSC with global row
 * ids; offsets have N+1 entries.  Output order of the reference: neg_idx, neg_off, pos_idx, pos_off. */
void orc_ter_csc(const int32_t* w, int N, int K, int32_t* neg_idx, int32_t* neg_off,
                 int32_t* pos_idx, int32_t* pos_off) {
    int nb_neg = 0, nb_pos = 0;
    for (int y = 0; y < N; y++) {
        neg_off[y] = nb_neg;
        pos_off[y] = nb_pos;
        for (int x = 0; x < K; x++) {
            const int32_t v = w[(size_t)x * N + y];
            if (v == -1) neg_idx[nb_neg++] = x;
            else if (v == 1) pos_idx[nb_pos++] = x;
        }
    }
    neg_off[N] = nb_neg;
    pos_off[N] = nb_pos;
}

/* convert_to_ter_tiled_csc (ter_spmm_wrapper.cu:92-152; TernaryCSC.py:50-94): same lists with
 * tile-local row ids and a [start,end) pair per (column, tile).  The reference walks TILE_K rows in
 * every tile even when K is not a multiple of TILE_K (an out-of-bounds read); here rows >= K count
 * as zero. */
void orc_ter_tiled_csc(const int32_t* w, int N, int K, int T, int32_t* neg_idx, int32_t* neg_off_t,
                       int32_t* pos_idx, int32_t* pos_off_t) {
    const int tiles = (K + T - 1) / T;
    int32_t* tmp_no = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N + 1));
    int32_t* tmp_po = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N + 1));
    orc_ter_csc(w, N, K, neg_idx, tmp_no, pos_idx, tmp_po);
    free(tmp_no); free(tmp_po);
    int nb_neg = 0, nb_pos = 0;
    for (int y = 0; y < N; y++) {
        for (int t = 0; t < tiles; t++) {
            const int offset = t * T;
            neg_off_t[((size_t)y * tiles + t) * 2 + 0] = nb_neg;
            pos_off_t[((size_t)y * tiles + t) * 2 + 0] = nb_pos;
            for (int x = 0; x < T; x++) {
                const int row = t * T + x;
                if (row >= K) break;
                const int32_t v = w[(size_t)row * N + y];
                if (v == -1) { neg_idx[nb_neg] -= offset; nb_neg++; }
                else if (v == 1) { pos_idx[nb_pos] -= offset; nb_pos++; }
            }
            neg_off_t[((size_t)y * tiles + t) * 2 + 1] = nb_neg;
            pos_off_t[((size_t)y * tiles + t) * 2 + 1] = nb_pos;
        }
    }
}

/* inter_tile_swizzle (ter_spmm_wrapper.cu:9-27): per column, tile ids sorted by list length.  The
 * reference uses std::sort (unstable) with a strict < comparator; ties therefore have no defined
 * order.  This restatement is a stable sort, and tests compare sorted-by-length property only. */
void orc_inter_tile_swizzle(int N, int tiles, const int32_t* off, int32_t* tile_idx) {
    for (int i = 0; i < N; i++) {
        int32_t* out = tile_idx + (size_t)i * tiles;
        for (int t = 0; t < tiles; t++) out[t] = t;
        for (int a = 1; a < tiles; a++) {          /* insertion sort, stable */
            const int32_t v = out[a];
            const int32_t* ov = off + ((size_t)i * tiles + v) * 4;
            const int lv = ov[2] - ov[0];
            int b = a - 1;
            while (b >= 0) {
                const int32_t* ob = off + ((size_t)i * tiles + out[b]) * 4;
                if (ob[2] - ob[0] > lv) { out[b + 1] = out[b]; b--; } else break;
            }
            out[b + 1] = v;
        }
    }
}

static int ceil_mult(int v, int m) { return (v + m - 1) / m * m; }

/* convert_to_ter_tiled_mcsc -- the merged tiled CSC that is the reference's GPU weight format.
 *   lossy == 0 : the lossless Python twin (TernaryCSC.py:97-156): per (column, tile) min(pos,neg)
 *                interleaved (p,q) pairs, then the left-over same-sign indices; offsets
 *                {pair_start, pair_end, rem_end, sign}, sign = +1 when neg <= pos else -1.
 *   lossy == 1 : the C++ packer actually used by the extension (ter_spmm_wrapper.cu:156-315),
 *                including its truncation of list lengths to multiples of 4 (:277-291), its padding
 *                rule (:198-230, :258-261) and the fact that the remainder is written directly
 *                behind the *unpadded* pair region (:266-275) while the offsets skip the padding.
 * idx must hold idx_cap entries and is zero-filled first (the reference value-initialises its
 * vector).  Returns the number of meaningful entries: the reference's vector length (cnt_pos+cnt_neg
 * without padding, the padded total with padding), or -1 if idx_cap is too small.
 * tile_idx (may be NULL) receives inter_tile_swizzle of the offsets. */
int64_t orc_ter_tiled_mcsc(const int32_t* w, int N, int K, int T, int padding, int padding_size,
                           int lossy, int32_t* idx, int64_t idx_cap, int32_t* off,
                           int32_t* tile_idx) {
    const int tiles = (K + T - 1) / T;
    int64_t cp, cn;
    orc_count_nnz(w, N, K, &cp, &cn);
    int32_t* neg_idx = (int32_t*)calloc((size_t)cn + 1, sizeof(int32_t));
    int32_t* pos_idx = (int32_t*)calloc((size_t)cp + 1, sizeof(int32_t));
    int32_t* neg_off = (int32_t*)malloc(sizeof(int32_t) * (size_t)N * tiles * 2);
    int32_t* pos_off = (int32_t*)malloc(sizeof(int32_t) * (size_t)N * tiles * 2);
    orc_ter_tiled_csc(w, N, K, T, neg_idx, neg_off, pos_idx, pos_off);

    int64_t total = cp + cn;
    if (lossy && padding) {                        /* ter_spmm_wrapper.cu:198-230 */
        total = 0;
        for (size_t i = 0; i < (size_t)N * tiles; i++) {
            const int neg = neg_off[i * 2 + 1] - neg_off[i * 2];
            const int pos = pos_off[i * 2 + 1] - pos_off[i * 2];
            const int mn = neg <= pos ? neg : pos, mx = neg <= pos ? pos : neg;
            total += ceil_mult(mn * 2, padding_size) + ceil_mult(mx - mn, padding_size);
        }
    }
    if (total > idx_cap) { free(neg_idx); free(pos_idx); free(neg_off); free(pos_off); return -1; }
    memset(idx, 0, sizeof(int32_t) * (size_t)idx_cap);

    int64_t prev_cnt = 0, prev_nnz = 0;
    for (int y = 0; y < N; y++) {
        for (int t = 0; t < tiles; t++) {
            const size_t ti = (size_t)y * tiles + t;
            const int ns = neg_off[ti * 2], ne = neg_off[ti * 2 + 1];
            const int ps = pos_off[ti * 2], pe = pos_off[ti * 2 + 1];
            const int neg = ne - ns, pos = pe - ps;
            const int flag_min_neg = neg <= pos;
            const int mn = flag_min_neg ? neg : pos, mx = flag_min_neg ? pos : neg;
            int cnt_inter = mn * 2;
            const int cnt_inter_pad = (lossy && padding) ? ceil_mult(cnt_inter, padding_size) : cnt_inter;
            for (int k = 0; k < mn; k++) {
                idx[prev_nnz + 2 * k + 0] = pos_idx[ps + k];
                idx[prev_nnz + 2 * k + 1] = neg_idx[ns + k];
            }
            for (int k = cnt_inter; k < cnt_inter_pad; k++)   /* (p,p) padding, :258-261 */
                idx[prev_nnz + k] = (ps < cp) ? pos_idx[ps] : 0;
            int cnt_rem = mx - mn;
            const int cnt_rem_pad = (lossy && padding) ? ceil_mult(cnt_rem, padding_size) : cnt_rem;
            for (int k = mn; k < mx; k++) {
                const int64_t dst = prev_nnz + k + mn;
                if (dst < idx_cap) idx[dst] = flag_min_neg ? pos_idx[ps + k] : neg_idx[ns + k];
            }
            if (lossy) {                           /* :277-291 */
                if (cnt_rem % 2 == 1) cnt_rem--;
                if (cnt_inter % 4 != 0) cnt_inter -= 2;
                if (cnt_rem % 4 != 0) cnt_rem -= 2;
            }
            int32_t* o = off + ti * 4;
            if (lossy && padding) {
                o[0] = (int32_t)prev_cnt;
                o[1] = (int32_t)(prev_cnt + cnt_inter_pad);
                o[2] = (int32_t)(prev_cnt + cnt_inter_pad + cnt_rem);
                prev_cnt += cnt_inter_pad + cnt_rem_pad;
            } else {
                o[0] = (int32_t)prev_cnt;
                o[1] = (int32_t)(prev_cnt + cnt_inter);
                o[2] = (int32_t)(prev_cnt + cnt_inter + cnt_rem);
                prev_cnt += cnt_inter + cnt_rem;
            }
            o[3] = flag_min_neg ? 1 : -1;
            /* the C++ packer restarts writing at the (possibly truncated) running count (:299-300);
             * the Python twin advances by the true number of entries (TernaryCSC.py:154). */
            prev_nnz = lossy ? prev_cnt : prev_nnz + neg + pos;
        }
    }
    if (tile_idx) orc_inter_tile_swizzle(N, tiles, off, tile_idx);
    free(neg_idx); free(pos_idx); free(neg_off); free(pos_off);
    return total;
}

/* What a kernel must compute from the merged tiled arrays: the intent of ter_tiled_mcsc_spmv
 * (ter_spmm_kernel.cuh:45-68) and ter_tiled_mcsc_spmm (:186-299), evaluated in fp64 over every list
 * entry, with the tile base applied to the remainder as well (the reference SpMV omits it at :63,
 * which is a defect, not a format rule).
 *   Y[m][n] = scale * sum_t ( sum_pairs x[tT+p]-x[tT+q]  +  sign_t * sum_rem x[tT+r] )
 * X is [M][K] row-major (x_colmajor == 0) or [K][M] (x_colmajor != 0, the layout the reference SpMM
 * reads, :173). Y is [M][N] row-major. */
void orc_mcsc_product_f64(const double* X, int x_colmajor, const int32_t* idx, const int32_t* off,
                          int M, int N, int K, int T, double scale, double* Y) {
    const int tiles = (K + T - 1) / T;
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            double acc = 0.0;
            for (int t = 0; t < tiles; t++) {
                const int32_t* o = off + ((size_t)n * tiles + t) * 4;
                const int base = t * T;
#define XV(r) (x_colmajor ? X[(size_t)(base + (r)) * M + m] : X[(size_t)m * K + base + (r)])
                for (int i = o[0]; i + 1 < o[1]; i += 2) acc += XV(idx[i]) - XV(idx[i + 1]);
                double part = 0.0;
                for (int i = o[1]; i < o[2]; i++) part += XV(idx[i]);
                acc += (double)o[3] * part;
#undef XV
            }
            Y[(size_t)m * N + n] = acc * scale;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* CPU-side formats (ternaryLLM_CPU/src/TCSC.hpp).  W is int8 [K][N] row-major.                       */
/* ------------------------------------------------------------------------------------------------ */

/* SparseFormat (TCSC.hpp:13-33): ">= 1" is positive, "<= -1" negative; int16 global row ids. */
void orc_sparse_format(const int8_t* W, int K, int N, int32_t* col_start_pos, int32_t* col_start_neg,
                       int16_t* row_index_pos, int16_t* row_index_neg) {
    int sp = 0, sn = 0;
    for (int n = 0; n < N; n++) {
        col_start_pos[n] = sp;
        col_start_neg[n] = sn;
        for (int k = 0; k < K; k++) {
            const int8_t v = W[(size_t)k * N + n];
            if (v >= 1) row_index_pos[sp++] = (int16_t)k;
            else if (v <= -1) row_index_neg[sn++] = (int16_t)k;
        }
    }
    col_start_pos[N] = sp;
    col_start_neg[N] = sn;
}

/* MergedTCSC (TCSC.hpp:41-89): per column interleaved (p,q) pairs then the left-over entries;
 * metadata {align_start, align_end, remain_end, remain_val} with remain_val in {+1,0,-1}. */
void orc_merged_tcsc(const int32_t* csp, const int32_t* csn, const int16_t* rip, const int16_t* rin,
                     int N, int32_t* metadata, int16_t* row_index) {
    int remain_end = 0, ip = 0, in = 0, w = 0;
    for (int n = 0; n < N; n++) {
        const int cp = csp[n + 1] - csp[n], cn = csn[n + 1] - csn[n];
        int align_end, remain_val;
        if (cp >= cn) {
            align_end = cn * 2;
            remain_val = (cp == cn) ? 0 : 1;
            for (int k = 0; k < cn; k++) { row_index[w++] = rip[ip++]; row_index[w++] = rin[in++]; }
            for (int k = 0; k < cp - cn; k++) row_index[w++] = rip[ip++];
        } else {
            align_end = cp * 2;
            remain_val = -1;
            for (int k = 0; k < cp; k++) { row_index[w++] = rip[ip++]; row_index[w++] = rin[in++]; }
            for (int k = 0; k < cn - cp; k++) row_index[w++] = rin[in++];
        }
        metadata[n * 4 + 0] = remain_end;
        metadata[n * 4 + 1] = remain_end + align_end;
        remain_end += cp + cn;
        metadata[n * 4 + 2] = remain_end;
        metadata[n * 4 + 3] = remain_val;
    }
}

static int imin(int a, int b) { return a < b ? a : b; }
static int imax(int a, int b) { return a > b ? a : b; }

/* MergedTCSC_Group (TCSC.hpp:99-283 six-argument constructor when simd <= 0, :285-408 seven-argument
 * constructor when simd >= 1).  method: 0 "min", 1 "mid", 2 "max", 3 anything else ("uniform").
 * Returns the number of row_index entries written (or -1 on overflow of either capacity) and stores
 * the metadata length in *meta_len. */
int64_t orc_merged_group(const int32_t* csp, const int32_t* csn, const int16_t* rip,
                         const int16_t* rin, int N, int G, int method, int interleaved, int simd,
                         int32_t* metadata, int64_t meta_cap, int16_t* row_index, int64_t ri_cap,
                         int64_t* meta_len) {
    int64_t w = 0, ml = 0;
    int align_pointer = 0;
    int* col_pos = (int*)malloc(sizeof(int) * (size_t)G);
    int* col_neg = (int*)malloc(sizeof(int) * (size_t)G);
#define PUSH_RI(v) do { if (w >= ri_cap) goto overflow; row_index[w++] = (int16_t)(v); } while (0)
#define PUSH_MD(v) do { if (ml >= meta_cap) goto overflow; metadata[ml++] = (int32_t)(v); } while (0)
    for (int n = 0; n < N; n += G) {
        int align_min = 65536, align_mid = 0, longest_align = 0, mid_longest_align = 0;
        for (int i = 0; i < G; i++) {
            col_pos[i] = csp[n + i + 1] - csp[n + i];
            col_neg[i] = csn[n + i + 1] - csn[n + i];
            const int mn = imin(col_pos[i], col_neg[i]);
            align_min = imin(mn, align_min);
            align_mid = imax(mn, align_mid);
            if (mn > longest_align) { longest_align = mn; mid_longest_align = i; }
        }
        /* common prefix */
        if (interleaved) {
            const int step = simd >= 1 ? simd : 1;   /* the 7-argument form strides columns by SIMD_SIZE (:310-315) */
            for (int k = 0; k < align_min; k++)
                for (int i = 0; i < G; i += step) {
                    PUSH_RI(rip[csp[n + i] + k]);
                    PUSH_RI(rin[csn[n + i] + k]);
                }
        } else if (simd > 1) {                       /* :318-330 */
            for (int k = 0; k < align_min; k++)
                for (int i = 0; i < G; i += simd) {
                    for (int s = 0; s < simd; s++) PUSH_RI(rip[csp[n + i + s] + k]);
                    for (int s = 0; s < simd; s++) PUSH_RI(rin[csn[n + i + s] + k]);
                }
        } else {                                     /* :137-144, :331-338 */
            for (int k = 0; k < align_min; k++) {
                for (int i = 0; i < G; i++) PUSH_RI(rip[csp[n + i] + k]);
                for (int i = 0; i < G; i++) PUSH_RI(rin[csn[n + i] + k]);
            }
        }
        if (method == 0) {                           /* "min", :146-174 */
            PUSH_MD(align_pointer);
            align_pointer += align_min * G * 2;
            PUSH_MD(align_pointer);
            for (int i = 0; i < G; i++) {
                for (int k = csp[n + i] + align_min; k < csp[n + i + 1]; k++) PUSH_RI(rip[k]);
                align_pointer += csp[n + i + 1] - (csp[n + i] + align_min);
                PUSH_MD(align_pointer);
                for (int k = csn[n + i] + align_min; k < csn[n + i + 1]; k++) PUSH_RI(rin[k]);
                align_pointer += csn[n + i + 1] - (csn[n + i] + align_min);
                PUSH_MD(align_pointer);
            }
        } else if (method == 1 || method == 2) {     /* "mid" :175-219, "max" :220-238 */
            for (int k = align_min; k < align_mid; k++)
                for (int i = 0; i < G; i++) {
                    if (k < imin(col_pos[i], col_neg[i])) {
                        PUSH_RI(rip[csp[n + i] + k]);
                        PUSH_RI(rin[csn[n + i] + k]);
                    } else {
                        const int same = rip[csp[n + mid_longest_align] + k];
                        PUSH_RI(same);
                        PUSH_RI(same);
                    }
                }
            PUSH_MD(align_pointer);
            align_pointer += align_mid * G * 2;
            PUSH_MD(align_pointer);
            if (method == 1)
                for (int i = 0; i < G; i++) {
                    if (col_pos[i] > col_neg[i]) {
                        for (int k = csp[n + i] + col_neg[i]; k < csp[n + i + 1]; k++) PUSH_RI(rip[k]);
                        align_pointer += csp[n + i + 1] - (csp[n + i] + col_neg[i]);
                        PUSH_MD(align_pointer);
                        PUSH_MD(+1);
                    } else {
                        for (int k = csn[n + i] + col_pos[i]; k < csn[n + i + 1]; k++) PUSH_RI(rin[k]);
                        align_pointer += csn[n + i + 1] - (csn[n + i] + col_pos[i]);
                        PUSH_MD(align_pointer);
                        PUSH_MD(-1);
                    }
                }
        } else {                                     /* "uniform", :239-243 */
            if (n == 0) PUSH_MD(align_min * 2);
        }
    }
    free(col_pos); free(col_neg);
    *meta_len = ml;
    return w;
overflow:
    free(col_pos); free(col_neg);
    *meta_len = ml;
    return -1;
#undef PUSH_RI
#undef PUSH_MD
}

/* ------------------------------------------------------------------------------------------------ */
/* How the reference CPU kernels read those arrays, expressed as "decode back to a dense matrix":    */
/* Wd[k][n] accumulates +1 per positive reference and -1 per negative reference (so the (a,a)        */
/* padding pairs of the "mid"/"max" groupings cancel exactly as they do in the kernels).              */
/* kind:                                                                                              */
/*   0 naive split CSC      (GEMM_CPU_FP32_colMajor_TCSC_Naive, GEMM_CPU_FP32.cpp:22-41):             */
/*       meta = col_start_neg[N+1] followed by col_start_pos[N+1]; ri = neg ids then pos ids, with   */
/*       aux = number of neg ids.                                                                     */
/*   1 MergedTCSC           (…_Merged_8x1_AVX2_OpenMP, GEMM_CPU_FP32.cpp:509-538)                     */
/*   2 Group "min"          (…_Merged_GroupMin_8xG4_AVX2_OpenMP :956-1042; GEMV …_G16 :14929-14958)   */
/*   3 Group "mid"          (…_Merged_GroupMid_8xG4_AVX2_OpenMP)                                      */
/*   4 Group "max"          (…_Aligned_GroupMax_8xG4_AVX2_OpenMP)                                     */
/*   5 Uniform              (…_Uniform_8xG4_AVX2_OpenMP; meta[0] = non-zeros per column)              */
/* prefix layout for kinds 2..5: chunk == 0 -> column-interleaved pairs p0 q0 p1 q1 …; chunk == S>0   */
/* -> per k, for each block of S columns, S positives then S negatives (S == G is the plain           */
/* "interleaved=false" layout; S == 8 / 16 are the _CS8 / _CS16 variants).                            */
/* ri32 selects int32 row ids (the gather kernels) instead of int16.                                  */
/* Returns 0, or -1 for an unknown kind.                                                              */
/* ------------------------------------------------------------------------------------------------ */
static inline int ri_at(const void* ri, int ri32, int64_t i) {
    return ri32 ? ((const int32_t*)ri)[i] : (int)((const int16_t*)ri)[i];
}

int orc_cpu_decode_dense(int kind, int G, int chunk, const int32_t* meta, const void* ri, int ri32,
                         int64_t aux, int N, int K, int8_t* Wd) {
    memset(Wd, 0, (size_t)N * K);
#define ADDW(k, n, s) Wd[(size_t)(k) * N + (n)] = (int8_t)(Wd[(size_t)(k) * N + (n)] + (s))
    if (kind == 0) {
        const int32_t* cneg = meta;
        const int32_t* cpos = meta + (N + 1);
        for (int n = 0; n < N; n++) {
            for (int i = cneg[n]; i < cneg[n + 1]; i++) ADDW(ri_at(ri, ri32, i), n, -1);
            for (int i = cpos[n]; i < cpos[n + 1]; i++) ADDW(ri_at(ri, ri32, aux + i), n, +1);
        }
        return 0;
    }
    if (kind == 1) {
        for (int n = 0; n < N; n++) {
            const int32_t* m = meta + (size_t)n * 4;
            for (int i = m[0]; i < m[1]; i += 2) {
                ADDW(ri_at(ri, ri32, i), n, +1);
                ADDW(ri_at(ri, ri32, i + 1), n, -1);
            }
            for (int i = m[1]; i < m[2]; i++) ADDW(ri_at(ri, ri32, i), n, m[3]);
        }
        return 0;
    }
    if (kind >= 2 && kind <= 5) {
        const int groups = N / G;
        for (int g = 0; g < groups; g++) {
            const int32_t* m;
            int64_t s, e;
            if (kind == 5) { m = meta; s = (int64_t)g * G * meta[0]; e = s + (int64_t)G * meta[0]; }
            else {
                const int per = kind == 4 ? 2 : 2 + 2 * G;
                m = meta + (size_t)g * per; s = m[0]; e = m[1];
            }
            for (int64_t k = s; k < e; k += 2 * G) {
                if (chunk == 0) {
                    for (int i = 0; i < G; i++) {
                        ADDW(ri_at(ri, ri32, k + 2 * i), g * G + i, +1);
                        ADDW(ri_at(ri, ri32, k + 2 * i + 1), g * G + i, -1);
                    }
                } else {
                    for (int c = 0; c < G; c += chunk)
                        for (int i = 0; i < chunk; i++) {
                            ADDW(ri_at(ri, ri32, k + 2 * c + i), g * G + c + i, +1);
                            ADDW(ri_at(ri, ri32, k + 2 * c + chunk + i), g * G + c + i, -1);
                        }
                }
            }
            if (kind == 2) {
                int64_t prev = m[1];
                for (int i = 0; i < G; i++) {
                    for (int64_t k = prev; k < m[2 + 2 * i]; k++) ADDW(ri_at(ri, ri32, k), g * G + i, +1);
                    for (int64_t k = m[2 + 2 * i]; k < m[3 + 2 * i]; k++) ADDW(ri_at(ri, ri32, k), g * G + i, -1);
                    prev = m[3 + 2 * i];
                }
            } else if (kind == 3) {
                int64_t prev = m[1];
                for (int i = 0; i < G; i++) {
                    for (int64_t k = prev; k < m[2 + 2 * i]; k++) ADDW(ri_at(ri, ri32, k), g * G + i, m[3 + 2 * i]);
                    prev = m[2 + 2 * i];
                }
            }
        }
        return 0;
    }
    return -1;
#undef ADDW
}

/* int8 kernels (GEMM_CPU_INT8.cpp:3-84): add/sub with _mm256_add_epi8 -> modular int8 accumulation,
 * int8 result.  Because reduction mod 256 commutes with addition, this equals the exact integer
 * product truncated to int8.  X [M][K] row-major, Y [M][N] row-major. */
void orc_int8_wrap(const int8_t* X, const int8_t* W, int8_t* Y, int M, int N, int K) {
    int64_t* t = (int64_t*)malloc(sizeof(int64_t) * (size_t)M * N);
    orc_dense_i64(X, W, t, M, N, K);
    for (size_t i = 0; i < (size_t)M * N; i++) Y[i] = (int8_t)(uint8_t)(t[i] & 0xff);
    free(t);
}

/* Naive_SiLU_Dot<float> (ternaryLLM_CPU/src/initData.hpp:204-210): X[i] = X[i]*XB[i]/(1+exp(-X[i])),
 * in place, evaluated in fp32 with the C library exp (the scalar version that the reference uses as
 * the yard-stick for its vectorised approximations, main.cpp:1470-1482). */
void orc_silu_mul_f32(int len, float* X, const float* XB) {
    for (int i = 0; i < len; i++) X[i] = X[i] * XB[i] / (1.0f + expf(-X[i]));
}

/* Same in fp64 for tolerance checks of fused kernels. */
void orc_silu_mul_f64(int len, double* X, const double* XB) {
    for (int i = 0; i < len; i++) X[i] = X[i] * XB[i] / (1.0 + exp(-X[i]));
}

/* The composition of TernaryMLP<T>::forward (ternaryLLM_CPU/src/LlamaModel.hpp:343-452) and
 * LlamaTernaryMLP.forward (ternaryLLM_GPU/TernaryLLM/TernaryMLP.py:33-35):
 *   y = down( silu(gate(x)) * up(x) ),  with per-tensor scales applied to each product.
 * h_round: 0 keep h in fp64; 1 round h to fp16; 2 round h to bf16; 3 round h to fp32 -- matching the
 * dtype in which a fused kernel hands h to the down projection.  Rounding helpers are below. */
static double round_to_f32(double v) { return (double)(float)v; }
static double round_to_bf16(double v) {
    float f = (float)v; uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7f800000u) == 0x7f800000u) return (double)f;
    u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u; memcpy(&f, &u, 4); return (double)f;
}
static double round_to_f16(double v) {
    /* round-to-nearest-even to binary16 via integer arithmetic on the fp32 encoding */
    float f = (float)v; uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = x & 0x80000000u; x &= 0x7fffffffu;
    float r;
    if (x >= 0x47800000u) { r = INFINITY; }
    else if (x < 0x38800000u) {                    /* subnormal half or zero: quantum 2^-24 */
        const float a = fabsf(f) * 16777216.0f;    /* exact scaling */
        r = (float)nearbyint((double)a) / 16777216.0f;
    } else {
        uint32_t y = x + 0xfffu + ((x >> 13) & 1u); y &= 0xffffe000u; memcpy(&r, &y, 4);
    }
    uint32_t o; memcpy(&o, &r, 4); o |= sign; memcpy(&r, &o, 4);
    return (double)r;
}
double orc_round(double v, int mode) {
    return mode == 1 ? round_to_f16(v) : mode == 2 ? round_to_bf16(v) : mode == 3 ? round_to_f32(v) : v;
}

void orc_mlp_f64(const double* X, const int8_t* Wg, const int8_t* Wu, const int8_t* Wd, double sg,
                 double su, double sd, int h_round, double* Y, int M, int hidden, int inter) {
    double* g = (double*)malloc(sizeof(double) * (size_t)M * inter);
    double* u = (double*)malloc(sizeof(double) * (size_t)M * inter);
    orc_dense_f64(X, Wg, sg, g, M, inter, hidden);
    orc_dense_f64(X, Wu, su, u, M, inter, hidden);
    orc_silu_mul_f64(M * inter, g, u);
    for (size_t i = 0; i < (size_t)M * inter; i++) g[i] = orc_round(g[i], h_round);
    orc_dense_f64(g, Wd, sd, Y, M, hidden, inter);
    free(g); free(u);
}
