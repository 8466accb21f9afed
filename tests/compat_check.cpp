// Test helper: exposes a handful of the generated reference-named wrappers of include/tllm_cpu_compat.hpp to ctypes,
// one per parameter-list family.  Compiled by tests/test_cpu_compat.py; not part of the library.
#include "tllm_cpu_compat.hpp"

#define GUARD(call)                  \
    try {                            \
        call;                        \
        return 0;                    \
    } catch (const std::exception&) { \
        return -1;                   \
    }

extern "C" {
int chk_f1(const float* X, const int32_t* meta, const int16_t* ri, float* out, int M, int N, int K) {
    GUARD(GEMM_CPU_FP32_colMajor_TCSC_Merged_GroupMin_8xG16_AVX2_OpenMP(X, meta, ri, out, M, N, K))
}
int chk_f2(const float* X, int nzpc, const int16_t* ri, float* out, int M, int N, int K) {
    GUARD(GEMM_CPU_FP32_colMajor_TCSC_Uniform_16xG16_AVX512_OpenMP(X, nzpc, ri, out, M, N, K))
}
int chk_f3(float* X, int32_t* meta, int32_t* ri, float* out, int M, int N, int K) {
    GUARD(GEMM_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_4xG8_AVX2_OpenMP(X, meta, ri, out, M, N, K))
}
int chk_f4(const float* x, const int32_t* meta, const int32_t* ri, float* out, int N, int K) {
    GUARD(GEMV_CPU_FP32_rowMajor_TCSC_Merged_GroupMin_G32_AVX2_OpenMP(x, meta, ri, out, N, K))
}
int chk_f4u(const float* x, int nzpc, const int32_t* ri, float* out, int N, int K) {
    GUARD(GEMV_CPU_FP32_rowMajor_TCSC_Uniform_G16_CS8_AVX2_OpenMP(x, nzpc, ri, out, N, K))
}
int chk_f5(float* X, int16_t* ni, int32_t* np_, int16_t* pi, int32_t* pp, float* out, int rows, int cols, int inners) {
    GUARD(GEMM_CPU_FP32_colMajor_TCSC_Naive(X, ni, np_, pi, pp, out, rows, cols, inners))
}
int chk_f6(const int8_t* X, const int32_t* meta, const int16_t* ri, int8_t* out, int M, int N, int K) {
    GUARD(GEMM_CPU_INT8_colMajor_TCSC_Merged_GroupMin_64xG4_AVX2_OpenMP(X, meta, ri, out, M, N, K))
}
int chk_f6u(const int8_t* X, int nzpc, const int16_t* ri, int8_t* out, int M, int N, int K) {
    GUARD(GEMM_CPU_INT8_colMajor_TCSC_Uniform_64xG4_AVX2_OpenMP(X, nzpc, ri, out, M, N, K))
}

// the direct product with bias on an object that has SparseFormat's four members (TCSC.hpp:6-34)
struct FourArrays {
    std::vector<int> col_start_pos, col_start_neg;
    std::vector<int16_t> row_index_pos, row_index_neg;
};
int chk_sparse_gemm(float* X, const int16_t* neg_idx, const int32_t* neg_ptr, const int16_t* pos_idx, const int32_t* pos_ptr, float* bias, float* Y, int M,
                    int N, int K) {
    FourArrays W;
    W.col_start_neg.assign(neg_ptr, neg_ptr + N + 1);
    W.col_start_pos.assign(pos_ptr, pos_ptr + N + 1);
    W.row_index_neg.assign(neg_idx, neg_idx + neg_ptr[N]);
    W.row_index_pos.assign(pos_idx, pos_idx + pos_ptr[N]);
    GUARD(tllm_compat::sparseGEMM(X, W, bias, Y, M, N, K))
}
// the grouped format builder on its own (host only): counts come back through n_meta / n_ri
int chk_build_group16(const int8_t* w, int K, int N, int G, int uniform, int interleaved, int* meta, int* n_meta, int16_t* ri, int* n_ri) {
    std::vector<int> m;
    std::vector<int16_t> r;
    if (!tllm_compat::build_group_format<int16_t>(w, K, N, G, uniform != 0, interleaved != 0, &m, &r)) return -1;
    if ((int)m.size() > *n_meta || (int)r.size() > *n_ri) return -2;
    std::copy(m.begin(), m.end(), meta);
    std::copy(r.begin(), r.end(), ri);
    *n_meta = (int)m.size(), *n_ri = (int)r.size();
    return 0;
}
// TernaryMLP<int32_t>: one row, X overwritten; TernaryMLP<int16_t>: M_ROW % 32 == 0, X is [K][M]
int chk_mlp32(const int8_t* WU, const int8_t* WG, const int8_t* WD, int K, int N, int uniform, float* X, float* Ya, float* Yb, int* group) {
    try {
        tllm_compat::TernaryMLP<int32_t> mlp(WU, WG, WD, K, N, uniform != 0, true, true);
        *group = mlp.Group;
        mlp.forward(X, Ya, Yb, 1, N, K);
        mlp.forward(X, Ya, Yb, 1, N, K);      // the block applied twice: the second call reuses the packed handle
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}
int chk_mlp16(const int8_t* WU, const int8_t* WG, const int8_t* WD, int K, int N, int M, float* X, float* Ya, float* Yb, int* group) {
    try {
        tllm_compat::TernaryMLP<int16_t> mlp(WU, WG, WD, K, N, false, false, false);
        *group = mlp.Group;
        mlp.forward(X, Ya, Yb, M, N, K);
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}
int chk_mlp_random(int K, int N, float sparsity, int uniform, float* X, float* Ya, float* Yb) {
    try {
        tllm_compat::TernaryMLP<int32_t> mlp(K, N, sparsity, 0.f, uniform != 0, false, true);
        mlp.forward(X, Ya, Yb, 1, N, K);
        int bad = 0;
        try {
            mlp.forward(X, Ya, Yb, 2, N, K);   // the int32_t class takes one row only
        } catch (const std::exception&) {
            bad = 1;
        }
        return bad ? 0 : -2;
    } catch (const std::exception&) {
        return -1;
    }
}
}
