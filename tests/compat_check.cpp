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
}
