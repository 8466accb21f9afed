// ref_shim.cpp -- TEST INFRASTRUCTURE ONLY.
//
// One translation unit that compiles the reference's CPU kernels and format builders
// (ternaryLLM_CPU/src/GEMM_CPU_FP32.cpp, GEMM_CPU_INT8.cpp, TCSC.hpp) exactly as they are and exposes
// them through a small extern "C" surface, so that tests can (a) pin the C restatement in oracle.c
// against the reference's own code and (b) time the reference CPU path as the benchmark's CPU baseline.
// Built by oracle/build_ref.py, which also generates ref_table.inc (kernel name -> function pointer,
// limited to kernels that are both declared and defined).
//
// The only intervention is mapping the aligned AVX load/store intrinsics to their unaligned forms: the
// kernels apply them to addresses that are merely element-aligned, which MSVC (the reference's
// compiler) tolerates by emitting unaligned moves and g++ does not.
#include <immintrin.h>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>
#include <omp.h>

#define _mm256_load_ps _mm256_loadu_ps
#define _mm256_store_ps _mm256_storeu_ps
#define _mm256_load_si256 _mm256_loadu_si256
#define _mm256_store_si256 _mm256_storeu_si256
#define _mm512_load_ps _mm512_loadu_ps
#define _mm512_store_ps _mm512_storeu_ps
#define _mm512_load_si512 _mm512_loadu_si512
#define _mm512_store_si512 _mm512_storeu_si512

#include "GEMM_CPU_FP32.cpp"
#include "GEMM_CPU_INT8.cpp"
#include "TCSC.hpp"

template <typename F>
struct Entry {
    const char* name;
    F fn;
};
#include "ref_table.inc"

template <typename F>
static F lookup(const Entry<F>* t, const char* name) {
    for (; t->name; ++t)
        if (std::strcmp(t->name, name) == 0) return t->fn;
    return nullptr;
}

template <typename F>
static int list_names(const Entry<F>* t, char* buf, int cap) {
    int used = 0;
    for (; t->name; ++t) {
        const int l = (int)std::strlen(t->name);
        if (used + l + 2 > cap) return -1;
        std::memcpy(buf + used, t->name, l);
        used += l;
        buf[used++] = '\n';
    }
    if (cap > 0) buf[used] = 0;
    return used;
}

template <typename T>
static int64_t copy_out(const std::vector<T>& v, T* dst, int64_t cap) {
    if ((int64_t)v.size() > cap) return -1;
    if (!v.empty()) std::memcpy(dst, v.data(), v.size() * sizeof(T));
    return (int64_t)v.size();
}

extern "C" {

void ref_set_threads(int n) { omp_set_num_threads(n); }
int ref_max_threads() { return omp_get_max_threads(); }

// family: 1..9 = F1,F2,F3,F4,F4U,F5,F6,F6U,FD ; newline separated names into buf
int ref_list(int family, char* buf, int cap) {
    switch (family) {
        case 1: return list_names(TABLE_F1, buf, cap);
        case 2: return list_names(TABLE_F2, buf, cap);
        case 3: return list_names(TABLE_F3, buf, cap);
        case 4: return list_names(TABLE_F4, buf, cap);
        case 5: return list_names(TABLE_F4U, buf, cap);
        case 6: return list_names(TABLE_F5, buf, cap);
        case 7: return list_names(TABLE_F6, buf, cap);
        case 8: return list_names(TABLE_F6U, buf, cap);
        case 9: return list_names(TABLE_FD, buf, cap);
    }
    return -1;
}

int ref_f1(const char* name, const float* X, const int32_t* meta, const int16_t* ri, float* out, int M, int N, int K) {
    auto f = lookup(TABLE_F1, name); if (!f) return -1; f(X, meta, ri, out, M, N, K); return 0;
}
int ref_f2(const char* name, const float* X, int32_t nz, const int16_t* ri, float* out, int M, int N, int K) {
    auto f = lookup(TABLE_F2, name); if (!f) return -1; f(X, nz, ri, out, M, N, K); return 0;
}
int ref_f3(const char* name, float* X, int32_t* meta, int32_t* ri, float* out, int M, int N, int K) {
    auto f = lookup(TABLE_F3, name); if (!f) return -1; f(X, meta, ri, out, M, N, K); return 0;
}
int ref_f4(const char* name, const float* X, const int32_t* meta, const int32_t* ri, float* out, int N, int K) {
    auto f = lookup(TABLE_F4, name); if (!f) return -1; f(X, meta, ri, out, N, K); return 0;
}
int ref_f4u(const char* name, const float* X, int32_t nz, const int32_t* ri, float* out, int N, int K) {
    auto f = lookup(TABLE_F4U, name); if (!f) return -1; f(X, nz, ri, out, N, K); return 0;
}
int ref_f5(const char* name, float* X, int16_t* ni, int32_t* np, int16_t* pi, int32_t* pp, float* out, int M, int N, int K) {
    auto f = lookup(TABLE_F5, name); if (!f) return -1; f(X, ni, np, pi, pp, out, M, N, K); return 0;
}
int ref_f6(const char* name, const int8_t* X, const int32_t* meta, const int16_t* ri, int8_t* out, int M, int N, int K) {
    auto f = lookup(TABLE_F6, name); if (!f) return -1; f(X, meta, ri, out, M, N, K); return 0;
}
int ref_f6u(const char* name, const int8_t* X, int32_t nz, const int16_t* ri, int8_t* out, int M, int N, int K) {
    auto f = lookup(TABLE_F6U, name); if (!f) return -1; f(X, nz, ri, out, M, N, K); return 0;
}
int ref_fd(const char* name, float* X, int8_t* W, float* out, int M, int N, int K) {
    auto f = lookup(TABLE_FD, name); if (!f) return -1; f(X, W, out, M, N, K); return 0;
}

// SparseFormat (TCSC.hpp:6-34).  csp/csn need N+1 entries; rip/rin need cap entries.
int64_t ref_sparse_format(const int8_t* W, int K, int N, int32_t* csp, int32_t* csn, int16_t* rip, int16_t* rin,
                          int64_t cap, int64_t* n_neg) {
    SparseFormat s(W, K, N);
    std::memcpy(csp, s.col_start_pos.data(), sizeof(int) * (N + 1));
    std::memcpy(csn, s.col_start_neg.data(), sizeof(int) * (N + 1));
    *n_neg = copy_out(s.row_index_neg, rin, cap);
    return copy_out(s.row_index_pos, rip, cap);
}

// MergedTCSC (TCSC.hpp:36-90)
int64_t ref_merged_tcsc(const int8_t* W, int K, int N, int32_t* meta, int16_t* ri, int64_t cap) {
    SparseFormat s(W, K, N);
    MergedTCSC m(s, K, N);
    std::memcpy(meta, m.metadata.data(), sizeof(int) * m.metadata.size());
    return copy_out(m.row_index, ri, cap);
}

// MergedTCSC_Group (TCSC.hpp:92-409); simd <= 0 selects the six-argument constructor.
int64_t ref_merged_group(const int8_t* W, int K, int N, int G, const char* method, int interleaved, int simd,
                         int32_t* meta, int64_t meta_cap, int16_t* ri, int64_t ri_cap, int64_t* meta_len) {
    SparseFormat s(W, K, N);
    if (simd <= 0) {
        MergedTCSC_Group g(s, K, N, G, std::string(method), interleaved != 0);
        *meta_len = copy_out(g.metadata, (int*)meta, meta_cap);
        return copy_out(g.row_index, ri, ri_cap);
    }
    MergedTCSC_Group g(s, K, N, G, std::string(method), interleaved != 0, simd);
    *meta_len = copy_out(g.metadata, (int*)meta, meta_cap);
    return copy_out(g.row_index, ri, ri_cap);
}

// sparseGEMM<float> (TCSC.hpp:413-430): the only place the reference applies a bias.
void ref_sparse_gemm_f32(float* X, const int8_t* W, float* bias, float* Y, int M, int N, int K) {
    SparseFormat s(W, K, N);
    sparseGEMM<float>(X, s, bias, Y, M, N, K);
}

}  // extern "C"
