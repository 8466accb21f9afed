// kernels.cuh -- sm_100a device code of libtllm shared by its kernels, and the small kernels.
//
//   helpers               mbarrier / bulk-copy / programmatic-dependent-launch wrappers, bounded waits, typed loads
//   mcsc_spmm_kernel      the product directly on the reference's merged tiled CSC arrays
//                         (what ter_tiled_mcsc_spmv / ter_tiled_mcsc_spmm compute,
//                         ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:24-78, :106-308), for callers that hold
//                         those arrays.
//   silu_mul_kernel       SiLU(g)*u (ternaryLLM_CPU/src/initData.hpp:204-210).
//   bias_add_kernel       Y += bias per column (the bias of sparseGEMM, ternaryLLM_CPU/src/TCSC.hpp:413-430).
//   add_rmsnorm_kernel    residual add + RMSNorm between two products of a decoder layer (the reference leaves
//                         this to stock Hugging Face modules).
//
// The decode product itself is in bstream_kernel.cuh, the tensor-core product in mma_kernel.cuh.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tllm.h"

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

template <typename T>
__device__ __forceinline__ T bits_as(uint32_t v);
template <>
__device__ __forceinline__ float bits_as<float>(uint32_t v) { return __uint_as_float(v); }
template <>
__device__ __forceinline__ int bits_as<int>(uint32_t v) { return (int)v; }

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

// activation element i of a raw tile staged in shared memory
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
static __global__ void silu_mul_kernel(void* g, const void* u, int dtype, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = load_act_f32(g, dtype, (size_t)i), bq = load_act_f32(u, dtype, (size_t)i);
    store_out(g, dtype, (size_t)i, silu_mul(a, bq));
}

// y[i] += bias[i % columns], both of `dtype` (fp32 sum, rounded once; int32 adds exactly)
static __global__ void bias_add_kernel(void* y, const void* bias, int dtype, long long n, int columns) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int c = (int)(i % columns);
    if (dtype == TLLM_I32) ((int*)y)[i] += ((const int*)bias)[c];
    else store_out(y, dtype, (size_t)i, load_act_f32(y, dtype, (size_t)i) + load_act_f32(bias, dtype, (size_t)c));
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
