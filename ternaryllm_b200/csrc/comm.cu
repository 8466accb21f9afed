// comm.cu -- one-shot all-reduce over peer memory, fused with the residual add and RMSNorm that follow it.
//
// In a tensor-parallel decoder layer the row-sharded products (O and down) leave a full-width partial result
// [rows][hidden] on every GPU; what the layer needs next is  x += sum over ranks;  h = RMSNorm(x).  (The
// reference has no distributed code; the contract is the usual tensor-parallel partitioning.)  This file does
// that in one kernel per GPU instead of an NCCL all-reduce plus a glue kernel:
//
//   push    every rank stores its fp32 partial row into its slot of every peer's receive buffer -- plain 16-byte
//           stores to peer-mapped memory over NVLink -- then releases a flag per peer (system-scope fence, then
//           the epoch number);
//   wait    one thread per peer polls this GPU's own flags until they show the epoch (bounded: about a second,
//           then the block gives up and reports through the status word);
//   reduce  all ranks add the slots in rank order (so every GPU computes the same bits), add the sum to the
//           residual row, and normalise.
//
// One thread block per activation row.  Receive buffers and flags are double-buffered by epoch parity: a rank
// can start all-reduce e+1 while a slower rank still reads the slots of e, and nobody can start e+2 before
// everybody has pushed e+1.  No TMA, no multicast, no library kernel touches peer memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <vector>

#include "../../include/tllm.h"
#include "kernels.cuh"
#include "util.h"

namespace tllm {

#define COMM_MAX_WORLD 16
#define COMM_MAX_SPLIT 8        // thread blocks that share one activation row
#define COMM_ERR_PEER_WAIT 201

struct CommParams {
    const float* partial;               // [rows][hidden] this rank's partial sums
    float* recv[COMM_MAX_WORLD];        // every rank's receive buffer [2][world][max_rows][hidden] (own one included)
    uint32_t* flags[COMM_MAX_WORLD];    // every rank's flags [2][world][max_rows][COMM_MAX_SPLIT]
    uint32_t* epoch;                    // [max_rows] all-reduces this row has been through (local)
    float* ssq;                         // [2][max_rows][COMM_MAX_SPLIT] the slices' sums of squares (local)
    unsigned int* arrive;               // [2][max_rows] blocks of the row that have stored theirs (local)
    int split;                          // thread blocks per row
    void* x;
    const void* weight;
    void* h;
    int* status;
    long long wait_clocks;
    int world, rank, max_rows, hidden;
    float eps;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One activation row is handled by `split` thread blocks, each a contiguous slice of the hidden dimension: the push to
// the peers then leaves from several SMs at once (a single SM's stores over NVLink were the slowest part with four or
// more ranks), and every block waits only for its own slice of the peers' rows.  The sum of squares of the row is put
// together through global memory: every block stores its slice's part, arrives on a counter, waits (bounded) until all
// blocks of the row have arrived and adds the parts in slice order -- all blocks, and all ranks, get the same bits.
// The blocks of a row are at most COMM_MAX_SPLIT of one launch, far fewer than SMs, so they are resident together.
template <typename T>
__global__ void __launch_bounds__(512) push_allreduce_add_rmsnorm_kernel(const __grid_constant__ CommParams p) {
    constexpr int NV = RmsVec<T>::N;   // values of T per 16 bytes
    __shared__ float red[32];
    __shared__ float total_s;
    const int r = blockIdx.x / p.split, sl = blockIdx.x % p.split, tid = threadIdx.x, nt = blockDim.x;
    const int slice = p.hidden / p.split;                  // values of this block's slice
    const size_t off = (size_t)sl * slice;                 // first value of the slice inside the row
    const int nvec4 = slice / 4, nvec = slice / NV;
    // The partial sums, the residual row and this row's epoch come from kernels earlier in the stream.
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t e = p.epoch[r] + 1u;
    const size_t set = e & 1u;
    if (sl == 0 && tid == 0) {                             // the other buffer set's barrier words are free again: clear them for call e + 1
        p.arrive[(set ^ 1u) * p.max_rows + r] = 0u;
    }
    const float4* mine = (const float4*)(p.partial + (size_t)r * p.hidden + off);
    // ---- push this rank's slice into its slot on every peer ----
    for (int q = 1; q < p.world; ++q) {
        const int peer = (p.rank + q) % p.world;   // start with the neighbour: ranks do not all hit the same GPU first
        float4* dst = (float4*)(p.recv[peer] + ((set * p.world + p.rank) * p.max_rows + r) * (size_t)p.hidden + off);
        for (int i = tid; i < nvec4; i += nt) dst[i] = __ldcg(mine + i);
    }
    __syncthreads();
    if (tid < p.world && tid != p.rank) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + ((set * p.world + p.rank) * p.max_rows + r) * COMM_MAX_SPLIT + sl, e);
    }
    // ---- what does not depend on the peers is read while their rows are on the way: the residual row and the norm weight
    T* x = (T*)p.x + (size_t)r * p.hidden + off;
    T* h = (T*)p.h + (size_t)r * p.hidden + off;
    const T* wgt = p.weight ? (const T*)p.weight + off : nullptr;
    constexpr int KEEP = 2;             // vectors of the slice a thread keeps in registers
    float keep[KEEP][8], gain[KEEP][8];
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int vi = tid + k * nt;
        if (vi < nvec) {
            RmsVec<T>::load(x + (size_t)vi * NV, keep[k]);
            if (wgt) RmsVec<T>::load(wgt + (size_t)vi * NV, gain[k]);
        }
    }
    // ---- wait for this slice of every peer's row ----
    if (tid < p.world && tid != p.rank) {
        const uint32_t* f = p.flags[p.rank] + ((set * p.world + tid) * p.max_rows + r) * COMM_MAX_SPLIT + sl;
        if (ld_acquire_sys(f) != e) {
            const long long t0 = clock64();
            while (ld_acquire_sys(f) != e) {
                if (clock64() - t0 > p.wait_clocks) {   // give up: the result is undefined and the status word says so
                    atomicExch(p.status, COMM_ERR_PEER_WAIT);
                    break;
                }
            }
        }
    }
    __syncthreads();
    // ---- x += sum over ranks (rank order) ----
    const float* mine_recv = p.recv[p.rank] + (set * p.world * p.max_rows + r) * (size_t)p.hidden + off;   // slot of rank 0, row r, this slice
    const size_t slot_stride = (size_t)p.max_rows * p.hidden;
    float ss = 0.f;
    auto first_pass = [&](int vi, float (&v)[8]) {      // v holds the residual values on entry
        float s[8];
#pragma unroll
        for (int i = 0; i < NV; ++i) s[i] = 0.f;
        for (int src = 0; src < p.world; ++src) {
            const float* row = src == p.rank ? (const float*)mine : mine_recv + src * slot_stride;
#pragma unroll
            for (int i = 0; i < NV; i += 4) {
                const float4 a = __ldcg((const float4*)(row + (size_t)vi * NV + i));
                s[i] += a.x, s[i + 1] += a.y, s[i + 2] += a.z, s[i + 3] += a.w;
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) v[i] = RmsVec<T>::round(v[i] + s[i]);
        RmsVec<T>::store(x + (size_t)vi * NV, v);
#pragma unroll
        for (int i = 0; i < NV; ++i) ss += v[i] * v[i];
    };
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int vi = tid + k * nt;
        if (vi < nvec) first_pass(vi, keep[k]);
    }
    for (int vi = tid + KEEP * nt; vi < nvec; vi += nt) {
        float v[8];
        RmsVec<T>::load(x + (size_t)vi * NV, v);
        first_pass(vi, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    // ---- the row's sum of squares: this slice's part out, all slices' parts in (slice order) ----
    if (tid == 0) {
        float part = 0.f;
        for (int w = 0; w < (nt + 31) / 32; ++w) part += red[w];
        float tot = part;
        if (p.split > 1) {
            float* parts = p.ssq + (set * p.max_rows + r) * COMM_MAX_SPLIT;
            unsigned int* arr = p.arrive + set * p.max_rows + r;
            __stcg(parts + sl, part);
            __threadfence();
            atomicAdd(arr, 1u);
            const long long t0 = clock64();
            while (*(volatile unsigned int*)arr < (unsigned int)p.split) {
                if (clock64() - t0 > p.wait_clocks) {   // a block of this row never came: report, use what is there
                    atomicExch(p.status, COMM_ERR_PEER_WAIT);
                    break;
                }
            }
            __threadfence();
            tot = 0.f;
            for (int i = 0; i < p.split; ++i) tot += __ldcg(parts + i);
        }
        total_s = tot;
        if (sl == 0) p.epoch[r] = e;                       // every block of the row has read the epoch by now
    }
    __syncthreads();
    const float inv = rsqrtf(total_s / (float)p.hidden + p.eps);
    auto second_pass = [&](int vi, float (&v)[8], const float (&g)[8]) {
        if (wgt) {
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] = v[i] * inv * g[i];
        } else {
#pragma unroll
            for (int i = 0; i < NV; ++i) v[i] = v[i] * inv;
        }
        RmsVec<T>::store(h + (size_t)vi * NV, v);
    };
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        const int vi = tid + k * nt;
        if (vi < nvec) second_pass(vi, keep[k], gain[k]);
    }
    for (int vi = tid + KEEP * nt; vi < nvec; vi += nt) {
        float v[8], g[8];
        RmsVec<T>::load(x + (size_t)vi * NV, v);
        if (wgt) RmsVec<T>::load(wgt + (size_t)vi * NV, g);
        second_pass(vi, v, g);
    }
}

}  // namespace tllm

using namespace tllm;

struct tllm_comm {
    int world = 1, rank = 0, max_rows = 0, hidden = 0, device = 0;
    float* recv = nullptr;          // own receive buffer
    uint32_t* flags = nullptr;      // own flags
    uint32_t* epoch = nullptr;
    float* ssq = nullptr;
    unsigned int* arrive = nullptr;
    int* status = nullptr;
    float* peer_recv[COMM_MAX_WORLD] = {};
    uint32_t* peer_flags[COMM_MAX_WORLD] = {};
    bool opened[COMM_MAX_WORLD] = {};      // mapped with cudaIpcOpenMemHandle (to be closed)
    bool connected = false;
    long long wait_clocks = 2000000000LL;   // about a second of SM clocks
    size_t recv_bytes = 0, flag_bytes = 0;
};

#define CC_TRY(expr)                                                                                       \
    do {                                                                                                   \
        cudaError_t e_ = (expr);                                                                           \
        if (e_ != cudaSuccess) return fail(TLLM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

extern "C" {

int tllm_comm_create(int world, int rank, int max_rows, int hidden, tllm_comm** out) {
    if (!out || world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world || max_rows < 1 || hidden < 8 || hidden % 8)
        return fail(TLLM_ERR_ARG, "tllm_comm_create: bad argument (world 1..%d, hidden a multiple of 8)", COMM_MAX_WORLD);
    *out = nullptr;
    tllm_comm* c = new tllm_comm();
    c->world = world, c->rank = rank, c->max_rows = max_rows, c->hidden = hidden;
    c->recv_bytes = (size_t)2 * world * max_rows * hidden * sizeof(float);
    c->flag_bytes = (size_t)2 * world * max_rows * COMM_MAX_SPLIT * sizeof(uint32_t);
    cudaError_t e = cudaGetDevice(&c->device);
    if (e == cudaSuccess) e = cudaMalloc(&c->recv, c->recv_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->flags, c->flag_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&c->epoch, (size_t)max_rows * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMalloc(&c->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&c->ssq, (size_t)2 * max_rows * COMM_MAX_SPLIT * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&c->arrive, (size_t)2 * max_rows * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(c->arrive, 0, (size_t)2 * max_rows * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(c->flags, 0, c->flag_bytes);
    if (e == cudaSuccess) e = cudaMemset(c->epoch, 0, (size_t)max_rows * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(c->status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        tllm_comm_destroy(c);
        return fail(TLLM_ERR_CUDA, "tllm_comm_create: %s", cudaGetErrorString(e));
    }
    c->peer_recv[rank] = c->recv;
    c->peer_flags[rank] = c->flags;
    c->connected = world == 1;
    *out = c;
    return TLLM_OK;
}

int tllm_comm_handle_bytes(void) { return 2 * (int)sizeof(cudaIpcMemHandle_t); }

int tllm_comm_export(tllm_comm* c, void* handle) {
    if (!c || !handle) return fail(TLLM_ERR_ARG, "tllm_comm_export: NULL");
    cudaIpcMemHandle_t h[2];
    CC_TRY(cudaIpcGetMemHandle(&h[0], c->recv));
    CC_TRY(cudaIpcGetMemHandle(&h[1], c->flags));
    std::memcpy(handle, h, sizeof h);
    return TLLM_OK;
}

int tllm_comm_connect(tllm_comm* c, const void* handles) {
    if (!c || !handles) return fail(TLLM_ERR_ARG, "tllm_comm_connect: NULL");
    int dev = 0;
    CC_TRY(cudaGetDevice(&dev));
    if (dev != c->device) return fail(TLLM_ERR_ARG, "tllm_comm_connect: device %d is current, the communicator lives on %d", dev, c->device);
    const cudaIpcMemHandle_t* h = (const cudaIpcMemHandle_t*)handles;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank || c->peer_recv[r]) continue;
        void *a = nullptr, *b = nullptr;
        CC_TRY(cudaIpcOpenMemHandle(&a, h[2 * r], cudaIpcMemLazyEnablePeerAccess));
        CC_TRY(cudaIpcOpenMemHandle(&b, h[2 * r + 1], cudaIpcMemLazyEnablePeerAccess));
        c->peer_recv[r] = (float*)a;
        c->peer_flags[r] = (uint32_t*)b;
        c->opened[r] = true;
    }
    c->connected = true;
    return TLLM_OK;
}

int tllm_comm_attach(tllm_comm* c, int peer, void* recv, void* flags) {
    if (!c || peer < 0 || peer >= c->world || peer == c->rank || !recv || !flags) return fail(TLLM_ERR_ARG, "tllm_comm_attach: bad argument");
    c->peer_recv[peer] = (float*)recv;
    c->peer_flags[peer] = (uint32_t*)flags;
    bool all = true;
    for (int r = 0; r < c->world; ++r) all = all && c->peer_recv[r] && c->peer_flags[r];
    c->connected = all;
    return TLLM_OK;
}

int tllm_comm_buffers(tllm_comm* c, void** recv, void** flags, int64_t* recv_bytes, int64_t* flag_bytes) {
    if (!c) return fail(TLLM_ERR_ARG, "tllm_comm_buffers: NULL");
    if (recv) *recv = c->recv;
    if (flags) *flags = c->flags;
    if (recv_bytes) *recv_bytes = (int64_t)c->recv_bytes;
    if (flag_bytes) *flag_bytes = (int64_t)c->flag_bytes;
    return TLLM_OK;
}

int tllm_comm_set_wait_limit(tllm_comm* c, double milliseconds) {
    if (!c || !(milliseconds > 0)) return fail(TLLM_ERR_ARG, "tllm_comm_set_wait_limit: bad argument");
    int khz = 0;
    CC_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device));
    c->wait_clocks = (long long)(milliseconds * (double)khz);
    return TLLM_OK;
}

int tllm_comm_check(tllm_comm* c) {
    if (!c) return fail(TLLM_ERR_ARG, "tllm_comm_check: NULL");
    int st = 0;
    CC_TRY(cudaMemcpy(&st, c->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(c->status, 0, sizeof(int));
        return fail(TLLM_ERR_KERNEL, "all-reduce: a peer's row never arrived within the wait limit (code %d); the ranks' epochs may differ now: "
                                     "destroy the communicator on every rank", st);
    }
    return TLLM_OK;
}

int tllm_comm_destroy(tllm_comm* c) {
    if (!c) return TLLM_OK;
    for (int r = 0; r < c->world; ++r)
        if (c->opened[r]) {
            cudaIpcCloseMemHandle(c->peer_recv[r]);
            cudaIpcCloseMemHandle(c->peer_flags[r]);
        }
    cudaFree(c->recv);
    cudaFree(c->flags);
    cudaFree(c->epoch);
    cudaFree(c->ssq);
    cudaFree(c->arrive);
    cudaFree(c->status);
    delete c;
    return TLLM_OK;
}

int tllm_allreduce_add_rmsnorm(tllm_comm* c, const float* partial, void* x, const void* weight, void* h, int dtype, int rows, float eps, void* stream) {
    if (!c || !partial || !x || !h) return fail(TLLM_ERR_ARG, "tllm_allreduce_add_rmsnorm: NULL pointer");
    if (rows < 0 || rows > c->max_rows) return fail(TLLM_ERR_ARG, "tllm_allreduce_add_rmsnorm: %d rows, the communicator was created for %d", rows, c->max_rows);
    if (dtype != TLLM_F32 && dtype != TLLM_F16 && dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "tllm_allreduce_add_rmsnorm: unsupported dtype");
    if (!c->connected) return fail(TLLM_ERR_ARG, "tllm_allreduce_add_rmsnorm: the communicator is not connected to its peers");
    if (((uintptr_t)partial | (uintptr_t)x | (uintptr_t)h | (uintptr_t)weight) % 16) return fail(TLLM_ERR_ARG, "tllm_allreduce_add_rmsnorm: pointers must be 16-byte aligned");
    int dev = 0;
    CC_TRY(cudaGetDevice(&dev));
    if (dev != c->device) return fail(TLLM_ERR_ARG, "tllm_allreduce_add_rmsnorm: device %d is current, the communicator lives on %d", dev, c->device);
    if (rows == 0) return TLLM_OK;
    CommParams p{};
    p.partial = partial;
    for (int r = 0; r < c->world; ++r) {
        p.recv[r] = c->peer_recv[r];
        p.flags[r] = c->peer_flags[r];
    }
    p.epoch = c->epoch;
    p.ssq = c->ssq;
    p.arrive = c->arrive;
    p.x = x, p.weight = weight, p.h = h;
    p.status = c->status;
    p.wait_clocks = c->wait_clocks;
    p.world = c->world, p.rank = c->rank, p.max_rows = c->max_rows, p.hidden = c->hidden;
    p.eps = eps;
    const int vec = dtype == TLLM_F32 ? 4 : 8;
    // slices of at least 1024 values, a whole number of 16-byte vectors each, at most COMM_MAX_SPLIT of them.
    // Measured: with one or two ranks a single block per row (up to 512 threads, two vectors each in registers) is
    // faster; with four ranks the split is (134.9 against 131.8 tokens/s at batch 1).
    int split = 1;
    while (c->world >= 4 && split < COMM_MAX_SPLIT && c->hidden % (split * 2 * 8) == 0 && c->hidden / (split * 2) >= 1024) split *= 2;
    p.split = split;
    int threads = (c->hidden / split / vec + 1) / 2;  // two vectors per thread stay in registers
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : (threads + 31) / 32 * 32);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(rows * split));
    cfg.blockDim = dim3((unsigned)threads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (dtype == TLLM_F32) CC_TRY(cudaLaunchKernelEx(&cfg, push_allreduce_add_rmsnorm_kernel<float>, p));
    else if (dtype == TLLM_F16) CC_TRY(cudaLaunchKernelEx(&cfg, push_allreduce_add_rmsnorm_kernel<__half>, p));
    else CC_TRY(cudaLaunchKernelEx(&cfg, push_allreduce_add_rmsnorm_kernel<__nv_bfloat16>, p));
    note_launch();
    return TLLM_OK;
}

}  // extern "C"
