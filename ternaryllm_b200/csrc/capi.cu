// capi.cu -- the C ABI of libtllm (declared in include/tllm.h): handles, launches, host staging.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include <cudaTypedefs.h>

#include "bstream_kernel.cuh"
#include "kernels.cuh"
#include "mma_kernel.cuh"
#include "nibble_format.h"
#include "nibble_kernel.cuh"
#include "nibble_rows_kernel.cuh"
#include "util.h"

namespace tllm {

static thread_local std::string g_err;
static std::atomic<int64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

#define CU_TRY(expr)                                                                                       \
    do {                                                                                                   \
        cudaError_t e_ = (expr);                                                                           \
        if (e_ != cudaSuccess) return fail(TLLM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

static size_t dtype_size(int dt) {
    switch (dt) {
        case TLLM_F32: case TLLM_I32: return 4;
        case TLLM_F16: case TLLM_BF16: return 2;
        case TLLM_I8: return 1;
    }
    return 0;
}

// Which kernel takes a call: -1 = decide per call from a cost model of the two kernels (the default), 0 = never the
// tensor-core kernel, n > 0 = from n activation rows on.  TLLM_MMA_MIN_ROWS sets the initial value.
static std::atomic<int> g_mm_min_rows{-2};
static std::atomic<int64_t> g_mm_launches{0};
static int mm_min_rows() {
    int v = g_mm_min_rows.load(std::memory_order_relaxed);
    if (v == -2) {
        const char* e = getenv("TLLM_MMA_MIN_ROWS");
        v = e ? atoi(e) : -1;
        if (v < -1) v = -1;
        g_mm_min_rows.store(v, std::memory_order_relaxed);
    }
    return v;
}
// Cost model measured on B200 (CUDA-graph replays of back-to-back products, weights streamed from HBM), microseconds:
// a gather launch of up to four rows costs about GATHER_FIXED + nnz * g(rows padded to 1, 2, 4), more rows take
// ceil(rows / 4) launches; the batched tensor-core kernel about 9.8 + 0.205e-6 per matrix entry whatever the row count
// up to 64; the decode tensor-core kernel is modelled below.  Every call goes to the kernel the model finds fastest.
static const double GATHER_FIXED_US = 2.9;
static const double GATHER_PS_PER_NNZ[3] = {0.48, 0.68, 1.35};
// The decode tensor-core kernel: -1 = cost model, 0 = never, n > 0 = always for calls of up to n rows.
static std::atomic<int> g_nb_max_rows{-1};
static std::atomic<int64_t> g_nb_launches{0};
#ifdef NB_DEBUG
static int g_nb_debug_tx = 0;   // diagnostic builds only: bytes a weight tile's copy is expected to report
static int g_nb_debug_stages = 0, g_nb_debug_flags = 0;
#endif
// one launch of the decode tensor-core kernel: half a byte per entry at 5.2 TB/s around 6.7 us of start-up (building B
// once the preceding kernel has finished) and hand-over between blocks, 0.9 us more for every further row
static const double NB_FIXED_US = 6.7, NB_ROW_US = 0.9, NB_US_PER_ENTRY = 0.5 / 5.2e6;
static double gather_model_us(int64_t nnz, int rows) {
    const int full = rows / 4, tail = rows % 4;
    const int idx = tail <= 1 ? 0 : (tail == 2 ? 1 : 2);
    return full * (GATHER_FIXED_US + nnz * GATHER_PS_PER_NNZ[2] * 1e-6) + (tail ? GATHER_FIXED_US + nnz * GATHER_PS_PER_NNZ[idx] * 1e-6 : 0.0);
}
// more rows than one such launch takes: the pieces kernel + the many-row kernel, up to 64 (32 fp32) rows per launch.
// Measured per launch with 32 / 64 / 128 / 256 piece rows: start-up and hand-over grow with the rows, and the stream
// slows down as the B tiles it re-reads from L2 and the MMAs grow with the piece rows.
static const double NR_FIXED_US[4] = {13.5, 19.2, 26.9, 42.6}, NR_US_PER_MENTRY[4] = {0.081, 0.075, 0.090, 0.158};
static double nibble_model_us(int64_t entries, int rows, int rows_per_launch) {
    if (rows <= rows_per_launch) return NB_FIXED_US + entries * NB_US_PER_ENTRY + (rows - 1) * NB_ROW_US;
    const int per2 = rows_per_launch * (NR_MAX_NB / NB_ROWS), pieces = NB_ROWS / rows_per_launch;
    double t = 0;
    for (int r0 = 0; r0 < rows; r0 += per2) {
        const int m = rows - r0 < per2 ? rows - r0 : per2;
        int i = 0;
        while ((32 << i) < m * pieces) ++i;
        t += NR_FIXED_US[i] + entries * 1e-6 * NR_US_PER_MENTRY[i];
    }
    return t;
}
static double mm_model_us(int64_t entries, int rows) { return 9.8 + entries * 0.205e-6 * (rows <= 64 ? 1.0 : rows / 64.0); }
static bool mm_model_prefers_tensor(int64_t nnz, int64_t entries, int rows) {
    if (rows < 2) return false;
    return mm_model_us(entries, rows) < gather_model_us(nnz, rows);
}

}  // namespace tllm

using namespace tllm;

struct tllm_weight {
    BsLayout lay;
    float scale = 1.f;
    int device = 0;
    int max_rows = 4;                 // rows of one gather launch
    uint32_t max_meta_words = 0;      // longest block table
    uint4* d_stream = nullptr;
    uint32_t* d_meta = nullptr;
    TsCtaDesc* d_cta = nullptr;
    void* d_partial = nullptr;
    unsigned int* d_counters = nullptr;
    int* d_status = nullptr;
    size_t stream_bytes = 0, meta_bytes = 0, scratch_bytes = 0;
    // staging for the host-buffer entry points
    void* d_x = nullptr;
    void* d_y = nullptr;
    void* d_bias = nullptr;
    void* h_pin = nullptr;
    int* h_status = nullptr;        // pinned copy of the status word, read back with every host-buffer call
    size_t x_cap = 0, y_cap = 0, bias_cap = 0, pin_cap = 0;
    cudaStream_t own_stream = nullptr;
    // tensor-core kernel: dense two-bit copy of W and its split scratch
    uint4* d_bits = nullptr;
    float* d_mm_partial = nullptr;
    unsigned int* d_mm_counters = nullptr;
    size_t bits_bytes = 0;
    int mm_n_tiles = 0, mm_kb = 0, mm_grid = 0;
    // decode tensor-core kernel: transposed four-bit copy of W, its tensor map, schedule and hand-over scratch
    uint8_t* d_nib = nullptr;
    size_t nib_bytes = 0;
    CUtensorMap nib_map;
    int nb_kb = 0, nb_kbs = 0, nb_splits = 0, nb_tiles = 0, nb_gj = 0, nb_uk = 2;
    float* d_nb_partial = nullptr;
    unsigned int* d_nb_counters = nullptr;
    uint32_t* d_nb_sched = nullptr;
    // many-row variant: the activation pieces of a call, their tensor maps (32 / 64 / 128 / 256 piece rows), scratch
    uint8_t* d_nr_pieces = nullptr;
    float* d_nr_row_pow = nullptr;
    float* d_nr_partial = nullptr;
    unsigned int* d_nr_counters = nullptr;
    CUtensorMap nr_map[4];
    int nb_k_pad = 0, nr_grid = 0;
    // the activation tensor map of the last tensor-core launch (encoding one costs more than a short launch)
    CUtensorMap tmap;
    const void* tmap_x = nullptr;
    int tmap_dtype = -1, tmap_rows = 0, tmap_ld = 0, tmap_nt = 0;
};

struct tllm_mlp {
    tllm_weight* gate_up = nullptr;   // columns interleaved: 2c = gate column c, 2c+1 = up column c
    tllm_weight* down = nullptr;
    int hidden = 0, inter = 0;
    float s_gate = 1.f, s_up = 1.f;
    void* d_h = nullptr;
    size_t h_cap = 0;
    // staging for the host-buffer entry point
    void* d_x = nullptr;
    void* d_y = nullptr;
    size_t x_cap = 0, y_cap = 0;
};

namespace {

// scratch of one gather launch: the handle's own, or the library's built-in array (tllm_spmm_static_scratch)
struct Scratch {
    void* partial;
    unsigned int* counters;
};

template <typename ACC, int MP>
int launch_bs(const BsParams& p, int grid, size_t smem, cudaStream_t st) {
    auto kern = bstream_spmm_kernel<ACC, MP>;
    static std::mutex mu;
    static bool configured[64] = {};
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(mu);
        if (dev < 64 && !configured[dev]) {
            CU_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            configured[dev] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(BS_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CU_TRY(cudaLaunchKernelEx(&cfg, kern, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TLLM_OK;
}

int check_types(int x_dtype, int y_dtype, const char* who) {
    if (x_dtype == TLLM_I8) {
        if (y_dtype != TLLM_I32) return fail(TLLM_ERR_ARG, "%s: int8 activations produce int32 results (y_dtype must be TLLM_I32)", who);
        return TLLM_OK;
    }
    if (x_dtype != TLLM_F32 && x_dtype != TLLM_F16 && x_dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "%s: unsupported x_dtype %d", who, x_dtype);
    if (y_dtype != TLLM_F32 && y_dtype != TLLM_F16 && y_dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "%s: unsupported y_dtype %d", who, y_dtype);
    return TLLM_OK;
}

// The handle's buffers live on one device; a call made with another device current would launch there with
// pointers from two GPUs.
int check_device(const tllm_weight* w, const char* who) {
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    if (dev != w->device) return fail(TLLM_ERR_ARG, "%s: the weight lives on device %d but device %d is current", who, w->device, dev);
    return TLLM_OK;
}

// ---- tensor-core path -----------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    });
    return fn;
}

// true when the tensor-core kernel can take this call: fp16 / bf16 row-major activations whose rows TMA can address
bool mm_usable(const tllm_weight* w, const void* X, int x_dtype, int x_layout, int x_ld, int rows) {
    // (a TMA box is 64 values wide: narrower matrices stay on the gather kernel)
    if (!w->d_bits || (x_dtype != TLLM_F16 && x_dtype != TLLM_BF16) || x_layout != TLLM_ROW_MAJOR || ((uintptr_t)X % 16) || ((size_t)x_ld * 2 % 16) ||
        w->lay.inners < MM_TILE_K || tensor_map_encoder() == nullptr)
        return false;
    const int thr = mm_min_rows();
    if (thr == 0) return false;
    if (thr > 0) return rows >= thr;
    return mm_model_prefers_tensor(w->lay.nnz, (int64_t)w->lay.inners * w->lay.columns, rows);
}

// the whole product of `rows` activation rows in one launch of the tensor-core kernel
int run_mm(tllm_weight* w, const void* X, int x_dtype, int x_ld, int rows, void* Y, int y_dtype, int y_ld, int epilogue, float scale,
           float scale2, cudaStream_t st) {
    const BsLayout& L = w->lay;
    MmParams p{};
    p.bits = w->d_bits;
    p.Y = Y;
    p.partial = w->d_mm_partial;
    p.counters = w->d_mm_counters;
    p.status = w->d_status;
    p.M = rows;
    p.K = L.inners;
    p.N = L.columns;
    p.KB = w->mm_kb;
    p.n_tiles = w->mm_n_tiles;
    p.Nt = rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256;
    p.m_tiles = (rows + p.Nt - 1) / p.Nt;
    p.y_dtype = y_dtype;
    p.epilogue = epilogue;
    p.y_ld = y_ld;
    // slices per unit and ring depths: narrow activation tiles take four slices per hand-over and a deep ring of
    // bit tiles (the stream from HBM is what matters there), wide ones keep the operand ring deep instead
    p.UK = p.Nt <= 64 ? 4 : 2;
    p.S = p.Nt == 128 ? 3 : 2;
    p.R = p.Nt == 64 ? 4 : 8;
    p.KBU = (p.KB + p.UK - 1) / p.UK;
    p.split = p.Nt <= MM_SPLIT_MAX_NT ? 1 : 0;
    const uint32_t fmt = x_dtype == TLLM_BF16 ? 1u : 0u;
    // instruction descriptor: fp32 accumulate (bits 4-5 = 1), A and B formats (bits 7-9, 10-12), both K-major,
    // N / 8 in bits 17-22, M / 16 in bits 24-28
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.Nt >> 3) << 17) | ((uint32_t)(MM_TILE_N >> 4) << 24);
    p.tmem_cols = 2u * (uint32_t)p.Nt < 32u ? 32u : 2u * (uint32_t)p.Nt;
    // fp16 holds +-1.0 (0x3C00 / 0xBC00); bf16 holds +-2.0 (0x4000 / 0xC000, whose low byte is zero like fp16's)
    // and the factor 1/2 moves into the scale
    p.pool = fmt ? 0x00C04000u : 0x00BC3C00u;
    p.scale = fmt ? scale * 0.5f : scale;
    p.scale2 = fmt ? scale2 * 0.5f : scale2;

    if (w->tmap_x != X || w->tmap_dtype != x_dtype || w->tmap_rows != rows || w->tmap_ld != x_ld || w->tmap_nt != p.Nt) {
        const cuuint64_t dims[2] = {(cuuint64_t)L.inners, (cuuint64_t)rows};
        const cuuint64_t strides[1] = {(cuuint64_t)x_ld * 2u};
        const cuuint32_t box[2] = {MM_TILE_K, (cuuint32_t)p.Nt};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult cr = tensor_map_encoder()(&w->tmap, fmt ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(X), dims,
                                                 strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            w->tmap_x = nullptr;
            return fail(TLLM_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)cr);
        }
        w->tmap_x = X, w->tmap_dtype = x_dtype, w->tmap_rows = rows, w->tmap_ld = x_ld, w->tmap_nt = p.Nt;
    }

    const size_t smem = 1024 + (size_t)p.S * p.UK * (MM_A_STAGE_BYTES + (size_t)p.Nt * 128) + (size_t)p.R * p.UK * MM_CHUNK_BYTES + 512;
    if (smem > 227 * 1024) return fail(TLLM_ERR_ARG, "tensor-core kernel: ring configuration needs %zu bytes of shared memory", smem);
    void (*kern)(CUtensorMap, MmParams) = p.UK == 4 ? mma_spmm_kernel<4> : mma_spmm_kernel<2>;
    static std::mutex mu;
    static bool configured[64][2] = {};
    {
        std::lock_guard<std::mutex> lk(mu);
        const int slot = p.UK == 4 ? 1 : 0;
        if (w->device < 64 && !configured[w->device][slot]) {
            CU_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            configured[w->device][slot] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    // never more blocks than work items: the hand-over between the blocks that share a tile counts on every
    // block in a tile's range of owners holding at least one unit of it
    const long long tiles = (long long)p.n_tiles * p.m_tiles, items = p.split ? tiles * p.KBU : tiles;
    cfg.gridDim = dim3((unsigned)(items < w->mm_grid ? items : w->mm_grid));
    cfg.blockDim = dim3(MM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    CU_TRY(cudaLaunchKernelEx(&cfg, kern, w->tmap, p));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    g_mm_launches.fetch_add(1, std::memory_order_relaxed);
    return TLLM_OK;
}

// ---- decode tensor-core path ---------------------------------------------------------------------------------
int nb_rows_per_launch(int x_dtype) { return x_dtype == TLLM_F32 ? NB_ROWS / 8 : NB_ROWS / 4; }

// true when the decode tensor-core kernel can and should take this call
bool nb_usable(const tllm_weight* w, int x_dtype, int x_layout, int rows) {
    if (!w->d_nib || (x_dtype != TLLM_F16 && x_dtype != TLLM_BF16 && x_dtype != TLLM_F32) || x_layout != TLLM_ROW_MAJOR) return false;
    if (mm_min_rows() == 0) return false;
    const int thr = g_nb_max_rows.load(std::memory_order_relaxed);
    if (thr == 0) return false;
    if (thr > 0) return rows <= thr;
    const int64_t entries = (int64_t)w->lay.inners * w->lay.columns;
    return nibble_model_us(entries, rows, nb_rows_per_launch(x_dtype)) < gather_model_us(w->lay.nnz, rows);
}

int upload_nibbles(tllm_weight* w, const int8_t* dense, int inners, int columns, int sms) {
    if (tensor_map_encoder() == nullptr) return TLLM_OK;      // no driver entry point: the handle simply has no such copy
    NbHostImage img;
    nb_pack_dense(dense, inners, columns, &img);
    w->nib_bytes = img.codes.size();
    CU_TRY(cudaMalloc(&w->d_nib, w->nib_bytes));
    CU_TRY(cudaMemcpy(w->d_nib, img.codes.data(), w->nib_bytes, cudaMemcpyHostToDevice));
    const cuuint64_t dims[2] = {(cuuint64_t)img.k_pad, (cuuint64_t)img.n_pad};
    const cuuint64_t strides[1] = {(cuuint64_t)img.k_pad / 2};
    const cuuint32_t box[2] = {NB_TILE_K, NB_TILE_N};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = tensor_map_encoder()(&w->nib_map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, w->d_nib, dims, strides, box, estr,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(TLLM_ERR_CUDA, "cuTensorMapEncodeTiled (four-bit weight planes) failed with code %d", (int)cr);
    // One block per SM, two tiles per unit, K ranges of up to 32 blocks.  (Two blocks per SM with one tile per unit and
    // ranges of 16 -- a block's start-up and hand-over overlapping the other's streaming -- measured 5 to 35 % slower.)
    static_assert(NB_FMT_TILE == NB_TILE_K && NB_FMT_TILE == NB_TILE_N && NB_FMT_MAX_KBS == NB_MAX_KBS && NB_FMT_UK == 2,
                  "the host schedule and the kernel (launched as nibble_spmm_kernel<2>) disagree");
    NbSchedule plan;
    nb_make_schedule(img.k_pad, img.n_pad, sms, &plan);
    w->nb_uk = plan.uk, w->nb_kb = plan.kb, w->nb_tiles = plan.tiles, w->nb_kbs = plan.kbs, w->nb_splits = plan.splits, w->nb_gj = plan.gj;
    const std::vector<uint32_t>& sched = plan.words;
    const size_t partial_bytes = (size_t)w->nb_splits * ((size_t)w->nb_tiles + w->nb_gj) * (NB_ROWS / 4) * NB_TILE_N * sizeof(float);
    const size_t counter_bytes = (size_t)w->nb_tiles * 4 * sizeof(unsigned int);
    CU_TRY(cudaMalloc(&w->d_nb_sched, sched.size() * sizeof(uint32_t)));
    CU_TRY(cudaMemcpy(w->d_nb_sched, sched.data(), sched.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
    CU_TRY(cudaMalloc(&w->d_nb_partial, partial_bytes));
    CU_TRY(cudaMalloc(&w->d_nb_counters, counter_bytes));
    CU_TRY(cudaMemset(w->d_nb_counters, 0, counter_bytes));
    w->scratch_bytes += partial_bytes + counter_bytes;
    // the many-row variant: pieces of up to NR_MAX_NB piece rows, one tensor map per B height, two hand-over slots per block
    w->nb_k_pad = img.k_pad;
    w->nr_grid = sms;
    const size_t pieces_bytes = (size_t)NR_MAX_NB * img.k_pad, nr_partial_bytes = (size_t)2 * sms * NB_TILE_N * NR_MAX_ROWS * sizeof(float);
    CU_TRY(cudaMalloc(&w->d_nr_pieces, pieces_bytes));
    CU_TRY(cudaMemset(w->d_nr_pieces, 0, pieces_bytes));
    CU_TRY(cudaMalloc(&w->d_nr_row_pow, NR_MAX_ROWS * sizeof(float)));
    CU_TRY(cudaMalloc(&w->d_nr_partial, nr_partial_bytes));
    CU_TRY(cudaMalloc(&w->d_nr_counters, counter_bytes));
    CU_TRY(cudaMemset(w->d_nr_counters, 0, counter_bytes));
    w->scratch_bytes += pieces_bytes + nr_partial_bytes + counter_bytes;
    for (int i = 0; i < 4; ++i) {
        const cuuint64_t pdims[2] = {(cuuint64_t)img.k_pad, (cuuint64_t)NR_MAX_NB};
        const cuuint64_t pstrides[1] = {(cuuint64_t)img.k_pad};
        const cuuint32_t pbox[2] = {NB_TILE_K, (cuuint32_t)(32 << i)};
        const CUresult pr = tensor_map_encoder()(&w->nr_map[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->d_nr_pieces, pdims, pstrides, pbox, estr,
                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (pr != CUDA_SUCCESS) return fail(TLLM_ERR_CUDA, "cuTensorMapEncodeTiled (activation pieces) failed with code %d", (int)pr);
    }
    CU_TRY(cudaDeviceSynchronize());
    return TLLM_OK;
}

// more rows than one launch of nibble_spmm_kernel takes: the pieces kernel and the many-row kernel, up to NR_MAX_NB piece rows per pair
int run_nr(tllm_weight* w, const void* X, int x_dtype, int x_ld, int rows, void* Y, int y_dtype, int y_ld, int epilogue, float scale, float scale2,
           cudaStream_t st) {
    const BsLayout& L = w->lay;
    static std::mutex mu;
    static bool configured[64] = {};
    {
        std::lock_guard<std::mutex> lk(mu);
        if (w->device < 64 && !configured[w->device]) {
            CU_TRY(cudaFuncSetAttribute(nibble_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            configured[w->device] = true;
        }
    }
    const int P = x_dtype == TLLM_F32 ? 8 : 4, per = NR_MAX_NB / P;
    const size_t xe = dtype_size(x_dtype), ye = dtype_size(y_dtype);
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    for (int r0 = 0; r0 < rows; r0 += per) {
        const int M = rows - r0 < per ? rows - r0 : per;
        int mi = 0;
        while ((32 << mi) < M * P) ++mi;
        const int NB = 32 << mi;
        NpParams q{};
        q.X = (const char*)X + (size_t)r0 * x_ld * xe;
        q.pieces = w->d_nr_pieces;
        q.row_pow = w->d_nr_row_pow;
        q.M = M, q.K = L.inners, q.k_pad = w->nb_k_pad, q.x_dtype = x_dtype, q.x_ld = x_ld, q.P = P;
        cudaLaunchConfig_t c1{};
        c1.gridDim = dim3((unsigned)M);
        c1.blockDim = dim3(256);
        c1.stream = st;
        c1.attrs = at;
        c1.numAttrs = 1;
        CU_TRY(cudaLaunchKernelEx(&c1, nibble_pieces_kernel, q));
        NrParams p{};
        p.row_pow = w->d_nr_row_pow;
        p.Y = (char*)Y + (size_t)r0 * y_ld * ye;
        p.partial = w->d_nr_partial;
        p.counters = w->d_nr_counters;
        p.status = w->d_status;
        p.M = M, p.N = L.columns;
        p.y_dtype = y_dtype, p.y_ld = y_ld, p.epilogue = epilogue;
        p.P = P, p.NB = NB, p.KB = w->nb_kb, p.n_tiles = w->nb_tiles;
        const size_t stage = (size_t)NR_UK * (NB_A_STAGE_BYTES + (size_t)NB * 128);
        p.S = (int)std::min<size_t>(NB_MAX_STAGES, (200 * 1024) / stage);
        p.idesc = (1u << 4) | (5u << 7) | (1u << 10) | ((uint32_t)(NB >> 3) << 17) | ((uint32_t)(NB_TILE_N >> 4) << 24);
        p.tmem_cols = (uint32_t)(2 * NB);
        p.scale = scale, p.scale2 = scale2;
        const long long units = (long long)p.n_tiles * ((p.KB + NR_UK - 1) / NR_UK);
        cudaLaunchConfig_t c2{};
        c2.gridDim = dim3((unsigned)(units < w->nr_grid ? units : w->nr_grid));
        c2.blockDim = dim3(NR_THREADS);
        c2.dynamicSmemBytes = 1024 + (size_t)p.S * stage + 1024;
        c2.stream = st;
        c2.attrs = at;
        c2.numAttrs = 1;
        CU_TRY(cudaLaunchKernelEx(&c2, nibble_rows_kernel, w->nib_map, w->nr_map[mi], p));
        g_launches.fetch_add(2, std::memory_order_relaxed);
        g_nb_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return TLLM_OK;
}

// `rows` activation rows through the decode tensor-core kernel: one launch for up to four rows (two for fp32), the many-row
// pair of kernels above that
int run_nb(tllm_weight* w, const void* X, int x_dtype, int x_ld, int rows, void* Y, int y_dtype, int y_ld, int epilogue, float scale, float scale2,
           cudaStream_t st) {
    if (rows > nb_rows_per_launch(x_dtype)) return run_nr(w, X, x_dtype, x_ld, rows, Y, y_dtype, y_ld, epilogue, scale, scale2, st);
    const BsLayout& L = w->lay;
    static std::mutex mu;
    static bool configured[64] = {};
    {
        std::lock_guard<std::mutex> lk(mu);
        if (w->device < 64 && !configured[w->device]) {
            CU_TRY(cudaFuncSetAttribute(nibble_spmm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            configured[w->device] = true;
        }
    }
    NbParams p{};
    p.partial = w->d_nb_partial;
    p.counters = w->d_nb_counters;
    p.sched = w->d_nb_sched;
    p.status = w->d_status;
    p.K = L.inners;
    p.N = L.columns;
    p.x_dtype = x_dtype;
    p.x_ld = x_ld;
    p.y_dtype = y_dtype;
    p.y_ld = y_ld;
    p.epilogue = epilogue;
    p.P = x_dtype == TLLM_F32 ? 8 : 4;
    p.KB = w->nb_kb;
    p.KBS = w->nb_kbs;
    p.k_splits = w->nb_splits;
    p.n_tiles = w->nb_tiles;
    p.Gj = w->nb_gj;
    p.S = NB_MAX_STAGES;
    // instruction descriptor: fp32 accumulate (bits 4-5 = 1), A = e2m1 (5, bits 7-9), B = e5m2 (1, bits 10-12), both
    // K-major, N / 8 in bits 17-22, M / 16 in bits 24-28
    p.idesc = (1u << 4) | (5u << 7) | (1u << 10) | ((uint32_t)(NB_ROWS >> 3) << 17) | ((uint32_t)(NB_TILE_N >> 4) << 24);
    p.tmem_cols = 32;
    p.tx_bytes = NB_A_TILE_BYTES;
#ifdef NB_DEBUG
    if (g_nb_debug_tx) p.tx_bytes = (uint32_t)g_nb_debug_tx;
    if (g_nb_debug_stages) p.S = g_nb_debug_stages;
    p.debug = g_nb_debug_flags;
#endif
    p.scale = scale;
    p.scale2 = scale2;
    const size_t smem = 1024 + (size_t)p.S * w->nb_uk * NB_A_STAGE_BYTES + (size_t)p.KBS * NB_ROWS * 128 + 512;
    const size_t xe = dtype_size(x_dtype), ye = dtype_size(y_dtype);
    const int per = nb_rows_per_launch(x_dtype);
    for (int r0 = 0; r0 < rows; r0 += per) {
        p.M = rows - r0 < per ? rows - r0 : per;
        p.X = (const char*)X + (size_t)r0 * x_ld * xe;
        p.Y = (char*)Y + (size_t)r0 * y_ld * ye;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)(p.k_splits * p.Gj));
        cfg.blockDim = dim3(NB_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        CU_TRY(cudaLaunchKernelEx(&cfg, nibble_spmm_kernel<2>, w->nib_map, p));
        g_launches.fetch_add(1, std::memory_order_relaxed);
        g_nb_launches.fetch_add(1, std::memory_order_relaxed);
    }
    return TLLM_OK;
}

enum KernelChoice { KERNEL_GATHER, KERNEL_MMA, KERNEL_NIBBLE };
KernelChoice choose_kernel(const tllm_weight* w, const void* X, int x_dtype, int x_layout, int x_ld, int rows) {
    const bool nb = nb_usable(w, x_dtype, x_layout, rows), mm = mm_usable(w, X, x_dtype, x_layout, x_ld, rows);
    if (nb && g_nb_max_rows.load(std::memory_order_relaxed) > 0) return KERNEL_NIBBLE;     // pinned
    if (mm && mm_min_rows() > 0) return KERNEL_MMA;                                         // pinned
    if (nb && mm) {
        const int64_t entries = (int64_t)w->lay.inners * w->lay.columns;
        return mm_model_us(entries, rows) < nibble_model_us(entries, rows, nb_rows_per_launch(x_dtype)) ? KERNEL_MMA : KERNEL_NIBBLE;
    }
    return nb ? KERNEL_NIBBLE : (mm ? KERNEL_MMA : KERNEL_GATHER);
}

// K-tiles whose activation tables one launch keeps in shared memory at the same time (the rest follow, one barrier-
// separated group after the other): small tables leave room for four blocks per SM
#ifndef BS_RESIDENT_MAX
#define BS_RESIDENT_MAX 2
#endif
int resident_tiles(int mp, int tiles_per_cta) {
    const int fit = BS_RESIDENT_MAX / mp > 0 ? BS_RESIDENT_MAX / mp : 1;
    return tiles_per_cta < fit ? tiles_per_cta : fit;
}

// one gather launch of at most four rows
int run_bs(tllm_weight* w, const void* X, int x_dtype, int x_layout, int x_ld, int rows, void* Y, int y_dtype, int y_ld,
           int epilogue, float scale, float scale2, const Scratch& scr, cudaStream_t st) {
    const BsLayout& L = w->lay;
    const int mp = rows <= 1 ? 1 : (rows == 2 ? 2 : 4);
    BsParams p{};
    p.stream = w->d_stream;
    p.meta = w->d_meta;
    p.X = X;
    p.Y = Y;
    p.partial = scr.partial;
    p.counters = scr.counters;
    p.status = w->d_status;
    p.x_dtype = x_dtype;
    p.x_layout = x_layout;
    p.y_dtype = y_dtype;
    p.M = rows;
    p.K = L.inners;
    p.N = L.columns;
    p.T = L.tile_rows;
    p.col_blocks = L.col_blocks;
    p.k_splits = L.k_splits;
    p.tiles_per_cta = L.tiles_per_cta;
    p.max_cols = L.max_cols_per_block;
    p.resident = resident_tiles(mp, L.tiles_per_cta);
    p.epilogue = epilogue;
    p.y_ld = y_ld;
    p.x_ld = x_ld;
    const size_t e = dtype_size(x_dtype);
    p.x_vec = x_layout == TLLM_ROW_MAJOR && ((uintptr_t)X % 16 == 0) && ((size_t)x_ld * e % 16 == 0) && (L.inners % 16 == 0) && (L.tile_rows % 16 == 0);
    p.l2_prefetch_bytes = 256u * 1024u;
    p.scale = scale;
    p.scale2 = scale2;
    const BsSmem sm = bs_smem_layout(mp, p.resident, L.tiles_per_cta, L.max_cols_per_block, w->max_meta_words, BS_STAGE_BYTES);
    p.off_table = sm.off_table, p.off_cells = sm.off_cells, p.off_meta = sm.off_meta, p.off_bars = sm.off_bars, p.off_stage = sm.off_stage;
    if (sm.total > 227u * 1024u) return fail(TLLM_ERR_ARG, "gather kernel: this weight needs %u bytes of shared memory per block", sm.total);
    p.cta_ext = w->d_cta;
    std::memcpy(p.cta, L.cta.data(), sizeof(TsCtaDesc) * (size_t)(L.num_ctas < BS_MAX_PARAM_BLOCKS ? L.num_ctas : BS_MAX_PARAM_BLOCKS));
    if (x_dtype == TLLM_I8) {
        if (mp == 1) return launch_bs<int, 1>(p, L.num_ctas, sm.total, st);
        if (mp == 2) return launch_bs<int, 2>(p, L.num_ctas, sm.total, st);
        return launch_bs<int, 4>(p, L.num_ctas, sm.total, st);
    }
    if (mp == 1) return launch_bs<float, 1>(p, L.num_ctas, sm.total, st);
    if (mp == 2) return launch_bs<float, 2>(p, L.num_ctas, sm.total, st);
    return launch_bs<float, 4>(p, L.num_ctas, sm.total, st);
}

// the gather product of any number of rows: launches of up to max_rows rows
int run_gather(tllm_weight* w, const void* X, int x_dtype, int x_layout, int x_ld, int rows, void* Y, int y_dtype, int y_ld, int epilogue,
               float scale, float scale2, const Scratch& scr, cudaStream_t st) {
    const size_t xe = dtype_size(x_dtype), ye = dtype_size(y_dtype);
    for (int r0 = 0; r0 < rows; r0 += w->max_rows) {
        const int m = rows - r0 < w->max_rows ? rows - r0 : w->max_rows;
        const char* xp = (const char*)X + (x_layout == TLLM_ROW_MAJOR ? (size_t)r0 * x_ld : (size_t)r0) * xe;
        char* yp = (char*)Y + (size_t)r0 * y_ld * ye;
        const int r = run_bs(w, xp, x_dtype, x_layout, x_ld, m, yp, y_dtype, y_ld, epilogue, scale, scale2, scr, st);
        if (r) return r;
    }
    return TLLM_OK;
}

int upload(tllm_weight* w, const BsHostImage& img, float scale, int max_rows) {
    w->lay = img.lay;
    w->scale = scale;
    w->max_rows = max_rows;
    w->max_meta_words = 0;
    for (const TsCtaDesc& d : img.lay.cta) w->max_meta_words = d.meta_words > w->max_meta_words ? d.meta_words : w->max_meta_words;
    CU_TRY(cudaGetDevice(&w->device));
    w->stream_bytes = img.stream.size();
    w->meta_bytes = img.meta.size() * sizeof(uint32_t);
    CU_TRY(cudaMalloc(&w->d_stream, w->stream_bytes + 512));
    CU_TRY(cudaMalloc(&w->d_meta, w->meta_bytes + 16));
    CU_TRY(cudaMemcpy(w->d_stream, img.stream.data(), w->stream_bytes, cudaMemcpyHostToDevice));
    CU_TRY(cudaMemcpy(w->d_meta, img.meta.data(), w->meta_bytes, cudaMemcpyHostToDevice));
    CU_TRY(cudaMalloc(&w->d_cta, img.lay.cta.size() * sizeof(TsCtaDesc)));
    CU_TRY(cudaMemcpy(w->d_cta, img.lay.cta.data(), img.lay.cta.size() * sizeof(TsCtaDesc), cudaMemcpyHostToDevice));
    const size_t partial_bytes = img.lay.k_splits > 1 ? (size_t)img.lay.k_splits * max_rows * img.lay.columns * 4 : 16;
    const size_t counter_bytes = (size_t)img.lay.col_blocks * sizeof(unsigned int);
    w->scratch_bytes = partial_bytes + counter_bytes + sizeof(int);
    CU_TRY(cudaMalloc(&w->d_partial, partial_bytes));
    CU_TRY(cudaMalloc(&w->d_counters, counter_bytes));
    CU_TRY(cudaMalloc(&w->d_status, sizeof(int)));
    CU_TRY(cudaMemset(w->d_counters, 0, counter_bytes));
    CU_TRY(cudaMemset(w->d_status, 0, sizeof(int)));
    CU_TRY(cudaDeviceSynchronize());
    return TLLM_OK;
}

int upload_bit_tiles(tllm_weight* w, const std::vector<uint32_t>& bits, int sms) {
    w->bits_bytes = bits.size() * sizeof(uint32_t);
    w->mm_grid = sms;
    CU_TRY(cudaMalloc(&w->d_bits, w->bits_bytes));
    CU_TRY(cudaMemcpy(w->d_bits, bits.data(), w->bits_bytes, cudaMemcpyHostToDevice));
    const size_t partial_bytes = (size_t)2 * sms * MM_TILE_N * MM_SPLIT_MAX_NT * sizeof(float);
    const size_t counter_bytes = (size_t)w->mm_n_tiles * 4 * sizeof(unsigned int);
    CU_TRY(cudaMalloc(&w->d_mm_partial, partial_bytes));
    CU_TRY(cudaMalloc(&w->d_mm_counters, counter_bytes));
    CU_TRY(cudaMemset(w->d_mm_counters, 0, counter_bytes));
    w->scratch_bytes += partial_bytes + counter_bytes;
    CU_TRY(cudaDeviceSynchronize());
    return TLLM_OK;
}

int upload_bits(tllm_weight* w, const int8_t* dense, int inners, int columns, int sms) {
    std::vector<uint32_t> bits;
    mm_pack_bits(dense, inners, columns, &bits, &w->mm_n_tiles, &w->mm_kb);
    return upload_bit_tiles(w, bits, sms);
}

int device_sms(int* sms) {
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    CU_TRY(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    int max_smem = 0;
    CU_TRY(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    if (max_smem < 227 * 1024)
        return fail(TLLM_ERR_ARG, "this device offers %d bytes of shared memory per block; the kernels need 232448 (built for sm_100a)", max_smem);
    return TLLM_OK;
}

int create_from_dense(const int8_t* dense, int inners, int columns, float scale, const tllm_pack_opts* opts, tllm_weight** out) {
    if (!out) return fail(TLLM_ERR_ARG, "weight create: out is NULL");
    *out = nullptr;
    int sms = 0;
    int rc = device_sms(&sms);
    if (rc) return rc;
    BsHostImage img;
    const char* msg = bs_pack_dense(dense, inners, columns, opts, sms, &img);
    if (msg) return fail(TLLM_ERR_ARG, "%s", msg);
    int max_rows = (opts && opts->max_rows > 0) ? opts->max_rows : 4;
    if (max_rows > 4) max_rows = 4;
    tllm_weight* w = new tllm_weight();
    rc = upload(w, img, scale, max_rows);
    if (rc == TLLM_OK && !(opts && opts->no_bit_tiles)) rc = upload_bits(w, dense, inners, columns, sms);
    if (rc == TLLM_OK && !(opts && opts->no_nibbles)) rc = upload_nibbles(w, dense, inners, columns, sms);
    if (rc != TLLM_OK) {
        tllm_weight_destroy(w);
        return rc;
    }
    *out = w;
    return TLLM_OK;
}

int ensure(void** p, size_t* cap, size_t need, bool pinned) {
    if (*cap >= need) return TLLM_OK;
    if (*p) {
        if (pinned) CU_TRY(cudaFreeHost(*p));
        else CU_TRY(cudaFree(*p));
        *p = nullptr;
        *cap = 0;
    }
    size_t n = need < 4096 ? 4096 : need;
    if (pinned) CU_TRY(cudaMallocHost(p, n));
    else CU_TRY(cudaMalloc(p, n));
    *cap = n;
    return TLLM_OK;
}

// Y[rows][columns] (row-major, on the device) += bias[columns], both of y_dtype
int add_bias(void* Y, const void* bias, int y_dtype, int rows, int columns, cudaStream_t st) {
    const long long n = (long long)rows * columns;
    bias_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(Y, bias, y_dtype, n, columns);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TLLM_OK;
}

}  // namespace

namespace tllm {
void bs_fill_info(const BsLayout& L, tllm_weight_info* info) {
    info->inners = L.inners;
    info->columns = L.columns;
    info->tile_rows = L.tile_rows;
    info->tiles = L.tiles;
    info->col_blocks = L.col_blocks;
    info->k_splits = L.k_splits;
    info->tiles_per_cta = L.tiles_per_cta;
    info->num_ctas = L.num_ctas;
    info->units = (int)L.units;
    info->nnz = L.nnz;
    info->algorithmic_bytes = 2 * L.nnz + 16 * (int64_t)L.columns * ((L.inners + 511) / 512);
}
}  // namespace tllm

#ifdef BS_TRACE
extern "C" int tllm_debug_set_trace(void* device_buffer) {
    CU_TRY(cudaMemcpyToSymbol(tllm::g_bs_trace, &device_buffer, sizeof(void*)));
    return TLLM_OK;
}
#endif

extern "C" {

const char* tllm_last_error(void) { return g_err.c_str(); }
int tllm_version(void) { return 200; }
int64_t tllm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
int64_t tllm_mma_launch_count(void) { return g_mm_launches.load(std::memory_order_relaxed); }
int tllm_set_mma_min_rows(int rows) {
    const int prev = mm_min_rows();
    g_mm_min_rows.store(rows < 0 ? -1 : rows, std::memory_order_relaxed);
    return prev;
}

// ---- packed copies of the reference's device arrays, keyed by the arrays' addresses and the shape --------------------
namespace {
struct TerCacheEntry {
    const void* row_idx;
    const void* col_off;
    int columns, inners, tile_k, device;
    tllm_weight* w;
};
std::mutex g_ter_mu;
std::vector<TerCacheEntry> g_ter_cache;

tllm_weight* ter_cache_find(const void* row_idx, const void* col_off, int columns, int inners, int tile_k) {
    std::lock_guard<std::mutex> lk(g_ter_mu);
    if (g_ter_cache.empty()) return nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    for (const TerCacheEntry& e : g_ter_cache)
        if (e.row_idx == row_idx && e.col_off == col_off && e.columns == columns && e.inners == inners && e.tile_k == tile_k && e.device == dev) return e.w;
    return nullptr;
}
}  // namespace

int tllm_ter_spmm_prepare(const int16_t* row_idx, const int32_t* col_off, int columns, int inners, int tile_k) {
    if (!row_idx || !col_off || columns <= 0 || inners <= 0 || tile_k <= 0) return fail(TLLM_ERR_ARG, "tllm_ter_spmm_prepare: bad argument");
    if (ter_cache_find(row_idx, col_off, columns, inners, tile_k)) return TLLM_OK;
    // the row-index array's length is the largest list end
    const size_t n_off = (size_t)columns * ((size_t)(inners + tile_k - 1) / tile_k) * 4;
    std::vector<int32_t> off(n_off);
    CU_TRY(cudaMemcpy(off.data(), col_off, n_off * sizeof(int32_t), cudaMemcpyDeviceToHost));
    int64_t len = 0;
    for (size_t i = 0; i < n_off; i += 4) len = std::max<int64_t>(len, off[i + 2]);
    tllm_weight* w = nullptr;
    const int rc = tllm_weight_create_mcsc_device(row_idx, len, col_off, columns, inners, tile_k, 1.0f, nullptr, &w);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(g_ter_mu);
    g_ter_cache.push_back(TerCacheEntry{row_idx, col_off, columns, inners, tile_k, w->device, w});
    return TLLM_OK;
}

int tllm_ter_spmm_forget(const int16_t* row_idx, const int32_t* col_off) {
    std::vector<tllm_weight*> dead;
    {
        std::lock_guard<std::mutex> lk(g_ter_mu);
        for (size_t i = 0; i < g_ter_cache.size();) {
            if ((!row_idx && !col_off) || (g_ter_cache[i].row_idx == row_idx && g_ter_cache[i].col_off == col_off)) {
                dead.push_back(g_ter_cache[i].w);
                g_ter_cache.erase(g_ter_cache.begin() + (long)i);
            } else ++i;
        }
    }
    for (tllm_weight* w : dead) tllm_weight_destroy(w);
    return (int)dead.size();
}

int tllm_set_nibble_max_rows(int rows) {
    return g_nb_max_rows.exchange(rows < 0 ? -1 : rows, std::memory_order_relaxed);
}

#ifdef NB_DEBUG
int tllm_debug_set_nb_tx(int bytes) {
    g_nb_debug_tx = bytes;
    return 0;
}
int tllm_debug_set_nb_flags(int flags) {
    g_nb_debug_flags = flags;
    return 0;
}
int tllm_debug_set_nb_stages(int stages) {
    g_nb_debug_stages = stages;
    return 0;
}
int tllm_debug_set_nb_trace(void* device_buffer) {
    CU_TRY(cudaMemcpyToSymbol(tllm::g_nb_trace, &device_buffer, sizeof(void*)));
    return TLLM_OK;
}
#endif
int64_t tllm_nibble_launch_count(void) { return g_nb_launches.load(std::memory_order_relaxed); }

int tllm_ter_spmm(const void* X, int x_dtype, int x_layout, const int16_t* row_idx, const int32_t* col_off,
                  const int16_t* col_tile_idx, void* Y, int y_dtype, int batch, int rows, int columns,
                  int inners, int tile_k, float scale, int uniformed, int padded, void* stream) {
    (void)col_tile_idx;
    (void)uniformed;
    (void)padded;
    if (batch == 0) return TLLM_OK;   // the reference launches nothing for a 2-D input (TernaryLinear.py:168)
    if (!X || !row_idx || !col_off || !Y) return fail(TLLM_ERR_ARG, "tllm_ter_spmm: NULL pointer");
    if (batch < 0 || rows <= 0 || columns <= 0 || inners <= 0 || tile_k <= 0) return fail(TLLM_ERR_ARG, "tllm_ter_spmm: bad shape");
    const int rc = check_types(x_dtype, y_dtype, "tllm_ter_spmm");
    if (rc) return rc;
    if (batch > 65535) return fail(TLLM_ERR_ARG, "tllm_ter_spmm: batch too large");
    if (tllm_weight* w = ter_cache_find(row_idx, col_off, columns, inners, tile_k)) {
        // these arrays were repacked by tllm_ter_spmm_prepare: the product runs on the packed copy
        const BsLayout& L = w->lay;
        cudaStream_t st = (cudaStream_t)stream;
        const size_t xe = dtype_size(x_dtype), ye = dtype_size(y_dtype);
        if (x_layout == TLLM_ROW_MAJOR) {
            const long long m = (long long)batch * rows;      // the batch is contiguous: one product of batch * rows rows
            if (m > 0x7fffffffLL) return fail(TLLM_ERR_ARG, "tllm_ter_spmm: batch * rows too large");
            const KernelChoice kc = choose_kernel(w, X, x_dtype, x_layout, inners, (int)m);
            if (kc == KERNEL_NIBBLE) return run_nb(w, X, x_dtype, inners, (int)m, Y, y_dtype, columns, 0, scale, 0.f, st);
            if (kc == KERNEL_MMA) return run_mm(w, X, x_dtype, inners, (int)m, Y, y_dtype, columns, 0, scale, 0.f, st);
            return run_gather(w, X, x_dtype, x_layout, inners, (int)m, Y, y_dtype, columns, 0, scale, 0.f, Scratch{w->d_partial, w->d_counters}, st);
        }
        for (int b = 0; b < batch; ++b) {
            const int rc2 = run_gather(w, (const char*)X + (size_t)b * rows * inners * xe, x_dtype, x_layout, rows, rows,
                                       (char*)Y + (size_t)b * rows * columns * ye, y_dtype, columns, 0, scale, 0.f, Scratch{w->d_partial, w->d_counters}, st);
            if (rc2) return rc2;
        }
        (void)L;
        return TLLM_OK;
    }
    constexpr int MC = 4;
    dim3 grid((columns + 7) / 8, (rows + MC - 1) / MC, batch), block(256);
    if (grid.y > 65535) return fail(TLLM_ERR_ARG, "tllm_ter_spmm: too many rows for one call");
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == TLLM_I8)
        mcsc_spmm_kernel<int, MC><<<grid, block, 0, st>>>(X, x_dtype, x_layout, row_idx, col_off, Y, y_dtype, rows, columns, inners, tile_k, scale);
    else
        mcsc_spmm_kernel<float, MC><<<grid, block, 0, st>>>(X, x_dtype, x_layout, row_idx, col_off, Y, y_dtype, rows, columns, inners, tile_k, scale);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TLLM_OK;
}

int tllm_weight_create_dense(const int8_t* w, int inners, int columns, float scale, const tllm_pack_opts* opts, tllm_weight** out) {
    if (!w || inners <= 0 || columns <= 0) return fail(TLLM_ERR_ARG, "tllm_weight_create_dense: bad argument");
    const size_t n = (size_t)inners * columns;
    for (size_t i = 0; i < n; ++i)
        if (w[i] < -1 || w[i] > 1) return fail(TLLM_ERR_ARG, "tllm_weight_create_dense: entry %zu is %d, not ternary", i, (int)w[i]);
    return create_from_dense(w, inners, columns, scale, opts, out);
}

int tllm_weight_create_mcsc(const int32_t* row_idx, const int32_t* col_off, int columns, int inners, int tile_k, float scale,
                            const tllm_pack_opts* opts, tllm_weight** out) {
    if (!row_idx || !col_off || columns <= 0 || inners <= 0 || tile_k <= 0) return fail(TLLM_ERR_ARG, "tllm_weight_create_mcsc: bad argument");
    std::vector<int8_t> dense;
    const char* msg = decode_mcsc(row_idx, col_off, columns, inners, tile_k, &dense);
    if (msg) return fail(TLLM_ERR_ARG, "%s", msg);
    return create_from_dense(dense.data(), inners, columns, scale, opts, out);
}

int tllm_weight_create_ssr(const uint8_t* image, size_t bytes, int inners, int columns, float scale, const tllm_pack_opts* opts, tllm_weight** out) {
    if (!image || inners <= 0 || columns <= 0) return fail(TLLM_ERR_ARG, "tllm_weight_create_ssr: bad argument");
    std::vector<int8_t> dense((size_t)inners * (size_t)columns);
    const int rc = tllm_ssr_decode(image, bytes, inners, columns, dense.data());      // validates the whole image first
    if (rc != TLLM_OK) return rc;
    return create_from_dense(dense.data(), inners, columns, scale, opts, out);
}

int tllm_weight_create_mcsc_device(const int16_t* row_idx, int64_t row_idx_len, const int32_t* col_off, int columns, int inners, int tile_k,
                                   float scale, const tllm_pack_opts* opts, tllm_weight** out) {
    if (!row_idx || !col_off || columns <= 0 || inners <= 0 || tile_k <= 0 || row_idx_len < 0)
        return fail(TLLM_ERR_ARG, "tllm_weight_create_mcsc_device: bad argument");
    const size_t n_off = (size_t)columns * ((size_t)(inners + tile_k - 1) / tile_k) * 4;
    std::vector<int16_t> ri16((size_t)row_idx_len);
    std::vector<int32_t> off(n_off);
    if (row_idx_len) CU_TRY(cudaMemcpy(ri16.data(), row_idx, ri16.size() * sizeof(int16_t), cudaMemcpyDeviceToHost));
    CU_TRY(cudaMemcpy(off.data(), col_off, off.size() * sizeof(int32_t), cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < n_off; i += 4)
        if (off[i] < 0 || off[i + 1] < off[i] || off[i + 2] < off[i + 1] || off[i + 2] > row_idx_len)
            return fail(TLLM_ERR_ARG, "tllm_weight_create_mcsc_device: list offsets of entry %zu leave the row-index array", i / 4);
    std::vector<int32_t> ri(ri16.begin(), ri16.end());
    return tllm_weight_create_mcsc(ri.data(), off.data(), columns, inners, tile_k, scale, opts, out);
}

int tllm_weight_create_cpu_format(int kind, int group, int chunk, const int32_t* meta, const void* ri, int ri32, int64_t aux,
                                  int columns, int inners, float scale, const tllm_pack_opts* opts, tllm_weight** out) {
    if (!meta || !ri || columns <= 0 || inners <= 0) return fail(TLLM_ERR_ARG, "tllm_weight_create_cpu_format: bad argument");
    std::vector<int8_t> dense;
    const char* msg = decode_cpu_format(kind, group, chunk, meta, ri, ri32, aux, columns, inners, &dense);
    if (msg) return fail(TLLM_ERR_ARG, "%s", msg);
    return create_from_dense(dense.data(), inners, columns, scale, opts, out);
}

int tllm_weight_destroy(tllm_weight* w) {
    if (!w) return TLLM_OK;
    cudaFree(w->d_stream);
    cudaFree(w->d_meta);
    cudaFree(w->d_cta);
    cudaFree(w->d_bits);
    cudaFree(w->d_mm_partial);
    cudaFree(w->d_mm_counters);
    cudaFree(w->d_nib);
    cudaFree(w->d_nb_partial);
    cudaFree(w->d_nb_counters);
    cudaFree(w->d_nb_sched);
    cudaFree(w->d_nr_pieces);
    cudaFree(w->d_nr_row_pow);
    cudaFree(w->d_nr_partial);
    cudaFree(w->d_nr_counters);
    cudaFree(w->d_partial);
    cudaFree(w->d_counters);
    cudaFree(w->d_status);
    cudaFree(w->d_x);
    cudaFree(w->d_y);
    cudaFree(w->d_bias);
    if (w->h_pin) cudaFreeHost(w->h_pin);
    if (w->h_status) cudaFreeHost(w->h_status);
    if (w->own_stream) cudaStreamDestroy(w->own_stream);
    delete w;
    return TLLM_OK;
}

int tllm_weight_get_info(const tllm_weight* w, tllm_weight_info* info) {
    if (!w || !info) return fail(TLLM_ERR_ARG, "tllm_weight_get_info: NULL");
    std::memset(info, 0, sizeof *info);
    bs_fill_info(w->lay, info);
    info->max_rows = w->max_rows;
    info->stream_bytes = (int64_t)w->stream_bytes;
    info->meta_bytes = (int64_t)w->meta_bytes;
    info->scratch_bytes = (int64_t)w->scratch_bytes;
    info->bit_tile_bytes = (int64_t)w->bits_bytes;
    info->nibble_bytes = (int64_t)w->nib_bytes;
    info->scale = w->scale;
    return TLLM_OK;
}

// ---- packed-weight files: header, column ranges, block descriptors, index stream, block tables, bit tiles ----------
namespace {
struct WeightFileHeader {
    char magic[8];                // "TLLMW002"
    int32_t inners, columns, tile_rows, tiles, col_blocks, k_splits, tiles_per_cta, num_ctas, max_cols_per_block, max_rows, mm_n_tiles, mm_kb;
    int64_t nnz, total_vecs, units, meta_words, bits_words;
    float scale;
    int32_t reserved[7];
};
bool read_exact(FILE* f, void* p, size_t n) { return n == 0 || fread(p, 1, n, f) == n; }
bool write_exact(FILE* f, const void* p, size_t n) { return n == 0 || fwrite(p, 1, n, f) == n; }
}  // namespace

int tllm_weight_save(const tllm_weight* w, const char* path) {
    if (!w || !path) return fail(TLLM_ERR_ARG, "tllm_weight_save: NULL argument");
    const BsLayout& L = w->lay;
    WeightFileHeader h{};
    std::memcpy(h.magic, "TLLMW002", 8);
    h.inners = L.inners, h.columns = L.columns, h.tile_rows = L.tile_rows, h.tiles = L.tiles, h.col_blocks = L.col_blocks;
    h.k_splits = L.k_splits, h.tiles_per_cta = L.tiles_per_cta, h.num_ctas = L.num_ctas, h.max_cols_per_block = L.max_cols_per_block;
    h.max_rows = w->max_rows, h.mm_n_tiles = w->mm_n_tiles, h.mm_kb = w->mm_kb;
    h.nnz = L.nnz, h.total_vecs = L.total_vecs, h.units = L.units;
    h.meta_words = (int64_t)(w->meta_bytes / sizeof(uint32_t));
    h.bits_words = (int64_t)(w->bits_bytes / sizeof(uint32_t));
    h.scale = w->scale;
    std::vector<unsigned char> stream(w->stream_bytes), meta(w->meta_bytes), bits(w->bits_bytes);
    int prev = 0;
    CU_TRY(cudaGetDevice(&prev));
    CU_TRY(cudaSetDevice(w->device));
    CU_TRY(cudaMemcpy(stream.data(), w->d_stream, w->stream_bytes, cudaMemcpyDeviceToHost));
    CU_TRY(cudaMemcpy(meta.data(), w->d_meta, w->meta_bytes, cudaMemcpyDeviceToHost));
    if (w->bits_bytes) CU_TRY(cudaMemcpy(bits.data(), w->d_bits, w->bits_bytes, cudaMemcpyDeviceToHost));
    CU_TRY(cudaSetDevice(prev));
    FILE* f = fopen(path, "wb");
    if (!f) return fail(TLLM_ERR_ARG, "tllm_weight_save: cannot open %s for writing", path);
    const bool ok = write_exact(f, &h, sizeof h) && write_exact(f, L.col_start.data(), L.col_start.size() * sizeof(int32_t)) &&
                    write_exact(f, L.cta.data(), L.cta.size() * sizeof(TsCtaDesc)) && write_exact(f, stream.data(), stream.size()) &&
                    write_exact(f, meta.data(), meta.size()) && write_exact(f, bits.data(), bits.size());
    if (fclose(f) != 0 || !ok) return fail(TLLM_ERR_ARG, "tllm_weight_save: short write to %s", path);
    return TLLM_OK;
}

int tllm_weight_load(const char* path, tllm_weight** out) {
    if (!path || !out) return fail(TLLM_ERR_ARG, "tllm_weight_load: NULL argument");
    *out = nullptr;
    FILE* f = fopen(path, "rb");
    if (!f) return fail(TLLM_ERR_ARG, "tllm_weight_load: cannot open %s", path);
    WeightFileHeader h{};
    BsHostImage img;
    std::vector<uint32_t> bits;
    bool ok = read_exact(f, &h, sizeof h) && std::memcmp(h.magic, "TLLMW002", 8) == 0;
    ok = ok && h.num_ctas > 0 && h.num_ctas <= BS_MAX_BLOCKS && h.col_blocks > 0 && h.col_blocks <= h.num_ctas && h.total_vecs >= 0 && h.meta_words >= 0 &&
         h.bits_words >= 0 && h.total_vecs < ((int64_t)1 << 32) && h.meta_words < ((int64_t)1 << 34) && h.bits_words < ((int64_t)1 << 38);
    if (ok) {
        BsLayout& L = img.lay;
        L.inners = h.inners, L.columns = h.columns, L.tile_rows = h.tile_rows, L.tiles = h.tiles, L.col_blocks = h.col_blocks;
        L.k_splits = h.k_splits, L.tiles_per_cta = h.tiles_per_cta, L.num_ctas = h.num_ctas, L.max_cols_per_block = h.max_cols_per_block;
        L.nnz = h.nnz, L.total_vecs = h.total_vecs, L.units = h.units;
        L.col_start.resize((size_t)h.col_blocks + 1);
        L.cta.resize((size_t)h.num_ctas);
        img.stream.resize((size_t)h.total_vecs * 16);
        img.meta.resize((size_t)h.meta_words);
        bits.resize((size_t)h.bits_words);
        ok = read_exact(f, L.col_start.data(), L.col_start.size() * sizeof(int32_t)) && read_exact(f, L.cta.data(), L.cta.size() * sizeof(TsCtaDesc)) &&
             read_exact(f, img.stream.data(), img.stream.size()) && read_exact(f, img.meta.data(), img.meta.size() * sizeof(uint32_t)) &&
             read_exact(f, bits.data(), bits.size() * sizeof(uint32_t));
    }
    fclose(f);
    if (!ok) return fail(TLLM_ERR_ARG, "tllm_weight_load: %s is not a packed-weight file of this library (or is truncated)", path);
    if (const char* msg = bs_validate(img)) return fail(TLLM_ERR_ARG, "tllm_weight_load: %s", msg);
    const int64_t want_bits = (int64_t)((h.columns + 127) / 128) * ((h.inners + 63) / 64) * 128 * 4;
    if (h.bits_words != 0 && (h.bits_words != want_bits || h.mm_n_tiles != (h.columns + 127) / 128 || h.mm_kb != (h.inners + 63) / 64))
        return fail(TLLM_ERR_ARG, "tllm_weight_load: bit tiles of %s do not match the matrix shape", path);
    int sms = 0;
    int rc = device_sms(&sms);
    if (rc) return rc;
    tllm_weight* w = new tllm_weight();
    rc = upload(w, img, h.scale, h.max_rows > 0 && h.max_rows <= 4 ? h.max_rows : 4);
    if (rc == TLLM_OK && h.bits_words) {
        w->mm_n_tiles = h.mm_n_tiles;
        w->mm_kb = h.mm_kb;
        rc = upload_bit_tiles(w, bits, sms);
    }
    if (rc == TLLM_OK) {   // the four-bit planes are not stored: they are rebuilt from the lists
        std::vector<int8_t> dense((size_t)h.inners * h.columns);
        bs_unpack_dense(img, dense.data());
        rc = upload_nibbles(w, dense.data(), h.inners, h.columns, sms);
    }
    if (rc != TLLM_OK) {
        tllm_weight_destroy(w);
        return rc;
    }
    *out = w;
    return TLLM_OK;
}

int tllm_weight_set_scale(tllm_weight* w, float scale) {
    if (!w) return fail(TLLM_ERR_ARG, "tllm_weight_set_scale: NULL");
    w->scale = scale;
    return TLLM_OK;
}

int tllm_weight_check(tllm_weight* w) {
    if (!w) return fail(TLLM_ERR_ARG, "tllm_weight_check: NULL");
    int st = 0;
    CU_TRY(cudaMemcpy(&st, w->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        cudaMemset(w->d_status, 0, sizeof(int));
        cudaMemset(w->d_counters, 0, (size_t)w->lay.col_blocks * sizeof(unsigned int));
        if (w->d_mm_counters) cudaMemset(w->d_mm_counters, 0, (size_t)w->mm_n_tiles * 4 * sizeof(unsigned int));
        if (w->d_nb_counters) cudaMemset(w->d_nb_counters, 0, (size_t)w->nb_tiles * 4 * sizeof(unsigned int));
        if (w->d_nr_counters) cudaMemset(w->d_nr_counters, 0, (size_t)w->nb_tiles * 4 * sizeof(unsigned int));
        return fail(TLLM_ERR_KERNEL, "a bounded wait ran out inside the kernel (code %d: %s)", st,
                    st == MM_ERR_WAIT ? "tensor-core pipeline stalled" : (st == NB_ERR_WAIT ? "decode tensor-core pipeline stalled" : "block table never arrived"));
    }
    return TLLM_OK;
}

int tllm_spmm(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, void* Y, int y_dtype, void* stream) {
    if (!w || !X || !Y) return fail(TLLM_ERR_ARG, "tllm_spmm: NULL pointer");
    if (rows <= 0) return fail(TLLM_ERR_ARG, "tllm_spmm: rows must be positive");
    if (x_layout != TLLM_ROW_MAJOR && x_layout != TLLM_COL_MAJOR) return fail(TLLM_ERR_ARG, "tllm_spmm: bad x_layout");
    int rc = check_types(x_dtype, y_dtype, "tllm_spmm");
    if (rc) return rc;
    rc = check_device(w, "tllm_spmm");
    if (rc) return rc;
    const BsLayout& L = w->lay;
    const int x_ld = x_layout == TLLM_ROW_MAJOR ? L.inners : rows;
    const KernelChoice kc = choose_kernel(w, X, x_dtype, x_layout, x_ld, rows);
    if (kc == KERNEL_NIBBLE) return run_nb(w, X, x_dtype, x_ld, rows, Y, y_dtype, L.columns, 0, w->scale, 0.f, (cudaStream_t)stream);
    if (kc == KERNEL_MMA) return run_mm(w, X, x_dtype, x_ld, rows, Y, y_dtype, L.columns, 0, w->scale, 0.f, (cudaStream_t)stream);
    return run_gather(w, X, x_dtype, x_layout, x_ld, rows, Y, y_dtype, L.columns, 0, w->scale, 0.f, Scratch{w->d_partial, w->d_counters},
                      (cudaStream_t)stream);
}

int tllm_spmm_host_bias(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, const void* bias, void* Y, int y_dtype, int y_layout) {
    if (!w || !X || !Y) return fail(TLLM_ERR_ARG, "tllm_spmm_host: NULL pointer");
    if (rows <= 0) return fail(TLLM_ERR_ARG, "tllm_spmm_host: rows must be positive");
    int rc = check_types(x_dtype, y_dtype, "tllm_spmm_host");
    if (rc) return rc;
    rc = check_device(w, "tllm_spmm_host");
    if (rc) return rc;
    const BsLayout& L = w->lay;
    const size_t xb = (size_t)rows * L.inners * dtype_size(x_dtype), yb = (size_t)rows * L.columns * dtype_size(y_dtype);
    if (!w->own_stream) CU_TRY(cudaStreamCreateWithFlags(&w->own_stream, cudaStreamNonBlocking));
    if (!w->h_status) CU_TRY(cudaMallocHost((void**)&w->h_status, sizeof(int)));
    int r = ensure(&w->d_x, &w->x_cap, xb, false);
    if (r) return r;
    r = ensure(&w->d_y, &w->y_cap, yb, false);
    if (r) return r;
    CU_TRY(cudaMemcpyAsync(w->d_x, X, xb, cudaMemcpyHostToDevice, w->own_stream));
    if (bias) {
        r = ensure(&w->d_bias, &w->bias_cap, (size_t)L.columns * dtype_size(y_dtype), false);
        if (r) return r;
        CU_TRY(cudaMemcpyAsync(w->d_bias, bias, (size_t)L.columns * dtype_size(y_dtype), cudaMemcpyHostToDevice, w->own_stream));
    }
    r = tllm_spmm(w, w->d_x, x_dtype, x_layout, rows, w->d_y, y_dtype, w->own_stream);
    if (r) return r;
    if (bias) {
        r = add_bias(w->d_y, w->d_bias, y_dtype, rows, L.columns, w->own_stream);
        if (r) return r;
    }
    if (y_layout == TLLM_ROW_MAJOR) {
        CU_TRY(cudaMemcpyAsync(Y, w->d_y, yb, cudaMemcpyDeviceToHost, w->own_stream));
        CU_TRY(cudaMemcpyAsync(w->h_status, w->d_status, sizeof(int), cudaMemcpyDeviceToHost, w->own_stream));
        CU_TRY(cudaStreamSynchronize(w->own_stream));
    } else {
        r = ensure(&w->h_pin, &w->pin_cap, yb, true);
        if (r) return r;
        CU_TRY(cudaMemcpyAsync(w->h_pin, w->d_y, yb, cudaMemcpyDeviceToHost, w->own_stream));
        CU_TRY(cudaMemcpyAsync(w->h_status, w->d_status, sizeof(int), cudaMemcpyDeviceToHost, w->own_stream));
        CU_TRY(cudaStreamSynchronize(w->own_stream));
        const size_t e = dtype_size(y_dtype);
        const char* src = (const char*)w->h_pin;
        char* dst = (char*)Y;
        for (int m = 0; m < rows; ++m)
            for (int n = 0; n < L.columns; ++n) std::memcpy(dst + ((size_t)n * rows + m) * e, src + ((size_t)m * L.columns + n) * e, e);
    }
    // the status word came back with the result; only a non-zero one needs the (synchronising) full check
    return *w->h_status ? tllm_weight_check(w) : TLLM_OK;
}

int tllm_spmm_host(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, void* Y, int y_dtype, int y_layout) {
    return tllm_spmm_host_bias(w, X, x_dtype, x_layout, rows, nullptr, Y, y_dtype, y_layout);
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------------
// tllm_spmm_static_scratch: the same product as tllm_spmm, for callers that must not allocate.
//
// Some callers run where device allocation is off the table: a serving loop whose memory pool was carved up
// at start-up and is policed for late cudaMalloc calls, code that executes under a framework allocator it
// must not bypass, or a latency-critical path where an allocation (which may synchronise the device) is not
// acceptable.  tllm_spmm itself allocates nothing either, but the handle it uses had its split-K scratch
// allocated with cudaMalloc when it was created.  This entry point does not use that scratch: partial sums
// and arrival counters live in the fixed array below, which every GPU that loads this library carries until
// the process exits.  Its size is the limit on what one call may ask for.  (The 4-byte status word stays the
// handle's own -- it exists since the handle was created -- so that tllm_weight_check reports a kernel that
// gave up on a wait on this path as on every other.)
// ------------------------------------------------------------------------------------------------------
#define TLLM_STATIC_SCRATCH_CELLS (1u << 20)   // 4-byte partial sums: k_splits * rows_per_launch * columns must fit
#define TLLM_STATIC_COUNTERS 4096u
#define TLLM_STATIC_SCRATCH_BYTES (TLLM_STATIC_SCRATCH_CELLS * 4u + TLLM_STATIC_COUNTERS * 4u)

static __device__ __align__(256) unsigned char g_static_scratch[TLLM_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void* g_static_ptr[64] = {};   // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel could use: the
// device address has to be asked for, once per device, with that device current.
int static_scratch_address(void** out) {
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TLLM_ERR_ARG, "tllm_spmm_static_scratch: device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* ptr = nullptr;
        CU_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) return fail(TLLM_ERR_CUDA, "tllm_spmm_static_scratch: cudaGetSymbolAddress returned a null address");
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return TLLM_OK;
}
}  // namespace

extern "C" int tllm_spmm_static_scratch(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, void* Y, int y_dtype,
                                        void* stream) {
    if (!w || !X || !Y) return fail(TLLM_ERR_ARG, "tllm_spmm_static_scratch: NULL pointer");
    if (rows <= 0) return fail(TLLM_ERR_ARG, "tllm_spmm_static_scratch: rows must be positive");
    if (x_layout != TLLM_ROW_MAJOR && x_layout != TLLM_COL_MAJOR) return fail(TLLM_ERR_ARG, "tllm_spmm_static_scratch: bad x_layout");
    int rc = check_types(x_dtype, y_dtype, "tllm_spmm_static_scratch");
    if (rc) return rc;
    rc = check_device(w, "tllm_spmm_static_scratch");
    if (rc) return rc;
    const BsLayout& L = w->lay;
    const int per_launch = rows < w->max_rows ? rows : w->max_rows;
    const uint64_t cells = L.k_splits > 1 ? (uint64_t)L.k_splits * (uint64_t)per_launch * (uint64_t)L.columns : 0;
    if (cells > TLLM_STATIC_SCRATCH_CELLS)
        return fail(TLLM_ERR_ARG,
                    "tllm_spmm_static_scratch: %d K-splits x %d rows x %d columns = %llu partial sums exceed the built-in scratch of %u; "
                    "use tllm_spmm, fewer rows per call, or a weight packed with fewer K-splits",
                    L.k_splits, per_launch, L.columns, (unsigned long long)cells, (unsigned)TLLM_STATIC_SCRATCH_CELLS);
    if ((unsigned)L.col_blocks > TLLM_STATIC_COUNTERS) return fail(TLLM_ERR_ARG, "tllm_spmm_static_scratch: too many column blocks for the built-in counters");
    void* base = nullptr;
    rc = static_scratch_address(&base);
    if (rc) return rc;
    unsigned char* scratch = (unsigned char*)base;
    unsigned int* counters = (unsigned int*)(scratch + (size_t)TLLM_STATIC_SCRATCH_CELLS * 4u);
    cudaStream_t st = (cudaStream_t)stream;
    // The array keeps whatever the previous call left.  Partial sums are overwritten before they are read;
    // the counters must start at zero, so they are cleared here, in stream order.
    CU_TRY(cudaMemsetAsync(counters, 0, (size_t)TLLM_STATIC_COUNTERS * 4u, st));
    const int x_ld = x_layout == TLLM_ROW_MAJOR ? L.inners : rows;
    return run_gather(w, X, x_dtype, x_layout, x_ld, rows, Y, y_dtype, L.columns, 0, w->scale, 0.f, Scratch{scratch, counters}, st);
}

extern "C" {

int tllm_mlp_create(const int8_t* w_gate, const int8_t* w_up, const int8_t* w_down, int hidden, int intermediate, float s_gate,
                    float s_up, float s_down, const tllm_pack_opts* opts, tllm_mlp** out) {
    if (!w_gate || !w_up || !w_down || hidden <= 0 || intermediate <= 0 || !out) return fail(TLLM_ERR_ARG, "tllm_mlp_create: bad argument");
    *out = nullptr;
    std::vector<int8_t> gu((size_t)hidden * 2 * intermediate);
    for (int k = 0; k < hidden; ++k) {
        const int8_t* g = w_gate + (size_t)k * intermediate;
        const int8_t* u = w_up + (size_t)k * intermediate;
        int8_t* d = gu.data() + (size_t)k * 2 * intermediate;
        for (int c = 0; c < intermediate; ++c) {
            d[2 * c] = g[c];
            d[2 * c + 1] = u[c];
        }
    }
    tllm_mlp* m = new tllm_mlp();
    m->hidden = hidden;
    m->inter = intermediate;
    m->s_gate = s_gate;
    m->s_up = s_up;
    int rc = tllm_weight_create_dense(gu.data(), hidden, 2 * intermediate, 1.f, opts, &m->gate_up);
    if (rc == TLLM_OK) rc = tllm_weight_create_dense(w_down, intermediate, hidden, s_down, opts, &m->down);
    if (rc == TLLM_OK) {
        m->h_cap = (size_t)16 * intermediate * 4;
        cudaError_t e = cudaMalloc(&m->d_h, m->h_cap);
        if (e != cudaSuccess) rc = fail(TLLM_ERR_CUDA, "cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    if (rc != TLLM_OK) {
        tllm_mlp_destroy(m);
        return rc;
    }
    *out = m;
    return TLLM_OK;
}

int tllm_mlp_create_cpu_format(int kind, int group, int chunk, int ri32, const int32_t* meta_gate, const void* ri_gate,
                               const int32_t* meta_up, const void* ri_up, const int32_t* meta_down, const void* ri_down, int hidden,
                               int intermediate, const tllm_pack_opts* opts, tllm_mlp** out) {
    if (!meta_gate || !ri_gate || !meta_up || !ri_up || !meta_down || !ri_down || hidden <= 0 || intermediate <= 0 || !out)
        return fail(TLLM_ERR_ARG, "tllm_mlp_create_cpu_format: bad argument");
    if (kind < 1 || kind > 5) return fail(TLLM_ERR_ARG, "tllm_mlp_create_cpu_format: kind must be 1..5 (the single-array formats)");
    *out = nullptr;
    std::vector<int8_t> g, u, d;
    const char* msg = tllm::decode_cpu_format(kind, group, chunk, meta_gate, ri_gate, ri32, 0, intermediate, hidden, &g);
    if (!msg) msg = tllm::decode_cpu_format(kind, group, chunk, meta_up, ri_up, ri32, 0, intermediate, hidden, &u);
    if (!msg) msg = tllm::decode_cpu_format(kind, group, chunk, meta_down, ri_down, ri32, 0, hidden, intermediate, &d);
    if (msg) return fail(TLLM_ERR_ARG, "tllm_mlp_create_cpu_format: %s", msg);
    return tllm_mlp_create(g.data(), u.data(), d.data(), hidden, intermediate, 1.f, 1.f, 1.f, opts, out);
}

int tllm_mlp_destroy(tllm_mlp* m) {
    if (!m) return TLLM_OK;
    tllm_weight_destroy(m->gate_up);
    tllm_weight_destroy(m->down);
    cudaFree(m->d_h);
    cudaFree(m->d_x);
    cudaFree(m->d_y);
    delete m;
    return TLLM_OK;
}

int tllm_mlp_forward(tllm_mlp* m, const void* X, int x_dtype, int rows, void* Y, void* H, void* stream) {
    return tllm_mlp_forward_ex(m, X, x_dtype, rows, Y, x_dtype, H, stream);
}

int tllm_mlp_forward_ex(tllm_mlp* m, const void* X, int x_dtype, int rows, void* Y, int y_dtype, void* H, void* stream) {
    if (!m || !X || !Y) return fail(TLLM_ERR_ARG, "tllm_mlp_forward: NULL pointer");
    if (y_dtype != TLLM_F32 && y_dtype != TLLM_F16 && y_dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "tllm_mlp_forward: unsupported y_dtype");
    if (rows <= 0) return fail(TLLM_ERR_ARG, "tllm_mlp_forward: rows must be positive");
    if (x_dtype != TLLM_F32 && x_dtype != TLLM_F16 && x_dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "tllm_mlp_forward: unsupported dtype");
    if (!H && (size_t)rows * m->inter * dtype_size(x_dtype) > m->h_cap) return fail(TLLM_ERR_ARG, "tllm_mlp_forward: pass H for more than 16 rows");
    int rc = check_device(m->gate_up, "tllm_mlp_forward");
    if (rc) return rc;
    char* h = (char*)(H ? H : m->d_h);
    cudaStream_t st = (cudaStream_t)stream;
    // the two products pick their kernel independently (gate and up share the first one: its epilogue applies SiLU and the product)
    const KernelChoice k1 = choose_kernel(m->gate_up, X, x_dtype, TLLM_ROW_MAJOR, m->hidden, rows);
    if (k1 == KERNEL_NIBBLE) rc = run_nb(m->gate_up, X, x_dtype, m->hidden, rows, h, x_dtype, m->inter, 1, m->s_gate, m->s_up, st);
    else if (k1 == KERNEL_MMA) rc = run_mm(m->gate_up, X, x_dtype, m->hidden, rows, h, x_dtype, m->inter, 1, m->s_gate, m->s_up, st);
    else rc = run_gather(m->gate_up, X, x_dtype, TLLM_ROW_MAJOR, m->hidden, rows, h, x_dtype, m->inter, 1, m->s_gate, m->s_up,
                         Scratch{m->gate_up->d_partial, m->gate_up->d_counters}, st);
    if (rc) return rc;
    const KernelChoice k2 = choose_kernel(m->down, h, x_dtype, TLLM_ROW_MAJOR, m->inter, rows);
    if (k2 == KERNEL_NIBBLE) return run_nb(m->down, h, x_dtype, m->inter, rows, Y, y_dtype, m->hidden, 0, m->down->scale, 0.f, st);
    if (k2 == KERNEL_MMA) return run_mm(m->down, h, x_dtype, m->inter, rows, Y, y_dtype, m->hidden, 0, m->down->scale, 0.f, st);
    return run_gather(m->down, h, x_dtype, TLLM_ROW_MAJOR, m->inter, rows, Y, y_dtype, m->hidden, 0, m->down->scale, 0.f,
                      Scratch{m->down->d_partial, m->down->d_counters}, st);
}

// [a][b] -> [b][a] for elements of `e` bytes
static void transpose_bytes(const void* src, void* dst, size_t a, size_t b, size_t e) {
    const char* s = (const char*)src;
    char* d = (char*)dst;
    for (size_t i = 0; i < a; ++i)
        for (size_t j = 0; j < b; ++j) memcpy(d + (j * a + i) * e, s + (i * b + j) * e, e);
}

int tllm_mlp_forward_host(tllm_mlp* m, void* X, int x_dtype, int x_layout, int rows, void* H) {
    if (!m || !X) return fail(TLLM_ERR_ARG, "tllm_mlp_forward_host: NULL pointer");
    if (rows <= 0) return fail(TLLM_ERR_ARG, "tllm_mlp_forward_host: rows must be positive");
    if (x_dtype != TLLM_F32 && x_dtype != TLLM_F16 && x_dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "tllm_mlp_forward_host: unsupported dtype");
    if (x_layout != TLLM_ROW_MAJOR && x_layout != TLLM_COL_MAJOR) return fail(TLLM_ERR_ARG, "tllm_mlp_forward_host: unknown layout");
    tllm_weight* w = m->gate_up;
    int rc = check_device(w, "tllm_mlp_forward_host");
    if (rc) return rc;
    const size_t e = dtype_size(x_dtype), xb = (size_t)rows * m->hidden * e, hb = (size_t)rows * m->inter * e;
    if (!w->own_stream) CU_TRY(cudaStreamCreateWithFlags(&w->own_stream, cudaStreamNonBlocking));
    if (!w->h_status) CU_TRY(cudaMallocHost((void**)&w->h_status, sizeof(int)));
    rc = ensure(&m->d_x, &m->x_cap, xb, false);
    if (rc) return rc;
    rc = ensure(&m->d_y, &m->y_cap, xb, false);
    if (rc) return rc;
    rc = ensure(&m->d_h, &m->h_cap, hb, false);
    if (rc) return rc;
    // a column-major caller ([hidden][rows], rows contiguous) is turned on the host: the block itself is row-major
    const bool turn = x_layout == TLLM_COL_MAJOR && rows > 1;
    std::vector<char> tx, th;
    void* hx = X;
    if (turn) {
        tx.resize(xb);
        transpose_bytes(X, tx.data(), (size_t)m->hidden, (size_t)rows, e);
        hx = tx.data();
        if (H) th.resize(hb);
    }
    CU_TRY(cudaMemcpyAsync(m->d_x, hx, xb, cudaMemcpyHostToDevice, w->own_stream));
    rc = tllm_mlp_forward(m, m->d_x, x_dtype, rows, m->d_y, m->d_h, w->own_stream);
    if (rc) return rc;
    CU_TRY(cudaMemcpyAsync(hx, m->d_y, xb, cudaMemcpyDeviceToHost, w->own_stream));
    if (H) CU_TRY(cudaMemcpyAsync(turn ? (void*)th.data() : H, m->d_h, hb, cudaMemcpyDeviceToHost, w->own_stream));
    CU_TRY(cudaMemcpyAsync(w->h_status, w->d_status, sizeof(int), cudaMemcpyDeviceToHost, w->own_stream));
    CU_TRY(cudaStreamSynchronize(w->own_stream));
    if (turn) {
        transpose_bytes(tx.data(), X, (size_t)rows, (size_t)m->hidden, e);
        if (H) transpose_bytes(th.data(), H, (size_t)rows, (size_t)m->inter, e);
    }
    if (*w->h_status) return tllm_weight_check(w);
    return tllm_weight_check(m->down);
}

int tllm_mlp_get_info(const tllm_mlp* m, tllm_weight_info* gate_up, tllm_weight_info* down) {
    if (!m) return fail(TLLM_ERR_ARG, "tllm_mlp_get_info: NULL");
    if (gate_up) tllm_weight_get_info(m->gate_up, gate_up);
    if (down) tllm_weight_get_info(m->down, down);
    return TLLM_OK;
}

int tllm_add_rmsnorm(void* x, const void* delta, const void* weight, void* h, int dtype, int rows, int hidden, float eps, void* stream) {
    if (!x || !h || rows < 0 || hidden <= 0) return fail(TLLM_ERR_ARG, "tllm_add_rmsnorm: bad argument");
    if (dtype != TLLM_F32 && dtype != TLLM_F16 && dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "tllm_add_rmsnorm: unsupported dtype");
    const int vec = dtype == TLLM_F32 ? 4 : 8;
    if (hidden % vec || ((uintptr_t)x | (uintptr_t)h | (uintptr_t)delta | (uintptr_t)weight) % 16)
        return fail(TLLM_ERR_ARG, "tllm_add_rmsnorm: hidden must be a multiple of %d and the pointers 16-byte aligned", vec);
    if (rows == 0) return TLLM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == TLLM_F32) add_rmsnorm_kernel<float><<<(unsigned)rows, 256, 0, st>>>((float*)x, (const float*)delta, (const float*)weight, (float*)h, hidden, eps);
    else if (dtype == TLLM_F16) add_rmsnorm_kernel<__half><<<(unsigned)rows, 256, 0, st>>>((__half*)x, (const __half*)delta, (const __half*)weight, (__half*)h, hidden, eps);
    else add_rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)weight, (__nv_bfloat16*)h, hidden, eps);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TLLM_OK;
}

int tllm_silu_mul(void* g, const void* u, int dtype, int64_t n, void* stream) {
    if (!g || !u || n < 0) return fail(TLLM_ERR_ARG, "tllm_silu_mul: bad argument");
    if (dtype != TLLM_F32 && dtype != TLLM_F16 && dtype != TLLM_BF16) return fail(TLLM_ERR_ARG, "tllm_silu_mul: unsupported dtype");
    if (n == 0) return TLLM_OK;
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(g, u, dtype, (long long)n);
    CU_TRY(cudaGetLastError());
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return TLLM_OK;
}

}  // extern "C"
