/*
 * tllm.h -- C ABI of the B200-native ternary sparse product  Y = X . W . s,  W in {-1,0,+1}.
 *
 * Plain C, plain pointers and sizes; no torch or C++ types cross this boundary.  Every entry point
 * below replaces one interface of fpgasystems/ternaryLLM; the citation (path within that repository,
 * file:line) says which.  All functions return 0 on success and a negative code on failure;
 * tllm_last_error() then holds a message for the calling thread.  Nothing here falls back to a CPU
 * implementation: a missing or unusable CUDA device is an error.
 */
#ifndef TLLM_H_
#define TLLM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TLLM_OK 0
#define TLLM_ERR_ARG (-1)      /* bad argument / unsupported shape */
#define TLLM_ERR_CUDA (-2)     /* a CUDA runtime call failed */
#define TLLM_ERR_KERNEL (-3)   /* a kernel reported a bounded wait that ran out (see tllm_last_error) */
#define TLLM_ERR_NOMEM (-4)

/* element types of activations / results */
#define TLLM_F32 0
#define TLLM_F16 1
#define TLLM_BF16 2
#define TLLM_I8 3              /* int8 activations, exact int32 accumulation */
#define TLLM_I32 4             /* result type for TLLM_I8 activations */

/* activation layouts */
#define TLLM_ROW_MAJOR 0       /* X is [M][K], K contiguous (what the reference's Python modules hold) */
#define TLLM_COL_MAJOR 1       /* X is [K][M], M contiguous (what ter_tiled_mcsc_spmm indexes,
                                  ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:173, and what the col-major CPU
                                  kernels take, ternaryLLM_CPU/src/GEMM_CPU_FP32.cpp:509-538) */

const char* tllm_last_error(void);
int tllm_version(void);
/* number of kernels this library has launched in the calling process (for benchmarks' bookkeeping) */
int64_t tllm_launch_count(void);
/* of those, launches of the tensor-core (tcgen05) kernel */
int64_t tllm_mma_launch_count(void);
/* Which kernel tllm_spmm / tllm_mlp_forward run for fp16 / bf16 row-major activations: the gather kernel on the
 * index lists, or the tensor-core kernel on the dense two-bit copy of W (the reference has one kernel for M = 1
 * and one for M > 1, ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:352-372, and no tensor-core path).
 *   rows < 0  decide per call (default) from a measured cost model: one row never takes this kernel; from two rows on
 *             it is a candidate whenever the model finds it faster than the gather kernel, and the call then goes to
 *             the faster of it and the decode tensor-core kernels (tllm_set_nibble_max_rows)
 *   rows = 0  never the tensor-core kernel
 *   rows > 0  the tensor-core kernel from that many activation rows on
 * Process-wide; returns the previous setting.  The environment variable TLLM_MMA_MIN_ROWS sets the initial one. */
int tllm_set_mma_min_rows(int rows);
/* Which kernel takes a call of a few rows: the gather kernel on the index lists, or the decode tensor-core kernels that
 * stream the four-bit copy of W by TMA (half a byte per entry whatever the sparsity; the gather kernel's cost grows with
 * the non-zeros): one launch for up to 4 rows (fp32: 2), a pair of launches (activation pieces, then the product) for up
 * to 64 rows (fp32: 32), several pairs above that.
 *   rows < 0  decide per call from a measured cost model of the two (default)
 *   rows = 0  never the decode tensor-core kernel
 *   rows > 0  always, for calls of up to that many rows
 * tllm_set_mma_min_rows(0) switches this kernel off as well.  Process-wide; returns the previous setting. */
int tllm_set_nibble_max_rows(int rows);
/* launches of the decode tensor-core kernel so far in this process */
int64_t tllm_nibble_launch_count(void);

/* --------------------------------------------------------------------------------------------------
 * Host-side packers: the four callables of the reference's `ter_spmm` extension module
 * (ternaryLLM_GPU/csrc/ter_spmm_wrapper.cu:350-355).  w is int32 [inners][columns] row-major on the
 * host with entries in {-1,0,1}; outputs are caller-allocated.
 * -------------------------------------------------------------------------------------------------- */

/* counts of +1 / -1 entries (TernaryLinear.py:104-105) */
int tllm_count_nnz(const int32_t* w, int columns, int inners, int64_t* cnt_pos, int64_t* cnt_neg);

/* convert_to_ter_csc (ter_spmm_wrapper.cu:39-78): neg_idx[cnt_neg], neg_off[columns+1],
 * pos_idx[cnt_pos], pos_off[columns+1] -- the reference returns them in this order. */
int tllm_convert_to_ter_csc(const int32_t* w, int columns, int inners, int32_t* neg_idx, int32_t* neg_off,
                            int32_t* pos_idx, int32_t* pos_off);

/* convert_to_ter_tiled_csc (ter_spmm_wrapper.cu:92-152): tile-local ids and [start,end) per
 * (column, tile): neg_off / pos_off hold columns*ceil(inners/tile_k)*2 entries.  Rows past `inners`
 * in the last tile count as zero (the reference reads out of bounds there). */
int tllm_convert_to_ter_tiled_csc(const int32_t* w, int columns, int inners, int tile_k, int32_t* neg_idx,
                                  int32_t* neg_off, int32_t* pos_idx, int32_t* pos_off);

/* convert_to_ter_tiled_mcsc (ter_spmm_wrapper.cu:156-315): merged tiled CSC.
 *   mode 0: lossless (the behaviour of the reference's Python twin, TernaryCSC.py:97-156); `padding`
 *           pads the pair region of every list with neutral (p,p) pairs to a multiple of padding_size
 *           and never drops an entry.
 *   mode 1: bit-compatible with the reference's C++ packer, including its truncation of list lengths
 *           to multiples of four (:277-291).  For drop-in comparisons only: it does not encode W.
 * tllm_ter_tiled_mcsc_len gives the number of row-index entries to allocate.  off has
 * columns*tiles*4 entries {pair_start, pair_end, rem_end, sign}; tile_idx (columns*tiles, may be NULL)
 * receives the per-column tile order by list length (inter_tile_swizzle, :9-27). */
int64_t tllm_ter_tiled_mcsc_len(const int32_t* w, int columns, int inners, int tile_k, int padding,
                                int padding_size, int mode);
int tllm_convert_to_ter_tiled_mcsc(const int32_t* w, int columns, int inners, int tile_k, int padding,
                                   int padding_size, int mode, int32_t* row_idx, int64_t row_idx_cap,
                                   int32_t* off, int32_t* tile_idx);

/* --------------------------------------------------------------------------------------------------
 * ter_spmm on the reference's own arrays (ter_spmm_wrapper.cu:318-348 -> ter_spmm_kernel.cuh:510-531).
 * All pointers are DEVICE pointers.  X holds `batch` matrices of rows x inners (layout as given);
 * Y receives batch x rows x columns, row-major, in y_dtype.  row_idx are int16 tile-local ids, col_off
 * the four int32 per (column, tile); col_tile_idx is accepted and unused, like in the reference
 * (ter_spmm_kernel.cuh:159-160).  Every list entry is honoured (pairs, then sign * remainder, with the
 * tile base applied to both), whatever `uniformed` / `padded` say.  Launches on `stream`
 * (a cudaStream_t; NULL = legacy default stream); no allocation, no synchronisation.
 * -------------------------------------------------------------------------------------------------- */
int tllm_ter_spmm(const void* X, int x_dtype, int x_layout, const int16_t* row_idx, const int32_t* col_off,
                  const int16_t* col_tile_idx, void* Y, int y_dtype, int batch, int rows, int columns,
                  int inners, int tile_k, float scale, int uniformed, int padded, void* stream);
/* Repacks one weight held in the reference's device arrays (row_idx int16, col_off int32, as
 * ternaryLLM_GPU/TernaryLLM/TernaryLinear.py:144-146 registers them) into this library's formats, once, and remembers
 * it under the arrays' addresses, the shape and the current device.  Every later tllm_ter_spmm call with the same
 * arrays runs the packed kernels (gather, or a tensor-core kernel where the cost model prefers it) instead of the
 * one-warp-per-column kernel on the arrays as they are -- so code written against the reference's three buffers gets
 * the fast path without holding a handle.  Copies the arrays to the host, allocates and synchronises: call it at
 * set-up time, not inside a stream capture.  The arrays must not change or be freed while remembered;
 * tllm_ter_spmm_forget(row_idx, col_off) drops one weight (both NULL: all) and returns how many it dropped. */
int tllm_ter_spmm_prepare(const int16_t* row_idx, const int32_t* col_off, int columns, int inners, int tile_k);
int tllm_ter_spmm_forget(const int16_t* row_idx, const int32_t* col_off);

/* --------------------------------------------------------------------------------------------------
 * Packed weights in the library's own B200 stream format (the replacement for
 * convert_ternary_weights + the three TernaryLinear buffers, TernaryLinear.py:87-113,144-146), and the
 * product on them (the replacement for TernaryLinear.forward, :152-182).
 * -------------------------------------------------------------------------------------------------- */
typedef struct tllm_weight tllm_weight;

typedef struct tllm_pack_opts {
    int tile_rows;        /* rows of a K-tile: a multiple of 32, at most 4096; 0 = 4096 (one-byte ids cover 128 row groups
                             of 32 rows; smaller tiles only make sense for tests of the multi-tile paths) */
    int num_ctas;         /* thread blocks to schedule for; 0 = number of SMs of the current device */
    int reserved0;        /* must be 0 */
    int max_rows;         /* rows of one gather launch, 1..4 (the split-K scratch is sized for it); 0 = 4 */
    int k_splits;         /* thread blocks that share one column range along K; 0 = choose (1 = no split-K scratch) */
    int no_bit_tiles;     /* 1 = do not keep the dense two-bit copy of W that the batched tensor-core kernel reads
                             (columns*inners/4 bytes); 0 = keep it */
    int no_nibbles;       /* 1 = do not keep the four-bit transposed copy of W that the decode tensor-core kernel streams
                             (columns*inners/2 bytes); 0 = keep it.  With neither copy every call runs the gather kernel. */
    int reserved[1];
} tllm_pack_opts;

typedef struct tllm_weight_info {
    int inners, columns, tile_rows, tiles, col_blocks, k_splits, tiles_per_cta, num_ctas;
    int units;                 /* (warp, K-tile, column range) work units of the index stream */
    int max_rows;
    int64_t nnz;               /* true non-zeros of W */
    int64_t stream_bytes;      /* index stream as stored: one byte per id, padding and list flags included */
    int64_t meta_bytes;        /* block tables as stored */
    int64_t scratch_bytes;     /* split-K partial sums + counters owned by the handle */
    int64_t algorithmic_bytes; /* 2*nnz + 16*columns*ceil(inners/512): the reference layout's weight bytes */
    int64_t bit_tile_bytes;    /* dense two-bit copy read by the batched tensor-core kernel (0 if not kept) */
    int64_t nibble_bytes;      /* four-bit transposed copy streamed by the decode tensor-core kernel (0 if not kept) */
    float scale;
} tllm_weight_info;

/* Float weights -> ternary weights and a per-tensor scale, host memory, w and out [inners][columns] row-major
 * (the reference's ternarize_weights is a stub that raises, ternaryLLM_GPU/TernaryLLM/TernaryLinear.py:19-20).
 * target_sparsity in (0,1): the round(target_sparsity * n) entries of smallest magnitude become 0; otherwise entries
 * with |w| <= threshold_factor * mean|w| become 0 (threshold_factor <= 0 means 0.7, the ternary-weight-network rule).
 * The others become sign(w); *scale = mean |w| of the kept entries (the least-squares scale). */
int tllm_ternarize(const float* w, int inners, int columns, float threshold_factor, float target_sparsity,
                   int8_t* out, float* scale);
/* from a dense ternary matrix, int8 [inners][columns] row-major, host memory */
int tllm_weight_create_dense(const int8_t* w, int inners, int columns, float scale,
                             const tllm_pack_opts* opts, tllm_weight** out);
/* from the reference's merged tiled CSC arrays on the host (row ids as int32, as the packers return them) */
int tllm_weight_create_mcsc(const int32_t* row_idx, const int32_t* col_off, int columns, int inners,
                            int tile_k, float scale, const tllm_pack_opts* opts, tllm_weight** out);
/* from the reference's merged tiled CSC arrays as the reference's modules hold them: int16 row ids and the four int32
 * per (column, tile), both in DEVICE memory (TernaryLinear.py:144-146).  Copies them to the host, checks every list
 * offset against row_idx_len, decodes and repacks: the one-off step that lets code written against the reference's three
 * buffers run the fast kernels (tllm_ter_spmm consumes the arrays as they are, one warp per column). */
int tllm_weight_create_mcsc_device(const int16_t* row_idx, int64_t row_idx_len, const int32_t* col_off, int columns,
                                   int inners, int tile_k, float scale, const tllm_pack_opts* opts, tllm_weight** out);
/* from the reference's CPU formats (ternaryLLM_CPU/src/TCSC.hpp), host memory:
 *   kind 0 SparseFormat (:6-34): meta = col_start_neg[N+1] ++ col_start_pos[N+1], ri = neg ids ++ pos ids,
 *          aux = number of neg ids
 *   kind 1 MergedTCSC (:36-90); kind 2/3/4 MergedTCSC_Group "min"/"mid"/"max" (:92-409);
 *   kind 5 uniform (meta[0] = non-zeros per column).
 * group = columns per group; chunk = 0 for the column-interleaved prefix, otherwise the number of
 * consecutive positives (then negatives) per block (group size for interleaved=false, 8 / 16 for the
 * _CS8 / _CS16 layouts); ri32 selects int32 row ids. */
int tllm_weight_create_cpu_format(int kind, int group, int chunk, const int32_t* meta, const void* ri,
                                  int ri32, int64_t aux, int columns, int inners, float scale,
                                  const tllm_pack_opts* opts, tllm_weight** out);
/* Diagnostic that needs no GPU: packs w for `num_sms` thread blocks on the host, checks the invariants the
 * kernel relies on (every (tile, column) covered once, ids inside their tile, list counts, no lane more than a ring
 * ahead of the reduced slots, reduce points only behind complete slots), unpacks into w_out (inners*columns int8)
 * and fills info. */
int tllm_pack_roundtrip(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                        int8_t* w_out, tllm_weight_info* info);
/* Diagnostic that needs no GPU: how the decode tensor-core kernel's grid shares a weight of this shape on num_sms SMs.
 * dims[6] = {K blocks of 128 rows, column tiles of 128, K blocks per range, ranges, thread blocks per range, K blocks
 * per unit}; words (NULL = dims only) = (1 + ranges) * tiles entries: words[t] = thread blocks that hold a part of column
 * tile t, words[(1 + j) * tiles + t] = first | last << 16 block of range j on tile t.  No counterpart in the reference. */
int tllm_nibble_schedule(int inners, int columns, int num_sms, int* dims, uint32_t* words, size_t capacity_words);
/* Test hook that needs no GPU: packs w, overwrites one field of the packed image (what: 1 table word `where`, 2 stream
 * byte `where`, 3 tile_rows, 4 tiles, 5 col_blocks, 6 k_splits, 7 tiles_per_cta, 8..9 / 12..13 a block descriptor's
 * table words / first vector / table offset / vectors, 10 column range `where`, 11 inners; 0 = nothing) with `value` and
 * runs the validator that tllm_weight_load runs before it uploads anything.  Returns its verdict. */
int tllm_pack_corrupt_check(const int8_t* w, int inners, int columns, const tllm_pack_opts* opts, int num_sms,
                            int what, int64_t where, uint32_t value);
/* Shared-segment rows: this library's own sparse-segment image of a ternary matrix, host memory only.  The reference
 * names such an encoding but holds no definition of it (SSR/README.md cites a paper; the one consumer,
 * ternaryLLM_GPU/csrc/ter_spmm_kernel.cuh:159-160, is commented out), so these two functions have no counterpart there.
 * The 8 columns of a group share, per segment of 256 rows, one ascending list of the rows any of them uses (a byte
 * each) and a 16-bit word of two-bit codes per listed row: 2 + 3n bytes per (group, segment).  It is a storage and
 * interchange form for matrices of 90 % zeros and more; no kernel reads it -- decode, then tllm_weight_create_dense.
 * tllm_ssr_encode: w int8 [inners][columns] row-major; image == NULL only reports the size in *bytes.
 * tllm_ssr_decode: validates the whole image (sizes, offsets, ascending rows, code words) before w_out is trusted. */
int tllm_ssr_encode(const int8_t* w, int inners, int columns, uint8_t* image, size_t capacity, size_t* bytes);
int tllm_ssr_decode(const uint8_t* image, size_t bytes, int inners, int columns, int8_t* w_out);
/* a handle from such an image: decoded and validated on the host, then packed like tllm_weight_create_dense */
int tllm_weight_create_ssr(const uint8_t* image, size_t bytes, int inners, int columns, float scale,
                           const tllm_pack_opts* opts, tllm_weight** out);
int tllm_weight_destroy(tllm_weight* w);
int tllm_weight_get_info(const tllm_weight* w, tllm_weight_info* info);
/* Packed-weight files: everything a handle holds on the device (index stream, block tables, block descriptors, the
 * dense two-bit copy if kept, the scale) in one file, so that a model is packed once and loaded without repacking.
 * The reference keeps its packed arrays as module buffers in a PyTorch state dict
 * (ternaryLLM_GPU/TernaryLLM/TernaryLinear.py:144-146); this is the equivalent for handles.  A file written on a
 * device with another SM count loads and runs (the gather kernel's block schedule is part of the file).  A file is
 * validated in full on the host before anything is uploaded; a damaged or foreign file is refused with TLLM_ERR_ARG. */
int tllm_weight_save(const tllm_weight* w, const char* path);
int tllm_weight_load(const char* path, tllm_weight** out);
/* change the per-tensor scale s (host value; takes effect for later calls) */
int tllm_weight_set_scale(tllm_weight* w, float scale);

/* Reads the handle's device status word (this synchronises with the device).  Returns TLLM_ERR_KERNEL if
 * a kernel gave up on one of its bounded waits since the last check -- its output is then undefined --
 * and clears the condition. */
int tllm_weight_check(tllm_weight* w);

/* Y[rows][columns] = X . W . s   on device pointers, launched on `stream`; the device that holds the handle must be
 * current.  The gather kernel takes max_rows (at most four) rows per launch, larger row counts run as several
 * launches or on the tensor-core kernel (tllm_set_mma_min_rows).  Calls on one handle must not overlap on the GPU
 * (they share the handle's scratch); calls on different handles may. */
int tllm_spmm(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, void* Y, int y_dtype,
              void* stream);

/* Same with HOST buffers: copies X to the device, runs, copies Y back and synchronises.  This is the
 * form behind the CPU entry points (GEMM_CPU_FP32.hpp:40-185, GEMM_CPU_INT8.hpp:11-29): caller-owned host
 * arrays in, host arrays out.  y_layout TLLM_COL_MAJOR writes Y as [columns][rows], the col-major
 * kernels' result layout (GEMM_CPU_FP32.cpp:534). */
int tllm_spmm_host(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, void* Y, int y_dtype,
                   int y_layout);
/* Same plus a bias: Y[m][n] = (X . W . s)[m][n] + bias[n], bias a host array of `columns` values of y_dtype (NULL = no
 * bias).  The one place the reference adds a bias is sparseGEMM<T> (ternaryLLM_CPU/src/TCSC.hpp:413-430). */
int tllm_spmm_host_bias(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, const void* bias,
                        void* Y, int y_dtype, int y_layout);

/* The same product for callers that are not allowed to allocate device memory -- a serving loop whose
 * memory budget was fixed at start-up, code living under a framework allocator it must not bypass, a path
 * where an allocation's implicit synchronisation is unacceptable.  (No counterpart in the reference: its
 * extension allocates its result on every call, ter_spmm_wrapper.cu:334.)  Inputs and outputs are the
 * caller's device buffers; the split-K partial sums and arrival counters live in a fixed array inside the
 * library (about 4 MiB, held by every GPU that loads the library until the process exits) instead of the
 * scratch the handle got from cudaMalloc.  Nothing is allocated or freed here.  Always the gather kernel.
 *   Limit:  k_splits * min(rows, max_rows) * columns  <=  1 048 576 partial sums (weights packed without a
 *           K-split need none), and at most 4096 column blocks; anything larger is refused with TLLM_ERR_ARG
 *           and a message (see tllm_weight_get_info).
 *   First call on a device looks up the array's device address (once per device, with that device current);
 *           make that first call outside any stream capture.
 *   All calls share the one array: the counters are cleared in stream order at every call, but two calls that
 *           overlap on the GPU (different streams) race and give wrong results.
 *   A kernel that gave up on a bounded wait reports through the handle's status word as on every other path:
 *           tllm_weight_check(w). */
int tllm_spmm_static_scratch(tllm_weight* w, const void* X, int x_dtype, int x_layout, int rows, void* Y,
                             int y_dtype, void* stream);

/* --------------------------------------------------------------------------------------------------
 * Fused ternary MLP block  y = down( silu(gate(x)) * up(x) )  (TernaryMLP.py:33-35;
 * TernaryMLP<T>::forward, ternaryLLM_CPU/src/LlamaModel.hpp:343-452): gate and up share one activation
 * table and one launch whose epilogue applies SiLU and the product; down follows as a second, dependent launch
 * whose weight stream is prefetched while the first kernel drains (two launches per block, h through HBM).
 * -------------------------------------------------------------------------------------------------- */
typedef struct tllm_mlp tllm_mlp;
int tllm_mlp_create(const int8_t* w_gate, const int8_t* w_up, const int8_t* w_down, int hidden,
                    int intermediate, float s_gate, float s_up, float s_down, const tllm_pack_opts* opts,
                    tllm_mlp** out);
int tllm_mlp_destroy(tllm_mlp* m);
/* X [rows][hidden] -> Y [rows][hidden]; H (device, rows*intermediate elements of x_dtype) receives the
 * intermediate activations and may be NULL to use the handle's own buffer. */
int tllm_mlp_forward(tllm_mlp* m, const void* X, int x_dtype, int rows, void* Y, void* H, void* stream);
/* Same with the result type chosen by the caller (TLLM_F32 keeps the down projection's sums unrounded: what a
 * tensor-parallel layer hands to the all-reduce). */
int tllm_mlp_forward_ex(tllm_mlp* m, const void* X, int x_dtype, int rows, void* Y, int y_dtype, void* H, void* stream);
/* Same with HOST buffers and the reference's in-place convention (TernaryMLP<T>::forward overwrites its input with the
 * block's output, LlamaModel.hpp:165-270 and :343-452): X ([rows][hidden] for TLLM_ROW_MAJOR, [hidden][rows] for
 * TLLM_COL_MAJOR as the reference's colMajor kernels take it) is copied to the device, the block runs, the result is
 * copied back over X in the same layout; H (host, rows*intermediate values in that layout, may be NULL) receives
 * silu(gate)*up. Synchronises. */
int tllm_mlp_forward_host(tllm_mlp* m, void* X, int x_dtype, int x_layout, int rows, void* H);
/* The block from three weights in one of the reference's single-array CPU formats (kinds 1..5 of
 * tllm_weight_create_cpu_format; gate and up are [hidden] x [intermediate], down is [intermediate] x [hidden]): what
 * TernaryMLP<T> keeps in WG_/WU_/WD_metadata and _rowindex (LlamaModel.hpp:95-100, :276-281). Scales are 1. */
int tllm_mlp_create_cpu_format(int kind, int group, int chunk, int ri32, const int32_t* meta_gate, const void* ri_gate,
                               const int32_t* meta_up, const void* ri_up, const int32_t* meta_down,
                               const void* ri_down, int hidden, int intermediate, const tllm_pack_opts* opts,
                               tllm_mlp** out);
int tllm_mlp_get_info(const tllm_mlp* m, tllm_weight_info* gate_up, tllm_weight_info* down);

/* Exact SiLU(x)*y epilogue on its own (Naive_SiLU_Dot, ternaryLLM_CPU/src/initData.hpp:204-210):
 * g[i] = g[i]*u[i]/(1+exp(-g[i])) in fp32, device pointers. */
int tllm_silu_mul(void* g, const void* u, int dtype, int64_t n, void* stream);

/* Glue between two products of a decoder layer, one launch: x[rows][hidden] += delta (skipped when delta is NULL),
 * then h = x * rsqrt(mean(x^2) + eps) * weight (weight = 1 when NULL); fp32 sums, all tensors of one float type,
 * device pointers aligned to 16 bytes, hidden a multiple of 8 (4 for fp32).  The reference leaves the residual add and LlamaRMSNorm to stock Hugging Face modules
 * (ternaryLLM_GPU/TernaryLLM/TernaryLlama.py); this entry point exists so that a decode step launches two
 * kernels per layer for them instead of a dozen element-wise ones. */
int tllm_add_rmsnorm(void* x, const void* delta, const void* weight, void* h, int dtype, int rows, int hidden,
                     float eps, void* stream);

/* --------------------------------------------------------------------------------------------------
 * Tensor-parallel glue: the all-reduce that follows a row-sharded product (O and down projections), fused with
 * the residual add and RMSNorm that follow it, in one kernel per GPU over peer-mapped memory.  The reference has
 * no distributed code; the partitioning is the usual one (column-sharded QKV / gate / up, row-sharded O / down).
 *
 *   x[r] += sum over ranks of partial_rank[r]        (fp32 partial sums, added in rank order on every GPU: all
 *   h[r]  = x[r] * rsqrt(mean(x[r]^2) + eps) * w      ranks compute identical bits; x rounded once to its type)
 *
 * One process per GPU.  Every rank creates a communicator (receive slots for max_rows x hidden partial sums from
 * each rank, double-buffered, plus flags), exports two inter-process memory handles (tllm_comm_handle_bytes bytes),
 * the caller all-gathers them with whatever it uses for rendezvous (torch.distributed in this package) and every
 * rank connects.  Each call pushes the rank's rows into its slot on every peer with plain stores over NVLink,
 * releases a flag per peer, waits (bounded: tllm_comm_set_wait_limit, default about a second) for the peers' flags
 * and reduces.  All ranks must make the same sequence of calls with the same row counts.  A wait that runs out
 * leaves the result undefined and is reported by tllm_comm_check, after which the communicator must be destroyed
 * on every rank.  No cluster-multicast loads and no library kernels touch peer memory.
 * tllm_comm_attach wires a peer to buffers the caller names (tests on one GPU: a stand-in peer whose slot and flag
 * the host fills). */
typedef struct tllm_comm tllm_comm;
int tllm_comm_create(int world, int rank, int max_rows, int hidden, tllm_comm** out);
int tllm_comm_handle_bytes(void);
int tllm_comm_export(tllm_comm* c, void* handle);
int tllm_comm_connect(tllm_comm* c, const void* handles /* world * tllm_comm_handle_bytes(), in rank order */);
int tllm_comm_attach(tllm_comm* c, int peer, void* recv, void* flags);
int tllm_comm_buffers(tllm_comm* c, void** recv, void** flags, int64_t* recv_bytes, int64_t* flag_bytes);
int tllm_comm_set_wait_limit(tllm_comm* c, double milliseconds);
int tllm_comm_check(tllm_comm* c);
int tllm_comm_destroy(tllm_comm* c);
int tllm_allreduce_add_rmsnorm(tllm_comm* c, const float* partial, void* x, const void* weight, void* h, int dtype,
                               int rows, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TLLM_H_ */
