/*
 * trspmm.h — C ABI of libtrspmm.so: the hybrid sparse hot path (format builder, fused
 * TC-block / 2:4 mma.sp / CSR-remainder SpMM, SDDMM) as hand-written CUDA for sm_100a.
 *
 * Conventions
 *   - every entry point returns 0 on success, a negative TRS_E_* value for an argument error
 *     found on the host before anything was launched, or a positive cudaError_t value;
 *   - no exception crosses this boundary; trs_strerror() explains any returned code;
 *   - pointers are plain device pointers unless the name says "host"; sizes are element counts;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - there is no CPU fallback: without a CUDA device every compute entry returns an error.
 *
 * The file:line citations name the interface of the reference project each entry replaces.
 */
#ifndef TRSPMM_H_
#define TRSPMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRS_OK 0
#define TRS_E_ARG (-1)        /* null pointer / non-positive size / unsupported value          */
#define TRS_E_WINDOW (-2)     /* window outside 1..16 (mGCN_online.cpp:888, block_online.cpp:553) */
#define TRS_E_OFFSETS (-3)    /* a prefix array is not monotone or does not start at 0          */
#define TRS_E_SHAPE (-4)      /* array lengths inconsistent with each other                     */
#define TRS_E_COLUMN (-5)     /* a column id outside [-1, kOri)                                 */
#define TRS_E_ROW (-6)        /* a row id outside [0, mOri)                                     */
#define TRS_E_WORKSPACE (-7)  /* caller-provided workspace too small                            */
#define TRS_E_NOT_CANONICAL (-8) /* CSR columns not ascending / duplicated inside a row         */
#define TRS_E_NO_DEVICE (-9)  /* no usable CUDA device                                          */
#define TRS_E_LIMIT (-10)     /* size beyond a documented fixed limit                           */

#define TRS_OUT_F32 0 /* what the reference returns (mGCN_online.cpp:934) */
#define TRS_OUT_F16 1

typedef uint16_t trs_half; /* IEEE binary16 bits */

/* The arrays block_sptc_2to4_online returns (block_online.cpp:844-870) that the forward pass
 * consumes (mGCN_online.cpp:760-800), with the value arrays already cast to fp16 as
 * mdataset2_online.py:151-153 does.  All pointers live in the same memory space. */
typedef struct trs_format {
    /* dense 16x8 tensor-core blocks */
    const int32_t* t_row_offset;   /* [parts_t + 1]  prefix of blocks per part               */
    const int32_t* t_block_offset; /* [blocks + 1]   prefix of values per block              */
    const int32_t* t_column;       /* [blocks * 8]   column per slot, -1 padded              */
    const trs_half* t_value;       /* [tc_nnz]                                               */
    const int32_t* t_window_row;   /* [parts_t]      first global row of the part's window   */
    const int64_t* t_binary;       /* [blocks * 2]   occupancy bitmaps rows 0-7 / 8-15       */
    int32_t parts_t;
    int32_t blocks;
    /* CUDA-core CSR remainder: long parts, then short parts */
    const int32_t* c_row_offset;   /* [parts_c + 1] */
    const int32_t* c_row;          /* [parts_c]     */
    const int32_t* c_column;
    const trs_half* c_value;
    int32_t parts_c;
    const int32_t* cs_row_offset;  /* [parts_c_short + 1] */
    const int32_t* cs_row;
    const int32_t* cs_column;
    const trs_half* cs_value;
    int32_t parts_c_short;
    /* packed 2:4 tiles for mma.sp m16n8k16 */
    const int32_t* s_window_tile_offset; /* [num_windows + 1] */
    const int32_t* s_tile_column;        /* [tiles * 16]      */
    const uint32_t* s_packed_a;          /* [tiles * 64]      */
    const uint32_t* s_packed_meta;       /* [tiles * 8]       */
    int32_t num_windows;
    int32_t tiles;
} trs_format;

typedef struct trs_spmm_plan trs_spmm_plan; /* opaque */

/* Per-call timings in milliseconds (device time, CUDA events), the slots of the reference's
 * return tuple [C, ms, ms_tc, ms_cuda_long, ms_cuda_short, ms_sptc] (mGCN_online.cpp:1130-1137).
 * The three routes run fused in one kernel here, so only `total` is a measurement. */
typedef struct trs_timing {
    float total_ms;
    float tc_ms, cuda_long_ms, cuda_short_ms, sptc_ms; /* always 0: fused */
    float h2d_ms, d2h_ms;
} trs_timing;

const char* trs_strerror(int code);
int trs_version(void);
int trs_device_count(void);

/* ---- SpMM: plan over device-resident format arrays ---------------------------------------
 * Replaces the device half of spmm_forward_fp16_tcu_cuda_sptc_mma_parallel_online
 * (mGCN_online.cpp:760-1138 -> mGCNkernel_online.cu:1529-1727).  The plan validates the
 * arrays on the device (monotone prefixes, column / row ranges), derives per-window work
 * items and keeps only small index arrays of its own; the format arrays stay caller-owned and
 * must outlive the plan.  `validate` = 0 skips the range checks. */
int trs_spmm_plan_create(const trs_format* dev_format, int m_rows, int k_cols, int window,
                         int validate, void* stream, trs_spmm_plan** out_plan);
int trs_spmm_plan_destroy(trs_spmm_plan* plan);
/* Scratch the run needs for feature width F (partial sums of windows split across CTAs). */
int trs_spmm_workspace_bytes(const trs_spmm_plan* plan, int F, size_t* bytes);
/* C[m_rows, F] = A' * B[k_cols, F]; fp16 inputs, fp32 accumulate; C fully written (no memset
 * needed), fp32 or fp16 per out_dtype.  Asynchronous on `stream`; allocates nothing. */
int trs_spmm_run(const trs_spmm_plan* plan, const trs_half* B, void* C, int F, int out_dtype,
                 void* workspace, size_t workspace_bytes, void* stream);
/* Same with an epilogue fused into the single write of C.  TRS_EPILOGUE_RELU: C = max(A'B, 0), the
 * activation of a GCN layer H = ReLU(A (X W)) (no layer code exists in the reference; the SpMM it
 * would call is mGCN_online.cpp:760). */
#define TRS_EPILOGUE_RELU 1
int trs_spmm_run_ex(const trs_spmm_plan* plan, const trs_half* B, void* C, int F, int out_dtype, int flags,
                    void* workspace, size_t workspace_bytes, void* stream);
/* SpMM fused with the exchange that follows it in a sharded GCN layer (no counterpart in the
 * reference, which has neither layers nor multi-GPU code).  The plan covers this GPU's row range of
 * a matrix with N_total rows; the fp16 result rows (ReLU optional) are written straight from the
 * kernel's epilogue into n_dst (<= 8) buffers of shape [N_total, F] at rows row0 + local row:
 * this GPU's copy and its NVLink peers' copies (peer-mapped device pointers, e.g. from CUDA IPC or
 * torch symmetric memory), as plain 16-byte stores of whole 256-byte row segments.  When every
 * rank has run it and the ranks have synchronised, each holds the whole matrix: the all-gather is
 * gone.  Needs F % 8 == 0 and 16-byte aligned buffers. */
int trs_spmm_run_bcast(const trs_spmm_plan* plan, const trs_half* B, void* const* dst, int n_dst,
                       long long row0, int F, int flags, void* workspace, size_t workspace_bytes,
                       void* stream);
/* Dense row-block product fused with the exchange that follows it in a row-sharded GCN layer (no
 * counterpart in the reference): Z[row0 + r, :] = H[r, :] * W for this GPU's `rows` rows of the
 * hidden matrix (H: [rows, K] fp16, W: [K, N] fp16 row-major, fp32 accumulate), the fp16 rows of Z
 * written by the same kernel into n_dst (<= 8) buffers of shape [N_total, N]: this GPU's copy and
 * its NVLink peers' (peer-mapped pointers), 16-byte stores of whole rows.  K a multiple of 16 up
 * to 256, N in {32, 64, 128}, N <= K, all pointers 16-byte aligned.  Asynchronous on `stream`. */
int trs_rows_gemm_bcast(const trs_half* H, const trs_half* W, void* const* dst, int n_dst, long long row0,
                        int rows, int K, int N, void* stream);
/* The same product with the rows stored once through an NVLink multicast address (multimem.st):
 * `multicast_dst` is the multicast mapping of the [N_total, N] buffers of all ranks (e.g. the
 * multicast_ptr of a torch symmetric-memory handle); the switch delivers every store to every bound
 * GPU, this one included, so the sender issues each row once whatever the number of ranks. */
int trs_rows_gemm_mcast(const trs_half* H, const trs_half* W, void* multicast_dst, long long row0, int rows,
                        int K, int N, void* stream);
/* Health word of the plan's kernels.  No kernel of the library waits on a flag or barrier another
 * warp or kernel sets, so there is no wait that could give up: always 0.  Kept for callers of
 * earlier versions. */
int trs_spmm_status(const trs_spmm_plan* plan, int* status);
/* trs_spmm_run for callers that can neither allocate device memory nor be handed any: hosts that
 * gave the whole device to their own memory pool at start-up, and latency-critical loops where
 * cudaMalloc / cudaFree would stall every stream.  This entry has no counterpart in the
 * reference.  It runs the same kernels as trs_spmm_run, keeping the partial sums of split
 * windows in a fixed array inside the library (TRS_STATIC_SCRATCH_BYTES per GPU, held from
 * library load to process exit) and allocates nothing, on the host or the device.
 *   - returns TRS_E_LIMIT when the plan needs more scratch for this F than the array holds
 *     (trs_spmm_static_scratch_bytes tells the need); nothing is launched then;
 *   - the first call on each device looks up the array's device address; make that call before
 *     any stream capture starts on that device;
 *   - all calls on a device share the one array: calls whose kernels may overlap on the GPU
 *     (different streams) race on it, so keep them ordered.  No clearing is needed between
 *     calls: every slot a call reads is fully written by that call first. */
#define TRS_STATIC_SCRATCH_BYTES (8u << 20)
int trs_spmm_run_static(const trs_spmm_plan* plan, const trs_half* B, void* C, int F, int out_dtype,
                        void* stream);
int trs_spmm_static_scratch_bytes(const trs_spmm_plan* plan, int F, size_t* bytes);
/* trs_spmm_run_ex restricted to the row windows [window_begin, window_end) of the plan: only the
 * rows of those windows are written.  Lets a caller pipeline a large SpMM against whatever
 * consumes its rows (a device->host copy, an exchange).  No counterpart in the reference. */
int trs_spmm_run_windows(const trs_spmm_plan* plan, const trs_half* B, void* C, int F, int out_dtype,
                         int flags, void* workspace, size_t workspace_bytes, void* stream,
                         int window_begin, int window_end);
int trs_spmm_num_windows(const trs_spmm_plan* plan);
/* Number of kernels one trs_spmm_run launches (1, or 2 when some window is split). */
int trs_spmm_launches(const trs_spmm_plan* plan);

/* ---- SpMM with HOST buffers: the reference's calling convention ------------------------------
 * trs_spmm_forward_host mirrors spmm_forward_fp16_tcu_cuda_sptc_mma_parallel_online
 * (mGCN_online.cpp:760-800): every array is a host pointer, device memory is allocated,
 * filled, used `epoches` times and released inside the call, C is fp32 [mOri, dimN] on the host.
 * The compat entries with SPTC-only inputs (forward_fp16_sptc_mma_packed_online,
 * mGCN_online.cpp:654-757) are the same call with the other array groups empty. */
int trs_spmm_forward_host(const trs_format* host_format, const trs_half* rhs_host, float* out_host,
                          int dimN, int mOri, int kOri, int window, int epoches, trs_timing* timing);

/* Resident-format variant for host callers: the format is uploaded once into a handle; each
 * call copies B host->device, runs, and copies C device->host. */
typedef struct trs_resident trs_resident;
int trs_resident_create(const trs_format* host_format, int mOri, int kOri, int window,
                        int max_dimN, trs_resident** out);
/* Same, over format arrays that already live on the device (e.g. a builder's output); the
 * arrays stay caller-owned and must outlive the handle. */
int trs_resident_create_device(const trs_format* dev_format, int mOri, int kOri, int window,
                               int max_dimN, trs_resident** out);
/* One call, complete on return.  The result rows travel back to the host in window chunks while
 * later chunks are still being computed.  timing (optional): h2d_ms, total_ms (kernels) and
 * d2h_ms (first to last output copy; overlaps total_ms). */
int trs_resident_forward(trs_resident* h, const trs_half* rhs_host, void* out_host, int dimN,
                         int out_dtype, trs_timing* timing);
/* The same call without the wait, for a stream of SpMMs over one matrix (the reference's callers
 * loop over spmm_forward_fp16_tcu_cuda_sptc_mma_parallel_online, mGCN_online.cpp:760, with a
 * host->device and a device->host copy in every call; no asynchronous form exists there).  The
 * handle keeps two device slots and three streams, so the input copy of call i+1 overlaps the
 * kernels and the output copy of call i.  rhs_host / out_host must stay valid, and out_host
 * unread, until trs_resident_wait returns; pinned host memory is needed for the overlap.
 * trs_resident_wait blocks until every submitted call is complete and returns the first error. */
int trs_resident_submit(trs_resident* h, const trs_half* rhs_host, void* out_host, int dimN,
                        int out_dtype);
int trs_resident_wait(trs_resident* h);
int trs_resident_destroy(trs_resident* h);

/* ---- un-packed SPTC arrays -> SpMM (compat) -------------------------------------------------
 * forward_fp16_sptc_online / forward_fp16_sptc_mma_online (mGCN_online.cpp:202-400, 404-652)
 * take s_column[G,4], s_value[G,window,2] fp32, s_pos[G,window,2] i8 and a per-group window
 * (or per-window offsets).  Host pointers; C fp32 on the host. */
int trs_sptc_unpacked_forward_host(const int32_t* s_column, const float* s_value, const int8_t* s_pos,
                                   const int32_t* s_window, const int32_t* s_offsets, int groups,
                                   int num_windows, const trs_half* rhs_host, float* out_host,
                                   int window, int dimN, int mOri, int kOri, int epoches,
                                   trs_timing* timing);

/* ---- format builder ---------------------------------------------------------------------------
 * Replaces Libra5BlockOnline.block_sptc_2to4_online (block_online.cpp:545-871): device CSR in,
 * the 29 arrays of block_online.cpp:844-870 out, bit-exact, built by GPU kernels.  `wide`,
 * `sptc_min_util` and `sptc_threshold` of the reference signature are accepted by the Python
 * shim and ignored here exactly as the reference ignores them (block_online.cpp:548-553).
 * skip_tc / unit_min_nnz carry the reference's LIBRA_SKIP_TC / LIBRA_SPTC_UNIT_MIN_NNZ
 * environment switches (block_online.cpp:564-567).  Input must be canonical CSR (columns
 * strictly ascending inside each row), which is what the reference's caller produces. */
#define TRS_BUILD_NUM_ARRAYS 29
typedef struct trs_build_config {
    int32_t part_t;      /* partSize_t: TC blocks per part                 */
    int32_t part_c;      /* partSize_c: entries per long CUDA-core part    */
    int32_t short_size;  /* shortSize: longest short CUDA-core part        */
    int32_t density;     /* minimum rows per column for a TC column        */
    int32_t window;      /* rows per window, 1..16                         */
    float tc_min_util;   /* minimum nnz / (window * 8) of a kept TC chunk  */
    int32_t skip_tc;     /* LIBRA_SKIP_TC                                  */
    int32_t unit_min_nnz;/* LIBRA_SPTC_UNIT_MIN_NNZ (reference default 2)  */
    int32_t strict;      /* 0: bit-exact with the reference, which drops the third and fourth
                          * non-zero a row has inside one 4-column group (block_online.cpp:683-695);
                          * 1: lossless — those entries join the row's CUDA-core part, so that the
                          * format encodes A exactly (arrays then differ from the reference's) */
} trs_build_config;

typedef struct trs_build_stats_t {
    long long nnz, dropped_nnz, distinct_window_columns, units;
    long long tc_nnz, csr_nnz, groups, tiles, tc_blocks;
    float build_ms; /* device time of the whole build */
} trs_build_stats_t;

typedef struct trs_builder trs_builder; /* opaque; owns the output arrays on the device */

int trs_build_create(const int32_t* rowptr, const int32_t* col, const float* values, int n_rows,
                     const trs_build_config* cfg, void* stream, trs_builder** out);
int trs_build_destroy(trs_builder* b);
/* The same build with every byte of device memory owned by the caller (the reference allocates
 * its outputs itself, block_online.cpp:844-870; a host that pools its device memory cannot let a
 * plug-in call cudaMalloc): trs_build_query gives an upper bound of the arena one build needs from
 * the matrix sizes alone; trs_build_fill builds with outputs and temporaries cut out of `arena`
 * (256-byte aligned device memory) and calls neither cudaMalloc nor cudaFree.  The builder it
 * returns points into the arena: the arrays stay valid until the caller reuses that memory;
 * trs_build_destroy frees only the small host object.  TRS_E_WORKSPACE when the arena is too small
 * (nothing is left half-built).  trs_build_arena_used reports the high-water mark of a finished
 * build, so that a caller building many matrices of one shape can size the arena from the first. */
int trs_build_query(int n_rows, long long nnz, const trs_build_config* cfg, size_t* arena_bytes);
int trs_build_fill(const int32_t* rowptr, const int32_t* col, const float* values, int n_rows,
                   const trs_build_config* cfg, void* arena, size_t arena_bytes, void* stream,
                   trs_builder** out);
int trs_build_arena_used(const trs_builder* b, size_t* bytes);
/* element counts of the 29 arrays, in the reference's return order */
int trs_build_sizes(const trs_builder* b, long long sizes[TRS_BUILD_NUM_ARRAYS]);
int trs_build_stats(const trs_builder* b, trs_build_stats_t* stats);
/* device pointer of array `id` (owned by the builder) */
const void* trs_build_array(const trs_builder* b, int id);
/* copy array `id` into caller memory (host or device) */
int trs_build_copy(const trs_builder* b, int id, void* dst, int dst_is_host, void* stream);
/* trs_format over the builder's arrays with the value arrays converted to fp16 (what
 * mdataset2_online.py:151-153 does on the host); valid until the builder is destroyed */
int trs_build_format(trs_builder* b, trs_format* out, void* stream);
/* the std::sort emulation used by the matching stage, run on the host (test hook) */
int trs_debug_stdsort_order(const unsigned char* keys, int n, int* out, int* heap_sorts);

/* ---- 2:4 matching statistics -------------------------------------------------------------------
 * Deterministic GPU versions of the reference's statistic-only matchers; device CSR in, one
 * record out (the reference returns the same numbers as a Python dict):
 *   variant 0  matching_utils.match_2to4             (block_matching_window_para_dr.cpp:361-449)
 *   variant 1  matching_utils_hash.match_2to4_hash   (block_matching_hash.cpp:373-441)
 *   variant 2  matching_utils_bucket.match_2to4_bucket (block_matching_bucket.cpp:430-499)
 *   variant 3  matching_utils_online.match_2to4_online (block_matching_online.cu:85-431, 554-649):
 *              the reference builds the window's column list in the slot order of a 2048-entry
 *              open-addressing table filled by racing threads; this is its result for the
 *              schedule in which the rows of a window insert one after the other (window = 16,
 *              columns beyond the 2048th distinct one of a window are lost, as in the reference)
 *   variant 4  matching_utils_cuda.match_2to4 (block_match_cuda.cu:822-1201, 1216-1612): the rules
 *              of the reference's multi-block kernels (hash-table compaction order, overlap <= 12,
 *              best score, search windows by window size) for the schedule in which its warps run
 *              one at a time and the window's entries are inserted in ascending column order;
 *              rows with ascending column ids are assumed.
 * dense_threshold / t_max are used by variants 0 and 3 only (the others fix their thresholds). */
typedef struct trs_match_stats {
    int32_t total_rows, total_cols;
    long long total_nnz;
    double sparsity;
    int32_t num_row_panels;
    long long num_groups;        /* "num_sptc_groups" of variant 0 */
    long long num_tc_blocks;     /* variant 0 only */
    long long num_16x16_blocks, block_padding_groups, fine_fallback, coarse_fallback, fake_zeros;
    long long tc_total_nnz, tc_block_count; /* variant 0 only */
    int32_t tc_block_max_nnz, tc_block_min_nnz;
    long long fake_zeros_exact; /* variant 1: 2*rows*groups - nnz, the per-row count block_match_cuda.cu:260-280 makes */
    long long dense_to_tc_cols, dense_to_sptc_cols; /* variants 0 and 3: pooled columns routed to TC blocks / fallback groups */
} trs_match_stats;
int trs_match24_stats(int variant, const int32_t* rowptr, const int32_t* col, int n_rows, int window,
                      int dense_threshold, int t_max, void* stream, trs_match_stats* out);

/* ---- SDDMM (no counterpart in the reference; defined by BASELINE config 3) -----------------
 * out[e] = fp16( sum_k fp32(X[row(e),k]) * fp32(Y[col(e),k]) ) for every CSR entry e.
 * The call reads rowptr[0] and rowptr[n_rows] back to the host first (one stream synchronise per
 * call; TRS_E_OFFSETS when they are not 0 / non-negative), then launches on `stream`.  The pattern
 * is not validated beyond that: the kernel never reads outside X, Y or rowptr, and an entry whose
 * column lies outside [0, n_cols) comes back as NaN.  Use the plan below for a checked pattern. */
int trs_sddmm(const int32_t* rowptr, const int32_t* col, const trs_half* X, const trs_half* Y,
              trs_half* out, int n_rows, int n_cols, int K, void* stream);
/* Planned SDDMM for a pattern that is used many times (training epochs): the plan groups the
 * entries by (16-row window, column), so that each distinct Y row of a window is gathered once
 * and the dot products run on the tensor cores (mma m16n8k16, fp32 accumulate) for K = 32, 64,
 * 128 with 16-byte aligned X / Y; other shapes run the entry-parallel kernel of trs_sddmm.  The
 * pattern must be canonical CSR (columns ascending and unique inside a row) and stay valid and
 * unchanged while the plan lives (checked at creation: TRS_E_COLUMN for a column outside
 * [0, n_cols), TRS_E_NOT_CANONICAL otherwise).  Results equal trs_sddmm's up to fp32 summation order.
 * No counterpart in the reference. */
typedef struct trs_sddmm_plan trs_sddmm_plan;
int trs_sddmm_plan_create(const int32_t* rowptr, const int32_t* col, int n_rows, int n_cols,
                          void* stream, trs_sddmm_plan** out);
int trs_sddmm_plan_run(const trs_sddmm_plan* plan, const trs_half* X, const trs_half* Y,
                       trs_half* out, int K, void* stream);
/* distinct (window, column) pairs and 8-column blocks of the plan */
int trs_sddmm_plan_info(const trs_sddmm_plan* plan, long long* n_pairs, long long* n_blocks);
int trs_sddmm_plan_destroy(trs_sddmm_plan* plan);

#ifdef __cplusplus
}
#endif
#endif /* TRSPMM_H_ */
