// Fused per-window SpMM over the reference's hybrid format, for sm_100a.
//
// One CTA owns one work item = a 16-row window (or a slice of a heavy window's k-steps) and all
// F output features of it.  A "k-step" is 16 columns of the window:
//   * a packed 2:4 tile  (s_tile_column / s_packed_a / s_packed_meta, block_online.cpp:796-841)
//     -> one mma.sp m16n8k16 per 8 features, or
//   * a pair of dense 16x8 TC blocks (t_column / t_binary / t_value, block_online.cpp:444-540)
//     -> one dense mma m16n8k16 per 8 features.
// The 16 B rows of a step are gathered with 16-byte cp.async into a padded shared-memory tile
// through a multi-stage pipeline and fed to the tensor cores with ldmatrix.trans; accumulation
// is fp32 in registers across the whole item.  The CSR remainder parts of the window
// (c_* / cs_* arrays, block_online.cpp:397-439) are added by the lanes that own the row, and C
// is written exactly once: no memset, no atomics, no second output buffer, no add kernel
// (compare mGCNkernel_online.cu:1589-1590, 1689-1712).  Heavy windows are cut into several
// items that write fp32 partial sums to scratch; a second kernel adds them in a fixed order,
// so results are bit-identical from run to run.
#include <cub/device/device_scan.cuh>

#include <string.h>

#include <mutex>
#include <vector>

#include "trs_common.cuh"

namespace trs {

constexpr int kStages = 4;
constexpr int kIdxAhead = 2 * kStages - 2;  // column ids are fetched this many steps ahead
constexpr int kIdxRing = 8;                 // slots of 16 column ids; >= kIdxAhead + 1
constexpr int kARegionBytes = 768;   // sparse: 256 B A + 32 B meta; dense: 16 rows x 48 B
constexpr int kDenseRowHalfs = 24;   // 48-byte row stride of the expanded dense A tile

struct Item {        // 32 bytes: everything a CTA needs to start, in one load
    int window;      // window id
    int step_begin;  // k-steps of the window this item covers
    int step_end;
    int slot;        // -1: write C; >=0: write partial sums to scratch slot
    int tile0;       // first packed tile of the window
    int ntiles;      // packed tiles of the window (steps [0, ntiles) are tiles, the rest TC pairs)
    int blk0;        // TC block range of the window
    int blk_end;
};

struct Heavy {
    int window;
    int slot_begin;
    int slot_end;
};

struct WindowRanges {
    int* blk_begin;  // TC block range per window
    int* blk_end;
    int* c_begin;    // long CSR parts per window
    int* c_end;
    int* cs_begin;   // short CSR parts per window
    int* cs_end;
};

struct KernelArgs {
    trs_format f;
    WindowRanges wr;
    const Item* items;
    const __half* B;
    void* C;
    float* scratch;
    const __half* tc_dense;        // [blocks][16][8] expanded TC blocks (plan-owned)
    const unsigned char* zeros;    // 512 zero bytes: source of padded (-1) columns / absent blocks
    int* status;                   // device word: non-zero after a pipeline wait gave up
    int m_rows, k_cols, window, F, out_half;
    int relu;                      // 1: C = max(A'B, 0) (GCN layer epilogue)
    void* peers[8];                // fused exchange: the fp16 rows are written into every one of these
    int n_peers;                   //   [N_total, F] buffers (this GPU's and its NVLink peers'), 0 = off
    long long peer_row0;           //   at global row peer_row0 + local row
};

// ----------------------------------------------------------------------------------------------
// plan preparation kernels
// ----------------------------------------------------------------------------------------------
__global__ void k_part_ranges(const int* __restrict__ key, const int* __restrict__ prefix, int n, int div,
                              int num_windows, int* __restrict__ begin, int* __restrict__ end, int use_prefix) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n) return;
    int w = key[p] / div;
    if (w < 0 || w >= num_windows) return;  // reported by validation
    int lo = use_prefix ? prefix[p] : p;
    int hi = use_prefix ? prefix[p + 1] : p + 1;
    if (p == 0 || key[p - 1] / div != w) begin[w] = lo;
    if (p == n - 1 || key[p + 1] / div != w) end[w] = hi;
}

__global__ void k_count_items(trs_format f, WindowRanges wr, int num_windows, int chunk, int* __restrict__ n_items,
                              int* __restrict__ n_heavy, int* __restrict__ n_slots) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= num_windows) return;
    int tiles = 0;
    if (w < f.num_windows) tiles = f.s_window_tile_offset[w + 1] - f.s_window_tile_offset[w];
    int blocks = wr.blk_end[w] - wr.blk_begin[w];
    int steps = tiles + (blocks + 1) / 2;
    int items = steps <= chunk ? 1 : (steps + chunk - 1) / chunk;
    n_items[w] = items;
    n_heavy[w] = items > 1 ? 1 : 0;
    n_slots[w] = items > 1 ? items : 0;
}

__global__ void k_fill_items(trs_format f, WindowRanges wr, int num_windows, int chunk,
                             const int* __restrict__ item_off, const int* __restrict__ heavy_off,
                             const int* __restrict__ slot_off, Item* __restrict__ items, Heavy* __restrict__ heavy) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= num_windows) return;
    int tiles = 0;
    if (w < f.num_windows) tiles = f.s_window_tile_offset[w + 1] - f.s_window_tile_offset[w];
    int blocks = wr.blk_end[w] - wr.blk_begin[w];
    int steps = tiles + (blocks + 1) / 2;
    int n = item_off[w + 1] - item_off[w];
    const int tile0 = (w < f.num_windows) ? f.s_window_tile_offset[w] : 0;
    const int blk0 = wr.blk_begin[w], blk_end = wr.blk_end[w];
    if (n == 1) {
        items[item_off[w]] = Item{w, 0, steps, -1, tile0, tiles, blk0, blk_end};
        return;
    }
    // split evenly so that no item is much shorter than the others
    int per = (steps + n - 1) / n;
    for (int i = 0; i < n; ++i) {
        int b = min(i * per, steps), e = min(b + per, steps);
        items[item_off[w] + i] = Item{w, b, e, slot_off[w] + i, tile0, tiles, blk0, blk_end};
    }
    heavy[heavy_off[w]] = Heavy{w, slot_off[w], slot_off[w] + n};
}

// Validation: every violated rule ORs one bit into *err.
enum { V_OFFSETS = 1, V_COLUMN = 2, V_ROW = 4, V_SHAPE = 8 };

__global__ void k_check_prefix(const int* __restrict__ a, int n, int expect_last, int* err) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (i == 0 && a[0] != 0) atomicOr(err, V_OFFSETS);
    if (i + 1 < n && a[i + 1] < a[i]) atomicOr(err, V_OFFSETS);
    if (i == n - 1 && expect_last >= 0 && a[i] != expect_last) atomicOr(err, V_SHAPE);
}
__global__ void k_check_range(const int* __restrict__ a, long long n, int lo, int hi, int bit, int* err) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int v = a[i];
    if (v < lo || v >= hi) atomicOr(err, bit);
}
__global__ void k_check_sorted(const int* __restrict__ a, int n, int* err) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i + 1 < n && a[i + 1] < a[i]) atomicOr(err, V_OFFSETS);
}

// ----------------------------------------------------------------------------------------------
// the fused window kernel
// ----------------------------------------------------------------------------------------------
// CSR remainder parts of the window (first item only) and the single write of the item's result:
// C rows (fp32 or fp16) or, for a slice of a split window, fp32 partial sums in scratch.
// Accumulators are in mma fragment layout: acc[n][2h + i] = row g + 8h, feature fcol + 8n + i.
__device__ __forceinline__ void add_csr_parts(float (&acc)[4][4], const Item& it, const KernelArgs& a, int fbase,
                                              int wid, int g, int t) {
    const int w = it.window;
    const size_t F = (size_t)a.F;
    // ---- CSR remainder parts: added by the first item of the window --------------------------
    if (it.step_begin == 0) {
        const int fcol = fbase + wid * 32 + 2 * t;  // + 8*n
        for (int pass = 0; pass < 2; ++pass) {
            const int pb = pass ? a.wr.cs_begin[w] : a.wr.c_begin[w];
            const int pe = pass ? a.wr.cs_end[w] : a.wr.c_end[w];
            const int* roff = pass ? a.f.cs_row_offset : a.f.c_row_offset;
            const int* rrow = pass ? a.f.cs_row : a.f.c_row;
            const int* rcol = pass ? a.f.cs_column : a.f.c_column;
            const __half* rval = (const __half*)(pass ? a.f.cs_value : a.f.c_value);
            for (int p = pb; p < pe; ++p) {
                const int lr = rrow[p] - w * a.window;
                if ((lr & 7) != g || lr < 0 || lr >= 16) continue;
                const int hi = lr >> 3;
                for (int e = roff[p]; e < roff[p + 1]; ++e) {
                    const int c = rcol[e];
                    const float v = __half2float(rval[e]);
                    const __half* brow = a.B + (size_t)c * F;
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        const int f = fcol + n * 8;
                        const float x0 = f < a.F ? v * __half2float(brow[f]) : 0.f;
                        const float x1 = f + 1 < a.F ? v * __half2float(brow[f + 1]) : 0.f;
                        if (hi) { acc[n][2] += x0; acc[n][3] += x1; }
                        else { acc[n][0] += x0; acc[n][1] += x1; }
                    }
                }
            }
        }
    }
}

__device__ __forceinline__ void finish_item(float (&acc)[4][4], const Item& it, const KernelArgs& a, int fbase,
                                            int wid, int g, int t) {
    const int w = it.window;
    const size_t F = (size_t)a.F;
    add_csr_parts(acc, it, a, fbase, wid, g, t);
    // ---- epilogue ----------------------------------------------------------------------------
    const int fcol = fbase + wid * 32 + 2 * t;
    if (it.slot >= 0) {
        float* dst = a.scratch + (size_t)it.slot * 16 * F;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const int f = fcol + n * 8;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float* d = dst + (size_t)(g + 8 * h) * F + f;
                if (f < a.F) d[0] = acc[n][2 * h];
                if (f + 1 < a.F) d[1] = acc[n][2 * h + 1];
            }
        }
        return;
    }
    if (a.relu) {
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = fmaxf(acc[n][i], 0.f);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int lr = g + 8 * h;
        const long long row = (long long)w * a.window + lr;
        if (lr >= a.window || row >= a.m_rows) continue;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            const int f = fcol + n * 8;
            if (a.out_half) {
                __half* d = (__half*)a.C + (size_t)row * F + f;
                if (f + 1 < a.F && (a.F & 1) == 0) { const __half2 hv = __floats2half2_rn(acc[n][2 * h], acc[n][2 * h + 1]); __stcs((unsigned int*)d, *(const unsigned int*)&hv); }
                else {
                    if (f < a.F) d[0] = __float2half_rn(acc[n][2 * h]);
                    if (f + 1 < a.F) d[1] = __float2half_rn(acc[n][2 * h + 1]);
                }
            } else {
                float* d = (float*)a.C + (size_t)row * F + f;
                if (f + 1 < a.F && (a.F & 1) == 0) __stcs((float2*)d, make_float2(acc[n][2 * h], acc[n][2 * h + 1]));
                else {
                    if (f < a.F) d[0] = acc[n][2 * h];
                    if (f + 1 < a.F) d[1] = acc[n][2 * h + 1];
                }
            }
        }
    }
}

// Fused exchange epilogue (fp16 rows into several [N_total, F] buffers, e.g. the hidden matrix of a
// GCN layer on every GPU of the box): the accumulators are converted once, staged as a 16 x FS
// fp16 tile in shared memory, and each thread then writes 16-byte pieces of whole rows to every
// destination — 256-byte contiguous row segments, which is what NVLink peer stores want.
// `tile` must hold 16 * (FS * 2 + 16) bytes and be free (pipeline drained, block synchronised).
template <int FS, int THREADS>
__device__ __forceinline__ void finish_item_bcast(float (&acc)[4][4], const Item& it, const KernelArgs& a, int fbase,
                                                  int wid, int g, int t, unsigned char* tile) {
    constexpr int PITCH = FS * 2 + 16;
    if (a.relu) {
#pragma unroll
        for (int n = 0; n < 4; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = fmaxf(acc[n][i], 0.f);
    }
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int h = 0; h < 2; ++h)
            *(__half2*)(tile + (g + 8 * h) * PITCH + (wid * 32 + n * 8 + 2 * t) * 2) =
                __floats2half2_rn(acc[n][2 * h], acc[n][2 * h + 1]);
    __syncthreads();
    constexpr int CPR = FS / 8;
    for (int c = threadIdx.x; c < 16 * CPR; c += THREADS) {
        const int lr = c / CPR, ch = c % CPR;
        const int f = fbase + ch * 8;
        const long long row = (long long)it.window * a.window + lr;
        if (lr >= a.window || row >= a.m_rows || f >= a.F) continue;
        const uint4 v = *(const uint4*)(tile + lr * PITCH + ch * 16);
        const size_t off = (size_t)(a.peer_row0 + row) * (size_t)a.F + f;
        for (int d = 0; d < a.n_peers; ++d) *(uint4*)((__half*)a.peers[d] + off) = v;
    }
}

template <int WARPS>
struct Tile {
    static constexpr int FS = WARPS * 32;          // features per CTA
    static constexpr int ROWB = FS * 2 + 16;       // padded B-row bytes: conflict-free ldmatrix
    static constexpr int BBYTES = 16 * ROWB;
    static constexpr int STAGE = BBYTES + kARegionBytes;
    static constexpr int SMEM = STAGE * kStages + kIdxRing * 64;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int CPR = FS / 8;             // 16-byte chunks per B row
};

template <int WARPS, bool ALIGNED>
__global__ void __launch_bounds__(WARPS * 32) k_window_spmm(const KernelArgs a) {
    using T = Tile<WARPS>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int wid = tid >> 5;
    const int g = lane >> 2;   // fragment row group
    const int t = lane & 3;    // thread in group
    const int fbase = blockIdx.y * T::FS;

    const Item it = a.items[blockIdx.x];
    const int w = it.window;
    const int tile0 = it.tile0, ntiles = it.ntiles, blk0 = it.blk0, blk_end = it.blk_end;
    const int nsteps = it.step_end - it.step_begin;
    const size_t F = (size_t)a.F;
    int* idx_ring = (int*)(smem + T::STAGE * kStages);

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    // Column ids of step m (relative to the item) -> ring slot m % kIdxRing, by threads 0..3.
    auto issue_idx = [&](int m) {
        if (tid >= 4 || m >= nsteps) return;
        const int s = it.step_begin + m;
        int* dst = idx_ring + (m % kIdxRing) * 16 + tid * 4;
        if (s < ntiles) {
            cp_async16(smem_u32(dst), a.f.s_tile_column + (size_t)(tile0 + s) * 16 + tid * 4, 16);
        } else {
            const int b = blk0 + 2 * (s - ntiles) + (tid >> 1);
            if (b < blk_end) cp_async16(smem_u32(dst), a.f.t_column + (size_t)b * 8 + (tid & 1) * 4, 16);
            else { dst[0] = -1; dst[1] = -1; dst[2] = -1; dst[3] = -1; }
        }
    };

    // each thread copies chunk (row0, ch) and (row0 + 8, ch) of every step when ALIGNED
    const int ch = tid % T::CPR;
    const int row0 = tid / T::CPR;  // 0..7

    auto issue = [&](int j) {  // j: step index relative to the item
        const int s = it.step_begin + j;
        unsigned char* st = smem + (j % kStages) * T::STAGE;
        const int* cols = idx_ring + (j % kIdxRing) * 16;
        // ---- B rows
        if (ALIGNED) {
            const int c0 = cols[row0], c1 = cols[row0 + 8];
            const int f = fbase + ch * 8;
            const bool fin = f < a.F;  // F % 8 == 0 here, so a chunk is inside or outside
            const __half* src0 = (c0 >= 0 && fin) ? a.B + (size_t)c0 * F + f : a.B;
            const __half* src1 = (c1 >= 0 && fin) ? a.B + (size_t)c1 * F + f : a.B;
            cp_async16(smem_u32(st + row0 * T::ROWB + ch * 16), src0, (c0 >= 0 && fin) ? 16 : 0);
            cp_async16(smem_u32(st + (row0 + 8) * T::ROWB + ch * 16), src1, (c1 >= 0 && fin) ? 16 : 0);
        } else {
            for (int i = tid; i < 16 * T::FS; i += T::THREADS) {
                const int r = i / T::FS, fo = i % T::FS;
                const int c = cols[r];
                __half v = __float2half(0.f);
                if (c >= 0 && fbase + fo < a.F) v = a.B[(size_t)c * F + fbase + fo];
                *(__half*)(st + r * T::ROWB + fo * 2) = v;
            }
        }
        // ---- A operand
        unsigned char* as = st + T::BBYTES;
        if (s < ntiles) {
            const size_t tile = (size_t)(tile0 + s);
            if (tid < 16) cp_async16(smem_u32(as + tid * 16), a.f.s_packed_a + tile * 64 + tid * 4, 16);
            else if (tid < 18) cp_async16(smem_u32(as + 256 + (tid - 16) * 16), a.f.s_packed_meta + tile * 8 + (tid - 16) * 4, 16);
        } else {
            const int b0 = blk0 + 2 * (s - ntiles);
            for (int i = tid; i < 256; i += T::THREADS) {
                const int r = i >> 4, k = i & 15;
                const int b = b0 + (k >> 3);
                __half v = __float2half(0.f);
                if (b < blk_end) {
                    const unsigned long long lo = (unsigned long long)a.f.t_binary[(size_t)b * 2];
                    const unsigned long long hi = (unsigned long long)a.f.t_binary[(size_t)b * 2 + 1];
                    const int bit = (r & 7) * 8 + (k & 7);
                    const unsigned long long m = r < 8 ? lo : hi;
                    if ((m >> bit) & 1ull) {
                        int rank = __popcll(m & ((1ull << bit) - 1ull));
                        if (r >= 8) rank += __popcll(lo);
                        v = ((const __half*)a.f.t_value)[(size_t)a.f.t_block_offset[b] + rank];
                    }
                }
                ((__half*)as)[r * kDenseRowHalfs + k] = v;
            }
        }
    };

    auto compute = [&](int j) {
        const int s = it.step_begin + j;
        const unsigned char* st = smem + (j % kStages) * T::STAGE;
        const unsigned char* as = st + T::BBYTES;
        // ldmatrix row address of this lane: matrix m = lane/8 -> k rows (m&1)*8.., features (m>>1)*8..
        const int m = lane >> 3;
        const int krow = (lane & 7) + (m & 1) * 8;
        const uint32_t baddr = smem_u32(st + krow * T::ROWB + (wid * 32 + (m >> 1) * 8) * 2);
        if (s < ntiles) {
            const uint2 av = *(const uint2*)(as + lane * 8);
            const uint32_t meta = *(const uint32_t*)(as + 256 + g * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_sp_16816(acc[2 * h], av.x, av.y, b0, b1, meta);
                mma_sp_16816(acc[2 * h + 1], av.x, av.y, b2, b3, meta);
            }
        } else {
            const uint32_t a0 = *(const uint32_t*)(as + g * 48 + t * 4);
            const uint32_t a1 = *(const uint32_t*)(as + (g + 8) * 48 + t * 4);
            const uint32_t a2 = *(const uint32_t*)(as + g * 48 + 16 + t * 4);
            const uint32_t a3 = *(const uint32_t*)(as + (g + 8) * 48 + 16 + t * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_16816(acc[2 * h], a0, a1, a2, a3, b0, b1);
                mma_16816(acc[2 * h + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    };

    // ---- software pipeline over the k-steps ------------------------------------------------
    // Two rings: column ids run kIdxAhead steps ahead of the compute, the gathered B rows
    // kStages-1 steps.  Group g_k (the k-th commit after the id prologue) carries the B rows of
    // step k and the ids of step k + kStages - 1; waiting until at most kStages-2 groups are
    // pending at iteration j therefore completes both the rows of step j and the ids that the
    // row gather issued in this iteration needs.
#pragma unroll
    for (int m = 0; m < kIdxAhead; ++m) issue_idx(m);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kStages - 1; ++j) {
        if (j < nsteps) issue(j);
        cp_async_commit();
    }
    for (int j = 0; j < nsteps; ++j) {
        cp_async_wait<kStages - 2>();
        __syncthreads();
        issue_idx(j + kIdxAhead);
        if (j + kStages - 1 < nsteps) issue(j + kStages - 1);
        cp_async_commit();
        compute(j);
    }
    cp_async_wait<0>();

    finish_item(acc, it, a, fbase, wid, g, t);
}

// ----------------------------------------------------------------------------------------------
// Lean variant of the cp.async kernel for the aligned case (F % 8 == 0, 16-byte aligned arrays).
// Same pipeline and numerics as k_window_spmm<WARPS, true>; what changes is the instruction
// count of the inner loop, which ncu showed to be the limiter (81 % issue-active, 131 warp
// instructions per k-step):
//   * stage and ring slots are compile-time constants (loop unrolled by the stage count),
//   * source addresses are one 32-bit multiply-add (16-byte units) plus one wide add,
//   * the dense TC operand comes pre-expanded from the plan through the same cp.async pipeline
//     (no bitmap decoding in the loop),
//   * all shared-memory addresses are hoisted out of the loop.
// ----------------------------------------------------------------------------------------------
// Shared memory of the lean kernel: the A operand of a step needs 512 bytes at most (two expanded
// TC blocks; a packed tile with its metadata is 288).  With 4 stages that would leave room for 11
// CTAs of 128 threads per SM, but holding the register allocation to the 40 registers this needs
// (a launch bound of 11, or 12 with 3 stages) was measured slower on B200 (3.80 vs 3.3 ms at R-MAT
// scale 21, 0.174 vs 0.158 ms on the clustered case): the kernel then re-computes addresses it
// otherwise keeps in registers.  So no minimum is requested (a minimum of 1 would let the compiler
// take 74 registers: 6 CTAs per SM, 3.81 ms): 48 registers, 10 CTAs per SM.
template <int WARPS, int STAGES>
struct LeanTile {
    static constexpr int FS = WARPS * 32;
    static constexpr int ROWB = FS * 2 + 16;
    static constexpr int BBYTES = 16 * ROWB;
    static constexpr int STAGE = BBYTES + 512;
    static constexpr int RING = STAGES <= 4 ? 8 : 16;   // id ring slots: a power of two above 2 * STAGES - 2
    static constexpr int SMEM = STAGE * STAGES + RING * 64;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int CPR = FS / 8;
};

template <int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32) k_window_spmm_lean(const KernelArgs a) {
    using T = LeanTile<WARPS, STAGES>;
    constexpr int kStages = STAGES;                 // shadows the file-wide stage count
    constexpr int kIdxAhead = 2 * STAGES - 2;       // column ids are fetched this many steps ahead (ring of T::RING)
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int fbase = blockIdx.y * T::FS;

    const Item it = a.items[blockIdx.x];
    const int nsteps = it.step_end - it.step_begin;
    const int nsparse = min(max(it.ntiles - it.step_begin, 0), nsteps);  // steps [0, nsparse) are packed tiles

    const uint32_t smem0 = smem_u32(smem);
    const uint32_t ring0 = smem0 + T::STAGE * kStages;
    const int* ring = (const int*)(smem + T::STAGE * kStages);

    const int ch = tid % T::CPR, row0 = tid / T::CPR;
    const uint32_t pitch16 = (uint32_t)a.F >> 3;             // 16-byte units per B row
    const uint32_t chunk16 = ((uint32_t)fbase >> 3) + ch;    // this thread's chunk inside a row
    const bool fin = fbase + ch * 8 < a.F;
    const uint4* Bq = (const uint4*)a.B;
    const uint32_t dst0 = smem0 + row0 * T::ROWB + ch * 16;
    const int mtx = lane >> 3;
    const uint32_t boff = smem0 + ((lane & 7) + (mtx & 1) * 8) * T::ROWB + (wid * 32 + (mtx >> 1) * 8) * 2;
    const unsigned char* a_lane = smem + T::BBYTES;          // + stage * STAGE

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    auto issue_idx = [&](int m) {
        if (tid < 4 && m < nsteps) {
            const int s = it.step_begin + m;
            const uint32_t dst = ring0 + (m & (T::RING - 1)) * 64 + tid * 16;
            if (s < it.ntiles) {
                cp_async16(dst, a.f.s_tile_column + (size_t)(it.tile0 + s) * 16 + tid * 4, 16);
            } else {
                const int b = it.blk0 + 2 * (s - it.ntiles) + (tid >> 1);
                if (b < it.blk_end) cp_async16(dst, a.f.t_column + (size_t)b * 8 + (tid & 1) * 4, 16);
                else *(int4*)(smem + T::STAGE * kStages + (m & (T::RING - 1)) * 64 + tid * 16) = make_int4(-1, -1, -1, -1);
            }
        }
    };

    auto issue = [&](int j, int stage) {
        const int* cols = ring + (j & (T::RING - 1)) * 16;
        const int c0 = cols[row0], c1 = cols[row0 + 8];
        const uint32_t o0 = (uint32_t)max(c0, 0) * pitch16 + chunk16;
        const uint32_t o1 = (uint32_t)max(c1, 0) * pitch16 + chunk16;
        cp_async16(dst0 + stage * T::STAGE, Bq + o0, (c0 >= 0 && fin) ? 16 : 0);
        cp_async16(dst0 + stage * T::STAGE + 8 * T::ROWB, Bq + o1, (c1 >= 0 && fin) ? 16 : 0);
        if (tid < 32) {  // A operand: warp 0
            const int s = it.step_begin + j;
            const uint32_t adst = smem0 + stage * T::STAGE + T::BBYTES + tid * 16;
            if (s < it.ntiles) {
                const size_t tile = (size_t)(it.tile0 + s);
                if (tid < 16) cp_async16(adst, a.f.s_packed_a + tile * 64 + tid * 4, 16);
                else if (tid < 18) cp_async16(adst, a.f.s_packed_meta + tile * 8 + (tid - 16) * 4, 16);
            } else {
                const int b = it.blk0 + 2 * (s - it.ntiles) + (tid >> 4);
                const bool live = b < it.blk_end;
                cp_async16(adst, a.tc_dense + (size_t)(live ? b : it.blk0) * 128 + (tid & 15) * 8, live ? 16 : 0);
            }
        }
    };

    auto compute = [&](int j, int stage) {
        const unsigned char* as = a_lane + stage * T::STAGE;
        const uint32_t baddr = boff + stage * T::STAGE;
        if (j < nsparse) {
            const uint2 av = *(const uint2*)(as + lane * 8);
            const uint32_t meta = *(const uint32_t*)(as + 256 + g * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_sp_16816(acc[2 * h], av.x, av.y, b0, b1, meta);
                mma_sp_16816(acc[2 * h + 1], av.x, av.y, b2, b3, meta);
            }
        } else {
            const uint32_t a0 = *(const uint32_t*)(as + g * 16 + t * 4);
            const uint32_t a1 = *(const uint32_t*)(as + (g + 8) * 16 + t * 4);
            const uint32_t a2 = *(const uint32_t*)(as + 256 + g * 16 + t * 4);
            const uint32_t a3 = *(const uint32_t*)(as + 256 + (g + 8) * 16 + t * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_16816(acc[2 * h], a0, a1, a2, a3, b0, b1);
                mma_16816(acc[2 * h + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    };

#pragma unroll
    for (int m = 0; m < kIdxAhead; ++m) issue_idx(m);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kStages - 1; ++j) {
        if (j < nsteps) issue(j, j);
        cp_async_commit();
    }
    for (int j0 = 0; j0 < nsteps; j0 += kStages) {
#pragma unroll
        for (int u = 0; u < kStages; ++u) {
            const int j = j0 + u;
            if (j < nsteps) {
                cp_async_wait<kStages - 2>();
                __syncthreads();
                issue_idx(j + kIdxAhead);
                if (j + kStages - 1 < nsteps) issue(j + kStages - 1, (u + kStages - 1) % kStages);
                cp_async_commit();
                compute(j, u);
            }
        }
    }
    cp_async_wait<0>();
    if (a.n_peers > 0 && it.slot < 0) {
        __syncthreads();  // every warp is done with the pipeline buffers
        add_csr_parts(acc, it, a, fbase, wid, g, t);
        finish_item_bcast<T::FS, T::THREADS>(acc, it, a, fbase, wid, g, t, smem);
        return;
    }
    finish_item(acc, it, a, fbase, wid, g, t);
}

// ----------------------------------------------------------------------------------------------
// Warp-specialised variant: one producer warp feeds the stages with bulk (TMA) copies, WARPS
// consumer warps only wait, load fragments and issue MMAs.  Per k-step the producer issues one
// 256-byte-class bulk copy per B row (lanes 0..15) plus the A operand (lanes 16, 17), all
// completing on the stage's "full" mbarrier; consumers release the stage through its "empty"
// mbarrier.  This removes the per-thread address arithmetic and the block-wide barrier of the
// cp.async variant from the inner loop, which ncu showed to be instruction-issue bound.
// Requirements (checked by the launcher): F % 8 == 0 and 16-byte aligned B and format arrays.
// Every mbarrier wait is bounded; on a timeout the CTA records it in *status and stops.
// ----------------------------------------------------------------------------------------------
constexpr int kBulkStages = 6;

template <int WARPS>
struct BulkTile {
    static constexpr int FS = WARPS * 32;
    static constexpr int ROWB = FS * 2 + 16;
    static constexpr int BBYTES = 16 * ROWB;
    static constexpr int ABYTES = 512;  // sparse: 256 B A + 32 B meta; dense: two 16x8 blocks
    static constexpr int STAGE = BBYTES + ABYTES;
    static constexpr int IDS_OFF = STAGE * kBulkStages;
    static constexpr int BAR_OFF = IDS_OFF + 1024;
    static constexpr int SMEM = BAR_OFF + 16 * kBulkStages;
    static constexpr int THREADS = (WARPS + 1) * 32;
};

template <int WARPS>
__global__ void __launch_bounds__((WARPS + 1) * 32) k_window_spmm_bulk(const KernelArgs a) {
    using T = BulkTile<WARPS>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int wid = tid >> 5;
    const int fbase = blockIdx.y * T::FS;

    const Item it = a.items[blockIdx.x];
    const int tile0 = it.tile0, ntiles = it.ntiles, blk0 = it.blk0, blk_end = it.blk_end;
    const int nsteps = it.step_end - it.step_begin;
    const size_t F = (size_t)a.F;
    const uint32_t full0 = smem_u32(smem + T::BAR_OFF);
    const uint32_t empty0 = full0 + 8 * kBulkStages;

    if (tid == 0) {
        for (int s = 0; s < kBulkStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, WARPS);
        }
        mbar_init_fence();
    }
    __syncthreads();

    if (wid == WARPS) {
        // ------------------------------ producer warp -----------------------------------------
        const uint32_t rowbytes = (uint32_t)min(T::FS, a.F - fbase) * 2u;
        int* ids = (int*)(smem + T::IDS_OFF);
        int4 nx0, nx1;  // this lane's share of the next 16 steps' column ids
        auto load_ids = [&](int base) {  // lane l: step base + l/2, columns (l%2)*8 .. +7
            nx0 = make_int4(-1, -1, -1, -1);
            nx1 = nx0;
            const int m = base + (lane >> 1);
            if (m >= nsteps) return;
            const int s = it.step_begin + m;
            const int4* src = nullptr;
            if (s < ntiles) src = (const int4*)(a.f.s_tile_column + (size_t)(tile0 + s) * 16 + (lane & 1) * 8);
            else {
                const int b = blk0 + 2 * (s - ntiles) + (lane & 1);
                if (b < blk_end) src = (const int4*)(a.f.t_column + (size_t)b * 8);
            }
            if (src) { nx0 = __ldg(src); nx1 = __ldg(src + 1); }
        };
        load_ids(0);
        bool ok = true;
        for (int j = 0; j < nsteps; ++j) {
            if ((j & 15) == 0) {
                __syncwarp();
                ((int4*)ids)[lane * 2] = nx0;
                ((int4*)ids)[lane * 2 + 1] = nx1;
                __syncwarp();
                load_ids(j + 16);
            }
            const int st = j % kBulkStages;
            const uint32_t ph = (uint32_t)(j / kBulkStages) & 1u;
            if (!mbar_wait_bounded(empty0 + 8 * st, ph ^ 1u)) { ok = false; break; }
            const int s = it.step_begin + j;
            unsigned char* stp = smem + st * T::STAGE;
            const uint32_t bar = full0 + 8 * st;
            const bool sparse = s < ntiles;
            if (lane == 0) mbar_arrive_expect_tx(bar, 16u * rowbytes + (sparse ? 288u : 512u));
            __syncwarp();
            if (lane < 16) {
                const int c = ids[(j & 15) * 16 + lane];
                const void* src = c >= 0 ? (const void*)(a.B + (size_t)c * F + fbase) : (const void*)a.zeros;
                bulk_g2s(smem_u32(stp + lane * T::ROWB), src, rowbytes, bar);
            } else if (lane == 16) {
                const void* src = sparse ? (const void*)(a.f.s_packed_a + (size_t)(tile0 + s) * 64)
                                         : (const void*)(a.tc_dense + (size_t)(blk0 + 2 * (s - ntiles)) * 128);
                bulk_g2s(smem_u32(stp + T::BBYTES), src, 256u, bar);
            } else if (lane == 17) {
                if (sparse) {
                    bulk_g2s(smem_u32(stp + T::BBYTES + 256), a.f.s_packed_meta + (size_t)(tile0 + s) * 8, 32u, bar);
                } else {
                    const int b = blk0 + 2 * (s - ntiles) + 1;
                    const void* src = b < blk_end ? (const void*)(a.tc_dense + (size_t)b * 128) : (const void*)a.zeros;
                    bulk_g2s(smem_u32(stp + T::BBYTES + 256), src, 256u, bar);
                }
            }
        }
        if (!ok && lane == 0) atomicExch(a.status, 1);
        return;
    }

    // ---------------------------------- consumer warps ------------------------------------------
    const int g = lane >> 2, t = lane & 3;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const int m = lane >> 3;
    const int krow = (lane & 7) + (m & 1) * 8;
    const uint32_t boff = krow * T::ROWB + (wid * 32 + (m >> 1) * 8) * 2;
    bool ok = true;
    for (int j = 0; j < nsteps; ++j) {
        const int st = j % kBulkStages;
        const uint32_t ph = (uint32_t)(j / kBulkStages) & 1u;
        if (!mbar_wait_bounded(full0 + 8 * st, ph)) { ok = false; break; }
        const unsigned char* stp = smem + st * T::STAGE;
        const unsigned char* as = stp + T::BBYTES;
        const uint32_t baddr = smem_u32(stp) + boff;
        if (it.step_begin + j < ntiles) {
            const uint2 av = *(const uint2*)(as + lane * 8);
            const uint32_t meta = *(const uint32_t*)(as + 256 + g * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_sp_16816(acc[2 * h], av.x, av.y, b0, b1, meta);
                mma_sp_16816(acc[2 * h + 1], av.x, av.y, b2, b3, meta);
            }
        } else {
            const uint32_t a0 = *(const uint32_t*)(as + g * 16 + t * 4);
            const uint32_t a1 = *(const uint32_t*)(as + (g + 8) * 16 + t * 4);
            const uint32_t a2 = *(const uint32_t*)(as + 256 + g * 16 + t * 4);
            const uint32_t a3 = *(const uint32_t*)(as + 256 + (g + 8) * 16 + t * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_16816(acc[2 * h], a0, a1, a2, a3, b0, b1);
                mma_16816(acc[2 * h + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * st);
    }
    if (!ok) {
        if (lane == 0) atomicExch(a.status, 2);
        return;
    }
    finish_item(acc, it, a, fbase, wid, g, t);
}

// Expands the bitmap + packed values of every TC block into a dense 16x8 fp16 tile.
__global__ void k_expand_tc(const long long* __restrict__ t_binary, const int* __restrict__ t_block_offset,
                            const __half* __restrict__ t_value, int blocks, __half* __restrict__ dense) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)blocks * 128) return;
    const int b = (int)(i >> 7), r = (int)((i >> 3) & 15), k = (int)(i & 7);
    const unsigned long long lo = (unsigned long long)t_binary[(size_t)b * 2];
    const unsigned long long hi = (unsigned long long)t_binary[(size_t)b * 2 + 1];
    const unsigned long long msk = r < 8 ? lo : hi;
    const int bit = (r & 7) * 8 + k;
    __half v = __float2half(0.f);
    if ((msk >> bit) & 1ull) {
        int rank = __popcll(msk & ((1ull << bit) - 1ull));
        if (r >= 8) rank += __popcll(lo);
        v = t_value[(size_t)t_block_offset[b] + rank];
    }
    dense[i] = v;
}

// ----------------------------------------------------------------------------------------------
// Persistent "flat stream" variant.  All k-steps of the matrix form one list ordered by window
// (a window's packed tiles, then its TC block pairs); the plan cuts the list into one contiguous
// chunk per resident CTA, balanced by steps plus a fixed cost per window.  A CTA streams through
// its chunk with the gather pipeline never draining: when a window ends it writes the 16 rows
// while the loads of the next windows are already in flight.  This removes the per-window
// pipeline fill / drain of the item-per-CTA kernels, which dominates for windows of a few dozen
// steps.  Per step the kernel reads an 8-byte descriptor (tile or TC-pair index, window id,
// first/last-of-window flags) that runs kMetaAhead steps ahead of the compute; column ids run
// kIdxAhead ahead and B rows kStages-1 ahead, all through cp.async groups.
// Windows cut by a chunk boundary write fp32 partial sums to two fixed scratch slots per CTA;
// k_reduce_flat adds them in chunk order (deterministic).
// ----------------------------------------------------------------------------------------------
constexpr int kMetaAhead = 10;
constexpr int kMetaRing = 16;
constexpr unsigned kDescLast = 0x80000000u, kDescFirst = 0x40000000u, kDescTc = 0x20000000u,
                   kDescTcSecond = 0x10000000u, kDescIndex = 0x0FFFFFFFu;

struct FlatArgs {
    const int2* meta;         // [S] {descriptor, window}
    const int* chunk_begin;   // [G + 1]
    int G;
};

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) k_window_spmm_flat(const KernelArgs a, const FlatArgs fa) {
    using T = Tile<WARPS>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int fbase = blockIdx.y * T::FS;
    const int chunk = blockIdx.x;
    const int g0 = fa.chunk_begin[chunk];
    const int nsteps = fa.chunk_begin[chunk + 1] - g0;
    if (nsteps <= 0) return;

    const uint32_t smem0 = smem_u32(smem);
    constexpr int RING_OFF = T::STAGE * kStages;            // ids ring: kIdxRing x 64 B
    constexpr int META_OFF = RING_OFF + kIdxRing * 64;      // meta ring: kMetaRing x 8 B
    const int* ring = (const int*)(smem + RING_OFF);
    const int2* mring = (const int2*)(smem + META_OFF);

    const int ch = tid % T::CPR, row0 = tid / T::CPR;
    const uint32_t pitch16 = (uint32_t)a.F >> 3;
    const uint32_t chunk16 = ((uint32_t)fbase >> 3) + ch;
    const bool fin = fbase + ch * 8 < a.F;
    const uint4* Bq = (const uint4*)a.B;
    const uint32_t dst0 = smem0 + row0 * T::ROWB + ch * 16;
    const int mtx = lane >> 3;
    const uint32_t boff = smem0 + ((lane & 7) + (mtx & 1) * 8) * T::ROWB + (wid * 32 + (mtx >> 1) * 8) * 2;
    const unsigned char* a_lane = smem + T::BBYTES;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    auto issue_meta = [&](int m) {
        if (tid == 0 && m < nsteps)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem0 + META_OFF + (m & (kMetaRing - 1)) * 8),
                         "l"(fa.meta + (size_t)(g0 + m)));
    };
    auto issue_idx = [&](int m) {
        if (tid < 4 && m < nsteps) {
            const unsigned desc = (unsigned)mring[m & (kMetaRing - 1)].x;
            const unsigned index = desc & kDescIndex;
            const uint32_t dst = smem0 + RING_OFF + (m & (kIdxRing - 1)) * 64 + tid * 16;
            if (!(desc & kDescTc)) {
                cp_async16(dst, a.f.s_tile_column + (size_t)index * 16 + tid * 4, 16);
            } else if (tid < 2 || (desc & kDescTcSecond)) {
                cp_async16(dst, a.f.t_column + (size_t)(index + (tid >> 1)) * 8 + (tid & 1) * 4, 16);
            } else {
                *(int4*)(smem + RING_OFF + (m & (kIdxRing - 1)) * 64 + tid * 16) = make_int4(-1, -1, -1, -1);
            }
        }
    };
    auto issue = [&](int j, int stage) {
        const int* cols = ring + (j & (kIdxRing - 1)) * 16;
        const int c0 = cols[row0], c1 = cols[row0 + 8];
        const uint32_t o0 = (uint32_t)max(c0, 0) * pitch16 + chunk16;
        const uint32_t o1 = (uint32_t)max(c1, 0) * pitch16 + chunk16;
        cp_async16(dst0 + stage * T::STAGE, Bq + o0, (c0 >= 0 && fin) ? 16 : 0);
        cp_async16(dst0 + stage * T::STAGE + 8 * T::ROWB, Bq + o1, (c1 >= 0 && fin) ? 16 : 0);
        if (tid < 32) {
            const unsigned desc = (unsigned)mring[j & (kMetaRing - 1)].x;
            const size_t index = desc & kDescIndex;
            const uint32_t adst = smem0 + stage * T::STAGE + T::BBYTES + tid * 16;
            if (!(desc & kDescTc)) {
                if (tid < 16) cp_async16(adst, a.f.s_packed_a + index * 64 + tid * 4, 16);
                else if (tid < 18) cp_async16(adst, a.f.s_packed_meta + index * 8 + (tid - 16) * 4, 16);
            } else {
                const bool live = tid < 16 || (desc & kDescTcSecond);
                cp_async16(adst, a.tc_dense + (index + (live ? (tid >> 4) : 0)) * 128 + (tid & 15) * 8, live ? 16 : 0);
            }
        }
    };
    auto compute = [&](bool dense, int stage) {
        const unsigned char* as = a_lane + stage * T::STAGE;
        const uint32_t baddr = boff + stage * T::STAGE;
        if (!dense) {
            const uint2 av = *(const uint2*)(as + lane * 8);
            const uint32_t meta = *(const uint32_t*)(as + 256 + g * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_sp_16816(acc[2 * h], av.x, av.y, b0, b1, meta);
                mma_sp_16816(acc[2 * h + 1], av.x, av.y, b2, b3, meta);
            }
        } else {
            const uint32_t a0 = *(const uint32_t*)(as + g * 16 + t * 4);
            const uint32_t a1 = *(const uint32_t*)(as + (g + 8) * 16 + t * 4);
            const uint32_t a2 = *(const uint32_t*)(as + 256 + g * 16 + t * 4);
            const uint32_t a3 = *(const uint32_t*)(as + 256 + (g + 8) * 16 + t * 4);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + h * 32, b0, b1, b2, b3);
                mma_16816(acc[2 * h], a0, a1, a2, a3, b0, b1);
                mma_16816(acc[2 * h + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    };

    // ---- prologue: three dependent fills, paid once per chunk -------------------------------------
#pragma unroll
    for (int m = 0; m < kMetaAhead; ++m) issue_meta(m);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int m = 0; m < kIdxAhead; ++m) issue_idx(m);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kStages - 1; ++j) {
        if (j < nsteps) issue(j, j);
        cp_async_commit();
    }
    bool piece_first = true;  // does the current piece contain its window's first step?  (set below)
    bool piece_open = false;
    for (int j0 = 0; j0 < nsteps; j0 += kStages) {
#pragma unroll
        for (int u = 0; u < kStages; ++u) {
            const int j = j0 + u;
            if (j < nsteps) {
                cp_async_wait<kStages - 2>();
                __syncthreads();
                issue_meta(j + kMetaAhead);
                issue_idx(j + kIdxAhead);
                if (j + kStages - 1 < nsteps) issue(j + kStages - 1, (u + kStages - 1) % kStages);
                cp_async_commit();
                const int2 mt = mring[j & (kMetaRing - 1)];
                const unsigned desc = (unsigned)mt.x;
                if (!piece_open) { piece_open = true; piece_first = (desc & kDescFirst) != 0; }
                compute((desc & kDescTc) != 0, u);
                if ((desc & kDescLast) || j == nsteps - 1) {
                    // the piece ends here: whole window -> C; otherwise a partial-sum slot
                    const bool whole = piece_first && (desc & kDescLast);
                    Item it;
                    it.window = mt.y;
                    it.step_begin = piece_first ? 0 : 1;  // only the piece with the first step adds the CSR parts
                    it.step_end = 0;
                    it.slot = whole ? -1 : (piece_first ? 2 * chunk + 1 : 2 * chunk);
                    it.tile0 = it.ntiles = it.blk0 = it.blk_end = 0;
                    finish_item(acc, it, a, fbase, wid, g, t);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int k = 0; k < 4; ++k) acc[i][k] = 0.f;
                    piece_open = false;
                }
            }
        }
    }
    cp_async_wait<0>();
}

// Windows without any k-step (empty, or CSR parts only): zeros plus the CSR parts.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) k_window_nosteps(const KernelArgs a, const int* __restrict__ windows) {
    using T = Tile<WARPS>;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    Item it;
    it.window = windows[blockIdx.x];
    it.step_begin = 0; it.step_end = 0; it.slot = -1;
    it.tile0 = it.ntiles = it.blk0 = it.blk_end = 0;
    finish_item(acc, it, a, blockIdx.y * T::FS, wid, lane >> 2, lane & 3);
}

// One block per chunk boundary: if the boundary cuts a window and is the first cut of that window,
// add the window's pieces in chunk order and write its rows.
__global__ void k_reduce_flat(const FlatArgs fa, const float* __restrict__ scratch, void* C, int F, int m_rows, int window,
                              int out_half, int relu) {
    const int c = blockIdx.x + 1;  // boundary between chunk c-1 and chunk c
    const int b = fa.chunk_begin[c];
    if (b <= fa.chunk_begin[c - 1] && c > 1) {
        // empty chunk c-1: the cut (if any) belongs to an earlier boundary with the same position
        if (fa.chunk_begin[c - 1] == b) return;
    }
    if (b >= fa.chunk_begin[fa.G]) return;
    const int2 here = fa.meta[b];
    if ((unsigned)here.x & kDescFirst) return;  // the boundary falls between two windows
    const int w = here.y;
    // first cut of this window?  the chunk before must hold the window's first step
    int cp = c - 1;
    while (cp > 0 && fa.chunk_begin[cp] == b) --cp;  // skip empty chunks at the same position
    const int pb = fa.chunk_begin[cp];
    if (fa.meta[pb].y == w && !((unsigned)fa.meta[pb].x & kDescFirst)) return;  // the window was already cut earlier
    const int per = 16 * F;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int lr = i / F, f = i % F;
        const long long row = (long long)w * window + lr;
        if (lr >= window || row >= m_rows) continue;
        float s = scratch[(size_t)(2 * cp + 1) * per + i];  // tail piece of the chunk with the first step
        for (int cc = c; cc < fa.G; ++cc) {
            const int bb = fa.chunk_begin[cc];
            if (bb >= fa.chunk_begin[cc + 1]) continue;  // empty chunk
            const int2 m2 = fa.meta[bb];
            if (m2.y != w || ((unsigned)m2.x & kDescFirst)) break;
            s += scratch[(size_t)(2 * cc) * per + i];       // head piece of a later chunk
        }
        if (relu) s = fmaxf(s, 0.f);
        if (out_half) ((__half*)C)[(size_t)row * F + f] = __float2half_rn(s);
        else ((float*)C)[(size_t)row * F + f] = s;
    }
}

// step descriptors: one thread per step
__global__ void k_fill_meta(trs_format f, WindowRanges wr, const int* __restrict__ win_step_off, int W, int S,
                            int2* __restrict__ meta) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= S) return;
    int lo = 0, hi = W;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (win_step_off[mid] <= s) lo = mid; else hi = mid; }
    const int w = lo;
    const int first = win_step_off[w], last = win_step_off[w + 1] - 1;
    const int tile0 = w < f.num_windows ? f.s_window_tile_offset[w] : 0;
    const int ntiles = w < f.num_windows ? f.s_window_tile_offset[w + 1] - tile0 : 0;
    const int local = s - first;
    unsigned desc;
    if (local < ntiles) desc = (unsigned)(tile0 + local);
    else {
        const int blk = wr.blk_begin[w] + 2 * (local - ntiles);
        desc = kDescTc | (unsigned)blk | (blk + 1 < wr.blk_end[w] ? kDescTcSecond : 0u);
    }
    if (s == first) desc |= kDescFirst;
    if (s == last) desc |= kDescLast;
    meta[s] = make_int2((int)desc, w);
}

__global__ void k_window_steps(trs_format f, WindowRanges wr, int W, int* __restrict__ steps) {
    const int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w > W) return;
    int n = 0;
    if (w < W) {
        if (w < f.num_windows) n = f.s_window_tile_offset[w + 1] - f.s_window_tile_offset[w];
        n += (wr.blk_end[w] - wr.blk_begin[w] + 1) / 2;
    }
    steps[w] = n;
}

// Adds the partial sums of a split window in slot order and writes its 16 rows of C.
struct PeerDst {
    void* ptr[8];
    int n;
    long long row0;
};

__global__ void k_reduce_heavy(const Heavy* __restrict__ heavy, const float* __restrict__ scratch, void* C, int F,
                               int m_rows, int window, int out_half, int relu, PeerDst pd) {
    const Heavy h = heavy[blockIdx.x];
    const int per = 16 * F;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int lr = i / F, f = i % F;
        const long long row = (long long)h.window * window + lr;
        if (lr >= window || row >= m_rows) continue;
        float s = 0.f;
        for (int sl = h.slot_begin; sl < h.slot_end; ++sl) s += scratch[(size_t)sl * per + i];
        if (relu) s = fmaxf(s, 0.f);
        if (pd.n > 0) {
            for (int d = 0; d < pd.n; ++d) ((__half*)pd.ptr[d])[(size_t)(pd.row0 + row) * F + f] = __float2half_rn(s);
        } else if (out_half) ((__half*)C)[(size_t)row * F + f] = __float2half_rn(s);
        else ((float*)C)[(size_t)row * F + f] = s;
    }
}

}  // namespace trs

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
using namespace trs;

struct trs_spmm_plan {
    trs_format f;
    int m_rows, k_cols, window, num_windows, chunk;
    DevBuf<int> ranges;  // 6 * num_windows
    WindowRanges wr;
    DevBuf<Item> items;
    DevBuf<Heavy> heavy;
    DevBuf<__half> tc_dense;          // expanded TC blocks for the bulk-copy kernel
    DevBuf<unsigned char> zeros;      // 512 zero bytes + the status word behind them
    int n_items, n_heavy, n_slots;
    std::vector<int> h_item_off, h_heavy_off;  // host copies of the per-window prefixes (num_windows + 1 each)
    bool bulk_ok;                     // bulk-copy kernel requested and usable
    bool arrays_aligned;              // index / tile arrays are 16-byte aligned
    // persistent flat-stream kernel
    bool flat_ok = false;
    int flat_G = 0, flat_S = 0, n_nosteps = 0;
    DevBuf<int2> step_meta;
    DevBuf<int> chunk_begin, nosteps;
};

static int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v ? atoi(v) : dflt;
}

static int validate_on_device(const trs_format& f, int m_rows, int k_cols, int window, int num_windows,
                              cudaStream_t st) {
    int* d_err = nullptr;
    TRS_CUDA(cudaMalloc(&d_err, sizeof(int)));
    cudaMemsetAsync(d_err, 0, sizeof(int), st);
    auto grid = [](long long n) { return (unsigned)((n + 255) / 256); };
    if (f.parts_t > 0) {
        k_check_prefix<<<grid(f.parts_t + 1), 256, 0, st>>>(f.t_row_offset, f.parts_t + 1, f.blocks, d_err);
        k_check_prefix<<<grid(f.blocks + 1), 256, 0, st>>>(f.t_block_offset, f.blocks + 1, -1, d_err);
        k_check_range<<<grid((long long)f.blocks * 8), 256, 0, st>>>(f.t_column, (long long)f.blocks * 8, -1, k_cols, V_COLUMN, d_err);
        k_check_range<<<grid(f.parts_t), 256, 0, st>>>(f.t_window_row, f.parts_t, 0, num_windows * 16, V_ROW, d_err);
        k_check_sorted<<<grid(f.parts_t), 256, 0, st>>>(f.t_window_row, f.parts_t, d_err);
    }
    for (int pass = 0; pass < 2; ++pass) {
        const int n = pass ? f.parts_c_short : f.parts_c;
        if (n <= 0) continue;
        const int* off = pass ? f.cs_row_offset : f.c_row_offset;
        const int* row = pass ? f.cs_row : f.c_row;
        k_check_prefix<<<grid(n + 1), 256, 0, st>>>(off, n + 1, -1, d_err);
        k_check_range<<<grid(n), 256, 0, st>>>(row, n, 0, m_rows, V_ROW, d_err);
        k_check_sorted<<<grid(n), 256, 0, st>>>(row, n, d_err);
    }
    // column ids of the CSR parts: their count is the last prefix entry, which lives on the device
    for (int pass = 0; pass < 2; ++pass) {
        const int n = pass ? f.parts_c_short : f.parts_c;
        if (n <= 0) continue;
        int last = 0;
        cudaError_t e2 = cudaMemcpyAsync(&last, (pass ? f.cs_row_offset : f.c_row_offset) + n, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (e2 == cudaSuccess) e2 = cudaStreamSynchronize(st);
        if (e2 != cudaSuccess) { cudaFree(d_err); return (int)e2; }
        if (last > 0)
            k_check_range<<<grid(last), 256, 0, st>>>(pass ? f.cs_column : f.c_column, last, 0, k_cols, V_COLUMN, d_err);
    }
    if (f.num_windows > 0) {
        k_check_prefix<<<grid(f.num_windows + 1), 256, 0, st>>>(f.s_window_tile_offset, f.num_windows + 1, f.tiles, d_err);
        if (f.tiles > 0)
            k_check_range<<<grid((long long)f.tiles * 16), 256, 0, st>>>(f.s_tile_column, (long long)f.tiles * 16, -1, k_cols, V_COLUMN, d_err);
    }
    int h_err = 0;
    cudaError_t e = cudaMemcpyAsync(&h_err, d_err, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_err);
    if (e != cudaSuccess) return (int)e;
    if (h_err & V_OFFSETS) return TRS_E_OFFSETS;
    if (h_err & V_SHAPE) return TRS_E_SHAPE;
    if (h_err & V_COLUMN) return TRS_E_COLUMN;
    if (h_err & V_ROW) return TRS_E_ROW;
    return TRS_OK;
}

// Flat-stream structures: steps per window -> prefix -> per-step descriptors; the step list is cut
// into one chunk per resident CTA, balanced by steps + a fixed cost per window end.
static int build_flat(trs_spmm_plan* p, cudaStream_t st) {
    const int W = p->num_windows;
    DevBuf<int> steps, off;
    DevBuf<unsigned char> tmp;
    int rc = steps.alloc((size_t)W + 1);
    if (!rc) rc = off.alloc((size_t)W + 1);
    auto done = [&](int code) { steps.release(); off.release(); tmp.release(); return code; };
    if (rc) return done(rc);
    k_window_steps<<<(unsigned)((W + 1 + 255) / 256), 256, 0, st>>>(p->f, p->wr, W, steps.p);
    size_t tb = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tb, steps.p, off.p, W + 1, st);
    rc = tmp.alloc(tb + 16);
    if (rc) return done(rc);
    cub::DeviceScan::ExclusiveSum(tmp.p, tb, steps.p, off.p, W + 1, st);
    std::vector<int> h_off((size_t)W + 1);
    cudaError_t e = cudaMemcpyAsync(h_off.data(), off.p, sizeof(int) * ((size_t)W + 1), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return done((int)e);
    const int S = h_off[W];
    p->flat_S = S;
    // windows without steps get their own tiny kernel
    std::vector<int> nos;
    for (int w = 0; w < W; ++w)
        if (h_off[w + 1] == h_off[w]) nos.push_back(w);
    p->n_nosteps = (int)nos.size();
    rc = p->nosteps.alloc(nos.size());
    if (rc) return done(rc);
    if (!nos.empty()) cudaMemcpyAsync(p->nosteps.p, nos.data(), sizeof(int) * nos.size(), cudaMemcpyHostToDevice, st);
    // chunk boundaries
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // one chunk per CTA that can be resident at once (the F = 128 kernel is the largest one)
    int occ = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k_window_spmm_flat<4>, 128, Tile<4>::SMEM + kMetaRing * 8);
    const int per_sm = max(1, env_int("TRS_FLAT_CTAS_PER_SM", occ > 0 ? occ : 8));
    int G = sms * per_sm;
    if (S < G * 8) G = max(1, S / 8);
    const double win_cost = (double)env_int("TRS_FLAT_WINDOW_COST", 4);
    std::vector<int> cb((size_t)G + 1, S);
    cb[0] = 0;
    if (S > 0) {
        // cost position of step s inside window w: s + win_cost * (non-empty windows finished before w)
        const double total = (double)S + win_cost * (double)(W - (int)nos.size());
        int w = 0;
        double done_windows = 0;  // non-empty windows fully before w
        for (int c = 1; c < G; ++c) {
            const double target = total * c / G;
            while (w < W && (double)h_off[w + 1] + win_cost * (done_windows + (h_off[w + 1] > h_off[w] ? 1 : 0)) <= target) {
                if (h_off[w + 1] > h_off[w]) done_windows += 1;
                ++w;
            }
            int s = w < W ? (int)(target - win_cost * done_windows) : S;
            if (w < W) s = min(max(s, h_off[w]), h_off[w + 1]);
            cb[c] = max(cb[c - 1], min(s, S));
        }
    }
    p->flat_G = G;
    rc = p->chunk_begin.alloc((size_t)G + 1);
    if (!rc) rc = p->step_meta.alloc((size_t)max(S, 1));
    if (rc) return done(rc);
    cudaMemcpyAsync(p->chunk_begin.p, cb.data(), sizeof(int) * ((size_t)G + 1), cudaMemcpyHostToDevice, st);
    if (S > 0)
        k_fill_meta<<<(unsigned)((S + 255) / 256), 256, 0, st>>>(p->f, p->wr, off.p, W, S, p->step_meta.p);
    e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return done((int)e);
    p->flat_ok = true;
    return done(0);
}

// CSR value-count checks need the last prefix entry; done with the column range check so that a
// short column array cannot be over-read: the caller states the lengths implicitly through the
// prefix arrays, exactly as the reference does (mGCN_online.cpp:982-1042 copies numel() items).
extern "C" int trs_spmm_plan_create(const trs_format* dev_format, int m_rows, int k_cols, int window, int validate,
                                    void* stream, trs_spmm_plan** out_plan) {
    if (!dev_format || !out_plan) return TRS_E_ARG;
    *out_plan = nullptr;
    if (m_rows <= 0 || k_cols <= 0) return TRS_E_ARG;
    if (window <= 0 || window > 16) return TRS_E_WINDOW;
    const trs_format& f = *dev_format;
    if (f.parts_t < 0 || f.blocks < 0 || f.parts_c < 0 || f.parts_c_short < 0 || f.num_windows < 0 || f.tiles < 0)
        return TRS_E_ARG;
    if (f.blocks > 0 && window != 16) return TRS_E_WINDOW;  // TC parts address rows as window_id * 16
    if (f.parts_t > 0 && !(f.t_row_offset && f.t_block_offset && f.t_column && f.t_value && f.t_window_row && f.t_binary))
        return TRS_E_ARG;
    if (f.parts_c > 0 && !(f.c_row_offset && f.c_row && f.c_column && f.c_value)) return TRS_E_ARG;
    if (f.parts_c_short > 0 && !(f.cs_row_offset && f.cs_row && f.cs_column && f.cs_value)) return TRS_E_ARG;
    if (f.num_windows > 0 && !f.s_window_tile_offset) return TRS_E_ARG;
    if (f.tiles > 0 && !(f.s_tile_column && f.s_packed_a && f.s_packed_meta)) return TRS_E_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return TRS_E_NO_DEVICE;

    cudaStream_t st = (cudaStream_t)stream;
    const int W = max(ceil_div(m_rows, window), f.num_windows);
    if (validate) {
        int rc = validate_on_device(f, m_rows, k_cols, window, W, st);
        if (rc != TRS_OK) return rc;
    }

    trs_spmm_plan* p = new trs_spmm_plan();
    p->f = f;
    p->m_rows = m_rows; p->k_cols = k_cols; p->window = window; p->num_windows = W;
    p->chunk = max(8, env_int("TRS_CHUNK_STEPS", 256));
    int rc = p->ranges.alloc((size_t)6 * W);
    if (rc) { delete p; return rc; }
    cudaMemsetAsync(p->ranges.p, 0, sizeof(int) * 6 * W, st);
    p->wr = WindowRanges{p->ranges.p, p->ranges.p + W, p->ranges.p + 2 * W, p->ranges.p + 3 * W,
                         p->ranges.p + 4 * W, p->ranges.p + 5 * W};
    auto grid = [](long long n) { return (unsigned)((n + 255) / 256); };
    if (f.parts_t > 0)
        k_part_ranges<<<grid(f.parts_t), 256, 0, st>>>(f.t_window_row, f.t_row_offset, f.parts_t, 16, W,
                                                        p->wr.blk_begin, p->wr.blk_end, 1);
    if (f.parts_c > 0)
        k_part_ranges<<<grid(f.parts_c), 256, 0, st>>>(f.c_row, nullptr, f.parts_c, window, W, p->wr.c_begin, p->wr.c_end, 0);
    if (f.parts_c_short > 0)
        k_part_ranges<<<grid(f.parts_c_short), 256, 0, st>>>(f.cs_row, nullptr, f.parts_c_short, window, W,
                                                              p->wr.cs_begin, p->wr.cs_end, 0);
    // counts -> exclusive scans (three arrays of W + 1)
    DevBuf<int> cnt, off;
    DevBuf<unsigned char> tmp;
    rc = cnt.alloc((size_t)3 * (W + 1));
    if (!rc) rc = off.alloc((size_t)3 * (W + 1));
    size_t tmp_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, cnt.p, off.p, W + 1, st);
    if (!rc) rc = tmp.alloc(tmp_bytes + 16);
    auto fail = [&](int code) { cnt.release(); off.release(); tmp.release(); trs_spmm_plan_destroy(p); return code; };
    if (rc) return fail(rc);
    cudaMemsetAsync(cnt.p, 0, sizeof(int) * 3 * (W + 1), st);
    k_count_items<<<grid(W), 256, 0, st>>>(f, p->wr, W, p->chunk, cnt.p, cnt.p + (W + 1), cnt.p + 2 * (W + 1));
    for (int i = 0; i < 3; ++i)
        cub::DeviceScan::ExclusiveSum(tmp.p, tmp_bytes, cnt.p + (size_t)i * (W + 1), off.p + (size_t)i * (W + 1), W + 1, st);
    int totals[3] = {0, 0, 0};
    for (int i = 0; i < 3; ++i)
        cudaMemcpyAsync(&totals[i], off.p + (size_t)i * (W + 1) + W, sizeof(int), cudaMemcpyDeviceToHost, st);
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail((int)e);
    p->n_items = totals[0]; p->n_heavy = totals[1]; p->n_slots = totals[2];
    // per-window prefixes on the host, so that a run can be restricted to a window range
    p->h_item_off.resize((size_t)W + 1);
    p->h_heavy_off.resize((size_t)W + 1);
    e = cudaMemcpy(p->h_item_off.data(), off.p, sizeof(int) * ((size_t)W + 1), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess)
        e = cudaMemcpy(p->h_heavy_off.data(), off.p + (W + 1), sizeof(int) * ((size_t)W + 1), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail((int)e);
    rc = p->items.alloc(p->n_items);
    if (!rc) rc = p->heavy.alloc(p->n_heavy);
    if (rc) return fail(rc);
    k_fill_items<<<grid(W), 256, 0, st>>>(f, p->wr, W, p->chunk, off.p, off.p + (W + 1), off.p + 2 * (W + 1),
                                           p->items.p, p->heavy.p);
    // data of the bulk-copy kernel: 512 zero bytes (+ status word) and the expanded TC blocks
    rc = p->zeros.alloc(512 + 16);
    if (!rc) rc = p->tc_dense.alloc((size_t)f.blocks * 128);
    if (rc) return fail(rc);
    cudaMemsetAsync(p->zeros.p, 0, 512 + 16, st);
    if (f.blocks > 0)
        k_expand_tc<<<grid((long long)f.blocks * 128), 256, 0, st>>>((const long long*)f.t_binary, f.t_block_offset,
                                                                      (const __half*)f.t_value, f.blocks, p->tc_dense.p);
    e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) e = cudaGetLastError();
    cnt.release(); off.release(); tmp.release();
    if (e != cudaSuccess) { trs_spmm_plan_destroy(p); return (int)e; }
    const uintptr_t align_or = (uintptr_t)f.s_tile_column | (uintptr_t)f.s_packed_a | (uintptr_t)f.s_packed_meta |
                               (uintptr_t)f.t_column;
    // The warp-specialised bulk-copy kernel is opt-in (TRS_SPMM_KERNEL=bulk): measured on B200 it
    // is slower than the cp.async kernel because 256-byte bulk copies cost ~7 cycles each in the
    // copy engine; it is kept for wider rows and as the structure a gather4 tensor copy would use.
    const char* kv = getenv("TRS_SPMM_KERNEL");
    p->arrays_aligned = (align_or & 15) == 0;
    p->bulk_ok = p->arrays_aligned && kv && strcmp(kv, "bulk") == 0;
    // The persistent flat-stream schedule is opt-in (TRS_SPMM_KERNEL=flat).  Measured on B200 it is
    // slower than one CTA per window (4.95 vs 3.23 ms at R-MAT scale 21): the gather is bound by how
    // many bytes the SM keeps in flight, the flat kernel fits 8 CTAs per SM instead of 10, and the
    // pipeline bubbles it removes were not the limiter.
    if (p->arrays_aligned && kv && strcmp(kv, "flat") == 0) {
        rc = build_flat(p, st);
        if (rc) { trs_spmm_plan_destroy(p); return rc; }
    }
    *out_plan = p;
    return TRS_OK;
}

extern "C" int trs_spmm_status(const trs_spmm_plan* p, int* status) {
    if (!p || !status) return TRS_E_ARG;
    TRS_CUDA(cudaDeviceSynchronize());
    TRS_CUDA(cudaMemcpy(status, p->zeros.p + 512, sizeof(int), cudaMemcpyDeviceToHost));
    return TRS_OK;
}

extern "C" int trs_spmm_plan_destroy(trs_spmm_plan* p) {
    if (!p) return TRS_OK;
    p->ranges.release();
    p->items.release();
    p->heavy.release();
    p->tc_dense.release();
    p->zeros.release();
    p->step_meta.release();
    p->chunk_begin.release();
    p->nosteps.release();
    delete p;
    return TRS_OK;
}

static size_t items_scratch_bytes(const trs_spmm_plan* p, int F) { return (size_t)p->n_slots * 16 * (size_t)F * sizeof(float); }
static size_t flat_scratch_bytes(const trs_spmm_plan* p, int F) {
    return p->flat_ok ? (size_t)2 * p->flat_G * 16 * (size_t)F * sizeof(float) : 0;
}
static bool flat_usable(const trs_spmm_plan* p, int F) { return p->flat_ok && p->flat_S > 0 && F % 8 == 0; }

extern "C" int trs_spmm_workspace_bytes(const trs_spmm_plan* p, int F, size_t* bytes) {
    if (!p || !bytes || F <= 0) return TRS_E_ARG;
    // the flat-stream kernel needs two slots per chunk; an unaligned B falls back to the item
    // kernels, so report what either path may ask for
    const size_t a = items_scratch_bytes(p, F), b = flat_usable(p, F) ? flat_scratch_bytes(p, F) : 0;
    *bytes = a > b ? a : b;
    return TRS_OK;
}

extern "C" int trs_spmm_static_scratch_bytes(const trs_spmm_plan* p, int F, size_t* bytes) {
    if (!p || !bytes || F <= 0) return TRS_E_ARG;
    *bytes = items_scratch_bytes(p, F);
    return TRS_OK;
}

extern "C" int trs_spmm_launches(const trs_spmm_plan* p) {
    if (!p) return 0;
    if (p->flat_ok && p->flat_S > 0) return 1 + (p->flat_G > 1 ? 1 : 0) + (p->n_nosteps > 0 ? 1 : 0);
    return p->n_heavy > 0 ? 2 : 1;
}

template <int WARPS>
static int launch_flat_kernel(const trs_spmm_plan* p, const KernelArgs& a, cudaStream_t st) {
    using T = Tile<WARPS>;
    constexpr int SMEM = T::SMEM + kMetaRing * 8;
    FlatArgs fa{p->step_meta.p, p->chunk_begin.p, p->flat_G};
    const int slabs = ceil_div(a.F, T::FS);
    TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_flat<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    k_window_spmm_flat<WARPS><<<dim3(p->flat_G, slabs), T::THREADS, SMEM, st>>>(a, fa);
    TRS_LAUNCH_CHECK();
    if (p->n_nosteps > 0) {
        k_window_nosteps<WARPS><<<dim3(p->n_nosteps, slabs), T::THREADS, 0, st>>>(a, p->nosteps.p);
        TRS_LAUNCH_CHECK();
    }
    if (p->flat_G > 1) {
        k_reduce_flat<<<p->flat_G - 1, 256, 0, st>>>(fa, a.scratch, a.C, a.F, a.m_rows, a.window, a.out_half, a.relu);
        TRS_LAUNCH_CHECK();
    }
    return TRS_OK;
}

template <int WARPS>
static int launch_bulk_kernel(const KernelArgs& a, int n_items, cudaStream_t st) {
    using T = BulkTile<WARPS>;
    dim3 grid(n_items, ceil_div(a.F, T::FS));
    TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_bulk<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
    k_window_spmm_bulk<WARPS><<<grid, T::THREADS, T::SMEM, st>>>(a);
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

template <int WARPS>
static int launch_window_kernel(const KernelArgs& a, int n_items, bool lean_ok, cudaStream_t st) {
    using T = Tile<WARPS>;
    const bool aligned = (a.F % 8 == 0) && (((uintptr_t)a.B & 15) == 0);
    dim3 grid(n_items, ceil_div(a.F, T::FS));
    static const bool use_lean = [] { const char* v = getenv("TRS_SPMM_KERNEL"); return !(v && strcmp(v, "cpasync_v1") == 0); }();
    if (aligned && lean_ok && use_lean) {
        // Three stages are the default: measured 1-2 % faster than four at R-MAT scale 21 (3.18 vs 3.23 ms,
        // 3.24 vs 3.28 ms on two boxes) and equal on the clustered case; five stages (8 CTAs per SM) and
        // 2-warp CTAs with the feature slabs on gridDim.y were slower (3.50 and 3.67 ms).
        static const int lean_stages = [] { const char* v = getenv("TRS_LEAN_STAGES"); return v && atoi(v) == 4 ? 4 : 3; }();
        if (lean_stages == 3) {
            using L = LeanTile<WARPS, 3>;
            TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_lean<WARPS, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM));
            TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_lean<WARPS, 3>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
            k_window_spmm_lean<WARPS, 3><<<grid, L::THREADS, L::SMEM, st>>>(a);
        } else {
            using L = LeanTile<WARPS, 4>;
            TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_lean<WARPS, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM));
            TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_lean<WARPS, 4>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
            k_window_spmm_lean<WARPS, 4><<<grid, L::THREADS, L::SMEM, st>>>(a);
        }
    } else if (aligned) {
        TRS_CUDA(cudaFuncSetAttribute(k_window_spmm<WARPS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
        k_window_spmm<WARPS, true><<<grid, T::THREADS, T::SMEM, st>>>(a);
    } else {
        TRS_CUDA(cudaFuncSetAttribute(k_window_spmm<WARPS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
        k_window_spmm<WARPS, false><<<grid, T::THREADS, T::SMEM, st>>>(a);
    }
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

extern "C" int trs_spmm_run(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, void* workspace,
                            size_t workspace_bytes, void* stream) {
    return trs_spmm_run_ex(p, B, C, F, out_dtype, 0, workspace, workspace_bytes, stream);
}

static int run_impl(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags, void* workspace,
                    size_t workspace_bytes, void* stream, bool items_only, void* const* peers = nullptr, int n_peers = 0,
                    long long peer_row0 = 0, int w0 = 0, int w1 = -1);

extern "C" int trs_spmm_run_ex(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags,
                               void* workspace, size_t workspace_bytes, void* stream) {
    return run_impl(p, B, C, F, out_dtype, flags, workspace, workspace_bytes, stream, false);
}

extern "C" int trs_spmm_run_windows(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags,
                                    void* workspace, size_t workspace_bytes, void* stream, int window_begin,
                                    int window_end) {
    if (window_end < 0) return TRS_E_ARG;
    return run_impl(p, B, C, F, out_dtype, flags, workspace, workspace_bytes, stream, /*items_only=*/true, nullptr, 0, 0,
                    window_begin, window_end);
}

extern "C" int trs_spmm_num_windows(const trs_spmm_plan* p) { return p ? p->num_windows : TRS_E_ARG; }

extern "C" int trs_spmm_run_bcast(const trs_spmm_plan* p, const trs_half* B, void* const* dst, int n_dst, long long row0,
                                  int F, int flags, void* workspace, size_t workspace_bytes, void* stream) {
    if (!p || !dst || n_dst < 1 || n_dst > 8 || row0 < 0) return TRS_E_ARG;
    for (int d = 0; d < n_dst; ++d)
        if (!dst[d] || ((uintptr_t)dst[d] & 15)) return TRS_E_ARG;
    if (F % 8 != 0 || ((uintptr_t)B & 15) || !p->arrays_aligned) return TRS_E_ARG;  // the 16-byte row pieces need it
    return run_impl(p, B, dst[0], F, TRS_OUT_F16, flags, workspace, workspace_bytes, stream, /*items_only=*/true, dst, n_dst, row0);
}

static int run_impl(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags, void* workspace,
                    size_t workspace_bytes, void* stream, bool items_only, void* const* peers, int n_peers,
                    long long peer_row0, int w0, int w1) {
    if (!p || !B || !C || F <= 0) return TRS_E_ARG;
    if (w1 < 0) w1 = p->num_windows;
    if (w0 < 0 || w0 > w1 || w1 > p->num_windows) return TRS_E_ARG;
    if (w0 == w1) return TRS_OK;
    // window range -> item / split-window ranges (both lists are in window order)
    const int i0 = p->h_item_off[w0], n_items = p->h_item_off[w1] - i0;
    const int h0 = p->h_heavy_off[w0], n_heavy = p->h_heavy_off[w1] - h0;
    if (flags & ~TRS_EPILOGUE_RELU) return TRS_E_ARG;
    if (out_dtype != TRS_OUT_F32 && out_dtype != TRS_OUT_F16) return TRS_E_ARG;
    const bool flat = !items_only && w0 == 0 && w1 == p->num_windows && flat_usable(p, F) && (((uintptr_t)B & 15) == 0);
    size_t need = flat ? flat_scratch_bytes(p, F) : items_scratch_bytes(p, F);
    if (flat && p->flat_G <= 1) need = 0;
    if (need > 0 && (!workspace || workspace_bytes < need)) return TRS_E_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    KernelArgs a;
    a.f = p->f; a.wr = p->wr; a.items = p->items.p + i0;
    a.B = (const __half*)B; a.C = C; a.scratch = (float*)workspace;
    a.m_rows = p->m_rows; a.k_cols = p->k_cols; a.window = p->window; a.F = F; a.out_half = out_dtype == TRS_OUT_F16;
    a.relu = (flags & TRS_EPILOGUE_RELU) ? 1 : 0;
    a.n_peers = n_peers; a.peer_row0 = peer_row0;
    for (int d = 0; d < 8; ++d) a.peers[d] = d < n_peers ? peers[d] : nullptr;
    a.tc_dense = p->tc_dense.p; a.zeros = p->zeros.p; a.status = (int*)(p->zeros.p + 512);
    int rc;
    if (flat) {
        if (F <= 32) return launch_flat_kernel<1>(p, a, st);
        if (F <= 64) return launch_flat_kernel<2>(p, a, st);
        return launch_flat_kernel<4>(p, a, st);
    }
    const bool bulk = p->bulk_ok && n_peers == 0 && (F % 8 == 0) && (((uintptr_t)B & 15) == 0);
    if (bulk) {
        if (F <= 32) rc = launch_bulk_kernel<1>(a, n_items, st);
        else if (F <= 64) rc = launch_bulk_kernel<2>(a, n_items, st);
        else rc = launch_bulk_kernel<4>(a, n_items, st);  // F > 128: feature slabs of 128 on gridDim.y
    } else if (F <= 32) rc = launch_window_kernel<1>(a, n_items, p->arrays_aligned, st);
    else if (F <= 64) rc = launch_window_kernel<2>(a, n_items, p->arrays_aligned, st);
    else rc = launch_window_kernel<4>(a, n_items, p->arrays_aligned, st);
    if (rc) return rc;
    if (n_heavy > 0) {
        PeerDst pd;
        pd.n = a.n_peers; pd.row0 = a.peer_row0;
        for (int d = 0; d < 8; ++d) pd.ptr[d] = a.peers[d];
        k_reduce_heavy<<<n_heavy, 256, 0, st>>>(p->heavy.p + h0, (const float*)workspace, C, F, p->m_rows, p->window, a.out_half, a.relu, pd);
        TRS_LAUNCH_CHECK();
    }
    return TRS_OK;
}

// ----------------------------------------------------------------------------------------------
// SpMM without any allocation: partial sums in a fixed, library-owned device array
// ----------------------------------------------------------------------------------------------
// Some hosts cannot give this library scratch memory at call time: applications that hand the
// whole device memory to their own pool at start-up (a later cudaMalloc from a plug-in fails or
// fragments that pool) and latency-critical loops in which cudaMalloc / cudaFree would stall
// every stream of the device.  For them trs_spmm_run_static runs the window-per-CTA kernels
// (k_window_spmm_lean / k_window_spmm + k_reduce_heavy), whose scratch need is small and known
// from the plan, with the partial sums of split windows kept in the array below instead of a
// caller-provided workspace.  Every GPU that loads the library holds these bytes until exit.
//
// In host code the array's name is only a stand-in for the symbol; the device address is asked
// for once per device (cudaGetSymbolAddress with that device current) and cached.
static __device__ __align__(256) unsigned char g_static_scratch[TRS_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};
bool g_static_scratch_ready[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;
}  // namespace

extern "C" int trs_spmm_run_static(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype,
                                   void* stream) {
    if (!p || !B || !C || F <= 0) return TRS_E_ARG;
    const size_t need = (size_t)p->n_slots * 16 * (size_t)F * sizeof(float);
    if (need > (size_t)TRS_STATIC_SCRATCH_BYTES) return TRS_E_LIMIT;
    int dev = -1;
    TRS_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return TRS_E_LIMIT;
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_ready[dev]) {  // first call on this device: look the symbol up
            void* ptr = nullptr;
            TRS_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
            g_static_scratch_ptr[dev] = ptr;
            g_static_scratch_ready[dev] = true;
        }
        scratch = g_static_scratch_ptr[dev];
    }
    // Nothing in the array has to start at zero: every slot a call reads is first written in
    // full by that call's window kernel.
    return run_impl(p, B, C, F, out_dtype, 0, scratch, (size_t)TRS_STATIC_SCRATCH_BYTES, stream, /*items_only=*/true);
}
