// Fused per-window SpMM over the reference's hybrid format, for sm_100a.
//
// One work item = a 16-row window (or a slice of a heavy window's k-steps) and up to 128 output
// features of it.  A "k-step" is 16 columns of the window:
//   * a packed 2:4 tile  (s_tile_column / s_packed_a / s_packed_meta, block_online.cpp:796-841)
//     -> one mma.sp m16n8k16 per 8 features, or
//   * a pair of dense 16x8 TC blocks (t_column / t_binary / t_value, block_online.cpp:444-540)
//     -> one dense mma m16n8k16 per 8 features, or
//   * 16 entries of the window's CSR remainder -> one dense mma m16n8k16 per 8 features.
// The default kernel gives every item to ONE warp: the warp gathers the 16 B rows of a step with
// 16-byte cp.async into its own shared-memory ring, feeds them to the tensor cores with
// ldmatrix.trans and keeps the fp32 accumulators of all 16 x FS outputs in registers across the
// item.  No block-wide barrier exists anywhere in the loop; measured on B200, the barrier per
// k-step of a CTA-cooperative gather, not the bytes in flight, was what held the gather rate at
// 8.7 TB/s where warp-private rings reach 14 TB/s on the same column stream.
// The CSR remainder parts of the window (c_* / cs_* arrays, block_online.cpp:397-439; kernels
// mGCNkernel.cu:976-1042, 1119-1171) run through the same pipeline: the plan expands them into
// groups of 16 entries, a group's 16 columns are gathered like a tile's and multiplied by a
// 16 x 16 A tile holding entry k in column k (the fallback kernel for unaligned operands adds
// them with scalar loads instead), and C is written exactly once:
// no memset, no atomics, no second output buffer, no add kernel (compare
// mGCNkernel_online.cu:1589-1590, 1689-1712).  Heavy windows are cut into several items that
// write fp32 partial sums to scratch; a second kernel adds them in a fixed order, so results are
// bit-identical from run to run.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <string.h>

#include <mutex>
#include <vector>

#include "trs_common.cuh"

namespace trs {

constexpr int kStages = 4;           // CTA-cooperative kernels (fallback for unaligned inputs)
constexpr int kIdxAhead = 2 * kStages - 2;  // column ids are fetched this many steps ahead
constexpr int kIdxRing = 8;                 // slots of 16 column ids; >= kIdxAhead + 1
constexpr int kARegionBytes = 768;   // sparse: 256 B A + 32 B meta; dense: 16 rows x 48 B
constexpr int kDenseRowHalfs = 24;   // 48-byte row stride of the expanded dense A tile

struct Item {        // 64 bytes: everything a warp / CTA needs to start
    int window;      // window id
    int step_begin;  // k-steps of the window this item covers
    int step_end;
    int slot;        // -1: write C; >=0: write partial sums to scratch slot
    int tile0;       // first packed tile of the window
    int ntiles;      // packed tiles of the window (steps [0, ntiles) are tiles, the rest TC pairs)
    int blk0;        // TC block range of the window
    int blk_end;
    int c_begin;     // long CSR parts this item adds (a split window's parts are spread over its items)
    int c_end;
    int cs_begin;    // short CSR parts this item adds
    int cs_end;
    int ce0;         // the same CSR entries as groups of 16 (plan-owned expansion): first group, count
    int ce_n;
    int pad[2];
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
    int* ce_begin;   // first group of 16 expanded CSR entries per window ([W + 1], exclusive scan of ce_count)
    int* ce_count;
};

struct KernelArgs {
    trs_format f;
    const Item* items;
    int n_items;
    const __half* B;
    void* C;
    float* scratch;
    const __half* tc_dense;        // [blocks][16][8] expanded TC blocks (plan-owned)
    const int* ce_col;             // [groups][16] column ids of the CSR remainder entries, -1 = padding (plan-owned)
    const unsigned* ce_rv;         // [groups][16] fp16 value | local row << 16
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

// CSR remainder entries of a window (long parts first, then short parts), expanded at plan time
// into groups of 16 entries - column id and (fp16 value, local row) - so that the warp kernel can
// run them through its gather pipeline as k-steps of their own: 16 gathered B rows times a
// 16 x 16 A tile that holds entry k in column k (one non-zero per column).
__global__ void k_ce_count(trs_format f, WindowRanges wr, int num_windows) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w > num_windows) return;
    int n = 0;
    if (w < num_windows) {
        if (wr.c_end[w] > wr.c_begin[w]) n += f.c_row_offset[wr.c_end[w]] - f.c_row_offset[wr.c_begin[w]];
        if (wr.cs_end[w] > wr.cs_begin[w]) n += f.cs_row_offset[wr.cs_end[w]] - f.cs_row_offset[wr.cs_begin[w]];
    }
    wr.ce_count[w] = n > 0 ? (n + 15) / 16 : 0;
}
__global__ void k_ce_fill(trs_format f, WindowRanges wr, int num_windows, int window, int pass, long long capacity,
                          int* __restrict__ ce_col, unsigned* __restrict__ ce_rv) {
    const int n = pass ? f.parts_c_short : f.parts_c;
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n) return;
    const int* roff = pass ? f.cs_row_offset : f.c_row_offset;
    const int* rrow = pass ? f.cs_row : f.c_row;
    const int* rcol = pass ? f.cs_column : f.c_column;
    const __half* rval = (const __half*)(pass ? f.cs_value : f.c_value);
    const int w = rrow[p] / window;
    if (w < 0 || w >= num_windows) return;  // reported by validation
    const int lr = rrow[p] - w * window;
    long long dst = (long long)wr.ce_begin[w] * 16 + (roff[p] - (pass ? f.cs_row_offset[wr.cs_begin[w]] : f.c_row_offset[wr.c_begin[w]]));
    if (pass && wr.c_end[w] > wr.c_begin[w]) dst += f.c_row_offset[wr.c_end[w]] - f.c_row_offset[wr.c_begin[w]];
    for (int e = roff[p]; e < roff[p + 1]; ++e, ++dst) {
        if (dst < 0 || dst >= capacity) return;
        ce_col[dst] = rcol[e];
        ce_rv[dst] = (unsigned)__half_as_ushort(rval[e]) | ((unsigned)lr << 16);
    }
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
    const int cb = wr.c_begin[w], cn = wr.c_end[w] - cb, sb = wr.cs_begin[w], sn = wr.cs_end[w] - sb;
    const int g0 = wr.ce_begin[w], gn = wr.ce_count[w];
    if (n == 1) {
        items[item_off[w]] = Item{w, 0, steps, -1, tile0, tiles, blk0, blk_end, cb, cb + cn, sb, sb + sn, g0, gn, {0, 0}};
        return;
    }
    // split evenly so that no item is much shorter than the others; the window's CSR parts are
    // spread over the items the same way
    int per = (steps + n - 1) / n;
    for (int i = 0; i < n; ++i) {
        int b = min(i * per, steps), e = min(b + per, steps);
        items[item_off[w] + i] = Item{w, b, e, slot_off[w] + i, tile0, tiles, blk0, blk_end,
                                      cb + (int)((long long)cn * i / n), cb + (int)((long long)cn * (i + 1) / n),
                                      sb + (int)((long long)sn * i / n), sb + (int)((long long)sn * (i + 1) / n),
                                      g0 + (int)((long long)gn * i / n),
                                      (int)((long long)gn * (i + 1) / n) - (int)((long long)gn * i / n), {0, 0}};
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
// Launch-order class of an item: long items first, so that the last wave of the grid consists of
// short ones (one item per warp: a long item that starts late would keep its SM busy alone).
__global__ void k_item_class(const Item* __restrict__ items, int n, unsigned char* __restrict__ cls) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int steps = items[i].step_end - items[i].step_begin + items[i].ce_n;
    cls[i] = (unsigned char)(31 - min(steps, 255) / 8);   // 32 classes of 8 steps (four classes measured 4 - 6 % slower, 64 or 256 the same)
}

// The TC kernels read t_value[t_block_offset[b] + rank] with rank taken from the block's two
// bitmaps, so the bitmaps' population must equal the block's share of t_value.
__global__ void k_check_tc_popcount(const long long* __restrict__ t_binary, const int* __restrict__ t_block_offset,
                                    int blocks, int* err) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const int bits = __popcll((unsigned long long)t_binary[2 * (size_t)b]) + __popcll((unsigned long long)t_binary[2 * (size_t)b + 1]);
    if (bits != t_block_offset[b + 1] - t_block_offset[b]) atomicOr(err, V_SHAPE);
}
__global__ void k_check_sorted(const int* __restrict__ a, int n, int* err) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i + 1 < n && a[i + 1] < a[i]) atomicOr(err, V_OFFSETS);
}

// ----------------------------------------------------------------------------------------------
// CTA-cooperative kernels
// ----------------------------------------------------------------------------------------------
// CSR remainder parts of the item and the single write of the item's result:
// C rows (fp32 or fp16) or, for a slice of a split window, fp32 partial sums in scratch.
// Accumulators are in mma fragment layout: acc[n][2h + i] = row g + 8h, feature fcol + 8n + i.
__device__ __forceinline__ void add_csr_parts(float (&acc)[4][4], const Item& it, const KernelArgs& a, int fbase,
                                              int wid, int g, int t) {
    const int w = it.window;
    const size_t F = (size_t)a.F;
    // ---- CSR remainder parts of this item (scalar loop: this path serves unaligned inputs only) ---
    {
        const int fcol = fbase + wid * 32 + 2 * t;  // + 8*n
        for (int pass = 0; pass < 2; ++pass) {
            const int pb = pass ? it.cs_begin : it.c_begin;
            const int pe = pass ? it.cs_end : it.c_end;
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

template <int WARPS>
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


    auto issue = [&](int j) {  // j: step index relative to the item
        const int s = it.step_begin + j;
        unsigned char* st = smem + (j % kStages) * T::STAGE;
        const int* cols = idx_ring + (j % kIdxRing) * 16;
        // ---- B rows: plain 2-byte loads (any alignment, any F)
        for (int i = tid; i < 16 * T::FS; i += T::THREADS) {
            const int r = i / T::FS, fo = i % T::FS;
            const int c = cols[r];
            __half v = __float2half(0.f);
            if (c >= 0 && fbase + fo < a.F) v = a.B[(size_t)c * F + fbase + fo];
            *(__half*)(st + r * T::ROWB + fo * 2) = v;
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
// Default kernel: one warp per work item, no block-wide synchronisation.
// ----------------------------------------------------------------------------------------------
// FS = features per warp (32 / 64 / 128; F > FS adds feature slabs on gridDim.y).  Per k-step the
// warp copies the 16 gathered rows (FS * 2 bytes each) with 16 / (256 / FS) cp.async instructions
// of 16 bytes per lane into a stage of its own ring - rows unpadded, the 16-byte chunks of a row
// swizzled by the row number so that ldmatrix is conflict-free - and the column ids of a later
// step into a small id ring.  The A operand (8 bytes of packed values and one metadata word per
// lane, or the four fragment words of two expanded TC blocks) is a coalesced stream read once; it
// goes straight into registers STAGES - 1 steps ahead, so the ring holds gathered rows only:
// 3 x 4 KB + 256 B per warp at FS = 128, which lets 16 one-warp CTAs (four per scheduler, 128
// registers each) share an SM - shared memory would take 17, but the fifth warp of one scheduler
// would cap every warp at 96 registers, which measured slower.  Commit groups give the ordering
// (see the group accounting at the loop); lanes meet in one __syncwarp per step.
// Requirements (checked by the launcher): F % 8 == 0, B / C / scratch and the tile arrays 16-byte
// aligned.
template <int FS, int STAGES>
struct WarpTile {
    static constexpr int NT = FS / 8;               // n-tiles (8 features) per warp
    static constexpr int CPR = FS / 8;              // 16-byte chunks per gathered row
    static constexpr int RPI = 32 / CPR;            // rows one cp.async warp-instruction covers
    static constexpr int NCP = 16 / RPI;            // cp.async instructions per lane and step
    static constexpr int ROWB = FS * 2;             // no padding: the chunks of a row are swizzled
    static constexpr int STAGE = 16 * ROWB;         // the B rows only; the A operand rides in registers
    static constexpr int IDA = 2 * STAGES - 2;      // ids run this many steps ahead
    static constexpr int RING = IDA <= 4 ? 4 : 8;   // id ring slots (64 B each), >= IDA
    static constexpr int SMEM = STAGE * STAGES + RING * 64;
    static_assert(STAGES >= 2 && STAGES <= 4, "id ring holds 8 steps");
    static_assert(SMEM >= 16 * (FS * 4 + 16), "the epilogue stages a 16 x FS fp32 tile in the ring");
    // chunk c of row r sits at position c ^ swz(r): the 8 rows one ldmatrix phase reads land in 8
    // different 16-byte bank groups (rows of 64 B share a 128-byte line in pairs)
    __device__ static constexpr int swz(int r) { return FS == 32 ? ((r >> 1) & 3) : (r & 7); }
};

// Epilogue of a warp-owned item.  Accumulators are in mma fragment layout: acc[n][2h + i] = row
// g + 8h, feature fbase + 8n + 2t + i.  The result tile is staged in the warp's (drained) ring and
// leaves in 16-byte pieces of whole rows: fp32 partial sums to a scratch slot, or fp16 / fp32
// rows of C, or fp16 rows into every peer buffer of the fused exchange.
template <int FS>
__device__ __forceinline__ void finish_item_warp(float (&acc)[FS / 8][4], const Item& it, const KernelArgs& a, int fbase,
                                                 int lane, unsigned char* ring) {
    constexpr int NT = FS / 8;
    const int g = lane >> 2, t = lane & 3;
    const bool partial = it.slot >= 0;
    if (a.relu && !partial) {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = fmaxf(acc[n][i], 0.f);
    }
    const bool half_out = !partial && (a.out_half || a.n_peers > 0);
    if (half_out) {
        constexpr int PITCH = FS * 2 + 16;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int h = 0; h < 2; ++h)
                *(__half2*)(ring + (g + 8 * h) * PITCH + (8 * n + 2 * t) * 2) = __floats2half2_rn(acc[n][2 * h], acc[n][2 * h + 1]);
        __syncwarp();
        constexpr int CPR = FS / 8;
        for (int c = lane; c < 16 * CPR; c += 32) {
            const int lr = c / CPR, ch = c % CPR;
            const int f = fbase + ch * 8;
            const long long row = (long long)it.window * a.window + lr;
            if (lr >= a.window || row >= a.m_rows || f >= a.F) continue;
            const uint4 v = *(const uint4*)(ring + lr * PITCH + ch * 16);
            if (a.n_peers > 0) {
                const size_t off = (size_t)(a.peer_row0 + row) * (size_t)a.F + f;
                for (int d = 0; d < a.n_peers; ++d) *(uint4*)((__half*)a.peers[d] + off) = v;
            } else {
                __stcs((uint4*)((__half*)a.C + (size_t)row * a.F + f), v);
            }
        }
    } else {
        constexpr int PITCH = FS * 4 + 16;
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int h = 0; h < 2; ++h)
                *(float2*)(ring + (g + 8 * h) * PITCH + (8 * n + 2 * t) * 4) = make_float2(acc[n][2 * h], acc[n][2 * h + 1]);
        __syncwarp();
        constexpr int CPR = FS / 4;
        float* dst = partial ? a.scratch + (size_t)it.slot * 16 * (size_t)a.F : (float*)a.C;
        for (int c = lane; c < 16 * CPR; c += 32) {
            const int lr = c / CPR, ch = c % CPR;
            const int f = fbase + ch * 4;
            const long long row = (long long)it.window * a.window + lr;
            if (f >= a.F) continue;
            if (!partial && (lr >= a.window || row >= a.m_rows)) continue;
            const float4 v = *(const float4*)(ring + lr * PITCH + ch * 16);
            float4* d = (float4*)(dst + (partial ? (size_t)lr : (size_t)row) * a.F + f);
            if (partial) *d = v;
            else __stcs(d, v);
        }
    }
}

template <int FS, int STAGES, int MINB>
__global__ void __launch_bounds__(32, MINB) k_window_spmm_warp(const KernelArgs a) {
    using T = WarpTile<FS, STAGES>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x;
    const int g = lane >> 2;
    const int fbase = blockIdx.y * FS;

    const Item it = a.items[blockIdx.x];
    const int nmain = it.step_end - it.step_begin;
    const int nsparse = min(max(it.ntiles - it.step_begin, 0), nmain);   // steps [0, nsparse) are packed tiles,
    const int nsteps = nmain + it.ce_n;                                  // [nsparse, nmain) TC pairs, the rest CSR groups

    const uint32_t smem0 = smem_u32(smem);
    const uint32_t ring0 = smem0 + T::STAGE * STAGES;
    const unsigned char* ringp = smem + T::STAGE * STAGES;

    // gather role of this lane: chunk `ch` of rows sub * NCP + k, k = 0 .. NCP-1
    const int ch = lane % T::CPR, sub = lane / T::CPR;
    const uint32_t pitch16 = (uint32_t)a.F >> 3;             // 16-byte units per B row
    const uint32_t chunk16 = ((uint32_t)fbase >> 3) + ch;    // this lane's chunk inside a row
    const bool fin = fbase + ch * 8 < a.F;
    const uint4* Bq = (const uint4*)a.B;
    const uint32_t dst0 = smem0 + (sub * T::NCP) * T::ROWB;
    // ldmatrix role: matrix lane / 8 -> k rows (m & 1) * 8 .., features (m >> 1) * 8 ..
    const int mtx = lane >> 3;
    const int lrow = (lane & 7) + (mtx & 1) * 8;
    const uint32_t boff = smem0 + lrow * T::ROWB;
    const int lswz = T::swz(lrow), lchunk = mtx >> 1;
    const int t = lane & 3;

    float acc[T::NT][4];
#pragma unroll
    for (int i = 0; i < T::NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    auto issue_idx = [&](int m) {
        if (lane < 4 && m < nsteps) {
            const int s = it.step_begin + m;
            const uint32_t dst = ring0 + (m & (T::RING - 1)) * 64 + lane * 16;
            if (m >= nmain) {
                cp_async16(dst, a.ce_col + (size_t)(it.ce0 + m - nmain) * 16 + lane * 4, 16);
            } else if (s < it.ntiles) {
                cp_async16(dst, a.f.s_tile_column + (size_t)(it.tile0 + s) * 16 + lane * 4, 16);
            } else {
                const int b = it.blk0 + 2 * (s - it.ntiles) + (lane >> 1);
                if (b < it.blk_end) cp_async16(dst, a.f.t_column + (size_t)b * 8 + (lane & 1) * 4, 16);
                else *(int4*)(smem + T::STAGE * STAGES + (m & (T::RING - 1)) * 64 + lane * 16) = make_int4(-1, -1, -1, -1);
            }
        }
    };

    auto issue = [&](int j, int stage) {
        const int* cols = (const int*)(ringp + (j & (T::RING - 1)) * 64) + sub * T::NCP;
        int c[T::NCP];
        if constexpr (T::NCP == 8) {
            const int4 x = *(const int4*)cols, y = *(const int4*)(cols + 4);
            c[0] = x.x; c[1] = x.y; c[2] = x.z; c[3] = x.w;
            c[4] = y.x; c[5] = y.y; c[6] = y.z; c[7] = y.w;
        } else if constexpr (T::NCP == 4) {
            const int4 x = *(const int4*)cols;
            c[0] = x.x; c[1] = x.y; c[2] = x.z; c[3] = x.w;
        } else {
            const int2 x = *(const int2*)cols;
            c[0] = x.x; c[1] = x.y;
        }
        const uint32_t d = dst0 + stage * T::STAGE;
#pragma unroll
        for (int k = 0; k < T::NCP; ++k) {
            const uint32_t o = (uint32_t)max(c[k], 0) * pitch16 + chunk16;
            cp_async16(d + k * T::ROWB + ((ch ^ T::swz(sub * T::NCP + k)) << 4), Bq + o, (c[k] >= 0 && fin) ? 16 : 0);
        }
    };

    // A operand of step j, straight into registers (a coalesced stream, read once): a packed tile
    // gives this lane its 8 bytes of values (x, y) and its metadata word (z); a pair of TC blocks
    // gives the four fragment words of the dense 16 x 16 tile
    auto load_a = [&](int j) -> uint4 {
        uint4 r = make_uint4(0u, 0u, 0u, 0u);
        if (j >= nsteps) return r;
        const int s = it.step_begin + j;
        if (j >= nmain) {  // entries 2t, 2t+1, 2t+8, 2t+9 of the group, as stored (value | row << 16)
            const unsigned* rv = a.ce_rv + (size_t)(it.ce0 + j - nmain) * 16 + 2 * t;
            const uint2 lo = __ldg((const uint2*)rv), hi = __ldg((const uint2*)(rv + 8));
            r = make_uint4(lo.x, lo.y, hi.x, hi.y);
        } else if (s < it.ntiles) {
            const size_t tile = (size_t)(it.tile0 + s);
            const uint2 v = __ldg((const uint2*)(a.f.s_packed_a + tile * 64) + lane);
            r.x = v.x; r.y = v.y;
            r.z = (uint32_t)__ldg(a.f.s_packed_meta + tile * 8 + g);
        } else {
            const int b = it.blk0 + 2 * (s - it.ntiles);
            const uint32_t* d0 = (const uint32_t*)(a.tc_dense + (size_t)b * 128);
            r.x = __ldg(d0 + g * 4 + t);
            r.y = __ldg(d0 + (g + 8) * 4 + t);
            if (b + 1 < it.blk_end) {
                r.z = __ldg(d0 + 64 + g * 4 + t);
                r.w = __ldg(d0 + 64 + (g + 8) * 4 + t);
            }
        }
        return r;
    };

    auto compute = [&](int j, int stage, const uint4& av) {
        const uint32_t baddr = boff + stage * T::STAGE;
        if (j < nsparse) {
#pragma unroll
            for (int h = 0; h < T::NT / 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + (((2 * h + lchunk) ^ lswz) << 4), b0, b1, b2, b3);
                mma_sp_16816(acc[2 * h], av.x, av.y, b0, b1, av.z);
                mma_sp_16816(acc[2 * h + 1], av.x, av.y, b2, b3, av.z);
            }
        } else {
            uint32_t a0 = av.x, a1 = av.y, a2 = av.z, a3 = av.w;
            if (j >= nmain) {
                // CSR group: A[r][k] = value of entry k if its row is r.  Fragment words: rows g / g + 8,
                // columns (2t, 2t+1) and (2t+8, 2t+9)
                auto pick = [](uint32_t e, uint32_t row) -> uint32_t { return (e >> 16) == row ? (e & 0xffffu) : 0u; };
                const uint32_t rlo = (uint32_t)g, rhi = (uint32_t)g + 8u;
                a0 = pick(av.x, rlo) | (pick(av.y, rlo) << 16);
                a1 = pick(av.x, rhi) | (pick(av.y, rhi) << 16);
                a2 = pick(av.z, rlo) | (pick(av.w, rlo) << 16);
                a3 = pick(av.z, rhi) | (pick(av.w, rhi) << 16);
            }
#pragma unroll
            for (int h = 0; h < T::NT / 2; ++h) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(baddr + (((2 * h + lchunk) ^ lswz) << 4), b0, b1, b2, b3);
                mma_16816(acc[2 * h], a0, a1, a2, a3, b0, b1);
                mma_16816(acc[2 * h + 1], a0, a1, a2, a3, b2, b3);
            }
        }
    };

    // Group accounting.  The prologue group carries the ids of steps 0 .. IDA-1 and is waited for
    // in full.  Then group k (k = 0, 1, ...) carries the rows of step k and, from k = STAGES-1 on,
    // the ids of step k - (STAGES-1) + IDA.  At iteration j all groups but the newest STAGES-2 are
    // complete, i.e. groups 0 .. j: the rows of step j, and the ids up to step j + IDA - STAGES + 1
    // = j + STAGES - 1, exactly what the gather issued in this iteration reads.
#pragma unroll
    for (int m = 0; m < T::IDA; ++m) issue_idx(m);
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    uint4 areg[STAGES];
#pragma unroll
    for (int j = 0; j < STAGES - 1; ++j) {
        if (j < nsteps) issue(j, j);
        cp_async_commit();
        areg[j] = load_a(j);
    }

    for (int j0 = 0; j0 < nsteps; j0 += STAGES) {
#pragma unroll
        for (int u = 0; u < STAGES; ++u) {
            const int j = j0 + u;
            if (j < nsteps) {
                cp_async_wait<STAGES - 2>();
                __syncwarp();
                issue_idx(j + T::IDA);
                if (j + STAGES - 1 < nsteps) issue(j + STAGES - 1, (u + STAGES - 1) % STAGES);
                cp_async_commit();
                areg[(u + STAGES - 1) % STAGES] = load_a(j + STAGES - 1);
                compute(j, u, areg[u]);
            }
        }
    }
    cp_async_wait<0>();
    __syncwarp();
    finish_item_warp<FS>(acc, it, a, fbase, lane, smem);
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
    DevBuf<Item> items;               // in window order (window-range runs index it by window)
    DevBuf<Item> items_sorted;        // the same items, long ones first (whole-matrix runs)
    DevBuf<Heavy> heavy;
    DevBuf<__half> tc_dense;          // TC blocks expanded to dense 16 x 8 fp16 tiles
    DevBuf<int> ce_col;               // CSR remainder entries in groups of 16: column ids (-1 = padding)
    DevBuf<unsigned> ce_rv;           //   and fp16 value | local row << 16
    int n_items, n_heavy, n_slots;
    std::vector<int> h_item_off, h_heavy_off;  // host copies of the per-window prefixes (num_windows + 1 each)
    bool arrays_aligned;              // index / tile arrays are 16-byte aligned
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
    // The checks below size their reads by prefix entries, so the verdict on the prefixes comes first.
    {
        int h_pre = 0;
        cudaError_t e1 = cudaMemcpyAsync(&h_pre, d_err, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (e1 == cudaSuccess) e1 = cudaStreamSynchronize(st);
        if (e1 != cudaSuccess) { cudaFree(d_err); return (int)e1; }
        if (h_pre & V_OFFSETS) { cudaFree(d_err); return TRS_E_OFFSETS; }
        if (h_pre & V_SHAPE) { cudaFree(d_err); return TRS_E_SHAPE; }
    }
    if (f.blocks > 0)
        k_check_tc_popcount<<<grid(f.blocks), 256, 0, st>>>((const long long*)f.t_binary, f.t_block_offset, f.blocks, d_err);
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
    // Longest run of k-steps one warp takes (longer windows are split into several items that write
    // partial sums).  Shorter items for small shards (64 to 256 by the shard's number of steps) were
    // measured and not kept: R-MAT scale 20 on one GPU 0.83 against 0.81 ms, a four-rank shard 0.46
    // against 0.42 ms - the extra partial sums cost more than the shorter critical path wins.
    p->chunk = max(8, env_int("TRS_CHUNK_STEPS", 256));
    // per-window ranges of TC blocks and CSR parts (needed only while the items are made)
    DevBuf<int> ranges, cnt, off;
    DevBuf<unsigned char> tmp;
    auto fail = [&](int code) { ranges.release(); cnt.release(); off.release(); tmp.release(); trs_spmm_plan_destroy(p); return code; };
    int rc = ranges.alloc((size_t)6 * W + 2 * ((size_t)W + 1));
    if (rc) return fail(rc);
    cudaMemsetAsync(ranges.p, 0, sizeof(int) * ((size_t)6 * W + 2 * ((size_t)W + 1)), st);
    WindowRanges wr{ranges.p, ranges.p + W, ranges.p + 2 * W, ranges.p + 3 * W, ranges.p + 4 * W, ranges.p + 5 * W,
                    ranges.p + (size_t)6 * W, ranges.p + (size_t)6 * W + (W + 1)};
    auto grid = [](long long n) { return (unsigned)((n + 255) / 256); };
    if (f.parts_t > 0)
        k_part_ranges<<<grid(f.parts_t), 256, 0, st>>>(f.t_window_row, f.t_row_offset, f.parts_t, 16, W,
                                                        wr.blk_begin, wr.blk_end, 1);
    if (f.parts_c > 0)
        k_part_ranges<<<grid(f.parts_c), 256, 0, st>>>(f.c_row, nullptr, f.parts_c, window, W, wr.c_begin, wr.c_end, 0);
    if (f.parts_c_short > 0)
        k_part_ranges<<<grid(f.parts_c_short), 256, 0, st>>>(f.cs_row, nullptr, f.parts_c_short, window, W,
                                                              wr.cs_begin, wr.cs_end, 0);
    // counts -> exclusive scans (three arrays of W + 1)
    rc = cnt.alloc((size_t)3 * (W + 1));
    if (!rc) rc = off.alloc((size_t)3 * (W + 1));
    size_t tmp_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, cnt.p, off.p, W + 1, st);
    if (!rc) rc = tmp.alloc(tmp_bytes + 16);
    if (rc) return fail(rc);
    cudaMemsetAsync(cnt.p, 0, sizeof(int) * 3 * (W + 1), st);
    // CSR remainder entries, expanded into groups of 16 per window
    {
        k_ce_count<<<grid(W + 1), 256, 0, st>>>(f, wr, W);
        cub::DeviceScan::ExclusiveSum(tmp.p, tmp_bytes, wr.ce_count, wr.ce_begin, W + 1, st);
        int groups = 0;
        cudaError_t ee = cudaMemcpyAsync(&groups, wr.ce_begin + W, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (ee == cudaSuccess) ee = cudaStreamSynchronize(st);
        if (ee != cudaSuccess) return fail((int)ee);
        if (groups < 0) return fail(TRS_E_OFFSETS);
        const size_t cap = (size_t)groups * 16;
        rc = p->ce_col.alloc(cap);
        if (!rc) rc = p->ce_rv.alloc(cap);
        if (rc) return fail(rc);
        if (cap > 0) {
            cudaMemsetAsync(p->ce_col.p, 0xff, cap * sizeof(int), st);
            cudaMemsetAsync(p->ce_rv.p, 0, cap * sizeof(unsigned), st);
            if (f.parts_c > 0)
                k_ce_fill<<<grid(f.parts_c), 256, 0, st>>>(f, wr, W, window, 0, (long long)cap, p->ce_col.p, p->ce_rv.p);
            if (f.parts_c_short > 0)
                k_ce_fill<<<grid(f.parts_c_short), 256, 0, st>>>(f, wr, W, window, 1, (long long)cap, p->ce_col.p, p->ce_rv.p);
        }
    }
    k_count_items<<<grid(W), 256, 0, st>>>(f, wr, W, p->chunk, cnt.p, cnt.p + (W + 1), cnt.p + 2 * (W + 1));
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
    k_fill_items<<<grid(W), 256, 0, st>>>(f, wr, W, p->chunk, off.p, off.p + (W + 1), off.p + 2 * (W + 1),
                                           p->items.p, p->heavy.p);
    // launch order of whole-matrix runs: a stable sort by length class, 32 classes (window order inside a class)
    if (p->n_items > 0) {
        DevBuf<unsigned char> cls, cls_out, sort_tmp;
        rc = p->items_sorted.alloc(p->n_items);
        if (!rc) rc = cls.alloc(p->n_items);
        if (!rc) rc = cls_out.alloc(p->n_items);
        size_t sort_bytes = 0;
        cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, cls.p, cls_out.p, p->items.p, p->items_sorted.p, p->n_items, 0, 5, st);
        if (!rc) rc = sort_tmp.alloc(sort_bytes + 16);
        if (!rc) {
            k_item_class<<<grid(p->n_items), 256, 0, st>>>(p->items.p, p->n_items, cls.p);
            cub::DeviceRadixSort::SortPairs(sort_tmp.p, sort_bytes, cls.p, cls_out.p, p->items.p, p->items_sorted.p, p->n_items, 0, 5, st);
            e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) rc = (int)e;
        }
        cls.release(); cls_out.release(); sort_tmp.release();
        if (rc) return fail(rc);
    }
    rc = p->tc_dense.alloc((size_t)f.blocks * 128);
    if (rc) return fail(rc);
    if (f.blocks > 0)
        k_expand_tc<<<grid((long long)f.blocks * 128), 256, 0, st>>>((const long long*)f.t_binary, f.t_block_offset,
                                                                      (const __half*)f.t_value, f.blocks, p->tc_dense.p);
    e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail((int)e);
    ranges.release(); cnt.release(); off.release(); tmp.release();
    const uintptr_t align_or = (uintptr_t)f.s_tile_column | (uintptr_t)f.s_packed_a | (uintptr_t)f.s_packed_meta |
                               (uintptr_t)f.t_column;
    p->arrays_aligned = (align_or & 15) == 0;
    *out_plan = p;
    return TRS_OK;
}

// No kernel of this library waits on a flag or a barrier that another warp or kernel sets (the
// window kernels synchronise inside one warp or one CTA only), so there is no wait that could
// give up: the status word is always 0.  Kept for callers of earlier versions.
extern "C" int trs_spmm_status(const trs_spmm_plan* p, int* status) {
    if (!p || !status) return TRS_E_ARG;
    *status = 0;
    return TRS_OK;
}

extern "C" int trs_spmm_plan_destroy(trs_spmm_plan* p) {
    if (!p) return TRS_OK;
    p->items.release();
    p->items_sorted.release();
    p->heavy.release();
    p->tc_dense.release();
    p->ce_col.release();
    p->ce_rv.release();
    delete p;
    return TRS_OK;
}

static size_t items_scratch_bytes(const trs_spmm_plan* p, int F) { return (size_t)p->n_slots * 16 * (size_t)F * sizeof(float); }

extern "C" int trs_spmm_workspace_bytes(const trs_spmm_plan* p, int F, size_t* bytes) {
    if (!p || !bytes || F <= 0) return TRS_E_ARG;
    *bytes = items_scratch_bytes(p, F);
    return TRS_OK;
}

extern "C" int trs_spmm_static_scratch_bytes(const trs_spmm_plan* p, int F, size_t* bytes) {
    if (!p || !bytes || F <= 0) return TRS_E_ARG;
    *bytes = items_scratch_bytes(p, F);
    return TRS_OK;
}

extern "C" int trs_spmm_launches(const trs_spmm_plan* p) {
    if (!p) return 0;
    return p->n_heavy > 0 ? 2 : 1;
}

template <int FS, int STAGES, int MINB>
static int launch_warp_kernel(const KernelArgs& a, cudaStream_t st) {
    using T = WarpTile<FS, STAGES>;
    dim3 grid(a.n_items, ceil_div(a.F, FS));
    TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_warp<FS, STAGES, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
    TRS_CUDA(cudaFuncSetAttribute(k_window_spmm_warp<FS, STAGES, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                  cudaSharedmemCarveoutMaxShared));
    k_window_spmm_warp<FS, STAGES, MINB><<<grid, 32, T::SMEM, st>>>(a);
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

template <int WARPS>
static int launch_cta_kernel(const KernelArgs& a, cudaStream_t st) {
    using T = Tile<WARPS>;
    dim3 grid(a.n_items, ceil_div(a.F, T::FS));
    TRS_CUDA(cudaFuncSetAttribute(k_window_spmm<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM));
    k_window_spmm<WARPS><<<grid, T::THREADS, T::SMEM, st>>>(a);
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

extern "C" int trs_spmm_run(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, void* workspace,
                            size_t workspace_bytes, void* stream) {
    return trs_spmm_run_ex(p, B, C, F, out_dtype, 0, workspace, workspace_bytes, stream);
}

static int run_impl(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags, void* workspace,
                    size_t workspace_bytes, void* stream, void* const* peers = nullptr, int n_peers = 0,
                    long long peer_row0 = 0, int w0 = 0, int w1 = -1);

extern "C" int trs_spmm_run_ex(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags,
                               void* workspace, size_t workspace_bytes, void* stream) {
    return run_impl(p, B, C, F, out_dtype, flags, workspace, workspace_bytes, stream);
}

extern "C" int trs_spmm_run_windows(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags,
                                    void* workspace, size_t workspace_bytes, void* stream, int window_begin,
                                    int window_end) {
    if (window_end < 0) return TRS_E_ARG;
    return run_impl(p, B, C, F, out_dtype, flags, workspace, workspace_bytes, stream, nullptr, 0, 0, window_begin, window_end);
}

extern "C" int trs_spmm_num_windows(const trs_spmm_plan* p) { return p ? p->num_windows : TRS_E_ARG; }

extern "C" int trs_spmm_run_bcast(const trs_spmm_plan* p, const trs_half* B, void* const* dst, int n_dst, long long row0,
                                  int F, int flags, void* workspace, size_t workspace_bytes, void* stream) {
    if (!p || !dst || n_dst < 1 || n_dst > 8 || row0 < 0) return TRS_E_ARG;
    for (int d = 0; d < n_dst; ++d)
        if (!dst[d] || ((uintptr_t)dst[d] & 15)) return TRS_E_ARG;
    if (F % 8 != 0 || ((uintptr_t)B & 15) || !p->arrays_aligned) return TRS_E_ARG;  // the 16-byte row pieces need it
    return run_impl(p, B, dst[0], F, TRS_OUT_F16, flags, workspace, workspace_bytes, stream, dst, n_dst, row0);
}

static int run_impl(const trs_spmm_plan* p, const trs_half* B, void* C, int F, int out_dtype, int flags, void* workspace,
                    size_t workspace_bytes, void* stream, void* const* peers, int n_peers, long long peer_row0, int w0,
                    int w1) {
    if (!p || !B || !C || F <= 0) return TRS_E_ARG;
    if (w1 < 0) w1 = p->num_windows;
    if (w0 < 0 || w0 > w1 || w1 > p->num_windows) return TRS_E_ARG;
    if (w0 == w1) return TRS_OK;
    // window range -> item / split-window ranges (both lists are in window order)
    const int i0 = p->h_item_off[w0], n_items = p->h_item_off[w1] - i0;
    const int h0 = p->h_heavy_off[w0], n_heavy = p->h_heavy_off[w1] - h0;
    if (flags & ~TRS_EPILOGUE_RELU) return TRS_E_ARG;
    if (out_dtype != TRS_OUT_F32 && out_dtype != TRS_OUT_F16) return TRS_E_ARG;
    const size_t need = items_scratch_bytes(p, F);
    if (need > 0 && (!workspace || workspace_bytes < need)) return TRS_E_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    KernelArgs a;
    a.f = p->f; a.n_items = n_items;
    a.items = (w0 == 0 && w1 == p->num_windows) ? p->items_sorted.p : p->items.p + i0;
    a.B = (const __half*)B; a.C = C; a.scratch = (float*)workspace;
    a.m_rows = p->m_rows; a.k_cols = p->k_cols; a.window = p->window; a.F = F; a.out_half = out_dtype == TRS_OUT_F16;
    a.relu = (flags & TRS_EPILOGUE_RELU) ? 1 : 0;
    a.n_peers = n_peers; a.peer_row0 = peer_row0;
    for (int d = 0; d < 8; ++d) a.peers[d] = d < n_peers ? peers[d] : nullptr;
    a.tc_dense = p->tc_dense.p;
    a.ce_col = p->ce_col.p; a.ce_rv = p->ce_rv.p;
    // The warp-owner kernel moves everything in 16-byte pieces; anything else takes the fallback.
    const bool aligned = p->arrays_aligned && (F % 8 == 0) &&
                         ((((uintptr_t)B | (uintptr_t)C | (uintptr_t)workspace) & 15) == 0);
    // Three stages (two k-steps in flight per warp) and 16 warps per SM (four per scheduler)
    // measured fastest at R-MAT scale 21: 2.72 ms, against 3.16 ms for four stages (13 warps) and
    // 3.05 ms for 17 warps of 96 registers; 64-feature slabs for F = 128 (24 warps per SM, twice
    // the steps) were slower too, and so was asking L2 for the rows (or the packed tiles) of later
    // steps with prefetch instructions two to four steps ahead (2.9 - 3.3 ms; bulk prefetches 4.1 ms).
    int rc;
    if (!aligned) {
        if (n_peers > 0) return TRS_E_ARG;
        if (F <= 32) rc = launch_cta_kernel<1>(a, st);
        else if (F <= 64) rc = launch_cta_kernel<2>(a, st);
        else rc = launch_cta_kernel<4>(a, st);
    } else if (F <= 32) rc = launch_warp_kernel<32, 3, 32>(a, st);
    else if (F <= 64) rc = launch_warp_kernel<64, 3, 28>(a, st);   // 72 registers: seven warps per scheduler (0.49 against 0.51 ms with six; eight spill: 0.57 ms)
    else rc = launch_warp_kernel<128, 3, 16>(a, st);   // F > 128: feature slabs of 128 on gridDim.y
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
// (k_window_spmm_warp / k_window_spmm + k_reduce_heavy), whose scratch need is small and known
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
    return run_impl(p, B, C, F, out_dtype, 0, scratch, (size_t)TRS_STATIC_SCRATCH_BYTES, stream);
}
