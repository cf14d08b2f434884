// SDDMM: out[e] = fp16( sum_k fp32(X[row(e),k]) * fp32(Y[col(e),k]) ) for every CSR entry e.
//
// The reference has no SDDMM operator; the definition is fixed by the benchmark
// configuration (X, Y dense fp16, fp32 accumulate, fp16 result in CSR order).
//
// Work is split by ENTRY, not by row, so power-law rows cost nothing extra: a warp takes a run
// of consecutive entries, an 8-lane group takes one entry at a time and reads the 128-byte
// slices of X[row] and Y[col] with one 16-byte load per lane, multiplies in fp32 and reduces
// with three shuffles.  The row of an entry is found once per warp by binary search in the row
// pointers and then advanced linearly.
#include <stdlib.h>
#include <string.h>

#include <cub/cub.cuh>

#include "trs_common.cuh"

namespace trs {

constexpr int kEntriesPerWarp = 512;

__device__ __forceinline__ float dot8(const uint4& x, const uint4& y) {
    const __half2* xh = reinterpret_cast<const __half2*>(&x);
    const __half2* yh = reinterpret_cast<const __half2*>(&y);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 a = __half22float2(xh[i]);
        const float2 b = __half22float2(yh[i]);
        s = fmaf(a.x, b.x, s);
        s = fmaf(a.y, b.y, s);
    }
    return s;
}

constexpr int kUnroll = 8;  // entries in flight per 8-lane group

template <bool VEC>
__global__ void __launch_bounds__(256) k_sddmm(const int* __restrict__ rowptr, const int* __restrict__ col,
                                               const __half* __restrict__ X, const __half* __restrict__ Y,
                                               __half* __restrict__ out, int n_rows, int n_cols, long long nnz, int K) {
    // Inputs are not validated by a pass of their own on this entry (trs_sddmm_plan_create does
    // that for planned patterns), so the kernel bounds what it dereferences: the row walk stops at
    // the last row, and an entry whose column lies outside [0, n_cols) reads row 0 of Y and is
    // written as NaN instead of gathering out of range.
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 3, sl = lane & 7;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long e0 = warp * kEntriesPerWarp;
    if (e0 >= nnz) return;
    const long long e1 = min(e0 + (long long)kEntriesPerWarp, nnz);
    // row containing e0: largest r with rowptr[r] <= e0
    int lo = 0, hi = n_rows;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)rowptr[mid] <= e0) lo = mid; else hi = mid;
    }
    int row = lo;
    if (VEC && K == 64) {
        // fast path: one 16-byte slice of X[row] and Y[col] per lane.  The Y slices of kUnroll
        // entries are requested before any is consumed, so an 8-lane group keeps kUnroll random
        // 128-byte rows in flight; X[row] changes rarely and is (re)read at use (an L1 hit).
        int xrow = -1;
        uint4 xv = make_uint4(0, 0, 0, 0);
        for (long long eb = e0; eb < e1; eb += 4 * kUnroll) {
            uint4 yv[kUnroll];
            int rows[kUnroll];
            unsigned bad = 0;
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const long long e = eb + sub + 4 * u;
                rows[u] = -1;
                yv[u] = make_uint4(0, 0, 0, 0);
                if (e < e1) {
                    while (row + 1 < n_rows && (long long)rowptr[row + 1] <= e) ++row;
                    rows[u] = row;
                    int c = col[e];
                    if ((unsigned)c >= (unsigned)n_cols) { c = 0; bad |= 1u << u; }
                    yv[u] = __ldg(reinterpret_cast<const uint4*>(Y + (size_t)c * 64) + sl);
                }
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                if (rows[u] >= 0 && rows[u] != xrow) {
                    xrow = rows[u];
                    xv = __ldg(reinterpret_cast<const uint4*>(X + (size_t)xrow * 64) + sl);
                }
                float s = dot8(xv, yv[u]);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if (rows[u] >= 0 && sl == 0) out[eb + sub + 4 * u] = (bad >> u) & 1u ? __ushort_as_half((unsigned short)0x7e00) : __float2half_rn(s);
            }
        }
        return;
    }
    for (long long eb = e0; eb < e1; eb += 4) {
        const long long e = eb + sub;
        const bool live = e < e1;
        float s = 0.f;
        bool bad = false;
        if (live) {
            while (row + 1 < n_rows && (long long)rowptr[row + 1] <= e) ++row;
            int c = col[e];
            if ((unsigned)c >= (unsigned)n_cols) { c = 0; bad = true; }
            const __half* xr = X + (size_t)row * K;
            const __half* yr = Y + (size_t)c * K;
            if (VEC) {
                for (int k = sl * 8; k < K; k += 64) {
                    const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xr + k));
                    const uint4 yv = __ldg(reinterpret_cast<const uint4*>(yr + k));
                    s += dot8(xv, yv);
                }
            } else {
                for (int k = sl; k < K; k += 8) s = fmaf(__half2float(xr[k]), __half2float(yr[k]), s);
            }
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (live && sl == 0) out[e] = bad ? __ushort_as_half((unsigned short)0x7e00) : __float2half_rn(s);
    }
}

// ----------------------------------------------------------------------------------------------
// Planned, tensor-core SDDMM
// ----------------------------------------------------------------------------------------------
// The entry-parallel kernel above gathers one Y row per ENTRY and spends ~19 warp instructions
// per entry on conversions, FMAs and shuffles.  With a plan over the pattern the work is done per
// (16-row window, column) PAIR instead: the distinct columns of a window, ascending, are cut into
// blocks of 8; for a block one warp multiplies the window's X tile (16 x K) with the 8 gathered
// Y rows on the tensor cores (mma m16n8k16, fp32 accumulate) and stores only the dot products
// the pattern has.  The contraction runs over the feature dimension, which is contiguous in
// both operands, so the fragments are filled by plain 16-byte loads: lane (g, t) reads bytes
// [64 c + 16 t, +16) of X[row g], X[row g + 8] and Y[col g] for every 32-feature chunk c — the
// same feature positions on both sides, which is all the MMA needs (the order of the k index
// inside a chunk is free).
//
// Block record (128 bytes, one cache line): 8 column ids (-1 = unused slot), a 16 x 8 bitmap of
// the entries present (bit 8 r + n), the window id, and for each of the 16 rows the CSR index of
// its first entry inside the block.  Columns ascend inside a CSR row and a block holds a
// contiguous run of the window's sorted distinct columns, so the entries of a row inside a block
// are consecutive in CSR order: entry (r, n) = start[r] + popcount(rowbits(r) below bit n).
// The pattern must be canonical CSR (columns ascending and unique per row).
struct SddmmBlock {
    int col[8];
    unsigned bits[4];
    int window;
    int pad[3];
    int start[16];
};
static_assert(sizeof(SddmmBlock) == 128, "one cache line per block");

__device__ __forceinline__ int row_of_entry(const int* __restrict__ rowptr, int n_rows, long long e) {
    int lo = 0, hi = n_rows;  // largest r with rowptr[r] <= e
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if ((long long)rowptr[mid] <= e) lo = mid; else hi = mid;
    }
    return lo;
}

// Also validates the pattern: err |= 1 for a column outside [0, n_cols), |= 2 for columns that are
// not strictly ascending inside a row (the plan's entry addressing relies on canonical CSR).
__global__ void ksp_keys(const int* __restrict__ rowptr, const int* __restrict__ col, int n_rows, int n_cols,
                         long long nnz, unsigned long long* __restrict__ key, int* __restrict__ ent,
                         int* __restrict__ err) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = row_of_entry(rowptr, n_rows, e);
    const int c = col[e];
    if (c < 0 || c >= n_cols) { atomicOr(err, 1); return; }
    if (e > (long long)rowptr[r] && col[e - 1] >= c) atomicOr(err, 2);
    key[e] = ((unsigned long long)(r >> 4) << 32) | (unsigned)col[e];
    ent[e] = (int)e;
}

__global__ void ksp_heads(const unsigned long long* __restrict__ key, long long nnz, int* __restrict__ head) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    head[i] = (i == 0 || key[i] != key[i - 1]) ? 1 : 0;
}

// first_pair[w] = number of distinct (window, column) pairs in windows < w, for w in [0, W]
__global__ void ksp_window_pairs(const unsigned long long* __restrict__ key, const int* __restrict__ pair_idx,
                                 long long nnz, int total_pairs, int W, int* __restrict__ first_pair,
                                 int* __restrict__ blocks_of) {
    const int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w > W) return;
    auto lower = [&](int win) -> int {  // pairs before the first sorted entry of window >= win
        long long lo = 0, hi = nnz;     // first i with key[i] >> 32 >= win
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if ((int)(key[mid] >> 32) < win) lo = mid + 1; else hi = mid;
        }
        return lo < nnz ? pair_idx[lo] : total_pairs;
    };
    const int mine = lower(w);
    first_pair[w] = mine;
    if (w < W) blocks_of[w] = (lower(w + 1) - mine + 7) >> 3;
}

__global__ void ksp_init_blocks(SddmmBlock* __restrict__ blk, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one int of a record per thread
    if (i >= n * 32) return;
    const int f = (int)(i & 31);
    int v = 0;
    if (f < 8) v = -1;
    else if (f >= 16) v = 0x7fffffff;
    ((int*)blk)[i] = v;
}

__global__ void ksp_fill(const unsigned long long* __restrict__ key, const int* __restrict__ ent,
                         const int* __restrict__ pair_idx, const int* __restrict__ head,
                         const int* __restrict__ first_pair, const int* __restrict__ blk_off,
                         const int* __restrict__ rowptr, int n_rows, long long nnz, SddmmBlock* __restrict__ blk) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const unsigned long long k = key[i];
    const int w = (int)(k >> 32);
    const int local = pair_idx[i] - first_pair[w];
    SddmmBlock* b = blk + (size_t)blk_off[w] + (local >> 3);
    const int n = local & 7;
    const int e = ent[i];
    const int r = row_of_entry(rowptr, n_rows, e) - (w << 4);
    atomicOr(&b->bits[r >> 2], 1u << (((r & 3) << 3) + n));
    atomicMin(&b->start[r], e);
    if (head[i]) {
        b->col[n] = (int)(unsigned)k;
        if (n == 0) b->window = w;
    }
}

constexpr int kSddmmBlocksPerWarp = 48;

// One warp walks kSddmmBlocksPerWarp consecutive blocks, one block at a time, with both dependent
// loads of a block taken off the warp's critical path: the
// 128-byte records run kRecAhead blocks ahead and the 8 gathered Y rows kRowAhead blocks ahead,
// all as 16-byte cp.async copies into the warp's own rings in shared memory (one commit group per
// block, lanes meet in one __syncwarp per block, no block-wide barrier).  The odd Y rows land with
// the two 64-byte halves of every 128 bytes swapped (chunk c at position c ^ 4): a 16-byte access
// is served eight lanes at a time, those are the lanes (g, t) of two consecutive rows g with four
// chunks each, and the swap puts the two rows into different halves of the 128-byte bank line, so
// the copies and the fragment reads - lane (g, t) takes chunks 4 ch + t of row g - are
// conflict-free without padding (rows of 64 bytes already alternate halves).  Holding the rows in
// registers instead (plain 16-byte loads two blocks ahead, no shared-memory round trip) measured
// slower: 0.127 against 0.109 ms on the clustered pattern.
constexpr int kRecRing = 8, kRecAhead = 6, kRowAhead = 3, kRowStages = 4;

template <int KCH>
struct SddmmRing {
    static constexpr int ROWB = KCH * 64;                 // bytes of a Y row (K halfs)
    static constexpr int CPR = KCH * 4;                   // 16-byte chunks per row
    static constexpr int STAGE = 8 * ROWB;
    static constexpr int WARP_SMEM = kRecRing * 128 + kRowStages * STAGE;
    static constexpr int SMEM = 4 * WARP_SMEM;
};

template <int KCH, int MINB>
__global__ void __launch_bounds__(128, MINB) k_sddmm_tc_ring(const SddmmBlock* __restrict__ blk, long long n_blocks,
                                                             const __half* __restrict__ X, const __half* __restrict__ Y,
                                                             __half* __restrict__ out, int n_rows, int blocks_per_warp) {
    using R = SddmmRing<KCH>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + wid;
    const long long b0 = warp * blocks_per_warp;
    if (b0 >= n_blocks) return;
    const int nb = (int)(min(b0 + (long long)blocks_per_warp, n_blocks) - b0);
    unsigned char* recs = smem + wid * R::WARP_SMEM;
    unsigned char* rows = recs + kRecRing * 128;
    const uint32_t recs0 = smem_u32(recs), rows0 = smem_u32(rows);
    constexpr int ROW16 = KCH * 4;
    const uint4* Xq = (const uint4*)X + t;
    const uint4* Yq = (const uint4*)Y;

    // `slot` / `stage` arguments are the ring positions of block j, passed separately so that they are
    // compile-time constants inside the unrolled loop below
    auto issue_rec = [&](int j, int slot) {   // record of block j -> record ring (8 lanes x 16 B)
        if (j < nb && lane < 8) cp_async16(recs0 + slot * 128 + lane * 16, (const uint4*)(blk + b0 + j) + lane, 16);
    };
    // Y rows of block j (its record is in the ring): lane copies chunks (lane & 3) + 4 i of row lane >> 2
    auto issue_rows = [&](int j, int slot, int stage) {
        if (j >= nb) return;
        const int c = *(const int*)(recs + slot * 128 + g * 4);
        const uint4* src = Yq + (size_t)max(c, 0) * ROW16;
        const uint32_t dst = rows0 + stage * R::STAGE + g * R::ROWB;
#pragma unroll
        for (int i = 0; i < KCH; ++i) {
            const int chunk = t + 4 * i;
            cp_async16(dst + ((chunk ^ ((g & 1) << 2)) & (R::CPR - 1)) * 16, src + chunk, c >= 0 ? 16 : 0);
        }
    };
    // group accounting: prologue = records 0 .. kRecAhead-1 (waited for), then one group per block j
    // holding the rows of block j + kRowAhead and the record of block j + kRecAhead; the rows of
    // blocks 0 .. kRowAhead-1 are kRowAhead groups of their own.  At iteration j all but the newest
    // kRowAhead-1 groups are complete: the rows of block j and the record of block j + kRowAhead.
#pragma unroll
    for (int j = 0; j < kRecAhead; ++j) issue_rec(j, j);
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int j = 0; j < kRowAhead; ++j) {
        issue_rows(j, j, j);
        cp_async_commit();
    }

    int cur_w = -1;
    uint4 xa[KCH], xb[KCH];
#pragma unroll
    for (int c = 0; c < KCH; ++c) xa[c] = xb[c] = make_uint4(0, 0, 0, 0);
    static_assert(kRecRing == 8 && kRowStages == 4, "the loop is unrolled by the record ring");
    for (int j0 = 0; j0 < nb; j0 += kRecRing) {
#pragma unroll
        for (int u = 0; u < kRecRing; ++u) {
            const int j = j0 + u;
            if (j >= nb) break;
            cp_async_wait<kRowAhead - 1>();
            __syncwarp();
            issue_rec(j + kRecAhead, (u + kRecAhead) & (kRecRing - 1));
            issue_rows(j + kRowAhead, (u + kRowAhead) & (kRecRing - 1), (u + kRowAhead) & (kRowStages - 1));
            cp_async_commit();
            const unsigned char* rec = recs + u * 128;
            const int w = *(const int*)(rec + 48);
            const unsigned wa = *(const unsigned*)(rec + 32 + (g >> 2) * 4), wb = *(const unsigned*)(rec + 32 + ((g >> 2) + 2) * 4);
            if (w != cur_w) {  // warp-uniform
                cur_w = w;
                const int ra = min(w * 16 + g, n_rows - 1), rb = min(w * 16 + g + 8, n_rows - 1);
#pragma unroll
                for (int ch = 0; ch < KCH; ++ch) {
                    xa[ch] = __ldg(Xq + (size_t)ra * ROW16 + ch * 4);
                    xb[ch] = __ldg(Xq + (size_t)rb * ROW16 + ch * 4);
                }
            }
            const unsigned char* yrow = rows + (u & (kRowStages - 1)) * R::STAGE + g * R::ROWB;
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ch = 0; ch < KCH; ++ch) {
                const uint4 y = *(const uint4*)(yrow + (((4 * ch + t) ^ ((g & 1) << 2)) & (R::CPR - 1)) * 16);
                mma_16816(d, xa[ch].x, xb[ch].x, xa[ch].y, xb[ch].y, y.x, y.y);
                mma_16816(d, xa[ch].z, xb[ch].z, xa[ch].w, xb[ch].w, y.z, y.w);
            }
            const unsigned ba = (wa >> ((g & 3) << 3)) & 0xffu, bbits = (wb >> ((g & 3) << 3)) & 0xffu;
            const int n0 = 2 * t;
            if ((ba >> n0) & 3u) {
                const int s = *(const int*)(rec + 64 + g * 4) + __popc(ba & ((1u << n0) - 1u));
                if ((ba >> n0) & 1u) out[s] = __float2half_rn(d[0]);
                if ((ba >> n0) & 2u) out[s + ((ba >> n0) & 1u)] = __float2half_rn(d[1]);
            }
            if ((bbits >> n0) & 3u) {
                const int s = *(const int*)(rec + 64 + (g + 8) * 4) + __popc(bbits & ((1u << n0) - 1u));
                if ((bbits >> n0) & 1u) out[s] = __float2half_rn(d[2]);
                if ((bbits >> n0) & 2u) out[s + ((bbits >> n0) & 1u)] = __float2half_rn(d[3]);
            }
        }
    }
    cp_async_wait<0>();
}


}  // namespace trs

struct trs_sddmm_plan {
    const int32_t* rowptr = nullptr;  // caller-owned pattern (used by the fallback kernel)
    const int32_t* col = nullptr;
    int n_rows = 0, n_cols = 0;
    long long nnz = 0, n_blocks = 0, n_pairs = 0;
    trs::DevBuf<trs::SddmmBlock> blocks;
};

extern "C" int trs_sddmm_plan_destroy(trs_sddmm_plan* p) {
    if (!p) return TRS_OK;
    p->blocks.release();
    delete p;
    return TRS_OK;
}

extern "C" int trs_sddmm_plan_create(const int32_t* rowptr, const int32_t* col, int n_rows, int n_cols, void* stream,
                                     trs_sddmm_plan** out) {
    using namespace trs;
    if (!out) return TRS_E_ARG;
    *out = nullptr;
    if (!rowptr || n_rows <= 0 || n_cols <= 0) return TRS_E_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return TRS_E_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    int ends[2] = {0, 0};
    TRS_CUDA(cudaMemcpyAsync(&ends[0], rowptr, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaMemcpyAsync(&ends[1], rowptr + n_rows, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    if (ends[0] != 0 || ends[1] < 0) return TRS_E_OFFSETS;
    const long long nnz = ends[1];
    if (nnz > 0 && !col) return TRS_E_ARG;
    trs_sddmm_plan* p = new trs_sddmm_plan();
    p->rowptr = rowptr; p->col = col; p->n_rows = n_rows; p->n_cols = n_cols; p->nnz = nnz;
    if (nnz == 0) { *out = p; return TRS_OK; }

    const int W = (n_rows + 15) / 16;
    DevBuf<unsigned long long> key_a, key_b;
    DevBuf<int> ent_a, ent_b, head, pair_idx, first_pair, blocks_of, blk_off;
    DevBuf<unsigned char> tmp;
    auto cleanup = [&]() {
        key_a.release(); key_b.release(); ent_a.release(); ent_b.release(); head.release(); pair_idx.release();
        first_pair.release(); blocks_of.release(); blk_off.release(); tmp.release();
    };
    auto fail = [&](int code) { cleanup(); trs_sddmm_plan_destroy(p); return code; };
    int rc = key_a.alloc(nnz);
    if (!rc) rc = key_b.alloc(nnz);
    if (!rc) rc = ent_a.alloc(nnz);
    if (!rc) rc = ent_b.alloc(nnz);
    if (!rc) rc = head.alloc(nnz);
    if (!rc) rc = pair_idx.alloc(nnz);
    if (!rc) rc = first_pair.alloc((size_t)W + 1);
    if (!rc) rc = blocks_of.alloc((size_t)W + 1);
    if (!rc) rc = blk_off.alloc((size_t)W + 1);
    if (rc) return fail(rc);
    auto grid = [](long long n) { return (unsigned)((n + 255) / 256); };
    DevBuf<int> d_err;
    rc = d_err.alloc(1);
    if (rc) return fail(rc);
    cudaMemsetAsync(d_err.p, 0, sizeof(int), st);
    ksp_keys<<<grid(nnz), 256, 0, st>>>(rowptr, col, n_rows, n_cols, nnz, key_a.p, ent_a.p, d_err.p);
    {
        int herr = 0;
        cudaError_t ee = cudaMemcpyAsync(&herr, d_err.p, sizeof(int), cudaMemcpyDeviceToHost, st);
        if (ee == cudaSuccess) ee = cudaStreamSynchronize(st);
        d_err.release();
        if (ee != cudaSuccess) return fail((int)ee);
        if (herr & 1) return fail(TRS_E_COLUMN);
        if (herr & 2) return fail(TRS_E_NOT_CANONICAL);
    }
    int wbits = 1;
    while ((1ll << wbits) < W) ++wbits;
    cub::DoubleBuffer<unsigned long long> kb(key_a.p, key_b.p);
    cub::DoubleBuffer<int> vb(ent_a.p, ent_b.p);
    size_t bytes = 0, bytes2 = 0, bytes3 = 0;
    cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, bytes, kb, vb, (int)nnz, 0, 32 + wbits, st);
    if (e == cudaSuccess) e = cub::DeviceScan::InclusiveSum(nullptr, bytes2, head.p, pair_idx.p, (int)nnz, st);
    if (e == cudaSuccess) e = cub::DeviceScan::ExclusiveSum(nullptr, bytes3, blocks_of.p, blk_off.p, W + 1, st);
    if (e != cudaSuccess) return fail((int)e);
    if (bytes2 > bytes) bytes = bytes2;
    if (bytes3 > bytes) bytes = bytes3;
    rc = tmp.alloc(bytes + 16);
    if (rc) return fail(rc);
    e = cub::DeviceRadixSort::SortPairs(tmp.p, bytes, kb, vb, (int)nnz, 0, 32 + wbits, st);
    if (e != cudaSuccess) return fail((int)e);
    const unsigned long long* key = kb.Current();
    const int* ent = vb.Current();
    ksp_heads<<<grid(nnz), 256, 0, st>>>(key, nnz, head.p);
    e = cub::DeviceScan::InclusiveSum(tmp.p, bytes, head.p, pair_idx.p, (int)nnz, st);  // pair id + 1
    if (e != cudaSuccess) return fail((int)e);
    int total_pairs = 0;
    e = cudaMemcpyAsync(&total_pairs, pair_idx.p + (nnz - 1), sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail((int)e);
    // pair_idx holds inclusive sums: pair id of sorted entry i = pair_idx[i] - 1.  ksp_window_pairs
    // and ksp_fill only use differences against first_pair, which is taken from the same array.
    e = cudaMemsetAsync(blocks_of.p, 0, sizeof(int) * ((size_t)W + 1), st);
    if (e != cudaSuccess) return fail((int)e);
    ksp_window_pairs<<<grid(W + 1), 256, 0, st>>>(key, pair_idx.p, nnz, total_pairs + 1, W, first_pair.p, blocks_of.p);
    e = cub::DeviceScan::ExclusiveSum(tmp.p, bytes, blocks_of.p, blk_off.p, W + 1, st);
    if (e != cudaSuccess) return fail((int)e);
    int n_blocks = 0;
    e = cudaMemcpyAsync(&n_blocks, blk_off.p + W, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail((int)e);
    p->n_blocks = n_blocks;
    p->n_pairs = total_pairs;
    rc = p->blocks.alloc((size_t)n_blocks);
    if (rc) return fail(rc);
    ksp_init_blocks<<<grid((long long)n_blocks * 32), 256, 0, st>>>(p->blocks.p, n_blocks);
    ksp_fill<<<grid(nnz), 256, 0, st>>>(key, ent, pair_idx.p, head.p, first_pair.p, blk_off.p, rowptr, n_rows, nnz,
                                       p->blocks.p);
    e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail((int)e);
    cleanup();
    *out = p;
    return TRS_OK;
}

extern "C" int trs_sddmm_plan_info(const trs_sddmm_plan* p, long long* n_pairs, long long* n_blocks) {
    if (!p) return TRS_E_ARG;
    if (n_pairs) *n_pairs = p->n_pairs;
    if (n_blocks) *n_blocks = p->n_blocks;
    return TRS_OK;
}

extern "C" int trs_sddmm(const int32_t* rowptr, const int32_t* col, const trs_half* X, const trs_half* Y, trs_half* out,
                         int n_rows, int n_cols, int K, void* stream);

extern "C" int trs_sddmm_plan_run(const trs_sddmm_plan* p, const trs_half* X, const trs_half* Y, trs_half* out, int K,
                                  void* stream) {
    if (!p || !X || !Y || K <= 0) return TRS_E_ARG;
    if (p->nnz == 0) return TRS_OK;
    if (!out) return TRS_E_ARG;
    const bool tc = (K == 32 || K == 64 || K == 128) && (((uintptr_t)X & 15) == 0) && (((uintptr_t)Y & 15) == 0);
    if (!tc) return trs_sddmm(p->rowptr, p->col, X, Y, out, p->n_rows, p->n_cols, K, stream);
    cudaStream_t st = (cudaStream_t)stream;
    const int bpw = trs::kSddmmBlocksPerWarp;
    const long long warps = trs::ceil_div64(p->n_blocks, bpw);
    const unsigned grid = (unsigned)trs::ceil_div64(warps, 4);
    const __half *x = (const __half*)X, *y = (const __half*)Y;
    auto launch = [&](auto kernel, int smem) -> int {
        TRS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kernel<<<grid, 128, smem, st>>>(p->blocks.p, p->n_blocks, x, y, (__half*)out, p->n_rows, bpw);
        return TRS_OK;
    };
    int rc;
    if (K == 32) rc = launch(trs::k_sddmm_tc_ring<1, 8>, trs::SddmmRing<1>::SMEM);
    else if (K == 64) rc = launch(trs::k_sddmm_tc_ring<2, 8>, trs::SddmmRing<2>::SMEM);
    else rc = launch(trs::k_sddmm_tc_ring<4, 5>, trs::SddmmRing<4>::SMEM);
    if (rc) return rc;
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

extern "C" int trs_sddmm(const int32_t* rowptr, const int32_t* col, const trs_half* X, const trs_half* Y, trs_half* out,
                         int n_rows, int n_cols, int K, void* stream) {
    if (!rowptr || !X || !Y || n_rows <= 0 || n_cols <= 0 || K <= 0) return TRS_E_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return TRS_E_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    int ends[2] = {0, 0};
    TRS_CUDA(cudaMemcpyAsync(&ends[0], rowptr, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaMemcpyAsync(&ends[1], rowptr + n_rows, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    if (ends[0] != 0 || ends[1] < 0) return TRS_E_OFFSETS;
    const long long nnz = ends[1];
    if (nnz == 0) return TRS_OK;
    if (!col || !out) return TRS_E_ARG;
    const long long warps = trs::ceil_div64(nnz, trs::kEntriesPerWarp);
    const unsigned blocks = (unsigned)trs::ceil_div64(warps, 8);
    const bool vec = (K % 8 == 0) && (((uintptr_t)X & 15) == 0) && (((uintptr_t)Y & 15) == 0);
    if (vec)
        trs::k_sddmm<true><<<blocks, 256, 0, st>>>(rowptr, col, (const __half*)X, (const __half*)Y, (__half*)out, n_rows, n_cols, nnz, K);
    else
        trs::k_sddmm<false><<<blocks, 256, 0, st>>>(rowptr, col, (const __half*)X, (const __half*)Y, (__half*)out, n_rows, n_cols, nnz, K);
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}
