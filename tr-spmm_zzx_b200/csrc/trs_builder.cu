// GPU format builder: CSR -> the reference's three-way hybrid format, bit-exact.
//
// Replaces block_sptc_2to4_online (TR-source/Block/block_online.cpp:545-871), which walks the
// windows serially on one CPU thread with hash maps and an O(U^2) unit graph.  Here every stage
// is a data-parallel pass over device arrays:
//
//   1. key = (window, column, local row) per entry, radix sort      -> per-window column lists
//      (the reference's col_info map, block_online.cpp:589-603)
//   2. run heads -> one record per (window, column): count, 16-bit row mask, first entry
//   3. stable sort by (window, 16 - count): the (count desc, column asc) order both funnels
//      use (block_online.cpp:226-230, 281-285)
//   4. TC funnel: leading columns with count >= density in chunks of 8, kept when
//      nnz/(window*8) >= tc_min_util (block_online.cpp:215-253)
//   5. units = consecutive pairs of the remaining columns (the first-fit of
//      block_online.cpp:287-326 always takes the next column because its bit test cannot fail)
//   6. matching (block_online.cpp:332-392): the unit graph is complete, so degrees are all
//      equal, the node order is libstdc++ std::sort of unit nnz (emulated step for step, see
//      trs_stdsort.cuh) and the partner of a node is the lowest-index unmatched other unit
//   7. group emission, per-row (value, position) slots with the reference's "first two kept,
//      the rest dropped" rule (block_online.cpp:629-703)
//   8. TC blocks, bitmaps, values, parts (block_online.cpp:444-540)
//   9. CUDA-core row parts from the columns of an unmatched sparse unit (block_online.cpp:397-439,
//      706-733)
//  10. 16x16 mma.sp tile packing (block_online.cpp:796-841; trs_pack.cu)
//
// Input contract: canonical CSR (columns strictly ascending inside a row), window in 1..16.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_reduce.cuh>
#include <cub/device/device_scan.cuh>

#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "trs_common.cuh"
#include "trs_stdsort.cuh"

namespace trs {

typedef unsigned long long u64;

struct BuildCfg {
    int part_t, part_c, short_size, density, window;
    float tc_min_util;
    int skip_tc, unit_min_nnz;
    int strict;  // 1: lossless — entries the reference drops go to the CUDA-core parts instead
};

// ---------------------------------------------------------------------------------------------
// stage kernels
// ---------------------------------------------------------------------------------------------
__global__ void kb_mark_rows(const int* __restrict__ rowptr, int n_rows, int* __restrict__ rowid, int* err) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int b = rowptr[r], e = rowptr[r + 1];
    if (e < b) { atomicOr(err, 1); return; }
    if (e > b) rowid[b] = r;
}

struct MaxOp {
    __device__ __forceinline__ int operator()(int a, int b) const { return a > b ? a : b; }
};

__global__ void kb_make_keys(const int* __restrict__ col, const int* __restrict__ rowid, long long nnz, int window,
                             int col_bits, u64* __restrict__ keys, int* __restrict__ edge, int* err) {
    long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = rowid[e], c = col[e];
    if (c < 0) atomicOr(err, 2);
    if (e + 1 < nnz && rowid[e + 1] == r && col[e + 1] <= c) atomicOr(err, 2);  // not canonical
    const int w = r / window, lr = r - w * window;
    keys[e] = ((u64)w << (col_bits + 4)) | ((u64)(unsigned)c << 4) | (u64)lr;
    edge[e] = (int)e;
}

__global__ void kb_heads(const u64* __restrict__ keys, long long nnz, int* __restrict__ head) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    head[i] = (i == 0 || (keys[i] >> 4) != (keys[i - 1] >> 4)) ? 1 : 0;
}

// wc_id (inclusive scan of heads) -> start position of every (window, column) record
__global__ void kb_wcol_start(const int* __restrict__ head, const int* __restrict__ wc_incl, long long nnz,
                              int* __restrict__ wc_start) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    if (head[i]) wc_start[wc_incl[i] - 1] = (int)i;
}

__global__ void kb_wcol_info(const u64* __restrict__ keys, const int* __restrict__ wc_start, int D, int col_bits,
                             int density, int skip_tc, int* __restrict__ wc_win, int* __restrict__ wc_col,
                             unsigned char* __restrict__ wc_count, unsigned short* __restrict__ wc_mask,
                             int* __restrict__ win_ncol, int* __restrict__ win_ncand, unsigned* __restrict__ key2) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= D) return;
    const int b = wc_start[j], e = wc_start[j + 1];
    const u64 k0 = keys[b];
    unsigned mask = 0;
    for (int i = b; i < e; ++i) mask |= 1u << (unsigned)(keys[i] & 15);
    const int w = (int)(k0 >> (col_bits + 4));
    const int count = e - b;
    wc_win[j] = w;
    wc_col[j] = (int)((k0 >> 4) & ((1ull << col_bits) - 1ull));
    wc_count[j] = (unsigned char)count;
    wc_mask[j] = (unsigned short)mask;
    // per-window counters, one atomic per warp and window (hub windows hold 10^5+ records)
    const unsigned active = __activemask();
    const unsigned peers = __match_any_sync(active, w);
    const bool cand = !skip_tc && count >= density;
    const unsigned cand_peers = __ballot_sync(active, cand) & peers;
    if ((threadIdx.x & 31) == __ffs(peers) - 1) {
        atomicAdd(&win_ncol[w], __popc(peers));
        if (cand_peers) atomicAdd(&win_ncand[w], __popc(cand_peers));
    }
    key2[j] = ((unsigned)w << 4) | (unsigned)(16 - count);
}

// Position p of the (count desc, col asc) order: TC membership of the column there.
__global__ void kb_tc_select(const int* __restrict__ ord, const int* __restrict__ wc_win,
                             const unsigned char* __restrict__ wc_count, const int* __restrict__ wc_begin,
                             const int* __restrict__ win_ncand, int D, int window, float tc_min_util,
                             int* __restrict__ not_tc, int* __restrict__ lead) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= D) return;
    const int j = ord[p];
    const int w = wc_win[j];
    const int wb = wc_begin[w];
    const int o = p - wb;
    const int ncand = win_ncand[w];
    int is_tc = 0, is_lead = 0;
    if (o < ncand) {
        const int cs = wb + (o / 8) * 8;
        const int ce = min(cs + 8, wb + ncand);
        int real_nnz = 0;
        for (int q = cs; q < ce; ++q) real_nnz += wc_count[ord[q]];
        const float util = __fdiv_rn((float)real_nnz, (float)(window * 8));
        if (!(util < tc_min_util)) { is_tc = 1; is_lead = (o % 8 == 0); }
    }
    not_tc[p] = !is_tc;
    lead[p] = is_lead;
}

__global__ void kb_compact(const int* __restrict__ ord, const int* __restrict__ not_tc, const int* __restrict__ lead,
                           const int* __restrict__ s_idx, const int* __restrict__ b_idx, const int* __restrict__ wc_win,
                           const int* __restrict__ wc_begin, const int* __restrict__ win_ncand, int D,
                           int* __restrict__ cand, int* __restrict__ blk_pos, int* __restrict__ blk_len) {
    int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= D) return;
    if (not_tc[p]) cand[s_idx[p]] = ord[p];
    if (lead[p]) {
        const int w = wc_win[ord[p]];
        const int end = wc_begin[w] + win_ncand[w];
        const int b = b_idx[p];
        blk_pos[b] = p;
        blk_len[b] = min(8, end - p);
    }
}

// per window: candidate range, units, pair slots, block range
__global__ void kb_window_counts(const int* __restrict__ wc_begin, const int* __restrict__ s_idx,
                                 const int* __restrict__ b_idx, int W, int part_t, int* __restrict__ win_cb,
                                 int* __restrict__ win_U, int* __restrict__ win_slots, int* __restrict__ win_bb,
                                 int* __restrict__ win_parts) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= W) return;
    const int pb = wc_begin[w], pe = wc_begin[w + 1];
    const int cb = s_idx[pb], ns = s_idx[pe] - cb;
    const int U = (ns + 1) / 2;
    win_cb[w] = cb;
    win_U[w] = U;
    win_slots[w] = (U + 1) / 2;
    const int bb = b_idx[pb], nb = b_idx[pe] - bb;
    win_bb[w] = bb;
    win_parts[w] = nb == 0 ? 0 : (nb <= part_t ? 1 : (nb + part_t - 1) / part_t);
}

// unit nnz: one thread per sparse-route candidate, even local index writes its unit
__global__ void kb_unit_nnz(const int* __restrict__ cand, int S, const int* __restrict__ wc_win,
                            const unsigned char* __restrict__ wc_count, const int* __restrict__ win_cb,
                            const int* __restrict__ win_ub, const int* __restrict__ win_cb_next_unused,
                            const int* __restrict__ win_U, unsigned char* __restrict__ unit_nnz) {
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= S) return;
    const int j = cand[s];
    const int w = wc_win[j];
    const int ls = s - win_cb[w];
    if (ls & 1) return;
    int nnz = wc_count[j];
    // the partner is the next candidate if it belongs to the same window
    if (s + 1 < S && wc_win[cand[s + 1]] == w) nnz += wc_count[cand[s + 1]];
    unit_nnz[win_ub[w] + (ls >> 1)] = (unsigned char)nnz;
}

struct UnitLess {
    const unsigned char* nnz;
    __host__ __device__ bool operator()(int a, int b) const { return nnz[a] > nnz[b]; }
};

// Matching of one window's units by one thread.  pair_a/pair_b get the groups in emission
// order: matched pairs in greedy order, then the unmatched unit (if it is kept).
__global__ void kb_match(const int* __restrict__ win_U, const int* __restrict__ win_ub,
                         const int* __restrict__ win_pb, int W, int unit_min_nnz,
                         const unsigned char* __restrict__ unit_nnz, int* __restrict__ order_buf,
                         unsigned char* __restrict__ matched_buf, int* __restrict__ pair_a, int* __restrict__ pair_b,
                         int* __restrict__ win_G, int* __restrict__ win_cuda_unit, const int* __restrict__ sel,
                         int n_sel) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_sel) return;
    const int w = sel ? sel[t] : t;
    const int U = win_U[w];
    int G = 0, cuda_unit = -1;
    if (U > 0) {
        const unsigned char* nnz = unit_nnz + win_ub[w];
        int* order = order_buf + win_ub[w];
        unsigned char* matched = matched_buf + win_ub[w];
        for (int i = 0; i < U; ++i) { order[i] = i; matched[i] = 0; }
        StdSort<UnitLess> sorter(order, UnitLess{nnz});
        sorter.sort(U);
        int* pa = pair_a + win_pb[w];
        int* pb = pair_b + win_pb[w];
        int lowest = 0;
        for (int k = 0; k < U; ++k) {
            const int idx = order[k];
            if (matched[idx]) continue;
            while (lowest < U && matched[lowest]) ++lowest;
            int partner = lowest;
            if (partner == idx) {
                ++partner;
                while (partner < U && matched[partner]) ++partner;
            }
            if (partner >= U) continue;  // idx stays unmatched
            matched[idx] = 1;
            matched[partner] = 1;
            pa[G] = idx;
            pb[G] = partner;
            ++G;
        }
        if (U & 1) {  // exactly one unit is left over
            int left = 0;
            while (matched[left]) ++left;
            if ((int)nnz[left] >= unit_min_nnz) { pa[G] = left; pb[G] = -1; ++G; }
            else cuda_unit = left;
        }
    }
    win_G[w] = G;
    win_cuda_unit[w] = cuda_unit;
}

// ---------------------------------------------------------------------------------------------
// Matching of a HEAVY window (tens of thousands to millions of units, the hub windows of a
// power-law graph) by one thread block.  Same result as kb_match, different execution:
//   * the std::sort emulation runs its partitions cooperatively.  An unguarded Hoare partition
//     swaps the k-th element >= pivot from the left with the k-th element <= pivot from the
//     right while the former lies left of the latter; with rank(i) = how many such elements
//     precede i, every thread can decide locally whether its element takes part and where its
//     partner is.  K swaps happen, the cut is min(position of the (K+1)-th left stopper, position
//     of the K-th right stopper) — checked against libstdc++ on the host, see tests;
//   * ranges of at most kParRange elements are finished by single threads with the sequential
//     emulation (introsort loop + the insertion pass restricted to the range);
//   * the greedy pass stays sequential (each step depends on all earlier ones) but runs out of
//     shared memory: a bitmask of matched units and tiles of the sorted order.
// ---------------------------------------------------------------------------------------------
constexpr int kMediumUnits = 96;    // above: one warp per window
constexpr int kHeavyUnits = 2048;    // above: one 256-thread block per window
constexpr int kOrderTile = 2048;

__global__ void kb_split_windows(const int* __restrict__ win_U, int W, int* __restrict__ light, int* __restrict__ medium,
                                 int* __restrict__ heavy, int* __restrict__ counters /* n_light, n_medium, n_heavy, max U */) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= W) return;
    const int U = win_U[w];
    if (U > kHeavyUnits) heavy[atomicAdd(&counters[2], 1)] = w;
    else if (U > kMediumUnits) medium[atomicAdd(&counters[1], 1)] = w;
    else light[atomicAdd(&counters[0], 1)] = w;
    atomicMax(&counters[3], U);
}

template <int kHeavyThreads, int kParRange>
__global__ void __launch_bounds__(kHeavyThreads) kb_match_coop(
    const int* __restrict__ win_U, const int* __restrict__ win_ub, const int* __restrict__ win_pb, int unit_min_nnz,
    const unsigned char* __restrict__ unit_nnz, int* __restrict__ order_buf, unsigned char* __restrict__ matched_buf,
    int* __restrict__ pair_a, int* __restrict__ pair_b, int* __restrict__ win_G, int* __restrict__ win_cuda_unit,
    const int* __restrict__ sel, int mask_words_cap) {
    extern __shared__ unsigned int dyn[];   // [mask_words_cap] matched bitmask, then [kOrderTile] order tile
    __shared__ int s_stack[64][3];
    __shared__ int s_small[kHeavyThreads][3];
    __shared__ int s_scan[kHeavyThreads];
    __shared__ int s_sp, s_nsmall, s_K, s_lnext, s_cur[3], s_G, s_cuda;
    const int tid = threadIdx.x;
    const int w = sel[blockIdx.x];
    const int U = win_U[w];
    const unsigned char* nnz = unit_nnz + win_ub[w];
    int* order = order_buf + win_ub[w];
    int* swapL = pair_a + win_pb[w];   // scratch during the sort, pair list afterwards
    int* swapR = pair_b + win_pb[w];
    for (int i = tid; i < U; i += kHeavyThreads) order[i] = i;
    if (tid == 0) {
        s_stack[0][0] = 0; s_stack[0][1] = U; s_stack[0][2] = 2 * StdSort<UnitLess>::floor_log2(U);
        s_sp = 1; s_nsmall = 0;
    }
    __syncthreads();
    StdSort<UnitLess> S(order, UnitLess{nnz});

    auto block_excl_scan = [&](int v, int& total) -> int {  // exclusive scan over threads (in order)
        s_scan[tid] = v;
        __syncthreads();
        for (int off = 1; off < kHeavyThreads; off <<= 1) {
            const int t = tid >= off ? s_scan[tid - off] : 0;
            __syncthreads();
            s_scan[tid] += t;
            __syncthreads();
        }
        total = s_scan[kHeavyThreads - 1];
        const int ex = s_scan[tid] - v;
        __syncthreads();
        return ex;
    };
    auto run_small = [&]() {  // every thread finishes one small range
        __syncthreads();
        if (tid < s_nsmall) {
            const int f = s_small[tid][0], l = s_small[tid][1], d = s_small[tid][2];
            if (d < 0) S.heap_sort(f, l - f);
            else { S.introsort_range(f, l, d); S.insertion_range(f, l); }
        }
        __syncthreads();
        if (tid == 0) s_nsmall = 0;
        __syncthreads();
    };

    while (true) {
        __syncthreads();
        const int sp_now = s_sp;   // read by everyone before thread 0 pops
        __syncthreads();
        if (sp_now == 0) break;
        if (tid == 0) {
            --s_sp;
            s_cur[0] = s_stack[s_sp][0]; s_cur[1] = s_stack[s_sp][1]; s_cur[2] = s_stack[s_sp][2];
        }
        __syncthreads();
        const int first = s_cur[0], last = s_cur[1];
        int depth = s_cur[2];
        if (last - first <= kParRange || depth == 0) {
            if (last - first > 1) {
                if (tid == 0) {
                    s_small[s_nsmall][0] = first; s_small[s_nsmall][1] = last;
                    s_small[s_nsmall][2] = (last - first > kParRange) ? -1 : depth;   // -1: depth exhausted -> heap sort
                    ++s_nsmall;
                }
                __syncthreads();
                if (s_nsmall == kHeavyThreads) run_small();
            }
            continue;
        }
        --depth;
        if (tid == 0) S.move_median_to_first(first, first + 1, first + (last - first) / 2, last - 1);
        __syncthreads();
        const int pvk = nnz[order[first]];
        const int lo = first + 1, n = last - lo;
        const int chunk = (n + kHeavyThreads - 1) / kHeavyThreads;
        const int cb = min(lo + tid * chunk, last), ce = min(cb + chunk, last);
        // pass 1: stoppers per chunk.  left stopper: key <= pivot key (not less than the pivot in
        // the descending order); right stopper: key >= pivot key
        int cL = 0, cR = 0;
        for (int i = cb; i < ce; ++i) {
            const int k = nnz[order[i]];
            cL += (k <= pvk);
            cR += (k >= pvk);
        }
        int totL, totR;
        const int baseL = block_excl_scan(cL, totL);
        const int exR = block_excl_scan(cR, totR);
        const int baseRright = totR - exR - cR;   // right stoppers in later chunks
        // pass 2a: which left stoppers swap; K = their number
        int lrank = baseL, rem = cR, myswaps = 0;
        for (int i = cb; i < ce; ++i) {
            const int k = nnz[order[i]];
            int right_of_i = baseRright + rem;
            if (k >= pvk) { right_of_i -= 1; rem -= 1; }
            if (k <= pvk) {
                ++lrank;
                if (right_of_i >= lrank) { swapL[lrank - 1] = i; ++myswaps; }
            }
        }
        int K;
        (void)block_excl_scan(myswaps, K);
        if (tid == 0) s_lnext = 0x7fffffff;
        __syncthreads();
        // pass 2b: the partners on the right, and the (K+1)-th left stopper
        lrank = baseL; rem = cR;
        for (int i = cb; i < ce; ++i) {
            const int k = nnz[order[i]];
            if (k >= pvk) {
                const int rrank = baseRright + rem;   // rank from the right, 1-based
                if (rrank <= K) swapR[rrank - 1] = i;
                rem -= 1;
            }
            if (k <= pvk) {
                ++lrank;
                if (lrank == K + 1) s_lnext = i;
            }
        }
        __syncthreads();
        const int cut = min(s_lnext, K >= 1 ? swapR[K - 1] : 0x7fffffff);
        __syncthreads();
        for (int k = tid; k < K; k += kHeavyThreads) {
            const int a = swapL[k], b = swapR[k];
            const int t = order[a]; order[a] = order[b]; order[b] = t;
        }
        __syncthreads();
        if (tid == 0) {
            s_stack[s_sp][0] = cut; s_stack[s_sp][1] = last; s_stack[s_sp][2] = depth; ++s_sp;
            s_stack[s_sp][0] = first; s_stack[s_sp][1] = cut; s_stack[s_sp][2] = depth; ++s_sp;
        }
    }
    run_small();

    // ---- greedy pass (block_online.cpp:365-386), thread 0 over shared-memory tiles --------------
    const int words = (U + 31) / 32;
    const bool in_smem = words <= mask_words_cap;
    unsigned int* mask = dyn;
    int* tile = (int*)(dyn + mask_words_cap);
    unsigned char* matched = matched_buf + win_ub[w];
    if (in_smem) { for (int i = tid; i < words; i += kHeavyThreads) mask[i] = 0u; }
    else { for (int i = tid; i < U; i += kHeavyThreads) matched[i] = 0; }
    if (tid == 0) { s_G = 0; s_cuda = -1; s_cur[0] = 0; }
    __syncthreads();
    auto is_set = [&](int i) -> bool { return in_smem ? ((mask[i >> 5] >> (i & 31)) & 1u) != 0 : matched[i] != 0; };
    auto set_bit = [&](int i) { if (in_smem) mask[i >> 5] |= 1u << (i & 31); else matched[i] = 1; };
    for (int k0 = 0; k0 < U; k0 += kOrderTile) {
        const int len = min(kOrderTile, U - k0);
        for (int i = tid; i < len; i += kHeavyThreads) tile[i] = order[k0 + i];
        __syncthreads();
        if (tid == 0) {
            int G = s_G, lowest = s_cur[0];
            for (int k = 0; k < len; ++k) {
                const int idx = tile[k];
                if (is_set(idx)) continue;
                while (lowest < U && is_set(lowest)) ++lowest;
                int partner = lowest;
                if (partner == idx) {
                    ++partner;
                    while (partner < U && is_set(partner)) ++partner;
                }
                if (partner >= U) continue;
                set_bit(idx); set_bit(partner);
                swapL[G] = idx; swapR[G] = partner;   // pair_a / pair_b of this window
                ++G;
            }
            s_G = G; s_cur[0] = lowest;
        }
        __syncthreads();
    }
    if (tid == 0) {
        int G = s_G;
        if (U & 1) {
            int left = 0;
            while (is_set(left)) ++left;
            if ((int)nnz[left] >= unit_min_nnz) { swapL[G] = left; swapR[G] = -1; ++G; }
            else s_cuda = left;
        }
        win_G[w] = G;
        win_cuda_unit[w] = s_cuda;
    }
}

__device__ __forceinline__ int find_window(const int* __restrict__ prefix, int W, int x) {
    // largest w in [0, W) with prefix[w] <= x   (prefix non-decreasing, prefix[W] > x)
    int lo = 0, hi = W;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

// one thread per pair slot: the group's columns, sorted ascending
__global__ void kb_emit_groups(const int* __restrict__ win_pb, const int* __restrict__ win_G,
                               const int* __restrict__ s_offset, const int* __restrict__ win_cb,
                               const int* __restrict__ win_U, const int* __restrict__ wc_begin,
                               const int* __restrict__ s_idx, int W, int total_slots, const int* __restrict__ pair_a,
                               const int* __restrict__ pair_b, const int* __restrict__ cand,
                               const int* __restrict__ wc_col, int* __restrict__ s_column, int* __restrict__ s_window,
                               int* __restrict__ grp_wcol) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= total_slots) return;
    const int w = find_window(win_pb, W, q);
    const int k = q - win_pb[w];
    if (k >= win_G[w]) return;
    const int g = s_offset[w] + k;
    const int cb = win_cb[w];
    const int ns = s_idx[wc_begin[w + 1]] - cb;
    int ids[4], cols[4], n = 0;
    const int ua = pair_a[q], ub = pair_b[q];
    for (int side = 0; side < 2; ++side) {
        const int u = side ? ub : ua;
        if (u < 0) continue;
        for (int i = 0; i < 2; ++i) {
            const int ls = 2 * u + i;
            if (ls < ns) { ids[n] = cand[cb + ls]; cols[n] = wc_col[ids[n]]; ++n; }
        }
    }
    for (int i = 1; i < n; ++i) {  // insertion sort by column id
        const int c = cols[i], id = ids[i];
        int k2 = i - 1;
        while (k2 >= 0 && cols[k2] > c) { cols[k2 + 1] = cols[k2]; ids[k2 + 1] = ids[k2]; --k2; }
        cols[k2 + 1] = c; ids[k2 + 1] = id;
    }
    for (int p = 0; p < 4; ++p) {
        s_column[(size_t)g * 4 + p] = p < n ? cols[p] : -1;
        grp_wcol[(size_t)g * 4 + p] = p < n ? ids[p] : -1;
    }
    s_window[g] = w;
}

// one thread per (group, local row): mask byte and the first two (value, position) slots.
// In strict mode the non-zeros beyond the second one (which the reference drops) are recorded in
// `extra_key` / `extra_at` (key = row << 32 | column) so that they can join the row's CUDA-core part.
__global__ void kb_emit_rows(const int* __restrict__ grp_wcol, long long total, int window,
                             const unsigned short* __restrict__ wc_mask, const int* __restrict__ wc_start,
                             const int* __restrict__ wc_col, const int* __restrict__ s_window,
                             const int* __restrict__ edge, const float* __restrict__ val,
                             unsigned char* __restrict__ s_mask, float* __restrict__ s_value,
                             signed char* __restrict__ s_pos, unsigned long long* __restrict__ dropped,
                             unsigned long long* __restrict__ extra_key, int* __restrict__ extra_at,
                             unsigned long long* __restrict__ extra_count, int* __restrict__ row_extra, int write_arrays) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long g = i / window;
    const int lr = (int)(i - g * window);
    unsigned mask = 0;
    int slots = 0;
    float rv[2] = {0.f, 0.f};
    int rp[2] = {-1, -1};
    for (int p = 0; p < 4; ++p) {
        const int j = grp_wcol[g * 4 + p];
        if (j < 0) break;
        const unsigned m = wc_mask[j];
        if (!((m >> lr) & 1u)) continue;
        mask |= 1u << p;
        const int at = wc_start[j] + __popc(m & ((1u << lr) - 1u));
        if (slots < 2) {
            rv[slots] = val[edge[at]];
            rp[slots] = p;
        } else if (extra_key) {
            const unsigned long long k = atomicAdd(extra_count, 1ull);
            const long long row = (long long)s_window[g] * window + lr;
            extra_key[k] = ((unsigned long long)row << 32) | (unsigned)wc_col[j];
            extra_at[k] = at;
            atomicAdd(&row_extra[row], 1);
        }
        ++slots;
    }
    if (!write_arrays) return;
    if (slots > 2) atomicAdd(dropped, (unsigned long long)(slots - 2));
    s_mask[i] = (unsigned char)mask;
    s_value[i * 2] = rv[0];
    s_value[i * 2 + 1] = rv[1];
    s_pos[i * 2] = (signed char)rp[0];
    s_pos[i * 2 + 1] = (signed char)rp[1];
}

// one thread per TC block: columns ascending, bitmaps, value count; records each column's slot
__global__ void kb_tc_blocks(const int* __restrict__ blk_pos, const int* __restrict__ blk_len, int NB,
                             const int* __restrict__ ord, const int* __restrict__ wc_col,
                             const unsigned short* __restrict__ wc_mask, int* __restrict__ t_column,
                             long long* __restrict__ t_binary, int* __restrict__ blk_nnz, int* __restrict__ wc_slot) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= NB) return;
    const int p0 = blk_pos[b], len = blk_len[b];
    int ids[8], cols[8];
    for (int i = 0; i < len; ++i) { ids[i] = ord[p0 + i]; cols[i] = wc_col[ids[i]]; }
    for (int i = 1; i < len; ++i) {
        const int c = cols[i], id = ids[i];
        int k = i - 1;
        while (k >= 0 && cols[k] > c) { cols[k + 1] = cols[k]; ids[k + 1] = ids[k]; --k; }
        cols[k + 1] = c; ids[k + 1] = id;
    }
    u64 lo = 0, hi = 0;
    for (int k = 0; k < 8; ++k) {
        t_column[(size_t)b * 8 + k] = k < len ? cols[k] : -1;
        if (k >= len) continue;
        wc_slot[ids[k]] = b * 8 + k;
        const unsigned m = wc_mask[ids[k]];
        for (int r = 0; r < 8; ++r) {
            if ((m >> r) & 1u) lo |= 1ull << (r * 8 + k);
            if ((m >> (r + 8)) & 1u) hi |= 1ull << (r * 8 + k);
        }
    }
    t_binary[(size_t)b * 2] = (long long)lo;
    t_binary[(size_t)b * 2 + 1] = (long long)hi;
    blk_nnz[b] = __popcll(lo) + __popcll(hi);
}

// one thread per sorted entry: entries of TC columns go to their slot of t_value
__global__ void kb_tc_values(const u64* __restrict__ keys, const int* __restrict__ edge,
                             const int* __restrict__ wc_incl, long long nnz, const int* __restrict__ wc_slot,
                             const long long* __restrict__ t_binary, const int* __restrict__ t_block_offset,
                             const float* __restrict__ val, float* __restrict__ t_value) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const int slot = wc_slot[wc_incl[i] - 1];
    if (slot < 0) return;
    const int b = slot >> 3, k = slot & 7;
    const int lr = (int)(keys[i] & 15);
    const u64 lo = (u64)t_binary[(size_t)b * 2], hi = (u64)t_binary[(size_t)b * 2 + 1];
    const int bit = (lr & 7) * 8 + k;
    int rank;
    if (lr < 8) rank = __popcll(lo & ((1ull << bit) - 1ull));
    else rank = __popcll(lo) + __popcll(hi & ((1ull << bit) - 1ull));
    t_value[(size_t)t_block_offset[b] + rank] = val[edge[i]];
}

__global__ void kb_tc_parts(const int* __restrict__ wc_begin, const int* __restrict__ b_idx,
                            const int* __restrict__ win_bb, const int* __restrict__ part_off,
                            const int* __restrict__ win_cuda_unit, int W, int part_t, int* __restrict__ t_row_offset,
                            int* __restrict__ t_window_row, int* __restrict__ t_atomic) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w == 0) t_row_offset[0] = 0;
    if (w >= W) return;
    const int bb = win_bb[w];
    const int nb = b_idx[wc_begin[w + 1]] - bb;
    if (nb == 0) return;
    const int p0 = part_off[w];
    if (nb <= part_t) {
        t_row_offset[p0 + 1] = bb + nb;
        t_window_row[p0] = w * 16;
        t_atomic[p0] = win_cuda_unit[w] >= 0 ? 1 : 0;
        return;
    }
    const int np = (nb + part_t - 1) / part_t;
    for (int q = 0; q < np; ++q) {
        t_row_offset[p0 + q + 1] = bb + min((q + 1) * part_t, nb);
        t_window_row[p0 + q] = w * 16;
        t_atomic[p0 + q] = 1;
    }
}

// CUDA-core leftovers: the (at most two) columns of the window's rejected unit.  Per row the
// entries come in ascending column order = CSR order.
struct CudaRow {
    int n;
    int cols[2];
    int at[2];  // position in the sorted entry array
};
__device__ __forceinline__ CudaRow cuda_row(int r, int window, const int* win_cuda_unit, const int* win_cb,
                                            const int* wc_begin, const int* s_idx, const int* cand, const int* wc_col,
                                            const unsigned short* wc_mask, const int* wc_start) {
    CudaRow out;
    out.n = 0;
    const int w = r / window, lr = r - w * window;
    const int u = win_cuda_unit[w];
    if (u < 0) return out;
    const int cb = win_cb[w];
    const int ns = s_idx[wc_begin[w + 1]] - cb;
    for (int i = 0; i < 2; ++i) {
        const int ls = 2 * u + i;
        if (ls >= ns) break;
        const int j = cand[cb + ls];
        const unsigned m = wc_mask[j];
        if (!((m >> lr) & 1u)) continue;
        out.cols[out.n] = wc_col[j];
        out.at[out.n] = wc_start[j] + __popc(m & ((1u << lr) - 1u));
        ++out.n;
    }
    if (out.n == 2 && out.cols[0] > out.cols[1]) {
        int t = out.cols[0]; out.cols[0] = out.cols[1]; out.cols[1] = t;
        t = out.at[0]; out.at[0] = out.at[1]; out.at[1] = t;
    }
    return out;
}

// split rule of block_online.cpp:415-439 as (long parts, short parts, long nnz, short nnz)
__device__ __forceinline__ void split_counts(int n, int part_c, int short_size, int& nl, int& ns, int& zl, int& zs) {
    nl = ns = zl = zs = 0;
    if (n <= 0) return;
    if (n <= short_size) { ns = 1; zs = n; return; }
    if (n <= part_c) { nl = 1; zl = n; return; }
    nl = n / part_c;
    zl = nl * part_c;
    const int residue = n % part_c;
    if (residue > 0) {
        if (residue <= short_size) { ns = 1; zs = residue; }
        else { nl += 1; zl += residue; }
    }
}

__global__ void kb_cuda_count(int n_rows, int window, int part_c, int short_size, const int* win_cuda_unit,
                              const int* win_cb, const int* wc_begin, const int* s_idx, const int* cand,
                              const int* wc_col, const unsigned short* wc_mask, const int* wc_start,
                              const int* __restrict__ row_extra, int* __restrict__ cnt /* 4 arrays of n_rows + 1 */) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const CudaRow cr = cuda_row(r, window, win_cuda_unit, win_cb, wc_begin, s_idx, cand, wc_col, wc_mask, wc_start);
    int nl, ns, zl, zs;
    split_counts(cr.n + (row_extra ? row_extra[r] : 0), part_c, short_size, nl, ns, zl, zs);
    const size_t stride = (size_t)n_rows + 1;
    cnt[r] = nl; cnt[stride + r] = ns; cnt[2 * stride + r] = zl; cnt[3 * stride + r] = zs;
}

// The row's leftover entries in ascending column order: the (at most two) entries of the window's
// rejected unit merged with the row's strict-mode extras (sorted by column beforehand).
__global__ void kb_cuda_fill(int n_rows, int window, int part_c, int short_size, const int* win_cuda_unit,
                             const int* win_cb, const int* wc_begin, const int* s_idx, const int* b_idx,
                             const int* cand, const int* wc_col, const unsigned short* wc_mask, const int* wc_start,
                             const int* edge, const float* val, const int* __restrict__ off,
                             const int* __restrict__ extra_off, const unsigned long long* __restrict__ extra_key,
                             const int* __restrict__ extra_at,
                             int* c_row_offset, int* c_row, int* c_atomic, int* c_column, float* c_value,
                             int* cs_row_offset, int* cs_row, int* cs_atomic, int* cs_column, float* cs_value) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r == 0) { c_row_offset[0] = 0; cs_row_offset[0] = 0; }
    if (r >= n_rows) return;
    const CudaRow cr = cuda_row(r, window, win_cuda_unit, win_cb, wc_begin, s_idx, cand, wc_col, wc_mask, wc_start);
    const int xb = extra_off ? extra_off[r] : 0, xe = extra_off ? extra_off[r + 1] : 0;
    const int n = cr.n + (xe - xb);
    if (n <= 0) return;
    const int w = r / window;
    const int base_atomic = (b_idx[wc_begin[w + 1]] - b_idx[wc_begin[w]]) > 0 ? 1 : 0;
    const size_t stride = (size_t)n_rows + 1;
    int pl = off[r], ps = off[stride + r], zl = off[2 * stride + r], zs = off[3 * stride + r];
    int iu = 0, ix = xb;  // cursors of the two sorted sources
    auto next = [&](int& c, float& v) {
        const int xc = ix < xe ? (int)(extra_key[ix] & 0xffffffffull) : 0x7fffffff;
        if (iu < cr.n && cr.cols[iu] < xc) { c = cr.cols[iu]; v = val[edge[cr.at[iu]]]; ++iu; }
        else { c = xc; v = val[edge[extra_at[ix]]]; ++ix; }
    };
    auto put = [&](int atomic, int cnt, bool residue) {
        for (int i = 0; i < cnt; ++i) {
            int c; float v;
            next(c, v);
            if (residue) { cs_column[zs + i] = c; cs_value[zs + i] = v; }
            else { c_column[zl + i] = c; c_value[zl + i] = v; }
        }
        if (residue) { zs += cnt; cs_row[ps] = r; cs_atomic[ps] = atomic; cs_row_offset[ps + 1] = zs; ++ps; }
        else { zl += cnt; c_row[pl] = r; c_atomic[pl] = atomic; c_row_offset[pl + 1] = zl; ++pl; }
    };
    if (n <= short_size) { put(base_atomic, n, true); return; }
    if (n <= part_c) { put(base_atomic, n, false); return; }
    for (int i = 0; i < n / part_c; ++i) put(1, part_c, false);
    const int residue = n % part_c;
    if (residue > 0) put(1, residue, residue <= short_size);
}

__global__ void kb_tiles(const int* __restrict__ tile_off, const int* __restrict__ s_offset, int W, int T,
                         int* __restrict__ s_tile_window, int* __restrict__ s_tile_group) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int w = find_window(tile_off, W, t);
    s_tile_window[t] = w;
    s_tile_group[t] = s_offset[w] + 4 * (t - tile_off[w]);
}

__global__ void kb_win_tiles(const int* __restrict__ win_G, int W, int* __restrict__ win_T) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w < W) win_T[w] = (win_G[w] + 3) / 4;
}

__global__ void kb_iota(int* __restrict__ p, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = i;
}

__global__ void kb_to_half(const float* __restrict__ src, long long n, __half* __restrict__ dst) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __float2half_rn(src[i]);
}

}  // namespace trs

// ---------------------------------------------------------------------------------------------
// host orchestration
// ---------------------------------------------------------------------------------------------
using namespace trs;

struct trs_builder {
    BuildCfg cfg;
    Arena arena_store;
    Arena* arena = nullptr;   // set: outputs and scratch come from the caller's memory
    int n_rows = 0, W = 0;
    long long nnz = 0;
    // the 29 arrays, reference order (block_online.cpp:844-870)
    DevBuf<int> t_row_offset, t_block_offset, t_column, t_window_row, t_atomic;
    DevBuf<float> t_value;
    DevBuf<long long> t_binary;
    DevBuf<int> c_row_offset, c_row, c_atomic, c_column;
    DevBuf<float> c_value;
    DevBuf<int> cs_row_offset, cs_row, cs_atomic, cs_column;
    DevBuf<float> cs_value;
    DevBuf<int> s_column, s_window, s_offset, s_tile_window, s_tile_group, s_tile_column, s_window_tile_offset;
    DevBuf<unsigned char> s_mask;
    DevBuf<float> s_value;
    DevBuf<signed char> s_pos;
    DevBuf<uint32_t> s_packed_a, s_packed_meta;
    DevBuf<__half> t_value_h, c_value_h, cs_value_h;
    long long sizes[TRS_BUILD_NUM_ARRAYS];
    unsigned long long dropped = 0;
    long long distinct_cols = 0, units = 0;
    float build_ms = 0.f;

    void release() {
        t_row_offset.release(); t_block_offset.release(); t_column.release(); t_window_row.release();
        t_atomic.release(); t_value.release(); t_binary.release();
        c_row_offset.release(); c_row.release(); c_atomic.release(); c_column.release(); c_value.release();
        cs_row_offset.release(); cs_row.release(); cs_atomic.release(); cs_column.release(); cs_value.release();
        s_column.release(); s_window.release(); s_offset.release(); s_tile_window.release(); s_tile_group.release();
        s_tile_column.release(); s_window_tile_offset.release(); s_mask.release(); s_value.release(); s_pos.release();
        s_packed_a.release(); s_packed_meta.release(); t_value_h.release(); c_value_h.release(); cs_value_h.release();
    }
};

namespace {

struct Scratch {  // frees everything it handed out (or gives it back to the caller's arena)
    Arena* arena = nullptr;
    std::vector<void*> ptrs;
    std::vector<size_t> bytes;
    ~Scratch() {
        for (size_t i = ptrs.size(); i-- > 0;)
            if (ptrs[i]) {
                if (arena) arena->give_back(ptrs[i], bytes[i]);
                else cudaFree(ptrs[i]);
            }
    }
    template <class T>
    int get(size_t n, T** out) {
        void* d = nullptr;
        const size_t nb = (n ? n : 1) * sizeof(T);
        if (arena) {
            d = arena->take(nb);
            if (!d) { *out = nullptr; return TRS_E_WORKSPACE; }
        } else {
            cudaError_t e = cudaMalloc(&d, nb);
            if (e != cudaSuccess) { *out = nullptr; return (int)e; }
        }
        ptrs.push_back(d);
        bytes.push_back(nb);
        *out = (T*)d;
        return 0;
    }
    void drop(void* p) {
        for (size_t i = 0; i < ptrs.size(); ++i)
            if (ptrs[i] == p) {
                if (arena) arena->give_back(p, bytes[i]);
                else cudaFree(p);
                ptrs[i] = nullptr;
            }
    }
};

inline unsigned grid_for(long long n, int block = 256) { return (unsigned)((n + block - 1) / block); }

int bits_for(long long max_value) {  // bits needed to store values in [0, max_value]
    int b = 1;
    while ((1ll << b) <= max_value && b < 62) ++b;
    return b;
}

#define TRS_TRY(expr) do { int _rc = (expr); if (_rc) return _rc; } while (0)

struct Cub {
    Scratch& sc;
    void* tmp = nullptr;
    size_t cap = 0;
    cudaStream_t st;
    Cub(Scratch& s, cudaStream_t stream) : sc(s), st(stream) {}
    int reserve(size_t bytes) {
        if (bytes <= cap) return 0;
        if (tmp) sc.drop(tmp);
        unsigned char* p;
        TRS_TRY(sc.get<unsigned char>(bytes, &p));
        tmp = p; cap = bytes;
        return 0;
    }
    int exclusive_sum(const int* in, int* out, long long n) {
        size_t bytes = 0;
        TRS_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, bytes, in, out, n, st));
        TRS_TRY(reserve(bytes));
        TRS_CUDA(cub::DeviceScan::ExclusiveSum(tmp, bytes, in, out, n, st));
        return 0;
    }
    int inclusive_sum(const int* in, int* out, long long n) {
        size_t bytes = 0;
        TRS_CUDA(cub::DeviceScan::InclusiveSum(nullptr, bytes, in, out, n, st));
        TRS_TRY(reserve(bytes));
        TRS_CUDA(cub::DeviceScan::InclusiveSum(tmp, bytes, in, out, n, st));
        return 0;
    }
    int inclusive_max(int* inout, long long n) {
        size_t bytes = 0;
        TRS_CUDA(cub::DeviceScan::InclusiveScan(nullptr, bytes, inout, inout, MaxOp(), n, st));
        TRS_TRY(reserve(bytes));
        TRS_CUDA(cub::DeviceScan::InclusiveScan(tmp, bytes, inout, inout, MaxOp(), n, st));
        return 0;
    }
    int max_reduce(const int* in, int* out, long long n) {
        size_t bytes = 0;
        TRS_CUDA(cub::DeviceReduce::Max(nullptr, bytes, in, out, n, st));
        TRS_TRY(reserve(bytes));
        TRS_CUDA(cub::DeviceReduce::Max(tmp, bytes, in, out, n, st));
        return 0;
    }
    template <class K, class V>
    int sort_pairs(K* k_in, K* k_out, V* v_in, V* v_out, long long n, int end_bit, K** k_res, V** v_res) {
        cub::DoubleBuffer<K> kb(k_in, k_out);
        cub::DoubleBuffer<V> vb(v_in, v_out);
        size_t bytes = 0;
        TRS_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, bytes, kb, vb, n, 0, end_bit, st));
        TRS_TRY(reserve(bytes));
        TRS_CUDA(cub::DeviceRadixSort::SortPairs(tmp, bytes, kb, vb, n, 0, end_bit, st));
        *k_res = kb.Current();
        *v_res = vb.Current();
        return 0;
    }
};

int read_int(const int* dev, cudaStream_t st, int* out) {
    TRS_CUDA(cudaMemcpyAsync(out, dev, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    return 0;
}

int do_build(trs_builder* B, const int* rowptr, const int* col, const float* val, cudaStream_t st) {
    const BuildCfg& cfg = B->cfg;
    const int n = B->n_rows, window = cfg.window;
    const int W = B->W;
    Scratch sc;
    sc.arena = B->arena;
    Cub cub_(sc, st);
    int* d_err;
    TRS_TRY(sc.get<int>(4, &d_err));
    TRS_CUDA(cudaMemsetAsync(d_err, 0, 4 * sizeof(int), st));

    int first = 0, last = 0;
    TRS_CUDA(cudaMemcpyAsync(&first, rowptr, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_TRY(read_int(rowptr + n, st, &last));
    if (first != 0 || last < 0) return TRS_E_OFFSETS;
    const long long nnz = last;
    B->nnz = nnz;

    // outputs that exist even for an empty matrix
    TRS_TRY(B->s_offset.alloc_from(B->arena, (size_t)W + 1));
    TRS_TRY(B->s_window_tile_offset.alloc_from(B->arena, (size_t)W + 1));
    TRS_TRY(B->t_row_offset.alloc_from(B->arena, 1));
    TRS_TRY(B->t_block_offset.alloc_from(B->arena, 1));
    TRS_TRY(B->c_row_offset.alloc_from(B->arena, 1));
    TRS_TRY(B->cs_row_offset.alloc_from(B->arena, 1));
    TRS_CUDA(cudaMemsetAsync(B->s_offset.p, 0, sizeof(int) * (W + 1), st));
    TRS_CUDA(cudaMemsetAsync(B->s_window_tile_offset.p, 0, sizeof(int) * (W + 1), st));
    TRS_CUDA(cudaMemsetAsync(B->t_row_offset.p, 0, sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(B->t_block_offset.p, 0, sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(B->c_row_offset.p, 0, sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(B->cs_row_offset.p, 0, sizeof(int), st));
    if (nnz == 0) {
        int h = 0;
        kb_mark_rows<<<grid_for(n), 256, 0, st>>>(rowptr, n, d_err, d_err);  // only the monotonicity check fires
        TRS_TRY(read_int(d_err, st, &h));
        return (h & 1) ? TRS_E_OFFSETS : TRS_OK;
    }

    // ---- 1. row ids, keys, sort ----------------------------------------------------------------
    int* rowid;
    TRS_TRY(sc.get<int>(nnz, &rowid));
    TRS_CUDA(cudaMemsetAsync(rowid, 0, sizeof(int) * nnz, st));
    kb_mark_rows<<<grid_for(n), 256, 0, st>>>(rowptr, n, rowid, d_err);
    TRS_LAUNCH_CHECK();
    {
        int h = 0;
        TRS_TRY(read_int(d_err, st, &h));
        if (h & 1) return TRS_E_OFFSETS;  // a decreasing row pointer would also corrupt the scatter above
    }
    TRS_TRY(cub_.inclusive_max(rowid, nnz));
    int* d_max;
    TRS_TRY(sc.get<int>(1, &d_max));
    TRS_TRY(cub_.max_reduce(col, d_max, nnz));
    int max_col = 0;
    TRS_TRY(read_int(d_max, st, &max_col));
    if (max_col < 0) return TRS_E_NOT_CANONICAL;
    const int col_bits = bits_for(max_col);
    const int w_bits = bits_for(W > 0 ? W - 1 : 0);

    u64 *keys_a, *keys_b, *keys;
    int *edge_a, *edge_b, *edge;
    TRS_TRY(sc.get<u64>(nnz, &keys_a));
    TRS_TRY(sc.get<u64>(nnz, &keys_b));
    TRS_TRY(sc.get<int>(nnz, &edge_a));
    TRS_TRY(sc.get<int>(nnz, &edge_b));
    kb_make_keys<<<grid_for(nnz), 256, 0, st>>>(col, rowid, nnz, window, col_bits, keys_a, edge_a, d_err);
    TRS_LAUNCH_CHECK();
    TRS_TRY(cub_.sort_pairs(keys_a, keys_b, edge_a, edge_b, nnz, 4 + col_bits + w_bits, &keys, &edge));
    {
        int h = 0;
        TRS_TRY(read_int(d_err, st, &h));
        if (h & 2) return TRS_E_NOT_CANONICAL;
    }
    sc.drop(rowid);
    sc.drop(keys == keys_a ? (void*)keys_b : (void*)keys_a);
    sc.drop(edge == edge_a ? (void*)edge_b : (void*)edge_a);

    // ---- 2. one record per (window, column) ----------------------------------------------------
    int *head, *wc_incl;
    TRS_TRY(sc.get<int>(nnz, &head));
    TRS_TRY(sc.get<int>(nnz, &wc_incl));
    kb_heads<<<grid_for(nnz), 256, 0, st>>>(keys, nnz, head);
    TRS_LAUNCH_CHECK();
    TRS_TRY(cub_.inclusive_sum(head, wc_incl, nnz));
    int D = 0;
    TRS_TRY(read_int(wc_incl + (nnz - 1), st, &D));
    B->distinct_cols = D;
    int *wc_start, *wc_win, *wc_col, *win_ncol, *win_ncand, *wc_begin;
    unsigned char* wc_count;
    unsigned short* wc_mask;
    unsigned *key2_a, *key2_b, *key2;
    int *ord_a, *ord_b, *ord;
    TRS_TRY(sc.get<int>((size_t)D + 1, &wc_start));
    TRS_TRY(sc.get<int>(D, &wc_win));
    TRS_TRY(sc.get<int>(D, &wc_col));
    TRS_TRY(sc.get<unsigned char>(D, &wc_count));
    TRS_TRY(sc.get<unsigned short>(D, &wc_mask));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_ncol));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_ncand));
    TRS_TRY(sc.get<int>((size_t)W + 1, &wc_begin));
    TRS_TRY(sc.get<unsigned>(D, &key2_a));
    TRS_TRY(sc.get<unsigned>(D, &key2_b));
    TRS_TRY(sc.get<int>(D, &ord_a));
    TRS_TRY(sc.get<int>(D, &ord_b));
    TRS_CUDA(cudaMemsetAsync(win_ncol, 0, sizeof(int) * (W + 1), st));
    TRS_CUDA(cudaMemsetAsync(win_ncand, 0, sizeof(int) * (W + 1), st));
    kb_wcol_start<<<grid_for(nnz), 256, 0, st>>>(head, wc_incl, nnz, wc_start);
    const int nnz_i = (int)nnz;
    TRS_CUDA(cudaMemcpyAsync(wc_start + D, &nnz_i, sizeof(int), cudaMemcpyHostToDevice, st));
    kb_wcol_info<<<grid_for(D), 256, 0, st>>>(keys, wc_start, D, col_bits, cfg.density, cfg.skip_tc, wc_win, wc_col,
                                               wc_count, wc_mask, win_ncol, win_ncand, key2_a);
    TRS_LAUNCH_CHECK();
    TRS_TRY(cub_.exclusive_sum(win_ncol, wc_begin, W + 1));
    sc.drop(head);

    // ---- 3. (count desc, col asc) order inside each window ---------------------------------------
    kb_iota<<<grid_for(D), 256, 0, st>>>(ord_a, D);
    TRS_LAUNCH_CHECK();
    TRS_TRY(cub_.sort_pairs(key2_a, key2_b, ord_a, ord_b, (long long)D, 4 + w_bits, &key2, &ord));  // LSD radix: stable

    // ---- 4. TC funnel ----------------------------------------------------------------------------
    int *not_tc, *lead, *s_idx, *b_idx;
    TRS_TRY(sc.get<int>((size_t)D + 1, &not_tc));
    TRS_TRY(sc.get<int>((size_t)D + 1, &lead));
    TRS_TRY(sc.get<int>((size_t)D + 1, &s_idx));
    TRS_TRY(sc.get<int>((size_t)D + 1, &b_idx));
    TRS_CUDA(cudaMemsetAsync(not_tc + D, 0, sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(lead + D, 0, sizeof(int), st));
    kb_tc_select<<<grid_for(D), 256, 0, st>>>(ord, wc_win, wc_count, wc_begin, win_ncand, D, window, cfg.tc_min_util,
                                               not_tc, lead);
    TRS_LAUNCH_CHECK();
    TRS_TRY(cub_.exclusive_sum(not_tc, s_idx, (long long)D + 1));
    TRS_TRY(cub_.exclusive_sum(lead, b_idx, (long long)D + 1));
    int S = 0, NB = 0;
    TRS_CUDA(cudaMemcpyAsync(&S, s_idx + D, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_TRY(read_int(b_idx + D, st, &NB));
    int *cand, *blk_pos, *blk_len;
    TRS_TRY(sc.get<int>(S, &cand));
    TRS_TRY(sc.get<int>(NB, &blk_pos));
    TRS_TRY(sc.get<int>(NB, &blk_len));
    kb_compact<<<grid_for(D), 256, 0, st>>>(ord, not_tc, lead, s_idx, b_idx, wc_win, wc_begin, win_ncand, D, cand,
                                             blk_pos, blk_len);
    TRS_LAUNCH_CHECK();

    // ---- 5. units ---------------------------------------------------------------------------------
    int *win_cb, *win_U, *win_slots, *win_bb, *win_parts, *win_ub, *win_pb, *part_off;
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_cb));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_U));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_slots));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_bb));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_parts));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_ub));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_pb));
    TRS_TRY(sc.get<int>((size_t)W + 1, &part_off));
    TRS_CUDA(cudaMemsetAsync(win_U + W, 0, sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(win_slots + W, 0, sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(win_parts + W, 0, sizeof(int), st));
    kb_window_counts<<<grid_for(W), 256, 0, st>>>(wc_begin, s_idx, b_idx, W, cfg.part_t, win_cb, win_U, win_slots,
                                                   win_bb, win_parts);
    TRS_LAUNCH_CHECK();
    TRS_TRY(cub_.exclusive_sum(win_U, win_ub, W + 1));
    TRS_TRY(cub_.exclusive_sum(win_slots, win_pb, W + 1));
    TRS_TRY(cub_.exclusive_sum(win_parts, part_off, W + 1));
    int TU = 0, TS = 0, NP = 0;
    TRS_CUDA(cudaMemcpyAsync(&TU, win_ub + W, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaMemcpyAsync(&TS, win_pb + W, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_TRY(read_int(part_off + W, st, &NP));
    B->units = TU;
    unsigned char *unit_nnz, *matched;
    int *order_buf, *pair_a, *pair_b, *win_G, *win_cuda_unit;
    TRS_TRY(sc.get<unsigned char>(TU, &unit_nnz));
    TRS_TRY(sc.get<unsigned char>(TU, &matched));
    TRS_TRY(sc.get<int>(TU, &order_buf));
    TRS_TRY(sc.get<int>(TS, &pair_a));
    TRS_TRY(sc.get<int>(TS, &pair_b));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_G));
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_cuda_unit));
    TRS_CUDA(cudaMemsetAsync(win_G + W, 0, sizeof(int), st));
    if (S > 0) {
        kb_unit_nnz<<<grid_for(S), 256, 0, st>>>(cand, S, wc_win, wc_count, win_cb, win_ub, nullptr, win_U, unit_nnz);
        TRS_LAUNCH_CHECK();
    }

    // ---- 6. matching -----------------------------------------------------------------------------
    // small windows: one thread each; medium: one warp each; heavy (hubs): one 256-thread block each
    int *sel_light, *sel_medium, *sel_heavy, *sel_cnt;
    TRS_TRY(sc.get<int>((size_t)W + 1, &sel_light));
    TRS_TRY(sc.get<int>((size_t)W + 1, &sel_medium));
    TRS_TRY(sc.get<int>((size_t)W + 1, &sel_heavy));
    TRS_TRY(sc.get<int>(4, &sel_cnt));
    TRS_CUDA(cudaMemsetAsync(sel_cnt, 0, 4 * sizeof(int), st));
    kb_split_windows<<<grid_for(W), 256, 0, st>>>(win_U, W, sel_light, sel_medium, sel_heavy, sel_cnt);
    TRS_LAUNCH_CHECK();
    int h_cnt[4] = {0, 0, 0, 0};
    TRS_CUDA(cudaMemcpyAsync(h_cnt, sel_cnt, 4 * sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    if (h_cnt[0] > 0) {
        kb_match<<<grid_for(h_cnt[0], 64), 64, 0, st>>>(win_U, win_ub, win_pb, W, cfg.unit_min_nnz, unit_nnz, order_buf,
                                                          matched, pair_a, pair_b, win_G, win_cuda_unit, sel_light, h_cnt[0]);
        TRS_LAUNCH_CHECK();
    }
    if (h_cnt[1] > 0) {
        const int cap_words = (kHeavyUnits + 31) / 32;
        const size_t smem = (size_t)cap_words * 4 + (size_t)kOrderTile * 4;
        kb_match_coop<32, 64><<<h_cnt[1], 32, smem, st>>>(win_U, win_ub, win_pb, cfg.unit_min_nnz, unit_nnz, order_buf, matched,
                                                          pair_a, pair_b, win_G, win_cuda_unit, sel_medium, cap_words);
        TRS_LAUNCH_CHECK();
    }
    if (h_cnt[2] > 0) {
        // shared memory: bitmask of matched units (as many words as fit) + one tile of the order
        const int max_words = (h_cnt[3] + 31) / 32;
        const int cap_words = std::min(max_words, (200 * 1024 - kOrderTile * 4) / 4);
        const size_t smem = (size_t)cap_words * 4 + (size_t)kOrderTile * 4;
        TRS_CUDA(cudaFuncSetAttribute(kb_match_coop<256, 1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kb_match_coop<256, 1024><<<h_cnt[2], 256, smem, st>>>(win_U, win_ub, win_pb, cfg.unit_min_nnz, unit_nnz, order_buf,
                                                              matched, pair_a, pair_b, win_G, win_cuda_unit, sel_heavy,
                                                              cap_words);
        TRS_LAUNCH_CHECK();
    }
    TRS_TRY(cub_.exclusive_sum(win_G, B->s_offset.p, W + 1));
    int G = 0;
    TRS_TRY(read_int(B->s_offset.p + W, st, &G));

    // ---- 7. groups ---------------------------------------------------------------------------------
    int* grp_wcol;
    TRS_TRY(sc.get<int>((size_t)G * 4, &grp_wcol));
    TRS_TRY(B->s_column.alloc_from(B->arena, (size_t)G * 4));
    TRS_TRY(B->s_window.alloc_from(B->arena, G));
    TRS_TRY(B->s_mask.alloc_from(B->arena, (size_t)G * window));
    TRS_TRY(B->s_value.alloc_from(B->arena, (size_t)G * window * 2));
    TRS_TRY(B->s_pos.alloc_from(B->arena, (size_t)G * window * 2));
    unsigned long long* d_dropped;
    TRS_TRY(sc.get<unsigned long long>(1, &d_dropped));
    TRS_CUDA(cudaMemsetAsync(d_dropped, 0, sizeof(unsigned long long), st));
    if (G > 0) {
        kb_emit_groups<<<grid_for(TS), 256, 0, st>>>(win_pb, win_G, B->s_offset.p, win_cb, win_U, wc_begin, s_idx, W, TS,
                                                      pair_a, pair_b, cand, wc_col, B->s_column.p, B->s_window.p, grp_wcol);
        TRS_LAUNCH_CHECK();
        kb_emit_rows<<<grid_for((long long)G * window), 256, 0, st>>>(grp_wcol, (long long)G * window, window, wc_mask,
                                                                       wc_start, wc_col, B->s_window.p, edge, val,
                                                                       B->s_mask.p, B->s_value.p, B->s_pos.p, d_dropped,
                                                                       nullptr, nullptr, nullptr, nullptr, 1);
        TRS_LAUNCH_CHECK();
    }
    // strict mode: collect what was dropped, ordered by (row, column)
    int* row_extra = nullptr;
    int* extra_off = nullptr;
    unsigned long long* extra_key = nullptr;
    int* extra_at = nullptr;
    if (cfg.strict && G > 0) {
        unsigned long long h_dropped = 0;
        TRS_CUDA(cudaMemcpyAsync(&h_dropped, d_dropped, sizeof(h_dropped), cudaMemcpyDeviceToHost, st));
        TRS_CUDA(cudaStreamSynchronize(st));
        if (h_dropped > 0) {
            unsigned long long *key_a, *key_b, *d_xcount;
            int *at_a, *at_b;
            TRS_TRY(sc.get<unsigned long long>(h_dropped, &key_a));
            TRS_TRY(sc.get<unsigned long long>(h_dropped, &key_b));
            TRS_TRY(sc.get<int>(h_dropped, &at_a));
            TRS_TRY(sc.get<int>(h_dropped, &at_b));
            TRS_TRY(sc.get<unsigned long long>(1, &d_xcount));
            TRS_TRY(sc.get<int>((size_t)n + 1, &row_extra));
            TRS_TRY(sc.get<int>((size_t)n + 1, &extra_off));
            TRS_CUDA(cudaMemsetAsync(d_xcount, 0, sizeof(unsigned long long), st));
            TRS_CUDA(cudaMemsetAsync(row_extra, 0, sizeof(int) * ((size_t)n + 1), st));
            kb_emit_rows<<<grid_for((long long)G * window), 256, 0, st>>>(grp_wcol, (long long)G * window, window, wc_mask,
                                                                           wc_start, wc_col, B->s_window.p, edge, val, nullptr,
                                                                           nullptr, nullptr, nullptr, key_a, at_a, d_xcount,
                                                                           row_extra, 0);
            TRS_LAUNCH_CHECK();
            TRS_TRY(cub_.sort_pairs(key_a, key_b, at_a, at_b, (long long)h_dropped, 32 + bits_for(n), &extra_key, &extra_at));
            TRS_TRY(cub_.exclusive_sum(row_extra, extra_off, (long long)n + 1));
            TRS_CUDA(cudaMemsetAsync(d_dropped, 0, sizeof(unsigned long long), st));   // nothing is lost in this mode
        }
    }

    // ---- 8. TC blocks, values, parts ------------------------------------------------------------
    int *blk_nnz, *wc_slot;
    TRS_TRY(sc.get<int>((size_t)NB + 1, &blk_nnz));
    TRS_TRY(sc.get<int>(D, &wc_slot));
    TRS_CUDA(cudaMemsetAsync(wc_slot, 0xFF, sizeof(int) * (size_t)D, st));
    TRS_CUDA(cudaMemsetAsync(blk_nnz + NB, 0, sizeof(int), st));
    B->t_block_offset.release();
    TRS_TRY(B->t_block_offset.alloc_from(B->arena, (size_t)NB + 1));
    TRS_TRY(B->t_column.alloc_from(B->arena, (size_t)NB * 8));
    TRS_TRY(B->t_binary.alloc_from(B->arena, (size_t)NB * 2));
    int tc_nnz = 0;
    if (NB > 0) {
        kb_tc_blocks<<<grid_for(NB), 256, 0, st>>>(blk_pos, blk_len, NB, ord, wc_col, wc_mask, B->t_column.p, B->t_binary.p,
                                                    blk_nnz, wc_slot);
        TRS_LAUNCH_CHECK();
    }
    TRS_TRY(cub_.exclusive_sum(blk_nnz, B->t_block_offset.p, (long long)NB + 1));
    TRS_TRY(read_int(B->t_block_offset.p + NB, st, &tc_nnz));
    TRS_TRY(B->t_value.alloc_from(B->arena, tc_nnz));
    if (NB > 0) {
        kb_tc_values<<<grid_for(nnz), 256, 0, st>>>(keys, edge, wc_incl, nnz, wc_slot, B->t_binary.p, B->t_block_offset.p,
                                                     val, B->t_value.p);
        TRS_LAUNCH_CHECK();
    }
    B->t_row_offset.release();
    TRS_TRY(B->t_row_offset.alloc_from(B->arena, (size_t)NP + 1));
    TRS_TRY(B->t_window_row.alloc_from(B->arena, NP));
    TRS_TRY(B->t_atomic.alloc_from(B->arena, NP));
    kb_tc_parts<<<grid_for(W), 256, 0, st>>>(wc_begin, b_idx, win_bb, part_off, win_cuda_unit, W, cfg.part_t,
                                              B->t_row_offset.p, B->t_window_row.p, B->t_atomic.p);
    TRS_LAUNCH_CHECK();

    // ---- 9. CUDA-core row parts ---------------------------------------------------------------
    int *cnt4, *off4;
    const size_t stride = (size_t)n + 1;
    TRS_TRY(sc.get<int>(4 * stride, &cnt4));
    TRS_TRY(sc.get<int>(4 * stride, &off4));
    TRS_CUDA(cudaMemsetAsync(cnt4, 0, sizeof(int) * 4 * stride, st));
    kb_cuda_count<<<grid_for(n), 256, 0, st>>>(n, window, cfg.part_c, cfg.short_size, win_cuda_unit, win_cb, wc_begin, s_idx,
                                                cand, wc_col, wc_mask, wc_start, row_extra, cnt4);
    TRS_LAUNCH_CHECK();
    int tot[4] = {0, 0, 0, 0};
    for (int i = 0; i < 4; ++i) {
        TRS_TRY(cub_.exclusive_sum(cnt4 + i * stride, off4 + i * stride, (long long)stride));
        TRS_CUDA(cudaMemcpyAsync(&tot[i], off4 + i * stride + n, sizeof(int), cudaMemcpyDeviceToHost, st));
    }
    TRS_CUDA(cudaStreamSynchronize(st));
    B->c_row_offset.release(); B->cs_row_offset.release();
    TRS_TRY(B->c_row_offset.alloc_from(B->arena, (size_t)tot[0] + 1));
    TRS_TRY(B->c_row.alloc_from(B->arena, tot[0]));
    TRS_TRY(B->c_atomic.alloc_from(B->arena, tot[0]));
    TRS_TRY(B->c_column.alloc_from(B->arena, tot[2]));
    TRS_TRY(B->c_value.alloc_from(B->arena, tot[2]));
    TRS_TRY(B->cs_row_offset.alloc_from(B->arena, (size_t)tot[1] + 1));
    TRS_TRY(B->cs_row.alloc_from(B->arena, tot[1]));
    TRS_TRY(B->cs_atomic.alloc_from(B->arena, tot[1]));
    TRS_TRY(B->cs_column.alloc_from(B->arena, tot[3]));
    TRS_TRY(B->cs_value.alloc_from(B->arena, tot[3]));
    kb_cuda_fill<<<grid_for(n), 256, 0, st>>>(n, window, cfg.part_c, cfg.short_size, win_cuda_unit, win_cb, wc_begin, s_idx,
                                               b_idx, cand, wc_col, wc_mask, wc_start, edge, val, off4, extra_off, extra_key,
                                               extra_at, B->c_row_offset.p,
                                               B->c_row.p, B->c_atomic.p, B->c_column.p, B->c_value.p, B->cs_row_offset.p,
                                               B->cs_row.p, B->cs_atomic.p, B->cs_column.p, B->cs_value.p);
    TRS_LAUNCH_CHECK();

    // ---- 10. tiles -----------------------------------------------------------------------------------
    int* win_T;
    TRS_TRY(sc.get<int>((size_t)W + 1, &win_T));
    TRS_CUDA(cudaMemsetAsync(win_T + W, 0, sizeof(int), st));
    kb_win_tiles<<<grid_for(W), 256, 0, st>>>(win_G, W, win_T);
    TRS_TRY(cub_.exclusive_sum(win_T, B->s_window_tile_offset.p, W + 1));
    int T = 0;
    TRS_TRY(read_int(B->s_window_tile_offset.p + W, st, &T));
    TRS_TRY(B->s_tile_window.alloc_from(B->arena, T));
    TRS_TRY(B->s_tile_group.alloc_from(B->arena, T));
    TRS_TRY(B->s_tile_column.alloc_from(B->arena, (size_t)T * 16));
    TRS_TRY(B->s_packed_a.alloc_from(B->arena, (size_t)T * 64));
    TRS_TRY(B->s_packed_meta.alloc_from(B->arena, (size_t)T * 8));
    if (T > 0) {
        kb_tiles<<<grid_for(T), 256, 0, st>>>(B->s_window_tile_offset.p, B->s_offset.p, W, T, B->s_tile_window.p,
                                               B->s_tile_group.p);
        TRS_LAUNCH_CHECK();
        TRS_TRY(pack_tiles(B->s_column.p, B->s_value.p, (const int8_t*)B->s_pos.p, B->s_offset.p, B->s_tile_window.p,
                           B->s_tile_group.p, T, window, B->s_tile_column.p, B->s_packed_a.p, B->s_packed_meta.p, st));
    }
    TRS_CUDA(cudaMemcpyAsync(&B->dropped, d_dropped, sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

void fill_sizes(trs_builder* B) {
    long long* z = B->sizes;
    z[0] = B->t_row_offset.n; z[1] = B->t_block_offset.n; z[2] = B->t_column.n; z[3] = B->t_value.n;
    z[4] = B->t_window_row.n; z[5] = B->t_atomic.n; z[6] = B->t_binary.n;
    z[7] = B->c_row_offset.n; z[8] = B->c_row.n; z[9] = B->c_atomic.n; z[10] = B->c_column.n; z[11] = B->c_value.n;
    z[12] = B->cs_row_offset.n; z[13] = B->cs_row.n; z[14] = B->cs_atomic.n; z[15] = B->cs_column.n; z[16] = B->cs_value.n;
    z[17] = B->s_column.n; z[18] = B->s_mask.n; z[19] = B->s_value.n; z[20] = B->s_pos.n; z[21] = B->s_window.n;
    z[22] = B->s_offset.n; z[23] = B->s_tile_window.n; z[24] = B->s_tile_group.n; z[25] = B->s_tile_column.n;
    z[26] = B->s_packed_a.n; z[27] = B->s_packed_meta.n; z[28] = B->s_window_tile_offset.n;
}

const void* array_ptr(const trs_builder* B, int id, size_t* elem) {
    switch (id) {
        case 0: *elem = 4; return B->t_row_offset.p;    case 1: *elem = 4; return B->t_block_offset.p;
        case 2: *elem = 4; return B->t_column.p;        case 3: *elem = 4; return B->t_value.p;
        case 4: *elem = 4; return B->t_window_row.p;    case 5: *elem = 4; return B->t_atomic.p;
        case 6: *elem = 8; return B->t_binary.p;        case 7: *elem = 4; return B->c_row_offset.p;
        case 8: *elem = 4; return B->c_row.p;           case 9: *elem = 4; return B->c_atomic.p;
        case 10: *elem = 4; return B->c_column.p;       case 11: *elem = 4; return B->c_value.p;
        case 12: *elem = 4; return B->cs_row_offset.p;  case 13: *elem = 4; return B->cs_row.p;
        case 14: *elem = 4; return B->cs_atomic.p;      case 15: *elem = 4; return B->cs_column.p;
        case 16: *elem = 4; return B->cs_value.p;       case 17: *elem = 4; return B->s_column.p;
        case 18: *elem = 1; return B->s_mask.p;         case 19: *elem = 4; return B->s_value.p;
        case 20: *elem = 1; return B->s_pos.p;          case 21: *elem = 4; return B->s_window.p;
        case 22: *elem = 4; return B->s_offset.p;       case 23: *elem = 4; return B->s_tile_window.p;
        case 24: *elem = 4; return B->s_tile_group.p;   case 25: *elem = 4; return B->s_tile_column.p;
        case 26: *elem = 4; return B->s_packed_a.p;     case 27: *elem = 4; return B->s_packed_meta.p;
        case 28: *elem = 4; return B->s_window_tile_offset.p;
    }
    *elem = 0;
    return nullptr;
}

}  // namespace

static int build_impl(const int32_t* rowptr, const int32_t* col, const float* values, int n_rows,
                      const trs_build_config* cfg, void* arena, size_t arena_bytes, bool use_arena, void* stream,
                      trs_builder** out) {
    if (!rowptr || !cfg || !out || n_rows <= 0) return TRS_E_ARG;
    *out = nullptr;
    if (cfg->window <= 0 || cfg->window > 16) return TRS_E_WINDOW;
    if (cfg->part_t <= 0 || cfg->part_c <= 0 || cfg->short_size < 0 || cfg->density < 0) return TRS_E_ARG;
    if (use_arena && (!arena || ((uintptr_t)arena & 255))) return TRS_E_ARG;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return TRS_E_NO_DEVICE;
    trs_builder* B = new trs_builder();
    if (use_arena) {
        B->arena_store.base = (unsigned char*)arena;
        B->arena_store.cap = arena_bytes;
        B->arena = &B->arena_store;
    }
    B->cfg = BuildCfg{cfg->part_t, cfg->part_c, cfg->short_size, cfg->density, cfg->window, cfg->tc_min_util,
                      cfg->skip_tc, cfg->unit_min_nnz, cfg->strict ? 1 : 0};
    B->n_rows = n_rows;
    B->W = ceil_div(n_rows, cfg->window);
    cudaStream_t st = (cudaStream_t)stream;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0, st);
    int rc = do_build(B, rowptr, col, values, st);
    cudaEventRecord(e1, st);
    cudaError_t es = cudaStreamSynchronize(st);
    if (!rc && es != cudaSuccess) rc = (int)es;
    if (!rc) cudaEventElapsedTime(&B->build_ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (rc) { B->release(); delete B; return rc; }
    fill_sizes(B);
    *out = B;
    return TRS_OK;
}

extern "C" int trs_build_create(const int32_t* rowptr, const int32_t* col, const float* values, int n_rows,
                                const trs_build_config* cfg, void* stream, trs_builder** out) {
    return build_impl(rowptr, col, values, n_rows, cfg, nullptr, 0, false, stream, out);
}

// Upper bound of the device memory one build can need (outputs + temporaries), from the sizes
// alone: every count the builder allocates by is bounded by the number of entries (distinct
// (window, column) pairs <= nnz, units <= pairs / 2 + windows, groups <= pairs / 4 + windows, ...).
extern "C" int trs_build_query(int n_rows, long long nnz, const trs_build_config* cfg, size_t* arena_bytes) {
    if (!cfg || !arena_bytes || n_rows <= 0 || nnz < 0) return TRS_E_ARG;
    if (cfg->window <= 0 || cfg->window > 16) return TRS_E_WINDOW;
    const size_t W = (size_t)ceil_div(n_rows, cfg->window) + 1;
    const size_t e = (size_t)nnz;
    size_t b = 0;
    b += e * 40;                      // row ids, two 64-bit key buffers, two edge buffers, heads, running counts
    b += e * 72;                      // per-(window, column) records, their two sort buffers, TC / SPTC index maps
    b += (e / 2 + W) * 8 + (e / 4 + W) * 24;   // units, pairs, group column lists
    if (cfg->strict) b += e * 28 + (size_t)n_rows * 8;
    b += W * 4 * 32;                  // per-window counters and prefixes
    b += e / 2 + ((size_t)64 << 20);  // CUB temporary storage
    // outputs: SPTC groups (196 B each) and tiles (360 B each), TC blocks, CSR parts, fp16 value copies
    b += (e / 4 + W) * 196 + (e / 16 + 2 * W) * 360;
    b += e * 12 + (e / 8 + W) * 64 + e * 14 + W * 32;
    b += 256 * 160;                   // alignment of every block
    *arena_bytes = b;
    return TRS_OK;
}

extern "C" int trs_build_fill(const int32_t* rowptr, const int32_t* col, const float* values, int n_rows,
                              const trs_build_config* cfg, void* arena, size_t arena_bytes, void* stream,
                              trs_builder** out) {
    return build_impl(rowptr, col, values, n_rows, cfg, arena, arena_bytes, true, stream, out);
}

extern "C" int trs_build_arena_used(const trs_builder* B, size_t* bytes) {
    if (!B || !bytes) return TRS_E_ARG;
    *bytes = B->arena ? B->arena->high : 0;
    return TRS_OK;
}

extern "C" int trs_build_destroy(trs_builder* B) {
    if (!B) return TRS_OK;
    B->release();
    delete B;
    return TRS_OK;
}

extern "C" int trs_build_sizes(const trs_builder* B, long long* sizes) {
    if (!B || !sizes) return TRS_E_ARG;
    memcpy(sizes, B->sizes, sizeof(B->sizes));
    return TRS_OK;
}

extern "C" int trs_build_stats(const trs_builder* B, trs_build_stats_t* s) {
    if (!B || !s) return TRS_E_ARG;
    s->nnz = B->nnz;
    s->dropped_nnz = (long long)B->dropped;
    s->distinct_window_columns = B->distinct_cols;
    s->units = B->units;
    s->tc_nnz = B->sizes[3];
    s->csr_nnz = B->sizes[11] + B->sizes[16];
    s->groups = B->sizes[21];
    s->tiles = B->sizes[23];
    s->tc_blocks = B->sizes[2] / 8;
    s->build_ms = B->build_ms;
    return TRS_OK;
}

extern "C" const void* trs_build_array(const trs_builder* B, int id) {
    size_t elem;
    return B ? array_ptr(B, id, &elem) : nullptr;
}

extern "C" int trs_build_copy(const trs_builder* B, int id, void* dst, int dst_is_host, void* stream) {
    if (!B || id < 0 || id >= TRS_BUILD_NUM_ARRAYS) return TRS_E_ARG;
    size_t elem;
    const void* src = array_ptr(B, id, &elem);
    const size_t bytes = (size_t)B->sizes[id] * elem;
    if (bytes == 0) return TRS_OK;
    if (!dst) return TRS_E_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    TRS_CUDA(cudaMemcpyAsync(dst, src, bytes, dst_is_host ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice, st));
    if (dst_is_host) TRS_CUDA(cudaStreamSynchronize(st));
    return TRS_OK;
}

extern "C" int trs_build_format(trs_builder* B, trs_format* out, void* stream) {
    if (!B || !out) return TRS_E_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    struct Conv { DevBuf<float>* src; DevBuf<__half>* dst; } conv[3] = {
        {&B->t_value, &B->t_value_h}, {&B->c_value, &B->c_value_h}, {&B->cs_value, &B->cs_value_h}};
    for (auto& c : conv) {
        if (c.dst->p || c.src->n == 0) continue;
        int rc = c.dst->alloc_from(B->arena, c.src->n);
        if (rc) return rc;
        kb_to_half<<<grid_for((long long)c.src->n), 256, 0, st>>>(c.src->p, (long long)c.src->n, c.dst->p);
        TRS_LAUNCH_CHECK();
    }
    memset(out, 0, sizeof(*out));
    out->t_row_offset = B->t_row_offset.p; out->t_block_offset = B->t_block_offset.p; out->t_column = B->t_column.p;
    out->t_value = (const trs_half*)B->t_value_h.p; out->t_window_row = B->t_window_row.p;
    out->t_binary = (const int64_t*)B->t_binary.p;
    out->parts_t = (int)B->t_window_row.n; out->blocks = (int)(B->t_column.n / 8);
    out->c_row_offset = B->c_row_offset.p; out->c_row = B->c_row.p; out->c_column = B->c_column.p;
    out->c_value = (const trs_half*)B->c_value_h.p; out->parts_c = (int)B->c_row.n;
    out->cs_row_offset = B->cs_row_offset.p; out->cs_row = B->cs_row.p; out->cs_column = B->cs_column.p;
    out->cs_value = (const trs_half*)B->cs_value_h.p; out->parts_c_short = (int)B->cs_row.n;
    out->s_window_tile_offset = B->s_window_tile_offset.p; out->s_tile_column = B->s_tile_column.p;
    out->s_packed_a = B->s_packed_a.p; out->s_packed_meta = B->s_packed_meta.p;
    out->num_windows = B->W; out->tiles = (int)B->s_tile_window.n;
    return TRS_OK;
}

// Host-side run of the std::sort emulation (the same code the matching kernel runs), so that
// it can be checked against libstdc++ without a GPU.
extern "C" int trs_debug_stdsort_order(const unsigned char* keys, int n, int* out, int* heap_sorts) {
    if (n < 0 || (n > 0 && (!keys || !out))) return TRS_E_ARG;
    for (int i = 0; i < n; ++i) out[i] = i;
    StdSort<UnitLess> s(out, UnitLess{keys});
    s.sort(n);
    if (heap_sorts) *heap_sorts = s.heap_sorts;
    return TRS_OK;
}
