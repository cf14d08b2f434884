// 2:4 matching STATISTICS on the GPU: deterministic device versions of the reference's three CPU
// matchers, one warp per 16-row window.
//
//   variant 0  matching_utils.match_2to4            TR-source/Block/block_matching_window_para_dr.cpp:90-261
//   variant 1  matching_utils_hash.match_2to4_hash  TR-source/Block/block_matching_hash.cpp:104-283
//   variant 2  matching_utils_bucket.match_2to4_bucket  TR-source/Block/block_matching_bucket.cpp:130-360
//   variant 3  matching_utils_online.match_2to4_online  TR-source/Block/block_matching_online.cu:85-431
//              (the dual-routing rules of variant 0 over the columns in the SLOT ORDER of the
//              reference's 2048-entry open-addressing table, for the schedule in which the window's
//              rows insert one after the other; at most 2048 distinct columns per window survive)
//   variant 4  matching_utils_cuda.match_2to4          TR-source/Block/block_match_cuda.cu:822-1201, 1216-1612
//              (best-score pairing and grouping over the columns in the compaction order of the
//              reference's per-window hash table, for the schedule in which its warps run one at a time)
//
// All three are greedy first-fit scans over the window's columns (sorted by column id) and then
// over the pairs they produced; every step depends on which columns earlier steps consumed, so a
// window is processed serially — but each scan ("first unused candidate in the next 32 / 1024 /
// 16 with ...") is evaluated by the 32 lanes at once with ballots, which gives exactly the
// candidate the serial loop would take.  Windows are independent; their integer statistics are
// added up with atomics (sums, min, max: order-free, hence deterministic).
// None of the reference functions returns format arrays; the contract is the statistics record.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_reduce.cuh>
#include <cub/device/device_scan.cuh>

#include <string.h>

#include <vector>

#include "trs_common.cuh"

namespace trs {

typedef unsigned long long u64;

struct MStats {  // device-side accumulators
    long long groups, tc_blocks, blocks16, pad_groups, fine_fb, coarse_fb, fake_zeros;
    long long tc_total_nnz, tc_block_count;
    int tc_max_nnz, tc_min_nnz;
    long long fake_exact;  // 2 * win_rows * groups - nnz of the grouped columns (exact padding count)
    long long pool_to_tc, pool_to_sptc;  // pooled columns routed to TC blocks / to 2-column fallback groups
};

struct WinCols {
    const int* begin;            // [W + 1] first column record of every window
    const unsigned short* mask;  // [D] row masks, columns ascending inside a window
};

struct Work {  // per-window scratch lives at the window's offset in these arrays
    unsigned char* matched;   // [D]
    unsigned short* pG1;      // [D] pairs
    unsigned short* pG2;
    unsigned char* pn1;       // nnz of the pair's first / second column (second = 0 when absent)
    unsigned char* pn2;
    unsigned char* pused;
    unsigned char* pool;      // [D] nnz of pooled columns (variant 0)
    int* idx_a;               // [D] bucket lists (variant 2) / mask-sorted order (variant 1)
    int* idx_b;
    int* idx_c;
};

__device__ __forceinline__ int warp_min_key(int key) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) key = min(key, __shfl_xor_sync(0xffffffffu, key, o));
    return key;
}

// candidate j = base + lane for lanes < count: first zero-cost one, else the cheapest within t_max
// (lowest lane on ties); -1 when none.  `ok` = candidate exists and is unmatched.
__device__ __forceinline__ int pick_partner(bool ok, int cost, int t_max, int lane) {
    const unsigned zero = __ballot_sync(0xffffffffu, ok && cost == 0);
    if (zero) return __ffs(zero) - 1;
    const int key = (ok && cost <= t_max) ? cost * 64 + lane : (1 << 20);
    const int best = warp_min_key(key);
    return best >= (1 << 20) ? -1 : (best & 63);
}

// Coarse step shared by all variants: pairs [0, np) in creation order, scan window `gw` pairs
// ahead (exclusive end i + gw + plus_one).  found(i, j) / lonely(i) are called by lane 0.
template <class Found, class Lonely>
__device__ __forceinline__ void group_pairs(int np, int gw, int plus_one, const unsigned short* G1,
                                            const unsigned short* G2, unsigned char* used, int lane, Found found,
                                            Lonely lonely) {
    for (int i = 0; i < np; ++i) {
        if (used[i]) continue;
        const unsigned short a1 = G1[i], a2 = G2[i];
        const int j_end = min(i + gw + plus_one, np);
        int hit = -1;
        for (int j0 = i + 1; j0 < j_end && hit < 0; j0 += 32) {
            const int j = j0 + lane;
            bool ok = j < j_end && !used[j];
            if (ok) ok = (((a1 & G2[j]) | (a2 & G1[j])) == 0);
            const unsigned m = __ballot_sync(0xffffffffu, ok);
            if (m) hit = j0 + __ffs(m) - 1;
        }
        if (lane == 0) {
            used[i] = 1;
            if (hit >= 0) { used[hit] = 1; found(i, hit); }
            else lonely(i);
        }
        __syncwarp();
    }
}

__device__ __forceinline__ void flush_window(MStats* st, int groups, long long fake, int fine, int coarse) {
    const int blocks = (groups + 3) / 4;
    atomicAdd((u64*)&st->groups, (u64)groups);
    atomicAdd((u64*)&st->blocks16, (u64)blocks);
    atomicAdd((u64*)&st->pad_groups, (u64)(blocks * 4 - groups));
    atomicAdd((u64*)&st->fine_fb, (u64)fine);
    atomicAdd((u64*)&st->coarse_fb, (u64)coarse);
    atomicAdd((u64*)&st->fake_zeros, (u64)fake);
}

// ---------------------------------------------------------------------------------------------
// variant 0: sliding window + dense-pool dual routing
// ---------------------------------------------------------------------------------------------
// `fixed_rows` > 0: every padding count uses that many rows, whatever the window really holds
// (block_matching_online.cu:332, 384 use the constant 32 = 2 x 16).
__global__ void km_para_dr(WinCols wc, Work wk, int W, int n_rows, int window, int dense_threshold, int t_max,
                           int fixed_rows, MStats* st) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= W) return;
    const int b = wc.begin[w], n = wc.begin[w + 1] - b;
    if (n == 0) return;
    const int win_rows = fixed_rows > 0 ? fixed_rows : min(window, n_rows - w * window);
    const unsigned short* m = wc.mask + b;
    unsigned short *G1 = wk.pG1 + b, *G2 = wk.pG2 + b;
    unsigned char *n1 = wk.pn1 + b, *n2 = wk.pn2 + b, *used = wk.pused + b, *pool = wk.pool + b;
    for (int i = lane; i < n; i += 32) used[i] = 0;
    __syncwarp();
    int np = 0, nd = 0, fine = 0, coarse = 0, groups = 0;
    long long fake = 0;
    // fine step (block_matching_window_para_dr.cpp:126-158).  A column can only be matched by one
    // of the 32 columns before it, so the matched flags of the columns ahead are a 32-bit window
    // kept in a register (bit k = column i + 1 + k), identical in every lane: the serial loop then
    // reads only the read-only masks from memory.
    unsigned ahead = 0u;
    bool cur = false;  // column i is matched
    for (int i = 0; i < n; ++i) {
        if (!cur) {
            const unsigned mi = m[i];
            const int j_end = min(i + 1 + 32, n);
            const int j = i + 1 + lane;
            const bool ok = j < j_end && !((ahead >> lane) & 1u);
            const int cost = ok ? __popc(mi & m[j]) : 99;
            const int pick = pick_partner(ok, cost, t_max, lane);
            if (lane == 0) {
                if (pick >= 0) {
                    const int bj = i + 1 + pick;
                    G1[np] = (unsigned short)(mi & m[bj]);
                    G2[np] = (unsigned short)(mi | m[bj]);
                    n1[np] = (unsigned char)__popc(mi);
                    n2[np] = (unsigned char)__popc((unsigned)m[bj]);
                } else {
                    pool[nd] = (unsigned char)__popc(mi);
                }
            }
            if (pick >= 0) { ahead |= 1u << pick; ++np; } else { ++nd; ++fine; }
        }
        cur = ahead & 1u;
        ahead >>= 1;
    }
    __syncwarp();
    // coarse step (:169-204)
    group_pairs(np, 1024, 1, G1, G2, used, lane,
                [&](int i, int j) { fake += 2 * win_rows - ((int)n1[i] + n2[i] + n1[j] + n2[j]); ++groups; },
                [&](int i) { pool[nd] = n1[i]; pool[nd + 1] = n2[i]; nd += 2; coarse += 2; });
    nd = __shfl_sync(0xffffffffu, nd, 0);
    if (lane != 0) return;
    // dual routing of the pool (:210-249)
    int processed = 0, tc_blocks = 0, tmax = 0, tmin = 999999;
    long long tc_nnz = 0;
    while (nd - processed >= dense_threshold) {
        int bn = 0;
        for (int k = 0; k < dense_threshold; ++k) bn += pool[processed + k];
        tc_nnz += bn; ++tc_blocks;
        tmax = max(tmax, bn); tmin = min(tmin, bn);
        processed += dense_threshold;
    }
    for (int idx = processed; idx < nd; idx += 2) {
        int fb = pool[idx] + (idx + 1 < nd ? pool[idx + 1] : 0);
        fake += 2 * win_rows - fb;
        ++groups;
    }
    flush_window(st, groups, fake, fine, coarse);
    atomicAdd((u64*)&st->pool_to_tc, (u64)processed);
    atomicAdd((u64*)&st->pool_to_sptc, (u64)(nd - processed));
    if (tc_blocks) {
        atomicAdd((u64*)&st->tc_blocks, (u64)tc_blocks);
        atomicAdd((u64*)&st->tc_block_count, (u64)tc_blocks);
        atomicAdd((u64*)&st->tc_total_nnz, (u64)tc_nnz);
        atomicMax(&st->tc_max_nnz, tmax);
        atomicMin(&st->tc_min_nnz, tmin);
    }
}

// ---------------------------------------------------------------------------------------------
// variant 1: complement-hash fast path + sliding window
// idx_a = the window's column indices ordered by (mask, index): the chains of the reference's
// hash table (head insertion => a chain is walked from the highest index down).
// ---------------------------------------------------------------------------------------------
__global__ void km_hash(WinCols wc, Work wk, int W, int n_rows, int window, MStats* st) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= W) return;
    const int b = wc.begin[w], n = wc.begin[w + 1] - b;
    if (n == 0) return;
    const int win_rows = min(window, n_rows - w * window);
    const unsigned short* m = wc.mask + b;
    unsigned char* matched = wk.matched + b;
    unsigned short *G1 = wk.pG1 + b, *G2 = wk.pG2 + b;
    unsigned char *n1 = wk.pn1 + b, *used = wk.pused + b;
    const int* by_mask = wk.idx_a + b;  // local column indices sorted by (mask, index)
    int* top = wk.idx_b + b;            // top[r] for a run starting at sorted position r: next candidate position
    long long win_nnz = 0;
    for (int i = lane; i < n; i += 32) { matched[i] = 0; used[i] = 0; top[i] = -2; win_nnz += __popc((unsigned)m[i]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) win_nnz += __shfl_xor_sync(0xffffffffu, win_nnz, o);
    __syncwarp();
    int np = 0, fine = 0, coarse = 0, groups = 0;
    long long fake = 0;
    // phase 1 (block_matching_hash.cpp:142-163).  The lookups only depend on the masks, so the
    // whole warp resolves them first, in parallel: run_lo[i] = sorted position where the run of
    // column i's complement mask starts (-1: no such run), and top[start of a run] = its last
    // position.  The chain walk itself is serial by nature and stays with lane 0, now without any
    // binary search on its critical path.
    int* run_lo = wk.idx_c + b;
    auto lower = [&](unsigned key) {  // first sorted position whose mask is >= key
        int lo = 0, hi = n;
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (m[by_mask[mid]] < key) lo = mid + 1; else hi = mid; }
        return lo;
    };
    for (int i = lane; i < n; i += 32) {
        const unsigned ideal = (~(unsigned)m[i]) & 0xFFFFu;
        const int lo = lower(ideal);
        run_lo[i] = (lo < n && m[by_mask[lo]] == ideal) ? lo : -1;
        const unsigned mq = m[by_mask[i]];   // i as a sorted position: is it the last of its run?
        if (i == n - 1 || m[by_mask[i + 1]] != mq) top[lower(mq)] = i;
    }
    __syncwarp();
    if (lane == 0) {
        for (int i = 0; i < n; ++i) {
            if (matched[i]) continue;
            const int lo = run_lo[i];
            if (lo < 0) continue;
            int p = top[lo];   // highest not yet discarded position of the run
            while (p >= lo && matched[by_mask[p]]) --p;
            top[lo] = p;
            if (p < lo) continue;
            const int j = by_mask[p];
            matched[i] = 1; matched[j] = 1;
            G1[np] = 0; G2[np] = (unsigned short)(m[i] | m[j]); n1[np] = 0;  // nnz stays 0, as in the reference
            ++np;
        }
    }
    np = __shfl_sync(0xffffffffu, np, 0);
    __syncwarp();
    // phase 2 (:170-221).  Phase 1 is over, so its matched flags are read-only now; the flags of the
    // 32 columns ahead sit in a register window (bit k = column i + 1 + k), refilled from the array
    // 32 positions at a time, and the matches of this phase are recorded in the window only.
    unsigned ahead = __ballot_sync(0xffffffffu, 1 + lane < n && matched[1 + lane]);
    int fbase = 33;
    unsigned feed = __ballot_sync(0xffffffffu, fbase + lane < n && matched[fbase + lane]);
    bool cur = matched[0] != 0;
    for (int i = 0; i < n; ++i) {
        if (!cur) {
            const unsigned mi = m[i];
            const int j_end = min(i + 1 + 32, n);
            const int j = i + 1 + lane;
            const bool ok = j < j_end && !((ahead >> lane) & 1u);
            const int cost = ok ? __popc(mi & m[j]) : 99;
            const int pick = pick_partner(ok, cost, 8, lane);
            if (lane == 0) {
                if (pick >= 0) {
                    const int bj = i + 1 + pick;
                    G1[np] = (unsigned short)(mi & m[bj]);
                    G2[np] = (unsigned short)(mi | m[bj]);
                    n1[np] = (unsigned char)(__popc(mi) + __popc((unsigned)m[bj]));
                } else {
                    G1[np] = 0; G2[np] = (unsigned short)mi; n1[np] = (unsigned char)__popc(mi);
                }
            }
            if (pick >= 0) ahead |= 1u << pick; else ++fine;
            ++np;
        }
        const int nx = i + 33;   // the column that enters the window
        if (nx - fbase == 32) {
            fbase += 32;
            feed = __ballot_sync(0xffffffffu, fbase + lane < n && matched[fbase + lane]);
        }
        cur = ahead & 1u;
        ahead = (ahead >> 1) | (((feed >> (nx - fbase)) & 1u) << 31);
    }
    __syncwarp();
    // coarse step (:227-277)
    group_pairs(np, 1024, 1, G1, G2, used, lane,
                [&](int i, int j) { fake += 2 * win_rows - ((int)n1[i] + n1[j]); ++groups; },
                [&](int i) { fake += 2 * win_rows - (int)n1[i]; ++groups; coarse += 2; });
    if (lane == 0) {
        flush_window(st, groups, fake, fine, coarse);
        atomicAdd((u64*)&st->fake_exact, (u64)(2ll * win_rows * groups - win_nnz));
    }
}

// ---------------------------------------------------------------------------------------------
// variant 2: top-heavy / bottom-heavy / balanced buckets
// ---------------------------------------------------------------------------------------------
// find_best_in_bucket (block_matching_bucket.cpp:99-124): candidates in list order, matched ones
// skipped, stop after 16 unmatched candidates; `skip` is excluded (balanced x balanced phase).
__device__ __forceinline__ int best_in_bucket(const unsigned short* m, unsigned mi, const int* list, int len,
                                              int* first_live, const unsigned char* matched, int skip, int lane) {
    int p = *first_live;
    while (p < len && matched[list[p]]) ++p;   // the matched prefix never comes back
    *first_live = p;
    int seen = 0, best_key = 1 << 20, best_idx = -1;
    for (; p < len && seen < 16; p += 32) {
        const int q = p + lane;
        const int idx = q < len ? list[q] : -1;
        const bool live = idx >= 0 && idx != skip && !matched[idx];
        const unsigned lm = __ballot_sync(0xffffffffu, live);
        const int rank = seen + __popc(lm & ((1u << lane) - 1u));   // unmatched candidates before this one
        const bool ok = live && rank < 16;
        const int cost = ok ? __popc(mi & m[idx]) : 99;
        const unsigned zero = __ballot_sync(0xffffffffu, ok && cost == 0);
        if (zero) return __shfl_sync(0xffffffffu, idx, __ffs(zero) - 1);
        // cheapest so far, earliest candidate on ties: key = cost * 4096 + rank
        const int key = (ok && cost <= 8) ? cost * 4096 + rank : (1 << 20);
        const int kmin = warp_min_key(key);
        if (kmin < best_key) {
            best_key = kmin;
            const unsigned who = __ballot_sync(0xffffffffu, key == kmin);
            best_idx = __shfl_sync(0xffffffffu, idx, __ffs(who) - 1);
        }
        seen += __popc(lm);
    }
    return best_idx;
}

__global__ void km_bucket(WinCols wc, Work wk, int W, int n_rows, int window, MStats* st) {
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= W) return;
    const int b = wc.begin[w], n = wc.begin[w + 1] - b;
    if (n == 0) return;
    const unsigned short* m = wc.mask + b;
    unsigned char* matched = wk.matched + b;
    unsigned short *G1 = wk.pG1 + b, *G2 = wk.pG2 + b;
    unsigned char* used = wk.pused + b;
    int *top = wk.idx_a + b, *bot = wk.idx_b + b, *bal = wk.idx_c + b;
    for (int i = lane; i < n; i += 32) { matched[i] = 0; used[i] = 0; }
    // bucket lists in ascending index order (block_matching_bucket.cpp:72-91)
    int nt = 0, nb = 0, nl = 0;
    long long win_nnz = 0;
    for (int i0 = 0; i0 < n; i0 += 32) {
        const int i = i0 + lane;
        int kind = -1;
        if (i < n) {
            const unsigned mk = m[i];
            const int t = __popc(mk & 0x00FFu), bo = __popc(mk & 0xFF00u);
            kind = t > bo ? 0 : (bo > t ? 1 : 2);
            win_nnz += t + bo;
        }
        const unsigned mt = __ballot_sync(0xffffffffu, kind == 0), mb = __ballot_sync(0xffffffffu, kind == 1),
                       ml = __ballot_sync(0xffffffffu, kind == 2);
        const unsigned below = (1u << lane) - 1u;
        if (kind == 0) top[nt + __popc(mt & below)] = i;
        if (kind == 1) bot[nb + __popc(mb & below)] = i;
        if (kind == 2) bal[nl + __popc(ml & below)] = i;
        nt += __popc(mt); nb += __popc(mb); nl += __popc(ml);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) win_nnz += __shfl_xor_sync(0xffffffffu, win_nnz, o);
    __syncwarp();
    int np = 0, fine = 0, coarse = 0, groups = 0;
    int cur[1];  // first live position of the list being scanned
    auto pair_up = [&](int i, int j) {
        if (lane == 0) {
            matched[i] = 1; matched[j] = 1;
            G1[np] = (unsigned short)(m[i] & m[j]);
            G2[np] = (unsigned short)(m[i] | m[j]);
        }
        ++np;
        __syncwarp();
    };
    // phase 1: top x bottom (:172-192)
    cur[0] = 0;
    for (int k = 0; k < nt; ++k) {
        const int i = top[k];
        if (matched[i]) continue;
        const int j = best_in_bucket(m, m[i], bot, nb, cur, matched, -1, lane);
        if (j >= 0) pair_up(i, j);
    }
    // phase 2: leftovers x balanced (:195-236)
    cur[0] = 0;
    for (int pass = 0; pass < 2; ++pass) {
        const int* lst = pass ? bot : top;
        const int len = pass ? nb : nt;
        for (int k = 0; k < len; ++k) {
            const int i = lst[k];
            if (matched[i]) continue;
            const int j = best_in_bucket(m, m[i], bal, nl, cur, matched, -1, lane);
            if (j >= 0) pair_up(i, j);
        }
    }
    // phase 3: balanced x balanced (:239-272)
    cur[0] = 0;
    for (int k = 0; k < nl; ++k) {
        const int i = bal[k];
        if (matched[i]) continue;
        const int j = best_in_bucket(m, m[i], bal, nl, cur, matched, i, lane);
        if (j >= 0) pair_up(i, j);
    }
    // phase 4: singles (:275-288)
    for (int i = 0; i < n; ++i) {
        if (matched[i]) continue;
        if (lane == 0) { matched[i] = 1; G1[np] = 0; G2[np] = m[i]; }
        ++np; ++fine;
        __syncwarp();
    }
    // coarse step, window 16 without the +1 (:294-337)
    group_pairs(np, 16, 0, G1, G2, used, lane, [&](int, int) { ++groups; }, [&](int) { ++groups; coarse += 2; });
    groups = __shfl_sync(0xffffffffu, groups, 0);
    coarse = __shfl_sync(0xffffffffu, coarse, 0);
    // every column sits in exactly one group: sum over groups of (32 - nnz) (:348-357)
    if (lane == 0) flush_window(st, groups, 32ll * groups - win_nnz, fine, coarse);
}

// ---------------------------------------------------------------------------------------------
// front end: (window, column) records with row masks, columns ascending inside a window
// ---------------------------------------------------------------------------------------------
__global__ void km_mark_rows(const int* __restrict__ rowptr, int n_rows, int* __restrict__ rowid, int* err) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int b = rowptr[r], e = rowptr[r + 1];
    if (e < b) { atomicOr(err, 1); return; }
    if (e > b) rowid[b] = r;
}
struct MaxOp2 {
    __device__ __forceinline__ int operator()(int a, int b) const { return a > b ? a : b; }
};
__global__ void km_keys(const int* __restrict__ col, const int* __restrict__ rowid, long long nnz, int window,
                        int col_bits, u64* __restrict__ keys, int* err) {
    long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= nnz) return;
    const int r = rowid[e], c = col[e];
    if (c < 0) atomicOr(err, 2);
    const int w = r / window, lr = r - w * window;
    keys[e] = ((u64)w << (col_bits + 4)) | ((u64)(unsigned)c << 4) | (u64)lr;
}
__global__ void km_heads(const u64* __restrict__ keys, long long nnz, int* __restrict__ head) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nnz) head[i] = (i == 0 || (keys[i] >> 4) != (keys[i - 1] >> 4)) ? 1 : 0;
}
__global__ void km_records(const u64* __restrict__ keys, const int* __restrict__ head, const int* __restrict__ incl,
                           long long nnz, int col_bits, unsigned* __restrict__ mask32, int* __restrict__ win_ncol,
                           int* __restrict__ rec_col) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const int j = incl[i] - 1;
    atomicOr(&mask32[j], 1u << (unsigned)(keys[i] & 15));
    if (head[i]) {
        atomicAdd(&win_ncol[(int)(keys[i] >> (col_bits + 4))], 1);
        if (rec_col) rec_col[j] = (int)((keys[i] >> 4) & ((1ull << col_bits) - 1ull));
    }
}

// Variant 3 front end.  The reference inserts the window's entries into a 2048-slot table
// (slot = col % 2048, linear probing, block_matching_online.cu:157-177) and compacts it in slot
// order (:184-197).  For the schedule in which row 0 inserts all its entries, then row 1, ...,
// a column is inserted when its first row is reached, in ascending column order inside that row:
// insertion order = (lowest set bit of the row mask, column id).  One warp per window replays the
// insertions in a shared-memory table (lane 0 probes; the 32 lanes find the next candidates with
// ballots), stops when the table is full - later columns are lost, as in the reference - and
// writes the surviving row masks in slot order.
constexpr int kOnlineSlots = 2048;
__global__ void __launch_bounds__(128) km_online_order(WinCols wc, const int* __restrict__ rec_col, int W,
                                                       const int* __restrict__ out_begin,
                                                       unsigned short* __restrict__ out_mask) {
    __shared__ int table[4][kOnlineSlots];   // record index + 1, 0 = empty
    const int wslot = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w = blockIdx.x * 4 + wslot;
    if (w >= W) return;
    const int b = wc.begin[w], n = wc.begin[w + 1] - b;
    if (n == 0) return;
    int* tab = table[wslot];
    for (int i = lane; i < kOnlineSlots; i += 32) tab[i] = 0;
    __syncwarp();
    int inserted = 0;
    for (int r = 0; r < 16 && inserted < kOnlineSlots; ++r) {
        for (int j0 = 0; j0 < n && inserted < kOnlineSlots; j0 += 32) {
            const int j = j0 + lane;
            const unsigned m = j < n ? wc.mask[b + j] : 0u;
            unsigned bal = __ballot_sync(0xffffffffu, m != 0u && (__ffs(m) - 1) == r);
            if (lane == 0) {
                while (bal && inserted < kOnlineSlots) {
                    const int jj = j0 + __ffs(bal) - 1;
                    bal &= bal - 1;
                    int slot = rec_col[b + jj] % kOnlineSlots;
                    while (tab[slot] != 0) slot = (slot + 1) % kOnlineSlots;   // a free slot exists: inserted < slots
                    tab[slot] = jj + 1;
                    ++inserted;
                }
            }
            inserted = __shfl_sync(0xffffffffu, inserted, 0);
        }
    }
    __syncwarp();
    int out = out_begin[w];
    for (int s0 = 0; s0 < kOnlineSlots; s0 += 32) {
        const int v = tab[s0 + lane];
        const unsigned occ = __ballot_sync(0xffffffffu, v != 0);
        if (v != 0) out_mask[out + __popc(occ & ((1u << lane) - 1u))] = wc.mask[b + v - 1];
        out += __popc(occ);
    }
}
__global__ void km_online_counts(const int* __restrict__ begin, int W, int* __restrict__ cnt) {
    int w = blockIdx.x * blockDim.x + threadIdx.x;
    if (w <= W) cnt[w] = w < W ? min(begin[w + 1] - begin[w], kOnlineSlots) : 0;
}

// ---------------------------------------------------------------------------------------------
// Variant 4: matching_utils_cuda.match_2to4 (TR-source/Block/block_match_cuda.cu:822-1201).
// The reference builds, per window, an open-addressing table of 2 x window_nnz slots in global
// memory (home slot = col * 2654435761 mod 2^32 mod size, linear probing, :861-880), compacts it
// thread by thread - thread t of a block of T threads owns the slots t, t + T, ..., so the
// compacted order is (slot mod T, slot) with T = 64 for windows of at most 512 non-zeros and 1024
// otherwise (:883-927, 1284-1306, 1495-1506) - and then lets the warps of the block race for the
// columns and for the pairs (:949-1201).  Restated here for one schedule the reference can take:
// the entries of the window are inserted in ascending column order (an interleaving of the row
// threads that keeps every thread's own CSR order, for rows with ascending columns), and one warp
// at a time takes the next column / pair index from the shared counter, so every claim succeeds.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) km_cuda_order(WinCols wc, const int* __restrict__ rec_col,
                                                     const int* __restrict__ rowptr, int n_rows, int window, int W,
                                                     int* __restrict__ table, unsigned short* __restrict__ out_mask) {
    __shared__ int cnt_s[4][1024];
    const int wslot = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w = blockIdx.x * 4 + wslot;
    if (w >= W) return;
    const int b = wc.begin[w], n = wc.begin[w + 1] - b;
    if (n == 0) return;
    const int r0 = w * window, r1 = min(r0 + window, n_rows);
    const int e0 = rowptr[r0], wnnz = rowptr[r1] - e0;
    const unsigned hs = (unsigned)wnnz << 1;
    int* tab = table + ((size_t)e0 << 1);           // zero-filled: record index + 1
    const int T = wnnz <= 512 ? 64 : 1024;
    int* cnt = cnt_s[wslot];
    for (int i = lane; i < T; i += 32) cnt[i] = 0;
    if (lane == 0) {
        for (int j = 0; j < n; ++j) {
            unsigned slot = ((unsigned)rec_col[b + j] * 2654435761u) % hs;
            while (tab[slot] != 0) { if (++slot == hs) slot = 0; }   // n <= window_nnz < hs: a free slot exists
            tab[slot] = j + 1;
            ++cnt[slot % (unsigned)T];
        }
    }
    __syncwarp();
    // exclusive prefix of the per-thread counts
    int carry = 0;
    for (int t0 = 0; t0 < T; t0 += 32) {
        const int v = cnt[t0 + lane];
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const int y = __shfl_up_sync(0xffffffffu, x, o); if (lane >= o) x += y; }
        cnt[t0 + lane] = carry + x - v;
        carry += __shfl_sync(0xffffffffu, x, 31);
    }
    __syncwarp();
    for (int t = lane; t < T; t += 32) {
        int out = b + cnt[t];
        for (unsigned slot = (unsigned)t; slot < hs; slot += (unsigned)T) {
            const int v = tab[slot];
            if (v != 0) out_mask[out++] = wc.mask[b + v - 1];
        }
    }
}

// padding of a group made of pair a and pair b (b = 0, 0 for a lone pair): every row of the window
// holding fewer than two of the four columns is filled up to two (block_match_cuda.cu:260-280)
__device__ __forceinline__ int cuda_fake_zeros(unsigned a1, unsigned a2, unsigned b1, unsigned b2, unsigned rowmask) {
    const unsigned zero = ~(a2 | b2) & rowmask;
    const unsigned one = ((a2 & ~a1 & ~b2) | (b2 & ~b1 & ~a2)) & rowmask;
    return 2 * __popc(zero) + __popc(one);
}

__global__ void __launch_bounds__(128) km_cuda(WinCols wc, Work wk, int W, int n_rows, int window, MStats* st) {
    const int lane = threadIdx.x & 31;
    const int w = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= W) return;
    const int b = wc.begin[w], n = wc.begin[w + 1] - b;
    if (n == 0) return;
    const int win_rows = min(window, n_rows - w * window);
    const unsigned rowmask = (1u << win_rows) - 1u;
    const unsigned short* m = wc.mask + b;
    unsigned char* matched = wk.matched + b;
    unsigned short *G1 = wk.pG1 + b, *G2 = wk.pG2 + b;
    unsigned char *pn = wk.pn1 + b, *used = wk.pused + b;
    for (int i = lane; i < n; i += 32) { matched[i] = 0; used[i] = 0; }
    __syncwarp();
    // 1:2 pairing (block_match_cuda.cu:949-1062): overlap of at most 12 rows, lowest
    // overlap * 64 + (16 - nnz of the partner), lowest index on ties
    const int sw = n > 16384 ? 64 : n > 4096 ? 128 : 512;
    int np = 0, fine = 0;
    for (int i = 0; i < n; ++i) {
        if (matched[i]) continue;
        const unsigned mi = m[i];
        const int j_end = min(n, i + 1 + sw);
        unsigned best = 0xffffffffu;
        for (int j = i + 1 + lane; j < j_end; j += 32) {
            if (matched[j]) continue;
            const unsigned mj = m[j];
            const int overlap = __popc(mi & mj);
            if (overlap > 12) continue;
            const unsigned key = ((unsigned)(overlap * 64 + 16 - __popc(mj)) << 16) | (unsigned)(j - i);
            best = min(best, key);
        }
        best = __reduce_min_sync(0xffffffffu, best);
        if (lane == 0) {
            matched[i] = 1;
            if (best != 0xffffffffu) {
                const int j = i + (int)(best & 0xffffu);
                const unsigned mj = m[j];
                matched[j] = 1;
                G1[np] = (unsigned short)(mi & mj); G2[np] = (unsigned short)(mi | mj);
                pn[np] = (unsigned char)(__popc(mi) + __popc(mj));
            } else {
                G1[np] = 0; G2[np] = (unsigned short)mi;
                pn[np] = (unsigned char)__popc(mi);
            }
        }
        if (best == 0xffffffffu) ++fine;
        ++np;
        __syncwarp();
    }
    // 2:4 grouping (block_match_cuda.cu:1086-1201): no row with more than two of the four columns,
    // most non-zeros first, lowest index on ties
    const int gw = np > 8192 ? 128 : np > 2048 ? 256 : 1024;
    int groups = 0, coarse = 0;
    long long fake = 0;
    for (int i = 0; i < np; ++i) {
        if (used[i]) continue;
        const unsigned a1 = G1[i], a2 = G2[i];
        const int na = pn[i];
        const int j_end = min(np, i + 1 + gw);
        unsigned best = 0xffffffffu;
        for (int j = i + 1 + lane; j < j_end; j += 32) {
            if (used[j]) continue;
            const unsigned b1 = G1[j], b2 = G2[j];
            if ((a1 & b2) | (a2 & b1)) continue;
            const unsigned key = ((unsigned)(64 - (na + (int)pn[j])) << 16) | (unsigned)(j - i);
            best = min(best, key);
        }
        best = __reduce_min_sync(0xffffffffu, best);
        ++groups;
        if (best != 0xffffffffu) {
            const int j = i + (int)(best & 0xffffu);
            fake += cuda_fake_zeros(a1, a2, G1[j], G2[j], rowmask);
            if (lane == 0) used[j] = 1;
        } else {
            coarse += 2;
            fake += cuda_fake_zeros(a1, a2, 0u, 0u, rowmask);
        }
        if (lane == 0) used[i] = 1;
        __syncwarp();
    }
    if (lane == 0) flush_window(st, groups, fake, fine, coarse);
}

__global__ void km_narrow(const unsigned* __restrict__ mask32, int D, unsigned short* __restrict__ mask16) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < D) mask16[j] = (unsigned short)mask32[j];
}
// key for the by-mask order of variant 1: (window, mask); payload = local column index
__global__ void km_mask_keys(const int* __restrict__ begin, const unsigned short* __restrict__ mask, int W, int D,
                             unsigned long long* __restrict__ key, int* __restrict__ local) {
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= D) return;
    int lo = 0, hi = W;
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (begin[mid] <= j) lo = mid; else hi = mid; }
    key[j] = ((u64)lo << 16) | mask[j];
    local[j] = j - begin[lo];
}

}  // namespace trs

using namespace trs;

namespace {
struct Bag {
    std::vector<void*> ptrs;
    ~Bag() { for (void* p : ptrs) cudaFree(p); }
    template <class T>
    int get(size_t n, T** out) {
        void* d = nullptr;
        cudaError_t e = cudaMalloc(&d, (n ? n : 1) * sizeof(T));
        if (e != cudaSuccess) { *out = nullptr; return (int)e; }
        ptrs.push_back(d);
        *out = (T*)d;
        return 0;
    }
};
inline unsigned gridm(long long n, int block = 256) { return (unsigned)((n + block - 1) / block); }
int bits_needed(long long max_value) { int b = 1; while ((1ll << b) <= max_value && b < 62) ++b; return b; }
#define M_TRY(expr) do { int _rc = (expr); if (_rc) return _rc; } while (0)
}  // namespace

extern "C" int trs_match24_stats(int variant, const int32_t* rowptr, const int32_t* col, int n_rows, int window,
                                 int dense_threshold, int t_max, void* stream, trs_match_stats* out) {
    if (!rowptr || !out || n_rows <= 0) return TRS_E_ARG;
    if (variant < 0 || variant > 4) return TRS_E_ARG;
    if (window <= 0 || window > 16) return TRS_E_WINDOW;
    if ((variant == 0 || variant == 3) && (dense_threshold <= 0 || t_max < 0)) return TRS_E_ARG;
    if (variant == 3 && window != 16) return TRS_E_WINDOW;   // the reference kernel fixes 16 rows per window
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return TRS_E_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    memset(out, 0, sizeof(*out));
    Bag bag;
    int ends[2] = {0, 0};
    TRS_CUDA(cudaMemcpyAsync(&ends[0], rowptr, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaMemcpyAsync(&ends[1], rowptr + n_rows, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    if (ends[0] != 0 || ends[1] < 0) return TRS_E_OFFSETS;
    const long long nnz = ends[1];
    const int W = ceil_div(n_rows, window);
    out->total_rows = n_rows;
    out->total_nnz = nnz;
    out->num_row_panels = W;
    out->tc_block_min_nnz = 999999;
    if (nnz == 0 || !col) return TRS_E_ARG;  // the reference rejects empty matrices too

    int *d_err, *rowid, *d_max;
    M_TRY(bag.get<int>(2, &d_err));
    M_TRY(bag.get<int>(nnz, &rowid));
    M_TRY(bag.get<int>(1, &d_max));
    TRS_CUDA(cudaMemsetAsync(d_err, 0, 2 * sizeof(int), st));
    TRS_CUDA(cudaMemsetAsync(rowid, 0, sizeof(int) * nnz, st));
    km_mark_rows<<<gridm(n_rows), 256, 0, st>>>(rowptr, n_rows, rowid, d_err);
    unsigned char* tmp = nullptr;
    size_t tmp_bytes = 0, need = 0;
    auto reserve = [&](size_t b) -> int { if (b <= tmp_bytes) return 0; M_TRY(bag.get<unsigned char>(b, &tmp)); tmp_bytes = b; return 0; };
    TRS_CUDA(cub::DeviceScan::InclusiveScan(nullptr, need, rowid, rowid, MaxOp2(), nnz, st));
    M_TRY(reserve(need));
    TRS_CUDA(cub::DeviceScan::InclusiveScan(tmp, need, rowid, rowid, MaxOp2(), nnz, st));
    TRS_CUDA(cub::DeviceReduce::Max(nullptr, need, col, d_max, nnz, st));
    M_TRY(reserve(need));
    TRS_CUDA(cub::DeviceReduce::Max(tmp, need, col, d_max, nnz, st));
    int max_col = 0, herr = 0;
    TRS_CUDA(cudaMemcpyAsync(&max_col, d_max, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    if (herr & 1) return TRS_E_OFFSETS;
    if (max_col < 0) return TRS_E_COLUMN;
    out->total_cols = max_col + 1;
    out->sparsity = 1.0 - (double)nnz / ((double)n_rows * (double)(max_col + 1));
    const int col_bits = bits_needed(max_col), w_bits = bits_needed(W - 1);

    u64 *k_a, *k_b;
    M_TRY(bag.get<u64>(nnz, &k_a));
    M_TRY(bag.get<u64>(nnz, &k_b));
    km_keys<<<gridm(nnz), 256, 0, st>>>(col, rowid, nnz, window, col_bits, k_a, d_err);
    cub::DoubleBuffer<u64> kb(k_a, k_b);
    TRS_CUDA(cub::DeviceRadixSort::SortKeys(nullptr, need, kb, (int)nnz, 0, 4 + col_bits + w_bits, st));
    M_TRY(reserve(need));
    TRS_CUDA(cub::DeviceRadixSort::SortKeys(tmp, need, kb, (int)nnz, 0, 4 + col_bits + w_bits, st));
    const u64* keys = kb.Current();
    int *head, *incl;
    M_TRY(bag.get<int>(nnz, &head));
    M_TRY(bag.get<int>(nnz, &incl));
    km_heads<<<gridm(nnz), 256, 0, st>>>(keys, nnz, head);
    TRS_CUDA(cub::DeviceScan::InclusiveSum(nullptr, need, head, incl, nnz, st));
    M_TRY(reserve(need));
    TRS_CUDA(cub::DeviceScan::InclusiveSum(tmp, need, head, incl, nnz, st));
    int D = 0;
    TRS_CUDA(cudaMemcpyAsync(&D, incl + (nnz - 1), sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaMemcpyAsync(&herr, d_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    if (herr & 2) return TRS_E_COLUMN;
    unsigned* mask32;
    unsigned short* mask16;
    int *win_ncol, *begin;
    M_TRY(bag.get<unsigned>(D, &mask32));
    M_TRY(bag.get<unsigned short>(D, &mask16));
    M_TRY(bag.get<int>((size_t)W + 1, &win_ncol));
    M_TRY(bag.get<int>((size_t)W + 1, &begin));
    TRS_CUDA(cudaMemsetAsync(mask32, 0, sizeof(unsigned) * (size_t)D, st));
    TRS_CUDA(cudaMemsetAsync(win_ncol, 0, sizeof(int) * ((size_t)W + 1), st));
    int* rec_col = nullptr;
    if (variant == 3 || variant == 4) M_TRY(bag.get<int>(D, &rec_col));
    km_records<<<gridm(nnz), 256, 0, st>>>(keys, head, incl, nnz, col_bits, mask32, win_ncol, rec_col);
    km_narrow<<<gridm(D), 256, 0, st>>>(mask32, D, mask16);
    TRS_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, need, win_ncol, begin, W + 1, st));
    M_TRY(reserve(need));
    TRS_CUDA(cub::DeviceScan::ExclusiveSum(tmp, need, win_ncol, begin, W + 1, st));

    Work wk;
    memset(&wk, 0, sizeof(wk));
    M_TRY(bag.get<unsigned char>(D, &wk.matched));
    M_TRY(bag.get<unsigned short>(D, &wk.pG1));
    M_TRY(bag.get<unsigned short>(D, &wk.pG2));
    M_TRY(bag.get<unsigned char>(D, &wk.pn1));
    M_TRY(bag.get<unsigned char>(D, &wk.pn2));
    M_TRY(bag.get<unsigned char>(D, &wk.pused));
    M_TRY(bag.get<unsigned char>((size_t)D + 2, &wk.pool));
    M_TRY(bag.get<int>(D, &wk.idx_a));
    M_TRY(bag.get<int>(D, &wk.idx_b));
    M_TRY(bag.get<int>(D, &wk.idx_c));
    MStats* d_stats;
    M_TRY(bag.get<MStats>(1, &d_stats));
    MStats init;
    memset(&init, 0, sizeof(init));
    init.tc_min_nnz = 999999;
    TRS_CUDA(cudaMemcpyAsync(d_stats, &init, sizeof(init), cudaMemcpyHostToDevice, st));
    WinCols wc{begin, mask16};
    const unsigned blocks = gridm((long long)W * 32, 128);
    if (variant == 0) {
        km_para_dr<<<blocks, 128, 0, st>>>(wc, wk, W, n_rows, window, dense_threshold, t_max, 0, d_stats);
    } else if (variant == 3) {
        int *cnt2, *begin2;
        unsigned short* mask2;
        M_TRY(bag.get<int>((size_t)W + 1, &cnt2));
        M_TRY(bag.get<int>((size_t)W + 1, &begin2));
        M_TRY(bag.get<unsigned short>(D, &mask2));
        km_online_counts<<<gridm(W + 1), 256, 0, st>>>(begin, W, cnt2);
        TRS_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, need, cnt2, begin2, W + 1, st));
        M_TRY(reserve(need));
        TRS_CUDA(cub::DeviceScan::ExclusiveSum(tmp, need, cnt2, begin2, W + 1, st));
        km_online_order<<<gridm(W, 4), 128, 0, st>>>(wc, rec_col, W, begin2, mask2);
        WinCols wc2{begin2, mask2};
        km_para_dr<<<blocks, 128, 0, st>>>(wc2, wk, W, n_rows, window, dense_threshold, t_max, 16, d_stats);
    } else if (variant == 4) {
        int* table;
        unsigned short* mask2;
        M_TRY(bag.get<int>((size_t)nnz * 2, &table));
        M_TRY(bag.get<unsigned short>(D, &mask2));
        TRS_CUDA(cudaMemsetAsync(table, 0, sizeof(int) * (size_t)nnz * 2, st));
        km_cuda_order<<<gridm(W, 4), 128, 0, st>>>(wc, rec_col, rowptr, n_rows, window, W, table, mask2);
        WinCols wc2{begin, mask2};
        km_cuda<<<blocks, 128, 0, st>>>(wc2, wk, W, n_rows, window, d_stats);
    } else if (variant == 1) {
        // columns of every window ordered by (mask, index): stable sort of (window, mask) keys
        u64 *mk_a, *mk_b;
        int* loc_b;
        M_TRY(bag.get<u64>(D, &mk_a));
        M_TRY(bag.get<u64>(D, &mk_b));
        M_TRY(bag.get<int>(D, &loc_b));
        km_mask_keys<<<gridm(D), 256, 0, st>>>(begin, mask16, W, D, mk_a, wk.idx_c);
        cub::DoubleBuffer<u64> mk(mk_a, mk_b);
        cub::DoubleBuffer<int> ml(wk.idx_c, loc_b);
        TRS_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, mk, ml, D, 0, 16 + w_bits, st));
        M_TRY(reserve(need));
        TRS_CUDA(cub::DeviceRadixSort::SortPairs(tmp, need, mk, ml, D, 0, 16 + w_bits, st));
        TRS_CUDA(cudaMemcpyAsync(wk.idx_a, ml.Current(), sizeof(int) * (size_t)D, cudaMemcpyDeviceToDevice, st));
        km_hash<<<blocks, 128, 0, st>>>(wc, wk, W, n_rows, window, d_stats);
    } else {
        km_bucket<<<blocks, 128, 0, st>>>(wc, wk, W, n_rows, window, d_stats);
    }
    TRS_LAUNCH_CHECK();
    MStats h;
    TRS_CUDA(cudaMemcpyAsync(&h, d_stats, sizeof(h), cudaMemcpyDeviceToHost, st));
    TRS_CUDA(cudaStreamSynchronize(st));
    out->num_groups = h.groups;
    out->num_tc_blocks = h.tc_blocks;
    out->num_16x16_blocks = h.blocks16;
    out->block_padding_groups = h.pad_groups;
    out->fine_fallback = h.fine_fb;
    out->coarse_fallback = h.coarse_fb;
    out->fake_zeros = h.fake_zeros;
    out->tc_total_nnz = h.tc_total_nnz;
    out->tc_block_count = h.tc_block_count;
    out->tc_block_max_nnz = h.tc_max_nnz;
    out->tc_block_min_nnz = h.tc_min_nnz;
    out->fake_zeros_exact = h.fake_exact;
    out->dense_to_tc_cols = h.pool_to_tc;
    out->dense_to_sptc_cols = h.pool_to_sptc;
    return TRS_OK;
}
