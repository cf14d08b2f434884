// CPU restatement of the reference's three-stage format builder.
//
// TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA builder is compared
// against.  Nothing the product ships links or loads it.
//
// Parity status: PINNED.  tests/test_oracle_golden.py compares every array this
// restatement emits against fixtures produced by the reference's own compiled
// builder (tests/golden/make_golden.py), and, when oracle/_ref is present,
// against the compiled reference directly on fresh seeded inputs.
//
// The restatement follows TR-source/Block/block_online.cpp of the reference:
//   window loop + column info .......... block_online.cpp:584-603
//   TC column selection ................ block_online.cpp:215-253
//   2-column units ..................... block_online.cpp:267-328
//   unit matching ...................... block_online.cpp:332-392
//   group emission + per-row encode .... block_online.cpp:629-703
//   CUDA-core row split ................ block_online.cpp:397-439, 706-733
//   TC part assembly ................... block_online.cpp:444-540
//   serialisation ...................... block_online.cpp:737-776
//   16x16 mma.sp tile packing .......... block_online.cpp:190-210, 796-841
//
// Two facts about the reference algorithm are used (and re-checked at run time
// when `exhaustive` is set):
//   * the column vectors only ever carry the even bit of every 2-bit row field, so
//     the O(1) compatibility check (block_online.cpp:85-88) passes for every pair;
//     the compatibility graph is complete and every degree equals U-1;
//   * the node order of the greedy matching comes from libstdc++'s std::sort with a
//     comparator that has ties, so this file calls std::sort itself with the same
//     comparator on the same initial permutation.
//
// Input contract: canonical CSR (columns ascending and duplicate-free per row).

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

namespace {

struct ColInfo {
    int col = 0;
    int count = 0;
    uint32_t vec = 0;                       // bit 2r set iff local row r holds the column
    std::vector<std::pair<int, int>> rows;  // (local_row, csr_edge)
};

struct Unit {
    int col1 = -1, col2 = -1;
    uint32_t vec = 0;
    int nnz = 0;
};

inline bool units_match_check(uint32_t a, uint32_t b) {  // block_online.cpp:85-88
    const uint32_t c = a | b;
    return (((a & b) | ((c << 1) & c)) & 0xaaaaaaaau) == 0;
}

// fp32 -> fp16 bits, round to nearest even (what c10::Half's constructor does;
// block_online.cpp:178-183).
inline uint16_t f32_to_f16_bits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((x > 0x7f800000u) ? 0x0200u : 0u));
    }
    if (x >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (x < 0x38800000u) {  // subnormal half or zero
        if (x < 0x33000000u) return (uint16_t)sign;  // < 2^-25 rounds to zero
        const int e = (int)(x >> 23);
        const uint32_t m = (x & 0x007fffffu) | 0x00800000u;
        const int shift = 126 - e;  // 14..24
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = (x - 0x38000000u) >> 13;
    const uint32_t rem = x & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
}

inline int pack_half2(float lo, float hi) {  // block_online.cpp:184-188
    return (int)((uint32_t)f32_to_f16_bits(lo) | ((uint32_t)f32_to_f16_bits(hi) << 16));
}

struct Format {
    std::vector<int> t_row_offset{0}, t_block_offset{0}, t_column, t_window_row, t_atomic;
    std::vector<float> t_value;
    std::vector<int64_t> t_binary;
    std::vector<int> c_row_offset{0}, c_row, c_atomic, c_column;
    std::vector<float> c_value;
    std::vector<int> cs_row_offset{0}, cs_row, cs_atomic, cs_column;
    std::vector<float> cs_value;
    std::vector<int> s_column, s_window, s_offset{0};
    std::vector<uint8_t> s_mask;
    std::vector<float> s_value;
    std::vector<int8_t> s_pos;
    std::vector<int> s_tile_window, s_tile_group, s_tile_column, s_packed_a, s_packed_meta;
    std::vector<int> s_window_tile_offset{0};
    long long check_failures = 0;  // pairs for which the compatibility check was false
    long long dropped_nnz = 0;     // entries beyond the first two of a (group,row)
};

void slot_normalise(const Format& f, int group_id, int group_limit, int row, int window,
                    float& v0, float& v1, int& p0, int& p1) {  // block_online.cpp:190-210
    v0 = 0.f; v1 = 0.f; p0 = 0; p1 = 1;
    if (group_id >= group_limit || row >= window) return;
    const size_t base = ((size_t)group_id * window + row) * 2;
    const int pos0 = f.s_pos[base], pos1 = f.s_pos[base + 1];
    const float val0 = f.s_value[base], val1 = f.s_value[base + 1];
    if (pos0 < 0 && pos1 < 0) return;
    if (pos0 >= 0 && pos1 >= 0) {
        if (pos0 <= pos1) { p0 = pos0; p1 = pos1; v0 = val0; v1 = val1; }
        else { p0 = pos1; p1 = pos0; v0 = val1; v1 = val0; }
        return;
    }
    const int real_pos = pos0 >= 0 ? pos0 : pos1;
    const float real_val = pos0 >= 0 ? val0 : val1;
    const int dummy = real_pos == 0 ? 1 : 0;
    if (dummy < real_pos) { p0 = dummy; p1 = real_pos; v0 = 0.f; v1 = real_val; }
    else { p0 = real_pos; p1 = dummy; v0 = real_val; v1 = 0.f; }
}

Format* build(const int* row, const int* column, const float* values, int rows,
              int part_t, int part_c, int short_size, int density, int window,
              float tc_min_util, int skip_tc, int unit_min_nnz, int exhaustive) {
    Format* F = new Format();
    const int tc_wide = 8;
    const int num_windows = (rows + window - 1) / window;

    for (int win = 0; win < num_windows; ++win) {
        const int row_start = win * window;
        const int row_stop = std::min(row_start + window, rows);

        // ---- column info (block_online.cpp:589-603): columns ascending ------------
        std::vector<std::pair<int, std::pair<int, int>>> trip;  // (col, (local_row, edge))
        for (int r = row_start; r < row_stop; ++r)
            for (int e = row[r]; e < row[r + 1]; ++e) trip.push_back({column[e], {r - row_start, e}});
        std::stable_sort(trip.begin(), trip.end(),
                         [](const auto& a, const auto& b) { return a.first < b.first; });
        std::vector<ColInfo> cols;
        for (const auto& t : trip) {
            if (cols.empty() || cols.back().col != t.first) {
                cols.emplace_back();
                cols.back().col = t.first;
            }
            ColInfo& ci = cols.back();
            if (!ci.rows.empty() && ci.rows.back().first == t.second.first) continue;  // dedup per row
            ci.count++;
            ci.vec += (uint32_t)1 << (2 * t.second.first);
            ci.rows.push_back(t.second);
        }
        const int ncol = (int)cols.size();
        auto by_count_then_col = [&](int a, int b) {
            if (cols[a].count != cols[b].count) return cols[a].count > cols[b].count;
            return cols[a].col < cols[b].col;
        };

        // ---- stage 1: TC columns (block_online.cpp:215-253) --------------------------
        // route[i]: -1 undecided, 0 TC, 1 SPTC, 2 CUDA
        std::vector<int> route(ncol, -1);
        std::vector<std::vector<int>> tc_groups;  // column *indices*, ascending col id
        if (!skip_tc) {
            std::vector<int> cand;
            for (int i = 0; i < ncol; ++i)
                if (cols[i].count >= density) cand.push_back(i);
            std::sort(cand.begin(), cand.end(), by_count_then_col);
            for (int start = 0; start < (int)cand.size(); start += tc_wide) {
                const int end = std::min(start + tc_wide, (int)cand.size());
                int real_nnz = 0;
                std::vector<int> group;
                for (int i = start; i < end; ++i) { real_nnz += cols[cand[i]].count; group.push_back(cand[i]); }
                const float util = (float)real_nnz / (float)(window * tc_wide);
                if (util < tc_min_util) continue;
                std::sort(group.begin(), group.end());  // index order == column-id order
                for (int i : group) route[i] = 0;
                tc_groups.push_back(group);
            }
        }
        const bool has_tc = !tc_groups.empty();

        // ---- stage 2a: units (block_online.cpp:267-328) ------------------------------
        std::vector<int> cand;
        for (int i = 0; i < ncol; ++i)
            if (route[i] != 0) cand.push_back(i);
        std::sort(cand.begin(), cand.end(), by_count_then_col);
        std::vector<Unit> units;
        {
            std::vector<char> used(cand.size(), 0);
            for (int i = 0; i < (int)cand.size(); ++i) {
                if (used[i]) continue;
                used[i] = 1;
                const ColInfo& a = cols[cand[i]];
                int best_j = -1;
                for (int j = i + 1; j < (int)cand.size(); ++j) {
                    if (used[j]) continue;
                    if (units_match_check(a.vec, cols[cand[j]].vec)) { best_j = j; break; }
                    F->check_failures++;
                }
                Unit u;
                u.col1 = cand[i];
                u.vec = a.vec;
                u.nnz = a.count;
                if (best_j >= 0) {
                    used[best_j] = 1;
                    u.col2 = cand[best_j];
                    u.vec |= cols[cand[best_j]].vec;
                    u.nnz += cols[cand[best_j]].count;
                }
                units.push_back(u);
            }
        }

        // ---- stage 2b: matching (block_online.cpp:332-392) ---------------------------
        const int U = (int)units.size();
        std::vector<int> degree(U, U > 0 ? U - 1 : 0);
        if (exhaustive) {
            std::fill(degree.begin(), degree.end(), 0);
            for (int i = 0; i < U; ++i)
                for (int j = i + 1; j < U; ++j) {
                    if (units_match_check(units[i].vec, units[j].vec)) { degree[i]++; degree[j]++; }
                    else F->check_failures++;
                }
        }
        std::vector<int> order(U);
        for (int i = 0; i < U; ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](int a, int b) {
            if (degree[a] != degree[b]) return degree[a] > degree[b];
            return units[a].nnz > units[b].nnz;
        });
        std::vector<char> matched(U, 0);
        std::vector<std::pair<int, int>> match_pairs;
        int lowest = 0;  // every index below it is matched (only used when !exhaustive)
        for (int idx : order) {
            if (matched[idx]) continue;
            int best = -1, best_degree = -1;
            while (lowest < U && matched[lowest]) ++lowest;
            // neighbours ascending; the graph is complete so every other unit is one
            for (int nb = exhaustive ? 0 : lowest; nb < U; ++nb) {
                if (nb == idx || matched[nb]) continue;
                if (exhaustive && !units_match_check(units[idx].vec, units[nb].vec)) continue;
                if (degree[nb] > best_degree ||
                    (degree[nb] == best_degree && units[nb].nnz > units[best].nnz)) {
                    best = nb;
                    best_degree = degree[nb];
                }
                if (!exhaustive) break;  // nnz is non-increasing in index: first unmatched wins
            }
            if (best >= 0) {
                matched[idx] = matched[best] = 1;
                match_pairs.push_back({idx, best});
            }
        }

        // ---- stage 2c: groups (block_online.cpp:629-666) ----------------------------
        const int g_begin = (int)F->s_window.size();
        auto emit_group = [&](std::vector<int> g) {
            std::sort(g.begin(), g.end());
            for (int i : g) route[i] = 1;
            F->s_window.push_back(win);
            for (int p = 0; p < 4; ++p) F->s_column.push_back(p < (int)g.size() ? cols[g[p]].col : -1);
            // per-row encode (block_online.cpp:669-701)
            for (int lr = 0; lr < window; ++lr) {
                uint8_t mask = 0;
                int slots = 0;
                float rv[2] = {0.f, 0.f};
                int8_t rp[2] = {-1, -1};
                for (int p = 0; p < (int)g.size(); ++p) {
                    const auto& rr = cols[g[p]].rows;
                    auto it = std::find_if(rr.begin(), rr.end(), [&](const auto& x) { return x.first == lr; });
                    if (it == rr.end()) continue;
                    mask |= (uint8_t)(1 << p);
                    if (slots < 2) { rv[slots] = values[it->second]; rp[slots] = (int8_t)p; }
                    else F->dropped_nnz++;
                    slots++;
                }
                F->s_mask.push_back(mask);
                for (int s = 0; s < 2; ++s) { F->s_value.push_back(rv[s]); F->s_pos.push_back(rp[s]); }
            }
        };
        for (const auto& p : match_pairs) {
            std::vector<int> g;
            g.push_back(units[p.first].col1);
            if (units[p.first].col2 >= 0) g.push_back(units[p.first].col2);
            if (units[p.second].col1 >= 0) g.push_back(units[p.second].col1);
            if (units[p.second].col2 >= 0) g.push_back(units[p.second].col2);
            emit_group(g);
        }
        for (int i = 0; i < U; ++i) {
            if (matched[i] || units[i].nnz < unit_min_nnz) continue;
            std::vector<int> g;
            g.push_back(units[i].col1);
            if (units[i].col2 >= 0) g.push_back(units[i].col2);
            emit_group(g);
        }
        F->s_offset.push_back((int)F->s_window.size());
        (void)g_begin;

        // ---- stage 3: CUDA-core leftovers (block_online.cpp:706-733, 397-439) --------
        bool has_cuda_fallback = false;
        for (int i = 0; i < ncol; ++i)
            if (route[i] < 0) { route[i] = 2; has_cuda_fallback = true; }
        auto col_index = [&](int c) {
            auto it = std::lower_bound(cols.begin(), cols.end(), c,
                                       [](const ColInfo& ci, int v) { return ci.col < v; });
            return (int)(it - cols.begin());
        };
        auto col_route = [&](int c) { return route[col_index(c)]; };

        // ---- TC parts (block_online.cpp:444-540, serialised at 749-758) ---------------
        if (has_tc) {
            const int blocks = (int)tc_groups.size();
            std::vector<uint64_t> lo(blocks, 0), hi(blocks, 0);
            std::vector<std::vector<float>> vals(blocks);
            std::vector<int> tc_slot(ncol, -1);  // column index -> block * 8 + k
            for (int b = 0; b < blocks; ++b)
                for (int p = 0; p < (int)tc_groups[b].size(); ++p) tc_slot[tc_groups[b][p]] = b * 8 + p;
            for (int r = row_start; r < row_stop; ++r) {
                const int lr = r - row_start;
                for (int e = row[r]; e < row[r + 1]; ++e) {
                    const int slot = tc_slot[col_index(column[e])];
                    if (slot < 0) continue;
                    const int b = slot >> 3, k = slot & 7;
                    const uint64_t bit = (uint64_t)1 << ((lr & 7) * 8 + k);
                    if (lr >= 8) hi[b] |= bit; else lo[b] |= bit;
                    vals[b].push_back(values[e]);
                }
            }
            for (int b = 0; b < blocks; ++b) {
                for (int p = 0; p < 8; ++p)
                    F->t_column.push_back(p < (int)tc_groups[b].size() ? cols[tc_groups[b][p]].col : -1);
                F->t_binary.push_back((int64_t)lo[b]);
                F->t_binary.push_back((int64_t)hi[b]);
                F->t_value.insert(F->t_value.end(), vals[b].begin(), vals[b].end());
                F->t_block_offset.push_back(F->t_block_offset.back() + (int)vals[b].size());
            }
            const int code = win * 16;
            if (blocks <= part_t) {
                F->t_row_offset.push_back(F->t_row_offset.back() + blocks);
                F->t_atomic.push_back(has_cuda_fallback ? 1 : 0);
                F->t_window_row.push_back(code);
            } else {
                for (int p = 0; p < blocks / part_t; ++p) {
                    F->t_row_offset.push_back(F->t_row_offset.back() + part_t);
                    F->t_atomic.push_back(1);
                    F->t_window_row.push_back(code);
                }
                if (blocks % part_t) {
                    F->t_row_offset.push_back(F->t_row_offset.back() + blocks % part_t);
                    F->t_atomic.push_back(1);
                    F->t_window_row.push_back(code);
                }
            }
        }

        // ---- CUDA-core row parts ---------------------------------------------------------
        const int base_atomic = has_tc ? 1 : 0;
        for (int r = row_start; r < row_stop; ++r) {
            std::vector<int> cc;
            std::vector<float> cv;
            for (int e = row[r]; e < row[r + 1]; ++e)
                if (col_route(column[e]) == 2) { cc.push_back(column[e]); cv.push_back(values[e]); }
            const int n = (int)cc.size();
            if (n <= 0) continue;
            auto put = [&](int atomic, int off, int cnt, bool residue) {
                auto& ro = residue ? F->cs_row_offset : F->c_row_offset;
                auto& rr = residue ? F->cs_row : F->c_row;
                auto& ra = residue ? F->cs_atomic : F->c_atomic;
                auto& rc = residue ? F->cs_column : F->c_column;
                auto& rv = residue ? F->cs_value : F->c_value;
                ro.push_back(ro.back() + cnt);
                rr.push_back(r);
                ra.push_back(atomic);
                rc.insert(rc.end(), cc.begin() + off, cc.begin() + off + cnt);
                rv.insert(rv.end(), cv.begin() + off, cv.begin() + off + cnt);
            };
            if (n <= short_size) put(base_atomic, 0, n, true);
            else if (n <= part_c) put(base_atomic, 0, n, false);
            else {
                int off = 0;
                for (int p = 0; p < n / part_c; ++p) { put(1, off, part_c, false); off += part_c; }
                const int residue = n % part_c;
                if (residue > 0) put(1, off, residue, residue <= short_size);
            }
        }
    }

    // ---- tile packing (block_online.cpp:796-841) --------------------------------------------
    for (int win = 0; win < num_windows; ++win) {
        const int gb = F->s_offset[win], ge = F->s_offset[win + 1];
        for (int base = gb; base < ge; base += 4) {
            F->s_tile_window.push_back(win);
            F->s_tile_group.push_back(base);
            for (int k = 0; k < 16; ++k) {
                const int gid = base + (k >> 2);
                F->s_tile_column.push_back(gid < ge ? F->s_column[(size_t)gid * 4 + (k & 3)] : -1);
            }
            for (int rg = 0; rg < 8; ++rg) {
                float ar0[8], ar1[8];
                int m0[4], m1[4], m2[4], m3[4];
                for (int ch = 0; ch < 4; ++ch) {
                    float v0, v1; int p0, p1;
                    slot_normalise(*F, base + ch, ge, rg, window, v0, v1, p0, p1);
                    ar0[ch * 2] = v0; ar0[ch * 2 + 1] = v1; m0[ch] = p0; m1[ch] = p1;
                    slot_normalise(*F, base + ch, ge, rg + 8, window, v0, v1, p0, p1);
                    ar1[ch * 2] = v0; ar1[ch * 2 + 1] = v1; m2[ch] = p0; m3[ch] = p1;
                }
                uint32_t meta = 0;
                for (int ch = 0; ch < 4; ++ch) {
                    meta |= ((uint32_t)(m0[ch] & 3) | ((uint32_t)(m1[ch] & 3) << 2)) << (ch * 4);
                    meta |= ((uint32_t)(m2[ch] & 3) | ((uint32_t)(m3[ch] & 3) << 2)) << (16 + ch * 4);
                }
                F->s_packed_meta.push_back((int)meta);
                for (int t = 0; t < 4; ++t) {
                    F->s_packed_a.push_back(pack_half2(ar0[t * 2], ar0[t * 2 + 1]));
                    F->s_packed_a.push_back(pack_half2(ar1[t * 2], ar1[t * 2 + 1]));
                }
            }
        }
        F->s_window_tile_offset.push_back((int)F->s_tile_window.size());
    }
    return F;
}

template <class T>
void copy_out(const std::vector<T>& v, void* dst) {
    if (!v.empty()) std::memcpy(dst, v.data(), v.size() * sizeof(T));
}

}  // namespace

extern "C" {

// Array ids follow the return order of block_sptc_2to4_online (block_online.cpp:844-870).
enum { ORACLE_NUM_ARRAYS = 29 };

void* trs_oracle_build(const int* row, const int* column, const float* values, int rows,
                       int part_t, int part_c, int short_size, int density, int window,
                       float tc_min_util, int skip_tc, int unit_min_nnz, int exhaustive) {
    if (window <= 0 || window > 16) return nullptr;
    return build(row, column, values, rows, part_t, part_c, short_size, density, window,
                 tc_min_util, skip_tc, unit_min_nnz, exhaustive);
}

long long trs_oracle_size(void* h, int id) {
    const Format& f = *(Format*)h;
    switch (id) {
        case 0: return f.t_row_offset.size();   case 1: return f.t_block_offset.size();
        case 2: return f.t_column.size();       case 3: return f.t_value.size();
        case 4: return f.t_window_row.size();   case 5: return f.t_atomic.size();
        case 6: return f.t_binary.size();       case 7: return f.c_row_offset.size();
        case 8: return f.c_row.size();          case 9: return f.c_atomic.size();
        case 10: return f.c_column.size();      case 11: return f.c_value.size();
        case 12: return f.cs_row_offset.size(); case 13: return f.cs_row.size();
        case 14: return f.cs_atomic.size();     case 15: return f.cs_column.size();
        case 16: return f.cs_value.size();      case 17: return f.s_column.size();
        case 18: return f.s_mask.size();        case 19: return f.s_value.size();
        case 20: return f.s_pos.size();         case 21: return f.s_window.size();
        case 22: return f.s_offset.size();      case 23: return f.s_tile_window.size();
        case 24: return f.s_tile_group.size();  case 25: return f.s_tile_column.size();
        case 26: return f.s_packed_a.size();    case 27: return f.s_packed_meta.size();
        case 28: return f.s_window_tile_offset.size();
        case 100: return f.check_failures;
        case 101: return f.dropped_nnz;
    }
    return -1;
}

void trs_oracle_copy(void* h, int id, void* dst) {
    const Format& f = *(Format*)h;
    switch (id) {
        case 0: copy_out(f.t_row_offset, dst); break;   case 1: copy_out(f.t_block_offset, dst); break;
        case 2: copy_out(f.t_column, dst); break;       case 3: copy_out(f.t_value, dst); break;
        case 4: copy_out(f.t_window_row, dst); break;   case 5: copy_out(f.t_atomic, dst); break;
        case 6: copy_out(f.t_binary, dst); break;       case 7: copy_out(f.c_row_offset, dst); break;
        case 8: copy_out(f.c_row, dst); break;          case 9: copy_out(f.c_atomic, dst); break;
        case 10: copy_out(f.c_column, dst); break;      case 11: copy_out(f.c_value, dst); break;
        case 12: copy_out(f.cs_row_offset, dst); break; case 13: copy_out(f.cs_row, dst); break;
        case 14: copy_out(f.cs_atomic, dst); break;     case 15: copy_out(f.cs_column, dst); break;
        case 16: copy_out(f.cs_value, dst); break;      case 17: copy_out(f.s_column, dst); break;
        case 18: copy_out(f.s_mask, dst); break;        case 19: copy_out(f.s_value, dst); break;
        case 20: copy_out(f.s_pos, dst); break;         case 21: copy_out(f.s_window, dst); break;
        case 22: copy_out(f.s_offset, dst); break;      case 23: copy_out(f.s_tile_window, dst); break;
        case 24: copy_out(f.s_tile_group, dst); break;  case 25: copy_out(f.s_tile_column, dst); break;
        case 26: copy_out(f.s_packed_a, dst); break;    case 27: copy_out(f.s_packed_meta, dst); break;
        case 28: copy_out(f.s_window_tile_offset, dst); break;
    }
}

void trs_oracle_free(void* h) { delete (Format*)h; }

// std::sort with the matching comparator on an identity permutation, exposed so that
// the CUDA builder's own introsort emulation can be checked against libstdc++ on the host.
// keys[i] = unit nnz; out[i] = the permutation std::sort leaves (block_online.cpp:358-363
// with all degrees equal).
void trs_oracle_std_sort_order(const int* keys, int n, int* out) {
    for (int i = 0; i < n; ++i) out[i] = i;
    std::sort(out, out + n, [&](int a, int b) { return keys[a] > keys[b]; });
}

uint16_t trs_oracle_f32_to_f16(float f) { return f32_to_f16_bits(f); }

// McIlroy's "killer adversary" played against libstdc++'s std::sort with a descending
// comparator: the returned keys make that same sort exhaust its depth limit.
void trs_oracle_adversary(int n, int* keys) {
    std::vector<int> val(n, n - 1), perm(n);
    const int gas = n - 1;
    int nsolid = 0, candidate = 0;
    for (int i = 0; i < n; ++i) perm[i] = i;
    std::sort(perm.begin(), perm.end(), [&](int x, int y) {
        if (val[x] == gas && val[y] == gas) { if (x == candidate) val[x] = nsolid++; else val[y] = nsolid++; }
        if (val[x] == gas) candidate = x; else if (val[y] == gas) candidate = y;
        return val[x] < val[y];
    });
    for (int i = 0; i < n; ++i) keys[i] = n - val[i];  // descending comparator sees the same order
}

}  // extern "C"
