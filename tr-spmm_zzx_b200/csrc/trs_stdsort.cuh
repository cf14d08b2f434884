// Step-for-step emulation of libstdc++'s std::sort (introsort) on an int array, usable from
// host and device code.
//
// Why it exists: the reference orders the units of a window with std::sort and a comparator
// that has ties (TR-source/Block/block_online.cpp:358-363), so its output depends on how
// libstdc++ happens to move equal keys.  A bit-exact builder has to move them the same way.
// The algorithm below is the published libstdc++ one (bits/stl_algo.h, bits/stl_heap.h, GCC 13):
//   sort            = introsort_loop(first, last, 2*floor(log2(n))) + final_insertion_sort
//   introsort_loop  = while range > 16: depth exhausted -> heap sort of the range; else
//                     median-of-three of (first+1, mid, last-1) moved to first, unguarded
//                     Hoare partition of (first+1, last) around *first, recurse on the right part
//   final insertion = guarded insertion sort of the first 16, unguarded linear inserts after
// `less(a, b)` must be the strict weak order the caller would hand to std::sort.
#pragma once

#ifdef __CUDACC__
#define TRS_HD __host__ __device__
#else
#define TRS_HD
#endif

namespace trs {

template <class Less>
struct StdSort {
    int* a;
    Less less;
    int heap_sorts = 0;  // how many ranges fell back to heap sort (diagnostics / tests)

    TRS_HD StdSort(int* arr, Less l) : a(arr), less(l) {}

    TRS_HD static int floor_log2(int n) {
        int r = 0;
        while (n > 1) { n >>= 1; ++r; }
        return r;
    }
    TRS_HD void swap(int i, int j) { const int t = a[i]; a[i] = a[j]; a[j] = t; }

    // std::__move_median_to_first(result, a, b, c)
    TRS_HD void move_median_to_first(int result, int x, int y, int z) {
        if (less(a[x], a[y])) {
            if (less(a[y], a[z])) swap(result, y);
            else if (less(a[x], a[z])) swap(result, z);
            else swap(result, x);
        } else if (less(a[x], a[z])) swap(result, x);
        else if (less(a[y], a[z])) swap(result, z);
        else swap(result, y);
    }

    // std::__unguarded_partition(first, last, pivot)
    TRS_HD int unguarded_partition(int first, int last, int pivot) {
        while (true) {
            while (less(a[first], a[pivot])) ++first;
            --last;
            while (less(a[pivot], a[last])) --last;
            if (!(first < last)) return first;
            swap(first, last);
            ++first;
        }
    }

    // ---- heap sort of [base, base + len): std::__partial_sort(first, last, last) ----------
    TRS_HD void push_heap(int base, int hole, int top, int value) {
        int parent = (hole - 1) / 2;
        while (hole > top && less(a[base + parent], value)) {
            a[base + hole] = a[base + parent];
            hole = parent;
            parent = (hole - 1) / 2;
        }
        a[base + hole] = value;
    }
    TRS_HD void adjust_heap(int base, int hole, int len, int value) {
        const int top = hole;
        int child = hole;
        while (child < (len - 1) / 2) {
            child = 2 * (child + 1);
            if (less(a[base + child], a[base + child - 1])) --child;
            a[base + hole] = a[base + child];
            hole = child;
        }
        if ((len & 1) == 0 && child == (len - 2) / 2) {
            child = 2 * (child + 1);
            a[base + hole] = a[base + child - 1];
            hole = child - 1;
        }
        push_heap(base, hole, top, value);
    }
    TRS_HD void heap_sort(int base, int len) {
        ++heap_sorts;
        if (len >= 2) {  // make_heap
            int parent = (len - 2) / 2;
            while (true) {
                const int value = a[base + parent];
                adjust_heap(base, parent, len, value);
                if (parent == 0) break;
                --parent;
            }
        }
        int last = len;  // sort_heap
        while (last > 1) {
            --last;
            const int value = a[base + last];
            a[base + last] = a[base];
            adjust_heap(base, 0, last, value);
        }
    }

    // ---- insertion sorts -----------------------------------------------------------------
    TRS_HD void unguarded_linear_insert(int last) {
        const int val = a[last];
        int next = last - 1;
        while (less(val, a[next])) {
            a[last] = a[next];
            last = next;
            --next;
        }
        a[last] = val;
    }
    TRS_HD void insertion_sort(int first, int last) {
        if (first == last) return;
        for (int i = first + 1; i != last; ++i) {
            if (less(a[i], a[first])) {
                const int val = a[i];
                for (int k = i; k > first; --k) a[k] = a[k - 1];
                a[first] = val;
            } else {
                unguarded_linear_insert(i);
            }
        }
    }

    // std::__introsort_loop(a + first, a + last, depth): leaves ranges of <= 16 elements unsorted.
    // The recursion takes the right part and loops on the left one; the two are disjoint, so the
    // order in which they are processed is free and an explicit stack does.
    TRS_HD void introsort_range(int first0, int last0, int depth0) {
        int st_first[64], st_last[64], st_depth[64];
        int sp = 1;
        st_first[0] = first0; st_last[0] = last0; st_depth[0] = depth0;
        while (sp > 0) {
            --sp;
            int first = st_first[sp], last = st_last[sp], depth = st_depth[sp];
            while (last - first > 16) {
                if (depth == 0) {
                    heap_sort(first, last - first);
                    break;
                }
                --depth;
                const int mid = first + (last - first) / 2;
                move_median_to_first(first, first + 1, mid, last - 1);
                const int cut = unguarded_partition(first + 1, last, first);
                if (last - cut > 16 && sp < 64) {
                    st_first[sp] = cut; st_last[sp] = last; st_depth[sp] = depth;
                    ++sp;
                }
                last = cut;
            }
        }
    }

    // What std::__final_insertion_sort does to the elements of [first, last) when that range is a
    // union of whole partition leaves: no element moves past a leaf boundary (everything to the
    // left of a leaf is not greater), so a guarded insertion sort of the range alone is identical.
    TRS_HD void insertion_range(int first, int last) { insertion_sort(first, last); }

    // std::sort(a, a + n, less)
    TRS_HD void sort(int n) {
        if (n <= 0) return;
        introsort_range(0, n, 2 * floor_log2(n));
        if (n > 16) {
            insertion_sort(0, 16);
            for (int i = 16; i != n; ++i) unguarded_linear_insert(i);
        } else {
            insertion_sort(0, n);
        }
    }
};

}  // namespace trs
