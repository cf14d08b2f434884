// Shared helpers for libtrspmm's translation units (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "trspmm.h"

#define TRS_CUDA(expr)                                     \
    do {                                                   \
        cudaError_t _e = (expr);                           \
        if (_e != cudaSuccess) return (int)_e;             \
    } while (0)

#define TRS_LAUNCH_CHECK()                                 \
    do {                                                   \
        cudaError_t _e = cudaGetLastError();               \
        if (_e != cudaSuccess) return (int)_e;             \
    } while (0)

namespace trs {

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline long long ceil_div64(long long a, long long b) { return (a + b - 1) / b; }

// Caller-owned device memory handed to a call that would otherwise allocate: blocks are cut off
// the front (256-byte aligned); a block given back is kept on a free list and handed out again
// to the next request it fits, which is what keeps the footprint of a pass with many temporaries
// near its peak instead of its sum.  Not thread-safe: one arena serves one call at a time.
struct Arena {
    unsigned char* base = nullptr;
    size_t cap = 0, used = 0, high = 0;
    struct Free { unsigned char* p; size_t bytes; };
    Free free_list[64];
    int n_free = 0;
    unsigned char* take(size_t bytes) {
        bytes = (bytes + 255) & ~(size_t)255;
        if (bytes == 0) bytes = 256;
        int best = -1;
        for (int i = 0; i < n_free; ++i)
            if (free_list[i].bytes >= bytes && (best < 0 || free_list[i].bytes < free_list[best].bytes)) best = i;
        if (best >= 0 && free_list[best].bytes <= bytes + bytes / 4) {   // close fit: reuse whole
            unsigned char* p = free_list[best].p;
            free_list[best] = free_list[--n_free];
            return p;
        }
        if (used + bytes > cap) return nullptr;
        unsigned char* p = base + used;
        used += bytes;
        if (used > high) high = used;
        return p;
    }
    void give_back(void* p, size_t bytes) {
        bytes = (bytes + 255) & ~(size_t)255;
        if (bytes == 0) bytes = 256;
        if ((unsigned char*)p + bytes == base + used) { used -= bytes; return; }   // last block: shrink
        if (n_free < 64) free_list[n_free++] = Free{(unsigned char*)p, bytes};
    }
};

// Simple owning device buffer for plan-lifetime index arrays; with an arena the memory is the
// caller's and release() only forgets it.
template <class T>
struct DevBuf {
    T* p = nullptr;
    size_t n = 0;
    bool owned = true;
    int alloc(size_t count) { return alloc_from(nullptr, count); }
    int alloc_from(Arena* arena, size_t count) {
        n = count;
        if (count == 0) { p = nullptr; return 0; }
        if (arena) {
            p = (T*)arena->take(count * sizeof(T));
            owned = false;
            return p ? 0 : TRS_E_WORKSPACE;
        }
        owned = true;
        cudaError_t e = cudaMalloc((void**)&p, count * sizeof(T));
        return e == cudaSuccess ? 0 : (int)e;
    }
    void release() {
        if (p && owned) cudaFree(p);
        p = nullptr;
        n = 0;
    }
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16-byte asynchronous global->shared copy; src_bytes = 0 writes zeros instead.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8,f32) += A(16x16 with 2:4 sparsity, stored 16x8 f16) * B(16x8 f16).
// `meta`: bits 4c..4c+3 = the two kept positions (p0 | p1<<2, p0<p1) of 4-column chunk c for
// row lane/4; bits 16+4c.. the same for row lane/4+8.  All four lanes of a quad pass the same
// word, so the thread selector is immaterial.
__device__ __forceinline__ void mma_sp_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, uint32_t b1,
                                             uint32_t meta) {
    asm volatile(
        "mma.sp::ordered_metadata.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5}, {%6,%7}, {%0,%1,%2,%3}, %8, 0x0;\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(b1), "r"(meta));
}

// D(16x8,f32) += A(16x16 f16) * B(16x8 f16)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- mbarrier + bulk copies (TMA, untiled, one CTA as destination) -------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports false (the caller flags the error and
// unwinds); a healthy pipeline completes within a few polls.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> this CTA's shared memory, completion counted in bytes on an mbarrier; 16-byte
// aligned addresses and a size that is a multiple of 16
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// trs_pack.cu
int pack_tiles(const int* s_column, const float* s_value, const int8_t* s_pos, const int* s_offset,
               const int* tile_window, const int* tile_group, long long tiles, int window, int* s_tile_column,
               uint32_t* packed_a, uint32_t* packed_meta, cudaStream_t st);

}  // namespace trs
