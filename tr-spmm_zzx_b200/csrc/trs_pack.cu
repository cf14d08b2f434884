// 16x16 mma.sp tile packing on the device (restates block_online.cpp:190-210, 796-841).
//
// One thread packs one (tile, row-pair g / g+8): for each of the tile's four 4-column groups the
// two stored (value, position) slots of the row are normalised to ordered positions p0 < p1 (a
// missing slot gets a dummy position holding 0.0), the values are rounded fp32 -> fp16
// (nearest even) and written as the A registers of lane 4g+t, and the eight 2-bit positions per
// row go into one 32-bit metadata word (low half row g, high half row g+8).
#include "trs_common.cuh"

namespace trs {

__device__ __forceinline__ void slot_normalise(const float* __restrict__ s_value, const int8_t* __restrict__ s_pos,
                                               int group, int group_end, int row, int window, float& v0, float& v1,
                                               int& p0, int& p1) {
    v0 = 0.f; v1 = 0.f; p0 = 0; p1 = 1;
    if (group >= group_end || row >= window) return;
    const size_t base = ((size_t)group * window + row) * 2;
    const int q0 = s_pos[base], q1 = s_pos[base + 1];
    const float x0 = s_value[base], x1 = s_value[base + 1];
    if (q0 < 0 && q1 < 0) return;
    if (q0 >= 0 && q1 >= 0) {
        if (q0 <= q1) { p0 = q0; p1 = q1; v0 = x0; v1 = x1; }
        else { p0 = q1; p1 = q0; v0 = x1; v1 = x0; }
        return;
    }
    const int rp = q0 >= 0 ? q0 : q1;
    const float rv = q0 >= 0 ? x0 : x1;
    const int dummy = rp == 0 ? 1 : 0;
    if (dummy < rp) { p0 = dummy; p1 = rp; v0 = 0.f; v1 = rv; }
    else { p0 = rp; p1 = dummy; v0 = rv; v1 = 0.f; }
}

__device__ __forceinline__ uint32_t pack_half2_rn(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}

__global__ void k_pack_tiles(const int* __restrict__ s_column, const float* __restrict__ s_value,
                             const int8_t* __restrict__ s_pos, const int* __restrict__ s_offset,
                             const int* __restrict__ tile_window, const int* __restrict__ tile_group, long long tiles,
                             int window, int* __restrict__ s_tile_column, uint32_t* __restrict__ packed_a,
                             uint32_t* __restrict__ packed_meta) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tiles * 8) return;
    const long long tile = idx >> 3;
    const int rg = (int)(idx & 7);
    const int win = tile_window[tile];
    const int base = tile_group[tile];
    const int gend = s_offset[win + 1];
    // two of the tile's 16 column ids per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int k = rg * 2 + i;
        const int gid = base + (k >> 2);
        s_tile_column[tile * 16 + k] = gid < gend ? s_column[(size_t)gid * 4 + (k & 3)] : -1;
    }
    uint32_t meta = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float v0, v1, w0, w1;
        int p0, p1, q0, q1;
        slot_normalise(s_value, s_pos, base + c, gend, rg, window, v0, v1, p0, p1);
        slot_normalise(s_value, s_pos, base + c, gend, rg + 8, window, w0, w1, q0, q1);
        meta |= ((uint32_t)(p0 & 3) | ((uint32_t)(p1 & 3) << 2)) << (c * 4);
        meta |= ((uint32_t)(q0 & 3) | ((uint32_t)(q1 & 3) << 2)) << (16 + c * 4);
        packed_a[tile * 64 + rg * 8 + c * 2] = pack_half2_rn(v0, v1);
        packed_a[tile * 64 + rg * 8 + c * 2 + 1] = pack_half2_rn(w0, w1);
    }
    packed_meta[tile * 8 + rg] = meta;
}

int pack_tiles(const int* s_column, const float* s_value, const int8_t* s_pos, const int* s_offset,
               const int* tile_window, const int* tile_group, long long tiles, int window, int* s_tile_column,
               uint32_t* packed_a, uint32_t* packed_meta, cudaStream_t st) {
    if (tiles <= 0) return TRS_OK;
    const long long threads = tiles * 8;
    k_pack_tiles<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(s_column, s_value, s_pos, s_offset, tile_window,
                                                                   tile_group, tiles, window, s_tile_column, packed_a,
                                                                   packed_meta);
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

}  // namespace trs
