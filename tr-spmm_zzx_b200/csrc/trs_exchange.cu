// Dense row-block product fused with the exchange that follows it in a row-sharded GCN layer:
//   Z[row0 + r, :] = H[r, :] * W        (H: this GPU's rows of the hidden matrix, fp16; W: K x N, fp16)
// written from the kernel's epilogue into every destination buffer - this GPU's copy of Z and its
// NVLink peers' copies (peer-mapped pointers) - as 16-byte stores of whole rows.  One kernel does
// the GEMM and the all-gather: no library GEMM, no collective launch, no second pass over Z.
// The reference has neither layers nor multi-GPU code; the layer shape comes from the GCN
// benchmark configuration (features 256 -> 128 -> 64).
//
// The product is memory-bound (K = 128, N = 64: 256 B read and 128 B x destinations written per
// row against 16 K multiply-adds), so the kernel is laid out for streaming: W sits in shared
// memory once per CTA, each warp takes 16-row tiles in a grid-stride loop, loads its tile with
// 16-byte loads, runs K / 16 x N / 8 mma.m16n8k16 (fp32 accumulate) and stores the fp16 rows.
#include "trs_common.cuh"

namespace trs {

struct RowDst {
    void* ptr[8];
    int n;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(addr));
}

constexpr int kGemmWarps = 8;

// One 16-byte store through an NVLink multicast address: the switch delivers it to every GPU bound
// to the multicast object (this one included), so the sender issues each row once instead of once
// per peer.
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

// NT = N / 8 (compile-time so that the accumulators stay in registers); MC: dst.ptr[0] is a
// multicast address and takes the one store per row piece
template <int NT, bool MC>
__global__ void __launch_bounds__(kGemmWarps * 32) k_rows_gemm_bcast(const __half* __restrict__ H, const __half* __restrict__ W,
                                                                     RowDst dst, long long row0, int rows, int K) {
    constexpr int N = NT * 8;
    extern __shared__ __align__(16) unsigned char smem[];
    const int wpitch = (N + 8) * 2;                 // bytes per W row (padded: conflict-free ldmatrix)
    const int hpitch = (K + 8) * 2;                 // bytes per tile row
    unsigned char* Ws = smem;
    unsigned char* Hs = smem + (size_t)K * wpitch + (size_t)(threadIdx.x >> 5) * 16 * hpitch;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // W -> shared memory, once per CTA
    for (int c = threadIdx.x; c < K * NT; c += blockDim.x) {
        const int k = c / NT, ch = c % NT;
        *(uint4*)(Ws + k * wpitch + ch * 16) = __ldg((const uint4*)(W + (size_t)k * N) + ch);
    }
    __syncthreads();
    const int tiles = (rows + 15) / 16;
    const int kchunks = K / 8;                      // 16-byte chunks per H row
    for (int tile = blockIdx.x * kGemmWarps + wid; tile < tiles; tile += gridDim.x * kGemmWarps) {
        const int r_base = tile * 16;
        for (int c = lane; c < 16 * kchunks; c += 32) {
            const int r = c / kchunks, ch = c % kchunks;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r_base + r < rows) v = __ldg((const uint4*)(H + (size_t)(r_base + r) * K) + ch);
            *(uint4*)(Hs + r * hpitch + ch * 16) = v;
        }
        __syncwarp();
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;
        const uint32_t a_addr = smem_u32(Hs) + (lane & 15) * hpitch + (lane >> 4) * 16;
        const uint32_t b_addr = smem_u32(Ws) + (lane & 15) * wpitch;
        for (int k0 = 0; k0 < K; k0 += 16) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(a_addr + k0 * 2, a0, a1, a2, a3);
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                uint32_t b0, b1;
                ldmatrix_x2_trans(b_addr + k0 * wpitch + n * 16, b0, b1);
                mma_16816(acc[n], a0, a1, a2, a3, b0, b1);
            }
        }
        __syncwarp();
        // fp16 rows staged in the tile buffer (pitch of the W rows), then whole rows out in 16-byte pieces
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            *(__half2*)(Hs + g * wpitch + (n * 8 + 2 * t) * 2) = __floats2half2_rn(acc[n][0], acc[n][1]);
            *(__half2*)(Hs + (g + 8) * wpitch + (n * 8 + 2 * t) * 2) = __floats2half2_rn(acc[n][2], acc[n][3]);
        }
        __syncwarp();
        for (int c = lane; c < 16 * NT; c += 32) {
            const int r = c / NT, ch = c % NT;
            if (r_base + r >= rows) continue;
            const uint4 v = *(const uint4*)(Hs + r * wpitch + ch * 16);
            const size_t off = (size_t)(row0 + r_base + r) * N + ch * 8;
            if (MC) multimem_st_16((__half*)dst.ptr[0] + off, v);
            else
                for (int d = 0; d < dst.n; ++d) *(uint4*)((__half*)dst.ptr[d] + off) = v;
        }
        __syncwarp();
    }
}

}  // namespace trs

static int rows_gemm_launch(const trs_half* H, const trs_half* W, void* const* dst, int n_dst, bool multicast,
                            long long row0, int rows, int K, int N, void* stream) {
    using namespace trs;
    if (!H || !W || !dst || n_dst < 1 || n_dst > 8 || row0 < 0 || rows < 0) return TRS_E_ARG;
    if (K < 16 || K > 256 || K % 16 != 0) return TRS_E_ARG;
    if (N != 32 && N != 64 && N != 128) return TRS_E_ARG;
    if (((uintptr_t)H | (uintptr_t)W) & 15) return TRS_E_ARG;
    RowDst rd;
    rd.n = n_dst;
    for (int d = 0; d < 8; ++d) {
        rd.ptr[d] = d < n_dst ? dst[d] : nullptr;
        if (d < n_dst && (!dst[d] || ((uintptr_t)dst[d] & 15))) return TRS_E_ARG;
    }
    if (rows == 0) return TRS_OK;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) return TRS_E_NO_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    // the tile buffer is reused for the N-wide output rows: its rows must hold either
    const int hpitch = (K + 8) * 2, wpitch = (N + 8) * 2;
    if (wpitch > hpitch) return TRS_E_ARG;   // N > K is not laid out for (not a GCN layer shape)
    const int smem = K * wpitch + kGemmWarps * 16 * hpitch;
    const int tiles = (rows + 15) / 16;
    int grid = (tiles + kGemmWarps - 1) / kGemmWarps;
    if (grid > 148 * 4) grid = 148 * 4;   // four CTAs of 256 threads fit an SM at N = 64 (53 KB, 64 registers)
    const __half *h = (const __half*)H, *w = (const __half*)W;
    auto launch = [&](auto kernel) -> int {
        TRS_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kernel<<<grid, kGemmWarps * 32, smem, st>>>(h, w, rd, row0, rows, K);
        return TRS_OK;
    };
    int rc;
    if (multicast) rc = N == 32 ? launch(k_rows_gemm_bcast<4, true>) : N == 64 ? launch(k_rows_gemm_bcast<8, true>) : launch(k_rows_gemm_bcast<16, true>);
    else rc = N == 32 ? launch(k_rows_gemm_bcast<4, false>) : N == 64 ? launch(k_rows_gemm_bcast<8, false>) : launch(k_rows_gemm_bcast<16, false>);
    if (rc) return rc;
    TRS_LAUNCH_CHECK();
    return TRS_OK;
}

extern "C" int trs_rows_gemm_bcast(const trs_half* H, const trs_half* W, void* const* dst, int n_dst, long long row0,
                                   int rows, int K, int N, void* stream) {
    return rows_gemm_launch(H, W, dst, n_dst, false, row0, rows, K, N, stream);
}

extern "C" int trs_rows_gemm_mcast(const trs_half* H, const trs_half* W, void* multicast_dst, long long row0, int rows,
                                   int K, int N, void* stream) {
    void* d[1] = {multicast_dst};
    return rows_gemm_launch(H, W, d, 1, true, row0, rows, K, N, stream);
}
