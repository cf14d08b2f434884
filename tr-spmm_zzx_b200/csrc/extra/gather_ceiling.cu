// Stand-alone micro-benchmark: how fast can a B200 pull random fixed-size rows of a dense matrix
// through L2 with plain 16-byte loads?  This is the ceiling of any SpMM that gathers one B row
// per (window, column) pair.  Not part of libtrspmm.so.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o gather_ceiling tr-spmm_zzx_b200/csrc/extra/gather_ceiling.cu
//   ./gather_ceiling
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include <vector>
#include <cstdint>
template <int UNROLL, int ROWB>
__global__ void gather(const uint4* __restrict__ B, const int* __restrict__ idx, long long nidx, unsigned nrows, unsigned long long* sink) {
    // a group of ROWB/16 lanes reads one row with 16B loads
    constexpr int LPR = ROWB / 16;            // lanes per row
    constexpr int RPW = 32 / LPR;             // rows per warp-instruction
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    unsigned acc = 0;
    for (long long base = warp * UNROLL * RPW; base + UNROLL * RPW <= nidx; base += nwarps * UNROLL * RPW) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const unsigned r = (unsigned)__ldg(idx + base + u * RPW + lane / LPR) % nrows;  // nrows counts ROWB-byte rows
            v[u] = __ldg(B + (size_t)r * LPR + (lane % LPR));
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) acc += v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    if (acc == 0x12345678u) atomicAdd(sink, 1ull);
}
__global__ void stream_read(const uint4* __restrict__ B, size_t n, unsigned long long* sink) {
    unsigned acc = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = __ldg(B + i); acc += v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x12345678u) atomicAdd(sink, 1ull);
}
int main() {
    unsigned long long* sink; cudaMalloc(&sink, 8);
    const long long nidx = 1 << 24;   // 16M row reads = 4 GB of traffic at 256B
    int* d_idx; cudaMalloc(&d_idx, nidx * 4);
    for (size_t mb : {16, 48, 96, 192, 512, 2048}) {
        const size_t rows = mb * 1024 * 1024 / 256;
        uint4* B; cudaMalloc(&B, rows * 256); cudaMemset(B, 1, rows * 256);
        std::vector<int> h(nidx);
        uint64_t s = 88172645463325252ull;
        for (auto& x : h) { s ^= s << 13; s ^= s >> 7; s ^= s << 17; x = (int)(s % rows); }
        cudaMemcpy(d_idx, h.data(), nidx * 4, cudaMemcpyHostToDevice);
        cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
        auto run = [&](const char* name, auto launch, double bytes) {
            for (int i = 0; i < 2; ++i) launch();
            cudaEventRecord(a);
            for (int i = 0; i < 5; ++i) launch();
            cudaEventRecord(b); cudaEventSynchronize(b);
            float ms; cudaEventElapsedTime(&ms, a, b); ms /= 5;
            cudaError_t e = cudaGetLastError(); if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); exit(1); }
            printf("B=%4zu MB %-28s %.3f ms  %.2f TB/s\n", mb, name, ms, bytes / ms / 1e9);
        };
        run("gather256 unroll4 (1024thr)", [&] { gather<4, 256><<<148 * 2, 1024>>>(B, d_idx, nidx, (unsigned)rows, sink); }, nidx * 256.0);
        run("gather256 unroll8 (512thr)", [&] { gather<8, 256><<<148 * 4, 512>>>(B, d_idx, nidx, (unsigned)rows, sink); }, nidx * 256.0);
        run("gather512 unroll8 (512thr)", [&] { gather<8, 512><<<148 * 4, 512>>>((const uint4*)B, d_idx, nidx / 2, (unsigned)(rows / 2), sink); }, nidx / 2 * 512.0);
        run("gather128 unroll8 (512thr)", [&] { gather<8, 128><<<148 * 4, 512>>>((const uint4*)B, d_idx, nidx, (unsigned)(rows * 2), sink); }, nidx * 128.0);
        run("stream read", [&] { stream_read<<<148 * 8, 512>>>(B, rows * 16, sink); }, rows * 256.0);
        cudaFree(B);
    }
    printf("%s\n", cudaGetErrorString(cudaDeviceSynchronize()));
    return 0;
}
