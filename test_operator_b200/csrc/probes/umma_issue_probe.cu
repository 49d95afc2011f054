// Standalone probe (not part of the library): how fast threads of a CTA can feed the tensor pipe of a B200 with
// tcgen05.mma (kind::f16, K = 16) in the way the kernels of this library do - chunks of four UMMAs on operands that
// rotate through a ring in shared memory, a tcgen05.commit behind every chunk - with one issuing thread or two (each
// thread on accumulators of its own, so no order between them is needed), for
//   cta_group::1  M 128 x N {64, 128, 256}, one CTA or one per SM
//   cta_group::2  M 256 x N {64, 128, 256}, one 2-CTA cluster
// Operand values are irrelevant (whatever is in shared memory); results are never read.  Every wait is bounded.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o umma_issue_probe umma_issue_probe.cu && ./umma_issue_probe
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at line %d\n", cudaGetErrorString(e), __LINE__); exit(1); } } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(16 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | ((uint64_t)2 << 61);
}
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {   // bf16 x bf16 -> fp32, both operands K-major
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok = 0;
    for (int it = 0; !ok && it < 4000000; ++it)
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// ---- cta_group::1 --------------------------------------------------------------------------------------------
// flags: bit 0 two issuing threads (warps 0 and 1), bit 1 no commit per chunk
__global__ void __launch_bounds__(128) probe_1cta(long long* out, int n_chunks, int N, int flags, int slot) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bar_done[2], bar_chunk[16];
    __shared__ uint32_t tslot;
    const int tid = threadIdx.x;
    for (int i = tid; i < 224 * 1024 / 4; i += 128) ((uint32_t*)smem)[i] = 0x3c003c00u;   // bf16 1.0
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_done[i])));
        for (int i = 0; i < 16; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_chunk[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (tid < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tslot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tslot;
    const bool two = flags & 1;
    const int x = tid >> 5;
    if ((tid & 31) == 0 && (x == 0 || (two && x == 1))) {
        const uint32_t idesc = make_idesc(128, N);
        const uint32_t sb = smem_u32(smem);
        const long long t0 = clock64();
        int n = 0;
        for (int c = x; c < n_chunks; c += two ? 2 : 1, ++n) {
            // A: a ring of five 16 KB chunks behind nine resident 16 KB chunks of B; accumulators of 128 columns
            const uint32_t a = sb + 9 * 16384 + (c % 5) * 16384, b = sb + ((c / 2) % 9) * 16384;
            const uint32_t acc = tmem + x * 256 + ((n / 9) & 1) * 128;
            const uint64_t ad = make_desc(a), bd = make_desc(b);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)   // 32 bytes further along K = +2 in the address field
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                             ::"r"(acc), "l"(ad + 2 * kk), "l"(bd + 2 * kk), "r"(idesc), "r"((uint32_t)(n % 9 + kk)) : "memory");
            if (!(flags & 2))
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar_chunk[c % 16])) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar_done[x])) : "memory");
        const bool ok = bounded_wait(smem_u32(&bar_done[x]), 0);
        const long long t1 = clock64();
        if (blockIdx.x == 0 && x == 0) { out[slot * 2] = t1 - t0; out[slot * 2 + 1] = ok; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

// ---- cta_group::2 --------------------------------------------------------------------------------------------
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128) probe_2cta(long long* out, int n_chunks, int N, int flags, int slot) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bar_done[2], bar_chunk[4];
    __shared__ uint32_t tslot;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int tid = threadIdx.x;
    for (int i = tid; i < 160 * 1024 / 4; i += 128) ((uint32_t*)smem)[i] = 0x3c003c00u;
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_done[i])));
        for (int i = 0; i < 4; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_chunk[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (tid < 32) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tslot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tslot;
    const bool two = flags & 1;
    const int x = tid >> 5;
    if (rank == 0 && (tid & 31) == 0 && (x == 0 || (two && x == 1))) {
        const uint32_t idesc = make_idesc(256, N);
        const uint32_t sb = smem_u32(smem);
        const long long t0 = clock64();
        int n = 0;
        for (int c = x; c < n_chunks; c += two ? 2 : 1, ++n) {
            const uint32_t a = sb + (c % 5) * 16384, b = sb + 81920 + (c % 4) * 16384;
            // one issuer: two buffers of 256 columns; two issuers: each its own pair of N <= 128 column buffers
            const uint32_t acc = two ? tmem + x * 256 + ((n / 9) & 1) * 128 : tmem + ((n / 9) & 1) * 256;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                             ::"r"(acc), "l"(make_desc(a + kk * 32)), "l"(make_desc(b + kk * 32)), "r"(idesc), "r"((uint32_t)(n % 9 + kk)) : "memory");
            if (!(flags & 2))     // delivered to both CTAs of the pair, as the kernels do
                asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                             ::"r"(smem_u32(&bar_chunk[2 * x + (n & 1)])), "h"((uint16_t)3) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar_done[x])) : "memory");
        const bool ok = bounded_wait(smem_u32(&bar_done[x]), 0);
        const long long t1 = clock64();
        if (x == 0) { out[slot * 2] = t1 - t0; out[slot * 2 + 1] = ok; }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

int main() {
    long long* d;
    CK(cudaMalloc(&d, 64 * 2 * 8));
    CK(cudaMemset(d, 0, 64 * 2 * 8));
    CK(cudaFuncSetAttribute(probe_1cta, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    CK(cudaFuncSetAttribute(probe_2cta, cudaFuncAttributeMaxDynamicSharedMemorySize, 164 * 1024));
    int n_sm = 0;
    CK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, 0));
    const int n = 4608;
    struct Cfg { int group, N, flags, grid; };
    const Cfg cfg[] = {{1, 128, 0, 1}, {1, 128, 2, 1}, {1, 128, 1, 1}, {1, 128, 1, n_sm}, {1, 64, 0, 1}, {1, 64, 1, 1}, {1, 256, 2, 1},
                       {2, 256, 0, 2}, {2, 256, 2, 2}, {2, 128, 0, 2}, {2, 128, 1, 2}, {2, 64, 0, 2}, {2, 64, 1, 2}};
    const int nc = sizeof(cfg) / sizeof(cfg[0]);
    for (int rep = 0; rep < 2; ++rep)
        for (int i = 0; i < nc; ++i) {
            if (cfg[i].group == 1) probe_1cta<<<cfg[i].grid, 128, 226 * 1024>>>(d, n, cfg[i].N, cfg[i].flags, i);
            else probe_2cta<<<cfg[i].grid, 128, 164 * 1024>>>(d, n, cfg[i].N, cfg[i].flags, i);
            CK(cudaDeviceSynchronize());
        }
    long long h[64 * 2];
    CK(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
    for (int i = 0; i < nc; ++i)
        printf("cta_group::%d M %3d N %3d  issuing threads %d  commit per chunk %d  CTAs %3d : %6.1f cycles per chunk of 4 UMMAs = %5.1f per UMMA (all issuers together; completed %lld)\n",
               cfg[i].group, cfg[i].group * 128, cfg[i].N, (cfg[i].flags & 1) + 1, !(cfg[i].flags & 2), cfg[i].grid, (double)h[i * 2] / n,
               (double)h[i * 2] / n / 4, h[i * 2 + 1]);
    return 0;
}
