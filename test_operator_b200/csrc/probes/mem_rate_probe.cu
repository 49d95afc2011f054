// Standalone probe (not part of the library): how fast a B200 takes fp32 reductions, stores and gathers on random
// 2304-byte rows (one dKV row) or 1152-byte rows (one kv row) of a 75 MB buffer, per SM and chip-wide, for the
// instruction forms the dKV scatter and the kv gather could use:
//   cp.reduce.async.bulk (whole row / three pieces / one issuing warp), red.global.add.v4.f32 warp-per-row,
//   red.global.add.f32 coalesced (what smla_dkv_pair_kernel issues), red.v4 lane-per-row, st.global.v4,
//   ld.global.nc.v4 gathers and cp.async.bulk gathers; plus hot-row (contention) cases.
// Every wait is bounded.  Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o mem_rate_probe mem_rate_probe.cu && ./mem_rate_probe
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} }while(0)

__device__ __forceinline__ uint32_t hash32(uint32_t x){ x ^= x>>16; x*=0x7feb352dU; x^=x>>15; x*=0x846ca68bU; x^=x>>16; return x; }

// mode 0: TMA bulk reduce from smem, one row (row_bytes) per op, issued by lane 0 of each warp.
__global__ void k_bulk_reduce(float* dst, int n_rows, int row_floats, int seg_floats, int rows_per_cta, uint32_t window, uint32_t base){
  extern __shared__ __align__(128) float sm[];
  int nstage = 8;
  for (int i = threadIdx.x; i < nstage*seg_floats; i += blockDim.x) sm[i] = 1.0f;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  int warp = threadIdx.x/32, lane = threadIdx.x%32, nw = blockDim.x/32;
  int nseg = row_floats/seg_floats;
  if (lane==0){
    for (int r = warp; r < rows_per_cta; r += nw){
      uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
      uint32_t row = base + (h % window);
      for (int s=0;s<nseg;s++){
        float* g = dst + (size_t)row*row_floats + s*seg_floats;
        uint32_t sa = (uint32_t)__cvta_generic_to_shared(sm + ((r+s)%nstage)*seg_floats);
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" :: "l"(g), "r"(sa), "r"(seg_floats*4) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group.read 4;" ::: "memory");
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
}

// mode 1: red.global.add.v4.f32, warp per row, 512B per instruction
__global__ void k_red_v4(float* dst, int n_rows, int row_floats, int rows_per_cta, uint32_t window, uint32_t base){
  int warp = threadIdx.x/32, lane = threadIdx.x%32, nw = blockDim.x/32;
  int nvec = row_floats/4;
  for (int r = warp; r < rows_per_cta; r += nw){
    uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
    uint32_t row = base + (h % window);
    float* g = dst + (size_t)row*row_floats;
    for (int v = lane; v < nvec; v += 32){
      asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(g + v*4), "f"(1.f),"f"(1.f),"f"(1.f),"f"(1.f) : "memory");
    }
  }
}
// mode 2: red.global.add.f32 scalar coalesced, 128B per instruction
__global__ void k_red_s(float* dst, int n_rows, int row_floats, int rows_per_cta, uint32_t window, uint32_t base){
  int warp = threadIdx.x/32, lane = threadIdx.x%32, nw = blockDim.x/32;
  for (int r = warp; r < rows_per_cta; r += nw){
    uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
    uint32_t row = base + (h % window);
    float* g = dst + (size_t)row*row_floats;
    for (int v = lane; v < row_floats; v += 32){
      asm volatile("red.global.add.f32 [%0], %1;" :: "l"(g + v), "f"(1.f) : "memory");
    }
  }
}
// mode 3: thread-per-row red.v4 (each lane a different row, 16B each): the "straight from tcgen05.ld 32x32b" pattern
__global__ void k_red_v4_rowperlane(float* dst, int n_rows, int row_floats, int rows_per_cta, uint32_t window, uint32_t base){
  int warp = threadIdx.x/32, lane = threadIdx.x%32, nw = blockDim.x/32;
  int nvec = row_floats/4;
  for (int r0 = warp*32; r0 < rows_per_cta; r0 += nw*32){
    int r = r0 + lane;
    uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
    uint32_t row = base + (h % window);
    float* g = dst + (size_t)row*row_floats;
    for (int v = 0; v < nvec; v++){
      asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" :: "l"(g + v*4), "f"(1.f),"f"(1.f),"f"(1.f),"f"(1.f) : "memory");
    }
  }
}
// mode 4: plain st.global.v4 warp per row (write bandwidth comparison)
__global__ void k_st_v4(float* dst, int n_rows, int row_floats, int rows_per_cta, uint32_t window, uint32_t base){
  int warp = threadIdx.x/32, lane = threadIdx.x%32, nw = blockDim.x/32;
  int nvec = row_floats/4;
  for (int r = warp; r < rows_per_cta; r += nw){
    uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
    uint32_t row = base + (h % window);
    float4* g = (float4*)(dst + (size_t)row*row_floats);
    for (int v = lane; v < nvec; v += 32) g[v] = make_float4(1,1,1,1);
  }
}
// mode 5: gather: ld.global.nc.v4 of random bf16 rows (row_floats*4 bytes... we pass bytes/16 as nvec)
__global__ void k_gather(const uint4* src, int nvec, int rows_per_cta, uint32_t window, uint32_t base, uint4* out){
  int warp = threadIdx.x/32, lane = threadIdx.x%32, nw = blockDim.x/32;
  uint4 acc = make_uint4(0,0,0,0);
  for (int r = warp; r < rows_per_cta; r += nw){
    uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
    uint32_t row = base + (h % window);
    const uint4* g = src + (size_t)row*nvec;
    for (int v = lane; v < nvec; v += 32){ uint4 x = __ldg(g+v); acc.x ^= x.x; acc.y ^= x.y; acc.z^=x.z; acc.w^=x.w; }
  }
  if (acc.x == 0x12345678u) out[threadIdx.x] = acc;
}
// mode 6: bulk gather via cp.async.bulk global->smem of full rows, mbarrier-free variant using bulk_group? (loads need mbarrier) -> use mbarrier with bounded wait
__global__ void k_bulk_gather(const char* src, int row_bytes, int rows_per_cta, uint32_t window, uint32_t base, int* err){
  extern __shared__ __align__(128) char smc[];
  __shared__ __align__(8) unsigned long long bar[8];
  const int NS = 8; const int RPS = 16; // rows per stage
  int tid = threadIdx.x;
  if (tid==0){ for(int i=0;i<NS;i++){ uint32_t b=(uint32_t)__cvta_generic_to_shared(&bar[i]); asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(b)); } asm volatile("fence.mbarrier_init.release.cluster;":::"memory"); }
  __syncthreads();
  if (tid < 32){
    int lane = tid;
    int nsteps = rows_per_cta / RPS;
    for (int st = 0; st < nsteps + NS; st++){
      if (st >= NS){ // wait for stage st-NS
        int s = (st-NS)%NS; uint32_t ph = ((st-NS)/NS)&1; uint32_t b=(uint32_t)__cvta_generic_to_shared(&bar[s]);
        uint32_t ok=0; int it=0;
        while(!ok && it < 2000000){ asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(b), "r"(ph) : "memory"); it++; }
        if(!ok){ if(lane==0) *err = 1; return; }
      }
      if (st < nsteps){
        int s = st%NS; uint32_t b=(uint32_t)__cvta_generic_to_shared(&bar[s]);
        if (lane==0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(b), "r"(RPS*row_bytes) : "memory");
        __syncwarp();
        if (lane < RPS){
          int r = st*RPS + lane;
          uint32_t h = hash32(blockIdx.x*1315423911u + r*2654435761u + 12345u);
          uint32_t row = base + (h % window);
          uint32_t sa = (uint32_t)__cvta_generic_to_shared(smc + (size_t)(s*RPS+lane)*row_bytes);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" :: "r"(sa), "l"(src + (size_t)row*row_bytes), "r"(row_bytes), "r"(b) : "memory");
        }
      }
    }
  }
}

int main(int argc, char** argv){
  int n_rows = 32768, row_floats = 576;
  float* d; size_t bytes = (size_t)n_rows*row_floats*4;
  CK(cudaMalloc(&d, bytes)); CK(cudaMemset(d, 0, bytes));
  int* derr; CK(cudaMalloc(&derr, 4)); CK(cudaMemset(derr,0,4));
  cudaDeviceProp p; CK(cudaGetDeviceProperties(&p,0)); int nsm = p.multiProcessorCount;
  printf("device %s SMs %d L2 %d MB clock %d kHz\n", p.name, nsm, p.l2CacheSize>>20, p.clockRate);
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  CK(cudaFuncSetAttribute(k_bulk_reduce, cudaFuncAttributeMaxDynamicSharedMemorySize, 8*2304+128));
  CK(cudaFuncSetAttribute(k_bulk_gather, cudaFuncAttributeMaxDynamicSharedMemorySize, 8*16*1152+128));
  auto run = [&](const char* name, int mode, int grid, int threads, int rows_per_cta, int seg_floats, uint32_t window, int rowf){
    float best = 1e30f;
    for (int it=0; it<3; it++){
      cudaEventRecord(e0);
      switch(mode){
        case 0: k_bulk_reduce<<<grid,threads,8*seg_floats*4>>>(d,n_rows,rowf,seg_floats,rows_per_cta,window,0); break;
        case 1: k_red_v4<<<grid,threads>>>(d,n_rows,rowf,rows_per_cta,window,0); break;
        case 2: k_red_s<<<grid,threads>>>(d,n_rows,rowf,rows_per_cta,window,0); break;
        case 3: k_red_v4_rowperlane<<<grid,threads>>>(d,n_rows,rowf,rows_per_cta,window,0); break;
        case 4: k_st_v4<<<grid,threads>>>(d,n_rows,rowf,rows_per_cta,window,0); break;
        case 5: k_gather<<<grid,threads>>>((const uint4*)d, 72, rows_per_cta, window*2, 0, (uint4*)d); break; // 1152B rows over same 75MB
        case 6: k_bulk_gather<<<grid,32,8*16*1152>>>((const char*)d, 1152, rows_per_cta, window*2, 0, derr); break;
      }
      cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); CK(cudaGetLastError());
      float ms; cudaEventElapsedTime(&ms,e0,e1); if(ms<best) best=ms;
    }
    double rowbytes = (mode>=5)? 1152.0 : rowf*4.0;
    double gb = (double)grid*rows_per_cta*rowbytes/1e9;
    printf("%-34s grid %4d thr %4d rows/cta %6d win %6u : %8.3f ms  %8.1f GB/s  (%.1f B/clk/SM @1.9GHz)\n", name, grid, threads, rows_per_cta, window, best, gb/(best*1e-3), gb*1e9/(best*1e-3)/grid/1.9e9);
  };
  for (int grid : {1, 16, nsm, 2*nsm}){
    int rpc = grid==1 ? 4096 : 8192;
    run("bulk_reduce row2304", 0, grid, 256, rpc, 576, 32768, 576);
    run("bulk_reduce 3x768", 0, grid, 256, rpc, 192, 32768, 576);
    run("bulk_reduce row2304 1warp", 0, grid, 32, rpc, 576, 32768, 576);
    run("red.v4 warp/row", 1, grid, 256, rpc, 0, 32768, 576);
    run("red.v4 warp/row 1024thr", 1, grid, 1024, rpc, 0, 32768, 576);
    run("red.f32 coalesced", 2, grid, 256, rpc, 0, 32768, 576);
    run("red.v4 row-per-lane", 3, grid, 256, rpc, 0, 32768, 576);
    run("st.v4 warp/row", 4, grid, 256, rpc, 0, 32768, 576);
    run("gather ldg.v4 1152B", 5, grid, 256, rpc*2, 0, 32768, 576);
    run("gather ldg.v4 1152B 1024thr", 5, grid, 1024, rpc*2, 0, 32768, 576);
    run("gather cp.async.bulk 1152B", 6, grid, 32, rpc*2, 0, 32768, 576);
  }
  // contention: hot window
  run("bulk_reduce row2304 hot4096", 0, nsm, 256, 8192, 576, 4096, 576);
  run("bulk_reduce row2304 hot256", 0, nsm, 256, 8192, 576, 256, 576);
  run("red.v4 warp/row hot4096", 1, nsm, 256, 8192, 0, 4096, 576);
  run("red.v4 warp/row hot256", 1, nsm, 256, 8192, 0, 256, 576);
  int herr; CK(cudaMemcpy(&herr, derr, 4, cudaMemcpyDeviceToHost)); printf("err flag %d\n", herr);
  // sanity: sum of dst should equal total adds
  printf("done\n");
  return 0;
}
