// tcgen05.mma issue-rate probe for sm_100a: how many clocks one M = 128, K = 16 bf16 instruction
// takes when a single thread issues a long dependent chain into one TMEM accumulator.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o mma_rate tcgen05_mma_rate.cu && ./mma_rate
//
// Variants: 0 = one lane issues, descriptors rebuilt per instruction; 1 = one lane, descriptor
// words hoisted; 2 / 3 = the whole warp runs the loop and elects the issuing lane per instruction.
// SS = both operands in shared memory (128-byte swizzle), TS = A in tensor memory.
// Every variant reaches the pipe's rate (N/2 clocks) except SS with N = 64, which is bound by the
// 128 B/clk shared-memory read bandwidth (6 KB of operands per 32-clock instruction).
// The issue loop must stay branch-free: a data-dependent branch between instructions costs
// tens of clocks per instruction (a run-time "mode" switch in an earlier version of this probe
// made every instruction take 94-118 clocks regardless of N).
// Not part of the library.
#include "../ptx.cuh"
#include <cstdio>
using namespace ua;
__device__ __forceinline__ void umma_ss_lh(uint32_t d, uint32_t alo, uint32_t ahi, uint32_t blo, uint32_t bhi, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}\n" ::"r"(d), "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_ts_lh(uint32_t d, uint32_t a, uint32_t blo, uint32_t bhi, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}\n" ::"r"(d), "r"(a), "r"(blo), "r"(bhi), "r"(idesc), "r"(acc) : "memory");
}
// V0: lane 0 only, descriptor built per MMA. V1: lane 0 only, hoisted lo/hi words.
// V2: whole warp runs the loop, elect per MMA, descriptor built per MMA. V3: whole warp + hoisted.
template <int V, int MODE>
__global__ void __launch_bounds__(160,1) k(int N, int iters, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint32_t tbase; __shared__ uint64_t bar[4];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 96*1024/4; i += blockDim.x) ((uint32_t*)sm)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) { for (int i=0;i<4;++i) mbar_init(&bar[i], 1); fence_mbar_init(); }
  if (warp == 0) { tmem_alloc(&tbase, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  uint32_t tb = tbase;
  if (warp == 1 && (lane == 0 || V >= 2)) {
    uint32_t idesc = make_idesc_bf16(128, N, 0, 0);
    uint32_t a_addr = smem_u32(sm), b_addr = smem_u32(sm + 32768);
    uint32_t d = tb;
    uint32_t hi = (uint32_t)(make_smem_desc_sw128(0, 16, 1024) >> 32);
    uint32_t alo = (a_addr & 0x3FFFF) >> 4 | (1u << 16), blo = (b_addr & 0x3FFFF) >> 4 | (1u << 16);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk>>2)*16384 + (kk&3)*32;
        if (V == 0 || V == 2) {
          uint64_t bd = make_smem_desc_sw128(b_addr + off, 16, 1024);
          uint64_t ad = make_smem_desc_sw128(a_addr + off, 16, 1024);
          if (V == 0 || elect_one()) {
            if (MODE == 0) umma_ss(d, ad, bd, idesc, 1); else umma_ts(d, tb + 448 + kk * 8, bd, idesc, 1);
          }
        } else {
          if (V == 1 || elect_one()) {
            if (MODE == 0) umma_ss_lh(d, alo + (off >> 4), hi, blo + (off >> 4), hi, idesc, 1);
            else umma_ts_lh(d, tb + 448 + kk * 8, blo + (off >> 4), hi, idesc, 1);
          }
        }
      }
    }
    long long t1 = clock64();
    if (V < 2 || elect_one()) tc_commit(&bar[0]);
    while (!mbar_try_wait(&bar[0], 0)) {}
    long long t2 = clock64();
    if (blockIdx.x == 0 && lane == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before_sync(); __syncthreads();
  if (warp == 0) { tc_fence_after_sync(); tmem_dealloc(tb, 512); }
}
template <int V, int MODE> void run(int N, long long* out) {
  long long h[2]; int iters = 200;
  cudaFuncSetAttribute(k<V, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100*1024);
  k<V, MODE><<<148, 160, 100*1024>>>(N, iters, out);
  cudaError_t e = cudaDeviceSynchronize();
  cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost);
  printf("%s N=%3d variant %d: issue %.1f complete %.1f clk/MMA %s\n", MODE ? "TS" : "SS", N, V, h[0] / (8.0 * iters), h[1] / (8.0 * iters), e == cudaSuccess ? "" : cudaGetErrorString(e));
}
int main() {
  long long* out; cudaMalloc(&out, 64);
  for (int N : {64, 128, 256}) {
    run<0,0>(N,out); run<1,0>(N,out); run<2,0>(N,out); run<3,0>(N,out);
    run<0,1>(N,out); run<1,1>(N,out); run<2,1>(N,out); run<3,1>(N,out);
  }
  return 0;
}
