// tcgen05.mma issue-rate measurement for sm_100a (a cost-model input: how many clocks one
// M = 128, K = 16 bf16 instruction takes when a single thread issues a long chain into one TMEM
// accumulator). Run by `python -m ultraattn_b200.drivers.cluster_profile --one mma_rate`.
//
// The reference measures its machine with two external profilers (third_party/kernel_profiler,
// third_party/comm_test; scripts/Makefile:90-96) that are not shipped with it; this is one of
// this framework's equivalents at instruction granularity.
//
// Variants: 0 = one lane issues, descriptors rebuilt per instruction; 1 = one lane, descriptor
// words hoisted; 2 / 3 = the whole warp runs the loop and elects the issuing lane per instruction.
// mode 0 (SS) = both operands in shared memory (128-byte swizzle), mode 1 (TS) = A in tensor
// memory. Every variant reaches the pipe's rate (N/2 clocks) except SS with N = 64, which is
// bound by the 128 B/clk shared-memory read bandwidth (6 KB of operands per 32-clock instruction).
// The issue loop must stay branch-free: a data-dependent branch between instructions costs tens
// of clocks per instruction.
#include "host_common.cuh"
#include "ptx.cuh"

namespace ua {

__device__ __forceinline__ void umma_ss_lh(uint32_t d, uint32_t alo, uint32_t ahi, uint32_t blo,
                                           uint32_t bhi, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}\n" ::"r"(d),
      "r"(alo), "r"(ahi), "r"(blo), "r"(bhi), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_ts_lh(uint32_t d, uint32_t a, uint32_t blo, uint32_t bhi,
                                           uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}\n" ::"r"(d),
      "r"(a), "r"(blo), "r"(bhi), "r"(idesc), "r"(acc)
      : "memory");
}

template <int V, int MODE>
__global__ void __launch_bounds__(160, 1) mma_rate_kernel(int N, int iters, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint32_t tbase;
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tbase, 512);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = tbase;
  WaitCtx wc{&abort_flag, status, 1000000000ull};   // one second, then the kernel reports and returns
  if (warp == 1 && (lane == 0 || V >= 2)) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, 0);
    const uint32_t a_addr = smem_u32(sm), b_addr = smem_u32(sm + 32768);
    const uint32_t d = tb;
    const uint32_t hi = static_cast<uint32_t>(make_smem_desc_sw128(0, 16, 1024) >> 32);
    const uint32_t alo = (a_addr & 0x3FFFF) >> 4 | (1u << 16), blo = (b_addr & 0x3FFFF) >> 4 | (1u << 16);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
        if (V == 0 || V == 2) {
          const uint64_t bd = make_smem_desc_sw128(b_addr + off, 16, 1024);
          const uint64_t ad = make_smem_desc_sw128(a_addr + off, 16, 1024);
          if (V == 0 || elect_one()) {
            if (MODE == 0) umma_ss(d, ad, bd, idesc, 1);
            else umma_ts(d, tb + 448 + kk * 8, bd, idesc, 1);
          }
        } else {
          if (V == 1 || elect_one()) {
            if (MODE == 0) umma_ss_lh(d, alo + (off >> 4), hi, blo + (off >> 4), hi, idesc, 1);
            else umma_ts_lh(d, tb + 448 + kk * 8, blo + (off >> 4), hi, idesc, 1);
          }
        }
      }
    }
    const long long t1 = clock64();
    if (V < 2 || elect_one()) tc_commit(&bar);
    mbar_wait(&bar, 0, wc, 900);
    const long long t2 = clock64();
    if (blockIdx.x == 0 && lane == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tb, 512);
  }
}

template <int V, int MODE>
static int launch_rate(int N, int iters, long long* out, int* status, cudaStream_t stream) {
  UA_CUDA(cudaFuncSetAttribute(mma_rate_kernel<V, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
  mma_rate_kernel<V, MODE><<<148, 160, 100 * 1024, stream>>>(N, iters, out, status);
  UA_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace ua

// out_dev: two 64-bit clock counts (issue loop only; until the last instruction completed) of
// CTA 0 over 8 * iters instructions. variant 0..3, mode 0 = SS, 1 = TS, N in {64, 128, 256}.
extern "C" int ua_mma_rate(int variant, int mode, int N, int iters, long long* out_dev, int* status,
                           cudaStream_t stream) {
  using namespace ua;
  if (N != 64 && N != 128 && N != 256) UA_FAIL("ua_mma_rate: N must be 64, 128 or 256");
  switch (variant * 2 + (mode ? 1 : 0)) {
    case 0: return launch_rate<0, 0>(N, iters, out_dev, status, stream);
    case 1: return launch_rate<0, 1>(N, iters, out_dev, status, stream);
    case 2: return launch_rate<1, 0>(N, iters, out_dev, status, stream);
    case 3: return launch_rate<1, 1>(N, iters, out_dev, status, stream);
    case 4: return launch_rate<2, 0>(N, iters, out_dev, status, stream);
    case 5: return launch_rate<2, 1>(N, iters, out_dev, status, stream);
    case 6: return launch_rate<3, 0>(N, iters, out_dev, status, stream);
    case 7: return launch_rate<3, 1>(N, iters, out_dev, status, stream);
  }
  UA_FAIL("ua_mma_rate: variant must be 0..3");
}
