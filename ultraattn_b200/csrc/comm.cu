// Device-side synchronisation between the GPUs of one NVSwitch domain over symmetric memory.
//
// ua_barrier: every rank writes an epoch number into its slot of every peer's signal pad (a
// release store at system scope, travelling as a plain peer store over NVLink) and then waits
// until all peers' epochs have arrived in its own pad. Epochs only grow, so the pads never need
// resetting and a late reader cannot miss a signal. The wait is bounded: when the time budget
// runs out the kernel records an error in the status word and returns, leaving the context
// usable (the host raises). This replaces the reference's host-driven synchronisation — an 8 GiB
// NCCL all-reduce issued only to line the ranks up before timing (search_algo/benchmark.py:593-594)
// and 1-element warm-up all-reduces (tests/distributed/device_communicators/pynccl.py:195-199).
//
// ua_multimem_bcast / ua_multimem_reduce: NVLS primitives on the multicast address of a symmetric
// buffer (one-to-all block broadcast, all-to-one gradient reduction, one-shot all-reduce); they
// replace the reference's per-peer ncclSend/ncclRecv fan-out of shared blocks
// (orchestrated_attn/orchestrated_attn_impl.py:103-141) and its ring all-reduce call sites.
//
// ua_wait_flag: waits (bounded) for a single 32-bit flag; used by tests of the time-out path: a
// flag that nothing sets makes the wait run out and the status word is checked on the host.
#include "host_common.cuh"
#include "ptx.cuh"

namespace ua {

constexpr int MAX_RANKS = 16;

struct BarrierParams {
  uint32_t* pads[MAX_RANKS];   // pads[r] = rank r's signal pad (peer-mapped addresses)
  int rank;
  int world;
  int channel;                 // independent barriers use different channels
  uint32_t epoch;
  unsigned long long budget_ns;
  int* status;
};

__global__ void barrier_kernel(const __grid_constant__ BarrierParams p) {
  const int peer = threadIdx.x;
  if (peer >= p.world) return;
  // make this GPU's earlier writes (to local and peer memory) visible before the signal
  __threadfence_system();
  uint32_t* remote = p.pads[peer] + p.channel * MAX_RANKS + p.rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(p.epoch) : "memory");
  const uint32_t* mine = p.pads[p.rank] + p.channel * MAX_RANKS + peer;
  unsigned long long t0 = 0;
  for (unsigned it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int>(v - p.epoch) >= 0) break;
    if ((it & 0x3F) == 0x3F) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > p.budget_ns) {
        if (p.status != nullptr && atomicCAS(p.status, 0, UA_ERR_FLAG_TIMEOUT) == 0) {
          p.status[1] = 900 + p.channel;
          p.status[2] = peer;
          p.status[3] = static_cast<int>(p.epoch);
        }
        return;
      }
    }
    __nanosleep(100);
  }
  __threadfence_system();
}

__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t target, unsigned long long budget_ns,
                                 int* status) {
  unsigned long long t0 = 0;
  for (unsigned it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - target) >= 0) return;
    if ((it & 0x3F) == 0x3F) {
      const unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > budget_ns) {
        if (status != nullptr && atomicCAS(status, 0, UA_ERR_FLAG_TIMEOUT) == 0) {
          status[1] = 950;
          status[2] = 0;
          status[3] = static_cast<int>(target);
        }
        return;
      }
    }
    __nanosleep(100);
  }
}

// dst[i] += src[i] (fp32) with vector reductions; dst may be a peer GPU's memory (the adds travel
// as NVLink reduction packets). Optionally clears src afterwards so that it can accumulate the
// next step's partial sums.
__global__ void __launch_bounds__(256)
peer_add_kernel(float* __restrict__ dst, float* __restrict__ src, long n_vec4, int zero_src) {
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec4; i += stride) {
    const float4 v = *reinterpret_cast<const float4*>(src + i * 4);
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + i * 4), "f"(v.x),
                 "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
    if (zero_src) *reinterpret_cast<float4*>(src + i * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}


// dst[i] = src[i] in 16-byte vectors by `gridDim.x` CTAs with the access pattern of the attention
// kernels' staging copies (four independent loads in flight per thread, `ld.global.cg`): src is
// usually a peer GPU's memory. Used to measure how staging throughput grows with the number of
// CTAs that copy (an input of the fused path's cost model).
__global__ void __launch_bounds__(512)
peer_pull_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long n16) {
  const long per = (n16 + gridDim.x - 1) / gridDim.x;
  const long lo = static_cast<long>(blockIdx.x) * per;
  const long hi = lo + per < n16 ? lo + per : n16;
  const long stride = blockDim.x;
  long i = lo + threadIdx.x;
  for (; i + 3 * stride < hi; i += 4 * stride) {
    const uint4 a = __ldcg(src + i);
    const uint4 b = __ldcg(src + i + stride);
    const uint4 c = __ldcg(src + i + 2 * stride);
    const uint4 d = __ldcg(src + i + 3 * stride);
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < hi; i += stride) dst[i] = __ldcg(src + i);
}

// ---- NVLS (NVSwitch multicast) primitives ---------------------------------------------------------
// `mc` is the multicast address of a symmetric buffer: one store to it lands in every rank's
// replica, one load-reduce from it returns the sum over all replicas, both performed by the switch.
// None of these kernels waits on another rank: the callers bracket them with the device barrier.

// every replica[i] = src[i]; 16 bytes per thread and iteration (any dtype, copied as bits)
__global__ void __launch_bounds__(256)
multimem_bcast_kernel(float4* __restrict__ mc, const float4* __restrict__ src, long n16) {
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const float4 v = src[i];
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc + i),
                 "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
  }
}

// dst[i] = sum over replicas of mc[i]  (fp32, or bf16 pairs accumulated in fp32 inside the switch)
template <bool BF16>
__global__ void __launch_bounds__(256)
multimem_reduce_kernel(float4* __restrict__ dst, const float4* __restrict__ mc, long n16,
                       float4* __restrict__ mc_out) {
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    float4 v;
    if (BF16) {
      uint32_t a, b, c, d;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(mc + i) : "memory");
      v = make_float4(__uint_as_float(a), __uint_as_float(b), __uint_as_float(c), __uint_as_float(d));
    } else {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc + i) : "memory");
    }
    if (dst != nullptr) dst[i] = v;
    if (mc_out != nullptr)
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_out + i),
                   "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                   : "memory");
  }
}

}  // namespace ua

using namespace ua;

extern "C" int ua_peer_pull(void* dst, const void* src, long nbytes, int n_ctas, cudaStream_t stream) {
  if (nbytes % 16 != 0 || n_ctas < 1) UA_FAIL("ua_peer_pull: size must be a multiple of 16 bytes, n_ctas >= 1");
  if (nbytes == 0) return 0;
  peer_pull_kernel<<<static_cast<unsigned>(n_ctas), 512, 0, stream>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src), nbytes / 16);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_peer_add_f32(void* dst, void* src, long n, int zero_src, int num_sms,
                               cudaStream_t stream) {
  if (n % 4 != 0) UA_FAIL("ua_peer_add_f32: n must be a multiple of 4");
  if (n == 0) return 0;
  const long n4 = n / 4;
  long blocks = (n4 + 255) / 256;
  if (blocks > static_cast<long>(num_sms) * 8) blocks = static_cast<long>(num_sms) * 8;
  peer_add_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<float*>(dst), static_cast<float*>(src), n4, zero_src);
  UA_CUDA(cudaGetLastError());
  return 0;
}

// pads: host array of `world` device pointers (peer-mapped signal pads, >= 16*channels uint32 each)
extern "C" int ua_barrier(void* const* pads, int rank, int world, int channel, unsigned epoch,
                          double budget_s, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS) UA_FAIL("ua_barrier: world must be in [1, %d]", MAX_RANKS);
  BarrierParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < world; ++i) p.pads[i] = static_cast<uint32_t*>(pads[i]);
  p.rank = rank; p.world = world; p.channel = channel; p.epoch = epoch;
  p.budget_ns = static_cast<unsigned long long>(budget_s * 1e9);
  p.status = status;
  barrier_kernel<<<1, 32, 0, stream>>>(p);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_wait_flag(const void* flag, unsigned target, double budget_s, int* status,
                            cudaStream_t stream) {
  wait_flag_kernel<<<1, 1, 0, stream>>>(static_cast<const uint32_t*>(flag), target,
                                        static_cast<unsigned long long>(budget_s * 1e9), status);
  UA_CUDA(cudaGetLastError());
  return 0;
}

static unsigned nvls_blocks(long n16, int num_sms) {
  long blocks = (n16 + 255) / 256;
  if (blocks > static_cast<long>(num_sms) * 4) blocks = static_cast<long>(num_sms) * 4;
  return static_cast<unsigned>(blocks);
}

// Broadcast `nbytes` of local memory into every rank's replica of a symmetric buffer.
extern "C" int ua_multimem_bcast(void* mc_dst, const void* src, long nbytes, int num_sms,
                                 cudaStream_t stream) {
  if (mc_dst == nullptr) UA_FAIL("ua_multimem_bcast: no multicast address (NVLS unavailable)");
  if (nbytes % 16 != 0 || (reinterpret_cast<uintptr_t>(mc_dst) | reinterpret_cast<uintptr_t>(src)) % 16 != 0)
    UA_FAIL("ua_multimem_bcast: addresses and size must be multiples of 16 bytes");
  if (nbytes == 0) return 0;
  const long n16 = nbytes / 16;
  multimem_bcast_kernel<<<nvls_blocks(n16, num_sms), 256, 0, stream>>>(
      static_cast<float4*>(mc_dst), static_cast<const float4*>(src), n16);
  UA_CUDA(cudaGetLastError());
  return 0;
}

// In-switch sum over the replicas of a symmetric buffer. dst (local, may be null) receives the
// sum; mc_out (multicast, may be null) receives it in every replica (with mc_out == mc_src and
// every rank covering a disjoint slice this is a one-shot all-reduce). bf16 != 0: elements are
// bf16 (accumulated in fp32 inside the switch), else fp32.
extern "C" int ua_multimem_reduce(void* dst, const void* mc_src, void* mc_out, long nbytes, int bf16,
                                  int num_sms, cudaStream_t stream) {
  if (mc_src == nullptr) UA_FAIL("ua_multimem_reduce: no multicast address (NVLS unavailable)");
  if (nbytes % 16 != 0 || (reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(mc_src) |
                           reinterpret_cast<uintptr_t>(mc_out)) % 16 != 0)
    UA_FAIL("ua_multimem_reduce: addresses and size must be multiples of 16 bytes");
  if (nbytes == 0) return 0;
  const long n16 = nbytes / 16;
  if (bf16)
    multimem_reduce_kernel<true><<<nvls_blocks(n16, num_sms), 256, 0, stream>>>(
        static_cast<float4*>(dst), static_cast<const float4*>(mc_src), n16, static_cast<float4*>(mc_out));
  else
    multimem_reduce_kernel<false><<<nvls_blocks(n16, num_sms), 256, 0, stream>>>(
        static_cast<float4*>(dst), static_cast<const float4*>(mc_src), n16, static_cast<float4*>(mc_out));
  UA_CUDA(cudaGetLastError());
  return 0;
}
