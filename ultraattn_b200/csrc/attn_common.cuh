// Data structures shared by the block-sparse attention forward and backward kernels.
//
// The attention problem handed to a kernel is a list of "block rows" (forward) or "block
// columns" (backward). A forward block row is a range of Bq query tokens plus a list of
// key/value segments it attends to; each segment names the buffer it lives in (`src`, an index
// into a small table of tensor maps, so that a segment may sit in this GPU's own K/V, in a
// staging buffer filled from a peer, or directly in a peer GPU's memory), its first token, its
// length and whether it is causal relative to the query block.
//
// This is the device-side form of the block table of the planner (reference:
// search_algo/bsa_config.py BSA_Repr, search_algo/utils.py:135-149 Block_Type {EMPTY, FULL,
// CAUSAL}); EMPTY blocks simply have no segment.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

namespace ua {

constexpr int ATTN_MAX_SRC = 10;   // tensor-map slots for K/V (fwd) or Q-side (bwd) sources
constexpr int ATTN_D = 128;        // head dimension these kernels are built for
constexpr int ATTN_TILE = 128;     // query / key tile edge

// One key/value segment attended by a query block (forward), or one query segment attending a
// key block (backward).
struct AttnSeg {
  int src;      // source slot
  int start;    // first token inside the source buffer
  int len;      // tokens
  int causal;   // 0: every (q,k) pair allowed; 1: key c allowed for query r iff c <= r + diag
  int diag;     // (r and c are 0-based inside the query block / the segment)
  int wait_flag;   // 0: data is in place; f > 0: wait until stage_flags[f - 1] >= wait_count
  int wait_count;
  int pad2;
};

// One chunk of the in-kernel staging prologue: copy n_vec16 16-byte vectors from src (usually a
// peer GPU's memory, read with plain peer loads over NVLink) to dst (this GPU's staging mirror),
// then bump stage_flags[flag].
struct CopyTask {
  const uint4* src;
  uint4* dst;
  long n_vec16;
  int flag;
  int pad;
};

struct StageParams {
  const CopyTask* tasks;
  int n_tasks;
  int n_copy_ctas;         // the first n_copy_ctas CTAs (linear id) share the tasks round-robin
  unsigned int* flags;     // monotonically increasing counters, never reset
  int epoch;               // call number (1, 2, ...): a block is ready at wait_count * epoch
};

#ifdef __CUDACC__
// Staging prologue, executed by every thread of the first n_copy_ctas CTAs before they take up
// their own tile. The copy never waits on anything, so a CTA that later waits for a staged block
// only ever waits on work that is unconditionally in progress.
__device__ __forceinline__ void run_stage_prologue(const StageParams& sp, int cta_linear) {
  if (sp.n_tasks == 0 || cta_linear >= sp.n_copy_ctas) return;
  for (int t = cta_linear; t < sp.n_tasks; t += sp.n_copy_ctas) {
    const CopyTask task = sp.tasks[t];
    const long n = task.n_vec16;
    long i = threadIdx.x;
    const long stride = blockDim.x;
    // 4 independent 16-byte peer loads in flight per thread
    for (; i + 3 * stride < n; i += 4 * stride) {
      const uint4 a = __ldcg(task.src + i);
      const uint4 b = __ldcg(task.src + i + stride);
      const uint4 c = __ldcg(task.src + i + 2 * stride);
      const uint4 d = __ldcg(task.src + i + 3 * stride);
      task.dst[i] = a;
      task.dst[i + stride] = b;
      task.dst[i + 2 * stride] = c;
      task.dst[i + 3 * stride] = d;
    }
    for (; i < n; i += stride) task.dst[i] = __ldcg(task.src + i);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(sp.flags + task.flag, 1u);
  }
}

// Bounded wait (single thread) until a staged block is complete. Returns false on time-out.
__device__ __forceinline__ bool wait_staged(const unsigned int* flags, int wait_flag, int wait_count,
                                            unsigned long long budget_ns) {
  if (wait_flag == 0) return true;
  const unsigned int* f = flags + (wait_flag - 1);
  unsigned long long t0 = 0;
  for (unsigned it = 0;; ++it) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (static_cast<int>(v - static_cast<unsigned>(wait_count)) >= 0) break;
    if ((it & 0xFF) == 0xFF) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      if (now - t0 > budget_ns) return false;
    }
    __nanosleep(200);
  }
  // staged data was written with generic-proxy stores; TMA reads it through the async proxy
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}
#endif

}  // namespace ua
