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
  int n_copy_ctas;         // the first n_copy_ctas CTAs (linear id) help with the copies even if they wait for nothing
  unsigned int* flags;     // monotonically increasing counters, never reset
  int epoch;               // call number (1, 2, ...): a block is ready at wait_count * epoch
  unsigned int* ticket;    // next unclaimed copy task of this launch (zeroed by the host before the launch)
};

// Optional per-CTA time stamps of a launch, available in the normal build (set through
// ua_set_kernel_trace): CTA i of the grid writes four 64-bit words at buf[4 * i]: globaltimer at
// its start, after its share of the staging copies, at its end, and (SM id << 32 | work item).
// The fused kernels do their transfers themselves, so a timeline shows them as one launch; these
// stamps keep staging, compute and idle tails attributable.
struct KernelTrace {
  unsigned long long* buf;
  int cap;                 // CTAs that fit
};

#ifdef __CUDACC__
__device__ __forceinline__ void trace_stamp(const KernelTrace& kt, int cta_linear, int slot) {
  if (kt.buf != nullptr && cta_linear < kt.cap && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    kt.buf[4 * static_cast<long>(cta_linear) + slot] = t;
  }
}
__device__ __forceinline__ void trace_ident(const KernelTrace& kt, int cta_linear, int item) {
  if (kt.buf != nullptr && cta_linear < kt.cap && threadIdx.x == 0) {
    unsigned int smid;
    asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
    kt.buf[4 * static_cast<long>(cta_linear) + 3] = (static_cast<unsigned long long>(smid) << 32) |
                                                   static_cast<unsigned int>(item);
  }
}
#endif

#ifdef __CUDACC__
// Staging prologue. The copy tasks of a launch form a queue; a CTA takes tasks from it (one atomic
// ticket per task) until the queue is empty. Every CTA that is going to wait for a staged block
// does this BEFORE its first wait (`take_part`), and so do the first n_copy_ctas CTAs of the grid.
// A copy never waits on anything. So whenever a CTA waits, every task has already been claimed
// by a CTA that is running and will finish it: the wait can only be for work that is in progress,
// whatever order the hardware dispatches the CTAs in. `slot`: one int of shared memory.
__device__ __forceinline__ void drain_stage_queue(const StageParams& sp, bool take_part, int cta_linear,
                                                  int* slot) {
  if (sp.n_tasks == 0 || sp.ticket == nullptr) return;
  if (!take_part && cta_linear >= sp.n_copy_ctas) return;      // (uniform over the CTA)
  for (;;) {
    __syncthreads();
    if (threadIdx.x == 0) *slot = static_cast<int>(atomicAdd(sp.ticket, 1u));
    __syncthreads();
    const int t = *slot;
    if (t >= sp.n_tasks) break;
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
