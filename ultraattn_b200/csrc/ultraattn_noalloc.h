/* Allocation-free entry point of libultraattn_sm100.so.
 *
 * This function has no counterpart in the reference framework; it exists for users of this
 * library whose code is not allowed to allocate device memory at the point where attention's
 * backward has to run: work recorded inside a CUDA-graph capture or a latency-critical serving
 * loop (an allocation there is illegal or stalls the device), a plug-in hosted by another
 * program whose memory pool it must not touch, or a job that has already given every free byte of
 * HBM to its own allocator, so that cudaMalloc can only fail.
 *
 * What it computes: dQ, dK, dV of dense attention (full or causal) for one sequence,
 *     q, d_o, dq : [tokens, n_heads,    128] bf16, contiguous
 *     k, v, dk, dv: [tokens, n_kv_heads, 128] bf16, contiguous
 *     lse, dvec  : [n_heads, tokens] fp32  (the forward's log-sum-exp and D = rowsum(dO * O))
 * exactly like ua_attn_bwd() with one key/value block and one query segment, followed by the
 * fp32 -> bf16 conversion of dQ.
 *
 * Where its scratch lives: the fp32 dQ accumulator and the launch tables sit in a fixed device
 * array inside the library (64 MiB + 4.5 KiB, held by every GPU that loads the library until the
 * process ends). Hence the limits  tokens <= 65536  and  tokens * n_heads <= 131072;  larger
 * problems are rejected with a non-zero return code and a message from ua_last_error().
 * The call itself performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *
 * Rules for callers:
 *   - The first call on each device resolves the array's device address (a one-time host-side
 *     set-up for that device). Make that first call outside of any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left
 *     in it. The function clears what has to start at zero on `stream` before it launches, but
 *     two calls whose GPU work overlaps in time (different streams, or two host threads) race
 *     on the array: serialise them.
 *   - `status` may be NULL; otherwise it points to 4 device ints that receive an error record if a
 *     bounded wait inside the kernel runs out.
 *
 * Returns 0 on success, -1 on error.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int ua_attn_bwd_dense_noalloc(const void* q, const void* k, const void* v, const void* d_o,
                              const float* lse, const float* dvec, void* dq, void* dk, void* dv,
                              int tokens, int n_heads, int n_kv_heads, int causal,
                              float softmax_scale, int* status, cudaStream_t stream);

const char* ua_last_error(void);

#ifdef __cplusplus
}
#endif
