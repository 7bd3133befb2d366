// Memory-bound kernels of the attention runtime and of the Llama-style model around it:
//   * k-way online-softmax merge of partial (O, lse) pairs (reference: the PyTorch-eager
//     update_out_and_lse, ring_flash_attn/utils.py:38-99, and the Triton _rescale_kernel,
//     easy_context/dist_flash_attn/lightseq_async_attn.py:32-108),
//   * D = rowsum(dO * O), the "softmax_d" input of the backward
//     (orchestrated_attn/utils.py:148-188 carries it inside Input_Row_Bwd),
//   * fp32 -> bf16 conversion of gradient accumulators,
//   * RMSNorm, rotary embedding, SwiGLU (forward and backward), the token cross-entropy over bf16
//     logits (forward: log-sum-exp and loss per token; backward: softmax minus one-hot, in place)
//     and a fused Adam step.
// All of them are one pass over HBM with 16-byte accesses.
#include "host_common.cuh"
#include "ptx.cuh"

namespace ua {

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------------------
// k-way merge. One warp per (token, head): D = 128 bf16 = 256 B = 32 lanes x 8 B... we use
// 16 lanes x 16 B per row, two rows per warp.
// dst (O, lse) = merge(srcs[0..k)); dst may alias srcs[0].
// O layout [tokens, heads, 128] with row stride (elements) per source; lse layout [heads, tokens]
// with head stride per source.
// ---------------------------------------------------------------------------------------------
constexpr int MERGE_MAX = 9;
struct MergeParams {
  const __nv_bfloat16* o_src[MERGE_MAX];
  const float* lse_src[MERGE_MAX];
  long o_stride[MERGE_MAX];
  long lse_hstride[MERGE_MAX];
  __nv_bfloat16* o_dst;
  float* lse_dst;
  long o_dst_stride;
  long lse_dst_hstride;
  int k;
  int tokens;
  int heads;
};

// Block = one token x 16 heads x 16 lanes (16 bytes of the 256-byte head row each); K sources.
template <int K>
__global__ void __launch_bounds__(256) lse_merge_kernel(const __grid_constant__ MergeParams p) {
  const int sub = threadIdx.x & 15;                       // 16-byte chunk inside the 256 B row
  const int tok = blockIdx.x;
  const int head = blockIdx.y * 16 + (threadIdx.x >> 4);
  if (head >= p.heads) return;
  float lses[K];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < K; ++i) {
    lses[i] = p.lse_src[i][head * p.lse_hstride[i] + tok];
    mx = fmaxf(mx, lses[i]);
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float tot = 0.f;
  if (mx > -INFINITY) {
#pragma unroll
    for (int i = 0; i < K; ++i) {
      const float w = __expf(lses[i] - mx);
      tot += w;
      if (w != 0.f) {
        const uint4 v = *reinterpret_cast<const uint4*>(
            p.o_src[i] + static_cast<long>(tok) * p.o_stride[i] + head * 128 + sub * 8);
        const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] += w * bf_lo(ws[q]);
          acc[2 * q + 1] += w * bf_hi(ws[q]);
        }
      }
    }
  }
  const float inv = tot > 0.f ? 1.f / tot : 0.f;
  uint4 o;
  o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  o.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
  o.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(p.o_dst + static_cast<long>(tok) * p.o_dst_stride + head * 128 +
                            sub * 8) = o;
  if (sub == 0)
    p.lse_dst[head * p.lse_dst_hstride + tok] = tot > 0.f ? mx + __logf(tot) : -INFINITY;
}

// ---------------------------------------------------------------------------------------------
// D[head, tok] = sum_d dO[tok, head, d] * O[tok, head, d]   (16 lanes per row)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rowdot_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
              float* __restrict__ out, long o_stride, long do_stride, long out_hstride, int tokens,
              int heads) {
  const int sub = threadIdx.x & 15;
  const long rid = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  float acc = 0.f;
  int tok = 0, head = 0;
  const bool valid = rid < static_cast<long>(tokens) * heads;
  if (valid) {
    tok = static_cast<int>(rid / heads);
    head = static_cast<int>(rid % heads);
    const uint4 a = *reinterpret_cast<const uint4*>(o + static_cast<long>(tok) * o_stride +
                                                    head * 128 + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(d_o + static_cast<long>(tok) * do_stride +
                                                    head * 128 + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) acc += bf_lo(aw[q]) * bf_lo(bw[q]) + bf_hi(aw[q]) * bf_hi(bw[q]);
  }
#pragma unroll
  for (int o2 = 8; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o2);
  if (valid && sub == 0) out[head * out_hstride + tok] = acc;
}

// ---------------------------------------------------------------------------------------------
// dst(bf16) = scale * src(fp32)   (optionally dst += )
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
cast_scale_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long n,
                  float scale, int accumulate) {
  const long i = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    const float4 a = *reinterpret_cast<const float4*>(src + i);
    const float4 b = *reinterpret_cast<const float4*>(src + i + 4);
    float f[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                  b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    if (accumulate) {
      const uint4 old = *reinterpret_cast<const uint4*>(dst + i);
      const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) { f[2 * q] += bf_lo(ow[q]); f[2 * q + 1] += bf_hi(ow[q]); }
    }
    uint4 o;
    o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
    o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(dst + i) = o;
  } else {
    for (long j = i; j < n; ++j) {
      float f = src[j] * scale;
      if (accumulate) f += __bfloat162float(dst[j]);
      dst[j] = __float2bfloat16(f);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w. One warp per row; row length H % 256 == 0.
// rstd is saved for the backward.
// Residual fusion: with `res` the kernels normalise xsum = x + res (rounded to bf16, which is what
// the next layer sees) and also store xsum; in the backward `dres` (the gradient that reaches
// xsum through the residual branch) is added to dx, so the two element-wise additions around a
// norm in a transformer block cost no passes of their own.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 add_bf16x8(const uint4& a, const uint4& b) {
  const uint32_t as[4] = {a.x, a.y, a.z, a.w};
  const uint32_t bs[4] = {b.x, b.y, b.z, b.w};
  uint32_t o[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) o[q] = pack_bf16x2(bf_lo(as[q]) + bf_lo(bs[q]), bf_hi(as[q]) + bf_hi(bs[q]));
  return make_uint4(o[0], o[1], o[2], o[3]);
}
template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int H,
                   float eps, const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ xsum) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const __nv_bfloat16* xr = x + static_cast<long>(warp) * H;
  const int nv = H / 256;  // 16-byte vectors per lane
  uint4 v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if (i < nv) {
      v[i] = *reinterpret_cast<const uint4*>(xr + (i * 32 + lane) * 8);
      if (res != nullptr) {
        const long off = static_cast<long>(warp) * H + (i * 32 + lane) * 8;
        v[i] = add_bf16x8(v[i], *reinterpret_cast<const uint4*>(res + off));
        *reinterpret_cast<uint4*>(xsum + off) = v[i];
      }
      const uint32_t ws[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) ss += bf_lo(ws[q]) * bf_lo(ws[q]) + bf_hi(ws[q]) * bf_hi(ws[q]);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / H + eps);
  if (lane == 0 && rstd != nullptr) rstd[warp] = r;
  __nv_bfloat16* yr = y + static_cast<long>(warp) * H;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    if (i < nv) {
      const uint4 wv = *reinterpret_cast<const uint4*>(w + (i * 32 + lane) * 8);
      const uint32_t xs[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        o[q] = pack_bf16x2(bf_lo(xs[q]) * r * bf_lo(ws[q]), bf_hi(xs[q]) * r * bf_hi(ws[q]));
      *reinterpret_cast<uint4*>(yr + (i * 32 + lane) * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Same block organisation as the fused backward below for H a multiple of 2048: eight warps own one
// column slice each of R rows at a time, the row-wide sum of squares goes through shared memory.
template <int NCH, int R>
__global__ void __launch_bounds__(256, 2)
rmsnorm_fwd_sliced_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int H,
                          float eps, const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ xsum) {
  __shared__ float part[2][R][8];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int col0 = warp * (H / 8) + lane * 8;
  uint4 wv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) wv[j] = *reinterpret_cast<const uint4*>(w + col0 + j * 256);
  int buf = 0;
  for (int r0 = blockIdx.x * R; r0 < rows; r0 += static_cast<int>(gridDim.x) * R, buf ^= 1) {
    uint4 xv[R][NCH];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = min(r0 + r, rows - 1);
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const long off = static_cast<long>(row) * H + col0 + j * 256;
        xv[r][j] = *reinterpret_cast<const uint4*>(x + off);
        if (res != nullptr) {
          xv[r][j] = add_bf16x8(xv[r][j], *reinterpret_cast<const uint4*>(res + off));
          if (r0 + r < rows) *reinterpret_cast<uint4*>(xsum + off) = xv[r][j];
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const uint32_t xs[4] = {xv[r][j].x, xv[r][j].y, xv[r][j].z, xv[r][j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) ss += bf_lo(xs[q]) * bf_lo(xs[q]) + bf_hi(xs[q]) * bf_hi(xs[q]);
      }
      ss = warp_sum(ss);
      if (lane == 0) part[buf][r][warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += part[buf][r][k];
      const float rr = rsqrtf(ss / H + eps);
      const bool live = r0 + r < rows;
      if (live && threadIdx.x == 0 && rstd != nullptr) rstd[r0 + r] = rr;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const uint32_t xs[4] = {xv[r][j].x, xv[r][j].y, xv[r][j].z, xv[r][j].w};
        const uint32_t ws[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          o[q] = pack_bf16x2(bf_lo(xs[q]) * rr * bf_lo(ws[q]), bf_hi(xs[q]) * rr * bf_hi(ws[q]));
        if (live)
          *reinterpret_cast<uint4*>(y + static_cast<long>(r0 + r) * H + col0 + j * 256) =
              make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// dx = rstd * (g*w - x * rstd^2 * mean(g*w*x)). One warp per row, two passes over the row (the
// second one hits L1/L2) so that nothing but the running dot product is kept in registers.
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                      const __nv_bfloat16* __restrict__ g, const float* __restrict__ rstd,
                      __nv_bfloat16* __restrict__ dx, int rows, int H,
                      const __nv_bfloat16* __restrict__ dres) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float r = rstd[row];
  const __nv_bfloat16* xr = x + static_cast<long>(row) * H;
  const __nv_bfloat16* gr = g + static_cast<long>(row) * H;
  float dot = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    const uint4 xv = *reinterpret_cast<const uint4*>(xr + c);
    const uint4 gv = *reinterpret_cast<const uint4*>(gr + c);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + c);
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
    const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q)
      dot += bf_lo(gs[q]) * bf_lo(ws[q]) * bf_lo(xs[q]) + bf_hi(gs[q]) * bf_hi(ws[q]) * bf_hi(xs[q]);
  }
  dot = warp_sum(dot);
  const float cc = dot * r * r / H;
  __nv_bfloat16* dxr = dx + static_cast<long>(row) * H;
  for (int c = lane * 8; c < H; c += 256) {
    const uint4 xv = *reinterpret_cast<const uint4*>(xr + c);
    const uint4 gv = *reinterpret_cast<const uint4*>(gr + c);
    const uint4 wv = *reinterpret_cast<const uint4*>(w + c);
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
    const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
    const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
    uint4 dr = make_uint4(0u, 0u, 0u, 0u);
    if (dres != nullptr) dr = *reinterpret_cast<const uint4*>(dres + static_cast<long>(row) * H + c);
    const uint32_t ds[4] = {dr.x, dr.y, dr.z, dr.w};
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q)
      o[q] = pack_bf16x2(r * (bf_lo(gs[q]) * bf_lo(ws[q]) - bf_lo(xs[q]) * cc) + bf_lo(ds[q]),
                         r * (bf_hi(gs[q]) * bf_hi(ws[q]) - bf_hi(xs[q]) * cc) + bf_hi(ds[q]));
    *reinterpret_cast<uint4*>(dxr + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// dw[col] += sum over a slice of rows of g * x * rstd. Thread = 8 columns x one row slice.
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                      const float* __restrict__ rstd, float* __restrict__ dw, int rows, int H,
                      int rows_per_slice) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  const int r0 = blockIdx.y * rows_per_slice;
  const int r1 = min(rows, r0 + rows_per_slice);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  auto add_row = [&](const uint4& xv, const uint4& gv, float r) {
    const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
    const uint32_t gs[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc[2 * q] += bf_lo(gs[q]) * bf_lo(xs[q]) * r;
      acc[2 * q + 1] += bf_hi(gs[q]) * bf_hi(xs[q]) * r;
    }
  };
  int row = r0;
  for (; row + 4 <= r1; row += 4) {          // four rows (eight 16-byte loads) in flight per thread
    uint4 xv[4], gv[4];
    float rr[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      xv[u] = *reinterpret_cast<const uint4*>(x + static_cast<long>(row + u) * H + c);
      gv[u] = *reinterpret_cast<const uint4*>(g + static_cast<long>(row + u) * H + c);
      rr[u] = rstd[row + u];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) add_row(xv[u], gv[u], rr[u]);
  }
  for (; row < r1; ++row)
    add_row(*reinterpret_cast<const uint4*>(x + static_cast<long>(row) * H + c),
            *reinterpret_cast<const uint4*>(g + static_cast<long>(row) * H + c), rstd[row]);
#pragma unroll
  for (int q = 0; q < 8; ++q) atomicAdd(dw + c + q, acc[q]);
}

// Fused form of the two kernels above for H a multiple of 2048: x and g are read once. A block of
// eight warps walks groups of R rows; warp w owns the column slice [w H/8, (w+1) H/8) of every
// row, so its dw partial sums stay in registers for the whole walk (one atomicAdd per column and
// block at the end). The row-wide dot product that dx needs is assembled through shared memory.
template <int NCH, int R>     // NCH: 16-byte chunks per lane and row (H / 2048); R: rows per group
__global__ void __launch_bounds__(256, 2)
rmsnorm_bwd_fused_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         const __nv_bfloat16* __restrict__ g, const float* __restrict__ rstd,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int rows, int H,
                         const __nv_bfloat16* __restrict__ dres) {
  __shared__ float part[2][R][8];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int col0 = warp * (H / 8) + lane * 8;       // chunk j sits at col0 + j * 256
  uint4 wv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) wv[j] = *reinterpret_cast<const uint4*>(w + col0 + j * 256);
  float acc[NCH][8];
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[j][q] = 0.f;
  int buf = 0;
  for (int r0 = blockIdx.x * R; r0 < rows; r0 += static_cast<int>(gridDim.x) * R, buf ^= 1) {
    uint4 xv[R][NCH], gv[R][NCH];
    float rs[R], dot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = min(r0 + r, rows - 1);          // rows past the end repeat the last one
      rs[r] = rstd[row];
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        xv[r][j] = *reinterpret_cast<const uint4*>(x + static_cast<long>(row) * H + col0 + j * 256);
        gv[r][j] = *reinterpret_cast<const uint4*>(g + static_cast<long>(row) * H + col0 + j * 256);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d = 0.f;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const uint32_t xs[4] = {xv[r][j].x, xv[r][j].y, xv[r][j].z, xv[r][j].w};
        const uint32_t gs[4] = {gv[r][j].x, gv[r][j].y, gv[r][j].z, gv[r][j].w};
        const uint32_t ws[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
          d += bf_lo(gs[q]) * bf_lo(ws[q]) * bf_lo(xs[q]) + bf_hi(gs[q]) * bf_hi(ws[q]) * bf_hi(xs[q]);
      }
      d = warp_sum(d);
      if (lane == 0) part[buf][r][warp] = d;
    }
    __syncthreads();          // the other buffer is free again: its readers passed this barrier
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) d += part[buf][r][k];
      dot[r] = d;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool live = r0 + r < rows;
      const float rr = live ? rs[r] : 0.f;            // a repeated tail row adds nothing to dw
      const float cc = dot[r] * rr * rr / H;
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const uint32_t xs[4] = {xv[r][j].x, xv[r][j].y, xv[r][j].z, xv[r][j].w};
        const uint32_t gs[4] = {gv[r][j].x, gv[r][j].y, gv[r][j].z, gv[r][j].w};
        const uint32_t ws[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
        uint4 dr = make_uint4(0u, 0u, 0u, 0u);
        if (dres != nullptr && live)
          dr = *reinterpret_cast<const uint4*>(dres + static_cast<long>(r0 + r) * H + col0 + j * 256);
        const uint32_t ds[4] = {dr.x, dr.y, dr.z, dr.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float xl = bf_lo(xs[q]), xh = bf_hi(xs[q]), gl = bf_lo(gs[q]), gh = bf_hi(gs[q]);
          o[q] = pack_bf16x2(rr * (gl * bf_lo(ws[q]) - xl * cc) + bf_lo(ds[q]),
                             rr * (gh * bf_hi(ws[q]) - xh * cc) + bf_hi(ds[q]));
          acc[j][2 * q] += gl * xl * rr;
          acc[j][2 * q + 1] += gh * xh * rr;
        }
        if (live)
          *reinterpret_cast<uint4*>(dx + static_cast<long>(r0 + r) * H + col0 + j * 256) =
              make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int q = 0; q < 8; ++q) atomicAdd(dw + col0 + j * 256 + q, acc[j][q]);
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding (rotate-half convention of Llama): for pair (i, i+64) of a 128-wide head,
//   y[i] = x[i] cos - x[i+64] sin ; y[i+64] = x[i+64] cos + x[i] sin.
// cos/sin tables are fp32 [positions, 64]; pos[tok] gives the position of each token (so that a
// context-parallel shard or a remapped block order rotates with its global position).
// The backward is the same kernel with sin negated (`inverse` = 1). In place allowed.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
            const int* __restrict__ pos, long tokens, int heads, long x_tok_stride,
            long y_tok_stride, int inverse) {
  // 8 lanes per (token, head): lane handles 8 low elements and the matching 8 high elements
  const long gid = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long rid = gid >> 3;
  const int sub = static_cast<int>(gid & 7);
  if (rid >= tokens * heads) return;
  const long tok = rid / heads;
  const int head = static_cast<int>(rid % heads);
  const int ps = pos[tok];
  const __nv_bfloat16* xr = x + tok * x_tok_stride + head * 128;
  __nv_bfloat16* yr = y + tok * y_tok_stride + head * 128;
  const uint4 lo = *reinterpret_cast<const uint4*>(xr + sub * 8);
  const uint4 hi = *reinterpret_cast<const uint4*>(xr + 64 + sub * 8);
  const float4 c0 = *reinterpret_cast<const float4*>(cos_t + static_cast<long>(ps) * 64 + sub * 8);
  const float4 c1 = *reinterpret_cast<const float4*>(cos_t + static_cast<long>(ps) * 64 + sub * 8 + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sin_t + static_cast<long>(ps) * 64 + sub * 8);
  const float4 s1 = *reinterpret_cast<const float4*>(sin_t + static_cast<long>(ps) * 64 + sub * 8 + 4);
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  if (inverse) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sn[i] = -sn[i];
  }
  const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w};
  const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
  uint32_t ol[4], oh[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float a0 = bf_lo(lw[q]), a1 = bf_hi(lw[q]);
    const float b0 = bf_lo(hw[q]), b1 = bf_hi(hw[q]);
    ol[q] = pack_bf16x2(a0 * cs[2 * q] - b0 * sn[2 * q], a1 * cs[2 * q + 1] - b1 * sn[2 * q + 1]);
    oh[q] = pack_bf16x2(b0 * cs[2 * q] + a0 * sn[2 * q], b1 * cs[2 * q + 1] + a1 * sn[2 * q + 1]);
  }
  *reinterpret_cast<uint4*>(yr + sub * 8) = make_uint4(ol[0], ol[1], ol[2], ol[3]);
  *reinterpret_cast<uint4*>(yr + 64 + sub * 8) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
}

// ---------------------------------------------------------------------------------------------
// SwiGLU on a fused [rows, 2F] gate|up projection: y = silu(gate) * up.
// backward: dgate = dy * up * sig * (1 + gate * (1 - sig)); dup = dy * silu(gate)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, long rows,
                  int F) {
  const long gid = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (gid >= rows * F) return;
  const long r = gid / F;
  const int c = static_cast<int>(gid % F);
  const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
  const uint32_t gs[4] = {g.x, g.y, g.z, g.w};
  const uint32_t us[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float g0 = bf_lo(gs[q]), g1 = bf_hi(gs[q]);
    const float s0 = g0 / (1.f + __expf(-g0)), s1 = g1 / (1.f + __expf(-g1));
    o[q] = pack_bf16x2(s0 * bf_lo(us[q]), s1 * bf_hi(us[q]));
  }
  *reinterpret_cast<uint4*>(y + r * F + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dy,
                  __nv_bfloat16* __restrict__ dgu, long rows, int F) {
  const long gid = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (gid >= rows * F) return;
  const long r = gid / F;
  const int c = static_cast<int>(gid % F);
  const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
  const uint4 d = *reinterpret_cast<const uint4*>(dy + r * F + c);
  const uint32_t gs[4] = {g.x, g.y, g.z, g.w};
  const uint32_t us[4] = {u.x, u.y, u.z, u.w};
  const uint32_t ds[4] = {d.x, d.y, d.z, d.w};
  uint32_t og[4], ou[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float gg[2] = {bf_lo(gs[q]), bf_hi(gs[q])};
    float uu[2] = {bf_lo(us[q]), bf_hi(us[q])};
    float dd[2] = {bf_lo(ds[q]), bf_hi(ds[q])};
    float rg[2], ru[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float sig = 1.f / (1.f + __expf(-gg[h]));
      rg[h] = dd[h] * uu[h] * sig * (1.f + gg[h] * (1.f - sig));
      ru[h] = dd[h] * gg[h] * sig;
    }
    og[q] = pack_bf16x2(rg[0], rg[1]);
    ou[q] = pack_bf16x2(ru[0], ru[1]);
  }
  *reinterpret_cast<uint4*>(dgu + r * 2 * F + c) = make_uint4(og[0], og[1], og[2], og[3]);
  *reinterpret_cast<uint4*>(dgu + r * 2 * F + F + c) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
}

// ---------------------------------------------------------------------------------------------
// Adam / AdamW on an fp32 master copy with bf16 gradients; writes the bf16 working weights.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
            const __nv_bfloat16* __restrict__ grad, __nv_bfloat16* __restrict__ param, long n,
            float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
            float grad_scale) {
  const long i = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 4 <= n) {
    float4 w4 = *reinterpret_cast<float4*>(master + i);
    float4 m4 = *reinterpret_cast<float4*>(m + i);
    float4 v4 = *reinterpret_cast<float4*>(v + i);
    const uint2 g2 = *reinterpret_cast<const uint2*>(grad + i);
    float g[4] = {bf_lo(g2.x) * grad_scale, bf_hi(g2.x) * grad_scale, bf_lo(g2.y) * grad_scale,
                  bf_hi(g2.y) * grad_scale};
    float* wp = reinterpret_cast<float*>(&w4);
    float* mp = reinterpret_cast<float*>(&m4);
    float* vp = reinterpret_cast<float*>(&v4);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      mp[q] = beta1 * mp[q] + (1.f - beta1) * g[q];
      vp[q] = beta2 * vp[q] + (1.f - beta2) * g[q] * g[q];
      const float upd = (mp[q] / bc1) / (sqrtf(vp[q] / bc2) + eps);
      wp[q] = wp[q] - lr * (upd + wd * wp[q]);
    }
    *reinterpret_cast<float4*>(master + i) = w4;
    *reinterpret_cast<float4*>(m + i) = m4;
    *reinterpret_cast<float4*>(v + i) = v4;
    uint2 o;
    o.x = pack_bf16x2(wp[0], wp[1]);
    o.y = pack_bf16x2(wp[2], wp[3]);
    *reinterpret_cast<uint2*>(param + i) = o;
  } else {
    for (long j = i; j < n; ++j) {
      const float gg = __bfloat162float(grad[j]) * grad_scale;
      m[j] = beta1 * m[j] + (1.f - beta1) * gg;
      v[j] = beta2 * v[j] + (1.f - beta2) * gg * gg;
      const float upd = (m[j] / bc1) / (sqrtf(v[j] / bc2) + eps);
      master[j] = master[j] - lr * (upd + wd * master[j]);
      param[j] = __float2bfloat16(master[j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Token cross-entropy over bf16 logits [T, V] (V a multiple of 8, rows 16-byte aligned). One block
// per token. Forward: lse[t] = log sum_v exp(logit[t, v]) by an online (max, sum) pass with 16-byte
// loads, loss[t] = lse[t] - logit[t, target[t]]. Backward, in place over the logits:
// d[t, v] = g * (exp(logit[t, v] - lse[t]) - [v == target[t]]), rounded to bf16. The logits are
// read once per pass and never exist in fp32 in memory.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
xent_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                float* __restrict__ lse, float* __restrict__ loss, long ld, int V) {
  const long t = blockIdx.x;
  const uint4* row = reinterpret_cast<const uint4*>(logits + t * ld);
  float m = -INFINITY, sum = 0.f;
  for (int i = threadIdx.x; i < V / 8; i += blockDim.x) {
    const uint4 q = row[i];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    float x[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) { x[2 * k] = bf_lo(w[k]); x[2 * k + 1] = bf_hi(w[k]); }
    float mx = x[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) mx = fmaxf(mx, x[k]);
    if (mx == -INFINITY) continue;                       // eight masked-out entries add nothing
    if (mx > m) { sum *= __expf(m - mx); m = mx; }
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += __expf(x[k] - m);
  }
  // combine the (max, sum) pairs: inside a warp by shuffles, across warps through shared memory
  __shared__ float sm[8], ss[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xFFFFFFFFu, m, o);
    const float s2 = __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    const float mn = fmaxf(m, m2);
    sum = (mn == -INFINITY) ? 0.f : sum * __expf(m - mn) + s2 * __expf(m2 - mn);
    m = mn;
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; ss[threadIdx.x >> 5] = sum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float mt = sm[0], st = ss[0];
    for (int wv = 1; wv < static_cast<int>(blockDim.x >> 5); ++wv) {
      const float mn = fmaxf(mt, sm[wv]);
      st = (mn == -INFINITY) ? 0.f : st * __expf(mt - mn) + ss[wv] * __expf(sm[wv] - mn);
      mt = mn;
    }
    const float l = mt + __logf(st);
    lse[t] = l;
    const int tg = targets[t];
    loss[t] = (tg >= 0 && tg < V) ? l - __bfloat162float(logits[t * ld + tg]) : 0.f;   // ignored target: no loss
  }
}

__global__ void __launch_bounds__(256)
xent_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                const float* __restrict__ lse, const float* __restrict__ g, long ld, int V) {
  const long t = blockIdx.x;
  uint4* row = reinterpret_cast<uint4*>(logits + t * ld);
  const float l = lse[t];
  const int tg = targets[t];
  const float scale = (tg >= 0 && tg < V) ? *g : 0.f;
  for (int i = threadIdx.x; i < V / 8; i += blockDim.x) {
    const uint4 q = row[i];
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float a = __expf(bf_lo(w[k]) - l), b = __expf(bf_hi(w[k]) - l);
      if (i * 8 + 2 * k == tg) a -= 1.f;
      if (i * 8 + 2 * k + 1 == tg) b -= 1.f;
      o[k] = pack_bf16x2(a * scale, b * scale);
    }
    row[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace ua

using namespace ua;

extern "C" int ua_lse_merge(const void* const* o_srcs, const float* const* lse_srcs,
                            const long* o_strides, const long* lse_hstrides, int k, void* o_dst,
                            float* lse_dst, long o_dst_stride, long lse_dst_hstride, int tokens,
                            int heads, cudaStream_t stream) {
  if (k < 1 || k > MERGE_MAX) UA_FAIL("ua_lse_merge: k must be in [1, %d]", MERGE_MAX);
  MergeParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < k; ++i) {
    p.o_src[i] = static_cast<const __nv_bfloat16*>(o_srcs[i]);
    p.lse_src[i] = lse_srcs[i];
    p.o_stride[i] = o_strides[i];
    p.lse_hstride[i] = lse_hstrides[i];
  }
  p.o_dst = static_cast<__nv_bfloat16*>(o_dst);
  p.lse_dst = lse_dst;
  p.o_dst_stride = o_dst_stride;
  p.lse_dst_hstride = lse_dst_hstride;
  p.k = k; p.tokens = tokens; p.heads = heads;
  if (tokens == 0 || heads == 0) return 0;
  const dim3 grid(static_cast<unsigned>(tokens), static_cast<unsigned>((heads + 15) / 16), 1);
  switch (k) {
#define UA_MERGE_CASE(K) case K: lse_merge_kernel<K><<<grid, 256, 0, stream>>>(p); break;
    UA_MERGE_CASE(1) UA_MERGE_CASE(2) UA_MERGE_CASE(3) UA_MERGE_CASE(4) UA_MERGE_CASE(5)
    UA_MERGE_CASE(6) UA_MERGE_CASE(7) UA_MERGE_CASE(8) UA_MERGE_CASE(9)
#undef UA_MERGE_CASE
    default: UA_FAIL("ua_lse_merge: k must be in [1, 9]");
  }
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_rowdot(const void* o, const void* d_o, float* out, long o_stride, long do_stride,
                         long out_hstride, int tokens, int heads, cudaStream_t stream) {
  const long threads = static_cast<long>(tokens) * heads * 16;
  if (threads == 0) return 0;
  rowdot_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), out, o_stride,
      do_stride, out_hstride, tokens, heads);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_cast_scale(const float* src, void* dst, long n, float scale, int accumulate,
                             cudaStream_t stream) {
  if (n == 0) return 0;
  const long threads = (n + 7) / 8;
  cast_scale_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      src, static_cast<__nv_bfloat16*>(dst), n, scale, accumulate);
  UA_CUDA(cudaGetLastError());
  return 0;
}

static int rmsnorm_fwd_launch(const void* x, const void* res, const void* w, void* xsum, void* y, float* rstd,
                              int rows, int H, float eps, cudaStream_t stream) {
  if (H % 256 != 0 || H > 8192) UA_FAIL("ua_rmsnorm_fwd: H must be a multiple of 256, <= 8192");
  if (rows == 0) return 0;
  const unsigned blocks = (static_cast<long>(rows) * 32 + 255) / 256;
  auto xx = static_cast<const __nv_bfloat16*>(x);
  auto ww = static_cast<const __nv_bfloat16*>(w);
  auto yy = static_cast<__nv_bfloat16*>(y);
  auto rr = static_cast<const __nv_bfloat16*>(res);
  auto xs = static_cast<__nv_bfloat16*>(xsum);
  if (H % 2048 == 0) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long want = (static_cast<long>(rows) + 3) / 4;
    const unsigned nb = static_cast<unsigned>(want < 8L * sms ? want : 8L * sms);
    switch (H / 2048) {
      case 1: rmsnorm_fwd_sliced_kernel<1, 4><<<nb, 256, 0, stream>>>(xx, ww, yy, rstd, rows, H, eps, rr, xs); break;
      case 2: rmsnorm_fwd_sliced_kernel<2, 4><<<nb, 256, 0, stream>>>(xx, ww, yy, rstd, rows, H, eps, rr, xs); break;
      case 3: rmsnorm_fwd_sliced_kernel<3, 4><<<nb, 256, 0, stream>>>(xx, ww, yy, rstd, rows, H, eps, rr, xs); break;
      default: rmsnorm_fwd_sliced_kernel<4, 4><<<nb, 256, 0, stream>>>(xx, ww, yy, rstd, rows, H, eps, rr, xs); break;
    }
    UA_CUDA(cudaGetLastError());
    return 0;
  }
  if (H <= 4096) rmsnorm_fwd_kernel<16><<<blocks, 256, 0, stream>>>(xx, ww, yy, rstd, rows, H, eps, rr, xs);
  else rmsnorm_fwd_kernel<32><<<blocks, 256, 0, stream>>>(xx, ww, yy, rstd, rows, H, eps, rr, xs);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int H,
                              float eps, cudaStream_t stream) {
  return rmsnorm_fwd_launch(x, nullptr, w, nullptr, y, rstd, rows, H, eps, stream);
}

// xsum = x + res (bf16), y = RMSNorm(xsum) * w, in one pass.
extern "C" int ua_add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* xsum, void* y,
                                  float* rstd, int rows, int H, float eps, cudaStream_t stream) {
  if (res == nullptr || xsum == nullptr) UA_FAIL("ua_add_rmsnorm_fwd: res and xsum are required");
  return rmsnorm_fwd_launch(x, res, w, xsum, y, rstd, rows, H, eps, stream);
}

// dw must be zeroed by the caller (fp32, H entries); it is accumulated into.
static int rmsnorm_bwd_launch(const void* x, const void* w, const void* g, const float* rstd, const void* dres,
                              void* dx, float* dw, int rows, int H, cudaStream_t stream) {
  auto dr = static_cast<const __nv_bfloat16*>(dres);
  if (H % 256 != 0) UA_FAIL("ua_rmsnorm_bwd: H must be a multiple of 256");
  if (rows == 0) return 0;
  if (H % 2048 == 0 && H <= 8192) {
    // fused single-pass kernel: a few persistent blocks per SM, each walking its share of the rows
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int R = H <= 2048 ? 4 : 2;
    long want = (static_cast<long>(rows) + R - 1) / R;
    const unsigned nb = static_cast<unsigned>(want < 6L * sms ? want : 6L * sms);
    auto xx = static_cast<const __nv_bfloat16*>(x);
    auto ww = static_cast<const __nv_bfloat16*>(w);
    auto gg = static_cast<const __nv_bfloat16*>(g);
    auto dd = static_cast<__nv_bfloat16*>(dx);
    switch (H / 2048) {
      case 1: rmsnorm_bwd_fused_kernel<1, 4><<<nb, 256, 0, stream>>>(xx, ww, gg, rstd, dd, dw, rows, H, dr); break;
      case 2: rmsnorm_bwd_fused_kernel<2, 2><<<nb, 256, 0, stream>>>(xx, ww, gg, rstd, dd, dw, rows, H, dr); break;
      case 3: rmsnorm_bwd_fused_kernel<3, 2><<<nb, 256, 0, stream>>>(xx, ww, gg, rstd, dd, dw, rows, H, dr); break;
      default: rmsnorm_bwd_fused_kernel<4, 2><<<nb, 256, 0, stream>>>(xx, ww, gg, rstd, dd, dw, rows, H, dr); break;
    }
    UA_CUDA(cudaGetLastError());
    return 0;
  }
  const unsigned blocks = (static_cast<long>(rows) * 32 + 255) / 256;
  rmsnorm_bwd_dx_kernel<<<blocks, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(g), rstd, static_cast<__nv_bfloat16*>(dx), rows, H, dr);
  UA_CUDA(cudaGetLastError());
  const int rows_per_slice = 64;
  dim3 grid((H / 8 + 255) / 256, (rows + rows_per_slice - 1) / rows_per_slice);
  rmsnorm_bwd_dw_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                  static_cast<const __nv_bfloat16*>(g), rstd, dw,
                                                  rows, H, rows_per_slice);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_rmsnorm_bwd(const void* x, const void* w, const void* g, const float* rstd,
                              void* dx, float* dw, int rows, int H, cudaStream_t stream) {
  return rmsnorm_bwd_launch(x, w, g, rstd, nullptr, dx, dw, rows, H, stream);
}

// dx = d RMSNorm / dx (g) + dres: the gradient of xsum when xsum also feeds a residual branch.
extern "C" int ua_rmsnorm_bwd_res(const void* x, const void* w, const void* g, const float* rstd,
                                  const void* dres, void* dx, float* dw, int rows, int H,
                                  cudaStream_t stream) {
  return rmsnorm_bwd_launch(x, w, g, rstd, dres, dx, dw, rows, H, stream);
}

extern "C" int ua_rope(const void* x, void* y, const float* cos_t, const float* sin_t,
                       const int* pos, long tokens, int heads, long x_tok_stride,
                       long y_tok_stride, int inverse, cudaStream_t stream) {
  const long threads = tokens * heads * 8;
  if (threads == 0) return 0;
  rope_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), cos_t, sin_t, pos,
      tokens, heads, x_tok_stride, y_tok_stride, inverse);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_swiglu_fwd(const void* gu, void* y, long rows, int F, cudaStream_t stream) {
  if (F % 8 != 0) UA_FAIL("ua_swiglu_fwd: F must be a multiple of 8");
  const long threads = rows * F / 8;
  if (threads == 0) return 0;
  swiglu_fwd_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(y), rows, F);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_swiglu_bwd(const void* gu, const void* dy, void* dgu, long rows, int F,
                             cudaStream_t stream) {
  if (F % 8 != 0) UA_FAIL("ua_swiglu_bwd: F must be a multiple of 8");
  const long threads = rows * F / 8;
  if (threads == 0) return 0;
  swiglu_bwd_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(dgu), rows, F);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_adam(float* master, float* m, float* v, const void* grad, void* param, long n,
                       float lr, float beta1, float beta2, float eps, float wd, int step,
                       float grad_scale, cudaStream_t stream) {
  if (n == 0) return 0;
  const float bc1 = 1.f - powf(beta1, static_cast<float>(step));
  const float bc2 = 1.f - powf(beta2, static_cast<float>(step));
  const long threads = (n + 3) / 4;
  adam_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
      master, m, v, static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(param), n,
      lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int ua_xent_fwd(const void* logits, const int* targets, float* lse, float* loss, long tokens,
                           long ld, int V, cudaStream_t stream) {
  if (V % 8 != 0 || ld % 8 != 0) UA_FAIL("ua_xent_fwd: vocabulary and row stride must be multiples of 8");
  if (tokens == 0) return 0;
  xent_fwd_kernel<<<static_cast<unsigned>(tokens), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(logits), targets, lse, loss, ld, V);
  UA_CUDA(cudaGetLastError());
  return 0;
}

// In place: logits become g * (softmax - one-hot); g is a device scalar (the incoming gradient).
extern "C" int ua_xent_bwd(void* logits, const int* targets, const float* lse, const float* g, long tokens,
                           long ld, int V, cudaStream_t stream) {
  if (V % 8 != 0 || ld % 8 != 0) UA_FAIL("ua_xent_bwd: vocabulary and row stride must be multiples of 8");
  if (tokens == 0) return 0;
  xent_bwd_kernel<<<static_cast<unsigned>(tokens), 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(logits), targets, lse, g, ld, V);
  UA_CUDA(cudaGetLastError());
  return 0;
}

extern "C" const char* ua_last_error() { return ua::err_buf(); }
