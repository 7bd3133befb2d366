// bf16 GEMM on tcgen05 tensor cores with TMEM accumulators (sm_100a).
//
//   C[M,N] = A[M,K] * B[K,N]      (fp32 accumulate, bf16 out)
//
// A may be stored K-contiguous ([M,K] row-major) or M-contiguous ([K,M] row-major); B may be
// stored K-contiguous ([N,K] row-major, the torch `linear` weight) or N-contiguous ([K,N]
// row-major). That covers y = x W^T, dx = dy W and dW = dy^T x without any transpose copy.
//
// One persistent CTA per SM walks output tiles. Warp 0 feeds a shared-memory ring with TMA, warp 1
// issues tcgen05.mma, the remaining warps drain the accumulator from TMEM. Two tile shapes:
//  * 128 x 256 (MH = 1): 4 stages, two 256-column TMEM accumulators so the epilogue of tile i
//    overlaps the main loop of tile i+1; used when there are few tiles.
//  * 256 x 256 (MH = 2): two M = 128 instructions per k-step share the B tile in shared memory
//    (acc 0 | acc 1 = all 512 TMEM columns, 3 stages, 8 epilogue warps). The shared-memory port
//    bounds this kernel (TMA writes + operand reads), and the taller tile needs 160 B per tensor
//    clock instead of 192; used when the problem has at least four waves of such tiles.
//
// Two optional fusions serve the head-parallel (Ulysses) attention path, where an all-to-all
// normally sits next to a projection GEMM (reference: comm_lib/comm_utils.py:32-45 A2AComm and
// head_parallel_attn/deepspeed_ulysses_attn.py):
//  * scatter epilogue: output columns are split into `n_dst` equal groups and group g is stored
//    to base pointer c_dst[g] (a peer GPU's buffer) at row offset `dst_row_off` — the GEMM
//    writes the all-to-all's result directly;
//  * gather prologue: the K dimension is split into `n_src` equal groups and group g of A is
//    loaded by TMA (unicast) from tensor map tmA[g] (a peer GPU's buffer) at row offset
//    `a_row_off` — the GEMM reads the all-to-all's input directly.
#include "host_common.cuh"
#include "ptx.cuh"

namespace ua {

constexpr int GEMM_BN = 256;
constexpr int GEMM_BK = 64;
constexpr int GEMM_MAX_PEERS = 8;
template <int MH> struct GemmCfg {
  static constexpr int BM = 128 * MH;
  static constexpr int STAGES = MH == 1 ? 4 : 3;
  static constexpr int ACC_BUFS = MH == 1 ? 2 : 1;
  static constexpr int EPI_WARPS = 4 * MH;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
};

struct GemmParams {
  CUtensorMap tmA[GEMM_MAX_PEERS];
  CUtensorMap tmB;
  __nv_bfloat16* c_dst[GEMM_MAX_PEERS];
  int M, N, K;
  int ldc;            // leading dimension of every destination buffer (elements)
  int a_mn_major;     // 1: A stored [K,M] (M contiguous)
  int b_mn_major;     // 1: B stored [K,N] (N contiguous)
  int n_src;          // gather prologue: number of K groups (1 = plain)
  int k_per_src;      // K / n_src
  int a_row_off;      // row offset of A inside every source buffer
  int n_dst;          // scatter epilogue: number of column groups (1 = plain)
  int cols_per_dst;   // N / n_dst
  int dst_row_off;    // row offset inside every destination buffer
  int* status;
};

// Tile order of the persistent kernels: tiles are walked in bands of GEMM_GROUP_M tile rows, down
// the band first, so that the tiles in flight at any moment (one per SM or SM pair) cover a
// compact block of the output: a few row panels of A and a few column panels of B, which then
// stay in L2 between the tiles that share them. With the plain "all tile rows of one tile column"
// order a wave touches 148 different A panels (more than the L2 holds for large M) and every A
// panel is fetched from HBM again for every tile column.
constexpr int GEMM_GROUP_M = 8;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = GEMM_GROUP_M * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * GEMM_GROUP_M;
  const int rows = min(GEMM_GROUP_M, m_tiles - first_m);
  const int in_group = tile - group * per_group;
  mt = first_m + in_group % rows;
  nt = in_group / rows;
}

template <int MH>
struct __align__(1024) GemmSmem {
  uint8_t a[GemmCfg<MH>::STAGES][GemmCfg<MH>::BM * GEMM_BK * 2];   // 16 KB per 128 rows and stage
  uint8_t b[GemmCfg<MH>::STAGES][GEMM_BN * GEMM_BK * 2];           // 32 KB per stage
  uint64_t full[GemmCfg<MH>::STAGES];
  uint64_t empty[GemmCfg<MH>::STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int MH>
__global__ void __launch_bounds__(GemmCfg<MH>::THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ GemmParams p) {
  constexpr int GEMM_STAGES = GemmCfg<MH>::STAGES;
  constexpr int ACC_BUFS = GemmCfg<MH>::ACC_BUFS;
  constexpr int TILE_M = GemmCfg<MH>::BM;
  extern __shared__ uint8_t smem_raw[];
  GemmSmem<MH>& s = *reinterpret_cast<GemmSmem<MH>*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < GEMM_STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 32 * GemmCfg<MH>::EPI_WARPS);
    }
    s.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  WaitCtx wc{&s.abort_flag, p.status, 4000000000ull};

  const int m_tiles = (p.M + TILE_M - 1) / TILE_M;
  const int n_tiles = (p.N + GEMM_BN - 1) / GEMM_BN;
  const int total = m_tiles * n_tiles;
  const int k_blocks = (p.K + GEMM_BK - 1) / GEMM_BK;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (lane == 0) {
      for (int i = 0; i < p.n_src; ++i) tma_prefetch_desc(&p.tmA[i]);
      tma_prefetch_desc(&p.tmB);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, mt, nt);
        const int m0 = mt * TILE_M;
        const int n0 = nt * GEMM_BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % GEMM_STAGES;
          const uint32_t ph = (it / GEMM_STAGES) & 1;
          if (!mbar_wait(&s.empty[st], ph ^ 1, wc, 10)) break;
          mbar_arrive_expect_tx(&s.full[st], (TILE_M + GEMM_BN) * GEMM_BK * 2);
          const int k0 = kb * GEMM_BK;
          const int src = k0 / p.k_per_src;
          const int ksrc = k0 - src * p.k_per_src;
          if (!p.a_mn_major) {
            // one box of TILE_M rows x 64 k (rows of 128 B; the second 128 rows start at +16 KB)
            tma_load_2d(s.a[st], &p.tmA[src], &s.full[st], ksrc, p.a_row_off + m0);
          } else {
            // [K,M] storage: 64-wide M panels of 64 k-rows each, two per 128 rows
            for (int pm = 0; pm < 2 * MH; ++pm)
              tma_load_2d(s.a[st] + pm * 8192, &p.tmA[src], &s.full[st], m0 + pm * 64, p.a_row_off + ksrc);
          }
          if (!p.b_mn_major) {
            tma_load_2d(s.b[st], &p.tmB, &s.full[st], k0, n0);
          } else {
            for (int pn = 0; pn < GEMM_BN / 64; ++pn)
              tma_load_2d(s.b[st] + pn * 8192, &p.tmB, &s.full[st], n0 + pn * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, GEMM_BN, p.a_mn_major, p.b_mn_major);
      // K-major tile: rows of 128 B, 8-row groups 1024 B apart; 16 k-elements = 32 B.
      // MN-major tile: 64-element panels 8192 B apart (LBO), 8 k-rows = 1024 B (SBO);
      //                16 k-rows = 2048 B.
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn_major ? 2048u : 32u;
      uint32_t it = 0;
      uint32_t tcount = 0;
      for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++tcount) {
        const int buf = ACC_BUFS == 2 ? (tcount & 1) : 0;
        const uint32_t aph = ACC_BUFS == 2 ? ((tcount >> 1) & 1) : (tcount & 1);
        if (!mbar_wait(&s.acc_empty[buf], aph ^ 1, wc, 20)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * GEMM_BN;      // MH = 2: halves at columns 0 and 256
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % GEMM_STAGES;
          const uint32_t ph = (it / GEMM_STAGES) & 1;
          if (!mbar_wait(&s.full[st], ph, wc, 21)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.a[st]);
          const uint32_t b_addr = smem_u32(s.b[st]);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
#pragma unroll
            for (int h = 0; h < MH; ++h) {
              const uint64_t ad = make_smem_desc_sw128(a_addr + h * 16384 + k * a_kstep, a_lbo, 1024);
              umma_ss(d_tmem + h * GEMM_BN, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          tc_commit(&s.empty[st]);
        }
        if (!ok) break;
        tc_commit(&s.acc_full[buf]);
      }
    }
  } else {
    // ------------------------------- epilogue (4 warps) -------------------------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;                 // which 128 rows of the tile (MH = 2: warps 6-9 take the second)
    const int row_in_tile = half * 128 + quad * 32 + lane;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++tcount) {
      const int buf = ACC_BUFS == 2 ? (tcount & 1) : 0;
      const uint32_t aph = ACC_BUFS == 2 ? ((tcount >> 1) & 1) : (tcount & 1);
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, mt, nt);
      const int m0 = mt * TILE_M;
      const int n0 = nt * GEMM_BN;
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s.acc_full[buf], aph, wc, 30))) break;
      tc_fence_after_sync();
      const int row = m0 + row_in_tile;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + (buf + half) * GEMM_BN;
#pragma unroll 1
      for (int c = 0; c < GEMM_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_x32(taddr + c * 32, v);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          const int g = col0 / p.cols_per_dst;
          const int cin = col0 - g * p.cols_per_dst;
          __nv_bfloat16* dst = p.c_dst[g] + static_cast<size_t>(p.dst_row_off + row) * p.ldc + cin;
          if (col0 + 32 <= p.N) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
              d4[q] = o;
            }
          } else {
            for (int q = 0; q < 32 && col0 + q < p.N; ++q)
              dst[q] = __float2bfloat16(__uint_as_float(v[q]));
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&s.acc_empty[buf]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair form (cta_group::2): a cluster of two CTAs on two SMs computes one 256 x 256 tile.
// Each CTA loads its own 128 rows of A and its own half (128 of 256) of the B tile; the tensor
// cores of both SMs read both halves, so every B byte is written to shared memory once and read
// by two SMs. That halves the shared-memory traffic per FLOP of the B operand, which is what
// bounds the single-CTA kernel above (TMA writes + operand reads exceed the 128 B/clk port).
// The even CTA (leader) issues the MMAs for the pair and owns the "full" and "accumulator empty"
// barriers; every TMA load of either CTA signals the leader's barrier (plain unicast loads: no
// cluster-multicast load anywhere), tcgen05.commit arrives on the per-stage "empty" barrier and on
// the "accumulator full" barrier of both CTAs.
// ------------------------------------------------------------------------------------------------
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_BM = 256;            // rows per cluster tile (128 per CTA)
constexpr int PAIR_THREADS = 64 + 32 * 4;

struct __align__(1024) PairSmem {
  uint8_t a[PAIR_STAGES][128 * GEMM_BK * 2];   // this CTA's 128 rows: 16 KB per stage
  uint8_t b[PAIR_STAGES][128 * GEMM_BK * 2];   // this CTA's half of the B tile: 16 KB per stage
  uint64_t full[PAIR_STAGES];                  // used in the leader only
  uint64_t empty[PAIR_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];                       // used in the leader only (both CTAs' epilogues arrive)
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  PairSmem& s = *reinterpret_cast<PairSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();        // 0 = leader, 1 = peer
  const bool leader = cta == 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < PAIR_STAGES; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.acc_full[i], 1);
      mbar_init(&s.acc_empty[i], 2 * 4);         // one arrival per epilogue warp of both CTAs
    }
    s.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&s.tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                            // the peer's barriers exist before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  WaitCtx wc{&s.abort_flag, p.status, 4000000000ull};

  const int m_tiles = (p.M + PAIR_BM - 1) / PAIR_BM;
  const int n_tiles = (p.N + GEMM_BN - 1) / GEMM_BN;
  const int total = m_tiles * n_tiles;
  const int k_blocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      for (int i = 0; i < p.n_src; ++i) tma_prefetch_desc(&p.tmA[i]);
      tma_prefetch_desc(&p.tmB);
      uint32_t it = 0;
      for (int tile = cluster_id; tile < total; tile += n_clusters) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, mt, nt);
        const int m0 = mt * PAIR_BM + static_cast<int>(cta) * 128;
        const int n0 = nt * GEMM_BN + static_cast<int>(cta) * 128;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (!mbar_wait(&s.empty[st], ph ^ 1, wc, 40)) { ok = false; break; }
          // the leader announces the bytes of both CTAs; the peer's loads complete on the same barrier
          if (leader) mbar_arrive_expect_tx(&s.full[st], 2 * (128 + 128) * GEMM_BK * 2);
          const uint32_t bar = mapa_shared(smem_u32(&s.full[st]), 0);
          const int k0 = kb * GEMM_BK;
          const int src = k0 / p.k_per_src;
          const int ksrc = k0 - src * p.k_per_src;
          if (!p.a_mn_major) {
            tma_load_2d_pair(s.a[st], &p.tmA[src], bar, ksrc, p.a_row_off + m0);
          } else {
            for (int pm = 0; pm < 2; ++pm)
              tma_load_2d_pair(s.a[st] + pm * 8192, &p.tmA[src], bar, m0 + pm * 64, p.a_row_off + ksrc);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(s.b[st], &p.tmB, bar, k0, n0);
          } else {
            for (int pn = 0; pn < 2; ++pn)
              tma_load_2d_pair(s.b[st] + pn * 8192, &p.tmB, bar, n0 + pn * 64, k0);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_bf16(256, GEMM_BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn_major ? 2048u : 32u;
      uint32_t it = 0;
      uint32_t tcount = 0;
      for (int tile = cluster_id; tile < total; tile += n_clusters, ++tcount) {
        const int buf = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&s.acc_empty[buf], aph ^ 1, wc, 50)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * GEMM_BN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int st = it % PAIR_STAGES;
          const uint32_t ph = (it / PAIR_STAGES) & 1;
          if (!mbar_wait(&s.full[st], ph, wc, 51)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(s.a[st]);
          const uint32_t b_addr = smem_u32(s.b[st]);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
            umma_ss_pair(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is free again in both CTAs once these MMAs have read it
          tc_commit_pair(&s.empty[st], 3);
        }
        if (!ok) break;
        tc_commit_pair(&s.acc_full[buf], 3);
      }
    }
  } else {
    // ------------------------------- epilogue (4 warps per CTA) -----------------------------
    const int quad = warp & 3;
    const int row_in_tile = static_cast<int>(cta) * 128 + quad * 32 + lane;
    uint32_t tcount = 0;
    for (int tile = cluster_id; tile < total; tile += n_clusters, ++tcount) {
      const int buf = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, mt, nt);
      const int m0 = mt * PAIR_BM;
      const int n0 = nt * GEMM_BN;
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s.acc_full[buf], aph, wc, 60))) break;
      tc_fence_after_sync();
      const int row = m0 + row_in_tile;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * GEMM_BN;
#pragma unroll 1
      for (int c = 0; c < GEMM_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_x32(taddr + c * 32, v);
        tmem_wait_ld();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          const int g = col0 / p.cols_per_dst;
          const int cin = col0 - g * p.cols_per_dst;
          __nv_bfloat16* dst = p.c_dst[g] + static_cast<size_t>(p.dst_row_off + row) * p.ldc + cin;
          if (col0 + 32 <= p.N) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
              d4[q] = o;
            }
          } else {
            for (int q = 0; q < 32 && col0 + q < p.N; ++q)
              dst[q] = __float2bfloat16(__uint_as_float(v[q]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&s.acc_empty[buf]), 0));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();      // nobody leaves while the other CTA may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace ua

using namespace ua;

static int g_gemm_smem_set[2][64] = {{0}};

template <int MH>
static int launch_gemm(const GemmParams& p, int grid, cudaStream_t stream) {
  const int smem_bytes = sizeof(GemmSmem<MH>) + 1024;
  int dev = 0;
  UA_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !g_gemm_smem_set[MH - 1][dev]) {
    UA_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<MH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes));
    g_gemm_smem_set[MH - 1][dev] = 1;
  }
  gemm_bf16_kernel<MH><<<grid, GemmCfg<MH>::THREADS, smem_bytes, stream>>>(p);
  UA_CUDA(cudaGetLastError());
  return 0;
}


static int g_pair_smem_set[64] = {0};
static int g_pair_mode = 0;      // 0: single-CTA tiles, 1: CTA pairs (set before a launch by ua_gemm_pair_mode)

// Which form the following ua_gemm_bf16 calls of this process use: 0 = one CTA per tile, 1 = a pair
// of CTAs per 256 x 256 tile. Neither is faster for every shape (measured on Llama-2-7B shapes at
// 64k tokens: pairs win the 12288-wide QKV projection, single CTAs the others).
extern "C" void ua_gemm_pair_mode(int mode) { g_pair_mode = mode; }

static int launch_gemm_pair(const GemmParams& p, int num_sms, cudaStream_t stream) {
  const int smem_bytes = sizeof(PairSmem) + 1024;
  int dev = 0;
  UA_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !g_pair_smem_set[dev]) {
    UA_CUDA(cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    g_pair_smem_set[dev] = 1;
  }
  const int m_tiles = (p.M + PAIR_BM - 1) / PAIR_BM;
  const int n_tiles = (p.N + GEMM_BN - 1) / GEMM_BN;
  int clusters = m_tiles * n_tiles;
  if (clusters > num_sms / 2) clusters = num_sms / 2;
  if (clusters < 1) return 0;
  gemm_bf16_pair_kernel<<<2 * clusters, PAIR_THREADS, smem_bytes, stream>>>(p);
  UA_CUDA(cudaGetLastError());
  return 0;
}

// a_ptrs / c_ptrs: arrays of n_src / n_dst device pointers (host arrays).
// lda / ldb / ldc in elements. Requirements: K % 8 == 0, lda % 8 == 0, ldb % 8 == 0,
// cols_per_dst % 32 == 0 when n_dst > 1, k_per_src % 64 == 0 when n_src > 1.
extern "C" int ua_gemm_bf16(const void* const* a_ptrs, int n_src, long a_rows_total, int lda,
                            int a_row_off, int a_mn_major, const void* b, int ldb, int b_mn_major,
                            void* const* c_ptrs, int n_dst, int ldc, int dst_row_off, int M, int N,
                            int K, int* status, int num_sms, cudaStream_t stream) {
  if (n_src < 1 || n_src > GEMM_MAX_PEERS || n_dst < 1 || n_dst > GEMM_MAX_PEERS)
    UA_FAIL("ua_gemm_bf16: n_src/n_dst out of range");
  if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || ldc % 8 != 0)
    UA_FAIL("ua_gemm_bf16: K, lda, ldb, ldc must be multiples of 8");
  if (K % n_src != 0 || N % n_dst != 0) UA_FAIL("ua_gemm_bf16: K %% n_src or N %% n_dst != 0");
  if (n_src > 1 && (K / n_src) % GEMM_BK != 0) UA_FAIL("ua_gemm_bf16: K/n_src must be a multiple of 64");
  if (n_dst > 1 && (N / n_dst) % 32 != 0) UA_FAIL("ua_gemm_bf16: N/n_dst must be a multiple of 32");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.n_src = n_src; p.k_per_src = K / n_src; p.a_row_off = a_row_off;
  p.n_dst = n_dst; p.cols_per_dst = N / n_dst; p.dst_row_off = dst_row_off;
  p.status = status;
  for (int i = 0; i < n_dst; ++i) p.c_dst[i] = static_cast<__nv_bfloat16*>(c_ptrs[i]);
  // tile height: 256 rows when that still leaves at least four waves of tiles (UA_GEMM_MH forces)
  int mh = (static_cast<long>((M + 255) / 256) * ((N + GEMM_BN - 1) / GEMM_BN) >= 4L * num_sms) ? 2 : 1;
  if (const char* e = getenv("UA_GEMM_MH")) mh = atoi(e) == 2 ? 2 : 1;
  // CTA pairs (256 x 256 tile over two SMs): chosen per call by ua_gemm_pair_mode (the Python
  // wrapper times both forms once per shape and keeps the faster), or forced by UA_GEMM_PAIR=0 / 1
  bool pair = g_pair_mode > 0;
  if (const char* e = getenv("UA_GEMM_PAIR")) pair = atoi(e) != 0;
  if (pair) mh = 1;        // per-CTA boxes of the pair kernel are those of the 128-row kernel
  for (int i = 0; i < n_src; ++i) {
    if (!a_mn_major) {
      // [rows, k_per_src] K contiguous
      uint64_t dims[2] = {static_cast<uint64_t>(p.k_per_src), static_cast<uint64_t>(a_rows_total)};
      uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
      uint32_t box[2] = {GEMM_BK, static_cast<uint32_t>(128 * mh)};
      if (make_tmap_2byte(&p.tmA[i], a_ptrs[i], 2, dims, str, box)) return -1;
    } else {
      // [k rows, M] M contiguous; a_rows_total counts k rows
      uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(a_rows_total)};
      uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
      uint32_t box[2] = {64, GEMM_BK};
      if (make_tmap_2byte(&p.tmA[i], a_ptrs[i], 2, dims, str, box)) return -1;
    }
  }
  if (!b_mn_major) {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {GEMM_BK, static_cast<uint32_t>(pair ? 128 : GEMM_BN)};   // a pair loads half a tile per CTA
    if (make_tmap_2byte(&p.tmB, b, 2, dims, str, box)) return -1;
  } else {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    uint32_t box[2] = {64, GEMM_BK};
    if (make_tmap_2byte(&p.tmB, b, 2, dims, str, box)) return -1;
  }
  if (pair) return launch_gemm_pair(p, num_sms, stream);
  const int m_tiles = (M + 128 * mh - 1) / (128 * mh);
  const int n_tiles = (N + GEMM_BN - 1) / GEMM_BN;
  int grid = m_tiles * n_tiles;
  if (grid > num_sms) grid = num_sms;
  if (grid < 1) return 0;
  if (mh == 2) return launch_gemm<2>(p, grid, stream);
  return launch_gemm<1>(p, grid, stream);
  return 0;
}
