// Block-sparse flash-attention backward for sm_100a (tcgen05 + TMEM + TMA), five GEMMs per tile.
//
// Replaces the backward of the flash-attention fork that the reference calls with a precomputed
// softmax_d (orchestrated_attn/orchestrated_attn_impl.py:574-597): inputs are Q, K, V, dO, the
// forward's lse and D = rowsum(dO * O); O itself is never read.
//
// CTA = one 128-key tile of one key/value head. It keeps dK and dV for that tile in tensor memory
// while it walks every 128-query tile that attends to it (all query heads of the GQA group, all
// query segments of the block column). Per step (128 keys x 128 queries):
//     S^T  = K Q^T                 (128 x 128, TMEM)
//     dP^T = V dO^T                (TMEM)
//     P^T  = exp2(S^T * scale - lse)            -> bf16 into TMEM (A operand of dV)
//            (-lse / scale and -D are added by the tensor core: a ninth 16-wide reduction step
//            multiplies ones with three bf16 parts of each row term)
//     dV  += P^T dO                (A from TMEM, B = dO as an N-major operand)
//     dS^T = P^T * (dP^T - D)                    -> bf16 into shared memory
//     dQ^T = K^T dS^T              (TMEM, where dP^T was; drained by a warpgroup: registers ->
//                                   shared memory -> TMA reduce-add into the fp32 dQ accumulator)
//     dK  += dS^T Q                (A from shared memory, B = Q as an N-major operand)
// Everything is computed transposed so that P^T and dS^T come out with keys on the TMEM lanes,
// the layout the dV / dK products need for their A operand.
//
// All five products use N = 128 (40 instructions of 64 tensor-pipe clocks per step). That fills
// tensor memory (dK 128 | dV 128 | S^T 128 | dP^T/dQ^T 128 columns), so nothing is double-buffered;
// instead the issue order keeps the softmax warps fed: S^T of the next step is issued right behind
// dV of this one (the tensor pipe runs in issue order, so it may overwrite P^T), which makes it
// ready while the warps still turn dP^T into dS^T; dK fills the time the drain warpgroup needs to
// read dQ^T out before dP^T of the next step may overwrite it. lse and D of the next step are
// fetched into registers one step ahead.
//
//   warps 0-7 : two softmax warpgroups; thread (key, half) handles 64 of the 128 query columns of
//               its key row; in the epilogue one warpgroup stores dK, the other dV
//   warps 8-11: dQ drain warpgroup (one thread per head-dim element): each warp reads its whole
//               32 x 128 slice into registers (handing tensor memory back at once); the four warps
//               transpose it into three rotating [16 queries][128] staging tiles and one thread
//               issues cp.reduce.async.bulk.tensor (fp32 add at the memory side, 512-byte rows)
//               into the dQ accumulator; two reduces are in flight while the next tile is staged
//   warp  12  : TMA producer (K, V once; Q double-buffered; dO single-buffered)
//   warp  13  : tcgen05.mma issuer, TMEM allocation
// dK/dV leave the CTA either as bf16 stores (the CTA is their only producer) or as fp32
// red.add into an accumulator that may live in a peer GPU's memory (partial gradients of a
// key/value block computed away from its owner).
#include "attn_common.cuh"
#include "host_common.cuh"
#include "ptx.cuh"

namespace ua {

constexpr int BWD_THREADS = 512;              // four warpgroups (the last one: TMA, MMA, two idle warps)
constexpr int BWD_TMA_WARP = 12;
constexpr int BWD_MMA_WARP = 13;
constexpr int BWD_QT = 128;                // queries per step
constexpr int BWD_TILE_BYTES = ATTN_TILE * ATTN_D * 2;   // 32 KB: [2 halves][128 rows][128 B]
#ifndef UA_BWD_DQ_DIRECT
#define UA_BWD_DQ_DIRECT 0
#endif
// dQ leaves the CTA through a shared-memory transpose and TMA reduce-add (default), or straight
// from registers (one warp-wide 128-byte red.global.add per query row and 32 head-dim elements).
// Measured at S = 16k, 32 heads: 1.03 PFLOP/s with the TMA reduce, 0.88 with the direct form (its
// 512 reduction instructions per step crowd the load/store queue the softmax warps depend on).
constexpr bool BWD_DQ_DIRECT = UA_BWD_DQ_DIRECT != 0;
#ifndef UA_BWD_POLY_EXP_OF_8
#define UA_BWD_POLY_EXP_OF_8 0
#endif
constexpr int BWD_POLY_EXP_OF_8 = UA_BWD_POLY_EXP_OF_8;    // of every 8 exponentials, how many are polynomial

struct BwdCol {
  int kv_src;     // slot in tmK / tmV
  int kv_start;   // first key token inside that source
  int kv_len;     // keys in this block column
  int seg_begin;  // [seg_begin, seg_end) into segs (query segments)
  int seg_end;
  int g_slot;     // slot in the dK/dV output tables
  int g_start;    // first output row inside that slot
  int pad;
  int kv_wait_flag;   // staging flag of the key/value block (0: in place)
  int kv_wait_count;
};

struct BwdParams {
  CUtensorMap tmK[ATTN_MAX_SRC];
  CUtensorMap tmV[ATTN_MAX_SRC];
  CUtensorMap tmQ[ATTN_MAX_SRC];    // box of 128 rows
  CUtensorMap tmdO[ATTN_MAX_SRC];   // box of 128 rows
  const float* lse_ptr[ATTN_MAX_SRC];
  const float* dvec_ptr[ATTN_MAX_SRC];
  long lse_head_stride[ATTN_MAX_SRC];
  long lse_batch_stride[ATTN_MAX_SRC];
  int q_tokens[ATTN_MAX_SRC];       // tokens in each query-side source (bounds for lse / D)
  CUtensorMap tmdQ[ATTN_MAX_SRC];   // fp32 [batch, tokens, q heads, 128] accumulators, box 128x1x16
  float* dq_ptr[ATTN_MAX_SRC];      // the same accumulators as plain pointers
  long dq_row_stride[ATTN_MAX_SRC];     // elements between tokens
  long dq_batch_stride[ATTN_MAX_SRC];
  void* dk_ptr[ATTN_MAX_SRC];       // bf16 (store mode) or fp32 (add mode) [tokens, kv heads, 128]
  void* dv_ptr[ATTN_MAX_SRC];
  long dkv_row_stride[ATTN_MAX_SRC];
  long dkv_batch_stride[ATTN_MAX_SRC];
  int dkv_add_f32[ATTN_MAX_SRC];    // 1: fp32 red.add, 0: bf16 store
  const BwdCol* cols;
  const AttnSeg* segs;
  const int2* tiles;                // (column index, 128-key tile inside the column)
  int n_tiles;
  int n_kv_heads;
  int kv_group;
  float scale;                      // softmax scale
  float scale_log2;
  int* status;
  StageParams stage;                // optional in-kernel staging of remote blocks
  KernelTrace trace;                // optional per-CTA time stamps
};

struct __align__(1024) BwdSmem {
  uint8_t k[BWD_TILE_BYTES];
  uint8_t v[BWD_TILE_BYTES];
  uint8_t q[2][BWD_TILE_BYTES];
  uint8_t d_o[BWD_TILE_BYTES];
  uint8_t ds[BWD_TILE_BYTES];              // dS^T: two 64-query panels of [128 keys][128 B], swizzled
  float dq_stage[3][16 * 128];             // three tiles of [16 queries][128 head-dim] fp32 shared by the drain warps
  // One extra 16-wide reduction step folds the row terms into the products: S^T and dP^T come out
  // of the tensor core as S^T - lse / scale and dP^T - D. aug[stage]: per query 16 bf16 (columns 0-2:
  // three bf16 parts of -lse * log2(e) / scale_log2, columns 4-6: parts of -D, rest 0); ones_lse /
  // ones_d: per key 16 bf16 with ones in columns 0-2 resp. 4-6. Only the first 8 columns of each
  // operand are stored: the second 8 columns of both row-term stages are one shared block of zeros,
  // so what the ones operands present there (whatever finite data follows them) multiplies zero.
  // Layout: K-major without swizzle,
  // row r's first 8 columns at r * 16, the other 8 at 2048 + r * 16.
  uint8_t ones_lse[2048];     // first 8 columns only; the second chunk of a ones operand may alias any finite data
  uint8_t ones_d[2048];
  uint8_t aug[2][2048];       // first 8 columns of each stage; both share aug_zero as their second chunk
  uint8_t aug_zero[2048];
  uint64_t kv_full;
  uint64_t q_full[2];
  uint64_t q_empty[2];
  uint64_t do_full;
  uint64_t do_empty;
  uint64_t s_full;       // S^T ready               (tcgen05.commit)
  uint64_t dp_full;      // dP^T ready              (tcgen05.commit)
  uint64_t p_ready;      // P^T written to TMEM     (8 softmax warps, one arrival each)
  uint64_t ds_ready;     // dS^T written to smem    (8 softmax warps, one arrival each)
  uint64_t dq_full;      // dQ^T ready              (tcgen05.commit)
  uint64_t dq_free;      // dQ^T read out of TMEM   (4 drain warps, one arrival each)
  uint64_t dkv_full;
  uint64_t aug0_ready;   // the first step's row terms are in shared memory (8 softmax warps, one arrival each)
  uint32_t tmem_base;
  int abort_flag;
  int stage_slot;
};

static_assert(sizeof(BwdSmem) <= 232448, "BwdSmem exceeds the 227 KB a CTA may use");

// First 128-query tile of a segment that can see the key tile starting at column c0.
__device__ __forceinline__ int seg_first_qt(const AttnSeg& sg, int c0) {
  if (!sg.causal) return 0;
  const int r_min = c0 - sg.diag;   // smallest query index that sees key c0
  return r_min <= 0 ? 0 : r_min / BWD_QT;
}
__device__ __forceinline__ int seg_num_qt(const AttnSeg& sg) {
  return (sg.len + BWD_QT - 1) / BWD_QT;
}


// Optional pipeline trace (compile with -DUA_BWD_PROF): CTA (0, 0) records clock64() at the
// hand-over points of one step of every role into g_bwd_prof; ua_bwd_prof_read copies it out.
#ifdef UA_BWD_PROF
__device__ long long g_bwd_prof[64];
#define BWD_PROF(cond, slot) do { if ((cond) && blockIdx.x == 0 && blockIdx.y == 0) g_bwd_prof[slot] = clock64(); } while (0)
#else
#define BWD_PROF(cond, slot) do { } while (0)
#endif
constexpr int BWD_PROF_STEP = 8;

// Walks the (query head of the group, query segment, 128-query tile) steps of one key tile in the
// order every role of the CTA uses.
struct BwdStepIter {
  int g, e, t, nq;
  bool new_seg;      // first step of a (head, segment) pair
  AttnSeg sg;
  __device__ __forceinline__ void seek(const BwdParams& p, const BwdCol& col, int c0) {
    // (g, e) valid; find the next segment with work from here on
    for (;;) {
      sg = p.segs[e];
      nq = seg_num_qt(sg);
      t = seg_first_qt(sg, c0);
      if (t < nq) return;
      if (++e >= col.seg_end) { e = col.seg_begin; ++g; }
      if (g >= p.kv_group) return;     // callers never step past the last step
    }
  }
  __device__ __forceinline__ void first(const BwdParams& p, const BwdCol& col, int c0) {
    g = 0; e = col.seg_begin; new_seg = true;
    seek(p, col, c0);
  }
  __device__ __forceinline__ void next(const BwdParams& p, const BwdCol& col, int c0) {
    new_seg = false;
    if (++t < nq) return;
    new_seg = true;
    if (++e >= col.seg_end) { e = col.seg_begin; ++g; }
    if (g < p.kv_group) seek(p, col, c0);
  }
};

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// P^T of one thread's 64 queries: exp2(x * scale_log2) with x = S^T - lse / scale as it comes out
// of the tensor core, packed to bf16 pairs. MASK applies the causal / key-tail mask (tiles that
// need none skip the compares).
template <bool MASK>
__device__ __forceinline__ void bwd_phase_a(uint32_t t_st, float scale_log2, bool key_ok, int r_first,
                                            uint32_t (&pk)[32]) {
  float sv[2][32];
  tmem_ld_x32(t_st, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
  tmem_ld_x32(t_st + 32, reinterpret_cast<uint32_t(&)[32]>(sv[1]));
  tmem_wait_ld();
  const uint64_t sc2 = f2_pack(scale_log2, scale_log2);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#pragma unroll
    for (int c = 0; c < 32; c += 2) {
      float x0, x1;
      f2_unpack(f2_mul(f2_pack(sv[h][c], sv[h][c + 1]), sc2), x0, x1);     // two products per instruction
      // optionally some exponentials run on the FMA pipe; measured slower (the phase is bound by
      // instruction issue, not by the special-function unit), so the default is none
      const float p0 = (c & 7) < BWD_POLY_EXP_OF_8 ? poly_exp2(x0) : fast_exp2(x0);
      const float p1 = ((c + 1) & 7) < BWD_POLY_EXP_OF_8 ? poly_exp2(x1) : fast_exp2(x1);
      sv[h][c] = (!MASK || (key_ok && (h * 32 + c) >= r_first)) ? p0 : 0.f;
      sv[h][c + 1] = (!MASK || (key_ok && (h * 32 + c + 1) >= r_first)) ? p1 : 0.f;
    }
#pragma unroll
    for (int c = 0; c < 16; ++c) pk[h * 16 + c] = pack_bf16x2(sv[h][2 * c], sv[h][2 * c + 1]);
  }
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  // The operand tiles need 1 KB alignment and the CTA uses all 227 KB, so there is no room to align
  // by hand: the dynamic shared memory window itself has to start on a 1 KB boundary (it does on
  // sm_100 with no static shared memory). If it ever does not, fail loudly instead of computing
  // with misplaced swizzle atoms.
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0 && p.status != nullptr && atomicCAS(p.status, 0, UA_ERR_SMEM_ALIGN) == 0)
      p.status[1] = 999;
    return;
  }
  BwdSmem& s = *reinterpret_cast<BwdSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int kv_head = blockIdx.x / p.n_tiles;
  const int2 tl = p.tiles[blockIdx.x % p.n_tiles];
  const int batch = blockIdx.y;
  const BwdCol col = p.cols[tl.x];
  const int cta_linear = blockIdx.y * gridDim.x + blockIdx.x;
  trace_stamp(p.trace, cta_linear, 0);
  trace_ident(p.trace, cta_linear, tl.x);
  {
    // does this CTA read a staged block? then it first helps to empty the copy queue
    bool waits = col.kv_wait_flag != 0;
    for (int e = col.seg_begin; e < col.seg_end && !waits; ++e) waits = p.segs[e].wait_flag != 0;
    drain_stage_queue(p.stage, waits, cta_linear, &s.stage_slot);
  }
  trace_stamp(p.trace, cta_linear, 1);
  const int c0 = tl.y * ATTN_TILE;              // column-relative first key of this CTA

  if (threadIdx.x == 0) {
    mbar_init(&s.kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.q_empty[i], 1);
    }
    mbar_init(&s.do_full, 1);
    mbar_init(&s.do_empty, 1);
    mbar_init(&s.s_full, 1);
    mbar_init(&s.dp_full, 1);
    mbar_init(&s.p_ready, 8);
    mbar_init(&s.ds_ready, 8);
    mbar_init(&s.dq_full, 1);
    mbar_init(&s.dq_free, 4);
    mbar_init(&s.dkv_full, 1);
    mbar_init(&s.aug0_ready, 8);
    s.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == BWD_MMA_WARP) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  // constant operands of the extra reduction step; the unused half of the row-term tiles stays 0
  for (int r = threadIdx.x; r < 256; r += BWD_THREADS) {
    const int row = r & 127;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    if (r < 128) {
      *reinterpret_cast<uint4*>(s.ones_lse + row * 16) = make_uint4(0x3F803F80u, 0x00003F80u, 0u, 0u);
      *reinterpret_cast<uint4*>(s.aug_zero + row * 16) = zero;
      *reinterpret_cast<uint4*>(s.aug[0] + row * 16) = zero;
    } else {
      *reinterpret_cast<uint4*>(s.ones_d + row * 16) = make_uint4(0u, 0u, 0x3F803F80u, 0x00003F80u);
      *reinterpret_cast<uint4*>(s.aug[1] + row * 16) = zero;
    }
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  WaitCtx wc{&s.abort_flag, p.status, 4000000000ull};

  // number of (head, segment, query tile) steps; identical in every role
  int steps_per_head = 0;
  for (int e = col.seg_begin; e < col.seg_end; ++e) {
    const AttnSeg sg = p.segs[e];
    const int n = seg_num_qt(sg) - seg_first_qt(sg, c0);
    steps_per_head += n > 0 ? n : 0;
  }
  const int n_steps = steps_per_head * p.kv_group;

  if (warp >= BWD_TMA_WARP) {
    // last warpgroup (TMA, MMA, two idle warps): the drain warpgroup takes most of its registers.
    // The instruction sits inside this branch so that the other roles keep their full budget.
    reg_dealloc<96>();
  if (warp == BWD_TMA_WARP) {
    // =============================== TMA producer ===========================================
    if (lane == 0 && n_steps > 0) {
      const int krow = col.kv_start + c0;
      bool ok = true;
      if (!wait_staged(p.stage.flags, col.kv_wait_flag, col.kv_wait_count * p.stage.epoch, wc.budget_ns)) {
        report_error(wc, UA_ERR_FLAG_TIMEOUT, 120, col.kv_wait_flag);
        ok = false;
      }
      mbar_arrive_expect_tx(&s.kv_full, 2 * BWD_TILE_BYTES);
      tma_load_4d(s.k, &p.tmK[col.kv_src], &s.kv_full, 0, kv_head, krow, batch);
      tma_load_4d(s.k + 16384, &p.tmK[col.kv_src], &s.kv_full, 64, kv_head, krow, batch);
      tma_load_4d(s.v, &p.tmV[col.kv_src], &s.kv_full, 0, kv_head, krow, batch);
      tma_load_4d(s.v + 16384, &p.tmV[col.kv_src], &s.kv_full, 64, kv_head, krow, batch);
      uint32_t i = 0;
      for (int g = 0; g < p.kv_group && ok; ++g) {
        const int head = kv_head * p.kv_group + g;
        for (int e = col.seg_begin; e < col.seg_end && ok; ++e) {
          const AttnSeg sg = p.segs[e];
          const int nq = seg_num_qt(sg);
          if (seg_first_qt(sg, c0) < nq &&
              !wait_staged(p.stage.flags, sg.wait_flag, sg.wait_count * p.stage.epoch, wc.budget_ns)) {
            report_error(wc, UA_ERR_FLAG_TIMEOUT, 121, sg.wait_flag);
            ok = false;
            break;
          }
          for (int t = seg_first_qt(sg, c0); t < nq; ++t, ++i) {
            const int st = i & 1;
            const int qrow = sg.start + t * BWD_QT;
            if (!mbar_wait(&s.q_empty[st], ((i >> 1) & 1) ^ 1, wc, 100)) { ok = false; break; }
            mbar_arrive_expect_tx(&s.q_full[st], BWD_TILE_BYTES);
            tma_load_4d(s.q[st], &p.tmQ[sg.src], &s.q_full[st], 0, head, qrow, batch);
            tma_load_4d(s.q[st] + 16384, &p.tmQ[sg.src], &s.q_full[st], 64, head, qrow, batch);
            if (!mbar_wait(&s.do_empty, (i & 1) ^ 1, wc, 101)) { ok = false; break; }
            mbar_arrive_expect_tx(&s.do_full, BWD_TILE_BYTES);
            tma_load_4d(s.d_o, &p.tmdO[sg.src], &s.do_full, 0, head, qrow, batch);
            tma_load_4d(s.d_o + 16384, &p.tmdO[sg.src], &s.do_full, 64, head, qrow, batch);
          }
        }
      }
    }
  } else if (warp == BWD_MMA_WARP) {
    // =============================== MMA issuer =============================================
    if (lane == 0 && n_steps > 0) {
      const uint32_t idesc_kk = make_idesc_bf16(128, 128, 0, 0);   // S^T, dP^T: both K-major
      const uint32_t idesc_kn = make_idesc_bf16(128, 128, 0, 1);   // dV, dK: B N-major
      const uint32_t idesc_nn = make_idesc_bf16(128, 128, 1, 1);   // dQ^T: A, B MN-major
      const uint32_t t_dk = tmem_base + 0;
      const uint32_t t_dv = tmem_base + 128;
      const uint32_t t_st = tmem_base + 256;     // S^T, later P^T (packed) at columns 0-31, 64-95
      const uint32_t t_dp = tmem_base + 384;     // dP^T, later dQ^T
      // one base descriptor per operand view; every instruction adds its (16-byte unit) offset to
      // the address field, which cannot carry out of it for addresses inside shared memory
      const uint64_t k_kmaj = make_smem_desc_sw128(smem_u32(s.k), 16, 1024);        // A of S^T
      const uint64_t k_mmaj = make_smem_desc_sw128(smem_u32(s.k), 16384, 1024);     // A of dQ^T
      const uint64_t v_kmaj = make_smem_desc_sw128(smem_u32(s.v), 16, 1024);        // A of dP^T
      const uint64_t do_kmaj = make_smem_desc_sw128(smem_u32(s.d_o), 16, 1024);     // B of dP^T
      const uint64_t do_nmaj = make_smem_desc_sw128(smem_u32(s.d_o), 16384, 1024);  // B of dV
      const uint64_t ds_kmaj = make_smem_desc_sw128(smem_u32(s.ds), 16, 1024);      // A of dK
      const uint64_t ds_nmaj = make_smem_desc_sw128(smem_u32(s.ds), 16384, 1024);   // B of dQ^T
      const uint64_t q_kmaj0 = make_smem_desc_sw128(smem_u32(s.q[0]), 16, 1024);    // B of S^T
      const uint64_t q_nmaj0 = make_smem_desc_sw128(smem_u32(s.q[0]), 16384, 1024); // B of dK
      const uint64_t ones_lse_d = make_smem_desc_noswz(smem_u32(s.ones_lse), 2048, 128);
      const uint64_t ones_d_d = make_smem_desc_noswz(smem_u32(s.ones_d), 2048, 128);
      // stage 0: chunks at aug[0] and aug_zero (4096 apart); stage 1: at aug[1] and aug_zero (2048 apart)
      const uint64_t aug_desc[2] = {make_smem_desc_noswz(smem_u32(s.aug[0]), 4096, 128),
                                    make_smem_desc_noswz(smem_u32(s.aug[1]), 2048, 128)};
      constexpr uint64_t Q_STAGE = BWD_TILE_BYTES >> 4;
      // K-major operands: 16 elements of the reduction = 32 B, the two 64-element halves 16384 B apart
      auto koff = [](int kk) -> uint64_t { return static_cast<uint64_t>(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4); };
      // MN-major operands: 16 rows of the reduction = 2048 B
      auto noff = [](int kk) -> uint64_t { return static_cast<uint64_t>((kk * 2048) >> 4); };
      auto issue_st = [&](int st) {
        const uint64_t qd = q_kmaj0 + st * Q_STAGE;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(t_st, k_kmaj + koff(kk), qd + koff(kk), idesc_kk, kk > 0 ? 1u : 0u);
        umma_ss(t_st, ones_lse_d, aug_desc[st], idesc_kk, 1u);     // - lse / scale
      };
      auto issue_dp = [&](int st) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(t_dp, v_kmaj + koff(kk), do_kmaj + koff(kk), idesc_kk, kk > 0 ? 1u : 0u);
        umma_ss(t_dp, ones_d_d, aug_desc[st], idesc_kk, 1u);       // - D
      };
      bool ok = true;
      do {
        if (!mbar_wait(&s.kv_full, 0, wc, 200)) { ok = false; break; }
        if (!mbar_wait(&s.q_full[0], 0, wc, 201)) { ok = false; break; }
        if (!mbar_wait(&s.aug0_ready, 0, wc, 208)) { ok = false; break; }
        tc_fence_after_sync();
        issue_st(0);
        tc_commit(&s.s_full);
        if (!mbar_wait(&s.do_full, 0, wc, 202)) { ok = false; break; }
        tc_fence_after_sync();
        issue_dp(0);
        tc_commit(&s.dp_full);
        for (int i = 0; i < n_steps; ++i) {
          const int st = i & 1;
          const uint32_t ph = i & 1;
          const uint64_t qn = q_nmaj0 + st * Q_STAGE;
          const bool more = i + 1 < n_steps;
          // dV += P^T dO : A = P^T in TMEM (queries 0-63 packed at columns 0-31, 64-127 at 64-95),
          // B = dO as an N-major operand (16 query rows = 2048 B, d-halves 16384 B apart)
          BWD_PROF(i == BWD_PROF_STEP, 0);
          if (!mbar_wait(&s.p_ready, ph, wc, 203)) { ok = false; break; }
          BWD_PROF(i == BWD_PROF_STEP, 1);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ts(t_dv, t_st + (kk >> 2) * 64 + (kk & 3) * 8, do_nmaj + noff(kk), idesc_kn,
                    (i > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&s.do_empty);
          // S^T of the next step right behind it: it overwrites P^T(i), which dV(i) reads first
          // because the tensor pipe executes in issue order
          if (more) {
            if (!mbar_wait(&s.q_full[st ^ 1], ((i + 1) >> 1) & 1, wc, 205)) { ok = false; break; }
            tc_fence_after_sync();
            BWD_PROF(i == BWD_PROF_STEP, 2);
            issue_st(st ^ 1);
            tc_commit(&s.s_full);
          }
          BWD_PROF(i == BWD_PROF_STEP, 3);
          // dQ^T = K^T dS^T : A = K as an M-major operand, B = dS^T as an N-major operand (two
          // 64-query panels 16384 B apart); lands where dP^T was
          if (!mbar_wait(&s.ds_ready, ph, wc, 204)) { ok = false; break; }
          BWD_PROF(i == BWD_PROF_STEP, 4);
          tc_fence_after_sync();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(t_dp, k_mmaj + noff(kk), ds_nmaj + noff(kk), idesc_nn, kk > 0 ? 1u : 0u);
          tc_commit(&s.dq_full);
          // dK += dS^T Q : A = dS^T in shared memory (K-major over queries: panel kk/4, 32 B per
          // step), B = Q as an N-major operand; runs while the drain warpgroup reads dQ^T
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(t_dk, ds_kmaj + koff(kk), qn + noff(kk), idesc_kn, (i > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&s.q_empty[st]);
          BWD_PROF(i == BWD_PROF_STEP, 5);
          if (more) {
            if (!mbar_wait(&s.do_full, (i + 1) & 1, wc, 206)) { ok = false; break; }
            BWD_PROF(i == BWD_PROF_STEP, 6);
            // dP^T(i+1) lands where dQ^T(i) is: wait until the drain warpgroup has read it
            if (!mbar_wait(&s.dq_free, ph, wc, 207)) { ok = false; break; }
            BWD_PROF(i == BWD_PROF_STEP, 7);
            tc_fence_after_sync();
            issue_dp(st ^ 1);
            tc_commit(&s.dp_full);
            BWD_PROF(i == BWD_PROF_STEP, 8);
          }
        }
        if (ok) tc_commit(&s.dkv_full);
      } while (false);
    }
  }
  } else if (warp < 8) {
    // =============================== softmax warpgroups =====================================
    const int wg = warp >> 2;                        // which half of the 128 query columns
    const int quad = warp & 3;
    const int key_t = quad * 32 + lane;              // key inside the tile
    const int key_c = c0 + key_t;                    // key inside the block column
    const bool key_ok = key_c < col.kv_len;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_st = tmem_base + lane_base + 256 + wg * 64;
    const uint32_t t_dp = tmem_base + lane_base + 384 + wg * 64;
    bool ok = true;
    // Row terms (lse, D) of the 128 queries of a step: warp w, lanes 0-15 handle queries
    // 16 w .. 16 w + 15. They are fetched two steps ahead and written into the extra operand tile
    // one step ahead, so that S^T of the next step can be issued as soon as P^T of this one exists.
    // Per (head, segment) values are looked up once per segment: the kernel parameters they come
    // from are indexed dynamically, which is too slow for the per-step path.
    const float* lse_g = nullptr;
    const float* dv_g = nullptr;
    int row_lim = 0;                     // rows of the segment that exist in its source
    const float inv_scale_log2 = 1.4426950408889634f / p.scale_log2;
    auto fetch = [&](const BwdStepIter& it, float& lv, float& dv) -> bool {
      if (it.new_seg) {
        const AttnSeg& sg = it.sg;
        if (sg.wait_flag != 0) {
          // lse / D of a staged segment are read with plain loads: make sure they landed
          int w_ok = 1;
          if (lane == 0) w_ok = wait_staged(p.stage.flags, sg.wait_flag, sg.wait_count * p.stage.epoch, wc.budget_ns) ? 1 : 0;
          w_ok = __shfl_sync(0xFFFFFFFFu, w_ok, 0);
          if (!w_ok) return false;
        }
        const int head = kv_head * p.kv_group + it.g;
        const long off = batch * p.lse_batch_stride[sg.src] + head * p.lse_head_stride[sg.src] + sg.start;
        lse_g = p.lse_ptr[sg.src] + off;
        dv_g = p.dvec_ptr[sg.src] + off;
        row_lim = min(sg.len, p.q_tokens[sg.src] - sg.start);
      }
      const int r = it.t * BWD_QT + warp * 16 + lane;
      lv = INFINITY;                     // rows outside the segment: lse = +inf -> P = 0
      dv = 0.f;
      if (lane < 16 && r < row_lim) {
        lv = lse_g[r];                   // consumed a step later: nothing waits for it here
        dv = dv_g[r];
      }
      return true;
    };
    // three bf16 parts of x (their sum has about 24 significant bits)
    auto split3 = [](float x, uint32_t& hm, uint32_t& l0) {
      const __nv_bfloat16 h = __float2bfloat16_rn(x);
      const float r1 = x - __bfloat162float(h);
      const __nv_bfloat16 m = __float2bfloat16_rn(r1);
      const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
      hm = static_cast<uint32_t>(__bfloat16_as_ushort(h)) | (static_cast<uint32_t>(__bfloat16_as_ushort(m)) << 16);
      l0 = static_cast<uint32_t>(__bfloat16_as_ushort(l));
    };
    auto write_aug = [&](int stage, float lv, float dv) {
      if (lane < 16) {
        // a row that attends to nothing (lse = -inf) or does not exist (+inf) gets a huge negative
        // term: its probabilities come out as exactly 0
        const float nl = (lv == INFINITY || lv == -INFINITY) ? -3.0e38f : -lv * inv_scale_log2;
        uint32_t a0, a1, b0, b1;
        split3(nl, a0, a1);
        split3(-dv, b0, b1);
        *reinterpret_cast<uint4*>(s.aug[stage] + (warp * 16 + lane) * 16) = make_uint4(a0, a1, b0, b1);
      }
      fence_proxy_async_smem();
    };
    BwdStepIter cur, fut;
    float lv = INFINITY, dv = 0.f;
    if (n_steps > 0) {
      cur.first(p, col, c0);
      fut = cur;
      ok = fetch(fut, lv, dv);
      if (ok) {
        write_aug(0, lv, dv);
        mbar_arrive_warp(&s.aug0_ready);
        if (n_steps > 1) {
          fut.next(p, col, c0);
          ok = fetch(fut, lv, dv);
        }
      }
    }
    for (int i = 0; i < n_steps && ok; ++i) {
      const uint32_t ph = i & 1;
      const AttnSeg& sg = cur.sg;
      const bool prof = i == BWD_PROF_STEP && quad == 0 && lane == 0;
      const int pslot = 16 + wg * 16;
      (void)prof; (void)pslot;
      BWD_PROF(prof, pslot + 0);
      // row terms of step i+1 into the operand tile (its previous user, step i-1, is complete: this
      // thread has consumed dP^T(i-1)); the arrival on p_ready below publishes them
      if (i + 1 < n_steps) write_aug((i + 1) & 1, lv, dv);
      BWD_PROF(prof, pslot + 7);
      // visible iff key_c <= r + diag  <=>  r >= key_c - diag   (r relative to this half)
      const int r_first = sg.causal ? (key_c - sg.diag - cur.t * BWD_QT - wg * 64) : 0;
      // the row terms of step i+2 travel while this step computes
      if (i + 2 < n_steps) {
        fut.next(p, col, c0);
        if (!fetch(fut, lv, dv)) { ok = false; break; }
      }

      // ---- phase A: P^T = exp2((S^T - lse / scale) * scale) -> TMEM (packed bf16) ------------
      BWD_PROF(prof, pslot + 1);
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s.s_full, ph, wc, 300))) { ok = false; break; }
      BWD_PROF(prof, pslot + 2);
      tc_fence_after_sync();
      uint32_t pk[32];                 // this thread's 64 probabilities, packed; kept for phase B
      if (__all_sync(0xFFFFFFFFu, key_ok && r_first <= 0))
        bwd_phase_a<false>(t_st, p.scale_log2, key_ok, r_first, pk);
      else
        bwd_phase_a<true>(t_st, p.scale_log2, key_ok, r_first, pk);
      // packed P^T of this half goes to the first 32 columns of this half's own S^T columns
      // (the other warpgroup may still be reading its fp32 half)
      BWD_PROF(prof, pslot + 3);
      tmem_st_x32(t_st, pk);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(&s.p_ready);
      BWD_PROF(prof, pslot + 4);

      // ---- phase B: dS^T = P^T * (dP^T - D) -> shared memory ------------------------------
      if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s.dp_full, ph, wc, 301))) { ok = false; break; }
      BWD_PROF(prof, pslot + 5);
      tc_fence_after_sync();
      uint8_t* ds_panel = s.ds + wg * 16384;     // this half's 64-query panel
      {
        uint32_t dp[2][32];
        tmem_ld_x32(t_dp, dp[0]);
        tmem_ld_x32(t_dp + 32, dp[1]);
        tmem_wait_ld();
        BWD_PROF(prof, pslot + 8);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {          // 8 queries = one 16-byte chunk
            uint32_t w4[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              // (dP - D), as it comes out of the tensor core, rounded to bf16 pairs, times the bf16
              // probabilities (masked ones are 0)
              const uint32_t x = pack_bf16x2(__uint_as_float(dp[h][ch * 8 + 2 * c]),
                                             __uint_as_float(dp[h][ch * 8 + 2 * c + 1]));
              w4[c] = mul_bf16x2(pk[h * 16 + ch * 4 + c], x);
            }
            *reinterpret_cast<uint4*>(ds_panel + sw128_offset(key_t, h * 4 + ch)) =
                make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      }
      BWD_PROF(prof, pslot + 9);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(&s.ds_ready);
      BWD_PROF(prof, pslot + 6);
      if (i + 1 < n_steps) cur.next(p, col, c0);
    }
    // ---------------------------------- dK / dV epilogue ------------------------------------
    if (n_steps > 0 && ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait(&s.dkv_full, 0, wc, 310));
    tc_fence_after_sync();
    const int slot = col.g_slot;
    const long grow = static_cast<long>(col.g_start + key_c);
    const long goff = batch * p.dkv_batch_stride[slot] + grow * p.dkv_row_stride[slot] +
                      static_cast<long>(kv_head) * ATTN_D;
#pragma unroll 1
    for (int which = wg; which <= wg; ++which) {      // warpgroup 0 stores dK, warpgroup 1 dV
      const uint32_t t_acc = tmem_base + lane_base + which * 128;
      const float mul = which == 0 ? p.scale : 1.0f;
      void* base = which == 0 ? p.dk_ptr[slot] : p.dv_ptr[slot];
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t av[32];
        if (n_steps > 0) {
          tmem_ld_x32(t_acc + c * 32, av);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) av[q] = 0u;
        }
        if (!key_ok) continue;
        if (p.dkv_add_f32[slot]) {
          if (n_steps == 0) continue;
          float* dst = static_cast<float*>(base) + goff + c * 32;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + q * 4),
                         "f"(__uint_as_float(av[q * 4 + 0]) * mul),
                         "f"(__uint_as_float(av[q * 4 + 1]) * mul),
                         "f"(__uint_as_float(av[q * 4 + 2]) * mul),
                         "f"(__uint_as_float(av[q * 4 + 3]) * mul)
                         : "memory");
          }
        } else {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(base) + goff + c * 32;
          uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(av[q * 8 + 0]) * mul, __uint_as_float(av[q * 8 + 1]) * mul);
            o.y = pack_bf16x2(__uint_as_float(av[q * 8 + 2]) * mul, __uint_as_float(av[q * 8 + 3]) * mul);
            o.z = pack_bf16x2(__uint_as_float(av[q * 8 + 4]) * mul, __uint_as_float(av[q * 8 + 5]) * mul);
            o.w = pack_bf16x2(__uint_as_float(av[q * 8 + 6]) * mul, __uint_as_float(av[q * 8 + 7]) * mul);
            d4[q] = o;
          }
        }
      }
    }
  } else {
    // =============================== dQ drain warpgroup =====================================
    reg_alloc<160>();        // holds a whole 128-query dQ^T slice in registers
    const int quad = warp & 3;                       // TMEM lanes quad*32.. = head-dim slice
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t t_dq = tmem_base + lane_base + 384;
    float* stage = s.dq_stage[0];
    bool ok = true;
    uint32_t i = 0;
    uint32_t n_chunk = 0;
    for (int g = 0; g < p.kv_group && ok; ++g) {
      const int head = kv_head * p.kv_group + g;
      for (int e = col.seg_begin; e < col.seg_end && ok; ++e) {
        const AttnSeg sg = p.segs[e];
        const int nq = seg_num_qt(sg);
        const CUtensorMap* tdq = &p.tmdQ[sg.src];
        const long rs = p.dq_row_stride[sg.src];
        float* dq_col = p.dq_ptr[sg.src] + batch * p.dq_batch_stride[sg.src] +
                        static_cast<long>(head) * ATTN_D + quad * 32 + lane;
        const int tokens = p.q_tokens[sg.src];
        for (int t = seg_first_qt(sg, c0); t < nq; ++t, ++i) {
          BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0, 48);
          if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s.dq_full, i & 1, wc, 400))) { ok = false; break; }
          BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0, 49);
          tc_fence_after_sync();
          const int qrow = sg.start + t * BWD_QT;
          // read the whole slice and hand TMEM back at once: dP^T of the next step is waiting for it
          uint32_t dv[4][32];
#pragma unroll
          for (int h = 0; h < 4; ++h) tmem_ld_x32(t_dq + h * 32, dv[h]);
          tmem_wait_ld();
          tc_fence_before_sync();
          mbar_arrive_warp(&s.dq_free);
          BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0, 50);
          if (BWD_DQ_DIRECT) {
            // lane = head-dim element, register = query: the 32 lanes of one instruction cover 128
            // contiguous bytes of one query row
            float* dst = dq_col + static_cast<long>(qrow) * rs;
            const int n_valid = min(BWD_QT, tokens - qrow);      // rows that exist in the accumulator
            if (n_valid == BWD_QT) {
#pragma unroll
              for (int h = 0; h < 4; ++h)
#pragma unroll
                for (int c = 0; c < 32; ++c)
                  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (h * 32 + c) * rs),
                               "f"(__uint_as_float(dv[h][c]) * p.scale) : "memory");
            } else {
#pragma unroll
              for (int h = 0; h < 4; ++h)
#pragma unroll
                for (int c = 0; c < 32; ++c)
                  if (h * 32 + c < n_valid)
                    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (h * 32 + c) * rs),
                                 "f"(__uint_as_float(dv[h][c]) * p.scale) : "memory");
            }
          } else {
#pragma unroll
            for (int h = 0; h < 8; ++h) {              // 16 queries at a time, three staging tiles in turn
              // The four warps fill one [16 queries][128 head-dim] tile (a 32-wide slice each) and one
              // thread issues a single reduce with 512-byte rows. The reduce issued three chunks
              // ago (same tile) must have finished reading it; the last two may still be in flight.
              if (quad == 0 && lane == 0) tma_store_wait_read_all_but<2>();
              asm volatile("bar.sync 1, 128;" ::: "memory");
              BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0 && (h & 1) == 0, 52 + (h >> 1) * 3);
              float* tile = stage + ((n_chunk + h) % 3) * 2048;
#pragma unroll
              for (int c = 0; c < 16; ++c)
                tile[c * 128 + quad * 32 + lane] = __uint_as_float(dv[h >> 1][(h & 1) * 16 + c]) * p.scale;
              fence_proxy_async_smem();
              asm volatile("bar.sync 1, 128;" ::: "memory");
              BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0 && (h & 1) == 0, 53 + (h >> 1) * 3);
              if (quad == 0 && lane == 0) {
                tma_reduce_add_4d(tdq, tile, 0, head, qrow + h * 16, batch);
                tma_store_commit();
              }
              BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0 && (h & 1) == 0, 54 + (h >> 1) * 3);
            }
          }
          n_chunk += 8;
          BWD_PROF(i == BWD_PROF_STEP && quad == 0 && lane == 0, 51);
        }
      }
    }
    if (lane == 0) tma_store_wait_all();
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  trace_stamp(p.trace, cta_linear, 2);
  if (warp == BWD_MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ua

using namespace ua;

#ifdef UA_BWD_PROF
extern "C" int ua_bwd_prof_read(long long* host64) {
  UA_CUDA(cudaMemcpyFromSymbol(host64, g_bwd_prof, sizeof(long long) * 64));
  return 0;
}
#endif

struct UaTensorSrc {
  const void* ptr;
  long tokens;
  long heads;
  long batch;
  long token_stride;
  long head_stride;
  long batch_stride;
};
// query-side extras of one source
struct UaBwdQSide {
  const float* lse;        // [batch, heads, tokens]
  const float* dvec;       // same layout
  long lse_head_stride;
  long lse_batch_stride;
  float* dq;               // fp32 [batch, tokens, heads, 128], heads*128 contiguous per token
  long dq_row_stride;      // elements between tokens
  long dq_batch_stride;
};
struct UaBwdKvOut {
  void* dk;
  void* dv;
  long row_stride;
  long batch_stride;
  int add_f32;
  int pad;
};

static int encode_src_box(CUtensorMap* tm, const UaTensorSrc& t, uint32_t rows) {
  uint64_t dims[4] = {ATTN_D, static_cast<uint64_t>(t.heads), static_cast<uint64_t>(t.tokens),
                      static_cast<uint64_t>(t.batch)};
  uint64_t str[3] = {static_cast<uint64_t>(t.head_stride) * 2,
                     static_cast<uint64_t>(t.token_stride) * 2,
                     static_cast<uint64_t>(t.batch_stride > 0 ? t.batch_stride : t.token_stride * t.tokens) * 2};
  uint32_t box[4] = {64, 1, rows, 1};
  return make_tmap_2byte(tm, t.ptr, 4, dims, str, box);
}

static int g_bwd_smem_set[64] = {0};

extern "C" int ua_attn_bwd(const UaTensorSrc* q_src, const UaTensorSrc* do_src,
                           const UaBwdQSide* q_side, int n_q, const UaTensorSrc* k_src,
                           const UaTensorSrc* v_src, int n_kv, const UaBwdKvOut* kv_out, int n_out,
                           const void* cols_dev, const void* segs_dev, const void* tiles_dev,
                           int n_tiles, int n_heads, int n_kv_heads, int batch,
                           float softmax_scale, int* status, const void* copy_tasks_dev,
                           int n_copy_tasks, int n_copy_ctas, unsigned int* stage_flags,
                           int stage_epoch, unsigned int* stage_ticket, cudaStream_t stream) {
  if (n_q > ATTN_MAX_SRC || n_kv > ATTN_MAX_SRC || n_out > ATTN_MAX_SRC)
    UA_FAIL("ua_attn_bwd: too many sources (max %d)", ATTN_MAX_SRC);
  if (n_tiles <= 0) return 0;
  BwdParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < n_q; ++i) {
    if (encode_src_box(&p.tmQ[i], q_src[i], BWD_QT)) return -1;
    if (encode_src_box(&p.tmdO[i], do_src[i], BWD_QT)) return -1;
    p.lse_ptr[i] = q_side[i].lse;
    p.dvec_ptr[i] = q_side[i].dvec;
    p.lse_head_stride[i] = q_side[i].lse_head_stride;
    p.lse_batch_stride[i] = q_side[i].lse_batch_stride;
    p.q_tokens[i] = static_cast<int>(q_src[i].tokens);
    {
      const UaTensorSrc& t = q_src[i];
      uint64_t dims[4] = {ATTN_D, static_cast<uint64_t>(t.heads), static_cast<uint64_t>(t.tokens),
                          static_cast<uint64_t>(t.batch)};
      const long bstr = q_side[i].dq_batch_stride > 0 ? q_side[i].dq_batch_stride
                                                      : q_side[i].dq_row_stride * t.tokens;
      uint64_t str[3] = {ATTN_D * 4ull, static_cast<uint64_t>(q_side[i].dq_row_stride) * 4,
                         static_cast<uint64_t>(bstr) * 4};
      uint32_t box[4] = {128, 1, 16, 1};
      if (make_tmap_f32(&p.tmdQ[i], q_side[i].dq, 4, dims, str, box)) return -1;
      p.dq_ptr[i] = q_side[i].dq;
      p.dq_row_stride[i] = q_side[i].dq_row_stride;
      p.dq_batch_stride[i] = bstr;
    }
  }
  for (int i = 0; i < n_kv; ++i) {
    if (encode_src_box(&p.tmK[i], k_src[i], ATTN_TILE)) return -1;
    if (encode_src_box(&p.tmV[i], v_src[i], ATTN_TILE)) return -1;
  }
  for (int i = 0; i < n_out; ++i) {
    p.dk_ptr[i] = kv_out[i].dk;
    p.dv_ptr[i] = kv_out[i].dv;
    p.dkv_row_stride[i] = kv_out[i].row_stride;
    p.dkv_batch_stride[i] = kv_out[i].batch_stride;
    p.dkv_add_f32[i] = kv_out[i].add_f32;
  }
  p.cols = static_cast<const BwdCol*>(cols_dev);
  p.segs = static_cast<const AttnSeg*>(segs_dev);
  p.tiles = static_cast<const int2*>(tiles_dev);
  p.n_tiles = n_tiles;
  p.n_kv_heads = n_kv_heads;
  p.kv_group = n_heads / n_kv_heads;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  p.stage.tasks = static_cast<const CopyTask*>(copy_tasks_dev);
  p.stage.n_tasks = n_copy_tasks;
  {
    const long grid_ctas = static_cast<long>(n_tiles) * n_kv_heads * batch;
    p.stage.n_copy_ctas = static_cast<int>(n_copy_ctas < grid_ctas ? n_copy_ctas : grid_ctas);
  }
  p.stage.flags = stage_flags;
  p.stage.epoch = stage_epoch;
  p.stage.ticket = stage_ticket;
  {
    int tdev = 0;
    UA_CUDA(cudaGetDevice(&tdev));
    const TraceSlot ts = tdev < 64 ? trace_registry()[1 * 64 + tdev] : TraceSlot{nullptr, 0};
    p.trace.buf = ts.buf;
    p.trace.cap = ts.cap;
  }
  if (n_copy_tasks > 0) {
    if (stage_ticket == nullptr) UA_FAIL("ua_attn_bwd: copy tasks need a ticket counter");
    UA_CUDA(cudaMemsetAsync(stage_ticket, 0, sizeof(unsigned int), stream));
  }
  const int smem_bytes = sizeof(BwdSmem);
  int dev = 0;
  UA_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !g_bwd_smem_set[dev]) {
    UA_CUDA(cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes));
    g_bwd_smem_set[dev] = 1;
  }
  dim3 grid(n_tiles * n_kv_heads, batch, 1);
  attn_bwd_kernel<<<grid, BWD_THREADS, smem_bytes, stream>>>(p);
  UA_CUDA(cudaGetLastError());
  return 0;
}

// =================================================================================================
// Allocation-free dense backward (declared in ultraattn_noalloc.h)
// =================================================================================================
// Same kernel as above, for callers that must not allocate device memory while they run: code
// inside a CUDA-graph capture or a real-time serving loop, a plug-in living in a host process
// whose memory pool it may not touch, or a process that has already handed all free HBM to its
// own allocator (cudaMalloc would fail or stall there). The fp32 dQ accumulator and the small
// launch tables, which ua_attn_bwd() expects the caller to provide, live in the file-scope
// device array below instead. Every GPU that loads this library holds the array until the
// process exits.
namespace ua {

constexpr long NOALLOC_MAX_QH_TOKENS = 131072;     // tokens * query heads, at most
constexpr int NOALLOC_MAX_TOKENS = 65536;
constexpr long NOALLOC_DQ_BYTES = NOALLOC_MAX_QH_TOKENS * ATTN_D * 4;           // 64 MiB
constexpr long NOALLOC_COL_OFF = NOALLOC_DQ_BYTES;
constexpr long NOALLOC_SEG_OFF = NOALLOC_COL_OFF + 256;
constexpr long NOALLOC_TILE_OFF = NOALLOC_SEG_OFF + 256;
constexpr long NOALLOC_BYTES = NOALLOC_TILE_OFF + (NOALLOC_MAX_TOKENS / ATTN_TILE) * 8;

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

// In host code the array's name is only a stand-in: the device address is looked up once per
// device (with that device current) and cached here.
static unsigned char* g_noalloc_ptr[64] = {nullptr};

__global__ void noalloc_fill_tables(BwdCol* col, AttnSeg* seg, int2* tiles, int tokens, int causal) {
  const int n_tiles = (tokens + ATTN_TILE - 1) / ATTN_TILE;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    BwdCol c;
    c.kv_src = 0; c.kv_start = 0; c.kv_len = tokens; c.seg_begin = 0; c.seg_end = 1;
    c.g_slot = 0; c.g_start = 0; c.pad = 0; c.kv_wait_flag = 0; c.kv_wait_count = 0;
    *col = c;
    AttnSeg s;
    s.src = 0; s.start = 0; s.len = tokens; s.causal = causal; s.diag = 0;
    s.wait_flag = 0; s.wait_count = 0; s.pad2 = 0;
    *seg = s;
  }
  // key tile t of a causal problem is visited by all query sub-tiles at or below it, so the
  // heaviest tiles are the first ones: ascending order is already heaviest-first
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n_tiles; t += gridDim.x * blockDim.x)
    tiles[t] = make_int2(0, t);
}

__global__ void noalloc_cast_dq(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long n) {
  const long stride = static_cast<long>(gridDim.x) * blockDim.x * 4;
  for (long i = (static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    const float4 v = *reinterpret_cast<const float4*>(src + i);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + i) = o;
  }
}

}  // namespace ua

extern "C" int ua_attn_bwd_dense_noalloc(const void* q, const void* k, const void* v, const void* d_o,
                                         const float* lse, const float* dvec, void* dq, void* dk,
                                         void* dv, int tokens, int n_heads, int n_kv_heads,
                                         int causal, float softmax_scale, int* status,
                                         cudaStream_t stream) {
  if (tokens <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0)
    UA_FAIL("ua_attn_bwd_dense_noalloc: bad shape (tokens=%d, heads=%d, kv heads=%d)", tokens, n_heads,
            n_kv_heads);
  if (tokens > NOALLOC_MAX_TOKENS || static_cast<long>(tokens) * n_heads > NOALLOC_MAX_QH_TOKENS)
    UA_FAIL("ua_attn_bwd_dense_noalloc: %d tokens x %d heads exceeds the built-in scratch "
            "(at most %d tokens and tokens*heads <= %ld); use ua_attn_bwd with caller-owned scratch",
            tokens, n_heads, NOALLOC_MAX_TOKENS, NOALLOC_MAX_QH_TOKENS);
  int dev = 0;
  UA_CUDA(cudaGetDevice(&dev));
  if (dev >= 64) UA_FAIL("ua_attn_bwd_dense_noalloc: device index %d not supported", dev);
  if (g_noalloc_ptr[dev] == nullptr) {
    // one-time set-up for this device: resolve the device address of the scratch array
    void* p = nullptr;
    UA_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
  }
  unsigned char* base = g_noalloc_ptr[dev];
  float* dq32 = reinterpret_cast<float*>(base);
  BwdCol* col = reinterpret_cast<BwdCol*>(base + NOALLOC_COL_OFF);
  AttnSeg* seg = reinterpret_cast<AttnSeg*>(base + NOALLOC_SEG_OFF);
  int2* tiles = reinterpret_cast<int2*>(base + NOALLOC_TILE_OFF);
  const int n_tiles = (tokens + ATTN_TILE - 1) / ATTN_TILE;
  const long n_dq = static_cast<long>(tokens) * n_heads * ATTN_D;

  BwdParams p;
  memset(&p, 0, sizeof(p));
  UaTensorSrc tq = {q, tokens, n_heads, 1, static_cast<long>(n_heads) * ATTN_D, ATTN_D, 0};
  UaTensorSrc tdo = {d_o, tokens, n_heads, 1, static_cast<long>(n_heads) * ATTN_D, ATTN_D, 0};
  UaTensorSrc tk = {k, tokens, n_kv_heads, 1, static_cast<long>(n_kv_heads) * ATTN_D, ATTN_D, 0};
  UaTensorSrc tv = {v, tokens, n_kv_heads, 1, static_cast<long>(n_kv_heads) * ATTN_D, ATTN_D, 0};
  if (encode_src_box(&p.tmQ[0], tq, BWD_QT)) return -1;
  if (encode_src_box(&p.tmdO[0], tdo, BWD_QT)) return -1;
  if (encode_src_box(&p.tmK[0], tk, ATTN_TILE)) return -1;
  if (encode_src_box(&p.tmV[0], tv, ATTN_TILE)) return -1;
  {
    uint64_t dims[4] = {ATTN_D, static_cast<uint64_t>(n_heads), static_cast<uint64_t>(tokens), 1};
    uint64_t str[3] = {ATTN_D * 4ull, static_cast<uint64_t>(n_heads) * ATTN_D * 4,
                       static_cast<uint64_t>(n_dq) * 4};
    uint32_t box[4] = {128, 1, 16, 1};
    if (make_tmap_f32(&p.tmdQ[0], dq32, 4, dims, str, box)) return -1;
    p.dq_ptr[0] = dq32;
    p.dq_row_stride[0] = static_cast<long>(n_heads) * ATTN_D;
    p.dq_batch_stride[0] = n_dq;
  }
  p.lse_ptr[0] = lse;
  p.dvec_ptr[0] = dvec;
  p.lse_head_stride[0] = tokens;
  p.lse_batch_stride[0] = static_cast<long>(tokens) * n_heads;
  p.q_tokens[0] = tokens;
  p.dk_ptr[0] = dk;
  p.dv_ptr[0] = dv;
  p.dkv_row_stride[0] = static_cast<long>(n_kv_heads) * ATTN_D;
  p.dkv_batch_stride[0] = static_cast<long>(tokens) * n_kv_heads * ATTN_D;
  p.dkv_add_f32[0] = 0;
  p.cols = col;
  p.segs = seg;
  p.tiles = tiles;
  p.n_tiles = n_tiles;
  p.n_kv_heads = n_kv_heads;
  p.kv_group = n_heads / n_kv_heads;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  p.stage.tasks = nullptr;
  p.stage.n_tasks = 0;
  p.stage.n_copy_ctas = 0;
  p.stage.flags = nullptr;
  p.stage.epoch = 1;
  p.stage.ticket = nullptr;
  p.trace.buf = nullptr;
  p.trace.cap = 0;

  const int smem_bytes = sizeof(BwdSmem);
  if (!g_bwd_smem_set[dev]) {
    UA_CUDA(cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    g_bwd_smem_set[dev] = 1;
  }
  // the array keeps the previous call's contents: the accumulator has to start from zero
  UA_CUDA(cudaMemsetAsync(dq32, 0, static_cast<size_t>(n_dq) * 4, stream));
  noalloc_fill_tables<<<4, 256, 0, stream>>>(col, seg, tiles, tokens, causal ? 1 : 0);
  UA_CUDA(cudaGetLastError());
  dim3 grid(n_tiles * n_kv_heads, 1, 1);
  attn_bwd_kernel<<<grid, BWD_THREADS, smem_bytes, stream>>>(p);
  UA_CUDA(cudaGetLastError());
  long blocks = (n_dq / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  noalloc_cast_dq<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      dq32, static_cast<__nv_bfloat16*>(dq), n_dq);
  UA_CUDA(cudaGetLastError());
  return 0;
}
