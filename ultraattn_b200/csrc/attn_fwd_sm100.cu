// Block-sparse flash-attention forward for sm_100a: TMA-fed tcgen05.mma with S/P and O
// accumulators in tensor memory.
//
// Replaces, for this framework, the forward of the flash-attention fork that the reference calls
// at orchestrated_attn/orchestrated_attn_impl.py:326-337 (one call per scheduled tile) and the
// running-state Triton kernel at easy_context/dist_flash_attn/lightseq_async_attn.py:110-215.
// Differences by design: one launch walks a whole list of key/value segments per query block
// (carrying the running max / sum / O in registers and TMEM, so no merge kernel between tiles),
// segments may live in different buffers (own K/V, a staging ring, a peer GPU's memory reached
// through a unicast TMA tensor map), and the epilogue can either overwrite (O, lse) or merge into
// an existing partial (O, lse) — possibly a mailbox in a peer GPU's memory.
//
// CTA = 256 query rows x 1 head: two 128-row sub-tiles processed ping-pong so that the tensor
// core works on one sub-tile while the softmax warps work on the other. TPR = threads per query
// row (template parameter):
//   TPR = 1 (320 threads, default): warps 0-3 softmax / correction / epilogue for sub-tile 0 (one thread per
//            query row, 128 score columns each), warps 4-7 the same for sub-tile 1
//   TPR = 2 (640 threads, UA_FWD_TPR=2): two warpgroups per sub-tile; the two threads of a row take 64
//            score columns each (both can reach the row's TMEM lane), exchange their row maxima
//            through shared memory once per tile and each keep a partial row sum. The softmax of
//            a 128 x 128 tile is a chain of dependent latencies (TMEM load, max, exp2, pack, TMEM
//            store) that one warp per scheduler cannot hide; four warps per scheduler can. As
//            measured (S = 16k, 32 heads) this form is slower than TPR = 1 all the same, 876 against
//            1192 TFLOP/s: 104 registers per softmax thread leave spills in its inner loop and
//            the exchange adds a barrier per tile. It is kept as a tested variant.
//   then one TMA producer warp (Q once, then the K and V rings) and one tcgen05.mma issuer warp
//   (one elected thread; it also owns the TMEM allocation)
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P (bf16) overwrites the first
// 64 columns of its S region and is consumed from TMEM as the A operand of the PV product.
#include "attn_common.cuh"
#include "host_common.cuh"
#include "ptx.cuh"

namespace ua {

constexpr int FWD_KV_STAGES = 2;
template <int TPR> struct FwdCfg {
  static constexpr int SOFTMAX_WARPS = 8 * TPR;
  static constexpr int TMA_WARP = SOFTMAX_WARPS;
  static constexpr int MMA_WARP = SOFTMAX_WARPS + 1;
  // TPR = 2: five warpgroups (the last one: TMA, MMA and two idle warps), so that every scheduler
  // hosts the same number of warps and the register file can be re-balanced by warpgroup
  static constexpr int THREADS = TPR == 2 ? 640 : 32 * (SOFTMAX_WARPS + 2);
  static constexpr int NC = ATTN_TILE / TPR;      // score columns per thread
  // register split of the TPR = 2 form (see the role dispatch in the kernel)
  static constexpr int REGS_LAUNCH = 96, REGS_LOAD = 64, REGS_SOFTMAX = 104;
  static_assert(4 * REGS_SOFTMAX + REGS_LOAD <= 5 * REGS_LAUNCH, "setmaxnreg may only redistribute the launch-time pool");
};
#ifndef UA_FWD_POLY_EXP_PERIOD
#define UA_FWD_POLY_EXP_PERIOD 0
#endif
constexpr int FWD_POLY_EXP_PERIOD = UA_FWD_POLY_EXP_PERIOD;   // every n-th pair of exponentials is polynomial (0: none)
constexpr int FWD_TILE_BYTES = ATTN_TILE * ATTN_D * 2;  // 32 KB: [2 d-halves][128 rows][128 B]

struct FwdRow {
  int q_src;      // slot in tmQ
  int q_start;    // first query token inside that source
  int q_len;      // query tokens in this block row
  int seg_begin;  // [seg_begin, seg_end) into segs
  int seg_end;
  int o_slot;     // slot in the output tables
  int o_start;    // first output row inside that slot
  int accumulate; // 1: merge with the (O, lse) already stored there
  int q_wait_flag;   // staging flag of the query block (0: in place), see AttnSeg::wait_flag
  int q_wait_count;
};

struct FwdParams {
  CUtensorMap tmQ[ATTN_MAX_SRC];
  CUtensorMap tmK[ATTN_MAX_SRC];
  CUtensorMap tmV[ATTN_MAX_SRC];
  __nv_bfloat16* o_ptr[ATTN_MAX_SRC];
  float* lse_ptr[ATTN_MAX_SRC];
  long o_row_stride[ATTN_MAX_SRC];   // elements between consecutive tokens (Nh * D)
  long o_batch_stride[ATTN_MAX_SRC];
  long lse_head_stride[ATTN_MAX_SRC];
  long lse_batch_stride[ATTN_MAX_SRC];
  const FwdRow* rows;
  const AttnSeg* segs;
  const int2* tiles;   // (row index, 256-row tile index inside the row), heaviest first
  int n_tiles;
  int n_heads;
  int kv_group;        // query heads per key/value head
  float scale_log2;    // softmax scale * log2(e)
  int* status;
  StageParams stage;   // optional in-kernel staging of remote K/V (and Q) blocks
  KernelTrace trace;   // optional per-CTA time stamps
};

struct __align__(1024) FwdSmem {
  uint8_t q[2][FWD_TILE_BYTES];
  uint8_t k[FWD_KV_STAGES][FWD_TILE_BYTES];
  uint8_t v[FWD_KV_STAGES][FWD_TILE_BYTES];
  uint64_t q_full[2];
  uint64_t k_full[FWD_KV_STAGES];
  uint64_t k_empty[FWD_KV_STAGES];
  uint64_t v_full[FWD_KV_STAGES];
  uint64_t v_empty[FWD_KV_STAGES];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_full;
  uint32_t tmem_base;
  int abort_flag;
  int stage_slot;
  float xchg[2][2][ATTN_TILE];    // [sub-tile][column half][row]: row maxima / row sums exchanged between the two threads of a row
  uint64_t xbar[2];               // the 8 warps of a sub-tile meet here (an mbarrier, so that the wait is bounded)
};
static_assert(sizeof(FwdSmem) + 1024 <= 232448, "FwdSmem exceeds the 227 KB a CTA may use");

// Number of 128-key tiles of a segment that the 256-row tile starting at block-relative row r0
// has to visit (tiles entirely above the causal diagonal for both sub-tiles are skipped).
__device__ __forceinline__ int seg_tiles(const AttnSeg& sg, int r0, int rows_here) {
  int n = (sg.len + ATTN_TILE - 1) / ATTN_TILE;
  if (sg.causal) {
    const int last = r0 + rows_here - 1 + sg.diag;  // largest allowed key index
    if (last < 0) return 0;
    const int nc = last / ATTN_TILE + 1;
    n = nc < n ? nc : n;
  }
  return n;
}

// Optional pipeline trace (compile with -DUA_FWD_PROF): CTA (0, 0) records clock64() at the
// hand-over points of one key tile of every role into g_fwd_prof; ua_fwd_prof_read copies it out.
#ifdef UA_FWD_PROF
__device__ long long g_fwd_prof[64];
#define FWD_PROF(cond, slot) do { if ((cond) && blockIdx.x == 0 && blockIdx.y == 0) g_fwd_prof[slot] = clock64(); } while (0)
#else
#define FWD_PROF(cond, slot) do { } while (0)
#endif
constexpr int FWD_PROF_TILE = 8;


template <int TPR>
__global__ void __launch_bounds__(FwdCfg<TPR>::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ FwdParams p) {
  using Cfg = FwdCfg<TPR>;
  constexpr int NC = Cfg::NC;
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& s = *reinterpret_cast<FwdSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int head = blockIdx.x / p.n_tiles;
  const int2 tl = p.tiles[blockIdx.x % p.n_tiles];
  const int batch = blockIdx.y;
  const FwdRow row = p.rows[tl.x];
  const int cta_linear = blockIdx.y * gridDim.x + blockIdx.x;
  trace_stamp(p.trace, cta_linear, 0);
  trace_ident(p.trace, cta_linear, tl.x);
  {
    // does this CTA read a staged block? then it first helps to empty the copy queue
    bool waits = row.q_wait_flag != 0;
    for (int e = row.seg_begin; e < row.seg_end && !waits; ++e) waits = p.segs[e].wait_flag != 0;
    drain_stage_queue(p.stage, waits, cta_linear, &s.stage_slot);
  }
  trace_stamp(p.trace, cta_linear, 1);
  const int r0 = tl.y * 256;                                    // block-relative first row
  const int rows_here = min(256, row.q_len - r0);               // valid query rows of this CTA
  const int kv_head = head / p.kv_group;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s.q_full[i], 1);
      mbar_init(&s.s_full[i], 1);
      mbar_init(&s.p_full[i], 4 * TPR);     // one arrival per softmax warp
      mbar_init(&s.xbar[i], 8);
    }
    for (int i = 0; i < FWD_KV_STAGES; ++i) {
      mbar_init(&s.k_full[i], 1);
      mbar_init(&s.k_empty[i], 1);
      mbar_init(&s.v_full[i], 1);
      mbar_init(&s.v_empty[i], 1);
    }
    mbar_init(&s.o_full, 1);
    s.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == Cfg::MMA_WARP) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = s.tmem_base;
  WaitCtx wc{&s.abort_flag, p.status, 4000000000ull};

  // total number of key tiles this CTA visits (identical in every role)
  int n_total = 0;
  for (int e = row.seg_begin; e < row.seg_end; ++e) n_total += seg_tiles(p.segs[e], r0, rows_here);

  if (warp >= Cfg::SOFTMAX_WARPS) {
  // 20 warps are launched with 96 registers per thread, and that launch-time total (5 x 96 per
  // scheduler lane) is the whole pool that setmaxnreg can redistribute: an increase that asks for
  // more than the decreases have returned never completes. The last warpgroup (TMA, MMA, two idle
  // warps) goes down to 64 and the four softmax warpgroups, which hold 64 scores per thread, go up
  // to 104: 4 x 104 + 64 = 5 x 96. (The instruction sits inside the role's branch so that the
  // compiler budgets each role separately.)
  if constexpr (TPR == 2) reg_dealloc<FwdCfg<2>::REGS_LOAD>();
  if (warp == Cfg::TMA_WARP) {
    // =============================== TMA producer ===========================================
    if (lane == 0 && n_total > 0) {
      const CUtensorMap* tq = &p.tmQ[row.q_src];
      tma_prefetch_desc(tq);
      bool ok = true;
      if (!wait_staged(p.stage.flags, row.q_wait_flag, row.q_wait_count * p.stage.epoch, wc.budget_ns)) {
        report_error(wc, UA_ERR_FLAG_TIMEOUT, 110, row.q_wait_flag);
        ok = false;
      }
      for (int w = 0; w < 2 && ok; ++w) {
        mbar_arrive_expect_tx(&s.q_full[w], FWD_TILE_BYTES);
        const int qrow = row.q_start + r0 + w * ATTN_TILE;
        tma_load_4d(s.q[w], tq, &s.q_full[w], 0, head, qrow, batch);
        tma_load_4d(s.q[w] + 16384, tq, &s.q_full[w], 64, head, qrow, batch);
      }
      uint32_t j = 0;
      for (int e = row.seg_begin; e < row.seg_end && ok; ++e) {
        const AttnSeg sg = p.segs[e];
        const int nt = seg_tiles(sg, r0, rows_here);
        const CUtensorMap* tk = &p.tmK[sg.src];
        const CUtensorMap* tv = &p.tmV[sg.src];
        if (nt > 0 && !wait_staged(p.stage.flags, sg.wait_flag, sg.wait_count * p.stage.epoch, wc.budget_ns)) {
          report_error(wc, UA_ERR_FLAG_TIMEOUT, 111, sg.wait_flag);
          ok = false;
          break;
        }
        for (int t = 0; t < nt; ++t, ++j) {
          const int st = j % FWD_KV_STAGES;
          const uint32_t ph = (j / FWD_KV_STAGES) & 1;
          const int krow = sg.start + t * ATTN_TILE;
          if (!mbar_wait(&s.k_empty[st], ph ^ 1, wc, 100)) { ok = false; break; }
          mbar_arrive_expect_tx(&s.k_full[st], FWD_TILE_BYTES);
          tma_load_4d(s.k[st], tk, &s.k_full[st], 0, kv_head, krow, batch);
          tma_load_4d(s.k[st] + 16384, tk, &s.k_full[st], 64, kv_head, krow, batch);
          if (!mbar_wait(&s.v_empty[st], ph ^ 1, wc, 101)) { ok = false; break; }
          mbar_arrive_expect_tx(&s.v_full[st], FWD_TILE_BYTES);
          tma_load_4d(s.v[st], tv, &s.v_full[st], 0, kv_head, krow, batch);
          tma_load_4d(s.v[st] + 16384, tv, &s.v_full[st], 64, kv_head, krow, batch);
        }
      }
    }
  } else if (warp == Cfg::MMA_WARP) {
    // =============================== MMA issuer =============================================
    if (lane == 0 && n_total > 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S = Q K^T, both K-major
      const uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);   // O += P V, V is N-major
      const uint32_t tS[2] = {tmem_base + 0, tmem_base + 128};
      const uint32_t tO[2] = {tmem_base + 256, tmem_base + 384};
      auto issue_s = [&](int w, int st) {
        const uint32_t qa = smem_u32(s.q[w]);
        const uint32_t ka = smem_u32(s.k[st]);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_ss(tS[w], make_smem_desc_sw128(qa + off, 16, 1024),
                  make_smem_desc_sw128(ka + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int w, int st, bool acc) {
        const uint32_t va = smem_u32(s.v[st]);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A: 16 keys = 8 packed columns of P; B: 16 key rows = 2048 B, d-halves 16384 B apart
          umma_ts(tO[w], tS[w] + kk * 8, make_smem_desc_sw128(va + kk * 2048, 16384, 1024),
                  idesc_o, (acc || kk > 0) ? 1u : 0u);
        }
      };
      bool ok = true;
      do {
        if (!mbar_wait(&s.q_full[0], 0, wc, 200)) { ok = false; break; }
        if (!mbar_wait(&s.k_full[0], 0, wc, 201)) { ok = false; break; }
        tc_fence_after_sync();
        issue_s(0, 0);
        tc_commit(&s.s_full[0]);
        if (!mbar_wait(&s.q_full[1], 0, wc, 202)) { ok = false; break; }
        tc_fence_after_sync();
        issue_s(1, 0);
        tc_commit(&s.s_full[1]);
        tc_commit(&s.k_empty[0]);
        for (int j = 0; j < n_total; ++j) {
          const int st = j % FWD_KV_STAGES;
          const uint32_t ph = (j / FWD_KV_STAGES) & 1;
          const int stn = (j + 1) % FWD_KV_STAGES;
          const uint32_t phn = ((j + 1) / FWD_KV_STAGES) & 1;
          const bool more = (j + 1 < n_total);
          FWD_PROF(j == FWD_PROF_TILE, 0);
          if (!mbar_wait(&s.v_full[st], ph, wc, 203)) { ok = false; break; }
          if (!mbar_wait(&s.p_full[0], j & 1, wc, 204)) { ok = false; break; }
          FWD_PROF(j == FWD_PROF_TILE, 1);
          tc_fence_after_sync();
          issue_pv(0, st, j > 0);
          if (more) {
            if (!mbar_wait(&s.k_full[stn], phn, wc, 205)) { ok = false; break; }
            tc_fence_after_sync();
            issue_s(0, stn);
            tc_commit(&s.s_full[0]);
          }
          FWD_PROF(j == FWD_PROF_TILE, 2);
          if (!mbar_wait(&s.p_full[1], j & 1, wc, 206)) { ok = false; break; }
          FWD_PROF(j == FWD_PROF_TILE, 3);
          tc_fence_after_sync();
          issue_pv(1, st, j > 0);
          tc_commit(&s.v_empty[st]);
          if (more) {
            issue_s(1, stn);
            tc_commit(&s.s_full[1]);
            tc_commit(&s.k_empty[stn]);
          }
          FWD_PROF(j == FWD_PROF_TILE, 4);
        }
        if (ok) tc_commit(&s.o_full);
      } while (false);
      (void)ok;
    }
  }
  } else {
    // =============================== softmax + epilogue =====================================
    if constexpr (TPR == 2) reg_alloc<FwdCfg<2>::REGS_SOFTMAX>();
    const int w = warp / (4 * TPR);          // sub-tile
    const int part = (warp >> 2) % TPR;      // which NC-column slice of the row this thread handles
    const int quad = warp & 3;               // TMEM lane quadrant of this warp
    const int r_tile = quad * 32 + lane;     // row inside the 128-row sub-tile
    const int r_blk = r0 + w * ATTN_TILE + r_tile;   // row inside the query block
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + w * 128;
    const uint32_t tSp = tS + part * NC;             // this thread's score columns
    const uint32_t tPp = tS + part * (NC / 2);       // ... and where its packed probabilities go
    const uint32_t tO = tmem_base + lane_base + 256 + w * 128;
    const float NEG_INF = -INFINITY;

    uint32_t xph = 0;        // phase of the sub-tile's exchange barrier
    // all 256 threads of the sub-tile have passed this point (bounded like every other wait)
    auto subtile_sync = [&]() -> bool {
      mbar_arrive_warp(&s.xbar[w]);
      const bool good = mbar_wait(&s.xbar[w], xph & 1, wc, 330 + w);
      ++xph;
      return good;
    };
    float m_use = NEG_INF;   // running reference max, log2 units (already scaled); identical in both threads of a row
    float l = 0.f;           // row sum over this thread's columns
    bool ok = true;
    uint32_t j = 0;
    for (int e = row.seg_begin; e < row.seg_end && ok; ++e) {
      const AttnSeg sg = p.segs[e];
      const int nt = seg_tiles(sg, r0, rows_here);
      for (int t = 0; t < nt; ++t, ++j) {
        const bool prof = (j == FWD_PROF_TILE || j == FWD_PROF_TILE + 1) && quad == 0 && lane == 0 && part == 0;
        const int pslot = 8 + w * 24 + (static_cast<int>(j) - FWD_PROF_TILE) * 8;
        (void)prof; (void)pslot;
        FWD_PROF(prof, pslot + 0);
        if (!__all_sync(0xFFFFFFFFu, mbar_wait(&s.s_full[w], j & 1, wc, 300 + w))) { ok = false; break; }
        FWD_PROF(prof, pslot + 1);
        tc_fence_after_sync();
        float sv[NC];
        {
          uint32_t(&raw)[NC] = reinterpret_cast<uint32_t(&)[NC]>(sv);
#pragma unroll
          for (int c = 0; c < NC / 32; ++c)
            tmem_ld_x32(tSp + c * 32, reinterpret_cast<uint32_t(&)[32]>(raw[c * 32]));
          tmem_wait_ld();
        }
        FWD_PROF(prof, pslot + 2);
        // masking: key index c (segment-relative) allowed iff c < len and (c <= r + diag)
        const int c0 = t * ATTN_TILE + part * NC;
        int limit = sg.len - c0;                               // columns < limit are in range
        if (sg.causal) limit = min(limit, r_blk + sg.diag - c0 + 1);
        if (limit < NC) {
#pragma unroll
          for (int i = 0; i < NC; ++i) sv[i] = (i < limit) ? sv[i] : NEG_INF;
        }
        // eight independent running maxima, two new values per instruction: one dependent chain of
        // compares would cost more than the exponentials
        float mx8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(sv[i], sv[8 + i]);
#pragma unroll
        for (int i = 16; i < NC; i += 16)
#pragma unroll
          for (int k = 0; k < 8; ++k) mx8[k] = fmax3(mx8[k], sv[i + k], sv[i + 8 + k]);
        float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]));
        mx = fmax3(mx, mx8[6], mx8[7]);
        if constexpr (TPR == 2) {
          // the row maximum over all 128 columns: exchange with the thread that holds the other half.
          // (The slot is free again: its reader of the previous tile arrived at p_full before the
          // products this tile's scores waited for could be issued.)
          s.xchg[w][part][r_tile] = mx;
          if (!__all_sync(0xFFFFFFFFu, subtile_sync())) { ok = false; break; }
          mx = fmaxf(mx, s.xchg[w][part ^ 1][r_tile]);
        }
        mx *= p.scale_log2;
        const float m_new = fmaxf(m_use, mx);
        // lazy rescale: only when the running max grew by more than 2^8 (warp-uniform branch,
        // because the TMEM accesses below are warp-collective)
        const bool need = (m_new - m_use > 8.0f) || (m_use == NEG_INF && m_new > NEG_INF);
        if (j == 0) {
          m_use = m_new;
        } else if (__any_sync(0xFFFFFFFFu, need)) {
          const float alpha = need ? fast_exp2(m_use - m_new) : 1.0f;
          if (need) m_use = m_new;
          l *= alpha;
          // each thread of the row rescales its share of the 128 output columns
#pragma unroll 1
          for (int c = part * (4 / TPR); c < (part + 1) * (4 / TPR); ++c) {
            uint32_t ov[32];
            tmem_ld_x32(tO + c * 32, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_x32(tO + c * 32, ov);
          }
        }
        FWD_PROF(prof, pslot + 3);
        const float m_eff = (m_use == NEG_INF) ? 0.f : m_use;
        // multiply-add and row sum on packed pairs; four independent partial sums
        const uint64_t sc2 = f2_pack(p.scale_log2, p.scale_log2);
        const uint64_t nm2 = f2_pack(-m_eff, -m_eff);
        uint64_t ls2[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) ls2[k] = f2_pack(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < NC / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1;
            f2_unpack(f2_fma(f2_pack(sv[c * 32 + 2 * i], sv[c * 32 + 2 * i + 1]), sc2, nm2), x0, x1);
            // optionally one pair in every FWD_POLY_EXP_PERIOD runs on the FMA pipe (packed cubic)
            const bool poly = FWD_POLY_EXP_PERIOD > 0 && (i % (FWD_POLY_EXP_PERIOD > 0 ? FWD_POLY_EXP_PERIOD : 1)) == (FWD_POLY_EXP_PERIOD > 0 ? FWD_POLY_EXP_PERIOD : 1) - 1;
            float p0, p1;
            if (poly) {
              f2_unpack(poly_exp2_x2(x0, x1), p0, p1);
            } else {
              p0 = fast_exp2(x0);
              p1 = fast_exp2(x1);
            }
            ls2[i & 3] = f2_add(ls2[i & 3], f2_pack(p0, p1));
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st_x16(tPp + c * 16, pk);
        }
        float ls4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float a, b;
          f2_unpack(ls2[k], a, b);
          ls4[k] = a + b;
        }
        l += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        FWD_PROF(prof, pslot + 4);
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive_warp(&s.p_full[w]);
        FWD_PROF(prof, pslot + 5);
      }
    }
    if constexpr (TPR == 2) {
      // the row sum over all columns (m_use is the same in both threads)
      if (ok) ok = __all_sync(0xFFFFFFFFu, subtile_sync());      // the last exchange of maxima has been read
      s.xchg[w][part][r_tile] = l;
      if (ok) ok = __all_sync(0xFFFFFFFFu, subtile_sync());
      l += s.xchg[w][part ^ 1][r_tile];
    }

    // ---------------------------------- epilogue --------------------------------------------
    const bool valid_row = (w * ATTN_TILE + r_tile) < rows_here;
    const long orow = static_cast<long>(row.o_start + r_blk);
    __nv_bfloat16* optr = p.o_ptr[row.o_slot] + batch * p.o_batch_stride[row.o_slot] +
                          orow * p.o_row_stride[row.o_slot] + static_cast<long>(head) * ATTN_D;
    float* lptr = p.lse_ptr[row.o_slot] + batch * p.lse_batch_stride[row.o_slot] +
                  head * p.lse_head_stride[row.o_slot] + orow;
    if (n_total > 0 && ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait(&s.o_full, 0, wc, 310 + w));
    tc_fence_after_sync();
    float lse = NEG_INF;
    float inv = 0.f;
    // (a row whose keys were all masked has m_use = -inf; the polynomial exponential leaves about
    // 2^-126 per masked entry in l, which must not count as probability mass)
    if (n_total > 0 && l > 0.f && m_use > NEG_INF) {
      lse = (m_use + log2f(l)) * 0.6931471805599453f;
      inv = 1.0f / l;
    }
    float w_old = 0.f, w_new = 1.f;
    float lse_old = NEG_INF;
    if (row.accumulate) {
      if (valid_row) lse_old = *lptr;
      // (both threads of a row have read the old lse before one of them overwrites it below)
      if constexpr (TPR == 2) { if (ok) ok = __all_sync(0xFFFFFFFFu, subtile_sync()); }
    }
    if (row.accumulate && valid_row) {
      const float mx = fmaxf(lse_old, lse);
      if (mx == NEG_INF) {
        w_old = 0.f; w_new = 0.f;
      } else {
        const float eo = __expf(lse_old - mx), en = __expf(lse - mx);
        const float tot = eo + en;
        w_old = eo / tot; w_new = en / tot;
        lse = mx + __logf(tot);
      }
    }
    const float fnew = inv * w_new;
#pragma unroll 1
    for (int c = part * (4 / TPR); c < (part + 1) * (4 / TPR); ++c) {
      uint32_t ov[32];
      if (n_total > 0) {
        tmem_ld_x32(tO + c * 32, ov);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) ov[i] = 0u;
      }
      if (valid_row) {
        uint4* d4 = reinterpret_cast<uint4*>(optr + c * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = (fnew == 0.f) ? 0.f : __uint_as_float(ov[q * 8 + i]) * fnew;
          if (row.accumulate) {
            const uint4 old = d4[q];
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float lo = __uint_as_float(ow[i] << 16);
              const float hi = __uint_as_float(ow[i] & 0xFFFF0000u);
              f[2 * i] += w_old * lo;
              f[2 * i + 1] += w_old * hi;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]);
          o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]);
          o.w = pack_bf16x2(f[6], f[7]);
          d4[q] = o;
        }
      }
    }
    if (valid_row && part == 0) *lptr = lse;
  }

  tc_fence_before_sync();
  __syncthreads();
  trace_stamp(p.trace, cta_linear, 2);
  if (warp == Cfg::MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ua

using namespace ua;

// Register (or, with buf = NULL, remove) the per-CTA trace buffer of the current device:
// which = 0 forward, 1 backward; buf = 4 * cap 64-bit words of device memory (see KernelTrace).
extern "C" int ua_set_kernel_trace(int which, unsigned long long* buf, int cap) {
  int dev = 0;
  UA_CUDA(cudaGetDevice(&dev));
  if (which < 0 || which > 1 || dev >= 64) UA_FAIL("ua_set_kernel_trace: bad kernel or device index");
  trace_registry()[which * 64 + dev] = TraceSlot{buf, buf != nullptr ? cap : 0};
  return 0;
}

// Hits and misses of the host-side tensor-map cache since the library was loaded.
extern "C" int ua_tmap_cache_stats(unsigned long long* hits, unsigned long long* misses) {
  TmapCache& c = tmap_cache();
  while (c.busy.test_and_set(std::memory_order_acquire)) {}
  *hits = c.hits;
  *misses = c.misses;
  c.busy.clear(std::memory_order_release);
  return 0;
}

#ifdef UA_FWD_PROF
extern "C" int ua_fwd_prof_read(long long* host64) {
  UA_CUDA(cudaMemcpyFromSymbol(host64, g_fwd_prof, sizeof(long long) * 64));
  return 0;
}
#endif

// Host-side description of one tensor source: [batch, tokens, heads, 128] bf16 with the given
// strides (elements).
struct UaTensorSrc {
  const void* ptr;
  long tokens;
  long heads;
  long batch;
  long token_stride;
  long head_stride;
  long batch_stride;
};
struct UaOutDst {
  void* o_ptr;
  float* lse_ptr;
  long o_row_stride;
  long o_batch_stride;
  long lse_head_stride;
  long lse_batch_stride;
};

static int encode_src(CUtensorMap* tm, const UaTensorSrc& t) {
  uint64_t dims[4] = {ATTN_D, static_cast<uint64_t>(t.heads), static_cast<uint64_t>(t.tokens),
                      static_cast<uint64_t>(t.batch)};
  uint64_t str[3] = {static_cast<uint64_t>(t.head_stride) * 2,
                     static_cast<uint64_t>(t.token_stride) * 2,
                     static_cast<uint64_t>(t.batch_stride > 0 ? t.batch_stride : t.token_stride * t.tokens) * 2};
  uint32_t box[4] = {64, 1, ATTN_TILE, 1};
  return make_tmap_2byte(tm, t.ptr, 4, dims, str, box);
}

static int g_fwd_smem_set[2][64] = {{0}};

// rows / segs / tiles are device pointers (prepared once per plan); q/k/v/out tables are host
// arrays of n_q / n_kv / n_out entries.
extern "C" int ua_attn_fwd(const UaTensorSrc* q_src, int n_q, const UaTensorSrc* k_src,
                           const UaTensorSrc* v_src, int n_kv, const UaOutDst* outs, int n_out,
                           const void* rows_dev, const void* segs_dev, const void* tiles_dev,
                           int n_tiles, int n_heads, int n_kv_heads, int batch,
                           float softmax_scale, int* status, const void* copy_tasks_dev,
                           int n_copy_tasks, int n_copy_ctas, unsigned int* stage_flags,
                           int stage_epoch, unsigned int* stage_ticket, cudaStream_t stream) {
  if (n_q > ATTN_MAX_SRC || n_kv > ATTN_MAX_SRC || n_out > ATTN_MAX_SRC)
    UA_FAIL("ua_attn_fwd: too many sources (max %d)", ATTN_MAX_SRC);
  if (n_tiles <= 0) return 0;
  FwdParams p;
  memset(&p, 0, sizeof(p));
  for (int i = 0; i < n_q; ++i)
    if (encode_src(&p.tmQ[i], q_src[i])) return -1;
  for (int i = 0; i < n_kv; ++i) {
    if (encode_src(&p.tmK[i], k_src[i])) return -1;
    if (encode_src(&p.tmV[i], v_src[i])) return -1;
  }
  for (int i = 0; i < n_out; ++i) {
    p.o_ptr[i] = static_cast<__nv_bfloat16*>(outs[i].o_ptr);
    p.lse_ptr[i] = outs[i].lse_ptr;
    p.o_row_stride[i] = outs[i].o_row_stride;
    p.o_batch_stride[i] = outs[i].o_batch_stride;
    p.lse_head_stride[i] = outs[i].lse_head_stride;
    p.lse_batch_stride[i] = outs[i].lse_batch_stride;
  }
  p.rows = static_cast<const FwdRow*>(rows_dev);
  p.segs = static_cast<const AttnSeg*>(segs_dev);
  p.tiles = static_cast<const int2*>(tiles_dev);
  p.n_tiles = n_tiles;
  p.n_heads = n_heads;
  p.kv_group = n_heads / n_kv_heads;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  p.stage.tasks = static_cast<const CopyTask*>(copy_tasks_dev);
  p.stage.n_tasks = n_copy_tasks;
  {
    const long grid_ctas = static_cast<long>(n_tiles) * n_heads * batch;
    p.stage.n_copy_ctas = static_cast<int>(n_copy_ctas < grid_ctas ? n_copy_ctas : grid_ctas);
  }
  p.stage.flags = stage_flags;
  p.stage.epoch = stage_epoch;
  p.stage.ticket = stage_ticket;
  {
    int tdev = 0;
    UA_CUDA(cudaGetDevice(&tdev));
    const TraceSlot ts = tdev < 64 ? trace_registry()[0 * 64 + tdev] : TraceSlot{nullptr, 0};
    p.trace.buf = ts.buf;
    p.trace.cap = ts.cap;
  }
  if (n_copy_tasks > 0) {
    if (stage_ticket == nullptr) UA_FAIL("ua_attn_fwd: copy tasks need a ticket counter");
    UA_CUDA(cudaMemsetAsync(stage_ticket, 0, sizeof(unsigned int), stream));
  }
  const int smem_bytes = sizeof(FwdSmem) + 1024;
  int dev = 0;
  UA_CUDA(cudaGetDevice(&dev));
  // UA_FWD_TPR = 1 / 2: softmax threads per query row (see the top of this file)
  const char* env = getenv("UA_FWD_TPR");
  const int tpr = (env != nullptr && atoi(env) == 2) ? 2 : 1;
  if (dev < 64 && !g_fwd_smem_set[tpr - 1][dev]) {
    if (tpr == 2)
      UA_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    else
      UA_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    g_fwd_smem_set[tpr - 1][dev] = 1;
  }
  dim3 grid(n_tiles * n_heads, batch, 1);
  if (tpr == 2)
    attn_fwd_kernel<2><<<grid, FwdCfg<2>::THREADS, smem_bytes, stream>>>(p);
  else
    attn_fwd_kernel<1><<<grid, FwdCfg<1>::THREADS, smem_bytes, stream>>>(p);
  UA_CUDA(cudaGetLastError());
  return 0;
}
