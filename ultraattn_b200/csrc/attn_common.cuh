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
  int pad0, pad1, pad2;
};

}  // namespace ua
