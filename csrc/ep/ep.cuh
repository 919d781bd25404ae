// Parameter blocks shared by the expert-parallel (EP) kernels and their launchers.
//
// Vocabulary
//   rank mode   : one copy of a token per destination RANK (DeepEP normal-mode layout:
//                 recv_x[N_recv,H] + recv_topk_idx/weights). Items per token J = R,
//                 buckets B = R.
//   expert mode : one copy per (token, expert choice), receive rows already grouped by
//                 local expert (replaces the multihot/permute glue of
//                 `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:276-388`).
//                 J = K, B = E.
//   pos         : stable rank of an item inside its (source rank -> bucket) stream
//                 (token order), so layouts are deterministic.
//   row         : absolute row in the destination rank's receive region.
//   slot        : absolute row in the SOURCE rank's combine region where the result for
//                 that item is returned; slot = comb_base[bucket] + pos.
#pragma once
#include "../common.cuh"

namespace b200ep {

enum Channel : int {
  kChNotify = 0,
  kChDispatch = 1,
  kChCombine = 2,
  kChBarrier = 3,
  kChLLDispatch = 4,
  kChLLCombine = 5,
  kChLLPull = 6,      // low-latency combine, pull form: one arrival per call and rank
  kNumChannels = 8,
};

constexpr int kChunkTokens = 32;   // tokens per counting chunk (one warp of notify_send)
constexpr int kMaxItemsPerToken = 32;

// Byte offsets inside every rank's symmetric region (same on all ranks). Offsets of
// double-buffered regions are already resolved for this call's epoch parity by the host.
struct EpRegions {
  long long flags;         // int   [kNumChannels][kMaxRanks]
  long long counts;        // int   [R][R+E]      (this parity)
  long long recv_x;        // bytes [cap][row_bytes]
  long long recv_scales;   // float [cap][scale_cols]
  long long recv_topk_idx; // int64 [cap][K]
  long long recv_topk_w;   // float [cap][K]
  long long recv_meta;     // int2  [cap]  {slot at source, source rank}
  long long recv_prob;     // float [cap]
  long long comb_x;        // bytes [slot_cap][comb_row_bytes]
  long long comb_w;        // float [slot_cap][K]
  long long pull_info;     // int64 [kMaxRanks][4]: where rank d keeps the rows that a pulling combine reads
};

struct EpGeom {
  int rank, R, E, El, K, T;
  int mode;      // 0 = rank mode, 1 = expert mode
  int J, B;      // items per token, number of buckets
  int H;         // hidden size (elements)
  int cap;       // receive capacity in rows for this call
  int slot_cap;  // combine slot capacity for this call
  int epoch;     // flag value to publish (dispatch / combine epoch; notify epoch in notify_send)
  int epoch_wait;  // dispatch_send: notify epoch whose count vectors the prologue waits for
  int tail_wait;   // dispatch_send: 1 = the last CTA also waits for the peers' dispatch flags
  unsigned long long timeout_ns;
};

// Device-resident per-dispatch metadata (one int array, owned by the handle).
// Layout: [0]=N_recv  [1..1+El) recv per local expert  then prefix tables, see offsets.
struct EpMeta {
  int* n_recv;            // [1]
  int* recv_expert_cnt;   // [El]
  int* recv_expert_off;   // [El+1]  exclusive prefix of rows per local expert (expert mode)
  int* recv_src_off;      // [R+1]   exclusive prefix of rows per source rank (rank mode)
  int* send_base;         // [B]
  int* comb_base;         // [B]
  int* send_total;        // [1] number of slots used on this rank
};

}  // namespace b200ep
