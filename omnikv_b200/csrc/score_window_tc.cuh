// Window-selector scores on tcgen05 tensor cores (score_window_tc.cu): interface to omnikv_score_window.
#pragma once

#include "common.cuh"

namespace omnikv {

constexpr int kWindowTcMaxSplits = 64;

struct WinTcArgs {
  const void* qw;              // [B, H, W, d]
  const int* consider_len;     // device [B]
  float* part;                 // [B][H][16][S][2]  pass-1 partials (offset, sum), log2 domain
  float* tplane;               // [B][16][tplane_stride] running max over heads per window slot (log domain), between
                               // the launches of pass 2
  int64_t tplane_stride;
  float* score_out;            // [B, score_stride] or nullptr
  float* planes_out;           // [B, W, score_stride] or nullptr (max over the local heads per slot)
  int64_t score_stride;
  int B, H, KVH, G, W, S, selector, n_sms;
  float scale;
  int* status;
};

// Whether the tensor-memory path covers this head grouping (the query blocks of all KV heads must fit in shared
// memory beside the K ring; a thread holds one accumulator row of 16 G columns in registers).
bool window_tc_supported(int G, int KVH);
int window_tc_splits(int B, int KVH, int n_sms, int max_len);
int window_tc_launches(int G, int KVH);  // kernels one call launches
// tm_k: tensor map over the K cache [B, KVH, rows, 128] with boxes of 64 elements x 128 rows, 128-byte swizzle.
int window_tc_launch(int dtype, const WinTcArgs& a, const CUtensorMap& tm_k, int max_len, cudaStream_t st);

}  // namespace omnikv
