// Window-selector scores ("uniform" / "exp" / "softmax_before_last").
//
//   A[h,w,p]  = softmax over p' < C of (qw[h,w,:] . K[h/G,p',:] * scale)
//   score[p]  = sum_w weight_w * max_h A[h,w,p]
//
// The softmax normaliser of every (head, window slot) row has to be known before the max over
// heads, so K is streamed twice:
//   pass 1  grid (splits, KVH, B): per-row online (max, sum-exp) of the CTA's chunk of keys;
//           a small kernel merges the splits into (m, 1/l) per row;
//   pass 2  grid (chunks of 512 positions, KVH, B): a CTA normalises the logits of one KV head's query group
//           for its chunk, takes the max over the group's heads in registers and folds it into per-slot
//           planes with integer atomicMax (weights are >= 0; max is order independent: deterministic);
//           a small kernel then forms the weighted sum over the window slots.
// The [G x 16 window slots] x 128 query block of one KV head against a tile of keys is a dense
// contraction: bf16/fp16 run it on m16n8k16 tensor-core MMAs with the K tile staged by cp.async;
// fp32 uses CUDA cores.  Query rows are laid out head-major with the window padded to 16 slots,
// so one MMA m-tile is one head and the max over heads is a max over a thread's own accumulators.
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"
#include "score_window_tc.cuh"

namespace omnikv {
namespace {

constexpr int TILE = 64;
constexpr int NWARPS = 4;
constexpr int NTHREADS = NWARPS * 32;
constexpr int PITCH = 272;
constexpr int TILE_BYTES = TILE * PITCH;
constexpr int WPAD = 16;  // window slots per head after padding
constexpr int P1_STAGES = 3;
constexpr int P2_STAGES = 3;

// workspace layout: [pass-1 partials][merged statistics][per-slot planes]
size_t part_floats(int B, int H, int S) { return (size_t)B * H * WPAD * S * 2; }
size_t stats_floats(int B, int H) { return (size_t)B * H * WPAD * 2; }
size_t plane_stride_of(int max_len) { return (size_t)ceil_div(max_len, 4) * 4; }
size_t plane_floats(int B, int W, int max_len) { return (size_t)B * W * plane_stride_of(max_len); }

struct WinArgs {
  const void* qw;
  const void* k;
  int64_t k_sb, k_sh, k_sr;
  const int* consider_len;
  float* part;    // [B][H][WPAD][S][2]  pass-1 partial (m, l)
  float* stats;   // [B][H][WPAD][2]     (m, 1/l)
  float* score_out;
  float* planes_out;
  int64_t score_stride;
  float* planes;        // [B][W][plane_stride] max over heads per window slot (zero before pass 2)
  int64_t plane_stride;
  int B, H, KVH, G, W, S, selector, chunk2;
  float scale;
  int* status;          // device word for bounded-wait failures, or nullptr
};

__device__ __forceinline__ void split_range(int n, int S, int split, int& r0, int& r1) {
  int chunk = ceil_div(ceil_div(n, S), TILE) * TILE;
  r0 = split * chunk;
  r1 = min(n, r0 + chunk);
}

// K tile (64 rows of one KV head) -> padded shared-memory rows.
template <typename T>
__device__ __forceinline__ void issue_k_tile(unsigned char* dst, const T* kbase, int64_t k_sr, int row0, int r1, int tid) {
  const int cc = tid & 15, rowi = tid >> 4;
#pragma unroll
  for (int i = 0; i < TILE / 8; ++i) {
    const int row = rowi + 8 * i;
    const int R = row0 + row;
    const bool valid = R < r1;
    const T* src = valid ? kbase + (size_t)R * k_sr : kbase;
    cp_async16(dst + row * PITCH + cc * 16, src + cc * 8, valid);
  }
}

// The same tile through the tensor map: two boxes of 64 rows x 128 bytes, issued by ONE thread.
constexpr int TMA_TILE_BYTES = 2 * kTmaBoxBytes;
__device__ __forceinline__ void issue_k_tile_tma(unsigned char* dst, const CUtensorMap* map, int row0, int kvh, int b,
                                                 uint64_t* bar) {
  mbar_expect_tx(bar, TMA_TILE_BYTES);
  tma_load_4d(dst, map, 0, row0, kvh, b, bar);
  tma_load_4d(dst + kTmaBoxBytes, map, 64, row0, kvh, b, bar);
}

// Query rows of `nheads` heads starting at head h0 -> shared memory [nheads*16][PITCH], slots >= W zero.
template <typename T>
__device__ __forceinline__ void load_q(unsigned char* q_s, const T* qw_b, int h0, int nheads, int W, int tid) {
  // batches of eight loads, then their stores: written as load, store, load, store ... every iteration would
  // cost a round trip (the compiler keeps a load behind an earlier store through a generic pointer)
  const int total = nheads * WPAD * 16;
  for (int base = 0; base < total; base += 8 * NTHREADS) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + tid + u * NTHREADS;
      const int c = i & 15, r = i >> 4;
      const int hl = r / WPAD, w = r % WPAD;
      v[u] = make_uint4(0, 0, 0, 0);
      if (i < total && w < W) v[u] = *reinterpret_cast<const uint4*>(qw_b + ((size_t)(h0 + hl) * W + w) * kHeadDim + c * 8);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + tid + u * NTHREADS;
      if (i < total) *reinterpret_cast<uint4*>(q_s + (i >> 4) * PITCH + (i & 15) * 16) = v[u];
    }
  }
}

// acc[i][j][e]: head i of the group, n-tile j (8 keys), e as in the m16n8 C fragment
// (row g + 8*(e>>1) = window slot, column 2t + (e&1) = key).
template <typename T, int G, bool TMA>
__device__ __forceinline__ void qk_tile(float (&acc)[G][2][4], const unsigned char* q_s, const unsigned char* ks,
                                        int warp, int lane) {
  const int mi = lane >> 3;
#pragma unroll
  for (int i = 0; i < G; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    unsigned kf[4];
    const int krow = warp * 16 + 8 * (mi >> 1) + (lane & 7), kcolb = (kk * 16 + 8 * (mi & 1)) * 2;
    ldmatrix_x4(kf, TMA ? swz128(ks, krow, kcolb) : ks + krow * PITCH + kcolb);
#pragma unroll
    for (int i = 0; i < G; ++i) {
      unsigned qa[4];
      ldmatrix_x4(qa, q_s + (i * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * PITCH + (kk * 16 + 8 * (lane >> 4)) * 2);
      mma_16816<T>(acc[i][0], qa, kf[0], kf[1]);
      mma_16816<T>(acc[i][1], qa, kf[2], kf[3]);
    }
  }
}

__device__ __forceinline__ void merge_ml(float& m, float& l, float m2, float l2) {
  const float M = fmaxf(m, m2);
  const float Mu = (M == -INFINITY) ? 0.f : M;
  l = l * exp2f((m - Mu) * kLog2e) + l2 * exp2f((m2 - Mu) * kLog2e);
  m = M;
}

// ---- pass 1: per-row (max, sum-exp) over the CTA's chunk -------------------------------------
template <typename T, int G, bool TMA>
__global__ void __launch_bounds__(NTHREADS, 3) window_pass1_mma(const WinArgs a, const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[P1_STAGES];
  constexpr int KT = TMA ? TMA_TILE_BYTES : TILE_BYTES;  // bytes of a staged K tile
  unsigned char* smem = TMA ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023)
                            : smem_raw;
  unsigned char* q_s = smem + P1_STAGES * KT;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n = a.consider_len[b];
  int r0, r1;
  split_range(n, a.S, split, r0, r1);
  const int ntiles = r1 > r0 ? ceil_div(r1 - r0, TILE) : 0;
  const T* kbase = static_cast<const T*>(a.k) + (size_t)b * a.k_sb + (size_t)kvh * a.k_sh;

  if constexpr (TMA) {
    if (tid == 0) {
#pragma unroll
      for (int s = 0; s < P1_STAGES; ++s) mbar_init(&full_bar[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
#pragma unroll
      for (int s = 0; s < P1_STAGES - 1; ++s)
        if (s < ntiles) issue_k_tile_tma(smem + s * KT, &tm_k, r0 + s * TILE, kvh, b, &full_bar[s]);
    }
  } else {
#pragma unroll
    for (int s = 0; s < P1_STAGES - 1; ++s) {
      if (s < ntiles) issue_k_tile<T>(smem + s * KT, kbase, a.k_sr, r0 + s * TILE, r1, tid);
      cp_async_commit();
    }
  }
  load_q<T>(q_s, static_cast<const T*>(a.qw) + (size_t)b * a.H * a.W * kHeadDim, kvh * G, G, a.W, tid);
  __syncthreads();

  float m[G][2], l[G][2];
#pragma unroll
  for (int i = 0; i < G; ++i) m[i][0] = m[i][1] = -INFINITY, l[i][0] = l[i][1] = 0.f;

  for (int tile = 0; tile < ntiles; ++tile) {
    {
      const int nt = tile + P1_STAGES - 1;
      if constexpr (TMA) {
        __syncthreads();  // every thread is done with tile - 1: its slot may be refilled
        if (tid == 0 && nt < ntiles)
          issue_k_tile_tma(smem + (nt % P1_STAGES) * KT, &tm_k, r0 + nt * TILE, kvh, b, &full_bar[nt % P1_STAGES]);
        if (!mbar_wait(&full_bar[tile % P1_STAGES], (tile / P1_STAGES) & 1) && a.status) atomicExch(a.status, 5);
      } else {
        cp_async_wait<P1_STAGES - 2>();
        __syncthreads();
        if (nt < ntiles) issue_k_tile<T>(smem + (nt % P1_STAGES) * KT, kbase, a.k_sr, r0 + nt * TILE, r1, tid);
        cp_async_commit();
      }
    }
    float acc[G][2][4];
    qk_tile<T, G, TMA>(acc, q_s, smem + (tile % P1_STAGES) * KT, warp, lane);
    const int cbase = r0 + tile * TILE + warp * 16 + 2 * t;
#pragma unroll
    for (int i = 0; i < G; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int R = cbase + 8 * j + e;
            v[2 * j + e] = (R < r1) ? acc[i][j][2 * h + e] * a.scale : -INFINITY;
          }
        const float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
        const float M = fmaxf(m[i][h], mx);
        const float Mu = (M == -INFINITY) ? 0.f : M;
        const float ml2 = Mu * kLog2e;
        l[i][h] = l[i][h] * exp2f((m[i][h] - Mu) * kLog2e) +
                  ((exp2f(fmaf(v[0], kLog2e, -ml2)) + exp2f(fmaf(v[1], kLog2e, -ml2))) +
                   (exp2f(fmaf(v[2], kLog2e, -ml2)) + exp2f(fmaf(v[3], kLog2e, -ml2))));
        m[i][h] = M;
      }
  }
  cp_async_wait<0>();
  __syncthreads();
  // merge over the 4 key-lanes of a row, then over warps
  float* ml_s = reinterpret_cast<float*>(smem);  // [NWARPS][G*16][2]
#pragma unroll
  for (int i = 0; i < G; ++i)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int off = 1; off <= 2; off <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m[i][h], off);
        const float l2 = __shfl_xor_sync(0xffffffffu, l[i][h], off);
        merge_ml(m[i][h], l[i][h], m2, l2);
      }
      if (t == 0) {
        const int r = i * 16 + g + 8 * h;
        ml_s[(warp * G * 16 + r) * 2 + 0] = m[i][h];
        ml_s[(warp * G * 16 + r) * 2 + 1] = l[i][h];
      }
    }
  __syncthreads();
  for (int r = tid; r < G * 16; r += NTHREADS) {
    float M = -INFINITY, L = 0.f;
    for (int w = 0; w < NWARPS; ++w) merge_ml(M, L, ml_s[(w * G * 16 + r) * 2], ml_s[(w * G * 16 + r) * 2 + 1]);
    const int hl = r / 16, ws = r % 16;
    float* dst = a.part + ((((size_t)b * a.H + kvh * G + hl) * WPAD + ws) * a.S + split) * 2;
    dst[0] = M;
    dst[1] = L;
  }
}

// splits -> (m, 1/l) per row.  One thread per (b, h, slot).
__global__ void window_stats_merge(const float* __restrict__ part, float* __restrict__ stats, int rows, int S) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float M = -INFINITY, L = 0.f;
  for (int s = 0; s < S; ++s) merge_ml(M, L, part[((size_t)r * S + s) * 2], part[((size_t)r * S + s) * 2 + 1]);
  stats[(size_t)r * 2 + 0] = M;
  stats[(size_t)r * 2 + 1] = L > 0.f ? 1.f / L : 0.f;
}

__device__ __forceinline__ float slot_weight(int selector, int W, int w) {
  if (w >= W) return 0.f;
  if (selector == OMNIKV_SEL_UNIFORM) return 1.f;
  if (selector == OMNIKV_SEL_EXP) return exp2f((float)(w - (W - 1)));
  return w == W - 1 ? 1.f : 0.f;
}

// ---- pass 2: normalise, max over heads --------------------------------------------------------
// grid (ceil(max_len / P2_CHUNK), KVH, B).  A CTA streams the K rows of ONE KV head for its chunk of positions,
// normalises the logits of the head's query group with the statistics of pass 1, takes the max over the group's
// heads in registers and folds it into the plane planes[b][w][p] with an integer atomicMax (the weights are
// >= 0, so their bit patterns order like the values; max is order independent, so the result is deterministic).
// The planes start at zero; the weighted window sum over w is a separate small kernel.  Walking all KV heads
// inside one CTA with the running max in shared memory needed 111 KB per CTA and ran two CTAs of four warps per
// SM, latency bound at 3 us per tile; without that table a CTA needs 69 KB and three are resident.
constexpr int P2_CHUNK = 512;

template <typename T, int G, bool TMA>
__global__ void __launch_bounds__(NTHREADS, 3) window_pass2_mma(const WinArgs a, const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[P2_STAGES];
  constexpr int KT = TMA ? TMA_TILE_BYTES : TILE_BYTES;
  unsigned char* smem = TMA ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023)
                            : smem_raw;
  unsigned char* q_s = smem + P2_STAGES * KT;                                     // [G*16][PITCH]
  float* st_s = reinterpret_cast<float*>(q_s + (size_t)G * WPAD * PITCH);         // [G*16][2]
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int n = a.consider_len[b];
  const int r0 = blockIdx.x * P2_CHUNK;
  const int r1 = min(n, r0 + P2_CHUNK);
  if (r0 >= r1) return;
  const int ntiles = ceil_div(r1 - r0, TILE);
  const T* kb = static_cast<const T*>(a.k) + (size_t)b * a.k_sb + (size_t)kvh * a.k_sh;
  const T* qb = static_cast<const T*>(a.qw) + (size_t)b * a.H * a.W * kHeadDim;

  if constexpr (TMA) {
    if (tid == 0) {
#pragma unroll
      for (int s = 0; s < P2_STAGES; ++s) mbar_init(&full_bar[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
#pragma unroll
      for (int s = 0; s < P2_STAGES - 1; ++s)
        if (s < ntiles) issue_k_tile_tma(smem + s * KT, &tm_k, r0 + s * TILE, kvh, b, &full_bar[s]);
    }
  } else {
#pragma unroll
    for (int s = 0; s < P2_STAGES - 1; ++s) {
      if (s < ntiles) issue_k_tile<T>(smem + s * KT, kb, a.k_sr, r0 + s * TILE, r1, tid);
      cp_async_commit();
    }
  }
  load_q<T>(q_s, qb, kvh * G, G, a.W, tid);
  for (int i = tid; i < G * WPAD * 2; i += NTHREADS) st_s[i] = a.stats[((size_t)b * a.H + kvh * G) * WPAD * 2 + i];
  int* plane0 = reinterpret_cast<int*>(a.planes) + (size_t)b * a.W * a.plane_stride;

  for (int tile = 0; tile < ntiles; ++tile) {
    {
      const int nt = tile + P2_STAGES - 1;
      if constexpr (TMA) {
        __syncthreads();  // slot of tile - 1 is free (and, the first time, queries and statistics are in place)
        if (tid == 0 && nt < ntiles)
          issue_k_tile_tma(smem + (nt % P2_STAGES) * KT, &tm_k, r0 + nt * TILE, kvh, b, &full_bar[nt % P2_STAGES]);
        if (!mbar_wait(&full_bar[tile % P2_STAGES], (tile / P2_STAGES) & 1) && a.status) atomicExch(a.status, 5);
      } else {
        cp_async_wait<P2_STAGES - 2>();
        __syncthreads();  // the tile has landed (and, the first time, the queries and statistics are in place)
        if (nt < ntiles) issue_k_tile<T>(smem + (nt % P2_STAGES) * KT, kb, a.k_sr, r0 + nt * TILE, r1, tid);
        cp_async_commit();
      }
    }
    float acc[G][2][4];
    qk_tile<T, G, TMA>(acc, q_s, smem + (tile % P2_STAGES) * KT, warp, lane);
    const int cbase = r0 + tile * TILE + warp * 16 + 2 * t;
    float hm[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) hm[j][0] = hm[j][1] = hm[j][2] = hm[j][3] = 0.f;
#pragma unroll
    for (int i = 0; i < G; ++i)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float* st = st_s + (i * WPAD + g + 8 * h) * 2;
        const float ml2 = st[0] * kLog2e, inv_l = st[1];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float pw = exp2f(fmaf(acc[i][j][2 * h + e] * a.scale, kLog2e, -ml2)) * inv_l;
            hm[j][2 * h + e] = fmaxf(hm[j][2 * h + e], pw);
          }
      }
    // fold into the planes: entry (slot w, position R) for this thread's eight accumulator cells
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int w = g + 8 * (e >> 1), R = cbase + 8 * j + (e & 1);
        if (w < a.W && R < r1) atomicMax(plane0 + (size_t)w * a.plane_stride + R, __float_as_int(hm[j][e]));
      }
  }
  cp_async_wait<0>();
}

// score[b][p] = sum_w weight_w * planes[b][w][p]
__global__ void window_fold_planes(const float* __restrict__ planes, int64_t plane_stride, float* __restrict__ score_out,
                                   int64_t score_stride, int W, const int* __restrict__ consider_len, int selector) {
  const int b = blockIdx.y;
  const int n = consider_len[b];
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < n; p += gridDim.x * blockDim.x) {
    const float* pl = planes + (size_t)b * W * plane_stride + p;
    float acc = 0.f;
    for (int w = 0; w < W; ++w) acc = fmaf(slot_weight(selector, W, w), pl[(size_t)w * plane_stride], acc);
    score_out[(size_t)b * score_stride + p] = acc;
  }
}

// ---- fp32 CUDA-core variants -----------------------------------------------------------------
// One warp per key row (lane L holds dims 4L..4L+3); query rows of the KV head's group in shared
// memory.  PASS 1 accumulates (m, l) per query row; PASS 2 handles all KV heads of a key position.
constexpr int F32_MAXROWS = 8 * WPAD;  // G <= 8

__device__ __forceinline__ float warp_sum(float d) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
  return d;
}

__global__ void __launch_bounds__(NTHREADS) window_pass1_f32(const WinArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  float4* q_s = reinterpret_cast<float4*>(smem);  // [G*W][32]
  __shared__ float ml_s[NWARPS][F32_MAXROWS][2];
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.G, W = a.W, rows = G * W;
  const int n = a.consider_len[b];
  int r0, r1;
  split_range(n, a.S, split, r0, r1);
  const float* qb = static_cast<const float*>(a.qw) + ((size_t)b * a.H + kvh * G) * W * kHeadDim;
  for (int i = tid; i < rows * 32; i += NTHREADS) q_s[i] = reinterpret_cast<const float4*>(qb)[i];
  __syncthreads();
  const float* kbase = static_cast<const float*>(a.k) + (size_t)b * a.k_sb + (size_t)kvh * a.k_sh;
  // lane keeps the running (m, l) of query rows r = lane, lane+32, ...
  float m[F32_MAXROWS / 32], l[F32_MAXROWS / 32];
#pragma unroll
  for (int i = 0; i < F32_MAXROWS / 32; ++i) m[i] = -INFINITY, l[i] = 0.f;
  for (int R = r0 + warp; R < r1; R += NWARPS) {
    const float4 kx = __ldg(reinterpret_cast<const float4*>(kbase + (size_t)R * a.k_sr) + lane);
#pragma unroll
    for (int blk = 0; blk < F32_MAXROWS / 32; ++blk) {
      if (blk * 32 < rows) {
        float mine = -INFINITY;
        const int lim = min(32, rows - blk * 32);
        for (int rr = 0; rr < lim; ++rr) {
          const float4 qv = q_s[(blk * 32 + rr) * 32 + lane];
          float d = qv.x * kx.x;
          d = fmaf(qv.y, kx.y, d);
          d = fmaf(qv.z, kx.z, d);
          d = fmaf(qv.w, kx.w, d);
          d = warp_sum(d) * a.scale;
          if (rr == lane) mine = d;
        }
        if (lane < lim) merge_ml(m[blk], l[blk], mine, 1.f);
      }
    }
  }
#pragma unroll
  for (int blk = 0; blk < F32_MAXROWS / 32; ++blk) {
    ml_s[warp][blk * 32 + lane][0] = m[blk];
    ml_s[warp][blk * 32 + lane][1] = l[blk];
  }
  __syncthreads();
  for (int r = tid; r < rows; r += NTHREADS) {
    float M = -INFINITY, L = 0.f;
    for (int w = 0; w < NWARPS; ++w) merge_ml(M, L, ml_s[w][r][0], ml_s[w][r][1]);
    const int hl = r / W, ws = r % W;
    float* dst = a.part + ((((size_t)b * a.H + kvh * G + hl) * WPAD + ws) * a.S + split) * 2;
    dst[0] = M;
    dst[1] = L;
  }
}

constexpr int F32_CHUNK2 = 256;  // key positions per CTA in the fp32 pass 2

// grid (ceil(max_len / F32_CHUNK2), B).  KV heads are the outer loop (one group's queries in shared
// memory at a time); the running max over heads of every (position, slot) lives in shared memory.
__global__ void __launch_bounds__(NTHREADS) window_pass2_f32(const WinArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  float4* q_s = reinterpret_cast<float4*>(smem);  // [G*W][32]
  __shared__ float hm_s[F32_CHUNK2][WPAD];
  const int b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = a.G, W = a.W, H = a.H;
  const int n = a.consider_len[b];
  const int r0 = blockIdx.x * F32_CHUNK2;
  const int r1 = min(n, r0 + F32_CHUNK2);
  if (r0 >= r1) return;
  const float* kb = static_cast<const float*>(a.k) + (size_t)b * a.k_sb;
  const float* stats = a.stats + (size_t)b * H * WPAD * 2;
  for (int kvh = 0; kvh < a.KVH; ++kvh) {
    __syncthreads();
    const float* qb = static_cast<const float*>(a.qw) + ((size_t)b * H + kvh * G) * W * kHeadDim;
    for (int i = tid; i < G * W * 32; i += NTHREADS) q_s[i] = reinterpret_cast<const float4*>(qb)[i];
    __syncthreads();
    for (int R = r0 + warp; R < r1; R += NWARPS) {
      // lane w (< W) keeps the max over heads of the normalised weight of window slot w
      float hmax = 0.f;
      if (kvh > 0 && lane < WPAD) hmax = hm_s[R - r0][lane];
      const float4 kx = __ldg(reinterpret_cast<const float4*>(kb + (size_t)kvh * a.k_sh + (size_t)R * a.k_sr) + lane);
      for (int hl = 0; hl < G; ++hl) {
        for (int w = 0; w < W; ++w) {
          const float4 qv = q_s[(hl * W + w) * 32 + lane];
          float d = qv.x * kx.x;
          d = fmaf(qv.y, kx.y, d);
          d = fmaf(qv.z, kx.z, d);
          d = fmaf(qv.w, kx.w, d);
          d = warp_sum(d) * a.scale;
          if (w == lane) {
            const float* st = stats + ((kvh * G + hl) * WPAD + w) * 2;
            hmax = fmaxf(hmax, exp2f((d - st[0]) * kLog2e) * st[1]);
          }
        }
      }
      if (lane < WPAD) hm_s[R - r0][lane] = hmax;
    }
  }
  __syncthreads();
  for (int R = r0 + warp; R < r1; R += NWARPS) {
    const float hmax = lane < W ? hm_s[R - r0][lane] : 0.f;
    if (a.planes_out && lane < W) a.planes_out[((size_t)b * W + lane) * a.score_stride + R] = hmax;
    if (a.score_out) {
      const float v = warp_sum(slot_weight(a.selector, W, lane) * hmax);
      if (lane == 0) a.score_out[(size_t)b * a.score_stride + R] = v;
    }
  }
}

template <typename T, int G, bool TMA>
int launch_mma_copy(const WinArgs& a, const CUtensorMap& tm_k, int max_len, cudaStream_t st) {
  constexpr int KT = TMA ? TMA_TILE_BYTES : TILE_BYTES;
  const int smem1 = P1_STAGES * KT + G * WPAD * PITCH + (TMA ? 1024 : 0);
  const int smem2 = P2_STAGES * KT + G * WPAD * PITCH + G * WPAD * 2 * (int)sizeof(float) + (TMA ? 1024 : 0);
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_pass1_mma<T, G, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_pass2_mma<T, G, TMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
  // the planes receive atomic maxima: clear the part pass 2 may touch
  OMNIKV_CUDA_OK(cudaMemsetAsync(a.planes, 0, (size_t)a.B * a.W * a.plane_stride * sizeof(float), st));
  window_pass1_mma<T, G, TMA><<<dim3(a.S, a.KVH, a.B), NTHREADS, smem1, st>>>(a, tm_k);
  OMNIKV_CUDA_OK(cudaGetLastError());
  const int rows = a.B * a.H * WPAD;
  window_stats_merge<<<ceil_div(rows, 128), 128, 0, st>>>(a.part, a.stats, rows, a.S);
  OMNIKV_CUDA_OK(cudaGetLastError());
  window_pass2_mma<T, G, TMA><<<dim3(ceil_div(max_len, P2_CHUNK), a.KVH, a.B), NTHREADS, smem2, st>>>(a, tm_k);
  OMNIKV_CUDA_OK(cudaGetLastError());
  if (a.score_out) {
    window_fold_planes<<<dim3(min(1184, ceil_div(max_len, 256)), a.B), 256, 0, st>>>(
        a.planes, a.plane_stride, a.score_out, a.score_stride, a.W, a.consider_len, a.selector);
    OMNIKV_CUDA_OK(cudaGetLastError());
  }
  return OMNIKV_OK;
}

// K tiles travel through a TMA tensor map over rows [0, max_len) of the cache (rows past it read as zero and are
// masked anyway); when the map cannot be built, through 16-byte cp.async copies.
template <typename T, int G>
int launch_mma(const WinArgs& a, int n_chunks2, int max_len, cudaStream_t st) {
  (void)n_chunks2;
  CUtensorMap tm_k = {};
  constexpr bool is_bf16 = !std::is_same<T, __half>::value;
  // The Blackwell tensor path (tcgen05.mma, accumulators in tensor memory) when it covers the shape and the K
  // cache can be described by a tensor map with 128-row boxes; OMNIKV_WINDOW_TC=0 keeps the mma.sync kernels.
  static const bool tc_on = [] {
    const char* e = getenv("OMNIKV_WINDOW_TC");
    return !(e && e[0] == '0');
  }();
  if (tc_on && window_tc_supported(G, a.KVH) &&
      make_kv_tensor_map(&tm_k, is_bf16, a.k, max_len, a.KVH, a.B, a.k_sr, a.k_sh, a.k_sb, 128)) {
    int dev = 0, n_sms = 0;
    OMNIKV_CUDA_OK(cudaGetDevice(&dev));
    OMNIKV_CUDA_OK(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev));
    WinTcArgs t;
    t.qw = a.qw; t.consider_len = a.consider_len; t.part = a.part;
    t.tplane = a.stats + stats_floats(a.B, a.H); t.tplane_stride = (int64_t)plane_stride_of(max_len);
    t.score_out = a.score_out; t.planes_out = a.planes_out; t.score_stride = a.score_stride;
    t.B = a.B; t.H = a.H; t.KVH = a.KVH; t.G = G; t.W = a.W; t.S = window_tc_splits(a.B, a.KVH, n_sms, max_len);
    t.selector = a.selector; t.n_sms = n_sms; t.scale = a.scale; t.status = a.status;
    return window_tc_launch(is_bf16 ? OMNIKV_BF16 : OMNIKV_F16, t, tm_k, max_len, st);
  }
  static const bool tma_on = [] {
    const char* e = getenv("OMNIKV_WINDOW_TMA");
    return !(e && e[0] == '0');
  }();
  if (tma_on && make_kv_tensor_map(&tm_k, is_bf16, a.k, max_len, a.KVH, a.B, a.k_sr, a.k_sh, a.k_sb))
    return launch_mma_copy<T, G, true>(a, tm_k, max_len, st);
  return launch_mma_copy<T, G, false>(a, tm_k, max_len, st);
}

template <typename T>
int dispatch_mma(const WinArgs& a, int n_chunks2, int max_len, cudaStream_t st) {
  switch (a.G) {
    case 1: return launch_mma<T, 1>(a, n_chunks2, max_len, st);
    case 2: return launch_mma<T, 2>(a, n_chunks2, max_len, st);
    case 4: return launch_mma<T, 4>(a, n_chunks2, max_len, st);
    case 8: return launch_mma<T, 8>(a, n_chunks2, max_len, st);
    default: return OMNIKV_E_UNSUPPORTED;
  }
}

int launch_f32(const WinArgs& a, int max_len, cudaStream_t st) {
  if (a.G > 8) return OMNIKV_E_UNSUPPORTED;
  const int smem_q = a.G * a.W * 32 * (int)sizeof(float4);
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_pass1_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q));
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_pass2_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q));
  window_pass1_f32<<<dim3(a.S, a.KVH, a.B), NTHREADS, smem_q, st>>>(a);
  OMNIKV_CUDA_OK(cudaGetLastError());
  const int rows = a.B * a.H * WPAD;
  window_stats_merge<<<ceil_div(rows, 128), 128, 0, st>>>(a.part, a.stats, rows, a.S);
  OMNIKV_CUDA_OK(cudaGetLastError());
  window_pass2_f32<<<dim3(ceil_div(max_len, F32_CHUNK2), a.B), NTHREADS, smem_q, st>>>(a);
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

constexpr int kPass1Splits = 55;  // 8 KV heads x 55 = 440 CTAs = 3 per SM on 148 SMs
static_assert(kWindowTcMaxSplits >= kPass1Splits, "the partials are sized for the larger split count");


}  // namespace
}  // namespace omnikv

extern "C" size_t omnikv_score_window_workspace_bytes(int B, int H, int W, int max_len) {
  using namespace omnikv;
  if (B <= 0 || H <= 0 || W <= 0 || max_len <= 0) return 0;
  // pass-1 partials, merged statistics, and the per-slot planes of pass 2 (used when the caller gives none)
  (void)W;  // the planes are sized for the padded window: the tensor-memory path keeps 16 per-slot maxima per key there
  return (part_floats(B, H, kWindowTcMaxSplits) + stats_floats(B, H) + plane_floats(B, WPAD, max_len)) * sizeof(float);
}

extern "C" int omnikv_score_window(const omnikv_window_params* p, void* stream) {
  using namespace omnikv;
  if (!p || !p->qw || !p->k || !p->consider_len || (!p->score_out && !p->planes_out)) return OMNIKV_E_BADARG;
  if (p->B <= 0 || p->H <= 0 || p->KVH <= 0 || p->W <= 0 || p->max_len <= 0 || p->H % p->KVH) return OMNIKV_E_BADARG;
  if (p->head_dim != kHeadDim || p->W > WPAD) return OMNIKV_E_UNSUPPORTED;
  if (p->selector < OMNIKV_SEL_SOFTMAX_LAST || p->selector > OMNIKV_SEL_EXP) return OMNIKV_E_BADARG;
  if (p->score_stride < p->max_len) return OMNIKV_E_BADARG;
  const int esz = p->dtype == OMNIKV_F32 ? 4 : 2;
  const int vec = 16 / esz;
  if ((reinterpret_cast<uintptr_t>(p->qw) & 15) || (reinterpret_cast<uintptr_t>(p->k) & 15)) return OMNIKV_E_BADARG;
  if (p->k_stride_b % vec || p->k_stride_h % vec || p->k_stride_row % vec || p->k_stride_row < kHeadDim)
    return OMNIKV_E_BADARG;
  if (!p->workspace || p->workspace_bytes < omnikv_score_window_workspace_bytes(p->B, p->H, p->W, p->max_len))
    return OMNIKV_E_WORKSPACE;
  WinArgs a;
  a.qw = p->qw; a.k = p->k; a.k_sb = p->k_stride_b; a.k_sh = p->k_stride_h; a.k_sr = p->k_stride_row;
  a.consider_len = p->consider_len;
  a.part = static_cast<float*>(p->workspace);
  a.stats = a.part + part_floats(p->B, p->H, kWindowTcMaxSplits);
  a.score_out = p->score_out; a.planes_out = p->planes_out; a.score_stride = p->score_stride;
  if (p->planes_out) {  // the caller's planes (tensor parallelism: they are MAX-reduced over ranks, then folded)
    a.planes = p->planes_out; a.plane_stride = p->score_stride;
  } else {
    a.planes = a.stats + stats_floats(p->B, p->H); a.plane_stride = (int64_t)plane_stride_of(p->max_len);
  }
  a.B = p->B; a.H = p->H; a.KVH = p->KVH; a.G = p->H / p->KVH; a.W = p->W; a.S = kPass1Splits;
  a.selector = p->selector; a.scale = p->scale; a.status = p->status;
  // pass 2: chunks of whole tiles, about two CTAs' worth of chunks per SM over the batch
  int chunks = ceil_div(296, p->B);
  a.chunk2 = ceil_div(ceil_div(p->max_len, chunks), TILE) * TILE;
  const int n_chunks2 = ceil_div(p->max_len, a.chunk2);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (p->dtype) {
    case OMNIKV_BF16: return dispatch_mma<__nv_bfloat16>(a, n_chunks2, p->max_len, st);
    case OMNIKV_F16: return dispatch_mma<__half>(a, n_chunks2, p->max_len, st);
    case OMNIKV_F32: return launch_f32(a, p->max_len, st);
    default: return OMNIKV_E_UNSUPPORTED;
  }
}
