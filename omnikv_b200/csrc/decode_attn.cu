// Decode attention over a row list (dense cache / selected rows + tail), split-K flash-decode,
// with the filter layer's selection score emitted while K streams through.
//
// bf16 / fp16: K and V rows (256 B each) are staged through a 3-deep shared-memory ring with
// 16-byte cp.async copies (rows padded to 272 B so that ldmatrix is bank-conflict free), and the
// GQA group's queries meet them in m16n8k16 tensor-core MMAs: HBM-bound streaming where the MMA
// only keeps the issue slots free; every K/V byte is read once for all query heads of its KV head.
// fp32: CUDA-core kernel (tensor cores would have to round the operands to tf32).
//
// Grid (n_splits, KVH, B).  Every CTA owns one contiguous chunk of the sequence's row list and
// writes one un-normalised partial (o, m, l) per query head; the CTA that finishes last for a (sequence,
// KV head) merges that group's splits into the output, so an attention call is a single launch.
#include <stdlib.h>

#include <atomic>
#include <type_traits>

#include "common.cuh"

namespace omnikv {

struct AttnArgs {
  const void* q;
  int64_t q_sb, q_sh;
  void* out;
  const void* kA;
  const void* vA;
  int64_t a_sb, a_sh, a_sr;
  const int* idxA;
  const int* idx_row;  // row of the index table that batch entry b uses, or nullptr: row b
  int64_t idx_stride;
  const int* lenA;
  const void* kB;
  const void* vB;
  int64_t b_sb, b_sh, b_sr;
  const int* startB;
  const int* lenB;
  float* score_out;
  int64_t score_stride;
  const int* score_len;
  float* ws_o;
  float* ws_ml;
  unsigned* ws_cnt;   // [B*KVH] arrival counters of the splits, zero between launches
  int pdl_trigger;    // 1: the grid is fully resident, the next kernel may be scheduled early
  int coop_merge;     // 1: the splits of a (sequence, KV head) merge together (see coop_merge); needs a resident grid
  int trace_slot;     // profiling build: slot of the stamp array this launch writes
  int* status;        // device word for bounded-wait failures, or nullptr
  int B, H, KVH, G, S;
  float scale;
};

#ifdef OMNIKV_TRACE
// Profiling build only: per-CTA %globaltimer stamps of the mma kernel's stages, one slot per launch.
// [0] CTA start, [1] previous kernel complete, [2] prologue done, [3] tiles consumed, [4] partials written,
// [5] counted in (the last CTA of a group: merged), [6] 2000 + (sparse ? 1 : 0).
constexpr int kAttnTraceCtas = 320, kAttnTraceWords = 8;
__device__ unsigned long long g_attn_trace[kTraceSlots * kAttnTraceCtas * kAttnTraceWords];
__device__ __forceinline__ void attn_stamp(int launch, int word) {
  if (threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (cta < kAttnTraceCtas) g_attn_trace[(launch * kAttnTraceCtas + cta) * kAttnTraceWords + word] = t;
  }
}
#define ATTN_STAMP(i) attn_stamp(a.trace_slot, i)
#else
#define ATTN_STAMP(i)
#endif

namespace {

constexpr int TILE = 64;       // rows per pipeline stage
constexpr int NWARPS = 4;      // each warp owns 16 rows of every tile
constexpr int NTHREADS = NWARPS * 32;
constexpr int STAGES = 3;
constexpr int PITCH = 272;     // bytes per staged row: 256 + 16 pad
constexpr int TILE_BYTES = TILE * PITCH;
constexpr int Q_BYTES = 16 * PITCH;

// OMNIKV_ATTN_TMA=0 in the environment keeps dense layers on the cp.async variant.
inline bool g_attn_tma_enabled() {
  static const bool on = [] {
    const char* e = getenv("OMNIKV_ATTN_TMA");
    return !(e && e[0] == '0');
  }();
  return on;
}

bool g_attn_coop_enabled() {  // OMNIKV_ATTN_COOP=0: every merge by the last CTA of its group
  static const bool on = [] {
    const char* e = getenv("OMNIKV_ATTN_COOP");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <bool WITH_V, int ST = STAGES>
constexpr int mma_smem_bytes() {
  return ST * (WITH_V ? 2 : 1) * TILE_BYTES + Q_BYTES;
}

// Row range [r0, r1) of split `split` out of S for a list of n rows (chunks are TILE-aligned).  The chunk
// length comes from the LONGEST sequence of the batch: every CTA then has the same amount of work and a
// short sequence simply uses fewer of its S splits (the rest hand in empty partials).  Sizing the chunks
// per sequence instead left the CTAs of short sequences idle while the longest one finished.
__device__ __forceinline__ void split_range(int n, int n_max, int S, int split, int& r0, int& r1) {
  int chunk = ceil_div(ceil_div(n_max, S), TILE) * TILE;
  r0 = min(n, split * chunk);
  r1 = min(n, r0 + chunk);
}
__device__ __forceinline__ int batch_max_rows(const AttnArgs& a, int n) {
  int n_max = n;
  for (int bb = 0; bb < a.B; ++bb) n_max = max(n_max, a.lenA[bb] + (a.lenB ? a.lenB[bb] : 0));
  return n_max;
}

// After a CTA has written its partials: count it in; the CTA that completes the count of its (b, kvh)
// merges the S partials of the group's heads into the output (log-sum-exp merge) and clears the counter.
// Must be called by all NTHREADS threads.  One warp per head (the group's heads in parallel), a lane owns
// four output dims.  w_s: shared scratch of NWARPS * S floats.
template <typename T>
__device__ __forceinline__ void finish_group(const AttnArgs& a, int b, int kvh, float* w_s, int* flag_s) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned prev = atomicAdd(a.ws_cnt + b * a.KVH + kvh, 1u);
    *flag_s = (prev == (unsigned)(a.S - 1));
  }
  __syncthreads();
  if (!*flag_s) return;
  __threadfence();
  const int G = a.G, S = a.S;
  float* w = w_s + (size_t)warp * S;
  for (int r = warp; r < G; r += NWARPS) {
    const int h = kvh * G + r;
    const size_t base = (size_t)(b * a.H + h) * S;
    // Everything that does not depend on the weights is asked for at once: the (m, l) pairs of all splits (two
    // per lane cover 64 splits, the rest in a loop) AND the first sixteen partial outputs -- the merge is a chain
    // of L2 round trips on the critical path of every attention call, so it should be as short as possible.
    const float4* op = reinterpret_cast<const float4*>(a.ws_o + base * kHeadDim) + lane;
    const float2* mlp = reinterpret_cast<const float2*>(a.ws_ml + base * 2);
    float2 ml0 = make_float2(-INFINITY, 0.f), ml1 = ml0;
    if (lane < S) ml0 = __ldcg(mlp + lane);
    if (lane + 32 < S) ml1 = __ldcg(mlp + lane + 32);
    constexpr int PRE = 16;
    float4 o_pre[PRE];
#pragma unroll
    for (int s = 0; s < PRE; ++s) o_pre[s] = s < S ? __ldcg(op + (size_t)s * (kHeadDim / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    float M = fmaxf(ml0.x, ml1.x);
    for (int s = lane + 64; s < S; s += 32) M = fmaxf(M, __ldcg(a.ws_ml + (base + s) * 2));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float l = 0.f;
    __syncwarp();
    {
      const float w0 = (ml0.x == -INFINITY) ? 0.f : exp2f((ml0.x - Mu) * kLog2e);
      const float w1 = (ml1.x == -INFINITY) ? 0.f : exp2f((ml1.x - Mu) * kLog2e);
      if (lane < S) w[lane] = w0;
      if (lane + 32 < S) w[lane + 32] = w1;
      l = fmaf(ml0.y, w0, ml1.y * w1);
    }
    for (int s = lane + 64; s < S; s += 32) {
      const float2 ml = __ldcg(mlp + s);
      const float wt = (ml.x == -INFINITY) ? 0.f : exp2f((ml.x - Mu) * kLog2e);
      w[s] = wt;
      l = fmaf(ml.y, wt, l);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    __syncwarp();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < PRE; ++s) {
      if (s < S) {
        const float wt = w[s];
        acc.x = fmaf(o_pre[s].x, wt, acc.x);
        acc.y = fmaf(o_pre[s].y, wt, acc.y);
        acc.z = fmaf(o_pre[s].z, wt, acc.z);
        acc.w = fmaf(o_pre[s].w, wt, acc.w);
      }
    }
#pragma unroll 16
    for (int s = PRE; s < S; ++s) {
      const float4 o = __ldcg(op + (size_t)s * (kHeadDim / 4));
      const float wt = w[s];
      acc.x = fmaf(o.x, wt, acc.x);
      acc.y = fmaf(o.y, wt, acc.y);
      acc.z = fmaf(o.z, wt, acc.z);
      acc.w = fmaf(o.w, wt, acc.w);
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* dst = static_cast<T*>(a.out) + (size_t)b * a.q_sb + (size_t)h * a.q_sh + lane * 4;
    dst[0] = from_float<T>(acc.x * inv);
    dst[1] = from_float<T>(acc.y * inv);
    dst[2] = from_float<T>(acc.z * inv);
    dst[3] = from_float<T>(acc.w * inv);
  }
  if (tid == 0) a.ws_cnt[b * a.KVH + kvh] = 0u;
}

// The merge of MANY splits (a layer under tensor parallelism: 148 per KV head of a dense layer, 69 of a sparse one) by one last CTA is a chain of ten
// L2 round trips (10.8 us measured at four GPUs).  When the whole grid is resident (the host checks the occupancy),
// the splits of a (sequence, KV head) instead wait for one another -- thread 0 of every CTA counts itself in and
// polls the count, bounded by time -- and then EVERY CTA merges a slice of the group's G x 128 outputs: four output
// values per CTA, the S partials of them read by one warp in a single round trip (lane = split, up to eight per
// lane), combined with shuffles in a fixed order.  The CTA that leaves last clears both counters.
template <typename T>
__device__ __forceinline__ void coop_merge(const AttnArgs& a, int b, int kvh, int split, int* flag_s) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.S, G = a.G;
  unsigned* arrive = a.ws_cnt + b * a.KVH + kvh;
  unsigned* depart = a.ws_cnt + 2048 + b * a.KVH + kvh;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    atomicAdd(arrive, 1u);
    bool ok = ld_volatile_u32(arrive) >= (unsigned)S;
    if (!ok) {
      const unsigned long long t0 = globaltimer_ns();
      for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16 && !ok; ++i) ok = ld_volatile_u32(arrive) >= (unsigned)S;
        if (ok || globaltimer_ns() - t0 > kWaitNs) break;
      }
    }
    if (!ok && a.status) atomicExch(a.status, 5);
    *flag_s = ok ? 1 : 0;
  }
  __syncthreads();
  if (!*flag_s) return;
  __threadfence();
  const int total = G * kHeadDim;
  const int chunk = ceil_div(ceil_div(total, S), 4) * 4;  // output values of this CTA
  if (warp == 0) {
    for (int e = split * chunk; e < min(total, split * chunk + chunk); e += 4) {
      const int r = e / kHeadDim, d0 = e % kHeadDim, h = kvh * G + r;
      const size_t base = (size_t)(b * a.H + h) * S;
      float2 ml[8];
      float4 ov[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int sidx = lane + 32 * u;
        ml[u] = make_float2(-INFINITY, 0.f);
        ov[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sidx < S) {
          ml[u] = __ldcg(reinterpret_cast<const float2*>(a.ws_ml + (base + sidx) * 2));
          ov[u] = __ldcg(reinterpret_cast<const float4*>(a.ws_o + (base + sidx) * kHeadDim + d0));
        }
      }
      float M = -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) M = fmaxf(M, ml[u].x);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
      const float Mu = (M == -INFINITY) ? 0.f : M;
      float l = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float wt = (ml[u].x == -INFINITY) ? 0.f : exp2f((ml[u].x - Mu) * kLog2e);
        l = fmaf(ml[u].y, wt, l);
        acc.x = fmaf(ov[u].x, wt, acc.x);
        acc.y = fmaf(ov[u].y, wt, acc.y);
        acc.z = fmaf(ov[u].z, wt, acc.z);
        acc.w = fmaf(ov[u].w, wt, acc.w);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        l += __shfl_xor_sync(0xffffffffu, l, off);
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
      }
      if (lane == 0) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* dst = static_cast<T*>(a.out) + (size_t)b * a.q_sb + (size_t)h * a.q_sh + d0;
        dst[0] = from_float<T>(acc.x * inv);
        dst[1] = from_float<T>(acc.y * inv);
        dst[2] = from_float<T>(acc.z * inv);
        dst[3] = from_float<T>(acc.w * inv);
      }
    }
  }
  __syncthreads();
  if (tid == 0 && atomicAdd(depart, 1u) == (unsigned)(S - 1)) {  // every CTA of the group is past its wait
    atomicExch(arrive, 0u);
    atomicExch(depart, 0u);
  }
}

// BULK: how a tile's rows travel to shared memory.  true: one 256-byte bulk copy per row (the copy engine moves
// it and signals the stage's mbarrier) -- sixteen times fewer instructions and request slots than cp.async, which
// is what a sparse layer's scattered rows need (22.5 instead of 28.7 us per layer).  false: sixteen 16-byte
// cp.async per row; for a dense layer's long contiguous streams this keeps more requests in flight and is the
// faster of the two there (99.8 against 103.7 us per layer).
//
// MODE kCopyTma (a dense layer whose row capacity the caller states): a tile is four boxes of 64 rows x 128 bytes
// (K low half, K high half, V low, V high) fetched by ONE thread with cp.async.bulk.tensor through a 4-D tensor
// map [B, KVH, rows, d]; the map's 128-byte swizzle (16-byte chunk c of row r lands at chunk c ^ (r & 7)) makes
// the unpadded rows conflict-free for ldmatrix.  Rows past the sequence but inside the capacity arrive as they
// are in memory: their scores are masked and their V rows are zeroed in shared memory before use.
constexpr int kCopyCpAsync = 0, kCopyBulkRows = 1, kCopyTma = 2, kCopyBulkPairs = 3;
constexpr int PAIR_PITCH = 528;  // K row | V row of one cache position (512 bytes) + 16 pad: conflict-free for ldmatrix
constexpr int TMA_BOX_BYTES = kTmaBoxBytes;

template <typename T, bool WITH_V, bool WITH_SCORE, int MODE, int ST = STAGES>
__global__ void __launch_bounds__(NTHREADS, ST > STAGES ? 1 : 2) decode_attn_mma_kernel(const AttnArgs a,
                                                                      const __grid_constant__ CUtensorMap tm_k,
                                                                      const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int last_flag;
  // kCopyBulkPairs: the cache stores the V row of a position right behind its K row (the token-major layout of a
  // sparse layer), so ONE 512-byte bulk copy brings both: half as many copies -- the copy engine takes about 25
  // cycles per copy whatever its size, which bounds a CTA that streams scattered rows
  constexpr bool PAIR = MODE == kCopyBulkPairs;
  constexpr bool BULK = MODE == kCopyBulkRows || PAIR;
  constexpr int RP = PAIR ? PAIR_PITCH : PITCH;  // byte pitch of a staged row
  constexpr bool TMA = MODE == kCopyTma;
  constexpr int STAGE_BYTES = TMA ? (WITH_V ? 4 : 2) * TMA_BOX_BYTES : (WITH_V ? 2 : 1) * TILE_BYTES;
  // the swizzled boxes want 1024-byte alignment
  unsigned char* smem = TMA ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023)
                            : smem_raw;
  unsigned char* q_s = smem + ST * STAGE_BYTES;
  // byte address of the 16-byte piece at (row, byte column) of a staged K or V tile
  auto staged = [&](const unsigned char* tile_base, int row, int colb) -> const unsigned char* {
    if constexpr (TMA)
      return swz128(tile_base, row, colb);
    else
      return tile_base + row * RP + colb;
  };

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = a.G;
  // Programmatic dependent launch.  Of what this kernel reads, only q and the CURRENT token's K/V row (the last
  // row of the sequence) come from the kernel right before it (the QKV kernel); the lengths, the index list and
  // all older rows were written by kernels that had completed before that one could start.  So the lengths, the
  // index lookups and the copies of the first tiles go out BEFORE the wait and overlap the previous kernel's
  // last CTAs; the wait comes before q is read and before anything is written.  Only a split whose first
  // tiles already reach the last row waits first.  The successor may be scheduled early only when this grid is
  // fully resident (a.pdl_trigger, decided by the host from the grid size).
  ATTN_STAMP(0);
#ifdef OMNIKV_TRACE
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)
    g_attn_trace[(a.trace_slot * kAttnTraceCtas) * kAttnTraceWords + 6] = 2000ull + (a.idxA ? 1 : 0);
#endif
  const int nA = a.lenA[b];
  const int nB = a.lenB ? a.lenB[b] : 0;
  const int startB = a.startB ? a.startB[b] : 0;
  const int n = nA + nB;
  int r0, r1;
  split_range(n, a.B > 1 ? batch_max_rows(a, n) : n, a.S, split, r0, r1);
  const int ntiles = r1 > r0 ? ceil_div(r1 - r0, TILE) : 0;
  const bool early = ntiles > 0 && (r1 < n || ntiles > ST - 1);
  if (!early) {
    pdl_wait();
    if (a.pdl_trigger) pdl_trigger();
  }

  float* ws_o = a.ws_o;
  float* ws_ml = a.ws_ml;
  if (ntiles == 0) {  // empty split: neutral partial
    if (WITH_V) {
      for (int r = 0; r < G; ++r) {
        size_t base = ((size_t)(b * a.H + kvh * G + r) * a.S + split);
        ws_o[base * kHeadDim + tid] = 0.f;
        if (tid == 0) {
          ws_ml[base * 2 + 0] = -INFINITY;
          ws_ml[base * 2 + 1] = 0.f;
        }
      }
      if (a.coop_merge) coop_merge<T>(a, b, kvh, split, &last_flag);
      else finish_group<T>(a, b, kvh, reinterpret_cast<float*>(smem), &last_flag);
    }
    return;
  }

  const T* kA = static_cast<const T*>(a.kA) + (size_t)b * a.a_sb + (size_t)kvh * a.a_sh;
  const T* vA = WITH_V ? static_cast<const T*>(a.vA) + (size_t)b * a.a_sb + (size_t)kvh * a.a_sh : nullptr;
  const T* kB = a.kB ? static_cast<const T*>(a.kB) + (size_t)b * a.b_sb + (size_t)kvh * a.b_sh : nullptr;
  const T* vB = (WITH_V && a.vB) ? static_cast<const T*>(a.vB) + (size_t)b * a.b_sb + (size_t)kvh * a.b_sh : nullptr;
  const int* idx = a.idxA ? a.idxA + (size_t)(a.idx_row ? a.idx_row[b] : b) * a.idx_stride : nullptr;

  // A tile is issued in two steps: resolve() turns its rows into cache offsets (for a sparse layer this is a
  // lookup in the index list), issue() starts the copies.  resolve() of the NEXT tile runs right after issue() of
  // the current one, so the index loads are in flight during a whole tile of compute and never sit between a
  // warp and its copies (the copies are asm statements the compiler does not move loads across).
  auto row_offset = [&](int tile, int row) -> long long {
    const int R = r0 + tile * TILE + row;
    if (tile >= ntiles || R >= r1) return -1;
    if (R < nA) {
      const long long pos = idx ? (long long)__ldg(idx + R) : (long long)R;
      return pos * a.a_sr;
    }
    return ((long long)(startB + (R - nA)) * a.b_sr) | (1ll << 62);  // bit 62: segment B
  };
  // ---- BULK: thread t owns row t & 63 of every tile, K for t < 64 and V for t >= 64 ----
  __shared__ __align__(8) uint64_t full_bar[ST];
  const int my_row = tid & (TILE - 1);
  const bool my_v = tid >= TILE;
  constexpr unsigned ROW_BYTES = kHeadDim * sizeof(T);
  auto issue_bulk = [&](int tile, long long off) {
    const int slot = tile % ST;
    unsigned char* dst = smem + slot * STAGE_BYTES + (PAIR ? my_row * PAIR_PITCH : (my_v ? TILE_BYTES : 0) + my_row * PITCH);
    if (tid == 0) {  // bytes this stage will receive: its valid rows, K and V
      const int nvalid = min(TILE, r1 - (r0 + tile * TILE));
      mbar_expect_tx(&full_bar[slot], (unsigned)nvalid * ROW_BYTES * (WITH_V ? 2u : 1u));
    }
    if (my_v && (!WITH_V || PAIR)) return;
    if constexpr (PAIR) {
      if (off >= 0) {
        const bool segB = (off >> 62) != 0;
        const long long o = off & ~(1ll << 62);
        tma_bulk_g2s(dst, (segB ? kB : kA) + o, 2 * ROW_BYTES, &full_bar[slot]);
      } else {
#pragma unroll
        for (int c = 0; c < 2 * (int)ROW_BYTES / 16; ++c) *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(0, 0, 0, 0);
      }
      return;
    }
    if (off >= 0) {
      const bool segB = (off >> 62) != 0;
      const long long o = off & ~(1ll << 62);
      const T* src = (my_v ? (segB ? vB : vA) : (segB ? kB : kA)) + o;
      tma_bulk_g2s(dst, src, ROW_BYTES, &full_bar[slot]);
    } else {  // a row past the end of the chunk: zeros, so that 0 * V stays 0
#pragma unroll
      for (int c = 0; c < (int)ROW_BYTES / 16; ++c) *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(0, 0, 0, 0);
    }
  };
  // ---- cp.async: thread t copies 16-byte column t & 15 of rows (t >> 4) + 8 i ----
  constexpr int RPT = TILE / 8;  // rows per thread and tile
  const int cc = tid & 15, rowi = tid >> 4;
  auto resolve_cp = [&](int tile, long long (&off)[RPT]) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) off[i] = row_offset(tile, rowi + 8 * i);
  };
  auto issue_cp = [&](int slot, const long long (&off)[RPT]) {
    unsigned char* ks = smem + slot * STAGE_BYTES;
    unsigned char* vs = ks + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int row = rowi + 8 * i;
      const bool valid = off[i] >= 0;
      const bool segB = valid && (off[i] >> 62);
      const long long o = off[i] & ~(1ll << 62);
      const T* ksrc = valid ? (segB ? kB : kA) + o : kA;
      cp_async16(ks + row * PITCH + cc * 16, ksrc + cc * 8, valid);
      if (WITH_V) {
        const T* vsrc = valid ? (segB ? vB : vA) + o : vA;
        cp_async16(vs + row * PITCH + cc * 16, vsrc + cc * 8, valid);
      }
    }
  };

  auto issue_tma = [&](int tile) {  // one thread: the tile's boxes
    const int slot = tile % ST;
    unsigned char* dst = smem + slot * STAGE_BYTES;
    mbar_expect_tx(&full_bar[slot], STAGE_BYTES);
    const int row0 = r0 + tile * TILE;
    tma_load_4d(dst, &tm_k, 0, row0, kvh, b, &full_bar[slot]);
    tma_load_4d(dst + TMA_BOX_BYTES, &tm_k, 64, row0, kvh, b, &full_bar[slot]);
    if (WITH_V) {
      tma_load_4d(dst + 2 * TMA_BOX_BYTES, &tm_v, 0, row0, kvh, b, &full_bar[slot]);
      tma_load_4d(dst + 3 * TMA_BOX_BYTES, &tm_v, 64, row0, kvh, b, &full_bar[slot]);
    }
  };

  // the index lookups of the first ST tiles go out together, then the copies of the first ST-1 tiles
  long long offb_next = -1;
  long long offc_next[RPT];
  if constexpr (TMA) {
    if (tid == 0) {
#pragma unroll
      for (int s = 0; s < ST; ++s) mbar_init(&full_bar[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
#pragma unroll
      for (int s = 0; s < ST - 1; ++s)
        if (s < ntiles) issue_tma(s);
    }
    __syncthreads();
  } else if constexpr (BULK) {
    if (tid == 0) {
#pragma unroll
      for (int s = 0; s < ST; ++s) mbar_init(&full_bar[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    long long first[ST - 1];
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) first[s] = row_offset(s, my_row);
    offb_next = row_offset(ST - 1, my_row);
#pragma unroll
    for (int s = 0; s < ST - 1; ++s)
      if (s < ntiles) issue_bulk(s, first[s]);
  } else {
    long long first[ST - 1][RPT];
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) resolve_cp(s, first[s]);
    resolve_cp(ST - 1, offc_next);
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) {
      if (s < ntiles) issue_cp(s, first[s]);
      cp_async_commit();
    }
  }

  if (early) {
    pdl_wait();
    if (a.pdl_trigger) pdl_trigger();
  }
  ATTN_STAMP(1);
  // Q tile: 16 rows x 128, rows >= G are zero.  Both loads first, then the stores (one round trip, not two: the
  // compiler keeps a load behind an earlier store through a generic pointer).
  uint4 qv[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = tid + j * NTHREADS, r = i >> 4, c = i & 15;
    qv[j] = make_uint4(0, 0, 0, 0);
    if (r < G) {
      const T* qp = static_cast<const T*>(a.q) + (size_t)b * a.q_sb + (size_t)(kvh * G + r) * a.q_sh;
      qv[j] = *reinterpret_cast<const uint4*>(qp + c * 8);
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int i = tid + j * NTHREADS, r = i >> 4, c = i & 15;
    *reinterpret_cast<uint4*>(q_s + r * PITCH + c * 16) = qv[j];
  }
  __syncthreads();
  unsigned qf[8][4];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const int row = (lane & 7) + 8 * ((lane >> 3) & 1);
    const int col = kk * 16 + 8 * (lane >> 4);
    ldmatrix_x4(qf[kk], q_s + row * PITCH + col * 2);
  }

  ATTN_STAMP(2);  // copies of the first tiles issued, Q fragments loaded
  float m_row[2] = {-INFINITY, -INFINITY};
  float l_row[2] = {0.f, 0.f};
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const int mi = lane >> 3;  // which 8x8 matrix this lane addresses in ldmatrix.x4
  int score_lim = 0;
  if (WITH_SCORE) score_lim = min(a.score_len[b], nA);
  float* score_row = WITH_SCORE ? a.score_out + ((size_t)kvh * a.B + b) * a.score_stride : nullptr;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int nt = tile + ST - 1;
    if constexpr (TMA) {
      __syncthreads();  // every thread is done with tile - 1: its slot may be refilled
      if (tid == 0 && nt < ntiles) issue_tma(nt);
      if (!mbar_wait(&full_bar[tile % ST], (tile / ST) & 1) && a.status) atomicExch(a.status, 5);
      if (WITH_V && tile == ntiles - 1 && r0 + ntiles * TILE > r1) {
        // the last tile reaches past the sequence: those rows hold whatever the cache holds; clear their V
        unsigned char* vt = smem + (tile % ST) * STAGE_BYTES + 2 * TMA_BOX_BYTES;
        const int first_bad = r1 - (r0 + tile * TILE);
        for (int i = tid; i < (TILE - first_bad) * 16; i += NTHREADS) {
          const int row = first_bad + (i >> 4), piece = i & 15;  // 16 pieces of 16 bytes per 256-byte row
          *reinterpret_cast<uint4*>(vt + (piece >> 3) * TMA_BOX_BYTES + row * 128 + (piece & 7) * 16) = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
      }
    } else if constexpr (BULK) {
      // every thread is done with tile - 1, so its slot may be refilled; then wait for this tile's bytes
      __syncthreads();
      if (nt < ntiles) issue_bulk(nt, offb_next);
      offb_next = row_offset(nt + 1, my_row);
      if (!mbar_wait(&full_bar[tile % ST], (tile / ST) & 1) && a.status) atomicExch(a.status, 5);
    } else {
      cp_async_wait<ST - 2>();
      __syncthreads();
      if (nt < ntiles) issue_cp(nt % ST, offc_next);
      cp_async_commit();
      resolve_cp(nt + 1, offc_next);
    }
    const unsigned char* ks = smem + (tile % ST) * STAGE_BYTES;
    const unsigned char* vs = ks + (TMA ? 2 * TMA_BOX_BYTES : (PAIR ? (int)(kHeadDim * sizeof(T)) : TILE_BYTES));

    // S = Q K^T for this warp's 16 rows: two n-tiles of 8 rows
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      unsigned kf[4];
      const int row = warp * 16 + 8 * (mi >> 1) + (lane & 7);
      const int col = kk * 16 + 8 * (mi & 1);
      ldmatrix_x4(kf, staged(ks, row, col * 2));
      mma_16816<T>(s[0], qf[kk], kf[0], kf[1]);
      mma_16816<T>(s[1], qf[kk], kf[2], kf[3]);
    }
    const int tile_base = r0 + tile * TILE + warp * 16;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int R = tile_base + 8 * j + 2 * t + (e & 1);
        s[j][e] = (R < r1) ? s[j][e] * a.scale : -INFINITY;
      }

    if (WITH_SCORE) {
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float v = -INFINITY;
          if (g < G) v = s[j][e];
          if (g + 8 < G) v = fmaxf(v, s[j][2 + e]);
          v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
          v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
          v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
          const int R = tile_base + 8 * j + 2 * t + e;
          if (g == 0 && R < score_lim) score_row[R] = v;
        }
    }

    if (WITH_V) {
      unsigned pa[4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_row[h], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = exp2f((m_row[h] - m_use) * kLog2e);
        m_row[h] = m_new;
        const float ml2 = m_use * kLog2e;
        const float p0 = exp2f(fmaf(s[0][2 * h], kLog2e, -ml2));
        const float p1 = exp2f(fmaf(s[0][2 * h + 1], kLog2e, -ml2));
        const float p2 = exp2f(fmaf(s[1][2 * h], kLog2e, -ml2));
        const float p3 = exp2f(fmaf(s[1][2 * h + 1], kLog2e, -ml2));
        l_row[h] = l_row[h] * corr + ((p0 + p1) + (p2 + p3));
        pa[h] = pack2<T>(p0, p1);
        pa[2 + h] = pack2<T>(p2, p3);
#pragma unroll
        for (int nn = 0; nn < 16; ++nn) {
          o[nn][2 * h] *= corr;
          o[nn][2 * h + 1] *= corr;
        }
      }
      // O += P V : 8 steps of 16 output dims
#pragma unroll
      for (int nn = 0; nn < 8; ++nn) {
        unsigned vf[4];
        const int row = warp * 16 + 8 * (mi & 1) + (lane & 7);
        const int col = nn * 16 + 8 * (mi >> 1);
        ldmatrix_x4_trans(vf, staged(vs, row, col * 2));
        mma_16816<T>(o[2 * nn], pa, vf[0], vf[1]);
        mma_16816<T>(o[2 * nn + 1], pa, vf[2], vf[3]);
      }
    }
  }
  if constexpr (MODE == kCopyCpAsync) cp_async_wait<0>();
  ATTN_STAMP(3);  // all tiles consumed
  if (!WITH_V) return;
  __syncthreads();  // every warp is done with the ring: reuse it for the cross-warp merge

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 1);
    l_row[h] += __shfl_xor_sync(0xffffffffu, l_row[h], 2);
  }
  float* o_s = reinterpret_cast<float*>(smem);                  // [NWARPS][16][128]
  float* ml_s = o_s + NWARPS * 16 * kHeadDim;                   // [NWARPS][16][2]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    if (r < G) {
      float* dst = o_s + ((size_t)warp * 16 + r) * kHeadDim;
#pragma unroll
      for (int nn = 0; nn < 16; ++nn) {
        *reinterpret_cast<float2*>(dst + nn * 8 + 2 * t) = make_float2(o[nn][2 * h], o[nn][2 * h + 1]);
      }
      if (t == 0) {
        ml_s[(warp * 16 + r) * 2 + 0] = m_row[h];
        ml_s[(warp * 16 + r) * 2 + 1] = l_row[h];
      }
    }
  }
  __syncthreads();
  for (int r = 0; r < G; ++r) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, ml_s[(w * 16 + r) * 2]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float wgt = exp2f((ml_s[(w * 16 + r) * 2] - Mu) * kLog2e);
      acc += o_s[((size_t)w * 16 + r) * kHeadDim + tid] * wgt;
      l += ml_s[(w * 16 + r) * 2 + 1] * wgt;
    }
    if (a.S == 1) {  // one split: this is the result, no partials and no arrival count
      static_cast<T*>(a.out)[(size_t)b * a.q_sb + (size_t)(kvh * G + r) * a.q_sh + tid] =
          from_float<T>(l > 0.f ? acc / l : 0.f);
      continue;
    }
    const size_t base = ((size_t)(b * a.H + kvh * G + r) * a.S + split);
    ws_o[base * kHeadDim + tid] = acc;
    if (tid == 0) {
      ws_ml[base * 2 + 0] = M;
      ws_ml[base * 2 + 1] = l;
    }
  }
  if (a.S == 1) return;
  ATTN_STAMP(4);  // partials written
  // the shared scratch of finish_group starts behind the cross-warp merge area used above
  if (a.coop_merge) coop_merge<T>(a, b, kvh, split, &last_flag);
  else finish_group<T>(a, b, kvh, ml_s + NWARPS * 16 * 2, &last_flag);
  ATTN_STAMP(5);  // counted in (and, for the last CTA of the group, merged)
}

// ---------------------------------------------------------------------------------------------
// fp32 CUDA-core kernel.  One warp per row at a time (a 512-byte row is one coalesced request,
// lane L holds dims 4L..4L+3), four rows in flight per warp.
// ---------------------------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(NTHREADS) decode_attn_f32_kernel(const AttnArgs a, const bool with_v,
                                                                    const bool with_score) {
  __shared__ float o_s[NWARPS][G][kHeadDim];
  __shared__ float ml_s[NWARPS][G][2];
  __shared__ float w_s[NWARPS * 512];
  __shared__ int last_flag;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nA = a.lenA[b];
  const int nB = a.lenB ? a.lenB[b] : 0;
  const int n = nA + nB;
  int r0, r1;
  split_range(n, a.B > 1 ? batch_max_rows(a, n) : n, a.S, split, r0, r1);

  const float* kA = static_cast<const float*>(a.kA) + (size_t)b * a.a_sb + (size_t)kvh * a.a_sh;
  const float* vA = with_v ? static_cast<const float*>(a.vA) + (size_t)b * a.a_sb + (size_t)kvh * a.a_sh : nullptr;
  const float* kB = a.kB ? static_cast<const float*>(a.kB) + (size_t)b * a.b_sb + (size_t)kvh * a.b_sh : nullptr;
  const float* vB = (with_v && a.vB) ? static_cast<const float*>(a.vB) + (size_t)b * a.b_sb + (size_t)kvh * a.b_sh : nullptr;
  const int* idx = a.idxA ? a.idxA + (size_t)(a.idx_row ? a.idx_row[b] : b) * a.idx_stride : nullptr;
  const int startB = a.startB ? a.startB[b] : 0;
  const int score_lim = with_score ? min(a.score_len[b], nA) : 0;
  float* score_row = with_score ? a.score_out + ((size_t)kvh * a.B + b) * a.score_stride : nullptr;

  float4 qv[G];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const float* qp = static_cast<const float*>(a.q) + (size_t)b * a.q_sb + (size_t)(kvh * G + h) * a.q_sh;
    qv[h] = *reinterpret_cast<const float4*>(qp + lane * 4);
  }
  float m[G], l[G];
  float4 acc[G];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
    acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  constexpr int U = 4;
  for (int base = r0 + warp * U; base < r1; base += NWARPS * U) {
    float4 kx[U], vx[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int R = base + u;
      kx[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      vx[u] = kx[u];
      if (R < r1) {
        const float* kp;
        const float* vp = nullptr;
        if (R < nA) {
          const size_t pos = idx ? (size_t)idx[R] : (size_t)R;
          kp = kA + pos * a.a_sr;
          if (with_v) vp = vA + pos * a.a_sr;
        } else {
          const size_t pos = (size_t)(startB + (R - nA));
          kp = kB + pos * a.b_sr;
          if (with_v) vp = vB + pos * a.b_sr;
        }
        kx[u] = __ldg(reinterpret_cast<const float4*>(kp) + lane);
        if (with_v) vx[u] = __ldg(reinterpret_cast<const float4*>(vp) + lane);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int R = base + u;
      if (R >= r1) break;  // warp-uniform
      float sc[G];
      float best = -INFINITY;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float d = qv[h].x * kx[u].x;
        d = fmaf(qv[h].y, kx[u].y, d);
        d = fmaf(qv[h].z, kx[u].z, d);
        d = fmaf(qv[h].w, kx[u].w, d);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        sc[h] = d * a.scale;
        best = fmaxf(best, sc[h]);
      }
      if (with_score && lane == 0 && R < score_lim) score_row[R] = best;
      if (with_v) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float m_new = fmaxf(m[h], sc[h]);  // finite: sc is a finite dot product
          const float corr = exp2f((m[h] - m_new) * kLog2e);
          const float p = exp2f((sc[h] - m_new) * kLog2e);
          m[h] = m_new;
          l[h] = l[h] * corr + p;
          acc[h].x = fmaf(p, vx[u].x, acc[h].x * corr);
          acc[h].y = fmaf(p, vx[u].y, acc[h].y * corr);
          acc[h].z = fmaf(p, vx[u].z, acc[h].z * corr);
          acc[h].w = fmaf(p, vx[u].w, acc[h].w * corr);
        }
      }
    }
  }
  if (!with_v) return;
#pragma unroll
  for (int h = 0; h < G; ++h) {
    *reinterpret_cast<float4*>(&o_s[warp][h][lane * 4]) = acc[h];
    if (lane == 0) {
      ml_s[warp][h][0] = m[h];
      ml_s[warp][h][1] = l[h];
    }
  }
  __syncthreads();
  for (int h = 0; h < G; ++h) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, ml_s[w][h][0]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float accv = 0.f, lv = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = ml_s[w][h][0];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f((mw - Mu) * kLog2e);
      accv += o_s[w][h][tid] * wgt;
      lv += ml_s[w][h][1] * wgt;
    }
    const size_t base = ((size_t)(b * a.H + kvh * G + h) * a.S + split);
    a.ws_o[base * kHeadDim + tid] = accv;
    if (tid == 0) {
      a.ws_ml[base * 2 + 0] = M;
      a.ws_ml[base * 2 + 1] = lv;
    }
  }
  finish_group<float>(a, b, kvh, w_s, &last_flag);
}

template <typename T>
int launch_mma(AttnArgs a, bool with_v, bool with_score, int64_t a_rows, cudaStream_t st) {
  dim3 grid(a.S, a.KVH, a.B), block(NTHREADS);
  int dev = 0, n_sms = 0;
  OMNIKV_CUDA_OK(cudaGetDevice(&dev));
  OMNIKV_CUDA_OK(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev));
  a.pdl_trigger = ((long long)a.S * a.KVH * a.B <= 2ll * n_sms) ? 1 : 0;  // two CTAs of this kernel fit per SM
#ifdef OMNIKV_TRACE
  a.trace_slot = trace_next_slot();
#endif
  // scattered rows: one bulk copy per row; a contiguous cache of known capacity: tensor-map tiles; else cp.async
  int mode = a.idxA != nullptr ? kCopyBulkRows : kCopyCpAsync;
  CUtensorMap tm_k = {}, tm_v = {};
  constexpr bool is_bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;
  if (mode == kCopyCpAsync && a_rows > 0 && !a.lenB && g_attn_tma_enabled() &&
      make_kv_tensor_map(&tm_k, is_bf16, a.kA, a_rows, a.KVH, a.B, a.a_sr, a.a_sh, a.a_sb) &&
      (!with_v || make_kv_tensor_map(&tm_v, is_bf16, a.vA, a_rows, a.KVH, a.B, a.a_sr, a.a_sh, a.a_sb)))
    mode = kCopyTma;
  auto go = [&](auto kern, int smem) -> int {
    OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    // many splits (64 or more: one or two local KV heads under tensor parallelism) and a grid that is resident as a
    // whole: the splits merge together.  With fewer splits the CTAs that wait hold their SMs longer than the merge by
    // the last CTA costs (measured at 37 splits x 8 KV heads: 3.57 against 3.53 ms per step).
    a.coop_merge = 0;
    if (mode != kCopyCpAsync && with_v && a.S >= 64 && a.S <= 256 && a.B * a.KVH <= 2048 && g_attn_coop_enabled()) {
      int per_sm = 0;
      OMNIKV_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NTHREADS, smem));
      if ((long long)a.S * a.KVH * a.B <= (long long)per_sm * n_sms) a.coop_merge = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OMNIKV_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, a, tm_k, tm_v));
    return OMNIKV_OK;
  };
  const int smem_v = mma_smem_bytes<true>(), smem_k = mma_smem_bytes<false>();
  const int tma_v = STAGES * 4 * TMA_BOX_BYTES + Q_BYTES + 1024, tma_k = STAGES * 2 * TMA_BOX_BYTES + Q_BYTES + 1024;
  int rc;
#define OMNIKV_ATTN_GO(V, SC)                                                                         \
  (mode == kCopyTma        ? go(decode_attn_mma_kernel<T, V, SC, kCopyTma>, V ? tma_v : tma_k)        \
   : mode == kCopyBulkRows ? go(decode_attn_mma_kernel<T, V, SC, kCopyBulkRows>, V ? smem_v : smem_k) \
                           : go(decode_attn_mma_kernel<T, V, SC, kCopyCpAsync>, V ? smem_v : smem_k))
  // scattered rows of a cache whose V row lies right behind the K row of the same position: one copy per position
  const size_t row_b = kHeadDim * sizeof(T);
  const bool pairs = mode == kCopyBulkRows && with_v && !with_score && sizeof(T) == 2 &&
                     static_cast<const unsigned char*>(a.vA) == static_cast<const unsigned char*>(a.kA) + row_b &&
                     (!a.kB || static_cast<const unsigned char*>(a.vB) == static_cast<const unsigned char*>(a.kB) + row_b);
  if (pairs) rc = go(decode_attn_mma_kernel<T, true, false, kCopyBulkPairs>, smem_v);
  else if (with_v && with_score) rc = OMNIKV_ATTN_GO(true, true);
  else if (with_v) rc = OMNIKV_ATTN_GO(true, false);
  else rc = OMNIKV_ATTN_GO(false, true);
#undef OMNIKV_ATTN_GO
  if (rc != OMNIKV_OK) return rc;
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

// ---------------------------------------------------------------------------------------------
// fp32 selector-`last` scores of a contiguous cache, as a stream: the rows of one (sequence, KV head) are
// consecutive in memory, so a tile of 64 rows is ONE 32 KB bulk copy into a three-stage ring (a producer thread,
// mbarrier transaction counts), which keeps ~190 KB per SM in flight -- the register-staged kernel above holds 8 KB
// per CTA and is bound by the memory latency.  Eight consumer warps take eight rows of a tile each (lane L holds
// dims 4L..4L+3 of the row and of the G queries), the eight scores of a warp leave as one 32-byte store.
// ---------------------------------------------------------------------------------------------
constexpr int SL_ROWS = 64, SL_STAGES = 3, SL_WARPS = 8, SL_THREADS = (SL_WARPS + 1) * 32;
constexpr int SL_TILE_BYTES = SL_ROWS * kHeadDim * 4;
constexpr int SL_SMEM_BYTES = SL_STAGES * SL_TILE_BYTES + 128;

template <int G>
__global__ void __launch_bounds__(SL_THREADS) score_last_f32_stream_kernel(const AttnArgs a) {
  extern __shared__ __align__(128) unsigned char sl_smem_raw[];
  __shared__ uint64_t full[SL_STAGES], empty[SL_STAGES];
  __shared__ int fail;
  float* ring = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(sl_smem_raw) + 127) & ~(uintptr_t)127);
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = min(a.score_len[b], a.lenA[b]);  // rows that get a score
  int r0, r1;
  split_range(n, n, a.S, split, r0, r1);
  const int n_tiles = r1 > r0 ? ceil_div(r1 - r0, SL_ROWS) : 0;
  const float* k = static_cast<const float*>(a.kA) + (size_t)b * a.a_sb + (size_t)kvh * a.a_sh;
  float* score_row = a.score_out + ((size_t)kvh * a.B + b) * a.score_stride;
  if (tid == 0) {
    fail = 0;
    for (int s = 0; s < SL_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], SL_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  if (warp == SL_WARPS) {
    if (lane == 0) {
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % SL_STAGES;
        if (!mbar_wait(&empty[s], ((t / SL_STAGES) & 1) ^ 1, &fail)) {
          if (!fail && a.status) atomicExch(a.status, 5);
          fail = 1;
          break;
        }
        const int row = r0 + t * SL_ROWS;
        const unsigned bytes = (unsigned)min(SL_ROWS, r1 - row) * kHeadDim * 4;
        mbar_expect_tx(&full[s], bytes);
        tma_bulk_g2s(ring + (size_t)s * SL_ROWS * kHeadDim, k + (size_t)row * kHeadDim, bytes, &full[s]);
      }
    }
    return;  // copies in flight are waited for by the consumers (a consumer that gives up leaves them to the 2 s bound)
  }
  float4 qv[G];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const float* qp = static_cast<const float*>(a.q) + (size_t)b * a.q_sb + (size_t)(kvh * G + h) * a.q_sh;
    qv[h] = *reinterpret_cast<const float4*>(qp + lane * 4);
  }
  for (int t = 0; t < n_tiles; ++t) {
    const int s = t % SL_STAGES;
    if (!mbar_wait(&full[s], (t / SL_STAGES) & 1, &fail)) {
      if (!fail && a.status) atomicExch(a.status, 5);
      fail = 1;
      break;
    }
    const int row0 = r0 + t * SL_ROWS + warp * 8;  // this warp's eight rows
    const float4* tile = reinterpret_cast<const float4*>(ring + (size_t)s * SL_ROWS * kHeadDim) + warp * 8 * 32;
    float4 kx[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) kx[i] = tile[i * 32 + lane];
    float mine = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float best = -INFINITY;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float d = qv[h].x * kx[i].x;
        d = fmaf(qv[h].y, kx[i].y, d);
        d = fmaf(qv[h].z, kx[i].z, d);
        d = fmaf(qv[h].w, kx[i].w, d);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        best = fmaxf(best, d * a.scale);
      }
      if (lane == i) mine = best;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);  // the tile's rows are in registers: the stage may be refilled
    if (lane < 8 && row0 + lane < r1) score_row[row0 + lane] = mine;
  }
  if (fail) {
    // a wait ran out: let every copy that was asked for land (bounded) before the shared memory is given up
    for (int s = 0; s < SL_STAGES; ++s) mbar_wait(&full[s], 0);
  }
}

template <int G>
int launch_score_stream(const AttnArgs& a, cudaStream_t st) {
  auto kern = score_last_f32_stream_kernel<G>;
  static bool attr_set = false;
  if (!attr_set) {
    OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SL_SMEM_BYTES));
    attr_set = true;
  }
  kern<<<dim3(a.S, a.KVH, a.B), SL_THREADS, SL_SMEM_BYTES, st>>>(a);
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

int launch_f32(const AttnArgs& a, bool with_v, bool with_score, cudaStream_t st) {
  // scores only over a cache whose rows lie back to back: the streaming kernel
  if (!with_v && with_score && !a.idxA && !a.kB && a.a_sr == kHeadDim && a.a_sb % 4 == 0 && a.a_sh % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(a.kA) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0) {
    switch (a.G) {
      case 1: return launch_score_stream<1>(a, st);
      case 2: return launch_score_stream<2>(a, st);
      case 4: return launch_score_stream<4>(a, st);
      case 8: return launch_score_stream<8>(a, st);
      default: break;
    }
  }
  dim3 grid(a.S, a.KVH, a.B), block(NTHREADS);
  switch (a.G) {
    case 1: decode_attn_f32_kernel<1><<<grid, block, 0, st>>>(a, with_v, with_score); break;
    case 2: decode_attn_f32_kernel<2><<<grid, block, 0, st>>>(a, with_v, with_score); break;
    case 4: decode_attn_f32_kernel<4><<<grid, block, 0, st>>>(a, with_v, with_score); break;
    case 8: decode_attn_f32_kernel<8><<<grid, block, 0, st>>>(a, with_v, with_score); break;
    default: return OMNIKV_E_UNSUPPORTED;
  }
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace omnikv

extern "C" size_t omnikv_decode_attn_workspace_bytes(int B, int H, int n_splits) {
  if (B <= 0 || H <= 0 || n_splits <= 0) return 0;
  // [arrival counters: a fixed 16 KiB region, so that calls of different shapes sharing one workspace agree
  //  on where it is][o partials][m, l partials]
  return omnikv::kAttnCntBytes +
         (omnikv::attn_ws_o_floats(B, H, n_splits) + omnikv::attn_ws_ml_floats(B, H, n_splits)) * sizeof(float);
}

// Host-side validation of a call (everything except the workspace).  OMNIKV_OK or the status to return.
static int validate_attn_params(const omnikv_attn_params* p) {
  using namespace omnikv;
  if (!p || !p->q || !p->kA || !p->lenA) return OMNIKV_E_BADARG;
  if (p->B <= 0 || p->H <= 0 || p->KVH <= 0 || p->n_splits <= 0) return OMNIKV_E_BADARG;
  if (p->head_dim != kHeadDim) return OMNIKV_E_UNSUPPORTED;
  if (p->H % p->KVH != 0) return OMNIKV_E_BADARG;
  const int G = p->H / p->KVH;
  const bool with_v = p->out != nullptr;
  const bool with_score = p->score_out != nullptr;
  if (!with_v && !with_score) return OMNIKV_E_BADARG;
  if (with_v && !p->vA) return OMNIKV_E_BADARG;
  if (with_score && (!p->score_len || p->score_stride <= 0)) return OMNIKV_E_BADARG;
  if (p->idx_row && !p->idxA) return OMNIKV_E_BADARG;
  if (p->lenB && (!p->kB || !p->startB || (with_v && !p->vB))) return OMNIKV_E_BADARG;
  const int esz = p->dtype == OMNIKV_F32 ? 4 : 2;
  const int vec = 16 / esz;  // elements per 16-byte vector
  if (p->dtype != OMNIKV_F32 && p->dtype != OMNIKV_BF16 && p->dtype != OMNIKV_F16) return OMNIKV_E_UNSUPPORTED;
  if (!aligned16(p->q) || !aligned16(p->kA) || (p->vA && !aligned16(p->vA)) || (p->kB && !aligned16(p->kB)) ||
      (p->vB && !aligned16(p->vB)))
    return OMNIKV_E_BADARG;
  if (p->q_stride_b % vec || p->q_stride_h % vec || p->a_stride_b % vec || p->a_stride_h % vec ||
      p->a_stride_row % vec || p->a_stride_row < kHeadDim)
    return OMNIKV_E_BADARG;
  if (p->lenB && (p->b_stride_b % vec || p->b_stride_h % vec || p->b_stride_row % vec || p->b_stride_row < kHeadDim))
    return OMNIKV_E_BADARG;
  if (p->dtype == OMNIKV_F32 ? (G != 1 && G != 2 && G != 4 && G != 8) : (G > 16)) return OMNIKV_E_UNSUPPORTED;
  if (with_v && (p->n_splits > 512 || (size_t)p->B * p->KVH * 4 > kAttnCntBytes)) return OMNIKV_E_UNSUPPORTED;
  return OMNIKV_OK;
}

extern "C" int omnikv_decode_attn(const omnikv_attn_params* p, void* stream) {
  using namespace omnikv;
  if (const int rc = validate_attn_params(p)) return rc;
  const int G = p->H / p->KVH;
  const bool with_v = p->out != nullptr;
  const bool with_score = p->score_out != nullptr;
  if (with_v) {
    if (!p->workspace || p->workspace_bytes < omnikv_decode_attn_workspace_bytes(p->B, p->H, p->n_splits))
      return OMNIKV_E_WORKSPACE;
    if (!aligned16(p->workspace)) return OMNIKV_E_BADARG;
  }
  AttnArgs a;
  a.q = p->q; a.q_sb = p->q_stride_b; a.q_sh = p->q_stride_h; a.out = p->out;
  a.kA = p->kA; a.vA = p->vA; a.a_sb = p->a_stride_b; a.a_sh = p->a_stride_h; a.a_sr = p->a_stride_row;
  a.idxA = p->idxA; a.idx_row = p->idx_row; a.idx_stride = p->idx_stride; a.lenA = p->lenA;
  a.kB = p->lenB ? p->kB : nullptr; a.vB = p->lenB ? p->vB : nullptr;
  a.b_sb = p->b_stride_b; a.b_sh = p->b_stride_h; a.b_sr = p->b_stride_row;
  a.startB = p->startB; a.lenB = p->lenB;
  a.score_out = p->score_out; a.score_stride = p->score_stride; a.score_len = p->score_len;
  a.ws_cnt = static_cast<unsigned*>(p->workspace);
  a.ws_o = with_v ? reinterpret_cast<float*>(static_cast<unsigned char*>(p->workspace) + kAttnCntBytes) : nullptr;
  a.ws_ml = with_v ? a.ws_o + attn_ws_o_floats(p->B, p->H, p->n_splits) : nullptr;
  a.B = p->B; a.H = p->H; a.KVH = p->KVH; a.G = G; a.S = p->n_splits;
  a.scale = p->scale;
  a.pdl_trigger = 0;
  a.trace_slot = 0;
  a.status = p->status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (p->dtype) {
    case OMNIKV_BF16: return launch_mma<__nv_bfloat16>(a, with_v, with_score, p->a_rows, st);
    case OMNIKV_F16: return launch_mma<__half>(a, with_v, with_score, p->a_rows, st);
    default: return launch_f32(a, with_v, with_score, st);
  }
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library have no allocator to hand: a plugin that is only given tensors by a runtime
// that owns all device memory, a process with a memory budget fixed at start-up, a real-time loop that must
// not touch cudaMalloc (it can block and synchronise the device).  For
// them the split partials and arrival counters live in the array below, which is part of the library's
// image: every GPU that loads the library holds these 4 MiB until the process exits.
// ---------------------------------------------------------------------------------------------
namespace omnikv {
namespace {

static __device__ __align__(256) unsigned char g_no_alloc_scratch[OMNIKV_NO_ALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// device address of the array, per device ordinal; filled on a device's first call.  Several host threads may
// make that first call at once: they all look up the same address, and the slot is read and written atomically.
std::atomic<void*> g_no_alloc_ptr[kMaxDevices];

// The array's name is only a handle on the host; the device address has to be asked for, once per
// device and with that device current.
int no_alloc_scratch(void** out) {
  int dev = 0;
  OMNIKV_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return OMNIKV_E_UNSUPPORTED;
  void* ptr = g_no_alloc_ptr[dev].load(std::memory_order_acquire);
  if (!ptr) {
    OMNIKV_CUDA_OK(cudaGetSymbolAddress(&ptr, g_no_alloc_scratch));
    if (!ptr) return OMNIKV_E_CUDA;
    g_no_alloc_ptr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return OMNIKV_OK;
}

}  // namespace
}  // namespace omnikv

extern "C" int omnikv_decode_attn_no_alloc(const omnikv_attn_params* p, void* stream) {
  using namespace omnikv;
  // every check comes first: a refused call puts nothing on the stream and leaves the shared array alone
  if (!p) return OMNIKV_E_BADARG;
  if (p->B <= 0 || p->H <= 0 || p->n_splits <= 0) return OMNIKV_E_BADARG;
  if (p->out && omnikv_decode_attn_workspace_bytes(p->B, p->H, p->n_splits) > (size_t)OMNIKV_NO_ALLOC_SCRATCH_BYTES)
    return OMNIKV_E_WORKSPACE;  // B * H * n_splits is more than the built-in scratch can hold
  if (const int bad = validate_attn_params(p)) return bad;
  void* scratch = nullptr;
  const int rc = no_alloc_scratch(&scratch);
  if (rc != OMNIKV_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps what the previous call left.  Only the arrival counters have to start at zero (a call
  // that ran to completion leaves them so, one that was cut short may not): clear them on the same stream.
  OMNIKV_CUDA_OK(cudaMemsetAsync(scratch, 0, kAttnCntBytes, st));
  omnikv_attn_params q = *p;
  q.workspace = scratch;
  q.workspace_bytes = OMNIKV_NO_ALLOC_SCRATCH_BYTES;
  return omnikv_decode_attn(&q, stream);
}

#ifdef OMNIKV_TRACE
extern "C" int omnikv_debug_attn_trace(unsigned long long* host_out, int n_words) {
  return (int)cudaMemcpyFromSymbol(host_out, omnikv::g_attn_trace, (size_t)n_words * 8);
}
#endif
