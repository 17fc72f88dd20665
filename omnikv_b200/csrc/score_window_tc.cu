// Window-selector scores on the Blackwell tensor path (tcgen05.mma, accumulators in tensor memory).
//
//   A[h,w,p]  = softmax over p' < C of (qw[h,w,:] . K[h/G,p',:] * scale)
//   score[p]  = sum_w weight_w * max_h A[h,w,p]
//
// The contraction of a KV head's query block ([G heads x 16 window slots] x 128) with a tile of 128 keys is one
// tcgen05.mma group: the K tile (128 keys x 128, two TMA boxes with the 128-byte swizzle) is the A operand
// (M = 128 keys), the query block the B operand (N = 16 G columns), the fp32 accumulator [128 keys x N] lives in
// tensor memory: key p of the tile is TMEM lane p, so an epilogue thread owns ONE key and reads its N logits with
// tcgen05.ld.  One elected thread issues the MMAs, one the TMA copies, four warps do the arithmetic that is left --
// which is small, because both passes work on logarithms:
//
//   pass 1  grid (splits, KVH, B): c[h,w] = log2 sum_p 2^(x[h,w,p]), x = logit * scale * log2(e).  A thread keeps a
//           private sum per column for its keys, relative to a per-column offset shared by the CTA (set from the
//           first tile, raised -- rarely -- when a later logit exceeds it by more than 2^16); the 128 private sums
//           are added once at the end.  One exp2 per (key, column).
//   pass 2  grid (CTAs per sequence, B): max_h A[h,w,p] = 2^(max_h (x[h,w,p] - c[h,w])) because 2^x is monotonic,
//           so a thread takes the max over ALL heads of a key in the log domain (every KV head's query block is
//           resident in shared memory and the CTA walks the KV heads of its key tile) and needs 16 exp2 per key,
//           not 16 per (key, head).  The score of a key is complete inside one thread: no atomics, no planes.
//
// Both passes are HBM streams of K (pass 2 re-reads it: the normaliser has to be known before the max over heads).
// Every wait is bounded by time; on expiry the CTA raises a flag, every role leaves its loop, the tensor memory
// is released and a status code is written.
#include <type_traits>

#include "common.cuh"
#include "score_window_tc.cuh"
#include "tc05.cuh"

namespace omnikv {
namespace {

constexpr int TC_TILE = 128;                 // keys per MMA group = TMEM lanes
constexpr int TC_KTILE_BYTES = TC_TILE * 256;  // a staged K tile: two boxes of 128 rows x 128 bytes
constexpr int TC_BOX_BYTES = TC_TILE * 128;
constexpr int TC_THREADS = 192;              // warps 0-3: epilogue (TMEM lane quarters), 4: TMA producer, 5: MMA issuer
constexpr int TC_WPAD = 16;

// Instruction descriptor of this file's MMAs: both operands K-major, M = 128 keys, N columns.
template <typename T>
__device__ __forceinline__ unsigned instr_desc(int N) { return tc_instr_desc<T>(TC_TILE, N, false, false); }

// Query block of KV head `kvh` -> shared memory as the B operand: N = 16 G rows (head-major, window padded to 16
// slots, rows >= W zero) x 128, two boxes of [N rows x 128 bytes], 16-byte chunk c of row r at chunk c ^ (r & 7).
// Loads go out in batches of eight before their stores: written as load, store, load, store ... every iteration
// would cost a memory round trip (the compiler keeps a load behind an earlier store through a generic pointer).
template <typename T>
__device__ __forceinline__ void stage_q_block(unsigned char* dst, const T* qw_b, int h0, int G, int W, int tid, int nthreads) {
  const int N = G * TC_WPAD;
  const int total = N * 16;  // 16-byte chunks
  for (int base = 0; base < total; base += 8 * nthreads) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + tid + u * nthreads;
      const int r = i >> 4, c = i & 15;  // row, 16-byte chunk of the 256-byte row
      const int hl = r / TC_WPAD, w = r % TC_WPAD;
      v[u] = make_uint4(0, 0, 0, 0);
      if (i < total && w < W) v[u] = *reinterpret_cast<const uint4*>(qw_b + ((size_t)(h0 + hl) * W + w) * kHeadDim + c * 8);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + tid + u * nthreads;
      const int r = i >> 4, c = i & 15;
      if (i < total) {
        unsigned char* box = dst + (c >> 3) * (N * 128);
        *reinterpret_cast<uint4*>(box + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v[u];
      }
    }
  }
}

// Accumulators in flight: the MMAs of a tile, their completion signal and the epilogue's read of tensor memory are a
// chain of latencies; four buffers of N <= 64 columns (half of the 512 columns at most) keep it from pacing the stream.
constexpr int kAccBufs = 4;

struct TcShared {
  uint64_t full[6];
  uint64_t empty[6];
  uint64_t acc_full[4];
  uint64_t acc_empty[4];
  unsigned tmem_base;
  int fail;
  int issued;  // K tiles the producer has asked for (read at teardown after a failure)
};

// ---- the three roles, shared by both passes ------------------------------------------------------------------
// Sub-tile j of a CTA is (key tile tile_of(j), KV head kvh_of(j)); its K rows start at row0_of(j).
template <int STAGES, typename F>
__device__ __forceinline__ void produce_tiles(TcShared& sh, unsigned char* ring, const CUtensorMap* map, int n_sub, int b,
                                              F sub, int* status) {
  for (int j = 0; j < n_sub; ++j) {
    const int s = j % STAGES;
    if (!mbar_wait(&sh.empty[s], ((j / STAGES) & 1) ^ 1, &sh.fail)) {
      if (!sh.fail && status) atomicExch(status, 5);
      sh.fail = 1;
      return;
    }
    int row0, kvh;
    sub(j, row0, kvh);
    unsigned char* dst = ring + (size_t)s * TC_KTILE_BYTES;
    mbar_expect_tx(&sh.full[s], TC_KTILE_BYTES);
    tma_load_4d(dst, map, 0, row0, kvh, b, &sh.full[s]);
    tma_load_4d(dst + TC_BOX_BYTES, map, 64, row0, kvh, b, &sh.full[s]);
    sh.issued = j + 1;
  }
}

template <typename T, int STAGES, typename F>
__device__ __forceinline__ void issue_mmas(TcShared& sh, unsigned char* ring, unsigned char* q_s, int N, int n_sub, F sub,
                                           int* status) {
  const unsigned idesc = instr_desc<T>(N);
  for (int j = 0; j < n_sub; ++j) {
    const int s = j % STAGES, buf = j % kAccBufs;
    if (!mbar_wait(&sh.full[s], (j / STAGES) & 1, &sh.fail) ||
        !mbar_wait(&sh.acc_empty[buf], ((j / kAccBufs) & 1) ^ 1, &sh.fail)) {
      if (!sh.fail && status) atomicExch(status, 5);
      sh.fail = 1;
      return;
    }
    tc_fence_after();
    int row0, kvh_slot;
    sub(j, row0, kvh_slot);  // kvh_slot: which resident query block this sub-tile meets
    const unsigned a_base = smem_u32(ring + (size_t)s * TC_KTILE_BYTES);
    const unsigned b_base = smem_u32(q_s + (size_t)kvh_slot * N * 256);
    const unsigned d_tmem = sh.tmem_base + (unsigned)(buf * N);  // accumulator buf: columns [buf * N, +N)
#pragma unroll
    for (int k = 0; k < 8; ++k) {  // 8 steps of 16 elements along head_dim: 4 per 128-byte box row, then the other box
      const uint64_t a_desc = smem_desc_sw128(a_base + (k >> 2) * TC_BOX_BYTES + (k & 3) * 32);
      const uint64_t b_desc = smem_desc_sw128(b_base + (k >> 2) * (N * 128) + (k & 3) * 32);
      tc_mma(d_tmem, a_desc, b_desc, idesc, k > 0 ? 1u : 0u);
    }
    tc_commit(&sh.empty[s]);        // the K tile may be overwritten once these MMAs have read it
    tc_commit(&sh.acc_full[buf]);   // ... and the accumulator is complete
  }
}

// Epilogue side: wait for accumulator `j`, read NC of this thread's logits (columns col0 .. col0 + NC of its TMEM
// lane) into v, hand the buffer back.  lane_quarter = warp & 3 (a warp reaches the 32 lanes of its quarter only).
template <int NC>
__device__ __forceinline__ bool take_accumulator(TcShared& sh, int j, float (&v)[NC], int lane_quarter, int acc_col0,
                                                 int* status) {
  static_assert(NC % 16 == 0, "columns are read 16 at a time");
  const int buf = j % kAccBufs;
  if (!mbar_wait(&sh.acc_full[buf], (j / kAccBufs) & 1, &sh.fail)) {
    if (!sh.fail && status) atomicExch(status, 5);
    sh.fail = 1;
    return false;
  }
  tc_fence_after();
  const unsigned taddr = sh.tmem_base + ((unsigned)(lane_quarter * 32) << 16) + (unsigned)acc_col0;
#pragma unroll
  for (int c = 0; c < NC; c += 16) tmem_ld16(taddr + c, *reinterpret_cast<float(*)[16]>(&v[c]));
  tmem_ld_wait();
  tc_fence_before();
  mbar_arrive(&sh.acc_empty[buf]);
  return true;
}

// Setup in two halves: the first touches no global memory, the second publishes the staged query blocks.
template <int STAGES>
__device__ __forceinline__ void tc_setup_begin(TcShared& sh, unsigned ncols, int warp, int n_epilogue_threads) {
  if (threadIdx.x == 0) {
    sh.fail = 0;
    sh.issued = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (int i = 0; i < kAccBufs; ++i) {
      mbar_init(&sh.acc_full[i], 1);
      mbar_init(&sh.acc_empty[i], n_epilogue_threads);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {  // one warp allocates the tensor memory and gives the permit back
    tmem_alloc(&sh.tmem_base, ncols);
    tmem_relinquish();
  }
}

__device__ __forceinline__ void tc_setup_end() {
  // the query block was written with ordinary stores; the tensor core reads it through the async proxy
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

template <int STAGES>
__device__ __forceinline__ void tc_teardown(TcShared& sh, unsigned ncols, int warp, int producer_tid) {
  tc_fence_before();
  __syncthreads();  // every role is out of its loop: no MMA, copy or TMEM read of this CTA is still wanted
  if (sh.fail) {
    // a wait ran out: copies that were asked for may still be on their way into this CTA's shared memory.  Wait
    // (bounded) for each stage's last requested tile before the memory is given up.
    if ((int)threadIdx.x == producer_tid) {
      for (int s = 0; s < STAGES; ++s) {
        const int last = sh.issued - 1 - ((sh.issued - 1 - s) % STAGES + STAGES) % STAGES;  // last j < issued with j % STAGES == s
        if (sh.issued > s && last >= 0) mbar_wait(&sh.full[s], (last / STAGES) & 1);
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(sh.tmem_base, ncols);
  }
}

__host__ __device__ constexpr unsigned tmem_cols(int N) {  // kAccBufs accumulators of N columns, a power of two >= 32
  return kAccBufs * N <= 32 ? 32u : (kAccBufs * N <= 64 ? 64u : (kAccBufs * N <= 128 ? 128u : (kAccBufs * N <= 256 ? 256u : 512u)));
}

// ---- pass 1 ------------------------------------------------------------------------------------------------------
// 16 G accumulator columns per key.  With 32 columns or more two warps share a TMEM lane quarter and split the
// columns (eight epilogue warps, two per scheduler: one warp alone cannot hide its own latencies, and the exp2 and
// add per (key, column) of this pass made a four-warp epilogue the limit, not the K stream).
constexpr int P1_STAGES = 2;  // two CTAs per SM (see window_tc_pass1): 128 KB of K in flight per SM
template <int G>
struct P1Shape {
  static constexpr int N = G * TC_WPAD;
  static constexpr int HALVES = N >= 32 ? 2 : 1;
  static constexpr int NC = N / HALVES;        // columns per epilogue thread
  static constexpr int EPI = 128 * HALVES;     // epilogue threads
  static constexpr int THREADS = EPI + 64;     // + TMA producer warp + MMA warp
};

template <int EPI>
__device__ __forceinline__ unsigned bar_or_epi(bool pred) {  // OR over the epilogue threads (named barrier 1)
  unsigned r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.b32 p, %1, 0;\n"
      "barrier.cta.red.or.pred q, 1, %2, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(r)
      : "r"((unsigned)pred), "n"(EPI)
      : "memory");
  return r;
}
template <int EPI>
__device__ __forceinline__ void bar_sync_epi() { asm volatile("bar.sync 1, %0;\n" ::"n"(EPI) : "memory"); }

template <typename T, int G>
__global__ void __launch_bounds__(P1Shape<G>::THREADS, 2) window_tc_pass1(const WinTcArgs a, const __grid_constant__ CUtensorMap tm_k) {
  using S_ = P1Shape<G>;
  constexpr int N = S_::N, NC = S_::NC, EPI = S_::EPI, THREADS = S_::THREADS;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TcShared sh;
  __shared__ float off_s[N];    // per-column offset (log2 domain) shared by the CTA
  __shared__ float shift_s[N];
  __shared__ float cmax_s[4][N];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;
  unsigned char* q_s = smem + P1_STAGES * TC_KTILE_BYTES;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Launched as a programmatic dependent: the CTAs are scheduled while the previous kernel of the stream drains, and
  // touch no global memory before it has completed.  The trigger comes AFTER the wait, so a pass-2 CTA that starts
  // early knows that everything older than this launch (lengths, window queries, K) is complete and visible.
  pdl_wait();
  pdl_trigger();
  const int n = a.consider_len[b];
  // chunks are sized by the LONGEST sequence of the batch: every CTA then has the same amount of work, a short
  // sequence uses fewer of its S splits (the others hand in empty partials)
  int n_max = n;
  for (int bb = 0; bb < a.B; ++bb) n_max = max(n_max, a.consider_len[bb]);
  const int chunk = ceil_div(ceil_div(n_max, a.S), TC_TILE) * TC_TILE;
  const int r0 = min(n, split * chunk), r1 = min(n, r0 + chunk);
  const int n_sub = r1 > r0 ? ceil_div(r1 - r0, TC_TILE) : 0;
  float* part = a.part + ((((size_t)b * a.H + kvh * G) * TC_WPAD) * a.S + split) * 2;  // + (hl*16 + w) * S * 2
  if (n_sub == 0) {
    for (int c = tid; c < N; c += THREADS) {
      part[(size_t)c * a.S * 2 + 0] = -INFINITY;
      part[(size_t)c * a.S * 2 + 1] = 0.f;
    }
    return;
  }
  stage_q_block<T>(q_s, static_cast<const T*>(a.qw) + (size_t)b * a.H * a.W * kHeadDim, kvh * G, G, a.W, tid, THREADS);
  tc_setup_begin<P1_STAGES>(sh, tmem_cols(N), warp, EPI);
  tc_setup_end();
  if (warp == EPI / 32) {
    if (lane == 0) {
      auto psub = [&](int j, int& row0, int& kv) { row0 = r0 + j * TC_TILE; kv = kvh; };
      produce_tiles<P1_STAGES>(sh, ring, &tm_k, n_sub, b, psub, a.status);
    }
  } else if (warp == EPI / 32 + 1) {
    if (lane == 0) {
      auto sub = [&](int j, int& row0, int& slot) { row0 = r0 + j * TC_TILE; slot = 0; };
      issue_mmas<T, P1_STAGES>(sh, ring, q_s, N, n_sub, sub, a.status);
    }
  } else {
    const int quarter = warp & 3, half = warp >> 2;   // key = quarter * 32 + lane of the tile, columns [half * NC, +NC)
    const int key = quarter * 32 + lane, col0 = half * NC;
    const float k2 = a.scale * kLog2e;
    float l[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) l[c] = 0.f;
    if (tid < N) off_s[tid] = 0.f;
    bar_sync_epi<EPI>();
    for (int j = 0; j < n_sub; ++j) {
      float x[NC];
      const bool ok = take_accumulator<NC>(sh, j, x, quarter, (j % kAccBufs) * N + col0, a.status);
      const bool valid = ok && r0 + j * TC_TILE + key < r1;
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        x[c] = valid ? fmaf(x[c], k2, -off_s[col0 + c]) : -INFINITY;
        tmax = fmaxf(tmax, x[c]);
      }
      // The shared offsets are set from the first tile and raised when some logit has outgrown them by more than
      // 2^16 (a sum of 2^16-sized terms cannot overflow fp32, and smaller terms lose nothing that matters).
      if (bar_or_epi<EPI>(!ok || j == 0 || tmax > 16.f)) {
        if (bar_or_epi<EPI>(!ok)) break;  // a wait ran out somewhere: all epilogue threads leave together
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float m = x[c];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (lane == 0) cmax_s[quarter][col0 + c] = m;
        }
        bar_sync_epi<EPI>();
        if (tid < N) {
          float m = fmaxf(fmaxf(cmax_s[0][tid], cmax_s[1][tid]), fmaxf(cmax_s[2][tid], cmax_s[3][tid]));
          // first tile: the column's maximum becomes the offset (whatever its sign); later: only ever raise it
          const float s = (j == 0) ? (m == -INFINITY ? 0.f : m) : fmaxf(m, 0.f);
          shift_s[tid] = s;
          off_s[tid] += s;
        }
        bar_sync_epi<EPI>();
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const float s = shift_s[col0 + c];
          if (j > 0) l[c] *= ex2_fast(-s);
          x[c] -= s;
        }
        bar_sync_epi<EPI>();  // shift_s is free again before anybody could rewrite it
      }
      if (valid) {
#pragma unroll
        for (int c = 0; c < NC; ++c) l[c] += ex2_fast(x[c]);
      }
    }
    // add the 128 private sums of every column (through shared memory: the ring is idle by now)
    bar_sync_epi<EPI>();
    float* red = reinterpret_cast<float*>(ring);  // [128 keys][N + 1]
    if (!sh.fail) {
#pragma unroll
      for (int c = 0; c < NC; ++c) red[key * (N + 1) + col0 + c] = l[c];
    }
    bar_sync_epi<EPI>();
    if (tid < N && !sh.fail) {
      float tot = 0.f;
      for (int t = 0; t < 128; ++t) tot += red[t * (N + 1) + tid];
      part[(size_t)tid * a.S * 2 + 0] = off_s[tid];
      part[(size_t)tid * a.S * 2 + 1] = tot;
    }
  }
  tc_teardown<P1_STAGES>(sh, tmem_cols(N), warp, EPI);
}

// ---- pass 2 ------------------------------------------------------------------------------------------------------
// One launch per GROUP of KV heads whose query blocks fit in shared memory beside a four-tile K ring (64 KB of
// queries: four KV heads of a group of four query heads).  A launch walks its KV heads for every key tile and keeps
// the running max over heads per window slot in registers; between launches the 16 per-slot maxima of every key
// (log domain, 64 bytes per key against the 2 KB of K that a KV-head group streams for it) go through a plane in the
// workspace.  The last launch turns them into the score.  With a two-tile ring -- all that fits beside eight
// resident query blocks -- the stream ran at half the rate: the ring depth is the memory parallelism of an SM.
constexpr int P2_STAGES = 4;

template <typename T, int G>
__global__ void __launch_bounds__(TC_THREADS, 1) window_tc_pass2(const WinTcArgs a, const __grid_constant__ CUtensorMap tm_k,
                                                                 const int kvh0, const int n_kvh, const int first, const int last) {
  constexpr int N = G * TC_WPAD;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TcShared sh;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;
  unsigned char* q_s = smem + P2_STAGES * TC_KTILE_BYTES;                 // [n_kvh][N rows x 256 bytes]
  float* c2_s = reinterpret_cast<float*>(q_s + (size_t)n_kvh * N * 256);  // [n_kvh * N]
  // The CTAs of the (flat) grid are dealt to the sequences in proportion to their key tiles, every sequence at least
  // one: b = this CTA's sequence, `loc` its number among the sequence's `cnt` CTAs (tiles loc, loc + cnt, ...).
  int b = 0, loc = (int)blockIdx.x, cnt = (int)gridDim.x;
  if (a.B > 1) {
    long long total = 0;
    for (int bb = 0; bb < a.B; ++bb) total += ceil_div(a.consider_len[bb], TC_TILE);
    const int spare = (int)gridDim.x - a.B;
    int used = 0;
    for (int bb = 0; bb < a.B; ++bb)
      used += total > 0 ? (int)((long long)spare * ceil_div(a.consider_len[bb], TC_TILE) / total) : 0;
    const int left = spare - used;  // < B: one more each for the first sequences
    int start = 0;
    for (int bb = 0; bb < a.B; ++bb) {
      const int c = 1 + (total > 0 ? (int)((long long)spare * ceil_div(a.consider_len[bb], TC_TILE) / total) : 0) +
                    (bb < left ? 1 : 0);
      if ((int)blockIdx.x < start + c) {
        b = bb;
        loc = (int)blockIdx.x - start;
        cnt = c;
        break;
      }
      start += c;
    }
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = a.consider_len[b];
  const int n_tiles = ceil_div(n, TC_TILE);
  const int my_tiles = loc < n_tiles ? ceil_div(n_tiles - loc, cnt) : 0;
  // Launched as a programmatic dependent of pass 1 (or of the previous pass-2 launch): a CTA takes its SM as soon as
  // that launch's CTAs leave it, stages its query blocks, fills its K ring and runs its first MMAs.  Only the epilogue
  // warps read what the previous launch wrote (the partial normalisers, the plane of running maxima), and they wait
  // for it first.  The window queries and K are older than pass 1, which triggers only after its own wait.
  pdl_trigger();
  if (my_tiles == 0) {
    pdl_wait();  // a launch is complete only after its predecessor: later kernels rely on that order
    return;
  }
  const int n_sub = my_tiles * n_kvh;
  const T* qb = static_cast<const T*>(a.qw) + (size_t)b * a.H * a.W * kHeadDim;
  for (int kv = 0; kv < n_kvh; ++kv)
    stage_q_block<T>(q_s + (size_t)kv * N * 256, qb, (kvh0 + kv) * G, G, a.W, tid, TC_THREADS);
  tc_setup_begin<P2_STAGES>(sh, tmem_cols(N), warp, 128);
  tc_setup_end();
  auto sub = [&](int j, int& row0, int& kv) {
    row0 = (loc + (j / n_kvh) * cnt) * TC_TILE;
    kv = j % n_kvh;
  };
  if (warp == 4) {
    if (lane == 0) {
      auto psub = [&](int j, int& row0, int& kv) { sub(j, row0, kv); kv += kvh0; };
      produce_tiles<P2_STAGES>(sh, ring, &tm_k, n_sub, b, psub, a.status);
    }
  } else if (warp == 5) {
    if (lane == 0) issue_mmas<T, P2_STAGES>(sh, ring, q_s, N, n_sub, sub, a.status);
  } else {
    // log2 of the softmax normaliser of this launch's (head, slot) rows, from the splits of pass 1 (what a separate
    // merge kernel would do; here it runs while the first K tiles are on their way)
    pdl_wait();
    for (int i = tid; i < n_kvh * N; i += 128) {
      const float2* pr = reinterpret_cast<const float2*>(a.part) + (((size_t)b * a.H + kvh0 * G) * TC_WPAD + i) * a.S;
      float M = -INFINITY, L = 0.f;
      for (int s0 = 0; s0 < a.S; s0 += 16) {  // sixteen (offset, sum) pairs per round trip
        float2 ml[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) ml[u] = s0 + u < a.S ? pr[s0 + u] : make_float2(-INFINITY, 0.f);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          if (ml[u].y > 0.f) {
            const float Mn = fmaxf(M, ml[u].x);
            L = L * exp2f(M - Mn) + ml[u].y * exp2f(ml[u].x - Mn);
            M = Mn;
          }
        }
      }
      c2_s[i] = L > 0.f ? M + log2f(L) : INFINITY;  // an empty row normalises everything to 0
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    const float k2 = a.scale * kLog2e;
    float wgt[TC_WPAD];
#pragma unroll
    for (int w = 0; w < TC_WPAD; ++w) {
      float v = 0.f;
      if (w < a.W) v = a.selector == OMNIKV_SEL_UNIFORM ? 1.f : (a.selector == OMNIKV_SEL_EXP ? exp2f((float)(w - (a.W - 1))) : (w == a.W - 1 ? 1.f : 0.f));
      wgt[w] = v;
    }
    float t[TC_WPAD];
    float* tplane = a.tplane + (size_t)b * TC_WPAD * a.tplane_stride;  // [16][tplane_stride] per sequence
    for (int j = 0; j < n_sub; ++j) {
      float x[N];
      if (!take_accumulator<N>(sh, j, x, warp, (j % kAccBufs) * N, a.status)) break;
      const int kv = j % n_kvh;
      const int p = (loc + (j / n_kvh) * cnt) * TC_TILE + tid;
      if (kv == 0) {
#pragma unroll
        for (int w = 0; w < TC_WPAD; ++w) t[w] = (first || p >= n) ? -INFINITY : tplane[(size_t)w * a.tplane_stride + p];
      }
      const float* c2 = c2_s + kv * N;
#pragma unroll
      for (int c = 0; c < N; ++c) t[c % TC_WPAD] = fmaxf(t[c % TC_WPAD], fmaf(x[c], k2, -c2[c]));
      if (kv == n_kvh - 1 && p < n) {
        if (!last) {
#pragma unroll
          for (int w = 0; w < TC_WPAD; ++w) tplane[(size_t)w * a.tplane_stride + p] = t[w];
        } else {
          if (a.planes_out) {
#pragma unroll
            for (int w = 0; w < TC_WPAD; ++w)
              if (w < a.W) a.planes_out[((size_t)b * a.W + w) * a.score_stride + p] = ex2_fast(t[w]);
          }
          if (a.score_out) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < TC_WPAD; ++w) s = fmaf(wgt[w], ex2_fast(t[w]), s);
            a.score_out[(size_t)b * a.score_stride + p] = s;
          }
        }
      }
    }
  }
  tc_teardown<P2_STAGES>(sh, tmem_cols(N), warp, 128);
}

constexpr int kP2QueryBytes = 64 * 1024;  // query blocks resident per pass-2 launch (four KV heads of four query heads)

template <typename T, int G>
int launch_tc(const WinTcArgs& a, const CUtensorMap& tm_k, int max_len, cudaStream_t st) {
  constexpr int N = G * TC_WPAD;
  const int group = kP2QueryBytes / (N * 256) < a.KVH ? kP2QueryBytes / (N * 256) : a.KVH;  // KV heads per pass-2 launch
  const int smem1 = P1_STAGES * TC_KTILE_BYTES + N * 256 + 1024;
  const int smem2 = P2_STAGES * TC_KTILE_BYTES + group * N * 256 + group * N * (int)sizeof(float) + 1024;
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_tc_pass1<T, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_tc_pass2<T, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
  OMNIKV_CUDA_OK(launch_pdl_smem_args(window_tc_pass1<T, G>, dim3(a.S, a.KVH, a.B), dim3(P1Shape<G>::THREADS), smem1, st, a, tm_k));
  const int max_tiles = ceil_div(max_len, TC_TILE);
  // one CTA per SM (the query blocks and the ring fill its shared memory), never fewer than one per sequence
  int n_ctas = a.n_sms < a.B * max_tiles ? a.n_sms : a.B * max_tiles;
  if (n_ctas < a.B) n_ctas = a.B;
  for (int kvh0 = 0; kvh0 < a.KVH; kvh0 += group) {
    const int n_kvh = a.KVH - kvh0 < group ? a.KVH - kvh0 : group;
    OMNIKV_CUDA_OK(launch_pdl_smem_args(window_tc_pass2<T, G>, dim3(n_ctas), dim3(TC_THREADS), smem2, st, a, tm_k, kvh0, n_kvh,
                                        kvh0 == 0 ? 1 : 0, kvh0 + n_kvh >= a.KVH ? 1 : 0));
  }
  return OMNIKV_OK;
}

}  // namespace

bool window_tc_supported(int G, int KVH) {
  (void)KVH;
  return G == 1 || G == 2 || G == 4;  // 16 G accumulator columns and as many running sums per key
}

int window_tc_splits(int B, int KVH, int n_sms, int max_len) {
  int s = 2 * (n_sms / (B * KVH > 0 ? B * KVH : 1));  // one wave of two CTAs per SM
  // a batch has more (sequence, KV head) pairs than that: chunks of about 4096 keys, dealt out as CTAs retire, even
  // out sequences of different lengths
  if (B > 1 && s < ceil_div(max_len, 4096)) s = ceil_div(max_len, 4096);
  return s < 1 ? 1 : (s > kWindowTcMaxSplits ? kWindowTcMaxSplits : s);
}

int window_tc_launches(int G, int KVH) {
  const int N = G * TC_WPAD;
  const int group = kP2QueryBytes / (N * 256) < KVH ? kP2QueryBytes / (N * 256) : KVH;
  return 1 + ceil_div(KVH, group);
}

int window_tc_launch(int dtype, const WinTcArgs& a, const CUtensorMap& tm_k, int max_len, cudaStream_t st) {
#define OMNIKV_TC_GO(T)                                            \
  switch (a.G) {                                                   \
    case 1: return launch_tc<T, 1>(a, tm_k, max_len, st);          \
    case 2: return launch_tc<T, 2>(a, tm_k, max_len, st);          \
    case 4: return launch_tc<T, 4>(a, tm_k, max_len, st);          \
    default: return OMNIKV_E_UNSUPPORTED;                          \
  }
  if (dtype == OMNIKV_BF16) { OMNIKV_TC_GO(__nv_bfloat16) }
  if (dtype == OMNIKV_F16) { OMNIKV_TC_GO(__half) }
#undef OMNIKV_TC_GO
  return OMNIKV_E_UNSUPPORTED;
}

}  // namespace omnikv
