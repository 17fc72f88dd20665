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

namespace omnikv {
namespace {

constexpr int TC_TILE = 128;                 // keys per MMA group = TMEM lanes
constexpr int TC_KTILE_BYTES = TC_TILE * 256;  // a staged K tile: two boxes of 128 rows x 128 bytes
constexpr int TC_BOX_BYTES = TC_TILE * 128;
constexpr int TC_THREADS = 192;              // warps 0-3: epilogue (TMEM lane quarters), 4: TMA producer, 5: MMA issuer
constexpr int TC_WPAD = 16;

// ---- tcgen05 wrappers (cta_group::1) ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(unsigned* smem_dst, unsigned ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// D[tmem] (+)= A[smem desc] * B[smem desc]; both operands K-major, fp32 accumulate
__device__ __forceinline__ void tc_mma(unsigned d_tmem, uint64_t a_desc, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand stored as rows of 128 bytes with the 128-byte swizzle
// (what a TMA box of 64 16-bit elements x rows leaves, and what the query block is written as): 8-row groups
// are 1024 bytes apart (stride byte offset), version 1 (Blackwell), layout type 2 = SWIZZLE_128B.  `addr` is
// the byte address of the first element of this K step inside its 1024-byte-aligned box.
__device__ __forceinline__ uint64_t smem_desc_sw128(unsigned addr) {
  uint64_t d = (uint64_t)((addr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused with a swizzled K-major operand)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}
// Instruction descriptor: fp32 accumulator, A and B of the given 16-bit format, both K-major, M = 128, N columns.
template <typename T>
__device__ __forceinline__ unsigned instr_desc(int N) {
  constexpr unsigned fmt = std::is_same<T, __half>::value ? 0u : 1u;  // F16 = 0, BF16 = 1
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(TC_TILE >> 4) << 24);
}

__device__ __forceinline__ unsigned bar_or_128(bool pred) {  // OR over the 128 epilogue threads (named barrier 1)
  unsigned r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.b32 p, %1, 0;\n"
      "barrier.cta.red.or.pred q, 1, 128, p;\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(r)
      : "r"((unsigned)pred)
      : "memory");
  return r;
}
__device__ __forceinline__ void bar_epi() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

// Query block of KV head `kvh` -> shared memory as the B operand: N = 16 G rows (head-major, window padded to 16
// slots, rows >= W zero) x 128, two boxes of [N rows x 128 bytes], 16-byte chunk c of row r at chunk c ^ (r & 7).
template <typename T>
__device__ __forceinline__ void stage_q_block(unsigned char* dst, const T* qw_b, int h0, int G, int W, int tid, int nthreads) {
  const int N = G * TC_WPAD;
  for (int i = tid; i < N * 16; i += nthreads) {
    const int r = i >> 4, c = i & 15;  // row, 16-byte chunk of the 256-byte row
    const int hl = r / TC_WPAD, w = r % TC_WPAD;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (w < W) v = *reinterpret_cast<const uint4*>(qw_b + ((size_t)(h0 + hl) * W + w) * kHeadDim + c * 8);
    unsigned char* box = dst + (c >> 3) * (N * 128);
    *reinterpret_cast<uint4*>(box + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
  }
}

struct TcShared {
  uint64_t full[4];
  uint64_t empty[4];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
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
    const int s = j % STAGES, buf = j & 1;
    if (!mbar_wait(&sh.full[s], (j / STAGES) & 1, &sh.fail) ||
        !mbar_wait(&sh.acc_empty[buf], ((j >> 1) & 1) ^ 1, &sh.fail)) {
      if (!sh.fail && status) atomicExch(status, 5);
      sh.fail = 1;
      return;
    }
    tc_fence_after();
    int row0, kvh_slot;
    sub(j, row0, kvh_slot);  // kvh_slot: which resident query block this sub-tile meets
    const unsigned a_base = smem_u32(ring + (size_t)s * TC_KTILE_BYTES);
    const unsigned b_base = smem_u32(q_s + (size_t)kvh_slot * N * 256);
    const unsigned d_tmem = sh.tmem_base + (unsigned)(buf * N);
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

// Epilogue side: wait for accumulator `j`, read this thread's N logits into v (N <= 128), hand the buffer back.
template <int N>
__device__ __forceinline__ bool take_accumulator(TcShared& sh, int j, float (&v)[N], int warp, int* status) {
  const int buf = j & 1;
  if (!mbar_wait(&sh.acc_full[buf], (j >> 1) & 1, &sh.fail)) {
    if (!sh.fail && status) atomicExch(status, 5);
    sh.fail = 1;
    return false;
  }
  tc_fence_after();
  const unsigned taddr = sh.tmem_base + ((unsigned)(warp * 32) << 16) + (unsigned)(buf * N);
#pragma unroll
  for (int c = 0; c < N; c += 16) tmem_ld16(taddr + c, *reinterpret_cast<float(*)[16]>(&v[c]));
  tmem_ld_wait();
  tc_fence_before();
  mbar_arrive(&sh.acc_empty[buf]);
  return true;
}

template <int STAGES>
__device__ __forceinline__ void tc_setup(TcShared& sh, unsigned ncols, int warp) {
  if (threadIdx.x == 0) {
    sh.fail = 0;
    sh.issued = 0;
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.acc_full[i], 1);
      mbar_init(&sh.acc_empty[i], 128);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {  // one warp allocates the tensor memory and gives the permit back
    tmem_alloc(&sh.tmem_base, ncols);
    tmem_relinquish();
  }
  // the query block was written with ordinary stores; the tensor core reads it through the async proxy
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

template <int STAGES>
__device__ __forceinline__ void tc_teardown(TcShared& sh, unsigned ncols, int warp) {
  tc_fence_before();
  __syncthreads();  // every role is out of its loop: no MMA, copy or TMEM read of this CTA is still wanted
  if (sh.fail) {
    // a wait ran out: copies that were asked for may still be on their way into this CTA's shared memory.  Wait
    // (bounded) for each stage's last requested tile before the memory is given up.
    if (threadIdx.x == 128) {
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

__host__ __device__ constexpr unsigned tmem_cols(int N) { return 2 * N <= 32 ? 32u : (2 * N <= 64 ? 64u : (2 * N <= 128 ? 128u : 256u)); }

// ---- pass 1 ------------------------------------------------------------------------------------------------------
constexpr int P1_STAGES = 4;

template <typename T, int G>
__global__ void __launch_bounds__(TC_THREADS, 1) window_tc_pass1(const WinTcArgs a, const __grid_constant__ CUtensorMap tm_k) {
  constexpr int N = G * TC_WPAD;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TcShared sh;
  __shared__ float off_s[N];    // per-column offset b (log2 domain) shared by the CTA
  __shared__ float shift_s[N];
  __shared__ float cmax_s[4][N];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;
  unsigned char* q_s = smem + P1_STAGES * TC_KTILE_BYTES;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = a.consider_len[b];
  const int chunk = ceil_div(ceil_div(n, a.S), TC_TILE) * TC_TILE;
  const int r0 = min(n, split * chunk), r1 = min(n, r0 + chunk);
  const int n_sub = r1 > r0 ? ceil_div(r1 - r0, TC_TILE) : 0;
  float* part = a.part + ((((size_t)b * a.H + kvh * G) * TC_WPAD) * a.S + split) * 2;  // + (hl*16 + w) * S * 2
  if (n_sub == 0) {
    for (int c = tid; c < N; c += TC_THREADS) {
      part[(size_t)c * a.S * 2 + 0] = -INFINITY;
      part[(size_t)c * a.S * 2 + 1] = 0.f;
    }
    return;
  }
  stage_q_block<T>(q_s, static_cast<const T*>(a.qw) + (size_t)b * a.H * a.W * kHeadDim, kvh * G, G, a.W, tid, TC_THREADS);
  tc_setup<P1_STAGES>(sh, tmem_cols(N), warp);
  auto sub = [&](int j, int& row0, int& slot) { row0 = r0 + j * TC_TILE; slot = 0; };
  if (warp == 4) {
    if (lane == 0) {
      auto psub = [&](int j, int& row0, int& kv) { row0 = r0 + j * TC_TILE; kv = kvh; };
      produce_tiles<P1_STAGES>(sh, ring, &tm_k, n_sub, b, psub, a.status);
    }
  } else if (warp == 5) {
    if (lane == 0) issue_mmas<T, P1_STAGES>(sh, ring, q_s, N, n_sub, sub, a.status);
  } else {
    const float k2 = a.scale * kLog2e;
    float l[N];
#pragma unroll
    for (int c = 0; c < N; ++c) l[c] = 0.f;
    if (tid < N) off_s[tid] = 0.f;
    bar_epi();
    for (int j = 0; j < n_sub; ++j) {
      float x[N];
      const bool ok = take_accumulator<N>(sh, j, x, warp, a.status);
      const bool valid = ok && r0 + j * TC_TILE + tid < r1;
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < N; ++c) {
        x[c] = valid ? fmaf(x[c], k2, -off_s[c]) : -INFINITY;
        tmax = fmaxf(tmax, x[c]);
      }
      // The shared offsets are set from the first tile and raised when some logit has outgrown them by more than
      // 2^16 (a sum of 2^16-sized terms cannot overflow fp32, and smaller terms lose nothing that matters).
      if (bar_or_128(!ok || j == 0 || tmax > 16.f)) {
        if (bar_or_128(!ok)) break;  // a wait ran out somewhere: all 128 threads leave together
#pragma unroll
        for (int c = 0; c < N; ++c) {
          float m = x[c];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (lane == 0) cmax_s[warp][c] = m;
        }
        bar_epi();
        if (tid < N) {
          float m = fmaxf(fmaxf(cmax_s[0][tid], cmax_s[1][tid]), fmaxf(cmax_s[2][tid], cmax_s[3][tid]));
          // first tile: the column's maximum becomes the offset (whatever its sign); later: only ever raise it
          const float s = (j == 0) ? (m == -INFINITY ? 0.f : m) : fmaxf(m, 0.f);
          shift_s[tid] = s;
          off_s[tid] += s;
        }
        bar_epi();
#pragma unroll
        for (int c = 0; c < N; ++c) {
          const float s = shift_s[c];
          if (j > 0) l[c] *= exp2f(-s);
          x[c] -= s;
        }
        bar_epi();  // shift_s is free again before anybody could rewrite it
      }
      if (valid) {
#pragma unroll
        for (int c = 0; c < N; ++c) l[c] += exp2f(x[c]);
      }
    }
    // add the 128 private sums of every column (through shared memory: the ring is idle by now)
    bar_epi();
    float* red = reinterpret_cast<float*>(ring);  // [128][N + 1]
    if (!sh.fail) {
#pragma unroll
      for (int c = 0; c < N; ++c) red[tid * (N + 1) + c] = l[c];
    }
    bar_epi();
    if (tid < N && !sh.fail) {
      float tot = 0.f;
      for (int t = 0; t < 128; ++t) tot += red[t * (N + 1) + tid];
      part[(size_t)tid * a.S * 2 + 0] = off_s[tid];
      part[(size_t)tid * a.S * 2 + 1] = tot;
    }
  }
  tc_teardown<P1_STAGES>(sh, tmem_cols(N), warp);
}

// splits -> c = m + log2(l) per (b, h, slot) row.  One thread per row; (m, l) pairs are in the log2 domain.
__global__ void window_tc_merge(const float* __restrict__ part, float* __restrict__ c2, int rows, int S) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float M = -INFINITY;
  for (int s = 0; s < S; ++s)
    if (part[((size_t)r * S + s) * 2 + 1] > 0.f) M = fmaxf(M, part[((size_t)r * S + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < S; ++s) {
    const float l = part[((size_t)r * S + s) * 2 + 1];
    if (l > 0.f) L += l * exp2f(part[((size_t)r * S + s) * 2] - M);
  }
  c2[r] = L > 0.f ? M + log2f(L) : INFINITY;  // an empty row (padded window slot) normalises everything to 0
}

// ---- pass 2 ------------------------------------------------------------------------------------------------------
constexpr int P2_STAGES = 2;

template <typename T, int G>
__global__ void __launch_bounds__(TC_THREADS, 1) window_tc_pass2(const WinTcArgs a, const __grid_constant__ CUtensorMap tm_k) {
  constexpr int N = G * TC_WPAD;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TcShared sh;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;
  unsigned char* q_s = smem + P2_STAGES * TC_KTILE_BYTES;                   // [KVH][N rows x 256 bytes]
  float* c2_s = reinterpret_cast<float*>(q_s + (size_t)a.KVH * N * 256);  // [KVH * N]
  const int b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = a.consider_len[b];
  const int n_tiles = ceil_div(n, TC_TILE);
  const int my_tiles = (int)blockIdx.x < n_tiles ? ceil_div(n_tiles - (int)blockIdx.x, (int)gridDim.x) : 0;
  if (my_tiles == 0) return;
  const int n_sub = my_tiles * a.KVH;
  const T* qb = static_cast<const T*>(a.qw) + (size_t)b * a.H * a.W * kHeadDim;
  for (int kv = 0; kv < a.KVH; ++kv) stage_q_block<T>(q_s + (size_t)kv * N * 256, qb, kv * G, G, a.W, tid, TC_THREADS);
  for (int i = tid; i < a.KVH * N; i += TC_THREADS) c2_s[i] = a.c2[(size_t)b * a.H * TC_WPAD + i];
  tc_setup<P2_STAGES>(sh, tmem_cols(N), warp);
  const int KVH = a.KVH;
  auto sub = [&](int j, int& row0, int& kv) {
    row0 = ((int)blockIdx.x + (j / KVH) * (int)gridDim.x) * TC_TILE;
    kv = j % KVH;
  };
  if (warp == 4) {
    if (lane == 0) produce_tiles<P2_STAGES>(sh, ring, &tm_k, n_sub, b, sub, a.status);
  } else if (warp == 5) {
    if (lane == 0) issue_mmas<T, P2_STAGES>(sh, ring, q_s, N, n_sub, sub, a.status);
  } else {
    const float k2 = a.scale * kLog2e;
    float wgt[TC_WPAD];
#pragma unroll
    for (int w = 0; w < TC_WPAD; ++w) {
      float v = 0.f;
      if (w < a.W) v = a.selector == OMNIKV_SEL_UNIFORM ? 1.f : (a.selector == OMNIKV_SEL_EXP ? exp2f((float)(w - (a.W - 1))) : (w == a.W - 1 ? 1.f : 0.f));
      wgt[w] = v;
    }
    float t[TC_WPAD];
    for (int j = 0; j < n_sub; ++j) {
      float x[N];
      if (!take_accumulator<N>(sh, j, x, warp, a.status)) break;
      const int kv = j % KVH;
      if (kv == 0) {
#pragma unroll
        for (int w = 0; w < TC_WPAD; ++w) t[w] = -INFINITY;
      }
      const float* c2 = c2_s + kv * N;
#pragma unroll
      for (int c = 0; c < N; ++c) t[c % TC_WPAD] = fmaxf(t[c % TC_WPAD], fmaf(x[c], k2, -c2[c]));
      if (kv == KVH - 1) {
        const int p = ((int)blockIdx.x + (j / KVH) * (int)gridDim.x) * TC_TILE + tid;
        if (p < n) {
          if (a.planes_out) {
#pragma unroll
            for (int w = 0; w < TC_WPAD; ++w)
              if (w < a.W) a.planes_out[((size_t)b * a.W + w) * a.score_stride + p] = exp2f(t[w]);
          }
          if (a.score_out) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < TC_WPAD; ++w) s = fmaf(wgt[w], exp2f(t[w]), s);
            a.score_out[(size_t)b * a.score_stride + p] = s;
          }
        }
      }
    }
  }
  tc_teardown<P2_STAGES>(sh, tmem_cols(N), warp);
}

template <typename T, int G>
int launch_tc(const WinTcArgs& a, const CUtensorMap& tm_k, int max_len, cudaStream_t st) {
  constexpr int N = G * TC_WPAD;
  const int smem1 = P1_STAGES * TC_KTILE_BYTES + N * 256 + 1024;
  const int smem2 = P2_STAGES * TC_KTILE_BYTES + a.KVH * N * 256 + a.KVH * N * (int)sizeof(float) + 1024;
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_tc_pass1<T, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(window_tc_pass2<T, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
  window_tc_pass1<T, G><<<dim3(a.S, a.KVH, a.B), TC_THREADS, smem1, st>>>(a, tm_k);
  OMNIKV_CUDA_OK(cudaGetLastError());
  const int rows = a.B * a.H * TC_WPAD;
  window_tc_merge<<<ceil_div(rows, 128), 128, 0, st>>>(a.part, a.c2, rows, a.S);
  OMNIKV_CUDA_OK(cudaGetLastError());
  const int max_tiles = ceil_div(max_len, TC_TILE);
  int per_seq = ceil_div(a.n_sms, a.B);
  if (per_seq > max_tiles) per_seq = max_tiles;
  window_tc_pass2<T, G><<<dim3(per_seq, a.B), TC_THREADS, smem2, st>>>(a, tm_k);
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

}  // namespace

bool window_tc_supported(int G, int KVH) {
  if (G != 1 && G != 2 && G != 4) return false;  // 16 G accumulator columns and as many running sums per thread
  const int N = G * TC_WPAD;
  // pass 2 keeps every KV head's query block resident beside a two-tile ring
  return P2_STAGES * TC_KTILE_BYTES + KVH * N * 256 + KVH * N * 4 + 1024 <= 200 * 1024;
}

int window_tc_splits(int B, int KVH, int n_sms) {
  int s = n_sms / (B * KVH > 0 ? B * KVH : 1);  // one wave of one CTA per SM (a thread holds 128 fp32 values)
  return s < 1 ? 1 : (s > kWindowTcMaxSplits ? kWindowTcMaxSplits : s);
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
