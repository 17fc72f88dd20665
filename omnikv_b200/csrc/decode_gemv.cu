// Weight-streaming kernels of a batch-1 decode step: y = W x with the surrounding element-wise work
// fused in, so that a decoder layer is five launches instead of about twenty:
//
//   QKV   : RMSNorm(h) -> fused q/k/v projection -> RoPE -> q to a buffer, k and v rows straight into
//           the KV cache at the current position (replaces norm, 3 GEMVs, rotate, cat, append);
//   RESID : h += W x                       (output projection, MLP down projection);
//   GATEUP: RMSNorm(h) -> silu(Wg x) * (Wu x);
//   LOGITS: RMSNorm(h) -> fp32 logits and their arg-max (greedy token).
//
// All of them are HBM-bound streams over a bf16/fp16 row-major weight matrix.  A CTA walks chunks of
// weight rows; each chunk is two contiguous pieces of rows that a single elected thread copies into a
// shared-memory ring with TMA bulk copies (cp.async.bulk + mbarrier transaction counts), up to
// (STAGES-1) x 64 KB in flight per SM.  Eight consumer warps read the staged rows with conflict-free
// 16-byte shared loads; every warp keeps its slice of x in registers as fp32, so the inner loop is one
// shared load, eight conversions and eight FMAs per 16 bytes of weights, fp32 accumulation.
// One CTA per SM, persistent over its chunks.  Every mbarrier wait is bounded: if it runs out the CTA
// records an error code in a status word and leaves.
#include "common.cuh"

namespace omnikv {
namespace {

constexpr int GV_CONSUMER_WARPS = 8;
constexpr int GV_THREADS = (GV_CONSUMER_WARPS + 1) * 32;  // + one producer warp
constexpr int kTpMaxHidden = 8192;  // largest residual stream whose tensor-parallel partial sums a kernel consumes
constexpr int GV_STAGES = 3;
#ifndef GV_PACED_FILL
#define GV_PACED_FILL 1
#endif
constexpr unsigned GV_SPIN_LIMIT = kSpinLimit;

enum Epilogue { EPI_QKV = 0, EPI_RESID = 1, EPI_GATEUP = 2, EPI_LOGITS = 3 };

struct GemvArgs {
  const void* W;        // [N, K] row-major
  const void* x;        // [K] activations (bf16/fp16)
  const void* norm_w;   // [K] RMSNorm weight or nullptr (no normalisation)
  float eps;
  int N, K;
  int n_chunks;         // chunks of RPS rows
  int partner_rows;     // distance in rows between the two pieces of a chunk (EPI_QKV: 64, EPI_GATEUP: N/2)
  // EPI_RESID
  const void* resid;    // [N] or nullptr
  void* out;            // [N] (EPI_RESID, EPI_GATEUP: [N/2])
  // EPI_QKV
  void* q_out;          // [H*128]
  void* k_cache;        // row base of this sequence: element (kvh, pos, :) at kvh*kv_sh + pos*kv_sr
  void* v_cache;
  int64_t kv_sh, kv_sr;
  const int* pos;       // device: cache row to write
  const int* rope_pos;  // device: position id for the rotation
  const float* inv_freq;  // [64]
  int H, KVH;
  // EPI_LOGITS
  float* logits;                    // [N]
  unsigned long long* best;         // packed (key << 32 | ~index), reduced with atomicMax
  int row_offset;                   // global index of row 0 (vocabulary shards)
  int* status;                      // device status word (0 = ok)
  int* next_chunk;                  // device counter (zero at launch) for dynamic chunk scheduling, or nullptr:
                                    // static round-robin over the CTAs
  // ---- tensor parallelism: the SUM all-reduce of a row-parallel projection, fused over peer memory ----
  // producer side (EPI_RESID): this rank's partial outputs are stored straight into every rank's exchange
  // buffer; when the whole grid is done, a flag word is stored on every rank
  int tp_world;                     // 0/1: off
  uint2* tp_peer_ll[8];             // rank p's slot for MY partials: [N] x {fp32 bits, tag}
  // consumer side (phases with a norm): x = resid + sum over ranks of their partials, once every entry carries
  // this exchange's tag
  const uint2* tp_my_ll;            // local [8][K] x {fp32 bits, tag} of the slot to consume, or nullptr
  void* tp_h_out;                   // local [K]: CTA 0 stores the summed residual stream here
  const unsigned* tp_epoch;         // device word bumped once per decode step
  unsigned tp_seq;                  // tag = epoch * 256 + seq + 1
  int trace_slot;                   // profiling build: which slot of the stamp array this launch writes
  int tail_pool;                    // chunks at the end of the matrix handed out dynamically (0: all static)
  int* tail_next;                   // [2] device: next index of the pool, finished producers (self-resetting)
};

#ifdef OMNIKV_TRACE
// Profiling build only: per-CTA %globaltimer stamps of the single-phase kernel, one slot per launch.
// [0] CTA start, [1] previous kernel complete (dependent-launch wait passed), [6] staging area free, [7] activations
// staged (after the wait for the peers' flags, when there is an exchange), [2] activations in registers, [3] first
// chunk landed, [8] rows done, [4] consumers done (after the exchange tail: fence, count, flags), [5] last copy
// issued (producer thread), [9] flags raised (the CTA that finished last), [10] epilogue kind.
constexpr int kGemvTraceCtas = 160, kGemvTraceWords = 12;
__device__ unsigned long long g_gemv_trace[kTraceSlots * kGemvTraceCtas * kGemvTraceWords];
#define GEMV_STAMP(a, i)                                                                                       \
  do {                                                                                                         \
    unsigned long long t_;                                                                                     \
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t_));                                                    \
    if (blockIdx.x < kGemvTraceCtas)                                                                           \
      g_gemv_trace[((a).trace_slot * kGemvTraceCtas + blockIdx.x) * kGemvTraceWords + (i)] = t_;               \
  } while (0)
#else
#define GEMV_STAMP(a, i)
#endif

// Ask the memory system to bring [src, src + bytes) into L2; nothing waits for it.
__device__ __forceinline__ void l2_prefetch(const void* gmem_src, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(gmem_src), "r"(bytes) : "memory");
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(u[i] << 16);
    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& v, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// Shared-memory ring shared by the producer thread and the consumer warps of a CTA.
struct Ring {
  unsigned char* smem;      // GV_STAGES slots of slot_bytes
  uint64_t* full_bar;
  uint64_t* empty_bar;
  unsigned slot_bytes;
  int* slot_chunk;          // chunk held by each slot, -1 = the phase has no more chunks for this CTA
  unsigned char* stage_x;   // staging area for the phase's activations (and norm weights), 16-byte aligned
  unsigned stage_bytes;     // its size
  const volatile int* abort;  // ConsumerShared::fail
};

// First row of the two pieces of chunk c.
template <int HALF, int EPI>
__device__ __forceinline__ void piece_rows(const GemvArgs& a, int c, int& row0, int& row1) {
  if (EPI == EPI_QKV) {
    constexpr int per_head = 64 / HALF;
    const int head = c / per_head, j = c % per_head;
    row0 = head * 128 + j * HALF;
    row1 = row0 + 64;
  } else if (EPI == EPI_GATEUP) {
    row0 = c * HALF;
    row1 = row0 + a.partner_rows;
  } else {
    row0 = c * 2 * HALF;
    row1 = row0 + HALF;
  }
}

// KV: 16-byte vectors per lane per K-slice; WK: warps along K.  K = WK * KV * 256.
// RPS = 8 / WK rows per stage, in two pieces of RPS/2 rows.
// Producer side of one phase: called by ONE thread.  `it` is the CTA's running chunk number (ring position).
template <typename T, int KV, int WK, int EPI>
__device__ __forceinline__ bool produce_phase(const GemvArgs& a, const Ring& ring, int& it) {
  const volatile int* abort = ring.abort;  // raised by the consumers when they give up: stop producing
  constexpr int HALF = GV_CONSUMER_WARPS / WK / 2;
  constexpr int K = WK * KV * 256;
  constexpr unsigned PIECE_BYTES = HALF * K * 2;
  const T* W = static_cast<const T*>(a.W);
  int i = 0;
  int grab = -2;  // index taken from the tail pool and not used yet (-2: none)
  for (;; ++it) {
    const int slot = it % GV_STAGES;
    if (it >= GV_STAGES && !mbar_wait(&ring.empty_bar[slot], ((it / GV_STAGES) - 1) & 1, abort)) {
      if (!*abort) atomicExch(a.status, 1);
      return false;
    }
    // The first fill of the ring is paced: a chunk is asked for when the one before it has landed.  One
    // chunk per SM in flight already saturates HBM; three per SM at once (28 MB) only build a queue that the
    // consumers' loads of the activations -- issued a little later, and on the critical path of the whole
    // kernel -- would have to wait behind (measured: 3.5 us instead of about 1).
    if (GV_PACED_FILL && it > 0 && it < GV_STAGES && !mbar_wait(&ring.full_bar[it - 1], 0, abort)) {
      if (!*abort) atomicExch(a.status, 1);
      return false;
    }
    // next chunk: from the shared counter (whoever is ready takes the next one, so slow SMs take fewer),
    // or this CTA's static share
    int c;
    if (a.next_chunk) {
      c = atomicAdd(a.next_chunk, 1);
    } else if (a.tail_pool > 0) {
      // static share first; the LAST tail_pool chunks of the matrix go to whoever gets there first, one at a
      // time, the next grab already requested while the current chunk is being fetched
      const int n_static = a.n_chunks - a.tail_pool;
      c = (int)blockIdx.x + i * (int)gridDim.x;
      if (c < n_static) {
        ++i;
        if (grab == -2 && (int)blockIdx.x + (i + 1) * (int)gridDim.x >= n_static) grab = atomicAdd(a.tail_next, 1);
      } else {
        if (grab == -2) grab = atomicAdd(a.tail_next, 1);
        c = n_static + grab;
        grab = -2;
        if (c < a.n_chunks) grab = atomicAdd(a.tail_next, 1);
      }
    } else {
      c = (int)blockIdx.x + i * (int)gridDim.x;
      ++i;
    }
    if (c >= a.n_chunks) {  // end marker: the slot carries no data
      ring.slot_chunk[slot] = -1;
      mbar_arrive(&ring.full_bar[slot]);
      ++it;
      if (a.tail_pool > 0 && atomicAdd(a.tail_next + 1, 1) == (int)gridDim.x - 1) {  // last producer: reset
        a.tail_next[0] = 0;
        a.tail_next[1] = 0;
      }
      return true;
    }
    ring.slot_chunk[slot] = c;
    int row0, row1;
    piece_rows<HALF, EPI>(a, c, row0, row1);
    unsigned char* dst = ring.smem + (size_t)slot * ring.slot_bytes;
    mbar_expect_tx(&ring.full_bar[slot], 2 * PIECE_BYTES);
    tma_bulk_g2s(dst, W + (size_t)row0 * K, PIECE_BYTES, &ring.full_bar[slot]);
    tma_bulk_g2s(dst + PIECE_BYTES, W + (size_t)row1 * K, PIECE_BYTES, &ring.full_bar[slot]);
  }
}

// The shared-memory ring covers about 4 us of HBM time; the pause between two phases (grid barrier + loading
// the new activations) is longer.  So when the producer has issued the last copy of a phase it asks for the
// first chunks of the NEXT phase to be brought into L2 (this CTA's round-robin share of them); the ring's
// copies then find them there and HBM keeps working through the pause.
constexpr int GV_L2_AHEAD = 4;  // chunks per CTA

template <typename T, int KV, int WK, int EPI>
__device__ __forceinline__ void prefetch_phase_head(const GemvArgs& a) {
  constexpr int HALF = GV_CONSUMER_WARPS / WK / 2;
  constexpr int K = WK * KV * 256;
  constexpr unsigned PIECE_BYTES = HALF * K * 2;
  const T* W = static_cast<const T*>(a.W);
  for (int j = 0; j < GV_L2_AHEAD; ++j) {
    const int c = (int)blockIdx.x + j * (int)gridDim.x;
    if (c >= a.n_chunks) break;
    int row0, row1;
    piece_rows<HALF, EPI>(a, c, row0, row1);
    l2_prefetch(W + (size_t)row0 * K, PIECE_BYTES);
    l2_prefetch(W + (size_t)row1 * K, PIECE_BYTES);
  }
}

// Scratch in static shared memory used by the consumers.
struct ConsumerShared {
  float inv_freq[64];  // EPI_QKV: the rotary frequencies, staged once
  float part[2][GV_CONSUMER_WARPS][4];
  float ssq[GV_CONSUMER_WARPS];
  unsigned long long best[GV_CONSUMER_WARPS];
  int fail;
};

__device__ __forceinline__ void consumer_bar() {
  asm volatile("bar.sync 1, %0;\n" ::"n"(GV_CONSUMER_WARPS * 32) : "memory");
}

// Consumer side of one phase: called by the 256 consumer threads.  COHERENT: x and resid were written by
// other CTAs of this same launch, so they are read through L2 (ld.global.cg), never from a stale L1 line.
template <typename T, int KV, int WK, int EPI, bool COHERENT>
__device__ __forceinline__ bool consume_phase(const GemvArgs& a, const Ring& ring, ConsumerShared& cs, int& it) {
  constexpr int RPS = GV_CONSUMER_WARPS / WK;
  constexpr int HALF = RPS / 2;
  constexpr int K = WK * KV * 256;
  constexpr unsigned ROW_BYTES = K * 2;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wk = warp % WK;   // K-slice
  const int wr = warp / WK;   // row within the stage

  // The activations (and the norm weights) are fetched ONCE per CTA into shared memory -- every SM reads the
  // same few KB right after a barrier, and eight warps each fetching all of it made those L2 lines a hot
  // spot -- then every warp takes its slice as fp32 registers, times the norm weight.
  uint4* xs = reinterpret_cast<uint4*>(ring.stage_x);
  uint4* ns = xs + K / 8;
  float sq = 0.f;
  consumer_bar();  // the previous phase no longer reads the staging area
  if (threadIdx.x == 0) GEMV_STAMP(a, 6);
  // Partial sums of other ranks are consumed by the stand-alone kernel only, and for at most 8192 activations
  // (four vectors per thread, whose sums stay in registers; the host checks the size).
  constexpr bool TP_OK = !COHERENT && K <= kTpMaxHidden;
  const bool tp_consume = TP_OK && a.tp_world > 1 && a.tp_my_ll != nullptr;
  constexpr int NT_ = GV_CONSUMER_WARPS * 32;
  constexpr int NV_ = TP_OK ? (K / 8 + NT_ - 1) / NT_ : 1;  // 16-byte vectors of activations per thread
  float psum[NV_][8];
  if constexpr (TP_OK) if (tp_consume) {
    // Every rank's partial sums of the previous projection arrive in this GPU's memory as 8-byte entries
    // {value, tag}, each written by ONE 8-byte store, so an entry is either the old one or the new one, never
    // a mix, and the tag says which: no flag, no fence and no completion of the producing kernel is waited for
    // -- a thread reads its entries until all of them carry this exchange's tag (a few microseconds after the
    // slowest rank has computed them).  The ranks' values are added in rank order (the same sums on every rank).
    // This kernel does NOT wait for its predecessor's completion either (see decode_gemv_kernel): everything it
    // needs from that kernel -- the local rank's partials -- comes through the tagged entries, and whatever else
    // it reads was written by kernels that had completed before the predecessor computed a single row.
    const unsigned want = __ldcg(a.tp_epoch) * 256u + a.tp_seq + 1u;
#pragma unroll
    for (int i = 0; i < NV_; ++i) {
#pragma unroll
      for (int e = 0; e < 8; ++e) psum[i][e] = 0.f;
      const int v = tid + i * NT_;
      if (v >= K / 8) continue;
      for (int r = 0; r < a.tp_world; ++r) {
        const uint4* src = reinterpret_cast<const uint4*>(a.tp_my_ll + (size_t)r * K + (size_t)v * 8);
        uint4 e0, e1, e2, e3;
        unsigned long long t0 = 0ull;
        for (unsigned spin = 0;; ++spin) {
          e0 = __ldcv(src); e1 = __ldcv(src + 1); e2 = __ldcv(src + 2); e3 = __ldcv(src + 3);
          const bool ok = e0.y == want && e0.w == want && e1.y == want && e1.w == want && e2.y == want &&
                          e2.w == want && e3.y == want && e3.w == want;
          if (ok) break;
          if ((spin & 63u) == 63u) {  // bounded by time: an absent rank costs kWaitNs, then the kernel reports and returns
            const unsigned long long now = globaltimer_ns();
            if (t0 == 0ull) t0 = now;
            if (now - t0 > kWaitNs || cs.fail) {
              cs.fail = 1;
              atomicExch(a.status, 4);
              break;
            }
          }
        }
        psum[i][0] += __uint_as_float(e0.x); psum[i][1] += __uint_as_float(e0.z);
        psum[i][2] += __uint_as_float(e1.x); psum[i][3] += __uint_as_float(e1.z);
        psum[i][4] += __uint_as_float(e2.x); psum[i][5] += __uint_as_float(e2.z);
        psum[i][6] += __uint_as_float(e3.x); psum[i][7] += __uint_as_float(e3.z);
      }
    }
    consumer_bar();
    if (cs.fail) return false;
  }
  {
    // Every global load of this prologue is issued BEFORE the first store to shared memory: written as one
    // loop (load, store, load, store ...) the compiler keeps the order, since it cannot rule out that the two
    // generic pointers alias, and each iteration then costs a full round trip (seven in a row for K = 14336).
    constexpr int NT = GV_CONSUMER_WARPS * 32;
    constexpr int NV = (K / 8 + NT - 1) / NT;  // 16-byte vectors per thread
    const uint4* xg = reinterpret_cast<const uint4*>(a.x);
    const uint4* ng = reinterpret_cast<const uint4*>(a.norm_w);
    uint4 xr_[NV], nr_[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = tid + i * NT;
      xr_[i] = make_uint4(0, 0, 0, 0);
      nr_[i] = xr_[i];
      if (v < K / 8) {
        xr_[i] = (COHERENT || tp_consume) ? __ldcg(xg + v) : xg[v];
        if (ng) nr_[i] = ng[v];
      }
    }
    if constexpr (TP_OK) if (tp_consume) {  // residual + the ranks' partials (fp32), rounded once to the storage type; still no store
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = tid + i * NT;
        if (v >= K / 8) continue;
        float f[8];
        unpack8<T>(xr_[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += psum[i][e];
        xr_[i].x = pack2<T>(f[0], f[1]);
        xr_[i].y = pack2<T>(f[2], f[3]);
        xr_[i].z = pack2<T>(f[4], f[5]);
        xr_[i].w = pack2<T>(f[6], f[7]);
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = tid + i * NT;
      if (v >= K / 8) continue;
      const uint4 raw = xr_[i];
      if (tp_consume && blockIdx.x == 0 && a.tp_h_out) reinterpret_cast<uint4*>(a.tp_h_out)[v] = raw;
      xs[v] = raw;
      if (ng) {
        ns[v] = nr_[i];
        float f[8];
        unpack8<T>(raw, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) sq = fmaf(f[e], f[e], sq);
      }
    }
  }
  // Whatever else the epilogue needs from global memory is fetched HERE, once: a load issued in the steady
  // state waits behind this SM's own weight copies (up to three chunks, several microseconds) and the warp
  // that waits for it holds up every stage.  The residual vector goes to the free half of the staging area
  // (this epilogue has no norm weights); the rotary frequencies and the two positions to shared memory /
  // registers.
  const T* rs_s = nullptr;
  if (EPI == EPI_RESID && a.resid && a.tp_world <= 1 && (a.N & 7) == 0 &&
      (size_t)K * 2 + (size_t)a.N * 2 <= ring.stage_bytes &&
      (reinterpret_cast<uintptr_t>(a.resid) & 15) == 0) {
    const uint4* rg = reinterpret_cast<const uint4*>(a.resid);
    constexpr int NT = GV_CONSUMER_WARPS * 32;
    uint4 rr[4];  // loads first, stores after (see above); 4 x 256 vectors cover N <= 8192
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = tid + i * NT;
      rr[i] = make_uint4(0, 0, 0, 0);
      if (v < a.N / 8) rr[i] = COHERENT ? __ldcg(rg + v) : rg[v];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = tid + i * NT;
      if (v < a.N / 8) ns[v] = rr[i];
    }
    for (int v = tid + 4 * NT; v < a.N / 8; v += NT) ns[v] = COHERENT ? __ldcg(rg + v) : rg[v];
    rs_s = reinterpret_cast<const T*>(ns);
  }
  int rope_pos_r = 0, cache_pos_r = 0;
  if (EPI == EPI_QKV) {
    if (tid < 64) cs.inv_freq[tid] = a.inv_freq[tid];
    rope_pos_r = *a.rope_pos;
    cache_pos_r = *a.pos;
  }
  float rstd = 1.f;
  if (a.norm_w) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    if (lane == 0) cs.ssq[warp] = sq;
  }
  consumer_bar();
  if (threadIdx.x == 0) GEMV_STAMP(a, 7);
  if (a.norm_w) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < GV_CONSUMER_WARPS; ++w) tot += cs.ssq[w];
    rstd = rsqrtf(tot / (float)K + a.eps);
  }
  float xr[KV][8];
#pragma unroll
  for (int j = 0; j < KV; ++j) {
    unpack8<T>(xs[wk * KV * 32 + j * 32 + lane], xr[j]);
    if (a.norm_w) {
      float nw[8];
      unpack8<T>(ns[wk * KV * 32 + j * 32 + lane], nw);
#pragma unroll
      for (int e = 0; e < 8; ++e) xr[j][e] *= nw[e];
    }
  }
  if (threadIdx.x == 0) GEMV_STAMP(a, 2);
#ifdef OMNIKV_TRACE
  bool first_stage = true;
#endif
  unsigned long long my_best = 0ull;
  unsigned tp_tag = 0u;
  if (EPI == EPI_RESID && a.tp_world > 1) tp_tag = __ldcg(a.tp_epoch) * 256u + a.tp_seq + 1u;
  for (;; ++it) {
    const int slot = it % GV_STAGES;
    const bool ok = mbar_wait(&ring.full_bar[slot], (it / GV_STAGES) & 1);
#ifdef OMNIKV_TRACE
    if (first_stage && threadIdx.x == 0) GEMV_STAMP(a, 3);  // first chunk has landed
    first_stage = false;
#endif
    if (!ok) {  // the copy never landed: flag it; every consumer leaves together after the barrier below
      cs.fail = 1;
      atomicExch(a.status, 2);
    }
    const int chunk = ok ? ring.slot_chunk[slot] : -1;
    if (ok && chunk < 0) {  // end marker of the phase: hand the slot back and stop
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty_bar[slot]);
      ++it;
      break;
    }
    float acc = 0.f;
    if (ok) {
      const uint4* wsm = reinterpret_cast<const uint4*>(ring.smem + (size_t)slot * ring.slot_bytes + (size_t)wr * ROW_BYTES) + wk * KV * 32;
      float acc2[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < KV; ++j) {
        float wf[8];
        unpack8<T>(wsm[j * 32 + lane], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc2[e & 1] = fmaf(wf[e], xr[j][e], acc2[e & 1]);
      }
      acc = acc2[0] + acc2[1];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      __syncwarp();
      if (lane == 0) mbar_arrive(&ring.empty_bar[slot]);
    }
    if (lane == 0) cs.part[it & 1][wr][wk] = acc;
    consumer_bar();
    if (cs.fail) return false;  // uniform: written before the barrier, never cleared

    // ---- epilogue: HALF threads, each owning row p of piece 0 and row p of piece 1 ----
    if (tid < HALF) {
      const int p = tid;
      float r0 = 0.f, r1 = 0.f;
#pragma unroll
      for (int w = 0; w < WK; ++w) {
        r0 += cs.part[it & 1][p][w];
        r1 += cs.part[it & 1][p + HALF][w];
      }
      r0 *= rstd;
      r1 *= rstd;
      int row0, row1;
      piece_rows<HALF, EPI>(a, chunk, row0, row1);
      row0 += p;
      row1 += p;
      if (EPI == EPI_RESID && a.tp_world > 1) {
        // {value, tag} in one 8-byte store per entry, straight into every rank's buffer (the local one included)
        const uint2 v0 = make_uint2(__float_as_uint(r0), tp_tag), v1 = make_uint2(__float_as_uint(r1), tp_tag);
        for (int pr = 0; pr < a.tp_world; ++pr) {
          __stcg(a.tp_peer_ll[pr] + row0, v0);
          __stcg(a.tp_peer_ll[pr] + row1, v1);
        }
      } else if (EPI == EPI_RESID) {
        const T* rs = static_cast<const T*>(a.resid);
        T* out = static_cast<T*>(a.out);
        float b0 = 0.f, b1 = 0.f;
        if (rs_s) {
          b0 = to_float(rs_s[row0]);
          b1 = to_float(rs_s[row1]);
        } else if (rs) {
          if (COHERENT) {
            const unsigned short u0 = __ldcg(reinterpret_cast<const unsigned short*>(rs) + row0);
            const unsigned short u1 = __ldcg(reinterpret_cast<const unsigned short*>(rs) + row1);
            b0 = to_float(*reinterpret_cast<const T*>(&u0));
            b1 = to_float(*reinterpret_cast<const T*>(&u1));
          } else {
            b0 = to_float(rs[row0]);
            b1 = to_float(rs[row1]);
          }
        }
        out[row0] = from_float<T>(r0 + b0);
        out[row1] = from_float<T>(r1 + b1);
      } else if (EPI == EPI_GATEUP) {
        const float sg = r0 / (1.f + __expf(-r0));
        static_cast<T*>(a.out)[row0] = from_float<T>(sg * r1);
      } else if (EPI == EPI_LOGITS) {
        a.logits[row0] = r0;
        a.logits[row1] = r1;
        const unsigned long long c0 = ((unsigned long long)float_to_key(r0) << 32) | (0xffffffffu - (unsigned)(a.row_offset + row0));
        const unsigned long long c1 = ((unsigned long long)float_to_key(r1) << 32) | (0xffffffffu - (unsigned)(a.row_offset + row1));
        my_best = max(my_best, max(c0, c1));
      } else {  // EPI_QKV
        const int head = row0 >> 7, i2 = row0 & 127;  // i2 in [0, 64)
        float o0 = r0, o1 = r1;
        if (head < a.H + a.KVH) {
          float sn, cs_;
          sincosf((float)rope_pos_r * cs.inv_freq[i2], &sn, &cs_);
          o0 = r0 * cs_ - r1 * sn;
          o1 = r1 * cs_ + r0 * sn;
        }
        T* dst;
        if (head < a.H) {
          dst = static_cast<T*>(a.q_out) + (size_t)head * 128;
        } else if (head < a.H + a.KVH) {
          dst = static_cast<T*>(a.k_cache) + (size_t)(head - a.H) * a.kv_sh + (size_t)cache_pos_r * a.kv_sr;
        } else {
          dst = static_cast<T*>(a.v_cache) + (size_t)(head - a.H - a.KVH) * a.kv_sh + (size_t)cache_pos_r * a.kv_sr;
        }
        dst[i2] = from_float<T>(o0);
        dst[i2 + 64] = from_float<T>(o1);
      }
    }
  }
  if (threadIdx.x == 0) GEMV_STAMP(a, 8);
  if (EPI == EPI_LOGITS) {
    consumer_bar();
    if (tid < HALF) cs.best[tid] = my_best;
    consumer_bar();
    if (tid == 0) {
      unsigned long long b = 0ull;
#pragma unroll
      for (int i = 0; i < HALF; ++i) b = max(b, cs.best[i]);
      if (b != 0ull) atomicMax(a.best, b);
    }
  }
  return true;
}

__device__ __forceinline__ void ring_init(uint64_t* full_bar, uint64_t* empty_bar, ConsumerShared& cs) {
  if (threadIdx.x == 0) {
    cs.fail = 0;
#pragma unroll
    for (int s = 0; s < GV_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], GV_CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
}

// ---- one phase per launch ----------------------------------------------------------------------
template <typename T, int KV, int WK, int EPI>
__global__ void __launch_bounds__(GV_THREADS, 1) decode_gemv_kernel(const GemvArgs a) {
  constexpr int K = WK * KV * 256;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[GV_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[GV_STAGES];
  __shared__ ConsumerShared cs;
  __shared__ int slot_chunk[GV_STAGES];
  ring_init(full_bar, empty_bar, cs);
  constexpr unsigned SLOT = GV_CONSUMER_WARPS / WK * K * 2;
  Ring ring{smem, full_bar, empty_bar, SLOT, slot_chunk, smem + GV_STAGES * SLOT, (unsigned)K * 4u, &cs.fail};
  int it = 0;
  // Programmatic dependent launch: the grid is one CTA per SM, all resident, so the next kernel may be
  // scheduled behind it right away.  The producer starts streaming weights at once (they depend on nothing);
  // the consumers wait for the previous kernel before they touch activations or write any output.
  pdl_trigger();
  if (threadIdx.x == 0) {
    GEMV_STAMP(a, 0);
#ifdef OMNIKV_TRACE
    if (blockIdx.x < kGemvTraceCtas)
      g_gemv_trace[(a.trace_slot * kGemvTraceCtas + blockIdx.x) * kGemvTraceWords + 10] = 1000ull + EPI * 10 + (a.tp_world > 1 ? (a.tp_my_ll ? 2 : (EPI == EPI_RESID ? 1 : 0)) : 0);
#endif
  }
  if ((threadIdx.x >> 5) == GV_CONSUMER_WARPS) {
    if ((threadIdx.x & 31) == 0) {
      produce_phase<T, KV, WK, EPI>(a, ring, it);
      GEMV_STAMP(a, 5);  // last copy issued
    }
    return;
  }
  // A consumer of a tensor-parallel exchange does not wait for its predecessor to complete: what it needs from it
  // arrives as tagged entries (consume_phase).  Every other kernel reads plain memory and waits.
  if (!(a.tp_world > 1 && a.tp_my_ll != nullptr)) pdl_wait();
  if (threadIdx.x == 0) GEMV_STAMP(a, 1);
  consume_phase<T, KV, WK, EPI, false>(a, ring, cs, it);
  if (threadIdx.x == 0) GEMV_STAMP(a, 4);
}

// ---- the GEMV chain of a decoder layer in ONE cooperative launch -----------------------------------
// Phases: [output projection + residual] -> [RMSNorm + gate/up + SiLU] -> [down projection + residual]
// -> [RMSNorm + next layer's QKV + RoPE + append | final RMSNorm + logits + arg-max].  Between phases the
// activations (a few KB) go through global memory and a grid-wide barrier; the weight stream does not
// stop there: the producer thread keeps filling the ring with the next phase's rows, which depend on
// nothing, so HBM stays busy across the barrier and across the per-phase prologue.
struct ChainArgs {
  GemvArgs ph[4];
  int kind[4];          // ChainKind, or -1 when the phase is skipped
  unsigned* grid_sync;  // one word: arrivals | generation << 16; zero before the first launch, self-resetting
  const void* next_w;         // optional: weights the next launch reads first, prefetched into L2 at the end
  size_t next_w_bytes;
};
enum ChainKind { CK_O = 0, CK_GATEUP = 1, CK_DOWN = 2, CK_QKV = 3, CK_LOGITS = 4 };

// Called by ONE thread per CTA after a CTA-level barrier.  One 32-bit word: arrivals in the low half,
// generation in the high half.  The last arriver adds (1 << 16) - n_blocks, which clears the count and
// bumps the generation in a single atomic; the others poll for the generation to change.  Bounded.
__device__ __forceinline__ bool grid_barrier(unsigned* sync, unsigned n_blocks) {
  __threadfence();
  const unsigned old = atomicAdd(sync, 1u);
  if ((old & 0xffffu) == n_blocks - 1) {
    atomicAdd(sync, 0x10000u - n_blocks);
  } else {
    const unsigned gen = old >> 16;
    unsigned spin = 0;
    while ((ld_volatile_u32(sync) >> 16) == gen) {
      if (++spin > GV_SPIN_LIMIT) return false;
    }
  }
  __threadfence();
  return true;
}

template <typename T, int KVH_, int WKH_, int KVI_, int WKI_>
__global__ void __launch_bounds__(GV_THREADS, 1) decode_chain_kernel(const ChainArgs c) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[GV_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[GV_STAGES];
  __shared__ ConsumerShared cs;
  constexpr unsigned SLOT_H = GV_CONSUMER_WARPS / WKH_ * (WKH_ * KVH_ * 256) * 2;
  constexpr unsigned SLOT_I = GV_CONSUMER_WARPS / WKI_ * (WKI_ * KVI_ * 256) * 2;
  __shared__ int slot_chunk[GV_STAGES];
  ring_init(full_bar, empty_bar, cs);
  constexpr unsigned CHAIN_STAGE_BYTES = 4u * (WKH_ * KVH_ * 256) > 2u * (WKI_ * KVI_ * 256) ? 4u * (WKH_ * KVH_ * 256) : 2u * (WKI_ * KVI_ * 256);
  constexpr unsigned SLOT = SLOT_H > SLOT_I ? SLOT_H : SLOT_I;
  Ring ring{smem, full_bar, empty_bar, SLOT, slot_chunk, smem + GV_STAGES * SLOT, CHAIN_STAGE_BYTES, &cs.fail};
  int it = 0;
  if ((threadIdx.x >> 5) == GV_CONSUMER_WARPS) {
    if ((threadIdx.x & 31) == 0) {
      for (int p = 0; p < 4; ++p) {
        bool ok = true;
        switch (c.kind[p]) {
          case CK_O: ok = produce_phase<T, KVH_, WKH_, EPI_RESID>(c.ph[p], ring, it); break;
          case CK_GATEUP: ok = produce_phase<T, KVH_, WKH_, EPI_GATEUP>(c.ph[p], ring, it); break;
          case CK_DOWN: ok = produce_phase<T, KVI_, WKI_, EPI_RESID>(c.ph[p], ring, it); break;
          case CK_QKV: ok = produce_phase<T, KVH_, WKH_, EPI_QKV>(c.ph[p], ring, it); break;
          case CK_LOGITS: ok = produce_phase<T, KVH_, WKH_, EPI_LOGITS>(c.ph[p], ring, it); break;
          default: break;
        }
        if (!ok) break;
        int nx = p + 1;
        while (nx < 4 && c.kind[nx] < 0) ++nx;
        if (nx < 4) {
          switch (c.kind[nx]) {
            case CK_GATEUP: prefetch_phase_head<T, KVH_, WKH_, EPI_GATEUP>(c.ph[nx]); break;
            case CK_DOWN: prefetch_phase_head<T, KVI_, WKI_, EPI_RESID>(c.ph[nx]); break;
            case CK_QKV: prefetch_phase_head<T, KVH_, WKH_, EPI_QKV>(c.ph[nx]); break;
            case CK_LOGITS: prefetch_phase_head<T, KVH_, WKH_, EPI_LOGITS>(c.ph[nx]); break;
            default: break;
          }
        } else if (c.next_w) {
          // the weights the NEXT launch starts with: they wait in L2 while the attention kernel runs
          const size_t per = ((c.next_w_bytes / gridDim.x) / 16) * 16;
          const unsigned char* src = static_cast<const unsigned char*>(c.next_w) + (size_t)blockIdx.x * per;
          for (size_t off = 0; off < per; off += 65536) l2_prefetch(src + off, (unsigned)(per - off < 65536 ? per - off : 65536));
          break;
        }
      }
    }
    return;
  }
  bool first = true;
  for (int p = 0; p < 4; ++p) {
    if (c.kind[p] < 0) continue;
    if (!first) {
      // every CTA's outputs of the previous phase must be visible before this phase reads them
      consumer_bar();
      if (threadIdx.x == 0 && !grid_barrier(c.grid_sync, gridDim.x)) {
        cs.fail = 1;
        atomicExch(c.ph[p].status, 3);
      }
      consumer_bar();
      if (cs.fail) return;
    }
    first = false;
    bool ok = true;
    switch (c.kind[p]) {
      case CK_O: ok = consume_phase<T, KVH_, WKH_, EPI_RESID, true>(c.ph[p], ring, cs, it); break;
      case CK_GATEUP: ok = consume_phase<T, KVH_, WKH_, EPI_GATEUP, true>(c.ph[p], ring, cs, it); break;
      case CK_DOWN: ok = consume_phase<T, KVI_, WKI_, EPI_RESID, true>(c.ph[p], ring, cs, it); break;
      case CK_QKV: ok = consume_phase<T, KVH_, WKH_, EPI_QKV, true>(c.ph[p], ring, cs, it); break;
      case CK_LOGITS: ok = consume_phase<T, KVH_, WKH_, EPI_LOGITS, true>(c.ph[p], ring, cs, it); break;
      default: break;
    }
    if (!ok) return;
  }
}

__global__ void argmax_finalize_kernel(const unsigned long long* best, long long* token) {
  token[0] = (long long)(0xffffffffu - (unsigned)(best[0] & 0xffffffffull));
}

template <typename T, int KV, int WK, int EPI>
int launch_one(const GemvArgs& a, int n_sms, cudaStream_t st) {
  constexpr int K = WK * KV * 256;
  constexpr int RPS = GV_CONSUMER_WARPS / WK;
  const size_t smem = (size_t)GV_STAGES * RPS * K * 2 + (size_t)K * 4;  // ring + staged activations and norm weights
  auto kern = decode_gemv_kernel<T, KV, WK, EPI>;
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = a.n_chunks < n_sms ? a.n_chunks : n_sms;
  GemvArgs aa = a;
  if (aa.tail_next) {
    // The last chunks of a long matrix are handed out dynamically (two per CTA on average): SMs that stream a
    // little faster take more of them, which evens out the end of the kernel.  Worth it only when a CTA has
    // many chunks; calls alternate between the two counter pairs of the caller's buffer, so that a launch
    // that starts early (programmatic dependent launch) never shares a pair with the one before it.
    static unsigned toggle = 0;
    const int pool = 2 * grid;
    if (aa.tp_world <= 1 && aa.n_chunks >= 8 * grid) {
      aa.tail_pool = pool;
      aa.tail_next += 2 * (toggle++ & 1u);
    } else {
      aa.tail_next = nullptr;
    }
  }
#ifdef OMNIKV_TRACE
  GemvArgs b = aa;
  b.trace_slot = trace_next_slot();
  OMNIKV_CUDA_OK(launch_pdl(kern, dim3(grid), dim3(GV_THREADS), smem, st, b));
#else
  OMNIKV_CUDA_OK(launch_pdl(kern, dim3(grid), dim3(GV_THREADS), smem, st, aa));
#endif
  return OMNIKV_OK;
}

template <typename T, int EPI>
int dispatch_k(const GemvArgs& a, int n_sms, cudaStream_t st) {
  switch (a.K) {
    case 512: return launch_one<T, 2, 1, EPI>(a, n_sms, st);
    case 1024: return launch_one<T, 4, 1, EPI>(a, n_sms, st);
    case 1792: return launch_one<T, 7, 1, EPI>(a, n_sms, st);
    case 2048: return launch_one<T, 8, 1, EPI>(a, n_sms, st);
    case 3584: return launch_one<T, 14, 1, EPI>(a, n_sms, st);
    case 4096: return launch_one<T, 16, 1, EPI>(a, n_sms, st);
    case 7168: return launch_one<T, 14, 2, EPI>(a, n_sms, st);
    case 8192: return launch_one<T, 16, 2, EPI>(a, n_sms, st);
    case 14336: return launch_one<T, 14, 4, EPI>(a, n_sms, st);
    default: return OMNIKV_E_UNSUPPORTED;
  }
}

template <int EPI>
int dispatch(int dtype, const GemvArgs& a, cudaStream_t st) {
  int dev = 0, n_sms = 0;
  OMNIKV_CUDA_OK(cudaGetDevice(&dev));
  OMNIKV_CUDA_OK(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev));
  if (dtype == OMNIKV_BF16) return dispatch_k<__nv_bfloat16, EPI>(a, n_sms, st);
  if (dtype == OMNIKV_F16) return dispatch_k<__half, EPI>(a, n_sms, st);
  return OMNIKV_E_UNSUPPORTED;
}

template <typename T, int KVH_, int WKH_, int KVI_, int WKI_>
int launch_chain(const ChainArgs& c, int n_sms, cudaStream_t st) {
  constexpr unsigned SLOT_H = GV_CONSUMER_WARPS / WKH_ * (WKH_ * KVH_ * 256) * 2;
  constexpr unsigned SLOT_I = GV_CONSUMER_WARPS / WKI_ * (WKI_ * KVI_ * 256) * 2;
  constexpr int K_H = WKH_ * KVH_ * 256, K_I = WKI_ * KVI_ * 256;
  const size_t smem = (size_t)GV_STAGES * (SLOT_H > SLOT_I ? SLOT_H : SLOT_I) + (size_t)(4 * K_H > 2 * K_I ? 4 * K_H : 2 * K_I);
  auto kern = decode_chain_kernel<T, KVH_, WKH_, KVI_, WKI_>;
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int per_sm = 0;
  OMNIKV_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, GV_THREADS, smem));
  if (per_sm < 1) return OMNIKV_E_UNSUPPORTED;
  void* args[] = {const_cast<ChainArgs*>(&c)};
  // cooperative: every CTA must be resident, the phases are separated by grid-wide barriers
  OMNIKV_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), dim3(n_sms), dim3(GV_THREADS), args, smem, st));
  return OMNIKV_OK;
}

// Exchange buffer of one rank: [2 slots][8 ranks][hidden] entries of {fp32 partial, tag} (the fused projection +
// all-reduce kernels), then [2][8] flag words (used by omnikv_tp_allreduce_sum, which lays fp32/16-bit vectors over
// the first half of the entry area).
size_t tp_partials_bytes(int hidden) { return (size_t)2 * 8 * hidden * sizeof(uint2); }

// Producer fields: where MY partials of exchange `seq` go on every rank.
int tp_fill_producer(GemvArgs& a, const omnikv_tp_exchange* t, int n_rows) {
  if (!t || t->world <= 1) return OMNIKV_OK;
  if (t->world > 8 || t->rank < 0 || t->rank >= t->world || !t->epoch || t->hidden != n_rows) return OMNIKV_E_BADARG;
  const int slot = t->seq & 1;
  a.tp_world = t->world;
  for (int p = 0; p < t->world; ++p) {
    if (!t->peer_base[p]) return OMNIKV_E_BADARG;
    a.tp_peer_ll[p] = static_cast<uint2*>(t->peer_base[p]) + ((size_t)slot * 8 + t->rank) * t->hidden;
  }
  a.tp_epoch = t->epoch;
  a.tp_seq = (unsigned)t->seq;
  return OMNIKV_OK;
}

// Consumer fields: the local slot holding every rank's partials of exchange `seq`.
int tp_fill_consumer(GemvArgs& a, const omnikv_tp_exchange* t, int k, void* h_out) {
  if (!t || t->world <= 1) return OMNIKV_OK;
  if (t->world > 8 || t->rank < 0 || t->rank >= t->world || !t->epoch || t->hidden != k || !t->peer_base[t->rank])
    return OMNIKV_E_BADARG;
  if (k > kTpMaxHidden) return OMNIKV_E_UNSUPPORTED;
  const int slot = t->seq & 1;
  unsigned char* base = static_cast<unsigned char*>(t->peer_base[t->rank]);
  a.tp_world = t->world;
  a.tp_my_ll = reinterpret_cast<const uint2*>(base) + (size_t)slot * 8 * t->hidden;
  a.tp_h_out = h_out;
  a.tp_epoch = t->epoch;
  a.tp_seq = (unsigned)t->seq;
  return OMNIKV_OK;
}

int rows_per_stage(int K) {
  const int wk = K <= 4096 ? 1 : (K <= 8192 ? 2 : 4);
  return GV_CONSUMER_WARPS / wk;
}

inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace omnikv

extern "C" int omnikv_decode_qkv(int dtype, const void* h, const void* norm_w, float eps, const void* w_qkv, int hidden,
                                 int H, int KVH, int head_dim, const float* inv_freq, const int32_t* rope_pos,
                                 void* q_out, void* k_cache_seq, void* v_cache_seq, int64_t kv_stride_h,
                                 int64_t kv_stride_row, const int32_t* cache_pos, const omnikv_tp_exchange* tp_in,
                                 void* h_inout, int32_t* status, void* stream) {
  using namespace omnikv;
  if (!h || !norm_w || !w_qkv || !inv_freq || !rope_pos || !q_out || !k_cache_seq || !v_cache_seq || !cache_pos || !status)
    return OMNIKV_E_BADARG;
  if (head_dim != kHeadDim) return OMNIKV_E_UNSUPPORTED;
  if (!al16(h) || !al16(norm_w) || !al16(w_qkv)) return OMNIKV_E_BADARG;
  GemvArgs a = {};
  a.W = w_qkv; a.x = h; a.norm_w = norm_w; a.eps = eps; a.N = (H + 2 * KVH) * kHeadDim; a.K = hidden;
  a.n_chunks = a.N / rows_per_stage(hidden); a.partner_rows = 64;
  a.q_out = q_out; a.k_cache = k_cache_seq; a.v_cache = v_cache_seq; a.kv_sh = kv_stride_h; a.kv_sr = kv_stride_row;
  a.pos = cache_pos; a.rope_pos = rope_pos; a.inv_freq = inv_freq; a.H = H; a.KVH = KVH; a.status = status;
  if (const int rc = tp_fill_consumer(a, tp_in, hidden, h_inout)) return rc;
  return dispatch<EPI_QKV>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int omnikv_decode_gemv_residual(int dtype, const void* w, int N, int K, const void* x, const void* resid,
                                           void* out, const omnikv_tp_exchange* tp_out, int32_t* status,
                                           void* stream) {
  using namespace omnikv;
  const bool exchange = tp_out && tp_out->world > 1;
  if (!w || !x || (!out && !exchange) || !status || N <= 0) return OMNIKV_E_BADARG;
  if (!al16(w) || !al16(x)) return OMNIKV_E_BADARG;
  const int rps = rows_per_stage(K);
  if (N % rps) return OMNIKV_E_UNSUPPORTED;
  GemvArgs a = {};
  a.W = w; a.x = x; a.N = N; a.K = K; a.n_chunks = N / rps; a.resid = resid; a.out = out; a.status = status;
  if (const int rc = tp_fill_producer(a, tp_out, N)) return rc;
  return dispatch<EPI_RESID>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int omnikv_decode_gate_up(int dtype, const void* h, const void* norm_w, float eps, const void* w_gate_up,
                                     int hidden, int inter, void* act_out, const omnikv_tp_exchange* tp_in,
                                     void* h_inout, int32_t* sched, int32_t* status, void* stream) {
  using namespace omnikv;
  if (!h || !norm_w || !w_gate_up || !act_out || !status || inter <= 0) return OMNIKV_E_BADARG;
  if (!al16(h) || !al16(norm_w) || !al16(w_gate_up)) return OMNIKV_E_BADARG;
  const int half = rows_per_stage(hidden) / 2;
  if (inter % half) return OMNIKV_E_UNSUPPORTED;
  GemvArgs a = {};
  a.W = w_gate_up; a.x = h; a.norm_w = norm_w; a.eps = eps; a.N = 2 * inter; a.K = hidden;
  a.n_chunks = inter / half; a.partner_rows = inter; a.out = act_out; a.status = status; a.tail_next = sched;
  if (const int rc = tp_fill_consumer(a, tp_in, hidden, h_inout)) return rc;
  return dispatch<EPI_GATEUP>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int omnikv_decode_logits(int dtype, const void* h, const void* norm_w, float eps, const void* w_head,
                                    int hidden, int vocab_rows, int row_offset, float* logits,
                                    unsigned long long* best_scratch, int64_t* token_out,
                                    const omnikv_tp_exchange* tp_in, int32_t* status, void* stream) {
  using namespace omnikv;
  if (!h || !norm_w || !w_head || !logits || !best_scratch || !status || vocab_rows <= 0) return OMNIKV_E_BADARG;
  if (!al16(h) || !al16(norm_w) || !al16(w_head)) return OMNIKV_E_BADARG;
  const int rps = rows_per_stage(hidden);
  if (vocab_rows % rps) return OMNIKV_E_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  OMNIKV_CUDA_OK(cudaMemsetAsync(best_scratch, 0, sizeof(unsigned long long), st));
  GemvArgs a = {};
  a.W = w_head; a.x = h; a.norm_w = norm_w; a.eps = eps; a.N = vocab_rows; a.K = hidden; a.n_chunks = vocab_rows / rps;
  a.logits = logits; a.best = best_scratch; a.row_offset = row_offset; a.status = status;
  if (const int rc0 = tp_fill_consumer(a, tp_in, hidden, nullptr)) return rc0;
  const int rc = dispatch<EPI_LOGITS>(dtype, a, st);
  if (rc != OMNIKV_OK) return rc;
  if (token_out) {
    argmax_finalize_kernel<<<1, 1, 0, st>>>(best_scratch, reinterpret_cast<long long*>(token_out));
    OMNIKV_CUDA_OK(cudaGetLastError());
  }
  return OMNIKV_OK;
}

extern "C" int omnikv_decode_chain(const omnikv_chain_params* p, void* stream) {
  using namespace omnikv;
  if (!p || !p->h || !p->grid_sync || !p->status) return OMNIKV_E_BADARG;
  if (p->dtype != OMNIKV_BF16 && p->dtype != OMNIKV_F16) return OMNIKV_E_UNSUPPORTED;
  const int hidden = p->hidden, inter = p->inter;
  if (p->H * kHeadDim != hidden) return OMNIKV_E_UNSUPPORTED;  // the output projection is square
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ChainArgs c = {};
  for (int i = 0; i < 4; ++i) c.kind[i] = -1;
  c.grid_sync = p->grid_sync;
  int* counters = p->chunk_counters;  // 4 ints, zero at launch (dynamic scheduling), or NULL (static)
  c.next_w = p->next_w;
  c.next_w_bytes = p->next_w ? p->next_w_bytes : 0;
  const int rps_h = rows_per_stage(hidden), rps_i = rows_per_stage(inter);
  if (p->w_o) {
    if (!p->attn_out || !al16(p->w_o) || !al16(p->attn_out) || hidden % rps_h) return OMNIKV_E_BADARG;
    GemvArgs& a = c.ph[0];
    a.W = p->w_o; a.x = p->attn_out; a.N = hidden; a.K = hidden; a.n_chunks = hidden / rps_h;
    a.resid = p->h; a.out = p->h; a.status = p->status; a.next_chunk = counters ? counters + 0 : nullptr;
    c.kind[0] = CK_O;
  }
  if (p->w_gate_up) {
    if (!p->w_down || !p->post_norm_w || !p->act_scratch || !al16(p->w_gate_up) || !al16(p->w_down) ||
        !al16(p->act_scratch) || inter % (rps_h / 2) || hidden % rps_i)
      return OMNIKV_E_BADARG;
    GemvArgs& g = c.ph[1];
    g.W = p->w_gate_up; g.x = p->h; g.norm_w = p->post_norm_w; g.eps = p->eps; g.N = 2 * inter; g.K = hidden;
    g.n_chunks = inter / (rps_h / 2); g.partner_rows = inter; g.out = p->act_scratch; g.status = p->status;
    g.next_chunk = counters ? counters + 1 : nullptr;
    c.kind[1] = CK_GATEUP;
    GemvArgs& d = c.ph[2];
    d.W = p->w_down; d.x = p->act_scratch; d.N = hidden; d.K = inter; d.n_chunks = hidden / rps_i;
    d.resid = p->h; d.out = p->h; d.status = p->status; d.next_chunk = counters ? counters + 2 : nullptr;
    c.kind[2] = CK_DOWN;
  }
  if (p->w_qkv && p->w_head) return OMNIKV_E_BADARG;
  if (p->w_qkv) {
    if (!p->in_norm_w || !p->inv_freq || !p->rope_pos || !p->q_out || !p->k_cache_seq || !p->v_cache_seq ||
        !p->cache_pos || !al16(p->w_qkv))
      return OMNIKV_E_BADARG;
    GemvArgs& a = c.ph[3];
    a.W = p->w_qkv; a.x = p->h; a.norm_w = p->in_norm_w; a.eps = p->eps; a.N = (p->H + 2 * p->KVH) * kHeadDim;
    a.K = hidden; a.n_chunks = a.N / rps_h; a.partner_rows = 64;
    a.q_out = p->q_out; a.k_cache = p->k_cache_seq; a.v_cache = p->v_cache_seq; a.kv_sh = p->kv_stride_h;
    a.kv_sr = p->kv_stride_row; a.pos = p->cache_pos; a.rope_pos = p->rope_pos; a.inv_freq = p->inv_freq;
    a.H = p->H; a.KVH = p->KVH; a.status = p->status; a.next_chunk = counters ? counters + 3 : nullptr;
    c.kind[3] = CK_QKV;
  } else if (p->w_head) {
    if (!p->final_norm_w || !p->logits || !p->best_scratch || p->vocab_rows <= 0 || p->vocab_rows % rps_h ||
        !al16(p->w_head))
      return OMNIKV_E_BADARG;
    OMNIKV_CUDA_OK(cudaMemsetAsync(p->best_scratch, 0, sizeof(unsigned long long), st));
    GemvArgs& a = c.ph[3];
    a.W = p->w_head; a.x = p->h; a.norm_w = p->final_norm_w; a.eps = p->eps; a.N = p->vocab_rows; a.K = hidden;
    a.n_chunks = p->vocab_rows / rps_h; a.logits = p->logits; a.best = p->best_scratch; a.row_offset = 0;
    a.status = p->status; a.next_chunk = counters ? counters + 3 : nullptr;
    c.kind[3] = CK_LOGITS;
  }
  int dev = 0, n_sms = 0;
  OMNIKV_CUDA_OK(cudaGetDevice(&dev));
  OMNIKV_CUDA_OK(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev));
  int rc = OMNIKV_E_UNSUPPORTED;
  const bool bf = p->dtype == OMNIKV_BF16;
  if (hidden == 4096 && inter == 14336)
    rc = bf ? launch_chain<__nv_bfloat16, 16, 1, 14, 4>(c, n_sms, st) : launch_chain<__half, 16, 1, 14, 4>(c, n_sms, st);
  else if (hidden == 512 && inter == 1024)
    rc = bf ? launch_chain<__nv_bfloat16, 2, 1, 4, 1>(c, n_sms, st) : launch_chain<__half, 2, 1, 4, 1>(c, n_sms, st);
  else if (hidden == 2048 && inter == 7168)
    rc = bf ? launch_chain<__nv_bfloat16, 8, 1, 14, 2>(c, n_sms, st) : launch_chain<__half, 8, 1, 14, 2>(c, n_sms, st);
  if (rc != OMNIKV_OK) return rc;
  if (p->w_head && p->token_out) {
    argmax_finalize_kernel<<<1, 1, 0, st>>>(p->best_scratch, reinterpret_cast<long long*>(p->token_out));
    OMNIKV_CUDA_OK(cudaGetLastError());
  }
  return OMNIKV_OK;
}

extern "C" int omnikv_decode_chain_supported(int dtype, int hidden, int inter, int H) {
  if (dtype != OMNIKV_BF16 && dtype != OMNIKV_F16) return 0;
  if (H * omnikv::kHeadDim != hidden) return 0;
  return (hidden == 4096 && inter == 14336) || (hidden == 512 && inter == 1024) || (hidden == 2048 && inter == 7168);
}

extern "C" size_t omnikv_tp_exchange_bytes(int hidden) {
  if (hidden <= 0) return 0;
  return omnikv::tp_partials_bytes(hidden) + 2 * 8 * sizeof(unsigned) + 192;  // padded to a multiple of 256
}

#ifdef OMNIKV_TRACE
extern "C" int omnikv_debug_gemv_trace(unsigned long long* host_out, int n_words) {
  return (int)cudaMemcpyFromSymbol(host_out, omnikv::g_gemv_trace, (size_t)n_words * 8);
}
#endif
