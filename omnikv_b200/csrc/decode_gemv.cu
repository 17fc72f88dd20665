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
constexpr int GV_STAGES = 3;
constexpr unsigned GV_SPIN_LIMIT = 1u << 24;

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
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  const unsigned addr = smem_u32(bar);
  for (unsigned spin = 0; spin < GV_SPIN_LIMIT; ++spin) {
    unsigned ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_bulk_g2s(void* smem_dst, const void* gmem_src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
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

// KV: 16-byte vectors per lane per K-slice; WK: warps along K.  K = WK * KV * 256.
// RPS = 8 / WK rows per stage, in two pieces of RPS/2 rows.
template <typename T, int KV, int WK, int EPI>
__global__ void __launch_bounds__(GV_THREADS, 1) decode_gemv_kernel(const GemvArgs a) {
  constexpr int RPS = GV_CONSUMER_WARPS / WK;
  constexpr int HALF = RPS / 2;
  constexpr int K = WK * KV * 256;
  constexpr unsigned ROW_BYTES = K * 2;
  constexpr unsigned PIECE_BYTES = HALF * ROW_BYTES;
  constexpr unsigned STAGE_BYTES = 2 * PIECE_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full_bar[GV_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[GV_STAGES];
  __shared__ float part[2][RPS][WK];
  __shared__ float ssq[GV_CONSUMER_WARPS];
  __shared__ unsigned long long best_s[RPS];
  __shared__ int fail_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_mine = a.n_chunks > (int)blockIdx.x ? (a.n_chunks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (tid == 0) {
    fail_s = 0;
#pragma unroll
    for (int s = 0; s < GV_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], GV_CONSUMER_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  // first row of the two pieces of chunk c
  auto piece_rows = [&](int c, int& row0, int& row1) {
    if (EPI == EPI_QKV) {
      constexpr int per_head = 64 / HALF;
      const int head = c / per_head, j = c % per_head;
      row0 = head * 128 + j * HALF;
      row1 = row0 + 64;
    } else if (EPI == EPI_GATEUP) {
      row0 = c * HALF;
      row1 = row0 + a.partner_rows;
    } else {
      row0 = c * RPS;
      row1 = row0 + HALF;
    }
  };

  if (warp == GV_CONSUMER_WARPS) {
    // ---------------- producer: one thread feeds the ring ----------------
    if (lane == 0) {
      const T* W = static_cast<const T*>(a.W);
      for (int it = 0; it < n_mine; ++it) {
        const int slot = it % GV_STAGES;
        if (it >= GV_STAGES) {
          if (!mbar_wait(&empty_bar[slot], ((it / GV_STAGES) - 1) & 1)) {
            atomicExch(a.status, 1);
            break;
          }
        }
        int row0, row1;
        piece_rows((int)blockIdx.x + it * (int)gridDim.x, row0, row1);
        unsigned char* dst = smem + (size_t)slot * STAGE_BYTES;
        mbar_expect_tx(&full_bar[slot], STAGE_BYTES);
        tma_bulk_g2s(dst, W + (size_t)row0 * K, PIECE_BYTES, &full_bar[slot]);
        tma_bulk_g2s(dst + PIECE_BYTES, W + (size_t)row1 * K, PIECE_BYTES, &full_bar[slot]);
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int wk = warp % WK;   // K-slice
  const int wr = warp / WK;   // row within the stage
  // this warp's slice of x as fp32, times the norm weight; sum of squares of the raw x
  float xr[KV][8];
  float sq = 0.f;
  {
    const uint4* xv = reinterpret_cast<const uint4*>(static_cast<const T*>(a.x) + (size_t)wk * KV * 256);
    const uint4* nv = a.norm_w ? reinterpret_cast<const uint4*>(static_cast<const T*>(a.norm_w) + (size_t)wk * KV * 256) : nullptr;
#pragma unroll
    for (int j = 0; j < KV; ++j) {
      unpack8<T>(xv[j * 32 + lane], xr[j]);
      if (nv) {
        float nw[8];
        unpack8<T>(nv[j * 32 + lane], nw);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sq = fmaf(xr[j][e], xr[j][e], sq);
          xr[j][e] *= nw[e];
        }
      }
    }
  }
  float rstd = 1.f;
  if (a.norm_w) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    if (lane == 0) ssq[warp] = sq;
    asm volatile("bar.sync 1, %0;\n" ::"n"(GV_CONSUMER_WARPS * 32) : "memory");
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < WK; ++w) tot += ssq[w];  // warps 0..WK-1 cover K once
    rstd = rsqrtf(tot / (float)K + a.eps);
  }

  unsigned long long my_best = 0ull;
  for (int it = 0; it < n_mine; ++it) {
    const int slot = it % GV_STAGES;
    bool ok = mbar_wait(&full_bar[slot], (it / GV_STAGES) & 1);
    if (!ok) {  // the copy never landed: flag it; every consumer leaves together after the barrier below
      fail_s = 1;
      atomicExch(a.status, 2);
    }
    float acc = 0.f;
    if (ok) {
      const uint4* wsm = reinterpret_cast<const uint4*>(smem + (size_t)slot * STAGE_BYTES + (size_t)wr * ROW_BYTES) + wk * KV * 32;
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
      if (lane == 0) mbar_arrive(&empty_bar[slot]);
    }
    if (lane == 0) part[it & 1][wr][wk] = acc;
    asm volatile("bar.sync 1, %0;\n" ::"n"(GV_CONSUMER_WARPS * 32) : "memory");
    if (fail_s) break;  // uniform: written before the barrier, never cleared

    // ---- epilogue: HALF threads, each owning row p of piece 0 and row p of piece 1 ----
    if (tid < HALF) {
      const int p = tid;
      float r0 = 0.f, r1 = 0.f;
#pragma unroll
      for (int w = 0; w < WK; ++w) {
        r0 += part[it & 1][p][w];
        r1 += part[it & 1][p + HALF][w];
      }
      r0 *= rstd;
      r1 *= rstd;
      int row0, row1;
      piece_rows((int)blockIdx.x + it * (int)gridDim.x, row0, row1);
      row0 += p;
      row1 += p;
      if (EPI == EPI_RESID) {
        const T* rs = static_cast<const T*>(a.resid);
        T* out = static_cast<T*>(a.out);
        out[row0] = from_float<T>(r0 + (rs ? to_float(rs[row0]) : 0.f));
        out[row1] = from_float<T>(r1 + (rs ? to_float(rs[row1]) : 0.f));
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
        const int head = row0 >> 7, i = row0 & 127;  // i in [0, 64)
        float o0 = r0, o1 = r1;
        if (head < a.H + a.KVH) {
          float sn, cs;
          sincosf((float)(*a.rope_pos) * a.inv_freq[i], &sn, &cs);
          o0 = r0 * cs - r1 * sn;
          o1 = r1 * cs + r0 * sn;
        }
        T* dst;
        if (head < a.H) {
          dst = static_cast<T*>(a.q_out) + (size_t)head * 128;
        } else if (head < a.H + a.KVH) {
          dst = static_cast<T*>(a.k_cache) + (size_t)(head - a.H) * a.kv_sh + (size_t)(*a.pos) * a.kv_sr;
        } else {
          dst = static_cast<T*>(a.v_cache) + (size_t)(head - a.H - a.KVH) * a.kv_sh + (size_t)(*a.pos) * a.kv_sr;
        }
        dst[i] = from_float<T>(o0);
        dst[i + 64] = from_float<T>(o1);
      }
    }
  }
  if (EPI == EPI_LOGITS) {
    if (tid < HALF) best_s[tid] = my_best;
    asm volatile("bar.sync 1, %0;\n" ::"n"(GV_CONSUMER_WARPS * 32) : "memory");
    if (tid == 0) {
      unsigned long long b = 0ull;
#pragma unroll
      for (int i = 0; i < HALF; ++i) b = max(b, best_s[i]);
      if (n_mine > 0) atomicMax(a.best, b);
    }
  }
}

__global__ void argmax_finalize_kernel(const unsigned long long* best, long long* token) {
  token[0] = (long long)(0xffffffffu - (unsigned)(best[0] & 0xffffffffull));
}

template <typename T, int KV, int WK, int EPI>
int launch_one(const GemvArgs& a, int n_sms, cudaStream_t st) {
  constexpr int K = WK * KV * 256;
  constexpr int RPS = GV_CONSUMER_WARPS / WK;
  const size_t smem = (size_t)GV_STAGES * RPS * K * 2;
  auto kern = decode_gemv_kernel<T, KV, WK, EPI>;
  OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int grid = a.n_chunks < n_sms ? a.n_chunks : n_sms;
  kern<<<grid, GV_THREADS, smem, st>>>(a);
  OMNIKV_CUDA_OK(cudaGetLastError());
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
                                 int64_t kv_stride_row, const int32_t* cache_pos, int32_t* status, void* stream) {
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
  return dispatch<EPI_QKV>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int omnikv_decode_gemv_residual(int dtype, const void* w, int N, int K, const void* x, const void* resid,
                                           void* out, int32_t* status, void* stream) {
  using namespace omnikv;
  if (!w || !x || !out || !status || N <= 0) return OMNIKV_E_BADARG;
  if (!al16(w) || !al16(x)) return OMNIKV_E_BADARG;
  const int rps = rows_per_stage(K);
  if (N % rps) return OMNIKV_E_UNSUPPORTED;
  GemvArgs a = {};
  a.W = w; a.x = x; a.N = N; a.K = K; a.n_chunks = N / rps; a.resid = resid; a.out = out; a.status = status;
  return dispatch<EPI_RESID>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int omnikv_decode_gate_up(int dtype, const void* h, const void* norm_w, float eps, const void* w_gate_up,
                                     int hidden, int inter, void* act_out, int32_t* status, void* stream) {
  using namespace omnikv;
  if (!h || !norm_w || !w_gate_up || !act_out || !status || inter <= 0) return OMNIKV_E_BADARG;
  if (!al16(h) || !al16(norm_w) || !al16(w_gate_up)) return OMNIKV_E_BADARG;
  const int half = rows_per_stage(hidden) / 2;
  if (inter % half) return OMNIKV_E_UNSUPPORTED;
  GemvArgs a = {};
  a.W = w_gate_up; a.x = h; a.norm_w = norm_w; a.eps = eps; a.N = 2 * inter; a.K = hidden;
  a.n_chunks = inter / half; a.partner_rows = inter; a.out = act_out; a.status = status;
  return dispatch<EPI_GATEUP>(dtype, a, static_cast<cudaStream_t>(stream));
}

extern "C" int omnikv_decode_logits(int dtype, const void* h, const void* norm_w, float eps, const void* w_head,
                                    int hidden, int vocab_rows, int row_offset, float* logits,
                                    unsigned long long* best_scratch, int64_t* token_out, int32_t* status,
                                    void* stream) {
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
  const int rc = dispatch<EPI_LOGITS>(dtype, a, st);
  if (rc != OMNIKV_OK) return rc;
  if (token_out) {
    argmax_finalize_kernel<<<1, 1, 0, st>>>(best_scratch, reinterpret_cast<long long*>(token_out));
    OMNIKV_CUDA_OK(cudaGetLastError());
  }
  return OMNIKV_OK;
}
