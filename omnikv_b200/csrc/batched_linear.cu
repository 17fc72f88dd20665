// Weight-streaming projections of a batched decode step (up to 16 tokens) on the Blackwell tensor path.
//
//   y[b, n] = sum_k W[n, k] * x'[b, k]      x' = x, or RMSNorm(x) * norm_w (the 1/rms factor is applied to y)
//
// with the epilogues of a decoder layer: plain store (fused QKV projection, logits in fp32), residual add (output
// and down projection), SiLU(gate) * up (gate/up projection).  These are the third-party decoder modules the
// reference calls around its selection path (modeling/omnikv.py:156, :219-236, :361-373) at batch > 1.
//
// For 16 tokens a projection is still a stream of the weight matrix (16 flop per byte), but 16 multiply-adds per
// weight are too many for the CUDA cores at HBM speed, so the arithmetic goes to tcgen05: a tile of 128 weight rows
// x 64 columns (one TMA box, 128-byte swizzle) is the A operand (M = 128 rows = TMEM lanes), the activations
// [16 tokens x 64] the B operand (N = 16), the fp32 accumulator [128 x 16] lives in tensor memory and an epilogue
// thread owns ONE output row and reads its 16 token values with tcgen05.ld.
//
// Work split: unit = (block of 128 rows, slice of the K dimension).  A CTA serves ONE slice (its activations,
// at most 16 x 2048, stay in shared memory beside an eight-stage ring of weight tiles) and walks row blocks;
// S slices x (CTAs / S) row-block walkers fill the GPU for any matrix shape (the host picks S).  With S > 1 every
// unit leaves its partial sums in a workspace and the CTA that completes a row block's count adds the S partials
// in slice order (deterministic) and runs the epilogue -- no CTA ever waits for another one.  The sum of squares of
// the RMSNorm travels the same way (one more partial per slice).
// Every wait is bounded by time; on expiry the CTA raises a flag, all roles leave, copies in flight are waited for
// (bounded), tensor memory is released and status 7 is written.
#include "common.cuh"
#include "tc05.cuh"

namespace omnikv {
namespace {

constexpr int BL_M = 128;                      // weight rows per tile = TMEM lanes
constexpr int BL_NT = 16;                      // token columns of the accumulator
constexpr int BL_KC = 64;                      // K columns per stage (one 128-byte swizzled box row)
constexpr int BL_STAGE_BYTES = BL_M * 128;     // 16 KB
constexpr int BL_XBOX_BYTES = BL_NT * 128;     // activations of one K chunk: 16 rows x 128 bytes
constexpr int BL_STAGES = 8;
constexpr int BL_MAX_CHUNKS = 32;              // K chunks per slice (2048 columns: 64 KB of activations)
constexpr int BL_THREADS = 192;                // warps 0-3 epilogue / staging, 4 TMA producer, 5 MMA issuer
constexpr int BL_SMEM_BYTES = BL_STAGES * BL_STAGE_BYTES + BL_MAX_CHUNKS * BL_XBOX_BYTES + 1024;
constexpr int BL_MAX_ROW_BLOCKS = 4096, BL_MAX_SLICES = 32;
constexpr size_t BL_COUNTER_BYTES = BL_MAX_ROW_BLOCKS * sizeof(int);
constexpr size_t BL_SS_BYTES = BL_MAX_SLICES * BL_NT * sizeof(float);

enum { EPI_STORE = 0, EPI_STORE_F32 = 1, EPI_RESIDUAL = 2, EPI_SWIGLU = 3 };

struct BlArgs {
  const void* x;
  int64_t ldx;
  const void* norm_w;
  float eps;
  void* out;
  int64_t ldo;
  const void* resid;
  int64_t ldr;
  float* part;    // [R][S][Bt][128]
  float* ss;      // [S][16] sum of squares of x over the slice
  int* counters;  // [R], zero between calls
  int Bt, N, K, S, R, chunks, epi, inter;
  int* status;
};

struct BlShared {
  uint64_t full[BL_STAGES], empty[BL_STAGES];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t x_full;
  unsigned tmem_base;
  int fail;
  int issued;
  int last;
  float ss_own[BL_NT];
  float rstd[BL_NT];
};

__device__ __forceinline__ unsigned bl_vote_or(bool pred) {  // OR over the 128 epilogue threads (named barrier 1)
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
__device__ __forceinline__ void bl_bar() { asm volatile("bar.sync 1, 128;\n" ::: "memory"); }

template <typename T>
__device__ __forceinline__ float2 unpack2(unsigned u);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(unsigned u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(unsigned u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
template <typename T>
__device__ __forceinline__ unsigned pack2f(float a, float b);
template <>
__device__ __forceinline__ unsigned pack2f<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}
template <>
__device__ __forceinline__ unsigned pack2f<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

// Activations of this CTA's K slice -> shared memory as the B operand: per K chunk of 64 a box of [16 tokens x 128
// bytes], 16-byte piece q of token b at piece q ^ (b & 7).  Eight threads per token; tokens >= Bt are zero.  With a
// norm weight the elements are scaled by it (the 1/rms factor is applied to the accumulator).  Returns, to the
// eight threads of a token, the sum of squares of the token's raw elements over the slice.
template <typename T>
__device__ __forceinline__ float stage_x(unsigned char* x_s, const BlArgs& a, int c0, int nch, int tid) {
  const int b = tid >> 3, t8 = tid & 7;
  const T* xr = static_cast<const T*>(a.x) + (size_t)b * a.ldx;
  const T* nw = static_cast<const T*>(a.norm_w);
  const int total = nch * 8;  // 16-byte pieces of a token's slice
  float ss = 0.f;
  for (int base = 0; base < total; base += 64) {  // eight pieces per thread per round, loads before stores
    uint4 v[8], w[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int q = base + t8 + 8 * u;
      const int col = c0 * BL_KC + q * 8;
      v[u] = make_uint4(0, 0, 0, 0);
      w[u] = v[u];
      if (q < total && b < a.Bt && col < a.K) {
        v[u] = *reinterpret_cast<const uint4*>(xr + col);
        if (nw) w[u] = *reinterpret_cast<const uint4*>(nw + col);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int q = base + t8 + 8 * u;
      if (q >= total) continue;
      uint4 o = v[u];
      if (nw) {
        const unsigned* vi = reinterpret_cast<const unsigned*>(&v[u]);
        const unsigned* wi = reinterpret_cast<const unsigned*>(&w[u]);
        unsigned* oi = reinterpret_cast<unsigned*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 xv = unpack2<T>(vi[i]), wv = unpack2<T>(wi[i]);
          ss = fmaf(xv.x, xv.x, fmaf(xv.y, xv.y, ss));
          oi[i] = pack2f<T>(xv.x * wv.x, xv.y * wv.y);
        }
      }
      *reinterpret_cast<uint4*>(x_s + (q >> 3) * BL_XBOX_BYTES + b * 128 + (((q & 7) ^ (b & 7)) << 4)) = o;
    }
  }
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  return ss;
}

template <typename T>
__global__ void __launch_bounds__(BL_THREADS, 1)
batched_linear_kernel(const BlArgs a, const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ BlShared sh;
  __shared__ float ss_all[BL_MAX_SLICES * BL_NT];
  __shared__ float ex[BL_M][BL_NT + 1];  // SiLU(gate) * up: gate rows and up rows of a tile meet here
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* ring = smem;
  unsigned char* x_s = smem + BL_STAGES * BL_STAGE_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.S, nper = (int)gridDim.x / S;
  const int s = (int)blockIdx.x % S, g = (int)blockIdx.x / S;
  const int c0 = (int)((long long)s * a.chunks / S), c1 = (int)((long long)(s + 1) * a.chunks / S);
  const int nch = c1 - c0;
  const int n_units = g < a.R ? (a.R - g + nper - 1) / nper : 0;
  const bool swiglu = a.epi == EPI_SWIGLU;

  if (tid == 0) {
    sh.fail = 0;
    sh.issued = 0;
    for (int i = 0; i < BL_STAGES; ++i) {
      mbar_init(&sh.full[i], 1);
      mbar_init(&sh.empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.acc_full[i], 1);
      mbar_init(&sh.acc_empty[i], 128);
    }
    mbar_init(&sh.x_full, 128);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(&sh.tmem_base, 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_trigger();
  const unsigned tmem = sh.tmem_base;

  if (warp == 4) {
    // ---- TMA producer: the weights do not depend on the kernel before, so this starts at once -----------------
    if (lane == 0) {
      int it = 0;
      for (int u = 0; u < n_units && !sh.fail; ++u) {
        const int rb = g + u * nper;
        for (int c = 0; c < nch; ++c, ++it) {
          const int st = it % BL_STAGES;
          if (!mbar_wait(&sh.empty[st], ((it / BL_STAGES) & 1) ^ 1, &sh.fail)) {
            if (!sh.fail && a.status) atomicExch(a.status, 7);
            sh.fail = 1;
            break;
          }
          unsigned char* dst = ring + (size_t)st * BL_STAGE_BYTES;
          mbar_expect_tx(&sh.full[st], BL_STAGE_BYTES);
          const int col = (c0 + c) * BL_KC;
          if (swiglu) {  // 64 gate rows and the 64 up rows that belong to them
            tma_load_2d(dst, &tm_w, col, rb * 64, &sh.full[st]);
            tma_load_2d(dst + 64 * 128, &tm_w, col, a.inter + rb * 64, &sh.full[st]);
          } else {
            tma_load_2d(dst, &tm_w, col, rb * BL_M, &sh.full[st]);
          }
          sh.issued = it + 1;
        }
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer -------------------------------------------------------------------------------------------
    if (lane == 0) {
      const unsigned idesc = tc_instr_desc<T>(BL_M, BL_NT, false, false);
      const unsigned x_base = smem_u32(x_s);
      bool ok = mbar_wait(&sh.x_full, 0, &sh.fail);
      int it = 0;
      for (int u = 0; ok && u < n_units; ++u) {
        const int buf = u & 1;
        if (!mbar_wait(&sh.acc_empty[buf], ((u >> 1) & 1) ^ 1, &sh.fail)) { ok = false; break; }
        const unsigned d_tmem = tmem + (unsigned)buf * BL_NT;
        for (int c = 0; c < nch; ++c, ++it) {
          const int st = it % BL_STAGES;
          if (!mbar_wait(&sh.full[st], (it / BL_STAGES) & 1, &sh.fail)) { ok = false; break; }
          tc_fence_after();
          const unsigned w_base = smem_u32(ring + (size_t)st * BL_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma(d_tmem, smem_desc_sw128(w_base + k * 32), smem_desc_sw128(x_base + c * BL_XBOX_BYTES + k * 32), idesc,
                   (c | k) ? 1u : 0u);
          tc_commit(&sh.empty[st]);
        }
        if (ok) tc_commit(&sh.acc_full[buf]);
      }
      if (!ok) {
        if (!sh.fail && a.status) atomicExch(a.status, 7);
        sh.fail = 1;
      }
    }
  } else {
    // ---- staging, then epilogue: thread = output row of the tile ----------------------------------------------
    pdl_wait();  // the activations (and the workspace) belong to the kernel before until it has completed
    const float ss8 = stage_x<T>(x_s, a, c0, nch, tid);
    if ((tid & 7) == 0) {
      sh.ss_own[tid >> 3] = ss8;
      if (S > 1 && a.norm_w) a.ss[s * BL_NT + (tid >> 3)] = ss8;  // every CTA of the slice writes the same value
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the tensor core reads x through the async proxy
    mbar_arrive(&sh.x_full);
    const T* resid = static_cast<const T*>(a.resid);
    bool rstd_ready = false;
    for (int u = 0; u < n_units; ++u) {
      const int rb = g + u * nper, buf = u & 1;
      const bool got = mbar_wait(&sh.acc_full[buf], (u >> 1) & 1, &sh.fail);
      if (bl_vote_or(!got)) {  // the 128 threads leave together
        if (!sh.fail && a.status) atomicExch(a.status, 7);
        sh.fail = 1;
        break;
      }
      tc_fence_after();
      float y[BL_NT];
      tmem_ld16(tmem + ((unsigned)(warp * 32) << 16) + (unsigned)buf * BL_NT, y);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&sh.acc_empty[buf]);
      bool mine = true;  // this CTA runs the epilogue of the row block
      if (S > 1) {
        float* p = a.part + ((size_t)rb * S + s) * a.Bt * BL_M + tid;
#pragma unroll
        for (int b = 0; b < BL_NT; ++b)
          if (b < a.Bt) __stcg(p + b * BL_M, y[b]);
        __threadfence();
        bl_bar();
        if (tid == 0) {
          const int old = atomicAdd(&a.counters[rb], 1);
          sh.last = (old == S - 1);
          if (old == S - 1) a.counters[rb] = 0;  // nobody else touches it any more in this call
        }
        bl_bar();
        mine = sh.last != 0;
        if (mine) {
          __threadfence();
#pragma unroll
          for (int b = 0; b < BL_NT; ++b) y[b] = 0.f;
          // slice order: the same sum whichever CTA arrives last.  Four slices' loads go out together.
          for (int sl0 = 0; sl0 < S; sl0 += 4) {
            float t[4][BL_NT];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float* q = a.part + ((size_t)rb * S + min(sl0 + u, S - 1)) * a.Bt * BL_M + tid;
#pragma unroll
              for (int b = 0; b < BL_NT; ++b) t[u][b] = (b < a.Bt) ? __ldcg(q + b * BL_M) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (sl0 + u < S) {
#pragma unroll
                for (int b = 0; b < BL_NT; ++b) y[b] += t[u][b];
              }
          }
        }
      }
      if (mine) {
        if (a.norm_w) {
          if (!rstd_ready) {  // once per CTA: every slice's sum of squares is visible to a row block's last arriver
            for (int i = tid; i < S * BL_NT; i += 128) ss_all[i] = (S > 1) ? __ldcg(a.ss + i) : sh.ss_own[i];
            bl_bar();
            if (tid < BL_NT) {
              float tot = 0.f;
              for (int sl = 0; sl < S; ++sl) tot += ss_all[sl * BL_NT + tid];
              sh.rstd[tid] = rsqrtf(tot / (float)a.K + a.eps);
            }
            bl_bar();
            rstd_ready = true;
          }
#pragma unroll
          for (int b = 0; b < BL_NT; ++b) y[b] *= sh.rstd[b];
        }
        if (swiglu) {
#pragma unroll
          for (int b = 0; b < BL_NT; ++b) ex[tid][b] = y[b];
          bl_bar();
          const int j = tid & 63, b0 = (tid >> 6) * 8;  // rows 0-63 write tokens 0-7, rows 64-127 tokens 8-15
          const int n = rb * 64 + j;
          if (n < a.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int b = b0 + i;
              if (b < a.Bt) {
                const float gt = ex[j][b], up = ex[64 + j][b];
                static_cast<T*>(a.out)[(size_t)b * a.ldo + n] = from_float<T>(gt / (1.f + __expf(-gt)) * up);
              }
            }
          }
        } else {
          const int n = rb * BL_M + tid;
          if (n < a.N) {
#pragma unroll
            for (int b = 0; b < BL_NT; ++b) {
              if (b >= a.Bt) continue;
              if (a.epi == EPI_STORE_F32) {
                static_cast<float*>(a.out)[(size_t)b * a.ldo + n] = y[b];
              } else {
                float v = y[b];
                if (a.epi == EPI_RESIDUAL) v += to_float<T>(resid[(size_t)b * a.ldr + n]);
                static_cast<T*>(a.out)[(size_t)b * a.ldo + n] = from_float<T>(v);
              }
            }
          }
        }
      }
      bl_bar();  // ex and last are reused by the next unit
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (sh.fail) {
    if (tid == 128) {  // wait (bounded) for the last requested tile of every stage before the memory is given up
      for (int st = 0; st < BL_STAGES; ++st) {
        const int last = sh.issued - 1 - ((sh.issued - 1 - st) % BL_STAGES + BL_STAGES) % BL_STAGES;
        if (sh.issued > st && last >= 0) mbar_wait(&sh.full[st], (last / BL_STAGES) & 1);
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 32);
  }
}

// Slices of K: the count that minimises (row-block rounds) x (chunks per slice) with at most BL_MAX_CHUNKS chunks.
struct BlPlan {
  int S, R, chunks, grid;
};
BlPlan plan(int rows_out, int K, bool swiglu, int n_sms) {
  BlPlan p;
  p.chunks = ceil_div(K, BL_KC);
  p.R = swiglu ? ceil_div(rows_out, 64) : ceil_div(rows_out, BL_M);
  long long best = -1;
  p.S = 1;
  for (int S = 1; S <= BL_MAX_SLICES && S <= p.chunks && S <= n_sms; ++S) {
    const int per = ceil_div(p.chunks, S);
    if (per > BL_MAX_CHUNKS) continue;
    const int nper = n_sms / S;
    // time ~ weight tiles streamed by the busiest CTA, plus the cost of merging S partials per row block
    const long long cost = (long long)ceil_div(p.R, nper) * (per * 8 + (S > 1 ? S + 4 : 0));
    if (best < 0 || cost < best) {
      best = cost;
      p.S = S;
    }
  }
  p.grid = (n_sms / p.S) * p.S;
  if (best < 0) p.S = 0;
  return p;
}

int device_sms(int* n_sms) {
  static int cached = 0;
  if (!cached) {
    int dev = 0, n = 0;
    OMNIKV_CUDA_OK(cudaGetDevice(&dev));
    OMNIKV_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    cached = n;
  }
  *n_sms = cached;
  return OMNIKV_OK;
}

template <typename T>
int launch_bl(const omnikv_batched_linear_params* p, const BlPlan& pl, cudaStream_t st) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  const bool swiglu = p->epilogue == EPI_SWIGLU;
  CUtensorMap tm;
  if (!make_matrix_tensor_map(&tm, bf16, p->w, p->w_rows, p->K, p->w_stride_row, swiglu ? 64 : BL_M))
    return OMNIKV_E_UNSUPPORTED;
  BlArgs a;
  a.x = p->x;
  a.ldx = p->x_stride_tok;
  a.norm_w = p->norm_w;
  a.eps = p->eps;
  a.out = p->out;
  a.ldo = p->out_stride_tok;
  a.resid = p->residual;
  a.ldr = p->residual_stride_tok;
  unsigned char* ws = static_cast<unsigned char*>(p->workspace);
  a.counters = reinterpret_cast<int*>(ws);
  a.ss = reinterpret_cast<float*>(ws + BL_COUNTER_BYTES);
  a.part = reinterpret_cast<float*>(ws + BL_COUNTER_BYTES + BL_SS_BYTES);
  a.Bt = p->n_tokens;
  a.N = swiglu ? p->w_rows / 2 : p->w_rows;
  a.K = p->K;
  a.S = pl.S;
  a.R = pl.R;
  a.chunks = pl.chunks;
  a.epi = p->epilogue;
  a.inter = p->w_rows / 2;
  a.status = p->status;
  auto kern = batched_linear_kernel<T>;
  static bool attr_set[2] = {false, false};
  if (!attr_set[bf16 ? 1 : 0]) {
    OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BL_SMEM_BYTES));
    attr_set[bf16 ? 1 : 0] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(BL_THREADS);
  cfg.dynamicSmemBytes = BL_SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  OMNIKV_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, a, tm));
  return OMNIKV_OK;
}

size_t bl_workspace_bytes(const BlPlan& pl, int n_tokens) {
  return BL_COUNTER_BYTES + BL_SS_BYTES + (pl.S > 1 ? (size_t)pl.R * pl.S * n_tokens * BL_M * sizeof(float) : 0);
}

}  // namespace
}  // namespace omnikv

extern "C" size_t omnikv_batched_linear_workspace_bytes(int n_tokens, int w_rows, int K, int epilogue) {
  using namespace omnikv;
  int n_sms = 0;
  if (device_sms(&n_sms) != OMNIKV_OK || n_tokens <= 0 || w_rows <= 0 || K <= 0) return 0;
  const bool swiglu = epilogue == EPI_SWIGLU;
  const BlPlan pl = plan(swiglu ? w_rows / 2 : w_rows, K, swiglu, n_sms);
  return bl_workspace_bytes(pl, n_tokens);
}

extern "C" int omnikv_batched_linear(const omnikv_batched_linear_params* p, void* stream) {
  using namespace omnikv;
  if (!p || !p->w || !p->x || !p->out || !p->workspace) return OMNIKV_E_BADARG;
  if (p->dtype != OMNIKV_BF16 && p->dtype != OMNIKV_F16) return OMNIKV_E_UNSUPPORTED;
  if (p->n_tokens <= 0 || p->n_tokens > BL_NT || p->w_rows <= 0 || p->K <= 0 || p->K % 8) return OMNIKV_E_UNSUPPORTED;
  if (p->epilogue < EPI_STORE || p->epilogue > EPI_SWIGLU) return OMNIKV_E_BADARG;
  if (p->epilogue == EPI_RESIDUAL && !p->residual) return OMNIKV_E_BADARG;
  if (p->epilogue == EPI_SWIGLU && (p->w_rows % 128)) return OMNIKV_E_UNSUPPORTED;  // gate and up halves in blocks of 64
  if (p->x_stride_tok % 8 || (reinterpret_cast<uintptr_t>(p->x) & 15) ||
      (p->norm_w && (reinterpret_cast<uintptr_t>(p->norm_w) & 15)))
    return OMNIKV_E_BADARG;
  int n_sms = 0;
  int rc = device_sms(&n_sms);
  if (rc != OMNIKV_OK) return rc;
  const bool swiglu = p->epilogue == EPI_SWIGLU;
  const BlPlan pl = plan(swiglu ? p->w_rows / 2 : p->w_rows, p->K, swiglu, n_sms);
  if (pl.S == 0 || pl.R > BL_MAX_ROW_BLOCKS) return OMNIKV_E_UNSUPPORTED;
  if (p->workspace_bytes < bl_workspace_bytes(pl, p->n_tokens)) return OMNIKV_E_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return p->dtype == OMNIKV_BF16 ? launch_bl<__nv_bfloat16>(p, pl, st) : launch_bl<__half>(p, pl, st);
}
