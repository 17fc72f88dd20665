// ABI bookkeeping, the KV append, the offload gather and the window-plane fold.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace omnikv {

namespace {
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
PFN_encodeTiled encode_tiled_fn() {
  static PFN_encodeTiled fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_encodeTiled>(p);
  }();
  return fn;
}

}  // namespace

// 4-D map [B, KVH, rows, d] of 16-bit elements over a K or V cache given by element strides; box 64 x box_rows rows,
// 128-byte swizzle.  False when the layout cannot be described (the caller then uses the cp.async variant).
bool make_kv_tensor_map(CUtensorMap* map, bool is_bf16, const void* base, int64_t rows, int KVH, int B, int64_t sr,
                        int64_t sh, int64_t sb, int box_rows) {
  PFN_encodeTiled enc = encode_tiled_fn();
  if (!enc || rows <= 0 || rows > 0x7fffffffll) return false;
  // a dimension of extent 1 still needs a legal stride
  if (KVH == 1 && (sh <= 0 || sh % 8)) sh = sr * rows;
  if (B == 1 && (sb <= 0 || sb % 8)) sb = sh * KVH;
  if (sr % 8 || sh % 8 || sb % 8 || sr <= 0 || sh <= 0 || sb <= 0) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)kHeadDim, (cuuint64_t)rows, (cuuint64_t)KVH, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)sr * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};  // bytes, dims 1..3
  const cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


bool make_matrix_tensor_map(CUtensorMap* map, bool is_bf16, const void* base, int64_t rows, int64_t cols, int64_t ld,
                            int box_rows) {
  PFN_encodeTiled enc = encode_tiled_fn();
  if (!enc || rows <= 0 || cols <= 0 || ld % 8 || ld < cols || (reinterpret_cast<uintptr_t>(base) & 15)) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return enc(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static thread_local char g_last_error[256] = "";

int record_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
  (void)cudaGetLastError();  // clear the sticky-less error state
  return OMNIKV_E_CUDA;
}

#ifdef OMNIKV_TRACE
static int g_trace_slot = 0;
int trace_next_slot() { return g_trace_slot++ % kTraceSlots; }
#endif

bool pdl_enabled() {
  static const int on = [] {
    const char* e = getenv("OMNIKV_PDL");
    return (e && e[0] == '0') ? 0 : 1;
  }();
  return on != 0;
}

namespace {

// k_new/v_new [B, KVH, d] -> row pos[b] of the caches.  One 16-byte vector per thread.
template <int ESZ>
__global__ void kv_append_kernel(const unsigned char* k_new, const unsigned char* v_new, unsigned char* k_cache,
                                 unsigned char* v_cache, int KVH, int64_t new_sb, int64_t new_sh, int64_t c_sb,
                                 int64_t c_sh, int64_t c_sr, const int* pos) {
  constexpr int VECS = kHeadDim * ESZ / 16;  // 16-byte vectors per row
  const int b = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= KVH * VECS) return;
  const int h = i / VECS, c = i % VECS;
  const int64_t p = pos[b];
  if (p < 0) return;
  const size_t src = ((size_t)b * new_sb + (size_t)h * new_sh) * ESZ + (size_t)c * 16;
  const size_t dst = ((size_t)b * c_sb + (size_t)h * c_sh + (size_t)p * c_sr) * ESZ + (size_t)c * 16;
  *reinterpret_cast<uint4*>(k_cache + dst) = *reinterpret_cast<const uint4*>(k_new + src);
  *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v_new + src);
}

// The current token of every sequence, straight from the fused QKV projection: one thread per rotary pair
// (i, i + 64) of a head.  q and k are rotated by angle rope_pos[b] * inv_freq[i] (computed in fp32, rounded
// once); q goes to q_out, k and v to row cache_pos[b] of the layer's cache.
template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const T* __restrict__ qkv, int64_t qkv_sb, int H, int KVH,
                                                          const float* __restrict__ inv_freq,
                                                          const int* __restrict__ rope_pos, T* __restrict__ q_out,
                                                          int64_t q_sb, T* k_cache, T* v_cache, int64_t c_sb,
                                                          int64_t c_sh, int64_t c_sr, const int* __restrict__ cache_pos) {
  // the attention kernel that follows may be scheduled at once: before its own wait for this grid it only reads
  // lengths, index lists and cache rows OTHER than the ones written here
  pdl_trigger();
  const int b = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int heads = H + 2 * KVH;
  if (t >= heads * 64) return;
  const int hh = t >> 6, i = t & 63;
  const T* src = qkv + (size_t)b * qkv_sb + (size_t)hh * kHeadDim;
  float x0 = to_float(src[i]), x1 = to_float(src[i + 64]);
  if (hh < H + KVH) {
    float sn, cs;
    sincosf((float)rope_pos[b] * inv_freq[i], &sn, &cs);
    const float r0 = x0 * cs - x1 * sn, r1 = x1 * cs + x0 * sn;
    x0 = r0;
    x1 = r1;
  }
  T* dst;
  if (hh < H) {
    dst = q_out + (size_t)b * q_sb + (size_t)hh * kHeadDim;
  } else {
    const int64_t p = cache_pos[b];
    if (p < 0) return;
    const bool is_k = hh < H + KVH;
    const int kvh = is_k ? hh - H : hh - H - KVH;
    dst = (is_k ? k_cache : v_cache) + (size_t)b * c_sb + (size_t)kvh * c_sh + (size_t)p * c_sr;
  }
  dst[i] = from_float<T>(x0);
  dst[i + 64] = from_float<T>(x1);
}

// The observation window's queries straight from the q projection: qlin[b][w] = H heads x head_dim, every one rotated
// at the CURRENT position of its sequence (as the reference's window selectors do, modeling/omnikv.py:52-57, :66-71),
// written as [B, H, W, head_dim] for omnikv_score_window.  fp32 arithmetic, rounded once.
template <typename T>
__global__ void __launch_bounds__(256) rope_window_kernel(const T* __restrict__ qlin, int64_t sb, int64_t sw, int H, int W,
                                                          const float* __restrict__ inv_freq,
                                                          const int* __restrict__ rope_pos, T* __restrict__ out) {
  const int b = blockIdx.z, w = blockIdx.y;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= H * 64) return;
  const int hh = t >> 6, i = t & 63;
  const T* src = qlin + (size_t)b * sb + (size_t)w * sw + (size_t)hh * kHeadDim;
  const float x0 = to_float(src[i]), x1 = to_float(src[i + 64]);
  float sn, cs;
  sincosf((float)rope_pos[b] * inv_freq[i], &sn, &cs);
  T* dst = out + (((size_t)b * H + hh) * W + w) * kHeadDim;
  dst[i] = from_float<T>(x0 * cs - x1 * sn);
  dst[i + 64] = from_float<T>(x1 * cs + x0 * sn);
}

// act[b][j] = silu(gu[b][j]) * gu[b][inter + j]: the SwiGLU product of a fused gate/up projection.
template <typename T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gu, int64_t gu_sb, T* __restrict__ act,
                                                       int64_t act_sb, int inter) {
  const int b = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= inter) return;
  const float g = to_float(gu[(size_t)b * gu_sb + j]), u = to_float(gu[(size_t)b * gu_sb + inter + j]);
  act[(size_t)b * act_sb + j] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// h[b] += delta[b] (when delta is given; rounded to T, as the residual stream is stored), out[b] = RMSNorm(h[b]) * w.
// One CTA per token, 256 threads; a thread visits the same elements in both passes.
template <typename T>
__global__ void __launch_bounds__(256) add_rms_norm_kernel(T* __restrict__ h, int64_t h_st, const T* __restrict__ delta,
                                                           int64_t d_st, const T* __restrict__ w, float eps,
                                                           T* __restrict__ out, int64_t o_st, int hidden) {
  __shared__ float red[8];
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x;
  T* hr = h + (size_t)b * h_st;
  const T* dr = delta ? delta + (size_t)b * d_st : nullptr;
  float ss = 0.f;
  for (int i = tid; i < hidden; i += 256) {
    float v = to_float(hr[i]);
    if (dr) {
      v = to_float(from_float<T>(v + to_float(dr[i])));
      hr[i] = from_float<T>(v);
    }
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)hidden + eps);
  for (int i = tid; i < hidden; i += 256) {  // the thread re-reads what it read or wrote above (L1 / L2 hits)
    const float v = to_float(hr[i]);
    out[(size_t)b * o_st + i] = from_float<T>(v * rstd * to_float(w[i]));
  }
}

// The same with 16-byte vectors, every load of a thread issued before its first store (hidden a multiple of the
// vector width and at most 1024 vectors per token: 8192 elements in 16 bits).
template <typename T>
__global__ void __launch_bounds__(256) add_rms_norm_vec_kernel(T* __restrict__ h, int64_t h_st, const T* __restrict__ delta,
                                                               int64_t d_st, const T* __restrict__ w, float eps,
                                                               T* __restrict__ out, int64_t o_st, int hidden) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[8];
  const int b = blockIdx.x, tid = threadIdx.x, nvec = hidden / V;
  uint4 wv[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {  // the norm weight does not depend on the kernel before
    const int i = tid + u * 256;
    wv[u] = i < nvec ? reinterpret_cast<const uint4*>(w)[i] : make_uint4(0, 0, 0, 0);
  }
  pdl_wait();
  uint4* h4 = reinterpret_cast<uint4*>(h + (size_t)b * h_st);
  const uint4* d4 = delta ? reinterpret_cast<const uint4*>(delta + (size_t)b * d_st) : nullptr;
  uint4 hv[4], dv[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = tid + u * 256;
    hv[u] = make_uint4(0, 0, 0, 0);
    dv[u] = hv[u];
    if (i < nvec) {
      hv[u] = h4[i];
      if (d4) dv[u] = d4[i];
    }
  }
  float x[4][V];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const T* he = reinterpret_cast<const T*>(&hv[u]);
    const T* de = reinterpret_cast<const T*>(&dv[u]);
    T* oe = reinterpret_cast<T*>(&hv[u]);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      float v = to_float(he[e]);
      if (d4) {
        oe[e] = from_float<T>(v + to_float(de[e]));
        v = to_float(oe[e]);
      }
      x[u][e] = v;
      ss = fmaf(v, v, ss);
    }
    const int i = tid + u * 256;
    if (d4 && i < nvec) h4[i] = hv[u];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)hidden + eps);
  uint4* o4 = reinterpret_cast<uint4*>(out + (size_t)b * o_st);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int i = tid + u * 256;
    if (i >= nvec) continue;
    uint4 ov;
    T* oe = reinterpret_cast<T*>(&ov);
    const T* we = reinterpret_cast<const T*>(&wv[u]);
#pragma unroll
    for (int e = 0; e < V; ++e) oe[e] = from_float<T>(x[u][e] * rstd * to_float(we[e]));
    o4[i] = ov;
  }
}

// Host-link gather.  One selected token is one contiguous chunk of n_layers*2*KVH rows in pinned
// host memory; row r of the chunk (layer l, K|V c, head h) goes to staged[l][c][h][j][:].
// A warp copies rows with one 16-byte load per lane per step, several rows in flight.
__global__ void __launch_bounds__(256) offload_gather_kernel(const unsigned char* __restrict__ host_kv,
                                                             int64_t token_stride, int rows_per_token,
                                                             int row_bytes, const int* __restrict__ idx,
                                                             const int* __restrict__ n_idx, int cap,
                                                             unsigned char* __restrict__ staged) {
  const int n = min(*n_idx, cap);
  const int vec_per_row = row_bytes / 16;
  const long long total = (long long)n * rows_per_token * vec_per_row;
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;
  for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < total; v0 += stride * U) {
    uint4 buf[U];
    long long dst[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + u * stride;
      dst[u] = -1;
      if (v < total) {
        const int c = (int)(v % vec_per_row);
        const long long rr = v / vec_per_row;
        const int r = (int)(rr % rows_per_token);
        const int j = (int)(rr / rows_per_token);
        const unsigned char* src = host_kv + (size_t)idx[j] * token_stride + (size_t)r * row_bytes + (size_t)c * 16;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(buf[u].x), "=r"(buf[u].y), "=r"(buf[u].z), "=r"(buf[u].w)
                     : "l"(src));
        dst[u] = ((long long)r * cap + j) * row_bytes + (long long)c * 16;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (dst[u] >= 0) *reinterpret_cast<uint4*>(staged + dst[u]) = buf[u];
  }
}

// Lazy re-gather rule, one CTA per sequence.  Both lists are ascending and free of duplicates, so the
// intersection is counted by a binary search of every new entry in the list in use.
__global__ void __launch_bounds__(1024) idx_commit_kernel(const int* __restrict__ new_idx, int64_t new_stride,
                                                          const int* __restrict__ new_count, int* live_idx,
                                                          int64_t live_stride, int* live_count, int capacity,
                                                          double skip_threshold, int* applied, int* gather_n,
                                                          int* overlap) {
  __shared__ int s_inter;
  const int b = blockIdx.x, tid = threadIdx.x;
  const int n = min(new_count[b], capacity), m = min(live_count[b], capacity);
  const int* nw = new_idx + (size_t)b * new_stride;
  int* lv = live_idx + (size_t)b * live_stride;
  if (tid == 0) s_inter = 0;
  __syncthreads();
  int c = 0;
  if (m > 0) {
    for (int j = tid; j < n; j += blockDim.x) {
      const int v = nw[j];
      int lo = 0, hi = m;  // first position with lv[pos] >= v
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (lv[mid] < v) lo = mid + 1; else hi = mid;
      }
      c += (lo < m && lv[lo] == v) ? 1 : 0;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
  if ((tid & 31) == 0 && c) atomicAdd(&s_inter, c);
  __syncthreads();  // also: every read of the list in use is done before it is overwritten
  const int inter = s_inter;
  const bool take = m == 0 || n == 0 || !((double)inter / (double)n > skip_threshold);
  if (take)
    for (int j = tid; j < n; j += blockDim.x) lv[j] = nw[j];
  if (tid == 0) {
    if (take) live_count[b] = n;
    applied[b] = take ? 1 : 0;
    if (gather_n) gather_n[b] = take ? n : 0;
    if (overlap) overlap[b] = inter;
  }
}

__global__ void window_fold_kernel(const float* __restrict__ planes, float* __restrict__ score_out, int W,
                                   int64_t score_stride, const int* __restrict__ consider_len, int selector) {
  const int b = blockIdx.y;
  const int n = consider_len[b];
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < n; p += gridDim.x * blockDim.x) {
    const float* pl = planes + (size_t)b * W * score_stride + p;
    float acc = 0.f;
    if (selector == OMNIKV_SEL_SOFTMAX_LAST) {
      acc = pl[(size_t)(W - 1) * score_stride];
    } else {
      for (int w = 0; w < W; ++w) {
        const float v = pl[(size_t)w * score_stride];
        acc = (selector == OMNIKV_SEL_EXP) ? fmaf(acc, 0.5f, v) : acc + v;
      }
    }
    score_out[(size_t)b * score_stride + p] = acc;
  }
}

}  // namespace
}  // namespace omnikv

extern "C" int omnikv_abi_version(void) { return OMNIKV_ABI_VERSION; }

extern "C" const char* omnikv_strerror(int status) {
  switch (status) {
    case OMNIKV_OK: return "ok";
    case OMNIKV_E_BADARG: return "bad argument (null pointer, non-positive size, stride or alignment)";
    case OMNIKV_E_UNSUPPORTED: return "unsupported shape or dtype";
    case OMNIKV_E_WORKSPACE: return "workspace missing or too small";
    case OMNIKV_E_CUDA: return "CUDA runtime error (see omnikv_last_cuda_error)";
    default: return "unknown status";
  }
}

extern "C" const char* omnikv_last_cuda_error(void) { return omnikv::g_last_error; }

extern "C" int omnikv_kv_append(int dtype, const void* k_new, const void* v_new, void* k_cache, void* v_cache, int B,
                                int KVH, int head_dim, int64_t new_stride_b, int64_t new_stride_h,
                                int64_t cache_stride_b, int64_t cache_stride_h, int64_t cache_stride_row,
                                const int32_t* pos, void* stream) {
  using namespace omnikv;
  if (!k_new || !v_new || !k_cache || !v_cache || !pos || B <= 0 || KVH <= 0) return OMNIKV_E_BADARG;
  if (head_dim != kHeadDim) return OMNIKV_E_UNSUPPORTED;
  const int esz = dtype == OMNIKV_F32 ? 4 : 2;
  const int vec = 16 / esz;
  if (new_stride_b % vec || new_stride_h % vec || cache_stride_b % vec || cache_stride_h % vec || cache_stride_row % vec)
    return OMNIKV_E_BADARG;
  const int threads = 128;
  const int work = KVH * kHeadDim * esz / 16;
  dim3 grid((work + threads - 1) / threads, B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto kn = static_cast<const unsigned char*>(k_new);
  auto vn = static_cast<const unsigned char*>(v_new);
  auto kc = static_cast<unsigned char*>(k_cache);
  auto vc = static_cast<unsigned char*>(v_cache);
  if (esz == 4)
    kv_append_kernel<4><<<grid, threads, 0, st>>>(kn, vn, kc, vc, KVH, new_stride_b, new_stride_h, cache_stride_b,
                                                  cache_stride_h, cache_stride_row, pos);
  else
    kv_append_kernel<2><<<grid, threads, 0, st>>>(kn, vn, kc, vc, KVH, new_stride_b, new_stride_h, cache_stride_b,
                                                  cache_stride_h, cache_stride_row, pos);
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

extern "C" int omnikv_rope_append(int dtype, const void* qkv, int64_t qkv_stride_b, int B, int H, int KVH,
                                  int head_dim, const float* inv_freq, const int32_t* rope_pos, void* q_out,
                                  int64_t q_stride_b, void* k_cache, void* v_cache, int64_t cache_stride_b,
                                  int64_t cache_stride_h, int64_t cache_stride_row, const int32_t* cache_pos,
                                  void* stream) {
  using namespace omnikv;
  if (!qkv || !inv_freq || !rope_pos || !q_out || !k_cache || !v_cache || !cache_pos || B <= 0 || H <= 0 || KVH <= 0)
    return OMNIKV_E_BADARG;
  if (head_dim != kHeadDim) return OMNIKV_E_UNSUPPORTED;
  dim3 grid(ceil_div((H + 2 * KVH) * 64, 256), B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define OMNIKV_ROPE_LAUNCH(T)                                                                                    \
  rope_append_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(qkv), qkv_stride_b, H, KVH, inv_freq, rope_pos, \
                                              static_cast<T*>(q_out), q_stride_b, static_cast<T*>(k_cache),         \
                                              static_cast<T*>(v_cache), cache_stride_b, cache_stride_h,             \
                                              cache_stride_row, cache_pos)
  switch (dtype) {
    case OMNIKV_BF16: OMNIKV_ROPE_LAUNCH(__nv_bfloat16); break;
    case OMNIKV_F16: OMNIKV_ROPE_LAUNCH(__half); break;
    case OMNIKV_F32: OMNIKV_ROPE_LAUNCH(float); break;
    default: return OMNIKV_E_UNSUPPORTED;
  }
#undef OMNIKV_ROPE_LAUNCH
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

extern "C" int omnikv_rope_window(int dtype, const void* qlin, int64_t stride_b, int64_t stride_w, int B, int W, int H,
                                  int head_dim, const float* inv_freq, const int32_t* rope_pos, void* out, void* stream) {
  using namespace omnikv;
  if (!qlin || !inv_freq || !rope_pos || !out || B <= 0 || W <= 0 || H <= 0 || B > 65535 || W > 65535) return OMNIKV_E_BADARG;
  if (head_dim != kHeadDim) return OMNIKV_E_UNSUPPORTED;
  dim3 grid(ceil_div(H * 64, 256), W, B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case OMNIKV_BF16:
      rope_window_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(qlin), stride_b, stride_w, H,
                                                              W, inv_freq, rope_pos, static_cast<__nv_bfloat16*>(out));
      break;
    case OMNIKV_F16:
      rope_window_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(qlin), stride_b, stride_w, H, W, inv_freq,
                                                       rope_pos, static_cast<__half*>(out));
      break;
    case OMNIKV_F32:
      rope_window_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(qlin), stride_b, stride_w, H, W, inv_freq,
                                                      rope_pos, static_cast<float*>(out));
      break;
    default: return OMNIKV_E_UNSUPPORTED;
  }
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

extern "C" int omnikv_silu_mul(int dtype, const void* gate_up, int64_t gate_up_stride_b, void* act,
                               int64_t act_stride_b, int B, int inter, void* stream) {
  using namespace omnikv;
  if (!gate_up || !act || B <= 0 || inter <= 0) return OMNIKV_E_BADARG;
  dim3 grid(ceil_div(inter, 256), B);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case OMNIKV_BF16:
      silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gate_up), gate_up_stride_b,
                                                           static_cast<__nv_bfloat16*>(act), act_stride_b, inter);
      break;
    case OMNIKV_F16:
      silu_mul_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(gate_up), gate_up_stride_b,
                                                    static_cast<__half*>(act), act_stride_b, inter);
      break;
    case OMNIKV_F32:
      silu_mul_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(gate_up), gate_up_stride_b,
                                                   static_cast<float*>(act), act_stride_b, inter);
      break;
    default: return OMNIKV_E_UNSUPPORTED;
  }
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

extern "C" int omnikv_add_rms_norm(int dtype, void* h, int64_t h_stride_tok, const void* delta, int64_t delta_stride_tok,
                                   const void* norm_w, float eps, void* out, int64_t out_stride_tok, int n_tokens,
                                   int hidden, void* stream) {
  using namespace omnikv;
  if (!h || !norm_w || !out || n_tokens <= 0 || hidden <= 0) return OMNIKV_E_BADARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
#define OMNIKV_ARN_LAUNCH(T)                                                                                        \
  const int V = 16 / (int)sizeof(T);                                                                                \
  const bool vec = hidden % V == 0 && hidden / V <= 1024 && aligned(h) && aligned(delta) && aligned(norm_w) &&      \
                   aligned(out) && h_stride_tok % V == 0 && delta_stride_tok % V == 0 && out_stride_tok % V == 0;   \
  OMNIKV_CUDA_OK(launch_pdl_args(vec ? add_rms_norm_vec_kernel<T> : add_rms_norm_kernel<T>, dim3(n_tokens), dim3(256), st, static_cast<T*>(h), h_stride_tok, \
                                 static_cast<const T*>(delta), delta_stride_tok, static_cast<const T*>(norm_w), eps,  \
                                 static_cast<T*>(out), out_stride_tok, hidden))
  switch (dtype) {
    case OMNIKV_BF16: { OMNIKV_ARN_LAUNCH(__nv_bfloat16); break; }
    case OMNIKV_F16: { OMNIKV_ARN_LAUNCH(__half); break; }
    case OMNIKV_F32: { OMNIKV_ARN_LAUNCH(float); break; }
    default: return OMNIKV_E_UNSUPPORTED;
  }
#undef OMNIKV_ARN_LAUNCH
  return OMNIKV_OK;
}

extern "C" int omnikv_offload_gather(const void* host_kv, int64_t token_stride_bytes, int n_layers_in_group, int KVH,
                                     int head_dim, int elem_bytes, const int32_t* idx, const int32_t* n_idx,
                                     int n_idx_capacity, void* staged, int n_ctas, void* stream) {
  using namespace omnikv;
  if (!host_kv || !idx || !n_idx || !staged || n_layers_in_group <= 0 || KVH <= 0 || n_idx_capacity <= 0 || n_ctas <= 0)
    return OMNIKV_E_BADARG;
  if (head_dim != kHeadDim || (elem_bytes != 2 && elem_bytes != 4)) return OMNIKV_E_UNSUPPORTED;
  const int row_bytes = head_dim * elem_bytes;
  const int rows_per_token = n_layers_in_group * 2 * KVH;
  if (token_stride_bytes < (int64_t)rows_per_token * row_bytes || token_stride_bytes % 16) return OMNIKV_E_BADARG;
  offload_gather_kernel<<<n_ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(host_kv), token_stride_bytes, rows_per_token, row_bytes, idx, n_idx,
      n_idx_capacity, static_cast<unsigned char*>(staged));
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

extern "C" int omnikv_idx_commit(const int32_t* new_idx, int64_t new_stride, const int32_t* new_count,
                                 int32_t* live_idx, int64_t live_stride, int32_t* live_count, int B, int capacity,
                                 double skip_threshold, int32_t* applied, int32_t* gather_n, int32_t* overlap,
                                 void* stream) {
  using namespace omnikv;
  if (!new_idx || !new_count || !live_idx || !live_count || !applied || B <= 0 || capacity <= 0)
    return OMNIKV_E_BADARG;
  if (new_stride < capacity || live_stride < capacity || new_idx == live_idx) return OMNIKV_E_BADARG;
  idx_commit_kernel<<<B, 1024, 0, static_cast<cudaStream_t>(stream)>>>(new_idx, new_stride, new_count, live_idx,
                                                                       live_stride, live_count, capacity,
                                                                       skip_threshold, applied, gather_n, overlap);
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

extern "C" int omnikv_window_fold(const float* planes, float* score_out, int B, int W, int64_t score_stride,
                                  const int32_t* consider_len, int max_len, int selector, void* stream) {
  using namespace omnikv;
  if (!planes || !score_out || !consider_len || B <= 0 || W <= 0 || max_len <= 0 || score_stride < max_len)
    return OMNIKV_E_BADARG;
  if (selector < OMNIKV_SEL_SOFTMAX_LAST || selector > OMNIKV_SEL_EXP) return OMNIKV_E_BADARG;
  dim3 grid(min(1184, (max_len + 255) / 256), B);
  window_fold_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(planes, score_out, W, score_stride,
                                                                         consider_len, selector);
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}

#ifdef OMNIKV_TRACE
extern "C" void omnikv_debug_trace_reset(void) { omnikv::g_trace_slot = 0; }
#endif
