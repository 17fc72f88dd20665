// Causal prefill attention on the Blackwell tensor path (tcgen05.mma, accumulators in tensor memory).
//
//   out[b, i, h, :] = softmax over keys j <= q_pos0 + i of (q[b,h,i,:] . k[b,h/G,j,:] * scale) . v[b,h/G,j,:]
//
// the attention the decoder runs over the prompt before the first decode step (the reference calls flash-attn
// there through transformers' decoder layer, modeling/omnikv.py:219-227).  One CTA owns 128 consecutive queries
// of one head and walks the key tiles of 128 rows that the causal mask leaves:
//
//   S  = Q K^T     Q tile [128 x 128] = A operand, K tile [128 keys x 128] = B operand, both K-major as two TMA
//                  boxes with the 128-byte swizzle; fp32 accumulator [128 queries x 128 keys] in tensor memory:
//                  TMEM lane = query, so a softmax thread owns ONE query row and reads its logits with tcgen05.ld
//   P  = 2^(S c - m)  written by the softmax threads as 16-bit into shared memory with the same swizzle
//   PV = P V       P = A operand (K-major over keys), the V tile as it lies in memory ([keys x 128]: rows run
//                  along the contraction) = MN-major B operand; accumulator [128 queries x 128] in tensor memory
//   O  = O alpha + PV   in the softmax threads' registers (one query row: 2 x 64 fp32)
//
// Roles: eight softmax warps (two per TMEM lane quarter, so that each scheduler has two warps to overlap: both take
// the row maximum, each exponentiates half of the keys and accumulates half of the output columns), one thread issues
// the TMA copies, one the MMAs.  S and PV
// are double-buffered in tensor memory (4 x 128 columns), K and V tiles in two-stage rings, so the tensor pipe
// computes S of tile j+1 and PV of tile j-1 while the softmax threads work on tile j.
// Every wait is bounded by time; on expiry the CTA raises a flag, every role leaves its loop, copies in flight are
// waited for (bounded), the tensor memory is released and a status code is written.
#include "common.cuh"
#include "tc05.cuh"

namespace omnikv {
namespace {

constexpr int PF_TILE = 128;                  // queries per CTA = keys per tile = TMEM lanes
constexpr int PF_TILE_BYTES = PF_TILE * 256;  // [128 rows x 128] 16-bit: two boxes of 128 rows x 128 bytes
constexpr int PF_BOX_BYTES = PF_TILE * 128;
constexpr int PF_STAGES = 2;
constexpr int PF_THREADS = 320;  // warps 0-7 softmax (two per TMEM lane quarter), 8 TMA producer, 9 MMA issuer
constexpr unsigned PF_TMEM_COLS = 512;  // S0 | S1 | PV0 | PV1, 128 columns each
constexpr int PF_SMEM_BYTES = PF_TILE_BYTES * (1 + 2 * PF_STAGES + 1) + 1024;  // Q, K ring, V ring, P, alignment

struct PfArgs {
  void* out;
  int64_t o_sb, o_sn, o_sh;  // element strides of out[b, i, h, :]
  int H, G, Sq, Skv, q_pos0;
  float scale_log2;  // scale * log2(e)
  int* status;
};

struct PfShared {
  uint64_t q_full;
  uint64_t k_full[PF_STAGES], k_empty[PF_STAGES];
  uint64_t v_full[PF_STAGES], v_empty[PF_STAGES];
  uint64_t s_full[2], s_empty[2];
  uint64_t pv_full[2], pv_empty[2];
  uint64_t p_full, p_empty;
  unsigned tmem_base;
  int fail;
  int k_issued, v_issued, q_issued;
};

__device__ __forceinline__ void pf_fail(PfShared& sh, int* status) {
  if (!sh.fail && status) atomicExch(status, 6);
  sh.fail = 1;
}

template <typename T>
__device__ __forceinline__ unsigned pack2(float a, float b);
template <>
__device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}
template <>
__device__ __forceinline__ unsigned pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}

template <typename T>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_attn_kernel(const PfArgs a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ PfShared sh;
  __shared__ float l_s[2][PF_TILE];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;
  unsigned char* k_ring = q_s + PF_TILE_BYTES;
  unsigned char* v_ring = k_ring + PF_STAGES * PF_TILE_BYTES;
  unsigned char* p_s = v_ring + PF_STAGES * PF_TILE_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;  // the longest rows of the causal triangle start first
  const int h = blockIdx.y, b = blockIdx.z, kvh = h / a.G;
  const int q0 = qblk * PF_TILE;
  const int last_q = min(q0 + PF_TILE, a.Sq) - 1;
  const int n_tiles = (a.q_pos0 + last_q) / PF_TILE + 1;  // key tiles with at least one visible key

  if (tid == 0) {
    sh.fail = 0;
    sh.k_issued = sh.v_issued = sh.q_issued = 0;
    mbar_init(&sh.q_full, 1);
    for (int s = 0; s < PF_STAGES; ++s) {
      mbar_init(&sh.k_full[s], 1);
      mbar_init(&sh.k_empty[s], 1);
      mbar_init(&sh.v_full[s], 1);
      mbar_init(&sh.v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sh.s_full[i], 1);
      mbar_init(&sh.s_empty[i], 256);
      mbar_init(&sh.pv_full[i], 1);
      mbar_init(&sh.pv_empty[i], 256);
    }
    mbar_init(&sh.p_full, 256);
    mbar_init(&sh.p_empty, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(&sh.tmem_base, PF_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = sh.tmem_base;

  if (warp == 8) {
    // ---- TMA producer ------------------------------------------------------------------------------------
    if (tid == 256) {
      mbar_expect_tx(&sh.q_full, PF_TILE_BYTES);
      tma_load_4d(q_s, &tm_q, 0, q0, h, b, &sh.q_full);
      tma_load_4d(q_s + PF_BOX_BYTES, &tm_q, 64, q0, h, b, &sh.q_full);
      sh.q_issued = 1;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % PF_STAGES;
        const unsigned par = ((j / PF_STAGES) & 1) ^ 1;
        if (!mbar_wait(&sh.k_empty[s], par, &sh.fail)) { pf_fail(sh, a.status); break; }
        unsigned char* kd = k_ring + (size_t)s * PF_TILE_BYTES;
        mbar_expect_tx(&sh.k_full[s], PF_TILE_BYTES);
        tma_load_4d(kd, &tm_k, 0, j * PF_TILE, kvh, b, &sh.k_full[s]);
        tma_load_4d(kd + PF_BOX_BYTES, &tm_k, 64, j * PF_TILE, kvh, b, &sh.k_full[s]);
        sh.k_issued = j + 1;
        if (!mbar_wait(&sh.v_empty[s], par, &sh.fail)) { pf_fail(sh, a.status); break; }
        unsigned char* vd = v_ring + (size_t)s * PF_TILE_BYTES;
        mbar_expect_tx(&sh.v_full[s], PF_TILE_BYTES);
        tma_load_4d(vd, &tm_v, 0, j * PF_TILE, kvh, b, &sh.v_full[s]);
        tma_load_4d(vd + PF_BOX_BYTES, &tm_v, 64, j * PF_TILE, kvh, b, &sh.v_full[s]);
        sh.v_issued = j + 1;
      }
    }
  } else if (warp == 9) {
    // ---- MMA issuer ----------------------------------------------------------------------------------------
    if (tid == 288) {
      const unsigned idesc_s = tc_instr_desc<T>(PF_TILE, PF_TILE, false, false);
      const unsigned idesc_pv = tc_instr_desc<T>(PF_TILE, kHeadDim, false, true);
      const unsigned q_base = smem_u32(q_s), p_base = smem_u32(p_s);
      bool ok = mbar_wait(&sh.q_full, 0, &sh.fail);
      // PV of tile i: P (128 queries x 128 keys, K-major) x V tile (MN-major), 8 steps of 16 keys
      auto issue_pv = [&](int i) -> bool {
        const int s = i % PF_STAGES, buf = i & 1;
        if (!mbar_wait(&sh.p_full, i & 1, &sh.fail) || !mbar_wait(&sh.v_full[s], (i / PF_STAGES) & 1, &sh.fail) ||
            !mbar_wait(&sh.pv_empty[buf], ((i >> 1) & 1) ^ 1, &sh.fail))
          return false;
        tc_fence_after();
        const unsigned v_base = smem_u32(v_ring + (size_t)s * PF_TILE_BYTES);
        const unsigned d_tmem = tmem + 256u + (unsigned)buf * 128u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t a_desc = smem_desc_sw128(p_base + (k >> 2) * PF_BOX_BYTES + (k & 3) * 32);
          const uint64_t b_desc = smem_desc_sw128_mn(v_base + k * 2048, PF_BOX_BYTES, 1024);
          tc_mma(d_tmem, a_desc, b_desc, idesc_pv, k > 0 ? 1u : 0u);
        }
        tc_commit(&sh.v_empty[s]);
        tc_commit(&sh.p_empty);
        tc_commit(&sh.pv_full[buf]);
        return true;
      };
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int s = j % PF_STAGES, buf = j & 1;
        if (!mbar_wait(&sh.k_full[s], (j / PF_STAGES) & 1, &sh.fail) ||
            !mbar_wait(&sh.s_empty[buf], ((j >> 1) & 1) ^ 1, &sh.fail)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned k_base = smem_u32(k_ring + (size_t)s * PF_TILE_BYTES);
        const unsigned d_tmem = tmem + (unsigned)buf * 128u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 16 elements of head_dim per step: 4 per 128-byte box row, then the other box
          const uint64_t a_desc = smem_desc_sw128(q_base + (k >> 2) * PF_BOX_BYTES + (k & 3) * 32);
          const uint64_t b_desc = smem_desc_sw128(k_base + (k >> 2) * PF_BOX_BYTES + (k & 3) * 32);
          tc_mma(d_tmem, a_desc, b_desc, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&sh.k_empty[s]);
        tc_commit(&sh.s_full[buf]);
        if (j > 0) ok = issue_pv(j - 1);
      }
      if (ok) ok = issue_pv(n_tiles - 1);
      if (!ok) pf_fail(sh, a.status);
    }
  } else {
    // ---- softmax: two threads per query row (warps w and w + 4 share TMEM lane quarter w) -------------------
    // Each takes the row maximum over all 128 logits of the tile (cheap, and it spares an exchange), but
    // exponentiates and writes only ITS half of the key columns of P, and accumulates ITS half of the output columns.
    const int quarter = warp & 3, hf = warp >> 2;
    const int row = quarter * 32 + (tid & 31);  // TMEM lane
    const int pos = a.q_pos0 + q0 + row;        // last visible key of this query
    const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16);
    const float c = a.scale_log2;
    constexpr int HC = kHeadDim / 2;  // columns per thread: 64 keys of P, 64 dims of O
    float m = -INFINITY, l = 0.f, alpha_pending = 1.f;
    float o[HC];
#pragma unroll
    for (int i = 0; i < HC; ++i) o[i] = 0.f;
    bool ok = true;
    // O = O * alpha_pending + PV_i (this thread's 64 output columns)
    auto take_pv = [&](int i) -> bool {
      const int buf = i & 1;
      if (!mbar_wait(&sh.pv_full[buf], (i >> 1) & 1, &sh.fail)) return false;
      tc_fence_after();
      const unsigned t = lane_addr + 256u + (unsigned)buf * 128u + (unsigned)hf * HC;
#pragma unroll
      for (int cb = 0; cb < HC; cb += 32) {
        float v[32];
        tmem_ld16(t + cb, *reinterpret_cast<float(*)[16]>(&v[0]));
        tmem_ld16(t + cb + 16, *reinterpret_cast<float(*)[16]>(&v[16]));
        tmem_ld_wait();
#pragma unroll
        for (int i2 = 0; i2 < 32; ++i2) o[cb + i2] = fmaf(o[cb + i2], alpha_pending, v[i2]);
      }
      tc_fence_before();
      mbar_arrive(&sh.pv_empty[buf]);
      return true;
    };
    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      if (!mbar_wait(&sh.s_full[buf], (j >> 1) & 1, &sh.fail)) { ok = false; break; }
      tc_fence_after();
      const unsigned t = lane_addr + (unsigned)buf * 128u;
      const int key0 = j * PF_TILE;
      const bool masked = key0 + PF_TILE - 1 > a.q_pos0 + q0;  // some query of this CTA does not see the whole tile
      // pass A: the row's maximum over the whole tile (raw logits; the scale is positive)
      float mraw = -INFINITY;
#pragma unroll
      for (int cb = 0; cb < PF_TILE; cb += 32) {
        float v[32];
        tmem_ld16(t + cb, *reinterpret_cast<float(*)[16]>(&v[0]));
        tmem_ld16(t + cb + 16, *reinterpret_cast<float(*)[16]>(&v[16]));
        tmem_ld_wait();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + cb + i <= pos) mraw = fmaxf(mraw, v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mraw = fmaxf(mraw, v[i]);
        }
      }
      // key 0 is visible to every query, so the maximum is finite from the first tile on
      const float mx = fmaxf(m, mraw * c);
      const float alpha = ex2_fast(m - mx);
      m = mx;
      // the previous tile's PV product has read P: fold it into O before alpha_pending changes, then reuse P
      if (j > 0) {
        if (!mbar_wait(&sh.p_empty, (j - 1) & 1, &sh.fail)) { ok = false; break; }
        if (!take_pv(j - 1)) { ok = false; break; }
      }
      alpha_pending = alpha;
      // pass B: this thread's 64 keys: P = 2^(S c - m) as 16-bit into box `hf` of P, partial row sum
      float sum = 0.f;
#pragma unroll
      for (int cb = 0; cb < HC; cb += 32) {
        float v[32];
        tmem_ld16(t + hf * HC + cb, *reinterpret_cast<float(*)[16]>(&v[0]));
        tmem_ld16(t + hf * HC + cb + 16, *reinterpret_cast<float(*)[16]>(&v[16]));
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p = ex2_fast(fmaf(v[i], c, -mx));
          if (masked && key0 + hf * HC + cb + i > pos) p = 0.f;
          v[i] = p;
          sum += p;
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {  // 8 keys = one 16-byte chunk of the row's 128-byte line in its 64-key box
          const int chunk = (cb >> 3) + ch;  // 0..7 inside the box
          uint4 w;
          w.x = pack2<T>(v[ch * 8 + 0], v[ch * 8 + 1]);
          w.y = pack2<T>(v[ch * 8 + 2], v[ch * 8 + 3]);
          w.z = pack2<T>(v[ch * 8 + 4], v[ch * 8 + 5]);
          w.w = pack2<T>(v[ch * 8 + 6], v[ch * 8 + 7]);
          *reinterpret_cast<uint4*>(p_s + hf * PF_BOX_BYTES + row * 128 + ((chunk ^ (row & 7)) << 4)) = w;
        }
      }
      l = fmaf(l, alpha, sum);
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // P is read by the tensor core (async proxy)
      mbar_arrive(&sh.p_full);
      tc_fence_before();
      mbar_arrive(&sh.s_empty[buf]);
    }
    ok = ok && mbar_wait(&sh.p_empty, (n_tiles - 1) & 1, &sh.fail) && take_pv(n_tiles - 1);
    // the two halves of a row meet for the normaliser (every softmax thread reaches this barrier)
    l_s[hf][row] = l;
    asm volatile("bar.sync 1, 256;\n" ::: "memory");
    if (ok) {
      if (q0 + row < a.Sq) {
        const float inv = 1.f / (l + l_s[hf ^ 1][row]);
        T* dst = reinterpret_cast<T*>(a.out) + (size_t)b * a.o_sb + (size_t)(q0 + row) * a.o_sn + (size_t)h * a.o_sh +
                 hf * HC;
#pragma unroll
        for (int i = 0; i < HC; i += 8) {
          uint4 w;
          w.x = pack2<T>(o[i] * inv, o[i + 1] * inv);
          w.y = pack2<T>(o[i + 2] * inv, o[i + 3] * inv);
          w.z = pack2<T>(o[i + 4] * inv, o[i + 5] * inv);
          w.w = pack2<T>(o[i + 6] * inv, o[i + 7] * inv);
          *reinterpret_cast<uint4*>(dst + i) = w;
        }
      }
    } else {
      pf_fail(sh, a.status);
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (sh.fail) {
    // copies that were asked for may still be on their way into this CTA's shared memory: wait (bounded) for the
    // last requested tile of every stage before the memory is given up
    if (tid == 256) {
      if (sh.q_issued) mbar_wait(&sh.q_full, 0);
      for (int s = 0; s < PF_STAGES; ++s) {
        const int kl = sh.k_issued - 1 - ((sh.k_issued - 1 - s) % PF_STAGES + PF_STAGES) % PF_STAGES;
        if (sh.k_issued > s && kl >= 0) mbar_wait(&sh.k_full[s], (kl / PF_STAGES) & 1);
        const int vl = sh.v_issued - 1 - ((sh.v_issued - 1 - s) % PF_STAGES + PF_STAGES) % PF_STAGES;
        if (sh.v_issued > s && vl >= 0) mbar_wait(&sh.v_full[s], (vl / PF_STAGES) & 1);
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, PF_TMEM_COLS);
  }
}

template <typename T>
int launch_prefill(const omnikv_prefill_params* p, cudaStream_t stream) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  CUtensorMap tq, tk, tv;
  if (!make_kv_tensor_map(&tq, bf16, p->q, p->Sq, p->H, p->B, p->q_stride_row, p->q_stride_h, p->q_stride_b, PF_TILE) ||
      !make_kv_tensor_map(&tk, bf16, p->k, p->Skv, p->KVH, p->B, p->k_stride_row, p->k_stride_h, p->k_stride_b, PF_TILE) ||
      !make_kv_tensor_map(&tv, bf16, p->v, p->Skv, p->KVH, p->B, p->v_stride_row, p->v_stride_h, p->v_stride_b, PF_TILE))
    return OMNIKV_E_UNSUPPORTED;
  PfArgs a;
  a.out = p->out;
  a.o_sb = p->o_stride_b;
  a.o_sn = p->o_stride_row;
  a.o_sh = p->o_stride_h;
  a.H = p->H;
  a.G = p->H / p->KVH;
  a.Sq = p->Sq;
  a.Skv = p->Skv;
  a.q_pos0 = p->q_pos0;
  a.scale_log2 = p->scale * 1.4426950408889634f;
  a.status = p->status;
  static bool attr_set[2] = {false, false};
  auto kern = prefill_attn_kernel<T>;
  if (!attr_set[bf16 ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_BYTES);
    if (e != cudaSuccess) return record_cuda_error(e, "omnikv_prefill_attn (shared memory)");
    attr_set[bf16 ? 1 : 0] = true;
  }
  dim3 grid((unsigned)ceil_div(p->Sq, PF_TILE), (unsigned)p->H, (unsigned)p->B);
  kern<<<grid, PF_THREADS, PF_SMEM_BYTES, stream>>>(a, tq, tk, tv);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return record_cuda_error(e, "omnikv_prefill_attn");
  return OMNIKV_OK;
}

}  // namespace

template <typename T>
int launch_prefill2(const omnikv_prefill_params* p, cudaStream_t stream);  // prefill_attn2.cu
}  // namespace omnikv

extern "C" int omnikv_prefill_attn(const omnikv_prefill_params* p, void* stream) {
  using namespace omnikv;
  if (!p || !p->q || !p->k || !p->v || !p->out) return OMNIKV_E_BADARG;
  if (p->head_dim != kHeadDim) return OMNIKV_E_UNSUPPORTED;
  if (p->dtype != OMNIKV_BF16 && p->dtype != OMNIKV_F16)
    return OMNIKV_E_UNSUPPORTED;
  if (p->B <= 0 || p->H <= 0 || p->KVH <= 0 || p->H % p->KVH || p->Sq <= 0 || p->q_pos0 < 0 ||
      p->Skv < p->q_pos0 + p->Sq || p->H > 65535 || p->B > 65535)
    return OMNIKV_E_BADARG;
  if (p->o_stride_row % 8 || p->o_stride_h % 8 || p->o_stride_b % 8 || (reinterpret_cast<uintptr_t>(p->out) & 15))
    return OMNIKV_E_BADARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->variant == 1) return p->dtype == OMNIKV_BF16 ? launch_prefill<__nv_bfloat16>(p, s) : launch_prefill<__half>(p, s);
  if (p->variant != 0) return OMNIKV_E_BADARG;
  return p->dtype == OMNIKV_BF16 ? launch_prefill2<__nv_bfloat16>(p, s) : launch_prefill2<__half>(p, s);
}
