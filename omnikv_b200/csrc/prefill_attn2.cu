// Causal prefill attention, two query tiles per CTA with P and O in tensor memory.
//
// Same contract as prefill_attn.cu (out[b, i, h, :] = softmax over keys j <= q_pos0 + i of q.k * scale, times v).
// What differs is how a CTA is kept busy.  In the one-tile kernel the chain of a key tile
// (S ready -> row maximum -> exp2 -> P -> PV -> fold into O) runs mostly one stage after the other and the tensor
// pipe idles two thirds of the time.  Here a CTA owns TWO tiles of 128 queries, each with its own softmax warpgroup,
// and the one MMA thread alternates between them: while warpgroup 0 exponentiates its logits the tensor pipe runs
// PV and the next S of tile 1, and the other way round.  To make room for the second tile
//
//   P   is written back into tensor memory by the softmax threads (tcgen05.st, two 16-bit values per 32-bit column,
//       over the logits they have just read) and is the A operand of the PV product FROM tensor memory -- no shared
//       memory for P, no proxy fence;
//   O   accumulates in tensor memory across key tiles (the PV product adds onto it); the softmax thread rescales its
//       row there (tcgen05.ld, multiply, tcgen05.st) only when the running maximum has grown by more than 2^8 since
//       the reference maximum was set -- P stays below 256, the normaliser is kept against the same reference, so
//       the result is the same; after the first few key tiles of a row this almost never happens;
//   K/V tiles (two-stage rings) are shared by both query tiles: half the loads per query.
//
// Tensor memory: S0 | S1 | O0 | O1, 128 columns each (all 512).  Shared memory: Q0, Q1, K ring, V ring = 192 KB.
// Every tcgen05.commit covers all MMAs issued before it, so when the logits of key tile j of a query tile arrive, the
// PV product of tile j - 1 (issued earlier) has completed: the softmax thread may touch O and overwrite the old P.
// Every wait is bounded by time; on expiry the CTA raises a flag, every role leaves its loop, copies in flight are
// waited for (bounded), the tensor memory is released and status 6 is written.
#include "common.cuh"
#include "tc05.cuh"

namespace omnikv {
namespace {

constexpr int P2_TILE = 128;
constexpr int P2_TILE_BYTES = P2_TILE * 256;
constexpr int P2_BOX_BYTES = P2_TILE * 128;
constexpr int P2_STAGES = 2;
constexpr int P2_THREADS = 320;  // warps 0-3: softmax of query tile 0, 4-7: of tile 1, 8: TMA producer, 9: MMA issuer
constexpr unsigned P2_TMEM_COLS = 512;
constexpr int P2_SMEM_BYTES = P2_TILE_BYTES * (2 + 2 * P2_STAGES) + 1024;
constexpr float P2_RESCALE_GAP = 8.f;  // log2 units the maximum may grow before O and l are rescaled

struct Pf2Args {
  void* out;
  int64_t o_sb, o_sn, o_sh;
  int H, G, Sq, Skv, q_pos0;
  float scale_log2;
  int* status;
};

struct Pf2Shared {
  uint64_t q_full;
  uint64_t k_full[P2_STAGES], k_empty[P2_STAGES];
  uint64_t v_full[P2_STAGES], v_empty[P2_STAGES];
  uint64_t s_full[2], p_full[2], o_done[2];
  unsigned tmem_base;
  int fail;
  int k_issued, v_issued, q_issued;
};

__device__ __forceinline__ void pf2_fail(Pf2Shared& sh, int* status) {
  if (!sh.fail && status) atomicExch(status, 6);
  sh.fail = 1;
}

template <typename T>
__device__ __forceinline__ unsigned pk2(float a, float b);
template <>
__device__ __forceinline__ unsigned pk2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}
template <>
__device__ __forceinline__ unsigned pk2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}

template <typename T>
__global__ void __launch_bounds__(P2_THREADS, 1)
prefill_attn2_kernel(const Pf2Args a, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ Pf2Shared sh;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = smem;                                    // two query tiles
  unsigned char* k_ring = q_s + 2 * P2_TILE_BYTES;
  unsigned char* v_ring = k_ring + P2_STAGES * P2_TILE_BYTES;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qblk = (int)gridDim.x - 1 - (int)blockIdx.x;  // the longest rows of the causal triangle start first
  const int h = blockIdx.y, b = blockIdx.z, kvh = h / a.G;
  const int q0 = qblk * 2 * P2_TILE;
  // key tiles of each query tile: up to the tile of its last query's position (0 for a tile past the end)
  int nt[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int first = q0 + q * P2_TILE;
    nt[q] = first < a.Sq ? (a.q_pos0 + min(first + P2_TILE, a.Sq) - 1) / P2_TILE + 1 : 0;
  }
  const int ntm = max(nt[0], nt[1]);

  if (tid == 0) {
    sh.fail = 0;
    sh.k_issued = sh.v_issued = sh.q_issued = 0;
    mbar_init(&sh.q_full, 1);
    for (int s = 0; s < P2_STAGES; ++s) {
      mbar_init(&sh.k_full[s], 1);
      mbar_init(&sh.k_empty[s], 1);
      mbar_init(&sh.v_full[s], 1);
      mbar_init(&sh.v_empty[s], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&sh.s_full[q], 1);
      mbar_init(&sh.p_full[q], 128);
      mbar_init(&sh.o_done[q], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncwarp();
  if (warp == 0) {
    tmem_alloc(&sh.tmem_base, P2_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = sh.tmem_base;

  if (warp == 8) {
    // ---- TMA producer ------------------------------------------------------------------------------------
    if (tid == 256) {
      mbar_expect_tx(&sh.q_full, 2 * P2_TILE_BYTES);
#pragma unroll
      for (int q = 0; q < 2; ++q) {  // rows past the end of the sequence arrive as zeros
        tma_load_4d(q_s + q * P2_TILE_BYTES, &tm_q, 0, q0 + q * P2_TILE, h, b, &sh.q_full);
        tma_load_4d(q_s + q * P2_TILE_BYTES + P2_BOX_BYTES, &tm_q, 64, q0 + q * P2_TILE, h, b, &sh.q_full);
      }
      sh.q_issued = 1;
      for (int j = 0; j < ntm; ++j) {
        const int s = j % P2_STAGES;
        const unsigned par = ((j / P2_STAGES) & 1) ^ 1;
        if (!mbar_wait(&sh.k_empty[s], par, &sh.fail)) { pf2_fail(sh, a.status); break; }
        unsigned char* kd = k_ring + (size_t)s * P2_TILE_BYTES;
        mbar_expect_tx(&sh.k_full[s], P2_TILE_BYTES);
        tma_load_4d(kd, &tm_k, 0, j * P2_TILE, kvh, b, &sh.k_full[s]);
        tma_load_4d(kd + P2_BOX_BYTES, &tm_k, 64, j * P2_TILE, kvh, b, &sh.k_full[s]);
        sh.k_issued = j + 1;
        if (!mbar_wait(&sh.v_empty[s], par, &sh.fail)) { pf2_fail(sh, a.status); break; }
        unsigned char* vd = v_ring + (size_t)s * P2_TILE_BYTES;
        mbar_expect_tx(&sh.v_full[s], P2_TILE_BYTES);
        tma_load_4d(vd, &tm_v, 0, j * P2_TILE, kvh, b, &sh.v_full[s]);
        tma_load_4d(vd + P2_BOX_BYTES, &tm_v, 64, j * P2_TILE, kvh, b, &sh.v_full[s]);
        sh.v_issued = j + 1;
      }
    }
  } else if (warp == 9) {
    // ---- MMA issuer: alternates between the two query tiles --------------------------------------------------
    if (tid == 288) {
      const unsigned idesc_s = tc_instr_desc<T>(P2_TILE, P2_TILE, false, false);
      const unsigned idesc_pv = tc_instr_desc<T>(P2_TILE, kHeadDim, false, true);
      const unsigned q_base = smem_u32(q_s);
      // S of key tile j of query tile q -> columns [128 q, 128 q + 128)
      auto issue_s = [&](int q, int j) {
        const unsigned k_base = smem_u32(k_ring + (size_t)(j % P2_STAGES) * P2_TILE_BYTES);
        const unsigned qa = q_base + q * P2_TILE_BYTES;
        const unsigned d_tmem = tmem + (unsigned)q * 128u;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma(d_tmem, smem_desc_sw128(qa + (k >> 2) * P2_BOX_BYTES + (k & 3) * 32),
                 smem_desc_sw128(k_base + (k >> 2) * P2_BOX_BYTES + (k & 3) * 32), idesc_s, k > 0 ? 1u : 0u);
        tc_commit(&sh.s_full[q]);
      };
      // O_q (+)= P_q V_j: P from tensor memory (eight 32-bit columns per step of 16 keys), V MN-major
      auto issue_pv = [&](int q, int j) {
        const unsigned v_base = smem_u32(v_ring + (size_t)(j % P2_STAGES) * P2_TILE_BYTES);
        const unsigned p_tmem = tmem + (unsigned)q * 128u;
        const unsigned d_tmem = tmem + 256u + (unsigned)q * 128u;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_ts(d_tmem, p_tmem + (unsigned)k * 8u, smem_desc_sw128_mn(v_base + k * 2048, P2_BOX_BYTES, 1024), idesc_pv,
                    (j > 0 || k > 0) ? 1u : 0u);
        tc_commit(&sh.o_done[q]);
      };
      bool ok = mbar_wait(&sh.q_full, 0, &sh.fail) && (ntm == 0 || mbar_wait(&sh.k_full[0], 0, &sh.fail));
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < 2; ++q)
          if (nt[q] > 0) issue_s(q, 0);
        if (ntm > 0) tc_commit(&sh.k_empty[0]);
      }
      for (int j = 0; ok && j < ntm; ++j) {
        const bool more = j + 1 < ntm;
        if ((more && !mbar_wait(&sh.k_full[(j + 1) % P2_STAGES], ((j + 1) / P2_STAGES) & 1, &sh.fail)) ||
            !mbar_wait(&sh.v_full[j % P2_STAGES], (j / P2_STAGES) & 1, &sh.fail)) {
          ok = false;
          break;
        }
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (j < nt[q]) {
            if (!mbar_wait(&sh.p_full[q], j & 1, &sh.fail)) { ok = false; break; }
            tc_fence_after();
            issue_pv(q, j);
          }
          if (j + 1 < nt[q]) issue_s(q, j + 1);  // overwrites P of tile j: the MMAs run in the order they are issued
        }
        if (!ok) break;
        if (more) tc_commit(&sh.k_empty[(j + 1) % P2_STAGES]);
        tc_commit(&sh.v_empty[j % P2_STAGES]);
      }
      if (!ok) pf2_fail(sh, a.status);
    }
  } else {
    // ---- softmax: warpgroup q = warp >> 2 owns query tile q, thread = query row ------------------------------
    const int q = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + (tid & 31);
    const int qrow = q0 + q * P2_TILE + row;       // query index inside the chunk
    const int pos = a.q_pos0 + qrow;               // last visible key
    const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16);
    const unsigned s_addr = lane_addr + (unsigned)q * 128u;         // logits, then P over them
    const unsigned o_addr = lane_addr + 256u + (unsigned)q * 128u;  // output accumulator
    const float c = a.scale_log2;
    const int my_nt = nt[q];
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_nt; ++j) {
      if (!mbar_wait(&sh.s_full[q], j & 1, &sh.fail)) { ok = false; break; }
      tc_fence_after();
      const int key0 = j * P2_TILE;
      const bool masked = key0 + P2_TILE - 1 > a.q_pos0 + q0 + q * P2_TILE;  // some query of this tile sees only part
      // pass A: the row's maximum (raw logits; the scale is positive); 64 columns per round trip to tensor memory
      float mraw = -INFINITY;
#pragma unroll
      for (int cb = 0; cb < P2_TILE; cb += 64) {
        float v[64];
#pragma unroll
        for (int u = 0; u < 4; ++u) tmem_ld16(s_addr + cb + 16 * u, *reinterpret_cast<float(*)[16]>(&v[16 * u]));
        tmem_ld_wait();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (key0 + cb + i <= pos) mraw = fmaxf(mraw, v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) mraw = fmaxf(mraw, v[i]);
        }
      }
      // The reference maximum m moves only when the row's maximum has outgrown it by more than the gap (and on the
      // first tile).  A fully masked tile (only possible for rows past the end of the sequence) leaves it alone.
      const float mx = mraw * c;
      const bool grow = mx > m + P2_RESCALE_GAP;  // false for mx = -inf; true on the first tile (m = -inf)
      const float alpha = grow ? ex2_fast(m - mx) : 1.f;
      if (grow) m = mx;
      // the PV product of tile j - 1 has completed (see the note on commits at the top): rescale O where needed
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll
        for (int cb = 0; cb < kHeadDim; cb += 16) {
          float v[16];
          unsigned r[16];
          tmem_ld16(o_addr + cb, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(v[i] * alpha);
          tmem_st16(o_addr + cb, r);
        }
      }
      l *= alpha;
      // pass B: P = 2^(S c - m) as 16-bit pairs into the columns the logits came from, row sum
      const float mref = (m == -INFINITY) ? 0.f : m;
      float sum = 0.f;
      float vb[2][32];
      tmem_ld16(s_addr, *reinterpret_cast<float(*)[16]>(&vb[0][0]));
      tmem_ld16(s_addr + 16, *reinterpret_cast<float(*)[16]>(&vb[0][16]));
      tmem_ld_wait();
#pragma unroll
      for (int ci = 0; ci < P2_TILE / 32; ++ci) {
        const int cb = ci * 32;
        float(&v)[32] = vb[ci & 1];
        if (ci + 1 < P2_TILE / 32) {  // the next chunk travels while this one is exponentiated
          tmem_ld16(s_addr + cb + 32, *reinterpret_cast<float(*)[16]>(&vb[(ci + 1) & 1][0]));
          tmem_ld16(s_addr + cb + 48, *reinterpret_cast<float(*)[16]>(&vb[(ci + 1) & 1][16]));
        }
        unsigned r[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_fast(fmaf(v[i], c, -mref));
          float p1 = ex2_fast(fmaf(v[i + 1], c, -mref));
          if (masked) {
            if (key0 + cb + i > pos) p0 = 0.f;
            if (key0 + cb + i + 1 > pos) p1 = 0.f;
          }
          sum += p0 + p1;
          r[i >> 1] = pk2<T>(p0, p1);
        }
        // columns [cb / 2, cb / 2 + 16): logits this thread has already read (the chunk in flight starts at cb + 32)
        tmem_st16(s_addr + (cb >> 1), r);
        if (ci + 1 < P2_TILE / 32) tmem_ld_wait();
      }
      l += sum;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&sh.p_full[q]);
    }
    // the last PV product, then the row: O / l
    if (ok && my_nt > 0 && !mbar_wait(&sh.o_done[q], (my_nt - 1) & 1, &sh.fail)) ok = false;
    if (ok && my_nt > 0) {
      tc_fence_after();
      // every lane takes part in the warp-wide tensor-memory reads; only rows inside the sequence are stored
      const float inv = 1.f / l;
      T* dst = reinterpret_cast<T*>(a.out) + (size_t)b * a.o_sb + (size_t)qrow * a.o_sn + (size_t)h * a.o_sh;
#pragma unroll
      for (int cb = 0; cb < kHeadDim; cb += 32) {
        float v[32];
        tmem_ld16(o_addr + cb, *reinterpret_cast<float(*)[16]>(&v[0]));
        tmem_ld16(o_addr + cb + 16, *reinterpret_cast<float(*)[16]>(&v[16]));
        tmem_ld_wait();
        if (qrow < a.Sq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pk2<T>(v[i] * inv, v[i + 1] * inv);
            w.y = pk2<T>(v[i + 2] * inv, v[i + 3] * inv);
            w.z = pk2<T>(v[i + 4] * inv, v[i + 5] * inv);
            w.w = pk2<T>(v[i + 6] * inv, v[i + 7] * inv);
            *reinterpret_cast<uint4*>(dst + cb + i) = w;
          }
        }
      }
    } else if (!ok) {
      pf2_fail(sh, a.status);
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (sh.fail) {
    if (tid == 256) {  // wait (bounded) for the last requested tile of every stage before the memory is given up
      if (sh.q_issued) mbar_wait(&sh.q_full, 0);
      for (int s = 0; s < P2_STAGES; ++s) {
        const int kl = sh.k_issued - 1 - ((sh.k_issued - 1 - s) % P2_STAGES + P2_STAGES) % P2_STAGES;
        if (sh.k_issued > s && kl >= 0) mbar_wait(&sh.k_full[s], (kl / P2_STAGES) & 1);
        const int vl = sh.v_issued - 1 - ((sh.v_issued - 1 - s) % P2_STAGES + P2_STAGES) % P2_STAGES;
        if (sh.v_issued > s && vl >= 0) mbar_wait(&sh.v_full[s], (vl / P2_STAGES) & 1);
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, P2_TMEM_COLS);
  }
}

}  // namespace

// Launch of the two-tile kernel (called by omnikv_prefill_attn).
template <typename T>
int launch_prefill2(const omnikv_prefill_params* p, cudaStream_t stream) {
  const bool bf16 = std::is_same<T, __nv_bfloat16>::value;
  CUtensorMap tq, tk, tv;
  if (!make_kv_tensor_map(&tq, bf16, p->q, p->Sq, p->H, p->B, p->q_stride_row, p->q_stride_h, p->q_stride_b, P2_TILE) ||
      !make_kv_tensor_map(&tk, bf16, p->k, p->Skv, p->KVH, p->B, p->k_stride_row, p->k_stride_h, p->k_stride_b, P2_TILE) ||
      !make_kv_tensor_map(&tv, bf16, p->v, p->Skv, p->KVH, p->B, p->v_stride_row, p->v_stride_h, p->v_stride_b, P2_TILE))
    return OMNIKV_E_UNSUPPORTED;
  Pf2Args a;
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
  auto kern = prefill_attn2_kernel<T>;
  if (!attr_set[bf16 ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P2_SMEM_BYTES);
    if (e != cudaSuccess) return record_cuda_error(e, "omnikv_prefill_attn (shared memory)");
    attr_set[bf16 ? 1 : 0] = true;
  }
  dim3 grid((unsigned)ceil_div(p->Sq, 2 * P2_TILE), (unsigned)p->H, (unsigned)p->B);
  kern<<<grid, P2_THREADS, P2_SMEM_BYTES, stream>>>(a, tq, tk, tv);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return record_cuda_error(e, "omnikv_prefill_attn");
  return OMNIKV_OK;
}
template int launch_prefill2<__nv_bfloat16>(const omnikv_prefill_params*, cudaStream_t);
template int launch_prefill2<__half>(const omnikv_prefill_params*, cudaStream_t);

}  // namespace omnikv
