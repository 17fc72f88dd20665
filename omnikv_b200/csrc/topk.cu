// Top-k selector: MSB-first radix select on order-preserving keys, then an ordered compaction
// that emits the selected positions in ascending order -- no sort.
//
// One thread-block cluster per sequence.  Every CTA of the cluster keeps its contiguous slice of
// the keys resident in shared memory (the scores are read from L2/HBM exactly once); the four
// 8-bit digit histograms are built with warp-aggregated shared-memory atomics and summed across
// the cluster through distributed shared memory.  Integer atomics only: the result is deterministic.
//
// This kernel never lets its successor be scheduled early (no griddepcontrol.launch_dependents, although most SMs
// are idle while one cluster selects): the decode attention kernels read the index list and its count BEFORE their
// own dependent-launch wait, which is only sound because the kernel right behind the selector cannot start -- and
// so cannot let its own successors start -- before the selector has completed.
#include <cooperative_groups.h>

#include <stdlib.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace omnikv {
namespace {

constexpr int TK_THREADS = 1024;
constexpr int TK_WARPS = TK_THREADS / 32;
constexpr int TK_MAX_CLUSTER = 16;  // 16 needs the non-portable cluster size attribute; 8 is the portable limit
constexpr int TK_RESIDENT_KEYS = 49152;  // 192 KiB of keys per CTA

struct TopkArgs {
  const float* scores;
  int n_planes;
  int64_t plane_stride, batch_stride;
  const int* len;
  const int* k;
  const int* append_n;
  int* idx_out;
  int64_t idx_stride;
  int* count_out;
  unsigned* gkeys;  // workspace [B][max_len] when the slice does not fit shared memory
  int max_len;
  int vec4;         // scores, strides and slices allow 16-byte loads
};

struct TkShared {
  unsigned hist[256];                // this CTA's histogram of the current digit
  unsigned total[2][256];            // cluster-wide histogram, filled by remote atomics from every CTA (double-buffered)
  unsigned cnt_all[TK_MAX_CLUSTER][2];  // (greater, equal) counts of every CTA, pushed by their owners
  unsigned warp_gt[TK_WARPS], warp_eq[TK_WARPS];
  unsigned sel_digit, sel_remaining;
};

template <bool RESIDENT>
__global__ void __launch_bounds__(TK_THREADS, 1) topk_kernel(const TopkArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  TkShared& sh = *reinterpret_cast<TkShared*>(smem_raw);
  unsigned* skeys = reinterpret_cast<unsigned*>(smem_raw + ((sizeof(TkShared) + 15) / 16) * 16);

  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int csize = (int)cluster.num_blocks();
  const int b = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int n = max(0, min(a.len[b], a.max_len));
  const int kk = max(0, min(a.k[b], n));
  const int app = a.append_n ? max(0, a.append_n[b]) : 0;
  int* out = a.idx_out + (size_t)b * a.idx_stride;

  // contiguous slice of this CTA, 4-aligned
  const int slice = ceil_div(ceil_div(n, csize), 4) * 4;
  const int s0 = min(n, crank * slice);
  const int s1 = min(n, s0 + slice);
  const int cnt = s1 - s0;
  unsigned* gk = RESIDENT ? nullptr : a.gkeys + (size_t)b * a.max_len + s0;

  // ---- load: max over planes, map to keys ---------------------------------------------------
  // four consecutive scores per thread and plane (16-byte loads, all planes' loads of an iteration in flight)
  const float* sc = a.scores + (size_t)b * a.batch_stride + s0;
  for (int i = tid; i < 256; i += TK_THREADS) sh.total[0][i] = sh.total[1][i] = 0;
  if (a.vec4) {
    const int n4 = cnt >> 2;
    for (int i4 = tid; i4 < n4; i4 += TK_THREADS) {
      float4 v = __ldcg(reinterpret_cast<const float4*>(sc) + i4);
      for (int p = 1; p < a.n_planes; ++p) {
        const float4 w = __ldcg(reinterpret_cast<const float4*>(sc + (size_t)p * a.plane_stride) + i4);
        v.x = (w.x > v.x || w.x != w.x) ? w.x : v.x;  // NaN wins, as in torch.topk
        v.y = (w.y > v.y || w.y != w.y) ? w.y : v.y;
        v.z = (w.z > v.z || w.z != w.z) ? w.z : v.z;
        v.w = (w.w > v.w || w.w != w.w) ? w.w : v.w;
      }
      const uint4 key = make_uint4(float_to_key(v.x), float_to_key(v.y), float_to_key(v.z), float_to_key(v.w));
      if (RESIDENT) reinterpret_cast<uint4*>(skeys)[i4] = key; else reinterpret_cast<uint4*>(gk)[i4] = key;
    }
  }
  for (int i = (a.vec4 ? (cnt & ~3) : 0) + tid; i < cnt; i += TK_THREADS) {
    float v = sc[i];
    for (int p = 1; p < a.n_planes; ++p) {
      const float w = sc[(size_t)p * a.plane_stride + i];
      v = (w > v || w != w) ? w : v;
    }
    const unsigned key = float_to_key(v);
    if (RESIDENT) skeys[i] = key; else gk[i] = key;
  }
  cluster.sync();  // every CTA's totals are zeroed before anyone adds to them

  // ---- radix select --------------------------------------------------------------------------
  // Each pass: local histogram of the digit (shared-memory atomics, aggregated per warp), pushed into EVERY
  // CTA's cluster-wide histogram with remote atomics, one cluster barrier, then every CTA scans its own copy.
  unsigned prefix = 0, mask = 0;
  unsigned remaining = (unsigned)kk;
  if (kk > 0) {
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      unsigned* tot = sh.total[pass & 1];
      for (int i = tid; i < 256; i += TK_THREADS) {
        sh.hist[i] = 0;
        sh.total[(pass + 1) & 1][i] = 0;  // the next pass's buffer: nobody adds to it before the barrier below
      }
      __syncthreads();
      for (int i0 = 0; i0 < cnt; i0 += TK_THREADS) {
        const int i = i0 + tid;
        bool act = false;
        unsigned bin = 0;
        if (i < cnt) {
          const unsigned key = RESIDENT ? skeys[i] : gk[i];
          act = (key & mask) == prefix;
          bin = (key >> shift) & 255u;
        }
        const unsigned actmask = __ballot_sync(0xffffffffu, act);
        if (act) {
          const unsigned peers = __match_any_sync(actmask, bin);
          if ((unsigned)lane == (unsigned)(__ffs(peers) - 1)) atomicAdd(&sh.hist[bin], (unsigned)__popc(peers));
        }
      }
      __syncthreads();
      for (int i = tid; i < 256 * csize; i += TK_THREADS) {
        const int bin = i & 255, r = i >> 8;
        const unsigned v = sh.hist[bin];
        if (v) atomicAdd(cluster.map_shared_rank(&tot[bin], r), v);
      }
      cluster.sync();
      if (warp == 0) {
        // find the digit d with count(bins > d) < remaining <= count(bins >= d); 8 bins per lane,
        // lane 0 holds the highest bins
        unsigned c[8];
        unsigned mine = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          c[j] = tot[255 - (lane * 8 + j)];
          mine += c[j];
        }
        unsigned incl = mine;  // inclusive scan over lanes
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const unsigned v = __shfl_up_sync(0xffffffffu, incl, off);
          if (lane >= off) incl += v;
        }
        const unsigned excl = incl - mine;
        if (excl < remaining && remaining <= incl) {
          unsigned run = excl;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (run < remaining && remaining <= run + c[j]) {
              sh.sel_digit = 255 - (lane * 8 + j);
              sh.sel_remaining = remaining - run;
            }
            run += c[j];
          }
        }
      }
      __syncthreads();
      prefix |= sh.sel_digit << shift;
      mask |= 255u << shift;
      remaining = sh.sel_remaining;
    }
  }
  const unsigned T = prefix;  // key of the k-th largest score; `remaining` ties of it are taken

  // ---- ordered compaction --------------------------------------------------------------------
  // each warp owns a contiguous sub-slice of the CTA's slice
  const int wslice = ceil_div(ceil_div(cnt, TK_WARPS), 32) * 32;
  const int w0 = min(cnt, warp * wslice);
  const int w1 = min(cnt, w0 + wslice);
  unsigned my_gt = 0, my_eq = 0;
  if (kk > 0) {
    for (int i = w0 + lane; i < w1; i += 32) {
      const unsigned key = RESIDENT ? skeys[i] : gk[i];
      my_gt += key > T;
      my_eq += key == T;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    my_gt += __shfl_xor_sync(0xffffffffu, my_gt, off);
    my_eq += __shfl_xor_sync(0xffffffffu, my_eq, off);
  }
  if (lane == 0) {
    sh.warp_gt[warp] = my_gt;
    sh.warp_eq[warp] = my_eq;
  }
  __syncthreads();
  if (tid < csize) {  // thread r pushes this CTA's counts into CTA r's table
    unsigned g = 0, e = 0;
    for (int w = 0; w < TK_WARPS; ++w) {
      g += sh.warp_gt[w];
      e += sh.warp_eq[w];
    }
    unsigned* dst = cluster.map_shared_rank(&sh.cnt_all[crank][0], tid);
    dst[0] = g;
    dst[1] = e;
  }
  cluster.sync();  // counts of every CTA have arrived in this CTA's table
  // positions selected / ties seen before this CTA, then before this warp
  unsigned eq_before = 0, sel_before = 0;
  for (int r = 0; r < crank; ++r) {
    const unsigned rg = sh.cnt_all[r][0];
    const unsigned re = sh.cnt_all[r][1];
    const unsigned take = (remaining > eq_before) ? min(re, remaining - eq_before) : 0u;
    sel_before += rg + take;
    eq_before += re;
  }
  for (int w = 0; w < warp; ++w) {
    const unsigned rg = sh.warp_gt[w], re = sh.warp_eq[w];
    const unsigned take = (remaining > eq_before) ? min(re, remaining - eq_before) : 0u;
    sel_before += rg + take;
    eq_before += re;
  }
  if (kk > 0) {
    const unsigned lt_mask = (1u << lane) - 1u;
    for (int i0 = w0; i0 < w1; i0 += 32) {
      const int i = i0 + lane;
      bool gt = false, eq = false;
      if (i < w1) {
        const unsigned key = RESIDENT ? skeys[i] : gk[i];
        gt = key > T;
        eq = key == T;
      }
      const unsigned eqm = __ballot_sync(0xffffffffu, eq);
      const unsigned eq_rank = eq_before + __popc(eqm & lt_mask);
      const bool sel = gt || (eq && eq_rank < remaining);
      const unsigned selm = __ballot_sync(0xffffffffu, sel);
      if (sel) out[sel_before + __popc(selm & lt_mask)] = s0 + i;
      sel_before += __popc(selm);
      eq_before += __popc(eqm);
    }
  }
  // appended window positions and the count
  if (crank == 0) {
    for (int i = tid; i < app; i += TK_THREADS) out[kk + i] = n + i;
    if (tid == 0) a.count_out[b] = kk + app;
  }
  cluster.sync();  // no CTA may exit while a peer can still read its shared memory
}

}  // namespace
}  // namespace omnikv

extern "C" size_t omnikv_topk_workspace_bytes(int B, int max_len) {
  if (B <= 0 || max_len <= 0) return 0;
  // only used when a CTA's slice does not fit shared memory; always sized so callers need no case split
  return (size_t)B * (size_t)max_len * sizeof(unsigned);
}

extern "C" int omnikv_topk(const float* scores, int n_planes, int64_t plane_stride, int64_t batch_stride,
                           const int32_t* len, const int32_t* k, const int32_t* append_n, int B, int max_len,
                           int32_t* idx_out, int64_t idx_stride, int32_t* count_out, void* workspace,
                           size_t workspace_bytes, void* stream) {
  using namespace omnikv;
  if (!scores || !len || !k || !idx_out || !count_out) return OMNIKV_E_BADARG;
  if (B <= 0 || max_len <= 0 || n_planes <= 0 || idx_stride <= 0) return OMNIKV_E_BADARG;
  if (n_planes > 1 && plane_stride <= 0) return OMNIKV_E_BADARG;
  TopkArgs a;
  a.scores = scores; a.n_planes = n_planes; a.plane_stride = plane_stride; a.batch_stride = batch_stride;
  a.len = len; a.k = k; a.append_n = append_n; a.idx_out = idx_out; a.idx_stride = idx_stride;
  a.count_out = count_out; a.gkeys = static_cast<unsigned*>(workspace); a.max_len = max_len;
  a.vec4 = ((reinterpret_cast<uintptr_t>(scores) & 15) == 0 && batch_stride % 4 == 0 &&
            (n_planes == 1 || plane_stride % 4 == 0) && (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0) &&
            max_len % 4 == 0) ? 1 : 0;

  // Slices of at most 8192 keys per CTA (1024 for a single sequence); a cluster of 16 (above the portable limit of 8) when the device can
  // co-schedule one, since the load of the score planes and every histogram pass scale with the CTA count.
  static const int max_cluster = [] {
    const char* e = getenv("OMNIKV_TOPK_CLUSTER");
    const int v = e ? atoi(e) : TK_MAX_CLUSTER;
    return v >= 1 && v <= TK_MAX_CLUSTER ? v : TK_MAX_CLUSTER;
  }();
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  decltype(&topk_kernel<true>) kern = nullptr;
  int csize = 1;
  for (int limit = max_cluster;; limit = 8) {
    csize = 1;
    // a single sequence leaves the other SMs idle anyway: slices down to 1024 keys (every phase is a latency chain
    // whose length goes with the slice); a batch keeps 8192 keys per CTA so that its clusters fit the device together
    const int slice_keys = B == 1 ? 1024 : 8192;
    while (csize < limit && ceil_div(max_len, csize) > slice_keys) csize *= 2;
    const int slice = ceil_div(ceil_div(max_len, csize), 4) * 4;
    const bool resident = slice <= TK_RESIDENT_KEYS;
    if (!resident && (!workspace || workspace_bytes < omnikv_topk_workspace_bytes(B, max_len))) return OMNIKV_E_WORKSPACE;
    const size_t smem = ((sizeof(TkShared) + 15) / 16) * 16 + (resident ? (size_t)slice * sizeof(unsigned) : 0);
    kern = resident ? topk_kernel<true> : topk_kernel<false>;
    OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (csize > 8) OMNIKV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    cfg = {};
    cfg.gridDim = dim3(csize, B, 1);
    cfg.blockDim = dim3(TK_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (csize <= 8) break;
    // a cluster of 16 CTAs of this size must be schedulable at once on this device; else the portable 8
    int n_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&n_clusters, kern, &cfg) == cudaSuccess && n_clusters >= 1) break;
    (void)cudaGetLastError();
  }
  OMNIKV_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, a));
  return OMNIKV_OK;
}
