// Shared device helpers for the omnikv_b200 kernels (sm_100a).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "omnikv_b200.h"

namespace omnikv {

constexpr int kHeadDim = 128;
constexpr float kLog2e = 1.4426950408889634f;

// Records the last CUDA error text for omnikv_last_cuda_error(); returns OMNIKV_E_CUDA.
int record_cuda_error(cudaError_t e, const char* where);

#define OMNIKV_CUDA_OK(call)                                         \
  do {                                                               \
    cudaError_t e__ = (call);                                        \
    if (e__ != cudaSuccess) return omnikv::record_cuda_error(e__, #call); \
  } while (0)

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch ----------------------------------------------------------------
// A kernel launched with launch_pdl() may start while its predecessor in the stream is still running.
// pdl_trigger(): this CTA allows the NEXT kernel's CTAs to be scheduled (they take SMs as CTAs of this grid
// exit).  pdl_wait(): blocks until the PREVIOUS kernel has completed and its writes are visible; everything
// that reads or overwrites data shared with earlier kernels must come after it.  Both are no-ops for a
// kernel launched without the attribute.  Only grids that are fully resident may trigger early.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

bool pdl_enabled();  // OMNIKV_PDL=0 in the environment turns it off

#ifdef OMNIKV_TRACE
// Profiling build only (-DOMNIKV_TRACE, `python -m omnikv_b200.build --trace`): the weight-streaming and attention
// kernels stamp %globaltimer at their stages into per-launch slots; the host numbers the launches in issue order.
constexpr int kTraceSlots = 256;
int trace_next_slot();   // slot of the launch being issued (wraps at kTraceSlots)
#endif

template <typename Kern, typename Args>
inline cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t st, const Args& a) {
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
  return cudaLaunchKernelEx(&cfg, kern, a);
}

// The same for a kernel that takes its arguments one by one.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_args(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ... and needs dynamic shared memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_smem_args(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
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
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.volatile.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}

// ---- mbarrier + bulk copies (TMA, untiled) -------------------------------------------------------------
// Every wait in these kernels is bounded, by TIME (a poll of an mbarrier may itself block for a while, so a poll
// count bounds nothing): a waiter that has not been served after kWaitNs gives up and reports it.  kSpinLimit
// bounds the few remaining plain spin loops (grid barrier).
constexpr unsigned kSpinLimit = 1u << 24;
constexpr unsigned long long kWaitNs = 2000000000ull;  // 2 s

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
__device__ __forceinline__ bool mbar_try_wait(unsigned addr, unsigned parity) {
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
  return ok != 0;
}
// Wait for the phase with the given parity; false if it has not completed within kWaitNs.  `abort` (optional):
// a shared-memory flag another thread of the CTA raises when it has given up; the wait then ends at once.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, const volatile int* abort = nullptr) {
  const unsigned addr = smem_u32(bar);
  if (mbar_try_wait(addr, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 8; ++i)
      if (mbar_try_wait(addr, parity)) return true;
    if (abort && *abort) return false;
    if (globaltimer_ns() - t0 > kWaitNs) return false;
  }
}
__device__ __forceinline__ void tma_bulk_g2s(void* smem_dst, const void* gmem_src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}


// ---- waits on words another GPU (or another CTA) writes ------------------------------------------------
// Waits until *flag has reached `want` (flags only grow; compared as a signed difference so that a wrap of the
// 32-bit counter is harmless).  Bounded by TIME: a peer that never arrives costs kPeerWaitNs, after which the
// caller records a status code and returns, leaving the context usable.
constexpr unsigned long long kPeerWaitNs = kWaitNs;
__device__ __forceinline__ bool wait_flag_reached(const unsigned* flag, unsigned want) {
  if ((int)(ld_volatile_u32(flag) - want) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if ((int)(ld_volatile_u32(flag) - want) >= 0) return true;
    if (globaltimer_ns() - t0 > kPeerWaitNs) return false;
  }
}

// ---- TMA tensor-map tiles of a K or V cache ----------------------------------------------------------------
// A tile of 64 rows x 256 bytes (head_dim 128, 16-bit) is two boxes of 64 rows x 128 bytes; the map's 128-byte
// swizzle stores the 16-byte chunk c of row r at chunk c ^ (r & 7) of that row, which makes the unpadded rows
// conflict-free for ldmatrix.  A box must start on a 1024-byte boundary of shared memory.
constexpr int kTmaBoxBytes = 64 * 128;

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n" ::
          "r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// Address of the 16-byte piece at (row, byte column < 256) of a staged tile [box of the low 128 bytes | box of the high].
__device__ __forceinline__ const unsigned char* swz128(const unsigned char* tile_base, int row, int colb) {
  return tile_base + (colb >> 7) * kTmaBoxBytes + row * 128 + ((((colb & 127) >> 4) ^ (row & 7)) << 4);
}

// Host: 4-D map [B, KVH, rows, d = 128] of 16-bit elements over a cache given by element strides; box 64 elements
// x box_rows rows (at most 256), 128-byte swizzle, out-of-range rows read as zero.  False when the driver entry point
// is missing or the layout cannot be described (callers then use their cp.async variant).
bool make_kv_tensor_map(CUtensorMap* map, bool is_bf16, const void* base, int64_t rows, int KVH, int B, int64_t sr,
                        int64_t sh, int64_t sb, int box_rows = 64);

// 2-D tiles of a row-major 16-bit matrix [rows, cols] (a weight): box 64 columns x box_rows rows, 128-byte swizzle,
// rows and columns past the end read as zero.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int col, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::
          "r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(col), "r"(row), "r"(smem_u32(bar))
      : "memory");
}
bool make_matrix_tensor_map(CUtensorMap* map, bool is_bf16, const void* base, int64_t rows, int64_t cols, int64_t ld,
                            int box_rows);

// ---- cp.async (16-byte, L1-bypassing) with zero fill when !valid ---------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
  unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem_src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---- ldmatrix ---------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem_row) {
  unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_row) {
  unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}

// ---- m16n8k16 MMA, fp32 accumulate ------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// pack two floats into one 32-bit register of two 16-bit values (lo = first element)
template <typename T>
__device__ __forceinline__ unsigned pack2(float lo, float hi);
template <>
__device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
template <>
__device__ __forceinline__ unsigned pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }

// Order-preserving map float -> uint32 (larger float <=> larger key; any NaN ranks top).
__device__ __forceinline__ unsigned float_to_key(float f) {
  if (f != f) return 0xffffffffu;
  unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Split-K partial layout in the decode-attention workspace:
//   o  : float [B][H][S][128]   (un-normalised, relative to m)
//   ml : float [B][H][S][2]     (m = running max in log2 domain, l = sum of weights)
struct AttnWorkspace {
  float* o;
  float* ml;
};
constexpr size_t kAttnCntBytes = 16384;  // split-arrival counters at the start of the decode-attention workspace
__host__ __device__ inline size_t attn_ws_o_floats(int B, int H, int S) { return (size_t)B * H * S * kHeadDim; }
__host__ __device__ inline size_t attn_ws_ml_floats(int B, int H, int S) { return (size_t)B * H * S * 2; }

}  // namespace omnikv
