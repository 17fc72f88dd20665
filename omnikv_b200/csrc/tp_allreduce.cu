// Small collectives over peer-mapped memory (NVLink): SUM all-reduce (the hidden state of a batched decode step), MAX
// all-reduce (the filter layers' fp32 score planes: order independent, so every rank ends with bit-identical planes
// and runs the same top-k) and all-gather (the vocabulary-sharded logits).  Below, for the SUM:
//
// At 8 ranks the hidden state of a decode step is tens to hundreds of KB: an all-reduce of that size is
// latency, and a ring or tree pays several hops.  Here every rank stores its vector straight into a slot of
// EVERY rank's exchange buffer (one hop, plain peer stores), the CTA that finishes last raises this rank's
// flag on every rank, and every rank then adds the world's vectors in rank order -- so all ranks compute
// bit-identical sums -- in fp32, rounding once.  One kernel per call on each GPU; the kernels of different
// GPUs wait for one another's flags with a bounded spin (a rank's flag depends only on that rank's own
// stores, never on a peer, so there is no cycle).  The grid is small enough to be resident at once.
//
// Exchange buffer layout is that of omnikv_tp_exchange (two alternating slots).  Slot and flag value come from
// a DEVICE-side counter of the calls made on this exchange object (slot = calls & 1, flag = calls + 1), which
// every rank advances identically: consecutive calls therefore always alternate slots, whatever the number of
// calls per decode step and also when a captured step is replayed.  (A rank can only be two calls ahead of a
// peer after that peer has raised the flag of the call in between, i.e. has finished reading the older slot.)
// Nothing is ever reset.  Plain peer loads and stores only.
#include "common.cuh"

namespace omnikv {
namespace {

constexpr int AR_THREADS = 256;
constexpr int AR_MAX_CTAS = 64;

struct ArArgs {
  void* x;                 // [n_vec] 16-byte vectors, reduced in place
  int n_vec;
  int world, rank;
  uint4* peer_slot[8];     // rank p's region for MY vector in slot 0 (slot 1: + 8 * slot_stride_vec)
  unsigned* peer_flag[8];  // rank p's flag word for (slot 0, me) (slot 1: + 8)
  const uint4* my_slots;   // local: [2 slots][8][slot_stride_vec]
  size_t slot_stride_vec;
  const unsigned* my_flags;  // local [2 slots][8]
  unsigned* done;          // local: [0] counter of finished CTAs (self-resetting), [1] calls made so far
  int* status;
  void* out;               // gather: [world][n_vec] vectors
};
enum { OP_SUM = 0, OP_MAX = 1, OP_GATHER = 2 };

template <typename T>
__device__ __forceinline__ void add8(const uint4& v, float (&acc)[8]);
template <>
__device__ __forceinline__ void add8<float>(const uint4& v, float (&acc)[8]) {
  acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
  acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void add8<__nv_bfloat16>(const uint4& v, float (&acc)[8]) {
  const unsigned u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(u[i] << 16);
    acc[2 * i + 1] += __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void add8<__half>(const uint4& v, float (&acc)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    acc[2 * i] += t.x;
    acc[2 * i + 1] += t.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  return make_uint4(pack2<T>(acc[0], acc[1]), pack2<T>(acc[2], acc[3]), pack2<T>(acc[4], acc[5]), pack2<T>(acc[6], acc[7]));
}
template <>
__device__ __forceinline__ uint4 pack8<float>(const float (&acc)[8]) {
  return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
}

template <typename T, int OP>
__global__ void __launch_bounds__(AR_THREADS) tp_allreduce_kernel(const ArArgs a) {
  __shared__ int fail;
  __shared__ unsigned call_s;
  const int tid = threadIdx.x;
  const int stride = gridDim.x * AR_THREADS;
  uint4* x = static_cast<uint4*>(a.x);
  if (tid == 0) {
    fail = 0;
    // the number of this call: read before this CTA counts itself in, so before the last CTA can bump it
    call_s = ld_volatile_u32(a.done + 1);
  }
  __syncthreads();
  const unsigned call = call_s;
  const unsigned slot = call & 1u;
  // 1. my vector into my slot on every rank (the local one included)
  for (int v = blockIdx.x * AR_THREADS + tid; v < a.n_vec; v += stride) {
    const uint4 val = x[v];
    for (int p = 0; p < a.world; ++p) (a.peer_slot[p] + (size_t)slot * 8 * a.slot_stride_vec)[v] = val;
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    // all of this CTA's stores are ordered before its count; the CTA that completes the count raises this
    // rank's flag on every rank and advances the call counter for the next launch
    const unsigned val = call + 1u;
    if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
      atomicExch(a.done, 0u);
      atomicExch(a.done + 1, val);
      __threadfence_system();
      for (int p = 0; p < a.world; ++p)
        asm volatile("st.volatile.global.u32 [%0], %1;\n" ::"l"(a.peer_flag[p] + slot * 8), "r"(val) : "memory");
    }
    // 2. every rank's vector must have landed here (wait bounded by time)
    for (int r = 0; r < a.world; ++r) {
      if (!wait_flag_reached(a.my_flags + slot * 8 + r, val)) {
        fail = 1;
        atomicExch(a.status, 4);
        break;
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  if (fail) return;
  const uint4* mine = a.my_slots + (size_t)slot * 8 * a.slot_stride_vec;
  if constexpr (OP == OP_GATHER) {
    // 3. the ranks' vectors one behind the other
    uint4* out = static_cast<uint4*>(a.out);
    for (int r = 0; r < a.world; ++r)
      for (int v = blockIdx.x * AR_THREADS + tid; v < a.n_vec; v += stride)
        out[(size_t)r * a.n_vec + v] = __ldcg(mine + (size_t)r * a.slot_stride_vec + v);
  } else if constexpr (OP == OP_MAX) {
    // 3. element-wise maximum of fp32 vectors (any order gives the same bits)
    for (int v = blockIdx.x * AR_THREADS + tid; v < a.n_vec; v += stride) {
      uint4 m = __ldcg(mine + v);
      for (int r = 1; r < a.world; ++r) {
        const uint4 o = __ldcg(mine + (size_t)r * a.slot_stride_vec + v);
        m.x = __float_as_uint(fmaxf(__uint_as_float(m.x), __uint_as_float(o.x)));
        m.y = __float_as_uint(fmaxf(__uint_as_float(m.y), __uint_as_float(o.y)));
        m.z = __float_as_uint(fmaxf(__uint_as_float(m.z), __uint_as_float(o.z)));
        m.w = __float_as_uint(fmaxf(__uint_as_float(m.w), __uint_as_float(o.w)));
      }
      x[v] = m;
    }
  } else {
    // 3. sum in rank order, fp32, rounded once
    for (int v = blockIdx.x * AR_THREADS + tid; v < a.n_vec; v += stride) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < a.world; ++r) add8<T>(__ldcg(mine + (size_t)r * a.slot_stride_vec + v), acc);
      x[v] = pack8<T>(acc);
    }
  }
}

}  // namespace
}  // namespace omnikv

namespace omnikv {
namespace {
int tp_collective(int op, int dtype, void* x, int64_t n, void* out, const omnikv_tp_exchange* t, int32_t* status,
                  void* stream) {
  if (!x || n <= 0 || !t || !status) return OMNIKV_E_BADARG;
  if (op == OP_GATHER && !out) return OMNIKV_E_BADARG;
  if (op == OP_MAX && dtype != OMNIKV_F32) return OMNIKV_E_UNSUPPORTED;
  if (t->world <= 1) return OMNIKV_OK;
  if (t->world > 8 || t->rank < 0 || t->rank >= t->world || !t->done_counter || t->hidden <= 0)
    return OMNIKV_E_BADARG;
  const int esz = dtype == OMNIKV_F32 ? 4 : 2;
  if (dtype != OMNIKV_F32 && dtype != OMNIKV_BF16 && dtype != OMNIKV_F16) return OMNIKV_E_UNSUPPORTED;
  const size_t bytes = (size_t)n * esz;
  const size_t slot_bytes = (size_t)t->hidden * sizeof(float);  // one (slot, rank) region of the exchange buffer
  if (bytes % 16 || (reinterpret_cast<uintptr_t>(x) & 15) || slot_bytes % 16) return OMNIKV_E_BADARG;
  if (bytes > slot_bytes) return OMNIKV_E_WORKSPACE;
  ArArgs a = {};
  a.x = x; a.n_vec = (int)(bytes / 16); a.world = t->world; a.rank = t->rank;
  const size_t flags_off = (size_t)2 * 8 * slot_bytes * 2;  // behind the entry area (8 bytes per element of `hidden`)
  for (int p = 0; p < t->world; ++p) {
    if (!t->peer_base[p]) return OMNIKV_E_BADARG;
    unsigned char* base = static_cast<unsigned char*>(t->peer_base[p]);
    a.peer_slot[p] = reinterpret_cast<uint4*>(base + (size_t)t->rank * slot_bytes);
    a.peer_flag[p] = reinterpret_cast<unsigned*>(base + flags_off) + t->rank;
  }
  unsigned char* mine = static_cast<unsigned char*>(t->peer_base[t->rank]);
  a.my_slots = reinterpret_cast<const uint4*>(mine);
  a.slot_stride_vec = slot_bytes / 16;
  a.my_flags = reinterpret_cast<const unsigned*>(mine + flags_off);
  a.done = t->done_counter; a.status = status; a.out = out;
  int grid = ceil_div(a.n_vec, AR_THREADS);
  if (grid > AR_MAX_CTAS) grid = AR_MAX_CTAS;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (op == OP_GATHER) {
    tp_allreduce_kernel<float, OP_GATHER><<<grid, AR_THREADS, 0, st>>>(a);  // moves 16-byte vectors: any element type
  } else if (op == OP_MAX) {
    tp_allreduce_kernel<float, OP_MAX><<<grid, AR_THREADS, 0, st>>>(a);
  } else {
    switch (dtype) {
      case OMNIKV_BF16: tp_allreduce_kernel<__nv_bfloat16, OP_SUM><<<grid, AR_THREADS, 0, st>>>(a); break;
      case OMNIKV_F16: tp_allreduce_kernel<__half, OP_SUM><<<grid, AR_THREADS, 0, st>>>(a); break;
      default: tp_allreduce_kernel<float, OP_SUM><<<grid, AR_THREADS, 0, st>>>(a); break;
    }
  }
  OMNIKV_CUDA_OK(cudaGetLastError());
  return OMNIKV_OK;
}
}  // namespace
}  // namespace omnikv

extern "C" int omnikv_tp_allreduce_sum(int dtype, void* x, int64_t n, const omnikv_tp_exchange* t, int32_t* status,
                                       void* stream) {
  return omnikv::tp_collective(omnikv::OP_SUM, dtype, x, n, nullptr, t, status, stream);
}
extern "C" int omnikv_tp_allreduce_max(void* x, int64_t n, const omnikv_tp_exchange* t, int32_t* status, void* stream) {
  return omnikv::tp_collective(omnikv::OP_MAX, OMNIKV_F32, x, n, nullptr, t, status, stream);
}
extern "C" int omnikv_tp_allgather(int dtype, const void* x, int64_t n, void* out, const omnikv_tp_exchange* t,
                                   int32_t* status, void* stream) {
  return omnikv::tp_collective(omnikv::OP_GATHER, dtype, const_cast<void*>(x), n, out, t, status, stream);
}
