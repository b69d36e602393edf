// Shared device/host helpers for the qdecode kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/qdecode.h"

typedef __nv_bfloat16 bf16;

// ---- host side: error text + launch helper ---------------------------------
void q_set_error(const char* fmt, ...);
bool q_pdl_enabled();

#define Q_CHECK_ARG(cond, ...)                                   \
  do {                                                           \
    if (!(cond)) { q_set_error(__VA_ARGS__); return Q_ERR_ARG; } \
  } while (0)

// Vectorised kernels load and store 8 or 16 bytes at a time: a pointer that is not aligned
// would fault on the device, so it is refused on the host. Null passes (optional operands).
#define Q_CHECK_ALIGN(ptr, bytes, who)                                                        \
  Q_CHECK_ARG((((uintptr_t)(ptr)) & ((bytes) - 1)) == 0, "%s: %s must be %d-byte aligned", who, #ptr, (int)(bytes))

#define Q_CHECK_CUDA(expr)                                                     \
  do {                                                                         \
    cudaError_t _e = (expr);                                                   \
    if (_e != cudaSuccess) {                                                   \
      q_set_error("%s failed: %s", #expr, cudaGetErrorString(_e));             \
      return Q_ERR_CUDA;                                                       \
    }                                                                          \
  } while (0)

// Launches `kernel` with the programmatic-dependent-launch attribute so that its
// prologue may overlap the previous kernel's tail. Every kernel here executes
// pdl_wait() before it touches memory another kernel of the step writes.
template <typename... KArgs, typename... Args>
static inline cudaError_t q_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                   size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = q_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Same, for a kernel whose CTAs form thread-block clusters of `cluster_x` along x.
template <typename... KArgs, typename... Args>
static inline cudaError_t q_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = q_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

int q_sm_count();

// Device index of the calling thread's current device, or -1 (also -1 above 63: the
// per-device caches below hold 64 entries).
static inline int q_device_index() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return -1; }
  return (dev >= 0 && dev < 64) ? dev : -1;
}

// Defines `int* fn()`: the device address of a file-scope __device__ status word on the
// current device (looked up once per device and cached), or null.
#define Q_DEFINE_STATUS_ADDR(fn, symbol)                                             \
  int* fn() {                                                                        \
    static int* cached[64] = {nullptr};                                              \
    const int dev = q_device_index();                                                \
    if (dev < 0) return nullptr;                                                     \
    if (!cached[dev]) {                                                              \
      void* p = nullptr;                                                             \
      if (cudaGetSymbolAddress(&p, symbol) != cudaSuccess) { cudaGetLastError(); return nullptr; } \
      cached[dev] = (int*)p;                                                         \
    }                                                                                \
    return cached[dev];                                                              \
  }

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is a per-device setting: `done` is a
// static size_t[64] of the largest size configured so far on each device.
template <typename F>
static inline cudaError_t q_ensure_smem(F* kernel, size_t bytes, size_t* done) {
  const int dev = q_device_index();
  if (dev < 0) return cudaErrorInvalidDevice;
  if (bytes <= done[dev]) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) done[dev] = bytes;
  return e;
}

// The step's last kernel copies the four status words (see q_device_status) to out, so
// that the host can read them with the tokens instead of synchronising the device.
struct StatusTap {
  const int* src[4];
  int32_t* out;      // null = no copy
};
int q_logits_argmax_tap(const float* d_branch, const q_gemm_plan_t* plan, void* d_logits, float* d_val,
                        int32_t* d_idx, int64_t* d_tokens, int32_t* d_pos, int pos_inc,
                        void* d_block_scratch, int rows, int vocab, int vocab_offset, StatusTap tap,
                        void* stream);
int q_argmax_merge_tap(const float* d_val, const int32_t* d_idx, int shards, int rows, int64_t* d_tokens,
                       int32_t* d_pos, int pos_inc, StatusTap tap, void* stream);
int q_argmax_merge_peers_tap(const float* d_val, const int32_t* d_idx, const q_peers_t* peers, int rows,
                             int64_t* d_tokens, int32_t* d_pos, int pos_inc, StatusTap tap, void* stream);

// Split-K plan over at most `max_workers` CTAs (q_gemm_plan uses the SM count), and the
// launch of a projection on a plan the caller already holds.
int q_gemm_plan_workers(int M, int N, int K, int max_workers, q_gemm_plan_t* plan);
int q_gemm_launch_planned(const void* d_x, const void* d_w_tiled, float* d_partials,
                          const q_gemm_plan_t* plan, void* stream);
// The same for the tcgen05 kernel (plan from q_gemm_tc_plan, weight in the 128 x 64 tiling).
int q_gemm_tc_launch(const void* d_x, const void* d_w_tc, float* d_partials, const q_gemm_plan_t* plan,
                     void* stream);

// q_swiglu on partials whose columns are in q_gemm_swiglu's interleaved gate/up order
// (interleaved = 1) or in [gate | up] order (0).
int q_swiglu_layout(const float* d_branch, const q_gemm_plan_t* plan, void* d_out, int rows, int inter,
                    int interleaved, void* stream);

// Measurement aid: a per-launch record {first CTA start, first CTA past the dependency
// wait, last warp end, last CTA start} in %globaltimer ns. Launchers pass q_tl_next(kind) as
// the kernel's last argument: null unless option "timeline" is on, else the next record.
enum q_tl_kind { Q_TL_GEMM = 1, Q_TL_GEMM_TC = 2, Q_TL_ATTENTION = 3, Q_TL_ADD_NORM = 4, Q_TL_SWIGLU = 5,
                 Q_TL_EMBED = 6, Q_TL_ARGMAX = 7, Q_TL_PEER_ADD_NORM = 8 };
unsigned long long* q_tl_next(int kind);

// This rank's view of the tensor-parallel peers (q_peers_t with the pointers checked).
struct PeerView {
  int rank, world;
  float* recv[Q_MAX_PEERS];      // rank r's receive area [2 halves][world][rows][cols] pairs of 8 bytes
  uint32_t* flags[Q_MAX_PEERS];
  uint32_t* epoch;     // [0] call counter of the add+norm exchange, [1] its ticket, [2] counter of the token exchange
};

int q_peer_view(const q_peers_t* peers, PeerView* out, const char* who);

// Split-K plan passed by value to consumer kernels. u == 0 means "one plain
// fp32 [rows][cols] buffer".
struct PlanView {
  int u;       // units per worker
  int C;       // chunks per group
  int gshift;  // log2(weight rows per group): 4 (stream-K units) or 7 (tcgen05 tiles)
  int nblk;    // tcgen05 plan of more than 256 rows: weight blocks per row chunk of 256 (else 0)
  long long slot_stride;  // M*N floats
};

static inline PlanView plan_view(const q_gemm_plan_t* p) {
  PlanView v;
  if (p) {
    v.u = p->units_per_worker;
    v.C = p->chunks_per_group;
    v.gshift = p->group_rows == 128 ? 7 : 4;
    v.nblk = (p->group_rows == 128 && p->M > 256) ? (p->N + 127) / 128 : 0;
    v.slot_stride = (long long)p->M * p->N;
  } else {
    v.u = 0; v.C = 0; v.gshift = 4; v.nblk = 0; v.slot_stride = 0;
  }
  return v;
}

// ---- device side ---------------------------------------------------------------
#ifdef __CUDACC__

// {value, call counter} pairs of the peer exchange: an 8-byte store is single-copy atomic, so a
// pair that carries this call's counter HAS arrived with its value.
__device__ __forceinline__ void st_pair2(void* p, float a, float b, unsigned e) {
  // two {value, counter} pairs, each element an 8-byte single-copy-atomic store
  asm volatile("st.volatile.global.v2.b64 [%0], {%1, %2};" ::"l"(p),
               "l"(((unsigned long long)e << 32) | __float_as_uint(a)),
               "l"(((unsigned long long)e << 32) | __float_as_uint(b)) : "memory");
}
__device__ __forceinline__ void ld_pair2(const void* p, unsigned long long& a, unsigned long long& b) {
  asm volatile("ld.volatile.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}

__device__ __forceinline__ void st_pair1(void* p, float a, unsigned e) {
  asm volatile("st.volatile.global.b64 [%0], %1;" ::"l"(p), "l"(((unsigned long long)e << 32) | __float_as_uint(a))
               : "memory");
}

__device__ __forceinline__ unsigned long long tl_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void tl_begin(unsigned long long* tl) {
  if (tl != nullptr && threadIdx.x == 0) {
    const unsigned long long t = tl_now();
    atomicMin(tl, t);
    atomicMax(tl + 3, t);
  }
}
__device__ __forceinline__ void tl_waited(unsigned long long* tl) {
  if (tl != nullptr && threadIdx.x == 0) atomicMin(tl + 1, tl_now());
}
// Called by every thread of the CTA that is still running at the kernel's end.
__device__ __forceinline__ void tl_end(unsigned long long* tl) {
  if (tl != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(tl + 2, tl_now());
  }
}

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Number of split-K slots that hold a partial for column n (of row `row`: plans of more than
// 256 rows count their groups per row chunk).
__device__ __forceinline__ int plan_count(const PlanView& pv, int n, int row = 0) {
  if (pv.u == 0) return 1;
  const unsigned g = ((unsigned)n >> pv.gshift) + (unsigned)(row >> 8) * (unsigned)pv.nblk;
  const unsigned C = (unsigned)pv.C, u = (unsigned)pv.u;
  const unsigned first = (g * C) / u;
  const unsigned last = ((g + 1) * C - 1) / u;
  return (int)(last - first + 1);
}

// Sum of the partial slots of element (m, n) in slot order 0..count-1. Every
// partial buffer has at least two slots, so slot 1 is loaded unconditionally
// (in parallel with slot 0) and only used when it holds data.
__device__ __forceinline__ float plan_sum(const float* __restrict__ P, const PlanView& pv,
                                          long long idx, int n, int row = 0) {
  float s = P[idx];
  if (pv.u != 0) {
    const float s1 = P[idx + pv.slot_stride];
    const int cnt = plan_count(pv, n, row);
    if (cnt > 1) s += s1;
    for (int k = 2; k < cnt; ++k) s += P[idx + k * pv.slot_stride];
  }
  return s;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; `red` is shared float[32]. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// Byte offset of element (token r, dim d) inside one swizzled 64x128 bf16 page tile.
__device__ __forceinline__ int kv_tile_offset_bytes(int r, int d) {
  int chunk = (d >> 3) ^ (r & 7);
  return r * 256 + chunk * 16 + (d & 7) * 2;
}

#endif  // __CUDACC__
