// Split-K weight-streaming GEMM for at most 64 activation rows.
//
// Y[M,N] = X[M,K] . W[N,K]^T with bf16 operands and fp32 accumulation, written
// as fp32 partial sums that the fused consumers add and round once
// (reference: engine/kernels/skinny_gemm.py:28-46 computes the same partials
// with a fixed split count; the decomposition here is different).
//
// The weight matrix is cut into units of 16 rows x 32 k (1 KB). Units are
// numbered group-major and every warp of the grid streams ONE contiguous run of
// `u` units, so all warps move the same number of bytes whatever N and K are.
// A warp feeds the weight rows to the tensor cores as the A operand of
// mma.m16n8k16 straight from its 128-bit global loads (no shared-memory
// staging): lane (g,t) loads 16 bytes of row g and of row g+8 at k offset 8t and
// uses them for two MMAs; the k positions inside an MMA are a fixed permutation
// of the real ones, and the activation fragment is loaded with the same
// permutation, so the dot products are unchanged. The batch rows sit in the MMA
// N dimension (8 per tile), which keeps tensor-core padding waste negligible.
//
// A ring of DEPTH chunks per warp is kept in flight. The first DEPTH weight
// chunks are requested BEFORE griddepcontrol.wait, i.e. while the kernel that
// produces X is still running.
#include "common.cuh"

namespace {

constexpr int WARPS = 16;      // warps per CTA
constexpr int DEPTH = 6;       // weight chunks in flight per warp

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT = number of 8-row activation tiles (M <= 8*NT).
template <int NT>
__global__ void __launch_bounds__(WARPS * 32)
k_gemm_streamk(const bf16* __restrict__ X, const bf16* __restrict__ W, float* __restrict__ P,
               int M, int N, int K, int C, long long total, int u) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const long long w = (long long)blockIdx.x * WARPS + (threadIdx.x >> 5);
  const long long start = w * u;
  long long end = start + u;
  if (end > total) end = total;
  if (start >= total) {
    pdl_wait();
    return;
  }
  const int n_units = (int)(end - start);

  // Position of the prefetch cursor (unit start+issued): group and chunk.
  int pf_group = (int)(start / C);
  int pf_chunk = (int)(start - (long long)pf_group * C);

  uint4 ra[DEPTH], rb[DEPTH];
  auto issue = [&](int slot) {
    int r0 = pf_group * 16 + g;
    int r1 = r0 + 8;
    r0 = r0 < N ? r0 : N - 1;   // ragged last group: reload a valid row, masked at store
    r1 = r1 < N ? r1 : N - 1;
    const bf16* p0 = W + (size_t)r0 * K + pf_chunk * 32 + t * 8;
    const bf16* p1 = W + (size_t)r1 * K + pf_chunk * 32 + t * 8;
    ra[slot] = ldg_stream(p0);
    rb[slot] = ldg_stream(p1);
    if (++pf_chunk == C) { pf_chunk = 0; ++pf_group; }
  };

#pragma unroll
  for (int j = 0; j < DEPTH; ++j)
    if (j < n_units) issue(j);

  pdl_wait();   // X (and the partial buffer's previous readers) are complete from here on

  int group = (int)(start / C);
  int chunk = (int)(start - (long long)group * C);
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

  const long long slot_stride = (long long)M * N;

  for (int base = 0; base < n_units; base += DEPTH) {
#pragma unroll
    for (int j = 0; j < DEPTH; ++j) {
      const int i = base + j;
      if (i < n_units) {
        const uint4 a = ra[j], b = rb[j];
        if (i + DEPTH < n_units) issue(j);
        const int koff = chunk * 32 + t * 8;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int m = nt * 8 + g;
          uint4 x = make_uint4(0, 0, 0, 0);
          if (m < M) x = ldg_cached(X + (size_t)m * K + koff);
          mma16816(acc[nt], a.x, b.x, a.y, b.y, x.x, x.y);
          mma16816(acc[nt], a.z, b.z, a.w, b.w, x.z, x.w);
        }
        const bool last_of_group = (chunk == C - 1);
        if (last_of_group || i == n_units - 1) {
          // flush this segment: slot = worker index relative to the group's first worker
          const long long first = ((long long)group * C) / u;
          float* out = P + (w - first) * slot_stride;
          const int n0 = group * 16 + g;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const int m0 = nt * 8 + 2 * t;
            if (m0 < M) {
              if (n0 < N) out[(size_t)m0 * N + n0] = acc[nt][0];
              if (n0 + 8 < N) out[(size_t)m0 * N + n0 + 8] = acc[nt][2];
            }
            if (m0 + 1 < M) {
              if (n0 < N) out[(size_t)(m0 + 1) * N + n0] = acc[nt][1];
              if (n0 + 8 < N) out[(size_t)(m0 + 1) * N + n0 + 8] = acc[nt][3];
            }
            acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
          }
        }
        if (last_of_group) { chunk = 0; ++group; } else { ++chunk; }
      }
    }
  }
}

// Sums the slots of each element into one fp32 value (tensor-parallel path).
__global__ void k_reduce_partials(const float* __restrict__ P, float* __restrict__ out,
                                  PlanView pv, int M, int N) {
  pdl_launch_dependents();
  pdl_wait();
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = (long long)M * N;
  if (i >= total) return;
  int n = (int)(i % N);
  out[i] = plan_sum(P, pv, i, n);
}

}  // namespace

extern "C" int q_gemm_plan(int M, int N, int K, q_gemm_plan_t* plan) {
  Q_CHECK_ARG(plan != nullptr, "q_gemm_plan: null plan");
  Q_CHECK_ARG(M >= 1 && M <= Q_MAX_ROWS, "q_gemm_plan: rows %d outside 1..%d", M, Q_MAX_ROWS);
  Q_CHECK_ARG(N >= 1 && K >= 32 && K % 32 == 0,
              "q_gemm_plan: need N >= 1 and K a positive multiple of 32 (N=%d K=%d)", N, K);
  int sms = q_sm_count();
  if (sms <= 0) return Q_ERR_CUDA;
  const int C = K / 32;
  const int groups = (N + 15) / 16;
  const long long total = (long long)groups * C;
  long long warps = (long long)sms * WARPS;
  long long u = (total + warps - 1) / warps;
  if (u < 1) u = 1;
  long long workers = (total + u - 1) / u;
  // slots = max over groups of the number of workers that touch the group
  int slots = 1;
  for (long long gidx = 0; gidx < groups; ++gidx) {
    long long first = (gidx * C) / u;
    long long last = ((gidx + 1) * C - 1) / u;
    int cnt = (int)(last - first + 1);
    if (cnt > slots) slots = cnt;
  }
  plan->M = M; plan->N = N; plan->K = K;
  plan->chunks_per_group = C;
  plan->groups = groups;
  plan->units_per_worker = (int)u;
  plan->workers = (int)workers;
  plan->slots = slots;
  plan->grid = (int)((workers + WARPS - 1) / WARPS);
  plan->block = WARPS * 32;
  return Q_OK;
}

extern "C" int q_gemm_splitk(const void* d_x, const void* d_w, float* d_partials,
                             int M, int N, int K, void* stream) {
  Q_CHECK_ARG(d_x && d_w && d_partials, "q_gemm_splitk: null pointer");
  Q_CHECK_ARG(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_w & 15) == 0,
              "q_gemm_splitk: x and w must be 16-byte aligned");
  q_gemm_plan_t p;
  int rc = q_gemm_plan(M, N, K, &p);
  if (rc) return rc;
  const long long total = (long long)p.groups * p.chunks_per_group;
  cudaStream_t s = (cudaStream_t)stream;
  const bf16* X = (const bf16*)d_x;
  const bf16* W = (const bf16*)d_w;
  cudaError_t e;
  dim3 grid(p.grid), block(p.block);
  if (M <= 8)
    e = q_launch(k_gemm_streamk<1>, grid, block, 0, s, X, W, d_partials, M, N, K,
                 p.chunks_per_group, total, p.units_per_worker);
  else if (M <= 16)
    e = q_launch(k_gemm_streamk<2>, grid, block, 0, s, X, W, d_partials, M, N, K,
                 p.chunks_per_group, total, p.units_per_worker);
  else if (M <= 32)
    e = q_launch(k_gemm_streamk<4>, grid, block, 0, s, X, W, d_partials, M, N, K,
                 p.chunks_per_group, total, p.units_per_worker);
  else
    e = q_launch(k_gemm_streamk<8>, grid, block, 0, s, X, W, d_partials, M, N, K,
                 p.chunks_per_group, total, p.units_per_worker);
  Q_CHECK_CUDA(e);
  return Q_OK;
}

extern "C" int q_reduce_partials(const float* d_partials, const q_gemm_plan_t* plan,
                                 float* d_out, void* stream) {
  Q_CHECK_ARG(d_partials && plan && d_out, "q_reduce_partials: null pointer");
  long long total = (long long)plan->M * plan->N;
  int block = 256;
  int grid = (int)((total + block - 1) / block);
  Q_CHECK_CUDA(q_launch(k_reduce_partials, dim3(grid), dim3(block), 0, (cudaStream_t)stream,
                        d_partials, d_out, plan_view(plan), plan->M, plan->N));
  return Q_OK;
}
