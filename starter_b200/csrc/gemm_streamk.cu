// Split-K weight-streaming GEMM for at most 64 activation rows, over weights
// pre-tiled at load time so that every warp streams one contiguous byte range.
//
// Y[M,N] = X[M,K] . W[N,K]^T with bf16 operands and fp32 accumulation, written
// as fp32 partial sums that the fused consumers add and round once
// (reference: engine/kernels/skinny_gemm.py:28-46 computes the same partials
// with a fixed split count over row-major weights; packing weights at load time
// is what engine/mlp.py:12-15 and engine/qk_norm_rope.py:25-30 do for gate|up and
// q|k|v; the tiling here goes further).
//
// Tiled layout ("units"). The matrix is cut into units of 16 rows x 32 k = 1 KB,
// stored group-major (16-row group, then k chunk). Inside a unit the bytes are in
// the order the tensor-core fragments want them: 32 pieces of 16 B for rows
// 0..7 (piece l = row l/4, k offset 8*(l%4)), then 32 pieces for rows 8..15.
// Rows past N are stored as zeros, so there is no ragged edge.
//
// Decomposition. CTA c owns the contiguous run of U units [c*U, (c+1)*U) (same
// bytes for every CTA, one CTA per SM); warp w of the CTA owns the contiguous
// 1/8 of that run. A warp therefore streams ONE linear byte range: lane 0 brings
// it into a private 2-stage shared-memory ring with cp.async.bulk (TMA, 8 KB per
// copy, mbarrier transaction counts), all lanes read back their own 2 x 16 B per
// unit as the A fragment of two mma.m16n8k16 (the k positions inside an MMA are a
// fixed permutation of the real ones and the activation fragment uses the same
// permutation). The batch rows sit in the MMA N dimension (8 per tile).
//
// A warp that covers a 16-row group completely writes that group's result
// straight to slot 0. The (at most two) ragged ends of a warp's run go to shared
// memory and are added across the CTA's warps after one __syncthreads, so a group
// receives one partial per CTA that touches it: at most 2 slots for all Qwen3-4B
// shapes.
//
// Overlap with the producer of X. Before griddepcontrol.wait every warp fills its ring:
// weights do not depend on the previous kernel, so HBM keeps streaming while the kernel
// that produces X is still running (with the add+norm prologue only the first stage is
// requested that early, see below). One CTA per SM: a second co-resident CTA measured
// slower, its copies queue in front of the running kernel's. An L2 prefetch of the run
// (cp.async.bulk.prefetch.L2) is an option that is off by default for the same reason.
//
// Every mbarrier wait is bounded; a wait that runs out sets the status word of
// this file (read by q_device_status) and the warp stops consuming.
#include "common.cuh"

extern int g_gemm_prefetch_kb;   // set through q_set_option
extern int g_gemm_debug_flags;   // set through q_set_option: 4 = record the per-CTA trace
extern int g_gemm_trace_launch;  // >= 0: only that GEMM launch (counted from when it was set) records
extern int g_gemm_launches;
extern int g_peer_wait_iters;     // q_set_option "peer_wait_iters"

namespace {

#ifndef QG_WARPS
#define QG_WARPS 8
#endif
#ifndef QG_STAGE_UNITS
#define QG_STAGE_UNITS 8
#endif
#ifndef QG_STAGES
#define QG_STAGES 2
#endif
constexpr int WARPS = QG_WARPS;
constexpr int THREADS = WARPS * 32;
constexpr int STAGE_UNITS = QG_STAGE_UNITS;  // units (KB) per bulk copy
constexpr int STAGES = QG_STAGES;
constexpr unsigned WAIT_LIMIT = 1u << 22;

__device__ int g_gemm_status[4];
// Measurement aid (debug flag 4): per CTA {smid, start, past the dependency wait, prologue done,
// first stage landed, loop end, exit, prologue operands arrived} in ns.
__device__ unsigned long long g_gemm_trace[256 * 8];

__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned smid() {
  unsigned s;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(s));
  return s;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (it > 256) __nanosleep(32);
  }
  return false;
}
// Weights are read once per step and are far larger than L2: their lines are marked
// evict-first so that they do not push out what the step re-reads (partials, residual,
// gains, rotary rows, the KV pages of short contexts).
__device__ __forceinline__ uint64_t stream_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
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

// silu(gate) * up with the reference's rounding points (engine/kernels/decode_fused.py:161-169):
// both sums round to bf16, silu rounds, the product rounds.
__device__ __forceinline__ bf16 swiglu_bf16(float gate, float up) {
  const float gt = bf16_round(gate), u = bf16_round(up);
  return __float2bfloat16_rn(bf16_round(gt / (1.0f + expf(-gt))) * u);
}

// One partial of output element (m, n), slot `slot`, to every rank's receive area (PEER == 1).
__device__ __forceinline__ void peer_push(const PeerView& pw, unsigned e, int slot, int M, int N, int m, int n,
                                          float v) {
  const size_t idx = ((((size_t)(e & 1u) * pw.world + pw.rank) * 2 + slot) * M + m) * N + n;
#pragma unroll
  for (int r = 0; r < Q_MAX_PEERS; ++r)
    if (r < pw.world) st_pair1(reinterpret_cast<char*>(pw.recv[r]) + idx * 8, v, e);
}

// Optional prologue: instead of reading a ready activation matrix, every CTA builds it
// from the previous projection's partials: resid_out = bf16(resid_in + bf16(sum of
// slots)); X = RMSNorm(resid_out) * gain (engine/kernels/decode_fused.py:19-44). All CTAs
// compute the same rows into their shared memory; CTA 0 alone stores resid_out (a different
// buffer than resid_in, which the other CTAs are still reading). This removes the
// single-CTA add+norm kernel between two GEMMs, and the prologue's one memory round trip
// runs while the ring is filling.
struct NormPrologue {
  const float* prev;          // partials of the previous projection [slots][M][K]
  PlanView prev_plan;
  const bf16* resid_in;       // [M][K]
  bf16* resid_out;            // [M][K]
  const bf16* gain;           // [K]
  float eps;
};

// NT = number of 8-row activation tiles (M <= 8*NT). PRO: activation rows come from the
// add+norm prologue (in shared memory) instead of global memory. ACT: the weight is a
// gate|up pair interleaved in blocks of 8 rows (rows 16i..16i+7 = gate rows 8i..8i+7, rows
// 16i+8..16i+15 = the matching up rows), every CTA owns WHOLE 16-row groups, and the
// epilogue writes silu(gate) * up as bf16 [M][N/2] into P instead of fp32 partials
// (engine/kernels/skinny_gemm.py:49-72): one MMA tile holds a gate row in c0/c1 and its up
// row in c2/c3 of the same thread, so no exchange is needed.
//
// PEER (tensor parallel over peer memory, 1-8 rows): 1 = the epilogue does not write partial
// slots but stores every partial, paired with the call counter, into the receive area of
// EVERY rank (its own too): [half][rank][2 slots][M][N] pairs of 8 bytes; 2 = the add+norm
// prologue does not read local slots but polls (bounded) the own receive area for all ranks'
// pairs of the previous projection and adds them in (rank, slot) order, and the last CTA
// through the prologue publishes the new call counter. The two are the halves of one
// exchange: the projection before pushes, the projection after polls, no kernel in between.
// Halves alternate with the counter, as in k_add_rmsnorm_peers.
template <int NT, bool PRO, bool ACT, int SU, int PEER = 0>
__global__ void __launch_bounds__(THREADS, (WARPS * STAGES * SU * 1024 <= 100 * 1024 ? 2 : 1))
k_gemm_streamk(const bf16* __restrict__ X, const unsigned char* __restrict__ Wt,
               float* __restrict__ P, int M, int N, int K, int C, int total, int U,
               int prefetch_bytes, int dbg, NormPrologue pro, PeerView pw, int peer_wait,
               unsigned long long* tl) {
  extern __shared__ __align__(1024) unsigned char smem[];
  float* red = reinterpret_cast<float*>(smem + WARPS * STAGES * SU * 1024);            // [WARPS][2][NT*128]
  int* tags = reinterpret_cast<int*>(red + WARPS * 2 * NT * 128);      // [WARPS][2] group or -1
  uint64_t* bars = reinterpret_cast<uint64_t*>(tags + WARPS * 2);      // [WARPS][STAGES]
  bf16* xsm = reinterpret_cast<bf16*>(bars + WARPS * STAGES);          // PRO: [M][K] activations
  const int XLD = PRO ? K + 32 : K;        // row stride; +64 B keeps the 8 rows of a fragment off one bank
  float* psum = reinterpret_cast<float*>(xsm + (PRO ? (size_t)M * XLD : 0));   // PRO: 32 floats

  tl_begin(tl);
  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const bool trace = (dbg & 4) && tid == 0 && blockIdx.x < 256;
  if (trace) {
    g_gemm_trace[blockIdx.x * 8 + 0] = smid();
    g_gemm_trace[blockIdx.x * 8 + 1] = gtime();
  }
  // stream-K: units [c U, (c+1) U). ACT: groups [c G / grid, (c+1) G / grid) with G = total / C.
  const int cs = ACT ? (int)(((long long)blockIdx.x * (total / C)) / gridDim.x) * C : blockIdx.x * U;
  const int ce = ACT ? (int)(((long long)(blockIdx.x + 1) * (total / C)) / gridDim.x) * C : min(total, cs + U);
  const int len = ce > cs ? ce - cs : 0;
  // the warp's contiguous run [ws, we)
  const int ws = cs + (int)(((long long)warp * len) / WARPS);
  const int we = cs + (int)(((long long)(warp + 1) * len) / WARPS);
  const int n_units = we - ws;
  const unsigned char* src = Wt + (size_t)ws * 1024;

  const uint32_t ring = smem_u32(smem) + warp * (STAGES * SU * 1024);
  const uint32_t bar0 = smem_u32(&bars[warp * STAGES]);
  const int n_stages = (n_units + SU - 1) / SU;
  const uint64_t policy = stream_policy();

  if (lane == 0) {
    if (prefetch_bytes > 0 && n_units > 0)
      l2_prefetch(src, (uint32_t)min(n_units * 1024, prefetch_bytes));
    for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // With the prologue only the first stage is requested here: the prologue's few KB of
    // dependent loads would otherwise queue behind the whole ring's worth of bulk copies
    // (measured: 3.5 us instead of ~1.5 us from the dependency wait to the first MMA).
    for (int s = 0; s < (PRO ? ((dbg & 8) ? 0 : 1) : STAGES) && s < n_stages; ++s) {
      const uint32_t bytes = (uint32_t)min(SU, n_units - s * SU) * 1024u;
      mbar_expect_tx(bar0 + 8 * s, bytes);
      bulk_g2s(ring + s * (SU * 1024), src + (size_t)s * SU * 1024, bytes, bar0 + 8 * s,
               policy);
    }
  }
  if (lane < 2) tags[warp * 2 + lane] = -1;
  __syncwarp();

  // The norm gains do not depend on the previous kernel: asked for before the wait.
  uint2 gn[3] = {make_uint2(0, 0), make_uint2(0, 0), make_uint2(0, 0)};
  if (PRO) {
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int col = 4 * tid + j * 1024;
      gn[j] = *reinterpret_cast<const uint2*>(pro.gain + (col < K ? col : 0));
    }
  }

  pdl_wait();   // X and the previous readers of P are complete from here on
  tl_waited(tl);
  if (trace) g_gemm_trace[blockIdx.x * 8 + 2] = gtime();

  // call counter of the peer exchange this launch takes part in (same in every CTA: the counter
  // word moves only when all CTAs of a polling launch are through their prologue)
  unsigned pe = 0;
  if (PEER != 0) pe = *reinterpret_cast<volatile unsigned*>(pw.epoch) + 1u;
  if (PRO) {
    // add + norm: thread t owns columns 4t..4t+3 (+1024 j); all loads first
    constexpr int VB = 3;                       // K <= 3072 (checked on the host)
    bool ok = true;                             // PEER == 2: no wait for a peer has run out yet
    for (int m = 0; m < M; ++m) {
      float4 s0[VB], s1[VB];
      uint2 xr[VB];
#pragma unroll
      for (int j = 0; j < VB; ++j) {
        const int col = 4 * tid + j * 1024;
        const int cc = col < K ? col : 0;
        if (PEER != 2) {
          s0[j] = *reinterpret_cast<const float4*>(pro.prev + (size_t)m * K + cc);
          s1[j] = pro.prev_plan.u != 0
                      ? *reinterpret_cast<const float4*>(pro.prev + (size_t)m * K + cc + pro.prev_plan.slot_stride)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        xr[j] = *reinterpret_cast<const uint2*>(pro.resid_in + (size_t)m * K + cc);
      }
      if (m == 0 && lane == 0) {
        // the rest of the ring, behind the prologue's loads in the memory system's queues
        for (int s = (dbg & 8) ? 0 : 1; s < STAGES && s < n_stages; ++s) {
          const uint32_t bytes = (uint32_t)min(SU, n_units - s * SU) * 1024u;
          mbar_expect_tx(bar0 + 8 * s, bytes);
          bulk_g2s(ring + s * (SU * 1024), src + (size_t)s * SU * 1024, bytes,
                   bar0 + 8 * s, policy);
        }
      }
      // PEER == 2: every rank's pairs of this thread's columns - slot 0 and, where the previous
      // plan has one for the group, slot 1 - two ranks' worth of loads in flight per poll, the
      // sums added in (rank, slot) order.
      float peer_acc[VB][4];
      if (PEER == 2) {
#pragma unroll
        for (int j = 0; j < VB; ++j) peer_acc[j][0] = peer_acc[j][1] = peer_acc[j][2] = peer_acc[j][3] = 0.f;
        int extra_j[VB];
#pragma unroll
        for (int j = 0; j < VB; ++j) {
          const int col = 4 * tid + j * 1024;
          extra_j[j] = col < K ? plan_count(pro.prev_plan, col) - 1 : -1;     // -1: no column
        }
        const size_t half = (size_t)(pe & 1u) * pw.world;
        const char* mine = reinterpret_cast<const char*>(pw.recv[pw.rank]);
        for (int r0 = 0; r0 < pw.world; r0 += 2) {
          unsigned long long a[2][VB][2][2];
          bool here = false;
          for (int i = 0; ok && i < peer_wait; ++i) {
            here = true;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (r0 + q >= pw.world) break;
#pragma unroll
              for (int j = 0; j < VB; ++j) {
#pragma unroll
                for (int sl = 0; sl < 2; ++sl) {
                  a[q][j][sl][0] = a[q][j][sl][1] = 0;
                  if (sl > extra_j[j]) continue;
                  const size_t idx = (((half + (r0 + q)) * 2 + sl) * M + m) * K + (4 * tid + j * 1024);
                  unsigned long long b0, b1, b2, b3;
                  ld_pair2(mine + idx * 8, b0, b1);
                  ld_pair2(mine + idx * 8 + 16, b2, b3);
                  here = here && (unsigned)(b0 >> 32) == pe && (unsigned)(b1 >> 32) == pe &&
                         (unsigned)(b2 >> 32) == pe && (unsigned)(b3 >> 32) == pe;
                  a[q][j][sl][0] = (b0 & 0xffffffffull) | (b1 << 32);
                  a[q][j][sl][1] = (b2 & 0xffffffffull) | (b3 << 32);
                }
              }
            }
            if (here) break;
            if (i > 64) __nanosleep(i > 65536 ? 2000 : (i > 4096 ? 400 : 40));
          }
          if (!here) { ok = false; atomicExch(&g_gemm_status[0], 4); }
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            if (r0 + q >= pw.world) break;
#pragma unroll
            for (int j = 0; j < VB; ++j)
#pragma unroll
              for (int sl = 0; sl < 2; ++sl) {
                if (sl > extra_j[j]) continue;
                peer_acc[j][0] += __uint_as_float((unsigned)a[q][j][sl][0]);
                peer_acc[j][1] += __uint_as_float((unsigned)(a[q][j][sl][0] >> 32));
                peer_acc[j][2] += __uint_as_float((unsigned)a[q][j][sl][1]);
                peer_acc[j][3] += __uint_as_float((unsigned)(a[q][j][sl][1] >> 32));
              }
          }
        }
      }
      float tot[VB][4];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VB; ++j) {
        const int col = 4 * tid + j * 1024;
        if (col < K) {
          const int extra = plan_count(pro.prev_plan, col) - 1;
          float s[4] = {0.f, 0.f, 0.f, 0.f};
          if (PEER == 2) {
            s[0] = peer_acc[j][0]; s[1] = peer_acc[j][1]; s[2] = peer_acc[j][2]; s[3] = peer_acc[j][3];
          } else {
            s[0] = s0[j].x; s[1] = s0[j].y; s[2] = s0[j].z; s[3] = s0[j].w;
            if (extra > 0) { s[0] += s1[j].x; s[1] += s1[j].y; s[2] += s1[j].z; s[3] += s1[j].w; }
            for (int k = 2; k <= extra; ++k) {
              const float4 sk = *reinterpret_cast<const float4*>(pro.prev + (size_t)m * K + col +
                                                                 (long long)k * pro.prev_plan.slot_stride);
              s[0] += sk.x; s[1] += sk.y; s[2] += sk.z; s[3] += sk.w;
            }
          }
          const float r[4] = {bf_lo(xr[j].x), bf_hi(xr[j].x), bf_lo(xr[j].y), bf_hi(xr[j].y)};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            tot[j][e] = bf16_round(r[e] + bf16_round(s[e]));
            ss += tot[j][e] * tot[j][e];
          }
        }
      }
      if (trace && m == 0) g_gemm_trace[blockIdx.x * 8 + 7] = gtime();    // operands arrived
      ss = block_sum(ss, psum);
      const float inv = rsqrtf(ss / (float)K + pro.eps);
#pragma unroll
      for (int j = 0; j < VB; ++j) {
        const int col = 4 * tid + j * 1024;
        if (col < K) {
          const float g4[4] = {bf_lo(gn[j].x), bf_hi(gn[j].x), bf_lo(gn[j].y), bf_hi(gn[j].y)};
          uint2 ro, xo;
          ro.x = pack_bf16(tot[j][0], tot[j][1]);
          ro.y = pack_bf16(tot[j][2], tot[j][3]);
          xo.x = pack_bf16(bf16_round(tot[j][0] * inv) * g4[0], bf16_round(tot[j][1] * inv) * g4[1]);
          xo.y = pack_bf16(bf16_round(tot[j][2] * inv) * g4[2], bf16_round(tot[j][3] * inv) * g4[3]);
          *reinterpret_cast<uint2*>(xsm + (size_t)m * XLD + col) = xo;
          if (blockIdx.x == 0) *reinterpret_cast<uint2*>(pro.resid_out + (size_t)m * K + col) = ro;
        }
      }
    }
    __syncthreads();
    if (PEER == 2 && tid == 0) {
      // every CTA has read the counter word before it takes a ticket: the last one moves it on
      const unsigned ticket = atomicAdd(pw.epoch + 1, 1u);
      if (ticket == gridDim.x - 1) {
        pw.epoch[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile unsigned*>(pw.epoch) = pe;
      }
    }
  }
  if (trace) g_gemm_trace[blockIdx.x * 8 + 3] = gtime();

  // Warm L1 with the activation rows (every CTA reads all of X, a few KB).
  if (!PRO) {
    const int lines = (M * K * 2 + 127) >> 7;
    if (lines <= 320)
      for (int i = tid; i < lines; i += THREADS)
        asm volatile("prefetch.global.L1 [%0];" ::"l"(reinterpret_cast<const char*>(X) + ((size_t)i << 7)));
  }

  // mma.sync has a long latency on this part (~280 cycles): consecutive MMAs go to
  // SETS independent accumulators, added when a 16-row group (or the run) ends.
  constexpr int SETS = NT == 1 ? 8 : (NT == 2 ? 4 : 2);   // <= 2 * XB
  float acc[SETS][NT][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[s][i][0] = acc[s][i][1] = acc[s][i][2] = acc[s][i][3] = 0.f;
  int group = ws / C;
  int chunk = ws - group * C;
  int seg_first_chunk = chunk;          // first chunk of the current segment
  int n_boundary = 0, units_done = 0;
  bool alive = true;
  constexpr int XB = NT == 1 ? 8 : (NT == 2 ? 4 : (NT == 4 ? 4 : 2));   // units per activation batch
  // activation row pointers of this lane (row nt*8+g, k offset 8t), null past M
  const bf16* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + g;
    xrow[nt] = m < M ? (PRO ? xsm : X) + (size_t)m * XLD + t * 8 : nullptr;
  }

  for (int st = 0; st < n_stages && alive; ++st) {
    const int sidx = st % STAGES;
    if (!mbar_wait(bar0 + 8 * sidx, (st / STAGES) & 1)) {
      atomicExch(&g_gemm_status[0], 1);
      alive = false;
      break;
    }
    if (trace && st == 0) g_gemm_trace[blockIdx.x * 8 + 4] = gtime();
    const int in_stage = min(SU, n_units - st * SU);
    uint32_t sbase = ring + sidx * (SU * 1024) + lane * 16;
    int done = 0;
    while (done < in_stage) {
      // up to XB units that lie inside one 16-row group; their activation fragments are
      // requested together so that the (L1/L2) latencies overlap, then the MMAs run
      const int n = min(min(in_stage - done, C - chunk), XB);
      uint4 xs[XB][NT];
#pragma unroll
      for (int j = 0; j < XB; ++j) {
        const int koff = (chunk + j) * 32;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          xs[j][nt] = make_uint4(0, 0, 0, 0);
          if (j < n && xrow[nt] != nullptr)
            xs[j][nt] = PRO ? *reinterpret_cast<const uint4*>(xrow[nt] + koff) : ldg_cached(xrow[nt] + koff);
        }
      }
#pragma unroll
      for (int j = 0; j < XB; ++j) {
        if (j < n) {
          const uint4 a = lds128(sbase + j * 1024), b = lds128(sbase + j * 1024 + 512);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 x = xs[j][nt];
            mma16816(acc[(2 * j) % SETS][nt], a.x, b.x, a.y, b.y, x.x, x.y);
            mma16816(acc[(2 * j + 1) % SETS][nt], a.z, b.z, a.w, b.w, x.z, x.w);
          }
        }
      }
      done += n; chunk += n; units_done += n; sbase += n * 1024;
      const bool group_end = (chunk == C);
      if (group_end || units_done == n_units) {
        float tot[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float v = 0.f;
#pragma unroll
            for (int s = 0; s < SETS; ++s) { v += acc[s][nt][e]; acc[s][nt][e] = 0.f; }
            tot[nt][e] = v;
          }
        if (group_end && seg_first_chunk == 0) {
          // the warp covered the whole group: it is the only contributor (slot 0)
          const int n0 = group * 16 + g;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const int m0 = nt * 8 + 2 * t;
            if (ACT) {
              bf16* A = reinterpret_cast<bf16*>(P);
              const int half = N >> 1, col = group * 8 + g;
              if (col < half) {
                if (m0 < M) A[(size_t)m0 * half + col] = swiglu_bf16(tot[nt][0], tot[nt][2]);
                if (m0 + 1 < M) A[(size_t)(m0 + 1) * half + col] = swiglu_bf16(tot[nt][1], tot[nt][3]);
              }
              continue;
            }
            if (PEER == 1) {
              if (m0 < M) {
                if (n0 < N) peer_push(pw, pe, 0, M, N, m0, n0, tot[nt][0]);
                if (n0 + 8 < N) peer_push(pw, pe, 0, M, N, m0, n0 + 8, tot[nt][2]);
              }
              if (m0 + 1 < M) {
                if (n0 < N) peer_push(pw, pe, 0, M, N, m0 + 1, n0, tot[nt][1]);
                if (n0 + 8 < N) peer_push(pw, pe, 0, M, N, m0 + 1, n0 + 8, tot[nt][3]);
              }
              continue;
            }
            if (m0 < M) {
              if (n0 < N) P[(size_t)m0 * N + n0] = tot[nt][0];
              if (n0 + 8 < N) P[(size_t)m0 * N + n0 + 8] = tot[nt][2];
            }
            if (m0 + 1 < M) {
              if (n0 < N) P[(size_t)(m0 + 1) * N + n0] = tot[nt][1];
              if (n0 + 8 < N) P[(size_t)(m0 + 1) * N + n0 + 8] = tot[nt][3];
            }
          }
        } else {
          // ragged end of the run: park it in shared memory for the CTA reduction
          float* mine = red + ((size_t)warp * 2 + n_boundary) * (NT * 128);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
            *reinterpret_cast<float4*>(mine + nt * 128 + lane * 4) =
                make_float4(tot[nt][0], tot[nt][1], tot[nt][2], tot[nt][3]);
          if (lane == 0) tags[warp * 2 + n_boundary] = group;
          ++n_boundary;
        }
        seg_first_chunk = 0;
        if (group_end) { chunk = 0; ++group; }
      }
    }
    // refill the stage just consumed
    __syncwarp();
    const int nxt = st + STAGES;
    if (lane == 0 && nxt < n_stages) {
      const uint32_t bytes = (uint32_t)min(SU, n_units - nxt * SU) * 1024u;
      mbar_expect_tx(bar0 + 8 * sidx, bytes);
      bulk_g2s(ring + sidx * (SU * 1024), src + (size_t)nxt * SU * 1024, bytes,
               bar0 + 8 * sidx, policy);
    }
  }

  if (trace) g_gemm_trace[blockIdx.x * 8 + 5] = gtime();
  // ---- add the ragged ends across the CTA: one partial per (CTA, group) ----
  __syncthreads();
  // The warp that holds the FIRST parked entry of a group adds all entries of that
  // group in fixed order and writes the CTA's partial of the group.
  const long long slot_stride = (long long)M * N;
  for (int mine = warp * 2; mine < warp * 2 + 2; ++mine) {
    const int gg = tags[mine];
    if (gg < 0) continue;
    bool fresh = true;
    for (int s2 = 0; s2 < mine; ++s2) fresh = fresh && (tags[s2] != gg);
    if (!fresh) continue;
    const unsigned first = ACT ? blockIdx.x : ((unsigned)gg * (unsigned)C) / (unsigned)U;
    float* out = P + (long long)((int)blockIdx.x - (int)first) * slot_stride;
    const int n0 = gg * 16 + g;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s2 = mine; s2 < WARPS * 2; ++s2) {
        if (tags[s2] == gg) {
          const float4 v = *reinterpret_cast<const float4*>(red + (size_t)s2 * (NT * 128) + nt * 128 + lane * 4);
          sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
      }
      const int m0 = nt * 8 + 2 * t;
      if (ACT) {
        bf16* A = reinterpret_cast<bf16*>(P);
        const int half = N >> 1, col = gg * 8 + g;
        if (col < half) {
          if (m0 < M) A[(size_t)m0 * half + col] = swiglu_bf16(sum.x, sum.z);
          if (m0 + 1 < M) A[(size_t)(m0 + 1) * half + col] = swiglu_bf16(sum.y, sum.w);
        }
        continue;
      }
      if (PEER == 1) {
        const int slot = (int)blockIdx.x - (int)first;
        if (m0 < M) {
          if (n0 < N) peer_push(pw, pe, slot, M, N, m0, n0, sum.x);
          if (n0 + 8 < N) peer_push(pw, pe, slot, M, N, m0, n0 + 8, sum.z);
        }
        if (m0 + 1 < M) {
          if (n0 < N) peer_push(pw, pe, slot, M, N, m0 + 1, n0, sum.y);
          if (n0 + 8 < N) peer_push(pw, pe, slot, M, N, m0 + 1, n0 + 8, sum.w);
        }
        continue;
      }
      if (m0 < M) {
        if (n0 < N) out[(size_t)m0 * N + n0] = sum.x;
        if (n0 + 8 < N) out[(size_t)m0 * N + n0 + 8] = sum.z;
      }
      if (m0 + 1 < M) {
        if (n0 < N) out[(size_t)(m0 + 1) * N + n0] = sum.y;
        if (n0 + 8 < N) out[(size_t)(m0 + 1) * N + n0 + 8] = sum.w;
      }
    }
  }
  if (trace) g_gemm_trace[blockIdx.x * 8 + 6] = gtime();
  tl_end(tl);
}

// Sums the slots of each element into one fp32 value (tensor-parallel path).
__global__ void k_reduce_partials(const float* __restrict__ P, float* __restrict__ out,
                                  PlanView pv, int M, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)M * N;
  if ((N & 3) == 0) {
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    const int n = (int)(i % N);
    const float4 a = *reinterpret_cast<const float4*>(P + i);
    const float4 b = pv.u != 0 ? *reinterpret_cast<const float4*>(P + i + pv.slot_stride)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
    const int extra = plan_count(pv, n, (int)(i / N)) - 1;
    float4 s = a;
    if (extra > 0) { s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w; }
    // slots 2..9 are requested together (the tcgen05 plan splits long-K projections ~10 ways)
    float4 t8[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      t8[k] = (k + 2 <= extra) ? *reinterpret_cast<const float4*>(P + i + (long long)(k + 2) * pv.slot_stride)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k + 2 <= extra) { s.x += t8[k].x; s.y += t8[k].y; s.z += t8[k].z; s.w += t8[k].w; }
    for (int k = 10; k <= extra; ++k) {
      const float4 t = *reinterpret_cast<const float4*>(P + i + (long long)k * pv.slot_stride);
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    *reinterpret_cast<float4*>(out + i) = s;
    return;
  }
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int n = (int)(i % N);
  out[i] = plan_sum(P, pv, i, n, (int)(i / N));
}

// Row-major [N][K] <-> tiled units. One thread per 16-byte piece of the tiled side.
__global__ void k_pack_weight(const uint4* __restrict__ src, uint4* __restrict__ dst, int N, int K,
                              int C, long long pieces, int to_tiled) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  const long long unit = i >> 6;
  const int piece = (int)(i & 63);
  const int half = piece >> 5, lane = piece & 31;
  const int group = (int)(unit / C), chunk = (int)(unit - (long long)group * C);
  const int row = group * 16 + half * 8 + (lane >> 2);
  const long long rm = ((long long)row * K + chunk * 32 + (lane & 3) * 8) >> 3;   // in 16-byte pieces
  if (to_tiled) {
    dst[i] = row < N ? src[rm] : make_uint4(0, 0, 0, 0);
  } else if (row < N) {
    dst[rm] = src[i];
  }
}

template <int NT, int SU = STAGE_UNITS>
constexpr int gemm_smem() {
  return WARPS * STAGES * SU * 1024 + WARPS * 2 * NT * 128 * 4 + WARPS * 2 * 4 + WARPS * STAGES * 8;
}

int debug_flags_of_this_launch() {
  if (g_gemm_trace_launch < 0) return g_gemm_debug_flags;
  return (g_gemm_launches++ == g_gemm_trace_launch ? 4 : 0) | (g_gemm_debug_flags & ~4);
}

// SU = 1 KB units per bulk copy (a warp's ring is STAGES * SU KB)
template <int NT, bool ACT, int SU = STAGE_UNITS>
cudaError_t launch_gemm(const q_gemm_plan_t& p, const bf16* X, const unsigned char* W, float* P,
                        cudaStream_t s) {
  static size_t done[64] = {0};          // the attribute is a per-device setting
  cudaError_t e0 = q_ensure_smem(k_gemm_streamk<NT, false, ACT, SU>, (size_t)gemm_smem<NT, SU>(), done);
  if (e0 != cudaSuccess) return e0;
  NormPrologue none = {};
  const int grid = ACT ? (p.groups < p.grid ? p.groups : p.grid) : p.grid;
  return q_launch(k_gemm_streamk<NT, false, ACT, SU>, dim3(grid), dim3(p.block), (size_t)gemm_smem<NT, SU>(), s, X,
                  W, P, p.M, p.N, p.K, p.chunks_per_group, p.groups * p.chunks_per_group,
                  p.units_per_worker, g_gemm_prefetch_kb * 1024 / WARPS, debug_flags_of_this_launch(), none,
                  PeerView{}, 0, q_tl_next(Q_TL_GEMM));
}

// The same launch with the peer-push epilogue (1-8 rows, no SwiGLU): partials go to every
// rank's receive area instead of P.
cudaError_t launch_gemm_push(const q_gemm_plan_t& p, const bf16* X, const unsigned char* W, const PeerView& pw,
                             cudaStream_t s) {
  static size_t done[64] = {0};
  auto kern = k_gemm_streamk<1, false, false, STAGE_UNITS, 1>;
  cudaError_t e0 = q_ensure_smem(kern, (size_t)gemm_smem<1, STAGE_UNITS>(), done);
  if (e0 != cudaSuccess) return e0;
  NormPrologue none = {};
  return q_launch(kern, dim3(p.grid), dim3(p.block), (size_t)gemm_smem<1, STAGE_UNITS>(), s, X, W, (float*)nullptr,
                  p.M, p.N, p.K, p.chunks_per_group, p.groups * p.chunks_per_group, p.units_per_worker, 0,
                  debug_flags_of_this_launch(), none, pw, 0, q_tl_next(Q_TL_GEMM));
}

template <bool ACT>
cudaError_t launch_gemm_norm(const q_gemm_plan_t& p, const unsigned char* W, float* P,
                             const NormPrologue& pro, cudaStream_t s) {
  const size_t smem = (size_t)gemm_smem<1>() + (size_t)p.M * (p.K + 32) * 2 + 32 * 4;
  static size_t done[64] = {0};
  cudaError_t e0 = q_ensure_smem(k_gemm_streamk<1, true, ACT, STAGE_UNITS>, smem, done);
  if (e0 != cudaSuccess) return e0;
  const int grid = ACT ? (p.groups < p.grid ? p.groups : p.grid) : p.grid;
  return q_launch(k_gemm_streamk<1, true, ACT, STAGE_UNITS>, dim3(grid), dim3(p.block), smem, s, (const bf16*)nullptr, W,
                  P, p.M, p.N, p.K, p.chunks_per_group, p.groups * p.chunks_per_group,
                  p.units_per_worker, 0, debug_flags_of_this_launch(), pro, PeerView{}, 0, q_tl_next(Q_TL_GEMM));
}

// ... and with the prologue that polls the receive area for all ranks' partials of the previous
// projection (pro.prev is unused, pro.prev_plan says which slots exist).
template <bool ACT>
cudaError_t launch_gemm_norm_poll(const q_gemm_plan_t& p, const unsigned char* W, float* P,
                                  const NormPrologue& pro, const PeerView& pw, cudaStream_t s) {
  const size_t smem = (size_t)gemm_smem<1>() + (size_t)p.M * (p.K + 32) * 2 + 32 * 4;
  static size_t done[64] = {0};
  auto kern = k_gemm_streamk<1, true, ACT, STAGE_UNITS, 2>;
  cudaError_t e0 = q_ensure_smem(kern, smem, done);
  if (e0 != cudaSuccess) return e0;
  const int grid = ACT ? (p.groups < p.grid ? p.groups : p.grid) : p.grid;
  return q_launch(kern, dim3(grid), dim3(p.block), smem, s, (const bf16*)nullptr, W, P, p.M, p.N, p.K,
                  p.chunks_per_group, p.groups * p.chunks_per_group, p.units_per_worker, 0,
                  debug_flags_of_this_launch(), pro, pw, g_peer_wait_iters, q_tl_next(Q_TL_GEMM));
}

}  // namespace

extern "C" int q_debug_gemm_trace(unsigned long long* out, int n_ctas) {
  Q_CHECK_ARG(out && n_ctas >= 1 && n_ctas <= 256, "q_debug_gemm_trace: bad argument");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_gemm_trace, sizeof(unsigned long long) * 8 * n_ctas));
  return Q_OK;
}

Q_DEFINE_STATUS_ADDR(q_gemm_status_addr, g_gemm_status)

extern "C" int q_gemm_plan(int M, int N, int K, q_gemm_plan_t* plan) {
  int sms = q_sm_count();
  if (sms <= 0) return Q_ERR_CUDA;
  return q_gemm_plan_workers(M, N, K, sms, plan);
}

int q_gemm_plan_workers(int M, int N, int K, int max_workers, q_gemm_plan_t* plan) {
  Q_CHECK_ARG(plan != nullptr, "q_gemm_plan: null plan");
  Q_CHECK_ARG(max_workers >= 1, "q_gemm_plan: no workers");
  Q_CHECK_ARG(M >= 1 && M <= Q_MAX_ROWS, "q_gemm_plan: rows %d outside 1..%d", M, Q_MAX_ROWS);
  Q_CHECK_ARG(N >= 1 && K >= 32 && K % 32 == 0,
              "q_gemm_plan: need N >= 1 and K a positive multiple of 32 (N=%d K=%d)", N, K);
  const int C = K / 32;
  const int groups = (N + 15) / 16;
  Q_CHECK_ARG((long long)groups * C < (1ll << 30), "q_gemm_plan: weight too large");
  const int sms = max_workers;
  const long long total = (long long)groups * C;
  long long u = (total + sms - 1) / sms;
  if (u < 1) u = 1;
  const long long workers = (total + u - 1) / u;
  // A group of C units is touched by at most ceil((C-1)/u)+1 consecutive CTAs;
  // consumers may always read two slots, so never report fewer.
  long long slots = (C - 1 + u - 1) / u + 1;
  if (slots > workers) slots = workers;
  if (slots < 2) slots = 2;
  plan->M = M; plan->N = N; plan->K = K;
  plan->chunks_per_group = C;
  plan->groups = groups;
  plan->units_per_worker = (int)u;
  plan->workers = (int)workers;
  plan->slots = (int)slots;
  plan->grid = (int)workers;
  plan->block = THREADS;
  plan->group_rows = 16;
  return Q_OK;
}

extern "C" int64_t q_packed_weight_bytes(int N, int K) {
  if (N < 1 || K < 32 || K % 32) return -1;
  return (int64_t)((N + 15) / 16) * (K / 32) * 1024;
}

static int pack_common(const void* src, void* dst, int N, int K, int to_tiled, void* stream,
                       const char* who) {
  Q_CHECK_ARG(src && dst, "%s: null pointer", who);
  Q_CHECK_ARG(N >= 1 && K >= 32 && K % 32 == 0, "%s: need N >= 1 and K a multiple of 32", who);
  Q_CHECK_ARG(((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0,
              "%s: pointers must be 16-byte aligned", who);
  const int C = K / 32;
  const long long pieces = (long long)((N + 15) / 16) * C * 64;
  const int block = 256;
  const long long grid = (pieces + block - 1) / block;
  Q_CHECK_ARG(grid < (1ll << 31), "%s: weight too large", who);
  k_pack_weight<<<(unsigned)grid, block, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, N, K,
                                                                     C, pieces, to_tiled);
  Q_CHECK_CUDA(cudaGetLastError());
  return Q_OK;
}

extern "C" int q_pack_weight(const void* d_rowmajor, void* d_tiled, int N, int K, void* stream) {
  return pack_common(d_rowmajor, d_tiled, N, K, 1, stream, "q_pack_weight");
}

extern "C" int q_unpack_weight(const void* d_tiled, void* d_rowmajor, int N, int K, void* stream) {
  return pack_common(d_tiled, d_rowmajor, N, K, 0, stream, "q_unpack_weight");
}

extern "C" int q_gemm_splitk(const void* d_x, const void* d_w_tiled, float* d_partials,
                             int M, int N, int K, void* stream) {
  Q_CHECK_ARG(d_x && d_w_tiled && d_partials, "q_gemm_splitk: null pointer");
  Q_CHECK_ARG(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_w_tiled & 15) == 0,
              "q_gemm_splitk: x and w must be 16-byte aligned");
  q_gemm_plan_t p;
  int rc = q_gemm_plan(M, N, K, &p);
  if (rc) return rc;
  return q_gemm_launch_planned(d_x, d_w_tiled, d_partials, &p, stream);
}

int q_gemm_launch_planned(const void* d_x, const void* d_w_tiled, float* d_partials,
                          const q_gemm_plan_t* plan, void* stream) {
  const q_gemm_plan_t& p = *plan;
  const int M = p.M;
  cudaStream_t s = (cudaStream_t)stream;
  const bf16* X = (const bf16*)d_x;
  const unsigned char* W = (const unsigned char*)d_w_tiled;
  cudaError_t e;
  if (M <= 8) e = launch_gemm<1, false>(p, X, W, d_partials, s);
  else if (M <= 16) e = launch_gemm<2, false>(p, X, W, d_partials, s);
  else if (M <= 32) e = launch_gemm<4, false>(p, X, W, d_partials, s);
  else e = launch_gemm<8, false>(p, X, W, d_partials, s);
  Q_CHECK_CUDA(e);
  return Q_OK;
}

// ---- projection without any allocation: partials in a library-owned static array ----
//
// Some hosts of this library must not allocate device memory at all: a serving
// loop that has handed every byte to its own pool allocator, a plugin whose
// runtime gives it buffers but forbids calls into the CUDA allocator, or code that
// runs while a stream is being captured or inside a latency-critical section,
// where cudaMalloc/cudaFree would synchronise the whole device. For them the
// split-K partials (the GEMM's only scratch memory) live in this fixed array
// instead of a caller buffer. The array costs Q_STATIC_SCRATCH_FLOATS * 4 bytes
// on every GPU that loads the library, until the process exits.
#define Q_STATIC_SCRATCH_FLOATS (2 * 8 * 20480)
static __device__ __align__(256) float g_static_partials[Q_STATIC_SCRATCH_FLOATS];

// In host code `g_static_partials` is only a handle for the runtime, not a device
// address: the real address is asked for once per device, with that device
// current, and cached.
static int static_scratch_address(float** out) {
  static float* cached[64] = {nullptr};
  int dev = -1;
  Q_CHECK_CUDA(cudaGetDevice(&dev));
  Q_CHECK_ARG(dev >= 0 && dev < 64, "q_linear_f32_static: device index %d not supported", dev);
  if (!cached[dev]) {
    void* p = nullptr;
    Q_CHECK_CUDA(cudaGetSymbolAddress(&p, g_static_partials));
    Q_CHECK_ARG(p != nullptr, "q_linear_f32_static: no address for the static scratch");
    cached[dev] = (float*)p;
  }
  *out = cached[dev];
  return Q_OK;
}

extern "C" int64_t q_static_scratch_floats(void) { return Q_STATIC_SCRATCH_FLOATS; }

extern "C" int q_linear_f32_static(const void* d_x, const void* d_w_tiled, float* d_out, int M, int N,
                                   int K, void* stream) {
  Q_CHECK_ARG(d_x && d_w_tiled && d_out, "q_linear_f32_static: null pointer");
  Q_CHECK_ALIGN(d_out, 16, "q_linear_f32_static");
  q_gemm_plan_t p;
  int rc = q_gemm_plan(M, N, K, &p);
  if (rc) return rc;
  const long long need = (long long)p.slots * M * N;
  Q_CHECK_ARG(need <= Q_STATIC_SCRATCH_FLOATS,
              "q_linear_f32_static: %d x %d output needs %lld scratch floats, the static array holds %d "
              "(use q_gemm_splitk with a caller buffer for larger shapes)",
              M, N, need, Q_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc) return rc;
  // Every slot that a consumer reads is rewritten by the GEMM of this call, so nothing
  // has to be cleared; the array keeps the last call's partials afterwards.
  rc = q_gemm_splitk(d_x, d_w_tiled, scratch, M, N, K, stream);
  if (rc) return rc;
  return q_reduce_partials(scratch, &p, d_out, stream);
}

extern "C" int q_gemm_splitk_addnorm(const void* d_resid_in, const float* d_prev, const q_gemm_plan_t* prev_plan,
                                     const void* d_gain, void* d_resid_out, const void* d_w_tiled,
                                     float* d_partials, int M, int N, int K, float eps, void* stream) {
  Q_CHECK_ARG(d_resid_in && d_prev && d_gain && d_resid_out && d_w_tiled && d_partials,
              "q_gemm_splitk_addnorm: null pointer");
  Q_CHECK_ARG(d_resid_in != d_resid_out, "q_gemm_splitk_addnorm: the residual cannot be updated in place");
  Q_CHECK_ALIGN(d_resid_in, 8, "q_gemm_splitk_addnorm"); Q_CHECK_ALIGN(d_prev, 16, "q_gemm_splitk_addnorm");
  Q_CHECK_ALIGN(d_gain, 8, "q_gemm_splitk_addnorm"); Q_CHECK_ALIGN(d_resid_out, 8, "q_gemm_splitk_addnorm");
  Q_CHECK_ALIGN(d_w_tiled, 16, "q_gemm_splitk_addnorm"); Q_CHECK_ALIGN(d_partials, 4, "q_gemm_splitk_addnorm");
  Q_CHECK_ARG(M >= 1 && M <= 8 && K % 4 == 0 && K <= 3072,
              "q_gemm_splitk_addnorm: needs 1..8 rows and K a multiple of 4 up to 3072 (M=%d K=%d)", M, K);
  if (prev_plan)
    Q_CHECK_ARG(prev_plan->M == M && prev_plan->N == K, "q_gemm_splitk_addnorm: previous plan is [%d,%d]",
                prev_plan->M, prev_plan->N);
  q_gemm_plan_t p;
  int rc = q_gemm_plan(M, N, K, &p);
  if (rc) return rc;
  NormPrologue pro;
  pro.prev = d_prev;
  pro.prev_plan = plan_view(prev_plan);
  pro.resid_in = (const bf16*)d_resid_in;
  pro.resid_out = (bf16*)d_resid_out;
  pro.gain = (const bf16*)d_gain;
  pro.eps = eps;
  Q_CHECK_CUDA(launch_gemm_norm<false>(p, (const unsigned char*)d_w_tiled, d_partials, pro, (cudaStream_t)stream));
  return Q_OK;
}

static int swiglu_shape_ok(int M, int inter, int K, const char* who) {
  Q_CHECK_ARG(M >= 1 && M <= Q_MAX_ROWS && inter >= 8 && inter % 8 == 0 && K >= 32 && K % 32 == 0,
              "%s: need 1..%d rows, inter a multiple of 8 and K a multiple of 32 (M=%d inter=%d K=%d)", who,
              Q_MAX_ROWS, M, inter, K);
  return Q_OK;
}

extern "C" int q_gemm_swiglu(const void* d_x, const void* d_w_tiled, void* d_act, int M, int inter, int K,
                             void* stream) {
  Q_CHECK_ARG(d_x && d_w_tiled && d_act, "q_gemm_swiglu: null pointer");
  Q_CHECK_ARG(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_w_tiled & 15) == 0,
              "q_gemm_swiglu: x and w must be 16-byte aligned");
  int rc = swiglu_shape_ok(M, inter, K, "q_gemm_swiglu");
  if (rc) return rc;
  q_gemm_plan_t p;
  rc = q_gemm_plan(M, 2 * inter, K, &p);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const bf16* X = (const bf16*)d_x;
  const unsigned char* W = (const unsigned char*)d_w_tiled;
  float* out = reinterpret_cast<float*>(d_act);
  cudaError_t e;
  if (M <= 8) e = launch_gemm<1, true>(p, X, W, out, s);
  else if (M <= 16) e = launch_gemm<2, true>(p, X, W, out, s);
  else if (M <= 32) e = launch_gemm<4, true>(p, X, W, out, s);
  else e = launch_gemm<8, true>(p, X, W, out, s);
  Q_CHECK_CUDA(e);
  return Q_OK;
}

extern "C" int q_gemm_swiglu_addnorm(const void* d_resid_in, const float* d_prev, const q_gemm_plan_t* prev_plan,
                                     const void* d_gain, void* d_resid_out, const void* d_w_tiled,
                                     void* d_act, int M, int inter, int K, float eps, void* stream) {
  Q_CHECK_ARG(d_resid_in && d_prev && d_gain && d_resid_out && d_w_tiled && d_act,
              "q_gemm_swiglu_addnorm: null pointer");
  Q_CHECK_ARG(d_resid_in != d_resid_out, "q_gemm_swiglu_addnorm: the residual cannot be updated in place");
  Q_CHECK_ALIGN(d_resid_in, 8, "q_gemm_swiglu_addnorm"); Q_CHECK_ALIGN(d_prev, 16, "q_gemm_swiglu_addnorm");
  Q_CHECK_ALIGN(d_gain, 8, "q_gemm_swiglu_addnorm"); Q_CHECK_ALIGN(d_resid_out, 8, "q_gemm_swiglu_addnorm");
  Q_CHECK_ALIGN(d_w_tiled, 16, "q_gemm_swiglu_addnorm"); Q_CHECK_ALIGN(d_act, 2, "q_gemm_swiglu_addnorm");
  Q_CHECK_ARG(M >= 1 && M <= 8 && K % 4 == 0 && K <= 3072,
              "q_gemm_swiglu_addnorm: needs 1..8 rows and K a multiple of 4 up to 3072 (M=%d K=%d)", M, K);
  int rc = swiglu_shape_ok(M, inter, K, "q_gemm_swiglu_addnorm");
  if (rc) return rc;
  if (prev_plan)
    Q_CHECK_ARG(prev_plan->M == M && prev_plan->N == K, "q_gemm_swiglu_addnorm: previous plan is [%d,%d]",
                prev_plan->M, prev_plan->N);
  q_gemm_plan_t p;
  rc = q_gemm_plan(M, 2 * inter, K, &p);
  if (rc) return rc;
  NormPrologue pro;
  pro.prev = d_prev;
  pro.prev_plan = plan_view(prev_plan);
  pro.resid_in = (const bf16*)d_resid_in;
  pro.resid_out = (bf16*)d_resid_out;
  pro.gain = (const bf16*)d_gain;
  pro.eps = eps;
  Q_CHECK_CUDA(launch_gemm_norm<true>(p, (const unsigned char*)d_w_tiled, reinterpret_cast<float*>(d_act), pro,
                                      (cudaStream_t)stream));
  return Q_OK;
}

// ---- tensor parallel over peer memory, 1-8 rows: the exchange inside the projections ----
// (see the PEER template parameter)

// X[M,K] @ W^T, every partial pushed to every rank's receive area.
extern "C" int q_gemm_push(const void* d_x, const void* d_w_tiled, const q_gemm_plan_t* plan, const q_peers_t* peers,
                           void* stream) {
  Q_CHECK_ARG(d_x && d_w_tiled && plan && peers, "q_gemm_push: null pointer");
  Q_CHECK_ARG(plan->M >= 1 && plan->M <= 8 && plan->slots <= 2 && plan->group_rows == 16,
              "q_gemm_push: needs a stream-K plan of 1..8 rows with at most two slots");
  Q_CHECK_ALIGN(d_x, 16, "q_gemm_push"); Q_CHECK_ALIGN(d_w_tiled, 16, "q_gemm_push");
  PeerView pw;
  int rc = q_peer_view(peers, &pw, "q_gemm_push");
  if (rc) return rc;
  Q_CHECK_CUDA(launch_gemm_push(*plan, (const bf16*)d_x, (const unsigned char*)d_w_tiled, pw, (cudaStream_t)stream));
  return Q_OK;
}

static int addnorm_peers_common(const void* d_resid_in, const q_peers_t* peers, const q_gemm_plan_t* prev_plan,
                                const void* d_gain, void* d_resid_out, const void* d_w_tiled, void* d_out, int M,
                                int K, float eps, NormPrologue* pro, PeerView* pw, const char* who) {
  Q_CHECK_ARG(d_resid_in && peers && prev_plan && d_gain && d_resid_out && d_w_tiled && d_out, "%s: null pointer", who);
  Q_CHECK_ARG(d_resid_in != d_resid_out, "%s: the residual cannot be updated in place", who);
  Q_CHECK_ALIGN(d_resid_in, 8, who); Q_CHECK_ALIGN(d_gain, 8, who); Q_CHECK_ALIGN(d_resid_out, 8, who);
  Q_CHECK_ALIGN(d_w_tiled, 16, who); Q_CHECK_ALIGN(d_out, 4, who);
  Q_CHECK_ARG(M >= 1 && M <= 8 && K % 4 == 0 && K <= 3072, "%s: needs 1..8 rows and K a multiple of 4 up to 3072", who);
  Q_CHECK_ARG(prev_plan->M == M && prev_plan->N == K && prev_plan->slots <= 2 && prev_plan->group_rows == 16,
              "%s: the pushing projection's plan must be a stream-K plan [%d,%d] with at most two slots", who, M, K);
  int rc = q_peer_view(peers, pw, who);
  if (rc) return rc;
  pro->prev = nullptr;
  pro->prev_plan = plan_view(prev_plan);
  pro->resid_in = (const bf16*)d_resid_in;
  pro->resid_out = (bf16*)d_resid_out;
  pro->gain = (const bf16*)d_gain;
  pro->eps = eps;
  return Q_OK;
}

// q_gemm_splitk_addnorm with the previous projection's partials of ALL ranks taken from the
// receive area (pushed by q_gemm_push on every rank).
extern "C" int q_gemm_splitk_addnorm_peers(const void* d_resid_in, const q_peers_t* peers, const q_gemm_plan_t* prev_plan,
                                           const void* d_gain, void* d_resid_out, const void* d_w_tiled, float* d_partials,
                                           int M, int N, int K, float eps, void* stream) {
  NormPrologue pro;
  PeerView pw;
  int rc = addnorm_peers_common(d_resid_in, peers, prev_plan, d_gain, d_resid_out, d_w_tiled, d_partials, M, K, eps,
                                &pro, &pw, "q_gemm_splitk_addnorm_peers");
  if (rc) return rc;
  q_gemm_plan_t p;
  rc = q_gemm_plan(M, N, K, &p);
  if (rc) return rc;
  Q_CHECK_CUDA(launch_gemm_norm_poll<false>(p, (const unsigned char*)d_w_tiled, d_partials, pro, pw, (cudaStream_t)stream));
  return Q_OK;
}

// q_gemm_swiglu_addnorm likewise.
extern "C" int q_gemm_swiglu_addnorm_peers(const void* d_resid_in, const q_peers_t* peers, const q_gemm_plan_t* prev_plan,
                                           const void* d_gain, void* d_resid_out, const void* d_w_tiled, void* d_act, int M,
                                           int inter, int K, float eps, void* stream) {
  NormPrologue pro;
  PeerView pw;
  int rc = addnorm_peers_common(d_resid_in, peers, prev_plan, d_gain, d_resid_out, d_w_tiled, d_act, M, K, eps, &pro,
                                &pw, "q_gemm_swiglu_addnorm_peers");
  if (rc) return rc;
  rc = swiglu_shape_ok(M, inter, K, "q_gemm_swiglu_addnorm_peers");
  if (rc) return rc;
  q_gemm_plan_t p;
  rc = q_gemm_plan(M, 2 * inter, K, &p);
  if (rc) return rc;
  Q_CHECK_CUDA(launch_gemm_norm_poll<true>(p, (const unsigned char*)d_w_tiled, reinterpret_cast<float*>(d_act), pro, pw,
                                           (cudaStream_t)stream));
  return Q_OK;
}

extern "C" int q_reduce_partials(const float* d_partials, const q_gemm_plan_t* plan,
                                 float* d_out, void* stream) {
  Q_CHECK_ARG(d_partials && plan && d_out, "q_reduce_partials: null pointer");
  Q_CHECK_ALIGN(d_partials, 16, "q_reduce_partials"); Q_CHECK_ALIGN(d_out, 16, "q_reduce_partials");
  long long total = (long long)plan->M * plan->N;
  if ((plan->N & 3) == 0) total /= 4;
  int block = 256;
  int grid = (int)((total + block - 1) / block);
  Q_CHECK_CUDA(q_launch(k_reduce_partials, dim3(grid), dim3(block), 0, (cudaStream_t)stream,
                        d_partials, d_out, plan_view(plan), plan->M, plan->N));
  return Q_OK;
}
