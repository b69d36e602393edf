// Whole decode step as ONE persistent cooperative kernel (small batch).
//
// The multi-kernel step (capi.cu) pays a kernel boundary ~360 times per token;
// at batch 1 the weight stream of a whole layer is only ~31 us long, so those
// boundaries dominate. Here one CTA per SM stays resident for the whole step and
// the phases are separated by grid barriers instead (reference: one captured
// graph of ~335 kernel nodes, engine/decode_step.py:33-60, engine/decode.py:97-108).
//
// Per layer:  A  add+RMSNorm (or embedding) -> QKV GEMM            | barrier
//             B  q/k norm + RoPE + KV write -> split-KV attention,  |
//                last split of a kv head merges the splits         | barrier
//             C  O-proj GEMM                                       | barrier
//             D  add+RMSNorm -> gate|up GEMM                       | barrier
//             E  SwiGLU (spread over the grid)                     | barrier
//             F  down GEMM                                         | barrier
// then the final norm + lm_head GEMM, barrier, and a grid-wide argmax whose last
// CTA writes the token and bumps the position.
//
// What makes the barriers cheap: a CTA issues the TMA copies of its NEXT GEMM's
// first 128 KB (its whole shared-memory ring) BEFORE it arrives at the barrier,
// so HBM keeps streaming weights while the CTAs synchronise and run the small
// prologues. The residual stream lives in every CTA's shared memory (all CTAs
// compute the same add+norm), so no phase depends on one CTA writing it.
//
// The GEMM phases use the same tiled weights, per-warp contiguous runs, mma
// fragments and slot scheme as k_gemm_streamk; the attention phase is the
// k_attn_split algorithm with the rope prologue and the merge folded in. Cast
// boundaries are identical to the multi-kernel step (see fused_ops.cu).
//
// Every data item another CTA wrote in this launch is read with ld.global.cg
// (L1 is not coherent across SMs). Every spin (grid barrier, mbarrier) is
// bounded: when a limit runs out the kernel records a status code and carries
// on to the end instead of hanging.
#include "common.cuh"
#include "mega_step.h"

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int STAGE_UNITS = 8;
constexpr int STAGES = 2;
constexpr int STAGE_BYTES = STAGE_UNITS * 1024;
constexpr int RING_BYTES = WARPS * STAGES * STAGE_BYTES;     // 128 KB
constexpr int RED_FLOATS = WARPS * 2 * 128;                  // ragged-end accumulators
constexpr unsigned SPIN_LIMIT = 1u << 22;

constexpr int ATT_TILE = 64 * 128 * 2;                       // one K or V tile
constexpr int ATT_STAGE = 2 * ATT_TILE;
constexpr int ATT_NS = 3;

__device__ int g_mega_status[4];
// Measurement aid: phase time stamps (ns) of layer `trace_layer` for CTAs 0 and 100.
__device__ unsigned long long g_mega_trace[2 * 32 + 4 * 160];
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define STAMP(i)                                                                        \
  do {                                                                                   \
    if (c.trace_gemm > 0 && threadIdx.x == 0) g_mega_trace[(blockIdx.x == 0 ? 0 : 32) + (i)] = gtime(); \
  } while (0)
#define TRACE(i)                                                                         \
  do {                                                                                   \
    if (tracing && threadIdx.x == 0) g_mega_trace[(blockIdx.x == 0 ? 0 : 32) + (i)] = gtime(); \
  } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if (it > 256) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ldcg_f(const float* p) { return __ldcg(p); }

// Partial-sum read of element idx (column n) written by other CTAs in this launch.
__device__ __forceinline__ float psum_cg(const float* P, const mega_plan_t& pl, long long stride,
                                         long long idx, int n) {
  const unsigned g = (unsigned)n >> 4, C = (unsigned)pl.C, u = (unsigned)pl.U;
  const unsigned first = (g * C) / u, last = ((g + 1) * C - 1) / u;
  float s = ldcg_f(P + idx);
  const float s1 = ldcg_f(P + idx + stride);
  if (last > first) s += s1;
  for (unsigned k = 2; k <= last - first; ++k) s += ldcg_f(P + idx + (long long)k * stride);
  return s;
}

struct Ctx {
  unsigned char* ring;        // RING_BYTES (attention reuses it)
  float* red;                 // RED_FLOATS
  int* tags;                  // WARPS*2
  uint64_t* gbars;            // WARPS*STAGES  (GEMM ring)
  uint64_t* abars;            // 2*ATT_NS      (attention ring)
  bf16* xs;                   // GEMM activation operand [M][Kmax]
  bf16* resid;                // residual stream [M][H]
  float* scratch;             // 64 floats for block reductions + small broadcast
  bf16* knew;                 // [128] newest key of this CTA's kv head
  bf16* vnew;                 // [128]
  bf16* cosrow;               // [128] rotary table row of the current position
  bf16* sinrow;               // [128]
  int pos;                    // position of the current token (read once per launch)
  uint32_t g_count;           // per-warp GEMM stage counter (mbarrier phase tracking)
  uint32_t a_count;           // attention stage counter (CTA-wide, same in all threads)
  int trace_gemm;             // measurement aid: >0 = stamp this GEMM's stages into g_mega_trace[17..]
  unsigned epoch;             // grid barrier epoch
};

// ---- grid barrier (split: arrive, then do independent work, then wait) ------------------
__device__ __noinline__ void grid_arrive(const mega_params_t& p, Ctx& c) {
  __syncthreads();
  c.epoch += 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(&p.sync[0], 1u);
  }
}

__device__ __noinline__ void grid_wait(const mega_params_t& p, Ctx& c) {
  if (threadIdx.x == 0) {
    const unsigned target = c.epoch * gridDim.x;
    unsigned it = 0;
    // once any wait in this launch has run out, nobody spins again
    while (*reinterpret_cast<volatile int*>(&g_mega_status[0]) == 0) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.sync) : "memory");
      if (v >= target) break;
      if (++it > SPIN_LIMIT) { atomicExch(&g_mega_status[0], 1); break; }
      if (it > 64) __nanosleep(20);
    }
    __threadfence();
  }
  __syncthreads();
}

__device__ __forceinline__ void grid_barrier(const mega_params_t& p, Ctx& c) {
  grid_arrive(p, c);
  grid_wait(p, c);
}

// ---- GEMM phase --------------------------------------------------------------------
struct GemmRun {
  const unsigned char* src;
  int ws, n_units, n_stages;
  uint32_t base;              // stage counter value of stage 0 of this GEMM
};

// Issues the first ring-full of the warp's run. Weights never depend on earlier
// phases, so this is called BEFORE the barrier that precedes the GEMM.
__device__ __noinline__ GemmRun gemm_prime(const unsigned char* Wt, const mega_plan_t& pl, Ctx& c) {
  GemmRun r;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cs = blockIdx.x * pl.U;
  const int ce = min(pl.total, cs + pl.U);
  const int len = ce > cs ? ce - cs : 0;
  r.ws = cs + (int)(((long long)warp * len) / WARPS);
  const int we = cs + (int)(((long long)(warp + 1) * len) / WARPS);
  r.n_units = we - r.ws;
  r.n_stages = (r.n_units + STAGE_UNITS - 1) / STAGE_UNITS;
  r.src = Wt + (size_t)r.ws * 1024;
  r.base = c.g_count;
  if (lane == 0) {
    // the ring may just have been written through the generic proxy (attention merge)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const uint32_t ring = smem_u32(c.ring) + warp * (STAGES * STAGE_BYTES);
    for (int s = 0; s < STAGES && s < r.n_stages; ++s) {
      const uint32_t slot = (r.base + s) % STAGES;
      const uint32_t bar = smem_u32(&c.gbars[warp * STAGES + slot]);
      const uint32_t bytes = (uint32_t)min(STAGE_UNITS, r.n_units - s * STAGE_UNITS) * 1024u;
      mbar_expect_tx(bar, bytes);
      bulk_g2s(ring + slot * STAGE_BYTES, r.src + (size_t)s * STAGE_BYTES, bytes, bar);
    }
  }
  c.g_count += r.n_stages;
  return r;
}

// Asks the TMA unit to pull (part of) this warp's run of a LATER GEMM into L2, so that HBM
// keeps streaming during the latency-bound phases (attention, norms, barriers). Bytes
// [skip, skip + cap) of the run; the first RING bytes usually arrive through gemm_prime.
__device__ __noinline__ void l2_prefetch_run(const unsigned char* Wt, const mega_plan_t& pl, int skip_units,
                                             int cap_units) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane != 0 || cap_units <= 0) return;
  const int cs = blockIdx.x * pl.U;
  const int ce = min(pl.total, cs + pl.U);
  const int len = ce > cs ? ce - cs : 0;
  const int ws = cs + (int)(((long long)warp * len) / WARPS);
  const int we = cs + (int)(((long long)(warp + 1) * len) / WARPS);
  int lo = ws + skip_units, hi = min(we, lo + cap_units);
  while (lo < hi) {
    const int n = min(hi - lo, 32);                      // 32 KB per instruction
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(Wt + (size_t)lo * 1024),
                 "r"((uint32_t)n * 1024u) : "memory");
    lo += n;
  }
}

// Streams the run, X fragments from shared memory (xs[M][K]), partials to P.
// mma.sync has a long latency on this part (~280 cycles), so consecutive MMAs go
// to NSETS independent accumulators that are added when a 16-row group ends.
constexpr int NSETS = 8;

__device__ __noinline__ void gemm_run(const GemmRun& r, const mega_plan_t& pl, int M, const bf16* xs,
                                      float* __restrict__ P, Ctx& c) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int C = pl.C, N = pl.N, K = pl.K;
  const uint32_t ring = smem_u32(c.ring) + warp * (STAGES * STAGE_BYTES);
  const uint32_t xbase = smem_u32(xs) + (uint32_t)(g * K + t * 8) * 2u;
  if (lane < 2) c.tags[warp * 2 + lane] = -1;
  __syncwarp();
  float acc[NSETS][4];
#pragma unroll
  for (int s = 0; s < NSETS; ++s) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;
  int group = r.ws / C;
  int chunk = r.ws - group * C;
  int seg_first = chunk, n_boundary = 0, units_done = 0;
  for (int st = 0; st < r.n_stages; ++st) {
    const uint32_t slot = (r.base + st) % STAGES;
    const uint32_t bar = smem_u32(&c.gbars[warp * STAGES + slot]);
    if (!mbar_wait(bar, ((r.base + st) / STAGES) & 1)) {
      atomicExch(&g_mega_status[0], 2);
      break;
    }
    const int in_stage = min(STAGE_UNITS, r.n_units - st * STAGE_UNITS);
    uint32_t sbase = ring + slot * STAGE_BYTES + lane * 16;
    int done = 0;
    while (done < in_stage) {
      const int n = min(in_stage - done, C - chunk);     // units of this stage inside one group
      const uint32_t xaddr = xbase + (uint32_t)chunk * 64u;
#pragma unroll
      for (int j = 0; j < STAGE_UNITS; ++j) {
        if (j < n) {
          const uint4 a = lds128(sbase + j * 1024), b = lds128(sbase + j * 1024 + 512);
          uint4 x = make_uint4(0, 0, 0, 0);
          if (g < M) x = lds128(xaddr + j * 64);
          mma16816(acc[(2 * j) % NSETS], a.x, b.x, a.y, b.y, x.x, x.y);
          mma16816(acc[(2 * j + 1) % NSETS], a.z, b.z, a.w, b.w, x.z, x.w);
        }
      }
      done += n; chunk += n; units_done += n; sbase += n * 1024;
      const bool group_end = (chunk == C);
      if (group_end || units_done == r.n_units) {
        float tot[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < NSETS; ++s) { v += acc[s][e]; acc[s][e] = 0.f; }
          tot[e] = v;
        }
        if (group_end && seg_first == 0) {
          const int n0 = group * 16 + g, m0 = 2 * t;
          if (m0 < M) {
            if (n0 < N) P[(size_t)m0 * N + n0] = tot[0];
            if (n0 + 8 < N) P[(size_t)m0 * N + n0 + 8] = tot[2];
          }
          if (m0 + 1 < M) {
            if (n0 < N) P[(size_t)(m0 + 1) * N + n0] = tot[1];
            if (n0 + 8 < N) P[(size_t)(m0 + 1) * N + n0 + 8] = tot[3];
          }
        } else {
          float* mine = c.red + ((size_t)warp * 2 + n_boundary) * 128;
          *reinterpret_cast<float4*>(mine + lane * 4) = make_float4(tot[0], tot[1], tot[2], tot[3]);
          if (lane == 0) c.tags[warp * 2 + n_boundary] = group;
          ++n_boundary;
        }
        seg_first = 0;
        if (group_end) { chunk = 0; ++group; }
      }
    }
    __syncwarp();
    const int nxt = st + STAGES;
    if (lane == 0 && nxt < r.n_stages) {
      const uint32_t bytes = (uint32_t)min(STAGE_UNITS, r.n_units - nxt * STAGE_UNITS) * 1024u;
      mbar_expect_tx(bar, bytes);
      bulk_g2s(ring + slot * STAGE_BYTES, r.src + (size_t)nxt * STAGE_BYTES, bytes, bar);
    }
  }
  __syncthreads();
  // Ragged ends: the warp that holds the FIRST parked entry of a group adds all entries
  // of that group (fixed order) and writes the CTA's partial of the group.
  const long long stride = (long long)M * N;
  int tg[WARPS * 2];
#pragma unroll
  for (int s = 0; s < WARPS * 2; s += 4) {
    const int4 v = *reinterpret_cast<const int4*>(c.tags + s);
    tg[s] = v.x; tg[s + 1] = v.y; tg[s + 2] = v.z; tg[s + 3] = v.w;
  }
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const int mine = warp * 2 + which;
    int gg = -1;
    bool fresh = true;
#pragma unroll
    for (int s2 = 0; s2 < WARPS * 2; ++s2) {
      if (s2 == mine) gg = tg[s2];
    }
    if (gg < 0) continue;
#pragma unroll
    for (int s2 = 0; s2 < WARPS * 2; ++s2) fresh = fresh && !(s2 < mine && tg[s2] == gg);
    if (!fresh) continue;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s2 = 0; s2 < WARPS * 2; ++s2) {
      if (s2 >= mine && tg[s2] == gg) {
        const float4 v = *reinterpret_cast<const float4*>(c.red + (size_t)s2 * 128 + lane * 4);
        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
      }
    }
    const unsigned first = ((unsigned)gg * (unsigned)C) / (unsigned)pl.U;
    float* out = P + (long long)((int)blockIdx.x - (int)first) * stride;
    const int n0 = gg * 16 + g, m0 = 2 * t;
    if (m0 < M) {
      if (n0 < N) out[(size_t)m0 * N + n0] = sum.x;
      if (n0 + 8 < N) out[(size_t)m0 * N + n0 + 8] = sum.z;
    }
    if (m0 + 1 < M) {
      if (n0 < N) out[(size_t)(m0 + 1) * N + n0] = sum.y;
      if (n0 + 8 < N) out[(size_t)(m0 + 1) * N + n0 + 8] = sum.w;
    }
  }
  // red/tags are written again only after the next grid barrier (a __syncthreads)
}

// ---- block reduction ------------------------------------------------------------------
__device__ __forceinline__ float block_sum_s(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < WARPS ? red[lane] : 0.f;
  return warp_sum(t);
}

// ---- prologues: produce the residual (resid) and the normed GEMM operand (xs) ---------
// xs[m][*] = bf16(bf16(resid*inv) * gain) given the per-row sum of squares `ss`.
__device__ __forceinline__ void scale_row_to_xs(const mega_params_t& p, Ctx& c, const bf16* gain, int K,
                                                int m, float ss) {
  const int H = p.H;
  const float inv = rsqrtf(ss / (float)H + p.eps);
  for (int col = threadIdx.x; col < H; col += THREADS) {
    const float v = bf16_round(__bfloat162float(c.resid[m * H + col]) * inv);
    c.xs[m * K + col] = __float2bfloat16_rn(v * __bfloat162float(gain[col]));
  }
}

__device__ __forceinline__ size_t tiled_elem(long long row, int col, int C) {
  const long long unit = (row >> 4) * C + (col >> 5);
  const int piece = (int)(row & 7) * 4 + ((col & 31) >> 3);
  return (size_t)unit * 512 + (size_t)((row >> 3) & 1) * 256 + piece * 8 + (col & 7);
}

constexpr int PB = 12;  // columns per thread whose global loads are issued together (3072 per batch)
constexpr int VB = 4;   // float4 batches per thread in the add+norm vector path (4096 columns)

__device__ __noinline__ void prologue_embed(const mega_params_t& p, Ctx& c, const bf16* gain) {
  const int H = p.H, C = H >> 5;
  const bf16* E = reinterpret_cast<const bf16*>(p.embed);
  for (int m = 0; m < p.M; ++m) {
    long long tok = p.tokens[m];
    tok = tok < 0 ? 0 : (tok >= p.full_vocab ? p.full_vocab - 1 : tok);
    float ss = 0.f;
    for (int base = threadIdx.x; base < H; base += THREADS * PB) {
      bf16 v[PB];
#pragma unroll
      for (int j = 0; j < PB; ++j) {
        const int col = base + j * THREADS;
        v[j] = col < H ? E[tiled_elem(tok, col, C)] : __float2bfloat16_rn(0.f);
      }
#pragma unroll
      for (int j = 0; j < PB; ++j) {
        const int col = base + j * THREADS;
        if (col < H) {
          c.resid[m * H + col] = v[j];
          const float f = __bfloat162float(v[j]);
          ss += f * f;
        }
      }
    }
    STAMP(18);
    ss = block_sum_s(ss, c.scratch);
    STAMP(19);
    scale_row_to_xs(p, c, gain, H, m, ss);
    STAMP(20);
  }
  __syncthreads();
  STAMP(21);
}

// resid = bf16(resid + bf16(sum of partial slots)); xs = RMSNorm(resid) * gain
// Fast path (H <= 3072): every thread keeps its <= 12 columns in registers, all global
// loads (two partial slots and the gain) are issued together, one pass.
__device__ __noinline__ void prologue_add_norm(const mega_params_t& p, Ctx& c, const float* P,
                                               const mega_plan_t& pl, const bf16* gain) {
  const int H = p.H;
  const long long stride = (long long)p.M * H;
  const unsigned C = (unsigned)pl.C, u = (unsigned)pl.U;
  STAMP(17);
  // which 16-column groups have a second slot (one division pair per group, not per column)
  int* two = reinterpret_cast<int*>(c.red);        // red is idle between GEMM phases
  for (int gi = threadIdx.x; gi < (H >> 4); gi += THREADS) {
    const unsigned first = ((unsigned)gi * C) / u, last = (((unsigned)gi + 1) * C - 1) / u;
    two[gi] = (int)(last - first);
  }
  __syncthreads();
  if (H <= THREADS * 4 * VB && (H & 3) == 0 && (H >> 4) <= RED_FLOATS) {
    // Vector path: thread t owns columns 4t..4t+3 (+1024 j): float4 loads of both slots
    // and an 8-byte load of the gains, all issued before anything is used.
    for (int m = 0; m < p.M; ++m) {
      float4 s0[VB], s1[VB];
      uint2 gn[VB];
#pragma unroll
      for (int j = 0; j < VB; ++j) {
        const int col = 4 * threadIdx.x + j * THREADS * 4;
        const int cc = col < H ? col : 0;
        s0[j] = __ldcg(reinterpret_cast<const float4*>(P + (long long)m * H + cc));
        s1[j] = __ldcg(reinterpret_cast<const float4*>(P + (long long)m * H + cc + stride));
        gn[j] = *reinterpret_cast<const uint2*>(gain + cc);
      }
      float tot[VB][4];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < VB; ++j) {
        const int col = 4 * threadIdx.x + j * THREADS * 4;
        if (col < H) {
          const int extra = two[col >> 4];       // the 4 columns share one 16-column group
          float s[4] = {s0[j].x, s0[j].y, s0[j].z, s0[j].w};
          if (extra > 0) { s[0] += s1[j].x; s[1] += s1[j].y; s[2] += s1[j].z; s[3] += s1[j].w; }
          for (int k = 2; k <= extra; ++k) {
            const float4 sk = __ldcg(reinterpret_cast<const float4*>(P + (long long)m * H + col + (long long)k * stride));
            s[0] += sk.x; s[1] += sk.y; s[2] += sk.z; s[3] += sk.w;
          }
          const uint2 rr = *reinterpret_cast<const uint2*>(c.resid + m * H + col);
          const float r[4] = {bf_lo(rr.x), bf_hi(rr.x), bf_lo(rr.y), bf_hi(rr.y)};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            tot[j][e] = bf16_round(r[e] + bf16_round(s[e]));
            ss += tot[j][e] * tot[j][e];
          }
        }
      }
      STAMP(18);
      ss = block_sum_s(ss, c.scratch);
      STAMP(19);
      const float inv = rsqrtf(ss / (float)H + p.eps);
#pragma unroll
      for (int j = 0; j < VB; ++j) {
        const int col = 4 * threadIdx.x + j * THREADS * 4;
        if (col < H) {
          const float g4[4] = {bf_lo(gn[j].x), bf_hi(gn[j].x), bf_lo(gn[j].y), bf_hi(gn[j].y)};
          uint2 ro, xo;
          ro.x = pack_bf16(tot[j][0], tot[j][1]);
          ro.y = pack_bf16(tot[j][2], tot[j][3]);
          xo.x = pack_bf16(bf16_round(tot[j][0] * inv) * g4[0], bf16_round(tot[j][1] * inv) * g4[1]);
          xo.y = pack_bf16(bf16_round(tot[j][2] * inv) * g4[2], bf16_round(tot[j][3] * inv) * g4[3]);
          *reinterpret_cast<uint2*>(c.resid + m * H + col) = ro;
          *reinterpret_cast<uint2*>(c.xs + m * H + col) = xo;
        }
      }
      STAMP(20);
    }
  } else {
    for (int m = 0; m < p.M; ++m) {
      float ss = 0.f;
      for (int col = threadIdx.x; col < H; col += THREADS) {
        const float y = bf16_round(psum_cg(P, pl, stride, (long long)m * H + col, col));
        const bf16 t = __float2bfloat16_rn(__bfloat162float(c.resid[m * H + col]) + y);
        c.resid[m * H + col] = t;
        const float f = __bfloat162float(t);
        ss += f * f;
      }
      ss = block_sum_s(ss, c.scratch);
      scale_row_to_xs(p, c, gain, H, m, ss);
    }
  }
  __syncthreads();
  STAMP(21);
}

__device__ __noinline__ void stage_x(const mega_params_t& p, Ctx& c, const bf16* src, int K) {
  const int pieces = p.M * K / 8;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(c.xs);
  for (int i = threadIdx.x; i < pieces; i += THREADS) d[i] = __ldcg(s + i);
  __syncthreads();
}

// ---- attention phase ----------------------------------------------------------------------
// CTA `item` = (sequence b, kv head kh, split). T = 1, G <= 16.
__device__ __noinline__ void attention_phase(const mega_params_t& p, Ctx& c, const mega_layer_t& L,
                                                const float* PQ) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.attn_S, nq = p.nq, nkv = p.nkv, G = nq / nkv;
  const int items = p.M * nkv * S;
  if ((int)blockIdx.x >= items) return;
  const int bh = blockIdx.x / S, split = blockIdx.x % S;
  const int b = bh / nkv, kh = bh % nkv;
  const int pos = c.pos;
  const int max_limit = pos + 1;
  const int tiles_used = (max_limit + Q_PAGE_TOKENS - 1) / Q_PAGE_TOKENS;
  const int per = (tiles_used + S - 1) / S;
  const int tile0 = split * per;
  const int tile1 = min(tiles_used, tile0 + per);
  const int ntiles = tile1 > tile0 ? tile1 - tile0 : 0;
  const int new_tile = pos / Q_PAGE_TOKENS, new_row = pos % Q_PAGE_TOKENS;
  const bool owns_new = ntiles > 0 && new_tile >= tile0 && new_tile < tile1;

  STAMP(22);
  unsigned char* stages = c.ring;                         // ATT_NS * ATT_STAGE = 96 KB
  unsigned char* qtile = c.ring + ATT_NS * ATT_STAGE;     // 16 rows * 256 B
  const uint32_t abar = smem_u32(c.abars);
  const uint32_t a_base = c.a_count;
  c.a_count += (uint32_t)ntiles;

  // ---- producer first, so that the KV tiles are in flight during the rope prologue ----
  if (warp == 4 && lane == 0) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int it = 0; it < ntiles && it < ATT_NS; ++it) {
      const uint32_t slot = (a_base + it) % ATT_NS;
      const int page = p.block_table[(size_t)b * p.pages_per_seq + tile0 + it];
      const size_t off = ((size_t)page * nkv + kh) * ATT_TILE;
      mbar_expect_tx(abar + 8 * slot, ATT_STAGE);
      bulk_g2s(smem_u32(stages + slot * ATT_STAGE), L.kpool + off, ATT_TILE, abar + 8 * slot);
      bulk_g2s(smem_u32(stages + slot * ATT_STAGE + ATT_TILE), L.vpool + off, ATT_TILE, abar + 8 * slot);
    }
  }

  // ---- q/k head norm + RoPE (+ v), from the QKV partials ----
  // One warp per head; lane l owns dims 4l..4l+3 (one float4 per slot), the rotate-half
  // partner dims (d +- 64) live in lane l ^ 16.
  {
    const int width = (nq + 2 * nkv) * 128;
    const long long stride = (long long)p.M * width;
    const float eps = p.eps;
    const unsigned Cq = (unsigned)p.qkv.C, uq = (unsigned)p.qkv.U;
    for (int h = warp; h < G + 2; h += WARPS) {
      const bool is_q = h < G, is_v = h == G + 1;
      const int head = is_q ? kh * G + h : (is_v ? nq + nkv + kh : nq + kh);   // column block
      const long long src = (long long)b * width + (long long)head * 128 + 4 * lane;
      const float4 s0 = __ldcg(reinterpret_cast<const float4*>(PQ + src));
      const float4 s1 = __ldcg(reinterpret_cast<const float4*>(PQ + src + stride));
      const uint2 graw = is_v ? make_uint2(0, 0)
                              : *reinterpret_cast<const uint2*>((is_q ? L.q_gain : L.k_gain) + 4 * lane);
      const unsigned gq = (unsigned)(head * 128 + 4 * lane) >> 4;
      const unsigned first = (gq * Cq) / uq, last = ((gq + 1) * Cq - 1) / uq;
      float x[4] = {s0.x, s0.y, s0.z, s0.w};
      if (last > first) { x[0] += s1.x; x[1] += s1.y; x[2] += s1.z; x[3] += s1.w; }
      for (unsigned k = 2; k <= last - first; ++k) {
        const float4 sk = __ldcg(reinterpret_cast<const float4*>(PQ + src + (long long)k * stride));
        x[0] += sk.x; x[1] += sk.y; x[2] += sk.z; x[3] += sk.w;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = bf16_round(x[e]);
      if (is_v) {
        uint2 o;
        o.x = pack_bf16(x[0], x[1]);
        o.y = pack_bf16(x[2], x[3]);
        *reinterpret_cast<uint2*>(c.vnew + 4 * lane) = o;
        continue;
      }
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / 128.f + eps);
      const float gv[4] = {bf_lo(graw.x), bf_hi(graw.x), bf_lo(graw.y), bf_hi(graw.y)};
      const uint2 craw = *reinterpret_cast<const uint2*>(c.cosrow + 4 * lane);
      const uint2 sraw = *reinterpret_cast<const uint2*>(c.sinrow + 4 * lane);
      const float cs[4] = {bf_lo(craw.x), bf_hi(craw.x), bf_lo(craw.y), bf_hi(craw.y)};
      const float sn[4] = {bf_lo(sraw.x), bf_hi(sraw.x), bf_lo(sraw.y), bf_hi(sraw.y)};
      float out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float n = bf16_round(bf16_round(x[e] * inv) * gv[e]);
        const float partner = __shfl_xor_sync(0xffffffffu, n, 16);
        const float rot = lane < 16 ? -partner : partner;     // dims < 64 take -x[d+64]
        out[e] = bf16_round(n * cs[e]) + bf16_round(rot * sn[e]);
      }
      uint2 o;
      o.x = pack_bf16(out[0], out[1]);
      o.y = pack_bf16(out[2], out[3]);
      if (is_q) {
        // dims 4l..4l+3 sit in 16-byte chunk l/2 of query row h (rows are swizzled like KV tiles)
        const int ch = lane >> 1;
        *reinterpret_cast<uint2*>(qtile + h * 256 + ((ch ^ (h & 7)) << 4) + (lane & 1) * 8) = o;
      } else {
        *reinterpret_cast<uint2*>(c.knew + 4 * lane) = o;
      }
    }
    // rows G..15 of the query tile are zero
    for (int i = tid; i < (16 - G) * 16; i += THREADS) {
      const int r = G + (i >> 4), ch = i & 15;
      *reinterpret_cast<uint4*>(qtile + r * 256 + ((ch ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
    }
  }
  __syncthreads();
  STAMP(23);
  if (owns_new && tid < 32) {
    // the newest key/value row goes to its page for later steps (16 lanes x 16 B each)
    const int page = p.block_table[(size_t)b * p.pages_per_seq + new_tile];
    const size_t tile = ((size_t)page * nkv + kh) * ATT_TILE;
    if (lane < 16) {
      const int off = new_row * 256 + ((lane ^ (new_row & 7)) << 4);
      *reinterpret_cast<uint4*>(L.kpool + tile + off) = *reinterpret_cast<const uint4*>(c.knew + lane * 8);
      *reinterpret_cast<uint4*>(L.vpool + tile + off) = *reinterpret_cast<const uint4*>(c.vnew + lane * 8);
    }
  }

  if (warp == 4) {
    // ---- producer: remaining tiles ----
    if (lane == 0) {
      for (int it = ATT_NS; it < ntiles; ++it) {
        const uint32_t slot = (a_base + it) % ATT_NS;
        // wait until the 4 consumers released the previous use of this slot
        if (!mbar_wait(abar + 8 * (ATT_NS + slot), ((a_base + it) / ATT_NS - 1) & 1)) {
          atomicExch(&g_mega_status[0], 3);
          break;
        }
        const int page = p.block_table[(size_t)b * p.pages_per_seq + tile0 + it];
        const size_t off = ((size_t)page * nkv + kh) * ATT_TILE;
        mbar_expect_tx(abar + 8 * slot, ATT_STAGE);
        bulk_g2s(smem_u32(stages + slot * ATT_STAGE), L.kpool + off, ATT_TILE, abar + 8 * slot);
        bulk_g2s(smem_u32(stages + slot * ATT_STAGE + ATT_TILE), L.vpool + off, ATT_TILE, abar + 8 * slot);
      }
    }
  } else if (warp < 4) {
    // ---- consumers ----
    const int g = lane >> 2, t4 = lane & 3;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
    const uint32_t q_base = smem_u32(qtile);
    for (int it = 0; it < ntiles; ++it) {
      const uint32_t slot = (a_base + it) % ATT_NS;
      if (!mbar_wait(abar + 8 * slot, ((a_base + it) / ATT_NS) & 1)) {
        atomicExch(&g_mega_status[0], 4);
        break;
      }
      unsigned char* kt = stages + slot * ATT_STAGE;
      unsigned char* vt = kt + ATT_TILE;
      const int key_base = (tile0 + it) * Q_PAGE_TOKENS;
      const int my_key0 = key_base + warp * 16;
      if (my_key0 + 16 > max_limit) {
        for (int i = lane; i < 16 * 16; i += 32) {
          const int kr = warp * 16 + (i >> 4);
          if (key_base + kr >= max_limit)
            *reinterpret_cast<uint4*>(vt + kr * 256 + ((i & 15) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      if (tile0 + it == new_tile && (new_row >> 4) == warp) {
        // patch the newest key/value row (computed above, not yet visible to the bulk copy)
        if (lane < 16) {
          const int off = new_row * 256 + ((lane ^ (new_row & 7)) << 4);
          *reinterpret_cast<uint4*>(kt + off) = *reinterpret_cast<const uint4*>(c.knew + lane * 8);
          *reinterpret_cast<uint4*>(vt + off) = *reinterpret_cast<const uint4*>(c.vnew + lane * 8);
        }
      }
      __syncwarp();
      const uint32_t k_base = smem_u32(kt), v_base = smem_u32(vt);
      float sacc[2][4], sodd[2][4];    // even / odd k steps: two independent MMA chains per key tile
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
        sodd[j][0] = sodd[j][1] = sodd[j][2] = sodd[j][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
        {
          const int row = (lane & 7) + 8 * ((lane >> 3) & 1);
          const int ch = 2 * ks + (lane >> 4);
          ldsm_x4(q_base + row * 256 + ((ch ^ (row & 7)) << 4), a0, a1, a2, a3);
        }
        {
          const int mi = lane >> 3;
          const int key = warp * 16 + 8 * (mi >> 1) + (lane & 7);
          const int ch = 2 * ks + (mi & 1);
          ldsm_x4(k_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        }
        if (ks & 1) {
          mma16816(sodd[0], a0, a1, a2, a3, b0, b1);
          mma16816(sodd[1], a0, a1, a2, a3, b2, b3);
        } else {
          mma16816(sacc[0], a0, a1, a2, a3, b0, b1);
          mma16816(sacc[1], a0, a1, a2, a3, b2, b3);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[j][e] += sodd[j][e];
      float pr[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = my_key0 + 8 * j + 2 * t4 + e;
            float v = sacc[j][2 * h + e] * p.scale_log2;
            v = key < max_limit ? v : -INFINITY;
            sacc[j][2 * h + e] = v;
            mx = fmaxf(mx, v);
          }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[h], mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float resc = exp2f(m_run[h] - m_safe);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float pv = exp2f(sacc[j][2 * h + e] - m_safe);
            pr[j][2 * h + e] = pv;
            sum += pv;
          }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[h] = l_run[h] * resc + sum;
        m_run[h] = m_new;
#pragma unroll
        for (int n = 0; n < 16; ++n) { oacc[n][2 * h] *= resc; oacc[n][2 * h + 1] *= resc; }
      }
      const uint32_t pa0 = pack_bf16(pr[0][0], pr[0][1]), pa1 = pack_bf16(pr[0][2], pr[0][3]);
      const uint32_t pa2 = pack_bf16(pr[1][0], pr[1][1]), pa3 = pack_bf16(pr[1][2], pr[1][3]);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        uint32_t b0, b1, b2, b3;
        const int mi = lane >> 3;
        const int key = warp * 16 + 8 * (mi & 1) + (lane & 7);
        const int ch = 2 * dp + (mi >> 1);
        ldsm_x4_t(v_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        mma16816(oacc[2 * dp], pa0, pa1, pa2, pa3, b0, b1);
        mma16816(oacc[2 * dp + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(abar + 8 * (ATT_NS + slot));
    }
    // park the warp's state for the CTA merge (after the ring is idle)
    STAMP(24);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    float* mo = reinterpret_cast<float*>(stages);            // [4][16][128]
    float* mml = mo + 4 * 16 * 128;                          // [4][16][2]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      float* dst = mo + ((size_t)warp * 16 + r) * 128;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        dst[8 * n + 2 * t4] = oacc[n][2 * h];
        dst[8 * n + 2 * t4 + 1] = oacc[n][2 * h + 1];
      }
      if (t4 == 0) {
        mml[((size_t)warp * 16 + r) * 2] = m_run[h];
        mml[((size_t)warp * 16 + r) * 2 + 1] = l_run[h];
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const int d = tid;
    for (int r = 0; r < G; ++r) {
      float mw[4], Mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) { mw[w] = mml[((size_t)w * 16 + r) * 2]; Mx = fmaxf(Mx, mw[w]); }
      const float Ms = Mx == -INFINITY ? 0.f : Mx;
      float Lsum = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float wt = exp2f(mw[w] - Ms);
        Lsum += wt * mml[((size_t)w * 16 + r) * 2 + 1];
        O += wt * mo[((size_t)w * 16 + r) * 128 + d];
      }
      if (S == 1) {
        p.attended[((size_t)b * nq + kh * G + r) * 128 + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
      } else {
        const size_t row = ((size_t)bh * S + split) * G + r;
        p.attn_o[row * 128 + d] = O;
        if (d == 0) { p.attn_ml[row * 2] = Mx; p.attn_ml[row * 2 + 1] = Lsum; }
      }
    }
  }
  if (S == 1) { __syncthreads(); return; }

  // ---- the last split of this kv head to finish merges all splits ----
  __syncthreads();
  STAMP(25);
  if (tid == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(&p.sync[4 + bh], 1u);
    reinterpret_cast<volatile int*>(c.scratch)[40] = (ticket == (unsigned)(S - 1));
    if (ticket == (unsigned)(S - 1)) p.sync[4 + bh] = 0;    // ready for the next layer
    __threadfence();
  }
  __syncthreads();
  STAMP(26);
  if (reinterpret_cast<volatile int*>(c.scratch)[40]) {
    for (int r = warp; r < G; r += WARPS) {
      const size_t base = ((size_t)bh * S) * G + r;           // + split * G
      float m = -INFINITY, l = 0.f;
      if (lane < S) {
        m = __ldcg(p.attn_ml + (base + (size_t)lane * G) * 2);
        l = __ldcg(p.attn_ml + (base + (size_t)lane * G) * 2 + 1);
      }
      float Mx = warp_max(m);
      if (Mx == -INFINITY) Mx = 0.f;
      const float wgt = l > 0.f ? exp2f(m - Mx) : 0.f;
      const float Lsum = warp_sum(wgt * l);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s0 = 0; s0 < S; s0 += 16) {
        float4 o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {           // all loads of the batch first
          const int s = s0 + j < S ? s0 + j : S - 1;
          o[j] = __ldcg(reinterpret_cast<const float4*>(p.attn_o + (base + (size_t)s * G) * 128) + lane);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float ws = (s0 + j < S) ? __shfl_sync(0xffffffffu, wgt, (s0 + j) & 31) : 0.f;
          acc[0] += ws * o[j].x; acc[1] += ws * o[j].y; acc[2] += ws * o[j].z; acc[3] += ws * o[j].w;
        }
      }
      const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
      uint2 packed;
      packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
      packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<uint2*>(p.attended + ((size_t)b * nq + kh * G + r) * 128 + lane * 4) = packed;
    }
  }
  __syncthreads();
}

// ---- SwiGLU phase (spread over the grid) -----------------------------------------------------
__device__ __noinline__ void swiglu_phase(const mega_params_t& p, const float* PG) {
  const int I = p.I;
  const long long stride = (long long)p.M * 2 * I;
  const unsigned C = (unsigned)p.gu.C, u = (unsigned)p.gu.U;
  if ((I & 3) == 0) {
    const long long quads = (long long)p.M * (I >> 2);
    for (long long qd = (long long)blockIdx.x * THREADS + threadIdx.x; qd < quads;
         qd += (long long)gridDim.x * THREADS) {
      const int m = (int)(qd / (I >> 2)), col = (int)(qd % (I >> 2)) * 4;
      // the layer's gate|up rows are interleaved in blocks of 8 (see q_gemm_swiglu): act
      // columns col..col+3 have their gate sums at 16*(col/8) + col%8 and their up sums 8 further
      const long long base = (long long)m * 2 * I;
      const int gcol = 16 * (col >> 3) + (col & 7), ucol = gcol + 8;
      const float4 g0 = __ldcg(reinterpret_cast<const float4*>(PG + base + gcol));
      const float4 g1 = __ldcg(reinterpret_cast<const float4*>(PG + base + gcol + stride));
      const float4 u0 = __ldcg(reinterpret_cast<const float4*>(PG + base + ucol));
      const float4 u1 = __ldcg(reinterpret_cast<const float4*>(PG + base + ucol + stride));
      const unsigned gg = (unsigned)gcol >> 4;
      const unsigned eg = ((gg + 1) * C - 1) / u - (gg * C) / u;
      const unsigned eu = eg;
      float gs[4] = {g0.x, g0.y, g0.z, g0.w}, us[4] = {u0.x, u0.y, u0.z, u0.w};
      if (eg > 0) { gs[0] += g1.x; gs[1] += g1.y; gs[2] += g1.z; gs[3] += g1.w; }
      if (eu > 0) { us[0] += u1.x; us[1] += u1.y; us[2] += u1.z; us[3] += u1.w; }
      for (unsigned k = 2; k <= eg; ++k) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(PG + base + gcol + (long long)k * stride));
        gs[0] += t.x; gs[1] += t.y; gs[2] += t.z; gs[3] += t.w;
      }
      for (unsigned k = 2; k <= eu; ++k) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(PG + base + ucol + (long long)k * stride));
        us[0] += t.x; us[1] += t.y; us[2] += t.z; us[3] += t.w;
      }
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float gt = bf16_round(gs[e]), up = bf16_round(us[e]);
        o[e] = bf16_round(gt / (1.0f + expf(-gt))) * up;
      }
      uint2 pk;
      pk.x = pack_bf16(o[0], o[1]);
      pk.y = pack_bf16(o[2], o[3]);
      *reinterpret_cast<uint2*>(p.act + (long long)m * I + col) = pk;
    }
    return;
  }
  const long long total = (long long)p.M * I;
  for (long long i = (long long)blockIdx.x * THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * THREADS) {
    const int m = (int)(i / I), col = (int)(i % I);
    const long long base = (long long)m * 2 * I;
    const int gcol = 16 * (col >> 3) + (col & 7), ucol = gcol + 8;
    const float gt = bf16_round(psum_cg(PG, p.gu, stride, base + gcol, gcol));
    const float up = bf16_round(psum_cg(PG, p.gu, stride, base + ucol, ucol));
    const float a = bf16_round(gt / (1.0f + expf(-gt)));
    p.act[i] = __float2bfloat16_rn(a * up);
  }
}

// ---- logits + argmax phase ----------------------------------------------------------------
__device__ __forceinline__ void better(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__device__ __forceinline__ void argmax_phase(const mega_params_t& p, Ctx& c, const float* PL) {
  const int V = p.V, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long stride = (long long)p.M * V;
  const int per = (V + gridDim.x - 1) / gridDim.x;
  const int c0 = blockIdx.x * per, c1 = min(V, c0 + per);
  float* sv = c.scratch;
  int* si = reinterpret_cast<int*>(c.scratch + 16);
  for (int m = 0; m < p.M; ++m) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int col = c0 + tid; col < c1; col += THREADS) {
      const long long i = (long long)m * V + col;
      const bf16 r = __float2bfloat16_rn(psum_cg(PL, p.head, stride, i, col));
      if (p.logits) p.logits[i] = r;
      float v = __bfloat162float(r);
      if (v != v) v = -INFINITY;
      better(bv, bi, v, col);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      better(bv, bi, ov, oi);
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int k = 1; k < WARPS; ++k) better(bv, bi, sv[k], si[k]);
      p.blk_val[(size_t)m * gridDim.x + blockIdx.x] = bv;
      p.blk_idx[(size_t)m * gridDim.x + blockIdx.x] = bi;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(&p.sync[2], 1u);
    reinterpret_cast<volatile int*>(c.scratch)[40] = (ticket == gridDim.x - 1);
    __threadfence();
  }
  __syncthreads();
  if (!reinterpret_cast<volatile int*>(c.scratch)[40]) return;
  for (int m = warp; m < p.M; m += WARPS) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = lane; k < (int)gridDim.x; k += 32)
      better(bv, bi, __ldcg(p.blk_val + (size_t)m * gridDim.x + k), __ldcg(p.blk_idx + (size_t)m * gridDim.x + k));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      better(bv, bi, ov, oi);
    }
    if (lane == 0) {
      if (bi == 0x7fffffff) bi = 0;
      p.arg_val[m] = bv;
      p.arg_idx[m] = bi;
      p.tokens[m] = bi;
    }
  }
  if (tid == 0) {
    p.pos[0] += 1;
    p.sync[2] = 0;
    p.sync[0] = 0;      // every CTA is past the last grid barrier: reset for the next launch
  }
}

__global__ void __launch_bounds__(THREADS, 1)
k_decode_mega(const __grid_constant__ mega_params_t p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  Ctx c;
  c.ring = smem;
  unsigned char* q = smem + RING_BYTES;
  c.red = reinterpret_cast<float*>(q); q += RED_FLOATS * 4;
  c.scratch = reinterpret_cast<float*>(q); q += 64 * 4;
  c.tags = reinterpret_cast<int*>(q); q += WARPS * 2 * 4;
  c.gbars = reinterpret_cast<uint64_t*>(q); q += WARPS * STAGES * 8;
  c.abars = reinterpret_cast<uint64_t*>(q); q += 2 * ATT_NS * 8;
  c.knew = reinterpret_cast<bf16*>(q); q += 256;
  c.vnew = reinterpret_cast<bf16*>(q); q += 256;
  c.cosrow = reinterpret_cast<bf16*>(q); q += 256;
  c.sinrow = reinterpret_cast<bf16*>(q); q += 256;
  c.resid = reinterpret_cast<bf16*>(q); q += (size_t)p.M * p.H * 2;
  c.xs = reinterpret_cast<bf16*>(q);
  c.g_count = 0;
  c.trace_gemm = 0;
  c.a_count = 0;
  c.epoch = 0;

  const int tid = threadIdx.x;
  c.pos = p.pos[0];
  if (tid < 128) {
    c.cosrow[tid] = p.cos[(size_t)c.pos * 128 + tid];
    c.sinrow[tid] = p.sin[(size_t)c.pos * 128 + tid];
  }
  if (tid == 0) {
    for (int i = 0; i < WARPS * STAGES; ++i) mbar_init(smem_u32(&c.gbars[i]), 1);
    for (int i = 0; i < ATT_NS; ++i) {
      mbar_init(smem_u32(&c.abars[i]), 1);
      mbar_init(smem_u32(&c.abars[ATT_NS + i]), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  const int Kmax = p.xs_cols;
  float* buf0 = p.buf0;
  float* buf1 = p.buf1;

  GemmRun run = gemm_prime(p.layers[0].wqkv, p.qkv, c);
  prologue_embed(p, c, p.layers[0].ln_in);
  for (int l = 0; l < p.L; ++l) {
    const mega_layer_t& Lw = p.layers[l];
    const bool tracing = (l == p.trace_layer) && (blockIdx.x == 0 || blockIdx.x == 100);
    TRACE(0);
    // A: QKV projection (operand xs = normed hidden, prepared by the previous prologue)
    c.trace_gemm = tracing ? 1 : 0;
    gemm_run(run, p.qkv, p.M, c.xs, buf0, c);
    if (p.prefetch_units > 0) {          // attention is long: O-proj and gate|up can come in behind it
      l2_prefetch_run(Lw.wo, p.o, 0, p.prefetch_units);
      l2_prefetch_run(Lw.wgu, p.gu, 0, p.prefetch_units);
    }
    TRACE(1);
    grid_barrier(p, c);
    TRACE(2);
    // B: attention (reuses the ring), then prime O-proj
    attention_phase(p, c, Lw, buf0);
    TRACE(3);
    grid_arrive(p, c);
    run = gemm_prime(Lw.wo, p.o, c);         // the copy issue overlaps the barrier wait
    grid_wait(p, c);
    TRACE(4);
    // C: O projection
    stage_x(p, c, p.attended, p.o.K);
    TRACE(5);
    if (l == p.trace_layer && threadIdx.x == 0) {
      unsigned sm;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
      g_mega_trace[64 + blockIdx.x] = sm;
    }
    gemm_run(run, p.o, p.M, c.xs, buf1, c);
    if (l == p.trace_layer && threadIdx.x == 0) g_mega_trace[64 + 160 + blockIdx.x] = gtime();
    TRACE(6);
    grid_arrive(p, c);
    run = gemm_prime(Lw.wgu, p.gu, c);
    grid_wait(p, c);
    TRACE(7);
    // D: add + norm, gate|up projection
    prologue_add_norm(p, c, buf1, p.o, Lw.ln_post);
    c.trace_gemm = 0;
    TRACE(8);
    if (l == p.trace_layer && threadIdx.x == 0) g_mega_trace[64 + 320 + blockIdx.x] = gtime();
    gemm_run(run, p.gu, p.M, c.xs, buf0, c);
    if (l == p.trace_layer && threadIdx.x == 0) g_mega_trace[64 + 480 + blockIdx.x] = gtime();
    TRACE(9);
    run = gemm_prime(Lw.wdown, p.down, c);
    if (p.prefetch_units > 0) l2_prefetch_run(Lw.wdown, p.down, STAGES * STAGE_UNITS, p.prefetch_units);
    grid_barrier(p, c);
    TRACE(10);
    // E: SwiGLU
    swiglu_phase(p, buf0);
    TRACE(11);
    grid_barrier(p, c);
    TRACE(12);
    // F: down projection
    stage_x(p, c, p.act, p.down.K);
    TRACE(13);
    gemm_run(run, p.down, p.M, c.xs, buf1, c);
    TRACE(14);
    const bool last = (l + 1 == p.L);
    run = last ? gemm_prime(p.lm_head, p.head, c) : gemm_prime(p.layers[l + 1].wqkv, p.qkv, c);
    if (p.prefetch_units > 0) {
      if (last) l2_prefetch_run(p.lm_head, p.head, STAGES * STAGE_UNITS, p.prefetch_units);
      else l2_prefetch_run(p.layers[l + 1].wqkv, p.qkv, STAGES * STAGE_UNITS, p.prefetch_units);
    }
    grid_barrier(p, c);
    TRACE(15);
    prologue_add_norm(p, c, buf1, p.down, last ? p.ln_final : p.layers[l + 1].ln_in);
    TRACE(16);
  }
  (void)Kmax;
  gemm_run(run, p.head, p.M, c.xs, buf0, c);
  grid_barrier(p, c);
  argmax_phase(p, c, buf0);
}

}  // namespace

int q_mega_trace_read(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_mega_trace, sizeof(unsigned long long) * (64 + 640)) == cudaSuccess ? 0 : -1;
}

int q_mega_status_read(int32_t out[4]) {
  return cudaMemcpyFromSymbol(out, g_mega_status, sizeof(int) * 4) == cudaSuccess ? 0 : -1;
}

size_t q_mega_smem_bytes(int M, int H, int xs_cols) {
  return (size_t)RING_BYTES + RED_FLOATS * 4 + 64 * 4 + WARPS * 2 * 4 + WARPS * STAGES * 8 + 2 * ATT_NS * 8 +
         1024 + (size_t)M * H * 2 + (size_t)M * xs_cols * 2 + 64;
}

cudaError_t q_mega_launch(const mega_params_t& p, int grid, cudaStream_t stream) {
  const size_t smem = q_mega_smem_bytes(p.M, p.H, p.xs_cols);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(k_decode_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, k_decode_mega, p);
}
