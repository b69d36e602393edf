// Split-KV GQA attention for 1..8 query tokens per sequence over a paged bf16 KV
// cache (reference: engine/kernels/small_query_attention.py:41-110 is the
// single-token version over a contiguous cache).
//
// One CTA = one (sequence, kv head) x one key split. Warp 4 is the producer: a
// single lane walks the block table and brings each 64-key page tile (K 16 KB +
// V 16 KB, already XOR-swizzled in global memory) into a shared-memory ring with
// cp.async.bulk + mbarrier transaction counts. Warps 0..3 are consumers: every
// consumer owns 16 of the 64 keys of each tile, computes S = Q K^T and P V with
// mma.m16n8k16 (all T*G query rows of the kv head share the tile), and keeps its
// own online-softmax state; the four states are merged once at the end through
// shared memory. Cast boundaries: fp32 scores from bf16 q,k; fp32 statistics;
// P rounded to bf16 for P V; fp32 accumulation; a single bf16 rounding after all
// splits are merged (k_attn_merge).
//
// Every mbarrier wait is bounded: when it runs out the thread records a code in
// the device status word and the CTA stops consuming, so a lost copy can never
// hang the GPU.
#include "common.cuh"

extern int g_attn_no_cluster;   // q_set_option "attn_no_cluster": merge splits through global memory

namespace {

constexpr int NS = 3;                      // ring stages
constexpr int TILE_BYTES = 64 * 128 * 2;   // one K or V page tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr int MAX_CLUSTER = 16;            // most key splits that merge inside one thread-block cluster
constexpr unsigned WAIT_LIMIT = 1u << 22;

__device__ int g_status[4];
// Measurement aid: phase stamps (ns) of CTA (0,0) of the last decode-attention launch that had a
// timeline record: start, past the wait, heads normed, tiles done, CTA merged, cluster merged, end.
__device__ unsigned long long g_attn_trace[8];

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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait; false when the limit ran out.
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
    if (it > 64) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
}

// RT = number of 16-row query tiles (T*G <= 16*RT).
template <int RT>
__global__ void __launch_bounds__(THREADS)
k_attn_split(const bf16* __restrict__ Q, const char* __restrict__ kpool,
             const char* __restrict__ vpool, const int32_t* __restrict__ block_table,
             int pages_per_seq, const int32_t* __restrict__ pos_ptr, float* __restrict__ part_o,
             float* __restrict__ part_ml, bf16* __restrict__ out, int T, int G, int nq, int nkv,
             int S, float scale_log2) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* stages = smem;                               // NS * STAGE_BYTES
  unsigned char* qtile = smem + NS * STAGE_BYTES;             // RT*16 rows * 256 B
  uint64_t* bars = reinterpret_cast<uint64_t*>(qtile + RT * 16 * 256);  // full[NS], empty[NS]
  __shared__ int s_fail;

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y, split = blockIdx.x;
  const int b = bh / nkv, kh = bh % nkv;
  const int R = T * G;

  if (tid == 0) {
    s_fail = 0;
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[NS + i]), CONSUMERS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // pos, the block table and every key/value row older than this step's query block were
  // written by earlier steps (earlier graph launches), so they may be read before the
  // dependency wait; only tiles that can hold the T newest rows must wait for the kernel
  // that writes them.
  const int pos = pos_ptr[0];
  const int max_limit = pos + T;                                   // keys visible to the last row
  const int tiles_used = (max_limit + Q_PAGE_TOKENS - 1) / Q_PAGE_TOKENS;
  // tiles are dealt out evenly: the first (tiles_used % S) splits get one more
  const int tbase = tiles_used / S, trem = tiles_used - tbase * S;
  const int tile0 = split * tbase + min(split, trem);
  const int tile1 = tile0 + tbase + (split < trem ? 1 : 0);
  const int ntiles = tile1 - tile0;
  const int first_new_tile = pos / Q_PAGE_TOKENS;                  // tiles >= this may change in this step

  if (warp == CONSUMERS) {
    // ---------------- producer ----------------
    if (lane == 0) {
      bool waited = false;
      for (int it = 0; it < ntiles; ++it) {
        const int s = it % NS;
        if (!waited && tile0 + it >= first_new_tile) {
          pdl_wait();
          waited = true;
        }
        if (it >= NS) {
          if (!mbar_wait(smem_u32(&bars[NS + s]), ((it / NS) - 1) & 1)) {
            atomicExch(&g_status[0], 1);
            atomicExch(&s_fail, 1);
            break;
          }
        }
        const int page = block_table[(size_t)b * pages_per_seq + tile0 + it];
        const size_t off = ((size_t)page * nkv + kh) * TILE_BYTES;
        const uint32_t bar = smem_u32(&bars[s]);
        mbar_expect_tx(bar, STAGE_BYTES);
        bulk_g2s(smem_u32(stages + s * STAGE_BYTES), kpool + off, TILE_BYTES, bar);
        bulk_g2s(smem_u32(stages + s * STAGE_BYTES + TILE_BYTES), vpool + off, TILE_BYTES, bar);
      }
      if (!waited) pdl_wait();
    }
  } else {
    // ---------------- consumers ----------------
    pdl_wait();                 // Q (and the newest K/V rows) come from the previous kernel
    // Q tile -> shared memory (swizzled rows of 256 B); rows >= R are zero.
    for (int c = tid; c < RT * 16 * 16; c += CONSUMERS * 32) {
      const int r = c >> 4, ch = c & 15;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < R) {
        const int t = r / G, gq = r % G;
        const bf16* src = Q + (((size_t)(b * T + t)) * nq + kh * G + gq) * 128 + ch * 8;
        v = *reinterpret_cast<const uint4*>(src);
      }
      *reinterpret_cast<uint4*>(qtile + r * 256 + ((ch ^ (r & 7)) << 4)) = v;
    }
    consumer_sync();

    const int g = lane >> 2, t4 = lane & 3;
    float m_run[RT][2], l_run[RT][2];
    float oacc[RT][16][4];
    int limit[RT][2];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        m_run[rt][h] = -INFINITY;
        l_run[rt][h] = 0.f;
        const int r = rt * 16 + g + 8 * h;
        limit[rt][h] = r < R ? pos + r / G + 1 : max_limit;
      }
#pragma unroll
      for (int n = 0; n < 16; ++n) oacc[rt][n][0] = oacc[rt][n][1] = oacc[rt][n][2] = oacc[rt][n][3] = 0.f;
    }
    const uint32_t q_base = smem_u32(qtile);
    bool alive = true;

    for (int it = 0; it < ntiles && alive; ++it) {
      const int s = it % NS;
      if (!mbar_wait(smem_u32(&bars[s]), (it / NS) & 1)) {
        atomicExch(&g_status[0], 2);
        alive = false;
        break;
      }
      unsigned char* kt = stages + s * STAGE_BYTES;
      unsigned char* vt = kt + TILE_BYTES;
      const int key_base = (tile0 + it) * Q_PAGE_TOKENS;
      const int my_key0 = key_base + warp * 16;
      if (my_key0 + 16 > max_limit) {
        // rows past the newest key may hold stale bits: clear the V rows so that
        // 0 * garbage cannot produce NaN in P V.
        for (int c = lane; c < 16 * 16; c += 32) {
          const int kr = warp * 16 + (c >> 4);
          if (key_base + kr >= max_limit)
            *reinterpret_cast<uint4*>(vt + kr * 256 + ((c & 15) << 4)) = make_uint4(0, 0, 0, 0);
        }
        __syncwarp();
      }
      const uint32_t k_base = smem_u32(kt), v_base = smem_u32(vt);

#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        float sacc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
          {
            const int row = rt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
            const int ch = 2 * ks + (lane >> 4);
            ldsm_x4(q_base + row * 256 + ((ch ^ (row & 7)) << 4), a0, a1, a2, a3);
          }
          {
            const int mi = lane >> 3;
            const int key = warp * 16 + 8 * (mi >> 1) + (lane & 7);
            const int ch = 2 * ks + (mi & 1);
            ldsm_x4(k_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
          }
          mma16816(sacc[0], a0, a1, a2, a3, b0, b1);
          mma16816(sacc[1], a0, a1, a2, a3, b2, b3);
        }
        // online softmax for rows g (h=0) and g+8 (h=1)
        float p[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float mx = -INFINITY;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int key = my_key0 + 8 * j + 2 * t4 + e;
              float v = sacc[j][2 * h + e] * scale_log2;
              v = key < limit[rt][h] ? v : -INFINITY;
              sacc[j][2 * h + e] = v;
              mx = fmaxf(mx, v);
            }
          }
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float m_new = fmaxf(m_run[rt][h], mx);
          const float m_safe = m_new == -INFINITY ? 0.f : m_new;
          const float resc = exp2f(m_run[rt][h] - m_safe);   // exp2(-inf) = 0 on the first tile
          float sum = 0.f;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float pv = exp2f(sacc[j][2 * h + e] - m_safe);
              p[j][2 * h + e] = pv;
              sum += pv;
            }
          }
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          l_run[rt][h] = l_run[rt][h] * resc + sum;
          m_run[rt][h] = m_new;
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            oacc[rt][n][2 * h] *= resc;
            oacc[rt][n][2 * h + 1] *= resc;
          }
        }
        const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]);
        const uint32_t pa1 = pack_bf16(p[0][2], p[0][3]);
        const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]);
        const uint32_t pa3 = pack_bf16(p[1][2], p[1][3]);
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          uint32_t b0, b1, b2, b3;
          const int mi = lane >> 3;
          const int key = warp * 16 + 8 * (mi & 1) + (lane & 7);
          const int ch = 2 * dp + (mi >> 1);
          ldsm_x4_t(v_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
          mma16816(oacc[rt][2 * dp], pa0, pa1, pa2, pa3, b0, b1);
          mma16816(oacc[rt][2 * dp + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[NS + s]));
    }
    if (!alive) atomicExch(&s_fail, 1);

    // ---- merge the four consumer states through shared memory ----
    consumer_sync();   // every consumer is done with the ring
    if (s_fail == 0) {
      float* mo = reinterpret_cast<float*>(stages);                      // [4][RT*16][128]
      float* mml = mo + CONSUMERS * RT * 16 * 128;                       // [4][RT*16][2]
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = rt * 16 + g + 8 * h;
          float* dst = mo + ((size_t)warp * RT * 16 + r) * 128;
#pragma unroll
          for (int n = 0; n < 16; ++n) {
            dst[8 * n + 2 * t4] = oacc[rt][n][2 * h];
            dst[8 * n + 2 * t4 + 1] = oacc[rt][n][2 * h + 1];
          }
          if (t4 == 0) {
            mml[((size_t)warp * RT * 16 + r) * 2] = m_run[rt][h];
            mml[((size_t)warp * RT * 16 + r) * 2 + 1] = l_run[rt][h];
          }
        }
      }
      consumer_sync();
      const int d = tid;  // 128 consumer threads = 128 dims
      for (int r = 0; r < R; ++r) {
        float mw[CONSUMERS], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
          mw[w] = mml[((size_t)w * RT * 16 + r) * 2];
          M = fmaxf(M, mw[w]);
        }
        const float Ms = M == -INFINITY ? 0.f : M;
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMERS; ++w) {
          const float wt = exp2f(mw[w] - Ms);
          L += wt * mml[((size_t)w * RT * 16 + r) * 2 + 1];
          O += wt * mo[((size_t)w * RT * 16 + r) * 128 + d];
        }
        if (S == 1) {
          const int t = r / G, gq = r % G;
          const float res = L > 0.f ? O / L : 0.f;
          out[(((size_t)(b * T + t)) * nq + kh * G + gq) * 128 + d] = __float2bfloat16_rn(res);
        } else {
          const size_t row = ((size_t)bh * S + split) * R + r;
          part_o[row * 128 + d] = O;
          if (d == 0) {
            part_ml[row * 2] = M;
            part_ml[row * 2 + 1] = L;
          }
        }
      }
    }
  }
}

// One warp per (sequence, token, q head): lanes hold one split each for the
// log-sum-exp weights (shuffle reductions), then every lane sums 4 dims.
__global__ void __launch_bounds__(128)
k_attn_merge(const float* __restrict__ part_o, const float* __restrict__ part_ml,
             bf16* __restrict__ out, int batch, int T, int G, int nq, int nkv, int S) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= batch * T * nq) return;
  const int head = item % nq, bt = item / nq;
  const int b = bt / T, t = bt % T;
  const int kh = head / G, gq = head % G;
  const int R = T * G, r = t * G + gq;
  const size_t base = ((size_t)(b * nkv + kh) * S) * R + r;   // + split * R
  float m = -INFINITY, l = 0.f;
  if (lane < S) {
    m = part_ml[(base + (size_t)lane * R) * 2];
    l = part_ml[(base + (size_t)lane * R) * 2 + 1];
  }
  float M = warp_max(m);
  if (M == -INFINITY) M = 0.f;
  const float wgt = l > 0.f ? exp2f(m - M) : 0.f;
  const float L = warp_sum(wgt * l);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  // every split wrote its (possibly neutral, all-zero) partial; 16 loads are issued together
  for (int s0 = 0; s0 < S; s0 += 16) {
    float4 o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int s = s0 + j < S ? s0 + j : S - 1;
      o[j] = *reinterpret_cast<const float4*>(part_o + (base + (size_t)s * R) * 128 + lane * 4);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float ws = (s0 + j < S) ? __shfl_sync(0xffffffffu, wgt, (s0 + j) & 31) : 0.f;
      acc[0] += ws * o[j].x; acc[1] += ws * o[j].y; acc[2] += ws * o[j].z; acc[3] += ws * o[j].w;
    }
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  bf16* dst = out + ((size_t)bt * nq + head) * 128 + lane * 4;
  uint2 packed;
  packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
  packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(dst) = packed;
}


// ---- single-token decode attention with everything around it folded in -----------------
// q/k head norm + RoPE + K/V page write (engine/kernels/decode_fused.py:59-118), the
// split-KV attention above for T = 1, and the split merge (k_attn_merge) as the job of
// the last split of a kv head to finish (a ticket counter, no spinning): one kernel per
// layer instead of three. The newest key/value row is computed here, so NOTHING this
// kernel streams from the KV pages depends on the previous kernel: the producer requests
// all its tiles before the dependency wait, and the consumer that owns the newest key
// patches that row into the shared-memory tile (and the owner split writes it to the page
// for later steps).
// CL: the S splits of a kv head are one thread-block cluster (S <= 16) and merge through
// distributed shared memory: every CTA parks its (max, sum, O) rows in its own shared
// memory, the cluster synchronises once, and CTA r of the cluster combines 1/S of the
// (row, dim) outputs from all S CTAs in split order. No global round trips, no tickets.
template <bool CL, int DG>
__global__ void __launch_bounds__((4 * DG + 1) * 32)
k_attn_decode(const float* __restrict__ PQ, PlanView pv, const bf16* __restrict__ QG,
              const bf16* __restrict__ KG, const bf16* __restrict__ COS, const bf16* __restrict__ SIN,
              const int32_t* __restrict__ pos_ptr, char* __restrict__ kpool, char* __restrict__ vpool,
              const int32_t* __restrict__ block_table, int pages_per_seq, float* __restrict__ part_o,
              float* __restrict__ part_ml, unsigned int* __restrict__ tickets, bf16* __restrict__ out,
              int rows, int G, int nq, int nkv, int S, float scale_log2, float eps, int ring_stages,
              unsigned long long* tl) {
  // Ring depth is a launch parameter here: a split that can never see more than one or
  // two tiles asks for that much shared memory only, so this CTA fits on an SM beside a
  // weight-streaming GEMM CTA (the next projection primes its ring during the attention).
  const int NS = ring_stages;
  constexpr int DC = 4 * DG;                 // consumer warps: DG groups of four, one tile per group at a time
  constexpr int DT = (DC + 1) * 32;          // threads; warp DC is the producer
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* stages = smem;                               // NS * STAGE_BYTES
  unsigned char* qtile = smem + NS * STAGE_BYTES;             // 16 rows * 256 B
  uint64_t* bars = reinterpret_cast<uint64_t*>(qtile + 16 * 256);       // full[NS], empty[NS]
  bf16* knew = reinterpret_cast<bf16*>(bars + 2 * NS);        // [128]
  bf16* vnew = knew + 128;                                    // [128]
  // Cluster merge: every CTA of the cluster stores its part of the rows THIS CTA combines
  // here ([S][share] sums, then from float G*128+16 on [S][G][2] max / sum of weights), outside the ring, which a
  // slower CTA is still using when a faster one delivers.
  float* recv = reinterpret_cast<float*>(vnew + 128);
  __shared__ int s_last;

  tl_begin(tl);
  const bool stamp = tl != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
  if (stamp) g_attn_trace[0] = tl_now();
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y, split = blockIdx.x;
  const int b = bh / nkv, kh = bh % nkv;
  if (tid == 0) {
    for (int i = 0; i < NS; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[NS + i]), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // position and block table were written by earlier steps: safe before the wait. The
  // producer warp fetches this sequence's block-table row together with the position (one
  // memory round trip instead of two before the first KV copy can be issued).
  int my_page = 0;
  if (warp == DC && lane < pages_per_seq) my_page = block_table[(size_t)b * pages_per_seq + lane];
  const int pos = pos_ptr[0];
  const int max_limit = pos + 1;
  const int tiles_used = (max_limit + Q_PAGE_TOKENS - 1) / Q_PAGE_TOKENS;
  // tiles are dealt out evenly: the first (tiles_used % S) splits get one more
  const int tbase = tiles_used / S, trem = tiles_used - tbase * S;
  const int tile0 = split * tbase + min(split, trem);
  const int tile1 = tile0 + tbase + (split < trem ? 1 : 0);
  const int ntiles = tile1 - tile0;
  const int new_tile = pos / Q_PAGE_TOKENS, new_row = pos % Q_PAGE_TOKENS;
  const bool owns_new = ntiles > 0 && new_tile >= tile0 && new_tile < tile1;

  if (warp == DC) {
    for (int it = 0; it < ntiles && it < NS; ++it) {
      const int tile = tile0 + it;
      int page = __shfl_sync(0xffffffffu, my_page, tile & 31);
      if (tile >= 32) page = block_table[(size_t)b * pages_per_seq + tile];
      if (lane == 0) {
        const size_t off = ((size_t)page * nkv + kh) * TILE_BYTES;
        const uint32_t bar = smem_u32(&bars[it]);
        mbar_expect_tx(bar, STAGE_BYTES);
        bulk_g2s(smem_u32(stages + it * STAGE_BYTES), kpool + off, TILE_BYTES, bar);
        bulk_g2s(smem_u32(stages + it * STAGE_BYTES + TILE_BYTES), vpool + off, TILE_BYTES, bar);
      }
    }
  }

  // Gains and the rotary row of this position do not depend on the projection: the warp's
  // first item asks for them before the wait, so only the partials are fetched after it.
  uint2 graw0 = make_uint2(0, 0), craw0 = make_uint2(0, 0), sraw0 = make_uint2(0, 0);
  if (warp < G + 1) {
    graw0 = *reinterpret_cast<const uint2*>((warp < G ? QG : KG) + 4 * lane);
    craw0 = *reinterpret_cast<const uint2*>(COS + (size_t)pos * 128 + 4 * lane);
    sraw0 = *reinterpret_cast<const uint2*>(SIN + (size_t)pos * 128 + 4 * lane);
  }

  pdl_wait();          // the QKV partials are complete from here on
  tl_waited(tl);
  if (stamp) g_attn_trace[1] = tl_now();

  // ---- q/k head norm + RoPE (+ v): lane l owns dims 4l..4l+3. Items 0..G-1 are the query
  // heads; item G is the key head TOGETHER with the value head (its loads ride along), so
  // that with 4 query heads per kv head every warp has one item and one memory round trip.
  {
    const int width = (nq + 2 * nkv) * 128;
    for (int h = warp; h < G + 1; h += DC + 1) {
      const bool is_q = h < G;
      const int head = is_q ? kh * G + h : nq + kh;
      const long long src = (long long)b * width + (long long)head * 128 + 4 * lane;
      const long long vsrc = (long long)b * width + (long long)(nq + nkv + kh) * 128 + 4 * lane;
      // Up to four partial slots per column (the tcgen05 plan splits the packed projection
      // four ways) are requested together; anything beyond comes one at a time.
      const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
      const int extra = plan_count(pv, head * 128 + 4 * lane) - 1;
      const int vextra = is_q ? 0 : plan_count(pv, (nq + nkv + kh) * 128 + 4 * lane) - 1;
      float4 sq[4], sv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        sq[k] = (k == 0 || (pv.u != 0 && k <= extra)) ? *reinterpret_cast<const float4*>(PQ + src + (long long)k * pv.slot_stride) : z4;
        sv[k] = (!is_q && (k == 0 || (pv.u != 0 && k <= vextra)))
                    ? *reinterpret_cast<const float4*>(PQ + vsrc + (long long)k * pv.slot_stride) : z4;
      }
      uint2 graw = graw0, craw = craw0, sraw = sraw0;
      if (h != warp) {
        graw = *reinterpret_cast<const uint2*>((is_q ? QG : KG) + 4 * lane);
        craw = *reinterpret_cast<const uint2*>(COS + (size_t)pos * 128 + 4 * lane);
        sraw = *reinterpret_cast<const uint2*>(SIN + (size_t)pos * 128 + 4 * lane);
      }
      if (!is_q) {
        float x[4] = {sv[0].x, sv[0].y, sv[0].z, sv[0].w};
#pragma unroll
        for (int k = 1; k < 4; ++k)
          if (k <= vextra) { x[0] += sv[k].x; x[1] += sv[k].y; x[2] += sv[k].z; x[3] += sv[k].w; }
        for (int k = 4; k <= vextra; ++k) {
          const float4 sk = *reinterpret_cast<const float4*>(PQ + vsrc + (long long)k * pv.slot_stride);
          x[0] += sk.x; x[1] += sk.y; x[2] += sk.z; x[3] += sk.w;
        }
        uint2 o;
        o.x = pack_bf16(x[0], x[1]);
        o.y = pack_bf16(x[2], x[3]);
        *reinterpret_cast<uint2*>(vnew + 4 * lane) = o;
      }
      float x[4] = {sq[0].x, sq[0].y, sq[0].z, sq[0].w};
#pragma unroll
      for (int k = 1; k < 4; ++k)
        if (k <= extra) { x[0] += sq[k].x; x[1] += sq[k].y; x[2] += sq[k].z; x[3] += sq[k].w; }
      for (int k = 4; k <= extra; ++k) {
        const float4 sk = *reinterpret_cast<const float4*>(PQ + src + (long long)k * pv.slot_stride);
        x[0] += sk.x; x[1] += sk.y; x[2] += sk.z; x[3] += sk.w;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = bf16_round(x[e]);
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / 128.f + eps);
      const float gv[4] = {bf_lo(graw.x), bf_hi(graw.x), bf_lo(graw.y), bf_hi(graw.y)};
      const float cs[4] = {bf_lo(craw.x), bf_hi(craw.x), bf_lo(craw.y), bf_hi(craw.y)};
      const float sn[4] = {bf_lo(sraw.x), bf_hi(sraw.x), bf_lo(sraw.y), bf_hi(sraw.y)};
      float outv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float n = bf16_round(bf16_round(x[e] * inv) * gv[e]);
        const float partner = __shfl_xor_sync(0xffffffffu, n, 16);
        const float rot = lane < 16 ? -partner : partner;
        outv[e] = bf16_round(n * cs[e]) + bf16_round(rot * sn[e]);
      }
      uint2 o;
      o.x = pack_bf16(outv[0], outv[1]);
      o.y = pack_bf16(outv[2], outv[3]);
      if (is_q) {
        *reinterpret_cast<uint2*>(qtile + h * 256 + (((lane >> 1) ^ (h & 7)) << 4) + (lane & 1) * 8) = o;
      } else {
        *reinterpret_cast<uint2*>(knew + 4 * lane) = o;
      }
    }
    for (int i = tid; i < (16 - G) * 16; i += DT) {       // query rows G..15 are zero
      const int r = G + (i >> 4), ch = i & 15;
      *reinterpret_cast<uint4*>(qtile + r * 256 + ((ch ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
    }
  }
  __syncthreads();
  if (stamp) g_attn_trace[2] = tl_now();
  if (owns_new && tid < 16) {
    // the newest key/value row goes to its page for later steps
    const int page = block_table[(size_t)b * pages_per_seq + new_tile];
    const size_t tile = ((size_t)page * nkv + kh) * TILE_BYTES;
    const int off = new_row * 256 + ((tid ^ (new_row & 7)) << 4);
    *reinterpret_cast<uint4*>(kpool + tile + off) = *reinterpret_cast<const uint4*>(knew + tid * 8);
    *reinterpret_cast<uint4*>(vpool + tile + off) = *reinterpret_cast<const uint4*>(vnew + tid * 8);
  }

  if (warp == DC) {
    if (lane == 0) {
      for (int it = NS; it < ntiles; ++it) {
        const int s = it % NS;
        if (!mbar_wait(smem_u32(&bars[NS + s]), ((it / NS) - 1) & 1)) {
          atomicExch(&g_status[0], 1);
          break;
        }
        const int page = block_table[(size_t)b * pages_per_seq + tile0 + it];
        const size_t off = ((size_t)page * nkv + kh) * TILE_BYTES;
        const uint32_t bar = smem_u32(&bars[s]);
        mbar_expect_tx(bar, STAGE_BYTES);
        bulk_g2s(smem_u32(stages + s * STAGE_BYTES), kpool + off, TILE_BYTES, bar);
        bulk_g2s(smem_u32(stages + s * STAGE_BYTES + TILE_BYTES), vpool + off, TILE_BYTES, bar);
      }
    }
  } else {
    const int g = lane >> 2, t4 = lane & 3;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float oacc[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
    const uint32_t q_base = smem_u32(qtile);
    const int grp = warp >> 2, wk = warp & 3;       // tile lane of the warp's group, key quarter of the warp
    for (int it = grp; it < ntiles; it += DG) {
      const int s = it % NS;
      if (!mbar_wait(smem_u32(&bars[s]), (it / NS) & 1)) {
        atomicExch(&g_status[0], 2);
        break;
      }
      unsigned char* kt = stages + s * STAGE_BYTES;
      unsigned char* vt = kt + TILE_BYTES;
      const int key_base = (tile0 + it) * Q_PAGE_TOKENS;
      const int my_key0 = key_base + wk * 16;
      if (my_key0 + 16 > max_limit) {
        for (int i = lane; i < 16 * 16; i += 32) {
          const int kr = wk * 16 + (i >> 4);
          if (key_base + kr >= max_limit)
            *reinterpret_cast<uint4*>(vt + kr * 256 + ((i & 15) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      if (tile0 + it == new_tile && (new_row >> 4) == wk && lane < 16) {
        const int off = new_row * 256 + ((lane ^ (new_row & 7)) << 4);
        *reinterpret_cast<uint4*>(kt + off) = *reinterpret_cast<const uint4*>(knew + lane * 8);
        *reinterpret_cast<uint4*>(vt + off) = *reinterpret_cast<const uint4*>(vnew + lane * 8);
      }
      __syncwarp();
      const uint32_t k_base = smem_u32(kt), v_base = smem_u32(vt);
      // the eight k-steps go to four independent accumulator sets (an MMA's result is ~280
      // cycles away), added at the end
      float sset[4][2][4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 2; ++j) sset[q][j][0] = sset[q][j][1] = sset[q][j][2] = sset[q][j][3] = 0.f;
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
          const int key = wk * 16 + 8 * (mi >> 1) + (lane & 7);
          const int ch = 2 * ks + (mi & 1);
          ldsm_x4(k_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        }
        mma16816(sset[ks & 3][0], a0, a1, a2, a3, b0, b1);
        mma16816(sset[ks & 3][1], a0, a1, a2, a3, b2, b3);
      }
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[j][e] = (sset[0][j][e] + sset[1][j][e]) + (sset[2][j][e] + sset[3][j][e]);
      float pr[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = my_key0 + 8 * j + 2 * t4 + e;
            float v = sacc[j][2 * h + e] * scale_log2;
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
            const float pv2 = exp2f(sacc[j][2 * h + e] - m_safe);
            pr[j][2 * h + e] = pv2;
            sum += pv2;
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
        const int key = wk * 16 + 8 * (mi & 1) + (lane & 7);
        const int ch = 2 * dp + (mi >> 1);
        ldsm_x4_t(v_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
        mma16816(oacc[2 * dp], pa0, pa1, pa2, pa3, b0, b1);
        mma16816(oacc[2 * dp + 1], pa0, pa1, pa2, pa3, b2, b3);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[NS + s]));
    }
    if (stamp) g_attn_trace[3] = tl_now();
    // merge the consumer warps' states through shared memory (only the G real query rows)
    asm volatile("bar.sync 1, %0;" ::"n"(DC * 32) : "memory");
    float* mo = reinterpret_cast<float*>(stages);            // [DC][G][128]
    float* mml = mo + DC * G * 128;                          // [DC][G][2]
    if (g < G) {
      float* dst = mo + ((size_t)warp * G + g) * 128;
#pragma unroll
      for (int n = 0; n < 16; ++n)
        *reinterpret_cast<float2*>(dst + 8 * n + 2 * t4) = make_float2(oacc[n][0], oacc[n][1]);
      if (t4 == 0) {
        mml[((size_t)warp * G + g) * 2] = m_run[0];
        mml[((size_t)warp * G + g) * 2 + 1] = l_run[0];
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DC * 32) : "memory");
    const int d = tid & 127;
    for (int r = tid >> 7; r < G; r += DG) {
      float mw[DC], Mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < DC; ++w) { mw[w] = mml[((size_t)w * G + r) * 2]; Mx = fmaxf(Mx, mw[w]); }
      const float Ms = Mx == -INFINITY ? 0.f : Mx;
      float Lsum = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < DC; ++w) {
        const float wt = exp2f(mw[w] - Ms);
        Lsum += wt * mml[((size_t)w * G + r) * 2 + 1];
        O += wt * mo[((size_t)w * G + r) * 128 + d];
      }
      if (S == 1) {
        out[((size_t)b * nq + kh * G + r) * 128 + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
      } else if (CL) {
        // deliver to the CTA that combines this (row, dim): slot `split` of its receive area
        const int total = G * 128, share = (total + S - 1) / S;
        const int v = r * 128 + d, owner = v / share;
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(recv)), "r"(owner));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote + (uint32_t)(split * share + (v - owner * share)) * 4u), "f"(O) : "memory");
        if (d < S) {
          // the row's max and sum of weights go to every CTA of the cluster (thread d -> CTA d)
          const uint32_t ml_off = (uint32_t)((total + 16) + (split * G + r) * 2) * 4u;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(recv)), "r"(d));
          asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote + ml_off), "f"(Mx), "f"(Lsum) : "memory");
        }
      } else {
        const size_t row = ((size_t)bh * S + split) * G + r;
        part_o[row * 128 + d] = O;
        if (d == 0) { part_ml[row * 2] = Mx; part_ml[row * 2 + 1] = Lsum; }
      }
    }
  }
  if (stamp) g_attn_trace[4] = tl_now();
  if (S == 1) { tl_end(tl); return; }
  if (CL) {
    // every thread of every CTA of the cluster arrives (idle splits too: they parked sum 0)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (stamp) g_attn_trace[5] = tl_now();
    // Everything this CTA combines is in its own receive area now: no remote reads, so no
    // second barrier before it may leave.
    const int total = G * 128;
    const int share = (total + S - 1) / S;
    const float* rml = recv + (total + 16);
    for (int i = tid; i < share; i += DT) {
      const int v = split * share + i;
      if (v >= total) break;
      const int r = v >> 7, d = v & 127;
      float Mx = -INFINITY;
      for (int s = 0; s < S; ++s) {
        const float2 ml = *reinterpret_cast<const float2*>(rml + (s * G + r) * 2);
        Mx = fmaxf(Mx, ml.y > 0.f ? ml.x : -INFINITY);
      }
      if (Mx == -INFINITY) Mx = 0.f;
      float Lsum = 0.f, O = 0.f;
      for (int s = 0; s < S; ++s) {
        const float2 ml = *reinterpret_cast<const float2*>(rml + (s * G + r) * 2);
        const float wgt = ml.y > 0.f ? exp2f(ml.x - Mx) : 0.f;
        Lsum += wgt * ml.y;
        O += wgt * recv[s * share + i];
      }
      const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
      out[((size_t)b * nq + kh * G + r) * 128 + d] = __float2bfloat16_rn(O * inv);
    }
    if (stamp) g_attn_trace[6] = tl_now();
    tl_end(tl);
    return;
  }

  // ---- the last split of this kv head to finish merges all splits (fixed split order) ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(&tickets[bh], 1u);
    s_last = (ticket == (unsigned)(S - 1));
    if (s_last) tickets[bh] = 0;         // ready for the next layer / launch
    __threadfence();
  }
  __syncthreads();
  if (!s_last) { tl_end(tl); return; }
  for (int r = warp; r < G; r += DC + 1) {
    const size_t base = ((size_t)bh * S) * G + r;
    float m = -INFINITY, l = 0.f;
    if (lane < S) {
      m = __ldcg(part_ml + (base + (size_t)lane * G) * 2);
      l = __ldcg(part_ml + (base + (size_t)lane * G) * 2 + 1);
    }
    float Mx = warp_max(m);
    if (Mx == -INFINITY) Mx = 0.f;
    const float wgt = l > 0.f ? exp2f(m - Mx) : 0.f;
    const float Lsum = warp_sum(wgt * l);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s0 = 0; s0 < S; s0 += 16) {
      float4 o[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int s = s0 + j < S ? s0 + j : S - 1;
        o[j] = __ldcg(reinterpret_cast<const float4*>(part_o + (base + (size_t)s * G) * 128) + lane);
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
    *reinterpret_cast<uint2*>(out + ((size_t)b * nq + kh * G + r) * 128 + lane * 4) = packed;
  }
  tl_end(tl);
}

// ---------------------------------------------------------------------------------------------
// Causal attention over a whole prompt (the prompt pass; reference: engine/prefill.py:45-52 calls
// the library's scaled-dot-product attention there). One CTA = one (sequence, kv head, block of
// 128/G prompt tokens): its 128 query rows (token-major, the G query heads of the kv head side
// by side) share every K/V page tile. Warps 0..7 each own 16 query rows and all 64 keys of a
// tile - S = Q K^T, online softmax and P V with mma.m16n8k16, no merge between warps; one lane
// walks the block table and keeps the two-stage ring full. Keys come from the pages the head-norm + RoPE
// kernel has just filled, tiles past the block's last token are never fetched, and the
// diagonal tiles are masked per row. Same cast boundaries as the decode kernels.
constexpr int PF_WARPS = 8;
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_NS = 2;
constexpr size_t PF_SMEM = PF_NS * STAGE_BYTES + 128 * 256 + 2 * PF_NS * 8;

__global__ void __launch_bounds__(PF_THREADS, 2)
k_attn_prefill(const bf16* __restrict__ Q, const char* __restrict__ kpool, const char* __restrict__ vpool,
               const int32_t* __restrict__ block_table, int pages_per_seq,
               const int32_t* __restrict__ pos_ptr, bf16* __restrict__ out, int T, int G, int gshift,
               int nq, int nkv, float scale_log2) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* stages = smem;                                   // PF_NS * STAGE_BYTES
  unsigned char* qtile = smem + PF_NS * STAGE_BYTES;              // 128 rows * 256 B
  uint64_t* bars = reinterpret_cast<uint64_t*>(qtile + 128 * 256);  // full[PF_NS], empty[PF_NS]

  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, kh = blockIdx.y;
  const int QB = 128 >> gshift;                                   // prompt tokens per CTA
  const int q0 = (gridDim.x - 1 - blockIdx.x) * QB;              // latest blocks (most key tiles) first
  if (tid == 0) {
    for (int i = 0; i < PF_NS; ++i) {
      mbar_init(smem_u32(&bars[i]), 1);
      mbar_init(smem_u32(&bars[PF_NS + i]), PF_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();                       // q and this pass's K/V rows come from the kernel before
  const int pos = pos_ptr[0];
  const int tok_end = min(q0 + QB, T);                            // tokens of this block: [q0, tok_end)
  const int max_limit = pos + tok_end;                            // keys visible to the last row
  const int ntiles = (max_limit + Q_PAGE_TOKENS - 1) / Q_PAGE_TOKENS;

  // Lane 0 of warp 0 is also the producer: it asks for the first tiles here and for tile
  // it + PF_NS when every warp has let go of tile it (no ninth warp: 256 threads leave each
  // thread 128 registers with two CTAs on an SM).
  auto fetch_tile = [&](int it) {
    const int s = it % PF_NS;
    const int page = block_table[(size_t)b * pages_per_seq + it];
    const size_t off = ((size_t)page * nkv + kh) * TILE_BYTES;
    const uint32_t bar = smem_u32(&bars[s]);
    mbar_expect_tx(bar, STAGE_BYTES);
    bulk_g2s(smem_u32(stages + s * STAGE_BYTES), kpool + off, TILE_BYTES, bar);
    bulk_g2s(smem_u32(stages + s * STAGE_BYTES + TILE_BYTES), vpool + off, TILE_BYTES, bar);
  };
  if (tid == 0)
    for (int it = 0; it < ntiles && it < PF_NS; ++it) fetch_tile(it);

  // ---------------- consumers ----------------
  // Q block -> shared memory (swizzled rows of 256 B); rows of tokens past the prompt are zero.
  for (int c = tid; c < 128 * 16; c += PF_WARPS * 32) {
    const int r = c >> 4, ch = c & 15;
    const int t = q0 + (r >> gshift), gq = r & (G - 1);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < T) v = *reinterpret_cast<const uint4*>(Q + (((size_t)b * T + t) * nq + kh * G + gq) * 128 + ch * 8);
    *reinterpret_cast<uint4*>(qtile + r * 256 + ((ch ^ (r & 7)) << 4)) = v;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(PF_WARPS * 32) : "memory");

  const int g = lane >> 2, t4 = lane & 3;
  float m_run[2], l_run[2], oacc[16][4];
  int limit[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    m_run[h] = -INFINITY;
    l_run[h] = 0.f;
    const int t = q0 + ((warp * 16 + g + 8 * h) >> gshift);
    limit[h] = t < T ? pos + t + 1 : 0;                           // a row past the prompt sees nothing
  }
#pragma unroll
  for (int n = 0; n < 16; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
  // keys this warp's 16 rows can see: tiles past that are skipped by the warp (still released)
  const int t_last = min(q0 + ((warp * 16 + 15) >> gshift), T - 1);
  const int warp_limit = pos + t_last + 1;
  const uint32_t q_base = smem_u32(qtile);

  for (int it = 0; it < ntiles; ++it) {
    const int s = it % PF_NS;
    if (!mbar_wait(smem_u32(&bars[s]), (it / PF_NS) & 1)) {
      atomicExch(&g_status[0], 6);
      return;
    }
    unsigned char* kt = stages + s * STAGE_BYTES;
    unsigned char* vt = kt + TILE_BYTES;
    const int key_base = it * Q_PAGE_TOKENS;
    if (key_base + Q_PAGE_TOKENS > max_limit) {
      // rows past the newest key may hold stale bits: clear those V rows so that 0 * garbage
      // cannot produce NaN in P V. Every warp clears all of them itself (the same zeros from
      // eight warps), so no barrier is needed before it reads the tile.
      for (int c = lane; c < 64 * 16; c += 32) {
        const int kr = c >> 4;
        if (key_base + kr >= max_limit)
          *reinterpret_cast<uint4*>(vt + kr * 256 + ((c & 15) << 4)) = make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
    }
    if (key_base < warp_limit) {
      const uint32_t k_base = smem_u32(kt), v_base = smem_u32(vt);
      float sacc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        // Q fragment of this k-step (re-read per tile: keeping all eight in registers costs
        // the second CTA per SM)
        uint32_t qa[8][4];
        {
          const int row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
          const int ch = 2 * ks + (lane >> 4);
          ldsm_x4(q_base + row * 256 + ((ch ^ (row & 7)) << 4), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
        }
#pragma unroll
        for (int kb = 0; kb < 4; ++kb) {                          // 16 keys per ldmatrix
          uint32_t b0, b1, b2, b3;
          const int mi = lane >> 3;
          const int key = kb * 16 + 8 * (mi >> 1) + (lane & 7);
          const int ch = 2 * ks + (mi & 1);
          ldsm_x4(k_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
          mma16816(sacc[2 * kb], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
          mma16816(sacc[2 * kb + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
        }
      }
      // online softmax for rows g (h=0) and g+8 (h=1) over the tile's 64 keys
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key_base + 8 * j + 2 * t4 + e;
            float v = sacc[j][2 * h + e] * scale_log2;
            v = key < limit[h] ? v : -INFINITY;
            sacc[j][2 * h + e] = v;
            mx = fmaxf(mx, v);
          }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[h], mx);
        const float m_safe = m_new == -INFINITY ? 0.f : m_new;
        const float resc = exp2f(m_run[h] - m_safe);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float pv = exp2f(sacc[j][2 * h + e] - m_safe);
            sacc[j][2 * h + e] = pv;
            sum += pv;
          }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_run[h] = l_run[h] * resc + sum;
        m_run[h] = m_new;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          oacc[n][2 * h] *= resc;
          oacc[n][2 * h + 1] *= resc;
        }
      }
#pragma unroll
      for (int kb = 0; kb < 4; ++kb) {                            // P V, 16 keys per step
        const uint32_t pa0 = pack_bf16(sacc[2 * kb][0], sacc[2 * kb][1]);
        const uint32_t pa1 = pack_bf16(sacc[2 * kb][2], sacc[2 * kb][3]);
        const uint32_t pa2 = pack_bf16(sacc[2 * kb + 1][0], sacc[2 * kb + 1][1]);
        const uint32_t pa3 = pack_bf16(sacc[2 * kb + 1][2], sacc[2 * kb + 1][3]);
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          uint32_t b0, b1, b2, b3;
          const int mi = lane >> 3;
          const int key = kb * 16 + 8 * (mi & 1) + (lane & 7);
          const int ch = 2 * dp + (mi >> 1);
          ldsm_x4_t(v_base + key * 256 + ((ch ^ (key & 7)) << 4), b0, b1, b2, b3);
          mma16816(oacc[2 * dp], pa0, pa1, pa2, pa3, b0, b1);
          mma16816(oacc[2 * dp + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bars[PF_NS + s]));
    if (tid == 0 && it + PF_NS < ntiles) {
      // a wait that runs out leaves the tile unrequested: the consumers' own bounded wait
      // for it then ends the CTA
      if (mbar_wait(smem_u32(&bars[PF_NS + s]), (it / PF_NS) & 1)) fetch_tile(it + PF_NS);
      else atomicExch(&g_status[0], 5);
    }
    __syncwarp();
  }

  // one rounding to bf16; the row's 128 dims go to out[(b*T + t)][head][128]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    const int t = q0 + (r >> gshift);
    if (t >= T) continue;
    const float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
    bf16* dst = out + (((size_t)b * T + t) * nq + kh * G + (r & (G - 1))) * 128;
#pragma unroll
    for (int n = 0; n < 16; ++n)
      *reinterpret_cast<uint32_t*>(dst + 8 * n + 2 * t4) = pack_bf16(oacc[n][2 * h] * inv, oacc[n][2 * h + 1] * inv);
  }
}

constexpr size_t attn_decode_smem(int ns) { return ns * STAGE_BYTES + 16 * 256 + 2 * ns * 8 + 2 * 128 * 2 + 64 + (8 * 128 + 16 + MAX_CLUSTER * 8 * 2) * 4; }

template <int RT>
constexpr size_t attn_smem() { return NS * STAGE_BYTES + RT * 16 * 256 + 2 * NS * 8; }

}  // namespace

extern "C" int q_attention_splits(int batch, int n_kv_heads, int capacity) {
  if (batch < 1 || n_kv_heads < 1 || capacity < 1) return 1;
  int sms = q_sm_count();
  if (sms <= 0) sms = 148;
  const int vh = batch * n_kv_heads;
  const int tiles = (capacity + Q_PAGE_TOKENS - 1) / Q_PAGE_TOKENS;
  // Two CTAs fit on an SM. All CTAs of a launch should be resident at once: a second wave
  // cannot request its K/V tiles before a slot frees, and measured ~15 % at 32 sequences of
  // 2 K keys (two splits per kv head = 1.7 waves) against one split per kv head in one wave.
  int desired = (2 * sms) / vh;
  if (desired < 1) desired = 1;
  int s = desired < tiles ? desired : tiles;
  // Up to 8 splits merge inside a thread-block cluster (no global round trip); that is
  // worth more than finer splits while a split still sees at most 4 tiles. (Clusters of up to
  // 16 are supported by the kernel; 12 splits of at most two tiles each, whose 70 KB CTAs fit
  // on an SM beside a projection CTA, measured slower at batch 1 / 1 K keys: 10.0 against
  // 9.1 us per layer - the scheduler packs two such CTAs onto one SM and the O projection
  // still starts late there.)
  if (s > 8 && tiles <= 32) s = 8;
  if (s > 32) s = 32;
  if (s < 1) s = 1;
  return s;
}

extern "C" int q_attention(const void* d_q, const q_kv_layout_t* kv, const int32_t* d_pos,
                           float* d_scratch_o, float* d_scratch_ml, void* d_out, int batch, int T,
                           int n_q_heads, int splits, float scale, void* stream) {
  Q_CHECK_ARG(d_q && kv && d_pos && d_out, "q_attention: null pointer");
  Q_CHECK_ARG(kv->d_kpool && kv->d_vpool && kv->d_block_table && kv->pages_per_seq >= 1 &&
                  kv->n_kv_heads >= 1,
              "q_attention: incomplete KV layout");
  const int nkv = kv->n_kv_heads;
  Q_CHECK_ARG(batch >= 1 && T >= 1 && n_q_heads >= nkv && n_q_heads % nkv == 0,
              "q_attention: bad batch/T/heads");
  const int G = n_q_heads / nkv;
  Q_CHECK_ARG(T * G <= 32, "q_attention: T*G = %d exceeds 32 query rows per kv head", T * G);
  Q_CHECK_ARG(splits >= 1 && splits <= 32, "q_attention: splits %d outside 1..32", splits);
  Q_CHECK_ARG(splits == 1 || (d_scratch_o && d_scratch_ml), "q_attention: split scratch missing");
  Q_CHECK_ARG((long long)batch * nkv <= 65535, "q_attention: too many (sequence, kv head) pairs");
  Q_CHECK_ARG(((uintptr_t)kv->d_kpool & 15) == 0 && ((uintptr_t)kv->d_vpool & 15) == 0 &&
                  ((uintptr_t)d_q & 15) == 0,
              "q_attention: pools and q must be 16-byte aligned");
  Q_CHECK_ALIGN(d_scratch_o, 16, "q_attention"); Q_CHECK_ALIGN(d_scratch_ml, 8, "q_attention");
  Q_CHECK_ALIGN(d_out, 8, "q_attention");
  cudaStream_t s = (cudaStream_t)stream;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(splits, batch * nkv), block(THREADS);
  cudaError_t e;
  static size_t done1[64] = {0}, done2[64] = {0};
  if (T * G <= 16) {
    Q_CHECK_CUDA(q_ensure_smem(k_attn_split<1>, attn_smem<1>(), done1));
    e = q_launch(k_attn_split<1>, grid, block, attn_smem<1>(), s, (const bf16*)d_q,
                 (const char*)kv->d_kpool, (const char*)kv->d_vpool, kv->d_block_table,
                 kv->pages_per_seq, d_pos, d_scratch_o, d_scratch_ml, (bf16*)d_out, T, G, n_q_heads,
                 nkv, splits, scale_log2);
  } else {
    Q_CHECK_CUDA(q_ensure_smem(k_attn_split<2>, attn_smem<2>(), done2));
    e = q_launch(k_attn_split<2>, grid, block, attn_smem<2>(), s, (const bf16*)d_q,
                 (const char*)kv->d_kpool, (const char*)kv->d_vpool, kv->d_block_table,
                 kv->pages_per_seq, d_pos, d_scratch_o, d_scratch_ml, (bf16*)d_out, T, G, n_q_heads,
                 nkv, splits, scale_log2);
  }
  Q_CHECK_CUDA(e);
  if (splits > 1) {
    const int items = batch * T * n_q_heads;
    Q_CHECK_CUDA(q_launch(k_attn_merge, dim3((items + 3) / 4), dim3(128), 0, s, d_scratch_o,
                          d_scratch_ml, (bf16*)d_out, batch, T, G, n_q_heads, nkv, splits));
  }
  return Q_OK;
}

extern "C" int q_attention_prefill(const void* d_q, const q_kv_layout_t* kv, const int32_t* d_pos,
                                   void* d_out, int batch, int T, int n_q_heads, float scale,
                                   void* stream) {
  Q_CHECK_ARG(d_q && kv && d_pos && d_out, "q_attention_prefill: null pointer");
  Q_CHECK_ARG(kv->d_kpool && kv->d_vpool && kv->d_block_table && kv->pages_per_seq >= 1 &&
                  kv->n_kv_heads >= 1,
              "q_attention_prefill: incomplete KV layout");
  const int nkv = kv->n_kv_heads;
  Q_CHECK_ARG(batch >= 1 && batch <= 65535 && nkv <= 65535 && T >= 1 && n_q_heads >= nkv &&
                  n_q_heads % nkv == 0,
              "q_attention_prefill: bad batch/T/heads");
  const int G = n_q_heads / nkv;
  Q_CHECK_ARG(G <= 8 && (G & (G - 1)) == 0,
              "q_attention_prefill: %d query heads per kv head (1, 2, 4 or 8 supported)", G);
  Q_CHECK_ALIGN(d_q, 16, "q_attention_prefill"); Q_CHECK_ALIGN(d_out, 4, "q_attention_prefill");
  Q_CHECK_ALIGN(kv->d_kpool, 16, "q_attention_prefill"); Q_CHECK_ALIGN(kv->d_vpool, 16, "q_attention_prefill");
  int gshift = 0;
  while ((1 << gshift) < G) ++gshift;
  const int QB = 128 >> gshift;
  static size_t done[64] = {0};
  Q_CHECK_CUDA(q_ensure_smem(k_attn_prefill, PF_SMEM, done));
  Q_CHECK_CUDA(q_launch(k_attn_prefill, dim3((T + QB - 1) / QB, nkv, batch), dim3(PF_THREADS), PF_SMEM,
                        (cudaStream_t)stream, (const bf16*)d_q, (const char*)kv->d_kpool,
                        (const char*)kv->d_vpool, kv->d_block_table, kv->pages_per_seq, d_pos,
                        (bf16*)d_out, T, G, gshift, n_q_heads, nkv, scale * 1.4426950408889634f));
  return Q_OK;
}

extern "C" int q_attention_decode(const float* d_qkv_partials, const q_gemm_plan_t* plan,
                                  const void* d_q_gain, const void* d_k_gain, const void* d_cos,
                                  const void* d_sin, const int32_t* d_pos, const q_kv_layout_t* kv,
                                  float* d_scratch_o, float* d_scratch_ml, uint32_t* d_tickets,
                                  void* d_out, int batch, int n_q_heads, int splits, float scale,
                                  float eps, void* stream) {
  Q_CHECK_ARG(d_qkv_partials && d_q_gain && d_k_gain && d_cos && d_sin && d_pos && kv && d_out,
              "q_attention_decode: null pointer");
  Q_CHECK_ARG(kv->d_kpool && kv->d_vpool && kv->d_block_table && kv->pages_per_seq >= 1 &&
                  kv->n_kv_heads >= 1,
              "q_attention_decode: incomplete KV layout");
  const int nkv = kv->n_kv_heads;
  Q_CHECK_ARG(batch >= 1 && batch <= Q_MAX_ROWS && n_q_heads >= nkv && n_q_heads % nkv == 0,
              "q_attention_decode: bad batch/heads");
  const int G = n_q_heads / nkv;
  Q_CHECK_ARG(G <= 8, "q_attention_decode: %d query heads per kv head exceed 8", G);
  Q_CHECK_ARG(splits >= 1 && splits <= 32, "q_attention_decode: splits %d outside 1..32", splits);
  Q_CHECK_ARG((long long)batch * nkv <= 65535, "q_attention_decode: too many (sequence, kv head) pairs");
  if (plan) {
    Q_CHECK_ARG(plan->M == batch && plan->N == (n_q_heads + 2 * nkv) * 128,
                "q_attention_decode: plan does not match the packed projection");
  }
  Q_CHECK_ALIGN(d_qkv_partials, 16, "q_attention_decode"); Q_CHECK_ALIGN(d_q_gain, 8, "q_attention_decode");
  Q_CHECK_ALIGN(d_k_gain, 8, "q_attention_decode"); Q_CHECK_ALIGN(d_cos, 8, "q_attention_decode");
  Q_CHECK_ALIGN(d_sin, 8, "q_attention_decode"); Q_CHECK_ALIGN(kv->d_kpool, 16, "q_attention_decode");
  Q_CHECK_ALIGN(kv->d_vpool, 16, "q_attention_decode"); Q_CHECK_ALIGN(d_scratch_o, 16, "q_attention_decode");
  Q_CHECK_ALIGN(d_scratch_ml, 8, "q_attention_decode"); Q_CHECK_ALIGN(d_out, 8, "q_attention_decode");
  // most tiles one split can be handed: ceil(tiles / splits) over the page capacity
  int ring = (kv->pages_per_seq + splits - 1) / splits;
  ring = ring < 1 ? 1 : (ring > NS ? NS : ring);
  // Three warp groups (one tile each at a time) when every CTA of the launch gets an SM of its
  // own; otherwise one group, so that two CTAs still fit on an SM. A ring stage must always be
  // consumed by the same group (its mbarrier parity is tracked per group), so the three groups
  // need the three-stage ring.
  int sms = q_sm_count();
  if (sms <= 0) sms = 148;
  const bool wide = splits > 1 && (long long)splits * batch * nkv <= sms && ring == 3 && NS == 3;
  const int dc = wide ? 12 : 4;
  const dim3 block((dc + 1) * 32);
  static size_t done[4][64] = {{0}};
  Q_CHECK_CUDA(q_ensure_smem(k_attn_decode<false, 1>, attn_decode_smem(NS), done[0]));
  Q_CHECK_CUDA(q_ensure_smem(k_attn_decode<true, 1>, attn_decode_smem(NS), done[1]));
  Q_CHECK_CUDA(q_ensure_smem(k_attn_decode<false, 3>, attn_decode_smem(NS), done[2]));
  Q_CHECK_CUDA(q_ensure_smem(k_attn_decode<true, 3>, attn_decode_smem(NS), done[3]));
  // the merge scratch (consumer states, then the CTA's own rows) reuses the ring
  const int scratch_stages = (G * (dc + 1) * 130 * 4 + STAGE_BYTES - 1) / STAGE_BYTES;
  if (ring < scratch_stages) ring = scratch_stages;
  Q_CHECK_ARG(ring <= NS, "q_attention_decode: merge scratch does not fit the ring");
  bool cluster = splits >= 2 && splits <= MAX_CLUSTER && !g_attn_no_cluster;
  if (cluster && splits > 8) {
    // more than 8 CTAs per cluster is an opt-in size; whether such clusters can be placed
    // at all is asked once per device and split count
    static int placeable[64][MAX_CLUSTER + 1];          // 0 unknown, 1 yes, -1 no
    const int dev = q_device_index();
    if (dev < 0) cluster = false;
    else {
      if (placeable[dev][splits] == 0) {
        int n = 0;
        cudaError_t e1 = cudaFuncSetAttribute(k_attn_decode<true, 1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e1 == cudaSuccess)
          e1 = cudaFuncSetAttribute(k_attn_decode<true, 3>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(splits, batch * nkv);
        cfg.blockDim = dim3(13 * 32);
        cfg.dynamicSmemBytes = attn_decode_smem(NS);
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaError_t e2 = e1 == cudaSuccess ? cudaOccupancyMaxActiveClusters(&n, k_attn_decode<true, 3>, &cfg) : e1;
        if (e2 != cudaSuccess) cudaGetLastError();
        placeable[dev][splits] = (e2 == cudaSuccess && n >= 1) ? 1 : -1;
      }
      cluster = placeable[dev][splits] == 1;
    }
  }
  Q_CHECK_ARG(cluster || splits == 1 || (d_scratch_o && d_scratch_ml && d_tickets),
              "q_attention_decode: split scratch or tickets missing (needed when the splits cannot merge in a cluster)");
  const float sl2 = scale * 1.4426950408889634f;
#define Q_ATTN_DECODE_ARGS                                                                              \
  d_qkv_partials, plan_view(plan), (const bf16*)d_q_gain, (const bf16*)d_k_gain, (const bf16*)d_cos,   \
      (const bf16*)d_sin, d_pos, (char*)kv->d_kpool, (char*)kv->d_vpool, kv->d_block_table,             \
      kv->pages_per_seq, d_scratch_o, d_scratch_ml, d_tickets, (bf16*)d_out, batch, G, n_q_heads, nkv,  \
      splits, sl2, eps, ring, q_tl_next(Q_TL_ATTENTION)
  const dim3 grid(splits, batch * nkv);
  const size_t smem = attn_decode_smem(ring);
  cudaStream_t st = (cudaStream_t)stream;
  if (cluster) {
    if (wide) Q_CHECK_CUDA(q_launch_cluster(k_attn_decode<true, 3>, grid, block, smem, st, (unsigned)splits, Q_ATTN_DECODE_ARGS));
    else Q_CHECK_CUDA(q_launch_cluster(k_attn_decode<true, 1>, grid, block, smem, st, (unsigned)splits, Q_ATTN_DECODE_ARGS));
  } else {
    if (wide) Q_CHECK_CUDA(q_launch(k_attn_decode<false, 3>, grid, block, smem, st, Q_ATTN_DECODE_ARGS));
    else Q_CHECK_CUDA(q_launch(k_attn_decode<false, 1>, grid, block, smem, st, Q_ATTN_DECODE_ARGS));
  }
#undef Q_ATTN_DECODE_ARGS
  return Q_OK;
}

extern "C" int q_debug_attn_trace(unsigned long long* out) {
  Q_CHECK_ARG(out != nullptr, "q_debug_attn_trace: null pointer");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_attn_trace, sizeof(unsigned long long) * 8));
  return Q_OK;
}

Q_DEFINE_STATUS_ADDR(q_attn_status_addr, g_status)
