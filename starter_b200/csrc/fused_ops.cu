// Element-wise consumers of the split-K partials. Each one reproduces the bf16
// rounding points of the native model exactly; fp32 reductions are free to
// reorder.
//   1. a Linear output rounds once fp32->bf16 after all partials are summed
//   2. residual add: bf16(x + y) of two bf16 values
//   3. RMSNorm: fp32 x*rsqrt(mean(x^2)+eps) -> bf16 -> times bf16 gain -> bf16
//   4. per-head q/k norm: as 3 over 128 values; V untouched
//   5. RoPE: bf16(bf16(n*cos) + bf16(rot*sin)), partner = (col+64) mod 128
//   6. SwiGLU: bf16(bf16(silu(bf16 g)) * bf16 u)
//   8. argmax over bf16 logits, lowest index on ties
// (reference: engine/kernels/decode_fused.py:19-118, engine/kernels/rmsnorm.py:12-36)
#include "common.cuh"

extern int g_peer_wait_iters;   // q_set_option "peer_wait_iters"

namespace {

// Greedy pick: larger value wins, equal values go to the lower index.
__device__ __forceinline__ void arg_better(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

// ---- RMSNorm (plain) -------------------------------------------------------
__global__ void __launch_bounds__(256)
k_rmsnorm(const bf16* __restrict__ X, const bf16* __restrict__ G, bf16* __restrict__ O,
          int cols, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  const bf16* x = X + row * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = __bfloat162float(x[c]);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)cols + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = bf16_round(__bfloat162float(x[c]) * inv);
    O[row * cols + c] = __float2bfloat16_rn(v * __bfloat162float(G[c]));
  }
}

// ---- embedding gather + RMSNorm --------------------------------------------
// The table is the (tied) lm_head weight in the tiled GEMM layout: element
// (row, c) lives in unit (row/16, c/32), half (row%16)/8, piece (row%8)*4 + (c%32)/8.
__device__ __forceinline__ size_t tiled_offset(long long row, int c, int C) {
  const long long unit = (row >> 4) * C + (c >> 5);
  const int piece = (int)(row & 7) * 4 + ((c & 31) >> 3);
  return (size_t)unit * 512 + (size_t)((row >> 3) & 1) * 256 + piece * 8 + (c & 7);   // in elements
}

__global__ void __launch_bounds__(256)
k_embed_rmsnorm(const int64_t* __restrict__ tokens, const bf16* __restrict__ E,
                const bf16* __restrict__ G, bf16* __restrict__ Xo, bf16* __restrict__ No,
                int cols, int vocab, float eps, unsigned long long* tl) {
  __shared__ float red[32];
  tl_begin(tl);
  pdl_launch_dependents();
  pdl_wait();
  tl_waited(tl);
  const size_t row = blockIdx.x;
  long long tok = tokens[row];
  if (tok < 0) tok = 0;
  if (tok >= vocab) tok = vocab - 1;
  const int C = cols >> 5;
  // 8 consecutive columns are one 16-byte piece of the tiled table
  float ss = 0.f;
  for (int c8 = threadIdx.x; c8 < (cols >> 3); c8 += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(E + tiled_offset(tok, c8 * 8, C));
    *reinterpret_cast<uint4*>(Xo + row * cols + c8 * 8) = raw;
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = bf_lo(w[e]), hi = bf_hi(w[e]);
      ss += lo * lo + hi * hi;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)cols + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = bf16_round(__bfloat162float(Xo[row * cols + c]) * inv);
    No[row * cols + c] = __float2bfloat16_rn(v * __bfloat162float(G[c]));
  }
  tl_end(tl);
}

// ---- residual add + RMSNorm on partials ------------------------------------
// One CTA per row. Thread t owns columns 4t..4t+3 (+1024 j): both partial slots come in
// with 16-byte loads that are all issued before anything is used (a row is a few KB in
// L2, so the kernel is one memory round trip + one block reduction).
constexpr int ADD_VB = 10;     // 256 threads * 4 columns * 10 = 10240 columns

__device__ __forceinline__ int plan_extra(const PlanView& pv, int n, int row) {   // slots beyond the first
  return plan_count(pv, n, row) - 1;
}

// THREADS = 256, or 1024 for rows of up to 4096 columns (VB = 1): a row is then spread over
// four times the threads, each with a third of the loads in flight.
template <int VB, int THREADS = 256>
__global__ void __launch_bounds__(THREADS)
k_add_rmsnorm(const bf16* __restrict__ Xin, const float* __restrict__ P, PlanView pv,
              const bf16* __restrict__ G, bf16* __restrict__ Tout, bf16* __restrict__ Nout,
              int cols, float eps, unsigned long long* tl) {
  __shared__ float red[32];
  tl_begin(tl);
  pdl_launch_dependents();
  pdl_wait();
  tl_waited(tl);
  const size_t row = blockIdx.x;
  const float* p0 = P + row * cols;
  const bool two = pv.u != 0;
  float4 s0[VB], s1[VB];
  uint2 xr[VB], gn[VB];
#pragma unroll
  for (int j = 0; j < VB; ++j) {
    const int col = 4 * threadIdx.x + j * 1024;
    const int cc = col < cols ? col : 0;
    s0[j] = *reinterpret_cast<const float4*>(p0 + cc);
    s1[j] = two ? *reinterpret_cast<const float4*>(p0 + cc + pv.slot_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
    xr[j] = *reinterpret_cast<const uint2*>(Xin + row * cols + cc);
    gn[j] = *reinterpret_cast<const uint2*>(G + cc);
  }
  // A projection whose output is narrow and whose K is long (O, down on the tcgen05 path) is
  // split up to ~10 ways: slots 2..9 are requested together as well (narrow rows only, the
  // registers of a wide row would not hold them); anything beyond comes one at a time.
  constexpr int EX = VB <= 3 ? 8 : 0;
  float4 sx[VB][EX > 0 ? EX : 1];
  if (EX > 0 && two) {
#pragma unroll
    for (int j = 0; j < VB; ++j) {
      const int col = 4 * threadIdx.x + j * 1024;
      const int cc = col < cols ? col : 0;
      const int extra = plan_extra(pv, cc, (int)row);
#pragma unroll
      for (int k = 0; k < EX; ++k)
        sx[j][k] = (k + 2 <= extra) ? *reinterpret_cast<const float4*>(p0 + cc + (long long)(k + 2) * pv.slot_stride)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  float tot[VB][4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VB; ++j) {
    const int col = 4 * threadIdx.x + j * 1024;
    if (col < cols) {
      const int extra = plan_extra(pv, col, (int)row);        // the 4 columns share one group
      float s[4] = {s0[j].x, s0[j].y, s0[j].z, s0[j].w};
      if (extra > 0) { s[0] += s1[j].x; s[1] += s1[j].y; s[2] += s1[j].z; s[3] += s1[j].w; }
      if (EX > 0 && two) {
#pragma unroll
        for (int k = 0; k < EX; ++k)
          if (k + 2 <= extra) { s[0] += sx[j][k].x; s[1] += sx[j][k].y; s[2] += sx[j][k].z; s[3] += sx[j][k].w; }
      }
      for (int k = 2 + EX; k <= extra; ++k) {
        const float4 sk = *reinterpret_cast<const float4*>(p0 + col + (long long)k * pv.slot_stride);
        s[0] += sk.x; s[1] += sk.y; s[2] += sk.z; s[3] += sk.w;
      }
      const float r[4] = {bf_lo(xr[j].x), bf_hi(xr[j].x), bf_lo(xr[j].y), bf_hi(xr[j].y)};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        tot[j][e] = bf16_round(r[e] + bf16_round(s[e]));
        ss += tot[j][e] * tot[j][e];
      }
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)cols + eps);
#pragma unroll
  for (int j = 0; j < VB; ++j) {
    const int col = 4 * threadIdx.x + j * 1024;
    if (col < cols) {
      const float g4[4] = {bf_lo(gn[j].x), bf_hi(gn[j].x), bf_lo(gn[j].y), bf_hi(gn[j].y)};
      uint2 to, no;
      to.x = pack_bf16(tot[j][0], tot[j][1]);
      to.y = pack_bf16(tot[j][2], tot[j][3]);
      no.x = pack_bf16(bf16_round(tot[j][0] * inv) * g4[0], bf16_round(tot[j][1] * inv) * g4[1]);
      no.y = pack_bf16(bf16_round(tot[j][2] * inv) * g4[2], bf16_round(tot[j][3] * inv) * g4[3]);
      *reinterpret_cast<uint2*>(Tout + row * cols + col) = to;
      *reinterpret_cast<uint2*>(Nout + row * cols + col) = no;
    }
  }
  tl_end(tl);
}


// ---- residual add + RMSNorm on the partials of ALL tensor-parallel ranks ----------------
// One CTA per row, one thread per four columns. The exchange carries its own arrival
// signal: every fp32 sum travels as an 8-byte pair {value, call counter}, stored with one
// 8-byte store (single-copy atomic), so there is no fence, no flag and no second trip:
//   1. the CTA adds this rank's split-K slots of its row (fp32, slot order) and stores the
//      pairs into EVERY peer's receive area through the peer mappings (posted writes);
//   2. it polls (bounded) its OWN receive area until the pairs of its row carry this call's
//      counter for every peer, adds all ranks' sums in rank order, rounds once, adds the
//      residual and normalises.
// The receive area has two halves used by alternate calls, so a rank may already push the
// next call's pairs while a slower peer still reads this call's; a half is written again two
// calls later, which a rank reaches only after every peer's pairs of the call between have
// arrived, i.e. after every peer finished this call. A stale pair can never look fresh: it
// carries an older counter. The call counter is bumped by the last CTA to finish (a
// ticket), so every CTA of a call reads the same value. All ranks make the same calls.
__device__ int g_peer_status;      // 1 = a wait for a peer ran out

// Bounded wait for `word` to reach `e` (wrap-around safe). The limit is in polling
// iterations; the back-off grows to 2 us per poll, so the default 2^21 is about 4 s: a peer
// whose host thread was descheduled for a moment must not look like a dead one.
__device__ __forceinline__ bool wait_arrival(const uint32_t* word, unsigned e, int limit) {
  for (int i = 0; i < limit; ++i) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
    if ((int)(v - e) >= 0) return true;
    if (i > 64) __nanosleep(i > 65536 ? 2000 : (i > 4096 ? 400 : 40));
  }
  return false;
}

constexpr int PEER_MAX_COLS = 4096;     // one thread per four columns, at most 1024 threads

__global__ void __launch_bounds__(1024)
k_add_rmsnorm_peers(const bf16* __restrict__ Xin, PeerView pw, const float* __restrict__ P, PlanView pv,
                    const bf16* __restrict__ G, bf16* __restrict__ Tout, bf16* __restrict__ Nout,
                    int rows, int cols, float eps, int wait_iters, unsigned long long* tl) {
  __shared__ float red[32];
  __shared__ unsigned s_epoch;
  tl_begin(tl);
  pdl_launch_dependents();
  pdl_wait();                         // this rank's projection has written its partials
  tl_waited(tl);
  const int tid = threadIdx.x, lane = tid & 31;
  const int row = blockIdx.x;
  // A warp covers 128 columns; lane l owns columns {2l, 2l+1} and {64+2l, 64+2l+1} of them, so
  // that each of its two 16-byte pair stores lines up with the other lanes' into 512
  // contiguous bytes (stores of 16 bytes scattered at a 32-byte stride crossed NVLink as
  // one small packet each and made the exchange packet-bound at 32 rows).
  const int cw = (tid >> 5) * 128 + 2 * lane;
  const int colv[2] = {cw, cw + 64};
  const bool live[2] = {colv[0] < cols, colv[1] < cols};
  if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned*>(pw.epoch) + 1u;
  // operands that do not depend on the peers: own slots, residual, gain
  const float2 z2 = make_float2(0.f, 0.f);
  float2 own[2];
  uint32_t xr[2], gn[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int c = live[h] ? colv[h] : 0;
    const float* p0 = P + (size_t)row * cols + c;
    const int extra = live[h] ? plan_count(pv, c) - 1 : -1;
    float2 sl[10];
#pragma unroll
    for (int k = 0; k < 10; ++k)
      sl[k] = (k <= extra && (k == 0 || pv.u != 0)) ? *reinterpret_cast<const float2*>(p0 + (long long)k * pv.slot_stride) : z2;
    xr[h] = live[h] ? *reinterpret_cast<const uint32_t*>(Xin + (size_t)row * cols + c) : 0u;
    gn[h] = live[h] ? *reinterpret_cast<const uint32_t*>(G + c) : 0u;
    float2 acc = sl[0];
#pragma unroll
    for (int k = 1; k < 10; ++k)
      if (k <= extra) { acc.x += sl[k].x; acc.y += sl[k].y; }
    for (int k = 10; k <= extra; ++k) {
      const float2 t = *reinterpret_cast<const float2*>(p0 + (long long)k * pv.slot_stride);
      acc.x += t.x; acc.y += t.y;
    }
    own[h] = acc;
  }
  __syncthreads();
  const unsigned e = s_epoch;
  // element offsets in 8-byte pairs: halves alternate with the call counter
  const size_t half_off = (size_t)(e & 1u) * pw.world * rows * cols;
  const size_t row_off = half_off + ((size_t)pw.rank * rows + row) * cols;
  // 1. push this rank's pairs to every peer
#pragma unroll
  for (int r = 0; r < Q_MAX_PEERS; ++r)
    if (r < pw.world && r != pw.rank) {
      char* dst = reinterpret_cast<char*>(pw.recv[r]);
      if (live[0]) st_pair2(dst + (row_off + colv[0]) * 8, own[0].x, own[0].y, e);
      if (live[1]) st_pair2(dst + (row_off + colv[1]) * 8, own[1].x, own[1].y, e);
    }
  // 2. collect the peers' pairs of this row from the own receive area, in rank order
  float tot[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  float ss = 0.f;
  {
    float2 acc[2] = {z2, z2};
    bool ok = true;
    // Four peers at a time: their loads are in flight together (one round trip per poll, not
    // one per peer), and the sums are still added in rank order.
    for (int r0 = 0; r0 < pw.world; r0 += 4) {
      unsigned long long a[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) a[j][0] = a[j][1] = a[j][2] = a[j][3] = 0;
      bool here = false;
      for (int i = 0; ok && i < wait_iters; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = r0 + j;
          if (r < pw.world && r != pw.rank) {
            const char* src = reinterpret_cast<const char*>(pw.recv[pw.rank]) + (half_off + ((size_t)r * rows + row) * cols) * 8;
            if (live[0]) ld_pair2(src + (size_t)colv[0] * 8, a[j][0], a[j][1]);
            if (live[1]) ld_pair2(src + (size_t)colv[1] * 8, a[j][2], a[j][3]);
          }
        }
        here = true;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = r0 + j;
          if (r < pw.world && r != pw.rank)
            here = here && (!live[0] || ((unsigned)(a[j][0] >> 32) == e && (unsigned)(a[j][1] >> 32) == e)) &&
                   (!live[1] || ((unsigned)(a[j][2] >> 32) == e && (unsigned)(a[j][3] >> 32) == e));
        }
        if (here) break;
        if (i > 64) __nanosleep(i > 65536 ? 2000 : (i > 4096 ? 400 : 40));
      }
      if (!here) { ok = false; atomicExch(&g_peer_status, 1); }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = r0 + j;
        if (r >= pw.world) break;
        float2 t[2] = {own[0], own[1]};
        if (r != pw.rank) {
          t[0] = make_float2(__uint_as_float((unsigned)a[j][0]), __uint_as_float((unsigned)a[j][1]));
          t[1] = make_float2(__uint_as_float((unsigned)a[j][2]), __uint_as_float((unsigned)a[j][3]));
        }
        acc[0].x += t[0].x; acc[0].y += t[0].y; acc[1].x += t[1].x; acc[1].y += t[1].y;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
      if (live[h]) {
        tot[h][0] = bf16_round(bf_lo(xr[h]) + bf16_round(acc[h].x));
        tot[h][1] = bf16_round(bf_hi(xr[h]) + bf16_round(acc[h].y));
        ss += tot[h][0] * tot[h][0] + tot[h][1] * tot[h][1];
      }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)cols + eps);
#pragma unroll
  for (int h = 0; h < 2; ++h)
    if (live[h]) {
      const uint32_t to = pack_bf16(tot[h][0], tot[h][1]);
      const uint32_t no = pack_bf16(bf16_round(tot[h][0] * inv) * bf_lo(gn[h]), bf16_round(tot[h][1] * inv) * bf_hi(gn[h]));
      *reinterpret_cast<uint32_t*>(Tout + (size_t)row * cols + colv[h]) = to;
      *reinterpret_cast<uint32_t*>(Nout + (size_t)row * cols + colv[h]) = no;
    }
  // the last CTA of the call publishes the new call counter
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned ticket = atomicAdd(pw.epoch + 1, 1u);
    if (ticket == gridDim.x - 1) {
      pw.epoch[1] = 0;
      *reinterpret_cast<volatile unsigned*>(pw.epoch) = e;
      __threadfence();
    }
  }
  tl_end(tl);
}

// ---- final token pick over the vocabulary shards, exchanged through peer memory ----------
// Every rank stores its per-row (max logit, index) pair into every rank's exchange area
// (plain peer stores), tells the peers with an arrival word and waits (bounded) for theirs;
// then each rank picks, per row, the largest value with the lowest index over the shards in
// its own area, writes the token and bumps the position. The area is double-buffered by the
// parity of the call counter, so a rank may run one call ahead of a peer that is still
// reading. Exchange area of rank r (inside its flag region, see q_peer_flag_bytes):
// arrival words at uint32 [64 + p], pairs at byte 512: [parity][shard][row] {float, int32}.
__global__ void __launch_bounds__(64)
k_argmax_merge_peers(const float* __restrict__ val, const int32_t* __restrict__ idx, PeerView pw, int rows,
                     int64_t* __restrict__ tokens, int32_t* __restrict__ pos_ptr, int pos_inc, int wait_iters,
                     StatusTap tap) {
  pdl_wait();
  const int tid = threadIdx.x;
  const unsigned e = *reinterpret_cast<volatile unsigned*>(pw.epoch + 2) + 1u;
  const int parity = (int)(e & 1u);
  if (tid < rows) {
    const float v = val[tid];
    const int i = idx[tid];
    for (int p = 0; p < pw.world; ++p) {
      char* area = reinterpret_cast<char*>(pw.flags[p]) + 512;
      float2* slot = reinterpret_cast<float2*>(area) + ((size_t)parity * pw.world + pw.rank) * Q_MAX_ROWS + tid;
      asm volatile("st.volatile.global.v2.f32 [%0], {%1, %2};" ::"l"(slot), "f"(v), "f"(__int_as_float(i)) : "memory");
    }
    __threadfence_system();
  }
  __syncthreads();
  if (tid < pw.world && tid != pw.rank) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pw.flags[tid] + 64 + pw.rank), "r"(e) : "memory");
    if (!wait_arrival(pw.flags[pw.rank] + 64 + tid, e, wait_iters)) atomicExch(&g_peer_status, 1);
  }
  __syncthreads();
  if (tid < rows) {
    const char* area = reinterpret_cast<const char*>(pw.flags[pw.rank]) + 512;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int s = 0; s < pw.world; ++s) {
      const float2* slot = reinterpret_cast<const float2*>(area) + ((size_t)parity * pw.world + s) * Q_MAX_ROWS + tid;
      float a, b;
      asm volatile("ld.volatile.global.v2.f32 {%0, %1}, [%2];" : "=f"(a), "=f"(b) : "l"(slot));
      arg_better(bv, bi, a, __float_as_int(b));
    }
    if (bi == 0x7fffffff) bi = 0;
    tokens[tid] = bi;
  }
  __syncthreads();
  if (tid == 0) {
    if (pos_ptr) pos_ptr[0] += pos_inc;
    pw.epoch[2] = e;
    if (tap.out) {
#pragma unroll
      for (int k = 0; k < 4; ++k) tap.out[k] = *reinterpret_cast<const volatile int*>(tap.src[k]);
    }
    __threadfence();
  }
  __syncthreads();
  pdl_launch_dependents();      // after the position write: the next step reads it early
}

// ---- SwiGLU on gate|up partials ---------------------------------------------
__global__ void __launch_bounds__(256)
k_swiglu(const float* __restrict__ P, PlanView pv, bf16* __restrict__ O, int rows, int inter,
         int interleaved, unsigned long long* tl) {
  tl_begin(tl);
  pdl_launch_dependents();
  pdl_wait();
  tl_waited(tl);
  const long long quads = (long long)rows * (inter >> 2);
  const long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= quads) return;
  const int m = (int)(q / (inter >> 2)), c = (int)(q % (inter >> 2)) * 4;
  const float* base = P + (long long)m * 2 * inter;
  const bool two = pv.u != 0;
  // columns of the gate and up sums of act columns c..c+3: [gate | up], or the layout of
  // q_gemm_swiglu's weight (blocks of 8 gate rows followed by their 8 up rows)
  const int gc = interleaved ? 16 * (c >> 3) + (c & 7) : c;
  const int uc = interleaved ? gc + 8 : inter + c;
  const float4 g0 = *reinterpret_cast<const float4*>(base + gc);
  const float4 u0 = *reinterpret_cast<const float4*>(base + uc);
  const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
  const int eg = plan_count(pv, gc, m) - 1, eu = plan_count(pv, uc, m) - 1;
  // Up to 256 rows the second slot is asked for without looking (one round trip, the lines
  // are in L2); the partials of a prompt pass are hundreds of MB, there only slots that hold
  // a partial are read.
  const bool many = pv.nblk != 0;
  const float4 g1 = two && (!many || eg > 0) ? *reinterpret_cast<const float4*>(base + gc + pv.slot_stride) : z;
  const float4 u1 = two && (!many || eu > 0) ? *reinterpret_cast<const float4*>(base + uc + pv.slot_stride) : z;
  float gs[4] = {g0.x, g0.y, g0.z, g0.w}, us[4] = {u0.x, u0.y, u0.z, u0.w};
  if (eg > 0) { gs[0] += g1.x; gs[1] += g1.y; gs[2] += g1.z; gs[3] += g1.w; }
  if (eu > 0) { us[0] += u1.x; us[1] += u1.y; us[2] += u1.z; us[3] += u1.w; }
  for (int k = 2; k <= eg; ++k) {
    const float4 t = *reinterpret_cast<const float4*>(base + gc + (long long)k * pv.slot_stride);
    gs[0] += t.x; gs[1] += t.y; gs[2] += t.z; gs[3] += t.w;
  }
  for (int k = 2; k <= eu; ++k) {
    const float4 t = *reinterpret_cast<const float4*>(base + uc + (long long)k * pv.slot_stride);
    us[0] += t.x; us[1] += t.y; us[2] += t.z; us[3] += t.w;
  }
  float o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float g = bf16_round(gs[e]), u = bf16_round(us[e]);
    o[e] = bf16_round(g / (1.0f + expf(-g))) * u;
  }
  uint2 pk;
  pk.x = pack_bf16(o[0], o[1]);
  pk.y = pack_bf16(o[2], o[3]);
  *reinterpret_cast<uint2*>(O + (long long)m * inter + c) = pk;
  tl_end(tl);
}

// ---- q/k head norm + RoPE + KV page write -------------------------------------
// One warp per (row, head) for q and k heads and one per v head; lane l owns dims
// 4l..4l+3 (one 16-byte load per partial slot), the rotate-half partner (d +- 64) is in
// lane l ^ 16.
__global__ void __launch_bounds__(128)
k_qkv_norm_rope_cache(const float* __restrict__ P, PlanView pv, const bf16* __restrict__ QG,
                      const bf16* __restrict__ KG, const bf16* __restrict__ COS,
                      const bf16* __restrict__ SIN, const int32_t* __restrict__ pos_ptr,
                      bf16* __restrict__ Q, char* __restrict__ kpool, char* __restrict__ vpool,
                      const int32_t* __restrict__ block_table, int pages_per_seq,
                      int rows, int T, int nq, int nkv, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int heads = nq + 2 * nkv;
  if (item >= rows * heads) return;
  const int m = item / heads, head = item % heads;       // head indexes the packed column blocks q|k|v
  const int b = m / T, tq = m % T;
  const int pos = pos_ptr[0] + tq;
  const int width = heads * 128;
  const bool is_q = head < nq, is_v = head >= nq + nkv;
  const long long src = (long long)m * width + (long long)head * 128 + 4 * lane;
  const float4 s0 = *reinterpret_cast<const float4*>(P + src);
  const int extra = plan_count(pv, head * 128 + 4 * lane, m) - 1;
  const float4 s1 = pv.u != 0 && (pv.nblk == 0 || extra > 0)
                        ? *reinterpret_cast<const float4*>(P + src + pv.slot_stride)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
  const uint2 graw = is_v ? make_uint2(0, 0) : *reinterpret_cast<const uint2*>((is_q ? QG : KG) + 4 * lane);
  const uint2 craw = *reinterpret_cast<const uint2*>(COS + (size_t)pos * 128 + 4 * lane);
  const uint2 sraw = *reinterpret_cast<const uint2*>(SIN + (size_t)pos * 128 + 4 * lane);
  float x[4] = {s0.x, s0.y, s0.z, s0.w};
  if (extra > 0) { x[0] += s1.x; x[1] += s1.y; x[2] += s1.z; x[3] += s1.w; }
  for (int k = 2; k <= extra; ++k) {
    const float4 sk = *reinterpret_cast<const float4*>(P + src + (long long)k * pv.slot_stride);
    x[0] += sk.x; x[1] += sk.y; x[2] += sk.z; x[3] += sk.w;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) x[e] = bf16_round(x[e]);
  uint2 o;
  if (is_v) {
    o.x = pack_bf16(x[0], x[1]);
    o.y = pack_bf16(x[2], x[3]);
  } else {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / 128.f + eps);
    const float gv[4] = {bf_lo(graw.x), bf_hi(graw.x), bf_lo(graw.y), bf_hi(graw.y)};
    const float cs[4] = {bf_lo(craw.x), bf_hi(craw.x), bf_lo(craw.y), bf_hi(craw.y)};
    const float sn[4] = {bf_lo(sraw.x), bf_hi(sraw.x), bf_lo(sraw.y), bf_hi(sraw.y)};
    float out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float n = bf16_round(bf16_round(x[e] * inv) * gv[e]);
      const float partner = __shfl_xor_sync(0xffffffffu, n, 16);
      const float rot = lane < 16 ? -partner : partner;
      out[e] = bf16_round(n * cs[e]) + bf16_round(rot * sn[e]);   // rounded to bf16 at the store
    }
    o.x = pack_bf16(out[0], out[1]);
    o.y = pack_bf16(out[2], out[3]);
  }
  if (is_q) {
    *reinterpret_cast<uint2*>(Q + ((size_t)m * nq + head) * 128 + 4 * lane) = o;
  } else {
    const int kh = is_v ? head - nq - nkv : head - nq;
    const int page = block_table[(size_t)b * pages_per_seq + pos / Q_PAGE_TOKENS];
    const int r = pos % Q_PAGE_TOKENS;
    const size_t tile = ((size_t)page * nkv + kh) * (Q_PAGE_TOKENS * 128 * 2);
    char* pool = is_v ? vpool : kpool;
    // dims 4l..4l+3 sit in 16-byte chunk l/2 of token row r
    *reinterpret_cast<uint2*>(pool + tile + r * 256 + (((lane >> 1) ^ (r & 7)) << 4) + (lane & 1) * 8) = o;
  }
}

// ---- scatter rotated K/V rows into pages (prefill helper) -----------------------
__global__ void __launch_bounds__(128)
k_kv_scatter(const bf16* __restrict__ Kin, const bf16* __restrict__ Vin, char* __restrict__ kpool,
             char* __restrict__ vpool, const int32_t* __restrict__ block_table,
             int pages_per_seq, int nkv, int len, int start) {
  // grid: (len, nkv, batch); 128 threads = one per dim
  const int p = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
  const int pos = start + p;
  const int page = block_table[(size_t)b * pages_per_seq + pos / Q_PAGE_TOKENS];
  const int r = pos % Q_PAGE_TOKENS;
  const size_t tile = ((size_t)page * nkv + h) * (Q_PAGE_TOKENS * 128 * 2);
  const size_t src = (((size_t)b * nkv + h) * len + p) * 128 + d;
  const int off = kv_tile_offset_bytes(r, d);
  *reinterpret_cast<bf16*>(kpool + tile + off) = Kin[src];
  *reinterpret_cast<bf16*>(vpool + tile + off) = Vin[src];
}

// ---- logits + argmax ----------------------------------------------------------------
// grid (blocks_per_row, rows). Each CTA rounds its slice of logits to bf16,
// optionally stores them, and finds (max, lowest index). The last CTA of a row
// (ticket counter) picks the row winner over the per-CTA results in index order.
constexpr int ARG_COLS = 4096;  // columns per CTA

struct ArgScratch {
  // layout: [rows] tickets (uint32) | [rows][blocks] val (float) | [rows][blocks] idx (int)
  unsigned int* tickets;
  float* val;
  int* idx;
};


__global__ void __launch_bounds__(256)
k_logits_argmax(const float* __restrict__ P, PlanView pv, bf16* __restrict__ logits,
                float* __restrict__ out_val, int32_t* __restrict__ out_idx,
                int64_t* __restrict__ tokens, int32_t* __restrict__ pos_ptr, int pos_inc,
                unsigned int* __restrict__ tickets, float* __restrict__ bval,
                int* __restrict__ bidx, int vocab, int vocab_offset, StatusTap tap,
                unsigned long long* tl) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ bool is_last;
  tl_begin(tl);
  // Kernels of the NEXT step read *pos_ptr before their own dependency wait (the
  // attention producer does), so dependents are released only at the very end, after
  // the position has been bumped.
  pdl_wait();
  tl_waited(tl);
  const int row = blockIdx.y, nblk = gridDim.x;
  const int c0 = blockIdx.x * ARG_COLS;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((vocab & 3) == 0) {
    // 4 columns per thread and step, 16-byte loads of both slots issued together
    const float* p0 = P + (long long)row * vocab;
    const bool two = pv.u != 0;
    for (int c = c0 + 4 * threadIdx.x; c < c0 + ARG_COLS && c < vocab; c += 1024) {
      const float4 a = *reinterpret_cast<const float4*>(p0 + c);
      const float4 b = two ? *reinterpret_cast<const float4*>(p0 + c + pv.slot_stride)
                           : make_float4(0.f, 0.f, 0.f, 0.f);
      const int extra = plan_count(pv, c, row) - 1;
      float s[4] = {a.x, a.y, a.z, a.w};
      if (extra > 0) { s[0] += b.x; s[1] += b.y; s[2] += b.z; s[3] += b.w; }
      for (int k = 2; k <= extra; ++k) {
        const float4 t = *reinterpret_cast<const float4*>(p0 + c + (long long)k * pv.slot_stride);
        s[0] += t.x; s[1] += t.y; s[2] += t.z; s[3] += t.w;
      }
      if (logits) {
        uint2 pk;
        pk.x = pack_bf16(s[0], s[1]);
        pk.y = pack_bf16(s[2], s[3]);
        *reinterpret_cast<uint2*>(logits + (long long)row * vocab + c) = pk;
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = bf16_round(s[e]);
        if (v != v) v = -INFINITY;  // NaN never wins
        arg_better(bv, bi, v, c + e);
      }
    }
  } else {
    for (int c = c0 + threadIdx.x; c < c0 + ARG_COLS && c < vocab; c += 256) {
      long long i = (long long)row * vocab + c;
      bf16 r = __float2bfloat16_rn(plan_sum(P, pv, i, c, row));
      if (logits) logits[i] = r;
      float v = __bfloat162float(r);
      if (v != v) v = -INFINITY;  // NaN never wins
      arg_better(bv, bi, v, c);
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    arg_better(bv, bi, ov, oi);
  }
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; ++k) arg_better(bv, bi, sv[k], si[k]);
    bval[(size_t)row * nblk + blockIdx.x] = bv;
    bidx[(size_t)row * nblk + blockIdx.x] = bi;
    __threadfence();
    unsigned int ticket = atomicAdd(&tickets[row], 1u);
    is_last = (ticket == (unsigned int)(nblk - 1));
  }
  __syncthreads();
  if (!is_last) {
    pdl_launch_dependents();
    return;
  }
  __threadfence();
  bv = -INFINITY;
  bi = 0x7fffffff;
  for (int k = threadIdx.x; k < nblk; k += 256) {
    float v = __ldcg(&bval[(size_t)row * nblk + k]);
    int i = __ldcg(&bidx[(size_t)row * nblk + k]);
    arg_better(bv, bi, v, i);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    arg_better(bv, bi, ov, oi);
  }
  __syncthreads();
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < 8; ++k) arg_better(bv, bi, sv[k], si[k]);
    if (bi == 0x7fffffff) bi = 0;
    out_val[row] = bv;
    out_idx[row] = bi + vocab_offset;
    if (tokens) tokens[row] = (int64_t)(bi + vocab_offset);
    if (pos_ptr && row == 0) pos_ptr[0] += pos_inc;
    if (tap.out && row == 0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) tap.out[k] = *reinterpret_cast<const volatile int*>(tap.src[k]);
    }
    tickets[row] = 0;  // ready for the next launch (graph replay)
    __threadfence();
  }
  __syncthreads();
  tl_end(tl);
  pdl_launch_dependents();
}

__global__ void k_argmax_merge(const float* __restrict__ val, const int32_t* __restrict__ idx,
                               int shards, int rows, int64_t* __restrict__ tokens,
                               int32_t* __restrict__ pos_ptr, int pos_inc, StatusTap tap) {
  pdl_wait();
  int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < rows) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int s = 0; s < shards; ++s) arg_better(bv, bi, val[(size_t)s * rows + row], idx[(size_t)s * rows + row]);
    if (bi == 0x7fffffff) bi = 0;
    tokens[row] = bi;
    if (row == 0 && pos_ptr) pos_ptr[0] += pos_inc;
    if (row == 0 && tap.out) {
#pragma unroll
      for (int k = 0; k < 4; ++k) tap.out[k] = *reinterpret_cast<const volatile int*>(tap.src[k]);
    }
  }
  __threadfence();
  pdl_launch_dependents();      // after the position write: see k_logits_argmax
}

}  // namespace

#define S(x) ((cudaStream_t)(x))

extern "C" int q_rmsnorm(const void* d_x, const void* d_gain, void* d_out, int rows, int cols,
                         float eps, void* stream) {
  Q_CHECK_ARG(d_x && d_gain && d_out && rows >= 1 && cols >= 1, "q_rmsnorm: bad argument");
  Q_CHECK_ALIGN(d_x, 2, "q_rmsnorm"); Q_CHECK_ALIGN(d_gain, 2, "q_rmsnorm"); Q_CHECK_ALIGN(d_out, 2, "q_rmsnorm");
  Q_CHECK_CUDA(q_launch(k_rmsnorm, dim3(rows), dim3(256), 0, S(stream), (const bf16*)d_x,
                        (const bf16*)d_gain, (bf16*)d_out, cols, eps));
  return Q_OK;
}

extern "C" int q_embed_rmsnorm(const int64_t* d_tokens, const void* d_embed, const void* d_gain,
                               void* d_x, void* d_normed, int rows, int cols, int vocab, float eps,
                               void* stream) {
  Q_CHECK_ARG(d_tokens && d_embed && d_gain && d_x && d_normed && rows >= 1 && cols >= 32 &&
                  cols % 32 == 0 && vocab >= 1,
              "q_embed_rmsnorm: bad argument (cols must be a multiple of 32)");
  Q_CHECK_ALIGN(d_tokens, 8, "q_embed_rmsnorm"); Q_CHECK_ALIGN(d_embed, 16, "q_embed_rmsnorm");
  Q_CHECK_ALIGN(d_x, 16, "q_embed_rmsnorm"); Q_CHECK_ALIGN(d_normed, 2, "q_embed_rmsnorm");
  Q_CHECK_ALIGN(d_gain, 2, "q_embed_rmsnorm");
  Q_CHECK_CUDA(q_launch(k_embed_rmsnorm, dim3(rows), dim3(256), 0, S(stream), d_tokens,
                        (const bf16*)d_embed, (const bf16*)d_gain, (bf16*)d_x, (bf16*)d_normed, cols,
                        vocab, eps, q_tl_next(Q_TL_EMBED)));
  return Q_OK;
}

static int check_plan(const q_gemm_plan_t* plan, int rows, int cols, const char* who) {
  if (plan) {
    Q_CHECK_ARG(plan->M == rows && plan->N == cols, "%s: plan is for [%d,%d], tensor is [%d,%d]", who,
                plan->M, plan->N, rows, cols);
    Q_CHECK_ARG(plan->units_per_worker >= 1 && plan->chunks_per_group >= 1, "%s: empty plan", who);
  }
  return Q_OK;
}

extern "C" int q_add_rmsnorm(const void* d_x_in, const float* d_branch, const q_gemm_plan_t* plan,
                             const void* d_gain, void* d_total_out, void* d_normed_out, int rows,
                             int cols, float eps, void* stream) {
  Q_CHECK_ARG(d_x_in && d_branch && d_gain && d_total_out && d_normed_out, "q_add_rmsnorm: null pointer");
  Q_CHECK_ARG(rows >= 1 && cols >= 4 && cols % 4 == 0 && cols <= 1024 * ADD_VB,
              "q_add_rmsnorm: cols %d must be a multiple of 4 in 4..%d", cols, 1024 * ADD_VB);
  Q_CHECK_ALIGN(d_branch, 16, "q_add_rmsnorm"); Q_CHECK_ALIGN(d_x_in, 8, "q_add_rmsnorm");
  Q_CHECK_ALIGN(d_gain, 8, "q_add_rmsnorm"); Q_CHECK_ALIGN(d_total_out, 8, "q_add_rmsnorm");
  Q_CHECK_ALIGN(d_normed_out, 8, "q_add_rmsnorm");
  int rc = check_plan(plan, rows, cols, "q_add_rmsnorm");
  if (rc) return rc;
  const bool wide = cols > 1024 && cols <= 4096 && plan != nullptr && plan->slots > 2;
  auto kern = wide ? k_add_rmsnorm<1, 1024>
                   : cols <= 1024 ? k_add_rmsnorm<1> : cols <= 3072 ? k_add_rmsnorm<3> : k_add_rmsnorm<ADD_VB>;
  Q_CHECK_CUDA(q_launch(kern, dim3(rows), dim3(wide ? 1024 : 256), 0, S(stream), (const bf16*)d_x_in,
                        d_branch, plan_view(plan), (const bf16*)d_gain, (bf16*)d_total_out,
                        (bf16*)d_normed_out, cols, eps, q_tl_next(Q_TL_ADD_NORM)));
  return Q_OK;
}


int q_peer_view(const q_peers_t* peers, PeerView* out, const char* who) {
  Q_CHECK_ARG(peers->world >= 2 && peers->world <= Q_MAX_PEERS && peers->rank >= 0 &&
                  peers->rank < peers->world && peers->epoch,
              "%s: bad rank/world or no counter words", who);
  out->rank = peers->rank;
  out->world = peers->world;
  out->epoch = peers->epoch;
  for (int r = 0; r < Q_MAX_PEERS; ++r) {
    out->recv[r] = r < peers->world ? peers->partials[r] : nullptr;
    out->flags[r] = r < peers->world ? peers->flags[r] : nullptr;
    Q_CHECK_ARG(r >= peers->world || (out->recv[r] && out->flags[r]), "%s: rank %d unmapped", who, r);
    Q_CHECK_ARG(((uintptr_t)out->recv[r] & 15) == 0 && ((uintptr_t)out->flags[r] & 15) == 0,
                "%s: peer buffers must be 16-byte aligned", who);
  }
  return Q_OK;
}

extern "C" int q_add_rmsnorm_peers(const void* d_x_in, const q_peers_t* peers, const float* d_own_branch,
                                   const q_gemm_plan_t* plan, const void* d_gain, void* d_total_out,
                                   void* d_normed_out, int rows, int cols, float eps, void* stream) {
  Q_CHECK_ARG(d_x_in && peers && d_own_branch && d_gain && d_total_out && d_normed_out,
              "q_add_rmsnorm_peers: null pointer");
  Q_CHECK_ARG(rows >= 1 && rows <= Q_MAX_ROWS && cols >= 4 && cols % 4 == 0 && cols <= PEER_MAX_COLS,
              "q_add_rmsnorm_peers: needs 1..%d rows and cols a multiple of 4 up to %d", Q_MAX_ROWS, PEER_MAX_COLS);
  Q_CHECK_ARG((((uintptr_t)d_x_in | (uintptr_t)d_gain | (uintptr_t)d_total_out | (uintptr_t)d_normed_out) & 7) == 0,
              "q_add_rmsnorm_peers: bf16 operands must be 8-byte aligned");
  Q_CHECK_ALIGN(d_own_branch, 16, "q_add_rmsnorm_peers");
  int rc = check_plan(plan, rows, cols, "q_add_rmsnorm_peers");
  if (rc) return rc;
  PeerView pw;
  rc = q_peer_view(peers, &pw, "q_add_rmsnorm_peers");
  if (rc) return rc;
  const int threads = ((cols + 127) / 128) * 32;        // one warp per 128 columns
  Q_CHECK_CUDA(q_launch(k_add_rmsnorm_peers, dim3(rows), dim3(threads), 0, S(stream), (const bf16*)d_x_in, pw,
                        d_own_branch, plan_view(plan), (const bf16*)d_gain, (bf16*)d_total_out,
                        (bf16*)d_normed_out, rows, cols, eps, g_peer_wait_iters, q_tl_next(Q_TL_PEER_ADD_NORM)));
  return Q_OK;
}

extern "C" int64_t q_peer_flag_bytes(void) {
  // 512 bytes of arrival words, then [2 parities][Q_MAX_PEERS shards][Q_MAX_ROWS] pairs of 8 bytes
  return 512 + 2ll * Q_MAX_PEERS * Q_MAX_ROWS * 8;
}

int q_argmax_merge_peers_tap(const float* d_val, const int32_t* d_idx, const q_peers_t* peers, int rows,
                             int64_t* d_tokens, int32_t* d_pos, int pos_inc, StatusTap tap, void* stream) {
  Q_CHECK_ARG(d_val && d_idx && peers && d_tokens && rows >= 1 && rows <= Q_MAX_ROWS,
              "q_argmax_merge_peers: bad argument");
  PeerView pw;
  int rc = q_peer_view(peers, &pw, "q_argmax_merge_peers");
  if (rc) return rc;
  Q_CHECK_CUDA(q_launch(k_argmax_merge_peers, dim3(1), dim3(64), 0, S(stream), d_val, d_idx, pw, rows, d_tokens,
                        d_pos, pos_inc, g_peer_wait_iters, tap));
  return Q_OK;
}

extern "C" int q_argmax_merge_peers(const float* d_val, const int32_t* d_idx, const q_peers_t* peers, int rows,
                                    int64_t* d_tokens, int32_t* d_pos, int pos_inc, void* stream) {
  StatusTap none = {};
  return q_argmax_merge_peers_tap(d_val, d_idx, peers, rows, d_tokens, d_pos, pos_inc, none, stream);
}

Q_DEFINE_STATUS_ADDR(q_peer_status_addr, g_peer_status)

int q_swiglu_layout(const float* d_branch, const q_gemm_plan_t* plan, void* d_out, int rows, int inter,
                    int interleaved, void* stream) {
  Q_CHECK_ARG(d_branch && d_out && rows >= 1 && inter >= 4 && inter % 4 == 0,
              "q_swiglu: bad argument (inter must be a multiple of 4)");
  Q_CHECK_ARG(((uintptr_t)d_branch & 15) == 0 && ((uintptr_t)d_out & 7) == 0,
              "q_swiglu: the partials must be 16-byte and the output 8-byte aligned");
  Q_CHECK_ARG(!interleaved || inter % 8 == 0, "q_swiglu: the interleaved layout needs inter %% 8 == 0");
  int rc = check_plan(plan, rows, 2 * inter, "q_swiglu");
  if (rc) return rc;
  long long total = (long long)rows * (inter / 4);
  Q_CHECK_CUDA(q_launch(k_swiglu, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, S(stream),
                        d_branch, plan_view(plan), (bf16*)d_out, rows, inter, interleaved, q_tl_next(Q_TL_SWIGLU)));
  return Q_OK;
}

extern "C" int q_swiglu(const float* d_branch, const q_gemm_plan_t* plan, void* d_out, int rows,
                        int inter, void* stream) {
  return q_swiglu_layout(d_branch, plan, d_out, rows, inter, 0, stream);
}

extern "C" int q_swiglu_interleaved(const float* d_branch, const q_gemm_plan_t* plan, void* d_out, int rows,
                                    int inter, void* stream) {
  return q_swiglu_layout(d_branch, plan, d_out, rows, inter, 1, stream);
}

extern "C" int q_qkv_norm_rope_cache(const float* d_branch, const q_gemm_plan_t* plan,
                                     const void* d_q_gain, const void* d_k_gain, const void* d_cos,
                                     const void* d_sin, const int32_t* d_pos, void* d_q_out,
                                     const q_kv_layout_t* kv, int batch, int T, int n_q_heads,
                                     float eps, void* stream) {
  Q_CHECK_ARG(d_branch && d_q_gain && d_k_gain && d_cos && d_sin && d_pos && d_q_out && kv,
              "q_qkv_norm_rope_cache: null pointer");
  Q_CHECK_ARG(kv->d_kpool && kv->d_vpool && kv->d_block_table && kv->pages_per_seq >= 1 &&
                  kv->n_kv_heads >= 1,
              "q_qkv_norm_rope_cache: incomplete KV layout");
  Q_CHECK_ARG(batch >= 1 && T >= 1 && n_q_heads >= 1 && (long long)batch * T <= (1 << 20),
              "q_qkv_norm_rope_cache: bad batch/T");
  const int rows = batch * T, nkv = kv->n_kv_heads;
  Q_CHECK_ALIGN(d_branch, 16, "q_qkv_norm_rope_cache"); Q_CHECK_ALIGN(d_q_gain, 8, "q_qkv_norm_rope_cache");
  Q_CHECK_ALIGN(d_k_gain, 8, "q_qkv_norm_rope_cache"); Q_CHECK_ALIGN(d_cos, 8, "q_qkv_norm_rope_cache");
  Q_CHECK_ALIGN(d_sin, 8, "q_qkv_norm_rope_cache"); Q_CHECK_ALIGN(d_q_out, 8, "q_qkv_norm_rope_cache");
  Q_CHECK_ALIGN(kv->d_kpool, 16, "q_qkv_norm_rope_cache"); Q_CHECK_ALIGN(kv->d_vpool, 16, "q_qkv_norm_rope_cache");
  int rc = check_plan(plan, rows, (n_q_heads + 2 * nkv) * 128, "q_qkv_norm_rope_cache");
  if (rc) return rc;
  const int items = rows * (n_q_heads + 2 * nkv);
  Q_CHECK_CUDA(q_launch(k_qkv_norm_rope_cache, dim3((items + 3) / 4), dim3(128), 0, S(stream),
                        d_branch, plan_view(plan), (const bf16*)d_q_gain, (const bf16*)d_k_gain,
                        (const bf16*)d_cos, (const bf16*)d_sin, d_pos, (bf16*)d_q_out,
                        (char*)kv->d_kpool, (char*)kv->d_vpool, kv->d_block_table, kv->pages_per_seq,
                        rows, T, n_q_heads, nkv, eps));
  return Q_OK;
}

extern "C" int q_kv_scatter(const void* d_k, const void* d_v, const q_kv_layout_t* kv, int batch,
                            int len, int start, void* stream) {
  Q_CHECK_ARG(d_k && d_v && kv && kv->d_kpool && kv->d_vpool && kv->d_block_table,
              "q_kv_scatter: null pointer");
  Q_CHECK_ARG(batch >= 1 && len >= 1 && start >= 0 && batch <= 65535 && kv->n_kv_heads <= 65535,
              "q_kv_scatter: bad sizes");
  Q_CHECK_ARG((start + len + Q_PAGE_TOKENS - 1) / Q_PAGE_TOKENS <= kv->pages_per_seq,
              "q_kv_scatter: positions exceed the block table");
  k_kv_scatter<<<dim3(len, kv->n_kv_heads, batch), 128, 0, S(stream)>>>(
      (const bf16*)d_k, (const bf16*)d_v, (char*)kv->d_kpool, (char*)kv->d_vpool, kv->d_block_table,
      kv->pages_per_seq, kv->n_kv_heads, len, start);
  Q_CHECK_CUDA(cudaGetLastError());
  return Q_OK;
}

static inline int arg_blocks(int vocab) { return (vocab + ARG_COLS - 1) / ARG_COLS; }

extern "C" int64_t q_argmax_scratch_bytes(int rows, int vocab) {
  if (rows < 1 || vocab < 1) return 0;
  int64_t nblk = arg_blocks(vocab);
  int64_t tick = ((int64_t)rows * 4 + 255) / 256 * 256;
  return tick + (int64_t)rows * nblk * 8;
}

extern "C" int q_logits_argmax(const float* d_branch, const q_gemm_plan_t* plan, void* d_logits,
                               float* d_val, int32_t* d_idx, int64_t* d_tokens, int32_t* d_pos,
                               int pos_inc, void* d_block_scratch, int rows, int vocab,
                               int vocab_offset, void* stream) {
  StatusTap none = {};
  return q_logits_argmax_tap(d_branch, plan, d_logits, d_val, d_idx, d_tokens, d_pos, pos_inc,
                             d_block_scratch, rows, vocab, vocab_offset, none, stream);
}

int q_logits_argmax_tap(const float* d_branch, const q_gemm_plan_t* plan, void* d_logits, float* d_val,
                        int32_t* d_idx, int64_t* d_tokens, int32_t* d_pos, int pos_inc,
                        void* d_block_scratch, int rows, int vocab, int vocab_offset, StatusTap tap,
                        void* stream) {
  Q_CHECK_ARG(d_branch && d_val && d_idx && d_block_scratch, "q_logits_argmax: null pointer");
  Q_CHECK_ARG(rows >= 1 && rows <= Q_MAX_ROWS && vocab >= 1, "q_logits_argmax: bad sizes");
  Q_CHECK_ALIGN(d_branch, 16, "q_logits_argmax"); Q_CHECK_ALIGN(d_logits, 8, "q_logits_argmax");
  Q_CHECK_ALIGN(d_block_scratch, 4, "q_logits_argmax"); Q_CHECK_ALIGN(d_tokens, 8, "q_logits_argmax");
  int rc = check_plan(plan, rows, vocab, "q_logits_argmax");
  if (rc) return rc;
  const int nblk = arg_blocks(vocab);
  char* base = (char*)d_block_scratch;
  int64_t tick = ((int64_t)rows * 4 + 255) / 256 * 256;
  unsigned int* tickets = (unsigned int*)base;
  float* bval = (float*)(base + tick);
  int* bidx = (int*)(base + tick + (int64_t)rows * nblk * 4);
  Q_CHECK_CUDA(q_launch(k_logits_argmax, dim3(nblk, rows), dim3(256), 0, S(stream), d_branch,
                        plan_view(plan), (bf16*)d_logits, d_val, d_idx, d_tokens, d_pos, pos_inc,
                        tickets, bval, bidx, vocab, vocab_offset, tap, q_tl_next(Q_TL_ARGMAX)));
  return Q_OK;
}

int q_argmax_merge_tap(const float* d_val, const int32_t* d_idx, int shards, int rows, int64_t* d_tokens,
                       int32_t* d_pos, int pos_inc, StatusTap tap, void* stream) {
  Q_CHECK_ARG(d_val && d_idx && d_tokens && shards >= 1 && rows >= 1, "q_argmax_merge: bad argument");
  Q_CHECK_CUDA(q_launch(k_argmax_merge, dim3((rows + 63) / 64), dim3(64), 0, S(stream), d_val, d_idx,
                        shards, rows, d_tokens, d_pos, pos_inc, tap));
  return Q_OK;
}

extern "C" int q_argmax_merge(const float* d_val, const int32_t* d_idx, int shards, int rows,
                              int64_t* d_tokens, int32_t* d_pos, int pos_inc, void* stream) {
  StatusTap none = {};
  return q_argmax_merge_tap(d_val, d_idx, shards, rows, d_tokens, d_pos, pos_inc, none, stream);
}
