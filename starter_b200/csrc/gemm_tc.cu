// Weight-streaming GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory) for 9 .. 256 activation rows.
//
// Y[M,N] = X[M,K] . W[N,K]^T, bf16 operands, fp32 accumulation, written as the same fp32
// split-K partial slots that the stream-K kernel of gemm_streamk.cu produces, so the fused
// consumers (add+norm, SwiGLU, head norm + RoPE, argmax) read either
// (reference: engine/kernels/skinny_gemm.py:28-46 at BLOCK_M = 32 / 64, one tl.dot per tile).
//
// Operands are swapped so that the batch never pads the large MMA dimension: the WEIGHT rows
// fill the M = 128 slot of the instruction and the activation rows sit in its N slot (16, 32,
// 64, 128 or 256). One 128 x 64 weight tile is one contiguous 16 KB block in HBM that already
// is the shared-memory image the MMA wants (K-major, 128-byte swizzle: 8-row x 128-byte atoms,
// the 16-byte chunk index of row r XOR-ed with r % 8), so a plain bulk copy brings it in; the
// matching 64-k slice of the activations comes through a TMA tensor map with the same swizzle
// (rows past M are zero-filled by the copy engine).
//
// Roles inside a CTA (one CTA per SM, 192 threads):
//   warp 0   producer: one lane keeps a ring of `stages` (weight tile, activation tile) pairs
//            full; the first `stages` weight tiles are requested before the dependency wait
//            (weights do not depend on the previous kernel), the activation tiles after it;
//   warp 1   one lane issues four tcgen05.mma (k = 16 each) per tile into one of two
//            accumulator buffers in tensor memory and commits the stage back to the producer;
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (lane = weight row, column =
//            activation row) and store it as a partial slot, while the MMA warp already
//            fills the other buffer.
// Work split: stream-K over tiles in (128-row block, k tile) order; CTA c owns tiles
// [c U, (c+1) U). A block that two CTAs share gets one partial per CTA: slot = CTA - first CTA
// of the block, exactly the slot rule of the stream-K kernel with "group" = 128 rows.
//
// Every mbarrier wait is bounded. A wait that runs out records a code in this file's status
// word and raises a CTA-wide abort flag; every role then leaves its loop, the producer waits
// (bounded) for its copies in flight, tensor memory is freed and the kernel returns.
#include <cuda.h>
#include "common.cuh"

extern int g_gemm_debug_flags;   // q_set_option "gemm_debug_flags": 4 = per-CTA stamps, 16 = no MMA issue

namespace {

constexpr int TC_THREADS = 192;
constexpr int TILE_ROWS = 128;
constexpr int TILE_K = 64;
constexpr int W_TILE_BYTES = TILE_ROWS * TILE_K * 2;      // 16 KB
constexpr int SMEM_BUDGET = 222 * 1024;                   // ring bytes at most
constexpr unsigned WAIT_LIMIT = 1u << 22;

__device__ int g_tc_status[4];
// Measurement aid (debug flag 4): per CTA {start, set-up done, producer past the dependency
// wait, first stage landed, last MMA issued, last accumulator stored, exit, tiles} in ns.
__device__ unsigned long long g_tc_trace[256 * 8];
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

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
// Bounded wait; false when the limit ran out or another role raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (unsigned it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if (it > 128) {
      __nanosleep(32);
      if ((it & 255) == 0 && *abort_flag) return false;
    }
  }
  return false;
}
// The same without the abort flag (used to drain copies in flight after an abort).
__device__ __forceinline__ bool mbar_wait_plain(uint32_t bar, uint32_t parity) {
  for (unsigned it = 0; it < WAIT_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if (it > 128) __nanosleep(32);
  }
  return false;
}
__device__ __forceinline__ uint64_t stream_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
// 2-D tiled TMA load: box (64 k, m_pad rows) at element coordinates (x = k offset, y = row).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] . B[smem desc]^T, one thread issues.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major operand tile with 128-byte swizzle: start
// address / 16 in bits 0-13, leading-dimension offset (unused for swizzled K-major, 1),
// stride between 8-row atoms 1024 B / 16 in bits 32-45, descriptor version 1 in bits 46-47,
// layout type 2 (128-byte swizzle) in bits 61-63. Moving 16 k (32 bytes) along K inside the
// 128-byte atom adds 2 to the start-address field.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

struct TcShape {
  int M;          // activation rows of this launch (more than m_pad: row chunks of m_pad rows)
  int N;          // weight rows
  int KT;         // k tiles (K rounded up to 64, / 64)
  int nblk;       // 128-row weight blocks
  int total;      // tiles = row chunks * nblk * KT, in (row chunk, weight block, k tile) order
  int U;          // tiles per CTA
  int m_pad;      // MMA N: 16, 32, 64, 128 or 256
  int stages;     // ring depth
  int row0;       // first activation row (coordinate in the tensor map)
  long long slot_stride;   // floats between partial slots (rows of the whole output x N)
  int out_rows;   // rows of the whole output the partial buffer was sized for
};

__global__ void __launch_bounds__(TC_THREADS, 1)
k_gemm_tc(const __grid_constant__ CUtensorMap xmap, const unsigned char* __restrict__ W, float* __restrict__ P,
          TcShape sh, int dbg, unsigned long long* tl) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;            // tiles need 1024-byte alignment
  unsigned char* smem = smem_raw + (base - raw);
  const uint32_t stage_bytes = W_TILE_BYTES + (uint32_t)sh.m_pad * 128u;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)sh.stages * stage_bytes);
  // full[stages] | empty[stages] | acc_full[2] | acc_empty[2]
  const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8u * sh.stages;
  const uint32_t bar_acc_full = bar_empty + 8u * sh.stages, bar_acc_empty = bar_acc_full + 16u;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * sh.stages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  tl_begin(tl);
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool trace = (dbg & 4) && blockIdx.x < 256;
  unsigned long long* tr = g_tc_trace + blockIdx.x * 8;
  if (trace && tid == 0) tr[0] = gtime();
  const int t0 = blockIdx.x * sh.U;
  const int t1 = min(sh.total, t0 + sh.U);
  const int n_tiles = t1 > t0 ? t1 - t0 : 0;
  // tensor-memory columns: two accumulator buffers of m_pad columns, a power of two >= 32
  // (spreading the k-steps of a tile over several accumulators measured no faster)
  const int acc_cols = sh.m_pad;
  uint32_t ncols = 32;
  while (ncols < 2u * acc_cols) ncols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < sh.stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (trace && tid == 0) { tr[1] = gtime(); tr[7] = (unsigned long long)n_tiles; }

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      const uint64_t policy = stream_policy();
      const int first = min(sh.stages, n_tiles);
      const int per_chunk = sh.nblk * sh.KT;               // tiles of one pass over the weight
      for (int i = 0; i < first; ++i) {
        mbar_expect_tx(bar_full + 8 * i, stage_bytes);
        bulk_g2s(base + i * stage_bytes, W + (size_t)((t0 + i) % per_chunk) * W_TILE_BYTES, W_TILE_BYTES,
                 bar_full + 8 * i, policy);
      }
      pdl_wait();                       // the activations are complete from here on
      tl_waited(tl);
      if (trace) tr[2] = gtime();
      for (int i = 0; i < first; ++i) {
        const int kt = (t0 + i) % sh.KT;
        const int xrow = sh.row0 + ((t0 + i) / per_chunk) * sh.m_pad;
        tma_load_2d(base + i * stage_bytes + W_TILE_BYTES, &xmap, kt * TILE_K, xrow, bar_full + 8 * i);
      }
      // Refill loop. One thread issues everything, so its instruction count per tile is what
      // bounds the copy rate: stage index, barrier parity and k tile are carried along instead
      // of being divided out of the tile number.
      bool ok = true;
      int issued_tiles = first;
      {
        int st = 0;                                        // stage of tile `first`
        uint32_t parity = 0;                               // phase of empty[st] to wait for
        int kt = (t0 + first) % sh.KT;
        int in_chunk = (t0 + first) % per_chunk;           // tile index inside the weight pass
        int xrow = sh.row0 + ((t0 + first) / per_chunk) * sh.m_pad;
        uint32_t dst = base, full = bar_full, empty = bar_empty;
        const unsigned char* src = W + (size_t)in_chunk * W_TILE_BYTES;
        for (int i = first; i < n_tiles; ++i) {
          if (!mbar_wait(empty, parity, abort_flag)) {
            atomicExch(&g_tc_status[0], 1);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(full, stage_bytes);
          bulk_g2s(dst, src, W_TILE_BYTES, full, policy);
          tma_load_2d(dst + W_TILE_BYTES, &xmap, kt * TILE_K, xrow, full);
          issued_tiles = i + 1;
          src += W_TILE_BYTES;
          if (++kt == sh.KT) kt = 0;
          if (++in_chunk == per_chunk) { in_chunk = 0; src = W; xrow += sh.m_pad; }   // next row chunk
          if (++st == sh.stages) {
            st = 0; parity ^= 1u; dst = base; full = bar_full; empty = bar_empty;
          } else {
            dst += stage_bytes; full += 8; empty += 8;
          }
        }
      }
      // Copies in flight must land before the CTA may exit, also when a role gave up: the
      // last fill of every stage flips that stage's `full` barrier once more.
      const int issued = ok ? n_tiles : issued_tiles;
      for (int s = 0; s < sh.stages; ++s) {
        if (issued <= s) break;
        const int last = ((issued - 1 - s) / sh.stages) * sh.stages + s;
        if (!mbar_wait_plain(bar_full + 8 * s, (last / sh.stages) & 1)) atomicExch(&g_tc_status[0], 4);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(sh.m_pad >> 3) << 17) |
                             ((uint32_t)(TILE_ROWS >> 4) << 24);     // f32 accum, bf16 x bf16, K-major both
      // Like the producer, this thread's instruction count per tile matters (a loop with
      // three integer divisions per tile made the tensor pipe look like the bottleneck): all
      // indices are carried along, the four k-steps are unrolled.
      const uint32_t stage_units = stage_bytes >> 4;       // descriptor address units (16 B)
      const uint64_t desc0 = smem_desc(base);
      int seg = 0;
      int st = 0;
      int kt = t0 % sh.KT;
      uint32_t full_parity = 0;
      uint32_t full = bar_full, empty = bar_empty;
      uint64_t a_desc = desc0;
      uint32_t dacc = tmem_base;
      uint32_t acc_full_bar = bar_acc_full;
      for (int i = 0; i < n_tiles; ++i) {
        const bool seg_start = (i == 0) || kt == 0;
        if (seg_start) {
          const int buf = seg & 1;
          // the epilogue has drained this buffer (passes at once for the first two segments)
          if (!mbar_wait(bar_acc_empty + 8 * buf, ((seg >> 1) & 1) ^ 1, abort_flag)) {
            atomicExch(&g_tc_status[0], 2);
            *abort_flag = 1;
            break;
          }
          dacc = tmem_base + (uint32_t)(buf * acc_cols);
          acc_full_bar = bar_acc_full + 8 * buf;
        }
        if (!mbar_wait(full, full_parity, abort_flag)) {
          atomicExch(&g_tc_status[0], 2);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        if (trace && i == 0) tr[3] = gtime();
        const uint64_t b_desc = a_desc + (W_TILE_BYTES >> 4);
        if (!(dbg & 16)) {
#pragma unroll
          for (int k = 0; k < TILE_K / 16; ++k)
            tc_mma(dacc, a_desc + 2u * k, b_desc + 2u * k, idesc, (seg_start && k == 0) ? 0u : 1u);
        }
        tc_commit(empty);                             // the stage is free when these MMAs are done
        if (++kt == sh.KT) kt = 0;
        if (kt == 0 || i == n_tiles - 1) {
          tc_commit(acc_full_bar);                    // ... and so is the accumulator
          ++seg;
        }
        if (++st == sh.stages) {
          st = 0; full_parity ^= 1u; full = bar_full; empty = bar_empty; a_desc = desc0;
        } else {
          full += 8; empty += 8; a_desc += stage_units;
        }
      }
      if (trace) tr[4] = gtime();
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    pdl_wait();                         // earlier readers of the partial buffer are done
    const int q = warp & 3;             // this warp may read tensor-memory lanes 32q .. 32q+31
    int seg = 0;
    int i = 0;
    while (i < n_tiles) {
      const int t = t0 + i;
      const int block = t / sh.KT, kt = t - block * sh.KT;
      const int len = min(n_tiles - i, sh.KT - kt);
      const int buf = seg & 1;
      // all lanes poll; the verdict is made warp-uniform (tcgen05.ld needs the whole warp)
      const int landed = mbar_wait(bar_acc_full + 8 * buf, (seg >> 1) & 1, abort_flag) ? 1 : 0;
      if (!__all_sync(0xffffffffu, landed)) {
        if (lane == 0) {
          atomicExch(&g_tc_status[0], 3);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after();
      const int first_cta = (int)(((long long)block * sh.KT) / sh.U);
      float* out = P + (long long)((int)blockIdx.x - first_cta) * sh.slot_stride;
      const int chunk = block / sh.nblk, wblock = block - chunk * sh.nblk;
      const int m0 = chunk * sh.m_pad;                      // first row of this segment's row chunk
      const int n = wblock * TILE_ROWS + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * acc_cols);
      for (int c0 = 0; c0 < sh.m_pad; c0 += 16) {
        if (m0 + c0 >= sh.M) break;     // warp-uniform
        float v[16];
        tc_ld16(taddr + c0, v);
        if (n < sh.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < sh.M) out[(size_t)(sh.row0 + m) * sh.N + n] = v[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      i += len;
      ++seg;
    }
    if (trace && warp == 2 && lane == 0) tr[5] = gtime();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(ncols) : "memory");
  }
  if (trace && tid == 0) tr[6] = gtime();
  tl_end(tl);
}

// Row-major [N][K] <-> 128 x 64 tiles in the swizzled shared-memory image. One thread per
// 16-byte chunk of the tiled side; rows past N and k past K are zero.
__global__ void k_pack_t128(const uint4* __restrict__ src, uint4* __restrict__ dst, int N, int K, int KT,
                            long long chunks, int to_tiled) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= chunks) return;
  const long long tile = i >> 10;                  // 1024 chunks of 16 B per tile
  const int in_tile = (int)(i & 1023);
  const int r = in_tile >> 3;                      // row inside the tile (128 B per row)
  const int phys = in_tile & 7;                    // physical chunk inside the row
  const int logical = phys ^ (r & 7);              // k chunk it holds
  const int block = (int)(tile / KT), kt = (int)(tile - (long long)block * KT);
  const int row = block * TILE_ROWS + r;
  const int k = kt * TILE_K + logical * 8;
  const bool inside = row < N && k < K;            // K is a multiple of 8
  const long long rm = ((long long)row * K + k) >> 3;
  if (to_tiled) {
    dst[i] = inside ? src[rm] : make_uint4(0, 0, 0, 0);
  } else if (inside) {
    dst[rm] = src[i];
  }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime (the library does not link
// against libcuda, so it still loads on a host without a driver).
encode_tiled_fn encoder() {
  static encode_tiled_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    fn = (encode_tiled_fn)p;
  }
  return fn;
}

int pad_rows(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

int stages_for(int m_pad) {
  const int stage = W_TILE_BYTES + m_pad * 128;
  int s = SMEM_BUDGET / stage;
  return s > 12 ? 12 : s;
}

size_t tc_smem(int m_pad, int stages) {
  return 1024 + (size_t)stages * (W_TILE_BYTES + m_pad * 128) + (2 * stages + 4) * 8 + 16;
}

}  // namespace

Q_DEFINE_STATUS_ADDR(q_tc_status_addr, g_tc_status)

extern "C" int q_debug_tc_trace(unsigned long long* out, int n_ctas) {
  Q_CHECK_ARG(out && n_ctas >= 1 && n_ctas <= 256, "q_debug_tc_trace: bad argument");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(unsigned long long) * 8 * n_ctas));
  return Q_OK;
}

extern "C" int64_t q_packed_weight_bytes_tc(int N, int K) {
  if (N < 1 || K < 32 || K % 32) return -1;
  return (int64_t)((N + TILE_ROWS - 1) / TILE_ROWS) * ((K + TILE_K - 1) / TILE_K) * W_TILE_BYTES;
}

static int pack_tc_common(const void* src, void* dst, int N, int K, int to_tiled, void* stream, const char* who) {
  Q_CHECK_ARG(src && dst, "%s: null pointer", who);
  Q_CHECK_ARG(N >= 1 && K >= 32 && K % 32 == 0, "%s: need N >= 1 and K a multiple of 32", who);
  Q_CHECK_ARG(((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0, "%s: pointers must be 16-byte aligned", who);
  const int KT = (K + TILE_K - 1) / TILE_K;
  const long long chunks = (long long)((N + TILE_ROWS - 1) / TILE_ROWS) * KT * 1024;
  const long long grid = (chunks + 255) / 256;
  Q_CHECK_ARG(grid < (1ll << 31), "%s: weight too large", who);
  k_pack_t128<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, N, K, KT, chunks,
                                                                to_tiled);
  Q_CHECK_CUDA(cudaGetLastError());
  return Q_OK;
}

extern "C" int q_pack_weight_tc(const void* d_rowmajor, void* d_tiled, int N, int K, void* stream) {
  return pack_tc_common(d_rowmajor, d_tiled, N, K, 1, stream, "q_pack_weight_tc");
}

extern "C" int q_unpack_weight_tc(const void* d_tiled, void* d_rowmajor, int N, int K, void* stream) {
  return pack_tc_common(d_tiled, d_rowmajor, N, K, 0, stream, "q_unpack_weight_tc");
}

extern "C" int q_gemm_tc_plan(int M, int N, int K, q_gemm_plan_t* plan) {
  Q_CHECK_ARG(plan != nullptr, "q_gemm_tc_plan: null plan");
  Q_CHECK_ARG(M >= 1, "q_gemm_tc_plan: no rows");
  Q_CHECK_ARG(N >= 1 && K >= 32 && K % 32 == 0,
              "q_gemm_tc_plan: need N >= 1 and K a positive multiple of 32 (N=%d K=%d)", N, K);
  int sms = q_sm_count();
  if (sms <= 0) sms = 148;
  const int KT = (K + TILE_K - 1) / TILE_K;
  // More than 256 rows: row chunks of 256, one launch over (row chunk, weight block, k tile);
  // a "group" of the plan is then one (row chunk, weight block) pair.
  const int row_chunks = (M + 255) / 256;
  const long long blocks = (long long)((N + TILE_ROWS - 1) / TILE_ROWS) * row_chunks;
  const long long total = blocks * KT;
  Q_CHECK_ARG(total < (1ll << 30), "q_gemm_tc_plan: too many tiles");
  long long u = (total + sms - 1) / sms;
  if (u < 1) u = 1;
  const long long workers = (total + u - 1) / u;
  long long slots = (KT - 1 + u - 1) / u + 1;
  if (slots > workers) slots = workers;
  if (slots < 2) slots = 2;
  plan->M = M; plan->N = N; plan->K = K;
  plan->chunks_per_group = KT;
  plan->groups = (int)blocks;
  plan->units_per_worker = (int)u;
  plan->workers = (int)workers;
  plan->slots = (int)slots;
  plan->grid = (int)workers;
  plan->block = TC_THREADS;
  plan->group_rows = TILE_ROWS;
  return Q_OK;
}

// Launches the projection for rows [0, plan->M) of X (leading dimension K): one launch; above
// 256 rows every CTA walks (row chunk, weight block, k tile) in that order, so the weight is
// streamed once per 256 rows (from L2 after the first pass where it fits).
int q_gemm_tc_launch(const void* d_x, const void* d_w_tc, float* d_partials, const q_gemm_plan_t* plan,
                     void* stream) {
  const q_gemm_plan_t& p = *plan;
  Q_CHECK_ARG(p.group_rows == TILE_ROWS, "q_gemm_tc: the plan was not made by q_gemm_tc_plan");
  encode_tiled_fn enc = encoder();
  if (!enc) { q_set_error("q_gemm_tc: the driver has no cuTensorMapEncodeTiled"); return Q_ERR_CUDA; }
  static size_t smem_done[64] = {0};
  const int m_pad = pad_rows(p.M);
  const int stages = stages_for(m_pad);
  const int nblk = (p.N + TILE_ROWS - 1) / TILE_ROWS;
  Q_CHECK_ARG(p.groups == nblk * ((p.M + 255) / 256), "q_gemm_tc: the plan does not match its own shape");
  CUtensorMap map;
  const cuuint64_t gdim[2] = {(cuuint64_t)p.K, (cuuint64_t)p.M};
  const cuuint64_t gstride[1] = {(cuuint64_t)p.K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)m_pad};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(d_x), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { q_set_error("q_gemm_tc: cuTensorMapEncodeTiled failed (%d)", (int)r); return Q_ERR_CUDA; }
  TcShape sh;
  sh.M = p.M; sh.N = p.N; sh.KT = p.chunks_per_group; sh.nblk = nblk; sh.total = p.groups * p.chunks_per_group;
  sh.U = p.units_per_worker; sh.m_pad = m_pad; sh.stages = stages; sh.row0 = 0;
  sh.slot_stride = (long long)p.M * p.N; sh.out_rows = p.M;
  const size_t smem = tc_smem(m_pad, stages);
  Q_CHECK_CUDA(q_ensure_smem(k_gemm_tc, smem, smem_done));
  Q_CHECK_CUDA(q_launch(k_gemm_tc, dim3(p.grid), dim3(TC_THREADS), smem, (cudaStream_t)stream, map,
                        (const unsigned char*)d_w_tc, d_partials, sh, g_gemm_debug_flags,
                        q_tl_next(Q_TL_GEMM_TC)));
  return Q_OK;
}

extern "C" int q_gemm_tc(const void* d_x, const void* d_w_tc, float* d_partials, int M, int N, int K,
                         void* stream) {
  Q_CHECK_ARG(d_x && d_w_tc && d_partials, "q_gemm_tc: null pointer");
  Q_CHECK_ARG(((uintptr_t)d_x & 15) == 0 && ((uintptr_t)d_w_tc & 1023) == 0 && ((uintptr_t)d_partials & 3) == 0,
              "q_gemm_tc: x must be 16-byte aligned and the tiled weight 1024-byte aligned");
  Q_CHECK_ARG(K % 8 == 0, "q_gemm_tc: K must be a multiple of 8");
  q_gemm_plan_t p;
  int rc = q_gemm_tc_plan(M, N, K, &p);
  if (rc) return rc;
  return q_gemm_tc_launch(d_x, d_w_tc, d_partials, &p, stream);
}
