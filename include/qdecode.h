/*
 * qdecode.h - C ABI of libqdecode.so: the Qwen3 greedy-decode hot path as
 * hand-written sm_100a CUDA kernels.
 *
 * Conventions (all entry points):
 *   - return 0 on success, a negative q_status on error; q_last_error() gives
 *     the message of the calling thread's last failure. Nothing throws, aborts
 *     or traps.
 *   - every pointer named d_* is a DEVICE pointer borrowed from the caller (the
 *     caller owns it and keeps it alive until the stream work has finished).
 *     Outputs are caller-allocated so that addresses are stable under CUDA
 *     graph capture.
 *   - `stream` is a cudaStream_t passed as void*. No entry point allocates,
 *     synchronises or reads device values on the host (except where stated),
 *     so all of them may be captured in a CUDA graph.
 *   - bf16 tensors are row-major, innermost dimension contiguous.
 *
 * Each declaration cites the reference interface (jadenpxrk/starter, path
 * within that project) it replaces.
 */
#ifndef QDECODE_H
#define QDECODE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum q_status {
  Q_OK = 0,
  Q_ERR_ARG = -1,      /* bad shape / null pointer / unsupported size */
  Q_ERR_CUDA = -2,     /* a CUDA runtime call failed */
  Q_ERR_STATE = -3,    /* engine not fully bound */
  Q_ERR_DEVICE = -4    /* device status word reported a bounded wait ran out */
} q_status;

#define Q_PAGE_TOKENS 64   /* tokens per KV page (one attention key tile) */
#define Q_HEAD_DIM 128     /* the only supported head dimension */
#define Q_MAX_ROWS 64      /* most activation rows (batch x query tokens) per GEMM */

const char* q_last_error(void);
int q_version(void);

/* Programmatic dependent launch between consecutive kernels (default on).
 * Off = plain stream-ordered launches. */
int q_set_pdl(int enabled);

/* Tuning knobs (process-wide, host side only; no reference counterpart).
 *   "gemm_prefetch_kb": L2 prefetch window per GEMM CTA in KB (0 = off, default).
 *   "norm_in_gemm": 1 (default) = with up to 8 rows on one GPU, q_decode_step runs residual add +
 *       RMSNorm as the prologue of the projection that consumes them (q_gemm_splitk_addnorm).
 *   "attn_no_cluster": 1 = q_attention_decode merges 2..8 key splits through global memory and a
 *       ticket like it does above 8 splits, instead of inside a thread-block cluster (default 0).
 *   "peer_wait_iters": polling iterations (about 1 us each once the wait has backed off) after which
 *       q_add_rmsnorm_peers / q_argmax_merge_peers give up on a peer and set status word 3 (default 2^21).
 *   "peer_in_gemm": largest tensor-parallel world (default 2, 0 = never) for which
 *       q_decode_step_peers at 1-8 rows exchanges inside the projections: the O and down
 *       projections store their partials into every rank's receive area from their epilogue and
 *       the next projection's add+norm prologue polls them, instead of q_add_rmsnorm_peers as
 *       a kernel of its own (the step then has the five launches per layer of one GPU).
 *   "tc_min_rows": fewest rows for which q_decode_step uses the tcgen05 projections when the
 *       engine has the 128 x 64 tiling of its weights bound (default 9).
 *   "gemm_debug_flags": measurement aid, 4 = per-CTA time stamps for q_debug_gemm_trace, 8 = a
 *       projection with the add+norm prologue requests none of its weights before its dependency wait.
 *   "gemm_trace_launch": measurement aid, n >= 0 = only the n-th GEMM launch from now records
 *       its CTA trace (so one projection inside a captured step can be looked at), -1 off.
 *   "timeline": measurement aid, 1 = per-launch time stamps for q_debug_timeline.
 * Unknown names return Q_ERR_ARG. */
int q_set_option(const char* name, int value);

/* Measurement aid: with option "gemm_debug_flags" bit 4 set, every GEMM CTA records
 * {SM id, start, past the dependency wait, prologue done, first stage landed, loop end,
 * exit, prologue operands in registers} (ns, %globaltimer); this copies the records of the last recording launch to the
 * host (8 values per CTA). */
int q_debug_gemm_trace(unsigned long long* out, int n_ctas);
/* The same for the tcgen05 projection: {start, set-up done, producer past the dependency wait,
 * first stage landed, last MMA issued, last accumulator stored, exit, tiles of the CTA}. With
 * "gemm_debug_flags" bit 16 the kernel issues no MMA (copies only: the load pipeline alone). */
int q_debug_tc_trace(unsigned long long* out, int n_ctas);

/* Measurement aid: with option "timeline" = 1 (set before the launches, and before a graph
 * capture that should carry it), the kernels of q_decode_step's default path record, per
 * launch in launch order, {first CTA start, first CTA past its dependency wait, last warp
 * end, last CTA start} in %globaltimer ns. Copies up to max_records records (4 values each)
 * of the most recent execution, re-arms the records and returns the count (or a negative
 * q_status). At most 4096 launches are recorded after the option is set.
 * q_debug_timeline_kinds gives the kernel kind of each record: 1 stream-K projection,
 * 2 tcgen05 projection, 3 decode attention, 4 add+norm, 5 SwiGLU, 6 embedding + norm,
 * 7 logits + argmax, 8 add+norm over peer memory. */
int q_debug_timeline(unsigned long long* out, int max_records);
int q_debug_timeline_kinds(int32_t* out, int max_records);

/* Measurement aid: with option "timeline" on, CTA (0,0) of the decode-attention kernel stamps
 * {start, past the dependency wait, heads normed, tiles done, CTA merged, cluster merged, end, 0}
 * (ns); this copies the stamps of the last such launch (8 values). */
int q_debug_attn_trace(unsigned long long* out);

/* ---- split-K weight-streaming GEMM --------------------------------------
 * Replaces engine/kernels/skinny_gemm.py:100-109 (linear_partials) and the
 * split planning at :86-91 (split_count).
 *
 * P[slot][m][n] (fp32) holds partial sums of X[M,K] . W[N,K]^T. The work is
 * cut into units of 16 weight rows x 32 k; every CTA of the grid (a "worker")
 * takes one contiguous run of `units_per_worker` units, so a 16-row group is
 * covered by `count(group)` consecutive workers, and worker w writes slot
 * w - first_worker(group). A consumer sums slots 0..count-1 in order and
 * rounds once to bf16. q_gemm_plan gives the numbers a consumer needs; P always
 * has at least two slots. */
typedef struct q_gemm_plan_t {
  int32_t M, N, K;
  int32_t chunks_per_group;   /* K / 32 */
  int32_t groups;             /* ceil(N / 16) */
  int32_t units_per_worker;   /* u */
  int32_t workers;            /* CTAs that get work */
  int32_t slots;              /* max count(group); P needs slots*M*N floats */
  int32_t grid, block;        /* launch shape used */
  int32_t group_rows;         /* weight rows per group: 16 (q_gemm_plan) or 128 (q_gemm_tc_plan) */
} q_gemm_plan_t;

int q_gemm_plan(int M, int N, int K, q_gemm_plan_t* plan);

/* Weight tiling, done once at load time (the reference packs at load time too:
 * engine/mlp.py:12-15, engine/qk_norm_rope.py:25-30). A row-major bf16 [N][K]
 * matrix (torch Linear layout) becomes q_packed_weight_bytes(N,K) bytes of 1 KB
 * units (16 rows x 32 k, group-major, rows past N zero) in the order the GEMM
 * streams them. q_unpack_weight is the inverse. Not capturable-sensitive: plain
 * kernels on `stream`. */
int64_t q_packed_weight_bytes(int N, int K);
int q_pack_weight(const void* d_rowmajor, void* d_tiled, int N, int K, void* stream);
int q_unpack_weight(const void* d_tiled, void* d_rowmajor, int N, int K, void* stream);

/* d_w_tiled is a weight in the tiled layout above. */
int q_gemm_splitk(const void* d_x, const void* d_w_tiled, float* d_partials,
                  int M, int N, int K, void* stream);

/* engine/kernels/decode_fused.py:140-158 (add_rms_norm) folded into the projection that
 * consumes it (engine/decode_step.py:50-59 calls them back to back): every CTA rebuilds
 * resid_out = bf16(resid_in + bf16(sum of d_prev slots)) and X = RMSNorm(resid_out) * gain
 * in shared memory and then streams its weights; d_resid_out (written once, must differ
 * from d_resid_in) is the new residual. 1..8 rows, K <= 3072. prev_plan NULL = d_prev is
 * one plain fp32 [M][K] buffer. */
int q_gemm_splitk_addnorm(const void* d_resid_in, const float* d_prev, const q_gemm_plan_t* prev_plan,
                          const void* d_gain, void* d_resid_out, const void* d_w_tiled,
                          float* d_partials, int M, int N, int K, float eps, void* stream);

/* engine/kernels/skinny_gemm.py:49-72,112-121 (linear_silu_mul): act[M][inter] (bf16) =
 * silu(x @ gate.T) * (x @ up.T) in ONE launch, no partials. d_w_tiled is the tiled layout of
 * the [2*inter, K] matrix whose rows interleave the two projections in blocks of 8: rows
 * 16i..16i+7 = gate rows 8i..8i+7, rows 16i+8..16i+15 = up rows 8i..8i+7 (so one tensor-core
 * tile holds a gate row and its up row in the same thread). Every CTA owns whole 16-row
 * groups. inter must be a multiple of 8. */
int q_gemm_swiglu(const void* d_x, const void* d_w_tiled, void* d_act, int M, int inter, int K,
                  void* stream);

/* The same with q_gemm_splitk_addnorm's prologue in front (1..8 rows, K <= 3072). */
int q_gemm_swiglu_addnorm(const void* d_resid_in, const float* d_prev, const q_gemm_plan_t* prev_plan,
                          const void* d_gain, void* d_resid_out, const void* d_w_tiled, void* d_act,
                          int M, int inter, int K, float eps, void* stream);

/* Sums the slots of a plan into one fp32 [M,N] buffer (no rounding). Used
 * before a tensor-parallel all-reduce, which must add fp32 partials. */
int q_reduce_partials(const float* d_partials, const q_gemm_plan_t* plan,
                      float* d_out, void* stream);

/* ---- the same projection on the tcgen05 tensor cores, for 9 rows and more ----------
 * Replaces engine/kernels/skinny_gemm.py:28-46 at BLOCK_M 32 / 64 and the cuBLAS calls of
 * the prompt pass (engine/prefill.py:40-52). The weight is tiled a second way: 128 rows x
 * 64 k tiles of 16 KB, row-block-major then k, each tile stored as the K-major shared-memory
 * image with 128-byte swizzle that tcgen05.mma reads (rows past N and k past K zero).
 * q_gemm_tc writes the same kind of partial slots as q_gemm_splitk, with a "group" of 128
 * weight rows: plan.group_rows = 128, chunks_per_group = k tiles, units_per_worker = tiles
 * per CTA. More than 256 rows run as row chunks of 256 inside the same launch, tiles in
 * (row chunk, weight block, k tile) order (one weight pass per chunk); the plan's groups
 * are then the (row chunk, weight block) pairs, groups = ceil(M/256) * ceil(N/128), and the
 * slot count of element (m, n) is that of group (m / 256) * ceil(N/128) + n / 128. X is
 * row-major [M][K], 16-byte aligned; d_w_tc 1024-byte aligned. */
int64_t q_packed_weight_bytes_tc(int N, int K);
int q_pack_weight_tc(const void* d_rowmajor, void* d_tiled, int N, int K, void* stream);
int q_unpack_weight_tc(const void* d_tiled, void* d_rowmajor, int N, int K, void* stream);
int q_gemm_tc_plan(int M, int N, int K, q_gemm_plan_t* plan);
int q_gemm_tc(const void* d_x, const void* d_w_tc, float* d_partials, int M, int N, int K,
              void* stream);

/* No counterpart in the reference. d_out[M][N] (fp32) = X . W^T, i.e. q_gemm_splitk
 * followed by q_reduce_partials, for callers that may not allocate device memory
 * (their own pool owns all of it, their runtime forbids allocator calls, or they
 * run where cudaMalloc would stall the device): the partial sums live in a static
 * array inside the library instead of a caller buffer. Limits and rules:
 *   - slots * M * N must not exceed q_static_scratch_floats() (327,680 floats,
 *     1.25 MB per GPU, held from library load to process exit); larger shapes
 *     return Q_ERR_ARG and belong to q_gemm_splitk with a caller buffer;
 *   - the first call on each device looks up the array's address (with that
 *     device current) and caches it: make that first call outside any stream
 *     capture;
 *   - all calls share the one array, which keeps the previous call's partials:
 *     calls that overlap on the GPU (different streams) race; order them;
 *   - it calls no allocator of any kind. */
int64_t q_static_scratch_floats(void);
int q_linear_f32_static(const void* d_x, const void* d_w_tiled, float* d_out,
                        int M, int N, int K, void* stream);

/* ---- fused element-wise consumers ----------------------------------------*/

/* engine/kernels/rmsnorm.py:39-62 (rms_norm): out = bf16(x*rsqrt(mean x^2+eps))*w */
int q_rmsnorm(const void* d_x, const void* d_gain, void* d_out,
              int rows, int cols, float eps, void* stream);

/* engine/decode_step.py:38-39: embedding gather + first RMSNorm. d_embed is the
 * [vocab][cols] table in the TILED weight layout (it is the tied lm_head).
 * d_tokens int64[rows]; writes x (the residual stream) and normed. */
int q_embed_rmsnorm(const int64_t* d_tokens, const void* d_embed, const void* d_gain,
                    void* d_x, void* d_normed, int rows, int cols, int vocab,
                    float eps, void* stream);

/* engine/kernels/decode_fused.py:140-158 (add_rms_norm). The branch is either
 * split-K partials described by `plan` (plan != NULL) or one fp32 [rows,cols]
 * buffer (plan == NULL, e.g. after an all-reduce). total = bf16(x + bf16(sum)),
 * normed = bf16(total*rsqrt(mean total^2 + eps)) * gain. d_x_in may equal
 * d_total_out. */
int q_add_rmsnorm(const void* d_x_in, const float* d_branch, const q_gemm_plan_t* plan,
                  const void* d_gain, void* d_total_out, void* d_normed_out,
                  int rows, int cols, float eps, void* stream);

/* engine/kernels/skinny_gemm.py:66-72 epilogue / decode_fused.py:161-169
 * (silu_mul) on split-K partials of the packed gate|up projection
 * (columns [0,I) gate, [I,2I) up): out = bf16(bf16(silu(bf16 g)) * bf16 u). */
int q_swiglu(const float* d_branch, const q_gemm_plan_t* plan, void* d_out,
             int rows, int inter, void* stream);
/* The same on partials whose columns are in q_gemm_swiglu's weight order (blocks of 8 gate
 * columns followed by their 8 up columns): what the step runs above 8 rows on the stream-K
 * kernel. inter must be a multiple of 8. */
int q_swiglu_interleaved(const float* d_branch, const q_gemm_plan_t* plan, void* d_out,
                         int rows, int inter, void* stream);

/* Paged KV cache of one layer: pool[page][kv_head][64 tokens][128] bf16, the
 * 16-byte chunks of each token row XOR-swizzled by (token & 7) so that a page
 * tile can be bulk-copied to shared memory and read conflict-free.
 * block_table int32 [batch][pages_per_seq] maps a sequence's tile to a page. */
typedef struct q_kv_layout_t {
  void* d_kpool;
  void* d_vpool;
  const int32_t* d_block_table;
  int32_t pages_per_seq;
  int32_t n_kv_heads;        /* heads held in this pool (local heads under TP) */
} q_kv_layout_t;

/* engine/kernels/decode_fused.py:172-210 (qkv_norm_rope_cache), generalised to
 * T consecutive query tokens per sequence (row m = b*T + t sits at absolute
 * position *d_pos + t). Consumes the packed [q|k|v] projection partials, does
 * per-head RMSNorm + RoPE, writes Q [rows][n_q][128] and the K,V rows into
 * their page slots. cos/sin are bf16 [capacity][128] tables. */
int q_qkv_norm_rope_cache(const float* d_branch, const q_gemm_plan_t* plan,
                          const void* d_q_gain, const void* d_k_gain,
                          const void* d_cos, const void* d_sin, const int32_t* d_pos,
                          void* d_q_out, const q_kv_layout_t* kv,
                          int batch, int T, int n_q_heads, float eps, void* stream);

/* Scatters already-rotated K and V rows [batch][n_kv][len][128] (bf16) into the
 * pages at positions start..start+len-1. Host-side helper for prefill
 * (engine/kernels/prefill.py:19-63 writes cache[:, :, :T] the same way). */
int q_kv_scatter(const void* d_k, const void* d_v, const q_kv_layout_t* kv,
                 int batch, int len, int start, void* stream);

/* ---- attention -------------------------------------------------------------
 * engine/kernels/small_query_attention.py:113-158 (SmallQueryAttention.run) and
 * engine/flash_decode.py:78-83, generalised to T in 1..(32/G) query tokens per
 * sequence with a causal limit inside the query block: row (b,t,head) sees keys
 * [0, *d_pos + t + 1). Split-KV partials go to caller scratch, a second kernel
 * merges them and rounds once to bf16. out is [batch*T][n_q*128].
 *   d_scratch_o: float[batch*n_kv][splits][T*G][128]
 *   d_scratch_ml: float[batch*n_kv][splits][T*G][2]
 * q_attention_splits returns the split count to size those for a capacity. */
int q_attention_splits(int batch, int n_kv_heads, int capacity);

int q_attention(const void* d_q, const q_kv_layout_t* kv, const int32_t* d_pos,
                float* d_scratch_o, float* d_scratch_ml, void* d_out,
                int batch, int T, int n_q_heads, int splits, float scale,
                void* stream);

/* Causal attention over a whole prompt block of T tokens per sequence (the prompt pass;
 * engine/prefill.py:45-52 calls the library's scaled-dot-product attention there). d_q is
 * [batch*T][n_q][128] bf16 (normed, rotated); the keys and values are read from the pages,
 * which must already hold positions *d_pos .. *d_pos+T-1 of every sequence; row (b,t,head)
 * sees keys [0, *d_pos + t + 1). No split scratch: one CTA per (sequence, kv head, block of
 * 128/G tokens). G = n_q_heads / n_kv_heads must be 1, 2, 4 or 8. out is [batch*T][n_q*128]. */
int q_attention_prefill(const void* d_q, const q_kv_layout_t* kv, const int32_t* d_pos,
                        void* d_out, int batch, int T, int n_q_heads, float scale,
                        void* stream);

/* The three kernels above for the single-token decode step in ONE launch:
 * engine/kernels/decode_fused.py:172-210 (head norm + RoPE + K/V write into the page
 * slot *d_pos) + engine/kernels/small_query_attention.py:113-158 (split-KV attention and
 * merge). Consumes the packed [q|k|v] projection partials directly. d_tickets:
 * uint32[batch*n_kv], zeroed once by the caller (the last split to finish merges and
 * resets its ticket). Output [batch][n_q*128]. */
int q_attention_decode(const float* d_qkv_partials, const q_gemm_plan_t* plan,
                       const void* d_q_gain, const void* d_k_gain,
                       const void* d_cos, const void* d_sin, const int32_t* d_pos,
                       const q_kv_layout_t* kv, float* d_scratch_o, float* d_scratch_ml,
                       uint32_t* d_tickets, void* d_out, int batch, int n_q_heads,
                       int splits, float scale, float eps, void* stream);

/* ---- lm_head + argmax -------------------------------------------------------
 * engine/decode_step.py:60 (F.linear on lm_head) + engine/decode.py:106-107
 * (argmax, position += 1). Consumes the lm_head GEMM partials; writes bf16
 * logits [rows][vocab] if d_logits != NULL; picks per row the largest bf16
 * logit, lowest index on ties. d_val/d_idx get the per-row winner (idx +
 * vocab_offset, for vocab-sharded tensor parallelism); if d_tokens != NULL the
 * winner is also stored there as int64 and, if d_pos != NULL, *d_pos += pos_inc.
 * d_block_scratch: at least q_argmax_scratch_bytes(rows, vocab) bytes, zeroed
 * once by the caller before first use. */
int64_t q_argmax_scratch_bytes(int rows, int vocab);

int q_logits_argmax(const float* d_branch, const q_gemm_plan_t* plan,
                    void* d_logits, float* d_val, int32_t* d_idx,
                    int64_t* d_tokens, int32_t* d_pos, int pos_inc,
                    void* d_block_scratch, int rows, int vocab, int vocab_offset,
                    void* stream);

/* Final pick over tensor-parallel shards: val/idx are [shards][rows]; lowest
 * global index wins ties. Writes tokens and bumps *d_pos like above. */
int q_argmax_merge(const float* d_val, const int32_t* d_idx, int shards, int rows,
                   int64_t* d_tokens, int32_t* d_pos, int pos_inc, void* stream);

/* ---- whole decode step ------------------------------------------------------
 * engine/decode_step.py:33-60 (fused_decode_forward) + engine/decode.py:97-108
 * (DecodeState.step). The engine object only stores borrowed pointers and
 * launch plans; it owns no device memory. */
typedef struct q_config_t {
  int32_t hidden, inter, n_layers, n_q_heads, n_kv_heads, vocab;
  /* sizes above are the LOCAL shard sizes under tensor parallelism, except
   * hidden. vocab_offset = first vocabulary row of the local lm_head shard. */
  int32_t vocab_offset;
  int32_t full_vocab;        /* rows of the (replicated) embedding table */
  int32_t tp_size;           /* 1 = single GPU */
  int32_t max_rows;          /* batch * T upper bound, <= Q_MAX_ROWS */
  float rms_eps;
  float attn_scale;
} q_config_t;

typedef struct q_layer_weights_t {
  /* the four matrices are in the tiled layout of q_pack_weight */
  const void* wqkv;     /* [(n_q+2*n_kv)*128][hidden]  q rows | k rows | v rows */
  const void* wo;       /* [hidden][n_q*128] */
  const void* wgu;      /* [2*inter][hidden]  gate rows | up rows */
  const void* wdown;    /* [hidden][inter] */
  const void* ln_in;    /* [hidden] */
  const void* ln_post;  /* [hidden] */
  const void* q_gain;   /* [128] */
  const void* k_gain;   /* [128] */
  void* kpool;
  void* vpool;
  /* optional: the four matrices in q_pack_weight_tc's tiling (wgu_tc = [gate rows | up rows],
   * not interleaved). All four set = steps with tc_min_rows rows or more use q_gemm_tc. */
  const void* wqkv_tc;
  const void* wo_tc;
  const void* wgu_tc;
  const void* wdown_tc;
} q_layer_weights_t;

typedef struct q_state_t {
  const void* embed;        /* [full_vocab][hidden], tiled layout */
  const void* lm_head;      /* [vocab][hidden] tiled (local shard; == embed when tied, tp 1) */
  const void* ln_final;     /* [hidden] */
  const void* cos;          /* [capacity][128] bf16 */
  const void* sin;
  int64_t* tokens;          /* [batch] current token per sequence */
  int32_t* pos;             /* [1] position of the current token */
  const int32_t* block_table;
  int32_t pages_per_seq;
  int32_t batch;
  int32_t attn_splits;
  int32_t q_tokens;         /* query tokens per sequence T (0 or 1 = the plain decode step); rows =
                               batch * T: every row buffer below is sized for that many rows, tokens
                               holds batch * T candidate ids, row b*T + t sits at position *pos + t */
  /* scratch, all caller-allocated */
  void* x;                  /* bf16 [rows][hidden] residual stream */
  void* normed;             /* bf16 [rows][hidden] */
  void* q;                  /* bf16 [rows][n_q*128] */
  void* attended;           /* bf16 [rows][n_q*128] */
  void* act;                /* bf16 [rows][inter] */
  float* partials;          /* q_engine_partial_floats() floats */
  float* reduced;           /* fp32 [rows][hidden] (tensor parallel only, else NULL) */
  float* attn_o;            /* see q_attention */
  float* attn_ml;
  uint32_t* attn_tickets;   /* uint32[batch*n_kv], zeroed once (q_attention_decode) */
  void* logits;             /* bf16 [rows][vocab] or NULL */
  float* arg_val;           /* [rows] */
  int32_t* arg_idx;         /* [rows] */
  void* arg_scratch;        /* q_argmax_scratch_bytes() bytes, zeroed once */
  const void* lm_head_tc;   /* lm_head in q_pack_weight_tc's tiling, or NULL */
  int32_t* status_out;      /* int32[4] or NULL: the step's last kernel copies the four status
                               words of q_device_status here, so the host can read them with the
                               tokens instead of synchronising */
} q_state_t;

/* Tensor parallel over peer memory (no reference counterpart: the reference is single-GPU).
 * Every rank owns a receive area the other ranks can write (CUDA IPC / symmetric memory;
 * q_engine_peer_floats() floats: room for [2 halves][world][2 slots][rows][hidden] pairs of
 * the in-projection exchange, of which q_add_rmsnorm_peers uses [2 halves][world][rows][hidden] pairs {fp32 sum, call
 * counter}, 8 bytes each, the halves used by alternate calls) and a flag region (q_peer_flag_bytes() bytes) of arrival words and the
 * token-exchange pairs. partials[r] / flags[r] are rank r's receive area and flag region as
 * mapped into THIS process (entry `rank` is this rank's own); both are zeroed once before
 * the first step together with the counter words. */
#define Q_MAX_PEERS 8
typedef struct q_peers_t {
  int32_t rank, world;
  float* partials[Q_MAX_PEERS];
  uint32_t* flags[Q_MAX_PEERS];
  uint32_t* epoch;          /* uint32[4] of this rank, ordinary device memory, zeroed once: call
                               counter and CTA ticket of the add+norm exchange, call counter of the
                               token exchange */
} q_peers_t;

/* Bytes of the region flags[r] points to (zeroed once before the first step): 512 bytes of
 * arrival words (uint32 [p] for q_add_rmsnorm_peers, [64 + p] for q_argmax_merge_peers), then
 * the (value, index) pairs of the token exchange, [parity][shard][row]. */
int64_t q_peer_flag_bytes(void);

/* engine/kernels/decode_fused.py:140-158 with the cross-rank sum folded in: ONE kernel that
 * (1) adds this rank's split-K slots (d_own_branch: ordinary device memory, described by
 * `plan`; plan NULL = one fp32 [rows][cols] buffer) and stores every sum, paired with this
 * rank's call counter in one 8-byte store, into every peer's receive area (plain peer stores,
 * no fence and no separate flag: a pair that carries this call's counter HAS arrived),
 * (2) polls (bounded) its OWN receive area for the peers' pairs, (3) adds all ranks' sums in
 * rank order in fp32, rounds the total once, adds the residual and normalises like
 * q_add_rmsnorm. It
 * replaces q_reduce_partials + an all-reduce + q_add_rmsnorm. All ranks must make the same
 * sequence of calls. A wait that runs out sets q_device_status word 3. One CTA per row.
 * rows <= Q_MAX_ROWS, cols a multiple of 4 up to 4096. */
int q_add_rmsnorm_peers(const void* d_x_in, const q_peers_t* peers, const float* d_own_branch,
                        const q_gemm_plan_t* plan, const void* d_gain, void* d_total_out,
                        void* d_normed_out, int rows, int cols, float eps, void* stream);

/* The same exchange INSIDE the projections, for 1..8 rows (no reference counterpart). The
 * projection BEFORE an add+norm (O, down) runs as q_gemm_push: instead of writing partial
 * slots it stores every partial, paired with the call counter, into the receive area of every
 * rank - [half][rank][2 slots][M][N] pairs of 8 bytes, its own rank's too. The projection
 * AFTER the add+norm runs as q_gemm_splitk_addnorm_peers / q_gemm_swiglu_addnorm_peers:
 * q_gemm_splitk_addnorm / q_gemm_swiglu_addnorm whose prologue polls (bounded by option
 * "peer_wait_iters") the own receive area for all ranks' partials of the pushing projection
 * (prev_plan = that projection's plan: which slots exist), adds them in (rank, slot) order
 * and moves the call counter on. A wait that runs out sets q_device_status word 1 to 4. All
 * ranks make the same sequence of calls; the counter words are shared with
 * q_add_rmsnorm_peers (peers->epoch). plan / prev_plan: a q_gemm_plan of 1..8 rows with at
 * most two slots; K of the polling projection a multiple of 4 up to 3072. */
int q_gemm_push(const void* d_x, const void* d_w_tiled, const q_gemm_plan_t* plan,
                const q_peers_t* peers, void* stream);
int q_gemm_splitk_addnorm_peers(const void* d_resid_in, const q_peers_t* peers,
                                const q_gemm_plan_t* prev_plan, const void* d_gain,
                                void* d_resid_out, const void* d_w_tiled, float* d_partials,
                                int M, int N, int K, float eps, void* stream);
int q_gemm_swiglu_addnorm_peers(const void* d_resid_in, const q_peers_t* peers,
                                const q_gemm_plan_t* prev_plan, const void* d_gain,
                                void* d_resid_out, const void* d_w_tiled, void* d_act,
                                int M, int inter, int K, float eps, void* stream);

/* engine/decode.py:106-107 (argmax, position += 1) over vocabulary shards held by different
 * ranks, without a collective library call: every rank stores its per-row (value, index) pair
 * (d_val / d_idx, as q_logits_argmax leaves them) into every rank's exchange area with plain
 * peer stores, signals, waits (bounded, status word 3) for the others and picks the largest
 * value with the lowest index; tokens are written and *d_pos += pos_inc on every rank. */
int q_argmax_merge_peers(const float* d_val, const int32_t* d_idx, const q_peers_t* peers, int rows,
                         int64_t* d_tokens, int32_t* d_pos, int pos_inc, void* stream);

typedef struct q_engine q_engine;

int q_create(const q_config_t* cfg, q_engine** out);
int q_bind_layer(q_engine* e, int layer, const q_layer_weights_t* w);
int q_bind_state(q_engine* e, const q_state_t* s);
int64_t q_engine_partial_floats(const q_engine* e, int rows);
void q_destroy(q_engine* e);
/* Tensor parallel over peer memory: floats of the peer-readable partial buffer for `rows`,
 * and the binding (after q_bind_state). With peers bound, q_decode_step_peers runs the whole
 * sharded step - embed .. lm_head shard .. local argmax .. q_argmax_merge_peers - with
 * q_add_rmsnorm_peers in place of the two all-reduces per layer (or, see option
 * "peer_in_gemm", the same exchange inside the projections). No collective library call
 * is left in the step. q_bind_peers(e, NULL) unbinds; q_bind_state unbinds too. */
int64_t q_engine_peer_floats(const q_engine* e, int rows);
int q_bind_peers(q_engine* e, const q_peers_t* peers);
int q_decode_step_peers(q_engine* e, void* stream);

/* One full step for T=1 on a single GPU: embed .. argmax, tokens and pos updated:
 * 2 + 5 per layer + 1 kernels up to 8 rows (add+norm and SwiGLU folded into the projections),
 * 1 + 8 per layer + 2 above, all with programmatic dependent launch. */
int q_decode_step(q_engine* e, void* stream);

/* The same step in pieces, for tensor parallelism: the caller all-reduces
 * state.reduced (fp32 [rows][hidden]) between the pieces.
 *   q_step_begin:      embed + first norm
 *   q_step_attn:       QKV .. O-proj; leaves the local fp32 sum in `reduced`
 *   q_step_post_attn:  add+norm from `reduced`, gate/up, SwiGLU, down -> `reduced`
 *   q_step_post_mlp:   add+norm from `reduced` with the next gain
 *   q_step_head:       lm_head shard + local argmax into arg_val/arg_idx */
int q_step_begin(q_engine* e, void* stream);
int q_step_attn(q_engine* e, int layer, void* stream);
int q_step_post_attn(q_engine* e, int layer, void* stream);
int q_step_post_mlp(q_engine* e, int layer, void* stream);
int q_step_head(q_engine* e, void* stream);
/* ... and after the caller has all-gathered (arg_val, arg_idx) into [tp_size][rows] buffers:
 * the pick over the shards (q_argmax_merge) into state.tokens, position += 1. */
int q_step_merge(q_engine* e, const float* d_val, const int32_t* d_idx, void* stream);

/* The exact-verification step (the idea recorded at AGENTS.md:93-95 of the reference): with
 * state.q_tokens = T >= 1, runs T candidate tokens per sequence through all layers in one
 * pass over the weights - rows = batch * T through the same projections, q_qkv_norm_rope_cache
 * and q_attention with T tokens per sequence - and leaves, for every row, the greedy successor
 * of that row's prefix in state.arg_idx (and the logits in state.logits if set). Tokens and
 * position are NOT advanced: the caller accepts the longest prefix whose candidates equal the
 * successors before them, then sets state.tokens / *pos. Single GPU. */
int q_verify_step(q_engine* e, void* stream);

/* Reads the library's device status words of the current device (synchronises the device;
 * not capturable). A non-zero word means a bounded wait inside a kernel ran out and the
 * results since then are not to be trusted: out[0] attention (1 producer, 2 consumer),
 * out[1] stream-K GEMM ring (1), out[2] tcgen05 GEMM (1 producer, 2 MMA issuer, 3 epilogue,
 * 4 drain), out[3] tensor parallel over peer memory (1 = a peer's arrival word never came).
 * The words are sticky; q_clear_status zeroes them (synchronises too). */
int q_device_status(int32_t out[4]);
int q_clear_status(void);

#ifdef __cplusplus
}
#endif
#endif /* QDECODE_H */
