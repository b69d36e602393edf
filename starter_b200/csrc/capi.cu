// Engine object and step orchestration behind the C ABI. The engine stores
// borrowed device pointers and launch plans only; it owns no device memory and
// every step function just enqueues kernels on the caller's stream, so a whole
// step can be captured in one CUDA graph
// (reference: engine/decode_step.py:33-60, engine/decode.py:97-108).
#include <stdarg.h>
#include <string.h>
#include <new>
#include <vector>
#include "common.cuh"

static thread_local char g_err[512] = "";
static bool g_pdl = true;

void q_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
bool q_pdl_enabled() { return g_pdl; }

int q_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    // No usable device (e.g. a CPU-only host asking for a plan): plan for a B200.
    cudaGetLastError();
    return 148;
  }
  if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 148;
  }
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

int g_gemm_prefetch_kb = 0;
int g_gemm_debug_flags = 0;
int g_gemm_trace_launch = -1;    // measurement aid: the one GEMM launch that records its CTA trace
int g_gemm_launches = 0;
int g_attn_no_cluster = 0;        // 1 = decode attention merges its splits through global memory
// Largest tensor-parallel world whose 1-8 row step exchanges inside the projections (0 = never).
// Every CTA of the polling projection reads all ranks' pairs, so the cost grows with the world:
// measured at batch 1 it wins at 2 ranks (1.73 against 1.79 ms) and loses at 4 (1.71 against 1.61).
static int g_peer_in_gemm = 2;
static int g_norm_in_gemm = 1;   // 1 = residual add + RMSNorm as the prologue of the next projection
static int g_tc_min_rows = 9;    // fewest rows that take the tcgen05 projections (when their tiling is bound)
int g_peer_wait_iters = 1 << 21; // polling limit of the waits for a tensor-parallel peer

// Launch timeline (measurement aid): Q_TL_SLOTS records of 4 stamps, handed out in launch order.
#define Q_TL_SLOTS 4096
static __device__ unsigned long long g_timeline[Q_TL_SLOTS * 4];
static int g_tl_on = 0, g_tl_used = 0;
static int g_tl_kind[Q_TL_SLOTS];
static unsigned long long* g_tl_base = nullptr;

static int tl_reset() {
  static unsigned long long init[Q_TL_SLOTS * 4];
  for (int i = 0; i < Q_TL_SLOTS; ++i) {
    init[4 * i] = init[4 * i + 1] = ~0ull;
    init[4 * i + 2] = init[4 * i + 3] = 0ull;
  }
  return cudaMemcpyToSymbol(g_timeline, init, sizeof(init)) == cudaSuccess ? 0 : -1;
}

unsigned long long* q_tl_next(int kind) {
  if (!g_tl_on || g_tl_base == nullptr || g_tl_used >= Q_TL_SLOTS) return nullptr;
  g_tl_kind[g_tl_used] = kind;
  return g_tl_base + 4 * (g_tl_used++);
}

extern "C" int q_debug_timeline_kinds(int32_t* out, int max_records) {
  Q_CHECK_ARG(out && max_records >= 1, "q_debug_timeline_kinds: bad argument");
  const int n = g_tl_used < max_records ? g_tl_used : max_records;
  for (int i = 0; i < n; ++i) out[i] = g_tl_kind[i];
  return n;
}

extern "C" int q_debug_timeline(unsigned long long* out, int max_records) {
  Q_CHECK_ARG(out && max_records >= 1, "q_debug_timeline: bad argument");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  const int n = g_tl_used < max_records ? g_tl_used : max_records;
  if (n > 0) Q_CHECK_CUDA(cudaMemcpyFromSymbol(out, g_timeline, sizeof(unsigned long long) * 4 * n));
  if (tl_reset()) { q_set_error("q_debug_timeline: reset failed"); return Q_ERR_CUDA; }
  return n;
}

extern "C" int q_set_option(const char* name, int value) {
  Q_CHECK_ARG(name != nullptr, "q_set_option: null name");
  if (strcmp(name, "timeline") == 0) {
    g_tl_on = value != 0;
    g_tl_used = 0;
    if (g_tl_on) {
      void* p = nullptr;
      Q_CHECK_CUDA(cudaGetSymbolAddress(&p, g_timeline));
      g_tl_base = (unsigned long long*)p;
      if (tl_reset()) { q_set_error("q_set_option: timeline reset failed"); return Q_ERR_CUDA; }
    }
    return Q_OK;
  }
  if (strcmp(name, "gemm_prefetch_kb") == 0) {
    Q_CHECK_ARG(value >= 0 && value <= 8192, "q_set_option: gemm_prefetch_kb outside 0..8192");
    g_gemm_prefetch_kb = value;
    return Q_OK;
  }
  if (strcmp(name, "peer_in_gemm") == 0) {
    Q_CHECK_ARG(value >= 0 && value <= Q_MAX_PEERS, "q_set_option: peer_in_gemm outside 0..%d", Q_MAX_PEERS);
    g_peer_in_gemm = value;
    return Q_OK;
  }
  if (strcmp(name, "norm_in_gemm") == 0) {
    g_norm_in_gemm = value != 0;
    return Q_OK;
  }
  if (strcmp(name, "tc_min_rows") == 0) {
    Q_CHECK_ARG(value >= 1, "q_set_option: tc_min_rows must be >= 1");
    g_tc_min_rows = value;
    return Q_OK;
  }
  if (strcmp(name, "peer_wait_iters") == 0) {
    Q_CHECK_ARG(value >= 1, "q_set_option: peer_wait_iters must be >= 1");
    g_peer_wait_iters = value;
    return Q_OK;
  }
  if (strcmp(name, "attn_no_cluster") == 0) {
    g_attn_no_cluster = value != 0;
    return Q_OK;
  }
  if (strcmp(name, "gemm_trace_launch") == 0) {
    g_gemm_trace_launch = value;
    g_gemm_launches = 0;
    return Q_OK;
  }
  if (strcmp(name, "gemm_debug_flags") == 0) {
    g_gemm_debug_flags = value;     // measurement aid: 4 = per-CTA time stamps (q_debug_gemm_trace)
    return Q_OK;
  }
  q_set_error("q_set_option: unknown option '%s'", name);
  return Q_ERR_ARG;
}

// Every kernel file keeps its own status word (a bounded wait that ran out records a code
// there); these give the words' device addresses on the current device.
int* q_attn_status_addr();
int* q_gemm_status_addr();
int* q_tc_status_addr();
int* q_peer_status_addr();

static int status_addrs(int* addr[4]) {
  addr[0] = q_attn_status_addr();   // attention: 1 producer wait ran out, 2 consumer wait ran out
  addr[1] = q_gemm_status_addr();   // stream-K GEMM: 1 ring wait ran out
  addr[2] = q_tc_status_addr();     // tcgen05 GEMM: 1 producer, 2 MMA issuer, 3 epilogue wait ran out
  addr[3] = q_peer_status_addr();   // tensor parallel over peer memory: 1 = a peer's arrival word never came
  for (int i = 0; i < 4; ++i)
    if (!addr[i]) { q_set_error("could not locate the device status words"); return Q_ERR_CUDA; }
  return Q_OK;
}

extern "C" int q_device_status(int32_t out[4]) {
  Q_CHECK_ARG(out != nullptr, "q_device_status: null pointer");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  int* addr[4];
  int rc = status_addrs(addr);
  if (rc) return rc;
  for (int i = 0; i < 4; ++i)
    Q_CHECK_CUDA(cudaMemcpy(&out[i], addr[i], sizeof(int32_t), cudaMemcpyDeviceToHost));
  return Q_OK;
}

extern "C" int q_clear_status(void) {
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  int* addr[4];
  int rc = status_addrs(addr);
  if (rc) return rc;
  for (int i = 0; i < 4; ++i) Q_CHECK_CUDA(cudaMemset(addr[i], 0, sizeof(int32_t)));
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  return Q_OK;
}

extern "C" const char* q_last_error(void) { return g_err; }
extern "C" int q_version(void) { return 100; }
extern "C" int q_set_pdl(int enabled) {
  g_pdl = enabled != 0;
  return Q_OK;
}

struct q_engine {
  q_config_t cfg;
  std::vector<q_layer_weights_t> layers;
  std::vector<bool> bound;
  q_state_t st;
  bool has_state;
  int rows;                 // batch * tokens per sequence
  int T;                    // query tokens per sequence of the bound state
  bool tc;                  // projections run on the tcgen05 kernel
  q_gemm_plan_t p_qkv, p_o, p_gu, p_down, p_head;
  bool has_peers;
  q_peers_t peers;
};

// Plans of the five projections for `rows` activation rows, on the stream-K kernel (16-row
// groups) or the tcgen05 kernel (128-row blocks).
static int make_plans(q_engine* e, int rows, bool tc) {
  const q_config_t& c = e->cfg;
  int (*plan)(int, int, int, q_gemm_plan_t*) = tc ? q_gemm_tc_plan : q_gemm_plan;
  int rc;
  if ((rc = plan(rows, (c.n_q_heads + 2 * c.n_kv_heads) * 128, c.hidden, &e->p_qkv))) return rc;
  if ((rc = plan(rows, c.hidden, c.n_q_heads * 128, &e->p_o))) return rc;
  if ((rc = plan(rows, 2 * c.inter, c.hidden, &e->p_gu))) return rc;
  if ((rc = plan(rows, c.hidden, c.inter, &e->p_down))) return rc;
  if ((rc = plan(rows, c.vocab, c.hidden, &e->p_head))) return rc;
  e->rows = rows;
  e->tc = tc;
  return Q_OK;
}

static long long plan_floats(const q_gemm_plan_t& p) { return (long long)p.slots * p.M * p.N; }

static bool tc_weights_bound(const q_engine* e, const q_state_t* s) {
  if (s && !s->lm_head_tc) return false;
  for (size_t i = 0; i < e->layers.size(); ++i) {
    const q_layer_weights_t& w = e->layers[i];
    if (!e->bound[i] || !w.wqkv_tc || !w.wo_tc || !w.wgu_tc || !w.wdown_tc) return false;
  }
  return true;
}

extern "C" int q_create(const q_config_t* cfg, q_engine** out) {
  Q_CHECK_ARG(cfg && out, "q_create: null pointer");
  Q_CHECK_ARG(cfg->hidden >= 32 && cfg->hidden % 32 == 0, "q_create: hidden must be a multiple of 32");
  Q_CHECK_ARG(cfg->inter >= 32 && cfg->inter % 32 == 0, "q_create: inter must be a multiple of 32");
  Q_CHECK_ARG(cfg->n_layers >= 1 && cfg->n_q_heads >= 1 && cfg->n_kv_heads >= 1 &&
                  cfg->n_q_heads % cfg->n_kv_heads == 0 && cfg->n_q_heads / cfg->n_kv_heads <= 32,
              "q_create: bad head counts");
  Q_CHECK_ARG(cfg->vocab >= 1 && cfg->full_vocab >= cfg->vocab && cfg->vocab_offset >= 0,
              "q_create: bad vocabulary sizes");
  Q_CHECK_ARG(cfg->tp_size >= 1, "q_create: tp_size must be >= 1");
  Q_CHECK_ARG(cfg->max_rows >= 1 && cfg->max_rows <= Q_MAX_ROWS, "q_create: max_rows outside 1..%d",
              Q_MAX_ROWS);
  q_engine* e = new (std::nothrow) q_engine();
  if (!e) { q_set_error("q_create: out of host memory"); return Q_ERR_ARG; }
  e->cfg = *cfg;
  e->layers.resize(cfg->n_layers);
  e->bound.assign(cfg->n_layers, false);
  memset(&e->st, 0, sizeof(e->st));
  e->has_state = false;
  e->has_peers = false;
  e->rows = 0;
  e->T = 1;
  e->tc = false;
  *out = e;
  return Q_OK;
}

extern "C" void q_destroy(q_engine* e) { delete e; }

extern "C" int q_bind_layer(q_engine* e, int layer, const q_layer_weights_t* w) {
  Q_CHECK_ARG(e && w, "q_bind_layer: null pointer");
  Q_CHECK_ARG(layer >= 0 && layer < e->cfg.n_layers, "q_bind_layer: layer %d out of range", layer);
  Q_CHECK_ARG(w->wqkv && w->wo && w->wgu && w->wdown && w->ln_in && w->ln_post && w->q_gain &&
                  w->k_gain && w->kpool && w->vpool,
              "q_bind_layer: layer %d has a null tensor", layer);
  const void* tiled[8] = {w->wqkv, w->wo, w->wgu, w->wdown, w->wqkv_tc, w->wo_tc, w->wgu_tc, w->wdown_tc};
  for (int i = 0; i < 8; ++i)
    Q_CHECK_ARG(((uintptr_t)tiled[i] & (i < 4 ? 15 : 1023)) == 0,
                "q_bind_layer: tiled weights must be 16-byte (128 x 64 tiling: 1024-byte) aligned");
  const void* vecs[6] = {w->ln_in, w->ln_post, w->q_gain, w->k_gain, w->kpool, w->vpool};
  for (int i = 0; i < 6; ++i)
    Q_CHECK_ARG(((uintptr_t)vecs[i] & 15) == 0, "q_bind_layer: gains and KV pools must be 16-byte aligned");
  e->layers[layer] = *w;
  e->bound[layer] = true;
  return Q_OK;
}

static long long max_plan_floats(const q_engine* e) {
  long long m = plan_floats(e->p_qkv);
  if (plan_floats(e->p_o) > m) m = plan_floats(e->p_o);
  if (plan_floats(e->p_gu) > m) m = plan_floats(e->p_gu);
  if (plan_floats(e->p_down) > m) m = plan_floats(e->p_down);
  if (plan_floats(e->p_head) > m) m = plan_floats(e->p_head);
  return ((m + 63) / 64) * 64;
}

static long long hidden_plan_floats(const q_engine* e) {
  const long long m = plan_floats(e->p_o) > plan_floats(e->p_down) ? plan_floats(e->p_o) : plan_floats(e->p_down);
  return ((m + 63) / 64) * 64;
}

extern "C" int64_t q_engine_partial_floats(const q_engine* e, int rows) {
  if (!e || rows < 1 || rows > Q_MAX_ROWS) return -1;
  // large enough for either kernel: [all projections | O / down partials when the consumer
  // is the prologue of the next projection]
  long long need = 0;
  for (int tc = 0; tc < 2; ++tc) {
    q_engine tmp = *e;
    if (make_plans(&tmp, rows, tc != 0)) return -1;
    const long long n = max_plan_floats(&tmp) + hidden_plan_floats(&tmp);
    if (n > need) need = n;
  }
  return need;
}

extern "C" int q_bind_state(q_engine* e, const q_state_t* s) {
  Q_CHECK_ARG(e && s, "q_bind_state: null pointer");
  const int T = s->q_tokens < 1 ? 1 : s->q_tokens;
  Q_CHECK_ARG(s->batch >= 1 && s->batch * T <= e->cfg.max_rows, "q_bind_state: batch %d x %d tokens outside 1..%d rows",
              s->batch, T, e->cfg.max_rows);
  Q_CHECK_ARG(s->embed && s->lm_head && s->ln_final && s->cos && s->sin && s->tokens && s->pos &&
                  s->block_table && s->x && s->normed && s->q && s->attended && s->act &&
                  s->partials && s->arg_val && s->arg_idx && s->arg_scratch,
              "q_bind_state: a required pointer is null");
  Q_CHECK_ARG(s->pages_per_seq >= 1, "q_bind_state: pages_per_seq must be >= 1");
  Q_CHECK_ARG(s->attn_splits >= 1 && s->attn_splits <= 32, "q_bind_state: attn_splits outside 1..32");
  Q_CHECK_ARG(s->attn_splits == 1 || (s->attn_o && s->attn_ml), "q_bind_state: attention scratch missing");
  Q_CHECK_ARG(e->cfg.tp_size == 1 || s->reduced, "q_bind_state: tensor parallel needs `reduced`");
  const int G = e->cfg.n_q_heads / e->cfg.n_kv_heads;
  Q_CHECK_ARG(T == 1 || T * G <= 32, "q_bind_state: %d query tokens x %d heads per kv head exceed 32 rows", T, G);
  const void* vec16[] = {s->embed, s->lm_head, s->ln_final, s->cos, s->sin, s->x, s->normed, s->q, s->attended,
                         s->act, s->partials, s->reduced, s->attn_o, s->attn_ml, s->logits};
  for (size_t i = 0; i < sizeof(vec16) / sizeof(vec16[0]); ++i)
    Q_CHECK_ARG(((uintptr_t)vec16[i] & 15) == 0, "q_bind_state: tensor %zu is not 16-byte aligned", i);
  Q_CHECK_ARG(((uintptr_t)s->lm_head_tc & 1023) == 0, "q_bind_state: lm_head_tc must be 1024-byte aligned");
  const bool tc = s->batch * T >= g_tc_min_rows && tc_weights_bound(e, s);
  int rc = make_plans(e, s->batch * T, tc);
  if (rc) return rc;
  e->st = *s;
  e->T = T;
  e->has_state = true;
  e->has_peers = false;
  return Q_OK;
}

static int ready(q_engine* e, const char* who) {
  if (!e) { q_set_error("%s: null engine", who); return Q_ERR_ARG; }
  if (!e->has_state) { q_set_error("%s: q_bind_state has not been called", who); return Q_ERR_STATE; }
  for (size_t i = 0; i < e->bound.size(); ++i)
    if (!e->bound[i]) { q_set_error("%s: layer %zu is not bound", who, i); return Q_ERR_STATE; }
  return Q_OK;
}

#define TRY(x) do { int _rc = (x); if (_rc) return _rc; } while (0)

static q_kv_layout_t kv_of(const q_engine* e, int layer) {
  q_kv_layout_t kv;
  kv.d_kpool = e->layers[layer].kpool;
  kv.d_vpool = e->layers[layer].vpool;
  kv.d_block_table = e->st.block_table;
  kv.pages_per_seq = e->st.pages_per_seq;
  kv.n_kv_heads = e->cfg.n_kv_heads;
  return kv;
}

// One projection on whichever kernel the bound plans are for.
static int project(const q_engine* e, const void* x, const void* w_units, const void* w_tc, float* out,
                   const q_gemm_plan_t& plan, void* stream) {
  if (e->tc) return q_gemm_tc_launch(x, w_tc, out, &plan, stream);
  return q_gemm_launch_planned(x, w_units, out, &plan, stream);
}

// Where the hidden-size projections (O, down) leave their partials. With the add+norm
// prologue the next projection reads them while it writes its own, so they live in the
// second buffer behind the first (q_engine_partial_floats sizes both).
static float* hidden_partials(const q_engine* e, bool second) {
  return second ? e->st.partials + max_plan_floats(e) : e->st.partials;
}

// Up to 8 rows on one GPU: residual add + RMSNorm run as the prologue of the projection
// that consumes them, the residual alternating between st.x and st.normed.
static bool norm_in_gemm(const q_engine* e) {
  return e->cfg.tp_size == 1 && !e->tc && e->T == 1 && e->rows <= 8 && e->cfg.hidden % 4 == 0 &&
         e->cfg.hidden <= 3072 && g_norm_in_gemm;
}

// Tensor parallel, up to 8 rows: the cross-rank sums are exchanged inside the projections.
static bool peer_exchange_in_gemm(const q_engine* e) {
  return e->cfg.tp_size > 1 && e->has_peers && !e->tc && e->T == 1 && e->rows <= 8 && e->cfg.hidden % 4 == 0 &&
         e->cfg.hidden <= 3072 && e->p_o.slots <= 2 && e->p_down.slots <= 2 && e->cfg.tp_size <= g_peer_in_gemm;
}

// attention .. O projection, from the QKV partials in st.partials. o_partials == nullptr: the O
// projection pushes its partials to the tensor-parallel peers instead (1-8 rows).
static int attn_after_qkv(q_engine* e, int layer, float* o_partials, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  const q_layer_weights_t& w = e->layers[layer];
  q_kv_layout_t kv = kv_of(e, layer);
  if (e->T == 1 && s.attn_tickets && c.n_q_heads / c.n_kv_heads <= 8) {
    // head norm + RoPE + K/V write + attention + split merge in one launch
    TRY(q_attention_decode(s.partials, &e->p_qkv, w.q_gain, w.k_gain, s.cos, s.sin, s.pos, &kv, s.attn_o,
                           s.attn_ml, s.attn_tickets, s.attended, s.batch, c.n_q_heads, s.attn_splits,
                           c.attn_scale, c.rms_eps, stream));
  } else {
    TRY(q_qkv_norm_rope_cache(s.partials, &e->p_qkv, w.q_gain, w.k_gain, s.cos, s.sin, s.pos, s.q, &kv,
                              s.batch, e->T, c.n_q_heads, c.rms_eps, stream));
    TRY(q_attention(s.q, &kv, s.pos, s.attn_o, s.attn_ml, s.attended, s.batch, e->T, c.n_q_heads,
                    s.attn_splits, c.attn_scale, stream));
  }
  if (!o_partials) return q_gemm_push(s.attended, w.wo, &e->p_o, &e->peers, stream);
  return project(e, s.attended, w.wo, w.wo_tc, o_partials, e->p_o, stream);
}

// QKV projection .. attention .. O projection (partials left in `o_partials`).
static int attn_block(q_engine* e, int layer, float* o_partials, void* stream) {
  const q_state_t& s = e->st;
  const q_layer_weights_t& w = e->layers[layer];
  TRY(project(e, s.normed, w.wqkv, w.wqkv_tc, s.partials, e->p_qkv, stream));
  return attn_after_qkv(e, layer, o_partials, stream);
}

// gate|up projection + SwiGLU, then the down projection into `down_partials`. The stream-K
// weight has its gate / up rows interleaved in blocks of 8 (SwiGLU in the projection's
// epilogue up to 8 rows; above, on the partials); the tcgen05 weight is plain [gate | up].
static int mlp_block(q_engine* e, int layer, float* down_partials, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  const q_layer_weights_t& w = e->layers[layer];
  if (e->tc) {
    TRY(q_gemm_tc_launch(s.normed, w.wgu_tc, s.partials, &e->p_gu, stream));
    TRY(q_swiglu_layout(s.partials, &e->p_gu, s.act, e->rows, c.inter, 0, stream));
  } else if (e->rows <= 8) {
    TRY(q_gemm_swiglu(s.normed, w.wgu, s.act, e->rows, c.inter, c.hidden, stream));
  } else {
    // Above 8 rows the mma.sync projection is bound by instruction issue, not by memory, and
    // whole groups per CTA (8 or 9 of them) cost more than the SwiGLU launch saves: stream-K
    // partials, then SwiGLU on the interleaved columns.
    TRY(q_gemm_launch_planned(s.normed, w.wgu, s.partials, &e->p_gu, stream));
    TRY(q_swiglu_layout(s.partials, &e->p_gu, s.act, e->rows, c.inter, 1, stream));
  }
  return project(e, s.act, w.wdown, w.wdown_tc, down_partials, e->p_down, stream);
}

static const void* next_gain(const q_engine* e, int layer) {
  return layer + 1 < e->cfg.n_layers ? e->layers[layer + 1].ln_in : e->st.ln_final;
}

static StatusTap status_tap(const q_engine* e) {
  StatusTap tap = {};
  if (e->st.status_out) {
    int* addr[4];
    if (status_addrs(addr) == Q_OK) {
      for (int i = 0; i < 4; ++i) tap.src[i] = addr[i];
      tap.out = e->st.status_out;
    }
  }
  return tap;
}

extern "C" int q_step_begin(q_engine* e, void* stream) {
  TRY(ready(e, "q_step_begin"));
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  return q_embed_rmsnorm(s.tokens, s.embed, e->layers[0].ln_in, s.x, s.normed, e->rows, c.hidden,
                         c.full_vocab, c.rms_eps, stream);
}

extern "C" int q_step_attn(q_engine* e, int layer, void* stream) {
  TRY(ready(e, "q_step_attn"));
  Q_CHECK_ARG(layer >= 0 && layer < e->cfg.n_layers, "q_step_attn: layer out of range");
  Q_CHECK_ARG(e->st.reduced, "q_step_attn: state.reduced is null");
  TRY(attn_block(e, layer, e->st.partials, stream));
  return q_reduce_partials(e->st.partials, &e->p_o, e->st.reduced, stream);
}

extern "C" int q_step_post_attn(q_engine* e, int layer, void* stream) {
  TRY(ready(e, "q_step_post_attn"));
  Q_CHECK_ARG(layer >= 0 && layer < e->cfg.n_layers, "q_step_post_attn: layer out of range");
  Q_CHECK_ARG(e->st.reduced, "q_step_post_attn: state.reduced is null");
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_add_rmsnorm(s.x, s.reduced, nullptr, e->layers[layer].ln_post, s.x, s.normed, e->rows,
                    c.hidden, c.rms_eps, stream));
  TRY(mlp_block(e, layer, s.partials, stream));
  return q_reduce_partials(s.partials, &e->p_down, s.reduced, stream);
}

extern "C" int q_step_post_mlp(q_engine* e, int layer, void* stream) {
  TRY(ready(e, "q_step_post_mlp"));
  Q_CHECK_ARG(layer >= 0 && layer < e->cfg.n_layers, "q_step_post_mlp: layer out of range");
  Q_CHECK_ARG(e->st.reduced, "q_step_post_mlp: state.reduced is null");
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  return q_add_rmsnorm(s.x, s.reduced, nullptr, next_gain(e, layer), s.x, s.normed, e->rows,
                       c.hidden, c.rms_eps, stream);
}

// Logits round + per-row pick. `advance`: write the winners to st.tokens and bump the position
// (the single-token step on one GPU); otherwise only arg_val / arg_idx are written.
static int head_argmax(q_engine* e, bool advance, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  StatusTap tap = {};
  if (advance || e->T > 1) tap = status_tap(e);     // under tensor parallelism the merge kernel taps
  return q_logits_argmax_tap(s.partials, &e->p_head, s.logits, s.arg_val, s.arg_idx,
                             advance ? s.tokens : nullptr, advance ? s.pos : nullptr, 1, s.arg_scratch,
                             e->rows, c.vocab, c.vocab_offset, tap, stream);
}

static int head(q_engine* e, bool advance, void* stream) {
  const q_state_t& s = e->st;
  TRY(project(e, s.normed, s.lm_head, s.lm_head_tc, s.partials, e->p_head, stream));
  return head_argmax(e, advance, stream);
}

extern "C" int q_step_head(q_engine* e, void* stream) {
  TRY(ready(e, "q_step_head"));
  return head(e, e->cfg.tp_size == 1 && e->T == 1, stream);
}

// Final pick over the vocabulary shards gathered by the caller ([shards][rows]), with the
// status words copied out if the state asks for them.
extern "C" int q_step_merge(q_engine* e, const float* d_val, const int32_t* d_idx, void* stream) {
  TRY(ready(e, "q_step_merge"));
  const q_state_t& s = e->st;
  return q_argmax_merge_tap(d_val, d_idx, e->cfg.tp_size, e->rows, s.tokens, s.pos, 1, status_tap(e), stream);
}

// Receive area of the cross-rank sums: [2 halves][world][2 slots][rows][hidden] pairs {fp32
// partial, call counter} of 8 bytes per rank, counted in floats (the one-kernel exchange above
// 8 rows uses half of it: [2 halves][world][rows][hidden]).
extern "C" int64_t q_engine_peer_floats(const q_engine* e, int rows) {
  if (!e || rows < 1 || rows > Q_MAX_ROWS) return -1;
  return 2ll * 2ll * 2ll * e->cfg.tp_size * rows * e->cfg.hidden;
}

extern "C" int q_bind_peers(q_engine* e, const q_peers_t* peers) {
  Q_CHECK_ARG(e != nullptr, "q_bind_peers: null engine");
  if (peers == nullptr) {           // unbind: q_decode_step_peers is refused again
    e->has_peers = false;
    return Q_OK;
  }
  Q_CHECK_ARG(e->has_state, "q_bind_peers: bind the state first");
  Q_CHECK_ARG(peers->world == e->cfg.tp_size && peers->world >= 2 && peers->world <= Q_MAX_PEERS &&
                  peers->rank >= 0 && peers->rank < peers->world && peers->epoch,
              "q_bind_peers: world %d does not match tp_size %d (or bad rank / no counter words)", peers->world,
              e->cfg.tp_size);
  Q_CHECK_ARG(e->cfg.hidden % 4 == 0 && e->cfg.hidden <= 4096, "q_bind_peers: the peer step needs hidden <= 4096");
  for (int r = 0; r < peers->world; ++r)
    Q_CHECK_ARG(peers->partials[r] && peers->flags[r], "q_bind_peers: rank %d is not mapped", r);
  e->peers = *peers;
  e->has_peers = true;
  return Q_OK;
}

// The sharded step with the cross-rank sums exchanged through peer memory: per layer QKV,
// attention, O, add+norm over all ranks, gate|up + SwiGLU, down, add+norm over all ranks; then
// the lm_head shard, the local pick and the pick over the shards, exchanged the same way. No
// collective library call, and no launch besides the single-GPU step's own.
extern "C" int q_decode_step_peers(q_engine* e, void* stream) {
  TRY(ready(e, "q_decode_step_peers"));
  Q_CHECK_ARG(e->has_peers, "q_decode_step_peers: q_bind_peers has not been called");
  Q_CHECK_ARG(e->T == 1, "q_decode_step_peers: one query token per sequence");
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_step_begin(e, stream));
  if (peer_exchange_in_gemm(e)) {
    // 1-8 rows: five launches per layer as on one GPU. The O and down projections push their
    // partials to every rank, the projection after them adds all ranks' in its add+norm
    // prologue; the residual alternates between st.x and st.normed as in run_layers.
    const int rows = e->rows;
    TRY(q_gemm_launch_planned(s.normed, e->layers[0].wqkv, s.partials, &e->p_qkv, stream));
    for (int l = 0; l < c.n_layers; ++l) {
      TRY(attn_after_qkv(e, l, nullptr, stream));
      TRY(q_gemm_swiglu_addnorm_peers(s.x, &e->peers, &e->p_o, e->layers[l].ln_post, s.normed, e->layers[l].wgu,
                                      s.act, rows, c.inter, c.hidden, c.rms_eps, stream));
      TRY(q_gemm_push(s.act, e->layers[l].wdown, &e->p_down, &e->peers, stream));
      const bool last = l + 1 == c.n_layers;
      TRY(q_gemm_splitk_addnorm_peers(s.normed, &e->peers, &e->p_down, next_gain(e, l), s.x,
                                      last ? s.lm_head : e->layers[l + 1].wqkv, s.partials, rows,
                                      last ? c.vocab : e->p_qkv.N, c.hidden, c.rms_eps, stream));
    }
    TRY(head_argmax(e, false, stream));
    return q_argmax_merge_peers_tap(s.arg_val, s.arg_idx, &e->peers, e->rows, s.tokens, s.pos, 1, status_tap(e),
                                    stream);
  }
  for (int l = 0; l < c.n_layers; ++l) {
    TRY(attn_block(e, l, s.partials, stream));
    TRY(q_add_rmsnorm_peers(s.x, &e->peers, s.partials, &e->p_o, e->layers[l].ln_post, s.x, s.normed, e->rows,
                            c.hidden, c.rms_eps, stream));
    TRY(mlp_block(e, l, s.partials, stream));
    TRY(q_add_rmsnorm_peers(s.x, &e->peers, s.partials, &e->p_down, next_gain(e, l), s.x, s.normed, e->rows,
                            c.hidden, c.rms_eps, stream));
  }
  TRY(head(e, false, stream));
  return q_argmax_merge_peers_tap(s.arg_val, s.arg_idx, &e->peers, e->rows, s.tokens, s.pos, 1, status_tap(e),
                                  stream);
}

// The layers and the head for the bound row count; `advance` as in head_argmax.
static int run_layers(q_engine* e, bool advance, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_step_begin(e, stream));
  if (norm_in_gemm(e)) {
    // st.x holds the residual at every layer boundary; st.normed holds it between the
    // attention and the MLP half. Hidden-size partials go to the second buffer, which no
    // projection with a prologue writes.
    float* hp = hidden_partials(e, true);
    const int rows = e->rows;
    TRY(q_gemm_launch_planned(s.normed, e->layers[0].wqkv, s.partials, &e->p_qkv, stream));
    for (int l = 0; l < c.n_layers; ++l) {
      TRY(attn_after_qkv(e, l, hp, stream));
      TRY(q_gemm_swiglu_addnorm(s.x, hp, &e->p_o, e->layers[l].ln_post, s.normed, e->layers[l].wgu,
                                s.act, rows, c.inter, c.hidden, c.rms_eps, stream));
      TRY(q_gemm_launch_planned(s.act, e->layers[l].wdown, hp, &e->p_down, stream));
      const bool last = l + 1 == c.n_layers;
      TRY(q_gemm_splitk_addnorm(s.normed, hp, &e->p_down, next_gain(e, l), s.x,
                                last ? s.lm_head : e->layers[l + 1].wqkv, s.partials, rows,
                                last ? c.vocab : e->p_qkv.N, c.hidden, c.rms_eps, stream));
    }
    return head_argmax(e, advance, stream);
  }
  for (int l = 0; l < c.n_layers; ++l) {
    TRY(attn_block(e, l, s.partials, stream));
    TRY(q_add_rmsnorm(s.x, s.partials, &e->p_o, e->layers[l].ln_post, s.x, s.normed, e->rows,
                      c.hidden, c.rms_eps, stream));
    TRY(mlp_block(e, l, s.partials, stream));
    TRY(q_add_rmsnorm(s.x, s.partials, &e->p_down, next_gain(e, l), s.x, s.normed, e->rows, c.hidden,
                      c.rms_eps, stream));
  }
  return head(e, advance, stream);
}

extern "C" int q_decode_step(q_engine* e, void* stream) {
  TRY(ready(e, "q_decode_step"));
  Q_CHECK_ARG(e->cfg.tp_size == 1, "q_decode_step: single-GPU entry point called with tp_size %d",
              e->cfg.tp_size);
  Q_CHECK_ARG(e->T == 1, "q_decode_step: the bound state has %d query tokens per sequence (use q_verify_step)",
              e->T);
  return run_layers(e, true, stream);
}

// T query tokens per sequence through all layers: row b*T + t holds candidate token
// st.tokens[b*T + t] at position *st.pos + t and sees the keys before it, so arg_idx[b*T + t]
// is the greedy successor of that row's prefix. Tokens and position are left alone: the
// caller accepts a prefix and sets them. K/V rows of all T positions are written; rows past
// the accepted prefix are overwritten by the next call before anything reads them.
extern "C" int q_verify_step(q_engine* e, void* stream) {
  TRY(ready(e, "q_verify_step"));
  Q_CHECK_ARG(e->cfg.tp_size == 1, "q_verify_step: single GPU only");
  return run_layers(e, false, stream);
}
