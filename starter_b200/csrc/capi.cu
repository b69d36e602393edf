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
#include "mega_step.h"

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
static int g_fused_step = 0;     // 1 = use the persistent whole-step kernel when it applies
static int g_norm_in_gemm = 1;   // 1 = residual add + RMSNorm as the prologue of the next projection
static int g_trace_layer = -1;   // measurement aid: layer whose phases the whole-step kernel stamps

// Launch timeline (measurement aid): Q_TL_SLOTS records of 4 stamps, handed out in launch order.
#define Q_TL_SLOTS 1024
static __device__ unsigned long long g_timeline[Q_TL_SLOTS * 4];
static int g_tl_on = 0, g_tl_used = 0;
static unsigned long long* g_tl_base = nullptr;

static int tl_reset() {
  static unsigned long long init[Q_TL_SLOTS * 4];
  for (int i = 0; i < Q_TL_SLOTS; ++i) {
    init[4 * i] = init[4 * i + 1] = ~0ull;
    init[4 * i + 2] = init[4 * i + 3] = 0ull;
  }
  return cudaMemcpyToSymbol(g_timeline, init, sizeof(init)) == cudaSuccess ? 0 : -1;
}

unsigned long long* q_tl_next() {
  if (!g_tl_on || g_tl_base == nullptr || g_tl_used >= Q_TL_SLOTS) return nullptr;
  return g_tl_base + 4 * (g_tl_used++);
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
  if (strcmp(name, "trace_layer") == 0) {
    g_trace_layer = value;
    return Q_OK;
  }
  if (strcmp(name, "fused_step") == 0) {
    g_fused_step = value != 0;
    return Q_OK;
  }
  if (strcmp(name, "norm_in_gemm") == 0) {
    g_norm_in_gemm = value != 0;
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

int q_peer_status_read(int32_t* out);
int q_attn_status_read(int32_t out[4]);
int q_gemm_status_read(int32_t out[4]);

extern "C" int q_device_status(int32_t out[4]) {
  Q_CHECK_ARG(out != nullptr, "q_device_status: null pointer");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  int32_t a[4] = {0, 0, 0, 0}, g[4] = {0, 0, 0, 0}, m[4] = {0, 0, 0, 0};
  if (q_attn_status_read(a) || q_gemm_status_read(g) || q_mega_status_read(m)) {
    q_set_error("q_device_status: could not read the status words");
    return Q_ERR_CUDA;
  }
  out[0] = a[0];   // attention: 1 producer wait ran out, 2 consumer wait ran out
  out[1] = g[0];   // GEMM: 1 ring wait ran out
  out[2] = m[0];   // whole-step kernel: 1 grid barrier, 2 GEMM ring, 3/4 attention ring
  int32_t peer = 0;
  if (q_peer_status_read(&peer)) { q_set_error("q_device_status: could not read the status words"); return Q_ERR_CUDA; }
  out[3] = peer;   // tensor parallel over peer memory: 1 = a wait for a peer's arrival word ran out
  return Q_OK;
}

extern "C" int q_debug_step_trace(unsigned long long* out) {
  Q_CHECK_ARG(out != nullptr, "q_debug_step_trace: null pointer (needs 704 values)");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  if (q_mega_trace_read(out)) { q_set_error("q_debug_step_trace: read failed"); return Q_ERR_CUDA; }
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
  int rows;
  q_gemm_plan_t p_qkv, p_o, p_gu, p_down, p_head;
  bool mega_ok;
  int mega_grid;
  mega_params_t mega;
  bool has_peers;
  q_peers_t peers;
};

static int make_plans(q_engine* e, int rows) {
  const q_config_t& c = e->cfg;
  int rc;
  if ((rc = q_gemm_plan(rows, (c.n_q_heads + 2 * c.n_kv_heads) * 128, c.hidden, &e->p_qkv))) return rc;
  if ((rc = q_gemm_plan(rows, c.hidden, c.n_q_heads * 128, &e->p_o))) return rc;
  if ((rc = q_gemm_plan(rows, 2 * c.inter, c.hidden, &e->p_gu))) return rc;
  if ((rc = q_gemm_plan(rows, c.hidden, c.inter, &e->p_down))) return rc;
  if ((rc = q_gemm_plan(rows, c.vocab, c.hidden, &e->p_head))) return rc;
  e->rows = rows;
  return Q_OK;
}

static long long plan_floats(const q_gemm_plan_t& p) { return (long long)p.slots * p.M * p.N; }

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
  e->mega_ok = false;
  e->mega_grid = 0;
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
  e->layers[layer] = *w;
  e->bound[layer] = true;
  return Q_OK;
}

extern "C" int64_t q_engine_partial_floats(const q_engine* e, int rows) {
  if (!e || rows < 1 || rows > Q_MAX_ROWS) return -1;
  q_engine tmp = *e;
  if (make_plans(&tmp, rows)) return -1;
  long long m = plan_floats(tmp.p_qkv);
  if (plan_floats(tmp.p_o) > m) m = plan_floats(tmp.p_o);
  if (plan_floats(tmp.p_gu) > m) m = plan_floats(tmp.p_gu);
  if (plan_floats(tmp.p_down) > m) m = plan_floats(tmp.p_down);
  if (plan_floats(tmp.p_head) > m) m = plan_floats(tmp.p_head);
  // the fused step keeps the O-proj/down partials in a second buffer behind the first
  long long second = plan_floats(tmp.p_o) > plan_floats(tmp.p_down) ? plan_floats(tmp.p_o) : plan_floats(tmp.p_down);
  return ((m + 63) / 64) * 64 + second;
}

static long long first_partial_floats(const q_engine* e) {
  long long m = plan_floats(e->p_qkv);
  if (plan_floats(e->p_o) > m) m = plan_floats(e->p_o);
  if (plan_floats(e->p_gu) > m) m = plan_floats(e->p_gu);
  if (plan_floats(e->p_down) > m) m = plan_floats(e->p_down);
  if (plan_floats(e->p_head) > m) m = plan_floats(e->p_head);
  return ((m + 63) / 64) * 64;
}

extern "C" int64_t q_fused_scratch_bytes(const q_engine* e, int rows) {
  if (!e || rows < 1) return -1;
  const int sms = q_sm_count();
  return 1024 + (int64_t)e->cfg.n_layers * (int64_t)sizeof(mega_layer_t) + 64 +
         (int64_t)rows * sms * 8 + 64;
}

static mega_plan_t lite(const q_gemm_plan_t& p) {
  mega_plan_t m;
  m.N = p.N; m.K = p.K; m.C = p.chunks_per_group; m.total = p.groups * p.chunks_per_group;
  m.U = p.units_per_worker;
  return m;
}

// Decides whether the persistent whole-step kernel applies and fills its parameters.
static int setup_fused(q_engine* e) {
  e->mega_ok = false;
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  if (c.tp_size != 1 || !s.fused_scratch || e->rows > 8) return Q_OK;
  const int sms = q_sm_count();
  const int G = c.n_q_heads / c.n_kv_heads;
  if (G > 16 || e->rows * c.n_kv_heads > sms) return Q_OK;
  int xs_cols = c.hidden;
  if (c.n_q_heads * 128 > xs_cols) xs_cols = c.n_q_heads * 128;
  if (c.inter > xs_cols) xs_cols = c.inter;
  int dev = 0, max_smem = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
    cudaGetLastError();
    return Q_OK;
  }
  if (q_mega_smem_bytes(e->rows, c.hidden, xs_cols) > (size_t)max_smem) return Q_OK;
  int coop = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (!coop) return Q_OK;
  // every GEMM must fit the grid (one CTA per SM) and all plans share the grid size
  int grid = e->p_qkv.grid;
  const q_gemm_plan_t* plans[5] = {&e->p_qkv, &e->p_o, &e->p_gu, &e->p_down, &e->p_head};
  for (int i = 0; i < 5; ++i) if (plans[i]->grid > grid) grid = plans[i]->grid;
  if (grid < e->rows * c.n_kv_heads) grid = e->rows * c.n_kv_heads;   // one CTA per (sequence, kv head) at least
  if (grid > sms) return Q_OK;

  char* base = (char*)s.fused_scratch;
  mega_params_t& m = e->mega;
  memset(&m, 0, sizeof(m));
  m.sync = (unsigned*)base;
  mega_layer_t* table = (mega_layer_t*)(base + 1024);
  char* after = base + 1024 + (size_t)c.n_layers * sizeof(mega_layer_t);
  after = (char*)(((uintptr_t)after + 63) & ~(uintptr_t)63);
  m.blk_val = (float*)after;
  m.blk_idx = (int*)(after + (size_t)e->rows * sms * 4);
  std::vector<mega_layer_t> host(c.n_layers);
  for (int i = 0; i < c.n_layers; ++i) {
    const q_layer_weights_t& w = e->layers[i];
    if (!e->bound[i]) return Q_OK;       // bind layers first; q_bind_state can be called again
    host[i].wqkv = (const unsigned char*)w.wqkv; host[i].wo = (const unsigned char*)w.wo;
    host[i].wgu = (const unsigned char*)w.wgu; host[i].wdown = (const unsigned char*)w.wdown;
    host[i].ln_in = (const bf16*)w.ln_in; host[i].ln_post = (const bf16*)w.ln_post;
    host[i].q_gain = (const bf16*)w.q_gain; host[i].k_gain = (const bf16*)w.k_gain;
    host[i].kpool = (char*)w.kpool; host[i].vpool = (char*)w.vpool;
  }
  Q_CHECK_CUDA(cudaMemcpy(table, host.data(), host.size() * sizeof(mega_layer_t), cudaMemcpyHostToDevice));
  Q_CHECK_CUDA(cudaMemset(m.sync, 0, 1024));
  m.layers = table;
  m.M = e->rows; m.H = c.hidden; m.I = c.inter; m.L = c.n_layers; m.nq = c.n_q_heads; m.nkv = c.n_kv_heads;
  m.V = c.vocab; m.full_vocab = c.full_vocab; m.pages_per_seq = s.pages_per_seq; m.xs_cols = xs_cols;
  int S = s.attn_splits;
  const int fit = grid / (e->rows * c.n_kv_heads);
  if (S > fit) S = fit;
  if (S < 1) S = 1;
  m.attn_S = S;
  m.trace_layer = -1;
  m.eps = c.rms_eps;
  m.scale_log2 = c.attn_scale * 1.4426950408889634f;
  m.embed = (const unsigned char*)s.embed; m.lm_head = (const unsigned char*)s.lm_head;
  m.ln_final = (const bf16*)s.ln_final; m.cos = (const bf16*)s.cos; m.sin = (const bf16*)s.sin;
  m.tokens = s.tokens; m.pos = s.pos; m.block_table = s.block_table;
  m.buf0 = s.partials; m.buf1 = s.partials + first_partial_floats(e);
  m.attended = (bf16*)s.attended; m.act = (bf16*)s.act; m.attn_o = s.attn_o; m.attn_ml = s.attn_ml;
  m.logits = (bf16*)s.logits; m.arg_val = s.arg_val; m.arg_idx = s.arg_idx;
  m.qkv = lite(e->p_qkv); m.o = lite(e->p_o); m.gu = lite(e->p_gu); m.down = lite(e->p_down);
  m.head = lite(e->p_head);
  e->mega_grid = grid;
  e->mega_ok = true;
  return Q_OK;
}

extern "C" int q_bind_state(q_engine* e, const q_state_t* s) {
  Q_CHECK_ARG(e && s, "q_bind_state: null pointer");
  Q_CHECK_ARG(s->batch >= 1 && s->batch <= e->cfg.max_rows, "q_bind_state: batch %d outside 1..%d",
              s->batch, e->cfg.max_rows);
  Q_CHECK_ARG(s->embed && s->lm_head && s->ln_final && s->cos && s->sin && s->tokens && s->pos &&
                  s->block_table && s->x && s->normed && s->q && s->attended && s->act &&
                  s->partials && s->arg_val && s->arg_idx && s->arg_scratch,
              "q_bind_state: a required pointer is null");
  Q_CHECK_ARG(s->pages_per_seq >= 1, "q_bind_state: pages_per_seq must be >= 1");
  Q_CHECK_ARG(s->attn_splits >= 1 && s->attn_splits <= 32, "q_bind_state: attn_splits outside 1..32");
  Q_CHECK_ARG(s->attn_splits == 1 || (s->attn_o && s->attn_ml), "q_bind_state: attention scratch missing");
  Q_CHECK_ARG(e->cfg.tp_size == 1 || s->reduced, "q_bind_state: tensor parallel needs `reduced`");
  int rc = make_plans(e, s->batch);
  if (rc) return rc;
  e->st = *s;
  e->has_state = true;
  return setup_fused(e);
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

// Where the hidden-size projections (O, down) leave their partials. With the add+norm
// prologue the next projection reads them while it writes its own, so they live in the
// second buffer behind the first (q_engine_partial_floats sizes both).
static float* hidden_partials(const q_engine* e, bool second) {
  return second ? e->st.partials + first_partial_floats(e) : e->st.partials;
}

// Up to 8 rows on one GPU: residual add + RMSNorm run as the prologue of the projection
// that consumes them, the residual alternating between st.x and st.normed.
static bool norm_in_gemm(const q_engine* e) {
  return e->cfg.tp_size == 1 && e->rows <= 8 && e->cfg.hidden % 4 == 0 && e->cfg.hidden <= 3072 &&
         g_norm_in_gemm;
}

// attention .. O projection, from the QKV partials in st.partials.
static int attn_after_qkv(q_engine* e, int layer, float* o_partials, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  const q_layer_weights_t& w = e->layers[layer];
  q_kv_layout_t kv = kv_of(e, layer);
  if (s.attn_tickets && c.n_q_heads / c.n_kv_heads <= 8) {
    // head norm + RoPE + K/V write + attention + split merge in one launch
    TRY(q_attention_decode(s.partials, &e->p_qkv, w.q_gain, w.k_gain, s.cos, s.sin, s.pos, &kv, s.attn_o,
                           s.attn_ml, s.attn_tickets, s.attended, s.batch, c.n_q_heads, s.attn_splits,
                           c.attn_scale, c.rms_eps, stream));
  } else {
    TRY(q_qkv_norm_rope_cache(s.partials, &e->p_qkv, w.q_gain, w.k_gain, s.cos, s.sin, s.pos, s.q, &kv,
                              s.batch, 1, c.n_q_heads, c.rms_eps, stream));
    TRY(q_attention(s.q, &kv, s.pos, s.attn_o, s.attn_ml, s.attended, s.batch, 1, c.n_q_heads,
                    s.attn_splits, c.attn_scale, stream));
  }
  return q_gemm_launch_planned(s.attended, w.wo, o_partials, &e->p_o, stream);
}

// QKV projection .. attention .. O projection (partials left in st.partials).
static int attn_block(q_engine* e, int layer, void* stream) {
  const q_state_t& s = e->st;
  TRY(q_gemm_splitk(s.normed, e->layers[layer].wqkv, s.partials, e->rows, e->p_qkv.N, e->cfg.hidden,
                    stream));
  return attn_after_qkv(e, layer, s.partials, stream);
}

// gate|up projection + SwiGLU (the layer's gate|up weight is in q_gemm_swiglu's interleaved row
// order), then the down projection.
static int mlp_block(q_engine* e, int layer, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  if (e->rows <= 8) {
    TRY(q_gemm_swiglu(s.normed, e->layers[layer].wgu, s.act, e->rows, c.inter, c.hidden, stream));
  } else {
    // Above 8 rows the projection is bound by instruction issue, not by memory, and whole
    // groups per CTA (8 or 9 of them) cost more than the SwiGLU launch saves: stream-K
    // partials, then SwiGLU on the interleaved columns.
    TRY(q_gemm_splitk(s.normed, e->layers[layer].wgu, s.partials, e->rows, 2 * c.inter, c.hidden, stream));
    TRY(q_swiglu_layout(s.partials, &e->p_gu, s.act, e->rows, c.inter, 1, stream));
  }
  TRY(q_gemm_splitk(s.act, e->layers[layer].wdown, s.partials, e->rows, c.hidden, c.inter, stream));
  return Q_OK;
}

static const void* next_gain(const q_engine* e, int layer) {
  return layer + 1 < e->cfg.n_layers ? e->layers[layer + 1].ln_in : e->st.ln_final;
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
  TRY(attn_block(e, layer, stream));
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
  TRY(mlp_block(e, layer, stream));
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

static int head_argmax(q_engine* e, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  const bool single = c.tp_size == 1;
  return q_logits_argmax(s.partials, &e->p_head, s.logits, s.arg_val, s.arg_idx,
                         single ? s.tokens : nullptr, single ? s.pos : nullptr, 1, s.arg_scratch,
                         e->rows, c.vocab, c.vocab_offset, stream);
}

extern "C" int q_step_head(q_engine* e, void* stream) {
  TRY(ready(e, "q_step_head"));
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_gemm_splitk(s.normed, s.lm_head, s.partials, e->rows, c.vocab, c.hidden, stream));
  return head_argmax(e, stream);
}


// Peer-readable buffer: [O partials | down partials], each rounded up to 64 floats.
static long long peer_half_floats(const q_engine* e) {
  long long m = plan_floats(e->p_o) > plan_floats(e->p_down) ? plan_floats(e->p_o) : plan_floats(e->p_down);
  return ((m + 63) / 64) * 64;
}

extern "C" int64_t q_engine_peer_floats(const q_engine* e, int rows) {
  if (!e || rows < 1 || rows > Q_MAX_ROWS) return -1;
  q_engine tmp = *e;
  if (make_plans(&tmp, rows)) return -1;
  return 2 * peer_half_floats(&tmp);
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
              "q_bind_peers: world %d does not match tp_size %d (or bad rank / no epoch word)", peers->world,
              e->cfg.tp_size);
  Q_CHECK_ARG(e->rows <= 8 && e->cfg.hidden % 4 == 0 && e->cfg.hidden <= 3072,
              "q_bind_peers: the peer step takes up to 8 rows and hidden <= 3072");
  for (int r = 0; r < peers->world; ++r)
    Q_CHECK_ARG(peers->partials[r] && peers->flags[r], "q_bind_peers: rank %d is not mapped", r);
  e->peers = *peers;
  e->has_peers = true;
  return Q_OK;
}

// The sharded step with the cross-rank sums read from peer memory: per layer QKV, attention,
// O (partials -> peer buffer half 0), add+norm over all ranks, gate|up + SwiGLU, down (->
// half 1), add+norm over all ranks. The two halves alternate, which is what
// q_add_rmsnorm_peers needs; every other projection writes the private partial buffer.
extern "C" int q_decode_step_peers(q_engine* e, void* stream) {
  TRY(ready(e, "q_decode_step_peers"));
  Q_CHECK_ARG(e->has_peers, "q_decode_step_peers: q_bind_peers has not been called");
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  float* half0 = e->peers.partials[e->peers.rank];
  float* half1 = half0 + peer_half_floats(e);
  TRY(q_step_begin(e, stream));
  for (int l = 0; l < c.n_layers; ++l) {
    TRY(q_gemm_splitk(s.normed, e->layers[l].wqkv, s.partials, e->rows, e->p_qkv.N, c.hidden, stream));
    TRY(attn_after_qkv(e, l, half0, stream));
    TRY(q_add_rmsnorm_peers(s.x, &e->peers, half0, &e->p_o, e->layers[l].ln_post, s.x, s.normed, e->rows,
                            c.hidden, c.rms_eps, stream));
    TRY(q_gemm_swiglu(s.normed, e->layers[l].wgu, s.act, e->rows, c.inter, c.hidden, stream));
    TRY(q_gemm_splitk(s.act, e->layers[l].wdown, half1, e->rows, c.hidden, c.inter, stream));
    TRY(q_add_rmsnorm_peers(s.x, &e->peers, half1, &e->p_down, next_gain(e, l), s.x, s.normed, e->rows,
                            c.hidden, c.rms_eps, stream));
  }
  TRY(q_gemm_splitk(s.normed, s.lm_head, s.partials, e->rows, c.vocab, c.hidden, stream));
  return head_argmax(e, stream);
}

extern "C" int q_decode_step(q_engine* e, void* stream) {
  TRY(ready(e, "q_decode_step"));
  Q_CHECK_ARG(e->cfg.tp_size == 1, "q_decode_step: single-GPU entry point called with tp_size %d",
              e->cfg.tp_size);
  if (e->mega_ok && g_fused_step) {
    e->mega.trace_layer = g_trace_layer;
    e->mega.prefetch_units = g_gemm_prefetch_kb / 8;     // per warp (8 warps per CTA), 1 KB units
    Q_CHECK_CUDA(q_mega_launch(e->mega, e->mega_grid, (cudaStream_t)stream));
    return Q_OK;
  }
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_step_begin(e, stream));
  if (norm_in_gemm(e)) {
    // st.x holds the residual at every layer boundary; st.normed holds it between the
    // attention and the MLP half. Hidden-size partials go to the second buffer, which no
    // projection with a prologue writes.
    float* hp = hidden_partials(e, true);
    const int rows = e->rows;
    TRY(q_gemm_splitk(s.normed, e->layers[0].wqkv, s.partials, rows, e->p_qkv.N, c.hidden, stream));
    for (int l = 0; l < c.n_layers; ++l) {
      TRY(attn_after_qkv(e, l, hp, stream));
      TRY(q_gemm_swiglu_addnorm(s.x, hp, &e->p_o, e->layers[l].ln_post, s.normed, e->layers[l].wgu,
                                s.act, rows, c.inter, c.hidden, c.rms_eps, stream));
      TRY(q_gemm_splitk(s.act, e->layers[l].wdown, hp, rows, c.hidden, c.inter, stream));
      const bool last = l + 1 == c.n_layers;
      TRY(q_gemm_splitk_addnorm(s.normed, hp, &e->p_down, next_gain(e, l), s.x,
                                last ? s.lm_head : e->layers[l + 1].wqkv, s.partials, rows,
                                last ? c.vocab : e->p_qkv.N, c.hidden, c.rms_eps, stream));
    }
    return head_argmax(e, stream);
  }
  for (int l = 0; l < c.n_layers; ++l) {
    TRY(attn_block(e, l, stream));
    TRY(q_add_rmsnorm(s.x, s.partials, &e->p_o, e->layers[l].ln_post, s.x, s.normed, e->rows,
                      c.hidden, c.rms_eps, stream));
    TRY(mlp_block(e, l, stream));
    TRY(q_add_rmsnorm(s.x, s.partials, &e->p_down, next_gain(e, l), s.x, s.normed, e->rows, c.hidden,
                      c.rms_eps, stream));
  }
  return q_step_head(e, stream);
}
