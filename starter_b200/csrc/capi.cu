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

int g_gemm_prefetch_kb = 640;
int g_gemm_debug_flags = 0;

extern "C" int q_set_option(const char* name, int value) {
  Q_CHECK_ARG(name != nullptr, "q_set_option: null name");
  if (strcmp(name, "gemm_prefetch_kb") == 0) {
    Q_CHECK_ARG(value >= 0 && value <= 8192, "q_set_option: gemm_prefetch_kb outside 0..8192");
    g_gemm_prefetch_kb = value;
    return Q_OK;
  }
  if (strcmp(name, "gemm_debug_flags") == 0) {
    g_gemm_debug_flags = value;     // measurement aid: results are wrong when non-zero
    return Q_OK;
  }
  q_set_error("q_set_option: unknown option '%s'", name);
  return Q_ERR_ARG;
}

int q_attn_status_read(int32_t out[4]);
int q_gemm_status_read(int32_t out[4]);

extern "C" int q_device_status(int32_t out[4]) {
  Q_CHECK_ARG(out != nullptr, "q_device_status: null pointer");
  Q_CHECK_CUDA(cudaDeviceSynchronize());
  int32_t a[4] = {0, 0, 0, 0}, g[4] = {0, 0, 0, 0};
  if (q_attn_status_read(a) || q_gemm_status_read(g)) {
    q_set_error("q_device_status: could not read the status words");
    return Q_ERR_CUDA;
  }
  out[0] = a[0];   // attention: 1 producer wait ran out, 2 consumer wait ran out
  out[1] = g[0];   // GEMM: 1 ring wait ran out
  out[2] = out[3] = 0;
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
  e->rows = 0;
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
  return m;
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

// QKV projection .. attention .. O projection (partials left in st.partials).
static int attn_block(q_engine* e, int layer, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  const q_layer_weights_t& w = e->layers[layer];
  const int rows = e->rows;
  q_kv_layout_t kv = kv_of(e, layer);
  TRY(q_gemm_splitk(s.normed, w.wqkv, s.partials, rows, e->p_qkv.N, c.hidden, stream));
  TRY(q_qkv_norm_rope_cache(s.partials, &e->p_qkv, w.q_gain, w.k_gain, s.cos, s.sin, s.pos, s.q, &kv,
                            s.batch, 1, c.n_q_heads, c.rms_eps, stream));
  TRY(q_attention(s.q, &kv, s.pos, s.attn_o, s.attn_ml, s.attended, s.batch, 1, c.n_q_heads,
                  s.attn_splits, c.attn_scale, stream));
  TRY(q_gemm_splitk(s.attended, w.wo, s.partials, rows, c.hidden, c.n_q_heads * 128, stream));
  return Q_OK;
}

static int mlp_block(q_engine* e, int layer, void* stream) {
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  const q_layer_weights_t& w = e->layers[layer];
  const int rows = e->rows;
  TRY(q_gemm_splitk(s.normed, w.wgu, s.partials, rows, 2 * c.inter, c.hidden, stream));
  TRY(q_swiglu(s.partials, &e->p_gu, s.act, rows, c.inter, stream));
  TRY(q_gemm_splitk(s.act, w.wdown, s.partials, rows, c.hidden, c.inter, stream));
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

extern "C" int q_step_head(q_engine* e, void* stream) {
  TRY(ready(e, "q_step_head"));
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_gemm_splitk(s.normed, s.lm_head, s.partials, e->rows, c.vocab, c.hidden, stream));
  const bool single = c.tp_size == 1;
  return q_logits_argmax(s.partials, &e->p_head, s.logits, s.arg_val, s.arg_idx,
                         single ? s.tokens : nullptr, single ? s.pos : nullptr, 1, s.arg_scratch,
                         e->rows, c.vocab, c.vocab_offset, stream);
}

extern "C" int q_decode_step(q_engine* e, void* stream) {
  TRY(ready(e, "q_decode_step"));
  Q_CHECK_ARG(e->cfg.tp_size == 1, "q_decode_step: single-GPU entry point called with tp_size %d",
              e->cfg.tp_size);
  const q_config_t& c = e->cfg;
  const q_state_t& s = e->st;
  TRY(q_step_begin(e, stream));
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
