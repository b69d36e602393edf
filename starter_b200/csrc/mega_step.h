// Parameter block of the persistent whole-step kernel (mega_step.cu). Internal to
// the library: filled by capi.cu from the bound engine state.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

struct mega_plan_t { int N, K, C, total, U; };

struct mega_layer_t {
  const unsigned char *wqkv, *wo, *wgu, *wdown;     // tiled weights
  const __nv_bfloat16 *ln_in, *ln_post, *q_gain, *k_gain;
  char *kpool, *vpool;
};

struct mega_params_t {
  int M, H, I, L, nq, nkv, V, full_vocab, pages_per_seq, attn_S, xs_cols, trace_layer, prefetch_units;
  float eps, scale_log2;
  const mega_layer_t* layers;                        // device array [L]
  const unsigned char* embed;
  const unsigned char* lm_head;
  const __nv_bfloat16* ln_final;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  int64_t* tokens;
  int32_t* pos;
  const int32_t* block_table;
  float* buf0;                                       // QKV / gate|up / lm_head partials
  float* buf1;                                       // O-proj / down partials
  __nv_bfloat16* attended;
  __nv_bfloat16* act;
  float* attn_o;
  float* attn_ml;
  __nv_bfloat16* logits;                             // may be null
  float* arg_val;
  int32_t* arg_idx;
  unsigned* sync;          // [0] grid barrier, [2] argmax ticket, [4 + b*nkv + kh] attention tickets
  float* blk_val;          // [M][grid]
  int* blk_idx;            // [M][grid]
  mega_plan_t qkv, o, gu, down, head;
};

size_t q_mega_smem_bytes(int M, int H, int xs_cols);
cudaError_t q_mega_launch(const mega_params_t& p, int grid, cudaStream_t stream);
int q_mega_status_read(int32_t out[4]);
int q_mega_trace_read(unsigned long long* out);
