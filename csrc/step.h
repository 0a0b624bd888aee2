// Descriptors of the native step driver (csrc/step.cu).  Plain C structs of device pointers and sizes that the host
// fills once per model and once per set of step buffers; the driver never owns or frees what they point to.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZSE_STEP_W4 0  /* tiled INT4 (zse_repack_w4) */
#define ZSE_STEP_F16 1 /* dense fp16 [N, K] */

typedef struct {
  int32_t kind;
  int32_t N; /* output rows as the kernel sees them (gate + up counted together) */
  int32_t K;
  int32_t reserved;
  const void* data;
  const void* bias; /* fp16 [N] or NULL */
} ZseStepLinear;

typedef struct {
  ZseStepLinear qkv, o, gate_up, down;
  const void* ln1; /* fp16 [hidden] */
  const void* ln2;
} ZseStepLayer;

typedef struct {
  int32_t num_layers, hidden, num_heads, num_kv_heads, head_dim, inter, vocab_rows, rotary_dim, sm_count;
  int32_t attn_tc; /* != 0: prefill attention of head_dim 128 on the tcgen05 kernel (zse_attn_prefill_tc) */
  float eps, scale, embed_scale, reserved_f;
  const void* embed;      /* fp16 [vocab_rows, hidden] */
  const void* final_norm; /* fp16 [hidden] */
  const void* inv_freq;   /* fp32 [rotary_dim / 2] */
  ZseStepLinear lm_head;
  const ZseStepLayer* layers; /* host array of num_layers entries */
  const void* rope_table;     /* fp32 [max_position][64][2] cos/sin, or NULL (no fused QKV epilogue) */
  int32_t max_position;
  int32_t dec_mode;           /* decode-sized INT4 layers through zse_gemm_w4_dec: 1 gate/up, 2 fused QKV, 4 the rest,
                                 8 o / down with the residual add and the next RMSNorm in the same kernel */
} ZseStepModel;

typedef struct {
  int32_t max_tokens, max_blocks, qkv_plane_rows, qkv_max_planes, max_planes, logits_rows_cap, logits_ld, reserved;
  void* ids;          /* int32 [max_tokens] */
  void* positions;    /* int32 [max_tokens] */
  void* slots;        /* int64 [max_tokens] */
  void* block_tables; /* int32 [max_seqs, max_blocks] */
  void* seq_lens;     /* int32 [max_seqs] */
  void* cu_q;         /* int32 [max_seqs + 1] */
  void* q_pos0;       /* int32 [max_seqs] */
  void* logit_rows;   /* int64 [logits_rows_cap] */
  void* residual;     /* fp32 [max_tokens, hidden] */
  void* xnorm;        /* fp16 [max_tokens, hidden] */
  void* qkv;          /* fp16 [max_tokens, (nh + 2 nkv) hd] */
  void* attn_out;     /* fp16 [max_tokens, nh hd] */
  void* qkv_planes;   /* fp32 [qkv_max_planes, qkv_plane_rows, (nh + 2 nkv) hd] */
  void* act;          /* fp16 [max_tokens, inter] */
  void* gate_up_tmp;  /* fp16 [max_tokens, 2 inter], only for dense gate/up weights; may be NULL */
  void* partials;     /* fp32 [max_planes, max_tokens, hidden] */
  void* xsel;         /* fp16 [logits_rows_cap, hidden] */
  void* logits;       /* fp16 [logits_rows_cap, logits_ld] */
  void* attn_scratch; /* fp32, zse_attn_decode_scratch_floats(max_seqs, nh, hd, splits) */
  void* status;       /* 16-byte device status word */
  void* dec_ws;       /* workspace of zse_gemm_w4_dec (zse_gemm_w4_dec_workspace_bytes), or NULL */
  void* norm_ctx;     /* one-rank tensor-parallel context with push buffers (dec_mode & 8), or NULL */
} ZseStepBuffers;

/* 1 when the driver can run this model with these buffers, else 0 (the caller keeps its own wiring) */
int zse_step_supported(const ZseStepModel* model, const ZseStepBuffers* buffers);
/* One pass over tokens ids[0..M): kv = base of the pool [layers][blocks][2][nkv][block_size][hd] (fp16),
 * kv_layer_stride in elements.  decode != 0: one token per sequence; else packed causal attention with cu_q / q_pos0.
 * Leaves fp16 logits of rows logit_rows[0..n_logit_rows) in `logits`.  Returns 0 or the first ZSE_ERR_* code;
 * *launches_out = kernels launched. */
int zse_step_forward(const ZseStepModel* model, const ZseStepBuffers* buffers, void* kv, int64_t kv_layer_stride,
                     int block_size, int M, int decode, int num_seqs, int max_q_len, int n_logit_rows, int attn_splits,
                     void* stream, int* launches_out);

#ifdef __cplusplus
}
#endif
