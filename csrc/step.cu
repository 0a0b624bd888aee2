// Native step driver: one C call runs a whole pass of the Llama / Mistral / Qwen2 / Phi-3 decoder (embedding, every
// layer, final norm, logits) by launching the kernels of this library in order on one stream.
//
// The reference keeps a C launcher for its single-sequence decode step (`fast_decode_m1`,
// zse-engine/zse_engine/orchestrator/fast_dispatch.py:18-338: a loop over cuLaunchKernel compiled with gcc at run
// time, and disabled because its signatures drifted from the kernels).  This one serves every kind of pass (prefill,
// chunked prefill, verification, batched decode), is built with the library, and calls the same entry points the
// Python wiring calls, so the two cannot drift apart: `tests/test_engine_gpu.py` compares their logits bit for bit.
// The launch sequence is the one described in `zse_b200/models/decoder.py`.  Passes that need per-step host logic
// between kernels (tensor-parallel collectives, LoRA) stay on the Python wiring.
#include <cuda_runtime.h>

#include "api.h"
#include "step.h"

namespace {

constexpr int kEpiF16 = 0, kEpiSwiGLU = 1, kEpiPartial = 2;

struct Pass {
  const ZseStepModel* m;
  const ZseStepBuffers* b;
  void* stream;
  int M;
  int launches;
  int rc;

  bool ok() const { return rc == 0; }
  void did(int r, int n = 1) {
    if (rc == 0) {
      rc = r;
      launches += n;
    }
  }

  // y[M, N] (fp16, +bias) = x W^T
  void linear(const ZseStepLinear& w, const void* x, void* out, int ldo, int M_) {
    if (!ok()) return;
    if (w.kind == ZSE_STEP_W4)
      did(zse_gemm_w4(w.data, x, b->max_tokens, w.bias, out, M_, w.N, w.K, ldo, kEpiF16, 0, b->status, stream));
    else
      did(zse_gemm_f16(w.data, w.N, x, b->max_tokens, w.bias, out, M_, w.N, w.K, ldo, kEpiF16, 1, b->status, stream));
  }

  // fp32 split-K planes [planes][M][N]; returns how many were written
  int linear_partial(const ZseStepLinear& w, const void* x, void* planes, int max_planes, int x_cap) {
    if (!ok()) return 0;
    if (w.kind == ZSE_STEP_W4) {
      int ks = 0;
      int n = zse_gemm_w4_splits(M, w.N, w.K, ks);
      if (n > max_planes) {
        ks = max_planes;
        n = zse_gemm_w4_splits(M, w.N, w.K, ks);
      }
      did(zse_gemm_w4(w.data, x, x_cap, nullptr, planes, M, w.N, w.K, w.N, kEpiPartial, ks, b->status, stream));
      return n;
    }
    // dense fp16 weights: enough K-split planes to fill the GPU (same rule as the Python wiring)
    const int n_tiles = (w.N + 127) / 128;
    const int nt = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const int ctas = n_tiles * ((M + nt - 1) / nt);
    int want = (m->sm_count * (nt <= 64 ? 2 : 1)) / (ctas > 0 ? ctas : 1);
    if (want < 1) want = 1;
    int by_k = (w.K / 64) / 4;
    if (by_k < 1) by_k = 1;
    int ks = want < 8 ? want : 8;
    if (ks > by_k) ks = by_k;
    if (ks > max_planes) ks = max_planes;
    const int n = zse_gemm_f16_splits(M, w.N, w.K, ks);
    did(zse_gemm_f16(w.data, w.N, x, x_cap, nullptr, planes, M, w.N, w.K, w.N, kEpiPartial, ks, b->status, stream));
    return n;
  }

  // o / down of a decode-sized pass with "residual += y; xnorm = RMSNorm(residual) * next_norm" in the GEMM kernel
  // (the one-rank case of the tensor-parallel kernel).  Returns false when the layer has to take the two-kernel path.
  bool row_fused(const ZseStepLinear& w, const void* x, const void* next_norm, int* slot) {
    if (!ok() || !(m->dec_mode & 8) || b->norm_ctx == nullptr || b->dec_ws == nullptr || w.kind != ZSE_STEP_W4 ||
        M > 64 || w.bias != nullptr || w.N != m->hidden || !zse_gemm_w4_dec_supported(M, w.N, w.K, 4))
      return false;
    int plan[2] = {0, 0};
    zse_gemm_w4_dec_plan(w.N, w.K, 4, m->sm_count, plan);
    if (plan[1] <= 0) return false;
    did(zse_tp_gemm_dec_allreduce_norm(b->norm_ctx, w.data, 0, x, b->max_tokens, M, w.N, w.K, *slot, 0, -1, b->residual,
                                       next_norm, b->xnorm, m->eps, b->dec_ws, b->status, stream));
    *slot ^= 1;
    return true;
  }

  void add_norm(int planes, const void* weight) {
    if (!ok() || planes < 0) return;          // planes < 0: the projection's own kernel added and normalised
    did(zse_add_rmsnorm(b->residual, b->partials, planes, nullptr, weight, b->xnorm, M, m->hidden, m->eps, stream));
  }
};

}  // namespace

extern "C" int zse_step_supported(const ZseStepModel* m, const ZseStepBuffers* b) {
  if (m == nullptr || b == nullptr || m->layers == nullptr || m->num_layers <= 0) return 0;
  for (int i = 0; i < m->num_layers; ++i) {
    const ZseStepLayer& L = m->layers[i];
    // a dense gate/up projection needs the [M, 2I] scratch for the separate activation kernel
    if (L.gate_up.kind != ZSE_STEP_W4 && b->gate_up_tmp == nullptr) return 0;
  }
  return 1;
}

extern "C" int zse_step_forward(const ZseStepModel* m, const ZseStepBuffers* b, void* kv, int64_t kv_layer_stride,
                                int block_size, int M, int decode, int num_seqs, int max_q_len, int n_logit_rows,
                                int attn_splits, void* stream, int* launches_out) {
  if (launches_out != nullptr) *launches_out = 0;
  if (M <= 0) return 0;
  if (!zse_step_supported(m, b) || M > b->max_tokens) return ZSE_ERR_SHAPE;
  Pass p{m, b, stream, M, 0, 0};
  const int H = m->hidden, hd = m->head_dim, nh = m->num_heads, nkv = m->num_kv_heads;
  const int qkv_ld = (nh + 2 * nkv) * hd;
  // blocks in one layer of the pool [layers][blocks][2][nkv][block_size][hd]
  const int64_t per_block = int64_t(2) * nkv * block_size * hd;
  const int kv_blocks = per_block > 0 ? int(kv_layer_stride / per_block) : 0;
  p.did(zse_embedding(m->embed, b->ids, b->residual, M, H, m->vocab_rows, m->embed_scale, b->status, stream));
  int planes = 0, slot = 0;
  for (int li = 0; li < m->num_layers && p.ok(); ++li) {
    const ZseStepLayer& L = m->layers[li];
    void* kv_layer = static_cast<char*>(kv) + size_t(li) * size_t(kv_layer_stride) * 2;
    p.add_norm(planes, L.ln1);
    if ((m->dec_mode & 2) && b->dec_ws != nullptr && m->rope_table != nullptr && L.qkv.kind == ZSE_STEP_W4 && M <= 64 &&
        hd == 128 && m->rotary_dim == 128 &&
        zse_gemm_w4_dec_supported(M, L.qkv.N, L.qkv.K, 3)) {
      // decode-sized pass: projection, bias, RoPE and the cache write in one kernel
      if (p.ok())
        p.did(zse_gemm_w4_dec_qkv_rope(L.qkv.data, b->xnorm, b->max_tokens, L.qkv.bias, b->qkv, qkv_ld, M, L.qkv.K, nh,
                                       nkv, kv_layer, block_size, b->positions, b->slots, m->rope_table,
                                       m->max_position, b->dec_ws, b->status, stream));
    } else if (M <= b->qkv_plane_rows && L.qkv.kind == ZSE_STEP_W4) {
      const int n_q = p.linear_partial(L.qkv, b->xnorm, b->qkv_planes, b->qkv_max_planes, b->max_tokens);
      if (p.ok())
        p.did(zse_rope_kv_write(b->qkv, kv_layer, b->positions, b->slots, m->inv_freq, M, nh, nkv, hd, m->rotary_dim,
                                block_size, b->qkv_planes, n_q, L.qkv.bias, stream));
    } else {
      p.linear(L.qkv, b->xnorm, b->qkv, qkv_ld, M);
      if (p.ok())
        p.did(zse_rope_kv_write(b->qkv, kv_layer, b->positions, b->slots, m->inv_freq, M, nh, nkv, hd, m->rotary_dim,
                                block_size, nullptr, 0, nullptr, stream));
    }
    if (!p.ok()) break;
    if (decode)
      p.did(zse_attn_decode(b->qkv, qkv_ld, kv_layer, b->block_tables, b->max_blocks, b->seq_lens, b->attn_out,
                            nh * hd, b->attn_scratch, num_seqs, nh, nkv, hd, block_size, attn_splits, m->scale, stream),
            attn_splits > 1 ? 2 : 1);
    else if (m->attn_tc && hd == 128 && kv_blocks > 0)
      p.did(zse_attn_prefill_tc(b->qkv, qkv_ld, M, kv_layer, kv_blocks, b->block_tables, b->max_blocks, b->cu_q,
                                b->q_pos0, b->attn_out, nh * hd, num_seqs, max_q_len, nh, nkv, hd, block_size, m->scale,
                                0, b->status, stream));
    else
      p.did(zse_attn_prefill(b->qkv, qkv_ld, kv_layer, b->block_tables, b->max_blocks, b->cu_q, b->q_pos0, b->attn_out,
                             nh * hd, num_seqs, max_q_len, nh, nkv, hd, block_size, m->scale, stream));
    planes = p.row_fused(L.o, b->attn_out, L.ln2, &slot) ? -1
                                                          : p.linear_partial(L.o, b->attn_out, b->partials,
                                                                             b->max_planes, b->max_tokens);
    p.add_norm(planes, L.ln2);
    if (!p.ok()) break;
    if (L.gate_up.kind == ZSE_STEP_W4 && (m->dec_mode & 1) && b->dec_ws != nullptr && M <= 64 && m->inter % 8 == 0 &&
        zse_gemm_w4_dec_supported(M, L.gate_up.N, L.gate_up.K, kEpiSwiGLU)) {
      p.did(zse_gemm_w4_dec(L.gate_up.data, b->xnorm, b->max_tokens, nullptr, b->act, M, L.gate_up.N, L.gate_up.K,
                            m->inter, kEpiSwiGLU, b->dec_ws, b->status, stream));
    } else if (L.gate_up.kind == ZSE_STEP_W4) {
      p.did(zse_gemm_w4(L.gate_up.data, b->xnorm, b->max_tokens, nullptr, b->act, M, L.gate_up.N, L.gate_up.K,
                        m->inter, kEpiSwiGLU, 0, b->status, stream));
    } else {
      p.did(zse_gemm_f16(L.gate_up.data, L.gate_up.N, b->xnorm, b->max_tokens, nullptr, b->gate_up_tmp, M, L.gate_up.N,
                         L.gate_up.K, L.gate_up.N, kEpiF16, 1, b->status, stream));
      if (p.ok()) p.did(zse_swiglu(b->gate_up_tmp, b->act, M, L.gate_up.N / 2, 0, stream));
    }
    const void* next_norm = li + 1 < m->num_layers ? m->layers[li + 1].ln1 : m->final_norm;
    planes = p.row_fused(L.down, b->act, next_norm, &slot) ? -1
                                                           : p.linear_partial(L.down, b->act, b->partials,
                                                                              b->max_planes, b->max_tokens);
  }
  p.add_norm(planes, m->final_norm);
  if (n_logit_rows > 0 && p.ok()) {
    p.did(zse_gather_rows_f16(b->xnorm, H, b->logit_rows, b->xsel, n_logit_rows, H, M, b->status, stream));
    if (p.ok()) {
      const ZseStepLinear& w = m->lm_head;
      if (w.kind == ZSE_STEP_W4)
        p.did(zse_gemm_w4(w.data, b->xsel, b->logits_rows_cap, w.bias, b->logits, n_logit_rows, w.N, w.K, b->logits_ld,
                          kEpiF16, 0, b->status, stream));
      else
        p.did(zse_gemm_f16(w.data, w.N, b->xsel, b->logits_rows_cap, w.bias, b->logits, n_logit_rows, w.N, w.K,
                           b->logits_ld, kEpiF16, 1, b->status, stream));
    }
  }
  if (launches_out != nullptr) *launches_out = p.launches;
  return p.rc;
}
