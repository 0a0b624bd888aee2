// C ABI of libzse_b200.so.  Every function takes raw device pointers and a cudaStream_t (as void*), launches
// asynchronously on that stream and returns 0 or a negative ZSE_ERR_* code; nothing here allocates device memory
// unless its name says so.  A device-side failure (a bounded wait that ran out, an index check) is reported through
// the 16-byte status word the caller passes in (see zse_status_*).
#pragma once
#include <stdint.h>

#define ZSE_ERR_SHAPE (-1)
#define ZSE_ERR_ALIGN (-2)
#define ZSE_ERR_DRIVER (-3)
#define ZSE_ERR_LAUNCH (-4)
#define ZSE_ERR_LIMIT (-5)

#ifdef __cplusplus
extern "C" {
#endif

// ---- runtime.cu ---------------------------------------------------------------------------------------------
// Programmatic dependent launch for the kernels of the decode path (on by default; ZSE_PDL=0 switches it off).
void zse_set_pdl(int on);
int zse_get_pdl(void);

// ---- gemm.cu ------------------------------------------------------------------------------------------------
// epilogue: 0 = fp16 store (+bias), 1 = SwiGLU (N counts gate+up rows, output has N/2 columns), 2 = fp32 partial planes
int zse_gemm_w4(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M, int N, int K,
                int ldo, int epilogue, int k_split, void* status, void* stream);
int zse_gemm_w4_splits(int M, int N, int K, int k_split);
// the launcher's plan for a call: out4 = {tiles per wide CTA, K splits, cluster size, CTA shape: 0 wide, 1 narrow,
// -1 CUDA-core GEMV}
void zse_gemm_w4_plan(int M, int N, int K, int epilogue, int k_split, int sm_count, int* out4);
// ---- gemm_w4_dec.cu -----------------------------------------------------------------------------------------
// Decode-sized INT4 GEMM (M <= 64): one persistent CTA per SM over an even split of the weight stream.
// epilogue: 0 = fp16 store (+bias), 1 = SwiGLU, 2 = fp32 store.  `workspace`: zse_gemm_w4_dec_workspace_bytes bytes,
// zeroed once; one workspace serves the calls of ONE stream (calls that overlap on the GPU must not share it).
long long zse_gemm_w4_dec_workspace_bytes(int sm_count);
int zse_gemm_w4_dec_supported(int M, int N, int K, int epilogue);
int zse_gemm_w4_dec(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out, int M, int N,
                    int K, int ldo, int epilogue, void* workspace, void* status, void* stream);
// Fused QKV projection, head_dim 128, full rotary: bias + rotate-half RoPE (cos/sin table [max_position][64] of
// float2) + K/V rows into the paged cache [blocks][2][nkv][block_size][128]; qkv_out receives the rotated q heads.
int zse_gemm_w4_dec_qkv_rope(const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* qkv_out,
                             int ldo, int M, int K, int nh, int nkv, void* kv_layer, int block_size,
                             const void* positions_i32, const void* slots_i64, const void* cos_sin_f32x2,
                             int max_position, void* workspace, void* status, void* stream);
// the plan of a call: out2 = {CTAs, K segments per tile pair (0: the stream plan)}
void zse_gemm_w4_dec_plan(int N, int K, int epilogue, int sm_count, int* out2);
void zse_gemm_w4_dec_set_tuning(int min_steps, int max_split);

int zse_gemm_f16(const void* w, int w_rows_cap, const void* x, int x_rows_cap, const void* bias, void* out, int M,
                 int N, int K, int ldo, int epilogue, int k_split, void* status, void* stream);
int zse_gemm_f16_splits(int M, int N, int K, int k_split);

// ---- repack.cu ----------------------------------------------------------------------------------------------
// Row-major INT4 [N, K/2] + scales/zeros [N, K/128] -> tiled chunks.  interleave_rows > 0 builds a fused gate/up
// tensor: `packed` holds gate rows [0, interleave_rows) then up rows; output tile t = 64 gate rows + 64 up rows.
int64_t zse_w4_tiled_bytes(int N, int K);
int zse_repack_w4(const void* packed, const void* scales, const void* zeros, void* out_tiled, int N, int K,
                  int interleave_rows, void* stream);
int zse_dequant_w4(const void* packed, const void* scales, const void* zeros, void* out_f16, int64_t n_elements,
                   int group_size, void* stream);
int zse_dequant_w8(const void* q, const void* scales, void* out_f16, int64_t n_elements, int group_size, void* stream);
int zse_quantize_w4(const void* w_f16, void* packed, void* scales, void* zeros, int64_t n_groups, void* stream);

// ---- elementwise.cu -----------------------------------------------------------------------------------------
int zse_embedding(const void* table_f16, const void* ids_i32, void* out_f32, int M, int H, int vocab, float scale,
                  void* status, void* stream);
// residual[M,H] (fp32, in/out) += sum of n_partials fp32 planes (stride M*H) [+ add_f16]; out = rmsnorm(residual)*w
int zse_add_rmsnorm(void* residual, const void* partials, int n_partials, const void* add_f16, const void* weight,
                    void* out_f16, int M, int H, float eps, void* stream);
int zse_rmsnorm_f16(const void* x_f16, const void* weight, void* out_f16, int M, int H, float eps, void* stream);
// qkv fp16 [M, (nh+2nkv)*hd]; rotates q and k in place (rotate-half), writes k and v into the paged cache
// kv_layer: [num_blocks][2][nkv][block_size][hd] fp16; slot = block*block_size + offset, -1 = skip;
// inv_freq: fp32 [rotary_dim/2] (theta^(-2i/rotary_dim), with any rope scaling already applied by the host)
// planes != NULL: q/k/v are read as n_planes fp32 planes [n_planes][M][(nh+2nkv)*hd] plus bias_f16 (may be NULL)
// instead of from qkv, and qkv only receives the rotated q
int zse_rope_kv_write(void* qkv, void* kv_layer, const void* positions_i32, const void* slots_i64,
                      const void* inv_freq_f32, int M, int nh, int nkv, int hd, int rotary_dim, int block_size,
                      const void* planes_f32, int n_planes, const void* bias_f16, void* stream);
int zse_swiglu(const void* gate_up_f16, void* out_f16, int M, int I, int gelu, void* stream);
int zse_bias_add(void* x_f16, const void* bias_f16, int M, int N, void* stream);
// dst[r, :] = src[rows_i64[r], :] for r < n (fp16 rows of H elements, H and ld multiples of 8)
// Diagnostic: `ctas` CTAs read `bytes` of `buf` `repeats` times (16-byte loads past L1); the caller times the launch.
int zse_read_probe(const void* buf, long long bytes, int repeats, int ctas, void* sink_u32, void* stream);
int zse_gather_rows_f16(const void* src_f16, int ld, const void* rows_i64, void* dst_f16, int n, int H, int src_rows,
                        void* status, void* stream);

// ---- gemma.cu: Gemma-family layers ------------------------------------------------------------------------------
// qkv fp16 [M, ld]: q heads, k heads, v heads (no v columns when k_is_v: V is then the raw k projection).  Per head:
// RMSNorm (q, k with the given fp16 weights [hd], NULL = none; v without weight when norm_v), RoPE on pairs
// (i, i + hd/2) with freqs_f32[i] (0 = pair not rotated), q written back in place, k and v into the cache of this
// layer: element (block, half, kv_head, offset, d) at block*blk_stride + half*half_stride + (kv_head*block_size +
// offset)*hd + d.
int zse_headnorm_rope_kv_write(void* qkv, int ld, void* kv_layer, int64_t blk_stride, int64_t half_stride,
                               const void* positions_i32, const void* slots_i64, const void* freqs_f32,
                               const void* q_norm_w, const void* k_norm_w, int norm_v, int k_is_v, float eps, int M,
                               int nh, int nkv, int hd, int block_size, void* stream);
// paged attention for any even head_dim <= 512.  Decode: cu_q = q_pos0 = NULL, query t belongs to sequence t at
// position seq_lens[t]-1.  Prefill: queries packed by cu_q, first query of sequence s at position q_pos0[s].
// softcap > 0: scores = softcap*tanh(scores/softcap); window > 0: only the last `window` positions are seen.
int zse_attn_generic(const void* q, int ldq, const void* kv_layer, int64_t blk_stride, int64_t half_stride,
                     const void* block_tables_i32, int max_blocks, const void* seq_lens_i32, const void* cu_q_i32,
                     const void* q_pos0_i32, int num_seqs, void* out_f16, int ldo, int T, int nh, int nkv, int hd,
                     int block_size, float scale, float softcap, int window, void* stream);
// residual = (residual + RMSNorm(x)*w_post) * scalar_f16[0] (scalar may be NULL); out = RMSNorm(residual)*w_next
// (out may be NULL)
int zse_norm_add_rmsnorm(const void* x_f16, const void* w_post, void* residual_f32, const void* scalar_f16,
                         const void* w_next, void* out_f16, int M, int H, float eps, void* stream);
int zse_softcap_f16(void* x_f16, int ld, int M, int V, float cap, void* stream);

// ---- attention.cu -------------------------------------------------------------------------------------------
int64_t zse_attn_decode_scratch_floats(int num_seqs, int nh, int hd, int max_splits);
int zse_attn_decode(const void* q, int ldq, const void* kv_layer, const void* block_tables_i32, int max_blocks,
                    const void* seq_lens_i32, void* out_f16, int ldo, void* scratch_f32, int num_seqs, int nh, int nkv,
                    int hd, int block_size, int num_splits, float scale, void* stream);
// causal attention of `total_q` query tokens (several sequences packed) over the paged cache.
// cu_q: [num_seqs+1] prefix offsets of query tokens; q_pos0[s]: cache position of the first query token of seq s.
int zse_attn_prefill(const void* q, int ldq, const void* kv_layer, const void* block_tables_i32, int max_blocks,
                     const void* cu_q_i32, const void* q_pos0_i32, void* out_f16, int ldo, int num_seqs, int max_q_len,
                     int nh, int nkv, int hd, int block_size, float scale, void* stream);
// The same on the tcgen05 tensor cores (attention_tc.cu): head_dim 128, contiguous cache layer of `num_blocks` blocks,
// `total_rows` rows in q.  ZSE_ERR_SHAPE for shapes it does not cover.
int zse_attn_prefill_tc(const void* q, int ldq, int total_rows, const void* kv_layer, int num_blocks,
                        const void* block_tables, int max_blocks, const void* cu_q, const void* q_pos0, void* out,
                        int ldo, int num_seqs, int max_q_len, int nh, int nkv, int hd, int block_size, float scale,
                        int variant, void* status, void* stream);

// the same kernels with an explicit cache addressing (element (block, half, kv_head, offset, d) at block*blk_stride +
// half*half_stride + (kv_head*block_size + offset)*hd + d; strides in elements, multiples of 8), soft-capped scores
// (softcap > 0: cap*tanh(score/cap)) and a sliding window (window > 0: only the last `window` positions are seen).
// head_dim 64, 128 or 256.
int zse_attn_decode_ext(const void* q, int ldq, const void* kv_layer, int64_t blk_stride, int64_t half_stride,
                        const void* block_tables_i32, int max_blocks, const void* seq_lens_i32, void* out_f16, int ldo,
                        void* scratch_f32, int num_seqs, int nh, int nkv, int hd, int block_size, int num_splits,
                        float scale, float softcap, int window, void* stream);
int zse_attn_prefill_ext(const void* q, int ldq, const void* kv_layer, int64_t blk_stride, int64_t half_stride,
                         const void* block_tables_i32, int max_blocks, const void* cu_q_i32, const void* q_pos0_i32,
                         void* out_f16, int ldo, int num_seqs, int max_q_len, int nh, int nkv, int hd, int block_size,
                         float scale, float softcap, int window, void* stream);

// ---- sampling.cu --------------------------------------------------------------------------------------------
int zse_argmax(const void* logits_f16, int ld, void* out_i32, int M, int V, void* stream);
int zse_sample(const void* logits_f16, int ld, void* out_i32, int M, int V, const void* temperature_f32,
               const void* top_k_i32, const void* top_p_f32, const void* seeds_u64, uint64_t step, void* stream);
// sparse form: entry i scales logits[rows[i], tokens[i]] by penalty[rows[i]]^(1+log2(counts[i]))
int zse_apply_repetition_penalty(void* logits_f16, int ld, const void* rows_i32, const void* tokens_i32,
                                 const void* counts_i32, int n, const void* penalty_f32, int V, void* stream);

// ---- lora.cu ------------------------------------------------------------------------------------------------
// y[t, :] += scale[a] * B[a] (A[a] x[t, :]) with a = adapter_ids[t] (-1 = none); A: [n_adapters][r][K], B: [n_adapters][N][r]
int zse_lora_shrink(const void* x_f16, int ldx, const void* a_f16, const void* adapter_ids_i32, void* tmp_f32, int M,
                    int K, int rank, void* stream);
int zse_lora_expand(const void* tmp_f32, const void* b_f16, const void* adapter_ids_i32, const void* scales_f32,
                    void* y_f16, int ldy, int M, int N, int rank, void* stream);
// shrink + expand in one launch, the activation row read once per token (rank even, <= 64)
int zse_lora_apply(const void* x, int ldx, const void* a, const void* b, const void* ids, const void* scales, void* y,
                   int ldy, int M, int K, int N, int rank, void* stream);

// ---- comm.cu ------------------------------------------------------------------------------------------------
// Tensor-parallel context: peer-mapped symmetric buffers of every rank (row data [2][m_cap][H] fp16, flags
// [2][tp][m_cap] u32, exchange words [2][tp][m_cap] u64 + flags), optional multicast view of the row data.
void* zse_tp_ctx_create(int tp, int rank, int m_cap, int H, const uint64_t* data_ptrs, const uint64_t* flag_ptrs,
                        uint64_t mc_data, const uint64_t* xchg_ptrs, const uint64_t* xflag_ptrs);
void zse_tp_ctx_destroy(void* ctx);
int zse_tp_reduce_add_rmsnorm(void* ctx, void* residual, const void* partials, int n_planes, const void* weight,
                              void* out, int M, float eps, int slot, int use_multimem, void* status,
                              void* stream);
int zse_tp_reduce_add_rmsnorm_emulated(void* ctx, const uint64_t* residuals, const uint64_t* partials, int n_planes,
                                       const void* weight, const uint64_t* outs, int M, float eps,
                                       int slot, void* status, void* stream);
// Two-shot form for many rows (prefill): reduce-scatter by rows (row r is reduced by rank r % tp, which also keeps the
// only current copy of the fp32 residual row) + all-gather of the normalised rows, in one kernel.
int zse_tp_reduce_scatter_add_rmsnorm(void* ctx, void* residual, const void* partials, int n_planes,
                                      const void* weight, void* out, int M, float eps, int slot, int use_multimem,
                                      void* status, void* stream);
int zse_tp_reduce_scatter_add_rmsnorm_emulated(void* ctx, const uint64_t* residuals, const uint64_t* partials,
                                               int n_planes, const void* weight, const uint64_t* outs, int M,
                                               float eps, int slot, void* status, void* stream);
// Push exchange: the row-parallel INT4 GEMM sends its fp16 partial rows to every rank's inbox from its own epilogue
// (multimem.st through NVSwitch or one store per peer) and counts its CTAs in; the consumer waits for the counters,
// adds the tp rows of its own inbox in rank order, adds the residual and applies RMSNorm.
//   inbox_ptrs[r]  : rank r's inbox [2][tp][push_m_cap][H] fp16 as mapped into this process (symmetric memory)
//   arrive_ptrs[r] : rank r's counters [2][tp] u32 (symmetric memory, zero at start)
//   state_ptrs[r]  : 4 u32 of ordinary device memory of rank r (zero at start); only the own rank's is needed
int zse_tp_ctx_set_push(void* ctx, int push_m_cap, const uint64_t* inbox_ptrs, uint64_t mc_inbox,
                        const uint64_t* arrive_ptrs, uint64_t mc_arrive, const uint64_t* state_ptrs);
// returns the number of CTAs launched (what the consumer waits for from every rank) or a negative error
int zse_tp_gemm_w4_push(void* ctx, const void* w_tiled, const void* x, int x_rows_cap, int M, int N, int K, int slot,
                        int use_multimem, int rank_override, void* status, void* stream);
// Decode-sized passes (M <= 64): row-parallel projection (INT4 or INT8 tiles), the exchange of the partial rows, the
// residual add and the next RMSNorm in ONE kernel (gemm_w4_dec.cu).  tp = 1 contexts work too (nothing to exchange).
int zse_tp_gemm_dec_allreduce_norm(void* ctx, const void* w_tiled, int int8_weights, const void* x, int x_rows_cap,
                                   int M, int N, int K, int slot, int use_multimem, int rank_override, void* residual,
                                   const void* norm_w, void* xnorm, float eps, void* workspace, void* status,
                                   void* stream);
int zse_tp_sum_add_rmsnorm(void* ctx, void* residual, const void* weight, void* out, int M, float eps, int slot,
                           int expected_add, void* status, void* stream);
int zse_tp_sum_add_rmsnorm_emulated(void* ctx, const uint64_t* residuals, const void* weight, const uint64_t* outs,
                                    int M, float eps, int slot, int expected_add, void* status, void* stream);
// Sequence-parallel exchange for passes of more than 64 rows (prefill): token rows are owned in blocks of 64
// (block b -> rank b % tp).  The row-parallel GEMM scatters its fp16 partial tiles to the owners from its epilogue;
// the owner adds, applies residual + RMSNorm and stores the row into the gathered buffer of every rank; GEMMs that
// read the gathered buffer wait, in their prologue, for the row blocks of their own token tile.
//   inbox_ptrs[r]  : rank r's inbox [2][tp][own_cap][H] fp16   arrive_ptrs[r] : counters [2][tp][nblk_cap] u32
//   xg_ptrs[r]     : gathered activations [nblk_cap * 64][H]    gflag_ptrs[r]  : flags [nblk_cap] u32
//   state_ptrs[r]  : 4 + nblk_cap u32 of ordinary device memory of rank r (all zero at start)
int zse_tp_ctx_set_sp(void* ctx, int own_cap, int nblk_cap, const uint64_t* inbox_ptrs, const uint64_t* arrive_ptrs,
                      const uint64_t* xg_ptrs, uint64_t mc_xg, const uint64_t* gflag_ptrs, const uint64_t* state_ptrs);
int zse_tp_gemm_w4_scatter(void* ctx, const void* w_tiled, const void* x, int x_rows_cap, int M, int N, int K,
                           int slot, int rank_override, void* status, void* stream);
int zse_tp_gemm_w4_gathered(void* ctx, const void* w_tiled, const void* x, int x_rows_cap, const void* bias, void* out,
                            int M, int N, int K, int ldo, int epilogue, int k_split, int rank_override, void* status,
                            void* stream);
int zse_tp_sp_sum_norm_gather(void* ctx, void* residual, const void* weight, int M, float eps, int slot,
                              int use_multimem, void* status, void* stream);
int zse_tp_sp_sum_norm_gather_emulated(void* ctx, const uint64_t* residuals, const void* weight, int M, float eps,
                                       int slot, void* status, void* stream);
int zse_tp_sp_wait(void* ctx, int M, int rank_override, void* status, void* stream);
// All-gather of vocabulary-sharded logits rows over NVLink (peer stores + per-row flags): buf_ptrs[r] = rank r's gathered
// rows [2][rows_cap][tp * width] fp16, flag_ptrs[r] = its flags [2][tp][rows_cap] u32, both symmetric memory.
int zse_tp_ctx_set_gather(void* ctx, int rows_cap, int width, const uint64_t* buf_ptrs, const uint64_t* flag_ptrs);
int zse_tp_gather_rows(void* ctx, const void* logits, int ld, int M, int slot, void* status, void* stream);
int zse_tp_gather_rows_emulated(void* ctx, const uint64_t* logits, int ld, int M, int slot, void* status, void* stream);
int zse_tp_argmax(void* ctx, const void* logits, int ld, void* out, int M, int V_local, int vocab_stride,
                  int slot, void* status, void* stream);
int zse_tp_argmax_emulated(void* ctx, const uint64_t* logits, int ld, const uint64_t* outs, int M, int V_local,
                           int vocab_stride, int slot, void* status, void* stream);

// ---- runtime.cu ---------------------------------------------------------------------------------------------
int zse_status_read(const void* status_dev, uint32_t* out4);   // synchronous 16-byte copy
int zse_device_info(int* sm_count, int* cc_major, int* cc_minor, int64_t* total_mem, int64_t* free_mem);
const char* zse_build_info(void);

#ifdef __cplusplus
}
#endif
