/*
 * CPU oracle for the flint attention hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's fp32 CPU attention
 * (src/ref/ref_model.cpp:45-61 RMSNorm + NEOX RoPE, :107-149 attention with the
 * learned sink), plus the integer maps of the GPU kernels (ring slot, window
 * start, split ranges, rollback rule) and the seeded input generator shared by
 * every test.  Nothing in the shipped library links, loads or calls this file:
 * it is the checker, used by the tests, by the smoke check and by the CPU
 * baseline leg of the benchmark.
 *
 * Parity pin: the attention functions here are compared, output for output,
 * with the unmodified reference RefModel compiled from its own sources and run
 * on a synthetic all-F32 GGUF (see ref_driver.cpp and tests/golden/).
 */
#ifndef FLINT_ATTN_ORACLE_H
#define FLINT_ATTN_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Shape constants of the one model the reference supports (src/metal/flint_config.h:10-31). */
enum {
    FO_N_HEAD = 32,
    FO_N_HEAD_KV = 4,
    FO_HEAD_DIM = 128,
    FO_GQA = 8,
    FO_Q_DIM = 4096,
    FO_KV_DIM = 512,
    FO_QKV_DIM = 5120,
    FO_N_SWA = 513,      /* window, current token included */
    FO_MAX_CHUNK = 512,
    FO_SWA_RING = 1024
};
#define FO_RMS_EPS 1e-6f
#define FO_ROPE_THETA 10000.0f

/* ---- seeded synthetic inputs ------------------------------------------------
 * Counter-based: element i of stream `stream` under `seed` does not depend on
 * how many elements are asked for, so any slice of any tensor can be
 * regenerated anywhere (needed to rebuild the K/V of a rolled-back range). */
void fo_gen_normal(uint64_t seed, uint64_t stream, uint64_t first, uint64_t n, float mean, float std, float *out);
uint64_t fo_gen_u64(uint64_t seed, uint64_t stream, uint64_t index);

/* fp16 / bf16 round trips (round to nearest even), in place. */
void fo_round_f16(float *x, uint64_t n);
void fo_round_bf16(float *x, uint64_t n);
void fo_f32_to_f16_bits(const float *x, uint16_t *out, uint64_t n);
void fo_f16_bits_to_f32(const uint16_t *x, float *out, uint64_t n);
void fo_f32_to_bf16_bits(const float *x, uint16_t *out, uint64_t n);
void fo_bf16_bits_to_f32(const uint16_t *x, float *out, uint64_t n);

/* ---- arithmetic of the path ------------------------------------------------- */
/* src/ref/ref_model.cpp:45-50 */
void fo_rmsnorm(const float *x, const float *w, float *y, int n, float eps);
/* src/ref/ref_model.cpp:53-61 */
void fo_rope_neox(float *x, int d, int pos, float theta);
/* 64 values theta^(-2i/128), the same powf call as fo_rope_neox. */
void fo_inv_freq(float theta, float *out64);

/* Norm (+RoPE) of the 32 q heads and 4 k heads of one token's raw qkv row
 * (src/ref/ref_model.cpp:112-121).  v is left untouched. */
void fo_qk_norm_rope(float *qkv_row, const float *q_norm, const float *k_norm, int pos, int has_rope);

/* One token's attention for all 32 heads (src/ref/ref_model.cpp:125-149).
 * q: [32][128] after norm/RoPE.  kc/vc: [pos+1][512] fp32, row j = position j.
 * att: [32][128].  n_threads > 1 spreads heads over OpenMP threads; the
 * arithmetic per head is unchanged. */
void fo_attend(const float *q, const float *kc, const float *vc, const float *sinks, int pos, int is_swa,
               float *att, int n_threads);

/* A whole layer, token by token from position p0 (how RefModel::forward drives
 * it): raw qkv [T][5120] -> att [T][4096].  kc/vc: caller-owned [p0+T][512]
 * fp32 caches whose first p0 rows are already filled.  round_kv_f16 != 0
 * rounds each new K (after norm/RoPE) and V through IEEE half before it is
 * stored and used, which is what the GPU kernels do (src/metal/fused.metal:285-293,
 * src/main.mm:274-275); 0 is the reference's own fp32 cache. */
void fo_layer_forward(const float *qkv, int T, int p0, const float *q_norm, const float *k_norm, const float *sinks,
                      int is_swa, int has_rope, int round_kv_f16, float *kc, float *vc, float *att, int n_threads);

/* Single-token attention over an fp16-valued cache given in the GPU layout of
 * one sequence: k16/v16 [4][n_slots][128] half bits.  The new token's raw
 * q/k/v come from qkv_row (5120 floats); its K/V are rounded to half, written
 * to slot(pos) and used.  att [32][128].  Used for the large decode configs,
 * where a whole-history fp32 replay would be too slow. */
void fo_decode_token_f16cache(const float *qkv_row, int pos, const float *q_norm, const float *k_norm,
                              const float *sinks, int is_swa, int has_rope, uint16_t *k16, uint16_t *v16,
                              int64_t n_slots, float *att, int n_threads);

/* Partial attention over keys [j0, j1) of an fp32 cache (no sink): per head
 * un-normalised acc[128], running max m and sum l, as the split-K kernels
 * produce them (src/metal/fused.metal:324-327).  part: [32][130]. */
void fo_attend_partial(const float *q, const float *kc, const float *vc, int j0, int j1, float *part);
/* src/metal/fused.metal:332-350: merge n_split partial records per head and add the sink once.
 * part: [32][n_split][130]; out [32][128]. */
void fo_combine(const float *part, int n_split, const float *sinks, float *out);

/* The reference's second CPU statement of this path, the one its own attention unit test compares the GPU with
 * (src/main.mm:253-305): everything in double -- RMSNorm, RoPE angles from pow/cos/sin in double, scores, a two-pass
 * softmax with the sink -- with K (after norm/RoPE) and V rounded through IEEE half as the caches hold them.  In the
 * reference a full-attention layer has no RoPE (src/main.mm:244,262); here the two flags stay separate.
 * qkv: raw rows [n][5120] of positions 0..n-1.  For each of the n_pos probe positions and n_heads probe heads the
 * attention output goes to out[(ip * n_heads + ih) * 128 ..] as double. */
void fo_attend_double_f16(const float *qkv, int n, const float *q_norm, const float *k_norm, const float *sinks,
                          int is_swa, int has_rope, const int32_t *probe_pos, int n_pos, const int32_t *probe_heads,
                          int n_heads, double *out);
/* Inputs of the kind that test draws, (rand() % 2001 - 1000) / 500 (src/main.mm:247): uniform on the grid
 * {-2, -1.998, ..., 2}, here from the seeded generator (rand() itself is platform-specific). */
void fo_gen_grid(uint64_t seed, uint64_t stream, uint64_t first, uint64_t n, float *out);

/* ---- the attention stack of the whole model (projections, residual, logits) ----------------------------------
 * src/ref/ref_model.cpp:74-92: y[r] = float(sum_i double(w[r][i]) * x[i]), rows r of w [n_rows][k]. */
void fo_matvec(const float *w, const float *x, float *y, int n_rows, int k, int n_threads);
/* RefModel::forward (src/ref/ref_model.cpp:95-197) for a model whose feed-forward weights are zero, token by token
 * from position 0: embedding row, per layer rmsnorm -> q/k/v matvecs -> QK norm (+RoPE) -> attention over the
 * un-rounded fp32 cache -> o-proj matvec -> residual add; then output_norm and the vocabulary matvec.  All weights
 * as fp32 arrays (whatever precision they were rounded to beforehand):
 *   embd [n_vocab][E]; per layer l: attn_norm [L][E], wq [L][4096][E], wk [L][512][E], wv [L][512][E],
 *   q_norm [L][128], k_norm [L][128], sinks [L][32], wo [L][E][4096]; out_norm [E]; w_out [n_vocab][E].
 * logits [n_tok][n_vocab] and hidden [n_tok][E] (the residual stream after the last layer) are written for every
 * token; either may be NULL. */
void fo_stack_forward(const float *embd, const float *attn_norm, const float *wq, const float *wk, const float *wv,
                      const float *q_norm, const float *k_norm, const float *sinks, const float *wo,
                      const int32_t *is_swa, const int32_t *has_rope, const float *out_norm, const float *w_out,
                      const int32_t *tokens, int n_tok, int n_layer, int n_embd, int n_vocab, float *logits,
                      float *hidden, int n_threads);

/* ---- integer maps (bit-exact items) ------------------------------------------ */
/* src/metal/fused.metal:269-274, prefill.metal:106 */
int32_t fo_slot(int32_t pos, int is_swa);
/* src/metal/fused.metal:265, ref_model.cpp:127 */
int32_t fo_k_begin(int32_t pos, int is_swa);
/* src/engine.mm:737-743: the reference's own split policy. */
void fo_ref_split_policy(int32_t pos, int is_swa, int32_t *keys_per_split, int32_t *n_split);
/* server/src/main.rs:96-100: position prefill restarts from after rolling back to p. */
int32_t fo_rollback_restart(int32_t cached_len, int32_t p);
/* Which position owns each ring slot after positions [0, n) were written: owner[1024], -1 = never written. */
void fo_ring_owners(int32_t n, int32_t *owner);

#ifdef __cplusplus
}
#endif
#endif
