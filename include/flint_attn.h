/*
 * flint_attn -- C ABI of the B200 (sm_100a) attention hot path of flint-mac.
 *
 * Shape and conventions follow the reference's engine interface, src/capi.h:10-37:
 * an opaque handle created by *_open and freed only by *_close; `err` is a
 * caller-owned buffer (may be NULL) that receives a NUL-terminated, truncated
 * message; int32 status returns are 0 on success and -1 on failure; no C++
 * exception crosses the boundary; a handle is single-owner and NOT thread-safe,
 * the caller serialises calls (src/capi.h:1).  Host-buffer entry points are
 * synchronous like the reference's (src/engine.mm:930); the *_dev variants take
 * device pointers and a CUDA stream and return after enqueueing.
 *
 * What it replaces inside the reference engine: the two attention call sites,
 *   decode : k_attn_dec + k_attn_combine     src/engine.mm:735-766, src/metal/fused.metal:254-350
 *   prefill: k_qk_prefill + k_attn_prefill   src/engine.mm:1087-1104, src/metal/prefill.metal:100-266
 * with the per-layer K/V caches of src/engine.mm:509-511 held by this library.
 *
 * Fixed shapes (src/metal/flint_config.h:10-31): 32 query heads, 4 KV heads, head dim 128,
 * sliding window 513 keys (current token included), 1024-slot ring per SWA layer.
 * One token's projections are passed as the reference's packed row
 *   qkv[5120] = q[32][128] | k[4][128] | v[4][128]          (src/metal/fused.metal:211)
 * before QK RMSNorm / RoPE; attention output rows are [32][128] = 4096 values.
 */
#ifndef FLINT_ATTN_H
#define FLINT_ATTN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct flint_attn flint_attn;

/* Element types of the qkv input rows and of the attention output rows.  Row buffers start on a 16-byte boundary
 * (any device allocation does; so does every row of one, a row being 10240 or 20480 bytes). */
enum { FLINT_ATTN_F32 = 0, FLINT_ATTN_BF16 = 1 };

enum {
    FLINT_ATTN_N_HEAD = 32,
    FLINT_ATTN_N_HEAD_KV = 4,
    FLINT_ATTN_HEAD_DIM = 128,
    FLINT_ATTN_QKV_DIM = 5120,
    FLINT_ATTN_OUT_DIM = 4096,
    FLINT_ATTN_PARTIAL_DIM = 130 /* acc[128], m, l  (src/metal/fused.metal:324-327) */
};

/* Counterpart of flint_config (src/capi.h:12-17): what the engine needs to know to allocate its KV caches. */
typedef struct {
    int32_t device;                /* CUDA device ordinal this handle lives on */
    int32_t n_layers;              /* attention layers held */
    const int32_t *layer_is_swa;   /* [n_layers] 1: 513-key window + 1024-slot ring; 0: full context (n_ctx slots) */
    const int32_t *layer_has_rope; /* [n_layers] 1: NEOX RoPE on q and k (src/ref/ref_model.h:18 keeps both flags) */
    int32_t max_seqs;              /* independent sequences resident on this device */
    int32_t n_ctx;                 /* context length per sequence (src/capi.h:16) */
    int32_t kv_rank;               /* KV-range sharding of full layers over devices: this shard ... */
    int32_t kv_ranks;              /* ... of this many (0 or 1: not sharded) */
    int32_t kv_pages;              /* 0: every sequence owns n_ctx slots per full layer (src/engine.mm:509-511).
                                      > 0: full layers keep K/V in a pool of this many 64-key pages per layer, handed to
                                      sequences on demand through a block table (see flint_attn_seq_release) */
} flint_attn_config;

/* src/capi.h:20-21. NULL + message on failure. */
flint_attn *flint_attn_open(const flint_attn_config *cfg, char *err, int32_t err_len);
void flint_attn_close(flint_attn *a);

/* src/capi.h:23,25 (per sequence here: the reference is single-session). */
int32_t flint_attn_n_ctx(const flint_attn *a);
int32_t flint_attn_pos(const flint_attn *a, int32_t seq);

/* src/capi.h:27-29, src/engine.h:60: move the sequence back to `pos` (<= current).  O(1); caches are not
 * touched.  -1 if pos < 0 or pos > current (src/capi.mm:52-56).  After rolling back more than 511 tokens the
 * caller must prefill again from max(0, pos-512) for the SWA rings to be right (server/src/main.rs:96-100);
 * flint_attn_rollback_restart gives that position. */
int32_t flint_attn_truncate(flint_attn *a, int32_t seq, int32_t pos);
int32_t flint_attn_rollback_restart(int32_t cached_len, int32_t pos);

/* Engine::step / Engine::prefill advance the position once per token after ALL layers ran
 * (src/engine.mm:936, :1248).  Attention calls below read the position and do not move it. */
int32_t flint_attn_advance(flint_attn *a, int32_t n, const int32_t *seqs, int32_t n_tokens);

/* Per-layer learned parameters: blk.N.attn_q_norm / attn_k_norm [128], attn_sinks [32], fp32
 * (bound at src/engine.mm:747-749).  Host pointers; copied. */
int32_t flint_attn_set_layer(flint_attn *a, int32_t layer, const float *q_norm, const float *k_norm,
                             const float *sinks, char *err, int32_t err_len);

/* ---- decode: one new token for each of n sequences ---------------------------------------------
 * Replaces k_attn_dec(args, qkv, q_norm, k_norm, sinks, k_cache, v_cache, out, partial) and k_attn_combine
 * (src/metal/fused.metal:254-259, 332-334).  For sequence seqs[i] at position p = flint_attn_pos(seqs[i]):
 * RMSNorm(+RoPE at p) of row i's q and k, K/V of the token rounded to half and written to slot p (p & 1023 on
 * SWA layers), softmax over cached keys [max(0,p-512) or 0, p) plus the token itself plus the head's sink,
 * split over the key range inside the GPU and merged.  qkv: [n][5120]; out: [n][4096]. */
int32_t flint_attn_decode(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs, const void *qkv,
                          int32_t qkv_dtype, void *out, int32_t out_dtype, char *err, int32_t err_len);
int32_t flint_attn_decode_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs, const void *qkv_dev,
                              int32_t qkv_dtype, void *out_dev, int32_t out_dtype, void *cuda_stream, char *err,
                              int32_t err_len);

/* KV-range sharded decode (kv_ranks > 1; full layers): this device's keys only, no sink.  partial_dev:
 * [n][32][130] fp32 = un-normalised acc[128], max m (natural-log units), sum l per head -- the record of
 * src/metal/fused.metal:324-327.  The shard that owns position p folds and stores the new token. */
int32_t flint_attn_decode_partial_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs,
                                      const void *qkv_dev, int32_t qkv_dtype, float *partial_dev, void *cuda_stream,
                                      char *err, int32_t err_len);
/* src/metal/fused.metal:332-350 over gathered shards: partials_dev [n_parts][n][32][130] -> out [n][4096];
 * the sink enters here, once. */
int32_t flint_attn_combine_dev(flint_attn *a, int32_t layer, int32_t n, int32_t n_parts, const float *partials_dev,
                               void *out_dev, int32_t out_dtype, void *cuda_stream, char *err, int32_t err_len);

/* ---- KV-range sharded decode with the exchange inside the kernels (GPUs of one node, peer access) ----
 * No counterpart in the reference (one device).  Instead of decode_partial + an all-gather by a library + combine,
 * the decode kernel itself stores each finished record into a gather buffer in EVERY rank's memory (plain peer
 * stores over NVLink) and the last group of the launch publishes the step number in every rank's flag word; the
 * combine kernel waits (bounded, about a second) on its own rank's flag words and merges records that are by then
 * local.  Per step every rank calls post, then combine, on one stream; records are double-buffered by step parity.
 *
 *   xchg_create        allocates this rank's buffer for batches up to n_max tokens and returns its CUDA IPC handle
 *                      (FLINT_ATTN_IPC_HANDLE_BYTES bytes; ipc_handle_out may be NULL inside one process).
 *   xchg_connect       opens the other ranks' buffers: ipc_handles = kv_ranks handles in rank order (own one ignored).
 *   xchg_connect_local same for handles that live in ONE process: peer_bases[r] = flint_attn_xchg_base(handle r).
 *   decode_xchg_post   = decode_partial_dev, records to every rank.  Full layers only.
 *   combine_xchg       = combine_dev over the records of the step just posted.  A wait that ran out makes the next
 *                      flint_attn_check fail; the output of that call is then undefined.
 * Kernels of two ranks that share ONE GPU must not wait on one another: there, post for every rank before any
 * combine. */
enum { FLINT_ATTN_IPC_HANDLE_BYTES = 64 };
int32_t flint_attn_xchg_create(flint_attn *a, int32_t n_max, void *ipc_handle_out, char *err, int32_t err_len);
int32_t flint_attn_xchg_connect(flint_attn *a, const void *ipc_handles, char *err, int32_t err_len);
void *flint_attn_xchg_base(flint_attn *a);
int32_t flint_attn_xchg_connect_local(flint_attn *a, void *const *peer_bases, char *err, int32_t err_len);
int32_t flint_attn_decode_xchg_post_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs,
                                        const void *qkv_dev, int32_t qkv_dtype, void *cuda_stream, char *err,
                                        int32_t err_len);
int32_t flint_attn_combine_xchg_dev(flint_attn *a, int32_t layer, int32_t n, void *out_dev, int32_t out_dtype,
                                    void *cuda_stream, char *err, int32_t err_len);

/* ---- prefill: n_tok tokens of one sequence from its current position -----------------------------
 * Replaces the chunk loop k_qk_prefill + k_attn_prefill (src/engine.mm:1080-1104, src/metal/prefill.metal:100-266):
 * norm(+RoPE at p0+t), K/V to the cache (ring slot (p0+t) & 1023 on SWA layers), causal + window + sink flash
 * attention.  qkv: [n_tok][5120]; out: [n_tok][4096]. */
int32_t flint_attn_prefill(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, const void *qkv,
                           int32_t qkv_dtype, void *out, int32_t out_dtype, char *err, int32_t err_len);
int32_t flint_attn_prefill_dev(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, const void *qkv_dev,
                               int32_t qkv_dtype, void *out_dev, int32_t out_dtype, void *cuda_stream, char *err,
                               int32_t err_len);

/* ---- context-parallel prefill: a full layer whose key range is sharded over devices (kv_ranks > 1) -------------
 * The reference prefills on one device (its own note on the cost of long full-attention prompts: docs/DEVLOG.md:192).
 * Here every rank gets the same n_tok rows; each stores the K/V of the positions in its own range, attends all n_tok
 * queries to the keys it holds and returns a partial: un-normalised fp32 rows partial_o [n_tok][4096] and, per
 * (token, head), the pair (m in base-2 units, l) in partial_ml [n_tok][32][2]; the rank that holds position 0 adds
 * the sink.  After an all-gather of both arrays (rank-major), prefill_combine merges them by log-sum-exp
 * (src/metal/fused.metal:332-350 applied to prefill rows).  Sliding-window layers of such a handle are replicated
 * and use flint_attn_prefill_dev on every rank.  Works on an unsharded handle too (one part). */
int32_t flint_attn_prefill_partial_dev(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, const void *qkv_dev,
                                       int32_t qkv_dtype, float *partial_o_dev, float *partial_ml_dev, void *cuda_stream,
                                       char *err, int32_t err_len);
int32_t flint_attn_prefill_combine_dev(flint_attn *a, int32_t n_tok, int32_t n_parts, const float *partials_o_dev,
                                       const float *partials_ml_dev, void *out_dev, int32_t out_dtype, void *cuda_stream,
                                       char *err, int32_t err_len);

/* ---- the attention block with its projections ---------------------------------------------------------
 * The steps either side of attention in the reference engine: the q/k/v matvecs on the attn_norm-ed residual stream
 * (src/engine.mm:728-732; fused form k_qkv, src/metal/fused.metal:215-231) and the o-proj matvec with the residual
 * add (src/engine.mm:811; k_mv_res, src/metal/fused.metal:357-379).  The reference's weights are quantised; here
 * they are dense bf16 rows with the input dimension contiguous (the GGUF layout).  set_projections copies host
 * arrays: attn_norm fp32 [n_embd], wq [4096][n_embd], wk [512][n_embd], wv [512][n_embd], wo [n_embd][4096] as bf16
 * bits; n_embd a multiple of 256.
 *   decode_block : x_dev fp32 [n][n_embd], one new token for each of n sequences, updated in place:
 *                  x += W_o . attention(W_qkv . rmsnorm(x, attn_norm))     (src/ref/ref_model.cpp:108-151)
 *   prefill_block: the same for n_tok tokens of one sequence from its current position.
 * The q|k|v rows and the attention rows never leave the device (scratch of the handle).  Like the attention calls,
 * these read the position and do not move it (flint_attn_advance after all layers). */
int32_t flint_attn_set_projections(flint_attn *a, int32_t layer, int32_t n_embd, const float *attn_norm,
                                   const uint16_t *wq, const uint16_t *wk, const uint16_t *wv, const uint16_t *wo,
                                   char *err, int32_t err_len);
int32_t flint_attn_decode_block_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs, float *x_dev,
                                    void *cuda_stream, char *err, int32_t err_len);
int32_t flint_attn_prefill_block_dev(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, float *x_dev,
                                     void *cuda_stream, char *err, int32_t err_len);
/* The projection kernel by itself (the reference's matvec, src/ref/ref_model.cpp:74-92, with an optional RMSNorm of
 * the input rows folded in): out_dev fp32 [n][n_rows_w] = W . norm?(x), W = w_dev bf16 [n_rows_w][k] on the device,
 * x_dev fp32 [n][k], norm_w_dev fp32 [k] or NULL.  n_rows_w a multiple of 128, k a multiple of 256. */
int32_t flint_attn_project_dev(flint_attn *a, const uint16_t *w_dev, int32_t n_rows_w, int32_t k, const float *x_dev,
                               int32_t n, const float *norm_w_dev, float *out_dev, void *cuda_stream, char *err,
                               int32_t err_len);

/* Wait for everything this handle enqueued and report an asynchronous failure of the *_dev calls (a CUDA error,
 * or a kernel whose bounded wait ran out), in the way the reference turns cb.error into an exception after
 * waitUntilCompleted (src/engine.mm:930-932).  A device-side error is reported by one call and cleared. */
int32_t flint_attn_check(flint_attn *a, char *err, int32_t err_len);

/* ---- cache access for tests and cache pre-loading (counterpart of the Engine::debug_* hooks, src/engine.h:37-47)
 * Cache layout on the device, per layer: K and V separately, half [max_seqs][4][n_slots][128], n_slots = 1024
 * (SWA) or the shard's share of n_ctx (full).  k/v host arrays here: [4][n][128] half bits for slots
 * [slot0, slot0+n) of one sequence. */
int32_t flint_attn_n_slots(const flint_attn *a, int32_t layer);
int32_t flint_attn_read_kv(flint_attn *a, int32_t layer, int32_t seq, int32_t slot0, int32_t n, uint16_t *k,
                           uint16_t *v, char *err, int32_t err_len);
int32_t flint_attn_write_kv(flint_attn *a, int32_t layer, int32_t seq, int32_t slot0, int32_t n, const uint16_t *k,
                            const uint16_t *v, char *err, int32_t err_len);
/* Device addresses of a layer's K (which = 0) or V (1) cache, for zero-copy fills by a co-resident producer (the
 * page pool [kv_pages][4][64][128] of a paged layer). */
void *flint_attn_kv_dev(flint_attn *a, int32_t layer, int32_t which);
/* Declare that a sequence's caches already hold `pos` tokens (after flint_attn_write_kv / a device-side fill). */
int32_t flint_attn_set_pos(flint_attn *a, int32_t seq, int32_t pos);

/* ---- paged KV cache: sequences that join and leave ------------------------------------------------------
 * No counterpart in the reference, which serves one session from one contiguous cache (src/engine.mm:509-511,
 * server/src/main.rs:84).  With kv_pages > 0 a full-attention layer's cache is a pool of 64-key pages (one decode
 * tile each) shared by all max_seqs sequence slots; a sequence takes a page whenever its position enters a new
 * 64-key block (in decode, prefill or flint_attn_write_kv; the call fails with "KV page pool exhausted" and changes
 * nothing when none is free) and keeps its pages across flint_attn_truncate.  Sliding-window layers keep their
 * 1024-slot ring per sequence slot.  A serving loop admits a request into a free slot, runs it, and retires it:
 *   flint_attn_seq_release   position back to 0 and every page of the slot back to the pool.  Pages are reused by later
 *                            launches: call it once the sequence's last launch is enqueued, and keep all launches of a
 *                            handle on one stream (or synchronise) so that reuse stays ordered behind earlier readers.
 *   flint_attn_pages_free    pages currently free (-1 when the handle is not paged).
 * Results are the same as with contiguous caches; only where K/V rows live differs. */
int32_t flint_attn_seq_release(flint_attn *a, int32_t seq);
int32_t flint_attn_pages_free(const flint_attn *a);

/* ---- host-side planning, exposed for tests (no GPU needed) -----------------------------------------
 * The split-K work list the decode launch would use for n tokens at positions pos[]: one record of 8 int32 per
 * work item = { token, kv_head, j0, j1, fold_new_token, split, n_split, first_partial }.  Cached keys [j0, j1)
 * of the items of one (token, kv_head) tile [k_begin, pos) clipped to [kv_lo, kv_hi) exactly once; exactly one
 * item per (token, kv_head) has fold_new_token = 1 when kv_lo <= pos < kv_hi.  Own policy (the reference's,
 * src/engine.mm:742-743, is tuned for 32 splits on an M5).  Returns the item count, or -1 if cap is too small. */
int32_t flint_attn_plan_decode(int32_t n, const int32_t *pos, int32_t is_swa, int32_t kv_lo, int32_t kv_hi,
                               int32_t target_items, int32_t *items, int32_t cap);
/* Tuning knob: work items the planner aims for per launch (default: one wave of 2 CTAs on every SM). */
int32_t flint_attn_set_target_items(flint_attn *a, int32_t target_items);
/* Number of kernel launches this handle has enqueued so far. */
int64_t flint_attn_launch_count(const flint_attn *a);
/* Device timing of the attention launches alone, in the role of the reference's per-dispatch GPU timestamps
 * (Engine::enable_profiling / last_profile, src/engine.h:49-51): while on, every decode / prefill call is bracketed
 * by CUDA events on its stream.  flint_attn_kernel_ms waits for them, returns the summed milliseconds and the
 * number of bracketed calls since the last query, and starts over. */
int32_t flint_attn_set_timing(flint_attn *a, int32_t on);
double flint_attn_kernel_ms(flint_attn *a, int64_t *n_timed);

/* ---- decode without any allocation -----------------------------------------------------------------
 * No counterpart in the reference (whose engine allocates what it needs, src/engine.mm:509-521); added for
 * hosts that cannot allocate device memory when they need attention: a server whose own arena already owns the
 * GPU (the KV caches live there), a plug-in inside a framework that owns the allocator, or a latency-critical
 * section where a device allocation's implicit synchronisation is not acceptable.  The handle-based calls above
 * allocate (caches at open; scratch and staging on demand); this one calls no cudaMalloc / cudaFree /
 * cudaMallocHost and uses no handle.  Same kernel, same planner, same kernel variants and same arithmetic as
 * flint_attn_decode_dev.  "Allocates nothing" is about CUDA memory: the planner keeps its work list in
 * thread-local host vectors that grow on the host heap the first time a thread plans a batch of a given size.
 *
 * The caller owns and passes everything as device pointers: qkv rows [n][5120], out rows [n][4096], the K and V
 * caches of the n sequences, half [n][4][n_slots][128] (row i of the batch uses cache i; n_slots = 1024 on a
 * sliding-window layer, the context length otherwise), q_norm/k_norm [128] and sinks [32] in fp32.  pos is a
 * HOST array of the n token positions.  What the kernel needs beyond that (work list, split-K partial records,
 * arrival counters, RoPE table) sits in one fixed array inside the library image, about 10 MiB on every GPU that
 * loads the library, held until the process exits.  Limits: n <= FLINT_ATTN_NOALLOC_MAX_TOKENS and a split-K work
 * list of at most FLINT_ATTN_NOALLOC_MAX_ITEMS items; beyond either the call fails with a message and does nothing.
 *
 * The first call on each device resolves the array's device address, fills the RoPE table and clears the
 * counters with blocking operations on the default stream: make that first call before any stream capture begins.
 * A work list of up to 640 items travels in the kernel's parameters; a longer one is uploaded from a pageable host
 * buffer, which blocks the calling thread until the bytes are staged.  The positions are read on the host at call
 * time: whatever replays the enqueued work later replays it for those positions.
 * All calls on a device share the one array, and it keeps the previous call's partial records: two calls that may
 * overlap on the GPU (different streams, or different host threads) race on it -- issue them on one stream or
 * order them yourself.  Host-side it is not re-entrant either. */
enum { FLINT_ATTN_NOALLOC_MAX_TOKENS = 64, FLINT_ATTN_NOALLOC_MAX_ITEMS = 2048 };
int32_t flint_attn_decode_noalloc_dev(int32_t n, const int32_t *pos, const void *qkv_dev, int32_t qkv_dtype,
                                      void *out_dev, int32_t out_dtype, void *k_cache_dev, void *v_cache_dev,
                                      int32_t n_slots, int32_t is_swa, int32_t has_rope, const float *q_norm_dev,
                                      const float *k_norm_dev, const float *sinks_dev, void *cuda_stream, char *err,
                                      int32_t err_len);

#ifdef __cplusplus
}
#endif
#endif
