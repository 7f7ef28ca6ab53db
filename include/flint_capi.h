/*
 * flint_capi -- the reference engine's C interface, exported by the B200 attention library.
 *
 * The nine entry points below have the names, argument lists and return conventions of the reference's
 * src/capi.h:20-37, which is what its Rust server binds (server/src/ffi.rs:18-28): an opaque engine created by
 * flint_open and freed by flint_close, int32 returns with -1 on failure and the message copied (NUL-terminated,
 * truncated) into the caller's buffer, a single session that the caller serialises (src/capi.h:1), synchronous
 * calls.  A program written against src/capi.h links against this library unchanged.
 *
 * What runs behind them is the attention stack of the model -- embedding, per layer the attention block
 * x += W_o . attention(W_qkv . rmsnorm(x)), output norm, vocabulary projection, greedy argmax -- not the
 * feed-forward / mixture-of-experts half of the layers, which this library does not contain.
 *
 * Model file.  flint_config.model_path names a flat little-endian container, not GGUF:
 *     char    magic[8]   = "FLNTATT1"
 *     int32   n_layer, n_embd (multiple of 256), n_vocab (multiple of 128), 0
 *     int32   is_swa[n_layer]      1: 513-key sliding window (1024-slot ring), 0: full context
 *     int32   has_rope[n_layer]
 *     bf16    token_embd[n_vocab][n_embd]
 *     per layer: f32 attn_norm[n_embd]; bf16 attn_q[4096][n_embd], attn_k[512][n_embd], attn_v[512][n_embd];
 *                f32 attn_q_norm[128], attn_k_norm[128], attn_sinks[32]; bf16 attn_output[n_embd][4096]
 *     f32     output_norm[n_embd]
 *     bf16    output[n_vocab][n_embd]
 * Tensor names are the reference's GGUF names (src/ref/ref_model.cpp:100-151, :192-195); rows are stored with
 * the input dimension contiguous, as GGUF stores them.  metallib_dir and pool_gb are accepted and ignored.
 */
#ifndef FLINT_CAPI_H
#define FLINT_CAPI_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLINT_MODEL_MAGIC "FLNTATT1"

typedef struct flint_engine flint_engine;

/* src/capi.h:12-17 */
typedef struct {
    const char *model_path;   /* the container described above */
    const char *metallib_dir; /* unused here (no Metal libraries) */
    double pool_gb;           /* unused here (no expert streaming) */
    int32_t n_ctx;            /* context length; full-attention layers allocate their KV cache for it */
} flint_config;

/* src/capi.h:20-21: NULL + message on failure (err may be NULL). */
flint_engine *flint_open(const flint_config *cfg, char *err, int32_t err_len);
void flint_close(flint_engine *e);

/* src/capi.h:23-25.  The reference's vocabulary size is a constant of its one model (src/metal/flint_config.h:24);
 * here flint_n_vocab reports that constant, 150144, until a model file has been opened, and that file's afterwards. */
int32_t flint_n_ctx(const flint_engine *e);
int32_t flint_n_vocab(void);
int32_t flint_pos(const flint_engine *e);

/* src/capi.h:27-29: back to position pos (<= current), -1 otherwise.  The sliding-window rings keep the last 1024
 * positions: after going back more than 511 tokens the caller prefills again from max(0, pos - 512). */
int32_t flint_truncate(flint_engine *e, int32_t pos);

/* src/capi.h:31-34: n tokens from the current position / one token; the greedy next token, or -1 + message. */
int32_t flint_prefill(flint_engine *e, const int32_t *tokens, int32_t n, char *err, int32_t err_len);
int32_t flint_decode(flint_engine *e, int32_t token, char *err, int32_t err_len);

/* src/capi.h:36-37: flint_n_vocab() floats of the last prefill / decode, valid until the next call. */
const float *flint_logits(const flint_engine *e);

#ifdef __cplusplus
}
#endif
#endif
