/* A plain-C client of include/flint_attn.h: the call sequence the reference's server makes through its FFI
 * (server/src/ffi.rs:5-28 over src/capi.h: open, prefill the prompt, decode token by token, truncate on a prefix
 * hit, decode again, close), at the attention boundary.  Test infrastructure: it proves the header is valid C and
 * that the library can be driven without Python or C++.
 *
 *   c_abi_driver <libflint_attn.so> symbols   resolve every entry point used below, compute nothing (no GPU needed)
 *   c_abi_driver <libflint_attn.so> run       run the sequence on CUDA device 0 and check the rollback property:
 *                                             decoding a token, truncating it away and decoding the same row again
 *                                             gives bit-identical output
 */
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../include/flint_attn.h"

/* Function-pointer types taken from the header's own declarations, so a signature drift fails to compile. */
typedef __typeof__(&flint_attn_open) open_fn;
typedef __typeof__(&flint_attn_close) close_fn;
typedef __typeof__(&flint_attn_n_ctx) n_ctx_fn;
typedef __typeof__(&flint_attn_pos) pos_fn;
typedef __typeof__(&flint_attn_truncate) truncate_fn;
typedef __typeof__(&flint_attn_rollback_restart) restart_fn;
typedef __typeof__(&flint_attn_advance) advance_fn;
typedef __typeof__(&flint_attn_set_layer) set_layer_fn;
typedef __typeof__(&flint_attn_decode) decode_fn;
typedef __typeof__(&flint_attn_prefill) prefill_fn;

static void *must_sym(void *lib, const char *name) {
    void *p = dlsym(lib, name);
    if (!p) {
        fprintf(stderr, "missing symbol %s\n", name);
        exit(2);
    }
    return p;
}

/* deterministic pseudo-random rows in [-1, 1) */
static float frand(uint32_t *s) {
    *s = *s * 1664525u + 1013904223u;
    return (float)(*s >> 8) / 8388608.0f - 1.0f;
}

int main(int argc, char **argv) {
    if (argc != 3) {
        fprintf(stderr, "usage: %s <libflint_attn.so> symbols|run\n", argv[0]);
        return 2;
    }
    void *lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        fprintf(stderr, "dlopen: %s\n", dlerror());
        return 2;
    }
    open_fn f_open = (open_fn)must_sym(lib, "flint_attn_open");
    close_fn f_close = (close_fn)must_sym(lib, "flint_attn_close");
    n_ctx_fn f_n_ctx = (n_ctx_fn)must_sym(lib, "flint_attn_n_ctx");
    pos_fn f_pos = (pos_fn)must_sym(lib, "flint_attn_pos");
    truncate_fn f_truncate = (truncate_fn)must_sym(lib, "flint_attn_truncate");
    restart_fn f_restart = (restart_fn)must_sym(lib, "flint_attn_rollback_restart");
    advance_fn f_advance = (advance_fn)must_sym(lib, "flint_attn_advance");
    set_layer_fn f_set_layer = (set_layer_fn)must_sym(lib, "flint_attn_set_layer");
    decode_fn f_decode = (decode_fn)must_sym(lib, "flint_attn_decode");
    prefill_fn f_prefill = (prefill_fn)must_sym(lib, "flint_attn_prefill");

    /* host-only entry point: the rule of server/src/main.rs:96-100 */
    if (f_restart(2000, 1900) != 1900 || f_restart(2000, 1000) != 488 || f_restart(300, 0) != 0) {
        fprintf(stderr, "rollback_restart disagrees with the reference rule\n");
        return 1;
    }
    if (strcmp(argv[2], "symbols") == 0) {
        printf("symbols ok\n");
        return 0;
    }

    enum { N_PROMPT = 40, N_DECODE = 3, N_CTX = 256 };
    char err[256] = "";
    const int32_t is_swa[2] = {1, 0}, has_rope[2] = {1, 1};
    flint_attn_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.device = 0;
    cfg.n_layers = 2;
    cfg.layer_is_swa = is_swa;
    cfg.layer_has_rope = has_rope;
    cfg.max_seqs = 1;
    cfg.n_ctx = N_CTX;
    flint_attn *h = f_open(&cfg, err, (int32_t)sizeof(err));
    if (!h) {
        fprintf(stderr, "open failed: %s\n", err);
        return 1;
    }
    if (f_n_ctx(h) != N_CTX || f_pos(h, 0) != 0) return 1;

    uint32_t seed = 7;
    float q_norm[FLINT_ATTN_HEAD_DIM], k_norm[FLINT_ATTN_HEAD_DIM], sinks[FLINT_ATTN_N_HEAD];
    for (int i = 0; i < FLINT_ATTN_HEAD_DIM; i++) {
        q_norm[i] = 1.0f + 0.1f * frand(&seed);
        k_norm[i] = 1.0f + 0.1f * frand(&seed);
    }
    for (int i = 0; i < FLINT_ATTN_N_HEAD; i++) sinks[i] = frand(&seed);
    for (int layer = 0; layer < 2; layer++)
        if (f_set_layer(h, layer, q_norm, k_norm, sinks, err, (int32_t)sizeof(err)) != 0) {
            fprintf(stderr, "set_layer: %s\n", err);
            return 1;
        }

    const size_t row = FLINT_ATTN_QKV_DIM, orow = FLINT_ATTN_OUT_DIM;
    float *qkv = (float *)malloc(sizeof(float) * row * (N_PROMPT + N_DECODE));
    float *out = (float *)malloc(sizeof(float) * orow * N_PROMPT);
    float *first = (float *)malloc(sizeof(float) * orow * 2);
    float *again = (float *)malloc(sizeof(float) * orow * 2);
    if (!qkv || !out || !first || !again) return 1;
    for (size_t i = 0; i < row * (N_PROMPT + N_DECODE); i++) qkv[i] = frand(&seed);
    const int32_t seq0 = 0;

    /* prefill: every layer, then one advance (src/engine.mm:1248) */
    for (int layer = 0; layer < 2; layer++)
        if (f_prefill(h, layer, 0, N_PROMPT, qkv, FLINT_ATTN_F32, out, FLINT_ATTN_F32, err, (int32_t)sizeof(err)) != 0) {
            fprintf(stderr, "prefill: %s\n", err);
            return 1;
        }
    if (f_advance(h, 1, &seq0, N_PROMPT) != 0 || f_pos(h, 0) != N_PROMPT) return 1;

    /* decode token by token (src/engine.mm:936) */
    for (int t = 0; t < N_DECODE; t++) {
        for (int layer = 0; layer < 2; layer++) {
            float *dst = t == N_DECODE - 1 ? first + orow * layer : out;
            if (f_decode(h, layer, 1, &seq0, qkv + row * (N_PROMPT + t), FLINT_ATTN_F32, dst, FLINT_ATTN_F32, err,
                         (int32_t)sizeof(err)) != 0) {
                fprintf(stderr, "decode: %s\n", err);
                return 1;
            }
        }
        if (f_advance(h, 1, &seq0, 1) != 0) return 1;
    }
    /* prefix-cache hit: roll the last token back (src/capi.h:27-29) and decode the same row again */
    if (f_truncate(h, 0, N_PROMPT + N_DECODE + 1) != -1 || f_truncate(h, 0, -1) != -1) return 1;
    if (f_truncate(h, 0, N_PROMPT + N_DECODE - 1) != 0 || f_pos(h, 0) != N_PROMPT + N_DECODE - 1) return 1;
    for (int layer = 0; layer < 2; layer++)
        if (f_decode(h, layer, 1, &seq0, qkv + row * (N_PROMPT + N_DECODE - 1), FLINT_ATTN_F32, again + orow * layer,
                     FLINT_ATTN_F32, err, (int32_t)sizeof(err)) != 0) {
            fprintf(stderr, "decode after truncate: %s\n", err);
            return 1;
        }
    int bad = memcmp(first, again, sizeof(float) * orow * 2) != 0;
    double sum = 0;
    for (size_t i = 0; i < orow * 2; i++) {
        if (!isfinite(first[i])) bad = 1;
        sum += fabs((double)first[i]);
    }
    /* errors come back as -1 + message, never as a crash (src/capi.mm:27-73) */
    const int32_t seq_bad = 5;
    if (f_decode(h, 0, 1, &seq_bad, qkv, FLINT_ATTN_F32, out, FLINT_ATTN_F32, err, (int32_t)sizeof(err)) != -1 || !err[0])
        bad = 1;
    f_close(h);
    free(qkv); free(out); free(first); free(again);
    if (bad || sum == 0.0) {
        fprintf(stderr, "mismatch after rollback, or a dead output\n");
        return 1;
    }
    printf("run ok (mean |out| = %.4f)\n", sum / (double)(orow * 2));
    return 0;
}
