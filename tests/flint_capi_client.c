/* A plain-C stand-in for the reference's Rust server at its FFI boundary: it declares the nine functions the way
 * server/src/ffi.rs:18-28 does (through include/flint_capi.h, whose signatures are those of src/capi.h:20-37), LINKS
 * against the library like server/build.rs links libflint.a -- no dlopen, so a missing or misspelt symbol fails at
 * link time -- and replays the server's call sequence (server/src/main.rs:96-116, 166-187):
 *   open -> n_ctx / n_vocab / pos -> prefill(prompt) -> decode ... -> truncate (prefix reuse) -> decode -> logits -> close.
 * Test infrastructure.  (A Rust link test is not possible in this image: there is no rustc / cargo.)
 *
 *   flint_capi_client link-only                          references every symbol, calls nothing (no GPU needed)
 *   flint_capi_client <model file> <tokens.i32> <n_prompt> <n_decode> <n_back>
 *       prefill the first n_prompt tokens, decode the next n_decode (teacher-forced from the file), go back n_back
 *       tokens with flint_truncate and decode those again: prints one line per call, "<pos> <greedy token> <logit of
 *       that token> <sum of logits>", for the test to compare.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../include/flint_capi.h"

static void report(const flint_engine *e, int32_t next) {
    const float *lg = flint_logits(e);
    double sum = 0;
    const int32_t v = flint_n_vocab();
    for (int32_t i = 0; i < v; i++) sum += lg[i];
    printf("%d %d %.9g %.9g\n", flint_pos(e), next, lg[next], sum);
}

int main(int argc, char **argv) {
    if (argc == 2 && strcmp(argv[1], "link-only") == 0) {
        /* taking the addresses is enough to make the linker resolve all nine */
        const void *syms[] = {(void *)flint_open,     (void *)flint_close,   (void *)flint_n_ctx,
                              (void *)flint_n_vocab,  (void *)flint_pos,     (void *)flint_truncate,
                              (void *)flint_prefill,  (void *)flint_decode,  (void *)flint_logits};
        int n = 0;
        for (unsigned i = 0; i < sizeof(syms) / sizeof(syms[0]); i++) n += syms[i] != NULL;
        printf("linked %d symbols, n_vocab before any model = %d\n", n, flint_n_vocab());
        return n == 9 ? 0 : 1;
    }
    if (argc != 6) {
        fprintf(stderr, "usage: %s link-only | <model> <tokens.i32> <n_prompt> <n_decode> <n_back>\n", argv[0]);
        return 2;
    }
    const int n_prompt = atoi(argv[3]), n_decode = atoi(argv[4]), n_back = atoi(argv[5]);
    FILE *f = fopen(argv[2], "rb");
    if (!f) return 2;
    int32_t *tok = malloc(sizeof(int32_t) * (size_t)(n_prompt + n_decode));
    if (fread(tok, sizeof(int32_t), (size_t)(n_prompt + n_decode), f) != (size_t)(n_prompt + n_decode)) return 2;
    fclose(f);

    char err[1024] = {0}; /* server/src/ffi.rs:38 */
    flint_config cfg = {argv[1], "", 0.0, n_prompt + n_decode + 8};
    flint_engine *e = flint_open(&cfg, err, sizeof(err));
    if (!e) {
        fprintf(stderr, "flint_open: %s\n", err);
        return 1;
    }
    printf("n_ctx %d n_vocab %d pos %d\n", flint_n_ctx(e), flint_n_vocab(), flint_pos(e));
    /* errors come back as -1 + message and leave the engine usable */
    if (flint_prefill(e, tok, 0, err, sizeof(err)) != -1 || !err[0]) return 3;
    printf("empty prefill refused: %s\n", err);
    if (flint_truncate(e, 1) != -1 || flint_truncate(e, -1) != -1) return 3;

    int32_t next = flint_prefill(e, tok, n_prompt, err, sizeof(err));
    if (next < 0) {
        fprintf(stderr, "flint_prefill: %s\n", err);
        return 1;
    }
    report(e, next);
    for (int i = 0; i < n_decode; i++) {
        next = flint_decode(e, tok[n_prompt + i], err, sizeof(err));
        if (next < 0) {
            fprintf(stderr, "flint_decode: %s\n", err);
            return 1;
        }
        report(e, next);
    }
    /* prefix reuse: the next request shares all but the last n_back tokens (server/src/main.rs:96-105) */
    const int32_t keep = flint_pos(e) - n_back;
    if (flint_truncate(e, keep) != 0 || flint_pos(e) != keep) return 3;
    printf("truncated to %d\n", keep);
    for (int i = n_decode - n_back; i < n_decode; i++) {
        next = flint_decode(e, tok[n_prompt + i], err, sizeof(err));
        if (next < 0) return 1;
        report(e, next);
    }
    /* the context ends where the caller said */
    while (flint_pos(e) < flint_n_ctx(e)) {
        if (flint_decode(e, tok[0], err, sizeof(err)) < 0) return 1;
    }
    if (flint_decode(e, tok[0], err, sizeof(err)) != -1) return 3;
    printf("context full refused: %s\n", err);
    flint_close(e);
    printf("client ok\n");
    free(tok);
    return 0;
}
