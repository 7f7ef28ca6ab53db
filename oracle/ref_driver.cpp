// Driver for the UNMODIFIED reference CPU model (src/ref/ref_model.cpp), used only to pin the oracle.
// TEST INFRASTRUCTURE: never linked into the shipped library.
//
// The reference's RefModel::forward is whole-model (src/ref/ref_model.cpp:95-197).  It is fed a synthetic
// all-F32 GGUF (written by make_ref_gguf.py) whose q/k/v projections are selection matrices, whose output
// projection copies the attention result into embedding dimensions that are zero on input, and whose FFN
// weights are zero.  After forward(t) the residual stream therefore holds, in dims [5120, 9216), exactly the
// 4096 attention outputs of token t, which this program writes out as raw float32.
//
//   ref_attn <model.gguf> <n_tokens> <out.bin> [threads]
//
// Second mode, for the attention stack with real projections (a GGUF whose FFN weights are zero): feeds the token ids
// of a file through RefModel::forward one by one and writes, per token, the logits it returns and the residual stream
// after the last layer (last_hidden()).
//
//   ref_attn --stack <model.gguf> <tokens.i32> <logits.bin> <hidden.bin> [threads]
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

#include "ref/ref_model.h"

static int run_stack(int argc, char **argv) {
    if (argc < 6) {
        fprintf(stderr, "usage: %s --stack model.gguf tokens.i32 logits.bin hidden.bin [threads]\n", argv[0]);
        return 2;
    }
    try {
        const int threads = argc > 6 ? atoi(argv[6]) : 8;
        flint::GgufFile file(argv[2]);
        flint::ref::RefModel model(file, threads);
        FILE *ft = fopen(argv[3], "rb");
        if (!ft) throw std::runtime_error("cannot open the token file");
        std::vector<int32_t> tokens;
        int32_t t;
        while (fread(&t, sizeof(t), 1, ft) == 1) tokens.push_back(t);
        fclose(ft);
        FILE *fl = fopen(argv[4], "wb"), *fh = fopen(argv[5], "wb");
        if (!fl || !fh) throw std::runtime_error("cannot open an output file");
        for (int32_t tok : tokens) {
            const std::vector<float> logits = model.forward(tok);
            fwrite(logits.data(), sizeof(float), logits.size(), fl);
            const std::vector<float> &h = model.last_hidden();
            fwrite(h.data(), sizeof(float), h.size(), fh);
        }
        fclose(fl);
        fclose(fh);
    } catch (const std::exception &ex) {
        fprintf(stderr, "ref_attn: %s\n", ex.what());
        return 1;
    }
    return 0;
}

int main(int argc, char **argv) {
    if (argc > 1 && std::string(argv[1]) == "--stack") return run_stack(argc, argv);
    if (argc < 4) {
        fprintf(stderr, "usage: %s model.gguf n_tokens out.bin [threads]\n", argv[0]);
        return 2;
    }
    try {
        const int n_tok = atoi(argv[2]);
        const int threads = argc > 4 ? atoi(argv[4]) : 8;
        flint::GgufFile file(argv[1]);
        flint::ref::RefModel model(file, threads);
        const int q_dim = model.hp().n_head * model.hp().head_dim;
        const int att_off = q_dim + 2 * model.hp().n_head_kv * model.hp().head_dim;
        if (model.hp().n_embd != att_off + q_dim) throw std::runtime_error("unexpected embedding width");
        FILE *fp = fopen(argv[3], "wb");
        if (!fp) throw std::runtime_error("cannot open output");
        for (int t = 0; t < n_tok; t++) {
            model.forward(t);
            const std::vector<float> &h = model.last_hidden();
            fwrite(h.data() + att_off, sizeof(float), q_dim, fp);
        }
        fclose(fp);
    } catch (const std::exception &ex) {
        fprintf(stderr, "ref_attn: %s\n", ex.what());
        return 1;
    }
    return 0;
}
