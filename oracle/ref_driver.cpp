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
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <vector>

#include "ref/ref_model.h"

int main(int argc, char **argv) {
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
