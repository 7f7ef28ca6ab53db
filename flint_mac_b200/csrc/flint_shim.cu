// The reference's engine interface (src/capi.h:10-37: flint_open / close / n_ctx / n_vocab / pos / truncate / prefill /
// decode / logits) on top of the attention library, so that a caller written against that interface -- the Rust
// server binds exactly these nine symbols, server/src/ffi.rs:18-28 -- can link this library in its place.
//
// What stands behind the symbols here is the attention stack only: token embedding, then per layer
// x += W_o . attention(W_qkv . rmsnorm(x, attn_norm)), then output_norm and the vocabulary projection, greedy argmax.
// The feed-forward / mixture-of-experts half of every layer (src/engine.mm:813-899) is not part of this library; a
// model whose FFN weights are zero goes through the reference's CPU model (src/ref/ref_model.cpp:95-197) with the
// same arithmetic, which is how this file is tested.  The model file is not GGUF (its parser is outside this
// library's scope) but the flat container described in include/flint_capi.h.
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/flint_attn.h"
#include "../../include/flint_capi.h"
#include "attn_common.h"
#include "proj.h"

using namespace flint;

namespace {

void set_err(char *err, int32_t len, const char *msg) {  // src/capi.mm:17-22
    if (err && len > 0) {
        strncpy(err, msg, size_t(len) - 1);
        err[len - 1] = 0;
    }
}

#define SHIM_CK(call)                                                                                    \
    do {                                                                                                 \
        cudaError_t e_ = (call);                                                                         \
        if (e_ != cudaSuccess)                                                                           \
            throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e_) + " at " #call); \
    } while (0)

int32_t g_n_vocab = 150144;  // src/metal/flint_config.h:24 until a model file says otherwise

struct FileCloser {
    void operator()(FILE *f) const { if (f) fclose(f); }
};

void read_exact(FILE *f, void *dst, size_t bytes, const char *what) {
    if (fread(dst, 1, bytes, f) != bytes) throw std::runtime_error(std::string("model file ends inside ") + what);
}

}  // namespace

struct flint_engine {
    flint_attn *attn = nullptr;
    int n_layer = 0, n_embd = 0, n_vocab = 0, n_ctx = 0, device = 0;
    __nv_bfloat16 *embd = nullptr, *w_out = nullptr;  // [n_vocab][n_embd] each
    float *out_norm = nullptr;                         // [n_embd]
    float *x = nullptr;                                // residual stream rows [x_rows][n_embd]
    size_t x_rows = 0;
    int32_t *ids = nullptr;                            // token ids of the call, on the device
    size_t ids_cap = 0;
    float *logits_dev = nullptr, *logits_host = nullptr;
    int32_t *next_dev = nullptr;
    cudaStream_t stream = nullptr;

    ~flint_engine() {
        cudaSetDevice(device);
        if (attn) flint_attn_close(attn);
        cudaFree(embd); cudaFree(w_out); cudaFree(out_norm); cudaFree(x); cudaFree(ids); cudaFree(logits_dev);
        cudaFree(next_dev);
        if (logits_host) cudaFreeHost(logits_host);
        if (stream) cudaStreamDestroy(stream);
    }

    void attn_call(int32_t r, const char *err) {
        if (r != 0) throw std::runtime_error(err);
    }

    // Engine::prefill / Engine::step (src/engine.mm:968-1250, :902-946) without the feed-forward half.
    int32_t run(const int32_t *tokens, int n, bool prefill) {
        SHIM_CK(cudaSetDevice(device));
        if (n <= 0) throw std::runtime_error("empty prefill");  // src/engine.mm:975
        const int p0 = flint_attn_pos(attn, 0);
        if (p0 + n > n_ctx) throw std::runtime_error("context full");  // src/engine.mm:904, :976
        for (int i = 0; i < n; i++)
            if (tokens[i] < 0 || tokens[i] >= n_vocab) throw std::runtime_error("token id out of range");
        if (size_t(n) > x_rows) {
            SHIM_CK(cudaDeviceSynchronize());
            cudaFree(x);
            x = nullptr;
            x_rows = 0;
            const size_t rows = std::max<size_t>(size_t(n), 512);
            SHIM_CK(cudaMalloc(&x, rows * n_embd * sizeof(float)));
            x_rows = rows;
        }
        if (size_t(n) > ids_cap) {
            SHIM_CK(cudaDeviceSynchronize());
            cudaFree(ids);
            ids = nullptr;
            ids_cap = 0;
            SHIM_CK(cudaMalloc(&ids, std::max<size_t>(size_t(n), 512) * sizeof(int32_t)));
            ids_cap = std::max<size_t>(size_t(n), 512);
        }
        SHIM_CK(cudaMemcpyAsync(ids, tokens, size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice, stream));
        SHIM_CK(launch_embed_rows(embd, ids, n, n_embd, x, stream));
        char msg[512] = {0};
        const int32_t seq0 = 0;
        for (int il = 0; il < n_layer; il++) {
            const int32_t r = prefill ? flint_attn_prefill_block_dev(attn, il, 0, n, x, stream, msg, sizeof(msg))
                                      : flint_attn_decode_block_dev(attn, il, 1, &seq0, x, stream, msg, sizeof(msg));
            attn_call(r, msg);
        }
        // logits of the last position only (src/engine.mm:1236-1246): output_norm folded into the projection
        attn_call(flint_attn_project_dev(attn, reinterpret_cast<const uint16_t *>(w_out), n_vocab, n_embd,
                                         x + size_t(n - 1) * n_embd, 1, out_norm, logits_dev, stream, msg, sizeof(msg)),
                  msg);
        SHIM_CK(launch_argmax(logits_dev, n_vocab, next_dev, stream));
        int32_t next = -1;
        SHIM_CK(cudaMemcpyAsync(logits_host, logits_dev, size_t(n_vocab) * sizeof(float), cudaMemcpyDeviceToHost, stream));
        SHIM_CK(cudaMemcpyAsync(&next, next_dev, sizeof(next), cudaMemcpyDeviceToHost, stream));
        SHIM_CK(cudaStreamSynchronize(stream));  // synchronous like the reference (src/engine.mm:930)
        attn_call(flint_attn_check(attn, msg, sizeof(msg)), msg);
        if (flint_attn_advance(attn, 1, &seq0, n) != 0) throw std::runtime_error("context full");
        return next;
    }
};

extern "C" {

flint_engine *flint_open(const flint_config *cfg, char *err, int32_t err_len) {
    try {
        if (!cfg || !cfg->model_path) throw std::runtime_error("null config or model path");
        std::unique_ptr<FILE, FileCloser> f(fopen(cfg->model_path, "rb"));
        if (!f) throw std::runtime_error(std::string("cannot open model file ") + cfg->model_path);
        char magic[8];
        int32_t hdr[4];
        read_exact(f.get(), magic, 8, "the header");
        if (memcmp(magic, FLINT_MODEL_MAGIC, 8) != 0)
            throw std::runtime_error("not a flint attention-stack model file (GGUF loading is outside this library)");
        read_exact(f.get(), hdr, sizeof(hdr), "the header");
        const int n_layer = hdr[0], n_embd = hdr[1], n_vocab = hdr[2];
        if (n_layer <= 0 || n_layer > 1024 || n_embd <= 0 || n_embd % 256 != 0 || n_vocab <= 0 || n_vocab % 128 != 0)
            throw std::runtime_error("model header: layers > 0, n_embd a multiple of 256, n_vocab a multiple of 128");
        std::vector<int32_t> is_swa(n_layer), has_rope(n_layer);
        read_exact(f.get(), is_swa.data(), n_layer * 4, "the layer table");
        read_exact(f.get(), has_rope.data(), n_layer * 4, "the layer table");

        auto e = std::make_unique<flint_engine>();
        e->n_layer = n_layer; e->n_embd = n_embd; e->n_vocab = n_vocab;
        e->n_ctx = cfg->n_ctx > 0 ? cfg->n_ctx : 4096;  // src/capi.mm:39
        e->device = 0;
        flint_attn_config ac{};
        ac.device = e->device; ac.n_layers = n_layer;
        ac.layer_is_swa = is_swa.data(); ac.layer_has_rope = has_rope.data();
        ac.max_seqs = 1;  // single session (src/capi.h:1)
        ac.n_ctx = e->n_ctx;
        char msg[512] = {0};
        e->attn = flint_attn_open(&ac, msg, sizeof(msg));
        if (!e->attn) throw std::runtime_error(msg);
        SHIM_CK(cudaSetDevice(e->device));
        SHIM_CK(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
        const size_t E = size_t(n_embd), V = size_t(n_vocab);
        std::vector<uint16_t> big(std::max(V * E, size_t(kQDim) * E));
        auto upload_bf16 = [&](size_t n, const char *what) {
            read_exact(f.get(), big.data(), n * 2, what);
            __nv_bfloat16 *d = nullptr;
            SHIM_CK(cudaMalloc(&d, n * 2));
            SHIM_CK(cudaMemcpy(d, big.data(), n * 2, cudaMemcpyHostToDevice));
            return d;
        };
        e->embd = upload_bf16(V * E, "token_embd");
        std::vector<float> attn_norm(E), qn(kHeadDim), kn(kHeadDim), sinks(kNHead);
        std::vector<uint16_t> wq(size_t(kQDim) * E), wk(size_t(kKvDim) * E), wv(size_t(kKvDim) * E), wo(E * kQDim);
        for (int il = 0; il < n_layer; il++) {
            read_exact(f.get(), attn_norm.data(), E * 4, "attn_norm");
            read_exact(f.get(), wq.data(), wq.size() * 2, "attn_q");
            read_exact(f.get(), wk.data(), wk.size() * 2, "attn_k");
            read_exact(f.get(), wv.data(), wv.size() * 2, "attn_v");
            read_exact(f.get(), qn.data(), kHeadDim * 4, "attn_q_norm");
            read_exact(f.get(), kn.data(), kHeadDim * 4, "attn_k_norm");
            read_exact(f.get(), sinks.data(), kNHead * 4, "attn_sinks");
            read_exact(f.get(), wo.data(), wo.size() * 2, "attn_output");
            if (flint_attn_set_layer(e->attn, il, qn.data(), kn.data(), sinks.data(), msg, sizeof(msg)) != 0 ||
                flint_attn_set_projections(e->attn, il, n_embd, attn_norm.data(), wq.data(), wk.data(), wv.data(),
                                           wo.data(), msg, sizeof(msg)) != 0)
                throw std::runtime_error(msg);
        }
        std::vector<float> on(E);
        read_exact(f.get(), on.data(), E * 4, "output_norm");
        SHIM_CK(cudaMalloc(&e->out_norm, E * 4));
        SHIM_CK(cudaMemcpy(e->out_norm, on.data(), E * 4, cudaMemcpyHostToDevice));
        e->w_out = upload_bf16(V * E, "output");
        SHIM_CK(cudaMalloc(&e->logits_dev, V * sizeof(float)));
        SHIM_CK(cudaMallocHost(&e->logits_host, V * sizeof(float)));
        SHIM_CK(cudaMalloc(&e->next_dev, sizeof(int32_t)));
        memset(e->logits_host, 0, V * sizeof(float));
        g_n_vocab = n_vocab;
        return e.release();
    } catch (const std::exception &ex) {
        set_err(err, err_len, ex.what());
        return nullptr;
    }
}

void flint_close(flint_engine *e) { delete e; }

int32_t flint_n_ctx(const flint_engine *e) { return e->n_ctx; }
int32_t flint_n_vocab(void) { return g_n_vocab; }
int32_t flint_pos(const flint_engine *e) { return flint_attn_pos(e->attn, 0); }

int32_t flint_truncate(flint_engine *e, int32_t pos) { return flint_attn_truncate(e->attn, 0, pos); }  // capi.mm:52-56

int32_t flint_prefill(flint_engine *e, const int32_t *tokens, int32_t n, char *err, int32_t err_len) {
    try {
        if (!tokens && n > 0) throw std::runtime_error("null token array");
        return e->run(tokens, n, true);
    } catch (const std::exception &ex) {
        set_err(err, err_len, ex.what());
        return -1;
    }
}

int32_t flint_decode(flint_engine *e, int32_t token, char *err, int32_t err_len) {
    try {
        return e->run(&token, 1, false);
    } catch (const std::exception &ex) {
        set_err(err, err_len, ex.what());
        return -1;
    }
}

const float *flint_logits(const flint_engine *e) { return e->logits_host; }

}  // extern "C"
