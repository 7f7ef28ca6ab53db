/*
 * CPU oracle for the flint attention hot path -- TEST INFRASTRUCTURE ONLY.
 * See flint_attn_oracle.h.  Every function names the reference lines it restates.
 * Build without -ffast-math and without FMA contraction so that the float
 * operation order below is the one that runs (the reference is built -O2 for
 * baseline x86-64, src/../Makefile:5-6, which has neither).
 */
#include "flint_attn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ generator */
static inline uint64_t fo_mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint64_t fo_gen_u64(uint64_t seed, uint64_t stream, uint64_t index) {
    const uint64_t key = fo_mix(fo_mix(seed) ^ (stream * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
    return fo_mix(key ^ (index * 0xA0761D6478BD642Full));
}

void fo_gen_normal(uint64_t seed, uint64_t stream, uint64_t first, uint64_t n, float mean, float std, float *out) {
    const uint64_t key = fo_mix(fo_mix(seed) ^ (stream * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull));
#pragma omp parallel for schedule(static) if (n > 65536)
    for (uint64_t i = 0; i < n; i++) {
        const uint64_t a = fo_mix(key ^ ((first + i) * 0xA0761D6478BD642Full));
        const uint64_t b = fo_mix(a);
        const double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0); /* (0,1] */
        const double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);         /* [0,1) */
        const double z = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
        out[i] = (float)((double)mean + (double)std * z);
    }
}

/* ------------------------------------------------------------------ half / bf16 */
void fo_round_f16(float *x, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) x[i] = (float)(_Float16)x[i];
}

static inline uint16_t bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40); /* NaN */
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

void fo_round_bf16(float *x, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) {
        const uint32_t u = (uint32_t)bf16_bits(x[i]) << 16;
        memcpy(&x[i], &u, 4);
    }
}

void fo_f32_to_f16_bits(const float *x, uint16_t *out, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) {
        const _Float16 h = (_Float16)x[i];
        memcpy(&out[i], &h, 2);
    }
}

void fo_f16_bits_to_f32(const uint16_t *x, float *out, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) {
        _Float16 h;
        memcpy(&h, &x[i], 2);
        out[i] = (float)h;
    }
}

void fo_f32_to_bf16_bits(const float *x, uint16_t *out, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) out[i] = bf16_bits(x[i]);
}

void fo_bf16_bits_to_f32(const uint16_t *x, float *out, uint64_t n) {
    for (uint64_t i = 0; i < n; i++) {
        const uint32_t u = (uint32_t)x[i] << 16;
        memcpy(&out[i], &u, 4);
    }
}

/* ------------------------------------------------------------------ norm / rope */
/* src/ref/ref_model.cpp:45-50: double sum of squares, fp32 scale, (x*scale)*w. */
void fo_rmsnorm(const float *x, const float *w, float *y, int n, float eps) {
    double ss = 0;
    for (int i = 0; i < n; i++) ss += (double)x[i] * x[i];
    const float scale = 1.0f / sqrtf((float)(ss / n) + eps);
    for (int i = 0; i < n; i++) y[i] = x[i] * scale * w[i];
}

/* src/ref/ref_model.cpp:53-61: pair (i, i+d/2); freq = powf(theta, -2i/d); angle = pos*freq in fp32. */
void fo_rope_neox(float *x, int d, int pos, float theta) {
    for (int i = 0; i < d / 2; i++) {
        const float freq = powf(theta, -2.0f * i / d);
        const float a = pos * freq, c = cosf(a), s = sinf(a);
        const float x0 = x[i], x1 = x[i + d / 2];
        x[i] = x0 * c - x1 * s;
        x[i + d / 2] = x0 * s + x1 * c;
    }
}

void fo_inv_freq(float theta, float *out64) {
    for (int i = 0; i < FO_HEAD_DIM / 2; i++) out64[i] = powf(theta, -2.0f * i / FO_HEAD_DIM);
}

/* src/ref/ref_model.cpp:112-121 */
void fo_qk_norm_rope(float *row, const float *q_norm, const float *k_norm, int pos, int has_rope) {
    for (int h = 0; h < FO_N_HEAD; h++) {
        float *q = row + h * FO_HEAD_DIM;
        fo_rmsnorm(q, q_norm, q, FO_HEAD_DIM, FO_RMS_EPS);
        if (has_rope) fo_rope_neox(q, FO_HEAD_DIM, pos, FO_ROPE_THETA);
    }
    for (int h = 0; h < FO_N_HEAD_KV; h++) {
        float *k = row + FO_Q_DIM + h * FO_HEAD_DIM;
        fo_rmsnorm(k, k_norm, k, FO_HEAD_DIM, FO_RMS_EPS);
        if (has_rope) fo_rope_neox(k, FO_HEAD_DIM, pos, FO_ROPE_THETA);
    }
}

/* ------------------------------------------------------------------ attention */
/* One head of src/ref/ref_model.cpp:130-148.  s: scratch of pos+1 floats. */
static void attend_head(const float *qh, const float *kc, const float *vc, int kvh, float sink, int first, int pos,
                        float *s, float *out) {
    const int D = FO_HEAD_DIM, kv_dim = FO_KV_DIM;
    const float scale = 1.0f / sqrtf((float)D);
    float m = sink;
    for (int j = first; j <= pos; j++) {
        const float *kj = &kc[(size_t)j * kv_dim + kvh * D];
        float d = 0;
        for (int i = 0; i < D; i++) d += qh[i] * kj[i];
        s[j] = d * scale;
        m = fmaxf(m, s[j]);
    }
    double denom = expf(sink - m);
    double acc[FO_HEAD_DIM];
    for (int i = 0; i < D; i++) acc[i] = 0.0;
    for (int j = first; j <= pos; j++) {
        const double p = expf(s[j] - m);
        denom += p;
        const float *vj = &vc[(size_t)j * kv_dim + kvh * D];
        for (int i = 0; i < D; i++) acc[i] += p * vj[i];
    }
    for (int i = 0; i < D; i++) out[i] = (float)(acc[i] / denom);
}

void fo_attend(const float *q, const float *kc, const float *vc, const float *sinks, int pos, int is_swa, float *att,
               int n_threads) {
    const int first = is_swa ? (pos - FO_N_SWA + 1 > 0 ? pos - FO_N_SWA + 1 : 0) : 0;
    if (n_threads < 1) n_threads = 1;
#pragma omp parallel num_threads(n_threads) if (n_threads > 1)
    {
        float *s = (float *)malloc(sizeof(float) * (size_t)(pos + 1));
#pragma omp for schedule(dynamic, 1)
        for (int h = 0; h < FO_N_HEAD; h++)
            attend_head(q + h * FO_HEAD_DIM, kc, vc, h / FO_GQA, sinks[h], first, pos, s, att + h * FO_HEAD_DIM);
        free(s);
    }
}

void fo_layer_forward(const float *qkv, int T, int p0, const float *q_norm, const float *k_norm, const float *sinks,
                      int is_swa, int has_rope, int round_kv_f16, float *kc, float *vc, float *att, int n_threads) {
    float row[FO_QKV_DIM];
    for (int t = 0; t < T; t++) {
        const int pos = p0 + t;
        memcpy(row, qkv + (size_t)t * FO_QKV_DIM, sizeof(row));
        fo_qk_norm_rope(row, q_norm, k_norm, pos, has_rope);
        float *kdst = kc + (size_t)pos * FO_KV_DIM, *vdst = vc + (size_t)pos * FO_KV_DIM;
        memcpy(kdst, row + FO_Q_DIM, sizeof(float) * FO_KV_DIM);
        memcpy(vdst, row + FO_Q_DIM + FO_KV_DIM, sizeof(float) * FO_KV_DIM);
        if (round_kv_f16) {
            fo_round_f16(kdst, FO_KV_DIM);
            fo_round_f16(vdst, FO_KV_DIM);
        }
        fo_attend(row, kc, vc, sinks, pos, is_swa, att + (size_t)t * FO_Q_DIM, n_threads);
    }
}

void fo_decode_token_f16cache(const float *qkv_row, int pos, const float *q_norm, const float *k_norm,
                              const float *sinks, int is_swa, int has_rope, uint16_t *k16, uint16_t *v16,
                              int64_t n_slots, float *att, int n_threads) {
    float row[FO_QKV_DIM];
    memcpy(row, qkv_row, sizeof(row));
    fo_qk_norm_rope(row, q_norm, k_norm, pos, has_rope);
    /* write the new token's K/V (half) into its slot, as the kernel does */
    const int32_t slot = fo_slot(pos, is_swa);
    for (int kvh = 0; kvh < FO_N_HEAD_KV; kvh++) {
        fo_f32_to_f16_bits(row + FO_Q_DIM + kvh * FO_HEAD_DIM, k16 + ((size_t)kvh * n_slots + slot) * FO_HEAD_DIM,
                           FO_HEAD_DIM);
        fo_f32_to_f16_bits(row + FO_Q_DIM + FO_KV_DIM + kvh * FO_HEAD_DIM,
                           v16 + ((size_t)kvh * n_slots + slot) * FO_HEAD_DIM, FO_HEAD_DIM);
    }
    /* gather the visible window into a position-major fp32 cache and run the reference arithmetic on it */
    const int first = fo_k_begin(pos, is_swa);
    const int n = pos - first + 1;
    float *kc = (float *)malloc(sizeof(float) * (size_t)n * FO_KV_DIM);
    float *vc = (float *)malloc(sizeof(float) * (size_t)n * FO_KV_DIM);
#pragma omp parallel for schedule(static) num_threads(n_threads > 1 ? n_threads : 1) if (n_threads > 1)
    for (int j = 0; j < n; j++) {
        const int32_t s = fo_slot(first + j, is_swa);
        for (int kvh = 0; kvh < FO_N_HEAD_KV; kvh++) {
            fo_f16_bits_to_f32(k16 + ((size_t)kvh * n_slots + s) * FO_HEAD_DIM,
                               kc + (size_t)j * FO_KV_DIM + kvh * FO_HEAD_DIM, FO_HEAD_DIM);
            fo_f16_bits_to_f32(v16 + ((size_t)kvh * n_slots + s) * FO_HEAD_DIM,
                               vc + (size_t)j * FO_KV_DIM + kvh * FO_HEAD_DIM, FO_HEAD_DIM);
        }
    }
    /* positions are relative to `first`; the window is the whole gathered range */
    fo_attend(row, kc, vc, sinks, n - 1, 0, att, n_threads);
    free(kc);
    free(vc);
}

/* Per-head partial over [j0, j1): same score arithmetic, max/sum without the sink. */
void fo_attend_partial(const float *q, const float *kc, const float *vc, int j0, int j1, float *part) {
    const int D = FO_HEAD_DIM;
    const float scale = 1.0f / sqrtf((float)D);
    float *s = (float *)malloc(sizeof(float) * (size_t)(j1 > j0 ? j1 - j0 : 1));
    for (int h = 0; h < FO_N_HEAD; h++) {
        const int kvh = h / FO_GQA;
        float *p = part + (size_t)h * (D + 2);
        float m = -INFINITY;
        for (int j = j0; j < j1; j++) {
            const float *kj = &kc[(size_t)j * FO_KV_DIM + kvh * D];
            float d = 0;
            for (int i = 0; i < D; i++) d += q[h * D + i] * kj[i];
            s[j - j0] = d * scale;
            m = fmaxf(m, s[j - j0]);
        }
        double l = 0, acc[FO_HEAD_DIM];
        for (int i = 0; i < D; i++) acc[i] = 0;
        for (int j = j0; j < j1; j++) {
            const double w = expf(s[j - j0] - m);
            l += w;
            const float *vj = &vc[(size_t)j * FO_KV_DIM + kvh * D];
            for (int i = 0; i < D; i++) acc[i] += w * vj[i];
        }
        for (int i = 0; i < D; i++) p[i] = (float)acc[i];
        p[D] = m;
        p[D + 1] = (float)l;
    }
    free(s);
}

/* src/metal/fused.metal:332-350 */
void fo_combine(const float *part, int n_split, const float *sinks, float *out) {
    const int D = FO_HEAD_DIM, R = D + 2;
    for (int h = 0; h < FO_N_HEAD; h++) {
        const float *p0 = part + (size_t)h * n_split * R;
        const float sink = sinks[h];
        float M = sink;
        for (int s = 0; s < n_split; s++) M = fmaxf(M, p0[s * R + D]);
        float L = expf(sink - M);
        float A[FO_HEAD_DIM];
        for (int i = 0; i < D; i++) A[i] = 0;
        for (int s = 0; s < n_split; s++) {
            const float *p = p0 + s * R;
            const float ls = p[D + 1];
            if (ls == 0) continue;
            const float c = expf(p[D] - M);
            L += ls * c;
            for (int i = 0; i < D; i++) A[i] += p[i] * c;
        }
        for (int i = 0; i < D; i++) out[h * D + i] = A[i] / L;
    }
}

/* ------------------------------------------------------------------ integer maps */
/* ---- src/main.mm:253-305: the all-double statement with half-rounded K/V ------------------------------------ */
static void norm_rope_double(const float *in, const float *w, int pos, int has_rope, double *o) { /* main.mm:253-266 */
    double ss = 0;
    for (int d = 0; d < FO_HEAD_DIM; d++) ss += (double)in[d] * in[d];
    const double sc = 1.0 / sqrt(ss / FO_HEAD_DIM + FO_RMS_EPS);
    double t[FO_HEAD_DIM];
    for (int d = 0; d < FO_HEAD_DIM; d++) t[d] = in[d] * sc * w[d];
    for (int d = 0; d < FO_HEAD_DIM; d++) o[d] = t[d];
    if (!has_rope) return;
    for (int i = 0; i < FO_HEAD_DIM / 2; i++) {
        const double a = pos * pow((double)FO_ROPE_THETA, -2.0 * i / FO_HEAD_DIM), c = cos(a), s = sin(a);
        o[i] = t[i] * c - t[i + 64] * s;
        o[i + 64] = t[i] * s + t[i + 64] * c;
    }
}

void fo_attend_double_f16(const float *qkv, int n, const float *q_norm, const float *k_norm, const float *sinks,
                          int is_swa, int has_rope, const int32_t *probe_pos, int n_pos, const int32_t *probe_heads,
                          int n_heads, double *out) {
    const int QS = FO_QKV_DIM;
    double *K = (double *)malloc(sizeof(double) * (size_t)n * FO_KV_DIM);
    double *V = (double *)malloc(sizeof(double) * (size_t)n * FO_KV_DIM);
    double *sc = (double *)malloc(sizeof(double) * (size_t)(n + 1));
    /* all keys / values first, rounded through half (main.mm:268-278) */
    for (int p = 0; p < n; p++)
        for (int hk = 0; hk < FO_N_HEAD_KV; hk++) {
            double tmp[FO_HEAD_DIM];
            norm_rope_double(&qkv[(size_t)p * QS + FO_Q_DIM + hk * FO_HEAD_DIM], k_norm, p, has_rope, tmp);
            for (int d = 0; d < FO_HEAD_DIM; d++) {
                K[(size_t)p * FO_KV_DIM + hk * FO_HEAD_DIM + d] = (double)(_Float16)tmp[d];
                V[(size_t)p * FO_KV_DIM + hk * FO_HEAD_DIM + d] =
                    (double)(_Float16)qkv[(size_t)p * QS + FO_Q_DIM + FO_KV_DIM + hk * FO_HEAD_DIM + d];
            }
        }
    for (int ip = 0; ip < n_pos; ip++)
        for (int ih = 0; ih < n_heads; ih++) { /* main.mm:281-305 */
            const int p = probe_pos[ip], h = probe_heads[ih];
            double q[FO_HEAD_DIM];
            norm_rope_double(&qkv[(size_t)p * QS + h * FO_HEAD_DIM], q_norm, p, has_rope, q);
            const int kvh = h / FO_GQA, lo = is_swa ? (p - (FO_N_SWA - 1) > 0 ? p - (FO_N_SWA - 1) : 0) : 0;
            double m = sinks[h], l = 0, acc[FO_HEAD_DIM];
            for (int i = 0; i < FO_HEAD_DIM; i++) acc[i] = 0;
            for (int j = lo; j <= p; j++) {
                double d = 0;
                for (int i = 0; i < FO_HEAD_DIM; i++) d += q[i] * K[(size_t)j * FO_KV_DIM + kvh * FO_HEAD_DIM + i];
                sc[j] = d / sqrt((double)FO_HEAD_DIM);
                m = m > sc[j] ? m : sc[j];
            }
            l = exp(sinks[h] - m);
            for (int j = lo; j <= p; j++) {
                const double w = exp(sc[j] - m);
                l += w;
                for (int i = 0; i < FO_HEAD_DIM; i++) acc[i] += w * V[(size_t)j * FO_KV_DIM + kvh * FO_HEAD_DIM + i];
            }
            for (int i = 0; i < FO_HEAD_DIM; i++) out[((size_t)ip * n_heads + ih) * FO_HEAD_DIM + i] = acc[i] / l;
        }
    free(K);
    free(V);
    free(sc);
}

void fo_gen_grid(uint64_t seed, uint64_t stream, uint64_t first, uint64_t n, float *out) { /* main.mm:247 */
    for (uint64_t i = 0; i < n; i++) out[i] = ((int)(fo_gen_u64(seed, stream, first + i) % 2001) - 1000) / 500.0f;
}

/* ---- src/ref/ref_model.cpp:74-92, :95-197 with a zero feed-forward part ------------------------------------- */
void fo_matvec(const float *w, const float *x, float *y, int n_rows, int k, int n_threads) {
    if (n_threads < 1) n_threads = 1;
#pragma omp parallel for num_threads(n_threads) if (n_threads > 1 && n_rows >= 256) schedule(static)
    for (int r = 0; r < n_rows; r++) {
        const float *row = w + (size_t)r * k;
        double acc = 0;
        for (int i = 0; i < k; i++) acc += (double)row[i] * x[i];
        y[r] = (float)acc;
    }
}

void fo_stack_forward(const float *embd, const float *attn_norm, const float *wq, const float *wk, const float *wv,
                      const float *q_norm, const float *k_norm, const float *sinks, const float *wo,
                      const int32_t *is_swa, const int32_t *has_rope, const float *out_norm, const float *w_out,
                      const int32_t *tokens, int n_tok, int n_layer, int n_embd, int n_vocab, float *logits,
                      float *hidden, int n_threads) {
    const int E = n_embd;
    float *x = (float *)malloc(sizeof(float) * E), *xn = (float *)malloc(sizeof(float) * E);
    float *o = (float *)malloc(sizeof(float) * E);
    float row[FO_QKV_DIM], att[FO_Q_DIM];
    float **kc = (float **)malloc(sizeof(float *) * n_layer), **vc = (float **)malloc(sizeof(float *) * n_layer);
    for (int il = 0; il < n_layer; il++) {
        kc[il] = (float *)malloc(sizeof(float) * (size_t)n_tok * FO_KV_DIM);
        vc[il] = (float *)malloc(sizeof(float) * (size_t)n_tok * FO_KV_DIM);
    }
    for (int t = 0; t < n_tok; t++) {
        const int pos = t;
        memcpy(x, embd + (size_t)tokens[t] * E, sizeof(float) * E); /* ref_model.cpp:102 */
        for (int il = 0; il < n_layer; il++) {
            fo_rmsnorm(x, attn_norm + (size_t)il * E, xn, E, FO_RMS_EPS); /* :108 */
            fo_matvec(wq + (size_t)il * FO_Q_DIM * E, xn, row, FO_Q_DIM, E, n_threads); /* :109-111 */
            fo_matvec(wk + (size_t)il * FO_KV_DIM * E, xn, row + FO_Q_DIM, FO_KV_DIM, E, n_threads);
            fo_matvec(wv + (size_t)il * FO_KV_DIM * E, xn, row + FO_Q_DIM + FO_KV_DIM, FO_KV_DIM, E, n_threads);
            fo_qk_norm_rope(row, q_norm + il * FO_HEAD_DIM, k_norm + il * FO_HEAD_DIM, pos, has_rope[il]); /* :112-121 */
            memcpy(kc[il] + (size_t)pos * FO_KV_DIM, row + FO_Q_DIM, sizeof(float) * FO_KV_DIM); /* :122-124 */
            memcpy(vc[il] + (size_t)pos * FO_KV_DIM, row + FO_Q_DIM + FO_KV_DIM, sizeof(float) * FO_KV_DIM);
            fo_attend(row, kc[il], vc[il], sinks + il * FO_N_HEAD, pos, is_swa[il], att, n_threads); /* :125-149 */
            fo_matvec(wo + (size_t)il * E * FO_Q_DIM, att, o, E, FO_Q_DIM, n_threads); /* :150 */
            for (int i = 0; i < E; i++) x[i] += o[i]; /* :151 */
            /* the feed-forward half (:153-188) adds zero */
        }
        if (hidden) memcpy(hidden + (size_t)t * E, x, sizeof(float) * E);
        if (logits) {
            fo_rmsnorm(x, out_norm, xn, E, FO_RMS_EPS); /* :192 */
            fo_matvec(w_out, xn, logits + (size_t)t * n_vocab, n_vocab, E, n_threads); /* :194 */
        }
    }
    for (int il = 0; il < n_layer; il++) {
        free(kc[il]);
        free(vc[il]);
    }
    free(kc); free(vc); free(x); free(xn); free(o);
}

int32_t fo_slot(int32_t pos, int is_swa) { return is_swa ? (pos & (FO_SWA_RING - 1)) : pos; }

int32_t fo_k_begin(int32_t pos, int is_swa) {
    if (!is_swa) return 0;
    const int32_t b = pos - (FO_N_SWA - 1);
    return b > 0 ? b : 0;
}

void fo_ref_split_policy(int32_t pos, int is_swa, int32_t *keys_per_split, int32_t *n_split) {
    const int32_t n_keys = pos - fo_k_begin(pos, is_swa);
    int32_t kps = (n_keys + 31) / 32;
    if (kps < 256) kps = 256;
    int32_t ns = (n_keys + kps - 1) / kps;
    if (ns < 1) ns = 1;
    *keys_per_split = kps;
    *n_split = ns;
}

int32_t fo_rollback_restart(int32_t cached_len, int32_t p) {
    if (cached_len > p && cached_len - p > 511) p = p >= 512 ? p - 512 : 0;
    return p;
}

void fo_ring_owners(int32_t n, int32_t *owner) {
    for (int i = 0; i < FO_SWA_RING; i++) owner[i] = -1;
    for (int32_t p = 0; p < n; p++) owner[p & (FO_SWA_RING - 1)] = p;
}
