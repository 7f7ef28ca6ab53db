// Dense bf16 projections either side of attention: qkv = W_qkv . rmsnorm(x) and x += W_o . att
// (the reference's q/k/v matvecs and o-proj, src/engine.mm:728-732, :811; src/ref/ref_model.cpp:108-111, :150-151).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace flint {

constexpr int kProjMaxBatch = 64;   // activation rows per launch (larger batches go in chunks)
constexpr int kProjRowBlock = 128;  // weight rows per CTA; N must be a multiple of it

// Scratch that lives with the owner of the weights and grows on demand.
struct ProjWorkspace {
    __nv_bfloat16 *act_hi = nullptr, *act_lo = nullptr;  // [kProjMaxBatch][k_cap]: activations as bf16 high + low parts
    float *partial = nullptr;                            // [k splits][kProjMaxBatch][n_cap] fp32 partial sums
    int *tickets = nullptr;                              // one arrival counter per block of kProjRowBlock rows
    size_t k_cap = 0, partial_floats = 0, n_tickets = 0;
};

struct ProjCall {
    const __nv_bfloat16 *w;  // [N][K], K contiguous (the GGUF layout: dims[0] = K)
    const void *act;         // [B][K] fp32 or bf16 activations
    int act_dtype;           // kDtypeF32 / kDtypeBf16
    const float *norm_w;     // [K]: fused RMSNorm of each activation row (x * rsqrt(mean x^2 + eps) * norm_w), or null
    void *out;               // [B][N]
    int out_dtype;
    const float *residual;   // [B][N] fp32 added to the product (may be the same buffer as out), or null
    int B, N, K;
};

// out = (residual +) W . (rmsnorm?)(act)  for any B (chunks of kProjMaxBatch).  Launches on `stream`; *n_launches
// receives the number of kernels enqueued.
cudaError_t launch_proj(const ProjCall &c, ProjWorkspace &ws, int sm_count, cudaStream_t stream, int *n_launches);
void proj_workspace_free(ProjWorkspace &ws);

// rows[i] = table[ids[i]] (bf16 table [n_rows][K] -> fp32 [n][K]): the embedding look-up in front of the first layer.
cudaError_t launch_embed_rows(const __nv_bfloat16 *table, const int32_t *ids_dev, int n, int K, float *rows,
                              cudaStream_t stream);
// Index of the largest of n floats (first one on ties), written to *result_dev.
cudaError_t launch_argmax(const float *x, int n, int32_t *result_dev, cudaStream_t stream);

}  // namespace flint
