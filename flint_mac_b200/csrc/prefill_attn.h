// Prefill attention launcher (norm/RoPE/cache-write prologue + tcgen05 flash attention).
#pragma once

#include "attn_common.h"

namespace flint {

struct PrefillParams {
    const void *qkv;   // [n_tok][5120] fp32 or bf16, raw projections
    void *out;         // [n_tok][4096] fp32 or bf16
    const float *q_norm, *k_norm, *sinks, *inv_freq;
    __half *k_cache, *v_cache;  // this sequence's caches: [4][n_slots][128]
    int n_slots;
    int is_swa, has_rope;
    int p0, n_tok;     // positions p0 .. p0+n_tok-1
    int qkv_dtype, out_dtype;
    cudaEvent_t ev_attn_begin = nullptr, ev_attn_end = nullptr;  // optional: recorded around the attention kernel alone
    // Paged full-attention layer: k_cache / v_cache are the layer's page pools [n_pages][4][64][128] and block_table
    // (device, this sequence's row) maps the 64-key block b to its page.
    const int32_t *block_table = nullptr;
    int n_pages = 0, table_len = 0;
    // Full layer whose cache holds positions [kv_lo, kv_hi) only (row 0 = position kv_lo).  with_sink: this device
    // adds the learned sink (exactly one of the devices sharing a sequence does).
    int kv_lo = 0, kv_hi = 0x7fffffff, with_sink = 1;
    // Context-parallel prefill: instead of normalised rows in `out`, write this device's partial -- un-normalised
    // fp32 rows [n_tok][4096] and per (token, head) the pair (m in base-2 units, l), [n_tok][32][2] -- for
    // launch_prefill_combine after the devices have exchanged them.
    float *partial_o = nullptr;
    float *partial_ml = nullptr;
};

// Device scratch that lives with the handle and grows on demand: half-precision staging of the normalised,
// rotated Q and of the K/V rows a launch attends to.
struct PrefillWorkspace {
    void *buf = nullptr;
    size_t cap = 0;
    // which CTA runs which work units (see launch_prefill); rebuilt only when the launch geometry changes
    int *sched = nullptr;
    size_t sched_cap = 0;
    int sched_key[5] = {-1, -1, -1, -1, -1};  // n_tok, p0, is_swa, first key row, grid
    int sched_rounds = 0;
};

cudaError_t prefill_kernel_setup();
// A tensor map (128 bytes, written to map_out on the host) over a K or V cache seen as n_rows rows of 128 halves:
// {128, n_rows}, box {64 halves, 64 rows}, 128-byte swizzle -- what the decode kernel's TMA tile loads use.
cudaError_t make_kv_rows_map(void *map_out, const void *base, long long n_rows);
cudaError_t launch_prefill(const PrefillParams &p, PrefillWorkspace &ws, cudaStream_t stream, int *n_launches);
void prefill_workspace_free(PrefillWorkspace &ws);
// parts_o [n_parts][n_tok][4096] fp32, parts_ml [n_parts][n_tok][32][2] -> out [n_tok][4096]: log-sum-exp merge of the
// devices' partials (src/metal/fused.metal:332-350 applied to prefill rows; the sink is inside one part's l).
cudaError_t launch_prefill_combine(const float *parts_o, const float *parts_ml, int n_parts, int n_tok, void *out,
                                   int out_dtype, cudaStream_t stream);
// Reads the device-side error word of the last prefill launches (0 = none; 1 = a bounded wait ran out; 2 = shared
// memory was not 1024-byte aligned).  Blocking.  A non-zero word is cleared after it has been read.
cudaError_t prefill_error_flag(const PrefillWorkspace &ws, int *flag);

}  // namespace flint
