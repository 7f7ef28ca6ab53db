// Types shared by the host launcher and the sm_100a attention kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace flint {

// Fixed model shape (the reference's src/metal/flint_config.h:10-31).
constexpr int kNHead = 32;
constexpr int kNHeadKv = 4;
constexpr int kHeadDim = 128;
constexpr int kGqa = 8;
constexpr int kQDim = kNHead * kHeadDim;       // 4096
constexpr int kKvDim = kNHeadKv * kHeadDim;    // 512
constexpr int kQkvDim = kQDim + 2 * kKvDim;    // 5120
constexpr int kNSwa = 513;                     // window, current token included
constexpr int kSwaRing = 1024;
constexpr float kRmsEps = 1e-6f;
constexpr float kRopeTheta = 10000.0f;
constexpr int kPartialDim = kHeadDim + 2;      // acc[128], m, l
constexpr int kRecStride = 132;                // floats between split-K scratch records (16-byte aligned rows)
constexpr int kMaxPeers = 8;                    // ranks of a KV-range-sharded sequence (one NVSwitch domain)
constexpr int kMaxParamItems = 640;             // work items that fit the 32 KiB kernel-parameter space
constexpr int kMergeFan = 16;                  // splits folded by one CTA in the first merge level

constexpr int kDtypeF32 = 0;
constexpr int kDtypeBf16 = 1;

// One unit of decode work: the 8 query heads of one KV head of one token against cached keys [j0, j1).
struct DecItem {
    int32_t tok;       // row of this call's qkv / out
    int32_t seq;       // sequence index into the caches
    int32_t kvh;       // KV head 0..3
    int32_t pos;       // position of the new token
    int32_t j0, j1;    // cached key positions covered by this item
    int32_t fold;      // 1: also attends to the new token itself and stores its K/V
    int32_t split;     // index of this item among the n_split items of its (tok, kvh) group
    int32_t n_split;
    int32_t part0;     // first partial record of the group in the scratch buffer
    int32_t group;     // second-level ticket counter index (one per (tok, kvh) group)
    int32_t sub0;      // first first-level ticket / second-level record of the group (one per run of kMergeFan splits)
};
static_assert(sizeof(DecItem) == 48, "DecItem is uploaded as raw bytes");

struct DecParams {
    const DecItem *items;
    const void *qkv;        // [n][5120] fp32 or bf16
    void *out;              // [n][4096] fp32 or bf16 (mode 0)
    float *partial_out;     // [n][32][130] (mode 1: this device's keys only, no sink)
    const float *q_norm, *k_norm, *sinks, *inv_freq;
    __half *k_cache, *v_cache;  // [max_seqs][4][n_slots][128]
    float *scratch;         // split-K partial records [..][8][kRecStride]
    float *scratch2;        // second-level records, one per run of kMergeFan splits
    int *tickets;           // one arrival counter per run of kMergeFan splits; all counters are zero between launches
    int *tickets2;          // one arrival counter per (tok, kvh) group
    long long seq_stride;   // halves between consecutive sequences = 4 * n_slots * 128
    int n_slots;
    uint32_t slot_mask;     // 1023 on ring layers, 0xFFFFFFFF otherwise
    int kv_lo;              // position held by slot 0 of a (sharded) full layer
    int has_rope;
    int qkv_dtype, out_dtype;
    int mode;               // 0: final output with sink; 1: partial record output; 2: partial records to every peer
    // mode 2 (KV-range sharding with a peer-memory exchange): this device's record of token t and head h goes to
    // peer_out[r] + (t * 32 + h) * 130 for every peer r (each points at this rank's slot in that peer's gather
    // buffer); when the last (token, KV head) group of the launch has written, peer_flag[r][rank] = step.
    float *peer_out[kMaxPeers];
    uint32_t *peer_flag[kMaxPeers];
    int n_peers, rank;
    uint32_t step;
    int *groups_done;       // one counter, zero between launches
    int n_groups;
    // Paged full-attention layers: k_cache / v_cache are page pools [n_pages][4][64][128] and the 64-key block b of
    // sequence s lives in page block_table[s * table_stride + b].  Work items then start on multiples of 64 keys, so a
    // 64-key tile is exactly one page.
    const int32_t *block_table;
    int table_stride;
    int paged;
    // Full layers of a handle: K/V tiles arrive by TMA.  k_map / v_map point at CUtensorMap objects in device memory
    // that describe the layer's cache (or page pool) as rows of 128 halves, {128, rows}, box {64, 64}, 128-byte
    // swizzle; null: tiles are fetched with 16-byte cp.async (ring layers, caller-owned caches).
    const void *k_map, *v_map;
    int *error_flag;  // set when a bounded wait of the TMA variant runs out (null: not reported)
};
constexpr int kPageKeys = 64;                   // keys per KV page = one decode tile

struct CombineParams {
    const float *partials;  // [n_parts][n][32][130]
    const float *sinks;
    void *out;              // [n][4096]
    int n, n_parts, out_dtype;
    int part_stride;        // floats between consecutive parts (n * 32 * 130 when packed)
    // peer-memory exchange only: wait (bounded) until flags[r] == step for every part before reading
    const uint32_t *flags;  // null: do not wait
    uint32_t step;
    int *error_flag;
};

cudaError_t launch_decode(const DecParams &p, int n_items, cudaStream_t stream);
// Same kernel with the work list passed by value in the kernel parameters (n_items <= kMaxParamItems): no upload.
cudaError_t launch_decode_inline(const DecParams &p, const DecItem *host_items, int n_items, int sm_count,
                                 cudaStream_t stream);
cudaError_t launch_combine(const CombineParams &p, cudaStream_t stream);
cudaError_t decode_kernel_setup();  // opt-in shared memory size; once per device

}  // namespace flint
