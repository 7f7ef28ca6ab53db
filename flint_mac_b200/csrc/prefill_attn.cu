// Prefill attention for sm_100a: a norm/RoPE/cache-write prologue and a tcgen05 flash-attention kernel.
//
// Replaces the reference's k_qk_prefill + k_attn_prefill chunk loop (src/metal/prefill.metal:100-266,
// src/engine.mm:1080-1104).  Semantics kept: RMSNorm then NEOX RoPE at position p0+t on q and k, K/V stored as half in
// the cache slot (pos & 1023 on ring layers), causal + 513-key window mask per element, the learned sink as the
// initial running maximum with l0 = 1 so that it only enters the denominator (prefill.metal:162), P rounded to half
// before P.V (prefill.metal:223), fp32 scores / statistics / accumulators.
//
// Shape chosen for B200: one CTA owns 128 query rows = 16 consecutive positions x the 8 query heads of one KV head,
// so one K/V tile serves the whole GQA group and the key band of a Q tile is 512+16 keys wide instead of 512+128;
// a CTA works on two such Q tiles (32 positions) that share every K/V tile.
// Q, K and V tiles arrive by TMA (128-byte swizzle, no multicast) from half-precision staging written by the
// prologue; S = Q.K^T and O += P.V run on the 5th-generation tensor core (tcgen05.mma, kind::f16) with both
// accumulators in tensor memory; each thread owns one query row of S (tcgen05.ld 32x32b), so the softmax needs no
// shuffles; O is rescaled lazily (only when a row maximum grows by more than 2^8).
#include "prefill_attn.h"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <queue>
#include <utility>
#include <vector>

#include "ptx.cuh"
#include "tc5.cuh"

namespace flint {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kQPos = 16;              // query positions per 128-row Q tile (x 8 heads of the GQA group)
constexpr int kBM = kQPos * kGqa;      // 128 query rows per Q tile
constexpr int kQTiles = 2;             // Q tiles per CTA: they share every K/V tile and take turns on the tensor core
constexpr int kCtaPos = kQPos * kQTiles;  // 32 query positions per CTA
constexpr int kBN = 128;               // keys per tile: an MMA narrower than N = 128 runs at half rate
constexpr int kSlots = 3;              // 32 KiB tile slots: slot 0 takes every K tile in turn, slots 1 and 2 the V tiles alternately
constexpr int kHist = kNSwa - 1;       // 512 keys of history a sliding-window query can see
// Tensor memory (all 512 columns): scores S per Q tile (read into registers, then free for the next tile's scores) and the
// output accumulators.
constexpr int kTmemCols = 512;
constexpr int kColS = 0;               // + 128 * tile
constexpr int kColO = 256;             // + 128 * tile
constexpr int kThreadsAttn = (kQTiles * 4 + 4) * 32;  // 8 softmax warps, 1 TMA warp, 2 MMA warps, 1 idle warp that
                                                      // completes the third warpgroup (register reallocation is per warpgroup)

constexpr int kQBytes = kBM * kHeadDim * 2;   // 32 KiB per Q tile: two 64-dim halves of [128 rows][128 B]
constexpr int kTileBytes = kBN * kHeadDim * 2;  // 32 KiB per K or V tile: two 64-dim halves of [128 keys][128 B]
constexpr int kOffQ = 0;
constexpr int kOffKV = kOffQ + kQTiles * kQBytes;
constexpr int kOutBlockBytes = kQPos * kGqa * 128;  // one 128-byte-wide column block of one Q tile's output
constexpr int kPBytes = kBM * kBN * 2;        // 32 KiB per P tile (two 64-key halves of [128 rows][128 B]); shares the
                                              // staging block of its Q tile with the output rows of the unit's drain
constexpr int kOffStage = kOffKV + kSlots * kTileBytes;  // per Q tile 32 KiB: P tiles, and the output rows at the end of a unit
static_assert(kPBytes == 2 * kOutBlockBytes, "P and the output staging share one block per Q tile");
constexpr int kOffBar = kOffStage + kQTiles * 2 * kOutBlockBytes;
constexpr int kOffSched = kOffBar + 256;   // this CTA's list of work units (the first kSchedLocal of them)
constexpr int kSchedLocal = 640;
constexpr int kSmemBytes = kOffSched + kSchedLocal * 4;  // 232192 B: one CTA per SM
static_assert(kSmemBytes <= 232448, "shared memory of one CTA");

struct PfArgs {
    const int *sched;  // [n_rounds][gridDim.x] unit of CTA b in its round i, -1 = none; nullptr: round-robin
    int n_rounds, n_units;
    const __half *q_st;  // [32][n_tok][128] normalised, rotated, pre-scaled queries
    void *out;
    const float *sinks;
    int *error_flag;
    int out_dtype;
    int p0, n_tok, is_swa;
    int key_row0;  // key position held by row 0 of the K/V tensor maps
    // Key-range split (full layers, chunks with fewer units than SMs): every unit is cut into n_ksplit ranges of key
    // tiles; each range writes an un-normalised fp32 partial (rows s * t_pad + t of `out`) and its (m, l) per row.
    int n_ksplit, t_pad;
    float2 *part_ml;  // [n_ksplit * t_pad][32] (m in base-2 units, l)
    // paged full layer: the K/V maps cover the page pool {128 dims, 64 rows, n_pages * 4} and the 64-key block b of
    // the sequence is page block_table[b] (entries past the sequence's last page are negative)
    const int32_t *block_table;
    int table_len;
    // Key-range shard of a full layer (context-parallel prefill): this device holds keys [kr_lo, kr_hi) only; a unit's
    // keys are clipped to it, the sink enters on the device that says so, and the output is an un-normalised partial.
    int kr_lo, kr_hi, with_sink, cp_partial;
};

// ------------------------------------------------------------------------------------------------- prologue
// Packed two-float arithmetic (sm_100): a 64-bit register holds two floats.
__device__ __forceinline__ unsigned long long pack_f32x2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float &a, float &b) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v));
}
// (a, b) - m2, the operands given as float bit patterns
__device__ __forceinline__ void sub_f32x2(uint32_t a, uint32_t b, unsigned long long m2, float &o0, float &o1) {
    asm("{\n.reg .b64 x, z;\nmov.b64 x, {%2, %3};\nsub.rn.f32x2 z, x, %4;\nmov.b64 {%0, %1}, z;\n}\n"
        : "=f"(o0), "=f"(o1)
        : "r"(a), "r"(b), "l"(m2));
}
__device__ __forceinline__ void add_f32x2(unsigned long long &acc, float a, float b) {
    asm("{\n.reg .b64 x;\nmov.b64 x, {%1, %2};\nadd.rn.f32x2 %0, %0, x;\n}\n" : "+l"(acc) : "f"(a), "f"(b));
}

__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

struct PrologueArgs {
    const void *qkv;
    const float *q_norm, *k_norm, *inv_freq;
    __half *k_cache, *v_cache;  // [4][n_slots][128] of this sequence
    __half *q_st;               // [32][n_tok][128], pre-scaled by log2(e)/sqrt(128)
    __half *k_st, *v_st;        // [4][n_hist + n_tok][128] (ring layers only; null otherwise)
    int n_slots, is_swa, has_rope, qkv_dtype;
    int p0, n_tok, n_hist;
    const int32_t *block_table;  // paged full layer: k_cache / v_cache are page pools, slot = page * 64 + pos % 64
    int kv_lo, kv_hi;            // full layer: positions this device's cache holds (slot = pos - kv_lo); others are not stored
};

// A lane's share of an input row of 128: dims 4*sub..4*sub+3 and the four 64 further on, the partners of the first
// four under NEOX RoPE, so that the rotation needs no exchange between lanes.  Two 8-byte loads for bf16 rows, two
// 16-byte loads for fp32 rows; they stay packed in registers until the row is worked on, so that a warp has all its
// loads in flight first.
template <bool kBf16>
struct ProRaw;
template <>
struct ProRaw<true> {
    uint2 lo, hi;
    __device__ __forceinline__ void load(const void *base, size_t elem) {
        lo = *reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(base) + elem);
        hi = *reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(base) + elem + kHeadDim / 2);
    }
    __device__ __forceinline__ void unpack(float (&x)[8]) const {
        const uint32_t w[4] = {lo.x, lo.y, hi.x, hi.y};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <>
struct ProRaw<false> {
    float4 lo, hi;
    __device__ __forceinline__ void load(const void *base, size_t elem) {
        lo = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem);
        hi = *reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem + kHeadDim / 2);
    }
    __device__ __forceinline__ void unpack(float (&x)[8]) const {
        x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
    }
};

// x[0..3] -> dst[0..3], x[4..7] -> dst[64..67], as halves
__device__ __forceinline__ void pf_store_half44(__half *dst, const float (&v)[8]) {
    *reinterpret_cast<uint2 *>(dst) = make_uint2(pack_half2(v[0], v[1]), pack_half2(v[2], v[3]));
    *reinterpret_cast<uint2 *>(dst + kHeadDim / 2) = make_uint2(pack_half2(v[4], v[5]), pack_half2(v[6], v[7]));
}

// RMSNorm with weight, then NEOX RoPE with this token's (cos, sin) per owned pair of dims (the arithmetic of
// src/ref/ref_model.cpp:45-61; `extra` is 1 for keys), in packed two-float instructions: the kernel is bound by
// instruction issue.  A row of 128 lives in 16 lanes; the two halves of a warp hold two different rows.  x[j] and
// x[j + 4] are dims d and d + 64; cs2 / sn2 / nsn2 hold (cos, cos'), (sin, sin') and (-sin, -sin') of dims (d, d + 1)
// and (d + 2, d + 3); w2 the norm weights of dims (d, d+1), (d+2, d+3), (d+64, d+65), (d+66, d+67).
__device__ __forceinline__ void pf_norm_rope8(float (&x)[8], const unsigned long long (&w2)[4],
                                              const unsigned long long (&cs2)[2], const unsigned long long (&sn2)[2],
                                              const unsigned long long (&nsn2)[2], bool rope, float extra) {
    unsigned long long v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = pack_f32x2(x[2 * i], x[2 * i + 1]);
    unsigned long long acc = mul_f32x2(v[0], v[0]);
#pragma unroll
    for (int i = 1; i < 4; i++) acc = fma_f32x2(v[i], v[i], acc);
    float s0, s1;
    unpack_f32x2(acc, s0, s1);
    float ss = s0 + s1;
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float scale = 1.0f / sqrtf(ss / kHeadDim + kRmsEps) * extra;
    const unsigned long long scale2 = pack_f32x2(scale, scale);
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = mul_f32x2(mul_f32x2(v[i], scale2), w2[i]);
    if (rope) {
#pragma unroll
        for (int i = 0; i < 2; i++) {  // lo' = lo cos - hi sin, hi' = lo sin + hi cos
            const unsigned long long lo = v[i], hi = v[i + 2];
            v[i] = fma_f32x2(hi, nsn2[i], mul_f32x2(lo, cs2[i]));
            v[i + 2] = fma_f32x2(lo, sn2[i], mul_f32x2(hi, cs2[i]));
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) unpack_f32x2(v[i], x[2 * i], x[2 * i + 1]);
}

constexpr int kProRows = 10;  // input rows (heads) per warp: a token's 40 rows (32 q, 4 k, 4 v) take the four warps of a CTA

// New-token pass: one CTA of four warps per token, each warp with ten of its 40 head rows, two rows per pass (one per
// half-warp).  All loads of a warp go out before the first row is touched.  The token's 64 (cos, sin) pairs are
// evaluated once, by the first warp, and shared through shared memory.
template <bool kBf16>
__device__ __forceinline__ void prologue_rows(const PrologueArgs &a) {
    __shared__ float2 s_cs[kHeadDim / 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, pos = a.p0 + t, half = lane >> 4, sub = lane & 15;
    const bool rope = a.has_rope != 0;
    const size_t in0 = size_t(t) * kQkvDim + size_t(warp * kProRows + half) * kHeadDim + 4 * sub;

    ProRaw<kBf16> raw[kProRows / 2];
#pragma unroll
    for (int i = 0; i < kProRows / 2; i++) raw[i].load(a.qkv, in0 + size_t(2 * i) * kHeadDim);

    if (rope && warp == 0) {
        const float2 fr = reinterpret_cast<const float2 *>(a.inv_freq)[lane];
        float s0, c0, s1, c1;
        sincosf(float(pos) * fr.x, &s0, &c0);
        sincosf(float(pos) * fr.y, &s1, &c1);
        *reinterpret_cast<float4 *>(&s_cs[2 * lane]) = make_float4(c0, s0, c1, s1);
    }
    unsigned long long wq[4];
    {
        const float4 q0 = __ldg(reinterpret_cast<const float4 *>(a.q_norm) + sub);
        const float4 q1 = __ldg(reinterpret_cast<const float4 *>(a.q_norm) + 16 + sub);
        wq[0] = pack_f32x2(q0.x, q0.y); wq[1] = pack_f32x2(q0.z, q0.w);
        wq[2] = pack_f32x2(q1.x, q1.y); wq[3] = pack_f32x2(q1.z, q1.w);
    }
    const float sc = rsqrtf(float(kHeadDim)) * kLog2e;
    const int slot = a.is_swa ? (pos & (kSwaRing - 1)) : pos - a.kv_lo;  // prefill.metal:106
    const bool mine = a.is_swa || (pos >= a.kv_lo && pos < a.kv_hi);
    // On a ring layer tokens t and t + 1024 of one launch share a slot: only the last token that maps to a slot
    // stores there, so the ring's final contents do not depend on the order in which the CTAs run.
    const bool to_cache = mine && (!a.is_swa || t + kSwaRing >= a.n_tok);
    // paged layer: [page][kv head][64 slots][128] instead of [kv head][slot][128]
    const size_t page = a.block_table ? size_t(a.block_table[pos >> 6]) : 0;
    __syncthreads();
    unsigned long long cs[2], sn[2], nsn[2];
    cs[0] = cs[1] = pack_f32x2(1.f, 1.f);
    sn[0] = sn[1] = nsn[0] = nsn[1] = pack_f32x2(0.f, 0.f);
    if (rope) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float4 v = *reinterpret_cast<const float4 *>(&s_cs[4 * sub + 2 * j]);  // (cos, sin) of two dims
            cs[j] = pack_f32x2(v.x, v.z);
            sn[j] = pack_f32x2(v.y, v.w);
            nsn[j] = pack_f32x2(-v.y, -v.w);
        }
    }

#pragma unroll
    for (int i = 0; i < kProRows / 2; i++) {
        const int row = warp * kProRows + 2 * i + half;  // 0-31 q heads, 32-35 k heads, 36-39 v heads
        float x[8];
        raw[i].unpack(x);
        if (row < kNHead) {  // (both halves of the warp are on the same side of every row-kind boundary)
            pf_norm_rope8(x, wq, cs, sn, nsn, rope, sc);
            pf_store_half44(a.q_st + (size_t(row) * a.n_tok + t) * kHeadDim + 4 * sub, x);
            continue;
        }
        const bool is_k = row < kNHead + kNHeadKv;
        const int kvh = (row - kNHead) & (kNHeadKv - 1);
        if (is_k) {  // two of a token's twenty row pairs: the k weights are fetched here, not held all along
            const float4 k0 = __ldg(reinterpret_cast<const float4 *>(a.k_norm) + sub);
            const float4 k1 = __ldg(reinterpret_cast<const float4 *>(a.k_norm) + 16 + sub);
            const unsigned long long wk[4] = {pack_f32x2(k0.x, k0.y), pack_f32x2(k0.z, k0.w), pack_f32x2(k1.x, k1.y),
                                              pack_f32x2(k1.z, k1.w)};
            pf_norm_rope8(x, wk, cs, sn, nsn, rope, 1.0f);
        }
        if (to_cache) {
            __half *cache = is_k ? a.k_cache : a.v_cache;
            const size_t crow = a.block_table ? (page * kNHeadKv + kvh) * 64 + (pos & 63) : size_t(kvh) * a.n_slots + slot;
            pf_store_half44(cache + crow * kHeadDim + 4 * sub, x);
        }
        if (a.k_st) {
            __half *st = is_k ? a.k_st : a.v_st;
            pf_store_half44(st + (size_t(kvh) * (a.n_hist + a.n_tok) + a.n_hist + t) * kHeadDim + 4 * sub, x);
        }
    }
}

// History pass (ring layers with p0 > 0): one warp per (history row, kv head) copies the up to 512 keys before p0 out
// of the ring into the linear staging the attention kernel reads.  The history pass is its own, earlier launch: tokens
// p0+512.. of a long prompt land in the very ring slots the history occupies (which is why the reference prefills in
// chunks of at most 512, src/metal/flint_config.h:29-31).
__global__ void __launch_bounds__(256) k_prefill_history(const PrologueArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 8 + warp;
    if (row >= (long long)a.n_hist * kNHeadKv) return;
    const int r = int(row / kNHeadKv), kvh = int(row % kNHeadKv);
    const int pos = a.p0 - a.n_hist + r, slot = pos & (kSwaRing - 1);
    const size_t src = (size_t(kvh) * a.n_slots + slot) * kHeadDim + 4 * lane;
    const size_t dst = (size_t(kvh) * (a.n_hist + a.n_tok) + r) * kHeadDim + 4 * lane;
    *reinterpret_cast<uint2 *>(a.k_st + dst) = *reinterpret_cast<const uint2 *>(a.k_cache + src);
    *reinterpret_cast<uint2 *>(a.v_st + dst) = *reinterpret_cast<const uint2 *>(a.v_cache + src);
}

// (one kernel per input type: the bf16 one holds half the registers in flight and fits eight CTAs on an SM)
template <bool kBf16>
__global__ void __launch_bounds__(128, kBf16 ? 8 : 5) k_prefill_prologue(const PrologueArgs a) {
    // the attention kernel of this prefill may be scheduled as soon as SMs come free: it waits for this grid's
    // completion (griddepcontrol.wait) before it reads anything written here
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    prologue_rows<kBf16>(a);
}

// ------------------------------------------------------------------------------------------------- attention
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
    // Bounded by a count of polls, not by the clock: 2^24 polls are a quarter of a second when every poll returns at
    // once and longer when the hardware suspends the thread inside a poll, far beyond anything a healthy launch needs
    // (a launch may sit behind its predecessor on the stream for a while).  The loop is four instructions; with a
    // clock read and a second loop around it, inlined at some twenty waits, the kernel ran 3-4 % slower: its softmax
    // warps are short of instruction-cache, not of issue slots.  (An explicit suspend-time hint of a microsecond on
    // the poll, which would pin the upper end of the bound, cost 2 %: the waits then wake up later.)
#pragma unroll 1
    for (uint32_t n = 0; n < (1u << 24); n++)
        if (tc5::mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Barriers (8 bytes each, at kOffBar): the warps only ever talk through these.  Every barrier completes one phase
// per use, and each waiter counts its own uses, so the phase parities stay valid across the work units of a CTA.
enum {
    kBarSlotFull = 0,                       // [kSlots] TMA -> MMA warp: the K or V tile of the slot has landed
    kBarSlotEmpty = kBarSlotFull + kSlots,  // [kSlots] tensor core -> TMA warp: every product reading the slot is done
    kBarQFull = kBarSlotEmpty + kSlots,     // [2] TMA -> MMA warp: the Q tile of the unit is in shared memory
    kBarQEmpty = kBarQFull + 2,             // [2] tensor core -> TMA warp: the unit's last Q.K^T of this Q tile is done
    kBarSReady = kBarQEmpty + 2,            // [2] tensor core -> softmax warps: S = Q.K^T of the current tile
    kBarPReady = kBarSReady + 2,            // [2] softmax warps -> MMA warp: P is in its shared-memory tile (128 arrivals)
    kBarPvDone = kBarPReady + 2,            // [2] tensor core -> softmax warps: O += P.V of the current tile
    kBarOFree = kBarPvDone + 2,             // [2] softmax warps -> MMA warp: O of the finished unit has been read out (128)
    kBarSFree = kBarOFree + 2,              // [2] softmax warps -> MMA warp: S of the current tile is in registers (128)
    kNumBars = kBarSFree + 2
};

// A work unit: 32 consecutive query positions (two Q tiles of 16 positions x 8 heads) of one KV head, and, when the
// key range is split, one range of its key tiles.
struct Unit {
    int t0, kvh, q_first, q_last, klo, n_keys, n_tiles, split;
};
// Units are handed out longest first: late query blocks (full 544-key bands) before the first 16 blocks of the
// prompt, whose bands are shorter, so that the CTAs that get one unit more than the others get short ones.
// (Host and device: the host's schedule uses the same tile counts.)
__host__ __device__ inline Unit unit_geom_of(int u, int n_tok, int p0, int is_swa, int key_row0, int n_ksplit,
                                             int kr_lo = 0, int kr_hi = 0x7fffffff) {
    Unit g;
    const int uq = u / n_ksplit;
    g.split = u % n_ksplit;
    const int n_qb = (n_tok + kCtaPos - 1) / kCtaPos;
    g.t0 = (n_qb - 1 - uq / kNHeadKv) * kCtaPos;
    g.kvh = uq % kNHeadKv;
    g.q_first = p0 + g.t0;
    const int t_end = g.t0 + kCtaPos < n_tok ? g.t0 + kCtaPos : n_tok;
    g.q_last = p0 + t_end - 1;
    const int lo_swa = g.q_first - kHist > key_row0 ? g.q_first - kHist : key_row0;
    g.klo = is_swa ? lo_swa : (kr_lo > 0 ? kr_lo : 0);
    g.n_keys = (is_swa || g.q_last < kr_hi ? g.q_last + 1 : kr_hi) - g.klo;  // <= 0: the unit has no key on this device
    g.n_tiles = (g.n_keys + kBN - 1) / kBN;
    if (n_ksplit > 1) {  // the host guarantees at least 4 tiles per range; the last range takes the remainder
        const int per = g.n_tiles / n_ksplit;
        const int kt_a = g.split * per, kt_b = g.split == n_ksplit - 1 ? g.n_tiles : kt_a + per;
        const int left = g.n_keys - kt_a * kBN;
        g.klo += kt_a * kBN;
        g.n_keys = left < (kt_b - kt_a) * kBN ? left : (kt_b - kt_a) * kBN;
        g.n_tiles = kt_b - kt_a;
    }
    return g;
}
__device__ __forceinline__ Unit unit_geom(const PfArgs &a, int u) {
    return unit_geom_of(u, a.n_tok, a.p0, a.is_swa, a.key_row0, a.n_ksplit, a.kr_lo, a.kr_hi);
}

// The i-th unit of this CTA, or -1.  The host balances the units over the CTAs by their tile counts and lays each
// CTA's list out longest first; the CTA copies its list into shared memory at start (entries past kSchedLocal stay
// in global memory).  Without a table (at most one unit per CTA, or FLINT_ATTN_PREFILL_SCHEDULE=roundrobin in the
// environment) CTA b takes units b, b + grid, ...
__device__ __forceinline__ int unit_at(const PfArgs &a, const int *local, int i) {
    if (!a.sched) {
        const int u = int(blockIdx.x) + i * int(gridDim.x);
        return u < a.n_units ? u : -1;
    }
    if (i >= a.n_rounds) return -1;
    return i < kSchedLocal ? local[i] : __ldg(a.sched + size_t(i) * gridDim.x + blockIdx.x);
}

// Persistent: one CTA per SM, 384 threads, each CTA walks its list of units.
// Warps 0-3 own Q tile 0 of the unit (128 rows, one row per thread), warps 4-7 Q tile 1; warp 8 streams Q, K and V
// tiles with TMA (K and V alternate through a ring of three 32 KiB slots); warp 9 issues every tcgen05.mma.  The two
// Q tiles share each K/V tile and alternate on the tensor core: while one tile's warps run the softmax of a key tile,
// the tensor core does P.V and the next Q.K^T of the other -- across unit boundaries too, so the start-up of a unit
// (Q load, first scores) and the drain of the previous one (O / l, TMA store) overlap.  P goes through shared memory
// (so the next scores can be computed while the softmax runs); every product is 128 wide (N = 128; narrower MMAs
// run at half rate).
// (compiled per layer kind and output type: the code of the other three combinations would only take up
// instruction cache, which the softmax warps are short of)
template <bool kSwa, bool kOutF32>
__global__ void __launch_bounds__(kThreadsAttn, 1) k_prefill_attn(const __grid_constant__ CUtensorMap tm_q,
                                                                  const __grid_constant__ CUtensorMap tm_k,
                                                                  const __grid_constant__ CUtensorMap tm_v,
                                                                  const __grid_constant__ CUtensorMap tm_o,
                                                                  const PfArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    unsigned char *gen = smem_raw;
    if (base & 1023u) {  // swizzled tiles need 1024-byte alignment; nothing has been allocated yet
        if (threadIdx.x == 0) atomicExch(a.error_flag, 2);
        return;
    }
    auto bar = [&](int i) { return base + kOffBar + 8u * uint32_t(i); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(gen + kOffBar + 8 * kNumBars);
    volatile int *pace = reinterpret_cast<volatile int *>(gen + kOffBar + 8 * kNumBars + 8);  // units whose first tile Q tile 0 is through
    static_assert(8 * kNumBars + 16 <= 256, "barrier block");

    const int tid = threadIdx.x, warp = tid >> 5;
    int *sched_local = reinterpret_cast<int *>(gen + kOffSched);
    if (a.sched)
        for (int i = tid; i < min(a.n_rounds, kSchedLocal); i += kThreadsAttn)
            sched_local[i] = a.sched[size_t(i) * gridDim.x + blockIdx.x];

    if (tid == 0) {
        *pace = 0;
        for (int i = 0; i < kNumBars; i++) {
            const bool many = (i >= kBarPReady && i < kBarPReady + 2) || (i >= kBarOFree && i < kBarOFree + 4);
            const bool pair = i >= kBarSlotEmpty && i < kBarSlotEmpty + kSlots;  // one commit from each MMA issuer
            tc5::mbar_init(bar(i), many ? kBM : pair ? kQTiles : 1);
        }
        tc5::mbar_fence_init();
    }
    if (warp == 0) {
        tc5::tmem_alloc(base + kOffBar + 8 * kNumBars, kTmemCols);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    // Three warps share each SM sub-partition's 16K registers: the compiler's budget is 168 per thread.  The softmax
    // rows want ~200 (a whole 128-column score row in registers), the TMA / MMA warps few: move registers over.
    // (each role executes its own setmaxnreg first thing; warp 11 only completes the third warpgroup)
    if (warp >= 11) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n");
    } else if (warp == 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n");
        // =========================================================== TMA producer
        if ((tid & 31) == 0) {
            tc5::prefetch_tmap(&tm_q);
            tc5::prefetch_tmap(&tm_k);
            tc5::prefetch_tmap(&tm_v);
            // Programmatic dependent launch: this kernel may have been scheduled while the prologue still ran.  Nothing
            // the prologue writes (staged q, K/V staging, cache rows) is read before this wait, and every other warp of
            // the CTA only ever works on what this thread's loads bring in.
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
            int g = 0;  // tiles sent through the ring so far
            auto load_tile = [&](const CUtensorMap *map, const Unit &un, int kt) {
                // K of stream tile jt is done with as soon as both Q.K^T products of that tile are, early in the step;
                // V of tile jt only after its P.V products, a whole softmax later.  One slot that turns over every
                // step for K and two that alternate for V let K of tile jt+2 come in while V of tile jt is still
                // waited on, which a single ring through all three slots would not.
                const int jt = g >> 1;
                const int slot = (g & 1) ? 1 + (jt & 1) : 0, use = (g & 1) ? jt >> 1 : jt;
                g++;
                if (use >= 1 && !wait_bar(bar(kBarSlotEmpty + slot), (use - 1) & 1)) return false;
                const uint32_t dst = base + kOffKV + slot * kTileBytes, full = bar(kBarSlotFull + slot);
                const int row = un.klo + kt * kBN - a.key_row0;
                tc5::mbar_expect_tx(full, kTileBytes);
                if (a.block_table) {
                    // a 128-key tile is two pages; a page past the sequence's last one holds only keys that every
                    // query of the unit has masked, so any resident page stands in for it
                    for (int rh = 0; rh < 2; rh++) {
                        const int blk = (row >> 6) + rh;
                        int page = blk < a.table_len ? __ldg(a.block_table + blk) : -1;
                        if (page < 0) page = 0;
                        const uint32_t d = dst + rh * (kTileBytes / 4);
                        tc5::tma_load_3d(d, map, full, 0, 0, page * kNHeadKv + un.kvh);
                        tc5::tma_load_3d(d + kTileBytes / 2, map, full, 64, 0, page * kNHeadKv + un.kvh);
                    }
                    return true;
                }
                tc5::tma_load_3d(dst, map, full, 0, row, un.kvh);
                tc5::tma_load_3d(dst + kTileBytes / 2, map, full, 64, row, un.kvh);
                return true;
            };
            auto load_q = [&](const Unit &un, int w, int i) {
                if (i >= 1 && !wait_bar(bar(kBarQEmpty + w), (i - 1) & 1)) return false;
                const uint32_t dst = base + kOffQ + w * kQBytes, full = bar(kBarQFull + w);
                tc5::mbar_expect_tx(full, kQBytes);
                tc5::tma_load_3d(dst, &tm_q, full, 0, un.t0 + w * kQPos, un.kvh * kGqa);
                tc5::tma_load_3d(dst + kQBytes / 2, &tm_q, full, 64, un.t0 + w * kQPos, un.kvh * kGqa);
                return true;
            };
            for (int i = 0; ok; i++) {
                const int u = unit_at(a, sched_local, i);
                if (u < 0) break;
                const Unit un = unit_geom(a, u);
                // order of need: Q0, K(0), Q1, V(0), K(1), V(1), ...
                ok = load_q(un, 0, i) && load_tile(&tm_k, un, 0) && load_q(un, 1, i);
                for (int kt = 0; kt < un.n_tiles && ok; kt++) {
                    ok = load_tile(&tm_v, un, kt);
                    if (ok && kt + 1 < un.n_tiles) ok = load_tile(&tm_k, un, kt + 1);
                }
            }
            if (!ok) atomicExch(a.error_flag, 1);
        }
    } else if (warp == 9 || warp == 10) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n");
        // =========================================================== MMA issuers (warp-uniform code, one lane issues)
        // One issuer per Q tile: warp 9 for tile 0, warp 10 for tile 1.  Each walks the same stream of key tiles and
        // waits only on its own tile's softmax, so a tile whose softmax runs behind the other's never holds up the
        // other's products: the two tiles drift half a step apart, and one tile's exponentials (the special-function
        // unit) run under the other's loads, maxima and waits instead of at the same time.
        const int w = warp - 9;
        const uint32_t leader = (tid & 31) == 0;
        constexpr uint32_t kDescHi = tc5::desc_hi_sw128(1024);
        constexpr uint32_t kIdescPV = tc5::idesc_f16(kBM, kHeadDim, 0, 1);  // A = P (shared memory), B = V (MN-major)
        const uint32_t q_lo = tc5::desc_lo(base + kOffQ, 16) + w * (kQBytes >> 4);
        const uint32_t p_lo = tc5::desc_lo(base + kOffStage, 16) + w * (kPBytes >> 4);  // P tile: K-major, two 64-key halves
        const uint32_t k_lo = tc5::desc_lo(base + kOffKV, 16);               // K tile: K-major, two 64-dim halves
        const uint32_t v_lo = tc5::desc_lo(base + kOffKV, kTileBytes / 2);   // V tile: MN-major, LBO = the other 64 dims
        // The key tiles of all units of this CTA form one stream; tile j of the stream has its K in slot 0 (use j) and
        // its V in slot 1 + j % 2 (use j / 2).  For each tile: Q.K^T of the NEXT tile of the stream (S is free again as
        // soon as the softmax has read the current scores into registers), possibly of the next unit, then P.V of the
        // current one when its P has been written.
        struct Cursor {
            int i, kt, j;  // index of the unit in this CTA's list, tile in the unit, tile in the stream
            Unit un;
        };
        // keys of a tile that any query of the unit can see, rounded up to the MMA's N granularity
        auto tile_n = [&](const Cursor &c) { return min(kBN, (c.un.n_keys - c.kt * kBN + 15) & ~15); };
        auto advance = [&](Cursor &c) {  // returns false at the end of the stream
            if (c.kt + 1 < c.un.n_tiles) {
                c.kt++;
            } else {
                const int u = unit_at(a, sched_local, c.i + 1);
                if (u < 0) return false;
                c.i++;
                c.kt = 0;
                c.un = unit_geom(a, u);
            }
            c.j++;
            return true;
        };
        auto issue_qk = [&](const Cursor &c) {
            const int slot = 0;
            if (c.j >= 1 && !wait_bar(bar(kBarSFree + w), (c.j - 1) & 1)) return false;  // the previous scores are read out
            if (c.kt == 0 && !wait_bar(bar(kBarQFull + w), c.i & 1)) return false;
            if (!wait_bar(bar(kBarSlotFull + slot), c.j & 1)) return false;
            tc5::fence_after_sync();
            const uint32_t kst = k_lo + uint32_t(slot) * (kTileBytes >> 4);
            const uint32_t idesc = tc5::idesc_f16(kBM, tile_n(c), 0, 0);  // A = Q (K-major), B = K (K-major)
#pragma unroll
            for (int ks = 0; ks < kHeadDim / 16; ks++) {
                const uint32_t off = (ks >> 2) * ((kTileBytes / 2) >> 4) + (ks & 3) * 2;  // Q and K halves are both 16 KiB
                tc5::mma_f16_ss_lohi_w(tmem + kColS + w * kBN, q_lo + off, kst + off, kDescHi, idesc, ks > 0, leader);
            }
            tc5::mma_commit_w(bar(kBarSReady + w), leader);
            if (c.kt == c.un.n_tiles - 1) tc5::mma_commit_w(bar(kBarQEmpty + w), leader);  // last use of this Q tile
            tc5::mma_commit_w(bar(kBarSlotEmpty + slot), leader);  // (the slot is free when both issuers have said so)
            return true;
        };
        auto issue_pv = [&](const Cursor &c) {
            const int slot = 1 + (c.j & 1);
            if (!wait_bar(bar(kBarPReady + w), c.j & 1)) return false;
            if (c.kt == 0 && c.i >= 1 && !wait_bar(bar(kBarOFree + w), (c.i - 1) & 1)) return false;
            if (!wait_bar(bar(kBarSlotFull + slot), (c.j >> 1) & 1)) return false;
            tc5::fence_after_sync();
            const uint32_t vst = v_lo + uint32_t(slot) * (kTileBytes >> 4);
            const int n_steps = tile_n(c) / 16;
#pragma unroll
            for (int ks = 0; ks < kBN / 16; ks++)
                if (ks < n_steps)
                    tc5::mma_f16_ss_lohi_w(tmem + kColO + w * kHeadDim, p_lo + (ks >> 2) * ((kPBytes / 2) >> 4) + (ks & 3) * 2,
                                           vst + ks * (2048 >> 4), kDescHi, kIdescPV, (c.kt > 0 || ks > 0), leader);
            tc5::mma_commit_w(bar(kBarPvDone + w), leader);
            tc5::mma_commit_w(bar(kBarSlotEmpty + slot), leader);
            return true;
        };
        if (unit_at(a, sched_local, 0) >= 0) {
            Cursor cur{0, 0, 0, unit_geom(a, unit_at(a, sched_local, 0))};
            ok = issue_qk(cur);
            while (ok) {
                Cursor nxt = cur;
                const bool more = advance(nxt);
                // The next scores are issued as soon as the current ones have been read into registers, so they are
                // computed while the softmax of the current tile runs; P.V follows when P has been written.  Across a
                // unit boundary the order turns round: the next unit's Q tile is still on its way, and the last P.V is
                // what the softmax warps wait for before they can write the unit out.
                if (more && nxt.kt != 0) ok = issue_qk(nxt);
                ok = ok && issue_pv(cur);
                if (more && nxt.kt == 0) ok = ok && issue_qk(nxt);
                if (!more) break;
                cur = nxt;
            }
            if (!ok && leader) atomicExch(a.error_flag, 1);
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;\n");
        // =========================================================== softmax warps: one query row per thread
        const int w = warp >> 2;                   // Q tile of this warp
        const int r = tid & (kBM - 1);             // row in the tile = head-in-group * 16 + position-in-tile
        const int hl = r >> 4, qi = r & 15;
        const uint32_t lane_base = tmem + (uint32_t((warp & 3) * 32) << 16);
        const uint32_t colS = lane_base + kColS + w * kBN, colO = lane_base + kColO + w * kHeadDim;
        int j = 0;  // tiles of the stream seen so far (phase of the S / P / P.V barriers)
        for (int i = 0; ok; i++) {
        const int u = unit_at(a, sched_local, i);
        if (u < 0) break;
        const Unit un = unit_geom(a, u);
        const int kvh = un.kvh, t0 = un.t0, klo = un.klo, n_keys = un.n_keys, n_tiles = un.n_tiles;
        const int qt_first = un.q_first + w * kQPos;  // first / last position of this Q tile
        const int qt_last = min(qt_first + kQPos - 1, un.q_last);
        const int qpos = qt_first + qi;
        const float sink2 = a.sinks[kvh * kGqa + hl] * kLog2e;

        // prefill.metal:162: the sink enters through m0 = sink, l0 = 1 -- once per row, so with a split key range
        // only the first range carries it (the others start empty; their first tile is fully visible, so m gets finite)
        const bool has_sink = un.split == 0 && a.with_sink;
        float m = has_sink ? sink2 : -INFINITY, l = has_sink ? 1.0f : 0.0f;
        for (int kt = 0; kt < n_tiles && ok; kt++) {
            ok = __all_sync(0xffffffffu, wait_bar(bar(kBarSReady + w), j & 1));  // warp-uniform for tcgen05.ld
            if (!ok) break;
            tc5::fence_after_sync();
            const int kbase = klo + kt * kBN;
            const int n_cols = min(kBN, (n_keys - kt * kBN + 15) & ~15);  // columns the MMA wrote (same as the issuer)
            const int n_chunks = (n_cols + 31) >> 5;
            // visible columns of this row form one range [c_lo, c_hi] (prefill.metal:212); on a key-range shard the
            // unit's keys also end with the shard (k_end), before the causal limit of later queries
            const int k_end = klo + n_keys - 1;
            const int c_hi = min(qpos, k_end) - kbase;
            const int c_lo = kSwa ? qpos - kHist - kbase : -(1 << 30);
            // Per 32-column chunk, for the whole Q tile: 0 = every row sees every key (no per-element mask),
            // 1 = mixed, 2 = no row sees any key.  Only the two ends of the band are mixed.
            auto chunk_kind = [&](int ch) {
                const int key_lo = kbase + ch * 32, key_hi = key_lo + 31;
                if (key_lo > qt_last || key_lo > k_end || (kSwa && key_hi < qt_first - kHist)) return 2;
                if (key_hi <= qt_first && key_hi <= k_end && (!kSwa || key_lo >= qt_last - kHist)) return 0;
                return 1;
            };

            // the whole row of S into registers: all loads in flight at once, one wait
            uint32_t sr[kBN];
#pragma unroll
            for (int ch = 0; ch < kBN / 32; ch++)
                if (ch < n_chunks) tc5::tmem_ld32(colS + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[ch * 32]));
            tc5::tmem_wait_ld();
            tc5::fence_before_sync();
            tc5::mbar_arrive(bar(kBarSFree + w));  // S is in registers: the next scores may overwrite it
            // Band-edge tiles (the first and the last of a unit): invisible scores become -inf, per 32-column chunk and
            // only in chunks that some row of the Q tile sees partly; interior tiles skip all of it on uniform branches.
            if (chunk_kind(0) != 0 || chunk_kind(n_chunks - 1) != 0) {
                const uint32_t span = uint32_t(c_hi - c_lo);
#pragma unroll
                for (int ch = 0; ch < kBN / 32; ch++) {
                    if (ch < n_chunks && chunk_kind(ch) != 0) {
#pragma unroll
                        for (int c = 0; c < 32; c++)  // visible iff c_lo <= col <= c_hi
                            if (uint32_t(ch * 32 + c - c_lo) > span) sr[ch * 32 + c] = 0xff800000u;
                    }
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < kBN / 32; ch++) {
                if (ch < n_chunks) {
                    float t4[4];
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        t4[c] = max3(fmaxf(__uint_as_float(sr[ch * 32 + 8 * c]), __uint_as_float(sr[ch * 32 + 8 * c + 1])),
                                     max3(__uint_as_float(sr[ch * 32 + 8 * c + 2]), __uint_as_float(sr[ch * 32 + 8 * c + 3]),
                                          __uint_as_float(sr[ch * 32 + 8 * c + 4])),
                                     max3(__uint_as_float(sr[ch * 32 + 8 * c + 5]), __uint_as_float(sr[ch * 32 + 8 * c + 6]),
                                          __uint_as_float(sr[ch * 32 + 8 * c + 7])));
                    mx = fmaxf(mx, fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3])));
                }
            }
            // lazy rescale: keep the old reference maximum unless the row maximum outgrew it by more than 2^8
            float corr = 1.0f;
            if (kt == 0) {
                m = fmaxf(m, mx);
                l = has_sink ? fast_exp2(sink2 - m) : 0.0f;  // the sink's share of the denominator under the new maximum
            } else if (mx > m + 8.0f) {
                corr = fast_exp2(m - mx);
                m = mx;
                l *= corr;
            }
            if (j >= 1) {
                // O and the P buffer belong to the tensor core until P.V of the previous tile of the stream is done
                // (it usually is by now: it was issued a whole softmax ago)
                ok = __all_sync(0xffffffffu, wait_bar(bar(kBarPvDone + w), (j - 1) & 1));
                if (!ok) break;
                tc5::fence_after_sync();
            }
            if (kt == 0 && i >= 1) {  // the P buffer doubles as output staging: the previous unit's store must have read it
                if (r == 0) tc5::tma_store_wait_read();
                if (w == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
                else asm volatile("bar.sync 2, 128;\n" ::: "memory");
            }
            if (kt >= 1 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // rare
#pragma unroll 1
                for (int cb = 0; cb < kHeadDim; cb += 32) {
                    uint32_t rr[32];
                    tc5::tmem_ld32(colO + cb, rr);
                    tc5::tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; c++) rr[c] = __float_as_uint(__uint_as_float(rr[c]) * corr);
                    tc5::tmem_st32(colO + cb, rr);
                }
                tc5::tmem_wait_st();
                tc5::fence_before_sync();
            }
            // The two Q tiles work half a step apart.  A tile's exponentials alone keep the special-function unit
            // busy; when both tiles run them at once each takes twice as long, and the unit then idles through both
            // tiles' loads, maxima and waits.  With its own MMA issuer a tile that runs behind stays behind, so it is
            // enough to hold tile 1 back once per unit: it starts its first exponentials of the unit when tile 0 has
            // finished its own.  This is pacing only: the wait gives up after a few microseconds and nothing depends
            // on it.
            if (w == 1 && kt == 0) {
                const long long t_pace = clock64();
                while (*pace < i + 1 && clock64() - t_pace < 16384) {
                }
            }
            // probabilities: P (half) goes to this Q tile's shared-memory block in the K-major 128-byte-swizzled layout
            // of an MMA A operand: two 64-key halves of [128 rows][128 B]
            // A row that has not seen a visible key yet (a key-range shard that starts after its position) still has
            // m = -inf: its scores are all -inf, and against a finite stand-in they give p = 0 instead of a NaN.
            const float mref = m == -INFINITY ? 0.0f : m;
            // The subtraction of the reference maximum and the row sums run as packed two-float instructions: a
            // quarter fewer instructions in the exponential phase, whose issue slots and instruction fetches the two
            // softmax warps of a scheduler compete for.
            const unsigned long long mref2 = pack_f32x2(mref, mref);
            unsigned long long sum01 = pack_f32x2(0.f, 0.f), sum23 = sum01;
#pragma unroll
            for (int ch = 0; ch < kBN / 32; ch++) {
                if (ch < n_chunks) {
                    uint32_t pw[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        float d0, d1, d2, d3;
                        sub_f32x2(sr[ch * 32 + c], sr[ch * 32 + c + 1], mref2, d0, d1);
                        sub_f32x2(sr[ch * 32 + c + 2], sr[ch * 32 + c + 3], mref2, d2, d3);
                        const float p0 = fast_exp2(d0), p1 = fast_exp2(d1), p2 = fast_exp2(d2), p3 = fast_exp2(d3);
                        add_f32x2(sum01, p0, p1);
                        add_f32x2(sum23, p2, p3);
                        pw[c >> 1] = pack_half2(p0, p1);
                        pw[(c >> 1) + 1] = pack_half2(p2, p3);
                    }
                    unsigned char *prow = gen + kOffStage + w * kPBytes + (ch >> 1) * (kPBytes / 2) + r * 128;
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        *reinterpret_cast<uint4 *>(prow + ((((ch & 1) * 4 + q) ^ (r & 7)) << 4)) =
                            make_uint4(pw[4 * q], pw[4 * q + 1], pw[4 * q + 2], pw[4 * q + 3]);
                }
            }
            {
                float s0, s1, s2, s3;
                unpack_f32x2(sum01, s0, s1);
                unpack_f32x2(sum23, s2, s3);
                l += (s0 + s1) + (s2 + s3);
            }
            tc5::fence_proxy_async();
            tc5::mbar_arrive(bar(kBarPReady + w));
            if (w == 0 && kt == 0 && r == 0) *pace = i + 1;
            j++;
        }
        // ---- drain of the unit.  The scores of the last tile proved P.V of the tile before it done, so a parity wait
        // for the last tile is well defined.
        if (ok) ok = __all_sync(0xffffffffu, wait_bar(bar(kBarPvDone + w), (j - 1) & 1));
        if (!ok) break;
        {
            // O / l (prefill.metal:255-265) goes out through a staging tile of this Q tile: each thread drops its row
            // into an [8 heads][16 positions][128 B] swizzled block per 128-byte column block, then one thread hands
            // the blocks to TMA, which writes full lines and clips rows past the prompt.  bf16 rows fit the two staging
            // blocks at once; fp32 rows go out in two rounds.  The TMA store of a unit drains while the next unit runs.
            tc5::fence_after_sync();
            const bool partial = a.n_ksplit > 1 || a.cp_partial;
            const float inv_l = partial ? 1.0f : 1.0f / l;
            constexpr bool f32 = kOutF32;
            const int row0 = un.t0 + w * kQPos + un.split * a.t_pad;  // row of the output tensor this Q tile starts at
            if (partial && un.t0 + w * kQPos + qi < a.n_tok)
                a.part_ml[size_t(row0 + qi) * kNHead + kvh * kGqa + hl] = make_float2(m, l);
            const uint32_t stage_off = kOffStage + w * 2 * kOutBlockBytes;
            unsigned char *stg = gen + stage_off + r * 128;
            const int sw = r & 7;
            const bool tile_valid = t0 + w * kQPos < a.n_tok;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                if (half == 0 || f32) {  // the previous store out of these blocks must have read them
                    if (r == 0) tc5::tma_store_wait_read();
                    if (w == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");  // the four warps of this Q tile only
                    else asm volatile("bar.sync 2, 128;\n" ::: "memory");
                }
                // 64 columns of the accumulator row per round: both loads in flight, one wait
                uint32_t oo[64];
                tc5::tmem_ld32(colO + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&oo[0]));
                tc5::tmem_ld32(colO + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&oo[32]));
                tc5::tmem_wait_ld();
                if (half == 1) {  // O is in registers: the next unit may overwrite the accumulator
                    tc5::fence_before_sync();
                    tc5::mbar_arrive(bar(kBarOFree + w));
                }
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const uint32_t(&rr)[32] = *reinterpret_cast<const uint32_t(*)[32]>(&oo[q * 32]);
                    if (f32) {
                        unsigned char *blk = stg + q * kOutBlockBytes;
#pragma unroll
                        for (int c = 0; c < 8; c++)
                            *reinterpret_cast<float4 *>(blk + ((c ^ sw) << 4)) =
                                make_float4(__uint_as_float(rr[4 * c]) * inv_l, __uint_as_float(rr[4 * c + 1]) * inv_l,
                                            __uint_as_float(rr[4 * c + 2]) * inv_l, __uint_as_float(rr[4 * c + 3]) * inv_l);
                    } else {
                        unsigned char *blk = stg + half * kOutBlockBytes;
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            uint32_t wd[4];
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(rr[8 * c + 2 * e]) * inv_l,
                                                                               __uint_as_float(rr[8 * c + 2 * e + 1]) * inv_l);
                                wd[e] = *reinterpret_cast<const uint32_t *>(&b);
                            }
                            *reinterpret_cast<uint4 *>(blk + ((4 * q + c) ^ sw) * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
                        }
                    }
                }
                if (half == 1 || f32) {
                    tc5::fence_proxy_async();
                    if (w == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
                    else asm volatile("bar.sync 2, 128;\n" ::: "memory");
                    if (r == 0 && tile_valid) {
                        for (int b = 0; b < 2; b++)
                            tc5::tma_store_3d(&tm_o, base + stage_off + b * kOutBlockBytes, f32 ? half * 64 + b * 32 : b * 64,
                                              row0, kvh * kGqa);
                        tc5::tma_store_commit();
                    }
                }
            }
        }
        }  // units
        if (!ok && (tid & 31) == 0) atomicExch(a.error_flag, 1);  // a wait ran out: report, then the normal teardown
        if (r == 0) tc5::tma_store_wait_read();                    // shared memory must outlive the last store's reads
    }
    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc5::tmem_dealloc(tmem, kTmemCols);
}

// Merge of the key-range partials of one chunk: out[t][head][:] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M)
// (the log-sum-exp merge of src/metal/fused.metal:332-350 applied to prefill rows; the sink is inside range 0's l).
// One CTA per (token, 4 heads), thread = (head, 4 dims).
// With ml_out the result stays a partial: the un-normalised sum at the common maximum and its (M, L), for a later
// merge with the other devices' partials.
__global__ void __launch_bounds__(128) k_prefill_merge(const float *part_o, const float2 *part_ml, void *out, int out_dtype,
                                                       int n_tok, int t_pad, int n_ksplit, float2 *ml_out) {
    const int t = blockIdx.x / (kNHead / 4);
    const int head = (blockIdx.x % (kNHead / 4)) * 4 + (threadIdx.x >> 5);
    const int d = (threadIdx.x & 31) * 4;
    float M = -INFINITY;
    for (int s = 0; s < n_ksplit; s++) {
        const float2 ml = part_ml[(size_t(s) * t_pad + t) * kNHead + head];
        if (ml.y != 0.f) M = fmaxf(M, ml.x);
    }
    float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_ksplit; s++) {
        const float2 ml = part_ml[(size_t(s) * t_pad + t) * kNHead + head];
        if (ml.y == 0.f) continue;  // an empty part (no key of this row in the range): its rows were never written
        const float c = exp2f(ml.x - M);
        const float4 o = *reinterpret_cast<const float4 *>(part_o + (size_t(s) * t_pad + t) * kQDim + head * kHeadDim + d);
        L += ml.y * c;
        acc[0] += o.x * c; acc[1] += o.y * c; acc[2] += o.z * c; acc[3] += o.w * c;
    }
    const float inv = ml_out ? 1.0f : 1.0f / L;
    if (ml_out && d == 0) ml_out[size_t(t) * kNHead + head] = make_float2(L == 0.f ? 0.f : M, L);
    const size_t idx = size_t(t) * kQDim + head * kHeadDim + d;
    if (out_dtype == kDtypeF32) {
        *reinterpret_cast<float4 *>(static_cast<float *>(out) + idx) =
            make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    } else {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
        *reinterpret_cast<uint2 *>(static_cast<__nv_bfloat16 *>(out) + idx) =
            make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
}

// ------------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
int g_sm_count = 148;

// half tensor [n_outer][n_rows][128] viewed as 3-D {128, n_rows, n_outer}, box {64, box_rows, box_outer}
cudaError_t make_map(CUtensorMap *map, const void *base, int n_rows, int n_outer, int box_rows, int box_outer) {
    const cuuint64_t dims[3] = {cuuint64_t(kHeadDim), cuuint64_t(n_rows), cuuint64_t(n_outer)};
    const cuuint64_t strides[2] = {cuuint64_t(kHeadDim) * 2, cuuint64_t(n_rows) * kHeadDim * 2};
    const cuuint32_t box[3] = {64, cuuint32_t(box_rows), cuuint32_t(box_outer)};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// output [n_tok][32][128] (bf16 or f32) viewed as {128 dims, n_tok, 32 heads}; box = one 128-byte column block x 16
// tokens x 8 heads, so that the shared-memory tile has the kernel's row order (head-major)
cudaError_t make_out_map(CUtensorMap *map, void *base, int n_tok, int out_dtype) {
    const cuuint64_t es = out_dtype == kDtypeF32 ? 4 : 2;
    const cuuint64_t dims[3] = {cuuint64_t(kHeadDim), cuuint64_t(n_tok), cuuint64_t(kNHead)};
    const cuuint64_t strides[2] = {cuuint64_t(kQDim) * es, cuuint64_t(kHeadDim) * es};
    const cuuint32_t box[3] = {cuuint32_t(128 / es), cuuint32_t(kQPos), cuuint32_t(kGqa)};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode(map, out_dtype == kDtypeF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Which CTA runs which units.  Units differ in length (the first query blocks of a prompt see fewer keys; on a full
// layer the band grows with the position), so handing them out round-robin leaves some CTAs with up to a third more
// tiles than others.  Greedy longest-first assignment to the least loaded CTA by (key tiles + one tile of per-unit
// overhead); unit indices are already ordered longest first.  The table is kept until the geometry changes.
cudaError_t build_schedule(PrefillWorkspace &ws, const PfArgs &a, int n_units, int grid, cudaStream_t stream) {
    const int key[5] = {a.n_tok, a.p0, a.is_swa * 256 + a.n_ksplit, a.key_row0 ^ (a.kr_hi * 31), grid};
    if (ws.sched && memcmp(key, ws.sched_key, sizeof(key)) == 0) return cudaSuccess;
    std::vector<std::vector<int>> lists(grid);
    std::priority_queue<std::pair<int, int>, std::vector<std::pair<int, int>>, std::greater<std::pair<int, int>>> heap;
    for (int b = 0; b < grid; b++) heap.push({0, b});
    for (int u = 0; u < n_units; u++) {
        const int tiles = unit_geom_of(u, a.n_tok, a.p0, a.is_swa, a.key_row0, a.n_ksplit, a.kr_lo, a.kr_hi).n_tiles;
        const auto [load, b] = heap.top();
        heap.pop();
        lists[b].push_back(u);
        heap.push({load + tiles + 1, b});
    }
    size_t rounds = 0;
    for (const auto &l : lists) rounds = std::max(rounds, l.size());
    std::vector<int> table(rounds * grid, -1);
    for (int b = 0; b < grid; b++)
        for (size_t i = 0; i < lists[b].size(); i++) table[i * grid + b] = lists[b][i];
    cudaError_t e;
    if (table.size() > ws.sched_cap) {
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return e;  // an earlier launch may still read the old one
        cudaFree(ws.sched);
        ws.sched = nullptr;
        ws.sched_cap = 0;
        if ((e = cudaMalloc(&ws.sched, table.size() * 2 * sizeof(int))) != cudaSuccess) return e;
        ws.sched_cap = table.size() * 2;
    }
    // pageable source: staged by the runtime before the call returns, ordered on the stream behind earlier launches
    if ((e = cudaMemcpyAsync(ws.sched, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice, stream)) != cudaSuccess)
        return e;
    memcpy(ws.sched_key, key, sizeof(key));
    ws.sched_rounds = int(rounds);
    return cudaSuccess;
}

}  // namespace

cudaError_t prefill_kernel_setup() {
    if (!g_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (!fn || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(k_prefill_attn<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_prefill_attn<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_prefill_attn<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_prefill_attn<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    return e;
}

void prefill_workspace_free(PrefillWorkspace &ws) {
    cudaFree(ws.buf);
    cudaFree(ws.sched);
    ws = PrefillWorkspace{};
}

cudaError_t launch_prefill(const PrefillParams &p, PrefillWorkspace &ws, cudaStream_t stream, int *n_launches) {
    *n_launches = 0;
    const int T = p.n_tok;
    const int n_hist = p.is_swa ? (p.p0 < kHist ? p.p0 : kHist) : 0;
    auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
    const size_t q_bytes = up(size_t(kNHead) * T * kHeadDim * 2);
    const size_t kv_bytes = p.is_swa ? up(size_t(kNHeadKv) * (n_hist + T) * kHeadDim * 2) : 0;
    // Key-range split: a chunk on a full layer with fewer units than SMs and a long history leaves most of the GPU
    // idle (512 tokens = 64 units) while every unit walks hundreds of key tiles.  Each unit is then cut into ranges
    // of at least 4 key tiles, as many as fit the SMs, and a small kernel merges the partials.
    // A key-range shard [kv_lo, kv_hi) of a full layer only has work for query blocks that end at or after kv_lo.
    // Units are numbered from the last query block down, so those form a prefix of the numbering.
    const bool cp = p.partial_o != nullptr;
    const int kr_lo = p.is_swa ? 0 : p.kv_lo, kr_hi = p.is_swa ? 0x7fffffff : p.kv_hi;
    const int n_qb = (T + kCtaPos - 1) / kCtaPos;
    // (the last block ends at p0 + T - 1; if even that lies before kv_lo, no block has a key here)
    const int first_block = p.p0 + T - 1 < kr_lo ? n_qb : std::max(0, (kr_lo - p.p0) / kCtaPos);
    const int n_units_q = (n_qb - first_block) * kNHeadKv;
    // every unit handed to the kernel must own at least one key: a unit without keys would issue products of width 0
    if (n_units_q > 0 && (unit_geom_of(n_units_q - 1, T, p.p0, p.is_swa, p.is_swa ? p.p0 - n_hist : kr_lo, 1, kr_lo, kr_hi).n_keys <= 0 ||
                          unit_geom_of(0, T, p.p0, p.is_swa, p.is_swa ? p.p0 - n_hist : kr_lo, 1, kr_lo, kr_hi).n_keys <= 0))
        return cudaErrorInvalidValue;
    int n_ksplit = 1;
    if (!p.is_swa && n_units_q > 0 && n_units_q * 2 <= g_sm_count) {
        // the shortest unit's tiles (the first query block that has keys here)
        const int min_tiles = unit_geom_of(n_units_q - 1, T, p.p0, 0, 0, 1, kr_lo, kr_hi).n_tiles;
        n_ksplit = std::max(1, std::min(g_sm_count / n_units_q, min_tiles / 4));
    }
    const int t_pad = (T + kCtaPos - 1) / kCtaPos * kCtaPos;
    const size_t part_o_bytes = n_ksplit > 1 ? up(size_t(n_ksplit) * t_pad * kQDim * sizeof(float)) : 0;
    const size_t part_ml_bytes = n_ksplit > 1 ? up(size_t(n_ksplit) * t_pad * kNHead * sizeof(float2)) : 0;
    const size_t need = q_bytes + 2 * kv_bytes + part_o_bytes + part_ml_bytes + 1024;
    if (need > ws.cap) {
        cudaError_t e = cudaDeviceSynchronize();  // an earlier launch may still be reading the old staging
        if (e != cudaSuccess) return e;
        cudaFree(ws.buf);
        ws.buf = nullptr;
        ws.cap = 0;
        e = cudaMalloc(&ws.buf, need);
        if (e != cudaSuccess) return e;
        ws.cap = need;
        e = cudaMemset(ws.buf, 0, 1024);
        if (e != cudaSuccess) return e;
    }
    char *wbase = static_cast<char *>(ws.buf);
    int *err_flag = reinterpret_cast<int *>(wbase);
    __half *q_st = reinterpret_cast<__half *>(wbase + 1024);
    __half *k_st = p.is_swa ? reinterpret_cast<__half *>(wbase + 1024 + q_bytes) : nullptr;
    __half *v_st = p.is_swa ? reinterpret_cast<__half *>(wbase + 1024 + q_bytes + kv_bytes) : nullptr;
    float *part_o = reinterpret_cast<float *>(wbase + 1024 + q_bytes + 2 * kv_bytes);
    float2 *part_ml = reinterpret_cast<float2 *>(wbase + 1024 + q_bytes + 2 * kv_bytes + part_o_bytes);

    PrologueArgs pa{};
    pa.qkv = p.qkv; pa.q_norm = p.q_norm; pa.k_norm = p.k_norm; pa.inv_freq = p.inv_freq;
    pa.k_cache = p.k_cache; pa.v_cache = p.v_cache;
    pa.q_st = q_st; pa.k_st = k_st; pa.v_st = v_st;
    pa.n_slots = p.n_slots; pa.is_swa = p.is_swa; pa.has_rope = p.has_rope; pa.qkv_dtype = p.qkv_dtype;
    pa.p0 = p.p0; pa.n_tok = T; pa.n_hist = n_hist;
    pa.block_table = p.block_table;
    pa.kv_lo = p.is_swa ? 0 : p.kv_lo;
    pa.kv_hi = p.is_swa ? 0x7fffffff : p.kv_hi;
    cudaError_t e;
    // The prologue is launched last, directly in front of the attention kernel, so that the two are neighbours on the
    // stream: the attention kernel is launched with programmatic stream serialisation and sets itself up (tensor
    // memory, barriers, work list) on SMs the prologue has already left.
    auto launch_prologue = [&]() -> cudaError_t {
        if (n_hist > 0) {
            k_prefill_history<<<unsigned((n_hist * kNHeadKv + 7) / 8), 256, 0, stream>>>(pa);
            if (cudaError_t le = cudaGetLastError(); le != cudaSuccess) return le;
            (*n_launches)++;
        }
        if (pa.qkv_dtype == kDtypeBf16) k_prefill_prologue<true><<<unsigned(T), 128, 0, stream>>>(pa);
        else k_prefill_prologue<false><<<unsigned(T), 128, 0, stream>>>(pa);
        if (cudaError_t le = cudaGetLastError(); le != cudaSuccess) return le;
        (*n_launches)++;
        return cudaSuccess;
    };

    if (cp) {  // rows whose unit has no key on this device are never written: they must read as empty parts
        if ((e = cudaMemsetAsync(p.partial_ml, 0, size_t(T) * kNHead * sizeof(float2), stream)) != cudaSuccess) return e;
        if (n_units_q == 0) return launch_prologue();
    }
    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    if (n_ksplit > 1) e = make_out_map(&tm_o, part_o, n_ksplit * t_pad, kDtypeF32);  // partials: fp32, un-normalised
    else if (cp) e = make_out_map(&tm_o, p.partial_o, T, kDtypeF32);
    else e = make_out_map(&tm_o, p.out, T, p.out_dtype);
    if (e != cudaSuccess) return e;
    if ((e = make_map(&tm_q, q_st, T, kNHead, kQPos, kGqa)) != cudaSuccess) return e;
    const void *kb = p.is_swa ? static_cast<const void *>(k_st) : static_cast<const void *>(p.k_cache);
    const void *vb = p.is_swa ? static_cast<const void *>(v_st) : static_cast<const void *>(p.v_cache);
    const int kv_rows = p.is_swa ? n_hist + T : p.n_slots;
    if (p.block_table) {  // page pool: {128 dims, 64 rows of a page, pages x KV heads}, one 64-row box per load
        if ((e = make_map(&tm_k, kb, 64, p.n_pages * kNHeadKv, 64, 1)) != cudaSuccess) return e;
        if ((e = make_map(&tm_v, vb, 64, p.n_pages * kNHeadKv, 64, 1)) != cudaSuccess) return e;
    } else {
        if ((e = make_map(&tm_k, kb, kv_rows, kNHeadKv, kBN, 1)) != cudaSuccess) return e;
        if ((e = make_map(&tm_v, vb, kv_rows, kNHeadKv, kBN, 1)) != cudaSuccess) return e;
    }

    PfArgs a{};
    a.q_st = q_st;
    a.out = n_ksplit > 1 ? static_cast<void *>(part_o) : cp ? static_cast<void *>(p.partial_o) : p.out;
    a.sinks = p.sinks; a.error_flag = err_flag;
    a.out_dtype = n_ksplit > 1 || cp ? kDtypeF32 : p.out_dtype;
    a.p0 = p.p0; a.n_tok = T; a.is_swa = p.is_swa;
    a.key_row0 = p.is_swa ? p.p0 - n_hist : kr_lo;  // row 0 of a full layer's cache holds position kv_lo
    a.n_ksplit = n_ksplit; a.t_pad = t_pad;
    a.part_ml = n_ksplit > 1 ? part_ml : cp ? reinterpret_cast<float2 *>(p.partial_ml) : part_ml;
    a.kr_lo = kr_lo; a.kr_hi = kr_hi;
    a.with_sink = p.with_sink;
    a.cp_partial = cp ? 1 : 0;
    a.block_table = p.block_table; a.table_len = p.table_len;
    const int n_units = n_units_q * n_ksplit;
    const dim3 grid(n_units < g_sm_count ? n_units : g_sm_count);
    a.n_units = n_units;
    static const bool round_robin = [] {
        const char *v = getenv("FLINT_ATTN_PREFILL_SCHEDULE");
        return v && strcmp(v, "roundrobin") == 0;
    }();
    if (n_units > int(grid.x) && !round_robin) {
        if ((e = build_schedule(ws, a, n_units, int(grid.x), stream)) != cudaSuccess) return e;
        a.sched = ws.sched;
        a.n_rounds = ws.sched_rounds;
    }
    if ((e = launch_prologue()) != cudaSuccess) return e;
    if (p.ev_attn_begin && (e = cudaEventRecord(p.ev_attn_begin, stream)) != cudaSuccess) return e;
    {
        static const bool no_pdl = [] {
            const char *v = getenv("FLINT_ATTN_NO_PDL");
            return v && v[0] == '1';
        }();
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreadsAttn);
        cfg.dynamicSmemBytes = kSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = no_pdl ? 0 : 1;
        const bool f32 = a.out_dtype == kDtypeF32;
        if (a.is_swa) e = f32 ? cudaLaunchKernelEx(&cfg, k_prefill_attn<true, true>, tm_q, tm_k, tm_v, tm_o, a)
                              : cudaLaunchKernelEx(&cfg, k_prefill_attn<true, false>, tm_q, tm_k, tm_v, tm_o, a);
        else e = f32 ? cudaLaunchKernelEx(&cfg, k_prefill_attn<false, true>, tm_q, tm_k, tm_v, tm_o, a)
                     : cudaLaunchKernelEx(&cfg, k_prefill_attn<false, false>, tm_q, tm_k, tm_v, tm_o, a);
    }
    if (e != cudaSuccess) return e;
    (*n_launches)++;
    if (n_ksplit > 1) {
        k_prefill_merge<<<unsigned(T) * (kNHead / 4), 128, 0, stream>>>(
            part_o, part_ml, cp ? static_cast<void *>(p.partial_o) : p.out, cp ? kDtypeF32 : p.out_dtype, T, t_pad, n_ksplit,
            cp ? reinterpret_cast<float2 *>(p.partial_ml) : nullptr);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        (*n_launches)++;
    }
    if (p.ev_attn_end) cudaEventRecord(p.ev_attn_end, stream);
    return cudaSuccess;
}

cudaError_t make_kv_rows_map(void *map_out, const void *base, long long n_rows) {
    if (!g_encode) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cuuint64_t(kHeadDim), cuuint64_t(n_rows)};
    const cuuint64_t strides[1] = {cuuint64_t(kHeadDim) * 2};
    const cuuint32_t box[2] = {64, 64};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(static_cast<CUtensorMap *>(map_out), CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                                const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_prefill_combine(const float *parts_o, const float *parts_ml, int n_parts, int n_tok, void *out,
                                   int out_dtype, cudaStream_t stream) {
    if (n_tok <= 0 || n_parts <= 0) return cudaSuccess;
    k_prefill_merge<<<unsigned(n_tok) * (kNHead / 4), 128, 0, stream>>>(parts_o, reinterpret_cast<const float2 *>(parts_ml), out,
                                                                     out_dtype, n_tok, n_tok, n_parts, nullptr);
    return cudaGetLastError();
}

cudaError_t prefill_error_flag(const PrefillWorkspace &ws, int *flag) {
    *flag = 0;
    if (!ws.buf) return cudaSuccess;
    cudaError_t e = cudaMemcpy(flag, ws.buf, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && *flag) e = cudaMemset(ws.buf, 0, sizeof(int));  // reported once, then cleared
    return e;
}

}  // namespace flint
