// Fused decode attention for sm_100a.
//
// Replaces the reference's k_attn_dec + k_attn_combine (src/metal/fused.metal:254-350).  Same semantics:
// QK RMSNorm, NEOX RoPE, K/V of the new token rounded to half and written to its cache slot, online softmax over
// the cached keys of a split, the learned per-head sink added exactly once in the final merge.
//
// Different shape, chosen for B200.  One CTA works on one (token, KV head, key range) item and serves all 8 query
// heads of the GQA group from a single pass over K and V, so every cache byte leaves HBM once (the reference
// re-reads it once per query head and relies on its cache).  K/V rows stream through a 3-stage cp.async pipeline
// of 64-key tiles into XOR-swizzled shared memory.  Scores are computed transposed on the tensor cores,
// S^T[16 keys x 8 heads] = K[16 x 128] . Q^T[128 x 8] with mma.m16n8k16 (N = 8 is exactly the GQA group, so no
// padding work), probabilities are transposed in registers with movmatrix and O^T[128 dims x 8 heads] +=
// V^T . P^T.  Softmax statistics stay in fp32 and are reduced with warp shuffles.  The four warps of a CTA take
// 16 keys each of every tile and keep private (m, l, O) state, merged once at the end through shared memory like
// the reference's four simdgroups (fused.metal:301-318).  Splits of one (token, KV head) group write fp32 partial
// records {acc[128], m, l} (fused.metal:324-327); the last CTA of the group to finish (atomic ticket) merges them,
// so there is no second launch and no spin-wait anywhere.
#include <cstdlib>
#include <cstring>

#include "attn_common.h"
#include "ptx.cuh"

namespace flint {

namespace {

constexpr int kTileKeys = 64;
constexpr int kStagesWave = 3;   // two CTAs per SM: the usual launch, about one wave of items
constexpr int kStagesDeep = 6;   // one CTA per SM: launches with no more items than SMs keep twice the bytes in flight
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kRowBytes = kHeadDim * 2;             // 256
constexpr int kTileBytes = kTileKeys * kRowBytes;   // 16 KiB per K or V tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int kStages>
struct __align__(1024) DecSmem {
    unsigned char k[kStages][kTileBytes];
    unsigned char v[kStages][kTileBytes];
    alignas(16) unsigned long long full_bar[kStages];  // TMA variant: the K and V tile of the stage have landed
    alignas(16) __half q[kGqa][kHeadDim];   // normalised, rotated, pre-scaled query heads of the group
    __half knew[kHeadDim];      // the new token's K (after norm/RoPE) and V as stored in the cache
    __half vnew[kHeadDim];
    float red_m[kWarps][kGqa];
    float red_l[kWarps][kGqa];
    float rope_cos[kHeadDim / 2];  // cos / sin of pos * inv_freq[i], shared by the 8 query heads and the new key
    float rope_sin[kHeadDim / 2];
    int is_last;
};
// The per-warp output accumulators are merged through the (by then idle) K tiles.
static_assert(sizeof(float) * kWarps * kGqa * kHeadDim <= kStagesWave * kTileBytes, "merge buffer aliases the K tiles");
static_assert(sizeof(DecSmem<kStagesDeep>) + 1024 <= 227 * 1024, "one CTA per SM");

// Byte offset of 16-byte chunk `ch` (0..15) of row `row` inside a 64-row K or V tile in shared memory.
//  cp.async layout: rows of 256 bytes, chunk index XOR (row % 8): conflict-free for ldmatrix.
//  TMA layout: two halves of [64 rows][128 bytes] (dims 0-63, dims 64-127), each with the hardware's 128-byte swizzle,
//  which is the same XOR applied to the chunk index within the 128-byte row (tile bases are 1024-byte aligned).
template <bool kTma>
__device__ __forceinline__ uint32_t tile_off(int row, int ch) {
    if (kTma) return uint32_t((ch >> 3) * (kTileBytes / 2) + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
    return uint32_t(row * kRowBytes + ((ch ^ (row & 7)) << 4));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after ~2^28 SM cycles, far beyond anything a healthy launch needs.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 28)) return false;
    }
}
// One 64-column x 64-row box of a {128, rows} half tensor into shared memory (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// sin and cos of a float angle of any size.  The angle is brought into [-pi, pi] in double first (exact to ~1e-11 for
// the 1e5-radian angles of a 131072-token context), which keeps sincosf off its long-argument path: that path alone
// cost the CTAs of such a context about two microseconds before their first tile could be used.
__device__ __forceinline__ void sincos_reduced(float x, float *sn, float *cs) {
    const double xd = double(x);
    const double k = rint(xd * 0.15915494309189535);
    double r = fma(-k, 6.283185307179586, xd);
    r = fma(-k, 2.4492935982947064e-16, r);
    sincosf(float(r), sn, cs);
}

__device__ __forceinline__ float4 load_row4(const void *base, int dtype, size_t elem0, int lane) {
    if (dtype == kDtypeF32) return reinterpret_cast<const float4 *>(static_cast<const float *>(base) + elem0)[lane];
    const uint2 u = reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(base) + elem0)[lane];
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&u.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162 *>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

// One 128-wide head row spread over a warp, lane owning dims 4*lane..4*lane+3: RMSNorm with weight, then NEOX RoPE
// pairing dim i with i+64, i.e. lane with lane^16 (same arithmetic as src/ref/ref_model.cpp:45-61).  cs/sn hold
// cos/sin of pos * inv_freq[4*(lane&15) .. +3], computed once per CTA.
__device__ __forceinline__ float4 norm_rope(float4 v, float4 wv, float4 cs, float4 sn, int lane, bool rope) {
    const float ss = warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w);
    const float scale = 1.0f / sqrtf(ss / kHeadDim + kRmsEps);
    v.x = v.x * scale * wv.x;
    v.y = v.y * scale * wv.y;
    v.z = v.z * scale * wv.z;
    v.w = v.w * scale * wv.w;
    if (!rope) return v;
    const float x[4] = {v.x, v.y, v.z, v.w}, c[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
    float out[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float partner = __shfl_xor_sync(0xffffffffu, x[j], 16);
        out[j] = lane < 16 ? x[j] * c[j] - partner * sv[j] : partner * sv[j] + x[j] * c[j];
    }
    return make_float4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ void store_half4(__half *dst, float4 v) {
    const uint2 u = make_uint2(pack_half2(v.x, v.y), pack_half2(v.z, v.w));
    *reinterpret_cast<uint2 *>(dst) = u;
}

__device__ __forceinline__ void store_out(void *out, int dtype, size_t idx, float v) {
    if (dtype == kDtypeF32) static_cast<float *>(out)[idx] = v;
    else static_cast<__nv_bfloat16 *>(out)[idx] = __float2bfloat16_rn(v);
}

// 8 consecutive outputs of one head as one or two 16-byte stores.
__device__ __forceinline__ void store_out8(void *out, int dtype, size_t idx, const float (&v)[8]) {
    if (dtype == kDtypeF32) {
        float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(out) + idx);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t *>(&b);
        }
        *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(out) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

struct Merged {
    float M, L;
    float a[8];
};

// Mode 1 writes this device's record to partial_out; mode 2 writes it into every peer's gather buffer over NVLink
// (plain peer stores; the data lands in the peer's memory, so the peer reads it locally).
__device__ __forceinline__ int n_record_targets(const DecParams &p) { return p.mode == 2 ? p.n_peers : 1; }
__device__ __forceinline__ float *record_target(const DecParams &p, int t, int tok, int head) {
    float *base = p.mode == 2 ? p.peer_out[t] : p.partial_out;
    return base + (size_t(tok) * kNHead + head) * kPartialDim;
}

// Mode 2: after a (token, KV head) group has written its records everywhere, count it; the last group of the launch
// publishes the step number in every peer's flag word for this rank (release at system scope).
__device__ __forceinline__ void publish_group(const DecParams &p, int tid) {
    if (p.mode != 2) return;
    __syncthreads();
    if (tid != 0) return;
    __threadfence_system();  // cumulative over the CTA's stores, which the barrier ordered before it
    if (atomicAdd(p.groups_done, 1) == p.n_groups - 1) {
        *p.groups_done = 0;
        // ONE system-scope fence orders every record store (this CTA's and, through the counter, the other groups')
        // before the flag stores; the flag stores themselves are relaxed, so the peers are written back to back
        // instead of one fence round trip per peer.
        __threadfence_system();
        for (int t = 0; t < p.n_peers; t++)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;\n" ::"l"(p.peer_flag[t] + p.rank), "r"(p.step) : "memory");
    }
}

// Takes a ticket: returns the old count.  Acquire-release at device scope (see the split-K merge).
__device__ __forceinline__ int ticket_acq_rel(int *counter) {
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;\n" : "=r"(old) : "l"(counter) : "memory");
    return old;
}

// Fold n partial records of one head (fused.metal:332-350) into the running state (M, L, a): M = max m_s,
// L = sum l_s e^(m_s - M), a = sum acc_s e^(m_s - M); the sink enters as a record with m = sink, l = 1, acc = 0.
// `rec` points at record 0 of this thread's head; consecutive records of the same head are kGqa * kRecStride floats
// apart.  The thread owns dims [d0, d0 + 8).  Eight records per trip: their 24 loads are in flight together (a trip costs about a microsecond), and
// the loop stays small -- this code runs once per group, from a cold instruction cache, so its size is its cost.
__device__ __forceinline__ Merged merge_records(const float *rec, int n, int d0, bool with_sink, float sink) {
    constexpr int kStep = kGqa * kRecStride;
    constexpr int kTrip = 8;  // records per round trip to L2
    Merged r;
    float M = with_sink ? sink : -INFINITY, L = with_sink ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) r.a[j] = 0.f;
#pragma unroll 1
    for (int s0 = 0; s0 < n; s0 += kTrip) {
        float2 ml[kTrip];
        float4 x[kTrip], y[kTrip];
#pragma unroll
        for (int i = 0; i < kTrip; i++) {
            const float *q = rec + size_t(min(s0 + i, n - 1)) * kStep;  // past the end: re-read the last one, unused
            ml[i] = __ldcg(reinterpret_cast<const float2 *>(q + kHeadDim));
            x[i] = __ldcg(reinterpret_cast<const float4 *>(q + d0));
            y[i] = __ldcg(reinterpret_cast<const float4 *>(q + d0 + 4));
            if (s0 + i >= n) ml[i] = make_float2(-INFINITY, 0.f);
        }
        float cm = M;
#pragma unroll
        for (int i = 0; i < kTrip; i++) cm = fmaxf(cm, ml[i].x);
        const float keep = M == -INFINITY ? 0.f : __expf(M - cm);
        L *= keep;
#pragma unroll
        for (int j = 0; j < 8; j++) r.a[j] *= keep;
        M = cm;
#pragma unroll
        for (int i = 0; i < kTrip; i++) {
            // an empty part has m = -inf, l = 0 (fused.metal:344)
            const float c = ml[i].y == 0.f ? 0.f : __expf(ml[i].x - M);
            L += ml[i].y * c;
            r.a[0] += x[i].x * c; r.a[1] += x[i].y * c; r.a[2] += x[i].z * c; r.a[3] += x[i].w * c;
            r.a[4] += y[i].x * c; r.a[5] += y[i].y * c; r.a[6] += y[i].z * c; r.a[7] += y[i].w * c;
        }
    }
    r.M = M;
    r.L = L;
    return r;
}

template <int kStages, bool kTma>
__device__ __forceinline__ void decode_item(const DecParams &p, const DecItem &it) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // swizzled TMA tiles need 1024-byte alignment: the launch asks for 1 KiB more than the struct and rounds up here
    DecSmem<kStages> &sm = *reinterpret_cast<DecSmem<kStages> *>(
        smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int j0 = it.j0, j1 = it.j1;
    const int j_end = j1 + (it.fold ? 1 : 0);  // the new token sits right after the cached range of a fold item
    const int n_tiles = (j_end - j0 + kTileKeys - 1) / kTileKeys;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    // layout of the merge steps at the end: 16 threads per head, 8 dims per thread; the head's sink is fetched now
    const int mh = tid >> 4, md = (tid & 15) * 8;
    const int head = it.kvh * kGqa + mh;
    const float sink = p.sinks[head];

    const __half *kbase = p.k_cache + size_t(it.seq) * p.seq_stride + size_t(it.kvh) * p.n_slots * kHeadDim;
    const __half *vbase = p.v_cache + size_t(it.seq) * p.seq_stride + size_t(it.kvh) * p.n_slots * kHeadDim;
    const uint32_t ks_addr = smem_u32(&sm.k[0][0]), vs_addr = smem_u32(&sm.v[0][0]);

    auto load_tile = [&](int t) {
        const int stage = t % kStages;
        const int jt = j0 + t * kTileKeys;
        if (kTma) {
            // One thread asks for the whole tile: two 64-dim halves of K and of V, 32 KiB on one barrier.  Rows past
            // the item's range are real cache rows (later keys, or slots never written): they are masked below, and
            // the caches of a handle only ever hold finite values.
            if (tid == 0) {
                int y;
                if (p.paged) y = (p.block_table[size_t(it.seq) * p.table_stride + (jt >> 6)] * kNHeadKv + it.kvh) * kPageKeys;
                else y = (it.seq * kNHeadKv + it.kvh) * p.n_slots + (jt - p.kv_lo);
                const uint32_t bar = smem_u32(&sm.full_bar[stage]);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // earlier generic accesses to the stage
                mbar_expect_tx(bar, 2 * kTileBytes);
                tma_load_2d(ks_addr + stage * kTileBytes, p.k_map, bar, 0, y);
                tma_load_2d(ks_addr + stage * kTileBytes + kTileBytes / 2, p.k_map, bar, 64, y);
                tma_load_2d(vs_addr + stage * kTileBytes, p.v_map, bar, 0, y);
                tma_load_2d(vs_addr + stage * kTileBytes + kTileBytes / 2, p.v_map, bar, 64, y);
            }
            return;
        }
        // paged layer: this tile is one page (jt is a multiple of 64); its rows are slots 0..63 of the page
        const __half *kb = kbase, *vb = vbase;
        if (p.paged) {
            const size_t page = size_t(p.block_table[size_t(it.seq) * p.table_stride + (jt >> 6)]);
            const size_t off = (page * kNHeadKv + it.kvh) * kPageKeys * kHeadDim;
            kb = p.k_cache + off;
            vb = p.v_cache + off;
        }
#pragma unroll
        for (int i = 0; i < (kTileKeys * 16) / kThreads; i++) {
            const int c = tid + kThreads * i;
            const int row = c >> 4, ch = c & 15;
            const int j = jt + row;
            const bool valid = j < j1;  // cached keys only; other rows are zero-filled
            const int slot = !valid ? 0 : p.paged ? row : int(uint32_t(j) & p.slot_mask) - p.kv_lo;
            const size_t off = size_t(slot) * kHeadDim + ch * 8;
            const uint32_t dst = stage * kTileBytes + tile_off<false>(row, ch);
            cp_async16(ks_addr + dst, kb + off, valid ? 16u : 0u);
            cp_async16(vs_addr + dst, vb + off, valid ? 16u : 0u);
        }
    };


    // ---- prologue: q heads of the group (and the new token's k, v) -> shared memory --------------------------
    // The row loads go out first, then the first K/V tiles, so that neither waits behind the other's latency; the 64
    // rotation angles are evaluated once per CTA while all of them are in flight.
    const size_t row0 = size_t(it.tok) * kQkvDim;
    const bool rope = p.has_rope != 0;
    const bool fold_k = it.fold && warp == 0, fold_v = it.fold && warp == 1;
    const float4 wq = reinterpret_cast<const float4 *>(p.q_norm)[lane];
    float4 wk = wq;
    if (fold_k) wk = reinterpret_cast<const float4 *>(p.k_norm)[lane];
    float freq = 0.f;
    if (rope && tid < kHeadDim / 2) freq = p.inv_freq[tid];
    // Programmatic dependent launch: the next kernel of the stream may be scheduled while this one still runs, and
    // this one may have been scheduled while its predecessor still ran.  Everything above touched only kernel
    // parameters and the layer's constant tables; nothing produced by an earlier kernel (the q/k/v rows, cache
    // contents, split-K scratch and counters) is read or written before this wait, which returns once every
    // earlier kernel of the stream has completed and its writes are visible.
    if (kTma && tid == 0) {  // the maps are written once, when the handle is opened: fetching them early is safe
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(p.k_map)) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(p.v_map)) : "memory");
    }
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (kTma && tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; s++) mbar_init(smem_u32(&sm.full_bar[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    float4 q[2];
#pragma unroll
    for (int i = 0; i < 2; i++)
        q[i] = load_row4(p.qkv, p.qkv_dtype, row0 + size_t(it.kvh * kGqa + warp * 2 + i) * kHeadDim, lane);
    float4 kv_new = make_float4(0.f, 0.f, 0.f, 0.f);
    if (fold_k) kv_new = load_row4(p.qkv, p.qkv_dtype, row0 + kQDim + size_t(it.kvh) * kHeadDim, lane);
    if (fold_v) kv_new = load_row4(p.qkv, p.qkv_dtype, row0 + kQDim + kKvDim + size_t(it.kvh) * kHeadDim, lane);

#pragma unroll
    for (int t = 0; t < kStages - 1; t++) {
        if (t < n_tiles) load_tile(t);
        cp_async_commit();
    }

    {
        const float qscale = rsqrtf(float(kHeadDim)) * kLog2e;  // softmax runs in base 2
        if (rope && tid < kHeadDim / 2) {
            float sn, cs;
            sincos_reduced(float(it.pos) * freq, &sn, &cs);
            sm.rope_cos[tid] = cs;
            sm.rope_sin[tid] = sn;
        }
        __syncthreads();
        float4 cs = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rope) {
            cs = reinterpret_cast<const float4 *>(sm.rope_cos)[lane & 15];
            sn = reinterpret_cast<const float4 *>(sm.rope_sin)[lane & 15];
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float4 r = norm_rope(q[i], wq, cs, sn, lane, rope);
            r.x *= qscale; r.y *= qscale; r.z *= qscale; r.w *= qscale;
            store_half4(&sm.q[warp * 2 + i][4 * lane], r);
        }
        if (fold_k || fold_v) {
            if (fold_k) kv_new = norm_rope(kv_new, wk, cs, sn, lane, rope);
            store_half4(fold_k ? &sm.knew[4 * lane] : &sm.vnew[4 * lane], kv_new);
            if (p.paged) {
                const size_t page = size_t(p.block_table[size_t(it.seq) * p.table_stride + (it.pos >> 6)]);
                const size_t off = ((page * kNHeadKv + it.kvh) * kPageKeys + (it.pos & (kPageKeys - 1))) * kHeadDim;
                store_half4((fold_k ? p.k_cache : p.v_cache) + off + 4 * lane, kv_new);
            } else {
                const int slot = int(uint32_t(it.pos) & p.slot_mask) - p.kv_lo;
                store_half4(const_cast<__half *>(fold_k ? kbase : vbase) + size_t(slot) * kHeadDim + 4 * lane, kv_new);
            }
        }
    }
    __syncthreads();

    // B fragments of Q^T for the 8 k-steps: b0 = Q[head g][16k + 2t, +1], b1 = Q[head g][16k + 8 + 2t, +1]
    uint32_t bq[8][2];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        bq[k][0] = *reinterpret_cast<const uint32_t *>(&sm.q[g][16 * k + 2 * t4]);
        bq[k][1] = *reinterpret_cast<const uint32_t *>(&sm.q[g][16 * k + 8 + 2 * t4]);
    }

    // Per-thread state for heads 2*t4 and 2*t4+1: running max (replicated over g), partial sum (this thread's keys),
    // and O^T fragments o[dm] = dims 16*dm + {g, g+8} x heads {2*t4, 2*t4+1}.
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[8][4];
#pragma unroll
    for (int dm = 0; dm < 8; dm++) o[dm][0] = o[dm][1] = o[dm][2] = o[dm][3] = 0.f;

    const int new_tile = it.fold ? (it.pos - j0) / kTileKeys : -1;
    const int new_row = it.fold ? (it.pos - j0) % kTileKeys : -1;

    for (int t = 0; t < n_tiles; t++) {
        if (kTma) {
            // every thread waits for the tile itself (bounded); if any wait ran out, the whole CTA reports it and
            // leaves together (the barrier below carries the decision)
            const bool late = !mbar_wait_bounded(smem_u32(&sm.full_bar[t % kStages]), uint32_t(t / kStages) & 1u);
            if (__syncthreads_or(late)) {
                if (tid == 0 && p.error_flag) atomicExch(p.error_flag, 4);
                return;
            }
        } else {
            cp_async_wait<kStages - 2>();
            __syncthreads();
        }
        if (t + kStages - 1 < n_tiles) load_tile(t + kStages - 1);
        if (!kTma) cp_async_commit();

        const int stage = t % kStages;
        const int jw = j0 + t * kTileKeys + 16 * warp;  // first key of this warp's 16-row slice
        if (jw >= j_end) continue;                       // warp-uniform

        if (t == new_tile && (new_row >> 4) == warp) {
            // the new token's row comes from registers/shared memory, never from the cache slot being written
            const uint4 val = lane < 16 ? reinterpret_cast<const uint4 *>(sm.knew)[lane]
                                        : reinterpret_cast<const uint4 *>(sm.vnew)[lane - 16];
            unsigned char *tile = lane < 16 ? sm.k[stage] : sm.v[stage];
            const int ch = lane & 15;
            *reinterpret_cast<uint4 *>(tile + tile_off<kTma>(new_row, ch)) = val;
            __syncwarp();
        }

        // S^T (16 keys x 8 heads) = K . Q^T
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const uint32_t base = ks_addr + stage * kTileBytes;
            const int row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int k = 0; k < 8; k++) {
                uint32_t a[4];
                ldmatrix_x4(a, base + tile_off<kTma>(row, 2 * k + (lane >> 4)));
                mma_16816(s, a, bq[k][0], bq[k][1]);
            }
        }
        if (jw + g >= j_end) s[0] = s[1] = -INFINITY;
        if (jw + g + 8 >= j_end) s[2] = s[3] = -INFINITY;

        float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        // at least one key of the slice is valid, so the new maxima are finite
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float c0 = fast_exp2(m0 - mn0), c1 = fast_exp2(m1 - mn1);
        const float p0 = fast_exp2(s[0] - mn0), p1 = fast_exp2(s[1] - mn1);
        const float p2 = fast_exp2(s[2] - mn0), p3 = fast_exp2(s[3] - mn1);
        l0 = l0 * c0 + (p0 + p2);
        l1 = l1 * c1 + (p1 + p3);
        m0 = mn0;
        m1 = mn1;
        // P^T as the B operand: b0 = P[key 2t, 2t+1][head g], b1 = keys +8
        const uint32_t b0 = movmatrix_trans(pack_half2(p0, p1));
        const uint32_t b1 = movmatrix_trans(pack_half2(p2, p3));

        // O^T (128 dims x 8 heads) = O^T * corr + V^T . P^T
        {
            const uint32_t base = vs_addr + stage * kTileBytes;
            const int row = 16 * warp + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
            for (int dm = 0; dm < 8; dm++) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, base + tile_off<kTma>(row, 2 * dm + ((lane >> 3) & 1)));
                o[dm][0] *= c0; o[dm][1] *= c1; o[dm][2] *= c0; o[dm][3] *= c1;
                mma_16816(o[dm], a, b0, b1);
            }
        }
    }
    if (!kTma) cp_async_wait<0>();
    __syncthreads();  // every warp is done with the tiles: the K tiles become the merge buffer

    // ---- merge the four warps --------------------------------------------------------------------------------
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, off);
        l1 += __shfl_xor_sync(0xffffffffu, l1, off);
    }
    float *obuf = reinterpret_cast<float *>(&sm.k[0][0]);  // [warp][head][dim]
    if (g == 0) {
        sm.red_m[warp][2 * t4] = m0; sm.red_m[warp][2 * t4 + 1] = m1;
        sm.red_l[warp][2 * t4] = l0; sm.red_l[warp][2 * t4 + 1] = l1;
    }
#pragma unroll
    for (int dm = 0; dm < 8; dm++) {
        float *ow = obuf + size_t(warp) * kGqa * kHeadDim;
        ow[(2 * t4) * kHeadDim + 16 * dm + g] = o[dm][0];
        ow[(2 * t4 + 1) * kHeadDim + 16 * dm + g] = o[dm][1];
        ow[(2 * t4) * kHeadDim + 16 * dm + g + 8] = o[dm][2];
        ow[(2 * t4 + 1) * kHeadDim + 16 * dm + g + 8] = o[dm][3];
    }
    __syncthreads();

    // From here on a thread owns 8 dims of one head (16 threads per head), so each step is a couple of wide,
    // independent loads per thread instead of a loop over heads.
    const bool direct = it.n_split == 1;
    {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, sm.red_m[w][mh]);
        float L = 0.f, A[8];
#pragma unroll
        for (int j = 0; j < 8; j++) A[j] = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            const float lw = sm.red_l[w][mh];
            // a warp that saw no key has m = -inf, l = 0 and contributes nothing (fused.metal:314)
            const float c = lw == 0.f ? 0.f : fast_exp2(sm.red_m[w][mh] - M);
            const float4 x = *reinterpret_cast<const float4 *>(obuf + (size_t(w) * kGqa + mh) * kHeadDim + md);
            const float4 y = *reinterpret_cast<const float4 *>(obuf + (size_t(w) * kGqa + mh) * kHeadDim + md + 4);
            L += lw * c;
            A[0] += x.x * c; A[1] += x.y * c; A[2] += x.z * c; A[3] += x.w * c;
            A[4] += y.x * c; A[5] += y.y * c; A[6] += y.z * c; A[7] += y.w * c;
        }
        if (direct && p.mode == 0) {
            // single split: fold the sink here (fused.metal:319-322), all in base 2
            const float sink2 = sink * kLog2e;
            const float Mf = fmaxf(M, sink2), cs = fast_exp2(M - Mf);
            const float inv = cs / (L * cs + fast_exp2(sink2 - Mf));
#pragma unroll
            for (int j = 0; j < 8; j++) A[j] *= inv;
            store_out8(p.out, p.out_dtype, size_t(it.tok) * kQDim + head * kHeadDim + md, A);
        } else if (direct) {
            // this device's only record for the token: {acc[128], m, l}, m in natural-log units (fused.metal:324-327)
            for (int t = 0; t < n_record_targets(p); t++) {
                float *rec = record_target(p, t, it.tok, head);  // 130-float records: 8-byte aligned only
#pragma unroll
                for (int j = 0; j < 8; j += 2) *reinterpret_cast<float2 *>(rec + md + j) = make_float2(A[j], A[j + 1]);
                if (md == 0) { rec[kHeadDim] = M * kLn2; rec[kHeadDim + 1] = L; }
            }
        } else {
            float *rec = p.scratch + ((size_t(it.part0) + it.split) * kGqa + mh) * kRecStride;
            *reinterpret_cast<float4 *>(rec + md) = make_float4(A[0], A[1], A[2], A[3]);
            *reinterpret_cast<float4 *>(rec + md + 4) = make_float4(A[4], A[5], A[6], A[7]);
            if (md == 0) { rec[kHeadDim] = M * kLn2; rec[kHeadDim + 1] = L; }
        }
    }
    if (direct) {
        publish_group(p, tid);
        return;
    }

    // ---- split-K merge (fused.metal:332-350), done by whichever CTA finishes last -- no second launch, no waiting.
    // Two levels, so that a long sequence cut into hundreds of splits is not merged by a single CTA: the last CTA of
    // each run of 16 splits folds those records into one; the last of those to finish folds the runs and the sink.
    const int sub = it.split / kMergeFan, n_sub = (it.n_split + kMergeFan - 1) / kMergeFan;
    const int sub_size = min(kMergeFan, it.n_split - sub * kMergeFan);
    // The CTA's record stores are ordered before thread 0's ticket by the barrier, and the ticket is an acquire-release
    // atomic at device scope: its release side is cumulative, so one thread publishes for all; its acquire side plus
    // the second barrier cover the other threads, which read the records past L1 (ld.cg).  (A fence either side of a
    // relaxed atomic does the same but makes the last arriver wait twice more for a round trip to L2, the second time
    // for its own reset of the ticket.)
    __syncthreads();
    if (tid == 0) {
        const bool last = ticket_acq_rel(&p.tickets[it.sub0 + sub]) == sub_size - 1;
        if (last) p.tickets[it.sub0 + sub] = 0;  // ready for the next launch; nothing in this one waits for it
        sm.is_last = last;
    }
    __syncthreads();
    if (!sm.is_last) return;

    // One copy of the merge code serves both levels (see merge_records on code size).
    const float *src = p.scratch + ((size_t(it.part0) + sub * kMergeFan) * kGqa + mh) * kRecStride;
    int n_src = sub_size;
    bool final_level = n_sub == 1;
    Merged r;
    for (;;) {
        r = merge_records(src, n_src, md, final_level && p.mode == 0, sink);
        if (final_level) break;
        float *rec2 = p.scratch2 + ((size_t(it.sub0) + sub) * kGqa + mh) * kRecStride;
        *reinterpret_cast<float4 *>(rec2 + md) = make_float4(r.a[0], r.a[1], r.a[2], r.a[3]);
        *reinterpret_cast<float4 *>(rec2 + md + 4) = make_float4(r.a[4], r.a[5], r.a[6], r.a[7]);
        if (md == 0) { rec2[kHeadDim] = r.M; rec2[kHeadDim + 1] = r.L; }
        __syncthreads();
        if (tid == 0) {
            const bool last = ticket_acq_rel(&p.tickets2[it.group]) == n_sub - 1;
            if (last) p.tickets2[it.group] = 0;
            sm.is_last = last;
        }
        __syncthreads();
        if (!sm.is_last) return;
        src = p.scratch2 + (size_t(it.sub0) * kGqa + mh) * kRecStride;
        n_src = n_sub;
        final_level = true;
    }
    if (p.mode == 0) {
        const float inv = 1.0f / r.L;
#pragma unroll
        for (int j = 0; j < 8; j++) r.a[j] *= inv;
        store_out8(p.out, p.out_dtype, size_t(it.tok) * kQDim + head * kHeadDim + md, r.a);
    } else {
        for (int t = 0; t < n_record_targets(p); t++) {
            float *rec = record_target(p, t, it.tok, head);  // 130-float public record
#pragma unroll
            for (int j = 0; j < 8; j += 2) *reinterpret_cast<float2 *>(rec + md + j) = make_float2(r.a[j], r.a[j + 1]);
            if (md == 0) { rec[kHeadDim] = r.M; rec[kHeadDim + 1] = r.L; }
        }
        publish_group(p, tid);
    }
}

// The work list either sits in device memory (any length) or, when it is short enough, travels in the kernel's
// parameter space (large kernel parameters, up to 32 KiB): one wave on a 148-SM part is ~300 items of 48 bytes, so the
// usual launch needs no host-to-device copy in front of it.  The parameter block is copied by the driver at every
// launch, so the kernel comes in three capacities and a launch takes the smallest that fits (the smallest one stays
// inside the classic 4 KiB parameter space).
template <int kCap>
struct DecItemsParam {
    DecItem items[kCap];
};

template <bool kTma>
__global__ void __launch_bounds__(kThreads, 2) k_decode_attn(const DecParams p) {
    const DecItem it = p.items[blockIdx.x];
    decode_item<kStagesWave, kTma>(p, it);
}

template <int kCap, int kStages, bool kTma>
__global__ void __launch_bounds__(kThreads, kStages == kStagesWave ? 2 : 1)
    k_decode_attn_p(const __grid_constant__ DecParams p, const __grid_constant__ DecItemsParam<kCap> ip) {
    const DecItem it = ip.items[blockIdx.x];
    decode_item<kStages, kTma>(p, it);
}

template <int kStages>
constexpr size_t smem_bytes() {  // 1 KiB of slack for the 1024-byte alignment of the tiles
    return sizeof(DecSmem<kStages>) + 1024;
}

constexpr int kCapSmall = 76, kCapMid = 304;  // 304: one wave of items on a 148-SM part (two CTAs per SM) and a little more
static_assert(sizeof(DecParams) + sizeof(DecItemsParam<kCapSmall>) <= 4096, "small variant fits 4 KiB of parameters");
static_assert(sizeof(DecParams) + sizeof(DecItemsParam<kMaxParamItems>) <= 32764, "largest variant fits the limit");

// Launch with programmatic stream serialization: the kernel may be scheduled before its predecessor in the stream
// has finished (it waits inside, see decode_item), which hides launch latency between the short kernels of a decode
// step.  FLINT_ATTN_NO_PDL=1 in the environment turns it off.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), int n_items, size_t smem_bytes, cudaStream_t stream,
                       const Args &...args) {
    static const bool off = [] {
        const char *v = getenv("FLINT_ATTN_NO_PDL");
        return v && v[0] == '1';
    }();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(n_items));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = off ? 0 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int kCap, int kStages>
cudaError_t launch_inline(const DecParams &p, const DecItem *host_items, int n_items, cudaStream_t stream) {
    static thread_local DecItemsParam<kCap> ip;  // copied into the launch by the runtime before this returns
    memcpy(ip.items, host_items, sizeof(DecItem) * size_t(n_items));
    if (p.k_map) return launch_pdl(k_decode_attn_p<kCap, kStages, true>, n_items, smem_bytes<kStages>(), stream, p, ip);
    return launch_pdl(k_decode_attn_p<kCap, kStages, false>, n_items, smem_bytes<kStages>(), stream, p, ip);
}

template <typename K>
cudaError_t allow_smem(K kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
}

// Merge of per-device partial records (KV-range sharding): one CTA per (token, head), thread = dim.  With a
// peer-memory exchange the records were stored by the other GPUs; the CTA first waits until every rank has published
// this step.  The wait is bounded (about a second); when it runs out the kernel records an error and returns.
constexpr long long kPeerWaitCycles = 2000000000LL;  // about a second at the part's clocks
__global__ void __launch_bounds__(kHeadDim) k_combine_parts(const CombineParams p) {
    const int tok = blockIdx.x / kNHead, head = blockIdx.x % kNHead, d = threadIdx.x;
    if (p.flags) {
        __shared__ int timed_out;
        if (d == 0) {
            timed_out = 0;
            for (int r = 0; r < p.n_parts && !timed_out; r++) {
                uint32_t v = 0;
                const long long t0 = clock64();
                for (;;) {
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p.flags + r) : "memory");
                    // a peer may already be one step ahead (it writes the other record buffer then)
                    if (int32_t(v - p.step) >= 0 || clock64() - t0 > kPeerWaitCycles) break;
                    __nanosleep(200);
                }
                if (int32_t(v - p.step) < 0) timed_out = 1;
            }
            if (timed_out) atomicExch(p.error_flag, 3);
        }
        __syncthreads();
        if (timed_out) return;
    }
    const float sink = p.sinks[head];
    float M = sink;
    for (int s = 0; s < p.n_parts; s++)
        M = fmaxf(M, __ldcg(p.partials + size_t(s) * p.part_stride + (size_t(tok) * kNHead + head) * kPartialDim + kHeadDim));
    float L = __expf(sink - M), A = 0.f;
    for (int s = 0; s < p.n_parts; s++) {
        const float *rec = p.partials + size_t(s) * p.part_stride + (size_t(tok) * kNHead + head) * kPartialDim;
        const float ls = __ldcg(rec + kHeadDim + 1);
        if (ls == 0.f) continue;
        const float c = __expf(__ldcg(rec + kHeadDim) - M);
        L += ls * c;
        A += __ldcg(rec + d) * c;
    }
    store_out(p.out, p.out_dtype, size_t(tok) * kQDim + head * kHeadDim + d, A / L);
}

}  // namespace

cudaError_t decode_kernel_setup() {
    constexpr size_t wave = smem_bytes<kStagesWave>(), deep = smem_bytes<kStagesDeep>();
    cudaError_t e = allow_smem(k_decode_attn<false>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn<true>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapSmall, kStagesWave, false>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapMid, kStagesWave, false>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kMaxParamItems, kStagesWave, false>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapSmall, kStagesDeep, false>, deep);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapMid, kStagesDeep, false>, deep);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapSmall, kStagesWave, true>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapMid, kStagesWave, true>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kMaxParamItems, kStagesWave, true>, wave);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapSmall, kStagesDeep, true>, deep);
    if (e == cudaSuccess) e = allow_smem(k_decode_attn_p<kCapMid, kStagesDeep, true>, deep);
    return e;
}

cudaError_t launch_decode(const DecParams &p, int n_items, cudaStream_t stream) {
    if (n_items <= 0) return cudaSuccess;
    if (p.k_map) return launch_pdl(k_decode_attn<true>, n_items, smem_bytes<kStagesWave>(), stream, p);
    return launch_pdl(k_decode_attn<false>, n_items, smem_bytes<kStagesWave>(), stream, p);
}

cudaError_t launch_decode_inline(const DecParams &p, const DecItem *host_items, int n_items, int sm_count,
                                 cudaStream_t stream) {
    if (n_items <= 0) return cudaSuccess;
    if (n_items > kMaxParamItems) return cudaErrorInvalidValue;
    // No more items than SMs: every CTA has an SM to itself, so it takes the deep pipeline (twice the bytes in flight
    // per SM; a short launch is bound by latency, not by bandwidth).
    if (n_items <= sm_count && n_items <= kCapMid) {
        if (n_items <= kCapSmall) return launch_inline<kCapSmall, kStagesDeep>(p, host_items, n_items, stream);
        return launch_inline<kCapMid, kStagesDeep>(p, host_items, n_items, stream);
    }
    if (n_items <= kCapSmall) return launch_inline<kCapSmall, kStagesWave>(p, host_items, n_items, stream);
    if (n_items <= kCapMid) return launch_inline<kCapMid, kStagesWave>(p, host_items, n_items, stream);
    return launch_inline<kMaxParamItems, kStagesWave>(p, host_items, n_items, stream);
}

cudaError_t launch_combine(const CombineParams &p, cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    k_combine_parts<<<p.n * kNHead, kHeadDim, 0, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace flint
