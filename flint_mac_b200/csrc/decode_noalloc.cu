// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need attention: an inference server that
// handed the whole GPU to its own arena at start-up and keeps the KV caches there, a plug-in running inside a
// framework whose allocator owns every byte, or code in a latency-critical section where an allocation (which
// synchronises the device) is not acceptable.  The handle-based entry points allocate: caches at open, and the
// split-K scratch, the work-list staging and the I/O staging on demand.  flint_attn_decode_noalloc_dev does not.
// The caller passes every input and output (rows, caches, layer parameters) as device pointers it owns, and the
// only memory the kernel needs beyond those -- the work list, the split-K partial records, the per-group arrival
// counters and the RoPE frequency table -- lives in the fixed array below, which is part of the loaded library
// image on every GPU that loads it (about 10 MiB per GPU until the process exits).
//
// It runs the same kernel as flint_attn_decode_dev (k_decode_attn), with the same planner and the same choice of
// kernel variant: a work list of up to 640 items travels in the kernel's parameters (no copy at all in front of the
// launch); only a longer list is uploaded into the fixed array from a pageable host buffer, a copy for which the
// runtime blocks the calling thread until the bytes are staged.
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "../../include/flint_attn.h"
#include "attn_common.h"

using namespace flint;

namespace {

constexpr int kMaxTokens = FLINT_ATTN_NOALLOC_MAX_TOKENS;  // 64
constexpr int kMaxItems = FLINT_ATTN_NOALLOC_MAX_ITEMS;    // 2048

// Layout of the fixed scratch (byte offsets, each a multiple of 256).  A group of n splits is merged in runs of
// kMergeFan, so it needs ceil(n / kMergeFan) run counters / second-level records: at most kMaxRuns in total.
constexpr int kMaxGroups = kMaxTokens * kNHeadKv;
constexpr int kMaxRuns = kMaxItems / kMergeFan + kMaxGroups;
constexpr size_t kAlign = 256;
constexpr size_t up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }
constexpr size_t kOffFreq = 0;                                                        // float[64]
constexpr size_t kOffTickets = 256;                                                   // int[kMaxRuns + kMaxGroups]
constexpr size_t kTicketBytes = sizeof(int) * (kMaxRuns + kMaxGroups);
constexpr size_t kOffItems = up(kOffTickets + kTicketBytes);                          // DecItem[kMaxItems]
constexpr size_t kOffRecords = up(kOffItems + sizeof(DecItem) * kMaxItems);           // float[kMaxItems][8][kRecStride]
constexpr size_t kOffRecords2 = up(kOffRecords + sizeof(float) * kMaxItems * kGqa * kRecStride);  // float[kMaxRuns][8][kRecStride]
constexpr size_t kScratchBytes = kOffRecords2 + sizeof(float) * kMaxRuns * kGqa * kRecStride;

// In host code this name is only a handle for cudaGetSymbolAddress: it is NOT a device address and must never be
// handed to a kernel as a pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct DeviceState {
    bool ready = false;
    unsigned char *base = nullptr;  // device address of g_noalloc_scratch on this GPU
    int sm_count = 148;
};
DeviceState g_state[64];
DecItem g_items_host[kMaxItems];  // staging for the work list; pageable on purpose (no cudaMallocHost)
int32_t g_plan[8 * kMaxItems];

void fail(char *err, int32_t len, const char *msg) {
    if (err && len > 0) {
        strncpy(err, msg, size_t(len) - 1);
        err[len - 1] = 0;
    }
}

// One-time set-up for the current device: resolve the scratch address, write the RoPE table, zero the counters.
// Uses the legacy default stream with blocking copies, so it must not happen inside a stream capture.
const char *setup_device(int dev) {
    DeviceState &st = g_state[dev];
    void *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) return "cudaGetSymbolAddress failed for the fixed scratch array";
    float freq[kHeadDim / 2];
    for (int i = 0; i < kHeadDim / 2; i++) freq[i] = powf(kRopeTheta, -2.0f * i / kHeadDim);
    unsigned char *base = static_cast<unsigned char *>(ptr);
    if (cudaMemcpy(base + kOffFreq, freq, sizeof(freq), cudaMemcpyHostToDevice) != cudaSuccess)
        return "could not initialise the RoPE table in the fixed scratch array";
    if (cudaMemset(base + kOffTickets, 0, kTicketBytes) != cudaSuccess)
        return "could not clear the arrival counters in the fixed scratch array";
    if (decode_kernel_setup() != cudaSuccess) return "could not set the decode kernel's shared-memory size";
    if (cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return "could not read the device's SM count";
    if (cudaDeviceSynchronize() != cudaSuccess) return "device error during set-up";
    st.base = base;
    st.ready = true;
    return nullptr;
}

}  // namespace

extern "C" int32_t flint_attn_decode_noalloc_dev(int32_t n, const int32_t *pos, const void *qkv_dev, int32_t qkv_dtype,
                                                 void *out_dev, int32_t out_dtype, void *k_cache_dev,
                                                 void *v_cache_dev, int32_t n_slots, int32_t is_swa,
                                                 int32_t has_rope, const float *q_norm_dev, const float *k_norm_dev,
                                                 const float *sinks_dev, void *cuda_stream, char *err,
                                                 int32_t err_len) {
    char msg[200];
    if (n < 1 || n > kMaxTokens) {
        snprintf(msg, sizeof(msg), "flint_attn_decode_noalloc_dev: n = %d tokens, the fixed scratch holds 1..%d", n,
                 kMaxTokens);
        fail(err, err_len, msg);
        return -1;
    }
    if (!pos || !qkv_dev || !out_dev || !k_cache_dev || !v_cache_dev || !q_norm_dev || !k_norm_dev || !sinks_dev) {
        fail(err, err_len, "flint_attn_decode_noalloc_dev: null pointer argument");
        return -1;
    }
    if ((qkv_dtype != kDtypeF32 && qkv_dtype != kDtypeBf16) || (out_dtype != kDtypeF32 && out_dtype != kDtypeBf16)) {
        fail(err, err_len, "flint_attn_decode_noalloc_dev: bad dtype");
        return -1;
    }
    if (n_slots < 1 || (is_swa && n_slots != kSwaRing)) {
        fail(err, err_len, "flint_attn_decode_noalloc_dev: n_slots must be 1024 on a sliding-window layer and >= 1 otherwise");
        return -1;
    }
    for (int i = 0; i < n; i++)
        if (pos[i] < 0 || (!is_swa && pos[i] >= n_slots)) {
            fail(err, err_len, "flint_attn_decode_noalloc_dev: position outside the cache");
            return -1;
        }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
        fail(err, err_len, "flint_attn_decode_noalloc_dev: no current CUDA device");
        return -1;
    }
    if (dev >= int(sizeof(g_state) / sizeof(g_state[0]))) {
        fail(err, err_len, "flint_attn_decode_noalloc_dev: device ordinals above 63 are not supported");
        return -1;
    }
    if (!g_state[dev].ready) {
        if (const char *why = setup_device(dev)) {
            fail(err, err_len, why);
            return -1;
        }
    }
    // Same planner as the handle-based path; it reports -1 when the work list would not fit.
    const int target_items = 2 * g_state[dev].sm_count;  // one wave of two CTAs per SM, as the handle plans
    const int n_items = flint_attn_plan_decode(n, pos, is_swa, 0, is_swa ? INT32_MAX : n_slots, target_items, g_plan,
                                               kMaxItems);
    if (n_items < 0) {
        snprintf(msg, sizeof(msg), "flint_attn_decode_noalloc_dev: the split-K work list exceeds the fixed scratch (%d items)",
                 kMaxItems);
        fail(err, err_len, msg);
        return -1;
    }
    // Run counters / second-level records are handed out in group order, like the partial records.
    static int32_t group_splits[kMaxGroups], group_sub0[kMaxGroups];
    for (int g = 0; g < n * kNHeadKv; g++) group_splits[g] = 1;
    for (int i = 0; i < n_items; i++) group_splits[g_plan[8 * i] * kNHeadKv + g_plan[8 * i + 1]] = g_plan[8 * i + 6];
    int n_runs = 0;
    for (int g = 0; g < n * kNHeadKv; g++) {
        group_sub0[g] = n_runs;
        if (group_splits[g] > 1) n_runs += (group_splits[g] + kMergeFan - 1) / kMergeFan;
    }
    for (int i = 0; i < n_items; i++) {
        const int32_t *r = g_plan + 8 * i;
        DecItem &it = g_items_host[i];
        it = DecItem{};
        it.tok = r[0]; it.seq = r[0]; it.kvh = r[1]; it.pos = pos[r[0]];
        it.j0 = r[2]; it.j1 = r[3]; it.fold = r[4]; it.split = r[5]; it.n_split = r[6]; it.part0 = r[7];
        it.group = r[0] * kNHeadKv + r[1];
        it.sub0 = group_sub0[it.group];
    }
    unsigned char *base = g_state[dev].base;
    cudaStream_t st = cudaStream_t(cuda_stream);
    // The counters must start at zero.  The kernel leaves them at zero, but a launch that failed part-way would not.
    if (cudaMemsetAsync(base + kOffTickets, 0, kTicketBytes, st) != cudaSuccess) {
        fail(err, err_len, "flint_attn_decode_noalloc_dev: could not clear the arrival counters");
        return -1;
    }
    DecParams dp{};
    const bool inline_items = n_items <= kMaxParamItems;
    if (!inline_items) {
        // Pageable source: the runtime has staged the bytes by the time this returns, so the host array can be reused.
        if (cudaMemcpyAsync(base + kOffItems, g_items_host, sizeof(DecItem) * size_t(n_items), cudaMemcpyHostToDevice,
                            st) != cudaSuccess) {
            fail(err, err_len, "flint_attn_decode_noalloc_dev: work-list upload failed");
            return -1;
        }
    }
    dp.items = inline_items ? nullptr : reinterpret_cast<const DecItem *>(base + kOffItems);
    dp.qkv = qkv_dev;
    dp.out = out_dev;
    dp.partial_out = nullptr;
    dp.q_norm = q_norm_dev; dp.k_norm = k_norm_dev; dp.sinks = sinks_dev;
    dp.inv_freq = reinterpret_cast<const float *>(base + kOffFreq);
    dp.k_cache = static_cast<__half *>(k_cache_dev);
    dp.v_cache = static_cast<__half *>(v_cache_dev);
    dp.scratch = reinterpret_cast<float *>(base + kOffRecords);
    dp.scratch2 = reinterpret_cast<float *>(base + kOffRecords2);
    dp.tickets = reinterpret_cast<int *>(base + kOffTickets);  // left at zero by the kernel after every launch
    dp.tickets2 = dp.tickets + kMaxRuns;
    dp.seq_stride = (long long)kNHeadKv * n_slots * kHeadDim;
    dp.n_slots = n_slots;
    dp.slot_mask = is_swa ? uint32_t(kSwaRing - 1) : 0xFFFFFFFFu;
    dp.kv_lo = 0;
    dp.has_rope = has_rope;
    dp.qkv_dtype = qkv_dtype; dp.out_dtype = out_dtype;
    dp.mode = 0;
    const cudaError_t e = inline_items ? launch_decode_inline(dp, g_items_host, n_items, g_state[dev].sm_count, st)
                                       : launch_decode(dp, n_items, st);
    if (e != cudaSuccess) {
        snprintf(msg, sizeof(msg), "flint_attn_decode_noalloc_dev: launch failed: %s", cudaGetErrorString(e));
        fail(err, err_len, msg);
        return -1;
    }
    return 0;
}
