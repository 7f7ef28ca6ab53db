// Host side of the attention library: the handle behind include/flint_attn.h, KV-cache ownership, the split-K
// work planner and the C ABI.  Plays the role of the attention parts of the reference's Engine
// (src/engine.mm:509-511 cache allocation, :735-766 decode dispatch, :1080-1104 prefill chunk loop) and of its
// C boundary (src/capi.mm:17-74: try/catch at every entry, message copied into the caller's buffer).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/flint_attn.h"
#include "attn_common.h"
#include "prefill_attn.h"
#include "proj.h"

using namespace flint;

namespace {

void set_err(char *err, int32_t len, const char *msg) {  // src/capi.mm:17-22
    if (err && len > 0) {
        strncpy(err, msg, size_t(len) - 1);
        err[len - 1] = 0;
    }
}

#define CK(call)                                                                                      \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e_) + " at " #call); \
    } while (0)

struct Layer {
    bool is_swa = false, has_rope = false, has_weights = false;
    bool paged = false;  // full layer whose K/V live in a page pool [kv_pages][4][64][128] shared by all sequences
    int n_slots = 0;
    int kv_lo = 0, kv_hi = 0;  // positions a full layer holds on this device: [kv_lo, kv_hi)
    __half *k = nullptr, *v = nullptr;
    float *q_norm = nullptr, *k_norm = nullptr, *sinks = nullptr;  // device copies
    // projections either side of attention (optional): attn_norm [n_embd] fp32, W_qkv [5120][n_embd] bf16 (q rows,
    // then k rows, then v rows: the packed row of src/metal/fused.metal:211), W_o [n_embd][4096] bf16
    unsigned char *kv_maps = nullptr;  // full layers: two tensor maps (K, V) in device memory for the decode kernel's TMA loads
    int n_embd = 0;
    float *attn_norm = nullptr;
    __nv_bfloat16 *w_qkv = nullptr, *w_o = nullptr;
};

constexpr int kRing = 4;  // work lists in flight

int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Own split policy.  The reference's (src/engine.mm:742-743: at most 32 splits of at least 256 keys) fills an
// M5.  On a B200 every work item pays a few microseconds of start-up and merge, so the launch aims for ONE wave:
// about as many items as there are CTA slots (2 per SM), each as long as possible.  The chunk length is the total
// number of cached key rows of the launch divided by the slots; a (token, KV head) group gets round(keys / chunk)
// splits (at least one), so a batch of equally long sequences is not cut in two just because it is a little longer
// than the chunk.
// The planner runs in front of every launch, so it allocates nothing once its buffers have grown, and it orders
// the items through 64-bit (length, index) keys instead of moving 48-byte structs in a sort.
struct PlanScratch {
    std::vector<int> lo, hi;
    std::vector<DecItem> gen;
    std::vector<uint64_t> keys;
};

// The last work list of a layer, kept so that the usual next call -- the same batch, every position advanced by one
// -- is a patch of a few fields per item instead of a new plan (the planner is most of the host time of a call).
// A patched list keeps the split structure of the plan it came from, so it is rebuilt from scratch every kPlanMaxAge
// steps; by then a range has grown by at most one 64-key tile.
constexpr int kPlanMaxAge = 64;
constexpr int kPlanWays = 4;  // batches remembered per layer (a server may alternate between a few fixed batches)
struct PlanCache {
    bool valid = false;
    int target_items = 0, n_groups = 0, n_records = 0, n_subs = 0, age = 0;
    std::vector<int32_t> seqs, pos;
    std::vector<DecItem> items;
};

// One planning pass for a given number of CTA slots.  Returns the longest item's keys; `total_rows` gets the cached
// rows summed over all (sequence, KV head) groups.
static int plan_decode_for(int n, const int32_t *seqs, const int32_t *pos, bool is_swa, int kv_lo, int kv_hi,
                           int target_items, std::vector<DecItem> &items, int &n_groups, int &n_records, int &n_subs,
                           PlanScratch &ps, long long &total_rows) {
    long long total = 0;
    ps.lo.resize(n);
    ps.hi.resize(n);
    int *lo = ps.lo.data(), *hi = ps.hi.data();
    for (int i = 0; i < n; i++) {
        const int kb = is_swa ? std::max(pos[i] - (kNSwa - 1), 0) : 0;  // src/metal/fused.metal:265
        lo[i] = std::min(std::max(kb, kv_lo), pos[i]);
        hi[i] = std::max(lo[i], std::min(pos[i], kv_hi));
        total += hi[i] - lo[i];
    }
    total *= kNHeadKv;
    total_rows = total;
    if (target_items < 1) target_items = 1;
    // A window of at most 512 cached keys is never split: two 256-key items plus their merge take longer than one
    // 512-key item (12.4 vs 10.3 us per launch for 32 sequences).  Full layers split down to 256 keys: there a lone
    // CTA scanning 1024 keys is slower than four CTAs and a merge (14.4 vs 11.1 us).
    const int min_chunk = is_swa ? 512 : 256;
    int chunk = round_up(int(std::max<long long>(min_chunk, (total + target_items - 1) / target_items)), 64);
    // Rounding every group to its nearest number of splits can overshoot the target (64 groups x 5 splits = 320 items
    // for 296 slots: a second wave that nearly doubles the launch).  If it does, the chunk grows until the list fits.
    auto splits_of = [](int nk, int c) { return std::max(1, (nk + c / 2) / c); };  // the nearest count
    auto count_items = [&](int c) {
        long long items = 0;
        for (int i = 0; i < n; i++) {
            const int nk = hi[i] - lo[i];
            int n_split = splits_of(nk, c);
            const int per = std::max(64, round_up((nk + n_split - 1) / n_split, 64));
            items += std::max(1, (nk + per - 1) / per);
        }
        return items * kNHeadKv;
    };
    for (int tries = 0; tries < 8 && chunk > min_chunk && count_items(chunk) > target_items && n * kNHeadKv <= target_items; tries++)
        chunk = round_up(int((long long)chunk * count_items(chunk) / target_items) + 1, 64);
    n_groups = n * kNHeadKv;
    n_records = 0;
    n_subs = 0;
    std::vector<DecItem> &gen = items;  // generated in place; reordered below only when needed
    gen.clear();
    bool sorted = true;  // already longest first?
    int prev_len = INT32_MAX, max_len = 0;
    for (int i = 0; i < n; i++) {
        const int nk = hi[i] - lo[i];
        const bool own_new = kv_lo <= pos[i] && pos[i] < kv_hi;
        int n_split = splits_of(nk, chunk);
        const int per = std::max(64, round_up((nk + n_split - 1) / n_split, 64));
        n_split = std::max(1, (nk + per - 1) / per);
        for (int kvh = 0; kvh < kNHeadKv; kvh++) {
            const int part0 = n_records, sub0 = n_subs;
            if (n_split > 1) {
                n_records += n_split;
                n_subs += (n_split + kMergeFan - 1) / kMergeFan;
            }
            for (int s = 0; s < n_split; s++) {
                DecItem it{};
                it.tok = i;
                it.seq = seqs ? seqs[i] : i;
                it.kvh = kvh;
                it.pos = pos[i];
                it.j0 = lo[i] + s * per;
                it.j1 = std::min(hi[i], lo[i] + (s + 1) * per);
                it.fold = (own_new && s == n_split - 1) ? 1 : 0;
                it.split = s;
                it.n_split = n_split;
                it.part0 = part0;
                it.group = i * kNHeadKv + kvh;
                it.sub0 = sub0;
                const int len = it.j1 - it.j0;
                sorted = sorted && len <= prev_len;
                prev_len = len;
                max_len = std::max(max_len, len);
                gen.push_back(it);
            }
        }
    }
    // longest first: the block scheduler hands CTAs out in order, which makes this a greedy LPT schedule
    if (sorted) return max_len;
    const size_t m = items.size();
    ps.keys.resize(m);
    for (size_t i = 0; i < m; i++)  // ascending key = descending length, ties in generation order
        ps.keys[i] = (uint64_t(uint32_t(INT32_MAX - (items[i].j1 - items[i].j0))) << 32) | uint32_t(i);
    std::sort(ps.keys.begin(), ps.keys.end());
    ps.gen.assign(items.begin(), items.end());
    for (size_t i = 0; i < m; i++) items[i] = ps.gen[uint32_t(ps.keys[i])];
    return max_len;
}

// The work list of one decode launch.  A batch of equal sequences is cut into one wave of items (every item pays a
// few microseconds of start-up and merge: 8 x 8192 keys take 33 us as 128-288 items, 38-40 us as 384-592).  A ragged
// batch cut that way leaves one item per slot with lengths up to 1.5x the mean, and the launch lasts as long as its
// longest item; when the longest item of the one-wave list exceeds the mean slot load by more than a fifth the list
// is planned again for two waves of shorter items, which the longest-first order packs well (32 sequences of 1..32768
// keys: 190 -> 166 us; 64 such sequences: 405 -> 319 us; three or more waves are slower again).
void plan_decode(int n, const int32_t *seqs, const int32_t *pos, bool is_swa, int kv_lo, int kv_hi, int target_items,
                 std::vector<DecItem> &items, int &n_groups, int &n_records, int &n_subs, PlanScratch &ps) {
    long long total = 0;
    if (target_items < 1) target_items = 1;
    const int max_len = plan_decode_for(n, seqs, pos, is_swa, kv_lo, kv_hi, target_items, items, n_groups, n_records,
                                        n_subs, ps, total);
    if (!is_swa && n * kNHeadKv <= target_items && (long long)max_len * target_items * 5 > total * 6)
        plan_decode_for(n, seqs, pos, is_swa, kv_lo, kv_hi, 2 * target_items, items, n_groups, n_records, n_subs, ps,
                        total);
}

// Brings a cached work list to the positions `pos` when they equal the cached ones or are all one ahead, and nothing
// about who folds the new token changed.  Returns false when the list has to be planned again.
bool patch_plan(PlanCache &pc, int n, const int32_t *seqs, const int32_t *pos, bool is_swa, int kv_lo, int kv_hi,
                int target_items) {
    if (!pc.valid || pc.target_items != target_items || int(pc.pos.size()) != n) return false;
    if (memcmp(pc.seqs.data(), seqs, sizeof(int32_t) * size_t(n)) != 0) return false;
    const int d = n > 0 ? pos[0] - pc.pos[0] : 0;
    if (d != 0 && d != 1) return false;
    for (int i = 0; i < n; i++) {
        if (pos[i] - pc.pos[i] != d) return false;
        if ((kv_lo <= pos[i] && pos[i] < kv_hi) != (kv_lo <= pc.pos[i] && pc.pos[i] < kv_hi)) return false;
    }
    if (d == 0) return true;
    if (pc.age + 1 >= kPlanMaxAge) return false;
    pc.age++;
    for (DecItem &it : pc.items) {
        const int p = pos[it.tok];
        it.pos = p;
        if (it.split != it.n_split - 1) continue;  // only the last range of a group ends at the position
        const int kb = is_swa ? std::max(p - (kNSwa - 1), 0) : 0;
        const int lo = std::min(std::max(kb, kv_lo), p);
        if (it.n_split == 1) it.j0 = lo;  // a sliding window moves with the position (windows are never split)
        it.j1 = std::max(it.j0, std::min(p, kv_hi));
    }
    memcpy(pc.pos.data(), pos, sizeof(int32_t) * size_t(n));
    return true;
}

}  // namespace

struct flint_attn {
    int device = 0, max_seqs = 0, n_ctx = 0, kv_rank = 0, kv_ranks = 1;
    int sm_count = 148, target_items = 0;
    // Paged KV (kv_pages > 0): one block table and one free list serve every paged layer -- all full layers hold the
    // same positions of a sequence, so block b of sequence s is page table[s][b] in each layer's own pool.
    int kv_pages = 0, pages_per_seq = 0;
    std::vector<int32_t> table_host;   // [max_seqs][pages_per_seq], -1 = no page
    std::vector<int32_t> seq_blocks;   // blocks each sequence holds
    std::vector<int32_t> free_pages;   // stack of free page numbers
    int32_t *table_dev = nullptr;
    int *dec_err = nullptr;  // device word the decode kernel sets when a bounded wait runs out
    std::vector<Layer> layers;
    std::vector<int32_t> pos;
    float *inv_freq = nullptr;
    float *scratch = nullptr, *scratch2 = nullptr;
    size_t scratch_recs = 0, scratch2_recs = 0;
    int *tickets = nullptr;
    size_t n_tickets = 0;
    // pinned host staging for work lists + matching device buffers, reused round-robin behind events
    DecItem *ring_host[kRing] = {};
    DecItem *ring_dev[kRing] = {};
    size_t ring_cap[kRing] = {};
    cudaEvent_t ring_ev[kRing] = {};
    int ring_next = 0;
    cudaStream_t stream = nullptr;  // used by the host-buffer entry points
    void *io_dev = nullptr;         // device staging for host-buffer calls
    size_t io_cap = 0;
    PrefillWorkspace pf;
    ProjWorkspace proj_ws;
    float *block_buf = nullptr;  // [rows][5120 + 4096] fp32: the q|k|v rows and the attention rows of a block call
    size_t block_rows = 0;
    int64_t launches = 0;
    std::vector<PlanCache> plan_cache;  // kPlanWays per layer
    std::vector<int> plan_victim;       // per layer: the way the next unknown batch replaces
    PlanScratch plan_scratch;
    std::vector<int32_t> batch_pos;
    std::vector<uint32_t> seen;  // per sequence: the number of the last decode batch it appeared in
    uint32_t batch_no = 0;
    // peer-memory exchange of partial records (KV-range sharding): one cudaMalloc block per rank, opened by the
    // others through CUDA IPC.  Layout: [flags: kMaxPeers words | error word | groups-done counter] in the first 256
    // bytes, then records [2 buffers][ranks][xchg_n][32][130] floats (buffers alternate per step).
    unsigned char *xchg = nullptr;
    unsigned char *xchg_peer[kMaxPeers] = {};
    bool xchg_opened[kMaxPeers] = {};
    int xchg_n = 0;
    uint32_t xchg_step = 0;
    // optional device timing of the attention kernels alone (events around each launch)
    bool timing = false;
    std::vector<cudaEvent_t> ev_pool;
    size_t ev_used = 0;

    ~flint_attn() {
        cudaSetDevice(device);
        for (auto &L : layers) {
            cudaFree(L.k); cudaFree(L.v); cudaFree(L.q_norm); cudaFree(L.k_norm); cudaFree(L.sinks);
            cudaFree(L.attn_norm); cudaFree(L.w_qkv); cudaFree(L.w_o); cudaFree(L.kv_maps);
        }
        cudaFree(dec_err);
        proj_workspace_free(proj_ws);
        cudaFree(block_buf);
        cudaFree(table_dev);
        cudaFree(inv_freq); cudaFree(scratch); cudaFree(scratch2); cudaFree(tickets); cudaFree(io_dev);
        for (int i = 0; i < kRing; i++) {
            if (ring_host[i]) cudaFreeHost(ring_host[i]);
            cudaFree(ring_dev[i]);
            if (ring_ev[i]) cudaEventDestroy(ring_ev[i]);
        }
        prefill_workspace_free(pf);
        for (int r = 0; r < kMaxPeers; r++)
            if (xchg_opened[r]) cudaIpcCloseMemHandle(xchg_peer[r]);
        cudaFree(xchg);
        for (cudaEvent_t e : ev_pool) cudaEventDestroy(e);
        if (stream) cudaStreamDestroy(stream);
    }

    cudaEvent_t next_event() {
        if (ev_used == ev_pool.size()) {
            cudaEvent_t e;
            CK(cudaEventCreate(&e));
            ev_pool.push_back(e);
        }
        return ev_pool[ev_used++];
    }
    void time_mark(cudaStream_t st) {
        if (!timing) return;
        CK(cudaEventRecord(next_event(), st));
    }

    Layer &layer(int il) {
        if (il < 0 || il >= int(layers.size())) throw std::runtime_error("layer index out of range");
        Layer &L = layers[il];
        if (!L.has_weights) throw std::runtime_error("layer weights not set (flint_attn_set_layer)");
        return L;
    }

    // Make sure sequence `seq` owns the pages of positions [0, last_pos].  New table entries are uploaded on `st`, in
    // front of the launch that will read them (pageable source: staged before the call returns); entries that
    // kernels already in flight read are never rewritten.
    void ensure_pages(int seq, int last_pos, cudaStream_t st) {
        const int need = last_pos / kPageKeys + 1, have = seq_blocks[seq];
        if (need <= have) return;
        if (size_t(need - have) > free_pages.size())
            throw std::runtime_error("KV page pool exhausted (" + std::to_string(kv_pages) + " pages of 64 keys)");
        int32_t *row = table_host.data() + size_t(seq) * pages_per_seq;
        for (int b = have; b < need; b++) {
            row[b] = free_pages.back();
            free_pages.pop_back();
        }
        CK(cudaMemcpyAsync(table_dev + size_t(seq) * pages_per_seq + have, row + have, size_t(need - have) * sizeof(int32_t),
                           cudaMemcpyHostToDevice, st));
        seq_blocks[seq] = need;
    }

    void check_seqs(int n, const int32_t *seqs) const {
        if (n <= 0 || n > max_seqs) throw std::runtime_error("batch size out of range");
        for (int i = 0; i < n; i++)
            if (seqs[i] < 0 || seqs[i] >= max_seqs) throw std::runtime_error("sequence index out of range");
    }

    void ensure_io(size_t bytes) {
        if (bytes <= io_cap) return;
        cudaFree(io_dev);
        io_dev = nullptr;
        io_cap = 0;
        CK(cudaMalloc(&io_dev, bytes));
        io_cap = bytes;
    }

    // Upload a work list through the pinned ring; returns the device copy, valid for the next launch on `st`.
    const DecItem *upload_items(const std::vector<DecItem> &items, cudaStream_t st) {
        const int r = ring_next;
        ring_next = (ring_next + 1) % kRing;
        CK(cudaEventSynchronize(ring_ev[r]));  // the launch that last used this slot has consumed it
        const size_t need = items.size();
        if (need > ring_cap[r]) {
            if (ring_host[r]) cudaFreeHost(ring_host[r]);
            cudaFree(ring_dev[r]);
            ring_host[r] = nullptr;
            ring_dev[r] = nullptr;
            ring_cap[r] = 0;
            const size_t cap = std::max<size_t>(need * 2, 1024);
            CK(cudaMallocHost(&ring_host[r], cap * sizeof(DecItem)));
            CK(cudaMalloc(&ring_dev[r], cap * sizeof(DecItem)));
            ring_cap[r] = cap;
        }
        memcpy(ring_host[r], items.data(), need * sizeof(DecItem));
        CK(cudaMemcpyAsync(ring_dev[r], ring_host[r], need * sizeof(DecItem), cudaMemcpyHostToDevice, st));
        return ring_dev[r];
    }
    void mark_ring_used(const DecItem *dev, cudaStream_t st) {
        for (int i = 0; i < kRing; i++)
            if (ring_dev[i] == dev) CK(cudaEventRecord(ring_ev[i], st));
    }

    void ensure_scratch(int n_records, int n_subs, int n_groups) {
        auto grow = [&](float *&buf, size_t &have, size_t need, size_t floor_recs) {
            if (need <= have) return;
            CK(cudaDeviceSynchronize());  // earlier launches may still be using the old buffer
            cudaFree(buf);
            buf = nullptr;
            have = 0;
            const size_t recs = std::max<size_t>(need * 2, floor_recs);
            CK(cudaMalloc(&buf, recs * kGqa * kRecStride * sizeof(float)));
            have = recs;
        };
        grow(scratch, scratch_recs, size_t(n_records), 4096);
        grow(scratch2, scratch2_recs, size_t(n_subs), 1024);
        if (size_t(n_subs + n_groups) > n_tickets) {
            CK(cudaDeviceSynchronize());
            cudaFree(tickets);
            tickets = nullptr;
            n_tickets = 0;
            const size_t nt = std::max<size_t>(size_t(n_subs + n_groups) * 2, 4096);
            CK(cudaMalloc(&tickets, nt * sizeof(int)));
            CK(cudaMemset(tickets, 0, nt * sizeof(int)));
            n_tickets = nt;
        }
    }

    // Rows of a host-buffer call.  `mapped` is the device address of the caller's page-locked rows (null if they
    // are pageable): the kernel then reads them in place; otherwise they are copied to `staging` first.
    struct HostRows {
        const void *host = nullptr, *mapped = nullptr;
        void *staging = nullptr;
        size_t bytes = 0;
    };

    // mode 0: out [n][4096]; mode 1: partial_out [n][32][130]; mode 2: records to every peer's gather buffer
    void decode_dev(int il, int n, const int32_t *seqs, const void *qkv, int qkv_dtype, void *out, int out_dtype,
                    float *partial_out, int mode, cudaStream_t st, uint32_t step = 0, const HostRows *rows = nullptr) {
        CK(cudaSetDevice(device));
        Layer &L = layer(il);
        check_seqs(n, seqs);
        if (qkv_dtype != kDtypeF32 && qkv_dtype != kDtypeBf16) throw std::runtime_error("bad qkv dtype");
        if (mode == 0 && out_dtype != kDtypeF32 && out_dtype != kDtypeBf16) throw std::runtime_error("bad out dtype");
        if (mode == 0 && kv_ranks > 1 && !L.is_swa)
            throw std::runtime_error("full layers of a KV-sharded handle need decode_partial + combine");
        std::vector<int32_t> &p = batch_pos;
        p.resize(n);
        if (seen.size() != size_t(max_seqs)) seen.assign(max_seqs, 0);
        if (++batch_no == 0) {  // the counter wrapped: forget every stamp
            std::fill(seen.begin(), seen.end(), 0u);
            batch_no = 1;
        }
        for (int i = 0; i < n; i++) {
            p[i] = pos[seqs[i]];
            if (p[i] >= n_ctx) throw std::runtime_error("context full");  // src/engine.mm:904
            if (seen[seqs[i]] == batch_no) throw std::runtime_error("a sequence appears twice in one decode batch");
            seen[seqs[i]] = batch_no;
        }
        if (L.paged) {  // all or nothing: a batch that does not fit the pool takes no page
            size_t want = 0;
            for (int i = 0; i < n; i++) want += size_t(std::max(0, p[i] / kPageKeys + 1 - seq_blocks[seqs[i]]));
            if (want > free_pages.size())
                throw std::runtime_error("KV page pool exhausted (" + std::to_string(kv_pages) + " pages of 64 keys)");
            for (int i = 0; i < n; i++) ensure_pages(seqs[i], p[i], st);
        }
        PlanCache *hit = nullptr;
        for (int w = 0; w < kPlanWays && !hit; w++) {
            PlanCache &c = plan_cache[size_t(il) * kPlanWays + w];
            if (c.valid && int(c.seqs.size()) == n && c.seqs[0] == seqs[0] &&
                patch_plan(c, n, seqs, p.data(), L.is_swa, L.kv_lo, L.kv_hi, target_items))
                hit = &c;
        }
        if (!hit) {
            // replace the way that holds this batch at other positions, else the next victim
            int way = -1;
            for (int w = 0; w < kPlanWays && way < 0; w++) {
                const PlanCache &c = plan_cache[size_t(il) * kPlanWays + w];
                if (c.valid && int(c.seqs.size()) == n && memcmp(c.seqs.data(), seqs, sizeof(int32_t) * size_t(n)) == 0) way = w;
            }
            if (way < 0) way = plan_victim[il] = (plan_victim[il] + 1) % kPlanWays;
            hit = &plan_cache[size_t(il) * kPlanWays + way];
            hit->valid = false;
            plan_decode(n, seqs, p.data(), L.is_swa, L.kv_lo, L.kv_hi, target_items, hit->items, hit->n_groups,
                        hit->n_records, hit->n_subs, plan_scratch);
            hit->seqs.assign(seqs, seqs + n);
            hit->pos.assign(p.begin(), p.end());
            hit->target_items = target_items;
            hit->age = 0;
            hit->valid = true;
        }
        PlanCache &pc = *hit;
        const std::vector<DecItem> &items = pc.items;
        const int n_groups = pc.n_groups, n_records = pc.n_records, n_subs = pc.n_subs;
        if (rows) {
            // Page-locked rows are read by the kernel where they lie (each CTA fetches the 2-4 KB it needs over PCIe
            // behind its first K/V tiles) unless the groups are cut into many ranges, each of which would fetch the
            // same rows again; then, and for pageable rows, one copy brings them to the device first.
            if (rows->mapped && items.size() <= 2 * size_t(n_groups)) qkv = rows->mapped;
            else {
                CK(cudaMemcpyAsync(rows->staging, rows->host, rows->bytes, cudaMemcpyHostToDevice, st));
                qkv = rows->staging;
            }
        }
        ensure_scratch(n_records, n_subs, n_groups);
        const bool inline_items = items.size() <= size_t(kMaxParamItems);
        DecParams dp{};
        dp.items = inline_items ? nullptr : upload_items(items, st);
        dp.qkv = qkv;
        dp.out = out;
        dp.partial_out = partial_out;
        dp.q_norm = L.q_norm; dp.k_norm = L.k_norm; dp.sinks = L.sinks; dp.inv_freq = inv_freq;
        dp.k_cache = L.k; dp.v_cache = L.v;
        dp.scratch = scratch; dp.scratch2 = scratch2;
        dp.tickets = tickets; dp.tickets2 = tickets + n_subs;
        dp.seq_stride = (long long)kNHeadKv * L.n_slots * kHeadDim;
        dp.n_slots = L.n_slots;
        dp.slot_mask = L.is_swa ? uint32_t(kSwaRing - 1) : 0xFFFFFFFFu;
        dp.kv_lo = L.is_swa ? 0 : L.kv_lo;
        dp.has_rope = L.has_rope;
        dp.qkv_dtype = qkv_dtype; dp.out_dtype = out_dtype;
        dp.mode = mode;
        dp.paged = L.paged ? 1 : 0;
        dp.block_table = table_dev;
        dp.table_stride = pages_per_seq;
        dp.k_map = L.kv_maps;
        dp.v_map = L.kv_maps ? L.kv_maps + 128 : nullptr;
        dp.error_flag = dec_err;
        if (mode == 2) {
            const size_t rec_bytes = size_t(xchg_n) * kNHead * kPartialDim * sizeof(float);
            const size_t buf_off = 256 + size_t(step & 1) * kv_ranks * rec_bytes + size_t(kv_rank) * rec_bytes;
            for (int r = 0; r < kv_ranks; r++) {
                dp.peer_out[r] = reinterpret_cast<float *>(xchg_peer[r] + buf_off);
                dp.peer_flag[r] = reinterpret_cast<uint32_t *>(xchg_peer[r]);
            }
            dp.n_peers = kv_ranks;
            dp.rank = kv_rank;
            dp.step = step;
            dp.groups_done = reinterpret_cast<int *>(xchg + (kMaxPeers + 1) * sizeof(uint32_t));
            dp.n_groups = n_groups;
        }
        time_mark(st);
        if (inline_items) CK(launch_decode_inline(dp, items.data(), int(items.size()), sm_count, st));
        else CK(launch_decode(dp, int(items.size()), st));
        time_mark(st);
        launches++;
        if (!inline_items) mark_ring_used(dp.items, st);
    }
};

// ============================================================================ C ABI
#define API_TRY try {
#define API_CATCH(ret)                       \
    }                                        \
    catch (const std::exception &ex) {       \
        set_err(err, err_len, ex.what());    \
        return ret;                          \
    }

extern "C" {

flint_attn *flint_attn_open(const flint_attn_config *cfg, char *err, int32_t err_len) {
    flint_attn *a = nullptr;
    try {
        if (!cfg) throw std::runtime_error("null config");
        if (cfg->n_layers <= 0 || !cfg->layer_is_swa || !cfg->layer_has_rope) throw std::runtime_error("bad layer table");
        if (cfg->max_seqs <= 0 || cfg->n_ctx <= 0) throw std::runtime_error("max_seqs and n_ctx must be positive");
        const int ranks = cfg->kv_ranks > 1 ? cfg->kv_ranks : 1;
        if (cfg->kv_rank < 0 || cfg->kv_rank >= ranks) throw std::runtime_error("kv_rank out of range");
        if (cfg->kv_pages < 0) throw std::runtime_error("kv_pages must not be negative");
        if (cfg->kv_pages > 0 && ranks > 1) throw std::runtime_error("a paged KV cache cannot also be sharded by key range");
        int n_dev = 0;
        CK(cudaGetDeviceCount(&n_dev));
        if (cfg->device < 0 || cfg->device >= n_dev) throw std::runtime_error("no such CUDA device");
        CK(cudaSetDevice(cfg->device));
        cudaDeviceProp prop{};
        CK(cudaGetDeviceProperties(&prop, cfg->device));
        if (prop.major != 10)
            throw std::runtime_error("this library is built for sm_100a (B200) only; device is sm_" +
                                     std::to_string(prop.major) + std::to_string(prop.minor));
        a = new flint_attn();
        a->device = cfg->device;
        a->max_seqs = cfg->max_seqs;
        a->n_ctx = cfg->n_ctx;
        a->kv_rank = cfg->kv_rank;
        a->kv_ranks = ranks;
        a->sm_count = prop.multiProcessorCount;
        a->target_items = a->sm_count * 2;
        a->pos.assign(cfg->max_seqs, 0);
        if (cfg->kv_pages > 0) {
            a->kv_pages = cfg->kv_pages;
            a->pages_per_seq = (cfg->n_ctx + kPageKeys - 1) / kPageKeys;
            a->table_host.assign(size_t(cfg->max_seqs) * a->pages_per_seq, -1);
            a->seq_blocks.assign(cfg->max_seqs, 0);
            a->free_pages.resize(cfg->kv_pages);
            for (int i = 0; i < cfg->kv_pages; i++) a->free_pages[i] = cfg->kv_pages - 1 - i;  // page 0 is handed out first
            CK(cudaMalloc(&a->table_dev, a->table_host.size() * sizeof(int32_t)));
            CK(cudaMemset(a->table_dev, 0xff, a->table_host.size() * sizeof(int32_t)));
        }
        CK(cudaStreamCreateWithFlags(&a->stream, cudaStreamNonBlocking));
        for (int i = 0; i < kRing; i++) CK(cudaEventCreateWithFlags(&a->ring_ev[i], cudaEventDisableTiming));
        CK(decode_kernel_setup());
        CK(prefill_kernel_setup());
        CK(cudaMalloc(&a->dec_err, sizeof(int)));
        CK(cudaMemset(a->dec_err, 0, sizeof(int)));
        float freq[kHeadDim / 2];
        for (int i = 0; i < kHeadDim / 2; i++) freq[i] = powf(kRopeTheta, -2.0f * i / kHeadDim);  // ref_model.cpp:55
        CK(cudaMalloc(&a->inv_freq, sizeof(freq)));
        CK(cudaMemcpy(a->inv_freq, freq, sizeof(freq), cudaMemcpyHostToDevice));
        const int shard = (cfg->n_ctx + ranks - 1) / ranks;
        a->layers.resize(cfg->n_layers);
        a->plan_cache.resize(size_t(cfg->n_layers) * kPlanWays);
        a->plan_victim.assign(cfg->n_layers, 0);
        for (int il = 0; il < cfg->n_layers; il++) {
            Layer &L = a->layers[il];
            L.is_swa = cfg->layer_is_swa[il] != 0;
            L.has_rope = cfg->layer_has_rope[il] != 0;
            if (L.is_swa) {
                L.n_slots = kSwaRing;  // src/engine.mm:509
                L.kv_lo = 0;
                L.kv_hi = INT32_MAX;
            } else {
                L.kv_lo = std::min(cfg->n_ctx, a->kv_rank * shard);
                L.kv_hi = std::min(cfg->n_ctx, L.kv_lo + shard);
                L.n_slots = std::max(1, L.kv_hi - L.kv_lo);
            }
            L.paged = !L.is_swa && cfg->kv_pages > 0;
            const size_t bytes = L.paged ? size_t(cfg->kv_pages) * kNHeadKv * kPageKeys * kHeadDim * sizeof(__half)
                                         : size_t(cfg->max_seqs) * kNHeadKv * L.n_slots * kHeadDim * sizeof(__half);
            CK(cudaMalloc(&L.k, bytes));
            CK(cudaMalloc(&L.v, bytes));
            CK(cudaMemset(L.k, 0, bytes));
            CK(cudaMemset(L.v, 0, bytes));
            // Full layers feed the decode kernel's K/V tiles by TMA (FLINT_ATTN_NO_TMA=1 keeps the cp.async path).
            static const bool no_tma = [] {
                const char *v = getenv("FLINT_ATTN_NO_TMA");
                return v && v[0] == '1';
            }();
            if (!L.is_swa && !no_tma) {
                const long long rows = L.paged ? (long long)cfg->kv_pages * kNHeadKv * kPageKeys
                                               : (long long)cfg->max_seqs * kNHeadKv * L.n_slots;
                if (rows < (1ll << 31)) {  // TMA coordinates are 32-bit
                    alignas(64) unsigned char maps[256];
                    CK(make_kv_rows_map(maps, L.k, rows));
                    CK(make_kv_rows_map(maps + 128, L.v, rows));
                    CK(cudaMalloc(&L.kv_maps, sizeof(maps)));
                    CK(cudaMemcpy(L.kv_maps, maps, sizeof(maps), cudaMemcpyHostToDevice));
                }
            }
            CK(cudaMalloc(&L.q_norm, kHeadDim * sizeof(float)));
            CK(cudaMalloc(&L.k_norm, kHeadDim * sizeof(float)));
            CK(cudaMalloc(&L.sinks, kNHead * sizeof(float)));
        }
        CK(cudaDeviceSynchronize());
        return a;
    } catch (const std::exception &ex) {
        set_err(err, err_len, ex.what());
        delete a;
        return nullptr;
    }
}

void flint_attn_close(flint_attn *a) {
    if (!a) return;
    cudaSetDevice(a->device);
    cudaDeviceSynchronize();
    delete a;
}

int32_t flint_attn_n_ctx(const flint_attn *a) { return a->n_ctx; }

int32_t flint_attn_pos(const flint_attn *a, int32_t seq) {
    if (seq < 0 || seq >= a->max_seqs) return -1;
    return a->pos[seq];
}

int32_t flint_attn_truncate(flint_attn *a, int32_t seq, int32_t pos) {  // src/capi.mm:52-56
    if (seq < 0 || seq >= a->max_seqs) return -1;
    if (pos < 0 || pos > a->pos[seq]) return -1;
    a->pos[seq] = pos;
    return 0;
}

int32_t flint_attn_rollback_restart(int32_t cached_len, int32_t pos) {  // server/src/main.rs:96-100
    if (cached_len > pos && cached_len - pos > 511) pos = pos >= 512 ? pos - 512 : 0;
    return pos;
}

int32_t flint_attn_set_pos(flint_attn *a, int32_t seq, int32_t pos) {
    if (seq < 0 || seq >= a->max_seqs || pos < 0 || pos > a->n_ctx) return -1;
    a->pos[seq] = pos;
    return 0;
}

int32_t flint_attn_advance(flint_attn *a, int32_t n, const int32_t *seqs, int32_t n_tokens) {
    if (n < 0 || n_tokens < 0) return -1;
    for (int i = 0; i < n; i++)
        if (seqs[i] < 0 || seqs[i] >= a->max_seqs || a->pos[seqs[i]] + n_tokens > a->n_ctx) return -1;
    for (int i = 0; i < n; i++) a->pos[seqs[i]] += n_tokens;
    return 0;
}

int32_t flint_attn_set_layer(flint_attn *a, int32_t layer, const float *q_norm, const float *k_norm,
                             const float *sinks, char *err, int32_t err_len) {
    API_TRY
    if (layer < 0 || layer >= int(a->layers.size())) throw std::runtime_error("layer index out of range");
    if (!q_norm || !k_norm || !sinks) throw std::runtime_error("null weight pointer");
    CK(cudaSetDevice(a->device));
    Layer &L = a->layers[layer];
    CK(cudaMemcpy(L.q_norm, q_norm, kHeadDim * sizeof(float), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.k_norm, k_norm, kHeadDim * sizeof(float), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.sinks, sinks, kNHead * sizeof(float), cudaMemcpyHostToDevice));
    L.has_weights = true;
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_decode_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs, const void *qkv_dev,
                              int32_t qkv_dtype, void *out_dev, int32_t out_dtype, void *cuda_stream, char *err,
                              int32_t err_len) {
    API_TRY
    a->decode_dev(layer, n, seqs, qkv_dev, qkv_dtype, out_dev, out_dtype, nullptr, 0, cudaStream_t(cuda_stream));
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_decode_partial_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs,
                                      const void *qkv_dev, int32_t qkv_dtype, float *partial_dev, void *cuda_stream,
                                      char *err, int32_t err_len) {
    API_TRY
    a->decode_dev(layer, n, seqs, qkv_dev, qkv_dtype, nullptr, 0, partial_dev, 1, cudaStream_t(cuda_stream));
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_xchg_create(flint_attn *a, int32_t n_max, void *ipc_handle_out, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    if (a->xchg) throw std::runtime_error("exchange buffer already created");
    if (n_max < 1 || n_max > a->max_seqs) throw std::runtime_error("n_max out of range");
    if (a->kv_ranks > kMaxPeers) throw std::runtime_error("at most 8 ranks can share a sequence");
    const size_t bytes = 256 + 2 * size_t(a->kv_ranks) * n_max * kNHead * kPartialDim * sizeof(float);
    CK(cudaMalloc(&a->xchg, bytes));
    CK(cudaMemset(a->xchg, 0, bytes));
    a->xchg_n = n_max;
    a->xchg_step = 0;
    a->xchg_peer[a->kv_rank] = a->xchg;
    if (ipc_handle_out) {
        cudaIpcMemHandle_t h;
        CK(cudaIpcGetMemHandle(&h, a->xchg));
        static_assert(sizeof(h) == FLINT_ATTN_IPC_HANDLE_BYTES, "IPC handle size");
        memcpy(ipc_handle_out, &h, sizeof(h));
    }
    CK(cudaDeviceSynchronize());
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_xchg_connect(flint_attn *a, const void *ipc_handles, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    if (!a->xchg) throw std::runtime_error("create the exchange buffer first");
    for (int r = 0; r < a->kv_ranks; r++) {
        if (r == a->kv_rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char *>(ipc_handles) + size_t(r) * sizeof(h), sizeof(h));
        void *ptr = nullptr;
        CK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        a->xchg_peer[r] = static_cast<unsigned char *>(ptr);
        a->xchg_opened[r] = true;
    }
    return 0;
    API_CATCH(-1)
}

void *flint_attn_xchg_base(flint_attn *a) { return a->xchg; }

int32_t flint_attn_xchg_connect_local(flint_attn *a, void *const *peer_bases, char *err, int32_t err_len) {
    API_TRY
    if (!a->xchg) throw std::runtime_error("create the exchange buffer first");
    for (int r = 0; r < a->kv_ranks; r++)
        if (r != a->kv_rank) a->xchg_peer[r] = static_cast<unsigned char *>(peer_bases[r]);
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_decode_xchg_post_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs,
                                        const void *qkv_dev, int32_t qkv_dtype, void *cuda_stream, char *err,
                                        int32_t err_len) {
    API_TRY
    if (!a->xchg) throw std::runtime_error("create and connect the exchange buffer first");
    for (int r = 0; r < a->kv_ranks; r++)
        if (!a->xchg_peer[r]) throw std::runtime_error("exchange buffer not connected to every rank");
    if (n > a->xchg_n) throw std::runtime_error("batch larger than the exchange buffer");
    if (a->layer(layer).is_swa) throw std::runtime_error("sliding-window layers are not sharded: use decode_dev");
    // The step counter moves only once the launch is enqueued: a call that fails validation (context full, a
    // duplicate sequence, a CUDA error) must leave this rank on the step its peers expect next.
    const uint32_t step = a->xchg_step + 1;
    a->decode_dev(layer, n, seqs, qkv_dev, qkv_dtype, nullptr, 0, nullptr, 2, cudaStream_t(cuda_stream), step);
    a->xchg_step = step;
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_combine_xchg_dev(flint_attn *a, int32_t layer, int32_t n, void *out_dev, int32_t out_dtype,
                                    void *cuda_stream, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    Layer &L = a->layer(layer);
    if (!a->xchg || a->xchg_step == 0) throw std::runtime_error("nothing was posted");
    if (n <= 0 || n > a->xchg_n) throw std::runtime_error("bad combine shape");
    if (out_dtype != kDtypeF32 && out_dtype != kDtypeBf16) throw std::runtime_error("bad out dtype");
    const size_t rec_floats = size_t(a->xchg_n) * kNHead * kPartialDim;
    CombineParams cp{};
    cp.partials = reinterpret_cast<const float *>(a->xchg + 256) + size_t(a->xchg_step & 1) * a->kv_ranks * rec_floats;
    cp.sinks = L.sinks; cp.out = out_dev;
    cp.n = n; cp.n_parts = a->kv_ranks; cp.out_dtype = out_dtype;
    cp.part_stride = int(rec_floats);
    cp.flags = reinterpret_cast<const uint32_t *>(a->xchg);
    cp.step = a->xchg_step;
    cp.error_flag = reinterpret_cast<int *>(a->xchg + kMaxPeers * sizeof(uint32_t));
    CK(launch_combine(cp, cudaStream_t(cuda_stream)));
    a->launches++;
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_combine_dev(flint_attn *a, int32_t layer, int32_t n, int32_t n_parts, const float *partials_dev,
                               void *out_dev, int32_t out_dtype, void *cuda_stream, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    Layer &L = a->layer(layer);
    if (n <= 0 || n_parts <= 0) throw std::runtime_error("bad combine shape");
    if (out_dtype != kDtypeF32 && out_dtype != kDtypeBf16) throw std::runtime_error("bad out dtype");
    CombineParams cp{};
    cp.partials = partials_dev; cp.sinks = L.sinks; cp.out = out_dev;
    cp.n = n; cp.n_parts = n_parts; cp.out_dtype = out_dtype;
    cp.part_stride = n * kNHead * kPartialDim;
    CK(launch_combine(cp, cudaStream_t(cuda_stream)));
    a->launches++;
    return 0;
    API_CATCH(-1)
}

static size_t elem_size(int dtype) { return dtype == kDtypeF32 ? 4 : 2; }

int32_t flint_attn_decode(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs, const void *qkv,
                          int32_t qkv_dtype, void *out, int32_t out_dtype, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    if (n <= 0 || n > a->max_seqs) throw std::runtime_error("batch size out of range");
    if ((qkv_dtype != kDtypeF32 && qkv_dtype != kDtypeBf16) || (out_dtype != kDtypeF32 && out_dtype != kDtypeBf16))
        throw std::runtime_error("bad dtype");
    const size_t in_bytes = size_t(n) * kQkvDim * elem_size(qkv_dtype);
    const size_t in_pad = (in_bytes + 255) / 256 * 256;
    const size_t out_bytes = size_t(n) * kQDim * elem_size(out_dtype);
    a->ensure_io(in_pad + out_bytes);
    char *d_in = static_cast<char *>(a->io_dev), *d_out = d_in + in_pad;
    // Rows in page-locked host memory are accessed by the kernel itself: output rows are posted writes over PCIe
    // that overlap the kernel's tail, input rows are fetched by the CTAs that need them.  Pageable rows go through
    // a device staging buffer and a copy each way.
    auto mapped_address = [](const void *host) -> void * {
        cudaPointerAttributes attr{};
        if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
            attr.devicePointer && (reinterpret_cast<uintptr_t>(attr.devicePointer) & 15) == 0)
            return attr.devicePointer;
        cudaGetLastError();  // pageable memory makes the query fail on some drivers: not an error here
        return nullptr;
    };
    void *out_mapped = mapped_address(out);
    flint_attn::HostRows rows;
    rows.host = qkv;
    rows.mapped = mapped_address(qkv);
    rows.staging = d_in;
    rows.bytes = in_bytes;
    a->decode_dev(layer, n, seqs, d_in, qkv_dtype, out_mapped ? out_mapped : d_out, out_dtype, nullptr, 0, a->stream, 0,
                  &rows);
    if (!out_mapped) CK(cudaMemcpyAsync(out, d_out, out_bytes, cudaMemcpyDeviceToHost, a->stream));
    CK(cudaStreamSynchronize(a->stream));  // synchronous like the reference (src/engine.mm:930)
    return 0;
    API_CATCH(-1)
}

static void prefill_impl(flint_attn *a, int layer, int seq, int n_tok, const void *qkv, int qkv_dtype, void *out,
                         int out_dtype, cudaStream_t st, float *partial_o = nullptr, float *partial_ml = nullptr) {
    CK(cudaSetDevice(a->device));
    Layer &L = a->layer(layer);
    if (seq < 0 || seq >= a->max_seqs) throw std::runtime_error("sequence index out of range");
    if (n_tok <= 0) throw std::runtime_error("empty prefill");  // src/engine.mm:975
    const int p0 = a->pos[seq];
    if (p0 + n_tok > a->n_ctx) throw std::runtime_error("context full");  // src/engine.mm:976
    if (a->kv_ranks > 1 && !L.is_swa && !partial_o)
        throw std::runtime_error("full layers of a KV-sharded handle need prefill_partial + prefill_combine");
    if (partial_o && L.is_swa) throw std::runtime_error("sliding-window layers are not sharded: use prefill_dev");
    if (partial_o && !partial_ml) throw std::runtime_error("null partial buffer");
    if ((qkv_dtype != kDtypeF32 && qkv_dtype != kDtypeBf16) ||
        (!partial_o && out_dtype != kDtypeF32 && out_dtype != kDtypeBf16))
        throw std::runtime_error("bad dtype");
    if (reinterpret_cast<uintptr_t>(qkv) & 15) throw std::runtime_error("q/k/v rows must start on a 16-byte boundary");
    PrefillParams pp{};
    pp.qkv = qkv; pp.out = out;
    pp.qkv_dtype = qkv_dtype; pp.out_dtype = out_dtype;
    pp.q_norm = L.q_norm; pp.k_norm = L.k_norm; pp.sinks = L.sinks; pp.inv_freq = a->inv_freq;
    pp.k_cache = L.k + (L.paged ? 0 : size_t(seq) * kNHeadKv * L.n_slots * kHeadDim);
    pp.v_cache = L.v + (L.paged ? 0 : size_t(seq) * kNHeadKv * L.n_slots * kHeadDim);
    if (L.paged) {
        a->ensure_pages(seq, p0 + n_tok - 1, st);
        pp.block_table = a->table_dev + size_t(seq) * a->pages_per_seq;
        pp.n_pages = a->kv_pages;
        pp.table_len = a->pages_per_seq;
    }
    pp.n_slots = L.n_slots;
    pp.is_swa = L.is_swa; pp.has_rope = L.has_rope;
    pp.p0 = p0; pp.n_tok = n_tok;
    if (!L.is_swa) {
        pp.kv_lo = L.kv_lo;
        pp.kv_hi = L.kv_hi;
        pp.with_sink = a->kv_rank == 0;  // the shard that holds position 0 carries the sink
    }
    pp.partial_o = partial_o;
    pp.partial_ml = partial_ml;
    int n_launch = 0;
    if (a->timing) {  // the attention kernel alone; the prologue is a separate, bandwidth-bound launch
        pp.ev_attn_begin = a->next_event();
        pp.ev_attn_end = a->next_event();
    }
    CK(launch_prefill(pp, a->pf, st, &n_launch));
    a->launches += n_launch;
}

// The attention block of one layer as the reference engine runs it between two residual-stream states
// (src/engine.mm:728-811 for one token, :1060-1112 for a prompt; src/ref/ref_model.cpp:108-151):
//   qkv = W_qkv . rmsnorm(x, attn_norm);  att = attention(qkv);  x += W_o . att
// The q|k|v rows and the attention rows stay in a scratch buffer of this handle (20 KB and 16 KB per token, which
// live in L2 between the three launches); x is read and updated in place.
static void attn_block(flint_attn *a, int layer, int n_rows, const int32_t *seqs, int seq, bool prefill, float *x,
                       cudaStream_t st) {
    CK(cudaSetDevice(a->device));
    Layer &L = a->layer(layer);
    if (!L.w_qkv) throw std::runtime_error("layer projections not set (flint_attn_set_projections)");
    if (!x) throw std::runtime_error("null residual stream");
    if (n_rows <= 0) throw std::runtime_error(prefill ? "empty prefill" : "batch size out of range");
    if (size_t(n_rows) > a->block_rows) {
        CK(cudaDeviceSynchronize());
        cudaFree(a->block_buf);
        a->block_buf = nullptr;
        a->block_rows = 0;
        const size_t rows = std::max<size_t>(size_t(n_rows), 64);
        CK(cudaMalloc(&a->block_buf, rows * (kQkvDim + kQDim) * sizeof(float)));
        a->block_rows = rows;
    }
    float *qkv = a->block_buf, *att = a->block_buf + a->block_rows * kQkvDim;
    int n_launch = 0;
    ProjCall pc{};
    pc.w = L.w_qkv; pc.act = x; pc.act_dtype = kDtypeF32; pc.norm_w = L.attn_norm;
    pc.out = qkv; pc.out_dtype = kDtypeF32; pc.residual = nullptr;
    pc.B = n_rows; pc.N = kQkvDim; pc.K = L.n_embd;
    CK(launch_proj(pc, a->proj_ws, a->sm_count, st, &n_launch));
    a->launches += n_launch;
    if (prefill) prefill_impl(a, layer, seq, n_rows, qkv, kDtypeF32, att, kDtypeF32, st);
    else a->decode_dev(layer, n_rows, seqs, qkv, kDtypeF32, att, kDtypeF32, nullptr, 0, st);
    pc = ProjCall{};
    pc.w = L.w_o; pc.act = att; pc.act_dtype = kDtypeF32; pc.norm_w = nullptr;
    pc.out = x; pc.out_dtype = kDtypeF32; pc.residual = x;
    pc.B = n_rows; pc.N = L.n_embd; pc.K = kQDim;
    CK(launch_proj(pc, a->proj_ws, a->sm_count, st, &n_launch));
    a->launches += n_launch;
}

int32_t flint_attn_prefill_dev(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, const void *qkv_dev,
                               int32_t qkv_dtype, void *out_dev, int32_t out_dtype, void *cuda_stream, char *err,
                               int32_t err_len) {
    API_TRY
    prefill_impl(a, layer, seq, n_tok, qkv_dev, qkv_dtype, out_dev, out_dtype, cudaStream_t(cuda_stream));
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_prefill_partial_dev(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, const void *qkv_dev,
                                       int32_t qkv_dtype, float *partial_o_dev, float *partial_ml_dev, void *cuda_stream,
                                       char *err, int32_t err_len) {
    API_TRY
    if (!partial_o_dev || !partial_ml_dev) throw std::runtime_error("null partial buffer");
    prefill_impl(a, layer, seq, n_tok, qkv_dev, qkv_dtype, nullptr, kDtypeF32, cudaStream_t(cuda_stream), partial_o_dev,
                 partial_ml_dev);
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_prefill_combine_dev(flint_attn *a, int32_t n_tok, int32_t n_parts, const float *partials_o_dev,
                                       const float *partials_ml_dev, void *out_dev, int32_t out_dtype, void *cuda_stream,
                                       char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    if (n_tok <= 0 || n_parts <= 0 || !partials_o_dev || !partials_ml_dev || !out_dev)
        throw std::runtime_error("bad combine shape");
    if (out_dtype != kDtypeF32 && out_dtype != kDtypeBf16) throw std::runtime_error("bad out dtype");
    CK(launch_prefill_combine(partials_o_dev, partials_ml_dev, n_parts, n_tok, out_dev, out_dtype, cudaStream_t(cuda_stream)));
    a->launches++;
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_prefill(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, const void *qkv,
                           int32_t qkv_dtype, void *out, int32_t out_dtype, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    if (n_tok <= 0) throw std::runtime_error("empty prefill");
    if ((qkv_dtype != kDtypeF32 && qkv_dtype != kDtypeBf16) || (out_dtype != kDtypeF32 && out_dtype != kDtypeBf16))
        throw std::runtime_error("bad dtype");
    const size_t in_bytes = size_t(n_tok) * kQkvDim * elem_size(qkv_dtype);
    const size_t in_pad = (in_bytes + 255) / 256 * 256;
    const size_t out_bytes = size_t(n_tok) * kQDim * elem_size(out_dtype);
    a->ensure_io(in_pad + out_bytes);
    char *d_in = static_cast<char *>(a->io_dev), *d_out = d_in + in_pad;
    CK(cudaMemcpyAsync(d_in, qkv, in_bytes, cudaMemcpyHostToDevice, a->stream));
    prefill_impl(a, layer, seq, n_tok, d_in, qkv_dtype, d_out, out_dtype, a->stream);
    CK(cudaMemcpyAsync(out, d_out, out_bytes, cudaMemcpyDeviceToHost, a->stream));
    CK(cudaStreamSynchronize(a->stream));
    int flag = 0;
    CK(prefill_error_flag(a->pf, &flag));
    if (flag) throw std::runtime_error("prefill kernel reported device error " + std::to_string(flag));
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_set_projections(flint_attn *a, int32_t layer, int32_t n_embd, const float *attn_norm,
                                   const uint16_t *wq, const uint16_t *wk, const uint16_t *wv, const uint16_t *wo,
                                   char *err, int32_t err_len) {
    API_TRY
    if (layer < 0 || layer >= int(a->layers.size())) throw std::runtime_error("layer index out of range");
    if (!attn_norm || !wq || !wk || !wv || !wo) throw std::runtime_error("null weight pointer");
    if (n_embd <= 0 || n_embd % 256 != 0) throw std::runtime_error("n_embd must be a positive multiple of 256");
    CK(cudaSetDevice(a->device));
    Layer &L = a->layers[layer];
    CK(cudaDeviceSynchronize());
    cudaFree(L.attn_norm); cudaFree(L.w_qkv); cudaFree(L.w_o);
    L.attn_norm = nullptr; L.w_qkv = nullptr; L.w_o = nullptr;
    const size_t E = size_t(n_embd);
    CK(cudaMalloc(&L.attn_norm, E * sizeof(float)));
    CK(cudaMalloc(&L.w_qkv, size_t(kQkvDim) * E * 2));
    CK(cudaMalloc(&L.w_o, E * kQDim * 2));
    CK(cudaMemcpy(L.attn_norm, attn_norm, E * sizeof(float), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.w_qkv, wq, size_t(kQDim) * E * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.w_qkv + size_t(kQDim) * E, wk, size_t(kKvDim) * E * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.w_qkv + size_t(kQDim + kKvDim) * E, wv, size_t(kKvDim) * E * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(L.w_o, wo, E * kQDim * 2, cudaMemcpyHostToDevice));
    L.n_embd = n_embd;
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_decode_block_dev(flint_attn *a, int32_t layer, int32_t n, const int32_t *seqs, float *x_dev,
                                    void *cuda_stream, char *err, int32_t err_len) {
    API_TRY
    attn_block(a, layer, n, seqs, 0, false, x_dev, cudaStream_t(cuda_stream));
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_prefill_block_dev(flint_attn *a, int32_t layer, int32_t seq, int32_t n_tok, float *x_dev,
                                     void *cuda_stream, char *err, int32_t err_len) {
    API_TRY
    attn_block(a, layer, n_tok, nullptr, seq, true, x_dev, cudaStream_t(cuda_stream));
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_project_dev(flint_attn *a, const uint16_t *w_dev, int32_t n_rows_w, int32_t k, const float *x_dev,
                               int32_t n, const float *norm_w_dev, float *out_dev, void *cuda_stream, char *err,
                               int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    if (!w_dev || !x_dev || !out_dev) throw std::runtime_error("null pointer");
    if (n <= 0 || n_rows_w <= 0 || n_rows_w % kProjRowBlock != 0 || k <= 0 || k % 256 != 0)
        throw std::runtime_error("projection shape: rows a multiple of 128, k a multiple of 256");
    ProjCall pc{};
    pc.w = reinterpret_cast<const __nv_bfloat16 *>(w_dev);
    pc.act = x_dev; pc.act_dtype = kDtypeF32; pc.norm_w = norm_w_dev;
    pc.out = out_dev; pc.out_dtype = kDtypeF32; pc.residual = nullptr;
    pc.B = n; pc.N = n_rows_w; pc.K = k;
    int n_launch = 0;
    CK(launch_proj(pc, a->proj_ws, a->sm_count, cudaStream_t(cuda_stream), &n_launch));
    a->launches += n_launch;
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_check(flint_attn *a, char *err, int32_t err_len) {
    API_TRY
    CK(cudaSetDevice(a->device));
    CK(cudaDeviceSynchronize());
    // Each device error word is reported once and cleared, the way the reference raises once per failed command
    // buffer (src/engine.mm:930-932): later, healthy launches on this handle are not failed by an old error.
    int flag = 0;
    CK(prefill_error_flag(a->pf, &flag));
    if (flag) throw std::runtime_error("prefill kernel reported device error " + std::to_string(flag));
    CK(cudaMemcpy(&flag, a->dec_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) {
        CK(cudaMemset(a->dec_err, 0, sizeof(int)));
        throw std::runtime_error("decode kernel reported device error " + std::to_string(flag));
    }
    if (a->xchg) {
        int *word = reinterpret_cast<int *>(a->xchg + kMaxPeers * sizeof(uint32_t));
        CK(cudaMemcpy(&flag, word, sizeof(int), cudaMemcpyDeviceToHost));
        if (flag) {
            CK(cudaMemset(word, 0, sizeof(int)));
            throw std::runtime_error("the wait for a peer's partial records ran out (exchange error " + std::to_string(flag) + ")");
        }
    }
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_n_slots(const flint_attn *a, int32_t layer) {
    if (layer < 0 || layer >= int(a->layers.size())) return -1;
    return a->layers[layer].n_slots;
}

static void kv_copy(flint_attn *a, int layer, int seq, int slot0, int n, uint16_t *k, uint16_t *v, bool to_host) {
    CK(cudaSetDevice(a->device));
    if (layer < 0 || layer >= int(a->layers.size())) throw std::runtime_error("layer index out of range");
    Layer &L = a->layers[layer];
    if (seq < 0 || seq >= a->max_seqs) throw std::runtime_error("sequence index out of range");
    if (slot0 < 0 || n < 0 || slot0 + n > L.n_slots) throw std::runtime_error("slot range out of bounds");
    CK(cudaDeviceSynchronize());
    if (L.paged) {  // block by block through the table; writing allocates the pages it needs
        if (!to_host && n > 0) {
            a->ensure_pages(seq, slot0 + n - 1, nullptr);
            CK(cudaDeviceSynchronize());
        }
        for (int s = slot0; s < slot0 + n;) {
            const int b = s / kPageKeys, in_page = s % kPageKeys, cnt = std::min(kPageKeys - in_page, slot0 + n - s);
            const int page = b < a->seq_blocks[seq] ? a->table_host[size_t(seq) * a->pages_per_seq + b] : -1;
            for (int kvh = 0; kvh < kNHeadKv; kvh++) {
                const size_t hoff = (size_t(kvh) * n + (s - slot0)) * kHeadDim, bytes = size_t(cnt) * kHeadDim * 2;
                if (page < 0) {  // reading slots that were never written: zeros, as in a fresh contiguous cache
                    memset(k + hoff, 0, bytes);
                    memset(v + hoff, 0, bytes);
                    continue;
                }
                const size_t doff = ((size_t(page) * kNHeadKv + kvh) * kPageKeys + in_page) * kHeadDim;
                if (to_host) {
                    CK(cudaMemcpy(k + hoff, L.k + doff, bytes, cudaMemcpyDeviceToHost));
                    CK(cudaMemcpy(v + hoff, L.v + doff, bytes, cudaMemcpyDeviceToHost));
                } else {
                    CK(cudaMemcpy(L.k + doff, k + hoff, bytes, cudaMemcpyHostToDevice));
                    CK(cudaMemcpy(L.v + doff, v + hoff, bytes, cudaMemcpyHostToDevice));
                }
            }
            s += cnt;
        }
        return;
    }
    for (int kvh = 0; kvh < kNHeadKv; kvh++) {
        const size_t doff = ((size_t(seq) * kNHeadKv + kvh) * L.n_slots + slot0) * kHeadDim;
        const size_t hoff = size_t(kvh) * n * kHeadDim, bytes = size_t(n) * kHeadDim * 2;
        if (to_host) {
            CK(cudaMemcpy(k + hoff, L.k + doff, bytes, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(v + hoff, L.v + doff, bytes, cudaMemcpyDeviceToHost));
        } else {
            CK(cudaMemcpy(L.k + doff, k + hoff, bytes, cudaMemcpyHostToDevice));
            CK(cudaMemcpy(L.v + doff, v + hoff, bytes, cudaMemcpyHostToDevice));
        }
    }
}

int32_t flint_attn_read_kv(flint_attn *a, int32_t layer, int32_t seq, int32_t slot0, int32_t n, uint16_t *k,
                           uint16_t *v, char *err, int32_t err_len) {
    API_TRY
    kv_copy(a, layer, seq, slot0, n, k, v, true);
    return 0;
    API_CATCH(-1)
}

int32_t flint_attn_write_kv(flint_attn *a, int32_t layer, int32_t seq, int32_t slot0, int32_t n, const uint16_t *k,
                            const uint16_t *v, char *err, int32_t err_len) {
    API_TRY
    kv_copy(a, layer, seq, slot0, n, const_cast<uint16_t *>(k), const_cast<uint16_t *>(v), false);
    return 0;
    API_CATCH(-1)
}

void *flint_attn_kv_dev(flint_attn *a, int32_t layer, int32_t which) {
    if (layer < 0 || layer >= int(a->layers.size())) return nullptr;
    return which == 0 ? static_cast<void *>(a->layers[layer].k) : static_cast<void *>(a->layers[layer].v);
}

int32_t flint_attn_seq_release(flint_attn *a, int32_t seq) {
    if (seq < 0 || seq >= a->max_seqs) return -1;
    a->pos[seq] = 0;
    if (a->kv_pages > 0) {
        int32_t *row = a->table_host.data() + size_t(seq) * a->pages_per_seq;
        for (int b = a->seq_blocks[seq] - 1; b >= 0; b--) {
            a->free_pages.push_back(row[b]);
            row[b] = -1;
        }
        a->seq_blocks[seq] = 0;
    }
    return 0;
}

int32_t flint_attn_pages_free(const flint_attn *a) { return a->kv_pages > 0 ? int32_t(a->free_pages.size()) : -1; }

int32_t flint_attn_plan_decode(int32_t n, const int32_t *pos, int32_t is_swa, int32_t kv_lo, int32_t kv_hi,
                               int32_t target_items, int32_t *out, int32_t cap) {
    static thread_local std::vector<DecItem> items;
    static thread_local PlanScratch scratch;
    int n_groups = 0, n_records = 0, n_subs = 0;
    plan_decode(n, nullptr, pos, is_swa != 0, kv_lo, kv_hi, target_items, items, n_groups, n_records, n_subs, scratch);
    if (int(items.size()) > cap) return -1;
    for (size_t i = 0; i < items.size(); i++) {
        const DecItem &it = items[i];
        const int32_t rec[8] = {it.tok, it.kvh, it.j0, it.j1, it.fold, it.split, it.n_split, it.part0};
        memcpy(out + 8 * i, rec, sizeof(rec));
    }
    return int32_t(items.size());
}

int32_t flint_attn_set_target_items(flint_attn *a, int32_t target_items) {
    if (target_items < 1) return -1;
    a->target_items = target_items;
    return 0;
}

int64_t flint_attn_launch_count(const flint_attn *a) { return a->launches; }

int32_t flint_attn_set_timing(flint_attn *a, int32_t on) {
    a->timing = on != 0;
    a->ev_used = 0;
    return 0;
}

double flint_attn_kernel_ms(flint_attn *a, int64_t *n_timed) {
    double total = 0;
    int64_t n = 0;
    cudaSetDevice(a->device);
    for (size_t i = 0; i + 1 < a->ev_used; i += 2) {
        float ms = 0;
        if (cudaEventSynchronize(a->ev_pool[i + 1]) != cudaSuccess) break;
        if (cudaEventElapsedTime(&ms, a->ev_pool[i], a->ev_pool[i + 1]) != cudaSuccess) break;
        total += ms;
        n++;
    }
    a->ev_used = 0;
    if (n_timed) *n_timed = n;
    return total;
}

}  // extern "C"
