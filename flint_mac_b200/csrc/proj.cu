// Dense bf16 projections either side of attention for sm_100a: qkv = W_qkv . rmsnorm(x), x += W_o . att, and the
// logits of the last position.
//
// Replaces the reference's q/k/v matvecs with the attn_norm RMSNorm folded into the activation load and its o-proj
// matvec with the residual add folded into the store (src/engine.mm:728-732, :811; k_qkv src/metal/fused.metal:215-231,
// k_mv_res :357-379).  The reference multiplies quantised weight rows by one fp32 activation vector per thread group;
// here the weights are bf16 rows [N][K] streamed from HBM exactly once per launch and multiplied on the tensor cores
// against up to 64 activation rows at a time (decode batches; prefill goes through in 64-token chunks whose weights
// come from L2).  The kernel is bound by the weight stream: 2 bytes per weight against 2 * 64 flops.
//
// Activations reach the tensor core as a bf16 high part plus a bf16 low part (two products per weight fragment, fp32
// accumulate), which keeps 16 bits of their mantissa: the result differs from the reference's double-accumulated
// fp32 product (src/ref/ref_model.cpp:74-92) by the rounding of the fp32 accumulator only.
#include "proj.h"

#include <algorithm>

#include "attn_common.h"
#include "ptx.cuh"

namespace flint {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kSub = 128;              // k values per pipeline stage
constexpr int kActStride = kSub + 32;  // halves per activation row in shared memory: the 16-byte reads of a quarter
                                       // warp (4 k-offsets x 2 batch rows) then fall into distinct banks
constexpr int kStages = 2;
constexpr int kStepsPerSub = kSub / 32;  // one step = 32 k: every thread holds 16 bytes of each of its two weight rows
static_assert(kProjRowBlock == kWarps * 16, "one 16-row block of weights per warp");

struct PrepArgs {
    const void *act;
    const float *norm_w;
    __nv_bfloat16 *hi, *lo;  // [rows_padded][K]
    float *ssq;              // [rows_padded] sum of squares of the raw row
    int act_dtype, B, K;
};

// One CTA per activation row: v = x * norm_w (if any); hi = bf16(v), lo = bf16(v - hi); ssq = sum x^2.  Rows past B
// are written as zeros (they pad the batch to a multiple of 8 for the tensor-core tiles).
__global__ void __launch_bounds__(256) k_proj_prep(const PrepArgs a) {
    const int b = blockIdx.x, tid = threadIdx.x;
    __shared__ float red[8];
    float ss = 0.f;
    for (int k = tid * 4; k < a.K; k += 256 * 4) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < a.B) {
            if (a.act_dtype == kDtypeF32) {
                x = *reinterpret_cast<const float4 *>(static_cast<const float *>(a.act) + size_t(b) * a.K + k);
            } else {
                const uint2 u = *reinterpret_cast<const uint2 *>(static_cast<const __nv_bfloat16 *>(a.act) + size_t(b) * a.K + k);
                const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162 *>(&u.x);
                const __nv_bfloat162 q = *reinterpret_cast<const __nv_bfloat162 *>(&u.y);
                x = make_float4(__low2float(p), __high2float(p), __low2float(q), __high2float(q));
            }
        }
        ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        if (a.norm_w) {
            const float4 w = *reinterpret_cast<const float4 *>(a.norm_w + k);
            x.x *= w.x; x.y *= w.y; x.z *= w.z; x.w *= w.w;
        }
        const float v[4] = {x.x, x.y, x.z, x.w};
        __nv_bfloat16 h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            h[i] = __float2bfloat16_rn(v[i]);
            l[i] = __float2bfloat16_rn(v[i] - __bfloat162float(h[i]));
        }
        *reinterpret_cast<uint2 *>(a.hi + size_t(b) * a.K + k) = *reinterpret_cast<const uint2 *>(h);
        *reinterpret_cast<uint2 *>(a.lo + size_t(b) * a.K + k) = *reinterpret_cast<const uint2 *>(l);
    }
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float t = 0.f;
        for (int i = 0; i < 8; i++) t += red[i];  // fixed order: the result does not depend on scheduling
        a.ssq[b] = t;
    }
}

struct ProjArgs {
    const __nv_bfloat16 *w, *act_hi, *act_lo;
    const float *ssq;       // per activation row, or null when no RMSNorm is folded in
    float *partial;         // [n_split][rows_padded][N]
    int *tickets;           // [N / kProjRowBlock], zero between launches
    void *out;
    const float *residual;
    int out_dtype, B, N, K, k_per_cta, n_split;
};

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void *p) {  // read once: do not keep the line in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// CTA = 128 weight rows (16 per warp) x k_per_cta values of K, against NB * 8 activation rows.
// A dot product does not care in which order its terms are added, so the k index that a fragment position stands
// for is chosen freely: thread (g, t) of a warp takes 16 contiguous bytes (8 weights) of row g and of row g + 8 per
// 32-k step straight from global memory into registers -- no shared-memory staging of the weights -- and the
// activation fragments are read from shared memory with the same assignment (one 16-byte read per batch group).
template <int NB>
__global__ void __launch_bounds__(kThreads, 2) k_proj(const ProjArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16 *act_s = reinterpret_cast<__nv_bfloat16 *>(smem_raw);  // [kStages][2][NB * 8][kActStride]
    __shared__ int is_last;
    constexpr int kRows = NB * 8;
    constexpr int kStageHalves = 2 * kRows * kActStride;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * kProjRowBlock + warp * 16;
    const int k_begin = blockIdx.y * a.k_per_cta;
    const int n_sub = a.k_per_cta / kSub;
    const __nv_bfloat16 *wr0 = a.w + size_t(n0 + g) * a.K + k_begin + 8 * t;
    const __nv_bfloat16 *wr1 = wr0 + size_t(8) * a.K;

    float acc[NB][4];
#pragma unroll
    for (int j = 0; j < NB; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    auto load_act = [&](int s, int stage) {  // activation rows of sub-slice s -> shared memory (asynchronous)
        constexpr int kChunks = 2 * kRows * (kSub / 8);  // 16-byte pieces
        for (int c = tid; c < kChunks; c += kThreads) {
            const int part = c / (kRows * (kSub / 8)), rc = c % (kRows * (kSub / 8));
            const int row = rc / (kSub / 8), ch = rc % (kSub / 8);
            const __nv_bfloat16 *src = (part ? a.act_lo : a.act_hi) + size_t(row) * a.K + k_begin + s * kSub + ch * 8;
            cp_async16(smem_u32(act_s + stage * kStageHalves + (part * kRows + row) * kActStride + ch * 8), src, 16u);
        }
    };
    auto load_w = [&](int s, uint4 (&buf)[kStepsPerSub][2]) {
#pragma unroll
        for (int st = 0; st < kStepsPerSub; st++) {
            buf[st][0] = ld_stream16(wr0 + s * kSub + st * 32);
            buf[st][1] = ld_stream16(wr1 + s * kSub + st * 32);
        }
    };
    auto compute = [&](int stage, const uint4 (&buf)[kStepsPerSub][2]) {
        const __nv_bfloat16 *hi = act_s + stage * kStageHalves + g * kActStride + 8 * t;
        const __nv_bfloat16 *lo = hi + kRows * kActStride;
#pragma unroll
        for (int st = 0; st < kStepsPerSub; st++) {
            const uint4 v = buf[st][0], u = buf[st][1];
#pragma unroll
            for (int j = 0; j < NB; j++) {
                const uint4 bh = *reinterpret_cast<const uint4 *>(hi + j * 8 * kActStride + st * 32);
                const uint4 bl = *reinterpret_cast<const uint4 *>(lo + j * 8 * kActStride + st * 32);
                mma_bf16_16816(acc[j], v.x, u.x, v.y, u.y, bh.x, bh.y);
                mma_bf16_16816(acc[j], v.z, u.z, v.w, u.w, bh.z, bh.w);
                mma_bf16_16816(acc[j], v.x, u.x, v.y, u.y, bl.x, bl.y);
                mma_bf16_16816(acc[j], v.z, u.z, v.w, u.w, bl.z, bl.w);
            }
        }
    };

    // Two sub-slices in flight: the weights of the next one travel into registers and its activations into the
    // other shared-memory stage while the current one is multiplied.
    uint4 wa[kStepsPerSub][2], wb[kStepsPerSub][2];
    load_w(0, wa);
    load_act(0, 0);
    cp_async_commit();
    for (int s = 0; s < n_sub; s += 2) {
        if (s + 1 < n_sub) {
            load_w(s + 1, wb);
            load_act(s + 1, 1);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        compute(0, wa);
        __syncthreads();
        if (s + 2 < n_sub) {
            load_w(s + 2, wa);
            load_act(s + 2, 0);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (s + 1 < n_sub) compute(1, wb);
        __syncthreads();
    }
    cp_async_wait<0>();

    // accumulator layout: c0, c1 = (row g, batch 2t, 2t+1); c2, c3 = (row g + 8, same batch columns)
    auto finish = [&](int b, int n, float v) {
        if (b >= a.B) return;
        if (a.ssq) v *= rsqrtf(a.ssq[b] / float(a.K) + kRmsEps);  // the RMSNorm scale of the row (ref_model.cpp:45-50)
        const size_t idx = size_t(b) * a.N + n;
        if (a.residual) v += a.residual[idx];
        if (a.out_dtype == kDtypeF32) static_cast<float *>(a.out)[idx] = v;
        else static_cast<__nv_bfloat16 *>(a.out)[idx] = __float2bfloat16_rn(v);
    };
    if (a.n_split == 1) {
#pragma unroll
        for (int j = 0; j < NB; j++) {
            finish(8 * j + 2 * t, n0 + g, acc[j][0]);
            finish(8 * j + 2 * t + 1, n0 + g, acc[j][1]);
            finish(8 * j + 2 * t, n0 + g + 8, acc[j][2]);
            finish(8 * j + 2 * t + 1, n0 + g + 8, acc[j][3]);
        }
        return;
    }
    // Split over K: every CTA of a row block writes its partial sums; the last one to arrive adds them up in split
    // order (so the result does not depend on which CTA that is) and finishes the rows.
    float *mine = a.partial + size_t(blockIdx.y) * kRows * a.N;
#pragma unroll
    for (int j = 0; j < NB; j++) {
        mine[size_t(8 * j + 2 * t) * a.N + n0 + g] = acc[j][0];
        mine[size_t(8 * j + 2 * t + 1) * a.N + n0 + g] = acc[j][1];
        mine[size_t(8 * j + 2 * t) * a.N + n0 + g + 8] = acc[j][2];
        mine[size_t(8 * j + 2 * t + 1) * a.N + n0 + g + 8] = acc[j][3];
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const bool last = atomicAdd(&a.tickets[blockIdx.x], 1) == a.n_split - 1;
        if (last) {
            a.tickets[blockIdx.x] = 0;  // ready for the next launch
            __threadfence();
        }
        is_last = last;
    }
    __syncthreads();
    if (!is_last) return;
    const int nb0 = blockIdx.x * kProjRowBlock;
    for (int idx = tid; idx < a.B * kProjRowBlock; idx += kThreads) {
        const int b = idx / kProjRowBlock, n = nb0 + idx % kProjRowBlock;
        float v = 0.f;
        for (int s = 0; s < a.n_split; s++) v += __ldcg(a.partial + (size_t(s) * kRows + b) * a.N + n);
        finish(b, n, v);
    }
}

__global__ void __launch_bounds__(256) k_embed_rows(const __nv_bfloat16 *table, const int32_t *ids, int K, float *rows) {
    const int i = blockIdx.x;
    const __nv_bfloat16 *src = table + size_t(ids[i]) * K;
    for (int k = threadIdx.x * 2; k < K; k += 512) {
        const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162 *>(src + k);
        *reinterpret_cast<float2 *>(rows + size_t(i) * K + k) = make_float2(__low2float(p), __high2float(p));
    }
}

// One CTA: strided scan, then a tree in shared memory; ties go to the smaller index (the first maximum, as a
// sequential scan would find it).
__global__ void __launch_bounds__(1024) k_argmax(const float *x, int n, int32_t *result) {
    __shared__ float best_v[1024];
    __shared__ int best_i[1024];
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += 1024) {
        const float v = x[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    best_v[threadIdx.x] = bv;
    best_i[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 512; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = best_v[threadIdx.x + s];
            const int oi = best_i[threadIdx.x + s];
            if (ov > best_v[threadIdx.x] || (ov == best_v[threadIdx.x] && oi < best_i[threadIdx.x])) {
                best_v[threadIdx.x] = ov;
                best_i[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *result = best_i[0] == 0x7fffffff ? 0 : best_i[0];
}

template <int NB>
cudaError_t launch_one(const ProjArgs &a, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = size_t(kStages) * 2 * NB * 8 * kActStride * sizeof(__nv_bfloat16);
    static bool configured = false;  // per process; the attribute is per device, set again below if another device is current
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured || configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(k_proj<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        configured = true;
        configured_dev = dev;
    }
    k_proj<NB><<<grid, kThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

void proj_workspace_free(ProjWorkspace &ws) {
    cudaFree(ws.act_hi);
    cudaFree(ws.act_lo);
    cudaFree(ws.partial);
    cudaFree(ws.tickets);
    ws = ProjWorkspace{};
}

cudaError_t launch_proj(const ProjCall &c, ProjWorkspace &ws, int sm_count, cudaStream_t stream, int *n_launches) {
    *n_launches = 0;
    if (c.B <= 0) return cudaSuccess;
    if (c.N % kProjRowBlock != 0 || c.K % 256 != 0 || c.K <= 0 || c.N <= 0) return cudaErrorInvalidValue;
    cudaError_t e;
    // ---- scratch (grows; never shrinks)
    if (size_t(c.K) > ws.k_cap) {
        if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
        cudaFree(ws.act_hi);
        cudaFree(ws.act_lo);
        ws.act_hi = ws.act_lo = nullptr;
        ws.k_cap = 0;
        // act_hi, act_lo and the per-row sums of squares (behind act_lo)
        if ((e = cudaMalloc(&ws.act_hi, size_t(kProjMaxBatch) * c.K * 2)) != cudaSuccess) return e;
        if ((e = cudaMalloc(&ws.act_lo, size_t(kProjMaxBatch) * c.K * 2 + kProjMaxBatch * sizeof(float))) != cudaSuccess) return e;
        ws.k_cap = size_t(c.K);
    }
    const int n_rb = c.N / kProjRowBlock;
    if (size_t(n_rb) > ws.n_tickets) {
        if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
        cudaFree(ws.tickets);
        ws.tickets = nullptr;
        ws.n_tickets = 0;
        const size_t nt = std::max<size_t>(size_t(n_rb) * 2, 256);
        if ((e = cudaMalloc(&ws.tickets, nt * sizeof(int))) != cudaSuccess) return e;
        if ((e = cudaMemset(ws.tickets, 0, nt * sizeof(int))) != cudaSuccess) return e;
        ws.n_tickets = nt;
    }
    float *ssq = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(ws.act_lo) + ws.k_cap * kProjMaxBatch * 2);

    for (int b0 = 0; b0 < c.B; b0 += kProjMaxBatch) {
        const int bc = std::min(kProjMaxBatch, c.B - b0);
        const int nb = bc <= 8 ? 1 : bc <= 16 ? 2 : bc <= 32 ? 4 : 8;
        // Split over K so that the SMs carry equal loads: with s slices there are n_rb * s CTAs, the busiest SM runs
        // ceil(n_rb * s / SMs) of them one after the other in effect (co-resident CTAs share the tensor pipe), each K / s
        // long.  Slices of at least 256 k; a full batch keeps 512 so that the activation rows each CTA pulls from L2
        // stay comparable to its weight bytes.
        const int min_slice = nb == 8 ? 512 : 256;
        int n_split = 1;
        long long best = (long long)((n_rb + sm_count - 1) / sm_count) * c.K;
        for (int s = 2; c.K / s >= min_slice && c.K % (s * kSub) == 0; s *= 2) {
            const long long cost = (long long)((n_rb * s + sm_count - 1) / sm_count) * (c.K / s);
            if (cost < best) {
                best = cost;
                n_split = s;
            }
        }
        const size_t need = n_split > 1 ? size_t(n_split) * nb * 8 * c.N : 0;
        if (need > ws.partial_floats) {
            if ((e = cudaDeviceSynchronize()) != cudaSuccess) return e;
            cudaFree(ws.partial);
            ws.partial = nullptr;
            ws.partial_floats = 0;
            if ((e = cudaMalloc(&ws.partial, need * sizeof(float))) != cudaSuccess) return e;
            ws.partial_floats = need;
        }
        const size_t esz = c.act_dtype == kDtypeF32 ? 4 : 2, osz = c.out_dtype == kDtypeF32 ? 4 : 2;
        PrepArgs pa{};
        pa.act = static_cast<const unsigned char *>(c.act) + size_t(b0) * c.K * esz;
        pa.norm_w = c.norm_w;
        pa.hi = ws.act_hi; pa.lo = ws.act_lo; pa.ssq = ssq;
        pa.act_dtype = c.act_dtype; pa.B = bc; pa.K = c.K;
        k_proj_prep<<<nb * 8, 256, 0, stream>>>(pa);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        ProjArgs a{};
        a.w = c.w; a.act_hi = ws.act_hi; a.act_lo = ws.act_lo;
        a.ssq = c.norm_w ? ssq : nullptr;
        a.partial = ws.partial; a.tickets = ws.tickets;
        a.out = static_cast<unsigned char *>(c.out) + size_t(b0) * c.N * osz;
        a.residual = c.residual ? c.residual + size_t(b0) * c.N : nullptr;
        a.out_dtype = c.out_dtype; a.B = bc; a.N = c.N; a.K = c.K;
        a.k_per_cta = c.K / n_split; a.n_split = n_split;
        const dim3 grid(n_rb, n_split);
        e = nb == 1 ? launch_one<1>(a, grid, stream) : nb == 2 ? launch_one<2>(a, grid, stream)
          : nb == 4 ? launch_one<4>(a, grid, stream) : launch_one<8>(a, grid, stream);
        if (e != cudaSuccess) return e;
        *n_launches += 2;
    }
    return cudaSuccess;
}

cudaError_t launch_embed_rows(const __nv_bfloat16 *table, const int32_t *ids_dev, int n, int K, float *rows,
                              cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    k_embed_rows<<<n, 256, 0, stream>>>(table, ids_dev, K, rows);
    return cudaGetLastError();
}

cudaError_t launch_argmax(const float *x, int n, int32_t *result_dev, cudaStream_t stream) {
    k_argmax<<<1, 1024, 0, stream>>>(x, n, result_dev);
    return cudaGetLastError();
}

}  // namespace flint
