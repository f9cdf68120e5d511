// Fused batch-1 attention for one layer: scores, softmax and value product in one kernel, one thread-block
// cluster per head. Replaces the reference's three launches per layer (mat_vec_strided_kernel,
// native/mat_vec_kernel.cu:51-81; softmax_kernel, native/softmax_kernel.cu:10-52; vec_mat_kernel,
// native/vec_mat_kernel.cu:8-48) and keeps their fp16 rounding points: a score is rounded to fp16 after the
// scale, a probability is rounded to fp16 after the division by the global sum, the output is rounded once.
//
// The sequence is split over the CTAs of a cluster; the per-head maximum, the exp-sum and the partial
// outputs are exchanged through distributed shared memory, so probabilities are normalised with the same
// global max and sum the unfused kernels see. Short sequences take a single-CTA path with no cluster traffic.
#pragma once

#include <cooperative_groups.h>

#include "common.cuh"

namespace ml2 {

namespace cg = cooperative_groups;

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnCluster = 8;
constexpr int kAttnSingleCtaMax = 128;  // sequences up to this length are handled by cluster rank 0 alone
constexpr int kHeadMax = 128;           // head size supported by the fused kernel (4 dims per lane)

struct AttnParams {
    __half* out;            // [n_heads * head_size]
    const __half* q;        // [n_heads * head_size]
    const __half* k;        // layer base: [seq][row_stride]
    const __half* v;
    const int* pos_ptr;     // device-resident position (graph replay); null -> pos_imm
    int pos_imm;
    int n_heads, head_size;
    int row_stride;         // elements between cache rows (kv_dim of this rank)
    float scale;
    int chunk_cap;          // capacity (positions) of the score buffer in dynamic shared memory
};

// scores of positions [t0, t1) of one head into s_sc (fp16-rounded, held as float); returns the CTA-wide max
__device__ __forceinline__ float attn_scores_chunk(const AttnParams& p, const __half* kh, const uint2 qv, int t0, int t1, float* s_sc,
                                                   float* s_tmp)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mx = -INFINITY;
    for (int t = t0 + warp; t < t1; t += kAttnWarps) {
        const uint2 kv = *reinterpret_cast<const uint2*>(kh + (size_t)t * p.row_stride + lane * 4);
        float s = 0.f;
        s = fma_f16_f32(lo16(kv.x), lo16(qv.x), s);
        s = fma_f16_f32(hi16(kv.x), hi16(qv.x), s);
        s = fma_f16_f32(lo16(kv.y), lo16(qv.y), s);
        s = fma_f16_f32(hi16(kv.y), hi16(qv.y), s);
        s = warp_sum(s);
        const float sr = __half2float(__float2half_rn(s * p.scale));  // native/mat_vec_kernel.cu:72-73
        if (lane == 0) s_sc[t - t0] = sr;
        mx = fmaxf(mx, sr);
    }
    if (lane == 0) s_tmp[warp] = mx;
    __syncthreads();
    float m = s_tmp[0];
#pragma unroll
    for (int w = 1; w < kAttnWarps; ++w) m = fmaxf(m, s_tmp[w]);
    __syncthreads();
    return m;
}

// exp(score - max) in place; returns the CTA-wide sum (fixed order)
__device__ __forceinline__ float attn_exp_chunk(float* s_sc, int n, float mx, float* s_tmp)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += kAttnThreads) {
        const float e = expf(s_sc[i] - mx);  // native/softmax_kernel.cu:37
        s_sc[i] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) s_tmp[warp] = sum;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) t += s_tmp[w];
    __syncthreads();
    return t;
}

// partial value product of the chunk: s_acc[w][d] per warp, summed in warp order into s_out[d]
__device__ __forceinline__ void attn_values_chunk(const AttnParams& p, const __half* vh, int t0, int t1, const float* s_sc, float total,
                                                  float (*s_acc)[kHeadMax], float* s_out)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = t0 + warp; t < t1; t += kAttnWarps) {
        // probability rounded to fp16 (native/softmax_kernel.cu:46), fed to the value product as fp16
        const unsigned short pr = __half_as_ushort(__float2half_rn(s_sc[t - t0] / total));
        const uint2 vv = *reinterpret_cast<const uint2*>(vh + (size_t)t * p.row_stride + lane * 4);
        acc[0] = fma_f16_f32(pr, lo16(vv.x), acc[0]);
        acc[1] = fma_f16_f32(pr, hi16(vv.x), acc[1]);
        acc[2] = fma_f16_f32(pr, lo16(vv.y), acc[2]);
        acc[3] = fma_f16_f32(pr, hi16(vv.y), acc[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) s_acc[warp][lane * 4 + e] = acc[e];
    __syncthreads();
    if (threadIdx.x < kHeadMax) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) s += s_acc[w][threadIdx.x];
        s_out[threadIdx.x] = s;
    }
    __syncthreads();
}

__global__ void __cluster_dims__(kAttnCluster, 1, 1) __launch_bounds__(kAttnThreads)
    fused_attention_kernel(const AttnParams p)
{
    extern __shared__ float s_sc[];                 // [chunk_cap]
    __shared__ float s_acc[kAttnWarps][kHeadMax];
    __shared__ float s_out[kHeadMax];               // this CTA's partial output (read by rank 0 through DSMEM)
    __shared__ float s_tmp[kAttnWarps];
    __shared__ float s_xchg[2];                     // [0] local max, [1] local sum (read by all ranks through DSMEM)

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int head = blockIdx.x / kAttnCluster;
    const int lane = threadIdx.x & 31;

    pdl_launch_dependents();
    pdl_wait();

    const int pos = p.pos_ptr ? *p.pos_ptr : p.pos_imm;
    const int n = pos + 1;
    const __half* kh = p.k + (size_t)head * p.head_size;
    const __half* vh = p.v + (size_t)head * p.head_size;
    const uint2 qv = *reinterpret_cast<const uint2*>(p.q + (size_t)head * p.head_size + lane * 4);

    if (n <= kAttnSingleCtaMax) {
        // ---- short sequence: rank 0 alone, no cluster traffic (uniform decision across the cluster) ----
        if (rank != 0) return;
        const float mx = attn_scores_chunk(p, kh, qv, 0, n, s_sc, s_tmp);
        const float total = attn_exp_chunk(s_sc, n, mx, s_tmp);
        attn_values_chunk(p, vh, 0, n, s_sc, total, s_acc, s_out);
        if (threadIdx.x < p.head_size) p.out[(size_t)head * p.head_size + threadIdx.x] = __float2half_rn(s_out[threadIdx.x]);
        return;
    }

    const int chunk = min(ceil_div(n, kAttnCluster), p.chunk_cap);
    const int t0 = min(rank * chunk, n), t1 = min(t0 + chunk, n);

    const float mx_local = attn_scores_chunk(p, kh, qv, t0, t1, s_sc, s_tmp);
    if (threadIdx.x == 0) s_xchg[0] = mx_local;
    cluster.sync();
    float mx = -INFINITY;
#pragma unroll
    for (int r = 0; r < kAttnCluster; ++r) mx = fmaxf(mx, *cluster.map_shared_rank(&s_xchg[0], r));

    const float sum_local = attn_exp_chunk(s_sc, t1 - t0, mx, s_tmp);
    if (threadIdx.x == 0) s_xchg[1] = sum_local;
    cluster.sync();
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < kAttnCluster; ++r) total += *cluster.map_shared_rank(&s_xchg[1], r);

    attn_values_chunk(p, vh, t0, t1, s_sc, total, s_acc, s_out);
    cluster.sync();
    if (rank == 0 && threadIdx.x < p.head_size) {
        float s = 0.f;
#pragma unroll
        for (int r = 0; r < kAttnCluster; ++r) s += *cluster.map_shared_rank(&s_out[threadIdx.x], r);
        p.out[(size_t)head * p.head_size + threadIdx.x] = __float2half_rn(s);  // native/vec_mat_kernel.cu:41
    }
    cluster.sync();  // remote shared memory stays alive until rank 0 has read it
}

}  // namespace ml2
