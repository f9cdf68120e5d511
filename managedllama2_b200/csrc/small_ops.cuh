// The small operators of the decode path as stand-alone kernels (operator-level C ABI), plus the
// synthetic-tensor generators. Arithmetic and fp16 rounding points follow the reference kernels
// cited per function (native/*.cu of GilesBathgate/ManagedLlama2); launch shapes do not.
#pragma once

#include "common.cuh"

namespace ml2 {

// ---- block reductions (warp shuffles + one shared-memory hop, fixed order) ---------------------
__device__ __forceinline__ float block_sum(float v, float* s_buf /* >= 33 floats */)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) s_buf[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? s_buf[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) s_buf[32] = t;
    }
    __syncthreads();
    return s_buf[32];
}
__device__ __forceinline__ float block_max(float v, float* s_buf)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) s_buf[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? s_buf[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) s_buf[32] = t;
    }
    __syncthreads();
    return s_buf[32];
}

// ---- RMSNorm (native/rmsnorm_kernel.cu:8-42): fp32 squares, rms = 1/sqrtf(ss/n + eps),
// out = half(rms * gamma * x), one block. out may alias in.
static __global__ void __launch_bounds__(1024) rmsnorm_kernel(__half* out, const __half* in, const __half* gamma, int size, float eps)
{
    __shared__ float s_buf[33];
    pdl_wait();
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = __half2float(in[i]);
        ss += v * v;
    }
    ss = block_sum(ss, s_buf);
    const float rms = 1.0f / sqrtf(ss / (float)size + eps);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float norm = rms * __half2float(gamma[i]) * __half2float(in[i]);
        out[i] = __float2half_rn(norm);
    }
}

// ---- RoPE (native/rope_kernel.cu:3-31): rotate-half pairs (t, t + hs/2) in every head; q always,
// k for heads below n_kv_heads; angle = pos / theta^(2t/hs) with powf/cosf/sinf.
static __global__ void rope_kernel(__half* q, __half* k, int n_heads, int n_kv_heads, int head_size, int pos, float theta)
{
    pdl_wait();
    const int half_hs = head_size >> 1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_heads * half_hs) return;
    const int h = idx / half_hs, t = idx - h * half_hs;
    const int i = h * head_size + t, j = i + half_hs;
    const int head_dim = (t * 2) % head_size;
    const float freq = 1.0f / powf(theta, (float)head_dim / (float)head_size);
    const float val = (float)pos * freq;
    const float fcr = cosf(val), fci = sinf(val);
    const float q0 = __half2float(q[i]), q1 = __half2float(q[j]);
    q[i] = __float2half_rn(q0 * fcr - q1 * fci);
    q[j] = __float2half_rn(q0 * fci + q1 * fcr);
    if (h >= n_kv_heads) return;
    const float k0 = __half2float(k[i]), k1 = __half2float(k[j]);
    k[i] = __float2half_rn(k0 * fcr - k1 * fci);
    k[j] = __float2half_rn(k0 * fci + k1 * fcr);
}

// (cos, sin) table for the fused QKV epilogue: same expressions as rope_kernel, one entry per
// (position, pair index).
static __global__ void rope_table_kernel(float2* table, int seq_len, int head_size, float theta)
{
    const int half_hs = head_size >> 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)seq_len * half_hs) return;
    const int pos = (int)(idx / half_hs), t = (int)(idx - (long long)pos * half_hs);
    const int head_dim = (t * 2) % head_size;
    const float freq = 1.0f / powf(theta, (float)head_dim / (float)head_size);
    const float val = (float)pos * freq;
    table[idx] = make_float2(cosf(val), sinf(val));
}

// ---- embedding gather (native/embedding_kernel.cu:3-17)
static __global__ void embedding_kernel(__half* out, const __half* table, int size, const int* tokens, int pos)
{
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= size) return;
    const int token = tokens[pos];
    out[i] = table[(size_t)token * size + i];
}

// ---- argmax (native/argmax_kernel.cu:8-46), lowest index wins ties
static __global__ void __launch_bounds__(1024) argmax_kernel(const __half* in, int size, int* result, int pos, int write_token)
{
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_wait();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = __half2float(in[i]);
        if (v > best) {  // strided ascending: the first maximum of this thread's subsequence is kept
            best = v;
            best_i = i;
        }
    }
    auto better = [](float a, int ai, float b, int bi) { return a > b || (a == b && ai < bi); };
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nw ? s_val[lane] : -INFINITY;
        best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0 && write_token) result[pos] = (best_i == 0x7fffffff) ? 0 : best_i;
    }
}

// ---- attention scores (mat_vec_strided_kernel, native/mat_vec_kernel.cu:51-81):
// att[h*seq + t] = half(scale * sum_d q[h*hs+d] * K[t*dim + h*hs + d]); one warp per (t, h),
// 8-byte loads, grid sized by the live sequence length.
static __global__ void __launch_bounds__(256) attn_scores_kernel(__half* att, const __half* q, const __half* k, int head_size, int dim,
                                                          int seq, float scale)
{
    pdl_wait();
    const int h = blockIdx.y;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= seq) return;
    const int lane = threadIdx.x & 31;
    const __half* kr = k + (size_t)t * dim + (size_t)h * head_size;
    const __half* qr = q + (size_t)h * head_size;
    float sum = 0.f;
    for (int d = lane * 4; d < head_size; d += 128) {
        if (d + 4 <= head_size) {
            const uint2 kv = *reinterpret_cast<const uint2*>(kr + d);
            const uint2 qv = *reinterpret_cast<const uint2*>(qr + d);
            sum = fma_f16_f32(lo16(kv.x), lo16(qv.x), sum);
            sum = fma_f16_f32(hi16(kv.x), hi16(qv.x), sum);
            sum = fma_f16_f32(lo16(kv.y), lo16(qv.y), sum);
            sum = fma_f16_f32(hi16(kv.y), hi16(qv.y), sum);
        } else {
            for (int e = d; e < head_size; ++e) sum += __half2float(kr[e]) * __half2float(qr[e]);
        }
    }
    sum = warp_sum(sum);
    if (lane == 0) att[(size_t)h * seq + t] = __float2half_rn(sum * scale);
}

// ---- softmax (native/softmax_kernel.cu:10-52): per head over `size` fp16 scores, fp32 math,
// in place. Three passes over L2-resident scores instead of a fixed shared-memory array.
static __global__ void __launch_bounds__(1024) softmax_kernel(__half* att, int size)
{
    __shared__ float s_buf[33];
    pdl_wait();
    __half* a = att + (size_t)blockIdx.x * size;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < size; i += blockDim.x) m = fmaxf(m, __half2float(a[i]));
    m = block_max(m, s_buf);
    float sum = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) sum += expf(__half2float(a[i]) - m);
    sum = block_sum(sum, s_buf);
    for (int i = threadIdx.x; i < size; i += blockDim.x) a[i] = __float2half_rn(expf(__half2float(a[i]) - m) / sum);
}

// ---- attention values (vec_mat_kernel, native/vec_mat_kernel.cu:8-48):
// out[h*hs + d] = half(sum_t att[h*seq+t] * V[t*dim + h*hs + d]). Block per (head, 128-wide d slab):
// warp w sweeps t = w, w+nw, ...; lane owns 4 consecutive d (8-byte loads); warps are summed in order.
static __global__ void __launch_bounds__(1024) attn_values_kernel(__half* out, const __half* att, const __half* v, int head_size, int dim,
                                                           int seq)
{
    __shared__ float s_acc[32][128 + 4];
    pdl_wait();
    const int h = blockIdx.y;
    const int d0 = blockIdx.x * 128 + (threadIdx.x & 31) * 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (d0 < head_size) {
        const __half* vb = v + (size_t)h * head_size + d0;
        const __half* ar = att + (size_t)h * seq;
        for (int t = warp; t < seq; t += nw) {
            const unsigned short a = __half_as_ushort(ar[t]);
            if (d0 + 4 <= head_size) {
                const uint2 vv = *reinterpret_cast<const uint2*>(vb + (size_t)t * dim);
                acc[0] = fma_f16_f32(a, lo16(vv.x), acc[0]);
                acc[1] = fma_f16_f32(a, hi16(vv.x), acc[1]);
                acc[2] = fma_f16_f32(a, lo16(vv.y), acc[2]);
                acc[3] = fma_f16_f32(a, hi16(vv.y), acc[3]);
            } else {
                for (int e = 0; e < 4 && d0 + e < head_size; ++e)
                    acc[e] += __half2float(ar[t]) * __half2float(vb[(size_t)t * dim + e]);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) s_acc[warp][lane * 4 + e] = acc[e];
    __syncthreads();
    const int d = blockIdx.x * 128 + threadIdx.x;
    if (threadIdx.x < 128 && d < head_size) {
        float s = 0.f;
        for (int w = 0; w < nw; ++w) s += s_acc[w][threadIdx.x];
        out[(size_t)h * head_size + d] = __float2half_rn(s);
    }
}

// ---- dequantise to fp16, HostQWeight.Unpack (src/QWeight.cs:29-54) per output row
static __global__ void dequant_int4_kernel(__half* out, const uint32_t* w, const uint32_t* z, const __half* s, int rows, int cols,
                                    int wsize, int zsize, int ssize)
{
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one packed word each
    const long long total = (long long)cols * (rows / 8 + ((rows & 7) ? 1 : 0));
    const int wpr = ceil_div(rows, 8);
    if (idx >= total) return;
    const int c = (int)(idx / wpr), j = (int)(idx - (long long)c * wpr);
    const uint32_t word = w[(size_t)c * wsize + j];
    const int g = (j * 8) / kGroup;
    const int zero = (int)((z[(size_t)c * zsize + (g >> 3)] >> ((g & 7) * 4)) & 0xFu);
    const float scale = __half2float(s[(size_t)c * ssize + g]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int k = j * 8 + i;
        if (k < rows) {
            const int element = (int)((word >> (i * 4)) & 0xFu);
            out[(size_t)c * rows + k] = __float2half_rn((float)(element - zero) * scale);
        }
    }
}

// ---- counter-based synthetic tensors (bit-identical host/device) ---------------------------------
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__host__ __device__ __forceinline__ uint64_t synth_key(uint64_t seed, uint32_t tensor_id, uint32_t kind)
{
    return mix64(seed ^ mix64(((uint64_t)tensor_id << 8) | kind));
}
__host__ __device__ __forceinline__ uint64_t synth_at(uint64_t key, uint64_t index) { return mix64(key ^ (index * 0xD1B54A32D192ED03ull)); }

// nibbles of logical word (col, j): 8 nibbles = one half of a 64-bit draw
__host__ __device__ __forceinline__ uint32_t synth_weight_word(uint64_t key, int rows_full, int col, int j)
{
    const uint64_t widx = (uint64_t)col * (uint64_t)(rows_full / 8) + (uint64_t)j;
    const uint64_t h = synth_at(key, widx >> 1);
    return (uint32_t)((widx & 1) ? (h >> 32) : h);
}
__host__ __device__ __forceinline__ uint32_t synth_zero(uint64_t key, int groups_full, int col, int g)
{
    return (uint32_t)(synth_at(key, (uint64_t)col * groups_full + g) >> 60);
}
__host__ __device__ __forceinline__ float synth_scale_f32(uint64_t key, int groups_full, int col, int g)
{
    const uint32_t u24 = (uint32_t)(synth_at(key, (uint64_t)col * groups_full + g) >> 40);
    const float u = (float)u24 * (1.0f / 16777216.0f);
    return fmaf(u, 0.019f, 0.001f);
}
// Irwin-Hall(8) of 16-bit fields: integer sum, one fp32 multiply
__host__ __device__ __forceinline__ float synth_normal_f32(uint64_t key, uint64_t index, float sigma)
{
    const uint64_t a = synth_at(key, 2 * index), b = synth_at(key, 2 * index + 1);
    int s = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s += (int)((a >> (16 * i)) & 0xFFFFu);
        s += (int)((b >> (16 * i)) & 0xFFFFu);
    }
    return (float)(s - 262140) * (sigma * (1.0f / 53509.94f));
}

static __global__ void synth_qweight_kernel(uint32_t* weight, uint32_t* zeros, __half* scales, int rows_full, int col0, int ncols, int g0,
                                     int ngroups, uint64_t kw, uint64_t kz, uint64_t ks)
{
    const int rows = min(ngroups * kGroup, rows_full - g0 * kGroup);
    const int wsize = ceil_div(rows, 32) * 4, ssize = ceil_div(rows, kGroup), zsize = ceil_div(ssize, 8);
    const int groups_full = ceil_div(rows_full, kGroup);
    const long long nW = (long long)ncols * wsize, nZ = (long long)ncols * zsize, nS = (long long)ncols * ssize;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nW + nZ + nS; i += (long long)gridDim.x * blockDim.x) {
        if (i < nW) {
            const int c = (int)(i / wsize), j = (int)(i - (long long)c * wsize);
            const int jf = g0 * (kGroup / 8) + j;
            weight[i] = (jf * 8 < rows_full && j * 8 < rows) ? synth_weight_word(kw, rows_full, col0 + c, jf) : 0u;
        } else if (i < nW + nZ) {
            const long long k = i - nW;
            const int c = (int)(k / zsize), zw = (int)(k - (long long)c * zsize);
            uint32_t word = 0;
            for (int n = 0; n < 8; ++n) {
                const int g = zw * 8 + n;
                if (g < ssize) word |= synth_zero(kz, groups_full, col0 + c, g0 + g) << (4 * n);
            }
            zeros[k] = word;
        } else {
            const long long k = i - nW - nZ;
            const int c = (int)(k / ssize), g = (int)(k - (long long)c * ssize);
            scales[k] = __float2half_rn(synth_scale_f32(ks, groups_full, col0 + c, g0 + g));
        }
    }
}

static __global__ void synth_normal_kernel(__half* out, long long row0, long long nrows, int width, float sigma, uint64_t key)
{
    const long long n = nrows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = __float2half_rn(synth_normal_f32(key, (uint64_t)(row0 * width + i), sigma));
}

}  // namespace ml2
