// The sampling chain that follows the decode path (Sampler.Sample, src/Sampler.cs:40-70 of GilesBathgate/ManagedLlama2):
// temperature softmax over the logits, descending sort of the probabilities with their token ids, inclusive sum, and
// the first entry whose cumulative probability reaches the threshold. One CTA per step, like the reference's four
// kernels (native/softmax_logits_kernel.cu, sort_kernel.cu, cumulative_sum_kernel.cu, sample_top_p_kernel.cu); the
// work is a few tens of kilobytes, so it is latency that counts, not bandwidth. Rounding points are the reference's.
#include <cuda_fp16.h>

#include "../../include/ml2b200.h"
#include "host_common.hpp"

namespace ml2 {

constexpr int kSampThreads = 1024;
constexpr int kSortMax = 32768;   // composite 32-bit sort keys of the whole array live in shared memory

__device__ __forceinline__ float samp_block_sum(float v, float* s)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) s[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (int)(blockDim.x >> 5) ? s[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) s[32] = t;
    }
    __syncthreads();
    return s[32];
}
__device__ __forceinline__ float samp_block_max(float v, float* s)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) s[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (int)(blockDim.x >> 5) ? s[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) s[32] = t;
    }
    __syncthreads();
    return s[32];
}

// native/softmax_logits_kernel.cu:10-54. indices[t] = t; logits /= temperature (rounded to fp16); softmax with the
// fp16 roundings of the reference: exp values are stored as fp16, summed unrounded, and the stored fp16 values are
// divided by the sum.
__global__ void __launch_bounds__(kSampThreads) softmax_logits_kernel(__half* logits, int size, float temperature, int* indices)
{
    __shared__ float s_buf[33];
    float mx = -INFINITY;
    for (int t = threadIdx.x; t < size; t += blockDim.x) {
        indices[t] = t;
        const __half h = __float2half_rn(__half2float(logits[t]) / temperature);
        logits[t] = h;
        mx = fmaxf(mx, __half2float(h));
    }
    mx = samp_block_max(mx, s_buf);
    float sum = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = expf(__half2float(logits[i]) - mx);
        logits[i] = __float2half_rn(v);
        sum += v;
    }
    sum = samp_block_sum(sum, s_buf);
    for (int t = threadIdx.x; t < size; t += blockDim.x) logits[t] = __float2half_rn(__half2float(logits[t]) / sum);
}

// fp16 bits -> 16-bit code whose unsigned order is the numeric order (-0 below +0), and back
__device__ __forceinline__ uint32_t half_order_code(unsigned short b) { return (b & 0x8000u) ? (uint32_t)(unsigned short)~b : (uint32_t)(b | 0x8000u); }
__device__ __forceinline__ unsigned short half_from_code(uint32_t c) { return (c & 0x8000u) ? (unsigned short)(c & 0x7fffu) : (unsigned short)~c; }

// native/sort_kernel.cu:13-45: keys descending, values carried, equal keys keep their order (the reference's block
// radix sort is stable). Each element becomes one 32-bit word (order code of the key, then 65535 - position), the
// words are sorted by a bitonic network in shared memory, keys and values are rebuilt from the sorted words.
__global__ void __launch_bounds__(kSampThreads) sort_desc_kernel(__half* keys, int* values, int size, int n2)
{
    extern __shared__ uint32_t s_w[];
    const int tid = threadIdx.x, nt = blockDim.x;
    for (int i = tid; i < n2; i += nt)
        s_w[i] = i < size ? ((half_order_code(__half_as_ushort(keys[i])) << 16) | (uint32_t)(65535 - i)) : 0u;   // padding sorts last
    __syncthreads();
    for (int k = 2; k <= n2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = tid; t < (n2 >> 1); t += nt) {
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int l = i | j;
                const uint32_t a = s_w[i], b = s_w[l];
                const bool desc = (i & k) == 0;
                if ((a < b) == desc) { s_w[i] = b; s_w[l] = a; }
            }
            __syncthreads();
        }
    }
    // values are permuted in place: fetch all of them before any is written
    int mine[kSortMax / kSampThreads];
#pragma unroll
    for (int q = 0; q < kSortMax / kSampThreads; ++q) {
        const int r = tid + q * nt;
        mine[q] = r < size ? values[65535 - (int)(s_w[r] & 0xffffu)] : 0;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kSortMax / kSampThreads; ++q) {
        const int r = tid + q * nt;
        if (r < size) {
            values[r] = mine[q];
            keys[r] = __ushort_as_half(half_from_code(s_w[r] >> 16));
        }
    }
}

// native/cumulative_sum_kernel.cu:9-28: inclusive sum in fp32 over fp16 values, each output rounded to fp16.
// A thread owns a run of consecutive items; its running sum starts from the total of the runs before it.
__global__ void __launch_bounds__(kSampThreads) cumulative_sum_kernel(__half* values, int size)
{
    __shared__ float s_warp[33];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ipt = (size + (int)blockDim.x - 1) / (int)blockDim.x;
    const int i0 = tid * ipt, i1 = min(size, i0 + ipt);
    float local = 0.f;
    for (int i = i0; i < i1; ++i) local += __half2float(values[i]);
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = lane < (int)(blockDim.x >> 5) ? s_warp[lane] : 0.f;
        float wi = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += t;
        }
        s_warp[lane] = wi - w;   // exclusive prefix of the warp totals
    }
    __syncthreads();
    float run = s_warp[warp] + (incl - local);
    for (int i = i0; i < i1; ++i) {
        run += __half2float(values[i]);
        values[i] = __float2half_rn(run);
    }
}

// native/sample_top_p_kernel.cu:9-24: the first position whose value reaches the threshold (the last one if none does).
__global__ void __launch_bounds__(kSampThreads) sample_top_p_kernel(const __half* values, const int* indices, int size, float threshold,
                                                                   int* result, int pos)
{
    __shared__ int s_min[32];
    int mn = size - 1;
    for (int t = threadIdx.x; t < size; t += blockDim.x)
        if (__half2float(values[t]) >= threshold && t < mn) mn = t;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    if ((threadIdx.x & 31) == 0) s_min[threadIdx.x >> 5] = mn;
    __syncthreads();
    if (threadIdx.x < 32) {
        mn = threadIdx.x < (int)(blockDim.x >> 5) ? s_min[threadIdx.x] : size - 1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        if (threadIdx.x == 0) result[pos] = indices[mn];
    }
}

static int next_pow2(int v)
{
    int n = 2;
    while (n < v) n <<= 1;
    return n;
}

int sampler_softmax_logits(cudaStream_t st, void* logits, int size, float temperature, int* indices)
{
    softmax_logits_kernel<<<1, kSampThreads, 0, st>>>(static_cast<__half*>(logits), size, temperature, indices);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ML2_OK : fail(ML2_E_CUDA, "softmax_logits: %s", cudaGetErrorString(e));
}
int sampler_sort(cudaStream_t st, int device, void* keys, int* values, int size)
{
    const int n2 = next_pow2(size);
    static bool attr_set[64] = {};
    if (device >= 0 && device < 64 && !attr_set[device]) {
        const cudaError_t e = cudaFuncSetAttribute(sort_desc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSortMax * 4);
        if (e != cudaSuccess) return fail(ML2_E_CUDA, "sort: %s", cudaGetErrorString(e));
        attr_set[device] = true;
    }
    sort_desc_kernel<<<1, kSampThreads, (size_t)n2 * 4, st>>>(static_cast<__half*>(keys), values, size, n2);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ML2_OK : fail(ML2_E_CUDA, "sort: %s", cudaGetErrorString(e));
}
int sampler_cumulative_sum(cudaStream_t st, void* values, int size)
{
    cumulative_sum_kernel<<<1, kSampThreads, 0, st>>>(static_cast<__half*>(values), size);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ML2_OK : fail(ML2_E_CUDA, "cumulative_sum: %s", cudaGetErrorString(e));
}
int sampler_sample_top_p(cudaStream_t st, const void* values, const int* indices, int size, float threshold, int* tokens, int pos)
{
    sample_top_p_kernel<<<1, kSampThreads, 0, st>>>(static_cast<const __half*>(values), indices, size, threshold, tokens, pos);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ML2_OK : fail(ML2_E_CUDA, "sample_top_p: %s", cudaGetErrorString(e));
}

// Sampler.Sample for temperature != 0 (src/Sampler.cs:49-66): logits are consumed in place.
int sampler_chain(cudaStream_t st, int device, void* logits, int* indices, int size, float temperature, float top_p, float coin, int* tokens,
                  int next_pos)
{
    int rc = sampler_softmax_logits(st, logits, size, temperature, indices);
    float threshold = coin;
    if (rc == ML2_OK && !(top_p <= 0.f || top_p >= 1.f)) {
        rc = sampler_sort(st, device, logits, indices, size);
        threshold = coin * top_p;
    }
    if (rc == ML2_OK) rc = sampler_cumulative_sum(st, logits, size);
    if (rc == ML2_OK) rc = sampler_sample_top_p(st, logits, indices, size, threshold, tokens, next_pos);
    return rc;
}

}  // namespace ml2

using namespace ml2;

extern "C" {

int ml2_softmax_logits(ml2_ctx* h, void* logits, int size, float temperature, int* indices)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !logits || !indices) return fail(ML2_E_INVALID, "softmax_logits: null argument");
    if (size <= 0 || !(temperature > 0.f)) return fail(ML2_E_INVALID, "softmax_logits: size=%d temperature=%g", size, (double)temperature);
    cudaSetDevice(ctx->device);
    const int rc = sampler_softmax_logits(ctx->stream, logits, size, temperature, indices);
    if (rc == ML2_OK) ++ctx->launches;
    return rc;
}

int ml2_sort(ml2_ctx* h, void* keys, int* values, int size)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !keys || !values) return fail(ML2_E_INVALID, "sort: null argument");
    if (size <= 0 || size > kSortMax) return fail(ML2_E_INVALID, "sort: size=%d (1..%d supported)", size, kSortMax);
    cudaSetDevice(ctx->device);
    const int rc = sampler_sort(ctx->stream, ctx->device, keys, values, size);
    if (rc == ML2_OK) ++ctx->launches;
    return rc;
}

int ml2_cumulative_sum(ml2_ctx* h, void* values, int size)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !values) return fail(ML2_E_INVALID, "cumulative_sum: null argument");
    if (size <= 0) return fail(ML2_E_INVALID, "cumulative_sum: size=%d", size);
    cudaSetDevice(ctx->device);
    const int rc = sampler_cumulative_sum(ctx->stream, values, size);
    if (rc == ML2_OK) ++ctx->launches;
    return rc;
}

int ml2_sample_top_p(ml2_ctx* h, const void* values, const int* indices, int size, float threshold, int* tokens, int pos)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !values || !indices || !tokens) return fail(ML2_E_INVALID, "sample_top_p: null argument");
    if (size <= 0 || pos < 0) return fail(ML2_E_INVALID, "sample_top_p: size=%d pos=%d", size, pos);
    cudaSetDevice(ctx->device);
    const int rc = sampler_sample_top_p(ctx->stream, values, indices, size, threshold, tokens, pos);
    if (rc == ML2_OK) ++ctx->launches;
    return rc;
}

}  // extern "C"
