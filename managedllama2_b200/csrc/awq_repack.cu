// AWQ checkpoint tensors -> QWeight layout: the repacking of ModelConverter (src/ModelConverter.cs:196-328 of
// GilesBathgate/ManagedLlama2) on the device. Byte and nibble shuffling, bound by HBM; one pass, every byte read and
// written once.
//
//   format v0 (AutoAWQ GEMM tensors): qweight int32 [in][out / 8], qzeros int32 [groups][out / 8], scales fp16 [groups][out].
//     One source word holds 8 OUTPUTS of one input; its nibble j belongs to output 8 * (word index) + orderMap[j],
//     orderMap = {0, 2, 4, 6, 1, 3, 5, 7} (src/ModelConverter.cs:19). The target word (out, in / 8) holds 8 INPUTS of one
//     output, nibble i = input 8 * (word index) + i (RepackQData, :286-321): a transpose of a 4-bit matrix.
//     Where the number of inputs is not a multiple of 8 (zero points: 108 or 86 groups), the last word of an output is
//     filled up with the first values of the NEXT output, zeros after the last one (the reference packs from a
//     column-major scratch array with four spare elements, :288, :308-312); those nibbles are never read.
//   format v1: weights and zero points are in the target layout already; scales come as [out][zerosSize * 8] and are
//     cut to [out][scalesSize] (:262-275).
#include <cuda_fp16.h>

#include "../../include/ml2b200.h"
#include "host_common.hpp"

namespace ml2 {

// nibble position inside a source word of the output with offset c in its group of 8: inverse of orderMap
__device__ __forceinline__ int awq_nibble_of(int c) { return ((c & 1) << 2) | (c >> 1); }

__device__ __forceinline__ uint32_t awq_value(const uint32_t* __restrict__ in, int w8, int y, int x)
{
    return (in[(size_t)y * w8 + (x >> 3)] >> (4 * awq_nibble_of(x & 7))) & 0xFu;
}

// One thread per output: 8 target words (64 inputs) per pass, written as two 16-byte vectors when the row length allows.
__global__ void __launch_bounds__(256) awq_repack_qdata_kernel(const uint32_t* __restrict__ in, int height, int width, uint32_t* __restrict__ out)
{
    const int x = blockIdx.x * 256 + threadIdx.x;
    const int h8 = (height + 7) >> 3, w8 = (width + 7) >> 3;
    if (x >= width) return;
    const int yb0 = blockIdx.y * 8;
    for (int q = 0; q < 8 && yb0 + q < h8; ++q) {
        const int yb = yb0 + q;
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int y = yb * 8 + i;
            uint32_t v;
            if (y < height) {
                v = awq_value(in, w8, y, x);
            } else {
                // spill-over of the reference's packing: element height * x + y of the column-major scratch array,
                // i.e. the start of the following output(s); zeros beyond the last one
                const int over = y - height;
                const int cx = x + 1 + over / height, cy = over % height;
                v = cx < width ? awq_value(in, w8, cy, cx) : 0u;
            }
            word |= v << (4 * i);
        }
        out[(size_t)x * h8 + yb] = word;
    }
}

// scales fp16 [meta_height][width] -> [width][meta_height] (RepackScales, src/ModelConverter.cs:323-332)
__global__ void __launch_bounds__(256) awq_transpose_scales_kernel(const unsigned short* __restrict__ in, int meta_height, int width,
                                                                   unsigned short* __restrict__ out)
{
    __shared__ unsigned short tile[32][33];
    const int x0 = blockIdx.x * 32, y0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const int y = y0 + r, x = x0 + tx;
        tile[r][tx] = (y < meta_height && x < width) ? in[(size_t)y * width + x] : (unsigned short)0;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int x = x0 + r, y = y0 + tx;
        if (x < width && y < meta_height) out[(size_t)x * meta_height + y] = tile[tx][r];
    }
}

// format v1: scales [width][padded_height] -> [width][scales_size]
__global__ void __launch_bounds__(256) awq_compact_scales_kernel(const unsigned short* __restrict__ in, int scales_size, int padded_height,
                                                                 int width, unsigned short* __restrict__ out)
{
    const size_t n = (size_t)width * scales_size;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t x = i / scales_size, y = i - x * scales_size;
        out[i] = in[x * padded_height + y];
    }
}

}  // namespace ml2

using namespace ml2;

extern "C" {

int ml2_awq_repack_qdata(ml2_ctx* h, const uint32_t* in, int height, int width, uint32_t* out)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !in || !out) return fail(ML2_E_INVALID, "awq_repack_qdata: null argument");
    if (height <= 0 || width <= 0 || (width & 7)) return fail(ML2_E_INVALID, "awq_repack_qdata: height=%d width=%d (width must be a multiple of 8)", height, width);
    cudaSetDevice(ctx->device);
    const dim3 grid((unsigned)((width + 255) / 256), (unsigned)((((height + 7) >> 3) + 7) / 8));
    awq_repack_qdata_kernel<<<grid, 256, 0, ctx->stream>>>(in, height, width, out);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "awq_repack_qdata: %s", cudaGetErrorString(e));
    ++ctx->launches;
    return ML2_OK;
}

int ml2_awq_repack_scales(ml2_ctx* h, const void* in, int meta_height, int width, void* out)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !in || !out) return fail(ML2_E_INVALID, "awq_repack_scales: null argument");
    if (meta_height <= 0 || width <= 0) return fail(ML2_E_INVALID, "awq_repack_scales: meta_height=%d width=%d", meta_height, width);
    cudaSetDevice(ctx->device);
    const dim3 grid((unsigned)((width + 31) / 32), (unsigned)((meta_height + 31) / 32));
    awq_transpose_scales_kernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const unsigned short*>(in), meta_height, width,
                                                              static_cast<unsigned short*>(out));
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "awq_repack_scales: %s", cudaGetErrorString(e));
    ++ctx->launches;
    return ML2_OK;
}

int ml2_awq_compact_scales_v1(ml2_ctx* h, const void* in, int scales_size, int padded_height, int width, void* out)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !in || !out) return fail(ML2_E_INVALID, "awq_compact_scales_v1: null argument");
    if (scales_size <= 0 || padded_height < scales_size || width <= 0)
        return fail(ML2_E_INVALID, "awq_compact_scales_v1: scales_size=%d padded_height=%d width=%d", scales_size, padded_height, width);
    cudaSetDevice(ctx->device);
    const size_t n = (size_t)width * scales_size;
    const unsigned blocks = (unsigned)std::min<size_t>((n + 255) / 256, 148 * 8);
    awq_compact_scales_kernel<<<blocks, 256, 0, ctx->stream>>>(static_cast<const unsigned short*>(in), scales_size, padded_height, width,
                                                              static_cast<unsigned short*>(out));
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "awq_compact_scales_v1: %s", cudaGetErrorString(e));
    ++ctx->launches;
    return ML2_OK;
}

}  // extern "C"
