// Host-buffer int4 mat-vec for callers that must not see this library allocate device memory.
//
// The reference's hosts own every device byte: all buffers are C#-side `CudaDeviceVariable`s, native code
// only borrows pointers, and RunState sizes the KV cache from the free memory it observes. A library that
// calls cudaMalloc behind such a host changes the budget the host computed (and a host that hands the whole
// device to one memory pool has nothing left to give). `ml2_matvec_residual_int4_host` stages its two
// vectors in a buffer it allocates on demand; this variant stages them in a fixed array that is part of
// the library image instead, so it never allocates or frees anything.
#include "../../include/ml2b200.h"

#include <mutex>

#include "host_common.hpp"

namespace ml2 {

constexpr int kStaticMaxRows = 16384;  // widest input vector (elements)
constexpr int kStaticMaxCols = 16384;  // longest output vector (elements)
constexpr size_t kStaticInBytes = (size_t)kStaticMaxRows * 2;
constexpr size_t kStaticOutBytes = (size_t)kStaticMaxCols * 2;

// 64 KiB held by every GPU that loads the library, until the process exits. In host code this name is only
// a stand-in for the symbol; its device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticInBytes + kStaticOutBytes];

static std::mutex g_static_mutex;
static unsigned char* g_static_ptr[64] = {};

// One-time set-up for `device` (the caller has made it current): resolves the array's device address.
static int static_scratch_for(int device, unsigned char** out)
{
    if (device < 0 || device >= 64) return fail(ML2_E_INVALID, "static scratch: device %d out of range", device);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[device]) {
        unsigned char* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
        if (e != cudaSuccess || !p) return fail(ML2_E_CUDA, "static scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_ptr[device] = p;
    }
    *out = g_static_ptr[device];
    return ML2_OK;
}

}  // namespace ml2

using namespace ml2;

extern "C" int ml2_matvec_residual_int4_host_static(ml2_ctx* h, void* inout_host, const void* in_host, const ml2_qweight* w_dev,
                                                    int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !inout_host || !in_host || !w_dev) return fail(ML2_E_INVALID, "matvec_residual_int4_host_static: null argument");
    if (rows <= 0 || cols <= 0) return fail(ML2_E_INVALID, "matvec_residual_int4_host_static: rows=%d cols=%d", rows, cols);
    if (rows > kStaticMaxRows || cols > kStaticMaxCols)
        return fail(ML2_E_INVALID,
                    "matvec_residual_int4_host_static: rows=%d cols=%d exceed the fixed staging array (at most %d inputs and %d "
                    "outputs); use ml2_matvec_residual_int4_host or device buffers for larger vectors",
                    rows, cols, kStaticMaxRows, kStaticMaxCols);
    unsigned char* base = nullptr;
    int rc = use_device(ctx);   // on every call, not only the first: the symbol look-up and the copies below go to this device
    if (rc) return rc;
    if ((rc = static_scratch_for(ctx->device, &base))) return rc;
    // Both regions are fully overwritten by the copies below before the kernel reads them, so nothing has
    // to be cleared between calls; what an earlier call left behind is never observed.
    unsigned char* d_in = base;
    unsigned char* d_out = base + kStaticInBytes;
    cudaError_t e = cudaMemcpyAsync(d_in, in_host, (size_t)rows * 2, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_out, inout_host, (size_t)cols * 2, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "matvec_residual_int4_host_static: host to device: %s", cudaGetErrorString(e));
    if ((rc = ml2_matvec_residual_int4(h, d_out, d_in, w_dev, rows, cols))) return rc;
    e = cudaMemcpyAsync(inout_host, d_out, (size_t)cols * 2, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "matvec_residual_int4_host_static: device to host: %s", cudaGetErrorString(e));
    return ML2_OK;
}
