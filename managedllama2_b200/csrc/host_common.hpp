// Host-side types shared by the C-ABI translation units.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>

#include "common.cuh"

namespace ml2 {

struct Ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool pdl = false;
    DeviceStatus* status_dev = nullptr;
    void* scratch = nullptr;          // host-buffer entry points stage their vectors here
    size_t scratch_bytes = 0;
    long long launches = 0;
    long long wait_cycles = 20000000000ll;   // budget of every device-side wait, in SM clock cycles (about ten seconds)
};

struct MatVecPlan {
    int wsize, zsize, ssize, units;
    int kw, mw, rw, nstage;
    int chunk_bytes, woff_z, woff_s;
    int smem_bytes, ntiles, grid, threads;
};

enum class Fmt : int;
enum class Epi : int;
enum class Pro : int;
struct MatVecParams;

int fail(int code, const char* fmt, ...);
// Makes the context's device current for the calling thread (every entry point does this first: a thread may hold
// several contexts, or may have switched device in between).
int use_device(const Ctx* ctx);
int plan_matvec(const Ctx* ctx, Fmt fmt, Epi epi, int rows, int cols, int nmat, MatVecPlan* pl);
int launch_matvec(Ctx* ctx, Fmt fmt, Epi epi, Pro pro, const MatVecPlan& pl, MatVecParams prm, bool pdl);

// sampling chain (sampler.cu): Sampler.Sample for temperature != 0 on `st`; the logits are consumed in place
int sampler_chain(cudaStream_t st, int device, void* logits, int* indices, int size, float temperature, float top_p, float coin, int* tokens,
                  int next_pos);

}  // namespace ml2
