// C ABI, operator level: argument checks, launch planning and one entry point per Module.Forward
// of the reference (see include/ml2b200.h for the reference file:line of each).
#include "../../include/ml2b200.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "host_common.hpp"
#include "small_ops.cuh"
#include "stream_matvec.cuh"

namespace ml2 {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int use_device(const Ctx* ctx)
{
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e == cudaSuccess && cur != ctx->device) e = cudaSetDevice(ctx->device);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "cudaSetDevice(%d): %s", ctx->device, cudaGetErrorString(e));
    return ML2_OK;
}

// ---- launch planning for the streaming mat-vec ---------------------------------------------------
// Picks rows-per-warp (RW), chunks per stage (MW), ring depth and CTAs per SM so that (a) every bulk
// copy is 16-byte aligned, (b) a kernel stays within ~half an SM (shared memory, threads, registers)
// so the next kernel's weight prefetch can run beside it, (c) there are enough warps per SM to cover
// the dequantisation arithmetic.
int plan_matvec(const Ctx* ctx, Fmt fmt, Epi epi, int rows, int cols, int nmat, MatVecPlan* pl)
{
    MatVecPlan p{};
    if (rows <= 0 || cols <= 0) return fail(ML2_E_INVALID, "mat-vec: rows=%d cols=%d must be positive", rows, cols);
    if (fmt == Fmt::Int4) {
        p.ssize = ceil_div(rows, kGroup);
        p.wsize = ceil_div(rows, 32) * 4;
        p.zsize = ceil_div(p.ssize, 8);
        if (rows % 8) return fail(ML2_E_INVALID, "int4 mat-vec: rows=%d must be a multiple of 8", rows);
    } else {
        if (rows % 8) return fail(ML2_E_INVALID, "fp16 mat-vec: rows=%d must be a multiple of 8", rows);
        p.wsize = rows / 2;
        p.zsize = p.ssize = 0;
    }
    p.units = p.wsize / 4;
    p.kw = ceil_div(p.units, 32);
    if (p.kw > kMaxKW) return fail(ML2_E_INVALID, "mat-vec: d_in=%d too wide for one row per %d warps", rows, kMaxKW);

    const bool paired = (epi == Epi::SwiGLU || epi == Epi::QKVRope);
    // RW = 4 needs 4-row runs of zeros (16*zsize B: always) and scales (8*ssize B) to be 16-byte multiples.
    p.rw = 4;
    if (fmt == Fmt::Int4 && (p.ssize & 1)) p.rw = 8;
    if (paired && p.rw != 4) p.rw = 4;  // paired chunks are 4 rows; ragged scale runs take the slow copy path

    // chunks per stage: aim at >= 8 consumer warps per CTA
    int mw = paired ? 2 : 1;
    while (p.kw * mw < 8 && mw * p.rw < 16) mw += paired ? 2 : 1;
    if (mw < 1 || mw * p.rw > kMaxR || (paired && (mw & 1)) || (p.kw * mw + 2) * 32 > 1024)
        return fail(ML2_E_INVALID, "mat-vec plan: mw=%d invalid for kw=%d rw=%d", mw, p.kw, p.rw);
    p.mw = mw;

    auto a16 = [](int b) { return (b + 15) & ~15; };
    p.woff_z = a16(p.rw * p.wsize * 4);
    p.woff_s = p.woff_z + a16(p.rw * p.zsize * 4);
    p.chunk_bytes = p.woff_s + a16(p.rw * p.ssize * 2);
    const int stage_bytes = p.chunk_bytes * p.mw;

    const int smem_budget = 96 * 1024;
    int ctas = 0;
    const int threads = (p.kw * p.mw + 2) * 32;  // consumers + producer + finalizer
    if (ctas <= 0) {
        ctas = 1;
        // small CTAs: co-schedule several per SM while the ring of each keeps >= 3 stages
        while (ctas < 4 && (ctas + 1) * threads <= 640 && (ctas + 1) * 3 * stage_bytes <= smem_budget) ++ctas;
    }
    int nstage = smem_budget / ctas / stage_bytes;
    if (nstage > 8) nstage = 8;
    if (nstage < 2) nstage = 2;
    p.nstage = nstage;
    p.smem_bytes = nstage * stage_bytes;
    if (p.smem_bytes > 200 * 1024) return fail(ML2_E_INVALID, "mat-vec plan: stage of %d B does not fit shared memory", stage_bytes);

    if (epi == Epi::SwiGLU) {
        p.ntiles = ceil_div(ceil_div(cols, p.rw), p.mw / 2);
    } else if (epi == Epi::QKVRope) {
        p.ntiles = ceil_div(nmat * (cols / 2 / p.rw), p.mw / 2);
    } else {
        p.ntiles = ceil_div(nmat * ceil_div(cols, p.rw), p.mw);
    }
    p.grid = ctx->sm_count * ctas;
    if (p.grid > p.ntiles) p.grid = p.ntiles;
    p.threads = threads;
    *pl = p;
    return ML2_OK;
}

template <Fmt F, Epi E, Pro P>
static cudaError_t launch_rw(const Ctx* ctx, const MatVecPlan& pl, const MatVecParams& prm, bool pdl)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(pl.grid);
    cfg.blockDim = dim3(pl.threads);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e;
    // the opt-in to large dynamic shared memory is per function and per device: once is enough
    static bool attr_done[2][2][16] = {};
    const int dev = ctx->device & 15;
    const int big = pl.threads > 512 ? 1 : 0, r8 = pl.rw == 4 ? 0 : 1;
    const void* k = nullptr;
    if (!big && !r8) k = (const void*)stream_matvec_kernel<F, E, P, 4, 512>;
    if (!big && r8) k = (const void*)stream_matvec_kernel<F, E, P, 8, 512>;
    if (big && !r8) k = (const void*)stream_matvec_kernel<F, E, P, 4, 1024>;
    if (big && r8) k = (const void*)stream_matvec_kernel<F, E, P, 8, 1024>;
    if (!attr_done[big][r8][dev]) {
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_done[big][r8][dev] = true;
    }
    void* args[] = {const_cast<MatVecParams*>(&prm)};
    return cudaLaunchKernelExC(&cfg, k, args);
}

int launch_matvec(Ctx* ctx, Fmt fmt, Epi epi, Pro pro, const MatVecPlan& pl, MatVecParams prm, bool pdl)
{
    prm.wsize = pl.wsize; prm.zsize = pl.zsize; prm.ssize = pl.ssize; prm.units = pl.units;
    prm.kw = pl.kw; prm.mw = pl.mw; prm.nstage = pl.nstage; prm.chunk_bytes = pl.chunk_bytes;
    prm.woff_z = pl.woff_z; prm.woff_s = pl.woff_s; prm.ntiles = pl.ntiles;
    prm.status = ctx->status_dev;
    if (int rc = use_device(ctx)) return rc;
    cudaError_t e = cudaErrorInvalidValue;
#define ML2_CASE(F_, E_, P_) \
    if (fmt == F_ && epi == E_ && pro == P_) e = launch_rw<F_, E_, P_>(ctx, pl, prm, pdl);
    ML2_CASE(Fmt::Int4, Epi::Store, Pro::Plain)
    ML2_CASE(Fmt::Int4, Epi::Store, Pro::RMSNorm)
    ML2_CASE(Fmt::Int4, Epi::Residual, Pro::Plain)
    ML2_CASE(Fmt::Int4, Epi::SwiGLU, Pro::Plain)
    ML2_CASE(Fmt::Int4, Epi::SwiGLU, Pro::RMSNorm)
    ML2_CASE(Fmt::Int4, Epi::PartialF32, Pro::Plain)
    ML2_CASE(Fmt::Int4, Epi::QKVRope, Pro::RMSNorm)
    ML2_CASE(Fmt::F16, Epi::Store, Pro::Plain)
    ML2_CASE(Fmt::F16, Epi::Store, Pro::RMSNorm)
#undef ML2_CASE
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "mat-vec launch failed: %s", cudaGetErrorString(e));
    ++ctx->launches;
    return ML2_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_qw(const char* what, const ml2_qweight* q)
{
    if (!q || !q->weight || !q->zeros || !q->scales) return fail(ML2_E_INVALID, "%s: null QWeight array", what);
    if (!aligned16(q->weight) || (reinterpret_cast<uintptr_t>(q->zeros) & 3u) || (reinterpret_cast<uintptr_t>(q->scales) & 1u))
        return fail(ML2_E_INVALID, "%s: QWeight.Weight must be 16-byte aligned (Zeros 4, Scales 2)", what);
    return ML2_OK;
}
static QWPtrs qw(const ml2_qweight* q) { return QWPtrs{q->weight, q->zeros, static_cast<const __half*>(q->scales)}; }

static int check_cuda(const char* what)
{
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return ML2_OK;
}

template <typename... Args>
static int launch_small(Ctx* ctx, const char* what, void (*kernel)(Args...), dim3 grid, dim3 block, Args... args)
{
    if (int rc = use_device(ctx)) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->pdl ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    ++ctx->launches;
    return ML2_OK;
}

}  // namespace ml2

using namespace ml2;

extern "C" {

const char* ml2_last_error(void) { return g_err; }
int ml2_version(void) { return 100; }

int ml2_ctx_create(int device, ml2_ctx** out)
{
    if (!out) return fail(ML2_E_INVALID, "ml2_ctx_create: out is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) return fail(ML2_E_CUDA, "no CUDA device: %s", cudaGetErrorString(e));
    if (device < 0 || device >= n) return fail(ML2_E_INVALID, "device %d out of range (0..%d)", device, n - 1);
    if ((e = cudaSetDevice(device)) != cudaSuccess) return fail(ML2_E_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return fail(ML2_E_CUDA, "%s", cudaGetErrorString(e));
    if (prop.major != 10) return fail(ML2_E_INVALID, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    Ctx* c = new Ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->stream = nullptr;
    c->pdl = false;
    if ((e = cudaMalloc(&c->status_dev, sizeof(DeviceStatus))) != cudaSuccess ||
        (e = cudaMemset(c->status_dev, 0, sizeof(DeviceStatus))) != cudaSuccess) {
        delete c;
        return fail(ML2_E_CUDA, "status word: %s", cudaGetErrorString(e));
    }
    *out = reinterpret_cast<ml2_ctx*>(c);
    return ML2_OK;
}

int ml2_ctx_destroy(ml2_ctx* h)
{
    Ctx* c = reinterpret_cast<Ctx*>(h);
    if (!c) return ML2_OK;
    cudaSetDevice(c->device);
    if (c->status_dev) cudaFree(c->status_dev);
    if (c->scratch) cudaFree(c->scratch);
    delete c;
    return ML2_OK;
}

int ml2_ctx_set_stream(ml2_ctx* h, void* s)
{
    if (!h) return fail(ML2_E_INVALID, "null context");
    reinterpret_cast<Ctx*>(h)->stream = static_cast<cudaStream_t>(s);
    return ML2_OK;
}
int ml2_ctx_set_pdl(ml2_ctx* h, int on)
{
    if (!h) return fail(ML2_E_INVALID, "null context");
    reinterpret_cast<Ctx*>(h)->pdl = on != 0;
    return ML2_OK;
}
int ml2_ctx_set_wait_limit(ml2_ctx* h, long long sm_cycles)
{
    if (!h) return fail(ML2_E_INVALID, "null context");
    if (sm_cycles < 1000) return fail(ML2_E_INVALID, "wait limit of %lld cycles is too short", sm_cycles);
    reinterpret_cast<Ctx*>(h)->wait_cycles = sm_cycles;
    return ML2_OK;
}
int ml2_ctx_synchronize(ml2_ctx* h)
{
    if (!h) return fail(ML2_E_INVALID, "null context");
    if (int rc = use_device(reinterpret_cast<Ctx*>(h))) return rc;
    const cudaError_t e = cudaStreamSynchronize(reinterpret_cast<Ctx*>(h)->stream);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "synchronize: %s", cudaGetErrorString(e));
    return ML2_OK;
}
int ml2_ctx_status(ml2_ctx* h, unsigned* error, unsigned* detail)
{
    Ctx* c = reinterpret_cast<Ctx*>(h);
    if (!c) return fail(ML2_E_INVALID, "null context");
    if (int rc = use_device(c)) return rc;
    DeviceStatus st{};
    cudaError_t e = cudaMemcpyAsync(&st, c->status_dev, sizeof(st), cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e == cudaSuccess && st.error) e = cudaMemsetAsync(c->status_dev, 0, sizeof(st), c->stream);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "status: %s", cudaGetErrorString(e));
    if (error) *error = st.error;
    if (detail) *detail = st.detail;
    return st.error ? fail(ML2_E_DEVICE, "a kernel gave up waiting (code %u, tile %u)", st.error, st.detail) : ML2_OK;
}
long long ml2_ctx_launch_count(ml2_ctx* h) { return h ? reinterpret_cast<Ctx*>(h)->launches : 0; }

// ---- int4 family -------------------------------------------------------------------------------
int ml2_matvec_residual_int4(ml2_ctx* h, void* inout, const void* in, const ml2_qweight* w, int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !inout || !in) return fail(ML2_E_INVALID, "matvec_residual_int4: null argument");
    if (inout == in) return fail(ML2_E_INVALID, "matvec_residual_int4: input aliases the residual output");
    if (!aligned16(in)) return fail(ML2_E_INVALID, "matvec_residual_int4: input must be 16-byte aligned");
    int rc = check_qw("matvec_residual_int4", w);
    if (rc) return rc;
    MatVecPlan pl;
    if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::Residual, rows, cols, 1, &pl))) return rc;
    MatVecParams p{};
    p.mat[0] = qw(w);
    p.out[0] = static_cast<__half*>(inout);
    p.in = static_cast<const __half*>(in);
    p.rows = rows; p.cols = cols; p.nmat = 1;
    return launch_matvec(ctx, Fmt::Int4, Epi::Residual, Pro::Plain, pl, p, ctx->pdl);
}

int ml2_matvec_int4(ml2_ctx* h, void* out, const void* in, const ml2_qweight* w, int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out || !in) return fail(ML2_E_INVALID, "matvec_int4: null argument");
    if (!aligned16(in)) return fail(ML2_E_INVALID, "matvec_int4: input must be 16-byte aligned");
    int rc = check_qw("matvec_int4", w);
    if (rc) return rc;
    MatVecPlan pl;
    if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::Store, rows, cols, 1, &pl))) return rc;
    MatVecParams p{};
    p.mat[0] = qw(w);
    p.out[0] = static_cast<__half*>(out);
    p.in = static_cast<const __half*>(in);
    p.rows = rows; p.cols = cols; p.nmat = 1;
    return launch_matvec(ctx, Fmt::Int4, Epi::Store, Pro::Plain, pl, p, ctx->pdl);
}

int ml2_qkv_matvec_int4(ml2_ctx* h, void* q_out, void* k_out, void* v_out, const void* in, const ml2_qweight* q,
                        const ml2_qweight* k, const ml2_qweight* v, int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !q_out || !k_out || !v_out || !in) return fail(ML2_E_INVALID, "qkv_matvec_int4: null argument");
    if (!aligned16(in)) return fail(ML2_E_INVALID, "qkv_matvec_int4: input must be 16-byte aligned");
    int rc;
    if ((rc = check_qw("qkv_matvec_int4(query)", q)) || (rc = check_qw("qkv_matvec_int4(key)", k)) ||
        (rc = check_qw("qkv_matvec_int4(value)", v)))
        return rc;
    MatVecPlan pl;
    if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::Store, rows, cols, 3, &pl))) return rc;
    MatVecParams p{};
    p.mat[0] = qw(q); p.mat[1] = qw(k); p.mat[2] = qw(v);
    p.out[0] = static_cast<__half*>(q_out); p.out[1] = static_cast<__half*>(k_out); p.out[2] = static_cast<__half*>(v_out);
    p.in = static_cast<const __half*>(in);
    p.rows = rows; p.cols = cols; p.nmat = 3;
    return launch_matvec(ctx, Fmt::Int4, Epi::Store, Pro::Plain, pl, p, ctx->pdl);
}

int ml2_matvec_swiglu_int4(ml2_ctx* h, void* out, const void* in, const ml2_qweight* gate, const ml2_qweight* up, int rows,
                           int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out || !in) return fail(ML2_E_INVALID, "matvec_swiglu_int4: null argument");
    if (!aligned16(in)) return fail(ML2_E_INVALID, "matvec_swiglu_int4: input must be 16-byte aligned");
    int rc;
    if ((rc = check_qw("matvec_swiglu_int4(gate)", gate)) || (rc = check_qw("matvec_swiglu_int4(up)", up))) return rc;
    MatVecPlan pl;
    if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::SwiGLU, rows, cols, 2, &pl))) return rc;
    MatVecParams p{};
    p.mat[0] = qw(gate); p.mat[1] = qw(up);
    p.out[0] = static_cast<__half*>(out);
    p.in = static_cast<const __half*>(in);
    p.rows = rows; p.cols = cols; p.nmat = 2;
    return launch_matvec(ctx, Fmt::Int4, Epi::SwiGLU, Pro::Plain, pl, p, ctx->pdl);
}

int ml2_matvec_f16(ml2_ctx* h, void* out, const void* in, const void* matrix, int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out || !in || !matrix) return fail(ML2_E_INVALID, "matvec_f16: null argument");
    if (!aligned16(in) || !aligned16(matrix)) return fail(ML2_E_INVALID, "matvec_f16: input and matrix must be 16-byte aligned");
    MatVecPlan pl;
    int rc;
    if ((rc = plan_matvec(ctx, Fmt::F16, Epi::Store, rows, cols, 1, &pl))) return rc;
    MatVecParams p{};
    p.mat[0] = QWPtrs{static_cast<const uint32_t*>(matrix), nullptr, nullptr};
    p.out[0] = static_cast<__half*>(out);
    p.in = static_cast<const __half*>(in);
    p.rows = rows; p.cols = cols; p.nmat = 1;
    return launch_matvec(ctx, Fmt::F16, Epi::Store, Pro::Plain, pl, p, ctx->pdl);
}

int ml2_dequant_int4(ml2_ctx* h, void* out, const ml2_qweight* w, int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out) return fail(ML2_E_INVALID, "dequant_int4: null argument");
    int rc = check_qw("dequant_int4", w);
    if (rc) return rc;
    if (rows <= 0 || cols <= 0) return fail(ML2_E_INVALID, "dequant_int4: rows=%d cols=%d", rows, cols);
    const int ssize = ceil_div(rows, kGroup), wsize = ceil_div(rows, 32) * 4, zsize = ceil_div(ssize, 8);
    const long long total = (long long)cols * ceil_div(rows, 8);
    const QWPtrs q = qw(w);
    dequant_int4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(static_cast<__half*>(out), q.w, q.z, q.s, rows, cols,
                                                                                wsize, zsize, ssize);
    ++ctx->launches;
    return check_cuda("dequant_int4");
}

// ---- attention products and small operators ------------------------------------------------------
int ml2_matvec_strided(ml2_ctx* h, void* attention, const void* query, const void* key, int head_size, int dim, int n_heads,
                       int seq_length, float scale)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !attention || !query || !key) return fail(ML2_E_INVALID, "matvec_strided: null argument");
    if (head_size <= 0 || n_heads <= 0 || seq_length <= 0 || dim < head_size * n_heads)
        return fail(ML2_E_INVALID, "matvec_strided: head_size=%d heads=%d dim=%d seq=%d", head_size, n_heads, dim, seq_length);
    if ((head_size % 4) || (dim % 4) || (reinterpret_cast<uintptr_t>(query) & 7u) || (reinterpret_cast<uintptr_t>(key) & 7u))
        return fail(ML2_E_INVALID, "matvec_strided: head_size and dim must be multiples of 4 and pointers 8-byte aligned");
    return launch_small(ctx, "matvec_strided", attn_scores_kernel, dim3(ceil_div(seq_length, 8), n_heads), dim3(256),
                        static_cast<__half*>(attention), static_cast<const __half*>(query), static_cast<const __half*>(key), head_size,
                        dim, seq_length, scale);
}

int ml2_softmax(ml2_ctx* h, void* attention, int n_heads, int seq_length)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !attention) return fail(ML2_E_INVALID, "softmax: null argument");
    if (n_heads <= 0 || seq_length <= 0) return fail(ML2_E_INVALID, "softmax: heads=%d seq=%d", n_heads, seq_length);
    const int block = seq_length >= 1024 ? 1024 : (seq_length > 128 ? 256 : 128);
    return launch_small(ctx, "softmax", softmax_kernel, dim3(n_heads), dim3(block), static_cast<__half*>(attention), seq_length);
}

int ml2_vecmat(ml2_ctx* h, void* out, const void* value, const void* attention, int head_size, int dim, int n_heads, int seq_length)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out || !value || !attention) return fail(ML2_E_INVALID, "vecmat: null argument");
    if (head_size <= 0 || n_heads <= 0 || seq_length <= 0 || dim < head_size * n_heads)
        return fail(ML2_E_INVALID, "vecmat: head_size=%d heads=%d dim=%d seq=%d", head_size, n_heads, dim, seq_length);
    if ((head_size % 4) || (dim % 4) || (reinterpret_cast<uintptr_t>(value) & 7u))
        return fail(ML2_E_INVALID, "vecmat: head_size and dim must be multiples of 4 and value 8-byte aligned");
    const int warps = seq_length >= 256 ? 32 : (seq_length >= 32 ? 8 : 4);
    return launch_small(ctx, "vecmat", attn_values_kernel, dim3(ceil_div(head_size, 128), n_heads), dim3(warps * 32),
                        static_cast<__half*>(out), static_cast<const __half*>(attention), static_cast<const __half*>(value), head_size,
                        dim, seq_length);
}

int ml2_rmsnorm(ml2_ctx* h, void* out, const void* in, const void* weights, int size, float eps)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out || !in || !weights) return fail(ML2_E_INVALID, "rmsnorm: null argument");
    if (size <= 0) return fail(ML2_E_INVALID, "rmsnorm: size=%d", size);
    return launch_small(ctx, "rmsnorm", rmsnorm_kernel, dim3(1), dim3(1024), static_cast<__half*>(out), static_cast<const __half*>(in),
                        static_cast<const __half*>(weights), size, eps);
}

int ml2_rope(ml2_ctx* h, void* query, void* key, int n_heads, int n_kv_heads, int head_size, int pos, float theta)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !query || !key) return fail(ML2_E_INVALID, "rope: null argument");
    if (n_heads <= 0 || n_kv_heads < 0 || n_kv_heads > n_heads || head_size <= 0 || (head_size & 1) || pos < 0)
        return fail(ML2_E_INVALID, "rope: heads=%d kv_heads=%d head_size=%d pos=%d", n_heads, n_kv_heads, head_size, pos);
    const int n = n_heads * (head_size / 2);
    return launch_small(ctx, "rope", rope_kernel, dim3(ceil_div(n, 256)), dim3(256), static_cast<__half*>(query),
                        static_cast<__half*>(key), n_heads, n_kv_heads, head_size, pos, theta);
}

int ml2_embedding(ml2_ctx* h, void* out, const void* table, int size, const int* tokens, int pos)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out || !table || !tokens) return fail(ML2_E_INVALID, "embedding: null argument");
    if (size <= 0 || pos < 0) return fail(ML2_E_INVALID, "embedding: size=%d pos=%d", size, pos);
    return launch_small(ctx, "embedding", embedding_kernel, dim3(ceil_div(size, 256)), dim3(256), static_cast<__half*>(out),
                        static_cast<const __half*>(table), size, tokens, pos);
}

int ml2_argmax(ml2_ctx* h, const void* logits, int vocab_size, int* tokens, int next_pos, int write_token)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !logits || !tokens) return fail(ML2_E_INVALID, "argmax: null argument");
    if (vocab_size <= 0 || next_pos < 0) return fail(ML2_E_INVALID, "argmax: vocab=%d pos=%d", vocab_size, next_pos);
    return launch_small(ctx, "argmax", argmax_kernel, dim3(1), dim3(1024), static_cast<const __half*>(logits), vocab_size, tokens,
                        next_pos, write_token);
}

// ---- host-buffer variant ---------------------------------------------------------------------------
int ml2_matvec_residual_int4_host(ml2_ctx* h, void* inout_host, const void* in_host, const ml2_qweight* w_dev, int rows, int cols)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !inout_host || !in_host) return fail(ML2_E_INVALID, "matvec_residual_int4_host: null argument");
    if (rows <= 0 || cols <= 0) return fail(ML2_E_INVALID, "matvec_residual_int4_host: rows=%d cols=%d", rows, cols);
    const size_t in_b = ((size_t)rows * 2 + 255) & ~size_t(255), out_b = ((size_t)cols * 2 + 255) & ~size_t(255);
    if (ctx->scratch_bytes < in_b + out_b) {
        if (ctx->scratch) cudaFree(ctx->scratch);
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
        const cudaError_t e = cudaMalloc(&ctx->scratch, in_b + out_b);
        if (e != cudaSuccess) return fail(ML2_E_CUDA, "scratch: %s", cudaGetErrorString(e));
        ctx->scratch_bytes = in_b + out_b;
    }
    char* d_in = static_cast<char*>(ctx->scratch);
    char* d_out = d_in + in_b;
    cudaError_t e = cudaMemcpyAsync(d_in, in_host, (size_t)rows * 2, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_out, inout_host, (size_t)cols * 2, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "H2D: %s", cudaGetErrorString(e));
    const int rc = ml2_matvec_residual_int4(h, d_out, d_in, w_dev, rows, cols);
    if (rc) return rc;
    e = cudaMemcpyAsync(inout_host, d_out, (size_t)cols * 2, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "D2H: %s", cudaGetErrorString(e));
    return ML2_OK;
}

// ---- synthetic tensors -------------------------------------------------------------------------------
int ml2_synth_qweight(ml2_ctx* h, uint32_t* weight, uint32_t* zeros, void* scales, int rows_full, int col0, int ncols, int g0,
                      int ngroups, uint64_t seed, uint32_t tensor_id)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !weight || !zeros || !scales) return fail(ML2_E_INVALID, "synth_qweight: null argument");
    if (rows_full <= 0 || (rows_full % 32) || ncols <= 0 || g0 < 0 || ngroups <= 0 || g0 * kGroup >= rows_full)
        return fail(ML2_E_INVALID, "synth_qweight: rows_full=%d ncols=%d g0=%d ngroups=%d", rows_full, ncols, g0, ngroups);
    synth_qweight_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(weight, zeros, static_cast<__half*>(scales), rows_full, col0, ncols,
                                                                     g0, ngroups, synth_key(seed, tensor_id, 0),
                                                                     synth_key(seed, tensor_id, 1), synth_key(seed, tensor_id, 2));
    ++ctx->launches;
    return check_cuda("synth_qweight");
}

int ml2_synth_normal_f16(ml2_ctx* h, void* out, long long row0, long long nrows, int width, float sigma, uint64_t seed,
                         uint32_t tensor_id)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !out) return fail(ML2_E_INVALID, "synth_normal_f16: null argument");
    if (row0 < 0 || nrows <= 0 || width <= 0) return fail(ML2_E_INVALID, "synth_normal_f16: bad shape");
    synth_normal_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(static_cast<__half*>(out), row0, nrows, width, sigma,
                                                                    synth_key(seed, tensor_id, 3));
    ++ctx->launches;
    return check_cuda("synth_normal_f16");
}

int ml2_synth_qweight_host(uint32_t* weight, uint32_t* zeros, void* scales_v, int rows_full, int col0, int ncols, int g0, int ngroups,
                           uint64_t seed, uint32_t tensor_id)
{
    if (!weight || !zeros || !scales_v) return fail(ML2_E_INVALID, "synth_qweight_host: null argument");
    if (rows_full <= 0 || (rows_full % 32) || ncols <= 0 || g0 < 0 || ngroups <= 0 || g0 * kGroup >= rows_full)
        return fail(ML2_E_INVALID, "synth_qweight_host: bad shape");
    __half* scales = static_cast<__half*>(scales_v);
    const uint64_t kw = synth_key(seed, tensor_id, 0), kz = synth_key(seed, tensor_id, 1), ks = synth_key(seed, tensor_id, 2);
    const int rows = std::min(ngroups * kGroup, rows_full - g0 * kGroup);
    const int wsize = ceil_div(rows, 32) * 4, ssize = ceil_div(rows, kGroup), zsize = ceil_div(ssize, 8);
    const int groups_full = ceil_div(rows_full, kGroup);
    for (int c = 0; c < ncols; ++c) {
        for (int j = 0; j < wsize; ++j) {
            const int jf = g0 * (kGroup / 8) + j;
            weight[(size_t)c * wsize + j] = (jf * 8 < rows_full && j * 8 < rows) ? synth_weight_word(kw, rows_full, col0 + c, jf) : 0u;
        }
        for (int zw = 0; zw < zsize; ++zw) {
            uint32_t word = 0;
            for (int n = 0; n < 8; ++n) {
                const int g = zw * 8 + n;
                if (g < ssize) word |= synth_zero(kz, groups_full, col0 + c, g0 + g) << (4 * n);
            }
            zeros[(size_t)c * zsize + zw] = word;
        }
        for (int g = 0; g < ssize; ++g) scales[(size_t)c * ssize + g] = __float2half_rn(synth_scale_f32(ks, groups_full, col0 + c, g0 + g));
    }
    return ML2_OK;
}

int ml2_synth_normal_f16_host(void* out_v, long long row0, long long nrows, int width, float sigma, uint64_t seed, uint32_t tensor_id)
{
    if (!out_v || row0 < 0 || nrows <= 0 || width <= 0) return fail(ML2_E_INVALID, "synth_normal_f16_host: bad argument");
    __half* out = static_cast<__half*>(out_v);
    const uint64_t key = synth_key(seed, tensor_id, 3);
    for (long long i = 0; i < nrows * width; ++i) out[i] = __float2half_rn(synth_normal_f32(key, (uint64_t)(row0 * width + i), sigma));
    return ML2_OK;
}

}  // extern "C"
