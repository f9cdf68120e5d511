// C ABI, model level: Transformer.Forward of the reference (src/Transformer.cs:158-190) as five fused
// kernels per layer replayed from one CUDA graph, with optional tensor parallelism (one process per GPU).
//
// Per layer, single GPU:
//   1. RMSNorm + QKV int4 mat-vec + RoPE, k/v written straight into the cache row      (reference: 3 launches)
//   2. fused attention (scores, softmax, values)                                       (reference: 3 launches)
//   3. o-proj int4 mat-vec + residual
//   4. RMSNorm + gate/up int4 mat-vec + SwiGLU                                         (reference: 2 launches)
//   5. down int4 mat-vec + residual
// then RMSNorm + fp16 classifier and the arg-max. The position lives in device memory (StepState), so
// one graph serves every token; only the first node's parameters are refreshed per replay.
//
// Tensor parallel (tp > 1): QKV / gate / up sharded by output rows, o-proj / down by input groups of
// 128, KV cache by heads, classifier by vocabulary rows. o-proj and down produce fp32 partials that
// are summed with ncclAllReduce before the single fp16 rounding of the residual add, so every rank
// holds bit-identical activations.
#include "../../include/ml2b200.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstring>
#include <vector>

#include "attention.cuh"
#include "host_common.hpp"
#include "megakernel.cuh"
#include "small_ops.cuh"
#include "stream_matvec.cuh"

namespace ml2 {

// NCCL is bound at run time, and only when tensor parallelism is used: a process that already carries an
// NCCL (e.g. the one PyTorch ships) keeps exactly that copy; otherwise the system library is loaded.
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
static NcclApi g_nccl;

static int nccl_load()
{
    if (g_nccl.ok) return ML2_OK;
    const char* override_path = getenv("ML2_NCCL_LIB");
    void* h = nullptr;
    if (override_path && *override_path) h = dlopen(override_path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);  // already in the process
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(ML2_E_NCCL, "cannot load libnccl.so.2: %s", dlerror());
#define ML2_SYM(field, name)                                                       \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));       \
    if (!g_nccl.field) return fail(ML2_E_NCCL, "libnccl.so.2 lacks %s", name);
    ML2_SYM(GetUniqueId, "ncclGetUniqueId")
    ML2_SYM(CommInitRank, "ncclCommInitRank")
    ML2_SYM(CommDestroy, "ncclCommDestroy")
    ML2_SYM(AllReduce, "ncclAllReduce")
    ML2_SYM(AllGather, "ncclAllGather")
    ML2_SYM(GetErrorString, "ncclGetErrorString")
#undef ML2_SYM
    g_nccl.ok = true;
    return ML2_OK;
}

struct StepState {
    int pos;
    int next_pos;
    int write_token;
    int reserved;
};

// first node of the token graph: publishes the step and gathers the embedding row
// (native/embedding_kernel.cu:3-17)
__global__ void begin_step_kernel(StepState* st, int pos, int next_pos, int write_token, __half* x, const __half* table, int dim,
                                  const int* tokens)
{
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        st->pos = pos;
        st->next_pos = next_pos;
        st->write_token = write_token;
    }
    const int token = tokens[pos];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x) x[i] = table[(size_t)token * dim + i];
}

// argmax with the step taken from device memory (native/argmax_kernel.cu:8-46; lowest index wins ties)
__global__ void __launch_bounds__(1024) argmax_step_kernel(const __half* logits, int size, int* tokens, const StepState* st)
{
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    pdl_wait();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = __half2float(logits[i]);
        if (v > best) { best = v; best_i = i; }
    }
    auto better = [](float a, int ai, float b, int bi) { return a > b || (a == b && ai < bi); };
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
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
        if (lane == 0 && st->write_token) tokens[st->next_pos] = (best_i == 0x7fffffff) ? 0 : best_i;
    }
}

// x = half(float(x) + all-reduced partial): the residual add of the row-sharded mat-vecs
// (rounding point of native/mat_vec_kernel.cu:154-156)
__global__ void residual_add_f32_kernel(__half* x, const float* sum, int n)
{
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __float2half_rn(__half2float(x[i]) + sum[i]);
}

struct LayerW {
    ml2_qweight q, k, v, o, gate, up, down;
    const __half* rms_att;
    const __half* rms_ffn;
    bool bound = false;
};

struct Model {
    Ctx* ctx = nullptr;
    ml2_config cfg{};
    int tp = 1, rank = 0;
    // local (per-rank) shapes
    int heads_local = 0, dim_local = 0;    // attention width owned by this rank
    int hidden_local = 0;                   // hidden rows owned (whole groups of 128)
    int vocab_local = 0, vocab_row0 = 0;
    int head_size = 0;
    float eps = 1e-5f;
    std::vector<LayerW> layers;
    const __half* embed = nullptr;
    const __half* classifier = nullptr;     // local vocabulary rows
    const __half* rms_final = nullptr;
    // run state (src/RunState.cs:5-25); owned here unless bound by the caller
    __half *x = nullptr, *xb = nullptr, *h = nullptr, *q = nullptr, *logits = nullptr, *att = nullptr;
    __half *key_cache = nullptr, *value_cache = nullptr;
    int* tokens = nullptr;
    bool own_state = false;
    float* partial = nullptr;               // fp32 [dim], tp > 1
    __half* logits_local = nullptr;         // tp > 1
    float2* rope_table = nullptr;
    StepState* step = nullptr;
    ncclComm_t comm = nullptr;
    // graph
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaGraphNode_t first_node = nullptr;
    cudaStream_t stream = nullptr;          // owned non-blocking stream used for capture and replay
    bool use_graph = true;
    bool use_pdl = true;
    long long launches_per_token = 0;
    std::vector<void*> owned;
    // persistent per-token kernel (single launch per token)
    bool use_mega = true;
    bool mega_built = false, mega_ok = false;
    MegaOp* mega_ops = nullptr;
    MegaTile* mega_tiles = nullptr;         // every CTA's tile descriptors, in streaming order
    int* mega_tile_begin = nullptr;         // [grid + 1]
    unsigned short* mega_op_tiles = nullptr;   // [nops][grid]
    unsigned int* mega_done = nullptr;
    int mega_nops = 0, mega_nstage = 0, mega_slot = 0, mega_att_bytes = 0, mega_smem = 0, mega_grid = 0;
    unsigned int mega_seq = 0;
    long long* mega_prof = nullptr;
    bool want_prof = false;
    bool poisoned = false;                  // a kernel's wait ran out: counters are mid-token, forwards are refused until ml2_model_reset
    int last_pos = 0;                       // position of the latest forward (ml2_model_profile times the attention there)                 // cycle counters of the diagnostic instantiation (ML2_MEGA_PROF=1 at model creation)
    unsigned int* mega_done_ptr = nullptr;
    __half* logits_view = nullptr;          // where the full logits of the persistent kernel land
    int* sample_indices = nullptr;          // token ids carried through the sampler's sort (RunState.indices)
    // attention split over several CTAs per head (persistent kernel, long contexts)
    float* att_ml = nullptr;
    float* att_part = nullptr;
    unsigned int* att_cnt = nullptr;
    int att_split = 1;                      // CTAs per head when the split path is taken (1: never)
    int att_min_seq = 704;                  // shortest sequence that takes it
    unsigned int att_seq = 0;
    // tensor parallel persistent kernel: one peer-visible buffer per rank (counters, receive zones, logits)
    void* comm_local = nullptr;
    void* comm_peer[8] = {};
    bool comm_attached = false;
};

#define ML2_CUDA(call)                                                                       \
    do {                                                                                     \
        const cudaError_t e_ = (call);                                                       \
        if (e_ != cudaSuccess) return fail(ML2_E_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)
#define ML2_NCCL(call)                                                                       \
    do {                                                                                     \
        const ncclResult_t r_ = (call);                                                      \
        if (r_ != ncclSuccess) return fail(ML2_E_NCCL, "%s: %s", #call, g_nccl.GetErrorString(r_)); \
    } while (0)

static int dev_alloc(Model* m, void** p, size_t bytes)
{
    ML2_CUDA(cudaMalloc(p, bytes));
    ML2_CUDA(cudaMemsetAsync(*p, 0, bytes, m->stream));
    m->owned.push_back(*p);
    return ML2_OK;
}

static QWPtrs qwp(const ml2_qweight& q) { return QWPtrs{q.weight, q.zeros, static_cast<const __half*>(q.scales)}; }

template <typename... Args>
static int launch_k(Model* m, const char* what, void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, bool pdl, Args... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = m->ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && m->use_pdl) ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e != cudaSuccess) return fail(ML2_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
    ++m->ctx->launches;
    return ML2_OK;
}

// One token's worth of launches on ctx->stream (captured once, or issued eagerly).
static int enqueue_token(Model* m, int pos, int next_pos, int write_token)
{
    Ctx* ctx = m->ctx;
    const ml2_config& c = m->cfg;
    const int dim = c.dim;
    const bool pdl = m->use_pdl;
    int rc;
    const long long before = ctx->launches;

    if ((rc = launch_k(m, "begin_step", begin_step_kernel, dim3(ceil_div(dim, 256)), dim3(256), 0, false, m->step, pos, next_pos,
                       write_token, m->x, m->embed, dim, (const int*)m->tokens)))
        return rc;

    MatVecPlan pl_qkv, pl_o, pl_gu, pl_down, pl_cls;
    if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::QKVRope, dim, m->dim_local, 3, &pl_qkv))) return rc;
    if ((rc = plan_matvec(ctx, Fmt::Int4, m->tp > 1 ? Epi::PartialF32 : Epi::Residual, m->dim_local, dim, 1, &pl_o))) return rc;
    if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::SwiGLU, dim, m->hidden_local, 2, &pl_gu))) return rc;
    if ((rc = plan_matvec(ctx, Fmt::Int4, m->tp > 1 ? Epi::PartialF32 : Epi::Residual, m->hidden_local, dim, 1, &pl_down))) return rc;
    if ((rc = plan_matvec(ctx, Fmt::F16, Epi::Store, dim, m->vocab_local, 1, &pl_cls))) return rc;

    const size_t kv_layer = (size_t)c.seq_len * m->dim_local;
    const int chunk_cap = std::max(ceil_div(c.seq_len, kAttnCluster), kAttnSingleCtaMax);

    for (int l = 0; l < c.n_layers; ++l) {
        const LayerW& L = m->layers[l];
        __half* kc = m->key_cache + (size_t)l * kv_layer;
        __half* vc = m->value_cache + (size_t)l * kv_layer;
        {   // 1. rmsnorm + qkv + rope (src/Transformer.cs:167-173)
            MatVecParams p{};
            p.mat[0] = qwp(L.q); p.mat[1] = qwp(L.k); p.mat[2] = qwp(L.v);
            p.out[0] = m->q; p.out[1] = kc; p.out[2] = vc;
            p.in = m->x; p.gamma = L.rms_att; p.eps = m->eps;
            p.rope_table = m->rope_table; p.pos_ptr = &m->step->pos; p.kv_row_stride = m->dim_local;
            p.rows = dim; p.cols = m->dim_local; p.nmat = 3; p.head_size = m->head_size;
            if ((rc = launch_matvec(ctx, Fmt::Int4, Epi::QKVRope, Pro::RMSNorm, pl_qkv, p, pdl))) return rc;
        }
        {   // 2. attention (src/Transformer.cs:150-156)
            AttnParams a{};
            a.out = m->xb; a.q = m->q; a.k = kc; a.v = vc; a.pos_ptr = &m->step->pos;
            a.n_heads = m->heads_local; a.head_size = m->head_size; a.row_stride = m->dim_local;
            a.scale = 1.0f / sqrtf((float)m->head_size); a.chunk_cap = chunk_cap;
            if ((rc = launch_k(m, "attention", fused_attention_kernel, dim3(m->heads_local * kAttnCluster), dim3(kAttnThreads),
                               (size_t)chunk_cap * sizeof(float), true, a)))
                return rc;
        }
        {   // 3. o-proj + residual (:177)
            MatVecParams p{};
            p.mat[0] = qwp(L.o); p.in = m->xb; p.rows = m->dim_local; p.cols = dim; p.nmat = 1;
            if (m->tp > 1) {
                p.out_f32 = m->partial;
                if ((rc = launch_matvec(ctx, Fmt::Int4, Epi::PartialF32, Pro::Plain, pl_o, p, pdl))) return rc;
                ML2_NCCL(g_nccl.AllReduce(m->partial, m->partial, dim, ncclFloat, ncclSum, m->comm, ctx->stream));
                if ((rc = launch_k(m, "residual_add", residual_add_f32_kernel, dim3(ceil_div(dim, 256)), dim3(256), 0, false, m->x,
                                   (const float*)m->partial, dim)))
                    return rc;
            } else {
                p.out[0] = m->x;
                if ((rc = launch_matvec(ctx, Fmt::Int4, Epi::Residual, Pro::Plain, pl_o, p, pdl))) return rc;
            }
        }
        {   // 4. rmsnorm + gate/up + swiglu (:179-181)
            MatVecParams p{};
            p.mat[0] = qwp(L.gate); p.mat[1] = qwp(L.up); p.out[0] = m->h;
            p.in = m->x; p.gamma = L.rms_ffn; p.eps = m->eps;
            p.rows = dim; p.cols = m->hidden_local; p.nmat = 2;
            if ((rc = launch_matvec(ctx, Fmt::Int4, Epi::SwiGLU, Pro::RMSNorm, pl_gu, p, pdl && m->tp == 1))) return rc;
        }
        {   // 5. down + residual (:183)
            MatVecParams p{};
            p.mat[0] = qwp(L.down); p.in = m->h; p.rows = m->hidden_local; p.cols = dim; p.nmat = 1;
            if (m->tp > 1) {
                p.out_f32 = m->partial;
                if ((rc = launch_matvec(ctx, Fmt::Int4, Epi::PartialF32, Pro::Plain, pl_down, p, pdl))) return rc;
                ML2_NCCL(g_nccl.AllReduce(m->partial, m->partial, dim, ncclFloat, ncclSum, m->comm, ctx->stream));
                if ((rc = launch_k(m, "residual_add", residual_add_f32_kernel, dim3(ceil_div(dim, 256)), dim3(256), 0, false, m->x,
                                   (const float*)m->partial, dim)))
                    return rc;
            } else {
                p.out[0] = m->x;
                if ((rc = launch_matvec(ctx, Fmt::Int4, Epi::Residual, Pro::Plain, pl_down, p, pdl))) return rc;
            }
        }
    }
    {   // final rmsnorm + classifier (:187-189)
        MatVecParams p{};
        p.mat[0] = QWPtrs{reinterpret_cast<const uint32_t*>(m->classifier), nullptr, nullptr};
        p.out[0] = m->tp > 1 ? m->logits_local : m->logits;
        p.in = m->x; p.gamma = m->rms_final; p.eps = m->eps;
        p.rows = dim; p.cols = m->vocab_local; p.nmat = 1;
        if ((rc = launch_matvec(ctx, Fmt::F16, Epi::Store, Pro::RMSNorm, pl_cls, p, pdl && m->tp == 1))) return rc;
        if (m->tp > 1)
            ML2_NCCL(g_nccl.AllGather(m->logits_local, m->logits, m->vocab_local, ncclHalf, m->comm, ctx->stream));
    }
    if ((rc = launch_k(m, "argmax", argmax_step_kernel, dim3(1), dim3(1024), 0, m->tp == 1, (const __half*)m->logits, c.vocab_size,
                       m->tokens, (const StepState*)m->step)))
        return rc;
    m->launches_per_token = ctx->launches - before;
    return ML2_OK;
}


// Launches one kernel kind of one layer exactly as the token sequence does (no NCCL, no PDL); used by the
// profiler below. kind: 0 qkv, 1 attention, 2 o-proj, 3 gate/up, 4 down, 5 classifier.
// One kernel of the CUDA-graph path on its own (ml2_model_profile), chained to its predecessor with programmatic
// dependent launch as the token's graph chains them: the weight prefetch of a launch overlaps the tail of the one before.
static int enqueue_kind(Model* m, int kind, int l)
{
    Ctx* ctx = m->ctx;
    const ml2_config& c = m->cfg;
    const int dim = c.dim;
    int rc;
    MatVecPlan pl;
    const size_t kv_layer = (size_t)c.seq_len * m->dim_local;
    const LayerW& L = m->layers[l];
    __half* kc = m->key_cache + (size_t)l * kv_layer;
    __half* vc = m->value_cache + (size_t)l * kv_layer;
    MatVecParams p{};
    switch (kind) {
    case 0:
        if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::QKVRope, dim, m->dim_local, 3, &pl))) return rc;
        p.mat[0] = qwp(L.q); p.mat[1] = qwp(L.k); p.mat[2] = qwp(L.v);
        p.out[0] = m->q; p.out[1] = kc; p.out[2] = vc;
        p.in = m->x; p.gamma = L.rms_att; p.eps = m->eps;
        p.rope_table = m->rope_table; p.pos_ptr = &m->step->pos; p.kv_row_stride = m->dim_local;
        p.rows = dim; p.cols = m->dim_local; p.nmat = 3; p.head_size = m->head_size;
        return launch_matvec(ctx, Fmt::Int4, Epi::QKVRope, Pro::RMSNorm, pl, p, m->use_pdl);
    case 1: {
        AttnParams a{};
        const int chunk_cap = std::max(ceil_div(c.seq_len, kAttnCluster), kAttnSingleCtaMax);
        a.out = m->xb; a.q = m->q; a.k = kc; a.v = vc; a.pos_ptr = &m->step->pos;
        a.n_heads = m->heads_local; a.head_size = m->head_size; a.row_stride = m->dim_local;
        a.scale = 1.0f / sqrtf((float)m->head_size); a.chunk_cap = chunk_cap;
        const bool save = m->use_pdl;
        m->use_pdl = false;
        rc = launch_k(m, "attention", fused_attention_kernel, dim3(m->heads_local * kAttnCluster), dim3(kAttnThreads),
                      (size_t)chunk_cap * sizeof(float), false, a);
        m->use_pdl = save;
        return rc;
    }
    case 2:
    case 4: {
        const int rows = kind == 2 ? m->dim_local : m->hidden_local;
        const Epi e = m->tp > 1 ? Epi::PartialF32 : Epi::Residual;
        if ((rc = plan_matvec(ctx, Fmt::Int4, e, rows, dim, 1, &pl))) return rc;
        p.mat[0] = qwp(kind == 2 ? L.o : L.down); p.in = kind == 2 ? m->xb : m->h; p.rows = rows; p.cols = dim; p.nmat = 1;
        p.out[0] = m->x; p.out_f32 = m->partial;
        return launch_matvec(ctx, Fmt::Int4, e, Pro::Plain, pl, p, m->use_pdl);
    }
    case 3:
        if ((rc = plan_matvec(ctx, Fmt::Int4, Epi::SwiGLU, dim, m->hidden_local, 2, &pl))) return rc;
        p.mat[0] = qwp(L.gate); p.mat[1] = qwp(L.up); p.out[0] = m->h;
        p.in = m->x; p.gamma = L.rms_ffn; p.eps = m->eps;
        p.rows = dim; p.cols = m->hidden_local; p.nmat = 2;
        return launch_matvec(ctx, Fmt::Int4, Epi::SwiGLU, Pro::RMSNorm, pl, p, m->use_pdl);
    case 5:
        if ((rc = plan_matvec(ctx, Fmt::F16, Epi::Store, dim, m->vocab_local, 1, &pl))) return rc;
        p.mat[0] = QWPtrs{reinterpret_cast<const uint32_t*>(m->classifier), nullptr, nullptr};
        p.out[0] = m->tp > 1 ? m->logits_local : m->logits;
        p.in = m->x; p.gamma = m->rms_final; p.eps = m->eps;
        p.rows = dim; p.cols = m->vocab_local; p.nmat = 1;
        return launch_matvec(ctx, Fmt::F16, Epi::Store, Pro::RMSNorm, pl, p, m->use_pdl);
    }
    return fail(ML2_E_INVALID, "profile: kind %d", kind);
}

static double qweight_bytes(int rows, int cols)
{
    const int ss = ceil_div(rows, kGroup), ws = ceil_div(rows, 32) * 4, zs = ceil_div(ss, 8);
    return (double)cols * (ws * 4.0 + zs * 4.0 + ss * 2.0);
}

// ---- persistent per-token kernel: operator list and launch ------------------------------------------------------
// Plans one weight operator for a ring slot of `slot_bytes`: lane mapping (warps per group, groups, weight vectors per
// lane), the alignment granule of its rows and the rows of a full tile.
static bool mega_plan_op(MegaOp& op, int fmt, int rows, int cols, int nmat, bool paired, int slot_bytes)
{
    op.fmt = fmt;
    op.rows = rows;
    op.cols = cols;
    op.nmat = nmat;
    op.paired = paired ? 1 : 0;
    op.tp = 1;
    op.has_tiles = 1;
    if (fmt == 0) {
        if (rows % 32) return false;
        const int ssize = ceil_div(rows, kGroup), wsize = ceil_div(rows, 32) * 4, zsize = ceil_div(ssize, 8);
        op.wrow = wsize * 4;
        op.zrow = zsize * 4;
        op.srow = ssize * 2;
        op.units = wsize / 4;
    } else {
        if (rows % 8 || paired) return false;
        op.wrow = rows * 2;
        op.zrow = op.srow = 0;
        op.units = rows / 8;
    }
    // every bulk copy of a tile (rows x bytes per row, in each of the three arrays) must be a multiple of 16 bytes
    auto rows_for_16 = [](int row_bytes) {
        int n = 1;
        while ((n * row_bytes) % 16) n *= 2;
        return n;
    };
    op.gran = std::max(rows_for_16(op.wrow), std::max(op.zrow ? rows_for_16(op.zrow) : 1, op.srow ? rows_for_16(op.srow) : 1));
    if (cols % op.gran) return false;
    const int nruns = paired ? 2 : 1;
    auto a16 = [](int b) { return (b + 15) & ~15; };
    auto tile_bytes = [&](int units) { return nruns * (units * op.wrow + a16(units * op.zrow) + a16(units * op.srow)); };
    auto set_layout = [&](int rmax) {
        op.rmax = rmax;
        op.off_z = rmax * op.wrow;
        op.off_s = op.off_z + a16(rmax * op.zrow);
        op.run_bytes = op.off_s + a16(rmax * op.srow);
    };
    if (fmt == 0) {
        // int4 on the tensor cores: every working warp takes `np` whole quantisation groups of all rows of a tile; a
        // full tile is one or two blocks of 8 rows (SwiGLU: 8 gate rows and the 8 matching up rows)
        if (rows % kGroup) return false;
        op.ngrp = rows / kGroup;
        op.np = std::max(2, ceil_div(op.ngrp, kMegaConsumerWarps));   // two groups per warp keep the inputs in registers
        op.kw = ceil_div(op.ngrp, op.np);
        op.groups = 1;
        op.tab_n = (op.ngrp * 4 + 7) & ~7;
        int rmax = 0;
        for (int r = paired ? 8 : 16; r >= 8 && !rmax; r -= 8)
            if (r % op.gran == 0 && tile_bytes(r) <= slot_bytes) rmax = r;
        if (!rmax) return false;
        op.two = (paired || rmax == 16) ? 1 : 0;
        set_layout(rmax);
        return true;
    }
    // Lane mapping: a group of kw warps spans a row with np weight vectors per lane; G groups share every tile. The
    // best mapping keeps the most lanes busy: (row coverage) x (warps in a group).
    op.kw = 0;
    double best = -1.0;
    for (int np = 1; np <= 2; ++np) {
        const int kw = ceil_div(op.units, 32 * np);
        if (kw > kMegaConsumerWarps) continue;
        const int groups = std::min(kMegaMaxGroups, kMegaConsumerWarps / kw);
        const double score = (double)op.units / (kw * 32.0 * np) * (double)(groups * kw) / kMegaConsumerWarps;
        if (score > best + 1e-9 || (score > best - 1e-9 && groups > op.groups)) {
            best = std::max(best, score);
            op.kw = kw;
            op.np = np;
            op.groups = groups;
        }
    }
    if (op.kw == 0) return false;
    // Rows of a full tile: whole batches for every group (a batch is 4 / np physical rows of a group), whole granules,
    // at most kMegaGroupRows physical rows per group, and the tile has to fit the slot.
    const int batch_units = std::max(1, (4 / op.np) / nruns);
    int step = op.groups * batch_units;
    step = step / std::__gcd(step, op.gran) * op.gran;
    const int cap_units = op.groups * (kMegaGroupRows / nruns);
    int rmax = 0;
    for (int r = step; r <= cap_units && tile_bytes(r) <= slot_bytes; r += step) rmax = r;
    if (rmax == 0) {
        // a whole batch step does not fit: fall back to as many granules as do (groups then share a tile unevenly)
        for (int r = op.gran; r <= cap_units && tile_bytes(r) <= slot_bytes; r += op.gran) rmax = r;
    }
    if (rmax == 0) return false;
    op.tab_n = op.kw * 32 * op.np;
    set_layout(rmax);
    return true;
}

// The tiles of operator k on one CTA, appended to `out`. The operator's output rows (QKV: the rows of q, k and v one
// after the other) are cut into contiguous, balanced ranges of alignment granules, one per CTA (which CTAs get one granule
// more rotates from operator to operator). A range is streamed as full tiles followed by one remainder tile; a tile never
// spans two matrices. (int4: every tile costs the arithmetic of a full one, or of half a one up to 8 rows, so a range is
// best cut into as few tiles as possible.)
static void mega_tiles_of(const MegaOp& op, int k, int cta, int ncta, std::vector<MegaTile>& out)
{
    const int nseg = op.paired ? 1 : op.nmat, nruns = op.paired ? 2 : 1;
    const size_t first = out.size();
    const bool shared_counter = (op.kind == MOP_PARTIAL || op.kind == MOP_CLS) && op.tp > 1;
    const int c = (cta + op.rot) % ncta;
    const long long G = (long long)op.ngran * nseg;   // granules of all segments
    const long long g0 = c * G / ncta, g1 = (c + 1) * G / ncta;
    for (int seg = 0; seg < nseg; ++seg) {
        const long long s0 = std::max<long long>(g0, (long long)seg * op.ngran), s1 = std::min<long long>(g1, (long long)(seg + 1) * op.ngran);
        if (s1 <= s0) continue;
        int row = (int)(s0 - (long long)seg * op.ngran) * op.gran;
        int left = (int)(s1 - s0);   // granules
        while (left > 0) {
            const int ng = std::min(left, op.gmax);
            const int n = ng * op.gran;
            MegaTile T{};
            T.row = row;
            T.n = n;
            T.info = (uint32_t)k | ((uint32_t)seg << 16) | ((op.kind == MOP_QKV && seg > 0) ? kTileCacheRow : 0u);
            T.out = op.out[op.kind == MOP_QKV ? seg : 0];
            T.opbits = (uint32_t)op.kind | (op.paired ? 8u : 0u) | (op.fmt == 0 ? 16u : 0u) | (shared_counter ? 32u : 0u) |
                       ((uint32_t)op.kw << 8) | ((uint32_t)op.groups << 16);
            for (int r = 0; r < nruns; ++r) {
                const QWPtrs& q = op.mat[op.paired ? r : seg];
                const unsigned char* src[3] = {reinterpret_cast<const unsigned char*>(q.w), reinterpret_cast<const unsigned char*>(q.z),
                                               reinterpret_cast<const unsigned char*>(q.s)};
                const int row_bytes[3] = {op.wrow, op.zrow, op.srow}, dst[3] = {0, op.off_z, op.off_s};
                for (int part = 0; part < 3; ++part) {
                    if (!src[part] || !row_bytes[part]) continue;
                    MegaTileCopy& e = T.cp[r * 3 + part];
                    e.src = src[part] + (size_t)row * row_bytes[part];
                    e.bytes = (uint32_t)(n * row_bytes[part]);
                    e.dst = (uint32_t)(r * op.run_bytes + dst[part]);
                    T.total_bytes += e.bytes;
                }
            }
            out.push_back(T);
            row += n;
            left -= ng;
        }
    }
    if (out.size() > first) out.back().info |= kTileLast;
}

// Layout of the peer-visible communication buffer of one rank (tensor parallel persistent kernel).
struct CommLayout {
    size_t done_off, recv_off, logits_off, x2_off, total;
    int zones;
};
static CommLayout comm_layout(const Model* m)
{
    CommLayout L{};
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t nops = (size_t)5 * m->cfg.n_layers + 2;
    L.zones = 4;
    L.done_off = 0;
    L.recv_off = up(nops * sizeof(unsigned int));
    L.logits_off = L.recv_off + up((size_t)L.zones * m->tp * m->cfg.dim * sizeof(float));
    L.x2_off = L.logits_off + up((size_t)m->cfg.vocab_size * sizeof(__half));
    L.total = L.x2_off + up((size_t)m->cfg.dim * sizeof(__half));
    return L;
}

static int build_mega(Model* m)
{
    m->mega_built = true;
    m->mega_ok = false;
    if (!m->use_mega) return ML2_OK;
    const bool tp = m->tp > 1;
    if (tp && !m->comm_attached) return ML2_OK;   // without peer memory the graph + NCCL path is used
    const ml2_config& c = m->cfg;
    const int dim = c.dim, hs = m->head_size;
    if (m->heads_local > m->ctx->sm_count || hs != kHeadMax || m->tp > 8) return ML2_OK;
    if (dim > 8 * kMegaNormVecs * kMegaConsThreads) return ML2_OK;   // a normalised input vector is held in registers by the CTA
    const CommLayout CL = comm_layout(m);
    auto peer = [&](int q, size_t off) { return static_cast<unsigned char*>(m->comm_peer[q]) + off; };
    const size_t kv_layer = (size_t)c.seq_len * m->dim_local;
    // split attention: scratch for the exchange between the parts of a head, and the counters of their arrivals
    const int split = std::min(kMegaMaxSplit, m->ctx->sm_count / std::max(1, m->heads_local));
    if (!m->att_ml) {
        ML2_CUDA(cudaMalloc(&m->att_ml, (size_t)m->heads_local * kMegaMaxSplit * 2 * sizeof(float)));
        ML2_CUDA(cudaMalloc(&m->att_part, (size_t)m->heads_local * kMegaMaxSplit * hs * sizeof(float)));
        ML2_CUDA(cudaMalloc(&m->att_cnt, (size_t)m->heads_local * sizeof(unsigned int)));
        m->owned.push_back(m->att_ml);
        m->owned.push_back(m->att_part);
        m->owned.push_back(m->att_cnt);
    }
    ML2_CUDA(cudaMemsetAsync(m->att_cnt, 0, (size_t)m->heads_local * sizeof(unsigned int), m->stream));
    m->att_seq = 0;

    // The operator list for a ring slot of `slot_bytes`; false when some operator cannot be planned.
    std::vector<MegaOp> ops;
    auto plan_all = [&](int slot_bytes) -> bool {
        ops.clear();
        int rot = 0;
        auto push = [&](MegaOp& op) {
            op.rot = rot % m->ctx->sm_count;
            rot += 37;   // the CTAs that own one granule more than the others change from operator to operator
            if (op.has_tiles) {
                op.ngran = op.cols / op.gran;
                op.gmax = op.rmax / op.gran;
            }
            ops.push_back(op);
        };
        // residual stream: in place on one GPU; under tensor parallelism the update happens in the next norm
        // operator's prologue and ping-pongs between two buffers (readers of the old one may still be running)
        __half* x_cur = m->x;
        __half* x_alt = tp ? reinterpret_cast<__half*>(peer(m->rank, CL.x2_off)) : nullptr;
        int partial_ordinal = 0;
        const float* pending_recv = nullptr;   // receive zone holding the partials not yet folded into x
        auto norm_input = [&](MegaOp& op, const __half* gamma, bool first) {
            op.gamma = gamma;
            if (first) { op.pro = 2; op.in = x_cur; return; }
            if (tp) {
                op.pro = 3; op.tp = m->tp; op.in = x_cur; op.recv = pending_recv; op.x_next = x_alt;
                std::swap(x_cur, x_alt);
            } else {
                op.pro = 1; op.in = x_cur;
            }
        };
        auto partial_output = [&](MegaOp& op, int k_index) {
            op.kind = MOP_PARTIAL;
            op.tp = m->tp;
            const size_t zone = (size_t)(partial_ordinal % CL.zones) * m->tp * dim * sizeof(float);
            for (int q = 0; q < m->tp; ++q) {
                op.peer_out[q] = reinterpret_cast<float*>(peer(q, CL.recv_off + zone + (size_t)m->rank * dim * sizeof(float)));
                op.peer_done[q] = reinterpret_cast<unsigned int*>(peer(q, CL.done_off)) + k_index;
            }
            pending_recv = reinterpret_cast<const float*>(peer(m->rank, CL.recv_off + zone));
            ++partial_ordinal;
        };
        for (int l = 0; l < c.n_layers; ++l) {
            const LayerW& L = m->layers[l];
            __half* kc = m->key_cache + (size_t)l * kv_layer;
            __half* vc = m->value_cache + (size_t)l * kv_layer;
            MegaOp q{};
            q.kind = MOP_QKV;
            if (!mega_plan_op(q, 0, dim, m->dim_local, 3, false, slot_bytes)) return false;
            norm_input(q, L.rms_att, l == 0);
            q.mat[0] = qwp(L.q); q.mat[1] = qwp(L.k); q.mat[2] = qwp(L.v);
            q.out[0] = m->q; q.out[1] = kc; q.out[2] = vc;
            push(q);
            MegaOp a{};
            a.kind = MOP_ATTN; a.tp = 1; a.in = m->q; a.out[0] = m->xb; a.kcache = kc; a.vcache = vc;
            a.att_ml = m->att_ml; a.att_part = m->att_part; a.att_cnt = m->att_cnt; a.att_layer = l;
            push(a);
            MegaOp o{};
            o.kind = MOP_RESID; o.pro = 0;
            if (!mega_plan_op(o, 0, m->dim_local, dim, 1, false, slot_bytes)) return false;
            o.mat[0] = qwp(L.o); o.out[0] = x_cur; o.in = m->xb;
            o.att_part = m->att_part;   // input of the split attention path: partial outputs summed in the prologue
            if (tp) partial_output(o, (int)ops.size());
            push(o);
            MegaOp g{};
            g.kind = MOP_SWIGLU;
            if (!mega_plan_op(g, 0, dim, m->hidden_local, 2, true, slot_bytes)) return false;
            norm_input(g, L.rms_ffn, false);
            g.mat[0] = qwp(L.gate); g.mat[1] = qwp(L.up); g.out[0] = m->h;
            push(g);
            MegaOp d{};
            d.kind = MOP_RESID; d.pro = 0;
            if (!mega_plan_op(d, 0, m->hidden_local, dim, 1, false, slot_bytes)) return false;
            d.mat[0] = qwp(L.down); d.out[0] = x_cur; d.in = m->h;
            if (tp) partial_output(d, (int)ops.size());
            push(d);
        }
        MegaOp cl{};
        cl.kind = MOP_CLS;
        if (!mega_plan_op(cl, 1, dim, m->vocab_local, 1, false, slot_bytes)) return false;
        norm_input(cl, m->rms_final, false);
        cl.mat[0] = QWPtrs{reinterpret_cast<const uint32_t*>(m->classifier), nullptr, nullptr};
        cl.out[0] = m->logits;
        if (tp) {
            cl.tp = m->tp;   // (norm_input set it already for the input side)
            cl.out_row0 = m->vocab_row0;
            for (int q = 0; q < m->tp; ++q) {
                cl.peer_logits[q] = reinterpret_cast<__half*>(peer(q, CL.logits_off));
                cl.peer_done[q] = reinterpret_cast<unsigned int*>(peer(q, CL.done_off)) + (int)ops.size();
            }
            m->logits_view = reinterpret_cast<__half*>(peer(m->rank, CL.logits_off));
        } else {
            m->logits_view = m->logits;
        }
        push(cl);
        MegaOp am{};
        am.kind = MOP_ARGMAX; am.tp = 1;
        push(am);
        return true;
    };

    // everything the opt-in limit of one CTA leaves after the kernel's static shared memory (1 KB kept spare)
    int optin = 0;
    ML2_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, m->ctx->device));
    cudaFuncAttributes fa{};
    ML2_CUDA(cudaFuncGetAttributes(&fa, decode_token_kernel<true>));
    const int budget = optin - (int)fa.sharedSizeBytes - 1024;
    if (!plan_all(budget)) return ML2_OK;   // lane mappings do not depend on the slot size
    // scratch beside the ring: the prepared input table of a weight operator, or the attention's scores and partial outputs
    int scratch = c.seq_len * 4 + kMegaConsumerWarps * kHeadMax * 4;
    for (const MegaOp& op : ops) {
        if (!op.has_tiles) continue;
        const int tab_n = op.tab_n;
        scratch = std::max(scratch, op.fmt == 0 ? tab_n * 4 * 16 + (tab_n / 4) * 16 : tab_n * 16);
        if (op.pro != 0 && (op.fmt == 0 ? tab_n * 4 : tab_n) > kMegaNormVecs * kMegaConsThreads) return ML2_OK;
    }
    scratch = (scratch + 127) & ~127;
    int nstage = 0, slot = 0;
    for (int ns = 4; ns >= 2 && !nstage; --ns) {
        const int sb = ((budget - scratch) / ns) & ~127;
        if (sb < 1024 || !plan_all(sb)) continue;
        // the slot needs no more than the largest tile
        int need = 0;
        for (const MegaOp& op : ops)
            if (op.has_tiles) need = std::max(need, (op.paired ? 2 : 1) * op.run_bytes);
        nstage = ns;
        slot = std::min(sb, (need + 127) & ~127);
    }
    if (!nstage) return ML2_OK;
    // every array a tile is copied from must be 16-byte aligned (the rows of a tile start at a whole granule)
    for (const MegaOp& op : ops) {
        if (!op.has_tiles) continue;
        for (int q = 0; q < op.nmat; ++q) {
            const uintptr_t bits = reinterpret_cast<uintptr_t>(op.mat[q].w) | reinterpret_cast<uintptr_t>(op.mat[q].z) |
                                   reinterpret_cast<uintptr_t>(op.mat[q].s);
            if (bits & 15u) return ML2_OK;
        }
    }
    m->att_split = split >= 2 ? split : 1;
    m->mega_slot = slot;
    m->mega_nstage = nstage;
    m->mega_att_bytes = scratch;
    m->mega_smem = nstage * slot + scratch;
    m->mega_nops = (int)ops.size();
    m->mega_grid = m->ctx->sm_count;
    ML2_CUDA(cudaFuncSetAttribute(decode_token_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, m->mega_smem));
    ML2_CUDA(cudaFuncSetAttribute(decode_token_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, m->mega_smem));
    int per_sm = 0;
    ML2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_token_kernel<false>, kMegaThreads, m->mega_smem));
    if (per_sm < 1) return ML2_OK;
    if (ops.size() > 0xffffu) return ML2_OK;
    if (m->mega_ops) { cudaFree(m->mega_ops); m->mega_ops = nullptr; }
    ML2_CUDA(cudaMalloc(&m->mega_ops, ops.size() * sizeof(MegaOp)));
    ML2_CUDA(cudaMemcpyAsync(m->mega_ops, ops.data(), ops.size() * sizeof(MegaOp), cudaMemcpyHostToDevice, m->stream));
    // every CTA's tile list and its tile counts per operator
    {
        const int ncta = m->mega_grid;
        std::vector<MegaTile> tiles;
        std::vector<int> begin(ncta + 1, 0);
        std::vector<unsigned short> per_op(ops.size() * (size_t)ncta, 0);
        for (int c = 0; c < ncta; ++c) {
            begin[c] = (int)tiles.size();
            for (size_t k = 0; k < ops.size(); ++k) {
                if (!ops[k].has_tiles) continue;
                const size_t before = tiles.size();
                mega_tiles_of(ops[k], (int)k, c, ncta, tiles);
                if (tiles.size() - before > 0xffffu) return ML2_OK;
                per_op[k * ncta + c] = (unsigned short)(tiles.size() - before);
            }
        }
        begin[ncta] = (int)tiles.size();
        for (const MegaTile& T : tiles)
            for (const MegaTileCopy& e : T.cp)
                if ((reinterpret_cast<uintptr_t>(e.src) & 15u) || (e.bytes & 15u) || (e.dst & 15u)) return ML2_OK;   // bulk copies: 16-byte rule
        if (m->mega_tiles) { cudaFree(m->mega_tiles); m->mega_tiles = nullptr; }
        if (m->mega_tile_begin) { cudaFree(m->mega_tile_begin); m->mega_tile_begin = nullptr; }
        if (m->mega_op_tiles) { cudaFree(m->mega_op_tiles); m->mega_op_tiles = nullptr; }
        ML2_CUDA(cudaMalloc(&m->mega_tiles, std::max<size_t>(1, tiles.size()) * sizeof(MegaTile)));
        ML2_CUDA(cudaMalloc(&m->mega_tile_begin, begin.size() * sizeof(int)));
        ML2_CUDA(cudaMalloc(&m->mega_op_tiles, per_op.size() * sizeof(unsigned short)));
        ML2_CUDA(cudaMemcpy(m->mega_tiles, tiles.data(), tiles.size() * sizeof(MegaTile), cudaMemcpyHostToDevice));
        ML2_CUDA(cudaMemcpy(m->mega_tile_begin, begin.data(), begin.size() * sizeof(int), cudaMemcpyHostToDevice));
        ML2_CUDA(cudaMemcpy(m->mega_op_tiles, per_op.data(), per_op.size() * sizeof(unsigned short), cudaMemcpyHostToDevice));
    }
    if (tp) {
        m->mega_done_ptr = reinterpret_cast<unsigned int*>(peer(m->rank, CL.done_off));   // zeroed when the buffer was made
    } else {
        if (!m->mega_done) ML2_CUDA(cudaMalloc(&m->mega_done, ops.size() * sizeof(unsigned int)));
        ML2_CUDA(cudaMemsetAsync(m->mega_done, 0, ops.size() * sizeof(unsigned int), m->stream));
        m->mega_done_ptr = m->mega_done;
        m->mega_seq = 0;
    }
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    if (m->want_prof && !m->mega_prof) {
        ML2_CUDA(cudaMalloc(&m->mega_prof, (size_t)m->mega_grid * 64 * sizeof(long long)));
        ML2_CUDA(cudaMemset(m->mega_prof, 0, (size_t)m->mega_grid * 64 * sizeof(long long)));
    }
    m->mega_ok = true;
    return ML2_OK;
}

static int forward_mega(Model* m, int pos, int next_pos, int write_token)
{
    MegaParams prm{};
    prm.ops = m->mega_ops;
    prm.nops = m->mega_nops;
    prm.tiles = m->mega_tiles;
    prm.tile_begin = m->mega_tile_begin;
    prm.op_tiles = m->mega_op_tiles;
    prm.done = m->mega_done_ptr;
    prm.status = m->ctx->status_dev;
    prm.rope_table = m->rope_table;
    prm.embed = m->embed;
    prm.x = m->x;
    prm.tokens = m->tokens;
    prm.logits = m->logits_view;
    prm.pos = pos; prm.next_pos = next_pos; prm.write_token = write_token;
    prm.seq_no = ++m->mega_seq;
    prm.dim = m->cfg.dim; prm.head_size = m->head_size; prm.heads_local = m->heads_local;
    prm.kv_row_stride = m->dim_local; prm.vocab = m->cfg.vocab_size;
    prm.eps = m->eps; prm.scale = 1.0f / sqrtf((float)m->head_size);
    prm.nstage = m->mega_nstage; prm.slot_bytes = m->mega_slot; prm.att_cap = m->cfg.seq_len;
    prm.prof = m->mega_prof;
    prm.n_layers = m->cfg.n_layers;
    prm.att_split = (m->att_split > 1 && pos + 1 >= m->att_min_seq) ? m->att_split : 1;
    prm.att_seq = prm.att_split > 1 ? ++m->att_seq : m->att_seq;
    prm.wait_cycles = m->ctx->wait_cycles;
    void* args[] = {&prm};
    const void* fn = m->mega_prof ? (const void*)decode_token_kernel<true> : (const void*)decode_token_kernel<false>;
    ML2_CUDA(cudaLaunchCooperativeKernel(fn, dim3(m->mega_grid), dim3(kMegaThreads), args, (size_t)m->mega_smem, m->stream));
    ++m->ctx->launches;
    m->launches_per_token = 1;
    return ML2_OK;
}

// Reads the device error word together with whatever the caller just synchronised on. A kernel whose bounded wait ran
// out leaves garbage behind and the monotonic counters mid-token: the model refuses further forwards until it is reset.
static int check_device_status(Model* m)
{
    DeviceStatus st{};
    ML2_CUDA(cudaMemcpyAsync(&st, m->ctx->status_dev, sizeof(st), cudaMemcpyDeviceToHost, m->stream));
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    if (st.error) {
        m->poisoned = true;
        return fail(ML2_E_DEVICE, "a kernel gave up waiting (code %u, operator %u); call ml2_model_reset before the next forward", st.error, st.detail);
    }
    return ML2_OK;
}

static int check_bound(Model* m)
{
    if (!m->embed || !m->classifier || !m->rms_final) return fail(ML2_E_STATE, "model: globals are not bound");
    for (size_t l = 0; l < m->layers.size(); ++l)
        if (!m->layers[l].bound) return fail(ML2_E_STATE, "model: layer %zu is not bound", l);
    if (!m->x) return fail(ML2_E_STATE, "model: run state is not allocated or bound");
    return ML2_OK;
}

}  // namespace ml2

using namespace ml2;

extern "C" {

int ml2_nccl_unique_id(void* out128)
{
    if (!out128) return fail(ML2_E_INVALID, "ml2_nccl_unique_id: null buffer");
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    int rc = nccl_load();
    if (rc) return rc;
    ncclUniqueId id;
    ML2_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return ML2_OK;
}

int ml2_model_create(ml2_ctx* h, const ml2_config* cfg, int tp_size, int tp_rank, const void* nccl_id128, ml2_model** out)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !cfg || !out) return fail(ML2_E_INVALID, "ml2_model_create: null argument");
    const ml2_config& c = *cfg;
    if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.vocab_size <= 0 || c.seq_len <= 0)
        return fail(ML2_E_INVALID, "ml2_model_create: non-positive config field");
    if (c.n_kv_heads != c.n_heads)
        return fail(ML2_E_INVALID, "grouped-query attention (numKVHeads != numHeads) is not supported, as in the reference");
    if (c.dim % c.n_heads) return fail(ML2_E_INVALID, "dim %d is not a multiple of n_heads %d", c.dim, c.n_heads);
    const int hs = c.dim / c.n_heads;
    if (hs != kHeadMax) return fail(ML2_E_INVALID, "head size %d: the fused path supports 128 only", hs);
    if (c.dim % kGroup || c.hidden_dim % kGroup) return fail(ML2_E_INVALID, "dim and hidden_dim must be multiples of 128");
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail(ML2_E_INVALID, "tp_size=%d tp_rank=%d", tp_size, tp_rank);
    if (c.n_heads % tp_size) return fail(ML2_E_INVALID, "n_heads %d is not divisible by tp %d", c.n_heads, tp_size);
    if (c.vocab_size % tp_size) return fail(ML2_E_INVALID, "vocab_size %d is not divisible by tp %d", c.vocab_size, tp_size);
    if (tp_size > 1 && !nccl_id128) return fail(ML2_E_INVALID, "tp > 1 needs the shared NCCL unique id");

    ML2_CUDA(cudaSetDevice(ctx->device));
    Model* m = new Model();
    m->ctx = ctx;
    m->cfg = c;
    m->tp = tp_size;
    m->rank = tp_rank;
    m->head_size = hs;
    m->heads_local = c.n_heads / tp_size;
    m->dim_local = m->heads_local * hs;
    int g0, ng;
    ml2_tp_hidden_groups(c.hidden_dim, tp_size, tp_rank, &g0, &ng);
    m->hidden_local = ng * kGroup;
    m->vocab_local = c.vocab_size / tp_size;
    m->vocab_row0 = m->vocab_local * tp_rank;
    m->layers.resize(c.n_layers);
    const char* eg = getenv("ML2_NO_GRAPH");
    m->use_graph = !(eg && *eg == '1');
    const char* em = getenv("ML2_NO_MEGA");
    m->use_mega = !(em && *em == '1');
    const char* ep = getenv("ML2_NO_PDL");
    m->use_pdl = !(ep && *ep == '1');
    const char* epf = getenv("ML2_MEGA_PROF");
    m->want_prof = epf && *epf == '1';
    cudaStream_t caller_stream = ctx->stream;
    // everything below may fail half way: one exit that frees what was made and gives the caller's stream back
    auto build = [&]() -> int {
        ML2_CUDA(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
        ctx->stream = m->stream;
        int rc;
        if ((rc = dev_alloc(m, (void**)&m->step, sizeof(StepState)))) return rc;
        if ((rc = dev_alloc(m, (void**)&m->rope_table, (size_t)c.seq_len * (hs / 2) * sizeof(float2)))) return rc;
        rope_table_kernel<<<ceil_div(c.seq_len * (hs / 2), 256), 256, 0, m->stream>>>(m->rope_table, c.seq_len, hs, c.rope_theta);
        ++ctx->launches;
        if (tp_size > 1) {
            if ((rc = dev_alloc(m, (void**)&m->partial, (size_t)c.dim * sizeof(float)))) return rc;
            if ((rc = dev_alloc(m, (void**)&m->logits_local, (size_t)m->vocab_local * sizeof(__half)))) return rc;
            {   // peer-visible buffer of the persistent kernel (counters, receive zones, logits, second residual buffer)
                const CommLayout CL = comm_layout(m);
                ML2_CUDA(cudaMalloc(&m->comm_local, CL.total));
                ML2_CUDA(cudaMemsetAsync(m->comm_local, 0, CL.total, m->stream));
            }
            if ((rc = nccl_load())) return rc;
            ncclUniqueId id;
            memcpy(&id, nccl_id128, sizeof(id));
            ML2_NCCL(g_nccl.CommInitRank(&m->comm, tp_size, id, tp_rank));
        }
        ML2_CUDA(cudaStreamSynchronize(m->stream));
        return ML2_OK;
    };
    const int rc = build();
    if (rc) {
        char keep[512];
        snprintf(keep, sizeof(keep), "%s", ml2_last_error());
        ml2_model_destroy(reinterpret_cast<ml2_model*>(m));
        ctx->stream = caller_stream;
        return fail(rc, "%s", keep);
    }
    *out = reinterpret_cast<ml2_model*>(m);
    return ML2_OK;
}

void ml2_tp_hidden_groups(int hidden_dim, int tp_size, int tp_rank, int* g0, int* ngroups)
{
    // whole groups of 128, the first (groups % tp) ranks take one more
    const int groups = hidden_dim / kGroup;
    const int base = groups / tp_size, extra = groups % tp_size;
    const int n = base + (tp_rank < extra ? 1 : 0);
    const int start = tp_rank * base + (tp_rank < extra ? tp_rank : extra);
    if (g0) *g0 = start;
    if (ngroups) *ngroups = n;
}

int ml2_model_destroy(ml2_model* h)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return ML2_OK;
    cudaSetDevice(m->ctx->device);
    if (m->stream) cudaStreamSynchronize(m->stream);
    if (m->exec) cudaGraphExecDestroy(m->exec);
    if (m->graph) cudaGraphDestroy(m->graph);
    if (m->comm) g_nccl.CommDestroy(m->comm);
    for (int q = 0; q < m->tp; ++q)
        if (m->comm_attached && q != m->rank && m->comm_peer[q]) cudaIpcCloseMemHandle(m->comm_peer[q]);
    if (m->comm_local) cudaFree(m->comm_local);
    if (m->mega_ops) cudaFree(m->mega_ops);
    if (m->mega_tiles) cudaFree(m->mega_tiles);
    if (m->mega_tile_begin) cudaFree(m->mega_tile_begin);
    if (m->mega_op_tiles) cudaFree(m->mega_op_tiles);
    if (m->mega_done) cudaFree(m->mega_done);
    for (void* p : m->owned) cudaFree(p);
    if (m->ctx->stream == m->stream) m->ctx->stream = nullptr;
    if (m->stream) cudaStreamDestroy(m->stream);
    delete m;
    return ML2_OK;
}

int ml2_model_local_shape(ml2_model* h, int* dim_local, int* hidden_local, int* vocab_local, int* hidden_group0, int* vocab_row0)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    int g0, ng;
    ml2_tp_hidden_groups(m->cfg.hidden_dim, m->tp, m->rank, &g0, &ng);
    if (dim_local) *dim_local = m->dim_local;
    if (hidden_local) *hidden_local = m->hidden_local;
    if (vocab_local) *vocab_local = m->vocab_local;
    if (hidden_group0) *hidden_group0 = g0;
    if (vocab_row0) *vocab_row0 = m->vocab_row0;
    return ML2_OK;
}

int ml2_model_bind_globals(ml2_model* h, const void* embed, const void* classifier_local, const void* rms_final)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !embed || !classifier_local || !rms_final) return fail(ML2_E_INVALID, "bind_globals: null argument");
    if ((reinterpret_cast<uintptr_t>(classifier_local) & 15u) || (reinterpret_cast<uintptr_t>(rms_final) & 15u))
        return fail(ML2_E_INVALID, "bind_globals: classifier and norm weights must be 16-byte aligned");
    m->embed = static_cast<const __half*>(embed);
    m->classifier = static_cast<const __half*>(classifier_local);
    m->rms_final = static_cast<const __half*>(rms_final);
    return ML2_OK;
}

int ml2_model_bind_layer(ml2_model* h, int layer, const ml2_layer_weights* w)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !w) return fail(ML2_E_INVALID, "bind_layer: null argument");
    if (layer < 0 || layer >= m->cfg.n_layers) return fail(ML2_E_INVALID, "bind_layer: layer %d out of range", layer);
    const ml2_qweight* all[7] = {&w->query, &w->key, &w->value, &w->output, &w->gate, &w->up, &w->down};
    for (const ml2_qweight* q : all) {
        if (!q->weight || !q->zeros || !q->scales) return fail(ML2_E_INVALID, "bind_layer: null QWeight array");
        if ((reinterpret_cast<uintptr_t>(q->weight) & 15u) || (reinterpret_cast<uintptr_t>(q->zeros) & 15u) ||
            (reinterpret_cast<uintptr_t>(q->scales) & 15u))
            return fail(ML2_E_INVALID, "bind_layer: QWeight arrays must be 16-byte aligned");
    }
    if (!w->rms_attention || !w->rms_feed_forward || (reinterpret_cast<uintptr_t>(w->rms_attention) & 15u) ||
        (reinterpret_cast<uintptr_t>(w->rms_feed_forward) & 15u))
        return fail(ML2_E_INVALID, "bind_layer: norm weights must be non-null and 16-byte aligned");
    LayerW& L = m->layers[layer];
    L.q = w->query; L.k = w->key; L.v = w->value; L.o = w->output; L.gate = w->gate; L.up = w->up; L.down = w->down;
    L.rms_att = static_cast<const __half*>(w->rms_attention);
    L.rms_ffn = static_cast<const __half*>(w->rms_feed_forward);
    L.bound = true;
    m->mega_built = false;
    if (m->exec) { cudaGraphExecDestroy(m->exec); m->exec = nullptr; }
    return ML2_OK;
}

int ml2_model_alloc_runstate(ml2_model* h)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    if (m->x) return fail(ML2_E_STATE, "run state already present");
    const ml2_config& c = m->cfg;
    int rc;
    const size_t kv = (size_t)c.n_layers * c.seq_len * m->dim_local * sizeof(__half);
    if ((rc = dev_alloc(m, (void**)&m->x, (size_t)c.dim * 2)) || (rc = dev_alloc(m, (void**)&m->xb, (size_t)c.dim * 2)) ||
        (rc = dev_alloc(m, (void**)&m->h, (size_t)c.hidden_dim * 2)) || (rc = dev_alloc(m, (void**)&m->q, (size_t)c.dim * 2)) ||
        (rc = dev_alloc(m, (void**)&m->logits, (size_t)c.vocab_size * 2)) || (rc = dev_alloc(m, (void**)&m->key_cache, kv)) ||
        (rc = dev_alloc(m, (void**)&m->value_cache, kv)) || (rc = dev_alloc(m, (void**)&m->tokens, (size_t)(c.seq_len + 1) * sizeof(int))))
        return rc;
    m->own_state = true;
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    return ML2_OK;
}

int ml2_model_bind_runstate(ml2_model* h, const ml2_runstate* rs)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !rs) return fail(ML2_E_INVALID, "bind_runstate: null argument");
    if (m->own_state) return fail(ML2_E_STATE, "run state already allocated by the library");
    void* all[] = {rs->x, rs->xb, rs->h, rs->q, rs->logits, rs->key_cache, rs->value_cache, rs->tokens};
    for (void* p : all)
        if (!p || (reinterpret_cast<uintptr_t>(p) & 15u)) return fail(ML2_E_INVALID, "bind_runstate: buffers must be non-null and 16-byte aligned");
    m->x = (__half*)rs->x; m->xb = (__half*)rs->xb; m->h = (__half*)rs->h; m->q = (__half*)rs->q; m->logits = (__half*)rs->logits;
    m->key_cache = (__half*)rs->key_cache; m->value_cache = (__half*)rs->value_cache; m->tokens = (int*)rs->tokens;
    m->mega_built = false;
    if (m->exec) { cudaGraphExecDestroy(m->exec); m->exec = nullptr; }
    return ML2_OK;
}

int ml2_model_runstate(ml2_model* h, ml2_runstate* rs)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !rs) return fail(ML2_E_INVALID, "runstate: null argument");
    rs->x = m->x; rs->xb = m->xb; rs->h = m->h; rs->q = m->q; rs->logits = m->logits;
    rs->key_cache = m->key_cache; rs->value_cache = m->value_cache; rs->tokens = m->tokens;
    return ML2_OK;
}

int ml2_model_forward(ml2_model* h, int pos, int next_pos, int write_token)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    int rc = check_bound(m);
    if (rc) return rc;
    if (pos < 0 || pos >= m->cfg.seq_len || next_pos < 0 || next_pos > m->cfg.seq_len)
        return fail(ML2_E_INVALID, "forward: pos=%d next_pos=%d outside [0,%d)", pos, next_pos, m->cfg.seq_len);
    Ctx* ctx = m->ctx;
    if ((rc = use_device(ctx))) return rc;
    if (m->poisoned) return fail(ML2_E_STATE, "forward: an earlier kernel gave up waiting; call ml2_model_reset first");
    ctx->stream = m->stream;
    m->last_pos = pos;
    if (!m->mega_built && (rc = build_mega(m))) return rc;
    if (m->mega_ok) return forward_mega(m, pos, next_pos, write_token);
    if (!m->use_graph) return enqueue_token(m, pos, next_pos, write_token);

    if (!m->exec) {
        if (m->graph) { cudaGraphDestroy(m->graph); m->graph = nullptr; }
        const long long before = ctx->launches;
        ML2_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
        rc = enqueue_token(m, pos, next_pos, write_token);
        cudaGraph_t g = nullptr;
        const cudaError_t e = cudaStreamEndCapture(m->stream, &g);
        ctx->launches = before;  // captured, not launched
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        if (e != cudaSuccess) return fail(ML2_E_CUDA, "graph capture: %s", cudaGetErrorString(e));
        m->graph = g;
        ML2_CUDA(cudaGraphInstantiate(&m->exec, m->graph, 0));
        // the first kernel node carries the step; find it (root node of the captured chain)
        size_t n_roots = 0;
        ML2_CUDA(cudaGraphGetRootNodes(m->graph, nullptr, &n_roots));
        std::vector<cudaGraphNode_t> roots(n_roots);
        ML2_CUDA(cudaGraphGetRootNodes(m->graph, roots.data(), &n_roots));
        m->first_node = nullptr;
        for (cudaGraphNode_t nd : roots) {
            cudaGraphNodeType t;
            ML2_CUDA(cudaGraphNodeGetType(nd, &t));
            if (t == cudaGraphNodeTypeKernel) { m->first_node = nd; break; }
        }
        if (!m->first_node) return fail(ML2_E_CUDA, "graph capture: first kernel node not found");
    }
    // refresh the step carried by the first node, then replay
    cudaKernelNodeParams kp{};
    ML2_CUDA(cudaGraphKernelNodeGetParams(m->first_node, &kp));
    StepState* st = m->step;
    __half* x = m->x;
    const __half* table = m->embed;
    int dim = m->cfg.dim;
    const int* tokens = m->tokens;
    void* args[] = {&st, &pos, &next_pos, &write_token, &x, &table, &dim, &tokens};
    kp.kernelParams = args;
    ML2_CUDA(cudaGraphExecKernelNodeSetParams(m->exec, m->first_node, &kp));
    ML2_CUDA(cudaGraphLaunch(m->exec, m->stream));
    ctx->launches += m->launches_per_token;
    return ML2_OK;
}

long long ml2_model_launches_per_token(ml2_model* h) { return h ? reinterpret_cast<Model*>(h)->launches_per_token : 0; }

int ml2_model_synchronize(ml2_model* h)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    if (int rc = use_device(m->ctx)) return rc;
    return check_device_status(m);
}

int ml2_model_reset(ml2_model* h)
{
    // After ML2_E_DEVICE: waits for whatever is still running, clears the error word and brings every counter the
    // persistent kernel keeps between tokens back to its start (operator arrivals, split-attention arrivals, launch
    // numbers). Under tensor parallelism every rank must call it before any rank runs the next forward: the receive
    // zones and counters of a rank are written by its peers.
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    if (int rc = use_device(m->ctx)) return rc;
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    ML2_CUDA(cudaMemsetAsync(m->ctx->status_dev, 0, sizeof(DeviceStatus), m->stream));
    if (m->mega_done_ptr && m->mega_nops > 0) ML2_CUDA(cudaMemsetAsync(m->mega_done_ptr, 0, (size_t)m->mega_nops * sizeof(unsigned int), m->stream));
    if (m->att_cnt) ML2_CUDA(cudaMemsetAsync(m->att_cnt, 0, (size_t)m->heads_local * sizeof(unsigned int), m->stream));
    m->mega_seq = 0;
    m->att_seq = 0;
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    m->poisoned = false;
    return ML2_OK;
}

static int check_token_ids(const Model* m, const int* ids, int count, const char* what)
{
    for (int i = 0; i < count; ++i)
        if (ids[i] < 0 || ids[i] >= m->cfg.vocab_size)
            return fail(ML2_E_INVALID, "%s: token id %d at index %d is outside the vocabulary [0, %d)", what, ids[i], i, m->cfg.vocab_size);
    return ML2_OK;
}

int ml2_model_set_tokens(ml2_model* h, const int* tokens_host, int first, int count)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !tokens_host) return fail(ML2_E_INVALID, "set_tokens: null argument");
    if (!m->tokens) return fail(ML2_E_STATE, "set_tokens: run state missing");
    if (first < 0 || count < 0 || first + count > m->cfg.seq_len + 1) return fail(ML2_E_INVALID, "set_tokens: range");
    if (int rc = check_token_ids(m, tokens_host, count, "set_tokens")) return rc;
    if (int rc = use_device(m->ctx)) return rc;
    ML2_CUDA(cudaMemcpyAsync(m->tokens + first, tokens_host, (size_t)count * sizeof(int), cudaMemcpyHostToDevice, m->stream));
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    return ML2_OK;
}

int ml2_model_put_token_async(ml2_model* h, int pos, const int* token_pinned_host)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !token_pinned_host) return fail(ML2_E_INVALID, "put_token_async: null argument");
    if (!m->tokens) return fail(ML2_E_STATE, "put_token_async: run state missing");
    if (pos < 0 || pos > m->cfg.seq_len) return fail(ML2_E_INVALID, "put_token_async: pos");
    if (int rc = check_token_ids(m, token_pinned_host, 1, "put_token_async")) return rc;
    if (int rc = use_device(m->ctx)) return rc;
    ML2_CUDA(cudaMemcpyAsync(m->tokens + pos, token_pinned_host, sizeof(int), cudaMemcpyHostToDevice, m->stream));
    return ML2_OK;
}

int ml2_model_step_host(ml2_model* h, int pos, const int* token_in_pinned_host, int* token_out_host)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !token_in_pinned_host || !token_out_host) return fail(ML2_E_INVALID, "step_host: null argument");
    if (pos < 0 || pos + 1 > m->cfg.seq_len) return fail(ML2_E_INVALID, "step_host: pos=%d", pos);
    if (!m->tokens) return fail(ML2_E_STATE, "step_host: run state missing");
    if (int rc0 = check_token_ids(m, token_in_pinned_host, 1, "step_host")) return rc0;
    if (int rc0 = use_device(m->ctx)) return rc0;
    // host -> device: this step's input token; the step; device -> host: the sampled token (the reference's blocking
    // 4-byte read, src/Sampler.cs:69)
    ML2_CUDA(cudaMemcpyAsync(m->tokens + pos, token_in_pinned_host, sizeof(int), cudaMemcpyHostToDevice, m->stream));
    const int rc = ml2_model_forward(h, pos, pos + 1, 1);
    if (rc) return rc;
    ML2_CUDA(cudaMemcpyAsync(token_out_host, m->tokens + pos + 1, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    return check_device_status(m);   // synchronises: the token and the error word arrive together
}

int ml2_model_read_token(ml2_model* h, int pos, int* token_host)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !token_host) return fail(ML2_E_INVALID, "read_token: null argument");
    if (pos < 0 || pos > m->cfg.seq_len) return fail(ML2_E_INVALID, "read_token: pos");
    // the reference's only per-token synchronisation: a 4-byte blocking read (src/Sampler.cs:69)
    if (int rc = use_device(m->ctx)) return rc;
    ML2_CUDA(cudaMemcpyAsync(token_host, m->tokens + pos, sizeof(int), cudaMemcpyDeviceToHost, m->stream));
    return check_device_status(m);
}

int ml2_model_sample(ml2_model* h, int next_pos, float temperature, float top_p, float coin)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "sample: null model");
    if (next_pos < 0 || next_pos > m->cfg.seq_len) return fail(ML2_E_INVALID, "sample: next_pos=%d", next_pos);
    if (!(temperature > 0.f)) return fail(ML2_E_INVALID, "sample: temperature %g (0 is the greedy path of ml2_model_forward)", (double)temperature);
    if (m->cfg.vocab_size > 32768 && !(top_p <= 0.f || top_p >= 1.f))
        return fail(ML2_E_INVALID, "sample: top-p sorting supports vocabularies up to 32768 (this one has %d)", m->cfg.vocab_size);
    ML2_CUDA(cudaSetDevice(m->ctx->device));
    if (!m->sample_indices) {
        ML2_CUDA(cudaMalloc(&m->sample_indices, (size_t)m->cfg.vocab_size * sizeof(int)));   // RunState.indices (src/RunState.cs)
        m->owned.push_back(m->sample_indices);
    }
    __half* lg = (m->mega_ok && m->logits_view) ? m->logits_view : m->logits;
    const int rc = sampler_chain(m->stream, m->ctx->device, lg, m->sample_indices, m->cfg.vocab_size, temperature, top_p, coin, m->tokens, next_pos);
    if (rc == ML2_OK) m->ctx->launches += (top_p <= 0.f || top_p >= 1.f) ? 3 : 4;
    return rc;
}

int ml2_model_read_logits(ml2_model* h, void* logits_host_f16)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !logits_host_f16) return fail(ML2_E_INVALID, "read_logits: null argument");
    const __half* src = (m->mega_ok && m->logits_view) ? m->logits_view : m->logits;
    if (int rc = use_device(m->ctx)) return rc;
    ML2_CUDA(cudaMemcpyAsync(logits_host_f16, src, (size_t)m->cfg.vocab_size * 2, cudaMemcpyDeviceToHost, m->stream));
    return check_device_status(m);
}

int ml2_model_debug_prof(ml2_model* h, long long* out, int n)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !out || !m->mega_prof) return fail(ML2_E_STATE, "no profile buffer (set ML2_MEGA_PROF=1 before the first forward)");
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    ML2_CUDA(cudaMemcpy(out, m->mega_prof, (size_t)std::min(n, m->mega_grid * 64) * sizeof(long long), cudaMemcpyDeviceToHost));
    return ML2_OK;
}

int ml2_model_set_split_attention_from(ml2_model* h, int min_seq)
{
    // From this many cache rows on, the persistent kernel spreads every head's attention over several CTAs.
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    if (min_seq < 2) return fail(ML2_E_INVALID, "set_split_attention_from: %d (at least 2)", min_seq);
    m->att_min_seq = min_seq;
    return ML2_OK;
}

int ml2_model_debug_skip_launch(ml2_model* h)
{
    // Host-made desynchronisation for the failure-path test: advances the launch number the counters are compared
    // with, exactly what a rank that skipped a forward looks like to its peers. The next forward's dependency waits
    // can then never be met and run out after the context's wait limit; nothing on the device is touched here.
    Model* m = reinterpret_cast<Model*>(h);
    if (!m) return fail(ML2_E_INVALID, "null model");
    ++m->mega_seq;
    return ML2_OK;
}

int ml2_debug_tile_plan(int fmt, int rows, int cols, int nmat, int paired, int slot_bytes, int n_cta, long long* out8)
{
    // Host only (no CUDA call): plans one weight operator of the persistent kernel for a ring slot of `slot_bytes`,
    // builds every CTA's tile list and checks it. out8 = {planned, units covered, fewest tiles of a CTA, most tiles,
    // violations, units of a full tile, working warps, groups per warp}. A violation is a tile outside the operator's
    // rows or larger than a full tile, a copy that breaks the 16-byte rule of bulk copies or leaves the slot, a unit
    // covered twice or not at all, or a missing "last tile" mark.
    if (!out8 || rows <= 0 || cols <= 0 || nmat < 1 || nmat > 3 || n_cta < 1) return fail(ML2_E_INVALID, "debug_tile_plan: argument");
    for (int i = 0; i < 8; ++i) out8[i] = 0;
    MegaOp op{};
    op.kind = paired ? MOP_SWIGLU : (nmat == 3 ? MOP_QKV : MOP_RESID);
    if (!mega_plan_op(op, fmt, rows, cols, nmat, paired != 0, slot_bytes)) return ML2_OK;
    out8[0] = 1; out8[5] = op.rmax; out8[6] = op.kw; out8[7] = op.np;
    op.ngran = op.cols / op.gran;
    op.gmax = op.rmax / op.gran;
    op.rot = 37 % n_cta;
    // distinct, 16-byte aligned fake bases: only address arithmetic is checked
    const uintptr_t base = 0x10000000u;
    for (int q = 0; q < 3; ++q)
        op.mat[q] = QWPtrs{reinterpret_cast<const uint32_t*>(base + (uintptr_t)q * 0x10000000u),
                           fmt == 0 ? reinterpret_cast<const uint32_t*>(base + 0x40000000u + (uintptr_t)q * 0x01000000u) : nullptr,
                           fmt == 0 ? reinterpret_cast<const __half*>(base + 0x50000000u + (uintptr_t)q * 0x01000000u) : nullptr};
    const int nseg = paired ? 1 : nmat;
    std::vector<int> seen((size_t)cols * nseg, 0);
    long long bad = 0, covered = 0;
    int mint = 1 << 30, maxt = 0;
    for (int c = 0; c < n_cta; ++c) {
        std::vector<MegaTile> t;
        mega_tiles_of(op, 3, c, n_cta, t);
        mint = std::min(mint, (int)t.size());
        maxt = std::max(maxt, (int)t.size());
        for (size_t i = 0; i < t.size(); ++i) {
            const MegaTile& T = t[i];
            const int seg = (int)((T.info >> 16) & 3u);
            if (T.row < 0 || T.n <= 0 || T.row + T.n > cols || T.n > op.rmax || T.row % op.gran || T.n % op.gran || seg >= nseg) { ++bad; continue; }
            if (((T.info & kTileLast) != 0) != (i + 1 == t.size())) ++bad;
            for (int r = T.row; r < T.row + T.n; ++r) { ++seen[(size_t)seg * cols + r]; ++covered; }
            uint32_t total = 0;
            for (const MegaTileCopy& e : T.cp) {
                if (!e.bytes) continue;
                total += e.bytes;
                if ((reinterpret_cast<uintptr_t>(e.src) & 15u) || (e.bytes & 15u) || (e.dst & 15u) || e.dst + e.bytes > (uint32_t)slot_bytes) ++bad;
            }
            if (total != T.total_bytes) ++bad;
        }
    }
    for (int v : seen) bad += v != 1;
    // what the consumer warps read of a slot, whatever the tile's size: the rows of one block of 8 (two blocks: 16 rows, or
    // 8 rows of each of the two runs), their zero words and scales, all inside the tile's layout and the slot
    const int nruns = paired ? 2 : 1;
    if (fmt == 0) {
        const int block_rows = (op.two && !paired) ? 16 : 8;
        if (block_rows > op.rmax) ++bad;
        if (op.kw < 1 || op.kw > kMegaConsumerWarps || op.kw * op.np < op.ngrp || (op.kw - 1) * op.np >= op.ngrp) ++bad;   // every group has a warp, every warp a group
        if (block_rows * op.wrow > op.off_z || op.off_z + block_rows * op.zrow > op.off_s || op.off_s + block_rows * op.srow > op.run_bytes) ++bad;
        if (op.ngrp * 64 != op.wrow || op.tab_n < op.ngrp * 4 || (op.tab_n & 7)) ++bad;
    } else {
        if (op.rmax > op.groups * kMegaGroupRows || op.kw * op.groups > kMegaConsumerWarps || op.kw * 32 * op.np < op.units) ++bad;
        if (op.rmax * op.wrow > op.run_bytes) ++bad;
    }
    if (nruns * op.run_bytes > slot_bytes) ++bad;
    out8[1] = covered; out8[2] = mint; out8[3] = maxt; out8[4] = bad;
    return ML2_OK;
}

int ml2_model_comm_handle(ml2_model* h, void* out64)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !out64) return fail(ML2_E_INVALID, "comm_handle: null argument");
    if (m->tp < 2 || !m->comm_local) return fail(ML2_E_STATE, "comm_handle: the model is not tensor parallel");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t size");
    cudaIpcMemHandle_t hd;
    ML2_CUDA(cudaIpcGetMemHandle(&hd, m->comm_local));
    memcpy(out64, &hd, sizeof(hd));
    return ML2_OK;
}

int ml2_model_comm_attach(ml2_model* h, const void* handles, int n)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !handles) return fail(ML2_E_INVALID, "comm_attach: null argument");
    if (m->tp < 2 || !m->comm_local) return fail(ML2_E_STATE, "comm_attach: the model is not tensor parallel");
    if (n != m->tp || n > 8) return fail(ML2_E_INVALID, "comm_attach: %d handles for %d ranks (at most 8)", n, m->tp);
    if (m->comm_attached) return fail(ML2_E_STATE, "comm_attach: already attached");
    ML2_CUDA(cudaSetDevice(m->ctx->device));
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    for (int q = 0; q < n; ++q) {
        if (q == m->rank) { m->comm_peer[q] = m->comm_local; continue; }
        cudaIpcMemHandle_t hd;
        memcpy(&hd, static_cast<const char*>(handles) + (size_t)q * 64, sizeof(hd));
        void* ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int r = 0; r < q; ++r)
                if (r != m->rank && m->comm_peer[r]) { cudaIpcCloseMemHandle(m->comm_peer[r]); m->comm_peer[r] = nullptr; }
            return fail(ML2_E_CUDA, "comm_attach: cudaIpcOpenMemHandle(rank %d): %s", q, cudaGetErrorString(e));
        }
        m->comm_peer[q] = ptr;
    }
    m->comm_attached = true;
    m->mega_built = false;
    return ML2_OK;
}

int ml2_model_stream(ml2_model* h, void** stream)
{
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !stream) return fail(ML2_E_INVALID, "model_stream: null argument");
    *stream = m->stream;
    return ML2_OK;
}

int ml2_model_profile(ml2_model* h, int iters, double* avg_us, double* algo_bytes)
{
    // Times every kernel kind on its own: `iters` sweeps over all layers (distinct weights every launch, the
    // sweep is far larger than L2), CUDA events on the model's stream. Activations are whatever the last
    // forward left; the residual stream is restored afterwards.
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !avg_us || !algo_bytes) return fail(ML2_E_INVALID, "profile: null argument");
    int rc = check_bound(m);
    if (rc) return rc;
    if (iters < 1) return fail(ML2_E_INVALID, "profile: iters=%d", iters);
    Ctx* ctx = m->ctx;
    if ((rc = use_device(ctx))) return rc;
    ctx->stream = m->stream;
    const ml2_config& c = m->cfg;
    __half* x_save = nullptr;
    ML2_CUDA(cudaMalloc(&x_save, (size_t)c.dim * 2));
    ML2_CUDA(cudaMemcpyAsync(x_save, m->x, (size_t)c.dim * 2, cudaMemcpyDeviceToDevice, m->stream));
    // the attention is timed at the position of the latest forward (its cache rows are written up to there)
    const int pos = m->last_pos;
    {
        StepState st{pos, pos + 1, 0, 0};
        ML2_CUDA(cudaMemcpyAsync(m->step, &st, sizeof(st), cudaMemcpyHostToDevice, m->stream));
    }
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    cudaEvent_t e0, e1;
    ML2_CUDA(cudaEventCreate(&e0));
    ML2_CUDA(cudaEventCreate(&e1));
    const double n = pos + 1;
    const double kv_bytes = 2.0 * n * m->dim_local * 2.0 + 2.0 * m->dim_local * 2.0;
    const double bytes[6] = {
        3.0 * qweight_bytes(c.dim, m->dim_local) + 2.0 * c.dim * 2 + 3.0 * m->dim_local * 2,
        kv_bytes,
        qweight_bytes(m->dim_local, c.dim) + m->dim_local * 2.0 + 2.0 * c.dim * 2,
        2.0 * qweight_bytes(c.dim, m->hidden_local) + 2.0 * c.dim * 2 + m->hidden_local * 2.0,
        qweight_bytes(m->hidden_local, c.dim) + m->hidden_local * 2.0 + 2.0 * c.dim * 2,
        (double)m->vocab_local * c.dim * 2 + 2.0 * c.dim * 2 + m->vocab_local * 2.0};
    for (int kind = 0; kind < 6; ++kind) {
        const int per_iter = kind == 5 ? 1 : c.n_layers;
        const int reps = kind == 5 ? iters * 4 : iters;
        for (int l = 0; l < per_iter; ++l)
            if ((rc = enqueue_kind(m, kind, l))) return rc;  // warm-up sweep
        ML2_CUDA(cudaEventRecord(e0, m->stream));
        for (int it = 0; it < reps; ++it)
            for (int l = 0; l < per_iter; ++l)
                if ((rc = enqueue_kind(m, kind, l))) return rc;
        ML2_CUDA(cudaEventRecord(e1, m->stream));
        ML2_CUDA(cudaEventSynchronize(e1));
        float ms = 0.f;
        ML2_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        avg_us[kind] = (double)ms * 1e3 / ((double)reps * per_iter);
        algo_bytes[kind] = bytes[kind];
    }
    ML2_CUDA(cudaMemcpyAsync(m->x, x_save, (size_t)c.dim * 2, cudaMemcpyDeviceToDevice, m->stream));
    ML2_CUDA(cudaStreamSynchronize(m->stream));
    cudaFree(x_save);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return ML2_OK;
}

int ml2_model_generate(ml2_model* h, const int* prompt_host, int n_prompt, int steps, int* out_tokens_host, int* n_out)
{
    // Transformer.Generate (src/Transformer.cs:89-112) on token ids: prompt to the device once, then per
    // position one Forward and, past the prompt, the greedy sample read back as 4 bytes; stops on id < 3.
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !prompt_host || !out_tokens_host || !n_out) return fail(ML2_E_INVALID, "generate: null argument");
    if (n_prompt < 1 || steps < 0 || steps > m->cfg.seq_len - 1) return fail(ML2_E_INVALID, "generate: n_prompt=%d steps=%d", n_prompt, steps);
    if (n_prompt > m->cfg.seq_len) return fail(ML2_E_INVALID, "generate: prompt longer than the sequence length");
    int rc = ml2_model_set_tokens(h, prompt_host, 0, n_prompt);
    if (rc) return rc;
    int produced = 0;
    for (int pos = 0; pos < steps; ++pos) {
        const int next_pos = pos + 1;
        const int generate = next_pos >= n_prompt;
        if ((rc = ml2_model_forward(h, pos, next_pos, generate))) return rc;
        int token;
        if (generate) {
            if ((rc = ml2_model_read_token(h, next_pos, &token))) return rc;
        } else {
            token = prompt_host[next_pos];
        }
        if (token < 3) break;
        out_tokens_host[produced++] = token;
    }
    *n_out = produced;
    return check_device_status(m);
}

}  // extern "C"
