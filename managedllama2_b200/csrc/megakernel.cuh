// One persistent kernel per token: the whole operator sequence of Transformer.Forward
// (src/Transformer.cs:158-190 of GilesBathgate/ManagedLlama2) runs inside a single cooperative launch with
// one CTA per SM, so HBM streaming never stops at an operator boundary.
//
//   * producer warp   walks the token's operator list and streams every weight tile this CTA owns, operator
//                     after operator, into one shared-memory ring (1-D bulk async copies, mbarrier completion).
//                     Weights do not depend on activations, so it runs ahead of the arithmetic by the depth of
//                     the ring, across operator boundaries.
//   * consumer warps  organised in groups of `kw` warps (one group spans a whole weight row: lane owns 32 inputs
//                     = one 16-byte weight vector of every row). A group waits until the operator's input vector
//                     is complete (a device-wide counter, acquire), keeps its slice in registers (RMSNorm applied
//                     on the fly where the reference runs rmsnorm first), then takes tiles from the ring.
//   * finalizer warps sum the k-warp partials in a fixed order and run the operator's tail (residual add, RoPE,
//                     SwiGLU, stores) with the reference's fp16 rounding points; after its last tile of an
//                     operator a CTA publishes "my share is done" (release) on that operator's counter.
//   * attention       is an operator without weights, with the three steps and rounding points of the reference's
//                     scores / softmax / values kernels: one CTA per head for short contexts, several CTAs per head
//                     (parts of the sequence, maximum / exp-sum exchanged through global memory) for long ones.
//   * wide rows       (down-projection) are swept several times by a group of fewer warps, the prepared input
//                     slices parked in shared memory, so that all warps stay busy (mega_multisweep_op).
//
// Every wait is bounded; when a limit runs out the CTA records an error word, stops waiting and runs to its end.
#pragma once

#include "stream_matvec.cuh"

#ifndef ML2_MULTI
#define ML2_MULTI 1
#endif

namespace ml2 {

enum MegaOpKind : int { MOP_QKV = 0, MOP_ATTN = 1, MOP_RESID = 2, MOP_SWIGLU = 3, MOP_CLS = 4, MOP_ARGMAX = 5, MOP_PARTIAL = 6 };

struct MegaOp {
    int kind;
    int fmt;                 // 0 int4, 1 fp16 weights
    int pro;                 // 0 plain input, 1 RMSNorm(in, gamma), 2 RMSNorm(embedding row of the token, gamma),
                             // 3 RMSNorm(in + sum over ranks of recv, gamma): residual add of a row-sharded mat-vec
    int rows, cols, nmat;    // d_in, d_out per matrix, matrices
    int wsize, zsize, ssize; // per-output sizes (words, words, halves)
    int units;               // 16-byte vectors per row
    int kw, groups;          // warps per group, groups per CTA
    int nch, rwc;            // arithmetic chunks per tile, rows per chunk
    int nruns, run_rows;     // copy sets ("runs" of consecutive rows) per tile, rows per run: nruns * run_rows = nch * rwc
    int ntiles;
    int chunk_bytes, woff_z, woff_s;   // shared-memory bytes of one run and the offsets of its zeros / scales parts
    int rot;                 // rotation of the tile -> CTA assignment
    int tp;                  // ranks summed into the input (pro 3) / receiving the output (MOP_PARTIAL, sharded MOP_CLS)
    int out_row0;            // sharded classifier: first vocabulary row of this rank
    int passes;              // a group covers a row in `passes` sweeps of kw * 32 lane slots (1: input slice stays in registers)
    QWPtrs mat[3];
    __half* out[3];
    float* out_f32;
    const __half* in;        // pro 3: the residual stream BEFORE the all-reduced update
    const __half* gamma;
    const __half* kcache;    // attention: this layer's caches
    const __half* vcache;
    // tensor parallel, fused all-reduce over peer memory (plain peer stores, no multicast):
    const float* recv;       // pro 3: [tp][rows] fp32 partials that every rank (this one included) stored here
    __half* x_next;          // pro 3: where CTA 0 stores the updated residual stream
    float* peer_out[8];      // MOP_PARTIAL: this rank's row block inside every rank's receive zone
    __half* peer_logits[8];  // sharded MOP_CLS: every rank's full logits buffer
    unsigned int* peer_done[8];  // this operator's counter on every rank
    // attention split over several CTAs per head (long contexts):
    float* att_ml;           // [heads][split][2]: running maximum and exp-sum of every part
    float* att_part;         // [heads][split][head_size]: fp32 partial outputs (MOP_ATTN writes, the next operator sums them)
    unsigned int* att_cnt;   // [heads]: arrivals of the parts, monotonically increasing
    int att_layer;           // layer index (the counters advance once per layer and token)
    int pad2;
};

struct MegaParams {
    const MegaOp* ops;
    int nops;
    unsigned int* done;        // [nops] arrivals, monotonically increasing over tokens
    DeviceStatus* status;
    const float2* rope_table;
    const __half* embed;
    __half* x;
    int* tokens;
    const __half* logits;
    int pos, next_pos, write_token;
    unsigned int seq_no;       // 1, 2, 3, ... : arrivals expected on a counter = seq_no * gridDim.x
    int dim, head_size, heads_local, kv_row_stride, vocab;
    float eps, scale;
    int nstage, slot_bytes, att_cap;
    int att_split;             // CTAs per head for this token's attention (1: one CTA per head)
    unsigned int att_seq;      // 1, 2, 3, ... over the tokens that used the split path
    int n_layers;
    int debug;                 // bit 0: consumers skip the arithmetic (pipeline probe)
    long long* prof;           // optional [gridDim.x][64] cycle counters (diagnostics), may be null
};

constexpr int kMegaConsumerWarps = 21;   // 3 groups of 7, 4 of 5, 5 of 4
constexpr int kMegaFinalWarps = 2;
constexpr int kMegaWarps = kMegaConsumerWarps + 1 + kMegaFinalWarps;
constexpr int kMegaThreads = kMegaWarps * 32;
constexpr int kMegaMaxStages = 12;
constexpr int kMegaRedSlots = 8;
constexpr int kMegaMaxRows = 8;       // rows per tile
constexpr int kMegaMaxGroups = 5;
constexpr int kMegaMaxSplit = 8;     // CTAs per head of the split attention
constexpr int kAttUnroll = 4;        // cache rows a warp keeps in flight
constexpr uint32_t kBarCount = 64;    // fixed arrival count of the consumer-side mbarriers (see arrive_n)

__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t n)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct MegaChunk {
    int m, row0, nrows;
};

// arrivals one CTA makes on an operator's counter: every finalizer warp for weight operators, one thread otherwise
__host__ __device__ __forceinline__ unsigned int mega_arrivals(const MegaOp& op)
{
    const unsigned int per_rank = op.ntiles > 0 ? (unsigned int)kMegaFinalWarps : 1u;
    const bool shared = (op.kind == MOP_PARTIAL || op.kind == MOP_CLS) && op.tp > 1;   // every rank publishes on every rank
    return shared ? per_rank * (unsigned int)op.tp : per_rank;
}

__device__ __forceinline__ MegaChunk mega_chunk(const MegaOp& op, int head_size, int tile, int c)
{
    MegaChunk k;
    if (op.kind == MOP_SWIGLU) {
        k.m = c;  // chunk 0 = gate rows, chunk 1 = the same rows of up
        k.row0 = tile * op.rwc;
    } else if (op.kind == MOP_QKV) {
        const int half = head_size >> 1;
        const int ppm = (op.cols >> 1) / op.rwc;   // pairs per matrix
        k.m = tile / ppm;
        const int pp = tile - k.m * ppm;
        const int pph = half / op.rwc;
        const int head = pp / pph;
        k.row0 = head * head_size + (pp - head * pph) * op.rwc + c * half;  // rotate-half partners share a tile
    } else {
        k.m = 0;
        k.row0 = (tile * op.nch + c) * op.rwc;
    }
    int n = op.cols - k.row0;
    n = n < 0 ? 0 : (n > op.rwc ? op.rwc : n);
    k.nrows = (k.m < op.nmat) ? n : 0;
    return k;
}

// Copy set `run` of a tile: the consecutive rows one group of bulk copies brings in.
__device__ __forceinline__ MegaChunk mega_run(const MegaOp& op, int head_size, int tile, int run)
{
    if (op.kind == MOP_SWIGLU || op.kind == MOP_QKV) return mega_chunk(op, head_size, tile, run);
    MegaChunk k;
    k.m = 0;
    k.row0 = tile * op.run_rows;
    int n = op.cols - k.row0;
    n = n < 0 ? 0 : (n > op.run_rows ? op.run_rows : n);
    k.nrows = run == 0 ? n : 0;
    return k;
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v)
{
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Device-wide dependency: waits until `counter` has collected `expected` arrivals (bounded).
__device__ __forceinline__ void mega_wait_counter(const unsigned int* counter, unsigned int expected, volatile unsigned int* abort_flag,
                                                  DeviceStatus* status, unsigned int code, int op_index, bool sys_scope)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        const unsigned int seen = sys_scope ? ld_acquire_sys(counter) : ld_acquire_gpu(counter);
        if ((int)(seen - expected) >= 0) return;
        if ((i & 255u) == 255u && (*abort_flag || ld_acquire_gpu(&status->error))) { *abort_flag = 1; return; }
    }
    *abort_flag = 1;
    atomicExch(&status->error, code);
    status->detail = (unsigned int)op_index;
}

template <int NX>
__device__ __forceinline__ void mega_load_slice(const __half* src, int rows, int e0, uint32_t (&xr)[NX / 2])
{
#pragma unroll
    for (int v = 0; v < NX / 8; ++v) {
        const int e = e0 + v * 8;
        uint4 t = make_uint4(0, 0, 0, 0);
        if (e + 8 <= rows) t = *reinterpret_cast<const uint4*>(src + e);
        xr[v * 4 + 0] = t.x; xr[v * 4 + 1] = t.y; xr[v * 4 + 2] = t.z; xr[v * 4 + 3] = t.w;
    }
}

// RMSNorm of a slice held in registers (native/rmsnorm_kernel.cu:12-35); `tot` is the sum of squares of the vector.
template <int NX>
__device__ __forceinline__ void mega_norm_slice(const __half* gamma, int rows, int e0, float tot, float eps, uint32_t (&xr)[NX / 2])
{
    const float rms = 1.0f / sqrtf(tot / (float)rows + eps);
#pragma unroll
    for (int v = 0; v < NX / 8; ++v) {
        const int e = e0 + v * 8;
        if (e + 8 > rows) continue;
        const uint4 t = *reinterpret_cast<const uint4*>(gamma + e);
        const uint32_t g4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t xv = xr[v * 4 + i];
            const float lo = rms * half_bits_to_float(lo16(g4[i])) * half_bits_to_float(lo16(xv));
            const float hi = rms * half_bits_to_float(hi16(g4[i])) * half_bits_to_float(hi16(xv));
            xr[v * 4 + i] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
        }
    }
}

template <int NX>
__device__ __forceinline__ float slice_sumsq(const uint32_t (&xr)[NX / 2])
{
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NX / 2; ++i) {
        const float a = half_bits_to_float(lo16(xr[i])), b = half_bits_to_float(hi16(xr[i]));
        ss = fmaf(a, a, ss);
        ss = fmaf(b, b, ss);
    }
    return warp_sum(ss);
}

// Four rows of one lane slot: dequantise-and-multiply against the prepared slice `xq`; zero point and scale are
// applied once per row (aw / az / as: shared-memory addresses of the lane's weight vector, zero word and scale of row 0).
__device__ __forceinline__ void mega_int4_rows(const XSlice& xq, uint32_t aw, uint32_t az, uint32_t as, uint32_t w_row, uint32_t z_row,
                                               uint32_t s_row, int zshift, bool act, float (&v)[4])
{
    uint4 wv[4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(wv[r].x), "=r"(wv[r].y), "=r"(wv[r].z), "=r"(wv[r].w)
                     : "r"(aw + r * w_row));
    // two accumulators per row (A: nibbles 0, 2, 4, 6; B: the odd ones, scaled by 16), four rows in flight
    float A[4], B[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        A[r] = xq.a0;
        B[r] = xq.b0;
        word_dot(wv[r].x, xq.xp + 0, A[r], B[r], A[r]);
        word_dot(wv[r].y, xq.xp + 4, A[r], B[r], A[r]);
        word_dot(wv[r].z, xq.xp + 8, A[r], B[r], A[r]);
        word_dot(wv[r].w, xq.xp + 12, A[r], B[r], A[r]);
    }
    // zero point and scale are fetched after the products: they are needed only now, and eight fewer registers are
    // live during the inner loop
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        uint32_t zw;
        unsigned short sc;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw) : "r"(az + r * z_row));
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sc) : "r"(as + r * s_row));
        const float zf = (float)((zw >> zshift) & 0xFu);
        const float t = fmaf(B[r], 0.0625f, A[r]);
        const float res = half_bits_to_float(sc) * fmaf(-zf, xq.c1, t);
        v[r] = act ? res : 0.f;
    }
}

constexpr int kSliceVecs = 5;   // 16-byte vectors of a prepared slice parked in shared memory

// Prepared slice of lane slot `sidx` -> table [kSliceVecs][tab_n] (xp: 4 vectors, start values: 1).
__device__ __forceinline__ void mega_store_slice(uint4* tab, int tab_n, int sidx, const XSlice& t)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) tab[q * tab_n + sidx] = make_uint4(t.xp[4 * q], t.xp[4 * q + 1], t.xp[4 * q + 2], t.xp[4 * q + 3]);
    tab[(kSliceVecs - 1) * tab_n + sidx] = make_uint4(__float_as_uint(t.a0), __float_as_uint(t.b0), __float_as_uint(t.c1), 0u);
}

__device__ __forceinline__ void mega_load_slice_tab(uint32_t ta, uint32_t tstep, XSlice& xt)
{
    float pad;
#pragma unroll
    for (int q = 0; q < 4; ++q)
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(xt.xp[4 * q]), "=r"(xt.xp[4 * q + 1]), "=r"(xt.xp[4 * q + 2]), "=r"(xt.xp[4 * q + 3])
                     : "r"(ta + q * tstep));
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(xt.a0), "=f"(xt.b0), "=f"(xt.c1), "=f"(pad) : "r"(ta + (kSliceVecs - 1) * tstep));
}

// Shared-memory objects of the kernel that the multi-sweep consumer needs.
struct MegaShared {
    unsigned char* smem;     // ring, then the scratch area
    uint64_t* full_bar;
    uint64_t* empty_bar;
    uint64_t* done_bar;
    uint64_t* free_bar;
    float* red;              // [kMegaRedSlots][kMaxKW][kMegaMaxRows]
    unsigned int* abort_flag;
    DeviceStatus* status;
    int nstage, slot_bytes;
};

// Consumer side of an int4 operator whose rows are wider than one sweep of a group (op.passes > 1; plain input).
// Every lane slot's prepared slice is built once per operator and parked in shared memory; a group of kw warps sweeps
// a tile `passes` times, reloading the lane's slice per sweep, so that groups * kw warps stay busy where a single
// sweep would tie most of the warps to one row. A loop of its own, apart from the single-sweep loop of the kernel.
__device__ __forceinline__ void mega_multisweep_op(const MegaOp& op, int k, const MegaShared& sh, int first, int cnt, uint32_t n_base,
                                                   int st_base, uint32_t ph_base)
{
    constexpr int kConsThreads = kMegaConsumerWarps * 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ncta = gridDim.x;
    const int npass = op.passes;
    const int stride = op.kw * 32;
    const int tab_n = stride * npass;
    uint4* s_tab = reinterpret_cast<uint4*>(sh.smem + (size_t)sh.nstage * sh.slot_bytes);
    for (int sidx = tid; sidx < tab_n; sidx += kConsThreads) {
        uint32_t xr[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) xr[i] = 0u;
        if (sidx < op.units) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 t = *reinterpret_cast<const uint4*>(op.in + (size_t)sidx * 32 + v * 8);
                xr[4 * v] = t.x; xr[4 * v + 1] = t.y; xr[4 * v + 2] = t.z; xr[4 * v + 3] = t.w;
            }
        }
        XSlice t;
        make_xslice(xr, t);
        mega_store_slice(s_tab, tab_n, sidx, t);
    }
    named_bar_sync(1, kConsThreads);

    const int group = warp / op.kw;
    const int kw_id = warp - group * op.kw;
    if (group >= op.groups) return;
    const int u = kw_id * 32 + lane;
    const uint32_t w_row = (uint32_t)op.wsize * 4u, z_row = (uint32_t)op.zsize * 4u, s_row = (uint32_t)op.ssize * 2u;
    const uint32_t ring = smem_u32(sh.smem);
    const uint32_t tab = smem_u32(s_tab), tstep = (uint32_t)tab_n * 16u;
    const uint32_t my_arrive = (kw_id == 0) ? (kBarCount - (uint32_t)op.kw + 1u) : 1u;
    const bool writer = (lane & 7) == 0 && (lane >> 3) < op.rwc;
    int st = st_base + group;
    uint32_t ph = ph_base;
    while (st >= sh.nstage) { st -= sh.nstage; ph ^= 1u; }
    for (int i = group; i < cnt; i += op.groups) {
        const uint32_t n = n_base + (uint32_t)i;
        wait_or_abort(&sh.full_bar[st], ph, sh.abort_flag, sh.status, 2u, k);
        const int slot = (int)(n % kMegaRedSlots);
        float* red = sh.red + (size_t)slot * (kMaxKW * kMegaMaxRows);
        bool slot_ready = n < (uint32_t)kMegaRedSlots;
        float resid[2] = {0.f, 0.f};
        if (op.kind == MOP_RESID && kw_id == 0 && writer) {
            const int tile = first + i * ncta;
            for (int c = 0; c < op.nch; ++c) {
                const int row = (tile * op.nch + c) * op.rwc + (lane >> 3);
                if (row < op.cols) resid[c] = __half2float(op.out[0][row]);
            }
        }
        for (int c = 0; c < op.nch; ++c) {
            const int trow = c * op.rwc;
            const int run = trow / op.run_rows;
            const int rin0 = trow - run * op.run_rows;
            const uint32_t cbase = ring + (uint32_t)st * sh.slot_bytes + (uint32_t)run * op.chunk_bytes;
            const uint32_t cw = cbase + (uint32_t)rin0 * w_row;
            const uint32_t cz = cbase + op.woff_z + (uint32_t)rin0 * z_row;
            const uint32_t cs = cbase + op.woff_s + (uint32_t)rin0 * s_row;
            float tot[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < npass; ++j) {
                const int uj = u + j * stride;
                const bool act = uj < op.units;
                const int ua = act ? uj : 0;
                const int g = ua >> 2;
                XSlice xt;
                mega_load_slice_tab(tab + (uint32_t)uj * 16u, tstep, xt);
                float v[4];
                mega_int4_rows(xt, cw + (uint32_t)ua * 16u, cz + (uint32_t)(g >> 3) * 4u, cs + (uint32_t)g * 2u, w_row, z_row, s_row,
                               (g & 7) * 4, act, v);
#pragma unroll
                for (int r = 0; r < 4; ++r) tot[r] += v[r];
            }
            if (c == op.nch - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive_n(&sh.empty_bar[st], my_arrive);
            }
            transpose_reduce<4>(tot, lane);
            if (!slot_ready) {
                wait_or_abort(&sh.free_bar[slot], ((n / kMegaRedSlots) - 1u) & 1u, sh.abort_flag, sh.status, 4u, k);
                slot_ready = true;
            }
            if (writer) red[kw_id * kMegaMaxRows + c * op.rwc + (lane >> 3)] = tot[0];
            if (op.kind == MOP_RESID && kw_id == 0 && writer) red[op.kw * kMegaMaxRows + c * op.rwc + (lane >> 3)] = resid[c];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive_n(&sh.done_bar[slot], my_arrive);
        st += op.groups;
        while (st >= sh.nstage) { st -= sh.nstage; ph ^= 1u; }
    }
}

// kProf adds cycle counters around the waits (diagnostics); the production instantiation carries none.
template <bool kProf>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const MegaParams p)
{
    auto now = [&]() -> long long { return kProf ? clock64() : 0ll; };
    extern __shared__ __align__(128) unsigned char smem_raw[];   // [ring: nstage * slot_bytes][attention scores: att_cap floats]
    __shared__ __align__(8) uint64_t full_bar[kMegaMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMegaMaxStages];
    __shared__ __align__(8) uint64_t done_bar[kMegaRedSlots];
    __shared__ __align__(8) uint64_t free_bar[kMegaRedSlots];
    __shared__ float s_red[kMegaRedSlots][kMaxKW][kMegaMaxRows];
    __shared__ float s_part[2][1][kMaxKW];   // per-warp sum-of-squares partials, double-buffered by operator parity
    __shared__ float s_att_acc[kMegaConsumerWarps][kHeadMax];
    __shared__ float s_att_tmp[kMegaConsumerWarps];
    __shared__ float s_best_v[kMegaConsumerWarps];
    __shared__ int s_best_i[kMegaConsumerWarps];
    __shared__ unsigned int s_abort;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const unsigned int expected = p.seq_no * (unsigned int)ncta;
    constexpr int kConsThreads = kMegaConsumerWarps * 32;

    if (tid == 0) {
        for (int s = 0; s < p.nstage; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kBarCount);
        }
        for (int s = 0; s < kMegaRedSlots; ++s) {
            mbar_init(&done_bar[s], kBarCount);
            mbar_init(&free_bar[s], 1);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // tiles of operator `op` owned by this CTA: first + i * ncta, i < count
    auto my_first = [&](const MegaOp& op) { int f = cta - op.rot; f %= ncta; return f < 0 ? f + ncta : f; };
    auto my_count = [&](const MegaOp& op, int first) { return op.ntiles > first ? (op.ntiles - 1 - first) / ncta + 1 : 0; };

    if (warp == kMegaConsumerWarps) {
        // ================= producer =====================================================================
        const uint64_t pol = policy_evict_first();
        // ring position of this CTA's running tile counter, kept without divisions: stage index and use count parity
        int st = 0;
        uint32_t ph = 0;      // parity of (uses of this stage so far)
        bool wrapped = false;
        long long tp_wait = 0, tp_all0 = now();
        const bool nocopy = (p.debug & 8) != 0;
        for (int k = 0; k < p.nops; ++k) {
            // The per-tile chain of this warp bounds the streaming rate of the CTA: everything that does not change
            // from tile to tile is read once per operator into registers, tile addresses advance by increments.
            const MegaOp* gp = p.ops + k;
            const int ntiles = gp->ntiles;
            if (ntiles == 0) continue;
            const int kind = gp->kind, cols = gp->cols, rwc = gp->rwc, nruns = gp->nruns;
            const bool int4 = gp->fmt == 0;
            const bool paired = kind == MOP_SWIGLU || kind == MOP_QKV;
            const int rr = paired ? rwc : gp->run_rows;             // rows of one run
            const uint32_t wrow = (uint32_t)gp->wsize * 4u, zrow = int4 ? (uint32_t)gp->zsize * 4u : 0u, srow = int4 ? (uint32_t)gp->ssize * 2u : 0u;
            const uint32_t woff_z = gp->woff_z, woff_s = gp->woff_s;
            const uint32_t lane_off = (uint32_t)lane * (uint32_t)gp->chunk_bytes;
            int first = (cta - gp->rot) % ncta;
            if (first < 0) first += ncta;
            const int cnt = ntiles > first ? (ntiles - 1 - first) / ncta + 1 : 0;
            // QKV: tile -> (matrix, pair of row blocks); the two runs of a tile are rotate-half partners
            const int half = p.head_size >> 1;
            const int ppm = paired ? (cols >> 1) / rwc : 1, pph = paired ? half / rwc : 1;
            int qm = 0, qpp = 0;
            if (kind == MOP_QKV) { qm = first / ppm; qpp = first - qm * ppm; }
            QWPtrs q = gp->mat[kind == MOP_SWIGLU ? (lane & 1) : (qm < 2 ? qm : 2)];
            int tile = first;
            for (int i = 0; i < cnt; ++i, tile += ncta) {
                if (wrapped) {
                    const long long tw0 = now();
                    if (lane == 0) wait_parked_or_abort(&empty_bar[st], ph ^ 1u, &s_abort, p.status, 1u, k);
                    __syncwarp();
                    tp_wait += now() - tw0;
                }
                int row0;
                if (kind == MOP_QKV) {
                    const int head = qpp / pph;
                    row0 = head * p.head_size + (qpp - head * pph) * rwc + (lane & 1) * half;
                } else {
                    row0 = tile * rr;
                }
                int nrows = cols - row0;
                nrows = nrows < 0 ? 0 : (nrows > rr ? rr : nrows);
                const uint32_t bw = (uint32_t)nrows * wrow, bz = (uint32_t)nrows * zrow, bs = (uint32_t)nrows * srow;
                // every run of a tile holds the same number of rows (the operator plan admits full tiles only)
                if (lane == 0) mbar_arrive_expect_tx(&full_bar[st], nocopy ? 0u : (uint32_t)nruns * (bw + bz + bs));
                __syncwarp();
                if (lane < nruns && nrows > 0 && !nocopy) {
                    unsigned char* cb = smem_raw + (size_t)st * p.slot_bytes + lane_off;
                    bulk_g2s(cb, q.w + (size_t)row0 * (wrow >> 2), bw, &full_bar[st], pol);
                    if (int4) {
                        bulk_g2s(cb + woff_z, q.z + (size_t)row0 * (zrow >> 2), bz, &full_bar[st], pol);
                        bulk_g2s(cb + woff_s, q.s + (size_t)row0 * (srow >> 1), bs, &full_bar[st], pol);
                    }
                }
                if (kind == MOP_QKV) {
                    qpp += ncta;
                    if (qpp >= ppm) {
                        do { qpp -= ppm; ++qm; } while (qpp >= ppm);
                        q = gp->mat[qm < 2 ? qm : 2];
                    }
                }
                if (++st == p.nstage) { st = 0; ph ^= 1u; wrapped = true; }
            }
        }
        if (kProf && p.prof && lane == 0) {
            long long* o = p.prof + (size_t)cta * 64;
            o[32] = now() - tp_all0;
            o[33] = tp_wait;
        }
        return;
    }

    if (warp > kMegaConsumerWarps) {
        // ================= finalizers: fixed-order sum over k-warps + operator tail ========================
        const int fw = warp - kMegaConsumerWarps - 1;
        uint32_t n = 0;
        long long tf_wait = 0, tf_all0 = now(), tf_sum = 0, tf_store = 0, tf_rel = 0, tf_head = 0;
        for (int k = 0; k < p.nops; ++k) {
            // As in the producer, the operator's invariants sit in registers and nothing is divided per tile.
            const long long th0 = now();
            const MegaOp* gp = p.ops + k;
            const int ntiles = gp->ntiles;
            if (ntiles == 0) continue;   // attention / argmax are published by the consumers
            const int kind = gp->kind, cols = gp->cols, rwc = gp->rwc, kw = gp->kw, tp = gp->tp;
            const bool paired = kind == MOP_SWIGLU || kind == MOP_QKV;
            int first = (cta - gp->rot) % ncta;
            if (first < 0) first += ncta;
            const int cnt = ntiles > first ? (ntiles - 1 - first) / ncta + 1 : 0;
            const int half = p.head_size >> 1;
            const int ppm = paired ? (cols >> 1) / rwc : 1, pph = paired ? half / rwc : 1;
            int qm = 0, qpp = 0;
            if (kind == MOP_QKV) { qm = first / ppm; qpp = first - qm * ppm; }
            // lane roles: paired tiles use lanes [0, rwc) (one output row pair each); other tiles one lane per row
            const int nrow = paired ? rwc : gp->nch * rwc;
            const int roff = lane;                              // index of this lane's row inside the partial slot
            __half* const out0 = gp->out[0];
            __half* out_m = kind == MOP_QKV ? gp->out[qm < 2 ? qm : 2] : out0;
            const int rows_per_tile = paired ? rwc : gp->nch * rwc;
            tf_head += now() - th0 + (long long)(rows_per_tile + (int)(size_t)out_m) * 0;
            for (int i = 0; i < cnt; ++i, ++n) {
                const bool take = (int)(n % kMegaFinalWarps) == fw;
                if (take) {
                    const int tile = first + i * ncta;
                    const int slot = (int)(n % kMegaRedSlots);
                    const float* red = &s_red[slot][0][0];
                    const uint32_t par = (n / kMegaRedSlots) & 1u;
                    if (p.debug & 4) {
                        wait_parked_or_abort(&done_bar[slot], par, &s_abort, p.status, 3u, k);
                    } else if (paired) {
                        // rows ra (chunk 0) and rb (chunk 1) of this lane
                        int ra, rb;
                        if (kind == MOP_QKV) {
                            const int head = qpp / pph;
                            ra = head * p.head_size + (qpp - head * pph) * rwc + lane;
                            rb = ra + half;
                        } else {
                            ra = rb = tile * rwc + lane;
                        }
                        const bool mine = lane < rwc && ra < cols;
                        float2 cs = make_float2(1.f, 0.f);
                        if (kind == MOP_QKV && mine && qm < 2) cs = p.rope_table[(size_t)p.pos * half + ra % p.head_size];
                        const long long tw0 = now();
                        wait_parked_or_abort(&done_bar[slot], par, &s_abort, p.status, 3u, k);
                        tf_wait += now() - tw0;
                        float sa = 0.f, sb = 0.f;
                        if (mine) {
                            for (int w = 0; w < kw; ++w) {
                                sa += red[w * kMegaMaxRows + lane];
                                sb += red[w * kMegaMaxRows + rwc + lane];
                            }
                        }
                        // the partial slot is read: hand it back BEFORE the global stores, so that the release of
                        // this arrival does not have to wait for their acknowledgement
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&free_bar[slot]);
                        if (mine) {
                            if (kind == MOP_SWIGLU) {
                                float val = sa;                       // native/mat_vec_kernel.cu:218-222
                                val *= 1.0f / (1.0f + expf(-val));
                                val *= sb;
                                out0[ra] = __float2half_rn(val);
                            } else {
                                __half* o = out_m;
                                if (qm > 0) o += (long long)p.pos * p.kv_row_stride;
                                if (qm < 2) {
                                    // fp16 store of the mat-vec (native/mat_vec_kernel.cu:175), then RoPE on the rounded
                                    // values (native/rope_kernel.cu:15-25)
                                    const float a0 = __half2float(__float2half_rn(sa));
                                    const float b0 = __half2float(__float2half_rn(sb));
                                    o[ra] = __float2half_rn(a0 * cs.x - b0 * cs.y);
                                    o[rb] = __float2half_rn(a0 * cs.y + b0 * cs.x);
                                } else {
                                    o[ra] = __float2half_rn(sa);
                                    o[rb] = __float2half_rn(sb);
                                }
                            }
                        }
                    } else {
                        const int row = tile * rows_per_tile + roff;
                        const bool mine = lane < nrow && row < cols;
                        const long long tw0 = now();
                        wait_parked_or_abort(&done_bar[slot], par, &s_abort, p.status, 3u, k);
                        tf_wait += now() - tw0;
                        const long long ts0 = now();
                        float sum = 0.f, res = 0.f;
                        if (mine) {
                            for (int w = 0; w < kw; ++w) sum += red[w * kMegaMaxRows + roff];
                            // the residual value was fetched by the consumers (they hold the operator's dependency) and
                            // travels in the extra k-row of the partial slot
                            if (kind == MOP_RESID) res = red[kw * kMegaMaxRows + roff];
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&free_bar[slot]);   // before the global stores (see above)
                        const long long ts1 = now();
                        tf_sum += ts1 - ts0;
                        if (mine) {
                            if (kind == MOP_RESID)
                                out0[row] = __float2half_rn(sum + res);  // native/mat_vec_kernel.cu:154-156
                            else if (kind == MOP_PARTIAL) {
                                // row-sharded mat-vec: this rank's fp32 partial goes straight into every rank's receive
                                // zone (plain peer stores over NVLink); the residual add and the single fp16 rounding
                                // happen where the sum is consumed
                                for (int q = 0; q < tp; ++q) gp->peer_out[q][row] = sum;
                            } else if (tp > 1) {
                                // vocabulary-sharded classifier: every rank ends up with the full logits
                                const __half hv = __float2half_rn(sum);
                                for (int q = 0; q < tp; ++q) gp->peer_logits[q][gp->out_row0 + row] = hv;
                            } else {
                                out0[row] = __float2half_rn(sum);
                            }
                        }
                        tf_store += now() - ts1;
                    }
                    if (p.debug & 4) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&free_bar[slot]);
                    }
                }
                if (kind == MOP_QKV) {
                    qpp += ncta;
                    if (qpp >= ppm) {
                        do { qpp -= ppm; ++qm; } while (qpp >= ppm);
                        out_m = gp->out[qm < 2 ? qm : 2];
                    }
                }
            }
            // this CTA's share of operator k is written: publish it. The warp barrier orders every lane's stores
            // before lane 0's release, which is cumulative at device scope.
            const long long tr0 = now();
            __syncwarp();
            if ((kind == MOP_PARTIAL || kind == MOP_CLS) && tp > 1) {
                // published on every rank's counter: system-scope release after the peer stores of this warp
                if (lane < tp) red_release_sys_add(gp->peer_done[lane], 1u);
            } else if (lane == 0) {
                red_release_gpu_add(&p.done[k], 1u);
            }
            tf_rel += now() - tr0;
        }
        if (kProf && p.prof && lane == 0) {
            long long* o = p.prof + (size_t)cta * 64;
            o[34 + 2 * fw] = now() - tf_all0;
            o[35 + 2 * fw] = tf_wait;
            if (fw == 0) { o[40] = tf_sum; o[41] = tf_store; o[42] = tf_rel; o[43] = tf_head; }
        }
        return;
    }

    // ================= consumers =========================================================================
    uint32_t n_base = 0;  // running tile counter at the start of the current operator
    int st_base = 0;      // ring stage of that tile, and the parity of its use count
    uint32_t ph_base = 0;
    long long t_dep = 0, t_full = 0, t_free = 0, t_attn = 0, t_pro = 0, t_all0 = now();
    long long tk_dep[8] = {0,0,0,0,0,0,0,0}, tk_pro[8] = {0,0,0,0,0,0,0,0}, tk_run[8] = {0,0,0,0,0,0,0,0};
    for (int k = 0; k < p.nops; ++k) {
        const MegaOp op = p.ops[k];

        // ---- dependency: the previous operator's output is complete everywhere -----------------------------
        const int kk = (op.kind == MOP_RESID && op.rows > p.dim) ? 7 : op.kind;
        long long tq0 = now();
        // the previous operator's output is complete everywhere (acquire by one thread, then a CTA barrier)
        auto wait_dependency = [&]() {
            const long long td0 = now();
            if (k > 0) {
                if (tid == 0) {
                    const MegaOp& prev = p.ops[k - 1];
                    const bool sys = (prev.kind == MOP_PARTIAL || prev.kind == MOP_CLS) && prev.tp > 1;
                    mega_wait_counter(&p.done[k - 1], expected * mega_arrivals(prev), &s_abort, p.status, 5u, k, sys);
                }
                named_bar_sync(1, kConsThreads);
            }
            const long long dt = now() - td0;
            t_dep += dt;
            tk_dep[kk] += dt;
            tq0 += dt;   // keep the wait out of the prologue / attention accounting
        };

        if (op.kind == MOP_ATTN) {
            wait_dependency();
            // ---- attention (reference: mat_vec_strided / softmax / vec_mat kernels): `att_split` CTAs per head, each
            // over a contiguous part of the sequence (1 for short contexts, more when the cache rows are many) ----
            // Every part computes its scores (rounded to fp16 like native/mat_vec_kernel.cu:72-73), their maximum m_p and
            // exp-sum l_p; the parts of a head exchange (m_p, l_p) through global memory; the probabilities are rounded
            // to fp16 after the division by the GLOBAL sum (native/softmax_kernel.cu:46); the fp32 partial outputs are
            // summed by the operator that consumes them (single fp16 rounding, native/vec_mat_kernel.cu:41).
            const int S = p.att_split > 1 ? p.att_split : 1;
            if (cta < p.heads_local * S) {
                float* s_sc = reinterpret_cast<float*>(smem_raw + (size_t)p.nstage * p.slot_bytes);
                const int head = cta / S, part = cta - head * S;
                const int nseq = p.pos + 1;
                const int chunk = (nseq + S - 1) / S;
                const int t0 = part * chunk;
                const int t1 = min(nseq, t0 + chunk);
                const size_t stride = (size_t)p.kv_row_stride;
                const __half* kh = op.kcache + (size_t)head * p.head_size + lane * 4;
                const __half* vh = op.vcache + (size_t)head * p.head_size + lane * 4;
                const uint2 qv = *reinterpret_cast<const uint2*>(op.in + (size_t)head * p.head_size + lane * 4);
                float mx = -INFINITY;
                for (int b = t0 + warp * kAttUnroll; b < t1; b += kMegaConsumerWarps * kAttUnroll) {
                    uint2 kv[kAttUnroll];
#pragma unroll
                    for (int u = 0; u < kAttUnroll; ++u)
                        kv[u] = *reinterpret_cast<const uint2*>(kh + (size_t)min(b + u, t1 - 1) * stride);   // unconditional: all loads in flight together
                    float sc[kAttUnroll];
#pragma unroll
                    for (int u = 0; u < kAttUnroll; ++u) {
                        float a = 0.f;
                        a = fma_f16_f32(lo16(kv[u].x), lo16(qv.x), a);
                        a = fma_f16_f32(hi16(kv[u].x), hi16(qv.x), a);
                        a = fma_f16_f32(lo16(kv[u].y), lo16(qv.y), a);
                        a = fma_f16_f32(hi16(kv[u].y), hi16(qv.y), a);
                        sc[u] = a;
                    }
                    transpose_reduce<kAttUnroll>(sc, lane);   // lane (32 / kAttUnroll) * u holds row u
                    constexpr int kPer = 32 / kAttUnroll;
                    const int u = lane / kPer;
                    if ((lane % kPer) == 0 && b + u < t1) {
                        const float sr = __half2float(__float2half_rn(sc[0] * p.scale));
                        s_sc[b + u - t0] = sr;
                        mx = fmaxf(mx, sr);
                    }
                }
                mx = warp_max(mx);
                if (lane == 0) s_att_tmp[warp] = mx;
                named_bar_sync(1, kConsThreads);
                mx = s_att_tmp[0];
#pragma unroll
                for (int w = 1; w < kMegaConsumerWarps; ++w) mx = fmaxf(mx, s_att_tmp[w]);
                named_bar_sync(1, kConsThreads);
                float sum = 0.f;
                for (int i = tid; i < t1 - t0; i += kConsThreads) {
                    const float e = expf(s_sc[i] - mx);
                    s_sc[i] = e;
                    sum += e;
                }
                sum = warp_sum(sum);
                if (lane == 0) s_att_tmp[warp] = sum;
                named_bar_sync(1, kConsThreads);
                float lsum = 0.f;
#pragma unroll
                for (int w = 0; w < kMegaConsumerWarps; ++w) lsum += s_att_tmp[w];
                // exchange with the other parts of this head
                float* ml = op.att_ml + (size_t)head * S * 2;
                float gm = mx, total = lsum, fac = 1.0f;
                if (S > 1) {
                if (tid == 0) {
                    ml[part * 2] = mx;
                    ml[part * 2 + 1] = lsum;
                    __threadfence();
                    red_release_gpu_add(&op.att_cnt[head], 1u);
                    const unsigned int want = ((p.att_seq - 1u) * (unsigned int)p.n_layers + (unsigned int)op.att_layer + 1u) * (unsigned int)S;
                    mega_wait_counter(&op.att_cnt[head], want, &s_abort, p.status, 6u, k, false);
                }
                named_bar_sync(1, kConsThreads);
                gm = -INFINITY;
                for (int q = 0; q < S; ++q) gm = fmaxf(gm, __ldcg(&ml[q * 2]));
                total = 0.f;
                for (int q = 0; q < S; ++q) {
                    const float lq = __ldcg(&ml[q * 2 + 1]);
                    if (lq > 0.f) total += lq * expf(__ldcg(&ml[q * 2]) - gm);
                }
                fac = (t1 > t0) ? expf(mx - gm) : 0.f;
                }
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int b = t0 + warp * kAttUnroll; b < t1; b += kMegaConsumerWarps * kAttUnroll) {
                    uint2 vv[kAttUnroll];
#pragma unroll
                    for (int u = 0; u < kAttUnroll; ++u)
                        vv[u] = *reinterpret_cast<const uint2*>(vh + (size_t)min(b + u, t1 - 1) * stride);
#pragma unroll
                    for (int u = 0; u < kAttUnroll; ++u) {
                        if (b + u < t1) {
                            const unsigned short pr = __half_as_ushort(__float2half_rn(s_sc[b + u - t0] * fac / total));
                            acc[0] = fma_f16_f32(pr, lo16(vv[u].x), acc[0]);
                            acc[1] = fma_f16_f32(pr, hi16(vv[u].x), acc[1]);
                            acc[2] = fma_f16_f32(pr, lo16(vv[u].y), acc[2]);
                            acc[3] = fma_f16_f32(pr, hi16(vv[u].y), acc[3]);
                        }
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) s_att_acc[warp][lane * 4 + e] = acc[e];
                named_bar_sync(1, kConsThreads);
                if (tid < p.head_size) {
                    float o = 0.f;
#pragma unroll
                    for (int w = 0; w < kMegaConsumerWarps; ++w) o += s_att_acc[w][tid];
                    if (S > 1) op.att_part[((size_t)head * S + part) * p.head_size + tid] = o;
                    else op.out[0][(size_t)head * p.head_size + tid] = __float2half_rn(o);   // native/vec_mat_kernel.cu:41
                }
                __threadfence();
                named_bar_sync(1, kConsThreads);
            }
            if (tid == 0) red_release_gpu_add(&p.done[k], 1u);
            t_attn += now() - tq0;
            continue;
        }

        if (op.kind == MOP_ARGMAX) {
            wait_dependency();
            // ---- greedy sample on CTA 0 (native/argmax_kernel.cu:8-46, lowest index on ties) --------------------
            if (cta == 0) {
                float best = -INFINITY;
                int best_i = 0x7fffffff;
                for (int i = tid; i < p.vocab; i += kConsThreads) {
                    const float v = __half2float(p.logits[i]);
                    if (v > best) { best = v; best_i = i; }
                }
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
                }
                if (lane == 0) { s_best_v[warp] = best; s_best_i[warp] = best_i; }
                named_bar_sync(1, kConsThreads);
                if (tid == 0) {
                    for (int w = 1; w < kMegaConsumerWarps; ++w)
                        if (s_best_v[w] > best || (s_best_v[w] == best && s_best_i[w] < best_i)) { best = s_best_v[w]; best_i = s_best_i[w]; }
                    if (p.write_token) p.tokens[p.next_pos] = (best_i == 0x7fffffff) ? 0 : best_i;
                }
            }
            if (tid == 0) red_release_gpu_add(&p.done[k], 1u);
            continue;
        }

        // ---- weight operators ------------------------------------------------------------------------------
        const int first = my_first(op), cnt = my_count(op, first);
        const int group = warp / op.kw;
        const int kw_id = warp - group * op.kw;
        const bool in_group = group < op.groups;
        const int u = kw_id * 32 + lane;
        const bool active = in_group && u < op.units;
        const bool is_int4 = op.fmt == 0;
        const int nx = is_int4 ? 32 : 16;     // inputs per lane: one 16-byte weight vector (int4) or two (fp16)
        const int e0 = u * nx;

        // Input vector, once per CTA: every consumer thread fetches 8 consecutive elements (the RMSNorm weights for
        // them are fetched BEFORE the dependency wait, they are constants), the vector is normalised cooperatively
        // (native/rmsnorm_kernel.cu:12-35) and staged in shared memory; each lane then takes its slice from there.
        __half* s_vec = reinterpret_cast<__half*>(smem_raw + (size_t)p.nstage * p.slot_bytes);   // shares the attention scratch
        const int nvec8 = op.rows >> 3;   // 16-byte pieces of the vector
        uint4 gam[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        if (op.pro != 0) {
#pragma unroll
            for (int q = 0; q < 2; ++q)
                if (tid + q * kConsThreads < nvec8) gam[q] = *reinterpret_cast<const uint4*>(op.gamma + (size_t)(tid + q * kConsThreads) * 8);
        }
        wait_dependency();

        if (ML2_MULTI && op.passes > 1) {
            MegaShared sh;
            sh.smem = smem_raw; sh.full_bar = full_bar; sh.empty_bar = empty_bar; sh.done_bar = done_bar; sh.free_bar = free_bar;
            sh.red = &s_red[0][0][0]; sh.abort_flag = &s_abort;
            sh.status = p.status; sh.nstage = p.nstage; sh.slot_bytes = p.slot_bytes;
            const long long trun0 = now();
            mega_multisweep_op(op, k, sh, first, cnt, n_base, st_base, ph_base);
            tk_run[kk] += now() - trun0;
            n_base += (uint32_t)cnt;
            st_base += cnt % p.nstage;
            ph_base ^= (uint32_t)(cnt / p.nstage) & 1u;
            if (st_base >= p.nstage) { st_base -= p.nstage; ph_base ^= 1u; }
            continue;
        }

        XSlice xs;
        {
            const __half* src = op.in;
            if (op.pro == 2) src = p.embed + (size_t)p.tokens[p.pos] * op.rows;   // native/embedding_kernel.cu:6-12
            if (op.pro == 0 && op.att_part != nullptr && p.att_split > 1) {
                // input = attention output of the split path: fp32 partials of the parts, summed in part order and
                // rounded to fp16 once (native/vec_mat_kernel.cu:41)
                const int S = p.att_split;
                for (int i = tid; i < nvec8; i += kConsThreads) {
                    const int e = i * 8, head = e / p.head_size, d = e - head * p.head_size;
                    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    for (int q = 0; q < S; ++q) {
                        const float4* pp = reinterpret_cast<const float4*>(op.att_part + ((size_t)head * S + q) * p.head_size + d);
                        const float4 p0 = __ldcg(pp), p1 = __ldcg(pp + 1);
                        a[0] += p0.x; a[1] += p0.y; a[2] += p0.z; a[3] += p0.w;
                        a[4] += p1.x; a[5] += p1.y; a[6] += p1.z; a[7] += p1.w;
                    }
                    uint32_t o4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        o4[j] = (uint32_t)__half_as_ushort(__float2half_rn(a[2 * j])) | ((uint32_t)__half_as_ushort(__float2half_rn(a[2 * j + 1])) << 16);
                    *reinterpret_cast<uint4*>(s_vec + (size_t)i * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                }
            } else if (op.pro == 0) {
                for (int i = tid; i < nvec8; i += kConsThreads)
                    *reinterpret_cast<uint4*>(s_vec + (size_t)i * 8) = *reinterpret_cast<const uint4*>(src + (size_t)i * 8);
            } else {
                uint4 xv[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                float ss = 0.f;
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int i = tid + q * kConsThreads;
                    if (i < nvec8) {
                        xv[q] = *reinterpret_cast<const uint4*>(src + (size_t)i * 8);
                        if (op.pro == 2 && cta == 0) *reinterpret_cast<uint4*>(p.x + (size_t)i * 8) = xv[q];  // residual stream := embedding row
                        if (op.pro == 3) {
                            // residual add of a row-sharded mat-vec: x := half(float(x) + sum over ranks of their fp32
                            // partials), ranks in fixed order so that every rank rounds the same value
                            // (rounding point of native/mat_vec_kernel.cu:154-156)
                            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                            for (int r = 0; r < op.tp; ++r) {
                                const float4* pr = reinterpret_cast<const float4*>(op.recv + (size_t)r * op.rows + (size_t)i * 8);
                                const float4 p0 = pr[0], p1 = pr[1];
                                acc[0] += p0.x; acc[1] += p0.y; acc[2] += p0.z; acc[3] += p0.w;
                                acc[4] += p1.x; acc[5] += p1.y; acc[6] += p1.z; acc[7] += p1.w;
                            }
                            uint32_t w4r[4] = {xv[q].x, xv[q].y, xv[q].z, xv[q].w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float lo = half_bits_to_float(lo16(w4r[e])) + acc[2 * e];
                                const float hi = half_bits_to_float(hi16(w4r[e])) + acc[2 * e + 1];
                                w4r[e] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
                            }
                            xv[q] = make_uint4(w4r[0], w4r[1], w4r[2], w4r[3]);
                            if (cta == 0) *reinterpret_cast<uint4*>(op.x_next + (size_t)i * 8) = xv[q];
                        }
                        const uint32_t w4[4] = {xv[q].x, xv[q].y, xv[q].z, xv[q].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // fp16 x fp16 is exact in fp32: the mixed FMA gives fmaf(float(x), float(x), ss) bit for bit
                            ss = fma_f16_f32(lo16(w4[e]), lo16(w4[e]), ss);
                            ss = fma_f16_f32(hi16(w4[e]), hi16(w4[e]), ss);
                        }
                    }
                }
                ss = warp_sum(ss);
                float* part = &s_part[k & 1][0][0];
                if (lane == 0) part[warp] = ss;
                named_bar_sync(1, kConsThreads);
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kMegaConsumerWarps; ++w) tot += part[w];
                const float rms = 1.0f / sqrtf(tot / (float)op.rows + p.eps);
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int i = tid + q * kConsThreads;
                    if (i < nvec8) {
                        const uint32_t w4[4] = {xv[q].x, xv[q].y, xv[q].z, xv[q].w};
                        const uint32_t g4[4] = {gam[q].x, gam[q].y, gam[q].z, gam[q].w};
                        uint32_t o4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float lo = rms * half_bits_to_float(lo16(g4[e])) * half_bits_to_float(lo16(w4[e]));
                            const float hi = rms * half_bits_to_float(hi16(g4[e])) * half_bits_to_float(hi16(w4[e]));
                            o4[e] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
                        }
                        *reinterpret_cast<uint4*>(s_vec + (size_t)i * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                    }
                }
            }
            named_bar_sync(1, kConsThreads);
            uint32_t xr[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) xr[i] = 0u;
            if (active) {
                const uint4* sv = reinterpret_cast<const uint4*>(s_vec + e0);
                const int nv = is_int4 ? 4 : 2;
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    if (v < nv && e0 + v * 8 + 8 <= op.rows) {
                        const uint4 t = sv[v];
                        xr[4 * v] = t.x; xr[4 * v + 1] = t.y; xr[4 * v + 2] = t.z; xr[4 * v + 3] = t.w;
                    }
                }
            }
            if (is_int4) {
                make_xslice(xr, xs);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) xs.xp[i] = xr[i];
            }
        }

        t_pro += now() - tq0;
        tk_pro[kk] += now() - tq0;
        const long long trun0 = now();
        const int g = u >> 2;
        const int zshift = (g & 7) * 4;
        const uint32_t w_off = (uint32_t)(active ? u : 0) * (is_int4 ? 16u : 32u);
        const uint32_t z_off = op.woff_z + (uint32_t)(active ? (g >> 3) : 0) * 4u;
        const uint32_t s_off = op.woff_s + (uint32_t)(active ? g : 0) * 2u;
        const uint32_t w_row = (uint32_t)op.wsize * 4u, z_row = (uint32_t)op.zsize * 4u, s_row = (uint32_t)op.ssize * 2u;
        const uint32_t ring = smem_u32(smem_raw);
        // arrival weights: the fixed barrier count is met by (kw - 1) single arrivals + one weighted arrival per tile
        const uint32_t my_arrive = (kw_id == 0) ? (kBarCount - (uint32_t)op.kw + 1u) : 1u;

        // tiles i = group, group + groups, ... belong to this group (idle warps take none)
        int st = st_base + group;
        uint32_t ph = ph_base;
        while (st >= p.nstage) { st -= p.nstage; ph ^= 1u; }
        for (int i = group; in_group && i < cnt; i += op.groups) {
            const uint32_t n = n_base + (uint32_t)i;
            long long tw0 = now();
            wait_or_abort(&full_bar[st], ph, &s_abort, p.status, 2u, k);
            t_full += now() - tw0;
            const int slot = (int)(n % kMegaRedSlots);
            bool slot_ready = n < (uint32_t)kMegaRedSlots;
            float resid[2] = {0.f, 0.f};
            if (op.kind == MOP_RESID && kw_id == 0 && (lane & 7) == 0 && (lane >> 3) < op.rwc) {
                const int tile = first + i * ncta;
                for (int c = 0; c < op.nch; ++c) {
                    const int row = (tile * op.nch + c) * op.rwc + (lane >> 3);
                    if (row < op.cols) resid[c] = __half2float(op.out[0][row]);
                }
            }
            for (int c = 0; c < op.nch; ++c) {
                // chunk c = rows [c*rwc, c*rwc + rwc) of the tile; they sit in run (c*rwc / run_rows) at row rin0 of that run
                const int trow = c * op.rwc;
                const int run = (op.run_rows == 8) ? (trow >> 3) : (op.run_rows == 4 ? (trow >> 2) : (trow >> 1));
                const int rin0 = trow - run * op.run_rows;
                const uint32_t cbase = ring + (uint32_t)st * p.slot_bytes + (uint32_t)run * op.chunk_bytes;
                const uint32_t cb = cbase;   // weights of the run start here
                const uint32_t cw = cbase + (uint32_t)rin0 * w_row;
                const uint32_t cz = cbase + (uint32_t)rin0 * z_row;
                const uint32_t cs = cbase + (uint32_t)rin0 * s_row;
                (void)cb;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (p.debug & 1) {
                } else if (is_int4) {
                    mega_int4_rows(xs, cw + w_off, cz + z_off, cs + s_off, w_row, z_row, s_row, zshift, active, v);
                } else {
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        if (r < op.rwc) {
                            uint4 wv, wu;
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w)
                                         : "r"(cw + w_off + r * w_row));
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(wu.x), "=r"(wu.y), "=r"(wu.z), "=r"(wu.w)
                                         : "r"(cw + w_off + r * w_row + 16u));
                            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                            a0 = fma_f16_f32(lo16(wv.x), lo16(xs.xp[0]), a0);
                            a1 = fma_f16_f32(hi16(wv.x), hi16(xs.xp[0]), a1);
                            a2 = fma_f16_f32(lo16(wv.y), lo16(xs.xp[1]), a2);
                            a3 = fma_f16_f32(hi16(wv.y), hi16(xs.xp[1]), a3);
                            a0 = fma_f16_f32(lo16(wv.z), lo16(xs.xp[2]), a0);
                            a1 = fma_f16_f32(hi16(wv.z), hi16(xs.xp[2]), a1);
                            a2 = fma_f16_f32(lo16(wv.w), lo16(xs.xp[3]), a2);
                            a3 = fma_f16_f32(hi16(wv.w), hi16(xs.xp[3]), a3);
                            a0 = fma_f16_f32(lo16(wu.x), lo16(xs.xp[4]), a0);
                            a1 = fma_f16_f32(hi16(wu.x), hi16(xs.xp[4]), a1);
                            a2 = fma_f16_f32(lo16(wu.y), lo16(xs.xp[5]), a2);
                            a3 = fma_f16_f32(hi16(wu.y), hi16(xs.xp[5]), a3);
                            a0 = fma_f16_f32(lo16(wu.z), lo16(xs.xp[6]), a0);
                            a1 = fma_f16_f32(hi16(wu.z), hi16(xs.xp[6]), a1);
                            a2 = fma_f16_f32(lo16(wu.w), lo16(xs.xp[7]), a2);
                            a3 = fma_f16_f32(hi16(wu.w), hi16(xs.xp[7]), a3);
                            v[r] = active ? ((a0 + a1) + (a2 + a3)) : 0.f;
                        }
                    }
                }
                if (c == op.nch - 1) {
                    // last read of the stage by this warp: hand it back to the producer
                    __syncwarp();
                    if (lane == 0) mbar_arrive_n(&empty_bar[st], my_arrive);
                }
                if (!(p.debug & 2)) transpose_reduce<4>(v, lane);
                if (!slot_ready) {
                    long long tf0 = now();
                    wait_or_abort(&free_bar[slot], ((n / kMegaRedSlots) - 1u) & 1u, &s_abort, p.status, 4u, k);
                    t_free += now() - tf0;
                    slot_ready = true;
                }
                if ((lane & 7) == 0 && (lane >> 3) < op.rwc) s_red[slot][kw_id][c * op.rwc + (lane >> 3)] = v[0];
                if (op.kind == MOP_RESID && kw_id == 0 && (lane & 7) == 0 && (lane >> 3) < op.rwc)
                    s_red[slot][op.kw][c * op.rwc + (lane >> 3)] = resid[c];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_n(&done_bar[slot], my_arrive);
            st += op.groups;
            while (st >= p.nstage) { st -= p.nstage; ph ^= 1u; }
        }
        tk_run[kk] += now() - trun0;
        n_base += (uint32_t)cnt;
        st_base += cnt % p.nstage;   // one division per operator
        ph_base ^= (uint32_t)(cnt / p.nstage) & 1u;
        if (st_base >= p.nstage) { st_base -= p.nstage; ph_base ^= 1u; }
    }
    if (kProf && p.prof && tid == 0) {
        long long* o = p.prof + (size_t)cta * 64;
        o[0] = now() - t_all0; o[1] = t_dep; o[2] = t_full; o[3] = t_free; o[4] = t_attn; o[5] = t_pro;
        for (int q = 0; q < 8; ++q) { o[8 + q] = tk_dep[q]; o[16 + q] = tk_pro[q]; o[24 + q] = tk_run[q]; }
    }
}

}  // namespace ml2
