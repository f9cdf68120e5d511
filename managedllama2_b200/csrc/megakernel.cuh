// One persistent kernel per token: the whole operator sequence of Transformer.Forward
// (src/Transformer.cs:158-190 of GilesBathgate/ManagedLlama2) runs inside a single cooperative launch with
// one CTA per SM, so HBM streaming never stops at an operator boundary.
//
//   * producer warp   walks the token's operator list and streams every weight tile this CTA owns, operator
//                     after operator, into one shared-memory ring (1-D bulk async copies, mbarrier completion).
//                     Weights do not depend on activations, so it runs ahead of the arithmetic by the depth of
//                     the ring, across operator boundaries.
//   * rows            every operator's output rows are cut into contiguous, balanced ranges, one per CTA; a CTA
//                     streams its range as tiles of up to `rmax` rows (three copies per tile: packed weights, zero
//                     words, scales). Tile sizes are spread evenly over the range, so all CTAs run the same number
//                     of arithmetic steps.
//   * consumer warps  work in groups of `kw` warps (one group spans a whole weight row: a lane owns one or two
//                     16-byte weight vectors of every row, its inputs stationary in registers). ALL groups share a
//                     tile: group g takes rows g, g + G, ... of it. A group sums its k-warps through shared memory
//                     behind a named barrier and its first warp runs the operator's tail (residual add, SwiGLU,
//                     stores) with the reference's fp16 rounding points. No separate finalizer warps.
//   * hand-off        when a CTA has stored its share of an operator, ONE thread publishes it (release) on the
//                     operator's device-wide counter; the next operator starts when the counter is complete
//                     (acquire by one thread, CTA barrier), builds its prepared input table cooperatively
//                     (RMSNorm applied where the reference runs rmsnorm first) and goes on with tiles that the
//                     producer has already brought in.
//   * attention       is an operator without weights, with the steps and rounding points of the reference's
//                     rope / scores / softmax / values kernels: one CTA per head for short contexts, several CTAs
//                     per head (parts of the sequence, maximum / exp-sum exchanged through global memory) for long
//                     ones. The rotation of q and of the new key row (native/rope_kernel.cu) happens here.
//
// Every wait is bounded by a cycle budget; when it runs out the CTA records an error word, stops waiting and runs
// to its end.
#pragma once

#include "stream_matvec.cuh"

namespace ml2 {

enum MegaOpKind : int { MOP_QKV = 0, MOP_ATTN = 1, MOP_RESID = 2, MOP_SWIGLU = 3, MOP_CLS = 4, MOP_ARGMAX = 5, MOP_PARTIAL = 6 };

struct MegaOp {
    int kind;
    int fmt;                 // 0 int4, 1 fp16 weights
    int pro;                 // 0 plain input, 1 RMSNorm(in, gamma), 2 RMSNorm(embedding row of the token, gamma),
                             // 3 RMSNorm(in + sum over ranks of recv, gamma): residual add of a row-sharded mat-vec
    int rows, cols, nmat;    // d_in, d_out per matrix, matrices
    int paired;              // 1: a unit of work is row i of mat[0] together with row i of mat[1] (SwiGLU)
    int wrow, zrow, srow;    // bytes of one output row in the weight / zero / scale arrays (fp16 weights: 2 * rows, 0, 0)
    int units;               // 16-byte weight vectors (lane slots) per row
    int kw, groups, np;      // warps per group, groups per CTA, weight vectors per lane and row (1 or 2)
    int gran;                // rows per alignment granule: every tile is a whole number of granules
    int rmax;                // units (rows, or row pairs) of a full tile
    int off_z, off_s, run_bytes;   // shared-memory layout of one run (the rows of one matrix in a tile)
    int has_tiles;           // weight operator
    int rot, seg_rot;        // rotation of the CTA -> row range assignment, per operator and per segment
    int ngran, gmax;         // granules of a segment (cols / gran), granules of a full tile (rmax / gran)
    float inv_ncta, inv_gmax;   // reciprocals used by the tile arithmetic (1 / CTAs of the launch, 1 / gmax)
    int tp;                  // ranks summed into the input (pro 3) / receiving the output (MOP_PARTIAL, sharded MOP_CLS)
    int out_row0;            // sharded classifier: first vocabulary row of this rank
    int att_layer;           // layer index (the split-attention counters advance once per layer and token)
    QWPtrs mat[3];
    __half* out[3];
    const __half* in;        // pro 3: the residual stream BEFORE the all-reduced update
    const __half* gamma;
    __half* kcache;          // attention: this layer's caches (the new key row is rotated in place)
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
    unsigned int seq_no;       // 1, 2, 3, ... : arrivals expected on a counter = seq_no * gridDim.x (* tp where ranks share it)
    int dim, head_size, heads_local, kv_row_stride, vocab;
    float eps, scale;
    int nstage, slot_bytes, att_cap;
    int att_split;             // CTAs per head for this token's attention (1: one CTA per head)
    unsigned int att_seq;      // 1, 2, 3, ... over the tokens that used the split path
    int n_layers;
    long long wait_cycles;     // budget of every wait, in SM clock cycles
    long long* prof;           // optional [gridDim.x][64] cycle counters (diagnostics), may be null
};

constexpr int kMegaConsumerWarps = 21;   // 4 groups of 5, 3 of 7, 5 of 4, 2 of 10
constexpr int kMegaWarps = kMegaConsumerWarps + 2;   // + copy warp + tail warp
constexpr int kMegaThreads = kMegaWarps * 32;
constexpr int kMegaConsThreads = kMegaConsumerWarps * 32;
constexpr int kMegaMaxStages = 6;
constexpr int kMegaMaxGroups = 8;     // named barriers 2 .. 9
constexpr int kMegaGroupRows = 8;     // physical rows of one tile that one group may own
constexpr int kMegaRedBufs = 8;       // tiles whose k-warp partials may be waiting for their tail (more than the ring depth + 1)
constexpr int kMegaMaxSplit = 8;      // CTAs per head of the split attention
constexpr int kAttUnroll = 8;         // cache rows a warp keeps in flight
constexpr uint32_t kMegaBarCount = 64;  // fixed arrival count of the empty barriers: the working warps of an operator add up to it
constexpr int kMegaNormVecs = 3;      // 16-byte pieces of a normalised input vector one thread may hold

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v)
{
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p)
{
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_cg_v2(const void* p)
{
    uint2 v;
    asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// arrivals one rank's CTAs make on an operator's counter per token: one per CTA; where every rank publishes on every
// rank's counter (row-sharded mat-vec, vocabulary-sharded classifier) tp times as many
__host__ __device__ __forceinline__ unsigned int mega_arrivals(const MegaOp& op)
{
    const bool shared = (op.kind == MOP_PARTIAL || op.kind == MOP_CLS) && op.tp > 1;
    return shared ? (unsigned int)op.tp : 1u;
}

// ---- bounded waits ----------------------------------------------------------------------------------------------------
struct MegaWait {
    volatile unsigned int* abort_flag;   // shared memory: some role of this CTA gave up
    DeviceStatus* status;
    long long budget;                    // SM cycles
};

__device__ __forceinline__ void mega_give_up(const MegaWait& w, unsigned int code, int detail)
{
    *w.abort_flag = 1;
    if (atomicCAS(&w.status->error, 0u, code) == 0u) w.status->detail = (unsigned int)detail;
}

// A waiting thread must not take issue slots from the arithmetic warps of its scheduler: between polls it sleeps
// (`sleep_ns`; the suspend-time hint of try_wait alone turned out to park a thread only briefly, and a spinning thread
// costs a third of a scheduler's slots). It wakes to look at the barrier, the abort flag and the clock.
__device__ __forceinline__ void mega_wait_bar(uint64_t* bar, uint32_t parity, const MegaWait& w, unsigned int code, int detail,
                                              unsigned int sleep_ns)
{
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        if (mbar_try_wait_suspend(bar, parity, 1000u)) return;
        __nanosleep(sleep_ns);
        if (*w.abort_flag) return;
        if (clock64() - t0 > w.budget) break;
    }
    mega_give_up(w, code, detail);
}

__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t n)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}

// Device-wide dependency: waits until `counter` has collected `expected` arrivals.
__device__ __forceinline__ void mega_wait_counter(const unsigned int* counter, unsigned int expected, const MegaWait& w, unsigned int code,
                                                  int detail, bool sys_scope)
{
    const long long t0 = clock64();
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        const unsigned int seen = sys_scope ? ld_acquire_sys(counter) : ld_acquire_gpu(counter);
        if ((int)(seen - expected) >= 0) return;
        if ((i & 15u) == 15u) {
            if (*w.abort_flag || ld_acquire_gpu(&w.status->error)) { *w.abort_flag = 1; return; }
            if (clock64() - t0 > w.budget) break;
        }
    }
    mega_give_up(w, code, detail);
}

// ---- row ranges and tiles ------------------------------------------------------------------------------------------------
// Segment s of an operator (matrix s of QKV; the only segment otherwise) has cols / gran granules; CTA c owns a
// contiguous, balanced range of them, cut into tiles whose sizes differ by at most one granule.
struct MegaSeg {
    int row0;          // first unit of this CTA's range
    int nt;            // tiles
    int base, extra;   // granules per tile: base (+1 for the first `extra` tiles)
};

// x / d for 0 <= x < 2^23 and small d, without the integer-division routine (`inv_d` = 1 / d rounded to float)
__device__ __forceinline__ int mega_div(int x, int d, float inv_d)
{
    int q = __float2int_rz((float)x * inv_d);
    const int r = x - q * d;
    q += (r >= d ? 1 : 0) - (r < 0 ? 1 : 0);
    return q;
}

__device__ __forceinline__ MegaSeg mega_segment(const MegaOp& op, int seg, int cta, int ncta)
{
    MegaSeg s;
    int c = cta + op.rot + seg * op.seg_rot;
    c -= mega_div(c, ncta, op.inv_ncta) * ncta;
    const int G = op.ngran;                         // granules of the segment (< 2^23 / ncta)
    const int g0 = mega_div(c * G, ncta, op.inv_ncta), g1 = mega_div((c + 1) * G, ncta, op.inv_ncta);
    const int ng = g1 - g0;
    s.row0 = g0 * op.gran;
    s.nt = mega_div(ng + op.gmax - 1, op.gmax, op.inv_gmax);   // gmax = granules of a full tile
    s.base = 0;
    s.extra = 0;
    if (s.nt > 0) {
        s.base = mega_div(ng, s.nt, __frcp_rn((float)s.nt));
        s.extra = ng - s.base * s.nt;
    }
    return s;
}

__device__ __forceinline__ int mega_segments(const MegaOp& op) { return op.paired ? 1 : op.nmat; }

// ---- shared-memory objects --------------------------------------------------------------------------------------------
struct MegaShared {
    unsigned char* ring;      // nstage * slot_bytes, then the table / scratch area
    unsigned char* table;
    uint64_t* full_bar;
    uint64_t* empty_bar;
    float* red;               // [kMegaRedBufs][kMegaConsumerWarps][kMegaGroupRows]
    float* part;              // [2][kMegaConsumerWarps] sum-of-squares partials
    float* resid;             // [kMegaRedBufs][kMegaMaxGroups][kMegaGroupRows] residual values of the tiles in flight
};

// ---- prepared input table ---------------------------------------------------------------------------------------------
// int4 operators: lane slot u (32 consecutive inputs = one 16-byte weight vector of every row, one quarter of a
// quantisation group) owns five 16-byte vectors, stored as table[q * tab_n + u]:
//   q = 0..3   the inputs of packed word q as fp16 pairs (x0,x4) (x1,x5) (x2,x6) (x3,x7)   (see word_dot)
//   q = 4      accumulator start values -1024 * S(even inputs), -1024 * S(odd inputs), and the sum of the inputs
//              of the slot's whole quantisation group (zero-point term)
// fp16 operators: table[u] = the 8 inputs of slot u.
// Slots past the end of the row hold zeros.
__device__ __forceinline__ void mega_table_store_int4(uint4* tab, int tab_n, int i, uint4 t)
{
    // thread i holds inputs [8i, 8i + 8): word (i & 3) of slot (i >> 2); the four threads of a slot are adjacent lanes
    const uint32_t x0 = __byte_perm(t.x, t.z, 0x5410), x1 = __byte_perm(t.x, t.z, 0x7632);
    const uint32_t x2 = __byte_perm(t.y, t.w, 0x5410), x3 = __byte_perm(t.y, t.w, 0x7632);
    float ev = half_bits_to_float(lo16(t.x)) + half_bits_to_float(lo16(t.y)) + half_bits_to_float(lo16(t.z)) + half_bits_to_float(lo16(t.w));
    float od = half_bits_to_float(hi16(t.x)) + half_bits_to_float(hi16(t.y)) + half_bits_to_float(hi16(t.z)) + half_bits_to_float(hi16(t.w));
    ev += __shfl_xor_sync(0xffffffffu, ev, 1);
    od += __shfl_xor_sync(0xffffffffu, od, 1);
    ev += __shfl_xor_sync(0xffffffffu, ev, 2);
    od += __shfl_xor_sync(0xffffffffu, od, 2);
    float grp = ev + od;
    grp += __shfl_xor_sync(0xffffffffu, grp, 4);
    grp += __shfl_xor_sync(0xffffffffu, grp, 8);
    const int u = i >> 2, q = i & 3;
    tab[q * tab_n + u] = make_uint4(x0, x1, x2, x3);
    if (q == 0) tab[4 * tab_n + u] = make_uint4(__float_as_uint(-1024.f * ev), __float_as_uint(-1024.f * od), __float_as_uint(grp), 0u);
}

struct MegaSlice {
    uint32_t xp[16];
    float a0, b0, c1g;
};

template <bool INT4>
__device__ __forceinline__ void mega_load_slice(uint32_t tab, int tab_n, int u, MegaSlice& x)
{
    if (INT4) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 t = lds_v4(tab + (uint32_t)(v * tab_n + u) * 16u);
            x.xp[4 * v] = t.x; x.xp[4 * v + 1] = t.y; x.xp[4 * v + 2] = t.z; x.xp[4 * v + 3] = t.w;
        }
        const uint4 c = lds_v4(tab + (uint32_t)(4 * tab_n + u) * 16u);
        x.a0 = __uint_as_float(c.x); x.b0 = __uint_as_float(c.y); x.c1g = __uint_as_float(c.z);
    } else {
        const uint4 t = lds_v4(tab + (uint32_t)u * 16u);
        x.xp[0] = t.x; x.xp[1] = t.y; x.xp[2] = t.z; x.xp[3] = t.w;
        x.a0 = x.b0 = x.c1g = 0.f;
    }
}

// one 16-byte weight vector against the lane's prepared inputs
template <bool INT4>
__device__ __forceinline__ float mega_item(const uint4& wv, const MegaSlice& x)
{
#ifdef ML2_DIAG_NOMATH
    return __uint_as_float(wv.x ^ x.xp[0]);   // pipeline probe: loads stay, arithmetic goes
#endif
    if (INT4) {
        float A = x.a0, B = x.b0, D = 0.f;
        word_dot(wv.x, x.xp + 0, A, B, D);
        word_dot(wv.y, x.xp + 4, A, B, D);
        word_dot(wv.z, x.xp + 8, A, B, D);
        word_dot(wv.w, x.xp + 12, A, B, D);
        return fmaf(B, 0.0625f, A) + D;
    } else {
        float a = 0.f, b = 0.f;
        a = fma_f16_f32(lo16(wv.x), lo16(x.xp[0]), a);
        b = fma_f16_f32(hi16(wv.x), hi16(x.xp[0]), b);
        a = fma_f16_f32(lo16(wv.y), lo16(x.xp[1]), a);
        b = fma_f16_f32(hi16(wv.y), hi16(x.xp[1]), b);
        a = fma_f16_f32(lo16(wv.z), lo16(x.xp[2]), a);
        b = fma_f16_f32(hi16(wv.z), hi16(x.xp[2]), b);
        a = fma_f16_f32(lo16(wv.w), lo16(x.xp[3]), a);
        b = fma_f16_f32(hi16(wv.w), hi16(x.xp[3]), b);
        return a + b;
    }
}

// ---- arithmetic of one batch: four (row, vector) items of this lane -------------------------------------------------
// Item i = row (i / NP) of the batch, weight vector (i % NP) of the lane. After the dot products a transposing
// reduction inside each quad of lanes (= one quantisation group) leaves item j's group sum on lane j of the quad,
// which applies that row's zero point and scale ONCE (instead of every lane for every row); the quads are then
// summed. Returns the warp's row totals: row r on the lanes with ((lane & 3) / NP) == r.
// NP == 1: the lane's slice `xs0` stays in registers for the whole operator. NP == 2: both slices are reloaded from
// the table in shared memory for every batch (two of them do not fit the register budget of a 704-thread CTA).
//   wa[r]   shared-memory address of this lane's first weight vector in row r of the batch
//   du      byte distance to the lane's second vector (NP == 2)
//   za, sa  addresses of the zero word and the scale that THIS lane applies (its item's row and quantisation group)
template <bool INT4, int NP>
__device__ __forceinline__ float mega_batch(const MegaSlice& xs0, uint32_t tab, int tab_n, int u0, int u1, const uint32_t (&wa)[4 / NP],
                                            uint32_t du, uint32_t za, uint32_t sa, int zshift, int nitems, int lane)
{
    constexpr int NR = 4 / NP;
    uint4 wv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wv[i] = lds_v4(wa[i / NP] + ((i % NP) ? du : 0u));
    uint32_t zw = 0;
    unsigned short sc = 0;
    if (INT4) {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw) : "r"(za));
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sc) : "r"(sa));
    }
    float t[4] = {0.f, 0.f, 0.f, 0.f};
    float cg;
    if (NP == 1) {
        cg = xs0.c1g;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (i < nitems) t[i] = mega_item<INT4>(wv[i], xs0);   // warp-uniform: a short last batch costs only the rows it has
    } else {
        float cq[NP];
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            MegaSlice x;
            mega_load_slice<INT4>(tab, tab_n, q ? u1 : u0, x);
            cq[q] = x.c1g;
#pragma unroll
            for (int r = 0; r < NR; ++r)
                if (r * NP + q < nitems) t[r * NP + q] = mega_item<INT4>(wv[r * NP + q], x);
        }
        cg = (lane & 1) ? cq[NP - 1] : cq[0];
    }
    // 4 x 4 transposing reduction inside the quad: lane j of the quad ends with the quad's sum of item j
    const bool b2 = (lane & 2) != 0, b1 = (lane & 1) != 0;
    const float s0 = b2 ? t[0] : t[2], k0 = b2 ? t[2] : t[0];
    const float s1 = b2 ? t[1] : t[3], k1 = b2 ? t[3] : t[1];
    const float q0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 2);
    const float q1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 2);
    const float sn = b1 ? q0 : q1, kp = b1 ? q1 : q0;
    float v = kp + __shfl_xor_sync(0xffffffffu, sn, 1);
    if (INT4) {
        const float zf = (float)((zw >> zshift) & 0xFu);
        v = half_bits_to_float(sc) * fmaf(-zf, cg, v);
    }
    if (NP == 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    return v;
}

// ---- the operator's tail for one unit (the reference's rounding points) ---------------------------------------------
__device__ __forceinline__ void mega_epilogue(const MegaOp* __restrict__ gp, int kind, __half* outp, int row, float sa, float sb, float resid)
{
    switch (kind) {
    case MOP_QKV:
        // fp16 store of the mat-vec result (native/mat_vec_kernel.cu:175); k and v go straight into the cache row
        outp[row] = __float2half_rn(sa);
        break;
    case MOP_RESID:
        outp[row] = __float2half_rn(sa + resid);   // native/mat_vec_kernel.cu:154-156
        break;
    case MOP_SWIGLU: {
        float val = sa;                             // native/mat_vec_kernel.cu:218-222
        val *= 1.0f / (1.0f + expf(-val));
        val *= sb;
        outp[row] = __float2half_rn(val);
        break;
    }
    case MOP_PARTIAL: {
        // row-sharded mat-vec: this rank's fp32 partial goes straight into every rank's receive zone (plain peer
        // stores over NVLink); the residual add and the single fp16 rounding happen where the sum is consumed
        const int tp = gp->tp;
        for (int q = 0; q < tp; ++q) gp->peer_out[q][row] = sa;
        break;
    }
    default: {   // MOP_CLS
        const int tp = gp->tp;
        if (tp > 1) {
            // vocabulary-sharded classifier: every rank ends up with the full logits
            const __half hv = __float2half_rn(sa);
            const int r0 = gp->out_row0;
            for (int q = 0; q < tp; ++q) gp->peer_logits[q][r0 + row] = hv;
        } else {
            outp[row] = __float2half_rn(sa);        // native/mat_vec_kernel.cu:43
        }
        break;
    }
    }
}

struct MegaRing {
    int slot;
    uint32_t parity;
};
__device__ __forceinline__ void mega_ring_next(MegaRing& r, int nstage)
{
    if (++r.slot == nstage) { r.slot = 0; r.parity ^= 1u; }
}

// ---- consumer side of one weight operator ---------------------------------------------------------------------------
// Everything that does not change from tile to tile is worked out once per operator; a tile costs a wait, the batches,
// an arrival, the group's barrier and (first warp of the group) the tail.
template <bool INT4, int NP, bool kProf>
__device__ __forceinline__ void mega_consume(const MegaOp* __restrict__ gp, const MegaParams& p, int k, const MegaShared& sh, MegaRing& rp,
                                             uint32_t& tile_no, const MegaWait& w, long long& t_full, long long& t_batch)
{
    constexpr int NR = 4 / NP;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ncta = gridDim.x, cta = blockIdx.x;
    const int G = gp->groups, kw = gp->kw, kind = gp->kind;
    const bool paired = gp->paired != 0;
    const int group = warp / kw, kw_id = warp - group * kw;
    const bool in_group = group < G;
    const int kw32 = kw * 32, tab_n = kw32 * NP, units = gp->units;
    const uint32_t tab = smem_u32(sh.table);
    const int u0 = kw_id * 32 + lane, u1 = u0 + kw32;

    // NP == 1: this lane's slice is stationary in registers for the whole operator
    MegaSlice xs0;
    if (NP == 1) mega_load_slice<INT4>(tab, tab_n, u0, xs0);
    // arrival weight on a slot's empty barrier: the working warps of the operator add up to the barrier's fixed count
    const uint32_t my_arrive = (warp == 0) ? (kMegaBarCount - (uint32_t)(G * kw) + 1u) : 1u;

    const uint32_t wrow = (uint32_t)gp->wrow, zrow = (uint32_t)gp->zrow, srow = (uint32_t)gp->srow;
    const uint32_t run_bytes = (uint32_t)gp->run_bytes;
    // slots past the end of a row hold zero inputs; their addresses are clamped into the row
    const int ua0 = u0 < units ? u0 : units - 1, ua1 = u1 < units ? u1 : units - 1;
    // byte offsets inside a slot of this lane's first weight vector in the group's first row, and from row to row
    const uint32_t gw = (uint32_t)G * wrow, gz = (uint32_t)G * zrow, gs = (uint32_t)G * srow;
    const uint32_t w_lane = (uint32_t)group * wrow + (uint32_t)ua0 * 16u;
    const uint32_t du = (uint32_t)(ua1 - ua0) * 16u;
    // rows 1 .. 3 of a batch relative to its row 0 (paired: gate, up, next gate, next up)
    const uint32_t ro1 = paired ? run_bytes : gw, ro2 = paired ? gw : 2u * gw, ro3 = paired ? gw + run_bytes : 3u * gw;
    const uint32_t adv_w = (paired ? (uint32_t)(NR / 2) : (uint32_t)NR) * gw;
    const uint32_t adv_z = (paired ? (uint32_t)(NR / 2) : (uint32_t)NR) * gz, adv_s = (paired ? (uint32_t)(NR / 2) : (uint32_t)NR) * gs;
    // the zero word and scale this lane applies: item j = lane & 3 of the quad -> row j / NP of the batch, vector j % NP
    const int rj = (lane & 3) / NP;
    const int gj = (((lane & 3) % NP) ? ua1 : ua0) >> 2;   // quantisation group of that vector
    const uint32_t rz = paired ? (uint32_t)(rj & 1) * run_bytes + (uint32_t)(rj >> 1) * gz : (uint32_t)rj * gz;
    const uint32_t rs = paired ? (uint32_t)(rj & 1) * run_bytes + (uint32_t)(rj >> 1) * gs : (uint32_t)rj * gs;
    const uint32_t z_lane = (uint32_t)gp->off_z + (uint32_t)group * zrow + rz + (uint32_t)(gj >> 3) * 4u;
    const uint32_t s_lane = (uint32_t)gp->off_s + (uint32_t)group * srow + rs + (uint32_t)gj * 2u;
    const int zshift = (gj & 7) * 4;
    const bool storer = lane < 4 && (lane % NP) == 0;     // lane r * NP of quad 0 stores row r of a batch
    const int recipG = (65536 + G - 1) / G;                // x / G for the small x that occur below
    float* const red_w = sh.red + warp * kMegaGroupRows + (lane & 3) / NP;
    constexpr int kRedBuf = kMegaConsumerWarps * kMegaGroupRows;
    static_assert((kMegaRedBufs & (kMegaRedBufs - 1)) == 0 && kMegaRedBufs >= kMegaMaxStages + 2, "partial buffers");

    const uint32_t ring = smem_u32(sh.ring);
    const int nseg = mega_segments(*gp);
    const int gran = gp->gran;

    // The tail of a tile (sum over the k-warps, rounding, store) belongs to the service warp, which runs it when every
    // consumer warp has arrived on the slot's empty barrier: a consumer never blocks on a sibling. The partial sums wait
    // in one of kMegaRedBufs buffers (a warp is at most `nstage` tiles ahead of the tail).
    const __half* const xres = (kind == MOP_RESID) ? gp->out[0] : nullptr;
    if (!in_group) {
        // a warp without a group has no part in this operator's tiles (nor in their barriers): it only keeps its ring
        // position in step, then waits at the next operator's CTA barrier
        int tiles = 0;
        for (int seg = 0; seg < nseg; ++seg) tiles += mega_segment(*gp, seg, cta, ncta).nt;
        tile_no += (uint32_t)tiles;
        const int pos = rp.slot + tiles;
        const int wraps = mega_div(pos, p.nstage, __frcp_rn((float)p.nstage));
        rp.slot = pos - wraps * p.nstage;
        rp.parity ^= (uint32_t)wraps & 1u;
        return;
    }
    for (int seg = 0; seg < nseg; ++seg) {
        const MegaSeg sg = mega_segment(*gp, seg, cta, ncta);
        int rb = sg.row0 + group;   // first row of this group in the current tile
        // a segment's tiles come in two sizes: the first `extra` ones hold one granule more than the others
        for (int phase = 0; phase < 2; ++phase) {
            int ntile = phase == 0 ? sg.extra : sg.nt - sg.extra;
            int n = (sg.base + (phase == 0 ? 1 : 0)) * gran;                          // units in a tile of this size
            int cnt = n > group ? ((n - group + G - 1) * recipG) >> 16 : 0;          // units of this group
            int nrows = paired ? 2 * cnt : cnt;                                      // physical rows of this group
            // (kept opaque: under register pressure the compiler would recompute these at every use inside the tile loop)
            asm volatile("" : "+r"(n), "+r"(cnt), "+r"(nrows), "+r"(ntile));
            for (int ti = 0; ti < ntile; ++ti) {
                const long long tw0 = kProf ? clock64() : 0ll;
                mega_wait_bar(&sh.full_bar[rp.slot], rp.parity, w, 2u, k, 32u);
                if (kProf) t_full += clock64() - tw0;
                const int buf = (int)(tile_no & (uint32_t)(kMegaRedBufs - 1));
                const int bufo = buf * kRedBuf;
                // residual values for the tail: fetched here (the consumers hold the operator's dependency), parked beside the partials
                float resid = 0.f;
                const bool res_lane = xres != nullptr && kw_id == 0 && lane < cnt;
                if (res_lane) resid = __half2float(__ldcg(xres + rb + lane * G));
                const uint32_t sbase = ring + (uint32_t)rp.slot * (uint32_t)p.slot_bytes;
                uint32_t bw = sbase + w_lane, bz = sbase + z_lane, bs = sbase + s_lane;
                for (int p0 = 0; p0 < nrows; p0 += NR, bw += adv_w, bz += adv_z, bs += adv_s) {
                    const int left = nrows - p0;
                    uint32_t wa[NR];
                    wa[0] = bw;
                    if (NR > 1) wa[1 % NR] = bw + (left > 1 ? ro1 : 0u);    // rows past the end repeat row 0 (not stored)
                    if (NR > 2) {
                        wa[2 % NR] = bw + (left > 2 ? ro2 : 0u);
                        wa[3 % NR] = bw + (left > 3 ? ro3 : 0u);
                    }
                    const long long tb0 = kProf ? clock64() : 0ll;
                    const float v = mega_batch<INT4, NP>(xs0, tab, tab_n, u0, u1, wa, du, bz, bs, zshift, (left < NR ? left : NR) * NP, lane);
                    if (storer && rj < left) red_w[bufo + p0] = v;
                    if (kProf) t_batch += clock64() - tb0;
                }
                if (res_lane) sh.resid[(buf * kMegaMaxGroups + group) * kMegaGroupRows + lane] = resid;
                // last read of the slot and the partials of this warp are done: one arrival tells the copy and tail warps
                __syncwarp();
                if (lane == 0) mbar_arrive_n(&sh.empty_bar[rp.slot], my_arrive);
                rb += n;
                ++tile_no;
                mega_ring_next(rp, p.nstage);
            }
        }
    }
}

// ---- service warp: the stream of this CTA's tiles over the whole token ------------------------------------------------
// A cursor walks this CTA's tiles in order (operator by operator, segment by segment). Everything that changes only
// with the operator or the segment is kept in registers; a step inside a segment costs a handful of instructions.
struct MegaCursor {
    int k;             // operator (nops: past the end)
    int seg, nseg;     // segment of the operator
    int ti, nt;        // tile of the segment, tiles in the segment
    int n_lo, extra;   // units per tile: n_lo (+ gran for the first `extra` tiles)
    int gran;
    int row, n;        // first unit and units of the current tile
    int left;          // tiles of operator k that follow the current one on this CTA
    bool fresh;        // the cursor has just entered an operator or a segment (per-operator state must be reloaded)
};

__device__ __forceinline__ int mega_my_tiles(const MegaOp& op, int cta, int ncta)
{
    int t = 0;
    const int nseg = mega_segments(op);
    for (int s = 0; s < nseg; ++s) t += mega_segment(op, s, cta, ncta).nt;
    return t;
}

__device__ __forceinline__ void mega_cursor_segment(const MegaOp& op, int cta, int ncta, MegaCursor& c)
{
    // first segment >= c.seg with tiles (the caller knows there is one)
    for (; c.seg < c.nseg; ++c.seg) {
        const MegaSeg sg = mega_segment(op, c.seg, cta, ncta);
        if (sg.nt > 0) {
            c.ti = 0; c.nt = sg.nt; c.n_lo = sg.base * c.gran; c.extra = sg.extra; c.row = sg.row0;
            c.n = c.n_lo + (sg.extra > 0 ? c.gran : 0);
            return;
        }
    }
}

// positions `c` on the first tile of the first operator >= c.k that has tiles on this CTA
__device__ __forceinline__ void mega_cursor_seek(const MegaParams& p, int cta, int ncta, MegaCursor& c)
{
    for (; c.k < p.nops; ++c.k) {
        const MegaOp& op = p.ops[c.k];
        if (!op.has_tiles) continue;
        const int total = mega_my_tiles(op, cta, ncta);
        if (total == 0) continue;
        c.nseg = mega_segments(op);
        c.gran = op.gran;
        c.seg = 0;
        mega_cursor_segment(op, cta, ncta, c);
        c.left = total - 1;
        c.fresh = true;
        return;
    }
}

__device__ __forceinline__ void mega_cursor_next(const MegaParams& p, int cta, int ncta, MegaCursor& c)
{
    if (c.left != 0 && c.ti + 1 < c.nt) {   // the common step: next tile of the same segment
        --c.left;
        ++c.ti;
        c.row += c.n;
        c.n = c.n_lo + (c.ti < c.extra ? c.gran : 0);
        return;
    }
    if (c.left == 0) {
        ++c.k;
        mega_cursor_seek(p, cta, ncta, c);
        return;
    }
    --c.left;
    ++c.seg;
    mega_cursor_segment(p.ops[c.k], cta, ncta, c);
    c.fresh = true;   // the segment changed: matrix and output pointers change with it
}

// this CTA's share of operator k is stored: publish it (the warp barrier orders every lane's stores before the release)
__device__ __forceinline__ void mega_publish(const MegaParams& p, int k, int lane)
{
    const MegaOp& op = p.ops[k];
    __syncwarp();
    if ((op.kind == MOP_PARTIAL || op.kind == MOP_CLS) && op.tp > 1) {
        if (lane < op.tp) red_release_sys_add(op.peer_done[lane], 1u);   // on every rank's counter, after the peer stores
    } else if (lane == 0) {
        red_release_gpu_add(&p.done[k], 1u);
    }
}

// kProf adds cycle counters around the waits (diagnostics); the production instantiation carries none.
template <bool kProf>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const MegaParams p)
{
    auto now = [&]() -> long long { return kProf ? clock64() : 0ll; };
    extern __shared__ __align__(128) unsigned char smem_raw[];   // [ring: nstage * slot_bytes][input table | attention scores, partial outputs]
    __shared__ __align__(8) uint64_t full_bar[kMegaMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMegaMaxStages];
    __shared__ float s_red[kMegaRedBufs * kMegaConsumerWarps * kMegaGroupRows];
    __shared__ float s_part[2][kMegaConsumerWarps];
    __shared__ float s_resid[kMegaRedBufs * kMegaMaxGroups * kMegaGroupRows];
    __shared__ float s_att_tmp[kMegaConsumerWarps];
    __shared__ __align__(16) __half s_q[kHeadMax];
    __shared__ float s_best_v[kMegaConsumerWarps];
    __shared__ int s_best_i[kMegaConsumerWarps];
    __shared__ unsigned int s_abort;
    __shared__ unsigned int s_tailed;   // tiles whose tail has run (tail warp -> copy warp)
    __shared__ unsigned int s_released; // tiles known to be consumed (copy warp -> tail warp)
    // the consumers' view of the current operator and of the next one (fetched one operator ahead, so that no field of an
    // operator is a global-memory access on the hand-off path)
    __shared__ __align__(16) MegaOp s_ops[2];
    constexpr int kOpWords = (int)(sizeof(MegaOp) / sizeof(uint32_t));
    static_assert(sizeof(MegaOp) % sizeof(uint32_t) == 0 && kOpWords <= kMegaConsThreads, "operator descriptor");

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const unsigned int expected = p.seq_no * (unsigned int)ncta;

    if (tid == 0) {
        for (int s = 0; s < p.nstage; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kMegaBarCount);
        }
        s_abort = 0;
        s_tailed = 0;
        s_released = 0;
        mbar_fence_init();
    }
    if (tid < kOpWords) reinterpret_cast<uint32_t*>(&s_ops[0])[tid] = reinterpret_cast<const uint32_t*>(p.ops)[tid];
    __syncthreads();

    MegaWait w;
    w.abort_flag = &s_abort;
    w.status = p.status;
    w.budget = p.wait_cycles;

    if (warp == kMegaConsumerWarps) {
        // ================= copy warp ==========================================================================
        // Tile t of this CTA (counted over the whole token) lives in ring slot t % nstage. When all consumer warps have
        // arrived on a slot's empty barrier, the slot is refilled with the tile that is `nstage` further on. Weights
        // do not depend on activations, so the copies run ahead of the arithmetic across operator boundaries.
        const uint64_t pol = policy_evict_first();
        MegaRing ri{0, 0u};
        MegaCursor ci;
        ci.k = 0;
        mega_cursor_seek(p, cta, ncta, ci);
        uint32_t issued = 0;
        long long tp_wait = 0, tp_all0 = now();
        // this lane's copy: part (lane % 3) of run (lane / 3): weights, zero words, scales
        const int my_run = lane / 3, my_part = lane - my_run * 3;
        bool i_issuer = false;
        uint32_t i_rowbytes = 0, i_off = 0, i_allbytes = 0;
        const unsigned char* i_src = nullptr;
        while (ci.k < p.nops) {
            if (issued >= (uint32_t)p.nstage) {
                const long long tw0 = now();
                if (lane == 0) {
                    mega_wait_bar(&empty_bar[ri.slot], ri.parity ^ 1u, w, 1u, ci.k, 256u);
                    // tile (issued - nstage) is consumed. The tail warp learns that from the barrier's phase parity, which
                    // repeats after two refills: this counter settles it if the tail warp ever falls that far behind
                    *(volatile unsigned int*)&s_released = issued - (uint32_t)p.nstage + 1u;
                    // the tail warp reads the partial sums of a tile from one of kMegaRedBufs buffers and tells tiles
                    // apart by the barrier's phase parity: it must not fall further behind than that allows
                    const long long t0 = clock64();
                    while ((int)(issued - *(volatile unsigned int*)&s_tailed) > kMegaRedBufs - 1 && !s_abort) {
                        if (clock64() - t0 > w.budget) { mega_give_up(w, 7u, ci.k); break; }
                    }
                }
                __syncwarp();
                tp_wait += now() - tw0;
            }
            if (ci.fresh) {
                const MegaOp* __restrict__ gp = p.ops + ci.k;
                const int nruns = gp->paired ? 2 : 1;
                const uint32_t wrow = (uint32_t)gp->wrow, zrow = (uint32_t)gp->zrow, srow = (uint32_t)gp->srow;
                i_issuer = lane < 3 * nruns && (gp->fmt == 0 || my_part == 0);
                i_allbytes = (uint32_t)nruns * (wrow + zrow + srow);
                i_rowbytes = my_part == 0 ? wrow : (my_part == 1 ? zrow : srow);
                i_off = (uint32_t)my_run * (uint32_t)gp->run_bytes + (my_part == 0 ? 0u : (my_part == 1 ? (uint32_t)gp->off_z : (uint32_t)gp->off_s));
                if (i_issuer) {
                    const QWPtrs q = gp->mat[gp->paired ? my_run : ci.seg];
                    i_src = my_part == 0 ? reinterpret_cast<const unsigned char*>(q.w)
                                         : (my_part == 1 ? reinterpret_cast<const unsigned char*>(q.z) : reinterpret_cast<const unsigned char*>(q.s));
                    i_src += (size_t)ci.row * i_rowbytes;
                }
                ci.fresh = false;
            }
            const uint32_t n = (uint32_t)ci.n;
#ifdef ML2_DIAG_NOCOPY
            if (lane == 0) mbar_arrive(&full_bar[ri.slot]);   // pipeline probe: no weight copies
            i_issuer = false;
#else
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[ri.slot], n * i_allbytes);
#endif
            __syncwarp();
            if (i_issuer) {
                bulk_g2s(smem_raw + (size_t)ri.slot * p.slot_bytes + i_off, i_src, n * i_rowbytes, &full_bar[ri.slot], pol);
                i_src += (size_t)n * i_rowbytes;
            }
            mega_cursor_next(p, cta, ncta, ci);
            mega_ring_next(ri, p.nstage);
            ++issued;
        }
        if (kProf && p.prof && lane == 0) {
            long long* o = p.prof + (size_t)cta * 64;
            o[32] = now() - tp_all0;
            o[33] = tp_wait;
        }
        return;
    }

    if (warp == kMegaConsumerWarps + 1) {
        // ================= tail warp ===========================================================================
        // When all consumer warps have arrived on a slot's empty barrier, the tile that was in it gets its tail: the
        // fixed-order sum over the k-warps of every row's group, the operator's rounding and store. After the tail of
        // the operator's last tile on this CTA the operator is published (release) on its device-wide counter.
        MegaRing rf{0, 0u};
        MegaCursor cf;
        cf.k = 0;
        mega_cursor_seek(p, cta, ncta, cf);
        uint32_t tailed = 0;
        long long tf_wait = 0, tf_all0 = now();
        int f_kind = 0, f_G = 1, f_kw = 1, f_recipG = 65536;
        bool f_paired = false;
        __half* f_out = nullptr;
        const MegaOp* f_gp = p.ops;
        while (cf.k < p.nops) {
            if (cf.fresh) {
                f_gp = p.ops + cf.k;
                f_kind = f_gp->kind; f_G = f_gp->groups; f_kw = f_gp->kw; f_paired = f_gp->paired != 0;
                f_recipG = (65536 + f_G - 1) / f_G;
                f_out = f_gp->out[f_kind == MOP_QKV ? cf.seg : 0];
                if (f_kind == MOP_QKV && cf.seg > 0) f_out += (long long)p.pos * p.kv_row_stride;
                cf.fresh = false;
            }
            const long long tw0 = now();
            if (lane == 0 && !mbar_try_wait(&empty_bar[rf.slot], rf.parity)) {
                const long long t0 = clock64();
                for (uint32_t i = 0; i < (1u << 30); ++i) {
                    if (mbar_try_wait_suspend(&empty_bar[rf.slot], rf.parity, 1000u)) break;
                    __nanosleep(128u);
                    if ((int)(*(volatile unsigned int*)&s_released - tailed) > 0 || s_abort) break;
                    if (clock64() - t0 > w.budget) { mega_give_up(w, 3u, cf.k); break; }
                }
            }
            __syncwarp();
            tf_wait += now() - tw0;
            const int buf = (int)(tailed & (uint32_t)(kMegaRedBufs - 1));
            const float* red = s_red + buf * (kMegaConsumerWarps * kMegaGroupRows);
            for (int j = lane; j < cf.n; j += 32) {
                const int i = (j * f_recipG) >> 16, g = j - i * f_G;   // unit j is unit i of group g
                const float* rg = red + g * f_kw * kMegaGroupRows + (f_paired ? 2 * i : i);
                float sa = 0.f, sb = 0.f;
                for (int q = 0; q < f_kw; ++q) {
                    sa += rg[q * kMegaGroupRows];
                    if (f_paired) sb += rg[q * kMegaGroupRows + 1];
                }
                const float resid = (f_kind == MOP_RESID) ? s_resid[(buf * kMegaMaxGroups + g) * kMegaGroupRows + i] : 0.f;
                mega_epilogue(f_gp, f_kind, f_out, cf.row + j, sa, sb, resid);
            }
            if (cf.left == 0) mega_publish(p, cf.k, lane);
            ++tailed;
            __syncwarp();
            if (lane == 0) *(volatile unsigned int*)&s_tailed = tailed;   // the partial buffer is free again
            mega_cursor_next(p, cta, ncta, cf);
            mega_ring_next(rf, p.nstage);
        }
        if (kProf && p.prof && lane == 0) {
            long long* o = p.prof + (size_t)cta * 64;
            o[34] = now() - tf_all0;
            o[35] = tf_wait;
        }
        return;
    }

    // ================= consumers =========================================================================
    MegaShared sh;
    sh.ring = smem_raw;
    sh.table = smem_raw + (size_t)p.nstage * p.slot_bytes;
    sh.full_bar = full_bar;
    sh.empty_bar = empty_bar;
    sh.red = s_red;
    sh.part = &s_part[0][0];
    sh.resid = s_resid;
    MegaRing rp{0, 0u};
    uint32_t tile_no = 0;
    long long t_dep = 0, t_full = 0, t_attn = 0, t_pro = 0, t_batch = 0, t_all0 = now();
    long long tk_dep[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tk_pro[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tk_run[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < p.nops; ++k) {
        const MegaOp* gp = &s_ops[k & 1];
        const MegaOp& op = *gp;
        const int kk = (op.kind == MOP_RESID && op.rows > p.dim) ? 7 : op.kind;

        // RMSNorm weights do not depend on the previous operator: fetch them before the wait
        uint4 gam[kMegaNormVecs];
#pragma unroll
        for (int q = 0; q < kMegaNormVecs; ++q) gam[q] = make_uint4(0, 0, 0, 0);
        const int nvec8 = op.rows >> 3;   // 16-byte pieces of the input vector
        if (op.has_tiles && op.pro != 0) {
#pragma unroll
            for (int q = 0; q < kMegaNormVecs; ++q)
                if (tid + q * kMegaConsThreads < nvec8) gam[q] = *reinterpret_cast<const uint4*>(op.gamma + (size_t)(tid + q * kMegaConsThreads) * 8);
        }

        // ---- dependency: the previous operator's output is complete everywhere (acquire by one thread, CTA barrier).
        // The barrier also keeps this operator's table from overwriting what slow warps of the last one still read.
        {
            const long long td0 = now();
            if (k > 0 && tid == 0) {
                const MegaOp& prev = s_ops[(k - 1) & 1];
                const bool sys = (prev.kind == MOP_PARTIAL || prev.kind == MOP_CLS) && prev.tp > 1;
                mega_wait_counter(&p.done[k - 1], expected * mega_arrivals(prev), w, 5u, k, sys);
            }
            named_bar_sync(1, kMegaConsThreads);
            const long long dt = now() - td0;
            t_dep += dt;
            tk_dep[kk] += dt;
        }
        const long long tq0 = now();
        // next operator's descriptor: loaded now, parked in the other buffer (nobody reads it any more) a little later
        uint32_t next_word = 0;
        const bool fetch_next = tid < kOpWords && k + 1 < p.nops;
        if (fetch_next) next_word = __ldg(reinterpret_cast<const uint32_t*>(p.ops + k + 1) + tid);

        if (op.kind == MOP_ATTN) {
            // ---- attention (reference: rope / mat_vec_strided / softmax / vec_mat kernels): `att_split` CTAs per head,
            // each over a contiguous part of the sequence (1 for short contexts, more when the cache rows are many) ----
            // Every part computes its scores (rounded to fp16 like native/mat_vec_kernel.cu:72-73), their maximum m_p and
            // exp-sum l_p; the parts of a head exchange (m_p, l_p) through global memory; the probabilities are rounded
            // to fp16 after the division by the GLOBAL sum (native/softmax_kernel.cu:46); the fp32 partial outputs are
            // summed by the operator that consumes them (single fp16 rounding, native/vec_mat_kernel.cu:41).
            const int S = p.att_split > 1 ? p.att_split : 1;
            if (cta < p.heads_local * S) {
                float* s_sc = reinterpret_cast<float*>(sh.table);
                float (*s_att_acc)[kHeadMax] = reinterpret_cast<float (*)[kHeadMax]>(sh.table + (size_t)p.att_cap * sizeof(float));
                const int head = cta / S, part = cta - head * S;
                const int nseq = p.pos + 1;
                const int chunk = (nseq + S - 1) / S;
                const int t0 = part * chunk;
                const int t1 = min(nseq, t0 + chunk);
                const size_t stride = (size_t)p.kv_row_stride;
                const int hs = p.head_size, half = hs >> 1;
                // rotation of q and of the key row written by this token (native/rope_kernel.cu:15-25: fp32 on the fp16
                // values the mat-vec stored, rounded to fp16): q stays in shared memory, the key row goes back to the cache
                if (tid < half) {
                    const float2 cs = p.rope_table[(size_t)p.pos * half + tid];
                    const __half* qh = op.in + (size_t)head * hs;
                    const float a = __half2float(__ldcg(qh + tid)), b = __half2float(__ldcg(qh + tid + half));
                    s_q[tid] = __float2half_rn(a * cs.x - b * cs.y);
                    s_q[tid + half] = __float2half_rn(a * cs.y + b * cs.x);
                } else if (tid < hs && t1 == nseq && t1 > t0) {
                    const int d = tid - half;
                    const float2 cs = p.rope_table[(size_t)p.pos * half + d];
                    __half* kr = op.kcache + (size_t)p.pos * stride + (size_t)head * hs;
                    const float a = __half2float(__ldcg(kr + d)), b = __half2float(__ldcg(kr + d + half));
                    kr[d] = __float2half_rn(a * cs.x - b * cs.y);
                    kr[d + half] = __float2half_rn(a * cs.y + b * cs.x);
                }
                __threadfence_block();
                named_bar_sync(1, kMegaConsThreads);
                const __half* kh = op.kcache + (size_t)head * hs + lane * 4;
                const __half* vh = op.vcache + (size_t)head * hs + lane * 4;
                const uint2 qv = *reinterpret_cast<const uint2*>(s_q + lane * 4);
                // short parts (one sweep of the warps covers them): the value rows do not depend on the scores, fetch them
                // together with the key rows instead of one memory round trip later
                const bool one_sweep = t1 - t0 <= kMegaConsumerWarps * kAttUnroll;
                uint2 vv0[kAttUnroll];
                if (one_sweep) {
                    const int b = t0 + warp * kAttUnroll;
#pragma unroll
                    for (int u = 0; u < kAttUnroll; ++u) vv0[u] = (b < t1) ? ld_cg_v2(vh + (size_t)min(b + u, t1 - 1) * stride) : make_uint2(0u, 0u);
                }
                float mx = -INFINITY;
                for (int b = t0 + warp * kAttUnroll; b < t1; b += kMegaConsumerWarps * kAttUnroll) {
                    uint2 kv[kAttUnroll];
#pragma unroll
                    for (int u = 0; u < kAttUnroll; ++u)
                        kv[u] = ld_cg_v2(kh + (size_t)min(b + u, t1 - 1) * stride);   // unconditional: all loads in flight together
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
                named_bar_sync(1, kMegaConsThreads);
                mx = s_att_tmp[0];
#pragma unroll
                for (int q = 1; q < kMegaConsumerWarps; ++q) mx = fmaxf(mx, s_att_tmp[q]);
                named_bar_sync(1, kMegaConsThreads);
                float sum = 0.f;
                for (int i = tid; i < t1 - t0; i += kMegaConsThreads) {
                    const float e = expf(s_sc[i] - mx);
                    s_sc[i] = e;
                    sum += e;
                }
                sum = warp_sum(sum);
                if (lane == 0) s_att_tmp[warp] = sum;
                named_bar_sync(1, kMegaConsThreads);
                float lsum = 0.f;
#pragma unroll
                for (int q = 0; q < kMegaConsumerWarps; ++q) lsum += s_att_tmp[q];
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
                        mega_wait_counter(&op.att_cnt[head], want, w, 6u, k, false);
                    }
                    named_bar_sync(1, kMegaConsThreads);
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
                    for (int u = 0; u < kAttUnroll; ++u) vv[u] = one_sweep ? vv0[u] : ld_cg_v2(vh + (size_t)min(b + u, t1 - 1) * stride);
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
                named_bar_sync(1, kMegaConsThreads);
                if (tid < hs) {
                    float o = 0.f;
#pragma unroll
                    for (int q = 0; q < kMegaConsumerWarps; ++q) o += s_att_acc[q][tid];
                    if (S > 1) op.att_part[((size_t)head * S + part) * hs + tid] = o;
                    else op.out[0][(size_t)head * hs + tid] = __float2half_rn(o);   // native/vec_mat_kernel.cu:41
                }
            }
            if (fetch_next) reinterpret_cast<uint32_t*>(&s_ops[(k + 1) & 1])[tid] = next_word;
            named_bar_sync(1, kMegaConsThreads);
            if (tid == 0) red_release_gpu_add(&p.done[k], 1u);
            t_attn += now() - tq0;
            continue;
        }

        if (op.kind == MOP_ARGMAX) {
            // ---- greedy sample on CTA 0 (native/argmax_kernel.cu:8-46, lowest index on ties) --------------------
            if (cta == 0) {
                float best = -INFINITY;
                int best_i = 0x7fffffff;
                for (int i = tid; i < p.vocab; i += kMegaConsThreads) {
                    const float v = __half2float(__ldcg(p.logits + i));
                    if (v > best) { best = v; best_i = i; }
                }
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
                }
                if (lane == 0) { s_best_v[warp] = best; s_best_i[warp] = best_i; }
                named_bar_sync(1, kMegaConsThreads);
                if (tid == 0) {
                    for (int q = 1; q < kMegaConsumerWarps; ++q)
                        if (s_best_v[q] > best || (s_best_v[q] == best && s_best_i[q] < best_i)) { best = s_best_v[q]; best_i = s_best_i[q]; }
                    if (p.write_token) p.tokens[p.next_pos] = (best_i == 0x7fffffff) ? 0 : best_i;
                }
            }
            if (fetch_next) reinterpret_cast<uint32_t*>(&s_ops[(k + 1) & 1])[tid] = next_word;
            if (tid == 0) red_release_gpu_add(&p.done[k], 1u);
            continue;
        }

        // ---- weight operators: prepared input table, once per CTA ----------------------------------------------------
        const int my_tiles = mega_my_tiles(op, cta, ncta);
        const bool is_int4 = op.fmt == 0;
        const int tab_n = op.kw * 32 * op.np;
        uint4* tab = reinterpret_cast<uint4*>(sh.table);
        const int nthr = is_int4 ? tab_n * 4 : tab_n;   // table builders: one per 8 inputs, whole warps
        if (op.pro == 0) {
            const bool split_in = op.att_part != nullptr && p.att_split > 1;
            for (int i = tid; i < nthr; i += kMegaConsThreads) {
                uint4 t = make_uint4(0, 0, 0, 0);
                if (i < nvec8) {
                    if (split_in) {
                        // input = attention output of the split path: fp32 partials of the parts, summed in part order and
                        // rounded to fp16 once (native/vec_mat_kernel.cu:41)
                        const int S = p.att_split;
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
                        t = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                    } else {
                        t = ld_cg_v4(op.in + (size_t)i * 8);
                    }
                }
                if (is_int4) mega_table_store_int4(tab, tab_n, i, t);
                else tab[i] = t;
            }
        } else {
            const __half* src = op.in;
            if (op.pro == 2) {
                int token = p.tokens[p.pos];                           // native/embedding_kernel.cu:6-12
                token = token < 0 ? 0 : (token >= p.vocab ? p.vocab - 1 : token);
                src = p.embed + (size_t)token * op.rows;
            }
            uint4 xv[kMegaNormVecs];
            float ss = 0.f;
#pragma unroll
            for (int q = 0; q < kMegaNormVecs; ++q) {
                xv[q] = make_uint4(0, 0, 0, 0);
                const int i = tid + q * kMegaConsThreads;
                if (i < nvec8) {
                    xv[q] = ld_cg_v4(src + (size_t)i * 8);
                    if (op.pro == 2 && cta == 0) *reinterpret_cast<uint4*>(p.x + (size_t)i * 8) = xv[q];  // residual stream := embedding row
                    if (op.pro == 3) {
                        // residual add of a row-sharded mat-vec: x := half(float(x) + sum over ranks of their fp32
                        // partials), ranks in fixed order so that every rank rounds the same value
                        // (rounding point of native/mat_vec_kernel.cu:154-156)
                        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        for (int r = 0; r < op.tp; ++r) {
                            const float4* pr = reinterpret_cast<const float4*>(op.recv + (size_t)r * op.rows + (size_t)i * 8);
                            const float4 p0 = __ldcg(pr), p1 = __ldcg(pr + 1);
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
            float* part = sh.part + (k & 1) * kMegaConsumerWarps;
            if (lane == 0) part[warp] = ss;
            named_bar_sync(1, kMegaConsThreads);
            float tot = 0.f;
#pragma unroll
            for (int q = 0; q < kMegaConsumerWarps; ++q) tot += part[q];
            const float rms = 1.0f / sqrtf(tot / (float)op.rows + p.eps);   // native/rmsnorm_kernel.cu:26-27
#pragma unroll
            for (int q = 0; q < kMegaNormVecs; ++q) {
                const int i = tid + q * kMegaConsThreads;
                if (i < nthr) {
                    uint4 t = make_uint4(0, 0, 0, 0);
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
                        t = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                    }
                    if (is_int4) mega_table_store_int4(tab, tab_n, i, t);
                    else tab[i] = t;
                }
            }
        }
        if (fetch_next) reinterpret_cast<uint32_t*>(&s_ops[(k + 1) & 1])[tid] = next_word;
        named_bar_sync(1, kMegaConsThreads);
        t_pro += now() - tq0;
        tk_pro[kk] += now() - tq0;

        const long long trun0 = now();
        if (is_int4) {
            if (op.np == 1) mega_consume<true, 1, kProf>(gp, p, k, sh, rp, tile_no, w, t_full, t_batch);
            else mega_consume<true, 2, kProf>(gp, p, k, sh, rp, tile_no, w, t_full, t_batch);
        } else {
            if (op.np == 1) mega_consume<false, 1, kProf>(gp, p, k, sh, rp, tile_no, w, t_full, t_batch);
            else mega_consume<false, 2, kProf>(gp, p, k, sh, rp, tile_no, w, t_full, t_batch);
        }
        tk_run[kk] += now() - trun0;

        // ---- hand-off: the service warp publishes the operator after the tail of this CTA's last tile; a CTA that
        // owns no tile of it publishes here (its consumers have read whatever the prologue reads)
        if (my_tiles == 0) {
            if ((op.kind == MOP_PARTIAL || op.kind == MOP_CLS) && op.tp > 1) {
                if (tid < op.tp) red_release_sys_add(op.peer_done[tid], 1u);
            } else if (tid == 0) {
                red_release_gpu_add(&p.done[k], 1u);
            }
        }
    }
    if (s_abort) {
        // some wait ran out: bulk copies of this CTA may still be in flight; give them time to land before the CTA's
        // shared memory is handed to someone else
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) { }
    }
    if (kProf && p.prof && tid == 0) {
        long long* o = p.prof + (size_t)cta * 64;
        o[0] = now() - t_all0; o[1] = t_dep; o[2] = t_full; o[3] = t_batch; o[4] = t_attn; o[5] = t_pro;
        for (int q = 0; q < 8; ++q) { o[8 + q] = tk_dep[q]; o[16 + q] = tk_pro[q]; o[24 + q] = tk_run[q]; }
    }
}

}  // namespace ml2
