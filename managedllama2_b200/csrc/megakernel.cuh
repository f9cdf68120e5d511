// One persistent kernel per token: the whole operator sequence of Transformer.Forward
// (src/Transformer.cs:158-190 of GilesBathgate/ManagedLlama2) runs inside a single cooperative launch with
// one CTA per SM, so HBM streaming never stops at an operator boundary.
//
//   * rows            every operator's output rows are cut into contiguous, balanced ranges, one per CTA; a CTA
//                     streams its range as tiles of up to `rmax` rows (packed weights, zero words, scales). The host
//                     works this out once per model and leaves every CTA a flat list of tile descriptors (sources,
//                     sizes and shared-memory offsets of the tile's copies; first row, rows, operator, output).
//   * copy warp       walks the CTA's tile list and streams every tile, operator after operator, into one shared-memory
//                     ring (1-D bulk async copies, mbarrier completion). Weights do not depend on activations, so it
//                     runs ahead of the arithmetic by the depth of the ring, across operator boundaries.
//   * consumer warps  int4 operators: every warp takes one or two quantisation groups (128 inputs) of ALL rows of a
//                     tile on the tensor cores (warp-wide m16n8k16 steps on nibbles unpacked in registers, its inputs
//                     stationary in registers as B fragments) and leaves one partial sum per row in shared memory.
//                     fp16 operator (classifier): groups of `kw` warps span a row, group g takes rows g, g + G, ...
//   * tail warp       when all consumer warps have arrived on a slot's barrier, adds the warps' partial sums of the
//                     tile in a fixed order and runs the operator's tail (residual add, SwiGLU, stores) with the
//                     reference's fp16 rounding points; after the CTA's last tile of an operator it publishes the
//                     operator (release) on its device-wide counter.
//   * hand-off        the next operator starts when the counter is complete (acquire by one thread, CTA barrier),
//                     builds its prepared input table cooperatively (RMSNorm applied where the reference runs rmsnorm
//                     first) and goes on with tiles that the copy warp has already brought in.
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
    int kw, groups, np;      // fp16 weights: warps per group, groups per CTA, weight vectors per lane and row (1 or 2)
                             // int4 weights: working warps, 1, quantisation groups per warp
    int ngrp, tab_n, two;    // int4: quantisation groups per row; lane slots of the input table; a tile has a second block of 8 rows
    int gran;                // rows per alignment granule: every tile is a whole number of granules
    int rmax;                // units (rows, or row pairs) of a full tile
    int off_z, off_s, run_bytes;   // shared-memory layout of one run (the rows of one matrix in a tile)
    int has_tiles;           // weight operator
    int rot;                 // rotation of the CTA -> row range assignment (host)
    int ngran, gmax;         // granules of a segment (cols / gran), granules of a full tile (rmax / gran) (host)
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

// One tile of one CTA: everything the copy warp and the tail warp need, worked out by the host (128 bytes).
struct MegaTileCopy {
    const void* src;          // 16-byte aligned
    uint32_t bytes;           // multiple of 16; 0: unused entry
    uint32_t dst;             // byte offset inside the ring slot
};
struct MegaTile {
    MegaTileCopy cp[6];       // weights, zero words, scales of the tile's one or two runs
    int row, n;               // first unit (row, or gate / up row pair) and units
    uint32_t info;            // bits 0..15 operator index, 16..17 segment, 18: the CTA's last tile of the operator,
                              // 19: the output row is the cache row of the token's position (k and v)
    uint32_t total_bytes;     // sum over cp
    __half* out;              // output vector of the tile's segment
    uint32_t opbits;          // bits 0..2 operator kind, 3 paired, 4 int4 (tensor-core partial layout), 5 the operator's counter
                              // lives on every rank, 8..15 kw, 16..23 groups
    uint32_t pad;
};
static_assert(sizeof(MegaTile) == 128, "tile descriptor");
constexpr uint32_t kTileLast = 1u << 18, kTileCacheRow = 1u << 19;

struct MegaParams {
    const MegaOp* ops;
    int nops;
    const MegaTile* tiles;     // every CTA's tiles in the order it streams them
    const int* tile_begin;     // [gridDim.x + 1] offsets into `tiles`
    const unsigned short* op_tiles;   // [nops][gridDim.x] tiles of each operator on each CTA
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

constexpr int kMegaConsumerWarps = 21;   // 20 warps x 2 quantisation groups span a 5120-input row, 18 x 6 a 13824-input row
constexpr int kMegaServiceWarps = 2;     // copy warp and tail warp: warps 0 and 1 of the CTA (first or last made no measurable difference)
constexpr int kMegaServiceThreads = kMegaServiceWarps * 32;
constexpr int kMegaWarps = kMegaConsumerWarps + kMegaServiceWarps;
constexpr int kMegaThreads = kMegaWarps * 32;
constexpr int kMegaConsThreads = kMegaConsumerWarps * 32;
constexpr int kMegaMaxStages = 6;
constexpr int kMegaMaxGroups = 8;     // groups of warps that may share a tile (fp16 weights)
constexpr int kMegaGroupRows = 8;     // physical rows of one tile that one group may own (fp16 weights)
constexpr int kMegaRedRows = 16;      // partial sums one warp may leave per tile
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

// ---- shared-memory objects --------------------------------------------------------------------------------------------
struct MegaShared {
    unsigned char* ring;      // nstage * slot_bytes, then the table / scratch area
    unsigned char* table;
    uint64_t* full_bar;
    uint64_t* empty_bar;
    float* red;               // [kMegaRedBufs][kMegaConsumerWarps][kMegaRedRows] partial sums of the tiles in flight
    float* part;              // [2][kMegaConsumerWarps] sum-of-squares partials
    float* resid;             // [kMegaRedBufs][kMegaRedRows] residual values of the tiles in flight (int4 operators)
    const int* tile_row;      // [nstage] first unit of the tile in each slot ...
    const int* tile_n;        // ... and its units (written by the copy warp before the slot's copies)
};

// ---- prepared input table ---------------------------------------------------------------------------------------------
// int4 operators: lane slot u (32 consecutive inputs = one 16-byte weight vector of every row, one quarter of a
// quantisation group) owns four 16-byte vectors, stored as table[q * tab_n + u]:
//   q = 0..3   the inputs of packed word q as fp16 pairs (x0,x4) (x1,x5) (x2,x6) (x3,x7): the B fragments of the two
//              tensor-core steps that consume the word (see mega_mma_word)
// and every quantisation group G one more, table[4 * tab_n + G]:
//   .x  -(1024 * S(inputs under even nibbles) + 64 * S(inputs under odd nibbles)): start value of the accumulator, it
//       removes the exponent offsets of the unpacked nibbles;   .y  S(all inputs of the group): zero-point term
// fp16 operators: table[u] = the 8 inputs of slot u.
// Slots past the end of the row hold zeros.
__device__ __forceinline__ void mega_table_store_int4(uint4* tab, int tab_n, int i, uint4 t)
{
    // thread i holds inputs [8i, 8i + 8): word (i & 3) of slot (i >> 2); the 16 threads of a group are adjacent lanes
    const uint32_t x0 = __byte_perm(t.x, t.z, 0x5410), x1 = __byte_perm(t.x, t.z, 0x7632);
    const uint32_t x2 = __byte_perm(t.y, t.w, 0x5410), x3 = __byte_perm(t.y, t.w, 0x7632);
    float ev = half_bits_to_float(lo16(t.x)) + half_bits_to_float(lo16(t.y)) + half_bits_to_float(lo16(t.z)) + half_bits_to_float(lo16(t.w));
    float od = half_bits_to_float(hi16(t.x)) + half_bits_to_float(hi16(t.y)) + half_bits_to_float(hi16(t.z)) + half_bits_to_float(hi16(t.w));
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        ev += __shfl_xor_sync(0xffffffffu, ev, o);
        od += __shfl_xor_sync(0xffffffffu, od, o);
    }
    const int u = i >> 2, q = i & 3;
    tab[q * tab_n + u] = make_uint4(x0, x1, x2, x3);
    if ((i & 15) == 0) tab[4 * tab_n + (i >> 4)] = make_uint4(__float_as_uint(-(1024.f * ev + 64.f * od)), __float_as_uint(ev + od), 0u, 0u);
}

// ---- fp16 operator (the classifier): arithmetic of one batch -------------------------------------------------------
// one 16-byte weight vector (8 fp16 weights) against the 8 matching inputs
__device__ __forceinline__ float mega_item_f16(const uint4& wv, const uint4& x)
{
#ifdef ML2_DIAG_NOMATH
    return __uint_as_float(wv.x ^ x.x);   // pipeline probe: loads stay, arithmetic goes
#endif
    float a = 0.f, b = 0.f;
    a = fma_f16_f32(lo16(wv.x), lo16(x.x), a);
    b = fma_f16_f32(hi16(wv.x), hi16(x.x), b);
    a = fma_f16_f32(lo16(wv.y), lo16(x.y), a);
    b = fma_f16_f32(hi16(wv.y), hi16(x.y), b);
    a = fma_f16_f32(lo16(wv.z), lo16(x.z), a);
    b = fma_f16_f32(hi16(wv.z), hi16(x.z), b);
    a = fma_f16_f32(lo16(wv.w), lo16(x.w), a);
    b = fma_f16_f32(hi16(wv.w), hi16(x.w), b);
    return a + b;
}

// A batch is four (row, vector) items of this lane: item i = row (i / NP) of the batch, weight vector (i % NP) of the
// lane. Returns the warp's row totals: row r on the lanes with ((lane & 3) / NP) == r.
//   wa[r]   shared-memory address of this lane's first weight vector in row r of the batch
//   du      byte distance to the lane's second vector (NP == 2)
template <int NP>
__device__ __forceinline__ float mega_batch_f16(const uint4 (&xs)[NP], const uint32_t (&wa)[4 / NP], uint32_t du, int nitems, int lane)
{
    uint4 wv[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) wv[i] = lds_v4(wa[i / NP] + ((i % NP) ? du : 0u));
    float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (i < nitems) t[i] = mega_item_f16(wv[i], xs[i % NP]);   // warp-uniform: a short last batch costs only the rows it has
    // 4 x 4 transposing reduction inside the quad: lane j of the quad ends with the quad's sum of item j
    const bool b2 = (lane & 2) != 0, b1 = (lane & 1) != 0;
    const float s0 = b2 ? t[0] : t[2], k0 = b2 ? t[2] : t[0];
    const float s1 = b2 ? t[1] : t[3], k1 = b2 ? t[3] : t[1];
    const float q0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 2);
    const float q1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 2);
    const float sn = b1 ? q0 : q1, kp = b1 ? q1 : q0;
    float v = kp + __shfl_xor_sync(0xffffffffu, sn, 1);
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

// a consumer warp that has no part in an operator's tiles (nor in their barriers) only keeps its ring position in step
__device__ __forceinline__ void mega_skip_tiles(MegaRing& rp, uint32_t& tile_no, int tiles, int nstage)
{
    tile_no += (uint32_t)tiles;
    const int pos = rp.slot + tiles;
    const int wraps = pos / nstage;
    rp.slot = pos - wraps * nstage;
    rp.parity ^= (uint32_t)wraps & 1u;
}

// ---- consumer side of the fp16 operator ------------------------------------------------------------------------------
// Groups of `kw` warps span a weight row (a lane owns one or two 16-byte vectors of every row, its inputs stationary in
// registers); all groups share a tile: group g takes rows g, g + G, ... of it. Everything that does not change from tile
// to tile is worked out once per operator; a tile costs a wait, the batches and an arrival. The partial sums of a tile
// wait for the tail warp in one of kMegaRedBufs buffers (a warp is at most `nstage` tiles ahead of the tail).
template <int NP, bool kProf>
__device__ __forceinline__ void mega_consume_f16(const MegaOp* __restrict__ gp, const MegaParams& p, int k, const MegaShared& sh, MegaRing& rp,
                                                 uint32_t& tile_no, const MegaWait& w, int my_tiles, long long& t_full, long long& t_batch)
{
    constexpr int NR = 4 / NP;
    const int tid = (int)threadIdx.x - kMegaServiceThreads, lane = tid & 31, warp = tid >> 5;
    const int G = gp->groups, kw = gp->kw;
    const int group = warp / kw, kw_id = warp - group * kw;
    if (group >= G) {
        mega_skip_tiles(rp, tile_no, my_tiles, p.nstage);
        return;
    }
    const int kw32 = kw * 32, units = gp->units, rmax = gp->rmax;
    const uint32_t tab = smem_u32(sh.table);
    const int u0 = kw_id * 32 + lane, u1 = u0 + kw32;
    uint4 xs[NP];   // this lane's inputs: slots past the end of the row hold zeros in the table
    xs[0] = lds_v4(tab + (uint32_t)u0 * 16u);
    if (NP == 2) xs[NP - 1] = lds_v4(tab + (uint32_t)u1 * 16u);
    // arrival weight on a slot's empty barrier: the working warps of the operator add up to the barrier's fixed count
    const uint32_t my_arrive = (warp == 0) ? (kMegaBarCount - (uint32_t)(G * kw) + 1u) : 1u;
    const uint32_t wrow = (uint32_t)gp->wrow;
    // slots past the end of a row: their addresses are clamped into the row
    const int ua0 = u0 < units ? u0 : units - 1, ua1 = u1 < units ? u1 : units - 1;
    // byte offsets inside a slot of this lane's first weight vector in the group's first row, and from row to row
    const uint32_t gw = (uint32_t)G * wrow;
    const uint32_t w_lane = (uint32_t)group * wrow + (uint32_t)ua0 * 16u;
    const uint32_t du = (uint32_t)(ua1 - ua0) * 16u;
    const int rj = (lane & 3) / NP;
    const bool storer = lane < 4 && (lane % NP) == 0;     // lane r * NP of quad 0 stores row r of a batch
    const int recipG = (65536 + G - 1) / G;                // x / G for the small x that occur below
    float* const red_w = sh.red + warp * kMegaRedRows + rj;
    constexpr int kRedBuf = kMegaConsumerWarps * kMegaRedRows;
    static_assert((kMegaRedBufs & (kMegaRedBufs - 1)) == 0 && kMegaRedBufs >= kMegaMaxStages + 2, "partial buffers");
    const uint32_t ring = smem_u32(sh.ring);

    for (int ti = 0; ti < my_tiles; ++ti) {
        const long long tw0 = kProf ? clock64() : 0ll;
        mega_wait_bar(&sh.full_bar[rp.slot], rp.parity, w, 2u, k, 32u);
        if (kProf) t_full += clock64() - tw0;
        // rows in this tile (none once a wait has run out: the slot's row count may then be another operator's)
        const int n = *w.abort_flag ? 0 : min(sh.tile_n[rp.slot], rmax);
        const int nrows = n > group ? ((n - group + G - 1) * recipG) >> 16 : 0;      // rows of this group
        const int bufo = (int)(tile_no & (uint32_t)(kMegaRedBufs - 1)) * kRedBuf;
        uint32_t bw = ring + (uint32_t)rp.slot * (uint32_t)p.slot_bytes + w_lane;
        for (int p0 = 0; p0 < nrows; p0 += NR, bw += (uint32_t)NR * gw) {
            const int left = nrows - p0;
            uint32_t wa[NR];
            wa[0] = bw;
            if (NR > 1) wa[1 % NR] = bw + (left > 1 ? gw : 0u);    // rows past the end repeat row 0 (not stored)
            if (NR > 2) {
                wa[2 % NR] = bw + (left > 2 ? 2u * gw : 0u);
                wa[3 % NR] = bw + (left > 3 ? 3u * gw : 0u);
            }
            const long long tb0 = kProf ? clock64() : 0ll;
            const float v = mega_batch_f16<NP>(xs, wa, du, (left < NR ? left : NR) * NP, lane);
            if (storer && rj < left) red_w[bufo + p0] = v;
            if (kProf) t_batch += clock64() - tb0;
        }
        // last read of the slot and the partials of this warp are done: one arrival tells the copy and tail warps
        __syncwarp();
        if (lane == 0) mbar_arrive_n(&sh.empty_bar[rp.slot], my_arrive);
        ++tile_no;
        mega_ring_next(rp, p.nstage);
    }
}

// ---- int4 operators on the tensor cores -------------------------------------------------------------------------------
// The arithmetic of an int4 mat-vec is bound by instruction issue, not by the multiply-adds themselves: as scalar code
// a packed word costs 5 integer instructions to unpack and 8 multiply-adds. One warp-wide m16n8k16 step takes the
// unpacked words of 16 rows (two registers of a row's word per step) against the matching inputs, so a word costs its
// unpacking plus ONE further instruction. Only column 0 of the 16 x 8 result is used.
//   lane (g, t), g = lane / 4, t = lane % 4, holds for quantisation group G the 16-byte vector 4G + t of row g of the
//   tile's first block of 8 rows and of row g of the second block (rows 8..15; SwiGLU: the 8 up rows beside the 8
//   gate rows). Its B fragments are the table entries of slot 4G + t (the same for every g: only the lanes with
//   g == 0 feed column 0). After the 8 steps of a group the lanes with t == 0 hold the group's sums of rows g, g + 8.
// Unpacking: (w & 0x000f000f) | 0x64006400 = fp16 (1024 + n0, 1024 + n4); (w & 0x00f000f0) | 0x54005400 = fp16
// (64 + n1, 64 + n5) (the nibble sits 4 bits up in a mantissa whose unit is 1/16); the same on w >> 8. The offsets are
// taken out by the accumulator's start value.
__device__ __forceinline__ void mma_m16n8k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first step of an accumulator chain: no accumulator input (no registers to clear)
__device__ __forceinline__ void mma_m16n8k16_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

template <bool TWO, bool FIRST>
__device__ __forceinline__ void mega_mma_word(uint32_t wa, uint32_t wb, const uint4& xb, float (&acc0)[4], float (&acc1)[4])
{
    const uint32_t wa8 = wa >> 8;
    const uint32_t aa = and_or(wa, 0x000f000fu, 0x64006400u), ab = and_or(wa, 0x00f000f0u, 0x54005400u);
    const uint32_t ac = and_or(wa8, 0x000f000fu, 0x64006400u), ad = and_or(wa8, 0x00f000f0u, 0x54005400u);
    uint32_t ba = 0, bb = 0, bc = 0, bd = 0;
    if (TWO) {
        const uint32_t wb8 = wb >> 8;
        ba = and_or(wb, 0x000f000fu, 0x64006400u); bb = and_or(wb, 0x00f000f0u, 0x54005400u);
        bc = and_or(wb8, 0x000f000fu, 0x64006400u); bd = and_or(wb8, 0x00f000f0u, 0x54005400u);
    }
    if (FIRST) {
        mma_m16n8k16_first(acc0, aa, ba, ab, bb, xb.x, xb.y);   // nibbles 0, 4 | 1, 5 against (x0,x4) | (x1,x5)
        mma_m16n8k16_first(acc1, ac, bc, ad, bd, xb.z, xb.w);   // nibbles 2, 6 | 3, 7 against (x2,x6) | (x3,x7)
    } else {
        mma_m16n8k16(acc0, aa, ba, ab, bb, xb.x, xb.y);
        mma_m16n8k16(acc1, ac, bc, ad, bd, xb.z, xb.w);
    }
}

// Consumer side of one int4 operator. Warp q works on quantisation groups [q * upw, q * upw + upw) of ALL rows of every
// tile and leaves one partial sum per row; the tail warp adds the warps' partials in a fixed order. Rows of the slot past
// the end of a short tile hold whatever an earlier tile left there: any bit pattern unpacks to finite numbers, and nobody
// reads those rows' sums. The consumers do not follow the row ranges at all: the copy warp leaves a tile's first row and
// row count beside the slot (warp 0 needs them to fetch the residual values).
template <bool TWO, bool kProf>
__device__ __forceinline__ void mega_consume_mma(const MegaOp* __restrict__ gp, const MegaParams& p, int k, const MegaShared& sh, MegaRing& rp,
                                                 uint32_t& tile_no, const MegaWait& w, int my_tiles, long long& t_full, long long& t_batch)
{
    const int tid = (int)threadIdx.x - kMegaServiceThreads, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kw = gp->kw, upw = gp->np, tab_n = gp->tab_n;
    if (warp >= kw) {
        mega_skip_tiles(rp, tile_no, my_tiles, p.nstage);
        return;
    }
    const int grp0 = warp * upw;
    int cnt = gp->ngrp - grp0;
    cnt = cnt < upw ? cnt : upw;
    // arrival weight on a slot's empty barrier: the working warps of the operator add up to the barrier's fixed count
    const uint32_t my_arrive = (warp == 0) ? (kMegaBarCount - (uint32_t)kw + 1u) : 1u;
    const bool paired = gp->paired != 0;
    const uint32_t wrow = (uint32_t)gp->wrow, zrow = (uint32_t)gp->zrow, srow = (uint32_t)gp->srow;
    // second block: rows 8 .. 15 of the run, or (SwiGLU) rows 0 .. 7 of the second run
    const uint32_t blk_w = paired ? (uint32_t)gp->run_bytes : 8u * wrow;
    const uint32_t blk_z = paired ? (uint32_t)gp->run_bytes : 8u * zrow;
    const uint32_t blk_s = paired ? (uint32_t)gp->run_bytes : 8u * srow;
    const uint32_t w_lane = (uint32_t)g * wrow + (uint32_t)(grp0 * 4 + t) * 16u;
    const uint32_t z_lane = (uint32_t)gp->off_z + (uint32_t)g * zrow + (uint32_t)(grp0 >> 3) * 4u;
    const uint32_t s_lane = (uint32_t)gp->off_s + (uint32_t)g * srow + (uint32_t)grp0 * 2u;
    const uint32_t tab = smem_u32(sh.table);
    const uint32_t x_lane = tab + (uint32_t)(grp0 * 4 + t) * 16u;
    const uint32_t x_q = (uint32_t)tab_n * 16u;
    const uint32_t c_lane = tab + (uint32_t)(4 * tab_n + grp0) * 16u;
    constexpr int kRedBuf = kMegaConsumerWarps * kMegaRedRows;
    float* const red_w = sh.red + warp * kMegaRedRows + g;
    const uint32_t ring = smem_u32(sh.ring);
    const __half* const xres = (gp->kind == MOP_RESID && warp == 0) ? gp->out[0] : nullptr;

    for (int ti = 0; ti < my_tiles; ++ti) {
        const long long tw0 = kProf ? clock64() : 0ll;
        mega_wait_bar(&sh.full_bar[rp.slot], rp.parity, w, 2u, k, 32u);
        const long long tb0 = kProf ? clock64() : 0ll;
        if (kProf) t_full += tb0 - tw0;
        const int buf = (int)(tile_no & (uint32_t)(kMegaRedBufs - 1));
        // residual values for the tail: fetched here (the consumers hold the operator's dependency), parked beside the partials
        float resid = 0.f;
        bool res_lane = false;
        if (xres != nullptr && *w.abort_flag == 0u) {   // (not once a wait has run out: the slot's row and size may be stale)
            res_lane = lane < sh.tile_n[rp.slot];
            if (res_lane) resid = __half2float(__ldcg(xres + sh.tile_row[rp.slot] + lane));
        }
        const uint32_t sbase = ring + (uint32_t)rp.slot * (uint32_t)p.slot_bytes;
        float tot_a = 0.f, tot_b = 0.f;
        uint32_t aw = sbase + w_lane, ax = x_lane, ac = c_lane;
        int grp = grp0;
#pragma unroll 1
        for (int u = 0; u < cnt; ++u, aw += 64u, ax += 64u, ac += 16u, ++grp) {
            const uint4 va = lds_v4(aw);
            uint4 vb = make_uint4(0u, 0u, 0u, 0u);
            if (TWO) vb = lds_v4(aw + blk_w);
            const uint4 x0 = lds_v4(ax), x1 = lds_v4(ax + x_q), x2 = lds_v4(ax + 2u * x_q), x3 = lds_v4(ax + 3u * x_q);
            float c0, c1;
            asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(c0), "=f"(c1) : "r"(ac));
            // zero words and scales of this group for the lane's rows
            const uint32_t zo = (uint32_t)((grp >> 3) - (grp0 >> 3)) * 4u, so = (uint32_t)(grp - grp0) * 2u;
            uint32_t zwa, zwb = 0;
            unsigned short sca, scb = 0;
            asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zwa) : "r"(sbase + z_lane + zo));
            asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sca) : "r"(sbase + s_lane + so));
            if (TWO) {
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zwb) : "r"(sbase + z_lane + blk_z + zo));
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(scb) : "r"(sbase + s_lane + blk_s + so));
            }
            float acc0[4] = {c0, 0.f, c0, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
            mega_mma_word<TWO, false>(va.x, vb.x, x0, acc0, acc1);
            mega_mma_word<TWO, false>(va.y, vb.y, x1, acc0, acc1);
            mega_mma_word<TWO, false>(va.z, vb.z, x2, acc0, acc1);
            mega_mma_word<TWO, false>(va.w, vb.w, x3, acc0, acc1);
            const int zs = (grp & 7) * 4;
            const float za = (float)((zwa >> zs) & 0xFu);
            tot_a = fmaf(half_bits_to_float(sca), fmaf(-za, c1, acc0[0] + acc1[0]), tot_a);
            if (TWO) {
                const float zb = (float)((zwb >> zs) & 0xFu);
                tot_b = fmaf(half_bits_to_float(scb), fmaf(-zb, c1, acc0[2] + acc1[2]), tot_b);
            }
        }
        if (t == 0) {
            red_w[buf * kRedBuf] = tot_a;
            if (TWO) red_w[buf * kRedBuf + 8] = tot_b;
        }
        if (res_lane) sh.resid[buf * kMegaRedRows + lane] = resid;
        if (kProf) t_batch += clock64() - tb0;
        // last read of the slot and the partials of this warp are done: one arrival tells the copy and tail warps
        __syncwarp();
        if (lane == 0) mbar_arrive_n(&sh.empty_bar[rp.slot], my_arrive);
        ++tile_no;
        mega_ring_next(rp, p.nstage);
    }
}

// ---- the hot loop of the int4 operators, compiled as a function of its own --------------------------------------------
// Inlined into the kernel, the tile loop shares the register file of a 736-thread CTA (80 registers a thread) with
// everything else the kernel keeps alive, and spills. As a separate function it gets the whole budget: the caller's
// state is saved once per operator. Everything it touches is addressed by 32-bit shared-memory addresses.
struct MegaWaitShared {      // in shared memory: what a wait needs when it does not succeed at once
    long long budget;        // SM cycles
    DeviceStatus* status;
    unsigned int abort;      // some role of this CTA gave up
    unsigned int pad;
};
struct MegaLoop {
    uint32_t ring, full_bar, empty_bar, red, resid, tile_row, tile_n, table, wait;   // shared-memory addresses
    int nstage, slot_bytes, k, my_tiles;
};
struct MegaLoopState {
    int slot;
    uint32_t parity, tile_no;
};

__device__ __forceinline__ bool mbar_try_wait_a(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_suspend_a(uint32_t bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ unsigned short lds_u16(uint32_t a)
{
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts_f32(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }

// the barrier was not complete at the first look: sleep between polls, watch the abort flag and the clock
__device__ __noinline__ void mega_wait_slow(uint32_t bar, uint32_t parity, uint32_t ws, unsigned int code, int detail)
{
    const long long t0 = clock64();
    long long budget;
    asm volatile("ld.shared.s64 %0, [%1];" : "=l"(budget) : "r"(ws));
    for (uint32_t i = 0; i < (1u << 30); ++i) {
        if (mbar_try_wait_suspend_a(bar, parity, 1000u)) return;
        __nanosleep(32u);
        if (lds_u32(ws + 16u)) return;
        if (clock64() - t0 > budget) break;
    }
    DeviceStatus* status;
    asm volatile("ld.shared.u64 %0, [%1];" : "=l"(status) : "r"(ws + 8u));
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(ws + 16u), "r"(1u) : "memory");
    if (atomicCAS(&status->error, 0u, code) == 0u) status->detail = (unsigned int)detail;
}

// the arithmetic of one tile for one warp: two quantisation groups of the tile's one or two blocks of 8 rows
template <bool TWO>
__device__ __forceinline__ void mega_tile_math(uint32_t sbase, uint32_t a_w, uint32_t blk_w, uint32_t o1, uint32_t a_z, uint32_t a_zb, uint32_t a_s,
                                           uint32_t a_sb, uint32_t so1, int zs0, const uint4 (&xr0)[4], const uint4 (&xr1)[4], float c00, float c01,
                                           float c10, float c11, uint32_t red_a, int lane)
{
    float tot_a, tot_b = 0.f;
    {
        // first group
        const uint4 va = lds_v4(sbase + a_w);
        uint4 vb = make_uint4(0u, 0u, 0u, 0u);
        if (TWO) vb = lds_v4(sbase + a_w + blk_w);
        float acc0[4], acc1[4];
        mega_mma_word<TWO, true>(va.x, vb.x, xr0[0], acc0, acc1);
        mega_mma_word<TWO, false>(va.y, vb.y, xr0[1], acc0, acc1);
        mega_mma_word<TWO, false>(va.z, vb.z, xr0[2], acc0, acc1);
        mega_mma_word<TWO, false>(va.w, vb.w, xr0[3], acc0, acc1);
        tot_a = acc0[0] + acc1[0] + c00;
        if (TWO) tot_b = acc0[2] + acc1[2] + c00;
    }
    float sec_a, sec_b = 0.f;
    {
        // second group
        const uint4 va = lds_v4(sbase + a_w + o1);
        uint4 vb = make_uint4(0u, 0u, 0u, 0u);
        if (TWO) vb = lds_v4(sbase + a_w + blk_w + o1);
        float acc0[4], acc1[4];
        mega_mma_word<TWO, true>(va.x, vb.x, xr1[0], acc0, acc1);
        mega_mma_word<TWO, false>(va.y, vb.y, xr1[1], acc0, acc1);
        mega_mma_word<TWO, false>(va.z, vb.z, xr1[2], acc0, acc1);
        mega_mma_word<TWO, false>(va.w, vb.w, xr1[3], acc0, acc1);
        sec_a = acc0[0] + acc1[0] + c10;
        if (TWO) sec_b = acc0[2] + acc1[2] + c10;
    }
    {
        const uint32_t zw = lds_u32(sbase + a_z);
        const unsigned short s0 = lds_u16(sbase + a_s), s1 = lds_u16(sbase + a_s + so1);
        const float z0 = (float)((zw >> zs0) & 0xFu), z1 = (float)((zw >> (zs0 + 4)) & 0xFu);
        tot_a = half_bits_to_float(s0) * fmaf(-z0, c01, tot_a);
        tot_a = fmaf(half_bits_to_float(s1), fmaf(-z1, c11, sec_a), tot_a);
        if ((lane & 3) == 0) sts_f32(red_a, tot_a);
    }
    if (TWO) {
        const uint32_t zw = lds_u32(sbase + a_zb);
        const unsigned short s0 = lds_u16(sbase + a_sb), s1 = lds_u16(sbase + a_sb + so1);
        const float z0 = (float)((zw >> zs0) & 0xFu), z1 = (float)((zw >> (zs0 + 4)) & 0xFu);
        tot_b = half_bits_to_float(s0) * fmaf(-z0, c01, tot_b);
        tot_b = fmaf(half_bits_to_float(s1), fmaf(-z1, c11, sec_b), tot_b);
        if ((lane & 3) == 0) sts_f32(red_a + 32u, tot_b);
    }
}

// Exactly two quantisation groups per warp (an odd last one: zero inputs against the first group's weights): the warp's
// B fragments and group constants stay in registers for the whole operator, and a tile is straight-line code.
template <bool TWO, bool kProf>
__device__ __noinline__ MegaLoopState mega_consume_mma_reg(const MegaOp* __restrict__ gp, const MegaLoop a, MegaLoopState st, long long* prof)
{
    const int lane = threadIdx.x & 31, warp = ((int)threadIdx.x - kMegaServiceThreads) >> 5;
    const int kw = gp->kw;
    if (warp >= kw) {
        MegaRing rp{st.slot, st.parity};
        mega_skip_tiles(rp, st.tile_no, a.my_tiles, a.nstage);
        st.slot = rp.slot;
        st.parity = rp.parity;
        return st;
    }
    const uint32_t my_arrive = (warp == 0) ? (kMegaBarCount - (uint32_t)kw + 1u) : 1u;
    uint32_t blk_w, a_w, a_z, a_zb, a_s, a_sb, o1;
    int zs0;
    uint4 xr0[4], xr1[4];   // stationary inputs
    float c00, c01, c10 = 0.f, c11 = 0.f;
    {
        const int g = lane >> 2, t = lane & 3, grp0 = warp * 2, tab_n = gp->tab_n;
        const bool second = grp0 + 1 < gp->ngrp;
        const bool paired = gp->paired != 0;
        const uint32_t wrow = (uint32_t)gp->wrow, zrow = (uint32_t)gp->zrow, srow = (uint32_t)gp->srow;
        // second block: rows 8 .. 15 of the run, or (SwiGLU) rows 0 .. 7 of the second run
        blk_w = paired ? (uint32_t)gp->run_bytes : 8u * wrow;
        a_w = (uint32_t)g * wrow + (uint32_t)(grp0 * 4 + t) * 16u;
        o1 = second ? 64u : 0u;
        a_z = (uint32_t)gp->off_z + (uint32_t)g * zrow + (uint32_t)(grp0 >> 3) * 4u;   // both groups sit in one zero word
        a_zb = a_z + (paired ? (uint32_t)gp->run_bytes : 8u * zrow);
        a_s = (uint32_t)gp->off_s + (uint32_t)g * srow + (uint32_t)grp0 * 2u;
        a_sb = a_s + (paired ? (uint32_t)gp->run_bytes : 8u * srow);
        zs0 = (grp0 & 7) * 4;
        const uint32_t ax = a.table + (uint32_t)(grp0 * 4 + t) * 16u, xq = (uint32_t)tab_n * 16u, ac = a.table + (uint32_t)(4 * tab_n + grp0) * 16u;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            xr0[q] = lds_v4(ax + (uint32_t)q * xq);
            xr1[q] = second ? lds_v4(ax + (uint32_t)q * xq + 64u) : make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(c00), "=f"(c01) : "r"(ac));
        if (second) asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(c10), "=f"(c11) : "r"(ac + 16u));
    }
    const uint32_t so1 = o1 >> 5;   // 2 bytes on to the second group's scale, 0 without one
    const uint32_t red_w = a.red + (uint32_t)(warp * kMegaRedRows + (lane >> 2)) * 4u;
    constexpr uint32_t kRedBufBytes = kMegaConsumerWarps * kMegaRedRows * 4;
    const __half* const xres = (gp->kind == MOP_RESID && warp == 0) ? gp->out[0] : nullptr;
    int slot = st.slot;
    uint32_t parity = st.parity, tile_no = st.tile_no;
    long long t_full = 0, t_batch = 0;

    for (int ti = 0; ti < a.my_tiles; ++ti) {
        const long long tw0 = kProf ? clock64() : 0ll;
        const uint32_t fb = a.full_bar + (uint32_t)slot * 8u;
        if (!mbar_try_wait_a(fb, parity)) mega_wait_slow(fb, parity, a.wait, 2u, a.k);
        const long long tb0 = kProf ? clock64() : 0ll;
        if (kProf) t_full += tb0 - tw0;
        const uint32_t bufo = (tile_no & (uint32_t)(kMegaRedBufs - 1)) * kRedBufBytes;
        // residual values for the tail: fetched here (the consumers hold the operator's dependency), parked beside the partials
        if (xres != nullptr && lds_u32(a.wait + 16u) == 0u) {   // (not once a wait has run out: the slot's row and size may be stale)
            const int n = (int)lds_u32(a.tile_n + (uint32_t)slot * 4u);
            if (lane < n) {
                const int row = (int)lds_u32(a.tile_row + (uint32_t)slot * 4u);
                sts_f32(a.resid + ((tile_no & (uint32_t)(kMegaRedBufs - 1)) * (uint32_t)kMegaRedRows + (uint32_t)lane) * 4u,
                        __half2float(__ldcg(xres + row + lane)));
            }
        }
        const uint32_t sbase = a.ring + (uint32_t)slot * (uint32_t)a.slot_bytes;
#ifndef ML2_DIAG_NOMATH
        mega_tile_math<TWO>(sbase, a_w, blk_w, o1, a_z, a_zb, a_s, a_sb, so1, zs0, xr0, xr1, c00, c01, c10, c11, red_w + bufo, lane);
#endif
        if (kProf) t_batch += clock64() - tb0;
        // last read of the slot and the partials of this warp are done: one arrival tells the copy and tail warps
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(a.empty_bar + (uint32_t)slot * 8u), "r"(my_arrive) : "memory");
        ++tile_no;
        if (++slot == a.nstage) { slot = 0; parity ^= 1u; }
    }
    if (kProf) { prof[0] += t_full; prof[1] += t_batch; }
    st.slot = slot;
    st.parity = parity;
    st.tile_no = tile_no;
    return st;
}

// kProf adds cycle counters around the waits (diagnostics); the production instantiation carries none.
template <bool kProf>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const MegaParams p)
{
    auto now = [&]() -> long long { return kProf ? clock64() : 0ll; };
    extern __shared__ __align__(128) unsigned char smem_raw[];   // [ring: nstage * slot_bytes][input table | attention scores, partial outputs]
    __shared__ __align__(8) uint64_t full_bar[kMegaMaxStages];
    __shared__ __align__(8) uint64_t empty_bar[kMegaMaxStages];
    __shared__ float s_red[kMegaRedBufs * kMegaConsumerWarps * kMegaRedRows];
    __shared__ float s_part[2][kMegaConsumerWarps];
    __shared__ float s_resid[kMegaRedBufs * kMegaRedRows];
    __shared__ float s_att_tmp[kMegaConsumerWarps];
    __shared__ __align__(16) __half s_q[kHeadMax];
    __shared__ float s_best_v[kMegaConsumerWarps];
    __shared__ int s_best_i[kMegaConsumerWarps];
    __shared__ int s_tile_row[kMegaMaxStages], s_tile_n[kMegaMaxStages];
    __shared__ __align__(16) uint4 s_meta[kMegaRedBufs][2];   // the last 32 bytes of the descriptors of the tiles in flight (copy warp -> tail warp)
    __shared__ __align__(16) MegaWaitShared s_wait;
    volatile unsigned int& s_abort = s_wait.abort;
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
        s_wait.abort = 0;
        s_wait.budget = p.wait_cycles;
        s_wait.status = p.status;
        s_tailed = 0;
        s_released = 0;
        mbar_fence_init();
    }
    if (tid < kOpWords) reinterpret_cast<uint32_t*>(&s_ops[0])[tid] = reinterpret_cast<const uint32_t*>(p.ops)[tid];
    __syncthreads();

    MegaWait w;
    w.abort_flag = &s_wait.abort;
    w.status = p.status;
    w.budget = p.wait_cycles;

    if (warp == 0) {
        // ================= copy warp ==========================================================================
        // Tile t of this CTA (counted over the whole token) lives in ring slot t % nstage. When all consumer warps have
        // arrived on a slot's empty barrier, the slot is refilled with the tile that is `nstage` further on. Weights
        // do not depend on activations, so the copies run ahead of the arithmetic across operator boundaries.
        // Lanes 0 .. 5 own one copy of a tile each (their 16 bytes of the descriptor), lane 6 the tile's row, size and
        // byte count; the next tile's descriptor is fetched while this one waits for its slot.
        const uint64_t pol = policy_evict_first();
        const int t_begin = p.tile_begin[cta], ntile = p.tile_begin[cta + 1] - t_begin;
        const uint4* td = reinterpret_cast<const uint4*>(p.tiles + t_begin) + (lane < 8 ? lane : 7);
        constexpr size_t kStride = sizeof(MegaTile) / sizeof(uint4);
        auto fetch = [&](int i) -> uint4 {   // issued where it stands (not moved by the compiler): two tiles before it is needed
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (i < ntile)
                asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(td + (size_t)i * kStride));
            return v;
        };
        MegaRing ri{0, 0u};
        long long tp_wait = 0, tp_all0 = now();
        uint4 nxt = fetch(0), nxt2 = fetch(1);
        for (int i = 0; i < ntile; ++i) {
            const uint4 cur = nxt;
            nxt = nxt2;
            nxt2 = fetch(i + 2);
            if (i >= p.nstage) {
                const long long tw0 = now();
                if (lane == 0) {
                    mega_wait_bar(&empty_bar[ri.slot], ri.parity ^ 1u, w, 1u, i, 256u);
                    // tile (i - nstage) is consumed. The tail warp learns that from the barrier's phase parity, which
                    // repeats after two refills: this counter settles it if the tail warp ever falls that far behind
                    *(volatile unsigned int*)&s_released = (unsigned int)(i - p.nstage) + 1u;
                    // the tail warp reads the partial sums of a tile from one of kMegaRedBufs buffers and tells tiles
                    // apart by the barrier's phase parity: it must not fall further behind than that allows
                    const long long t0 = clock64();
                    while ((int)((unsigned int)i - *(volatile unsigned int*)&s_tailed) > kMegaRedBufs - 1 && !s_abort) {
                        if (clock64() - t0 > w.budget) { mega_give_up(w, 7u, i); break; }
                    }
                }
                __syncwarp();
                tp_wait += now() - tw0;
                if (s_abort) break;   // some wait ran out: no further copies
            }
            const uint32_t total = __shfl_sync(0xffffffffu, cur.w, 6);
            // the tile's row and size for the consumers, its whole tail part for the tail warp: ordered before their reads by the barriers
            if (lane == 6) { s_tile_row[ri.slot] = (int)cur.x; s_tile_n[ri.slot] = (int)cur.y; }
            if (lane == 6 || lane == 7) s_meta[i & (kMegaRedBufs - 1)][lane - 6] = cur;
            __syncwarp();
#ifdef ML2_DIAG_NOCOPY
            if (lane == 0) mbar_arrive(&full_bar[ri.slot]);   // pipeline probe: no weight copies
#else
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[ri.slot], total);
            __syncwarp();
            if (lane < 6 && cur.z != 0u) {
                const void* src = reinterpret_cast<const void*>((uint64_t)cur.x | ((uint64_t)cur.y << 32));
                bulk_g2s(smem_raw + (size_t)ri.slot * p.slot_bytes + cur.w, src, cur.z, &full_bar[ri.slot], pol);
            }
#endif
            mega_ring_next(ri, p.nstage);
        }
        if (kProf && p.prof && lane == 0) {
            long long* o = p.prof + (size_t)cta * 64;
            o[32] = now() - tp_all0;
            o[33] = tp_wait;
        }
        return;
    }

    if (warp == 1) {
        // ================= tail warp ===========================================================================
        // When all consumer warps have arrived on a slot's empty barrier, the tile that was in it gets its tail: the
        // fixed-order sum over the warps' partials of every row, the operator's rounding and store. After the tail of
        // the operator's last tile on this CTA the operator is published (release) on its device-wide counter.
        const int ntile = p.tile_begin[cta + 1] - p.tile_begin[cta];
        MegaRing rf{0, 0u};
        long long tf_wait = 0, tf_all0 = now(), tf_sum = 0, tf_next = 0, tf_pub = 0, tf_epi = 0;
        for (int i = 0; i < ntile; ++i) {
            const long long tw0 = now();
            if (lane == 0 && !mbar_try_wait(&empty_bar[rf.slot], rf.parity)) {
                const long long t0 = clock64();
                for (uint32_t it = 0; it < (1u << 30); ++it) {
                    if (mbar_try_wait_suspend(&empty_bar[rf.slot], rf.parity, 1000u)) break;
                    __nanosleep(128u);
                    if ((int)(*(volatile unsigned int*)&s_released - (unsigned int)i) > 0 || s_abort) break;
                    if (clock64() - t0 > w.budget) { mega_give_up(w, 3u, i); break; }
                }
            }
            __syncwarp();
            // some wait of this CTA ran out: the tiles that follow may never have been issued (no descriptor, no partial
            // sums); nothing is stored or published any more
            if (s_abort) break;
            const long long ts0 = now();
            tf_wait += ts0 - tw0;
            const int buf = i & (kMegaRedBufs - 1);
            // what the copy warp left about this tile (the last 32 bytes of its descriptor)
            const uint4 m0 = s_meta[buf][0], m1 = s_meta[buf][1];
            const int row = (int)m0.x, n = (int)m0.y;
            const int k = (int)(m0.z & 0xffffu);
            const int f_kind = (int)(m1.z & 7u), f_kw = (int)((m1.z >> 8) & 0xffu), f_G = (int)((m1.z >> 16) & 0xffu);
            const bool f_paired = (m1.z & 8u) != 0, f_mma = (m1.z & 16u) != 0;
            __half* f_out = reinterpret_cast<__half*>((uint64_t)m1.x | ((uint64_t)m1.y << 32));
            if (m0.z & kTileCacheRow) f_out += (long long)p.pos * p.kv_row_stride;
            const MegaOp* f_gp = p.ops + k;
            const float* red = s_red + buf * (kMegaConsumerWarps * kMegaRedRows);
#ifdef ML2_DIAG_NOTAIL
            if (false) {
#else
            if (f_mma) {
#endif
                // int4: every working warp left one partial per row (second block / up rows 8 further on). Two lanes per
                // unit add half of the warps each, in a fixed order; all loads are issued before the first addition.
                constexpr int kHalf = (kMegaConsumerWarps + 1) / 2;
                const int j = lane & 15, kh = (f_kw + 1) >> 1;
                const int q0 = lane < 16 ? 0 : kh, nq = lane < 16 ? kh : f_kw - kh;
                const float* rq = red + q0 * kMegaRedRows + j;
                float va[kHalf], vb[kHalf];
#pragma unroll
                for (int q = 0; q < kHalf; ++q) {
                    va[q] = q < nq ? rq[q * kMegaRedRows] : 0.f;
                    vb[q] = (f_paired && q < nq) ? rq[q * kMegaRedRows + 8] : 0.f;
                }
                float sa = 0.f, sb = 0.f;
#pragma unroll
                for (int q = 0; q < kHalf; ++q) { sa += va[q]; sb += vb[q]; }
                sa += __shfl_xor_sync(0xffffffffu, sa, 16);
                sb += __shfl_xor_sync(0xffffffffu, sb, 16);
                const long long te0 = now();
                tf_epi -= te0 - ts0;
                if (lane < n) {
                    const float resid = (f_kind == MOP_RESID) ? s_resid[buf * kMegaRedRows + lane] : 0.f;
                    mega_epilogue(f_gp, f_kind, f_out, row + lane, sa, sb, resid);
                }
#ifdef ML2_DIAG_NOTAIL
            } else if (false) {
#else
            } else {
#endif
                // fp16: unit j is row u of group g; the group's warps left its partial at row u
                const int f_recipG = (65536 + f_G - 1) / f_G;
                for (int j = lane; j < n; j += 32) {
                    const int u = (j * f_recipG) >> 16, g = j - u * f_G;
                    const float* rg = red + g * f_kw * kMegaRedRows + u;
                    float sa = 0.f;
                    for (int q = 0; q < f_kw; ++q) sa += rg[q * kMegaRedRows];
                    mega_epilogue(f_gp, f_kind, f_out, row + j, sa, 0.f, 0.f);
                }
            }
            const long long ts1 = now();
            tf_sum += ts1 - ts0;
            tf_epi += ts1 - ts0;
            // this CTA's share of the operator is stored: publish it (the warp barrier orders every lane's stores before the release)
            __syncwarp();
            const long long tpb0 = now();
            if (m0.z & kTileLast) {
                if (m1.z & 32u) {
                    if (lane < f_gp->tp) red_release_sys_add(f_gp->peer_done[lane], 1u);   // on every rank's counter, after the peer stores
                } else if (lane == 0) {
                    red_release_gpu_add(&p.done[k], 1u);
                }
            }
            tf_pub += now() - tpb0;
            if (lane == 0) *(volatile unsigned int*)&s_tailed = (unsigned int)i + 1u;   // the partial buffer is free again
            mega_ring_next(rf, p.nstage);
            tf_next += now() - ts1;
        }
        if (kProf && p.prof && lane == 0) {
            long long* o = p.prof + (size_t)cta * 64;
            o[34] = now() - tf_all0;
            o[35] = tf_wait;
            o[36] = tf_epi; o[37] = tf_sum; o[38] = tf_next; o[39] = tf_pub;
        }
        return;
    }

    // ================= consumers (numbered from 0 after the two service warps) ================================
    {
    const int tid = (int)threadIdx.x - kMegaServiceThreads;
    const int warp = tid >> 5;
    MegaShared sh;
    sh.ring = smem_raw;
    sh.table = smem_raw + (size_t)p.nstage * p.slot_bytes;
    sh.full_bar = full_bar;
    sh.empty_bar = empty_bar;
    sh.red = s_red;
    sh.part = &s_part[0][0];
    sh.resid = s_resid;
    sh.tile_row = s_tile_row;
    sh.tile_n = s_tile_n;
    MegaRing rp{0, 0u};
    uint32_t tile_no = 0;
    int next_tiles = p.op_tiles[cta];   // this CTA's tiles of operator 0; the next operator's count is fetched one operator ahead
    long long t_dep = 0, t_full = 0, t_attn = 0, t_pro = 0, t_batch = 0, t_all0 = now();
    long long tk_dep[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tk_pro[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tk_run[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tk_batch[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tk_full[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < p.nops; ++k) {
        const MegaOp* gp = &s_ops[k & 1];
        const MegaOp& op = *gp;
        const int my_tiles = next_tiles;
        if (k + 1 < p.nops) next_tiles = __ldg(p.op_tiles + (size_t)(k + 1) * ncta + cta);
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
        const bool is_int4 = op.fmt == 0;
        const int tab_n = op.tab_n;
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

        const long long trun0 = now(), tb_before = t_batch, tf_before = t_full;
        if (is_int4) {
            if (op.np <= 2) {
                MegaLoop la;
                la.ring = smem_u32(sh.ring); la.full_bar = smem_u32(full_bar); la.empty_bar = smem_u32(empty_bar);
                la.red = smem_u32(s_red); la.resid = smem_u32(s_resid); la.tile_row = smem_u32(s_tile_row); la.tile_n = smem_u32(s_tile_n);
                la.table = smem_u32(sh.table); la.wait = smem_u32(&s_wait);
                la.nstage = p.nstage; la.slot_bytes = p.slot_bytes; la.k = k; la.my_tiles = my_tiles;
                MegaLoopState ls{rp.slot, rp.parity, tile_no};
                long long pr[2] = {0, 0};
                ls = op.two ? mega_consume_mma_reg<true, kProf>(gp, la, ls, pr) : mega_consume_mma_reg<false, kProf>(gp, la, ls, pr);
                rp.slot = ls.slot; rp.parity = ls.parity; tile_no = ls.tile_no;
                if (kProf) { t_full += pr[0]; t_batch += pr[1]; }
            } else {
                if (op.two) mega_consume_mma<true, kProf>(gp, p, k, sh, rp, tile_no, w, my_tiles, t_full, t_batch);
                else mega_consume_mma<false, kProf>(gp, p, k, sh, rp, tile_no, w, my_tiles, t_full, t_batch);
            }
        } else {
            if (op.np == 1) mega_consume_f16<1, kProf>(gp, p, k, sh, rp, tile_no, w, my_tiles, t_full, t_batch);
            else mega_consume_f16<2, kProf>(gp, p, k, sh, rp, tile_no, w, my_tiles, t_full, t_batch);
        }
        tk_run[kk] += now() - trun0;
        tk_batch[kk] += t_batch - tb_before;
        tk_full[kk] += t_full - tf_before;

        // ---- hand-off: the tail warp publishes the operator after the tail of this CTA's last tile; a CTA that
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
        for (int q = 0; q < 8; ++q) { o[8 + q] = tk_dep[q]; o[16 + q] = tk_pro[q]; o[24 + q] = tk_run[q]; o[40 + q] = tk_batch[q]; o[48 + q] = tk_full[q]; }
    }
    }
}

}  // namespace ml2
