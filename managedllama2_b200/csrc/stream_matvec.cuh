// Streaming batch-1 mat-vec for sm_100a: out = epilogue(W . prologue(in)).
//
// One kernel template covers the reference's whole mat-vec family
// (native/mat_vec_kernel.cu of GilesBathgate/ManagedLlama2):
//   * AWQ int4 group-128 weights in the QWeight layout (sum_mat_vec_int4, :83-142) with the
//     residual (:144-164), QKV (:179-203) and SwiGLU (:206-234) epilogues, and
//   * plain fp16 weights (mat_vec_kernel, :14-49; the classifier).
//
// Design (not the reference's one-warp-per-output mapping):
//   * A producer warp streams whole weight rows (plus their zero words and scales) from HBM into
//     a ring of shared-memory stages with 1-D bulk async copies (TMA engine, mbarrier
//     completion, evict-first L2 hint). Weights never depend on the previous kernel, so the ring
//     is filled BEFORE the programmatic-dependent-launch wait: HBM keeps streaming across kernel
//     boundaries while the activations of the previous operator are still being produced.
//   * The input vector is stationary in registers: k-warp `kw`, lane `l` owns the 32 inputs
//     [32u, 32u+32) with u = 32*kw + l, i.e. exactly one 16-byte weight vector of every row, all
//     inside one quantisation group. Rows stream past it; every weight byte is read once.
//   * Dequantisation is two logic ops per nibble pair: (w & 0x000f000f) | 0x64006400 is the fp16
//     pair (1024+n, 1024+n'), (w & 0x00f000f0) | 0x64006400 is (1024+16n, 1024+16n'). They are fed
//     to the Blackwell mixed-precision FMA (fp16 x fp16 + fp32, exact product) against the fp16
//     inputs; the 1024 offsets are removed exactly by starting the two accumulators at
//     -1024*sum(x_even) and -1024*sum(x_odd). Zero point and scale are applied once per lane and
//     row: s * (sum x.n - z * sum x).
//   * Lane partials of RW rows are combined with a transposing shuffle reduction, k-warps are
//     summed in a fixed order through shared memory (deterministic), and the epilogue rounds to
//     fp16 exactly where the reference kernels do.
#pragma once

#include "common.cuh"

namespace ml2 {

enum class Fmt : int { Int4 = 0, F16 = 1 };
enum class Epi : int { Store = 0, Residual = 1, SwiGLU = 2, PartialF32 = 3, QKVRope = 4 };
enum class Pro : int { Plain = 0, RMSNorm = 1 };

struct QWPtrs {
    const uint32_t* w;  // [cols][wsize] packed nibbles (Int4) or fp16 rows viewed as words (F16)
    const uint32_t* z;  // [cols][zsize] packed zero points
    const __half* s;    // [cols][ssize] group scales
};

struct MatVecParams {
    QWPtrs mat[3];
    __half* out[3];            // Store / QKVRope: one output per matrix; Residual / SwiGLU: out[0]
    float* out_f32;            // PartialF32
    const __half* in;          // [rows]
    const __half* gamma;       // [rows], Pro::RMSNorm
    const float2* rope_table;  // [seq][head_size/2] (cos, sin), Epi::QKVRope
    const int* pos_ptr;        // device-resident position (graph replay); null -> pos_imm
    DeviceStatus* status;
    long long kv_row_stride;   // elements added to out[1], out[2] per position (QKVRope with pos_ptr)
    float eps;
    int pos_imm;
    int rows, cols;            // d_in, d_out (per matrix)
    int nmat;
    int wsize, zsize, ssize;   // per-output sizes: words, words, halves (F16: wsize = rows/2, others 0)
    int units;                 // 16-byte vectors per output row = wsize / 4
    int kw, mw;                // k-warps per row, chunks (row groups) per stage
    int nstage;                // ring depth
    int chunk_bytes;           // shared-memory bytes of one chunk (RW rows of weights, zeros, scales)
    int woff_z, woff_s;        // byte offsets of the zeros / scales sub-regions inside a chunk
    int ntiles;                // stage-tiles in the whole problem
    int head_size;
};

struct Chunk {
    int m, row0, nrows;
};

template <Epi E, int RW>
__device__ __forceinline__ Chunk chunk_of(const MatVecParams& p, int tile, int mw)
{
    Chunk c;
    if (E == Epi::SwiGLU) {
        const int pair = tile * (p.mw >> 1) + (mw >> 1);
        c.m = mw & 1;  // 0 = gate, 1 = up: the same output rows of both matrices share a stage
        c.row0 = pair * RW;
    } else if (E == Epi::QKVRope) {
        // rotate-half partners (i, i + head/2) of the same head share a stage
        const int pair = tile * (p.mw >> 1) + (mw >> 1);
        const int half = p.head_size >> 1;
        const int ppm = (p.cols >> 1) / RW;  // pairs per matrix
        c.m = pair / ppm;
        const int pp = pair - c.m * ppm;
        const int pph = half / RW;
        const int head = pp / pph;
        c.row0 = head * p.head_size + (pp - head * pph) * RW + (mw & 1) * half;
    } else {
        const int cid = tile * p.mw + mw;
        const int cpm = ceil_div(p.cols, RW);
        c.m = cid / cpm;
        c.row0 = (cid - c.m * cpm) * RW;
    }
    int n = p.cols - c.row0;
    n = n < 0 ? 0 : (n > RW ? RW : n);
    c.nrows = (c.m < p.nmat) ? n : 0;
    return c;
}

// Transposing reduction: every lane holds RW partial sums; afterwards lane (32/RW)*r holds the
// warp total of row r in v[0].
template <int RW>
__device__ __forceinline__ void transpose_reduce(float (&v)[RW], int lane)
{
    int off = 16;
#pragma unroll
    for (int n = RW; n > 1; n >>= 1) {
        const bool hi = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < n / 2; ++j) {
            const float send = hi ? v[j] : v[j + n / 2];
            const float keep = hi ? v[j + n / 2] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

// 8 nibbles of one word against the 8 matching inputs. xp[0..3] = (x0,x4) (x1,x5) (x2,x6) (x3,x7) as fp16 pairs.
//   a = (w & 0x000f000f) | 0x64006400   halves = fp16(1024 + n0), fp16(1024 + n4)          -> mixed FMAs with x0, x4 (acc A, D)
//   b = (w & 0x00f000f0) | 0x64006400   halves = fp16(1024 + 16*n1), fp16(1024 + 16*n5)    -> mixed FMAs with x1, x5 (acc B)
//   c, d: the same on w >> 8 (n2, n6 and n3, n7).
// The constant offsets (1024 * sum of the inputs) are removed by the accumulators' initial values; B carries a factor 16.
// The mixed FMA reads either half of a register at no cost (no extraction instruction is issued).
struct XSlice {
    uint32_t xp[16];   // fp16 pairs for the mixed FMAs
    float a0, b0;      // accumulator start values: -1024 * S(even inputs), -1024 * S(odd inputs)
    float c1;          // sum of all 32 inputs (zero-point term)
};

// (w & mask) | bits as ONE three-input logic instruction. Written as `(w & mask) | bits` in C++ the compiler emits an AND
// and an OR (measured: 9 instead of 5 integer-pipe instructions per packed word, and that pipe bounds this loop).
__device__ __forceinline__ uint32_t and_or(uint32_t w, uint32_t mask, uint32_t bits)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(d) : "r"(w), "r"(mask), "r"(bits));
    return d;
}

__device__ __forceinline__ void word_dot(uint32_t w, const uint32_t* xp, float& A, float& B, float& D)
{
    const uint32_t a = and_or(w, 0x000f000fu, 0x64006400u);
    const uint32_t b = and_or(w, 0x00f000f0u, 0x64006400u);
    const uint32_t w8 = w >> 8;
    const uint32_t c = and_or(w8, 0x000f000fu, 0x64006400u);
    const uint32_t d = and_or(w8, 0x00f000f0u, 0x64006400u);
    A = fma_f16_f32(lo16(a), lo16(xp[0]), A);
    D = fma_f16_f32(hi16(a), hi16(xp[0]), D);
    B = fma_f16_f32(lo16(b), lo16(xp[1]), B);
    B = fma_f16_f32(hi16(b), hi16(xp[1]), B);
    A = fma_f16_f32(lo16(c), lo16(xp[2]), A);
    D = fma_f16_f32(hi16(c), hi16(xp[2]), D);
    B = fma_f16_f32(lo16(d), lo16(xp[3]), B);
    B = fma_f16_f32(hi16(d), hi16(xp[3]), B);
}

__device__ __forceinline__ float half_bits_to_float(unsigned short h) { return __half2float(__ushort_as_half(h)); }

// Builds the stationary input slice of a lane from its 32 inputs in natural order (16 fp16 pairs). The sums come
// from mixed-precision FMAs against the constant -1024 (fp16 in, fp32 accumulate): no fp16 -> fp32 conversions,
// which issue at a fraction of the FMA rate.
__device__ __forceinline__ void make_xslice(const uint32_t (&xr)[16], XSlice& xs)
{
    constexpr unsigned short kM1024 = 0xE400;   // fp16 -1024
    float e0 = 0.f, e1 = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t h01 = xr[4 * j], h23 = xr[4 * j + 1], h45 = xr[4 * j + 2], h67 = xr[4 * j + 3];
        xs.xp[4 * j + 0] = __byte_perm(h01, h45, 0x5410);   // (x0, x4)
        xs.xp[4 * j + 1] = __byte_perm(h01, h45, 0x7632);   // (x1, x5)
        xs.xp[4 * j + 2] = __byte_perm(h23, h67, 0x5410);   // (x2, x6)
        xs.xp[4 * j + 3] = __byte_perm(h23, h67, 0x7632);   // (x3, x7)
        e0 = fma_f16_f32(lo16(h01), kM1024, e0);
        o0 = fma_f16_f32(hi16(h01), kM1024, o0);
        e1 = fma_f16_f32(lo16(h23), kM1024, e1);
        o1 = fma_f16_f32(hi16(h23), kM1024, o1);
        e0 = fma_f16_f32(lo16(h45), kM1024, e0);
        o0 = fma_f16_f32(hi16(h45), kM1024, o0);
        e1 = fma_f16_f32(lo16(h67), kM1024, e1);
        o1 = fma_f16_f32(hi16(h67), kM1024, o1);
    }
    xs.a0 = e0 + e1;                                   // -1024 * S(even inputs)
    xs.b0 = o0 + o1;                                   // -1024 * S(odd inputs)
    xs.c1 = (xs.a0 + xs.b0) * -0.0009765625f;          // S(all inputs): the scaling by 1/1024 is exact
}

// Loads the lane's input slice (NX halves starting at element e0), optionally applying RMSNorm
// (native/rmsnorm_kernel.cu:12-35: fp32 squares, rms = 1/sqrtf(ss/n + eps), out = half(rms*gamma*x)).
// Returns the slice as NX/2 packed half2 words in natural order.
template <Pro P, int NX>
__device__ __forceinline__ void load_input(const MatVecParams& p, int e0, bool first_mw, int kw_id, int ncons,
                                           float* s_part, uint32_t (&xr)[NX / 2])
{
    const int rows = p.rows;
#pragma unroll
    for (int v = 0; v < NX / 8; ++v) {
        const int e = e0 + v * 8;
        uint4 t = make_uint4(0, 0, 0, 0);
        if (e + 8 <= rows) {
            t = *reinterpret_cast<const uint4*>(p.in + e);
        } else if (e < rows) {
            unsigned short h[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = (e + i < rows) ? __half_as_ushort(p.in[e + i]) : (unsigned short)0;
            t = make_uint4(h[0] | (uint32_t)h[1] << 16, h[2] | (uint32_t)h[3] << 16, h[4] | (uint32_t)h[5] << 16,
                           h[6] | (uint32_t)h[7] << 16);
        }
        xr[v * 4 + 0] = t.x;
        xr[v * 4 + 1] = t.y;
        xr[v * 4 + 2] = t.z;
        xr[v * 4 + 3] = t.w;
    }
    if constexpr (P == Pro::RMSNorm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NX / 2; ++i) {
            const float a = half_bits_to_float(lo16(xr[i])), b = half_bits_to_float(hi16(xr[i]));
            ss = fmaf(a, a, ss);
            ss = fmaf(b, b, ss);
        }
        ss = warp_sum(ss);
        if (first_mw && (threadIdx.x & 31) == 0) s_part[kw_id] = ss;
        named_bar_sync(1, ncons);
        float tot = 0.f;
        for (int k = 0; k < p.kw; ++k) tot += s_part[k];
        const float rms = 1.0f / sqrtf(tot / (float)rows + p.eps);
#pragma unroll
        for (int v = 0; v < NX / 8; ++v) {
            const int e = e0 + v * 8;
            if (e >= rows) continue;
            unsigned short g[8];
            if (e + 8 <= rows) {
                const uint4 t = *reinterpret_cast<const uint4*>(p.gamma + e);
                g[0] = lo16(t.x); g[1] = hi16(t.x); g[2] = lo16(t.y); g[3] = hi16(t.y);
                g[4] = lo16(t.z); g[5] = hi16(t.z); g[6] = lo16(t.w); g[7] = hi16(t.w);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) g[i] = (e + i < rows) ? __half_as_ushort(p.gamma[e + i]) : (unsigned short)0;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t xv = xr[v * 4 + i];
                const float lo = rms * half_bits_to_float(g[2 * i]) * half_bits_to_float(lo16(xv));
                const float hi = rms * half_bits_to_float(g[2 * i + 1]) * half_bits_to_float(hi16(xv));
                xr[v * 4 + i] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) |
                                ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
            }
        }
    }
}

constexpr int kMaxKW = 32;   // d_in up to 32768 (int4) / 8192 (fp16)
constexpr int kMaxR = 16;    // rows per stage
constexpr int kMaxStages = 8;
constexpr int kRedSlots = 8; // tiles whose k-warp partials may be waiting for the finalizer

// Bounded wait shared by all roles: gives up when another role already flagged an abort, or when its own
// limit runs out (then flags the abort and records where). The kernel always runs to its end.
__device__ __forceinline__ void wait_or_abort(uint64_t* bar, uint32_t parity, volatile unsigned int* abort_flag,
                                              DeviceStatus* status, unsigned int code, int tile)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 1023u) == 1023u && *abort_flag) return;
    }
    *abort_flag = 1;
    if (status) {
        atomicExch(&status->error, code);
        status->detail = (unsigned int)tile;
    }
}

// The same for roles off the critical path (producer, finalizers): the hardware parks the thread between polls,
// so a waiting warp does not take issue slots from the arithmetic warps.
__device__ __forceinline__ void wait_parked_or_abort(uint64_t* bar, uint32_t parity, volatile unsigned int* abort_flag,
                                                     DeviceStatus* status, unsigned int code, int tile)
{
    for (uint32_t i = 0; i < (kSpinLimit >> 6); ++i) {
        if (mbar_try_wait_suspend(bar, parity, 20000u)) return;
        if ((i & 15u) == 15u && *abort_flag) return;
    }
    *abort_flag = 1;
    if (status) {
        atomicExch(&status->error, code);
        status->detail = (unsigned int)tile;
    }
}

// kMaxThreads: the largest block this instantiation is launched with (512 or 1024; the plan's block is
// (k-warps x chunks + 2) warps), so that the register allocation matches the real block size.
template <Fmt F, Epi E, Pro P, int RW, int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads, 1) stream_matvec_kernel(const MatVecParams p)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kMaxStages];    // producer -> consumers: stage landed
    __shared__ __align__(8) uint64_t empty_bar[kMaxStages];   // consumers -> producer: stage may be refilled
    __shared__ __align__(8) uint64_t done_bar[kRedSlots];     // consumers -> finalizer: partials of a tile complete
    __shared__ __align__(8) uint64_t free_bar[kRedSlots];     // finalizer -> consumers: partial slot may be reused
    __shared__ float s_red[kRedSlots][kMaxKW][kMaxR];
    __shared__ float s_part[kMaxKW];
    __shared__ unsigned int s_abort;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncw = p.kw * p.mw;      // consumer warps 0..ncw-1; warp ncw = producer; warp ncw+1 = finalizer
    const int ncons = ncw * 32;
    const int stage_bytes = p.chunk_bytes * p.mw;

    if (tid == 0) {
        for (int s = 0; s < p.nstage; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], ncw);
        }
        for (int s = 0; s < kRedSlots; ++s) {
            mbar_init(&done_bar[s], ncw);
            mbar_init(&free_bar[s], 1);
        }
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    const int my_tiles = (p.ntiles > (int)blockIdx.x) ? (p.ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == ncw) {
        // ---------------- producer warp: weights only, independent of the previous kernel --------
        const uint64_t pol = policy_evict_first();
        for (int i = 0; i < my_tiles; ++i) {
            const int tile = blockIdx.x + i * gridDim.x;
            const int st = i % p.nstage;
            if (i >= p.nstage) {
                if (lane == 0) wait_parked_or_abort(&empty_bar[st], ((i / p.nstage) - 1) & 1, &s_abort, p.status, 1u, tile);
                __syncwarp();
            }
            unsigned char* sbase = smem_raw + (size_t)st * stage_bytes;
            // lane m describes chunk m (one pass, in parallel); runs that are 16-byte aligned go through the
            // bulk-copy engine, anything else (ragged tail, odd strides) through a cooperative copy
            Chunk c{0, 0, 0};
            if (lane < p.mw) c = chunk_of<E, RW>(p, tile, lane);
            const QWPtrs q = p.mat[c.m < p.nmat ? c.m : 0];
            const uint32_t* gw = q.w + (size_t)c.row0 * p.wsize;
            const uint32_t bw = (uint32_t)c.nrows * p.wsize * 4u;
            bool fast = ((reinterpret_cast<uintptr_t>(gw) | bw) & 15u) == 0;
            const uint32_t* gz = nullptr;
            const __half* gs = nullptr;
            uint32_t bz = 0, bs = 0;
            if (F == Fmt::Int4) {
                gz = q.z + (size_t)c.row0 * p.zsize;
                gs = q.s + (size_t)c.row0 * p.ssize;
                bz = (uint32_t)c.nrows * p.zsize * 4u;
                bs = (uint32_t)c.nrows * p.ssize * 2u;
                fast = fast && (((reinterpret_cast<uintptr_t>(gz) | bz) & 15u) == 0) &&
                       (((reinterpret_cast<uintptr_t>(gs) | bs) & 15u) == 0);
            }
            const bool live = c.nrows > 0;
            uint32_t tx = (live && fast) ? (bw + bz + bs) : 0u;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
            const uint32_t slow_mask = __ballot_sync(0xffffffffu, live && !fast);
            if (slow_mask) {
                for (int mwi = 0; mwi < p.mw; ++mwi) {
                    if (!((slow_mask >> mwi) & 1u)) continue;
                    const Chunk cs = chunk_of<E, RW>(p, tile, mwi);
                    const QWPtrs& qs = p.mat[cs.m];
                    unsigned char* cb = sbase + (size_t)mwi * p.chunk_bytes;
                    const uint32_t* sw = qs.w + (size_t)cs.row0 * p.wsize;
                    uint32_t* dw = reinterpret_cast<uint32_t*>(cb);
                    for (int k = lane; k < cs.nrows * p.wsize; k += 32) dw[k] = sw[k];
                    if constexpr (F == Fmt::Int4) {
                        const uint32_t* sz = qs.z + (size_t)cs.row0 * p.zsize;
                        uint32_t* dz = reinterpret_cast<uint32_t*>(cb + p.woff_z);
                        for (int k = lane; k < cs.nrows * p.zsize; k += 32) dz[k] = sz[k];
                        const __half* ss = qs.s + (size_t)cs.row0 * p.ssize;
                        __half* ds = reinterpret_cast<__half*>(cb + p.woff_s);
                        for (int k = lane; k < cs.nrows * p.ssize; k += 32) ds[k] = ss[k];
                    }
                }
                __syncwarp();
            }
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[st], tx);
            __syncwarp();
            if (live && fast) {
                unsigned char* cb = sbase + (size_t)lane * p.chunk_bytes;
                bulk_g2s(cb, gw, bw, &full_bar[st], pol);
                if (F == Fmt::Int4) {
                    bulk_g2s(cb + p.woff_z, gz, bz, &full_bar[st], pol);
                    bulk_g2s(cb + p.woff_s, gs, bs, &full_bar[st], pol);
                }
            }
        }
        return;
    }

    if (warp == ncw + 1) {
        // ---------------- finalizer warp: fixed-order sum over k-warps, then the operator's tail ------
        pdl_wait();  // outputs (and the residual read) belong after the previous kernel
        const int pos = (E == Epi::QKVRope) ? (p.pos_ptr ? *p.pos_ptr : p.pos_imm) : 0;
        for (int i = 0; i < my_tiles; ++i) {
            const int tile = blockIdx.x + i * gridDim.x;
            const int slot = i % kRedSlots;
            const float* red = &s_red[slot][0][0];
            if constexpr (E == Epi::SwiGLU || E == Epi::QKVRope) {
                const int npair = (p.mw >> 1) * RW;
                const int pr = lane / RW, r = lane - pr * RW;
                const bool mine = lane < npair;
                Chunk ca{0, 0, 0}, cbk{0, 0, 0};
                if (mine) {
                    ca = chunk_of<E, RW>(p, tile, 2 * pr);
                    cbk = chunk_of<E, RW>(p, tile, 2 * pr + 1);
                }
                float2 cs = make_float2(1.f, 0.f);
                if (E == Epi::QKVRope && mine && r < ca.nrows && ca.m < 2)
                    cs = p.rope_table[(size_t)pos * (p.head_size >> 1) + (ca.row0 + r) % p.head_size];
                wait_parked_or_abort(&done_bar[slot], (i / kRedSlots) & 1, &s_abort, p.status, 3u, tile);
                if (mine && r < ca.nrows) {
                    float sa = 0.f, sb = 0.f;
                    for (int k = 0; k < p.kw; ++k) {
                        sa += red[k * kMaxR + (2 * pr) * RW + r];
                        sb += red[k * kMaxR + (2 * pr + 1) * RW + r];
                    }
                    if constexpr (E == Epi::SwiGLU) {
                        // native/mat_vec_kernel.cu:218-222
                        float val = sa;
                        val *= 1.0f / (1.0f + expf(-val));
                        val *= sb;
                        p.out[0][ca.row0 + r] = __float2half_rn(val);
                    } else {
                        __half* o = p.out[ca.m];
                        if (ca.m > 0 && p.pos_ptr) o += (long long)pos * p.kv_row_stride;
                        if (ca.m < 2) {
                            // fp16 store of the mat-vec result (native/mat_vec_kernel.cu:175), then RoPE on the
                            // rounded values (native/rope_kernel.cu:15-25)
                            const float a0 = __half2float(__float2half_rn(sa));
                            const float b0 = __half2float(__float2half_rn(sb));
                            o[ca.row0 + r] = __float2half_rn(a0 * cs.x - b0 * cs.y);
                            o[cbk.row0 + r] = __float2half_rn(a0 * cs.y + b0 * cs.x);
                        } else {
                            o[ca.row0 + r] = __float2half_rn(sa);
                            o[cbk.row0 + r] = __float2half_rn(sb);
                        }
                    }
                }
            } else {
                const int nrow = p.mw * RW;
                const int ch = lane / RW, r = lane - ch * RW;
                Chunk c{0, 0, 0};
                if (lane < nrow) c = chunk_of<E, RW>(p, tile, ch);
                const bool mine = lane < nrow && r < c.nrows;
                const int row = c.row0 + r;
                float resid = 0.f;
                if (E == Epi::Residual && mine) resid = __half2float(p.out[0][row]);  // issued before the wait
                wait_parked_or_abort(&done_bar[slot], (i / kRedSlots) & 1, &s_abort, p.status, 3u, tile);
                if (mine) {
                    float sum = 0.f;
                    for (int k = 0; k < p.kw; ++k) sum += red[k * kMaxR + lane];
                    if constexpr (E == Epi::Store) {
                        p.out[c.m][row] = __float2half_rn(sum);
                    } else if constexpr (E == Epi::Residual) {
                        p.out[0][row] = __float2half_rn(sum + resid);  // native/mat_vec_kernel.cu:154-156
                    } else {
                        p.out_f32[row] = sum;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&free_bar[slot]);
        }
        return;
    }
    if (warp > ncw + 1) return;

    // ---------------- consumer warps ------------------------------------------------------------
    const int kw_id = warp % p.kw;
    const int mw_id = warp / p.kw;
    const int u = kw_id * 32 + lane;          // this lane's 16-byte vector inside every row
    const bool active = u < p.units;
    constexpr int NX = (F == Fmt::Int4) ? 32 : 8;  // inputs per lane
    const int e0 = u * NX;

    pdl_wait();  // the previous kernel's output (our input vector) is complete and visible from here on

    uint32_t xr[NX / 2];
    load_input<P, NX>(p, active ? e0 : p.rows, mw_id == 0, kw_id, ncons, s_part, xr);

    XSlice xs;
    if constexpr (F == Fmt::Int4) {
        make_xslice(xr, xs);
    } else {
#pragma unroll
        for (int i = 0; i < NX / 2; ++i) xs.xp[i] = xr[i];
    }
    const int g = u >> 2;             // quantisation group of this lane's slice (Int4)
    const int zshift = (g & 7) * 4;
    // lane-invariant offsets inside a chunk
    const uint32_t chunk_base = smem_u32(smem_raw) + (uint32_t)mw_id * p.chunk_bytes;
    const uint32_t w_off = (uint32_t)(active ? u : 0) * 16u;
    const uint32_t z_off = p.woff_z + (uint32_t)(active ? (g >> 3) : 0) * 4u;
    const uint32_t s_off = p.woff_s + (uint32_t)(active ? g : 0) * 2u;
    const uint32_t w_row = (uint32_t)p.wsize * 4u, z_row = (uint32_t)p.zsize * 4u, s_row = (uint32_t)p.ssize * 2u;
    const bool writer = (lane & (32 / RW - 1)) == 0;
    float* red_dst = &s_red[0][kw_id][mw_id * RW + lane / (32 / RW)];  // + slot * kMaxKW * kMaxR

    for (int i = 0; i < my_tiles; ++i) {
        const int st = i % p.nstage;
        wait_or_abort(&full_bar[st], (i / p.nstage) & 1, &s_abort, p.status, 2u, i);
        const uint32_t cb = chunk_base + (uint32_t)st * stage_bytes;
        float v[RW];
        if constexpr (F == Fmt::Int4) {
            uint4 wv[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r)
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(wv[r].x), "=r"(wv[r].y), "=r"(wv[r].z), "=r"(wv[r].w)
                             : "r"(cb + w_off + r * w_row));
            uint32_t zw[RW];
            unsigned short sc[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(zw[r]) : "r"(cb + z_off + r * z_row));
                asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sc[r]) : "r"(cb + s_off + r * s_row));
            }
            float A[RW], B[RW], D[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                A[r] = xs.a0;
                B[r] = xs.b0;
                D[r] = 0.f;
                word_dot(wv[r].x, xs.xp + 0, A[r], B[r], D[r]);
                word_dot(wv[r].y, xs.xp + 4, A[r], B[r], D[r]);
                word_dot(wv[r].z, xs.xp + 8, A[r], B[r], D[r]);
                word_dot(wv[r].w, xs.xp + 12, A[r], B[r], D[r]);
            }
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const float zf = (float)((zw[r] >> zshift) & 0xFu);
                const float t = fmaf(B[r], 0.0625f, A[r]) + D[r];
                const float res = half_bits_to_float(sc[r]) * fmaf(-zf, xs.c1, t);
                v[r] = active ? res : 0.f;
            }
        } else {
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                uint4 wv;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w)
                             : "r"(cb + w_off + r * w_row));
                float a0 = 0.f, a1 = 0.f;
                a0 = fma_f16_f32(lo16(wv.x), lo16(xs.xp[0]), a0);
                a1 = fma_f16_f32(hi16(wv.x), hi16(xs.xp[0]), a1);
                a0 = fma_f16_f32(lo16(wv.y), lo16(xs.xp[1]), a0);
                a1 = fma_f16_f32(hi16(wv.y), hi16(xs.xp[1]), a1);
                a0 = fma_f16_f32(lo16(wv.z), lo16(xs.xp[2]), a0);
                a1 = fma_f16_f32(hi16(wv.z), hi16(xs.xp[2]), a1);
                a0 = fma_f16_f32(lo16(wv.w), lo16(xs.xp[3]), a0);
                a1 = fma_f16_f32(hi16(wv.w), hi16(xs.xp[3]), a1);
                v[r] = active ? (a0 + a1) : 0.f;
            }
        }
        // this warp is done with the stage: hand it back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[st]);

        // deposit the row sums of this warp's k-slice for the finalizer
        transpose_reduce<RW>(v, lane);
        const int slot = i % kRedSlots;
        if (i >= kRedSlots) wait_or_abort(&free_bar[slot], ((i / kRedSlots) - 1) & 1, &s_abort, p.status, 4u, i);
        if (writer) red_dst[slot * (kMaxKW * kMaxR)] = v[0];
        __syncwarp();
        if (lane == 0) mbar_arrive(&done_bar[slot]);
    }
}

}  // namespace ml2
