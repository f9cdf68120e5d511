/*
 * CPU oracle for the ManagedLlama2 decode hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the CPU-side definition of the
 * reference's int4 (AWQ, group 128) mat-vec family and of the small operators around it.
 * It is the checker the CUDA kernels are compared with; it is also the timed "CPU baseline"
 * of the benchmark. Nothing in the product library links, loads or calls it.
 *
 * Every function cites the reference file (path inside GilesBathgate/ManagedLlama2) and the
 * lines it follows. C# `Half` <-> `float` conversions are IEEE round-to-nearest-even, which is
 * what `_Float16` gives with GCC on x86-64; C# `MathF.*` maps onto the C library's
 * `expf/sqrtf/powf/sinf/cosf`.
 *
 * Parity pin: `orc_unpack_flat` reproduces the literal golden vector of the reference's
 * test/QWeightTestData.cs bit for bit (tests/test_oracle_golden.py).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef _Float16 f16;

#define ORC_API __attribute__((visibility("default")))

static inline int ceil_div(int a, int b) { return (a + (b - 1)) / b; }

/* The C# reference loops are single-threaded. The mat-vec loops over outputs can be spread over
 * host threads (each output is still one sequential fp32 sum, so results do not change); the
 * benchmark's CPU baseline uses this with every host core. 1 thread by default. */
static int g_threads = 1;
ORC_API void orc_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
ORC_API int orc_get_threads(void) { return g_threads; }

typedef void (*range_fn)(void* ctx, int begin, int end);
typedef struct { range_fn fn; void* ctx; int begin, end; } range_job;
static void* range_thread(void* p) { range_job* j = (range_job*)p; j->fn(j->ctx, j->begin, j->end); return NULL; }

static void parallel_for(int n, range_fn fn, void* ctx)
{
    int t = g_threads;
    if (t > n) t = n;
    if (t <= 1) { fn(ctx, 0, n); return; }
    pthread_t tid[256];
    range_job job[256];
    const int per = ceil_div(n, t);
    int started = 0;
    for (int i = 0; i < t; ++i) {
        int b = i * per, e = b + per > n ? n : b + per;
        if (b >= e) break;
        job[i] = (range_job){ fn, ctx, b, e };
        if (pthread_create(&tid[i], NULL, range_thread, &job[i]) != 0) { fn(ctx, b, e); tid[i] = 0; }
        started = i + 1;
    }
    for (int i = 0; i < started; ++i) if (tid[i]) pthread_join(tid[i], NULL);
}

/* ------------------------------------------------------------------------------------------
 * QWeight layout
 * ---------------------------------------------------------------------------------------- */

/* HostQWeight.Unpack, src/QWeight.cs:29-54, applied to ONE flat stream of `n_words` packed
 * words (8 nibbles each, least-significant nibble first). For x-th run of 4 words:
 * zIndex = x/32, sIndex = x/4, zero = (Zeros[zIndex] >> (sIndex*4)) & 0xF. C# masks a 32-bit
 * shift count to 5 bits, hence `(sIndex & 7) * 4` here. value = (element - zero) * (float)scale
 * with an int subtraction and an fp32 multiply, then rounded to fp16 (`ToHalf`, :53). */
ORC_API void orc_unpack_flat(const uint32_t* weight, const uint32_t* zeros, const f16* scales,
                             int n_words, f16* out)
{
    const int x_size = n_words / 4;
    for (int x = 0; x < x_size; ++x) {
        const int z_index = x / 32;
        const int s_index = x / 4;
        const int w_index = x * 4;
        const int zero = (int)((zeros[z_index] >> ((s_index & 7) * 4)) & 0xFu);
        const float scale = (float)scales[s_index];
        for (int w = 0; w < 4; ++w) {
            const uint32_t word = weight[w_index + w];
            const int o_index = w_index * 8 + w * 8;
            for (int i = 0; i < 8; ++i) {
                const int element = (int)((word >> (i * 4)) & 0xFu);
                const float v = (float)(element - zero) * scale;
                out[o_index + i] = (f16)v;
            }
        }
    }
}

/* HostQWeight.Pack, src/QWeight.cs:56-92. `data` holds n_scales*128 values; zeros are given one
 * per group (unpacked), scales as fp32. Quantisation truncates: (uint)(value/scale + zero) & 0xF
 * (:82-83); the scale is stored as fp16 (:88). */
ORC_API void orc_pack_flat(const f16* data, const float* scales, const uint32_t* zeros_unpacked,
                           int n_scales, uint32_t* weight, uint32_t* zeros, f16* scales_out)
{
    for (int i = 0; i < n_scales / 8; ++i) {
        uint32_t combined = 0;
        for (int z = 0; z < 8; ++z) combined |= (zeros_unpacked[i * 8 + z] & 0xFu) << (z * 4);
        zeros[i] = combined;
    }
    const int s_size = n_scales * 4;
    for (int s = 0; s < s_size; ++s) {
        const int s_index = s / 4;
        const int w_index = s * 4;
        const float scale = scales[s_index];
        const uint32_t zero = zeros_unpacked[s_index];
        for (int w = 0; w < 4; ++w) {
            uint32_t word = 0;
            const int o_index = w_index * 8 + w * 8;
            for (int i = 0; i < 8; ++i) {
                /* C#: (uint)(((float)data[..] / scale) + zero): the uint is widened to float for
                 * the addition and the sum is truncated towards zero. */
                const float q = ((float)data[o_index + i] / scale) + (float)zero;
                const uint32_t element = (uint32_t)(int64_t)q;
                word |= (element & 0xFu) << (i * 4);
            }
            weight[w_index + w] = word;
        }
        scales_out[s_index] = (f16)scale;
    }
}

/* Device layout of one matrix (src/TransformerWeights.cs:54-69, native/mat_vec_kernel.cu:98-116):
 * every output ("col") owns weightsSize = ceil(rows/32)*4 words, zerosSize = ceil(scalesSize/8)
 * words and scalesSize = ceil(rows/128) scales. Unpack is applied per output so that shapes whose
 * d_in is not a multiple of 1024 (padded zero words) are handled like the kernel handles them.
 * out is [cols][rows]. */
ORC_API void orc_unpack_rows(const uint32_t* weight, const uint32_t* zeros, const f16* scales,
                             int rows, int cols, f16* out)
{
    const int s_size = ceil_div(rows, 128);
    const int w_size = ceil_div(rows, 32) * 4;
    const int z_size = ceil_div(s_size, 8);
    for (int c = 0; c < cols; ++c) {
        const uint32_t* w = weight + (size_t)c * w_size;
        const uint32_t* z = zeros + (size_t)c * z_size;
        const f16* s = scales + (size_t)c * s_size;
        f16* o = out + (size_t)c * rows;
        for (int k = 0; k < rows; ++k) {
            const int g = k / 128;
            const int zero = (int)((z[g / 8] >> ((g & 7) * 4)) & 0xFu);
            const int element = (int)((w[k / 8] >> ((k & 7) * 4)) & 0xFu);
            o[k] = (f16)((float)(element - zero) * (float)s[g]);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * int4 mat-vec family: the C# test-local CPU references
 * ---------------------------------------------------------------------------------------- */

/* Sequential fp32 dot of one dequantised (fp16) weight row with x:
 * test/MatVecInt4Tests.cs:53-61 (identical loops at test/QKVMatVecInt4Tests.cs:64-87 and
 * test/SwiGLUMatVecInt4Tests.cs:55-70). */
static float dot_unpacked_row(const uint32_t* w, const uint32_t* z, const f16* s, const f16* x, int rows)
{
    float val = 0.0f;
    for (int k = 0; k < rows; ++k) {
        const int g = k / 128;
        const int zero = (int)((z[g / 8] >> ((g & 7) * 4)) & 0xFu);
        const int element = (int)((w[k / 8] >> ((k & 7) * 4)) & 0xFu);
        const f16 wk = (f16)((float)(element - zero) * (float)s[g]); /* Unpack rounds to Half */
        val += (float)wk * (float)x[k];
    }
    return val;
}

/* Arithmetic of the reference CUDA kernel for one output (native/mat_vec_kernel.cu:130-134):
 * sum += (float)x * (element - zero) * scale in fp32 with no intermediate fp16 rounding of the
 * weight; accumulated here in double so the result is order-independent ("exact" arbiter). */
static double dot_exact_row(const uint32_t* w, const uint32_t* z, const f16* s, const f16* x, int rows)
{
    double val = 0.0;
    for (int k = 0; k < rows; ++k) {
        const int g = k / 128;
        const int zero = (int)((z[g / 8] >> ((g & 7) * 4)) & 0xFu);
        const int element = (int)((w[k / 8] >> ((k & 7) * 4)) & 0xFu);
        val += (double)(float)x[k] * (double)(element - zero) * (double)(float)s[g];
    }
    return val;
}

typedef struct {
    const uint32_t* w;
    const uint32_t* z;
    const f16* s;
} orc_qweight;

static inline void row_ptrs(const orc_qweight* q, int rows, int c, const uint32_t** w, const uint32_t** z, const f16** s)
{
    const int s_size = ceil_div(rows, 128);
    const int w_size = ceil_div(rows, 32) * 4;
    const int z_size = ceil_div(s_size, 8);
    *w = q->w + (size_t)c * w_size;
    *z = q->z + (size_t)c * z_size;
    *s = q->s + (size_t)c * s_size;
}

/* Plain int4 mat-vec, fp32 result before the fp16 store. mode 0: C# reference (fp16-rounded
 * weights, sequential fp32 sum); mode 1: kernel arithmetic accumulated in double. */
typedef struct { float* out; const f16* x; orc_qweight q; int rows, mode; } mv4_ctx;
static void mv4_range(void* p, int b, int e)
{
    const mv4_ctx* a = (const mv4_ctx*)p;
    for (int c = b; c < e; ++c) {
        const uint32_t *rw, *rz;
        const f16* rs;
        row_ptrs(&a->q, a->rows, c, &rw, &rz, &rs);
        a->out[c] = a->mode == 0 ? dot_unpacked_row(rw, rz, rs, a->x, a->rows)
                                 : (float)dot_exact_row(rw, rz, rs, a->x, a->rows);
    }
}
ORC_API void orc_matvec_int4_f32(float* out, const f16* x, const uint32_t* w, const uint32_t* z, const f16* s,
                                 int rows, int cols, int mode)
{
    mv4_ctx a = { out, x, { w, z, s }, rows, mode };
    parallel_for(cols, mv4_range, &a);
}

/* MatVecInt4Tests.Expected, test/MatVecInt4Tests.cs:48-70: xout = (Half)((float)x_res + W.x).
 * `inout` is the residual stream (read, then overwritten); `in` is the multiplied vector. */
ORC_API void orc_matvec_residual_int4(f16* inout, const f16* in, const uint32_t* w, const uint32_t* z, const f16* s,
                                      int rows, int cols, int mode)
{
    float* tmp = (float*)malloc(sizeof(float) * (size_t)cols);
    orc_matvec_int4_f32(tmp, in, w, z, s, rows, cols, mode);
    for (int c = 0; c < cols; ++c) inout[c] = (f16)((float)inout[c] + tmp[c]);
    free(tmp);
}

/* QKVMatVecInt4Tests.Expected, test/QKVMatVecInt4Tests.cs:64-87: three independent mat-vecs, each
 * rounded to fp16. */
ORC_API void orc_qkv_matvec_int4(f16* q_out, f16* k_out, f16* v_out, const f16* in,
                                 const uint32_t* qw, const uint32_t* qz, const f16* qs,
                                 const uint32_t* kw, const uint32_t* kz, const f16* ks,
                                 const uint32_t* vw, const uint32_t* vz, const f16* vs,
                                 int rows, int cols, int mode)
{
    float* tmp = (float*)malloc(sizeof(float) * (size_t)cols);
    f16* outs[3] = { q_out, k_out, v_out };
    const uint32_t* ws[3] = { qw, kw, vw };
    const uint32_t* zs[3] = { qz, kz, vz };
    const f16* ss[3] = { qs, ks, vs };
    for (int m = 0; m < 3; ++m) {
        orc_matvec_int4_f32(tmp, in, ws[m], zs[m], ss[m], rows, cols, mode);
        for (int c = 0; c < cols; ++c) outs[m][c] = (f16)tmp[c];
    }
    free(tmp);
}

/* SwiGLUMatVecInt4Tests.Expected, test/SwiGLUMatVecInt4Tests.cs:72-92 (kernel:
 * native/mat_vec_kernel.cu:218-222): val = g; val *= 1/(1+expf(-val)); val *= u; fp16 store. */
ORC_API void orc_matvec_swiglu_int4(f16* out, const f16* in,
                                    const uint32_t* gw, const uint32_t* gz, const f16* gs,
                                    const uint32_t* uw, const uint32_t* uz, const f16* us,
                                    int rows, int cols, int mode)
{
    float* g = (float*)malloc(sizeof(float) * (size_t)cols);
    float* u = (float*)malloc(sizeof(float) * (size_t)cols);
    orc_matvec_int4_f32(g, in, gw, gz, gs, rows, cols, mode);
    orc_matvec_int4_f32(u, in, uw, uz, us, rows, cols, mode);
    for (int c = 0; c < cols; ++c) {
        float val = g[c];
        val *= 1.0f / (1.0f + expf(-val));
        val *= u[c];
        out[c] = (f16)val;
    }
    free(g);
    free(u);
}

/* ------------------------------------------------------------------------------------------
 * fp16 mat-vec, attention products, softmax, RMSNorm, RoPE, embedding, argmax
 * ---------------------------------------------------------------------------------------- */

/* MatVecTests.Expected, test/MatVecTests.cs:41-56: out[i] = (Half) sum_j (float)w[i*n+j]*(float)x[j];
 * n = rows (d_in), d = cols (d_out). */
typedef struct { f16* out; const f16* x; const f16* w; int rows; } mvf_ctx;
static void mvf_range(void* p, int b, int e)
{
    const mvf_ctx* a = (const mvf_ctx*)p;
    for (int i = b; i < e; ++i) {
        float val = 0.0f;
        const f16* wr = a->w + (size_t)i * a->rows;
        for (int j = 0; j < a->rows; ++j) val += (float)wr[j] * (float)a->x[j];
        a->out[i] = (f16)val;
    }
}
ORC_API void orc_matvec_f16(f16* out, const f16* x, const f16* w, int rows, int cols)
{
    mvf_ctx a = { out, x, w, rows };
    parallel_for(cols, mvf_range, &a);
}

/* MatVecStridedTests.Expected, test/MatVecStridedTests.cs:43-72: att[h*seq + t] =
 * (Half)(scale * sum_i q[h*hs+i] * k[t*kv_dim + (h/kv_mul)*hs + i]); scale = 1/sqrtf(hs).
 * `k` points at the layer's first cache row; row stride is kv_dim. */
ORC_API void orc_attn_scores(f16* att, const f16* q, const f16* k, int dim, int n_heads, int n_kv_heads, int seq_len)
{
    const int head_size = dim / n_heads;
    const float scale = 1.0f / sqrtf((float)head_size);
    const int kv_dim = dim * n_kv_heads / n_heads;
    const int kv_mul = n_heads / n_kv_heads;
    for (int h = 0; h < n_heads; ++h) {
        for (int t = 0; t < seq_len; ++t) {
            const f16* kr = k + (size_t)t * kv_dim + (size_t)(h / kv_mul) * head_size;
            float score = 0.0f;
            for (int i = 0; i < head_size; ++i) score += (float)q[h * head_size + i] * (float)kr[i];
            score *= scale;
            att[(size_t)h * seq_len + t] = (f16)score;
        }
    }
}

/* SoftmaxTests.Expected, test/SoftmaxTests.cs:31-59, once per head (the kernel runs one block per
 * head over att[h*size .. h*size+size), native/softmax_kernel.cu:15-16). */
ORC_API void orc_softmax(f16* att, int n_heads, int size)
{
    float* x = (float*)malloc(sizeof(float) * (size_t)size);
    for (int h = 0; h < n_heads; ++h) {
        f16* a = att + (size_t)h * size;
        for (int i = 0; i < size; ++i) x[i] = (float)a[i];
        float max_val = x[0];
        for (int i = 1; i < size; ++i)
            if (x[i] > max_val) max_val = x[i];
        float sum = 0.0f;
        for (int i = 0; i < size; ++i) {
            x[i] = expf(x[i] - max_val);
            sum += x[i];
        }
        for (int i = 0; i < size; ++i) a[i] = (f16)(x[i] / sum);
    }
    free(x);
}

/* VecMatTests.Expected, test/VecMatTests.cs:44-73: xb[h*hs+i] = (Half) sum_t att[h*seq+t] *
 * v[t*kv_dim + (h/kv_mul)*hs + i], accumulated over t in fp32. */
ORC_API void orc_attn_values(f16* out, const f16* att, const f16* v, int dim, int n_heads, int n_kv_heads, int seq_len)
{
    const int head_size = dim / n_heads;
    const int kv_dim = dim * n_kv_heads / n_heads;
    const int kv_mul = n_heads / n_kv_heads;
    float* xb = (float*)calloc((size_t)dim, sizeof(float));
    for (int h = 0; h < n_heads; ++h) {
        for (int t = 0; t < seq_len; ++t) {
            const f16* vr = v + (size_t)t * kv_dim + (size_t)(h / kv_mul) * head_size;
            const float a = (float)att[(size_t)h * seq_len + t];
            for (int i = 0; i < head_size; ++i) xb[h * head_size + i] += a * (float)vr[i];
        }
    }
    for (int i = 0; i < dim; ++i) out[i] = (f16)xb[i];
    free(xb);
}

/* RMSNorm. The reference kernel (native/rmsnorm_kernel.cu:12-35) squares in fp32 and forms
 * rms * gamma * x left to right; the C# test reference (test/RMSNormTests.cs:34-51) squares in
 * fp16 (`input[i] * input[i]` on Half) and forms gamma * (ss * x). fp16_square selects the
 * test's variant; the model oracle uses the kernel's. out may alias in. */
ORC_API void orc_rmsnorm(f16* out, const f16* in, const f16* gamma, int size, float eps, int fp16_square)
{
    float ss = 0.0f;
    for (int i = 0; i < size; ++i) {
        if (fp16_square) {
            const f16 sq = (f16)((float)in[i] * (float)in[i]);
            ss += (float)sq;
        } else {
            const float v = (float)in[i];
            ss += v * v;
        }
    }
    ss /= (float)size;
    ss += eps;
    ss = 1.0f / sqrtf(ss);
    for (int i = 0; i < size; ++i) {
        const float r = fp16_square ? (float)gamma[i] * (ss * (float)in[i]) : ss * (float)gamma[i] * (float)in[i];
        out[i] = (f16)r;
    }
}

/* RoPETests.Expected, test/RoPETests.cs:42-83 (kernel: native/rope_kernel.cu:6-25): rotate-half
 * pairs (i, i + hs/2) inside each head; freq = 1/powf(theta, ((i*2) % hs)/hs); angle = pos*freq;
 * q always, k (the cache row of this position) for heads below n_kv_heads. */
ORC_API void orc_rope(f16* q, f16* k_row, int dim, int n_heads, int n_kv_heads, int pos, float theta)
{
    const int head_size = dim / n_heads;
    const int kv_dim = dim * n_kv_heads / n_heads;
    const int half = head_size / 2;
    for (int h = 0; h < n_heads; ++h) {
        for (int t = 0; t < half; ++t) {
            const int i = h * head_size + t;
            const int j = half + i;
            const int head_dim = (i * 2) % head_size;
            const float freq = 1.0f / powf(theta, (float)head_dim / (float)head_size);
            const float val = (float)pos * freq;
            const float fci = sinf(val);
            const float fcr = cosf(val);
            {
                const float v0 = (float)q[i], v1 = (float)q[j];
                q[i] = (f16)(v0 * fcr - v1 * fci);
                q[j] = (f16)(v0 * fci + v1 * fcr);
            }
            if (i < kv_dim) {
                const float v0 = (float)k_row[i], v1 = (float)k_row[j];
                k_row[i] = (f16)(v0 * fcr - v1 * fci);
                k_row[j] = (f16)(v0 * fci + v1 * fcr);
            }
        }
    }
}

/* native/embedding_kernel.cu:6-12: out = table[token]. */
ORC_API void orc_embedding(f16* out, const f16* table, int size, int token)
{
    memcpy(out, table + (size_t)token * size, sizeof(f16) * (size_t)size);
}

/* ArgmaxTests.Expected, test/ArgmaxTests.cs:33-46: first index of the maximum (strict >). */
ORC_API int orc_argmax(const f16* logits, int n)
{
    int max_i = 0;
    f16 max_p = logits[0];
    for (int i = 1; i < n; ++i) {
        if (logits[i] > max_p) {
            max_i = i;
            max_p = logits[i];
        }
    }
    return max_i;
}

/* ------------------------------------------------------------------------------------------
 * One token through the model: Transformer.Forward, src/Transformer.cs:158-190, composed from the
 * pieces above with an fp16 store wherever the reference kernels store fp16.
 * ---------------------------------------------------------------------------------------- */

typedef struct {
    int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_theta;
} orc_config; /* same field order as src/Config.cs:6-17 */

typedef struct {
    orc_qweight q, k, v, o, gate, up, down;
    const f16* rms_att;
    const f16* rms_ffn;
} orc_layer; /* src/PerLayerWeight.cs:5-16 */

typedef struct {
    orc_config cfg;
    const f16* embed;      /* [vocab][dim] */
    const f16* classifier; /* [vocab][dim] */
    const f16* rms_final;  /* [dim] */
    const orc_layer* layers;
    /* run state, src/RunState.cs:5-25 */
    f16 *x, *xb, *h, *q, *att, *logits;
    f16 *key_cache, *value_cache; /* [layer][seq_len][kv_dim] */
    float eps;
    int mode; /* 0 = C# fp16-weight reference arithmetic, 1 = kernel arithmetic (double sum) */
} orc_model;

ORC_API void orc_forward(orc_model* m, int token, int pos)
{
    const orc_config* c = &m->cfg;
    const int dim = c->dim, hid = c->hidden_dim;
    const int kv_dim = dim * c->n_kv_heads / c->n_heads;
    const int seq = pos + 1;

    orc_embedding(m->x, m->embed, dim, token); /* :163 */
    for (int l = 0; l < c->n_layers; ++l) {
        const orc_layer* L = &m->layers[l];
        orc_rmsnorm(m->xb, m->x, L->rms_att, dim, m->eps, 0); /* :167 */
        const size_t layer_off = (size_t)l * c->seq_len * kv_dim; /* :169 */
        f16* k_row = m->key_cache + layer_off + (size_t)pos * kv_dim;
        f16* v_row = m->value_cache + layer_off + (size_t)pos * kv_dim;
        orc_qkv_matvec_int4(m->q, k_row, v_row, m->xb, L->q.w, L->q.z, L->q.s, L->k.w, L->k.z, L->k.s,
                            L->v.w, L->v.z, L->v.s, dim, dim, m->mode); /* :171 */
        orc_rope(m->q, k_row, dim, c->n_heads, c->n_kv_heads, pos, c->rope_theta); /* :173 */
        /* MultiHeadAttention, :150-156 */
        orc_attn_scores(m->att, m->q, m->key_cache + layer_off, dim, c->n_heads, c->n_kv_heads, seq);
        orc_softmax(m->att, c->n_heads, seq);
        orc_attn_values(m->xb, m->att, m->value_cache + layer_off, dim, c->n_heads, c->n_kv_heads, seq);
        orc_matvec_residual_int4(m->x, m->xb, L->o.w, L->o.z, L->o.s, dim, dim, m->mode); /* :177 */
        orc_rmsnorm(m->xb, m->x, L->rms_ffn, dim, m->eps, 0); /* :179 */
        orc_matvec_swiglu_int4(m->h, m->xb, L->gate.w, L->gate.z, L->gate.s, L->up.w, L->up.z, L->up.s,
                               dim, hid, m->mode); /* :181 */
        orc_matvec_residual_int4(m->x, m->h, L->down.w, L->down.z, L->down.s, hid, dim, m->mode); /* :183 */
    }
    orc_rmsnorm(m->x, m->x, m->rms_final, dim, m->eps, 0); /* :187 */
    orc_matvec_f16(m->logits, m->x, m->classifier, dim, c->vocab_size); /* :189 */
}
