/*
 * ml2b200 - C ABI of the B200 (sm_100a) decode hot path for ManagedLlama2.
 *
 * Two levels, both plain C (pointers and sizes only):
 *
 *  1. Operator level: one entry point per `Module.Forward` of the reference's C# operator classes
 *     (the src/ directory of GilesBathgate/ManagedLlama2). Arguments keep the reference's meaning: raw device
 *     pointers, `rows` = d_in, `cols` = d_out, offsets into the KV cache already applied by the
 *     caller (as `OffsetPointer` does, src/Extensions.cs:20-21). Launch geometry and the derived
 *     sizes (`scalesSize`, `weightsSize`, `zerosSize`, src/QKVMatVec.cs:22-24) are computed inside.
 *     Each C# subclass body becomes a single P/Invoke.
 *
 *  2. Model level: the per-token operator sequence of `Transformer.Forward`
 *     (src/Transformer.cs:158-190) as ONE persistent kernel launch per token (one CTA per SM; the
 *     operators hand over through device-wide counters, weights stream through a shared-memory ring
 *     across operator boundaries), with optional tensor parallelism: one process per GPU, the sum of
 *     the row-sharded mat-vecs fused into that kernel over peer memory. A CUDA graph of five fused
 *     kernels per layer (with NCCL all-reduces under tensor parallelism) is the alternative path.
 *
 * Every function returns 0 on success or a negative ML2_E_* code; `ml2_last_error()` gives the text
 * for the calling thread. Nothing throws, nothing traps the device, no call falls back to the CPU.
 * Buffers are owned by the caller unless stated; kernels only borrow them for the launch.
 * All launches go to the context's stream (default: the legacy NULL stream, as the reference's
 * `Module` uses, src/Module.cs:13).
 */
#ifndef ML2B200_H
#define ML2B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with -fvisibility=hidden */
#endif

#define ML2_OK 0
#define ML2_E_INVALID (-1)   /* bad size, null or misaligned pointer, unsupported shape */
#define ML2_E_CUDA (-2)      /* a CUDA runtime call failed; text in ml2_last_error() */
#define ML2_E_STATE (-3)     /* call made in the wrong state (e.g. forward before bind) */
#define ML2_E_DEVICE (-4)    /* a kernel's bounded wait ran out; status word in ml2_ctx_status() */
#define ML2_E_NCCL (-5)      /* an NCCL call failed */

typedef struct ml2_ctx ml2_ctx;
typedef struct ml2_model ml2_model;

/* Same eight fields, order and 32-byte layout as `Config` (src/Config.cs:6-17). */
typedef struct ml2_config {
    int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_theta;
} ml2_config;

/* The three device arrays of a `QWeight` (src/QWeight.cs:5-10). */
typedef struct ml2_qweight {
    const uint32_t* weight; /* [cols][ceil(rows/32)*4]  8 nibbles per word, LSB first */
    const uint32_t* zeros;  /* [cols][ceil(ceil(rows/128)/8)] 8 zero points per word */
    const void* scales;     /* fp16 [cols][ceil(rows/128)] */
} ml2_qweight;

const char* ml2_last_error(void);
int ml2_version(void);

/* ---- context ---------------------------------------------------------------------------- */
/* Replaces `new CudaContext(deviceID)` + per-Module PTX loading (src/Transformer.cs:48-49,
 * src/Module.cs:15-19): binds the calling thread's primary context of `device`. */
int ml2_ctx_create(int device, ml2_ctx** out);
int ml2_ctx_destroy(ml2_ctx* ctx);
int ml2_ctx_set_stream(ml2_ctx* ctx, void* cuda_stream);
/* Programmatic dependent launch between consecutive operator calls (default off at this level:
 * the reference's semantics are plain stream order). */
int ml2_ctx_set_pdl(ml2_ctx* ctx, int enabled);
int ml2_ctx_synchronize(ml2_ctx* ctx);
/* Budget of every device-side wait (mbarrier phases, operator counters, peer counters), in SM clock
 * cycles; default 2e10 (about ten seconds). A wait that runs out writes the error word and the kernel
 * runs to its end; the next synchronising call returns ML2_E_DEVICE. No counterpart in the reference
 * (its kernels never wait on one another). */
int ml2_ctx_set_wait_limit(ml2_ctx* ctx, long long sm_cycles);
/* Reads and clears the device error word written when a kernel's bounded wait expired. */
int ml2_ctx_status(ml2_ctx* ctx, unsigned* error, unsigned* detail);
/* Number of kernels this library has launched through `ctx` so far. */
long long ml2_ctx_launch_count(ml2_ctx* ctx);

/* ---- operator level: int4 (AWQ, group 128) mat-vec family --------------------------------- */
/* MatVecResidual.Forward (src/MatVecResidual.cs:15-23; mat_vec_residual_int4_kernel,
 * native/mat_vec_kernel.cu:144-164): inout[c] = half(float(inout[c]) + sum_r W[c][r]*in[r]).
 * `in` must not alias `inout`. */
int ml2_matvec_residual_int4(ml2_ctx* ctx, void* inout, const void* in, const ml2_qweight* w, int rows, int cols);
/* QKVMatVec.Forward (src/QKVMatVec.cs:19-30; qkv_mat_vec_kernel, native/mat_vec_kernel.cu:179-203).
 * q_out/k_out/v_out are the final destinations (cache row offset already applied). */
int ml2_qkv_matvec_int4(ml2_ctx* ctx, void* q_out, void* k_out, void* v_out, const void* in, const ml2_qweight* q,
                        const ml2_qweight* k, const ml2_qweight* v, int rows, int cols);
/* MatVecSwiGLU.Forward (src/MatVecSwiGLU.cs:15-23; mat_vec_swiglu_kernel,
 * native/mat_vec_kernel.cu:206-234): out[c] = half(silu(Wg.in)[c] * (Wu.in)[c]). */
int ml2_matvec_swiglu_int4(ml2_ctx* ctx, void* out, const void* in, const ml2_qweight* gate, const ml2_qweight* up,
                           int rows, int cols);
/* Plain int4 mat-vec with fp16 store (device function mat_vec_int4, native/mat_vec_kernel.cu:166-177). */
int ml2_matvec_int4(ml2_ctx* ctx, void* out, const void* in, const ml2_qweight* w, int rows, int cols);
/* MatVec.Forward (src/MatVec.cs:15-16; mat_vec_kernel, native/mat_vec_kernel.cu:14-49): fp16
 * matrix [cols][rows], out[c] = half(sum_r M[c][r]*in[r]). */
int ml2_matvec_f16(ml2_ctx* ctx, void* out, const void* in, const void* matrix, int rows, int cols);
/* Device-side HostQWeight.Unpack (src/QWeight.cs:29-54) per output row: out fp16 [cols][rows] =
 * half((nibble - zero) * scale). Used for the bit-exact layout check. */
int ml2_dequant_int4(ml2_ctx* ctx, void* out, const ml2_qweight* w, int rows, int cols);

/* ---- operator level: attention products and the small operators --------------------------- */
/* MatVecStrided.Forward (src/MatVecStrided.cs:16-17; mat_vec_strided_kernel,
 * native/mat_vec_kernel.cu:51-81): att[h*seq + t] = half(scale * q_h . K[t][h]), K row stride `dim`.
 * `key` already points at the layer's first cache row. */
int ml2_matvec_strided(ml2_ctx* ctx, void* attention, const void* query, const void* key, int head_size, int dim,
                       int n_heads, int seq_length, float scale);
/* Softmax.Forward (src/Softmax.cs:14; softmax_kernel, native/softmax_kernel.cu:10-52): in place,
 * one row of `seq_length` per head. No 8192 cap. */
int ml2_softmax(ml2_ctx* ctx, void* attention, int n_heads, int seq_length);
/* VecMat.Forward (src/VecMat.cs:17-18; vec_mat_kernel, native/vec_mat_kernel.cu:8-48):
 * out[h*hs + d] = half(sum_t att[h*seq + t] * V[t][h][d]). */
int ml2_vecmat(ml2_ctx* ctx, void* out, const void* value, const void* attention, int head_size, int dim, int n_heads,
               int seq_length);
/* RMSNorm.Forward (src/RMSNorm.cs:14; rmsnorm_kernel, native/rmsnorm_kernel.cu:8-42). out may alias in. */
int ml2_rmsnorm(ml2_ctx* ctx, void* out, const void* in, const void* weights, int size, float eps);
/* RoPERotation.Forward (src/RoPERotation.cs:19-24; rope_kernel, native/rope_kernel.cu:3-31):
 * rotates q and the key row `key` (offset already applied) in place. */
int ml2_rope(ml2_ctx* ctx, void* query, void* key, int n_heads, int n_kv_heads, int head_size, int pos, float theta);
/* Embedding.Forward (src/Embedding.cs:14; embedding_kernel, native/embedding_kernel.cu:3-17). */
int ml2_embedding(ml2_ctx* ctx, void* out, const void* table, int size, const int* tokens, int pos);
/* Argmax.Forward (src/Argmax.cs:14; argmax_kernel, native/argmax_kernel.cu:8-46): tokens[next_pos] =
 * argmax(logits) when write_token != 0. Ties resolve to the LOWEST index (the reference's kernel
 * leaves ties to a race, :32-36; its CPU test expects the first maximum, test/ArgmaxTests.cs:33-46). */
int ml2_argmax(ml2_ctx* ctx, const void* logits, int vocab_size, int* tokens, int next_pos, int write_token);

/* ---- host-buffer convenience (the same operators with the copies inside the call) ---------- */
/* Copies `in`/`inout` (host fp16) to scratch owned by the context, runs ml2_matvec_residual_int4 on
 * device-resident weights, copies the result back and synchronises. */
int ml2_matvec_residual_int4_host(ml2_ctx* ctx, void* inout_host, const void* in_host, const ml2_qweight* w_dev,
                                  int rows, int cols);
/* No counterpart in the reference. Same operation and result as ml2_matvec_residual_int4_host, for hosts
 * that must not see the library allocate: hosts that account for every device byte themselves (the
 * reference's C# side owns all device buffers and sizes its KV cache from the free memory it sees), or that
 * gave the whole device to one pool. The two vectors are staged in a fixed 64 KiB array inside the library
 * image (held by every GPU that loads the library), so the call makes no cudaMalloc / cudaFree and uses no
 * allocating routine. Limits: rows <= 16384 and cols <= 16384, larger sizes return ML2_E_INVALID. The first
 * call on a device looks up the array's address (one-time set-up); make that first call outside any stream
 * capture. All calls share the one array: calls whose GPU work overlaps (other streams, other threads or
 * contexts of the same process) race on it - serialise them. */
int ml2_matvec_residual_int4_host_static(ml2_ctx* ctx, void* inout_host, const void* in_host, const ml2_qweight* w_dev,
                                         int rows, int cols);

/* ---- synthetic tensors (counter-based, identical on host and device) ----------------------- */
/* Fills the window [col0, col0+ncols) x groups [g0, g0+ngroups) of a logical rows_full-wide QWeight
 * in QWeight layout with rows = ngroups*128 (or the ragged tail): nibbles and zero points uniform in
 * [0,15], scales half(0.001 + u*0.019). `tensor_id` separates tensors; values depend only on
 * (seed, tensor_id, logical coordinates), so a shard equals the slice of the full tensor. */
int ml2_synth_qweight(ml2_ctx* ctx, uint32_t* weight, uint32_t* zeros, void* scales, int rows_full, int col0, int ncols,
                      int g0, int ngroups, uint64_t seed, uint32_t tensor_id);
/* fp16 ~ N(0, sigma^2) (Irwin-Hall of integer fields: exact, no libm) for rows [row0,row0+nrows) of a
 * logical [*, width] tensor. */
int ml2_synth_normal_f16(ml2_ctx* ctx, void* out, long long row0, long long nrows, int width, float sigma, uint64_t seed,
                         uint32_t tensor_id);
/* Host versions (for the oracle side of parity tests). */
int ml2_synth_qweight_host(uint32_t* weight, uint32_t* zeros, void* scales, int rows_full, int col0, int ncols, int g0,
                           int ngroups, uint64_t seed, uint32_t tensor_id);
int ml2_synth_normal_f16_host(void* out, long long row0, long long nrows, int width, float sigma, uint64_t seed,
                              uint32_t tensor_id);

/* ---- model level -------------------------------------------------------------------------------- */
/* Device pointers of one layer, named as in PerLayerWeight (src/PerLayerWeight.cs:5-16). Under tensor
 * parallelism these are the rank's shards (see ml2_model_local_shape). */
typedef struct ml2_layer_weights {
    ml2_qweight query, key, value, output, gate, up, down;
    const void* rms_attention;    /* fp16 [dim] */
    const void* rms_feed_forward; /* fp16 [dim] */
} ml2_layer_weights;

/* Device buffers of RunState (src/RunState.cs:5-25). key/value caches are [layer][seq_len][kv_dim_local]. */
typedef struct ml2_runstate {
    void *x, *xb, *h, *q, *logits, *key_cache, *value_cache;
    int* tokens; /* [seq_len + 1] */
} ml2_runstate;

/* 128-byte NCCL unique id; rank 0 creates it, every rank passes the same bytes to ml2_model_create. */
int ml2_nccl_unique_id(void* out128);
/* Stands for the Transformer constructor (src/Transformer.cs:46-87) minus file reading: validates the
 * config (GQA is refused like the reference does, :53-56), builds the RoPE table, joins the NCCL group
 * when tp_size > 1 (one process per GPU). The model uses a stream of its own. */
int ml2_model_create(ml2_ctx* ctx, const ml2_config* cfg, int tp_size, int tp_rank, const void* nccl_id128, ml2_model** out);
int ml2_model_destroy(ml2_model* model);
/* Shard owned by this rank: attention width (heads*128), hidden rows (whole groups of 128, starting at
 * group hidden_group0), vocabulary rows (starting at vocab_row0). */
int ml2_model_local_shape(ml2_model* model, int* dim_local, int* hidden_local, int* vocab_local, int* hidden_group0,
                          int* vocab_row0);
void ml2_tp_hidden_groups(int hidden_dim, int tp_size, int tp_rank, int* group0, int* ngroups);
/* Borrow the caller's device arrays (TransformerWeights, src/TransformerWeights.cs:8-16). `classifier_local`
 * holds this rank's vocabulary rows. */
int ml2_model_bind_globals(ml2_model* model, const void* embed, const void* classifier_local, const void* rms_final);
int ml2_model_bind_layer(ml2_model* model, int layer, const ml2_layer_weights* w);
/* Run state: either allocated (and owned) by the library or borrowed from the caller. */
int ml2_model_alloc_runstate(ml2_model* model);
int ml2_model_bind_runstate(ml2_model* model, const ml2_runstate* rs);
int ml2_model_runstate(ml2_model* model, ml2_runstate* rs);
/* Transformer.Forward(position, nextPosition) followed by the greedy Sampler.Sample
 * (src/Transformer.cs:158-190, src/Sampler.cs:44-47): asynchronous; tokens[next_pos] is written on the
 * device when write_token != 0. One persistent-kernel launch (or one CUDA-graph replay) per call. Refused with
 * ML2_E_STATE after a kernel's bounded wait ran out, until ml2_model_reset. */
int ml2_model_forward(ml2_model* model, int pos, int next_pos, int write_token);
/* Waits for the model's stream and reads the device error word: ML2_E_DEVICE if a bounded wait ran out (as do
 * ml2_model_step_host, ml2_model_read_token, ml2_model_read_logits and ml2_model_generate, whose device-to-host
 * read carries the error word along). */
int ml2_model_synchronize(ml2_model* model);
/* After ML2_E_DEVICE: clears the error word and brings every counter the persistent kernel keeps between tokens
 * back to its start. Under tensor parallelism every rank calls it before any rank runs its next forward. No
 * counterpart in the reference (its kernels never wait on one another). */
int ml2_model_reset(ml2_model* model);
long long ml2_model_launches_per_token(ml2_model* model);
int ml2_model_set_tokens(ml2_model* model, const int* tokens_host, int first, int count);
/* Stream-ordered 4-byte host->device copy of one token id; `token_pinned_host` must stay valid until it ran. */
int ml2_model_put_token_async(ml2_model* model, int pos, const int* token_pinned_host);
int ml2_model_read_token(ml2_model* model, int pos, int* token_host);
/* One greedy decode step with HOST buffers, the per-token body of Transformer.Generate (src/Transformer.cs:96-104):
 * copies the input token id from (pinned) host memory to tokens[pos], runs Forward(pos, pos + 1) with the greedy
 * sample, copies tokens[pos + 1] back and waits for it. */
int ml2_model_step_host(ml2_model* model, int pos, const int* token_in_pinned_host, int* token_out_host);
int ml2_model_read_logits(ml2_model* model, void* logits_host_f16);
/* Tensor-parallel persistent kernel (one launch per token per GPU, all-reduce fused into the operator hand-off):
 * every rank owns one peer-visible buffer (counters, fp32 receive zones, logits). `ml2_model_comm_handle` writes
 * its 64-byte CUDA IPC handle; the host exchanges the handles of all ranks (any transport) and passes them, in
 * rank order, to `ml2_model_comm_attach`. Row-sharded mat-vecs then store their fp32 partials straight into every
 * rank's receive zone (plain peer stores over NVLink, no multicast), publish with a system-scope release on every
 * rank's counter, and the next operator adds the tp partials in rank order before the single fp16 rounding.
 * Without attached peers the tensor-parallel model runs the CUDA-graph + ncclAllReduce path. All ranks must call
 * ml2_model_forward the same number of times. */
int ml2_model_comm_handle(ml2_model* model, void* out64);
int ml2_model_comm_attach(ml2_model* model, const void* handles_rank_order, int n_ranks);
/* Diagnostics: per-CTA cycle counters of the last persistent-kernel launch, 64 values per CTA ([0..5] total,
 * dependency waits, ring waits, cycles inside the arithmetic batches, attention, prologue; [8..31] wait / prologue /
 * tile cycles per operator kind; [32..39] copy warp and tail warp: total and wait cycles, the tail's epilogue, sum,
 * hand-back and publish cycles; [40..55] arithmetic and ring-wait cycles per operator kind); needs ML2_MEGA_PROF=1 in
 * the environment when the model is created. */
int ml2_model_debug_prof(ml2_model* model, long long* out, int n);
/* Diagnostics (failure-path test): makes the model expect one more round of operator arrivals than its counters
 * hold, as after a rank skipped a forward; the next forward's waits then run out after the wait limit, the kernel
 * returns, and the synchronising call reports ML2_E_DEVICE. Touches nothing on the device. */
int ml2_model_debug_skip_launch(ml2_model* model);
/* Diagnostics, host only (no GPU needed): plans one weight operator of the persistent kernel (fmt 0 int4, 1 fp16;
 * `rows` inputs, `cols` outputs per matrix, `nmat` matrices, `paired` for gate / up) for a ring slot of `slot_bytes`
 * and `n_cta` CTAs, builds every CTA's tile list as the model does and checks it: every output row covered exactly
 * once, tiles inside the operator and no larger than a full tile, every bulk copy 16-byte aligned in source, size
 * and destination and inside the slot. out8 = {planned, rows covered, fewest / most tiles of a CTA, violations,
 * rows of a full tile, working warps, quantisation groups (fp16: weight vectors) per warp}. */
int ml2_debug_tile_plan(int fmt, int rows, int cols, int nmat, int paired, int slot_bytes, int n_cta, long long* out8);
/* Tuning: the sequence length from which the persistent kernel splits every head's attention over several CTAs
 * (default 704, the measured crossover on a B200 for the 13B shape; shorter sequences keep one CTA per head). */
int ml2_model_set_split_attention_from(ml2_model* model, int min_seq);
/* The CUDA stream the model launches on (for events or for ordering other work after it). */
int ml2_model_stream(ml2_model* model, void** cuda_stream);
/* Times each kernel kind alone over all layers (kinds: 0 qkv, 1 attention, 2 o-proj, 3 gate/up, 4 down,
 * 5 classifier): average microseconds per launch and the algorithmic bytes one launch moves. */
int ml2_model_profile(ml2_model* model, int iters, double* avg_us6, double* algo_bytes6);
/* Transformer.Generate on token ids (src/Transformer.cs:89-112): HOST buffers in and out, copies inside. */
int ml2_model_generate(ml2_model* model, const int* prompt_host, int n_prompt, int steps, int* out_tokens_host, int* n_out);


/* ---- sampling chain (Sampler.Sample, src/Sampler.cs:40-70) -----------------------------------
 * One call per Module of the reference; every kernel is one CTA on the context's stream, in place.
 * SoftmaxLogits.Forward (src/SoftmaxLogits.cs; native/softmax_logits_kernel.cu:10-60): indices[t] = t,
 * logits := softmax(logits / temperature) with the reference's fp16 rounding points. */
int ml2_softmax_logits(ml2_ctx* ctx, void* logits, int size, float temperature, int* indices);
/* Sort.Forward (src/Sort.cs; native/sort_kernel.cu:13-45): fp16 keys descending, int values carried, equal keys
 * keep their order. Any size from 1 to 32768 (the reference needs size = 125 * block size). */
int ml2_sort(ml2_ctx* ctx, void* keys, int* values, int size);
/* CumulativeSum.Forward (src/CumulativeSum.cs; native/cumulative_sum_kernel.cu:9-33): inclusive fp32 sum of fp16
 * values, each output rounded to fp16. Any size (the reference needs size = 32 * block size). */
int ml2_cumulative_sum(ml2_ctx* ctx, void* values, int size);
/* SampleTopP.Forward (src/SampleTopP.cs; native/sample_top_p_kernel.cu:9-29): tokens[pos] = indices[first t with
 * values[t] >= threshold], the last entry if none reaches it. */
int ml2_sample_top_p(ml2_ctx* ctx, const void* values, const int* indices, int size, float threshold, int* tokens, int pos);
/* Sampler.Sample for temperature != 0 (src/Sampler.cs:49-66) on the model's stream, after ml2_model_forward(...,
 * write_token = 0): softmax, sort when 0 < top_p < 1 (threshold = coin * top_p, else coin), cumulative sum, pick;
 * writes tokens[next_pos] and consumes the logits. `coin` is the host's uniform draw in [0,1). */
int ml2_model_sample(ml2_model* model, int next_pos, float temperature, float top_p, float coin);

/* ---- tokenizer (Tokenizer, src/Tokenizer.cs:27-171); host code, no GPU ------------------------------
 * `tokenizer.bin`: int32 maxTokenLength, then per piece float score, int32 byte length, UTF-8 bytes (:34-48).
 * Encode (:95-171): optional BOS, the " " dummy prefix for a non-empty prompt, one token per UTF-16 code unit with
 * the UTF-8 byte fallback (byte + 3), then the best-scoring adjacent pair is merged until none is a piece; optional
 * EOS. Decode (:57-86) is stateful like the reference's: <0xNN> pieces are collected until they form characters. */
typedef struct ml2_tokenizer ml2_tokenizer;
int ml2_tokenizer_open(const char* path, int vocab_size, ml2_tokenizer** out);
int ml2_tokenizer_close(ml2_tokenizer* tokenizer);
int ml2_tokenizer_encode(ml2_tokenizer* tokenizer, const char* prompt_utf8, int bos, int eos, int* out_tokens, int capacity, int* n_out);
int ml2_tokenizer_decode(ml2_tokenizer* tokenizer, int prev, int token, char* out_utf8, int capacity, int* n_out);

/* ---- AWQ checkpoint tensors -> QWeight layout (ModelConverter, src/ModelConverter.cs:196-332) ----------
 * Device buffers in, device buffers out. Format v0: `in` is an AutoAWQ tensor, int32 [height][width / 8] with the
 * nibble order map {0,2,4,6,1,3,5,7} (:19); `out` is u32 [width][ceil(height / 8)], 8 consecutive inputs per word
 * (RepackQData, :286-321; height = d_in for weights, the number of groups for zero points). */
int ml2_awq_repack_qdata(ml2_ctx* ctx, const uint32_t* in, int height, int width, uint32_t* out);
/* RepackScales (:323-332): fp16 [meta_height][width] -> [width][meta_height]. */
int ml2_awq_repack_scales(ml2_ctx* ctx, const void* in, int meta_height, int width, void* out);
/* Format v1 (:262-275): scales fp16 [width][padded_height] -> [width][scales_size]. */
int ml2_awq_compact_scales_v1(ml2_ctx* ctx, const void* in, int scales_size, int padded_height, int width, void* out);

/* ---- model.bin reader -------------------------------------------------------------------------
 * Stands for Config.LoadConfig (src/Config.cs:21-31) and the TransformerWeights constructor
 * (src/TransformerWeights.cs:20-41, 54-103): the file written by src/ModelConverter.cs:130-177 is mapped
 * read-only, the 32-byte header is checked (ropeTheta must be 10000), the tensor walk of the reference's reader
 * is repeated (globals: embedding, classifier, final norm; per layer the QWeights query, key, value, output, up,
 * gate, down as Weight / Zeros / Scales, then the two norm vectors) and the file must be consumed exactly.
 * Host-only calls: ml2_model_file_open / _close / _config / _tensor need no GPU. */
typedef struct ml2_model_file ml2_model_file;
typedef struct ml2_weights ml2_weights;
#define ML2_T_EMBED 0      /* global tensors: layer = -1, part = 0 */
#define ML2_T_CLASSIFIER 1
#define ML2_T_RMS_FINAL 2
#define ML2_T_QUERY 0      /* layer tensors; QWeights have part 0 = Weight, 1 = Zeros, 2 = Scales */
#define ML2_T_KEY 1
#define ML2_T_VALUE 2
#define ML2_T_OUTPUT 3
#define ML2_T_UP 4
#define ML2_T_GATE 5
#define ML2_T_DOWN 6
#define ML2_T_RMS_ATT 7
#define ML2_T_RMS_FFN 8
int ml2_model_file_open(const char* path, ml2_model_file** out);
int ml2_model_file_close(ml2_model_file* file);
int ml2_model_file_config(const ml2_model_file* file, ml2_config* out);
/* Pointer into the mapping and byte length of one array of the file. */
int ml2_model_file_tensor(const ml2_model_file* file, int layer, int tensor, int part, const void** data, uint64_t* bytes);
/* Host-only: the part of one QWeight (tensor ML2_T_QUERY .. ML2_T_DOWN) that rank `tp_rank` of `tp_size` owns, copied
 * into caller buffers (any of them may be null to ask for the sizes only). Outputs of query / key / value / up / gate
 * are cut by range; inputs of output / down as a window of whole groups of 128, zero points re-packed from the
 * window's first group. */
int ml2_model_file_shard(const ml2_model_file* file, int layer, int tensor, int tp_size, int tp_rank, void* weight_out, void* zeros_out,
                         void* scales_out, uint64_t* weight_bytes, uint64_t* zeros_bytes, uint64_t* scales_bytes);
/* Stands for the host-to-device copies of the Transformer constructor (src/Transformer.cs:58-61 and the
 * CudaDeviceVariable assignments of src/TransformerWeights.cs): copies the shard that rank `tp_rank` of `tp_size`
 * owns into one device allocation (outputs of query / key / value / gate / up and vocabulary rows by range, inputs
 * of output / down as a window of whole groups of 128 with the zero points re-packed from the window's start). */
int ml2_weights_upload(ml2_ctx* ctx, const ml2_model_file* file, int tp_size, int tp_rank, ml2_weights** out);
/* ml2_model_bind_globals + ml2_model_bind_layer for every layer. The weights must outlive the model. */
int ml2_weights_bind(const ml2_weights* weights, ml2_model* model);
int ml2_weights_layer(const ml2_weights* weights, int layer, ml2_layer_weights* out);
int ml2_weights_globals(const ml2_weights* weights, const void** embed, const void** classifier_local, const void** rms_final,
                        uint64_t* device_bytes);
int ml2_weights_free(ml2_weights* weights);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* ML2B200_H */
