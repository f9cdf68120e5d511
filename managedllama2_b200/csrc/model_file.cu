// model.bin reader: the file format of GilesBathgate/ManagedLlama2 (written by src/ModelConverter.cs:130-177, read by
// src/Config.cs:21-31 and src/TransformerWeights.cs:20-103) mapped read-only, checked like the reference checks it,
// and uploaded to the device as the shard one tensor-parallel rank owns.
//
//   header   32 bytes = Config {dim, hiddenDim, numLayers, numHeads, numKVHeads, vocabSize, seqLength (int32), ropeTheta (float)}
//   globals  fp16 embed[vocab][dim], fp16 classifier[vocab][dim], fp16 rms_final[dim]
//   layers   QWeights query, key, value, output, up, gate, down (each: Weight u32, Zeros u32, Scales fp16),
//            then fp16 rms_attention[dim], fp16 rms_feed_forward[dim]
//
// The reference refuses a file whose ropeTheta is not 10000 (src/Config.cs:27-28) and one that is not consumed exactly
// (src/TransformerWeights.cs:39-40); so does this reader.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <vector>

#include "../../include/ml2b200.h"
#include "host_common.hpp"

using namespace ml2;

#define ML2_CUDA(call)                                                                       \
    do {                                                                                     \
        const cudaError_t e_ = (call);                                                       \
        if (e_ != cudaSuccess) return fail(ML2_E_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
    } while (0)

namespace {

constexpr int kGroupRows = 128;

struct Span {
    uint64_t off = 0, bytes = 0;
};
struct QSpan {
    Span w, z, s;
    int rows = 0, cols = 0;
};
struct LayerSpans {
    QSpan q[7];   // file order: query, key, value, output, up, gate, down
    Span rms_att, rms_ffn;
};

inline int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace

struct ml2_model_file {
    int fd = -1;
    const unsigned char* base = nullptr;
    uint64_t size = 0;
    ml2_config cfg{};
    Span embed, classifier, rms_final;
    std::vector<LayerSpans> layers;
};

struct ml2_weights {
    int device = 0;
    int tp = 1, rank = 0;
    ml2_config cfg{};
    unsigned char* arena = nullptr;   // one device allocation holding every tensor of the shard
    uint64_t arena_bytes = 0;
    const void *embed = nullptr, *classifier = nullptr, *rms_final = nullptr;
    std::vector<ml2_layer_weights> layers;
};

int ml2_model_file_open(const char* path, ml2_model_file** out)
{
    if (!path || !out) return fail(ML2_E_INVALID, "model_file_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(ML2_E_INVALID, "model_file_open: %s: %s", path, strerror(errno));
    struct stat st {};
    if (fstat(fd, &st) != 0 || st.st_size < (off_t)sizeof(ml2_config)) {
        close(fd);
        return fail(ML2_E_INVALID, "model_file_open: %s is shorter than the 32-byte header", path);
    }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    if (map == MAP_FAILED) {
        close(fd);
        return fail(ML2_E_INVALID, "model_file_open: mmap of %s failed: %s", path, strerror(errno));
    }
    ml2_model_file* f = new ml2_model_file;
    f->fd = fd;
    f->base = static_cast<const unsigned char*>(map);
    f->size = (uint64_t)st.st_size;
    memcpy(&f->cfg, f->base, sizeof(ml2_config));
    const ml2_config& c = f->cfg;
    auto bad = [&](const char* why) {
        const int rc = fail(ML2_E_INVALID, "model_file_open: %s: %s", path, why);
        ml2_model_file_close(f);
        return rc;
    };
    if (c.rope_theta != 10000.0f) return bad("Invalid model config (ropeTheta must be 10000)");   // src/Config.cs:27-28
    if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.vocab_size <= 0 ||
        c.seq_len <= 0 || c.dim % c.n_heads)
        return bad("Invalid model config (non-positive or inconsistent sizes)");

    // the reader's walk (src/TransformerWeights.cs:33-37, 81-95)
    uint64_t off = sizeof(ml2_config);
    auto take = [&](uint64_t bytes) {
        Span s;
        s.off = off;
        s.bytes = bytes;
        off += bytes;
        return s;
    };
    const uint64_t dim = (uint64_t)c.dim, vocab = (uint64_t)c.vocab_size;
    const int kv_dim = (int)((int64_t)c.dim * c.n_kv_heads / c.n_heads);
    f->embed = take(vocab * dim * 2);
    f->classifier = take(vocab * dim * 2);
    f->rms_final = take(dim * 2);
    auto qweight = [&](int rows, int cols) {   // ReadQWeight, src/TransformerWeights.cs:54-69
        QSpan q;
        q.rows = rows;
        q.cols = cols;
        const uint64_t ssize = (uint64_t)cdiv(rows, kGroupRows), wsize = (uint64_t)cdiv(rows, 32) * 4, zsize = (uint64_t)cdiv((int)ssize, 8);
        q.w = take(wsize * (uint64_t)cols * 4);
        q.z = take(zsize * (uint64_t)cols * 4);
        q.s = take(ssize * (uint64_t)cols * 2);
        return q;
    };
    f->layers.resize((size_t)c.n_layers);
    for (LayerSpans& L : f->layers) {
        L.q[0] = qweight(c.dim, c.dim);
        L.q[1] = qweight(c.dim, kv_dim);
        L.q[2] = qweight(c.dim, kv_dim);
        L.q[3] = qweight(c.dim, c.dim);
        L.q[4] = qweight(c.dim, c.hidden_dim);   // up comes before gate in the file
        L.q[5] = qweight(c.dim, c.hidden_dim);
        L.q[6] = qweight(c.hidden_dim, c.dim);
        L.rms_att = take(dim * 2);
        L.rms_ffn = take(dim * 2);
    }
    if (off != f->size) {   // src/TransformerWeights.cs:39-40
        const int rc = fail(ML2_E_INVALID, "model_file_open: %s: Failed to read file. offset: %llu != length: %llu", path,
                            (unsigned long long)(off - sizeof(ml2_config)), (unsigned long long)(f->size - sizeof(ml2_config)));
        ml2_model_file_close(f);
        return rc;
    }
    *out = f;
    return ML2_OK;
}

int ml2_model_file_close(ml2_model_file* f)
{
    if (!f) return ML2_OK;
    if (f->base) munmap(const_cast<unsigned char*>(f->base), (size_t)f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
    return ML2_OK;
}

int ml2_model_file_config(const ml2_model_file* f, ml2_config* out)
{
    if (!f || !out) return fail(ML2_E_INVALID, "model_file_config: null argument");
    *out = f->cfg;
    return ML2_OK;
}

int ml2_model_file_tensor(const ml2_model_file* f, int layer, int tensor, int part, const void** data, uint64_t* bytes)
{
    if (!f || !data || !bytes) return fail(ML2_E_INVALID, "model_file_tensor: null argument");
    Span s;
    if (layer < 0) {
        if (tensor == ML2_T_EMBED) s = f->embed;
        else if (tensor == ML2_T_CLASSIFIER) s = f->classifier;
        else if (tensor == ML2_T_RMS_FINAL) s = f->rms_final;
        else return fail(ML2_E_INVALID, "model_file_tensor: global tensor %d", tensor);
        if (part != 0) return fail(ML2_E_INVALID, "model_file_tensor: part %d of a plain tensor", part);
    } else {
        if (layer >= (int)f->layers.size()) return fail(ML2_E_INVALID, "model_file_tensor: layer %d of %d", layer, (int)f->layers.size());
        const LayerSpans& L = f->layers[(size_t)layer];
        if (tensor >= ML2_T_QUERY && tensor <= ML2_T_DOWN) {
            const QSpan& q = L.q[tensor - ML2_T_QUERY];
            if (part < 0 || part > 2) return fail(ML2_E_INVALID, "model_file_tensor: part %d of a QWeight", part);
            s = part == 0 ? q.w : (part == 1 ? q.z : q.s);
        } else if (tensor == ML2_T_RMS_ATT || tensor == ML2_T_RMS_FFN) {
            if (part != 0) return fail(ML2_E_INVALID, "model_file_tensor: part %d of a plain tensor", part);
            s = tensor == ML2_T_RMS_ATT ? L.rms_att : L.rms_ffn;
        } else {
            return fail(ML2_E_INVALID, "model_file_tensor: layer tensor %d", tensor);
        }
    }
    *data = f->base + s.off;
    *bytes = s.bytes;
    return ML2_OK;
}

namespace {

// Geometry of one rank's part of a QWeight: a range of outputs (columns of the layout) and a window of whole
// quantisation groups of the inputs.
struct Shard {
    int col0, ncols, g0, ngroups;   // ngroups < 0: every input (no window)
};

struct Placed {
    uint64_t w, z, s;   // arena offsets
    int rows_local;
};

uint64_t align256(uint64_t v) { return (v + 255) & ~uint64_t(255); }

// bytes of the shard's three arrays
void shard_sizes(const QSpan& q, const Shard& sh, uint64_t* bw, uint64_t* bz, uint64_t* bs, int* rows_local)
{
    const int rows = sh.ngroups < 0 ? q.rows : std::min(sh.ngroups * kGroupRows, q.rows - sh.g0 * kGroupRows);
    const uint64_t ssize = (uint64_t)cdiv(rows, kGroupRows), wsize = (uint64_t)cdiv(rows, 32) * 4, zsize = (uint64_t)cdiv((int)ssize, 8);
    *bw = wsize * (uint64_t)sh.ncols * 4;
    *bz = zsize * (uint64_t)sh.ncols * 4;
    *bs = ssize * (uint64_t)sh.ncols * 2;
    *rows_local = rows;
}

// The shard of `q` as three host pointers. A column range is contiguous in all three arrays of the file (the pointers
// then point into the mapping); a window of groups is cut out of every column into `tmp` (weights: 16 words per group;
// scales: one per group; zero points: re-packed so that the window's first group sits in nibble 0 of word 0).
void cut_qweight(const ml2_model_file* f, const QSpan& q, const Shard& sh, std::vector<unsigned char>& tmp, const void** pw, const void** pz,
                 const void** ps, uint64_t* bw_out, uint64_t* bz_out, uint64_t* bs_out)
{
    const unsigned char* fw = f->base + q.w.off;
    const unsigned char* fz = f->base + q.z.off;
    const unsigned char* fs = f->base + q.s.off;
    const uint64_t ssize_f = (uint64_t)cdiv(q.rows, kGroupRows), wsize_f = (uint64_t)cdiv(q.rows, 32) * 4, zsize_f = (uint64_t)cdiv((int)ssize_f, 8);
    uint64_t bw, bz, bs;
    int rows_local;
    shard_sizes(q, sh, &bw, &bz, &bs, &rows_local);
    *bw_out = bw; *bz_out = bz; *bs_out = bs;
    const bool window = sh.ngroups >= 0 && !(sh.g0 == 0 && rows_local == q.rows);
    if (!window) {
        *pw = fw + (uint64_t)sh.col0 * wsize_f * 4;
        *pz = fz + (uint64_t)sh.col0 * zsize_f * 4;
        *ps = fs + (uint64_t)sh.col0 * ssize_f * 2;
        return;
    }
    const uint64_t ng = (uint64_t)cdiv(rows_local, kGroupRows);
    const uint64_t wsize_l = (uint64_t)cdiv(rows_local, 32) * 4, zsize_l = (ng + 7) / 8;
    tmp.assign((size_t)(bw + bz + bs), 0);
    uint32_t* tw = reinterpret_cast<uint32_t*>(tmp.data());
    uint32_t* tz = reinterpret_cast<uint32_t*>(tmp.data() + bw);
    uint16_t* ts = reinterpret_cast<uint16_t*>(tmp.data() + bw + bz);
    for (int c = 0; c < sh.ncols; ++c) {
        const uint64_t col = (uint64_t)(sh.col0 + c);
        const uint32_t* sw = reinterpret_cast<const uint32_t*>(fw) + col * wsize_f + (uint64_t)sh.g0 * 16;
        memcpy(tw + (uint64_t)c * wsize_l, sw, (size_t)wsize_l * 4);
        const uint16_t* ss = reinterpret_cast<const uint16_t*>(fs) + col * ssize_f + (uint64_t)sh.g0;
        memcpy(ts + (uint64_t)c * ng, ss, (size_t)ng * 2);
        const uint32_t* sz = reinterpret_cast<const uint32_t*>(fz) + col * zsize_f;
        uint32_t* dz = tz + (uint64_t)c * zsize_l;
        for (uint64_t j = 0; j < ng; ++j) {
            const uint64_t g = (uint64_t)sh.g0 + j;
            const uint32_t nib = (sz[g >> 3] >> (4 * (g & 7))) & 0xFu;
            dz[j >> 3] |= nib << (4 * (j & 7));
        }
    }
    *pw = tw;
    *pz = tz;
    *ps = ts;
}

int upload_qweight(const ml2_model_file* f, const QSpan& q, const Shard& sh, unsigned char* arena, const Placed& at,
                   std::vector<unsigned char>& tmp)
{
    const void *pw, *pz, *ps;
    uint64_t bw, bz, bs;
    cut_qweight(f, q, sh, tmp, &pw, &pz, &ps, &bw, &bz, &bs);
    ML2_CUDA(cudaMemcpy(arena + at.w, pw, bw, cudaMemcpyHostToDevice));
    ML2_CUDA(cudaMemcpy(arena + at.z, pz, bz, cudaMemcpyHostToDevice));
    ML2_CUDA(cudaMemcpy(arena + at.s, ps, bs, cudaMemcpyHostToDevice));
    return ML2_OK;
}

// shard geometry of the seven QWeights of a layer (file order) for one rank; false when the shapes do not split
bool layer_shards(const ml2_config& c, int tp_size, int tp_rank, Shard (&shards)[7], int* hidden_local_out)
{
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return false;
    if (c.n_heads % tp_size || c.vocab_size % tp_size || (c.dim / tp_size) % kGroupRows || (tp_size > 1 && c.hidden_dim % kGroupRows)) return false;
    const int dim_local = c.dim / tp_size;
    int hg0 = 0, hng = 0;
    ml2_tp_hidden_groups(c.hidden_dim, tp_size, tp_rank, &hg0, &hng);
    const int hidden_local = tp_size == 1 ? c.hidden_dim : hng * kGroupRows;
    const Shard sq{tp_rank * dim_local, dim_local, 0, -1};
    const Shard so{0, c.dim, tp_rank * (dim_local / kGroupRows), tp_size == 1 ? -1 : dim_local / kGroupRows};
    const Shard sf{tp_size == 1 ? 0 : hg0 * kGroupRows, hidden_local, 0, -1};
    const Shard sd{0, c.dim, hg0, tp_size == 1 ? -1 : hng};
    const Shard all[7] = {sq, sq, sq, so, sf, sf, sd};
    for (int i = 0; i < 7; ++i) shards[i] = all[i];
    if (hidden_local_out) *hidden_local_out = hidden_local;
    return true;
}

}  // namespace

int ml2_weights_upload(ml2_ctx* h, const ml2_model_file* f, int tp_size, int tp_rank, ml2_weights** out)
{
    Ctx* ctx = reinterpret_cast<Ctx*>(h);
    if (!ctx || !f || !out) return fail(ML2_E_INVALID, "weights_upload: null argument");
    *out = nullptr;
    const ml2_config& c = f->cfg;
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail(ML2_E_INVALID, "weights_upload: rank %d of %d", tp_rank, tp_size);
    if (c.n_kv_heads != c.n_heads)   // src/Transformer.cs:53-56
        return fail(ML2_E_INVALID, "weights_upload: grouped-query attention is not supported (the reference refuses it too)");
    if (c.n_heads % tp_size || c.vocab_size % tp_size || (c.dim / tp_size) % kGroupRows || (tp_size > 1 && c.hidden_dim % kGroupRows))
        return fail(ML2_E_INVALID, "weights_upload: heads=%d vocab=%d dim=%d hidden=%d do not split over %d ranks", c.n_heads, c.vocab_size,
                    c.dim, c.hidden_dim, tp_size);
    const int vocab_local = c.vocab_size / tp_size;
    Shard shards[7];
    layer_shards(c, tp_size, tp_rank, shards, nullptr);

    // arena layout
    uint64_t total = 0;
    auto place = [&](uint64_t bytes) {
        const uint64_t at = total;
        total += align256(bytes);
        return at;
    };
    const uint64_t dim2 = (uint64_t)c.dim * 2;
    const uint64_t at_embed = place((uint64_t)c.vocab_size * dim2), at_cls = place((uint64_t)vocab_local * dim2), at_rmsf = place(dim2);
    struct LayerAt {
        Placed q[7];
        uint64_t rms_att, rms_ffn;
    };
    std::vector<LayerAt> at((size_t)c.n_layers);
    for (int l = 0; l < c.n_layers; ++l) {
        for (int t = 0; t < 7; ++t) {
            uint64_t bw, bz, bs;
            int rl;
            shard_sizes(f->layers[(size_t)l].q[t], shards[t], &bw, &bz, &bs, &rl);
            at[(size_t)l].q[t] = Placed{place(bw), place(bz), place(bs), rl};
        }
        at[(size_t)l].rms_att = place(dim2);
        at[(size_t)l].rms_ffn = place(dim2);
    }

    ML2_CUDA(cudaSetDevice(ctx->device));
    ml2_weights* w = new ml2_weights;
    w->device = ctx->device;
    w->tp = tp_size;
    w->rank = tp_rank;
    w->cfg = c;
    w->arena_bytes = total;
    {
        const cudaError_t e = cudaMalloc(&w->arena, (size_t)total);
        if (e != cudaSuccess) {
            delete w;
            return fail(ML2_E_CUDA, "weights_upload: %llu bytes of device memory: %s", (unsigned long long)total, cudaGetErrorString(e));
        }
    }
    auto up = [&](uint64_t dst, const Span& s, uint64_t skip, uint64_t bytes) {
        return cudaMemcpy(w->arena + dst, f->base + s.off + skip, (size_t)bytes, cudaMemcpyHostToDevice);
    };
    int rc = ML2_OK;
    auto check = [&](cudaError_t e) {
        if (e != cudaSuccess && rc == ML2_OK) rc = fail(ML2_E_CUDA, "weights_upload: copy failed: %s", cudaGetErrorString(e));
    };
    check(up(at_embed, f->embed, 0, f->embed.bytes));
    check(up(at_cls, f->classifier, (uint64_t)tp_rank * vocab_local * dim2, (uint64_t)vocab_local * dim2));
    check(up(at_rmsf, f->rms_final, 0, dim2));
    w->embed = w->arena + at_embed;
    w->classifier = w->arena + at_cls;
    w->rms_final = w->arena + at_rmsf;
    w->layers.resize((size_t)c.n_layers);
    std::vector<unsigned char> tmp;
    for (int l = 0; l < c.n_layers && rc == ML2_OK; ++l) {
        const LayerSpans& L = f->layers[(size_t)l];
        ml2_qweight qs[7];
        for (int t = 0; t < 7 && rc == ML2_OK; ++t) {
            const Placed& p = at[(size_t)l].q[t];
            rc = upload_qweight(f, L.q[t], shards[t], w->arena, p, tmp);
            qs[t].weight = reinterpret_cast<const uint32_t*>(w->arena + p.w);
            qs[t].zeros = reinterpret_cast<const uint32_t*>(w->arena + p.z);
            qs[t].scales = w->arena + p.s;
        }
        check(up(at[(size_t)l].rms_att, L.rms_att, 0, dim2));
        check(up(at[(size_t)l].rms_ffn, L.rms_ffn, 0, dim2));
        ml2_layer_weights& lw = w->layers[(size_t)l];
        lw.query = qs[0]; lw.key = qs[1]; lw.value = qs[2]; lw.output = qs[3];
        lw.up = qs[4]; lw.gate = qs[5]; lw.down = qs[6];   // file order: up before gate
        lw.rms_attention = w->arena + at[(size_t)l].rms_att;
        lw.rms_feed_forward = w->arena + at[(size_t)l].rms_ffn;
    }
    if (rc != ML2_OK) {
        ml2_weights_free(w);
        return rc;
    }
    *out = w;
    return ML2_OK;
}

int ml2_weights_bind(const ml2_weights* w, ml2_model* model)
{
    if (!w || !model) return fail(ML2_E_INVALID, "weights_bind: null argument");
    int dl = 0, hl = 0, vl = 0, hg0 = 0, vr0 = 0;
    int rc = ml2_model_local_shape(model, &dl, &hl, &vl, &hg0, &vr0);
    if (rc != ML2_OK) return rc;
    if (dl != w->cfg.dim / w->tp || vl != w->cfg.vocab_size / w->tp || vr0 != w->rank * vl)
        return fail(ML2_E_INVALID, "weights_bind: the model's shard (dim %d, vocabulary %d from row %d) is not the one uploaded (rank %d of %d)", dl,
                    vl, vr0, w->rank, w->tp);
    rc = ml2_model_bind_globals(model, w->embed, w->classifier, w->rms_final);
    for (size_t l = 0; l < w->layers.size() && rc == ML2_OK; ++l) rc = ml2_model_bind_layer(model, (int)l, &w->layers[l]);
    return rc;
}

int ml2_weights_layer(const ml2_weights* w, int layer, ml2_layer_weights* out)
{
    if (!w || !out || layer < 0 || layer >= (int)w->layers.size()) return fail(ML2_E_INVALID, "weights_layer: layer %d", layer);
    *out = w->layers[(size_t)layer];
    return ML2_OK;
}

int ml2_weights_globals(const ml2_weights* w, const void** embed, const void** classifier_local, const void** rms_final, uint64_t* device_bytes)
{
    if (!w) return fail(ML2_E_INVALID, "weights_globals: null argument");
    if (embed) *embed = w->embed;
    if (classifier_local) *classifier_local = w->classifier;
    if (rms_final) *rms_final = w->rms_final;
    if (device_bytes) *device_bytes = w->arena_bytes;
    return ML2_OK;
}

int ml2_weights_free(ml2_weights* w)
{
    if (!w) return ML2_OK;
    if (w->arena) {
        cudaSetDevice(w->device);
        cudaFree(w->arena);
    }
    delete w;
    return ML2_OK;
}

int ml2_model_file_shard(const ml2_model_file* f, int layer, int tensor, int tp_size, int tp_rank, void* weight_out, void* zeros_out,
                         void* scales_out, uint64_t* weight_bytes, uint64_t* zeros_bytes, uint64_t* scales_bytes)
{
    if (!f) return fail(ML2_E_INVALID, "model_file_shard: null file");
    if (layer < 0 || layer >= (int)f->layers.size() || tensor < ML2_T_QUERY || tensor > ML2_T_DOWN)
        return fail(ML2_E_INVALID, "model_file_shard: layer %d tensor %d", layer, tensor);
    Shard shards[7];
    if (!layer_shards(f->cfg, tp_size, tp_rank, shards, nullptr))
        return fail(ML2_E_INVALID, "model_file_shard: the model does not split over %d ranks (rank %d)", tp_size, tp_rank);
    std::vector<unsigned char> tmp;
    const void *pw, *pz, *ps;
    uint64_t bw, bz, bs;
    cut_qweight(f, f->layers[(size_t)layer].q[tensor - ML2_T_QUERY], shards[tensor - ML2_T_QUERY], tmp, &pw, &pz, &ps, &bw, &bz, &bs);
    if (weight_bytes) *weight_bytes = bw;
    if (zeros_bytes) *zeros_bytes = bz;
    if (scales_bytes) *scales_bytes = bs;
    if (weight_out) memcpy(weight_out, pw, (size_t)bw);
    if (zeros_out) memcpy(zeros_out, pz, (size_t)bz);
    if (scales_out) memcpy(scales_out, ps, (size_t)bs);
    return ML2_OK;
}
