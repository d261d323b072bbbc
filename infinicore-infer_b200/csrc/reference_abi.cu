// The reference's C interface over this engine: the six symbols that its Python binding opens
// (scripts/libinfinicore_infer.py:84-137; declared in include/infinicore_infer/models/jiuge.h:50-110), plus
// duplicateKVCache.  A program written against the reference -- its own unmodified scripts/jiuge.py first of all --
// finds them in this library (put it, or a link to it, at $INFINI_ROOT/lib/libinfinicore_infer.so) and drives this
// engine: the reference's loader marshals the weights, its batching code marshals the requests.
//
// What arrives is the reference's packing (scripts/jiuge.py:139-352): the rows of the query and key matrices permuted
// inside each head for an adjacent-pair rotary operator, and the three MiniCPM scales already multiplied into the
// embedding, the output and down matrices and the final norm.  The rows are put back in the checkpoint's order (an
// exact operation; this engine rotates pair (j, j + head/2), which is the same function on unpermuted rows) and the
// model runs with all scales at 1.  Matrices arrive in bfloat16, or in float16 or float32 and are then rounded to
// bfloat16 (this engine's 16-bit type); norms in any of the three.  One device only.
//
// The reference's calls return nothing and end the process on an error (src/utils.hpp:10-34).  Here an error is printed
// to stderr; createJiugeModel then returns null, inferBatch fills its output with 0xFFFFFFFF and forwardBatch leaves
// its logits untouched.
#include <cuda_fp16.h>
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "model_api.h"

namespace {

enum RefDtype { REF_F16 = 12, REF_F32 = 13, REF_BF16 = 19 };       // infiniDtype_t, as scripts/libinfinicore_infer.py:7-27 lists it

struct RefMeta {
    int dt_logits;
    size_t nlayer, d, nh, nkvh, dh, di, dctx, dvoc;
    float epsilon, theta;
    uint32_t end_token;
};

struct RefWeights {
    size_t nlayer;
    int dt_norm, dt_mat;
    int transpose_linear_weights;
    const void *input_embd, *output_norm, *output_embd;
    const void *const *attn_norm, *const *attn_qkv, *const *attn_qkv_b, *const *attn_o, *const *ffn_norm, *const *ffn_gate_up,
        *const *ffn_down;
};

uint16_t bf16_of(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);      // NaN stays NaN
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);                       // round to nearest even
}
float f32_of(const void *p, size_t i, int dtype) {
    if (dtype == REF_F32) return ((const float *)p)[i];
    if (dtype == REF_F16) return __half2float(((const __half *)p)[i]);
    uint32_t u = (uint32_t)((const uint16_t *)p)[i] << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
size_t elem_size(int dtype) { return dtype == REF_F32 ? 4 : 2; }

// rows [r0, r0 + heads * dh) of a packed matrix back into the checkpoint's order: row 2j + s of a head came from row
// s * dh/2 + j (scripts/jiuge.py:217-227); `row_bytes` bytes per row
void depermute(const char *src, char *dst, size_t heads, size_t dh, size_t row_bytes) {
    const size_t half = dh / 2;
    for (size_t h = 0; h < heads; ++h)
        for (size_t j = 0; j < half; ++j)
            for (size_t s = 0; s < 2; ++s)
                memcpy(dst + (h * dh + s * half + j) * row_bytes, src + (h * dh + 2 * j + s) * row_bytes, row_bytes);
}

// a matrix of `n` elements in the reference's type as bfloat16
void to_bf16(const void *src, int dtype, size_t n, std::vector<uint16_t> &out) {
    out.resize(n);
    if (dtype == REF_BF16) memcpy(out.data(), src, 2 * n);
    else for (size_t i = 0; i < n; ++i) out[i] = bf16_of(f32_of(src, i, dtype));
}

struct Model {
    JkModel *jk = nullptr;
    RefMeta meta{};
};

std::string own_directory() {
    Dl_info info;
    if (dladdr((const void *)&own_directory, &info) == 0 || info.dli_fname == nullptr) return ".";
    char resolved[4096];
    const char *path = realpath(info.dli_fname, resolved) ? resolved : info.dli_fname;
    std::string s(path);
    const size_t slash = s.rfind('/');
    return slash == std::string::npos ? "." : s.substr(0, slash);
}

void complain(const char *what) { fprintf(stderr, "[infinicore_infer_b200] %s: %s\n", what, jkLastError()); }

}  // namespace

JK_EXPORT void *createJiugeModel(const RefMeta *meta, const RefWeights *w, int device, int ndev, const int *dev_ids) {
    (void)device;
    if (meta == nullptr || w == nullptr) { fprintf(stderr, "[infinicore_infer_b200] createJiugeModel: meta or weights missing\n"); return nullptr; }
    if (ndev != 1) { fprintf(stderr, "[infinicore_infer_b200] createJiugeModel: this engine runs on one device, ndev is %d\n", ndev); return nullptr; }
    if (w->transpose_linear_weights == 0) {
        fprintf(stderr, "[infinicore_infer_b200] createJiugeModel: matrices must come as [out, in] (transpose_linear_weights != 0)\n");
        return nullptr;
    }
    for (int dt : {meta->dt_logits, w->dt_norm, w->dt_mat})
        if (dt != REF_F16 && dt != REF_F32 && dt != REF_BF16) { fprintf(stderr, "[infinicore_infer_b200] createJiugeModel: data type %d\n", dt); return nullptr; }
    const size_t L = meta->nlayer, d = meta->d, nh = meta->nh, nkvh = meta->nkvh, dh = meta->dh, di = meta->di, V = meta->dvoc;
    const size_t nq = (nh + 2 * nkvh) * dh;
    JkModelMeta m{};
    m.nlayer = (int32_t)L; m.d = (int32_t)d; m.nh = (int32_t)nh; m.nkvh = (int32_t)nkvh; m.dh = (int32_t)dh; m.di = (int32_t)di;
    m.dctx = (int32_t)meta->dctx; m.dvoc = (int32_t)V;
    m.epsilon = meta->epsilon; m.theta = meta->theta;
    m.embed_scale = m.residual_scale = m.logit_scale = 1.f;         // the reference's loader multiplied them into the weights
    m.end_token = (int32_t)meta->end_token;

    // everything as this engine takes it: bfloat16 matrices in the checkpoint's row order, float32 norms and biases
    std::vector<uint16_t> embd, head;
    std::vector<float> final_norm(d);
    to_bf16(w->input_embd, meta->dt_logits, V * d, embd);
    const bool tied = w->output_embd == w->input_embd;
    if (!tied) to_bf16(w->output_embd, w->dt_mat, V * d, head);
    for (size_t i = 0; i < d; ++i) final_norm[i] = f32_of(w->output_norm, i, w->dt_norm);
    std::vector<std::vector<uint16_t>> qkv(L), o(L), gate_up(L), down(L);
    std::vector<std::vector<float>> norm1(L, std::vector<float>(d)), norm2(L, std::vector<float>(d)), bias(L);
    std::vector<const void *> p_qkv(L), p_o(L), p_gu(L), p_down(L), p_n1(L), p_n2(L), p_bias(L, nullptr);
    const size_t es = elem_size(w->dt_mat);
    std::vector<char> rows(nq * d * es);
    for (size_t l = 0; l < L; ++l) {
        const char *packed = (const char *)w->attn_qkv[l];
        depermute(packed, rows.data(), nh, dh, d * es);
        depermute(packed + nh * dh * d * es, rows.data() + nh * dh * d * es, nkvh, dh, d * es);
        memcpy(rows.data() + (nh + nkvh) * dh * d * es, packed + (nh + nkvh) * dh * d * es, nkvh * dh * d * es);
        to_bf16(rows.data(), w->dt_mat, nq * d, qkv[l]);
        to_bf16(w->attn_o[l], w->dt_mat, d * nh * dh, o[l]);
        to_bf16(w->ffn_gate_up[l], w->dt_mat, 2 * di * d, gate_up[l]);
        to_bf16(w->ffn_down[l], w->dt_mat, d * di, down[l]);
        for (size_t i = 0; i < d; ++i) {
            norm1[l][i] = f32_of(w->attn_norm[l], i, w->dt_norm);
            norm2[l][i] = f32_of(w->ffn_norm[l], i, w->dt_norm);
        }
        if (w->attn_qkv_b != nullptr && w->attn_qkv_b[l] != nullptr) {
            // the bias comes in the logits' type, permuted like the rows it belongs to
            std::vector<float> packed_b(nq), hf(nq);
            for (size_t i = 0; i < nq; ++i) packed_b[i] = f32_of(w->attn_qkv_b[l], i, meta->dt_logits);
            depermute((const char *)packed_b.data(), (char *)hf.data(), nh, dh, sizeof(float));
            depermute((const char *)(packed_b.data() + nh * dh), (char *)(hf.data() + nh * dh), nkvh, dh, sizeof(float));
            memcpy(hf.data() + (nh + nkvh) * dh, packed_b.data() + (nh + nkvh) * dh, nkvh * dh * sizeof(float));
            bias[l] = hf;
            p_bias[l] = bias[l].data();
        }
        p_qkv[l] = qkv[l].data(); p_o[l] = o[l].data(); p_gu[l] = gate_up[l].data(); p_down[l] = down[l].data();
        p_n1[l] = norm1[l].data(); p_n2[l] = norm2[l].data();
    }
    JkModelWeights jw{};
    jw.norm_dtype = 0;
    jw.input_embd = embd.data();
    jw.output_embd = tied ? embd.data() : head.data();
    jw.output_norm = final_norm.data();
    jw.attn_norm = p_n1.data(); jw.attn_qkv = p_qkv.data(); jw.attn_o = p_o.data(); jw.ffn_norm = p_n2.data();
    jw.ffn_gate_up = p_gu.data(); jw.ffn_down = p_down.data();
    jw.attn_qkv_b = (w->attn_qkv_b != nullptr) ? p_bias.data() : nullptr;

    const std::string dir = own_directory();
    JkModelOptions opt{};
    opt.device = dev_ids != nullptr ? dev_ids[0] : 0;
    opt.page_size = 16;
    // The reference gives every cache handle a whole context of its own; here all handles share one pool of pages.
    // INFINICORE_INFER_B200_CACHE_TOKENS sizes it; the default holds eight whole contexts.
    const char *tokens_env = getenv("INFINICORE_INFER_B200_CACHE_TOKENS");
    opt.cache_tokens = tokens_env != nullptr ? atoll(tokens_env) : 8LL * (long long)meta->dctx;
    opt.max_step_tokens = 8192;
    opt.kernel_dir = dir.c_str();
    Model *model = new Model();
    model->meta = *meta;
    model->jk = jkCreateModel(&m, &jw, &opt);
    if (model->jk == nullptr) {
        complain("createJiugeModel");
        delete model;
        return nullptr;
    }
    return model;
}

JK_EXPORT void destroyJiugeModel(void *model) {
    Model *m = (Model *)model;
    if (m == nullptr) return;
    jkDestroyModel(m->jk);
    delete m;
}

JK_EXPORT void *createKVCache(const void *model) {
    const Model *m = (const Model *)model;
    return m != nullptr ? jkCreateKVCache(m->jk) : nullptr;
}

JK_EXPORT void *duplicateKVCache(const void *model, const void *cache, uint32_t seq_len) {
    const Model *m = (const Model *)model;
    if (m == nullptr) return nullptr;
    JkKVCache *c = jkDuplicateKVCache(m->jk, (const JkKVCache *)cache, seq_len);
    if (c == nullptr) complain("duplicateKVCache");
    return c;
}

JK_EXPORT void dropKVCache(const void *model, void *cache) {
    const Model *m = (const Model *)model;
    if (m != nullptr) jkDropKVCache(m->jk, (JkKVCache *)cache);
}

JK_EXPORT void inferBatch(void *model, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
                          const uint32_t *req_pos, void **kv_caches, const float *temperature, const uint32_t *topk, const float *topp,
                          uint32_t *output) {
    Model *m = (Model *)model;
    if (m == nullptr || jkInferBatch(m->jk, tokens, ntok, req_lens, nreq, req_pos, (JkKVCache **)kv_caches, temperature, topk, topp,
                                     nullptr, output) != 0) {
        complain("inferBatch");
        for (uint32_t i = 0; output != nullptr && i < nreq; ++i) output[i] = 0xFFFFFFFFu;
    }
}

JK_EXPORT void forwardBatch(void *model, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
                            const uint32_t *req_pos, void **kv_caches, void *logits) {
    Model *m = (Model *)model;
    if (m == nullptr || logits == nullptr) { fprintf(stderr, "[infinicore_infer_b200] forwardBatch: no model or no place for the logits\n"); return; }
    const size_t n = (size_t)ntok * m->meta.dvoc;
    if (m->meta.dt_logits == REF_F32) {
        if (jkForwardBatch(m->jk, tokens, ntok, req_lens, nreq, req_pos, (JkKVCache **)kv_caches, (float *)logits) != 0) complain("forwardBatch");
        return;
    }
    std::vector<float> f(n);
    if (jkForwardBatch(m->jk, tokens, ntok, req_lens, nreq, req_pos, (JkKVCache **)kv_caches, f.data()) != 0) {
        complain("forwardBatch");
        return;
    }
    // the reference hands logits back in its activation type
    if (m->meta.dt_logits == REF_BF16) {
        uint16_t *out = (uint16_t *)logits;
        for (size_t i = 0; i < n; ++i) out[i] = bf16_of(f[i]);
    } else {
        __half *out = (__half *)logits;
        for (size_t i = 0; i < n; ++i) out[i] = __float2half(f[i]);
    }
}
