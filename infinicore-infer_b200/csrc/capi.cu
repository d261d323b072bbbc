// The C interface of model_api.h on top of the native step: weights and cache pages on the device, one page list per
// cache handle, and sampling.
//
// It is the same step as the Python engine's, made of the same pieces: the model is the launch records that the
// emitters of runner.cu write (the ones the Python parts call), jk_runner_run replays them, and the page pool, the
// layout and packing of a batch's metadata, the attention's work lists, the rotary tables and the uniform numbers are
// the functions of host_rules.h that the Python engine calls too.  This file only decides which pages a request holds
// and arranges the records in this architecture's block.  (The reference's counterpart is
// src/models/jiuge/jiuge.cpp:27-117 for the device resources and :300-350 for the two batch calls; its
// caches are contiguous per request, src/cache_manager/kvcache.cpp, these are paged.)
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "model_api.h"
#include "runner.h"

extern "C" const char *jk_runner_last_error();
extern "C" int jk_runner_launches();

namespace {
constexpr long long WORKSPACE_BYTES = 32ll << 20;
}  // namespace

struct JkKVCache {
    std::vector<int> pages;
};

struct JkModel {
    JkModelMeta meta{};
    int device = 0, page_size = 64, max_step_tokens = 2048, max_blocks = 0, max_requests = 0;
    RunnerEnv env{};
    std::vector<RunnerOp> ops;                   // the model as launch records: embedding, the layers, final norm, output product
    RunnerBuffers buffers{};
    std::vector<void *> k_pages, v_pages;        // per layer
    const float *cos_table = nullptr, *sin_table = nullptr;
    std::vector<void *> device_allocs;
    jk::PagePool *pool = nullptr;                // page 0 is never handed out: padding rows write there
    cudaStream_t stream = nullptr;
    int *meta_host = nullptr, *meta_dev = nullptr;
    int meta_words = 0, extra_words = 0;
    float *logits = nullptr;
    long long logits_rows = 0;
    int *out_dev = nullptr;                      // ids of the largest logits, then drawn ids: 2 * max_requests
    float *sample_dev = nullptr;                 // sampling parameters of a batch: 4 * max_requests
    size_t page_bytes = 0;                       // one page of one layer's keys (or values)
    int last_launches = 0;
    std::vector<void *> libraries;
};

namespace {

int cuda_fail(cudaError_t e, const char *what) {
    JK_FAIL(JK_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
}
#define CUDA_TRY(call, what)                                  \
    do {                                                      \
        cudaError_t e_ = (call);                              \
        if (e_ != cudaSuccess) return cuda_fail(e_, what);    \
    } while (0)

int device_alloc(JkModel *m, void **p, size_t bytes, const char *what) {
    CUDA_TRY(cudaMalloc(p, bytes ? bytes : 16), what);
    m->device_allocs.push_back(*p);
    return JK_OK;
}

int upload(JkModel *m, const void **dst, const void *src, size_t bytes, const char *what) {
    JK_REQUIRE(src != nullptr, "create model: %s is missing", what);
    void *p = nullptr;
    if (int rc = device_alloc(m, &p, bytes, what)) return rc;
    CUDA_TRY(cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice), what);
    *dst = p;
    return JK_OK;
}

// A norm's weights, whatever they are stored in, as float32 on the device.
int upload_norm(JkModel *m, const float **dst, const void *src, int dtype, int n, const char *what) {
    JK_REQUIRE(src != nullptr, "create model: %s is missing", what);
    std::vector<float> f((size_t)n);
    if (dtype == JK_F32) {
        memcpy(f.data(), src, sizeof(float) * n);
    } else {
        const uint16_t *h = (const uint16_t *)src;
        for (int i = 0; i < n; ++i) {
            const uint32_t bits = (uint32_t)h[i] << 16;
            memcpy(&f[i], &bits, 4);
        }
    }
    const void *p = nullptr;
    if (int rc = upload(m, &p, f.data(), sizeof(float) * n, what)) return rc;
    *dst = (const float *)p;
    return JK_OK;
}

int upload_rotary_tables(JkModel *m) {
    const int half = m->meta.dh / 2, P = m->meta.dctx;
    std::vector<float> c((size_t)P * half), s((size_t)P * half);
    jk::rotary_tables((double)m->meta.theta, half, P, 1.0, c.data(), s.data());
    const void *pc = nullptr, *ps = nullptr;
    if (int rc = upload(m, &pc, c.data(), c.size() * sizeof(float), "the cosine table")) return rc;
    if (int rc = upload(m, &ps, s.data(), s.size() * sizeof(float), "the sine table")) return rc;
    m->cos_table = (const float *)pc;
    m->sin_table = (const float *)ps;
    return JK_OK;
}

// The kernel modules by name from a folder, for a program that has no Python around it.
// The few-row products' own flag (a bounded wait for a tile of weights that ran out): read and cleared by this function.
int (*g_small_fault)() = nullptr;

int bind_from_directory(JkModel *m, const char *dir, bool need_gemm_tcgen05, bool need_attention_tcgen05) {
    auto open = [&](const char *module, void **handle) -> int {
        const std::string path = std::string(dir) + "/libjk_" + module + ".so";
        *handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (*handle == nullptr) JK_FAIL(JK_UNSUPPORTED, "create model: cannot load %s: %s", path.c_str(), dlerror());
        m->libraries.push_back(*handle);
        return JK_OK;
    };
    void *ew = nullptr, *ls = nullptr, *at = nullptr, *sa = nullptr, *gt = nullptr, *att = nullptr;
    if (int rc = open("elementwise", &ew)) return rc;
    if (int rc = open("linear_small", &ls)) return rc;
    if (int rc = open("attention", &at)) return rc;
    if (int rc = open("sampling", &sa)) return rc;
    if (need_gemm_tcgen05)
        if (int rc = open("gemm_tcgen05", &gt)) return rc;
    if (need_attention_tcgen05)
        if (int rc = open("attention_tcgen05", &att)) return rc;
    RunnerFns f{};
    bool missing = false;
    auto sym = [&](void *h, const char *name) -> void * {
        if (h == nullptr) return nullptr;
        void *p = dlsym(h, name);
        if (p == nullptr) missing = true;
        return p;
    };
    f.embed = (EmbedFn)sym(ew, "jk_embed");
    f.add_rmsnorm = (AddRmsnormFn)sym(ew, "jk_add_rmsnorm");
    f.residual_add = (ResidualAddFn)sym(ew, "jk_residual_add");
    f.gemm_f32 = (GemmF32Fn)sym(ew, "jk_gemm_f32");
    f.attention_rows = (AttentionRowsFn)sym(at, "jk_attention_rows");
    f.attention_prefill_supports = (Supports1Fn)sym(at, "jk_attention_prefill_supports");
    f.swiglu = (SwigluFn)sym(ew, "jk_swiglu");
    f.rope_kv = (RopeKvFn)sym(ew, "jk_rope_kv");
    f.linear_small = (LinearSmallFn)sym(ls, "jk_linear_small");
    f.linear_small_qkv = (LinearSmallQkvFn)sym(ls, "jk_linear_small_qkv");
    f.linear_small_supports = (SupportsFn)sym(ls, "jk_linear_small_supports");
    f.linear_small_qkv_supports = (SupportsFn)sym(ls, "jk_linear_small_qkv_supports");
    f.gemm_skinny = (GemmTcgen05Fn)sym(gt, "jk_gemm_skinny");
    f.linear_small_norm_supports = (SupportsFn)sym(ls, "jk_linear_small_norm_supports");
    f.linear_small_norm = (LinearSmallNormFn)sym(ls, "jk_linear_small_norm");
    f.linear_small_qkv_norm = (LinearSmallQkvNormFn)sym(ls, "jk_linear_small_qkv_norm");
    g_small_fault = (int (*)())sym(ls, "jk_linear_small_take_fault");
    f.gemm_tcgen05 = (GemmTcgen05Fn)sym(gt, "jk_gemm_tcgen05");
    f.gemm_tcgen05_qkv = (GemmTcgen05QkvFn)sym(gt, "jk_gemm_tcgen05_qkv");
    f.attention_decode = (AttentionDecodeFn)sym(at, "jk_attention_decode");
    f.attention_prefill = (AttentionPrefillFn)sym(at, "jk_attention_prefill");
    f.attention_tcgen05 = (AttentionTcgen05Fn)sym(att, "jk_attention_tcgen05");
    f.err_elementwise = (LastErrorFn)sym(ew, "jk_elementwise_last_error");
    f.err_linear_small = (LastErrorFn)sym(ls, "jk_linear_small_last_error");
    f.err_gemm_tcgen05 = (LastErrorFn)sym(gt, "jk_gemm_tcgen05_last_error");
    f.err_attention = (LastErrorFn)sym(at, "jk_attention_last_error");
    f.err_attention_tcgen05 = (LastErrorFn)sym(att, "jk_attention_tcgen05_last_error");
    f.argmax = (ArgmaxFn)sym(sa, "jk_argmax");
    f.sample = (SampleFn)sym(sa, "jk_sample");
    f.err_sampling = (LastErrorFn)sym(sa, "jk_sampling_last_error");
    if (missing) JK_FAIL(JK_UNSUPPORTED, "create model: a kernel module in %s lacks an entry point", dir);
    return jk_runner_bind(&f);
}

// The model as launch records, in the arrangement of this architecture's block (src/models/jiuge/jiuge.cpp:195-258):
// norm, attention, norm, feed-forward, each branch added into the stream; the records of each part come from the
// emitters that the Python parts use too.  Pointers that are not known yet (weights, pages) may be null: the same
// function sizes the kernel modules before anything is on the device.
void build_records(JkModel *m, const std::vector<const void *> &w_qkv, const std::vector<const float *> &b_qkv,
                   const std::vector<const void *> &w_o, const std::vector<const void *> &w_gate_up,
                   const std::vector<const void *> &w_down, const std::vector<const float *> &norm1,
                   const std::vector<const float *> &norm2, const void *embedding, const void *lm_head, const float *final_norm) {
    const JkModelMeta &a = m->meta;
    const float softmax_scale = 1.f / std::sqrt((float)a.dh);
    m->ops.clear();
    m->ops.resize((size_t)a.nlayer * 7 + 3);
    RunnerOp *at = m->ops.data();
    at += jk_emit_embedding(at, embedding, JK_BF16, a.d, a.embed_scale);
    for (int l = 0; l < a.nlayer; ++l) {
        at += jk_emit_rmsnorm(at, norm1[l], a.d, a.epsilon, 1.f, 0);
        at += jk_emit_attention(at, w_qkv[l], b_qkv[l], w_o[l], a.d, a.nh, a.nkvh, a.dh, 0, softmax_scale, a.residual_scale,
                                m->cos_table, m->sin_table, 0, a.dctx, m->k_pages.empty() ? nullptr : m->k_pages[l],
                                m->v_pages.empty() ? nullptr : m->v_pages[l], m->pool ? m->pool->num_pages() : 0, 0, 1, 0, 1);
        at += jk_emit_rmsnorm(at, norm2[l], a.d, a.epsilon, 1.f, 0);
        at += jk_emit_swiglu(at, w_gate_up[l], w_down[l], a.d, a.di, a.residual_scale);
    }
    at += jk_emit_rmsnorm(at, final_norm, a.d, a.epsilon, a.logit_scale, 1);
    at += jk_emit_output(at, lm_head, a.dvoc, a.d);
    m->ops.resize((size_t)(at - m->ops.data()));
}

void set_environment(JkModel *m, int sms) {
    RunnerEnv &e = m->env;
    e.dtype = JK_BF16;
    e.page_size = m->page_size;
    e.max_blocks = m->max_blocks;
    e.fused_norms = getenv("JK_NO_FUSED_NORM") == nullptr || getenv("JK_NO_FUSED_NORM")[0] != '1';
    e.routing = jk::Routing{};        // the measured thresholds are the defaults of host_rules.h
    e.routing.sms = sms;
}

int create(JkModel *m, const JkModelMeta *meta, const JkModelWeights *w, const JkModelOptions *opt) {
    JK_REQUIRE(meta && w, "create model: meta or weights missing");
    m->meta = *meta;
    const int L = meta->nlayer, d = meta->d, nh = meta->nh, nkvh = meta->nkvh, dh = meta->dh, di = meta->di, V = meta->dvoc;
    JK_REQUIRE(L > 0 && d > 0 && nh > 0 && nkvh > 0 && dh > 0 && di > 0 && V > 0 && meta->dctx > 0,
               "create model: a size is not positive");
    JK_REQUIRE(nh % nkvh == 0, "create model: %d heads do not divide into %d key/value heads", nh, nkvh);
    JK_REQUIRE(d % 8 == 0 && di % 8 == 0 && (nh * dh) % 8 == 0 && dh % 2 == 0,
               "create model: width %d, feed-forward width %d and head size %d must be multiples of 8, 8 and 2", d, di, dh);
    JK_REQUIRE(w->norm_dtype == JK_F32 || w->norm_dtype == JK_BF16, "create model: norm_dtype %d", w->norm_dtype);
    m->device = opt ? opt->device : 0;
    m->page_size = opt && opt->page_size ? opt->page_size : 64;
    m->max_step_tokens = opt && opt->max_step_tokens ? opt->max_step_tokens : 2048;
    const long long cache_tokens = opt && opt->cache_tokens ? opt->cache_tokens : meta->dctx;
    JK_REQUIRE(m->page_size > 0 && m->max_step_tokens > 0 && cache_tokens > 0, "create model: an option is negative");
    CUDA_TRY(cudaSetDevice(m->device), "create model: cudaSetDevice");
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, m->device), "create model: device properties");
    JK_REQUIRE(prop.major == 10, "create model: the kernels are built for sm_100a, device %d is sm_%d%d", m->device, prop.major,
               prop.minor);
    CUDA_TRY(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking), "create model: stream");
    m->max_blocks = (meta->dctx + m->page_size - 1) / m->page_size;
    const long long num_pages = (cache_tokens + m->page_size - 1) / m->page_size;
    m->pool = new jk::PagePool((int)num_pages + 1, 1);
    set_environment(m, prop.multiProcessorCount);

    // the kernels: which modules the records can reach is asked of the runner itself, on records without pointers
    const std::vector<const void *> none((size_t)L, nullptr);
    const std::vector<const float *> nonef((size_t)L, nullptr);
    build_records(m, none, nonef, none, none, none, nonef, nonef, nullptr, nullptr, nullptr);
    const bool need_gemm = jk_runner_needs_gemm_tcgen05(&m->env, m->ops.data(), (int)m->ops.size(), m->max_step_tokens) != 0;
    const bool need_attention = jk::attention_tcgen05_takes(dh, m->page_size);
    if (opt && opt->kernel_dir) {
        if (int rc = bind_from_directory(m, opt->kernel_dir, need_gemm, need_attention)) return rc;
    }
    const RunnerFns *fns = jk_runner_fns();
    JK_REQUIRE(fns != nullptr, "create model: no kernels are bound; give kernel_dir or call jk_runner_bind first");
    JK_REQUIRE(fns->argmax && fns->sample, "create model: the bound kernels lack the sampling entry points");
    JK_REQUIRE(!need_gemm || fns->gemm_tcgen05, "create model: steps of %d tokens need the tcgen05 product, which is not bound",
               m->max_step_tokens);

    // weights
    const void *embedding = nullptr, *lm_head = nullptr;
    const float *final_norm = nullptr;
    if (int rc = upload(m, &embedding, w->input_embd, (size_t)V * d * 2, "input_embd")) return rc;
    if (w->output_embd == w->input_embd || w->output_embd == nullptr) lm_head = embedding;
    else if (int rc = upload(m, &lm_head, w->output_embd, (size_t)V * d * 2, "output_embd")) return rc;
    if (int rc = upload_norm(m, &final_norm, w->output_norm, w->norm_dtype, d, "output_norm")) return rc;
    if (meta->theta > 0.f)
        if (int rc = upload_rotary_tables(m)) return rc;
    JK_REQUIRE(w->attn_norm && w->attn_qkv && w->attn_o && w->ffn_norm && w->ffn_gate_up && w->ffn_down,
               "create model: a list of layer weights is missing");
    void *status = nullptr;
    if (int rc = device_alloc(m, &status, sizeof(int), "status word")) return rc;
    CUDA_TRY(cudaMemset(status, 0, sizeof(int)), "status word");
    m->env.status = (int *)status;

    const int nq = (nh + 2 * nkvh) * dh;
    m->page_bytes = (size_t)nkvh * m->page_size * dh * 2;
    std::vector<const void *> w_qkv((size_t)L), w_o((size_t)L), w_gate_up((size_t)L), w_down((size_t)L);
    std::vector<const float *> b_qkv((size_t)L, nullptr), norm1((size_t)L), norm2((size_t)L);
    m->k_pages.resize((size_t)L); m->v_pages.resize((size_t)L);
    for (int l = 0; l < L; ++l) {
        if (int rc = upload(m, &w_qkv[l], w->attn_qkv[l], (size_t)nq * d * 2, "attn_qkv")) return rc;
        if (int rc = upload(m, &w_o[l], w->attn_o[l], (size_t)d * nh * dh * 2, "attn_o")) return rc;
        if (int rc = upload(m, &w_gate_up[l], w->ffn_gate_up[l], (size_t)2 * di * d * 2, "ffn_gate_up")) return rc;
        if (int rc = upload(m, &w_down[l], w->ffn_down[l], (size_t)d * di * 2, "ffn_down")) return rc;
        if (int rc = upload_norm(m, &norm1[l], w->attn_norm[l], w->norm_dtype, d, "attn_norm")) return rc;
        if (int rc = upload_norm(m, &norm2[l], w->ffn_norm[l], w->norm_dtype, d, "ffn_norm")) return rc;
        if (w->attn_qkv_b != nullptr && w->attn_qkv_b[l] != nullptr) {
            const void *b = nullptr;
            if (int rc = upload(m, &b, w->attn_qkv_b[l], sizeof(float) * nq, "attn_qkv_b")) return rc;
            b_qkv[l] = (const float *)b;
        }
        const size_t bytes = m->page_bytes * (size_t)m->pool->num_pages();
        if (int rc = device_alloc(m, &m->k_pages[l], bytes, "key pages")) return rc;
        if (int rc = device_alloc(m, &m->v_pages[l], bytes, "value pages")) return rc;
        // Every page starts as zeros.  Page 0 is read by padding rows; what cudaMalloc hands back need not be finite, and
        // no kernel should ever meet such bytes, not even with weight 0.
        CUDA_TRY(cudaMemset(m->k_pages[l], 0, bytes), "key pages");
        CUDA_TRY(cudaMemset(m->v_pages[l], 0, bytes), "value pages");
    }
    build_records(m, w_qkv, b_qkv, w_o, w_gate_up, w_down, norm1, norm2, embedding, lm_head, final_norm);

    // buffers of a step: as many bytes per slot as the records ask for, sized once (captured or not, nothing moves later)
    m->max_requests = m->max_step_tokens;
    long long bytes[RUNNER_SLOTS];
    if (int rc = jk_runner_slot_bytes(&m->env, m->ops.data(), (int)m->ops.size(), m->max_step_tokens, m->max_step_tokens, bytes)) {
        snprintf(jk_error_buffer(), 512, "%s", jk_runner_last_error());
        return rc;
    }
    bytes[SLOT_LOGITS] = 0;       // the logits grow with the batches that ask for many rows (see run_batch)
    for (int s = 0; s < RUNNER_SLOTS; ++s) {
        m->buffers.bytes[s] = bytes[s];
        if (bytes[s] > 0)
            if (int rc = device_alloc(m, &m->buffers.slot[s], (size_t)bytes[s], "a step's buffer")) return rc;
    }
    if (int rc = device_alloc(m, &m->buffers.workspace, WORKSPACE_BYTES, "workspace")) return rc;
    m->buffers.workspace_bytes = WORKSPACE_BYTES;
    m->buffers.sumsq_rows = (int)m->ops.size();
    void *p = nullptr;
    if (int rc = device_alloc(m, &p, sizeof(unsigned long long) * 16 * m->ops.size(), "sums of squares")) return rc;
    m->buffers.sumsq = (unsigned long long *)p;
    m->extra_words = jk::attention_short_rows_capacity(m->max_step_tokens) + jk::attention_tiles_capacity(m->max_step_tokens, m->max_requests);
    m->meta_words = jk::StepLayout(m->max_step_tokens, m->max_requests, 1, m->max_blocks, m->extra_words).total;
    CUDA_TRY(cudaMallocHost((void **)&m->meta_host, sizeof(int) * m->meta_words), "pinned metadata");
    if (int rc = device_alloc(m, &p, sizeof(int) * m->meta_words, "metadata")) return rc; m->meta_dev = (int *)p;
    if (int rc = device_alloc(m, &p, sizeof(int) * 2 * m->max_requests, "sampled ids")) return rc; m->out_dev = (int *)p;
    if (int rc = device_alloc(m, &p, sizeof(float) * 4 * m->max_requests, "sampling parameters")) return rc;
    m->sample_dev = (float *)p;
    CUDA_TRY(cudaDeviceSynchronize(), "create model");
    return JK_OK;
}

int grow(JkModel *m, void **buf, long long *have, long long need, size_t elem, const char *what) {
    if (need <= *have) return JK_OK;
    CUDA_TRY(cudaStreamSynchronize(m->stream), what);
    if (*buf) cudaFree(*buf);
    *buf = nullptr; *have = 0;
    CUDA_TRY(cudaMalloc(buf, (size_t)need * elem), what);
    *have = need;
    return JK_OK;
}

// Pages for every request up to the end of its portion; nothing is taken unless all of them fit.
int reserve_pages(JkModel *m, const uint32_t *req_lens, uint32_t nreq, const uint32_t *req_pos, JkKVCache **caches) {
    long long need = 0;
    for (uint32_t i = 0; i < nreq; ++i) {
        JK_REQUIRE(caches[i] != nullptr, "batch: request %u has no cache", i);
        for (uint32_t j = 0; j < i; ++j) JK_REQUIRE(caches[j] != caches[i], "batch: requests %u and %u share a cache", j, i);
        const long long end = (long long)req_pos[i] + req_lens[i];
        JK_REQUIRE(req_lens[i] > 0, "batch: request %u brings no token", i);
        JK_REQUIRE(end <= m->meta.dctx, "batch: request %u would reach position %lld, the model holds %d", i, end, m->meta.dctx);
        const long long held = (long long)caches[i]->pages.size();
        JK_REQUIRE((long long)req_pos[i] <= held * m->page_size,
                   "batch: request %u starts at position %u but its cache holds %lld tokens' pages", i, req_pos[i],
                   held * m->page_size);
        const long long want = (end + m->page_size - 1) / m->page_size;
        need += std::max(0ll, want - held);
    }
    if (need > (long long)m->pool->available())
        JK_FAIL(JK_UNSUPPORTED, "batch: %lld more cache pages are needed and %d are free; drop a cache or make the pool larger",
                need, m->pool->available());
    for (uint32_t i = 0; i < nreq; ++i) {
        const size_t want = ((size_t)req_pos[i] + req_lens[i] + m->page_size - 1) / m->page_size;
        const size_t held = caches[i]->pages.size();
        if (want > held) {
            caches[i]->pages.resize(want);
            m->pool->alloc((int)(want - held), caches[i]->pages.data() + held);
        }
    }
    return JK_OK;
}

// Runs the batch; the logits of `all_rows ? every row : each request's last row` are left in m->logits.
int run_batch(JkModel *m, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
              const uint32_t *req_pos, JkKVCache **caches, bool all_rows) {
    JK_REQUIRE(m && tokens && req_lens && req_pos && caches, "batch: an argument is missing");
    JK_REQUIRE(nreq > 0 && ntok > 0, "batch: no requests or no tokens");
    JK_REQUIRE((int)ntok <= m->max_step_tokens, "batch: %u tokens in one batch, the model was created for %d", ntok,
               m->max_step_tokens);
    long long sum = 0;
    for (uint32_t i = 0; i < nreq; ++i) sum += req_lens[i];
    JK_REQUIRE(sum == ntok, "batch: the requests' lengths add up to %lld, ntok is %u", sum, ntok);
    for (uint32_t t = 0; t < ntok; ++t)
        JK_REQUIRE(tokens[t] < (uint32_t)m->meta.dvoc, "batch: token %u is outside the vocabulary of %d", tokens[t], m->meta.dvoc);
    CUDA_TRY(cudaSetDevice(m->device), "batch: cudaSetDevice");
    if (int rc = reserve_pages(m, req_lens, nreq, req_pos, caches)) return rc;
    // the pinned buffer is free again: every call ends with a synchronisation of the stream
    const int T = (int)ntok, B = (int)nreq, mb = m->max_blocks;
    const int extra = jk::attention_short_rows_capacity(T) + jk::attention_tiles_capacity(T, B);
    const jk::StepLayout lay(T, B, 1, mb, extra);
    int *h = m->meta_host;
    memset(h, 0, sizeof(int) * lay.total);
    std::vector<int> want, lens(B), starts(B), table((size_t)B * mb, 0);
    int row = 0, longest = 0;
    for (int i = 0; i < B; ++i) {
        lens[i] = (int)req_lens[i]; starts[i] = (int)req_pos[i];
        if (all_rows) for (int t = 0; t < lens[i]; ++t) want.push_back(row + t);
        else want.push_back(row + lens[i] - 1);
        const std::vector<int> &pages = caches[i]->pages;
        for (size_t b = 0; b < pages.size() && (int)b < mb; ++b) table[(size_t)i * mb + b] = pages[b];
        longest = std::max(longest, starts[i] + lens[i]);
        row += lens[i];
    }
    const int *tables[1] = {table.data()};
    jk::pack_step(h, lay, B, B, (const int *)tokens, lens.data(), starts.data(), nullptr, want.data(), (int)want.size(), 1, mb, tables);
    int *short_rows = h + lay.extra, *tiles = short_rows + jk::attention_short_rows_capacity(T);
    const jk::AttentionLists lists = jk::attention_work_lists(B, B, lens.data(), starts.data(), short_rows, tiles);
    CUDA_TRY(cudaMemcpyAsync(m->meta_dev, h, sizeof(int) * lay.total, cudaMemcpyHostToDevice, m->stream), "batch: metadata");

    const int n_want = (int)want.size();
    long long logit_rows = m->logits_rows;
    if (int rc = grow(m, (void **)&m->logits, &logit_rows, n_want, sizeof(float) * m->meta.dvoc, "batch: logits")) return rc;
    m->logits_rows = logit_rows;
    m->buffers.slot[SLOT_LOGITS] = m->logits;
    m->buffers.bytes[SLOT_LOGITS] = (long long)sizeof(float) * m->meta.dvoc * m->logits_rows;

    RunnerStep st{};
    st.ntok = T; st.nreq = B; st.n_want = n_want;
    st.context = jk::context_bucket(longest, m->meta.dctx);
    const int *dv = m->meta_dev;
    st.tokens = dv + lay.tokens; st.positions = dv + lay.positions; st.row_req = dv + lay.row_req;
    st.req_start = dv + lay.req_start; st.req_pos = dv + lay.req_pos; st.want_rows = dv + lay.want_rows;
    st.block_tables[0] = dv + lay.tables[0];
    st.lists[0] = lists.n_short == T ? nullptr : dv + lay.extra;       // every row is a short row: no list is needed
    st.list_n[0] = lists.n_short;
    st.lists[1] = lists.n_tiles ? dv + lay.extra + jk::attention_short_rows_capacity(T) : nullptr;
    st.list_n[1] = lists.n_tiles;
    const int rc = jk_runner_run(&m->env, m->ops.data(), 0, (int)m->ops.size(), &st, &m->buffers, 0, m->stream);
    m->last_launches = jk_runner_launches();
    return rc;
}

// After the stream is idle: did a kernel give up a bounded wait?
int check_status(JkModel *m) {
    if (g_small_fault != nullptr && g_small_fault() > 0)
        JK_FAIL(JK_CUDA_ERROR, "batch: a few-row product gave up the bounded wait for its weights; the results of this batch are invalid");
    int status = 0;
    CUDA_TRY(cudaMemcpy(&status, m->env.status, sizeof(int), cudaMemcpyDeviceToHost), "batch: status word");
    if (status != 0) {
        cudaMemset(m->env.status, 0, sizeof(int));
        if (status == 4)
            JK_FAIL(JK_CUDA_ERROR, "batch: a row's sum of squares is beyond the range of the fixed-point counters; the results "
                                   "of this batch are invalid (JK_NO_FUSED_NORM=1 keeps the norm kernels, which have no such limit)");
        JK_FAIL(JK_CUDA_ERROR, "batch: a tcgen05 kernel gave up a bounded wait (status %d); the results of this batch are invalid", status);
    }
    return JK_OK;
}

}  // namespace

JK_EXPORT const char *jkLastError(void) { return jk_runner_last_error(); }

JK_EXPORT int jkKernelModules(const JkModelMeta *meta, const JkModelOptions *opt, char *out, int size) {
    JK_REQUIRE(meta && out && size > 0, "kernel modules: an argument is missing");
    JkModel probe;
    probe.meta = *meta;
    probe.page_size = opt && opt->page_size ? opt->page_size : 64;
    probe.max_blocks = (meta->dctx + probe.page_size - 1) / probe.page_size;
    int device = 0, sms = 148;
    cudaDeviceProp prop;
    if (cudaGetDevice(&device) == cudaSuccess && cudaGetDeviceProperties(&prop, opt ? opt->device : device) == cudaSuccess)
        sms = prop.multiProcessorCount;
    set_environment(&probe, sms);
    const std::vector<const void *> none((size_t)meta->nlayer, nullptr);
    const std::vector<const float *> nonef((size_t)meta->nlayer, nullptr);
    build_records(&probe, none, nonef, none, none, none, nonef, nonef, nullptr, nullptr, nullptr);
    std::string list = "elementwise,linear_small,attention,sampling,runner";
    if (jk_runner_needs_gemm_tcgen05(&probe.env, probe.ops.data(), (int)probe.ops.size(), opt && opt->max_step_tokens ? opt->max_step_tokens : 2048))
        list += ",gemm_tcgen05";
    if (jk::attention_tcgen05_takes(meta->dh, probe.page_size)) list += ",attention_tcgen05";
    JK_REQUIRE((int)list.size() < size, "kernel modules: the list needs %zu bytes", list.size() + 1);
    snprintf(out, size, "%s", list.c_str());
    return JK_OK;
}

JK_EXPORT JkModel *jkCreateModel(const JkModelMeta *meta, const JkModelWeights *weights, const JkModelOptions *options) {
    JkModel *m = new JkModel();
    if (create(m, meta, weights, options) != JK_OK) {
        const std::string keep = jk_error_buffer();       // the clean-up must not lose the message
        jkDestroyModel(m);
        snprintf(jk_error_buffer(), 512, "%s", keep.c_str());
        return nullptr;
    }
    return m;
}

JK_EXPORT void jkDestroyModel(JkModel *m) {
    if (m == nullptr) return;
    cudaSetDevice(m->device);
    if (m->stream) cudaStreamSynchronize(m->stream);
    for (void *p : m->device_allocs) cudaFree(p);
    if (m->logits) cudaFree(m->logits);
    if (m->meta_host) cudaFreeHost(m->meta_host);
    if (m->stream) cudaStreamDestroy(m->stream);
    // the kernel modules stay loaded: the runner's table still points into them
    delete m->pool;
    delete m;
}

JK_EXPORT JkKVCache *jkCreateKVCache(const JkModel *m) {
    if (m == nullptr) return nullptr;
    return new JkKVCache();
}

JK_EXPORT void jkDropKVCache(const JkModel *m, JkKVCache *c) {
    if (m == nullptr || c == nullptr) return;
    // the page taken last goes back first, so that it is the last of these to be handed out again
    std::vector<int> back(c->pages.rbegin(), c->pages.rend());
    m->pool->free(back.data(), (int)back.size());
    delete c;
}

JK_EXPORT JkKVCache *jkDuplicateKVCache(const JkModel *m, const JkKVCache *src, uint32_t seq_len) {
    if (m == nullptr || src == nullptr) return nullptr;
    const size_t pages = ((size_t)seq_len + m->page_size - 1) / m->page_size;
    char *err = jk_error_buffer();
    if (pages > src->pages.size()) {
        snprintf(err, 512, "duplicate cache: %u tokens asked for, the source holds pages for %zu", seq_len,
                 src->pages.size() * m->page_size);
        return nullptr;
    }
    if ((long long)pages > m->pool->available()) {
        snprintf(err, 512, "duplicate cache: %zu pages needed, %d free", pages, m->pool->available());
        return nullptr;
    }
    cudaSetDevice(m->device);
    JkKVCache *c = new JkKVCache();
    c->pages.resize(pages);
    m->pool->alloc((int)pages, c->pages.data());
    cudaError_t e = cudaSuccess;
    for (size_t l = 0; l < m->k_pages.size(); ++l)
        for (size_t b = 0; b < pages && e == cudaSuccess; ++b) {
            const size_t from = (size_t)src->pages[b] * m->page_bytes, to = (size_t)c->pages[b] * m->page_bytes;
            e = cudaMemcpyAsync((char *)m->k_pages[l] + to, (const char *)m->k_pages[l] + from, m->page_bytes, cudaMemcpyDeviceToDevice,
                                m->stream);
            if (e == cudaSuccess)
                e = cudaMemcpyAsync((char *)m->v_pages[l] + to, (const char *)m->v_pages[l] + from, m->page_bytes,
                                    cudaMemcpyDeviceToDevice, m->stream);
        }
    if (e == cudaSuccess) e = cudaStreamSynchronize(m->stream);
    if (e != cudaSuccess) {
        snprintf(err, 512, "duplicate cache: %s", cudaGetErrorString(e));
        jkDropKVCache(m, c);
        return nullptr;
    }
    return c;
}

JK_EXPORT int jkForwardBatch(JkModel *m, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
                             const uint32_t *req_pos, JkKVCache **caches, float *logits) {
    JK_REQUIRE(logits != nullptr, "forward batch: no place for the logits");
    if (int rc = run_batch(m, tokens, ntok, req_lens, nreq, req_pos, caches, true)) return rc;
    CUDA_TRY(cudaMemcpyAsync(logits, m->logits, sizeof(float) * (size_t)ntok * m->meta.dvoc, cudaMemcpyDeviceToHost, m->stream),
             "forward batch: logits");
    CUDA_TRY(cudaStreamSynchronize(m->stream), "forward batch");
    return check_status(m);
}

JK_EXPORT int jkInferBatch(JkModel *m, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
                           const uint32_t *req_pos, JkKVCache **caches, const float *temperature, const uint32_t *topk,
                           const float *topp, const uint64_t *seeds, uint32_t *output) {
    JK_REQUIRE(output != nullptr, "infer batch: no place for the tokens");
    if (int rc = run_batch(m, tokens, ntok, req_lens, nreq, req_pos, caches, false)) return rc;
    const RunnerFns *fns = jk_runner_fns();
    const int B = (int)nreq, V = m->meta.dvoc;
    JK_REQUIRE(B <= m->max_requests, "infer batch: %d requests, the model was created for %d", B, m->max_requests);
    std::vector<char> greedy(B);
    bool any_random = false;
    for (int i = 0; i < B; ++i) {
        greedy[i] = temperature == nullptr || temperature[i] <= 0.f || (topk != nullptr && topk[i] == 1);
        any_random = any_random || !greedy[i];
    }
    // ids of the largest logits in out_dev[0, B), drawn ids in out_dev[B, 2B)
    if (fns->argmax(m->logits, V, B, V, m->out_dev, nullptr, m->stream))
        JK_FAIL(JK_CUDA_ERROR, "infer batch: %s", fns->err_sampling ? fns->err_sampling() : "argmax failed");
    if (any_random) {
        std::vector<float> par(4 * (size_t)B, 0.f);       // temperature, top-k (as int), top-p, uniform number
        for (int i = 0; i < B; ++i) {
            par[i] = greedy[i] ? 1.f : temperature[i];
            const int k = topk ? (int)topk[i] : 0;
            memcpy(&par[B + i], &k, 4);
            par[2 * B + i] = topp ? topp[i] : 1.f;
            par[3 * B + i] = jk::uniform_for(seeds ? seeds[i] : 0, (uint64_t)req_pos[i] + req_lens[i]);
        }
        // the copy reads pageable memory: it has finished with `par` when it returns
        CUDA_TRY(cudaMemcpyAsync(m->sample_dev, par.data(), sizeof(float) * par.size(), cudaMemcpyHostToDevice, m->stream),
                 "infer batch: sampling parameters");
        if (fns->sample(m->logits, V, B, V, m->sample_dev, (const int *)(m->sample_dev + B), m->sample_dev + 2 * B,
                        m->sample_dev + 3 * B, m->out_dev + B, m->stream))
            JK_FAIL(JK_CUDA_ERROR, "infer batch: %s", fns->err_sampling ? fns->err_sampling() : "sampling failed");
    }
    std::vector<int> ids(2 * (size_t)B, 0);
    CUDA_TRY(cudaMemcpyAsync(ids.data(), m->out_dev, sizeof(int) * (any_random ? 2 : 1) * B, cudaMemcpyDeviceToHost, m->stream),
             "infer batch: ids");
    CUDA_TRY(cudaStreamSynchronize(m->stream), "infer batch");
    for (int i = 0; i < B; ++i) output[i] = (uint32_t)(greedy[i] ? ids[i] : ids[B + i]);
    return check_status(m);
}

JK_EXPORT int64_t jkFreePages(const JkModel *m) { return m && m->pool ? (int64_t)m->pool->available() : 0; }
JK_EXPORT int32_t jkLastLaunches(const JkModel *m) { return m ? m->last_launches : 0; }
