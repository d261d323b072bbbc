// The C interface of model_api.h on top of the native runner: weights and cache pages on the device,
// a page pool with per-request page lists, the packing of a batch's metadata, and sampling.
//
// It is the same step as the Python engine's: jk_runner_forward runs the kernels, this file only decides
// which pages a request holds and describes the batch.  (The reference's counterpart is
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

constexpr int TILE_ROWS = 128;      // rows of a query tile of the prefill attention kernels
constexpr int SHORT_ROWS = 8;       // a request with at most this many rows goes to the decode kernel
constexpr long long WORKSPACE_BYTES = 32ll << 20;

int align4(int n) { return (n + 3) & ~3; }

// Where each array of a step's metadata lies in the one buffer that is copied per step.
struct MetaLayout {
    int tokens, positions, row_req, req_start, req_pos, want_rows, short_rows, tiles, block_table, total;
    MetaLayout(int T, int B, int max_blocks) {
        int o = 0;
        tokens = o; o += align4(T);
        positions = o; o += align4(T);
        row_req = o; o += align4(T);
        req_start = o; o += align4(B + 1);
        req_pos = o; o += align4(B);
        want_rows = o; o += align4(T);
        short_rows = o; o += align4(T);
        tiles = o; o += align4(2 * (T / TILE_ROWS + B));
        block_table = o; o += align4(B * max_blocks);
        total = o;
    }
};

}  // namespace

struct JkKVCache {
    std::vector<int> pages;
};

struct JkModel {
    JkModelMeta meta{};
    int device = 0, page_size = 64, max_step_tokens = 2048, max_blocks = 0, max_requests = 0;
    long long num_pages = 0;
    RunnerModel rm{};
    std::vector<RunnerLayer> layers;
    RunnerScratch scratch{};
    std::vector<void *> device_allocs;
    mutable std::vector<int> free_pages;         // page 0 is never handed out: padding rows write there
    cudaStream_t stream = nullptr;
    int *meta_host = nullptr, *meta_dev = nullptr;
    int meta_words = 0;
    float *logits = nullptr;
    long long logits_rows = 0;
    float *decode_scratch = nullptr;
    long long decode_floats = 0;
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

// Angle of pair j at position p: p / theta^(j / half), computed in double and rounded once.
int upload_rotary_tables(JkModel *m) {
    const int half = m->meta.dh / 2, P = m->meta.dctx;
    std::vector<float> c((size_t)P * half), s((size_t)P * half);
    std::vector<double> inv(half);
    for (int j = 0; j < half; ++j) inv[j] = std::pow((double)m->meta.theta, -((double)j / half));
    for (int p = 0; p < P; ++p)
        for (int j = 0; j < half; ++j) {
            const double a = (double)p * inv[j];
            c[(size_t)p * half + j] = (float)std::cos(a);
            s[(size_t)p * half + j] = (float)std::sin(a);
        }
    const void *pc = nullptr, *ps = nullptr;
    if (int rc = upload(m, &pc, c.data(), c.size() * sizeof(float), "the cosine table")) return rc;
    if (int rc = upload(m, &ps, s.data(), s.size() * sizeof(float), "the sine table")) return rc;
    m->rm.cos_table = (const float *)pc;
    m->rm.sin_table = (const float *)ps;
    return JK_OK;
}

// The kernel modules by name from a folder, for a program that has no Python around it.
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

bool takes_tcgen05(const RunnerModel &m, int rows, int n, int k) {
    return runner_takes_tcgen05(m.sms, m.tcgen05_min_rows, m.tcgen05_min_tiles, m.tcgen05_min_fill_pct, rows, n, k);
}

// The gemm_tcgen05 module is loaded if a step can reach one of its kernels: the tiled one under the runner's
// routing, or the few-rows one (a block for every SM).
bool needs_gemm_tcgen05(const RunnerModel &rm, int max_step_tokens) {
    const int nq = (rm.heads + 2 * rm.kv_heads) * rm.head_dim;
    const int products[5][3] = {{nq, rm.hidden, RUNNER_F32}, {rm.hidden, rm.heads * rm.head_dim, RUNNER_RESIDUAL},
                                {rm.intermediate, rm.hidden, RUNNER_SWIGLU}, {rm.hidden, rm.intermediate, RUNNER_RESIDUAL},
                                {rm.vocab, rm.hidden, RUNNER_F32}};
    const long long need = rm.skinny_min_blocks > 0 ? rm.skinny_min_blocks : rm.sms;
    for (auto &p : products) {
        if (takes_tcgen05(rm, max_step_tokens, p[2] == RUNNER_SWIGLU ? 2 * p[0] : p[0], p[1])) return true;
        if (p[1] % 8 == 0 && runner_skinny_blocks(rm.sms, p[0], p[1], p[2]) >= need) return true;
    }
    return false;
}

bool tcgen05_attention_takes(int dh, int page) {
    return (dh == 64 || dh == 128) && (page == 8 || page == 16 || page == 32 || page == 64 || page == 128);
}

// How many ways the decode kernels cut each row's key range (the same rule as kernels.attention_decode_splits of
// the Python side).  Head sizes 64 and 128, the tensor-core kernel: as many cuts as make the blocks fill the SMs once
// (two blocks an SM, rounded) as long as a block keeps 256 keys, then up to two rounds of blocks as long as it keeps 1024.  Other
// head sizes: full waves of blocks (three an SM) against a block's fixed cost of about 128 keys' worth of time.
int decode_splits(int nrows, int nkvh, int group, int max_positions, int sms, int dh) {
    const int keys = std::max(1, max_positions / 2);
    if (dh == 64 || dh == 128) {
        const long long blocks = std::max(1, nrows * nkvh * ((group + 15) / 16));
        const long long slots = 2LL * sms;
        long long s = std::max(1LL, std::min({(2 * slots + blocks) / (2 * blocks), (long long)keys / 256, 32LL}));      // slots / blocks, rounded
        while (blocks * (s + 1) <= 2 * slots && keys / (s + 1) >= 1024 && s < 32) ++s;
        return (int)s;
    }
    const long long blocks = std::max(1, nrows * nkvh * (group > 4 ? (group + 3) / 4 : 1));
    const long long slots = (long long)sms * 3;
    int best = 1;
    double best_cost = -1;
    for (int s = 1; s <= 32; ++s) {
        if (s > 1 && (double)keys / s < 64) break;
        const long long waves = (blocks * s + slots - 1) / slots;
        const double cost = waves * (128 + (double)keys / s);
        if (best_cost < 0 || cost < best_cost * 0.97) best = s, best_cost = cost;
    }
    return best;
}

float uniform_for(uint64_t seed, uint64_t index) {      // the splitmix64 finaliser, top 24 bits
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + (index + 1) * 0xBF58476D1CE4E5B9ull;
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) / (float)(1 << 24);
}

int create(JkModel *m, const JkModelMeta *meta, const JkModelWeights *w, const JkModelOptions *opt) {
    JK_REQUIRE(meta && w, "create model: meta or weights missing");
    m->meta = *meta;
    const int L = meta->nlayer, d = meta->d, nh = meta->nh, nkvh = meta->nkvh, dh = meta->dh, di = meta->di, V = meta->dvoc;
    JK_REQUIRE(L > 0 && d > 0 && nh > 0 && nkvh > 0 && dh > 0 && di > 0 && V > 0 && meta->dctx > 0,
               "create model: a size is not positive");
    JK_REQUIRE(nh % nkvh == 0, "create model: %d heads do not divide into %d key/value heads", nh, nkvh);
    JK_REQUIRE(d % 32 == 0 && di % 32 == 0 && (nh * dh) % 32 == 0 && dh % 16 == 0 && dh <= 256,
               "create model: width %d, feed-forward width %d and head size %d must be multiples of 32, 32 and 16 "
               "(head size at most 256) for the kernels of this interface", d, di, dh);
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

    RunnerModel &rm = m->rm;
    rm.layers = L; rm.hidden = d; rm.heads = nh; rm.kv_heads = nkvh; rm.head_dim = dh; rm.intermediate = di; rm.vocab = V;
    rm.page_size = m->page_size;
    m->max_blocks = (meta->dctx + m->page_size - 1) / m->page_size;
    rm.max_blocks = m->max_blocks;
    m->num_pages = (cache_tokens + m->page_size - 1) / m->page_size;
    rm.num_pages = (int)m->num_pages + 1;
    rm.window = 0;
    rm.sms = prop.multiProcessorCount;
    rm.tcgen05_min_rows = 129;       // the routing's measured thresholds: see runner_takes_tcgen05
    rm.tcgen05_min_tiles = 200;
    rm.tcgen05_min_fill_pct = 80;
    rm.attention_tcgen05 = tcgen05_attention_takes(dh, m->page_size);
    rm.fused_norms = getenv("JK_NO_FUSED_NORM") == nullptr || getenv("JK_NO_FUSED_NORM")[0] != '1';
    rm.embed_dtype = JK_BF16;
    rm.embed_scale = meta->embed_scale; rm.residual_scale = meta->residual_scale; rm.logit_scale = meta->logit_scale;
    rm.softmax_scale = 1.f / std::sqrt((float)dh);
    rm.final_eps = meta->epsilon;

    // the kernels
    const int nq = (nh + 2 * nkvh) * dh;
    const bool need_gemm = needs_gemm_tcgen05(rm, m->max_step_tokens);
    if (opt && opt->kernel_dir) {
        if (int rc = bind_from_directory(m, opt->kernel_dir, need_gemm, rm.attention_tcgen05 != 0)) return rc;
    }
    const RunnerFns *fns = jk_runner_fns();
    JK_REQUIRE(fns != nullptr, "create model: no kernels are bound; give kernel_dir or call jk_runner_bind first");
    JK_REQUIRE(fns->argmax && fns->sample, "create model: the bound kernels lack the sampling entry points");
    JK_REQUIRE(!need_gemm || fns->gemm_tcgen05, "create model: steps of %d tokens need the tcgen05 product, which is not bound",
               m->max_step_tokens);
    JK_REQUIRE(!rm.attention_tcgen05 || fns->attention_tcgen05, "create model: the tcgen05 attention kernel is not bound");

    // weights
    if (int rc = upload(m, &rm.embedding, w->input_embd, (size_t)V * d * 2, "input_embd")) return rc;
    if (w->output_embd == w->input_embd || w->output_embd == nullptr) rm.lm_head = rm.embedding;
    else if (int rc = upload(m, &rm.lm_head, w->output_embd, (size_t)V * d * 2, "output_embd")) return rc;
    if (int rc = upload_norm(m, &rm.final_norm, w->output_norm, w->norm_dtype, d, "output_norm")) return rc;
    if (meta->theta > 0.f)
        if (int rc = upload_rotary_tables(m)) return rc;
    JK_REQUIRE(w->attn_norm && w->attn_qkv && w->attn_o && w->ffn_norm && w->ffn_gate_up && w->ffn_down,
               "create model: a list of layer weights is missing");
    void *status = nullptr;
    if (int rc = device_alloc(m, &status, sizeof(int), "status word")) return rc;
    CUDA_TRY(cudaMemset(status, 0, sizeof(int)), "status word");
    rm.status = (int *)status;

    m->page_bytes = (size_t)nkvh * m->page_size * dh * 2;
    m->layers.resize(L);
    for (int l = 0; l < L; ++l) {
        RunnerLayer &y = m->layers[l];
        if (int rc = upload(m, &y.w_qkv, w->attn_qkv[l], (size_t)nq * d * 2, "attn_qkv")) return rc;
        if (int rc = upload(m, &y.w_o, w->attn_o[l], (size_t)d * nh * dh * 2, "attn_o")) return rc;
        if (int rc = upload(m, &y.w_gate_up, w->ffn_gate_up[l], (size_t)2 * di * d * 2, "ffn_gate_up")) return rc;
        if (int rc = upload(m, &y.w_down, w->ffn_down[l], (size_t)d * di * 2, "ffn_down")) return rc;
        if (int rc = upload_norm(m, &y.norm1, w->attn_norm[l], w->norm_dtype, d, "attn_norm")) return rc;
        if (int rc = upload_norm(m, &y.norm2, w->ffn_norm[l], w->norm_dtype, d, "ffn_norm")) return rc;
        y.eps1 = y.eps2 = meta->epsilon;
        const size_t bytes = m->page_bytes * (size_t)rm.num_pages;
        if (int rc = device_alloc(m, &y.k_pages, bytes, "key pages")) return rc;
        if (int rc = device_alloc(m, &y.v_pages, bytes, "value pages")) return rc;
        // Every page starts as zeros.  Page 0 is read by padding rows; of the others a kernel that loads whole pages
        // (the tcgen05 attention, by TMA) also reads the slots beyond a request's last position, with weight 0 in
        // the P V product: what lies there must be finite, and memory that cudaMalloc hands back need not be.
        CUDA_TRY(cudaMemset(y.k_pages, 0, bytes), "key pages");
        CUDA_TRY(cudaMemset(y.v_pages, 0, bytes), "value pages");
    }
    m->free_pages.reserve(m->num_pages);
    for (long long p = m->num_pages; p >= 1; --p) m->free_pages.push_back((int)p);      // low pages go out first

    // buffers of a step
    const size_t T = m->max_step_tokens;
    RunnerScratch &s = m->scratch;
    void *p = nullptr;
    if (int rc = device_alloc(m, &p, T * d * 4, "x")) return rc; s.x = (float *)p;
    if (int rc = device_alloc(m, &s.h, T * d * 2, "h")) return rc;
    if (int rc = device_alloc(m, &p, T * nq * 4, "qkv")) return rc; s.qkv = (float *)p;
    if (int rc = device_alloc(m, &s.q, T * nh * dh * 2, "q")) return rc;
    if (int rc = device_alloc(m, &s.o, T * nh * dh * 2, "o")) return rc;
    if (int rc = device_alloc(m, &p, T * d * 4, "delta")) return rc; s.delta = (float *)p;
    if (int rc = device_alloc(m, &p, T * 2 * di * 4, "gate_up")) return rc; s.gate_up = (float *)p;
    if (int rc = device_alloc(m, &s.act, T * di * 2, "act")) return rc;
    if (int rc = device_alloc(m, &s.hw, T * d * 2, "hw")) return rc;
    if (int rc = device_alloc(m, &s.workspace, WORKSPACE_BYTES, "workspace")) return rc;
    s.workspace_bytes = WORKSPACE_BYTES;
    if (int rc = device_alloc(m, &p, sizeof(unsigned long long) * 2 * L * 16, "sums of squares")) return rc;
    s.sumsq = (unsigned long long *)p;
    m->max_requests = m->max_step_tokens;
    m->meta_words = MetaLayout(m->max_step_tokens, m->max_requests, m->max_blocks).total;
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
    if (need > (long long)m->free_pages.size())
        JK_FAIL(JK_UNSUPPORTED, "batch: %lld more cache pages are needed and %zu are free; drop a cache or make the pool larger",
                need, m->free_pages.size());
    for (uint32_t i = 0; i < nreq; ++i) {
        const size_t want = ((size_t)req_pos[i] + req_lens[i] + m->page_size - 1) / m->page_size;
        while (caches[i]->pages.size() < want) {
            caches[i]->pages.push_back(m->free_pages.back());
            m->free_pages.pop_back();
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
    CUDA_TRY(cudaSetDevice(m->device), "batch: cudaSetDevice");
    if (int rc = reserve_pages(m, req_lens, nreq, req_pos, caches)) return rc;
    // the pinned buffer is free again: every call ends with a synchronisation of the stream
    const int T = (int)ntok, B = (int)nreq, mb = m->max_blocks;
    const MetaLayout lay(T, B, mb);
    int *h = m->meta_host;
    memset(h, 0, sizeof(int) * lay.total);
    int row = 0, n_short = 0, n_want = 0, max_end = 0;
    struct Tile { int keys, req, row; };
    std::vector<Tile> tiles;
    for (int i = 0; i < B; ++i) {
        const int n = (int)req_lens[i], s = (int)req_pos[i];
        h[lay.req_start + i] = row;
        h[lay.req_pos + i] = s;
        for (int t = 0; t < n; ++t) {
            JK_REQUIRE(tokens[row + t] < (uint32_t)m->meta.dvoc, "batch: token %u is outside the vocabulary of %d", tokens[row + t],
                       m->meta.dvoc);
            h[lay.tokens + row + t] = (int)tokens[row + t];
            h[lay.positions + row + t] = s + t;
            h[lay.row_req + row + t] = i;
            if (all_rows) h[lay.want_rows + n_want++] = row + t;
        }
        if (!all_rows) h[lay.want_rows + n_want++] = row + n - 1;
        if (n <= SHORT_ROWS)
            for (int t = 0; t < n; ++t) h[lay.short_rows + n_short++] = row + t;
        else
            for (int t0 = 0; t0 < n; t0 += TILE_ROWS) tiles.push_back({s + t0, i, row + t0});
        const std::vector<int> &pages = caches[i]->pages;
        for (size_t b = 0; b < pages.size() && (int)b < mb; ++b) h[lay.block_table + i * mb + (int)b] = pages[b];
        max_end = std::max(max_end, s + n);
        row += n;
    }
    h[lay.req_start + B] = row;
    // the attention kernels start tiles in the order of the list: those that see the most keys first
    std::stable_sort(tiles.begin(), tiles.end(), [](const Tile &a, const Tile &b) { return a.keys > b.keys; });
    for (size_t t = 0; t < tiles.size(); ++t) {
        h[lay.tiles + 2 * (int)t] = tiles[t].req;
        h[lay.tiles + 2 * (int)t + 1] = tiles[t].row;
    }
    CUDA_TRY(cudaMemcpyAsync(m->meta_dev, h, sizeof(int) * lay.total, cudaMemcpyHostToDevice, m->stream), "batch: metadata");

    int splits = 1;
    if (n_short) {
        splits = decode_splits(n_short, m->meta.nkvh, m->meta.nh / m->meta.nkvh, m->meta.dctx, m->rm.sms, m->meta.dh);
        const long long need = splits > 1 ? (long long)n_short * m->meta.nh * splits * (m->meta.dh + 2) : 0;
        if (int rc = grow(m, (void **)&m->decode_scratch, &m->decode_floats, need, sizeof(float), "batch: attention scratch")) return rc;
        m->scratch.decode_scratch = m->decode_scratch;
    }
    long long logit_rows = m->logits_rows;
    if (int rc = grow(m, (void **)&m->logits, &logit_rows, n_want, sizeof(float) * m->meta.dvoc, "batch: logits")) return rc;
    m->logits_rows = logit_rows;

    RunnerStep st{};
    st.ntok = T; st.nreq = B; st.n_want = n_want; st.n_tiles = (int)tiles.size(); st.n_short = n_short; st.splits = splits;
    const int *dv = m->meta_dev;
    st.tokens = dv + lay.tokens; st.positions = dv + lay.positions; st.row_req = dv + lay.row_req;
    st.req_start = dv + lay.req_start; st.req_pos = dv + lay.req_pos; st.want_rows = dv + lay.want_rows;
    st.short_rows = n_short == T ? nullptr : dv + lay.short_rows;
    st.tiles = tiles.empty() ? nullptr : dv + lay.tiles;
    st.block_table = dv + lay.block_table;
    st.logits = m->logits;
    const int rc = jk_runner_forward(&m->rm, m->layers.data(), &st, &m->scratch, m->stream);
    m->last_launches = jk_runner_launches();
    return rc;
}

// After the stream is idle: did a kernel give up a bounded wait?
int check_status(JkModel *m) {
    int status = 0;
    CUDA_TRY(cudaMemcpy(&status, m->rm.status, sizeof(int), cudaMemcpyDeviceToHost), "batch: status word");
    if (status != 0) {
        cudaMemset(m->rm.status, 0, sizeof(int));
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
    RunnerModel rm{};
    rm.hidden = meta->d; rm.heads = meta->nh; rm.kv_heads = meta->nkvh; rm.head_dim = meta->dh; rm.intermediate = meta->di;
    rm.vocab = meta->dvoc;
    rm.sms = 148; rm.tcgen05_min_rows = 129; rm.tcgen05_min_tiles = 200; rm.tcgen05_min_fill_pct = 80;
    int device = 0;
    cudaDeviceProp prop;
    if (cudaGetDevice(&device) == cudaSuccess && cudaGetDeviceProperties(&prop, opt ? opt->device : device) == cudaSuccess)
        rm.sms = prop.multiProcessorCount;
    std::string list = "elementwise,linear_small,attention,sampling,runner";
    if (needs_gemm_tcgen05(rm, opt && opt->max_step_tokens ? opt->max_step_tokens : 2048)) list += ",gemm_tcgen05";
    if (tcgen05_attention_takes(meta->dh, opt && opt->page_size ? opt->page_size : 64)) list += ",attention_tcgen05";
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
    if (m->decode_scratch) cudaFree(m->decode_scratch);
    if (m->meta_host) cudaFreeHost(m->meta_host);
    if (m->stream) cudaStreamDestroy(m->stream);
    // the kernel modules stay loaded: the runner's table still points into them
    delete m;
}

JK_EXPORT JkKVCache *jkCreateKVCache(const JkModel *m) {
    if (m == nullptr) return nullptr;
    return new JkKVCache();
}

JK_EXPORT void jkDropKVCache(const JkModel *m, JkKVCache *c) {
    if (m == nullptr || c == nullptr) return;
    for (auto it = c->pages.rbegin(); it != c->pages.rend(); ++it) m->free_pages.push_back(*it);
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
    if (pages > m->free_pages.size()) {
        snprintf(err, 512, "duplicate cache: %zu pages needed, %zu free", pages, m->free_pages.size());
        return nullptr;
    }
    cudaSetDevice(m->device);
    JkKVCache *c = new JkKVCache();
    for (size_t b = 0; b < pages; ++b) {
        c->pages.push_back(m->free_pages.back());
        m->free_pages.pop_back();
    }
    cudaError_t e = cudaSuccess;
    for (const RunnerLayer &y : m->layers)
        for (size_t b = 0; b < pages && e == cudaSuccess; ++b) {
            const size_t from = (size_t)src->pages[b] * m->page_bytes, to = (size_t)c->pages[b] * m->page_bytes;
            e = cudaMemcpyAsync((char *)y.k_pages + to, (const char *)y.k_pages + from, m->page_bytes, cudaMemcpyDeviceToDevice, m->stream);
            if (e == cudaSuccess)
                e = cudaMemcpyAsync((char *)y.v_pages + to, (const char *)y.v_pages + from, m->page_bytes, cudaMemcpyDeviceToDevice,
                                    m->stream);
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
            par[3 * B + i] = uniform_for(seeds ? seeds[i] : 0, (uint64_t)req_pos[i] + req_lens[i]);
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

JK_EXPORT int64_t jkFreePages(const JkModel *m) { return m ? (int64_t)m->free_pages.size() : 0; }
JK_EXPORT int32_t jkLastLaunches(const JkModel *m) { return m ? m->last_launches : 0; }
