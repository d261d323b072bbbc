// The native step: replays a model's launch records (runner.h) for one batch.
//
// One call launches every kernel of a run of records (for the standard stack: the whole step, embedding to logits)
// where Python would make a dozen calls a layer.  Which kernel runs a record is decided here and nowhere else:
//
//   float32       every product on the CUDA cores (gemm_f32, no tensor cores), attention by the row kernel
//   bfloat16      products by the rules of host_rules.h (jk::product_route):
//                   rows <= 16          the weight-streaming kernels of linear_small.cu (q/k/v with rotation and cache
//                                       write in the epilogue, gate/up with SwiGLU in the epilogue)
//                   few rows, wide      the tcgen05 kernel with the weights on the MMA's M side (gemm_skinny.cu)
//                   many rows, wide     the tiled tcgen05 kernel (q/k/v epilogue, SwiGLU epilogue, residual add by TMA)
//                   else                cuBLAS, bfloat16 operands, float32 accumulation and output, with the rotary
//                                       kernel, the SwiGLU kernel and the fused add + norm kernel around it
//                 attention: tiles of requests with many rows -> attention_tcgen05 (or the mma.sync kernel);
//                            rows of requests with few rows -> the split-key decode kernel
//   steps of at most 16 rows run without norm kernels where three records in a row allow it (a product that adds into
//   the stream, a norm, the product after it): see fuse_norm below.
//
// The kernels live in their own shared objects; the caller hands their entry points over once (jk_runner_bind).
// Nothing is allocated here.
#include "common.cuh"
#include "runner.h"

#include <cublas_v2.h>
#include <mutex>

JK_DEFINE_ERROR_BUFFER(jk_runner)

static RunnerFns g_fns = {};
static bool g_bound = false;
JK_EXPORT const RunnerFns *jk_runner_fns() { return g_bound ? &g_fns : nullptr; }

JK_EXPORT int jk_runner_bind(const RunnerFns *fns) {
    JK_REQUIRE(fns != nullptr, "runner_bind: no table");
    // a table adds to what is bound already (two users of this library in one process may need different modules): an
    // entry that this caller leaves empty keeps what an earlier caller gave
    static_assert(sizeof(RunnerFns) % sizeof(void *) == 0, "the table is a list of pointers");
    void *const *from = (void *const *)fns;
    void **to = (void **)&g_fns;
    for (size_t i = 0; i < sizeof(RunnerFns) / sizeof(void *); ++i)
        if (from[i] != nullptr) to[i] = from[i];
    // the tcgen05 modules may be left out by a caller whose model or step size never reaches them (they are then not
    // even compiled); everything else is needed by every model
    const RunnerFns &f = g_fns;
    JK_REQUIRE(f.embed && f.add_rmsnorm && f.residual_add && f.swiglu && f.rope_kv && f.gemm_f32 && f.linear_small &&
               f.linear_small_qkv && f.linear_small_supports && f.linear_small_qkv_supports && f.linear_small_norm_supports &&
               f.linear_small_norm && f.linear_small_qkv_norm && f.attention_rows && f.attention_decode && f.attention_prefill &&
               f.attention_prefill_supports && f.err_elementwise && f.err_linear_small && f.err_attention,
               "runner_bind: an entry that every model needs is empty");
    JK_REQUIRE((f.gemm_tcgen05 != nullptr) == (f.gemm_tcgen05_qkv != nullptr) && (f.gemm_tcgen05 != nullptr) == (f.gemm_skinny != nullptr) &&
               (f.gemm_tcgen05 != nullptr) == (f.err_gemm_tcgen05 != nullptr) &&
               (f.attention_tcgen05 != nullptr) == (f.err_attention_tcgen05 != nullptr),
               "runner_bind: a module's entries come together");
    g_bound = true;
    return JK_OK;
}

static int g_launches = 0;      // kernels launched by the last jk_runner_run (the library's count as one each)
JK_EXPORT int jk_runner_launches() { return g_launches; }

#define RUN(module, call)                                                                                   \
    do {                                                                                                    \
        ++g_launches;                                                                                       \
        if (int rc_ = (call)) {                                                                             \
            snprintf(jk_error_buffer(), 512, "%s", g_fns.err_##module());                                   \
            return rc_;                                                                                     \
        }                                                                                                   \
    } while (0)

// ---- the library product: out[M, N] (float32) = act[M, K] * w[N, K]^T, bfloat16 operands --------------------
// cublasGemmEx with the library's own choice of kernel (it splits K for narrow outputs by itself), float32
// accumulation; the handle works in the caller's workspace so that nothing is allocated inside a capture.
static cublasHandle_t g_blas = nullptr;
static std::mutex g_blas_mutex;

static int lt_product(const void *act, const void *w, float *out, int M, int N, int K, const RunnerBuffers &b, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_blas_mutex);
    if (!g_blas && cublasCreate(&g_blas) != CUBLAS_STATUS_SUCCESS) JK_FAIL(JK_CUDA_ERROR, "runner: cublasCreate failed");
    JK_REQUIRE(b.workspace != nullptr && b.workspace_bytes > 0, "runner: the library's product needs a workspace");
    if (cublasSetStream(g_blas, stream) != CUBLAS_STATUS_SUCCESS ||
        cublasSetWorkspace(g_blas, b.workspace, (size_t)b.workspace_bytes) != CUBLAS_STATUS_SUCCESS)
        JK_FAIL(JK_CUDA_ERROR, "runner: the library refused the stream or the workspace");
    // row-major out[M, N] is column-major [N, M] = W^T (op T on the column-major [K, N]) * act (column-major [K, M])
    const float one = 1.f, zero = 0.f;
    ++g_launches;
    const cublasStatus_t st = cublasGemmEx(g_blas, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &one, w, CUDA_R_16BF, K, act, CUDA_R_16BF, K,
                                           &zero, out, CUDA_R_32F, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    if (st != CUBLAS_STATUS_SUCCESS) JK_FAIL(JK_CUDA_ERROR, "runner: the library's product of %d x %d x %d failed with %d", M, N, K, (int)st);
    return JK_OK;
}

namespace {

struct Run {
    const RunnerEnv &env;
    const RunnerStep &st;
    const RunnerBuffers &buf;
    cudaStream_t stream;
    bool pending = false;         // SLOT_DELTA holds a product that has not been added to the stream yet
    float pending_scale = 1.f;

    int elem() const { return env.dtype == JK_F32 ? 4 : 2; }
    bool tcgen05_bound() const { return g_fns.gemm_tcgen05 != nullptr; }
    jk::Route route(int rows, int n, int k, int kind) const {
        return jk::product_route(env.routing, rows, n, k, kind, g_fns.linear_small_supports(rows, n, k) != 0, tcgen05_bound());
    }
    // the slot's address, after a check that it holds `need` bytes
    int slot(int which, long long need, void **out, const char *what) const {
        JK_REQUIRE(which >= 0 && which < RUNNER_SLOTS && buf.slot[which] != nullptr, "runner: %s: slot %d is not there", what, which);
        JK_REQUIRE(need <= buf.bytes[which], "runner: %s needs %lld bytes in slot %d, which holds %lld", what, need, which, buf.bytes[which]);
        *out = buf.slot[which];
        return JK_OK;
    }
    float *x() const { return (float *)buf.slot[SLOT_X]; }
    float *delta() const { return (float *)buf.slot[SLOT_DELTA]; }
};

// out (float32 [rows, n]) = act * w^T (+ bias) by whichever kernel takes `rows`
int product_f32(Run &r, const void *act, const void *w, const float *bias, float *out, int rows, int n, int k) {
    if (r.env.dtype == JK_F32) {
        RUN(elementwise, g_fns.gemm_f32((const float *)act, k, (const float *)w, k, bias, out, n, rows, n, k, r.stream));
        return JK_OK;
    }
    // a bias outside q/k/v (whose bias the rotary kernel adds) does not occur in this architecture; no kernel adds one
    JK_REQUIRE(bias == nullptr, "runner: a bfloat16 product with a bias outside q/k/v is not built");
    const jk::Routing &ro = r.env.routing;
    switch (r.route(rows, n, k, jk::PRODUCT_F32)) {
        case jk::ROUTE_SMALL:
            RUN(linear_small, g_fns.linear_small(act, w, out, rows, n, k, n, 0, ro.sms, r.stream));
            break;
        case jk::ROUTE_SKINNY:
            RUN(gemm_tcgen05, g_fns.gemm_skinny(act, w, out, rows, n, k, n, 0, 1.f, r.env.status, ro.sms, r.stream));
            break;
        case jk::ROUTE_TCGEN05:
            RUN(gemm_tcgen05, g_fns.gemm_tcgen05(act, w, out, rows, n, k, n, 0, 1.f, r.env.status, ro.sms, r.stream));
            break;
        default:
            if (int rc = lt_product(act, w, out, rows, n, k, r.buf, r.stream)) return rc;
    }
    return JK_OK;
}

int flush_pending(Run &r, int T, int hidden) {
    if (!r.pending) return JK_OK;
    RUN(elementwise, g_fns.residual_add(r.x(), r.delta(), JK_F32, r.pending_scale, (long long)T * hidden, r.stream));
    r.pending = false;
    return JK_OK;
}

// Steps of few rows without norm kernels: three records in a row -- a product that adds into the stream, a norm over
// every row with factor 1, and a gate/up or q/k/v product that reads the norm's output -- run as two kernels.  The first
// adds itself into the float32 stream, writes bfloat16(x * norm weight) as the next product's activations and its
// tile's share of sum(x^2) per row into counters; the second multiplies its rows by 1 / sqrt(sum / width + eps) before
// its own epilogue.  The sums and the scaling are float32; what changes against the norm kernel is where the activations
// are rounded to bfloat16 (before the 1 / rms instead of after).
struct FusedNorm {
    const RunnerOp *norm = nullptr;       // the norm that the last residual product took over
    unsigned long long *sumsq = nullptr;
};

bool small_residual_ok(const Run &r, const RunnerOp &op, int T) {
    return r.env.dtype == JK_BF16 && r.env.fused_norms && T <= 16 && r.buf.sumsq != nullptr && op.out_slot == SLOT_X &&
           r.route(T, op.n, op.k, jk::PRODUCT_RESIDUAL) == jk::ROUTE_SMALL && g_fns.linear_small_norm_supports(T, op.n, op.k);
}
bool qkv_fusable(const Run &r, const RunnerOp &op) {
    return r.env.dtype == JK_BF16 && op.vec == nullptr && op.writes_cache && !op.interleaved && !r.env.routing.library_only;
}
bool consumer_takes_norm(const Run &r, const RunnerOp &norm, const RunnerOp &next, int T) {
    if (next.in_slot != norm.out_slot) return false;
    if (next.kind == OP_GATE_UP)
        return r.route(T, next.n, next.k, jk::PRODUCT_SWIGLU) == jk::ROUTE_SMALL && g_fns.linear_small_norm_supports(T, next.n, next.k);
    if (next.kind == OP_QKV) return qkv_fusable(r, next) && g_fns.linear_small_qkv_supports(T, next.k, next.head_dim);
    return false;
}

int run_embed(Run &r, const RunnerOp &op) {
    void *out;
    if (int rc = r.slot(op.out_slot, 4LL * r.st.ntok * op.n, &out, "the embedding")) return rc;
    RUN(elementwise, g_fns.embed(r.st.tokens, r.st.ntok, op.w, op.w_dtype, op.n, op.scale, (float *)out, r.stream));
    return JK_OK;
}

int run_norm(Run &r, const RunnerOp &op) {
    const int rows = op.wanted_rows ? r.st.n_want : r.st.ntok;
    if (rows == 0) return JK_OK;
    void *out;
    if (int rc = r.slot(op.out_slot, (long long)r.elem() * rows * op.n, &out, "a norm")) return rc;
    // the pending product is added by the same kernel: into the stream when every row is normalised; a norm over the
    // wanted rows only reads stream + product for its rows and leaves both as they are
    RUN(elementwise, g_fns.add_rmsnorm(r.x(), r.pending ? r.delta() : nullptr, JK_F32, r.pending_scale, op.vec, op.eps, op.scale, out,
                                       r.env.dtype, op.wanted_rows ? r.st.want_rows : nullptr, rows, op.n, r.stream));
    if (!op.wanted_rows) r.pending = false;
    return JK_OK;
}

int run_qkv(Run &r, const RunnerOp &op, const FusedNorm &fused) {
    const int T = r.st.ntok, nq = op.n, d = op.k, nh = op.heads, nkvh = op.kv_heads, dh = op.head_dim;
    const jk::Routing &ro = r.env.routing;
    void *h, *q;
    if (int rc = r.slot(op.in_slot, (long long)r.elem() * T * d, &h, "q/k/v's activations")) return rc;
    if (int rc = r.slot(op.out_slot, (long long)r.elem() * T * nh * dh, &q, "the queries")) return rc;
    const int *table = r.st.block_tables[op.cache_group];
    JK_REQUIRE(table != nullptr || !op.writes_cache, "runner: q/k/v writes the cache of group %d, whose block table the step lacks", op.cache_group);
    if (fused.norm != nullptr) {
        RUN(linear_small, g_fns.linear_small_qkv_norm(h, op.w, T, d, q, op.k_pages, op.v_pages, op.cos_table, op.sin_table,
                                                      r.st.positions, r.st.row_req, table, r.env.max_blocks, r.env.page_size, nh, nkvh,
                                                      dh, fused.sumsq, fused.norm->eps, ro.sms, r.stream));
        return JK_OK;
    }
    if (qkv_fusable(r, op)) {
        // the product's epilogue rotates and writes q and the cache itself: no float32 copy of the product, no rotary kernel
        if (r.tcgen05_bound() && jk::takes_tcgen05(ro, T, nq, d) && (dh == 64 || dh == 128)) {
            RUN(gemm_tcgen05, g_fns.gemm_tcgen05_qkv(h, op.w, T, d, q, op.k_pages, op.v_pages, op.cos_table, op.sin_table, r.st.positions,
                                                     r.st.row_req, table, r.env.max_blocks, r.env.page_size, nh, nkvh, dh,
                                                     r.env.status, ro.sms, r.stream));
            return JK_OK;
        }
        if (T <= 16 && g_fns.linear_small_qkv_supports(T, d, dh)) {
            RUN(linear_small, g_fns.linear_small_qkv(h, op.w, T, d, q, op.k_pages, op.v_pages, op.cos_table, op.sin_table, r.st.positions,
                                                     r.st.row_req, table, r.env.max_blocks, r.env.page_size, nh, nkvh, dh, ro.sms,
                                                     r.stream));
            return JK_OK;
        }
    }
    void *tmp;
    if (int rc = r.slot(SLOT_TMP, 4LL * T * nq, &tmp, "the q/k/v product")) return rc;
    if (int rc = product_f32(r, h, op.w, nullptr, (float *)tmp, T, nq, d)) return rc;
    RUN(elementwise, g_fns.rope_kv(tmp, JK_F32, nq, op.vec, r.st.positions, r.st.row_req, table, r.env.max_blocks, r.env.page_size,
                                   op.cos_table, op.sin_table, op.interleaved, q, op.k_pages, op.v_pages, r.env.dtype, T, nh, nkvh, dh,
                                   op.writes_cache, r.stream));
    return JK_OK;
}

int run_attention(Run &r, const RunnerOp &op) {
    const int T = r.st.ntok, nh = op.heads, nkvh = op.kv_heads, dh = op.head_dim, page = r.env.page_size;
    void *q, *o;
    if (int rc = r.slot(op.in_slot, (long long)r.elem() * T * nh * dh, &q, "the queries")) return rc;
    if (int rc = r.slot(op.out_slot, (long long)r.elem() * T * nh * dh, &o, "attention's output")) return rc;
    const int *table = r.st.block_tables[op.cache_group];
    JK_REQUIRE(table != nullptr, "runner: attention reads the cache of group %d, whose block table the step lacks", op.cache_group);
    const int n_short = r.st.list_n[op.list_short], n_tiles = r.st.list_n[op.list_tiles];
    const int *short_rows = r.st.lists[op.list_short], *tiles = r.st.lists[op.list_tiles];
    const bool tc = !r.env.legacy_tensor_cores && g_fns.attention_tcgen05 != nullptr && jk::attention_tcgen05_takes(dh, page);
    bool fast = r.env.dtype == JK_BF16 && !r.env.plain_attention && (n_short > 0 || n_tiles > 0) && dh % 8 == 0 && dh <= 256;
    if (fast && n_tiles > 0 && !(tc || g_fns.attention_prefill_supports(dh))) fast = false;
    if (!fast) {
        // one warp per (row, head): float32, and every shape the tensor-core kernels are not built for
        RUN(attention, g_fns.attention_rows(q, op.k_pages, op.v_pages, o, r.env.dtype, r.st.positions, r.st.row_req, table,
                                            r.env.max_blocks, page, T, nh, nkvh, dh, op.softmax_scale, op.window, r.stream));
        return JK_OK;
    }
    if (n_tiles > 0) {
        if (tc)
            RUN(attention_tcgen05, g_fns.attention_tcgen05(q, op.k_pages, op.v_pages, o, tiles, n_tiles, T, r.st.req_start, r.st.req_pos,
                                                           table, r.env.max_blocks, op.num_pages, page, nh, nkvh, dh, op.softmax_scale,
                                                           op.window, r.env.status, r.stream));
        else
            RUN(attention, g_fns.attention_prefill(q, op.k_pages, op.v_pages, o, tiles, n_tiles, jk::TILE_ROWS, r.st.req_start,
                                                   r.st.req_pos, table, r.env.max_blocks, page, nh, nkvh, dh, op.softmax_scale,
                                                   op.window, r.stream));
    }
    if (n_short > 0) {
        const int context = r.st.context > 0 ? r.st.context : op.max_positions;
        const int splits = jk::decode_splits(n_short, nkvh, nh / nkvh, jk::decode_keys_hint(context, op.window), r.env.routing.sms, dh);
        void *scratch = nullptr;
        const long long need = 4 * jk::decode_scratch_floats(n_short, nh, dh, splits);
        if (need > 0)
            if (int rc = r.slot(SLOT_DECODE, need, &scratch, "the split-key attention's partial results")) return rc;
        RUN(attention, g_fns.attention_decode(q, op.k_pages, op.v_pages, o, (float *)scratch, short_rows, n_short, r.st.positions,
                                              r.st.row_req, table, r.env.max_blocks, page, nh, nkvh, dh, op.softmax_scale, op.window,
                                              splits, r.stream));
    }
    return JK_OK;
}

// stream += scale * (in w^T): in the product's epilogue where that exists, else left pending for the next norm
int run_residual(Run &r, const RunnerOp &op, const RunnerOp *norm, const RunnerOp *consumer, int op_index, FusedNorm *fused) {
    const int T = r.st.ntok;
    const jk::Routing &ro = r.env.routing;
    void *act;
    if (int rc = r.slot(op.in_slot, (long long)r.elem() * T * op.k, &act, "a product's activations")) return rc;
    JK_REQUIRE(op.out_slot == SLOT_X, "runner: a residual product adds into the stream");
    if (int rc = flush_pending(r, T, op.n)) return rc;
    if (small_residual_ok(r, op, T)) {
        const bool take_norm = norm != nullptr && norm->kind == OP_NORM && !norm->wanted_rows && norm->scale == 1.f && norm->n == op.n &&
                               consumer != nullptr && consumer_takes_norm(r, *norm, *consumer, T) && op_index < r.buf.sumsq_rows;
        void *h = nullptr;
        unsigned long long *ss = nullptr;
        if (take_norm) {
            if (int rc = r.slot(norm->out_slot, 2LL * T * op.n, &h, "a norm")) return rc;
            ss = r.buf.sumsq + (size_t)op_index * 16;
            fused->norm = norm;
            fused->sumsq = ss;
        }
        RUN(linear_small, g_fns.linear_small_norm(act, op.w, r.x(), T, op.n, op.k, op.n, 3, nullptr, 0.f, h, take_norm ? norm->vec : nullptr,
                                                  ss, op.scale, r.env.status, ro.sms, r.stream));
        return JK_OK;
    }
    if (r.env.dtype == JK_BF16) {
        const jk::Route route = r.route(T, op.n, op.k, jk::PRODUCT_RESIDUAL);
        if (route == jk::ROUTE_SKINNY) {
            RUN(gemm_tcgen05, g_fns.gemm_skinny(act, op.w, r.x(), T, op.n, op.k, op.n, 2, op.scale, r.env.status, ro.sms, r.stream));
            return JK_OK;
        }
        if (route == jk::ROUTE_TCGEN05) {
            RUN(gemm_tcgen05, g_fns.gemm_tcgen05(act, op.w, r.x(), T, op.n, op.k, op.n, 2, op.scale, r.env.status, ro.sms, r.stream));
            return JK_OK;
        }
    }
    void *delta;
    if (int rc = r.slot(SLOT_DELTA, 4LL * T * op.n, &delta, "a product that waits for the next norm")) return rc;
    if (int rc = product_f32(r, act, op.w, nullptr, (float *)delta, T, op.n, op.k)) return rc;
    r.pending = true;
    r.pending_scale = op.scale;
    return JK_OK;
}

int run_gate_up(Run &r, const RunnerOp &op, const FusedNorm &fused) {
    const int T = r.st.ntok, di = op.n, d = op.k;
    const jk::Routing &ro = r.env.routing;
    void *h, *act;
    if (int rc = r.slot(op.in_slot, (long long)r.elem() * T * d, &h, "gate/up's activations")) return rc;
    if (int rc = r.slot(op.out_slot, (long long)r.elem() * T * di, &act, "the feed-forward's inner activations")) return rc;
    if (fused.norm != nullptr) {
        RUN(linear_small, g_fns.linear_small_norm(h, op.w, act, T, di, d, di, 1, fused.sumsq, fused.norm->eps, nullptr, nullptr, nullptr,
                                                  1.f, r.env.status, ro.sms, r.stream));
        return JK_OK;
    }
    if (r.env.dtype == JK_BF16) {
        switch (r.route(T, di, d, jk::PRODUCT_SWIGLU)) {
            case jk::ROUTE_SMALL:
                RUN(linear_small, g_fns.linear_small(h, op.w, act, T, di, d, di, 1, ro.sms, r.stream));
                return JK_OK;
            case jk::ROUTE_SKINNY:
                RUN(gemm_tcgen05, g_fns.gemm_skinny(h, op.w, act, T, di, d, di, 3, 1.f, r.env.status, ro.sms, r.stream));
                return JK_OK;
            case jk::ROUTE_TCGEN05:
                RUN(gemm_tcgen05, g_fns.gemm_tcgen05(h, op.w, act, T, di, d, di, 3, 1.f, r.env.status, ro.sms, r.stream));
                return JK_OK;
            default:
                break;
        }
    }
    void *tmp;
    if (int rc = r.slot(SLOT_TMP, 4LL * T * 2 * di, &tmp, "the gate/up product")) return rc;
    if (r.env.dtype == JK_F32) {
        RUN(elementwise, g_fns.gemm_f32((const float *)h, d, (const float *)op.w, d, nullptr, (float *)tmp, 2 * di, T, 2 * di, d, r.stream));
    } else {
        if (int rc = lt_product(h, op.w, (float *)tmp, T, 2 * di, d, r.buf, r.stream)) return rc;
    }
    RUN(elementwise, g_fns.swiglu(tmp, JK_F32, act, r.env.dtype, T, di, r.stream));
    return JK_OK;
}

int run_linear(Run &r, const RunnerOp &op) {
    const int rows = op.wanted_rows ? r.st.n_want : r.st.ntok;
    if (rows == 0) return JK_OK;
    void *in, *out;
    if (int rc = r.slot(op.in_slot, (long long)r.elem() * rows * op.k, &in, "a product's activations")) return rc;
    if (int rc = r.slot(op.out_slot, 4LL * rows * op.n, &out, "a product's output")) return rc;
    return product_f32(r, in, op.w, op.vec, (float *)out, rows, op.n, op.k);
}

}  // namespace

JK_EXPORT int jk_runner_run(const RunnerEnv *envp, const RunnerOp *ops, int first, int count, const RunnerStep *sp,
                            const RunnerBuffers *bp, int flush, cudaStream_t stream) {
    JK_REQUIRE(g_bound, "runner_run: jk_runner_bind has not been called");
    JK_REQUIRE(envp && ops && sp && bp && first >= 0 && count >= 0, "runner_run: an argument is missing");
    JK_REQUIRE(envp->dtype == JK_F32 || envp->dtype == JK_BF16, "runner_run: dtype %d", envp->dtype);
    Run r{*envp, *sp, *bp, stream};
    g_launches = 0;
    const int T = sp->ntok;
    if (T == 0 || count == 0) return JK_OK;
    JK_REQUIRE(bp->slot[SLOT_X] != nullptr, "runner_run: the stream's buffer is missing");
    bool may_fuse = false;
    if (envp->dtype == JK_BF16 && envp->fused_norms && T <= 16 && bp->sumsq != nullptr)
        for (int i = first; i < first + count && !may_fuse; ++i) may_fuse = ops[i].kind == OP_RESIDUAL;
    if (may_fuse) {
        ++g_launches;
        if (cudaMemsetAsync(bp->sumsq, 0, sizeof(unsigned long long) * 16 * (size_t)bp->sumsq_rows, stream) != cudaSuccess)
            JK_FAIL(JK_CUDA_ERROR, "runner: clearing the sums of squares failed");
    }
    FusedNorm fused;              // set by a residual product that took over the norm after it
    int hidden = 0;
    for (int i = first; i < first + count; ++i) {
        const RunnerOp &op = ops[i];
        int rc = JK_OK;
        switch (op.kind) {
            case OP_EMBED:
                hidden = op.n;
                rc = run_embed(r, op);
                break;
            case OP_NORM:
                hidden = op.n;
                if (fused.norm == &op) break;          // the product before did its work
                rc = run_norm(r, op);
                break;
            case OP_QKV: {
                const FusedNorm use = (fused.norm != nullptr && i > first && &ops[i - 1] == fused.norm) ? fused : FusedNorm{};
                rc = run_qkv(r, op, use);
                fused = FusedNorm{};
                break;
            }
            case OP_ATTENTION:
                rc = run_attention(r, op);
                break;
            case OP_RESIDUAL: {
                hidden = op.n;
                const RunnerOp *norm = i + 1 < first + count ? &ops[i + 1] : nullptr;
                const RunnerOp *consumer = i + 2 < first + count ? &ops[i + 2] : nullptr;
                fused = FusedNorm{};
                rc = run_residual(r, op, norm, consumer, i, &fused);
                break;
            }
            case OP_GATE_UP: {
                const FusedNorm use = (fused.norm != nullptr && i > first && &ops[i - 1] == fused.norm) ? fused : FusedNorm{};
                rc = run_gate_up(r, op, use);
                fused = FusedNorm{};
                break;
            }
            case OP_LINEAR:
                rc = run_linear(r, op);
                break;
            default:
                JK_FAIL(JK_BAD_ARGUMENT, "runner_run: record %d has kind %d", i, op.kind);
        }
        if (rc) return rc;
    }
    // A product that still waits for its addition: a caller that goes on with code of its own (flush) gets a whole stream;
    // at the end of a model nobody reads the stream again.
    if (r.pending && flush) {
        JK_REQUIRE(hidden > 0, "runner_run: a product waits for its addition but no record said how wide the stream is");
        if (int rc = flush_pending(r, T, hidden)) return rc;
    }
    return JK_OK;
}

// How many bytes each slot needs for steps of up to `max_rows` rows with up to `max_want` wanted rows.
JK_EXPORT int jk_runner_slot_bytes(const RunnerEnv *env, const RunnerOp *ops, int count, int max_rows, int max_want, long long *bytes) {
    JK_REQUIRE(env && ops && bytes && max_rows > 0 && max_want >= 0, "runner_slot_bytes: an argument is missing");
    const long long e = env->dtype == JK_F32 ? 4 : 2;
    for (int s = 0; s < RUNNER_SLOTS; ++s) bytes[s] = 0;
    auto need = [&](int slot, long long b) { if (slot >= 0 && slot < RUNNER_SLOTS && b > bytes[slot]) bytes[slot] = b; };
    for (int i = 0; i < count; ++i) {
        const RunnerOp &op = ops[i];
        const long long rows = op.wanted_rows ? max_want : max_rows;
        switch (op.kind) {
            case OP_EMBED: need(op.out_slot, 4 * rows * op.n); break;
            case OP_NORM: need(SLOT_X, 4LL * max_rows * op.n); need(op.out_slot, e * rows * op.n); break;
            case OP_QKV:
                need(op.in_slot, e * rows * op.k); need(op.out_slot, e * rows * op.heads * op.head_dim); need(SLOT_TMP, 4 * rows * op.n);
                break;
            case OP_ATTENTION: {
                need(op.in_slot, e * rows * op.heads * op.head_dim); need(op.out_slot, e * rows * op.heads * op.head_dim);
                // the worst step: more rows mean fewer cuts; every context bucket up to the longest
                long long worst = 0;
                for (int context = 256;; context *= 2) {
                    const int c = context < op.max_positions ? context : op.max_positions;
                    for (int n = 1; n <= max_rows; ++n) {
                        const int s = jk::decode_splits(n, op.kv_heads, op.heads / op.kv_heads, jk::decode_keys_hint(c, op.window),
                                                        env->routing.sms, op.head_dim);
                        worst = std::max(worst, jk::decode_scratch_floats(n, op.heads, op.head_dim, s));
                        if (s <= 1) break;
                    }
                    if (context >= op.max_positions) break;
                }
                need(SLOT_DECODE, 4 * worst);
                break;
            }
            case OP_RESIDUAL: need(op.in_slot, e * rows * op.k); need(SLOT_X, 4 * rows * op.n); need(SLOT_DELTA, 4 * rows * op.n); break;
            case OP_GATE_UP: need(op.in_slot, e * rows * op.k); need(op.out_slot, e * rows * op.n); need(SLOT_TMP, 4 * rows * 2 * op.n); break;
            case OP_LINEAR: need(op.in_slot, e * rows * op.k); need(op.out_slot, 4 * rows * op.n); break;
            default: JK_FAIL(JK_BAD_ARGUMENT, "runner_slot_bytes: record %d has kind %d", i, op.kind);
        }
    }
    return JK_OK;
}

// Whether records [0, count) can reach a kernel of the tcgen05 product module in a step of up to `max_rows` rows.
JK_EXPORT int jk_runner_needs_gemm_tcgen05(const RunnerEnv *env, const RunnerOp *ops, int count, int max_rows) {
    if (!env || !ops || env->dtype != JK_BF16 || env->routing.library_only) return 0;
    for (int i = 0; i < count; ++i) {
        const RunnerOp &op = ops[i];
        int kind;
        switch (op.kind) {
            case OP_QKV: case OP_LINEAR: kind = jk::PRODUCT_F32; break;
            case OP_RESIDUAL: kind = jk::PRODUCT_RESIDUAL; break;
            case OP_GATE_UP: kind = jk::PRODUCT_SWIGLU; break;
            default: continue;
        }
        for (int rows : {1, 16, 17, 128, 129, max_rows})
            if (rows <= max_rows || rows == 1) {
                const jk::Route rt = jk::product_route(env->routing, rows, op.n, op.k, kind, true, true);
                if (rt == jk::ROUTE_SKINNY || rt == jk::ROUTE_TCGEN05) return 1;
                // small_ok = true may hide the few-rows kernel behind the small-row one: ask again without it
                const jk::Route rt2 = jk::product_route(env->routing, rows, op.n, op.k, kind, false, true);
                if (rt2 == jk::ROUTE_SKINNY || rt2 == jk::ROUTE_TCGEN05) return 1;
            }
    }
    return 0;
}

// ---- emitters: the records of this architecture's standard parts -----------------------------------------------
static RunnerOp blank(int kind, int in_slot, int out_slot) {
    RunnerOp op;
    memset(&op, 0, sizeof(op));
    op.kind = kind; op.in_slot = in_slot; op.out_slot = out_slot;
    op.scale = 1.f;
    return op;
}

// Causal softmax attention over the paged cache (src/models/jiuge/jiuge.cpp:200-236): the fused q/k/v product with
// rotation and cache write, the attention itself, the output product added into the stream times `residual_scale`.
JK_EXPORT int jk_emit_attention(RunnerOp *out, const void *w_qkv, const float *b_qkv, const void *w_o, int hidden, int heads, int kv_heads,
                                int head_dim, int window, float softmax_scale, float residual_scale, const float *cos_table,
                                const float *sin_table, int interleaved, int max_positions, void *k_pages, void *v_pages, int num_pages,
                                int cache_group, int writes_cache, int list_short, int list_tiles) {
    RunnerOp qkv = blank(OP_QKV, SLOT_H, SLOT_Q);
    qkv.n = (heads + 2 * kv_heads) * head_dim; qkv.k = hidden;
    qkv.heads = heads; qkv.kv_heads = kv_heads; qkv.head_dim = head_dim; qkv.interleaved = interleaved; qkv.writes_cache = writes_cache;
    qkv.cache_group = cache_group; qkv.w = w_qkv; qkv.vec = b_qkv; qkv.cos_table = cos_table; qkv.sin_table = sin_table;
    qkv.k_pages = k_pages; qkv.v_pages = v_pages; qkv.num_pages = num_pages;
    RunnerOp att = blank(OP_ATTENTION, SLOT_Q, SLOT_O);
    att.heads = heads; att.kv_heads = kv_heads; att.head_dim = head_dim; att.window = window; att.softmax_scale = softmax_scale;
    att.cache_group = cache_group; att.list_short = list_short; att.list_tiles = list_tiles; att.max_positions = max_positions;
    att.k_pages = k_pages; att.v_pages = v_pages; att.num_pages = num_pages;
    RunnerOp o = blank(OP_RESIDUAL, SLOT_O, SLOT_X);
    o.n = hidden; o.k = heads * head_dim; o.w = w_o; o.scale = residual_scale;
    out[0] = qkv; out[1] = att; out[2] = o;
    return 3;
}

// SwiGLU feed-forward (src/models/jiuge/jiuge.cpp:247-249): gate | up with the activation, down added into the stream.
JK_EXPORT int jk_emit_swiglu(RunnerOp *out, const void *w_gate_up, const void *w_down, int hidden, int intermediate, float residual_scale) {
    RunnerOp gu = blank(OP_GATE_UP, SLOT_H, SLOT_ACT);
    gu.n = intermediate; gu.k = hidden; gu.w = w_gate_up;
    RunnerOp down = blank(OP_RESIDUAL, SLOT_ACT, SLOT_X);
    down.n = hidden; down.k = intermediate; down.w = w_down; down.scale = residual_scale;
    out[0] = gu; out[1] = down;
    return 2;
}

// RMSNorm over every row (into the next product's activations) or over the wanted rows (the final norm).
JK_EXPORT int jk_emit_rmsnorm(RunnerOp *out, const float *weight, int size, float eps, float out_scale, int wanted_rows) {
    RunnerOp op = blank(OP_NORM, SLOT_X, wanted_rows ? SLOT_HW : SLOT_H);
    op.n = size; op.vec = weight; op.eps = eps; op.scale = out_scale; op.wanted_rows = wanted_rows;
    out[0] = op;
    return 1;
}

JK_EXPORT int jk_emit_embedding(RunnerOp *out, const void *table, int dtype, int hidden, float scale) {
    RunnerOp op = blank(OP_EMBED, -1, SLOT_X);
    op.n = hidden; op.w = table; op.w_dtype = dtype; op.scale = scale;
    out[0] = op;
    return 1;
}

JK_EXPORT int jk_emit_output(RunnerOp *out, const void *w, int vocab, int hidden) {
    RunnerOp op = blank(OP_LINEAR, SLOT_HW, SLOT_LOGITS);
    op.n = vocab; op.k = hidden; op.w = w; op.wanted_rows = 1;
    out[0] = op;
    return 1;
}

// The size of a record, for a caller in another language that mirrors the struct.
JK_EXPORT int jk_runner_op_size() { return (int)sizeof(RunnerOp); }
// sizes[0..4]: RunnerOp, RunnerEnv, RunnerStep, RunnerBuffers, RunnerFns
JK_EXPORT void jk_runner_struct_sizes(int *sizes) {
    sizes[0] = (int)sizeof(RunnerOp); sizes[1] = (int)sizeof(RunnerEnv); sizes[2] = (int)sizeof(RunnerStep);
    sizes[3] = (int)sizeof(RunnerBuffers); sizes[4] = (int)sizeof(RunnerFns);
}
