// The step of the standard decoder stack, run from native code: one call launches every kernel of a
// step (embedding, the layers, the final norm, the output product) where the Python parts would make
// a dozen calls a layer.  It runs the same kernels with the same routing as the parts do:
//
//   rows <= 16            the weight-streaming kernels of linear_small.cu (q/k/v with rotation and cache
//                         write in the epilogue, gate/up with SwiGLU in the epilogue)
//   rows >= min_rows      the tcgen05 kernels of gemm_tcgen05.cu (q/k/v epilogue, SwiGLU epilogue, residual
//                         add by TMA)
//   in between            cuBLAS, bfloat16 operands, float32 accumulation and output, with the rotary
//                         kernel, the SwiGLU kernel and the fused add + norm kernel around it
//   attention             tiles of requests with many rows -> attention_tcgen05 (or the mma.sync kernel);
//                         rows of requests with few rows -> the split-key decode kernel
//
// The kernels live in their own shared objects; the caller hands their entry points over once
// (jk_runner_bind).  Everything a step needs arrives in four plain structs; nothing is allocated here.
// (The reference's counterpart is the per-device worker that runs inferDeviceBatch,
// src/models/jiuge/jiuge.cpp:126-305.)
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
    // the tcgen05 modules may be left out by a caller whose model or step size never reaches them (they are
    // then not even compiled); everything else is needed by every model
    JK_REQUIRE(fns->embed && fns->add_rmsnorm && fns->swiglu && fns->rope_kv && fns->linear_small && fns->linear_small_qkv &&
               fns->linear_small_supports && fns->linear_small_qkv_supports && fns->linear_small_norm_supports &&
               fns->linear_small_norm && fns->linear_small_qkv_norm && fns->attention_decode && fns->attention_prefill && fns->err_elementwise && fns->err_linear_small &&
               fns->err_attention, "runner_bind: an entry that every model needs is empty");
    JK_REQUIRE((fns->gemm_tcgen05 != nullptr) == (fns->gemm_tcgen05_qkv != nullptr) &&
               (fns->gemm_tcgen05 != nullptr) == (fns->gemm_skinny != nullptr) &&
               (fns->gemm_tcgen05 != nullptr) == (fns->err_gemm_tcgen05 != nullptr) &&
               (fns->attention_tcgen05 != nullptr) == (fns->err_attention_tcgen05 != nullptr),
               "runner_bind: a module's entries come together");
    // a table adds to what is bound already (two users of this library in one process may need different
    // modules): an entry that this caller leaves empty keeps what an earlier caller gave
    static_assert(sizeof(RunnerFns) % sizeof(void *) == 0, "the table is a list of pointers");
    void *const *from = (void *const *)fns;
    void **to = (void **)&g_fns;
    for (size_t i = 0; i < sizeof(RunnerFns) / sizeof(void *); ++i)
        if (from[i] != nullptr) to[i] = from[i];
    g_bound = true;
    return JK_OK;
}

static int g_launches = 0;      // kernels launched by the last jk_runner_forward (the library's count as one each)
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

static int lt_product(const void *act, const void *w, float *out, int M, int N, int K, const RunnerScratch &s, cudaStream_t stream) {
    std::lock_guard<std::mutex> lock(g_blas_mutex);
    if (!g_blas && cublasCreate(&g_blas) != CUBLAS_STATUS_SUCCESS) JK_FAIL(JK_CUDA_ERROR, "runner: cublasCreate failed");
    if (cublasSetStream(g_blas, stream) != CUBLAS_STATUS_SUCCESS ||
        cublasSetWorkspace(g_blas, s.workspace, (size_t)s.workspace_bytes) != CUBLAS_STATUS_SUCCESS)
        JK_FAIL(JK_CUDA_ERROR, "runner: the library refused the stream or the workspace");
    // row-major out[M, N] is column-major [N, M] = W^T (op T on the column-major [K, N]) * act (column-major [K, M])
    const float one = 1.f, zero = 0.f;
    ++g_launches;
    const cublasStatus_t st = cublasGemmEx(g_blas, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &one, w, CUDA_R_16BF, K, act, CUDA_R_16BF, K,
                                           &zero, out, CUDA_R_32F, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    if (st != CUBLAS_STATUS_SUCCESS) JK_FAIL(JK_CUDA_ERROR, "runner: the library's product of %d x %d x %d failed with %d", M, N, K, (int)st);
    return JK_OK;
}

static bool takes_tcgen05(const RunnerModel &m, int rows, int n, int k) {
    return g_fns.gemm_tcgen05 != nullptr && runner_takes_tcgen05(m.sms, m.tcgen05_min_rows, m.tcgen05_min_tiles, m.tcgen05_min_fill_pct, rows, n, k);
}

// Which kernel takes a product of at most 128 rows (the same rule as Runtime.few_rows_route of the parts): the
// few-rows tcgen05 kernel once it has a block for every SM; up to 16 rows the small-row kernel where it has a
// second block on the SM to overlap its load phase with (a slice of 16 rows x K fits twice), or so few tiles that
// they make one wave, or nothing better; else the library.
enum Route { ROUTE_LIBRARY, ROUTE_SMALL, ROUTE_SKINNY };
static Route few_rows_route(const RunnerModel &m, int rows, int n, int k, int kind) {
    if (rows > 128) return ROUTE_LIBRARY;
    const long long need = m.skinny_min_blocks > 0 ? m.skinny_min_blocks : m.sms;
    const bool skinny = g_fns.gemm_skinny != nullptr && k % 8 == 0 && runner_skinny_blocks(m.sms, n, k, kind) >= need;
    if (rows <= 16 && g_fns.linear_small_supports(rows, n, k)) {
        const long long out_rows = kind == RUNNER_SWIGLU ? 2LL * n : n;
        if (!skinny || 2 * (32LL * k + 8192) <= 227 * 1024 || (out_rows + 15) / 16 <= m.sms) return ROUTE_SMALL;
    }
    return skinny ? ROUTE_SKINNY : ROUTE_LIBRARY;
}

// out (float32 [rows, n]) = act * w^T by whichever kernel takes `rows`
static int product_f32(const RunnerModel &m, const RunnerScratch &s, const void *act, const void *w, float *out, int rows, int n,
                       int k, cudaStream_t stream) {
    const Route route = few_rows_route(m, rows, n, k, RUNNER_F32);
    if (route == ROUTE_SMALL) {
        RUN(linear_small, g_fns.linear_small(act, w, out, rows, n, k, n, 0, m.sms, stream));
    } else if (route == ROUTE_SKINNY) {
        RUN(gemm_tcgen05, g_fns.gemm_skinny(act, w, out, rows, n, k, n, 0, 1.f, m.status, m.sms, stream));
    } else if (takes_tcgen05(m, rows, n, k)) {
        RUN(gemm_tcgen05, g_fns.gemm_tcgen05(act, w, out, rows, n, k, n, 0, 1.f, m.status, m.sms, stream));
    } else {
        if (int rc = lt_product(act, w, out, rows, n, k, s, stream)) return rc;
    }
    return JK_OK;
}

// x += scale * (act * w^T): in the product's epilogue where that exists, else left pending for the next norm
static int product_into_residual(const RunnerModel &m, const RunnerScratch &s, const void *act, const void *w, int rows, int n,
                                 int k, bool *pending, cudaStream_t stream) {
    *pending = false;
    if (few_rows_route(m, rows, n, k, RUNNER_RESIDUAL) == ROUTE_SKINNY) {
        RUN(gemm_tcgen05, g_fns.gemm_skinny(act, w, s.x, rows, n, k, n, 2, m.residual_scale, m.status, m.sms, stream));
        return JK_OK;
    }
    if (takes_tcgen05(m, rows, n, k)) {
        RUN(gemm_tcgen05, g_fns.gemm_tcgen05(act, w, s.x, rows, n, k, n, 2, m.residual_scale, m.status, m.sms, stream));
        return JK_OK;
    }
    *pending = true;
    return product_f32(m, s, act, w, s.delta, rows, n, k, stream);
}

JK_EXPORT int jk_runner_forward(const RunnerModel *mp, const RunnerLayer *layers, const RunnerStep *sp, const RunnerScratch *cp,
                                cudaStream_t stream) {
    JK_REQUIRE(g_bound, "runner_forward: jk_runner_bind has not been called");
    JK_REQUIRE(mp && layers && sp && cp, "runner_forward: a struct is missing");
    const RunnerModel &m = *mp;
    const RunnerStep &st = *sp;
    const RunnerScratch &s = *cp;
    const int T = st.ntok, d = m.hidden, nh = m.heads, nkvh = m.kv_heads, dh = m.head_dim, di = m.intermediate;
    const int nq = (nh + 2 * nkvh) * dh;
    g_launches = 0;
    if (T == 0) return JK_OK;
    RUN(elementwise, g_fns.embed(st.tokens, T, m.embedding, m.embed_dtype, d, m.embed_scale, s.x, stream));
    // Steps of few rows run without norm kernels when all four products of a layer are the small-row tile kernel's:
    // o and down add themselves into x, leave bfloat16(x * next norm's weight) in s.h and the rows' sums of squares in
    // s.sumsq; q/k/v and gate/up scale their rows by 1 / rms.  Two kernels fewer in a layer's chain of nine.
    const bool fused = m.fused_norms && T <= 16 && s.sumsq != nullptr && g_fns.linear_small_qkv_supports(T, d, dh) &&
                       g_fns.linear_small_norm_supports(T, d, nh * dh) && g_fns.linear_small_norm_supports(T, di, d) &&
                       g_fns.linear_small_norm_supports(T, d, di) && few_rows_route(m, T, d, nh * dh, RUNNER_RESIDUAL) == ROUTE_SMALL &&
                       few_rows_route(m, T, di, d, RUNNER_SWIGLU) == ROUTE_SMALL && few_rows_route(m, T, d, di, RUNNER_RESIDUAL) == ROUTE_SMALL;
    if (fused) {
        ++g_launches;
        if (cudaMemsetAsync(s.sumsq, 0, sizeof(unsigned long long) * 2 * m.layers * 16, stream) != cudaSuccess)
            JK_FAIL(JK_CUDA_ERROR, "runner: clearing the sums of squares failed");
    }
    bool pending = false;       // s.delta holds a product that has not been added to x yet
    for (int l = 0; l < m.layers; ++l) {
        const RunnerLayer &L = layers[l];
        unsigned long long *ss1 = fused ? s.sumsq + (size_t)(2 * l) * 16 : nullptr;       // rows before norm1 of this layer
        unsigned long long *ss2 = fused ? s.sumsq + (size_t)(2 * l + 1) * 16 : nullptr;   // before norm2
        // ---- attention ----
        if (fused && l > 0) {
            // s.h and ss1 were left by the layer before
            RUN(linear_small, g_fns.linear_small_qkv_norm(s.h, L.w_qkv, T, d, s.q, L.k_pages, L.v_pages, m.cos_table, m.sin_table,
                                                          st.positions, st.row_req, st.block_table, m.max_blocks, m.page_size,
                                                          nh, nkvh, dh, ss1, L.eps1, m.sms, stream));
        } else {
        RUN(elementwise, g_fns.add_rmsnorm(s.x, pending ? s.delta : nullptr, JK_F32, m.residual_scale, L.norm1, L.eps1, 1.f, s.h,
                                           JK_BF16, nullptr, T, d, stream));
        pending = false;
        if (takes_tcgen05(m, T, nq, d) && (dh == 64 || dh == 128)) {
            RUN(gemm_tcgen05, g_fns.gemm_tcgen05_qkv(s.h, L.w_qkv, T, d, s.q, L.k_pages, L.v_pages, m.cos_table, m.sin_table,
                                                     st.positions, st.row_req, st.block_table, m.max_blocks, m.page_size, nh,
                                                     nkvh, dh, m.status, m.sms, stream));
        } else if (T <= 16 && g_fns.linear_small_qkv_supports(T, d, dh)) {
            RUN(linear_small, g_fns.linear_small_qkv(s.h, L.w_qkv, T, d, s.q, L.k_pages, L.v_pages, m.cos_table, m.sin_table,
                                                     st.positions, st.row_req, st.block_table, m.max_blocks, m.page_size, nh,
                                                     nkvh, dh, m.sms, stream));
        } else {
            if (int rc = product_f32(m, s, s.h, L.w_qkv, s.qkv, T, nq, d, stream)) return rc;
            RUN(elementwise, g_fns.rope_kv(s.qkv, JK_F32, nq, nullptr, st.positions, st.row_req, st.block_table, m.max_blocks,
                                           m.page_size, m.cos_table, m.sin_table, 0, s.q, L.k_pages, L.v_pages, JK_BF16, T, nh,
                                           nkvh, dh, 1, stream));
        }
        }
        if (st.n_tiles > 0) {
            if (m.attention_tcgen05 && g_fns.attention_tcgen05 != nullptr)
                RUN(attention_tcgen05, g_fns.attention_tcgen05(s.q, L.k_pages, L.v_pages, s.o, st.tiles, st.n_tiles, T, st.req_start,
                                                               st.req_pos, st.block_table, m.max_blocks, m.num_pages, m.page_size,
                                                               nh, nkvh, dh, m.softmax_scale, m.window, m.status, stream));
            else
                RUN(attention, g_fns.attention_prefill(s.q, L.k_pages, L.v_pages, s.o, st.tiles, st.n_tiles, 128, st.req_start,
                                                       st.req_pos, st.block_table, m.max_blocks, m.page_size, nh, nkvh, dh,
                                                       m.softmax_scale, m.window, stream));
        }
        if (st.n_short > 0)
            RUN(attention, g_fns.attention_decode(s.q, L.k_pages, L.v_pages, s.o, st.splits > 1 ? s.decode_scratch : nullptr,
                                                  st.short_rows, st.n_short, st.positions, st.row_req, st.block_table,
                                                  m.max_blocks, m.page_size, nh, nkvh, dh, m.softmax_scale, m.window, st.splits,
                                                  stream));
        if (fused) {
            // x += scale * o; s.h = bfloat16(x * norm2), ss2 = sum(x^2); gate/up reads them; down does the same for the
            // next layer's norm1 (the last layer's down only adds: the final norm has its own kernel)
            RUN(linear_small, g_fns.linear_small_norm(s.o, L.w_o, s.x, T, d, nh * dh, d, 3, nullptr, 0.f, s.h, L.norm2, ss2,
                                                      m.residual_scale, m.status, m.sms, stream));
            RUN(linear_small, g_fns.linear_small_norm(s.h, L.w_gate_up, s.act, T, di, d, di, 1, ss2, L.eps2, nullptr, nullptr, nullptr,
                                                      1.f, m.status, m.sms, stream));
            const bool last = l + 1 == m.layers;
            RUN(linear_small, g_fns.linear_small_norm(s.act, L.w_down, s.x, T, d, di, d, 3, nullptr, 0.f, last ? nullptr : s.h,
                                                      last ? nullptr : layers[l + 1].norm1, last ? nullptr : ss1 + 32,
                                                      m.residual_scale, m.status, m.sms, stream));
            continue;
        }
        if (int rc = product_into_residual(m, s, s.o, L.w_o, T, d, nh * dh, &pending, stream)) return rc;
        // ---- feed-forward ----
        RUN(elementwise, g_fns.add_rmsnorm(s.x, pending ? s.delta : nullptr, JK_F32, m.residual_scale, L.norm2, L.eps2, 1.f, s.h,
                                           JK_BF16, nullptr, T, d, stream));
        pending = false;
        const Route gate_up = few_rows_route(m, T, di, d, RUNNER_SWIGLU);
        if (gate_up == ROUTE_SMALL) {
            RUN(linear_small, g_fns.linear_small(s.h, L.w_gate_up, s.act, T, di, d, di, 1, m.sms, stream));
        } else if (gate_up == ROUTE_SKINNY) {
            RUN(gemm_tcgen05, g_fns.gemm_skinny(s.h, L.w_gate_up, s.act, T, di, d, di, 3, 1.f, m.status, m.sms, stream));
        } else if (takes_tcgen05(m, T, di, d)) {
            RUN(gemm_tcgen05, g_fns.gemm_tcgen05(s.h, L.w_gate_up, s.act, T, di, d, di, 3, 1.f, m.status, m.sms, stream));
        } else {
            if (int rc = lt_product(s.h, L.w_gate_up, s.gate_up, T, 2 * di, d, s, stream)) return rc;
            RUN(elementwise, g_fns.swiglu(s.gate_up, JK_F32, s.act, JK_BF16, T, di, stream));
        }
        if (int rc = product_into_residual(m, s, s.act, L.w_down, T, d, di, &pending, stream)) return rc;
    }
    // the logit scale rides on the final norm, which looks at the wanted rows only
    if (st.n_want > 0) {
        RUN(elementwise, g_fns.add_rmsnorm(s.x, pending ? s.delta : nullptr, JK_F32, m.residual_scale, m.final_norm, m.final_eps,
                                           m.logit_scale, s.hw, JK_BF16, st.want_rows, st.n_want, d, stream));
        if (int rc = product_f32(m, s, s.hw, m.lm_head, st.logits, st.n_want, m.vocab, d, stream)) return rc;
    }
    return JK_OK;
}
