// Types of the native runner (csrc/runner.cu) and of the C interface on top of it (csrc/capi.cu).
#pragma once

#include <cuda_runtime.h>

// ---- entry points of the kernel modules (signatures as in their sources) -------------------------------
extern "C" {
typedef int (*EmbedFn)(const int *, int, const void *, int, int, float, float *, cudaStream_t);
typedef int (*AddRmsnormFn)(float *, const void *, int, float, const float *, float, float, void *, int, const int *, int,
                            int, cudaStream_t);
typedef int (*SwigluFn)(const void *, int, void *, int, int, int, cudaStream_t);
typedef int (*RopeKvFn)(const void *, int, int, const float *, const int *, const int *, const int *, int, int,
                        const float *, const float *, int, void *, void *, void *, int, int, int, int, int, int,
                        cudaStream_t);
typedef int (*LinearSmallFn)(const void *, const void *, void *, int, int, int, int, int, int, cudaStream_t);
typedef int (*LinearSmallQkvFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                const int *, const int *, const int *, int, int, int, int, int, int, cudaStream_t);
typedef int (*GemmTcgen05Fn)(const void *, const void *, void *, int, int, int, int, int, float, int *, int, cudaStream_t);
typedef int (*GemmTcgen05QkvFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                const int *, const int *, const int *, int, int, int, int, int, int *, int, cudaStream_t);
typedef int (*AttentionDecodeFn)(const void *, const void *, const void *, void *, float *, const int *, int, const int *,
                                 const int *, const int *, int, int, int, int, int, float, int, int, cudaStream_t);
typedef int (*AttentionPrefillFn)(const void *, const void *, const void *, void *, const int *, int, int, const int *,
                                  const int *, const int *, int, int, int, int, int, float, int, cudaStream_t);
typedef int (*AttentionTcgen05Fn)(const void *, const void *, const void *, void *, const int *, int, int, const int *,
                                  const int *, const int *, int, int, int, int, int, int, float, int, int *, cudaStream_t);
typedef int (*SupportsFn)(int, int, int);
typedef int (*LinearSmallNormFn)(const void *, const void *, void *, int, int, int, int, int, const unsigned long long *, float,
                                 void *, const float *, unsigned long long *, float, int *, int, cudaStream_t);
typedef int (*LinearSmallQkvNormFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                    const int *, const int *, const int *, int, int, int, int, int,
                                    const unsigned long long *, float, int, cudaStream_t);
typedef const char *(*LastErrorFn)();
typedef int (*ArgmaxFn)(const float *, long long, int, int, int *, void *, cudaStream_t);
typedef int (*SampleFn)(const float *, long long, int, int, const float *, const int *, const float *, const float *, int *,
                        cudaStream_t);
}

struct RunnerFns {
    EmbedFn embed;
    AddRmsnormFn add_rmsnorm;
    SwigluFn swiglu;
    RopeKvFn rope_kv;
    LinearSmallFn linear_small;
    LinearSmallQkvFn linear_small_qkv;
    GemmTcgen05Fn gemm_tcgen05;
    GemmTcgen05QkvFn gemm_tcgen05_qkv;
    AttentionDecodeFn attention_decode;
    AttentionPrefillFn attention_prefill;
    AttentionTcgen05Fn attention_tcgen05;
    LastErrorFn err_elementwise, err_linear_small, err_gemm_tcgen05, err_attention, err_attention_tcgen05;
    // products of few rows: what the small-row kernels take, and the tcgen05 kernel with the weights on the MMA's M side
    // (part of the gemm_tcgen05 module: bound with it or not at all)
    SupportsFn linear_small_supports, linear_small_qkv_supports;
    GemmTcgen05Fn gemm_skinny;
    // few-row products of a chain in which RMSNorm has no kernel of its own
    SupportsFn linear_small_norm_supports;
    LinearSmallNormFn linear_small_norm;
    LinearSmallQkvNormFn linear_small_qkv_norm;
    // sampling (used by the C interface only; may be empty for a caller that samples by itself)
    ArgmaxFn argmax;
    SampleFn sample;
    LastErrorFn err_sampling;
};

// What never changes from step to step.
struct RunnerModel {
    int layers, hidden, heads, kv_heads, head_dim, intermediate, vocab;
    int page_size, max_blocks, num_pages, window;
    int sms, tcgen05_min_rows, tcgen05_min_tiles, tcgen05_min_fill_pct;
    int skinny_min_blocks;          // fewest blocks for which the few-rows tcgen05 kernel is used (0: one per SM)
    int fused_norms;                // 1: steps of at most 16 rows run without norm kernels where the small-row kernels allow
    int attention_tcgen05;          // 1: tiles go to the tcgen05 attention kernel, 0: to the mma.sync kernel
    int embed_dtype;                // JK_F32 or JK_BF16
    float embed_scale, residual_scale, logit_scale, softmax_scale, final_eps;
    const void *embedding;          // [vocab, hidden]
    const void *lm_head;            // [vocab, hidden] bfloat16
    const float *final_norm;        // [hidden]
    const float *cos_table;         // [positions, head_dim / 2] or null
    const float *sin_table;
    int *status;                    // the word in which the tcgen05 kernels record a wait that ran out
};

struct RunnerLayer {
    const void *w_qkv, *w_o, *w_gate_up, *w_down;      // bfloat16 [N, K]
    const float *norm1, *norm2;
    float eps1, eps2;
    void *k_pages, *v_pages;                           // bfloat16 [pages, kv_heads, page_size, head_dim]
};

// One step's batch (device arrays of the step's metadata buffer) and where its logits go.
struct RunnerStep {
    int ntok, nreq, n_want, n_tiles, n_short, splits;
    const int *tokens, *positions, *row_req, *req_start, *req_pos, *want_rows, *short_rows, *tiles, *block_table;
    float *logits;                  // [n_want, vocab]
};

// Buffers for `max_tokens` rows, made once by the caller.
struct RunnerScratch {
    float *x;                       // [T, hidden] the residual stream
    void *h;                        // bf16 [T, hidden]
    float *qkv;                     // [T, (heads + 2 kv_heads) * head_dim]
    void *q, *o;                    // bf16 [T, heads * head_dim]
    float *delta;                   // [T, hidden]
    float *gate_up;                 // [T, 2 * intermediate]
    void *act;                      // bf16 [T, intermediate]
    void *hw;                       // bf16 [max wanted rows, hidden]
    float *decode_scratch;          // partial results of the split-key attention
    void *workspace;                // for the library
    long long workspace_bytes;
    unsigned long long *sumsq;      // [2 * layers, 16] fixed-point sums of squares of the rows before each norm
};

// Whether the tiled tcgen05 product takes a product of `rows` x `n` over `k` (the same rule as Runtime.takes_tcgen05 of
// the parts).  Measured on the 1B, 2B and 8B shapes against the library's product with separate elementwise kernels:
// from `min_rows` rows on, a product with at least `min_tiles` output tiles of 128 x 128 whose rows fill their tiles of
// 128 to `min_fill_pct` per cent (80) is as fast or faster here (fused epilogues, dependent launch); products of fewer tiles go to
// the library, whose smaller tiles and cuts of K fill the SMs better.  Very wide outputs (the logits) are taken from 17 rows.
static inline bool runner_takes_tcgen05(int sms, int min_rows, int min_tiles, int min_fill_pct, int rows, int n, int k) {
    if (rows <= 16 || k % 8) return false;
    const long long row_tiles = (rows + 127) / 128;
    if (row_tiles * ((n + 255) / 256) >= 3LL * sms) return true;
    if (rows < min_rows || rows * 100LL < (long long)min_fill_pct * row_tiles * 128) return false;
    return row_tiles * ((n + 127) / 128) >= min_tiles;
}

// Blocks that the few-rows tcgen05 kernel (jk_gemm_skinny) starts for a product with `n` output features over `k`:
// tiles of 128 features (64 for SwiGLU, whose tile holds as many up rows again); a product that is added into
// the residual stream splits K until the blocks fill the SMs twice, as long as a block keeps 8 steps of 64.
enum RunnerProductKind { RUNNER_F32 = 0, RUNNER_RESIDUAL = 1, RUNNER_SWIGLU = 2 };
static inline long long runner_skinny_blocks(int sms, int n, int k, int kind) {
    const int nk = (k + 63) / 64;
    if (kind == RUNNER_SWIGLU) return (n + 63) / 64;
    const int tiles = (n + 127) / 128;
    int splits = 1;
    if (kind == RUNNER_RESIDUAL) {
        splits = 2 * sms / tiles;
        if (splits > nk / 8) splits = nk / 8;
        if (splits < 1) splits = 1;
    }
    const int ksteps = (nk + splits - 1) / splits;
    return (long long)tiles * ((nk + ksteps - 1) / ksteps);
}

extern "C" {
int jk_runner_bind(const RunnerFns *fns);
int jk_runner_forward(const RunnerModel *, const RunnerLayer *, const RunnerStep *, const RunnerScratch *, cudaStream_t);
const RunnerFns *jk_runner_fns();      // the bound table (null before jk_runner_bind)
}
