// The native step: a model is a list of launch records that its parts emitted once; a step replays them.
//
// A record (RunnerOp) names one operation of a layer kind: what it reads and writes (buffer slots), its weights and
// its constants.  It does not name a kernel: which kernel runs it depends on the step (how many rows, which precision)
// and is decided here, in one place, by the rules of host_rules.h.  The records know nothing of the model they belong
// to, and this file knows nothing of any architecture: a layer that can be said in these operations runs natively,
// whatever it is part of; what cannot is run by its own code between two runs of records.
// (The reference's counterpart is the hand-written layer loop of inferDeviceBatch, src/models/jiuge/jiuge.cpp:126-305.)
#pragma once

#include <cuda_runtime.h>

#include "host_rules.h"

// ---- entry points of the kernel modules (signatures as in their sources) -------------------------------
extern "C" {
typedef int (*EmbedFn)(const int *, int, const void *, int, int, float, float *, cudaStream_t);
typedef int (*AddRmsnormFn)(float *, const void *, int, float, const float *, float, float, void *, int, const int *, int,
                            int, cudaStream_t);
typedef int (*ResidualAddFn)(float *, const void *, int, float, long long, cudaStream_t);
typedef int (*SwigluFn)(const void *, int, void *, int, int, int, cudaStream_t);
typedef int (*RopeKvFn)(const void *, int, int, const float *, const int *, const int *, const int *, int, int,
                        const float *, const float *, int, void *, void *, void *, int, int, int, int, int, int,
                        cudaStream_t);
typedef int (*GemmF32Fn)(const float *, int, const float *, int, const float *, float *, int, int, int, int, cudaStream_t);
typedef int (*LinearSmallFn)(const void *, const void *, void *, int, int, int, int, int, int, cudaStream_t);
typedef int (*LinearSmallQkvFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                const int *, const int *, const int *, int, int, int, int, int, int, cudaStream_t);
typedef int (*GemmTcgen05Fn)(const void *, const void *, void *, int, int, int, int, int, float, int *, int, cudaStream_t);
typedef int (*GemmTcgen05QkvFn)(const void *, const void *, int, int, void *, void *, void *, const float *, const float *,
                                const int *, const int *, const int *, int, int, int, int, int, int *, int, cudaStream_t);
typedef int (*AttentionRowsFn)(const void *, const void *, const void *, void *, int, const int *, const int *, const int *, int,
                               int, int, int, int, int, float, int, cudaStream_t);
typedef int (*AttentionDecodeFn)(const void *, const void *, const void *, void *, float *, const int *, int, const int *,
                                 const int *, const int *, int, int, int, int, int, float, int, int, cudaStream_t);
typedef int (*AttentionPrefillFn)(const void *, const void *, const void *, void *, const int *, int, int, const int *,
                                  const int *, const int *, int, int, int, int, int, float, int, cudaStream_t);
typedef int (*AttentionTcgen05Fn)(const void *, const void *, const void *, void *, const int *, int, int, const int *,
                                  const int *, const int *, int, int, int, int, int, int, float, int, int *, cudaStream_t);
typedef int (*SupportsFn)(int, int, int);
typedef int (*Supports1Fn)(int);
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
    ResidualAddFn residual_add;
    SwigluFn swiglu;
    RopeKvFn rope_kv;
    GemmF32Fn gemm_f32;
    LinearSmallFn linear_small;
    LinearSmallQkvFn linear_small_qkv;
    GemmTcgen05Fn gemm_tcgen05;
    GemmTcgen05QkvFn gemm_tcgen05_qkv;
    AttentionRowsFn attention_rows;
    AttentionDecodeFn attention_decode;
    AttentionPrefillFn attention_prefill;
    Supports1Fn attention_prefill_supports;
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

// ---- records ---------------------------------------------------------------------------------------------------
// Buffers of a step, by slot.  An operation reads and writes slots; the caller says where each slot lies (and how many
// bytes it holds) when it runs the records, so the same records run over the runner's own buffers or over a caller's
// tensors.
enum RunnerSlot {
    SLOT_X = 0,         // float32 [T, hidden]: the residual stream
    SLOT_DELTA,         // float32 [T, hidden]: a product that has not been added to the stream yet
    SLOT_H,             // activations [T, width]: a norm's output, the operand of the next product
    SLOT_Q,             // activations [T, heads * head size]: rotated queries
    SLOT_O,             // activations [T, heads * head size]: attention's output
    SLOT_ACT,           // activations [T, intermediate]: the gated feed-forward's inner activations
    SLOT_HW,            // activations [wanted rows, hidden]: the final norm's output
    SLOT_LOGITS,        // float32 [wanted rows, vocabulary]
    SLOT_TMP,           // float32: the product before an unfused rotation or activation ([T, widest such product])
    SLOT_DECODE,        // float32: partial results of the split-key attention
    RUNNER_SLOTS
};

enum RunnerOpKind {
    OP_EMBED = 1,       // out[t] = scale * table[tokens[t]]                                         -> float32 stream
    OP_NORM,            // stream += pending; out = out_scale * rmsnorm(stream[rows]) * weight        rows: all | wanted
    OP_QKV,             // [q | k | v] = in w^T (+ bias); rotate q and k; q -> out, k and v -> their pages
    OP_ATTENTION,       // out = softmax(q K^T * scale, causal, window) V over the paged cache
    OP_RESIDUAL,        // stream += scale * (in w^T)   (left pending for the next norm where no kernel adds in place)
    OP_GATE_UP,         // out = silu(in w_gate^T) * (in w_up^T), w = [gate rows; up rows]
    OP_LINEAR,          // out (float32) = in w^T (+ bias)                                            rows: all | wanted
};

struct RunnerOp {
    int kind;
    int in_slot, out_slot;
    int wanted_rows;            // 1: the operation works on the step's wanted rows only (final norm, output product)
    int n, k;                   // products: output features (GATE_UP: the width after the activation), input features
    int heads, kv_heads, head_dim, window, interleaved, writes_cache;
    int cache_group;            // which of the step's block tables indexes the pages
    int list_short, list_tiles; // ATTENTION: which of the step's lists hold its short rows and its tiles
    int w_dtype;                // EMBED: JK_F32 or JK_BF16 table
    int max_positions;          // ATTENTION: the longest context (bounds the keys of a row)
    float eps, scale, softmax_scale;    // NORM: eps, scale = the output's factor; RESIDUAL, EMBED: scale
    const void *w;              // the matrix [n (2n for GATE_UP), k] in the compute type; EMBED: the table
    const float *vec;           // NORM: the weight; QKV, LINEAR: the bias or null
    const float *cos_table, *sin_table;     // [positions, head_dim / 2] or null
    void *k_pages, *v_pages;    // [pages, kv_heads, page_size, head_dim] in the compute type
    int num_pages;
};

// What does not change from step to step and is no part's business.
struct RunnerEnv {
    int dtype;                  // JK_F32: every product on the CUDA cores in float32; JK_BF16
    int page_size, max_blocks;  // of every cache group
    int fused_norms;            // 1: steps of at most 16 rows run without norm kernels where the small-row kernels allow
    int plain_attention;        // 1: bfloat16 attention through the row kernel too
    int legacy_tensor_cores;    // 1: prefill attention on mma.sync even where tcgen05 is built
    jk::Routing routing;
    int *status;                // the word in which kernels record a bounded wait that ran out
};

// One step's batch (device arrays of the step's metadata buffer).
struct RunnerStep {
    int ntok, nreq, n_want;
    int context;                // the context length the step is planned for (the bucket of the live lengths)
    const int *tokens, *positions, *row_req, *req_start, *req_pos, *want_rows;
    const int *block_tables[jk::MAX_CACHE_GROUPS];
    const int *lists[jk::MAX_STEP_LISTS];     // work lists that mixers asked for; null with n == ntok means "rows 0..ntok-1"
    int list_n[jk::MAX_STEP_LISTS];
};

struct RunnerBuffers {
    void *slot[RUNNER_SLOTS];
    long long bytes[RUNNER_SLOTS];
    void *workspace;                // for the library
    long long workspace_bytes;
    unsigned long long *sumsq;      // [sumsq_rows, 16] fixed-point sums of squares, one row per record
    int sumsq_rows;
};

extern "C" {
int jk_runner_bind(const RunnerFns *fns);
// Runs records [first, first + count) of `ops`.  A product that adds into the stream may wait in SLOT_DELTA for the next
// norm to add it; with `flush` one that still waits when the records end is added before the call returns (for a caller
// that goes on with code of its own), without it the wait ends with the call (nobody reads the stream after a model's
// last record).
int jk_runner_run(const RunnerEnv *, const RunnerOp *ops, int first, int count, const RunnerStep *, const RunnerBuffers *,
                  int flush, cudaStream_t);
int jk_runner_slot_bytes(const RunnerEnv *, const RunnerOp *ops, int count, int max_rows, int max_want, long long *bytes);
int jk_runner_needs_gemm_tcgen05(const RunnerEnv *, const RunnerOp *ops, int count, int max_rows);
const RunnerFns *jk_runner_fns();      // the bound table (null before jk_runner_bind)
int jk_runner_launches();
// Emitters: the records of this architecture's standard parts, written once for the Python parts and the C interface.
// Each writes its records at `out` and returns their number.
int jk_emit_attention(RunnerOp *out, const void *w_qkv, const float *b_qkv, const void *w_o, int hidden, int heads, int kv_heads,
                      int head_dim, int window, float softmax_scale, float residual_scale, const float *cos_table,
                      const float *sin_table, int interleaved, int max_positions, void *k_pages, void *v_pages, int num_pages,
                      int cache_group, int writes_cache, int list_short, int list_tiles);
int jk_emit_swiglu(RunnerOp *out, const void *w_gate_up, const void *w_down, int hidden, int intermediate, float residual_scale);
int jk_emit_rmsnorm(RunnerOp *out, const float *weight, int size, float eps, float out_scale, int wanted_rows);
int jk_emit_embedding(RunnerOp *out, const void *table, int dtype, int hidden, float scale);
int jk_emit_output(RunnerOp *out, const void *w, int vocab, int hidden);
}
