/* A C interface to the engine for one GPU: create a model from host weights, create per-request
 * caches, and run batches that either sample one token per request or return the logits of every row.
 *
 * The calls and their arguments follow the reference's include/infinicore_infer/models/jiuge.h:50-118
 * (createJiugeModel, createKVCache, duplicateKVCache, dropKVCache, inferBatch, forwardBatch) with
 * three differences: there is one device, so no device list; the three MiniCPM scales are fields of the
 * meta instead of being multiplied into the weights by the caller (scripts/jiuge.py:97-114 does that);
 * and every call returns a status instead of ending the process, with the message in jkLastError().
 *
 * A request's cache is a list of pages of one pool that the model owns; pages are taken as the
 * request grows and go back to the pool in jkDropKVCache.  One model is driven by one thread at a time.
 */
#ifndef INFINICORE_INFER_B200_MODEL_API_H
#define INFINICORE_INFER_B200_MODEL_API_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

struct JkModel;
struct JkKVCache;

typedef struct {
    int32_t nlayer, d, nh, nkvh, dh, di, dctx, dvoc;
    float epsilon;                    /* of every RMSNorm */
    float theta;                      /* rotary base; <= 0: no position encoding */
    float embed_scale;                /* embedding rows are multiplied by this (scale_emb; 1 if unscaled) */
    float residual_scale;             /* each branch is multiplied by this before it is added (scale_depth / sqrt(nlayer)) */
    float logit_scale;                /* the final norm's output is multiplied by this (d / dim_model_base as an integer quotient, i.e. hidden_size // dim_model_base; 1 if unscaled) */
    int32_t end_token;
} JkModelMeta;

/* All arrays are in host memory and are copied to the device by jkCreateModel. */
typedef struct {
    int32_t norm_dtype;               /* 0: float32, 1: bfloat16 (the norm weights; kept in float32 on the device) */
    const void *input_embd;           /* bfloat16 [dvoc, d] */
    const void *output_norm;          /* [d] */
    const void *output_embd;          /* bfloat16 [dvoc, d]; the same pointer as input_embd for tied embeddings */
    const void *const *attn_norm;     /* nlayer * [d] */
    const void *const *attn_qkv;      /* nlayer * bfloat16 [(nh + 2 nkvh) * dh, d]: q rows, then k rows, then v rows */
    const void *const *attn_o;        /* nlayer * bfloat16 [d, nh * dh] */
    const void *const *ffn_norm;      /* nlayer * [d] */
    const void *const *ffn_gate_up;   /* nlayer * bfloat16 [2 di, d]: gate rows, then up rows */
    const void *const *ffn_down;      /* nlayer * bfloat16 [d, di] */
    const void *const *attn_qkv_b;    /* null, or nlayer * float32 [(nh + 2 nkvh) * dh]: the q, k and v biases (an entry may be null) */
} JkModelWeights;

typedef struct {
    int32_t device;                   /* CUDA device ordinal */
    int32_t page_size;                /* tokens per cache page (0: 64) */
    int64_t cache_tokens;             /* tokens the page pool holds over all live requests (0: dctx) */
    int32_t max_step_tokens;          /* most tokens one batch may bring (0: 2048) */
    const char *kernel_dir;           /* folder of the built kernel modules (libjk_*.so); null: the table that
                                         jk_runner_bind was given by the embedding program */
} JkModelOptions;

struct JkModel *jkCreateModel(const JkModelMeta *, const JkModelWeights *, const JkModelOptions *);
void jkDestroyModel(struct JkModel *);

struct JkKVCache *jkCreateKVCache(const struct JkModel *);
/* A new cache that holds a copy of the first seq_len tokens of another. */
struct JkKVCache *jkDuplicateKVCache(const struct JkModel *, const struct JkKVCache *, uint32_t seq_len);
void jkDropKVCache(const struct JkModel *, struct JkKVCache *);

/* One batch: request i brings req_lens[i] tokens that start at position req_pos[i] of its cache.
 * Samples one token per request from the logits of its last row (temperature 0 or topk 1: the
 * largest logit; topk 0: no limit); seeds may be null (all 0).  The uniform number of a draw depends
 * on (seed, position of the sampled token) only. */
int jkInferBatch(struct JkModel *, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
                 const uint32_t *req_pos, struct JkKVCache **kv_caches, const float *temperature, const uint32_t *topk,
                 const float *topp, const uint64_t *seeds, uint32_t *output);

/* The same batch, no sampling: float32 logits of every row, [ntok, dvoc], to host memory. */
int jkForwardBatch(struct JkModel *, const uint32_t *tokens, uint32_t ntok, const uint32_t *req_lens, uint32_t nreq,
                   const uint32_t *req_pos, struct JkKVCache **kv_caches, float *logits);

/* The kernel modules (libjk_<name>.so in kernel_dir) that a model of these sizes and options loads, as a
 * comma-separated list: what a build step has to provide. */
int jkKernelModules(const JkModelMeta *, const JkModelOptions *, char *out, int size);

/* Pages of the pool that no cache holds. */
int64_t jkFreePages(const struct JkModel *);
/* Kernels launched by the last batch. */
int32_t jkLastLaunches(const struct JkModel *);
const char *jkLastError(void);

#ifdef __cplusplus
}
#endif
#endif
