/* A program without Python on the C interface (csrc/model_api.h): it makes a tiny model from numbers of its own,
 * runs a prompt whole and again in two portions plus single tokens, and compares the logits of the two ways;
 * then it generates a few tokens greedily.  Exit status 0 if all calls succeeded and the two ways agree.
 *
 *   cc -std=c99 c_api_program.c -o prog -L<build dir> -ljk_runner -Wl,-rpath,<build dir> -lm
 *   ./prog <build dir>        (the folder that holds libjk_*.so)
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "model_api.h"

static uint32_t lcg_state = 12345u;
static float uniform01(void) {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return (float)(lcg_state >> 8) / 16777216.0f;
}
static float gaussian(void) {                    /* sum of uniforms: close enough for weights */
    float s = 0.f;
    for (int i = 0; i < 6; ++i) s += uniform01();
    return (s - 3.0f) * 1.4142f;
}
static uint16_t to_bf16(float v) {               /* round to nearest even */
    uint32_t bits;
    memcpy(&bits, &v, 4);
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}
static uint16_t *matrix(size_t rows, size_t cols, float std) {
    uint16_t *m = (uint16_t *)malloc(rows * cols * sizeof(uint16_t));
    for (size_t i = 0; i < rows * cols; ++i) m[i] = to_bf16(gaussian() * std);
    return m;
}
static float *norm_weight(size_t n) {
    float *w = (float *)malloc(n * sizeof(float));
    for (size_t i = 0; i < n; ++i) w[i] = 1.0f + 0.02f * gaussian();
    return w;
}

#define LAYERS 2
#define CHECK(call)                                                           \
    do {                                                                      \
        if ((call) != 0) {                                                    \
            fprintf(stderr, "%s failed: %s\n", #call, jkLastError());         \
            return 1;                                                         \
        }                                                                     \
    } while (0)

int main(int argc, char **argv) {
    if (argc < 2) {
        fprintf(stderr, "usage: %s <folder of the built kernel modules>\n", argv[0]);
        return 2;
    }
    JkModelMeta meta;
    memset(&meta, 0, sizeof meta);
    meta.nlayer = LAYERS; meta.d = 128; meta.nh = 2; meta.nkvh = 1; meta.dh = 64; meta.di = 192; meta.dctx = 256; meta.dvoc = 333;
    meta.epsilon = 1e-5f; meta.theta = 10000.0f;
    meta.embed_scale = 5.0f; meta.residual_scale = 1.4f / sqrtf((float)LAYERS); meta.logit_scale = 1.0f / (128.0f / 32.0f);
    meta.end_token = 2;
    const float std = 0.09f;
    const size_t nq = (size_t)(meta.nh + 2 * meta.nkvh) * meta.dh;
    const void *attn_norm[LAYERS], *attn_qkv[LAYERS], *attn_o[LAYERS], *ffn_norm[LAYERS], *gate_up[LAYERS], *down[LAYERS];
    for (int l = 0; l < LAYERS; ++l) {
        attn_norm[l] = norm_weight(meta.d);
        attn_qkv[l] = matrix(nq, meta.d, std);
        attn_o[l] = matrix(meta.d, (size_t)meta.nh * meta.dh, std);
        ffn_norm[l] = norm_weight(meta.d);
        gate_up[l] = matrix(2 * (size_t)meta.di, meta.d, std);
        down[l] = matrix(meta.d, meta.di, std);
    }
    JkModelWeights w;
    memset(&w, 0, sizeof w);
    w.norm_dtype = 0;
    w.input_embd = matrix(meta.dvoc, meta.d, std);
    w.output_embd = w.input_embd;                /* tied */
    w.output_norm = norm_weight(meta.d);
    w.attn_norm = attn_norm; w.attn_qkv = attn_qkv; w.attn_o = attn_o; w.ffn_norm = ffn_norm; w.ffn_gate_up = gate_up; w.ffn_down = down;
    JkModelOptions opt;
    memset(&opt, 0, sizeof opt);
    opt.page_size = 16; opt.cache_tokens = 512; opt.max_step_tokens = 256; opt.kernel_dir = argv[1];

    struct JkModel *model = jkCreateModel(&meta, &w, &opt);
    if (model == NULL) {
        fprintf(stderr, "jkCreateModel failed: %s\n", jkLastError());
        return 1;
    }
    enum { N = 150 };
    uint32_t tokens[N];
    for (int i = 0; i < N; ++i) tokens[i] = (uint32_t)(uniform01() * meta.dvoc) % (uint32_t)meta.dvoc;
    float *whole = (float *)malloc(sizeof(float) * N * meta.dvoc), *cut = (float *)malloc(sizeof(float) * N * meta.dvoc);
    const int64_t pool = jkFreePages(model);

    struct JkKVCache *cache = jkCreateKVCache(model);
    uint32_t len = N, pos = 0;
    CHECK(jkForwardBatch(model, tokens, len, &len, 1, &pos, &cache, whole));
    jkDropKVCache(model, cache);

    cache = jkCreateKVCache(model);
    const uint32_t portions[] = {70, 2, 60};
    uint32_t done = 0;
    for (int p = 0; p < 3; ++p) {
        len = portions[p]; pos = done;
        CHECK(jkForwardBatch(model, tokens + done, len, &len, 1, &pos, &cache, cut + (size_t)done * meta.dvoc));
        done += len;
    }
    while (done < N) {                            /* the rest one token at a time */
        len = 1; pos = done;
        CHECK(jkForwardBatch(model, tokens + done, len, &len, 1, &pos, &cache, cut + (size_t)done * meta.dvoc));
        ++done;
    }
    double scale = 0.0, worst = 0.0;
    for (size_t i = 0; i < (size_t)N * meta.dvoc; ++i) {
        if (fabs(whole[i]) > scale) scale = fabs(whole[i]);
        if (fabs(whole[i] - cut[i]) > worst) worst = fabs(whole[i] - cut[i]);
    }
    printf("logits: largest %.3f, largest difference between the two ways of cutting %.4f\n", scale, worst);

    uint32_t next = 0, out = 0;
    float temperature = 0.f, topp = 1.f;
    uint32_t topk = 1;
    printf("greedy:");
    for (int i = 0; i < 8; ++i) {
        len = 1; pos = N + i;
        uint32_t tok = i == 0 ? tokens[N - 1] : next;
        if (i == 0) pos = N - 1;                  /* the last prompt token again: its cache entry is rewritten with the same values */
        else pos = N - 1 + i;
        CHECK(jkInferBatch(model, &tok, 1, &len, 1, &pos, &cache, &temperature, &topk, &topp, NULL, &out));
        next = out;
        printf(" %u", out);
    }
    printf("\n");
    jkDropKVCache(model, cache);
    const int leak = jkFreePages(model) != pool;
    jkDestroyModel(model);
    if (leak) { fprintf(stderr, "pages were lost\n"); return 1; }
    if (!(worst <= 0.025 * scale)) { fprintf(stderr, "the two ways of cutting disagree\n"); return 1; }
    return 0;
}
