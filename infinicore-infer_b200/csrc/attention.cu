// Causal softmax attention over the paged key/value cache.
//
// One contract for every way of cutting the work: a step holds rows; row t is a query at
// absolute position positions[t] of request row_req[t]; its keys are the cache entries of
// that request at positions lo..positions[t], lo = 0 or positions[t] - window + 1.  Keys and
// values of the step's own rows were written to the pages before this kernel runs, so a
// portion of a prompt, a single decoded token and a whole prompt are the same case.
// Pages: [num_pages, nkvh, page_size, dh]; block_table[r, b] is the page of request r that
// holds positions b*page_size .. (b+1)*page_size-1.  Query head h reads key/value head
// h / (nh / nkvh).
//
// Scores, the running maximum, the normaliser and the output accumulator are float32; a
// masked key contributes exactly zero.  Scores are never materialised.
// (reference: the per-request loop of two batched products and a causal softmax over a
// materialised [nh, s, t] buffer, src/models/jiuge/jiuge.cpp:206-233.)
#include "common.cuh"

JK_DEFINE_ERROR_BUFFER(jk_attention)

struct AttnArgs {
    const void *q;          // [T, nh, dh]
    const void *k_pages;    // [pages, nkvh, page_size, dh]
    const void *v_pages;
    void *out;              // [T, nh, dh]
    const int *positions;   // [T]
    const int *row_req;     // [T]
    const int *block_table; // [nreq, max_blocks]
    int T, nh, nkvh, dh, page_size, max_blocks, window;
    float scale;
};

// ---------------------------------------------------------------------------------------
// Row kernel: one warp per (row, query head).  Lanes take one key each for the scores, then
// one slice of the head each for the weighted values.  Any head size, any page size, both
// element types; the result for a row does not depend on what else is in the batch.
// ---------------------------------------------------------------------------------------
constexpr int ROW_WARPS = 4;
constexpr int ROW_MAX_DH = 512;

template <typename T, int NS>     // NS: slices of 32 elements that cover one head
__global__ void __launch_bounds__(ROW_WARPS * 32)
attention_row_kernel(AttnArgs a) {
    extern __shared__ float q_smem[];          // [ROW_WARPS][dh]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.y;
    const int h = blockIdx.x * ROW_WARPS + warp;
    if (h >= a.nh) return;
    const int dh = a.dh;
    const int hk = h / (a.nh / a.nkvh);
    const int pos = a.positions[t];
    const int *bt = a.block_table + (size_t)a.row_req[t] * a.max_blocks;
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;

    float *qs = q_smem + warp * dh;
    const T *qrow = (const T *)a.q + ((size_t)t * a.nh + h) * dh;
    for (int e = lane; e < dh; e += 32) qs[e] = to_f32(qrow[e]);
    __syncwarp();

    const T *kp = (const T *)a.k_pages;
    const T *vp = (const T *)a.v_pages;
    const size_t head_off = (size_t)hk * a.page_size * dh;
    const size_t page_stride = (size_t)a.nkvh * a.page_size * dh;

    float m = -INFINITY, l = 0.f;
    float acc[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) acc[i] = 0.f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j <= pos;
        size_t row_off = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / a.page_size];
            row_off = (size_t)page * page_stride + head_off + (size_t)(j % a.page_size) * dh;
            const T *kr = kp + row_off;
            float dot = 0.f;
            for (int e = 0; e < dh; ++e) dot = fmaf(qs[e], to_f32(kr[e]), dot);
            s = dot * a.scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);          // exp(-inf) = 0 on the first chunk
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NS; ++i) acc[i] *= corr;
        const int n = min(32, pos - j0 + 1);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const unsigned long long off = __shfl_sync(0xffffffffu, (unsigned long long)row_off, jj);
            const T *vr = vp + off;
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                const int e = lane + 32 * i;
                if (e < dh) acc[i] = fmaf(pj, to_f32(vr[e]), acc[i]);
            }
        }
    }
    T *orow = (T *)a.out + ((size_t)t * a.nh + h) * dh;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < NS; ++i) {
        const int e = lane + 32 * i;
        if (e < dh) orow[e] = from_f32<T>(acc[i] * inv);
    }
}

static int check_args(const AttnArgs &a) {
    JK_REQUIRE(a.T > 0 && a.nh > 0 && a.nkvh > 0 && a.dh > 0, "attention: T %d heads %d/%d head size %d",
               a.T, a.nh, a.nkvh, a.dh);
    JK_REQUIRE(a.nh % a.nkvh == 0, "attention: %d query heads are no multiple of %d key heads", a.nh, a.nkvh);
    JK_REQUIRE(a.page_size > 0 && a.max_blocks > 0, "attention: page size %d, blocks %d", a.page_size, a.max_blocks);
    JK_REQUIRE(a.window >= 0, "attention: window %d", a.window);
    return JK_OK;
}

JK_EXPORT int jk_attention_rows(const void *q, const void *k_pages, const void *v_pages, void *out,
                                int dtype, const int *positions, const int *row_req,
                                const int *block_table, int max_blocks, int page_size, int T, int nh,
                                int nkvh, int dh, float scale, int window, cudaStream_t stream) {
    if (T == 0) return JK_OK;
    AttnArgs a{q, k_pages, v_pages, out, positions, row_req, block_table,
               T, nh, nkvh, dh, page_size, max_blocks, window, scale};
    if (int rc = check_args(a)) return rc;
    JK_REQUIRE(dh <= ROW_MAX_DH, "attention: head size %d exceeds %d", dh, ROW_MAX_DH);
    JK_REQUIRE(T <= 65535, "attention: %d rows exceed one launch (65535)", T);
    dim3 grid((nh + ROW_WARPS - 1) / ROW_WARPS, T);
    const size_t smem = (size_t)ROW_WARPS * dh * sizeof(float);
#define LAUNCH_ROWS(T, NS) attention_row_kernel<T, NS><<<grid, ROW_WARPS * 32, smem, stream>>>(a)
#define LAUNCH_ROWS_T(T)                                \
    do {                                                \
        if (dh <= 32) LAUNCH_ROWS(T, 1);                \
        else if (dh <= 64) LAUNCH_ROWS(T, 2);           \
        else if (dh <= 128) LAUNCH_ROWS(T, 4);          \
        else if (dh <= 256) LAUNCH_ROWS(T, 8);          \
        else LAUNCH_ROWS(T, 16);                        \
    } while (0)
    if (dtype == JK_F32)
        LAUNCH_ROWS_T(float);
    else if (dtype == JK_BF16)
        LAUNCH_ROWS_T(__nv_bfloat16);
    else
        JK_FAIL(JK_UNSUPPORTED, "attention: dtype %d", dtype);
    JK_CHECK_LAUNCH("attention_rows");
    return JK_OK;
}
