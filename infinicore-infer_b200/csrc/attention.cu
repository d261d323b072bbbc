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
#include "host_rules.h"

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
    pdl_trigger();
    pdl_wait();
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
#define LAUNCH_ROWS(T, NS) jk_launch(attention_row_kernel<T, NS>, grid, dim3(ROW_WARPS * 32), smem, stream, a)
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

// =======================================================================================
// bfloat16 fast paths.  Both read the same pages and block tables as the row kernel above
// and compute the same function; they differ in how the work is cut.
// =======================================================================================

// ---------------------------------------------------------------------------------------
// Decode kernel: for rows of requests that bring few rows (a decoded token, a short
// portion).  Work item = (row, key/value head, split of the key range).  The `HG` query heads
// of a key/value head that one block handles share every key and value it loads.  A group
// of LPR lanes owns one key at a time: each lane loads 16 bytes of the key row (coalesced:
// the groups of a warp read consecutive rows), the group's partial dot products are summed
// with shuffles, and every group keeps its own running (max, sum, accumulator), so nothing
// synchronises inside the loop.  Groups, warps and splits are merged at the end with the
// usual rule  acc = sum_i exp(m_i - M) acc_i,  l = sum_i exp(m_i - M) l_i.
// The split partials go to scratch memory and a second kernel merges them.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Rows of one request in one launch of a decode kernel: at most this many (jk::SHORT_ROWS of the work lists), so the
// kernel before a launch writes keys at most this far back from a row's own position.
constexpr int DECODE_FRESH_ROWS = jk::SHORT_ROWS;

struct DecodeArgs {
    const __nv_bfloat16 *q;        // [T, nh, dh]
    const __nv_bfloat16 *k_pages;  // [pages, nkvh, page_size, dh]
    const __nv_bfloat16 *v_pages;
    __nv_bfloat16 *out;            // [T, nh, dh]
    float *part_acc;               // [nrows, nh, splits, dh]
    float *part_ml;                // [nrows, nh, splits, 2]
    const int *rows;               // [nrows] row indices, or null for 0..nrows-1
    const int *positions;
    const int *row_req;
    const int *block_table;
    int nrows, nh, nkvh, dh, page_size, max_blocks, window, splits, page_shift;
    float scale_log2;              // softmax scale * log2(e)
    int cluster;                   // 1: the splits of a row are one thread-block cluster and merge among themselves
};

constexpr int DEC_WARPS = 4;
constexpr int DEC_UNROLL = 4;      // keys a group handles per stage
constexpr int DEC_STAGES = 4;      // stages of keys and values in flight per thread

__device__ __forceinline__ float fast_exp2(float x) {     // 2^x to 22 bits; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void bf16x8_to_float(const uint4 &raw, float (&f)[8]) {
    const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        f[2 * e] = __uint_as_float(w[e] << 16);
        f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
}

template <int LPR, int HG, bool POW2>   // lanes per key row, query heads per block, page size a power of two
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(DecodeArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int GROUPS = DEC_WARPS * 32 / LPR;
    const int split = blockIdx.x;
    const int g = a.nh / a.nkvh;
    const int hgroups = (g + HG - 1) / HG;
    const int hk = blockIdx.y / hgroups;
    const int h0 = hk * g + (blockIdx.y % hgroups) * HG;        // first query head of this block
    const int nheads = min(HG, hk * g + g - h0);
    const int ri = blockIdx.z;
    const int t = a.rows ? a.rows[ri] : ri;
    const int pos = a.positions[t];
    const int *bt = a.block_table + (size_t)a.row_req[t] * a.max_blocks;
    const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
    const int nkeys = pos - lo + 1;
    int chunk = (nkeys + a.splits - 1) / a.splits;
    chunk = (chunk + GROUPS - 1) / GROUPS * GROUPS;
    const int k_begin = lo + split * chunk;
    const int k_end = min(pos + 1, k_begin + chunk);             // exclusive

    const int lane_in = threadIdx.x % LPR;                       // which 16 bytes of the row
    const int group = threadIdx.x / LPR;
    const int dh = a.dh;
    const bool lane_ok = lane_in * 8 < dh;
    const size_t head_off = (size_t)hk * a.page_size * dh + lane_in * 8;
    const size_t page_stride = (size_t)a.nkvh * a.page_size * dh;

    float qf[HG][8];
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
#pragma unroll
        for (int e = 0; e < 8; ++e) qf[hh][e] = 0.f;
        if (hh < nheads && lane_ok) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(a.q + ((size_t)t * a.nh + h0 + hh) * dh + lane_in * 8);
            const __nv_bfloat162 *p2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(p2[e]);
                qf[hh][2 * e] = f.x * a.scale_log2;
                qf[hh][2 * e + 1] = f.y * a.scale_log2;
            }
        }
    }
    float m[HG], l[HG], acc[HG][8];
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
        m[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[hh][e] = 0.f;
    }

    // Keys and values travel through a ring in shared memory that is private to each thread: the
    // thread that issues a 16-byte cp.async is the one that later reads it, so nothing but the
    // thread's own cp.async.wait_group orders them, and DEC_STAGES stages stay in flight whatever
    // the register budget.  The trip count is the same for every thread of the block and no thread
    // skips a shuffle: a key beyond the range scores -inf and so weighs exactly zero.
    extern __shared__ __align__(16) float dec_smem[];
    uint4 *ring = reinterpret_cast<uint4 *>(dec_smem);          // [DEC_STAGES][DEC_UNROLL][2][threads]
    const int nthreads = DEC_WARPS * 32;
    const int n_iter = (k_end - k_begin + GROUPS * DEC_UNROLL - 1) / (GROUPS * DEC_UNROLL);
    auto issue = [&](int it) {
        if (it < n_iter) {
            const int base = k_begin + it * GROUPS * DEC_UNROLL;
            uint4 *slot = ring + (size_t)(it % DEC_STAGES) * DEC_UNROLL * 2 * nthreads + threadIdx.x;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                const int j = base + group + u * GROUPS;
                if (j < k_end && lane_ok) {
                    const int blk = POW2 ? (j >> a.page_shift) : (j / a.page_size);
                    const int in_page = POW2 ? (j & (a.page_size - 1)) : (j - blk * a.page_size);
                    const size_t off = (size_t)bt[blk] * page_stride + head_off + (size_t)in_page * dh;
                    cp_async16(slot + (u * 2) * nthreads, a.k_pages + off);
                    cp_async16(slot + (u * 2 + 1) * nthreads, a.v_pages + off);
                }
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int s0 = 0; s0 < DEC_STAGES - 1; ++s0) issue(s0);
    for (int it = 0; it < n_iter; ++it) {
        issue(it + DEC_STAGES - 1);
        cp_async_wait<DEC_STAGES - 1>();
        const int base = k_begin + it * GROUPS * DEC_UNROLL;
        const uint4 *slot = ring + (size_t)(it % DEC_STAGES) * DEC_UNROLL * 2 * nthreads + threadIdx.x;
        uint4 kr[DEC_UNROLL], vr[DEC_UNROLL];
        bool ok[DEC_UNROLL];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            const int j = base + group + u * GROUPS;
            ok[u] = j < k_end;
            kr[u] = make_uint4(0, 0, 0, 0); vr[u] = make_uint4(0, 0, 0, 0);
            if (ok[u] && lane_ok) {
                kr[u] = slot[(u * 2) * nthreads];
                vr[u] = slot[(u * 2 + 1) * nthreads];
            }
        }
        float sc[HG][DEC_UNROLL];
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float kf[8];
            bf16x8_to_float(kr[u], kf);
#pragma unroll
            for (int hh = 0; hh < HG; ++hh) {
                float s = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) s = fmaf(qf[hh][e], kf[e], s);
                sc[hh][u] = s;
            }
        }
#pragma unroll
        for (int hh = 0; hh < HG; ++hh) {
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
#pragma unroll
                for (int o = LPR / 2; o > 0; o >>= 1) sc[hh][u] += __shfl_xor_sync(0xffffffffu, sc[hh][u], o);
                if (!ok[u]) sc[hh][u] = -INFINITY;
            }
            float m_new = m[hh];
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) m_new = fmaxf(m_new, sc[hh][u]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fast_exp2(m[hh] - m_use);
            m[hh] = m_new;
            float psum = 0.f;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) { sc[hh][u] = fast_exp2(sc[hh][u] - m_use); psum += sc[hh][u]; }
            l[hh] = l[hh] * corr + psum;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[hh][e] *= corr;
        }
#pragma unroll
        for (int u = 0; u < DEC_UNROLL; ++u) {
            float vf[8];
            bf16x8_to_float(vr[u], vf);
#pragma unroll
            for (int hh = 0; hh < HG; ++hh)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[hh][e] = fmaf(sc[hh][u], vf[e], acc[hh][e]);
        }
    }

    // merge the groups of this block (the ring's memory is free once every thread has left the loop)
    __syncthreads();
    float *s_ml = dec_smem;                                   // [GROUPS][HG][2]
    float *s_acc = dec_smem + GROUPS * HG * 2;                // [GROUPS][HG][LPR*8]
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
        if (lane_in == 0) {
            s_ml[(group * HG + hh) * 2] = m[hh];
            s_ml[(group * HG + hh) * 2 + 1] = l[hh];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) s_acc[((size_t)group * HG + hh) * (LPR * 8) + lane_in * 8 + e] = acc[hh][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nheads * dh; i += blockDim.x) {
        const int hh = i / dh, e = i - hh * dh;
        float M = -INFINITY;
        for (int gi = 0; gi < GROUPS; ++gi) M = fmaxf(M, s_ml[(gi * HG + hh) * 2]);
        float L = 0.f, A = 0.f;
        if (M > -INFINITY) {
            for (int gi = 0; gi < GROUPS; ++gi) {
                const float w = exp2f(s_ml[(gi * HG + hh) * 2] - M);
                L += w * s_ml[(gi * HG + hh) * 2 + 1];
                A += w * s_acc[((size_t)gi * HG + hh) * (LPR * 8) + e];
            }
        }
        const size_t slot = ((size_t)ri * a.nh + h0 + hh) * a.splits + split;
        if (a.splits == 1) {
            a.out[((size_t)t * a.nh + h0 + hh) * dh + e] = __float2bfloat16_rn(A / L);
        } else {
            a.part_acc[slot * dh + e] = A;
            if (e == 0) { a.part_ml[slot * 2] = M; a.part_ml[slot * 2 + 1] = L; }
        }
    }
}

// One block per (query head, row): merge the splits' partial results.
__global__ void attention_combine_kernel(DecodeArgs a) {
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x, ri = blockIdx.y;
    const int t = a.rows ? a.rows[ri] : ri;
    const size_t base = ((size_t)ri * a.nh + h) * a.splits;
    float M = -INFINITY;
    for (int s = 0; s < a.splits; ++s) M = fmaxf(M, a.part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < a.splits; ++s) {
        const float ms = a.part_ml[(base + s) * 2];
        if (ms > -INFINITY) L += exp2f(ms - M) * a.part_ml[(base + s) * 2 + 1];
    }
    for (int e = threadIdx.x; e < a.dh; e += blockDim.x) {
        float A = 0.f;
        for (int s = 0; s < a.splits; ++s) {
            const float ms = a.part_ml[(base + s) * 2];
            if (ms > -INFINITY) A += exp2f(ms - M) * a.part_acc[(base + s) * a.dh + e];
        }
        a.out[((size_t)t * a.nh + h) * a.dh + e] = __float2bfloat16_rn(A / L);
    }
}

template <int LPR, int HG, bool POW2>
static int launch_decode(const DecodeArgs &a, cudaStream_t stream) {
    constexpr int GROUPS = DEC_WARPS * 32 / LPR;
    const int g = a.nh / a.nkvh;
    const int hgroups = (g + HG - 1) / HG;
    dim3 grid(a.splits, a.nkvh * hgroups, a.nrows);
    const size_t merge_bytes = (size_t)GROUPS * HG * (2 + LPR * 8) * sizeof(float);
    const size_t ring_bytes = (size_t)DEC_STAGES * DEC_UNROLL * 2 * DEC_WARPS * 32 * sizeof(uint4);
    const size_t smem = merge_bytes > ring_bytes ? merge_bytes : ring_bytes;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<LPR, HG, POW2>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "attention_decode: %s", cudaGetErrorString(e));
    }
    jk_launch(attention_decode_kernel<LPR, HG, POW2>, grid, dim3(DEC_WARPS * 32), smem, stream, a);
    JK_CHECK_LAUNCH("attention_decode");
    if (a.splits > 1) {
        jk_launch(attention_combine_kernel, dim3(a.nh, a.nrows), dim3(64), 0, stream, a);
        JK_CHECK_LAUNCH("attention_combine");
    }
    return JK_OK;
}

static int decode_gqa(const DecodeArgs &a, cudaStream_t stream, bool *taken);      // further down, beside its helpers

// Scratch floats that `jk_attention_decode` needs for (nrows, nh, dh, splits).
JK_EXPORT long long jk_attention_decode_scratch_floats(int nrows, int nh, int dh, int splits) {
    if (splits <= 1) return 0;
    return (long long)nrows * nh * splits * (dh + 2);
}

JK_EXPORT int jk_attention_decode(const void *q, const void *k_pages, const void *v_pages, void *out,
                                  float *scratch, const int *rows, int nrows, const int *positions,
                                  const int *row_req, const int *block_table, int max_blocks,
                                  int page_size, int nh, int nkvh, int dh, float scale, int window,
                                  int splits, cudaStream_t stream) {
    if (nrows == 0) return JK_OK;
    JK_REQUIRE(nrows > 0 && nh > 0 && nkvh > 0 && nh % nkvh == 0, "attention_decode: rows %d heads %d/%d", nrows, nh, nkvh);
    JK_REQUIRE(dh % 8 == 0 && dh >= 8 && dh <= 256, "attention_decode: head size %d (takes multiples of 8 up to 256)", dh);
    JK_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "attention_decode: page size %d, blocks %d, window %d",
               page_size, max_blocks, window);
    JK_REQUIRE(splits >= 1 && splits <= 256, "attention_decode: %d splits", splits);
    JK_REQUIRE(splits == 1 || scratch != nullptr, "attention_decode: %d splits need scratch memory", splits);
    JK_REQUIRE(nrows <= 65535, "attention_decode: %d rows exceed one launch", nrows);
    DecodeArgs a{(const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_pages, (const __nv_bfloat16 *)v_pages,
                 (__nv_bfloat16 *)out, scratch,
                 scratch ? scratch + (size_t)nrows * nh * splits * dh : nullptr,
                 rows, positions, row_req, block_table,
                 nrows, nh, nkvh, dh, page_size, max_blocks, window, splits, 0,
                 scale * 1.4426950408889634f};
    const bool pow2 = (page_size & (page_size - 1)) == 0;
    while ((1 << a.page_shift) < page_size) ++a.page_shift;
    const int g = nh / nkvh;
    const int lanes = dh / 8;
    {
        bool taken = false;
        const int rc = decode_gqa(a, stream, &taken);
        if (taken) return rc;
    }
#define DEC_DISPATCH_P2(LPR, HG) return pow2 ? launch_decode<LPR, HG, true>(a, stream) : launch_decode<LPR, HG, false>(a, stream)
#define DEC_DISPATCH_HG(LPR)                                         \
    do {                                                             \
        if (g == 1) DEC_DISPATCH_P2(LPR, 1);                         \
        if (g == 2) DEC_DISPATCH_P2(LPR, 2);                         \
        if (g == 3) DEC_DISPATCH_P2(LPR, 3);                         \
        DEC_DISPATCH_P2(LPR, 4);                                     \
    } while (0)
    if (lanes <= 2) DEC_DISPATCH_HG(2);
    if (lanes <= 4) DEC_DISPATCH_HG(4);
    if (lanes <= 8) DEC_DISPATCH_HG(8);
    if (lanes <= 16) DEC_DISPATCH_HG(16);
    DEC_DISPATCH_HG(32);
#undef DEC_DISPATCH_HG
#undef DEC_DISPATCH_P2
}

// ---------------------------------------------------------------------------------------
// Prefill kernel: for requests that bring many rows.  Work item = (tile of 64 query rows of
// one request, query head); 4 warps of 16 rows.  Keys and values are gathered page by page
// into shared memory with cp.async (two buffers), scores and weighted values run on the
// tensor cores (mma.sync m16n8k16, bfloat16 in, float32 out), the softmax is the online one
// in float32 registers.  Rows beyond the request's end repeat its last row and are not stored.
// Shared rows are padded by 16 bytes, which makes every ldmatrix conflict-free for any head
// size that is a multiple of 16.
// ---------------------------------------------------------------------------------------
struct PrefillArgs {
    const __nv_bfloat16 *q;
    const __nv_bfloat16 *k_pages;
    const __nv_bfloat16 *v_pages;
    __nv_bfloat16 *out;
    const int *tiles;        // [ntiles][2]: batch entry, first row of the tile (row index in the step)
    const int *req_start;    // [nreq + 1]
    const int *req_pos;      // [nreq]
    const int *block_table;  // [nreq, max_blocks]
    int ntiles, nh, nkvh, page_size, max_blocks, window, tile_rows;
    float scale_log2;
};

constexpr int PF_BM = 64;


__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void *smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void *smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned *>(&v);
}

template <int DH, int BN>
__global__ void __launch_bounds__(128, DH <= 64 ? 4 : (DH <= 128 ? 2 : 1))
attention_prefill_kernel(PrefillArgs a) {
    pdl_trigger();
    pdl_wait();
    constexpr int STRIDE = DH + 8;            // elements per shared row
    constexpr int CH = DH / 8;                // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char pf_smem[];
    __nv_bfloat16 *Qs = reinterpret_cast<__nv_bfloat16 *>(pf_smem);
    __nv_bfloat16 *Ks = Qs + PF_BM * STRIDE;              // [2][BN][STRIDE]
    __nv_bfloat16 *Vs = Ks + 2 * BN * STRIDE;             // [2][BN][STRIDE]

    // the step's tiles are tile_rows rows long; a block takes 64 of them.  Blocks start in the order of
    // the tile list (the caller lists the tiles with the most keys first), all heads of a tile together.
    const int parts = a.tile_rows / PF_BM;
    const int idx = blockIdx.y;
    const int tile = idx / parts;
    const int h = blockIdx.x;
    const int hk = h / (a.nh / a.nkvh);
    const int r = a.tiles[2 * tile];
    const int row0 = a.tiles[2 * tile + 1] + (idx % parts) * PF_BM;
    if (row0 >= a.req_start[r + 1]) return;               // this part of the tile lies beyond the request
    const int nrows = min(PF_BM, a.req_start[r + 1] - row0);
    const int p0 = a.req_pos[r] + (row0 - a.req_start[r]);   // position of the tile's first row
    const int p_last = p0 + nrows - 1;
    const int lo = (a.window > 0 && p0 - a.window + 1 > 0) ? p0 - a.window + 1 : 0;
    const int *bt = a.block_table + (size_t)r * a.max_blocks;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t page_stride = (size_t)a.nkvh * a.page_size * DH;
    const size_t head_off = (size_t)hk * a.page_size * DH;

    // the query tile
    for (int c = tid; c < PF_BM * CH; c += 128) {
        const int row = c / CH, ch = c - row * CH;
        const int rr = min(row, nrows - 1);
        cp_async16(Qs + row * STRIDE + ch * 8, a.q + ((size_t)(row0 + rr) * a.nh + h) * DH + ch * 8);
    }
    auto load_kv = [&](int kv0, int buf) {
        __nv_bfloat16 *kd = Ks + buf * BN * STRIDE, *vd = Vs + buf * BN * STRIDE;
        for (int c = tid; c < BN * CH; c += 128) {
            const int row = c / CH, ch = c - row * CH;
            const int key = kv0 + row;
            if (key <= p_last) {
                const size_t off = (size_t)bt[key / a.page_size] * page_stride + head_off +
                                   (size_t)(key % a.page_size) * DH + ch * 8;
                cp_async16(kd + row * STRIDE + ch * 8, a.k_pages + off);
                cp_async16(vd + row * STRIDE + ch * 8, a.v_pages + off);
            } else {
                *reinterpret_cast<uint4 *>(kd + row * STRIDE + ch * 8) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(vd + row * STRIDE + ch * 8) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    const int kv_first = lo / BN * BN;
    load_kv(kv_first, 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // query fragments stay in registers
    unsigned qf[DH / 16][4];
#pragma unroll
    for (int kk = 0; kk < DH / 16; ++kk)
        ldmatrix_x4(qf[kk], Qs + (warp * 16 + (lane & 15)) * STRIDE + kk * 16 + (lane >> 4) * 8);

    const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
    const int pos_a = p0 + min(row_a, nrows - 1), pos_b = p0 + min(row_b, nrows - 1);
    const int lo_a = a.window > 0 ? pos_a - a.window + 1 : 0, lo_b = a.window > 0 ? pos_b - a.window + 1 : 0;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    float o[DH / 8][4];
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

    int buf = 0;
    for (int kv0 = kv_first; kv0 <= p_last; kv0 += BN, buf ^= 1) {
        if (kv0 + BN <= p_last) load_kv(kv0 + BN, buf ^ 1);       // prefetch the next tile
        cp_async_commit();

        const __nv_bfloat16 *kt = Ks + buf * BN * STRIDE, *vt = Vs + buf * BN * STRIDE;
        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
#pragma unroll
            for (int n2 = 0; n2 < BN / 16; ++n2) {
                unsigned b[4];
                ldmatrix_x4(b, kt + (n2 * 16 + (lane & 7) + ((lane >> 4) << 3)) * STRIDE + kk * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[2 * n2], qf[kk], b[0], b[1]);
                mma_bf16(s[2 * n2 + 1], qf[kk], b[2], b[3]);
            }
        }
        // mask and running maximum on the raw scores (the softmax scale is positive, so it commutes
        // with the maximum and is applied inside the exponent by one fused multiply-add)
        const bool all_visible = (kv0 + BN - 1 <= p0) && (a.window == 0 || kv0 >= p_last - a.window + 1);
        float mx_a = -INFINITY, mx_b = -INFINITY;
        if (!all_visible) {
#pragma unroll
            for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = kv0 + i * 8 + 2 * (lane & 3) + (c & 1);
                    const bool ok = c < 2 ? (j <= pos_a && j >= lo_a) : (j <= pos_b && j >= lo_b);
                    if (!ok) s[i][c] = -INFINITY;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) {
            mx_a = fmaxf(mx_a, fmaxf(s[i][0], s[i][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[i][2], s[i][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);          // raw maxima
        const float use_a = mn_a == -INFINITY ? 0.f : mn_a * a.scale_log2, use_b = mn_b == -INFINITY ? 0.f : mn_b * a.scale_log2;
        const float corr_a = fast_exp2(m_a * a.scale_log2 - use_a), corr_b = fast_exp2(m_b * a.scale_log2 - use_b);
        m_a = mn_a; m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) {
            s[i][0] = fast_exp2(fmaf(s[i][0], a.scale_log2, -use_a)); s[i][1] = fast_exp2(fmaf(s[i][1], a.scale_log2, -use_a));
            s[i][2] = fast_exp2(fmaf(s[i][2], a.scale_log2, -use_b)); s[i][3] = fast_exp2(fmaf(s[i][3], a.scale_log2, -use_b));
            sum_a += s[i][0] + s[i][1]; sum_b += s[i][2] + s[i][3];
        }
        l_a = l_a * corr_a + sum_a; l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
        // weighted values
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            unsigned p[4];
            p[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            p[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            p[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            p[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < DH / 16; ++d2) {
                unsigned b[4];
                ldmatrix_x4_trans(b, vt + (ks * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * STRIDE + d2 * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * d2], p, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], p, b[2], b[3]);
            }
        }
        cp_async_wait<0>();
        __syncthreads();
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = 1.f / l_a, inv_b = 1.f / l_b;
#pragma unroll
    for (int i = 0; i < DH / 8; ++i) {
        const int col = i * 8 + 2 * (lane & 3);
        if (row_a < nrows)
            *reinterpret_cast<__nv_bfloat162 *>(a.out + ((size_t)(row0 + row_a) * a.nh + h) * DH + col) =
                __floats2bfloat162_rn(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < nrows)
            *reinterpret_cast<__nv_bfloat162 *>(a.out + ((size_t)(row0 + row_b) * a.nh + h) * DH + col) =
                __floats2bfloat162_rn(o[i][2] * inv_b, o[i][3] * inv_b);
    }
}

template <int DH, int BN>
static int launch_prefill(const PrefillArgs &a, cudaStream_t stream) {
    const size_t smem = (size_t)(PF_BM + 4 * BN) * (DH + 8) * sizeof(__nv_bfloat16);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<DH, BN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "attention_prefill: %s", cudaGetErrorString(e));
    }
    jk_launch(attention_prefill_kernel<DH, BN>, dim3(a.nh, a.ntiles * (a.tile_rows / PF_BM)), dim3(128), smem, stream, a);
    JK_CHECK_LAUNCH("attention_prefill");
    return JK_OK;
}


// =======================================================================================
// Decode attention for grouped heads (several query heads per key/value head): the group is
// the M side of mma.sync m16n8k16, so a block reads its keys and values once for up to 16 query heads
// and does the two products on the tensor cores.  Grid (split, key/value head x head tile, row); a block
// walks over its range of keys in tiles of 64 that cp.async brings into a swizzled ring (three tiles of
// keys and values in flight); warp w takes keys 16w..16w+15 of every tile with its own running maximum,
// sum and accumulator, the four are merged through shared memory at the end.  Output as the kernel
// above: final rows when there is one split, partial (accumulator, maximum, sum) else.
// =======================================================================================
constexpr int GQ_STAGES = 3, GQ_HEADS = 16;

__device__ __forceinline__ void cp_async16_or_zero(void *smem, const void *gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;              // 0 bytes read: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}

// A float of another block of this block's cluster, at the place where `local` lies in this block.
__device__ __forceinline__ float ld_cluster_f32(const float *local, unsigned rank) {
    unsigned addr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(addr) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {      // every thread of every block of the cluster
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// NW warps take 16 keys each of a tile of NW * 16 keys: four as a rule; eight (tiles of 128 keys, one block an SM with
// heads of 128) for launches of so few blocks that every SM has at most one: a block's pace is set by the chain of a
// tile's instructions in each warp, and twice the warps pass twice the keys in the same time.
template <int DH, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_decode_gqa_kernel(DecodeArgs a) {
    constexpr int KEYS = NW * 16, NT = NW * 32;
    static_assert(DH == 64 || DH == 128, "the swizzle chunk ^ (key & 7) needs rows of 8 or 16 chunks");
    constexpr int CH = DH / 8;                     // 16-byte chunks of a key row
    constexpr int TILE = KEYS * CH;             // uint4 per tile of keys (or values)
    extern __shared__ uint4 gq_smem[];
    pdl_trigger();
    const int split = blockIdx.x, kh = blockIdx.y % a.nkvh, ht = blockIdx.y / a.nkvh, ri = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = a.nh / a.nkvh;
    const int h0 = kh * g + ht * GQ_HEADS;         // first query head of this block
    const int heads = min(GQ_HEADS, g - ht * GQ_HEADS);
    // Not yet the wait for the kernel before this one: what that kernel writes are the queries and, in the cache, the
    // keys and values of this step's own rows (at most DECODE_FRESH_ROWS positions back from a row's own: the work
    // lists send requests with more rows elsewhere).  The step's metadata and all older keys are there already, so the
    // block finds its pages and asks for its first tiles of old keys while the kernel before still runs.
    const int t = a.rows ? a.rows[ri] : ri;
    const int pos = a.positions[t], req = a.row_req[t];
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0, hi = pos + 1;
    const int tiles_all = (hi - lo + KEYS - 1) / KEYS;
    // at least two tiles per split (a block's fixed part costs more than a tile): short contexts use fewer of the
    // splits that the grid was sized for, the others report that they saw nothing
    const int per = max(2, (tiles_all + a.splits - 1) / a.splits);
    const int k0 = lo + split * per * KEYS, k1 = min(hi, k0 + per * KEYS);
    const size_t pbase = ((size_t)ri * a.nh + h0) * a.splits + split;      // + head * splits
    if (k0 >= k1 && !a.cluster) {                  // nothing for this split: the merge skips it (in a cluster the block
                                                   // goes on with no tiles: the others wait for it at the barriers)
        pdl_wait();                                // the scratch may still be read by a merge of the layer before
        if (a.splits > 1 && threadIdx.x < heads) {
            a.part_ml[(pbase + (size_t)threadIdx.x * a.splits) * 2] = -INFINITY;
            a.part_ml[(pbase + (size_t)threadIdx.x * a.splits) * 2 + 1] = 0.f;
        }
        return;
    }
    const int ntiles = (k1 - k0 + KEYS - 1) / KEYS;
    const int *bt = a.block_table + (size_t)req * a.max_blocks;

    // Where a tile's 64 keys lie (element offset of the key's row in the pages, -1 beyond the range) is worked out
    // once per tile by 64 threads into a table of two turns; the copies then cost a table read each.
    long long *tab = reinterpret_cast<long long *>(gq_smem + (size_t)GQ_STAGES * 2 * TILE);       // [2][KEYS]
    // in two halves: the read of the block table is issued at the start of an iteration and used at its end, so
    // that the warp does not sit on it
    auto locate_begin = [&](int i) -> int {
        const int kj = k0 + i * KEYS + threadIdx.x;
        return threadIdx.x < KEYS && kj < k1 ? bt[kj / a.page_size] : -1;
    };
    auto locate_end = [&](int i, int page) {
        if (threadIdx.x < KEYS) {
            const int kj = k0 + i * KEYS + threadIdx.x;
            tab[(i & 1) * KEYS + threadIdx.x] =
                page < 0 ? -1 : (((long long)page * a.nkvh + kh) * a.page_size + kj % a.page_size) * DH;
        }
    };
    auto locate_tile = [&](int i) { locate_end(i, locate_begin(i)); };
    // 16 bytes of key `key` of a tile lie at chunk ^ (key & 7): ldmatrix reads eight rows without conflicts.  A
    // thread copies the same chunk of every (128 / CH)-th key, so its swizzled chunk never changes.
    constexpr int KEYS_PER_PASS = NT / CH;
    const int my_key = threadIdx.x / CH, my_ch = threadIdx.x % CH;
    const int my_slot = my_key * CH + (my_ch ^ (my_key & 7));
    auto load_tile = [&](int i) {
        uint4 *kd = gq_smem + (size_t)(i % GQ_STAGES) * 2 * TILE + my_slot, *vd = kd + TILE;
        const long long *where = tab + (i & 1) * KEYS + my_key;
#pragma unroll
        for (int c = 0; c < KEYS / KEYS_PER_PASS; ++c) {
            const long long off = where[c * KEYS_PER_PASS];
            const bool valid = off >= 0;
            const size_t src = valid ? (size_t)off + my_ch * 8 : 0;
            cp_async16_or_zero(kd + c * KEYS_PER_PASS * CH, a.k_pages + src, valid);
            cp_async16_or_zero(vd + c * KEYS_PER_PASS * CH, a.v_pages + src, valid);
        }
    };
    locate_tile(0);
    locate_tile(1);
    __syncthreads();
    // the first tiles, as far as they hold old keys only
    const int old_hi = pos - (DECODE_FRESH_ROWS - 1);
    int first = 0;
    for (; first < GQ_STAGES - 1; ++first) {
        if (first < ntiles && min(k1, k0 + (first + 1) * KEYS) > old_hi) break;
        if (first < ntiles) load_tile(first);
        cp_async_commit();
    }
    pdl_wait();
    {
        // the queries of the group's heads are one contiguous piece of q; heads beyond the group read as zeros
        uint4 *qs = gq_smem + (size_t)GQ_STAGES * 2 * TILE + 2 * KEYS * sizeof(long long) / sizeof(uint4);
        const uint4 *qg = reinterpret_cast<const uint4 *>(a.q + ((size_t)t * a.nh + h0) * DH);
        for (int idx = threadIdx.x; idx < GQ_HEADS * CH; idx += NT) {
            const int head = idx / CH, ch = idx % CH;
            qs[head * CH + (ch ^ (head & 7))] = head < heads ? qg[idx] : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    for (int i = first; i < GQ_STAGES - 1; ++i) {
        if (i < ntiles) load_tile(i);
        cp_async_commit();
    }
    __syncthreads();                               // the first tables have been read (and the queries are written)
    locate_tile(2);
    // the group's queries as A fragments: rows are heads (zero beyond the group), 16 dims per step; they came
    // with the first tile's group of copies into their own 16 x DH corner of shared memory
    unsigned qf[DH / 16][4];
    {
        cp_async_wait<GQ_STAGES - 2>();
        __syncthreads();
        const uint4 *qs = gq_smem + (size_t)GQ_STAGES * 2 * TILE + 2 * KEYS * sizeof(long long) / sizeof(uint4);
        // matrices: (heads 0-7, dims 0-7), (heads 8-15, dims 0-7), (heads 0-7, dims 8-15), (heads 8-15, dims 8-15)
        const int head = (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
            const int ch = kk * 2 + (lane >> 4);
            ldmatrix_x4(qf[kk], qs + head * CH + (ch ^ (head & 7)));
        }
    }
    float o[DH / 8][4];
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // heads lane / 4 and lane / 4 + 8

    for (int i = 0; i < ntiles; ++i) {
        cp_async_wait<GQ_STAGES - 2>();
        __syncthreads();                           // tile i has landed for everyone; tile i - 1 is no longer read
        const int page_ahead = locate_begin(i + GQ_STAGES);
        if (i + GQ_STAGES - 1 < ntiles) load_tile(i + GQ_STAGES - 1);
        cp_async_commit();
        const uint4 *kt = gq_smem + (size_t)(i % GQ_STAGES) * 2 * TILE, *vt = kt + TILE;
        const int kw = k0 + i * KEYS + warp * 16;          // this warp's first key of the tile
        if (kw >= k1) {                                        // warp-uniform: no key of the tile is this warp's
            locate_end(i + GQ_STAGES, page_ahead);
            continue;
        }
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            float sd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};      // odd steps: two chains of half the length
            const int key = warp * 16 + ((lane >> 4) << 3) + (lane & 7);
            const uint4 *krow = kt + key * CH;
#pragma unroll
            for (int kk = 0; kk < DH / 16; ++kk) {
                // matrices: (keys 0-7, dims 0-7), (keys 0-7, dims 8-15), (keys 8-15, dims 0-7), (keys 8-15, dims 8-15)
                const int ch = kk * 2 + ((lane >> 3) & 1);
                unsigned b[4];
                ldmatrix_x4(b, krow + (ch ^ (key & 7)));
                mma_bf16(kk & 1 ? sd[0] : sc[0], qf[kk], b[0], b[1]);
                mma_bf16(kk & 1 ? sd[1] : sc[1], qf[kk], b[2], b[3]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[j][e] += sd[j][e];
        }
        // scores in the log2 domain; keys beyond the range count as minus infinity
        float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool in = kw + j * 8 + (lane & 3) * 2 + e < k1;
                sc[j][e] = in ? sc[j][e] * a.scale_log2 : -INFINITY;
                sc[j][2 + e] = in ? sc[j][2 + e] * a.scale_log2 : -INFINITY;
                t0 = fmaxf(t0, sc[j][e]);
                t1 = fmaxf(t1, sc[j][2 + e]);
            }
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
        t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
        // the warp's first key is in range, so both maxima are finite (a score itself is finite)
        const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
        const float c0 = fast_exp2(m0 - n0), c1 = fast_exp2(m1 - n1);
        m0 = n0; m1 = n1;
        unsigned pa[4];
        float p[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            p[j][0] = fast_exp2(sc[j][0] - n0); p[j][1] = fast_exp2(sc[j][1] - n0);
            p[j][2] = fast_exp2(sc[j][2] - n1); p[j][3] = fast_exp2(sc[j][3] - n1);
        }
        l0 = l0 * c0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
        l1 = l1 * c1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
        pa[0] = pack_bf16(p[0][0], p[0][1]); pa[1] = pack_bf16(p[0][2], p[0][3]);
        pa[2] = pack_bf16(p[1][0], p[1][1]); pa[3] = pack_bf16(p[1][2], p[1][3]);
        if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {           // a maximum moved: seldom after the first tiles
#pragma unroll
            for (int n = 0; n < DH / 8; ++n) { o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1; }
        }
#pragma unroll
        for (int d2 = 0; d2 < DH / 16; ++d2) {
            // transposed: (keys 0-7, dims 16 d2 ..+7), (keys 8-15, same dims), (keys 0-7, dims +8..+15), (keys 8-15, ...)
            const int key = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7), ch = d2 * 2 + (lane >> 4);
            unsigned b[4];
            ldmatrix_x4_trans(b, vt + key * CH + (ch ^ (key & 7)));
            mma_bf16(o[2 * d2], pa, b[0], b[1]);
            mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
        }
        locate_end(i + GQ_STAGES, page_ahead);     // into the table that the copies of tile i + 1 have read
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncthreads();                               // the ring is free: it carries the warps' results
    // [warp][head][DH + 8]: the accumulator, then maximum and sum; with this stride the 8-byte stores of a half warp
    // (four heads, dims 0..7) fall into 32 different banks
    constexpr int RS = DH + 8;
    float *red = reinterpret_cast<float *>(gq_smem);
    float *fin = red + NW * GQ_HEADS * RS, *fin_ml = fin + GQ_HEADS * DH;      // this block's result, for its cluster
    {
        float *mine = red + (size_t)warp * GQ_HEADS * RS;
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < DH / 8; ++n) {
            *reinterpret_cast<float2 *>(mine + r0 * RS + n * 8 + c0) = make_float2(o[n][0], o[n][1]);
            *reinterpret_cast<float2 *>(mine + (r0 + 8) * RS + n * 8 + c0) = make_float2(o[n][2], o[n][3]);
        }
        if ((lane & 3) == 0) {
            *reinterpret_cast<float2 *>(mine + r0 * RS + DH) = make_float2(m0, l0);
            *reinterpret_cast<float2 *>(mine + (r0 + 8) * RS + DH) = make_float2(m1, l1);
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < heads * DH; idx += NT) {
        const int r = idx / DH, e = idx % DH;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, red[((size_t)w * GQ_HEADS + r) * RS + DH]);
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float *src = red + ((size_t)w * GQ_HEADS + r) * RS;
            const float f = M == -INFINITY ? 0.f : fast_exp2(src[DH] - M);      // a warp without keys: 2^-inf = 0
            L += f * src[DH + 1];
            A += f * src[e];
        }
        if (a.cluster) {
            fin[r * DH + e] = A;
            if (e == 0) { fin_ml[2 * r] = M; fin_ml[2 * r + 1] = L; }
        } else if (a.splits == 1) {
            a.out[((size_t)t * a.nh + h0 + r) * DH + e] = __float2bfloat16_rn(A / L);
        } else {
            const size_t slot = pbase + (size_t)r * a.splits;
            a.part_acc[slot * DH + e] = A;
            if (e == 0) { a.part_ml[slot * 2] = M; a.part_ml[slot * 2 + 1] = L; }
        }
    }
    if (a.cluster) {
        // the splits of this row and head group are the blocks of one cluster: the first reads the others' results
        // out of their shared memory and writes the row (the same sums, in the same order, as the merge kernel)
        cluster_sync_all();
        if (split == 0) {
            for (int idx = threadIdx.x; idx < heads * DH; idx += NT) {
                const int r = idx / DH;
                float M = -INFINITY;
                for (int p = 0; p < a.splits; ++p) M = fmaxf(M, ld_cluster_f32(fin_ml + 2 * r, p));
                float L = 0.f, A = 0.f;
                for (int p = 0; p < a.splits; ++p) {
                    const float mp = ld_cluster_f32(fin_ml + 2 * r, p);
                    if (mp > -INFINITY) {
                        const float f = exp2f(mp - M);
                        L += f * ld_cluster_f32(fin_ml + 2 * r + 1, p);
                        A += f * ld_cluster_f32(fin + idx, p);
                    }
                }
                a.out[((size_t)t * a.nh + h0 + r) * DH + (idx % DH)] = __float2bfloat16_rn(A / L);
            }
        }
        cluster_sync_all();                        // nobody leaves while its shared memory may still be read
    }
}

template <int DH, int NW>
static int launch_decode_gqa_warps(const DecodeArgs &a, int sms, cudaStream_t stream) {
    constexpr int KEYS = NW * 16;
    const int g = a.nh / a.nkvh;
    const size_t ring = (size_t)GQ_STAGES * 2 * KEYS * DH * sizeof(__nv_bfloat16) + 2 * KEYS * sizeof(long long)
                        + (size_t)GQ_HEADS * DH * sizeof(__nv_bfloat16);       // tiles, the two tables, the queries
    const size_t merge = (size_t)NW * GQ_HEADS * (DH + 8) * sizeof(float) + (size_t)GQ_HEADS * (DH + 2) * sizeof(float);
    const size_t smem = ring > merge ? ring : merge;
    cudaError_t e = cudaFuncSetAttribute(attention_decode_gqa_kernel<DH, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "attention_decode: %s", cudaGetErrorString(e));
    dim3 grid(a.splits, a.nkvh * ((g + GQ_HEADS - 1) / GQ_HEADS), a.nrows);
    // Measured: with heads of 64 (52 KB of shared memory a block) clusters of two are faster than the merge kernel
    // (48.6 against 50.0 us at 8 x 4096 keys, 36 heads), and larger ones as long as all blocks are resident at once (a
    // single row: 14.1 us at eight splits); larger clusters in several waves, and any cluster of the 103 KB blocks of
    // heads of 128, wait for whole groups of free SMs and lose more than the merge kernel costs (37.6 against 30.9 us;
    // the blocks of eight warps, 203 KB each, in clusters of eight: 36.1 against 15.0 us at 8 rows x 4,096 keys).
    const long long blocks = (long long)grid.x * grid.y * grid.z;
    if (DH == 64 && NW == 4 && a.splits >= 2 && a.splits <= 8 && (a.splits == 2 || blocks <= 2LL * sms)) {
        // the splits are one cluster and merge through distributed shared memory: no merge kernel, no scratch
        DecodeArgs c = a;
        c.cluster = 1;
        const cudaError_t err = jk_launch_clusters(attention_decode_gqa_kernel<DH, NW>, a.splits, grid, dim3(NW * 32), smem, stream, c);
        if (err != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "attention_decode_gqa (clusters of %d): %s", a.splits, cudaGetErrorString(err));
        return JK_OK;
    }
    jk_launch(attention_decode_gqa_kernel<DH, NW>, grid, dim3(NW * 32), smem, stream, a);
    JK_CHECK_LAUNCH("attention_decode_gqa");
    if (a.splits > 1) {
        jk_launch(attention_combine_kernel, dim3(a.nh, a.nrows), dim3(64), 0, stream, a);
        JK_CHECK_LAUNCH("attention_combine");
    }
    return JK_OK;
}

template <int DH>
static int launch_decode_gqa(const DecodeArgs &a, cudaStream_t stream) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    static const bool wide_off = [] { const char *v = getenv("JK_GQA_NO_WIDE"); return v && v[0] == '1'; }();
    const long long blocks = (long long)a.splits * a.nkvh * ((a.nh / a.nkvh + GQ_HEADS - 1) / GQ_HEADS) * a.nrows;
    // (Heads of 64 gain less and not everywhere: 8 key/value heads, one row, 4,096 keys at 8 cuts 10.7 -> 8.2 us, but a
    // step of that shape at 512 keys loses 3 %, and where the cuts would have to be halved for it, 36 heads and two
    // rows, 20.4 -> 22.2 us: they keep blocks of four warps, whose cuts merge inside clusters.)
    if (DH == 128 && blocks <= sms && !wide_off) return launch_decode_gqa_warps<DH, 8>(a, sms, stream);
    return launch_decode_gqa_warps<DH, 4>(a, sms, stream);
}

// Head sizes 64 and 128 go to the tensor-core decode kernel, which reads keys and values once per group of query
// heads: measured against the kernel of the CUDA cores it is 1.1 times as fast without groups, 1.4 to 2 times at groups
// of 2 to 4 and five times at 16 (JK_GQA_MIN_GROUP=n keeps groups below n on the old kernel).  Other head sizes stay there.
static int decode_gqa(const DecodeArgs &a, cudaStream_t stream, bool *taken) {
    *taken = true;
    static const int min_group = [] { const char *v = getenv("JK_GQA_MIN_GROUP"); return v ? atoi(v) : 1; }();
    if (a.nh / a.nkvh >= min_group) {
        switch (a.dh) {
            case 64: return launch_decode_gqa<64>(a, stream);       // rows of 8 or 16 chunks: what the swizzle takes
            case 128: return launch_decode_gqa<128>(a, stream);
        }
    }
    *taken = false;
    return JK_OK;
}

// Head sizes the tensor-core kernel is built for; others go to the row kernel.
JK_EXPORT int jk_attention_prefill_supports(int dh) {
    return dh == 16 || dh == 32 || dh == 48 || dh == 64 || dh == 80 || dh == 96 || dh == 128 || dh == 256;
}

JK_EXPORT int jk_attention_prefill(const void *q, const void *k_pages, const void *v_pages, void *out,
                                   const int *tiles, int ntiles, int tile_rows, const int *req_start, const int *req_pos,
                                   const int *block_table, int max_blocks, int page_size, int nh, int nkvh,
                                   int dh, float scale, int window, cudaStream_t stream) {
    if (ntiles == 0) return JK_OK;
    JK_REQUIRE(ntiles > 0 && nh > 0 && nkvh > 0 && nh % nkvh == 0, "attention_prefill: tiles %d heads %d/%d", ntiles, nh, nkvh);
    JK_REQUIRE(ntiles * (tile_rows / PF_BM) <= 65535, "attention_prefill: %d tiles exceed one launch", ntiles);
    JK_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "attention_prefill: page size %d, blocks %d, window %d",
               page_size, max_blocks, window);
    PrefillArgs a{(const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_pages, (const __nv_bfloat16 *)v_pages,
                  (__nv_bfloat16 *)out, tiles, req_start, req_pos, block_table,
                  ntiles, nh, nkvh, page_size, max_blocks, window, tile_rows, scale * 1.4426950408889634f};
    JK_REQUIRE(tile_rows >= PF_BM && tile_rows % PF_BM == 0, "attention_prefill: tiles of %d rows (a multiple of %d is needed)", tile_rows, PF_BM);
    switch (dh) {
        case 16: return launch_prefill<16, 64>(a, stream);
        case 32: return launch_prefill<32, 64>(a, stream);
        case 48: return launch_prefill<48, 64>(a, stream);
        case 64: return launch_prefill<64, 64>(a, stream);
        case 80: return launch_prefill<80, 64>(a, stream);
        case 96: return launch_prefill<96, 64>(a, stream);
        case 128: return launch_prefill<128, 64>(a, stream);
        case 256: return launch_prefill<256, 32>(a, stream);
        default: JK_FAIL(JK_UNSUPPORTED, "attention_prefill: head size %d has no tensor-core kernel", dh);
    }
}

// =======================================================================================
// The decode kernel for callers that cannot allocate: the scratch for the split partials is an
// array in the library's own image (see attention_static_scratch.h for who needs this and for the
// rules of use).  Nothing above this line is changed by it.
// =======================================================================================
#include "attention_static_scratch.h"
#include <mutex>

static __device__ __align__(256) float g_static_scratch[JK_STATIC_SCRATCH_FLOATS];

// In host code `g_static_scratch` is only a handle for the symbol, not an address a kernel could
// use; the device address is looked up once per device and kept here.
constexpr int JK_MAX_DEVICES = 64;
static float *g_static_scratch_addr[JK_MAX_DEVICES] = {};
static std::mutex g_static_scratch_mutex;

static int static_scratch_address(float **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    JK_REQUIRE(dev >= 0 && dev < JK_MAX_DEVICES, "attention_decode_static: device %d is beyond the %d this library tracks",
               dev, JK_MAX_DEVICES);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        // first call on this device (it is the current one): ask the runtime where the array lives here
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            JK_FAIL(JK_CUDA_ERROR, "attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_scratch_addr[dev] = static_cast<float *>(p);
    }
    *out = g_static_scratch_addr[dev];
    return JK_OK;
}

JK_EXPORT int jk_attention_decode_static(const void *q, const void *k_pages, const void *v_pages, void *out,
                                         const int *rows, int nrows, const int *positions, const int *row_req,
                                         const int *block_table, int max_blocks, int page_size, int nh, int nkvh,
                                         int dh, float scale, int window, int splits, cudaStream_t stream) {
    if (nrows == 0) return JK_OK;
    JK_REQUIRE(nrows > 0 && nh > 0 && dh > 0 && splits >= 1, "attention_decode_static: rows %d heads %d head size %d splits %d",
               nrows, nh, dh, splits);
    const long long need = jk_attention_decode_scratch_floats(nrows, nh, dh, splits);
    JK_REQUIRE(need <= (long long)JK_STATIC_SCRATCH_FLOATS,
               "attention_decode_static: %d rows x %d heads x %d splits of head size %d need %lld floats of scratch, "
               "the built-in array holds %d; use fewer splits or rows, or jk_attention_decode with your own scratch",
               nrows, nh, splits, dh, need, (int)JK_STATIC_SCRATCH_FLOATS);
    float *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    // every partial slot that the merge kernel reads is written by the split kernel of this same call,
    // so what an earlier call left in the array needs no clearing
    return jk_attention_decode(q, k_pages, v_pages, out, need ? scratch : nullptr, rows, nrows, positions, row_req,
                               block_table, max_blocks, page_size, nh, nkvh, dh, scale, window, splits, stream);
}
