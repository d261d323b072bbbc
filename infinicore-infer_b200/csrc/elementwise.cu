// Row-wise kernels of the step: embedding gather, residual add + RMSNorm, rotary position
// encoding fused with the write of keys and values into cache pages, SwiGLU, and a
// float32 matrix product on the CUDA cores (the true 32-bit path).
//
// The residual stream is float32 in both precisions; products, norms and rotations are
// computed in float32 and rounded once when they are stored as bfloat16.
#include "common.cuh"

JK_DEFINE_ERROR_BUFFER(jk_elementwise)

// ---------------------------------------------------------------------------------------
// Embedding: x[i, :] = scale * E[tokens[i], :]      (reference: jiuge.cpp:164-168 does one
// device-to-device copy per token of a table that was scaled on the host, jiuge.py:194-197)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int *__restrict__ tokens, const TW *__restrict__ table,
                             float *__restrict__ out, int d, float scale) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const TW *src = table + (size_t)tokens[row] * d;
    float *dst = out + (size_t)row * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) dst[c] = scale * to_f32(src[c]);
}

JK_EXPORT int jk_embed(const int *tokens, int ntok, const void *table, int table_dtype, int d,
                       float scale, float *out, cudaStream_t stream) {
    if (ntok == 0) return JK_OK;
    JK_REQUIRE(ntok > 0 && d > 0, "embed: ntok %d, d %d", ntok, d);
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == JK_F32)
        jk_launch(embed_kernel<float>, dim3(ntok), dim3(threads), 0, stream, tokens, (const float *)table, out, d, scale);
    else if (table_dtype == JK_BF16)
        jk_launch(embed_kernel<__nv_bfloat16>, dim3(ntok), dim3(threads), 0, stream, tokens, (const __nv_bfloat16 *)table, out, d, scale);
    else
        JK_FAIL(JK_UNSUPPORTED, "embed: table dtype %d", table_dtype);
    JK_CHECK_LAUNCH("embed");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------
// Residual add + RMSNorm.  For output row i (source row r = rows ? rows[i] : i):
//     v = x[r] + delta_scale * delta[r]          (delta may be null)
//     x[r] = v                                   (only when rows is null)
//     out[i] = out_scale * v * w / sqrt(mean(v^2) + eps)
// One block per row; the row is held in shared memory between the two passes.
// (reference: rmsnorm at jiuge.cpp:198, :246, :262; the residual add is the beta=1 of the
// preceding product, inference_context.cpp:207-210.)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float4 load4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) {
    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16 *p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned *>(&lo); raw.y = *reinterpret_cast<const unsigned *>(&hi);
    *reinterpret_cast<uint2 *>(p) = raw;
}

// VEC: the width is a multiple of 4 and rows are 16-byte aligned, so four elements move at a time.
template <typename TD, typename TO, bool VEC>
__global__ void add_rmsnorm_kernel(float *__restrict__ x, const TD *__restrict__ delta,
                                   float delta_scale, const float *__restrict__ w, float eps,
                                   float out_scale, TO *__restrict__ out,
                                   const int *__restrict__ rows, int d) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float *xr = x + (size_t)r * d;
    const TD *dr = delta ? delta + (size_t)r * d : nullptr;
    float ss = 0.f;
    if (VEC) {
        for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
            float4 v = load4(xr + c);
            if (dr) {
                const float4 dv = load4(dr + c);
                v = make_float4(v.x + delta_scale * dv.x, v.y + delta_scale * dv.y, v.z + delta_scale * dv.z, v.w + delta_scale * dv.w);
                if (!rows) store4(xr + c, v);
            }
            store4(row_buf + c, v);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int c = threadIdx.x; c < d; c += blockDim.x) {
            float v = xr[c];
            if (dr) v += delta_scale * to_f32(dr[c]);
            row_buf[c] = v;
            if (dr && !rows) xr[c] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)d + eps) * out_scale;
    TO *o = out + (size_t)i * d;
    if (VEC) {
        for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
            const float4 v = load4(row_buf + c), g = load4(w + c);
            store4(o + c, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
        }
    } else {
        for (int c = threadIdx.x; c < d; c += blockDim.x) o[c] = from_f32<TO>((row_buf[c] * inv) * w[c]);
    }
}

// The same for steps of many rows: a warp per row, the row in registers (NV groups of four floats a lane), every load
// of a row on its way before the first is used, no shared memory and no barrier (a prefill of 2,048 tokens of the 2B
// shape: 9.94 -> 9.90 ms).
template <typename TD, typename TO, int NV>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float *__restrict__ x, const TD *__restrict__ delta, float delta_scale, const float *__restrict__ w, float eps,
                        float out_scale, TO *__restrict__ out, const int *__restrict__ rows, int nout, int d) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (i >= nout) return;
    const int r = rows ? rows[i] : i;
    float *xr = x + (size_t)r * d;
    const TD *dr = delta ? delta + (size_t)r * d : nullptr;
    float4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int c = (j * 32 + lane) * 4;
        v[j] = c < d ? load4(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (dr) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int c = (j * 32 + lane) * 4;
            if (c < d) {
                const float4 dv = load4(dr + c);
                v[j] = make_float4(v[j].x + delta_scale * dv.x, v[j].y + delta_scale * dv.y, v[j].z + delta_scale * dv.z, v[j].w + delta_scale * dv.w);
                if (!rows) store4(xr + c, v[j]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)d + eps) * out_scale;
    TO *o = out + (size_t)i * d;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int c = (j * 32 + lane) * 4;
        if (c < d) {
            const float4 g = load4(w + c);
            store4(o + c, make_float4(v[j].x * inv * g.x, v[j].y * inv * g.y, v[j].z * inv * g.z, v[j].w * inv * g.w));
        }
    }
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float *x, const void *delta, float delta_scale, const float *w,
                              float eps, float out_scale, void *out, const int *rows, int nout,
                              int d, cudaStream_t stream) {
    const size_t smem = (size_t)d * sizeof(float);
    JK_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: width %d needs %zu bytes of shared memory", d, smem);
    const bool vec = d % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                     ((uintptr_t)w % 16 == 0);
    if (smem > 48 * 1024) {
        cudaError_t e = vec ? cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                            : cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "add_rmsnorm: %s", cudaGetErrorString(e));
    }
    if (vec && nout >= 256 && d <= 24 * 128) {
        // many rows: a warp per row
        const int blocks = (nout + 7) / 8;
#define JK_ROWS_LAUNCH(NV_)                                                                                              \
        jk_launch(add_rmsnorm_rows_kernel<TD, TO, NV_>, dim3(blocks), dim3(256), 0, stream, x, (const TD *)delta, delta_scale, w, eps, \
                  out_scale, (TO *)out, rows, nout, d)
        if (d <= 8 * 128) JK_ROWS_LAUNCH(8);
        else if (d <= 16 * 128) JK_ROWS_LAUNCH(16);
        else JK_ROWS_LAUNCH(24);
#undef JK_ROWS_LAUNCH
        JK_CHECK_LAUNCH("add_rmsnorm");
        return JK_OK;
    }
    if (vec) {
        const int threads = d >= 4096 ? 512 : (d >= 1024 ? 256 : 128);
        jk_launch(add_rmsnorm_kernel<TD, TO, true>, dim3(nout), dim3(threads), smem, stream,
                  x, (const TD *)delta, delta_scale, w, eps, out_scale, (TO *)out, rows, d);
    } else {
        const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
        jk_launch(add_rmsnorm_kernel<TD, TO, false>, dim3(nout), dim3(threads), smem, stream,
                  x, (const TD *)delta, delta_scale, w, eps, out_scale, (TO *)out, rows, d);
    }
    JK_CHECK_LAUNCH("add_rmsnorm");
    return JK_OK;
}

JK_EXPORT int jk_add_rmsnorm(float *x, const void *delta, int delta_dtype, float delta_scale,
                             const float *w, float eps, float out_scale, void *out, int out_dtype,
                             const int *rows, int nout, int d, cudaStream_t stream) {
    if (nout == 0) return JK_OK;
    JK_REQUIRE(nout > 0 && d > 0, "add_rmsnorm: nout %d, d %d", nout, d);
    if (delta_dtype == JK_F32 && out_dtype == JK_F32)
        return launch_add_rmsnorm<float, float>(x, delta, delta_scale, w, eps, out_scale, out, rows, nout, d, stream);
    if (delta_dtype == JK_F32 && out_dtype == JK_BF16)
        return launch_add_rmsnorm<float, __nv_bfloat16>(x, delta, delta_scale, w, eps, out_scale, out, rows, nout, d, stream);
    if (delta_dtype == JK_BF16 && out_dtype == JK_BF16)
        return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(x, delta, delta_scale, w, eps, out_scale, out, rows, nout, d, stream);
    if (delta_dtype == JK_BF16 && out_dtype == JK_F32)
        return launch_add_rmsnorm<__nv_bfloat16, float>(x, delta, delta_scale, w, eps, out_scale, out, rows, nout, d, stream);
    JK_FAIL(JK_UNSUPPORTED, "add_rmsnorm: dtypes %d, %d", delta_dtype, out_dtype);
}

// x += delta_scale * delta, without a norm (used when a residual must be made whole).
template <typename TD>
__global__ void residual_add_kernel(float *__restrict__ x, const TD *__restrict__ delta,
                                    float delta_scale, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) x[i] += delta_scale * to_f32(delta[i]);
}

JK_EXPORT int jk_residual_add(float *x, const void *delta, int delta_dtype, float delta_scale,
                              long long n, cudaStream_t stream) {
    if (n == 0) return JK_OK;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (delta_dtype == JK_F32)
        jk_launch(residual_add_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, x, (const float *)delta, delta_scale, (size_t)n);
    else if (delta_dtype == JK_BF16)
        jk_launch(residual_add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, x, (const __nv_bfloat16 *)delta, delta_scale, (size_t)n);
    else
        JK_FAIL(JK_UNSUPPORTED, "residual_add: dtype %d", delta_dtype);
    JK_CHECK_LAUNCH("residual_add");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------
// SwiGLU: out[t, c] = silu(gu[t, c]) * gu[t, di + c],  silu(z) = z / (1 + exp(-z))
// (reference: jiuge.cpp:191-192, :248: gate is the first half of the fused product, up the second)
// ---------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI *__restrict__ gu, TO *__restrict__ out, int di, size_t total) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t t = i / di;
        const int c = (int)(i - t * di);
        const float g = to_f32(gu[t * 2 * di + c]);
        const float u = to_f32(gu[t * 2 * di + di + c]);
        out[i] = from_f32<TO>(g / (1.f + expf(-g)) * u);
    }
}

JK_EXPORT int jk_swiglu(const void *gu, int in_dtype, void *out, int out_dtype, int ntok, int di,
                        cudaStream_t stream) {
    if (ntok == 0) return JK_OK;
    JK_REQUIRE(ntok > 0 && di > 0, "swiglu: ntok %d, di %d", ntok, di);
    const size_t total = (size_t)ntok * di;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (in_dtype == JK_F32 && out_dtype == JK_F32)
        jk_launch(swiglu_kernel<float, float>, dim3((int)blocks), dim3(threads), 0, stream, (const float *)gu, (float *)out, di, total);
    else if (in_dtype == JK_F32 && out_dtype == JK_BF16)
        jk_launch(swiglu_kernel<float, __nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (const float *)gu, (__nv_bfloat16 *)out, di, total);
    else if (in_dtype == JK_BF16 && out_dtype == JK_BF16)
        jk_launch(swiglu_kernel<__nv_bfloat16, __nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (const __nv_bfloat16 *)gu, (__nv_bfloat16 *)out, di, total);
    else
        JK_FAIL(JK_UNSUPPORTED, "swiglu: dtypes %d -> %d", in_dtype, out_dtype);
    JK_CHECK_LAUNCH("swiglu");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------
// Rotary position encoding + cache write.  For token row t at position p of request r:
//   q_out[t, h, :]            = rot(qkv[t, h, :] + bias, p)                  h < nh
//   K[page, hk, off, :]       = rot(qkv[t, nh + hk, :] + bias, p)            hk < nkvh
//   V[page, hk, off, :]       = qkv[t, nh + nkvh + hk, :] + bias
// with page = block_table[r, p / page_size], off = p % page_size.  rot pairs element j with
// j + dh/2 (or 2j with 2j+1 when interleaved) at angle p / theta^(j / (dh/2)); cos and sin
// come from float32 tables [max_positions, dh/2].  A null table means no rotation.
// (reference: rope at jiuge.cpp:202-203, cache rows at jiuge.cpp:217-218, tables at
// jiuge_weight.hpp:134-186)
// ---------------------------------------------------------------------------------------
struct RopeKvArgs {
    const void *qkv;
    const float *bias;
    const int *positions;
    const int *row_req;
    const int *block_table;
    const float *cos_table;
    const float *sin_table;
    void *q_out;
    void *k_pages;
    void *v_pages;
    int ld_qkv, nh, nkvh, dh, page_size, max_blocks, interleaved, write_cache, heads_per_block, vec;
};

template <typename TI, typename TO>
__global__ void rope_kv_kernel(RopeKvArgs a) {
    pdl_trigger();
    pdl_wait();
    // blockIdx.x: token row; blockIdx.y: a chunk of `heads_per_block` heads out of the row's
    // nh query heads, nkvh key heads and nkvh value heads (in that order)
    const int t = blockIdx.x;
    const int pos = a.positions[t];
    const int half = a.dh / 2;
    const TI *src = (const TI *)a.qkv + (size_t)t * a.ld_qkv;
    const float *cs = a.cos_table ? a.cos_table + (size_t)pos * half : nullptr;
    const float *sn = a.sin_table ? a.sin_table + (size_t)pos * half : nullptr;
    size_t slot = 0;   // element offset of (page, head 0, off, 0) in the pages
    if (a.write_cache) {
        const int page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
        slot = ((size_t)page * a.nkvh * a.page_size + (pos % a.page_size)) * a.dh;
    }
    const size_t head_stride = (size_t)a.page_size * a.dh;
    const int total_heads = a.write_cache ? a.nh + 2 * a.nkvh : a.nh;
    const int h_begin = blockIdx.y * a.heads_per_block;
    const int h_end = min(total_heads, h_begin + a.heads_per_block);
    if (a.vec) {
        // four pairs at a time: elements j..j+3 of the first half with j+half..j+half+3 of the second
        const int q4 = half / 4;
        for (int i = threadIdx.x; i < (h_end - h_begin) * q4; i += blockDim.x) {
            const int h = h_begin + i / q4, j = (i % q4) * 4;
            const bool rotated = h < a.nh + a.nkvh;
            float4 x0 = load4(src + h * a.dh + j), x1 = load4(src + h * a.dh + half + j);
            if (a.bias) {
                const float4 b0 = load4(a.bias + h * a.dh + j), b1 = load4(a.bias + h * a.dh + half + j);
                x0 = make_float4(x0.x + b0.x, x0.y + b0.y, x0.z + b0.z, x0.w + b0.w);
                x1 = make_float4(x1.x + b1.x, x1.y + b1.y, x1.z + b1.z, x1.w + b1.w);
            }
            float4 y0 = x0, y1 = x1;
            if (cs && rotated) {
                const float4 c = load4(cs + j), sn4 = load4(sn + j);
                y0 = make_float4(x0.x * c.x - x1.x * sn4.x, x0.y * c.y - x1.y * sn4.y, x0.z * c.z - x1.z * sn4.z, x0.w * c.w - x1.w * sn4.w);
                y1 = make_float4(x0.x * sn4.x + x1.x * c.x, x0.y * sn4.y + x1.y * c.y, x0.z * sn4.z + x1.z * c.z, x0.w * sn4.w + x1.w * c.w);
            }
            TO *dst;
            if (h < a.nh) dst = (TO *)a.q_out + ((size_t)t * a.nh + h) * a.dh;
            else if (h < a.nh + a.nkvh) dst = (TO *)a.k_pages + slot + (size_t)(h - a.nh) * head_stride;
            else dst = (TO *)a.v_pages + slot + (size_t)(h - a.nh - a.nkvh) * head_stride;
            store4(dst + j, y0);
            store4(dst + half + j, y1);
        }
        return;
    }
    for (int i = threadIdx.x; i < (h_end - h_begin) * half; i += blockDim.x) {
        const int h = h_begin + i / half, j = i % half;
        const bool rotated = h < a.nh + a.nkvh;             // value heads are copied as they are
        const int e0 = (a.interleaved && rotated) ? 2 * j : j;
        const int e1 = (a.interleaved && rotated) ? 2 * j + 1 : j + half;
        float x0 = to_f32(src[h * a.dh + e0]), x1 = to_f32(src[h * a.dh + e1]);
        if (a.bias) { x0 += a.bias[h * a.dh + e0]; x1 += a.bias[h * a.dh + e1]; }
        float y0 = x0, y1 = x1;
        if (cs && rotated) {
            const float c = cs[j], s = sn[j];
            y0 = x0 * c - x1 * s;
            y1 = x0 * s + x1 * c;
        }
        TO *dst;
        if (h < a.nh) dst = (TO *)a.q_out + ((size_t)t * a.nh + h) * a.dh;
        else if (h < a.nh + a.nkvh) dst = (TO *)a.k_pages + slot + (size_t)(h - a.nh) * head_stride;
        else dst = (TO *)a.v_pages + slot + (size_t)(h - a.nh - a.nkvh) * head_stride;
        dst[e0] = from_f32<TO>(y0);
        dst[e1] = from_f32<TO>(y1);
    }
}

JK_EXPORT int jk_rope_kv(const void *qkv, int in_dtype, int ld_qkv, const float *bias,
                         const int *positions, const int *row_req, const int *block_table,
                         int max_blocks, int page_size, const float *cos_table,
                         const float *sin_table, int interleaved, void *q_out, void *k_pages,
                         void *v_pages, int out_dtype, int ntok, int nh, int nkvh, int dh,
                         int write_cache, cudaStream_t stream) {
    if (ntok == 0) return JK_OK;
    JK_REQUIRE(ntok > 0 && nh > 0 && nkvh >= 0 && dh > 0 && dh % 2 == 0,
               "rope_kv: ntok %d, heads %d/%d, head size %d", ntok, nh, nkvh, dh);
    JK_REQUIRE(!write_cache || (page_size > 0 && max_blocks > 0 && block_table && k_pages && v_pages),
               "rope_kv: cache write asked for without pages");
    JK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "rope_kv: one of cos/sin is null");
    RopeKvArgs a{qkv, bias, positions, row_req, block_table, cos_table, sin_table, q_out, k_pages,
                 v_pages, ld_qkv, nh, nkvh, dh, page_size, max_blocks, interleaved, write_cache, 0, 0};
    // four elements at a time when the layout allows it (pairs j, j + dh/2; everything 16-byte aligned)
    a.vec = !interleaved && dh % 8 == 0 && ld_qkv % 4 == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)q_out % 16 == 0) &&
            ((uintptr_t)k_pages % 16 == 0) && ((uintptr_t)v_pages % 16 == 0) && ((uintptr_t)bias % 16 == 0) &&
            ((uintptr_t)cos_table % 16 == 0) && ((uintptr_t)sin_table % 16 == 0);
    // few rows: cut each row's heads over several blocks so that the GPU is not left to ntok blocks
    const int total_heads = write_cache ? nh + 2 * nkvh : nh;
    int chunks = 1;
    while (ntok * chunks < 296 && chunks * 2 <= total_heads) chunks *= 2;
    a.heads_per_block = (total_heads + chunks - 1) / chunks;
    const dim3 grid(ntok, (total_heads + a.heads_per_block - 1) / a.heads_per_block);
    JK_REQUIRE(grid.y <= 65535, "rope_kv: too many head chunks");
    const int work = a.heads_per_block * dh / 2 / (a.vec ? 4 : 1);
    const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
    if (in_dtype == JK_F32 && out_dtype == JK_F32)
        jk_launch(rope_kv_kernel<float, float>, grid, dim3(threads), 0, stream, a);
    else if (in_dtype == JK_F32 && out_dtype == JK_BF16)
        jk_launch(rope_kv_kernel<float, __nv_bfloat16>, grid, dim3(threads), 0, stream, a);
    else if (in_dtype == JK_BF16 && out_dtype == JK_BF16)
        jk_launch(rope_kv_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(threads), 0, stream, a);
    else
        JK_FAIL(JK_UNSUPPORTED, "rope_kv: dtypes %d -> %d", in_dtype, out_dtype);
    JK_CHECK_LAUNCH("rope_kv");
    return JK_OK;
}

// ---------------------------------------------------------------------------------------
// float32 matrix product on the CUDA cores:  C[M, N] = A[M, K] * W[N, K]^T (+ bias[N]).
// Plain fused multiply-adds in float32: no tensor cores, hence no TF32 rounding of the
// operands.  Each output element sums over k in ascending order whatever M and N are, so a
// row's result does not depend on what else is in the batch.
// (reference: the products at jiuge.cpp:200, :236, :247, :249, :264 go to a library.)
// ---------------------------------------------------------------------------------------
constexpr int GF_BM = 64, GF_BN = 64, GF_BK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float *__restrict__ A, const float *__restrict__ W,
                const float *__restrict__ bias, float *__restrict__ C, int M, int N, int K,
                int lda, int ldw, int ldc) {
    pdl_trigger();
    pdl_wait();
    __shared__ float As[GF_BK][GF_BM + 1];
    __shared__ float Ws[GF_BK][GF_BN + 1];
    const int m0 = blockIdx.y * GF_BM, n0 = blockIdx.x * GF_BN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += GF_BK) {
        for (int i = threadIdx.x; i < GF_BM * GF_BK; i += 256) {
            const int r = i / GF_BK, c = i % GF_BK;
            As[c][r] = (m0 + r < M && k0 + c < K) ? A[(size_t)(m0 + r) * lda + k0 + c] : 0.f;
            Ws[c][r] = (n0 + r < N && k0 + c < K) ? W[(size_t)(n0 + r) * ldw + k0 + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GF_BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
        }
    }
}

JK_EXPORT int jk_gemm_f32(const float *A, int lda, const float *W, int ldw, const float *bias,
                          float *C, int ldc, int M, int N, int K, cudaStream_t stream) {
    if (M == 0 || N == 0) return JK_OK;
    JK_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_f32: M %d N %d K %d", M, N, K);
    dim3 grid((N + GF_BN - 1) / GF_BN, (M + GF_BM - 1) / GF_BM);
    JK_REQUIRE(grid.y <= 65535, "gemm_f32: M %d is too large for one launch", M);
    jk_launch(gemm_f32_kernel, grid, dim3(256), 0, stream, A, W, bias, C, M, N, K, lda, ldw, ldc);
    JK_CHECK_LAUNCH("gemm_f32");
    return JK_OK;
}
