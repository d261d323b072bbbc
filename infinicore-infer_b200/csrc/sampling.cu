// Sampling from rows of float32 logits: greedy, temperature, top-k, top-p.
//
// The reference hands one row of raw logits plus (random_val, topp, topk, temperature) to a
// library operator, once per request (src/models/jiuge/jiuge.cpp:282-289); temperature 0 or
// topk 1 means greedy (include/infinicore_infer/models/jiuge.h:85-87).  Here one block
// samples one row:
//   greedy       the largest logit, the lowest index among equals;
//   otherwise    w_i = exp((logit_i - max) / temperature); the candidate set is the largest
//                logits down to the first one at which either topk candidates or a share
//                topp of the whole mass is reached (candidates equal to that one included);
//                the token is the first candidate, in vocabulary order, whose running mass
//                exceeds u * (mass of the candidates).
// Masses are summed as 64-bit fixed point, so the result does not depend on the order in
// which threads add: the same (logits, u) always gives the same token.
#include "common.cuh"

JK_DEFINE_ERROR_BUFFER(jk_sampling)

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ int block_argmax(const float *row, int V, ArgMax *scratch) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best.v || (v == best.v && i < best.i)) best = ArgMax{v, i};
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = best;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = lane < (int)(blockDim.x >> 5) ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    int idx = scratch[32].i;
    if (idx == 0x7fffffff) idx = 0;     // a row of NaN or -inf only
    return idx;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float *__restrict__ logits, long long ld, int V, int *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgMax scratch[33];
    const int idx = block_argmax(logits + (size_t)blockIdx.x * ld, V, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

// Two stages for few rows of a large vocabulary: blocks take chunks of a row, then one block per row
// picks among the chunks' winners (the lowest index among equals in both stages).
constexpr int ARGMAX_CHUNK = 8192;

__global__ void __launch_bounds__(256)
argmax_chunks_kernel(const float *__restrict__ logits, long long ld, int V, ArgMax *__restrict__ part) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgMax scratch[33];
    const int r = blockIdx.y, c = blockIdx.x;
    const int lo = c * ARGMAX_CHUNK, n = min(ARGMAX_CHUNK, V - lo);
    const int idx = block_argmax(logits + (size_t)r * ld + lo, n, scratch);
    if (threadIdx.x == 0) part[(size_t)r * gridDim.x + c] = ArgMax{logits[(size_t)r * ld + lo + idx], lo + idx};
}

__global__ void argmax_merge_kernel(const ArgMax *__restrict__ part, int nchunks, int *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < nchunks; i += 32) best = better(best, part[(size_t)r * nchunks + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// Bytes of scratch that `jk_argmax` wants for this shape (0: it runs in one stage).
JK_EXPORT long long jk_argmax_scratch_bytes(int nrows, int V) {
    const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    if (chunks < 2 || nrows * 1 >= 148 * 2) return 0;
    return (long long)nrows * chunks * sizeof(ArgMax);
}

JK_EXPORT int jk_argmax(const float *logits, long long ld, int nrows, int V, int *out, void *scratch,
                        cudaStream_t stream) {
    if (nrows == 0) return JK_OK;
    JK_REQUIRE(nrows > 0 && V > 0 && ld >= V, "argmax: rows %d, vocabulary %d, stride %lld", nrows, V, ld);
    if (scratch != nullptr && jk_argmax_scratch_bytes(nrows, V) > 0) {
        const int chunks = (V + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
        JK_REQUIRE(nrows <= 65535, "argmax: %d rows exceed one launch", nrows);
        jk_launch(argmax_chunks_kernel, dim3(chunks, nrows), dim3(256), 0, stream, logits, ld, V, (ArgMax *)scratch);
        JK_CHECK_LAUNCH("argmax_chunks");
        jk_launch(argmax_merge_kernel, dim3(nrows), dim3(32), 0, stream, (const ArgMax *)scratch, chunks, out);
        JK_CHECK_LAUNCH("argmax_merge");
        return JK_OK;
    }
    jk_launch(argmax_kernel, dim3(nrows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, out);
    JK_CHECK_LAUNCH("argmax");
    return JK_OK;
}

__device__ __forceinline__ unsigned long long fixed_mass(float z, float m) {
    return (unsigned long long)(expf(z - m) * 4294967296.f);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float *__restrict__ logits, long long ld, int V,
              const float *__restrict__ temperature, const int *__restrict__ topk,
              const float *__restrict__ topp, const float *__restrict__ uniform,
              int *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ ArgMax am_scratch[33];
    __shared__ float f_scratch[33];
    __shared__ unsigned hist_cnt[256];
    __shared__ unsigned long long hist_mass[256];
    __shared__ unsigned long long seg_mass[SAMPLE_THREADS];
    __shared__ unsigned long long sh_u64[4];
    __shared__ unsigned sh_u32[4];

    const int r = blockIdx.x;
    const float *row = logits + (size_t)r * ld;
    const float temp = temperature[r];
    const int k_in = topk[r];
    const float p_in = topp[r];
    if (temp <= 0.f || k_in == 1) {
        const int idx = block_argmax(row, V, am_scratch);
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }
    const float inv_t = 1.f / temp;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) m = fmaxf(m, row[i] * inv_t);
    m = block_max(m, f_scratch);

    // every thread owns one contiguous segment of the vocabulary
    const int seg = (V + blockDim.x - 1) / blockDim.x;
    const int s0 = min(V, (int)threadIdx.x * seg), s1 = min(V, s0 + seg);

    unsigned long long mine = 0;
    for (int i = s0; i < s1; ++i) mine += fixed_mass(row[i] * inv_t, m);
    seg_mass[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long tot = 0;
        for (int i = 0; i < (int)blockDim.x; ++i) tot += seg_mass[i];
        sh_u64[0] = tot;
    }
    __syncthreads();
    const unsigned long long total = sh_u64[0];

    unsigned tau = 0;                       // candidates: ordered_key >= tau
    unsigned long long cand_mass = total;
    const bool cut_k = k_in > 1 && k_in < V;
    const bool cut_p = p_in < 1.f;
    if (cut_k || cut_p) {
        const unsigned kk = cut_k ? (unsigned)k_in : (unsigned)V;
        const unsigned long long limit = cut_p ? (unsigned long long)((double)fmaxf(p_in, 0.f) * (double)total) : total;
        unsigned prefix = 0;
        if (threadIdx.x == 0) { sh_u32[0] = 0; sh_u64[1] = 0; }   // count and mass above the prefix range
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int b = threadIdx.x; b < 256; b += blockDim.x) { hist_cnt[b] = 0; hist_mass[b] = 0; }
            __syncthreads();
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float z = row[i] * inv_t;
                const unsigned key = ordered_key(z);
                if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) {
                    const unsigned b = (key >> shift) & 255u;
                    atomicAdd(&hist_cnt[b], 1u);
                    atomicAdd(&hist_mass[b], fixed_mass(z, m));
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                unsigned c = sh_u32[0];
                unsigned long long ms = sh_u64[1];
                int sel = 0;
                for (int b = 255; b >= 0; --b) {
                    if (hist_cnt[b] == 0) continue;
                    sel = b;
                    if (c + hist_cnt[b] >= kk || ms + hist_mass[b] >= limit) break;
                    c += hist_cnt[b];
                    ms += hist_mass[b];
                }
                sh_u32[0] = c;
                sh_u64[1] = ms;
                sh_u32[1] = (unsigned)sel;
                sh_u64[2] = ms + hist_mass[sel];
            }
            __syncthreads();
            prefix |= sh_u32[1] << shift;
        }
        tau = prefix;
        cand_mass = sh_u64[2];
        __syncthreads();
    }

    // walk the candidates in vocabulary order
    mine = 0;
    for (int i = s0; i < s1; ++i) {
        const float z = row[i] * inv_t;
        if (ordered_key(z) >= tau) mine += fixed_mass(z, m);
    }
    seg_mass[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float u = uniform[r];
        u = fminf(fmaxf(u, 0.f), 0.99999994f);
        const unsigned long long target = (unsigned long long)((double)u * (double)cand_mass);
        unsigned long long cum = 0;
        int owner = -1;
        for (int i = 0; i < (int)blockDim.x; ++i) {
            if (cum + seg_mass[i] > target) { owner = i; break; }
            cum += seg_mass[i];
        }
        sh_u32[2] = (unsigned)owner;
        sh_u64[3] = cum;
        sh_u64[0] = target;
    }
    __syncthreads();
    const int owner = (int)sh_u32[2];
    if (owner < 0) {                        // no mass at all (cannot happen: the maximum has mass 2^32)
        const int idx = block_argmax(row, V, am_scratch);
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }
    if ((int)threadIdx.x == owner) {
        unsigned long long cum = sh_u64[3];
        const unsigned long long target = sh_u64[0];
        int pick = s0;
        for (int i = s0; i < s1; ++i) {
            const float z = row[i] * inv_t;
            if (ordered_key(z) >= tau) {
                cum += fixed_mass(z, m);
                pick = i;
                if (cum > target) break;
            }
        }
        out[r] = pick;
    }
}

JK_EXPORT int jk_sample(const float *logits, long long ld, int nrows, int V, const float *temperature,
                        const int *topk, const float *topp, const float *uniform, int *out,
                        cudaStream_t stream) {
    if (nrows == 0) return JK_OK;
    JK_REQUIRE(nrows > 0 && V > 0 && ld >= V, "sample: rows %d, vocabulary %d, stride %lld", nrows, V, ld);
    jk_launch(sample_kernel, dim3(nrows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature, topk, topp, uniform, out);
    JK_CHECK_LAUNCH("sample");
    return JK_OK;
}
