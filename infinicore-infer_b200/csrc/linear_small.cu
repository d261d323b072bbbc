// Matrix products for steps of few rows (decoding): out[M, N] = act[M, K] * W[N, K]^T, M <= 16.
//
// With so few rows the product is a stream of weights: every byte of W is read once and used
// for M multiply-adds, so the kernel is built around the loads.  The roles of the tensor-core
// operands are swapped: 16 rows of W (16 output features) are the A operand of
// mma.sync.m16n8k16 and up to 8 rows of activations are the B operand.  Because a dot product
// does not care in which order its terms are added, the k index is permuted so that every
// thread's operand registers come straight out of ONE 16-byte load: thread (g, t) of a warp
// loads W[n0 + g][k0 + 8t .. k0 + 8t + 7] and W[n0 + g + 8][same], and the activations are laid
// out in shared memory as [k / 8][row][8] so that its B registers are one conflict-free 16-byte
// load as well.  No shuffle, no ldmatrix, no transposition of weights.
//
// Two kernels share this layout.  `small_linear_tile_kernel` (below) takes every K whose 16-row tile
// fits in shared memory: one block per tile, the whole tile in flight at once.  `small_linear_kernel`
// takes longer K with a ring: a block's warps are split into (tiles of 16 features) x (slices of K).
// In both the slices' partial sums meet in shared memory and the first slice's warp runs the epilogue:
//   EPI_F32     out[m, n] = acc                       (float32; the residual add and the next
//                                                      norm are the consumer's)
//   EPI_SWIGLU  out[m, n] = silu(gate) * up           (bfloat16; the warp computes features n
//                                                      and N + n of a [2N, K] matrix together)
// The library is asked for the same products when M is larger (the reference sends all of its
// products to a library: src/models/inference_context.cpp:59-79).
#include "common.cuh"
#include "tma.cuh"

JK_DEFINE_ERROR_BUFFER(jk_linear_small)

enum { EPI_F32 = 0, EPI_SWIGLU = 1, EPI_QKV = 2, EPI_RESIDUAL = 3 };

// RMSNorm without a kernel of its own, for a chain of few-row products (decode steps).  The product before a norm
// (EPI_RESIDUAL) adds itself into the float32 residual stream, writes bfloat16(x * next norm's weight) as the next
// product's activations and adds its tile's share of sum(x^2) per row to a counter; the product after the norm reads
// those activations as they are and multiplies its accumulators by 1 / sqrt(sum / K + eps) per row before its own
// epilogue.  The counter is a 64-bit fixed-point number (26 fractional bits): integer additions give the same sum
// in whatever order the tiles arrive, so a step's results do not vary from run to run.
constexpr float SUMSQ_TO_FIXED = 67108864.f, SUMSQ_FROM_FIXED = 1.f / 67108864.f;
struct SmallNormFuse {
    const unsigned long long *in_sumsq;   // [M] of the activation rows, or null: no scaling
    float in_eps;
    __nv_bfloat16 *xb;                    // EPI_RESIDUAL: [M, N] activations for the next product, or null
    const float *next_w;                  // [N] the next norm's weight
    unsigned long long *out_sumsq;        // [M], or null
    float scale;                          // x += scale * product
    int *status;                          // receives 4 if a tile's sum of squares is beyond the counter's range, or null
};
constexpr float SUMSQ_TILE_LIMIT = 9007199254740992.f;      // 2^53 in fixed point: a thousand tiles cannot wrap the counter

// EPI_QKV: where the fused [q | k | v] projection's columns go (bfloat16 all).
struct SmallQkvDest {
    __nv_bfloat16 *q_out;          // [M, nh * dh]
    __nv_bfloat16 *k_pages;        // [pages, nkvh, page_size, dh]
    __nv_bfloat16 *v_pages;
    const float *cos_table;        // [positions, dh / 2], or null: no rotation
    const float *sin_table;
    const int *positions;          // [M]
    const int *row_req;            // [M]
    const int *block_table;        // [requests, max_blocks]
    int nh, nkvh, dh, page_size, max_blocks;
};

struct SmallLinearArgs {
    const __nv_bfloat16 *act;   // [M, K]
    const __nv_bfloat16 *w;     // [N, K]  (EPI_SWIGLU: [2N, K], gate rows then up rows)
    void *out;                  // EPI_F32: float [M, ldo]; EPI_SWIGLU: bfloat16 [M, ldo]
    int M, N, K, ldo, ksplit, n_units;
    SmallQkvDest qkv;           // EPI_QKV only
    SmallNormFuse norm;         // the tile kernel only
    int *fault;                 // the TMA tile kernel: receives 1 when its bounded wait runs out, 2 for misaligned shared memory
};

constexpr int SL_MAX_WARPS = 8;
constexpr int SL_RING = 256;        // ring bytes per thread: 16 loads of 16 bytes in flight
constexpr int SL_RING_SMALL = 128;  // when the activations take most of the shared memory

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The weights a thread needs travel through a ring in shared memory that is private to the thread
// (it issues the 16-byte cp.async and it reads the result), DEPTH blocks of 32 k ahead of the
// tensor-core instructions that consume them, across the boundaries of tiles.  The first blocks
// are on their way before the activations are staged.
template <int MT, int EPI, int RING>      // MT: tiles of 8 activation rows (1 or 2); RING: ring bytes per thread
__global__ void __launch_bounds__(SL_MAX_WARPS * 32)
small_linear_kernel(SmallLinearArgs a) {
    pdl_trigger();
    constexpr int NW = EPI == EPI_SWIGLU ? 2 : 1;          // weight tiles a warp streams together
    constexpr int DEPTH = RING / (NW * 2 * 16);
    extern __shared__ __align__(16) unsigned char sl_smem[];
    const int nthreads = blockDim.x, nwarps = blockDim.x >> 5;
    uint4 *act_s = reinterpret_cast<uint4 *>(sl_smem);                          // [K / 8][MT * 8] units of 8 bf16
    uint4 *ring = act_s + (size_t)(a.K / 8) * MT * 8;                           // [DEPTH][NW][2][threads]
    float *red_s = reinterpret_cast<float *>(ring + (size_t)DEPTH * NW * 2 * nthreads);   // [warps][NW][MT][4][32]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    const int tiles_per_unit = nwarps / a.ksplit;
    const int tile_in_unit = warp / a.ksplit, kslice = warp - tile_in_unit * a.ksplit;
    const int kblocks = a.K / 32;
    const int per_slice = (kblocks + a.ksplit - 1) / a.ksplit;
    const int kb_begin = min(kblocks, kslice * per_slice), kb_end = min(kblocks, kb_begin + per_slice);
    const int nkb = kb_end - kb_begin;
    const int my_units = blockIdx.x < a.n_units ? (a.n_units - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int total_items = my_units * nkb;                  // (unit, k block) pairs of this warp, in order

    auto issue = [&](int q) {
        if (q < total_items) {
            const int ui = q / nkb, kb = kb_begin + (q - ui * nkb);
            const int n0 = ((blockIdx.x + ui * gridDim.x) * tiles_per_unit + tile_in_unit) * 16;
            if (n0 < a.N) {
                uint4 *slot = ring + (size_t)(q % DEPTH) * NW * 2 * nthreads + threadIdx.x;
#pragma unroll
                for (int w = 0; w < NW; ++w) {
                    // rows are clamped inside the matrix; what a clamped row yields is not stored
                    const size_t r0 = (size_t)w * a.N + min(n0 + g, a.N - 1), r1 = (size_t)w * a.N + min(n0 + g + 8, a.N - 1);
                    cp_async16(slot + (w * 2) * nthreads, a.w + r0 * a.K + kb * 32 + t * 8);
                    cp_async16(slot + (w * 2 + 1) * nthreads, a.w + r1 * a.K + kb * 32 + t * 8);
                }
            }
        }
        cp_async_commit();
    };
#pragma unroll
    for (int q = 0; q < DEPTH - 1; ++q) issue(q);     // weights do not depend on the kernel before this one
    pdl_wait();

    // activations into shared memory, [k / 8][row][8]; rows beyond M are zero.  Plain loads, eight in
    // flight per thread: they come from L2 and must not queue behind the weights' cp.async traffic.
    const int total_units = (a.K / 8) * MT * 8;
    for (int i0 = threadIdx.x; i0 < total_units; i0 += nthreads * 8) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * nthreads;
            const int kb = i / (MT * 8), row = i - kb * (MT * 8);
            v[u] = make_uint4(0, 0, 0, 0);
            if (i < total_units && row < a.M) v[u] = *reinterpret_cast<const uint4 *>(a.act + (size_t)row * a.K + kb * 8);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * nthreads;
            if (i < total_units) act_s[i] = v[u];
        }
    }
    __syncthreads();

    int q = 0;
    for (int ui = 0; ui < my_units; ++ui) {
        const int n0 = ((blockIdx.x + ui * gridDim.x) * tiles_per_unit + tile_in_unit) * 16;
        float acc[NW][MT][4];
#pragma unroll
        for (int w = 0; w < NW; ++w)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[w][m][0] = acc[w][m][1] = acc[w][m][2] = acc[w][m][3] = 0.f;
        for (int kb = kb_begin; kb < kb_end; ++kb, ++q) {
            issue(q + DEPTH - 1);
            cp_async_wait<DEPTH - 1>();
            if (n0 < a.N) {
                const uint4 *slot = ring + (size_t)(q % DEPTH) * NW * 2 * nthreads + threadIdx.x;
                uint4 wv[NW][2];
#pragma unroll
                for (int w = 0; w < NW; ++w) { wv[w][0] = slot[(w * 2) * nthreads]; wv[w][1] = slot[(w * 2 + 1) * nthreads]; }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint4 b = act_s[(kb * 4 + t) * (MT * 8) + m * 8 + g];
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        mma16816(acc[w][m], wv[w][0].x, wv[w][1].x, wv[w][0].y, wv[w][1].y, b.x, b.y);
                        mma16816(acc[w][m], wv[w][0].z, wv[w][1].z, wv[w][0].w, wv[w][1].w, b.z, b.w);
                    }
                }
            }
        }
        // partial sums of the K slices meet in shared memory
        if (a.ksplit > 1) {
#pragma unroll
            for (int w = 0; w < NW; ++w)
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        red_s[(((warp * NW + w) * MT + m) * 4 + c) * 32 + lane] = acc[w][m][c];
            __syncthreads();
            if (kslice == 0) {
                for (int s = 1; s < a.ksplit; ++s)
#pragma unroll
                    for (int w = 0; w < NW; ++w)
#pragma unroll
                        for (int m = 0; m < MT; ++m)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                acc[w][m][c] += red_s[((((warp + s) * NW + w) * MT + m) * 4 + c) * 32 + lane];
            }
        }
        if (kslice == 0 && n0 < a.N) {
            // accumulator element c of tile m: feature n0 + g (+8 for c >= 2), row m*8 + 2t + (c & 1)
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int n = n0 + g + (c >> 1) * 8, row = m * 8 + 2 * t + (c & 1);
                    if (n < a.N && row < a.M) {
                        if (EPI == EPI_F32) {
                            reinterpret_cast<float *>(a.out)[(size_t)row * a.ldo + n] = acc[0][m][c];
                        } else {
                            const float gate = acc[0][m][c], up = acc[NW - 1][m][c];
                            reinterpret_cast<__nv_bfloat16 *>(a.out)[(size_t)row * a.ldo + n] =
                                __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
                        }
                    }
                }
        }
        if (a.ksplit > 1) __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------------
// The kernel for every K whose tile of 16 weight rows fits in shared memory (K <= 6400).  One block =
// one tile of 16 features, its warps on slices of K, and NOTHING is staged or looped over: every
// thread issues the cp.async copies of its whole share of the tile at once (before it waits for the
// kernel before it: weights depend on nothing), so that the whole matrix is in flight over the GPU
// from the first microsecond; a pure read of the matrix in this pattern takes 6.9 us for 32 MB where
// a ring of 256 bytes per thread with the same access pattern takes 11.7.  The copies are committed
// in four groups and the products start when the first has landed.  The activations are not staged
// either: a thread reads its 16 bytes per block of 32 k straight from global memory (they sit in L2,
// a few tens of KB that every block reads), a few blocks ahead.  Shared memory holds the tile only
// (private to each thread: it reads back what it copied, so no barrier stands between copy and use);
// the K slices' partial sums meet in the same memory once the products are done.
// The TMA variant (the default where the weights are 16-byte aligned) brings the same tile as boxes of 8 rows x 64 k
// that one lane of each warp asks for; what a thread reads from shared memory and everything after is the same.
//   EPI_SWIGLU here pairs 8 gate rows with their 8 up rows in one 16-row tile: a thread's accumulators
//   c0, c1 are then the gate and c2, c3 the up of the same feature and activation rows.
//   EPI_QKV (the fused [q | k | v] projection) pairs, in the same way, 8 features of a head's first half
//   with their partners in the second half, so that a thread holds both members of a rotary pair; it
//   rotates query and key heads (rotate-half, float32 cos/sin at the row's position), rounds to
//   bfloat16 and writes queries to q_out and keys and values into their cache pages through the block
//   table (what a separate kernel did with a float32 copy of the product in between:
//   src/models/jiuge/jiuge.cpp:200-218).
// ---------------------------------------------------------------------------------------------------
constexpr int ST_GROUPS = 4;        // commit groups of a thread's copies
constexpr int ST_AHEAD = 4;         // blocks of k the activation loads run ahead (the TMA variant with 16 rows: 2, see there)

constexpr int ST_MAX_WARPS = 16;

// TMA = true: the tile comes as boxes of 8 rows x 64 k (1 KB, 128-byte swizzle) that one lane of each warp asks for,
// the slices of K are whole boxes, and a warp waits on a barrier of its own; a thread then reads from the boxes the same
// 16 bytes that it would have copied by itself.  Whole 128-byte lines by bulk copies instead of 16-byte copies from every
// thread: measured on a long stream (the logits' matrix) the per-thread copies reach 4.3 TB/s, TMA boxes 6.2.

template <int MT, int EPI, bool TMA, int AHEAD = ST_AHEAD>
__global__ void __launch_bounds__(ST_MAX_WARPS * 32)
small_linear_tile_kernel(const __grid_constant__ CUtensorMap map_w, SmallLinearArgs a) {
    pdl_trigger();
    extern __shared__ __align__(1024) unsigned char st_smem[];
    uint4 *mine = reinterpret_cast<uint4 *>(st_smem) + threadIdx.x;       // [2 * per_slice][threads]   (not TMA)
    const int nthreads = blockDim.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;           // warp = K slice
    const int g = lane >> 2, t = lane & 3;
    const int kblocks = a.K / 32;
    // TMA: slices of whole boxes (two blocks of 32 k each)
    const int per_slice = TMA ? 2 * (((kblocks + 1) / 2 + a.ksplit - 1) / a.ksplit) : (kblocks + a.ksplit - 1) / a.ksplit;
    const int kb_begin = min(kblocks, warp * per_slice), kb_end = min(kblocks, kb_begin + per_slice);
    const int nkb = kb_end - kb_begin;
    const int per_group = (per_slice + ST_GROUPS - 1) / ST_GROUPS;
    unsigned char *boxes = st_smem + (size_t)warp * (per_slice / 2) * 2048;     // TMA: [box of the slice][rows g | rows g + 8][8 x 128 bytes]
    unsigned long long *tile_full = reinterpret_cast<unsigned long long *>(st_smem + (size_t)a.ksplit * (per_slice / 2) * 2048);   // TMA: [warps]
    if (TMA && (smem_u32(st_smem) & 1023u)) {                 // swizzled boxes need it; never seen
        if (threadIdx.x == 0 && a.fault != nullptr) *reinterpret_cast<volatile int *>(a.fault) = 2;
        return;
    }
    // weight rows of this thread: EPI_F32: features n0 + g and n0 + g + 8; EPI_SWIGLU: gate and up of n0 + g.
    // Rows are clamped inside the matrix; what a clamped row yields is not stored.
    const int n0 = blockIdx.x * (EPI == EPI_SWIGLU ? 8 : 16);
    // EPI_QKV: block -> (head, 8 pairs of it); rows j0 + g of the head's first half and of its second half
    const int qkv_tiles = EPI == EPI_QKV ? a.qkv.dh / 16 : 1;
    const int qkv_head = blockIdx.x / qkv_tiles, qkv_j0 = (blockIdx.x % qkv_tiles) * 8;
    size_t r0 = min(n0 + g, a.N - 1);
    size_t r1 = EPI == EPI_SWIGLU ? (size_t)a.N + min(n0 + g, a.N - 1) : (size_t)min(n0 + g + 8, a.N - 1);
    if (EPI == EPI_QKV) {
        r0 = (size_t)qkv_head * a.qkv.dh + qkv_j0 + g;
        r1 = r0 + a.qkv.dh / 2;
    }
    if (TMA) {
        // first rows of the tile's two groups of eight (rows beyond the matrix arrive as zeros)
        int row_lo = n0, row_hi = EPI == EPI_SWIGLU ? a.N + n0 : n0 + 8;
        if (EPI == EPI_QKV) {
            row_lo = qkv_head * a.qkv.dh + qkv_j0;
            row_hi = row_lo + a.qkv.dh / 2;
        }
        if (lane == 0) {
            mbar_init(&tile_full[warp], 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
            const int nbox = (nkb + 1) / 2;
            if (nbox > 0) {
                mbar_expect_tx(&tile_full[warp], (unsigned)nbox * 2048u);
                for (int c = 0; c < nbox; ++c) {
                    tma_load_2d(boxes + (size_t)c * 2048, &map_w, &tile_full[warp], kb_begin * 32 + c * 64, row_lo);
                    tma_load_2d(boxes + (size_t)c * 2048 + 1024, &map_w, &tile_full[warp], kb_begin * 32 + c * 64, row_hi);
                }
            }
        }
        __syncwarp();
    } else {
        const __nv_bfloat16 *p0 = a.w + r0 * a.K + (size_t)kb_begin * 32 + t * 8;
        const __nv_bfloat16 *p1 = a.w + r1 * a.K + (size_t)kb_begin * 32 + t * 8;
        for (int d = 0; d < per_slice; ++d) {
            if (d < nkb) {
                cp_async16(mine + (size_t)(2 * d) * nthreads, p0 + d * 32);
                cp_async16(mine + (size_t)(2 * d + 1) * nthreads, p1 + d * 32);
            }
            if ((d + 1) % per_group == 0 || d + 1 == per_slice) cp_async_commit();
        }
        // every thread commits the same number of groups: pad to ST_GROUPS
        for (int j = (per_slice + per_group - 1) / per_group; j < ST_GROUPS; ++j) cp_async_commit();
    }
    pdl_wait();          // the weights do not depend on the kernel before this one; the activations do

    // what the epilogue of the first warp needs from memory is asked for now, so that it has arrived by then
    float pre_ss[MT][2], pre_x[MT][4], pre_w[2];
    if (warp == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int row = m * 8 + 2 * t + j;
                pre_ss[m][j] = a.norm.in_sumsq != nullptr && row < a.M ? __ull2float_rn(a.norm.in_sumsq[row]) * SUMSQ_FROM_FIXED : 0.f;
            }
        if (EPI == EPI_RESIDUAL) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int n = n0 + g + h * 8;
                pre_w[h] = a.norm.next_w != nullptr && n < a.N ? a.norm.next_w[n] : 0.f;
            }
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int row = m * 8 + 2 * t + (c & 1), n = n0 + g + (c >> 1) * 8;
                    pre_x[m][c] = n < a.N && row < a.M ? reinterpret_cast<const float *>(a.out)[(size_t)row * a.ldo + n] : 0.f;
                }
        }
    }
    // EPI_QKV: the row's position, its rotation and (key and value heads) the place of its cache slot hang on two loads
    // in a row each; asked for now, they are there when the products are done
    float pre_cs[MT][2], pre_sn[MT][2];
    size_t pre_slot[MT][2];
    if (EPI == EPI_QKV && warp == 0) {
        const SmallQkvDest &d = a.qkv;
        const int half = d.dh / 2, j = qkv_j0 + g, h = qkv_head;
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int row = m * 8 + 2 * t + c;
                pre_cs[m][c] = 1.f; pre_sn[m][c] = 0.f; pre_slot[m][c] = 0;
                if (row >= a.M) continue;
                const int pos = d.positions[row];
                if (d.cos_table != nullptr && h < d.nh + d.nkvh) {
                    pre_cs[m][c] = d.cos_table[(size_t)pos * half + j];
                    pre_sn[m][c] = d.sin_table[(size_t)pos * half + j];
                }
                if (h >= d.nh) {
                    const int page = d.block_table[(size_t)d.row_req[row] * d.max_blocks + pos / d.page_size];
                    pre_slot[m][c] = ((size_t)page * d.nkvh * d.page_size + (pos % d.page_size)) * d.dh;
                }
            }
    }

    const __nv_bfloat16 *ap[MT];
    bool arow[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        arow[m] = m * 8 + g < a.M;
        ap[m] = a.act + (size_t)(arow[m] ? m * 8 + g : 0) * a.K + (size_t)kb_begin * 32 + t * 8;
    }
    float acc[MT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;
    uint4 bq[AHEAD][MT];
#pragma unroll
    for (int d = 0; d < AHEAD; ++d)
#pragma unroll
        for (int m = 0; m < MT; ++m)
            bq[d][m] = (arow[m] && d < nkb) ? *reinterpret_cast<const uint4 *>(ap[m] + d * 32) : make_uint4(0, 0, 0, 0);

    if (TMA && nkb > 0 && !mbar_wait(&tile_full[warp], 0)) {
        if (lane == 0 && a.fault != nullptr) *reinterpret_cast<volatile int *>(a.fault) = 1;     // the products below run on what is there
        mbar_wait(&tile_full[warp], 0);                          // copies still on their way get a second bounded time to land
    }
    for (int q0 = 0; q0 < nkb; q0 += AHEAD) {
#pragma unroll
        for (int d = 0; d < AHEAD; ++d) {
            const int q = q0 + d;
            if (q < nkb) {
                uint4 w0, w1;
                if (TMA) {
                    // 16 bytes t of the block's 64 in row g of both groups; the 16-byte pieces of a row are swizzled by the row
                    const unsigned char *box = boxes + (size_t)(q >> 1) * 2048 + g * 128 + (((((q & 1) << 2) + t) ^ g) << 4);
                    w0 = *reinterpret_cast<const uint4 *>(box);
                    w1 = *reinterpret_cast<const uint4 *>(box + 1024);
                } else {
                    if (q % per_group == 0) {                       // the group of copies this block of k belongs to
                        const int grp = q / per_group;
                        if (grp == 0) cp_async_wait<ST_GROUPS - 1>();
                        else if (grp == 1) cp_async_wait<ST_GROUPS - 2>();
                        else if (grp == 2) cp_async_wait<ST_GROUPS - 3>();
                        else cp_async_wait<0>();
                    }
                    w0 = mine[(size_t)(2 * q) * nthreads];
                    w1 = mine[(size_t)(2 * q + 1) * nthreads];
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    const uint4 b = bq[d][m];
                    mma16816(acc[m], w0.x, w1.x, w0.y, w1.y, b.x, b.y);
                    mma16816(acc[m], w0.z, w1.z, w0.w, w1.w, b.z, b.w);
                    if (arow[m] && q + AHEAD < nkb) bq[d][m] = *reinterpret_cast<const uint4 *>(ap[m] + (q + AHEAD) * 32);
                }
            }
        }
    }
    // partial sums of the K slices meet in shared memory (the tile's place: every product is done)
    if (a.ksplit > 1) {
        __syncthreads();
        float *red_s = reinterpret_cast<float *>(st_smem);               // [warps][MT][4][32]
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) red_s[((warp * MT + m) * 4 + c) * 32 + lane] = acc[m][c];
        __syncthreads();
        if (warp == 0) {
            for (int s = 1; s < a.ksplit; ++s)
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[m][c] += red_s[((s * MT + m) * 4 + c) * 32 + lane];
        }
    }
    if (warp == 0 && a.norm.in_sumsq != nullptr) {
        // the activations came without their norm's 1 / rms: it is a factor of the whole row of the product
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float inv = rsqrtf(pre_ss[m][j] / (float)a.K + a.norm.in_eps);
                acc[m][j] *= inv;
                acc[m][j + 2] *= inv;
            }
    }
    if (warp == 0 && EPI == EPI_RESIDUAL) {
        // element c of tile m: feature n0 + g (+8 for c >= 2), activation row m*8 + 2t + (c & 1)
        float *x = reinterpret_cast<float *>(a.out);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float ss[2] = {0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int row = m * 8 + 2 * t + (c & 1), n = n0 + g + (c >> 1) * 8;
                if (n < a.N && row < a.M) {
                    const float v = pre_x[m][c] + a.norm.scale * acc[m][c];
                    x[(size_t)row * a.ldo + n] = v;
                    if (a.norm.xb != nullptr) a.norm.xb[(size_t)row * a.N + n] = __float2bfloat16_rn(v * pre_w[c >> 1]);
                    ss[c & 1] += v * v;
                }
            }
            if (a.norm.out_sumsq != nullptr) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float v = ss[j];                                     // over the eight lanes that share t
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 16);
                    const int row = m * 8 + 2 * t + j;
                    if (g == 0 && row < a.M) {
                        float fx = v * SUMSQ_TO_FIXED;
                        if (!(fx < SUMSQ_TILE_LIMIT)) {                  // also a NaN: say so instead of wrapping around
                            if (a.norm.status != nullptr) atomicExch(a.norm.status, 4);
                            fx = SUMSQ_TILE_LIMIT;
                        }
                        atomicAdd(a.norm.out_sumsq + row, __float2ull_rn(fx));
                    }
                }
            }
        }
    } else if (warp == 0 && EPI == EPI_QKV) {
        const SmallQkvDest &d = a.qkv;
        const int half = d.dh / 2, j = qkv_j0 + g, h = qkv_head;
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int row = m * 8 + 2 * t + c;
                if (row >= a.M) continue;
                float y0 = acc[m][c], y1 = acc[m][c + 2];                 // elements j and j + half of head h
                if (d.cos_table != nullptr && h < d.nh + d.nkvh) {
                    const float cs = pre_cs[m][c], sn = pre_sn[m][c];
                    const float x0 = y0, x1 = y1;
                    y0 = x0 * cs - x1 * sn;
                    y1 = x0 * sn + x1 * cs;
                }
                __nv_bfloat16 *dst;
                if (h < d.nh) {
                    dst = d.q_out + ((size_t)row * d.nh + h) * d.dh;
                } else {
                    dst = (h < d.nh + d.nkvh ? d.k_pages + (size_t)(h - d.nh) * d.page_size * d.dh
                                             : d.v_pages + (size_t)(h - d.nh - d.nkvh) * d.page_size * d.dh) + pre_slot[m][c];
                }
                dst[j] = __float2bfloat16_rn(y0);
                dst[j + half] = __float2bfloat16_rn(y1);
            }
    } else if (warp == 0) {
        // accumulator element c of tile m: weight row g (+8 for c >= 2), activation row m*8 + 2t + (c & 1)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int c = 0; c < (EPI == EPI_SWIGLU ? 2 : 4); ++c) {
                const int row = m * 8 + 2 * t + (c & 1);
                if (EPI == EPI_F32) {
                    const int n = n0 + g + (c >> 1) * 8;
                    if (n < a.N && row < a.M) reinterpret_cast<float *>(a.out)[(size_t)row * a.ldo + n] = acc[m][c];
                } else {
                    const int n = n0 + g;
                    const float gate = acc[m][c], up = acc[m][c + 2];
                    if (n < a.N && row < a.M)
                        reinterpret_cast<__nv_bfloat16 *>(a.out)[(size_t)row * a.ldo + n] =
                            __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
                }
            }
    }
}

// Shared memory of the tile kernel: the tile, padded to whole slices (and room for the partial sums).
static size_t small_tile_smem(int K, int MT, int ksplit) {
    const int per_slice = (K / 32 + ksplit - 1) / ksplit;
    const size_t tile = (size_t)2 * per_slice * ksplit * 32 * 16;
    const size_t red = (size_t)ksplit * MT * 4 * 32 * sizeof(float);
    return tile > red ? tile : red;
}

// The slices of K of the TMA variant: as many warps (4 to 16) as share the boxes of 64 k out most evenly, more if equal.
// With 16 activation rows a thread holds 80 registers: ten warps at most, so that three blocks still share an SM.
// Measured in a 2B decode step (ms, batch 1 / 8 / 16 at 512 keys) for lookahead and warps: 4 and 12: 1.66, 2.02, 2.91;
// 4 and 9: 1.72, 2.05, 2.75; 2 and 9: 1.75, 2.16, 2.58; 6 and 12: 1.58, 2.04, 3.23; per-thread copies: 1.83, 2.07, 2.62.
static int tma_ksplit(int K, int MT) {
    const int boxes = (K + 63) / 64;
    int best = 1, best_waste = 1 << 30;
    for (int w = MT == 2 ? 10 : ST_MAX_WARPS; w >= 4; --w) {
        const int waste = (boxes + w - 1) / w * w - boxes;
        if (waste < best_waste) { best = w; best_waste = waste; }
    }
    return boxes < 4 ? boxes : best;
}
static size_t small_tile_smem_tma(int K, int MT, int ksplit) {
    const int boxes = (K + 63) / 64, per_warp = (boxes + ksplit - 1) / ksplit;
    const size_t tile = (size_t)ksplit * per_warp * 2048;
    const size_t red = (size_t)ksplit * MT * 4 * 32 * sizeof(float);
    return (tile > red ? tile : red) + ST_MAX_WARPS * sizeof(unsigned long long);
}
// The word that a tile kernel writes when its bounded wait runs out lies in pinned host memory that the device
// reaches too: the host reads it without a copy (after the stream is idle).  One word per process.
static int *fault_word() {
    static int *word = [] {
        int *p = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void **>(&p), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) return (int *)nullptr;
        *p = 0;
        return p;
    }();
    return word;
}
JK_EXPORT int jk_linear_small_take_fault() {
    int *w = fault_word();
    if (w == nullptr) return 0;
    const int v = *reinterpret_cast<volatile int *>(w);
    if (v != 0) *reinterpret_cast<volatile int *>(w) = 0;
    return v;
}

template <int MT, int EPI>
static int launch_tile(const SmallLinearArgs &a_in, size_t smem, cudaStream_t stream) {
    SmallLinearArgs a = a_in;
    const int tiles = EPI == EPI_SWIGLU ? (a.N + 7) / 8 : (a.N + 15) / 16;     // EPI_QKV: 16 features a tile as well
    static const bool tma_off = [] { const char *v = getenv("JK_SMALL_NO_TMA"); return v && v[0] == '1'; }();
    const int ks = tma_ksplit(a.K, MT);
    const size_t smem_tma = small_tile_smem_tma(a.K, MT, ks);
    CUtensorMap map_w;
    bool tma = !tma_off && (reinterpret_cast<uintptr_t>(a.w) & 15) == 0 && smem_tma <= 200 * 1024;
    if (tma) {
        const int rows = EPI == EPI_SWIGLU ? 2 * a.N : a.N;
        if (tensor_map_2d(a.w, rows, a.K, a.K, 8, 64, 2, &map_w) != JK_OK) tma = false;      // the other variant needs none
    }
    if (tma) {
        a.ksplit = ks;
        a.fault = fault_word();          // (unified addressing: the device uses the host's address)
        // How far the activation loads run ahead of the products: all the way where every block has an SM to itself
        // (registers are no object there and no load's latency shows: batch 8 at 512 keys 1.99 -> 1.92 ms a step); else 4
        // blocks of k.  With 16 rows: 4 and 2 (all the way costs 128 registers and spills: batch 16 2.52 -> 2.78 ms).
        static const int sms = [] {
            int dev = 0, n = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
            return n;
        }();
        // (Tiles of 8 rows for the products that have one tile of 16 per SM, twice the blocks of half the size: slower,
        // batch 8 at 512 keys 1.92 -> 2.18 ms a step; every block reads all the activation rows from L2, and twice the
        // blocks read them twice.)
        auto kernel = tiles <= sms ? small_linear_tile_kernel<MT, EPI, true, MT == 2 ? 4 : 12> : small_linear_tile_kernel<MT, EPI, true, MT == 2 ? 2 : ST_AHEAD>;
        if (smem_tma > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_tma);
            if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "linear_small: %s", cudaGetErrorString(e));
        }
        jk_launch(kernel, dim3(tiles), dim3(a.ksplit * 32), smem_tma, stream, map_w, a);
        JK_CHECK_LAUNCH("linear_small");
        return JK_OK;
    }
    memset(&map_w, 0, sizeof(map_w));
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(small_linear_tile_kernel<MT, EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "linear_small: %s", cudaGetErrorString(e));
    }
    jk_launch(small_linear_tile_kernel<MT, EPI, false>, dim3(tiles), dim3(a.ksplit * 32), smem, stream, map_w, a);
    JK_CHECK_LAUNCH("linear_small");
    return JK_OK;
}

static size_t small_linear_smem(int K, int MT, int warps, int ring) {
    return (size_t)(K / 8) * MT * 8 * 16 + (size_t)ring * warps * 32 + (size_t)warps * 2 * MT * 4 * 32 * sizeof(float);
}
// The deep ring unless the activations leave too little room for it.
static int small_linear_ring(int K, int MT, int warps) {
    return small_linear_smem(K, MT, warps, SL_RING) <= 170 * 1024 ? SL_RING : SL_RING_SMALL;
}

template <int MT, int EPI, int RING>
static int launch_small(const SmallLinearArgs &a, int ctas, int warps, size_t smem, cudaStream_t stream) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(small_linear_kernel<MT, EPI, RING>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "linear_small: %s", cudaGetErrorString(e));
    }
    jk_launch(small_linear_kernel<MT, EPI, RING>, dim3(ctas), dim3(warps * 32), smem, stream, a);
    JK_CHECK_LAUNCH("linear_small");
    return JK_OK;
}

// Does this kernel take the product?  (M rows, K a multiple of 32, the activations fit in shared memory.)
JK_EXPORT int jk_linear_small_supports(int M, int N, int K) {
    if (M < 1 || M > 16 || N < 1 || K < 32 || K % 32) return 0;
    const int MT = M <= 8 ? 1 : 2;
    // the tile kernel (a 16-row tile of W in shared memory) or the ring kernel (the activations in shared memory)
    int ksplit = ST_MAX_WARPS;
    while (ksplit > 1 && (K / 32) / ksplit < 2) ksplit /= 2;
    if (small_tile_smem(K, MT, ksplit) <= 200 * 1024) return 1;
    return small_linear_smem(K, MT, 8, small_linear_ring(K, MT, 8)) <= 200 * 1024;
}

// The fused [q | k | v] projection of at most 16 rows with rotation and cache write in its epilogue.
// Any head size that is a multiple of 16; K up to what a 16-row tile may take of shared memory.
JK_EXPORT int jk_linear_small_qkv_supports(int M, int K, int dh) {
    if (M < 1 || M > 16 || K < 32 || K % 32 || dh < 16 || dh % 16) return 0;
    int ksplit = ST_MAX_WARPS;
    while (ksplit > 1 && (K / 32) / ksplit < 2) ksplit /= 2;
    return small_tile_smem(K, M <= 8 ? 1 : 2, ksplit) <= 200 * 1024;
}

static int linear_small_qkv_impl(const void *act, const void *w, int M, int K, void *q_out, void *k_pages, void *v_pages,
                                 const float *cos_table, const float *sin_table, const int *positions,
                                 const int *row_req, const int *block_table, int max_blocks, int page_size, int nh,
                                 int nkvh, int dh, int sms, const SmallNormFuse &norm, cudaStream_t stream) {
    JK_REQUIRE(jk_linear_small_qkv_supports(M, K, dh), "linear_small_qkv: M %d K %d head size %d is outside what the kernel takes", M, K, dh);
    JK_REQUIRE(nh >= 1 && nkvh >= 1 && q_out && k_pages && v_pages && positions && row_req && block_table && max_blocks > 0 && page_size > 0,
               "linear_small_qkv: a destination or index array is missing");
    JK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "linear_small_qkv: cos and sin tables come together");
    if (sms <= 0) sms = 148;
    const int N = (nh + 2 * nkvh) * dh, MT = M <= 8 ? 1 : 2;
    const int n_tiles = N / 16;
    int ksplit = n_tiles < 2 * sms ? ST_MAX_WARPS : SL_MAX_WARPS;
    while (ksplit > 1 && (K / 32) / ksplit < 2) ksplit /= 2;
    const size_t smem = small_tile_smem(K, MT, ksplit);
    SmallLinearArgs a{(const __nv_bfloat16 *)act, (const __nv_bfloat16 *)w, nullptr, M, N, K, N, ksplit, 0,
                      SmallQkvDest{(__nv_bfloat16 *)q_out, (__nv_bfloat16 *)k_pages, (__nv_bfloat16 *)v_pages, cos_table,
                                   sin_table, positions, row_req, block_table, nh, nkvh, dh, page_size, max_blocks}, norm};
    if (MT == 1) return launch_tile<1, EPI_QKV>(a, smem, stream);
    return launch_tile<2, EPI_QKV>(a, smem, stream);
}

JK_EXPORT int jk_linear_small_qkv(const void *act, const void *w, int M, int K, void *q_out, void *k_pages, void *v_pages,
                                  const float *cos_table, const float *sin_table, const int *positions,
                                  const int *row_req, const int *block_table, int max_blocks, int page_size, int nh,
                                  int nkvh, int dh, int sms, cudaStream_t stream) {
    return linear_small_qkv_impl(act, w, M, K, q_out, k_pages, v_pages, cos_table, sin_table, positions, row_req, block_table,
                                 max_blocks, page_size, nh, nkvh, dh, sms, SmallNormFuse{}, stream);
}

// The same with activations that came without their norm's 1 / rms (see SmallNormFuse): `in_sumsq` holds the rows'
// sums of squares as the product before the norm left them, K is the norm's width.
JK_EXPORT int jk_linear_small_qkv_norm(const void *act, const void *w, int M, int K, void *q_out, void *k_pages, void *v_pages,
                                       const float *cos_table, const float *sin_table, const int *positions,
                                       const int *row_req, const int *block_table, int max_blocks, int page_size, int nh,
                                       int nkvh, int dh, const unsigned long long *in_sumsq, float in_eps, int sms,
                                       cudaStream_t stream) {
    JK_REQUIRE(in_sumsq != nullptr, "linear_small_qkv_norm: no sums of squares");
    SmallNormFuse norm{};
    norm.in_sumsq = in_sumsq;
    norm.in_eps = in_eps;
    return linear_small_qkv_impl(act, w, M, K, q_out, k_pages, v_pages, cos_table, sin_table, positions, row_req, block_table,
                                 max_blocks, page_size, nh, nkvh, dh, sms, norm, stream);
}

static size_t tile_kernel_smem(int M, int N, int K, int epilogue, int sms, int *ksplit_out) {
    const int n_tiles = epilogue == EPI_SWIGLU ? (N + 7) / 8 : (N + 15) / 16;
    int ksplit = n_tiles < 2 * (sms > 0 ? sms : 148) ? ST_MAX_WARPS : SL_MAX_WARPS;
    while (ksplit > 1 && (K / 32) / ksplit < 2) ksplit /= 2;
    if (ksplit_out) *ksplit_out = ksplit;
    return small_tile_smem(K, M <= 8 ? 1 : 2, ksplit);
}

// The products of a chain without norm kernels run on the tile kernel only (K up to what a 16-row tile may take
// of shared memory).
JK_EXPORT int jk_linear_small_norm_supports(int M, int N, int K) {
    if (M < 1 || M > 16 || N < 1 || K < 32 || K % 32) return 0;
    return tile_kernel_smem(M, N, K, EPI_F32, 148, nullptr) <= 200 * 1024 && tile_kernel_smem(M, N, K, EPI_SWIGLU, 148, nullptr) <= 200 * 1024;
}

static int linear_small_impl(const void *act, const void *w, void *out, int M, int N, int K, int ldo,
                             int epilogue, int sms, const SmallNormFuse &norm, bool fused, cudaStream_t stream) {
    JK_REQUIRE(jk_linear_small_supports(M, N, K), "linear_small: M %d N %d K %d is outside what the kernel takes "
               "(1..16 rows, K a multiple of 32)", M, N, K);
    JK_REQUIRE(epilogue == EPI_F32 || epilogue == EPI_SWIGLU || (fused && epilogue == EPI_RESIDUAL), "linear_small: epilogue %d", epilogue);
    JK_REQUIRE(ldo >= N, "linear_small: output stride %d < N %d", ldo, N);
    const int MT = M <= 8 ? 1 : 2;
    {
        // the tile kernel: all warps of a block on one tile, as many slices of K as leave each at least two
        // blocks of k; 16 warps when the tiles are too few to give every SM two blocks (the copies are
        // issued by more threads and each slice is shorter), else 8
        if (sms <= 0) sms = 148;
        const int n_tiles = epilogue == EPI_SWIGLU ? (N + 7) / 8 : (N + 15) / 16;
        int ksplit = n_tiles < 2 * sms ? ST_MAX_WARPS : SL_MAX_WARPS;
        while (ksplit > 1 && (K / 32) / ksplit < 2) ksplit /= 2;
        const size_t smem = small_tile_smem(K, MT, ksplit);
        if (smem <= 200 * 1024) {
            SmallLinearArgs a{(const __nv_bfloat16 *)act, (const __nv_bfloat16 *)w, out, M, N, K, ldo, ksplit, 0, SmallQkvDest{}, norm};
            if (MT == 1 && epilogue == EPI_F32) return launch_tile<1, EPI_F32>(a, smem, stream);
            if (MT == 2 && epilogue == EPI_F32) return launch_tile<2, EPI_F32>(a, smem, stream);
            if (MT == 1 && epilogue == EPI_RESIDUAL) return launch_tile<1, EPI_RESIDUAL>(a, smem, stream);
            if (MT == 2 && epilogue == EPI_RESIDUAL) return launch_tile<2, EPI_RESIDUAL>(a, smem, stream);
            if (MT == 1) return launch_tile<1, EPI_SWIGLU>(a, smem, stream);
            return launch_tile<2, EPI_SWIGLU>(a, smem, stream);
        }
        JK_REQUIRE(!fused, "linear_small_norm: K %d is beyond the tile kernel", K);
    }
    const int tiles = (N + 15) / 16;
    if (sms <= 0) sms = 148;
    // Blocks of 4 warps, several per SM; a block works on one tile of 16 features at a time with its
    // warps on slices of K (short chains, and the work is cut finely enough to balance over the SMs).
    // 8 warps on one tile when the matrix is small in N (few tiles to go round) or long in K (the
    // chain of loads per warp would be long); else 4
    const int warps = (tiles <= 2 * sms || K >= 4096) ? 8 : 4;
    int ksplit = warps;
    while (ksplit > 1 && (K / 32) / ksplit < 2) ksplit /= 2;
    const int tiles_per_unit = warps / ksplit;
    SmallLinearArgs a{(const __nv_bfloat16 *)act, (const __nv_bfloat16 *)w, out, M, N, K, ldo, ksplit,
                      (tiles + tiles_per_unit - 1) / tiles_per_unit, SmallQkvDest{}};
    const int ring = small_linear_ring(K, MT, warps);
    const size_t smem = small_linear_smem(K, MT, warps, ring);
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    if (per_sm > 6) per_sm = 6;
    if (per_sm < 1) per_sm = 1;
    const int ctas = a.n_units < sms * per_sm ? a.n_units : sms * per_sm;
#define SL_LAUNCH(MT_, EPI_)                                                                            \
    return ring == SL_RING ? launch_small<MT_, EPI_, SL_RING>(a, ctas, warps, smem, stream)             \
                           : launch_small<MT_, EPI_, SL_RING_SMALL>(a, ctas, warps, smem, stream)
    if (MT == 1 && epilogue == EPI_F32) SL_LAUNCH(1, EPI_F32);
    if (MT == 2 && epilogue == EPI_F32) SL_LAUNCH(2, EPI_F32);
    if (MT == 1) SL_LAUNCH(1, EPI_SWIGLU);
    SL_LAUNCH(2, EPI_SWIGLU);
#undef SL_LAUNCH
}

JK_EXPORT int jk_linear_small(const void *act, const void *w, void *out, int M, int N, int K, int ldo,
                              int epilogue, int sms, cudaStream_t stream) {
    return linear_small_impl(act, w, out, M, N, K, ldo, epilogue, sms, SmallNormFuse{}, false, stream);
}

// A product of a chain without norm kernels (see SmallNormFuse).  epilogue EPI_F32 or EPI_SWIGLU with `in_sumsq`: the
// activations came without their norm's 1 / rms, which the accumulators get per row before the epilogue (K is the norm's
// width).  epilogue EPI_RESIDUAL: `out` is the float32 residual stream x [M, ldo]: x += scale * product; if `xb` is given
// it receives bfloat16(x * next_w) [M, N] and `out_sumsq` [M] this product's share of sum(x^2) per row (the caller
// zeroes the counters before the first product of a step that adds to them; `status`, if given, receives 4 when a
// tile's sum of squares is beyond what the counters hold: activations of several thousand on average).
JK_EXPORT int jk_linear_small_norm(const void *act, const void *w, void *out, int M, int N, int K, int ldo, int epilogue,
                                   const unsigned long long *in_sumsq, float in_eps, void *xb, const float *next_w,
                                   unsigned long long *out_sumsq, float scale, int *status, int sms, cudaStream_t stream) {
    JK_REQUIRE(jk_linear_small_norm_supports(M, N, K), "linear_small_norm: M %d N %d K %d is outside what the tile kernel takes", M, N, K);
    JK_REQUIRE(out != nullptr && (xb == nullptr) == (next_w == nullptr) && (xb == nullptr) == (out_sumsq == nullptr),
               "linear_small_norm: the next product's activations, the norm's weight and the counters come together");
    JK_REQUIRE(epilogue == EPI_RESIDUAL || xb == nullptr, "linear_small_norm: only the residual epilogue writes activations");
    SmallNormFuse norm{in_sumsq, in_eps, (__nv_bfloat16 *)xb, next_w, out_sumsq, scale, status};
    return linear_small_impl(act, w, out, M, N, K, ldo, epilogue, sms, norm, true, stream);
}
