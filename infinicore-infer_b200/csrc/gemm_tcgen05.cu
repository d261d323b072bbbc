// Matrix products for steps of many rows (prefill): C[M, N] = A[M, K] * W[N, K]^T on the
// 5th-generation tensor cores of sm_100a, with the layer's elementwise work in the epilogue.
//
//   operands   bfloat16, both K-major (A rows are tokens, W rows are output features), brought
//              into shared memory by TMA (cp.async.bulk.tensor.2d) as 128-byte-swizzled tiles of
//              [rows][64] through a ring of STAGES stages guarded by full/empty mbarriers;
//   product    tcgen05.mma.cta_group::1.kind::f16, M = 128, N = BN, K = 16 per instruction, issued
//              by one elected thread, float32 accumulator in tensor memory (BN columns x 128 lanes);
//              tcgen05.commit hands a finished stage back to the TMA warp and the finished
//              accumulator to the epilogue;
//   tiles      a block is persistent: it walks over output tiles with two accumulators in tensor
//              memory, so that the epilogue of one tile runs while the next tile's products are issued;
//   epilogue   four warps read the accumulator with tcgen05.ld (each warp its quarter of the
//              lanes; a thread holds 32 consecutive columns of one row), stage 32 rows x 128 bytes in
//              swizzled shared memory and hand them to TMA (a store, or a reduce-add for the residual:
//              the memory system does x += value, the SM never reads x) and apply one of
//                EPI_F32       out[m, n]  = acc                      float32
//                EPI_BF16      out[m, n]  = acc                      bfloat16
//                EPI_RESIDUAL  out[m, n] += scale * acc              float32, in place (the residual stream)
//                EPI_SWIGLU    out[m, n]  = silu(acc[n]) * acc[N+n]  bfloat16; W is [2N, K], gate rows then
//                                                                    up rows, and a tile holds BN/2 of each.
//                EPI_QKV       the columns are heads [q | k | v]: query and key heads are rotated (rotate-half,
//                              angles from float32 cos/sin tables at the row's position) and rounded to
//                              bfloat16; queries go to q_out, keys and values straight into their cache
//                              pages through the block table (what a separate rotary kernel did with a
//                              float32 copy of the product in between: src/models/jiuge/jiuge.cpp:200-218).
// Rows, columns and the K range that a tile has beyond the matrices are zero-filled by TMA and
// never stored.  Warp roles: warp 0 TMA, warp 1 MMA (and owner of the tensor-memory allocation),
// warps 2..5 epilogue.  Every wait on an mbarrier is bounded; a wait that runs out records a code in
// `status`, the roles drain what is in flight, tensor memory is freed and the kernel returns.
//
// (The reference sends these products to a library: src/models/inference_context.cpp:59-79; the
// residual add is its beta = 1, the SwiGLU a separate operator, jiuge.cpp:236-249.)
#include "tcgen05.cuh"

JK_DEFINE_ERROR_BUFFER(jk_gemm_tcgen05)


// EPI_QKV: where the fused [q | k | v] projection's columns go (bfloat16 all).
struct QkvDest {
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

struct TgArgs {
    void *out;
    int M, N, K, ldo;
    float scale;
    int *status;       // device word: 0, or the code of the wait that ran out
    int direct;        // 1: the output's rows are not 16-byte aligned, store from registers instead of by TMA
    int ksplit;        // EPI_RESIDUAL by TMA only: a tile's K is cut into this many units whose partial products all add
                       // themselves into the output (0 or 1: none)
    QkvDest qkv;       // EPI_QKV only
};

template <int BN, int CTAS> struct TgSmem {
    static constexpr int STAGES = CTAS == 2 ? 6 : TG_STAGES;
    __nv_bfloat16 a[STAGES][TG_BM * TG_BK];          // 16 KB each, 1024-byte aligned
    __nv_bfloat16 b[STAGES][BN / CTAS * TG_BK];
    unsigned char stage_out[4][4096];                // per epilogue warp: 32 rows x 128 bytes, swizzled
    unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    unsigned tmem_base;
};

// One 16-byte piece of a staging row: piece `chunk` of row `row` sits at chunk ^ (row & 7), the
// 128-byte swizzle that the output's tensor map undoes.
__device__ __forceinline__ void stage_write(unsigned char *tile, int row, int chunk, uint4 v) {
    *reinterpret_cast<uint4 *>(tile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}

// The order in which workers walk the output tiles: groups of 8 rows of tiles, within a group down the rows first and
// then along the columns.  The tiles that run at the same time then share a few tiles of W (each read from memory
// once and from L2 by the other rows of the group) and the group's rows of A, whatever the size of W; walking along
// the columns first reads all of W once per row of tiles (at 268 MB of gate/up weights: 2 GB instead of 0.3).
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &tm, int &tn) {
    constexpr int GM = 8;
    const int per_group = GM * tiles_n;
    const int mg = tile / per_group, r = tile - mg * per_group;
    const int gm = min(GM, tiles_m - mg * GM);
    tm = mg * GM + r % gm;
    tn = r / gm;
}

template <int BN, int EPI, int CTAS>
__global__ void __launch_bounds__(TG_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, TgArgs a) {
    extern __shared__ unsigned char tg_raw[];
    using Smem = TgSmem<BN, CTAS>;
    Smem &s = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(tg_raw) + 1023) & ~uintptr_t(1023));
    constexpr int STAGES = Smem::STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // EPI_SWIGLU: a tile's B rows are BN/2 gate rows and the BN/2 up rows that belong to them
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? BN / 2 : BN;
    // bytes that land per stage, over the pair when there is one (the first block's barrier counts both)
    constexpr unsigned STAGE_BYTES = CTAS * (TG_BM + BN / CTAS) * TG_BK * sizeof(__nv_bfloat16);
    // a worker is a block, or a pair of blocks (a cluster of two: blocks 2c and 2c + 1) on a tile of 256 rows
    const int rank = CTAS == 2 ? (int)cluster_rank() : 0;
    const int worker = blockIdx.x / CTAS, workers = gridDim.x / CTAS;
    constexpr int TILE_M = TG_BM * CTAS;
    const int tiles_n = (a.N + OUT_COLS - 1) / OUT_COLS, tiles_m = (a.M + TILE_M - 1) / TILE_M;
    // a unit of work is a tile, or one of a tile's `ksplit` ranges of K (units of one tile follow one another, so
    // they run at the same time on different workers and add into the same tile of the output)
    const int ksplit = a.ksplit > 1 ? a.ksplit : 1;
    const int num_tiles = tiles_n * tiles_m * ksplit;
    const int nk_all = (a.K + TG_BK - 1) / TG_BK, nk_unit = (nk_all + ksplit - 1) / ksplit;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], 4 * CTAS); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        if (CTAS == 2) tmem_alloc_pair(&s.tmem_base, 2 * BN);
        else tmem_alloc(&s.tmem_base, 2 * BN);
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) cluster_sync();      // the other block's barriers exist before anything arrives on them
    tc_fence_after();
    const unsigned tmem = s.tmem_base;
    int failed = 0;
    // The next kernel may be scheduled only once every block holds its tensor memory: a later kernel that
    // took tensor memory on an SM and then waited for this grid, while a block of this grid still waited
    // for tensor memory there, would never end.
    pdl_trigger();
    // barriers and tensor memory are set up.  The weights depend on no kernel before this one: the producer asks for
    // the first stages' tiles of B at once and waits for the kernel before only then, for the activations (A); the
    // epilogue warps wait before their first access to what earlier kernels wrote.

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            // one stage's loads: `which` 1: the tile of B (and the count of the stage's bytes), 2: the tile of A, 3: both
            auto load_stage = [&](int st, int i, int m0, int n0, int which) {
                if (CTAS == 2) {
                    // each block loads its own rows of A and its half of the tile's rows of B (gate rows in the
                    // first block, up rows in the second for SwiGLU); the first block's barrier counts all bytes
                    if (rank == 0 && (which & 1)) mbar_expect_tx(&s.full[st], STAGE_BYTES);
                    const unsigned bar = cluster_addr(&s.full[st], 0);
                    const int w0 = EPI == EPI_SWIGLU ? (rank ? a.N + n0 : n0) : n0 + rank * (BN / 2);
                    if (which & 2) tma_load_2d_pair(s.a[st], &map_a, bar, i * TG_BK, m0);
                    if (which & 1) tma_load_2d_pair(s.b[st], &map_w, bar, i * TG_BK, w0);
                    return;
                }
                if (which & 1) mbar_expect_tx(&s.full[st], STAGE_BYTES);
                if (which & 2) tma_load_2d(s.a[st], &map_a, &s.full[st], i * TG_BK, m0);
                if (which & 1) {
                    tma_load_2d(s.b[st], &map_w, &s.full[st], i * TG_BK, n0);
                    if (EPI == EPI_SWIGLU)
                        tma_load_2d(s.b[st] + (BN / 2) * TG_BK, &map_w, &s.full[st], i * TG_BK, a.N + n0);
                }
            };
            // the stages that are free from the start, twice: the weights now, the activations after the wait
            for (int pass = 1; pass <= 2; ++pass) {
                int it = 0;
                for (int tile = worker; tile < num_tiles && it < STAGES; tile += workers) {
                    int tm, tn;
                    tile_coords(tile / ksplit, tiles_m, tiles_n, tm, tn);
                    const int m0 = tm * TILE_M + rank * TG_BM, n0 = tn * OUT_COLS;
                    const int k_first = (tile % ksplit) * nk_unit, nk = min(nk_unit, nk_all - k_first);
                    for (int i = k_first; i < k_first + nk && it < STAGES; ++i, ++it) load_stage(it, i, m0, n0, pass);
                }
                if (pass == 1) pdl_wait();
            }
            int it = 0;
            for (int tile = worker; tile < num_tiles && !failed; tile += workers) {
                int tm, tn;
                tile_coords(tile / ksplit, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * TILE_M + rank * TG_BM, n0 = tn * OUT_COLS;
                const int k_first = (tile % ksplit) * nk_unit, nk = min(nk_unit, nk_all - k_first);
                for (int i = k_first; i < k_first + nk; ++i, ++it) {
                    if (it < STAGES) continue;                       // asked for above
                    const int st = it % STAGES;
                    if (!mbar_wait(&s.empty[st], ((it / STAGES) - 1) & 1)) { failed = 1; break; }
                    load_stage(st, i, m0, n0, 3);
                }
            }
            if (failed) atomicExch(a.status, 1);
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0 && rank == 0) {      // of a pair, the first block issues for both
            constexpr unsigned idesc = instr_desc_bf16(BN, TILE_M);
            int it = 0, j = 0;
            for (int tile = worker; tile < num_tiles && !failed; tile += workers, ++j) {
                const int buf = j & 1;
                if (j >= 2 && !mbar_wait(&s.acc_empty[buf], ((j >> 1) - 1) & 1)) { failed = 2; break; }
                tc_fence_after();
                const unsigned acc = tmem + buf * BN;
                const int nk = min(nk_unit, nk_all - (tile % ksplit) * nk_unit);
                for (int i = 0; i < nk; ++i, ++it) {
                    const int st = it % STAGES;
                    if (!mbar_wait(&s.full[st], (it / STAGES) & 1)) { failed = 2; break; }
                    tc_fence_after();
                    const unsigned long long ad = smem_desc_sw128(s.a[st]), bd = smem_desc_sw128(s.b[st]);
#pragma unroll
                    for (int k = 0; k < TG_BK / 16; ++k) {    // 32 bytes further along K per instruction
                        if (CTAS == 2) umma_bf16_pair(acc, ad + 2 * k, bd + 2 * k, idesc, (i | k) ? 1u : 0u);
                        else umma_bf16(acc, ad + 2 * k, bd + 2 * k, idesc, (i | k) ? 1u : 0u);
                    }
                    // the stage is free (in both blocks) once these MMAs have read it
                    if (CTAS == 2) umma_commit_pair(&s.empty[st]);
                    else umma_commit(&s.empty[st]);
                }
                if (!failed) {
                    if (CTAS == 2) umma_commit_pair(&s.acc_full[buf]);
                    else umma_commit(&s.acc_full[buf]);
                }
            }
            if (failed) atomicExch(a.status, 2);
        }
    } else {
        // ---- epilogue: warps 2..5, each owns the 32 lanes (rows) warp % 4 of the accumulator ----
        pdl_wait();                       // what follows reads and writes what earlier kernels wrote
        const int quarter = warp & 3;
        unsigned char *stage = s.stage_out[quarter];
        int j = 0;
        // handing an accumulator back: the issuing block's barrier counts the epilogue warps of the whole pair
        auto release_accumulator = [&](int buf) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2) mbar_arrive_cluster(cluster_addr(&s.acc_empty[buf], 0));
                else mbar_arrive(&s.acc_empty[buf]);
            }
        };
        for (int tile = worker; tile < num_tiles; tile += workers, ++j) {
            int tm, tn;
            tile_coords(tile / ksplit, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * TILE_M + rank * TG_BM, n0 = tn * OUT_COLS;
            const int buf = j & 1;
            if (!mbar_wait(&s.acc_full[buf], (j >> 1) & 1)) { failed = 3; if (lane == 0) atomicExch(a.status, 3); break; }
            tc_fence_after();
            const unsigned acc = tmem + buf * BN + ((unsigned)(quarter * 32) << 16);
            const int row0 = m0 + quarter * 32, row = row0 + lane;
            if (EPI == EPI_QKV) {
                // thread = row: its position picks the angles and the cache slot; a head's two halves
                // are read from tensor memory 32 pairs at a time, rotated and stored 64 bytes at a time
                const QkvDest &d = a.qkv;
                const int half = d.dh / 2;
                int pos = 0;
                size_t slot = 0;
                if (row < a.M) {
                    pos = d.positions[row];
                    const int page = d.block_table[(size_t)d.row_req[row] * d.max_blocks + pos / d.page_size];
                    slot = ((size_t)page * d.nkvh * d.page_size + (pos % d.page_size)) * d.dh;
                }
                const float *cs = d.cos_table ? d.cos_table + (size_t)pos * half : nullptr;
                const float *sn = d.sin_table ? d.sin_table + (size_t)pos * half : nullptr;
                // this row's angles for 32 pairs; with heads of 64 they are the same for every head of the tile
                float cr[32], sr[32];
                auto load_angles = [&](int part) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cs + part + i));
                        const float4 s4 = __ldg(reinterpret_cast<const float4 *>(sn + part + i));
                        cr[i] = c4.x; cr[i + 1] = c4.y; cr[i + 2] = c4.z; cr[i + 3] = c4.w;
                        sr[i] = s4.x; sr[i + 1] = s4.y; sr[i + 2] = s4.z; sr[i + 3] = s4.w;
                    }
                };
                if (cs != nullptr && half == 32) load_angles(0);
#pragma unroll 1
                for (int c0 = 0; c0 < OUT_COLS; c0 += d.dh) {
                    if (n0 + c0 >= a.N) break;                             // warp-uniform
                    const int h = (n0 + c0) / d.dh;
                    __nv_bfloat16 *dst;
                    if (h < d.nh) dst = d.q_out + ((size_t)row * d.nh + h) * d.dh;
                    else if (h < d.nh + d.nkvh) dst = d.k_pages + slot + (size_t)(h - d.nh) * d.page_size * d.dh;
                    else dst = d.v_pages + slot + (size_t)(h - d.nh - d.nkvh) * d.page_size * d.dh;
                    const bool rotated = cs != nullptr && h < d.nh + d.nkvh;
#pragma unroll 1
                    for (int part = 0; part < half; part += 32) {
                        unsigned x0[32], x1[32];
                        tmem_ld32(acc + c0 + part, x0);
                        tmem_ld32(acc + c0 + half + part, x1);
                        if (rotated && half != 32) load_angles(part);
                        if (row < a.M) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                unsigned w0[4], w1[4];
#pragma unroll
                                for (int e = 0; e < 8; e += 2) {
                                    float y0[2], y1[2];
#pragma unroll
                                    for (int z = 0; z < 2; ++z) {
                                        const float u = __uint_as_float(x0[i + e + z]), v = __uint_as_float(x1[i + e + z]);
                                        y0[z] = rotated ? u * cr[i + e + z] - v * sr[i + e + z] : u;
                                        y1[z] = rotated ? u * sr[i + e + z] + v * cr[i + e + z] : v;
                                    }
                                    const __nv_bfloat162 b0 = __floats2bfloat162_rn(y0[0], y0[1]);
                                    const __nv_bfloat162 b1 = __floats2bfloat162_rn(y1[0], y1[1]);
                                    w0[e / 2] = *reinterpret_cast<const unsigned *>(&b0);
                                    w1[e / 2] = *reinterpret_cast<const unsigned *>(&b1);
                                }
                                *reinterpret_cast<uint4 *>(dst + part + i) = make_uint4(w0[0], w0[1], w0[2], w0[3]);
                                *reinterpret_cast<uint4 *>(dst + half + part + i) = make_uint4(w1[0], w1[1], w1[2], w1[3]);
                            }
                        }
                    }
                }
                release_accumulator(buf);
                continue;
            }
            // columns per pass: a staging row is 128 bytes = 32 floats or 64 bfloat16
            constexpr int PASS = (EPI == EPI_F32 || EPI == EPI_RESIDUAL) ? 32 : 64;
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += PASS) {
                const int col = n0 + c0;
                if (col >= a.N) break;                                     // warp-uniform
                if (!a.direct) {
                    if (lane == 0) bulk_wait_read();                       // the staging tile's last store has read it
                    __syncwarp();
                }
#pragma unroll
                for (int half = 0; half < PASS / 32; ++half) {
                    unsigned v[32];
                    tmem_ld32(acc + c0 + half * 32, v);
                    float f[32];
                    if (EPI == EPI_SWIGLU) {
                        unsigned u[32];
                        tmem_ld32(acc + BN / 2 + c0 + half * 32, u);
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float g = __uint_as_float(v[i]);
                            f[i] = g / (1.f + expf(-g)) * __uint_as_float(u[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]) * (EPI == EPI_RESIDUAL ? a.scale : 1.f);
                    }
                    if (a.direct) {
                        // rows of the output are not 16-byte aligned: plain guarded stores
                        if (row < a.M) {
                            for (int i = 0; i < 32; ++i) {
                                const int c = col + half * 32 + i;
                                if (c >= a.N) break;
                                if (EPI == EPI_F32) reinterpret_cast<float *>(a.out)[(size_t)row * a.ldo + c] = f[i];
                                else if (EPI == EPI_RESIDUAL) reinterpret_cast<float *>(a.out)[(size_t)row * a.ldo + c] += f[i];
                                else reinterpret_cast<__nv_bfloat16 *>(a.out)[(size_t)row * a.ldo + c] = __float2bfloat16_rn(f[i]);
                            }
                        }
                    } else if (PASS == 32) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            stage_write(stage, lane, i, make_uint4(__float_as_uint(f[4 * i]), __float_as_uint(f[4 * i + 1]),
                                                                   __float_as_uint(f[4 * i + 2]), __float_as_uint(f[4 * i + 3])));
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(f[8 * i], f[8 * i + 1]), p1 = __floats2bfloat162_rn(f[8 * i + 2], f[8 * i + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(f[8 * i + 4], f[8 * i + 5]), p3 = __floats2bfloat162_rn(f[8 * i + 6], f[8 * i + 7]);
                            stage_write(stage, lane, half * 4 + i,
                                        make_uint4(*reinterpret_cast<unsigned *>(&p0), *reinterpret_cast<unsigned *>(&p1),
                                                   *reinterpret_cast<unsigned *>(&p2), *reinterpret_cast<unsigned *>(&p3)));
                        }
                    }
                }
                if (!a.direct) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0 && row0 < a.M) {
                        // TMA clips what lies beyond the matrix; the box starts inside it, never at a negative coordinate
                        if (EPI == EPI_RESIDUAL) tma_reduce_add_2d(&map_out, stage, col, row0);
                        else tma_store_2d(&map_out, stage, col, row0);
                        bulk_commit();
                    }
                }
            }
            // this warp has read all it needs of the accumulator: hand the buffer back to the MMA warp
            release_accumulator(buf);
        }
        if (lane == 0) bulk_wait_all();
    }
    // A role that gave up leaves copies or MMAs in flight: give them a bounded time to land before
    // the block's shared and tensor memory are released.
    if (failed && lane == 0) {
        for (int st = 0; st < STAGES; ++st) mbar_wait(&s.full[st], 0);
    }
    tc_fence_before();
    __syncthreads();
    // of a pair, neither block leaves (or frees tensor memory) while the other may still read its shared
    // memory, write its accumulators or arrive on its barriers
    if (CTAS == 2) cluster_sync();
    tc_fence_after();
    if (warp == 1) {
        if (CTAS == 2) tmem_dealloc_pair(tmem, 2 * BN);
        else tmem_dealloc(tmem, 2 * BN);
    }
}

template <int BN, int EPI>
static int launch_tg(const CUtensorMap &ma, const CUtensorMap &mw, const CUtensorMap &mo, const TgArgs &a, int sms,
                     cudaStream_t stream) {
    const size_t smem = sizeof(TgSmem<BN, 1>) + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "gemm_tcgen05: %s", cudaGetErrorString(e));
    const int out_cols = EPI == EPI_SWIGLU ? BN / 2 : BN;
    const int tiles = ((a.N + out_cols - 1) / out_cols) * ((a.M + TG_BM - 1) / TG_BM) * (a.ksplit > 1 ? a.ksplit : 1);
    jk_launch(gemm_tcgen05_kernel<BN, EPI, 1>, dim3(tiles < sms ? tiles : sms), dim3(TG_THREADS), smem, stream, ma, mw, mo, a);
    JK_CHECK_LAUNCH("gemm_tcgen05");
    return JK_OK;
}

// The same product by pairs of blocks (clusters of two) on tiles of 256 x 256: `mw` has boxes of 128 rows.
template <int EPI>
static int launch_tg_pair(const CUtensorMap &ma, const CUtensorMap &mw, const CUtensorMap &mo, const TgArgs &a, int sms,
                          cudaStream_t stream) {
    auto kernel = gemm_tcgen05_kernel<256, EPI, 2>;
    const size_t smem = sizeof(TgSmem<256, 2>) + 1024;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "gemm_tcgen05: %s", cudaGetErrorString(e));
    const int out_cols = EPI == EPI_SWIGLU ? 128 : 256;
    const int tiles = ((a.N + out_cols - 1) / out_cols) * ((a.M + 2 * TG_BM - 1) / (2 * TG_BM)) * (a.ksplit > 1 ? a.ksplit : 1);
    // as many pairs as the device holds at once (each block takes an SM's whole shared memory)
    static int resident = 0;
    if (resident == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (sms / 2)); cfg.blockDim = dim3(TG_THREADS); cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = sms / 2;
        }
        resident = n < sms / 2 ? n : sms / 2;
    }
    const int pairs = tiles < resident ? tiles : resident;
    e = jk_launch_clusters(kernel, 2, dim3(2 * pairs), dim3(TG_THREADS), smem, stream, ma, mw, mo, a);
    if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "gemm_tcgen05 (pairs): %s", cudaGetErrorString(e));
    return JK_OK;
}

// Pairs of blocks take a product whose tiles of 256 x 256 make more than one wave over the SM pairs (each SM then
// reads half of B's bytes per flop from its shared memory, which is what bounds single blocks); a product of
// one wave is no faster that way, and single blocks spread it over more SMs.  JK_GEMM_PAIR=0 keeps every
// product on single blocks, JK_GEMM_PAIR=2 sends every product of more than 128 rows to pairs
// (jk_gemm_tcgen05_set_pairs does the same at run time, for tests).
static int g_pair_mode = -1;      // -1: not read yet
JK_EXPORT int jk_gemm_tcgen05_set_pairs(int mode) {      // 0, 1 (the rule above) or 2; returns the mode before
    const int before = g_pair_mode;
    g_pair_mode = mode < 0 ? 0 : mode > 2 ? 2 : mode;
    return before;
}
static int pair_mode() {
    if (g_pair_mode < 0) {
        const char *v = getenv("JK_GEMM_PAIR");
        g_pair_mode = v && v[0] >= '0' && v[0] <= '2' ? v[0] - '0' : 1;
    }
    return g_pair_mode;
}
static bool takes_pairs(int M, int N, int out_cols, int sms) {
    const int mode = pair_mode();
    if (mode == 0 || M <= TG_BM) return false;
    if (mode == 2) return true;
    // rows that fill tiles of 256 badly (640 = two and a half) leave a pair's second block idle on the last row of
    // tiles: single blocks then (measured at 640 rows of the 2B shape: 177 against 166 us a layer)
    const int padded = (M + 2 * TG_BM - 1) / (2 * TG_BM) * (2 * TG_BM);
    if ((padded - M) * 8 > M) return false;
    const long long tiles = (long long)((N + out_cols - 1) / out_cols) * (padded / (2 * TG_BM));
    return tiles > sms / 2;
}

// The fused [q | k | v] projection with rotation and cache write in its epilogue.  Head sizes 64 and 128
// (a 256-column tile holds whole heads, a head's halves are multiples of 32 columns).
JK_EXPORT int jk_gemm_tcgen05_qkv_supports(int dh) { return dh == 64 || dh == 128; }

JK_EXPORT int jk_gemm_tcgen05_qkv(const void *act, const void *w, int M, int K, void *q_out, void *k_pages, void *v_pages,
                                  const float *cos_table, const float *sin_table, const int *positions,
                                  const int *row_req, const int *block_table, int max_blocks, int page_size, int nh,
                                  int nkvh, int dh, int *status, int sms, cudaStream_t stream) {
    const int N = (nh + 2 * nkvh) * dh;
    JK_REQUIRE(jk_gemm_tcgen05_qkv_supports(dh), "gemm_tcgen05_qkv: head size %d (64 and 128 are built)", dh);
    JK_REQUIRE(M >= 1 && K >= 8 && K % 8 == 0 && nh >= 1 && nkvh >= 1, "gemm_tcgen05_qkv: M %d K %d heads %d/%d", M, K, nh, nkvh);
    JK_REQUIRE(status != nullptr && q_out && k_pages && v_pages && positions && row_req && block_table && max_blocks > 0 && page_size > 0,
               "gemm_tcgen05_qkv: a destination or index array is missing");
    JK_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "gemm_tcgen05_qkv: cos and sin tables come together");
    JK_REQUIRE((reinterpret_cast<uintptr_t>(act) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(q_out) & 15) == 0 && (reinterpret_cast<uintptr_t>(k_pages) & 15) == 0 &&
               (reinterpret_cast<uintptr_t>(v_pages) & 15) == 0, "gemm_tcgen05_qkv: operands must be 16-byte aligned");
    if (sms <= 0) sms = 148;
    CUtensorMap ma, mw;
    if (int rc = tensor_map_2d(act, M, K, K, TG_BM, TG_BK, 2, &ma)) return rc;
    const bool pair = takes_pairs(M, N, 256, sms);
    if (int rc = tensor_map_2d(w, N, K, K, pair ? 128 : 256, TG_BK, 2, &mw)) return rc;
    TgArgs a{nullptr, M, N, K, N, 1.f, status, 0, 0,
             QkvDest{(__nv_bfloat16 *)q_out, (__nv_bfloat16 *)k_pages, (__nv_bfloat16 *)v_pages, cos_table, sin_table,
                     positions, row_req, block_table, nh, nkvh, dh, page_size, max_blocks}};
    if (pair) return launch_tg_pair<EPI_QKV>(ma, mw, ma, a, sms, stream);
    return launch_tg<256, EPI_QKV>(ma, mw, ma, a, sms, stream);
}

JK_EXPORT int jk_gemm_tcgen05_supports(int M, int N, int K) { return M >= 1 && N >= 1 && K >= 8 && K % 8 == 0; }

JK_EXPORT int jk_gemm_tcgen05(const void *act, const void *w, void *out, int M, int N, int K, int ldo, int epilogue,
                              float scale, int *status, int sms, cudaStream_t stream) {
    JK_REQUIRE(jk_gemm_tcgen05_supports(M, N, K), "gemm_tcgen05: M %d N %d K %d (K must be a multiple of 8)", M, N, K);
    JK_REQUIRE(epilogue >= EPI_F32 && epilogue <= EPI_SWIGLU, "gemm_tcgen05: epilogue %d", epilogue);
    JK_REQUIRE(ldo >= N && status != nullptr, "gemm_tcgen05: output stride %d < N %d, or no status word", ldo, N);
    JK_REQUIRE((reinterpret_cast<uintptr_t>(act) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "gemm_tcgen05: operands must be 16-byte aligned");
    if (sms <= 0) sms = 148;
    const int w_rows = epilogue == EPI_SWIGLU ? 2 * N : N;
    const int out_bytes = (epilogue == EPI_F32 || epilogue == EPI_RESIDUAL) ? 4 : 2;
    CUtensorMap ma, mw, mo;
    if (int rc = tensor_map_2d(act, M, K, K, TG_BM, TG_BK, 2, &ma)) return rc;
    TgArgs a{out, M, N, K, ldo, scale, status, 0, 0, QkvDest{}};
    // the output goes out by TMA when its rows are 16-byte aligned, else straight from registers
    a.direct = ((size_t)ldo * out_bytes) % 16 != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0;
    if (a.direct) mo = ma;
    else if (int rc = tensor_map_2d(out, M, N, ldo, 32, 128 / out_bytes, out_bytes, &mo)) return rc;
    bool pair = takes_pairs(M, N, epilogue == EPI_SWIGLU ? 128 : 256, sms);
    if (epilogue == EPI_RESIDUAL && !a.direct) {
        // A product that adds itself into its output may cut K: the units of a tile add their partial products by the
        // same TMA reduce.  Up to three cuts (JK_GEMM_KSPLIT moves the limit), chosen so that the units fill their waves,
        // as long as a unit keeps 32 steps of K.  Measured at 768 x 4096 x 16384: 164 -> 112 us; at 1536 rows 168 -> 150 us.
        // Four cuts of 128 tiles on 74 pairs of SMs look better on paper (seven waves of quarters against two of whole
        // tiles) and are slower (211 against 190 us): a second wave that is three quarters empty runs faster than a full one.
        // Shorter units do not help a single wave either.  At 2048 x 2304 x 2304 (144 tiles for 148 SMs, 36 steps each):
        // whole tiles 20.8 us (the library's product of this shape: 19.5), two cuts of 18 steps 23.0, pairs of blocks 21.7,
        // tiles of 128 columns 30.2.  Two cuts of 18 steps do help 512 rows of that shape (16.0 -> 11.7 us) and then cost
        // 512 x 2304 x 5760 as much (20.8 -> 24.0), so the limit of 32 steps stays.
        const int nk = (K + TG_BK - 1) / TG_BK;
        const bool pairs_possible = pair_mode() != 0 && M > TG_BM;
        double best = 1e30;
        int best_s = 1;
        bool best_pair = pair;
        for (int use_pair = 0; use_pair <= (pairs_possible ? 1 : 0); ++use_pair) {
            const long long tiles = use_pair ? (long long)((N + 255) / 256) * ((M + 255) / 256) : (long long)((N + 255) / 256) * ((M + 127) / 128);
            const int workers = use_pair ? sms / 2 : sms;
            static const int max_cuts = [] { const char *v = getenv("JK_GEMM_KSPLIT"); return v ? atoi(v) : 3; }();
            for (int sp = 1; sp <= (max_cuts < 1 ? 1 : max_cuts); ++sp) {
                if (sp > 1 && nk / sp < 32) break;
                const long long waves = (tiles * sp + workers - 1) / workers;
                // time in tiles of 128 x 256 per SM; pairs do their share about 7 % faster once there is more than one
                // wave of them (a single wave is no faster, measured); a cut costs a little
                const double cost = (double)waves / sp * (use_pair ? (waves > 1 ? 0.93 : 1.03) : 1.0) * (1.0 + 0.03 * (sp - 1));
                if (cost < best - 1e-9) { best = cost; best_s = sp; best_pair = use_pair != 0; }
            }
        }
        if (pair_mode() == 2 && pairs_possible) best_pair = true;      // forced by a test
        pair = best_pair;
        a.ksplit = best_s;
        const int nk_unit = (nk + a.ksplit - 1) / a.ksplit;
        a.ksplit = (nk + nk_unit - 1) / nk_unit;                          // no unit without a step
    }
    if (epilogue == EPI_SWIGLU) {
        if (int rc = tensor_map_2d(w, w_rows, K, K, 128, TG_BK, 2, &mw)) return rc;
        if (pair) return launch_tg_pair<EPI_SWIGLU>(ma, mw, mo, a, sms, stream);
        return launch_tg<256, EPI_SWIGLU>(ma, mw, mo, a, sms, stream);
    }
    // a narrower tile when wide tiles would leave most SMs without one
    const int tiles_m = (M + TG_BM - 1) / TG_BM;
    const bool narrow = N <= 128 || tiles_m * ((N + 255) / 256) < sms * 3 / 4;
    if (pair && !narrow) {
        if (int rc = tensor_map_2d(w, w_rows, K, K, 128, TG_BK, 2, &mw)) return rc;
        switch (epilogue) {
            case EPI_F32: return launch_tg_pair<EPI_F32>(ma, mw, mo, a, sms, stream);
            case EPI_BF16: return launch_tg_pair<EPI_BF16>(ma, mw, mo, a, sms, stream);
            default: return launch_tg_pair<EPI_RESIDUAL>(ma, mw, mo, a, sms, stream);
        }
    }
    if (int rc = tensor_map_2d(w, w_rows, K, K, narrow ? 128 : 256, TG_BK, 2, &mw)) return rc;
#define TG_DISPATCH(BN_)                                                                 \
    switch (epilogue) {                                                                  \
        case EPI_F32: return launch_tg<BN_, EPI_F32>(ma, mw, mo, a, sms, stream);         \
        case EPI_BF16: return launch_tg<BN_, EPI_BF16>(ma, mw, mo, a, sms, stream);       \
        default: return launch_tg<BN_, EPI_RESIDUAL>(ma, mw, mo, a, sms, stream);         \
    }
    if (narrow) { TG_DISPATCH(128) }
    TG_DISPATCH(256)
#undef TG_DISPATCH
}
