// The product of 1 to 128 activation rows on the tcgen05 tensor cores with the weights on the MMA's M side.
// (Part of the module gemm_tcgen05; the tiled kernel for many rows is in gemm_tcgen05.cu.)
#include "tcgen05.cuh"

// ---- products of few rows (decode batches, short portions): weights on the MMA's M side -------------------
//
// With 17 to 128 activation rows the product is bound by reading W once.  A block takes 128 rows of W (for SwiGLU
// 64 gate rows and the 64 up rows that belong to them) and a range of K, and computes D^T[n, m] = W[n, :] . A[m, :]:
// W tiles are the MMA's A operand (M = 128), the activation rows (padded to a multiple of 32, zero-filled by TMA)
// its B operand (N = rows), so no tensor-core lane is spent on padding rows of a 128-row activation tile.  The first
// tiles of W are requested before the wait on the preceding kernel (weights are never written by a step).  A thread of
// the epilogue holds one output feature n and all rows m: for each m a warp writes 32 consecutive features.
//   SK_STORE   out[m, n]  = acc                      float32 (one block per 128 features, all of K)
//   SK_ADD     out[m, n] += scale * acc              float32 by red.global.add: blocks split K among themselves and
//                                                    add their partial sums (into the residual stream, or into an
//                                                    output that the caller zeroed)
//   SK_SWIGLU  out[m, n]  = silu(gate) * up          bfloat16; the up half of the lanes hands its values to the gate
//                                                    half through shared memory
enum { SK_STORE = 0, SK_ADD = 1, SK_SWIGLU = 2 };
constexpr int SK_MAX_STAGES = 8;

struct SkArgs {
    void *out;
    int M, N, K, ldo;
    float scale;
    int *status;
    int mpad;           // activation rows padded to a multiple of 32 (the MMA's N)
    int stages;         // depth of the ring
    int ksteps;         // 64-wide steps of K per block
};

template <int EPI>
__global__ void __launch_bounds__(TG_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, SkArgs a) {
    extern __shared__ unsigned char sk_raw[];
    unsigned char *ring = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(sk_raw) + 1023) & ~uintptr_t(1023));
    constexpr unsigned W_BYTES = 128 * TG_BK * sizeof(__nv_bfloat16);       // 16 KB
    constexpr int OUT_ROWS = EPI == SK_SWIGLU ? 64 : 128;                   // output features per block
    const unsigned act_bytes = (unsigned)a.mpad * TG_BK * sizeof(__nv_bfloat16);
    const unsigned stage_bytes = W_BYTES + act_bytes;                       // a multiple of 1024: tiles stay aligned
    struct Bars { unsigned long long full[SK_MAX_STAGES], empty[SK_MAX_STAGES], acc_full; unsigned tmem_base; };
    Bars &b = *reinterpret_cast<Bars *>(ring + (size_t)a.stages * stage_bytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * OUT_ROWS;
    const int nk = (a.K + TG_BK - 1) / TG_BK;
    const int ks0 = blockIdx.y * a.ksteps;
    const int steps = min(a.ksteps, nk - ks0);                              // >= 1 by the host's choice of the grid
    unsigned tmem_cols = 32;
    while ((int)tmem_cols < a.mpad) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < a.stages; ++i) { mbar_init(&b.full[i], 1); mbar_init(&b.empty[i], 1); }
        mbar_init(&b.acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&b.tmem_base, tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = b.tmem_base;
    int failed = 0;
    pdl_trigger();

    auto w_tile = [&](int st) { return ring + (size_t)st * stage_bytes; };
    auto a_tile = [&](int st) { return ring + (size_t)st * stage_bytes + W_BYTES; };
    if (warp == 0) {
        if (lane == 0) {
            auto load_w = [&](int i) {
                const int st = i % a.stages, kc = (ks0 + i) * TG_BK;
                mbar_expect_tx(&b.full[st], stage_bytes);
                if (EPI == SK_SWIGLU) {
                    tma_load_2d(w_tile(st), &map_w, &b.full[st], kc, n0);
                    tma_load_2d(w_tile(st) + W_BYTES / 2, &map_w, &b.full[st], kc, a.N + n0);
                } else {
                    tma_load_2d(w_tile(st), &map_w, &b.full[st], kc, n0);
                }
            };
            const int ahead = min(steps, a.stages);
            for (int i = 0; i < ahead; ++i) load_w(i);                     // weights: nothing to wait for
            pdl_wait();                                                    // the activations come from the kernel before
            for (int i = 0; i < ahead; ++i) tma_load_2d(a_tile(i), &map_a, &b.full[i], (ks0 + i) * TG_BK, 0);
            for (int i = ahead; i < steps; ++i) {
                const int st = i % a.stages;
                if (!mbar_wait(&b.empty[st], ((i / a.stages) - 1) & 1)) { failed = 1; break; }
                load_w(i);
                tma_load_2d(a_tile(st), &map_a, &b.full[st], (ks0 + i) * TG_BK, 0);
            }
            if (failed) atomicExch(a.status, 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = instr_desc_bf16(a.mpad);
            for (int i = 0; i < steps; ++i) {
                const int st = i % a.stages;
                if (!mbar_wait(&b.full[st], (i / a.stages) & 1)) { failed = 2; break; }
                tc_fence_after();
                const unsigned long long wd = smem_desc_sw128(w_tile(st)), ad = smem_desc_sw128(a_tile(st));
#pragma unroll
                for (int k = 0; k < TG_BK / 16; ++k) umma_bf16(tmem, wd + 2 * k, ad + 2 * k, idesc, (i | k) ? 1u : 0u);
                umma_commit(&b.empty[st]);
            }
            if (!failed) umma_commit(&b.acc_full);
            else atomicExch(a.status, 2);
        }
    } else {
        const int quarter = warp & 3;                                      // lanes (features) quarter * 32 ... of the accumulator
        pdl_wait();                                                        // before this block's first global write
        if (!mbar_wait(&b.acc_full, 0)) {
            failed = 3;
            if (lane == 0) atomicExch(a.status, 3);
        }
        tc_fence_after();
        const unsigned acc = tmem + ((unsigned)(quarter * 32) << 16);
        if (EPI == SK_SWIGLU) {
            // lanes 0..63 hold gate rows, lanes 64..127 the up rows of the same features; the ring is free
            // (every MMA that read it has completed) and carries the up values over: [row m][feature 0..63]
            float *xch = reinterpret_cast<float *>(ring);
            if (quarter >= 2 && !failed) {
                for (int c0 = 0; c0 < a.mpad; c0 += 32) {
                    unsigned v[32];
                    tmem_ld32(acc + c0, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) xch[(c0 + i) * 64 + (quarter - 2) * 32 + lane] = __uint_as_float(v[i]);
                }
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");             // the four epilogue warps, whatever their wait said
            if (quarter < 2 && !failed) {
                const int n = n0 + quarter * 32 + lane;
                __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(a.out);
                for (int c0 = 0; c0 < a.mpad; c0 += 32) {
                    unsigned v[32];
                    tmem_ld32(acc + c0, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int m = c0 + i;
                        const float g = __uint_as_float(v[i]), u = xch[m * 64 + quarter * 32 + lane];
                        if (m < a.M && n < a.N) out[(size_t)m * a.ldo + n] = __float2bfloat16_rn(g / (1.f + expf(-g)) * u);
                    }
                }
            }
        } else if (!failed) {
            const int n = n0 + quarter * 32 + lane;
            float *out = reinterpret_cast<float *>(a.out);
            for (int c0 = 0; c0 < a.mpad; c0 += 32) {
                unsigned v[32];
                tmem_ld32(acc + c0, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int m = c0 + i;
                    if (m < a.M && n < a.N) {
                        if (EPI == SK_ADD) atomicAdd(out + (size_t)m * a.ldo + n, a.scale * __uint_as_float(v[i]));
                        else out[(size_t)m * a.ldo + n] = __uint_as_float(v[i]);
                    }
                }
            }
        }
    }
    if (failed && lane == 0) {
        for (int st = 0; st < a.stages; ++st) mbar_wait(&b.full[st], 0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem, tmem_cols);
}

// 17 to 128 rows (fewer are taken too: the weight-streaming kernels of linear_small.cu are the better home for up to
// 16 rows unless K is beyond what they hold in shared memory).
JK_EXPORT int jk_gemm_skinny_supports(int M, int N, int K) { return M >= 1 && M <= 128 && N >= 1 && K >= 8 && K % 8 == 0; }

// epilogue: EPI_F32 (out = product, float32), EPI_RESIDUAL (out += scale * product, float32), EPI_SWIGLU (w is
// [2N, K]; out = silu(gate) * up, bfloat16).
JK_EXPORT int jk_gemm_skinny(const void *act, const void *w, void *out, int M, int N, int K, int ldo, int epilogue, float scale,
                             int *status, int sms, cudaStream_t stream) {
    JK_REQUIRE(jk_gemm_skinny_supports(M, N, K), "gemm_skinny: M %d N %d K %d (1 to 128 rows, K a multiple of 8)", M, N, K);
    JK_REQUIRE(epilogue == EPI_F32 || epilogue == EPI_RESIDUAL || epilogue == EPI_SWIGLU, "gemm_skinny: epilogue %d", epilogue);
    JK_REQUIRE(ldo >= N && status != nullptr && out != nullptr, "gemm_skinny: output stride %d < N %d, or a pointer is missing", ldo, N);
    JK_REQUIRE((reinterpret_cast<uintptr_t>(act) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "gemm_skinny: operands must be 16-byte aligned");
    if (sms <= 0) sms = 148;
    SkArgs a{out, M, N, K, ldo, scale, status, (M + 31) / 32 * 32, 0, 0};
    const int out_rows = epilogue == EPI_SWIGLU ? 64 : 128;
    const int tiles = (N + out_rows - 1) / out_rows;
    const int nk = (K + TG_BK - 1) / TG_BK;
    // two blocks fit an SM; K is split until the blocks fill the SMs twice over, as long as each keeps 8 steps
    int splits = 1;
    if (epilogue != EPI_SWIGLU) {
        splits = 2 * sms / tiles;
        if (splits > nk / 8) splits = nk / 8;
        if (splits < 1) splits = 1;
    }
    a.ksteps = (nk + splits - 1) / splits;
    splits = (nk + a.ksteps - 1) / a.ksteps;                              // no block without a step
    const size_t stage = 128 * TG_BK * 2 + (size_t)a.mpad * TG_BK * 2;
    a.stages = (int)((100 * 1024) / stage);                               // two blocks' rings per SM
    if (a.stages > SK_MAX_STAGES) a.stages = SK_MAX_STAGES;
    if (a.stages > a.ksteps) a.stages = a.ksteps < 2 ? 2 : a.ksteps;
    const size_t smem = a.stages * stage + 256 + 1024;
    CUtensorMap mw, ma;
    if (int rc = tensor_map_2d(w, epilogue == EPI_SWIGLU ? 2 * N : N, K, K, out_rows, TG_BK, 2, &mw)) return rc;
    if (int rc = tensor_map_2d(act, M, K, K, a.mpad, TG_BK, 2, &ma)) return rc;
    int kind = epilogue == EPI_SWIGLU ? SK_SWIGLU : epilogue == EPI_RESIDUAL ? SK_ADD : SK_STORE;
    if (kind == SK_STORE && splits > 1) {
        // partial sums of the blocks that share an output tile are added into a zeroed output
        const cudaError_t e = cudaMemset2DAsync(out, (size_t)ldo * 4, 0, (size_t)N * 4, M, stream);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "gemm_skinny: %s", cudaGetErrorString(e));
        kind = SK_ADD;
        a.scale = 1.f;
    }
    auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024 + 2048);
        if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "gemm_skinny: %s", cudaGetErrorString(e));
        jk_launch(kernel, dim3(tiles, splits), dim3(TG_THREADS), smem, stream, mw, ma, a);
        JK_CHECK_LAUNCH("gemm_skinny");
        return JK_OK;
    };
    if (kind == SK_SWIGLU) return launch(gemm_skinny_kernel<SK_SWIGLU>);
    if (kind == SK_ADD) return launch(gemm_skinny_kernel<SK_ADD>);
    return launch(gemm_skinny_kernel<SK_STORE>);
}

// K must keep rows 16-byte aligned for TMA; everything else is free.
