// Prefill attention on the 5th-generation tensor cores: causal softmax attention of 128-row query
// tiles over the paged key/value cache, both products by tcgen05.mma with accumulators in tensor
// memory, operands by TMA.  Same contract as the mma.sync kernel in attention.cu (which stays for
// head sizes and page sizes this one is not built for).
//
// One block = (128 query rows of one request, one query head); ten warps:
//   warp 0     TMA: the query tile once, then for every tile of 128 keys the pages that hold it
//              (block table -> page -> one box of page_size rows per page; lane = page), keys and
//              values into two stages each;
//   warp 1     issues the products:  S = Q K^T  (M 128, N 128, K = head size) into tensor memory,
//              and  O_h += P_h V_h  for the two halves h of the tile's keys (M 128, N = head size,
//              K = 64 keys each); K is a K-major operand, V an MN-major one (rows of the cache are
//              keys, which is the K dimension of P V), both straight from the 128-byte-swizzled tiles
//              that TMA wrote;
//   warps 2-9  softmax: thread = (query row, half of the tile's keys); warps w and w + 4 share the rows
//              of one lane quarter of tensor memory.  A thread reads its 64 scores, applies scale,
//              causal mask and window, keeps a reference maximum and the running sum in float32 and
//              writes P as bfloat16 into shared memory in the swizzled K-major layout the second
//              product reads.  The reference is raised only when the maximum exceeds it by more than
//              2^8 (then the accumulator and the sum are rescaled); until then probabilities are at most
//              256, exact in float32 and safe in bfloat16, and the final division by the sum makes the
//              choice of reference immaterial.  Each half has its own reference, sum and accumulator
//              (O_0 and O_1 in tensor memory), so the halves exchange nothing until the epilogue, which
//              brings them to a common reference:  O = (w_0 O_0 + w_1 O_1) / (w_0 l_0 + w_1 l_1).
//              The scores' place in tensor memory is released as soon as a warp holds its part in
//              registers, so the next tile's first product runs under this tile's softmax.
// Two such blocks fit an SM (head size 64), so one block's softmax overlaps the other's products.
// Measured with cycle counters inside the kernel (heads of 64): a product instruction of M 128 takes about 65 cycles
// to issue and run whether N is 128 or 64, so the eight products of P V cost twice the four of Q K^T; a key tile costs
// a softmax warp about 1,200 cycles of waits, loads and arrivals that nothing of its own overlaps, beside its
// arithmetic; an SM passes one key tile in about 1,600 cycles whatever the arrangement (blocks that stay and share
// the units out, one thread per row with P through tensor memory as the A operand: both built, equal, not kept).
// Every wait is bounded; a wait that runs out records a code in `status` and the block drains and leaves.
// (reference: the per-request loop of two batched products and a causal softmax over a materialised
// score buffer, src/models/jiuge/jiuge.cpp:206-233.)
#include "common.cuh"

#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

JK_DEFINE_ERROR_BUFFER(jk_attention_tcgen05)

constexpr int AT_BM = 128, AT_BN = 128, AT_HALF = 64, AT_THREADS = 320;
constexpr unsigned AT_SPIN_LIMIT = 1u << 20;
constexpr float AT_RESCALE_THRESHOLD = 8.f;      // in log2 units
// Of every 8 pairs of probabilities, this many are computed by a polynomial on the FMA pipes and the
// rest by the special-function unit (16 results a cycle and SM).  Measured at 36 heads of 64, 2,048 and 8,192 tokens:
// 0 of 8: 43.8 and 451 us, 1: 44.1 and 446, 2: 41.3 and 418, 3: 43.1 and 439, 4: 44.5 and 461.
constexpr int AT_POLY_OF_8 = 2;

struct AtArgs {
    __nv_bfloat16 *out;       // [T, nh, dh]
    const int *tiles;         // [ntiles][2]: batch entry, first row of the tile (row index in the step); most keys first
    const int *req_start;     // [nreq + 1]
    const int *req_pos;       // [nreq]
    const int *block_table;   // [nreq, max_blocks]
    int *status;
    int ntiles, nh, nkvh, page_size, max_blocks, window;
    float scale_log2;
};

// ---- PTX wrappers (see gemm_tcgen05.cu for the same set) -----------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity) {
    for (unsigned i = 0; i < AT_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void *smem, const CUtensorMap *map, unsigned long long *bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(unsigned *slot, unsigned columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned addr, unsigned columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(addr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// D (tensor memory) (+)= A B, operands by shared-memory descriptors.  Each descriptor comes as two 32-bit
// words: the high word is one constant per operand kind and the low word moves by a small constant from
// product to product, so the thread that issues spends one addition per operand.
__device__ __forceinline__ void umma_bf16_words(unsigned tmem_c, unsigned a_lo, unsigned a_hi, unsigned b_lo, unsigned b_hi,
                                                unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                 "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}\n"
                 ::"r"(tmem_c), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned addr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
// The same load without the wait: several may be in flight before one tmem_wait_ld().
__device__ __forceinline__ void tmem_ld32_issue(unsigned addr, unsigned *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(unsigned addr, const unsigned (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two float32 in one 64-bit register, for the packed arithmetic of sm_100 (one instruction, two results).
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for two x in [-125, 128) without the special-function unit: x = n + f with n the nearest
// integer (taken from the low mantissa bits of x + 1.5 * 2^23) and f in [-0.5, 0.5]; 2^f by a cubic
// (relative error 7.5e-5, far inside what a bfloat16 probability keeps); n goes into the exponent
// by an integer addition.
__device__ __forceinline__ void exp2_poly2(unsigned long long x2, float &e0, float &e1) {
    float x0, x1;
    unpack2(x2, x0, x1);
    const unsigned long long xc = pack2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
    const unsigned long long t = add2(xc, pack2(12582912.f, 12582912.f));
    const unsigned long long n = add2(t, pack2(-12582912.f, -12582912.f));
    const unsigned long long f = fma2(n, pack2(-1.f, -1.f), xc);
    unsigned long long p = fma2(f, pack2(0.055171459913253784f, 0.055171459913253784f), pack2(0.2426108568906784f, 0.2426108568906784f));
    p = fma2(p, f, pack2(0.6932609677314758f, 0.6932609677314758f));
    p = fma2(p, f, pack2(0.9999281167984009f, 0.9999281167984009f));
    float p0, p1, t0, t1;
    unpack2(p, p0, p1);
    unpack2(t, t0, t1);
    e0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(t0) << 23));
    e1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(t1) << 23));
}

// Shared-memory descriptors of the 128-byte-swizzled tiles (built in the issuing thread):
//   K-major operand [rows][64 bf16]: groups of 8 rows are 1024 bytes apart (stride offset), leading offset 1;
//   MN-major operand (the value tile as B of P V): memory rows are keys (the K dimension), 128 bytes =
//   64 elements of the head each; groups of 8 keys are 1024 bytes apart (stride offset), further
//   groups of 64 head elements one whole tile apart (leading offset);
//   version 1, layout type 2 (128-byte swizzle).
// D float32, A and B bfloat16, M = 128; b_mn: B is MN-major.
__host__ __device__ constexpr unsigned instr_desc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) | ((unsigned)(AT_BM >> 4) << 24);
}

template <int DH> struct AtSmem {
    static constexpr int SUB = DH / 64;                       // 64-wide sub-tiles along the head
    __nv_bfloat16 q[SUB][AT_BM * 64];                         // K-major, per sub-tile [128 rows][64]
    __nv_bfloat16 k[2][SUB][AT_BN * 64];                      // two stages
    __nv_bfloat16 v[2][SUB][AT_BN * 64];
    __nv_bfloat16 p[2][AT_BM * 64];                           // [128 rows][128 keys] as two sub-tiles of 64 keys
    unsigned long long q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_free, p_ready, pv_done, met[4];
    unsigned tmem_base;
};

template <int DH>
__global__ void __launch_bounds__(AT_THREADS, DH <= 64 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, AtArgs a) {
    constexpr int SUB = DH / 64;
    constexpr unsigned TMEM_COLS = DH <= 64 ? 256 : 512;      // S: 128 columns; two accumulators of DH columns
    extern __shared__ __align__(1024) unsigned char at_raw[];      // swizzled tiles need 1024-byte alignment
    AtSmem<DH> &s = *reinterpret_cast<AtSmem<DH> *>(at_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (smem_u32(at_raw) & 1023u) {                            // never seen; a wrong result is not an option
        if (threadIdx.x == 0) atomicExch(a.status, 14);
        return;
    }

    // blocks start in the order of the tile list (the caller lists the tiles with the most keys first),
    // all heads of a tile together
    const int tile = blockIdx.y;
    const int h = blockIdx.x;
    const int hk = h / (a.nh / a.nkvh);
    if (threadIdx.x == 0) {
        mbar_init(&s.q_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&s.k_full[i], 1); mbar_init(&s.k_empty[i], 1); mbar_init(&s.v_full[i], 1); mbar_init(&s.v_empty[i], 1); }
        mbar_init(&s.s_full, 1); mbar_init(&s.s_free, 8); mbar_init(&s.p_ready, 8); mbar_init(&s.pv_done, 1);
        for (int i = 0; i < 4; ++i) mbar_init(&s.met[i], 2);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_s = s.tmem_base, tmem_o = s.tmem_base + AT_BN;
    // Only now may the next kernel be scheduled: a later kernel that took tensor memory on this SM and
    // then waited for this grid, while a block of this grid still waited for tensor memory, would never end.
    pdl_trigger();
    pdl_wait();

    const int r = a.tiles[2 * tile];
    const int row0 = a.tiles[2 * tile + 1];
    const int nrows = min(AT_BM, a.req_start[r + 1] - row0);
    const int p0 = a.req_pos[r] + (row0 - a.req_start[r]);    // position of the tile's first row
    const int p_last = p0 + nrows - 1;
    const int lo = (a.window > 0 && p0 - a.window + 1 > 0) ? p0 - a.window + 1 : 0;
    const int kv_first = lo / AT_BN * AT_BN;
    const int n_kv = (p_last - kv_first) / AT_BN + 1;         // key tiles this query tile sees
    const int *bt = a.block_table + (size_t)r * a.max_blocks;
    const int pages_per_tile = AT_BN / a.page_size;
    int failed = 0;

    if (warp == 0) {
        // ---- TMA producer: the whole warp; lane = (page of the tile, 64-wide part of the head) ----
        if (lane == 0) {
            mbar_expect_tx(&s.q_full, AT_BM * DH * 2);
            for (int u = 0; u < SUB; ++u) tma_load_2d(s.q[u], &map_q, &s.q_full, h * DH + u * 64, row0);
        }
        const int boxes = pages_per_tile * SUB;                 // at most 16 pages x 2 parts
        for (int i = 0; i < n_kv && !failed; ++i) {
            const int st = i & 1, kv0 = kv_first + i * AT_BN;
            // this lane's page of the tile, read from the block table once for keys and values;
            // a page beyond what the request holds is never looked at: its keys are masked
            const int pg = lane / SUB, u = lane % SUB;
            const int blk = kv0 / a.page_size + pg;
            const int page = (lane < boxes && blk < a.max_blocks) ? bt[blk] : 0;
            const int grow = (page * a.nkvh + hk) * a.page_size;
            for (int kind = 0; kind < 2; ++kind) {               // 0: keys, 1: values
                unsigned long long *empty = kind ? &s.v_empty[st] : &s.k_empty[st];
                unsigned long long *full = kind ? &s.v_full[st] : &s.k_full[st];
                int ok = 1;
                if (i >= 2) {
                    if (lane == 0) ok = mbar_wait(empty, ((i >> 1) - 1) & 1) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                }
                if (!ok) { failed = 1; break; }
                if (lane == 0) mbar_expect_tx(full, AT_BN * DH * 2);
                __syncwarp();
                if (lane < boxes) {
                    __nv_bfloat16 *dst = (kind ? s.v[st][u] : s.k[st][u]) + pg * a.page_size * 64;
                    tma_load_2d(dst, kind ? &map_v : &map_k, full, u * 64, grow);
                }
            }
        }
        if (failed && lane == 0) atomicExch(a.status, 11);
    } else if (warp == 1) {
        // ---- product issuer ----
        if (lane == 0) {
            constexpr unsigned idesc_qk = instr_desc(AT_BN, false), idesc_pv = instr_desc(DH, true);
            // descriptor words, built once: low = start address and leading offset, high = stride
            // offset 1024, version 1, 128-byte swizzle
            constexpr unsigned desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            auto lo_k = [](const void *tile) { return ((smem_u32(tile) & 0x3FFFFu) >> 4) | (1u << 16); };
            auto lo_mn = [](const void *tile) { return ((smem_u32(tile) & 0x3FFFFu) >> 4) | ((unsigned)((AT_BN * 64 * 2) >> 4) << 16); };
            unsigned q_lo[SUB], k_lo[2][SUB], p_lo[2], v_lo[2];
#pragma unroll
            for (int u = 0; u < SUB; ++u) { q_lo[u] = lo_k(s.q[u]); k_lo[0][u] = lo_k(s.k[0][u]); k_lo[1][u] = lo_k(s.k[1][u]); }
            p_lo[0] = lo_k(s.p[0]); p_lo[1] = lo_k(s.p[1]);
            v_lo[0] = lo_mn(s.v[0][0]); v_lo[1] = lo_mn(s.v[1][0]);
            auto issue_qk = [&](int st) {
#pragma unroll
                for (int u = 0; u < SUB; ++u)
#pragma unroll
                    for (int k = 0; k < 4; ++k)          // 16 of the head's elements per instruction: 32 bytes further
                        umma_bf16_words(tmem_s, q_lo[u] + 2 * k, desc_hi, (st ? k_lo[1][u] : k_lo[0][u]) + 2 * k, desc_hi,
                                        idesc_qk, (u | k) ? 1u : 0u);
            };
            if (!mbar_wait(&s.q_full, 0) || !mbar_wait(&s.k_full[0], 0)) failed = 2;
            if (!failed) {
                tc_fence_after();
                issue_qk(0);
                umma_commit(&s.s_full);
                umma_commit(&s.k_empty[0]);
            }
            for (int i = 0; i < n_kv && !failed; ++i) {
                const int st = i & 1;
                if (i + 1 < n_kv) {
                    // the next scores as soon as the softmax warps hold these in registers
                    const int sn = (i + 1) & 1;
                    if (!mbar_wait(&s.s_free, i & 1) || !mbar_wait(&s.k_full[sn], ((i + 1) >> 1) & 1)) { failed = 2; break; }
                    tc_fence_after();
                    issue_qk(sn);
                    umma_commit(&s.s_full);
                    umma_commit(&s.k_empty[sn]);
                }
                if (!mbar_wait(&s.p_ready, i & 1)) { failed = 2; break; }          // P_i is written
                tc_fence_after();
                if (!mbar_wait(&s.v_full[st], (i >> 1) & 1)) { failed = 2; break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < AT_BN / 16; ++k) {   // 16 keys per instruction
                    // P: 32 bytes further in the row of sub-tile k / 4; V: 16 rows of 128 bytes further.
                    // Keys 0..63 of the tile add to the first accumulator, keys 64..127 to the second.
                    umma_bf16_words(tmem_o + (k / 4) * DH, p_lo[k / 4] + 2 * (k % 4), desc_hi,
                                    (st ? v_lo[1] : v_lo[0]) + ((k * 16 * 128) >> 4), desc_hi, idesc_pv, (i | (k % 4)) ? 1u : 0u);
                }
                umma_commit(&s.pv_done);
                umma_commit(&s.v_empty[st]);
            }
            if (failed) atomicExch(a.status, 12);
        }
    } else {
        // ---- softmax and epilogue: warps 2..9; thread = (row, half of the tile's keys) ----
        // Warps w and w + 4 share the 32 rows of tensor-memory lane quarter w % 4; one takes keys 0..63 of
        // every tile, the other keys 64..127.  Each half has a reference maximum, a sum and an output
        // accumulator of its own, so the two never talk until the end.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;                   // row of the tile
        const int pos = p0 + min(row, nrows - 1);              // rows beyond the request repeat its last row
        const int lo_row = a.window > 0 ? pos - a.window + 1 : 0;
        const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
        const unsigned tmem_sh = tmem_s + lane_addr + half * AT_HALF;     // this thread's scores
        const unsigned tmem_oh = tmem_o + lane_addr + half * DH;          // this half's accumulator
        float m_ref = -INFINITY, l = 0.f;                      // reference maximum (scaled, log2 units) and sum
        bool alive = true;
        for (int i = 0; i < n_kv; ++i) {
            const int kv0 = kv_first + i * AT_BN + half * AT_HALF;        // first key of this thread's part
            if (!__all_sync(0xffffffffu, mbar_wait(&s.s_full, i & 1))) { alive = false; break; }
            tc_fence_after();
            const bool all_visible = (kv0 + AT_HALF - 1 <= p0) && (a.window == 0 || kv0 >= p_last - a.window + 1);
            unsigned sv[AT_HALF];
#pragma unroll
            for (int c = 0; c < AT_HALF / 32; ++c) tmem_ld32_issue(tmem_sh + c * 32, sv + c * 32);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.s_free);             // the next scores may overwrite these
            if (!all_visible) {
                // keys kv0 + j with j in [first, first + span] are seen by this row; the others score -inf
                const int first = lo_row - kv0, span = pos - kv0 - first;
#pragma unroll
                for (int j = 0; j < AT_HALF; ++j)
                    if ((unsigned)(j - first) > (unsigned)span || span < 0) sv[j] = 0xff800000u;
            }
            // the maximum: four independent chains of three-input maxima
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < AT_HALF; j += 8) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    mx4[q] = max3(mx4[q], __uint_as_float(sv[j + 2 * q]), __uint_as_float(sv[j + 2 * q + 1]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2;   // the scale is positive
            // raise the reference only when it is far behind (or not set yet)
            float factor = 1.f;
            if (mx > m_ref + AT_RESCALE_THRESHOLD) {
                factor = m_ref == -INFINITY ? 0.f : ex2(m_ref - mx);
                m_ref = mx;
            }
            const float base = m_ref == -INFINITY ? 0.f : m_ref;
            // probabilities (2^-inf = 0 for the masked keys), packed to bfloat16; scale, shift and the
            // running sums two elements per instruction
            unsigned pk[AT_HALF / 2];
            const unsigned long long scale2 = pack2(a.scale_log2, a.scale_log2), shift2 = pack2(-base, -base);
            unsigned long long sum2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int j = 0; j < AT_HALF; j += 2) {
                const unsigned long long x2 = fma2(pack2(__uint_as_float(sv[j]), __uint_as_float(sv[j + 1])), scale2, shift2);
                float e0, e1;
                if (((j >> 1) & 7) < AT_POLY_OF_8) {
                    exp2_poly2(x2, e0, e1);
                } else {
                    float x0, x1;
                    unpack2(x2, x0, x1);
                    e0 = ex2(x0); e1 = ex2(x1);
                }
                sum2[(j >> 1) & 3] = add2(sum2[(j >> 1) & 3], pack2(e0, e1));
                const __nv_bfloat162 b = __floats2bfloat162_rn(e0, e1);
                pk[j / 2] = *reinterpret_cast<const unsigned *>(&b);
            }
            float sum, sum_hi;
            unpack2(add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3])), sum, sum_hi);
            sum += sum_hi;
            l = l * factor + sum;
            // the second product of the tile before must be done: it reads P and writes the accumulators
            if (i > 0 && !__all_sync(0xffffffffu, mbar_wait(&s.pv_done, (i - 1) & 1))) { alive = false; break; }
            tc_fence_after();
            if (__any_sync(0xffffffffu, factor != 1.f) && i > 0) {
                // rescale this warp's rows of its accumulator (rows that keep their reference multiply by 1)
#pragma unroll 1
                for (int c = 0; c < DH / 32; ++c) {
                    unsigned ov[32];
                    tmem_ld32(tmem_oh + c * 32, ov);
#pragma unroll
                    for (int j = 0; j < 32; ++j) ov[j] = __float_as_uint(__uint_as_float(ov[j]) * factor);
                    tmem_st32(tmem_oh + c * 32, ov);
                }
            }
            // P into shared memory: this half's 64 keys are one 128-byte row of sub-tile `half`,
            // 16-byte pieces swizzled
#pragma unroll
            for (int c = 0; c < AT_HALF / 8; ++c) {
                unsigned char *dst = reinterpret_cast<unsigned char *>(s.p[half]) + row * 128 + ((c ^ (row & 7)) << 4);
                *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            }
            // The tile's value rows beyond the last key that any row of this tile sees carry weight 0 in P V, but
            // 0 x NaN is NaN: slots of the request's last page that lie beyond its end hold whatever an earlier
            // holder of the page left there.  Those rows become zeros before the product reads them (only the last
            // tile of keys has any; the first half's threads take one key row each).
            if (i == n_kv - 1 && half == 0 && kv_first + i * AT_BN + AT_BN - 1 > p_last) {
                if (!__all_sync(0xffffffffu, mbar_wait(&s.v_full[i & 1], (i >> 1) & 1))) { alive = false; break; }
                if (kv_first + i * AT_BN + row > p_last) {
#pragma unroll
                    for (int u = 0; u < SUB; ++u) {
                        uint4 *vrow = reinterpret_cast<uint4 *>(s.v[i & 1][u] + row * 64);      // 128 bytes; the swizzle stays inside
#pragma unroll
                        for (int c = 0; c < 8; ++c) vrow[c] = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.p_ready);            // one arrival per softmax warp
        }
        if (alive && !__all_sync(0xffffffffu, mbar_wait(&s.pv_done, (n_kv - 1) & 1))) alive = false;
        tc_fence_after();
        // the halves meet: P's place in shared memory is free now and carries (reference, sum) across
        float2 *meet = reinterpret_cast<float2 *>(s.p[0]);      // [half][row]
        if (alive) {
            meet[half * AT_BM + row] = make_float2(m_ref, l);
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.met[quarter]);
            if (!__all_sync(0xffffffffu, mbar_wait(&s.met[quarter], 0))) alive = false;
        }
        if (!alive) { failed = 3; if (lane == 0) atomicExch(a.status, 13); }
        if (alive) {
            const float2 other = meet[(half ^ 1) * AT_BM + row];
            // a half that saw no key has reference -inf, sum 0 and an accumulator of zeros
            const float m_all = fmaxf(m_ref, other.x);
            const float w_mine = ex2(m_ref - m_all), w_other = ex2(other.x - m_all);
            const float inv = 1.f / (l * w_mine + other.y * w_other);
            const float w0 = (half ? w_other : w_mine) * inv, w1 = (half ? w_mine : w_other) * inv;
            // this thread writes columns [half * DH / 2, + DH / 2) of its row
            __nv_bfloat16 *dst = a.out + ((size_t)(row0 + row) * a.nh + h) * DH + half * (DH / 2);
#pragma unroll 1
            for (int c = 0; c < DH / 64; ++c) {
                unsigned o0[32], o1[32];
                tmem_ld32_issue(tmem_o + lane_addr + half * (DH / 2) + c * 32, o0);
                tmem_ld32_issue(tmem_o + lane_addr + DH + half * (DH / 2) + c * 32, o1);
                tmem_wait_ld();
                if (row < nrows) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        unsigned w[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float lo = __uint_as_float(o0[j + 2 * q]) * w0 + __uint_as_float(o1[j + 2 * q]) * w1;
                            const float hi = __uint_as_float(o0[j + 2 * q + 1]) * w0 + __uint_as_float(o1[j + 2 * q + 1]) * w1;
                            const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
                            w[q] = *reinterpret_cast<const unsigned *>(&b);
                        }
                        *reinterpret_cast<uint4 *>(dst + c * 32 + j) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    // a role that gave up may leave copies in flight: bounded time to land before memory is released
    if (failed && lane == 0) {
        mbar_wait(&s.q_full, 0);
        for (int st = 0; st < 2; ++st) { mbar_wait(&s.k_full[st], 0); mbar_wait(&s.v_full[st], 0); }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(s.tmem_base, TMEM_COLS);
}

// ---- host side -----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}
// A 2-D bfloat16 tensor map [rows, cols] with boxes of 64 columns x box_rows, 128-byte swizzle; cached.
static int tensor_map(const void *ptr, long long rows, int cols, int box_rows, CUtensorMap *out) {
    using Key = std::tuple<const void *, long long, int, int>;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const Key key(ptr, rows, cols, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return JK_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) JK_FAIL(JK_CUDA_ERROR, "attention_tcgen05: the driver has no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) JK_FAIL(JK_CUDA_ERROR, "attention_tcgen05: cuTensorMapEncodeTiled failed with %d", (int)r);
    if (cache.size() > 1024) cache.clear();
    cache[key] = m;
    *out = m;
    return JK_OK;
}

// Head sizes and page sizes this kernel is built for (the page must divide a tile of 128 keys and
// fill whole groups of 8 swizzled rows).
JK_EXPORT int jk_attention_tcgen05_supports(int dh, int page_size) {
    return (dh == 64 || dh == 128) && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128);
}

template <int DH>
static int launch_at(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const AtArgs &a, cudaStream_t stream) {
    const size_t smem = sizeof(AtSmem<DH>);
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) JK_FAIL(JK_CUDA_ERROR, "attention_tcgen05: %s", cudaGetErrorString(e));
    jk_launch(attention_tcgen05_kernel<DH>, dim3(a.nh, a.ntiles), dim3(AT_THREADS), smem, stream, mq, mk, mv, a);
    JK_CHECK_LAUNCH("attention_tcgen05");
    return JK_OK;
}

JK_EXPORT int jk_attention_tcgen05(const void *q, const void *k_pages, const void *v_pages, void *out, const int *tiles,
                                   int ntiles, int ntok, const int *req_start, const int *req_pos, const int *block_table,
                                   int max_blocks, int num_pages, int page_size, int nh, int nkvh, int dh, float scale,
                                   int window, int *status, cudaStream_t stream) {
    if (ntiles == 0) return JK_OK;
    JK_REQUIRE(jk_attention_tcgen05_supports(dh, page_size), "attention_tcgen05: head size %d with pages of %d is not built", dh, page_size);
    JK_REQUIRE(ntiles > 0 && nh > 0 && nkvh > 0 && nh % nkvh == 0 && ntiles <= 65535, "attention_tcgen05: tiles %d heads %d/%d", ntiles, nh, nkvh);
    JK_REQUIRE(max_blocks > 0 && window >= 0 && status != nullptr && num_pages > 0, "attention_tcgen05: bad arguments");
    CUtensorMap mq, mk, mv;
    if (int rc = tensor_map(q, ntok, nh * dh, AT_BM, &mq)) return rc;
    if (int rc = tensor_map(k_pages, (long long)num_pages * nkvh * page_size, dh, page_size, &mk)) return rc;
    if (int rc = tensor_map(v_pages, (long long)num_pages * nkvh * page_size, dh, page_size, &mv)) return rc;
    AtArgs a{(__nv_bfloat16 *)out, tiles, req_start, req_pos, block_table, status,
             ntiles, nh, nkvh, page_size, max_blocks, window, scale * 1.4426950408889634f};
    if (dh == 64) return launch_at<64>(mq, mk, mv, a, stream);
    return launch_at<128>(mq, mk, mv, a, stream);
}
