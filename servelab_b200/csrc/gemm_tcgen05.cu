// Weight-streaming matrix product on the 5th-generation tensor cores (tcgen05):
//   out[M, N] = x[M, K] . W[N, K]^T (+ bias[N]),  bfloat16 in, float32 accumulate in
//   tensor memory, bfloat16 or float32 out,  M <= 64 tokens ("swap-AB": the 128 rows
//   of a W tile are the M side of the MMA, the tokens are its N side).
//
// A decode step reads every weight once and does little arithmetic with it, so the
// kernel is built around moving W with as few instructions as possible:
//   * one thread issues TMA tile loads (cp.async.bulk.tensor, 128-byte swizzle) of
//     W [128 rows x 64 k] and x [tokens x 64 k] into a ring of shared-memory stages,
//     completion counted in bytes on an mbarrier per stage;
//   * one thread issues tcgen05.mma (M = 128, N = tokens padded to 16, K = 16, four
//     per stage) on shared-memory descriptors, accumulating into TMEM; a
//     tcgen05.commit per stage hands the stage back to the loader;
//   * four warps read the accumulator with tcgen05.ld and store it.
// The K range is split over gridDim.y blocks so that narrow outputs still occupy
// every SM; with more than one split the blocks write float32 partial sums and a
// second kernel adds them in a fixed order (deterministic).
//
// A second kernel (gemm_tc_cluster_kernel, further down) runs the K splits of a row tile as
// one thread-block cluster that adds its accumulators up through distributed shared memory,
// with epilogues that finish the result (store, q|k|v rotation and cache write, add into the
// residual stream); both kernels can build the x operand from the float32 residual stream
// (the RMS norm before the product) instead of fetching it.
//
// Every wait on an mbarrier is bounded: after SLB_TC_SPIN_LIMIT polls the role
// records a code in the status word, leaves its loop, and the block frees its TMEM
// and returns, so a wrong descriptor cannot hang the GPU.
//
// Reference analogue: F.linear in the decode step (servelab/parallel/
// tp_model.py:48-53,67-68,115-119), left to the library there.
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int TC_BM = 128;            // rows of W per block (MMA M)
constexpr int TC_BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int TC_MAX_TOK = 64;        // MMA N
constexpr int TC_MAX_STAGES = 12;     // the ring is as deep as shared memory allows
constexpr int TC_THREADS = 192;       // warp 0 loader, warp 1 MMA + TMEM, warps 2..5 epilogue
constexpr int TC_TMEM_COLS = 64;
constexpr uint32_t SLB_TC_SPIN_LIMIT = 1u << 18;
constexpr int A_STAGE_BYTES = TC_BM * TC_BK * 2;          // 16 KB of W per stage
constexpr size_t TC_SMEM_BUDGET = 200 * 1024;             // stages + barriers (one block per SM)
constexpr size_t TC_SMEM_TAIL = 256;                      // barriers and the TMEM address

// x tile of a stage: ntok16 rows of 128 bytes, rounded up so stages stay 1024-aligned
__host__ __device__ constexpr int b_stage_bytes(int ntok16) { return (ntok16 * TC_BK * 2 + 1023) / 1024 * 1024; }
__host__ __device__ constexpr int stages_for(int ntok16, int max_stages) {
    const int s = (int)((TC_SMEM_BUDGET - 1024 - TC_SMEM_TAIL) / (A_STAGE_BYTES + b_stage_bytes(ntok16)));
    const int cap = (max_stages > 0 && max_stages < TC_MAX_STAGES) ? max_stages : TC_MAX_STAGES;
    return s > cap ? cap : s;
}

__device__ int tc_status_word = 0;    // 0 ok; else (role << 8 | what) of the first timeout

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait for the phase with the given parity; false after the poll limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SLB_TC_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (stride byte offset), version 1 (Blackwell), layout 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);            // start address
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset
    d |= (uint64_t)1 << 46;                                // descriptor version
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
}

// Weights to pull into the L2 cache for the product that follows this one: the first
// `bytes` of that matrix, requested in pieces of chunk_bytes (a request costs the issuing
// warp tens of cycles whatever its size, so the pieces are large and few).  The requests
// are issued when this block's own tiles have all arrived, so they fill the time in which
// the small kernels between two products leave the memory idle.
struct Prefetch {
    const unsigned char* ptr;
    long long bytes;
    int chunk_bytes;
};
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// The x operand as the RMS norm of the float32 residual stream, built by the loader warp
// instead of fetched by TMA: x[tok][k] = resid[tok][k] * rstd[tok] * weight[k], with
// rstd[tok] = 1 / sqrt(sum_t sumsq[t][tok] / K + eps) from the partial sums of squares that
// the product before the norm left per row tile (its EPI_RESID epilogue).  Up to 16 tokens.
struct NormIn {
    const float* resid;                 // [M][ld], every update already added; null: x comes by TMA
    int ld;
    const float* sumsq;                 // [tiles][M]
    int tiles;
    const float* weight;                // [K]
    float eps;
};
constexpr int NORM_IN_MAX_TOK = 16;

__device__ __forceinline__ void mbar_arrive_plain(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// With NormIn the full barrier of a stage counts two arrivals: the loader thread's, with the
// bytes of the W tile it requests by TMA, and that of the warp that wrote the stage's x tile.
__device__ __forceinline__ void load_w_only(const CUtensorMap* map_w, unsigned char* a_stage, int stages,
                                            uint64_t* full, uint64_t* empty, int kb_begin, int iters,
                                            int n0, int* status, int code) {
    const int ahead = min(iters, stages);
    for (int i = 0; i < ahead; ++i) {                      // W is written by no kernel
        mbar_expect_tx(&full[i], A_STAGE_BYTES);
        tma_load_2d(a_stage + i * A_STAGE_BYTES, map_w, &full[i], (kb_begin + i) * TC_BK, n0);
    }
    for (int i = ahead; i < iters; ++i) {
        const int s = i % stages;
        if (!mbar_wait(&empty[s], ((i / stages) & 1) ^ 1)) {
            atomicCAS(status, 0, (1 << 8) | code);
            break;
        }
        mbar_expect_tx(&full[s], A_STAGE_BYTES);
        tma_load_2d(a_stage + s * A_STAGE_BYTES, map_w, &full[s], (kb_begin + i) * TC_BK, n0);
    }
}

// The x tiles, written by the four epilogue warps while the main loop runs (they have nothing
// else to do until the accumulator is complete): warp xw takes the k-blocks i = xw, xw + 4, ...
// of this block, so each has four k-blocks' time for the loads of one.  The residual rows and
// norm weights of its next k-block are loaded before the current one is converted.  Called
// after pdl_wait() by whole warps.
__device__ __forceinline__ void produce_x_normed(const NormIn& nin, unsigned char* b_stage, int b_stage_bytes_,
                                                 int stages, uint64_t* full, uint64_t* empty, int kb_begin,
                                                 int iters, int M, int K, int ntok16, int* status, int xw) {
    const int lane = threadIdx.x & 31;
    float rstd = 0.f;
    if (lane < M) {
        float ss = 0.f;
        for (int t = 0; t < nin.tiles; ++t) ss += nin.sumsq[(size_t)t * M + lane];
        rstd = 1.0f / sqrtf(ss / (float)K + nin.eps);
    }
    // A k-block's x tile is M * 8 chunks of 16 bytes; a lane handles chunk `lane` and
    // `lane + 32` of each half of 64 chunks (8 tokens).  Few registers on purpose: with
    // fewer than about 100 a thread, a third block fits on an SM beside two of the kernel
    // before this one and requests its first weight tiles while they finish.
    const int chunks = M * 8;
    for (int i = xw; i < iters; i += 4) {
        const int s = i % stages;
        const int k0 = (kb_begin + i) * TC_BK;
        unsigned char* tile = b_stage + s * b_stage_bytes_;
        bool waited = i < stages;                          // the first use of a stage needs no wait
        if (waited)
            for (int off = M * 128 + lane * 16; off < ntok16 * 128; off += 32 * 16)
                *reinterpret_cast<uint4*>(tile + off) = make_uint4(0, 0, 0, 0);   // rows beyond the tokens
        bool ok = true;
        for (int half = 0; half * 64 < chunks && ok; ++half) {
            float4 v[2][4];                                // residual (2) and weight (2) per chunk
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int idx = half * 64 + c * 32 + lane;
                const int tok = idx >> 3, k = k0 + (idx & 7) * 8;
                if (idx < chunks && k < K) {               // K is a multiple of 8
                    const float4* src = reinterpret_cast<const float4*>(nin.resid + (size_t)tok * nin.ld + k);
                    const float4* wsrc = reinterpret_cast<const float4*>(nin.weight + k);
                    v[c][0] = __ldcg(src);
                    v[c][1] = __ldcg(src + 1);
                    v[c][2] = __ldg(wsrc);
                    v[c][3] = __ldg(wsrc + 1);
                } else {
                    v[c][0] = v[c][1] = v[c][2] = v[c][3] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            if (!waited) {                                 // the loads are in flight meanwhile
                if (lane == 0) ok = mbar_wait(&empty[s], ((i / stages) & 1) ^ 1);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                waited = true;
                if (!ok) break;
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int idx = half * 64 + c * 32 + lane;
                const int tok = idx >> 3, j = idx & 7;
                const float r = __shfl_sync(0xffffffffu, rstd, tok & 31);
                if (idx < chunks) {
                    const float4 a = v[c][0], b = v[c][1], w0 = v[c][2], w1 = v[c][3];
                    __nv_bfloat162 o[4];
                    o[0] = __floats2bfloat162_rn(a.x * r * w0.x, a.y * r * w0.y);
                    o[1] = __floats2bfloat162_rn(a.z * r * w0.z, a.w * r * w0.w);
                    o[2] = __floats2bfloat162_rn(b.x * r * w1.x, b.y * r * w1.y);
                    o[3] = __floats2bfloat162_rn(b.z * r * w1.z, b.w * r * w1.w);
                    // 128-byte swizzle of a K-major tile: chunk j of row tok sits at chunk j ^ (tok & 7)
                    *reinterpret_cast<uint4*>(tile + tok * 128 + ((j ^ (tok & 7)) << 4)) =
                        *reinterpret_cast<const uint4*>(o);
                }
            }
        }
        if (!ok) {
            if (lane == 0) atomicCAS(status, 0, (4 << 8) | 1);
            break;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive_plain(&full[s]);
    }
    __syncwarp();
}

// grid (row tiles of W, K splits).  ntok16: tokens padded to a multiple of 16.
// splits == 1: `out` receives the result (+ bias) in its dtype; otherwise `partial`
// receives float32 [split][M][N].
template <typename TO, bool NORM_IN>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_decode_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    TO* __restrict__ out, int ldo, float* __restrict__ partial, const float* __restrict__ bias,
    int M, int N, int K, int ntok16, int max_stages, int* __restrict__ status, Prefetch pf, int swiglu,
    const NormIn nin) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int B_STAGE_BYTES = b_stage_bytes(ntok16);
    const int TC_STAGES = stages_for(ntok16, max_stages);
    unsigned char* a_stage = base;
    unsigned char* b_stage = base + TC_STAGES * A_STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + TC_STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
    uint64_t* empty = full + TC_MAX_STAGES;
    uint64_t* accum = empty + TC_MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TC_BM;
    const int splits = gridDim.y, split = blockIdx.y;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    const int per = (kblocks + splits - 1) / splits;
    const int kb_begin = min(kblocks, split * per);
    const int kb_end = min(kblocks, kb_begin + per);
    const int iters = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&full[s], NORM_IN ? 2 : 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                        // one warp allocates the accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ loader
        // W is written by no kernel, x by the preceding one: the W tiles of the first
        // stages are requested at once, the x tiles after the wait for that kernel.
        if constexpr (NORM_IN) {
            if (lane == 0) load_w_only(&map_w, a_stage, TC_STAGES, full, empty, kb_begin, iters, n0, status, 3);
        } else if (lane == 0) {
            const uint32_t bytes = A_STAGE_BYTES + (uint32_t)ntok16 * TC_BK * 2;
            const int ahead = min(iters, TC_STAGES);
            for (int i = 0; i < ahead; ++i) {                 // stages are empty at the start
                mbar_expect_tx(&full[i], bytes);
                tma_load_2d(a_stage + i * A_STAGE_BYTES, &map_w, &full[i], (kb_begin + i) * TC_BK, n0);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(b_stage + i * B_STAGE_BYTES, &map_x, &full[i], (kb_begin + i) * TC_BK, 0);
            for (int i = ahead; i < iters; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&empty[s], ((i / TC_STAGES) & 1) ^ 1)) {
                    atomicCAS(status, 0, (1 << 8) | 1);
                    break;
                }
                mbar_expect_tx(&full[s], bytes);
                const int k = (kb_begin + i) * TC_BK;
                tma_load_2d(a_stage + s * A_STAGE_BYTES, &map_w, &full[s], k, n0);
                tma_load_2d(b_stage + s * B_STAGE_BYTES, &map_x, &full[s], k, 0);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   ((uint32_t)(ntok16 >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < iters && ok; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&full[s], (i / TC_STAGES) & 1)) {
                    atomicCAS(status, 0, (2 << 8) | 1);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = umma_desc_sw128(smem_u32(a_stage + s * A_STAGE_BYTES));
                const uint64_t bdesc = umma_desc_sw128(smem_u32(b_stage + s * B_STAGE_BYTES));
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)     // 32 bytes further per K = 16 step
                    umma_bf16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&empty[s]);                      // stage free once these MMAs have read it
            }
            if (ok) umma_commit(accum);                      // accumulator complete
        }
    } else {
        // ------------------------------------------------------------ epilogue
        pdl_wait();                                          // nothing is written before the
                                                             // preceding kernel has finished
        if constexpr (NORM_IN)
            produce_x_normed(nin, b_stage, B_STAGE_BYTES, TC_STAGES, full, empty, kb_begin, iters, M, K, ntok16,
                             status, warp - 2);
        const int quarter = warp & 3;                        // TMEM lanes this warp may read
        const int row = quarter * 32 + lane;                 // row of the tile = row of W
        const int n = n0 + row;
        bool ok = true;
        if (iters > 0) {
            ok = mbar_wait(accum, 0);
            if (!ok) atomicCAS(status, 0, (3 << 8) | 1);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_launch_dependents();
        if (pf.ptr != nullptr) {
            const long long items = (pf.bytes + pf.chunk_bytes - 1) / pf.chunk_bytes;
            const long long stride = (long long)(gridDim.x * gridDim.y) * (TC_THREADS - 64);
            // consecutive pieces go to different blocks (one thread of a block at a time)
            const long long first = (long long)(threadIdx.x - 64) * (gridDim.x * gridDim.y) +
                                    (blockIdx.y * gridDim.x + blockIdx.x);
            for (long long it = first; it < items; it += stride) {
                const long long off = it * pf.chunk_bytes;
                const long long left = pf.bytes - off;
                prefetch_l2(pf.ptr + off, (uint32_t)(left < pf.chunk_bytes ? left : pf.chunk_bytes) & ~15u);
            }
        }
        if (swiglu) {
            // W holds gate and up rows alternating in runs of 64, so this tile's rows are 64
            // gates and their 64 ups: the upper two warps park the ups in shared memory (the
            // ring is idle: every tile has arrived and every MMA has run), the lower two
            // combine: out[tok, tile * 64 + r] = silu(gate_r) * up_r.  One K split only.
            float* ups = reinterpret_cast<float*>(a_stage);            // [64][ntok16 + 1]
            const int ld_ups = ntok16 + 1;
            if (row >= 64) {
                for (int c0 = 0; c0 < ntok16; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) ups[(row - 64) * ld_ups + c0 + j] = __uint_as_float(v[j]);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");             // the four epilogue warps
            if (row < 64) {
                const int col = (int)blockIdx.x * 64 + row;            // index of the gate
                for (int c0 = 0; c0 < ntok16; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (col < N / 2 && ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int tok = c0 + j;
                            if (tok >= M) break;
                            const float gt = __uint_as_float(v[j]);
                            const float up = ups[row * ld_ups + tok];
                            out[(size_t)tok * ldo + col] = from_float<TO>(gt / (1.0f + expf(-gt)) * up);
                        }
                    }
                }
            }
        } else
        for (int c0 = 0; c0 < ntok16; c0 += 16) {
            uint32_t v[16];
            if (iters > 0 && ok) {
                tmem_ld16(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
            if (n < N && ok) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = c0 + j;
                    if (tok >= M) break;
                    const float val = __uint_as_float(v[j]);
                    if (splits == 1)
                        out[(size_t)tok * ldo + n] = from_float<TO>(val + (bias ? bias[n] : 0.f));
                    else
                        partial[((size_t)split * M + tok) * N + n] = val;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TC_TMEM_COLS)
                     : "memory");
    }
}

// out[tok, n] = sum over splits (in order) of partial[s][tok][n] (+ bias[n])
template <typename TO>
__global__ void gemm_tc_reduce_kernel(const float* __restrict__ partial, TO* __restrict__ out, int ldo,
                                      const float* __restrict__ bias, int M, int N, int splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int tok = blockIdx.y;
    if (n >= N) return;
    float sum = 0.f;
    for (int s = 0; s < splits; ++s) sum += partial[((size_t)s * M + tok) * N + n];
    if (bias) sum += bias[n];
    out[(size_t)tok * ldo + n] = from_float<TO>(sum);
}

// ---- the K splits of a row tile as one thread-block cluster ----------------------
// grid (row tiles of W, K splits), cluster (1, K splits, 1): the blocks that share a row
// tile run at the same time and can read one another's shared memory.  Each block
// accumulates its K range in tensor memory as above, parks the result in its own shared
// memory, and after a cluster barrier block r adds up, in the order of the ranks, the
// tokens r, r + splits, ... of all blocks and finishes them: no partial sums in global
// memory, no second kernel, a fixed order of additions.
//
// What "finishes" means is the EPI parameter:
//   EPI_STORE  out[tok, n] = sum + bias[n]
//   EPI_ROPE   the q|k|v product of an attention layer: bias added, q and k rotated by the
//              token's position, q written to q_out, k and v into the token's slot of the
//              paged cache (the arithmetic of the kernel in rope_cache.cu).  A row tile
//              must hold whole heads: head sizes 16, 32, 64, 128.
//   EPI_RESID  resid[tok, n] += sum + bias[n] (the float32 residual stream), and the sum of
//              squares of the tile's 128 updated values of every token to sumsq[tile][tok]:
//              what the RMS norm that follows needs, so that the product after it can
//              build its normed input itself (NormIn above).
enum { EPI_STORE = 0, EPI_ROPE = 1, EPI_RESID = 2 };

struct ResidEpilogue {
    float* resid;                       // [M][ld]
    int ld;
    float* sumsq;                       // [row tiles][M]
};

struct RopeEpilogue {
    const float* bias;                  // [N] or null
    const int* positions;               // [M]
    const int* seq_of_token;            // [M]
    const int* block_table;             // [requests][max_pages]
    int max_pages, page_size;
    const float* inv_freq;              // [rotary_dim / 2] or null
    int rotary_dim;
    bf16* q_out;
    int ld_q;
    bf16* k_cache;                      // null: nothing is written to the cache
    bf16* v_cache;
    int H, Hkv, D;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// every thread of every block of the cluster, warps converged
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t a;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

template <int EPI, bool NORM_IN>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_cluster_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    bf16* __restrict__ out, int ldo, const float* __restrict__ bias, int M, int N, int K, int ntok16,
    int max_stages, int* __restrict__ status, const RopeEpilogue rope, const ResidEpilogue res,
    const NormIn nin) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int B_STAGE_BYTES = b_stage_bytes(ntok16);
    const int TC_STAGES = stages_for(ntok16, max_stages);
    unsigned char* a_stage = base;
    unsigned char* b_stage = base + TC_STAGES * A_STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + TC_STAGES * (A_STAGE_BYTES + B_STAGE_BYTES));
    uint64_t* empty = full + TC_MAX_STAGES;
    uint64_t* accum = empty + TC_MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    __shared__ float pair_vals[2][TC_BM];                    // EPI_ROPE: a token's row of the tile
    __shared__ float warp_sq[2][4];                          // EPI_RESID: sums of squares per warp

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TC_BM;
    const int splits = gridDim.y, split = blockIdx.y;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    const int per = (kblocks + splits - 1) / splits;
    const int kb_begin = min(kblocks, split * per);
    const int kb_end = min(kblocks, kb_begin + per);
    const int iters = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&full[s], NORM_IN ? 2 : 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_slot;
    float* acc = reinterpret_cast<float*>(a_stage);          // [ntok16][TC_BM] once the ring is idle

    if (warp == 0) {
        if constexpr (NORM_IN) {
            if (lane == 0) load_w_only(&map_w, a_stage, TC_STAGES, full, empty, kb_begin, iters, n0, status, 4);
        } else if (lane == 0) {
            const uint32_t bytes = A_STAGE_BYTES + (uint32_t)ntok16 * TC_BK * 2;
            const int ahead = min(iters, TC_STAGES);
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full[i], bytes);
                tma_load_2d(a_stage + i * A_STAGE_BYTES, &map_w, &full[i], (kb_begin + i) * TC_BK, n0);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(b_stage + i * B_STAGE_BYTES, &map_x, &full[i], (kb_begin + i) * TC_BK, 0);
            for (int i = ahead; i < iters; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&empty[s], ((i / TC_STAGES) & 1) ^ 1)) {
                    atomicCAS(status, 0, (1 << 8) | 2);
                    break;
                }
                mbar_expect_tx(&full[s], bytes);
                const int k = (kb_begin + i) * TC_BK;
                tma_load_2d(a_stage + s * A_STAGE_BYTES, &map_w, &full[s], k, n0);
                tma_load_2d(b_stage + s * B_STAGE_BYTES, &map_x, &full[s], k, 0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   ((uint32_t)(ntok16 >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            bool ok = true;
            for (int i = 0; i < iters && ok; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&full[s], (i / TC_STAGES) & 1)) {
                    atomicCAS(status, 0, (2 << 8) | 2);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t adesc = umma_desc_sw128(smem_u32(a_stage + s * A_STAGE_BYTES));
                const uint64_t bdesc = umma_desc_sw128(smem_u32(b_stage + s * B_STAGE_BYTES));
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)
                    umma_bf16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(accum);
        }
        __syncwarp();
    } else {
        // ------------------------------------------ epilogue, part 1: accumulator -> acc
        pdl_wait();
        if constexpr (NORM_IN)
            produce_x_normed(nin, b_stage, B_STAGE_BYTES, TC_STAGES, full, empty, kb_begin, iters, M, K, ntok16,
                             status, warp - 2);
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        bool ok = true;
        if (iters > 0) {
            ok = mbar_wait(accum, 0);
            if (!ok) atomicCAS(status, 0, (3 << 8) | 2);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_launch_dependents();
        for (int c0 = 0; c0 < ntok16; c0 += 16) {
            uint32_t v[16];
            if (iters > 0 && ok) {
                tmem_ld16(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[(c0 + j) * TC_BM + row] = __uint_as_float(v[j]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();                                      // every block's acc is complete

    if (warp >= 2) {
        // ------------------------------- epilogue, part 2: this block's share of the tokens
        const int row = (warp & 3) * 32 + lane;
        const int n = n0 + row;
        const uint32_t rank = cluster_rank(), nranks = cluster_size();
        int parity = 0;
        for (int tok = (int)rank; tok < M; tok += (int)nranks) {
            const uint32_t addr = smem_u32(acc + tok * TC_BM + row);
            float sum = 0.f;
            for (uint32_t p = 0; p < nranks; ++p) sum += ld_peer_f32(addr, p);
            if constexpr (EPI == EPI_STORE) {
                if (n < N) out[(size_t)tok * ldo + n] = __float2bfloat16_rn(sum + (bias ? bias[n] : 0.f));
            } else if constexpr (EPI == EPI_RESID) {
                float r = 0.f;
                if (n < N) {
                    float* dst = res.resid + (size_t)tok * res.ld + n;
                    r = *dst + (sum + (bias ? bias[n] : 0.f));
                    *dst = r;
                }
                const float sq = warp_sum(r * r);
                if (lane == 0) warp_sq[parity][warp & 3] = sq;
                asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps
                if (row == 0)
                    res.sumsq[(size_t)blockIdx.x * M + tok] =
                        ((warp_sq[parity][0] + warp_sq[parity][1]) + warp_sq[parity][2]) + warp_sq[parity][3];
                parity ^= 1;
            } else {
                const int D = rope.D;
                const int half = rope.inv_freq != nullptr ? rope.rotary_dim >> 1 : 0;
                float v = (n < N) ? sum + (rope.bias ? rope.bias[n] : 0.f) : 0.f;
                pair_vals[parity][row] = v;
                asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps
                if (n < N) {
                    const int j = n / D, e = n - j * D;
                    const bool is_v = j >= rope.H + rope.Hkv;
                    const int pos = rope.positions[tok];
                    if (!is_v && e < 2 * half) {
                        const int i = e < half ? e : e - half;
                        float sn, cs;
                        sincosf((float)pos * rope.inv_freq[i], &sn, &cs);
                        const float other = pair_vals[parity][e < half ? row + half : row - half];
                        v = e < half ? v * cs - other * sn : v * cs + other * sn;
                    }
                    bf16* dst = nullptr;
                    if (j < rope.H) {
                        dst = rope.q_out + (size_t)tok * rope.ld_q + (size_t)j * D;
                    } else if (rope.k_cache != nullptr) {
                        const int page = rope.block_table[(size_t)rope.seq_of_token[tok] * rope.max_pages +
                                                          pos / rope.page_size];
                        if (page >= 0) {
                            const int kvh = is_v ? j - rope.H - rope.Hkv : j - rope.H;
                            dst = (is_v ? rope.v_cache : rope.k_cache) +
                                  (((size_t)page * rope.Hkv + kvh) * rope.page_size + pos % rope.page_size) * D;
                        }
                    }
                    if (dst != nullptr) dst[e] = __float2bfloat16_rn(v);
                }
                parity ^= 1;
            }
        }
    }
    __syncwarp();
    cluster_sync_all();                                      // no block leaves while its acc is read
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TC_TMEM_COLS)
                     : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Tensor map of a row-major [rows, K] bfloat16 matrix with leading dimension ld,
// tiles of box_rows x 64 elements, 128-byte swizzle, zeros outside the matrix.
int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return SLB_ERR_BAD_ARG;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                          elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : SLB_ERR_BAD_ARG;
}

template <typename TO, bool NORM_IN>
int run(const bf16* x, int ldx, const bf16* W, int ldw, TO* out, int ldo, const float* bias,
        float* workspace, int M, int N, int K, int splits, int max_stages, int defer_sum,
        const Prefetch& pf, int swiglu, const NormIn& nin, cudaStream_t st) {
    CUtensorMap map_w, map_x = {};
    const int ntok16 = (M + 15) / 16 * 16;
    int rc = make_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc != 0) return rc;
    if (!NORM_IN) {
        rc = make_map(&map_x, x, M, K, ldx, ntok16);
        if (rc != 0) return rc;
    }
    static bool configured = false;                         // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_decode_kernel<TO, NORM_IN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)TC_SMEM_BUDGET);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const size_t TC_SMEM = 1024 + (size_t)stages_for(ntok16, max_stages) * (A_STAGE_BYTES + b_stage_bytes(ntok16)) +
                           TC_SMEM_TAIL;
    int* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&status, tc_status_word);
    if (e != cudaSuccess) return (int)e;
    rc = slb_launch(gemm_tc_decode_kernel<TO, NORM_IN>, dim3((N + TC_BM - 1) / TC_BM, splits), dim3(TC_THREADS),
                    TC_SMEM, st, map_w, map_x, out, ldo, workspace, bias, M, N, K, ntok16, max_stages, status, pf,
                    swiglu, nin);
    if (rc != 0 || splits == 1 || defer_sum) return rc;
    return slb_launch(gemm_tc_reduce_kernel<TO>, dim3((N + 255) / 256, M), dim3(256), 0, st,
                      (const float*)workspace, out, ldo, bias, M, N, splits);
}

// what a caller may pass as the norm that produces x
int check_norm_in(const NormIn& nin, int M, int K) {
    if (nin.resid == nullptr) return 0;
    if (M > NORM_IN_MAX_TOK) return SLB_ERR_TOO_LARGE;
    if (nin.sumsq == nullptr || nin.weight == nullptr || nin.tiles < 1 || nin.ld < K || nin.ld % 4 ||
        !(nin.eps >= 0.f) || ((uintptr_t)nin.resid | (uintptr_t)nin.weight) % 16)
        return SLB_ERR_BAD_ARG;
    return 0;
}

template <typename... KArgs, typename... Args>
int launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, int cluster_y, size_t smem,
                   cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)cluster_y;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = slb_pdl_enabled ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int TC_MAX_CLUSTER = 8;       // the portable cluster size

template <int EPI, bool NORM_IN>
int run_cluster(const bf16* x, int ldx, const bf16* W, int ldw, bf16* out, int ldo, const float* bias,
                int M, int N, int K, int splits, int max_stages, const RopeEpilogue& rope,
                const ResidEpilogue& res, const NormIn& nin, cudaStream_t st) {
    CUtensorMap map_w, map_x = {};
    const int ntok16 = (M + 15) / 16 * 16;
    int rc = make_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc != 0) return rc;
    if (!NORM_IN) {
        rc = make_map(&map_x, x, M, K, ldx, ntok16);
        if (rc != 0) return rc;
    }
    static bool configured = false;                         // per instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_cluster_kernel<EPI, NORM_IN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BUDGET);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int stages = stages_for(ntok16, max_stages);
    // the parked accumulator [ntok16][128] floats lives in the W stages of the ring
    if ((size_t)stages * A_STAGE_BYTES < (size_t)ntok16 * TC_BM * 4) return SLB_ERR_BAD_ARG;
    const size_t smem = 1024 + (size_t)stages * (A_STAGE_BYTES + b_stage_bytes(ntok16)) + TC_SMEM_TAIL;
    int* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&status, tc_status_word);
    if (e != cudaSuccess) return (int)e;
    return launch_cluster(gemm_tc_cluster_kernel<EPI, NORM_IN>, dim3((N + TC_BM - 1) / TC_BM, splits),
                          dim3(TC_THREADS), splits, smem, st, map_w, map_x, out, ldo, bias, M, N, K, ntok16,
                          max_stages, status, rope, res, nin);
}

// x == nullptr: the x operand is built from the residual stream (NormIn)
int check_cluster_args(const bf16* x, int ldx, const bf16* W, int ldw, int M, int N, int K, int splits) {
    if (K <= 0 || K % 8 || ldw % 8 || ldw < K || (uintptr_t)W % 16) return SLB_ERR_BAD_ARG;
    if (x != nullptr && (ldx % 8 || ldx < K || (uintptr_t)x % 16)) return SLB_ERR_BAD_ARG;
    if (M > TC_MAX_TOK) return SLB_ERR_TOO_LARGE;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > kblocks) return SLB_ERR_BAD_ARG;
    if (splits > TC_MAX_CLUSTER) return SLB_ERR_TOO_LARGE;
    return 0;
}

}  // namespace

extern "C" {

// out[M, N] = x . W^T (+ bias), bfloat16, the K splits of a row tile as one cluster (at most 8):
// no workspace, no second kernel.
int slb_gemm_tc_cluster_bf16(const bf16* x, int ldx, const bf16* W, int ldw, bf16* out, int ldo,
                             const float* bias, int M, int N, int K, int splits, int max_stages,
                             cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (ldo < N || out == nullptr) return SLB_ERR_BAD_ARG;
    const int rc = check_cluster_args(x, ldx, W, ldw, M, N, K, splits);
    if (rc != 0) return rc;
    if (x == nullptr) return SLB_ERR_BAD_ARG;
    return run_cluster<EPI_STORE, false>(x, ldx, W, ldw, out, ldo, bias, M, N, K, splits, max_stages,
                                         RopeEpilogue{}, ResidEpilogue{}, NormIn{}, st);
}

// resid[M, N] += x . W^T (+ bias) on the float32 residual stream, and sumsq[tile][tok] = the sum
// of squares of the updated values of row tile `tile` (ceil(N / 128) tiles) of token tok.
int slb_gemm_tc_resid_bf16(const bf16* x, int ldx, const bf16* W, int ldw, const float* bias, float* resid,
                           int ld_resid, float* sumsq, int M, int N, int K, int splits, int max_stages,
                           cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (x == nullptr || resid == nullptr || sumsq == nullptr || ld_resid < N) return SLB_ERR_BAD_ARG;
    const int rc = check_cluster_args(x, ldx, W, ldw, M, N, K, splits);
    if (rc != 0) return rc;
    const ResidEpilogue res = {resid, ld_resid, sumsq};
    return run_cluster<EPI_RESID, false>(x, ldx, W, ldw, nullptr, 0, bias, M, N, K, splits, max_stages,
                                         RopeEpilogue{}, res, NormIn{}, st);
}

// The q|k|v product of an attention layer with what follows it: W is [(H + 2 Hkv) D, K]
// (q heads, k heads, v heads), and the kernel adds the bias, rotates q and k by
// positions[tok] (angles pos * inv_freq[i], float32), writes q to q_out [M, H D] and k, v to
// the cache slot of the token (block_table[seq_of_token[tok]][pos / page_size]); k_cache ==
// null writes no cache.  Head sizes 16, 32, 64, 128.
// With norm_resid != null x is not read: the loader builds it as the RMS norm of the residual
// stream (NormIn: at most 16 tokens).
int slb_gemm_tc_qkv_rope_bf16(const bf16* x, int ldx, const bf16* W, int ldw, const float* bias,
                              const int* positions, const int* seq_of_token, const int* block_table,
                              int max_pages, int page_size, const float* inv_freq, int rotary_dim,
                              bf16* q_out, int ld_q, bf16* k_cache, bf16* v_cache, int M, int H, int Hkv,
                              int D, int K, int splits, int max_stages, const float* norm_resid,
                              int norm_ld, const float* norm_sumsq, int norm_tiles, const float* norm_weight,
                              float norm_eps, cudaStream_t st) {
    if (M <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || D < 16 || D > TC_BM || TC_BM % D || page_size <= 0 || max_pages <= 0)
        return SLB_ERR_BAD_ARG;
    if (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) || ld_q < H * D) return SLB_ERR_BAD_ARG;
    if (positions == nullptr || seq_of_token == nullptr || block_table == nullptr || q_out == nullptr ||
        (k_cache == nullptr) != (v_cache == nullptr))
        return SLB_ERR_BAD_ARG;
    const int N = (H + 2 * Hkv) * D;
    const NormIn nin = {norm_resid, norm_ld, norm_sumsq, norm_tiles, norm_weight, norm_eps};
    const bool normed = norm_resid != nullptr;
    if (!normed && x == nullptr) return SLB_ERR_BAD_ARG;
    int rc = check_cluster_args(normed ? nullptr : x, ldx, W, ldw, M, N, K, splits);
    if (rc != 0) return rc;
    rc = check_norm_in(nin, M, K);
    if (rc != 0) return rc;
    RopeEpilogue rope = {bias, positions, seq_of_token, block_table, max_pages, page_size, inv_freq,
                         inv_freq != nullptr ? rotary_dim : 0, q_out, ld_q, k_cache, v_cache, H, Hkv, D};
    if (normed)
        return run_cluster<EPI_ROPE, true>(x, ldx, W, ldw, nullptr, 0, nullptr, M, N, K, splits, max_stages,
                                           rope, ResidEpilogue{}, nin, st);
    return run_cluster<EPI_ROPE, false>(x, ldx, W, ldw, nullptr, 0, nullptr, M, N, K, splits, max_stages, rope,
                                        ResidEpilogue{}, nin, st);
}

// workspace: float32 [splits * M * N] when splits > 1 (may be null otherwise).
// max_stages: cap on the depth of the shared-memory ring (0: as deep as fits).
// defer_sum: with splits > 1, leave the partial sums [splits][M][N] in the workspace
// and launch no reduction (the consumer adds them; `out` and `bias` are unused).
// next_w (may be null): the weights the following product will read; their first
// next_bytes are requested into the L2 cache in pieces of next_chunk_bytes (both multiples
// of 16, the address 16-byte aligned).
int slb_gemm_tc_decode_bf16(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo,
                            const float* bias, float* workspace, int out_f32, int M, int N, int K,
                            int splits, int max_stages, int defer_sum, const void* next_w,
                            long long next_bytes, int next_chunk_bytes, int swiglu,
                            const float* norm_resid, int norm_ld, const float* norm_sumsq, int norm_tiles,
                            const float* norm_weight, float norm_eps, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    const NormIn nin = {norm_resid, norm_ld, norm_sumsq, norm_tiles, norm_weight, norm_eps};
    const bool normed = norm_resid != nullptr;               // x is built from the residual stream
    if (K <= 0 || K % 8 || ldw % 8 || ldw < K || (!swiglu && ldo < N)) return SLB_ERR_BAD_ARG;
    if (!normed && (ldx % 8 || ldx < K || (uintptr_t)x % 16)) return SLB_ERR_BAD_ARG;
    if ((uintptr_t)W % 16) return SLB_ERR_BAD_ARG;
    if (M > TC_MAX_TOK) return SLB_ERR_TOO_LARGE;
    int rc = check_norm_in(nin, M, K);
    if (rc != 0) return rc;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > kblocks || splits > 65535) return SLB_ERR_BAD_ARG;
    if (splits > 1 && workspace == nullptr) return SLB_ERR_BAD_ARG;
    // swiglu: W's rows are gates and ups alternating in runs of 64; out is [M, N / 2]
    if (swiglu && (splits != 1 || N % 128 || bias != nullptr || ldo < N / 2)) return SLB_ERR_BAD_ARG;
    // the ups of a tile wait in the idle ring: [64][tokens + 1] floats
    if (swiglu && (size_t)stages_for((M + 15) / 16 * 16, max_stages) * A_STAGE_BYTES < (size_t)64 * ((M + 15) / 16 * 16 + 1) * 4)
        return SLB_ERR_BAD_ARG;
    Prefetch pf = {nullptr, 0, 0};
    if (next_w != nullptr && next_bytes >= 16) {
        if (next_chunk_bytes < 16 || next_chunk_bytes % 16 || next_bytes % 16 || (uintptr_t)next_w % 16)
            return SLB_ERR_BAD_ARG;
        pf = {static_cast<const unsigned char*>(next_w), next_bytes, next_chunk_bytes};
    }
    if (normed) {
        if (out_f32)
            return run<float, true>(x, ldx, W, ldw, (float*)out, ldo, bias, workspace, M, N, K, splits,
                                    max_stages, defer_sum, pf, swiglu, nin, st);
        return run<bf16, true>(x, ldx, W, ldw, (bf16*)out, ldo, bias, workspace, M, N, K, splits, max_stages,
                               defer_sum, pf, swiglu, nin, st);
    }
    if (out_f32)
        return run<float, false>(x, ldx, W, ldw, (float*)out, ldo, bias, workspace, M, N, K, splits,
                                 max_stages, defer_sum, pf, swiglu, nin, st);
    return run<bf16, false>(x, ldx, W, ldw, (bf16*)out, ldo, bias, workspace, M, N, K, splits, max_stages,
                            defer_sum, pf, swiglu, nin, st);
}

// out[M, N] = sum of float32 partial sums [splits][M][N] (+ bias), in order.
int slb_split_sum(const float* parts, void* out, int ldo, const float* bias, int out_f32, int M, int N,
                  int splits, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (splits < 1 || ldo < N || M > 65535) return SLB_ERR_BAD_ARG;
    if (out_f32)
        return slb_launch(gemm_tc_reduce_kernel<float>, dim3((N + 255) / 256, M), dim3(256), 0, st, parts,
                          (float*)out, ldo, bias, M, N, splits);
    return slb_launch(gemm_tc_reduce_kernel<bf16>, dim3((N + 255) / 256, M), dim3(256), 0, st, parts,
                      (bf16*)out, ldo, bias, M, N, splits);
}

// 0 while no wait has timed out; else (role << 8 | code) of the first one.
// Reading synchronises with the device.
int slb_gemm_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tc_status_word, &zero, sizeof(int));
    }
    return v;
}
}
