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
// with epilogues that finish the result (store; q|k|v rotation and cache write).
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
constexpr int tc_cluster_single_max_tokens = 16;   // up to here the cluster form finishes one token at a time
constexpr int TC_MAX_STAGES = 12;     // the ring is as deep as shared memory allows
constexpr int TC_THREADS = 192;       // warp 0 loader, warp 1 MMA + TMEM, warps 2..5 epilogue
constexpr int TC_TMEM_COLS = 64;
constexpr int TC_MAX_CLUSTER = 8;       // K splits of a row tile that can form one cluster (the portable size)
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
// the same copy with an L2 eviction policy for the lines it brings (createpolicy)
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                                 int c0, int c1, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
          "l"(policy)
        : "memory");
}
// a W tile: streamed once a step
__device__ __forceinline__ void load_w_tile(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, bool evict_first, uint64_t policy) {
    if (evict_first) tma_load_2d_hint(smem_dst, map, bar, c0, c1, policy);
    else tma_load_2d(smem_dst, map, bar, c0, c1);
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

// grid (row tiles of W, K splits).  ntok16: tokens padded to a multiple of 16.
// splits == 1: `out` receives the result (+ bias) in its dtype; otherwise `partial`
// receives float32 [split][M][N].
// The x operand is the z of a product with the residual-and-norm epilogue (EPI_RESID below): every token's result is to be multiplied by
// rstd[tok], from the sums of squares that product left per row tile.  sumsq == null: no scale.
struct RowScale {
    const float* sumsq;                 // [M][tiles]
    int tiles;
    float width;                        // elements of a normed row
    float eps;
};
// rstd[t] = 1 / rms of token t's input row for all M tokens, by four warps (`warp4` 0..3) that a
// named barrier joins afterwards: a warp takes tokens warp4, warp4 + 4, ... (at most 16), its lanes
// the tiles (consecutive in memory), and the loads of eight tokens are issued before the first is
// used: they travel while the product's weight tiles keep the memory busy.  The order of additions
// is fixed.
__device__ __forceinline__ void rows_rstd(const RowScale& rs, int M, int warp4, int lane, float* rstd) {
    // Eight of a warp's tokens at a time (all of a step of up to 32 tokens), and no loop around the
    // loads of a token: loads inside a loop of unknown length are not moved ahead of the previous
    // token's additions, and 16 tokens then took 16 round trips (22 us).
    constexpr int GROUP = 8;
#pragma unroll 1
    for (int j0 = 0; warp4 + 4 * j0 < M; j0 += GROUP) {
        float lo[GROUP], hi[GROUP];                          // tiles lane and lane + 32 of each token
#pragma unroll
        for (int j = 0; j < GROUP; ++j) {
            const int t = warp4 + 4 * (j0 + j);
            const int at = t * rs.tiles + lane;
            lo[j] = (t < M && lane < rs.tiles) ? __ldcg(rs.sumsq + at) : 0.f;
            hi[j] = (t < M && lane + 32 < rs.tiles) ? __ldcg(rs.sumsq + at + 32) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < GROUP; ++j) {
            const int t = warp4 + 4 * (j0 + j);
            if (t >= M) break;                               // (the same for every lane)
            float part = lo[j] + hi[j];
            for (int tile = lane + 64; tile < rs.tiles; tile += 32)    // rows wider than 8,192
                part += __ldcg(rs.sumsq + (size_t)t * rs.tiles + tile);
            const float ss = warp_sum(part);
            if (lane == 0) rstd[t] = 1.0f / sqrtf(ss / rs.width + rs.eps);
        }
    }
}

// four consecutive outputs; dst is 8-byte aligned
__device__ __forceinline__ void store4_bf16(bf16* dst, const float (&o)[4]) {
    uint2 packed;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(o[0], o[1]); packed.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[2], o[3]); packed.y = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint2*>(dst) = packed;
}
// eight consecutive outputs; dst is 16-byte aligned for bfloat16 (32-byte for float)
__device__ __forceinline__ void store8(bf16* dst, const float (&o)[8]) {
    uint4 packed;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(o[0], o[1]); packed.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[2], o[3]); packed.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[4], o[5]); packed.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(o[6], o[7]); packed.w = *reinterpret_cast<uint32_t*>(&h);
    *reinterpret_cast<uint4*>(dst) = packed;
}
__device__ __forceinline__ void store8(float* dst, const float (&o)[8]) {
    *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(o[4], o[5], o[6], o[7]);
}

template <typename TO>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_decode_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    TO* __restrict__ out_all, int ldo, float* __restrict__ partial, const float* __restrict__ bias,
    int M_all, int N, int K, int ntok16, int max_stages, int* __restrict__ status, int swiglu,
    int flags, const RowScale rs_all, int tok_group, const SlbTraceArg tr) {
    __shared__ float rstd_s[TC_MAX_TOK];                    // RowScale: 1 / rms of every token's input row
    // tok_group > 0: the step's tokens in groups of that many (grid z), each block one group --
    // for matrices small enough to be read once per group from the L2 cache, so that a block
    // finishes few tokens however many the step has
    const int tok_base = tok_group > 0 ? (int)blockIdx.z * tok_group : 0;
    const int M = tok_group > 0 ? min(tok_group, M_all - tok_base) : M_all;
    TO* out = out_all != nullptr ? out_all + (size_t)tok_base * ldo : nullptr;
    RowScale rs = rs_all;
    if (rs.sumsq != nullptr) rs.sumsq += (size_t)tok_base * rs.tiles;
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
            mbar_init(&full[s], 1);
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
    if (flags & SLB_FLAG_PDL_EARLY) pdl_launch_dependents();
    const bool tracer = threadIdx.x == 64;                  // lane 0 of the first epilogue warp
    if (tracer) slb_trace_event(tr, 1, SLB_TR_START);

    if (warp == 0) {
        // ------------------------------------------------------------ loader
        // W is written by no kernel, x by the preceding one: the W tiles of the first
        // stages are requested at once, the x tiles after the wait for that kernel.
        if (lane == 0) {
            const uint32_t bytes = A_STAGE_BYTES + (uint32_t)ntok16 * TC_BK * 2;
            const bool w_first = (flags & SLB_FLAG_EVICT_FIRST) != 0;
            const uint64_t w_policy = w_first ? l2_evict_first_policy() : 0;
            const int ahead = min(iters, TC_STAGES);
            for (int i = 0; i < ahead; ++i) {                 // stages are empty at the start
                mbar_expect_tx(&full[i], bytes);
                load_w_tile(a_stage + i * A_STAGE_BYTES, &map_w, &full[i], (kb_begin + i) * TC_BK, n0, w_first, w_policy);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(b_stage + i * B_STAGE_BYTES, &map_x, &full[i], (kb_begin + i) * TC_BK, tok_base);
            for (int i = ahead; i < iters; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&empty[s], ((i / TC_STAGES) & 1) ^ 1)) {
                    atomicCAS(status, 0, (1 << 8) | 1);
                    break;
                }
                mbar_expect_tx(&full[s], bytes);
                const int k = (kb_begin + i) * TC_BK;
                load_w_tile(a_stage + s * A_STAGE_BYTES, &map_w, &full[s], k, n0, w_first, w_policy);
                tma_load_2d(b_stage + s * B_STAGE_BYTES, &map_x, &full[s], k, tok_base);
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
        if (tracer) slb_trace_event(tr, 1, SLB_TR_WAITED);
        const int quarter = warp & 3;                        // TMEM lanes this warp may read
        const bool scaled = rs.sumsq != nullptr;
        if (scaled) {                                        // in the shadow of the main loop
            rows_rstd(rs, M, quarter, lane, rstd_s);
            asm volatile("bar.sync 1, 128;" ::: "memory");               // the four epilogue warps
        }
        const int row = quarter * 32 + lane;                 // row of the tile = row of W
        const int n = n0 + row;
        bool ok = true;
        if (iters > 0) {
            ok = mbar_wait(accum, 0);
            if (!ok) atomicCAS(status, 0, (3 << 8) | 1);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_launch_dependents();
        if (tracer) slb_trace_event(tr, 1, SLB_TR_LOOP_DONE);
        if (swiglu) {
            // W holds gate and up rows alternating in runs of 64, so this tile's rows are 64
            // gates and their 64 ups.  Every warp parks its 32 rows in shared memory (the ring is
            // idle: every tile has arrived and every MMA has run); then a thread takes eight
            // neighbouring outputs of a token, out[tok, tile * 64 + c] = silu(gate_c) * up_c, and
            // stores them with one 16-byte access.  (Before, the two warps that hold the gates wrote
            // every token's value with a 2-byte store of its own: 7.5 us at 64 tokens.)  One K split.
            float* vals = reinterpret_cast<float*>(a_stage);           // [128][ntok16 + 1]
            const int ld = ntok16 + 1;
            for (int c0 = 0; c0 < ntok16; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) vals[row * ld + c0 + j] = __uint_as_float(v[j]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");             // the four epilogue warps
            const int t = (int)threadIdx.x - 64;
            const int c8 = (t & 7) * 8;                                // first of this thread's eight columns
            if (ok) {
                for (int tok = t >> 3; tok < M; tok += 16) {
                    const float rstd = scaled ? rstd_s[tok] : 1.f;
                    float o[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float gt = vals[(c8 + e) * ld + tok] * rstd;
                        const float up = vals[(64 + c8 + e) * ld + tok] * rstd;
                        o[e] = gt / (1.0f + expf(-gt)) * up;
                    }
                    TO* dst = out + (size_t)tok * ldo + (size_t)blockIdx.x * 64 + c8;
                    store8(dst, o);
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
                    const float val = __uint_as_float(v[j]) * (scaled ? rstd_s[tok] : 1.f);   // (partial sums too)
                    if (splits == 1)
                        out[(size_t)tok * ldo + n] = from_float<TO>(val + (bias ? bias[n] : 0.f));
                    else
                        partial[((size_t)split * M_all + tok_base + tok) * N + n] = val;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tracer) slb_trace_event(tr, 1, SLB_TR_END);
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
//   EPI_RESID  the product updates the float32 residual stream and prepares the RMS norm that
//              follows, so that no norm kernel runs: resid[tok, n] += sum + bias[n];
//              z[tok, n] = bfloat16(resid[tok, n] * norm_weight[n]) -- the normed row without its
//              factor 1 / rms, which is one number a token; sumsq[tok][tile] = the sum of squares of
//              the tile's 128 updated values.  The product that consumes z multiplies its result
//              by rstd[tok] = 1 / sqrt(sum over tiles of sumsq / N + eps) in its epilogue
//              (RowScale), because W (z rstd) = rstd (W z).
enum { EPI_STORE = 0, EPI_ROPE = 1, EPI_RESID = 2 };

struct ResidEpilogue {
    float* resid;                       // [M][ld] float32, updated in place
    int ld;
    const float* norm_weight;           // [N]
    bf16* z;                            // [M][ldz]
    int ldz;
    float* sumsq;                       // [M][row tiles]
};


struct RopeEpilogue {
    const float* bias;                  // [N] or null
    const int* positions;               // [M]
    const int* seq_of_token;            // [M]
    const int* block_table;             // [requests][max_pages]
    int max_pages, page_size, num_pages;
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
// The two halves of a cluster barrier that only says "I have read what I needed of your shared
// memory": arriving orders nothing (the values read have been used in arithmetic by then), so the
// block's stores to global memory after it are not waited for -- with a releasing arrival after
// them a block spent up to 4 us at the barrier while the next product's weight fetches kept the
// memory busy.
__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
// ... once `value` exists, i.e. once the remote loads it was computed from have returned: the
// value is first stored (volatile, to a word of this block's own shared memory that nothing
// reads), which needs it in a register, and the arrival follows the store.  Without that the
// compiler may place the arrival before the additions, and a block of the cluster could leave,
// and its shared memory be refilled by the next kernel, under a load in flight.
__device__ __forceinline__ void cluster_arrive_relaxed_after(float value, float* sink) {
    asm volatile("st.volatile.shared.f32 [%0], %1;\n\tbarrier.cluster.arrive.relaxed.aligned;"
                 ::"r"(smem_u32(sink)), "f"(value) : "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t a;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_peer_f32x4(uint32_t local_addr, uint32_t rank) {     // 16-byte aligned
    uint32_t a;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}

// What the q|k|v epilogue needs for element n of token tok besides the sum over the K splits:
// the bias, sine and cosine of the token's rotation, and where the result goes.  None of it
// depends on the product, so a block computes it for its first token while its main loop runs.
struct RopeTarget {
    float bias, sn, cs;
    bf16* dst;                          // null: nothing is stored (beyond N, no page, no cache)
    int other;                          // row of the tile that holds the rotation partner
    bool rotate, first_half;
};
// pos: the token's position; page: its entry of the block table (negative: nothing to write)
__device__ __forceinline__ RopeTarget rope_target(const RopeEpilogue& rope, int tok, int pos, int page, int n,
                                                  int row, int N) {
    RopeTarget t;
    t.bias = 0.f; t.sn = 0.f; t.cs = 1.f; t.dst = nullptr; t.other = row; t.rotate = false; t.first_half = true;
    if (n >= N) return t;
    const int D = rope.D;
    const int half = rope.inv_freq != nullptr ? rope.rotary_dim >> 1 : 0;
    const int j = n / D, e = n - j * D;
    const bool is_v = j >= rope.H + rope.Hkv;
    if (rope.bias) t.bias = rope.bias[n];
    if (!is_v && e < 2 * half) {
        const int i = e < half ? e : e - half;
        sincosf((float)pos * rope.inv_freq[i], &t.sn, &t.cs);
        t.rotate = true;
        t.first_half = e < half;
        t.other = e < half ? row + half : row - half;
    }
    if (j < rope.H) {
        t.dst = rope.q_out + (size_t)tok * rope.ld_q + (size_t)j * D + e;
    } else if (rope.k_cache != nullptr && page >= 0) {
        const int kvh = is_v ? j - rope.H - rope.Hkv : j - rope.H;
        t.dst = (is_v ? rope.v_cache : rope.k_cache) +
                (((size_t)page * rope.Hkv + kvh) * rope.page_size + pos % rope.page_size) * D + e;
    }
    return t;
}

template <int EPI, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_cluster_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    bf16* __restrict__ out_all, int ldo, const float* __restrict__ bias, int M_all, int N, int K, int ntok16,
    int max_stages, int* __restrict__ status, const RopeEpilogue rope_all, const ResidEpilogue res_all,
    const RowScale rs_all, int flags, int tok_group, const SlbTraceArg tr) {
    // tok_group > 0: the step's tokens in groups (grid z), as in gemm_tc_decode_kernel
    const int tok_base = tok_group > 0 ? (int)blockIdx.z * tok_group : 0;
    const int M = tok_group > 0 ? min(tok_group, M_all - tok_base) : M_all;
    bf16* out = out_all != nullptr ? out_all + (size_t)tok_base * ldo : nullptr;
    RopeEpilogue rope = rope_all;
    ResidEpilogue res = res_all;
    RowScale rs = rs_all;
    if (tok_base > 0) {
        if (EPI == EPI_ROPE) {
            rope.positions += tok_base;
            rope.seq_of_token += tok_base;
            rope.q_out += (size_t)tok_base * rope.ld_q;
        }
        if (EPI == EPI_RESID) {
            res.resid += (size_t)tok_base * res.ld;
            res.z += (size_t)tok_base * res.ldz;
            res.sumsq += (size_t)tok_base * gridDim.x;
        }
        if (rs.sumsq != nullptr) rs.sumsq += (size_t)tok_base * rs.tiles;
    }
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
    // Static shared memory is kept to a few hundred bytes on purpose: with the ring's 75 KB a
    // third block (of the kernel after this one) fits on an SM beside two of this kernel only
    // while a block needs less than about 76.5 KB in all, and that third block is what fetches
    // the next product's first weight tiles while this one finishes (a block 3 KB larger cost
    // 9 us a layer).  The rows that the rotation exchanges live in the idle x stages of the ring.
    __shared__ int tok_pos[TC_MAX_TOK], tok_page[TC_MAX_TOK]; // EPI_ROPE: position and cache page of every token
    __shared__ float rstd_s[TC_MAX_TOK];                      // RowScale: 1 / rms of every token's input row
    __shared__ float warp_sq[2][4];                           // EPI_RESID: sums of squares per epilogue warp
    float (*pair_vals)[TC_BM] = reinterpret_cast<float (*)[TC_BM]>(b_stage);         // [2][128]: 1 KB
    float* sink = reinterpret_cast<float*>(b_stage) + 2 * TC_BM;                     // [192] behind them

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
            mbar_init(&full[s], 1);
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
    RopeTarget first_target = {};                            // EPI_ROPE: for token `rank` of this block
    float first_sn[2][4] = {}, first_cs[2][4] = {};          // EPI_ROPE, WIDE: of this warp's first two tokens
    float resid_ahead0 = 0.f, resid_ahead1 = 0.f, norm_w = 0.f, bias_n = 0.f;   // EPI_RESID: fetched while the main loop runs
    // The q|k|v product of a step of few tokens lets its successor, the attention, be scheduled at
    // once: its blocks then look up their pages and request the keys of earlier steps while this
    // product's main loop runs (2.80 -> 2.77 ms a batch-8 step of the 7B shape, 2.66 -> 2.64 at batch
    // 1; from 32 tokens on the same cost 0.02 to 0.05 ms, so the many-token form does not do it).
    if ((flags & SLB_FLAG_PDL_EARLY) || (EPI == EPI_ROPE && !WIDE)) pdl_launch_dependents();
    const bool tracer = threadIdx.x == 64;                  // lane 0 of the first epilogue warp
    constexpr int TRACE_ID = EPI == EPI_ROPE ? 3 : (EPI == EPI_RESID ? 7 : 2);
    if (tracer) slb_trace_event(tr, TRACE_ID, SLB_TR_START);

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t bytes = A_STAGE_BYTES + (uint32_t)ntok16 * TC_BK * 2;
            const bool w_first = (flags & SLB_FLAG_EVICT_FIRST) != 0;
            const uint64_t w_policy = w_first ? l2_evict_first_policy() : 0;
            const int ahead = min(iters, TC_STAGES);
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full[i], bytes);
                load_w_tile(a_stage + i * A_STAGE_BYTES, &map_w, &full[i], (kb_begin + i) * TC_BK, n0, w_first, w_policy);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(b_stage + i * B_STAGE_BYTES, &map_x, &full[i], (kb_begin + i) * TC_BK, tok_base);
            for (int i = ahead; i < iters; ++i) {
                const int s = i % TC_STAGES;
                if (!mbar_wait(&empty[s], ((i / TC_STAGES) & 1) ^ 1)) {
                    atomicCAS(status, 0, (1 << 8) | 2);
                    break;
                }
                mbar_expect_tx(&full[s], bytes);
                const int k = (kb_begin + i) * TC_BK;
                load_w_tile(a_stage + s * A_STAGE_BYTES, &map_w, &full[s], k, n0, w_first, w_policy);
                tma_load_2d(b_stage + s * B_STAGE_BYTES, &map_x, &full[s], k, tok_base);
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
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        if constexpr (EPI == EPI_ROPE) {
            // Before the wait for the preceding kernel, which writes none of this (the step's
            // positions and block tables are in place before its first kernel starts): the
            // positions and cache pages of the step's tokens (one token a thread: dependent loads
            // from global memory, which would otherwise be waited for token by token), then what
            // this block's first token needs.
            const int t = (int)threadIdx.x - 64;
            if (t < M) {
                const int pos = rope.positions[t];
                int page = -1;
                if (rope.k_cache != nullptr) {
                    page = rope.block_table[(size_t)rope.seq_of_token[t] * rope.max_pages + pos / rope.page_size];
                    if (page >= rope.num_pages) {            // outside the cache: not written
                        atomicCAS(status, 0, (5 << 8) | 1);
                        page = -1;
                    }
                }
                tok_pos[t] = pos;
                tok_page[t] = page;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");               // the four epilogue warps
            const int tok0 = (int)cluster_rank();
            if (!WIDE && tok0 < M)
                first_target = rope_target(rope, tok0, tok_pos[tok0], tok_page[tok0], n0 + row, row, N);
            if constexpr (WIDE) {
                // sine and cosine of this warp's first two tokens, for this lane's four rows
                const int half = rope.inv_freq != nullptr ? rope.rotary_dim >> 1 : 0;
                const int n4 = n0 + 4 * lane, e0 = n4 % rope.D;
                if (n4 < N && n4 / rope.D < rope.H + rope.Hkv && e0 < 2 * half) {
                    const float4 fr = *reinterpret_cast<const float4*>(rope.inv_freq + (e0 < half ? e0 : e0 - half));
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int tok = (int)cluster_rank() + (quarter + 4 * u) * (int)cluster_size();
                        if (tok < M)
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                sincosf((float)tok_pos[tok] * (&fr.x)[c], &first_sn[u][c], &first_cs[u][c]);
                    }
                }
            }
        }
        pdl_wait();
        if (tracer) slb_trace_event(tr, TRACE_ID, SLB_TR_WAITED);
        if (rs.sumsq != nullptr) rows_rstd(rs, M, quarter, lane, rstd_s);   // in the shadow of the main loop
        if constexpr (EPI == EPI_RESID && !WIDE) {
            // what this thread's column needs of the first two tokens of this block's share
            const int tok0 = (int)cluster_rank(), tok1 = tok0 + (int)cluster_size();
            if (n0 + row < N) {
                norm_w = res.norm_weight[n0 + row];
                if (bias) bias_n = bias[n0 + row];
                if (tok0 < M) resid_ahead0 = __ldcg(res.resid + (size_t)tok0 * res.ld + n0 + row);
                if (tok1 < M) resid_ahead1 = __ldcg(res.resid + (size_t)tok1 * res.ld + n0 + row);
            }
        }
        bool ok = true;
        if (iters > 0) {
            ok = mbar_wait(accum, 0);
            if (!ok) atomicCAS(status, 0, (3 << 8) | 2);
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_launch_dependents();
        if (tracer) slb_trace_event(tr, TRACE_ID, SLB_TR_LOOP_DONE);
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
    if (tracer) slb_trace_event(tr, TRACE_ID, SLB_TR_END + 1);

    if (warp >= 2) {
        // ------------------------------- epilogue, part 2: this block's share of the tokens
        const int row = (warp & 3) * 32 + lane;
        const int n = n0 + row;
        const uint32_t rank = cluster_rank(), nranks = cluster_size();
        bool arrived = false;
        if constexpr (WIDE) {
            // Steps of more than 16 tokens, where a block finishes up to eight tokens: a warp takes a
            // whole token (a lane four consecutive rows of the tile, fetched from every block with
            // one 16-byte load), the four warps the block's tokens in turn.  The rotation partner
            // and the sum of squares of a token then lie within one warp: shuffles, no barrier.
            // (host: N is a multiple of 4, so a lane's four rows are all inside or all beyond N, and
            // what a lane reads and writes of a row is 8- or 16-byte aligned)
            const int w4 = warp & 3, r4 = 4 * lane, n4 = n0 + r4;
            const bool in = n4 < N;
            float4 nw = make_float4(0.f, 0.f, 0.f, 0.f), bs = nw, fr = nw;
            // the q|k|v form: where this lane's rows lie (the same for every token)
            int rope_j = 0, rope_e0 = 0, partner = lane;
            bool rotate = false, first_half = true, is_v = false;
            if constexpr (EPI == EPI_ROPE) {
                // (host: the width is a multiple of 16 and half the rotary size a multiple of 4, so the
                // four rows lie in one head and on one side of the rotation)
                const int half = rope.inv_freq != nullptr ? rope.rotary_dim >> 1 : 0;
                rope_j = n4 / rope.D;
                rope_e0 = n4 - rope_j * rope.D;
                is_v = rope_j >= rope.H + rope.Hkv;
                rotate = in && !is_v && rope_e0 < 2 * half;
                first_half = rope_e0 < half;
                if (rotate) {
                    partner = first_half ? lane + (half >> 2) : lane - (half >> 2);
                    fr = *reinterpret_cast<const float4*>(rope.inv_freq + (first_half ? rope_e0 : rope_e0 - half));
                }
                if (in && rope.bias) bs = *reinterpret_cast<const float4*>(rope.bias + n4);
            } else if (in) {
                if (EPI == EPI_RESID) nw = *reinterpret_cast<const float4*>(res.norm_weight + n4);
                if (bias) bs = *reinterpret_cast<const float4*>(bias + n4);
            }
            // what is left to do for a token once its sums v[0..3] (rows r4 .. r4 + 3) exist
            auto finish = [&](int tok, float (&v)[4], const float (&before)[4], bool first_turn, int u) {
                if (rs.sumsq != nullptr) {
                    const float rstd = rstd_s[tok];
#pragma unroll
                    for (int c = 0; c < 4; ++c) v[c] *= rstd;
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) v[c] += (&bs.x)[c];
                if constexpr (EPI == EPI_STORE) {
                    if (in) store4_bf16(out + (size_t)tok * ldo + n4, v);
                } else if constexpr (EPI == EPI_RESID) {
                    float sq = 0.f;
                    if (in) {
                        float r[4], zv[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            r[c] = before[c] + v[c];
                            zv[c] = r[c] * (&nw.x)[c];
                            sq += r[c] * r[c];
                        }
                        *reinterpret_cast<float4*>(res.resid + (size_t)tok * res.ld + n4) =
                            make_float4(r[0], r[1], r[2], r[3]);
                        store4_bf16(res.z + (size_t)tok * res.ldz + n4, zv);
                    }
                    sq = warp_sum(sq);
                    if (lane == 0) res.sumsq[(size_t)tok * gridDim.x + blockIdx.x] = sq;
                } else {
                    float other[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) other[c] = __shfl_sync(0xffffffffu, v[c], partner);
                    const int pos = tok_pos[tok], page = tok_page[tok];
                    if (rotate) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            float sn, cs;
                            if (first_turn) {                          // computed before the main loop ended
                                sn = first_sn[u][c];
                                cs = first_cs[u][c];
                            } else {
                                sincosf((float)pos * (&fr.x)[c], &sn, &cs);
                            }
                            v[c] = first_half ? v[c] * cs - other[c] * sn : v[c] * cs + other[c] * sn;
                        }
                    }
                    bf16* dst = nullptr;
                    if (in && rope_j < rope.H) {
                        dst = rope.q_out + (size_t)tok * rope.ld_q + (size_t)rope_j * rope.D + rope_e0;
                    } else if (in && rope.k_cache != nullptr && page >= 0) {
                        const int kvh = is_v ? rope_j - rope.H - rope.Hkv : rope_j - rope.H;
                        dst = (is_v ? rope.v_cache : rope.k_cache) +
                              (((size_t)page * rope.Hkv + kvh) * rope.page_size + pos % rope.page_size) * rope.D +
                              rope_e0;
                    }
                    if (dst != nullptr) store4_bf16(dst, v);
                }
            };
            // two tokens a turn, the remote values (and residual rows) of both requested before
            // either is used: a warp's tokens would otherwise cost a round trip each
            for (int tok = (int)rank + w4 * (int)nranks; tok < M; tok += 8 * (int)nranks) {
                const int tok2 = tok + 4 * (int)nranks;
                float4 part[2][TC_MAX_CLUSTER];
                float before[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int t = u == 0 ? tok : tok2;
                    const bool live = t < M;
                    const uint32_t addr = smem_u32(acc + (live ? t : 0) * TC_BM + r4);
#pragma unroll
                    for (uint32_t p = 0; p < (uint32_t)TC_MAX_CLUSTER; ++p)
                        part[u][p] = (live && p < nranks) ? ld_peer_f32x4(addr, p) : make_float4(0.f, 0.f, 0.f, 0.f);
                    if constexpr (EPI == EPI_RESID)
                        if (live && in) {
                            const float4 b4 = __ldcg(reinterpret_cast<const float4*>(res.resid + (size_t)t * res.ld + n4));
                            before[u][0] = b4.x; before[u][1] = b4.y; before[u][2] = b4.z; before[u][3] = b4.w;
                        }
                }
                float v[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (uint32_t p = 0; p < (uint32_t)TC_MAX_CLUSTER; ++p) {
                        v[u][0] += part[u][p].x; v[u][1] += part[u][p].y;
                        v[u][2] += part[u][p].z; v[u][3] += part[u][p].w;
                    }
                if (tok + 8 * (int)nranks >= M) {            // this warp's last values of other blocks are here
                    cluster_arrive_relaxed_after(((v[0][0] + v[0][1]) + (v[0][2] + v[0][3])) +
                                                     ((v[1][0] + v[1][1]) + (v[1][2] + v[1][3])),
                                                 sink + threadIdx.x);
                    arrived = true;
                }
                const bool first_turn = tok == (int)rank + w4 * (int)nranks;
                finish(tok, v[0], before[0], first_turn, 0);
                if (tok2 < M) finish(tok2, v[1], before[1], first_turn, 1);
            }
        } else {
        int parity = 0, turn = 0;
        for (int tok = (int)rank; tok < M; tok += (int)nranks) {
            // the blocks' values are fetched together and then added in rank order: a loop of
            // load-then-add would wait for every remote load in turn
            const uint32_t addr = smem_u32(acc + tok * TC_BM + row);
            float part[TC_MAX_CLUSTER];
#pragma unroll
            for (uint32_t p = 0; p < (uint32_t)TC_MAX_CLUSTER; ++p) part[p] = p < nranks ? ld_peer_f32(addr, p) : 0.f;
            float sum = 0.f;
#pragma unroll
            for (uint32_t p = 0; p < (uint32_t)TC_MAX_CLUSTER; ++p) sum += part[p];
            if (tok + (int)nranks >= M) {                    // the last values of other blocks are here
                cluster_arrive_relaxed_after(sum, sink + threadIdx.x);
                arrived = true;
            }
            if (rs.sumsq != nullptr) sum *= rstd_s[tok];
            if constexpr (EPI == EPI_STORE) {
                if (n < N) out[(size_t)tok * ldo + n] = __float2bfloat16_rn(sum + (bias ? bias[n] : 0.f));
            } else if constexpr (EPI == EPI_RESID) {
                float r = 0.f;
                if (n < N) {
                    float* dst = res.resid + (size_t)tok * res.ld + n;
                    const float before = turn == 0 ? resid_ahead0 : (turn == 1 ? resid_ahead1 : __ldcg(dst));
                    r = before + (sum + bias_n);
                    *dst = r;
                    res.z[(size_t)tok * res.ldz + n] = __float2bfloat16_rn(r * norm_w);
                }
                ++turn;
                const float sq = warp_sum(r * r);
                if (lane == 0) warp_sq[parity][warp & 3] = sq;
                asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps
                if (row == 0)
                    res.sumsq[(size_t)tok * gridDim.x + blockIdx.x] =
                        ((warp_sq[parity][0] + warp_sq[parity][1]) + warp_sq[parity][2]) + warp_sq[parity][3];
                parity ^= 1;
            } else {
                const RopeTarget t = tok == (int)rank ? first_target
                                                      : rope_target(rope, tok, tok_pos[tok], tok_page[tok], n, row, N);
                float v = sum + t.bias;
                pair_vals[parity][row] = v;
                asm volatile("bar.sync 1, 128;" ::: "memory");           // the four epilogue warps
                if (t.rotate) {
                    const float other = pair_vals[parity][t.other];
                    v = t.first_half ? v * t.cs - other * t.sn : v * t.cs + other * t.sn;
                }
                if (t.dst != nullptr) *t.dst = __float2bfloat16_rn(v);
                parity ^= 1;
            }
        }
        }
        if (!arrived) cluster_arrive_relaxed();              // (a block without a token of its own)
    } else {
        cluster_arrive_relaxed();
    }
    __syncwarp();
    cluster_wait();                                          // no block leaves while its acc is read
    if (tracer) slb_trace_event(tr, TRACE_ID, SLB_TR_END);
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

template <typename TO>
int run(const bf16* x, int ldx, const bf16* W, int ldw, TO* out, int ldo, const float* bias,
        float* workspace, int M, int N, int K, int splits, int max_stages, int defer_sum, int swiglu,
        const RowScale& rs, int tok_group, cudaStream_t st) {
    CUtensorMap map_w, map_x;
    const int Mb = tok_group > 0 ? (M < tok_group ? M : tok_group) : M;      // tokens a block sees
    const int groups = tok_group > 0 ? (M + tok_group - 1) / tok_group : 1;
    const int ntok16 = (Mb + 15) / 16 * 16;
    int rc = make_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc != 0) return rc;
    rc = make_map(&map_x, x, M, K, ldx, ntok16);
    if (rc != 0) return rc;
    static unsigned long long configured = 0;               // per instantiation, a bit per device
    rc = slb_configure(&configured, gemm_tc_decode_kernel<TO>, TC_SMEM_BUDGET);
    if (rc != 0) return rc;
    const size_t TC_SMEM = 1024 + (size_t)stages_for(ntok16, max_stages) * (A_STAGE_BYTES + b_stage_bytes(ntok16)) +
                           TC_SMEM_TAIL;
    int* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&status, tc_status_word);
    if (e != cudaSuccess) return (int)e;
    rc = slb_launch(gemm_tc_decode_kernel<TO>, dim3((N + TC_BM - 1) / TC_BM, splits, groups), dim3(TC_THREADS),
                    TC_SMEM, st, map_w, map_x, out, ldo, workspace, bias, M, N, K, ntok16, max_stages, status,
                    swiglu, slb_kernel_flags, rs, tok_group, slb_trace_arg());
    if (rc != 0 || splits == 1 || defer_sum) return rc;
    return slb_launch(gemm_tc_reduce_kernel<TO>, dim3((N + 255) / 256, M), dim3(256), 0, st,
                      (const float*)workspace, out, ldo, bias, M, N, splits);
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


template <int EPI>
int run_cluster(const bf16* x, int ldx, const bf16* W, int ldw, bf16* out, int ldo, const float* bias,
                int M, int N, int K, int splits, int max_stages, const RopeEpilogue& rope,
                const ResidEpilogue& res, const RowScale& rs, int tok_group, cudaStream_t st) {
    CUtensorMap map_w, map_x;
    const int Mb = tok_group > 0 ? (M < tok_group ? M : tok_group) : M;      // tokens a block sees
    const int groups = tok_group > 0 ? (M + tok_group - 1) / tok_group : 1;
    const int ntok16 = (Mb + 15) / 16 * 16;
    int rc = make_map(&map_w, W, N, K, ldw, TC_BM);
    if (rc != 0) return rc;
    rc = make_map(&map_x, x, M, K, ldx, ntok16);
    if (rc != 0) return rc;
    static unsigned long long configured = 0, configured_wide = 0;   // per instantiation, a bit per device
    // the warp-per-token epilogue: above 16 tokens, where its shapes allow it (see the kernel)
    auto aligned = [](const void* p, int ld, int elem_bytes, int bytes) {
        return p == nullptr || ((uintptr_t)p % bytes == 0 && ((size_t)ld * elem_bytes) % bytes == 0);
    };
    bool wide_ok = N % 4 == 0 && aligned(bias, 0, 4, 16);
    if (EPI == EPI_STORE) wide_ok = wide_ok && aligned(out, ldo, 2, 8);
    if (EPI == EPI_RESID)
        wide_ok = wide_ok && aligned(res.resid, res.ld, 4, 16) && aligned(res.z, res.ldz, 2, 8) &&
                  aligned(res.norm_weight, 0, 4, 16);
    if (EPI == EPI_ROPE)
        wide_ok = wide_ok && N % 16 == 0 && (rope.inv_freq == nullptr || rope.rotary_dim % 8 == 0) &&
                  aligned(rope.bias, 0, 4, 16) && aligned(rope.inv_freq, 0, 4, 16) &&
                  aligned(rope.q_out, rope.ld_q, 2, 8) && aligned(rope.k_cache, 0, 2, 8) &&
                  aligned(rope.v_cache, 0, 2, 8);
    // a thread a row while a block finishes at most two tokens, else a warp a token
    const bool few = (Mb <= tc_cluster_single_max_tokens && (Mb + splits - 1) / splits <= 2) || !wide_ok;
    rc = few ? slb_configure(&configured, gemm_tc_cluster_kernel<EPI, false>, TC_SMEM_BUDGET)
             : slb_configure(&configured_wide, gemm_tc_cluster_kernel<EPI, true>, TC_SMEM_BUDGET);
    if (rc != 0) return rc;
    const int stages = stages_for(ntok16, max_stages);
    // the parked accumulator [ntok16][128] floats lives in the W stages of the ring
    if ((size_t)stages * A_STAGE_BYTES < (size_t)ntok16 * TC_BM * 4) return SLB_ERR_BAD_ARG;
    // ... and the rows that the rotation exchanges (2 x 128 floats) in its x stages
    // and a word a thread (see cluster_arrive_relaxed_after)
    if ((size_t)stages * b_stage_bytes(ntok16) < (2 * TC_BM + TC_THREADS) * sizeof(float)) return SLB_ERR_BAD_ARG;
    const size_t smem = 1024 + (size_t)stages * (A_STAGE_BYTES + b_stage_bytes(ntok16)) + TC_SMEM_TAIL;
    int* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&status, tc_status_word);
    if (e != cudaSuccess) return (int)e;
    if (few)
        return launch_cluster(gemm_tc_cluster_kernel<EPI, false>, dim3((N + TC_BM - 1) / TC_BM, splits, groups),
                              dim3(TC_THREADS), splits, smem, st, map_w, map_x, out, ldo, bias, M, N, K, ntok16,
                              max_stages, status, rope, res, rs, slb_kernel_flags, tok_group, slb_trace_arg());
    return launch_cluster(gemm_tc_cluster_kernel<EPI, true>, dim3((N + TC_BM - 1) / TC_BM, splits, groups),
                          dim3(TC_THREADS), splits, smem, st, map_w, map_x, out, ldo, bias, M, N, K, ntok16,
                          max_stages, status, rope, res, rs, slb_kernel_flags, tok_group, slb_trace_arg());
}

// tok_group: 0, or the tokens a block takes (a multiple of 16 up to 64); the step's tokens are
// then cut into groups of that many
int check_tok_group(int tok_group) {
    return (tok_group < 0 || tok_group % 16 || tok_group > TC_MAX_TOK) ? SLB_ERR_BAD_ARG : 0;
}

int check_cluster_args(const bf16* x, int ldx, const bf16* W, int ldw, int M, int N, int K, int splits,
                       int tok_group) {
    if (K <= 0 || K % 8 || ldw % 8 || ldw < K || (uintptr_t)W % 16) return SLB_ERR_BAD_ARG;
    if (x == nullptr || ldx % 8 || ldx < K || (uintptr_t)x % 16) return SLB_ERR_BAD_ARG;
    if (check_tok_group(tok_group) != 0) return SLB_ERR_BAD_ARG;
    if (M > TC_MAX_TOK) return SLB_ERR_TOO_LARGE;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > kblocks) return SLB_ERR_BAD_ARG;
    if (splits > TC_MAX_CLUSTER) return SLB_ERR_TOO_LARGE;
    return 0;
}

}  // namespace

extern "C" {

// out[M, N] = x . W^T (+ bias), bfloat16, the K splits of a row tile as one cluster (at most 8):
// no workspace, no second kernel.  scale_sumsq: as for slb_gemm_tc_decode_bf16.
int slb_gemm_tc_cluster_bf16(const bf16* x, int ldx, const bf16* W, int ldw, bf16* out, int ldo,
                             const float* bias, int M, int N, int K, int splits, int max_stages,
                             const float* scale_sumsq, int scale_tiles, float scale_eps, int tok_group,
                             cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (ldo < N || out == nullptr) return SLB_ERR_BAD_ARG;
    const int rc = check_cluster_args(x, ldx, W, ldw, M, N, K, splits, tok_group);
    if (rc != 0) return rc;
    if (scale_sumsq != nullptr && scale_tiles <= 0) return SLB_ERR_BAD_ARG;
    const RowScale rs = {scale_sumsq, scale_tiles, (float)K, scale_eps};
    return run_cluster<EPI_STORE>(x, ldx, W, ldw, out, ldo, bias, M, N, K, splits, max_stages, RopeEpilogue{},
                                  ResidEpilogue{}, rs, tok_group, st);
}

// The product that closes a residual branch together with the RMS norm that follows it:
// resid[M, N] (float32) += x . W^T (+ bias); z[M, N] = bfloat16(resid * norm_weight), the normed
// rows without their factor 1 / rms; sumsq[M][row tiles] = per 128-column tile, the sum of squares
// of the updated resid.  The product that reads z passes sumsq on (scale_sumsq below) and multiplies
// its result by 1 / sqrt(sum(sumsq) / N + eps) per token.  sumsq needs (N + 127) / 128 * M floats.
int slb_gemm_tc_resid_norm_bf16(const bf16* x, int ldx, const bf16* W, int ldw, const float* bias,
                                float* resid, int ld_resid, const float* norm_weight, bf16* z, int ldz,
                                float* sumsq, int M, int N, int K, int splits, int max_stages,
                                int tok_group, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (resid == nullptr || norm_weight == nullptr || z == nullptr || sumsq == nullptr || ld_resid < N ||
        ldz < N)
        return SLB_ERR_BAD_ARG;
    const int rc = check_cluster_args(x, ldx, W, ldw, M, N, K, splits, tok_group);
    if (rc != 0) return rc;
    const ResidEpilogue res = {resid, ld_resid, norm_weight, z, ldz, sumsq};
    return run_cluster<EPI_RESID>(x, ldx, W, ldw, nullptr, 0, bias, M, N, K, splits, max_stages, RopeEpilogue{},
                                  res, RowScale{}, tok_group, st);
}

// The q|k|v product of an attention layer with what follows it: W is [(H + 2 Hkv) D, K]
// (q heads, k heads, v heads), and the kernel adds the bias, rotates q and k by
// positions[tok] (angles pos * inv_freq[i], float32), writes q to q_out [M, H D] and k, v to
// the cache slot of the token (block_table[seq_of_token[tok]][pos / page_size]); k_cache ==
// null writes no cache.  num_pages: pages in the cache (a table entry outside [0, num_pages)
// is not written and sets the status word).  Head sizes 16, 32, 64, 128.
int slb_gemm_tc_qkv_rope_bf16(const bf16* x, int ldx, const bf16* W, int ldw, const float* bias,
                              const int* positions, const int* seq_of_token, const int* block_table,
                              int max_pages, int page_size, int num_pages, const float* inv_freq,
                              int rotary_dim, bf16* q_out, int ld_q, bf16* k_cache, bf16* v_cache, int M,
                              int H, int Hkv, int D, int K, int splits, int max_stages,
                              const float* scale_sumsq, int scale_tiles, float scale_eps, int tok_group,
                              cudaStream_t st) {
    if (M <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || D < 16 || D > TC_BM || TC_BM % D || page_size <= 0 || max_pages <= 0)
        return SLB_ERR_BAD_ARG;
    if (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) || ld_q < H * D) return SLB_ERR_BAD_ARG;
    if (positions == nullptr || seq_of_token == nullptr || block_table == nullptr || q_out == nullptr ||
        (k_cache == nullptr) != (v_cache == nullptr) || (k_cache != nullptr && num_pages <= 0))
        return SLB_ERR_BAD_ARG;
    const int N = (H + 2 * Hkv) * D;
    const int rc = check_cluster_args(x, ldx, W, ldw, M, N, K, splits, tok_group);
    if (rc != 0) return rc;
    int* status = nullptr;
    if (cudaGetSymbolAddress((void**)&status, tc_status_word) != cudaSuccess) return SLB_ERR_BAD_ARG;
    RopeEpilogue rope = {bias, positions, seq_of_token, block_table, max_pages, page_size, num_pages, inv_freq,
                         inv_freq != nullptr ? rotary_dim : 0, q_out, ld_q, k_cache, v_cache, H, Hkv, D};
    if (scale_sumsq != nullptr && scale_tiles <= 0) return SLB_ERR_BAD_ARG;
    const RowScale rs = {scale_sumsq, scale_tiles, (float)K, scale_eps};
    return run_cluster<EPI_ROPE>(x, ldx, W, ldw, nullptr, 0, nullptr, M, N, K, splits, max_stages, rope,
                                 ResidEpilogue{}, rs, tok_group, st);
}

// workspace: float32 [splits * M * N] when splits > 1 (may be null otherwise).
// max_stages: cap on the depth of the shared-memory ring (0: as deep as fits).
// scale_sumsq [M][scale_tiles] (or null): x is the z of slb_gemm_tc_resid_norm_bf16, whose rows still
// lack their factor 1 / rms; the result of token t is multiplied by
// 1 / sqrt(sum over tiles of scale_sumsq[t][.] / K + scale_eps) before the bias and the activation.
// defer_sum: with splits > 1, leave the partial sums [splits][M][N] in the workspace
// and launch no reduction (the consumer adds them; `out` and `bias` are unused).
// swiglu: W's rows are gates and ups alternating in runs of 64; out is [M, N / 2] =
// silu(gate) * up (one K split, no bias).
int slb_gemm_tc_decode_bf16(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo,
                            const float* bias, float* workspace, int out_f32, int M, int N, int K,
                            int splits, int max_stages, int defer_sum, int swiglu,
                            const float* scale_sumsq, int scale_tiles, float scale_eps, int tok_group,
                            cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (check_tok_group(tok_group) != 0) return SLB_ERR_BAD_ARG;
    if (K <= 0 || K % 8 || ldw % 8 || ldw < K || (!swiglu && ldo < N)) return SLB_ERR_BAD_ARG;
    if (x == nullptr || ldx % 8 || ldx < K || (uintptr_t)x % 16 || (uintptr_t)W % 16) return SLB_ERR_BAD_ARG;
    if (M > TC_MAX_TOK) return SLB_ERR_TOO_LARGE;
    const int kblocks = (K + TC_BK - 1) / TC_BK;
    if (splits < 1 || splits > kblocks || splits > 65535) return SLB_ERR_BAD_ARG;
    if (splits > 1 && workspace == nullptr) return SLB_ERR_BAD_ARG;
    if (swiglu && (splits != 1 || N % 128 || bias != nullptr || ldo < N / 2)) return SLB_ERR_BAD_ARG;
    // (its outputs are stored eight at a time)
    if (swiglu && (ldo % 8 || (uintptr_t)out % (out_f32 ? 32 : 16))) return SLB_ERR_BAD_ARG;
    // the tile waits in the idle ring: [128][tokens + 1] floats
    if (swiglu && (size_t)stages_for((M + 15) / 16 * 16, max_stages) * A_STAGE_BYTES < (size_t)128 * ((M + 15) / 16 * 16 + 1) * 4)
        return SLB_ERR_BAD_ARG;
    if (scale_sumsq != nullptr && scale_tiles <= 0) return SLB_ERR_BAD_ARG;
    const RowScale rs = {scale_sumsq, scale_tiles, (float)K, scale_eps};
    if (out_f32)
        return run<float>(x, ldx, W, ldw, (float*)out, ldo, bias, workspace, M, N, K, splits, max_stages,
                          defer_sum, swiglu, rs, tok_group, st);
    return run<bf16>(x, ldx, W, ldw, (bf16*)out, ldo, bias, workspace, M, N, K, splits, max_stages, defer_sum,
                     swiglu, rs, tok_group, st);
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

// 0 while no wait has timed out and no page index was out of range; else (role << 8 | code)
// of the first event (role 5: a block-table entry outside the cache).  Reading synchronises
// with the device.
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
