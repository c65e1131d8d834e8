// Paged prefill attention on the 5th-generation tensor cores (tcgen05), bfloat16,
// head sizes 64 and 128, page sizes that are powers of two from 8.
//
// Work unit: 128 query rows x one kv head; the rows of a request are flattened as
// rho = local_token * g + head_in_group (whole tokens per tile: floor(128 / g) of
// them), so the g query heads of a group share every key/value tile.  Per 64-key
// tile, with both accumulators in tensor memory (TMEM):
//
//   loader warps    TMA tensor copies (128-byte swizzle) of the tile's pages of K (warp 0)
//                   and of V (warp 6) into two-stage shared-memory rings of their own
//                                                          -> k_full[stage], v_full[stage]
//   MMA warp        S = Q.K^T   (tcgen05.mma M=128 N=64,  K=16 x D/16)  -> s_full (scores ready,
//                                                                          keys may be replaced)
//                   O += P.V    (tcgen05.mma M=128 N=D,   K=16 x 4)     -> pv_done (values may
//                                                                          be replaced, O is final)
//   softmax warps   thread r owns row r: tcgen05.ld its 64 scores, mask, running max and
//                   sum in float32 (no shuffles: a row lives in one thread), P as
//                   bfloat16 back into tensor memory (tcgen05.st, over the scores it
//                   came from), where the second MMA reads its A operand  -> p_full
// The scores are double buffered: Q.K^T of the next tile runs while this tile's softmax
// does, and P of a tile never waits for the P.V of the one before.  Every barrier that
// is waited on by parity is one of a pair indexed by the tile's buffer, so that the
// side that signals can never be two phases ahead of the side that waits: the softmax
// warps may finish tile j + 1 before the MMA warp has seen P of tile j (both score
// buffers are filled ahead), and a single "P is ready" barrier would then have wrapped
// past the phase the MMA warp still waits for.
//
// The running maximum is only raised when the tile's maximum exceeds it by more than
// 2^8 (scores are in the base-2 domain); otherwise the stale maximum keeps being used
// (probabilities stay below 256, exact in the float32 sums), so the accumulator in
// TMEM is rescaled rarely.  Two blocks fit on an SM: one does its softmax while the
// other's MMAs run.
//
// Every mbarrier wait is bounded; a role that gives up records a code in the status
// word and leaves its loop; the block then frees its TMEM and returns without a result.
//
// Reference analogue: the torch loop over sequences (servelab/parallel/
// tp_model.py:136-157); masking and softmax follow it (r <= a, optional window).
#include <cuda.h>

#include "common.cuh"
#include "tma_util.cuh"

#if (SLB_HEAD_DIM == 64 || SLB_HEAD_DIM == 128)

namespace {

constexpr int D = SLB_HEAD_DIM;
constexpr int PANELS = D / 64;                 // 64-element (128-byte) column panels
constexpr int BM = 128, BN = 64;
constexpr int THREADS = 224;                   // warp 0 loads keys, 1 issues the MMAs, 2..5 softmax,
                                               // 6 loads values
constexpr int TMEM_COLS = 256;                 // two S buffers at columns 0..127, O at 128..128+D-1
constexpr int S_COL = 0, O_COL = 128;          // S buffer b sits at S_COL + 64 * b
constexpr int Q_BYTES = PANELS * BM * 128;
constexpr int KV_PANEL_BYTES = BN * 128;
constexpr int KV_TILE_BYTES = PANELS * KV_PANEL_BYTES;
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;
constexpr int OFF_V = OFF_K + 2 * KV_TILE_BYTES;
constexpr int OFF_BAR = OFF_V + 2 * KV_TILE_BYTES;
constexpr size_t TC_ATTN_SMEM = OFF_BAR + 128;
constexpr uint32_t SPIN_LIMIT = 1u << 18;     // a poll that suspends takes about 4 us: about a second
constexpr float RESCALE_THRESHOLD = 8.f;       // log2 of the largest probability tolerated

__device__ int tc_attn_status = 0;
// Where bounded waits gave up last, four ints per role (loader, MMA issuer, softmax):
// code, block, key tile, key tiles of the block.
__device__ int tc_attn_where[12] = {0};

__device__ __forceinline__ void gave_up(int* status, int code, int role, int tile, int ntiles) {
    atomicCAS(status, 0, code);
    tc_attn_where[role * 4 + 0] = code;
    tc_attn_where[role * 4 + 1] = (int)blockIdx.x;
    tc_attn_where[role * 4 + 2] = tile;
    tc_attn_where[role * 4 + 3] = ntiles;
}

using slb_tma::tma_load_2d;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
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
// The same wait for hand-overs on the critical path of a tile (scores ready, P ready):
// test_wait does not suspend the thread, so the waiter sees the phase within tens of
// cycles; bounded by SPIN_LIMIT * 64 polls (a poll that does not suspend is ~60 times
// shorter).
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SPIN_LIMIT * 64u; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// Shared-memory matrix descriptor, 128-byte swizzle, rows of 128 bytes in groups of 8
// (1024 bytes).  lbo16: leading byte offset >> 4 (distance of 64-element panels for an
// operand that is contiguous along M/N; unused for K-major operands).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo16) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(lbo16 & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
// same with the A operand in tensor memory (lane = row, 32-bit columns of two bfloat16)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}
// 2^x in one MUFU instruction (exp2f adds a range fix-up around it; the probabilities
// here are rounded to bfloat16 anyway, and -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

__global__ void __launch_bounds__(THREADS, 2) prefill_attention_tc_kernel(
    const bf16* __restrict__ q, int ldq, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int ldo,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_q,
    const int* __restrict__ ctx_len, const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
    int H, int Hkv, int ps, int box_rows, float scale_log2, int window, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    // All barriers come in pairs indexed by tile parity.  s_full[b]: Q.K^T of a tile is done
    // (its scores are ready and its keys may be replaced); pv_done[b]: its P.V is done (its
    // values may be replaced, the accumulator may be rescaled or read).
    uint64_t* k_full = reinterpret_cast<uint64_t*>(smem + OFF_BAR);     // [2]
    uint64_t* v_full = k_full + 2;                                      // [2]
    uint64_t* s_full = v_full + 2;                                      // [2]
    uint64_t* p_full = s_full + 2;                                      // [2], one per score buffer
    uint64_t* pv_done = p_full + 2;                                     // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);

    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are handed out in the order of their linear index: tile by tile from the last
    // (most keys) to the first, all kv heads of a tile together, so that no head's long
    // tiles start late.
    const int kvh = blockIdx.x % Hkv;
    const int tile = (int)(gridDim.x / Hkv) - 1 - (int)(blockIdx.x / Hkv);
    const int s = tile_seq[tile];
    const int row0 = tile_row0[tile];
    const int g = H / Hkv;
    const int q0 = cu_q[s];
    const int qlen = cu_q[s + 1] - q0;
    const int ctx = ctx_len[s];
    const int rows_per_tile = (BM / g) * g;
    const int nrows = min(rows_per_tile, qlen * g - row0);
    const int tok0 = row0 / g;
    const int pos_base = ctx - qlen;
    const int* table = block_table + (size_t)s * max_pages;
    const bool aligned = (smem_u32(smem) & 1023u) == 0;     // the swizzle needs 1024-byte alignment
    if (nrows <= 0 || !aligned) {
        if (!aligned && threadIdx.x == 0) atomicCAS(status, 0, 0x900);
        return;
    }
    const int p_first = pos_base + tok0;
    const int p_last = pos_base + tok0 + (nrows - 1) / g;
    int kbeg = 0;
    if (window > 0) kbeg = max(0, p_first - window + 1) / BN * BN;
    const int kend = p_last + 1;
    const int ntiles = (kend - kbeg + BN - 1) / BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&pv_done[i], 1);
        }
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&p_full[0], 128); mbar_init(&p_full[1], 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // K/V stages start as zeros so that rows no copy fills (absent pages) hold finite values
    for (int i = threadIdx.x; i < 4 * KV_TILE_BYTES / 16; i += THREADS)
        reinterpret_cast<uint4*>(smem + OFF_K)[i] = make_uint4(0, 0, 0, 0);
    // Q tile: the softmax threads copy their rows into the swizzled operand layout
    if (warp >= 2 && warp < 6) {
        const int r = (warp & 3) * 32 + lane;
        unsigned char* qs = smem + OFF_Q;
        if (r < nrows) {
            const int tl = r / g, hg = r - tl * g;
            const bf16* src = q + (size_t)(q0 + tok0 + tl) * ldq + (size_t)(kvh * g + hg) * D;
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint4 v = *reinterpret_cast<const uint4*>(src + c * 8);
                *reinterpret_cast<uint4*>(qs + (c >> 3) * (BM * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = v;
            }
        } else {
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                *reinterpret_cast<uint4*>(qs + (c >> 3) * (BM * 128) + r * 128 + ((c & 7) << 4)) =
                    make_uint4(0, 0, 0, 0);
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 || warp == 6) {
        // ---------------------------------------------------------------- loaders
        // Warp 0 fetches the keys, warp 6 the values, each through its own two-stage ring:
        // the keys of a tile may be replaced when its Q.K^T has run (two softmax periods
        // before the new ones are needed), the values when its P.V has.  Lane b looks up the
        // page of box b, one tile ahead of its use (a dependent global load), and issues the
        // box's copies (a copy costs the issuing warp 60 to 160 cycles: spread over lanes).
        const bool keys = warp == 0;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        unsigned char* ring = smem + (keys ? OFF_K : OFF_V);
        uint64_t* full = keys ? k_full : v_full;
        uint64_t* freed = keys ? s_full : pv_done;
        const int boxes = BN / box_rows;
        const int shift = __ffs(ps) - 1;                  // the launcher only takes powers of two
        auto lookup = [&](int j) {                        // first cache row of this lane's box, or -1
            int row = -1;
            if (lane < boxes && j < ntiles) {
                const int kp = kbeg + j * BN + lane * box_rows;
                if (kp < kend) {
                    const int page = table[kp >> shift];
                    if (page >= 0) row = (page * Hkv + kvh) * ps + (kp & (ps - 1));
                }
            }
            return row;
        };
        int row = lookup(0);
        for (int j = 0; j < ntiles; ++j) {
            const int st = j & 1;
            const int next_row = lookup(j + 1);
            if (!mbar_wait(&freed[st], ((j >> 1) & 1) ^ 1)) {
                if (lane == 0) gave_up(status, keys ? 0x101 : 0x102, 0, j, ntiles);
                break;
            }
            const unsigned got = __ballot_sync(0xffffffffu, row >= 0);
            if (lane == 0) {
                const uint32_t bytes = (uint32_t)__popc(got) * (uint32_t)box_rows * 128u * PANELS;
                if (bytes) mbar_expect_tx(&full[st], bytes); else mbar_arrive(&full[st]);
            }
            __syncwarp();
            if (row >= 0) {
#pragma unroll
                for (int p = 0; p < PANELS; ++p)
                    tma_load_2d(ring + st * KV_TILE_BYTES + p * KV_PANEL_BYTES + lane * box_rows * 128, map,
                                &full[st], p * 64, row);
            }
            row = next_row;
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                      ((uint32_t)(BM >> 4) << 24);
            const uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                      ((uint32_t)(D >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // operand descriptors are built once; a step along K or to another panel adds its
            // byte offset / 16 to the address field
            const uint64_t q_desc = umma_desc(smem_u32(smem + OFF_Q), 1);
            const uint64_t k_desc0 = umma_desc(smem_u32(smem + OFF_K), 1);
            const uint64_t v_desc0 = umma_desc(smem_u32(smem + OFF_V), KV_PANEL_BYTES >> 4);
            constexpr uint64_t STAGE_STEP = KV_TILE_BYTES >> 4;      // to the second stage
            // S = Q.K^T of tile t into score buffer t & 1 (which held the scores and then P of
            // tile t - 2; its P.V has been issued before)
            auto issue_qk = [&](int t) -> bool {
                const int st = t & 1;
                if (!mbar_spin(&k_full[st], (t >> 1) & 1)) { gave_up(status, 0x201, 1, t, ntiles); return false; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int p = 0; p < PANELS; ++p)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)          // 16 elements of D = 32 bytes per step
                        umma_bf16(tmem + S_COL + 64 * st, q_desc + ((p * (BM * 128) + kk * 32) >> 4),
                                  k_desc0 + st * STAGE_STEP + ((p * KV_PANEL_BYTES + kk * 32) >> 4), idesc_qk,
                                  (p > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&s_full[st]);
                return true;
            };
            bool ok = issue_qk(0);
            if (ok && ntiles > 1) ok = issue_qk(1);
            for (int j = 0; j < ntiles && ok; ++j) {
                const int st = j & 1;
                if (!mbar_spin(&p_full[st], (j >> 1) & 1)) { gave_up(status, 0x202, 1, j, ntiles); break; }
                if (!mbar_spin(&v_full[st], (j >> 1) & 1)) { gave_up(status, 0x203, 1, j, ntiles); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)              // 16 keys per step: P 8 columns, V 16 rows
                    umma_bf16_ts(tmem + O_COL, tmem + S_COL + 64 * st + kk * 8,
                                 v_desc0 + st * STAGE_STEP + ((kk * 16 * 128) >> 4), idesc_pv,
                                 (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&pv_done[st]);
                // the scores of tile j + 2 go where P of tile j was: issued after P.V of tile j
                // (the tensor core executes in issue order), while the softmax of j + 1 runs
                if (j + 2 < ntiles) ok = issue_qk(j + 2);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax + epilogue
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pos = r < nrows ? pos_base + tok0 + r / g : -1;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < ntiles && ok; ++j) {
            if (!mbar_spin(&s_full[j & 1], (j >> 1) & 1)) { if (lane == 0) gave_up(status, 0x301, 2, j, ntiles); ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t raw[2][32];
            tmem_ld32(tmem + lane_base + S_COL + 64 * (j & 1), raw[0]);
            tmem_ld32(tmem + lane_base + S_COL + 64 * (j & 1) + 32, raw[1]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int k0 = kbeg + j * BN;
            // raw scores stay unscaled; masked ones become -inf.  A tile that every row of
            // the block sees completely needs no mask (rows of padding compute garbage that
            // is never stored).
            const bool open = k0 + BN - 1 <= p_first && (window <= 0 || p_last - k0 < window);
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one
            if (open) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(raw[h][i]));
            } else {
                const int hi = min(BN, min(kend, pos + 1) - k0);      // visible keys: [lo, hi)
                const int lo = window > 0 ? max(0, pos - window + 1 - k0) : 0;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int c = h * 32 + i;
                        if (!(c >= lo && c < hi)) raw[h][i] = __float_as_uint(-INFINITY);
                        mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(raw[h][i]));
                    }
            }
            const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale_log2;   // scale > 0
            float alpha = 1.f;
            if (mt > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mt != -INFINITY)) {
                alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mt);
                m_ref = mt;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            float sm[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t packed[32];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = fast_exp2(fmaf(__uint_as_float(raw[h][i]), scale_log2, -m_use));
                    const float p1 = fast_exp2(fmaf(__uint_as_float(raw[h][i + 1]), scale_log2, -m_use));
                    sm[(i >> 1) & 3] += p0 + p1;
                    packed[h * 16 + i / 2] = pack2(p0, p1);
                }
            l = l * alpha + ((sm[0] + sm[1]) + (sm[2] + sm[3]));
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // the accumulator is rescaled (rarely): P.V of the previous tile must be done
                if (!mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1)) { if (lane == 0) gave_up(status, 0x302, 2, j, ntiles); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem + lane_base + O_COL + c0, ov);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                    tmem_st32(tmem + lane_base + O_COL + c0, ov);
                }
            }
            // P: 64 bfloat16 = 32 columns, written over the first half of this tile's scores
            tmem_st32(tmem + lane_base + S_COL + 64 * (j & 1), packed);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&p_full[j & 1]);
        }
        if (ok) {
            if (!mbar_wait(&pv_done[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1)) { if (lane == 0) gave_up(status, 0x303, 2, ntiles, ntiles); ok = false; }
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        pdl_launch_dependents();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int tl = r / g, hg = r - tl * g;
        bf16* dst = out + (size_t)(q0 + tok0 + tl) * ldo + (size_t)(kvh * g + hg) * D;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(tmem + lane_base + O_COL + c0, ov);            // warp-wide: every lane takes part
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (ok && r < nrows) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack2(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv);
                    v.y = pack2(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
                    v.z = pack2(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
                    v.w = pack2(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
                    *reinterpret_cast<uint4*>(dst + c0 + i) = v;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS)
                     : "memory");
    }
}

// the cache of one layer as a matrix [pages * kv heads * page size, D]; boxes of box_rows x 64
int make_cache_map(CUtensorMap* map, const void* ptr, long long rows, int box_rows) {
    return slb_tma::make_rows_map(map, ptr, D, rows, box_rows);
}

}  // namespace

extern "C" {

// 1 if the (head size, page size, group size) is taken by the tcgen05 prefill kernel
int slb_prefill_attention_tc_supported(int ps, int group) {
    return ps >= 8 && (ps & (ps - 1)) == 0 && group >= 1 && group <= BM;
}
// query rows per tile for a group of g query heads (whole tokens per tile)
int slb_prefill_attention_tc_tile_rows(int group) { return group >= 1 && group <= BM ? (BM / group) * group : 0; }

// num_pages: pages in k_cache / v_cache ([num_pages][Hkv][ps][D]).
int slb_prefill_attention_tc_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, bf16* out, int ldo,
                                  const int* block_table, int max_pages, const int* cu_q,
                                  const int* ctx_len, const int* tile_seq, const int* tile_row0,
                                  int num_tiles, int H, int Hkv, int ps, int num_pages, float scale,
                                  int window, cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || max_pages <= 0 || num_pages <= 0 || !(scale > 0.f))
        return SLB_ERR_BAD_ARG;
    if (!slb_prefill_attention_tc_supported(ps, H / Hkv)) return SLB_ERR_BAD_ARG;
    if (ldq % 8 || ldo % 8 || ((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) % 16)
        return SLB_ERR_BAD_ARG;
    if ((long long)num_tiles * Hkv > 0x7fffffffll) return SLB_ERR_TOO_LARGE;
    const int box_rows = ps < BN ? ps : BN;
    CUtensorMap map_k, map_v;
    const long long rows = (long long)num_pages * Hkv * ps;
    if (rows > 0x7fffffffll) return SLB_ERR_TOO_LARGE;    // box coordinates are 32-bit
    // (a block-table entry outside [0, num_pages) names rows outside the tensor map: the copy
    // reads zeros there, never memory outside the cache)
    int rc = make_cache_map(&map_k, kc, rows, box_rows);
    if (rc != 0) return rc;
    rc = make_cache_map(&map_v, vc, rows, box_rows);
    if (rc != 0) return rc;
    static unsigned long long configured = 0;              // a bit per device
    rc = slb_configure(&configured, prefill_attention_tc_kernel, TC_ATTN_SMEM);
    if (rc != 0) return rc;
    int* status = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&status, tc_attn_status);
    if (e != cudaSuccess) return (int)e;
    return slb_launch(prefill_attention_tc_kernel, dim3((unsigned)num_tiles * Hkv), dim3(THREADS), TC_ATTN_SMEM, st, q, ldq,
                      map_k, map_v, out, ldo, block_table, max_pages, cu_q, ctx_len, tile_seq, tile_row0, H, Hkv,
                      ps, box_rows, scale * 1.4426950408889634f, window, status);
}

// copies the twelve ints that say where waits gave up last (see tc_attn_where)
int slb_prefill_attention_tc_where(int* out12) {
    return (int)cudaMemcpyFromSymbol(out12, tc_attn_where, 12 * sizeof(int));
}

int slb_prefill_attention_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc_attn_status, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tc_attn_status, &zero, sizeof(int));
    }
    return v;
}
}

#else   // head sizes the tcgen05 kernel does not take

extern "C" {
int slb_prefill_attention_tc_supported(int, int) { return 0; }
int slb_prefill_attention_tc_tile_rows(int) { return 0; }
int slb_prefill_attention_tc_status(int) { return 0; }
int slb_prefill_attention_tc_where(int* out12) {
    for (int i = 0; i < 12; ++i) out12[i] = 0;
    return 0;
}
}

#endif
