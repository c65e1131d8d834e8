// Tensor-core paged attention for bfloat16, specialised at compile time for one
// head size (SLB_HEAD_DIM, a multiple of 16 up to 256).  Two kernels share their
// tile code:
//
//   prefill  any mix of prompt portions and single tokens.  Work unit: 64 query
//            rows x one kv head, the rows of a request flattened as
//            rho = local_token * g + head_in_group so that the g query heads of
//            a group share every key/value tile.  Four warps own 16 rows each and
//            walk all key tiles (64 keys) with an online softmax.
//   decode   steps of single tokens.  Work unit: (split of the keys, kv head,
//            request); the four warps split each 64-key tile among themselves,
//            the g query heads are the rows of one 16-row MMA tile.  Partial
//            results of the splits (float32 accumulator, running max and sum) go
//            to a scratch buffer and a second kernel combines them.
//
// Keys and values stream through shared memory with cp.async (two stages); scores
// and P.V run on mma.sync.m16n8k16 with float32 accumulation; the softmax is kept
// in float32 (base-2 exponentials of scores pre-multiplied by scale*log2 e).
// Masking: key r is visible to a query at position a iff r <= a and, with a
// window w > 0, a - r < w.  Page layout: [page][kv head][slot][SLB_HEAD_DIM].
//
// Reference analogue: the one-program-per-(sequence, head) Triton decode kernel
// (servelab/attention/triton/paged_attention.py:25-74), which has no tensor-core
// path, no sharing of loads across a group and no split of long contexts, and the
// torch loop that serves prompts (servelab/parallel/tp_model.py:136-157).
#include "common.cuh"
#include "mma_util.cuh"

#ifndef SLB_HEAD_DIM
#error "compile with -DSLB_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = SLB_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16, at most 256");
constexpr int LDS = D + 8;            // shared-memory row stride in elements (16-byte pad)
constexpr int BN = 64;                // keys per tile
constexpr int BM = 64;                // query rows per prefill tile
constexpr int NTHREADS = 128;
constexpr int CHUNKS = D / 8;         // 16-byte chunks per row
constexpr int KSTEPS = D / 16;        // k-steps of Q.K^T
constexpr int NT_O = D / 8;           // 8-wide column tiles of the output
constexpr int STAGE_ELEMS = 2 * BN * LDS;                 // K tile + V tile
constexpr int MAX_SPLITS = 32;
constexpr int DSTAGES = 3;            // key/value tiles buffered by the decode kernel

using namespace slb_mma;

__device__ int attn_status_word = 0;             // 0, or a code of the first wait that gave up

// One 64-key tile of K and V by bulk copies: thread t fetches row t % 64 of K (t < 64)
// or of V (t >= 64) with ONE instruction of D*2 bytes; every thread arrives once on
// `bar` (initialised with a count of NTHREADS), with the bytes it expects if it
// copies.  Rows at or beyond kend and rows whose page is absent are filled with
// zeros by ordinary stores.  Callers make sure all earlier reads of the stage are
// done (a block-wide barrier) before calling.
__device__ __forceinline__ void load_kv_tile_bulk(bf16* Ks, bf16* Vs, uint64_t* bar,
                                                  const bf16* __restrict__ kc,
                                                  const bf16* __restrict__ vc,
                                                  const int* __restrict__ table, int k0, int kend,
                                                  int kvh, int Hkv, int ps, int num_pages) {
    static_assert(NTHREADS == 2 * BN, "one row of K or V per thread");
    const int r = threadIdx.x & (BN - 1);
    const bool is_v = threadIdx.x >= BN;
    const int kp = k0 + r;
    bool ok = kp < kend;
    int page = -1, slot = 0;
    if (ok) {
        const bool pow2 = (ps & (ps - 1)) == 0;
        const int lp = pow2 ? kp >> (__ffs(ps) - 1) : kp / ps;
        slot = pow2 ? kp & (ps - 1) : kp - lp * ps;
        page = table[lp];
        if (page >= num_pages) {                            // outside the cache: read as zeros
            atomicCAS(&attn_status_word, 0, 0x40);
            page = -1;
        }
        ok = page >= 0;
    }
    bf16* dst = (is_v ? Vs : Ks) + r * LDS;
    if (ok) {
        const bf16* src = (is_v ? vc : kc) + (((size_t)page * Hkv + kvh) * ps + slot) * D;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_expect_tx(bar, D * 2);
        bulk_copy_g2s(dst, src, D * 2, bar);
    } else {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
        mbar_arrive(bar);
    }
}

// Issue the loads of one 64-key tile of K and V (keys k0 .. k0+63 of the request).
// Rows at or beyond kend, and rows whose page is absent, are zero-filled.
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ kc,
                                             const bf16* __restrict__ vc,
                                             const int* __restrict__ table, int k0, int kend,
                                             int kvh, int Hkv, int ps, int num_pages) {
    const bool pow2 = (ps & (ps - 1)) == 0;
    const int shift = __ffs(ps) - 1;
    for (int idx = threadIdx.x; idx < BN * CHUNKS; idx += NTHREADS) {
        const int r = idx / CHUNKS, c = idx - r * CHUNKS;
        const int kp = k0 + r;
        bool ok = kp < kend;
        const int lp = pow2 ? kp >> shift : kp / ps;
        const int slot = pow2 ? kp & (ps - 1) : kp - lp * ps;
        int page = -1;
        if (ok) page = table[lp];
        if (page >= num_pages) {                            // outside the cache: read as zeros
            atomicCAS(&attn_status_word, 0, 0x40);
            page = -1;
        }
        ok = ok && page >= 0;
        const size_t off = ok ? (((size_t)page * Hkv + kvh) * ps + slot) * D + c * 8 : 0;
        cp_async16(Ks + r * LDS + c * 8, kc + off, ok);
        cp_async16(Vs + r * LDS + c * 8, vc + off, ok);
    }
}

// The A fragments of a 16-row Q tile (rows at `Qs`, stride LDS), all k-steps.
__device__ __forceinline__ void load_q_frags(unsigned (&qf)[KSTEPS][4], const bf16* Qs) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
        ldmatrix_x4(qf[kk], Qs + (lane & 15) * LDS + kk * 16 + (lane >> 4) * 8);
}

// S[16 x 8*NT] += Q . K^T for NT/2 pairs of 8-key tiles starting at key row `krow`.
template <int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const unsigned (&qf)[KSTEPS][4],
                                        const bf16* Ks, int krow) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
            unsigned b[4];
            ldmatrix_x4(b, Ks + (krow + jp * 16 + (lane >> 4) * 8 + (lane & 7)) * LDS + kk * 16 +
                               ((lane >> 3) & 1) * 8);
            mma_bf16(s[2 * jp], qf[kk], b[0], b[1]);
            mma_bf16(s[2 * jp + 1], qf[kk], b[2], b[3]);
        }
    }
}

// O[16 x D] += P . V for NT/2 k-steps of 16 keys starting at key row `krow`; P comes
// from the score accumulators (already exponentiated).
template <int NT>
__device__ __forceinline__ void pv_tile(float (&o)[NT_O][4], const float (&p)[NT][4],
                                        const bf16* Vs, int krow) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int ks = 0; ks < NT / 2; ++ks) {
        unsigned a[4];
        a[0] = pack_bf16(p[2 * ks][0], p[2 * ks][1]);
        a[1] = pack_bf16(p[2 * ks][2], p[2 * ks][3]);
        a[2] = pack_bf16(p[2 * ks + 1][0], p[2 * ks + 1][1]);
        a[3] = pack_bf16(p[2 * ks + 1][2], p[2 * ks + 1][3]);
#pragma unroll
        for (int np = 0; np < NT_O / 2; ++np) {
            unsigned b[4];
            ldmatrix_x4_trans(b, Vs + (krow + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS +
                                     np * 16 + (lane >> 4) * 8);
            mma_bf16(o[2 * np], a, b[0], b[1]);
            mma_bf16(o[2 * np + 1], a, b[2], b[3]);
        }
    }
}

// Online-softmax update of one thread's two rows (lane/4 and lane/4 + 8) for a
// score tile whose first key sits at position kpos0.  pos_lo / pos_hi are the
// rows' query positions (-1: padding row, sees nothing).  Scores arrive raw and
// leave as probabilities relative to the new running max (kept in the base-2
// domain, i.e. already multiplied by scale*log2 e).  MASKED = false is the fast
// path for tiles every row of the warp sees completely.
template <int NT, bool MASKED>
__device__ __forceinline__ void softmax_tile(float (&s)[NT][4], float (&o)[NT_O][4], float (&m)[2],
                                             float (&l)[2], int kpos0, int kend, int pos_lo,
                                             int pos_hi, int window, float scale_log2) {
    const int tig = threadIdx.x & 3;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (MASKED) {
                const int kp = kpos0 + j * 8 + tig * 2 + (e & 1);
                const int pos = (e < 2) ? pos_lo : pos_hi;
                const bool vis = kp < kend && kp <= pos && (window <= 0 || pos - kp < window);
                if (!vis) s[j][e] = -INFINITY;
            }
            mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        }
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h] * scale_log2);      // scale_log2 > 0
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[h] = exp2f(m[h] - m_use);                            // 0 while nothing was seen
        m[h] = m_new;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            s[j][2 * h] = exp2f(fmaf(s[j][2 * h], scale_log2, -m_use));
            s[j][2 * h + 1] = exp2f(fmaf(s[j][2 * h + 1], scale_log2, -m_use));
            sum += s[j][2 * h] + s[j][2 * h + 1];
        }
        l[h] = l[h] * alpha[h] + sum;                              // partial over this thread's columns
    }
    // the accumulator is rescaled only when some row of the warp got a new max
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int n = 0; n < NT_O; ++n) {
            o[n][0] *= alpha[0];
            o[n][1] *= alpha[0];
            o[n][2] *= alpha[1];
            o[n][3] *= alpha[1];
        }
    }
}

// ------------------------------------------------------------------- prefill
__global__ void __launch_bounds__(NTHREADS) prefill_attention_kernel(
    const bf16* __restrict__ q, int ldq, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
    bf16* __restrict__ out, int ldo, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0, int H, int Hkv, int ps,
    int num_pages, float scale_log2, int window) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_wait();
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [BM][LDS], later the output stage
    bf16* stage0 = Qs + BM * LDS;                          // 2 x (K tile | V tile)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // tiles are listed in position order; the last ones see the most keys, so they are
    // started first, all kv heads of a tile together (blocks start in the order of their
    // linear index)
    const int kvh = blockIdx.x % Hkv;
    const int tile = (int)(gridDim.x / Hkv) - 1 - (int)(blockIdx.x / Hkv);
    const int s = tile_seq[tile];
    const int row0 = tile_row0[tile];
    const int g = H / Hkv;
    const int q0 = cu_q[s];
    const int qlen = cu_q[s + 1] - q0;
    const int ctx = ctx_len[s];
    const int nrows = min(BM, qlen * g - row0);
    if (nrows <= 0) return;
    const int pos_base = ctx - qlen;
    const int* table = block_table + (size_t)s * max_pages;

    // Q tile (rows beyond nrows are zero)
    for (int idx = tid; idx < BM * CHUNKS; idx += NTHREADS) {
        const int r = idx / CHUNKS, c = idx - r * CHUNKS;
        const bool ok = r < nrows;
        const int rho = row0 + (ok ? r : 0);
        const int tl = rho / g, hg = rho - tl * g;
        cp_async16(Qs + r * LDS + c * 8, q + (size_t)(q0 + tl) * ldq + (size_t)(kvh * g + hg) * D + c * 8, ok);
    }
    cp_async_commit();

    const int p_first = pos_base + row0 / g;
    const int p_last = pos_base + (row0 + nrows - 1) / g;
    int kbeg = 0;
    if (window > 0) kbeg = max(0, p_first - window + 1) / BN * BN;
    const int kend = p_last + 1;
    const int ntiles = (kend - kbeg + BN - 1) / BN;

    load_kv_tile(stage0, stage0 + BN * LDS, kc, vc, table, kbeg, kend, kvh, Hkv, ps, num_pages);
    cp_async_commit();

    // this thread's two rows
    const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
    const int pos_lo = r_lo < nrows ? pos_base + (row0 + r_lo) / g : -1;
    const int pos_hi = r_hi < nrows ? pos_base + (row0 + r_hi) / g : -1;
    const int wr_last = min(nrows - 1, warp * 16 + 15);
    const int warp_pos_max = warp * 16 < nrows ? pos_base + (row0 + wr_last) / g : -1;
    const bool warp_rows_full = warp * 16 + 15 < nrows;
    const int warp_pos_min = pos_base + (row0 + warp * 16) / g;

    unsigned qf[KSTEPS][4];
    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int t = 0; t < ntiles; ++t) {
        bf16* Ks = stage0 + (t & 1) * STAGE_ELEMS;
        bf16* Vs = Ks + BN * LDS;
        if (t + 1 < ntiles) {
            bf16* Kn = stage0 + ((t + 1) & 1) * STAGE_ELEMS;
            load_kv_tile(Kn, Kn + BN * LDS, kc, vc, table, kbeg + (t + 1) * BN, kend, kvh, Hkv, ps, num_pages);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (t == 0) load_q_frags(qf, Qs + warp * 16 * LDS);
        const int k0 = kbeg + t * BN;
        if (k0 <= warp_pos_max) {                          // else: every key is in this warp's future
            float sc[BN / 8][4];
            qk_tile<BN / 8>(sc, qf, Ks, 0);
            // all 64 keys visible to all 16 rows of the warp: no mask to evaluate
            const bool open = warp_rows_full && k0 + BN - 1 <= warp_pos_min &&
                              (window <= 0 || warp_pos_max - k0 < window);
            if (open)
                softmax_tile<BN / 8, false>(sc, o, m, l, k0, kend, pos_lo, pos_hi, window, scale_log2);
            else
                softmax_tile<BN / 8, true>(sc, o, m, l, k0, kend, pos_lo, pos_hi, window, scale_log2);
            pv_tile<BN / 8>(o, sc, Vs, 0);
        }
        __syncthreads();                                   // the stage may be refilled next round
    }

    pdl_launch_dependents();
    // normalise, stage the warp's 16 rows in its own Q rows, store 16 bytes at a time
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    const float inv_lo = l[0] > 0.f ? 1.f / l[0] : 0.f;
    const float inv_hi = l[1] > 0.f ? 1.f / l[1] : 0.f;
    bf16* Os = Qs + warp * 16 * LDS;
    __syncwarp();
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<unsigned*>(Os + (lane >> 2) * LDS + col) = pack_bf16(o[n][0] * inv_lo, o[n][1] * inv_lo);
        *reinterpret_cast<unsigned*>(Os + ((lane >> 2) + 8) * LDS + col) = pack_bf16(o[n][2] * inv_hi, o[n][3] * inv_hi);
    }
    __syncwarp();
    for (int idx = lane; idx < 16 * CHUNKS; idx += 32) {
        const int r = idx / CHUNKS, c = idx - r * CHUNKS;
        const int row = warp * 16 + r;
        if (row < nrows) {
            const int rho = row0 + row;
            const int tl = rho / g, hg = rho - tl * g;
            *reinterpret_cast<uint4*>(out + (size_t)(q0 + tl) * ldo + (size_t)(kvh * g + hg) * D + c * 8) =
                *reinterpret_cast<const uint4*>(Os + r * LDS + c * 8);
        }
    }
}

// -------------------------------------------------------------------- decode
// grid (num_splits, Hkv * head_tiles, S); q_len must be 1 for every request.
// Scratch: part_o [S][H][num_splits][D] float32 (unnormalised), part_ml
// [S][H][num_splits][2] float32 (running max in the base-2 domain, running sum).
__global__ void __launch_bounds__(NTHREADS) decode_attention_kernel(
    const bf16* __restrict__ q, int ldq, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
    bf16* __restrict__ out, int ldo, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ ctx_len, float* __restrict__ part_o, float* __restrict__ part_ml,
    int H, int Hkv, int ps, int num_pages, float scale_log2, int window, int num_splits, int head_tiles) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_wait();
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);          // [16][LDS]
    bf16* stage0 = Qs + 16 * LDS;
    float* red_o = reinterpret_cast<float*>(stage0);       // [4][16][D] after the key loop
    __shared__ float red_m[4][16], red_l[4][16];
    __shared__ __align__(8) uint64_t full_bar[DSTAGES];    // a stage's K and V rows have landed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / head_tiles, htile = blockIdx.y - kvh * head_tiles;
    const int s = blockIdx.z;
    const int g = H / Hkv;
    const int h0 = htile * 16;                             // first head of the group in this tile
    const int nrows = min(16, g - h0);
    const int ctx = ctx_len[s];
    const int pos = ctx - 1;
    const int* table = block_table + (size_t)s * max_pages;

    int kbeg = 0;
    if (window > 0) kbeg = max(0, pos - window + 1) / BN * BN;
    const int total_tiles = (ctx - kbeg + BN - 1) / BN;
    const int tiles_per_split = (total_tiles + num_splits - 1) / num_splits;
    const int t_begin = split * tiles_per_split;
    const int t_end = min(total_tiles, t_begin + tiles_per_split);
    const int ntiles = max(0, t_end - t_begin);
    const int kstart = kbeg + t_begin * BN;

    for (int idx = tid; idx < 16 * CHUNKS; idx += NTHREADS) {
        const int r = idx / CHUNKS, c = idx - r * CHUNKS;
        const bool ok = r < nrows;
        cp_async16(Qs + r * LDS + c * 8,
                   q + (size_t)s * ldq + (size_t)(kvh * g + h0 + (ok ? r : 0)) * D + c * 8, ok);
    }
    cp_async_commit();
    if (tid == 0) {
#pragma unroll
        for (int p = 0; p < DSTAGES; ++p) mbar_init(&full_bar[p], NTHREADS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // DSTAGES - 1 tiles are in flight ahead of the one being used
#pragma unroll
    for (int p = 0; p < DSTAGES - 1; ++p) {
        if (p < ntiles) {
            bf16* Kp = stage0 + p * STAGE_ELEMS;
            load_kv_tile_bulk(Kp, Kp + BN * LDS, &full_bar[p], kc, vc, table, kstart + p * BN, ctx,
                              kvh, Hkv, ps, num_pages);
        }
    }
    cp_async_wait<0>();                                     // the Q tile

    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const int pos_lo = r_lo < nrows ? pos : -1;
    const int pos_hi = r_hi < nrows ? pos : -1;
    unsigned qf[KSTEPS][4];
    float o[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    bool ok = true;
    for (int t = 0; t < ntiles; ++t) {
        bf16* Ks = stage0 + (t % DSTAGES) * STAGE_ELEMS;
        bf16* Vs = Ks + BN * LDS;
        const int tn = t + DSTAGES - 1;                      // its stage was freed by round t - 1
        if (tn < ntiles) {
            bf16* Kn = stage0 + (tn % DSTAGES) * STAGE_ELEMS;
            load_kv_tile_bulk(Kn, Kn + BN * LDS, &full_bar[tn % DSTAGES], kc, vc, table,
                              kstart + tn * BN, ctx, kvh, Hkv, ps, num_pages);
        }
        ok = mbar_wait(&full_bar[t % DSTAGES], (t / DSTAGES) & 1);
        if (t == 0) {
            __syncthreads();                                 // Q rows of the other threads
            load_q_frags(qf, Qs);
        }
        const int k0 = kstart + t * BN + warp * 16;         // this warp's 16 keys of the tile
        if (ok && k0 < ctx) {
            float sc[2][4];
            qk_tile<2>(sc, qf, Ks, warp * 16);
            // every key of this warp's 16 is inside the context and the window: no mask
            if (k0 + 15 < ctx && (window <= 0 || pos - k0 < window))
                softmax_tile<2, false>(sc, o, m, l, k0, ctx, pos_lo, pos_hi, window, scale_log2);
            else
                softmax_tile<2, true>(sc, o, m, l, k0, ctx, pos_lo, pos_hi, window, scale_log2);
            pv_tile<2>(o, sc, Vs, warp * 16);
        }
        // the stage may be refilled next round; if any thread's wait gave up, all stop
        if (!__syncthreads_and(ok)) {
            if (tid == 0) atomicCAS(&attn_status_word, 0, 1);
            // copies already requested must not land in memory of a later block: wait
            // for them once more (bounded), then leave without writing a result
            for (int tt = t; tt < min(ntiles, t + DSTAGES); ++tt)
                mbar_wait(&full_bar[tt % DSTAGES], (tt / DSTAGES) & 1);
            // the combine step must not merge what an earlier launch left in these slots:
            // mark this split of every head as empty (maximum -inf, sum 0)
            if (num_splits > 1 && tid < nrows) {
                const size_t pi = ((size_t)s * H + kvh * g + h0 + tid) * num_splits + split;
                part_ml[pi * 2] = -INFINITY;
                part_ml[pi * 2 + 1] = 0.f;
            }
            return;
        }
    }
    __syncthreads();

    pdl_launch_dependents();
    // merge the four warps (each saw a quarter of the keys)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    if ((lane & 3) == 0) {
        red_m[warp][r_lo] = m[0]; red_l[warp][r_lo] = l[0];
        red_m[warp][r_hi] = m[1]; red_l[warp][r_hi] = l[1];
    }
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        float* dst = red_o + ((size_t)warp * 16 + r_lo) * D + col;
        dst[0] = o[n][0]; dst[1] = o[n][1];
        dst[8 * D] = o[n][2]; dst[8 * D + 1] = o[n][3];
    }
    __syncthreads();
    for (int idx = tid; idx < nrows * D; idx += NTHREADS) {
        const int r = idx / D, d = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, red_m[w][r]);
        float L = 0.f, acc = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                if (red_m[w][r] == -INFINITY) continue;
                const float f = exp2f(red_m[w][r] - M);
                L += red_l[w][r] * f;
                acc += red_o[((size_t)w * 16 + r) * D + d] * f;
            }
        }
        const int head = kvh * g + h0 + r;
        if (num_splits == 1) {
            out[(size_t)s * ldo + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t pi = ((size_t)s * H + head) * num_splits + split;
            part_o[pi * D + d] = acc;
            if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
    }
}

// grid (H, S), D threads (rounded up to a warp): combine the splits of one head.
__global__ void decode_combine_kernel(const float* __restrict__ part_o,
                                      const float* __restrict__ part_ml, bf16* __restrict__ out,
                                      int ldo, int H, int num_splits) {
    pdl_launch_dependents();
    pdl_wait();
    const int head = blockIdx.x, s = blockIdx.y, d = threadIdx.x;
    if (d >= D) return;
    const size_t base = ((size_t)s * H + head) * num_splits;
    float M = -INFINITY;
    for (int i = 0; i < num_splits; ++i) M = fmaxf(M, part_ml[(base + i) * 2]);
    float L = 0.f, acc = 0.f;
    if (M != -INFINITY) {
        for (int i = 0; i < num_splits; ++i) {
            const float mi = part_ml[(base + i) * 2];
            if (mi == -INFINITY) continue;
            const float f = exp2f(mi - M);
            L += part_ml[(base + i) * 2 + 1] * f;
            acc += part_o[(base + i) * D + d] * f;
        }
    }
    out[(size_t)s * ldo + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

constexpr size_t PREFILL_SMEM = (size_t)(BM * LDS + 2 * STAGE_ELEMS) * sizeof(bf16);
constexpr size_t DECODE_STAGE_BYTES = (size_t)DSTAGES * STAGE_ELEMS * sizeof(bf16);
constexpr size_t DECODE_RED_BYTES = (size_t)4 * 16 * D * sizeof(float);
constexpr size_t DECODE_SMEM = (size_t)16 * LDS * sizeof(bf16) +
                               (DECODE_STAGE_BYTES > DECODE_RED_BYTES ? DECODE_STAGE_BYTES : DECODE_RED_BYTES);

}  // namespace

SLB_DEFINE_PDL_SWITCH

extern "C" {

int slb_attention_head_dim() { return D; }

// 0 unless a bounded wait inside an attention kernel gave up (the kernel then wrote
// nothing for its block).  Reading synchronises with the device.
int slb_attention_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, attn_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(attn_status_word, &zero, sizeof(int));
    }
    return v;
}
int slb_prefill_attention_tile_rows() { return BM; }
int slb_decode_attention_max_splits() { return MAX_SPLITS; }

// bytes of scratch the decode kernel needs for (S requests, H heads, num_splits)
long long slb_decode_attention_scratch_bytes(int S, int H, int num_splits) {
    if (num_splits <= 1) return 0;
    return (long long)S * H * num_splits * (D + 2) * (long long)sizeof(float);
}

int slb_prefill_attention_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, bf16* out,
                               int ldo, const int* block_table, int max_pages, const int* cu_q,
                               const int* ctx_len, const int* tile_seq, const int* tile_row0,
                               int num_tiles, int H, int Hkv, int ps, int num_pages, float scale,
                               int window, cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || ps <= 0 || max_pages <= 0 || num_pages <= 0 || !(scale > 0.f))
        return SLB_ERR_BAD_ARG;
    if (ldq % 8 || ldo % 8 || ((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)out) % 16)
        return SLB_ERR_BAD_ARG;                            // 16-byte copies
    if ((long long)num_tiles * Hkv > 0x7fffffffll) return SLB_ERR_TOO_LARGE;
    static unsigned long long configured = 0;              // a bit per device
    const int crc = slb_configure(&configured, prefill_attention_kernel, PREFILL_SMEM);
    if (crc != 0) return crc;
    return slb_launch(prefill_attention_kernel, dim3((unsigned)num_tiles * Hkv), dim3(NTHREADS), PREFILL_SMEM, st,
                      q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q, ctx_len, tile_seq,
                      tile_row0, H, Hkv, ps, num_pages, scale * 1.4426950408889634f, window);
}

// scratch: float32 buffer of at least slb_decode_attention_scratch_bytes(...) bytes
// (may be null when num_splits == 1).
int slb_decode_attention_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, bf16* out,
                              int ldo, const int* block_table, int max_pages, const int* ctx_len,
                              float* scratch, int S, int H, int Hkv, int ps, int num_pages,
                              float scale, int window, int num_splits, cudaStream_t st) {
    if (S <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || ps <= 0 || max_pages <= 0 || num_pages <= 0 || !(scale > 0.f))
        return SLB_ERR_BAD_ARG;
    if (num_splits < 1 || (num_splits > 1 && scratch == nullptr)) return SLB_ERR_BAD_ARG;
    if (ldq % 8 || ((uintptr_t)q | (uintptr_t)kc | (uintptr_t)vc) % 16) return SLB_ERR_BAD_ARG;
    if (num_splits > MAX_SPLITS || S > 65535) return SLB_ERR_TOO_LARGE;
    const int g = H / Hkv;
    const int head_tiles = (g + 15) / 16;
    if (Hkv * head_tiles > 65535) return SLB_ERR_TOO_LARGE;
    static unsigned long long configured = 0;              // a bit per device
    const int crc = slb_configure(&configured, decode_attention_kernel, DECODE_SMEM);
    if (crc != 0) return crc;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)S * H * num_splits * D : nullptr;
    const int rc = slb_launch(decode_attention_kernel, dim3(num_splits, Hkv * head_tiles, S),
                              dim3(NTHREADS), DECODE_SMEM, st, q, ldq, kc, vc, out, ldo, block_table,
                              max_pages, ctx_len, part_o, part_ml, H, Hkv, ps, num_pages,
                              scale * 1.4426950408889634f, window, num_splits, head_tiles);
    if (rc != 0 || num_splits == 1) return rc;
    return slb_launch(decode_combine_kernel, dim3(H, S), dim3((D + 31) / 32 * 32), 0, st,
                      (const float*)part_o, (const float*)part_ml, out, ldo, H, num_splits);
}

}  // extern "C"

// --------------------------------------------------------------------------
// The same decode attention for callers that may not allocate (see no_alloc.h).
// --------------------------------------------------------------------------
#include "no_alloc.h"

namespace {

constexpr long long NOALLOC_SCRATCH_BYTES = 4ll << 20;
constexpr int NOALLOC_MAX_DEVICES = 64;

// The scratch lives in the library image.  In host code this name is only a
// handle for the runtime, not an address a kernel could use: the device address
// is looked up per device below.
static __device__ __align__(256) float noalloc_scratch[NOALLOC_SCRATCH_BYTES / sizeof(float)];

float* noalloc_scratch_on_device[NOALLOC_MAX_DEVICES] = {nullptr};

// Device address of the scratch on the current device; looked up on first use.
int noalloc_scratch_address(float** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SLB_ERR_BAD_ARG;
    if (noalloc_scratch_on_device[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return SLB_ERR_BAD_ARG;
        noalloc_scratch_on_device[dev] = p;
    }
    *ptr = noalloc_scratch_on_device[dev];
    return 0;
}

}  // namespace

extern "C" {

long long slb_decode_attention_noalloc_capacity_bytes(void) { return NOALLOC_SCRATCH_BYTES; }

const char* slb_decode_attention_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "success";
        case SLB_ERR_BAD_ARG: return "an argument is not taken (sizes, alignment, or device index)";
        case SLB_ERR_TOO_LARGE:
            return "S * H * num_splits * (head_dim + 2) * 4 bytes exceed the built-in scratch "
                   "(slb_decode_attention_noalloc_capacity_bytes), or a launch dimension is too "
                   "large: use fewer splits or fewer requests per call";
        default: return "CUDA runtime error (the code is a cudaError_t)";
    }
}

int slb_decode_attention_bf16_noalloc(const bf16* q, int ldq, const bf16* kc, const bf16* vc,
                                      bf16* out, int ldo, const int* block_table, int max_pages,
                                      const int* ctx_len, int S, int H, int Hkv, int ps, int num_pages,
                                      float scale, int window, int num_splits, cudaStream_t st) {
    if (S <= 0) return 0;
    if (H <= 0 || num_splits < 1) return SLB_ERR_BAD_ARG;
    if (slb_decode_attention_scratch_bytes(S, H, num_splits) > NOALLOC_SCRATCH_BYTES)
        return SLB_ERR_TOO_LARGE;
    float* scratch = nullptr;
    const int rc = noalloc_scratch_address(&scratch);
    if (rc != 0) return rc;
    return slb_decode_attention_bf16(q, ldq, kc, vc, out, ldo, block_table, max_pages, ctx_len,
                                     scratch, S, H, Hkv, ps, num_pages, scale, window, num_splits, st);
}

}  // extern "C"
