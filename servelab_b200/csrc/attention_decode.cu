// Paged attention for steps of single tokens (bfloat16), specialised at compile
// time for one head size (SLB_HEAD_DIM, a multiple of 16 up to 256).
//
// Work unit: (split of the keys, kv head [x tile of 8 or 16 query heads], request).
// A block has one producer warp and DW consumer warps.  The producer walks the
// block's 64-key tiles, looks the pages up in the block table and fetches each page's
// rows of K and of V as TMA boxes (page rows x 64 elements, 128-byte swizzle) into a
// ring of shared-memory stages: 16 copies of 2 KB a tile at page size 16 and head
// size 128, where row-wise bulk copies needed 128 (a warp issues a copy every ~40 ns,
// which bounded the earlier kernel).  A stage is handed over by an mbarrier that
// counts the bytes ("full") and handed back by one that counts the consumer warps
// ("empty"), so no block-wide barrier sits in the loop.  Every consumer warp takes 16
// keys of a tile and computes the TRANSPOSED problem on mma.sync.m16n8k16:
//
//     S^T[key, head] = K[key, :] . Q^T[:, head]         (M = 16 keys, N = 8 heads)
//     O^T[d,   head] += V^T[d, key] . P^T[key, head]    (M = 16 of D, N = 8 heads)
//
// so the g query heads of a group are the 8-wide N side: a group of up to 8 heads
// wastes nothing (the row-major form pads them to 16 rows), the accumulator is
// half as large, and P^T becomes the B operand of the second product by one
// `movmatrix` per 8 keys.  The softmax is float32 in the base-2 domain with a LAZY
// reference: a head's reference maximum moves only when a score exceeds it by more
// than 2^8 (checked with one warp vote per slice; no shuffles in the steady state),
// which changes nothing in exact arithmetic because numerator and denominator use
// the same reference.  The warps of a block merge through shared memory.  The splits of
// one request merge in one of two ways, both inside the one launch.  With at most eight
// splits the blocks of a request's (kv head, head tile) are a thread-block cluster: each
// parks its merged result in its own shared memory and, after a cluster barrier, block r
// combines a slice of the outputs from all of them through distributed shared memory, in
// the order of the ranks (no scratch, no counter, no round trip through the L2 cache).
// With more splits they write partial results to scratch in global memory and the block
// that arrives last on a per-(request, head tile) counter combines them.
//
// Taken: head sizes that are multiples of 64, page sizes that are powers of two from
// 8 (what a box copy needs); other sizes use the kernel in attention_mma.cu.
//
// Masking: key r is visible to the query at position a = ctx - 1 iff r <= a and,
// with a window w > 0, a - r < w.  Page layout: [page][kv head][slot][SLB_HEAD_DIM].
// Pages hold finite values in every slot (the cache starts as zeros), so a masked key
// may carry any stale row; boxes that are not fetched at all (beyond the context, a
// page already given back by a window, or a table entry outside the cache, which also
// sets the status word) are zero-filled in shared memory.
// Every mbarrier wait is bounded; a wait that gives up sets a status word, the
// block waits (bounded) for its own copies in flight and writes no result.
//
// Reference analogue: the one-program-per-(sequence, head) Triton decode kernel
// (servelab/attention/triton/paged_attention.py:25-74).
#include <cuda.h>

#include "common.cuh"
#include "mma_util.cuh"
#include "tma_util.cuh"

#ifndef SLB_HEAD_DIM
#error "compile with -DSLB_HEAD_DIM=<head size>"
#endif

#if (SLB_HEAD_DIM % 64 == 0)

namespace {

using namespace slb_mma;
using slb_tma::tma_load_3d;

constexpr int D = SLB_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16, at most 256");
constexpr int LDS = D + 8;                 // shared-memory row stride in elements (16-byte pad)
constexpr int CHUNKS = D / 8;              // 16-byte chunks per row
constexpr int KSTEPS = D / 16;             // k-steps of K . Q^T
constexpr int MT = D / 16;                 // 16-row tiles of O^T
constexpr int DW = 4;                      // consumer warps
constexpr int BN = 16 * DW;                // keys per tile
constexpr int NTHREADS = 32 * (DW + 1);
constexpr int PANELS = D / 64;             // 64-element (128-byte) column panels of a tile
constexpr int PANEL_BYTES = BN * 128;
constexpr int TILE_BYTES = PANELS * PANEL_BYTES;           // K or V of one tile, swizzled
constexpr int STAGE_BYTES = 2 * TILE_BYTES;                // K tile + V tile
constexpr int MAX_STAGES = 4;
constexpr int MAX_SPLITS = 64;
constexpr int MAX_CLUSTER_SPLITS = 8;      // splits that can form one cluster (the portable size)
constexpr float LAZY_LOG2 = 8.f;           // the reference moves when exceeded by 2^8

__device__ int dec_status_word = 0;        // 0, or a code of the first wait that gave up (0x10 producer,
                                           // 0x20 consumer) or 0x40: a table entry outside the cache
__device__ int dec_splits_used = 0;        // the most splits any request has used since the last reset

// transpose of an 8x8 matrix of 16-bit elements held one row pair per thread
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

__device__ __forceinline__ void cluster_sync_all_threads() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* mine, uint32_t rank) {
    uint32_t a;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(mine)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

// Offsets inside a stage.  A page's box lands as [panel][row][64 elements]: key row r
// of the tile sits in box r / box_rows at row rr = r % box_rows, and 16-byte chunk c of
// panel p of that row at
//     box * (PANELS * box_rows * 128) + p * (box_rows * 128) + rr * 128 + ((c ^ (rr & 7)) << 4)
// (the 128-byte swizzle of the copy; box_rows is a multiple of 8, so rr & 7 == r & 7).
struct BoxGeometry {
    int box_rows, boxes, box_shift, panel_bytes, box_bytes;
    __device__ __forceinline__ int row_offset(int r) const {
        return (r >> box_shift) * box_bytes + (r & (box_rows - 1)) * 128;
    }
};
__device__ __forceinline__ BoxGeometry box_geometry(int rows) {
    BoxGeometry geo;
    geo.box_rows = rows;
    geo.boxes = BN / rows;
    geo.box_shift = 31 - __clz(rows);                      // rows is a power of two
    geo.panel_bytes = rows * 128;
    geo.box_bytes = PANELS * rows * 128;
    return geo;
}

// One tile's copies, issued by the calling warp.  Lane b handles box b (box_rows keys of
// one page, every panel, in ONE tiled copy each for K and V); `page` is that box's entry
// of the block table.  Boxes that are not fetched are zero-filled by the whole warp with
// ordinary stores; lane 0 arrives on `bar` (count 1) with the bytes of all copies.
__device__ __forceinline__ void produce_tile(unsigned char* Kd, unsigned char* Vd, uint64_t* bar,
                                             const CUtensorMap* map_k, const CUtensorMap* map_v,
                                             int page, int k0, int ctx, int kvh, int Hkv, int ps,
                                             const BoxGeometry& geo, bool evict_first) {
    const int lane = threadIdx.x & 31;
    int row0 = -1;                                         // first cache row of this lane's box
    if (lane < geo.boxes) {
        const int kp = k0 + lane * geo.box_rows;
        if (kp < ctx && page >= 0) row0 = (page * Hkv + kvh) * ps + (kp & (ps - 1));
    }
    const unsigned fetched = __ballot_sync(0xffffffffu, row0 >= 0);
    if (fetched != (1u << geo.boxes) - 1u) {
        for (int b = 0; b < geo.boxes; ++b) {
            if (fetched >> b & 1u) continue;
            for (int i = lane * 16; i < geo.box_bytes; i += 32 * 16) {
                *reinterpret_cast<uint4*>(Kd + b * geo.box_bytes + i) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(Vd + b * geo.box_bytes + i) = make_uint4(0, 0, 0, 0);
            }
        }
        // these rows are overwritten through the async proxy in a later round
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
    }
    if (lane == 0) {
        const uint32_t bytes = (uint32_t)__popc(fetched) * (uint32_t)geo.box_bytes * 2u;
        if (bytes) mbar_arrive_expect_tx(bar, bytes); else mbar_arrive(bar);
    }
    __syncwarp();
    if (row0 >= 0) {
        if (evict_first) {                                 // the cache is streamed once a step
            const uint64_t policy = l2_evict_first_policy();
            slb_tma::tma_load_3d_hint(Kd + lane * geo.box_bytes, map_k, bar, 0, row0, 0, policy);
            slb_tma::tma_load_3d_hint(Vd + lane * geo.box_bytes, map_v, bar, 0, row0, 0, policy);
        } else {
            tma_load_3d(Kd + lane * geo.box_bytes, map_k, bar, 0, row0, 0);
            tma_load_3d(Vd + lane * geo.box_bytes, map_v, bar, 0, row0, 0);
        }
    }
}

// grid (num_splits, Hkv * head_tiles, S); q_len is 1 for every request.  NH: 8-head
// tiles per block.  Scratch (only with num_splits > 1): part_o [S][H][num_splits][D]
// float32 (unnormalised), part_ml [S][H][num_splits][2] (reference max in the base-2
// domain, sum), counters [S][Hkv * head_tiles] ints that are zero between launches.
template <int NH, bool CLUSTER>
__global__ void __launch_bounds__(NTHREADS) decode_attention_ws_kernel(
    const bf16* __restrict__ q, int ldq, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int ldo,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ ctx_len,
    float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters, int H,
    int Hkv, int ps, int box_rows, float scale_log2, int window, int num_splits, int head_tiles,
    int stages, float split_coef, int unsplit_tiles, int num_pages, int flags,
    const SlbTraceArg tr) {
    constexpr int HR = 8 * NH;                             // query heads per block
    constexpr int QCH = (HR * CHUNKS + 32 * DW - 1) / (32 * DW);   // 16-byte chunks of Q a consumer thread moves
    extern __shared__ unsigned char smem_raw[];
    // the swizzle pattern of a box repeats every 1024 bytes of shared-memory address
    unsigned char* stage0 = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    bf16* Qs = reinterpret_cast<bf16*>(stage0 + (size_t)stages * STAGE_BYTES);    // [HR][LDS]
    float* red_o = reinterpret_cast<float*>(stage0);       // [DW][registers][32] after the key loop
    // cluster form: this block's merged result for the other blocks of the cluster to read,
    // behind red_o: [HR][D] unnormalised sums, then [HR][2] (reference maximum, sum)
    float* cl_o = red_o + (size_t)DW * (NH * (D / 16) * 4) * 32;
    float* cl_ml = cl_o + HR * D;
    __shared__ float red_m[DW][HR], red_l[DW][HR];
    __shared__ __align__(8) uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES];
    __shared__ int failed, issued, last_block;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / head_tiles, htile = blockIdx.y - kvh * head_tiles;
    const int s = blockIdx.z;
    const int g = H / Hkv;
    const int h0 = htile * HR;                             // first head of the group in this block
    const int nrows = min(HR, g - h0);

    // context length and block table are written by the host before the step: they may be
    // read before the preceding kernel has finished
    const int ctx = ctx_len[s];
    const int pos = ctx - 1;
    const int* table = block_table + (size_t)s * max_pages;

    int kbeg = 0;
    if (window > 0) kbeg = max(0, pos - window + 1) / BN * BN;
    const int total_tiles = (ctx - kbeg + BN - 1) / BN;
    // How many of the launch's num_splits this request uses: none beyond one while it has
    // few tiles; otherwise about split_coef * sqrt(tiles) tiles per split (the cost of a
    // split grows with the number of splits the last block combines, the cost of a tile
    // with the tiles per split).  Blocks of unused splits leave at once.
    int use_splits = 1;
    if (num_splits > 1 && total_tiles > unsplit_tiles) {
        // (cluster form: combining costs about the same whatever the number of splits, so a request
        // takes as many as the launch has, down to two tiles a split)
        const int least = CLUSTER ? 2 : (int)ceilf(split_coef * sqrtf((float)total_tiles));
        const int per = max(least, (total_tiles + num_splits - 1) / num_splits);
        use_splits = (total_tiles + per - 1) / per;
        if (!CLUSTER && use_splits > 8 && use_splits <= 12) use_splits = 8;   // the last block reads eight at a time
    }
    // Cluster form: the launch's splits come as clusters of `csize` blocks; a request that uses more
    // splits than a cluster has uses several clusters ("groups"), each of which combines its own
    // splits through shared memory and leaves one partial result in global memory; the groups'
    // results are combined slice by slice by whichever block finishes a slice last.
    const int csize = CLUSTER ? min(num_splits, MAX_CLUSTER_SPLITS) : 1;
    if (CLUSTER && use_splits > csize) {
        // several clusters cost about 3 us more than one (partial results through global memory): worth
        // it when a block then has at least four tiles (of about 0.8 us) fewer
        const int per_one = (total_tiles + csize - 1) / csize;
        const int per_many = (total_tiles + use_splits - 1) / use_splits;
        if (per_one - per_many < 4) use_splits = (total_tiles + per_one - 1) / per_one;
    }
    const int group = CLUSTER ? split / csize : 0, crank = CLUSTER ? split - group * csize : 0;
    const int groups_used = CLUSTER ? (use_splits + csize - 1) / csize : 1;
    if (CLUSTER && group >= groups_used) return;           // a whole cluster
    // (in the cluster form every block stays for the cluster's barriers; one beyond the
    // request's splits has no tiles)
    if (!CLUSTER && split >= use_splits) return;
    if (use_splits > 1 && split == 0 && blockIdx.y == 0 && threadIdx.x == 0)
        atomicMax(&dec_splits_used, use_splits);           // what tests read to see that requests were split
    if (CLUSTER && use_splits == 1 && split > 0) return;   // the whole cluster takes this branch or none
    if (flags & SLB_FLAG_PDL_EARLY) pdl_launch_dependents();
    if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_START);
    const int tiles_per_split = (total_tiles + use_splits - 1) / use_splits;
    const int t_begin = split * tiles_per_split;
    const int ntiles = max(0, min(total_tiles, t_begin + tiles_per_split) - t_begin);
    const int kstart = kbeg + t_begin * BN;
    const int kstop = min(ctx, kstart + ntiles * BN);

    if (tid == 0) {
        for (int p = 0; p < stages; ++p) {
            mbar_init(&full_bar[p], 1);
            mbar_init(&empty_bar[p], DW);
        }
        failed = 0;
        issued = 0;
        last_block = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const BoxGeometry geo = box_geometry(box_rows);
    const int ps_shift = __ffs(ps) - 1;                    // the launcher takes powers of two only
    // Block-table entries are read 32 boxes at a time: lane l holds the page of box
    // 32 * group + l of this block's keys.
    auto lookup = [&](int group) {
        const int kp = kstart + (group * 32 + lane) * geo.box_rows;
        int page = kp < kstop ? table[kp >> ps_shift] : -1;
        if (page >= num_pages) {                           // outside the cache: not fetched
            atomicCAS(&dec_status_word, 0, 0x40);
            page = -1;
        }
        return page;
    };
    // The first `stages` tiles are requested by warps 0 .. stages-1 at once (one warp
    // issues a tile's copies in roughly a microsecond); the producer warp takes over from
    // tile `stages` on.
    const int burst = min(stages, ntiles);
    int first_pages = -1;
    if (warp < burst) first_pages = lookup((warp * geo.boxes) >> 5);

    // Only the request's newest key and value are written in this step (by the kernel
    // before this one, into the request's last tile); every earlier tile was written by
    // earlier steps and is requested at once, while that kernel still runs.
    const bool last_tile_in_burst = warp < burst && t_begin + warp == total_tiles - 1;
    auto produce_first = [&]() {
        const int page = __shfl_sync(0xffffffffu, first_pages, (warp * geo.boxes + lane) & 31);
        unsigned char* Kd = stage0 + (size_t)warp * STAGE_BYTES;
        produce_tile(Kd, Kd + TILE_BYTES, &full_bar[warp], &map_k, &map_v, page, kstart + warp * BN, ctx,
                     kvh, Hkv, ps, geo, (flags & SLB_FLAG_EVICT_FIRST) != 0);
    };
    if (warp < burst && !last_tile_in_burst) produce_first();
    pdl_wait();                                            // q and this step's K/V rows
    if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_WAITED);
    if (last_tile_in_burst) produce_first();

    if (warp == DW) {
        // ------------------------------------------------------------ producer
        // the lookup is a dependent global load: entries are fetched one group ahead of use
        if (lane == 0) issued = burst;
        int group = (stages * geo.boxes) >> 5;
        int cur = ntiles > stages ? lookup(group) : -1, nxt = ntiles > stages ? lookup(group + 1) : -1;
        for (int t = stages; t < ntiles; ++t) {
            const int st = t % stages;
            const int box0 = t * geo.boxes;                // index of the tile's first box
            if ((box0 >> 5) != group) {
                group = box0 >> 5;
                cur = nxt;
                nxt = lookup(group + 1);
            }
            const int page = __shfl_sync(0xffffffffu, cur, (box0 + lane) & 31);
            if (!mbar_wait(&empty_bar[st], ((t / stages) - 1) & 1)) {
                if (lane == 0) { atomicCAS(&dec_status_word, 0, 0x10); failed = 1; }
                break;
            }
            unsigned char* Kd = stage0 + (size_t)st * STAGE_BYTES;
            produce_tile(Kd, Kd + TILE_BYTES, &full_bar[st], &map_k, &map_v, page, kstart + t * BN, ctx,
                         kvh, Hkv, ps, geo, (flags & SLB_FLAG_EVICT_FIRST) != 0);
            if (lane == 0) issued = t + 1;
        }
    }

    // per-thread state of a consumer: heads 2t, 2t+1 of each 8-head tile (t = lane & 3)
    float o[NH][MT][4];
    float m_ref[NH][2], l[NH][2];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[nh][mt][e] = 0.f;
        m_ref[nh][0] = m_ref[nh][1] = -INFINITY;
        l[nh][0] = l[nh][1] = 0.f;
    }

    if (warp < DW) {
        // ----------------------------------------------------------- consumers
        // the Q rows of the block's heads, zero for heads beyond the group
        {
            uint4 qv[QCH];
#pragma unroll
            for (int i = 0; i < QCH; ++i) {
                const int idx = tid + i * 32 * DW;
                const int r = idx / CHUNKS, c = idx - r * CHUNKS;
                qv[i] = make_uint4(0, 0, 0, 0);
                if (idx < HR * CHUNKS && r < nrows)
                    qv[i] = *reinterpret_cast<const uint4*>(q + (size_t)s * ldq +
                                                            (size_t)(kvh * g + h0 + r) * D + c * 8);
            }
#pragma unroll
            for (int i = 0; i < QCH; ++i) {
                const int idx = tid + i * 32 * DW;
                const int r = idx / CHUNKS, c = idx - r * CHUNKS;
                if (idx < HR * CHUNKS) *reinterpret_cast<uint4*>(Qs + r * LDS + c * 8) = qv[i];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * DW) : "memory");    // the consumer warps only
        }
        unsigned qf[NH][KSTEPS][2];                        // B fragments of Q^T, all k-steps
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
            for (int kk = 0; kk + 1 < KSTEPS; kk += 2) {
                unsigned r[4];
                ldmatrix_x4(r, Qs + (nh * 8 + (lane & 7)) * LDS + kk * 16 + (lane >> 3) * 8);
                qf[nh][kk][0] = r[0]; qf[nh][kk][1] = r[1];
                qf[nh][kk + 1][0] = r[2]; qf[nh][kk + 1][1] = r[3];
            }
        }
        const int kr = lane >> 2;                          // this thread's keys: kr and kr + 8
        // this lane's ldmatrix rows in the K tile (A operand as stored) and the V tile
        // (A operand transposed), and which 16-byte half of a 16-element column step
        const int k_off = geo.row_offset(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8), k_half = lane >> 4;
        const int v_off = geo.row_offset(warp * 16 + (lane & 7) + (lane >> 4) * 8), v_half = (lane >> 3) & 1;
        const int sw = lane & 7;
        constexpr int VPRE = D <= 128 ? MT : 0;            // V fragments fetched before the softmax
        for (int t = 0; t < ntiles; ++t) {
            const int st = t % stages;
            if (!mbar_wait(&full_bar[st], (t / stages) & 1)) {
                if (lane == 0) { atomicCAS(&dec_status_word, 0, 0x20); failed = 1; }
                break;
            }
            const unsigned char* Ks = stage0 + (size_t)st * STAGE_BYTES;
            const unsigned char* Vs = Ks + TILE_BYTES;
            const int k0 = kstart + t * BN + warp * 16;    // position of this warp's first key
            if (k0 < ctx) {
                // every shared-memory read of the slice is issued before the first MMA needs
                // its result (the asm statements keep their order)
                unsigned ka[KSTEPS][4];
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk)
                    ldmatrix_x4(ka[kk], Ks + (kk >> 2) * geo.panel_bytes + k_off +
                                            ((((kk & 3) * 2 + k_half) ^ sw) << 4));
                unsigned va[VPRE > 0 ? VPRE : 1][4];
#pragma unroll
                for (int mt = 0; mt < VPRE; ++mt)
                    ldmatrix_x4_trans(va[mt], Vs + (mt >> 2) * geo.panel_bytes + v_off +
                                                  ((((mt & 3) * 2 + v_half) ^ sw) << 4));
                // S^T = K . Q^T, four accumulators per head tile: MMA chains two deep
                float sacc[4][NH][4];
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sacc[c][nh][e] = 0.f;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh)
                        mma_bf16(sacc[kk & 3][nh], ka[kk], qf[nh][kk][0], qf[nh][kk][1]);
                }
                const bool open = k0 + 15 < ctx && (window <= 0 || pos - k0 < window);
                float x[NH][4];
                bool grow = false;
#pragma unroll
                for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        x[nh][e] = ((sacc[0][nh][e] + sacc[1][nh][e]) + (sacc[2][nh][e] + sacc[3][nh][e])) * scale_log2;
                        if (!open) {
                            const int kp = k0 + kr + (e >> 1) * 8;
                            const bool vis = kp < ctx && (window <= 0 || pos - kp < window);
                            if (!vis) x[nh][e] = -INFINITY;
                        }
                    }
                    grow |= fmaxf(x[nh][0], x[nh][2]) > m_ref[nh][0] + LAZY_LOG2;
                    grow |= fmaxf(x[nh][1], x[nh][3]) > m_ref[nh][1] + LAZY_LOG2;
                }
                if (__any_sync(0xffffffffu, grow)) {
                    // move the references of all heads to the exact maxima seen so far
#pragma unroll
                    for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float mx = fmaxf(x[nh][h], x[nh][h + 2]);
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                            const float m_new = fmaxf(m_ref[nh][h], mx);
                            // nothing seen before: the accumulators are zero, any factor will do
                            const float alpha = m_ref[nh][h] == -INFINITY ? 1.f : exp2f(m_ref[nh][h] - m_new);
                            m_ref[nh][h] = m_new;
                            l[nh][h] *= alpha;
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                o[nh][mt][h] *= alpha;
                                o[nh][mt][h + 2] *= alpha;
                            }
                        }
                    }
                }
                unsigned pb[NH][2];                        // B fragments of P^T
#pragma unroll
                for (int nh = 0; nh < NH; ++nh) {
                    const float u0 = m_ref[nh][0] == -INFINITY ? 0.f : m_ref[nh][0];
                    const float u1 = m_ref[nh][1] == -INFINITY ? 0.f : m_ref[nh][1];
                    const float p0 = exp2f(x[nh][0] - u0), p1 = exp2f(x[nh][1] - u1);
                    const float p2 = exp2f(x[nh][2] - u0), p3 = exp2f(x[nh][3] - u1);
                    l[nh][0] += p0 + p2;
                    l[nh][1] += p1 + p3;
                    pb[nh][0] = movmatrix_trans(pack_bf16(p0, p1));
                    pb[nh][1] = movmatrix_trans(pack_bf16(p2, p3));
                }
                // O^T += V^T . P^T
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (mt < VPRE) {
#pragma unroll
                        for (int nh = 0; nh < NH; ++nh) mma_bf16(o[nh][mt], va[mt], pb[nh][0], pb[nh][1]);
                    } else {
                        unsigned a[4];
                        ldmatrix_x4_trans(a, Vs + (mt >> 2) * geo.panel_bytes + v_off +
                                                 ((((mt & 3) * 2 + v_half) ^ sw) << 4));
#pragma unroll
                        for (int nh = 0; nh < NH; ++nh) mma_bf16(o[nh][mt], a, pb[nh][0], pb[nh][1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[st]);    // the producer may refill the stage
        }
    }
    __syncthreads();
    pdl_launch_dependents();
    if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_LOOP_DONE);

    const bool bad = failed != 0;
    if (bad) {
        // copies already requested must not land in the shared memory of a later block
        if (tid == 0)
            for (int tt = max(0, issued - stages); tt < issued; ++tt)
                mbar_wait(&full_bar[tt % stages], (tt / stages) & 1);
        __syncthreads();
        if (CLUSTER && tid < HR) {                         // this split counts as empty
            cl_ml[tid * 2] = -INFINITY;
            cl_ml[tid * 2 + 1] = 0.f;
        }
    } else {
        // ---- merge the consumer warps (each saw a quarter of the keys) ----
        // Every warp holds the same fragment of O^T for its own keys: the fragments are
        // exchanged in register order (conflict-free), then warp w sums registers
        // [w * RPW, (w + 1) * RPW) of the four warps and stores its part of the result.
        constexpr int R = NH * MT * 4;                     // accumulator registers of a thread
        constexpr int RPW = R / DW;                        // registers a warp reduces
        static_assert(R % DW == 0 && (MT * 4) % RPW == 0, "a warp's registers belong to one head tile");
        if (warp < DW) {
#pragma unroll
            for (int nh = 0; nh < NH; ++nh) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float v = l[nh][h];
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 16);
                    if (lane < 4) {
                        red_m[warp][nh * 8 + lane * 2 + h] = m_ref[nh][h];
                        red_l[warp][nh * 8 + lane * 2 + h] = v;
                    }
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        red_o[((size_t)warp * R + (nh * MT + mt) * 4 + e) * 32 + lane] = o[nh][mt][e];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(32 * DW) : "memory");    // the consumer warps only
            const int nh = warp * RPW / (MT * 4);          // the head tile of this warp's registers
            float f[DW][2], L[2];
            bool any[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int hr = nh * 8 + (lane & 3) * 2 + h;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < DW; ++w) M = fmaxf(M, red_m[w][hr]);
                any[h] = M != -INFINITY;
                L[h] = 0.f;
#pragma unroll
                for (int w = 0; w < DW; ++w) {
                    f[w][h] = (any[h] && red_m[w][hr] != -INFINITY) ? exp2f(red_m[w][hr] - M) : 0.f;
                    L[h] += red_l[w][hr] * f[w][h];
                }
                const int head = kvh * g + h0 + hr;
                if (use_splits > 1 && hr < nrows && (warp * RPW) % (MT * 4) == 0 && lane < 4) {
                    if (CLUSTER) {
                        cl_ml[hr * 2] = M;
                        cl_ml[hr * 2 + 1] = L[h];
                    } else {
                        const size_t pi = ((size_t)s * H + head) * num_splits + split;
                        part_ml[pi * 2] = M;
                        part_ml[pi * 2 + 1] = L[h];
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < RPW; ++i) {
                const int reg = warp * RPW + i;            // (nh * MT + mt) * 4 + e
                const int e = reg & 3, mt = (reg >> 2) % MT, h = e & 1;
                float acc = 0.f;
#pragma unroll
                for (int w = 0; w < DW; ++w) acc += red_o[((size_t)w * R + reg) * 32 + lane] * f[w][h];
                const int hr = nh * 8 + (lane & 3) * 2 + h;
                const int d = mt * 16 + (lane >> 2) + (e >> 1) * 8;
                if (hr < nrows) {
                    const int head = kvh * g + h0 + hr;
                    if (use_splits == 1) {
                        out[(size_t)s * ldo + (size_t)head * D + d] =
                            __float2bfloat16_rn(L[h] > 0.f ? acc / L[h] : 0.f);
                    } else if (CLUSTER) {
                        cl_o[hr * D + d] = acc;
                    } else {
                        part_o[(((size_t)s * H + head) * num_splits + split) * D + d] = acc;
                    }
                }
            }
        }
    }
    if (use_splits == 1) {
        if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_END);
        return;
    }

    if constexpr (CLUSTER) {
        // ---- the blocks of the cluster combine a slice of the outputs each ----
        cluster_sync_all_threads();                        // every block's result is parked
        // (every block of the cluster takes a slice, also one beyond the request's splits, which has
        // parked an empty result: the slices are then the same in every group)
        const int total = nrows * D;
        const int chunk = (total + csize - 1) / csize;
        const int begin = crank * chunk, stop = min(total, (crank + 1) * chunk);
        const bool several = groups_used > 1;
        {
            for (int idx = begin + tid; idx < stop; idx += NTHREADS) {
                const int r = idx / D, d = idx - r * D;
                // all remote loads first, then the merge in the order of the ranks
                float mv[8], lv[8], ov[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const bool in = j < csize;
                    mv[j] = in ? ld_cluster_f32(cl_ml + r * 2, (uint32_t)j) : -INFINITY;
                    lv[j] = in ? ld_cluster_f32(cl_ml + r * 2 + 1, (uint32_t)j) : 0.f;
                    ov[j] = in ? ld_cluster_f32(cl_o + r * D + d, (uint32_t)j) : 0.f;
                }
                float M = -INFINITY, touched = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    M = fmaxf(M, mv[j]);
                    touched += lv[j] + ov[j];              // (every loaded value, also of empty splits)
                }
                float L = 0.f, acc = 0.f;
                if (M != -INFINITY) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (mv[j] == -INFINITY) continue;  // an empty split
                        const float f = exp2f(mv[j] - M);
                        L += lv[j] * f;
                        acc += ov[j] * f;
                    }
                }
                const int head = kvh * g + h0 + r;
                if (!several) {
                    out[(size_t)s * ldo + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
                } else {
                    // this group's partial result; its (maximum, sum) once per row and slice
                    part_o[(((size_t)s * H + head) * num_splits + group) * D + d] = acc;
                    if (d == 0 || idx == begin) {
                        const size_t pi = ((size_t)s * H + head) * num_splits + group * csize + crank;
                        part_ml[pi * 2] = M;
                        part_ml[pi * 2 + 1] = L;
                    }
                }
                // what was read has arrived once this store has its operand (see below)
                asm volatile("st.volatile.shared.f32 [%0], %1;" ::"r"(smem_u32(red_o + tid)), "f"(touched + M) : "memory");
            }
        }
        // A relaxed arrival: it orders nothing, so the stores above are not waited for (with a
        // releasing one a block spent microseconds here while the next product's weight fetches kept
        // the memory busy).  What was read from the other blocks has arrived: every loaded value went
        // into a volatile store to this block's own idle shared memory (red_o), which needs it in a
        // register, and the arrival follows those stores.
        asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
                                                           // nobody leaves while its result is read
        if (!several) {
            if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_END + 1);
            return;
        }
        // ---- several groups: the block that finishes slice `crank` last combines it ----
        __threadfence();
        __syncthreads();
        int* counter = counters + ((size_t)s * gridDim.y + blockIdx.y) * MAX_CLUSTER_SPLITS + crank;
        if (tid == 0) {
            int before;
            asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(before) : "l"(counter) : "memory");
            last_block = before == groups_used - 1;
            if (last_block) *counter = 0;                  // zero again for the next launch
        }
        __syncthreads();
        if (!last_block) {
            if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_END);
            return;
        }
        for (int idx = begin + tid; idx < stop; idx += NTHREADS) {
            const int r = idx / D, d = idx - r * D;
            const int head = kvh * g + h0 + r;
            const size_t base = ((size_t)s * H + head) * num_splits;
            float mv[MAX_SPLITS / MAX_CLUSTER_SPLITS], lv[MAX_SPLITS / MAX_CLUSTER_SPLITS],
                ov[MAX_SPLITS / MAX_CLUSTER_SPLITS];
#pragma unroll
            for (int j = 0; j < MAX_SPLITS / MAX_CLUSTER_SPLITS; ++j) {
                const bool in = j < groups_used;
                // the slice of group j that holds (r, d) wrote this row's maximum and sum
                const size_t pi = base + j * csize + crank;
                mv[j] = in ? __ldcg(part_ml + pi * 2) : -INFINITY;
                lv[j] = in ? __ldcg(part_ml + pi * 2 + 1) : 0.f;
                ov[j] = in ? __ldcg(part_o + (base + j) * D + d) : 0.f;
            }
            float M = -INFINITY;
#pragma unroll
            for (int j = 0; j < MAX_SPLITS / MAX_CLUSTER_SPLITS; ++j) M = fmaxf(M, mv[j]);
            float L = 0.f, acc = 0.f;
            if (M != -INFINITY) {
#pragma unroll
                for (int j = 0; j < MAX_SPLITS / MAX_CLUSTER_SPLITS; ++j) {
                    if (mv[j] == -INFINITY) continue;
                    const float f = exp2f(mv[j] - M);
                    L += lv[j] * f;
                    acc += ov[j] * f;
                }
            }
            out[(size_t)s * ldo + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        }
        if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_END + 1);
        return;
    }

    // ---- the block that arrives last combines the splits ----
    // The block barrier orders every thread's partial results before thread 0's release
    // on the counter; the last arrival acquires all earlier releases through the same
    // counter, and the second barrier hands that view to the block's other threads.
    __syncthreads();
    int* counter = counters + (size_t)s * gridDim.y + blockIdx.y;
    if (tid == 0) {
        int before;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(before) : "l"(counter) : "memory");
        last_block = before == use_splits - 1;
        if (last_block) *counter = 0;                      // zero again for the next launch
    }
    __syncthreads();
    if (!last_block) {
        if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_END);
        return;
    }
    for (int idx = tid; idx < nrows * D; idx += NTHREADS) {
        const int r = idx / D, d = idx - r * D;
        const int head = kvh * g + h0 + r;
        const size_t base = ((size_t)s * H + head) * num_splits;
        // one pass, eight splits' loads in flight together (they come from the L2); the
        // running reference moves as in the online softmax
        float M = -INFINITY, L = 0.f, acc = 0.f;
        for (int i0 = 0; i0 < use_splits; i0 += 8) {
            float mv[8], lv[8], ov[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool in = i0 + j < use_splits;
                mv[j] = in ? __ldcg(part_ml + (base + i0 + j) * 2) : -INFINITY;
                lv[j] = in ? __ldcg(part_ml + (base + i0 + j) * 2 + 1) : 0.f;
                ov[j] = in ? __ldcg(part_o + (base + i0 + j) * D + d) : 0.f;
            }
            float Mb = M;
#pragma unroll
            for (int j = 0; j < 8; ++j) Mb = fmaxf(Mb, mv[j]);
            if (Mb == -INFINITY) continue;                 // nothing seen so far
            const float keep = M == -INFINITY ? 0.f : exp2f(M - Mb);
            L *= keep;
            acc *= keep;
            M = Mb;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (mv[j] == -INFINITY) continue;          // an empty split: its sums are not read
                const float f = exp2f(mv[j] - M);
                L += lv[j] * f;
                acc += ov[j] * f;
            }
        }
        out[(size_t)s * ldo + (size_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    if (threadIdx.x == 0) slb_trace_event(tr, 4, SLB_TR_END + 1);     // end of a block that combined
}

// dynamic shared memory: 1024 bytes of slack for the alignment, the stages, the Q rows
constexpr size_t decode_smem(int nh, int stages) {
    return 1024 + (size_t)stages * STAGE_BYTES + (size_t)8 * nh * LDS * sizeof(bf16);
}
constexpr size_t MAX_DYNAMIC_SMEM = 220 * 1024;            // of the 227 KB a block may have
static_assert(decode_smem(2, 2) <= MAX_DYNAMIC_SMEM, "two stages must fit for every head size");
static_assert(((size_t)DW * 2 * (D / 16) * 4 * 32 + 16 * D + 16 * 2) * sizeof(float) <= 2 * (size_t)STAGE_BYTES,
              "the merge buffer and the parked result live in the first two stages");

template <int NH, bool CLUSTER>
int launch_decode(const bf16* q, int ldq, const CUtensorMap& map_k, const CUtensorMap& map_v, bf16* out,
                  int ldo, const int* block_table, int max_pages, const int* ctx_len, float* scratch,
                  int* counters, int S, int H, int Hkv, int ps, int box_rows, float scale, int window,
                  int num_splits, int stages, float split_coef, int unsplit_tiles, int num_pages,
                  cudaStream_t st) {
    const int g = H / Hkv;
    const int head_tiles = (g + 8 * NH - 1) / (8 * NH);
    if ((long long)Hkv * head_tiles > 65535) return SLB_ERR_TOO_LARGE;
    while (stages > 2 && decode_smem(NH, stages) > MAX_DYNAMIC_SMEM) --stages;
    const size_t smem = decode_smem(NH, stages);
    static unsigned long long configured = 0;              // per instantiation, a bit per device
    const int rc = slb_configure(&configured, decode_attention_ws_kernel<NH, CLUSTER>, MAX_DYNAMIC_SMEM);
    if (rc != 0) return rc;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)S * H * num_splits * D : nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(num_splits, Hkv * head_tiles, S);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (CLUSTER) {                                         // (up to eight of) the splits of a (request, head tile)
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = (unsigned)(num_splits < MAX_CLUSTER_SPLITS ? num_splits : MAX_CLUSTER_SPLITS);
        attr[nattr].val.clusterDim.y = 1;
        attr[nattr].val.clusterDim.z = 1;
        ++nattr;
    }
    if (slb_pdl_enabled) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    return (int)cudaLaunchKernelEx(&cfg, decode_attention_ws_kernel<NH, CLUSTER>, q, ldq, map_k, map_v, out,
                                   ldo, block_table, max_pages, ctx_len, part_o, part_ml, counters, H, Hkv, ps,
                                   box_rows, scale * 1.4426950408889634f, window, num_splits, head_tiles,
                                   stages, split_coef, unsplit_tiles, num_pages, slb_kernel_flags,
                                   slb_trace_arg());
}

}  // namespace

extern "C" {

// 1 if the kernel takes this page size (the head size is fixed by the library)
int slb_decode_attention_ws_supported(int ps) { return ps >= 8 && (ps & (ps - 1)) == 0; }

// 0 unless a bounded wait inside the kernel gave up (its block then wrote nothing) or a
// block-table entry pointed outside the cache (0x40; that page was read as zeros).
// Reading synchronises with the device.
int slb_decode_attention_ws_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, dec_status_word, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(dec_status_word, &zero, sizeof(int));
    }
    return v;
}
// The most splits any request has used in a launch since the last reset (0: every request
// ran unsplit).  Reading synchronises with the device.
int slb_decode_attention_ws_splits_used(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, dec_splits_used, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(dec_splits_used, &zero, sizeof(int));
    }
    return v;
}
int slb_decode_attention_ws_max_splits() { return MAX_SPLITS; }
int slb_decode_attention_ws_max_cluster_splits() { return MAX_CLUSTER_SPLITS; }
int slb_decode_attention_ws_tile_keys() { return BN; }

// float32 scratch for the partial results of (S requests, H heads, num_splits)
long long slb_decode_attention_ws_scratch_bytes(int S, int H, int num_splits) {
    if (num_splits <= 1) return 0;
    return (long long)S * H * num_splits * (D + 2) * (long long)sizeof(float);
}
// ints of the arrival counters (zero before the first launch; every launch leaves
// them zero) for S requests
long long slb_decode_attention_ws_counters(int S, int H, int Hkv) {
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0) return 0;
    const int g = H / Hkv;
    const int hr = g <= 8 ? 8 : 16;
    return (long long)S * Hkv * ((g + hr - 1) / hr) * MAX_CLUSTER_SPLITS;      // (one per slice in the cluster form)
}

// scratch and counters may be null when num_splits == 1.  num_pages: pages in k_cache /
// v_cache ([num_pages][Hkv][ps][D]).  stages: depth of the shared-memory ring, 2..4.
// num_splits is the most any request is split; a request of T 64-key tiles uses one split
// while T <= unsplit_tiles, else ceil(T / max(ceil(split_coef * sqrt(T)), ceil(T /
// num_splits))) of them (8 instead of 9..12); in the cluster form ceil(T / max(2, ceil(T /
// num_splits))).
int slb_decode_attention_ws_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc, bf16* out,
                                 int ldo, const int* block_table, int max_pages, const int* ctx_len,
                                 float* scratch, int* counters, int S, int H, int Hkv, int ps,
                                 int num_pages, float scale, int window, int num_splits, int stages,
                                 float split_coef, int unsplit_tiles, int cluster, cudaStream_t st) {
    if (S <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || max_pages <= 0 || num_pages <= 0 || !(scale > 0.f))
        return SLB_ERR_BAD_ARG;
    if (!slb_decode_attention_ws_supported(ps)) return SLB_ERR_BAD_ARG;
    // cluster != 0: the splits of a request combine through the shared memory of thread-block
    // clusters of up to MAX_CLUSTER_SPLITS blocks; with more splits than that (a multiple of it) every
    // cluster leaves a partial result in the scratch, and the results are combined slice by slice
    // through the counters.  Up to MAX_CLUSTER_SPLITS splits scratch and counters are not used.
    const bool clustered = cluster != 0 && num_splits > 1;
    if (clustered && num_splits > MAX_CLUSTER_SPLITS && num_splits % MAX_CLUSTER_SPLITS) return SLB_ERR_BAD_ARG;
    const bool needs_scratch = num_splits > 1 && (!clustered || num_splits > MAX_CLUSTER_SPLITS);
    if (num_splits < 1 || (needs_scratch && (scratch == nullptr || counters == nullptr)))
        return SLB_ERR_BAD_ARG;
    if (stages < 2 || stages > MAX_STAGES || !(split_coef >= 0.f) || unsplit_tiles < 0) return SLB_ERR_BAD_ARG;
    if (((uintptr_t)kc | (uintptr_t)vc) % 16 || ldq % 8 || (uintptr_t)q % 16) return SLB_ERR_BAD_ARG;
    if (num_splits > MAX_SPLITS || S > 65535) return SLB_ERR_TOO_LARGE;
    const long long rows = (long long)num_pages * Hkv * ps;
    if (rows > 0x7fffffffll) return SLB_ERR_TOO_LARGE;     // box coordinates are 32-bit
    const int box_rows = ps < BN ? ps : BN;
    CUtensorMap map_k, map_v;
    int rc = slb_tma::make_paneled_rows_map(&map_k, kc, D, rows, box_rows);
    if (rc != 0) return rc;
    rc = slb_tma::make_paneled_rows_map(&map_v, vc, D, rows, box_rows);
    if (rc != 0) return rc;
#define SLB_LAUNCH_DECODE(NH_, CL_)                                                                      \
    launch_decode<NH_, CL_>(q, ldq, map_k, map_v, out, ldo, block_table, max_pages, ctx_len, scratch,    \
                            counters, S, H, Hkv, ps, box_rows, scale, window, num_splits, stages,        \
                            split_coef, unsplit_tiles, num_pages, st)
    if (clustered) return H / Hkv <= 8 ? SLB_LAUNCH_DECODE(1, true) : SLB_LAUNCH_DECODE(2, true);
    return H / Hkv <= 8 ? SLB_LAUNCH_DECODE(1, false) : SLB_LAUNCH_DECODE(2, false);
#undef SLB_LAUNCH_DECODE
}

}  // extern "C"

#else   // head sizes whose rows are not whole 128-byte panels

extern "C" {
int slb_decode_attention_ws_supported(int) { return 0; }
int slb_decode_attention_ws_status(int) { return 0; }
int slb_decode_attention_ws_splits_used(int) { return 0; }
int slb_decode_attention_ws_max_splits() { return 1; }
int slb_decode_attention_ws_max_cluster_splits() { return 1; }
int slb_decode_attention_ws_tile_keys() { return 64; }
long long slb_decode_attention_ws_scratch_bytes(int, int, int) { return 0; }
long long slb_decode_attention_ws_counters(int, int, int) { return 0; }
int slb_decode_attention_ws_bf16(const bf16*, int, const bf16*, const bf16*, bf16*, int, const int*, int,
                                 const int*, float*, int*, int, int, int, int, int, float, int, int, int,
                                 float, int, int, cudaStream_t) {
    return SLB_ERR_BAD_ARG;
}
}

#endif
