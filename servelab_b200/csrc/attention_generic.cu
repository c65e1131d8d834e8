// Plain paged attention: any head size up to 256, any number of heads and groups,
// any page size, any mix of prompt portions and single decoded tokens, float32
// arithmetic throughout (inputs and outputs float32 or bfloat16).
//
// It is the attention of the 32-bit path and the plain kernel that stands beside
// the fast bfloat16 kernels (which are checked against it).
//
// Work unit: (tile of 32 query rows, kv head).  The query rows of one request and
// one kv head are flattened as rho = local_token * g + head_in_group, so that the
// g query heads sharing a kv head also share each loaded key/value tile.  Keys are
// visited in tiles of 32 aligned to absolute positions, in increasing order, with
// an online softmax per row (running max m, running sum l, float32 accumulator).
// A row's result therefore depends only on that row's query and the keys it may
// see: not on the other rows of the tile, not on how the prompt was cut, and not
// on which pages hold the keys.
//
// Masking: key position r is visible to a query at position a iff r <= a and, with
// a window w > 0, a - r < w.  The position of local token i of a request is
// ctx_len - q_len + i.
//
// Reference analogue: the per-sequence torch loop (servelab/parallel/
// tp_model.py:136-157): gather rows by block table, repeat_interleave for the
// groups, float32 scores * D^-1/2, causal mask, float32 softmax, float32 P.V.
#include "common.cuh"

#define AG_BM 32
#define AG_BN 32
#define AG_THREADS 256
#define AG_MAX_D 256

// 0, or 1 once a block-table entry pointed outside the cache (page >= num_pages): those keys
// were read as zeros instead of from outside the pool.
SLB_DEFINE_STATUS_WORD(generic_attention_status_word, slb_paged_attention_generic_status)

template <typename T>
__global__ void __launch_bounds__(AG_THREADS) paged_attention_generic_kernel(
    const T* __restrict__ q, int ldq, const T* __restrict__ kc, const T* __restrict__ vc,
    T* __restrict__ out, int ldo, const int* __restrict__ block_table, int max_pages,
    const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_row0,
    int H, int Hkv, int D, int ps, int num_pages, float scale, int window) {
    extern __shared__ float smem[];
    pdl_wait();
    const int ldd = D + 1;
    float* Qs = smem;
    float* Ks = Qs + AG_BM * ldd;
    float* Vs = Ks + AG_BN * ldd;
    float* Ps = Vs + AG_BN * ldd;                 // [AG_BM][AG_BN + 1]

    const int tid = threadIdx.x;
    const int kvh = blockIdx.y;
    const int s = tile_seq[blockIdx.x];
    const int row0 = tile_row0[blockIdx.x];
    const int g = H / Hkv;
    const int q0 = cu_q[s];
    const int qlen = cu_q[s + 1] - q0;
    const int ctx = ctx_len[s];
    const int nrows = min(AG_BM, qlen * g - row0);
    if (nrows <= 0) return;
    const int pos_base = ctx - qlen;

    for (int idx = tid; idx < AG_BM * D; idx += AG_THREADS) {
        const int r = idx / D, d = idx - r * D;
        float v = 0.f;
        if (r < nrows) {
            const int rho = row0 + r;
            const int tl = rho / g, hg = rho - tl * g;
            v = to_float(q[(size_t)(q0 + tl) * ldq + (size_t)(kvh * g + hg) * D + d]);
        }
        Qs[r * ldd + d] = v;
    }

    const int r = tid >> 3, c0 = tid & 7;
    const bool row_valid = r < nrows;
    const int my_pos = row_valid ? pos_base + (row0 + r) / g : -1;
    const int p_first = pos_base + row0 / g;
    const int p_last = pos_base + (row0 + nrows - 1) / g;
    int kbeg = 0;
    if (window > 0) kbeg = max(0, p_first - window + 1) / AG_BN * AG_BN;
    const int kend = p_last + 1;
    const int nj = (D + 7) >> 3;

    float m = -INFINITY, l = 0.f;
    float acc[AG_MAX_D / 8];
#pragma unroll
    for (int j = 0; j < AG_MAX_D / 8; ++j) acc[j] = 0.f;

    const int* table = block_table + (size_t)s * max_pages;
    for (int k0 = kbeg; k0 < kend; k0 += AG_BN) {
        __syncthreads();
        for (int idx = tid; idx < AG_BN * D; idx += AG_THREADS) {
            const int kr = idx / D, d = idx - kr * D;
            const int kp = k0 + kr;
            float kv = 0.f, vv = 0.f;
            if (kp < kend) {
                const int page = table[kp / ps];
                if (page >= num_pages) {
                    atomicCAS(&generic_attention_status_word, 0, 1);
                } else if (page >= 0) {
                    const size_t off = (((size_t)page * Hkv + kvh) * ps + kp % ps) * D + d;
                    kv = to_float(kc[off]);
                    vv = to_float(vc[off]);
                }
            }
            Ks[kr * ldd + d] = kv;
            Vs[kr * ldd + d] = vv;
        }
        __syncthreads();

        float sc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int d = 0; d < D; ++d) {
            const float qv = Qs[r * ldd + d];
#pragma unroll
            for (int j = 0; j < 4; ++j) sc[j] += qv * Ks[(c0 + 8 * j) * ldd + d];
        }
        float tmax = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int kp = k0 + c0 + 8 * j;
            const bool vis = row_valid && kp <= my_pos && (window <= 0 || my_pos - kp < window);
            sc[j] = vis ? sc[j] * scale : -INFINITY;
            tmax = fmaxf(tmax, sc[j]);
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
        const float m_new = fmaxf(m, tmax);
        float alpha = 1.f, psum = 0.f;
        float p[4] = {0.f, 0.f, 0.f, 0.f};
        if (m_new != -INFINITY) {
            alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                p[j] = (sc[j] == -INFINITY) ? 0.f : expf(sc[j] - m_new);
                psum += p[j];
            }
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int j = 0; j < 4; ++j) Ps[r * (AG_BN + 1) + c0 + 8 * j] = p[j];
        __syncwarp();                              // a row's 8 threads share a warp

#pragma unroll
        for (int j = 0; j < AG_MAX_D / 8; ++j) acc[j] *= alpha;
        for (int k = 0; k < AG_BN; ++k) {
            const float pv = Ps[r * (AG_BN + 1) + k];
#pragma unroll
            for (int j = 0; j < AG_MAX_D / 8; ++j) {
                const int c = c0 + 8 * j;
                if (j < nj && c < D) acc[j] += pv * Vs[k * ldd + c];
            }
        }
    }

    if (row_valid) {
        const int rho = row0 + r;
        const int tl = rho / g, hg = rho - tl * g;
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + (size_t)(q0 + tl) * ldo + (size_t)(kvh * g + hg) * D;
#pragma unroll
        for (int j = 0; j < AG_MAX_D / 8; ++j) {
            const int c = c0 + 8 * j;
            if (j < nj && c < D) o[c] = from_float<T>(acc[j] * inv);
        }
    }
}

template <typename T>
static int launch_generic(const T* q, int ldq, const T* kc, const T* vc, T* out, int ldo,
                          const int* block_table, int max_pages, const int* cu_q,
                          const int* ctx_len, const int* tile_seq, const int* tile_row0,
                          int num_tiles, int H, int Hkv, int D, int ps, int num_pages, float scale,
                          int window, cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0 || D <= 0 || ps <= 0 || max_pages <= 0 || num_pages <= 0)
        return SLB_ERR_BAD_ARG;
    if (D > AG_MAX_D || Hkv > 65535) return SLB_ERR_TOO_LARGE;
    const size_t smem = ((size_t)(AG_BM + 2 * AG_BN) * (D + 1) + AG_BM * (AG_BN + 1)) * sizeof(float);
    // the largest this kernel can ask for (head size AG_MAX_D), set once per device
    constexpr size_t SMEM_MAX = ((size_t)(AG_BM + 2 * AG_BN) * (AG_MAX_D + 1) + AG_BM * (AG_BN + 1)) * sizeof(float);
    static unsigned long long configured = 0;     // per template instance, a bit per device
    const int rc = slb_configure(&configured, paged_attention_generic_kernel<T>, SMEM_MAX);
    if (rc != 0) return rc;
    return slb_launch(paged_attention_generic_kernel<T>, dim3(num_tiles, Hkv), dim3(AG_THREADS), smem,
                      st, q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q, ctx_len, tile_seq,
                      tile_row0, H, Hkv, D, ps, num_pages, scale, window);
}

extern "C" {
int slb_paged_attention_generic_f32(const float* q, int ldq, const float* kc, const float* vc,
                                    float* out, int ldo, const int* block_table, int max_pages,
                                    const int* cu_q, const int* ctx_len, const int* tile_seq,
                                    const int* tile_row0, int num_tiles, int H, int Hkv, int D,
                                    int ps, int num_pages, float scale, int window, cudaStream_t st) {
    return launch_generic<float>(q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q, ctx_len,
                                 tile_seq, tile_row0, num_tiles, H, Hkv, D, ps, num_pages, scale, window, st);
}
int slb_paged_attention_generic_bf16(const bf16* q, int ldq, const bf16* kc, const bf16* vc,
                                     bf16* out, int ldo, const int* block_table, int max_pages,
                                     const int* cu_q, const int* ctx_len, const int* tile_seq,
                                     const int* tile_row0, int num_tiles, int H, int Hkv, int D,
                                     int ps, int num_pages, float scale, int window, cudaStream_t st) {
    return launch_generic<bf16>(q, ldq, kc, vc, out, ldo, block_table, max_pages, cu_q, ctx_len,
                                tile_seq, tile_row0, num_tiles, H, Hkv, D, ps, num_pages, scale, window, st);
}
// rows per tile of the generic kernel (the host builds the tile list with it)
int slb_paged_attention_generic_tile_rows() { return AG_BM; }
}
