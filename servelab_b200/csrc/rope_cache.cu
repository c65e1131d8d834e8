// q/k/v bias + rotary position encoding + write of keys and values into pages.
//
// Input is the fused q|k|v projection of each token ([T, (H + 2 Hkv) D], without
// bias).  Per (token, head) block: add the bias, rotate q and k heads by the
// token's position (rotate-half over the first rotary_dim elements: with halves
// x1|x2, x' = x1 cos - x2 sin | x2 cos + x1 sin, angle = pos * inv_freq[i], all in
// float32), store q to its own buffer and k (rotated) and v into the page that
// the request's block table names: slot = table[pos / ps] * ps + pos % ps.
//
// Reference analogues: qkv with bias (servelab/parallel/tp_model.py:48-53),
// apply_rope before the cache write (tp_model.py:128-129), pool.write
// (servelab/kv_cache/pool.py:68-78), the slot formula (servelab/kv_cache/
// manager.py:309-313).  Page layout here: [page][kv head][slot in page][D].
#include "common.cuh"

template <typename T>
__global__ void qkv_rope_cache_kernel(
    const T* __restrict__ qkv, int ld_qkv, const float* __restrict__ bias,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int max_pages, int page_size,
    const float* __restrict__ inv_freq, int rotary_dim,
    T* __restrict__ q_out, int ld_q, T* __restrict__ k_cache, T* __restrict__ v_cache,
    int H, int Hkv, int D) {
    const int t = blockIdx.x;
    const int j = blockIdx.y;                       // 0..H-1 q, H..H+Hkv-1 k, then v
    const int pos = positions[t];
    const T* x = qkv + (size_t)t * ld_qkv + (size_t)j * D;
    const float* b = bias ? bias + (size_t)j * D : nullptr;
    const bool is_q = j < H;
    const bool is_v = j >= H + Hkv;
    const bool rotate = !is_v && inv_freq != nullptr && rotary_dim > 0;
    const int half = rotary_dim >> 1;

    T* dst;
    if (is_q) {
        dst = q_out + (size_t)t * ld_q + (size_t)j * D;
    } else {
        const int kvh = is_v ? j - H - Hkv : j - H;
        const int page = block_table[(size_t)seq_of_token[t] * max_pages + pos / page_size];
        if (page < 0) return;                       // no page: nothing may be written
        T* base = is_v ? v_cache : k_cache;
        dst = base + (((size_t)page * Hkv + kvh) * page_size + pos % page_size) * D;
    }
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = to_float(x[i]) + (b ? b[i] : 0.f);
        if (rotate && i < rotary_dim) {
            const int fi = i < half ? i : i - half;
            const int pi = i < half ? i + half : i - half;
            const float other = to_float(x[pi]) + (b ? b[pi] : 0.f);
            float sn, cs;
            sincosf((float)pos * inv_freq[fi], &sn, &cs);
            v = i < half ? v * cs - other * sn : v * cs + other * sn;
        }
        dst[i] = from_float<T>(v);
    }
}

template <typename T>
static int launch_qkv_rope_cache(const T* qkv, int ld_qkv, const float* bias, const int* positions,
                                 const int* seq_of_token, const int* block_table, int max_pages,
                                 int page_size, const float* inv_freq, int rotary_dim, T* q_out,
                                 int ld_q, T* k_cache, T* v_cache, int T_, int H, int Hkv, int D,
                                 cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || D <= 0 || page_size <= 0 || max_pages <= 0) return SLB_ERR_BAD_ARG;
    if (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1)) return SLB_ERR_BAD_ARG;
    const bool write = k_cache != nullptr && v_cache != nullptr;
    const int heads = write ? H + 2 * Hkv : H;
    if (heads > 65535) return SLB_ERR_TOO_LARGE;
    int threads = 32;
    while (threads < 128 && threads < D) threads <<= 1;
    qkv_rope_cache_kernel<T><<<dim3(T_, heads), threads, 0, st>>>(
        qkv, ld_qkv, bias, positions, seq_of_token, block_table, max_pages, page_size, inv_freq,
        rotary_dim, q_out, ld_q, k_cache, v_cache, H, Hkv, D);
    return slb_launch_status();
}

extern "C" {
int slb_qkv_rope_cache_f32(const float* qkv, int ld_qkv, const float* bias, const int* positions,
                           const int* seq_of_token, const int* block_table, int max_pages,
                           int page_size, const float* inv_freq, int rotary_dim, float* q_out,
                           int ld_q, float* k_cache, float* v_cache, int T, int H, int Hkv, int D,
                           cudaStream_t st) {
    return launch_qkv_rope_cache<float>(qkv, ld_qkv, bias, positions, seq_of_token, block_table,
                                        max_pages, page_size, inv_freq, rotary_dim, q_out, ld_q,
                                        k_cache, v_cache, T, H, Hkv, D, st);
}
int slb_qkv_rope_cache_bf16(const bf16* qkv, int ld_qkv, const float* bias, const int* positions,
                            const int* seq_of_token, const int* block_table, int max_pages,
                            int page_size, const float* inv_freq, int rotary_dim, bf16* q_out,
                            int ld_q, bf16* k_cache, bf16* v_cache, int T, int H, int Hkv, int D,
                            cudaStream_t st) {
    return launch_qkv_rope_cache<bf16>(qkv, ld_qkv, bias, positions, seq_of_token, block_table,
                                       max_pages, page_size, inv_freq, rotary_dim, q_out, ld_q,
                                       k_cache, v_cache, T, H, Hkv, D, st);
}
}
