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

// 0, or 1 once a block-table entry pointed outside the cache (page >= num_pages): that key
// and value were not written.  A table can only be wrong through a fault of the host side;
// the kernels skip the access and say so instead of writing outside the pool.
SLB_DEFINE_STATUS_WORD(cache_write_status_word, slb_cache_write_status)

__device__ __forceinline__ bool page_in_cache(int page, int num_pages) {
    if (page >= num_pages) {
        atomicCAS(&cache_write_status_word, 0, 1);
        return false;
    }
    return page >= 0;
}

// One block per token.  A head is D/2 "slots" of two elements: slot i < rot/2 is the
// rotation pair (i, i + rot/2); the slots after that are pairs of neighbouring
// elements beyond the rotary part, which pass through.  Thread (i, lane-of-heads)
// computes sin/cos of its slot once and walks the heads with them.
template <typename T>
__global__ void qkv_rope_cache_kernel(
    const T* __restrict__ qkv, int ld_qkv, const float* __restrict__ bias,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
    const float* __restrict__ inv_freq, int rotary_dim,
    T* __restrict__ q_out, int ld_q, T* __restrict__ k_cache, T* __restrict__ v_cache,
    int H, int Hkv, int D, int slots_per_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int i = threadIdx.x % slots_per_head;
    const int head_lane = threadIdx.x / slots_per_head;
    const int head_lanes = blockDim.x / slots_per_head;
    if (i >= D / 2) return;
    const int pos = positions[t];
    const int half = (inv_freq != nullptr) ? rotary_dim >> 1 : 0;
    const bool rot = i < half;
    float sn = 0.f, cs = 1.f;
    if (rot) sincosf((float)pos * inv_freq[i], &sn, &cs);
    // the two elements of this slot in a rotated head, and in a head that is copied
    const int e0 = rot ? i : 2 * half + 2 * (i - half);
    const int e1 = rot ? i + half : e0 + 1;
    const int c0 = 2 * i, c1 = 2 * i + 1;
    const bool write = k_cache != nullptr && v_cache != nullptr;
    size_t kv_base = 0;
    bool have_page = false;
    if (write) {
        const int page = block_table[(size_t)seq_of_token[t] * max_pages + pos / page_size];
        have_page = page_in_cache(page, num_pages);    // no page: nothing may be written
        kv_base = ((size_t)(have_page ? page : 0) * Hkv * page_size + pos % page_size) * D;
    }
    const T* x = qkv + (size_t)t * ld_qkv;
    const int heads = write ? H + 2 * Hkv : H;
    for (int j = head_lane; j < heads; j += head_lanes) {
        const bool is_v = j >= H + Hkv;
        const int a = is_v ? c0 : e0, b = is_v ? c1 : e1;
        const size_t off = (size_t)j * D;
        float va = to_float(x[off + a]), vb = to_float(x[off + b]);
        if (bias) { va += bias[off + a]; vb += bias[off + b]; }
        if (rot && !is_v) {
            const float ra = va * cs - vb * sn;
            vb = vb * cs + va * sn;
            va = ra;
        }
        T* dst;
        if (j < H) {
            dst = q_out + (size_t)t * ld_q + off;
        } else {
            if (!have_page) continue;
            const int kvh = is_v ? j - H - Hkv : j - H;
            dst = (is_v ? v_cache : k_cache) + kv_base + (size_t)kvh * page_size * D;
        }
        dst[a] = from_float<T>(va);
        dst[b] = from_float<T>(vb);
    }
}

// The projection as float32 partial sums [nparts][T][ld_qkv] of a product split along K
// (decode steps): one block per (head, token), so that a step of few tokens still fills
// the GPU; thread i owns slot i of the head as in the kernel above and adds the parts in
// their order.
template <typename T>
__global__ void qkv_rope_cache_parts_kernel(
    const float* __restrict__ parts, int nparts, size_t part_stride, int ld_qkv,
    const float* __restrict__ bias, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int max_pages,
    int page_size, int num_pages, const float* __restrict__ inv_freq, int rotary_dim,
    T* __restrict__ q_out, int ld_q, T* __restrict__ k_cache, T* __restrict__ v_cache,
    int H, int Hkv, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int j = blockIdx.x, t = blockIdx.y, i = threadIdx.x;
    if (i >= D / 2) return;
    const int pos = positions[t];
    const int half = (inv_freq != nullptr) ? rotary_dim >> 1 : 0;
    const bool is_v = j >= H + Hkv;
    const bool rot = i < half && !is_v;
    // the two elements of this slot: a rotation pair, or neighbours that pass through
    const int a = rot ? i : (is_v ? 2 * i : (i < half ? i : 2 * half + 2 * (i - half)));
    const int b = rot ? i + half : (is_v ? 2 * i + 1 : (i < half ? i + half : a + 1));
    const size_t off = (size_t)j * D;
    const float* px = parts + (size_t)t * ld_qkv + off;
    float va = 0.f, vb = 0.f;
    for (int p = 0; p < nparts; ++p) {
        va += px[p * part_stride + a];
        vb += px[p * part_stride + b];
    }
    if (bias) { va += bias[off + a]; vb += bias[off + b]; }
    if (rot) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        const float ra = va * cs - vb * sn;
        vb = vb * cs + va * sn;
        va = ra;
    }
    T* dst;
    if (j < H) {
        dst = q_out + (size_t)t * ld_q + off;
    } else {
        const int page = block_table[(size_t)seq_of_token[t] * max_pages + pos / page_size];
        if (!page_in_cache(page, num_pages)) return;   // no page: nothing may be written
        const int kvh = is_v ? j - H - Hkv : j - H;
        dst = (is_v ? v_cache : k_cache) +
              (((size_t)page * Hkv + kvh) * page_size + pos % page_size) * D;
    }
    dst[a] = from_float<T>(va);
    dst[b] = from_float<T>(vb);
}

// The same with 16-byte accesses, for layouts whose rotary and pass-through parts are
// whole vectors (VEC = 16 bytes of T).  One block per token: the first rotary_dim / 2
// threads compute the token's sines and cosines once into shared memory; then the
// block walks "units" of 2 * VEC elements: in a rotated head unit u < half / VEC is the
// VEC rotation pairs (u VEC + e, u VEC + e + half); every other unit is 2 * VEC
// neighbouring elements that pass through (the tail of a rotated head, a value head).
template <typename T>
__global__ void qkv_rope_cache_vec_kernel(
    const T* __restrict__ qkv, int ld_qkv, const float* __restrict__ bias,
    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
    const int* __restrict__ block_table, int max_pages, int page_size, int num_pages,
    const float* __restrict__ inv_freq, int rotary_dim,
    T* __restrict__ q_out, int ld_q, T* __restrict__ k_cache, T* __restrict__ v_cache,
    int H, int Hkv, int D) {
    constexpr int VEC = 16 / (int)sizeof(T);
    extern __shared__ float trig[];                    // cos[half] then sin[half]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = (inv_freq != nullptr) ? rotary_dim >> 1 : 0;
    const bool write = k_cache != nullptr && v_cache != nullptr;
    const int units_per_head = D / (2 * VEC);
    const int rot_units = half / VEC;
    const int heads = write ? H + 2 * Hkv : H;
    const int units = heads * units_per_head;
    const T* x = qkv + (size_t)t * ld_qkv;

    // where unit w reads and writes inside its head: a rotation pair, or neighbours
    auto place = [&](int w, int& j, int& a, int& b, bool& rot, bool& is_v) {
        j = w / units_per_head;
        const int u = w - j * units_per_head;
        is_v = j >= H + Hkv;
        rot = !is_v && u < rot_units;
        a = rot ? u * VEC : (is_v ? 2 * VEC * u : 2 * half + 2 * VEC * (u - rot_units));
        b = rot ? a + half : a + VEC;
    };
    const int pos = positions[t];
    size_t kv_base = 0;
    bool have_page = false;
    if (write) {
        const int page = block_table[(size_t)seq_of_token[t] * max_pages + pos / page_size];
        have_page = page_in_cache(page, num_pages);    // no page: nothing may be written
        kv_base = ((size_t)(have_page ? page : 0) * Hkv * page_size + pos % page_size) * D;
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        trig[i] = cs;
        trig[half + i] = sn;
    }
    __syncthreads();
    for (int w = threadIdx.x; w < units; w += blockDim.x) {
        int j, a, b; bool rot, is_v;
        place(w, j, a, b, rot, is_v);
        const size_t off = (size_t)j * D;
        T va[VEC], vb[VEC];
        *reinterpret_cast<uint4*>(va) = *reinterpret_cast<const uint4*>(x + off + a);
        *reinterpret_cast<uint4*>(vb) = *reinterpret_cast<const uint4*>(x + off + b);
        float fa[VEC], fb[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            fa[e] = to_float(va[e]);
            fb[e] = to_float(vb[e]);
        }
        if (bias) {                                    // a and b are multiples of VEC: 16-byte loads
#pragma unroll
            for (int e = 0; e < VEC; e += 4) {
                const float4 ba = *reinterpret_cast<const float4*>(bias + off + a + e);
                const float4 bb = *reinterpret_cast<const float4*>(bias + off + b + e);
                fa[e] += ba.x; fa[e + 1] += ba.y; fa[e + 2] += ba.z; fa[e + 3] += ba.w;
                fb[e] += bb.x; fb[e + 1] += bb.y; fb[e + 2] += bb.z; fb[e + 3] += bb.w;
            }
        }
        if (rot) {
#pragma unroll
            for (int e = 0; e < VEC; e += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(trig + a + e);
                const float4 s4 = *reinterpret_cast<const float4*>(trig + half + a + e);
                const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float ra = fa[e + k] * cs[k] - fb[e + k] * sn[k];
                    fb[e + k] = fb[e + k] * cs[k] + fa[e + k] * sn[k];
                    fa[e + k] = ra;
                }
            }
        }
        T* dst;
        if (j < H) {
            dst = q_out + (size_t)t * ld_q + off;
        } else {
            if (!have_page) continue;
            const int kvh = is_v ? j - H - Hkv : j - H;
            dst = (is_v ? v_cache : k_cache) + kv_base + (size_t)kvh * page_size * D;
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            va[e] = from_float<T>(fa[e]);
            vb[e] = from_float<T>(fb[e]);
        }
        *reinterpret_cast<uint4*>(dst + a) = *reinterpret_cast<const uint4*>(va);
        *reinterpret_cast<uint4*>(dst + b) = *reinterpret_cast<const uint4*>(vb);
    }
}

template <typename T>
static int launch_qkv_rope_cache(const T* qkv, int ld_qkv, const float* parts, int nparts,
                                 long long part_stride, const float* bias, const int* positions,
                                 const int* seq_of_token, const int* block_table, int max_pages,
                                 int page_size, int num_pages, const float* inv_freq, int rotary_dim, T* q_out,
                                 int ld_q, T* k_cache, T* v_cache, int T_, int H, int Hkv, int D,
                                 cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (H <= 0 || Hkv <= 0 || D <= 0 || (D & 1) || page_size <= 0 || max_pages <= 0)
        return SLB_ERR_BAD_ARG;
    if (k_cache != nullptr && num_pages <= 0) return SLB_ERR_BAD_ARG;
    if (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1)) return SLB_ERR_BAD_ARG;
    if (D > 1024) return SLB_ERR_TOO_LARGE;
    int slots = 1;
    while (slots < D / 2) slots <<= 1;                 // power of two >= D/2, at most 512
    const int heads = H + 2 * Hkv;
    int lanes = 256 / slots;
    if (lanes < 1) lanes = 1;
    if (lanes > heads) lanes = heads;
    int threads = slots * lanes;
    threads = (threads + 31) / 32 * 32;
    if ((qkv == nullptr) == (nparts <= 0)) return SLB_ERR_BAD_ARG;      // exactly one input form
    constexpr int VEC = 16 / (int)sizeof(T);
    const int rot = inv_freq != nullptr ? rotary_dim : 0;
    const bool vec_ok = nparts <= 0 && D % (2 * VEC) == 0 && rot % (2 * VEC) == 0 &&
                        ld_qkv % VEC == 0 && ld_q % VEC == 0 &&
                        ((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) % 16 == 0;
    if (vec_ok) {
        const int units = heads * (D / (2 * VEC));
        // as few equal passes over the units as blocks of up to 512 threads allow (288 units:
        // one pass of 288 threads, not a full pass of 256 and one that keeps a single warp busy)
        const int passes = (units + 511) / 512;
        int vthreads = ((units + passes - 1) / passes + 31) / 32 * 32;
        if (vthreads < rot / 2) vthreads = ((rot / 2 + 31) / 32 * 32 < 1024) ? (rot / 2 + 31) / 32 * 32 : 1024;
        return slb_launch(qkv_rope_cache_vec_kernel<T>, dim3(T_), dim3(vthreads), (size_t)rot * sizeof(float), st,
                          qkv, ld_qkv, bias, positions, seq_of_token, block_table, max_pages, page_size, num_pages,
                          inv_freq, rotary_dim, q_out, ld_q, k_cache, v_cache, H, Hkv, D);
    }
    if (nparts > 0) {
        if (T_ > 65535) return SLB_ERR_TOO_LARGE;
        const bool write = k_cache != nullptr && v_cache != nullptr;
        return slb_launch(qkv_rope_cache_parts_kernel<T>, dim3(write ? heads : H, T_),
                          dim3((D / 2 + 31) / 32 * 32), 0, st, parts, nparts, (size_t)part_stride,
                          ld_qkv, bias, positions, seq_of_token, block_table, max_pages, page_size, num_pages,
                          inv_freq, rotary_dim, q_out, ld_q, k_cache, v_cache, H, Hkv, D);
    }
    return slb_launch(qkv_rope_cache_kernel<T>, dim3(T_), dim3(threads), 0, st, qkv, ld_qkv, bias,
                      positions, seq_of_token, block_table, max_pages, page_size, num_pages, inv_freq, rotary_dim,
                      q_out, ld_q, k_cache, v_cache, H, Hkv, D, slots);
}

extern "C" {
int slb_qkv_rope_cache_f32(const float* qkv, int ld_qkv, const float* bias, const int* positions,
                           const int* seq_of_token, const int* block_table, int max_pages,
                           int page_size, int num_pages, const float* inv_freq, int rotary_dim, float* q_out,
                           int ld_q, float* k_cache, float* v_cache, int T, int H, int Hkv, int D,
                           cudaStream_t st) {
    return launch_qkv_rope_cache<float>(qkv, ld_qkv, nullptr, 0, 0, bias, positions, seq_of_token, block_table,
                                        max_pages, page_size, num_pages, inv_freq, rotary_dim, q_out, ld_q,
                                        k_cache, v_cache, T, H, Hkv, D, st);
}
int slb_qkv_rope_cache_bf16(const bf16* qkv, int ld_qkv, const float* bias, const int* positions,
                            const int* seq_of_token, const int* block_table, int max_pages,
                            int page_size, int num_pages, const float* inv_freq, int rotary_dim, bf16* q_out,
                            int ld_q, bf16* k_cache, bf16* v_cache, int T, int H, int Hkv, int D,
                            cudaStream_t st) {
    return launch_qkv_rope_cache<bf16>(qkv, ld_qkv, nullptr, 0, 0, bias, positions, seq_of_token, block_table,
                                       max_pages, page_size, num_pages, inv_freq, rotary_dim, q_out, ld_q,
                                       k_cache, v_cache, T, H, Hkv, D, st);
}
// the fused q|k|v projection arrives as float32 partial sums [nparts][T][ld_qkv]
int slb_qkv_rope_cache_parts_bf16(const float* parts, int nparts, long long part_stride, int ld_qkv,
                                  const float* bias, const int* positions, const int* seq_of_token,
                                  const int* block_table, int max_pages, int page_size, int num_pages,
                                  const float* inv_freq, int rotary_dim, bf16* q_out, int ld_q,
                                  bf16* k_cache, bf16* v_cache, int T, int H, int Hkv, int D,
                                  cudaStream_t st) {
    return launch_qkv_rope_cache<bf16>(nullptr, ld_qkv, parts, nparts, part_stride, bias, positions,
                                       seq_of_token, block_table, max_pages, page_size, num_pages, inv_freq,
                                       rotary_dim, q_out, ld_q, k_cache, v_cache, T, H, Hkv, D, st);
}
}
