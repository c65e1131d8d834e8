// Embedding gather, fused residual-add + RMSNorm, SwiGLU.
//
// The residual stream is float32 in both the 32-bit and the bfloat16 path: the
// residual sum and the whole norm are computed in float32, only the normed
// activations handed to the next matrix product take the compute dtype.
//
// Reference analogues: F.embedding (servelab/parallel/tp_model.py:123), RMSNorm
// (servelab/attention/triton/paged_attention.py:76-91: one program per row,
// float32 x*rsqrt(mean(x^2)+eps)*w), silu(gate)*up (tp_model.py:67-68).
#include "common.cuh"

// Vector helpers: 4 consecutive elements as float4 (float32: one 16-byte access,
// bfloat16: one 8-byte access).  Callers guarantee the alignment.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&lo);
    raw.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

// out[t, :] = table[ids[t], :] * scale as float32.  An id outside [0, vocab) yields a
// row of zeros (callers validate ids on the host).  VEC: h % 4 == 0.
template <typename T, bool VEC>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int h, int vocab, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * h;
    float* o = out + (size_t)t * h;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
            float4 v = ok ? load4(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
            store4(o + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) o[i] = ok ? to_float(row[i]) * scale : 0.f;
    }
}

// logits[r, v] = cap * tanh(logits[r, v] * scale / cap) (cap > 0), or logits * scale: what
// some architectures do to their logits after the LM head.  In place, float32.
__global__ void logit_transform_kernel(float* __restrict__ logits, int ld, int V, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    float* row = logits + (size_t)blockIdx.y * ld;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < V; v += gridDim.x * blockDim.x) {
        const float x = row[v] * scale;
        row[v] = cap > 0.f ? cap * tanhf(x / cap) : x;
    }
}

// One block per output row r.  src = row_map ? row_map[r] : r.
//   v = resid[src] + delta[src]        (delta may be null)
//   if no row_map: resid[src] = v      (the stream is updated in place)
//   out[r] = v * (1/sqrt(mean(v^2) + eps)) * weight
// The update may instead arrive as `nparts` float32 partial sums (a matrix product
// split along K): parts[p * part_stride + src * h + i], added in the order of p,
// plus an optional float32 bias `pbias[i]`.
// The sum of squares is accumulated per thread over a strided walk and then
// reduced over the block; both depend only on h and the block size, never on the
// batch.  VEC: h % 4 == 0 (all rows then start 16-byte aligned).
// The partial sums are fetched eight at a time before any is added (the additions keep the
// order of p): a loop of load-then-add would wait for every load in turn, ten round trips
// to the L2 cache for a product split ten ways.
template <typename TD>
__device__ __forceinline__ float4 delta4(const TD* d, const float* parts, int nparts,
                                         size_t part_stride, const float* pbias, int i) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (d) v = load4(d + i);
    if (pbias) b = load4(pbias + i);
    for (int p0 = 0; p0 < nparts; p0 += 8) {
        float4 q[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            q[j] = p0 + j < nparts ? __ldcg(reinterpret_cast<const float4*>(parts + (size_t)(p0 + j) * part_stride + i))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 8; ++j) { v.x += q[j].x; v.y += q[j].y; v.z += q[j].z; v.w += q[j].w; }
    }
    v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    return v;
}
template <typename TD>
__device__ __forceinline__ float delta1(const TD* d, const float* parts, int nparts,
                                        size_t part_stride, const float* pbias, int i) {
    float v = d ? to_float(d[i]) : 0.f;
    for (int p = 0; p < nparts; ++p) v += parts[p * part_stride + i];
    if (pbias) v += pbias[i];
    return v;
}

// NV: float4 a thread keeps in registers between the two passes (rows of up to 16 * blockDim
// elements; longer rows are read again in the second pass).
constexpr int NORM_NV = 4;

template <typename TD, typename TO, bool VEC, bool PARTS>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const float* __restrict__ parts, int nparts, size_t part_stride,
                                   const float* __restrict__ pbias,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ row_map, int h, float eps,
                                   const SlbTraceArg tr) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    if (threadIdx.x == 0) slb_trace_event(tr, 5, SLB_TR_START);
    // the norm weights are written by no kernel: they are fetched while the kernel before
    // this one still runs
    const bool in_regs = VEC && h <= (int)blockDim.x * 4 * NORM_NV;
    float4 wv[NORM_NV];
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NORM_NV; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * 4;
            wv[j] = i < h ? load4(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    pdl_wait();
    if (threadIdx.x == 0) slb_trace_event(tr, 5, SLB_TR_WAITED);
    const int r = blockIdx.x;
    const int src = row_map ? row_map[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)src * h : nullptr;
    const float* pp = PARTS ? parts + (size_t)src * h : nullptr;
    if (!PARTS) nparts = 0;
    const bool has_delta = d != nullptr || PARTS;
    const bool write_back = (row_map == nullptr) && has_delta;
    TO* o = out + (size_t)r * h;
    float ss = 0.f;
    if (in_regs) {
        // one pass over global memory: the row stays in registers between the sum of squares
        // and the scaling (same order of additions per thread as the two-pass form)
        float4 xv[NORM_NV];
#pragma unroll
        for (int j = 0; j < NORM_NV; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * 4;
            xv[j] = i < h ? load4(x + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (has_delta) {
            // every load of the update before the first store of the stream (a store between
            // two loads would make the second wait for the first)
            float4 dv[NORM_NV];
#pragma unroll
            for (int j = 0; j < NORM_NV; ++j) {
                const int i = (threadIdx.x + j * blockDim.x) * 4;
                dv[j] = i < h ? delta4(d, pp, nparts, part_stride, pbias, i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < NORM_NV; ++j) {
                const int i = (threadIdx.x + j * blockDim.x) * 4;
                xv[j].x += dv[j].x; xv[j].y += dv[j].y; xv[j].z += dv[j].z; xv[j].w += dv[j].w;
                if (write_back && i < h) store4(x + i, xv[j]);
            }
        }
        if (threadIdx.x == 0) slb_trace_event(tr, 5, SLB_TR_LOOP_DONE);
#pragma unroll
        for (int j = 0; j < NORM_NV; ++j) {
            ss += xv[j].x * xv[j].x;
            ss += xv[j].y * xv[j].y;
            ss += xv[j].z * xv[j].z;
            ss += xv[j].w * xv[j].w;
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)h + eps);
#pragma unroll
        for (int j = 0; j < NORM_NV; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * 4;
            if (i < h)
                store4(o + i, make_float4(xv[j].x * rstd * wv[j].x, xv[j].y * rstd * wv[j].y,
                                          xv[j].z * rstd * wv[j].z, xv[j].w * rstd * wv[j].w));
        }
        if (threadIdx.x == 0) slb_trace_event(tr, 5, SLB_TR_END);
        return;
    }
    if (VEC) {
        for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
            float4 v = load4(x + i);
            if (has_delta) {
                const float4 dv = delta4(d, pp, nparts, part_stride, pbias, i);
                v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            }
            if (write_back) store4(x + i, v);
            ss += v.x * v.x;
            ss += v.y * v.y;
            ss += v.z * v.z;
            ss += v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float v = x[i];
            if (has_delta) v += delta1(d, pp, nparts, part_stride, pbias, i);
            if (write_back) x[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)h + eps);
    if (VEC) {
        for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
            float4 v = load4(x + i);
            if (has_delta && !write_back) {
                const float4 dv = delta4(d, pp, nparts, part_stride, pbias, i);
                v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            }
            const float4 w = load4(weight + i);
            store4(o + i, make_float4(v.x * rstd * w.x, v.y * rstd * w.y, v.z * rstd * w.z,
                                      v.w * rstd * w.w));
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float v = x[i];
            if (has_delta && !write_back) v += delta1(d, pp, nparts, part_stride, pbias, i);
            o[i] = from_float<TO>(v * rstd * weight[i]);
        }
    }
    if (threadIdx.x == 0) slb_trace_event(tr, 5, SLB_TR_END);
}

// ---- the same norm for an update that arrives as K-split partial sums (decode steps) ----
// A step of few tokens has few rows: a row is shared by a cluster of NORM_CLUSTER blocks
// (a column range each), so that adding the partial sums is spread over the GPU.  Every
// block reduces its own sum of squares, publishes it in its shared memory and reads the
// others' through the cluster's distributed shared memory, in the order of the ranks
// (the row's result depends on h and the cluster size only, never on the batch).
constexpr int NORM_CLUSTER = 8;

__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float load_cluster_shared(const float* mine, unsigned rank) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(mine);
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// grid (NORM_CLUSTER, rows), cluster (NORM_CLUSTER, 1, 1); chunk: columns per block (a
// multiple of 4, at most 4 * blockDim.x); h % 4 == 0.
template <typename TO>
__global__ void add_rmsnorm_parts_cluster_kernel(float* __restrict__ resid,
                                                 const float* __restrict__ parts, int nparts,
                                                 size_t part_stride, const float* __restrict__ pbias,
                                                 const float* __restrict__ weight, TO* __restrict__ out,
                                                 const int* __restrict__ row_map, int h, int chunk,
                                                 float eps, const SlbTraceArg tr) {
    __shared__ float scratch[33];
    __shared__ float my_ss;
    pdl_launch_dependents();
    if (threadIdx.x == 0) slb_trace_event(tr, 6, SLB_TR_START);
    const unsigned rank = cluster_ctarank();
    const int r = blockIdx.y;
    const int i = (int)rank * chunk + threadIdx.x * 4;
    const bool active = (int)threadIdx.x * 4 < chunk && i < h;
    // the norm weights are written by no kernel: fetched while the kernel before this one runs
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) w = load4(weight + i);
    pdl_wait();
    if (threadIdx.x == 0) slb_trace_event(tr, 6, SLB_TR_WAITED);
    const int src = row_map ? row_map[r] : r;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active) {
        float* x = resid + (size_t)src * h;
        v = load4(x + i);
        const float4 dv = delta4<float>(nullptr, parts + (size_t)src * h, nparts, part_stride, pbias, i);
        v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
        if (row_map == nullptr) store4(x + i, v);          // the stream is updated in place
    }
    float ss = v.x * v.x;
    ss += v.y * v.y;
    ss += v.z * v.z;
    ss += v.w * v.w;
    if (threadIdx.x == 0) slb_trace_event(tr, 6, SLB_TR_LOOP_DONE);
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) my_ss = ss;
    cluster_arrive();
    cluster_wait();
    if (threadIdx.x == 0) slb_trace_event(tr, 6, 4);
    float part[NORM_CLUSTER];                              // all remote loads first, then the sum
#pragma unroll
    for (unsigned c = 0; c < NORM_CLUSTER; ++c) part[c] = load_cluster_shared(&my_ss, c);
    float total = 0.f;
#pragma unroll
    for (unsigned c = 0; c < NORM_CLUSTER; ++c) total += part[c];
    cluster_arrive();                                      // this block has read the others' sums
    const float rstd = 1.0f / sqrtf(total / (float)h + eps);
    if (active) {
        store4(out + (size_t)r * h + i, make_float4(v.x * rstd * w.x, v.y * rstd * w.y,
                                                    v.z * rstd * w.z, v.w * rstd * w.w));
    }
    cluster_wait();                                        // nobody still reads this block's sum
    if (threadIdx.x == 0) slb_trace_event(tr, 6, SLB_TR_END);
}

// out[t, i] = silu(gate_i) * up_i, silu(z) = z / (1 + exp(-z)), in float32.  Layout of a
// row of gu: block == 0: all gates, then all ups (gate_i at i, up_i at inter + i);
// block > 0: gates and ups alternate in runs of `block` (gate_i at (i / block) * 2 * block +
// i % block, up_i `block` further), the order in which a product with row-interleaved
// weights delivers them.
// V elements per thread and step: 8 (bfloat16 with inter, block, ld_gu and ld_out multiples
// of 8: 16-byte accesses), 4 (multiples of 4) or 1.
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + expf(-g)) * u; }
// For results that are rounded to bfloat16: the hardware exponential and reciprocal (errors of
// a few 1e-7 relative, a thousand times below the rounding), a third of the instructions
// (42.4 against 47.8 us for 2,048 tokens of the 7B shape).
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
    return g * __frcp_rn(1.0f + __expf(-g)) * u;
}

template <typename T, int V>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              int ld_gu, int ld_out, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y;
    const T* row = gu + (size_t)t * ld_gu;
    T* o = out + (size_t)t * ld_out;
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (i >= inter) return;
    const int gi = block > 0 ? (i / block) * 2 * block + i % block : i;     // where gate_i sits
    const int ui = block > 0 ? gi + block : inter + i;                      // where up_i sits
    if constexpr (V == 8) {
        // two 16-byte loads of 8 bfloat16 each, one 16-byte store
        const uint4 graw = *reinterpret_cast<const uint4*>(row + gi);
        const uint4 uraw = *reinterpret_cast<const uint4*>(row + ui);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&graw);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uraw);
        uint4 res;
        __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
            r2[e] = __floats2bfloat162_rn(silu_mul_fast(g.x, u.x), silu_mul_fast(g.y, u.y));
        }
        *reinterpret_cast<uint4*>(o + i) = res;
    } else if constexpr (V == 4) {
        const float4 g = load4(row + gi), u = load4(row + ui);
        store4(o + i, make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z),
                                  silu_mul(g.w, u.w)));
    } else {
        o[i] = from_float<T>(silu_mul(to_float(row[gi]), to_float(row[ui])));
    }
}

static int norm_threads(int h) {
    int t = ((h + 15) / 16 + 31) / 32 * 32;        // about four vectors of 4 per thread, all in flight
    return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

template <typename T>
static int launch_embedding(const int* ids, const T* table, float* out, int T_, int h, int vocab,
                            float scale, cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (h <= 0 || vocab <= 0) return SLB_ERR_BAD_ARG;
    if (h % 4 == 0)
        return slb_launch(embedding_kernel<T, true>, dim3(T_), dim3(256), 0, st, ids, table, out, h, vocab, scale);
    return slb_launch(embedding_kernel<T, false>, dim3(T_), dim3(256), 0, st, ids, table, out, h, vocab, scale);
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float* resid, const TD* delta, const float* parts, int nparts,
                              long long part_stride, const float* pbias, const float* weight,
                              TO* out, const int* row_map, int rows, int h, float eps,
                              cudaStream_t st) {
    if (rows <= 0) return 0;
    if (h <= 0 || nparts < 0 || (nparts > 0 && parts == nullptr)) return SLB_ERR_BAD_ARG;
    const dim3 grid(rows), block(norm_threads(h));
    const bool vec = h % 4 == 0 && part_stride % 4 == 0;
#define SLB_NORM_LAUNCH(V, P)                                                                   \
    return slb_launch(add_rmsnorm_kernel<TD, TO, V, P>, grid, block, 0, st, resid, delta, parts, \
                      nparts, (size_t)part_stride, pbias, weight, out, row_map, h, eps, slb_trace_arg())
    if (nparts > 0) {
        if (vec) SLB_NORM_LAUNCH(true, true);
        SLB_NORM_LAUNCH(false, true);
    }
    if (vec) SLB_NORM_LAUNCH(true, false);
    SLB_NORM_LAUNCH(false, false);
#undef SLB_NORM_LAUNCH
}

template <typename T>
static int launch_swiglu(const T* gu, T* out, int T_, int inter, int ld_gu, int ld_out, int block,
                         cudaStream_t st) {
    if (T_ <= 0) return 0;
    if (inter <= 0 || T_ > 65535 || block < 0 || (block > 0 && inter % block)) return SLB_ERR_BAD_ARG;
    if constexpr (sizeof(T) == 2) {
        if (inter % 8 == 0 && block % 8 == 0 && ld_gu % 8 == 0 && ld_out % 8 == 0 &&
            ((uintptr_t)gu | (uintptr_t)out) % 16 == 0)
            return slb_launch(swiglu_kernel<T, 8>, dim3((inter / 8 + 255) / 256, T_), dim3(256), 0, st,
                              gu, out, inter, ld_gu, ld_out, block);
    }
    if (inter % 4 == 0 && block % 4 == 0 && ld_gu % 4 == 0 && ld_out % 4 == 0)
        return slb_launch(swiglu_kernel<T, 4>, dim3((inter / 4 + 255) / 256, T_), dim3(256), 0, st,
                          gu, out, inter, ld_gu, ld_out, block);
    return slb_launch(swiglu_kernel<T, 1>, dim3((inter + 255) / 256, T_), dim3(256), 0, st, gu,
                      out, inter, ld_gu, ld_out, block);
}

SLB_DEFINE_PDL_SWITCH

extern "C" {

// out[t] = table[ids[t]] * scale as float32 (scale 1 for architectures without an embedding scale)
int slb_embedding_f32(const int* ids, const float* table, float* out, int T, int h, int vocab,
                      float scale, cudaStream_t st) {
    return launch_embedding<float>(ids, table, out, T, h, vocab, scale, st);
}
int slb_embedding_bf16(const int* ids, const bf16* table, float* out, int T, int h, int vocab,
                       float scale, cudaStream_t st) {
    return launch_embedding<bf16>(ids, table, out, T, h, vocab, scale, st);
}

// logits [R, V] float32 (leading dimension ld), in place: multiplied by scale, then with
// cap > 0 bounded to cap * tanh(x / cap).
int slb_logit_transform(float* logits, int ld, int R, int V, float scale, float cap, cudaStream_t st) {
    if (R <= 0 || V <= 0) return 0;
    if (ld < V || R > 65535 || !(cap >= 0.f)) return SLB_ERR_BAD_ARG;
    const int blocks = (V + 1023) / 1024 < 64 ? (V + 1023) / 1024 : 64;
    return slb_launch(logit_transform_kernel, dim3(blocks, R), dim3(256), 0, st, logits, ld, V, scale, cap);
}

int slb_add_rmsnorm_f32(float* resid, const float* delta, const float* weight, float* out,
                        const int* row_map, int rows, int h, float eps, cudaStream_t st) {
    return launch_add_rmsnorm<float, float>(resid, delta, nullptr, 0, 0, nullptr, weight, out,
                                            row_map, rows, h, eps, st);
}
int slb_add_rmsnorm_bf16(float* resid, const bf16* delta, const float* weight, bf16* out,
                         const int* row_map, int rows, int h, float eps, cudaStream_t st) {
    return launch_add_rmsnorm<bf16, bf16>(resid, delta, nullptr, 0, 0, nullptr, weight, out, row_map,
                                          rows, h, eps, st);
}
// the update arrives as `nparts` float32 partial sums [nparts][rows_total][h] (+ bias)
int slb_add_rmsnorm_parts_bf16(float* resid, const float* parts, int nparts, long long part_stride,
                               const float* pbias, const float* weight, bf16* out,
                               const int* row_map, int rows, int h, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    const int chunk = ((h / 4 + NORM_CLUSTER - 1) / NORM_CLUSTER) * 4;     // columns per block
    if (nparts > 0 && parts != nullptr && h > 0 && h % 4 == 0 && part_stride % 4 == 0 &&
        chunk / 4 <= 1024 && rows <= 65535) {
        int threads = (chunk / 4 + 31) / 32 * 32;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(NORM_CLUSTER, rows);
        cfg.blockDim = dim3(threads);
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = NORM_CLUSTER;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = slb_pdl_enabled ? 2 : 1;
        return (int)cudaLaunchKernelEx(&cfg, add_rmsnorm_parts_cluster_kernel<bf16>, resid, parts, nparts,
                                       (size_t)part_stride, pbias, weight, out, row_map, h, chunk, eps,
                                       slb_trace_arg());
    }
    return launch_add_rmsnorm<bf16, bf16>(resid, nullptr, parts, nparts, part_stride, pbias, weight,
                                          out, row_map, rows, h, eps, st);
}

// block: 0, or the run length in which gates and ups alternate in a row of gu
int slb_swiglu_f32(const float* gu, float* out, int T, int inter, int ld_gu, int ld_out, int block,
                   cudaStream_t st) {
    return launch_swiglu<float>(gu, out, T, inter, ld_gu, ld_out, block, st);
}
int slb_swiglu_bf16(const bf16* gu, bf16* out, int T, int inter, int ld_gu, int ld_out, int block,
                    cudaStream_t st) {
    return launch_swiglu<bf16>(gu, out, T, inter, ld_gu, ld_out, block, st);
}

}  // extern "C"
