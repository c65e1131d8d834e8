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

// out[t, :] = table[ids[t], :] as float32.  An id outside [0, vocab) yields a
// row of zeros (callers validate ids on the host).
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int h, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * h;
    float* o = out + (size_t)t * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) o[i] = ok ? to_float(row[i]) : 0.f;
}

// One block per output row r.  src = row_map ? row_map[r] : r.
//   v = resid[src] + delta[src]        (delta may be null)
//   if no row_map: resid[src] = v      (the stream is updated in place)
//   out[r] = v * (1/sqrt(mean(v^2) + eps)) * weight
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const float* __restrict__ weight, TO* __restrict__ out,
                                   const int* __restrict__ row_map, int h, float eps) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int src = row_map ? row_map[r] : r;
    float* x = resid + (size_t)src * h;
    const TD* d = delta ? delta + (size_t)src * h : nullptr;
    const bool write_back = (row_map == nullptr) && (d != nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float v = x[i];
        if (d) v += to_float(d[i]);
        if (write_back) x[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)h + eps);
    TO* o = out + (size_t)r * h;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float v = x[i];
        if (d && !write_back) v += to_float(d[i]);
        o[i] = from_float<TO>(v * rstd * weight[i]);
    }
}

// out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(z) = z / (1 + exp(-z)), in float32.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              int ld_gu, int ld_out) {
    const int t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const float g = to_float(gu[(size_t)t * ld_gu + i]);
    const float u = to_float(gu[(size_t)t * ld_gu + inter + i]);
    out[(size_t)t * ld_out + i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

static int norm_threads(int h) {
    int t = 32;
    while (t < 1024 && t * 4 < h) t <<= 1;
    return t;
}

extern "C" {

int slb_embedding_f32(const int* ids, const float* table, float* out, int T, int h, int vocab,
                      cudaStream_t st) {
    if (T <= 0) return 0;
    if (h <= 0 || vocab <= 0) return SLB_ERR_BAD_ARG;
    embedding_kernel<float><<<T, 256, 0, st>>>(ids, table, out, h, vocab);
    return slb_launch_status();
}
int slb_embedding_bf16(const int* ids, const bf16* table, float* out, int T, int h, int vocab,
                       cudaStream_t st) {
    if (T <= 0) return 0;
    if (h <= 0 || vocab <= 0) return SLB_ERR_BAD_ARG;
    embedding_kernel<bf16><<<T, 256, 0, st>>>(ids, table, out, h, vocab);
    return slb_launch_status();
}

int slb_add_rmsnorm_f32(float* resid, const float* delta, const float* weight, float* out,
                        const int* row_map, int rows, int h, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (h <= 0) return SLB_ERR_BAD_ARG;
    add_rmsnorm_kernel<float, float><<<rows, norm_threads(h), 0, st>>>(resid, delta, weight, out,
                                                                      row_map, h, eps);
    return slb_launch_status();
}
int slb_add_rmsnorm_bf16(float* resid, const bf16* delta, const float* weight, bf16* out,
                         const int* row_map, int rows, int h, float eps, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (h <= 0) return SLB_ERR_BAD_ARG;
    add_rmsnorm_kernel<bf16, bf16><<<rows, norm_threads(h), 0, st>>>(resid, delta, weight, out,
                                                                    row_map, h, eps);
    return slb_launch_status();
}

int slb_swiglu_f32(const float* gu, float* out, int T, int inter, int ld_gu, int ld_out,
                   cudaStream_t st) {
    if (T <= 0) return 0;
    if (inter <= 0 || T > 65535) return SLB_ERR_BAD_ARG;
    swiglu_kernel<float><<<dim3((inter + 255) / 256, T), 256, 0, st>>>(gu, out, inter, ld_gu, ld_out);
    return slb_launch_status();
}
int slb_swiglu_bf16(const bf16* gu, bf16* out, int T, int inter, int ld_gu, int ld_out,
                    cudaStream_t st) {
    if (T <= 0) return 0;
    if (inter <= 0 || T > 65535) return SLB_ERR_BAD_ARG;
    swiglu_kernel<bf16><<<dim3((inter + 255) / 256, T), 256, 0, st>>>(gu, out, inter, ld_gu, ld_out);
    return slb_launch_status();
}

}  // extern "C"
