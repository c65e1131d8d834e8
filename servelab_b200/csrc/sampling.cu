// Sampling on the device from float32 logits: greedy (argmax, lowest index among
// equal maxima), temperature, top-k and top-p.
//
// Semantics follow the reference sampler (servelab/engine/sampler.py:22-45):
// temperature 0 is argmax; else p = softmax(logits / max(T, 1e-6)); with top_k > 0
// only the k largest stay (top_p is then ignored, as in the reference); else with
// top_p < 1 entries are kept while their descending inclusive cumulative
// probability does not exceed top_p (the largest always stays); the rest is
// renormalised and one token drawn.
//
// The draw itself differs on purpose: instead of a host generator consumed in
// batch order, each draw takes u = Philox4x32-10(key = seed; counter = (position,
// stream)) and picks the first index, in index order, whose inclusive cumulative
// kept mass exceeds u * total.  A draw thus depends only on (seed, request
// stream, output position), never on the batch.
//
// One block of 1024 threads per row.  Thresholds for top-k / top-p are found by
// bisection on the order-preserving integer image of the scaled logits (32 passes
// over the row, exact for distinct values; equal values at the threshold all stay).
#include "common.cuh"

#define SM_THREADS 1024

__device__ __forceinline__ uint32_t philox_first_word(uint64_t seed, uint64_t stream,
                                                      uint32_t counter) {
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    uint32_t c0 = counter, c1 = (uint32_t)stream, c2 = (uint32_t)(stream >> 32), c3 = 0u;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    return c0;
}

__device__ __forceinline__ uint32_t ordered_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// (value, index) max with the lower index winning ties; result to all threads
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        float tv = lane < nw ? sv[lane] : -INFINITY;
        int ti = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, tv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, ti, o);
            if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
        }
        if (lane == 0) { sv[32] = tv; si[32] = ti; }
    }
    __syncthreads();
    v = sv[32];
    idx = si[32];
}

__global__ void __launch_bounds__(SM_THREADS) sample_rows_kernel(
    const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p,
    const unsigned long long* __restrict__ seed, const unsigned long long* __restrict__ stream,
    const int* __restrict__ position, int* __restrict__ out) {
    __shared__ float scratch[33];
    pdl_wait();
    __shared__ float sv[33];
    __shared__ int si[33];
    __shared__ float warp_tot[32];
    __shared__ int result;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    const float temp = temperature ? temperature[row] : 0.f;

    // greedy: first index of the maximum (also the fallback of a draw)
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    if (V % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
        // four values a load (a block reads its 600 KB row three times faster); every thread still
        // visits its indices in ascending order
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (int i = tid; i < V / 4; i += SM_THREADS) {
            const float4 v = x4[i];
            if (v.x > bv) { bv = v.x; bi = 4 * i; }
            if (v.y > bv) { bv = v.y; bi = 4 * i + 1; }
            if (v.z > bv) { bv = v.z; bi = 4 * i + 2; }
            if (v.w > bv) { bv = v.w; bi = 4 * i + 3; }
        }
    } else {
        for (int i = tid; i < V; i += SM_THREADS) {
            const float v = x[i];
            if (v > bv) { bv = v; bi = i; }       // strided visit keeps the lowest index per thread
        }
    }
    block_argmax(bv, bi, sv, si);
    if (bi < 0 || bi >= V) bi = 0;                // a row of NaNs: keep a valid id
    if (temp == 0.f) {
        if (tid == 0) out[row] = bi;
        return;
    }

    const float tc = fmaxf(temp, 1e-6f);
    const float mx = bv / tc;
    float zs = 0.f;
    for (int i = tid; i < V; i += SM_THREADS) zs += expf(x[i] / tc - mx);
    const float Z = block_sum(zs, scratch);

    // threshold key: tokens with ordered_key(x/tc) >= thr stay
    uint32_t thr = 0u;
    const int k = top_k ? top_k[row] : -1;
    const float pp = top_p ? top_p[row] : 1.f;
    if (k > 0 && k < V) {
        uint32_t prefix = 0u;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            float cnt = 0.f;
            for (int i = tid; i < V; i += SM_THREADS) cnt += ordered_key(x[i] / tc) >= cand ? 1.f : 0.f;
            cnt = block_sum(cnt, scratch);        // exact: counts below 2^24
            if (cnt >= (float)k) prefix = cand;
        }
        thr = prefix;
    } else if (k <= 0 && pp < 1.f) {
        const float limit = pp * Z;
        uint32_t prefix = 0u;                     // largest key whose tail mass still exceeds the limit
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            float mass = 0.f;
            for (int i = tid; i < V; i += SM_THREADS) {
                const float s = x[i] / tc;
                if (ordered_key(s) >= cand) mass += expf(s - mx);
            }
            mass = block_sum(mass, scratch);
            if (mass > limit) prefix = cand;
        }
        const uint32_t kmax = ordered_key(mx);
        thr = prefix == 0xffffffffu ? kmax : min(prefix + 1u, kmax);
    }

    // inverse CDF in index order over contiguous chunks
    const int chunk = (V + SM_THREADS - 1) / SM_THREADS;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
    float mine = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float s = x[i] / tc;
        if (ordered_key(s) >= thr) mine += expf(s - mx);
    }
    // inclusive scan of the chunk sums
    const int lane = tid & 31, warp = tid >> 5;
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (tid == 0) result = -1;
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    float before = 0.f;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    float total = 0.f;
    for (int w = 0; w < SM_THREADS / 32; ++w) total += warp_tot[w];
    incl += before;
    float excl = __shfl_up_sync(0xffffffffu, incl, 1);   // the previous thread's inclusive sum
    if (lane == 0) excl = before;

    const uint32_t word = philox_first_word(seed[row], stream[row], (uint32_t)position[row]);
    const float u = (float)(word >> 8) * (1.0f / 16777216.0f);
    float target = u * total;
    if (target >= total) target = nextafterf(total, 0.f);
    if (mine > 0.f && excl <= target && incl > target) {
        float run = excl;
        int pick = -1;
        for (int i = lo; i < hi; ++i) {
            const float s = x[i] / tc;
            if (ordered_key(s) >= thr) {
                run += expf(s - mx);
                pick = i;                          // last kept index so far
                if (run > target) break;
            }
        }
        result = pick;
    }
    __syncthreads();
    if (tid == 0) out[row] = result >= 0 ? result : bi;
}

extern "C" {
// temperature/top_k/top_p/seed/stream/position are per-row device arrays;
// temperature == nullptr means every row is greedy.
int slb_sample_rows(const float* logits, int ld, int R, int V, const float* temperature,
                    const int* top_k, const float* top_p, const unsigned long long* seed,
                    const unsigned long long* stream, const int* position, int* out,
                    cudaStream_t st) {
    if (R <= 0) return 0;
    if (V <= 0 || ld < V) return SLB_ERR_BAD_ARG;
    if (temperature && (!seed || !stream || !position)) return SLB_ERR_BAD_ARG;
    return slb_launch(sample_rows_kernel, dim3(R), dim3(SM_THREADS), 0, st, logits, ld, V,
                      temperature, top_k, top_p, seed, stream, position, out);
}
}
