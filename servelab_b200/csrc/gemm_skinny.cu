// Weight-streaming matrix product for a handful of tokens (decode steps):
//   out[M, N] = x[M, K] . W[N, K]^T (+ bias[N]),  bfloat16 in, float32 accumulate,
//   bfloat16 or float32 out,  M <= 64,  K a multiple of 8.
//
// With few tokens the product is bound by reading W once from HBM.  Each block
// owns 16*RT rows of W; its 8 warps split K among themselves (a warp walks its K
// range in chunks of 32), so even a narrow output has enough warps streaming.
// Rows of W are the M side of mma.sync.m16n8k16, the tokens are the N side (8 per
// tile).  A lane fetches 16 contiguous bytes of "its" W row (rows g and g+8) and of
// "its" token's activations and feeds them to two MMAs: the k index inside a chunk
// is permuted the same way for both operands, which leaves the dot product
// unchanged and lets every quad of lanes read 64 contiguous bytes of a row.  W is
// loaded with the no-allocate hint (it is used once), x through L1.  The warps'
// partial sums meet in shared memory in a fixed order, so results are
// deterministic and a token's result does not depend on the other tokens.
//
// Reference analogue: F.linear in the decode step (servelab/parallel/
// tp_model.py:48-53,67-68,115-119), which the reference leaves to the library.
#include "common.cuh"

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// RT: 16-row tiles of W per block; NT: 8-token tiles (M <= 8*NT).
template <int RT, int NT, typename TO>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(
    const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw, TO* __restrict__ out,
    int ldo, const float* __restrict__ bias, int M, int N, int K) {
    __shared__ float red[SK_WARPS][RT * 16][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int n0 = blockIdx.x * RT * 16;

    // this warp's K range, in chunks of 32
    const int chunks = (K + 31) / 32;
    const int per_warp = (chunks + SK_WARPS - 1) / SK_WARPS;
    const int c_begin = warp * per_warp;
    const int c_end = min(chunks, c_begin + per_warp);

    const bf16* wrow[RT][2];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        wrow[r][0] = W + (size_t)min(n0 + r * 16 + g, N - 1) * ldw;
        wrow[r][1] = W + (size_t)min(n0 + r * 16 + g + 8, N - 1) * ldw;
    }
    const bf16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        xok[t] = t * 8 + g < M;
        xrow[t] = x + (size_t)(xok[t] ? t * 8 + g : 0) * ldx;
    }

    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[r][t][e] = 0.f;

    constexpr int UNROLL = (RT * NT >= 8) ? 1 : ((RT >= 4 || NT >= 4) ? 2 : 4);
    uint4 wv[UNROLL][RT][2];
    // The weights of the first round are fetched before waiting for the kernel that
    // produces x: W is written by no kernel, so this read may overlap its tail.
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int k = (c_begin + u) * 32 + tig * 8;
        const bool kok = (c_begin + u) < c_end && k < K;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            wv[u][r][0] = kok ? ld_stream16(wrow[r][0] + k) : make_uint4(0, 0, 0, 0);
            wv[u][r][1] = kok ? ld_stream16(wrow[r][1] + k) : make_uint4(0, 0, 0, 0);
        }
    }
    pdl_wait();
    for (int c0 = c_begin; c0 < c_end; c0 += UNROLL) {
        uint4 xv[UNROLL][NT];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (c0 + u) * 32 + tig * 8;
            const bool kok = (c0 + u) < c_end && k < K;
            if (c0 != c_begin) {
#pragma unroll
                for (int r = 0; r < RT; ++r) {
                    wv[u][r][0] = kok ? ld_stream16(wrow[r][0] + k) : make_uint4(0, 0, 0, 0);
                    wv[u][r][1] = kok ? ld_stream16(wrow[r][1] + k) : make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int t = 0; t < NT; ++t)
                xv[u][t] = (kok && xok[t]) ? __ldg(reinterpret_cast<const uint4*>(xrow[t] + k))
                                           : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    mma16816(acc[r][t], wv[u][r][0].x, wv[u][r][1].x, wv[u][r][0].y, wv[u][r][1].y,
                             xv[u][t].x, xv[u][t].y);
                    mma16816(acc[r][t], wv[u][r][0].z, wv[u][r][1].z, wv[u][r][0].w, wv[u][r][1].w,
                             xv[u][t].z, xv[u][t].w);
                }
    }

    pdl_launch_dependents();                 // the next kernel may start its prologue now
    // partial sums of the warps -> shared memory -> fixed-order sum -> out
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            red[warp][r * 16 + g][t * 8 + tig * 2] = acc[r][t][0];
            red[warp][r * 16 + g][t * 8 + tig * 2 + 1] = acc[r][t][1];
            red[warp][r * 16 + g + 8][t * 8 + tig * 2] = acc[r][t][2];
            red[warp][r * 16 + g + 8][t * 8 + tig * 2 + 1] = acc[r][t][3];
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < RT * 16 * NT * 8; idx += SK_THREADS) {
        const int row = idx % (RT * 16), tok = idx / (RT * 16);
        const int n = n0 + row;
        if (n >= N || tok >= M) continue;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) sum += red[w][row][tok];
        if (bias) sum += bias[n];
        out[(size_t)tok * ldo + n] = from_float<TO>(sum);
    }
}

template <int RT, int NT, typename TO>
static int launch(const bf16* x, int ldx, const bf16* W, int ldw, TO* out, int ldo,
                  const float* bias, int M, int N, int K, cudaStream_t st) {
    return slb_launch(gemm_skinny_kernel<RT, NT, TO>, dim3((N + RT * 16 - 1) / (RT * 16)),
                      dim3(SK_THREADS), 0, st, x, ldx, W, ldw, out, ldo, bias, M, N, K);
}

template <int NT, typename TO>
static int launch_rt(int rt, const bf16* x, int ldx, const bf16* W, int ldw, TO* out, int ldo,
                     const float* bias, int M, int N, int K, cudaStream_t st) {
    if constexpr (NT <= 2) {
        if (rt >= 4) return launch<4, NT, TO>(x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
    }
    if constexpr (NT <= 4) {
        if (rt >= 2) return launch<2, NT, TO>(x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
    }
    return launch<1, NT, TO>(x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
}

// rt_hint: 16-row tiles of W per block (1, 2 or 4); 0 lets the launcher choose.
template <typename TO>
static int dispatch(const bf16* x, int ldx, const bf16* W, int ldw, TO* out, int ldo,
                    const float* bias, int M, int N, int K, int rt_hint, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return SLB_ERR_BAD_ARG;
    if (((uintptr_t)x | (uintptr_t)W) % 16) return SLB_ERR_BAD_ARG;
    if (M > 64) return SLB_ERR_TOO_LARGE;
    // wide outputs take more rows per block, so the activations are re-read less often
    int rt = rt_hint > 0 ? rt_hint : 1;          // one tile per block measured fastest
    if (M <= 8) return launch_rt<1, TO>(rt, x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
    if (M <= 16) return launch_rt<2, TO>(rt, x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
    if (M <= 32) return launch_rt<4, TO>(rt, x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
    return launch_rt<8, TO>(rt, x, ldx, W, ldw, out, ldo, bias, M, N, K, st);
}

}  // namespace

extern "C" {
// out_f32 != 0: `out` is float32, else bfloat16
int slb_gemm_skinny_bf16(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo,
                         const float* bias, int out_f32, int M, int N, int K, int rt_hint,
                         cudaStream_t st) {
    if (out_f32)
        return dispatch<float>(x, ldx, W, ldw, (float*)out, ldo, bias, M, N, K, rt_hint, st);
    return dispatch<bf16>(x, ldx, W, ldw, (bf16*)out, ldo, bias, M, N, K, rt_hint, st);
}
int slb_gemm_skinny_max_tokens() { return 64; }
}
