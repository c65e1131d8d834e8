// Shared helpers of the servelab_b200 kernels (sm_100a).
//
// Conventions of every launcher in this library:
//   * extern "C", plain pointers and ints, the CUDA stream as the last argument;
//   * the return value is 0 on success, a cudaError_t from the launch, or a
//     negative SLB_ERR_* code when the arguments are refused (never a wrong
//     result for an unsupported size);
//   * no launcher allocates device memory or synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SLB_ERR_BAD_ARG (-1)      // a size or pointer the kernel does not take
#define SLB_ERR_TOO_LARGE (-2)    // beyond a stated maximum

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions depends only on blockDim, so a row's result does not
// depend on what else is in the batch.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                      // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

static inline int slb_launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch ------------------------------------------
// Every kernel of this library calls pdl_wait() before it touches activations: it
// blocks until the preceding kernel of the stream has finished and its writes are
// visible.  pdl_launch_dependents() lets the next kernel be scheduled: the short
// kernels call it at their start (what follows them is a matrix product, which
// fetches its first weight tiles while they run), the long ones when their main
// loop is done (blocks that only wait would otherwise share the SMs with blocks
// that work).  What a kernel does before pdl_wait() may only read data that no
// kernel of the step writes (weights).  Launches go through
// slb_launch(), which sets the launch attribute when the switch is on; without
// the attribute both device calls do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

extern int slb_pdl_enabled;          // defined once per shared library (SLB_DEFINE_PDL_SWITCH)
// Switches of the long kernels (matrix products, decode attention), handed to them as one word:
//   SLB_FLAG_PDL_EARLY    they let their successor be scheduled at their start instead of after
//                         their main loop, so that its blocks become resident beside theirs
//                         wherever an SM has room and fetch their first weight tiles meanwhile
//                         (off: measured slower, 2.89 against 2.85 ms a batch-8 step of the 7B
//                         shape -- the early fetches compete with the running product for the
//                         memory, while fetches during its epilogue use time in which the
//                         memory is idle; early starts of only the attention, only the o and
//                         down products, or norms that release their successor late: 2.85,
//                         2.95, 2.88 ms.  The one exception that pays is in the kernel itself:
//                         the q|k|v product of a step of few tokens, whose successor -- the
//                         attention -- has look-ups and old keys to fetch meanwhile);
//   SLB_FLAG_EVICT_FIRST  what they stream once a step (weights, cached keys and values) is
//                         fetched with the L2 policy "evict first", so that the few hundred KB of
//                         activations between the kernels (the float32 residual stream above
//                         all) stay in the L2 cache instead of being pushed out by 400 MB of
//                         weights a layer and fetched from HBM again by the next norm.
enum { SLB_FLAG_PDL_EARLY = 1, SLB_FLAG_EVICT_FIRST = 2 };
extern int slb_kernel_flags;
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// ---- device timeline (measurements) -------------------------------------------
// With a buffer set (slb_set_trace), one thread of every block of the decode-step kernels
// records when the block started, when its wait for the preceding kernel returned, when its
// main loop was done and when it ended: the nanosecond timer of the device and the SM's
// number.  Every (launch, block, event) has a slot of its own, so recording is two plain
// stores and no atomic operation delays the thread that records:
//   slot = ((seq % SLB_TR_LAUNCHES) * SLB_TR_BLOCKS + block % SLB_TR_BLOCKS) * SLB_TR_EVENTS + event
//   buf[2 * slot] = timer, buf[2 * slot + 1] = kernel << 48 | event << 40 | sm << 24 | block
// (blocks beyond SLB_TR_BLOCKS share slots: of a large grid a sample is kept).  Without a
// buffer the calls cost a predicated branch.
constexpr int SLB_TR_LAUNCHES = 2048, SLB_TR_PER_LIBRARY = 512, SLB_TR_BLOCKS = 512, SLB_TR_EVENTS = 5;
struct SlbTraceArg {
    unsigned long long* buf;
    int seq;
};
extern unsigned long long* slb_trace_ptr;     // host side, per library; null = off
extern int slb_trace_seq, slb_trace_base;     // launches counted, first launch slot of this library
static inline SlbTraceArg slb_trace_arg() {
    SlbTraceArg a;
    a.buf = slb_trace_ptr;
    a.seq = slb_trace_ptr != nullptr ? slb_trace_base + slb_trace_seq++ % SLB_TR_PER_LIBRARY : 0;
    return a;
}
enum { SLB_TR_START = 0, SLB_TR_WAITED = 1, SLB_TR_LOOP_DONE = 2, SLB_TR_END = 3 };
__device__ __forceinline__ void slb_trace_event(const SlbTraceArg& tr, int kernel_id, int event) {
    if (tr.buf == nullptr) return;
    unsigned long long now;
    unsigned smid;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    const unsigned long long block = blockIdx.x + gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    const size_t slot = ((size_t)(tr.seq % SLB_TR_LAUNCHES) * SLB_TR_BLOCKS + (size_t)(block % SLB_TR_BLOCKS)) *
                            SLB_TR_EVENTS + (size_t)event;
    tr.buf[2 * slot] = now;
    tr.buf[2 * slot + 1] = ((unsigned long long)kernel_id << 48) | ((unsigned long long)event << 40) |
                           ((unsigned long long)(smid & 0xffff) << 24) | (block & 0xffffff);
}

// cudaFuncSetAttribute(max dynamic shared memory) once per device for one kernel: `done` is
// the caller's static word for that kernel (bit d = done on device d); the attribute belongs
// to the device that is current, so a process that uses several devices sets it on each.
template <typename Kernel>
static inline int slb_configure(unsigned long long* done, Kernel kernel, size_t smem) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SLB_ERR_BAD_ARG;
    if (dev >= 0 && dev < 64 && (*done >> dev & 1ull)) return 0;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) *done |= 1ull << dev;
    return 0;
}

template <typename... KArgs, typename... Args>
static inline int slb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = slb_pdl_enabled ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// A status word on the device with its host accessor `fn(reset)`: 0, or the code of the first
// event recorded since the last reset.  Reading synchronises with the device.
#define SLB_DEFINE_STATUS_WORD(var, fn)                                               \
    __device__ int var = 0;                                                           \
    extern "C" int fn(int reset) {                                                    \
        int v = 0;                                                                    \
        if (cudaMemcpyFromSymbol(&v, var, sizeof(int)) != cudaSuccess) return -1;     \
        if (reset && v != 0) {                                                        \
            const int zero = 0;                                                       \
            cudaMemcpyToSymbol(var, &zero, sizeof(int));                              \
        }                                                                             \
        return v;                                                                     \
    }

#define SLB_DEFINE_PDL_SWITCH                                                         \
    int slb_pdl_enabled = 0;                                                          \
    int slb_kernel_flags = SLB_FLAG_EVICT_FIRST;                                      \
    extern "C" int slb_set_pdl(int on) {                                              \
        const int old = slb_pdl_enabled;                                              \
        slb_pdl_enabled = on ? 1 : 0;                                                 \
        return old;                                                                   \
    }                                                                                 \
    extern "C" int slb_set_kernel_flags(int flags) {                                  \
        const int old = slb_kernel_flags;                                             \
        slb_kernel_flags = flags;                                                     \
        return old;                                                                   \
    }                                                                                 \
    unsigned long long* slb_trace_ptr = nullptr;                                      \
    int slb_trace_seq = 0;                                                            \
    int slb_trace_base = 0;                                                           \
    extern "C" int slb_set_trace(unsigned long long* buf, int library_index) {        \
        slb_trace_ptr = buf;                                                          \
        slb_trace_seq = 0;                                                            \
        slb_trace_base = (library_index % (SLB_TR_LAUNCHES / SLB_TR_PER_LIBRARY)) * SLB_TR_PER_LIBRARY; \
        return 0;                                                                     \
    }
