// Shared helpers of the kernels: element types, conversions, warp and block
// reductions, the launch-error convention of the exported functions.
//
// Every exported function is `extern "C"`, takes raw device pointers and a
// stream, and returns 0 or a negative code; the message of the last refusal is
// kept per thread and read with hos_last_error().  A function that cannot take
// a size says so and launches nothing.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

namespace hos {

typedef __nv_bfloat16 bf16;

enum DType : int { kF32 = 0, kBF16 = 1 };

// ---- error reporting ---------------------------------------------------------------
inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}
#define HOS_REFUSE(...)                                                     \
    do {                                                                    \
        snprintf(hos::error_buffer(), 512, __VA_ARGS__);                    \
        return -1;                                                          \
    } while (0)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        snprintf(error_buffer(), 512, "%s: %s", what, cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

// ---- bounded waits -------------------------------------------------------------------
// Every spin on an mbarrier has a limit.  A kernel whose wait runs out sets a flag on the device,
// writes one of these codes into a word of pinned host memory (if the host gave one: the
// hos_*_set_error_word functions), leaves and frees what it holds.  The host looks at the word
// after any synchronisation, at no cost, and raises an error instead of handing out the step's result.
enum GiveUpCode : int { kGiveUpGemmTc = 1, kGiveUpAttnDecode = 2, kGiveUpAttnPrefill = 3 };

// ---- programmatic dependent launch -----------------------------------------------------
// Kernels that follow one another on a stream are launched so that the next one may be set
// up (its CTAs placed, its prologue run) while the one before is still finishing.  Every such
// kernel calls pdl_wait() before it reads or writes anything in global memory: that returns
// once the kernels before it are complete and their writes visible.  pdl_launch_dependents()
// lets the kernel after it be set up in turn.  Both are no-ops for a kernel launched the
// ordinary way.  Measured on Gemma-2 2B sizes the attribute gains 3% on a
// 2,048-token prompt and loses 5% on a decode step at batch 8 (the step's kernels are short and
// the graph replays them back to back anyway, and the loss is the same 5% whether a kernel lets its
// successor go at its start or only after its main loop); issuing the first weight loads of the few-rows
// products before the wait changed nothing at batch 8 and gained 3% at batch 1.  So the engine
// switches it on for prompt steps and off for single-token steps (hos_set_pdl); HOS_PDL=0 or 1 in
// the environment fixes it for all.  One pair uses it always: the decode attention kernel fetches
// old keys while the q/k/v projection before it still runs (launch_ahead).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() { pdl_wait(); pdl_launch_dependents(); }

// Whether launch_pdl() launches ahead: the caller of the library says so per step (hos_set_pdl:
// prompts gain from it, single-token steps do not); HOS_PDL=1 or 0 in the environment overrides it.
inline int& pdl_state() {
    static int on = 0;
    return on;
}
inline int pdl_env() {
    static int env = -2;                   // -1: not set
    if (env == -2) {
        const char* e = getenv("HOS_PDL");
        env = (e && e[0]) ? (e[0] != '0' ? 1 : 0) : -1;
    }
    return env;
}
inline bool pdl_enabled() { return pdl_env() >= 0 ? pdl_env() == 1 : pdl_state() == 1; }
// One definition per library however many of its files include this header.
extern "C" __attribute__((weak)) void hos_set_pdl(int on) { hos::pdl_state() = on ? 1 : 0; }

// `ahead`: the kernel may be set up while the one before it on the stream is still running (if that
// one lets it: pdl_launch_dependents()), and must call pdl_wait() before it touches what that one wrote.
template <typename... KArgs, typename... Args>
inline void launch_ahead(bool ahead, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ahead ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);      // the caller reads the error with check_launch()
}

// The ordinary launch of every kernel here: ahead of its turn only if HOS_PDL asks for it.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    launch_ahead(pdl_enabled(), kernel, grid, block, smem, stream, args...);
}

inline int sm_count_cached() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// ---- conversions -------------------------------------------------------------------
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// ---- reductions --------------------------------------------------------------------
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
// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  All threads
// get the result.  Safe to call repeatedly with the same scratch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : 0.f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
    return warp_max(t);
}

// Soft-cap c*tanh(v/c), identity when c <= 0.  Precise tanhf: the 32-bit path
// and the logits use this one.
__device__ __forceinline__ float softcap_precise(float v, float c) {
    return c > 0.f ? c * tanhf(v / c) : v;
}

// tanh-form GELU: 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float c = 0.79788452f;   // sqrt(2/pi) as 32-bit arithmetic gives it: sqrtf(2.f / 3.14159274f)
    return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
}

// The gate activations of the bfloat16 products' epilogues, at a handful of instructions per element (an epilogue
// thread has a whole row's share of a tile to itself: with tanhf and an IEEE division, 60 instructions per
// element, the epilogue of a 256 x 128 gated tile took 6 us and was bound by instruction issue).
// gelu: 0.5 x (1 + tanh u) = x / (1 + e^{-2u}) exactly, u = sqrt(2/pi) (x + 0.044715 x^3); there is no cancellation
// where tanh u is near -1.  silu: x / (1 + e^{-x}).  ex2.approx and rcp.approx: a relative error of a few 1e-7.
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    constexpr float k0 = -2.f * 0.79788452f * 1.44269504f;       // -2 sqrt(2/pi) log2(e)
    constexpr float k1 = k0 * 0.044715f;
    return x * rcp_approx(1.f + ex2_approx(x * fmaf(k1, x * x, k0)));
}
__device__ __forceinline__ float silu_fast(float x) {
    return x * rcp_approx(1.f + ex2_approx(-1.44269504f * x));
}

}  // namespace hos
