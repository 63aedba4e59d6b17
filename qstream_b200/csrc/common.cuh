// Shared declarations of the kernel library: element types, error reporting, loads.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and the CUDA
// stream to launch on, allocates nothing, and returns 0 or a non-zero code after
// storing a message that `qs_last_error()` returns (the manner of QStream's
// error code plus detail string, src/error.c:14-53).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>

#define QS_API extern "C" __attribute__((visibility("default")))

enum QsDtype { QS_F32 = 0, QS_BF16 = 1 };

enum QsActivation { QS_ACT_NONE = 0, QS_ACT_GELU_TANH = 1, QS_ACT_GELU_ERF = 2 };

// Codes follow QsError in errors.py (QStream include/qsf/error.h:14-32).
enum { QS_OK = 0, QS_ERR_INVALID_INPUT = 11, QS_ERR_INTERNAL = 15 };

int qs_fail(int code, const char* fmt, ...);
int qs_check_launch(const char* what);

#define QS_REQUIRE(cond, ...) do { if (!(cond)) return qs_fail(QS_ERR_INVALID_INPUT, __VA_ARGS__); } while (0)

// Programmatic dependent launch.  A kernel calls `grid_dep_launch()` once it no longer minds the next
// kernel of the stream being scheduled beside it, and a kernel launched with `qs_launch_dependent`
// calls `grid_dep_wait()` before it first touches memory the previous kernel wrote (or writes memory
// the previous kernel read): what precedes the wait - barrier set-up, TMEM allocation, loads of
// weights that no kernel writes - overlaps the previous kernel's tail.  Every such kernel executes the
// wait before it ends, so completion of a kernel implies completion of all kernels before it.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
cudaError_t qs_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A vector operand (norm weight, bias) whose stored type is known only at run time.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
    return dtype == QS_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// Needs 16-byte (bfloat16) or 32-byte (float32) alignment of p + c.
// Eight consecutive elements of a weight or bias vector stored as float32 or bfloat16 (c a multiple of 8).
__device__ __forceinline__ void load8_as_f32(const void* p, int dtype, int c, float (&f)[8]) {
    if (dtype == QS_F32) {
        const float4 a = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + c)[0];
        const float4 b = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + c)[1];
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + c);
        const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) { f[2 * j] = __uint_as_float(u[j] << 16); f[2 * j + 1] = __uint_as_float(u[j] & 0xffff0000u); }
    }
}

__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
    if (dtype == QS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

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

// Sum over a block in a fixed order (warp butterflies, then the warp totals in
// index order), so the result does not depend on scheduling.  `scratch` holds at
// least 33 floats.  All threads get the total.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = 0.f;
        for (int i = 0; i < n_warps; ++i) t += scratch[i];
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float gelu_tanh(float v) {
    // 0.5 v (1 + tanh(sqrt(2/pi) (v + 0.044715 v^3))): QStream src/kernels_scalar.c:135-142
    const float c = 0.7978845608028654f;
    return 0.5f * v * (1.0f + tanhf(c * (v + 0.044715f * v * v * v)));
}

// The same function with tanh(u) = 1 - 2 / (exp(2u) + 1) on the fast exponential: a handful of
// instructions instead of tanhf's forty, absolute error below 1e-6.  For epilogues that must keep up
// with the tensor cores; the float32 engine uses gelu_tanh.
__device__ __forceinline__ float gelu_tanh_fast(float v) {
    const float c = 0.7978845608028654f;
    const float u = c * (v + 0.044715f * v * v * v);
    const float t = 1.0f - __fdividef(2.0f, __expf(2.0f * u) + 1.0f);
    return 0.5f * v * (1.0f + t);
}

__device__ __forceinline__ float gelu_erf(float v) {
    return 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
}

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == QS_ACT_GELU_TANH) return gelu_tanh(v);
    if (act == QS_ACT_GELU_ERF) return gelu_erf(v);
    return v;
}

__device__ __forceinline__ float apply_activation_fast(float v, int act) {
    if (act == QS_ACT_GELU_TANH) return gelu_tanh_fast(v);
    if (act == QS_ACT_GELU_ERF) return gelu_erf(v);
    return v;
}
