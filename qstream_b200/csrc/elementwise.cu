// Error reporting, embedding lookup, LayerNorm, row gather and residual add.
//
// Each kernel has a plain reference with the same formula in tests/plain_gptj.py.
#include "common.cuh"

#include <stdarg.h>
#include <stdio.h>

// ----------------------------------------------------------------------------- errors

static thread_local char g_error[512] = "";

int qs_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int qs_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "%s: %s", what, cudaGetErrorString(e));
    return QS_OK;
}

QS_API const char* qs_last_error(void) { return g_error; }

QS_API int qs_abi_version(void) { return 1; }

// ----------------------------------------------------------------------------- embedding

// out[t, :] = table[token[t], :]   (QStream src/engine.c:710-765; no position term).
// Token ids are checked by the caller; an id outside the table is clamped here so
// that a bad id can never read outside the table.
template <typename TO, typename TT>
__global__ void embedding_kernel(TO* __restrict__ out, const TT* __restrict__ table,
                                 const int32_t* __restrict__ tokens, int D, int V) {
    const int t = blockIdx.x;
    int id = tokens[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const TT* row = table + (size_t)id * D;
    TO* dst = out + (size_t)t * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = from_f32<TO>(to_f32(row[i]));
}

QS_API int qs_embedding(void* out, int out_dtype, const void* table, int table_dtype,
                        const int32_t* tokens, int T, int D, int V, cudaStream_t stream) {
    if (T == 0) return QS_OK;
    QS_REQUIRE(T > 0 && D > 0 && V > 0, "embedding: bad sizes T=%d D=%d V=%d", T, D, V);
    const int threads = D >= 1024 ? 256 : 128;
#define LAUNCH(TO, TT) embedding_kernel<TO, TT><<<T, threads, 0, stream>>>( \
        (TO*)out, (const TT*)table, tokens, D, V)
    if (out_dtype == QS_F32 && table_dtype == QS_F32) LAUNCH(float, float);
    else if (out_dtype == QS_F32 && table_dtype == QS_BF16) LAUNCH(float, __nv_bfloat16);
    else if (out_dtype == QS_BF16 && table_dtype == QS_F32) LAUNCH(__nv_bfloat16, float);
    else if (out_dtype == QS_BF16 && table_dtype == QS_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return qs_fail(QS_ERR_INVALID_INPUT, "embedding: unknown dtype %d/%d", out_dtype, table_dtype);
#undef LAUNCH
    return qs_check_launch("embedding");
}

// ----------------------------------------------------------------------------- LayerNorm

// mean = sum x / D; var = sum (x - mean)^2 / D (two passes); y = (x - mean) / sqrt(var + eps) * w + b
// (QStream src/kernels_scalar.c:151-171).  Statistics in 32-bit whatever the storage type.
// One block per row; the row is held in shared memory as 32-bit floats.
template <typename T>
__global__ void layernorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                                 const void* __restrict__ w, int w_dtype,
                                 const void* __restrict__ b, int b_dtype,
                                 int D, float eps, size_t ldx, size_t ldo) {
    extern __shared__ float row[];
    __shared__ float scratch[33];
    grid_dep_launch();
    grid_dep_wait();
    const T* src = x + (size_t)blockIdx.x * ldx;
    T* dst = out + (size_t)blockIdx.x * ldo;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = to_f32(src[i]);
        row[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)D;
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float d = row[i] - mean;
        q += d * d;
    }
    const float var = block_sum(q, scratch) / (float)D;
    const float rstd = 1.0f / sqrtf(var + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float y = (row[i] - mean) * rstd * load_as_f32(w, w_dtype, i);
        if (b) y += load_as_f32(b, b_dtype, i);
        dst[i] = from_f32<T>(y);
    }
}

// The same for bfloat16 rows whose width is a multiple of 8: one block of 128 threads per row, the row
// kept in registers as NV 16-byte pieces per thread (width <= 1024 * NV), all of a thread's loads in
// flight at once, statistics by the block's fixed-order sum.  At 40 registers sixteen blocks share an SM,
// so 2,048 rows are one wave.  (One warp per row with the whole row in a lane's registers, 160 of them,
// moved 1.5 TB/s on 2,048 rows of 4,096.)  EARLY (few rows, a decode step): the thread's pieces of weight and
// bias, which no kernel writes, are fetched before the wait for the previous kernel instead of after the two
// sums, where their way from memory would be on the step's critical path; the arithmetic is the same.
template <int NV, bool EARLY>
__global__ void __launch_bounds__(128)
layernorm_row_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                     const void* __restrict__ w, int w_dtype, const void* __restrict__ b, int b_dtype,
                     int D, float eps, size_t ldx, size_t ldo) {
    __shared__ float scratch[33];
    grid_dep_launch();
    float we[EARLY ? NV : 1][8], be[EARLY ? NV : 1][8];
    if (EARLY) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (i * 128 + threadIdx.x) * 8;
            if (c < D) {
                load8_as_f32(w, w_dtype, c, we[i]);
                if (b) load8_as_f32(b, b_dtype, c, be[i]);
            }
        }
    }
    grid_dep_wait();
    const __nv_bfloat16* src = x + (size_t)blockIdx.x * ldx;
    uint4 raw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 128 + threadIdx.x) * 8;
        raw[i] = c < D ? *reinterpret_cast<const uint4*>(src + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) s += __uint_as_float(u[j] << 16) + __uint_as_float(u[j] & 0xffff0000u);
    }
    const float mean = block_sum(s, scratch) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if ((i * 128 + threadIdx.x) * 8 < D) {
            const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float d0 = __uint_as_float(u[j] << 16) - mean, d1 = __uint_as_float(u[j] & 0xffff0000u) - mean;
                q += d0 * d0 + d1 * d1;
            }
        }
    const float rstd = 1.0f / sqrtf(block_sum(q, scratch) / (float)D + eps);
    __nv_bfloat16* dst = out + (size_t)blockIdx.x * ldo;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 128 + threadIdx.x) * 8;
        if (c < D) {
            const uint32_t u[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
            uint32_t o[4];
            float wf[8], bf[8];
            if (EARLY) {
#pragma unroll
                for (int j = 0; j < 8; ++j) { wf[j] = we[i][j]; bf[j] = be[i][j]; }
            } else {
                load8_as_f32(w, w_dtype, c, wf);
                if (b) load8_as_f32(b, b_dtype, c, bf);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float y0 = (__uint_as_float(u[j] << 16) - mean) * rstd * wf[2 * j];
                float y1 = (__uint_as_float(u[j] & 0xffff0000u) - mean) * rstd * wf[2 * j + 1];
                if (b) { y0 += bf[2 * j]; y1 += bf[2 * j + 1]; }
                const __nv_bfloat162 pb = __floats2bfloat162_rn(y0, y1);
                o[j] = *reinterpret_cast<const uint32_t*>(&pb);
            }
            *reinterpret_cast<uint4*>(dst + c) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

QS_API int qs_layernorm(void* out, const void* x, int dtype, const void* w, int w_dtype,
                        const void* b, int b_dtype, int rows, int D, float eps,
                        long long ldx, long long ldo, int settled, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && D > 0, "layernorm: bad sizes rows=%d D=%d", rows, D);
    // bfloat16 rows of 16-byte pieces: the row in registers, whatever the number of rows (prefill and decode
    // steps then run the same arithmetic)
    if (dtype == QS_BF16 && D % 8 == 0 && D <= 8192 && ldx % 8 == 0 && ldo % 8 == 0 &&
        ((uintptr_t)x % 16) == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)w % (w_dtype == QS_F32 ? 32 : 16)) == 0 &&
        (!b || ((uintptr_t)b % (b_dtype == QS_F32 ? 32 : 16)) == 0)) {
        const int nv = (D + 1023) / 1024;
#define GO1(NV, EARLY) qs_launch_dependent(layernorm_row_kernel<NV, EARLY>, dim3(rows), dim3(128), 0, stream, (__nv_bfloat16*)out, \
            (const __nv_bfloat16*)x, w, w_dtype, b, b_dtype, D, eps, (size_t)ldx, (size_t)ldo)
#define GO(NV) do { if (rows <= 64 && settled) GO1(NV, true); else GO1(NV, false); } while (0)
        if (nv <= 1) GO(1); else if (nv <= 2) GO(2); else if (nv <= 4) GO(4); else GO(8);
#undef GO1
#undef GO
        return qs_check_launch("layernorm");
    }
    const size_t smem = (size_t)D * sizeof(float);
    QS_REQUIRE(smem <= 200 * 1024, "layernorm: width %d does not fit one block's shared memory (max %d)",
               D, 200 * 1024 / 4);
    // few rows: many threads per row for latency; many rows: smaller blocks, more rows per SM
    const int threads = rows >= 512 ? (D >= 1024 ? 256 : 128) : (D >= 4096 ? 1024 : (D >= 2048 ? 512 : (D >= 512 ? 256 : 128)));
    cudaError_t e = cudaSuccess;
    if (dtype == QS_F32) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = qs_launch_dependent(layernorm_kernel<float>, dim3(rows), dim3(threads), smem, stream,
            (float*)out, (const float*)x, w, w_dtype, b, b_dtype, D, eps, (size_t)ldx, (size_t)ldo);
    } else if (dtype == QS_BF16) {
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(layernorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = qs_launch_dependent(layernorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, stream,
            (__nv_bfloat16*)out, (const __nv_bfloat16*)x, w, w_dtype, b, b_dtype, D, eps, (size_t)ldx, (size_t)ldo);
    } else {
        return qs_fail(QS_ERR_INVALID_INPUT, "layernorm: unknown dtype %d", dtype);
    }
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "layernorm: %s", cudaGetErrorString(e));
    return qs_check_launch("layernorm");
}

// ----------------------------------------------------------------------------- gather rows

// out[i, :] = x[rows[i], :]: the rows whose logits are wanted, picked before the
// final norm and the head so that only they pay for the vocabulary projection.
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ x,
                                   const int32_t* __restrict__ rows, int D, size_t ldx) {
    const T* src = x + (size_t)rows[blockIdx.x] * ldx;
    T* dst = out + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
}

QS_API int qs_gather_rows(void* out, const void* x, int dtype, const int32_t* rows, int n, int D,
                          long long ldx, cudaStream_t stream) {
    if (n == 0) return QS_OK;
    QS_REQUIRE(n > 0 && D > 0, "gather_rows: bad sizes n=%d D=%d", n, D);
    if (dtype == QS_F32) gather_rows_kernel<float><<<n, 256, 0, stream>>>((float*)out, (const float*)x, rows, D, (size_t)ldx);
    else if (dtype == QS_BF16) gather_rows_kernel<__nv_bfloat16><<<n, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)x, rows, D, (size_t)ldx);
    else return qs_fail(QS_ERR_INVALID_INPUT, "gather_rows: unknown dtype %d", dtype);
    return qs_check_launch("gather_rows");
}

// ----------------------------------------------------------------------------- residual add

// out = a + b (+ c), summed in 32-bit and rounded once.  For parts that cannot add
// the residual in their last kernel.
template <typename T>
__global__ void add_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                           const T* __restrict__ c, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = to_f32(a[i]) + to_f32(b[i]);
        if (c) v += to_f32(c[i]);
        out[i] = from_f32<T>(v);
    }
}

QS_API int qs_add(void* out, const void* a, const void* b, const void* c, int dtype, long long n,
                  cudaStream_t stream) {
    if (n == 0) return QS_OK;
    QS_REQUIRE(n > 0, "add: bad size %lld", n);
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    if (dtype == QS_F32) add_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, (const float*)a, (const float*)b, (const float*)c, (size_t)n);
    else if (dtype == QS_BF16) add_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, (size_t)n);
    else return qs_fail(QS_ERR_INVALID_INPUT, "add: unknown dtype %d", dtype);
    return qs_check_launch("add");
}
