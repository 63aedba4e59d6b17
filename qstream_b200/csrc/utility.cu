// Utility kernels: seeded random fill, type conversion at upload, finite check, canary words.
//
// QStream has none of these as kernels: its weights come from a file only, its
// `check_nan` switch scans a layer's output on the host (src/engine.c:1176-1187), and
// its arena has no guard words.  Each kernel here has a host twin with the same
// arithmetic (weights/random_init.py for the generator; numpy in the tests).
#include "common.cuh"
#include "sm100.cuh"

// ----------------------------------------------------------------------------- random fill
//
// Element i of a tensor is a pure function of (key, i): bits = mix(key + (i + 1) * golden), the
// SplitMix64 stream of seed `key` at place i.  From the bits: m1 = top 24 bits + 1 (1 .. 2^24),
// k2 = the next 24 bits.  A normal deviate is Box-Muller's sqrt(-2 ln(m1 / 2^24)) * cos(2 pi k2 / 2^24).
// The logarithm and the cosine are computed here, in double, from additions, multiplications, one
// division and one square root only, each rounded to nearest and never fused, so that the host twin
// (the same operations on numpy arrays) gives the same bits: library logarithms and cosines differ
// between machines in the last place.

#define QS_GOLDEN 0x9E3779B97F4A7C15ull

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }

// ln(m / 2^24), m an integer in 1 .. 2^24
__device__ __forceinline__ double ln_of_fraction(uint32_t m) {
    const double x = (double)m;                                   // exact
    const uint64_t raw = (uint64_t)__double_as_longlong(x);
    int e = (int)(raw >> 52) - 1023;
    double f = __longlong_as_double((long long)((raw & 0x000FFFFFFFFFFFFFull) | 0x3FF0000000000000ull));   // [1, 2)
    if (f > 1.4142135623730951) { f = mul_rn(f, 0.5); e += 1; }
    const double s = __ddiv_rn(add_rn(f, -1.0), add_rn(f, 1.0));     // |s| < 0.172
    const double s2 = mul_rn(s, s);
    double p = 1.0 / 15.0;                                        // 2 atanh(s) = 2 s (1 + s^2/3 + s^4/5 + ...)
    p = add_rn(mul_rn(p, s2), 1.0 / 13.0);
    p = add_rn(mul_rn(p, s2), 1.0 / 11.0);
    p = add_rn(mul_rn(p, s2), 1.0 / 9.0);
    p = add_rn(mul_rn(p, s2), 1.0 / 7.0);
    p = add_rn(mul_rn(p, s2), 1.0 / 5.0);
    p = add_rn(mul_rn(p, s2), 1.0 / 3.0);
    p = add_rn(mul_rn(p, s2), 1.0);
    const double ln_f = mul_rn(mul_rn(2.0, s), p);
    return add_rn(ln_f, mul_rn((double)(e - 24), 0.6931471805599453));
}

// cos(2 pi k / 2^24), k an integer in 0 .. 2^24 - 1: quadrant and octant by integer arithmetic,
// Taylor polynomials on [0, pi/4]
__device__ __forceinline__ double cos_of_turn(uint32_t k) {
    const uint32_t quadrant = k >> 22, j = k & 0x3FFFFFu;
    const bool swap = j > 0x200000u;
    const uint32_t jj = swap ? 0x400000u - j : j;
    const double x = mul_rn((double)jj, 3.141592653589793 / 2.0 / 4194304.0);
    const double x2 = mul_rn(x, x);
    double c = 1.0 / 20922789888000.0;                            // x^16 / 16!
    c = add_rn(mul_rn(c, x2), -1.0 / 87178291200.0);
    c = add_rn(mul_rn(c, x2), 1.0 / 479001600.0);
    c = add_rn(mul_rn(c, x2), -1.0 / 3628800.0);
    c = add_rn(mul_rn(c, x2), 1.0 / 40320.0);
    c = add_rn(mul_rn(c, x2), -1.0 / 720.0);
    c = add_rn(mul_rn(c, x2), 1.0 / 24.0);
    c = add_rn(mul_rn(c, x2), -0.5);
    c = add_rn(mul_rn(c, x2), 1.0);
    double s = -1.0 / 1307674368000.0;                            // x^15 / 15!
    s = add_rn(mul_rn(s, x2), 1.0 / 6227020800.0);
    s = add_rn(mul_rn(s, x2), -1.0 / 39916800.0);
    s = add_rn(mul_rn(s, x2), 1.0 / 362880.0);
    s = add_rn(mul_rn(s, x2), -1.0 / 5040.0);
    s = add_rn(mul_rn(s, x2), 1.0 / 120.0);
    s = add_rn(mul_rn(s, x2), -1.0 / 6.0);
    s = add_rn(mul_rn(s, x2), 1.0);
    s = mul_rn(s, x);
    const double cos_t = swap ? s : c, sin_t = swap ? c : s;     // of the angle inside the quadrant
    switch (quadrant) {
        case 0: return cos_t;
        case 1: return -sin_t;
        case 2: return -cos_t;
        default: return sin_t;
    }
}

enum { QS_FILL_NORMAL = 0, QS_FILL_AROUND_ONE = 1, QS_FILL_INT = 2 };
enum { QS_OUT_F32 = 0, QS_OUT_BF16 = 1, QS_OUT_I32 = 2 };

__global__ void random_fill_kernel(void* __restrict__ out, int out_type, long long n, uint64_t key, int kind,
                                   double a, long long first) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint64_t bits = mix64(key + (uint64_t)(first + i + 1) * QS_GOLDEN);
        if (kind == QS_FILL_INT) {
            reinterpret_cast<int32_t*>(out)[i] = (int32_t)(bits % (uint64_t)a);
            continue;
        }
        double v;
        if (kind == QS_FILL_NORMAL) {
            const uint32_t m1 = (uint32_t)(bits >> 40) + 1u, k2 = (uint32_t)(bits >> 16) & 0xFFFFFFu;
            const double r = __dsqrt_rn(mul_rn(-2.0, ln_of_fraction(m1)));
            v = mul_rn(mul_rn(r, cos_of_turn(k2)), a);
        } else {                                                  // 1 + (2 u - 1) a, u = top 24 bits / 2^24
            const double u = mul_rn((double)(uint32_t)(bits >> 40), 1.0 / 16777216.0);
            v = add_rn(1.0, mul_rn(add_rn(mul_rn(2.0, u), -1.0), a));
        }
        const float f = __double2float_rn(v);
        if (out_type == QS_OUT_F32) reinterpret_cast<float*>(out)[i] = f;
        else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(f);
    }
}

// Fill out[0 .. n) with elements first .. first + n of the stream `key`.
// kind 0: N(0, a); kind 1: 1 + U(-a, a); kind 2: integers in [0, a) (out_type int32).
QS_API int qs_random_fill(void* out, int out_type, long long n, unsigned long long key, int kind, double a,
                          long long first, cudaStream_t stream) {
    if (n == 0) return QS_OK;
    QS_REQUIRE(n > 0 && first >= 0, "random fill: n=%lld first=%lld", n, first);
    QS_REQUIRE(kind >= QS_FILL_NORMAL && kind <= QS_FILL_INT, "random fill: unknown kind %d", kind);
    QS_REQUIRE((kind == QS_FILL_INT) == (out_type == QS_OUT_I32) && out_type >= 0 && out_type <= QS_OUT_I32,
               "random fill: kind %d does not go with element type %d", kind, out_type);
    QS_REQUIRE(kind != QS_FILL_INT || (a >= 1.0 && a <= 2147483648.0), "random fill: integers below %g", a);
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    random_fill_kernel<<<blocks, threads, 0, stream>>>(out, out_type, n, key, kind, a, first);
    return qs_check_launch("random fill");
}

// ----------------------------------------------------------------------------- conversion at upload

enum { QS_IN_F32 = 0, QS_IN_BF16 = 1, QS_IN_F16 = 2 };

__device__ __forceinline__ float half_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
    if (exp == 0) {                                               // zero or subnormal: man * 2^-24
        const float f = (float)man * 5.9604644775390625e-8f;
        return __uint_as_float(__float_as_uint(f) | sign);
    }
    if (exp == 31) return __uint_as_float(sign | 0x7F800000u | (man << 13));
    return __uint_as_float(sign | ((exp + 112u) << 23) | (man << 13));
}

__global__ void convert_kernel(void* __restrict__ out, int out_type, const void* __restrict__ in, int in_type,
                               long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float f;
        if (in_type == QS_IN_F32) f = reinterpret_cast<const float*>(in)[i];
        else if (in_type == QS_IN_BF16) f = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(in)[i] << 16);
        else f = half_bits_to_f32(reinterpret_cast<const uint16_t*>(in)[i]);
        if (out_type == QS_OUT_F32) reinterpret_cast<float*>(out)[i] = f;
        else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(f);
    }
}

// out[i] = in[i] converted: float32 / bfloat16 / float16 in, float32 or bfloat16 (round to nearest even) out.
QS_API int qs_convert(void* out, int out_type, const void* in, int in_type, long long n, cudaStream_t stream) {
    if (n == 0) return QS_OK;
    QS_REQUIRE(n > 0 && (out_type == QS_OUT_F32 || out_type == QS_OUT_BF16) && in_type >= 0 && in_type <= QS_IN_F16,
               "convert: n=%lld types %d -> %d", n, in_type, out_type);
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    convert_kernel<<<blocks, threads, 0, stream>>>(out, out_type, in, in_type, n);
    return qs_check_launch("convert");
}

// ----------------------------------------------------------------------------- finite check

// record[0] = 1 once a value that is not finite has been seen; the first block to see one also writes
// record[1] = tag, record[2] = row, record[3] = column.  Nothing traps: the host reads the record.
template <typename T>
__global__ void check_finite_kernel(const T* __restrict__ x, int rows, int width, size_t ld, int tag,
                                    const int32_t* __restrict__ row_slot, int32_t* __restrict__ record) {
    grid_dep_launch();
    grid_dep_wait();
    const long long n = (long long)rows * width;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int r = (int)(i / width), c = (int)(i - (long long)r * width);
        if (row_slot != nullptr && row_slot[r] < 0) continue;     // padding rows hold nothing
        const float v = to_f32(x[(size_t)r * ld + c]);
        if (!(fabsf(v) <= 3.4028234663852886e38f)) {              // false for NaN and for +-Inf
            if (atomicCAS(record, 0, 1) == 0) { record[1] = tag; record[2] = r; record[3] = c; }
            return;
        }
    }
}

// Scan x [rows, width] (row pitch ld); rows whose `row_slot` entry is negative are skipped (row_slot may
// be null).  `record`: four int32 on the device, zero before the first scan of a step.
QS_API int qs_check_finite(const void* x, int dtype, int rows, int width, long long ld, int tag,
                           const int32_t* row_slot, int32_t* record, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && width > 0 && ld >= width && record != nullptr, "finite check: rows=%d width=%d ld=%lld",
               rows, width, ld);
    const long long n = (long long)rows * width;
    const int threads = 256;
    const long long want = (n + threads * 4 - 1) / (threads * 4);
    const int blocks = (int)(want < 148 * 8 ? (want < 1 ? 1 : want) : 148 * 8);
    cudaError_t e;
    if (dtype == QS_F32)
        e = qs_launch_dependent(check_finite_kernel<float>, dim3(blocks), dim3(threads), 0, stream,
                                (const float*)x, rows, width, (size_t)ld, tag, row_slot, record);
    else if (dtype == QS_BF16)
        e = qs_launch_dependent(check_finite_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream,
                                (const __nv_bfloat16*)x, rows, width, (size_t)ld, tag, row_slot, record);
    else return qs_fail(QS_ERR_INVALID_INPUT, "finite check: unknown dtype %d", dtype);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "finite check: %s", cudaGetErrorString(e));
    return qs_check_launch("finite check");
}

// ----------------------------------------------------------------------------- canary words

__global__ void canary_fill_kernel(uint32_t* __restrict__ p, long long n, uint32_t pattern) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        p[i] = pattern ^ (uint32_t)i;
}

// damaged[0] counts words that no longer hold their pattern; damaged[1] = index of one of them.
__global__ void canary_check_kernel(const uint32_t* __restrict__ p, long long n, uint32_t pattern,
                                    int32_t* __restrict__ damaged) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        if (p[i] != (pattern ^ (uint32_t)i)) {
            if (atomicAdd(damaged, 1) == 0) damaged[1] = (int32_t)(i < 0x7fffffff ? i : 0x7fffffff);
        }
}

// Guard words at the edge of a buffer: word i holds pattern ^ i.  `qs_canary_check` adds the number of
// damaged words to damaged[0] (two int32 on the device).
QS_API int qs_canary_fill(void* p, long long n_words, unsigned int pattern, cudaStream_t stream) {
    if (n_words == 0) return QS_OK;
    QS_REQUIRE(n_words > 0 && ((uintptr_t)p & 3) == 0, "canary fill: n=%lld", n_words);
    const int blocks = (int)((n_words + 255) / 256 < 1184 ? (n_words + 255) / 256 : 1184);
    canary_fill_kernel<<<blocks, 256, 0, stream>>>((uint32_t*)p, n_words, pattern);
    return qs_check_launch("canary fill");
}

QS_API int qs_canary_check(const void* p, long long n_words, unsigned int pattern, int32_t* damaged,
                           cudaStream_t stream) {
    if (n_words == 0) return QS_OK;
    QS_REQUIRE(n_words > 0 && ((uintptr_t)p & 3) == 0 && damaged != nullptr, "canary check: n=%lld", n_words);
    const int blocks = (int)((n_words + 255) / 256 < 1184 ? (n_words + 255) / 256 : 1184);
    canary_check_kernel<<<blocks, 256, 0, stream>>>((const uint32_t*)p, n_words, pattern, damaged);
    return qs_check_launch("canary check");
}

// ----------------------------------------------------------------------------- tokens from the sampler

// dst[j] = src[idx[j]] for j < n where idx[j] >= 0: the step's token buffer takes its tokens from the
// sampler's output on the device; rows with a negative index keep what the host wrote.
__global__ void take_tokens_kernel(int32_t* __restrict__ dst, const int32_t* __restrict__ src,
                                   const int32_t* __restrict__ idx, int n, int n_src) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const int k = idx[j];
    if (k >= 0 && k < n_src) dst[j] = src[k];
}

QS_API int qs_take_tokens(int32_t* dst, const int32_t* src, const int32_t* idx, int n, int n_src, cudaStream_t stream) {
    if (n == 0) return QS_OK;
    QS_REQUIRE(n > 0 && n_src > 0 && dst && src && idx, "take tokens: n=%d of %d", n, n_src);
    take_tokens_kernel<<<(n + 127) / 128, 128, 0, stream>>>(dst, src, idx, n, n_src);
    return qs_check_launch("take tokens");
}

// ----------------------------------------------------------------------------- cache pages that change hands

// Zero page `pages[blockIdx.x]` of every entry: base + entry * entry_bytes + page * page_bytes.
__global__ void zero_pages_kernel(uint8_t* __restrict__ base, size_t entry_bytes, size_t page_bytes,
                                  const int32_t* __restrict__ pages, int n_total_pages) {
    const int page = pages[blockIdx.x];
    if (page < 0 || page >= n_total_pages) return;
    uint4* p = reinterpret_cast<uint4*>(base + (size_t)blockIdx.y * entry_bytes + (size_t)page * page_bytes);
    const size_t n = page_bytes / 16;
    for (size_t i = (size_t)blockIdx.z * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.z * blockDim.x)
        p[i] = make_uint4(0u, 0u, 0u, 0u);
}

// A page that held another sequence's values is cleared before it is handed on, unless the step that
// takes it writes all of its rows: the tensor-core prefill attention multiplies the rows past a
// sequence's end by weights of exactly zero, and 0 * Inf is NaN.
QS_API int qs_zero_pages(void* base, long long entry_bytes, long long page_bytes, int n_entries,
                         const int32_t* pages, int n_pages, int n_total_pages, cudaStream_t stream) {
    if (n_pages == 0 || n_entries == 0) return QS_OK;
    QS_REQUIRE(n_pages > 0 && n_entries > 0 && n_entries <= 65535 && page_bytes > 0 && page_bytes % 16 == 0 &&
               entry_bytes % 16 == 0 && ((uintptr_t)base % 16) == 0,
               "zero pages: %d pages of %lld bytes in %d entries", n_pages, page_bytes, n_entries);
    const int z = (int)((page_bytes / 16 + 255) / 256 < 8 ? (page_bytes / 16 + 255) / 256 : 8);
    zero_pages_kernel<<<dim3(n_pages, n_entries, z), 256, 0, stream>>>((uint8_t*)base, (size_t)entry_bytes,
                                                                     (size_t)page_bytes, pages, n_total_pages);
    return qs_check_launch("zero pages");
}

// ----------------------------------------------------------------------------- the bounded wait, by itself

// A wait on a barrier that nothing will ever complete, with the polling loop that every kernel of the
// library uses (sm100::mbar_try_wait under a limit): after `polls` polls it gives up, records code 199
// in `status` and returns.  The context stays usable.  For tests of the path a kernel takes when one of its
// waits runs out; no kernel of the model calls this.
__global__ void bounded_wait_selftest_kernel(int32_t* __restrict__ status, uint32_t polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        sm100::mbar_init(&bar, 1);
        sm100::mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        bool done = false;
        for (uint32_t i = 0; i < polls && !done; ++i) done = sm100::mbar_try_wait(&bar, 0);
        if (!done) atomicExch(status, 199);
    }
    __syncthreads();
}

QS_API int qs_selftest_bounded_wait(int32_t* status, int polls, cudaStream_t stream) {
    QS_REQUIRE(status != nullptr && polls > 0 && polls <= (1 << 16), "bounded wait self-test: polls=%d", polls);
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, (uint32_t)polls);
    return qs_check_launch("bounded wait self-test");
}
