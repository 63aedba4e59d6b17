// Decode attention for bfloat16: one query token per sequence against its paged cache, with the
// keys cut into splits of 256 (four pages of 64) that run as separate CTAs, and a merge kernel.
//
// The kernel is bound by the bytes of K and V it streams (one multiply-add per byte and head),
// so it runs on the CUDA cores with 16-byte loads; scores, maxima, exponentials, sums and the
// output accumulator are 32-bit.  A split's boundaries depend only on absolute key positions
// and the merge adds the splits in ascending order, so a sequence's result depends on its own
// length only, not on the batch or on where its pages lie.
//
//   s[u] = q.k[u] / sqrt(dh) over keys first <= u <= pos     (QStream src/engine.c:888-906)
//   softmax with max subtraction                             (src/kernels_scalar.c:188-213)
//   o = sum_u a[u] v[u]                                      (src/engine.c:913-922)
#include "common.cuh"

namespace {

constexpr int PAGE = 64;
constexpr int WARPS = 4;
constexpr int SPLIT = PAGE * WARPS;          // keys per CTA

__device__ __forceinline__ void bf16x8_to_f32(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Lanes are grouped GS to a key (GS = the power of two >= dh / 16, at most 32); lane `c` of a group
// owns the 16-byte chunks c, c + GS, ... (NCH of them) of the head.  KPL = 32 / GS keys are
// handled per warp instruction.
template <int NCH, int UNROLL>
__global__ void __launch_bounds__(WARPS * 32)
decode_split_kernel(float* __restrict__ partial, const __nv_bfloat16* __restrict__ q, size_t ldq,
                    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                    const int32_t* __restrict__ page_table, int max_pages,
                    const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                    int n_heads, int n_kv_heads, int dh, int gs_log2, float scale, int window, int max_splits,
                    int32_t* __restrict__ status) {
    __shared__ float s_scores[WARPS][PAGE];
    __shared__ float s_m[WARPS], s_l[WARPS];
    extern __shared__ float s_acc[];                 // [WARPS][dh]

    const int split = blockIdx.x, head = blockIdx.y, t = blockIdx.z;
    const int slot = tok_slot[t];
    if (slot < 0) return;
    const int pos = tok_pos[t];
    if (pos < 0 || pos >= max_splits * SPLIT) {       // outside what the grid and the scratch cover: report, touch nothing
        if (threadIdx.x == 0 && split == 0) atomicExch(status, 1);
        return;
    }
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    if (split * SPLIT > pos || (split + 1) * SPLIT <= first) return;       // no visible key in this split

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int GS = 1 << gs_log2, KPL = 32 >> gs_log2;
    const int chunk = lane & (GS - 1), sub = lane >> gs_log2;
    const int n_chunks = dh >> 3;
    const int kvh = head / (n_heads / n_kv_heads);

    // this lane's part of the query, in 32-bit
    float qf[NCH][8];
    const __nv_bfloat16* qrow = q + (size_t)t * ldq + (size_t)head * dh;
#pragma unroll
    for (int i = 0; i < NCH; ++i) {
        const int c = chunk + i * GS;
        if (c < n_chunks) bf16x8_to_f32(*reinterpret_cast<const uint4*>(qrow + c * 8), qf[i]);
        else {
#pragma unroll
            for (int j = 0; j < 8; ++j) qf[i][j] = 0.f;
        }
    }

    float acc[NCH][8];
#pragma unroll
    for (int i = 0; i < NCH; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int key0 = split * SPLIT + warp * PAGE;     // this warp's page of keys
    if (key0 <= pos && key0 + PAGE > first) {
        const int page = page_table[(size_t)slot * max_pages + (key0 >> 6)];
        if (page < 0) {
            if (lane == 0) atomicExch(status, 3);
        } else {
            const size_t base = ((size_t)page * n_kv_heads + kvh) * PAGE * dh;
            const __nv_bfloat16* kp = k_cache + base;
            const __nv_bfloat16* vp = v_cache + base;
            const int n_keys = min(PAGE, pos - key0 + 1);
            // scores of the page's keys, UNROLL warp loads in flight at a time
            for (int it0 = 0; it0 * KPL < n_keys; it0 += UNROLL) {
                uint4 raw[UNROLL][NCH];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int kk = (it0 + u) * KPL + sub;
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const int c = chunk + i * GS;
                        raw[u][i] = (kk < n_keys && c < n_chunks)
                            ? __ldg(reinterpret_cast<const uint4*>(kp + (size_t)kk * dh + c * 8)) : make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int kk = (it0 + u) * KPL + sub;
                    float dot = 0.f;
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        float kf[8];
                        bf16x8_to_f32(raw[u][i], kf);
#pragma unroll
                        for (int j = 0; j < 8; ++j) dot = fmaf(qf[i][j], kf[j], dot);
                    }
                    for (int o = GS >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                    if (chunk == 0 && kk < PAGE) s_scores[warp][kk] = (kk < n_keys && key0 + kk >= first) ? dot * scale : -INFINITY;
                }
            }
            __syncwarp();
            // softmax weights of the page: lane handles keys lane and lane + 32
            float s0 = lane < n_keys ? s_scores[warp][lane] : -INFINITY;
            float s1 = lane + 32 < n_keys ? s_scores[warp][lane + 32] : -INFINITY;
            m = warp_max(fmaxf(s0, s1));
            const float p0 = m == -INFINITY ? 0.f : expf(s0 - m);
            const float p1 = m == -INFINITY ? 0.f : expf(s1 - m);
            l = warp_sum(p0 + p1);
            __syncwarp();
            s_scores[warp][lane] = p0;
            s_scores[warp][lane + 32] = p1;
            __syncwarp();
            // weighted values
            for (int it0 = 0; it0 * KPL < n_keys; it0 += UNROLL) {
                uint4 raw[UNROLL][NCH];
                float pw[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int kk = (it0 + u) * KPL + sub;
                    pw[u] = kk < n_keys ? s_scores[warp][kk] : 0.f;
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        const int c = chunk + i * GS;
                        raw[u][i] = (kk < n_keys && c < n_chunks)
                            ? __ldg(reinterpret_cast<const uint4*>(vp + (size_t)kk * dh + c * 8)) : make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        float vf[8];
                        bf16x8_to_f32(raw[u][i], vf);
#pragma unroll
                        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(pw[u], vf[j], acc[i][j]);
                    }
                }
            }
            // add the KPL key groups of the warp (they hold different keys of the same dims)
            for (int o = GS; o < 32; o <<= 1) {
#pragma unroll
                for (int i = 0; i < NCH; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] += __shfl_xor_sync(0xffffffffu, acc[i][j], o);
            }
        }
    }

    // merge the four warps in warp order
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
    if (sub == 0) {
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int c = chunk + i * GS;
            if (c < n_chunks) {
#pragma unroll
                for (int j = 0; j < 8; ++j) s_acc[(size_t)warp * dh + c * 8 + j] = acc[i][j];
            }
        }
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, s_m[w]);
    float* out = partial + (((size_t)t * n_heads + head) * max_splits + split) * (dh + 2);
    for (int d = threadIdx.x; d < dh; d += blockDim.x) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w)
            if (s_m[w] != -INFINITY) o += s_acc[(size_t)w * dh + d] * expf(s_m[w] - M);
        out[d] = o;
    }
    if (threadIdx.x == 0) {
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w)
            if (s_m[w] != -INFINITY) L += s_l[w] * expf(s_m[w] - M);
        out[dh] = M;
        out[dh + 1] = L;
    }
}

// One block per (token, head): add the splits' partial results in ascending split order.
__global__ void decode_merge_kernel(__nv_bfloat16* __restrict__ out, size_t ldo, const float* __restrict__ partial,
                                    const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                    int n_heads, int dh, int window, int max_splits) {
    grid_dep_launch();
    const int head = blockIdx.x, t = blockIdx.y;
    __nv_bfloat16* o = out + (size_t)t * ldo + (size_t)head * dh;
    if (tok_slot[t] < 0) {
        for (int d = threadIdx.x; d < dh; d += blockDim.x) o[d] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos = tok_pos[t];
    if (pos < 0 || pos >= max_splits * SPLIT) {       // the split kernel has reported it; a defined row, no access
        for (int d = threadIdx.x; d < dh; d += blockDim.x) o[d] = __float2bfloat16_rn(0.f);
        return;
    }
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int s_lo = first / SPLIT, s_hi = pos / SPLIT, n = s_hi - s_lo + 1;
    const float* base = partial + ((size_t)t * n_heads + head) * max_splits * (dh + 2);
    // The splits' maxima, sums and weights exp(m_s - M) are fetched and computed once per block, a split per
    // thread; every sum below then runs over shared memory or over loads that are all in flight together, in
    // ascending split order as before.  (With one thread walking 64 splits' global memory in a row - a context
    // of 16,384 - the merge took 20 us, as long as a third of the split kernel.)
    extern __shared__ float s_all[];                  // [3][max_splits]: weights, maxima, sums
    float* s_w = s_all;
    float* s_m = s_all + max_splits;
    float* s_l = s_all + 2 * max_splits;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        s_m[i] = base[(size_t)(s_lo + i) * (dh + 2) + dh];
        s_l[i] = base[(size_t)(s_lo + i) * (dh + 2) + dh + 1];
    }
    __syncthreads();
    float M = -INFINITY;
    for (int i = 0; i < n; ++i) M = fmaxf(M, s_m[i]);
    for (int i = threadIdx.x; i < n; i += blockDim.x) s_w[i] = s_m[i] != -INFINITY ? expf(s_m[i] - M) : 0.f;
    __syncthreads();
    float L = 0.f;
    for (int i = 0; i < n; ++i)
        if (s_w[i] != 0.f) L += s_l[i] * s_w[i];
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    constexpr int AHEAD = 8;                          // loads in flight per thread
    for (int d = threadIdx.x; d < dh; d += blockDim.x) {
        float acc = 0.f;
        for (int i0 = 0; i0 < n; i0 += AHEAD) {
            float v[AHEAD];
#pragma unroll
            for (int u = 0; u < AHEAD; ++u)           // a split without visible keys wrote nothing: its cell is read and not used
                v[u] = i0 + u < n ? base[(size_t)(s_lo + i0 + u) * (dh + 2) + d] : 0.f;
#pragma unroll
            for (int u = 0; u < AHEAD; ++u)
                if (i0 + u < n && s_w[i0 + u] != 0.f) acc += v[u] * s_w[i0 + u];
        }
        o[d] = __float2bfloat16_rn(acc * inv);
    }
}

}  // namespace

// How many floats of scratch `qs_attention_decode` needs.
QS_API long long qs_attention_decode_scratch(int T_tokens, int n_heads, int dh, int max_context) {
    const long long max_splits = (max_context + SPLIT - 1) / SPLIT;
    return (long long)T_tokens * n_heads * max_splits * (dh + 2);
}

// out [T, n_heads * dh] bfloat16.  One query token per row; `max_context` bounds every row's
// position + 1 and fixes the grid, so the same launch serves every length (CUDA graphs).
// `scratch`: float32, at least qs_attention_decode_scratch(...) elements; contents need no
// initialisation.  A row whose position is negative or not below max_context rounded up to 256 sets
// status 1 and gets zeros; `tok_slot` entries must be negative (padding) or rows of `page_table`.
QS_API int qs_attention_decode(void* out, long long ldo, const void* q, long long ldq, const void* k_cache,
                               const void* v_cache, const int32_t* page_table, int max_pages, int page_tokens,
                               const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens, int n_heads,
                               int n_kv_heads, int dh, float scale, int window, int max_context,
                               float* scratch, int32_t* status, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && dh > 0 && max_context > 0, "attention_decode: bad sizes");
    QS_REQUIRE(page_tokens == PAGE, "attention_decode: pages of %d tokens, the kernel is built for %d", page_tokens, PAGE);
    QS_REQUIRE(n_heads % n_kv_heads == 0, "attention_decode: %d query heads are no multiple of %d key heads", n_heads, n_kv_heads);
    QS_REQUIRE(dh % 8 == 0 && dh <= 512, "attention_decode: head size %d must be a multiple of 8, at most 512", dh);
    QS_REQUIRE(ldq % 8 == 0 && ((uintptr_t)q % 16) == 0, "attention_decode: queries must be 16-byte aligned rows");
    QS_REQUIRE(T_tokens <= 65535 && n_heads <= 65535, "attention_decode: sizes exceed the grid");
    const int max_splits = (max_context + SPLIT - 1) / SPLIT;
    QS_REQUIRE(max_splits <= 4096, "attention_decode: a context of %d exceeds what the merge kernel holds (%d)", max_context, 4096 * SPLIT);
    const int n_chunks = dh / 8;
    // Two 16-byte chunks per lane: half as many lanes share a key, so a score costs one shuffle step
    // less and a warp instruction covers twice the keys.  The grouping depends on the head size only
    // (it fixes the order of the sums); how many loads a lane keeps in flight does not change a bit
    // of the result and follows the size of the grid.
    int gs_log2 = 0;
    while ((2 << gs_log2) < n_chunks && gs_log2 < 5) ++gs_log2;
    int nch = (n_chunks + (1 << gs_log2) - 1) >> gs_log2;
    // Head sizes of 3 or 5 times a power of two chunks would leave a quarter to three eighths of the lanes'
    // chunk slots empty with two chunks per lane: three or five chunks per lane fill them all.  Measured at
    // 192 and 320: 25 us instead of 33 us, 29 us instead of 54 us (16 sequences of 1,000 keys); at 48 and 80,
    // where a key would be left to two lanes, it is slower (32 us for 27 us, 42 us for 38 us) and not used.
    for (int per = 3; per <= 5; per += 2) {
        const int gs = n_chunks / per;
        if (n_chunks % per == 0 && gs >= 8 && gs <= 32 && (gs & (gs - 1)) == 0) {
            nch = per;
            gs_log2 = 0;
            while ((1 << gs_log2) < gs) ++gs_log2;
        }
    }
    dim3 grid(max_splits, n_heads, T_tokens);
    const size_t smem = (size_t)WARPS * dh * sizeof(float);
    static int sm_counts[64] = {0};                  // per device; a race only repeats the query
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    int sm_count = sm_counts[dev];
    if (sm_count == 0) {
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sm_count = 1;
        sm_counts[dev] = sm_count;
    }
    const bool few_ctas = (long long)max_splits * n_heads * T_tokens <= 2LL * sm_count;
#define GO(NCH, UNROLL) decode_split_kernel<NCH, UNROLL><<<grid, WARPS * 32, smem, stream>>>( \
        scratch, (const __nv_bfloat16*)q, (size_t)ldq, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
        page_table, max_pages, tok_slot, tok_pos, n_heads, n_kv_heads, dh, gs_log2, scale, window, max_splits, status)
    if (nch == 1) GO(1, 8);
    else if (nch == 3) GO(3, 4);
    else if (nch == 5) GO(5, 2);
    else if (few_ctas) GO(2, 8);
    else GO(2, 4);
#undef GO
    int rc = qs_check_launch("attention_decode");
    if (rc != QS_OK) return rc;
    decode_merge_kernel<<<dim3(n_heads, T_tokens), dh >= 128 ? 128 : 64, (size_t)3 * max_splits * sizeof(float), stream>>>(
        (__nv_bfloat16*)out, (size_t)ldo, scratch, tok_slot, tok_pos, n_heads, dh, window, max_splits);
    return qs_check_launch("attention_decode merge");
}

// ----------------------------------------------------------------------------- no allocation
//
// The same decode attention for callers that cannot allocate device memory (see
// qstream_no_alloc.h): the partial results of the key splits go to a fixed array in the
// library instead of a buffer from the caller.
#include "qstream_no_alloc.h"

// In host code this name is only a handle for cudaGetSymbolAddress, not a device address.
static __device__ __align__(256) float g_decode_static_scratch[QS_DECODE_STATIC_SCRATCH_FLOATS];

#include <mutex>

namespace {
constexpr int kMaxDevices = 64;
float* g_decode_static_ptr[kMaxDevices] = {nullptr};
std::mutex g_decode_static_mutex;                  // set-up from two host threads at once
}  // namespace

QS_API int qs_attention_decode_static(void* out, long long ldo, const void* q, long long ldq,
                                      const void* k_cache, const void* v_cache,
                                      const int32_t* page_table, int max_pages, int page_tokens,
                                      const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens,
                                      int n_heads, int n_kv_heads, int dh, float scale, int window,
                                      int max_context, int32_t* status, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && n_heads > 0 && dh > 0 && max_context > 0, "attention_decode_static: bad sizes");
    const long long need = qs_attention_decode_scratch(T_tokens, n_heads, dh, max_context);
    QS_REQUIRE(need <= (long long)QS_DECODE_STATIC_SCRATCH_FLOATS,
               "attention_decode_static: the call needs %lld floats of scratch, the built-in array holds %d "
               "(tokens * heads * ceil(context / 256) * (head size + 2))", need, QS_DECODE_STATIC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "attention_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    QS_REQUIRE(device >= 0 && device < kMaxDevices, "attention_decode_static: device %d out of range", device);
    float* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_decode_static_mutex);
        if (!g_decode_static_ptr[device]) {         // first call on this device: find the array's device address
            float* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_decode_static_scratch);
            if (e != cudaSuccess || !p)
                return qs_fail(QS_ERR_INTERNAL, "attention_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_decode_static_ptr[device] = p;
        }
        scratch = g_decode_static_ptr[device];
    }
    return qs_attention_decode(out, ldo, q, ldq, k_cache, v_cache, page_table, max_pages, page_tokens, tok_slot,
                               tok_pos, T_tokens, n_heads, n_kv_heads, dh, scale, window, max_context,
                               scratch, status, stream);
}
