// Rotary position encoding fused with the write of keys and values into the paged
// cache, and causal attention of each token over its sequence's cache.
//
// Cache entry layout: K and V each [n_pages][n_kv_heads][page_tokens][head_dim].
// A sequence (slot) owns a row of `page_table` ([n_slots][max_pages], int32); position
// p of the sequence lies in page page_table[slot][p / page_tokens] at row
// p % page_tokens.  A token with slot < 0 is padding: nothing is read or written for it.
#include "common.cuh"

namespace {

// ----------------------------------------------------------------------------- rotary + store

// For every token and head: rotate pairs (2j, 2j+1), 2j < R, of q (in place) and k by the
// angle pos * base^(-2j/R), taken from a 32-bit table [max_pos][R/2][2] = (cos, sin):
//   a' = a cos - b sin ; b' = a sin + b cos            (QStream src/engine.c:216-218)
// then keep the rotated k and the v in the cache (rope before store: src/engine.c:871-880).
// The rotation is evaluated in 32-bit and rounded once.  q == nullptr: keys/values only.
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                  size_t ldq, size_t ldk, size_t ldv,
                                  int n_heads, int n_kv_heads, int dh, int R,
                                  const float* __restrict__ cos_sin, int max_pos,
                                  const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                  const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  int32_t* __restrict__ status) {
    // blockIdx.x = token; the gridDim.y blocks of a token share its (head, pair of dims) items of q, then k and v
    grid_dep_launch();
    grid_dep_wait();
    const int t = blockIdx.x;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;
    const int pos = tok_pos[t];
    const int page_tokens = 1 << page_shift;
    const bool rotate = cos_sin != nullptr && R > 0;
    if (rotate && (pos < 0 || pos >= max_pos)) { if (threadIdx.x == 0) atomicExch(status, 1); return; }
    const float* cs = rotate ? cos_sin + (size_t)pos * R : nullptr;      // R/2 pairs of (cos, sin)
    const int half = dh >> 1;

    if (q && rotate) {
        const int rp = R >> 1;                                           // rotated pairs per head
        for (int e = tid; e < n_heads * rp; e += stride) {
            const int head = e / rp, j = e - head * rp;
            T* row = q + (size_t)t * ldq + (size_t)head * dh;
            const float c = cs[2 * j], sn = cs[2 * j + 1];
            const float a = to_f32(row[2 * j]), b = to_f32(row[2 * j + 1]);
            row[2 * j] = from_f32<T>(a * c - b * sn);
            row[2 * j + 1] = from_f32<T>(a * sn + b * c);
        }
    }
    if (n_kv_heads == 0) return;
    const int page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    if (page < 0) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    const size_t in_page = (size_t)(pos & (page_tokens - 1)) * dh;
    for (int e = tid; e < n_kv_heads * half; e += stride) {
        const int kvh = e / half, j = e - kvh * half;
        const size_t dst_off = ((size_t)page * n_kv_heads + kvh) * page_tokens * dh + in_page;
        const T* krow = k + (size_t)t * ldk + (size_t)kvh * dh;
        T* kdst = k_cache + dst_off;
        if (rotate && 2 * j < R) {
            const float c = cs[2 * j], sn = cs[2 * j + 1];
            const float a = to_f32(krow[2 * j]), b = to_f32(krow[2 * j + 1]);
            kdst[2 * j] = from_f32<T>(a * c - b * sn);
            kdst[2 * j + 1] = from_f32<T>(a * sn + b * c);
        } else {
            kdst[2 * j] = krow[2 * j];
            kdst[2 * j + 1] = krow[2 * j + 1];
        }
        const T* vrow = v + (size_t)t * ldv + (size_t)kvh * dh;
        T* vdst = v_cache + dst_off;
        vdst[2 * j] = vrow[2 * j];
        vdst[2 * j + 1] = vrow[2 * j + 1];
    }
}

// The same for bfloat16 with 16-byte accesses: an item is eight consecutive dims (four rotary pairs).
// Needs head size and rotary width multiples of 8 and 16-byte aligned rows.
__device__ __forceinline__ uint4 rotate8(const uint4 raw, const float* __restrict__ cs8) {
    // cs8: (cos, sin) of the four pairs, eight floats
    const float4 a = reinterpret_cast<const float4*>(cs8)[0], b = reinterpret_cast<const float4*>(cs8)[1];
    const float c[4] = {a.x, a.z, b.x, b.z}, sn[4] = {a.y, a.w, b.y, b.w};
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float x = __uint_as_float(w[i] << 16), y = __uint_as_float(w[i] & 0xffff0000u);
        const __nv_bfloat162 r = __floats2bfloat162_rn(x * c[i] - y * sn[i], x * sn[i] + y * c[i]);
        o[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void rope_store_vec_kernel(__nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                      const __nv_bfloat16* __restrict__ v, size_t ldq, size_t ldk, size_t ldv,
                                      int n_heads, int n_kv_heads, int dh, int R,
                                      const float* __restrict__ cos_sin, int max_pos,
                                      const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                                      const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                                      __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                      int32_t* __restrict__ status, int settled) {
    grid_dep_launch();
    // `settled`: the step's slots, positions and pages and the table of angles were complete before the
    // previous kernel of the stream began.  Then they are fetched (the table's row only as far as L2) while
    // that kernel still runs.
    if (!settled) grid_dep_wait();
    const int t = blockIdx.x;
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, stride = gridDim.y * blockDim.x;
    const int slot = tok_slot[t];
    const int pos = tok_pos[t];
    const bool rotate = cos_sin != nullptr && R > 0;
    const bool pos_ok = !rotate || (pos >= 0 && pos < max_pos);
    const float* cs = rotate && pos_ok ? cos_sin + (size_t)pos * R : nullptr;
    int page = -1;
    if (slot >= 0 && n_kv_heads > 0 && pos >= 0 && (pos >> page_shift) < max_pages)
        page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    if (cs && slot >= 0 && threadIdx.x * 32 < R)
        asm volatile("prefetch.global.L2 [%0];" :: "l"(cs + threadIdx.x * 32));
    if (settled) grid_dep_wait();
    if (slot < 0) return;
    const int page_tokens = 1 << page_shift;
    if (!pos_ok) { if (threadIdx.x == 0) atomicExch(status, 1); return; }
    const int rc = R >> 3, hc = dh >> 3;                                 // 16-byte chunks of the rotary part / of a head
    if (q && rotate) {
        for (int e = tid; e < n_heads * rc; e += stride) {
            const int head = e / rc, c = e - head * rc;
            uint4* p = reinterpret_cast<uint4*>(q + (size_t)t * ldq + (size_t)head * dh + c * 8);
            *p = rotate8(*p, cs + c * 8);
        }
    }
    if (n_kv_heads == 0) return;
    if (page < 0) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    const size_t in_page = (size_t)(pos & (page_tokens - 1)) * dh;
    for (int e = tid; e < n_kv_heads * hc; e += stride) {
        const int kvh = e / hc, c = e - kvh * hc;
        const size_t dst = ((size_t)page * n_kv_heads + kvh) * page_tokens * dh + in_page + c * 8;
        uint4 kk = *reinterpret_cast<const uint4*>(k + (size_t)t * ldk + (size_t)kvh * dh + c * 8);
        if (rotate && c < rc) kk = rotate8(kk, cs + c * 8);
        *reinterpret_cast<uint4*>(k_cache + dst) = kk;
        *reinterpret_cast<uint4*>(v_cache + dst) = *reinterpret_cast<const uint4*>(v + (size_t)t * ldv + (size_t)kvh * dh + c * 8);
    }
}

// ----------------------------------------------------------------------------- attention

// One warp per (token, query head).  Keys are visited 32 at a time in position order:
// lane l scores key base+l (s = q.k / sqrt(dh), QStream src/engine.c:888-906), the
// running maximum and sum are updated (softmax with max subtraction,
// src/kernels_scalar.c:188-213, in its streaming form) and the 32 weighted values are
// added in key order (src/engine.c:913-922).  Scores, maximum, exponentials, sum and
// the output accumulator are 32-bit.  The order of the sums depends only on the
// token's own position, never on the batch or on where the pages lie.
// Lane l owns output dims l, l+32, ...: NACC = ceil(dh / 32) accumulators.
template <typename T, int NACC>
__global__ void __launch_bounds__(128)
attention_kernel(T* __restrict__ out, const T* __restrict__ q, size_t ldo, size_t ldq,
                 const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 const int32_t* __restrict__ page_table, int max_pages, int page_shift,
                 const int32_t* __restrict__ tok_slot, const int32_t* __restrict__ tok_pos,
                 int T_tokens, int n_heads, int n_kv_heads, int dh, float scale, int window,
                 int32_t* __restrict__ status) {
    extern __shared__ float q_smem[];               // [warps][dh]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)T_tokens * n_heads) return;
    const int t = (int)(item / n_heads), head = (int)(item % n_heads);
    T* o = out + (size_t)t * ldo + (size_t)head * dh;
    const int slot = tok_slot[t];
    if (slot < 0) {                                 // padding: defined output, no cache access
        for (int d = lane; d < dh; d += 32) o[d] = from_f32<T>(0.f);
        return;
    }
    const int pos = tok_pos[t];
    const int kvh = head / (n_heads / n_kv_heads);  // QStream src/engine.c:884,889
    const int page_tokens = 1 << page_shift;
    const int32_t* pages = page_table + (size_t)slot * max_pages;

    float* qs = q_smem + (size_t)warp * dh;
    const T* qrow = q + (size_t)t * ldq + (size_t)head * dh;
    for (int d = lane; d < dh; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();

    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;

    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        const bool live = key <= pos;
        float s = -INFINITY;
        const T* vrow = nullptr;
        if (live) {
            const int page = pages[key >> page_shift];
            if (page < 0) { atomicExch(status, 3); }
            else {
                const size_t off = (((size_t)page * n_kv_heads + kvh) * page_tokens + (key & (page_tokens - 1))) * dh;
                const T* krow = k_cache + off;
                vrow = v_cache + off;
                float dot = 0.f;
                for (int d = 0; d < dh; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = live && vrow ? expf(s - m_new) : 0.f;
        const float alpha = m == -INFINITY ? 0.f : expf(m - m_new);
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const int n_keys = min(32, pos - base + 1);
        for (int j = 0; j < n_keys; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const T* vj = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, (unsigned long long)vrow, j));
            if (!vj) continue;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dh) acc[i] = fmaf(pj, to_f32(vj[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dh) o[d] = from_f32<T>(acc[i] * inv);
    }
}

template <typename T>
int launch_attention(void* out, const void* q, long long ldo, long long ldq, const void* k_cache,
                     const void* v_cache, const int32_t* page_table, int max_pages, int page_shift,
                     const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens, int n_heads,
                     int n_kv_heads, int dh, float scale, int window, int32_t* status,
                     cudaStream_t stream) {
    const int warps = 4;
    const long long items = (long long)T_tokens * n_heads;
    const int blocks = (int)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * dh * sizeof(float);
#define GO(NACC) attention_kernel<T, NACC><<<blocks, warps * 32, smem, stream>>>( \
        (T*)out, (const T*)q, (size_t)ldo, (size_t)ldq, (const T*)k_cache, (const T*)v_cache, \
        page_table, max_pages, page_shift, tok_slot, tok_pos, T_tokens, n_heads, n_kv_heads, dh, \
        scale, window, status)
    const int nacc = (dh + 31) / 32;
    if (nacc <= 1) GO(1);
    else if (nacc <= 2) GO(2);
    else if (nacc <= 4) GO(4);
    else if (nacc <= 8) GO(8);
    else GO(16);
#undef GO
    return qs_check_launch("attention");
}

}  // namespace

// `settled` != 0: slots, positions, page table and the table of angles were complete before the previous kernel
// of the stream began (they came by a copy, or from an earlier step), so the kernel may read them early.
QS_API int qs_rope_store(void* q, const void* k, const void* v, int dtype,
                         long long ldq, long long ldk, long long ldv,
                         int n_heads, int n_kv_heads, int dh, int R,
                         const float* cos_sin, int max_pos,
                         const int32_t* tok_slot, const int32_t* tok_pos,
                         const int32_t* page_table, int max_pages, int page_tokens,
                         void* k_cache, void* v_cache, int T_tokens, int32_t* status,
                         int settled, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && n_heads >= 0 && n_kv_heads >= 0 && n_heads + n_kv_heads > 0 && dh > 0, "rope_store: bad sizes");
    QS_REQUIRE(n_kv_heads == 0 || (k && v && k_cache && v_cache), "rope_store: keys and values without a cache to keep them");
    QS_REQUIRE(dh % 2 == 0, "rope_store: head size %d must be even", dh);
    QS_REQUIRE(R >= 0 && R % 2 == 0 && R <= dh, "rope_store: rotary width %d must be even and within the head size %d", R, dh);
    QS_REQUIRE(page_tokens > 0 && (page_tokens & (page_tokens - 1)) == 0, "rope_store: page size %d is no power of two", page_tokens);
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    const int work = (n_heads + 2 * n_kv_heads) * dh / 2;
    const int threads = work >= 2048 ? 256 : (work >= 512 ? 128 : 64);
    int per_token = 1;                       // few tokens (decode): several blocks per token
    if (T_tokens < 256) { per_token = (n_kv_heads * dh / 2 + threads - 1) / threads; if (per_token > 16) per_token = 16; if (per_token < 1) per_token = 1; }
    dim3 grid(T_tokens, per_token);
    const bool aligned = dh % 8 == 0 && R % 8 == 0 && ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 &&
                         ((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0 &&
                         ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)cos_sin % 16) == 0;
    if (dtype == QS_BF16 && aligned) {
        const int work8 = (n_heads * (R / 8) + n_kv_heads * (dh / 8));
        const int threads8 = work8 >= 512 ? 128 : 64;
        int per = 1;
        if (T_tokens < 256) { per = (n_kv_heads * (dh / 8) + threads8 - 1) / threads8; if (per > 16) per = 16; if (per < 1) per = 1; }
        cudaError_t e = qs_launch_dependent(rope_store_vec_kernel, dim3(T_tokens, per), dim3(threads8), 0, stream,
            (__nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (size_t)ldq, (size_t)ldk, (size_t)ldv,
            n_heads, n_kv_heads, dh, R, cos_sin, max_pos, tok_slot, tok_pos, page_table, max_pages, shift,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, status, settled);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "rope_store: %s", cudaGetErrorString(e));
        return qs_check_launch("rope_store");
    }
    if (dtype == QS_F32)
        qs_launch_dependent(rope_store_kernel<float>, grid, dim3(threads), 0, stream, (float*)q, (const float*)k, (const float*)v,
            (size_t)ldq, (size_t)ldk, (size_t)ldv, n_heads, n_kv_heads, dh, R, cos_sin, max_pos, tok_slot, tok_pos,
            page_table, max_pages, shift, (float*)k_cache, (float*)v_cache, status);
    else if (dtype == QS_BF16)
        qs_launch_dependent(rope_store_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)q, (const __nv_bfloat16*)k,
            (const __nv_bfloat16*)v, (size_t)ldq, (size_t)ldk, (size_t)ldv, n_heads, n_kv_heads, dh, R, cos_sin, max_pos,
            tok_slot, tok_pos, page_table, max_pages, shift, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, status);
    else return qs_fail(QS_ERR_INVALID_INPUT, "rope_store: unknown dtype %d", dtype);
    return qs_check_launch("rope_store");
}

QS_API int qs_attention(void* out, const void* q, int dtype, long long ldo, long long ldq,
                        const void* k_cache, const void* v_cache,
                        const int32_t* page_table, int max_pages, int page_tokens,
                        const int32_t* tok_slot, const int32_t* tok_pos, int T_tokens,
                        int n_heads, int n_kv_heads, int dh, float scale, int window,
                        int32_t* status, cudaStream_t stream) {
    if (T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && dh > 0, "attention: bad sizes");
    QS_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d query heads are no multiple of %d key heads", n_heads, n_kv_heads);
    QS_REQUIRE(dh <= 512, "attention: head size %d above 512", dh);
    QS_REQUIRE(page_tokens > 0 && (page_tokens & (page_tokens - 1)) == 0, "attention: page size %d is no power of two", page_tokens);
    QS_REQUIRE(window >= 0, "attention: negative window");
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    if (dtype == QS_F32)
        return launch_attention<float>(out, q, ldo, ldq, k_cache, v_cache, page_table, max_pages, shift, tok_slot,
                                       tok_pos, T_tokens, n_heads, n_kv_heads, dh, scale, window, status, stream);
    if (dtype == QS_BF16)
        return launch_attention<__nv_bfloat16>(out, q, ldo, ldq, k_cache, v_cache, page_table, max_pages, shift,
                                               tok_slot, tok_pos, T_tokens, n_heads, n_kv_heads, dh, scale, window,
                                               status, stream);
    return qs_fail(QS_ERR_INVALID_INPUT, "attention: unknown dtype %d", dtype);
}
