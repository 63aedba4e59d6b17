// Sampling on the device: argmax, repeat penalty, temperature, top-k, top-p and the
// inverse-CDF draw, with the meanings of QStream's src/sampling.c.
//
// One block works on one row of 32-bit logits [V].  Nothing is written to the logits
// by the sampler itself (the repeat penalty is a kernel of its own); filters are kept
// as thresholds.  All sums are taken in a fixed order, so a row's token depends only
// on its logits, its options and its draw r, not on the other rows.
#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_LIST = 1024;            // most elements that the sampler's short way lists after top-k

// Monotone map of a float to an unsigned key (larger float -> larger key).
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = -INFINITY;
        for (int i = 0; i < n_warps; ++i) t = fmaxf(t, scratch[i]);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Greedy: strict '>' scan from element 0, so the lowest index wins ties, a NaN is never chosen over a
// number, and a row that begins with NaN yields 0 (src/sampling.c:214-224).  Value and index are packed
// into one 64-bit key whose maximum is that element: the value's order key above, the complement of
// the index below.
__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
    if (v != v) return i == 0 ? ~0ull : 0ull;
    if (v == 0.0f) v = 0.0f;                          // -0 and +0 compare equal
    return ((unsigned long long)order_key(v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(int32_t* __restrict__ out, const float* __restrict__ logits, int V, size_t ld) {
    __shared__ unsigned long long best[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    unsigned long long key = 0;
    // scalar head up to a 16-byte boundary, 16-byte body, scalar tail
    const int head = min(V, (int)((4 - ((reinterpret_cast<uintptr_t>(row) >> 2) & 3)) & 3));
    const int n4 = (V - head) >> 2;
    if ((int)threadIdx.x < head) key = argmax_key(row[threadIdx.x], threadIdx.x);
    const float4* body = reinterpret_cast<const float4*>(row + head);
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
        const float4 v = body[j];
        const int i = head + 4 * j;
        unsigned long long k0 = argmax_key(v.x, i), k1 = argmax_key(v.y, i + 1);
        unsigned long long k2 = argmax_key(v.z, i + 2), k3 = argmax_key(v.w, i + 3);
        k0 = k0 > k1 ? k0 : k1;
        k2 = k2 > k3 ? k2 : k3;
        k0 = k0 > k2 ? k0 : k2;
        key = key > k0 ? key : k0;
    }
    for (int i = head + 4 * n4 + threadIdx.x; i < V; i += blockDim.x) {
        const unsigned long long k = argmax_key(row[i], i);
        key = key > k ? key : k;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = key > other ? key : other;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) best[warp] = key;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        key = lane < n_warps ? best[lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
            key = key > other ? key : other;
        }
        // ~0: the row begins with NaN.  0 cannot be left over: element 0 is a number or has won.
        if (lane == 0) out[blockIdx.x] = key == 0ull || key == ~0ull ? 0 : (int32_t)(0xffffffffu - (uint32_t)key);
    }
}

// Divide positive and multiply negative logits of the recent tokens by the penalty,
// once per occurrence, in the order of the window (src/sampling.c:59-74).
__global__ void repeat_penalty_kernel(float* __restrict__ logits, int V, size_t ld,
                                      const int32_t* __restrict__ recent, int window,
                                      const int32_t* __restrict__ n_recent, float penalty) {
    // One thread per entry of the window.  The thread of a token's first occurrence applies the penalty as
    // often as the token occurs, one division or multiplication after the other as a walk through the window
    // would, so the result is the same bits; the tokens' loads and stores go side by side instead of one
    // round trip after the other (64 entries: some 45 us in one thread).
    const int row = blockIdx.x;
    float* x = logits + (size_t)row * ld;
    const int n = min(n_recent[row], window);
    const int32_t* mine = recent + (size_t)row * window;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int t = mine[i];
        if (t < 0 || t >= V) continue;
        bool first = true;
        for (int j = 0; j < i; ++j) first = first && mine[j] != t;
        if (!first) continue;
        int times = 0;
        for (int j = i; j < n; ++j) times += mine[j] == t ? 1 : 0;
        float v = x[t];
        for (int c = 0; c < times; ++c) v = v > 0.f ? v / penalty : v * penalty;
        x[t] = v;
    }
}

// Temperature, top-k, top-p, softmax, inverse-CDF (src/sampling.c:227-250), for a
// temperature >= 0.01 (the caller sends greedy rows to argmax_kernel).
//   y = x / T (unless T == 1)                                              (:50-56)
//   top-k: y below the k-th largest is dropped, ties at it stay            (:77-118)
//   top-p: of softmax(y), in descending order (equal values: lower index first), keep
//          through the first element whose cumulative probability exceeds p (:121-175)
//   draw: first index with cumulative probability >= r; if none, the last kept (:199-211)
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(int32_t* __restrict__ out, const float* __restrict__ logits, int V, size_t ld,
              float temperature, int top_k, float top_p, const float* __restrict__ draws) {
    __shared__ float scratch[33];
    __shared__ float chunk_sum[SAMPLE_THREADS];
    __shared__ int chunk_ties[SAMPLE_THREADS];
    __shared__ int result;
    __shared__ int hist[256];
    __shared__ uint32_t sel_prefix;
    __shared__ int sel_remaining, list_n, list_kept;
    const float* x = logits + (size_t)blockIdx.x * ld;
    const float inv_t = temperature == 1.0f ? 1.0f : 1.0f / temperature;
    const int tid = threadIdx.x;

    // The k-th largest key, one byte of it per pass over the row: a count of the candidates' next byte
    // (integers: the order of the additions does not matter), then the byte at which the count from the top
    // reaches what is still wanted.  (One bit per pass, 32 passes with a sum over the block each, took 150 us
    // of a 300 us kernel at a vocabulary of 50,400.)
    uint32_t k_key = 0;                              // keep everything
    // Without top-k, top-p alone mostly keeps a few elements too: the SAMPLE_LIST largest are listed as if k were
    // that, with the sum over the whole row as the total; if their share does not reach p, the general way is gone.
    const bool real_k = top_k > 0 && top_k < V;
    const bool stand_in = !real_k && top_p > 0.f && top_p < 1.f;
    const int k_sel = real_k ? top_k : min(V, SAMPLE_LIST);
    if (real_k || stand_in) {
        if (tid == 0) { sel_prefix = 0; sel_remaining = k_sel; }
        for (int shift = 24; shift >= 0 && k_sel < V; shift -= 8) {
            if (tid < 256) hist[tid] = 0;
            __syncthreads();
            const uint32_t prefix = sel_prefix;
            for (int i = tid; i < V; i += blockDim.x) {
                const uint32_t key = order_key(x[i] * inv_t);
                if (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(key >> shift) & 255u], 1);
            }
            __syncthreads();
            if (tid == 0) {
                int want = sel_remaining, d = 255;
                for (; d > 0; --d) {
                    if (hist[d] >= want) break;
                    want -= hist[d];
                }
                sel_prefix = prefix | ((uint32_t)d << shift);
                sel_remaining = want;
            }
            __syncthreads();
        }
        k_key = k_sel < V ? sel_prefix : 0u;

        // The elements that top-k keeps (k of them, and the ties at the k-th value) are few: they are listed,
        // put in the order that top-p wants (falling value, equal values by rising index), and one thread does
        // the sums over them as src/sampling.c:121-211 does, in 32-bit.  A list that overflows (a very large
        // k, or thousands of equal logits) goes the general way below.
        __shared__ float l_y[SAMPLE_LIST], s_y[SAMPLE_LIST], s_w[SAMPLE_LIST];
        __shared__ int l_i[SAMPLE_LIST], s_i[SAMPLE_LIST];
        if (tid == 0) list_n = 0;
        __syncthreads();
        for (int i = tid; i < V; i += blockDim.x) {
            const float y = x[i] * inv_t;
            if (order_key(y) >= k_key) {
                const int at = atomicAdd(&list_n, 1);
                if (at < SAMPLE_LIST) { l_y[at] = y; l_i[at] = i; }
            }
        }
        __syncthreads();
        const int m = list_n;
        if (m <= SAMPLE_LIST) {
            for (int a = tid; a < m; a += blockDim.x) {              // rank in (value falling, index rising)
                const uint32_t ka = order_key(l_y[a]);
                const int ia = l_i[a];
                int rank = 0;
                for (int b = 0; b < m; ++b) {
                    const uint32_t kb = order_key(l_y[b]);
                    rank += (kb > ka || (kb == ka && l_i[b] < ia)) ? 1 : 0;
                }
                s_y[rank] = l_y[a];
                s_i[rank] = ia;
            }
            __syncthreads();
            const float top = s_y[0];
            for (int a = tid; a < m; a += blockDim.x) s_w[a] = expf(s_y[a] - top);
            float z_row = 0.f;
            if (stand_in) {                                          // the total is the whole row's
                for (int i = tid; i < V; i += blockDim.x) z_row += expf(x[i] * inv_t - top);
                z_row = block_sum(z_row, scratch);
            }
            __syncthreads();
            if (tid == 0) {
                int kept = m;
                float z = z_row;
                if (!stand_in)
                    for (int a = 0; a < m; ++a) z += s_w[a];
                if (top_p > 0.f && top_p < 1.f && z > 0.f) {
                    const float limit = top_p * z;
                    float run = 0.f;
                    bool found = false;
                    for (int a = 0; a < m && !found; ++a) {
                        run += s_w[a];
                        if (run > limit) { kept = a + 1; found = true; }
                    }
                    if (stand_in && !found && m < V) kept = -1;      // the list does not hold the whole of top-p
                } else if (stand_in && m < V) kept = -1;
                list_kept = kept;
            }
            __syncthreads();
            const int kept = list_kept;
            if (kept >= 0) {
                for (int a = tid; a < kept; a += blockDim.x) {           // the kept ones by rising index
                    const int ia = s_i[a];
                    int rank = 0;
                    for (int b = 0; b < kept; ++b) rank += s_i[b] < ia ? 1 : 0;
                    l_i[rank] = ia;
                    l_y[rank] = s_w[a];
                }
                __syncthreads();
                if (tid == 0) {
                    float total = 0.f;
                    for (int a = 0; a < kept; ++a) total += l_y[a];
                    const float target = draws[blockIdx.x] * total;
                    int r = -1, last = 0;
                    float run = 0.f;
                    for (int a = 0; a < kept; ++a) {
                        if (!(l_y[a] > 0.f)) continue;                   // a weight of zero (or NaN) is never drawn
                        last = l_i[a];
                        run += l_y[a];
                        if (r < 0 && run >= target) r = l_i[a];
                    }
                    out[blockIdx.x] = r >= 0 ? r : last;                 // none reached the target: the last kept, else 0
                }
                return;
            }
        }
        if (stand_in) k_key = 0;                                     // the general way filters by top-p alone
        __syncthreads();
    }

    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, x[i] * inv_t);
    mx = block_max(mx, scratch);

    float z = 0.f;
    for (int i = tid; i < V; i += blockDim.x) {
        const float y = x[i] * inv_t;
        if (order_key(y) >= k_key) z += expf(y - mx);
    }
    z = block_sum(z, scratch);

    // top-p: the key of the element at which the cumulative sum first exceeds p, and how
    // many of the elements equal to it (in index order) are kept
    uint32_t p_key = 0;
    int ties_kept = 0x7fffffff;
    if (top_p > 0.f && top_p < 1.f && z > 0.f) {
        const float limit = top_p * z;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t trial = p_key | (1u << bit);
            float s = 0.f;
            for (int i = tid; i < V; i += blockDim.x) {
                const float y = x[i] * inv_t;
                const uint32_t key = order_key(y);
                if (key >= k_key && key >= trial) s += expf(y - mx);
            }
            if (block_sum(s, scratch) > limit) p_key = trial;
        }
        float above = 0.f, at = 0.f;
        for (int i = tid; i < V; i += blockDim.x) {
            const float y = x[i] * inv_t;
            const uint32_t key = order_key(y);
            if (key >= k_key && key > p_key) above += expf(y - mx);
            if (key >= k_key && key == p_key) at = expf(y - mx);
        }
        above = block_sum(above, scratch);
        at = block_max(at, scratch);
        ties_kept = 1;
        if (at > 0.f) while (above + (float)ties_kept * at <= limit && ties_kept < V) ++ties_kept;
    }
    const uint32_t keep_key = p_key > k_key ? p_key : k_key;   // keys below this are dropped

    // chunked pass in index order: every thread owns a contiguous range
    const bool tie_rule = ties_kept != 0x7fffffff;
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int c0 = min(V, tid * per), c1 = min(V, c0 + per);
    int local_ties = 0;
    if (tie_rule)
        for (int i = c0; i < c1; ++i) local_ties += order_key(x[i] * inv_t) == p_key ? 1 : 0;
    chunk_ties[tid] = local_ties;
    if (tid == 0) result = 0x7fffffff;
    __syncthreads();
    int ties_before = 0;                              // elements equal to the cut-off value before this chunk
    if (tie_rule)
        for (int j = 0; j < tid; ++j) ties_before += chunk_ties[j];

    // weight of element i in the final distribution (0 if filtered); `rank` counts ties
    auto weight = [&](int i, int& rank) -> float {
        const float y = x[i] * inv_t;
        const uint32_t key = order_key(y);
        if (key < keep_key) return 0.f;
        if (tie_rule && key == p_key && rank++ >= ties_kept) return 0.f;
        return expf(y - mx);
    };

    float local = 0.f;
    {
        int rank = ties_before;
        for (int i = c0; i < c1; ++i) local += weight(i, rank);
    }
    chunk_sum[tid] = local;
    __syncthreads();
    if (tid == 0) {                                   // ordered prefix: chunk_sum[j] becomes the sum before chunk j
        float run = 0.f;
        for (int j = 0; j < blockDim.x; ++j) { const float c = chunk_sum[j]; chunk_sum[j] = run; run += c; }
        scratch[0] = run;
    }
    __syncthreads();
    const float total = scratch[0];
    const float target = draws[blockIdx.x] * total;
    const float before = chunk_sum[tid];
    // The first index whose cumulative weight reaches the target lies in the chunk with
    // before < target <= before + local; the walk below repeats the additions of `local`
    // exactly, so that chunk finds it.
    if (c0 < c1 && before + local >= target && (before < target || target <= 0.f)) {
        float part = 0.f;
        int rank = ties_before;
        for (int i = c0; i < c1; ++i) {
            const float wgt = weight(i, rank);
            if (wgt == 0.f) continue;
            part += wgt;
            if (before + part >= target) { atomicMin(&result, i); break; }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int r = result;
        if (r == 0x7fffffff) {                        // empty or non-finite distribution: last kept, else 0
            r = 0;
            int rank = 0;
            for (int i = 0; i < V; ++i) if (weight(i, rank) > 0.f) r = i;
        }
        out[blockIdx.x] = r;
    }
}

}  // namespace

QS_API int qs_argmax(int32_t* out, const float* logits, int rows, int V, long long ld, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && V > 0 && ld >= V, "argmax: bad sizes rows=%d V=%d ld=%lld", rows, V, ld);
    argmax_kernel<<<rows, V >= 4096 ? 1024 : 256, 0, stream>>>(out, logits, V, (size_t)ld);
    return qs_check_launch("argmax");
}

QS_API int qs_repeat_penalty(float* logits, int rows, int V, long long ld, const int32_t* recent,
                             int window, const int32_t* n_recent, float penalty, cudaStream_t stream) {
    if (rows == 0 || penalty <= 1.0f) return QS_OK;
    QS_REQUIRE(rows > 0 && V > 0 && window > 0, "repeat_penalty: bad sizes");
    repeat_penalty_kernel<<<rows, 64, 0, stream>>>(logits, V, (size_t)ld, recent, window, n_recent, penalty);
    return qs_check_launch("repeat_penalty");
}

QS_API int qs_sample(int32_t* out, const float* logits, int rows, int V, long long ld, float temperature,
                     int top_k, float top_p, const float* draws, cudaStream_t stream) {
    if (rows == 0) return QS_OK;
    QS_REQUIRE(rows > 0 && V > 0 && ld >= V, "sample: bad sizes rows=%d V=%d ld=%lld", rows, V, ld);
    QS_REQUIRE(temperature >= 0.01f, "sample: temperature %g is greedy; use argmax", (double)temperature);
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(out, logits, V, (size_t)ld, temperature, top_k, top_p, draws);
    return qs_check_launch("sample");
}
