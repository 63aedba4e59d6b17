// Prefill attention for bfloat16 on the 5th-generation tensor cores: 128 query rows of one
// sequence and head per CTA against the sequence's paged cache, one page of 64 keys at a time.
//
//   S = Q K^T        tcgen05.mma, Q [128 x dh] and K [64 x dh] both K-major in shared memory (TMA,
//                    128-byte swizzle), S [128 x 64] float32 in TMEM (two buffers)
//   softmax          four warps, one thread per query row: tcgen05.ld S, scale, causal / window mask,
//                    running maximum and sum in 32-bit, P = exp2(s - m) rounded to bfloat16 (the sum is
//                    taken over the unrounded weights) and
//                    written to shared memory in the swizzled K-major layout the MMA reads
//   O += P V         tcgen05.mma, V [64 keys x dh] as the page lies in the cache (MN-major), O
//                    [128 x dh] float32 in TMEM; O is rescaled in TMEM only when a row's maximum has
//                    grown by more than 2^8 since the scale it was accumulated under
//   out = O / l      read back, normalised, rounded to bfloat16
//
// Formulas: scores q.k / sqrt(dh) over keys u <= position (QStream src/engine.c:888-906), softmax
// with maximum subtraction (src/kernels_scalar.c:188-213), weighted sum of values (src/engine.c:913-922).
//
// Warp roles (192 threads): warp 0 = TMA producer (walks the page table), warp 1 = TMEM owner and
// MMA issuer, warps 2..5 = softmax and epilogue (warp w owns TMEM lanes 32 * (w % 4) .. +31).
// A row's result depends on its own sequence only: keys are visited page by page in position order
// whatever else is in the batch and wherever the pages lie.
//
// Sizes: head size a multiple of 16 up to 256 (tiles are padded to 64 columns with TMA's zero fill);
// any number of heads and groups; pages of 64 tokens.
#include "common.cuh"
#include "sm100.cuh"

#include <mutex>
#include <unordered_map>

using namespace sm100;

namespace {

constexpr int BM = 128;          // query rows per CTA = TMEM lanes
constexpr int BN = 64;           // keys per block = one cache page
constexpr int KC = 64;           // columns of one swizzled tile (128 bytes of bfloat16)
constexpr int THREADS = 320;      // producer warp, MMA warp, eight softmax warps
constexpr float RESCALE_THRESHOLD = 8.0f;        // log2 units

struct TileInfo { int row_start, n_rows, qpos0, slot; };

// 2^x on the special-function unit (relative error about 2^-22; -inf gives 0).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The value rounded up (toward +inf) to one whose low 16 bits are zero; -inf and +inf stay.
__device__ __forceinline__ float round_up_16(float x) {
    const uint32_t u = __float_as_uint(x);
    if ((u & 0xffffu) == 0u) return x;
    return __uint_as_float(x > 0.f ? (u + 0x10000u) & 0xffff0000u : u & 0xffff0000u);
}

template <int NKC> constexpr int kv_stages() { return NKC == 4 ? 2 : (NKC == 3 ? 3 : 4); }
template <int NKC> constexpr int q_bytes() { return BM * KC * 2 * NKC; }
template <int NKC> constexpr int kv_tile_bytes() { return BN * KC * 2 * NKC; }      // one of K or V
constexpr int P_BYTES = BM * BN * 2;            // one buffer of softmax weights; there are two
template <int NKC> constexpr int smem_bytes() {
    return q_bytes<NKC>() + 2 * kv_stages<NKC>() * kv_tile_bytes<NKC>() + 2 * P_BYTES + 1024 + 512 + 4 * BM * 2;
}

template <int NKC>
__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out, size_t ldo,
                         const TileInfo* __restrict__ tiles, const int32_t* __restrict__ page_table, int max_pages,
                         int n_heads, int n_kv_heads, int dh, float scale_log2, int window,
                         int32_t* __restrict__ status) {
    constexpr int STAGES = kv_stages<NKC>();
    constexpr int KV_TILE = kv_tile_bytes<NKC>();
    constexpr uint32_t TMEM_COLS = NKC <= 2 ? 256 : 512;
    constexpr uint32_t O_COL = 2 * BN;                   // S buffers at columns 0 and 64, O from 128

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;
    uint8_t* kv_smem = q_smem + q_bytes<NKC>();          // per stage: K tile then V tile
    uint8_t* p_smem = kv_smem + 2 * STAGES * KV_TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + 2 * P_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = k_full + STAGES;
    uint64_t* k_empty = v_full + STAGES;                  // a K tile is free once its Q K^T has completed,
    uint64_t* v_empty = k_empty + STAGES;                 // a V tile once its P V has: the next keys load under the softmax
    uint64_t* s_full = v_empty + STAGES;                  // [2]
    uint64_t* p_full = s_full + 2;                        // [2]
    uint64_t* p_free = p_full + 2;                        // [2]
    uint64_t* pv_done = p_free + 2;
    uint64_t* o_done = pv_done + 1;                       // the last P V of the tile has completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
    volatile uint32_t* aborted = tmem_slot + 1;
    uint16_t* row_max = reinterpret_cast<uint16_t*>(bars + 64);    // [2 buffers][2 halves][BM], 512 bytes behind the barriers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heads are the fast grid dimension and the tiles come longest first: CTAs start in order of falling
    // work, so the last ones to start are the shortest (a causal tile's work grows with its position)
    const TileInfo tile = tiles[blockIdx.y];
    if (tile.n_rows <= 0) return;             // an unused entry of a tile list of fixed length (captured steps): the whole CTA leaves
    const int head = blockIdx.x;
    const int kvh = head / (n_heads / n_kv_heads);
    const int qpos_last = tile.qpos0 + tile.n_rows - 1;
    const int first_key = window > 0 ? max(0, tile.qpos0 - window + 1) : 0;
    const int block_first = first_key / BN;
    const int n_blocks = qpos_last / BN - block_first + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_empty[s], 1); }
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(&p_full[0], 2 * BM);
        mbar_init(&p_full[1], 2 * BM);
        mbar_init(&p_free[0], 1);
        mbar_init(&p_free[1], 1);
        mbar_init(pv_done, 1);
        mbar_init(o_done, 1);
        *aborted = 0;
        mbar_fence_init();
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (elect_one()) {
            mbar_expect_tx(q_full, q_bytes<NKC>());
#pragma unroll
            for (int c = 0; c < NKC; ++c)
                tma_load_2d(q_smem + c * BM * KC * 2, &map_q, q_full, head * dh + c * KC, tile.row_start);
            const int32_t* pages = page_table + (size_t)tile.slot * max_pages;
            auto tile_row = [&](int j) {
                int page = pages[block_first + j];
                if (page < 0) { atomicExch(status, 3); page = 0; }       // still fill the stage so nobody waits for it
                return (page * n_kv_heads + kvh) * BN;
            };
            auto load_k = [&](int j) -> bool {
                const int st = j % STAGES;
                if (!mbar_wait(&k_empty[st], ((j / STAGES) & 1) ^ 1)) { atomicExch(status, 111); *aborted = 1; return false; }
                const int row = tile_row(j);
                uint8_t* k_tile = kv_smem + (size_t)st * 2 * KV_TILE;
                mbar_expect_tx(&k_full[st], KV_TILE);
#pragma unroll
                for (int c = 0; c < NKC; ++c) tma_load_2d(k_tile + c * BN * KC * 2, &map_k, &k_full[st], c * KC, row);
                return true;
            };
            auto load_v = [&](int j) -> bool {
                const int st = j % STAGES;
                if (!mbar_wait(&v_empty[st], ((j / STAGES) & 1) ^ 1)) { atomicExch(status, 110); *aborted = 1; return false; }
                const int row = tile_row(j);
                uint8_t* v_tile = kv_smem + (size_t)st * 2 * KV_TILE + KV_TILE;
                mbar_expect_tx(&v_full[st], KV_TILE);
#pragma unroll
                for (int c = 0; c < NKC; ++c) tma_load_2d(v_tile + c * BN * KC * 2, &map_v, &v_full[st], c * KC, row);
                return true;
            };
            // in the order in which the slots come free: keys of block j + 1 (after Q K^T of block j + 1 - STAGES),
            // then values of block j (after P V of block j - STAGES)
            bool ok = load_k(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                if (j + 1 < n_blocks) ok = load_k(j + 1);
                if (ok) ok = load_v(j);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            const uint32_t idesc_qk = idesc_bf16_f32(BM, BN);
            const uint32_t idesc_pv = idesc_bf16_f32_b_mn(BM, dh);
            const int k_steps = (dh + 15) / 16;
            bool ok = mbar_wait(q_full, 0);
            if (!ok) { atomicExch(status, 112); *aborted = 1; }
            auto issue_qk = [&](int j) -> bool {
                const int st = j % STAGES;
                if (!mbar_wait(&k_full[st], (j / STAGES) & 1)) { atomicExch(status, 113); *aborted = 1; return false; }
                tc_fence_after_sync();
                const uint32_t qa = smem_u32(q_smem);
                const uint32_t ka = smem_u32(kv_smem + (size_t)st * 2 * KV_TILE);
                for (int k = 0; k < k_steps; ++k) {
                    const uint32_t c = k >> 2, kk = k & 3;       // 64-column tile, 16-column step inside it
                    mma_bf16(tmem_base + (uint32_t)((j & 1) * BN),
                             smem_desc_sw128(qa + c * BM * KC * 2 + kk * 32),
                             smem_desc_sw128(ka + c * BN * KC * 2 + kk * 32), idesc_qk, k != 0);
                }
                mma_commit(&s_full[j & 1]);
                mma_commit(&k_empty[st]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_blocks && ok; ++j) {
                if (j + 1 < n_blocks) ok = issue_qk(j + 1);
                if (!ok) break;
                const int st = j % STAGES;
                if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1)) { atomicExch(status, 114); *aborted = 1; break; }
                if (!mbar_wait(&v_full[st], (j / STAGES) & 1)) { atomicExch(status, 115); *aborted = 1; break; }
                tc_fence_after_sync();
                const uint32_t pa = smem_u32(p_smem + (j & 1) * P_BYTES);
                const uint32_t va = smem_u32(kv_smem + (size_t)st * 2 * KV_TILE + KV_TILE);
#pragma unroll
                for (int k = 0; k < BN / 16; ++k) {
                    // P: K-major, 16 keys = 32 bytes inside the 128-byte row.  V: MN-major, 16 keys = two groups
                    // of eight 128-byte rows = 2048 bytes; 64-column blocks of the head lie 8192 bytes apart.
                    mma_bf16(tmem_base + O_COL, smem_desc_sw128(pa + k * 32),
                             smem_desc_sw128_mn(va + k * 2048, BN * KC * 2, 1024), idesc_pv, (j | k) != 0);
                }
                mma_commit(&v_empty[st]);
                mma_commit(&p_free[j & 1]);
                mma_commit(pv_done);
            }
            // The end of the tile has a barrier of its own.  `pv_done` only tells its phases apart by their
            // parity, and a softmax thread that has not waited for it in the last blocks (no rescaling) may reach
            // the end while the last but one P V is still running: a wait for the last one's parity then
            // passes at once, and the thread would read O - and reuse the weights' buffers - too early.
            mma_commit(o_done);
            if (!ok || *aborted) {                   // let the softmax warps fall through their waits
                mma_commit(&s_full[0]); mma_commit(&s_full[1]); mma_commit(pv_done);
                mma_commit(&p_free[0]); mma_commit(&p_free[1]);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax and epilogue
        // Eight warps, two threads per query row: warps 2..5 take key columns 0..31 of a block, warps 6..9
        // columns 32..63 (a warp may touch the TMEM lanes 32 (warp % 4) .. +31, so both see the same rows).
        // The two threads of a row exchange their block maxima through shared memory (one named barrier per
        // block), keep partial row sums that are added at the end, and share the columns of O between them.
        // No thread leaves the loop early: a wait that ran out clears `ok` and the thread goes on to every
        // barrier without touching anything.
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r = quad * 32 + lane;
        const bool valid = r < tile.n_rows;
        const int qpos = valid ? tile.qpos0 + r : -1;
        const int lo = (window > 0 && valid) ? max(0, qpos - window + 1) : 0;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blocks; ++j) {
            if (ok && !mbar_wait(&s_full[j & 1], (j >> 1) & 1)) { atomicExch(status, 116); ok = false; }
            if (*aborted) ok = false;
            tc_fence_after_sync();
            uint32_t raw[32];
            tmem_load_32x32(tmem_base + lane_base + (uint32_t)((j & 1) * BN + half * 32), raw);
            tmem_load_wait();
            const int key0 = (block_first + j) * BN + half * 32;
            const bool all_visible = key0 + 31 <= qpos && key0 >= lo;
            // raw scores stay in `raw`; masked ones become -inf.  The maximum is taken over four independent chains.
            if (!all_visible) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int key = key0 + c;
                    if (key > qpos || key < lo) raw[c] = 0xff800000u;       // -inf
                }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
#pragma unroll
                for (int u = 0; u < 4; ++u) mx[u] = fmaxf(mx[u], __uint_as_float(raw[c + u]));
            }
            // The maximum only steadies the exponentials: any common value at or above the true one serves.  The
            // two threads exchange theirs rounded up to 16 bits (half the shared memory) and both use the
            // larger of the two rounded values.
            const float mine = round_up_16(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
            uint16_t* xch = row_max + (j & 1) * 2 * BM;   // two buffers: block j + 2 writes only after everyone passed barrier j + 1
            xch[half * BM + r] = (uint16_t)(__float_as_uint(mine) >> 16);
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");      // the row's two threads sit in warps quad + 2 and quad + 6: a barrier of their own per quarter
            const float theirs = __uint_as_float((uint32_t)xch[(half ^ 1) * BM + r] << 16);
            const float bmax = fmaxf(mine, theirs) * scale_log2;                      // scale_log2 > 0
            // Two buffers of weights: this block's buffer is free once the P V of block j - 2 has completed
            // (a barrier per buffer), so these exponentials run under the P V of block j - 1.
            if (ok && j > 1 && !mbar_wait(&p_free[j & 1], ((j >> 1) - 1) & 1)) { atomicExch(status, 117); ok = false; }
            const bool grow = ok && (bmax > m + RESCALE_THRESHOLD || (m == -INFINITY && bmax > -INFINITY));
            if (__any_sync(0xffffffffu, grow)) {         // tcgen05.ld/st are warp-wide: the whole warp goes
                const float m_new = grow ? bmax : m;
                const float alpha = (m == -INFINITY) ? 0.f : fast_exp2(m - m_new);     // 1 where the row keeps its scale
                if (j > 0) {
                    // O may only be touched between two P V products; the row's two threads take every other chunk
                    if (ok && !mbar_wait(pv_done, (j - 1) & 1)) { atomicExch(status, 119); ok = false; }
                    tc_fence_after_sync();
                    for (int c = half; c * 32 < dh; c += 2) {
                        uint32_t o[32];
                        tmem_load_32x32(tmem_base + lane_base + O_COL + (uint32_t)(c * 32), o);
                        tmem_load_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_store_32x32(tmem_base + lane_base + O_COL + (uint32_t)(c * 32), o);
                    }
                    tmem_store_wait();
                }
                l *= alpha;
                m = m_new;
            }
            // P = exp2(s * scale - m) (one FMA and one ex2 per score), rounded to bfloat16 and written in the
            // swizzled K-major layout; the row sum is taken in 32-bit over two independent chains.
            if (ok) {
                uint8_t* prow = p_smem + (j & 1) * P_BYTES + (size_t)r * 128;
                const float neg_m = m == -INFINITY ? -INFINITY : -m;          // a row with no visible key so far: all weights 0
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c = ch * 8 + 2 * i;
                        const float sa = __uint_as_float(raw[c]), sb = __uint_as_float(raw[c + 1]);
                        const float a = neg_m == -INFINITY ? 0.f : fast_exp2(fmaf(sa, scale_log2, neg_m));
                        const float b = neg_m == -INFINITY ? 0.f : fast_exp2(fmaf(sb, scale_log2, neg_m));
                        ps0 += a;
                        ps1 += b;
                        const __nv_bfloat162 pb = __floats2bfloat162_rn(a, b);
                        w[i] = *reinterpret_cast<const uint32_t*>(&pb);
                    }
                    *reinterpret_cast<uint4*>(prow + (((half * 4 + ch) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                l += ps0 + ps1;
                fence_proxy_async_smem();
                tc_fence_before_sync();
                mbar_arrive(&p_full[j & 1]);
            }
        }
        if (ok && !mbar_wait(o_done, 0)) { atomicExch(status, 118); ok = false; }
        // the row's sum: the two partial sums in the order of their columns
        float* lsum = reinterpret_cast<float*>(p_smem);   // the weights' buffers are free now
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
        lsum[half * BM + r] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
        const float l_all = lsum[r] + lsum[BM + r];
        if (ok && !*aborted) {
            tc_fence_after_sync();
            const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
            __nv_bfloat16* orow = out + (size_t)(tile.row_start + r) * ldo + (size_t)head * dh;
            for (int c = half; c * 32 < dh; c += 2) {
                uint32_t o[32];
                tmem_load_32x32(tmem_base + lane_base + O_COL + (uint32_t)(c * 32), o);
                tmem_load_wait();
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        if (c * 32 + i < dh) {
                            uint32_t w[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const __nv_bfloat162 pb = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * u]) * inv,
                                                                                 __uint_as_float(o[i + 2 * u + 1]) * inv);
                                w[u] = *reinterpret_cast<const uint32_t*>(&pb);
                            }
                            *reinterpret_cast<uint4*>(orow + c * 32 + i) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ----------------------------------------------------------------------------- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Tensor map of a row-major bfloat16 matrix [rows, cols], row stride ld elements, boxes of box_rows x 64
// elements with the 128-byte swizzle and zero fill outside.
int make_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return qs_fail(QS_ERR_INTERNAL, "attention_prefill: the driver offers no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)KC, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return qs_fail(QS_ERR_INTERNAL, "attention_prefill: cuTensorMapEncodeTiled failed with %d (rows=%lld cols=%lld ld=%lld)",
                       (int)r, rows, cols, ld);
    return QS_OK;
}

template <int NKC>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, long long ldo,
           const TileInfo* tiles, int n_tiles, const int32_t* page_table, int max_pages, int n_heads, int n_kv_heads,
           int dh, float scale_log2, int window, int32_t* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<NKC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             smem_bytes<NKC>());
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "attention_prefill: shared memory of %d bytes refused: %s",
                                             smem_bytes<NKC>(), cudaGetErrorString(e));
        configured = true;
    }
    attention_prefill_kernel<NKC><<<dim3(n_heads, n_tiles), THREADS, smem_bytes<NKC>(), stream>>>(
        mq, mk, mv, (__nv_bfloat16*)out, (size_t)ldo, tiles, page_table, max_pages, n_heads, n_kv_heads, dh,
        scale_log2, window, status);
    return qs_check_launch("attention_prefill");
}

}  // namespace

// q [T, >= n_heads * dh] bfloat16 (row stride ldq), out [T, n_heads * dh] bfloat16 (row stride ldo).
// tiles: device array of n_tiles x {row_start, n_rows (<= 128), position of the first row, slot}: the
// query rows of each sequence cut into pieces of at most 128.  The cache entry is
// [n_pages][n_kv_heads][64][dh].  Keys up to each row's own position must already be in the cache.
QS_API int qs_attention_prefill(void* out, long long ldo, const void* q, long long ldq, int T_tokens,
                                const void* k_cache, const void* v_cache, int n_pages,
                                const int32_t* page_table, int max_pages, int page_tokens,
                                const int32_t* tiles, int n_tiles, int n_heads, int n_kv_heads, int dh,
                                float scale, int window, int32_t* status, cudaStream_t stream) {
    if (n_tiles == 0 || T_tokens == 0) return QS_OK;
    QS_REQUIRE(T_tokens > 0 && n_tiles > 0 && n_heads > 0 && n_kv_heads > 0 && n_pages > 0, "attention_prefill: bad sizes");
    QS_REQUIRE(page_tokens == BN, "attention_prefill: pages of %d tokens, the kernel is built for %d", page_tokens, BN);
    QS_REQUIRE(n_heads % n_kv_heads == 0, "attention_prefill: %d query heads are no multiple of %d key heads", n_heads, n_kv_heads);
    QS_REQUIRE(dh % 16 == 0 && dh >= 16 && dh <= 256, "attention_prefill: head size %d must be a multiple of 16 up to 256", dh);
    QS_REQUIRE(ldq % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)out % 16) == 0,
               "attention_prefill: rows must be 16-byte aligned");
    QS_REQUIRE(n_tiles <= 65535, "attention_prefill: %d tiles of queries are too many for the grid", n_tiles);
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = make_map(&mq, q, T_tokens, (long long)n_heads * dh, ldq, BM)) != QS_OK) return rc;
    const long long kv_rows = (long long)n_pages * n_kv_heads * BN;
    if ((rc = make_map(&mk, k_cache, kv_rows, dh, dh, BN)) != QS_OK) return rc;
    if ((rc = make_map(&mv, v_cache, kv_rows, dh, dh, BN)) != QS_OK) return rc;
    const float scale_log2 = scale * 1.4426950408889634f;
    const TileInfo* ti = reinterpret_cast<const TileInfo*>(tiles);
    const int nkc = (dh + KC - 1) / KC;
#define GO(NKC) return launch<NKC>(mq, mk, mv, out, ldo, ti, n_tiles, page_table, max_pages, n_heads, n_kv_heads, dh, \
                                   scale_log2, window, status, stream)
    if (nkc == 1) GO(1);
    if (nkc == 2) GO(2);
    if (nkc == 3) GO(3);
    GO(4);
#undef GO
}
