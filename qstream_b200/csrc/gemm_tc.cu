// C = act(A W^T + bias) + res1 + res2 for bfloat16 A [M, K] and W [N, K] on the 5th-generation
// tensor cores: TMA brings 128-byte-swizzled K-major tiles into a ring of shared-memory
// stages, one elected thread issues tcgen05.mma (kind::f16, float32 accumulator in TMEM),
// four warps read the accumulator back with tcgen05.ld and apply the epilogue in 32-bit.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner and MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32 * (w % 4) .. +31).
//
// Two operand arrangements of the same kernel:
//   rows of A on the MMA's M side (128 per tile), rows of W on its N side (BN per tile): many tokens;
//   SWAP: rows of W on the M side, the few tokens of a decode step on the N side (BN = 16..64),
//         so no tensor-core row is spent on padding and every CTA streams its own slab of W.
// Each output element is accumulated over K in one TMEM cell in ascending k, so a row's result
// does not depend on the other rows of the batch.
//
// Sizes: any M, N; K a multiple of 8 (TMA row pitch of 16 bytes); tails are zero-filled by TMA.
#include "common.cuh"
#include "sm100.cuh"

#include <mutex>
#include <unordered_map>

using namespace sm100;

namespace {

constexpr int BM = 128;             // rows of the M-side operand per tile = TMEM lanes
constexpr int BK = 64;              // 64 bfloat16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET_BIG = 200 * 1024;     // many tokens: one CTA per SM, deep ring
constexpr int SMEM_BUDGET_SWAP = 100 * 1024;    // few tokens: two CTAs per SM stream weights side by side
constexpr int TARGET_CTAS = 2 * 148;            // CTAs resident at once in the weight-streaming arrangement
constexpr int MIN_KB_PER_SPLIT = 8;             // k-blocks of 64 a split-K slice keeps at least

struct Epilogue {
    void* C; int c_dtype; long long ldc;
    const void* bias; int bias_dtype; int act;
    const __nv_bfloat16* res1; const __nv_bfloat16* res2; long long ldr;
    int M, N;                       // tokens, output features
};

template <int BN> constexpr int stage_bytes() { return BM * BK * 2 + BN * BK * 2; }
template <int BN, bool SWAP> constexpr int num_stages() {
    return (SWAP ? SMEM_BUDGET_SWAP : SMEM_BUDGET_BIG) / stage_bytes<BN>();
}
template <int BN, bool SWAP> constexpr int smem_bytes() { return num_stages<BN, SWAP>() * stage_bytes<BN>() + 1024 + 256; }

__device__ __forceinline__ void store_out(const Epilogue& ep, int m, int n, float v) {
    if (ep.bias) v += load_as_f32(ep.bias, ep.bias_dtype, n);
    v = apply_activation(v, ep.act);
    if (ep.res1) v += __bfloat162float(ep.res1[(size_t)m * ep.ldr + n]);
    if (ep.res2) v += __bfloat162float(ep.res2[(size_t)m * ep.ldr + n]);
    store_from_f32(ep.C, ep.c_dtype, (size_t)m * ep.ldc + n, v);
}

template <int BN, bool SWAP>
__global__ void __launch_bounds__(THREADS, SWAP ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
               const Epilogue ep, const int K, float* __restrict__ ws, int32_t* __restrict__ counters,
               int32_t* __restrict__ status) {
    constexpr int STAGES = num_stages<BN, SWAP>();
    constexpr int STAGE = stage_bytes<BN>();
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr int CH = BN < 32 ? 16 : 32;             // accumulator columns read per tcgen05.ld

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    volatile uint32_t* aborted = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p0 = blockIdx.x * BM;                   // first row of the M-side operand
    const int q0 = blockIdx.y * BN;                   // first row of the N-side operand
    // split-K: CTA z of gridDim.z accumulates k-blocks [kb_begin, kb_end)
    const int total_kb = (K + BK - 1) / BK;
    const int splits = gridDim.z;
    const int kb_begin = (int)((long long)blockIdx.z * total_kb / splits);
    const int num_kb = (int)((long long)(blockIdx.z + 1) * total_kb / splits) - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        *aborted = 0;
        mbar_fence_init();
        prefetch_tensormap(&map_p);
        prefetch_tensormap(&map_q);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            for (int kb = 0; kb < num_kb; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (kb / STAGES) & 1;
                if (!mbar_wait(&empty[s], phase ^ 1)) { atomicExch(status, 101); *aborted = 1; break; }
                uint8_t* tile = smem + s * STAGE;
                mbar_expect_tx(&full[s], STAGE);
                tma_load_2d(tile, &map_p, &full[s], (kb_begin + kb) * BK, p0);
                tma_load_2d(tile + BM * BK * 2, &map_q, &full[s], (kb_begin + kb) * BK, q0);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
            bool ok = true;
            for (int kb = 0; kb < num_kb && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t phase = (kb / STAGES) & 1;
                if (!mbar_wait(&full[s], phase)) { atomicExch(status, 102); *aborted = 1; ok = false; break; }
                tc_fence_after_sync();
                const uint32_t a_addr = smem_u32(smem + s * STAGE);
                const uint64_t da = smem_desc_sw128(a_addr);
                const uint64_t db = smem_desc_sw128(a_addr + BM * BK * 2);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // 16 elements of K = 32 bytes = 2 units of the descriptor's address field
                    mma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                }
                mma_commit(&empty[s]);                // the stage is free once these MMAs have read it
            }
            mma_commit(acc_ready);                    // arrives even after a failed wait, so nobody hangs on it
        }
    } else {
        const int quad = warp & 3;
        bool ok = mbar_wait(acc_ready, 0);
        if (!ok) atomicExch(status, 103);
        ok = ok && *aborted == 0;
        tc_fence_after_sync();
        const int r = quad * 32 + lane;               // this thread's TMEM lane
        const int p = p0 + r;                         // its row of the M-side operand
        auto emit = [&](int c, const float (&v)[CH]) {
            if constexpr (!SWAP) {
                if (p < ep.M) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int n = q0 + c * CH + j;
                        if (n < ep.N) store_out(ep, p, n, v[j]);
                    }
                }
            } else {
                if (p < ep.N) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int m = q0 + c * CH + j;
                        if (m < ep.M) store_out(ep, m, p, v[j]);
                    }
                }
            }
        };
        if (splits == 1) {
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < BN / CH; ++c) {
                    uint32_t raw[CH];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * CH);
                    if constexpr (CH == 32) tmem_load_32x32(taddr, raw); else tmem_load_32x16(taddr, raw);
                    tmem_load_wait();
                    float v[CH];
#pragma unroll
                    for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(raw[j]);
                    emit(c, v);
                }
            }
        } else {
            // Split-K: every slice leaves its 32-bit partial tile in the workspace; the CTA that arrives
            // last adds the slices in slice order (its own included, read back like the others), so the
            // sum does not depend on which CTA finished when.
            const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
            float* mine = ws + ((tile * splits + blockIdx.z) * BN) * BM;
#pragma unroll 1
            for (int c = 0; c < BN / CH; ++c) {
                uint32_t raw[CH];
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * CH);
                if constexpr (CH == 32) tmem_load_32x32(taddr, raw); else tmem_load_32x16(taddr, raw);
                tmem_load_wait();
#pragma unroll
                for (int j = 0; j < CH; ++j) mine[(size_t)(c * CH + j) * BM + r] = ok ? __uint_as_float(raw[j]) : 0.f;
            }
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");            // the four epilogue warps
            if (threadIdx.x == 64) {
                const int prev = atomicAdd(&counters[tile], 1);
                *last_flag = (prev == splits - 1) ? 1u : 0u;
                if (prev == splits - 1) counters[tile] = 0;           // ready for the next launch
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*last_flag) {
                __threadfence();
#pragma unroll 1
                for (int c = 0; c < BN / CH; ++c) {
                    float v[CH];
#pragma unroll
                    for (int j = 0; j < CH; ++j) v[j] = 0.f;
                    for (int z = 0; z < splits; ++z) {
                        const float* part = ws + ((tile * splits + z) * BN) * BM;
#pragma unroll
                        for (int j = 0; j < CH; ++j) v[j] += __ldcg(&part[(size_t)(c * CH + j) * BM + r]);
                    }
                    emit(c, v);
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ----------------------------------------------------------------------------- persistent kernel (many tokens)

// Wait that also gives up when another role of the CTA has recorded a failure.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* aborted) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *aborted) return false;
    }
    return false;
}

template <int BN> constexpr int p_stages() { return SMEM_BUDGET_BIG / stage_bytes<BN>(); }
template <int BN> constexpr int p_smem_bytes() { return p_stages<BN>() * stage_bytes<BN>() + 1024 + 512; }

// One CTA per SM walks over output tiles of 128 x BN (tile t = n_tile * m_tiles + m_tile, so CTAs that
// run together share rows of W and all of A stays in L2).  Two accumulators in TMEM: while the four
// epilogue warps drain tile i, the MMA warp already accumulates tile i + 1 into the other one, and the
// TMA producer runs ahead across tile borders through the same ring of stages.
template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          const Epilogue ep, const int K, const int m_tiles, const int n_tiles,
                          int32_t* __restrict__ status) {
    constexpr int STAGES = p_stages<BN>();
    constexpr int STAGE = stage_bytes<BN>();
    constexpr uint32_t TMEM_COLS = 2 * BN;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;              // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* aborted = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (K + BK - 1) / BK;
    const int total_tiles = m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        *aborted = 0;
        mbar_fence_init();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_w);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t it = 0;
            for (int t = blockIdx.x; t < total_tiles && !*aborted; t += gridDim.x) {
                const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort(&empty[s], ((it / STAGES) & 1) ^ 1, aborted)) { atomicExch(status, 121); *aborted = 1; break; }
                    uint8_t* tile = smem + s * STAGE;
                    mbar_expect_tx(&full[s], STAGE);
                    tma_load_2d(tile, &map_a, &full[s], kb * BK, m0);
                    tma_load_2d(tile + BM * BK * 2, &map_w, &full[s], kb * BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
            uint32_t it = 0;
            int i = 0;
            for (int t = blockIdx.x; t < total_tiles && !*aborted; t += gridDim.x, ++i) {
                const int buf = i & 1;
                if (!wait_or_abort(&acc_empty[buf], ((i >> 1) & 1) ^ 1, aborted)) { atomicExch(status, 122); *aborted = 1; break; }
                tc_fence_after_sync();
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_or_abort(&full[s], (it / STAGES) & 1, aborted)) { atomicExch(status, 123); *aborted = 1; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + s * STAGE);
                    const uint64_t da = smem_desc_sw128(a_addr);
                    const uint64_t db = smem_desc_sw128(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_bf16(tmem_base + (uint32_t)(buf * BN), da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    mma_commit(&empty[s]);
                }
                mma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const bool vec_ok = ep.c_dtype == QS_BF16 && (ep.ldc % 8) == 0 && ((uintptr_t)ep.C % 16) == 0 &&
                            (!ep.res1 || ((ep.ldr % 8) == 0 && ((uintptr_t)ep.res1 % 16) == 0)) &&
                            (!ep.res2 || ((uintptr_t)ep.res2 % 16) == 0);
        int i = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, ++i) {
            const int buf = i & 1;
            const int m = (t % m_tiles) * BM + r, n0 = (t / m_tiles) * BN;
            if (!wait_or_abort(&acc_full[buf], (i >> 1) & 1, aborted)) { atomicExch(status, 124); *aborted = 1; break; }
            tc_fence_after_sync();
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t raw[32];
                tmem_load_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN + c * 32), raw);
                tmem_load_wait();
                const int nc = n0 + c * 32;
                if (m >= ep.M || nc >= ep.N) continue;
                if (vec_ok && nc + 32 <= ep.N) {
                    // 32 consecutive outputs of one row: bias and activation on the accumulator, residuals
                    // added in 32-bit, one rounding, four 16-byte stores
                    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(ep.C) + (size_t)m * ep.ldc + nc;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float x = __uint_as_float(raw[g * 8 + j]);
                            if (ep.bias) x += load_as_f32(ep.bias, ep.bias_dtype, nc + g * 8 + j);
                            v[j] = apply_activation(x, ep.act);
                        }
                        if (ep.res1) {
                            const uint4 rr = *reinterpret_cast<const uint4*>(ep.res1 + (size_t)m * ep.ldr + nc + g * 8);
                            const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) { v[2 * j] += __uint_as_float(w[j] << 16); v[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u); }
                        }
                        if (ep.res2) {
                            const uint4 rr = *reinterpret_cast<const uint4*>(ep.res2 + (size_t)m * ep.ldr + nc + g * 8);
                            const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) { v[2 * j] += __uint_as_float(w[j] << 16); v[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u); }
                        }
                        uint32_t o[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const __nv_bfloat162 pb = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            o[j] = *reinterpret_cast<const uint32_t*>(&pb);
                        }
                        *reinterpret_cast<uint4*>(crow + g * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (nc + j < ep.N) store_out(ep, m, nc + j, __uint_as_float(raw[j]));
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&acc_empty[buf]);
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

struct MapKey {
    const void* ptr; long long rows, cols, ld; int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        for (long long v : {k.rows, k.cols, k.ld, (long long)k.box_rows}) h = h * 1000003u ^ (size_t)v;
        return h;
    }
};

// Tensor map of a row-major bfloat16 matrix [rows, cols] with row stride ld (elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zero fill outside.  Maps are cached by their key.
int tensor_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    const MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return QS_OK; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return qs_fail(QS_ERR_INTERNAL, "gemm_tc: the driver offers no cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return qs_fail(QS_ERR_INTERNAL, "gemm_tc: cuTensorMapEncodeTiled failed with %d (rows=%lld cols=%lld ld=%lld)",
                       (int)r, rows, cols, ld);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return QS_OK;
}

// How many split-K slices the weight-streaming arrangement uses: a function of N and K only, never of
// the number of tokens, so that a token's result does not depend on its batch.
int choose_splits(int N, int K) {
    const int tiles = (N + BM - 1) / BM;
    const int total_kb = (K + BK - 1) / BK;
    int splits = (TARGET_CTAS + tiles / 2) / tiles;
    if (splits > total_kb / MIN_KB_PER_SPLIT) splits = total_kb / MIN_KB_PER_SPLIT;
    return splits < 1 ? 1 : splits;
}

template <int BN, bool SWAP>
int launch(const CUtensorMap& mp, const CUtensorMap& mq, const Epilogue& ep, int p_rows, int q_rows, int K,
           int splits, float* ws, int32_t* counters, int32_t* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             smem_bytes<BN, SWAP>());
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gemm_tc: shared memory of %d bytes refused: %s",
                                             smem_bytes<BN, SWAP>(), cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((p_rows + BM - 1) / BM, (q_rows + BN - 1) / BN, splits);
    gemm_tc_kernel<BN, SWAP><<<grid, THREADS, smem_bytes<BN, SWAP>(), stream>>>(mp, mq, ep, K, ws, counters, status);
    return qs_check_launch("gemm_tc");
}

template <int BN>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mw, const Epilogue& ep, int M, int N, int K,
                      int32_t* status, cudaStream_t stream) {
    static bool configured = false;
    static int sm_count = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             p_smem_bytes<BN>());
        int dev = 0;
        if (e == cudaSuccess) e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gemm_tc: set-up of the persistent kernel failed: %s",
                                             cudaGetErrorString(e));
        configured = true;
    }
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const long long total = (long long)m_tiles * n_tiles;
    const int grid = (int)(total < sm_count ? total : sm_count);
    gemm_tc_persistent_kernel<BN><<<grid, THREADS, p_smem_bytes<BN>(), stream>>>(ma, mw, ep, K, m_tiles, n_tiles, status);
    return qs_check_launch("gemm_tc persistent");
}

}  // namespace

// A: [M, K] bfloat16, row stride lda; W: [N, K] bfloat16 contiguous; C: [M, N] bfloat16 or float32.
// res1/res2: bfloat16 [M, N] with row stride ldr, or null.  status: device int32 that receives a
// non-zero code if a bounded wait inside the kernel ran out.
// ws / counters: scratch for split-K in the weight-streaming arrangement (M <= 64): `ws_floats` floats
// and `n_counters` int32 that are ZERO before the first call (the kernel leaves them zero).  Without
// them (null) the product runs unsplit.  Calls that share the scratch must not overlap on the GPU.
QS_API int qs_gemm_tc(void* C, int c_dtype, const void* A, const void* W, const void* bias, int bias_dtype, int act,
                      const void* res1, const void* res2, int M, int N, int K, long long lda, long long ldc,
                      long long ldr, float* ws, long long ws_floats, int32_t* counters, int n_counters,
                      int32_t* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return QS_OK;
    QS_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    QS_REQUIRE(K % 8 == 0 && lda % 8 == 0, "gemm_tc: K=%d and the row stride %lld must be multiples of 8", K, lda);
    QS_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_tc: operands must be 16-byte aligned");
    QS_REQUIRE(c_dtype == QS_F32 || c_dtype == QS_BF16, "gemm_tc: unknown output type %d", c_dtype);
    Epilogue ep{C, c_dtype, ldc, bias, bias_dtype, act, (const __nv_bfloat16*)res1, (const __nv_bfloat16*)res2, ldr, M, N};
    CUtensorMap ma, mw;
    int rc;
    if (M > 64) {
        QS_REQUIRE((M + BM - 1) / BM <= 65535 * 1 && (N + 127) / 128 <= 65535, "gemm_tc: sizes exceed the grid");
        if ((rc = tensor_map(&ma, A, M, K, lda, BM)) != QS_OK) return rc;
        const int bn = N > 128 ? 256 : 128;
        if ((rc = tensor_map(&mw, W, N, K, K, bn)) != QS_OK) return rc;
        if (bn == 256) return launch_persistent<256>(ma, mw, ep, M, N, K, status, stream);
        return launch_persistent<128>(ma, mw, ep, M, N, K, status, stream);
    }
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    int splits = choose_splits(N, K);
    const long long tiles = (N + BM - 1) / BM;
    if (!ws || !counters || tiles > n_counters || tiles * splits * 64 * BM > ws_floats) splits = 1;
    if ((rc = tensor_map(&mw, W, N, K, K, BM)) != QS_OK) return rc;
    if ((rc = tensor_map(&ma, A, M, K, lda, bn)) != QS_OK) return rc;
    if (bn == 16) return launch<16, true>(mw, ma, ep, N, M, K, splits, ws, counters, status, stream);
    if (bn == 32) return launch<32, true>(mw, ma, ep, N, M, K, splits, ws, counters, status, stream);
    return launch<64, true>(mw, ma, ep, N, M, K, splits, ws, counters, status, stream);
}
