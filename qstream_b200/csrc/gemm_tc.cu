// C = act(A W^T + bias) + res1 + res2 for bfloat16 A [M, K] and W [N, K] on the 5th-generation
// tensor cores: TMA brings 128-byte-swizzled K-major tiles into a ring of shared-memory
// stages, one elected thread issues tcgen05.mma (kind::f16, float32 accumulator in TMEM),
// four warps read the accumulator back with tcgen05.ld and apply the epilogue in 32-bit.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner and MMA issuer,
// warps 2..5 = epilogue (warp w reads TMEM lanes 32 * (w % 4) .. +31).
//
// Two kernels:
//   many tokens (M > 128): rows of A on the MMA's M side, rows of W on its N side; a persistent CTA per SM
//       walks over 128 x 256 output tiles with two TMEM accumulators, so the epilogue of one tile runs
//       under the main loop of the next;
//   few tokens (M <= 128): rows of W on the M side and the tokens on the N side (16, 32, 64 or 128), so no
//       tensor-core row is spent on padding; one CTA per SM streams whole tiles of W, or - for a narrow
//       N - an even share of all k-blocks (stream-K) with a deterministic reduction of partial tiles.
// Each output element is accumulated over K in ascending k (in one TMEM cell, or in a fixed sequence of
// partial sums), so a row's result does not depend on the other rows of the batch.
//
// Sizes: any M, N; K a multiple of 8 (TMA row pitch of 16 bytes); tails are zero-filled by TMA.
#include "common.cuh"
#include "sm100.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

using namespace sm100;

namespace {

constexpr int BM = 128;             // rows of the M-side operand per tile = TMEM lanes
constexpr int BK = 64;              // 64 bfloat16 = one 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int SMEM_BUDGET_BIG = 200 * 1024;     // one CTA per SM with a deep ring of stages
constexpr int MIN_KB_PER_SPLIT = 8;             // k-blocks of 64 a CTA's share keeps at least

struct Epilogue {
    void* C; int c_dtype; long long ldc;
    const void* bias; int bias_dtype; int act;
    const __nv_bfloat16* res1; const __nv_bfloat16* res2; long long ldr;
    int M, N;                       // tokens, output features
};

template <int BN> constexpr int stage_bytes() { return BM * BK * 2 + BN * BK * 2; }

__device__ __forceinline__ void store_out(const Epilogue& ep, int m, int n, float v) {
    if (ep.bias) v += load_as_f32(ep.bias, ep.bias_dtype, n);
    v = apply_activation_fast(v, ep.act);
    if (ep.res1) v += __bfloat162float(ep.res1[(size_t)m * ep.ldr + n]);
    if (ep.res2) v += __bfloat162float(ep.res2[(size_t)m * ep.ldr + n]);
    store_from_f32(ep.C, ep.c_dtype, (size_t)m * ep.ldc + n, v);
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
        const bool bias_vec = ep.bias && ((uintptr_t)ep.bias % 32) == 0;
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
                        float v[8], bv[8];
                        if (ep.bias) {
                            if (bias_vec) load8_as_f32(ep.bias, ep.bias_dtype, nc + g * 8, bv);
                            else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) bv[j] = load_as_f32(ep.bias, ep.bias_dtype, nc + g * 8 + j);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float x = __uint_as_float(raw[g * 8 + j]);
                            if (ep.bias) x += bv[j];
                            v[j] = apply_activation_fast(x, ep.act);
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

// ----------------------------------------------------------------------------- persistent kernel on CTA pairs

// per CTA and stage: 128 rows of A and its half of the PAIR_BN rows of W, 64 wide
// Epilogue warps of the pair kernel: four, or eight (each TMEM lane quarter then has two warps that share the
// tile's columns).  Eight were measured: a product of one round of tiles gains 7 % (256 x 16384 x 4096: 39 -> 36 us),
// one whose k-ranges are cut loses 6 to 9 %, and 2,048-token products stay where they are or lose 2 %.
constexpr int PAIR_EPILOGUE_THREADS = 128;
constexpr int PAIR_THREADS = 64 + PAIR_EPILOGUE_THREADS;      // producer warp, MMA warp, epilogue warps
template <int PAIR_BN> constexpr int pair_stage() { return BM * BK * 2 + (PAIR_BN / 2) * BK * 2; }
template <int PAIR_BN> constexpr int pair_stages() { return SMEM_BUDGET_BIG / pair_stage<PAIR_BN>(); }
template <int PAIR_BN> constexpr int pair_smem() { return pair_stages<PAIR_BN>() * pair_stage<PAIR_BN>() + 1024 + 512 + PAIR_BN * 4; }

// Like wait_or_abort, and it also gives up when any CTA of the grid has reported a failure.
__device__ __forceinline__ bool wait_or_abort_grid(uint64_t* bar, uint32_t parity, volatile uint32_t* aborted,
                                                   const int32_t* status) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && (*aborted || *reinterpret_cast<const volatile int32_t*>(status) != 0)) return false;
    }
    return false;
}

// Where tile number `tile` lies: tiles are walked group by group of `gm` pairs of row tiles, inside a group
// column tile by column tile, rows fastest.  The rows of A that the CTA pairs work on at a time then stay
// within one group, which the host sizes to fit L2: without groups, with more rows of A than L2 holds (8,192
// tokens and more at K = 4096), every round of tiles read all of A from memory again.
__device__ __forceinline__ void pair_tile_coords(int tile, int m_pairs, int n_tiles, int gm, int& m, int& n) {
    const int per_group = gm * n_tiles;
    const int g = tile / per_group, idx = tile - g * per_group;
    const int here = min(gm, m_pairs - g * gm);       // the last group may hold fewer rows
    n = idx / here;
    m = g * gm + (idx - n * here);
}

// Two CTAs on neighbouring SMs work on one 256 x PAIR_BN output tile (PAIR_BN = 256, or 192 where that wastes
// less of the last round of tiles) with tcgen05.mma.cta_group::2: each CTA
// loads its own 128 rows of A and its own half of the W tile - half the shared-memory traffic
// per flop of the single-CTA kernel - and holds its 128 x PAIR_BN half of the accumulator in its TMEM.  The
// even CTA (the leader) issues the MMAs for both; all TMA bytes of a stage are counted on the leader's
// barrier; tcgen05.commit tells both CTAs when a stage or an accumulator may be used again; the other
// CTA's epilogue warps signal the leader across the cluster.  No load uses multicast.
template <int PAIR_BN>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const Epilogue ep, const int K, const int m_pairs, const int n_tiles, const int splits, const int gm,
                    float* __restrict__ ws, int32_t* __restrict__ counters, int32_t* __restrict__ status) {
    constexpr int PAIR_STAGE = pair_stage<PAIR_BN>();
    constexpr int PAIR_STAGES = pair_stages<PAIR_BN>();
    constexpr uint32_t TMEM_COLS = 512;             // two accumulators of PAIR_BN columns; a power of two
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + PAIR_STAGES * PAIR_STAGE);
    uint64_t* empty = full + PAIR_STAGES;
    uint64_t* acc_full = empty + PAIR_STAGES;         // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2], the leader's counts both CTAs' epilogue threads
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* aborted = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;
    float* s_bias = reinterpret_cast<float*>(smem + PAIR_STAGES * PAIR_STAGE + 512);     // [PAIR_BN]: the tile's bias

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs_grid = gridDim.x >> 1;
    const int num_kb = (K + BK - 1) / BK;
    // A work unit is a tile, or (splits > 1: fewer tiles than CTA pairs) one of `splits` equal parts of a
    // tile's k-range; the parts of a tile are neighbouring units, so they run at the same time.
    const int total_tiles = m_pairs * n_tiles * splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * PAIR_EPILOGUE_THREADS); }
        *aborted = 0;
        mbar_fence_init();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_w);
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();                                   // both CTAs' barriers exist before anyone signals across
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    grid_dep_launch();                                // the next kernel may set itself up beside this one
    if (warp == 0) {
        if (elect_one()) {
            // Launched as a programmatic dependent: the weights, which no kernel writes, fill the ring while the
            // previous kernel may still be running; the rows of A of those stages follow once it has completed.
            uint32_t it = 0;
            bool waited = false;
            int late_kb[PAIR_STAGES], late_m0[PAIR_STAGES];
            auto catch_up = [&]() {
                grid_dep_wait();
                waited = true;
                const int n_late = (int)min(it, (uint32_t)PAIR_STAGES);
                for (int s = 0; s < n_late; ++s)
                    tma_load_2d_pair(smem + s * PAIR_STAGE, &map_a, &full[s], late_kb[s] * BK, late_m0[s]);
            };
            for (int t = pair; t < total_tiles && !*aborted; t += n_pairs_grid) {
                const int tile = t / splits, part = t - tile * splits;
                int tm, tn;
                pair_tile_coords(tile, m_pairs, n_tiles, gm, tm, tn);
                const int m0 = tm * 2 * BM + (int)rank * BM;
                const int n0 = tn * PAIR_BN + (int)rank * (PAIR_BN / 2);
                const int kb_end = (int)((long long)(part + 1) * num_kb / splits);
                for (int kb = (int)((long long)part * num_kb / splits); kb < kb_end; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    if (!waited && it >= (uint32_t)PAIR_STAGES) catch_up();
                    if (!wait_or_abort_grid(&empty[s], ((it / PAIR_STAGES) & 1) ^ 1, aborted, status)) { atomicExch(status, 151); *aborted = 1; break; }
                    uint8_t* st = smem + s * PAIR_STAGE;
                    if (rank == 0) mbar_expect_tx(&full[s], 2 * PAIR_STAGE);     // both CTAs' bytes
                    if (waited) tma_load_2d_pair(st, &map_a, &full[s], kb * BK, m0);
                    else { late_kb[s] = kb; late_m0[s] = m0; }
                    tma_load_2d_pair(st + BM * BK * 2, &map_w, &full[s], kb * BK, n0);
                }
            }
            if (!waited) catch_up();
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, PAIR_BN);
            uint32_t it = 0;
            int i = 0;
            for (int t = pair; t < total_tiles && !*aborted; t += n_pairs_grid, ++i) {
                const int buf = i & 1;
                if (!wait_or_abort_grid(&acc_empty[buf], ((i >> 1) & 1) ^ 1, aborted, status)) { atomicExch(status, 152); *aborted = 1; break; }
                tc_fence_after_sync();
                const int part = t % splits;
                const int kb_begin = (int)((long long)part * num_kb / splits), kb_end = (int)((long long)(part + 1) * num_kb / splits);
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    if (!wait_or_abort_grid(&full[s], (it / PAIR_STAGES) & 1, aborted, status)) { atomicExch(status, 153); *aborted = 1; break; }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(smem + s * PAIR_STAGE);
                    const uint64_t da = smem_desc_sw128(a_addr);
                    const uint64_t db = smem_desc_sw128(a_addr + BM * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_bf16_pair(tmem_base + (uint32_t)(buf * PAIR_BN), da + 2 * k, db + 2 * k, idesc, kb != kb_begin || k != 0);
                    mma_commit_pair(&empty[s], 3);
                }
                mma_commit_pair(&acc_full[buf], 3);
            }
        }
    } else {
        // a warp reads the quarter of the TMEM lanes that its number allows (warp % 4) and its share of the columns
        const int quad = warp & 3, half = (warp - 2) >> 2;
        const int r = quad * 32 + lane;
        constexpr int HALF_CHUNKS = PAIR_BN / 32 / (PAIR_EPILOGUE_THREADS / 128);      // chunks of 32 columns per warp
        const bool vec_ok = ep.c_dtype == QS_BF16 && (ep.ldc % 8) == 0 && ((uintptr_t)ep.C % 16) == 0 &&
                            (!ep.res1 || ((ep.ldr % 8) == 0 && ((uintptr_t)ep.res1 % 16) == 0)) &&
                            (!ep.res2 || ((uintptr_t)ep.res2 % 16) == 0);
        const uint32_t leader_acc_empty[2] = {map_to_cta(&acc_empty[0], 0), map_to_cta(&acc_empty[1], 0)};
        grid_dep_wait();                                  // residuals, outputs and the workspace belong to earlier kernels until now
        int i = 0;
        for (int t = pair; t < total_tiles; t += n_pairs_grid, ++i) {
            const int buf = i & 1;
            const int tile = t / splits, part = t - tile * splits;
            int tm, tn;
            pair_tile_coords(tile, m_pairs, n_tiles, gm, tm, tn);
            const int m = tm * 2 * BM + (int)rank * BM + r, n0 = tn * PAIR_BN;
            // The tile's bias goes to shared memory once, before the wait for the sums: read per group of
            // columns from global memory it cost every thread 32 round trips in a row (a warp is alone on
            // its scheduler here, and loads do not move across the stores between them): 9 of the 21 us that
            // a 256 x 256 tile's epilogue took.
            if (*aborted) break;                                         // a thread that gave up a wait meets no barrier again
            if (ep.bias) {
                asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_THREADS) : "memory");            // the previous tile's readers are done
                for (int j = threadIdx.x - 64; j < PAIR_BN; j += PAIR_EPILOGUE_THREADS)
                    s_bias[j] = n0 + j < ep.N ? load_as_f32(ep.bias, ep.bias_dtype, n0 + j) : 0.f;
                asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_THREADS) : "memory");
            }
            if (!wait_or_abort_grid(&acc_full[buf], (i >> 1) & 1, aborted, status)) { atomicExch(status, 154); *aborted = 1; break; }
            tc_fence_after_sync();
            // this thread's pieces of the residuals for 32 columns, asked for before the sums are waited for
            uint4 pre1[4], pre2[4];
            auto prefetch = [&](int c) {
                const int nc = n0 + c * 32;
                if (m >= ep.M || !(vec_ok && nc + 32 <= ep.N)) return;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    if (ep.res1) pre1[g] = *reinterpret_cast<const uint4*>(ep.res1 + (size_t)m * ep.ldr + nc + g * 8);
                    if (ep.res2) pre2[g] = *reinterpret_cast<const uint4*>(ep.res2 + (size_t)m * ep.ldr + nc + g * 8);
                }
            };
            // bias, activation, residuals and the store of 32 columns of this thread's row
            auto finish = [&](int c, const uint32_t (&raw)[32]) {
                const int nc = n0 + c * 32;
                if (m >= ep.M || nc >= ep.N) return;
                if (vec_ok && nc + 32 <= ep.N) {
                    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(ep.C) + (size_t)m * ep.ldc + nc;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float v[8], bv[8];
                        if (ep.bias) {
                            const float4 b0 = *reinterpret_cast<const float4*>(s_bias + c * 32 + g * 8);
                            const float4 b1 = *reinterpret_cast<const float4*>(s_bias + c * 32 + g * 8 + 4);
                            bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
                            bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float x = __uint_as_float(raw[g * 8 + j]);
                            if (ep.bias) x += bv[j];
                            v[j] = apply_activation_fast(x, ep.act);
                        }
                        if (ep.res1) {
                            const uint4 rr = pre1[g];
                            const uint32_t w[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) { v[2 * j] += __uint_as_float(w[j] << 16); v[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u); }
                        }
                        if (ep.res2) {
                            const uint4 rr = pre2[g];
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
            };
            if (splits == 1) {
#pragma unroll 1
                for (int c = half * HALF_CHUNKS; c < (half + 1) * HALF_CHUNKS; ++c) {
                    uint32_t raw[32];
                    prefetch(c);
                    tmem_load_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * PAIR_BN + c * 32), raw);
                    tmem_load_wait();
                    finish(c, raw);
                }
                tc_fence_before_sync();
                mbar_arrive_cluster(leader_acc_empty[buf]);   // the leader's MMA warp waits for both CTAs' epilogues
            } else {
                // This CTA's 128 rows of the part's sums go to the workspace ([column][row]: a warp's stores are
                // contiguous); a counter per (tile, CTA of the pair) tells the last part to arrive, which adds the
                // parts in the order of their k-ranges and finishes the tile.  Nobody waits for anybody.
                float* mine = ws + ((size_t)t * 2 + rank) * BM * PAIR_BN;
#pragma unroll 1
                for (int c = half * HALF_CHUNKS; c < (half + 1) * HALF_CHUNKS; ++c) {
                    uint32_t raw[32];
                    tmem_load_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * PAIR_BN + c * 32), raw);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) mine[(size_t)(c * 32 + j) * BM + r] = __uint_as_float(raw[j]);
                }
                tc_fence_before_sync();
                mbar_arrive_cluster(leader_acc_empty[buf]);
                __threadfence();
                if (*aborted) break;
                asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_THREADS) : "memory");
                if (threadIdx.x == 64) {
                    const int prev = atomicAdd(&counters[tile * 2 + (int)rank], 1);
                    const bool last = prev == splits - 1;
                    *last_flag = last ? 1u : 0u;
                    if (last) counters[tile * 2 + (int)rank] = 0;     // ready for the next launch
                }
                asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_THREADS) : "memory");
                if (*last_flag) {
                    __threadfence();
                    const float* first = ws + ((size_t)(tile * splits) * 2 + rank) * BM * PAIR_BN;
#pragma unroll 1
                    for (int c = half * HALF_CHUNKS; c < (half + 1) * HALF_CHUNKS; ++c) {
                        float v[32];
                        prefetch(c);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0.f;
                        for (int p = 0; p < splits; ++p) {
                            const float* src = first + (size_t)p * 2 * BM * PAIR_BN;
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += __ldcg(&src[(size_t)(c * 32 + j) * BM + r]);
                        }
                        uint32_t raw[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(v[j]);
                        finish(c, raw);
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(PAIR_EPILOGUE_THREADS) : "memory");        // last_flag is read by all before it is reused
                (void)part;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();                                   // nobody leaves while the other may still signal it
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ----------------------------------------------------------------------------- stream-K kernel (few tokens)


// The CTA that holds work unit u when U units are dealt to G CTAs as [c U / G, (c + 1) U / G).
__device__ __forceinline__ int owner_of(long long u, long long U, int G) { return (int)(((u + 1) * G - 1) / U); }

// Decode-sized products (at most 64 tokens) are bound by the bytes of W.  Rows of W sit on the MMA's M
// side (tiles of 128 output features), the tokens on its N side (BN = 16, 32 or 64).  The work - every
// (tile, 64-wide k-block) pair, tile-major - is dealt in equal contiguous shares to gridDim.x CTAs, each
// streaming its share through one uninterrupted TMA ring that fills the SM's shared memory.  When the
// host picks gridDim.x = tiles, a share is exactly one tile and no partial sums exist.  A share may begin and end inside a tile: such partial sums go to a workspace slot of the
// CTA, an arrival counter per tile tells the last contributor, and that CTA adds the partial tiles in
// ascending k (ascending CTA) order and runs the epilogue.  No CTA ever waits for another.  The dealing
// depends on N, K and the device only, so a token's result does not depend on its batch.
constexpr int MAX_STREAM_STAGES = 40;
constexpr int STREAM_PAD = BM * BK * 2;          // the MMA always reads 128 rows from a slot: room behind the last one

template <int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                      const Epilogue ep, const int K, const int tiles, const int tile_rows, const int STAGES,
                      float* __restrict__ ws, int32_t* __restrict__ counters, int32_t* __restrict__ status) {
    // A tile is `tile_rows` (a multiple of 8, at most 128) output features high: narrow or uneven N is cut
    // into as many equal tiles as there are SMs.  The MMA still spans 128 rows; rows past tile_rows hold
    // whatever lies behind the slot and are never stored.
    const int STAGE = tile_rows * BK * 2 + BN * BK * 2;
    constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr int CH = 16;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(base);
    uint64_t* empty = full + MAX_STREAM_STAGES;
    uint64_t* acc_full = empty + MAX_STREAM_STAGES;   // [2]
    uint64_t* acc_empty = acc_full + 2;               // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* aborted = tmem_slot + 1;
    volatile uint32_t* last_flag = tmem_slot + 2;
    uint8_t* smem = base + 1024;                      // the ring of stages

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (K + BK - 1) / BK;
    const long long U = (long long)tiles * total_kb;
    const int G = gridDim.x, cta = blockIdx.x;
    const long long u_begin = (long long)cta * U / G, u_end = (long long)(cta + 1) * U / G;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 128); }
        *aborted = 0;
        mbar_fence_init();
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    grid_dep_launch();                                // the next kernel may be scheduled as CTAs of this one leave

    // The loops of the two single threads carry their tile, k-block, stage and phase along: a division
    // in a lone thread's dependent chain costs as much as the copy it is about to start.
    const int tile_begin = (int)(u_begin / total_kb), kb_begin = (int)(u_begin - (long long)tile_begin * total_kb);
    const int count = (int)(u_end - u_begin);

    if (warp == 0) {
        if (elect_one()) {
            // The weights are written by no kernel: the ring is filled with tiles of W right away, while the
            // previous kernel may still be running; the tokens' tiles follow once it has completed.
            const int ahead = min(STAGES, count);
            int tile = tile_begin, kb = kb_begin;
            for (int i = 0; i < ahead; ++i) {
                mbar_expect_tx(&full[i], STAGE);
                tma_load_2d(smem + i * STAGE, &map_w, &full[i], kb * BK, tile * tile_rows);
                if (++kb == total_kb) { kb = 0; ++tile; }
            }
            grid_dep_wait();
            kb = kb_begin;
            for (int i = 0; i < ahead; ++i) {
                tma_load_2d(smem + i * STAGE + tile_rows * BK * 2, &map_a, &full[i], kb * BK, 0);
                if (++kb == total_kb) kb = 0;
            }
            int s = ahead == STAGES ? 0 : ahead;
            uint32_t parity = ahead == STAGES ? 0u : 1u;      // the phase of empty[s] that frees the slot
            for (int i = ahead; i < count; ++i) {
                if (!wait_or_abort(&empty[s], parity, aborted)) { atomicExch(status, 131); *aborted = 1; break; }
                uint8_t* st = smem + s * STAGE;
                mbar_expect_tx(&full[s], STAGE);
                tma_load_2d(st, &map_w, &full[s], kb * BK, tile * tile_rows);
                tma_load_2d(st + tile_rows * BK * 2, &map_a, &full[s], kb * BK, 0);
                if (++kb == total_kb) { kb = 0; ++tile; }
                if (++s == STAGES) { s = 0; parity ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
            int s = 0, kb0 = kb_begin, left = count, seg = 0;
            uint32_t parity = 0;
            for (; left > 0; ++seg) {
                const int n = min(total_kb - kb0, left);
                const int buf = seg & 1;
                if (!wait_or_abort(&acc_empty[buf], ((seg >> 1) & 1) ^ 1, aborted)) { atomicExch(status, 132); *aborted = 1; break; }
                tc_fence_after_sync();
                bool ok = true;
                for (int kb = 0; kb < n; ++kb) {
                    if (!wait_or_abort(&full[s], parity, aborted)) { atomicExch(status, 133); *aborted = 1; ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t w_addr = smem_u32(smem + s * STAGE);
                    const uint64_t dw = smem_desc_sw128(w_addr);
                    const uint64_t da = smem_desc_sw128(w_addr + tile_rows * BK * 2);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_bf16(tmem_base + (uint32_t)(buf * BN), dw + 2 * k, da + 2 * k, idesc, (kb | k) != 0);
                    mma_commit(&empty[s]);
                    if (++s == STAGES) { s = 0; parity ^= 1u; }
                }
                mma_commit(&acc_full[buf]);
                if (!ok) break;
                left -= n;
                kb0 = 0;
            }
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;                   // TMEM lane = output feature within the tile
        grid_dep_wait();                                  // residuals, outputs and the workspace belong to earlier kernels until now
        // 16-byte stores and residual loads need features in whole groups of eight and aligned rows
        const bool vec_ok = (ep.N % 8) == 0 && (ep.ldc % 8) == 0 &&
                            ((uintptr_t)ep.C % (ep.c_dtype == QS_BF16 ? 16 : 32)) == 0 &&
                            (!ep.res1 || ((ep.ldr % 8) == 0 && ((uintptr_t)ep.res1 % 16) == 0)) &&
                            (!ep.res2 || ((ep.ldr % 8) == 0 && ((uintptr_t)ep.res2 % 16) == 0));
        int seg = 0, tile = tile_begin, kb0 = kb_begin, left = count;
        for (; left > 0; ++seg, ++tile, kb0 = 0) {
            const int n = min(total_kb - kb0, left);
            left -= n;
            const int buf = seg & 1;
            const int feat = r < tile_rows ? tile * tile_rows + r : ep.N;       // rows past the tile's height are not stored
            // What the epilogue reads besides the sums is fetched before the wait for them, so that its way from
            // memory is not the kernel's tail: the bias and, with at most 16 tokens, the residuals' pieces.
            const float bias_v = (feat < ep.N && ep.bias) ? load_as_f32(ep.bias, ep.bias_dtype, feat) : 0.f;
            const int sub = lane & 7;
            const int group_row = r - sub;                                    // the group's first TMEM lane
            const int group_feat = tile * tile_rows + group_row;
            const bool group_ok = group_row < tile_rows && group_feat < ep.N;  // all eight or none (multiples of 8)
            constexpr bool EARLY_RES = BN == CH;
            uint4 early1[EARLY_RES ? CH / 8 : 1], early2[EARLY_RES ? CH / 8 : 1];
            if (EARLY_RES && vec_ok && group_ok) {
#pragma unroll
                for (int blk = 0; blk < CH / 8; ++blk) {
                    const int m = blk * 8 + sub;
                    if (m >= ep.M) continue;
                    if (ep.res1) early1[blk] = *reinterpret_cast<const uint4*>(ep.res1 + (size_t)m * ep.ldr + group_feat);
                    if (ep.res2) early2[blk] = *reinterpret_cast<const uint4*>(ep.res2 + (size_t)m * ep.ldr + group_feat);
                }
            }
            if (!wait_or_abort(&acc_full[buf], (seg >> 1) & 1, aborted)) { atomicExch(status, 134); *aborted = 1; break; }
            tc_fence_after_sync();
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
            auto load_acc = [&](int c, float (&v)[CH]) {
                uint32_t raw[CH];
                tmem_load_32x16(tacc + c * CH, raw);
                tmem_load_wait();
#pragma unroll
                for (int j = 0; j < CH; ++j) v[j] = __uint_as_float(raw[j]);
            };
            // This thread holds one output feature for CH tokens.  A warp's store of one token is 64 bytes of
            // 2-byte elements, and such stores cost about 200 cycles each (86 with 4-byte elements), one after the
            // other: 64 tokens took 13,000 cycles.  So, where the layout allows 16-byte stores, groups of eight
            // lanes transpose 8 x 8 blocks by shuffles: a lane then holds eight neighbouring features of one
            // token and stores them at once.  Bias and activation come before the transpose (they go by
            // feature), residuals and the one rounding after it.
            auto emit = [&](int c, const float (&v)[CH]) {
                const int m0 = c * CH;
                if (vec_ok) {
                    float y[CH];
#pragma unroll
                    for (int j = 0; j < CH; ++j) y[j] = apply_activation_fast(v[j] + bias_v, ep.act);
#pragma unroll
                    for (int blk = 0; blk < CH / 8; ++blk) {
#pragma unroll
                        for (int s = 4; s >= 1; s >>= 1) {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                if (i & s) continue;
                                float& lo = y[blk * 8 + i];
                                float& hi = y[blk * 8 + (i | s)];
                                const float got = __shfl_xor_sync(0xffffffffu, (lane & s) ? lo : hi, s);
                                if (lane & s) lo = got; else hi = got;
                            }
                        }
                        const int m = m0 + blk * 8 + sub;                      // y[blk * 8 + i] = feature group_feat + i of token m
                        if (!group_ok || m >= ep.M) continue;
                        float x[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) x[i] = y[blk * 8 + i];
                        if (ep.res1) {
                            const uint4 rr = EARLY_RES ? early1[EARLY_RES ? blk : 0]
                                                       : *reinterpret_cast<const uint4*>(ep.res1 + (size_t)m * ep.ldr + group_feat);
                            const uint32_t w4[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) { x[2 * i] += __uint_as_float(w4[i] << 16); x[2 * i + 1] += __uint_as_float(w4[i] & 0xffff0000u); }
                        }
                        if (ep.res2) {
                            const uint4 rr = EARLY_RES ? early2[EARLY_RES ? blk : 0]
                                                       : *reinterpret_cast<const uint4*>(ep.res2 + (size_t)m * ep.ldr + group_feat);
                            const uint32_t w4[4] = {rr.x, rr.y, rr.z, rr.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) { x[2 * i] += __uint_as_float(w4[i] << 16); x[2 * i + 1] += __uint_as_float(w4[i] & 0xffff0000u); }
                        }
                        if (ep.c_dtype == QS_BF16) {
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const __nv_bfloat162 pb = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
                                o[i] = *reinterpret_cast<const uint32_t*>(&pb);
                            }
                            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(ep.C) + (size_t)m * ep.ldc + group_feat) =
                                make_uint4(o[0], o[1], o[2], o[3]);
                        } else {
                            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(ep.C) + (size_t)m * ep.ldc + group_feat);
                            dst[0] = make_float4(x[0], x[1], x[2], x[3]);
                            dst[1] = make_float4(x[4], x[5], x[6], x[7]);
                        }
                    }
                    return;
                }
                if (feat >= ep.N) return;
                const __nv_bfloat16* r1 = ep.res1 ? ep.res1 + (size_t)m0 * ep.ldr + feat : nullptr;
                const __nv_bfloat16* r2 = ep.res2 ? ep.res2 + (size_t)m0 * ep.ldr + feat : nullptr;
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    if (m0 + j < ep.M) {
                        float x = apply_activation_fast(v[j] + bias_v, ep.act);
                        if (r1) x += __bfloat162float(r1[(size_t)j * ep.ldr]);
                        if (r2) x += __bfloat162float(r2[(size_t)j * ep.ldr]);
                        store_from_f32(ep.C, ep.c_dtype, (size_t)(m0 + j) * ep.ldc + feat, x);
                    }
                }
            };
            if (n == total_kb) {                          // the whole tile was accumulated here
#pragma unroll 1
                for (int c = 0; c < BN / CH; ++c) {
                    float v[CH];
                    load_acc(c, v);
                    emit(c, v);
                }
            } else {
                // a CTA has at most two partial tiles: the one its share begins in (slot 0) and the one it ends in (slot 1)
                float* mine = ws + ((size_t)cta * 2 + (seg == 0 ? 0 : 1)) * BN * BM;
#pragma unroll 1
                for (int c = 0; c < BN / CH; ++c) {
                    float pv[CH];
                    load_acc(c, pv);
#pragma unroll
                    for (int j = 0; j < CH; ++j)
                        if (r < tile_rows) mine[(size_t)(c * CH + j) * BM + r] = pv[j];
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int c_first = owner_of((long long)tile * total_kb, U, G);
                const int c_last = owner_of((long long)(tile + 1) * total_kb - 1, U, G);
                if (threadIdx.x == 64) {
                    const int prev = atomicAdd(&counters[tile], 1);
                    const bool last = prev == c_last - c_first;
                    *last_flag = last ? 1u : 0u;
                    if (last) counters[tile] = 0;         // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
#pragma unroll 1
                    for (int c = 0; c < BN / CH; ++c) {
                        float v[CH];
#pragma unroll
                        for (int j = 0; j < CH; ++j) v[j] = 0.f;
                        for (int cc = c_first; cc <= c_last && r < tile_rows; ++cc) {
                            const int first_tile = (int)(((long long)cc * U / G) / total_kb);
                            const float* part = ws + ((size_t)cc * 2 + (first_tile == tile ? 0 : 1)) * BN * BM;
#pragma unroll
                            for (int j = 0; j < CH; ++j) v[j] += __ldcg(&part[(size_t)(c * CH + j) * BM + r]);
                        }
                        emit(c, v);
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");        // last_flag is read by all before it is reused
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

template <int BN>
int launch_stream(const void* W, long long ldw, const CUtensorMap& ma, const Epilogue& ep, int N, int K, float* ws,
                  long long ws_floats, int32_t* counters, int n_counters, int32_t* status, int smem_kb, cudaStream_t stream) {
    static bool configured = false;
    static int sm_count = 0;
    constexpr int SMEM_MAX = 224 * 1024;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_stream_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX);
        int dev = 0;
        if (e == cudaSuccess) e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gemm_tc: set-up of the stream-K kernel failed: %s",
                                             cudaGetErrorString(e));
        configured = true;
    }
    // One CTA per SM with a ring that fills its shared memory.  N is cut into tiles of equal height (a
    // multiple of 8 rows, at most 128), as many as fill the SMs an integral number of times, so that every
    // SM streams its share of W.  Tiles lower than about 64 rows pay more per k-block than they move, so a
    // narrow N gets fewer, higher tiles, each cut along K into `splits` equal parts for as many CTAs: they
    // add their partial tiles in the order of their k-ranges (the stream-K path of the kernel).  The dealing
    // depends on N, K and the device only.
    const long long total_kb = (K + BK - 1) / BK;
    const long long waves = ((long long)N + (long long)BM * sm_count - 1) / ((long long)BM * sm_count);
    long long splits = 1;
    if (waves == 1 && ws && counters) {
        splits = (long long)sm_count * 64 / N;
        if (splits > total_kb / MIN_KB_PER_SPLIT) splits = total_kb / MIN_KB_PER_SPLIT;
        if (splits < 1) splits = 1;
    }
    const long long slots = waves * sm_count / splits;           // tiles that run at a time
    long long rows = (N + slots - 1) / slots;
    rows = (rows + 7) / 8 * 8;
    if (rows > BM) rows = BM;
    const long long tiles = (N + rows - 1) / rows;
    long long G = tiles * splits;
    if (splits > 1 && (tiles > n_counters || G * 2 * BN * BM > ws_floats)) G = tiles;
    const int stage = (int)rows * BK * 2 + BN * BK * 2;
    // the caller may bound a CTA's shared memory, so that CTAs of two products (on two streams) share an SM
    const int smem_limit = smem_kb > 0 && smem_kb * 1024 < SMEM_MAX ? smem_kb * 1024 : SMEM_MAX;
    int stages = (smem_limit - 2048 - STREAM_PAD) / stage;
    if (stages < 2) stages = 2;
    if (stages > MAX_STREAM_STAGES) stages = MAX_STREAM_STAGES;
    const int smem = 2048 + stages * stage + STREAM_PAD;
    CUtensorMap mw;
    int rc = tensor_map(&mw, W, N, K, ldw, (int)rows);
    if (rc != QS_OK) return rc;
    cudaError_t e = qs_launch_dependent(gemm_tc_stream_kernel<BN>, dim3((unsigned)G), dim3(THREADS), (size_t)smem, stream,
                                        mw, ma, ep, K, (int)tiles, (int)rows, stages, ws, counters, status);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gemm_tc stream: %s", cudaGetErrorString(e));
    return qs_check_launch("gemm_tc stream");
}

// Fewer tiles than CTA pairs (a few hundred tokens against a narrow N): each tile's k-range is cut into
// equal parts for as many pairs as stand idle, at least 16 k-blocks each; their partial sums meet in the
// workspace (see the kernel).  The cut depends on M, N, K and the device.
long long pair_splits(long long tiles, int max_clusters, int K, int pair_bn, const float* ws, long long ws_floats,
                      const int32_t* counters, int n_counters) {
    if (!ws || !counters || tiles * 2 > max_clusters) return 1;
    long long splits = max_clusters / tiles;

    const long long most = ((K + BK - 1) / BK) / 16;
    if (splits > most) splits = most;
    if (splits > 3) splits = 3;            // measured at 256 x 4096 x 20480: 84, 61, 58, 66, 100 us with 1, 2, 3, 4, 6 parts
    if (splits < 1 || tiles * 2 > n_counters || tiles * splits * 2 * BM * pair_bn > ws_floats) splits = 1;
    return splits;
}

// The CTA-pair kernel as a cluster launch; 0 clusters means this device cannot run it at all.
template <int PAIR_BN>
int pair_max_clusters() {
    static int state = 0;                 // 0 = not probed, 1 = usable, -1 = not usable
    static int max_clusters = 0;
    if (state == 0) {
        state = -1;
        if (cudaFuncSetAttribute(gemm_tc_pair_kernel<PAIR_BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 pair_smem<PAIR_BN>()) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2); cfg.blockDim = dim3(PAIR_THREADS); cfg.dynamicSmemBytes = pair_smem<PAIR_BN>();
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<PAIR_BN>, &cfg) == cudaSuccess && n > 0) { max_clusters = n; state = 1; }
        }
        cudaGetLastError();
    }
    return state == 1 ? max_clusters : 0;
}

template <int PAIR_BN>
int launch_pair(const CUtensorMap& ma, const void* W, long long ldw, const Epilogue& ep, int M, int N, int K, float* ws,
                long long ws_floats, int32_t* counters, int n_counters, int32_t* status, cudaStream_t stream) {
    const int max_clusters = pair_max_clusters<PAIR_BN>();
    CUtensorMap mw;
    int rc = tensor_map(&mw, W, N, K, ldw, PAIR_BN / 2);
    if (rc != QS_OK) return rc;
    const int m_pairs = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + PAIR_BN - 1) / PAIR_BN;
    const long long tiles = (long long)m_pairs * n_tiles;
    const long long splits = pair_splits(tiles, max_clusters, K, PAIR_BN, ws, ws_floats, counters, n_counters);
    const long long total = tiles * splits;
    const int clusters = (int)(total < max_clusters ? total : max_clusters);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters); cfg.blockDim = dim3(PAIR_THREADS); cfg.dynamicSmemBytes = pair_smem<PAIR_BN>(); cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    // Rows of A per group of tiles: 32 MB, about a quarter of L2 (126 MB here), at least one pair of row tiles.
    // Measured with groups of 16, 32 and 64 MB against none: 16,384 tokens 2005 -> 1559 us (x 16384 x 4096), 1661 ->
    // 1234 us (x 12288 x 4096), 2327 -> 2014 us (x 4096 x 20480) at 32 MB; 8,192 tokens 5 to 7 % faster; 4,096
    // tokens the same; at 2,048 tokens the product over K = 20480 was 2 % slower in groups, so up to there
    // the tiles keep the plain order.
    long long gm = ((long long)32 << 20) / ((long long)2 * BM * K * 2);
    if (gm < 1) gm = 1;
    if (gm > m_pairs || m_pairs <= 8) gm = m_pairs;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<PAIR_BN>, ma, mw, ep, K, m_pairs, n_tiles, (int)splits, (int)gm,
                                       ws, counters, status);
    if (e != cudaSuccess) return qs_fail(QS_ERR_INTERNAL, "gemm_tc pair: %s", cudaGetErrorString(e));
    return qs_check_launch("gemm_tc pair");
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

// A: [M, K] bfloat16, row stride lda; W: [N, K] bfloat16, row stride ldw (a matrix, or columns of a wider
// one); C: [M, N] bfloat16 or float32.
// res1/res2: bfloat16 [M, N] with row stride ldr, or null.  status: device int32 that receives a
// non-zero code if a bounded wait inside the kernel ran out.
// ws / counters: scratch for split-K in the weight-streaming arrangement (M <= 128): `ws_floats` floats
// and `n_counters` int32 that are ZERO before the first call (the kernel leaves them zero).  Without
// them (null) the product runs unsplit.  Calls that share the scratch must not overlap on the GPU.
// `smem_kb` > 0 bounds the shared memory of a CTA of the weight-streaming arrangement (M <= 128): with half of
// an SM's each, the CTAs of two products that run on two streams share the SMs instead of taking turns.
QS_API int qs_gemm_tc(void* C, int c_dtype, const void* A, const void* W, const void* bias, int bias_dtype, int act,
                      const void* res1, const void* res2, int M, int N, int K, long long lda, long long ldw,
                      long long ldc, long long ldr, float* ws, long long ws_floats, int32_t* counters, int n_counters,
                      int32_t* status, int smem_kb, cudaStream_t stream) {
    if (M == 0 || N == 0) return QS_OK;
    QS_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    QS_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ldw >= K,
               "gemm_tc: K=%d and the row strides %lld, %lld must be multiples of 8, the matrix's at least K", K, lda, ldw);
    QS_REQUIRE(((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0, "gemm_tc: operands must be 16-byte aligned");
    QS_REQUIRE(c_dtype == QS_F32 || c_dtype == QS_BF16, "gemm_tc: unknown output type %d", c_dtype);
    Epilogue ep{C, c_dtype, ldc, bias, bias_dtype, act, (const __nv_bfloat16*)res1, (const __nv_bfloat16*)res2, ldr, M, N};
    CUtensorMap ma, mw;
    int rc;
    if (M > 128) {
        QS_REQUIRE((M + BM - 1) / BM <= 65535 * 1 && (N + 127) / 128 <= 65535, "gemm_tc: sizes exceed the grid");
        if ((rc = tensor_map(&ma, A, M, K, lda, BM)) != QS_OK) return rc;
        if (M > BM && N > 128) {                     // enough rows for a pair of CTAs: tiles of 256 rows
            const int c256 = pair_max_clusters<256>(), c192 = pair_max_clusters<192>();
            if (c256 > 0) {
                // Tiles 192 wide where the rounds over the CTA pairs then cost less, a narrower tile's lower
                // efficiency (measured: about a tenth) included: 384 tiles of 256 are 6 rounds over 74 pairs, the same
                // matrix in 512 tiles of 192 is 7 rounds of three quarters the length.
                // The cost of a width: rounds of work units over the pairs, times a unit's share of K, times the width.
                const long long m_pairs = (M + 2 * BM - 1) / (2 * BM);
                auto cost = [&](long long width, int pairs) {
                    const long long tiles = m_pairs * ((N + width - 1) / width);
                    const long long splits = pair_splits(tiles, pairs, K, (int)width, ws, ws_floats, counters, n_counters);
                    return (tiles * splits + pairs - 1) / pairs * width * ((K + splits - 1) / splits);
                };
                const long long r256 = cost(256, c256);
                const long long r192 = c192 > 0 ? cost(192, c192) : r256;
                if (r192 * 112 < r256 * 100)
                    return launch_pair<192>(ma, W, ldw, ep, M, N, K, ws, ws_floats, counters, n_counters, status, stream);
                return launch_pair<256>(ma, W, ldw, ep, M, N, K, ws, ws_floats, counters, n_counters, status, stream);
            }
        }
        const int bn = N > 128 ? 256 : 128;
        if ((rc = tensor_map(&mw, W, N, K, ldw, bn)) != QS_OK) return rc;
        if (bn == 256) return launch_persistent<256>(ma, mw, ep, M, N, K, status, stream);
        return launch_persistent<128>(ma, mw, ep, M, N, K, status, stream);
    }
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    if ((rc = tensor_map(&ma, A, M, K, lda, bn)) != QS_OK) return rc;
    if (bn == 16) return launch_stream<16>(W, ldw, ma, ep, N, K, ws, ws_floats, counters, n_counters, status, smem_kb, stream);
    if (bn == 32) return launch_stream<32>(W, ldw, ma, ep, N, K, ws, ws_floats, counters, n_counters, status, smem_kb, stream);
    if (bn == 64) return launch_stream<64>(W, ldw, ma, ep, N, K, ws, ws_floats, counters, n_counters, status, smem_kb, stream);
    return launch_stream<128>(W, ldw, ma, ep, N, K, ws, ws_floats, counters, n_counters, status, smem_kb, stream);
}
