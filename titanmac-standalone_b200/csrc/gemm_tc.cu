// Linear layer on tcgen05: C[M, N] = A[M, K] · W[N, K]ᵀ (+ bias[N]) (+ exact GELU), 16-bit inputs, fp32
// accumulation in tensor memory, 16-bit output.  The layout of torch.nn.functional.linear: activations
// row-major, weight [out_features, in_features] - both operands K-major, no transposes anywhere.
//
// A persistent CTA per SM walks over 128 x BN output tiles (consecutive tiles share their rows of A, so those
// stay in L2 while the weight panels change).  Warp roles:
//   warp 0      TMA producer: A and W tiles of 64 K-elements into a ring of shared-memory stages
//   warp 1      issues the tcgen05.mma of every stage (one elected thread); allocates / frees tensor memory
//   warps 2-9   epilogue: tensor memory -> registers -> bias / GELU -> 16-bit -> shared memory -> TMA store;
//               warp w reads the 32 lanes of its number modulo 4, warps 2-5 the first half of the columns,
//               warps 6-9 the second
// The accumulator is double-buffered in tensor memory (2 x BN columns): the epilogue of a tile runs under the
// matrix products of the next one.  Every mbarrier wait is bounded and reports TMW_ERR_DEVICE_TIMEOUT through
// the device status word.
#include <cuda.h>

#include <cstdio>
#include <mutex>

#include "tc_ptx.cuh"
#include "tmw_common.cuh"

namespace tmw {
namespace {

using namespace ptx;

constexpr int GM = 128;        // rows of an output tile
constexpr int GK = 64;         // K elements per stage: one 128-byte swizzle row
constexpr int kPanel = 32;     // columns per staging panel of the output (64 bytes, 64-byte swizzle)
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = 32 * (2 + kEpiWarps);

template <int BN>
struct GemmSmem {
    static constexpr int kStageA = GM * GK * 2;
    static constexpr int kStageB = BN * GK * 2;
    static constexpr int kStage = kStageA + kStageB;
    static constexpr int kOut = GM * BN * 2;  // staging of one output tile: BN / 32 panels of 128 rows x 64 bytes
    static constexpr int kStages = (232448 - 2048 - kOut) / kStage;
    static constexpr int kBars = kStages * kStage + kOut;  // offset of the barrier area
    static constexpr int kTotal = kBars + 1024 + 1024;     // barriers, alignment slack
    static_assert(kStages >= 3, "pipeline depth");
};

struct GemmParams {
    int m, n, k;
    int epilogue;        // tmw_epilogue
    const void* bias;    // [n] in the dtype of the operands, or nullptr
    int* status;
};

// Exact (erf-based) GELU, 0.5 x (1 + erf(x / sqrt 2)), with erf from the rational approximation 7.1.26 of
// Abramowitz & Stegun (absolute error below 1.5e-7, i.e. fp32 rounding noise against the 16-bit result): one
// reciprocal, one exponential and a degree-5 polynomial instead of the library's branchy erff - the epilogue of
// a 128 x 256 tile evaluates it 32 768 times and must stay shorter than the tile's matrix products.
__device__ __forceinline__ float gelu_erf(float x) {
    const float z = fabsf(x) * 0.70710678118654752f;
    const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    const float erf_abs = 1.0f - poly * t * __expf(-z * z);  // erf(|x| / sqrt 2)
    return 0.5f * x * (1.0f + copysignf(erf_abs, x));
}

template <int BN, bool BF16>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
    using L = GemmSmem<BN>;
    constexpr int S = L::kStages;
    constexpr uint32_t kTmemCols = 512;  // two accumulators of BN <= 256 columns
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* bar_area = smem + L::kBars;
    const uint32_t bar_base = smem_base + L::kBars;
    // barrier slots: full[S] | empty[S] | acc_full[2] | acc_empty[2]
    auto full = [&](int s) -> uint32_t { return bar_base + 8 * s; };
    auto empty = [&](int s) -> uint32_t { return bar_base + 8 * (S + s); };
    auto acc_full = [&](int b) -> uint32_t { return bar_base + 8 * (2 * S + b); };
    auto acc_empty = [&](int b) -> uint32_t { return bar_base + 8 * (2 * S + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_area + 8 * (2 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_area + 8 * (2 * S + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (p.n + BN - 1) / BN, m_tiles = (p.m + GM - 1) / GM;
    const int tiles = n_tiles * m_tiles;
    const int k_blocks = (p.k + GK - 1) / GK;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
        for (int s = 0; s < S; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer ----------------
        int n = 0;  // stages filled so far
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int row0 = (tile / n_tiles) * GM, col0 = (tile % n_tiles) * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++n) {
                const int s = n % S;
                mbar_wait(empty(s), ((n / S) & 1) ^ 1, abort_flag, p.status);
                if (lane == 0) {
                    mbar_expect_tx(full(s), L::kStage);
                    const uint32_t dst = smem_base + s * L::kStage;
                    tma_load_2d(dst, &map_a, full(s), kb * GK, row0);
                    tma_load_2d(dst + L::kStageA, &map_w, full(s), kb * GK, col0);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue ----------------
        const uint32_t idesc = idesc_kmajor(BF16 ? 1u : 0u, BN);
        int n = 0, t = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            mbar_wait(acc_empty(buf), ((t >> 1) & 1) ^ 1, abort_flag, p.status);  // the epilogue has drained it
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++n) {
                const int s = n % S;
                mbar_wait(full(s), (n / S) & 1, abort_flag, p.status);
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t a_desc = kmajor_desc(smem_base + s * L::kStage);
                    const uint64_t b_desc = kmajor_desc(smem_base + s * L::kStage + L::kStageA);
#pragma unroll
                    for (int kk = 0; kk < GK / 16; ++kk)
                        mma_ss(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                    tc_commit(empty(s));  // the stage is free once these products have read it
                    if (kb == k_blocks - 1) tc_commit(acc_full(buf));
                }
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int g = warp & 3;             // lane group of tensor memory this warp may read
        const int half = (warp - 2) >> 2;   // column half
        const int row = g * 32 + lane;      // row of the tile
        constexpr int kPanels = BN / kPanel;
        constexpr int kHalfPanels = (kPanels + 1) / 2;  // panels of the first half (the second gets the rest)
        const int panel0 = half == 0 ? 0 : kHalfPanels;
        const int panel1 = half == 0 ? kHalfPanels : kPanels;
        uint8_t* stage = smem + S * L::kStage;
        const bool epi_leader = warp == 2 && lane == 0;
        int t = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++t) {
            const int buf = t & 1;
            const int row0 = (tile / n_tiles) * GM, col0 = (tile % n_tiles) * BN;
            mbar_wait(acc_full(buf), (t >> 1) & 1, abort_flag, p.status);
            tc_fence_after();
            // the previous tile's store must have read the staging buffer before it is overwritten
            if (epi_leader) tma_store_wait_read();
            named_barrier_sync(1, kEpiWarps * 32);
            const uint32_t t_addr = tmem_base + ((uint32_t)(g * 32) << 16) + buf * BN;
            if (panel0 == panel1 && lane == 0) mbar_arrive(acc_empty(buf));  // a tile of one panel: nothing to read
            for (int pn = panel0; pn < panel1; ++pn) {
                uint32_t acc[32];
                tmem_ld32(t_addr + pn * kPanel, acc);
                tc_wait_ld();
                if (pn == panel1 - 1) {
                    // this warp has read all of its columns: hand the accumulator back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(buf));
                }
                const int col = col0 + pn * kPanel;  // first column of the panel
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
                if (p.bias != nullptr) {
                    // bias of 32 columns: 64 bytes, the same for every row (broadcast loads)
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col + j < p.n) {  // n is a multiple of 8
                            float b8[8];
                            if (BF16) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.bias) + col + j, b8);
                            else load8<__half>(static_cast<const __half*>(p.bias) + col + j, b8);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[j + e] += b8[e];
                        }
                    }
                }
                if (p.epilogue == TMW_EPILOGUE_GELU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
                }
                // 32 columns = 64 bytes = four 16-byte chunks of this row in panel pn (64-byte swizzle)
                uint8_t* prow = stage + pn * (GM * 64) + row * 64;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (BF16) {
                            const __nv_bfloat162 hh = __floats2bfloat162_rn(v[c * 8 + 2 * e], v[c * 8 + 2 * e + 1]);
                            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        } else {
                            const __half2 hh = __floats2half2_rn(v[c * 8 + 2 * e], v[c * 8 + 2 * e + 1]);
                            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        }
                    }
                    *reinterpret_cast<uint4*>(prow + ((c ^ ((row >> 1) & 3)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
            named_barrier_sync(2, kEpiWarps * 32);
            if (epi_leader) {
                for (int pn = 0; pn < kPanels; ++pn)
                    if (col0 + pn * kPanel < p.n)
                        tma_store_2d(&map_c, smem_u32(stage + pn * (GM * 64)), col0 + pn * kPanel, row0);
                tma_store_commit();
            }
        }
        if (epi_leader) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (*abort_flag) {
            // a wait expired in this CTA: give copies and products that may still be in flight time to finish
            const long long t0 = clock64();
            while (clock64() - t0 < 400000) __nanosleep(1000);
        }
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------
// The same product on CTA pairs: two CTAs of a cluster (two SMs) share 256 x BN output tiles.  Each CTA
// loads its 128 rows of A and its BN / 2 rows of W, so a W tile crosses L2 -> SM once per 256 output rows instead
// of once per 128 (the single-CTA kernel is bound by exactly that traffic).  The first CTA of the pair issues
// tcgen05.mma.cta_group::2 for both; each CTA keeps its 128 x BN half of the accumulator in its own tensor
// memory and runs its own epilogue.  Barriers: "full" lives in the first CTA and counts the bytes of both CTAs'
// loads; "empty" and "accumulator full" are arrived on in both CTAs by one commit; "accumulator empty" lives in
// the first CTA and collects the epilogue warps of both.
// ---------------------------------------------------------------------------------
template <int BN>
struct PairSmem {
    static constexpr int kStageA = GM * GK * 2;
    static constexpr int kStageB = (BN / 2) * GK * 2;
    static constexpr int kStage = kStageA + kStageB;
    static constexpr int kOut = GM * BN * 2;
    static constexpr int kStages = (232448 - 2048 - kOut) / kStage;
    static constexpr int kBars = kStages * kStage + kOut;
    static constexpr int kTotal = kBars + 1024 + 1024;
    static_assert(kStages >= 3, "pipeline depth");
    static_assert(kStage % 1024 == 0 && kStageA % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
};

template <int BN, bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
    using L = PairSmem<BN>;
    constexpr int S = L::kStages;
    constexpr uint32_t kTmemCols = 512;
    extern __shared__ uint8_t smem_raw[];
    // the same offsets in both CTAs of the pair (the dynamic shared memory of a kernel starts at the same
    // address in every CTA)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* bar_area = smem + L::kBars;
    const uint32_t bar_base = smem_base + L::kBars;
    auto full = [&](int s) -> uint32_t { return bar_base + 8 * s; };
    auto empty = [&](int s) -> uint32_t { return bar_base + 8 * (S + s); };
    auto acc_full = [&](int b) -> uint32_t { return bar_base + 8 * (2 * S + b); };
    auto acc_empty = [&](int b) -> uint32_t { return bar_base + 8 * (2 * S + 2 + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_area + 8 * (2 * S + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_area + 8 * (2 * S + 4) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: issues the products, 1: partner
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int n_tiles = (p.n + BN - 1) / BN, m_tiles = (p.m + 2 * GM - 1) / (2 * GM);
    const int tiles = n_tiles * m_tiles;
    const int k_blocks = (p.k + GK - 1) / GK;
    // columns a tile multiplies: BN, or for the last tile of a row what is left of N (in steps of 32) - a product
    // over columns that do not exist would cost its full time
    auto n_of = [&](int tile) -> int {
        const int rem = p.n - (tile % n_tiles) * BN;
        return rem >= BN ? BN : (rem + 31) / 32 * 32;
    };

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
        for (int s = 0; s < S; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 2 * kEpiWarps);  // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), kTmemCols);
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the partner's barriers exist before anything is signalled across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- producer (both CTAs) ----------------
        int n = 0;
        for (int tile = pair; tile < tiles; tile += pairs) {
            const int row0 = (tile / n_tiles) * (2 * GM) + (int)rank * GM;
            // each CTA supplies half of the tile's columns (the box is BN / 2 rows; a narrow tile uses its first rows)
            const int col0 = (tile % n_tiles) * BN + (int)rank * (n_of(tile) / 2);
            for (int kb = 0; kb < k_blocks; ++kb, ++n) {
                const int s = n % S;
                mbar_wait(empty(s), ((n / S) & 1) ^ 1, abort_flag, p.status);
                if (lane == 0) {
                    if (rank == 0) mbar_expect_tx(full(s), 2 * L::kStage);  // both CTAs' bytes
                    const uint32_t bar0 = map_to_cta(full(s), 0);
                    const uint32_t dst = smem_base + s * L::kStage;
                    tma_load_2d_pair(dst, &map_a, bar0, kb * GK, row0);
                    tma_load_2d_pair(dst + L::kStageA, &map_w, bar0, kb * GK, col0);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- tensor-core issue (first CTA of the pair only) ----------------
        if (rank == 0) {
            int n = 0, t = 0;
            for (int tile = pair; tile < tiles; tile += pairs, ++t) {
                const int buf = t & 1;
                const uint32_t idesc = idesc_kmajor(BF16 ? 1u : 0u, (uint32_t)n_of(tile), 2 * GM);
                mbar_wait(acc_empty(buf), ((t >> 1) & 1) ^ 1, abort_flag, p.status);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++n) {
                    const int s = n % S;
                    mbar_wait(full(s), (n / S) & 1, abort_flag, p.status);
                    tc_fence_after();
                    if (lane == 0) {
                        const uint64_t a_desc = kmajor_desc(smem_base + s * L::kStage);
                        const uint64_t b_desc = kmajor_desc(smem_base + s * L::kStage + L::kStageA);
#pragma unroll
                        for (int kk = 0; kk < GK / 16; ++kk)
                            mma_ss_pair(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kb | kk) ? 1u : 0u);
                        tc_commit_pair(empty(s));
                        if (kb == k_blocks - 1) tc_commit_pair(acc_full(buf));
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, each its own 128 rows) ----------------
        const int g = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = g * 32 + lane;
        constexpr int kPanels = BN / kPanel;
        uint8_t* stage = smem + S * L::kStage;
        const bool epi_leader = warp == 2 && lane == 0;
        int t = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++t) {
            const int buf = t & 1;
            const int row0 = (tile / n_tiles) * (2 * GM) + (int)rank * GM, col0 = (tile % n_tiles) * BN;
            // the tile's panels of 32 columns, split between the two warps of a lane group
            const int panels = n_of(tile) / kPanel, half_panels = (panels + 1) / 2;
            const int panel0 = half == 0 ? 0 : half_panels;
            const int panel1 = half == 0 ? half_panels : panels;
            mbar_wait(acc_full(buf), (t >> 1) & 1, abort_flag, p.status);
            tc_fence_after();
            if (epi_leader) tma_store_wait_read();
            named_barrier_sync(1, kEpiWarps * 32);
            const uint32_t t_addr = tmem_base + ((uint32_t)(g * 32) << 16) + buf * BN;
            if (panel0 == panel1 && lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty(buf), 0));
            for (int pn = panel0; pn < panel1; ++pn) {
                uint32_t acc[32];
                tmem_ld32(t_addr + pn * kPanel, acc);
                tc_wait_ld();
                if (pn == panel1 - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty(buf), 0));
                }
                const int col = col0 + pn * kPanel;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
                if (p.bias != nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (col + j < p.n) {
                            float b8[8];
                            if (BF16) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.bias) + col + j, b8);
                            else load8<__half>(static_cast<const __half*>(p.bias) + col + j, b8);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[j + e] += b8[e];
                        }
                    }
                }
                if (p.epilogue == TMW_EPILOGUE_GELU) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
                }
                uint8_t* prow = stage + pn * (GM * 64) + row * 64;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (BF16) {
                            const __nv_bfloat162 hh = __floats2bfloat162_rn(v[c * 8 + 2 * e], v[c * 8 + 2 * e + 1]);
                            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        } else {
                            const __half2 hh = __floats2half2_rn(v[c * 8 + 2 * e], v[c * 8 + 2 * e + 1]);
                            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        }
                    }
                    *reinterpret_cast<uint4*>(prow + ((c ^ ((row >> 1) & 3)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
            named_barrier_sync(2, kEpiWarps * 32);
            if (epi_leader && row0 < p.m) {
                for (int pn = 0; pn < kPanels; ++pn)
                    if (col0 + pn * kPanel < p.n)
                        tma_store_2d(&map_c, smem_u32(stage + pn * (GM * 64)), col0 + pn * kPanel, row0);
                tma_store_commit();
            }
        }
        if (epi_leader) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();  // nothing of the partner (its barriers, its shared memory) is touched after this
    if (warp == 1) {
        tc_fence_after();
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 400000) __nanosleep(1000);
        }
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// Map over a row-major [rows, cols] matrix with leading dimension ld (elements): boxes of box_rows x box_cols.
// Encoded maps are kept per host thread, keyed by everything that goes into them.
struct Map2dKey {
    const void* base;
    int64_t ld;
    int32_t dtype, rows, cols, box_rows, box_cols, swizzle;
    bool operator==(const Map2dKey& o) const {
        return base == o.base && ld == o.ld && dtype == o.dtype && rows == o.rows && cols == o.cols &&
               box_rows == o.box_rows && box_cols == o.box_cols && swizzle == o.swizzle;
    }
};
bool make_map_2d(CUtensorMap* map, const void* base, int dtype, int rows, int cols, int64_t ld, int box_rows,
                 int box_cols, CUtensorMapSwizzle swizzle) {
    constexpr int kEntries = 64;
    struct Cache { Map2dKey key[kEntries]; CUtensorMap map[kEntries]; bool used[kEntries] = {false}; int next = 0; };
    static thread_local Cache cache;
    const Map2dKey key{base, ld, dtype, rows, cols, box_rows, box_cols, (int32_t)swizzle};
    for (int i = 0; i < kEntries; ++i)
        if (cache.used[i] && cache.key[i] == key) {
            *map = cache.map[i];
            return true;
        }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUtensorMapDataType dt = dtype == TMW_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char text[96];
        snprintf(text, sizeof(text), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        set_error_text(text);
        return false;
    }
    const int slot = cache.next;
    cache.next = (cache.next + 1) % kEntries;
    cache.key[slot] = key;
    cache.map[slot] = *map;
    cache.used[slot] = true;
    return true;
}

int sm_count() {
    constexpr int kMaxDevices = 64;
    static int cache[kMaxDevices] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

template <int BN>
int launch_gemm(const tmw_linear_desc& d, const void* a, const void* w, const void* bias, void* c, cudaStream_t stream) {
    using L = GemmSmem<BN>;
    CUtensorMap ma, mw, mc;
    if (!make_map_2d(&ma, a, d.dtype, d.m, d.k, d.lda, GM, GK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_2d(&mw, w, d.dtype, d.n, d.k, d.ldw, BN, GK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_2d(&mc, c, d.dtype, d.m, d.n, d.ldc, GM, kPanel, CU_TENSOR_MAP_SWIZZLE_64B))
        return TMW_ERR_CUDA;
    GemmParams p;
    p.m = d.m; p.n = d.n; p.k = d.k;
    p.epilogue = d.epilogue;
    p.bias = bias;
    p.status = device_status_word();
    if (p.status == nullptr) return TMW_ERR_CUDA;
    const int tiles = ((d.m + GM - 1) / GM) * ((d.n + BN - 1) / BN);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    auto run = [&](auto kern) -> int {
        const int rc = allow_shared_memory(reinterpret_cast<const void*>(kern), L::kTotal);
        if (rc != TMW_OK) return rc;
        kern<<<grid, kGemmThreads, L::kTotal, stream>>>(ma, mw, mc, p);
        return TMW_OK;
    };
    const int st = d.dtype == TMW_BF16 ? run(gemm_tc_kernel<BN, true>) : run(gemm_tc_kernel<BN, false>);
    if (st != TMW_OK) return st;
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

// How many CTA pairs of the kernel the device runs at once (asked once per kernel and device).
int max_active_pairs(const void* kern, int smem_bytes) {
    constexpr int kMaxDevices = 64, kMaxKernels = 16;
    struct Entry { const void* kern; int pairs[kMaxDevices]; };
    static std::mutex mutex;
    static Entry table[kMaxKernels] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return sm_count() / 2;
    std::lock_guard<std::mutex> lock(mutex);
    Entry* e = nullptr;
    for (int i = 0; i < kMaxKernels && e == nullptr; ++i) {
        if (table[i].kern == kern) e = &table[i];
        else if (table[i].kern == nullptr) { table[i].kern = kern; e = &table[i]; }
    }
    if (e != nullptr && e->pairs[dev] > 0) return e->pairs[dev];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = sm_count() / 2;
    }
    if (e != nullptr) e->pairs[dev] = n;
    return n;
}

template <int BN>
int launch_gemm_pair(const tmw_linear_desc& d, const void* a, const void* w, const void* bias, void* c,
                     cudaStream_t stream) {
    using L = PairSmem<BN>;
    CUtensorMap ma, mw, mc;
    if (!make_map_2d(&ma, a, d.dtype, d.m, d.k, d.lda, GM, GK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_2d(&mw, w, d.dtype, d.n, d.k, d.ldw, BN / 2, GK, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_map_2d(&mc, c, d.dtype, d.m, d.n, d.ldc, GM, kPanel, CU_TENSOR_MAP_SWIZZLE_64B))
        return TMW_ERR_CUDA;
    GemmParams p;
    p.m = d.m; p.n = d.n; p.k = d.k;
    p.epilogue = d.epilogue;
    p.bias = bias;
    p.status = device_status_word();
    if (p.status == nullptr) return TMW_ERR_CUDA;
    const int tiles = ((d.m + 2 * GM - 1) / (2 * GM)) * ((d.n + BN - 1) / BN);
    auto run = [&](auto kern) -> int {
        const void* fn = reinterpret_cast<const void*>(kern);
        const int rc = allow_shared_memory(fn, L::kTotal);
        if (rc != TMW_OK) return rc;
        const int resident = max_active_pairs(fn, L::kTotal);
        const int pairs = tiles < resident ? tiles : resident;
        kern<<<2 * pairs, kGemmThreads, L::kTotal, stream>>>(ma, mw, mc, p);
        return TMW_OK;
    };
    const int st = d.dtype == TMW_BF16 ? run(gemm_tc_pair_kernel<BN, true>) : run(gemm_tc_pair_kernel<BN, false>);
    if (st != TMW_OK) return st;
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

}  // namespace

int launch_linear(const tmw_linear_desc& d, const void* a, const void* w, const void* bias, void* c, cudaStream_t stream) {
    const int m_tiles = (d.m + GM - 1) / GM;
    if (m_tiles <= 2) {
        // Few rows (a decode step): the weights are streamed once and the work is spread by narrow column tiles -
        // the widest tile that still gives most SMs a tile of their own.
        const int want = sm_count() * 2 / 3;
        auto tiles = [&](int bn) { return m_tiles * ((d.n + bn - 1) / bn); };
        if (tiles(256) >= want) return launch_gemm<256>(d, a, w, bias, c, stream);
        if (tiles(128) >= want) return launch_gemm<128>(d, a, w, bias, c, stream);
        if (tiles(64) >= want) return launch_gemm<64>(d, a, w, bias, c, stream);
        return launch_gemm<32>(d, a, w, bias, c, stream);
    }
    // Many rows: CTA pairs on 256 x 256 tiles, the shape that moves the fewest operand bytes per product.  That
    // stream (L2 -> shared memory) is what bounds the kernel, so the wide tile wins even where the last tile of a
    // row is partly empty: measured at M = 32 896, K = 640 for N = 1920 / 640 with tiles of 256 | 192 | 160 | 128
    // columns: 71.9 | 77.4 | 85.6 | 103.8 us and 31.0 | 33.1 | 33.2 | 39.4 us.
    return launch_gemm_pair<256>(d, a, w, bias, c, stream);
}

}  // namespace tmw
