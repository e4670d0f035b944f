// Backward of the windowed attention core on tcgen05: dQ, dK, dV over the visible pairs only, every matrix
// product on the 5th-generation tensor cores with accumulators AND the 16-bit intermediates (P, dS) in tensor
// memory, tiles staged by TMA.  Whole sequences (q_pos0 = 0, k_pos0 = n_persistent), 16-bit types, head_dim 64
// or 128; the plain windowed mask, or (kernels instantiated with GENERAL) the mask of the block-sparse class.
//
// Same mathematics as the other backward paths of this library (c = scale * log2 e, lse from the forward):
//   S = Q Kᵀ,  P = exp2(S c - lse) o mask,  dP = dO Vᵀ,  D_i = dO_i · O_i,  dS = P o (dP - D)
//   dV = Pᵀ dO,  dK = scale · dSᵀ Q,  dQ = scale · dS K
// and the same split into two launches of ONE kernel template - no atomics, results independent of the schedule:
//   !ROWS_ARE_KEYS : a CTA owns 128 queries and walks over the 64-key tiles of their windows -> dQ   (runs first)
//   ROWS_ARE_KEYS  : a CTA owns 128 keys and walks over the 64-query tiles that can see them  -> dK, dV
// The rows a CTA owns sit on the 128 lanes of tensor memory.  Per (row tile, column tile):
//   X = R1 C1ᵀ and Y = R2 C2ᵀ                (R1,R2 = K,V or Q,dO of the rows;  C1,C2 = Q,dO or K,V of the columns)
//   eight warps, two threads per row, turn X into P and Y into dS (16 columns at a time) and write both back into
//   tensor memory as 16-bit values OVER X and Y,
//   then  acc += Pᵀ-or-dS (from tensor memory) · column tile (from shared memory, read as an MN-major operand).
// Warps: 0 TMA producer (and the columns' statistics), 1 and 2 issue the tcgen05.mma (one elected thread each, each
// its own chain of products; warp 1 allocates tensor memory), 3 idle, 4-11 the element-wise work and the output.
// The first launch leaves every row's (log-sum-exp, D) in scratch memory for the second.  Every mbarrier wait is
// bounded (TMW_ERR_DEVICE_TIMEOUT in the status word).
#include <cuda.h>

#include <cstdio>
#include <mutex>
#include <type_traits>

#include "tc_ptx.cuh"
#include "tmw_common.cuh"

namespace tmw {
namespace {

using namespace ptx;

constexpr int BT = 128;          // rows of a tile (the lanes of tensor memory)
constexpr int kBwdThreads = 384;  // 12 warps: see the roles at the kernel
// Columns per tile and depth of the column-tile ring.  head_dim 64: 64 columns, so that X | Y | accumulators fit
// into 256 tensor-memory columns and TWO CTAs share an SM - the chain of a tile pair (products, hand-over, load
// from tensor memory, exponentials, hand-over, products) is serial inside a CTA, and a second CTA is what fills
// its gaps.  head_dim 128: 128 columns, one CTA per SM (the accumulators alone take 256 columns).
template <int DH>
struct Geo {
    static constexpr int kCW = DH == 64 ? 64 : 128;
    static constexpr int kStages = DH == 64 ? 4 : 2;
    static constexpr int kCtasPerSm = DH == 64 ? 2 : 1;
};

struct BwdParams {
    int rows, window, np;        // L, w, Np
    int dim_order;               // bit i: tensor i (0=q 1=k 2=v 3=o/dO 4=dq 5=dk 6=dv) has its head axis before its row axis
    float scale, scale_log2;
    const void* o;               // for D_i = dO_i . O_i
    const void* d_o;
    long long os[3];             // {batch, head, row} strides of o and d_o, elements
    const float* lse;            // [batch, heads, rows]
    // Scratch memory [batch * heads][2][rows_pad] (fp32; rows_pad a multiple of 128), or nullptr.  The launch whose
    // rows are queries computes every row's D anyway and leaves (lse, D) here; the launch whose rows are keys,
    // run after it, then fetches its column statistics with one 16-byte load per lane instead of reading two
    // rows of O and dO per column.
    float* stats;
    int rows_pad;
    int n_bx, heads, batch;      // row tiles per (batch, head); grid = n_bx * heads * batch
    // The mask of the block-sparse class (kernels instantiated with GENERAL): block > 0 moves the left edge of a
    // query's window in steps of `block` rows (first_visible_pos), and the persistent QUERY rows see every key;
    // lse then comes in two planes, [batch, heads, rows - np] for the sequence rows and, at lse_pers,
    // [batch, heads, np] for the persistent rows.
    int block;
    const float* lse_pers;
    int* status;
};

template <int DH>
struct BwdSmem {
    static constexpr int CW = Geo<DH>::kCW, S = Geo<DH>::kStages;
    static constexpr int kTile = BT * DH * 2;                   // a row tile
    static constexpr int kSub = BT * 128;                       // its 64-column sub-tiles: 128 rows x 128 bytes
    static constexpr int kCTile = CW * DH * 2;                  // a column tile
    static constexpr int kCSub = CW * 128;
    static constexpr int kR1 = 0, kR2 = kTile;                  // row tiles (later: staging of the outputs)
    static constexpr int kC = 2 * kTile;                        // S x (C1 | C2)
    static constexpr int kVec = kC + S * 2 * kCTile;            // per stage and column: lse and D (fp32)
    static constexpr int kBars = kVec + S * 2 * CW * 4;
    static constexpr int kTotal = kBars + 256 + 1024;
};

// barrier slots: R_FULL | C_FULL[4] | C_EMPTY[4] | XY_FULL | PDS_READY | ACC_DONE | V_FULL[4]
enum { BAR_R_FULL = 0, BAR_C_FULL = 1, BAR_C_EMPTY = 5, BAR_XY_FULL = 9, BAR_PDS_READY = 10, BAR_ACC_DONE = 11, BAR_V_FULL = 12,
       BAR_N = 16 };

// D = dO . O of one query row (fp32), straight from global memory (two rows of head_dim 16-bit values)
template <int DH, bool BF16>
__device__ __forceinline__ float delta_of(const BwdParams& p, int batch, int head, int qrow) {
    if (qrow >= p.rows) return 0.f;
    const long long off = (long long)batch * p.os[0] + (long long)head * p.os[1] + (long long)qrow * p.os[2];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < DH; c += 8) {
        float a[8], b[8];
        if (BF16) {
            load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.o) + off + c, a);
            load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.d_o) + off + c, b);
        } else {
            load8<__half>(static_cast<const __half*>(p.o) + off + c, a);
            load8<__half>(static_cast<const __half*>(p.d_o) + off + c, b);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e & 3] = fmaf(a[e], b[e], acc[e & 3]);
    }
    return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

// column tiles [first, first + count) that the rows [r0, r1) of a tile interact with, in two segments
struct ColPlan {
    int a0, n0;  // first segment (tiles that hold persistent rows / all query tiles)
    int a1, n1;  // second segment
};

// last query that sees sequence key k through its window (block > 0: the window's left edge is block-aligned)
__device__ __forceinline__ int last_query_of_key(int k, int np, int w, int block) {
    return block > 0 ? np + ((k - np + w) / block) * block + block - 1 : k + w;
}

// `block` > 0 selects the block-sparse class's mask (then the persistent query rows see every key as well)
template <bool ROWS_ARE_KEYS, int CW>
__device__ __forceinline__ ColPlan col_plan(int r0, int L, int w, int np, int block) {
    ColPlan c = {0, 0, 0, 0};
    const int r1 = min(L, r0 + BT);
    const int n_tiles = (L + CW - 1) / CW;
    const int np_tiles = (np + CW - 1) / CW;
    if (ROWS_ARE_KEYS) {
        if (r0 < np) {  // the tile holds persistent keys: every query sees them
            c.n0 = n_tiles;
            return c;
        }
        if (block > 0) c.n0 = np_tiles;  // the persistent queries see every key
        c.a1 = max(r0 / CW, c.n0);
        c.n1 = max(0, min(L - 1, last_query_of_key(r1 - 1, np, w, block)) / CW - c.a1 + 1);
        return c;
    }
    if (block > 0 && r0 < np) {  // the tile holds persistent queries: they see every key
        c.n0 = n_tiles;
        return c;
    }
    c.n0 = np_tiles;  // persistent keys
    if (r1 > np) {
        const int lo = first_visible_pos(max(r0, np), np, w, block);
        c.a1 = max(lo / CW, np_tiles);
        c.n1 = max(0, (r1 - 1) / CW - c.a1 + 1);
    }
    return c;
}

template <int DH, bool BF16, bool ROWS_ARE_KEYS, bool GENERAL>
__global__ void __launch_bounds__(kBwdThreads, Geo<DH>::kCtasPerSm)
bwd_tc_kernel(const __grid_constant__ CUtensorMap map_r1, const __grid_constant__ CUtensorMap map_r2,
              const __grid_constant__ CUtensorMap map_c1, const __grid_constant__ CUtensorMap map_c2,
              const __grid_constant__ CUtensorMap map_out1, const __grid_constant__ CUtensorMap map_out2,
              const BwdParams p) {
    using L = BwdSmem<DH>;
    constexpr int NSUB = DH / 64;
    constexpr int CW = Geo<DH>::kCW, kColStages = Geo<DH>::kStages;
    constexpr uint32_t kX = 0, kY = CW, kAcc1 = 2 * CW, kAcc2 = 2 * CW + DH;
    constexpr uint32_t kNeed = 2 * CW + (ROWS_ARE_KEYS ? 2 : 1) * DH;
    constexpr uint32_t kTmemCols = kNeed <= 256 ? 256 : 512;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    uint8_t* bar_area = smem + L::kBars;
    const uint32_t bar_base = smem_base + L::kBars;
    auto bar = [&](int slot) -> uint32_t { return bar_base + slot * 8; };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_area + BAR_N * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_area + BAR_N * 8 + 8);
    float* vec = reinterpret_cast<float*>(smem + L::kVec);  // [stage][lse | D][column]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // One-dimensional grid.  The row tile that holds the persistent keys walks over EVERY query tile (all queries
    // see those keys), several times the work of any other tile: those CTAs get the first block indices, so they
    // start first and the short ones fill in around them instead of the long ones forming the tail of the launch.
    int tile_x, head, batch;
    {
        const int n_bh = p.heads * p.batch;
        int id = (int)blockIdx.x, bh;
        if ((ROWS_ARE_KEYS || GENERAL) && p.np > 0 && p.n_bx > 1) {
            if (id < n_bh) { tile_x = 0; bh = id; }
            else { id -= n_bh; tile_x = 1 + id % (p.n_bx - 1); bh = id / (p.n_bx - 1); }
        } else {
            tile_x = id % p.n_bx;
            bh = id / p.n_bx;
        }
        head = bh % p.heads;
        batch = bh / p.heads;
    }
    const int r0 = tile_x * BT;
    const int wblock = GENERAL ? p.block : 0;
    const ColPlan plan = col_plan<ROWS_ARE_KEYS, CW>(r0, p.rows, p.window, p.np, wblock);
    const int n_cols = plan.n0 + plan.n1;
    auto col_tile = [&](int n) -> int { return n < plan.n0 ? plan.a0 + n : plan.a1 + (n - plan.n0); };
    // coordinate order of a tensor map: (dh, rows, heads, batch) or (dh, heads, rows, batch)
    auto coords = [&](int which, int row, int& c1, int& c2) {
        if ((p.dim_order >> which) & 1) { c1 = head; c2 = row; } else { c1 = row; c2 = head; }
    };
    // which tensors play which role
    constexpr int kR1 = ROWS_ARE_KEYS ? 1 : 0, kR2 = ROWS_ARE_KEYS ? 2 : 3;   // K,V | Q,dO
    constexpr int kC1 = ROWS_ARE_KEYS ? 0 : 1, kC2 = ROWS_ARE_KEYS ? 3 : 2;   // Q,dO | K,V
    constexpr int kO1 = ROWS_ARE_KEYS ? 6 : 4, kO2 = 5;                       // dV,dK | dQ

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_r1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_r2) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c2) : "memory");
        mbar_init(bar(BAR_R_FULL), 1);
        for (int s = 0; s < kColStages; ++s) {
            mbar_init(bar(BAR_C_FULL + s), 1);
            mbar_init(bar(BAR_C_EMPTY + s), 2);  // both issuing warps
        }
        for (int s = 0; s < kColStages; ++s) mbar_init(bar(BAR_V_FULL + s), 1);
        mbar_init(bar(BAR_XY_FULL), 2);    // X by one issuing warp, Y by the other
        mbar_init(bar(BAR_PDS_READY), 8);  // the eight element-wise warps
        mbar_init(bar(BAR_ACC_DONE), 2);
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
        if (lane == 0) {
            mbar_expect_tx(bar(BAR_R_FULL), 2 * L::kTile);
            int c1, c2;
            coords(kR1, r0, c1, c2);
            for (int u = 0; u < NSUB; ++u)
                tma_load_4d(smem_base + L::kR1 + u * L::kSub, &map_r1, bar(BAR_R_FULL), u * 64, c1, c2, batch);
            coords(kR2, r0, c1, c2);
            for (int u = 0; u < NSUB; ++u)
                tma_load_4d(smem_base + L::kR2 + u * L::kSub, &map_r2, bar(BAR_R_FULL), u * 64, c1, c2, batch);
        }
        for (int n = 0; n < n_cols; ++n) {
            const int s = n % kColStages;
            mbar_wait(bar(BAR_C_EMPTY + s), ((n / kColStages) & 1) ^ 1, abort_flag, p.status);
            if (lane == 0) {
                mbar_expect_tx(bar(BAR_C_FULL + s), 2 * L::kCTile);
                const uint32_t dst = smem_base + L::kC + s * 2 * L::kCTile;
                const int row = col_tile(n) * CW;
                int c1, c2;
                coords(kC1, row, c1, c2);
                for (int u = 0; u < NSUB; ++u)
                    tma_load_4d(dst + u * L::kCSub, &map_c1, bar(BAR_C_FULL + s), u * 64, c1, c2, batch);
                coords(kC2, row, c1, c2);
                for (int u = 0; u < NSUB; ++u)
                    tma_load_4d(dst + L::kCTile + u * L::kCSub, &map_c2, bar(BAR_C_FULL + s), u * 64, c1, c2, batch);
            }
            if (ROWS_ARE_KEYS) {
                // columns are queries: their log-sum-exp and D = dO . O, a few tiles ahead of the warps that use
                // them (the loads would otherwise sit on those warps' critical path once per column tile)
                float* v_lse = vec + s * 2 * CW;
                const long long bh = (long long)batch * p.heads + head;
                if (p.stats != nullptr) {
                    // [lse | D] of the tile's CW columns: 2 * CW / 4 loads of 16 bytes
                    const float* src = p.stats + bh * 2 * p.rows_pad + col_tile(n) * CW;
                    for (int i = lane; i < 2 * CW / 4; i += 32) {
                        const int half = i / (CW / 4), c4 = i % (CW / 4);
                        *reinterpret_cast<float4*>(v_lse + half * CW + c4 * 4) =
                            *reinterpret_cast<const float4*>(src + (long long)half * p.rows_pad + c4 * 4);
                    }
                } else {
                    for (int i = lane; i < CW; i += 32) {
                        const int qrow = col_tile(n) * CW + i;
                        v_lse[i] = qrow >= p.rows ? 0.f
                                   : !GENERAL ? p.lse[bh * p.rows + qrow]
                                   : qrow >= p.np ? p.lse[bh * (p.rows - p.np) + (qrow - p.np)] : p.lse_pers[bh * p.np + qrow];
                        v_lse[CW + i] = delta_of<DH, BF16>(p, batch, head, qrow);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_V_FULL + s));
            }
            __syncwarp();
        }
    } else if (warp == 1 || warp == 2) {
        // ---------------- tensor-core issue: two warps, each with its own chain of products ----------------
        // warp 1:  X = R1 C1^T,  then (rows are keys)  dV += P^T dO          (P lies over X)
        // warp 2:  Y = R2 C2^T,  then  dK += dS^T Q  or  dQ += dS K           (dS lies over Y)
        // The products of one thread execute in issue order, so each warp's next X / Y overwrites the P / dS that
        // its own earlier product has consumed.  Two issuing threads because one thread feeds the pipe with short
        // products (N = 64, K = 16) at well below the rate the pipe runs them.  (The whole warp runs the loop and
        // computes the operands; one lane issues - a lone lane inside a divergent branch issues markedly slower.)
        const bool leader = lane == 0;
        const bool second = warp == 2;
        const uint32_t fmt = BF16 ? 1u : 0u;
        const uint32_t idesc_xy = idesc_kmajor(fmt, CW);
        const uint32_t idesc_acc = idesc_b_mnmajor(fmt, DH);
        const bool has_acc = second || ROWS_ARE_KEYS;
        // the 16-bit intermediates of 16 columns (one k-step) sit in 8 tensor-memory columns; each half of the
        // column tile keeps its packed values inside its own half (see the element-wise warps)
        auto packed_col = [](int kk) -> uint32_t { return (uint32_t)((kk / (CW / 32)) * (CW / 2) + (kk % (CW / 32)) * 8); };
        mbar_wait(bar(BAR_R_FULL), 0, abort_flag, p.status);
        for (int n = 0; n < n_cols; ++n) {
            const int s = n % kColStages;
            const uint32_t c_addr = smem_base + L::kC + s * 2 * L::kCTile;
            mbar_wait(bar(BAR_C_FULL + s), (n / kColStages) & 1, abort_flag, p.status);
            tc_fence_after();
            // both operands K-major over head_dim
            const uint32_t r_addr = smem_base + (second ? L::kR2 : L::kR1);
            const uint32_t c_tile = c_addr + (second ? L::kCTile : 0);
#pragma unroll
            for (int kk = 0; kk < DH / 16; ++kk) {
                const uint64_t ad = kmajor_desc(r_addr + (kk / 4) * L::kSub + (kk % 4) * 32);
                const uint64_t bd = kmajor_desc(c_tile + (kk / 4) * L::kCSub + (kk % 4) * 32);
                if (leader) mma_ss(tmem_base + (second ? kY : kX), ad, bd, idesc_xy, kk > 0 ? 1u : 0u);
            }
            if (leader) tc_commit(bar(BAR_XY_FULL));
            __syncwarp();
            // (the next column tile has usually landed: seeing it now takes that wait off the path hand-over ->
            // products of this tile -> X / Y of the next)
            if (n + 1 < n_cols)
                mbar_wait(bar(BAR_C_FULL + (n + 1) % kColStages), ((n + 1) / kColStages) & 1, abort_flag, p.status);
            mbar_wait(bar(BAR_PDS_READY), n & 1, abort_flag, p.status);
            tc_fence_after();
            if (has_acc) {
                // A = P or dS from tensor memory, B = the other column tile read MN-major:
                // warp 1: dV += P^T dO (B = C2);  warp 2: dK += dS^T Q  or  dQ += dS K (B = C1)
                const uint32_t a_base = tmem_base + (second ? kY : kX);
                const uint32_t d_acc = tmem_base + ((second && ROWS_ARE_KEYS) ? kAcc2 : kAcc1);
                const uint64_t b0 = mnmajor_desc(second ? c_addr : c_addr + L::kCTile, L::kCSub);
                const uint32_t acc = n > 0 ? 1u : 0u;
#pragma unroll
                for (int kk = 0; kk < CW / 16; ++kk) {
                    if (leader) mma_ts(d_acc, a_base + packed_col(kk), b0 + kk * 128, idesc_acc, kk > 0 ? 1u : acc);
                }
            }
            if (leader) {
                tc_commit(bar(BAR_C_EMPTY + s));
                if (n == n_cols - 1) tc_commit(bar(BAR_ACC_DONE));
            }
            __syncwarp();
        }
    } else if (warp >= 4) {
        // ---------------- element-wise warps: two threads per row of the tile, half of the columns each ----------------
        const int g = warp & 3;                    // lane group of tensor memory this warp may touch
        const int half = (warp - 4) >> 2;          // which half of the column tile (and of the output columns)
        const int row = g * 32 + lane;
        const int tid256 = (warp - 4) * 32 + lane;  // 0 .. 255 among the eight warps
        const int pos_row = r0 + row;              // position of this thread's key (ROWS_ARE_KEYS) or query
        const uint32_t t_row = tmem_base + ((uint32_t)(g * 32) << 16);
        const long long bh = (long long)batch * p.heads + head;
        // log-sum-exp of a query row (GENERAL: the persistent rows have a plane of their own)
        auto lse_of = [&](int q) -> float {
            if (q >= p.rows) return 0.f;
            if (GENERAL) return q >= p.np ? p.lse[bh * (p.rows - p.np) + (q - p.np)] : p.lse_pers[bh * p.np + q];
            return p.lse[bh * p.rows + q];
        };
        constexpr int HC = CW / 2;                 // columns per thread and tile
        const int cbase = half * HC;

        // rows are queries: this thread's own statistics, once
        float lse_own = 0.f, d_own = 0.f;
        if (!ROWS_ARE_KEYS) {
            lse_own = lse_of(pos_row);
            d_own = delta_of<DH, BF16>(p, batch, head, pos_row);
            if (p.stats != nullptr && half == 0) {  // rows beyond the sequence get (0, 0), like the bounds-checked path
                p.stats[bh * 2 * p.rows_pad + pos_row] = lse_own;
                p.stats[bh * 2 * p.rows_pad + p.rows_pad + pos_row] = d_own;
            }
        }

        for (int n = 0; n < n_cols; ++n) {
            const int c0 = col_tile(n) * CW;  // position of column 0
            const float* v_lse = vec + (n % kColStages) * 2 * CW;  // written by the producer warp for this stage
            const float* v_d = v_lse + CW;
            if (ROWS_ARE_KEYS) mbar_wait(bar(BAR_V_FULL + n % kColStages), (n / kColStages) & 1, abort_flag, p.status);
            // every pair of the tile visible?  (then no per-element test)
            const int rlo = r0, rhi = min(p.rows, r0 + BT) - 1, clo = c0, chi = min(p.rows, c0 + CW) - 1;
            bool full;
            if (ROWS_ARE_KEYS)  // rows = keys [rlo, rhi], columns = queries [clo, chi]
                full = r0 + BT <= p.rows && c0 + CW <= p.rows &&
                       (rhi < p.np || (GENERAL && chi < p.np) ||
                        (rlo >= p.np && clo >= p.np && rhi <= clo && chi <= last_query_of_key(rlo, p.np, p.window, wblock)));
            else               // rows = queries, columns = keys
                full = r0 + BT <= p.rows && c0 + CW <= p.rows &&
                       (chi < p.np || (GENERAL && rhi < p.np) ||
                        (clo >= p.np && rlo >= p.np && chi <= rlo && clo >= first_visible_pos(rhi, p.np, p.window, wblock)));

            // Columns of this tile that this thread's row sees: [vlo, vhi] (relative to the tile) and the columns
            // below npc - the persistent keys when the rows are queries, the persistent queries (block-sparse
            // class: they see every key) when the rows are keys.  Two instructions per element.
            int vlo = 1, vhi = 0, npc = 0;
            if (pos_row < p.rows) {
                if (ROWS_ARE_KEYS) {
                    if (GENERAL) npc = p.np - c0;
                    if (pos_row < p.np) { vlo = 0; vhi = p.rows - 1 - c0; }
                    else { vlo = pos_row - c0; vhi = min(last_query_of_key(pos_row, p.np, p.window, wblock), p.rows - 1) - c0; }
                } else {
                    npc = p.np - c0;
                    if (pos_row >= p.np) { vlo = first_visible_pos(pos_row, p.np, p.window, wblock) - c0; vhi = pos_row - c0; }
                    else if (GENERAL) { vlo = 0; vhi = p.rows - 1 - c0; }
                }
            }
            const int vbase = cbase - vlo;                 // column - vlo = vbase + (column - cbase)
            const unsigned vspan = (unsigned)max(vhi - vlo, -1);   // vhi < vlo: empty (0xffffffff would mean everything)
            const bool vnone = vhi < vlo;
            const int pbase = npc - cbase;                 // column < npc  <=>  (column - cbase) < pbase

            mbar_wait(bar(BAR_XY_FULL), n & 1, abort_flag, p.status);
            tc_fence_after();
            // 16 columns at a time.  The body exists twice, with and without the per-element mask, as straight-line
            // code (a run-time test inside it would split it into one basic block per element and serialise the
            // elements' dependency chains).  The 16-bit results go back OVER the fp32 inputs, each thread's inside
            // its own half of the columns: chunk j's 8 packed columns lie in columns this thread has already read.
            auto process = [&](auto masked_tag) {
                constexpr bool MASKED = decltype(masked_tag)::value;
#pragma unroll
                for (int j = 0; j < HC / 16; ++j) {
                    uint32_t x[16], y[16];
                    tmem_ld16(t_row + kX + cbase + j * 16, x);
                    tmem_ld16(t_row + kY + cbase + j * 16, y);
                    tc_wait_ld();
                    uint32_t pp[8], ds[8];
#pragma unroll
                    for (int e4 = 0; e4 < 16; e4 += 4) {
                        float l[4], dd[4];
                        if (ROWS_ARE_KEYS) {  // the columns' statistics, four columns per shared-memory load
                            const float4 l4 = *reinterpret_cast<const float4*>(v_lse + cbase + j * 16 + e4);
                            const float4 d4 = *reinterpret_cast<const float4*>(v_d + cbase + j * 16 + e4);
                            l[0] = l4.x; l[1] = l4.y; l[2] = l4.z; l[3] = l4.w;
                            dd[0] = d4.x; dd[1] = d4.y; dd[2] = d4.z; dd[3] = d4.w;
                        } else {
                            l[0] = l[1] = l[2] = l[3] = lse_own;
                            dd[0] = dd[1] = dd[2] = dd[3] = d_own;
                        }
                        float pv[4], dv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float pr = fast_exp2(fmaf(__uint_as_float(x[e4 + e]), p.scale_log2, -l[e]));
                            const float dsv = pr * (__uint_as_float(y[e4 + e]) - dd[e]);
                            if (MASKED) {
                                const int rel = j * 16 + e4 + e;  // column - cbase, a compile-time constant
                                bool vis = ((unsigned)(vbase + rel) <= vspan) & !vnone;
                                if (!ROWS_ARE_KEYS || GENERAL) vis |= rel < pbase;
                                pv[e] = vis ? pr : 0.f;
                                dv[e] = vis ? dsv : 0.f;
                            } else {
                                pv[e] = pr;
                                dv[e] = dsv;
                            }
                        }
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            if (BF16) {
                                const __nv_bfloat162 a2 = __floats2bfloat162_rn(pv[e], pv[e + 1]);
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(dv[e], dv[e + 1]);
                                pp[(e4 + e) / 2] = *reinterpret_cast<const uint32_t*>(&a2);
                                ds[(e4 + e) / 2] = *reinterpret_cast<const uint32_t*>(&b2);
                            } else {
                                const __half2 a2 = __floats2half2_rn(pv[e], pv[e + 1]);
                                const __half2 b2 = __floats2half2_rn(dv[e], dv[e + 1]);
                                pp[(e4 + e) / 2] = *reinterpret_cast<const uint32_t*>(&a2);
                                ds[(e4 + e) / 2] = *reinterpret_cast<const uint32_t*>(&b2);
                            }
                        }
                    }
                    if (ROWS_ARE_KEYS) tmem_st8(t_row + kX + cbase + j * 8, pp);
                    tmem_st8(t_row + kY + cbase + j * 8, ds);
                }
            };
            // a warp none of whose rows sees any of its columns (rows beyond the diagonal or the window's edge, or the
            // sequence keys of a tile that far queries only reach through the persistent keys) writes zeros unread
            const bool mine_empty = vnone || vhi < cbase || vlo >= cbase + HC;
            const bool nothing = !full && __all_sync(0xffffffffu, mine_empty && ((ROWS_ARE_KEYS && !GENERAL) || pbase <= 0 || pos_row >= p.rows));
            if (nothing) {
                const uint32_t zero[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll
                for (int j = 0; j < HC / 16; ++j) {
                    if (ROWS_ARE_KEYS) tmem_st8(t_row + kX + cbase + j * 8, zero);
                    tmem_st8(t_row + kY + cbase + j * 8, zero);
                }
            } else if (full) {
                process(std::false_type{});
            } else {
                process(std::true_type{});
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BAR_PDS_READY));
        }

        // ---------------- output: accumulators -> 16 bits -> shared memory (swizzled) -> TMA store ----------------
        // (each of a row's two threads takes half of the output columns)
        mbar_wait(bar(BAR_ACC_DONE), 0, abort_flag, p.status);
        tc_fence_after();
        constexpr int kOutputs = ROWS_ARE_KEYS ? 2 : 1;
#pragma unroll
        for (int which = 0; which < kOutputs; ++which) {
            // dV is taken as it is; dK and dQ carry the softmax scale
            const float mul = (ROWS_ARE_KEYS && which == 0) ? 1.0f : p.scale;
            uint8_t* stage = smem + (which == 0 ? L::kR1 : L::kR2);  // the row tiles are no longer needed
#pragma unroll
            for (int c = 0; c < DH / 32; ++c) {
                uint32_t o[16];
                const int col0 = half * (DH / 2) + c * 16;
                tmem_ld16(t_row + (which == 0 ? kAcc1 : kAcc2) + col0, o);
                tc_wait_ld();
#pragma unroll
                for (int g8 = 0; g8 < 2; ++g8) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = __uint_as_float(o[g8 * 8 + 2 * e]) * mul;
                        const float b = __uint_as_float(o[g8 * 8 + 2 * e + 1]) * mul;
                        if (BF16) {
                            const __nv_bfloat162 hh = __floats2bfloat162_rn(a, b);
                            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        } else {
                            const __half2 hh = __floats2half2_rn(a, b);
                            w[e] = *reinterpret_cast<const uint32_t*>(&hh);
                        }
                    }
                    const int col = col0 + g8 * 8;
                    uint8_t* dst = stage + (col / 64) * L::kSub + row * 128 + ((((col % 64) / 8) ^ (row & 7)) * 16);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        fence_proxy_async_smem();
        named_barrier_sync(2, 2 * BT);
        if (tid256 == 0) {
            int c1, c2;
            coords(kO1, r0, c1, c2);
            for (int u = 0; u < NSUB; ++u)
                tma_store_4d(&map_out1, smem_u32(smem + L::kR1 + u * L::kSub), u * 64, c1, c2, batch);
            if (ROWS_ARE_KEYS) {
                coords(kO2, r0, c1, c2);
                for (int u = 0; u < NSUB; ++u)
                    tma_store_4d(&map_out2, smem_u32(smem + L::kR2 + u * L::kSub), u * 64, c1, c2, batch);
            }
            tma_store_commit();
            tma_store_wait_all();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (*abort_flag) {
            const long long t0 = clock64();
            while (clock64() - t0 < 400000) __nanosleep(1000);
        }
        tmem_dealloc(tmem_base, kTmemCols);
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

struct Strides4 {
    int64_t row, head, batch;
    bool heads_first;
    bool ok;  // positive multiples of 16 bytes below 2^40 bytes: what a tensor map accepts
};
Strides4 strides_of(int batch, int heads, int rows, int dh, const int64_t stride[3]) {
    Strides4 m;
    m.row = rows > 1 ? stride[2] : dh;
    m.head = heads > 1 ? stride[1] : m.row * rows;
    const int64_t inner_span = m.head * heads > m.row * rows ? m.head * heads : m.row * rows;
    m.batch = batch > 1 ? stride[0] : inner_span;
    m.heads_first = m.head < m.row;
    const int64_t limit = ((int64_t)1 << 40) / 2;
    m.ok = m.row > 0 && m.head > 0 && m.batch > 0 && m.row < limit && m.head < limit && m.batch < limit &&
           m.row % 8 == 0 && m.head % 8 == 0 && m.batch % 8 == 0;
    return m;
}

// map over a [batch, heads, rows, dh] tensor: boxes of box_rows rows x 64 columns of one (batch, head), 128-byte swizzle
bool make_map4(CUtensorMap* map, const void* base, int dtype, int batch, int heads, int rows, int dh, const Strides4& m,
               int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4];
    dims[0] = (cuuint64_t)dh;
    box[0] = 64;
    if (m.heads_first) {
        dims[1] = (cuuint64_t)heads; strides[0] = (cuuint64_t)m.head * 2; box[1] = 1;
        dims[2] = (cuuint64_t)rows;  strides[1] = (cuuint64_t)m.row * 2;  box[2] = (cuuint32_t)box_rows;
    } else {
        dims[1] = (cuuint64_t)rows;  strides[0] = (cuuint64_t)m.row * 2;  box[1] = (cuuint32_t)box_rows;
        dims[2] = (cuuint64_t)heads; strides[1] = (cuuint64_t)m.head * 2; box[2] = 1;
    }
    dims[3] = (cuuint64_t)batch;
    strides[2] = (cuuint64_t)m.batch * 2;
    box[3] = 1;
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == TMW_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, elem_strides,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char text[96];
        snprintf(text, sizeof(text), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        set_error_text(text);
        return false;
    }
    return true;
}

// Stream-ordered scratch memory comes from a pool of the library's own (one per device, created on first use,
// kept for the life of the process): freed blocks stay in the pool, so a call costs no trip to the driver's
// allocator after the first, and the device's default pool and its settings are left alone.
cudaMemPool_t scratch_pool() {
    constexpr int kMaxDevices = 64;
    static std::mutex mutex;
    static cudaMemPool_t pools[kMaxDevices] = {};
    static bool tried[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if (!tried[dev]) {
        tried[dev] = true;
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) == cudaSuccess) {
            unsigned long long keep = ~0ull;
            (void)cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            pools[dev] = pool;
        } else {
            (void)cudaGetLastError();
        }
    }
    return pools[dev];
}

template <int DH>
int launch_bwd_tc(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o, const void* d_o,
                  const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream, int window_block) {
    using L = BwdSmem<DH>;
    const int B = d.batch, H = d.heads, R = d.q_rows;
    const Strides4 sq = strides_of(B, H, R, DH, d.q_stride), sk = strides_of(B, H, R, DH, d.k_stride);
    const Strides4 sv = strides_of(B, H, R, DH, d.v_stride), so = strides_of(B, H, R, DH, d.o_stride);
    constexpr int CW = Geo<DH>::kCW;
    // row-tile maps (boxes of 128 rows; also the outputs) and column-tile maps (boxes of CW rows)
    CUtensorMap mq, mk, mv, mdo, mdq, mdk, mdv, cq, ck, cv, cdo;
    if (!make_map4(&mq, q, d.dtype, B, H, R, DH, sq, BT) || !make_map4(&mk, k, d.dtype, B, H, R, DH, sk, BT) ||
        !make_map4(&mv, v, d.dtype, B, H, R, DH, sv, BT) || !make_map4(&mdo, d_o, d.dtype, B, H, R, DH, so, BT) ||
        !make_map4(&mdq, dq, d.dtype, B, H, R, DH, sq, BT) || !make_map4(&mdk, dk, d.dtype, B, H, R, DH, sk, BT) ||
        !make_map4(&mdv, dv, d.dtype, B, H, R, DH, sv, BT) || !make_map4(&cq, q, d.dtype, B, H, R, DH, sq, CW) ||
        !make_map4(&ck, k, d.dtype, B, H, R, DH, sk, CW) || !make_map4(&cv, v, d.dtype, B, H, R, DH, sv, CW) ||
        !make_map4(&cdo, d_o, d.dtype, B, H, R, DH, so, CW))
        return TMW_ERR_CUDA;
    BwdParams p;
    p.rows = R; p.window = d.window; p.np = d.n_persistent;
    p.dim_order = (sq.heads_first ? 1 : 0) | (sk.heads_first ? 2 : 0) | (sv.heads_first ? 4 : 0) | (so.heads_first ? 8 : 0) |
                  (sq.heads_first ? 16 : 0) | (sk.heads_first ? 32 : 0) | (sv.heads_first ? 64 : 0);
    p.scale = d.scale != 0.f ? d.scale : 1.0f / sqrtf((float)DH);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.o = o; p.d_o = d_o;
    for (int i = 0; i < 3; ++i) p.os[i] = d.o_stride[i];
    p.lse = lse;
    p.block = window_block;
    p.lse_pers = window_block > 0 ? lse + (size_t)B * H * (R - d.n_persistent) : nullptr;
    p.status = device_status_word();
    if (p.status == nullptr) return TMW_ERR_CUDA;
    // scratch memory for the rows' (lse, D), ordered on the caller's stream; without it the launch whose rows are
    // keys computes D itself
    p.rows_pad = (R + BT - 1) / BT * BT;
    p.stats = nullptr;
    {
        void* mem = nullptr;
        cudaMemPool_t pool = scratch_pool();
        if (pool != nullptr &&
            cudaMallocFromPoolAsync(&mem, (size_t)B * H * 2 * p.rows_pad * sizeof(float), pool, stream) == cudaSuccess)
            p.stats = static_cast<float*>(mem);
        else
            (void)cudaGetLastError();
    }
    p.n_bx = (R + BT - 1) / BT; p.heads = H; p.batch = B;
    const dim3 grid(p.n_bx * H * B, 1, 1);
    auto run = [&](auto kern, const CUtensorMap& r1, const CUtensorMap& r2, const CUtensorMap& c1, const CUtensorMap& c2,
                   const CUtensorMap& o1, const CUtensorMap& o2) -> int {
        const int rc = allow_shared_memory(reinterpret_cast<const void*>(kern), L::kTotal);
        if (rc != TMW_OK) return rc;
        kern<<<grid, kBwdThreads, L::kTotal, stream>>>(r1, r2, c1, c2, o1, o2, p);
        return TMW_OK;
    };
    // dQ first: rows are queries (Q, dO), columns are keys (K, V); it also leaves the rows' statistics
    const bool bf16 = d.dtype == TMW_BF16, general = window_block > 0;
    int st = general ? (bf16 ? run(bwd_tc_kernel<DH, true, false, true>, mq, mdo, ck, cv, mdq, mdq)
                             : run(bwd_tc_kernel<DH, false, false, true>, mq, mdo, ck, cv, mdq, mdq))
                     : (bf16 ? run(bwd_tc_kernel<DH, true, false, false>, mq, mdo, ck, cv, mdq, mdq)
                             : run(bwd_tc_kernel<DH, false, false, false>, mq, mdo, ck, cv, mdq, mdq));
    // dK, dV: rows are keys (K, V), columns are queries (Q, dO)
    if (st == TMW_OK)
        st = general ? (bf16 ? run(bwd_tc_kernel<DH, true, true, true>, mk, mv, cq, cdo, mdv, mdk)
                             : run(bwd_tc_kernel<DH, false, true, true>, mk, mv, cq, cdo, mdv, mdk))
                     : (bf16 ? run(bwd_tc_kernel<DH, true, true, false>, mk, mv, cq, cdo, mdv, mdk)
                             : run(bwd_tc_kernel<DH, false, true, false>, mk, mv, cq, cdo, mdv, mdk));
    const cudaError_t launched = cudaGetLastError();
    if (p.stats != nullptr) (void)cudaFreeAsync(p.stats, stream);
    if (st != TMW_OK) return st;
    TMW_CUDA_TRY(launched);
    return TMW_OK;
}

}  // namespace

// the plain windowed mask over whole sequences, 16-bit types, head_dim 64 or 128, layouts a tensor map can describe
bool prefill_backward_tc_supports(const tmw_prefill_desc& d) {
    if (d.dtype != TMW_BF16 && d.dtype != TMW_F16) return false;
    if (d.head_dim != 64 && d.head_dim != 128) return false;
    if (d.batch > 65535 || d.heads > 65535) return false;
    if ((int64_t)d.q_rows + d.window + 2 * BT >= (int64_t)1 << 29) return false;  // (+ a block size of up to 2^20)
    return strides_of(d.batch, d.heads, d.q_rows, d.head_dim, d.q_stride).ok &&
           strides_of(d.batch, d.heads, d.q_rows, d.head_dim, d.k_stride).ok &&
           strides_of(d.batch, d.heads, d.q_rows, d.head_dim, d.v_stride).ok &&
           strides_of(d.batch, d.heads, d.q_rows, d.head_dim, d.o_stride).ok;
}

int launch_prefill_backward_tc(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o,
                               const void* d_o, const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream,
                               int window_block) {
    return d.head_dim == 64 ? launch_bwd_tc<64>(d, q, k, v, o, d_o, lse, dq, dk, dv, stream, window_block)
                            : launch_bwd_tc<128>(d, q, k, v, o, d_o, lse, dq, dk, dv, stream, window_block);
}

}  // namespace tmw
