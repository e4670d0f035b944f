// Tensor-core prefill kernel for B200: sliding-window attention with persistent prefix
// keys on tcgen05 (5th-generation tensor cores) with accumulators in tensor memory.
//
// One CTA owns 256 consecutive query rows of one (batch, head) as two 128-row query
// tiles.  Its 12 warps have fixed roles:
//   warp  0     TMA producer: Q tiles, then the K tiles of the window
//   warp  1     TMA producer: persistent K/V tile, then the V tiles; allocates / frees tensor memory
//   warp  2     issues the tcgen05.mma of query tile 0 (one elected thread)
//   warp  3     issues the tcgen05.mma of query tile 1
//   warps 4-7   softmax group of query tile 0      (one thread per query row)
//   warps 8-11  softmax group of query tile 1
// (the issuing warps come first so that they are the oldest warps of their schedulers)
// head_dim 64 runs one query tile per CTA and two CTAs per SM instead (8 warps), or - windows of 192 keys and
// more - with TWO threads per score row (12 warps: warps w and w + 4 share the 32 rows of their lane group,
// take 64 of a key tile's 128 columns each and exchange the row maximum and sum through shared memory).
// Key positions are cut into 128-key tiles anchored at (first query position - w), so
// the second query tile always needs the same tiles shifted by one: both tiles share
// every K/V tile that is loaded, and tiles that lie outside a query tile's window are
// never multiplied.  The persistent keys are one extra, always-first tile kept in its
// own shared-memory buffer.
//
// Per (query tile, key tile):  S = Q Kᵀ (fp32, tensor memory)  ->  the softmax group
// reads its row of S, updates the running maximum lazily (the output accumulator in
// tensor memory is only rescaled when the maximum grew by more than 2^8), writes
// P = exp2(S·c - m) as 16-bit values back into tensor memory over S  ->  O += P V with P
// read from tensor memory.  The two query tiles alternate on the tensor pipe, so one
// tile's softmax overlaps the other tile's matrix products.
//
// Every wait on an mbarrier is bounded: on expiry the kernel records
// TMW_ERR_DEVICE_TIMEOUT in the device status word, stops waiting anywhere and runs
// to completion (with meaningless output) so that tensor memory is freed and the
// context stays usable.
#include <cuda.h>

#include <cstdio>
#include <mutex>
#include <type_traits>

#include "tmw_common.cuh"

namespace tmw {
namespace {

// Threads and register budget per query tiles of a CTA.  Two tiles: 384 threads launched with 168 registers
// (one CTA per SM).  One tile: 256 threads launched with 128 registers (two CTAs per SM).  The four
// producer / issuing warps shrink to kRegsService, the softmax warps grow to kRegsSoftmax; setmaxnreg.inc
// blocks until the registers it asks for have been released INSIDE THE CTA and nothing bounds that wait, so
// the numbers must add up.
template <int TILES, int RS>
struct Budget {
    static_assert(RS == 1 || (RS == 2 && TILES == 1), "two threads per score row: one-tile CTAs only");
    static constexpr int kThreads = 128 + TILES * 128 * RS;
    static constexpr int kCtasPerSm = TILES == 2 ? 1 : 2;
    // one thread per row: 168 | 80 | 208 (two tiles), 128 | 56 | 200 (one tile);  two threads per row: 80 | 40 | 96
    static constexpr int kRegsLaunch = RS == 2 ? 80 : TILES == 2 ? 168 : 128;
    static constexpr int kRegsService = RS == 2 ? 40 : TILES == 2 ? 80 : 56;
    static constexpr int kRegsSoftmax = RS == 2 ? 96 : TILES == 2 ? 208 : 200;
    static_assert(kThreads * kRegsLaunch <= 65536 / kCtasPerSm, "register file");
    static_assert(128 * (kRegsLaunch - kRegsService) >= TILES * 128 * RS * (kRegsSoftmax - kRegsLaunch),
                  "setmaxnreg: the issuing warps must release what the softmax warps request");
};
constexpr int BM = 128;  // query rows per tile
constexpr int BN = 128;  // keys per tile
constexpr long long kWaitLimitCycles = 2000000000LL;  // about one second
// The two softmax groups of a two-tile CTA take turns with their exponentials for head_dim 128 (measured: +10 %
// at head_dim 128 / window 1024, -6 % at head_dim 64 / window 512, where it is off).
template <int DH>
struct Alternate { static constexpr bool value = DH == 128; };

// tensor-memory columns (32-bit each, 128 lanes): S0 | S1 | O0 | O1; P aliases S
// head_dim 64 : S0 0 | S1 128 | P0 256 | P1 320 | O0 384 | O1 448   (P has its own columns: the next QK
//                may overwrite S while the softmax group still turns the previous S into P)
// head_dim 128: S0 0 | S1 128 | O0 256 | O1 384                      (P is written over S)
// one query tile per CTA (256 columns, two CTAs share the SM's 512):
// head_dim 64 : S 0 | P 128 | O 192        head_dim 128: S 0 | O 128
template <int DH, int TILES>
struct TmemMap {
    static constexpr bool kSplitP = DH == 64;
    static constexpr uint32_t kCols = TILES * 256;
    __host__ __device__ static constexpr uint32_t s(int t) { return t == 0 ? 0u : 128u; }
    __host__ __device__ static constexpr uint32_t p(int t) {
        return TILES == 1 ? (kSplitP ? 128u : 0u) : kSplitP ? (t == 0 ? 256u : 320u) : s(t);
    }
    __host__ __device__ static constexpr uint32_t o(int t) {
        return TILES == 1 ? (kSplitP ? 192u : 128u) : kSplitP ? (t == 0 ? 384u : 448u) : (t == 0 ? 256u : 384u);
    }
};


struct TcParams {
    int q_rows, k_rows, window, np, np_pad, q_pos0, k_pos0;
    int block;        // 0 or the block size of the block-granular window (first_visible_pos)
    int window_plan;  // window + block - 1: the widest window any row can have, used to lay out the key tiles
    int all_keys;     // 1: every query row of the call sees every key row, unmasked
    int dim_order;  // bit i set: tensor i (0=q,1=k,2=v,3=o) has its head axis before its row axis in the map
    float scale_log2;
    int* status;
    float* lse;  // optional [batch, heads, q_rows]: log2 of the row's softmax denominator, in the scaled-by-log2(e) domain
    // Sequence-sharded call whose K/V buffer is filled by other GPUs (tmw_halo_push): key rows [0, np) may be read
    // once *pers_flag >= flag_value, key rows [np, np + halo_rows) once *halo_flag >= flag_value.  nullptr: no wait.
    const int* pers_flag;
    const int* halo_flag;
    int flag_value;
    int halo_rows;
    long long flag_wait_limit;
};

// Bounded wait of a producer warp for a flag that another GPU raises in this GPU's memory after it has written
// rows of the K/V buffer (release at system scope).  The rows are then read by TMA, i.e. through the asynchronous
// proxy, hence the proxy fence after the acquire.  On expiry: TMW_ERR_DEVICE_TIMEOUT in the status word
// (status[1] = -1 marks a flag, not an mbarrier), and nobody in the CTA waits any more.
__device__ __forceinline__ void flag_wait(const int* flag, int value, long long limit, volatile int* abort_flag,
                                          int* status) {
    if ((threadIdx.x & 31) == 0) {
        const long long t0 = clock64();
        for (;;) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v >= value || *abort_flag) break;
            if (clock64() - t0 > limit) {
                *abort_flag = 1;
                if (atomicCAS(status, 0, (int)TMW_ERR_DEVICE_TIMEOUT) == 0) {
                    status[1] = -1;
                    status[2] = (int)(blockIdx.x | (blockIdx.y << 16));
                    status[3] = (int)(blockIdx.z | ((threadIdx.x >> 5) << 16));
                }
                break;
            }
            __nanosleep(100);
        }
        asm volatile("fence.proxy.async;" ::: "memory");
    }
    __syncwarp();
}

// ---------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory; once it is set nobody waits any more.  The first
// wait that expires on the device also records where it was: status[1] = shared-memory offset of the
// barrier and parity, status[2] = blockIdx.x | blockIdx.y << 16, status[3] = blockIdx.z | warp << 16.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                if (atomicCAS(status, 0, (int)TMW_ERR_DEVICE_TIMEOUT) == 0) {
                    status[1] = (int)((bar & 0xffffu) | (parity << 16));
                    status[2] = (int)(blockIdx.x | (blockIdx.y << 16));
                    status[3] = (int)(blockIdx.z | ((threadIdx.x >> 5) << 16));
                }
                return;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two fp32 values in one 64-bit register, for the packed f32x2 arithmetic of sm_100
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}

#define TMW_R8(a, o)                                                                                        \
    "=r"(a[o + 0]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]),        \
        "=r"(a[o + 6]), "=r"(a[o + 7])
#define TMW_I8(a, o)                                                                                        \
    "r"(a[o + 0]), "r"(a[o + 1]), "r"(a[o + 2]), "r"(a[o + 3]), "r"(a[o + 4]), "r"(a[o + 5]), "r"(a[o + 6]), \
        "r"(a[o + 7])

// 32 lanes x 32 consecutive columns: thread t of the warp gets lane (base lane + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : TMW_R8(r, 0), TMW_R8(r, 8), TMW_R8(r, 16), TMW_R8(r, 24)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : TMW_R8(r, 0), TMW_R8(r, 8)
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
        ::"r"(taddr), TMW_I8(r, 0)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), TMW_I8(r, 0), TMW_I8(r, 8)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), TMW_I8(r, 0), TMW_I8(r, 8), TMW_I8(r, 16), TMW_I8(r, 24)
        : "memory");
}

// Shared-memory matrix descriptors (128-byte swizzle, version 1 for sm_100) are built in the kernel as
//   bits [0,14)  start address >> 4       bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4  bits [46,48) version = 1    bits [61,64) layout = 2 (SWIZZLE_128B)

// Instruction descriptor for kind::f16: fp32 accumulate, A K-major; B K-major or MN-major.
//   [4,6) D format (1 = f32)  [7,10) A format  [10,13) B format (0 = f16, 1 = bf16)
//   [15] A major  [16] B major (1 = MN)  [17,23) N >> 3  [24,29) M >> 4
__device__ __forceinline__ uint32_t make_idesc(uint32_t fmt, uint32_t b_mn_major, uint32_t n) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn_major << 16) | ((n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ---------------------------------------------------------------------------------
// Schedule of one CTA, computed identically by every role
// ---------------------------------------------------------------------------------
struct QtPlan {
    int p_lo;      // position of the tile's first query row
    int rows;      // valid query rows (0: tile absent)
    int has_pers;  // 1 if the persistent tile is item 0
    int a;         // first window tile index
    int n_win;     // number of window tiles
    int n_items;   // has_pers + n_win
};

struct CtaPlan {
    int anchor;  // position of key 0 of window tile 0
    QtPlan qt[2];
    int x_begin, x_end;  // window tiles [x_begin, x_end) are loaded
};

__device__ __forceinline__ int floor_div(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }

// `wblock` / `all_keys`: the block-granular window and the unmasked mode; the kernel instantiated for the
// plain windowed mask passes constants, so that none of this costs it an instruction
__device__ __forceinline__ CtaPlan make_plan(const TcParams& p, int block, int tiles, int wblock, bool all_keys) {
    CtaPlan c;
    const int r0 = block * tiles * BM;
    c.anchor = p.q_pos0 + r0 - (wblock > 0 ? p.window_plan : p.window);
    c.x_begin = 1 << 30;
    c.x_end = 0;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        QtPlan& q = c.qt[t];
        q.p_lo = p.q_pos0 + r0 + t * BM;
        q.rows = t < tiles ? max(0, min(BM, p.q_rows - (r0 + t * BM))) : 0;
        q.has_pers = (q.rows > 0 && p.np > 0) ? 1 : 0;
        const int p_hi = q.p_lo + q.rows - 1;
        if (all_keys) {
            c.anchor = p.k_pos0;  // key tile x starts at key row np + x * BN
            q.a = 0;
            q.n_win = q.rows > 0 ? (p.k_rows - p.np + BN - 1) / BN : 0;
            if (q.rows > 0) {
                c.x_begin = 0;
                c.x_end = max(c.x_end, q.n_win);
            }
        } else if (q.rows > 0 && p_hi >= p.np) {
            const int g_lo = first_visible_pos(max(q.p_lo, p.np), p.np, p.window, wblock);
            q.a = floor_div(g_lo - c.anchor, BN);
            q.n_win = floor_div(p_hi - c.anchor, BN) - q.a + 1;
            c.x_begin = min(c.x_begin, q.a);
            c.x_end = max(c.x_end, q.a + q.n_win);
        } else {
            q.a = 0;
            q.n_win = 0;
        }
        q.n_items = q.has_pers + q.n_win;
    }
    if (c.x_end == 0) c.x_begin = 0;
    return c;
}

// ---------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------
template <int DH, int KS, int VS, int TILES>
struct TcSmem {
    static constexpr int kTileBytes = BN * DH * 2;       // one K or V or Q tile
    static constexpr int kSubTileBytes = BN * 128;       // 128 rows x 64 columns of 16-bit
    static constexpr int kQ = 0;                         // TILES tiles
    static constexpr int kK = kQ + TILES * kTileBytes;   // KS tiles
    static constexpr int kV = kK + KS * kTileBytes;      // VS tiles
    static constexpr int kP = kV + VS * kTileBytes;      // persistent K then V: np_pad x DH x 2 bytes each
    // after the tiles: barriers (512 bytes), then the exchange area of rows that two threads share (3 KB)
    static int total_bytes(int np_pad) { return kP + 2 * np_pad * DH * 2 + 4096 + 1024 /*alignment*/; }
};

// barrier slots inside the barrier area
enum BarSlot {
    BAR_Q_FULL = 0,        // [2]
    BAR_KP_FULL = 2,       // persistent K and V
    BAR_S_FULL = 3,        // [2]
    BAR_P_READY = 5,       // [2]
    BAR_O_DONE = 7,        // [2]
    BAR_K_FULL = 9,        // [KS <= 4]
    BAR_K_EMPTY = 13,      // [KS]
    BAR_V_FULL = 17,       // [VS <= 4]
    BAR_V_EMPTY = 21,      // [VS]
    BAR_S_FREE = 25,       // [2] softmax group has S in registers (only when P has its own columns)
    BAR_PV_DONE = 27,      // [2] P V of the previous item has finished (only when P has its own columns)
    BAR_TURN = 29,         // [2] the other softmax group has finished its exponentials (alternation)
    BAR_COUNT = 31
};

// GENERAL = false: the plain windowed mask (every mode parameter a compile-time constant);
// GENERAL = true: block-granular window and / or the unmasked "all keys" mode, read from the parameters.
template <int DH, int KS, int VS, bool BF16, int TILES, bool GENERAL, int RS>
__global__ void __launch_bounds__(Budget<TILES, RS>::kThreads, Budget<TILES, RS>::kCtasPerSm)
prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                  const __grid_constant__ CUtensorMap map_kp, const __grid_constant__ CUtensorMap map_vp,
                  const TcParams p) {
    using L = TcSmem<DH, KS, VS, TILES>;
    constexpr uint32_t kTmemCols = TmemMap<DH, TILES>::kCols;
    constexpr int NSUB = DH / 64;  // 64-column sub-tiles per tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t pers_bytes = (uint32_t)p.np_pad * DH * 2;
    const uint32_t bar_base = smem_base + L::kP + 2 * pers_bytes;
    uint8_t* bar_area = smem + L::kP + 2 * pers_bytes;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_area + BAR_COUNT * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_area + BAR_COUNT * 8 + 8);
    auto bar = [&](int slot) -> uint32_t { return bar_base + slot * 8; };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y, batch = blockIdx.z;
    const int wblock = GENERAL ? p.block : 0;
    const bool all_keys = GENERAL && p.all_keys != 0;
    const CtaPlan plan = make_plan(p, blockIdx.x, TILES, wblock, all_keys);

    if (threadIdx.x == 0) {
        // the tensor maps live in the kernel parameters; fetch them into the descriptor cache early
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kp) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_vp) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_o) : "memory");
        mbar_init(bar(BAR_Q_FULL + 0), 1);
        mbar_init(bar(BAR_Q_FULL + 1), 1);
        mbar_init(bar(BAR_KP_FULL), 1);
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar(BAR_S_FULL + t), 1);
            mbar_init(bar(BAR_P_READY + t), RS * BM / 32);  // one arrival per softmax warp
            mbar_init(bar(BAR_O_DONE + t), 1);
            mbar_init(bar(BAR_S_FREE + t), RS * BM / 32);
            mbar_init(bar(BAR_PV_DONE + t), 1);
            mbar_init(bar(BAR_TURN + t), BM / 32);
        }
        for (int s = 0; s < KS; ++s) {
            mbar_init(bar(BAR_K_FULL + s), 1);
            mbar_init(bar(BAR_K_EMPTY + s), TILES);  // one arrival per issuing warp
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(bar(BAR_V_FULL + s), 1);
            mbar_init(bar(BAR_V_EMPTY + s), TILES);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // coordinate order of each tensor map: (dh, rows, heads, batch) or (dh, heads, rows, batch)
    auto coords = [&](int which, int row, int& c1, int& c2) {
        if ((p.dim_order >> which) & 1) { c1 = head; c2 = row; } else { c1 = row; c2 = head; }
    };

    if (warp < 4) {
        // register budget: see Budget
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Budget<TILES, RS>::kRegsService) : "memory");
        // Every role warp runs its loop with all 32 lanes (so the warp never splits into a running
        // lane and 31 lanes parked at the final barrier); one lane issues the asynchronous operations.
        const bool leader = lane == 0;
        if (warp == 0) {
            // ---------------- producer: Q tiles, then K tiles ----------------
#pragma unroll
            for (int t = 0; t < TILES; ++t) {
                if (plan.qt[t].rows == 0 || !leader) continue;
                mbar_expect_tx(bar(BAR_Q_FULL + t), L::kTileBytes);
                int c1, c2;
                coords(0, (blockIdx.x * TILES + t) * BM, c1, c2);
                for (int s = 0; s < NSUB; ++s)
                    tma_load_4d(smem_base + L::kQ + t * L::kTileBytes + s * L::kSubTileBytes, &map_q,
                                bar(BAR_Q_FULL + t), s * 64, c1, c2, batch);
            }
            int n = 0;
            bool halo_seen = p.halo_flag == nullptr;
            for (int x = plan.x_begin; x < plan.x_end; ++x, ++n) {
                const int s = n % KS;
                if (!halo_seen && p.np + plan.anchor + x * BN - p.k_pos0 < p.np + p.halo_rows) {
                    flag_wait(p.halo_flag, p.flag_value, p.flag_wait_limit, abort_flag, p.status);
                    halo_seen = true;
                }
                mbar_wait(bar(BAR_K_EMPTY + s), ((n / KS) & 1) ^ 1, abort_flag, p.status);
                if (leader) {
                    mbar_expect_tx(bar(BAR_K_FULL + s), L::kTileBytes);
                    int c1, c2;
                    coords(1, p.np + plan.anchor + x * BN - p.k_pos0, c1, c2);
                    for (int u = 0; u < NSUB; ++u)
                        tma_load_4d(smem_base + L::kK + s * L::kTileBytes + u * L::kSubTileBytes, &map_k,
                                    bar(BAR_K_FULL + s), u * 64, c1, c2, batch);
                }
                __syncwarp();
            }
        } else if (warp == 1) {
            // ---------------- producer: persistent K/V, then V tiles ----------------
            // (the persistent maps end at row np: rows np .. np_pad - 1 of the tile arrive as zeros)
            if (p.np > 0 && p.pers_flag != nullptr)
                flag_wait(p.pers_flag, p.flag_value, p.flag_wait_limit, abort_flag, p.status);
            if (p.np > 0 && leader) {
                mbar_expect_tx(bar(BAR_KP_FULL), 2 * pers_bytes);
                int c1, c2;
                coords(1, 0, c1, c2);
                for (int u = 0; u < NSUB; ++u)
                    tma_load_4d(smem_base + L::kP + u * p.np_pad * 128, &map_kp, bar(BAR_KP_FULL), u * 64, c1, c2, batch);
                coords(2, 0, c1, c2);
                for (int u = 0; u < NSUB; ++u)
                    tma_load_4d(smem_base + L::kP + pers_bytes + u * p.np_pad * 128, &map_vp, bar(BAR_KP_FULL), u * 64,
                                c1, c2, batch);
            }
            int n = 0;
            bool halo_seen = p.halo_flag == nullptr;
            for (int x = plan.x_begin; x < plan.x_end; ++x, ++n) {
                const int s = n % VS;
                if (!halo_seen && p.np + plan.anchor + x * BN - p.k_pos0 < p.np + p.halo_rows) {
                    flag_wait(p.halo_flag, p.flag_value, p.flag_wait_limit, abort_flag, p.status);
                    halo_seen = true;
                }
                mbar_wait(bar(BAR_V_EMPTY + s), ((n / VS) & 1) ^ 1, abort_flag, p.status);
                if (leader) {
                    mbar_expect_tx(bar(BAR_V_FULL + s), L::kTileBytes);
                    int c1, c2;
                    coords(2, p.np + plan.anchor + x * BN - p.k_pos0, c1, c2);
                    for (int u = 0; u < NSUB; ++u)
                        tma_load_4d(smem_base + L::kV + s * L::kTileBytes + u * L::kSubTileBytes, &map_v,
                                    bar(BAR_V_FULL + s), u * 64, c1, c2, batch);
                }
                __syncwarp();
            }
        } else if (warp - 2 < TILES) {
            // ---------------- tensor-core issue: warp 2 drives query tile 0, warp 3 query tile 1 ----------------
            // Each warp issues, for its own query tile, QK of item i+1 right after PV of item i (P aliases S, and
            // tcgen05 operations of one thread execute in issue order).  A K/V stage is free again once BOTH
            // warps have arrived on its "empty" barrier: a warp that multiplies the tile arrives through
            // tcgen05.commit after its last use, a warp that does not need the tile arrives once it has seen
            // the tile land (so that the arrival is counted in the right phase).  All bookkeeping is kept
            // incremental and in registers: this instruction stream paces the softmax groups.
            const int t = warp - 2;
            const uint32_t fmt = BF16 ? 1u : 0u;
            const uint32_t idesc_qk_win = make_idesc(fmt, 0, BN);
            const uint32_t idesc_qk_pers = make_idesc(fmt, 0, (uint32_t)max(p.np_pad, 16));
            const uint32_t idesc_pv = make_idesc(fmt, 1, DH);
            // high word of every descriptor: stride byte offset 1024, version 1, 128-byte swizzle
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            auto desc_of = [](uint32_t lo) -> uint64_t { return ((uint64_t)kDescHi << 32) | lo; };
            // low word: start address >> 4 | leading byte offset >> 4 << 16
            auto lo_of = [](uint32_t addr, uint32_t lbo) -> uint32_t { return ((addr >> 4) & 0x3fffu) | ((lbo >> 4) << 16); };
            const QtPlan q = t == 0 ? plan.qt[0] : plan.qt[1];
            const int n_tiles = plan.x_end - plan.x_begin;        // window tiles loaded by the producers
            const int n_first = q.n_win > 0 ? q.a - plan.x_begin : n_tiles;  // my tiles: [n_first, n_first + n_win)
            using TM = TmemMap<DH, TILES>;
            const uint32_t s_tmem = tmem_base + TM::s(t);
            const uint32_t p_tmem = tmem_base + TM::p(t);
            const uint32_t o_tmem = tmem_base + TM::o(t);
            const uint32_t a_lo = lo_of(smem_base + L::kQ + t * L::kTileBytes, 16);
            const uint32_t s_bar = bar(BAR_S_FULL + t), p_bar = bar(BAR_P_READY + t);

            // ring cursors: the next K tile / V tile this warp has not yet passed
            int kn = 0, k_stage = 0;
            uint32_t k_par = 0;
            int vn = 0, v_stage = 0;
            uint32_t v_par = 0;
            auto k_advance = [&]() { ++kn; if (++k_stage == KS) { k_stage = 0; k_par ^= 1u; } };
            auto v_advance = [&]() { ++vn; if (++v_stage == VS) { v_stage = 0; v_par ^= 1u; } };
            // Tiles this warp never multiplies: see them land, then hand the stage back.  K and V tiles are
            // taken alternately — a warp that sat on the K ring alone would starve the V ring (and with it
            // the other warp) as soon as it had more tiles to pass than the ring has stages.
            auto skip_tiles_until = [&](int n_stop) {
                while (kn < n_stop || vn < n_stop) {
                    if (kn < n_stop && kn <= vn) {
                        mbar_wait(bar(BAR_K_FULL + k_stage), k_par, abort_flag, p.status);
                        if (leader) mbar_arrive(bar(BAR_K_EMPTY + k_stage));
                        k_advance();
                    } else {
                        mbar_wait(bar(BAR_V_FULL + v_stage), v_par, abort_flag, p.status);
                        if (leader) mbar_arrive(bar(BAR_V_EMPTY + v_stage));
                        v_advance();
                    }
                }
            };

            auto qk_pers = [&]() {
                mbar_wait(bar(BAR_KP_FULL), 0, abort_flag, p.status);
                const uint32_t b_lo = lo_of(smem_base + L::kP, 16);
                const uint32_t b_sub = (uint32_t)p.np_pad * 8;  // sub-tile stride >> 4
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < DH / 16; ++kk) {
                    const uint64_t ad = desc_of(a_lo + (kk / 4) * (L::kSubTileBytes >> 4) + (kk % 4) * 2);
                    const uint64_t bd = desc_of(b_lo + (kk / 4) * b_sub + (kk % 4) * 2);
                    if (leader) mma_ss(s_tmem, ad, bd, idesc_qk_pers, kk > 0 ? 1u : 0u);
                }
                if (leader) tc_commit(s_bar);
                __syncwarp();
            };
            // QK of the window tile under the K cursor (waits for the tile, releases its stage)
            auto qk_win = [&]() {
                mbar_wait(bar(BAR_K_FULL + k_stage), k_par, abort_flag, p.status);
                const uint32_t b_lo = lo_of(smem_base + L::kK + k_stage * L::kTileBytes, 16);
                const uint32_t e_bar = bar(BAR_K_EMPTY + k_stage);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < DH / 16; ++kk) {
                    const uint64_t ad = desc_of(a_lo + (kk / 4) * (L::kSubTileBytes >> 4) + (kk % 4) * 2);
                    const uint64_t bd = desc_of(b_lo + (kk / 4) * (L::kSubTileBytes >> 4) + (kk % 4) * 2);
                    if (leader) mma_ss(s_tmem, ad, bd, idesc_qk_win, kk > 0 ? 1u : 0u);
                }
                if (leader) {
                    tc_commit(s_bar);
                    tc_commit(e_bar);
                }
                __syncwarp();
                k_advance();
            };
            auto pv_pers = [&]() {
                const uint32_t b_lo = lo_of(smem_base + L::kP + pers_bytes, (uint32_t)p.np_pad * 128);
                tc_fence_after();
                for (int kk = 0; kk < p.np_pad / 16; ++kk) {
                    const uint64_t bd = desc_of(b_lo + kk * 128);
                    if (leader) mma_ts(o_tmem, p_tmem + kk * 8, bd, idesc_pv, kk > 0 ? 1u : 0u);
                }
                __syncwarp();
            };
            // PV of the window tile under the V cursor; acc0 = 0 only for the very first product of the tile
            auto pv_win = [&](uint32_t acc0) {
                mbar_wait(bar(BAR_V_FULL + v_stage), v_par, abort_flag, p.status);
                // B = V tile, MN-major: 16 keys = two 8-row groups of 1024 bytes per k-step
                const uint32_t b_lo = lo_of(smem_base + L::kV + v_stage * L::kTileBytes, L::kSubTileBytes);
                const uint32_t e_bar = bar(BAR_V_EMPTY + v_stage);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    const uint64_t bd = desc_of(b_lo + kk * 128);
                    if (leader) mma_ts(o_tmem, p_tmem + kk * 8, bd, idesc_pv, kk > 0 ? 1u : acc0);
                }
                if (leader) tc_commit(e_bar);
                __syncwarp();
                v_advance();
            };

            if (q.n_items > 0) {
                mbar_wait(bar(BAR_Q_FULL + t), 0, abort_flag, p.status);
                if (q.n_win > 0) skip_tiles_until(n_first);  // at most one tile: the other query tile's first
                if (q.has_pers) qk_pers(); else qk_win();
#pragma unroll 1
                for (int i = 0; i < q.n_items; ++i) {
                    if (TM::kSplitP && i + 1 < q.n_items) {
                        // S of item i is in the softmax group's registers: the next S may be produced
                        // while the group is still busy with the exponentials of item i
                        mbar_wait(bar(BAR_S_FREE + t), i & 1, abort_flag, p.status);
                        qk_win();
                    }
                    mbar_wait(p_bar, i & 1, abort_flag, p.status);
                    if (i < q.has_pers) pv_pers(); else pv_win(i > 0 ? 1u : 0u);
                    if (TM::kSplitP) {
                        if (leader) tc_commit(bar(i + 1 < q.n_items ? BAR_PV_DONE + t : BAR_O_DONE + t));
                    } else {
                        if (i + 1 < q.n_items) qk_win();
                        else if (leader) tc_commit(bar(BAR_O_DONE + t));
                    }
                }
            }
            // hand back the stages of the tiles behind my last one (or all of them if I had none)
            skip_tiles_until(n_tiles);
        }
    } else {
        // ---------------- softmax groups ----------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Budget<TILES, RS>::kRegsSoftmax) : "memory");
        // one thread per score row, or (RS == 2) two: warps w and w + 4 share the rows of their lane group and
        // take 64 of a key tile's 128 columns each, half of the output columns, and exchange the row maxima
        // and sums through shared memory
        const int t = RS == 2 ? 0 : (warp >> 2) - 1;   // query tile of this group
        const int half = RS == 2 ? (warp >> 2) - 1 : 0;
        const int row = threadIdx.x & (BM - 1);        // row of the tile == tensor-memory lane
        constexpr int NCH = 4 / RS;                    // 32-column chunks per thread
        const int c_first = half * NCH;                // this thread's first chunk
        float* xmax = reinterpret_cast<float*>(bar_area + 512);        // [item parity][half][row]
        float* xsum = xmax + 4 * BM;                                   // [half][row]
        const QtPlan q = t == 0 ? plan.qt[0] : plan.qt[1];
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        using TM = TmemMap<DH, TILES>;
        const uint32_t s_addr = tmem_base + lane_addr + TM::s(t);
        const uint32_t p_addr = tmem_base + lane_addr + TM::p(t);
        const uint32_t o_addr = tmem_base + lane_addr + TM::o(t);
        const int pos = q.p_lo + row;
        float m_used = -INFINITY;  // maximum the stored P and O are relative to (log2 domain)
        float l_sum = 0.f;

        // Alternation of the two softmax groups: both share the four schedulers and their special-function
        // units, and left alone they fall into step and queue for the exponentials together.  Group 0 goes
        // first; a group starts the exponentials of round r only after the other group has issued those of
        // its previous round.  Both groups run max(items of tile 0, items of tile 1) rounds.
        constexpr bool kAlternate = TILES == 2 && Alternate<DH>::value;
        const int rounds = kAlternate ? max(plan.qt[0].n_items, plan.qt[1].n_items) : 0;
        const uint32_t my_turn = bar(BAR_TURN + t), other_turn = bar(BAR_TURN + (t ^ 1));

        for (int item = 0; item < q.n_items; ++item) {
            // visible columns of this row inside the tile: [j_lo, j_hi]
            int j_lo, j_hi, ncols;
            bool full;
            if (item < q.has_pers) {
                j_lo = 0;
                j_hi = p.np - 1;
                ncols = p.np_pad;
                full = false;
            } else {
                const int g0 = plan.anchor + (q.a + item - q.has_pers) * BN;
                if (all_keys) {
                    j_lo = 0;
                    j_hi = p.k_pos0 + (p.k_rows - p.np) - 1 - g0;  // the last key row that exists
                } else if (pos >= p.np) {
                    j_lo = first_visible_pos(pos, p.np, p.window, wblock) - g0;
                    j_hi = pos - g0;
                } else {
                    j_lo = 1;
                    j_hi = 0;
                }
                ncols = BN;
                // every row of the tile sees every key of the tile (decided per tile, not per row)
                full = all_keys ? j_hi >= BN - 1
                                : q.p_lo >= p.np && g0 >= p.np && g0 + BN - 1 <= q.p_lo &&
                                      g0 >= first_visible_pos(q.p_lo + BM - 1, p.np, p.window, wblock);
            }
            const int nchunks = (ncols + 31) / 32;
            // 32-column chunks in which no row of this warp sees a key (beyond the diagonal, or before the
            // window's left edge): not loaded, not exponentiated, P = 0
            // (cc counts this thread's chunks, c = c_first + cc is the chunk's place in the tile)
            bool hid[NCH];
#pragma unroll
            for (int cc = 0; cc < NCH; ++cc) {
                const int c = c_first + cc;
                hid[cc] = !full && __all_sync(0xffffffffu, j_hi - c * 32 < 0 || j_lo - c * 32 > 31);
            }

            mbar_wait(bar(BAR_S_FULL + t), item & 1, abort_flag, p.status);
            tc_fence_after();

            uint32_t s[NCH][32];
#pragma unroll
            for (int cc = 0; cc < NCH; ++cc)
                if (c_first + cc < nchunks && !hid[cc]) tmem_ld32(s_addr + (c_first + cc) * 32, s[cc]);
            tc_wait_ld();
            if (TM::kSplitP) {
                // S is in registers now: let the issuing warp overwrite it with the next item's scores
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(BAR_S_FREE + t));
            }

            // mask (only the chunks in which some row of the warp has a hidden key), then the row maximum
            // over four independent chains of 3-input max
            if (!full) {
#pragma unroll
                for (int cc = 0; cc < NCH; ++cc)
                    if (c_first + cc < nchunks && !hid[cc]) {
                        const int c = c_first + cc;
                        const int lo = j_lo - c * 32, hi = j_hi - c * 32;  // visible columns of the chunk: [lo, hi]
                        if (!__all_sync(0xffffffffu, lo <= 0 && hi >= 31)) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < lo || j > hi) s[cc][j] = 0xff800000u;  // -inf
                        }
                    }
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int cc = 0; cc < NCH; ++cc)
                if (c_first + cc < nchunks && !hid[cc]) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            mx[k] = max3(mx[k], __uint_as_float(s[cc][j + 2 * k]), __uint_as_float(s[cc][j + 2 * k + 1]));
                        }
                    }
                }
            float tile_max = max3(fmaxf(mx[0], mx[1]), mx[2], mx[3]);
            tile_max *= p.scale_log2;  // scale > 0, so the maximum commutes with the scaling
            if (RS == 2) {
                // the row's other half: through shared memory, two buffers in turn (a buffer is written again two
                // items later, behind the next item's barrier, when both threads of every row have read it)
                float* xm = xmax + (item & 1) * 2 * BM;
                xm[half * BM + row] = tile_max;
                named_barrier_sync(3 + (warp & 3), 64);  // the two warps that share these 32 rows
                tile_max = fmaxf(tile_max, xm[(half ^ 1) * BM + row]);
            }

            if (TM::kSplitP && item > 0) {
                // the previous P V must have finished before O is rescaled or P is overwritten.  (Keeping the
                // exponentials in registers until then, to take this wait off the path previous P -> P V ->
                // this P, was measured: the 64 extra live registers spill and the kernel is 1.5 x slower.)
                mbar_wait(bar(BAR_PV_DONE + t), (item - 1) & 1, abort_flag, p.status);
                tc_fence_after();
            }
            // lazy maximum: keep the old reference unless the new maximum is more than 2^8 above it
            const bool grow = tile_max > m_used + 8.0f;
            if (item == 0) {
                m_used = tile_max;
            } else if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_used, tile_max);
                const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(m_used - m_new);
                m_used = m_new;
                l_sum *= alpha;
                if (RS == 2) {
                    // this thread's half of the output columns, 16 at a time: the scores stay live in registers
#pragma unroll
                    for (int cc = 0; cc < DH / 32; ++cc) {
                        uint32_t o[16];
                        tmem_ld16(o_addr + half * (DH / 2) + cc * 16, o);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                        tmem_st16(o_addr + half * (DH / 2) + cc * 16, o);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < DH / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld32(o_addr + c * 32, o);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                        tmem_st32(o_addr + c * 32, o);
                    }
                }
            }

            // P = exp2(S * c - m) on the special-function unit, packed two 16-bit values per column
            const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
            const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2);
            const uint64_t negm2 = pack2(neg_m, neg_m);
            uint64_t lacc[2] = {0ull, 0ull};  // four partial row sums
            if (kAlternate) mbar_wait(my_turn, (uint32_t)(item & 1) ^ (t == 0 ? 1u : 0u), abort_flag, p.status);
#pragma unroll
            for (int cc = 0; cc < NCH; ++cc)
                if (c_first + cc < nchunks) {
                    const int c = c_first + cc;
                    // 32 score columns -> 16 packed columns per store (two threads per row: 16 -> 8, fewer
                    // registers in flight)
                    constexpr int PART = RS == 2 ? 8 : 16;  // column pairs per store
#pragma unroll
                    for (int part = 0; part < 16 / PART; ++part) {
                        uint32_t packed[PART];
                        if (hid[cc]) {
#pragma unroll
                            for (int i = 0; i < PART; ++i) packed[i] = 0u;
                        } else {
#pragma unroll
                            for (int i = 0; i < PART; ++i) {
                                const int j = (part * PART + i) * 2;
                                const uint64_t x = fma2(pack2(__uint_as_float(s[cc][j]), __uint_as_float(s[cc][j + 1])),
                                                        scale2, negm2);
                                float x0, x1;
                                unpack2(x, x0, x1);
                                const float e0 = fast_exp2(x0);
                                const float e1 = fast_exp2(x1);
                                lacc[i & 1] = add2(lacc[i & 1], pack2(e0, e1));
                                if (BF16) {
                                    const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
                                    packed[i] = *reinterpret_cast<const uint32_t*>(&h);
                                } else {
                                    const __half2 h = __floats2half2_rn(e0, e1);
                                    packed[i] = *reinterpret_cast<const uint32_t*>(&h);
                                }
                            }
                        }
                        if constexpr (RS == 2) tmem_st8(p_addr + c * 16 + part * 8, packed);
                        else tmem_st16(p_addr + c * 16, packed);
                    }
                }
            {
                float a0, a1, a2, a3;
                unpack2(lacc[0], a0, a1);
                unpack2(lacc[1], a2, a3);
                l_sum += (a0 + a1) + (a2 + a3);
            }
            if (kAlternate) {
                __syncwarp();
                if (lane == 0) mbar_arrive(other_turn);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(BAR_P_READY + t));
        }

        for (int r = q.n_items; r < rounds; ++r) {  // keep the hand-over going for the group with more items
            mbar_wait(my_turn, (uint32_t)(r & 1) ^ (t == 0 ? 1u : 0u), abort_flag, p.status);
            __syncwarp();
            if (lane == 0) mbar_arrive(other_turn);
        }

        if (q.n_items > 0) {
            // ---------------- epilogue: O / l -> shared memory (swizzled) -> TMA store ----------------
            mbar_wait(bar(BAR_O_DONE + t), 0, abort_flag, p.status);
            tc_fence_after();
            if (RS == 2) {  // the row's sum: both halves
                xsum[half * BM + row] = l_sum;
                named_barrier_sync(1, RS * BM);
                l_sum += xsum[(half ^ 1) * BM + row];
            }
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
            if (p.lse != nullptr && row < q.rows && half == 0)
                p.lse[((long long)batch * gridDim.y + head) * p.q_rows + (blockIdx.x * TILES + t) * BM + row] =
                    m_used + log2f(l_sum);
            uint8_t* stage = smem + L::kQ + t * L::kTileBytes;  // the Q tile is no longer needed
#pragma unroll
            for (int cc = 0; cc < DH / 32 / RS; ++cc) {  // this thread's share of the output columns
                const int c = half * (DH / 32 / RS) + cc;
                uint32_t o[32];
                tmem_ld32(o_addr + c * 32, o);
                tc_wait_ld();
#pragma unroll
                for (int g = 0; g < 4; ++g) {  // 8 columns = one 16-byte chunk
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float a = __uint_as_float(o[g * 8 + 2 * e]) * inv;
                        const float b = __uint_as_float(o[g * 8 + 2 * e + 1]) * inv;
                        if (BF16) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                            w[e] = *reinterpret_cast<const uint32_t*>(&h);
                        } else {
                            const __half2 h = __floats2half2_rn(a, b);
                            w[e] = *reinterpret_cast<const uint32_t*>(&h);
                        }
                    }
                    const int col = c * 32 + g * 8;          // first column of the chunk
                    const int sub = col / 64;                // 64-column sub-tile
                    const int chunk = (col % 64) / 8;        // 16-byte chunk inside the 128-byte row
                    uint8_t* dst = stage + sub * L::kSubTileBytes + row * 128 + ((chunk ^ (row & 7)) * 16);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async_smem();
            named_barrier_sync(1 + t, RS * BM);
            if (row == 0 && half == 0) {
                int c1, c2;
                coords(3, (blockIdx.x * TILES + t) * BM, c1, c2);
                for (int u = 0; u < NSUB; ++u)
                    tma_store_4d(&map_o, smem_u32(stage + u * L::kSubTileBytes), u * 64, c1, c2, batch);
                tma_store_commit_and_wait();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (*abort_flag) {
            // a wait expired somewhere in this CTA: give asynchronous copies and matrix products that may
            // still be in flight time to finish before tensor memory and shared memory are handed back
            const long long t0 = clock64();
            while (clock64() - t0 < 400000) __nanosleep(1000);
        }
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------
// Host side: tensor maps and launch
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

// Strides (in elements) that the tensor maps of a [batch, heads, rows, dh] tensor use.  The stride of an
// extent-1 axis is never used for addressing; it gets a harmless valid value.
struct MapStrides {
    int64_t row, head, batch;
    bool heads_first;  // the head axis has the smaller stride and comes before the row axis in the map
};
MapStrides map_strides(int batch, int heads, int rows, int dh, const int64_t stride[3]) {
    MapStrides m;
    m.row = rows > 1 ? stride[2] : dh;
    m.head = heads > 1 ? stride[1] : m.row * rows;
    const int64_t inner_span = m.head * heads > m.row * rows ? m.head * heads : m.row * rows;
    m.batch = batch > 1 ? stride[0] : inner_span;
    m.heads_first = m.head < m.row;
    return m;
}

// What cuTensorMapEncodeTiled accepts: strides that are positive multiples of 16 bytes below 2^40 bytes.
// (Broadcast views with a zero stride and the like go to the CUDA-core kernel.)
bool map_strides_ok(const MapStrides& m) {
    const int64_t limit = ((int64_t)1 << 40) / 2;
    return m.row > 0 && m.head > 0 && m.batch > 0 && m.row < limit && m.head < limit && m.batch < limit &&
           m.row % 8 == 0 && m.head % 8 == 0 && m.batch % 8 == 0;
}

// Encoded maps are kept per host thread, keyed by everything that goes into them: a caller that runs the same
// buffers again (a layer inside a captured or repeated step) pays for the six driver calls once.
struct MapKey {
    const void* base;
    int64_t row, head, batch_stride;
    int32_t dtype, batch, heads, rows, dh, box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && row == o.row && head == o.head && batch_stride == o.batch_stride && dtype == o.dtype &&
               batch == o.batch && heads == o.heads && rows == o.rows && dh == o.dh && box_rows == o.box_rows;
    }
};
struct MapCache {
    static constexpr int kEntries = 64;
    MapKey key[kEntries];
    CUtensorMap map[kEntries];
    bool used[kEntries] = {false};
    int next = 0;
};

// Map over rows [0, rows) of a [batch, heads, *, dh] tensor laid out by `m`: a box of box_rows rows x 64
// columns of one (batch, head).  Rows of a box at or beyond `rows` are filled with zeros on load and dropped
// on store.  Returns false on failure.
bool make_map(CUtensorMap* map, const void* base, int dtype, int batch, int heads, int rows, int dh,
              const MapStrides& m, int box_rows) {
    static thread_local MapCache cache;
    const MapKey key{base, m.row, m.head, m.batch, dtype, batch, heads, rows, dh, box_rows};
    for (int i = 0; i < MapCache::kEntries; ++i)
        if (cache.used[i] && cache.key[i] == key) {
            *map = cache.map[i];
            return true;
        }
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[4];
    cuuint64_t strides[3];
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
    const int slot = cache.next;
    cache.next = (cache.next + 1) % MapCache::kEntries;
    cache.key[slot] = key;
    cache.map[slot] = *map;
    cache.used[slot] = true;
    return true;
}

int np_pad_of(int np) { return np > 0 ? ((np + 15) / 16) * 16 : 0; }

template <int DH, int KS, int VS, int TILES, int RS>
int launch_tc(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, void* o, cudaStream_t stream,
              int window_block, bool all_keys, float* lse, const tmw_halo_wait* wait) {
    using L = TcSmem<DH, KS, VS, TILES>;
    const int np_pad = np_pad_of(d.n_persistent);
    CUtensorMap mq, mk, mv, mo, mkp, mvp;
    const MapStrides sq = map_strides(d.batch, d.heads, d.q_rows, DH, d.q_stride);
    const MapStrides sk = map_strides(d.batch, d.heads, d.k_rows, DH, d.k_stride);
    const MapStrides sv = map_strides(d.batch, d.heads, d.k_rows, DH, d.v_stride);
    const MapStrides so = map_strides(d.batch, d.heads, d.q_rows, DH, d.o_stride);
    // The persistent tile is a box of np_pad rows of a map that ENDS at row np: the rows between np and
    // np_pad are zero-filled instead of being read from the first sequence rows (whatever those hold - even
    // Inf or NaN bits of a buffer that is still being filled - must not reach 0 x V in the P V product).
    const int np_rows = d.n_persistent > 0 ? d.n_persistent : 1;
    if (!make_map(&mq, q, d.dtype, d.batch, d.heads, d.q_rows, DH, sq, BM) ||
        !make_map(&mk, k, d.dtype, d.batch, d.heads, d.k_rows, DH, sk, BN) ||
        !make_map(&mv, v, d.dtype, d.batch, d.heads, d.k_rows, DH, sv, BN) ||
        !make_map(&mo, o, d.dtype, d.batch, d.heads, d.q_rows, DH, so, BM) ||
        !make_map(&mkp, k, d.dtype, d.batch, d.heads, np_rows, DH, sk, np_pad > 0 ? np_pad : 16) ||
        !make_map(&mvp, v, d.dtype, d.batch, d.heads, np_rows, DH, sv, np_pad > 0 ? np_pad : 16))
        return TMW_ERR_CUDA;
    TcParams p;
    p.q_rows = d.q_rows; p.k_rows = d.k_rows; p.window = d.window; p.np = d.n_persistent; p.np_pad = np_pad;
    p.block = window_block;
    p.window_plan = d.window + (window_block > 0 ? window_block - 1 : 0);
    p.all_keys = all_keys ? 1 : 0;
    p.lse = lse;
    p.pers_flag = wait != nullptr ? wait->pers_flag : nullptr;
    p.halo_flag = wait != nullptr ? wait->halo_flag : nullptr;
    p.flag_value = wait != nullptr ? wait->value : 0;
    p.halo_rows = wait != nullptr ? wait->halo_rows : 0;
    p.flag_wait_limit = wait != nullptr && wait->wait_limit_cycles > 0 ? wait->wait_limit_cycles : kWaitLimitCycles;
    p.q_pos0 = d.q_pos0; p.k_pos0 = d.k_pos0;
    p.dim_order = (sq.heads_first ? 1 : 0) | (sk.heads_first ? 2 : 0) | (sv.heads_first ? 4 : 0) | (so.heads_first ? 8 : 0);
    const float scale = d.scale != 0.f ? d.scale : 1.0f / sqrtf((float)DH);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = device_status_word();
    if (p.status == nullptr) return TMW_ERR_CUDA;
    const int smem_bytes = L::total_bytes(np_pad);
    dim3 grid((d.q_rows + TILES * BM - 1) / (TILES * BM), d.heads, d.batch);
    constexpr int kThreadsTc = Budget<TILES, RS>::kThreads;
    const bool general = window_block > 0 || all_keys;
    auto run = [&](auto kern) -> int {
        const int rc = allow_shared_memory(reinterpret_cast<const void*>(kern), smem_bytes);
        if (rc != TMW_OK) return rc;
        kern<<<grid, kThreadsTc, smem_bytes, stream>>>(mq, mk, mv, mo, mkp, mvp, p);
        return TMW_OK;
    };
    int st;
    if (d.dtype == TMW_BF16)
        st = general ? run(prefill_tc_kernel<DH, KS, VS, true, TILES, true, RS>) : run(prefill_tc_kernel<DH, KS, VS, true, TILES, false, RS>);
    else
        st = general ? run(prefill_tc_kernel<DH, KS, VS, false, TILES, true, RS>) : run(prefill_tc_kernel<DH, KS, VS, false, TILES, false, RS>);
    if (st != TMW_OK) return st;
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

constexpr int kMaxDynamicSmem = 232448;  // 227 KB per CTA on sm_100
constexpr int kTwoCtaSmem = (233472 - 2 * 1024) / 2;  // 228 KB per SM, 1 KB per CTA reserved by the system

}  // namespace

bool prefill_tc_supports(const tmw_prefill_desc& d, const void*, const void*, const void*, const void*) {
    if (d.dtype != TMW_BF16 && d.dtype != TMW_F16) return false;
    if (d.head_dim != 64 && d.head_dim != 128) return false;
    if (d.batch > 65535 || d.heads > 65535) return false;
    const int np_pad = np_pad_of(d.n_persistent);
    if (np_pad > 128) return false;
    const int need = d.head_dim == 64 ? TcSmem<64, 3, 3, 2>::total_bytes(np_pad) : TcSmem<128, 2, 2, 2>::total_bytes(np_pad);
    if (need > kMaxDynamicSmem) return false;
    // positions are combined in 32-bit arithmetic inside the kernel
    if ((int64_t)d.q_pos0 + d.q_rows + d.window + 4 * BN >= (int64_t)1 << 30) return false;
    // layouts a tensor map cannot describe
    if (!map_strides_ok(map_strides(d.batch, d.heads, d.q_rows, d.head_dim, d.q_stride)) ||
        !map_strides_ok(map_strides(d.batch, d.heads, d.k_rows, d.head_dim, d.k_stride)) ||
        !map_strides_ok(map_strides(d.batch, d.heads, d.k_rows, d.head_dim, d.v_stride)) ||
        !map_strides_ok(map_strides(d.batch, d.heads, d.q_rows, d.head_dim, d.o_stride)))
        return false;
    return true;
}

int launch_prefill_tc(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, void* o,
                      cudaStream_t stream, int window_block, bool all_keys, float* lse, const tmw_halo_wait* wait) {
    if (d.head_dim == 64) {
        // One query tile per CTA and two CTAs per SM when two such CTAs fit into shared memory (they do
        // unless there are many persistent keys): independent CTAs drift apart, so one CTA's exponentials,
        // start-up and output phase overlap the other's matrix products.
        if (TcSmem<64, 3, 2, 1>::total_bytes(np_pad_of(d.n_persistent)) <= kTwoCtaSmem) {
            // Two threads per score row (twice the softmax warps, half the dependent chain per key tile each) once a
            // query tile has enough key tiles for that to outweigh the exchange between the two threads: measured
            // on 8 x 10 heads x 4112 rows, window 128 | 512 | 2048: 91.0 | 141.5 | 293.9 us against 87.2 | 152.6 | 300.9.
            if (d.window >= 192)
                return launch_tc<64, 3, 2, 1, 2>(d, q, k, v, o, stream, window_block, all_keys, lse, wait);
            return launch_tc<64, 3, 2, 1, 1>(d, q, k, v, o, stream, window_block, all_keys, lse, wait);
        }
        return launch_tc<64, 3, 3, 2, 1>(d, q, k, v, o, stream, window_block, all_keys, lse, wait);
    }
    return launch_tc<128, 2, 2, 2, 1>(d, q, k, v, o, stream, window_block, all_keys, lse, wait);
}

}  // namespace tmw
