// Backward of the windowed attention core on the warp-level tensor-core path (nvcuda::wmma, 16-bit inputs,
// fp32 accumulation), for head_dim 64 and 128.  Same mathematics and the same two-kernel split as the
// CUDA-core version in prefill_bwd.cu - a dQ kernel that owns 64 query rows and walks over the 64-key blocks
// of their windows, a dK/dV kernel that owns 64 keys and walks over the query blocks that can see them - but
// the five matrix products per (query block, key block) pair run as 16x16x16 tensor-core tiles:
//
//   S  = Q K^T          dP = dO V^T                (fp32 tiles to shared memory)
//   P  = exp2(S c - lse) o mask,  dS = P o (dP - D)  (element-wise, rounded to the 16-bit type)
//   dV += P^T dO        dK += dS^T Q               dQ += dS K
//
// Everything between the products goes through shared memory, which keeps the fragment layouts of the wmma
// API opaque.  The tiles a kernel walks over (K / V in the dQ kernel, Q / dO in the dK/dV kernel) are requested
// one pair ahead with cp.async into a second buffer pair, so a round's loads overlap the previous round's
// products.  Whole sequences only, like the CUDA-core version.
#include <math_constants.h>
#include <mma.h>

#include "tmw_common.cuh"

namespace tmw {
namespace {

using namespace nvcuda;

constexpr int BR = 64;        // query rows per block
constexpr int BC = 64;        // keys per block
constexpr int kWarps = 8;
constexpr int kThreadsMma = kWarps * 32;

struct MmaBwdParams {
    const void* q;
    const void* k;
    const void* v;
    const void* o;
    const void* d_o;
    const float* lse;
    void* dq;
    void* dk;
    void* dv;
    int rows, window, np;
    int block;        // 0: per-token window; > 0: block-granular left edge (first_visible_pos)
    int pers_global;  // 1: the np persistent query rows see every key; lse then comes as
                      //    [batch, heads, rows - np] followed by [batch, heads, np]
    long long qs[3], ks[3], vs[3], os[3];
    float scale, scale_log2;
};

// log-sum-exp of query row `row` of (batch b, head h); gridDim.z is the batch size
__device__ __forceinline__ float lse_at(const MmaBwdParams& p, int b, int h, int heads, int row) {
    const long long bh = (long long)b * heads + h;
    if (!p.pers_global) return p.lse[bh * p.rows + row];
    if (row >= p.np) return p.lse[bh * (p.rows - p.np) + (row - p.np)];
    return p.lse[(long long)gridDim.z * heads * (p.rows - p.np) + bh * p.np + row];
}

// Row strides in shared memory, padded by 16 bytes so that the 16 rows a tensor-core tile load touches fall
// into different banks (an unpadded 128-byte row stride puts all of them on the same ones).
template <int DH>
struct Ld {
    static constexpr int kT = DH + 8;   // 16-bit tiles [64 x DH]: K, V, Q, dO (and O while D is computed)
    static constexpr int kP = 64 + 8;   // 16-bit [64 x 64]: P, dS
    static constexpr int kS = 64 + 4;   // fp32 [64 x 64]: S, dP
    static constexpr int kOut = DH + 4; // fp32 [64 x DH]: results on the way out (in the S and dP buffers)
};

template <typename T, int DH>
struct MmaSmem {
    static constexpr int kTile = 64 * Ld<DH>::kT * 2;
    static constexpr int kPBytes = 64 * Ld<DH>::kP * 2;
    static constexpr int kSBytes = 64 * Ld<DH>::kS * 4;
    static constexpr int kK = 0, kV = kTile, kQ = 2 * kTile, kDO = 3 * kTile;
    static constexpr int kP = 4 * kTile, kDS = kP + kPBytes;   // contiguous: together they also hold an O tile
    static constexpr int kS = kDS + kPBytes, kDP = kS + kSBytes;  // contiguous: together they stage a result
    static constexpr int kLse = kDP + kSBytes, kD = kLse + 64 * 4;
    static constexpr int kBytes = kD + 64 * 4;
    static_assert(kTile <= 2 * kPBytes, "an O tile must fit into the P and dS buffers");
    static_assert(64 * Ld<DH>::kOut * 4 <= 2 * kSBytes, "an fp32 result tile must fit into the S and dP buffers");
    static_assert(kTile % 32 == 0 && kPBytes % 32 == 0 && kSBytes % 32 == 0, "tensor-core tile loads want 32-byte alignment");
};

// copies rows [r0, r0 + 64) of a [rows, DH] tensor (row stride in elements) into a dense 16-bit tile; rows at or
// beyond `limit` become zeros
template <typename T, int DH>
__device__ __forceinline__ void load_tile(T* tile, const T* base, long long row_stride, int r0, int limit) {
    constexpr int CPR = DH / 8;
    for (int c = threadIdx.x; c < 64 * CPR; c += kThreadsMma) {
        const int j = c / CPR, col = (c % CPR) * 8;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r0 + j < limit) val = *reinterpret_cast<const uint4*>(base + (long long)(r0 + j) * row_stride + col);
        *reinterpret_cast<uint4*>(tile + j * Ld<DH>::kT + col) = val;
    }
}

// the same copy with cp.async: 16 bytes per request straight into shared memory, no register staging, so all
// requests of a round's tiles are in flight at once; rows at or beyond `limit` are zero-filled (source size 0)
template <typename T, int DH>
__device__ __forceinline__ void load_tile_async(T* tile, const T* base, long long row_stride, int r0, int limit) {
    constexpr int CPR = DH / 8;
    for (int c = threadIdx.x; c < 64 * CPR; c += kThreadsMma) {
        const int j = c / CPR, col = (c % CPR) * 8;
        const bool live = r0 + j < limit;
        const T* src = live ? base + (long long)(r0 + j) * row_stride + col : base;
        const unsigned dst = (unsigned)__cvta_generic_to_shared(tile + j * Ld<DH>::kT + col);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
    }
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// out[64 x 64] (fp32, shared) = A[64 x DH] * B[64 x DH]^T, both 16-bit row-major tiles; 8 warps, 16 x 32 each
template <typename T, int DH>
__device__ __forceinline__ void gemm_abt(float* out, const T* a, const T* b) {
    const int warp = threadIdx.x >> 5;
    const int m0 = (warp >> 1) * 16, n0 = (warp & 1) * 32;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2];
    wmma::fill_fragment(acc[0], 0.f);
    wmma::fill_fragment(acc[1], 0.f);
    constexpr int LT = Ld<DH>::kT, LS = Ld<DH>::kS;
#pragma unroll
    for (int kk = 0; kk < DH; kk += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> fa;
        wmma::load_matrix_sync(fa, a + m0 * LT + kk, LT);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::col_major> fb;  // B^T: element (k, n) = b[n][k]
            wmma::load_matrix_sync(fb, b + (n0 + t * 16) * LT + kk, LT);
            wmma::mma_sync(acc[t], fa, fb, acc[t]);
        }
    }
    wmma::store_matrix_sync(out + m0 * LS + n0, acc[0], LS, wmma::mem_row_major);
    wmma::store_matrix_sync(out + m0 * LS + n0 + 16, acc[1], LS, wmma::mem_row_major);
}

// accumulators of a [64 x DH] result spread over 8 warps: warp w owns the 16-row band (w / 2) and the column
// tiles n = (w % 2) * DH / 32 + t, t < DH / 32
template <int DH>
struct Acc64 {
    static constexpr int NT = DH / 32;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> f[NT];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int t = 0; t < NT; ++t) wmma::fill_fragment(f[t], 0.f);
    }
};

// acc[64 x DH] += A^T B with A = a[64(k) x 64(m)] (16-bit, row-major, used transposed) and B = b[64(k) x DH]
template <typename T, int DH>
__device__ __forceinline__ void gemm_atb_acc(Acc64<DH>& acc, const T* a, const T* b) {
    const int warp = threadIdx.x >> 5;
    const int m0 = (warp >> 1) * 16, nbase = (warp & 1) * (DH / 2);
#pragma unroll
    for (int kk = 0; kk < 64; kk += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::col_major> fa;  // A^T: element (m, k) = a[k][m]
        wmma::load_matrix_sync(fa, a + kk * Ld<DH>::kP + m0, Ld<DH>::kP);
#pragma unroll
        for (int t = 0; t < Acc64<DH>::NT; ++t) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::row_major> fb;
            wmma::load_matrix_sync(fb, b + kk * Ld<DH>::kT + nbase + t * 16, Ld<DH>::kT);
            wmma::mma_sync(acc.f[t], fa, fb, acc.f[t]);
        }
    }
}
// acc[64 x DH] += A B with A = a[64(m) x 64(k)] (16-bit, row-major) and B = b[64(k) x DH]
template <typename T, int DH>
__device__ __forceinline__ void gemm_ab_acc(Acc64<DH>& acc, const T* a, const T* b) {
    const int warp = threadIdx.x >> 5;
    const int m0 = (warp >> 1) * 16, nbase = (warp & 1) * (DH / 2);
#pragma unroll
    for (int kk = 0; kk < 64; kk += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> fa;
        wmma::load_matrix_sync(fa, a + m0 * Ld<DH>::kP + kk, Ld<DH>::kP);
#pragma unroll
        for (int t = 0; t < Acc64<DH>::NT; ++t) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::row_major> fb;
            wmma::load_matrix_sync(fb, b + kk * Ld<DH>::kT + nbase + t * 16, Ld<DH>::kT);
            wmma::mma_sync(acc.f[t], fa, fb, acc.f[t]);
        }
    }
}
// stages the accumulators as fp32 [64 x DH] in shared memory, then writes rows [r0, r0 + 64) < limit, times `mul`
template <typename T, int DH>
__device__ __forceinline__ void store_acc(Acc64<DH>& acc, float* stage, T* base, long long row_stride, int r0, int limit,
                                          float mul) {
    const int warp = threadIdx.x >> 5;
    const int m0 = (warp >> 1) * 16, nbase = (warp & 1) * (DH / 2);
#pragma unroll
    for (int t = 0; t < Acc64<DH>::NT; ++t)
        wmma::store_matrix_sync(stage + m0 * Ld<DH>::kOut + nbase + t * 16, acc.f[t], Ld<DH>::kOut, wmma::mem_row_major);
    __syncthreads();
    constexpr int CPR = DH / 8;
    for (int c = threadIdx.x; c < 64 * CPR; c += kThreadsMma) {
        const int j = c / CPR, col = (c % CPR) * 8;
        if (r0 + j < limit) {
            float t[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = stage[j * Ld<DH>::kOut + col + e] * mul;
            store8<T>(base + (long long)(r0 + j) * row_stride + col, t);
        }
    }
}

// lse and D = sum_d dO O of the 64 staged query rows (O tile in `o_tile`, dO tile in `do_tile`)
template <typename T, int DH>
__device__ __forceinline__ void row_stats(float* lse_s, float* d_s, const T* o_tile, const T* do_tile,
                                          const MmaBwdParams& p, int b, int h, int i0, int limit) {
    // four threads per row
    const int row = threadIdx.x >> 2, part = threadIdx.x & 3;
    float sum = 0.f;
    for (int c = part * (DH / 4); c < (part + 1) * (DH / 4); ++c)
        sum = fmaf(to_f32<T>(o_tile[row * Ld<DH>::kT + c]), to_f32<T>(do_tile[row * Ld<DH>::kT + c]), sum);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (part == 0) {
        d_s[row] = sum;
        lse_s[row] = i0 + row < limit ? lse_at(p, b, h, gridDim.y, i0 + row) : 0.f;
    }
}

// P and dS of one (query block, key block) pair from S and dP.  `key_pos(c)` = position of key column c, or -1 for
// a persistent key; a column is hidden by returning -2.
template <typename T, int DH, typename KeyPos>
__device__ __forceinline__ void softmax_grad(T* p_s, T* ds_s, const float* s_s, const float* dp_s, const float* lse_s,
                                             const float* d_s, int i0, int rows, const MmaBwdParams& p, int wblock,
                                             bool pers_global, KeyPos key_pos) {
    const int np = p.np;
    const float scale_log2 = p.scale_log2;
    // four adjacent columns per thread (a warp covers two whole rows): 16-byte reads of S and dP, 8-byte writes of
    // P and dS; the padded row strides keep both aligned
    constexpr int CW = 4, TPR = 64 / CW;
    static_assert(Ld<DH>::kS % 4 == 0 && Ld<DH>::kP % 4 == 0, "row strides must keep 16-byte / 8-byte alignment");
    for (int e = threadIdx.x; e < 64 * TPR; e += kThreadsMma) {
        const int r = e / TPR, c = (e % TPR) * CW;
        const int i = i0 + r;
        const int es = r * Ld<DH>::kS + c, ep = r * Ld<DH>::kP + c;
        __align__(16) float sv[CW];
        __align__(16) float dpv[CW];
        *reinterpret_cast<float4*>(sv) = *reinterpret_cast<const float4*>(s_s + es);
        *reinterpret_cast<float4*>(dpv) = *reinterpret_cast<const float4*>(dp_s + es);
        const int lo = i >= np ? first_visible_pos(i, np, p.window, wblock) : 0;
        const float lse = lse_s[r], d = d_s[r];
        __align__(8) T pr[CW];
        __align__(8) T dsr[CW];
#pragma unroll
        for (int x = 0; x < CW; ++x) {
            const int g = key_pos(c + x);
            // persistent key: always; sequence key: the persistent rows see it only in the block-sparse class, a
            // sequence row sees it inside its (possibly block-granular) causal window
            const bool vis = i < rows && (g == -1 || (g >= 0 && (i < np ? pers_global : g <= i && g >= lo)));
            float pv = 0.f;
            if (vis) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pv) : "f"(sv[x] * scale_log2 - lse));
            pr[x] = from_f32<T>(pv);
            dsr[x] = from_f32<T>(pv * (dpv[x] - d));
        }
        *reinterpret_cast<uint2*>(p_s + ep) = *reinterpret_cast<const uint2*>(pr);
        *reinterpret_cast<uint2*>(ds_s + ep) = *reinterpret_cast<const uint2*>(dsr);
    }
}

// ---------------------------------------------------------------------------------------------------------
// GENERAL = false: the plain windowed mask, every mode parameter a compile-time constant (the block-sparse
// logic costs the common case nothing); GENERAL = true: block-granular window and global persistent rows.
template <typename T, int DH, bool GENERAL>
__global__ void __launch_bounds__(kThreadsMma, DH == 64 ? 2 : 1) bwd_mma_dkv_kernel(const MmaBwdParams p, int n_seq_blocks) {
    using L = MmaSmem<T, DH>;
    const int wblock = GENERAL ? p.block : 0;
    const bool pers_global = GENERAL && p.pers_global != 0;
    extern __shared__ __align__(128) unsigned char smem[];
    T* k_s = reinterpret_cast<T*>(smem + L::kK);
    T* v_s = reinterpret_cast<T*>(smem + L::kV);
    T* p_s = reinterpret_cast<T*>(smem + L::kP);
    T* ds_s = reinterpret_cast<T*>(smem + L::kDS);
    float* s_s = reinterpret_cast<float*>(smem + L::kS);
    float* dp_s = reinterpret_cast<float*>(smem + L::kDP);
    float* lse_s = reinterpret_cast<float*>(smem + L::kLse);
    float* d_s = reinterpret_cast<float*>(smem + L::kD);

    const int h = blockIdx.y, b = blockIdx.z;
    const bool pers = (int)blockIdx.x >= n_seq_blocks;
    const int k0 = pers ? ((int)blockIdx.x - n_seq_blocks) * BC : p.np + (int)blockIdx.x * BC;
    const int k_end = pers ? min(p.np, k0 + BC) : min(p.rows, k0 + BC);
    const T* qg = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
    const T* kg = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
    const T* vg = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
    const T* og = static_cast<const T*>(p.o) + b * p.os[0] + h * p.os[1];
    const T* dog = static_cast<const T*>(p.d_o) + b * p.os[0] + h * p.os[1];
    load_tile<T, DH>(k_s, kg, p.ks[2], k0, k_end);
    load_tile<T, DH>(v_s, vg, p.vs[2], k0, k_end);
    Acc64<DH> dk, dv;
    dk.zero();
    dv.zero();
    // query rows that see these keys: the rows from the key's own position to the last row whose (possibly
    // block-granular) window reaches it, and in the block-sparse class also the np persistent rows, which come
    // first as rounds of their own ([0, np) never overlaps [k0, ...) because k0 >= np; their rows end at np so
    // that a prefix round never touches sequence rows)
    const int reach = p.window + (wblock > 0 ? wblock - 1 : 0);
    const int main_lo = pers ? 0 : k0;
    const int main_hi = pers ? p.rows - 1 : (int)min((long long)p.rows - 1, (long long)k_end - 1 + reach);
    const int n_prefix = (!pers && pers_global && p.np > 0) ? (p.np + BR - 1) / BR : 0;
    const int n_rounds = n_prefix + (main_hi - main_lo) / BR + 1;
    auto round_rows = [&](int r, int& i0, int& limit) {
        if (r < n_prefix) {
            i0 = r * BR;
            limit = p.np;
        } else {
            i0 = main_lo + (r - n_prefix) * BR;
            limit = main_hi + 1;
        }
    };
    // Q and dO tiles alternate between two buffer pairs: round r + 1's tiles are requested (cp.async) before
    // round r computes
    auto q_buf = [&](int r) { return reinterpret_cast<T*>(smem + ((r & 1) ? L::kBytes : L::kQ)); };
    auto do_buf = [&](int r) { return reinterpret_cast<T*>(smem + ((r & 1) ? L::kBytes + L::kTile : L::kDO)); };
    auto request = [&](int r) {
        if (r < n_rounds) {
            int i0, limit;
            round_rows(r, i0, limit);
            load_tile_async<T, DH>(q_buf(r), qg, p.qs[2], i0, limit);
            load_tile_async<T, DH>(do_buf(r), dog, p.os[2], i0, limit);
        }
        async_commit();  // an empty group past the end keeps the wait count uniform
    };
    auto key_pos = [&](int c) { return k0 + c < k_end ? (pers ? -1 : k0 + c) : -2; };
    // D = sum_d dO O per query row: four threads per row, each with DH / 4 elements of O straight from global
    // memory in registers (requested before the round's barrier, used after the first two products)
    const int st_row = threadIdx.x >> 2, st_col = (threadIdx.x & 3) * (DH / 4);
    constexpr int OV = DH / 32;
    request(0);
    for (int r = 0; r < n_rounds; ++r) {
        int i0, limit;
        round_rows(r, i0, limit);
        T* q_s = q_buf(r);
        T* do_s = do_buf(r);
        const bool st_live = i0 + st_row < limit;
        uint4 o_reg[OV];
#pragma unroll
        for (int e = 0; e < OV; ++e)
            o_reg[e] = st_live ? *reinterpret_cast<const uint4*>(og + (long long)(i0 + st_row) * p.os[2] + st_col + e * 8)
                               : make_uint4(0, 0, 0, 0);
        const float st_lse = st_live ? lse_at(p, b, h, gridDim.y, i0 + st_row) : 0.f;
        async_wait<0>();
        __syncthreads();  // this round's Q / dO have landed; the previous round's products have read the other
                          // buffer pair, p_s and ds_s
        request(r + 1);
        gemm_abt<T, DH>(s_s, q_s, k_s);
        gemm_abt<T, DH>(dp_s, do_s, v_s);
        {
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < OV; ++e) {
                const T* ov = reinterpret_cast<const T*>(&o_reg[e]);
#pragma unroll
                for (int x = 0; x < 8; ++x)
                    sum = fmaf(to_f32<T>(ov[x]), to_f32<T>(do_s[st_row * Ld<DH>::kT + st_col + e * 8 + x]), sum);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if ((threadIdx.x & 3) == 0) {
                d_s[st_row] = sum;
                lse_s[st_row] = st_lse;
            }
        }
        __syncthreads();
        softmax_grad<T, DH>(p_s, ds_s, s_s, dp_s, lse_s, d_s, i0, limit, p, wblock, pers_global, key_pos);
        __syncthreads();
        gemm_atb_acc<T, DH>(dv, p_s, do_s);
        gemm_atb_acc<T, DH>(dk, ds_s, q_s);
    }
    __syncthreads();
    T* dkg = static_cast<T*>(p.dk) + b * p.ks[0] + h * p.ks[1];
    T* dvg = static_cast<T*>(p.dv) + b * p.vs[0] + h * p.vs[1];
    store_acc<T, DH>(dk, s_s, dkg, p.ks[2], k0, k_end, p.scale);
    __syncthreads();
    store_acc<T, DH>(dv, s_s, dvg, p.vs[2], k0, k_end, 1.0f);
}

// ---------------------------------------------------------------------------------------------------------
template <typename T, int DH, bool GENERAL>
__global__ void __launch_bounds__(kThreadsMma) bwd_mma_dq_kernel(const MmaBwdParams p) {
    using L = MmaSmem<T, DH>;
    const int wblock = GENERAL ? p.block : 0;
    const bool pers_global = GENERAL && p.pers_global != 0;
    extern __shared__ __align__(128) unsigned char smem[];
    T* q_s = reinterpret_cast<T*>(smem + L::kQ);
    T* do_s = reinterpret_cast<T*>(smem + L::kDO);
    T* p_s = reinterpret_cast<T*>(smem + L::kP);
    T* ds_s = reinterpret_cast<T*>(smem + L::kDS);
    float* s_s = reinterpret_cast<float*>(smem + L::kS);
    float* dp_s = reinterpret_cast<float*>(smem + L::kDP);
    float* lse_s = reinterpret_cast<float*>(smem + L::kLse);
    float* d_s = reinterpret_cast<float*>(smem + L::kD);

    const int h = blockIdx.y, b = blockIdx.z;
    const int i0 = blockIdx.x * BR;
    const T* qg = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
    const T* kg = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
    const T* vg = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
    const T* og = static_cast<const T*>(p.o) + b * p.os[0] + h * p.os[1];
    const T* dog = static_cast<const T*>(p.d_o) + b * p.os[0] + h * p.os[1];
    load_tile<T, DH>(q_s, qg, p.qs[2], i0, p.rows);
    load_tile<T, DH>(do_s, dog, p.os[2], i0, p.rows);
    load_tile<T, DH>(p_s, og, p.os[2], i0, p.rows);
    __syncthreads();
    row_stats<T, DH>(lse_s, d_s, p_s, do_s, p, b, h, i0, p.rows);
    Acc64<DH> dq;
    dq.zero();
    // key blocks: the persistent keys in blocks of 64, then the positions [glo, i_last] of this block's windows
    const int i_last = min(i0 + BR, p.rows) - 1;
    const bool all_seq = pers_global && i0 < p.np;  // a persistent row in this block: every sequence key
    const int glo = all_seq ? p.np : first_visible_pos(max(i0, p.np), p.np, p.window, wblock);
    const int ghi = all_seq ? p.rows - 1 : i_last;
    const int n_pers_blocks = (p.np + BC - 1) / BC;
    const int n_win_blocks = (all_seq || i_last >= p.np) && ghi >= glo ? (ghi - glo) / BC + 1 : 0;
    // K and V tiles alternate between two buffer pairs: round jb + 1's tiles are requested (cp.async) before
    // round jb computes
    auto k_buf = [&](int jb) { return reinterpret_cast<T*>(smem + ((jb & 1) ? L::kBytes : L::kK)); };
    auto v_buf = [&](int jb) { return reinterpret_cast<T*>(smem + ((jb & 1) ? L::kBytes + L::kTile : L::kV)); };
    const int n_blocks = n_pers_blocks + n_win_blocks;
    auto block_range = [&](int jb, int& k0, int& k_end) {
        const bool pers = jb < n_pers_blocks;
        k0 = pers ? jb * BC : glo + (jb - n_pers_blocks) * BC;
        k_end = pers ? min(p.np, k0 + BC) : min(ghi + 1, k0 + BC);
    };
    auto request = [&](int jb) {
        if (jb < n_blocks) {
            int k0, k_end;
            block_range(jb, k0, k_end);
            load_tile_async<T, DH>(k_buf(jb), kg, p.ks[2], k0, k_end);
            load_tile_async<T, DH>(v_buf(jb), vg, p.vs[2], k0, k_end);
        }
        async_commit();  // an empty group past the end keeps the wait count uniform
    };
    request(0);
    for (int jb = 0; jb < n_blocks; ++jb) {
        const bool pers = jb < n_pers_blocks;
        int k0, k_end;
        block_range(jb, k0, k_end);
        T* k_s = k_buf(jb);
        T* v_s = v_buf(jb);
        __syncthreads();  // the previous round's product has read the other K buffer and ds_s; row_stats has read p_s
        request(jb + 1);
        async_wait<1>();  // this round's tiles have landed (the next round's may still be in flight)
        __syncthreads();
        gemm_abt<T, DH>(s_s, q_s, k_s);
        gemm_abt<T, DH>(dp_s, do_s, v_s);
        __syncthreads();
        auto key_pos = [&](int c) { return k0 + c < k_end ? (pers ? -1 : k0 + c) : -2; };
        softmax_grad<T, DH>(p_s, ds_s, s_s, dp_s, lse_s, d_s, i0, p.rows, p, wblock, pers_global, key_pos);
        __syncthreads();
        gemm_ab_acc<T, DH>(dq, ds_s, k_s);
    }
    __syncthreads();
    T* dqg = static_cast<T*>(p.dq) + b * p.qs[0] + h * p.qs[1];
    store_acc<T, DH>(dq, s_s, dqg, p.qs[2], i0, p.rows, p.scale);
}

template <typename T, int DH>
int launch_mma(const MmaBwdParams& p, int batch, int heads, cudaStream_t stream) {
    using L = MmaSmem<T, DH>;
    const bool general = p.block > 0 || p.pers_global != 0;
    auto kq = general ? bwd_mma_dq_kernel<T, DH, true> : bwd_mma_dq_kernel<T, DH, false>;
    auto kkv = general ? bwd_mma_dkv_kernel<T, DH, true> : bwd_mma_dkv_kernel<T, DH, false>;
    constexpr int kDqBytes = L::kBytes + 2 * L::kTile;  // second buffer pair: K / V in the dQ kernel, Q / dO in the other
    TMW_CUDA_TRY(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqBytes));
    TMW_CUDA_TRY(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqBytes));
    const dim3 gq((p.rows + BR - 1) / BR, heads, batch);
    kq<<<gq, kThreadsMma, kDqBytes, stream>>>(p);
    TMW_CUDA_TRY(cudaGetLastError());
    const int n_seq = (p.rows - p.np + BC - 1) / BC, n_pers = (p.np + BC - 1) / BC;
    const dim3 gk(n_seq + n_pers, heads, batch);
    kkv<<<gk, kThreadsMma, kDqBytes, stream>>>(p, n_seq);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

}  // namespace

bool prefill_backward_mma_supports(const tmw_prefill_desc& d) {
    return (d.dtype == TMW_BF16 || d.dtype == TMW_F16) && (d.head_dim == 64 || d.head_dim == 128) && d.batch <= 65535 &&
           d.heads <= 65535;
}

int launch_prefill_backward_mma(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o,
                                const void* d_o, const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream,
                                int window_block, bool pers_global) {
    MmaBwdParams p;
    p.block = window_block;
    p.pers_global = pers_global ? 1 : 0;
    p.q = q; p.k = k; p.v = v; p.o = o; p.d_o = d_o; p.lse = lse; p.dq = dq; p.dk = dk; p.dv = dv;
    p.rows = d.q_rows; p.window = d.window; p.np = d.n_persistent;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = d.q_stride[i]; p.ks[i] = d.k_stride[i]; p.vs[i] = d.v_stride[i]; p.os[i] = d.o_stride[i];
    }
    p.scale = d.scale != 0.f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    if (d.dtype == TMW_BF16)
        return d.head_dim == 64 ? launch_mma<__nv_bfloat16, 64>(p, d.batch, d.heads, stream)
                                : launch_mma<__nv_bfloat16, 128>(p, d.batch, d.heads, stream);
    return d.head_dim == 64 ? launch_mma<__half, 64>(p, d.batch, d.heads, stream)
                            : launch_mma<__half, 128>(p, d.batch, d.heads, stream);
}

}  // namespace tmw
