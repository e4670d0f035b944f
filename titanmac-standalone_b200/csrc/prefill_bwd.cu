// Backward of the windowed attention core on CUDA cores (fp32 arithmetic): given dO, the saved
// output O and the per-row log-sum-exp of the forward, it returns dQ, dK and dV with the same tile
// skipping as the forward - no key outside a query's window is touched, no L x L matrix exists.
//
//   P = exp2(S c - lse)      (S = Q K^T, c = scale log2 e, lse from the forward, masked pairs give 0)
//   D_i = sum_d dO_id O_id
//   dS = P o (dO V^T - D)
//   dQ = scale dS K          dK = scale dS^T Q          dV = P^T dO
//
// Two kernels.  bwd_dq: a CTA owns query rows (one row per LPR adjacent lanes, like the forward kernel) and
// walks over the persistent keys and the keys of its window.  bwd_dkv: a CTA owns key rows and walks over
// the queries that can see them - the next `window` rows for a sequence key, every row for a persistent key.
// Whole sequences only (q_pos0 = 0, k_pos0 = n_persistent, q_rows = k_rows).
#include <math_constants.h>

#include "tmw_common.cuh"

namespace tmw {
namespace {

constexpr int kThreads = 128;

template <int DH>
struct BwdShape {
    static constexpr int LPR = DH <= 32 ? 1 : (DH == 96 ? 4 : DH / 32);  // lanes per row
    static constexpr int DPL = DH / LPR;                                  // elements per lane
    static constexpr int CH = DPL / 8;                                    // 8-element chunks per lane
    static constexpr int ROWS = kThreads / LPR;                           // rows owned by a CTA
    static constexpr int BN = DH <= 128 ? 32 : 16;                        // rows per shared-memory tile
    static_assert(DPL % 8 == 0 && DPL <= 32, "lane slice must be 8..32 elements");
};

struct BwdParams {
    const void* q;
    const void* k;
    const void* v;
    const void* o;
    const void* d_o;
    const float* lse;
    void* dq;
    void* dk;
    void* dv;
    int rows, window, np;  // rows = L
    int block;        // 0: per-token window; > 0: block-granular left edge (first_visible_pos)
    int pers_global;  // 1: the np persistent query rows see every key (the block-sparse class); then the
                      //    log-sum-exp comes in two planes: [batch, heads, rows - np] for the sequence rows,
                      //    followed by [batch, heads, np] for the persistent rows
    long long qs[3], ks[3], vs[3], os[3];  // q / dq, k / dk, v / dv, o / dO share strides pairwise
    float scale, scale_log2;
};

// log-sum-exp of query row `row` of (batch b, head h)
__device__ __forceinline__ float lse_at(const BwdParams& p, int b, int h, int heads, int row) {
    const long long bh = (long long)b * heads + h;
    if (!p.pers_global) return p.lse[bh * p.rows + row];
    if (row >= p.np) return p.lse[bh * (p.rows - p.np) + (row - p.np)];
    return p.lse[(long long)gridDim.z * heads * (p.rows - p.np) + bh * p.np + row];
}
// does the query at position i see the key at position g (g < np: a persistent key)?
__device__ __forceinline__ bool sees(const BwdParams& p, int i, int g) {
    if (g < p.np) return true;
    if (i < p.np) return p.pers_global != 0;
    return g <= i && g >= first_visible_pos(i, p.np, p.window, p.block);
}

// this lane's slice of a row: chunks sub, sub + LPR, ... of 8 elements each
template <typename T, int DH>
__device__ __forceinline__ void load_slice(const T* row, int sub, float (&out)[BwdShape<DH>::DPL]) {
    using S = BwdShape<DH>;
#pragma unroll
    for (int c = 0; c < S::CH; ++c) {
        float tmp[8];
        load8<T>(row + (sub + c * S::LPR) * 8, tmp);
#pragma unroll
        for (int e = 0; e < 8; ++e) out[c * 8 + e] = tmp[e];
    }
}
template <typename T, int DH>
__device__ __forceinline__ void store_slice(T* row, int sub, const float (&in)[BwdShape<DH>::DPL], float mul) {
    using S = BwdShape<DH>;
#pragma unroll
    for (int c = 0; c < S::CH; ++c) {
        float tmp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = in[c * 8 + e] * mul;
        store8<T>(row + (sub + c * S::LPR) * 8, tmp);
    }
}
// dot product of this lane's register slice with the matching slice of a shared-memory row
template <int DH>
__device__ __forceinline__ float dot_slice(const float (&a)[BwdShape<DH>::DPL], const float* smem_row, int sub) {
    using S = BwdShape<DH>;
    float part = 0.f;
#pragma unroll
    for (int c = 0; c < S::CH; ++c) {
        const float4 x = *reinterpret_cast<const float4*>(smem_row + (sub + c * S::LPR) * 8);
        const float4 y = *reinterpret_cast<const float4*>(smem_row + (sub + c * S::LPR) * 8 + 4);
        part = fmaf(a[c * 8 + 0], x.x, part);
        part = fmaf(a[c * 8 + 1], x.y, part);
        part = fmaf(a[c * 8 + 2], x.z, part);
        part = fmaf(a[c * 8 + 3], x.w, part);
        part = fmaf(a[c * 8 + 4], y.x, part);
        part = fmaf(a[c * 8 + 5], y.y, part);
        part = fmaf(a[c * 8 + 6], y.z, part);
        part = fmaf(a[c * 8 + 7], y.w, part);
    }
    return part;
}
// acc += w * (slice of a shared-memory row)
template <int DH>
__device__ __forceinline__ void axpy_slice(float (&acc)[BwdShape<DH>::DPL], float w, const float* smem_row, int sub) {
    using S = BwdShape<DH>;
#pragma unroll
    for (int c = 0; c < S::CH; ++c) {
        const float4 x = *reinterpret_cast<const float4*>(smem_row + (sub + c * S::LPR) * 8);
        const float4 y = *reinterpret_cast<const float4*>(smem_row + (sub + c * S::LPR) * 8 + 4);
        acc[c * 8 + 0] = fmaf(w, x.x, acc[c * 8 + 0]);
        acc[c * 8 + 1] = fmaf(w, x.y, acc[c * 8 + 1]);
        acc[c * 8 + 2] = fmaf(w, x.z, acc[c * 8 + 2]);
        acc[c * 8 + 3] = fmaf(w, x.w, acc[c * 8 + 3]);
        acc[c * 8 + 4] = fmaf(w, y.x, acc[c * 8 + 4]);
        acc[c * 8 + 5] = fmaf(w, y.y, acc[c * 8 + 5]);
        acc[c * 8 + 6] = fmaf(w, y.z, acc[c * 8 + 6]);
        acc[c * 8 + 7] = fmaf(w, y.w, acc[c * 8 + 7]);
    }
}
template <int LPR>
__device__ __forceinline__ float reduce_row(float x) {
#pragma unroll
    for (int off = 1; off < LPR; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    return x;
}
// stages `n` rows (first at row index r0, rows beyond `limit` as zeros) of a [.., rows, DH] tensor as fp32
template <typename T, int DH, int BN>
__device__ __forceinline__ void stage_rows(float (*tile)[DH], const T* base, long long row_stride, int r0, int limit) {
    constexpr int CPR = DH / 8;
    for (int c = threadIdx.x; c < BN * CPR; c += kThreads) {
        const int j = c / CPR, col = (c % CPR) * 8;
        float t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (r0 + j < limit) load8<T>(base + (long long)(r0 + j) * row_stride + col, t);
        *reinterpret_cast<float4*>(&tile[j][col]) = make_float4(t[0], t[1], t[2], t[3]);
        *reinterpret_cast<float4*>(&tile[j][col + 4]) = make_float4(t[4], t[5], t[6], t[7]);
    }
}

// ---------------------------------------------------------------------------------------------------------
template <typename T, int DH>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(const BwdParams p) {
    using S = BwdShape<DH>;
    __shared__ __align__(16) float k_tile[S::BN][DH];
    __shared__ __align__(16) float v_tile[S::BN][DH];
    const int tid = threadIdx.x, sub = tid % S::LPR, r0 = blockIdx.x * S::ROWS;
    const int row = r0 + tid / S::LPR;
    const bool valid = row < p.rows;
    const int h = blockIdx.y, b = blockIdx.z;
    const T* qg = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
    const T* kg = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
    const T* vg = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
    const T* og = static_cast<const T*>(p.o) + b * p.os[0] + h * p.os[1];
    const T* dog = static_cast<const T*>(p.d_o) + b * p.os[0] + h * p.os[1];
    T* dqg = static_cast<T*>(p.dq) + b * p.qs[0] + h * p.qs[1];

    float qreg[S::DPL], doreg[S::DPL], acc[S::DPL];
#pragma unroll
    for (int e = 0; e < S::DPL; ++e) qreg[e] = doreg[e] = acc[e] = 0.f;
    float dsum = 0.f, lse = 0.f;
    if (valid) {
        load_slice<T, DH>(qg + (long long)row * p.qs[2], sub, qreg);
        load_slice<T, DH>(dog + (long long)row * p.os[2], sub, doreg);
        float oreg[S::DPL];
        load_slice<T, DH>(og + (long long)row * p.os[2], sub, oreg);
#pragma unroll
        for (int e = 0; e < S::DPL; ++e) dsum = fmaf(doreg[e], oreg[e], dsum);
        lse = lse_at(p, b, h, gridDim.y, row);
    }
    dsum = reduce_row<S::LPR>(dsum);

    // virtual key index u: [0, np) persistent keys, then the positions [glo, ghi] of this CTA's windows
    const int p_last = min(r0 + S::ROWS, p.rows) - 1;
    const bool all_seq = p.pers_global && r0 < p.np;  // a persistent row in this CTA: every sequence key
    const int glo = all_seq ? p.np : first_visible_pos(max(r0, p.np), p.np, p.window, p.block);
    const int ghi = all_seq ? p.rows - 1 : p_last;
    const int n_win = (all_seq || p_last >= p.np) && ghi >= glo ? ghi - glo + 1 : 0;
    const int n_keys = p.np + n_win;
    for (int u0 = 0; u0 < n_keys; u0 += S::BN) {
        __syncthreads();
        constexpr int CPR = DH / 8;
        for (int c = tid; c < S::BN * CPR; c += kThreads) {
            const int j = c / CPR, col = (c % CPR) * 8, u = u0 + j;
            float kt[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vt[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (u < n_keys) {
                const long long kr = u < p.np ? u : glo + (u - p.np);
                load8<T>(kg + kr * p.ks[2] + col, kt);
                load8<T>(vg + kr * p.vs[2] + col, vt);
            }
            *reinterpret_cast<float4*>(&k_tile[j][col]) = make_float4(kt[0], kt[1], kt[2], kt[3]);
            *reinterpret_cast<float4*>(&k_tile[j][col + 4]) = make_float4(kt[4], kt[5], kt[6], kt[7]);
            *reinterpret_cast<float4*>(&v_tile[j][col]) = make_float4(vt[0], vt[1], vt[2], vt[3]);
            *reinterpret_cast<float4*>(&v_tile[j][col + 4]) = make_float4(vt[4], vt[5], vt[6], vt[7]);
        }
        __syncthreads();
        const int jn = min(S::BN, n_keys - u0);
        for (int j = 0; j < jn; ++j) {
            const float s = reduce_row<S::LPR>(dot_slice<DH>(qreg, k_tile[j], sub));
            const float dp = reduce_row<S::LPR>(dot_slice<DH>(doreg, v_tile[j], sub));
            const int u = u0 + j;
            const int g = u < p.np ? u : glo + (u - p.np);
            const bool vis = valid && sees(p, row, g);
            const float pj = vis ? exp2f(s * p.scale_log2 - lse) : 0.f;
            axpy_slice<DH>(acc, pj * (dp - dsum), k_tile[j], sub);
        }
    }
    if (valid) store_slice<T, DH>(dqg + (long long)row * p.qs[2], sub, acc, p.scale);
}

// ---------------------------------------------------------------------------------------------------------
template <typename T, int DH>
__global__ void __launch_bounds__(kThreads) bwd_dkv_kernel(const BwdParams p, int n_seq_blocks) {
    using S = BwdShape<DH>;
    __shared__ __align__(16) float q_tile[S::BN][DH];
    __shared__ __align__(16) float do_tile[S::BN][DH];
    __shared__ float lse_s[S::BN], dsum_s[S::BN];
    const int tid = threadIdx.x, sub = tid % S::LPR;
    const int h = blockIdx.y, b = blockIdx.z;
    const bool pers_block = (int)blockIdx.x >= n_seq_blocks;
    // key rows owned by this CTA: [k0, k_end)
    const int k0 = pers_block ? ((int)blockIdx.x - n_seq_blocks) * S::ROWS : p.np + (int)blockIdx.x * S::ROWS;
    const int k_end = pers_block ? min(p.np, k0 + S::ROWS) : min(p.rows, k0 + S::ROWS);
    const int key = k0 + tid / S::LPR;
    const bool valid = key < k_end;
    const T* qg = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
    const T* kg = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
    const T* vg = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
    const T* og = static_cast<const T*>(p.o) + b * p.os[0] + h * p.os[1];
    const T* dog = static_cast<const T*>(p.d_o) + b * p.os[0] + h * p.os[1];
    T* dkg = static_cast<T*>(p.dk) + b * p.ks[0] + h * p.ks[1];
    T* dvg = static_cast<T*>(p.dv) + b * p.vs[0] + h * p.vs[1];
    float kreg[S::DPL], vreg[S::DPL], dk[S::DPL], dv[S::DPL];
#pragma unroll
    for (int e = 0; e < S::DPL; ++e) kreg[e] = vreg[e] = dk[e] = dv[e] = 0.f;
    if (valid) {
        load_slice<T, DH>(kg + (long long)key * p.ks[2], sub, kreg);
        load_slice<T, DH>(vg + (long long)key * p.vs[2], sub, vreg);
    }
    // query rows that can see a key of this CTA: every row for persistent keys, [k0, last key + window] else
    // A sequence key is seen by the rows from its own position to the last row whose (possibly block-granular)
    // window still reaches it, and, for the block-sparse class, by the np persistent rows: those come first as
    // a range of their own ([0, np) never overlaps [k0, ...) because k0 >= np).
    const int reach = p.window + (p.block > 0 ? p.block - 1 : 0);
    const int main_lo = pers_block ? 0 : k0;
    const int main_hi = pers_block ? p.rows - 1 : (int)min((long long)p.rows - 1, (long long)k_end - 1 + reach);
    const int n_ranges = (!pers_block && p.pers_global && p.np > 0) ? 2 : 1;
    for (int range = 0; range < n_ranges; ++range) {
    const int i_lo = (n_ranges == 2 && range == 0) ? 0 : main_lo;
    const int i_hi = (n_ranges == 2 && range == 0) ? p.np - 1 : main_hi;
    for (int i0 = i_lo; i0 <= i_hi; i0 += S::BN) {
        __syncthreads();
        stage_rows<T, DH, S::BN>(q_tile, qg, p.qs[2], i0, i_hi + 1);
        stage_rows<T, DH, S::BN>(do_tile, dog, p.os[2], i0, i_hi + 1);
        if (tid < S::BN) {
            lse_s[tid] = i0 + tid <= i_hi ? lse_at(p, b, h, gridDim.y, i0 + tid) : 0.f;
            dsum_s[tid] = 0.f;
        }
        __syncthreads();
        // D_i = sum_d dO_id O_id of the staged rows (O is read once here, not staged)
        constexpr int CPR = DH / 8;
        for (int c = tid; c < S::BN * CPR; c += kThreads) {
            const int j = c / CPR, col = (c % CPR) * 8;
            if (i0 + j <= i_hi) {
                float t[8];
                load8<T>(og + (long long)(i0 + j) * p.os[2] + col, t);
                float part = 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) part = fmaf(t[e], do_tile[j][col + e], part);
                atomicAdd(&dsum_s[j], part);
            }
        }
        __syncthreads();
        const int jn = min(S::BN, i_hi + 1 - i0);
        for (int j = 0; j < jn; ++j) {
            const int i = i0 + j;  // query position
            const float s = reduce_row<S::LPR>(dot_slice<DH>(kreg, q_tile[j], sub));
            const float dp = reduce_row<S::LPR>(dot_slice<DH>(vreg, do_tile[j], sub));
            const bool vis = valid && sees(p, i, key);
            const float pj = vis ? exp2f(s * p.scale_log2 - lse_s[j]) : 0.f;
            axpy_slice<DH>(dv, pj, do_tile[j], sub);
            axpy_slice<DH>(dk, pj * (dp - dsum_s[j]), q_tile[j], sub);
        }
    }
    }  // ranges
    if (valid) {
        store_slice<T, DH>(dkg + (long long)key * p.ks[2], sub, dk, p.scale);
        store_slice<T, DH>(dvg + (long long)key * p.vs[2], sub, dv, 1.0f);
    }
}

template <typename T, int DH>
int launch_t(const BwdParams& p, int batch, int heads, cudaStream_t stream) {
    using S = BwdShape<DH>;
    const dim3 gq((p.rows + S::ROWS - 1) / S::ROWS, heads, batch);
    bwd_dq_kernel<T, DH><<<gq, kThreads, 0, stream>>>(p);
    TMW_CUDA_TRY(cudaGetLastError());
    const int n_seq = (p.rows - p.np + S::ROWS - 1) / S::ROWS;
    const int n_pers = (p.np + S::ROWS - 1) / S::ROWS;
    const dim3 gk(n_seq + n_pers, heads, batch);
    bwd_dkv_kernel<T, DH><<<gk, kThreads, 0, stream>>>(p, n_seq);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

template <typename T>
int launch_dh(const BwdParams& p, int batch, int heads, int dh, cudaStream_t stream) {
    switch (dh) {
        case 8: return launch_t<T, 8>(p, batch, heads, stream);
        case 16: return launch_t<T, 16>(p, batch, heads, stream);
        case 32: return launch_t<T, 32>(p, batch, heads, stream);
        case 64: return launch_t<T, 64>(p, batch, heads, stream);
        case 96: return launch_t<T, 96>(p, batch, heads, stream);
        case 128: return launch_t<T, 128>(p, batch, heads, stream);
        case 256: return launch_t<T, 256>(p, batch, heads, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

}  // namespace

int launch_prefill_backward(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o,
                            const void* d_o, const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream,
                            int window_block, bool pers_global) {
    BwdParams p;
    p.block = window_block;
    p.pers_global = pers_global ? 1 : 0;
    p.q = q; p.k = k; p.v = v; p.o = o; p.d_o = d_o; p.lse = lse; p.dq = dq; p.dk = dk; p.dv = dv;
    p.rows = d.q_rows; p.window = d.window; p.np = d.n_persistent;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = d.q_stride[i]; p.ks[i] = d.k_stride[i]; p.vs[i] = d.v_stride[i]; p.os[i] = d.o_stride[i];
    }
    p.scale = d.scale != 0.f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
    p.scale_log2 = p.scale * 1.4426950408889634f;
    if (d.batch > 65535 || d.heads > 65535) return TMW_ERR_TOO_LARGE;
    switch (d.dtype) {
        case TMW_F32: return launch_dh<float>(p, d.batch, d.heads, d.head_dim, stream);
        case TMW_BF16: return launch_dh<__nv_bfloat16>(p, d.batch, d.heads, d.head_dim, stream);
        case TMW_F16: return launch_dh<__half>(p, d.batch, d.heads, d.head_dim, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

}  // namespace tmw
