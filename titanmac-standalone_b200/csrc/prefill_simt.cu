// CUDA-core prefill kernel: sliding-window attention with persistent prefix keys,
// fp32 accumulation everywhere.  It is the kernel behind the fp32 contract (max-abs
// 1e-5 against the reference) and the one that covers head sizes the tensor-core
// kernel does not.  Out-of-window keys are never loaded: a CTA walks the persistent
// keys and then only the key positions [first_row - w, last_row] of its query rows.
//
// Work split: a CTA owns ROWS = 128 / LPR consecutive query rows of one (batch,
// head); each row is held by LPR adjacent lanes, every lane keeping DH / LPR
// elements of the query and of the output accumulator in registers.  Keys and values
// are staged in shared memory as fp32 in tiles of BN keys (all lanes of a warp read
// the same key element, so the reads are broadcasts) and consumed in register
// sub-tiles of JB scores with one online-softmax update per sub-tile.
#include <math_constants.h>

#include "tmw_common.cuh"

namespace tmw {
namespace {

constexpr int kThreads = 128;
constexpr int JB = 16;

template <int DH>
struct SimtShape {
    static constexpr int LPR = DH <= 32 ? 1 : (DH == 96 ? 4 : DH / 32);  // lanes per query row
    static constexpr int DPL = DH / LPR;                                  // elements per lane
    static constexpr int CH = DPL / 8;                                    // 8-element chunks per lane
    static constexpr int ROWS = kThreads / LPR;                           // query rows per CTA
    static constexpr int BN = DH <= 128 ? 32 : 16;                        // keys per shared-memory tile
    static_assert(DPL % 8 == 0 && DPL <= 32, "lane slice must be 8..32 elements");
};

struct SimtParams {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    int q_rows, k_rows, window, np, q_pos0, k_pos0;
    int block;     // 0 or the block size of the block-granular window
    int all_keys;  // 1: no mask at all, every key row is visible to every query row of the call
    long long qs[3], ks[3], vs[3], os[3];
    float scale_log2;  // scale * log2(e)
    float* lse;        // optional [batch, heads, q_rows]: m + log2(l) of every row (log2 domain)
};

template <typename T, int DH>
__global__ void __launch_bounds__(kThreads) prefill_simt_kernel(const SimtParams p) {
    using S = SimtShape<DH>;
    __shared__ __align__(16) float k_tile[S::BN][DH];
    __shared__ __align__(16) float v_tile[S::BN][DH];

    const int tid = threadIdx.x;
    const int sub = tid % S::LPR;
    const int row_in_cta = tid / S::LPR;
    const int r0 = blockIdx.x * S::ROWS;
    const int row = r0 + row_in_cta;
    const bool valid = row < p.q_rows;
    const int h = blockIdx.y, b = blockIdx.z;

    const T* qg = static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1];
    const T* kg = static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1];
    const T* vg = static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1];
    T* og = static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1];

    // query slice of this lane: chunks sub, sub + LPR, ... of 8 elements each
    float qreg[S::DPL];
    float acc[S::DPL];
#pragma unroll
    for (int c = 0; c < S::CH; ++c) {
        float tmp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (valid) load8<T>(qg + (long long)row * p.qs[2] + (sub + c * S::LPR) * 8, tmp);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            qreg[c * 8 + e] = tmp[e];
            acc[c * 8 + e] = 0.f;
        }
    }
    float m = -CUDART_INF_F, l = 0.f;

    const int pos = p.q_pos0 + row;  // position of this lane's query
    const int p_first = p.q_pos0 + r0;
    const int p_last = p.q_pos0 + min(r0 + S::ROWS, p.q_rows) - 1;
    // window keys this CTA can need: positions [glo, ghi]
    const int glo = p.all_keys ? p.k_pos0 : first_visible_pos(max(p_first, p.np), p.np, p.window, p.block);
    const int ghi = p.all_keys ? p.k_pos0 + (p.k_rows - p.np) - 1 : p_last;
    const int n_win = (p.all_keys || p_last >= p.np) && ghi >= glo ? ghi - glo + 1 : 0;
    const int my_lo = pos >= p.np ? first_visible_pos(pos, p.np, p.window, p.block) : 0;
    const int n_keys = p.np + n_win;  // virtual key index u: [0,np) persistent, then the window

    for (int u0 = 0; u0 < n_keys; u0 += S::BN) {
        __syncthreads();
        // ---- stage BN keys and values as fp32 ----
        constexpr int CHUNKS_PER_ROW = DH / 8;
        for (int c = tid; c < S::BN * CHUNKS_PER_ROW; c += kThreads) {
            const int j = c / CHUNKS_PER_ROW;
            const int col = (c % CHUNKS_PER_ROW) * 8;
            const int u = u0 + j;
            float kt[8] = {0, 0, 0, 0, 0, 0, 0, 0}, vt[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (u < n_keys) {
                const long long kr = u < p.np ? u : (long long)p.np + (glo + (u - p.np)) - p.k_pos0;
                if (kr >= 0 && kr < p.k_rows) {
                    load8<T>(kg + kr * p.ks[2] + col, kt);
                    load8<T>(vg + kr * p.vs[2] + col, vt);
                }
            }
            *reinterpret_cast<float4*>(&k_tile[j][col]) = make_float4(kt[0], kt[1], kt[2], kt[3]);
            *reinterpret_cast<float4*>(&k_tile[j][col + 4]) = make_float4(kt[4], kt[5], kt[6], kt[7]);
            *reinterpret_cast<float4*>(&v_tile[j][col]) = make_float4(vt[0], vt[1], vt[2], vt[3]);
            *reinterpret_cast<float4*>(&v_tile[j][col + 4]) = make_float4(vt[4], vt[5], vt[6], vt[7]);
        }
        __syncthreads();

#pragma unroll 1
        for (int j0 = 0; j0 < S::BN; j0 += JB) {
            if (u0 + j0 >= n_keys) break;  // uniform over the CTA
            float s[JB];
            float tmax = -CUDART_INF_F;
#pragma unroll
            for (int jj = 0; jj < JB; ++jj) {
                const int j = j0 + jj;
                float part = 0.f;
#pragma unroll
                for (int c = 0; c < S::CH; ++c) {
                    const float4 a = *reinterpret_cast<const float4*>(&k_tile[j][(sub + c * S::LPR) * 8]);
                    const float4 bq = *reinterpret_cast<const float4*>(&k_tile[j][(sub + c * S::LPR) * 8 + 4]);
                    part = fmaf(qreg[c * 8 + 0], a.x, part);
                    part = fmaf(qreg[c * 8 + 1], a.y, part);
                    part = fmaf(qreg[c * 8 + 2], a.z, part);
                    part = fmaf(qreg[c * 8 + 3], a.w, part);
                    part = fmaf(qreg[c * 8 + 4], bq.x, part);
                    part = fmaf(qreg[c * 8 + 5], bq.y, part);
                    part = fmaf(qreg[c * 8 + 6], bq.z, part);
                    part = fmaf(qreg[c * 8 + 7], bq.w, part);
                }
#pragma unroll
                for (int off = 1; off < S::LPR; off <<= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
                const int u = u0 + j;
                const int g = u < p.np ? u : glo + (u - p.np);
                const bool vis = valid && u < n_keys &&
                                 (p.all_keys || u < p.np || (pos >= p.np && g <= pos && g >= my_lo));
                s[jj] = vis ? part * p.scale_log2 : -CUDART_INF_F;
                tmax = fmaxf(tmax, s[jj]);
            }
            if (tmax > -CUDART_INF_F) {  // same answer on every lane of a row
                const float m_new = fmaxf(m, tmax);
                const float alpha = exp2f(m - m_new);  // m = -inf gives 0
                m = m_new;
                l *= alpha;
#pragma unroll
                for (int e = 0; e < S::DPL; ++e) acc[e] *= alpha;
#pragma unroll
                for (int jj = 0; jj < JB; ++jj) {
                    const float pj = exp2f(s[jj] - m);  // s = -inf gives 0
                    l += pj;
                    const int j = j0 + jj;
#pragma unroll
                    for (int c = 0; c < S::CH; ++c) {
                        const float4 a = *reinterpret_cast<const float4*>(&v_tile[j][(sub + c * S::LPR) * 8]);
                        const float4 bq = *reinterpret_cast<const float4*>(&v_tile[j][(sub + c * S::LPR) * 8 + 4]);
                        acc[c * 8 + 0] = fmaf(pj, a.x, acc[c * 8 + 0]);
                        acc[c * 8 + 1] = fmaf(pj, a.y, acc[c * 8 + 1]);
                        acc[c * 8 + 2] = fmaf(pj, a.z, acc[c * 8 + 2]);
                        acc[c * 8 + 3] = fmaf(pj, a.w, acc[c * 8 + 3]);
                        acc[c * 8 + 4] = fmaf(pj, bq.x, acc[c * 8 + 4]);
                        acc[c * 8 + 5] = fmaf(pj, bq.y, acc[c * 8 + 5]);
                        acc[c * 8 + 6] = fmaf(pj, bq.z, acc[c * 8 + 6]);
                        acc[c * 8 + 7] = fmaf(pj, bq.w, acc[c * 8 + 7]);
                    }
                }
            }
        }
    }

    if (valid && sub == 0 && p.lse != nullptr)
        p.lse[((long long)b * gridDim.y + h) * p.q_rows + row] = m + log2f(l);
    if (valid) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < S::CH; ++c) {
            float tmp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = acc[c * 8 + e] * inv;
            store8<T>(og + (long long)row * p.os[2] + (sub + c * S::LPR) * 8, tmp);
        }
    }
}

template <typename T, int DH>
int launch_t(const SimtParams& p, int batch, int heads, cudaStream_t stream) {
    using S = SimtShape<DH>;
    if (p.q_rows == 0 || batch == 0 || heads == 0) return TMW_OK;
    dim3 grid((p.q_rows + S::ROWS - 1) / S::ROWS, heads, batch);
    prefill_simt_kernel<T, DH><<<grid, kThreads, 0, stream>>>(p);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

template <typename T>
int launch_dh(const SimtParams& p, int batch, int heads, int dh, cudaStream_t stream) {
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

int launch_prefill_simt(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, void* o,
                        cudaStream_t stream, int window_block, bool all_keys, float* lse) {
    SimtParams p;
    p.lse = lse;
    p.block = window_block;
    p.all_keys = all_keys ? 1 : 0;
    p.q = q; p.k = k; p.v = v; p.o = o;
    p.q_rows = d.q_rows; p.k_rows = d.k_rows; p.window = d.window; p.np = d.n_persistent;
    p.q_pos0 = d.q_pos0; p.k_pos0 = d.k_pos0;
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = d.q_stride[i]; p.ks[i] = d.k_stride[i]; p.vs[i] = d.v_stride[i]; p.os[i] = d.o_stride[i];
    }
    const float scale = d.scale != 0.f ? d.scale : 1.0f / sqrtf((float)d.head_dim);
    p.scale_log2 = scale * 1.4426950408889634f;
    if (d.batch > 65535 || d.heads > 65535) return TMW_ERR_TOO_LARGE;
    switch (d.dtype) {
        case TMW_F32: return launch_dh<float>(p, d.batch, d.heads, d.head_dim, stream);
        case TMW_BF16: return launch_dh<__nv_bfloat16>(p, d.batch, d.heads, d.head_dim, stream);
        case TMW_F16: return launch_dh<__half>(p, d.batch, d.heads, d.head_dim, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

}  // namespace tmw
