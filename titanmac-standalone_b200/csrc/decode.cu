// Decode against a ring cache of the last window+1 keys per (sequence, head), plus
// the persistent keys every query sees.  The step is bound by HBM traffic (about one
// multiply-add per byte read), so the kernel is organised around wide coalesced
// loads: a key row of head_dim elements is read by head_dim/8 adjacent lanes with
// one 16-byte load each, a warp covers 32/(head_dim/8) rows per load instruction and
// keeps UNROLL such instructions in flight for K and for V before it touches the
// softmax.  Dot products are finished with warp shuffles; each lane group keeps a
// private online-softmax state that is merged across groups and warps at the end.
#include <math_constants.h>

#include "tmw_common.cuh"

namespace tmw {
namespace {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = kDecodeThreads / 32;
constexpr int UNROLL = 4;

struct DecodeParams {
    void* k_ring;
    void* v_ring;
    const void* k_pers;
    const void* v_pers;
    const void* q;
    const void* k_new;
    const void* v_new;
    void* o;
    const int32_t* pos;
    long long qs[2], ns[2], os[2];
    int heads, slots, np;
    float scale_log2;
};

// LPK = lanes per key row = DH / 8
template <typename T, int DH>
__global__ void __launch_bounds__(kDecodeThreads) decode_kernel(const DecodeParams p) {
    constexpr int LPK = DH / 8;
    constexpr int RPW = 32 / LPK;                 // key rows per warp per load instruction
    constexpr int STEP = RPW * kDecodeWarps;      // key rows per CTA per load instruction
    static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must be 8 * 2^n, at most 256");

    const int h = blockIdx.x, b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane % LPK;  // which 8-element slice of the row
    const int grp = lane / LPK;  // which row of the warp's RPW rows

    const int t = p.pos[b];
    const int slot_new = t % p.slots;
    const int count = min(t + 1, p.slots);
    const long long ring_bh = ((long long)b * p.heads + h) * p.slots * DH;
    T* kr = static_cast<T*>(p.k_ring) + ring_bh;
    T* vr = static_cast<T*>(p.v_ring) + ring_bh;
    const T* kp = static_cast<const T*>(p.k_pers) + (long long)h * p.np * DH;
    const T* vp = static_cast<const T*>(p.v_pers) + (long long)h * p.np * DH;

    // 1. the new token's key and value go into their slot first
    if (tid < 2 * LPK) {
        const int c = tid % LPK;
        const bool is_v = tid >= LPK;
        const T* src = static_cast<const T*>(is_v ? p.v_new : p.k_new) + b * p.ns[0] + h * p.ns[1] + c * 8;
        T* dst = (is_v ? vr : kr) + (long long)slot_new * DH + c * 8;
        float tmp[8];
        load8<T>(src, tmp);
        store8<T>(dst, tmp);
    }
    float qreg[8];
    load8<T>(static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + sub * 8, qreg);
    __syncthreads();  // the slot written above is read below by other threads of this CTA

    float m = -CUDART_INF_F, l = 0.f;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int n_keys = p.np + count;

    for (int i0 = 0; i0 < n_keys; i0 += STEP * UNROLL) {
        float kf[UNROLL][8], vf[UNROLL][8];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int i = i0 + u * STEP + warp * RPW + grp;
            ok[u] = i < n_keys;
            const int ii = ok[u] ? i : 0;
            const T* ksrc = ii < p.np ? kp + (long long)ii * DH : kr + (long long)(ii - p.np) * DH;
            const T* vsrc = ii < p.np ? vp + (long long)ii * DH : vr + (long long)(ii - p.np) * DH;
            if (ok[u]) {
                load8<T>(ksrc + sub * 8, kf[u]);
                load8<T>(vsrc + sub * 8, vf[u]);
            }
        }
        float s[UNROLL];
        float tmax = -CUDART_INF_F;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float part = 0.f;
            if (ok[u]) {
#pragma unroll
                for (int e = 0; e < 8; ++e) part = fmaf(qreg[e], kf[u][e], part);
            }
#pragma unroll
            for (int off = 1; off < LPK; off <<= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
            s[u] = ok[u] ? part * p.scale_log2 : -CUDART_INF_F;
            tmax = fmaxf(tmax, s[u]);
        }
        if (tmax > -CUDART_INF_F) {
            const float m_new = fmaxf(m, tmax);
            const float alpha = exp2f(m - m_new);
            m = m_new;
            l *= alpha;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] *= alpha;
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (ok[u]) {
                    const float pj = exp2f(s[u] - m);
                    l += pj;
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(pj, vf[u][e], acc[e]);
                }
            }
        }
    }

    // 2. merge the RPW lane groups of the warp (lanes that hold the same slice)
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
        const float m_o = __shfl_xor_sync(0xffffffffu, m, off);
        const float l_o = __shfl_xor_sync(0xffffffffu, l, off);
        const float m_new = fmaxf(m, m_o);
        const float a = m_new > -CUDART_INF_F ? exp2f(m - m_new) : 0.f;
        const float a_o = m_new > -CUDART_INF_F ? exp2f(m_o - m_new) : 0.f;
        l = l * a + l_o * a_o;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float acc_o = __shfl_xor_sync(0xffffffffu, acc[e], off);
            acc[e] = acc[e] * a + acc_o * a_o;
        }
        m = m_new;
    }

    // 3. merge the warps through shared memory
    __shared__ float sm_m[kDecodeWarps], sm_l[kDecodeWarps];
    __shared__ float sm_acc[kDecodeWarps][DH];
    if (grp == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) sm_acc[warp][sub * 8 + e] = acc[e];
        if (sub == 0) {
            sm_m[warp] = m;
            sm_l[warp] = l;
        }
    }
    __syncthreads();
    if (tid < LPK) {
        float m_all = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) m_all = fmaxf(m_all, sm_m[w]);
        float l_all = 0.f;
        float out[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float a = sm_m[w] > -CUDART_INF_F ? exp2f(sm_m[w] - m_all) : 0.f;
            l_all += sm_l[w] * a;
#pragma unroll
            for (int e = 0; e < 8; ++e) out[e] += sm_acc[w][tid * 8 + e] * a;
        }
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] *= inv;
        store8<T>(static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1] + tid * 8, out);
    }
}

struct FillParams {
    void* k_ring;
    void* v_ring;
    const void* k;
    const void* v;
    long long ks[3], vs[3];
    int heads, slots, dh, rows, first_row, t0;
};

// One thread per 8-element chunk of a kept row; rows [first_row, rows) are kept.
template <typename T>
__global__ void cache_fill_kernel(const FillParams p) {
    const int h = blockIdx.y, b = blockIdx.z;
    const int chunks_per_row = p.dh / 8;
    const int n = (p.rows - p.first_row) * chunks_per_row;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n; c += gridDim.x * blockDim.x) {
        const int i = p.first_row + c / chunks_per_row;
        const int col = (c % chunks_per_row) * 8;
        const int slot = (p.t0 + i) % p.slots;
        const long long dst = (((long long)b * p.heads + h) * p.slots + slot) * p.dh + col;
        float tmp[8];
        load8<T>(static_cast<const T*>(p.k) + b * p.ks[0] + h * p.ks[1] + (long long)i * p.ks[2] + col, tmp);
        store8<T>(static_cast<T*>(p.k_ring) + dst, tmp);
        load8<T>(static_cast<const T*>(p.v) + b * p.vs[0] + h * p.vs[1] + (long long)i * p.vs[2] + col, tmp);
        store8<T>(static_cast<T*>(p.v_ring) + dst, tmp);
    }
}

template <typename T>
int launch_decode_dh(const DecodeParams& p, int batch, int heads, int dh, cudaStream_t stream) {
    dim3 grid(heads, batch);
    switch (dh) {
        case 8: decode_kernel<T, 8><<<grid, kDecodeThreads, 0, stream>>>(p); break;
        case 16: decode_kernel<T, 16><<<grid, kDecodeThreads, 0, stream>>>(p); break;
        case 32: decode_kernel<T, 32><<<grid, kDecodeThreads, 0, stream>>>(p); break;
        case 64: decode_kernel<T, 64><<<grid, kDecodeThreads, 0, stream>>>(p); break;
        case 128: decode_kernel<T, 128><<<grid, kDecodeThreads, 0, stream>>>(p); break;
        case 256: decode_kernel<T, 256><<<grid, kDecodeThreads, 0, stream>>>(p); break;
        default: return TMW_ERR_UNSUPPORTED;
    }
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

}  // namespace

int launch_decode(const tmw_cache_desc& c, const void* q, const void* k_new, const void* v_new, void* o,
                  const int64_t qs[2], const int64_t ns[2], const int64_t os[2], const int32_t* pos,
                  cudaStream_t stream) {
    if (c.batch == 0 || c.heads == 0) return TMW_OK;
    if (c.batch > 65535) return TMW_ERR_TOO_LARGE;
    DecodeParams p;
    p.k_ring = c.k_ring; p.v_ring = c.v_ring; p.k_pers = c.k_pers; p.v_pers = c.v_pers;
    p.q = q; p.k_new = k_new; p.v_new = v_new; p.o = o; p.pos = pos;
    for (int i = 0; i < 2; ++i) { p.qs[i] = qs[i]; p.ns[i] = ns[i]; p.os[i] = os[i]; }
    p.heads = c.heads; p.slots = c.window + 1; p.np = c.n_persistent;
    const float scale = c.scale != 0.f ? c.scale : 1.0f / sqrtf((float)c.head_dim);
    p.scale_log2 = scale * 1.4426950408889634f;
    switch (c.dtype) {
        case TMW_F32: return launch_decode_dh<float>(p, c.batch, c.heads, c.head_dim, stream);
        case TMW_BF16: return launch_decode_dh<__nv_bfloat16>(p, c.batch, c.heads, c.head_dim, stream);
        case TMW_F16: return launch_decode_dh<__half>(p, c.batch, c.heads, c.head_dim, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

int launch_cache_fill(const tmw_cache_desc& c, const void* k, const void* v, const int64_t ks[3],
                      const int64_t vs[3], int rows, int t0, cudaStream_t stream) {
    if (c.batch == 0 || c.heads == 0 || rows == 0) return TMW_OK;
    if (c.batch > 65535 || c.heads > 65535) return TMW_ERR_TOO_LARGE;
    FillParams p;
    p.k_ring = c.k_ring; p.v_ring = c.v_ring; p.k = k; p.v = v;
    for (int i = 0; i < 3; ++i) { p.ks[i] = ks[i]; p.vs[i] = vs[i]; }
    p.heads = c.heads; p.slots = c.window + 1; p.dh = c.head_dim; p.rows = rows;
    p.first_row = rows > p.slots ? rows - p.slots : 0;
    p.t0 = t0;
    const int n = (rows - p.first_row) * (c.head_dim / 8);
    dim3 grid((n + 255) / 256, c.heads, c.batch);
    switch (c.dtype) {
        case TMW_F32: cache_fill_kernel<float><<<grid, 256, 0, stream>>>(p); break;
        case TMW_BF16: cache_fill_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p); break;
        case TMW_F16: cache_fill_kernel<__half><<<grid, 256, 0, stream>>>(p); break;
        default: return TMW_ERR_UNSUPPORTED;
    }
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

}  // namespace tmw
