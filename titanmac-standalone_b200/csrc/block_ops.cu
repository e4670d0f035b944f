// Element-wise kernels around the attention call (all HBM-bound, 16-byte accesses).
//
// Residual add + RMSNorm in one pass over the rows: the element-wise work that surrounds the
// attention module in a TitanBlock (titans_core/blocks/titan_block.py:92-100 of the reference,
// norm formula titans_core/blocks/norms.py:55-58).  In PyTorch the residual add and the norm are
// seven small kernels and as many trips through HBM; here a row is read once, the sum is stored
// (it is the new residual stream) and the normalised row is written.  HBM-bound: one warp per row,
// 16-byte accesses, the row stays in registers between the two passes when it is short enough.
#include "tmw_common.cuh"

namespace tmw {
namespace {

constexpr int kWarpsPerBlock = 8;

// CTAs of `kernel` that fit on the whole GPU at once (the grid of a kernel whose threads loop over the work)
template <typename K>
int resident_ctas(K kernel, int threads) {
    int sms = 148, dev = 0, per_sm = 1;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    return sms * per_sm;
}

// NV = 8-element vectors per lane kept in registers; NV == 0: the row is read again for the second pass
// (it comes out of L1/L2: the same warp has just read or written it).
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
add_rmsnorm_kernel(const T* x, const T* __restrict__ res, const T* __restrict__ scale, float eps,
                   T* sum_out, T* __restrict__ y, long long rows, int dim) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * kWarpsPerBlock;
    // a resident grid: every warp walks over rows (a block that lives for one row per warp spends most of
    // its life being scheduled)
    for (long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); row < rows; row += warps) {
    const T* xr = x + row * dim;
    const T* rr = res != nullptr ? res + row * dim : nullptr;
    T* sr = sum_out != nullptr ? sum_out + row * dim : nullptr;
    T* yr = y + row * dim;
    const int nvec = dim / 8;

    // h = x + residual, rounded to the storage type like the reference's `x + f(x)`; the norm is taken of
    // the rounded values, in fp32
    auto load_h = [&](int v, float (&h)[8]) {
        load8<T>(xr + v * 8, h);
        if (rr != nullptr) {
            float r[8];
            load8<T>(rr + v * 8, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = to_f32<T>(from_f32<T>(h[i] + r[i]));
        }
    };

    float keep[NV > 0 ? NV : 1][8];
    float ss = 0.f;
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int v = lane + j * 32;
            if (v < nvec) {
                load_h(v, keep[j]);
                if (sr != nullptr && rr != nullptr) store8<T>(sr + v * 8, keep[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(keep[j][i], keep[j][i], ss);
            }
        }
    } else {
        for (int v = lane; v < nvec; v += 32) {
            float h[8];
            load_h(v, h);
            if (sr != nullptr && rr != nullptr) store8<T>(sr + v * 8, h);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(h[i], h[i], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    // the reference computes x / rms * scale; multiplying by the reciprocal differs by at most one fp32 ulp
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);

    auto emit = [&](int v, const float (&h)[8]) {
        float g[8], out[8];
        load8<T>(scale + v * 8, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = h[i] * inv * g[i];
        store8<T>(yr + v * 8, out);
    };
    if (NV > 0) {
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int v = lane + j * 32;
            if (v < nvec) emit(v, keep[j]);
        }
    } else {
        for (int v = lane; v < nvec; v += 32) {
            float h[8];
            if (sr != nullptr && rr != nullptr) load8<T>(sr + v * 8, h); else load_h(v, h);
            emit(v, h);
        }
    }
    }  // rows
}

template <typename T>
int launch_add_rmsnorm(long long rows, int dim, const void* x, const void* res, const void* scale, float eps,
                       void* sum_out, void* y, cudaStream_t stream) {
    const long long want = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int nv = (dim / 8 + 31) / 32;
    // one resident wave: every warp walks over its rows, nothing waits for a slot
#define TMW_NORM_CASE(N)                                                                                     \
    {                                                                                                        \
        static int wave = 0;                                                                                 \
        if (wave == 0) wave = resident_ctas(add_rmsnorm_kernel<T, N>, kWarpsPerBlock * 32);                  \
        const unsigned blocks = (unsigned)(want < wave ? want : wave);                                       \
        add_rmsnorm_kernel<T, N><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(                                \
            static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(scale), eps,        \
            static_cast<T*>(sum_out), static_cast<T*>(y), rows, dim);                                        \
    }
    switch (nv) {
        case 1: TMW_NORM_CASE(1); break;
        case 2: TMW_NORM_CASE(2); break;
        case 3: TMW_NORM_CASE(3); break;
        case 4: TMW_NORM_CASE(4); break;
        default: TMW_NORM_CASE(0); break;
    }
#undef TMW_NORM_CASE
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

// ---- exact GELU --------------------------------------------------------------------------------------
// 0.5 x (1 + erf(x / sqrt 2)), the default nn.GELU() of the reference's MLP (titans_core/blocks/mlp.py:58-65).
// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7, below fp32 rounding of the result): a reciprocal,
// five multiply-adds and one exp2 instead of the branchy library erff, so that the kernel stays bound by
// HBM (one read, one write) and not by arithmetic.
__device__ __forceinline__ float gelu_erf(float x) {
    const float z = fabsf(x) * 0.70710678118654752f;
    const float t = __fdividef(1.0f, fmaf(0.3275911f, z, 1.0f));
    float poly = fmaf(1.061405429f, t, -1.453152027f);
    poly = fmaf(poly, t, 1.421413741f);
    poly = fmaf(poly, t, -0.284496736f);
    poly = fmaf(poly, t, 0.254829592f);
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z * z * 1.4426950408889634f));
    const float erfc_z = poly * t * e;  // 1 - erf(z), z >= 0
    const float erf_abs = 1.0f - erfc_z;
    return 0.5f * x * (1.0f + copysignf(erf_abs, x));
}

constexpr int kGeluUnroll = 4;  // 16-byte loads in flight per thread

template <typename T>
__global__ void __launch_bounds__(256) gelu_kernel(const T* x, T* y, long long nvec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * kGeluUnroll) {
        float a[kGeluUnroll][8];
#pragma unroll
        for (int u = 0; u < kGeluUnroll; ++u)
            if (v0 + u * stride < nvec) load8<T>(x + (v0 + u * stride) * 8, a[u]);
#pragma unroll
        for (int u = 0; u < kGeluUnroll; ++u)
            if (v0 + u * stride < nvec) {
#pragma unroll
                for (int i = 0; i < 8; ++i) a[u][i] = gelu_erf(a[u][i]);
                store8<T>(y + (v0 + u * stride) * 8, a[u]);
            }
    }
}

template <typename T>
int launch_gelu(long long n, const void* x, void* y, cudaStream_t stream) {
    static int wave = 0;
    if (wave == 0) wave = resident_ctas(gelu_kernel<T>, 256);
    const long long nvec = n / 8;
    const long long want = (nvec + 256 * kGeluUnroll - 1) / (256 * kGeluUnroll);
    const unsigned blocks = (unsigned)(want < wave ? want : wave);
    gelu_kernel<T><<<blocks, 256, 0, stream>>>(static_cast<const T*>(x), static_cast<T*>(y), nvec);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

// ---- causal depthwise convolution along the rows ---------------------------------------------------------
// y[b, t, c] = sum_j w[c, j] * x[b, t - (TAPS-1) + j, c]: the Conv1d(groups = channels, padding = TAPS-1),
// trimmed to the input length, that the reference's block-sparse attention applies to Q, K and V
// (titans_core/attn/block_sparse_attention.py:77-92, 241-256).  One thread owns 8 adjacent channels and
// walks down a strip of rows with the last TAPS rows in registers: x is read once (plus TAPS-1 rows per
// strip), y written once.
constexpr int kConvStrip = 64;
constexpr int kConvThreads = 128;

template <typename T, int TAPS>
__global__ void __launch_bounds__(kConvThreads)
dwconv_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, int rows, int channels) {
    const int vec = blockIdx.x * kConvThreads + threadIdx.x;  // which group of 8 channels
    if (vec * 8 >= channels) return;
    const int t0 = blockIdx.y * kConvStrip;
    const int t1 = min(rows, t0 + kConvStrip);
    const long long base = (long long)blockIdx.z * rows * channels + vec * 8;
    float wr[TAPS][8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[j][c] = to_f32<T>(w[(long long)(vec * 8 + c) * TAPS + j]);
    float hist[TAPS][8];  // hist[j] = x[t - (TAPS-1) + j]
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {
        const int t = t0 - (TAPS - 1) + j;
        if (t >= 0) {
            load8<T>(x + base + (long long)t * channels, hist[j + 1]);
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) hist[j + 1][c] = 0.f;
        }
    }
    for (int t = t0; t < t1; ++t) {
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) hist[j][c] = hist[j + 1][c];
        load8<T>(x + base + (long long)t * channels, hist[TAPS - 1]);
        float out[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < TAPS; ++j) a = fmaf(wr[j][c], hist[j][c], a);
            out[c] = a;
        }
        store8<T>(y + base + (long long)t * channels, out);
    }
}

template <typename T, int TAPS>
int launch_dwconv_taps(int batch, int rows, int channels, const void* x, const void* w, void* y, cudaStream_t stream) {
    const dim3 grid((channels / 8 + kConvThreads - 1) / kConvThreads, (rows + kConvStrip - 1) / kConvStrip, batch);
    dwconv_kernel<T, TAPS><<<grid, kConvThreads, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(w),
                                                              static_cast<T*>(y), rows, channels);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

// Backward of the convolution.  dx[t] = sum_j w[j] dy[t + (TAPS-1) - j] looks ahead, so a thread walks its strip
// of rows from the bottom up with the TAPS rows dy[t .. t+TAPS-1] in registers.  dw[c][j] = sum over batch and rows
// of dy[t][c] x[t - (TAPS-1) + j][c]: a thread accumulates its strip's share and adds it to an fp32 buffer
// [channels, TAPS] (zero on entry) with atomics.
template <typename T, int TAPS>
__global__ void __launch_bounds__(kConvThreads)
dwconv_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy, T* __restrict__ dx,
                  float* __restrict__ dw, int rows, int channels) {
    const int vec = blockIdx.x * kConvThreads + threadIdx.x;
    if (vec * 8 >= channels) return;
    const int t0 = blockIdx.y * kConvStrip;
    const int t1 = min(rows, t0 + kConvStrip);
    const long long base = (long long)blockIdx.z * rows * channels + vec * 8;
    float wr[TAPS][8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wr[j][c] = to_f32<T>(w[(long long)(vec * 8 + c) * TAPS + j]);
    // ---- dx: bottom-up, ahead[m] = dy[t + m]
    float ahead[TAPS][8];
#pragma unroll
    for (int m = 0; m < TAPS - 1; ++m) {  // the state "before" row t1 - 1: dy[t1 + m]
        if (t1 + m < rows) {
            load8<T>(dy + base + (long long)(t1 + m) * channels, ahead[m]);
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) ahead[m][c] = 0.f;
        }
    }
    for (int t = t1 - 1; t >= t0; --t) {
#pragma unroll
        for (int m = TAPS - 1; m >= 1; --m)
#pragma unroll
            for (int c = 0; c < 8; ++c) ahead[m][c] = ahead[m - 1][c];
        load8<T>(dy + base + (long long)t * channels, ahead[0]);
        float out[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < TAPS; ++j) a = fmaf(wr[j][c], ahead[TAPS - 1 - j][c], a);
            out[c] = a;
        }
        store8<T>(dx + base + (long long)t * channels, out);
    }
    // ---- dw: top-down like the forward, hist[j] = x[t - (TAPS-1) + j]
    float hist[TAPS][8], acc[TAPS][8];
#pragma unroll
    for (int j = 0; j < TAPS; ++j)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[j][c] = 0.f;
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) {
        const int t = t0 - (TAPS - 1) + j;
        if (t >= 0) {
            load8<T>(x + base + (long long)t * channels, hist[j + 1]);
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) hist[j + 1][c] = 0.f;
        }
    }
    for (int t = t0; t < t1; ++t) {
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) hist[j][c] = hist[j + 1][c];
        load8<T>(x + base + (long long)t * channels, hist[TAPS - 1]);
        float g[8];
        load8<T>(dy + base + (long long)t * channels, g);
#pragma unroll
        for (int j = 0; j < TAPS; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[j][c] = fmaf(g[c], hist[j][c], acc[j][c]);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) atomicAdd(dw + (long long)(vec * 8 + c) * TAPS + j, acc[j][c]);
}

template <typename T, int TAPS>
int launch_dwconv_bwd_taps(int batch, int rows, int channels, const void* x, const void* w, const void* dy, void* dx,
                           float* dw, cudaStream_t stream) {
    const dim3 grid((channels / 8 + kConvThreads - 1) / kConvThreads, (rows + kConvStrip - 1) / kConvStrip, batch);
    dwconv_bwd_kernel<T, TAPS><<<grid, kConvThreads, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(w),
                                                                  static_cast<const T*>(dy), static_cast<T*>(dx), dw,
                                                                  rows, channels);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

template <typename T>
int launch_dwconv_bwd(int batch, int rows, int channels, int taps, const void* x, const void* w, const void* dy,
                      void* dx, float* dw, cudaStream_t stream) {
    switch (taps) {
        case 1: return launch_dwconv_bwd_taps<T, 1>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 2: return launch_dwconv_bwd_taps<T, 2>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 3: return launch_dwconv_bwd_taps<T, 3>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 4: return launch_dwconv_bwd_taps<T, 4>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 5: return launch_dwconv_bwd_taps<T, 5>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 6: return launch_dwconv_bwd_taps<T, 6>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 7: return launch_dwconv_bwd_taps<T, 7>(batch, rows, channels, x, w, dy, dx, dw, stream);
        case 8: return launch_dwconv_bwd_taps<T, 8>(batch, rows, channels, x, w, dy, dx, dw, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

template <typename T>
int launch_dwconv(int batch, int rows, int channels, int taps, const void* x, const void* w, void* y,
                  cudaStream_t stream) {
    switch (taps) {
        case 1: return launch_dwconv_taps<T, 1>(batch, rows, channels, x, w, y, stream);
        case 2: return launch_dwconv_taps<T, 2>(batch, rows, channels, x, w, y, stream);
        case 3: return launch_dwconv_taps<T, 3>(batch, rows, channels, x, w, y, stream);
        case 4: return launch_dwconv_taps<T, 4>(batch, rows, channels, x, w, y, stream);
        case 5: return launch_dwconv_taps<T, 5>(batch, rows, channels, x, w, y, stream);
        case 6: return launch_dwconv_taps<T, 6>(batch, rows, channels, x, w, y, stream);
        case 7: return launch_dwconv_taps<T, 7>(batch, rows, channels, x, w, y, stream);
        case 8: return launch_dwconv_taps<T, 8>(batch, rows, channels, x, w, y, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

}  // namespace
}  // namespace tmw

extern "C" int tmw_causal_dwconv(int32_t dtype, int32_t batch, int32_t rows, int32_t channels, int32_t taps,
                                 const void* x, const void* weight, void* y, void* stream) {
    using namespace tmw;
    if (batch < 0 || rows < 0 || channels <= 0) return TMW_ERR_INVALID_ARGUMENT;
    if (dtype != TMW_F32 && dtype != TMW_BF16 && dtype != TMW_F16) return TMW_ERR_INVALID_ARGUMENT;
    if (taps < 1 || taps > 8 || channels % 8 != 0) {
        set_error_text("tmw_causal_dwconv: 1 to 8 taps and a multiple of 8 channels");
        return TMW_ERR_UNSUPPORTED;
    }
    if (batch == 0 || rows == 0) return TMW_OK;
    if (x == nullptr || weight == nullptr || y == nullptr || x == y) return TMW_ERR_INVALID_ARGUMENT;
    if ((((uintptr_t)x | (uintptr_t)y) & 15) != 0) {
        set_error_text("tmw_causal_dwconv: x and y must be 16-byte aligned");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (batch > 65535 || (rows + kConvStrip - 1) / kConvStrip > 65535) return TMW_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TMW_F32: return launch_dwconv<float>(batch, rows, channels, taps, x, weight, y, s);
        case TMW_BF16: return launch_dwconv<__nv_bfloat16>(batch, rows, channels, taps, x, weight, y, s);
        default: return launch_dwconv<__half>(batch, rows, channels, taps, x, weight, y, s);
    }
}

extern "C" int tmw_causal_dwconv_backward(int32_t dtype, int32_t batch, int32_t rows, int32_t channels, int32_t taps,
                                          const void* x, const void* weight, const void* dy, void* dx, float* dw,
                                          void* stream) {
    using namespace tmw;
    if (batch < 0 || rows < 0 || channels <= 0) return TMW_ERR_INVALID_ARGUMENT;
    if (dtype != TMW_F32 && dtype != TMW_BF16 && dtype != TMW_F16) return TMW_ERR_INVALID_ARGUMENT;
    if (taps < 1 || taps > 8 || channels % 8 != 0) return TMW_ERR_UNSUPPORTED;
    if (batch == 0 || rows == 0) return TMW_OK;
    if (x == nullptr || weight == nullptr || dy == nullptr || dx == nullptr || dw == nullptr || dx == dy)
        return TMW_ERR_INVALID_ARGUMENT;
    if ((((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) & 15) != 0) return TMW_ERR_INVALID_ARGUMENT;
    if (batch > 65535 || (rows + kConvStrip - 1) / kConvStrip > 65535) return TMW_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TMW_F32: return launch_dwconv_bwd<float>(batch, rows, channels, taps, x, weight, dy, dx, dw, s);
        case TMW_BF16: return launch_dwconv_bwd<__nv_bfloat16>(batch, rows, channels, taps, x, weight, dy, dx, dw, s);
        default: return launch_dwconv_bwd<__half>(batch, rows, channels, taps, x, weight, dy, dx, dw, s);
    }
}

extern "C" int tmw_gelu(int32_t dtype, int64_t n, const void* x, void* y, void* stream) {
    using namespace tmw;
    if (n < 0 || (n > 0 && (x == nullptr || y == nullptr))) {
        set_error_text("tmw_gelu: null pointer or negative size");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (dtype != TMW_F32 && dtype != TMW_BF16 && dtype != TMW_F16) return TMW_ERR_INVALID_ARGUMENT;
    if (n % 8 != 0) {
        set_error_text("tmw_gelu: the element count must be a multiple of 8");
        return TMW_ERR_UNSUPPORTED;
    }
    if ((((uintptr_t)x | (uintptr_t)y) & 15) != 0) {
        set_error_text("tmw_gelu: both pointers must be 16-byte aligned");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (n == 0) return TMW_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TMW_F32: return launch_gelu<float>(n, x, y, s);
        case TMW_BF16: return launch_gelu<__nv_bfloat16>(n, x, y, s);
        default: return launch_gelu<__half>(n, x, y, s);
    }
}

extern "C" int tmw_add_rmsnorm(int32_t dtype, int64_t rows, int32_t dim, const void* x, const void* residual,
                               const void* scale, float eps, void* sum_out, void* y, void* stream) {
    using namespace tmw;
    if (rows < 0 || dim <= 0 || x == nullptr || scale == nullptr || y == nullptr || !(eps >= 0.f)) {
        set_error_text("tmw_add_rmsnorm: null pointer, negative size or negative eps");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (dtype != TMW_F32 && dtype != TMW_BF16 && dtype != TMW_F16) return TMW_ERR_INVALID_ARGUMENT;
    if (dim % 8 != 0) {
        set_error_text("tmw_add_rmsnorm: the row length must be a multiple of 8");
        return TMW_ERR_UNSUPPORTED;
    }
    const uintptr_t all = (uintptr_t)x | (uintptr_t)residual | (uintptr_t)scale | (uintptr_t)sum_out | (uintptr_t)y;
    if (all % 16 != 0) {
        set_error_text("tmw_add_rmsnorm: every pointer must be 16-byte aligned");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (rows == 0) return TMW_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TMW_F32: return launch_add_rmsnorm<float>(rows, dim, x, residual, scale, eps, sum_out, y, s);
        case TMW_BF16: return launch_add_rmsnorm<__nv_bfloat16>(rows, dim, x, residual, scale, eps, sum_out, y, s);
        default: return launch_add_rmsnorm<__half>(rows, dim, x, residual, scale, eps, sum_out, y, s);
    }
}
