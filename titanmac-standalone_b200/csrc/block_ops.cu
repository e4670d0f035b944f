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

// NV = 8-element vectors per lane kept in registers; NV == 0: the row is read again for the second pass
// (it comes out of L1/L2: the same warp has just read or written it).
template <typename T, int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
add_rmsnorm_kernel(const T* x, const T* __restrict__ res, const T* __restrict__ scale, float eps,
                   T* sum_out, T* __restrict__ y, long long rows, int dim) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
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
    const float rms = sqrtf(ss / (float)dim + eps);  // same operation order as the reference: x / rms * scale

    auto emit = [&](int v, const float (&h)[8]) {
        float g[8], out[8];
        load8<T>(scale + v * 8, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = h[i] / rms * g[i];
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
}

template <typename T>
int launch_add_rmsnorm(long long rows, int dim, const void* x, const void* res, const void* scale, float eps,
                       void* sum_out, void* y, cudaStream_t stream) {
    const unsigned blocks = (unsigned)((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const int nv = (dim / 8 + 31) / 32;
#define TMW_NORM_CASE(N)                                                                                     \
    add_rmsnorm_kernel<T, N><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(                                    \
        static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(scale), eps,            \
        static_cast<T*>(sum_out), static_cast<T*>(y), rows, dim)
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

}  // namespace
}  // namespace tmw

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
    if ((rows + kWarpsPerBlock - 1) / kWarpsPerBlock > 0x7fffffffLL) return TMW_ERR_TOO_LARGE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TMW_F32: return launch_add_rmsnorm<float>(rows, dim, x, residual, scale, eps, sum_out, y, s);
        case TMW_BF16: return launch_add_rmsnorm<__nv_bfloat16>(rows, dim, x, residual, scale, eps, sum_out, y, s);
        default: return launch_add_rmsnorm<__half>(rows, dim, x, residual, scale, eps, sum_out, y, s);
    }
}
