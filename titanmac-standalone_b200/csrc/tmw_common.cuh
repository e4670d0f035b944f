// Shared declarations of libtmw's translation units (internal; the public ABI is
// include/tmw.h).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "tmw.h"

namespace tmw {

// ---- element conversion ---------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Loads 8 consecutive elements (16 B for 16-bit types, 32 B for float) as floats.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&out)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&out)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&out)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
    }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&in)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&in)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(in[4], in[5], in[6], in[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&in)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&in)[8]) {
    uint4 raw;
    __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

__host__ __device__ inline size_t dtype_size(int dtype) { return dtype == TMW_F32 ? 4 : 2; }

// Position of the first sequence key that the sequence query at position `pos` (>= np) sees.
// block == 0: the query and its `window` predecessors (WindowedAttention, windowed_attention.py:136-150).
// block  > 0: the left edge moves in steps of `block` rows - the query in block b of the sequence sees the
//             keys from b * block - window on (BlockSparseAttention, block_sparse_attention.py:299-311).
__host__ __device__ inline int first_visible_pos(int pos, int np, int window, int block) {
    if (block > 0) {
        const int lo = ((pos - np) / block) * block - window;
        return np + (lo > 0 ? lo : 0);
    }
    const int lo = pos - window;
    return lo > np ? lo : np;
}

// ---- host-side plumbing shared by the entry points ---------------------------------
void set_cuda_error(cudaError_t e, const char* where);
void set_error_text(const char* text);
int* device_status_word();  // per-device int in global memory, 0 = fine
// opt-in of a kernel to `bytes` of dynamic shared memory, made once per kernel and device
int allow_shared_memory(const void* kern, int bytes);

// a library-owned stream for work that may overlap the caller's stream, with the events of the fork / join
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    std::mutex mutex;
};
SideStream* side_stream_of_current_device();  // nullptr if it cannot be made

#define TMW_CUDA_TRY(expr)                                   \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) {                             \
            ::tmw::set_cuda_error(_e, #expr);                \
            return TMW_ERR_CUDA;                             \
        }                                                    \
    } while (0)

// Argument checks shared by the decode entry points (defined with the entry points in api.cu).
int validate_decode_call(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new,
                         const void* o, const int64_t q_stride[2], const int64_t kv_new_stride[2],
                         const int64_t o_stride[2], const int32_t* pos);

// Kernel launchers (one per translation unit).
// window_block: 0 = per-token window, > 0 = block-granular left edge (see first_visible_pos);
// all_keys: every query row of the call sees every key, unmasked (the persistent rows of the block-sparse class)
// lse (optional): [batch, heads, q_rows] fp32, log2 of every row's softmax denominator in the domain of
// score * scale * log2(e) - what the backward pass needs to rebuild the probabilities
int launch_prefill_simt(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, void* o,
                        cudaStream_t stream, int window_block = 0, bool all_keys = false, float* lse = nullptr);
int launch_prefill_tc(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, void* o,
                      cudaStream_t stream, int window_block = 0, bool all_keys = false, float* lse = nullptr,
                      const tmw_halo_wait* wait = nullptr);
// window_block / pers_global select the mask of the block-sparse class (see first_visible_pos; pers_global: the
// persistent query rows see every key, and lse comes as [batch, heads, rows - np] followed by [batch, heads, np])
int launch_prefill_backward(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o,
                            const void* d_o, const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream,
                            int window_block = 0, bool pers_global = false);
// the same on the warp-level tensor-core path (16-bit types, head_dim 64 / 128)
bool prefill_backward_mma_supports(const tmw_prefill_desc& d);
int launch_prefill_backward_mma(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o,
                                const void* d_o, const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream,
                                int window_block = 0, bool pers_global = false);
// the same on tcgen05 (16-bit types, head_dim 64 / 128); window_block > 0: the block-sparse class's mask with its
// persistent query rows seeing every key and lse in two planes
bool prefill_backward_tc_supports(const tmw_prefill_desc& d);
int launch_prefill_backward_tc(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o,
                               const void* d_o, const float* lse, void* dq, void* dk, void* dv, cudaStream_t stream,
                               int window_block = 0);
bool prefill_tc_supports(const tmw_prefill_desc& d, const void* q, const void* k, const void* v, const void* o);
int launch_decode(const tmw_cache_desc& c, const void* q, const void* k_new, const void* v_new, void* o,
                  const int64_t qs[2], const int64_t ns[2], const int64_t os[2], const int32_t* pos,
                  int splits, float* scratch, unsigned int* counters, cudaStream_t stream);

// layout of the split-decode scratch memory: partial results, then (16-byte aligned) one counter per pair
inline size_t decode_partials_bytes(int batch, int heads, int head_dim, int splits) {
    const size_t n = (size_t)batch * heads * splits * ((size_t)head_dim + 2) * sizeof(float);
    return (n + 15) & ~(size_t)15;
}
int launch_linear(const tmw_linear_desc& d, const void* a, const void* w, const void* bias, void* c,
                  cudaStream_t stream);
int launch_cache_fill(const tmw_cache_desc& c, const void* k, const void* v, const int64_t ks[3],
                      const int64_t vs[3], int rows, int t0, cudaStream_t stream);

}  // namespace tmw
