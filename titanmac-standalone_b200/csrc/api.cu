// C-ABI entry points of libtmw: argument validation, kernel selection, error text.
// Everything that can be rejected is rejected here, on the host, before a launch.
#include <atomic>
#include <cstdio>
#include <mutex>
#include <cstring>

#include "tmw_common.cuh"

namespace tmw {

static thread_local char g_error_text[256] = "";

void set_error_text(const char* text) {
    std::snprintf(g_error_text, sizeof(g_error_text), "%s", text);
}

void set_cuda_error(cudaError_t e, const char* where) {
    std::snprintf(g_error_text, sizeof(g_error_text), "%s: %s (%s)", cudaGetErrorName(e), cudaGetErrorString(e),
                  where);
}

// One status word per device: a __device__ variable is instantiated in every
// context that loads this module.
__device__ int g_device_status[4] = {0, 0, 0, 0};  // [0] status, [1..3] where the first expired wait was

int* device_status_word() {
    constexpr int kMaxDevices = 64;
    // written once per device; two host threads making the first call on a device store the same value
    static std::atomic<int*> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (cache[dev].load(std::memory_order_acquire) == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
        cache[dev].store(static_cast<int*>(ptr), std::memory_order_release);
    }
    return cache[dev].load(std::memory_order_acquire);
}

// One side stream and two events per device, made on first use and kept for the life of the process (make
// that first use outside stream capture).  Calls that use them are serialised on the host by `mutex`.
SideStream* side_stream_of_current_device() {
    constexpr int kMaxDevices = 64;
    static SideStream table[kMaxDevices];
    static bool ready[kMaxDevices] = {false};
    static std::mutex init;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(init);
    if (!ready[dev]) {
        SideStream& t = table[dev];
        if (cudaStreamCreateWithFlags(&t.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&t.join, cudaEventDisableTiming) != cudaSuccess)
            return nullptr;
        ready[dev] = true;
    }
    return &table[dev];
}

// the opt-in to more than 48 KB of dynamic shared memory is per kernel and per device: made once
int allow_shared_memory(const void* kern, int bytes) {
    constexpr int kMaxDevices = 64, kMaxKernels = 32;
    struct Entry { const void* kern; int allowed[kMaxDevices]; };
    static std::mutex mutex;
    static Entry table[kMaxKernels] = {};
    int dev = 0;
    TMW_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mutex);
    Entry* e = nullptr;
    for (int i = 0; i < kMaxKernels && e == nullptr; ++i) {
        if (table[i].kern == kern) e = &table[i];
        else if (table[i].kern == nullptr) { table[i].kern = kern; e = &table[i]; }
    }
    if (e == nullptr || dev < 0 || dev >= kMaxDevices || e->allowed[dev] < bytes) {
        TMW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        if (e != nullptr && dev >= 0 && dev < kMaxDevices) e->allowed[dev] = bytes;
    }
    return TMW_OK;
}

namespace {

bool dtype_ok(int dtype) { return dtype == TMW_F32 || dtype == TMW_BF16 || dtype == TMW_F16; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool strides_ok(const int64_t* s, int n, int dtype) {
    const int64_t unit = 16 / (int64_t)dtype_size(dtype);  // elements per 16 bytes
    for (int i = 0; i < n; ++i)
        if (s[i] < 0 || s[i] % unit != 0) return false;
    return true;
}

int validate_prefill(const tmw_prefill_desc* d, const void* q, const void* k, const void* v, const void* o) {
    if (d == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (!dtype_ok(d->dtype)) return TMW_ERR_UNSUPPORTED;
    if (d->algo < TMW_ALGO_AUTO || d->algo > TMW_ALGO_MMA) return TMW_ERR_INVALID_ARGUMENT;
    if (d->batch < 0 || d->heads < 0 || d->head_dim <= 0 || d->q_rows < 0 || d->k_rows < 0 ||
        d->n_persistent < 0 || d->q_pos0 < 0)
        return TMW_ERR_INVALID_ARGUMENT;
    if (d->window < 0) return TMW_ERR_NEGATIVE_WINDOW;
    if (d->k_rows <= d->n_persistent) return TMW_ERR_PERSISTENT_GE_LEN;
    if (d->k_pos0 < d->n_persistent) return TMW_ERR_INVALID_ARGUMENT;
    if (!(d->scale >= 0.f)) return TMW_ERR_INVALID_ARGUMENT;
    if (d->batch == 0 || d->heads == 0 || d->q_rows == 0) return TMW_OK;
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return TMW_ERR_INVALID_ARGUMENT;
    if (!strides_ok(d->q_stride, 3, d->dtype) || !strides_ok(d->k_stride, 3, d->dtype) ||
        !strides_ok(d->v_stride, 3, d->dtype) || !strides_ok(d->o_stride, 3, d->dtype))
        return TMW_ERR_INVALID_ARGUMENT;
    // every sequence query must find its window inside the K/V buffers
    const int64_t np = d->n_persistent;
    const int64_t p_last = (int64_t)d->q_pos0 + d->q_rows - 1;
    if (p_last >= np) {
        const int64_t p_first = d->q_pos0 > np ? d->q_pos0 : np;
        const int64_t g_lo = p_first - d->window > np ? p_first - d->window : np;
        const int64_t k_last = (int64_t)d->k_pos0 + (d->k_rows - np) - 1;
        if (g_lo < d->k_pos0 || p_last > k_last) return TMW_ERR_KEY_RANGE;
    }
    return TMW_OK;
}

int validate_cache(const tmw_cache_desc* c) {
    if (c == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (!dtype_ok(c->dtype)) return TMW_ERR_UNSUPPORTED;
    if (c->batch < 0 || c->heads < 0 || c->head_dim <= 0 || c->n_persistent < 0) return TMW_ERR_INVALID_ARGUMENT;
    if (c->window < 0) return TMW_ERR_NEGATIVE_WINDOW;
    const int dh = c->head_dim;
    if (!(dh == 8 || dh == 16 || dh == 32 || dh == 64 || dh == 128 || dh == 256)) return TMW_ERR_UNSUPPORTED;
    if (!(c->scale >= 0.f)) return TMW_ERR_INVALID_ARGUMENT;
    if (c->batch == 0 || c->heads == 0) return TMW_OK;
    if (c->k_ring == nullptr || c->v_ring == nullptr || !aligned16(c->k_ring) || !aligned16(c->v_ring))
        return TMW_ERR_INVALID_ARGUMENT;
    if (c->n_persistent > 0 &&
        (c->k_pers == nullptr || c->v_pers == nullptr || !aligned16(c->k_pers) || !aligned16(c->v_pers)))
        return TMW_ERR_INVALID_ARGUMENT;
    return TMW_OK;
}

}  // namespace

// Checks shared by every decode entry point (everything except the scratch memory).
int validate_decode_call(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new,
                         const void* o, const int64_t q_stride[2], const int64_t kv_new_stride[2],
                         const int64_t o_stride[2], const int32_t* pos) {
    const int rc = validate_cache(cache);
    if (rc != TMW_OK) return rc;
    if (q_stride == nullptr || kv_new_stride == nullptr || o_stride == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (cache->batch == 0 || cache->heads == 0) return TMW_OK;
    if (q == nullptr || k_new == nullptr || v_new == nullptr || o == nullptr || pos == nullptr)
        return TMW_ERR_INVALID_ARGUMENT;
    if (!aligned16(q) || !aligned16(k_new) || !aligned16(v_new) || !aligned16(o)) return TMW_ERR_INVALID_ARGUMENT;
    if (!strides_ok(q_stride, 2, cache->dtype) || !strides_ok(kv_new_stride, 2, cache->dtype) ||
        !strides_ok(o_stride, 2, cache->dtype))
        return TMW_ERR_INVALID_ARGUMENT;
    return TMW_OK;
}

}  // namespace tmw

extern "C" {

int tmw_version(void) { return TMW_VERSION; }

const char* tmw_strerror(int status) {
    switch (status) {
        case TMW_OK: return "ok";
        case TMW_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, negative size, stride or alignment)";
        case TMW_ERR_UNSUPPORTED: return "unsupported dtype / head_dim / algorithm";
        case TMW_ERR_PERSISTENT_GE_LEN: return "n_persistent must be < length";
        case TMW_ERR_NEGATIVE_WINDOW: return "window must be non-negative";
        case TMW_ERR_KEY_RANGE: return "a query's window reaches outside the key/value buffers";
        case TMW_ERR_CUDA: return "CUDA call failed";
        case TMW_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
        case TMW_ERR_TOO_LARGE: return "size exceeds a fixed capacity of this entry point";
        default: return "unknown status";
    }
}

const char* tmw_last_cuda_error(void) { return tmw::g_error_text; }

int tmw_prefill(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, void* o,
                void* stream) {
    const int rc = tmw::validate_prefill(desc, q, k, v, o);
    if (rc != TMW_OK) return rc;
    if (desc->batch == 0 || desc->heads == 0 || desc->q_rows == 0) return TMW_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (desc->algo == TMW_ALGO_MMA) return TMW_ERR_UNSUPPORTED;  // a backward-only choice
    const bool tc_ok = tmw::prefill_tc_supports(*desc, q, k, v, o);
    if (desc->algo == TMW_ALGO_TCGEN05) {
        if (!tc_ok) return TMW_ERR_UNSUPPORTED;
        return tmw::launch_prefill_tc(*desc, q, k, v, o, s);
    }
    if (desc->algo == TMW_ALGO_AUTO && tc_ok) return tmw::launch_prefill_tc(*desc, q, k, v, o, s);
    return tmw::launch_prefill_simt(*desc, q, k, v, o, s);
}

int tmw_prefill_halo(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, void* o,
                     const tmw_halo_wait* wait, void* stream) {
    const int rc = tmw::validate_prefill(desc, q, k, v, o);
    if (rc != TMW_OK) return rc;
    if (wait == nullptr || wait->halo_rows < 0 || wait->halo_rows > desc->k_rows - desc->n_persistent)
        return TMW_ERR_INVALID_ARGUMENT;
    if (desc->batch == 0 || desc->heads == 0 || desc->q_rows == 0) return TMW_OK;
    if (desc->algo == TMW_ALGO_SIMT || !tmw::prefill_tc_supports(*desc, q, k, v, o)) {
        tmw::set_error_text("tmw_prefill_halo: only the tensor-core kernel polls the flags (bf16 / f16, head_dim 64 or 128)");
        return TMW_ERR_UNSUPPORTED;
    }
    return tmw::launch_prefill_tc(*desc, q, k, v, o, static_cast<cudaStream_t>(stream), 0, false, nullptr, wait);
}

int tmw_prefill_lse(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, void* o, float* lse,
                    void* stream) {
    const int rc = tmw::validate_prefill(desc, q, k, v, o);
    if (rc != TMW_OK) return rc;
    if (desc->batch == 0 || desc->heads == 0 || desc->q_rows == 0) return TMW_OK;
    if (lse == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool tc_ok = tmw::prefill_tc_supports(*desc, q, k, v, o);
    if (desc->algo == TMW_ALGO_TCGEN05 && !tc_ok) return TMW_ERR_UNSUPPORTED;
    if (desc->algo != TMW_ALGO_SIMT && tc_ok) return tmw::launch_prefill_tc(*desc, q, k, v, o, s, 0, false, lse);
    return tmw::launch_prefill_simt(*desc, q, k, v, o, s, 0, false, lse);
}

int tmw_prefill_backward(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, const void* o,
                         const void* d_o, const float* lse, void* dq, void* dk, void* dv, void* stream) {
    const int rc = tmw::validate_prefill(desc, q, k, v, o);
    if (rc != TMW_OK) return rc;
    if (desc->q_pos0 != 0 || desc->k_pos0 != desc->n_persistent || desc->q_rows != desc->k_rows) {
        tmw::set_error_text("tmw_prefill_backward: whole sequences only (q_pos0 = 0, k_pos0 = n_persistent, q_rows = k_rows)");
        return TMW_ERR_UNSUPPORTED;
    }
    if (desc->batch == 0 || desc->heads == 0 || desc->q_rows == 0) return TMW_OK;
    if (d_o == nullptr || lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (!tmw::aligned16(d_o) || !tmw::aligned16(dq) || !tmw::aligned16(dk) || !tmw::aligned16(dv))
        return TMW_ERR_INVALID_ARGUMENT;
    // desc->algo: TMW_ALGO_SIMT pins the CUDA-core kernels, TMW_ALGO_MMA the warp-level tensor-core kernels,
    // TMW_ALGO_TCGEN05 the tcgen05 kernels; TMW_ALGO_AUTO takes the fastest path that applies, in that order backwards
    const bool tc_ok = tmw::prefill_backward_tc_supports(*desc);
    if (desc->algo == TMW_ALGO_TCGEN05 && !tc_ok) return TMW_ERR_UNSUPPORTED;
    if ((desc->algo == TMW_ALGO_AUTO || desc->algo == TMW_ALGO_TCGEN05) && tc_ok)
        return tmw::launch_prefill_backward_tc(*desc, q, k, v, o, d_o, lse, dq, dk, dv, static_cast<cudaStream_t>(stream));
    if (desc->algo == TMW_ALGO_MMA && !tmw::prefill_backward_mma_supports(*desc)) return TMW_ERR_UNSUPPORTED;
    if (desc->algo != TMW_ALGO_SIMT && tmw::prefill_backward_mma_supports(*desc))
        return tmw::launch_prefill_backward_mma(*desc, q, k, v, o, d_o, lse, dq, dk, dv, static_cast<cudaStream_t>(stream));
    return tmw::launch_prefill_backward(*desc, q, k, v, o, d_o, lse, dq, dk, dv, static_cast<cudaStream_t>(stream));
}

int tmw_prefill_block_sparse(const tmw_prefill_desc* desc, int32_t block_size, const void* q, const void* k,
                             const void* v, void* o, void* stream) {
    return tmw_prefill_block_sparse_lse(desc, block_size, q, k, v, o, nullptr, stream);
}

int tmw_prefill_block_sparse_backward(const tmw_prefill_desc* desc, int32_t block_size, const void* q, const void* k,
                                      const void* v, const void* o, const void* d_o, const float* lse, void* dq,
                                      void* dk, void* dv, void* stream) {
    const int rc = tmw::validate_prefill(desc, q, k, v, o);
    if (rc != TMW_OK) return rc;
    if (block_size <= 0 || block_size > (1 << 20)) return TMW_ERR_INVALID_ARGUMENT;
    if (desc->q_pos0 != 0 || desc->k_pos0 != desc->n_persistent || desc->q_rows != desc->k_rows) {
        tmw::set_error_text("tmw_prefill_block_sparse_backward: whole sequences only");
        return TMW_ERR_UNSUPPORTED;
    }
    if (desc->batch == 0 || desc->heads == 0 || desc->q_rows == 0) return TMW_OK;
    if (d_o == nullptr || lse == nullptr || dq == nullptr || dk == nullptr || dv == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (!tmw::aligned16(d_o) || !tmw::aligned16(dq) || !tmw::aligned16(dk) || !tmw::aligned16(dv))
        return TMW_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool tc_ok = tmw::prefill_backward_tc_supports(*desc);
    if (desc->algo == TMW_ALGO_TCGEN05 && !tc_ok) return TMW_ERR_UNSUPPORTED;
    if ((desc->algo == TMW_ALGO_AUTO || desc->algo == TMW_ALGO_TCGEN05) && tc_ok)
        return tmw::launch_prefill_backward_tc(*desc, q, k, v, o, d_o, lse, dq, dk, dv, s, block_size);
    if (desc->algo != TMW_ALGO_SIMT && tmw::prefill_backward_mma_supports(*desc))
        return tmw::launch_prefill_backward_mma(*desc, q, k, v, o, d_o, lse, dq, dk, dv, s, block_size, true);
    return tmw::launch_prefill_backward(*desc, q, k, v, o, d_o, lse, dq, dk, dv, s, block_size, true);
}

int tmw_prefill_block_sparse_lse(const tmw_prefill_desc* desc, int32_t block_size, const void* q, const void* k,
                                 const void* v, void* o, float* lse, void* stream) {
    const int rc = tmw::validate_prefill(desc, q, k, v, o);
    if (rc != TMW_OK) return rc;
    if (block_size <= 0 || block_size > (1 << 20)) {
        tmw::set_error_text("tmw_prefill_block_sparse: block_size must be positive (at most 2^20)");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (desc->q_pos0 != 0 || desc->k_pos0 != desc->n_persistent || desc->q_rows != desc->k_rows) {
        tmw::set_error_text("tmw_prefill_block_sparse: whole sequences only (q_pos0 = 0, k_pos0 = n_persistent, q_rows = k_rows)");
        return TMW_ERR_UNSUPPORTED;
    }
    if (desc->batch == 0 || desc->heads == 0 || desc->q_rows == 0) return TMW_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    tmw_prefill_desc d = *desc;
    const bool tc_ok = tmw::prefill_tc_supports(d, q, k, v, o) && (int64_t)d.q_rows + d.window + block_size < ((int64_t)1 << 29);
    if (d.algo == TMW_ALGO_TCGEN05 && !tc_ok) return TMW_ERR_UNSUPPORTED;
    const bool use_tc = d.algo != TMW_ALGO_SIMT && tc_ok;
    const int np = d.n_persistent;
    // the log-sum-exp comes in two planes: [batch, heads, L - np] for the sequence rows (first launch), then
    // [batch, heads, np] for the persistent rows (second launch)
    float* lse_pers = lse != nullptr ? lse + (size_t)d.batch * d.heads * (d.q_rows - np) : nullptr;
    auto launch = [&](const tmw_prefill_desc& dd, const void* qq, void* oo, cudaStream_t st, bool all_keys) {
        float* l = all_keys ? lse_pers : lse;
        return use_tc ? tmw::launch_prefill_tc(dd, qq, k, v, oo, st, block_size, all_keys, l)
                      : tmw::launch_prefill_simt(dd, qq, k, v, oo, st, block_size, all_keys, l);
    };
    if (np == 0) return launch(d, q, o, s, false);
    // Two independent launches: the sequence rows [np, L) with the block-granular window, and the np
    // persistent query rows, which see every key (one query tile per (batch, head) walking over all key
    // tiles - it occupies only batch x heads CTAs for a long time).  They write different rows, so the
    // second one runs on a side stream of the library between two events (a fork / join that stream
    // capture accepts as well).
    tmw_prefill_desc seq = d, pers = d;
    const size_t esz = tmw::dtype_size(d.dtype);
    seq.q_rows = d.q_rows - np;
    seq.q_pos0 = np;
    const void* q_seq = static_cast<const char*>(q) + (size_t)np * d.q_stride[2] * esz;
    void* o_seq = static_cast<char*>(o) + (size_t)np * d.o_stride[2] * esz;
    pers.q_rows = np;
    tmw::SideStream* side = tmw::side_stream_of_current_device();
    if (side == nullptr) {  // no side stream: one after the other
        const int st = launch(seq, q_seq, o_seq, s, false);
        return st != TMW_OK ? st : launch(pers, q, o, s, true);
    }
    std::lock_guard<std::mutex> lock(side->mutex);
    TMW_CUDA_TRY(cudaEventRecord(side->fork, s));
    TMW_CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
    int st = launch(pers, q, o, side->stream, true);
    TMW_CUDA_TRY(cudaEventRecord(side->join, side->stream));
    const int st2 = launch(seq, q_seq, o_seq, s, false);
    TMW_CUDA_TRY(cudaStreamWaitEvent(s, side->join, 0));
    return st != TMW_OK ? st : st2;
}

int tmw_linear(const tmw_linear_desc* d, const void* a, const void* w, const void* bias, void* c, void* stream) {
    if (d == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (d->dtype != TMW_BF16 && d->dtype != TMW_F16) return TMW_ERR_UNSUPPORTED;
    if (d->epilogue != TMW_EPILOGUE_NONE && d->epilogue != TMW_EPILOGUE_GELU) return TMW_ERR_INVALID_ARGUMENT;
    if (d->m < 0 || d->n < 0 || d->k <= 0) return TMW_ERR_INVALID_ARGUMENT;
    if (d->k % 8 != 0 || d->n % 8 != 0 || d->lda % 8 != 0 || d->ldw % 8 != 0 || d->ldc % 8 != 0 || d->lda < d->k ||
        d->ldw < d->k || d->ldc < d->n) {
        tmw::set_error_text("tmw_linear: k, n and the leading dimensions must be multiples of 8 (16 bytes)");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    if (d->m == 0 || d->n == 0) return TMW_OK;
    if (a == nullptr || w == nullptr || c == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (!tmw::aligned16(a) || !tmw::aligned16(w) || !tmw::aligned16(c) || (bias != nullptr && !tmw::aligned16(bias)))
        return TMW_ERR_INVALID_ARGUMENT;
    // tensor-map limits: leading dimensions below 2^40 bytes (extents are 32-bit already)
    const int64_t limit = ((int64_t)1 << 40) / 2;
    if (d->lda >= limit || d->ldw >= limit || d->ldc >= limit) return TMW_ERR_UNSUPPORTED;
    return tmw::launch_linear(*d, a, w, bias, c, static_cast<cudaStream_t>(stream));
}

size_t tmw_cache_ring_bytes(int32_t dtype, int32_t batch, int32_t heads, int32_t head_dim, int32_t window) {
    if (!tmw::dtype_ok(dtype) || batch < 0 || heads < 0 || head_dim <= 0 || window < 0) return 0;
    return (size_t)batch * (size_t)heads * ((size_t)window + 1) * (size_t)head_dim * tmw::dtype_size(dtype);
}

int tmw_cache_fill(const tmw_cache_desc* cache, const void* k, const void* v, const int64_t k_stride[3],
                   const int64_t v_stride[3], int32_t rows, int32_t t0, void* stream) {
    const int rc = tmw::validate_cache(cache);
    if (rc != TMW_OK) return rc;
    if (rows < 0 || t0 < 0 || k_stride == nullptr || v_stride == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    if (cache->batch == 0 || cache->heads == 0 || rows == 0) return TMW_OK;
    if (k == nullptr || v == nullptr || !tmw::aligned16(k) || !tmw::aligned16(v)) return TMW_ERR_INVALID_ARGUMENT;
    if (!tmw::strides_ok(k_stride, 3, cache->dtype) || !tmw::strides_ok(v_stride, 3, cache->dtype))
        return TMW_ERR_INVALID_ARGUMENT;
    return tmw::launch_cache_fill(*cache, k, v, k_stride, v_stride, rows, t0, static_cast<cudaStream_t>(stream));
}

int tmw_decode(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new, void* o,
               const int64_t q_stride[2], const int64_t kv_new_stride[2], const int64_t o_stride[2],
               const int32_t* pos, void* stream) {
    const int rc = tmw::validate_decode_call(cache, q, k_new, v_new, o, q_stride, kv_new_stride, o_stride, pos);
    if (rc != TMW_OK) return rc;
    if (cache->batch == 0 || cache->heads == 0) return TMW_OK;
    return tmw::launch_decode(*cache, q, k_new, v_new, o, q_stride, kv_new_stride, o_stride, pos, 0, nullptr, nullptr,
                              static_cast<cudaStream_t>(stream));
}

size_t tmw_decode_split_scratch_bytes(const tmw_cache_desc* cache, int32_t splits) {
    if (tmw::validate_cache(cache) != TMW_OK || splits < 1 || splits > TMW_MAX_DECODE_SPLITS) return 0;
    return tmw::decode_partials_bytes(cache->batch, cache->heads, cache->head_dim, splits) +
           (size_t)cache->batch * (size_t)cache->heads * sizeof(unsigned int);
}

int tmw_decode_split(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new, void* o,
                     const int64_t q_stride[2], const int64_t kv_new_stride[2], const int64_t o_stride[2],
                     const int32_t* pos, int32_t splits, void* scratch, size_t scratch_bytes, void* stream) {
    const int rc = tmw::validate_decode_call(cache, q, k_new, v_new, o, q_stride, kv_new_stride, o_stride, pos);
    if (rc != TMW_OK) return rc;
    if (splits < 1 || splits > TMW_MAX_DECODE_SPLITS) return TMW_ERR_INVALID_ARGUMENT;
    if (cache->batch == 0 || cache->heads == 0) return TMW_OK;
    if (scratch == nullptr || !tmw::aligned16(scratch)) return TMW_ERR_INVALID_ARGUMENT;
    if (scratch_bytes < tmw_decode_split_scratch_bytes(cache, splits)) return TMW_ERR_TOO_LARGE;
    unsigned int* counters = reinterpret_cast<unsigned int*>(
        static_cast<char*>(scratch) + tmw::decode_partials_bytes(cache->batch, cache->heads, cache->head_dim, splits));
    return tmw::launch_decode(*cache, q, k_new, v_new, o, q_stride, kv_new_stride, o_stride, pos, splits,
                              static_cast<float*>(scratch), counters, static_cast<cudaStream_t>(stream));
}

int tmw_poll_status(void* stream) {
    TMW_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int* word = tmw::device_status_word();
    if (word == nullptr) return TMW_ERR_CUDA;
    int value[4] = {0, 0, 0, 0};
    TMW_CUDA_TRY(cudaMemcpy(value, word, sizeof(value), cudaMemcpyDeviceToHost));
    if (value[0] != 0) {
        const int zero[4] = {0, 0, 0, 0};
        TMW_CUDA_TRY(cudaMemcpy(word, zero, sizeof(zero), cudaMemcpyHostToDevice));
        char text[160];
        if (value[0] == TMW_ERR_INVALID_ARGUMENT) {
            tmw::set_error_text("a kernel met an invalid device-side argument (a negative entry of pos in a decode call)");
            return TMW_ERR_INVALID_ARGUMENT;
        }
        if (value[1] == -1)
            std::snprintf(text, sizeof(text), "device wait expired: a halo flag that another GPU should have raised (block %d, detail %d)",
                          value[2] & 0xffff, value[3]);
        else
            std::snprintf(text, sizeof(text), "device wait expired: barrier at shared offset %d parity %d, block (%d,%d,%d), warp %d",
                          value[1] & 0xffff, (value[1] >> 16) & 1, value[2] & 0xffff, (value[2] >> 16) & 0xffff,
                          value[3] & 0xffff, (value[3] >> 16) & 0xffff);
        tmw::set_error_text(text);
        return TMW_ERR_DEVICE_TIMEOUT;
    }
    return TMW_OK;
}

}  // extern "C"
