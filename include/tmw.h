/*
 * tmw.h — C ABI of libtmw: sliding-window attention with persistent prefix keys
 * for NVIDIA B200 (sm_100a).
 *
 * The library replaces the attention core of TitanMAC's WindowedAttention module
 * (reference project path: titans_core/attn/windowed_attention.py).  All
 * pointers are device pointers unless stated otherwise; sizes and strides are in
 * ELEMENTS; the innermost (head_dim) stride of every tensor is 1.  Every entry
 * point enqueues work on the CUDA stream it is given (a cudaStream_t passed as
 * void*, NULL = the default stream) and returns without synchronising.  Return
 * value: TMW_OK (0) or a negative tmw_status.  Nothing here throws, allocates
 * caller-visible memory or falls back to the CPU.
 *
 * Positions.  The reference treats the first n_persistent rows of its input as
 * "persistent" rows and the rest as sequence rows; positions in this header
 * count over that whole length L = n_persistent + T.  A query at position p
 * attends to
 *     every key position g <  n_persistent                       and, if
 *     p >= n_persistent, to the keys max(n_persistent, p - window) <= g <= p.
 * (windowed_attention.py:113-118 and :134-150; a query therefore sees window+1
 * sequence keys including itself.)
 */
#ifndef TMW_H_
#define TMW_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TMW_VERSION 100

#if defined(__GNUC__)
#define TMW_API __attribute__((visibility("default")))
#else
#define TMW_API
#endif

typedef enum tmw_status {
    TMW_OK = 0,
    TMW_ERR_INVALID_ARGUMENT = -1, /* NULL pointer, negative size, stride/alignment rule broken        */
    TMW_ERR_UNSUPPORTED = -2,      /* dtype / head_dim / algorithm combination that has no kernel       */
    TMW_ERR_PERSISTENT_GE_LEN = -3,/* n_persistent >= length (the reference raises ValueError, :97-100) */
    TMW_ERR_NEGATIVE_WINDOW = -4,  /* window < 0 (the reference raises ValueError, :102-103)            */
    TMW_ERR_KEY_RANGE = -5,        /* a query needs a key position the K/V buffers do not hold          */
    TMW_ERR_CUDA = -6,             /* a CUDA runtime or driver call failed; see tmw_last_cuda_error()   */
    TMW_ERR_DEVICE_TIMEOUT = -7,   /* a bounded device-side wait gave up (read back by tmw_poll_status) */
    TMW_ERR_TOO_LARGE = -8         /* a fixed capacity of the called entry point is exceeded            */
} tmw_status;

typedef enum tmw_dtype { TMW_F32 = 0, TMW_BF16 = 1, TMW_F16 = 2 } tmw_dtype;

typedef enum tmw_algo {
    TMW_ALGO_AUTO = 0,   /* tcgen05 kernel when it applies, otherwise the CUDA-core kernel       */
    TMW_ALGO_SIMT = 1,   /* CUDA-core kernel (every dtype, head_dim 8/16/32/64/96/128/256)       */
    TMW_ALGO_TCGEN05 = 2,/* tensor-core kernel (bf16/f16, head_dim 64 or 128)                    */
    TMW_ALGO_MMA = 3     /* backward only: the warp-level tensor-core kernels (mma.sync class)   */
} tmw_algo;

/*
 * Prefill: o = softmax(q kᵀ · scale + mask) v for a block of query rows.
 * Replaces the bool→additive mask conversion and the scaled-dot-product call of
 * WindowedAttention.forward (windowed_attention.py:307-323) together with the
 * dense mask of build_band_mask (:61-152), which is never materialised.
 *
 * q, o : [batch, heads, q_rows, head_dim]   addressed through *_stride[3] =
 * k, v : [batch, heads, k_rows, head_dim]   {batch, head, row} element strides.
 *
 * Query row r sits at position q_pos0 + r.  Key rows [0, n_persistent) are the
 * persistent keys; key row n_persistent + i sits at position k_pos0 + i.  The
 * unsharded call has q_pos0 = 0, k_pos0 = n_persistent and q_rows = k_rows = L.
 * A sequence-sharded rank passes its own rows as q and a K/V buffer laid out as
 * [persistent | halo from the left neighbour | own rows] with k_pos0 = position
 * of the first halo row.
 */
typedef struct tmw_prefill_desc {
    int32_t dtype;        /* tmw_dtype of q, k, v and o                                   */
    int32_t algo;         /* tmw_algo                                                     */
    int32_t batch, heads, head_dim;
    int32_t q_rows, k_rows;
    int32_t window;       /* w: a sequence query sees itself and the w previous keys      */
    int32_t n_persistent; /* Np                                                           */
    int32_t q_pos0;       /* position of query row 0                                      */
    int32_t k_pos0;       /* position of key row n_persistent (>= n_persistent)           */
    float scale;          /* 0 selects 1/sqrt(head_dim), the reference's default (:318)   */
    int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];
} tmw_prefill_desc;

TMW_API int tmw_prefill(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, void* o,
                void* stream);

/*
 * tmw_prefill that also returns, per query row, the log-sum-exp of its scores: lse[batch, heads, q_rows]
 * (fp32, contiguous) holds log2(sum_j exp2(s_ij * scale * log2 e)) over the visible keys - the one number
 * per row from which the backward pass rebuilds the probabilities.
 */
TMW_API int tmw_prefill_lse(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, void* o,
                            float* lse, void* stream);

/*
 * Backward of tmw_prefill for whole sequences (q_pos0 = 0, k_pos0 = n_persistent, q_rows = k_rows):
 * given d_o (gradient of o, addressed like o) and the o and lse of tmw_prefill_lse, writes dq, dk, dv
 * (addressed like q, k, v: the same strides).  Replaces what autograd does through the reference's mask
 * conversion and scaled-dot-product call (windowed_attention.py:307-323) - there over all L x L pairs,
 * here over the visible pairs only.  For bf16 / f16 with head_dim 64 or 128: tcgen05 kernels (products and the
 * 16-bit intermediates in tensor memory; desc->algo TMW_ALGO_AUTO or TMW_ALGO_TCGEN05), or the older warp-level
 * tensor-core kernels (TMW_ALGO_MMA); fp32 arithmetic on CUDA cores otherwise, or for every case with
 * TMW_ALGO_SIMT.  All of them accumulate in fp32.  The tcgen05 path keeps 8 bytes per (batch, head, row) between
 * its two launches in scratch memory that it takes, ordered on `stream`, from a memory pool of the library's own
 * (created on first use per device, kept until the process ends; usable while `stream` is being captured); if the
 * pool cannot be had it recomputes those numbers instead.
 */
TMW_API int tmw_prefill_backward(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v,
                                 const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv,
                                 void* stream);

/*
 * Prefill with the mask of the reference's BlockSparseAttention (its default attention class,
 * titans_core/attn/block_sparse_attention.py:258-343), for whole sequences (q_pos0 = 0,
 * k_pos0 = n_persistent, q_rows = k_rows = L; desc->window is its window_size):
 *   - the sequence row with sequence index t sees the persistent keys and the sequence keys
 *     max(0, floor(t / block_size) * block_size - window) .. t   (:299-311, :147-156);
 *   - the n_persistent persistent query rows see every key, later rows included (:283-291).
 * q, k, v are the tensors after that class's depthwise convolutions (tmw_causal_dwconv).
 * Replaces its Python loop over query blocks with per-block concatenation, mask and softmax.
 */
TMW_API int tmw_prefill_block_sparse(const tmw_prefill_desc* desc, int32_t block_size, const void* q, const void* k,
                                     const void* v, void* o, void* stream);

/*
 * tmw_prefill_block_sparse that also returns the row log-sum-exp (see tmw_prefill_lse), and its backward.
 * lse holds batch x heads x L floats in two planes: [batch, heads, L - n_persistent] for the sequence rows,
 * followed by [batch, heads, n_persistent] for the persistent rows.  The backward writes dq, dk, dv (addressed
 * like q, k, v) from d_o (addressed like o): what autograd does through the reference's per-block matmul /
 * softmax / matmul (block_sparse_attention.py:163-199, 258-343).  Kernels and desc->algo as for
 * tmw_prefill_backward (tcgen05 for bf16 / f16 with head_dim 64 or 128 unless another path is pinned).
 */
TMW_API int tmw_prefill_block_sparse_lse(const tmw_prefill_desc* desc, int32_t block_size, const void* q, const void* k,
                                         const void* v, void* o, float* lse, void* stream);
TMW_API int tmw_prefill_block_sparse_backward(const tmw_prefill_desc* desc, int32_t block_size, const void* q,
                                              const void* k, const void* v, const void* o, const void* d_o,
                                              const float* lse, void* dq, void* dk, void* dv, void* stream);

/*
 * Causal depthwise convolution along the rows: y[b, t, c] = sum_j weight[c, j] * x[b, t - (taps-1) + j, c],
 * rows before the first count as zero.  x, y: [batch, rows, channels] contiguous (channels a multiple of 8,
 * 16-byte aligned); weight: [channels, taps] contiguous, same dtype, 1 <= taps <= 8; y must not overlap x.
 * Replaces the three Conv1d(groups=d_model, padding=taps-1) calls with their transposes and trimming in
 * BlockSparseAttention.forward (block_sparse_attention.py:241-256) - with channels = 3 * d_model and the
 * three filters stacked it is one pass over the QKV projection output.
 */
TMW_API int tmw_causal_dwconv(int32_t dtype, int32_t batch, int32_t rows, int32_t channels, int32_t taps,
                              const void* x, const void* weight, void* y, void* stream);

/*
 * Backward of tmw_causal_dwconv: dx (like x) and dw (fp32 [channels, taps], ADDED to: zero it first) from dy.
 * Replaces autograd through the three Conv1d calls of block_sparse_attention.py:241-256.
 */
TMW_API int tmw_causal_dwconv_backward(int32_t dtype, int32_t batch, int32_t rows, int32_t channels, int32_t taps,
                                       const void* x, const void* weight, const void* dy, void* dx, float* dw,
                                       void* stream);

/*
 * Sequence-sharded prefill without a host-side collective on the step.  The reference has no distributed code;
 * this is the multi-GPU form of its attention core (windowed_attention.py:113-150: a row needs its window
 * predecessors and the persistent rows, nothing else), for one process per GPU with the neighbours' buffers
 * mapped into this process (CUDA IPC / peer access; how the pointers are exchanged is the caller's business).
 *
 * tmw_halo_push - one launch per destination rank, on `stream`:
 *   1. waits (bounded) until *wait_flag >= wait_value (wait_flag: in THIS GPU's memory, raised by the destination
 *      when it has finished reading what the previous push wrote; NULL = no wait),
 *   2. copies every src -> dst (dst: the destination rank's K/V buffer through its peer mapping; plain stores),
 *   3. stores signal_value to *signal_flag (in the destination's memory) with release semantics at system scope
 *      (signal_flag NULL = none; n_copies = 0 with a signal_flag makes the call a pure signal).
 * Pointers and sizes are multiples of 16 bytes; at most TMW_HALO_MAX_COPIES copies per call.  Launches of one
 * process must be ordered on one stream (they share a completion counter).  wait_limit_cycles <= 0 selects
 * about one second; an expired wait skips copies and signal and is reported by tmw_poll_status
 * (TMW_ERR_DEVICE_TIMEOUT).
 *
 * tmw_prefill_halo - tmw_prefill on the tensor-core kernel (TMW_ERR_UNSUPPORTED where that kernel does not
 * apply) for a K/V buffer [persistent | halo | own rows] whose first two parts are written by other GPUs: the
 * kernel's loader warps poll *pers_flag (key rows [0, n_persistent)) and *halo_flag (key rows [n_persistent,
 * n_persistent + halo_rows)) until they reach `value`, right before the first TMA load that touches those rows -
 * query tiles whose window lies in the rank's own rows never wait for the halo.  The flags live in this GPU's
 * memory; a NULL flag is not waited for.  Waits are bounded by wait_limit_cycles (<= 0: about one second).
 */
#define TMW_HALO_MAX_COPIES 8

typedef struct tmw_halo_copy {
    const void* src; /* local memory */
    void* dst;       /* local or peer-mapped memory */
    size_t bytes;
} tmw_halo_copy;

typedef struct tmw_halo_wait {
    const int32_t* pers_flag;
    const int32_t* halo_flag;
    int32_t value;
    int32_t halo_rows;
    int64_t wait_limit_cycles;
} tmw_halo_wait;

TMW_API int tmw_halo_push(const tmw_halo_copy* copies, int32_t n_copies, const int32_t* wait_flag, int32_t wait_value,
                          int32_t* signal_flag, int32_t signal_value, int64_t wait_limit_cycles, void* stream);

/*
 * Mapping a buffer of another process of the same node (one process per GPU), for the destinations and flags of
 * tmw_halo_push.  tmw_ipc_export describes the device allocation that holds ptr (allocations of cudaMalloc, which
 * is what PyTorch's default allocator hands out); the 80-byte description travels to the other process by any
 * means (the host side uses torch.distributed.all_gather_object).  tmw_ipc_open maps it with the CALLER'S current
 * device as the one whose kernels will use the address, and returns the address of the same byte as ptr.  Every
 * allocation is mapped once per process and device; tmw_ipc_close_all unmaps everything (call it, on every rank,
 * before any rank frees an exported buffer).
 */
typedef struct tmw_ipc_mem {
    unsigned char handle[64];
    uint64_t offset; /* of the buffer inside its allocation */
    uint64_t size;   /* of the allocation */
} tmw_ipc_mem;

TMW_API int tmw_ipc_export(const void* ptr, tmw_ipc_mem* out);
TMW_API int tmw_ipc_open(const tmw_ipc_mem* mem, void** ptr);
TMW_API int tmw_ipc_close_all(void);

/* Enables peer access from the current device to peer_device (needed before tmw_halo_push stores into that GPU's
 * memory through a mapping); already enabled is fine.  TMW_ERR_UNSUPPORTED when the devices have no peer path. */
TMW_API int tmw_enable_peer_access(int32_t peer_device);

TMW_API int tmw_prefill_halo(const tmw_prefill_desc* desc, const void* q, const void* k, const void* v, void* o,
                             const tmw_halo_wait* wait, void* stream);

/*
 * Linear layer on the tensor cores: c[m, n] = sum_k a[m, k] * w[n, k] (+ bias[n]) (then the exact, erf-based GELU
 * when epilogue is TMW_EPILOGUE_GELU) - torch.nn.functional.linear with its [out_features, in_features] weight.
 * a: [m, k] row-major with leading dimension lda, w: [n, k] with ldw, c: [m, n] with ldc (elements); bias: [n]
 * or NULL; everything in dtype (TMW_BF16 or TMW_F16), accumulation in fp32.  k, n and the leading dimensions
 * must be multiples of 8 and the pointers 16-byte aligned (TMW_ERR_INVALID_ARGUMENT otherwise).
 * Replaces the library GEMMs behind the module's two projections (windowed_attention.py:295 qkv_proj, :331
 * out_proj, both without bias) and behind the block's MLP, whose bias add and GELU ride in the epilogue
 * (titans_core/blocks/mlp.py:58-65: fc1 + bias -> GELU -> fc2 + bias).
 */
typedef enum tmw_epilogue { TMW_EPILOGUE_NONE = 0, TMW_EPILOGUE_GELU = 1 } tmw_epilogue;

typedef struct tmw_linear_desc {
    int32_t dtype;    /* tmw_dtype of a, w, bias and c: TMW_BF16 or TMW_F16 */
    int32_t m, n, k;
    int32_t epilogue; /* tmw_epilogue, applied after the bias */
    int64_t lda, ldw, ldc;
} tmw_linear_desc;

TMW_API int tmw_linear(const tmw_linear_desc* desc, const void* a, const void* w, const void* bias, void* c,
                       void* stream);

/*
 * Decode: one new token per sequence against a ring cache of the last window+1
 * keys.  The reference has no incremental decode (its generation helper re-runs
 * the full forward per token, examples/train_math.py:146-161); this entry point
 * returns what the last row of that forward returns.
 *
 * k_ring, v_ring : [batch, heads, slots, head_dim] contiguous, slots = window+1.
 * k_pers, v_pers : [heads, n_persistent, head_dim] contiguous, shared by the batch
 *                  (may be NULL when n_persistent == 0).
 * Token t of a sequence (t = 0 for its first sequence token) lives in slot
 * t % slots.
 */
typedef struct tmw_cache_desc {
    int32_t dtype;
    int32_t batch, heads, head_dim;
    int32_t window, n_persistent;
    void* k_ring;
    void* v_ring;
    const void* k_pers;
    const void* v_pers;
    float scale; /* 0 selects 1/sqrt(head_dim) */
} tmw_cache_desc;

/* Bytes of ONE ring (k or v) for the given geometry; 0 on bad arguments. */
TMW_API size_t tmw_cache_ring_bytes(int32_t dtype, int32_t batch, int32_t heads, int32_t head_dim, int32_t window);

/*
 * Copy K/V rows produced by a prefill into the ring.  k, v: [batch, heads, rows,
 * head_dim] through {batch, head, row} strides, row i being sequence token
 * t0 + i.  Only the last min(rows, window+1) rows are kept.
 */
TMW_API int tmw_cache_fill(const tmw_cache_desc* cache, const void* k, const void* v, const int64_t k_stride[3],
                   const int64_t v_stride[3], int32_t rows, int32_t t0, void* stream);

/*
 * One decode step.  q, k_new, v_new, o: [batch, heads, head_dim] through
 * {batch, head} strides.  pos: device array [batch] of int32, the sequence index
 * t >= 0 of the new token (the host cannot see a device array: a negative entry is
 * treated as 0 by the kernels and reported by tmw_poll_status as
 * TMW_ERR_INVALID_ARGUMENT).  The call stores k_new/v_new into slot t % (window+1) and
 * attends over the persistent keys and the min(t+1, window+1) newest slots.
 */
TMW_API int tmw_decode(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new, void* o,
               const int64_t q_stride[2], const int64_t kv_new_stride[2], const int64_t o_stride[2],
               const int32_t* pos, void* stream);

/*
 * The same step for small batches: the keys of every (sequence, head) pair are cut into `splits` ranges
 * (1..TMW_MAX_DECODE_SPLITS) that are scanned by separate CTAs; the CTA of a pair that finishes last merges
 * the partial results.  Partial results and one arrival counter per pair live in caller-provided scratch
 * memory (device, 16-byte aligned) of at least tmw_decode_split_scratch_bytes() bytes.  The scratch memory
 * must be ZERO-FILLED ONCE before its first use with a given geometry; every call leaves the counters at
 * zero again.  Two calls that use the same scratch memory must not overlap on the GPU.
 * Like tmw_decode it has no counterpart in the reference (examples/train_math.py:146-161 re-runs the
 * forward); it pays off below a few hundred pairs, where one CTA per pair cannot keep HBM busy.
 */
#define TMW_MAX_DECODE_SPLITS 16
TMW_API size_t tmw_decode_split_scratch_bytes(const tmw_cache_desc* cache, int32_t splits);
TMW_API int tmw_decode_split(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new, void* o,
                     const int64_t q_stride[2], const int64_t kv_new_stride[2], const int64_t o_stride[2],
                     const int32_t* pos, int32_t splits, void* scratch, size_t scratch_bytes, void* stream);

/*
 * tmw_decode_split for callers that cannot allocate device memory (no counterpart in the reference).
 *
 * Who needs it: a serving process that gave all of HBM to its own memory pool and forbids cudaMalloc
 * after start-up, or a decode loop in which an allocation - a synchronising driver call - is not
 * acceptable.  The scratch memory of the split launch is then a fixed 2 MiB array inside the library
 * (one per GPU that loads the library, held until the process exits) instead of a caller buffer.
 *
 * Limits: batch x heads <= 4096 and batch x heads x splits x (head_dim + 2) x 4 bytes <= 2 MiB - 16 KiB;
 * anything larger returns TMW_ERR_TOO_LARGE (tmw_last_cuda_error() says by how much).  The call never
 * calls cudaMalloc, cudaFree or any other allocating routine.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress with that device
 * current); make that first call outside any stream capture.  All calls on one GPU share the one array:
 * every call clears the arrival counters it needs and overwrites the partial results, so calls may follow
 * one another on a stream, but two calls that overlap on the GPU (different streams) race.
 */
TMW_API int tmw_decode_split_static(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new,
                            void* o, const int64_t q_stride[2], const int64_t kv_new_stride[2],
                            const int64_t o_stride[2], const int32_t* pos, int32_t splits, void* stream);

/*
 * Residual add + RMSNorm over contiguous rows [rows, dim] (dim a multiple of 8, pointers 16-byte aligned):
 *     h = x + residual          (residual may be NULL: h = x)
 *     sum_out = h               (sum_out may be NULL, and may be x itself: the residual stream in place)
 *     y = h / sqrt(mean(h^2) + eps) * scale
 * Replaces the element-wise PyTorch operations around the attention call in the reference's block:
 * the residual adds of titans_core/blocks/titan_block.py:94-100 and RMSNorm.forward,
 * titans_core/blocks/norms.py:55-58 (seven kernels there, one pass over HBM here).  h is rounded to the
 * storage type before the norm, as the reference's own addition does; the norm is computed in fp32.
 */
TMW_API int tmw_add_rmsnorm(int32_t dtype, int64_t rows, int32_t dim, const void* x, const void* residual,
                            const void* scale, float eps, void* sum_out, void* y, void* stream);

/*
 * y = 0.5 x (1 + erf(x / sqrt 2)) over n contiguous elements (n a multiple of 8, pointers 16-byte aligned;
 * y may be x).  Replaces the nn.GELU() between the two linears of the reference's MLP,
 * titans_core/blocks/mlp.py:58-65 (exact form, not the tanh approximation).  erf is evaluated with an
 * absolute error below 1.5e-7.
 */
TMW_API int tmw_gelu(int32_t dtype, int64_t n, const void* x, void* y, void* stream);

/* Library facts. */
TMW_API int tmw_version(void);
TMW_API const char* tmw_strerror(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
TMW_API const char* tmw_last_cuda_error(void);
/*
 * Device-side status word of the current device: 0, or TMW_ERR_DEVICE_TIMEOUT if a
 * kernel's bounded wait expired since the last poll.  Synchronises the given
 * stream, then clears the word.
 */
TMW_API int tmw_poll_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TMW_H_ */
