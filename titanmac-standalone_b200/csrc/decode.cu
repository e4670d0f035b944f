// Decode against a ring cache of the last window+1 keys per (sequence, head), plus
// the persistent keys every query sees.  The step is bound by HBM traffic (about one
// multiply-add per byte read), so the kernel is organised around wide coalesced
// loads: a key row of head_dim elements is read by head_dim/8 adjacent lanes with
// one 16-byte load each, a warp covers 32/(head_dim/8) rows per load instruction and
// keeps UNROLL such instructions in flight for K and for V before it touches the
// softmax.  Dot products are finished with warp shuffles; each lane group keeps a
// private online-softmax state that is merged across groups (and warps) at the end.
//
// Two launch shapes share the code: with many (sequence, head) pairs every pair gets
// ONE warp (no block-level merge, all pairs resident at once, so no wave
// quantisation); with few pairs a whole CTA of 8 warps shares one pair.
//
// 16-bit caches with more than half a pair per SM take decode_stream_kernel further
// down instead: the same arithmetic fed from shared memory, which bulk asynchronous
// copies keep filled three chunks ahead (measured on B200, 2560 pairs, window 512:
// 60 us against 68 us; 5120 pairs: 105 us against 129 us, the bandwidth of a plain copy).
#include <math_constants.h>

#include <cstdio>

#include <atomic>

#include "tmw_common.cuh"

#ifndef TMW_DECODE_STREAM
#define TMW_DECODE_STREAM 1
#endif

namespace tmw {
namespace {


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
    int batch, heads, slots, np;
    float scale_log2;
    int splits;              // > 0: the keys of a pair are cut into this many ranges, one CTA each
    float* scratch;          // [pairs][splits][DH + 2] partial results (accumulator, running maximum, sum)
    unsigned int* counters;  // [pairs] arrivals of a pair's CTAs; zero between launches
    int* status;             // device status word (bounded waits of the streaming kernel report here)
};

// 8 consecutive elements as raw bits, loaded through the read-only path without keeping
// the line in L1 (every ring byte is read exactly once per step).
template <typename T>
struct Raw8;
template <>
struct Raw8<float> {
    uint4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p));
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(p + 4));
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
        f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
    }
};
template <>
struct Raw8<__nv_bfloat16> {
    uint4 a;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p));
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <>
struct Raw8<__half> {
    uint4 a;
    __device__ __forceinline__ void load(const __half* p) {
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(p));
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
};

// WARPS = warps that share one (sequence, head) pair.  The launcher picks WARPS so that every pair is
// resident at once (no second, partly filled wave of CTAs):
//   WARPS 1: 2 pairs per 64-thread CTA, 9 CTAs per SM  -> up to 2664 pairs on 148 SMs
//   WARPS 2: 1 pair  per 64-thread CTA, 9 CTAs per SM  -> up to 1332 pairs
//   WARPS 4: 1 pair  per 128-thread CTA, 4 per SM      -> up to  592 pairs
//   WARPS 8: 1 pair  per 256-thread CTA, 2 per SM      -> up to  296 pairs
//
// SPLIT: few pairs (small batches).  A pair's keys are cut into p.splits ranges, each scanned by its own
// CTA, which leaves an unnormalised partial result in scratch memory and counts itself in; the CTA that
// arrives last merges the pair's partial results, writes the output and puts the counter back to zero.
template <typename T, int DH, int WARPS, bool SPLIT = false>
__global__ void __launch_bounds__(WARPS == 1 ? 64 : WARPS * 32, WARPS <= 2 ? 9 : (WARPS == 4 ? 4 : 2))
decode_kernel(const DecodeParams p) {
    // 16-byte loads in flight per lane for K, and again for V; fewer in the shapes with many resident
    // warps per SM, whose register budget per thread is 112
    constexpr int UNROLL = (WARPS <= 2 ? 4 : 8) / (sizeof(T) == 4 ? 2 : 1);
    constexpr int LPK = DH / 8;       // lanes per key row
    constexpr int RPW = 32 / LPK;     // key rows per warp per load instruction
    constexpr int STRIDE = RPW * WARPS;
    static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must be 8 * 2^n, at most 256");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pair = SPLIT ? blockIdx.x / p.splits : (WARPS == 1 ? blockIdx.x * 2 + warp : blockIdx.x);
    const int split = SPLIT ? blockIdx.x % p.splits : 0;
    if (pair >= p.batch * p.heads) return;  // whole warps leave together; no block barrier when WARPS == 1
    const int b = pair / p.heads, h = pair % p.heads;
    const int wslot = WARPS == 1 ? 0 : warp;  // which share of the keys this warp scans
    const int sub = lane % LPK;  // which 8-element slice of the row
    const int grp = lane / LPK;  // which row of the warp's RPW rows

    int t = p.pos[b];
    if (t < 0) {
        // a negative position would put the new row in front of the ring: treated as position 0 (nothing is
        // written out of bounds) and reported through the status word as an invalid argument
        if (lane == 0) atomicCAS(p.status, 0, (int)TMW_ERR_INVALID_ARGUMENT);
        t = 0;
    }
    const int slot_new = t % p.slots;
    const int count = min(t + 1, p.slots);
    const long long ring_bh = ((long long)b * p.heads + h) * p.slots * DH;
    T* kr = static_cast<T*>(p.k_ring) + ring_bh;
    T* vr = static_cast<T*>(p.v_ring) + ring_bh;
    const T* kp = static_cast<const T*>(p.k_pers) + (long long)h * p.np * DH;
    const T* vp = static_cast<const T*>(p.v_pers) + (long long)h * p.np * DH;
    const T* kn = static_cast<const T*>(p.k_new) + b * p.ns[0] + h * p.ns[1];
    const T* vn = static_cast<const T*>(p.v_new) + b * p.ns[0] + h * p.ns[1];

    float qreg[8];
    load8<T>(static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + sub * 8, qreg);

    // Virtual key index i: [0, np) persistent keys, np = the new token (read from k_new / v_new, so the
    // ring slot written below is never read back), then the count-1 older ring slots in slot order.
    const int n_all = p.np + count;
    const int per_split = SPLIT ? (n_all + p.splits - 1) / p.splits : n_all;
    const int k_lo = split * per_split;
    const int n_keys = min(n_all, k_lo + per_split);  // this CTA scans the virtual keys [k_lo, n_keys)
    float m = -CUDART_INF_F, l = 0.f;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};

    for (int i0 = k_lo; i0 < n_keys; i0 += STRIDE * UNROLL) {
        Raw8<T> kraw[UNROLL], vraw[UNROLL];
        bool ok[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int i = i0 + u * STRIDE + wslot * RPW + grp;
            ok[u] = i < n_keys;
            if (ok[u]) {
                const T* ksrc;
                const T* vsrc;
                if (i < p.np) {
                    ksrc = kp + (long long)i * DH;
                    vsrc = vp + (long long)i * DH;
                } else if (i == p.np) {
                    ksrc = kn;
                    vsrc = vn;
                } else {
                    const int j = i - p.np - 1;
                    const int slot = j < slot_new ? j : j + 1;
                    ksrc = kr + (long long)slot * DH;
                    vsrc = vr + (long long)slot * DH;
                }
                kraw[u].load(ksrc + sub * 8);
                vraw[u].load(vsrc + sub * 8);
            }
        }
        float s[UNROLL];
        float tmax = -CUDART_INF_F;
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float part = 0.f;
            if (ok[u]) {
                float kf[8];
                kraw[u].unpack(kf);
#pragma unroll
                for (int e = 0; e < 8; ++e) part = fmaf(qreg[e], kf[e], part);
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
                    float vf[8];
                    vraw[u].unpack(vf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(pj, vf[e], acc[e]);
                }
            }
        }
    }

    // the new token's key and value go into their ring slot for the following steps
    if (wslot == 0 && grp == 0 && split == 0) {
        float tmp[8];
        load8<T>(kn + sub * 8, tmp);
        store8<T>(kr + (long long)slot_new * DH + sub * 8, tmp);
        load8<T>(vn + sub * 8, tmp);
        store8<T>(vr + (long long)slot_new * DH + sub * 8, tmp);
    }

    // merge the RPW lane groups of the warp (lanes that hold the same slice)
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

    T* out = static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1];
    if (WARPS == 1) {
        if (grp == 0) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            float res[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) res[e] = acc[e] * inv;
            store8<T>(out + sub * 8, res);
        }
    } else {
        // merge the warps through shared memory
        __shared__ float sm_m[WARPS], sm_l[WARPS];
        __shared__ float sm_acc[WARPS][DH];
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
            for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, sm_m[w]);
            float l_all = 0.f;
            float res[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float a = sm_m[w] > -CUDART_INF_F ? exp2f(sm_m[w] - m_all) : 0.f;
                l_all += sm_l[w] * a;
#pragma unroll
                for (int e = 0; e < 8; ++e) res[e] += sm_acc[w][tid * 8 + e] * a;
            }
            if (SPLIT) {
                float* part = p.scratch + ((long long)pair * p.splits + split) * (DH + 2);
#pragma unroll
                for (int e = 0; e < 8; ++e) part[tid * 8 + e] = res[e];
                if (tid == 0) {
                    part[DH] = m_all;
                    part[DH + 1] = l_all;
                }
            } else {
                const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll
                for (int e = 0; e < 8; ++e) res[e] *= inv;
                store8<T>(out + tid * 8, res);
            }
        }
        if (SPLIT) {
            // last CTA of the pair merges (the usual fence / counter / fence hand-over through global memory)
            __shared__ int is_last;
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int prev = atomicAdd(p.counters + pair, 1u);
                is_last = prev == (unsigned int)p.splits - 1u;
            }
            __syncthreads();
            if (is_last) {
                __threadfence();
                const volatile float* all = p.scratch + (long long)pair * p.splits * (DH + 2);
                float m_all = -CUDART_INF_F;
                for (int sp = 0; sp < p.splits; ++sp) m_all = fmaxf(m_all, all[sp * (DH + 2) + DH]);
                for (int d = tid; d < DH; d += WARPS * 32) {
                    float l_all = 0.f, a_all = 0.f;
                    for (int sp = 0; sp < p.splits; ++sp) {
                        const float m_s = all[sp * (DH + 2) + DH];
                        const float a = m_s > -CUDART_INF_F ? exp2f(m_s - m_all) : 0.f;
                        l_all += all[sp * (DH + 2) + DH + 1] * a;
                        a_all += all[sp * (DH + 2) + d] * a;
                    }
                    out[d] = from_f32<T>(l_all > 0.f ? a_all / l_all : 0.f);
                }
                if (tid == 0) p.counters[pair] = 0u;  // ready for the next launch
            }
        }
    }
}


// -----------------------------------------------------------------------------------------------------
// Streaming variant for 16-bit caches with every pair resident (one warp per pair).
//
// The register variant above issues a batch of loads, waits for all of them and computes: between batches
// a warp has nothing in flight, and the measured bandwidth stays at three quarters of a plain copy.  Here
// the keys and values of a pair - contiguous in the ring - are brought into shared memory by bulk
// asynchronous copies (cp.async.bulk, completion counted on an mbarrier) in chunks of 2 KB for K and 2 KB
// for V, three chunks ahead of the arithmetic, so every warp keeps 12 KB in flight at all times without
// holding them in registers.  A stage is re-filled by the warp's lane 0 right after the warp has read it.
// The new token is taken from the projection output (registers); its ring slot still holds the token that
// falls out of the window, is skipped while scanning and overwritten at the end.  Waits are bounded.
// -----------------------------------------------------------------------------------------------------
constexpr int kStreamStages = 3;
constexpr int kStreamChunkBytes = 2048;
constexpr int kStreamWarpBytes = kStreamStages * 2 * kStreamChunkBytes;
constexpr int stream_smem_bytes(int warps) { return warps * kStreamWarpBytes + warps * kStreamStages * 8; }
constexpr long long kStreamWaitCycles = 2000000000LL;  // about one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& a, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& a, float (&f)[8]) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void unpack16<__half>(const uint4& a, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&a);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// WPP = warps per pair.  1: two pairs per 64-thread CTA, nine CTAs per SM (all pairs of a large batch resident);
// 2 and 4: one pair per CTA, the warps take the chunks in turn and merge their partial results through shared
// memory at the end (smaller batches: more bytes in flight per pair).
template <typename T, int DH, int WPP>
__global__ void __launch_bounds__(WPP == 1 ? 64 : WPP * 32, WPP == 1 ? 9 : (WPP == 2 ? 9 : 4))
decode_stream_kernel(const DecodeParams p) {
    static_assert(sizeof(T) == 2, "the streaming variant is for 16-bit caches");
    constexpr int LPK = DH / 8;                    // lanes per key row
    constexpr int RPW = 32 / LPK;                  // key rows per warp per pass
    constexpr int ROWB = DH * 2;                   // bytes per row
    constexpr int CH = kStreamChunkBytes / ROWB;   // rows per chunk
    constexpr int PASSES = CH / RPW;
    static_assert(CH % RPW == 0 && PASSES >= 1, "chunk geometry");
    extern __shared__ __align__(128) unsigned char stream_smem[];

    constexpr int NW = WPP == 1 ? 2 : WPP;  // warps per CTA
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = WPP == 1 ? blockIdx.x * 2 + warp : blockIdx.x;
    const int wslot = WPP == 1 ? 0 : warp;  // which share of the chunks this warp scans
    if (pair >= p.batch * p.heads) return;  // WPP == 1 only (whole warps; those warps never synchronise)
    unsigned char* stage_mem = stream_smem + warp * kStreamWarpBytes;
    const uint32_t stage_u32 = smem_u32(stage_mem);
    const uint32_t bar0 = smem_u32(stream_smem + NW * kStreamWarpBytes) + warp * kStreamStages * 8;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kStreamStages; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar0 + s * 8), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    const int b = pair / p.heads, h = pair % p.heads;
    const int sub = lane % LPK, grp = lane / LPK;
    int t = p.pos[b];
    if (t < 0) {
        // a negative position would put the new row in front of the ring: treated as position 0 (nothing is
        // written out of bounds) and reported through the status word as an invalid argument
        if (lane == 0) atomicCAS(p.status, 0, (int)TMW_ERR_INVALID_ARGUMENT);
        t = 0;
    }
    const int slot_new = t % p.slots;
    const int count = min(t + 1, p.slots);
    const long long ring_bh = ((long long)b * p.heads + h) * p.slots * DH;
    T* kr = static_cast<T*>(p.k_ring) + ring_bh;
    T* vr = static_cast<T*>(p.v_ring) + ring_bh;
    const T* kp = static_cast<const T*>(p.k_pers) + (long long)h * p.np * DH;
    const T* vp = static_cast<const T*>(p.v_pers) + (long long)h * p.np * DH;
    const T* kn = static_cast<const T*>(p.k_new) + b * p.ns[0] + h * p.ns[1];
    const T* vn = static_cast<const T*>(p.v_new) + b * p.ns[0] + h * p.ns[1];

    // chunk c: persistent rows first, then the ring rows [0, count) in slot order
    const int n_pc = (p.np + CH - 1) / CH;
    const int n_chunks = n_pc + (count + CH - 1) / CH;
    auto chunk_rows = [&](int c, int& r0, bool& ring) -> int {
        ring = c >= n_pc;
        r0 = (ring ? c - n_pc : c) * CH;
        return min(CH, (ring ? count : p.np) - r0);
    };
    // this warp's chunks are wslot, wslot + WPP, ...; n counts them
    const int my_chunks = n_chunks > wslot ? (n_chunks - wslot + WPP - 1) / WPP : 0;
    auto issue = [&](int n) {  // lane 0
        int r0;
        bool ring;
        const int nr = chunk_rows(n * WPP + wslot, r0, ring);
        const uint32_t bytes = (uint32_t)nr * ROWB;
        const uint32_t bar = bar0 + (n % kStreamStages) * 8;
        const uint32_t dst = stage_u32 + (n % kStreamStages) * 2 * kStreamChunkBytes;
        const T* ksrc = (ring ? kr : kp) + (long long)r0 * DH;
        const T* vsrc = (ring ? vr : vp) + (long long)r0 * DH;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst), "l"(ksrc), "r"(bytes), "r"(bar) : "memory");
        asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(dst + kStreamChunkBytes), "l"(vsrc), "r"(bytes), "r"(bar) : "memory");
    };
    if (lane == 0)
        for (int n = 0; n < min(kStreamStages, my_chunks); ++n) issue(n);

    // the new token (every lane group computes its score, group 0 owns it)
    float qreg[8];
    load8<T>(static_cast<const T*>(p.q) + b * p.qs[0] + h * p.qs[1] + sub * 8, qreg);
    float m, l, acc[8];
    {
        float kf[8], vf[8];
        load8<T>(kn + sub * 8, kf);
        load8<T>(vn + sub * 8, vf);
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) part = fmaf(qreg[e], kf[e], part);
#pragma unroll
        for (int off = 1; off < LPK; off <<= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        const bool owner = grp == 0 && wslot == 0;
        m = owner ? part * p.scale_log2 : -CUDART_INF_F;
        l = owner ? 1.f : 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = owner ? vf[e] : 0.f;
    }

    bool failed = false;
    for (int n = 0; n < my_chunks; ++n) {
        const int stage = n % kStreamStages;
        const uint32_t bar = bar0 + stage * 8;
        const uint32_t parity = (uint32_t)(n / kStreamStages) & 1u;
        if (!__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) {  // the whole warp takes the slow path together
            const long long t0 = clock64();
            bool expired = false;
            while (!mbar_try_wait(bar, parity)) {
                if (clock64() - t0 > kStreamWaitCycles) {
                    expired = true;
                    break;
                }
            }
            if (__any_sync(0xffffffffu, expired)) {
                failed = true;
                break;
            }
        }
        int r0;
        bool ring;
        const int nr = chunk_rows(n * WPP + wslot, r0, ring);
        const unsigned char* ks = stage_mem + stage * 2 * kStreamChunkBytes;
        const unsigned char* vs = ks + kStreamChunkBytes;

        float s[PASSES];
        bool ok[PASSES];
        float tmax = -CUDART_INF_F;
#pragma unroll
        for (int u = 0; u < PASSES; ++u) {
            const int row = u * RPW + grp;
            ok[u] = row < nr && !(ring && r0 + row == slot_new);
            const uint4 raw = *reinterpret_cast<const uint4*>(ks + row * ROWB + sub * 16);
            float kf[8];
            unpack16<T>(raw, kf);
            float part = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) part = fmaf(qreg[e], kf[e], part);
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
            for (int u = 0; u < PASSES; ++u) {
                if (ok[u]) {
                    const float pj = exp2f(s[u] - m);
                    l += pj;
                    const uint4 raw = *reinterpret_cast<const uint4*>(vs + (u * RPW + grp) * ROWB + sub * 16);
                    float vf[8];
                    unpack16<T>(raw, vf);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(pj, vf[e], acc[e]);
                }
            }
        }
        __syncwarp();  // every lane has read the stage: it may be filled again
        if (lane == 0 && n + kStreamStages < my_chunks) issue(n + kStreamStages);
    }
    if (failed) {
        // a copy did not arrive in time: report, give copies that may still be in flight time to land in this
        // CTA's shared memory, and leave the cache and the output untouched
        if (lane == 0) atomicCAS(p.status, 0, (int)TMW_ERR_DEVICE_TIMEOUT);
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) __nanosleep(1000);
        if (WPP == 1) return;
    }
    if (WPP > 1) {
        // all warps of the pair have finished scanning (also the way out after a failed wait: nobody
        // is left behind at the barrier, and nothing is written)
        __shared__ int any_failed;
        if (threadIdx.x == 0) any_failed = 0;
        __syncthreads();
        if (failed && lane == 0) any_failed = 1;
        __syncthreads();
        if (any_failed) return;
    }

    // the new token's key and value go into their ring slot for the following steps
    if (grp == 0 && wslot == 0) {
        float tmp[8];
        load8<T>(kn + sub * 8, tmp);
        store8<T>(kr + (long long)slot_new * DH + sub * 8, tmp);
        load8<T>(vn + sub * 8, tmp);
        store8<T>(vr + (long long)slot_new * DH + sub * 8, tmp);
    }
    // merge the RPW lane groups of the warp (lanes that hold the same slice)
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
    T* out = static_cast<T*>(p.o) + b * p.os[0] + h * p.os[1];
    if (WPP == 1) {
        if (grp == 0) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            float res[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) res[e] = acc[e] * inv;
            store8<T>(out + sub * 8, res);
        }
    } else {
        // merge the warps through shared memory
        __shared__ float sm_m[NW], sm_l[NW];
        __shared__ float sm_acc[NW][DH];
        if (grp == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) sm_acc[warp][sub * 8 + e] = acc[e];
            if (sub == 0) {
                sm_m[warp] = m;
                sm_l[warp] = l;
            }
        }
        __syncthreads();
        if (threadIdx.x < LPK) {
            float m_all = -CUDART_INF_F;
#pragma unroll
            for (int w = 0; w < NW; ++w) m_all = fmaxf(m_all, sm_m[w]);
            float l_all = 0.f;
            float res[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float a = sm_m[w] > -CUDART_INF_F ? exp2f(sm_m[w] - m_all) : 0.f;
                l_all += sm_l[w] * a;
#pragma unroll
                for (int e = 0; e < 8; ++e) res[e] += sm_acc[w][threadIdx.x * 8 + e] * a;
            }
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) res[e] *= inv;
            store8<T>(out + threadIdx.x * 8, res);
        }
    }
}

template <typename T, int DH, int WPP>
int launch_decode_stream(const DecodeParams& p, cudaStream_t stream) {
    if constexpr (sizeof(T) == 2 && (DH == 64 || DH == 128)) {
        auto kern = decode_stream_kernel<T, DH, WPP>;
        // nine 64-thread CTAs with 24 KB each per SM: ask for the largest shared-memory carve-out, once per
        // device (so that later calls, e.g. under stream capture, only launch)
        static bool configured[64] = {false};
        int dev = 0;
        TMW_CUDA_TRY(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            TMW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
            TMW_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              stream_smem_bytes(WPP == 1 ? 2 : WPP)));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
        const int pairs = p.batch * p.heads;
        if (WPP == 1) kern<<<(pairs + 1) / 2, 64, stream_smem_bytes(2), stream>>>(p);
        else kern<<<pairs, WPP * 32, stream_smem_bytes(WPP), stream>>>(p);
        TMW_CUDA_TRY(cudaGetLastError());
        return TMW_OK;
    } else {
        return TMW_ERR_UNSUPPORTED;
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

template <typename T, int DH>
int launch_decode_shape(const DecodeParams& p, cudaStream_t stream) {
    const int pairs = p.batch * p.heads;
    if (p.splits > 0) {
        decode_kernel<T, DH, 4, true><<<pairs * p.splits, 128, 0, stream>>>(p);
        TMW_CUDA_TRY(cudaGetLastError());
        return TMW_OK;
    }
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // 16-bit caches whose rows are whole 16-byte units at 16-byte aligned addresses take the streaming variant
    constexpr bool kStreamShape = sizeof(T) == 2 && (DH == 64 || DH == 128);
    const bool aligned = (((uintptr_t)p.k_ring | (uintptr_t)p.v_ring | (uintptr_t)p.k_pers | (uintptr_t)p.v_pers) & 15) == 0;
    if (TMW_DECODE_STREAM && kStreamShape && aligned) {
        // every shape runs as a single wave: 2 pairs per CTA x 9 CTAs per SM, 1 pair per 2-warp CTA x 9, or
        // 1 pair per 4-warp CTA x 4 (measured, us per layer at window 512: 2560 pairs 60, 800 pairs 20.8,
        // 640 pairs 18.5, 480 pairs 14.3, 320 pairs 11.8, 160 pairs 8.9)
        if (pairs > 9 * sms) return launch_decode_stream<T, DH, 1>(p, stream);
        if (pairs > 4 * sms) return launch_decode_stream<T, DH, 2>(p, stream);
        if (pairs > sms / 2) return launch_decode_stream<T, DH, 4>(p, stream);
    }
    if (pairs > 9 * sms) {
        decode_kernel<T, DH, 1><<<(pairs + 1) / 2, 64, 0, stream>>>(p);
    } else if (pairs > 4 * sms) {
        decode_kernel<T, DH, 2><<<pairs, 64, 0, stream>>>(p);
    } else if (pairs > 2 * sms) {
        decode_kernel<T, DH, 4><<<pairs, 128, 0, stream>>>(p);
    } else {
        decode_kernel<T, DH, 8><<<pairs, 256, 0, stream>>>(p);
    }
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

template <typename T>
int launch_decode_dh(const DecodeParams& p, int dh, cudaStream_t stream) {
    switch (dh) {
        case 8: return launch_decode_shape<T, 8>(p, stream);
        case 16: return launch_decode_shape<T, 16>(p, stream);
        case 32: return launch_decode_shape<T, 32>(p, stream);
        case 64: return launch_decode_shape<T, 64>(p, stream);
        case 128: return launch_decode_shape<T, 128>(p, stream);
        case 256: return launch_decode_shape<T, 256>(p, stream);
        default: return TMW_ERR_UNSUPPORTED;
    }
}

}  // namespace

int launch_decode(const tmw_cache_desc& c, const void* q, const void* k_new, const void* v_new, void* o,
                  const int64_t qs[2], const int64_t ns[2], const int64_t os[2], const int32_t* pos,
                  int splits, float* scratch, unsigned int* counters, cudaStream_t stream) {
    if (c.batch == 0 || c.heads == 0) return TMW_OK;
    if ((long long)c.batch * c.heads > (1LL << 30)) return TMW_ERR_TOO_LARGE;
    DecodeParams p;
    p.k_ring = c.k_ring; p.v_ring = c.v_ring; p.k_pers = c.k_pers; p.v_pers = c.v_pers;
    p.q = q; p.k_new = k_new; p.v_new = v_new; p.o = o; p.pos = pos;
    for (int i = 0; i < 2; ++i) { p.qs[i] = qs[i]; p.ns[i] = ns[i]; p.os[i] = os[i]; }
    p.batch = c.batch; p.heads = c.heads; p.slots = c.window + 1; p.np = c.n_persistent;
    p.splits = splits; p.scratch = scratch; p.counters = counters;
    p.status = device_status_word();
    if (p.status == nullptr) return TMW_ERR_CUDA;
    const float scale = c.scale != 0.f ? c.scale : 1.0f / sqrtf((float)c.head_dim);
    p.scale_log2 = scale * 1.4426950408889634f;
    switch (c.dtype) {
        case TMW_F32: return launch_decode_dh<float>(p, c.head_dim, stream);
        case TMW_BF16: return launch_decode_dh<__nv_bfloat16>(p, c.head_dim, stream);
        case TMW_F16: return launch_decode_dh<__half>(p, c.head_dim, stream);
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

// -----------------------------------------------------------------------------------------------------
// Split decode without any allocation.
//
// Some hosts may not allocate device memory around a decode step: an inference server that has handed
// all HBM to its own pool and forbids cudaMalloc after start-up, or a latency-critical loop in which an
// allocation (a synchronising driver call) is unacceptable.  For them the scratch memory of the split
// launch is a fixed array inside this library.  It exists once per GPU that loads the library and stays
// until the process exits; its size is the limit of this entry point.
//
// In host code the array's NAME is only a handle for the runtime, not a device address.  The device
// address is asked for once per device (cudaGetSymbolAddress, with that device current) and kept.
// -----------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticCounterBytes = 16 * 1024;            // 4096 arrival counters, always at the start
constexpr size_t kStaticScratchBytes = 2 * 1024 * 1024;      // the whole array: counters, then partial results
constexpr int kStaticMaxPairs = (int)(kStaticCounterBytes / sizeof(unsigned int));
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// device address of the array on the current device; nullptr (and the CUDA error recorded) on failure
unsigned char* static_scratch_on_current_device() {
    constexpr int kMaxDevices = 64;
    // written once per device; two host threads making the first call on a device store the same value
    static std::atomic<unsigned char*> address[kMaxDevices];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        tmw::set_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevice, "cudaGetDevice");
        return nullptr;
    }
    if (address[dev].load(std::memory_order_acquire) == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
        if (e != cudaSuccess) {
            tmw::set_cuda_error(e, "cudaGetSymbolAddress(g_decode_static_scratch)");
            return nullptr;
        }
        address[dev].store(static_cast<unsigned char*>(ptr), std::memory_order_release);
    }
    return address[dev].load(std::memory_order_acquire);
}

}  // namespace

extern "C" int tmw_decode_split_static(const tmw_cache_desc* cache, const void* q, const void* k_new, const void* v_new,
                                       void* o, const int64_t q_stride[2], const int64_t kv_new_stride[2],
                                       const int64_t o_stride[2], const int32_t* pos, int32_t splits, void* stream) {
    const int rc = tmw::validate_decode_call(cache, q, k_new, v_new, o, q_stride, kv_new_stride, o_stride, pos);
    if (rc != TMW_OK) return rc;
    if (splits < 1 || splits > TMW_MAX_DECODE_SPLITS) return TMW_ERR_INVALID_ARGUMENT;
    if (cache->batch == 0 || cache->heads == 0) return TMW_OK;
    const long long pairs = (long long)cache->batch * cache->heads;
    const size_t partial_bytes = tmw::decode_partials_bytes(cache->batch, cache->heads, cache->head_dim, splits);
    if (pairs > kStaticMaxPairs || partial_bytes > kStaticScratchBytes - kStaticCounterBytes) {
        char text[200];
        std::snprintf(text, sizeof(text),
                      "tmw_decode_split_static: %lld pairs x %d splits need %zu bytes of partial results; the built-in "
                      "scratch memory holds %d pairs and %zu bytes",
                      pairs, (int)splits, partial_bytes, kStaticMaxPairs, kStaticScratchBytes - kStaticCounterBytes);
        tmw::set_error_text(text);
        return TMW_ERR_TOO_LARGE;
    }
    unsigned char* base = static_scratch_on_current_device();
    if (base == nullptr) return TMW_ERR_CUDA;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the last call left in it.  Partial results are rewritten completely by every
    // launch; the arrival counters must start at zero, so they are cleared here (an aborted earlier launch
    // could have left them half counted).
    TMW_CUDA_TRY(cudaMemsetAsync(base, 0, (size_t)pairs * sizeof(unsigned int), s));
    return tmw::launch_decode(*cache, q, k_new, v_new, o, q_stride, kv_new_stride, o_stride, pos, splits,
                              reinterpret_cast<float*>(base + kStaticCounterBytes),
                              reinterpret_cast<unsigned int*>(base), s);
}
