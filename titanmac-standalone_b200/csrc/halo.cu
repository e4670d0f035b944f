// Device-side halo exchange for the sequence-sharded prefill: a rank pushes K/V rows straight into a
// neighbour's buffer through a peer-mapped pointer (plain 16-byte stores over NVLink), fences, and raises a
// flag in the neighbour's memory; the neighbour's attention kernel polls that flag (bounded) right before the
// first TMA load that touches the rows.  No host-side collective is on the step, nothing is read from a peer's
// memory, and TMA only ever reads local memory.
//
// One launch serves one destination:  wait (bounded) until *wait_flag >= wait_value  - the destination has
// finished reading what the previous push wrote -,  copy,  __threadfence_system,  and the block that finishes
// last stores signal_value to *signal_flag with release semantics at system scope.
#include <cuda.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "tmw_common.cuh"

namespace tmw {
namespace {

constexpr int kMaxCopies = TMW_HALO_MAX_COPIES;
constexpr int kPushThreads = 256;

struct PushParams {
    const uint4* src[kMaxCopies];
    uint4* dst[kMaxCopies];
    unsigned long long chunks[kMaxCopies];  // 16-byte units
    int n_copies;
    const int* wait_flag;
    int wait_value;
    int* signal_flag;
    int signal_value;
    long long wait_limit_cycles;
    unsigned int* done_counter;  // blocks that have finished their share (library memory, reset by the last one)
    int* status;
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kPushThreads) halo_push_kernel(const PushParams p) {
    __shared__ int give_up;
    if (threadIdx.x == 0) {
        give_up = 0;
        if (p.wait_flag != nullptr) {
            // bounded: the flag lives in this GPU's memory and is written by the destination rank
            const long long t0 = clock64();
            while (ld_acquire_sys(p.wait_flag) < p.wait_value) {
                if (clock64() - t0 > p.wait_limit_cycles) {
                    give_up = 1;
                    if (atomicCAS(p.status, 0, (int)TMW_ERR_DEVICE_TIMEOUT) == 0) {
                        p.status[1] = -1;  // not an mbarrier: a halo flag
                        p.status[2] = (int)blockIdx.x;
                        p.status[3] = p.wait_value;
                    }
                    break;
                }
                __nanosleep(200);
            }
        }
    }
    __syncthreads();
    if (!give_up) {
        for (int c = 0; c < p.n_copies; ++c) {
            const uint4* src = p.src[c];
            uint4* dst = p.dst[c];
            const unsigned long long n = p.chunks[c];
            for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
                 i += (unsigned long long)gridDim.x * blockDim.x)
                dst[i] = src[i];
        }
    }
    // every thread's stores are ordered before the flag at system scope: fence, block barrier, then one
    // atomic per block; the last block to arrive raises the flag
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int arrived = atomicAdd(p.done_counter, 1u) + 1u;
        if (arrived == gridDim.x) {
            *p.done_counter = 0u;  // ready for the next launch on this stream
            __threadfence_system();
            if (p.signal_flag != nullptr && !give_up) st_release_sys(p.signal_flag, p.signal_value);
        }
    }
}

// one counter per device for the "last block" decision; launches that use it are ordered on the caller's stream
__device__ unsigned int g_push_counter[8];

}  // namespace
}  // namespace tmw

extern "C" int tmw_halo_push(const tmw_halo_copy* copies, int32_t n_copies, const int32_t* wait_flag,
                             int32_t wait_value, int32_t* signal_flag, int32_t signal_value, int64_t wait_limit_cycles,
                             void* stream) {
    using namespace tmw;
    if (n_copies < 0 || n_copies > kMaxCopies || (n_copies > 0 && copies == nullptr)) return TMW_ERR_INVALID_ARGUMENT;
    PushParams p = {};
    size_t total = 0;
    for (int i = 0; i < n_copies; ++i) {
        const tmw_halo_copy& c = copies[i];
        if (c.bytes == 0) {
            p.src[i] = nullptr; p.dst[i] = nullptr; p.chunks[i] = 0;
            continue;
        }
        if (c.src == nullptr || c.dst == nullptr || (reinterpret_cast<uintptr_t>(c.src) & 15u) ||
            (reinterpret_cast<uintptr_t>(c.dst) & 15u) || (c.bytes & 15u)) {
            set_error_text("tmw_halo_push: sources, destinations and sizes must be multiples of 16 bytes");
            return TMW_ERR_INVALID_ARGUMENT;
        }
        p.src[i] = static_cast<const uint4*>(c.src);
        p.dst[i] = static_cast<uint4*>(c.dst);
        p.chunks[i] = c.bytes / 16;
        total += c.bytes;
    }
    p.n_copies = n_copies;
    p.wait_flag = wait_flag;
    p.wait_value = wait_value;
    p.signal_flag = signal_flag;
    p.signal_value = signal_value;
    p.wait_limit_cycles = wait_limit_cycles > 0 ? wait_limit_cycles : 2000000000LL;
    p.status = device_status_word();
    if (p.status == nullptr) return TMW_ERR_CUDA;
    void* counter = nullptr;
    TMW_CUDA_TRY(cudaGetSymbolAddress(&counter, g_push_counter));
    p.done_counter = static_cast<unsigned int*>(counter);
    // enough blocks to keep the link busy, few enough to stay a side show next to the attention kernel
    int blocks = (int)((total / 16 + kPushThreads * 8 - 1) / (kPushThreads * 8));
    blocks = blocks < 1 ? 1 : blocks > 64 ? 64 : blocks;
    halo_push_kernel<<<blocks, kPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    TMW_CUDA_TRY(cudaGetLastError());
    return TMW_OK;
}

// Peer access from the current device to `peer_device` (stores of tmw_halo_push into that GPU's memory need it).
// Idempotent: an access that is already enabled is not an error.
extern "C" int tmw_enable_peer_access(int32_t peer_device) {
    int dev = 0;
    TMW_CUDA_TRY(cudaGetDevice(&dev));
    if (peer_device == dev) return TMW_OK;
    int can = 0;
    TMW_CUDA_TRY(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    if (!can) {
        tmw::set_error_text("tmw_enable_peer_access: the two devices have no peer path");
        return TMW_ERR_UNSUPPORTED;
    }
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return TMW_OK;
    }
    TMW_CUDA_TRY(e);
    return TMW_OK;
}

// ---------------------------------------------------------------------------------
// Mapping another process's device memory (one process per GPU on one node).  The exporting rank describes the
// allocation that holds its buffer (CUDA IPC handle + the buffer's offset inside it); the importing rank opens
// it WITH ITS OWN DEVICE CURRENT, which is what makes the returned address valid for kernels that run on the
// importing GPU (a mapping opened under the exporter's device index is not).  An allocation can be opened only
// once per process, so the mappings are kept and handed out again.
// ---------------------------------------------------------------------------------
namespace tmw {
namespace {

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

GetAddressRangeFn address_range_fn() {
    static GetAddressRangeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<GetAddressRangeFn>(ptr);
    });
    return fn;
}

struct OpenMapping {
    cudaIpcMemHandle_t handle;
    int device;
    void* base;
};
std::mutex g_ipc_mutex;
std::vector<OpenMapping> g_ipc_open;

}  // namespace
}  // namespace tmw

extern "C" int tmw_ipc_export(const void* ptr, tmw_ipc_mem* out) {
    using namespace tmw;
    if (ptr == nullptr || out == nullptr) return TMW_ERR_INVALID_ARGUMENT;
    GetAddressRangeFn range = address_range_fn();
    if (range == nullptr) return TMW_ERR_CUDA;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) {
        set_error_text("tmw_ipc_export: not a device allocation of this process");
        return TMW_ERR_INVALID_ARGUMENT;
    }
    cudaIpcMemHandle_t h;
    TMW_CUDA_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    static_assert(sizeof(h) == sizeof(out->handle), "handle size");
    std::memcpy(out->handle, &h, sizeof(h));
    out->offset = (uint64_t)(reinterpret_cast<uintptr_t>(ptr) - (uintptr_t)base);
    out->size = (uint64_t)size;
    return TMW_OK;
}

extern "C" int tmw_ipc_open(const tmw_ipc_mem* mem, void** ptr) {
    using namespace tmw;
    if (mem == nullptr || ptr == nullptr || mem->offset >= mem->size) return TMW_ERR_INVALID_ARGUMENT;
    int dev = 0;
    TMW_CUDA_TRY(cudaGetDevice(&dev));
    cudaIpcMemHandle_t h;
    std::memcpy(&h, mem->handle, sizeof(h));
    std::lock_guard<std::mutex> lock(g_ipc_mutex);
    for (const OpenMapping& m : g_ipc_open)
        if (m.device == dev && std::memcmp(&m.handle, &h, sizeof(h)) == 0) {
            *ptr = static_cast<char*>(m.base) + mem->offset;
            return TMW_OK;
        }
    void* base = nullptr;
    TMW_CUDA_TRY(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    g_ipc_open.push_back(OpenMapping{h, dev, base});
    *ptr = static_cast<char*>(base) + mem->offset;
    return TMW_OK;
}

extern "C" int tmw_ipc_close_all(void) {
    using namespace tmw;
    std::lock_guard<std::mutex> lock(g_ipc_mutex);
    int rc = TMW_OK;
    for (const OpenMapping& m : g_ipc_open) {
        int cur = 0;
        if (cudaGetDevice(&cur) != cudaSuccess || cudaSetDevice(m.device) != cudaSuccess ||
            cudaIpcCloseMemHandle(m.base) != cudaSuccess)
            rc = TMW_ERR_CUDA;
        (void)cudaSetDevice(cur);
    }
    g_ipc_open.clear();
    if (rc != TMW_OK) set_cuda_error(cudaGetLastError(), "cudaIpcCloseMemHandle");
    return rc;
}
