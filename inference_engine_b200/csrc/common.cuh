// Shared helpers for the engine's kernels (sm_100a).
//
// Every exported function is plain C (`extern "C"`), takes raw device pointers and the
// stream to launch on, allocates nothing, and returns a cudaError_t as int.  Kernels never
// trap: an index that is out of range (a token id, a page, a slot) is recorded in a device
// error word and the access is skipped, so the context stays usable and the host can report
// what went wrong (the caller owns the error word and reads it when it likes).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define IE_API extern "C" __attribute__((visibility("default")))

enum IeDtype { IE_F32 = 0, IE_BF16 = 1 };

enum IeError {
    IE_OK = 0,
    IE_ERR_TOKEN_ID = 1,   // a token id outside the vocabulary
    IE_ERR_PAGE = 2,       // a page or slot outside the cache
    IE_ERR_POSITION = 3,   // a position outside the rotary table
    IE_ERR_TABLE = 4,      // a block-table entry that was given back (-1) was read
    IE_ERR_TIMEOUT = 5,    // a bounded wait inside a kernel ran out (value, where = block x, y)
};

// Every launch gets `err`, four ints in device memory owned by the caller:
// [0] = first error code seen, [1] = the offending value, [2] = where (row / token).
__device__ __forceinline__ void ie_report(int* err, int code, int value, int where) {
    if (err != nullptr && atomicCAS(&err[0], 0, code) == 0) {
        err[1] = value;
        err[2] = where;
    }
}

__device__ __forceinline__ float ie_load(const float* p) { return *p; }
__device__ __forceinline__ float ie_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void ie_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void ie_store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

#define IE_LAUNCH_CHECK() ((int)cudaGetLastError())

// Programmatic dependent launch.  A kernel launched with `ie_launch` may be scheduled while
// the kernel before it in the stream is still running (once all of that kernel's blocks have
// called ie_pdl_trigger or exited), so its launch latency and whatever it does before
// ie_pdl_wait -- index arithmetic, prefetching weights, which no earlier kernel writes --
// overlap the predecessor.  ie_pdl_wait returns when the predecessor grid has completed and its
// writes are visible; every kernel calls it before its first read of activations and before any
// global write, and every thread calls it, so "my predecessor is done" holds transitively.
__device__ __forceinline__ void ie_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ie_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::); }

// 1 (default): launch with the programmatic-serialization attribute; 0: plain launches.
inline int& ie_pdl_enabled() {
    static int enabled = 1;
    return enabled;
}

// The same launch as a grid of thread-block clusters of (cx, cy, cz) blocks: the blocks of a cluster
// run at the same time and can write into each other's shared memory.
template <typename... KArgs, typename... Args>
inline int ie_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ie_pdl_enabled() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// What is set on a kernel function (its dynamic shared memory limit) or asked of a device (its SM
// count) holds for the device that was current at the time, so "done already" is kept per device.
constexpr int IE_MAX_DEVICES = 64;
struct IePerDevice {
    bool done[IE_MAX_DEVICES] = {};
};

template <typename Kernel>
inline cudaError_t ie_allow_smem(IePerDevice& state, Kernel kernel, size_t bytes) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    bool known = dev >= 0 && dev < IE_MAX_DEVICES;
    if (known && state.done[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess && known) state.done[dev] = true;
    return e;
}

// SMs of the current device (148 if the runtime cannot say).
inline int ie_sm_count() {
    static int sms[IE_MAX_DEVICES] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= IE_MAX_DEVICES) return 148;
    if (sms[dev] == 0 &&
        (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0))
        sms[dev] = 148;
    return sms[dev];
}

template <typename... KArgs, typename... Args>
inline int ie_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                     Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ie_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
