// Shared helpers of the emberserve_b200 kernels (sm_100a only).
//
// Every launcher is an extern "C" function that takes raw device pointers, plain
// integers and a cudaStream_t, and returns 0 or one of the EMS_ERR_* codes below; the
// Python side (emberserve_b200/kernels.py) turns a non-zero code into an exception.
// Element types are passed as EMS_F32 / EMS_BF16 codes so that one entry point serves
// the true 32-bit path and the bfloat16 path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define EMS_F32 0
#define EMS_BF16 1

#define EMS_OK 0
#define EMS_ERR_DTYPE 1        // unknown element type code
#define EMS_ERR_SHAPE 2        // a size this kernel does not take
#define EMS_ERR_LAUNCH 3       // cudaGetLastError() after the launch was not cudaSuccess
#define EMS_ERR_SCRATCH 4      // scratch buffer too small
#define EMS_ERR_ALIGN 5        // pointer or stride not aligned as the kernel needs

#define EMS_EXPORT extern "C" __attribute__((visibility("default")))

namespace ems {

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Round a 32-bit value to the storage type and back: the value a later kernel reads.
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

// Load element i of an array whose element type is only known at run time.
__device__ __forceinline__ float load_any(const void* p, int dtype, size_t i) {
    return dtype == EMS_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

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

// Sum over the block; every thread gets the result.  `red` holds >= 33 floats.  The
// order of the additions depends only on blockDim, never on other rows of the batch.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // protect `red` from a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Lets a kernel that was launched as a programmatic dependent of this one (the tcgen05 GEMM
// that follows a norm, an attention or an activation kernel) start its prologue and its
// weight loads while this kernel still runs; that kernel waits before it reads our output.
// A no-op when nothing of the kind follows.
__device__ __forceinline__ void allow_dependent_launch() { asm volatile("griddepcontrol.launch_dependents;" ::); }

// First statement of a kernel that is launched with launch_pdl(): let the kernel after this
// one be scheduled early, then wait until the kernel before this one has completed (and its
// writes are visible).  Every kernel of a chain waits, so completion is transitive.
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::);
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? EMS_OK : EMS_ERR_LAUNCH; }

// Launch as a programmatic dependent of the kernel before it in the stream: the blocks may be
// scheduled while that kernel drains, which hides launch latency in chains of short kernels.
// The kernel must begin with pdl_prologue().
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) != cudaSuccess) {
        cudaGetLastError();
        return EMS_ERR_LAUNCH;
    }
    return launch_status();
}

}  // namespace ems
