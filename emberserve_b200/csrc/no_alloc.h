// ems_paged_attention_static_scratch: split-key paged decode attention for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in the reference (ashwinsreedhar28/emberserve is
// Python over torch and always allocates through torch); it exists for users of this
// library only.
//
// Who needs it.  ems_paged_attention with `splits` > 1 wants a scratch buffer for the
// partial results of the splits, and leaves it to the caller to allocate one.  Some
// callers cannot: a serving process that has handed all GPU memory to a pool with a fixed
// plan (a cudaMalloc there fails, or breaks the plan); a latency-bound loop in which
// cudaMalloc / cudaFree are forbidden because they synchronise the whole device; a plain C,
// Rust or Go program that links the .so and has no tensor library to allocate with.  For
// them the scratch lives inside the library, in a file-scope
// `static __device__ __align__(256)` array of EMS_STATIC_SCRATCH_BYTES (8 MiB).  Every GPU
// on which the library's code is loaded holds those 8 MiB until the process exits.
//
// Contract.
//  * Same arguments and same results as ems_paged_attention, without `scratch` and
//    `scratch_bytes`.  The caller still passes inputs and outputs.  It calls no cudaMalloc,
//    no cudaFree and no allocating library routine.
//  * Sizes: N * nh * splits * (D + 2) * 4 bytes must fit in EMS_STATIC_SCRATCH_BYTES;
//    otherwise the call launches nothing and returns EMS_ERR_SCRATCH (4).  With splits == 1
//    no scratch is used and any size passes.
//  * Set-up happens inside the first call on each device: with that device current, the
//    address of the array is taken with cudaGetSymbolAddress (in host code the array's name
//    is only a stand-in, not a device address) and kept.  Make that first call before any
//    stream capture.  If taking the address fails the call returns EMS_ERR_LAUNCH (3).
//    With CUDA's lazy module loading the array itself may only come to exist on a device when
//    this part of the library is first used there: a caller whose pool takes all free memory
//    makes the first call on each device BEFORE the pool does, or that call fails with
//    EMS_ERR_LAUNCH.  The address is kept for the life of the process and is stale after a
//    cudaDeviceReset: do not reset a device on which this entry point has been called.
//  * In bfloat16 with head sizes 64 / 128 the kernel is launched as a programmatic dependent
//    of the kernel before it in the stream: it requests every cached key and value tile
//    except each row's newest 16-key tile before it waits for that kernel.  A preceding kernel
//    that signals early (cudaTriggerProgrammaticLaunchCompletion, griddepcontrol.launch_dependents)
//    may therefore write only each row's newest key and value; one that writes older cache
//    positions must not signal early (an ordinary kernel never does).
//  * All calls on a device share the one array, and it keeps what the last call left in
//    it.  Nothing in it has to start at zero: every partial result that the merge step
//    reads is written earlier in the same call.  Two calls that may run at the same time on
//    one GPU (different streams, different threads) race on the array: order them.
#pragma once

#include <cuda_runtime.h>

#define EMS_STATIC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int ems_paged_attention_static_scratch(
    const void* q, long long q_stride, void* out, int dtype, const void* kcache, const void* vcache,
    const int* block_tables, int bt_stride, int page_size, const int* cu_q, const int* starts, int B,
    int N, int nh, int nkv, int D, int window, float scale, int max_q_len, int splits,
    cudaStream_t stream);

// The fixed capacity in bytes (EMS_STATIC_SCRATCH_BYTES), for callers that want to size
// `splits` to it.
long long ems_static_scratch_capacity(void);

#ifdef __cplusplus
}
#endif
