// Token selection on the device: argmax, and temperature sampling with optional top-k,
// top-p and repetition penalty, one block per row of 32-bit logits.
//
// Semantics follow emberserve/sampling.py:
//   :42-53    repetition penalty over the set of seen tokens: s > 0 ? s / p : s * p
//   :56-60    top-k by value: keep logits >= the k-th largest (ties at it survive)
//   :63-73    top-p: keep a token iff the probability mass of the tokens above it is < p
//   :110-145  greedy rows take the first maximum; the others divide by the temperature,
//             filter, take the softmax and draw one token
// The draw itself is ours: a counter-based generator (Philox4x32-10 keyed by the
// request's seed, counter = number of tokens the request has drawn so far) gives a
// uniform u, and the token is the first index whose cumulative probability exceeds u.
// So a request's tokens depend on its seed and logits only, not on the batch.
//
// No sorting: thresholds are found by a 4-pass radix descent over the order-preserving
// integer image of the floats; probability mass is accumulated in 64-bit fixed point so
// that the result does not depend on the order of the atomic additions.
#include "common.cuh"

namespace ems {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ uint4 philox4x32_10(uint2 key, uint4 ctr) {
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const unsigned hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const unsigned hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}

// first index of the maximum of x[0..V)
__device__ int block_argmax(const float* __restrict__ x, int V, float* red_v, int* red_i) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best || (v == best && i < bi) || bi == 0x7fffffff) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { red_v[warp] = best; red_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nwarps ? red_v[lane] : -INFINITY;
        bi = lane < nwarps ? red_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) red_i[32] = bi;
    }
    __syncthreads();
    return red_i[32];
}

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
    __shared__ float red_v[33];
    __shared__ int red_i[33];
    const int r = blockIdx.x;
    const int idx = block_argmax(logits + (size_t)r * V, V, red_v, red_i);
    if (threadIdx.x == 0) out[r] = idx;
}

// The same in two stages for few rows of a large vocabulary: blockIdx.y takes a slice of
// the row and leaves (ordered value, ~index) packed in 64 bits, largest first on ties of
// the value means smallest index; the second stage takes the maximum of the slices.
constexpr int ARGMAX_SLICE = 4096;

__global__ void argmax_slice_kernel(const float* __restrict__ logits, unsigned long long* __restrict__ tmp,
                                    int V, int slices) {
    __shared__ float red_v[33];
    __shared__ int red_i[33];
    const int r = blockIdx.x, sl = blockIdx.y;
    const int lo = sl * ARGMAX_SLICE, n = min(ARGMAX_SLICE, V - lo);
    const float* x = logits + (size_t)r * V + lo;
    const int idx = block_argmax(x, n, red_v, red_i);
    if (threadIdx.x == 0)
        tmp[(size_t)r * slices + sl] =
            ((unsigned long long)ordered_key(x[idx]) << 32) | (unsigned)(0x7fffffff - (lo + idx));
}

__global__ void argmax_merge_kernel(const unsigned long long* __restrict__ tmp, int* __restrict__ out,
                                    int slices) {
    const int r = blockIdx.x;
    unsigned long long best = 0;
    for (int i = threadIdx.x; i < slices; i += 32) best = max(best, tmp[(size_t)r * slices + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (threadIdx.x == 0) out[r] = 0x7fffffff - (int)(best & 0xffffffffull);
}

// logits[row, tok] = s > 0 ? s / penalty : s * penalty for every distinct tok of the row
__global__ void penalty_kernel(float* __restrict__ logits, int V, const int* __restrict__ row_ptr,
                               const int* __restrict__ token_ids, const float* __restrict__ penalty) {
    const int r = blockIdx.x;
    const float p = penalty[r];
    if (p == 1.0f) return;
    for (int i = row_ptr[r] + threadIdx.x; i < row_ptr[r + 1]; i += blockDim.x) {
        const int tok = token_ids[i];
        if (tok < 0 || tok >= V) continue;
        float* s = logits + (size_t)r * V + tok;
        *s = *s > 0.f ? *s / p : *s * p;
    }
}

struct SampleShared {
    float red[33];
    float red_v[33];
    int red_i[33];
    unsigned hist[256];
    unsigned long long mass[256];
    unsigned prefix, mask, remaining;
    unsigned long long mass_above;
    int crossed;
    float chunk[SAMPLE_THREADS];
    int found;
};

// One block per row.  temperature == 0 -> argmax.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ counters, int* __restrict__ out) {
    __shared__ SampleShared sh;
    const int r = blockIdx.x;
    const float* x = logits + (size_t)r * V;
    const float temp = temperature[r];
    if (temp == 0.f) {
        const int idx = block_argmax(x, V, sh.red_v, sh.red_i);
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }
    const int tid = threadIdx.x;
    // z = x / temp ; m = max z
    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x) mx = fmaxf(mx, x[i] / temp);
    mx = block_max(mx, sh.red);

    // ---- top-k: key of the k-th largest z -------------------------------------------
    unsigned thr_key = 0;  // keep keys >= thr_key
    const int k = top_k[r];
    if (k > 0 && k < V) {
        if (tid == 0) { sh.prefix = 0; sh.mask = 0; sh.remaining = (unsigned)k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < 256; i += blockDim.x) sh.hist[i] = 0;
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.mask;
            for (int i = tid; i < V; i += blockDim.x) {
                const unsigned key = ordered_key(x[i] / temp);
                if ((key & mask) == prefix) atomicAdd(&sh.hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned running = 0;
                int bsel = 0;
                for (int bin = 255; bin >= 0; --bin) {
                    if (running + sh.hist[bin] >= sh.remaining) { bsel = bin; break; }
                    running += sh.hist[bin];
                }
                sh.remaining -= running;
                sh.prefix = prefix | ((unsigned)bsel << shift);
                sh.mask = mask | (255u << shift);
            }
            __syncthreads();
        }
        thr_key = sh.prefix;
    }

    // ---- top-p over what top-k kept ---------------------------------------------------
    const float p = top_p[r];
    if (p < 1.0f) {
        // Z over the kept tokens, each thread a contiguous chunk, then a fixed-order sum
        const int per = (V + blockDim.x - 1) / blockDim.x;
        const int lo = min(V, tid * per), hi = min(V, lo + per);
        float z = 0.f;
        for (int i = lo; i < hi; ++i) {
            const float zi = x[i] / temp;
            if (ordered_key(zi) >= thr_key) z += expf(zi - mx);
        }
        const float Z = block_sum(z, sh.red);
        const float to_fixed = 1099511627776.0f / Z;  // 2^40 / Z
        const unsigned long long target = (unsigned long long)((double)p * 1099511627776.0);
        if (tid == 0) { sh.prefix = 0; sh.mask = 0; sh.mass_above = 0; sh.crossed = 1; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < 256; i += blockDim.x) sh.mass[i] = 0;
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.mask;
            for (int i = tid; i < V; i += blockDim.x) {
                const float zi = x[i] / temp;
                const unsigned key = ordered_key(zi);
                if (key >= thr_key && (key & mask) == prefix) {
                    const unsigned long long q = (unsigned long long)(expf(zi - mx) * to_fixed);
                    atomicAdd(&sh.mass[(key >> shift) & 255u], q);
                }
            }
            __syncthreads();
            if (tid == 0 && sh.crossed) {
                unsigned long long running = sh.mass_above;
                int bsel = -1;
                for (int bin = 255; bin >= 0; --bin) {
                    if (sh.mass[bin] == 0) continue;
                    if (running + sh.mass[bin] >= target) { bsel = bin; break; }
                    running += sh.mass[bin];
                }
                if (bsel < 0) {
                    sh.crossed = 0;  // rounding left the total below p: keep everything
                } else {
                    sh.mass_above = running;
                    sh.prefix = prefix | ((unsigned)bsel << shift);
                    sh.mask = mask | (255u << shift);
                }
            }
            __syncthreads();
        }
        if (sh.crossed) thr_key = max(thr_key, sh.prefix);
    }

    // ---- draw: first index whose cumulative probability exceeds u ----------------------
    const int per = (V + blockDim.x - 1) / blockDim.x;
    const int lo = min(V, tid * per), hi = min(V, lo + per);
    float part = 0.f;
    int last_kept = -1;
    for (int i = lo; i < hi; ++i) {
        const float zi = x[i] / temp;
        if (ordered_key(zi) >= thr_key) { part += expf(zi - mx); last_kept = i; }
    }
    sh.chunk[tid] = part;
    // last kept index of the row (fallback when rounding puts u*Z at or past the total)
    int lk = last_kept;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lk = max(lk, __shfl_xor_sync(0xffffffffu, lk, o));
    __syncthreads();
    if ((tid & 31) == 0) sh.red_i[tid >> 5] = lk;
    __syncthreads();
    if (tid == 0) {
        int best = -1;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) best = max(best, sh.red_i[w]);
        sh.found = best;
        // serial prefix over the chunk sums: the same order for every batch
        const uint4 rnd = philox4x32_10(
            make_uint2((unsigned)(seeds[r] & 0xffffffffull), (unsigned)(seeds[r] >> 32)),
            make_uint4((unsigned)(counters[r] & 0xffffffffull), (unsigned)(counters[r] >> 32), 0u, 0u));
        const float u = (float)(rnd.x >> 8) * (1.0f / 16777216.0f);
        float total = 0.f;
        for (int t = 0; t < (int)blockDim.x; ++t) total += sh.chunk[t];
        const float target = u * total;
        float run = 0.f;
        int sel = -1;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (run + sh.chunk[t] > target) { sel = t; break; }
            run += sh.chunk[t];
        }
        sh.red[0] = target - run;  // what is left to cover inside chunk `sel`
        sh.red_i[0] = sel;
    }
    __syncthreads();
    if (tid == sh.red_i[0]) {
        const float want = sh.red[0];
        float run = 0.f;
        int sel = last_kept;
        for (int i = lo; i < hi; ++i) {
            const float zi = x[i] / temp;
            if (ordered_key(zi) >= thr_key) {
                run += expf(zi - mx);
                if (run > want) { sel = i; break; }
            }
        }
        sh.found = sel;
    }
    __syncthreads();
    if (tid == 0) out[r] = sh.found;
}

}  // namespace ems

using namespace ems;

// Slices per row of the two-stage form; tmp must hold R * slices 64-bit words (0 = one stage).
EMS_EXPORT int ems_argmax_slices(int R, int V) {
    const int slices = (V + ARGMAX_SLICE - 1) / ARGMAX_SLICE;
    return (slices >= 4 && R * slices <= 65535 && R <= 256) ? slices : 0;
}

EMS_EXPORT int ems_argmax(const float* logits, int* out, int R, int V, unsigned long long* tmp,
                          cudaStream_t stream) {
    if (R <= 0) return EMS_OK;
    if (V <= 0) return EMS_ERR_SHAPE;
    const int slices = ems_argmax_slices(R, V);
    if (slices > 0 && tmp != nullptr) {
        argmax_slice_kernel<<<dim3(R, slices), 256, 0, stream>>>(logits, tmp, V, slices);
        argmax_merge_kernel<<<R, 32, 0, stream>>>(tmp, out, slices);
        return launch_status();
    }
    argmax_kernel<<<R, 1024, 0, stream>>>(logits, out, V);
    return launch_status();
}

EMS_EXPORT int ems_repetition_penalty(float* logits, int R, int V, const int* row_ptr,
                                      const int* token_ids, const float* penalty,
                                      cudaStream_t stream) {
    if (R <= 0) return EMS_OK;
    penalty_kernel<<<R, 256, 0, stream>>>(logits, V, row_ptr, token_ids, penalty);
    return launch_status();
}

EMS_EXPORT int ems_sample(const float* logits, int R, int V, const float* temperature,
                          const int* top_k, const float* top_p, const unsigned long long* seeds,
                          const unsigned long long* counters, int* out, cudaStream_t stream) {
    if (R <= 0) return EMS_OK;
    if (V <= 0) return EMS_ERR_SHAPE;
    sample_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, top_k, top_p, seeds,
                                                    counters, out);
    return launch_status();
}
