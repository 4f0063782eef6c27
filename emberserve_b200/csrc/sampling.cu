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

// hist[bin] += 1 (or mass[bin] += q) for the lanes with `valid`, one atomic per distinct bin of
// the warp: the scores of a row crowd into a few bins, and a shared-memory atomic per element on
// the same few words (64-bit ones are compare-and-swap loops) was most of the kernel's time.
// Every lane of the warp calls these.
__device__ __forceinline__ void warp_hist_add(unsigned* hist, bool valid, unsigned bin) {
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? bin : 0xffffffffu);
    if (valid && (threadIdx.x & 31) == (unsigned)(__ffs(peers) - 1)) atomicAdd(&hist[bin], (unsigned)__popc(peers));
}
// `qf` is the element's probability in 2^-40 units as a float in [0, 2^40]; what is added is
// floor(qf), split as a * 2^20 + b so that two 32-bit conversions and two 32-bit warp sums do
// (a <= 2^20 and b < 2^20, so sums over 32 lanes fit).
__device__ __forceinline__ void warp_mass_add(unsigned long long* mass, bool valid, unsigned bin, float qf) {
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? bin : 0xffffffffu);
    const unsigned a = (unsigned)(qf * 9.5367431640625e-07f);          // floor(qf / 2^20)
    const unsigned b = (unsigned)(qf - (float)a * 1048576.0f);          // exact: both are multiples of qf's ulp
    const unsigned sa = __reduce_add_sync(peers, a), sb = __reduce_add_sync(peers, b);
    if (valid && (threadIdx.x & 31) == (unsigned)(__ffs(peers) - 1))
        atomicAdd(&mass[bin], ((unsigned long long)sa << 20) + sb);
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
            for (int i0 = 0; i0 < V; i0 += blockDim.x) {  // whole warps stay in the loop
                const int i = i0 + tid;
                const unsigned key = i < V ? ordered_key(x[i] / temp) : 0u;
                const bool valid = i < V && (key & mask) == prefix;
                if (!__any_sync(0xffffffffu, valid)) continue;
                warp_hist_add(sh.hist, valid, (key >> shift) & 255u);
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
            for (int i0 = 0; i0 < V; i0 += blockDim.x) {
                const int i = i0 + tid;
                const float zi = i < V ? x[i] / temp : 0.f;
                const unsigned key = ordered_key(zi);
                const bool valid = i < V && key >= thr_key && (key & mask) == prefix;
                if (!__any_sync(0xffffffffu, valid)) continue;
                warp_mass_add(sh.mass, valid, (key >> shift) & 255u, valid ? expf(zi - mx) * to_fixed : 0.f);
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
        sh.red_i[0] = 0x7fffffff;
    }
    // prefix sums of the chunk sums, the same tree for every batch: inside each warp by shuffles,
    // then over the warps' totals
    const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    float incl = part;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) sh.red[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? sh.red[lane] : 0.f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        sh.red_v[lane] = w;  // inclusive totals of the warps
    }
    __syncthreads();
    const float before_warp = warp > 0 ? sh.red_v[warp - 1] : 0.f;
    incl += before_warp;
    const float total = sh.red_v[nwarps - 1];
    const uint4 rnd = philox4x32_10(
        make_uint2((unsigned)(seeds[r] & 0xffffffffull), (unsigned)(seeds[r] >> 32)),
        make_uint4((unsigned)(counters[r] & 0xffffffffull), (unsigned)(counters[r] >> 32), 0u, 0u));
    const float u = (float)(rnd.x >> 8) * (1.0f / 16777216.0f);
    const float target = u * total;
    if (incl > target) atomicMin(&sh.red_i[0], tid);  // the first chunk whose prefix passes the target
    __syncthreads();
    if (tid == sh.red_i[0]) sh.red[0] = target - (incl - part);  // what is left to cover inside it
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


// ---------------------------------------------------------------------------------------
// The same selection with a row spread over a thread-block cluster of 8 blocks.  One block per
// row leaves all but a few SMs idle at decode batch sizes and makes a dozen passes over the row
// from global memory, dividing by the temperature in each.  Here every block keeps its slice of
// z = x / temperature in shared memory (read and divided once) and the blocks of a row exchange
// their partial results (maxima, histograms, sums) through distributed shared memory.  All the
// combinations are in rank order or of integers, so the token drawn is the same as from the
// one-block kernel up to the order of the 32-bit additions of the draw.

constexpr int SC_CLUSTER = 8;
constexpr int SC_THREADS = 1024;

__device__ __forceinline__ void sc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned sc_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned sc_remote(const void* local, unsigned rank) {
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ unsigned sc_ld_u32(const void* local, unsigned rank) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(sc_remote(local, rank)) : "memory");
    return v;
}
__device__ __forceinline__ float sc_ld_f32(const void* local, unsigned rank) { return __uint_as_float(sc_ld_u32(local, rank)); }
__device__ __forceinline__ unsigned long long sc_ld_u64(const void* local, unsigned rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(sc_remote(local, rank)) : "memory");
    return v;
}

struct ClusterShared {
    float red[33];
    float red_v[33];
    int red_i[33];
    unsigned hist[2][256];             // this block's counts, two buffers used in turn
    unsigned long long mass[2][256];   // this block's probability mass (2^-40 units)
    unsigned ghist[256];               // the row's counts / mass, summed over the cluster
    unsigned long long gmass[256];
    float pub_f[2][2];                 // values published to the cluster, two slots used in turn
    int pub_i[2][2];
    unsigned prefix, mask, remaining;
    unsigned long long mass_above;
    int crossed, found, turn;
};

__global__ void __cluster_dims__(SC_CLUSTER, 1, 1) __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                      const unsigned long long* __restrict__ seeds,
                      const unsigned long long* __restrict__ counters, int* __restrict__ out) {
    __shared__ ClusterShared sh;
    extern __shared__ float zs[];  // this block's slice of z
    const int r = blockIdx.y, tid = threadIdx.x;
    const unsigned rank = sc_cluster_rank();
    const float* x = logits + (size_t)r * V;
    const float temp = temperature[r];
    const int per = (V + SC_CLUSTER - 1) / SC_CLUSTER;
    const int lo = min(V, (int)rank * per), n = min(V, lo + per) - lo;  // the slice [lo, lo + n)
    int phase = 0;  // which of the two published slots / histogram buffers is in use

    if (temp == 0.f) {  // greedy row: first maximum of the row
        const int idx = n > 0 ? block_argmax(x + lo, n, sh.red_v, sh.red_i) : 0;
        if (tid == 0) { sh.pub_f[0][0] = n > 0 ? x[lo + idx] : -INFINITY; sh.pub_i[0][0] = lo + idx; }
        sc_cluster_sync();
        if (rank == 0 && tid == 0) {
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (unsigned c = 0; c < SC_CLUSTER; ++c) {
                const float v = sc_ld_f32(&sh.pub_f[0][0], c);
                const int i = (int)sc_ld_u32(&sh.pub_i[0][0], c);
                if (v > best || (v == best && i < bi) || bi == 0x7fffffff) { best = v; bi = i; }
            }
            out[r] = bi;
        }
        sc_cluster_sync();  // nobody leaves while rank 0 may still read its shared memory
        return;
    }

    // ---- z = x / temp into shared memory, and the row's maximum -----------------------------
    float mx = -INFINITY;
    for (int i = tid; i < n; i += SC_THREADS) {
        const float z = x[lo + i] / temp;
        zs[i] = z;
        mx = fmaxf(mx, z);
    }
    mx = block_max(mx, sh.red);
    if (tid == 0) sh.pub_f[phase][0] = mx;
    sc_cluster_sync();
    mx = -INFINITY;
    for (unsigned c = 0; c < SC_CLUSTER; ++c) mx = fmaxf(mx, sc_ld_f32(&sh.pub_f[phase][0], c));
    phase ^= 1;

    // ---- top-k: key of the k-th largest z -----------------------------------------------------
    unsigned thr_key = 0;  // keep keys >= thr_key
    const int k = top_k[r];
    if (k > 0 && k < V) {
        if (tid == 0) { sh.prefix = 0; sh.mask = 0; sh.remaining = (unsigned)k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            unsigned* hist = sh.hist[phase];
            for (int i = tid; i < 256; i += SC_THREADS) hist[i] = 0;
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.mask;
            for (int i0 = 0; i0 < n; i0 += SC_THREADS) {  // whole warps stay in the loop
                const int i = i0 + tid;
                const unsigned key = i < n ? ordered_key(zs[i]) : 0u;
                const bool valid = i < n && (key & mask) == prefix;
                if (!__any_sync(0xffffffffu, valid)) continue;  // after the first pass few elements match
                warp_hist_add(hist, valid, (key >> shift) & 255u);
            }
            sc_cluster_sync();
            if (tid < 256) {
                unsigned total = 0;
                for (unsigned c = 0; c < SC_CLUSTER; ++c) total += sc_ld_u32(&hist[tid], c);
                sh.ghist[tid] = total;
            }
            __syncthreads();
            if (tid == 0) {  // every block of the row takes the same decision
                unsigned running = 0;
                int bsel = 0;
                for (int bin = 255; bin >= 0; --bin) {
                    if (running + sh.ghist[bin] >= sh.remaining) { bsel = bin; break; }
                    running += sh.ghist[bin];
                }
                sh.remaining -= running;
                sh.prefix = prefix | ((unsigned)bsel << shift);
                sh.mask = mask | (255u << shift);
            }
            __syncthreads();
            phase ^= 1;
        }
        thr_key = sh.prefix;
    }

    // ---- top-p over what top-k kept -------------------------------------------------------------
    const int cper = (n + SC_THREADS - 1) / SC_THREADS;       // a thread's contiguous chunk of the slice
    const int clo = min(n, tid * cper), chi = min(n, clo + cper);
    const float p = top_p[r];
    if (p < 1.0f) {
        float z = 0.f;
        for (int i = clo; i < chi; ++i)
            if (ordered_key(zs[i]) >= thr_key) z += expf(zs[i] - mx);
        z = block_sum(z, sh.red);
        if (tid == 0) sh.pub_f[phase][0] = z;
        sc_cluster_sync();
        float Z = 0.f;
        for (unsigned c = 0; c < SC_CLUSTER; ++c) Z += sc_ld_f32(&sh.pub_f[phase][0], c);  // rank order
        phase ^= 1;
        const float to_fixed = 1099511627776.0f / Z;  // 2^40 / Z
        const unsigned long long target = (unsigned long long)((double)p * 1099511627776.0);
        if (tid == 0) { sh.prefix = 0; sh.mask = 0; sh.mass_above = 0; sh.crossed = 1; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            unsigned long long* mass = sh.mass[phase];
            for (int i = tid; i < 256; i += SC_THREADS) mass[i] = 0;
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.mask;
            for (int i0 = 0; i0 < n; i0 += SC_THREADS) {
                const int i = i0 + tid;
                const float zi = i < n ? zs[i] : 0.f;
                const unsigned key = ordered_key(zi);
                const bool valid = i < n && key >= thr_key && (key & mask) == prefix;
                if (!__any_sync(0xffffffffu, valid)) continue;
                warp_mass_add(mass, valid, (key >> shift) & 255u, valid ? expf(zi - mx) * to_fixed : 0.f);
            }
            sc_cluster_sync();
            if (tid < 256) {
                unsigned long long total = 0;
                for (unsigned c = 0; c < SC_CLUSTER; ++c) total += sc_ld_u64(&mass[tid], c);
                sh.gmass[tid] = total;
            }
            __syncthreads();
            if (tid == 0 && sh.crossed) {
                unsigned long long running = sh.mass_above;
                int bsel = -1;
                for (int bin = 255; bin >= 0; --bin) {
                    if (sh.gmass[bin] == 0) continue;
                    if (running + sh.gmass[bin] >= target) { bsel = bin; break; }
                    running += sh.gmass[bin];
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
            phase ^= 1;
        }
        if (sh.crossed) thr_key = max(thr_key, sh.prefix);
    }

    // ---- draw: first index whose cumulative probability exceeds u ---------------------------------
    float part = 0.f;
    int last_kept = -1;
    for (int i = clo; i < chi; ++i)
        if (ordered_key(zs[i]) >= thr_key) { part += expf(zs[i] - mx); last_kept = lo + i; }
    const int lane = tid & 31, warp = tid >> 5;
    float incl = part;  // prefix sums of the chunk sums, the same tree for every batch
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    int lk = last_kept;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lk = max(lk, __shfl_xor_sync(0xffffffffu, lk, o));
    if (lane == 31) sh.red[warp] = incl;
    if (lane == 0) sh.red_i[warp] = lk;
    __syncthreads();
    if (warp == 0) {
        float w = sh.red[lane];
        int l = sh.red_i[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l = max(l, __shfl_xor_sync(0xffffffffu, l, o));
        sh.red_v[lane] = w;  // inclusive totals of the warps
        if (lane == 0) sh.pub_i[phase][0] = l;  // this block's last kept index
    }
    __syncthreads();
    if (tid == 0) sh.pub_f[phase][0] = sh.red_v[31];  // this block's total
    incl += warp > 0 ? sh.red_v[warp - 1] : 0.f;
    sc_cluster_sync();
    float before = 0.f, total = 0.f;
    int last_of_row = -1;
    for (unsigned c = 0; c < SC_CLUSTER; ++c) {  // rank order = index order
        const float t = sc_ld_f32(&sh.pub_f[phase][0], c);
        if (c < rank) before += t;
        total += t;
        last_of_row = max(last_of_row, (int)sc_ld_u32(&sh.pub_i[phase][0], c));
    }
    phase ^= 1;
    const uint4 rnd = philox4x32_10(
        make_uint2((unsigned)(seeds[r] & 0xffffffffull), (unsigned)(seeds[r] >> 32)),
        make_uint4((unsigned)(counters[r] & 0xffffffffull), (unsigned)(counters[r] >> 32), 0u, 0u));
    const float u = (float)(rnd.x >> 8) * (1.0f / 16777216.0f);
    const float target = u * total;
    if (tid == 0) sh.found = 0x7fffffff;
    __syncthreads();
    if (before + incl > target) atomicMin(&sh.found, (int)rank * SC_THREADS + tid);  // first chunk past the target
    __syncthreads();
    if (tid == 0) sh.pub_i[phase][0] = sh.found;
    sc_cluster_sync();
    int first = 0x7fffffff;
    for (unsigned c = 0; c < SC_CLUSTER; ++c) first = min(first, (int)sc_ld_u32(&sh.pub_i[phase][0], c));
    if (first == 0x7fffffff) {  // rounding put u * total at or past the total: the last kept token
        if (rank == 0 && tid == 0) out[r] = last_of_row;
    } else if (first == (int)rank * SC_THREADS + tid) {
        const float want = target - (before + incl - part);  // what is left to cover inside this chunk
        float run = 0.f;
        int sel = last_kept;
        for (int i = clo; i < chi; ++i) {
            if (ordered_key(zs[i]) >= thr_key) {
                run += expf(zs[i] - mx);
                if (run > want) { sel = lo + i; break; }
            }
        }
        out[r] = sel;
    }
    sc_cluster_sync();  // nobody leaves while a peer may still read its shared memory
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
    // A large vocabulary is spread over a cluster of blocks per row, each holding its slice of
    // the row in shared memory; small ones (and slices that would not fit) take one block per row.
    const size_t slice_bytes = (size_t)((V + SC_CLUSTER - 1) / SC_CLUSTER) * sizeof(float);
    if (V >= 8192 && slice_bytes <= 160 * 1024 && R <= 65535) {
        static int raised_on = -1;  // once per device
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return EMS_ERR_LAUNCH;
        if (raised_on != device) {
            if (cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     160 * 1024) != cudaSuccess)
                return EMS_ERR_LAUNCH;
            raised_on = device;
        }
        sample_cluster_kernel<<<dim3(SC_CLUSTER, R), SC_THREADS, slice_bytes, stream>>>(
            logits, V, temperature, top_k, top_p, seeds, counters, out);
        return launch_status();
    }
    sample_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, top_k, top_p, seeds,
                                                    counters, out);
    return launch_status();
}
