// y = x W^T (+ bias) for 17..128 rows of x: decode steps of many requests, short prompt
// portions, and steps that mix the two.  Still a bandwidth problem (every weight is read once
// and used a few dozen times), but with other proportions than at 1..16 rows: the activation
// tile of a stage is as large as the weight tile, and the float32 partials of a split K are
// 16..64 KB per block.  So this kernel keeps ONE block per SM with a ring as deep as shared
// memory allows (5..10 stages, 80..160 KB of weights in flight per SM), splits K only as far as
// all blocks of the product still start in one wave, and the owner of a share of the output
// rows keeps its own partial in the ring memory it has finished with instead of in the inbox.
//
// As in the kernel for few rows (gemm_tcgen05.cu) the WEIGHT matrix is on the 128-row side of
// tcgen05.mma and the tokens on its N side (32, 64 or 128 columns); weight and activation
// tiles arrive by TMA (128-byte swizzle, no multicast), the first ring of weight tiles before
// the wait on the kernel before.  The blocks that share K are a thread-block cluster: each lays
// its partial sums out in its ring memory, one slab per owner, and one bulk copy per owner
// (cp.async.bulk from shared memory into the owner's shared memory, counted by the owner's
// mbarrier) carries a slab into that owner's inbox; the owner adds the slabs in rank order.
//
// The reference's engine calls cuBLAS for these products (emberserve/model/qwen2.py:57-58,
// 77-79); at these row counts the library reaches about half of the memory bandwidth.
//
// Every wait on an mbarrier is bounded: if it runs out, the block records a code in the status
// word shared by the tcgen05 kernels (codes 31..35 here: producer, MMA issuer, epilogue, drain,
// arrival of the partials), stops issuing work, lets what it has in flight land, frees its
// tensor memory and returns.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace ems {

constexpr int G6_BM = 128;   // output features per block (MMA M)
constexpr int G6_BK = 64;    // K per stage: one 128-byte swizzle span of bf16
constexpr int G6_THREADS = 128;
// Rows of the inbox: what the OTHER blocks of the cluster push for the rows this block owns,
// (ksplit - 1) * owned(ksplit) with owned = 128 / ksplit rounded up to 4; the maximum over
// ksplit = 2..8 is 120 (at 6 and 7).
constexpr int G6_INBOX_ROWS = 120;
template <int NT> constexpr int g6_stages() { return NT <= 32 ? 10 : (NT <= 64 ? 8 : 5); }
template <int NT> constexpr int g6_smem_bytes() {
    return g6_stages<NT>() * (G6_BM * G6_BK * 2 + NT * G6_BK * 2) + G6_INBOX_ROWS * NT * 4 +
           (2 * g6_stages<NT>() + 2) * 8 + 16 + 1024;
}

struct Gemm6Params {
    bf16* y;             // [m_tok, n_out]
    const bf16* bias;    // [n_out] or null
    int* status;
    int m_tok, n_out, k_tiles, ksplit;
    int cols;            // m_tok rounded up to 4: the token columns that are pushed and summed
    int tiled;           // the weight map is that of the tiled copy (see tc_weight_map)
};

// NT: token columns of the MMA (32, 64 or 128); the activation tile of a stage has NT rows, of
// which the first m_tok exist (TMA fills the rest with zeros).
template <int NT>
__global__ void __launch_bounds__(G6_THREADS)
gemm_midm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         const Gemm6Params p) {
    constexpr int STAGES = g6_stages<NT>();
    constexpr uint32_t A_BYTES = G6_BM * G6_BK * 2;   // 16 KB of weights
    constexpr uint32_t B_BYTES = NT * G6_BK * 2;      // 4..16 KB of activations
    constexpr uint32_t INBOX_BYTES = G6_INBOX_ROWS * NT * 4;
    constexpr int LD = 16;  // accumulator columns per tensor-memory load
    // instruction descriptor: D float32, A and B bfloat16, both K-major, N = NT, M = 128
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) |
                               ((uint32_t)(G6_BM >> 4) << 24);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // carve: [A stages][B stages][inbox][barriers][tmem pointer]; the base is rounded up to 1024 bytes
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_s = base, b_s = base + STAGES * A_BYTES;
    float* inbox = reinterpret_cast<float*>(base_ptr + STAGES * (A_BYTES + B_BYTES));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + STAGES * (A_BYTES + B_BYTES) + INBOX_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, done_bar = empty0 + 8 * STAGES;
    const uint32_t inbox_bar = done_bar + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, ks = blockIdx.y;
    const int per = (p.k_tiles + p.ksplit - 1) / p.ksplit;
    const int kt_begin = ks * per, kt_end = min(p.k_tiles, kt_begin + per);
    const int nk = max(0, kt_end - kt_begin);
    // split K: rank `me` of the cluster owns output rows [me * owned, +owned) of the tile
    const bool split = p.ksplit > 1;
    const int me = split ? (int)cluster_rank() : 0;
    const int owned = (((G6_BM + p.ksplit - 1) / p.ksplit) + 3) & ~3;
    const int my_rows = max(0, min(owned, G6_BM - me * owned));
    const int cols = p.cols;

    auto load_w = [&](uint32_t dst, int kt, uint32_t bar) {  // the weight tile of K tile `kt` into a stage
        if (p.tiled) tma_load_2d(dst, &map_w, 0, (tile * p.k_tiles + kt) * G6_BM, bar);
        else tma_load_2d(dst, &map_w, kt * G6_BK, tile * G6_BM, bar);
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(done_bar, 1);
        mbar_init(inbox_bar, 1);
        // what the other blocks of the cluster will send here: a slab of owned x cols floats each
        if (split) mbar_expect_tx(inbox_bar, (uint32_t)((p.ksplit - 1) * owned * cols * 4));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the weights do not depend on the kernel before this one: the first ring of weight tiles
        // is requested at once; the activations follow after the dependency wait
        const int pre = min(nk, STAGES);
        for (int it = 0; it < pre; ++it) {
            mbar_expect_tx(full0 + 8 * it, A_BYTES + B_BYTES);
            load_w(a_s + it * A_BYTES, kt_begin + it, full0 + 8 * it);
        }
    }
    if (warp == 1) {  // tensor memory for the accumulator: NT columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)NT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // no block pushes into a peer before that peer's inbox barrier exists (the only cluster
    // barrier of the kernel; it is passed while the blocks still wait for the kernel before)
    if (split) cluster_sync_all();
    const uint32_t tmem_d = *tmem_slot;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (the first ring of weight tiles is on its way already) ----------
        const int pre = min(nk, STAGES);
        grid_dependency_wait();
        for (int it = 0; it < pre; ++it)
            tma_load_2d(b_s + it * B_BYTES, &map_x, (kt_begin + it) * G6_BK, 0, full0 + 8 * it);
        int armed = pre;
        for (int it = pre; it < nk && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, 31);
            if (!ok) break;
            mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
            const int k0 = (kt_begin + it) * G6_BK;
            load_w(a_s + s * A_BYTES, kt_begin + it, full0 + 8 * s);
            tma_load_2d(b_s + s * B_BYTES, &map_x, k0, 0, full0 + 8 * s);
            armed = it + 1;
        }
        if (!ok) {  // let the copies that were issued land before the block leaves
            for (int it = max(0, armed - STAGES); it < armed; ++it)
                mbar_wait(full0 + 8 * (it % STAGES), (uint32_t)(it / STAGES) & 1u, p.status, 34);
        }
    } else if (warp == 1) {
        // ---- MMA issue: the warp runs the loop, one elected lane issues ---------------------
        const bool issuer = elect_one();
        for (int it = 0; it < nk && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph, p.status, 32));
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = smem_desc_sw128(a_s + s * A_BYTES), db = smem_desc_sw128(b_s + s * B_BYTES);
            if (issuer) {
#pragma unroll
                for (int k = 0; k < G6_BK / 16; ++k)  // 16 K per MMA = 32 bytes = 2 descriptor units
                    tc_mma_bf16(tmem_d, da + 2 * k, db + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
                tc_commit(empty0 + 8 * s);  // arrives once these MMAs have read the stage
            }
            __syncwarp();
        }
        if (issuer) tc_commit(done_bar);    // arrives once every MMA issued above has completed
    }
    __syncwarp();

    // ---- epilogue: all four warps, 32 accumulator lanes (= output features) each -------
    grid_dependency_wait();  // (the producer has passed it already; this orders the stores below)
    allow_dependent_launch();
    bool done = true;
    if (lane == 0) done = mbar_wait(done_bar, 0, p.status, 33);
    done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
    tc_fence_after();
    const int row_local = warp * 32 + lane;
    const int row = tile * G6_BM + row_local;  // output feature of this thread
    const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
    const bool have = done && nk > 0;
    if (!split) {
        const float bias = (row < p.n_out && p.bias) ? __bfloat162float(p.bias[row]) : 0.f;
        if (have) {
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += LD) {
                if (c0 >= p.m_tok) break;
                float v[LD];
                tc_ld16(taddr + c0, v);
                if (row < p.n_out) {
#pragma unroll
                    for (int i = 0; i < LD; ++i)
                        if (c0 + i < p.m_tok) p.y[(size_t)(c0 + i) * p.n_out + row] = __float2bfloat16_rn(v[i] + bias);
                }
            }
        }
    } else {
        // The partials of the tile are laid out in this block's ring memory (no copy and no MMA
        // touches it any more) as one slab per owner, [owner][cols / 4][owned row][4 tokens]; then
        // ONE bulk copy per owner carries a slab into that owner's inbox (slot of this block among
        // the other senders) and completes its bytes on the owner's mbarrier.  The slab of the rows
        // this block owns stays where it is.  A block whose waits ran out must not write the ring
        // (copies may still land): it sends nothing, the owners' waits run out in turn and the
        // status word says so.
        const int dst_rank = row_local / owned;
        const int rl_mine = row_local % owned;
        const int slab_floats = owned * cols;
        float* stage = reinterpret_cast<float*>(base_ptr);
        if (done) {
            float* mine = stage + (size_t)dst_rank * slab_floats + rl_mine * 4;
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 32) {
                if (c0 >= cols) break;
                float v[32];
                if (have) tc_ld32(taddr + c0, v);
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    if (c0 + i >= cols) break;
                    const bool z = !have;  // a block without K sends zeros
                    *reinterpret_cast<float4*>(mine + (size_t)(c0 + i) * owned) =
                        make_float4(z ? 0.f : v[i], z ? 0.f : v[i + 1], z ? 0.f : v[i + 2], z ? 0.f : v[i + 3]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the bulk copies read what was stored
        }
        __syncthreads();
        if (done && (int)threadIdx.x < p.ksplit && (int)threadIdx.x != me) {
            const int r = threadIdx.x;
            const int sender_slot = me < r ? me : me - 1;
            bulk_push(smem_u32(inbox) + (uint32_t)(sender_slot * slab_floats) * 4u,
                      smem_u32(stage) + (uint32_t)(r * slab_floats) * 4u, (uint32_t)slab_floats * 4u, inbox_bar,
                      (uint32_t)r);
        }
        bool arrived = true;
        if (lane == 0) arrived = mbar_wait(inbox_bar, 0, p.status, 35);
        arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
        if (arrived) mbar_try_wait(inbox_bar, 0);  // (every thread observes the completed phase itself)
        // every copy INTO this block has landed; the others may leave once they know
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        arrived = arrived && done;
        // one item = four tokens of one owned row: 16 bytes per sender, side by side for the lanes
        const float* own_slab = stage + (size_t)me * slab_floats;
        for (int idx = threadIdx.x; idx < (cols >> 2) * my_rows && arrived; idx += G6_THREADS) {
            const int c4 = idx / my_rows, rl = idx % my_rows;
            const int orow = tile * G6_BM + me * owned + rl;
            if (orow >= p.n_out) continue;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int r = 0; r < p.ksplit; ++r) {  // in rank order: the same sum for every batch
                const float* src = (r == me ? own_slab : inbox + (size_t)((r < me ? r : r - 1) * slab_floats)) +
                                   (size_t)(c4 * owned + rl) * 4;
                const float4 v = *reinterpret_cast<const float4*>(src);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            const float bias = p.bias ? __bfloat162float(p.bias[orow]) : 0.f;
            const int n = c4 * 4;
            bf16* dst = p.y + (size_t)n * p.n_out + orow;
            if (n < p.m_tok) dst[0] = __float2bfloat16_rn(acc.x + bias);
            if (n + 1 < p.m_tok) dst[(size_t)p.n_out] = __float2bfloat16_rn(acc.y + bias);
            if (n + 2 < p.m_tok) dst[(size_t)2 * p.n_out] = __float2bfloat16_rn(acc.z + bias);
            if (n + 3 < p.m_tok) dst[(size_t)3 * p.n_out] = __float2bfloat16_rn(acc.w + bias);
        }
        // no block leaves (and gives up the shared memory its copies read) before every block of the
        // cluster has received what was sent to it
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)NT) : "memory");
    }
}

template <int NT>
static int launch_gemm6(const CUtensorMap& mw, const CUtensorMap& mx, const Gemm6Params& p, int tiles,
                        cudaStream_t stream) {
    auto kernel = gemm_midm_tcgen05_kernel<NT>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g6_smem_bytes<NT>()) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    cfg.gridDim = dim3(tiles, p.ksplit);
    cfg.blockDim = dim3(G6_THREADS);
    cfg.dynamicSmemBytes = g6_smem_bytes<NT>();
    cfg.stream = stream;
    int nattr = 0;
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see grid_dependency_wait
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
    if (p.ksplit > 1) {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = 1;
        attr[nattr].val.clusterDim.y = p.ksplit;
        attr[nattr].val.clusterDim.z = 1;
        ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    if (cudaLaunchKernelEx(&cfg, kernel, mw, mx, p) != cudaSuccess) {
        cudaGetLastError();
        return EMS_ERR_LAUNCH;
    }
    return launch_status();
}

}  // namespace ems

using namespace ems;

template <int NT>
static int max_clusters6(int ksplit) {
    auto kernel = gemm_midm_tcgen05_kernel<NT>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g6_smem_bytes<NT>()) != cudaSuccess)
        return -1;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    cfg.gridDim = dim3(1, ksplit);
    cfg.blockDim = dim3(G6_THREADS);
    cfg.dynamicSmemBytes = g6_smem_bytes<NT>();
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ksplit;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return n;
}

// How many clusters of `ksplit` blocks of the kernel for `m_tok` rows the device holds at once
// (a cluster lives inside one of the GPU's processing clusters, so this is less than SMs / ksplit).
EMS_EXPORT int ems_gemm_midm_max_clusters(int m_tok, int ksplit) {
    if (ksplit < 1 || ksplit > 8) return -1;
    if (m_tok <= 32) return max_clusters6<32>(ksplit);
    if (m_tok <= 64) return max_clusters6<64>(ksplit);
    return max_clusters6<128>(ksplit);
}

// y[m_tok, n_out] (bf16) = x[m_tok, k] (bf16, row-major) . w[n_out, k]^T (+ bias), m_tok <= 128;
// k a multiple of 8; 16-byte aligned x and w.  ksplit in 1..8 blocks share K as one thread-block
// cluster.  `tiled`: w is the tiled copy of the weight (tc_weight_map).  One block per SM: the caller chooses ksplit so that n_out / 128 * ksplit blocks start
// in one wave.
EMS_EXPORT int ems_gemm_midm(const void* x, const void* w, const void* bias, void* y, int m_tok, int n_out, int k,
                             int ksplit, int tiled, cudaStream_t stream) {
    if (m_tok <= 0 || n_out <= 0) return EMS_OK;
    if (m_tok > 128 || k <= 0 || k % 8 || ksplit < 1 || ksplit > 8) return EMS_ERR_SHAPE;  // 8: the portable cluster size
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)y % 2) || y == nullptr) return EMS_ERR_ALIGN;
    int* status_dev = tc_status_device_ptr();
    if (!status_dev) return EMS_ERR_LAUNCH;
    int* dev_ptr = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&dev_ptr), status_dev, 0) != cudaSuccess) return EMS_ERR_LAUNCH;
    const int nt = m_tok <= 32 ? 32 : (m_tok <= 64 ? 64 : 128);
    CUtensorMap mw, mx;
    if (!tc_weight_map(w, n_out, k, tiled != 0, &mw) || !tc_tensor_map_2d(x, m_tok, k, nt, &mx)) return EMS_ERR_LAUNCH;
    Gemm6Params p;
    p.y = reinterpret_cast<bf16*>(y); p.bias = reinterpret_cast<const bf16*>(bias); p.status = dev_ptr;
    p.m_tok = m_tok; p.n_out = n_out; p.k_tiles = (k + G6_BK - 1) / G6_BK; p.ksplit = ksplit;
    p.cols = (m_tok + 3) & ~3;
    p.tiled = tiled ? 1 : 0;
    const int tiles = (n_out + G6_BM - 1) / G6_BM;
    if (nt == 32) return launch_gemm6<32>(mw, mx, p, tiles, stream);
    if (nt == 64) return launch_gemm6<64>(mw, mx, p, tiles, stream);
    return launch_gemm6<128>(mw, mx, p, tiles, stream);
}
