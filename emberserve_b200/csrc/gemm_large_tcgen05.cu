// y = x W^T for many rows of x (prompt portions): a compute-bound GEMM on the fifth-generation
// tensor cores, two SMs to a tile, with the gated feed-forward's activation in its epilogue.
//
// Two blocks on neighbouring SMs form a cluster and share one 256 x 256 output tile
// (tcgen05.mma.cta_group::2): each block stages its own 128 token rows of x and HALF of the
// 256 weight rows of a K step (TMA, 128-byte swizzle, no multicast), so a K step of 64 costs
// each SM 32 KB of shared-memory fill for 128 x 256 x 64 multiply-adds, and the ring is six
// stages deep.  One warp of the leading block issues the MMAs for both (the whole warp runs
// the loop and an elected lane issues: with a lone diverged lane every tcgen05.commit cost
// the tensor pipe about 130 idle cycles, 583 k cycles a call against 500 k); the accumulator
// (128 lanes x 256 float32 columns per block) lives in tensor memory twice, so that the
// eight epilogue warps of each block drain tile t while the MMAs of tile t+1 run.  The grid
// is persistent: one cluster per SM pair walks the tiles in an order that keeps the tiles
// in flight on few weight rows (they are read from memory once and from L2 after that).
//
// GATED: the leading block stages 128 rows of the gate projection and its peer the same
// rows of the up projection, so the accumulator holds gate in columns 0..127 and up in
// 128..255 of the same token lane, and the epilogue stores silu(gate) * up: the [tokens, 2 I]
// intermediate never goes to memory.  The reference's engine calls cuBLAS and then a Triton
// kernel here (emberserve/model/qwen2.py:57-61, emberserve/model/ops_triton.py:62-91).
//
// Every wait on an mbarrier is bounded: if one runs out, the block records a code in the
// status word that the host reads, every role leaves its loop, the producers give their
// copies in flight time to land, both blocks meet at the cluster barrier and free their
// tensor memory.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace ems {

constexpr int GL_BM = 128;        // token rows per block (256 per pair)
constexpr int GL_BN = 128;        // weight rows staged per block and K step (256 per pair)
constexpr int GL_BK = 64;         // K per stage: one 128-byte swizzle span of bf16
constexpr int GL_STAGES = 6;
constexpr int GL_THREADS = 320;   // warp 0 TMA, warp 1 MMA and tensor memory, warps 2..9 epilogue
constexpr uint32_t GL_TILE_BYTES = GL_BM * GL_BK * 2;       // 16 KB (x tile and weight tile alike)
constexpr uint32_t GL_STAGE_BYTES = 2 * GL_TILE_BYTES;      // 32 KB per block
constexpr uint32_t GL_ACC_COLS = 256;
constexpr uint32_t GL_TMEM_COLS = 512;                      // two accumulators
constexpr int GL_SMEM = GL_STAGES * GL_STAGE_BYTES + (2 * GL_STAGES + 4) * 8 + 32 + 1024;

struct GemmLargeParams {
    bf16* y;            // GATED: [m_tok, n_out]; else [m_tok, n_out]
    const bf16* bias;   // plain only, or null
    int* status;
    int m_tok;
    int n_out;          // GATED: I (width of y; the weight has 2 I rows); else rows of the weight
    int k_tiles;
    int m_tiles;        // of 256 token rows
    int n_tiles;        // GATED: of 128 outputs; else of 256
    int tiled;          // the weight map is that of the tiled copy (tc_weight_map)
};

__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    return remote;
}
// TMA tile load whose completion is counted on a barrier that may belong to the peer block
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {  // `bar`: a shared::cluster address
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {  // `bar`: a shared::cluster address
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive float32 columns of this thread's accumulator lane; the caller waits
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float silu_times(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// One chunk of 32 accumulator columns of a token row to memory.  GATED: `a` = gate columns
// [c0, c0+32), `b` = the up columns of the same outputs; else `a` = columns [c0, c0+32) of y.
template <bool GATED>
__device__ __forceinline__ void gl_store_chunk(const GemmLargeParams& p, int token, int n_tile, int c0,
                                               const float (&a)[32], const float (&b)[32]) {
    if (token >= p.m_tok) return;
    if (GATED) {
        bf16* dst = p.y + (size_t)token * p.n_out + (size_t)n_tile * GL_BN + c0;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf16x2(silu_times(a[i], b[i]), silu_times(a[i + 1], b[i + 1]));
            o.y = pack_bf16x2(silu_times(a[i + 2], b[i + 2]), silu_times(a[i + 3], b[i + 3]));
            o.z = pack_bf16x2(silu_times(a[i + 4], b[i + 4]), silu_times(a[i + 5], b[i + 5]));
            o.w = pack_bf16x2(silu_times(a[i + 6], b[i + 6]), silu_times(a[i + 7], b[i + 7]));
            *reinterpret_cast<uint4*>(dst + i) = o;
        }
    } else {
        const int n0 = n_tile * 2 * GL_BN + c0;
        bf16* dst = p.y + (size_t)token * p.n_out + n0;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            if (n0 + i >= p.n_out) break;  // n_out is a multiple of 8
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = a[i + j] + (p.bias ? __bfloat162float(p.bias[n0 + i + j]) : 0.f);
            uint4 o;
            o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
            o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(dst + i) = o;
        }
    }
}

template <bool GATED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GL_THREADS)
gemm_large_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                          const GemmLargeParams p) {
    // instruction descriptor: D float32, A and B bfloat16, both K-major, N = 256, M = 256 over the pair
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) |
                               ((uint32_t)(256 >> 4) << 24);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // carve: [stages: x tile, weight tile][full, empty][tfull x2, tempty x2][tmem pointer][wait flags]
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + GL_STAGES * GL_STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * GL_STAGES;
    const uint32_t tfull0 = empty0 + 8 * GL_STAGES, tempty0 = tfull0 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * GL_STAGES + 4);
    volatile int* wait_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);  // two, used in turn

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();          // 0 leads: it issues the MMAs and owns full / tempty
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int total = p.m_tiles * p.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < GL_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 16); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both blocks: 512 columns in each block's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(GL_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers and tensor memory exist from here on
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (each block loads its own halves; completion counts on the leader) ----
        const uint32_t lead_full0 = map_to_rank(full0, 0);
        // this block's 128 weight rows of K step `kb` (row-major matrix, or its tiled copy)
        auto load_w = [&](uint32_t dst, int kb, int w_row, uint32_t bar) {
            if (p.tiled) tma_load_2d_pair(dst, &map_w, 0, ((w_row / GL_BN) * p.k_tiles + kb) * GL_BN, bar);
            else tma_load_2d_pair(dst, &map_w, kb * GL_BK, w_row, bar);
        };
        bool ok = true;
        int it = 0;
        // The weights do not depend on the kernel before this one (the launch is a programmatic
        // dependent): the weight halves of the first stages are requested at once, the token rows
        // after the dependency wait.
        const int pre = pair < total ? min(p.k_tiles, GL_STAGES) : 0;
        {
            const int n_tile = pair / p.m_tiles;
            const int w_row = GATED ? (int)rank * p.n_out + n_tile * GL_BN : n_tile * 2 * GL_BN + (int)rank * GL_BN;
            for (int kb = 0; kb < pre; ++kb) {
                if (rank == 0) mbar_expect_tx(full0 + 8 * kb, 2 * GL_STAGE_BYTES);
                load_w(base + kb * GL_STAGE_BYTES + GL_TILE_BYTES, kb, w_row, lead_full0 + 8 * kb);
            }
        }
        grid_dependency_wait();
        for (int tile = pair; tile < total && ok; tile += pairs) {
            const int n_tile = tile / p.m_tiles, m_tile = tile % p.m_tiles;
            const int x_row = m_tile * 2 * GL_BM + (int)rank * GL_BM;
            const int w_row = GATED ? (int)rank * p.n_out + n_tile * GL_BN : n_tile * 2 * GL_BN + (int)rank * GL_BN;
            for (int kb = 0; kb < p.k_tiles; ++kb, ++it) {
                const int s = it % GL_STAGES;
                const uint32_t dst = base + s * GL_STAGE_BYTES;
                if (it < pre) {  // armed above, the weight half is on its way
                    tma_load_2d_pair(dst, &map_x, kb * GL_BK, x_row, lead_full0 + 8 * s);
                    continue;
                }
                const uint32_t ph = (uint32_t)(it / GL_STAGES) & 1u;
                ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, 11);
                if (!ok) break;
                if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * GL_STAGE_BYTES);
                tma_load_2d_pair(dst, &map_x, kb * GL_BK, x_row, lead_full0 + 8 * s);
                load_w(dst + GL_TILE_BYTES, kb, w_row, lead_full0 + 8 * s);
            }
        }
        if (!ok)  // copies in flight may still land in this block's shared memory: give them time
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
    } else if (warp == 1 && rank == 0) {
        // ---- MMA issue (leading block only): the warp runs the loop, one elected lane issues ---
        const bool issuer = elect_one();
        const uint32_t peer_empty0 = map_to_rank(empty0, 1), peer_tfull0 = map_to_rank(tfull0, 1);
        bool ok = true;
        int it = 0, si = 0;
        for (int tile = pair; tile < total && ok; tile += pairs, ++si) {
            const int b = si & 1;
            const uint32_t tph = (uint32_t)(si >> 1) & 1u;
            // both blocks have drained this accumulator
            ok = __all_sync(0xffffffffu, mbar_wait(tempty0 + 8 * b, tph ^ 1u, p.status, 12));
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc_addr = tmem_d + (uint32_t)b * GL_ACC_COLS;
            for (int kb = 0; kb < p.k_tiles; ++kb, ++it) {
                const int s = it % GL_STAGES;
                const uint32_t ph = (uint32_t)(it / GL_STAGES) & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph, p.status, 13));
                if (!ok) break;
                tc_fence_after();
                const uint64_t da = smem_desc_sw128(base + s * GL_STAGE_BYTES);
                const uint64_t db = smem_desc_sw128(base + s * GL_STAGE_BYTES + GL_TILE_BYTES);
                if (issuer) {
#pragma unroll
                    for (int k = 0; k < GL_BK / 16; ++k)
                        tc_mma_bf16_pair(acc_addr, da + 2 * k, db + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty0 + 8 * s);   // the stage is free in both blocks once these MMAs have read it
                    tc_commit_pair(peer_empty0 + 8 * s);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (issuer) {
                tc_commit_pair(tfull0 + 8 * b);       // the accumulator is complete in both blocks
                tc_commit_pair(peer_tfull0 + 8 * b);
            }
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ---- epilogue: eight warps; a warp reads the 32 token lanes of its quarter of tensor memory
        // and one half of the accumulator's columns --------------------------------------------------
        const uint32_t lead_tempty0 = map_to_rank(tempty0, 0);
        const int quad = warp & 3;          // the lanes of tensor memory this warp may read
        const int half = (warp - 2) >> 2;   // which half of the columns
        const int row_local = quad * 32 + lane;
        // GATED: outputs [c_begin, c_end) of the tile's 128 (gate column c, up column 128 + c);
        // else accumulator columns [c_begin, c_end) of 256
        constexpr int SPAN = GATED ? GL_BN / 2 : GL_BN;
        const int c_begin = half * SPAN, c_end = c_begin + SPAN;
        bool ok = true;
        int si = 0;
        for (int tile = pair; tile < total && ok; tile += pairs, ++si) {
            const int n_tile = tile / p.m_tiles, m_tile = tile % p.m_tiles;
            const int b = si & 1;
            const uint32_t tph = (uint32_t)(si >> 1) & 1u;
            // one lane waits for the accumulator and tells the eight warps
            if (warp == 2 && lane == 0) wait_flag[si & 1] = mbar_wait(tfull0 + 8 * b, tph, p.status, 14) ? 1 : 0;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            ok = wait_flag[si & 1] != 0;
            if (!ok) break;
            tc_fence_after();
            const int token = m_tile * 2 * GL_BM + (int)rank * GL_BM + row_local;
            const uint32_t taddr = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)b * GL_ACC_COLS;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                uint32_t ra[32], rb[32];
                tc_ld32_nowait(taddr + c0, ra);
                if (GATED) tc_ld32_nowait(taddr + GL_BN + c0, rb);
                tc_ld_wait();
                float fa[32], fb[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) { fa[i] = __uint_as_float(ra[i]); fb[i] = GATED ? __uint_as_float(rb[i]) : 0.f; }
                gl_store_chunk<GATED>(p, token, n_tile, c0, fa, fb);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8 * b);
        }
    }
    __syncwarp();  // the lanes that had no role wait here for the one that had
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // nobody frees tensor memory or leaves while the pair still works
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(GL_TMEM_COLS) : "memory");
    }
}

template <bool GATED>
static int launch_gemm_large(const CUtensorMap& mx, const CUtensorMap& mw, const GemmLargeParams& p,
                             cudaStream_t stream) {
    auto kernel = gemm_large_tcgen05_kernel<GATED>;
    static int pairs_cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return EMS_ERR_LAUNCH;
    if (pairs_cached[dev] == 0) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GL_SMEM) != cudaSuccess)
            return EMS_ERR_LAUNCH;
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2)
            return EMS_ERR_LAUNCH;
        // how many pairs the device runs at once: not every SM need have a partner for a cluster of two
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sms); cfg.blockDim = dim3(GL_THREADS); cfg.dynamicSmemBytes = GL_SMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) {
            cudaGetLastError();
            clusters = sms / 2;
        }
        pairs_cached[dev] = clusters;
    }
    const int total = p.m_tiles * p.n_tiles;
    const int pairs = total < pairs_cached[dev] ? total : pairs_cached[dev];
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GL_THREADS);
    cfg.dynamicSmemBytes = GL_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    // may start while the kernel before it still runs: set-up and the first weight tiles overlap it
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, mx, mw, p) != cudaSuccess) {
        cudaGetLastError();
        return EMS_ERR_LAUNCH;
    }
    return launch_status();
}

}  // namespace ems

using namespace ems;

// 1 if ems_gemm_large_gated takes these sizes (bfloat16 only).
EMS_EXPORT int ems_gemm_large_gated_supported(int m_tok, int inter, int k) {
    return m_tok > 0 && inter > 0 && inter % GL_BN == 0 && k > 0 && k % 8 == 0;
}

// act[m_tok, inter] (bf16) = silu(x . w[0:inter]^T) * (x . w[inter:2*inter]^T), w: [2*inter, k],
// for any number of rows; inter a multiple of 128, k a multiple of 8, 16-byte aligned pointers.
EMS_EXPORT int ems_gemm_large_gated(const void* x, const void* w, void* act, int m_tok, int inter, int k, int tiled,
                                    cudaStream_t stream) {
    if (m_tok <= 0 || inter <= 0) return EMS_OK;
    if (!ems_gemm_large_gated_supported(m_tok, inter, k)) return EMS_ERR_SHAPE;
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)act % 16)) return EMS_ERR_ALIGN;
    int* status = tc_status_device_ptr();
    if (!status) return EMS_ERR_LAUNCH;
    int* status_dev = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev), status, 0) != cudaSuccess) return EMS_ERR_LAUNCH;
    CUtensorMap mx, mw;
    if (!tc_tensor_map_2d(x, m_tok, k, GL_BM, &mx) || !tc_weight_map(w, 2LL * inter, k, tiled != 0, &mw))
        return EMS_ERR_LAUNCH;
    GemmLargeParams p;
    p.y = reinterpret_cast<bf16*>(act); p.bias = nullptr; p.status = status_dev; p.m_tok = m_tok; p.n_out = inter;
    p.k_tiles = (k + GL_BK - 1) / GL_BK; p.m_tiles = (m_tok + 2 * GL_BM - 1) / (2 * GL_BM); p.n_tiles = inter / GL_BN;
    p.tiled = tiled ? 1 : 0;
    return launch_gemm_large<true>(mx, mw, p, stream);
}
