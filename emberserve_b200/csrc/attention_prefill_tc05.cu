// Paged causal grouped-query attention for prompt portions in bfloat16 on the
// fifth-generation tensor cores: both products of the flash-attention scheme are
// tcgen05.mma instructions whose accumulators, and the probabilities between them, stay in
// tensor memory.
//
// A block owns 256 "rows" of one request and one KV head, as two tiles A and B of 128 (a row
// is a (query token, query head of the group) pair, so the heads that share a KV head share
// every K/V tile), and walks the keys in tiles of 128 aligned to absolute positions.  Its warps
// have fixed roles that meet only through mbarriers:
//   loader (1 warp)     K and V tiles by TMA: pages are multiples of 16 keys, so 16 keys of one KV
//                       head are one box of a tensor map over the cache seen as a matrix
//                       [pages * kv heads * page size, D], found through the block table; eight
//                       boxes (per 64-column span) make a tile in the 128-byte-swizzled layout of
//                       the tensor cores; K and V have rings of two stages each, freed
//                       separately (K as soon as both S products have read it).  Rows of V that hold no key
//                       of this block (the end of the last tile, the start of a window) are
//                       zeroed after they land, since a zero probability times a stale
//                       non-number would still poison the row;
//   MMA (1 warp)        S_X = Q_X K^T (128 x 128 x D, K-major operands from shared memory, S in
//                       tensor memory), and O_X += P_X V (128 x D x 128) with P read from tensor
//                       memory and V consumed as it lies in the cache, keys by rows (an MN-major
//                       operand); X alternates between A and B, so the tensor pipe works on one
//                       tile while the other tile's softmax runs.  The warp runs its loop as a
//                       whole (addresses and descriptors are the same in every lane) and one
//                       elected lane issues the instructions;
//   softmax (2 x 4 warps) thread r of a group owns row r: it reads its lane of S (tcgen05.ld),
//                       masks, keeps the running maximum and sum in float32 (base-2
//                       exponentials), and writes P = 2^(s - m) as bfloat16 over S
//                       (tcgen05.st).  O is rescaled in tensor memory only when a row's maximum
//                       has grown by more than 2^8 since the reference point of its
//                       exponentials (that point, not the true maximum, is `m`; the quotient
//                       O / l does not depend on it).  At the end it divides O by l and stores.
//
// Formulas: emberserve/attn/base.py:105-128.  The reference has no kernel of this kind (it
// calls flash-attn, attn/paged_flash.py:232-279).  Every wait on an mbarrier is bounded; a
// wait that runs out writes a code to the status word of the tcgen05 kernels, the roles skip
// the rest of their work, and the block still frees its tensor memory.
#include <cuda.h>

#include "attention_decode_mma.cuh"

namespace ems {

// gemm_tcgen05.cu: the status word of the tcgen05 kernels, and cached tensor maps of row-major
// bfloat16 matrices with boxes of [box_rows, 64 columns] in the 128-byte swizzle
int* tc_status_device_ptr();
bool tc_tensor_map_2d(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out);

constexpr int T5_BQ = 128;       // rows per tile = MMA M
constexpr int T5_BK = 128;       // keys per tile
constexpr int T5_STAGES = 2;     // stages of the K ring and of the V ring
constexpr int T5_THREADS = 320;  // warps 0-3: softmax A, 4-7: softmax B, 8: MMA + tensor memory, 9: loader
constexpr uint32_t T5_SPIN_LIMIT = 1u << 18;
constexpr float T5_RESCALE_LOG2 = 8.0f;
// Room to align the tiles to 1024 bytes behind whatever the dynamic shared memory starts at.
constexpr int T5_ALIGN_SLACK = 1024;
constexpr long long T5_MAX_ROWS = 2147483647LL;  // rows of the cache matrix a 32-bit row index reaches

__device__ __forceinline__ uint32_t t5_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void t5_cp16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void t5_commit_group() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void t5_wait_group() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void t5_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void t5_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void t5_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void t5_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void t5_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void t5_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void t5_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ bool t5_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool t5_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    for (uint32_t i = 0; i < T5_SPIN_LIMIT; ++i)
        if (t5_try_wait(bar, parity)) return true;
    volatile int* word = status;
    if (*word == 0) *word = code;
    return false;
}
__device__ __forceinline__ void t5_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] B[smem]
__device__ __forceinline__ void t5_mma_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] B[smem]
__device__ __forceinline__ void t5_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
#define T5_R32(r) \
    "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), \
    "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), \
    "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), \
    "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
#define T5_IN32(r) \
    "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), \
    "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), \
    "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), \
    "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
// 32 consecutive columns of this thread's lane (no wait: follow with t5_ld_wait)
__device__ __forceinline__ void t5_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : T5_R32(r) : "r"(taddr));
}
__device__ __forceinline__ void t5_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void t5_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
        ::T5_IN32(r), "r"(taddr) : "memory");
}
__device__ __forceinline__ void t5_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr) : "memory");
}
__device__ __forceinline__ bool t5_elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void t5_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float t5_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t t5_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// 128-byte-swizzled tile descriptors (version 1, layout type 2).  K-major: rows of 128 bytes,
// 8-row groups `sbo` bytes apart.  MN-major: the same rows are K indices; 64-element groups of
// the MN dimension `lbo` bytes apart.
__device__ __forceinline__ uint64_t t5_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    const uint64_t lo = (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16);
    const uint64_t hi = (uint64_t)((sbo >> 4) & 0x3FFFu) | ((uint64_t)1 << 14) | ((uint64_t)2 << 29);
    return lo | (hi << 32);
}

template <int D> struct T5Layout {
    static constexpr int SPANS = D / 64;              // 128-byte spans per row of Q, K, V
    static constexpr int Q_SPAN = T5_BQ * 128;        // bytes of one span of a Q tile
    static constexpr int KV_SPAN = T5_BK * 128;       // bytes of one span of a K or V tile
    static constexpr int Q_BYTES = SPANS * Q_SPAN;    // one Q tile
    static constexpr int KV_BYTES = SPANS * KV_SPAN;  // one K or V tile
    static constexpr int NUM_BARS = 4 * T5_STAGES + 7;
    static constexpr int SMEM = 2 * Q_BYTES + 2 * T5_STAGES * KV_BYTES + NUM_BARS * 8 + 16 + T5_ALIGN_SLACK;
    // tensor memory columns: S_A, S_B (128 each; P overlays the first 64), O_A, O_B (D each)
    static constexpr uint32_t S_COL = 0, O_COL = 2 * T5_BK;
    static constexpr uint32_t TMEM_COLS = 512;
};

template <int D>
__global__ void __launch_bounds__(T5_THREADS, 1)
prefill_attention_tc05_kernel(const DecodeParams p, int* status, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, const int single) {
    using L = T5Layout<D>;
    // D float32, A and B bfloat16; S: both K-major, N = 128 keys; PV: B MN-major, N = D
    constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(T5_BK >> 3) << 17) | (8u << 24);
    constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | (8u << 24);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t base = (t5_smem(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - t5_smem(smem_raw));
    const uint32_t q_s = base, k_s = q_s + 2 * L::Q_BYTES, v_s = k_s + T5_STAGES * L::KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + 2 * L::Q_BYTES + 2 * T5_STAGES * L::KV_BYTES);
    const uint32_t bar0 = t5_smem(bars);
    // barriers: kfull, vfull, kempty, vempty (per stage), then sfull[X], pfull[X], ofull[X], vland
    auto kfull = [&](int st) { return bar0 + 8u * st; };
    auto vfull = [&](int st) { return bar0 + 8u * (T5_STAGES + st); };
    auto kempty = [&](int st) { return bar0 + 8u * (2 * T5_STAGES + st); };
    auto vempty = [&](int st) { return bar0 + 8u * (3 * T5_STAGES + st); };
    auto sfull = [&](int x) { return bar0 + 8u * (4 * T5_STAGES + x); };
    auto pfull = [&](int x) { return bar0 + 8u * (4 * T5_STAGES + 2 + x); };
    auto ofull = [&](int x) { return bar0 + 8u * (4 * T5_STAGES + 4 + x); };
    const uint32_t vland = bar0 + 8u * (4 * T5_STAGES + 6);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);

    // grid: x = (request, KV head), y = row tile.  Blocks are handed out x first, so the heavy row
    // tiles (late rows, many keys) of ALL heads and requests start before any light one: with the
    // tiles of one head after the other a second wave would begin with another head's heaviest.
    const int b = blockIdx.x / p.nkv, hk = blockIdx.x % p.nkv;
    const int G = p.G;
    const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0, start = p.starts[b];
    const int nrows = qlen * G;
    // `single`: the block owns one row tile (A) instead of two: twice the blocks, for portions whose
    // pairs of tiles would leave SMs idle; tile B's roles then have nothing to do
    const int r0 = (int)(gridDim.y - 1 - blockIdx.y) * (single ? 1 : 2) * T5_BQ;  // heavy row tiles first
    if (r0 >= nrows) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // key ranges: tile X sees keys below kend[X]; both walk the same key tiles from kt0
    const int last_a = min(nrows - 1, r0 + T5_BQ - 1), last_b = single ? last_a : min(nrows - 1, r0 + 2 * T5_BQ - 1);
    const bool have_b = !single && r0 + T5_BQ < nrows;
    const int kend_a = start + last_a / G + 1, kend_b = start + last_b / G + 1;
    const int k_begin = p.window > 0 ? max(0, start + r0 / G - p.window + 1) : 0;
    const int kt0 = (k_begin / T5_BK) * T5_BK;
    const int n_a = (kend_a - kt0 + T5_BK - 1) / T5_BK;
    const int n_b = have_b ? (kend_b - kt0 + T5_BK - 1) / T5_BK : 0;
    const int n_all = max(n_a, n_b), k_end = max(kend_a, kend_b);
    const int* table = p.bt + (size_t)b * p.bt_stride;

    if (tid == 0) {
        for (int i = 0; i < 4 * T5_STAGES; ++i) t5_mbar_init(bar0 + 8u * i, 1);
        t5_mbar_init(vland, 1);
        for (int x = 0; x < 2; ++x) {
            t5_mbar_init(sfull(x), 1);
            t5_mbar_init(pfull(x), T5_BQ);
            t5_mbar_init(ofull(x), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(t5_smem(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {   // both Q tiles, by everybody: [tile][span][row][128 bytes, 16-byte chunks swizzled by row]
        constexpr int CH = D / 8;
        for (int idx = tid; idx < (single ? 1 : 2) * T5_BQ * CH; idx += T5_THREADS) {
            const int row = idx / CH, c = idx % CH;
            const int gr = r0 + row;
            const bool valid = gr < nrows;
            const bf16* src = p.q;
            if (valid) src = p.q + (size_t)(q0 + gr / G) * p.q_stride + (size_t)(hk * G + gr % G) * D + c * 8;
            const int x = row / T5_BQ, rl = row % T5_BQ;
            t5_cp16(q_s + x * L::Q_BYTES + (c / 8) * L::Q_SPAN + rl * 128 + (((c % 8) ^ (rl & 7)) << 4), src, valid);
        }
        t5_commit_group();
        t5_wait_group<0>();
        t5_proxy_fence();  // what cp.async wrote becomes visible to the tensor cores' proxy
    }
    t5_fence_before();
    __syncthreads();
    t5_fence_after();
    const uint32_t tmem = *tmem_slot;
    bool ok = true;
    // every lane of a warp polls, so a wait that runs out ends the role for the whole warp
    auto wait_warp = [&](uint32_t bar, uint32_t parity, int code) {
        if (ok) ok = t5_wait(bar, parity, status, code);
        ok = __all_sync(0xffffffffu, ok);
        return ok;
    };

    if (warp == 9) {
        // ---- loader ------------------------------------------------------------------------
        constexpr uint32_t GROUP_BYTES = 16 * D * 2;  // 16 keys of one KV head
        constexpr int GROUPS = T5_BK / 16;
        uint32_t edges = 0;
        int issued = 0;
        for (int j = 0; j < n_all; ++j) {
            const int st = j % T5_STAGES;
            const uint32_t free_ph = (uint32_t)(j / T5_STAGES - 1) & 1u;
            const int kt = kt0 + j * T5_BK;
            // lane g < 8 finds the rows of key group g in the cache matrix (-1: no key of ours)
            const int key0 = kt + (lane & (GROUPS - 1)) * 16;
            int row = -1;
            if (key0 < k_end && key0 + 16 > k_begin)
                row = (table[key0 / p.page_size] * p.nkv + hk) * p.page_size + key0 % p.page_size;
            const uint32_t have = __ballot_sync(0xffffffffu, row >= 0) & ((1u << GROUPS) - 1);
            const uint32_t bytes = GROUP_BYTES * __popc(have);
            const bool edge = kt < k_begin || kt + T5_BK > k_end;  // some rows of the tile hold no key of ours
            if (j >= T5_STAGES && !wait_warp(kempty(st), free_ph, 11)) break;
            if (lane == 0) t5_expect_tx(kfull(st), bytes);
            __syncwarp();
            if (lane < GROUPS && row >= 0) {  // one lane per group issues its boxes
#pragma unroll
                for (int sp = 0; sp < L::SPANS; ++sp)
                    t5_tma_2d(k_s + st * L::KV_BYTES + sp * L::KV_SPAN + lane * 2048, &map_k, sp * 64, row, kfull(st));
            }
            if (j >= T5_STAGES && !wait_warp(vempty(st), free_ph, 12)) break;
            const uint32_t vbar = edge ? vland : vfull(st);
            if (lane == 0) t5_expect_tx(vbar, bytes);
            __syncwarp();
            if (lane < GROUPS && row >= 0) {
#pragma unroll
                for (int sp = 0; sp < L::SPANS; ++sp)
                    t5_tma_2d(v_s + st * L::KV_BYTES + sp * L::KV_SPAN + lane * 2048, &map_v, sp * 64, row, vbar);
            }
            issued = j + 1;
            if (edge) {
                // wait until V has landed, zero the rows without a key, then hand the tile over
                if (!wait_warp(vland, edges & 1u, 13)) break;
                ++edges;
                const uint32_t vdst = v_s + st * L::KV_BYTES;
                for (int idx = lane; idx < T5_BK * (D / 8); idx += 32) {
                    const int r = idx / (D / 8), c = idx % (D / 8);
                    const int key = kt + r;
                    if (key < k_begin || key >= k_end)  // whole rows: the swizzle only permutes within a row
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};"
                                     ::"r"(vdst + (c / 8) * L::KV_SPAN + r * 128 + (c % 8) * 16), "r"(0) : "memory");
                }
                t5_proxy_fence();
                __syncwarp();
                if (lane == 0) t5_arrive(vfull(st));
            }
        }
        if (!ok) {  // let the copies that were issued land before the block leaves
            for (int j = max(0, issued - T5_STAGES); j < issued; ++j) {
                t5_wait(kfull(j % T5_STAGES), (uint32_t)(j / T5_STAGES) & 1u, status, 20);
                t5_wait(vfull(j % T5_STAGES), (uint32_t)(j / T5_STAGES) & 1u, status, 20);
            }
        }
    } else if (warp == 8) {
        // ---- MMA issue: the warp runs the loop, one elected lane issues --------------------------
        const bool leader = t5_elect_one();
        const int n_of[2] = {n_a, n_b};
        auto issue_s = [&](int x, int j) {  // S_X(j) = Q_X K(j)^T
            const int st = j % T5_STAGES;
            const uint64_t dq = t5_desc(q_s + x * L::Q_BYTES, 16, 1024);
            const uint64_t dk = t5_desc(k_s + st * L::KV_BYTES, 16, 1024);
            if (leader) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)  // 16 elements of D: 32 bytes in a span, spans apart
                    t5_mma_ss(tmem + L::S_COL + x * T5_BK, dq + (uint64_t)((ks / 4) * (L::Q_SPAN >> 4) + 2 * (ks % 4)),
                              dk + (uint64_t)((ks / 4) * (L::KV_SPAN >> 4) + 2 * (ks % 4)), IDESC_S, ks > 0 ? 1u : 0u);
                t5_commit(sfull(x));
                if (x == 1 || j >= n_b) t5_commit(kempty(st));  // the last reader of this K tile
            }
            __syncwarp();
        };
        if (wait_warp(kfull(0), 0, 14)) {
            t5_fence_after();
            issue_s(0, 0);
            if (n_b > 0) issue_s(1, 0);
        }
        for (int j = 0; j < n_all && ok; ++j) {
            const int st = j % T5_STAGES;
            const uint32_t ring_ph = (uint32_t)(j / T5_STAGES) & 1u;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (j >= n_of[x] || !ok) continue;
                if (!wait_warp(pfull(x), (uint32_t)j & 1u, 15)) break;  // P_X(j) is written, O_X rescaled
                if (!wait_warp(vfull(st), ring_ph, 16)) break;
                t5_fence_after();
                // P: 16 keys = 8 columns of packed pairs.  V, MN-major: 16 keys = two 8-row groups
                // 1024 bytes apart (2048 bytes per step), D/64 spans KV_SPAN apart.
                const uint64_t dv = t5_desc(v_s + st * L::KV_BYTES, L::KV_SPAN, 1024);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < T5_BK / 16; ++kk)
                        t5_mma_ts(tmem + L::O_COL + x * D, tmem + L::S_COL + x * T5_BK + kk * 8,
                                  dv + (uint64_t)(kk * (2048 >> 4)), IDESC_PV, (j > 0 || kk > 0) ? 1u : 0u);
                    t5_commit(ofull(x));
                    if (x == 1 || j >= n_b) t5_commit(vempty(st));  // the last reader of this V tile
                }
                __syncwarp();
                if (j + 1 < n_of[x]) {
                    if (!wait_warp(kfull((j + 1) % T5_STAGES), (uint32_t)((j + 1) / T5_STAGES) & 1u, 17)) break;
                    t5_fence_after();
                    issue_s(x, j + 1);  // overwrites P_X(j) behind the products above (in issue order)
                }
            }
        }
        __syncwarp();
    } else {
        // ---- softmax: group X = warp / 4, thread = row ----------------------------------------
        const int x = warp >> 2, rl = tid & (T5_BQ - 1);
        const int n_mine = x == 0 ? n_a : n_b;
        const int my_row = r0 + x * T5_BQ + rl;
        const bool live = my_row < nrows;
        const int qpos = live ? start + my_row / G : -1;  // -1: sees no key
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + L::S_COL + x * T5_BK, o_addr = lane_base + L::O_COL + x * D;
        const float sl2 = p.scale_log2;
        float m_ref = -INFINITY, l_run = 0.f;  // reference point of the exponentials, running sum
        for (int j = 0; j < n_mine; ++j) {
            const int kt = kt0 + j * T5_BK;
            if (!wait_warp(sfull(x), (uint32_t)j & 1u, 18)) break;
            t5_fence_after();
            // visible keys of this row in the tile: lo <= i <= hi; only tiles on an edge pay for the mask
            const int hi = qpos - kt, lo = p.window > 0 ? qpos - p.window + 1 - kt : -(1 << 30);
            const bool masked = !__all_sync(0xffffffffu, hi >= T5_BK - 1 && lo <= 0);
            auto mask = [&](uint32_t (&v)[32], int c0) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (c0 + i > hi || c0 + i < lo) v[i] = 0xff800000u;  // -inf
            };
            // first pass over the row of S: its maximum
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c0 = 0; c0 < T5_BK; c0 += 64) {
                uint32_t va[32], vb[32];
                t5_ld32(s_addr + c0, va);
                t5_ld32(s_addr + c0 + 32, vb);
                t5_ld_wait();
                if (masked) {
                    mask(va, c0);
                    mask(vb, c0 + 32);
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(va[i]));
                    mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(vb[i]));
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = mx * sl2;  // -inf where the row sees nothing here
            const bool grow = m_new > m_ref + T5_RESCALE_LOG2 || (m_ref == -INFINITY && m_new > -INFINITY);
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                // O_X holds the tiles before this one once their last product has completed
                if (!wait_warp(ofull(x), (uint32_t)(j - 1) & 1u, 19)) break;
                t5_fence_after();
                const float f = grow ? t5_ex2(m_ref - m_new) : 1.0f;  // 0 from -inf: O and l are 0 there
                l_run *= f;
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t orr[32];
                    t5_ld32(o_addr + c0, orr);
                    t5_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * f);
                    t5_st32(o_addr + c0, orr);
                }
            }
            if (grow) m_ref = m_new;
            const float mb = m_ref == -INFINITY ? 0.f : m_ref;
            // second pass: P = 2^(s * scale - m) as bfloat16 pairs over the first half of S (the pairs
            // of columns [c0, c0 + 32) land in columns [c0 / 2, c0 / 2 + 16), which were read before)
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c0 = 0; c0 < T5_BK; c0 += 64) {
                uint32_t va[32], vb[32];
                t5_ld32(s_addr + c0, va);
                t5_ld32(s_addr + c0 + 32, vb);
                t5_ld_wait();
                if (masked) {
                    mask(va, c0);
                    mask(vb, c0 + 32);
                }
                uint32_t pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float e0 = t5_ex2(fmaf(__uint_as_float(va[i]), sl2, -mb));
                    const float e1 = t5_ex2(fmaf(__uint_as_float(va[i + 1]), sl2, -mb));
                    const float e2 = t5_ex2(fmaf(__uint_as_float(vb[i]), sl2, -mb));
                    const float e3 = t5_ex2(fmaf(__uint_as_float(vb[i + 1]), sl2, -mb));
                    ps4[(i >> 1) & 1] += e0 + e1;
                    ps4[2 + ((i >> 1) & 1)] += e2 + e3;
                    pa[i / 2] = t5_pack(e0, e1);
                    pb[i / 2] = t5_pack(e2, e3);
                }
                t5_st16(s_addr + c0 / 2, pa);
                t5_st16(s_addr + c0 / 2 + 16, pb);
            }
            l_run += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
            t5_st_wait();
            t5_fence_before();
            t5_arrive(pfull(x));
        }
        if (n_mine > 0 && wait_warp(ofull(x), (uint32_t)(n_mine - 1) & 1u, 21)) {
            t5_fence_after();
            const float inv = 1.0f / l_run;
            bf16* dst = p.out + ((size_t)(q0 + my_row / G) * p.nh + hk * G + my_row % G) * D;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t orr[32];
                t5_ld32(o_addr + c0, orr);
                t5_ld_wait();
                if (live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = t5_pack(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv);
                        w.y = t5_pack(__uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv);
                        w.z = t5_pack(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv);
                        w.w = t5_pack(__uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + i) = w;
                    }
                }
            }
        }
    }
    t5_fence_before();
    __syncthreads();
    if (warp == 8) {
        t5_fence_after();
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(L::TMEM_COLS) : "memory");
    }
}

template <int D>
int launch_prefill_tc05(const DecodeParams& p, int B, int max_q_len, cudaStream_t stream) {
    constexpr int smem = T5Layout<D>::SMEM;
    auto kernel = prefill_attention_tc05_kernel<D>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    int* status = tc_status_device_ptr();
    if (!status) return EMS_ERR_LAUNCH;
    // The kernel is not told how many pages the cache has (it trusts the block table, as the
    // other attention kernels do), so the maps cover the largest matrix the row index allows.
    CUtensorMap map_k, map_v;
    if (!tc_tensor_map_2d(p.kc, T5_MAX_ROWS, D, 16, &map_k) || !tc_tensor_map_2d(p.vc, T5_MAX_ROWS, D, 16, &map_v))
        return EMS_ERR_LAUNCH;
    long long tiles = ((long long)max_q_len * p.G + 2 * T5_BQ - 1) / (2 * T5_BQ);
    // Pairs of row tiles let the tensor pipe work on one tile during the other's softmax, but where
    // the pairs would not even fill half of the SMs, one tile per block and twice the blocks is
    // faster (7B heads, 512 tokens: 17.4 us against 21.3; 0.5B heads, 1024 tokens: 21.7 against 25.0;
    // from 1024 tokens at the 7B heads on, pairs win).  A row's result does not depend on the choice.
    static int sms_cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return EMS_ERR_LAUNCH;
    if (sms_cached[dev] == 0 &&
        cudaDeviceGetAttribute(&sms_cached[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    const int single = tiles * p.nkv * B * 2 <= sms_cached[dev] ? 1 : 0;
    if (single) tiles = ((long long)max_q_len * p.G + T5_BQ - 1) / T5_BQ;
    if (tiles > 65535 || (long long)p.nkv * B > 2147483647LL) return EMS_ERR_SHAPE;
    const dim3 grid((unsigned)(p.nkv * B), (unsigned)tiles, 1u);
    kernel<<<grid, T5_THREADS, smem, stream>>>(p, status, map_k, map_v, single);
    return launch_status();
}

// Head sizes 64 and 128 and pages of a multiple of 16 keys (a box of the tensor map is 16 keys
// of one page); everything else is left to the mma.sync kernel.
bool prefill_tc05_supported(int dtype, int D, int page_size, long long q_stride, const void* q, const void* out,
                            const void* kc, const void* vc) {
    if (dtype != EMS_BF16 || (D != 64 && D != 128) || page_size % 16) return false;
    if ((q_stride * 2) % 16 || ((uintptr_t)q % 16) || ((uintptr_t)out % 16) || ((uintptr_t)kc % 16) ||
        ((uintptr_t)vc % 16))
        return false;
    return true;
}

int run_prefill_tc05(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream) {
    return D == 64 ? launch_prefill_tc05<64>(p, B, max_q_len, stream) : launch_prefill_tc05<128>(p, B, max_q_len, stream);
}

}  // namespace ems
