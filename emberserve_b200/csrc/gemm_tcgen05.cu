// y = x W^T for few rows of x (decode steps): a weight-streaming GEMM on the fifth-generation
// tensor cores.
//
// With 1..64 token rows the product is a bandwidth problem: every weight is read once and
// used a few times.  So the WEIGHT matrix is put on the 128-row side of the MMA and the
// tokens on its N side (8..64 columns): a block owns 128 output features and a range of
// K, streams its weight tile through a ring of shared-memory stages with TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), and one elected thread issues
// tcgen05.mma (kind::f16, bfloat16 inputs, float32 accumulators in tensor memory) on the
// stages as they land; tcgen05.commit hands each stage back to the TMA producer.  When the
// block's K range is done the four warps read their 32 accumulator lanes from tensor
// memory (tcgen05.ld) and store them.  When K is split over several blocks so that all SMs
// stream, those blocks are one thread-block cluster: every block PUSHES its float32 partial
// rows into the shared memory of the block that owns them (st.async, counted by that block's
// mbarrier), and each owner adds what arrived in rank order, adds the bias and rounds once.
// A push is one trip through the cluster's network; no block waits at a cluster barrier
// after its K loop, and none pulls.
//
// The reference's engine calls cuBLAS for these products (emberserve/model/qwen2.py:57-58,
// 77-79,203); this kernel replaces the library where the row count is small.
//
// Every wait on an mbarrier is bounded: if it runs out, the block records a code in a
// status word that the host can read, stops issuing work, lets what it has in flight
// land, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace ems {

constexpr int G5_BM = 128;      // output features per block (MMA M)
constexpr int G5_BK = 64;       // K per stage: 64 bf16 = one 128-byte swizzle span
// Stages of the ring: as many as let two blocks share an SM beside the inbox of the split-K
// reduction (the blocks of the next kernel must be able to move in while this one drains, and two
// rings in flight feed the memory better).
#ifndef G5_DUAL_STAGES
#define G5_DUAL_STAGES 5
#endif
template <int NT, int COLS, bool DUAL> constexpr int g5_stages() {
    return DUAL ? G5_DUAL_STAGES : (NT <= 16 ? (COLS <= 8 ? 6 : 5) : (NT <= 32 ? 4 : 3));
}
constexpr int G5_THREADS = 128;
// Rows of the inbox: `ksplit` senders times the rows a block owns (128 / ksplit, rounded up to 4).
constexpr int G5_INBOX_ROWS = 128 + 4 * 8;
template <int COLS, bool DUAL> constexpr int g5_inbox_bytes() { return DUAL ? 0 : G5_INBOX_ROWS * COLS * 4; }

struct Gemm5Params {
    void* y;             // [M_tok, N_out] bf16, or float32 (y_f32: unsplit plain products only)
    int y_f32;
    const bf16* bias;    // [N_out] or null
    int* status;         // device-visible status word
    int m_tok, n_out, k_tiles;
    int ksplit;          // > 1: the ksplit blocks of a row tile are a cluster and reduce on chip
    int dual_offset;     // DUAL kernels: row distance between the two weight tiles
    // The weights as a TILED copy: the 128 x 64 tile (row tile r, K tile kt) is 16 KB of contiguous
    // memory at tile index r * k_tiles + kt, so that a TMA load reads whole DRAM pages instead of
    // 128 bytes from each of 128 rows.  0: the row-major matrix itself.
    int tiled;
    // The norm that stands BEHIND this product, begun in its epilogue (plain kernels, at most 16
    // rows): the product is added into the float32 residual stream `res` [m_tok, n_out] instead
    // of being stored, `scaled` gets bf16(res * gain), and every block leaves the sum of res^2
    // over its share of the columns, per row, in sumsq_out[(tile * ksplit + rank) * 16 + row].
    float* res;
    const bf16* gain;
    bf16* scaled;
    float* sumsq_out;
    // The norm that stands BEFORE this product, finished in its epilogue: the activations it was
    // given are res * gain of such a producer, and row n of the result is multiplied by
    // 1 / sqrt(sum_parts sumsq_in[part * 16 + n] * in_inv_width + in_eps) before the bias is added.
    const float* sumsq_in;
    int in_parts;
    float in_inv_width, in_eps;
};

constexpr int G5_NORM_ROWS = 16;  // rows (tokens) of a step up to which the norms are fused into the products

template <int N> __device__ __forceinline__ void tc_ld_cols(uint32_t taddr, float (&v)[N]);
template <> __device__ __forceinline__ void tc_ld_cols<16>(uint32_t taddr, float (&v)[16]) { tc_ld16(taddr, v); }

// NT: token columns of the MMA (16, 32 or 64; with 128 weight rows per MMA, multiples of 16).
// COLS: how many of them hold tokens, NT or, for up to 8 tokens, 8: then a stage holds only 8
// activation rows (one 1 KB swizzle atom), the MMA's upper 8 columns read whatever lies behind
// them in shared memory, and their accumulators are never looked at.  The kilobytes saved buy
// a sixth stage beside the inbox.
// DUAL: the block owns TWO weight tiles, rows [tile*128, +128) and the same rows `dual_offset`
// further down (gate and up projections of a gated feed-forward), accumulates both, and
// stores silu(first) * second: the activation never goes to memory unfused.
// Split K (ksplit > 1): the ksplit blocks of a row tile form a thread-block cluster and add
// their accumulators through distributed shared memory, in rank order.
template <int NT, int COLS, bool DUAL>
__global__ void __launch_bounds__(G5_THREADS)
gemm_smallm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           const Gemm5Params p) {
    constexpr int STAGES = g5_stages<NT, COLS, DUAL>();
    constexpr uint32_t W_BYTES = G5_BM * G5_BK * 2;               // 16 KB per weight tile
    constexpr uint32_t A_BYTES = (DUAL ? 2 : 1) * W_BYTES;
    constexpr uint32_t B_BYTES = COLS * G5_BK * 2;                // 1..8 KB
    constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * NT;
    constexpr uint32_t TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;
    constexpr uint32_t INBOX_BYTES = g5_inbox_bytes<COLS, DUAL>();
    constexpr int LD = 16;  // accumulator columns per tensor-memory load
    // instruction descriptor: D float32, A and B bfloat16, both K-major, N = NT, M = 128
    constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NT >> 3) << 17) |
                               ((uint32_t)(G5_BM >> 4) << 24);
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
    float* rstd_s = reinterpret_cast<float*>(bars + 2 * STAGES + 4);  // [16] scale of each row (norm before)
    float* ssq_s = rstd_s + G5_NORM_ROWS;                             // [16][32] partial sums (norm behind)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, ks = blockIdx.y;
    // this block's K tiles
    const int per = (p.k_tiles + p.ksplit - 1) / p.ksplit;
    const int kt_begin = ks * per, kt_end = min(p.k_tiles, kt_begin + per);
    const int nk = max(0, kt_end - kt_begin);
    // split K: rank `me` of the cluster owns output rows [me * owned, +owned) of the tile
    const bool split = !DUAL && p.ksplit > 1;
    const int me = split ? (int)cluster_rank() : 0;
    const int owned = (((G5_BM + p.ksplit - 1) / p.ksplit) + 3) & ~3;
    const int my_rows = max(0, min(owned, G5_BM - me * owned));

    // the weight tile(s) of K tile `kt` into a stage
    auto load_w = [&](uint32_t dst, int kt, uint32_t bar) {
        if (p.tiled) {
            tma_load_2d(dst, &map_w, 0, (tile * p.k_tiles + kt) * G5_BM, bar);
            if (DUAL) tma_load_2d(dst + W_BYTES, &map_w, 0, ((p.dual_offset / G5_BM + tile) * p.k_tiles + kt) * G5_BM, bar);
        } else {
            tma_load_2d(dst, &map_w, kt * G5_BK, tile * G5_BM, bar);
            if (DUAL) tma_load_2d(dst + W_BYTES, &map_w, kt * G5_BK, p.dual_offset + tile * G5_BM, bar);
        }
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(done_bar, 1);
        mbar_init(inbox_bar, 1);
        // what the blocks of the cluster (this one included) will push here: COLS floats per owned row each
        if (split && my_rows > 0) mbar_expect_tx(inbox_bar, (uint32_t)(p.ksplit * my_rows * COLS * 4));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The weights do not depend on the kernel before this one: the first ring of weight tiles
        // is requested at once, before the block has even set up its tensor memory (this thread
        // is the producer below); the activations follow after the dependency wait.
        const int pre = min(nk, STAGES);
        for (int it = 0; it < pre; ++it) {
            mbar_expect_tx(full0 + 8 * it, A_BYTES + B_BYTES);
            load_w(a_s + it * A_BYTES, kt_begin + it, full0 + 8 * it);
        }
    }
    if (warp == 1) {  // tensor memory for the accumulators: TMEM_COLS columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
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

    // What the epilogue of a split product will need from global memory for this thread's first
    // four outputs, asked for now, while the block waits and streams: bias and gain are weights
    // and are loaded; the residual row may still be written by a kernel before this one, so it is
    // only asked into L2 (a step has read hundreds of megabytes since it was last touched).
    const int quads = owned >> 2;
    const int my_n = threadIdx.x / quads, my_rl = (threadIdx.x % quads) * 4;
    const int my_orow = tile * G5_BM + me * owned + my_rl;
    const bool my_quad = split && (int)threadIdx.x < quads * p.m_tok && me * owned + my_rl + 3 < G5_BM &&
                         my_orow + 3 < p.n_out && (p.n_out & 3) == 0;
    uint2 gain_pre = make_uint2(0u, 0u), bias_pre = make_uint2(0u, 0u);
    if (my_quad) {
        if (p.bias) bias_pre = *reinterpret_cast<const uint2*>(p.bias + my_orow);
        if (p.res) {
            gain_pre = *reinterpret_cast<const uint2*>(p.gain + my_orow);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.res + (size_t)my_n * p.n_out + my_orow));
        }
    }

    if (warp == 0 && lane == 0) {
        // ---- TMA producer (the first ring of weight tiles is on its way already) ----------
        const int pre = min(nk, STAGES);
        grid_dependency_wait();
        for (int it = 0; it < pre; ++it)
            tma_load_2d(b_s + it * B_BYTES, &map_x, (kt_begin + it) * G5_BK, 0, full0 + 8 * it);
        int armed = pre;
        for (int it = pre; it < nk && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            ok = mbar_wait(empty0 + 8 * s, ph ^ 1u, p.status, 1);
            if (!ok) break;
            mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
            const int k0 = (kt_begin + it) * G5_BK;
            load_w(a_s + s * A_BYTES, kt_begin + it, full0 + 8 * s);
            tma_load_2d(b_s + s * B_BYTES, &map_x, k0, 0, full0 + 8 * s);
            armed = it + 1;
        }
        if (!ok) {  // let the copies that were issued land before the block leaves
            for (int it = max(0, armed - STAGES); it < armed; ++it)
                mbar_wait(full0 + 8 * (it % STAGES), (uint32_t)(it / STAGES) & 1u, p.status, 4);
        }
    } else if (warp == 1) {
        // ---- MMA issue: the warp runs the loop, one elected lane issues (a lone diverged lane
        // leaves the tensor pipe idle for a while after every commit) -----------------------
        const bool issuer = elect_one();
        for (int it = 0; it < nk && ok; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, ph, p.status, 2));
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = smem_desc_sw128(a_s + s * A_BYTES), db = smem_desc_sw128(b_s + s * B_BYTES);
            if (issuer) {
#pragma unroll
                for (int k = 0; k < G5_BK / 16; ++k) {  // 16 K per MMA = 32 bytes = 2 descriptor units
                    const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
                    tc_mma_bf16(tmem_d, da + 2 * k, db + 2 * k, IDESC, acc);
                    if (DUAL) tc_mma_bf16(tmem_d + NT, da + (W_BYTES >> 4) + 2 * k, db + 2 * k, IDESC, acc);
                }
                tc_commit(empty0 + 8 * s);  // arrives once these MMAs have read the stage
            }
            __syncwarp();
        }
        if (issuer) tc_commit(done_bar);    // arrives once every MMA issued above has completed
    }
    __syncwarp();

    // ---- epilogue: all four warps, 32 accumulator lanes (= output features) each -------
    grid_dependency_wait();  // (the producer has passed it already; this orders the stores below)
    allow_dependent_launch();  // a GEMM that follows may set up and fetch weights as blocks retire
    if (p.sumsq_in != nullptr && warp >= 2) {
        // the scale of each row, by the two warps that had nothing to do so far (they get here as
        // soon as the kernel before has completed): four threads per row add the partial sums
        // in a fixed pattern
        const int t = threadIdx.x - 64, n = t >> 2, j = t & 3;
        float sum = 0.f;
        for (int part = j; part < p.in_parts; part += 4) sum += p.sumsq_in[(size_t)part * G5_NORM_ROWS + n];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (j == 0) rstd_s[n] = 1.0f / sqrtf(sum * p.in_inv_width + p.in_eps);
    }
    bool done = true;
    if (lane == 0) done = mbar_wait(done_bar, 0, p.status, 3);
    done = __shfl_sync(0xffffffffu, done ? 1 : 0, 0) != 0;
    tc_fence_after();
    const bool scale_rows = p.sumsq_in != nullptr;
    if (scale_rows) __syncthreads();  // rstd_s is written
    const int row_local = warp * 32 + lane;
    const int row = tile * G5_BM + row_local;  // output feature of this thread
    const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
    const bool have = done && nk > 0;
    if (DUAL) {
        if (have) {
#pragma unroll
            for (int c0 = 0; c0 < COLS; c0 += LD) {
                float g[LD], u[LD];
                tc_ld_cols<LD>(taddr + c0, g);
                tc_ld_cols<LD>(taddr + NT + c0, u);
                if (row < p.n_out) {
                    bf16* y = reinterpret_cast<bf16*>(p.y);
#pragma unroll
                    for (int i = 0; i < LD; ++i)
                        if (c0 + i < p.m_tok) {
                            const float sc = scale_rows ? rstd_s[c0 + i] : 1.0f;
                            const float gi = g[i] * sc, ui = u[i] * sc;
                            y[(size_t)(c0 + i) * p.n_out + row] = __float2bfloat16_rn(gi / (1.0f + expf(-gi)) * ui);
                        }
                }
            }
        }
    } else if (split) {
        // push: this thread's accumulator row goes to the block that owns it, into the slot of
        // this block's rank; inbox layout [sender][owned row][token]
        const uint32_t dst_rank = (uint32_t)(row_local / owned);
        const uint32_t slot = smem_u32(inbox) + (uint32_t)((me * owned + row_local % owned) * COLS) * 4u;
#pragma unroll
        for (int c0 = 0; c0 < COLS; c0 += LD) {
            float v[LD];
            if (have) tc_ld_cols<LD>(taddr + c0, v);
#pragma unroll
            for (int i = 0; i < LD && c0 + i < COLS; i += 4) {
                const bool z = !have;  // a block without K (or whose waits ran out) pushes zeros: nobody waits in vain
                push_f32x4(slot + (uint32_t)(c0 + i) * 4u, inbox_bar, dst_rank, z ? 0.f : v[i], z ? 0.f : v[i + 1],
                           z ? 0.f : v[i + 2], z ? 0.f : v[i + 3]);
            }
        }
        // own: add what the ksplit blocks pushed for my rows, in rank order (the same for every batch)
        if (my_rows > 0) {
            // (norm behind) what this thread's first four outputs join, read while the pushes travel
            const bool norm_behind = p.res != nullptr;
            float4 res_pre = make_float4(0.f, 0.f, 0.f, 0.f);
            const bool pre = norm_behind && my_quad;
            if (pre) res_pre = *reinterpret_cast<const float4*>(p.res + (size_t)my_n * p.n_out + my_orow);
            bool arrived = true;
            if (lane == 0) arrived = mbar_wait(inbox_bar, 0, p.status, 5);
            arrived = __shfl_sync(0xffffffffu, arrived ? 1 : 0, 0) != 0;
            if (arrived) mbar_try_wait(inbox_bar, 0);  // (every thread observes the completed phase itself)
            bf16* y = reinterpret_cast<bf16*>(p.y);
            for (int idx = threadIdx.x; idx < quads * p.m_tok && arrived; idx += G5_THREADS) {
                const int n = idx / quads, rl = (idx % quads) * 4;
                const int orow = tile * G5_BM + me * owned + rl;
                if (norm_behind) ssq_s[n * 32 + idx % quads] = 0.f;
                if (me * owned + rl >= G5_BM || orow >= p.n_out) continue;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int r = 0; r < p.ksplit; ++r) {
                    const float* src = inbox + (size_t)((r * owned + rl) * COLS + n);
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[e] += src[e * COLS];
                }
                const float sc = scale_rows ? rstd_s[n] : 1.0f;
                if (my_quad && idx == (int)threadIdx.x) {  // the bias is in registers already
                    const float2 b01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bias_pre.x));
                    const float2 b23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bias_pre.y));
                    acc[0] = acc[0] * sc + b01.x; acc[1] = acc[1] * sc + b01.y;
                    acc[2] = acc[2] * sc + b23.x; acc[3] = acc[3] * sc + b23.y;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[e] *= sc;
                        if (orow + e < p.n_out && p.bias) acc[e] += __bfloat162float(p.bias[orow + e]);
                    }
                }
                if (norm_behind) {
                    // the product joins the residual stream here; the norm behind it gets its gain
                    // applied and its statistic begun
                    const size_t at = (size_t)n * p.n_out + orow;
                    float r[4], gn[4];
                    bool valid[4];
                    if (pre && idx == (int)threadIdx.x) {
                        r[0] = res_pre.x; r[1] = res_pre.y; r[2] = res_pre.z; r[3] = res_pre.w;
                        const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gain_pre.x));
                        const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gain_pre.y));
                        gn[0] = g01.x; gn[1] = g01.y; gn[2] = g23.x; gn[3] = g23.y;
#pragma unroll
                        for (int e = 0; e < 4; ++e) valid[e] = true;
                    } else {  // every load before the first store (the stores may alias them for all the compiler knows)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            valid[e] = me * owned + rl + e < G5_BM && orow + e < p.n_out;
                            r[e] = valid[e] ? p.res[at + e] : 0.f;
                            gn[e] = valid[e] ? __bfloat162float(p.gain[orow + e]) : 0.f;
                        }
                    }
                    float ss = 0.f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        r[e] += acc[e];
                        if (valid[e]) ss += r[e] * r[e];
                    }
                    if (pre && idx == (int)threadIdx.x) {
                        *reinterpret_cast<float4*>(p.res + at) = make_float4(r[0], r[1], r[2], r[3]);
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(r[0] * gn[0], r[1] * gn[1]);
                        const __nv_bfloat162 hi = __floats2bfloat162_rn(r[2] * gn[2], r[3] * gn[3]);
                        uint2 o;
                        o.x = *reinterpret_cast<const uint32_t*>(&lo); o.y = *reinterpret_cast<const uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(p.scaled + at) = o;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (valid[e]) {
                                p.res[at + e] = r[e];
                                p.scaled[at + e] = __float2bfloat16_rn(r[e] * gn[e]);
                            }
                    }
                    ssq_s[n * 32 + idx % quads] = ss;
                    continue;
                }
                bf16* dst = y + (size_t)n * p.n_out + orow;
                if (me * owned + rl + 3 < G5_BM && orow + 3 < p.n_out && ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0)) {
                    uint2 o;
                    __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0], acc[1]), hi = __floats2bfloat162_rn(acc[2], acc[3]);
                    o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(dst) = o;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (me * owned + rl + e < G5_BM && orow + e < p.n_out) dst[e] = __float2bfloat16_rn(acc[e]);
                }
            }
            if (norm_behind) {  // this block's share of each row's sum of squares, added in a fixed order
                __syncthreads();
                if (threadIdx.x < p.m_tok) {
                    float sum = 0.f;
                    for (int q = 0; q < quads; ++q) sum += ssq_s[threadIdx.x * 32 + q];
                    p.sumsq_out[(size_t)(tile * p.ksplit + me) * G5_NORM_ROWS + threadIdx.x] = arrived ? sum : 0.f;
                }
            }
        }
    } else {
        const bool norm_behind = p.res != nullptr;
        if (have) {
#pragma unroll
            for (int c0 = 0; c0 < COLS; c0 += LD) {
                float v[LD], r[LD];
                tc_ld_cols<LD>(taddr + c0, v);
                const float bias = (row < p.n_out && p.bias) ? __bfloat162float(p.bias[row]) : 0.f;
                bf16* y = reinterpret_cast<bf16*>(p.y);
                const float gn = (norm_behind && row < p.n_out) ? __bfloat162float(p.gain[row]) : 0.f;
                if (norm_behind) {  // every load before the first store
#pragma unroll
                    for (int i = 0; i < LD; ++i)
                        r[i] = (c0 + i < p.m_tok && row < p.n_out) ? p.res[(size_t)(c0 + i) * p.n_out + row] : 0.f;
                }
#pragma unroll
                for (int i = 0; i < LD; ++i) {
                    if (c0 + i >= p.m_tok) continue;
                    const float out = v[i] * (scale_rows ? rstd_s[c0 + i] : 1.0f) + bias;
                    if (!norm_behind) {
                        if (row < p.n_out) {
                            if (p.y_f32) reinterpret_cast<float*>(p.y)[(size_t)(c0 + i) * p.n_out + row] = out;
                            else y[(size_t)(c0 + i) * p.n_out + row] = __float2bfloat16_rn(out);
                        }
                        continue;
                    }
                    float sq = 0.f;
                    if (row < p.n_out) {
                        const size_t at = (size_t)(c0 + i) * p.n_out + row;
                        const float sum = r[i] + out;
                        p.res[at] = sum;
                        p.scaled[at] = __float2bfloat16_rn(sum * gn);
                        sq = sum * sum;
                    }
                    sq = warp_sum(sq);
                    if (lane == 0) ssq_s[(c0 + i) * 32 + warp] = sq;
                }
            }
        }
        if (norm_behind) {  // (p.m_tok <= 16 = COLS or less: one pass of the loop above)
            __syncthreads();
            if (threadIdx.x < p.m_tok) {
                float sum = 0.f;
                for (int w = 0; w < G5_THREADS / 32; ++w) sum += ssq_s[threadIdx.x * 32 + w];
                p.sumsq_out[(size_t)tile * G5_NORM_ROWS + threadIdx.x] = have ? sum : 0.f;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side: tensor maps and launch ---------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr; long long rows, cols; int box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^
               (std::hash<long long>()(k.cols) * 131) ^ (size_t)k.box_rows;
    }
};

// Tensor map of a row-major bf16 matrix [rows, cols], box [box_rows, 64 columns], 128-byte
// swizzle, zeros outside the matrix.  Maps are cached: the same weight is mapped once.
static bool tensor_map_2d(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)G5_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap map;
    if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, map);
    *out = map;
    return true;
}

// The tensor map of a weight [rows, cols] for 128-row boxes: of the row-major matrix, or of its
// tiled copy (rows and cols multiples of 128 and 64), which is a matrix of 64 columns whose rows
// [t * 128, +128) are tile t = row tile * (cols / 64) + K tile.
static bool weight_map(const void* w, long long rows, long long cols, bool tiled, CUtensorMap* out) {
    if (!tiled) return tensor_map_2d(w, rows, cols, G5_BM, out);
    if (rows % G5_BM || cols % G5_BK) return false;
    return tensor_map_2d(w, rows * (cols / G5_BK), G5_BK, G5_BM, out);
}

static int* status_word() {  // host-mapped, so the host reads it without a CUDA call
    static int* host = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        if (cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped) == cudaSuccess) *host = 0;
        else host = nullptr;
    });
    return host;
}

// The same word serves the other tcgen05 kernels of the library (the prompt attention).
int* tc_status_device_ptr() { return status_word(); }
bool tc_tensor_map_2d(const void* ptr, long long rows, long long cols, int box_rows, CUtensorMap* out) {
    return tensor_map_2d(ptr, rows, cols, box_rows, out);
}
bool tc_weight_map(const void* w, long long rows, long long cols, bool tiled, CUtensorMap* out) {
    return weight_map(w, rows, cols, tiled, out);
}

template <int NT, int COLS, bool DUAL> constexpr int g5_smem_bytes() {
    // (the last stage's MMA reads NT activation rows where only COLS were loaded: room for them)
    return g5_stages<NT, COLS, DUAL>() * ((DUAL ? 2 : 1) * G5_BM * G5_BK * 2 + COLS * G5_BK * 2) +
           (NT - COLS) * G5_BK * 2 * (DUAL ? 1 : 0) + g5_inbox_bytes<COLS, DUAL>() +
           (2 * g5_stages<NT, COLS, DUAL>() + 2) * 8 + 16 + (G5_NORM_ROWS + G5_NORM_ROWS * 32) * 4 + 1024;
}

template <int NT, int COLS, bool DUAL>
static void fill_launch(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int tiles, int ksplit, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(tiles, ksplit);
    cfg.blockDim = dim3(G5_THREADS);
    cfg.dynamicSmemBytes = g5_smem_bytes<NT, COLS, DUAL>();
    cfg.stream = stream;
    int nattr = 0;
    // may start while the kernel before it still runs (see grid_dependency_wait)
    attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[nattr].val.programmaticStreamSerializationAllowed = 1;
    ++nattr;
    if (ksplit > 1) {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = 1;
        attr[nattr].val.clusterDim.y = ksplit;
        attr[nattr].val.clusterDim.z = 1;
        ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
}

template <int NT, int COLS, bool DUAL>
static int launch_gemm5(const CUtensorMap& mw, const CUtensorMap& mx, const Gemm5Params& p, int tiles,
                        cudaStream_t stream) {
    auto kernel = gemm_smallm_tcgen05_kernel<NT, COLS, DUAL>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, g5_smem_bytes<NT, COLS, DUAL>()) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    fill_launch<NT, COLS, DUAL>(cfg, attr, tiles, p.ksplit, stream);
    if (cudaLaunchKernelEx(&cfg, kernel, mw, mx, p) != cudaSuccess) {
        cudaGetLastError();
        return EMS_ERR_LAUNCH;
    }
    return launch_status();
}

static inline int nt_for(int m_tok) { return m_tok <= 16 ? 16 : (m_tok <= 32 ? 32 : 64); }

}  // namespace ems

using namespace ems;

// 0 while no kernel of this file has recorded a failed wait; else the code of the first one
// (1 producer, 2 MMA issuer, 3 epilogue, 4 drain, 5 arrival of the split-K partials).
EMS_EXPORT int ems_gemm_smallm_status(void) {
    int* s = status_word();
    return s ? *s : -1;
}

// Set the word back to 0 once the host has acted on a code (no kernel of the library may be
// in flight: the caller has synchronised).
EMS_EXPORT void ems_tc_status_clear(void) {
    int* s = status_word();
    if (s) *s = 0;
}

// The norm before a product, to be finished in its epilogue (Gemm5Params::sumsq_in); false if the
// arguments do not make sense.
static bool fill_norm_before(Gemm5Params& p, const float* sumsq_in, int in_parts, int in_width, float in_eps) {
    p.sumsq_in = sumsq_in; p.in_parts = in_parts; p.in_eps = in_eps;
    p.in_inv_width = in_width > 0 ? 1.0f / (float)in_width : 0.f;
    return sumsq_in == nullptr || (p.m_tok <= G5_NORM_ROWS && in_parts > 0 && in_width > 0);
}

// y[m_tok, n_out] (bf16) = x[m_tok, k] (bf16, row-major) . w[n_out, k]^T (+ bias).
// m_tok <= 64; k a multiple of 8; 16-byte aligned pointers.  ksplit in 1..8 blocks share K: they
// form a thread-block cluster and add their accumulators on chip.
// With `res` (m_tok <= 16): the product is added into the float32 stream res[m_tok, n_out] instead of
// being stored in y, scaled[m_tok, n_out] = bf16(res * gain), and sumsq_out[tiles * ksplit, 16] gets
// every block's share of each row's sum of squares (the norm behind the product).  With `sumsq_in`
// (m_tok <= 16): row n of the product is multiplied by 1 / sqrt(sum over in_parts of
// sumsq_in[part, n] / in_width + in_eps) before the bias is added (the norm before it).
// `tiled`: w is the tiled copy of the weight (tc_weight_map).  `y_f32`: y is float32 and takes the
// sums unrounded (ksplit 1, no `res`).
EMS_EXPORT int ems_gemm_smallm(const void* x, const void* w, const void* bias, void* y, int m_tok, int n_out,
                               int k, int ksplit, float* res, const void* gain, void* scaled, float* sumsq_out,
                               const float* sumsq_in, int in_parts, int in_width, float in_eps, int tiled,
                               int y_f32, cudaStream_t stream) {
    if (m_tok <= 0 || n_out <= 0) return EMS_OK;
    // (float32 output, the logits of a language-model head: never rounded, so only where one block
    // holds the whole sum and stores it itself)
    if (y_f32 && (ksplit != 1 || res != nullptr || ((uintptr_t)y % 4))) return EMS_ERR_SHAPE;
    if (m_tok > 64 || k <= 0 || k % 8 || ksplit < 1 || ksplit > 8) return EMS_ERR_SHAPE;  // 8: the portable cluster size
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)y % 2)) return EMS_ERR_ALIGN;
    if (res != nullptr && (m_tok > G5_NORM_ROWS || gain == nullptr || scaled == nullptr || sumsq_out == nullptr))
        return EMS_ERR_SHAPE;
    if (res == nullptr && y == nullptr) return EMS_ERR_SHAPE;
    int* status = status_word();
    if (!status) return EMS_ERR_LAUNCH;
    int* status_dev = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev), status, 0) != cudaSuccess) return EMS_ERR_LAUNCH;
    const int nt = nt_for(m_tok);
    CUtensorMap mw, mx;
    if (!weight_map(w, n_out, k, tiled != 0, &mw) || !tensor_map_2d(x, m_tok, k, m_tok <= 8 ? 8 : nt, &mx)) return EMS_ERR_LAUNCH;
    Gemm5Params p;
    p.tiled = tiled ? 1 : 0;
    p.y_f32 = y_f32 ? 1 : 0;
    p.y = y; p.bias = reinterpret_cast<const bf16*>(bias);
    p.status = status_dev; p.m_tok = m_tok; p.n_out = n_out; p.k_tiles = (k + G5_BK - 1) / G5_BK; p.ksplit = ksplit;
    p.dual_offset = 0;
    p.res = res; p.gain = reinterpret_cast<const bf16*>(gain); p.scaled = reinterpret_cast<bf16*>(scaled);
    p.sumsq_out = sumsq_out;
    if (!fill_norm_before(p, sumsq_in, in_parts, in_width, in_eps)) return EMS_ERR_SHAPE;
    const int tiles = (n_out + G5_BM - 1) / G5_BM;
    if (m_tok <= 8) return launch_gemm5<16, 8, false>(mw, mx, p, tiles, stream);
    if (nt == 16) return launch_gemm5<16, 16, false>(mw, mx, p, tiles, stream);
    if (nt == 32) return launch_gemm5<32, 32, false>(mw, mx, p, tiles, stream);
    return launch_gemm5<64, 64, false>(mw, mx, p, tiles, stream);
}

// act[m_tok, inter] (bf16) = silu(x . w[0:inter]^T) * (x . w[inter:2*inter]^T): the gated
// feed-forward's first two projections and its activation in one kernel.  w: [2*inter, k].
// `sumsq_in` ...: the norm before the product, as for ems_gemm_smallm (both halves are scaled).
EMS_EXPORT int ems_gemm_smallm_gated(const void* x, const void* w, void* act, int m_tok, int inter, int k,
                                     const float* sumsq_in, int in_parts, int in_width, float in_eps, int tiled,
                                     cudaStream_t stream) {
    if (m_tok <= 0 || inter <= 0) return EMS_OK;
    if (m_tok > 64 || k <= 0 || k % 8) return EMS_ERR_SHAPE;
    if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)act % 2)) return EMS_ERR_ALIGN;
    int* status = status_word();
    if (!status) return EMS_ERR_LAUNCH;
    int* status_dev = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&status_dev), status, 0) != cudaSuccess) return EMS_ERR_LAUNCH;
    const int nt = nt_for(m_tok);
    CUtensorMap mw, mx;
    if (tiled && inter % G5_BM) return EMS_ERR_SHAPE;
    if (!weight_map(w, 2LL * inter, k, tiled != 0, &mw) || !tensor_map_2d(x, m_tok, k, m_tok <= 8 ? 8 : nt, &mx)) return EMS_ERR_LAUNCH;
    Gemm5Params p;
    p.tiled = tiled ? 1 : 0;
    p.y_f32 = 0;
    p.y = act; p.bias = nullptr; p.status = status_dev; p.m_tok = m_tok; p.n_out = inter;
    p.k_tiles = (k + G5_BK - 1) / G5_BK; p.ksplit = 1; p.dual_offset = inter;
    p.res = nullptr; p.gain = nullptr; p.scaled = nullptr; p.sumsq_out = nullptr;
    if (!fill_norm_before(p, sumsq_in, in_parts, in_width, in_eps)) return EMS_ERR_SHAPE;
    const int tiles = (inter + G5_BM - 1) / G5_BM;
    if (m_tok <= 8) return launch_gemm5<16, 8, true>(mw, mx, p, tiles, stream);
    if (nt == 16) return launch_gemm5<16, 16, true>(mw, mx, p, tiles, stream);
    if (nt == 32) return launch_gemm5<32, 32, true>(mw, mx, p, tiles, stream);
    return launch_gemm5<64, 64, true>(mw, mx, p, tiles, stream);
}
