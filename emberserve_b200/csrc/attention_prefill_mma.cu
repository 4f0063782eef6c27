// Paged causal grouped-query attention for prompt portions (and any mix of rows) in
// bfloat16 on the tensor cores: the flash-attention scheme over block tables.
//
// A block of four warps owns 64 "rows" of one request and one KV head, a row being
// (query token, query head of the group): row r -> token r / G, head r % G, so the G heads
// that share a KV head share every K/V tile.  Keys are walked in tiles of 64 whose
// boundaries are multiples of 64 in absolute position (the order of additions for a query
// does not depend on how the prompt was cut), double-buffered through shared memory with
// cp.async; pages are found through the block table row by row, so any page size works.
// S = Q K^T and O += P V are mma.sync m16n8k16 bf16 products with float32 accumulators;
// the online softmax is float32 with base-2 exponentials.  A window of W keys hides keys
// at positions <= p - W from the query at position p.
//
// Formulas: emberserve/attn/base.py:105-128.  The reference has no kernel of this kind:
// it calls flash-attn for fresh prompts and gathers the context for later portions
// (attn/paged_flash.py:232-279, attn/paged_triton.py:517-557).
#include "attention_decode_mma.cuh"

namespace ems {

constexpr int PF_WARPS = 4;
constexpr int PF_BQ = 64;   // rows per block (16 per warp)
constexpr int PF_BK = 64;   // keys per tile

__device__ __forceinline__ void pf_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void pf_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void pf_ldsm4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pf_ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x of a float32 by the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float pf_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// PAGE16: the page size is a multiple of 16, so every aligned group of 16 keys of a tile
// lies in one page, contiguously: a warp fetches one such group with one block-table lookup.
template <int D, bool PAGE16>
__global__ void __launch_bounds__(PF_WARPS * 32)
prefill_attention_mma_kernel(const DecodeParams p) {
    constexpr int CH = D / 8;                 // 16-byte chunks per row
    constexpr int ROW_BYTES = D * 2;
    constexpr int Q_BYTES = PF_BQ * ROW_BYTES;
    constexpr int KV_BYTES = PF_BK * ROW_BYTES;
    constexpr int KS = D / 16;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t q_s = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t kv_s = q_s + Q_BYTES;      // stage s: K at kv_s + s*2*KV_BYTES, V right after

    const int b = blockIdx.z, hk = blockIdx.y;
    const int G = p.G;
    const int q0 = p.cu_q[b], qlen = p.cu_q[b + 1] - q0, start = p.starts[b];
    const int nrows = qlen * G;
    // Row tiles are handed out last first: under the causal mask the last tile of a prompt has
    // the most keys, and the longest blocks should not be the ones that start last.
    const int r0 = (int)(gridDim.x - 1 - blockIdx.x) * PF_BQ;
    if (r0 >= nrows) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int tok_lo = r0 / G, tok_hi = min(nrows - 1, r0 + PF_BQ - 1) / G;
    const int p_lo = start + tok_lo, p_hi = start + tok_hi;
    const int k_begin = p.window > 0 ? max(0, p_lo - p.window + 1) : 0;
    const int k_end = p_hi + 1;
    const int kt0 = (k_begin / PF_BK) * PF_BK;
    const int ntiles = (k_end - kt0 + PF_BK - 1) / PF_BK;
    const int* table = p.bt + (size_t)b * p.bt_stride;

    // queries of the block -> shared memory (rows past the request are zeros)
    for (int idx = tid; idx < PF_BQ * CH; idx += PF_WARPS * 32) {
        const int row = idx / CH, chunk = idx % CH;
        const int gr = r0 + row;
        const bool valid = gr < nrows;
        const bf16* src = p.q;
        if (valid) src = p.q + (size_t)(q0 + gr / G) * p.q_stride + (size_t)(hk * G + gr % G) * D + chunk * 8;
        pf_cp_async16(q_s + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), src, valid);
    }
    auto issue_tile = [&](int t) {
        const uint32_t kdst = kv_s + (t & 1) * 2 * KV_BYTES, vdst = kdst + KV_BYTES;
        const int kt = kt0 + t * PF_BK;
        if (PAGE16) {
            // warp w fetches keys [kt + 16 w', kt + 16 w' + 16) for w' = w, w + 4, ... : one page each
            constexpr int ROWS_PER_IT = 32 / CH;
            for (int grp = warp; grp < PF_BK / 16; grp += PF_WARPS) {
                const int key0 = kt + grp * 16;
                const bool any = key0 < k_end && key0 + 16 > k_begin;
                size_t base = 0;
                if (any) {
                    const int page = table[key0 / p.page_size];
                    base = (((size_t)page * p.nkv + hk) * p.page_size + key0 % p.page_size) * D;
                }
                const bf16* ksrc = p.kc + base + lane * 8;
                const bf16* vsrc = p.vc + base + lane * 8;
#pragma unroll
                for (int it = 0; it < 16 / ROWS_PER_IT; ++it) {
                    const int row = grp * 16 + it * ROWS_PER_IT + lane / CH, chunk = lane % CH;
                    const int key = kt + row;
                    const bool valid = key >= k_begin && key < k_end;
                    const uint32_t sw = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
                    pf_cp_async16(kdst + sw, valid ? ksrc + it * 256 : p.kc, valid);
                    pf_cp_async16(vdst + sw, valid ? vsrc + it * 256 : p.vc, valid);
                }
            }
            return;
        }
        for (int idx = tid; idx < PF_BK * CH; idx += PF_WARPS * 32) {
            const int row = idx / CH, chunk = idx % CH;
            const int key = kt + row;
            const bool valid = key >= k_begin && key < k_end;
            size_t off = 0;
            if (valid) {
                const int page = table[key / p.page_size];
                off = (((size_t)page * p.nkv + hk) * p.page_size + key % p.page_size) * D + chunk * 8;
            }
            const uint32_t sw = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
            pf_cp_async16(kdst + sw, p.kc + off, valid);
            pf_cp_async16(vdst + sw, p.vc + off, valid);
        }
    };
    issue_tile(0);
    pf_commit();

    // the two rows of this thread inside the warp's 16: lane/4 and lane/4 + 8
    const int gr0 = r0 + warp * 16 + (lane >> 2), gr1 = gr0 + 8;
    const int qpos0 = gr0 < nrows ? start + gr0 / G : -1;   // -1: sees no key
    const int qpos1 = gr1 < nrows ? start + gr1 / G : -1;
    // positions covered by the warp's rows, to skip tiles that none of them can see
    const int wr_lo = r0 + warp * 16, wr_hi = min(nrows - 1, wr_lo + 15);
    const int wpos_lo = wr_lo < nrows ? start + wr_lo / G : -1;
    const int wpos_hi = wr_lo < nrows ? start + wr_hi / G : -1;

    uint32_t qf[KS][4];
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int t = 0; t < ntiles; ++t) {
        if (t + 1 < ntiles) issue_tile(t + 1);
        pf_commit();
        pf_wait<1>();
        __syncthreads();
        if (t == 0) {  // query fragments (the Q copy was in the first group)
            const int mat = lane >> 3, r = lane & 7;
            const int row = warp * 16 + (mat & 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int chunk = ks * 2 + (mat >> 1);
                pf_ldsm4(q_s + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), qf[ks]);
            }
        }
        const int kt = kt0 + t * PF_BK;
        const bool warp_sees = wpos_hi >= kt && (p.window <= 0 || kt + PF_BK - 1 > wpos_lo - p.window);
        if (warp_sees) {
            const uint32_t kst = kv_s + (t & 1) * 2 * KV_BYTES, vst = kst + KV_BYTES;
            float s[PF_BK / 8][4];
#pragma unroll
            for (int n = 0; n < PF_BK / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
            {
                const int mat = lane >> 3, r = lane & 7;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const int chunk = ks * 2 + (mat & 1);
#pragma unroll
                    for (int np = 0; np < PF_BK / 16; ++np) {
                        const int krow = np * 16 + (mat >> 1) * 8 + r;
                        uint32_t bfrag[4];
                        pf_ldsm4(kst + krow * ROW_BYTES + ((chunk ^ (krow & 7)) << 4), bfrag);
                        pf_mma(s[2 * np], qf[ks], bfrag[0], bfrag[1]);
                        pf_mma(s[2 * np + 1], qf[ks], bfrag[2], bfrag[3]);
                    }
                }
            }
            // mask (only tiles that touch the diagonal or the window's edge need one), online
            // softmax in base 2: p = 2^(s * scale_log2 - m), one FMA and one ex2 per score
            const bool full = kt + PF_BK - 1 <= wpos_lo && (p.window <= 0 || kt > wpos_hi - p.window);
            if (!full) {
#pragma unroll
                for (int n = 0; n < PF_BK / 8; ++n)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = kt + n * 8 + (lane & 3) * 2 + e;
                        const bool v0 = key <= qpos0 && (p.window <= 0 || key > qpos0 - p.window);
                        const bool v1 = key <= qpos1 && (p.window <= 0 || key > qpos1 - p.window);
                        if (!v0) s[n][e] = -INFINITY;
                        if (!v1) s[n][2 + e] = -INFINITY;
                    }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < PF_BK / 8; ++n) {
                mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
                mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float sl2 = p.scale_log2;
            const float mn0 = fmaxf(m0, mx0 * sl2), mn1 = fmaxf(m1, mx1 * sl2);
            // a row that has seen no key yet keeps max -inf; subtract 0 instead so that 2^(-inf) = 0
            const float mb0 = mn0 == -INFINITY ? 0.f : mn0, mb1 = mn1 == -INFINITY ? 0.f : mn1;
            const float a0 = pf_ex2(m0 - mb0), a1 = pf_ex2(m1 - mb1);
            m0 = mn0; m1 = mn1;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int n = 0; n < PF_BK / 8; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    s[n][e] = pf_ex2(fmaf(s[n][e], sl2, -mb0));
                    s[n][2 + e] = pf_ex2(fmaf(s[n][2 + e], sl2, -mb1));
                    ps0 += s[n][e];
                    ps1 += s[n][2 + e];
                }
            l0 = l0 * a0 + ps0;
            l1 = l1 * a1 + ps1;
#pragma unroll
            for (int n = 0; n < D / 8; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
            {
                const int mat = lane >> 3, r = lane & 7;
#pragma unroll
                for (int kc = 0; kc < PF_BK / 16; ++kc) {
                    uint32_t pa[4];
                    pa[0] = pf_pack(s[2 * kc][0], s[2 * kc][1]);
                    pa[1] = pf_pack(s[2 * kc][2], s[2 * kc][3]);
                    pa[2] = pf_pack(s[2 * kc + 1][0], s[2 * kc + 1][1]);
                    pa[3] = pf_pack(s[2 * kc + 1][2], s[2 * kc + 1][3]);
                    const int vrow = kc * 16 + (mat & 1) * 8 + r;
#pragma unroll
                    for (int np = 0; np < KS; ++np) {
                        const int chunk = np * 2 + (mat >> 1);
                        uint32_t bfrag[4];
                        pf_ldsm4t(vst + vrow * ROW_BYTES + ((chunk ^ (vrow & 7)) << 4), bfrag);
                        pf_mma(o[2 * np], pa, bfrag[0], bfrag[1]);
                        pf_mma(o[2 * np + 1], pa, bfrag[2], bfrag[3]);
                    }
                }
            }
        }
        __syncthreads();  // the stage is free for the tile after next
    }
    pf_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    const int c = (lane & 3) * 2;
    if (gr0 < nrows) {
        bf16* dst = p.out + ((size_t)(q0 + gr0 / G) * p.nh + hk * G + gr0 % G) * D;
        const float inv = 1.0f / l0;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + c) = __floats2bfloat162_rn(o[n][0] * inv, o[n][1] * inv);
    }
    if (gr1 < nrows) {
        bf16* dst = p.out + ((size_t)(q0 + gr1 / G) * p.nh + hk * G + gr1 % G) * D;
        const float inv = 1.0f / l1;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8 + c) = __floats2bfloat162_rn(o[n][2] * inv, o[n][3] * inv);
    }
}

template <int D, bool PAGE16>
int launch_prefill_mma(const DecodeParams& p, int B, int max_q_len, cudaStream_t stream) {
    constexpr int smem = PF_BQ * D * 2 + 2 * 2 * PF_BK * D * 2;
    auto kernel = prefill_attention_mma_kernel<D, PAGE16>;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    const long long tiles = ((long long)max_q_len * p.G + PF_BQ - 1) / PF_BQ;
    if (tiles > 2147483647LL || p.nkv > 65535 || B > 65535) return EMS_ERR_SHAPE;
    const dim3 grid((unsigned)tiles, (unsigned)p.nkv, (unsigned)B);
    kernel<<<grid, PF_WARPS * 32, smem, stream>>>(p);
    return launch_status();
}

bool prefill_mma_supported(int dtype, int D, long long q_stride, const void* q, const void* out,
                           const void* kc, const void* vc) {
    if (dtype != EMS_BF16 || (D != 64 && D != 128)) return false;
    if ((q_stride * 2) % 16 || ((uintptr_t)q % 16) || ((uintptr_t)out % 4) || ((uintptr_t)kc % 16) ||
        ((uintptr_t)vc % 16))
        return false;
    return true;
}

int run_prefill_mma(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream) {
    if (p.page_size % 16 == 0)
        return D == 64 ? launch_prefill_mma<64, true>(p, B, max_q_len, stream)
                       : launch_prefill_mma<128, true>(p, B, max_q_len, stream);
    return D == 64 ? launch_prefill_mma<64, false>(p, B, max_q_len, stream)
                   : launch_prefill_mma<128, false>(p, B, max_q_len, stream);
}

}  // namespace ems
