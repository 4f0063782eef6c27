// Paged grouped-query attention for decode rows (one query token per request) in
// bfloat16 on the tensor cores, split over the keys.
//
// A decode step reads every cached key and value once and does little arithmetic with
// them (2 * G * D multiply-adds per key for G query heads per KV head), so the kernel is
// built around the memory system: a block is four warps that never synchronise with each
// other until the very end; each warp owns every fourth 16-key tile of the block's key
// range and streams it through a private three-stage cp.async ring in shared memory
// (16 keys x D bf16 of K and of V per stage: one 4 KB page each at page size 16, D 128),
// so that many kilobytes per SM are always in flight.  The G query heads of the group are
// the rows of one m16 tile: S = Q K^T and O += P V are mma.sync m16n8k16 bf16 products
// with float32 accumulators; softmax is float32 (base-2 exponentials of scores scaled by
// log2(e) / sqrt(D)).  At the end the four warps' partial (max, sum, O) are merged in
// shared memory and written out, or handed to the merge kernel when the keys of a
// request are split over several blocks.  (Letting the block that finishes last merge the
// splits was tried and dropped: one block reading every partial costs as much at the end of
// the kernel as the merge kernel does behind it.)
//
// The kernel is launched as a programmatic dependent of the kernel before it: the tiles of keys
// that earlier steps cached (all but the tile that holds the row's new key) are requested
// before it waits for that kernel.  In the fused form that kernel is the qkv projection: the
// block rotates q itself, and the warp that owns the last tile rotates the new key, writes it
// and the new value into the cache and into its tile.
//
// Formulas: emberserve/attn/paged_torch.py:87-98 (decode form of base.py:105-128);
// the reference's own kernel of this kind is attn/paged_triton.py:100-183 (split-K
// partials merged by :185-208).
#include "attention_decode_mma.cuh"

namespace ems {

constexpr int DEC_WARPS_MIN = 4;
constexpr int DEC_STAGES_MIN = 3;  // tiles in flight per warp
constexpr int DEC_TK = 16;  // keys per warp tile

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x of a float32 by the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// PAGE16: the page size is a multiple of 16, so the 16 keys of a tile (tiles are aligned to
// multiples of 16 in absolute position) lie in one page, contiguously: one block-table
// lookup per tile instead of one per key row.
template <int D, bool PAGE16, int DEC_STAGES, int DEC_WARPS>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_mma_kernel(const DecodeParams p) {
    asm volatile("griddepcontrol.launch_dependents;" ::);
    constexpr int CH = D / 8;                  // 16-byte chunks per key row
    constexpr int ROW_BYTES = D * 2;
    constexpr int TILE_BYTES = DEC_TK * ROW_BYTES;           // K (or V) of one 16-key tile
    constexpr int WARP_BYTES = DEC_STAGES * 2 * TILE_BYTES;  // the warp's ring: K and V per stage
    constexpr int KS = D / 16;                 // k-steps of Q.K^T, and pairs of d-tiles of P.V
    extern __shared__ __align__(128) unsigned char smem_raw[];

    const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok = p.cu_q[b];
    const int ctx = p.starts[b] + 1;           // keys visible to the query: [k_begin, ctx)
    const int k_begin = p.window > 0 ? max(0, ctx - p.window) : 0;
    const int G = p.G;

    // this block's tiles (16 keys each, aligned to absolute positions), and this warp's
    const int tile_lo = k_begin / DEC_TK, tile_hi = (ctx - 1) / DEC_TK;  // inclusive
    const int ntiles = tile_hi - tile_lo + 1;
    const int per_split = (ntiles + p.splits - 1) / p.splits;
    const int t_begin = tile_lo + split * per_split;
    const int t_end = min(tile_hi + 1, t_begin + per_split);
    const int my_first = t_begin + warp;
    const int my_count = my_first < t_end ? (t_end - my_first + DEC_WARPS - 1) / DEC_WARPS : 0;

    unsigned char* ring = smem_raw + warp * WARP_BYTES;
    const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
    const int* table = p.bt + (size_t)b * p.bt_stride;
    // fused form with a write: the row's own key is not in the cache yet; its row of the last
    // tile is filled with zeros by the copy and patched once the tile has landed
    const int new_key = (p.fused && p.write_kv) ? ctx - 1 : -1;

    auto issue_tile = [&](int i) {  // stream the warp's i-th tile into stage i % DEC_STAGES
        const int tile = my_first + i * DEC_WARPS;
        const uint32_t kdst = ring_addr + (i % DEC_STAGES) * 2 * TILE_BYTES;
        const uint32_t vdst = kdst + TILE_BYTES;
        constexpr int ROWS_PER_IT = 32 / CH;
        if (PAGE16) {
            const int key0 = tile * DEC_TK;
            const int page = table[key0 / p.page_size];
            const size_t base = (((size_t)page * p.nkv + hk) * p.page_size + key0 % p.page_size) * D;
            const bf16* ksrc = p.kc + base + lane * 8;   // the tile is 16 * D contiguous elements
            const bf16* vsrc = p.vc + base + lane * 8;
#pragma unroll
            for (int it = 0; it < DEC_TK / ROWS_PER_IT; ++it) {
                const int row = it * ROWS_PER_IT + lane / CH, chunk = lane % CH;
                const int key = key0 + row;
                const bool valid = key >= k_begin && key < ctx && key != new_key;
                const uint32_t sw = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
                cp_async16(kdst + sw, valid ? ksrc + it * 256 : p.kc, valid);
                cp_async16(vdst + sw, valid ? vsrc + it * 256 : p.vc, valid);
            }
            return;
        }
#pragma unroll
        for (int it = 0; it < DEC_TK / ROWS_PER_IT; ++it) {
            const int row = it * ROWS_PER_IT + lane / CH, chunk = lane % CH;
            const int key = tile * DEC_TK + row;
            const bool valid = key >= k_begin && key < ctx && key != new_key;
            size_t off = 0;
            if (valid) {
                const int page = table[key / p.page_size];
                off = (((size_t)page * p.nkv + hk) * p.page_size + key % p.page_size) * D + chunk * 8;
            }
            const uint32_t sw = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
            cp_async16(kdst + sw, p.kc + off, valid);
            cp_async16(vdst + sw, p.vc + off, valid);
        }
    };

    // Tiles of keys that were cached by earlier steps do not depend on the kernel before this
    // one: request them first.  The tile that holds the row's own key (the last one) waits.
    int issued = 0;
#pragma unroll
    for (int s = 0; s < DEC_STAGES; ++s) {
        if (s < my_count && my_first + s * DEC_WARPS == tile_hi) break;
        if (s < my_count) issue_tile(s);
        cp_async_commit();
        ++issued;
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // query fragments: rows of the m16 tile are the G heads of the group (rows >= G are zero)
    uint32_t qf[KS][4];
    {
        const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
        const bf16* qrow = p.q + (size_t)tok * p.q_stride + (size_t)hk * G * D;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int col = ks * 16 + c;
            qf[ks][0] = r0 < G ? *reinterpret_cast<const uint32_t*>(qrow + r0 * D + col) : 0u;
            qf[ks][1] = r1 < G ? *reinterpret_cast<const uint32_t*>(qrow + r1 * D + col) : 0u;
            qf[ks][2] = r0 < G ? *reinterpret_cast<const uint32_t*>(qrow + r0 * D + col + 8) : 0u;
            qf[ks][3] = r1 < G ? *reinterpret_cast<const uint32_t*>(qrow + r1 * D + col + 8) : 0u;
        }
        if (p.fused && p.rot == D) {
            // rotate-half over the whole head: column j < D/2 pairs with j + D/2, which this thread
            // holds in the fragment KS/2 steps on (emberserve/model/ops.py:66-81); the same
            // expressions as the rotary kernel of the unfused path
            const float* cs = p.rope_table + (size_t)(ctx - 1) * (D / 2) * 2;
#pragma unroll
            for (int ks = 0; ks < KS / 2; ++ks)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = ks * 16 + c + (e >> 1) * 8;  // column of the low element of the pair
                    const float2 cs0 = *reinterpret_cast<const float2*>(cs + 2 * j);
                    const float2 cs1 = *reinterpret_cast<const float2*>(cs + 2 * (j + 1));
                    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&qf[ks][e]);
                    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&qf[ks + KS / 2][e]);
                    const float a0 = __bfloat162float(lo.x), a1 = __bfloat162float(lo.y);
                    const float b0 = __bfloat162float(hi.x), b1 = __bfloat162float(hi.y);
                    __nv_bfloat162 nlo, nhi;
                    nlo.x = __float2bfloat16_rn(a0 * cs0.x - b0 * cs0.y);
                    nhi.x = __float2bfloat16_rn(b0 * cs0.x + a0 * cs0.y);
                    nlo.y = __float2bfloat16_rn(a1 * cs1.x - b1 * cs1.y);
                    nhi.y = __float2bfloat16_rn(b1 * cs1.x + a1 * cs1.y);
                    qf[ks][e] = *reinterpret_cast<const uint32_t*>(&nlo);
                    qf[ks + KS / 2][e] = *reinterpret_cast<const uint32_t*>(&nhi);
                }
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // rows lane/4 and lane/4 + 8

    for (int s = issued; s < DEC_STAGES; ++s) {
        if (s < my_count) issue_tile(s);
        cp_async_commit();
    }

    for (int i = 0; i < my_count; ++i) {
        cp_async_wait<DEC_STAGES - 1>();
        __syncwarp();
        const uint32_t kst = ring_addr + (i % DEC_STAGES) * 2 * TILE_BYTES;
        const uint32_t vst = kst + TILE_BYTES;
        const int key0 = (my_first + i * DEC_WARPS) * DEC_TK;
        if (new_key >= 0 && my_first + i * DEC_WARPS == tile_hi) {
            // the row's own key and value: from the qkv row into the cache and into this tile
            const int row = new_key - key0;
            const bf16* kraw = p.q + (size_t)tok * p.q_stride + (size_t)(p.nh + hk) * D;
            const bf16* vraw = kraw + (size_t)p.nkv * D;
            const int page = table[new_key / p.page_size];
            const size_t off = (((size_t)page * p.nkv + hk) * p.page_size + new_key % p.page_size) * D;
            bf16* kdst = const_cast<bf16*>(p.kc) + off;
            bf16* vdst = const_cast<bf16*>(p.vc) + off;
            unsigned char* ktile = ring + (i % DEC_STAGES) * 2 * TILE_BYTES;
            unsigned char* vtile = ktile + TILE_BYTES;
            auto put = [&](unsigned char* tile, int col, bf16 v) {
                *reinterpret_cast<bf16*>(tile + row * ROW_BYTES + (((col >> 3) ^ (row & 7)) << 4) + (col & 7) * 2) = v;
            };
            if (p.rot == D) {
                const float* cs = p.rope_table + (size_t)new_key * (D / 2) * 2;
                for (int j = lane; j < D / 2; j += 32) {
                    const float c = cs[2 * j], sn = cs[2 * j + 1];
                    const float x1 = __bfloat162float(kraw[j]), x2 = __bfloat162float(kraw[j + D / 2]);
                    const bf16 o1 = __float2bfloat16_rn(x1 * c - x2 * sn), o2 = __float2bfloat16_rn(x2 * c + x1 * sn);
                    kdst[j] = o1;
                    kdst[j + D / 2] = o2;
                    put(ktile, j, o1);
                    put(ktile, j + D / 2, o2);
                }
            } else {
                for (int j = lane; j < D; j += 32) {
                    kdst[j] = kraw[j];
                    put(ktile, j, kraw[j]);
                }
            }
            for (int j = lane; j < D; j += 32) {
                vdst[j] = vraw[j];
                put(vtile, j, vraw[j]);
            }
            __syncwarp();
        }

        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        {
            const int mat = lane >> 3, r = lane & 7;
            const int krow = (mat >> 1) * 8 + r;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int chunk = ks * 2 + (mat & 1);
                uint32_t bfrag[4];
                ldmatrix_x4(kst + krow * ROW_BYTES + ((chunk ^ (krow & 7)) << 4), bfrag);
                mma_bf16_16816(s[0], qf[ks], bfrag[0], bfrag[1]);
                mma_bf16_16816(s[1], qf[ks], bfrag[2], bfrag[3]);
            }
        }
        // softmax of the tile, rows r0 (values [n][0..1]) and r1 (values [n][2..3]), in base 2:
        // p = 2^(s * scale_log2 - m), one FMA and one ex2 per score
        if (key0 < k_begin || key0 + DEC_TK > ctx) {  // only the first and the last tile need a mask
#pragma unroll
            for (int n = 0; n < 2; ++n)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + n * 8 + (lane & 3) * 2 + e;
                    if (key < k_begin || key >= ctx) { s[n][e] = -INFINITY; s[n][2 + e] = -INFINITY; }
                }
        }
        float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float sl2 = p.scale_log2;
        const float mn0 = fmaxf(m0, mx0 * sl2), mn1 = fmaxf(m1, mx1 * sl2);
        const float mb0 = mn0 == -INFINITY ? 0.f : mn0, mb1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = ex2_approx(m0 - mb0), a1 = ex2_approx(m1 - mb1);
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[n][e] = ex2_approx(fmaf(s[n][e], sl2, -mb0));
                s[n][2 + e] = ex2_approx(fmaf(s[n][2 + e], sl2, -mb1));
                ps0 += s[n][e];
                ps1 += s[n][2 + e];
            }
        l0 = l0 * a0 + ps0;  // per-thread share of the row sum; the quad is summed at the end
        l1 = l1 * a1 + ps1;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
        {
            const int mat = lane >> 3, r = lane & 7;
            const int vrow = (mat & 1) * 8 + r;
#pragma unroll
            for (int np = 0; np < KS; ++np) {
                const int chunk = np * 2 + (mat >> 1);
                uint32_t bfrag[4];
                ldmatrix_x4_trans(vst + vrow * ROW_BYTES + ((chunk ^ (vrow & 7)) << 4), bfrag);
                mma_bf16_16816(o[2 * np], pa, bfrag[0], bfrag[1]);
                mma_bf16_16816(o[2 * np + 1], pa, bfrag[2], bfrag[3]);
            }
        }
        __syncwarp();  // every lane is done with the stage before it is refilled
        if (i + DEC_STAGES < my_count) issue_tile(i + DEC_STAGES);
        cp_async_commit();
    }
    cp_async_wait<0>();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    __syncwarp();

    // the warp's partial result into its own (now idle) ring: m[16], l[16], o[16][D]
    float* wm = reinterpret_cast<float*>(ring);
    float* wl = wm + 16;
    float* wo = wl + 16;
    {
        const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
        if ((lane & 3) == 0) { wm[r0] = m0; wm[r1] = m1; wl[r0] = l0; wl[r1] = l1; }
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            wo[r0 * D + n * 8 + c] = o[n][0];
            wo[r0 * D + n * 8 + c + 1] = o[n][1];
            wo[r1 * D + n * 8 + c] = o[n][2];
            wo[r1 * D + n * 8 + c + 1] = o[n][3];
        }
    }
    __syncthreads();

    for (int idx = threadIdx.x; idx < G * D; idx += DEC_WARPS * 32) {
        const int g = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w)
            M = fmaxf(M, reinterpret_cast<const float*>(smem_raw + w * WARP_BYTES)[g]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* base = reinterpret_cast<const float*>(smem_raw + w * WARP_BYTES);
            const float mw = base[g];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += base[16 + g] * f;
            acc += base[32 + g * D + d] * f;
        }
        const size_t prow = (size_t)tok * p.nh + (size_t)hk * G + g;
        if (p.splits == 1) {
            p.out[prow * D + d] = __float2bfloat16_rn(acc / L);
        } else {
            p.part_o[(prow * p.splits + split) * D + d] = acc;
            if (d == 0) {
                p.part_ml[(prow * p.splits + split) * 2] = M * 0.69314718055994531f;  // to natural-log units
                p.part_ml[(prow * p.splits + split) * 2 + 1] = L;
            }
        }
    }
}

template <int D, bool PAGE16, int STAGES, int WARPS>
int launch_decode_mma_staged(const DecodeParams& p, int B, cudaStream_t stream, int device) {
    constexpr int smem = WARPS * STAGES * 2 * DEC_TK * D * 2;
    auto kernel = decode_attention_mma_kernel<D, PAGE16, STAGES, WARPS>;
    // (dynamic + the kernel's few static bytes pass the 48 KB default at D = 64); once per device
    static int raised_on = -1;
    if (raised_on != device) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return EMS_ERR_LAUNCH;
        raised_on = device;
    }
    const dim3 grid((unsigned)p.splits, (unsigned)p.nkv, (unsigned)B);
    return launch_pdl(kernel, grid, dim3(WARPS * 32), smem, stream, p);
}

template <int D, bool PAGE16>
int launch_decode_mma(const DecodeParams& p, int B, cudaStream_t stream) {
    static int sms_of[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return EMS_ERR_LAUNCH;
    if (sms_of[device] == 0 &&
        cudaDeviceGetAttribute(&sms_of[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return EMS_ERR_LAUNCH;
    if (p.nkv > 65535 || B > 65535) return EMS_ERR_SHAPE;
    // Four warps with rings of three tiles are 48 KB at head size 64: four blocks per SM.  While all
    // blocks of the step are resident at once at TWO per SM, eight warps per block are faster (a
    // request's keys are walked by twice the warps, so the longest request of the step ends sooner):
    // 128 rows x 2 KV heads with contexts spread over 64..1536 take 17.8 us against 20.6 (four warps
    // with six tiles in flight each, the same shared memory), with contexts of 1536 21.3 against
    // 23.3; with more blocks than that the small blocks win (256 rows, 1024 keys: 26 us against 34).
    if constexpr (D == 64) {
        if ((long long)p.splits * p.nkv * B <= 2LL * sms_of[device])
            return launch_decode_mma_staged<D, PAGE16, DEC_STAGES_MIN, 2 * DEC_WARPS_MIN>(p, B, stream, device);
    }
    return launch_decode_mma_staged<D, PAGE16, DEC_STAGES_MIN, DEC_WARPS_MIN>(p, B, stream, device);
}

// Whether the tensor-core decode kernel takes this case; otherwise the generic kernel runs.
bool decode_mma_supported(int dtype, int D, int G, long long q_stride, const void* q, const void* kc,
                          const void* vc) {
    if (dtype != EMS_BF16 || (D != 64 && D != 128) || G > 16) return false;
    if ((q_stride * 2) % 4 || ((uintptr_t)q % 4) || ((uintptr_t)kc % 16) || ((uintptr_t)vc % 16)) return false;
    return true;
}

bool decode_fused_supported(int D, int G, int rot, long long q_stride, const void* q, const void* kc,
                            const void* vc) {
    return decode_mma_supported(EMS_BF16, D, G, q_stride, q, kc, vc) && (rot == 0 || rot == D);
}

int run_decode_mma(const DecodeParams& p, int B, int D, cudaStream_t stream) {
    if (p.page_size % 16 == 0)
        return D == 64 ? launch_decode_mma<64, true>(p, B, stream) : launch_decode_mma<128, true>(p, B, stream);
    return D == 64 ? launch_decode_mma<64, false>(p, B, stream) : launch_decode_mma<128, false>(p, B, stream);
}

}  // namespace ems
