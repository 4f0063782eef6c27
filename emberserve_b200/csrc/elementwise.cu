// Row-wise kernels of the decoder: embedding gather, residual add + RMSNorm, SiLU-gate,
// rotary table, and rotary encoding fused with the write of keys and values into the
// paged cache.  All arithmetic is 32-bit; the storage type T is float (the true 32-bit
// path) or bfloat16 (the serving path).
//
// Formulas (reference, by file within emberserve):
//   RMSNorm            model/ops.py:51-55    y = w * cast(x * rsqrt(mean(x^2) + eps))
//   residual + norm    model/ops.py:58-63    residual += x, then RMSNorm(residual)
//   rotary (NeoX)      model/ops.py:66-81    o1 = x1*c - x2*s ; o2 = x2*c + x1*s
//   rotary table       model/rope.py:68-82   angle = pos * inv_freq[i]  (float32)
//   SiLU gate          model/ops.py:84-87    silu(gate) * up
//   cache write        kv/cache.py:54-61     slot = page * page_size + pos % page_size
// The residual stream is kept in 32 bits here (the reference rounds it to the
// activation type after every add); the norm's output is rounded to T before the
// multiplication by the weight, as the reference does.
#include "common.cuh"

namespace ems {

// ---------------------------------------------------------------------------------------
// embedding: residual[n, :] = float(table[tokens[n], :]).  A negative entry -(k + 1) stands for
// deferred[k]: a token that an earlier kernel of the stream has sampled and the host has not
// seen yet (the engine launches a step before it has read the step before it).

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                 const int* __restrict__ deferred, float* __restrict__ residual, int H) {
    pdl_prologue();
    const size_t n = blockIdx.x;
    int tok = tokens[n];
    if (tok < 0) tok = deferred ? deferred[-(tok + 1)] : 0;
    const T* src = table + (size_t)tok * H;
    float* dst = residual + n * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

// ---------------------------------------------------------------------------------------
// residual add + RMSNorm.  One block per output row.  Each thread touches the same
// columns in both passes, so it re-reads only what it wrote itself.

template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ delta, float* residual,
                                   const void* __restrict__ weight, int w_dtype,
                                   T* __restrict__ out, const int* __restrict__ rows, int H,
                                   float eps, int write_residual) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : r;
    float* res = residual + src * H;
    const T* dl = delta ? delta + src * H : nullptr;
    const bool store = dl && write_residual;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = res[i];
        if (dl) s += to_f32<T>(dl[i]);
        if (store) res[i] = s;
        ss += s * s;
    }
    const float total = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)H + eps);
    T* o = out + r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = res[i];
        if (dl && !store) s += to_f32<T>(dl[i]);
        const float y = round_to<T>(s * rstd);
        o[i] = from_f32<T>(y * load_any(weight, w_dtype, i));
    }
}

// The same, four columns per thread held in registers between the two phases (H a multiple
// of 4, at most 4 * VPT * blockDim).  A row of a decode step is then one round trip to
// memory instead of four dependent ones.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<const uint32_t*>(&a);
        t.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};

template <typename T, int VPT>
__global__ void add_rmsnorm_vec_kernel(const T* __restrict__ delta, float* residual,
                                       const void* __restrict__ weight, int w_dtype,
                                       T* __restrict__ out, const int* __restrict__ rows, int H,
                                       float eps, int write_residual) {
    pdl_prologue();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : r;
    float* res = residual + src * H;
    const T* dl = delta ? delta + src * H : nullptr;
    const bool store = dl && write_residual;
    float x[VPT][4];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int col = (v * blockDim.x + threadIdx.x) * 4;
        if (col < H) {
            Vec4<float>::load(res + col, x[v]);
            if (dl) {
                float d[4];
                Vec4<T>::load(dl + col, d);
#pragma unroll
                for (int i = 0; i < 4; ++i) x[v][i] += d[i];
            }
            if (store) Vec4<float>::store(res + col, x[v]);
#pragma unroll
            for (int i = 0; i < 4; ++i) ss += x[v][i] * x[v][i];
        }
    }
    const float total = block_sum(ss, red);
    const float rstd = 1.0f / sqrtf(total / (float)H + eps);
    T* o = out + r * H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int col = (v * blockDim.x + threadIdx.x) * 4;
        if (col < H) {
            float w[4], y[4];
            if (w_dtype == EMS_F32) Vec4<float>::load(reinterpret_cast<const float*>(weight) + col, w);
            else Vec4<bf16>::load(reinterpret_cast<const bf16*>(weight) + col, w);
#pragma unroll
            for (int i = 0; i < 4; ++i) y[i] = round_to<T>(x[v][i] * rstd) * w[i];
            Vec4<T>::store(o + col, y);
        }
    }
}

// ---------------------------------------------------------------------------------------
// out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I) {
    const size_t n = blockIdx.x;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= I) return;
    const float g = to_f32<T>(gate_up[n * 2 * I + i]);
    const float u = to_f32<T>(gate_up[n * 2 * I + I + i]);
    const float act = g / (1.0f + expf(-g));
    out[n * I + i] = from_f32<T>(act * u);
}

// Four columns per thread (I a multiple of 4).
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I) {
    allow_dependent_launch();
    const size_t n = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (i >= I) return;
    float g[4], u[4], y[4];
    Vec4<T>::load(gate_up + n * 2 * I + i, g);
    Vec4<T>::load(gate_up + n * 2 * I + I + i, u);
#pragma unroll
    for (int k = 0; k < 4; ++k) y[k] = g[k] / (1.0f + expf(-g[k])) * u[k];
    Vec4<T>::store(out + n * I + i, y);
}

// ---------------------------------------------------------------------------------------
// table[pos, i, 0] = cos(pos * inv_freq[i]); table[pos, i, 1] = sin(...)

__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ table,
                                  int max_pos, int half) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)max_pos * half) return;
    const int pos = (int)(idx / half), i = (int)(idx % half);
    const float angle = (float)pos * inv_freq[i];
    table[2 * idx] = cosf(angle);
    table[2 * idx + 1] = sinf(angle);
}

// ---------------------------------------------------------------------------------------
// Rotary encoding of q (in place) and k, and the write of k and v into the cache pages.
// qkv row: [q: nh*D | k: nkv*D | v: nkv*D].  Dimension i < rot/2 pairs with i + rot/2;
// dimensions >= rot are copied.  Cache layout: [page, kv_head, slot_in_page, D].

template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int nh, int nkv, int D,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ row_of_token,
                                     const float* __restrict__ table, int rot,
                                     T* __restrict__ kcache, T* __restrict__ vcache,
                                     const int* __restrict__ block_tables, int bt_stride,
                                     int page_size, int write_kv) {
    // blockIdx.y: a q head (< nh), then a k head (< nh + nkv), then a v head
    const size_t n = blockIdx.x;
    const int head = blockIdx.y;
    const int pos = positions[n];
    const int half = rot / 2;
    T* row = qkv + n * (size_t)(nh + 2 * nkv) * D;
    const float* cs = table ? table + (size_t)pos * half * 2 : nullptr;
    if (head < nh) {  // rotate q in place
        T* x = row + (size_t)head * D;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const float x1 = to_f32<T>(x[i]), x2 = to_f32<T>(x[i + half]);
            x[i] = from_f32<T>(x1 * c - x2 * s);
            x[i + half] = from_f32<T>(x2 * c + x1 * s);
        }
        return;
    }
    const int page = block_tables[(size_t)row_of_token[n] * bt_stride + pos / page_size];
    const int slot = pos % page_size;
    if (head < nh + nkv) {  // rotate k into its cache slot
        const int h = head - nh;
        const T* x = row + (size_t)head * D;
        T* dst = kcache + (((size_t)page * nkv + h) * page_size + slot) * D;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float c = cs[2 * i], s = cs[2 * i + 1];
            const float x1 = to_f32<T>(x[i]), x2 = to_f32<T>(x[i + half]);
            dst[i] = from_f32<T>(x1 * c - x2 * s);
            dst[i + half] = from_f32<T>(x2 * c + x1 * s);
        }
        for (int i = rot + threadIdx.x; i < D; i += blockDim.x) dst[i] = x[i];
    } else {  // copy v
        const int h = head - nh - nkv;
        const T* x = row + (size_t)head * D;
        T* dst = vcache + (((size_t)page * nkv + h) * page_size + slot) * D;
        for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = x[i];
    }
}

// The same with four pairs per work item and one block per token (all sizes multiples of 4):
// item = (head, group of 4 consecutive i), heads being q heads, then k heads, then v heads.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int nh, int nkv, int D,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ row_of_token,
                                         const float* __restrict__ table, int rot,
                                         T* __restrict__ kcache, T* __restrict__ vcache,
                                         const int* __restrict__ block_tables, int bt_stride,
                                         int page_size, int write_kv) {
    pdl_prologue();
    const size_t n = blockIdx.x;
    const int pos = positions[n];
    const int half = rot / 2;
    T* row = qkv + n * (size_t)(nh + 2 * nkv) * D;
    const float* cs = table ? table + (size_t)pos * half * 2 : nullptr;
    size_t cache_base = 0;
    if (write_kv) {
        const int page = block_tables[(size_t)row_of_token[n] * bt_stride + pos / page_size];
        cache_base = ((size_t)page * nkv * page_size + pos % page_size) * D;
    }
    const int per_rot = half / 4;            // rotated items per head
    const int per_tail = (D - rot) / 4;      // copied items per k head
    const int per_head = per_rot + per_tail;
    const int rot_heads = write_kv ? nh + nkv : nh;
    const int total = rot_heads * per_head + (write_kv ? nkv * (D / 4) : 0);
    for (int item = threadIdx.x; item < total; item += blockDim.x) {
        if (item < rot_heads * per_head) {
            const int head = item / per_head, j = item % per_head;
            const bool is_q = head < nh;
            T* x = row + (size_t)head * D;
            T* dst = is_q ? x : kcache + cache_base + (size_t)(head - nh) * page_size * D;
            if (j < per_rot) {
                const int i = j * 4;
                float x1[4], x2[4], c4[4], s4[4], o1[4], o2[4];
                Vec4<T>::load(x + i, x1);
                Vec4<T>::load(x + i + half, x2);
                const float4 ca = *reinterpret_cast<const float4*>(cs + 2 * i);
                const float4 cb = *reinterpret_cast<const float4*>(cs + 2 * i + 4);
                c4[0] = ca.x; s4[0] = ca.y; c4[1] = ca.z; s4[1] = ca.w;
                c4[2] = cb.x; s4[2] = cb.y; c4[3] = cb.z; s4[3] = cb.w;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o1[k] = x1[k] * c4[k] - x2[k] * s4[k];
                    o2[k] = x2[k] * c4[k] + x1[k] * s4[k];
                }
                Vec4<T>::store(dst + i, o1);
                Vec4<T>::store(dst + i + half, o2);
            } else if (!is_q) {  // unrotated tail of k; q's tail stays where it is
                const int i = rot + (j - per_rot) * 4;
                float t[4];
                Vec4<T>::load(x + i, t);
                Vec4<T>::store(dst + i, t);
            }
        } else {
            const int j = item - rot_heads * per_head;
            const int h = j / (D / 4), i = (j % (D / 4)) * 4;
            float t[4];
            Vec4<T>::load(row + (size_t)(nh + nkv + h) * D + i, t);
            Vec4<T>::store(vcache + cache_base + (size_t)h * page_size * D + i, t);
        }
    }
}

}  // namespace ems

using namespace ems;

EMS_EXPORT int ems_embedding(const void* table, int dtype, const int* tokens, const int* deferred,
                             float* residual, int N, int H, cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == EMS_F32)
        return launch_pdl(embedding_kernel<float>, dim3(N), dim3(threads), 0, stream, (const float*)table, tokens,
                          deferred, residual, H);
    if (dtype == EMS_BF16)
        return launch_pdl(embedding_kernel<bf16>, dim3(N), dim3(threads), 0, stream, (const bf16*)table, tokens,
                          deferred, residual, H);
    return EMS_ERR_DTYPE;
}

// delta may be null (first layer: the embedding is the residual).  rows may be null (all
// rows, out row r = residual row r) or hold `num_out` residual row indices (compact out).
EMS_EXPORT int ems_add_rmsnorm(const void* delta, float* residual, const void* weight, int w_dtype,
                               void* out, int dtype, const int* rows, int num_out, int H, float eps,
                               int write_residual, cudaStream_t stream) {
    if (num_out <= 0) return EMS_OK;
    if (w_dtype != EMS_F32 && w_dtype != EMS_BF16) return EMS_ERR_DTYPE;
    // The block size is a function of H alone, so a row's sum never depends on the batch.
    if (H % 4 == 0 && H <= 16384 && ((uintptr_t)residual % 16) == 0 && ((uintptr_t)weight % 16) == 0 &&
        ((uintptr_t)out % 16) == 0 && ((uintptr_t)delta % 16) == 0) {
        const int vecs = H / 4;
        const int vpt = (vecs + 1023) / 1024;                       // 1..4
        const int threads = ((vecs + vpt - 1) / vpt + 31) / 32 * 32;  // <= 1024
        int rc = EMS_OK;
#define EMS_NORM_VEC(T, V)                                                                         \
    rc = launch_pdl(add_rmsnorm_vec_kernel<T, V>, dim3(num_out), dim3(threads), 0, stream, (const T*)delta, \
                    residual, weight, w_dtype, (T*)out, rows, H, eps, write_residual)
        if (dtype == EMS_F32) {
            if (vpt == 1) EMS_NORM_VEC(float, 1); else if (vpt == 2) EMS_NORM_VEC(float, 2);
            else if (vpt == 3) EMS_NORM_VEC(float, 3); else EMS_NORM_VEC(float, 4);
        } else if (dtype == EMS_BF16) {
            if (vpt == 1) EMS_NORM_VEC(bf16, 1); else if (vpt == 2) EMS_NORM_VEC(bf16, 2);
            else if (vpt == 3) EMS_NORM_VEC(bf16, 3); else EMS_NORM_VEC(bf16, 4);
        } else {
            return EMS_ERR_DTYPE;
        }
#undef EMS_NORM_VEC
        return rc;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (dtype == EMS_F32)
        add_rmsnorm_kernel<float><<<num_out, threads, 0, stream>>>(
            (const float*)delta, residual, weight, w_dtype, (float*)out, rows, H, eps, write_residual);
    else if (dtype == EMS_BF16)
        add_rmsnorm_kernel<bf16><<<num_out, threads, 0, stream>>>(
            (const bf16*)delta, residual, weight, w_dtype, (bf16*)out, rows, H, eps, write_residual);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_silu_mul(const void* gate_up, void* out, int dtype, int N, int I,
                            cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    const int threads = 256;
    if (I % 4 == 0 && ((uintptr_t)gate_up % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const dim3 vgrid(N, (I / 4 + threads - 1) / threads);
        if (vgrid.y > 65535) return EMS_ERR_SHAPE;
        if (dtype == EMS_F32)
            silu_mul_vec_kernel<float><<<vgrid, threads, 0, stream>>>((const float*)gate_up, (float*)out, I);
        else if (dtype == EMS_BF16)
            silu_mul_vec_kernel<bf16><<<vgrid, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I);
        else
            return EMS_ERR_DTYPE;
        return launch_status();
    }
    const dim3 grid(N, (I + threads - 1) / threads);
    if (grid.y > 65535) return EMS_ERR_SHAPE;
    if (dtype == EMS_F32)
        silu_mul_kernel<float><<<grid, threads, 0, stream>>>((const float*)gate_up, (float*)out, I);
    else if (dtype == EMS_BF16)
        silu_mul_kernel<bf16><<<grid, threads, 0, stream>>>((const bf16*)gate_up, (bf16*)out, I);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}

EMS_EXPORT int ems_rope_table(const float* inv_freq, float* table, int max_pos, int half,
                              cudaStream_t stream) {
    const size_t total = (size_t)max_pos * half;
    if (total == 0) return EMS_OK;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(inv_freq, table, max_pos, half);
    return launch_status();
}

EMS_EXPORT int ems_rope_kv_write(void* qkv, int dtype, int N, int nh, int nkv, int D,
                                 const int* positions, const int* row_of_token, const float* table,
                                 int rotary_dim, void* kcache, void* vcache, const int* block_tables,
                                 int bt_stride, int page_size, int write_kv, cudaStream_t stream) {
    if (N <= 0) return EMS_OK;
    if (rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1)) return EMS_ERR_SHAPE;
    if (rotary_dim > 0 && table == nullptr) return EMS_ERR_SHAPE;
    const int esize = dtype == EMS_F32 ? 4 : 2;
    if (D % 4 == 0 && rotary_dim % 8 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)kcache % 16) == 0 &&
        ((uintptr_t)vcache % 16) == 0 && ((uintptr_t)table % 16) == 0 && (D * esize) % 8 == 0) {
        const int items = (write_kv ? nh + nkv : nh) * (D - rotary_dim / 2) / 4 + (write_kv ? nkv * D / 4 : 0);
        const int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
        if (dtype == EMS_F32)
            return launch_pdl(rope_kv_write_vec_kernel<float>, dim3(N), dim3(threads), 0, stream, (float*)qkv, nh,
                              nkv, D, positions, row_of_token, table, rotary_dim, (float*)kcache, (float*)vcache,
                              block_tables, bt_stride, page_size, write_kv);
        if (dtype == EMS_BF16)
            return launch_pdl(rope_kv_write_vec_kernel<bf16>, dim3(N), dim3(threads), 0, stream, (bf16*)qkv, nh,
                              nkv, D, positions, row_of_token, table, rotary_dim, (bf16*)kcache, (bf16*)vcache,
                              block_tables, bt_stride, page_size, write_kv);
        return EMS_ERR_DTYPE;
    }
    const int heads = write_kv ? nh + 2 * nkv : nh;
    if (heads > 65535) return EMS_ERR_SHAPE;
    const dim3 grid(N, heads);
    const int threads = D >= 128 ? 64 : 32;
    if (dtype == EMS_F32)
        rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>(
            (float*)qkv, nh, nkv, D, positions, row_of_token, table, rotary_dim, (float*)kcache,
            (float*)vcache, block_tables, bt_stride, page_size, write_kv);
    else if (dtype == EMS_BF16)
        rope_kv_write_kernel<bf16><<<grid, threads, 0, stream>>>(
            (bf16*)qkv, nh, nkv, D, positions, row_of_token, table, rotary_dim, (bf16*)kcache,
            (bf16*)vcache, block_tables, bt_stride, page_size, write_kv);
    else
        return EMS_ERR_DTYPE;
    return launch_status();
}
