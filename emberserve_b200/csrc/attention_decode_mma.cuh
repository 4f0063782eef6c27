// Interface of the tensor-core decode attention kernel (attention_decode_mma.cu) towards
// the dispatcher in attention_generic.cu.
#pragma once

#include "common.cuh"

namespace ems {

struct DecodeParams {
    const bf16* q;      // [N, q_stride], first nh*D columns
    bf16* out;          // [N, nh*D]
    const bf16* kc;     // [pages, nkv, page_size, D]
    const bf16* vc;
    const int* bt;      // [B, bt_stride]
    const int* cu_q;    // [B+1] packed token index of each row (rows have one token)
    const int* starts;  // [B] keys cached before this step; the query stands at that position
    float* part_o;      // [N*nh, splits, D]
    float* part_ml;     // [N*nh, splits, 2]  (max in natural-log units, sum)
    long long q_stride;
    int bt_stride, page_size, nh, nkv, G, window, splits;
    float scale_log2;   // log2(e) / sqrt(D)
    // The fused decode form (attention_decode_mma.cu): `q` is the raw qkv row [q | k | v]; the
    // kernel rotates q (and k) itself with `rope_table` [positions, rot / 2, (cos, sin)] and, with
    // write_kv, puts the row's new key and value into the cache (and into its own tile of them).
    const float* rope_table = nullptr;
    int rot = 0;        // 0 (no rotation) or D
    int fused = 0;
    int write_kv = 0;
};

bool decode_mma_supported(int dtype, int D, int G, long long q_stride, const void* q, const void* kc,
                          const void* vc);
int run_decode_mma(const DecodeParams& p, int B, int D, cudaStream_t stream);
bool decode_fused_supported(int D, int G, int rot, long long q_stride, const void* q, const void* kc,
                            const void* vc);

// The tensor-core kernel for prompt portions and mixed rows (attention_prefill_mma.cu);
// it uses the same parameter block (no split of the keys: part_o / part_ml unused).
bool prefill_mma_supported(int dtype, int D, long long q_stride, const void* q, const void* out,
                           const void* kc, const void* vc);
int run_prefill_mma(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream);

// The tcgen05 kernel for prompt portions (attention_prefill_tc05.cu): long prompts at head
// sizes 64 and 128 with pages of a multiple of 16 keys; same parameter block.
bool prefill_tc05_supported(int dtype, int D, int page_size, long long q_stride, const void* q, const void* out,
                            const void* kc, const void* vc);
int run_prefill_tc05(const DecodeParams& p, int B, int D, int max_q_len, cudaStream_t stream);

}  // namespace ems
