// Paged grouped-query attention on CUDA cores in 32-bit arithmetic, for any head size.
//
// This is the attention of the whole-model 32-bit path, and the kernel that takes the shapes the
// tensor-core kernels refuse.  One block per (token, query head).  A token at position p of its
// request sees keys lo..p, lo = 0 or p - window + 1, read from the request's pages; the keys of
// the tokens in this step are already in the pages when it runs.  Scores, softmax and the
// weighted sum are 32-bit; keys are consumed in tiles of 128 in position order, so the result of
// a token depends on its own keys only, not on the batch around it.
//
// Math: s = scale * q·k, p = softmax(s), o = p·v; query head h reads kv head h / (heads/kv_heads)
// (crates/mrun-engine/src/models/common.rs:129,199-205; causal alignment to the end of the keys,
// crates/mrun-engine/src/tensor/nuvec.rs:866-872).
#include "common.cuh"

using namespace mrun;

namespace {

constexpr int THREADS = 128;

template <typename TA>
__global__ void __launch_bounds__(THREADS)
paged_attention_generic_kernel(const TA* __restrict__ q, long q_stride, TA* __restrict__ out,
                               const TA* __restrict__ k_cache, const TA* __restrict__ v_cache,
                               const int* __restrict__ block_tables, int max_blocks,
                               const int* __restrict__ token_slot, const int* __restrict__ positions,
                               int heads, int kv_heads, int head_dim, int page_size, float scale,
                               int window) {
    extern __shared__ float smem[];
    float* qs = smem;                 // head_dim
    float* probs = qs + head_dim;     // THREADS
    int* rows = (int*)(probs + THREADS);  // THREADS: element offset / head_dim of each key's row
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int pos = positions[t];
    TA* dst = out + ((size_t)t * heads + h) * head_dim;
    if (pos < 0) {  // padding token
        for (int d = tid; d < head_dim; d += THREADS) dst[d] = from_float<TA>(0.f);
        return;
    }
    const int kvh = h / (heads / kv_heads);
    const int* table = block_tables + (size_t)token_slot[t] * max_blocks;
    const TA* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
    for (int d = tid; d < head_dim; d += THREADS) qs[d] = to_float(qrow[d]);
    __syncthreads();

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float m = -INFINITY, l = 0.f;
    float acc[8];  // head_dim <= 8 * THREADS = 1024
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

    for (int tile0 = lo; tile0 <= pos; tile0 += THREADS) {
        const int key = tile0 + tid;
        const bool valid = key <= pos;
        float s = -INFINITY;
        if (valid) {
            const int page = table[key / page_size];
            const long row = ((long)page * kv_heads + kvh) * page_size + key % page_size;
            rows[tid] = (int)row;
            const TA* kr = k_cache + row * head_dim;
            float dot = 0.f;
            for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
            s = dot * scale;
        }
        const float tile_max = block_max(s, scratch);
        const float m_new = fmaxf(m, tile_max);
        const float p = valid ? expf(s - m_new) : 0.f;
        probs[tid] = p;
        const float tile_sum = block_sum(p, scratch);  // has a __syncthreads after the probs store
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + tile_sum;
        m = m_new;
        const int n = min(THREADS, pos - tile0 + 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = tid + i * THREADS;
            if (d < head_dim) {
                float a = acc[i] * corr;
                for (int j = 0; j < n; ++j)
                    a = fmaf(probs[j], to_float(v_cache[(long)rows[j] * head_dim + d]), a);
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int d = tid + i * THREADS;
        if (d < head_dim) dst[d] = from_float<TA>(acc[i] * inv);
    }
}

}  // namespace

// q: row t starts at q + t * q_stride, heads contiguous [heads, head_dim].
// out: dense [tokens, heads * head_dim].  caches: [pages, kv_heads, page_size, head_dim].
// block_tables: [slots, max_blocks], one row per state slot; token_slot[t] picks the row; positions[t] < 0 = padding.
MRUN_API int mrun_paged_attention_generic(const void* q, long q_stride, void* out, const void* k_cache,
                                          const void* v_cache, int act_dtype, const int* block_tables,
                                          int max_blocks, const int* token_slot, const int* positions,
                                          int tokens, int heads, int kv_heads, int head_dim,
                                          int page_size, long cache_rows, float scale, int window,
                                          cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && page_size > 0 && max_blocks > 0,
                 "paged_attention_generic: bad sizes");
    MRUN_REQUIRE(heads % kv_heads == 0, "paged_attention_generic: heads=%d is not a multiple of kv_heads=%d",
                 heads, kv_heads);
    MRUN_REQUIRE(head_dim <= 8 * THREADS, "paged_attention_generic: head_dim=%d exceeds the supported %d",
                 head_dim, 8 * THREADS);
    MRUN_REQUIRE(heads <= 65535, "paged_attention_generic: heads=%d exceeds 65535", heads);
    MRUN_REQUIRE(cache_rows < (1L << 31), "paged_attention_generic: the cache has %ld rows, the limit is 2^31",
                 cache_rows);
    MRUN_REQUIRE(window >= 0, "paged_attention_generic: window=%d is negative", window);
    if (tokens == 0) return 0;
    const dim3 grid(tokens, heads);
    const size_t smem = (size_t)(head_dim + 2 * THREADS) * sizeof(float);
    if (act_dtype == MRUN_F32)
        paged_attention_generic_kernel<float><<<grid, THREADS, smem, stream>>>(
            (const float*)q, q_stride, (float*)out, (const float*)k_cache, (const float*)v_cache,
            block_tables, max_blocks, token_slot, positions, heads, kv_heads, head_dim, page_size, scale,
            window);
    else if (act_dtype == MRUN_BF16)
        paged_attention_generic_kernel<__nv_bfloat16><<<grid, THREADS, smem, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)k_cache,
            (const __nv_bfloat16*)v_cache, block_tables, max_blocks, token_slot, positions, heads, kv_heads,
            head_dim, page_size, scale, window);
    else
        return mrun_set_error("paged_attention_generic: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("paged_attention_generic");
    return 0;
}
