// What the mma.sync attention kernels of one head size share: the fragment loads and products,
// the description of raw q, k, v input that the decode kernels norm, rotate and store themselves,
// and the argument checks.  Compiled with -DMRUN_HEAD_DIM=<multiple of 16, at most 256>.
#pragma once

#include "attention_paging.cuh"
#include "common.cuh"

#ifndef MRUN_HEAD_DIM
#error "compile with -DMRUN_HEAD_DIM=<head size>"
#endif

namespace {

constexpr int D = MRUN_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16, at most 256");
constexpr int LD = D + 8;            // smem row stride in elements: odd number of 16-byte chunks
constexpr int BLOCK_N = 64;          // keys per tile
constexpr int THREADS = 128;
constexpr int CHUNKS = D / 8;        // 16-byte chunks per row
constexpr float LOG2E = 1.4426950408889634f;

using bf16 = __nv_bfloat16;

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes become zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// What the decode kernel does itself when the step's q, k and v arrive raw from the projection:
// per-head RMSNorm of q and k, rotation of both, and the write of the token's k and v into its
// page (the same arithmetic, in the same order, as the stand-alone kernel that prefill uses:
// norm, then rotation of pairs (j, j + rotary_dim / 2), v untouched).  `enabled` = 0: q is ready
// and the cache already holds the token.
struct FusedInput {
    int enabled;
    const float* q_weight;   // [D] or null: no norm
    const float* k_weight;
    float eps;
    const float2* rot;       // [tokens, rotary_dim / 2] (cos, sin) or null: no rotation
    int rotary_dim;
    const int* slots;        // [tokens] page * page_size + offset, negative or null: nothing is written
    bf16* k_cache;           // the pages, writable
    bf16* v_cache;
    // Not part of the raw input: when the kernel's tokens are a selection of the step's rows (the
    // single decode tokens of a step that also carries prompt portions), rows[t] is the row of q
    // and of out that token t stands for; null: token t is row t.  Only without raw input.
    const int* rows;
};

// One head vector (D elements at `src`): norm with `weight` (may be null), rotation with the
// token's table row `cs` (may be null), result as bf16 at `dst`.  One warp; `vec` holds D floats.
__device__ __forceinline__ void norm_rotate_head(const bf16* __restrict__ src, const float* __restrict__ weight,
                                                 float eps, const float2* __restrict__ cs, int rotary_dim,
                                                 float* vec, bf16* dst) {
    const int lane = threadIdx.x & 31;
    if constexpr (D % 64 == 0) {
        // Rotation over the whole head (or none): element e = lane + 32 i and its partner
        // e + D / 2 belong to the same lane, so nothing travels through shared memory, and the
        // head, the weight and the table row are requested together: one trip to memory, not three.
        if (cs == nullptr || rotary_dim == D) {
            constexpr int N = D % 64 == 0 ? D / 32 : 2, H = N / 2;      // (sizes that compile for every D)
            float v[N], w[N];
            float2 c[H];
#pragma unroll
            for (int i = 0; i < N; ++i) v[i] = __bfloat162float(src[lane + 32 * i]);
#pragma unroll
            for (int i = 0; i < N; ++i) w[i] = weight ? weight[lane + 32 * i] : 1.f;
#pragma unroll
            for (int i = 0; i < H; ++i) c[i] = cs ? cs[lane + 32 * i] : make_float2(1.f, 0.f);
            if (weight) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < N; ++i) ss += v[i] * v[i];
                ss = mrun::warp_sum(ss);
                const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
                for (int i = 0; i < N; ++i) v[i] = v[i] * inv * w[i];
            }
            if (cs) {
#pragma unroll
                for (int i = 0; i < H; ++i) {
                    const float x1 = v[i], x2 = v[i + H];
                    dst[lane + 32 * i] = __float2bfloat16_rn(x1 * c[i].x - x2 * c[i].y);
                    dst[lane + 32 * i + D / 2] = __float2bfloat16_rn(x2 * c[i].x + x1 * c[i].y);
                }
            } else {
#pragma unroll
                for (int i = 0; i < N; ++i) dst[lane + 32 * i] = __float2bfloat16_rn(v[i]);
            }
            __syncwarp();
            return;
        }
    }
    float ss = 0.f;
    for (int e = lane; e < D; e += 32) {
        const float v = __bfloat162float(src[e]);
        vec[e] = v;
        ss += v * v;
    }
    if (weight) {
        ss = mrun::warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        __syncwarp();
        for (int e = lane; e < D; e += 32) vec[e] = vec[e] * inv * weight[e];
    }
    __syncwarp();
    const int half = rotary_dim >> 1;
    if (cs) {
        for (int j = lane; j < half; j += 32) {
            const float x1 = vec[j], x2 = vec[j + half];
            const float2 c = cs[j];
            dst[j] = __float2bfloat16_rn(x1 * c.x - x2 * c.y);
            dst[j + half] = __float2bfloat16_rn(x2 * c.x + x1 * c.y);
        }
        for (int e = rotary_dim + lane; e < D; e += 32) dst[e] = __float2bfloat16_rn(vec[e]);
    } else {
        for (int e = lane; e < D; e += 32) dst[e] = __float2bfloat16_rn(vec[e]);
    }
    __syncwarp();
}

inline int check_common(const char* name, int heads, int kv_heads, int head_dim, int page_size, int max_blocks,
                 int window, int max_group) {
    MRUN_REQUIRE(head_dim == D, "%s: this library was built for head_dim=%d, got %d", name, D, head_dim);
    MRUN_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                 "%s: heads=%d must be a positive multiple of kv_heads=%d", name, heads, kv_heads);
    MRUN_REQUIRE(heads / kv_heads <= max_group, "%s: %d query heads per kv head exceed the supported %d", name,
                 heads / kv_heads, max_group);
    MRUN_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "%s: bad page_size/max_blocks/window", name);
    MRUN_REQUIRE(kv_heads <= 65535, "%s: kv_heads=%d exceeds 65535", name, kv_heads);
    return 0;
}


}  // namespace
