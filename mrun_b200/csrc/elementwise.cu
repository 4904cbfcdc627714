// Memory-bound kernels of the step: embedding gather, residual-add + RMSNorm, rotation table,
// per-head QK RMSNorm + rotary + key/value write into pages, gated activation.
//
// All arithmetic is 32-bit and each result is rounded once into the activation dtype.  The
// residual stream itself is kept in 32-bit in both precisions.
#include "common.cuh"

using namespace mrun;

// ------------------------------------------------------------------------------------------
// Embedding: out[t, :] = float(table[ids[t], :]).  An id outside [0, vocab) gives a zero row;
// the host checks ids before the step, this only keeps the kernel inside the table.
// Reference call site: crates/mrun-engine/src/load.rs:330-335.
// ------------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, int vocab) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const TW* row = table + (size_t)(ok ? id : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) dst[h] = ok ? to_float(row[h]) : 0.f;
}

MRUN_API int mrun_embed(const void* table, int table_dtype, const int* ids, float* out, int tokens,
                        int hidden, int vocab, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embed: bad sizes tokens=%d hidden=%d vocab=%d",
                 tokens, hidden, vocab);
    if (tokens == 0) return 0;
    if (table_dtype == MRUN_F32)
        embed_kernel<float><<<tokens, 256, 0, stream>>>((const float*)table, ids, out, hidden, vocab);
    else if (table_dtype == MRUN_BF16)
        embed_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, out,
                                                                 hidden, vocab);
    else
        return mrun_set_error("embed: unknown dtype code %d", table_dtype);
    MRUN_CHECK_LAUNCH("embed");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   v = resid[src] + delta[src]   (delta may be null)
//   if rows == null: resid[src] = v            (the stream advances)
//   out[r] = v * rsqrt(mean(v^2) + eps) * weight
// With `rows` the kernel reads row rows[r] and leaves the stream untouched (final norm at the
// wanted positions only).  eps is added to the mean of squares
// (crates/mrun-engine/src/models/gated_delta.rs:11-13 states the form).
// One block of 256 threads per row whatever the batch, so the order of additions is fixed.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                   const float* __restrict__ weight, float eps, TA* __restrict__ out,
                                   const int* __restrict__ rows, int hidden) {
    extern __shared__ float row_buf[];
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    float ss = 0.f;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        float v = resid[src + h];
        if (delta) v += to_float(delta[src + h]);
        row_buf[h] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    TA* dst = out + (size_t)r * hidden;
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const float v = row_buf[h];
        if (!rows && delta) resid[src + h] = v;
        dst[h] = from_float<TA>(v * inv * weight[h]);
    }
}

// The same operation for widths that are a multiple of 8 and at most 8192: every thread keeps up
// to four 8-element chunks in registers and moves them with 16-byte loads and stores, so a row
// takes one pass and the latency of a few independent loads.  One block of 256 threads per row
// whatever the batch: the order of additions depends on the width only.
template <typename TA> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

template <typename TA>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                       const float* __restrict__ weight, float eps, TA* __restrict__ out,
                       const int* __restrict__ rows, int hidden) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const int chunks = hidden >> 3;
    float v[4][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            Vec8<float>::load(resid + src + c * 8, v[i]);
            if (delta) {
                float d[8];
                Vec8<TA>::load(delta + src + c * 8, d);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[i][e] += d[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c < chunks) {
            if (!rows && delta) Vec8<float>::store(resid + src + c * 8, v[i]);
            float w[8], y[8];
            Vec8<float>::load(weight + c * 8, w);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = v[i][e] * inv * w[e];
            Vec8<TA>::store(out + (size_t)r * hidden + c * 8, y);
        }
    }
}

template <typename TA>
static int launch_add_rmsnorm(float* resid, const void* delta, const float* weight, float eps, void* out,
                              const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    const bool aligned = (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
    if (hidden % 8 == 0 && hidden <= 8192 && aligned) {
        MRUN_CHECK_CUDA(launch_kernel(add_rmsnorm_vec_kernel<TA>, dim3(n_rows), dim3(256), 0, stream, resid,
                                   (const TA*)delta, weight, eps, (TA*)out, rows, hidden), "add_rmsnorm");
        return 0;
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 48 * 1024)
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(add_rmsnorm_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem), "add_rmsnorm");
    add_rmsnorm_kernel<TA><<<n_rows, 256, smem, stream>>>(resid, (const TA*)delta, weight, eps, (TA*)out, rows,
                                                          hidden);
    return 0;
}

MRUN_API int mrun_add_rmsnorm(float* resid, const void* delta, const float* weight, float eps, void* out,
                              int act_dtype, const int* rows, int n_rows, int hidden,
                              cudaStream_t stream) {
    MRUN_REQUIRE(n_rows >= 0 && hidden > 0, "add_rmsnorm: bad sizes rows=%d hidden=%d", n_rows, hidden);
    MRUN_REQUIRE((size_t)hidden * sizeof(float) <= 200 * 1024, "add_rmsnorm: hidden=%d exceeds the supported 51200",
                 hidden);
    if (n_rows == 0) return 0;
    int rc;
    if (act_dtype == MRUN_F32)
        rc = launch_add_rmsnorm<float>(resid, delta, weight, eps, out, rows, n_rows, hidden, stream);
    else if (act_dtype == MRUN_BF16)
        rc = launch_add_rmsnorm<__nv_bfloat16>(resid, delta, weight, eps, out, rows, n_rows, hidden, stream);
    else
        return mrun_set_error("add_rmsnorm: unknown dtype code %d", act_dtype);
    if (rc) return rc;
    MRUN_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Rotation table: out[t, j] = (cos a, sin a), a = position[t] * inv_freq[j], the product and the
// functions in 64-bit, rounded once (the reference's explicit form computes the angle in
// 64-bit too, crates/mrun-engine/src/models/common.rs:264-270).  A negative position (padding)
// gives (1, 0).
// ------------------------------------------------------------------------------------------
__global__ void rotary_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                    float2* __restrict__ out, int tokens, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= tokens * half) return;
    const int t = i / half, j = i - t * half;
    const int p = positions[t];
    if (p < 0) {
        out[i] = make_float2(1.f, 0.f);
        return;
    }
    double s, c;
    sincos((double)p * inv_freq[j], &s, &c);
    out[i] = make_float2((float)c, (float)s);
}

MRUN_API int mrun_rotary_table(const int* positions, const double* inv_freq, float* out, int tokens,
                               int half, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && half > 0, "rotary_table: bad sizes tokens=%d half=%d", tokens, half);
    if (tokens == 0) return 0;
    const int n = tokens * half;
    rotary_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(positions, inv_freq, (float2*)out, tokens, half);
    MRUN_CHECK_LAUNCH("rotary_table");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Per-head RMSNorm of q and k, rotation of q and k, write of k and v into pages.
//   qkv: [tokens, (heads + 2 kv_heads) * head_dim], q heads first, then k heads, then v heads.
//   q is normed and rotated in place.  k (normed, rotated) and v (as is) go to
//   cache[page, kv_head, offset, :] with page * page_size + offset = slots[t]; a negative slot
//   skips the write (padding token, or a layer that only reads a cache).
// Order of operations: norm before rotation, v untouched
// (crates/mrun-engine/src/models/common.rs:183,194-198); pairing (j, j + rotary_dim/2)
// (crates/mrun-engine/src/models/common.rs:221,271-280).
// One warp per (token, head); the head's vector is staged in shared memory in 32-bit.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void qk_norm_rope_cache_kernel(TA* __restrict__ qkv, const float* __restrict__ q_weight,
                                          const float* __restrict__ k_weight, float eps,
                                          const float2* __restrict__ rot, int rotary_dim,
                                          const int* __restrict__ slots, TA* __restrict__ k_cache,
                                          TA* __restrict__ v_cache, int tokens, int heads, int kv_heads,
                                          int head_dim, int page_size) {
    extern __shared__ float vec_buf[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_token = heads + 2 * kv_heads;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long)tokens * per_token) return;
    const int t = (int)(item / per_token), slot_head = (int)(item - (long)t * per_token);
    float* vec = vec_buf + warp * head_dim;
    TA* src = qkv + ((size_t)t * per_token + slot_head) * head_dim;

    const bool is_q = slot_head < heads;
    const bool is_k = !is_q && slot_head < heads + kv_heads;
    const int kv_head = is_q ? 0 : (is_k ? slot_head - heads : slot_head - heads - kv_heads);
    const int slot = slots ? slots[t] : -1;
    if (!is_q && slot < 0) return;

    TA* dst;
    if (is_q) {
        dst = src;
    } else {
        const int page = slot / page_size, off = slot - page * page_size;
        TA* cache = is_k ? k_cache : v_cache;
        dst = cache + (((size_t)page * kv_heads + kv_head) * page_size + off) * head_dim;
    }

    if (!is_q && !is_k) {  // v: plain copy
        for (int e = lane; e < head_dim; e += 32) dst[e] = src[e];
        return;
    }

    float ss = 0.f;
    for (int e = lane; e < head_dim; e += 32) {
        const float v = to_float(src[e]);
        vec[e] = v;
        ss += v * v;
    }
    const float* weight = is_q ? q_weight : k_weight;
    if (weight) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)head_dim + eps);
        __syncwarp();
        for (int e = lane; e < head_dim; e += 32) vec[e] = vec[e] * inv * weight[e];
    }
    __syncwarp();
    const int half = rotary_dim >> 1;
    if (rot) {
        const float2* cs = rot + (size_t)t * half;
        for (int j = lane; j < half; j += 32) {
            const float x1 = vec[j], x2 = vec[j + half];
            const float2 c = cs[j];
            dst[j] = from_float<TA>(x1 * c.x - x2 * c.y);
            dst[j + half] = from_float<TA>(x2 * c.x + x1 * c.y);
        }
        for (int e = rotary_dim + lane; e < head_dim; e += 32) dst[e] = from_float<TA>(vec[e]);
    } else {
        for (int e = lane; e < head_dim; e += 32) dst[e] = from_float<TA>(vec[e]);
    }
}

// The same for bfloat16 with a head of 64, 128 or 256 values rotated as a whole (or not at all):
// LANES = head_dim / 8 lanes share a head, eight values (16 bytes) a lane, so a row is read and
// written in whole 16-byte pieces; the sum of squares and the rotation's partner values (the lane
// LANES / 2 further along holds j + head_dim / 2) travel by shuffles.  A group of lanes takes
// QK_HEADS_PER_GROUP consecutive heads of one token, so the token's cosines and sines and the
// norm weights are read once for all of them.  The arithmetic is the scalar kernel's, value by value.
constexpr int QK_HEADS_PER_GROUP = 4;    // the fastest of 2, 4 and 8 heads a lane group on B200

template <int LANES>
__global__ void __launch_bounds__(256, 4)
qk_norm_rope_cache_vec_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_weight,
                              const float* __restrict__ k_weight, float eps, const float2* __restrict__ rot,
                              const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache,
                              __nv_bfloat16* __restrict__ v_cache, int tokens, int heads, int kv_heads,
                              int page_size) {
    constexpr int HEAD_DIM = LANES * 8, HALF = HEAD_DIM / 2;
    const int per_token = heads + 2 * kv_heads;
    const int groups_per_token = (per_token + QK_HEADS_PER_GROUP - 1) / QK_HEADS_PER_GROUP;
    const long group = ((long)blockIdx.x * blockDim.x + threadIdx.x) / LANES;
    const int part = threadIdx.x % LANES;                 // which eight values of a head
    // the lanes of a group leave together, so the shuffles below see all of them
    if (group >= (long)tokens * groups_per_token) return;
    const int t = (int)(group / groups_per_token);
    const int head0 = (int)(group - (long)t * groups_per_token) * QK_HEADS_PER_GROUP;
    const int head1 = min(per_token, head0 + QK_HEADS_PER_GROUP);
    const int slot = slots ? slots[t] : -1;
    const unsigned lane = threadIdx.x & 31;
    const unsigned mask = LANES == 32 ? 0xffffffffu : (((1u << LANES) - 1u) << (lane & ~(unsigned)(LANES - 1)));
    const bool upper = part >= LANES / 2;

    float cs[16];                                          // (cos, sin) of the lane's eight pairs
    if (rot && head0 < heads + kv_heads) {
        const float4* src = reinterpret_cast<const float4*>(rot + (size_t)t * HALF + (part % (LANES / 2)) * 8);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 c = src[i];
            cs[4 * i] = c.x; cs[4 * i + 1] = c.y; cs[4 * i + 2] = c.z; cs[4 * i + 3] = c.w;
        }
    }
    const __nv_bfloat16* row = qkv + (size_t)t * per_token * HEAD_DIM + part * 8;
    uint4 raw[QK_HEADS_PER_GROUP];
#pragma unroll
    for (int i = 0; i < QK_HEADS_PER_GROUP; ++i)
        if (head0 + i < head1) raw[i] = *reinterpret_cast<const uint4*>(row + (size_t)(head0 + i) * HEAD_DIM);

#pragma unroll
    for (int i = 0; i < QK_HEADS_PER_GROUP; ++i) {
        const int head = head0 + i;
        if (head >= head1) break;
        const bool is_q = head < heads;
        const bool is_k = !is_q && head < heads + kv_heads;
        if (!is_q && slot < 0) continue;
        __nv_bfloat16* dst = qkv + ((size_t)t * per_token + head) * HEAD_DIM + part * 8;
        if (!is_q) {
            const int kv_head = is_k ? head - heads : head - heads - kv_heads;
            const int page = slot / page_size, off = slot - page * page_size;
            dst = (is_k ? k_cache : v_cache) + (((size_t)page * kv_heads + kv_head) * page_size + off) * HEAD_DIM + part * 8;
        }
        if (!is_q && !is_k) {                              // v: plain copy
            *reinterpret_cast<uint4*>(dst) = raw[i];
            continue;
        }
        float v[8];
        {
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(pairs[e]);
                v[2 * e] = f.x; v[2 * e + 1] = f.y;
            }
        }
        const float* weight = is_q ? q_weight : k_weight;
        if (weight) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(mask, ss, o);
            const float inv = rsqrtf(ss / (float)HEAD_DIM + eps);
            const float4 w0 = *reinterpret_cast<const float4*>(weight + part * 8);
            const float4 w1 = *reinterpret_cast<const float4*>(weight + part * 8 + 4);
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * inv * w[e];
        }
        if (rot) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float other = __shfl_xor_sync(mask, v[e], LANES / 2);
                // lower half: x1 cos - x2 sin; upper half: x2 cos + x1 sin
                v[e] = upper ? v[e] * cs[2 * e] + other * cs[2 * e + 1] : v[e] * cs[2 * e] - other * cs[2 * e + 1];
            }
        }
        uint4 packed;
        __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) out[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
        *reinterpret_cast<uint4*>(dst) = packed;
    }
}

template <int LANES>
cudaError_t launch_qk_vec(__nv_bfloat16* qkv, const float* q_weight, const float* k_weight, float eps, const float2* rot,
                          const int* slots, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, int tokens, int heads,
                          int kv_heads, int page_size, cudaStream_t stream) {
    const int per_token = heads + 2 * kv_heads;
    const long groups = (long)tokens * ((per_token + QK_HEADS_PER_GROUP - 1) / QK_HEADS_PER_GROUP);
    const long threads = groups * LANES;
    return launch_kernel(qk_norm_rope_cache_vec_kernel<LANES>, dim3((unsigned)((threads + 255) / 256)),
                      dim3(256), 0, stream, qkv, q_weight, k_weight, eps, rot, slots, k_cache, v_cache, tokens, heads,
                      kv_heads, page_size);
}

MRUN_API int mrun_qk_norm_rope_cache(void* qkv, int act_dtype, const float* q_weight, const float* k_weight,
                                     float eps, const float* rot, int rotary_dim, const int* slots,
                                     void* k_cache, void* v_cache, int tokens, int heads, int kv_heads,
                                     int head_dim, int page_size, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && head_dim > 0 && page_size > 0,
                 "qk_norm_rope_cache: bad sizes");
    MRUN_REQUIRE(head_dim <= 1024, "qk_norm_rope_cache: head_dim=%d exceeds the supported 1024", head_dim);
    MRUN_REQUIRE(rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
                 "qk_norm_rope_cache: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim,
                 head_dim);
    MRUN_REQUIRE((q_weight == nullptr) == (k_weight == nullptr),
                 "qk_norm_rope_cache: q and k norm weights come together");
    MRUN_REQUIRE(slots == nullptr || (k_cache && v_cache), "qk_norm_rope_cache: slots without a cache");
    if (tokens == 0) return 0;
    const bool aligned = ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
                         ((uintptr_t)q_weight & 15) == 0 && ((uintptr_t)k_weight & 15) == 0 && ((uintptr_t)rot & 15) == 0;
    if (act_dtype == MRUN_BF16 && aligned && (rot == nullptr || rotary_dim == head_dim) &&
        (head_dim == 64 || head_dim == 128 || head_dim == 256)) {
        __nv_bfloat16* x = (__nv_bfloat16*)qkv;
        __nv_bfloat16 *kc = (__nv_bfloat16*)k_cache, *vc = (__nv_bfloat16*)v_cache;
        const float2* r = (const float2*)rot;
        cudaError_t err = head_dim == 64 ? launch_qk_vec<8>(x, q_weight, k_weight, eps, r, slots, kc, vc, tokens, heads, kv_heads, page_size, stream)
                        : head_dim == 128 ? launch_qk_vec<16>(x, q_weight, k_weight, eps, r, slots, kc, vc, tokens, heads, kv_heads, page_size, stream)
                                          : launch_qk_vec<32>(x, q_weight, k_weight, eps, r, slots, kc, vc, tokens, heads, kv_heads, page_size, stream);
        MRUN_CHECK_CUDA(err, "qk_norm_rope_cache");
        MRUN_CHECK_LAUNCH("qk_norm_rope_cache");
        return 0;
    }
    const int warps = 4;
    const long items = (long)tokens * (heads + 2 * kv_heads);
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    if (act_dtype == MRUN_F32)
        MRUN_CHECK_CUDA(launch_kernel(qk_norm_rope_cache_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream,
                                   (float*)qkv, q_weight, k_weight, eps, (const float2*)rot, rotary_dim, slots,
                                   (float*)k_cache, (float*)v_cache, tokens, heads, kv_heads, head_dim, page_size),
                        "qk_norm_rope_cache");
    else if (act_dtype == MRUN_BF16)
        MRUN_CHECK_CUDA(launch_kernel(qk_norm_rope_cache_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem,
                                   stream, (__nv_bfloat16*)qkv, q_weight, k_weight, eps, (const float2*)rot,
                                   rotary_dim, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tokens, heads,
                                   kv_heads, head_dim, page_size),
                        "qk_norm_rope_cache");
    else
        return mrun_set_error("qk_norm_rope_cache: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("qk_norm_rope_cache");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Gated activation: out[t, i] = act(gate_i) * up_i in 32-bit; act by code: SiLU
// (z * sigmoid(z), crates/mrun-engine/src/models/activations.rs:46-59) or tanh-GELU.
// Layout of gate_up[t, :]: block == 0: all gates, then all ups (gate_i at i, up_i at inter + i).
// block == 8: runs of eight gates followed by the eight ups of the same outputs
// (gate_i at 16 (i / 8) + i % 8, up_i eight further), the row order the decode GEMM's fused
// epilogue wants of the stacked weight.
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gate_up, TA* __restrict__ out, long total, int inter,
                              int block, int act) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long t = i / inter;
    const int c = (int)(i - t * inter);
    const long gi = block ? t * 2 * inter + 2 * (c & ~7) + (c & 7) : t * 2 * inter + c;
    const long ui = block ? gi + 8 : gi + inter;
    const float g = to_float(gate_up[gi]);
    const float u = to_float(gate_up[ui]);
    out[i] = from_float<TA>(mrun::gated_mul<sizeof(TA) == 4>(act, g, u));
}

// Eight outputs per thread with 16-byte loads and stores, for widths that are a multiple of 8.
// One group a thread: with two or four groups in flight per thread the kernel was slower
// (by 10 to 50 per cent at 2,048 x 12,288 outputs).
template <typename TA>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const TA* __restrict__ gate_up, TA* __restrict__ out, long total8, int inter, int block, int act) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total8) return;
    const int per_row = inter >> 3;
    const long t = i / per_row;
    const int c = (int)(i - t * per_row) << 3;
    const TA* g_ptr = gate_up + t * 2 * inter + (block ? 2 * c : c);
    const TA* u_ptr = block ? g_ptr + 8 : g_ptr + inter;
    float g[8], u[8], y[8];
    Vec8<TA>::load(g_ptr, g);
    Vec8<TA>::load(u_ptr, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = mrun::gated_mul<sizeof(TA) == 4>(act, g[e], u[e]);
    Vec8<TA>::store(out + t * inter + c, y);
}

MRUN_API int mrun_swiglu(const void* gate_up, void* out, int act_dtype, int tokens, int inter, int block,
                         int act, cudaStream_t stream) {
    MRUN_REQUIRE_GATE(act, "swiglu");
    MRUN_REQUIRE(tokens >= 0 && inter > 0, "swiglu: bad sizes tokens=%d inter=%d", tokens, inter);
    MRUN_REQUIRE(block == 0 || (block == 8 && inter % 8 == 0),
                 "swiglu: the interleaved layout has runs of 8 and needs inter=%d to be a multiple of 8", inter);
    if (tokens == 0) return 0;
    const long total = (long)tokens * inter;
    const bool aligned = (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0;
    if (inter % 8 == 0 && aligned && (act_dtype == MRUN_F32 || act_dtype == MRUN_BF16)) {
        const long total8 = total / 8;
        const unsigned vblocks = (unsigned)((total8 + 255) / 256);
        if (act_dtype == MRUN_F32)
            swiglu_vec_kernel<float><<<vblocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, total8, inter,
                                                                block, act);
        else
            swiglu_vec_kernel<__nv_bfloat16><<<vblocks, 256, 0, stream>>>(
                (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, total8, inter, block, act);
        MRUN_CHECK_LAUNCH("swiglu");
        return 0;
    }
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_dtype == MRUN_F32)
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, total, inter, block, act);
    else if (act_dtype == MRUN_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                 (__nv_bfloat16*)out, total, inter, block, act);
    else
        return mrun_set_error("swiglu: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("swiglu");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Bias of a linear layer: y[t, n] += bias[n], the sum in 32-bit and rounded once to y's type
// (crates/mrun-engine/src/load.rs:302-305 adds an optional bias after the product).
// ------------------------------------------------------------------------------------------
template <typename TA>
__global__ void add_bias_kernel(TA* __restrict__ y, const float* __restrict__ bias, long total, int n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    y[i] = from_float<TA>(to_float(y[i]) + bias[(int)(i % n)]);
}

MRUN_API int mrun_add_bias(void* y, int act_dtype, const float* bias, int tokens, int n, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && n > 0, "add_bias: bad sizes tokens=%d n=%d", tokens, n);
    if (tokens == 0) return 0;
    const long total = (long)tokens * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_dtype == MRUN_F32)
        add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)y, bias, total, n);
    else if (act_dtype == MRUN_BF16)
        add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)y, bias, total, n);
    else
        return mrun_set_error("add_bias: unknown dtype code %d", act_dtype);
    MRUN_CHECK_LAUNCH("add_bias");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Scatter of 32-bit integers: dst[index[i]] = value[i].  Brings the block tables on the device up
// to date with the pages the host handed out or took back since the last step.
// ------------------------------------------------------------------------------------------
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ index,
                                   const int* __restrict__ value, int n, long dst_size) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long at = index[i];
    if (at >= 0 && at < dst_size) dst[at] = value[i];
}

MRUN_API int mrun_scatter_i32(int* dst, const int* index, const int* value, int n, long dst_size,
                              cudaStream_t stream) {
    MRUN_REQUIRE(n >= 0 && dst_size >= 0, "scatter_i32: bad sizes n=%d dst_size=%ld", n, dst_size);
    if (n == 0) return 0;
    scatter_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(dst, index, value, n, dst_size);
    MRUN_CHECK_LAUNCH("scatter_i32");
    return 0;
}

// ------------------------------------------------------------------------------------------
// Token feedback: ids[r] = previous[source[r]] where source[r] >= 0.  Lets a decode step take the
// tokens the step before it sampled straight from the device, before the host has read them
// (the reference feeds a sampled token before reading it back too,
// crates/mrun-engine/src/nuvec_engine.rs:1489-1500).
// ------------------------------------------------------------------------------------------
__global__ void select_tokens_kernel(int* __restrict__ ids, const int* __restrict__ previous,
                                     const int* __restrict__ source, int rows, int previous_rows) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int s = source[r];
    if (s >= 0 && s < previous_rows) ids[r] = previous[s];
}

MRUN_API int mrun_select_tokens(int* ids, const int* previous, const int* source, int rows, int previous_rows,
                                cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && previous_rows >= 0, "select_tokens: bad sizes rows=%d previous=%d", rows, previous_rows);
    if (rows == 0) return 0;
    select_tokens_kernel<<<(rows + 255) / 256, 256, 0, stream>>>(ids, previous, source, rows, previous_rows);
    MRUN_CHECK_LAUNCH("select_tokens");
    return 0;
}

