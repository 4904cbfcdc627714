// Next-token choice from 32-bit logits, one block per row: greedy argmax, or temperature sampling
// after the top-p, min-p and top-k filters, plus the repetition penalty that runs before them.
//
// Order of operations follows crates/mrun-engine/src/sample.rs:88-132: penalty on the raw
// logits; log-probabilities; greedy = argmax; otherwise top-p, then min-p, then top-k, each
// setting what it drops to -inf; then a categorical draw from lp / temperature.
//
// The categorical draw (not in the reference's own source) is a Gumbel-max draw:
//   token = argmax_i ( logit_i / T + g_i ),  g_i = -log(-log(u_i)),
//   u_i   = ((mix(key + i) >> 40) + 0.5) * 2^-24,   mix = SplitMix64's finaliser,
// with the logarithms in 64-bit, so that a plain host implementation draws the same token.
// The three filters reduce to one threshold on the log-probability: a token is kept when it is
// kept by each, and each keeps an upper set.
//   top-p keeps i  <=>  mass of tokens strictly more likely than i  <  p * total mass
//   min-p keeps i  <=>  lp_i >= max lp + log(min_p)
//   top-k keeps i  <=>  fewer than k tokens are strictly more likely than i
// (ties are all kept).  The first and third thresholds are found by bisection over the ordered
// bit patterns of the row's values, 32 counting passes each.
#include "common.cuh"

using namespace mrun;

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Monotone map float -> unsigned: a < b  <=>  key(a) < key(b)  (no NaNs).
__device__ __forceinline__ unsigned ordered_key(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_key(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct ArgMax {
    float value;
    int index;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
    return a;
}
__device__ ArgMax block_argmax(ArgMax v, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax other;
        other.value = __shfl_xor_sync(0xffffffffu, v.value, o);
        other.index = __shfl_xor_sync(0xffffffffu, v.index, o);
        v = better(v, other);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = scratch[lane];  // THREADS / 32 == 32 warps
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax other;
            other.value = __shfl_xor_sync(0xffffffffu, t.value, o);
            other.index = __shfl_xor_sync(0xffffffffu, t.index, o);
            t = better(t, other);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const int* __restrict__ top_k,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ keys,
              int* __restrict__ out) {
    __shared__ float scratch[33];
    __shared__ ArgMax arg_scratch[33];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * vocab;
    const float temp = temperature ? temperature[row] : 0.f;

    if (!(temp > 0.f)) {  // greedy
        ArgMax best{-INFINITY, 0x7fffffff};
        if ((((uintptr_t)x) & 15) == 0) {
            // four logits a load, four loads in flight
            const int quads = vocab >> 2;
            const float4* x4 = reinterpret_cast<const float4*>(x);
            for (int q0 = tid; q0 < quads; q0 += 4 * THREADS) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    v[u] = q0 + u * THREADS < quads ? x4[q0 + u * THREADS] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = (q0 + u * THREADS) << 2;
                    best = better(best, ArgMax{v[u].x, i});
                    best = better(best, ArgMax{v[u].y, i + 1});
                    best = better(best, ArgMax{v[u].z, i + 2});
                    best = better(best, ArgMax{v[u].w, i + 3});
                }
            }
            for (int i = (quads << 2) + tid; i < vocab; i += THREADS) best = better(best, ArgMax{x[i], i});
        } else {
            for (int i = tid; i < vocab; i += THREADS) best = better(best, ArgMax{x[i], i});
        }
        best = block_argmax(best, arg_scratch);
        if (tid == 0) out[row] = best.index;
        return;
    }

    const float p = top_p ? top_p[row] : 1.f;
    const int k = top_k ? top_k[row] : 0;
    const float mp = min_p ? min_p[row] : 0.f;
    float threshold = -INFINITY;  // on the logit itself (log-probability + lse)

    if ((p > 0.f && p < 1.f) || mp > 0.f || (k > 0 && k < vocab)) {
        float mx = -INFINITY;
        for (int i = tid; i < vocab; i += THREADS) mx = fmaxf(mx, x[i]);
        mx = block_max(mx, scratch);
        if (p > 0.f && p < 1.f) {
            float total = 0.f;
            for (int i = tid; i < vocab; i += THREADS) total += expf(x[i] - mx);
            total = block_sum(total, scratch);
            const float cut = total * p;
            // smallest key u with mass{x > value(u)} < cut
            unsigned lo = ordered_key(-INFINITY), hi = ordered_key(mx);  // hi satisfies: nothing is above the max
            while (lo < hi) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                const float v = from_ordered_key(mid);
                float above = 0.f;
                for (int i = tid; i < vocab; i += THREADS) {
                    const float xi = x[i];
                    if (xi > v) above += expf(xi - mx);
                }
                above = block_sum(above, scratch);
                if (above < cut) hi = mid; else lo = mid + 1;
            }
            threshold = fmaxf(threshold, from_ordered_key(lo));
        }
        if (mp > 0.f) threshold = fmaxf(threshold, mx + logf(mp));
        if (k > 0 && k < vocab) {
            unsigned lo = ordered_key(-INFINITY), hi = ordered_key(mx);
            while (lo < hi) {
                const unsigned mid = lo + ((hi - lo) >> 1);
                const float v = from_ordered_key(mid);
                float above = 0.f;  // counts below 2^24 are exact in fp32
                for (int i = tid; i < vocab; i += THREADS) above += x[i] > v ? 1.f : 0.f;
                above = block_sum(above, scratch);
                if (above < (float)k) hi = mid; else lo = mid + 1;
            }
            threshold = fmaxf(threshold, from_ordered_key(lo));
        }
    }

    const unsigned long long key = keys[row];
    const float inv_t = 1.f / temp;
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += THREADS) {
        const float xi = x[i];
        if (xi < threshold) continue;
        const unsigned long long bits = mix64(key + (unsigned long long)i);
        const double u = ((double)(bits >> 40) + 0.5) * (1.0 / 16777216.0);
        const float g = (float)(-log(-log(u)));
        best = better(best, ArgMax{xi * inv_t + g, i});
    }
    best = block_argmax(best, arg_scratch);
    if (tid == 0) out[row] = best.index;
}

// Constrained decoding: logits[rows[m], i] = -inf wherever bit i of mask m is clear or i is at or
// beyond the mask's own vocabulary (crates/mrun-engine/src/sample.rs:104-116: the reference's
// where(mask, logprobs, -inf); the filters and the draw after it see differences among the
// allowed tokens only, so masking the logits is the same).  words: [masks, words_a_mask] of 32
// tokens each, bit i % 32 of word i / 32 for token i.
__global__ void token_mask_kernel(float* __restrict__ logits, int vocab, const int* __restrict__ rows,
                                  const unsigned* __restrict__ words, int words_a_mask,
                                  const int* __restrict__ mask_vocab) {
    const int m = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vocab) return;
    const bool allowed = i < mask_vocab[m] && ((words[(size_t)m * words_a_mask + (i >> 5)] >> (i & 31)) & 1u);
    if (!allowed) logits[(size_t)rows[m] * vocab + i] = -INFINITY;
}

// logits[row, id] of each distinct id in recent[row, :n] is divided by the penalty when it is
// >= 0 and multiplied when negative (crates/mrun-engine/src/sample.rs:23-36).  A negative id
// is an empty place.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, int vocab,
                                          const int* __restrict__ recent, int n_recent,
                                          const float* __restrict__ penalty) {
    const int row = blockIdx.x, j = threadIdx.x;
    if (j >= n_recent) return;
    const float pen = penalty[row];
    if (pen == 1.f) return;
    const int* ids = recent + (size_t)row * n_recent;
    const int id = ids[j];
    if (id < 0 || id >= vocab) return;
    for (int e = 0; e < j; ++e)
        if (ids[e] == id) return;  // an earlier place handles this id
    float* v = logits + (size_t)row * vocab + id;
    *v = *v >= 0.f ? *v / pen : *v * pen;
}

// The n most likely tokens of a row with their log-probabilities, most likely first, ties by the
// smaller id (crates/mrun-engine/src/sample.rs:134-156).  lp_i = x_i - logsumexp(x), 32-bit.
// One block per row: the row's maximum and sum, then n selection rounds, each the argmax over the
// tokens that come after the one chosen in the round before.
__global__ void __launch_bounds__(THREADS)
top_logprobs_kernel(const float* __restrict__ logits, int vocab, int n, int* __restrict__ ids,
                    float* __restrict__ values) {
    __shared__ float scratch[33];
    __shared__ ArgMax arg_scratch[33];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * vocab;
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += THREADS) mx = fmaxf(mx, x[i]);
    mx = block_max(mx, scratch);
    float total = 0.f;
    for (int i = tid; i < vocab; i += THREADS) total += expf(x[i] - mx);
    total = block_sum(total, scratch);
    const float lse = mx + logf(total);
    ArgMax last{INFINITY, -1};                   // everything comes after this
    for (int round = 0; round < n; ++round) {
        ArgMax best{-INFINITY, 0x7fffffff};
        for (int i = tid; i < vocab; i += THREADS) {
            const float v = x[i];
            // after `last` in the order (value descending, id ascending)
            if (v < last.value || (v == last.value && i > last.index)) best = better(best, ArgMax{v, i});
        }
        best = block_argmax(best, arg_scratch);
        if (tid == 0) {
            ids[(size_t)row * n + round] = best.index;
            values[(size_t)row * n + round] = best.value - lse;
        }
        last = best;
    }
}

}  // namespace

// ids, values: [rows, n]; n at most the vocabulary.
MRUN_API int mrun_top_logprobs(const float* logits, int rows, int vocab, int n, int* ids, float* values,
                               cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && vocab > 0, "top_logprobs: bad sizes rows=%d vocab=%d", rows, vocab);
    MRUN_REQUIRE(n >= 1 && n <= vocab && n <= 1024, "top_logprobs: n=%d must be 1 .. min(vocab, 1024)", n);
    if (rows == 0) return 0;
    top_logprobs_kernel<<<rows, THREADS, 0, stream>>>(logits, vocab, n, ids, values);
    MRUN_CHECK_LAUNCH("top_logprobs");
    return 0;
}

// temperature/top_p/top_k/min_p/keys are per-row device arrays; a null array means the neutral
// value (0, 1, 0, 0).  temperature 0 = greedy (keys may then be null).
MRUN_API int mrun_sample(const float* logits, int rows, int vocab, const float* temperature,
                         const float* top_p, const int* top_k, const float* min_p,
                         const unsigned long long* keys, int* out, cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
    MRUN_REQUIRE(temperature == nullptr || keys != nullptr, "sample: temperature without draw keys");
    if (rows == 0) return 0;
    sample_kernel<<<rows, THREADS, 0, stream>>>(logits, vocab, temperature, top_p, top_k, min_p, keys, out);
    MRUN_CHECK_LAUNCH("sample");
    return 0;
}

MRUN_API int mrun_repetition_penalty(float* logits, int rows, int vocab, const int* recent, int n_recent,
                                     const float* penalty, cudaStream_t stream) {
    MRUN_REQUIRE(rows >= 0 && vocab > 0 && n_recent >= 0 && n_recent <= 1024,
                 "repetition_penalty: bad sizes rows=%d vocab=%d recent=%d", rows, vocab, n_recent);
    if (rows == 0 || n_recent == 0) return 0;
    repetition_penalty_kernel<<<rows, ((n_recent + 31) / 32) * 32, 0, stream>>>(logits, vocab, recent,
                                                                                  n_recent, penalty);
    MRUN_CHECK_LAUNCH("repetition_penalty");
    return 0;
}

// logits: float32 [*, vocab], changed in place.  rows[m]: the row that mask m applies to;
// words: [masks, words_a_mask] unsigned, words_a_mask >= ceil(vocab / 32); mask_vocab[m]: the tokens
// mask m covers (at most vocab; tokens beyond it are not allowed).
MRUN_API int mrun_apply_token_mask(float* logits, int vocab, const int* rows, const unsigned* words, int words_a_mask,
                                   const int* mask_vocab, int masks, cudaStream_t stream) {
    MRUN_REQUIRE(vocab > 0 && masks >= 0, "apply_token_mask: bad sizes vocab=%d masks=%d", vocab, masks);
    MRUN_REQUIRE(words_a_mask >= (vocab + 31) / 32, "apply_token_mask: %d words a mask do not cover %d tokens",
                 words_a_mask, vocab);
    MRUN_REQUIRE(masks <= 65535, "apply_token_mask: %d masks in one call exceed 65535", masks);
    if (masks == 0) return 0;
    token_mask_kernel<<<dim3((vocab + 255) / 256, masks), 256, 0, stream>>>(logits, vocab, rows, words, words_a_mask,
                                                                            mask_vocab);
    MRUN_CHECK_LAUNCH("apply_token_mask");
    return 0;
}
