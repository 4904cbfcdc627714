// Paged grouped-query attention for prompt portions on the fifth-generation tensor cores
// (tcgen05, accumulators in tensor memory), compiled for one head size that is a multiple of 64
// and at most 128: -DMRUN_HEAD_DIM=<64 | 128>.
//
// One thread block per (tile of query tokens, kv head).  The tile's 128 rows are (token, query
// head of the kv head's group) pairs, so a key/value tile read once serves the whole group.  Keys
// are consumed 128 at a time in position order with an online softmax:
//
//   warps 0..7   softmax.  Tensor-memory lane r is row r; warp w and warp w + 4 share the lanes
//                32 (w % 4) .., the first takes the row's keys 0..63 of a tile, the second keys
//                64..127.  A thread reads its half row of S = Q·Kᵀ (tcgen05.ld), masks it, meets
//                its partner for the row's maximum (through shared memory and a barrier of the
//                two warps), keeps the running maximum and its half of the sum in 32-bit, and
//                writes P = exp2(s - max) as packed bf16 into tensor memory (tcgen05.st, one of
//                two P buffers).  It rescales its half of the row of O when the
//                maximum has grown by more than 2^8 since the last rescale (until then P is
//                taken against the older maximum, which is exact: the final division uses the
//                same maximum);
//   warp 8       one lane issues the products: S = Q·Kᵀ into one of two S accumulators, up to two
//                tiles ahead of the softmax (an accumulator is free again once the softmax has
//                its scores in registers), and O += P[j]·V[j] as soon as P[j] is written.  P is
//                read from tensor memory, Q, K and V from shared memory, V as the MN-major
//                operand (its rows are keys, as the cache stores them);
//   warp 9       brings K tiles from the pages into a ring of two stages by TMA: a lane per page
//                of the tile looks the page up in the block table and copies its rows as
//                [rows x 64] boxes with the 128-byte swizzle; warp 10 the V tiles likewise.
//
// The roles hand tiles to one another through mbarriers; every wait is bounded by a cycle budget.
// When a wait runs out the block records a code in the status word, every role stops, the block
// frees its tensor memory and returns; the host reads the status word after the step and raises.
//
// A token at position p sees keys lo..p, lo = 0 or p - window + 1.  Pages that lie wholly
// outside the tile's range, or that were given back, are never dereferenced; their rows of a
// stage keep what an earlier tile left there (the V stages start as zeros), and every key outside
// a row's range is masked.  The page size must be a power of two (pages of 1 .. 128 keys divide
// a tile, larger pages hold whole tiles).
// Math as in the other attention kernels: s = scale * q·k, softmax in 32-bit, o = p·v
// (crates/mrun-engine/src/models/common.rs:129,199-205); P is rounded to bf16 for the second
// product, as the tensor cores take bf16 operands.
#include <cstdio>

#include "attention_paging.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

#ifndef MRUN_HEAD_DIM
#error "compile with -DMRUN_HEAD_DIM=<head size>"
#endif

#if MRUN_HEAD_DIM % 64 == 0 && MRUN_HEAD_DIM <= 128
#define MRUN_ATTN_TC5 1
#else
#define MRUN_ATTN_TC5 0
#endif

#if MRUN_ATTN_TC5

namespace {

using bf16 = __nv_bfloat16;
using namespace tc5;

constexpr int D = MRUN_HEAD_DIM;
constexpr int ROWS = 128;                    // query rows per block = MMA M
constexpr int KEYS = 128;                    // keys per tile = N of the first product, K of the second
constexpr int SPANS_D = D / 64;              // 64-wide spans of the head dimension
constexpr int SPAN_BYTES = 128 * 128;        // one swizzled tile of 128 rows x 64 bf16
constexpr int KV_BYTES = SPANS_D * SPAN_BYTES;          // one stage of K (or V): 128 keys x D
constexpr int Q_BYTES = SPANS_D * SPAN_BYTES;
constexpr int SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + 1024;                // Q, two stages of K and of V
constexpr int SOFTMAX_WARPS = 8, SOFTMAX_THREADS = SOFTMAX_WARPS * 32;
constexpr int MMA_WARP = 8, K_WARP = 9, V_WARP = 10;
constexpr int THREADS = SOFTMAX_THREADS + 3 * 32;                        // 352
constexpr unsigned TMEM_COLS = 512;          // S0 [0,128) S1 [128,256) P0 [256,320) P1 [320,384) O [384, 384 + D)
constexpr unsigned P_COL = 256, O_COL = 384;
constexpr int O_HALF = D / 2;                // columns of O a thread of a pair looks after
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.f;          // log2 of the growth of a row maximum that forces a rescale
constexpr long long WAIT_CYCLES = 3000000000LL;         // about 1.5 s at 2 GHz

enum : int { STATUS_OK = 0, STATUS_LOADER = 1, STATUS_MMA = 2, STATUS_SOFTMAX = 3 };


__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;        // 0: the destination is zero-filled, the source not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
// 2^x by the special-function unit (two units in the last place; P is rounded to bf16 after it).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// The two warps that share a quarter of the rows meet here (barrier 1 + quarter, 64 threads).
__device__ __forceinline__ void pair_sync(int quarter) {
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
}

struct Barriers {
    unsigned long long q_full;
    unsigned long long k_full[2], k_empty[2], v_full[2], v_empty[2];
    unsigned long long s_full[2], s_empty[2], p_full[2], pv_done;
};

__global__ void __launch_bounds__(THREADS, 1)
prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out,
                   const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ token_slot,
                   const int* __restrict__ positions, const int* __restrict__ tile_tok0,
                   const int* __restrict__ tile_ntok, int heads, int kv_heads, int page_size, int page_shift,
                   float scale_log2, int window, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = base;
    unsigned char* k_stages = q_tile + Q_BYTES;
    unsigned char* v_stages = k_stages + 2 * KV_BYTES;
    __shared__ Barriers bars;
    __shared__ unsigned tmem_base_slot;
    __shared__ int aborted;
    __shared__ float pair_max[2][2][ROWS];               // [tile parity][half][row]: the halves' maxima
    __shared__ float pair_sum[2][ROWS];                  // [half][row]: the halves' sums, at the end

    // Blocks start in the order of their index, x first: all kv heads of the first tile of the
    // list, which the host sorted by falling context length, then all of the second, ...
    const int tile = blockIdx.y, kvh = blockIdx.x;
    const int group = heads / kv_heads;
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_rows = ntok * group;
    // tokens of a tile are consecutive positions of one request
    const int pos_first = positions[tok0], pos_last = pos_first + ntok - 1;
    const int lo_tile = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int first_block = lo_tile / KEYS, last_block = pos_last / KEYS;
    const int n_tiles = last_block - first_block + 1;

    if (threadIdx.x == 0) {
        mbar_init(&bars.q_full, SOFTMAX_WARPS);                     // one arrival per softmax warp
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars.k_full[s], 32);                         // every lane of the loader warp arrives
            mbar_init(&bars.v_full[s], 32);
            mbar_init(&bars.k_empty[s], 1);
            mbar_init(&bars.v_empty[s], 1);
            mbar_init(&bars.s_full[s], 1);
            mbar_init(&bars.s_empty[s], SOFTMAX_WARPS);
            mbar_init(&bars.p_full[s], SOFTMAX_WARPS);
        }
        mbar_init(&bars.pv_done, 1);
        aborted = 0;
        mbar_init_fence();
    }
    // rows of a V stage that no copy ever fills must not hold NaN patterns: 0 * NaN is NaN
    for (int i = threadIdx.x; i < 2 * KV_BYTES / 16; i += THREADS)
        reinterpret_cast<uint4*>(v_stages)[i] = make_uint4(0, 0, 0, 0);
    fence_async_smem();
    __syncwarp();
    if (warp == 0) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp < SOFTMAX_WARPS) {
        // ------------------------------------------------------------------ softmax, half rows
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;                          // 0..127
        const unsigned lane_base = tmem_base + ((unsigned)(quarter * 32) << 16);
        // q rows: row r = (token r / group, head kvh * group + r % group); rows past n_rows are zero
        for (int c = threadIdx.x; c < ROWS * (D / 8); c += SOFTMAX_THREADS) {
            const int r = c / (D / 8), chunk = c - r * (D / 8);
            const bool valid = r < n_rows;
            const bf16* src = q;
            if (valid)
                src = q + (size_t)(tok0 + r / group) * q_stride + (size_t)(kvh * group + r % group) * D + chunk * 8;
            cp_async_16(q_tile + (chunk >> 3) * SPAN_BYTES + swizzled_offset(r, chunk & 7), src, valid);
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.q_full);

        const int row_pos = row < n_rows ? pos_first + row / group : -1;      // -1: padding row
        const int row_lo = (window > 0 && row_pos - window + 1 > 0) ? row_pos - window + 1 : 0;
        // the tile's last row sees the most recent keys, its first row the oldest
        const int lo_last = (window > 0 && pos_last - window + 1 > 0) ? pos_last - window + 1 : 0;
        float m_used = -INFINITY, l = 0.f;                           // l: this half's share of the row's sum
        bool alive = true;
        // A warp that gave up on a wait still walks through the remaining tiles, doing nothing but
        // meeting its partner at every barrier, so that no warp is left waiting at one.
        for (int j = 0; j < n_tiles; ++j) {
            const int buf = j & 1;
            if (alive && !__all_sync(0xffffffffu, mbar_wait(&bars.s_full[buf], (j >> 1) & 1, WAIT_CYCLES, &aborted))) alive = false;
            const int key_base = (first_block + j) * KEYS + half * 64;        // of this thread's first score
            // every row of the block sees every key of the tile: no comparisons
            const bool need_mask = (first_block + j) * KEYS + KEYS - 1 > pos_first || (first_block + j) * KEYS < lo_last ||
                                   n_rows < ROWS;
            float sc[64];
            float mx = -INFINITY;
            if (alive) {
                tc_fence_after();
                // the half row's 64 scores, read once
                unsigned raw[64];
                {
                    unsigned (&lo32)[32] = *reinterpret_cast<unsigned (*)[32]>(&raw[0]);
                    unsigned (&hi32)[32] = *reinterpret_cast<unsigned (*)[32]>(&raw[32]);
                    tmem_load32_start(lane_base + buf * KEYS + half * 64, lo32);
                    tmem_load32_start(lane_base + buf * KEYS + half * 64 + 32, hi32);
                    tmem_load_wait();
                }
                // the scores are in registers: the product after next may overwrite the accumulator
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars.s_empty[buf]);
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    pin(raw[i]);
                    sc[i] = __uint_as_float(raw[i]);
                }
                // the largest raw score first (the scale is positive, so it scales the maximum
                // alike); masked scores become -inf and later give p = 0
                if (need_mask) {
                    const int lo_rel = row_lo - key_base, hi_rel = row_pos - key_base;
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        if (i > hi_rel || i < lo_rel) sc[i] = -INFINITY;
                        mx = fmaxf(mx, sc[i]);
                    }
                } else {
                    float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int i = 0; i < 64; i += 4) {
                        mx4[0] = fmaxf(mx4[0], sc[i]); mx4[1] = fmaxf(mx4[1], sc[i + 1]);
                        mx4[2] = fmaxf(mx4[2], sc[i + 2]); mx4[3] = fmaxf(mx4[3], sc[i + 3]);
                    }
                    mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                }
            }
            // the other half of the row
            pair_max[buf][half][row] = mx;
            pair_sync(quarter);
            if (!alive) continue;
            mx = fmaxf(mx, pair_max[buf][half ^ 1][row]) * scale_log2;
            // the maximum the probabilities are taken against moves only by large steps; both
            // halves of a row decide alike, from the same numbers
            float m_new = m_used;
            if (mx > m_used + RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY)) m_new = mx;
            const bool moved = m_new != m_used && m_used != -INFINITY;       // O holds something to rescale
            const bool warp_moved = __any_sync(0xffffffffu, moved);
            if (warp_moved) {
                // O belongs to the second product of the tile before until that has finished
                if (j > 0 && !__all_sync(0xffffffffu, mbar_wait(&bars.pv_done, (j - 1) & 1, WAIT_CYCLES, &aborted))) {
                    alive = false;
                    continue;
                }
                tc_fence_after();
                const float corr = moved ? exp2f(m_used - m_new) : 1.f;
#pragma unroll 1
                for (int c = 0; c < O_HALF; c += 32) {
                    float v[32];
                    tmem_load32(lane_base + O_COL + half * O_HALF + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] *= corr;
                    tmem_store32(lane_base + O_COL + half * O_HALF + c, v);
                }
                l *= corr;
            }
            m_used = m_new;
            // p = 2^(s * scale - m): one fused multiply-add and one special-function call a score.
            // Masked scores are -inf and give 0; a row that has seen nothing yet keeps m_used = -inf.
            const float m_sub = m_used == -INFINITY ? 0.f : -m_used;
            // Two scores an instruction where the hardware has one (fma.f32x2, add.f32x2): these
            // warps are bound by the instructions they issue.
            const float2 scale2 = make_float2(scale_log2, scale_log2), m_sub2 = make_float2(m_sub, m_sub);
            float2 sums = make_float2(0.f, 0.f);
            float packed[32];                                         // two bf16 a word, even key low
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                const float2 x = __ffma2_rn(make_float2(sc[i], sc[i + 1]), scale2, m_sub2);
                const float2 p = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                sums = __fadd2_rn(sums, p);
                packed[i >> 1] = __uint_as_float(pack_bf16(p.x, p.y));
            }
            l += sums.x + sums.y;
            // the P buffer of this tile was read by the second product of the tile before last
            if (j >= 2 && !__all_sync(0xffffffffu, mbar_wait(&bars.v_empty[buf], ((j >> 1) - 1) & 1, WAIT_CYCLES, &aborted))) {
                alive = false;
                continue;
            }
            tmem_store32(lane_base + P_COL + buf * 64 + half * 32, packed);       // this half's keys: words 32 half ..
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_full[buf]);
        }
        // a warp leaves the loop as a whole, so every lane takes part in what follows
        if (alive && !__all_sync(0xffffffffu, mbar_wait(&bars.pv_done, (n_tiles - 1) & 1, WAIT_CYCLES, &aborted))) alive = false;
        if (!alive) {
            if (!*(volatile int*)&aborted) atomicExch(status, STATUS_SOFTMAX);
            atomicExch(&aborted, 1);
        }
        // the row's sum is the two halves' (the partner may have given up: it still comes here)
        pair_sum[half][row] = l;
        pair_sync(quarter);
        if (alive) {
            tc_fence_after();
            const float total = l + pair_sum[half ^ 1][row];
            const float inv = total > 0.f ? 1.f / total : 0.f;
            bf16* dst = out + ((size_t)(tok0 + row / group) * heads + kvh * group + row % group) * D + half * O_HALF;
#pragma unroll 1
            for (int c = 0; c < O_HALF; c += 32) {
                float v[32];
                tmem_load32(lane_base + O_COL + half * O_HALF + c, v);       // every lane of the warp takes part
                if (row < n_rows) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        *reinterpret_cast<uint4*>(dst + c + 8 * k) =
                            make_uint4(pack_bf16(v[8 * k] * inv, v[8 * k + 1] * inv),
                                       pack_bf16(v[8 * k + 2] * inv, v[8 * k + 3] * inv),
                                       pack_bf16(v[8 * k + 4] * inv, v[8 * k + 5] * inv),
                                       pack_bf16(v[8 * k + 6] * inv, v[8 * k + 7] * inv));
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc_qk = instruction_descriptor(ROWS, KEYS);
            constexpr unsigned idesc_pv = instruction_descriptor(ROWS, D, true);
            // The operand descriptors of stage 0, made once: this warp shares its scheduler with
            // two softmax warps, so every instruction it spends between two products delays them.
            // Stage 1 lies KV_BYTES further (the address field counts 16-byte units).
            unsigned long long q_desc[D / 16], k_desc[D / 16], v_desc[KEYS / 16];
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int off = (kk >> 2) * SPAN_BYTES + (kk & 3) * 32;       // 32 bytes further along d per step
                q_desc[kk] = smem_descriptor(q_tile + off);
                k_desc[kk] = smem_descriptor(k_stages + off);
            }
#pragma unroll
            for (int kk = 0; kk < KEYS / 16; ++kk)                            // sixteen rows (two groups) further per step
                v_desc[kk] = smem_descriptor(v_stages + kk * 2048, SPAN_BYTES, 1024);
            constexpr unsigned long long STAGE_STEP = KV_BYTES >> 4;
            bool alive = mbar_wait(&bars.q_full, 0, WAIT_CYCLES, &aborted);
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait(&bars.k_full[s], (j >> 1) & 1, WAIT_CYCLES, &aborted)) return false;
                if (j >= 2 && !mbar_wait(&bars.s_empty[s], ((j >> 1) - 1) & 1, WAIT_CYCLES, &aborted)) return false;
                tc_fence_after();
                const unsigned long long step = s * STAGE_STEP;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem_base + s * KEYS, q_desc[kk], k_desc[kk] + step, idesc_qk, kk > 0 ? 1u : 0u);
                umma_commit(&bars.s_full[s]);
                umma_commit(&bars.k_empty[s]);
                return true;
            };
            // the first products run two tiles ahead of the softmax, the second follow it
            if (alive) alive = issue_qk(0);
            if (alive && n_tiles > 1) alive = issue_qk(1);
            for (int j = 0; alive && j < n_tiles; ++j) {
                const int s = j & 1;
                if (!mbar_wait(&bars.v_full[s], (j >> 1) & 1, WAIT_CYCLES, &aborted)) { alive = false; break; }
                if (!mbar_wait(&bars.p_full[s], (j >> 1) & 1, WAIT_CYCLES, &aborted)) { alive = false; break; }
                tc_fence_after();
                const unsigned long long step = s * STAGE_STEP;
#pragma unroll
                for (int kk = 0; kk < KEYS / 16; ++kk)                        // P: eight columns (16 keys) further per step
                    umma_bf16_a_tmem(tmem_base + O_COL, tmem_base + P_COL + s * 64 + kk * 8, v_desc[kk] + step, idesc_pv,
                                     (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&bars.v_empty[s]);
                umma_commit(&bars.pv_done);
                if (j + 2 < n_tiles && !issue_qk(j + 2)) { alive = false; break; }
            }
            if (!alive) {
                if (!*(volatile int*)&aborted) atomicExch(status, STATUS_MMA);
                atomicExch(&aborted, 1);
            }
        }
    } else {
        // ------------------------------------------------------------------------------- loaders
        const bool keys_role = warp == K_WARP;                        // one warp for K, one for V
        const CUtensorMap* map = keys_role ? &map_k : &map_v;
        unsigned char* stages = keys_role ? k_stages : v_stages;
        unsigned long long* full = keys_role ? bars.k_full : bars.v_full;
        unsigned long long* empty = keys_role ? bars.k_empty : bars.v_empty;
        const int* table = block_tables + (size_t)token_slot[tok0] * max_blocks;
        // pages of up to 128 keys: 128 / page_size boxes of page_size rows; larger pages: one box
        const int box_rows = page_size < KEYS ? page_size : KEYS;
        const int boxes = KEYS / box_rows;
        bool alive = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            const bool free_now = j < 2 || mbar_wait(&empty[s], ((j >> 1) - 1) & 1, WAIT_CYCLES, &aborted);
            if (!__all_sync(0xffffffffu, free_now)) { alive = false; break; }
            const int key0 = (first_block + j) * KEYS;
            unsigned char* stage = stages + s * KV_BYTES;
            // a lane's boxes: lane, lane + 32, ...  It announces their bytes, then copies them.
            unsigned bytes = 0;
            for (int b = lane; b < boxes; b += 32) {
                const int first_key = key0 + b * box_rows;
                if (first_key <= pos_last && first_key + box_rows - 1 >= lo_tile && table[first_key >> page_shift] >= 0)
                    bytes += (unsigned)(box_rows * D * 2);
            }
            if (bytes) mbar_expect_tx(&full[s], bytes);
            else mbar_arrive(&full[s]);
            for (int b = lane; b < boxes; b += 32) {
                const int first_key = key0 + b * box_rows;
                if (first_key > pos_last || first_key + box_rows - 1 < lo_tile) continue;
                const int page = table[first_key >> page_shift];
                if (page < 0) continue;
#pragma unroll
                for (int h = 0; h < SPANS_D; ++h)
                    tma_load_4d(stage + h * SPAN_BYTES + b * box_rows * 128, map, h * 64,
                                first_key & (page_size - 1), kvh, page, &full[s]);
            }
        }
        if (!alive) {
            if (!*(volatile int*)&aborted) atomicExch(status, STATUS_LOADER);
            atomicExch(&aborted, 1);
        }
    }

    // ---------------------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)&aborted) {
        // copies that were requested may still be landing in this block's shared memory
        const long long start = clock64();
        while (clock64() - start < 4000000LL) __nanosleep(1000);
    }
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

}  // namespace

#endif  // MRUN_ATTN_TC5

// 1 when this library holds the tcgen05 prefill kernel (head sizes 64 and 128).
MRUN_API int mrun_attn_prefill_tc5_available() { return MRUN_ATTN_TC5; }

// Rows per tile of the tcgen05 kernel: a tile holds at most 128 / (heads / kv_heads) tokens.
MRUN_API int mrun_attn_prefill_tc5_rows() { return 128; }

// As mrun_attn_prefill, with tiles of at most 128 / (heads / kv_heads) tokens, a page size that is
// a power of two, and `pages` the number of pages of the two cache tensors.  `status` is one
// int on the device, zero before the first call; a non-zero value afterwards names the role whose
// wait ran out (1 loader, 2 products, 3 softmax) and the outputs of that launch are void.
MRUN_API int mrun_attn_prefill_tc5(const void* q, long q_stride, void* out, const void* k_cache,
                                   const void* v_cache, const int* block_tables, int max_blocks,
                                   const int* token_slot, const int* positions, const int* tile_tok0,
                                   const int* tile_ntok, int n_tiles, int heads, int kv_heads, int head_dim,
                                   int page_size, float scale, int window, long pages, int* status,
                                   cudaStream_t stream) {
#if MRUN_ATTN_TC5
    MRUN_REQUIRE(head_dim == D, "attn_prefill_tc5: this library was built for head_dim=%d, got %d", D, head_dim);
    MRUN_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                 "attn_prefill_tc5: heads=%d must be a positive multiple of kv_heads=%d", heads, kv_heads);
    MRUN_REQUIRE(heads / kv_heads <= ROWS, "attn_prefill_tc5: %d query heads per kv head exceed the supported %d",
                 heads / kv_heads, ROWS);
    MRUN_REQUIRE(page_size > 0 && max_blocks > 0 && window >= 0, "attn_prefill_tc5: bad page_size/max_blocks/window");
    MRUN_REQUIRE(n_tiles >= 0, "attn_prefill_tc5: n_tiles=%d", n_tiles);
    MRUN_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                 ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0,
                 "attn_prefill_tc5: q, out and the caches must be 16-byte aligned, q_stride a multiple of 8");
    MRUN_REQUIRE(status != nullptr, "attn_prefill_tc5: the status word is missing");
    MRUN_REQUIRE(page_shift_of(page_size) >= 0, "attn_prefill_tc5: page_size=%d is not a power of two", page_size);
    MRUN_REQUIRE(pages > 0 && pages < (1L << 31), "attn_prefill_tc5: pages=%ld", pages);
    if (n_tiles == 0) return 0;
    CUtensorMap map_k, map_v;
    const int box_rows = page_size < KEYS ? page_size : KEYS;
    if (int rc = paged_cache_map(&map_k, k_cache, pages, kv_heads, page_size, D, box_rows, "attn_prefill_tc5")) return rc;
    if (int rc = paged_cache_map(&map_v, v_cache, pages, kv_heads, page_size, D, box_rows, "attn_prefill_tc5")) return rc;
    static bool configured = false;
    if (!configured) {
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_BYTES), "attn_prefill_tc5");
        configured = true;
    }
    for (int done = 0; done < n_tiles; done += 65535) {          // the grid's second dimension ends at 65535
        const int now = n_tiles - done < 65535 ? n_tiles - done : 65535;
        prefill_tc5_kernel<<<dim3(kv_heads, now), THREADS, SMEM_BYTES, stream>>>(
            map_k, map_v, (const bf16*)q, q_stride, (bf16*)out, block_tables, max_blocks,
            token_slot, positions, tile_tok0 + done, tile_ntok + done, heads, kv_heads, page_size, page_shift_of(page_size),
            scale * LOG2E, window, status);
        MRUN_CHECK_LAUNCH("attn_prefill_tc5");
    }
    return 0;
#else
    return mrun_set_error("attn_prefill_tc5: not built for head_dim=%d (head sizes 64 and 128 only)", MRUN_HEAD_DIM);
#endif
}
