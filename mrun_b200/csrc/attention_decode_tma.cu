// Paged grouped-query attention for decode steps, keys and values brought by TMA: the same work
// list, plan, scratch and merge as the decode kernel of attention_mma.cu (a step's 64-key tiles of
// all (token, kv head) pairs dealt to the blocks; a pair shared between blocks is merged by the one
// that arrives last), with another way of moving the tiles:
//
//   warp 4       the producer.  It walks the block's tiles ahead of the others; for every tile a
//                lane per page looks the page up in the block table and copies its rows of K and
//                of V as [rows x 64] boxes (cp.async.bulk.tensor, 128-byte swizzle) into a ring
//                of two or three stages, each guarded by a full/empty pair of mbarriers.  It
//                does not stop at the end of a pair: while the other warps merge and write a
//                pair's result, the first tiles of the next pair are already on their way;
//   warps 0..3   the consumers: per pair the queries (ready, or normed and rotated here from the
//                raw projection rows), then per tile each warp takes 16 of the 64 keys with
//                mma.sync over ldmatrix fragments read through the swizzle, online softmax in
//                32-bit; the four warps' results meet in a small buffer of their own, so the
//                ring is never drained.
//
// A stage is 2 x 64 x D x 2 bytes without padding (the swizzle keeps ldmatrix free of bank
// conflicts), so two blocks with three stages each fit a multiprocessor at D = 128 and up to five
// tiles a multiprocessor are in flight.  Head sizes 64 and 128, page sizes that are powers of
// two, at most 16 query heads per kv head.  Every mbarrier wait is bounded; a wait that runs out
// sets the status word (the host reads it after the step and raises) and the block runs to its
// end without waiting again.
//
// A second kernel of the same parts (decode_cluster_kernel, below) serves steps with few pairs:
// a thread-block cluster takes one pair, cuts its tiles among its blocks and merges their partial
// results through distributed shared memory, with neither plan nor scratch.
//
// Math as in the other attention kernels (crates/mrun-engine/src/models/common.rs:129,199-205).
#include <cstdio>

#include "attention_frag.cuh"
#include "tcgen05.cuh"

#if MRUN_HEAD_DIM % 64 == 0 && MRUN_HEAD_DIM <= 128
#define MRUN_DECODE_TMA 1
#else
#define MRUN_DECODE_TMA 0
#endif

#if MRUN_DECODE_TMA

namespace {

using namespace tc5;

constexpr int SPANS = D / 64;                        // 64-wide spans of the head dimension
constexpr int SPAN_BYTES = BLOCK_N * 128;            // 64 rows x 128 bytes
constexpr int TILE_BYTES = SPANS * SPAN_BYTES;       // one K (or V) tile
constexpr int STAGE_BYTES = 2 * TILE_BYTES;          // K then V
constexpr int CONSUMERS = 128, TMA_THREADS = CONSUMERS + 32;
constexpr int MS = D + 2;                            // a merged row: D values, maximum, sum
constexpr long long WAIT_CYCLES = 3000000000LL;      // about 1.5 s at 2 GHz

enum : int { STATUS_PRODUCER = 1, STATUS_CONSUMER = 2 };

__host__ __device__ constexpr size_t tma_smem_bytes(int ring, int group) {
    return (size_t)ring * STAGE_BYTES + 1024                           // the ring, 1024-byte aligned
           + (size_t)16 * LD * sizeof(bf16)                             // q rows
           + (size_t)4 * group * MS * sizeof(float)                     // the four warps' results
           + (size_t)4 * D * sizeof(float) + 2 * D * sizeof(bf16);      // head staging, the step's own k and v
}

// Address of the 16-byte chunk `chunk` (0 .. D/8 - 1) of row `row` of a swizzled tile.
__device__ __forceinline__ const unsigned char* swz(const unsigned char* tile, int row, int chunk) {
    return tile + (chunk >> 3) * SPAN_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// One 16-row warp tile against the 16 keys krow0 .. krow0+15 of a swizzled K and V tile: the same
// arithmetic as attend_tile<16>, with the fragments fetched through the swizzle.
__device__ __forceinline__ void attend_slice(const bf16* q_tile, const unsigned char* k_tile, const unsigned char* v_tile,
                                             int krow0, int key_base, float scale_log2, const int (&row_pos)[2],
                                             const int (&row_lo)[2], float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
    const int lane = threadIdx.x & 31;
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a[4], b[4];
        ldmatrix_x4(a, q_tile + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8);
        ldmatrix_x4(b, swz(k_tile, krow0 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1)));
        mma_bf16(s[0], a, b[0], b[1]);
        mma_bf16(s[1], a, b[2], b[3]);
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            float v = s[nt][e] * scale_log2;
            const int key = key_base + krow0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            if (key > row_pos[r] || key < row_lo[r]) v = -INFINITY;
            s[nt][e] = v;
            mx[r] = fmaxf(mx[r], v);
        }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        corr[r] = (m[r] == -INFINITY) ? 0.f : exp2f(m[r] - m_new);
        m[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const float p = (m[r] == -INFINITY) ? 0.f : exp2f(s[nt][e] - m[r]);
            s[nt][e] = p;
            sum[r] += p;
        }
#pragma unroll
    for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + sum[r];       // per-thread partial; reduced at the end
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }
    unsigned a[4];
    a[0] = pack_bf16(s[0][0], s[0][1]);
    a[1] = pack_bf16(s[0][2], s[0][3]);
    a[2] = pack_bf16(s[1][0], s[1][1]);
    a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int dt = 0; dt < D / 8; dt += 2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, swz(v_tile, krow0 + (lane & 7) + ((lane >> 3) & 1) * 8, dt + (lane >> 4)));
        mma_bf16(o[dt], a, b[0], b[1]);
        mma_bf16(o[dt + 1], a, b[2], b[3]);
    }
}

// The pair that tile `u` of the flat list belongs to, found as the consumers and the producer walk
// the block's range: `tok`/`kvh` come in as the pair of the tile before (or the plan's start).
struct Segment {
    int kvh, tok, j0, len, pair_tiles, pair_start, pos, lo, first_block, last_block;
    bool complete;
};

__device__ __forceinline__ Segment next_segment(int seg, int u, int u_end, int& kvh, int& tok, int tiles_per_head,
                                                const int* __restrict__ prefix, const int* __restrict__ positions,
                                                int window) {
    if (seg > 0) {
        ++tok;
        if (u - kvh * tiles_per_head >= tiles_per_head) {
            ++kvh;
            tok = 0;
        }
    }
    const int r = u - kvh * tiles_per_head;
    while (prefix[tok + 1] <= r) ++tok;                          // skip tokens without tiles (padding)
    Segment sg;
    sg.kvh = kvh;
    sg.tok = tok;
    sg.pair_tiles = prefix[tok + 1] - prefix[tok];
    sg.j0 = r - prefix[tok];
    sg.len = min(u_end - u, sg.pair_tiles - sg.j0);
    sg.complete = sg.j0 == 0 && sg.len == sg.pair_tiles;
    sg.pair_start = kvh * tiles_per_head + prefix[tok];
    sg.pos = positions[tok];
    sg.lo = (window > 0 && sg.pos - window + 1 > 0) ? sg.pos - window + 1 : 0;
    sg.first_block = sg.lo / BLOCK_N + sg.j0;
    sg.last_block = sg.first_block + sg.len - 1;
    return sg;
}

// grid: `blocks` blocks, the number the plan was made for.  Scratch as for decode_kernel.
template <int RING>
__global__ void __launch_bounds__(TMA_THREADS)
decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                  const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ token_slot,
                  const int* __restrict__ positions, const int* __restrict__ tile_prefix,
                  const int4* __restrict__ assignment, int tokens, float* __restrict__ part_o,
                  float* __restrict__ part_ml, int* __restrict__ counters, int heads, int kv_heads, int page_size,
                  int page_shift, float scale_log2, int window, const FusedInput fused, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int group = heads / kv_heads;
    bf16* q_tile = reinterpret_cast<bf16*>(ring + RING * STAGE_BYTES);                   // [16][LD]
    float* merge = reinterpret_cast<float*>(q_tile + 16 * LD);                            // [4][group][MS]
    float (*head_vec)[D] = reinterpret_cast<float (*)[D]>(merge + 4 * group * MS);        // [4][D]
    bf16* new_k = reinterpret_cast<bf16*>(head_vec + 4);                                  // this step's own key, value
    bf16* new_v = new_k + D;
    __shared__ unsigned long long full_bar[RING], empty_bar[RING];
    __shared__ int ticket_shared, aborted;

    const int block_id = blockIdx.x, n_blocks_grid = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int4 mine = assignment[2 * block_id], shape = assignment[2 * block_id + 1];
    const int u_begin = mine.x, u_end = mine.y;
    const int tiles_per_head = shape.x, per = shape.y, splits = shape.z;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RING; ++s) {
            mbar_init(&full_bar[s], 32);                 // every lane of the producer arrives
            mbar_init(&empty_bar[s], 4);                 // one arrival per consumer warp
        }
        aborted = 0;
        mbar_init_fence();
    }
    // The producer looks its first run of tiles up (plan, positions: dependent loads from global
    // memory) while the block prepares its shared memory.  (Also reading the block-table entries
    // of the first tiles and prefetching the tensor maps here made the kernel slower.)
    Segment first_sg = {};
    int first_kvh = mine.z, first_tok = mine.w;
    if (warp == 4 && u_begin < u_end)
        first_sg = next_segment(0, u_begin, u_end, first_kvh, first_tok, tiles_per_head, tile_prefix, positions, window);
    // rows of a V tile that no copy fills must not hold NaN patterns: 0 * NaN is NaN
    for (int s = 0; s < RING; ++s)
        for (int i = threadIdx.x; i < TILE_BYTES / 16; i += TMA_THREADS)
            reinterpret_cast<uint4*>(ring + s * STAGE_BYTES + TILE_BYTES)[i] = make_uint4(0, 0, 0, 0);
    fence_async_smem();
    __syncthreads();

    if (warp == 4) {
        // ------------------------------------------------------------------------------ producer
        const int box_rows = page_size < BLOCK_N ? page_size : BLOCK_N;
        const int boxes = BLOCK_N / box_rows;
        int kvh = first_kvh, tok = first_tok, u = u_begin, it = 0;
        bool alive = true;
        for (int seg = 0; alive && u < u_end; ++seg) {
            const Segment sg = seg == 0 ? first_sg
                                        : next_segment(seg, u, u_end, kvh, tok, tiles_per_head, tile_prefix, positions, window);
            const int* table = block_tables + (size_t)token_slot[sg.tok] * max_blocks;
            for (int block = sg.first_block; block <= sg.last_block; ++block, ++it) {
                const int s = it % RING, use = it / RING;
                const bool free_now = use == 0 || mbar_wait(&empty_bar[s], (use - 1) & 1, WAIT_CYCLES, &aborted);
                if (!__all_sync(0xffffffffu, free_now)) { alive = false; break; }
                unsigned char* stage = ring + s * STAGE_BYTES;
                const int key0 = block * BLOCK_N;
                // a lane's boxes: lane, lane + 32, ...  It announces their bytes, then copies them.
                unsigned bytes = 0;
                for (int b = lane; b < boxes; b += 32) {
                    const int first_key = key0 + b * box_rows;
                    if (first_key <= sg.pos && first_key + box_rows - 1 >= sg.lo && table[first_key >> page_shift] >= 0)
                        bytes += (unsigned)(2 * box_rows * D * 2);
                }
                if (bytes) mbar_expect_tx(&full_bar[s], bytes);
                else mbar_arrive(&full_bar[s]);
                for (int b = lane; b < boxes; b += 32) {
                    const int first_key = key0 + b * box_rows;
                    if (first_key > sg.pos || first_key + box_rows - 1 < sg.lo) continue;
                    const int page = table[first_key >> page_shift];
                    if (page < 0) continue;
#pragma unroll
                    for (int h = 0; h < SPANS; ++h) {
                        tma_load_4d(stage + h * SPAN_BYTES + b * box_rows * 128, &map_k, h * 64,
                                    first_key & (page_size - 1), sg.kvh, page, &full_bar[s]);
                        tma_load_4d(stage + TILE_BYTES + h * SPAN_BYTES + b * box_rows * 128, &map_v, h * 64,
                                    first_key & (page_size - 1), sg.kvh, page, &full_bar[s]);
                    }
                }
            }
            u += sg.len;
        }
        if (!alive) {
            if (!*(volatile int*)&aborted) atomicExch(status, STATUS_PRODUCER);
            atomicExch(&aborted, 1);
        }
    } else {
        // ----------------------------------------------------------------------------- consumers
        // padding rows come out as zeros
        for (int t = block_id; t < tokens; t += n_blocks_grid)
            if (positions[t] < 0)
                for (int i = threadIdx.x; i < heads * D; i += CONSUMERS)
                    out[(size_t)(fused.rows ? fused.rows[t] : t) * heads * D + i] = __float2bfloat16_rn(0.f);

        // A warp whose wait ran out sets the flag and keeps walking (its later waits return at once,
        // its numbers are void), so that every barrier of the four warps is still met by all.
        int kvh = mine.z, tok = mine.w, u = u_begin, it = 0;
        bool alive = true;
        for (int seg = 0; u < u_end; ++seg) {
            const Segment sg = next_segment(seg, u, u_end, kvh, tok, tiles_per_head, tile_prefix, positions, window);
            const int pos = sg.pos, lo = sg.lo;
            const int b1 = pos / BLOCK_N;
            float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
            float o[D / 8][4];
#pragma unroll
            for (int dt = 0; dt < D / 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

            const bool owns_new_token = fused.enabled && sg.last_block == b1;
            const int q_row = fused.rows ? fused.rows[sg.tok] : sg.tok;        // the row of q and out
            if (!fused.enabled) {
                for (int c = threadIdx.x; c < 16 * CHUNKS; c += CONSUMERS) {
                    const int row = c / CHUNKS, chunk = c - row * CHUNKS;
                    uint4 value = make_uint4(0, 0, 0, 0);
                    if (row < group)
                        value = *reinterpret_cast<const uint4*>(q + (size_t)q_row * q_stride + (size_t)(sg.kvh * group + row) * D + chunk * 8);
                    *reinterpret_cast<uint4*>(q_tile + row * LD + chunk * 8) = value;
                }
            } else {
                // q, k and v arrive raw: [q heads | k heads | v heads] of D elements each in the token's row
                const bf16* token_row = q + (size_t)sg.tok * q_stride;
                const float2* cs = fused.rot ? fused.rot + (size_t)sg.tok * (fused.rotary_dim >> 1) : nullptr;
                // where the token's own key and value go: asked for now, used after the heads are made
                const int slot = (owns_new_token && fused.slots) ? fused.slots[sg.tok] : -1;
                for (int row = warp; row < 16; row += 4) {
                    if (row < group)
                        norm_rotate_head(token_row + (size_t)(sg.kvh * group + row) * D, fused.q_weight, fused.eps, cs,
                                         fused.rotary_dim, head_vec[warp], q_tile + row * LD);
                    else
                        for (int e = lane; e < D; e += 32) q_tile[row * LD + e] = __float2bfloat16_rn(0.f);
                }
                if (owns_new_token) {
                    // the block that holds the pair's last tile makes the token's own key and value: into
                    // the page for later steps, and into shared memory for this one
                    if (warp == 0)
                        norm_rotate_head(token_row + (size_t)(heads + sg.kvh) * D, fused.k_weight, fused.eps, cs,
                                         fused.rotary_dim, head_vec[0], new_k);
                    if (warp == 1)
                        for (int e = lane; e < D; e += 32) new_v[e] = token_row[(size_t)(heads + kv_heads + sg.kvh) * D + e];
                    consumer_sync();
                    if (slot >= 0) {
                        const int page = slot / page_size, off = slot - page * page_size;
                        const size_t at = (((size_t)page * kv_heads + sg.kvh) * page_size + off) * D;
                        for (int c = threadIdx.x; c < 2 * CHUNKS; c += CONSUMERS) {
                            const bool is_v = c >= CHUNKS;
                            const int chunk = is_v ? c - CHUNKS : c;
                            *reinterpret_cast<uint4*>((is_v ? fused.v_cache : fused.k_cache) + at + chunk * 8) =
                                *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + chunk * 8);
                        }
                    }
                }
            }
            consumer_sync();                                    // q (and the new key and value) are in place

            int row_pos[2], row_lo[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = (lane >> 2) + rr * 8;
                row_pos[rr] = row < group ? pos : -1;
                row_lo[rr] = lo;
            }
            for (int block = sg.first_block; block <= sg.last_block; ++block, ++it) {
                const int s = it % RING, use = it / RING;
                if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], use & 1, WAIT_CYCLES, &aborted)) && alive) {
                    alive = false;
                    if (lane == 0) {
                        if (!*(volatile int*)&aborted) atomicExch(status, STATUS_CONSUMER);
                        atomicExch(&aborted, 1);
                    }
                }
                unsigned char* k_tile = ring + s * STAGE_BYTES;
                unsigned char* v_tile = k_tile + TILE_BYTES;
                const int key_base = block * BLOCK_N;
                if (owns_new_token && block == b1) {
                    // the page row of this step's token was not written when the tile was requested
                    const int row = pos - key_base;
                    for (int c = threadIdx.x; c < 2 * CHUNKS; c += CONSUMERS) {
                        const bool is_v = c >= CHUNKS;
                        const int chunk = is_v ? c - CHUNKS : c;
                        *reinterpret_cast<uint4*>(const_cast<unsigned char*>(swz(is_v ? v_tile : k_tile, row, chunk))) =
                            *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + chunk * 8);
                    }
                    consumer_sync();
                }
                // warp w takes keys 16w .. 16w+15 of the tile
                if (key_base + warp * 16 <= pos && key_base + warp * 16 + 15 >= lo)
                    attend_slice(q_tile, k_tile, v_tile, warp * 16, key_base, scale_log2, row_pos, row_lo, m, l, o);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);
            }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
                l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
            }
            // the four warps meet: merge[warp][row < group][D + 2]
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = (lane >> 2) + rr * 8;
                if (row < group) {
                    float* dst = merge + (warp * group + row) * MS;
#pragma unroll
                    for (int dt = 0; dt < D / 8; ++dt) {
                        dst[dt * 8 + (lane & 3) * 2] = o[dt][2 * rr];
                        dst[dt * 8 + (lane & 3) * 2 + 1] = o[dt][2 * rr + 1];
                    }
                    if ((lane & 3) == 0) {
                        dst[D] = m[rr];
                        dst[D + 1] = l[rr];
                    }
                }
            }
            consumer_sync();
            const size_t my_slot = (size_t)block_id * 2 + (seg == 0 ? 0 : 1);
            // a thread takes four values of a row: the warps' maxima and sums are read once for them
            for (int i = threadIdx.x; i < group * (D / 4); i += CONSUMERS) {
                const int row = i / (D / 4), d = (i - row * (D / 4)) * 4;
                float mm = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[(w * group + row) * MS + D]);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float ll = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float* src = merge + (w * group + row) * MS;
                    const float c = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
                    const float2 lo2 = *reinterpret_cast<const float2*>(src + d), hi2 = *reinterpret_cast<const float2*>(src + d + 2);
                    acc.x += lo2.x * c; acc.y += lo2.y * c; acc.z += hi2.x * c; acc.w += hi2.y * c;
                    ll += src[D + 1] * c;
                }
                if (sg.complete) {
                    const float inv = ll > 0.f ? 1.f / ll : 0.f;
                    __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                    __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                    uint2 packed;
                    packed.x = *reinterpret_cast<unsigned*>(&lo2);
                    packed.y = *reinterpret_cast<unsigned*>(&hi2);
                    *reinterpret_cast<uint2*>(out + ((size_t)q_row * heads + sg.kvh * group + row) * D + d) = packed;
                } else {
                    *reinterpret_cast<float4*>(part_o + (my_slot * 16 + row) * D + d) = acc;
                    if (d == 0) *reinterpret_cast<float2*>(part_ml + (my_slot * 16 + row) * 2) = make_float2(mm, ll);
                }
            }
            if (!sg.complete) {
                // the blocks that share this pair are p_first .. p_last; the last to arrive merges their
                // pieces in block order
                int p_first, p_last;
                if (splits > 0) {            // the pair's own run of blocks: `splits` blocks a kv head
                    p_first = sg.kvh * splits + tile_prefix[tokens + 1 + sg.tok];
                    p_last = p_first + (sg.pair_tiles + per - 1) / per - 1;
                } else {
                    p_first = sg.pair_start / per;
                    p_last = (sg.pair_start + sg.pair_tiles - 1) / per;
                }
                __threadfence();
                consumer_sync();
                if (threadIdx.x == 0) ticket_shared = atomicAdd(&counters[sg.tok * kv_heads + sg.kvh], 1);
                consumer_sync();
                if (ticket_shared == p_last - p_first) {
                    __threadfence();
                    // A thread takes four values of a row.  The pieces are read four at a time, all
                    // loads of a round requested before any is used (one piece after the other the
                    // merge took a third of a block's time).
                    for (int i = threadIdx.x; i < group * (D / 4); i += CONSUMERS) {
                        const int row = i / (D / 4), d = (i - row * (D / 4)) * 4;
                        // block p's piece of this pair is its first segment iff its range starts inside the pair
                        auto slot_of = [&](int p) -> size_t {
                            return (size_t)p * 2 + ((splits > 0 || p * per >= sg.pair_start) ? 0 : 1);
                        };
                        float mm = -INFINITY;
                        for (int p0 = p_first; p0 <= p_last; p0 += 4) {
                            float ms[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                ms[k] = p0 + k <= p_last ? __ldcg(part_ml + (slot_of(p0 + k) * 16 + row) * 2) : -INFINITY;
#pragma unroll
                            for (int k = 0; k < 4; ++k) mm = fmaxf(mm, ms[k]);
                        }
                        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                        float ll = 0.f;
                        for (int p0 = p_first; p0 <= p_last; p0 += 4) {
                            float2 ml[4];
                            float4 po[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                ml[k] = make_float2(-INFINITY, 0.f);
                                po[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                                if (p0 + k <= p_last) {
                                    const size_t at = slot_of(p0 + k) * 16 + row;
                                    ml[k] = __ldcg(reinterpret_cast<const float2*>(part_ml + at * 2));
                                    po[k] = __ldcg(reinterpret_cast<const float4*>(part_o + at * D + d));
                                }
                            }
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float c = (ml[k].x == -INFINITY) ? 0.f : exp2f(ml[k].x - mm);
                                acc.x += po[k].x * c; acc.y += po[k].y * c; acc.z += po[k].z * c; acc.w += po[k].w * c;
                                ll += ml[k].y * c;
                            }
                        }
                        const float inv = ll > 0.f ? 1.f / ll : 0.f;
                        __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                        __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                        uint2 packed;
                        packed.x = *reinterpret_cast<unsigned*>(&lo2);
                        packed.y = *reinterpret_cast<unsigned*>(&hi2);
                        *reinterpret_cast<uint2*>(out + ((size_t)q_row * heads + sg.kvh * group + row) * D + d) = packed;
                    }
                    if (threadIdx.x == 0) counters[sg.tok * kv_heads + sg.kvh] = 0;
                }
            }
            consumer_sync();            // the merge area, q and ticket_shared are reused by the next segment
            u += sg.len;
        }
    }
    __syncthreads();
    if (*(volatile int*)&aborted) {
        // copies that were requested may still be landing in this block's shared memory
        const long long start = clock64();
        while (clock64() - start < 4000000LL) __nanosleep(1000);
    }
}

// ------------------------------------------------------------------------------------------
// The same attention for steps with few (token, kv head) pairs, one thread-block cluster a pair.
// The pair's tiles are cut evenly into as many pieces as the cluster has blocks (a function of
// the pair's own length and the cluster size, so no plan is read and a pair's cut does not depend
// on the other pairs of the step).  A block streams its piece as above, leaves its partial result
// (rows x D values, maximum, sum) in its own shared memory, the cluster meets at its hardware
// barrier, and the first block reads the pieces of the others through distributed shared memory
// in block order and writes the pair's heads: no scratch in global memory, no fence, no counter.
// grid (cluster size, tokens * kv_heads), cluster (cluster size, 1, 1); up to 8 query heads a kv head.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_address(const void* own_shared, unsigned rank) {
    unsigned local = (unsigned)__cvta_generic_to_shared(own_shared), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ float4 cluster_load4(unsigned address) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(address));
    return v;
}
__device__ __forceinline__ float2 cluster_load2(unsigned address) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "r"(address));
    return v;
}

template <int RING>
__global__ void __launch_bounds__(TMA_THREADS)
decode_cluster_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out,
                      const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ token_slot,
                      const int* __restrict__ positions, int heads, int kv_heads, int page_size, int page_shift,
                      float scale_log2, int window, const FusedInput fused, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int group = heads / kv_heads;
    bf16* q_tile = reinterpret_cast<bf16*>(ring + RING * STAGE_BYTES);                   // [16][LD]
    float* merge = reinterpret_cast<float*>(q_tile + 16 * LD);                            // [4][group][MS]
    float (*head_vec)[D] = reinterpret_cast<float (*)[D]>(merge + 4 * group * MS);        // [4][D]
    bf16* new_k = reinterpret_cast<bf16*>(head_vec + 4);
    bf16* new_v = new_k + D;
    // the block's piece takes the place of the queries once the tiles are done: [group][PS],
    // PS = D + 4 so that a row starts on 16 bytes (group <= 8: 8 x 132 floats fit 16 x LD bf16)
    constexpr int PS = D + 4;
    float* piece = reinterpret_cast<float*>(q_tile);
    __shared__ unsigned long long full_bar[RING], empty_bar[RING];
    __shared__ int aborted;

    const unsigned rank = blockIdx.x, pieces = gridDim.x;
    const int pair = blockIdx.y, tok = pair / kv_heads, kvh = pair - tok * kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[tok], slot_row = token_slot[tok];      // asked for together: one trip
    const int q_row = fused.rows ? fused.rows[tok] : tok;
    if (pos < 0) {                                   // a padding row: zeros, and the whole cluster leaves
        if (rank == 0)
            for (int i = threadIdx.x; i < group * D; i += TMA_THREADS)
                out[((size_t)q_row * heads + kvh * group) * D + i] = __float2bfloat16_rn(0.f);
        return;
    }
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int b0 = lo / BLOCK_N, b1 = pos / BLOCK_N, pair_tiles = b1 - b0 + 1;
    const int base = pair_tiles / (int)pieces, extra = pair_tiles - base * (int)pieces;
    const int len = base + ((int)rank < extra ? 1 : 0);
    const int first_block = b0 + (int)rank * base + min((int)rank, extra), last_block = first_block + len - 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RING; ++s) {
            mbar_init(&full_bar[s], 32);
            mbar_init(&empty_bar[s], 4);
        }
        aborted = 0;
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == 4) {
        // ------------------------------------------------------------------------------ producer
        const int box_rows = page_size < BLOCK_N ? page_size : BLOCK_N;
        const int boxes = BLOCK_N / box_rows;
        const int* table = block_tables + (size_t)slot_row * max_blocks;
        bool alive = true;
        int it = 0;
        // The pages of the next tiles are looked up 32 boxes at a time, one a lane, so that the
        // loop asks the block table once in several tiles and not once a tile (a dependent load
        // in front of every copy otherwise); pages smaller than two keys look up as they go.
        const bool windowed = boxes <= 32;
        const int tiles_a_window = windowed ? 32 / boxes : 1;
        int window_page = -1;
        for (int block = first_block; alive && block <= last_block; ++block, ++it) {
            const int s = it % RING, use = it / RING;
            const int in_window = it % tiles_a_window;
            if (windowed && in_window == 0) {
                const int first_key = block * BLOCK_N + lane * box_rows;
                window_page = (first_key <= pos && first_key + box_rows - 1 >= lo) ? table[first_key >> page_shift] : -1;
            }
            const bool free_now = use == 0 || mbar_wait(&empty_bar[s], (use - 1) & 1, WAIT_CYCLES, &aborted);
            if (!__all_sync(0xffffffffu, free_now)) { alive = false; break; }
            unsigned char* stage = ring + s * STAGE_BYTES;
            const int key0 = block * BLOCK_N;
            // lane b takes box b of the tile (boxes <= 32), or boxes b, b + 32, ... of it
            int my_page = -1;
            if (windowed) my_page = __shfl_sync(0xffffffffu, window_page, (in_window * boxes + lane) & 31);
            unsigned bytes = 0;
            for (int b = lane; b < boxes; b += 32) {
                const int first_key = key0 + b * box_rows;
                const bool wanted = first_key <= pos && first_key + box_rows - 1 >= lo;
                const int page = !wanted ? -1 : windowed ? my_page : table[first_key >> page_shift];
                if (page >= 0) {
                    bytes += (unsigned)(2 * box_rows * D * 2);
                    continue;
                }
                // Rows of a V tile that no copy fills must not hold NaN patterns (0 * NaN is NaN): the
                // lane that leaves a box out clears the box's V rows itself, before it arrives.
#pragma unroll
                for (int h = 0; h < SPANS; ++h) {
                    uint4* rows = reinterpret_cast<uint4*>(stage + TILE_BYTES + h * SPAN_BYTES + b * box_rows * 128);
                    for (int i = 0; i < box_rows * 8; ++i) rows[i] = make_uint4(0, 0, 0, 0);
                }
            }
            if (bytes) mbar_expect_tx(&full_bar[s], bytes);
            else mbar_arrive(&full_bar[s]);
            for (int b = lane; b < boxes; b += 32) {
                const int first_key = key0 + b * box_rows;
                if (first_key > pos || first_key + box_rows - 1 < lo) continue;
                const int page = windowed ? my_page : table[first_key >> page_shift];
                if (page < 0) continue;
#pragma unroll
                for (int h = 0; h < SPANS; ++h) {
                    tma_load_4d(stage + h * SPAN_BYTES + b * box_rows * 128, &map_k, h * 64,
                                first_key & (page_size - 1), kvh, page, &full_bar[s]);
                    tma_load_4d(stage + TILE_BYTES + h * SPAN_BYTES + b * box_rows * 128, &map_v, h * 64,
                                first_key & (page_size - 1), kvh, page, &full_bar[s]);
                }
            }
        }
        if (!alive) {
            if (!*(volatile int*)&aborted) atomicExch(status, STATUS_PRODUCER);
            atomicExch(&aborted, 1);
        }
    } else {
        // ----------------------------------------------------------------------------- consumers
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[D / 8][4];
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
        if (len > 0) {
            const bool owns_new_token = fused.enabled && last_block == b1;
            if (!fused.enabled) {
                for (int c = threadIdx.x; c < 16 * CHUNKS; c += CONSUMERS) {
                    const int row = c / CHUNKS, chunk = c - row * CHUNKS;
                    uint4 value = make_uint4(0, 0, 0, 0);
                    if (row < group)
                        value = *reinterpret_cast<const uint4*>(q + (size_t)q_row * q_stride + (size_t)(kvh * group + row) * D + chunk * 8);
                    *reinterpret_cast<uint4*>(q_tile + row * LD + chunk * 8) = value;
                }
            } else {
                const bf16* token_row = q + (size_t)tok * q_stride;
                const float2* cs = fused.rot ? fused.rot + (size_t)tok * (fused.rotary_dim >> 1) : nullptr;
                const int slot = (owns_new_token && fused.slots) ? fused.slots[tok] : -1;
                for (int row = warp; row < 16; row += 4) {
                    if (row < group)
                        norm_rotate_head(token_row + (size_t)(kvh * group + row) * D, fused.q_weight, fused.eps, cs,
                                         fused.rotary_dim, head_vec[warp], q_tile + row * LD);
                    else
                        for (int e = lane; e < D; e += 32) q_tile[row * LD + e] = __float2bfloat16_rn(0.f);
                }
                if (owns_new_token) {
                    if (warp == 0)
                        norm_rotate_head(token_row + (size_t)(heads + kvh) * D, fused.k_weight, fused.eps, cs,
                                         fused.rotary_dim, head_vec[0], new_k);
                    if (warp == 1)
                        for (int e = lane; e < D; e += 32) new_v[e] = token_row[(size_t)(heads + kv_heads + kvh) * D + e];
                    consumer_sync();
                    if (slot >= 0) {
                        const int page = slot / page_size, off = slot - page * page_size;
                        const size_t at = (((size_t)page * kv_heads + kvh) * page_size + off) * D;
                        for (int c = threadIdx.x; c < 2 * CHUNKS; c += CONSUMERS) {
                            const bool is_v = c >= CHUNKS;
                            const int chunk = is_v ? c - CHUNKS : c;
                            *reinterpret_cast<uint4*>((is_v ? fused.v_cache : fused.k_cache) + at + chunk * 8) =
                                *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + chunk * 8);
                        }
                    }
                }
            }
            consumer_sync();                                    // q (and the new key and value) are in place

            int row_pos[2], row_lo[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int row = (lane >> 2) + rr * 8;
                row_pos[rr] = row < group ? pos : -1;
                row_lo[rr] = lo;
            }
            bool alive = true;
            int it = 0;
            for (int block = first_block; block <= last_block; ++block, ++it) {
                const int s = it % RING, use = it / RING;
                if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], use & 1, WAIT_CYCLES, &aborted)) && alive) {
                    alive = false;
                    if (lane == 0) {
                        if (!*(volatile int*)&aborted) atomicExch(status, STATUS_CONSUMER);
                        atomicExch(&aborted, 1);
                    }
                }
                unsigned char* k_tile = ring + s * STAGE_BYTES;
                unsigned char* v_tile = k_tile + TILE_BYTES;
                const int key_base = block * BLOCK_N;
                if (owns_new_token && block == b1) {
                    const int row = pos - key_base;
                    for (int c = threadIdx.x; c < 2 * CHUNKS; c += CONSUMERS) {
                        const bool is_v = c >= CHUNKS;
                        const int chunk = is_v ? c - CHUNKS : c;
                        *reinterpret_cast<uint4*>(const_cast<unsigned char*>(swz(is_v ? v_tile : k_tile, row, chunk))) =
                            *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + chunk * 8);
                    }
                    consumer_sync();
                }
                if (key_base + warp * 16 <= pos && key_base + warp * 16 + 15 >= lo)
                    attend_slice(q_tile, k_tile, v_tile, warp * 16, key_base, scale_log2, row_pos, row_lo, m, l, o);
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);
            }
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
                l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
            }
        }
        // the four warps meet: merge[warp][row < group][D + 2] (a block without tiles brings nothing)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int row = (lane >> 2) + rr * 8;
            if (row < group) {
                float* dst = merge + (warp * group + row) * MS;
#pragma unroll
                for (int dt = 0; dt < D / 8; ++dt) {
                    dst[dt * 8 + (lane & 3) * 2] = o[dt][2 * rr];
                    dst[dt * 8 + (lane & 3) * 2 + 1] = o[dt][2 * rr + 1];
                }
                if ((lane & 3) == 0) {
                    dst[D] = m[rr];
                    dst[D + 1] = l[rr];
                }
            }
        }
        consumer_sync();                                        // also: nobody reads the queries any more
        for (int i = threadIdx.x; i < group * (D / 4); i += CONSUMERS) {
            const int row = i / (D / 4), d = (i - row * (D / 4)) * 4;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[(w * group + row) * MS + D]);
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float ll = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float* src = merge + (w * group + row) * MS;
                const float c = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
                const float2 lo2 = *reinterpret_cast<const float2*>(src + d), hi2 = *reinterpret_cast<const float2*>(src + d + 2);
                acc.x += lo2.x * c; acc.y += lo2.y * c; acc.z += hi2.x * c; acc.w += hi2.y * c;
                ll += src[D + 1] * c;
            }
            if (pieces == 1) {
                const float inv = ll > 0.f ? 1.f / ll : 0.f;
                __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                uint2 packed;
                packed.x = *reinterpret_cast<unsigned*>(&lo2);
                packed.y = *reinterpret_cast<unsigned*>(&hi2);
                *reinterpret_cast<uint2*>(out + ((size_t)q_row * heads + kvh * group + row) * D + d) = packed;
            } else {
                *reinterpret_cast<float4*>(piece + row * PS + d) = acc;
                if (d == 0) *reinterpret_cast<float2*>(piece + row * PS + D) = make_float2(mm, ll);
            }
        }
    }
    if (pieces > 1) {
        cluster_sync_all();                                     // every block's piece is in its shared memory
        if (rank == 0 && warp < 4) {
            for (int i = threadIdx.x; i < group * (D / 4); i += CONSUMERS) {
                const int row = i / (D / 4), d = (i - row * (D / 4)) * 4;
                // four pieces a round, all of a round's loads requested before any is used; the
                // running maximum rescales what the rounds before have added
                float mm = -INFINITY, ll = 0.f;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (unsigned p0 = 0; p0 < pieces; p0 += 4) {
                    float2 ml[4];
                    float4 po[4];
#pragma unroll
                    for (unsigned k = 0; k < 4; ++k) {
                        ml[k] = make_float2(-INFINITY, 0.f);
                        po[k] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (p0 + k < pieces) {
                            ml[k] = cluster_load2(cluster_address(piece + row * PS + D, p0 + k));
                            po[k] = cluster_load4(cluster_address(piece + row * PS + d, p0 + k));
                        }
                    }
                    float round_max = mm;
#pragma unroll
                    for (unsigned k = 0; k < 4; ++k) round_max = fmaxf(round_max, ml[k].x);
                    const float keep = (mm == -INFINITY) ? 0.f : exp2f(mm - round_max);
                    acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
                    ll *= keep;
                    mm = round_max;
#pragma unroll
                    for (unsigned k = 0; k < 4; ++k) {
                        const float c = (ml[k].x == -INFINITY) ? 0.f : exp2f(ml[k].x - mm);
                        acc.x += po[k].x * c; acc.y += po[k].y * c; acc.z += po[k].z * c; acc.w += po[k].w * c;
                        ll += ml[k].y * c;
                    }
                }
                const float inv = ll > 0.f ? 1.f / ll : 0.f;
                __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                uint2 packed;
                packed.x = *reinterpret_cast<unsigned*>(&lo2);
                packed.y = *reinterpret_cast<unsigned*>(&hi2);
                *reinterpret_cast<uint2*>(out + ((size_t)q_row * heads + kvh * group + row) * D + d) = packed;
            }
        }
        cluster_sync_all();                                     // the pieces may go: the first block has read them
    }
    if (*(volatile int*)&aborted) {
        const long long start = clock64();
        while (clock64() - start < 4000000LL) __nanosleep(1000);
    }
}

// Three stages where two blocks of them fit a multiprocessor, else two.
int ring_for(int group) { return 2 * (tma_smem_bytes(3, group) + 1024) <= 227 * 1024 ? 3 : 2; }

template <int RING>
int configure(int group, int* per_sm) {
    const size_t smem = tma_smem_bytes(RING, group);
    static size_t allowed = 0;                   // the attribute is raised once per size, not per launch
    if (smem > allowed) {
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(decode_tma_kernel<RING>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "attn_decode_tma");
        allowed = smem;
    }
    if (per_sm)
        MRUN_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(per_sm, decode_tma_kernel<RING>, TMA_THREADS, smem),
                        "attn_decode_tma");
    return 0;
}

}  // namespace

#endif  // MRUN_DECODE_TMA

// 1 when this library holds the TMA decode kernel (head sizes 64 and 128).
MRUN_API int mrun_attn_decode_tma_available() { return MRUN_DECODE_TMA; }

// Blocks of the TMA decode kernel that fit on one multiprocessor with `group` query heads per kv
// head (for choosing the number of blocks of a launch); 0 when the kernel is not available.
MRUN_API int mrun_attn_decode_tma_occupancy(int group) {
#if MRUN_DECODE_TMA
    if (group < 1 || group > 16) return 0;
    int per_sm = 0;
    const int rc = ring_for(group) == 3 ? configure<3>(group, &per_sm) : configure<2>(group, &per_sm);
    return rc == 0 ? per_sm : 0;
#else
    (void)group;
    return 0;
#endif
}

#if MRUN_DECODE_TMA
namespace {
template <int RING>
int launch_cluster(const CUtensorMap& map_k, const CUtensorMap& map_v, const void* q, long q_stride, void* out,
                   const int* block_tables, int max_blocks, const int* token_slot, const int* positions, int tokens,
                   int cluster, int heads, int kv_heads, int page_size, float scale, int window, const FusedInput& in,
                   int* status, cudaStream_t stream) {
    const int group = heads / kv_heads;
    const size_t smem = tma_smem_bytes(RING, group);
    static size_t allowed = 0;
    if (smem > allowed) {
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(decode_cluster_kernel<RING>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "attn_decode_cluster");
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(decode_cluster_kernel<RING>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1),
                        "attn_decode_cluster");
        allowed = smem;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(cluster, tokens * kv_heads);
    config.blockDim = dim3(TMA_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = cluster;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    MRUN_CHECK_CUDA(cudaLaunchKernelEx(&config, decode_cluster_kernel<RING>, map_k, map_v, (const bf16*)q, q_stride, (bf16*)out,
                                       block_tables, max_blocks, token_slot, positions, heads, kv_heads, page_size,
                                       page_shift_of(page_size), scale * LOG2E, window, in, status),
                    "attn_decode_cluster");
    return 0;
}
}  // namespace
#endif

// The largest cluster (a power of two, at most 16) of the cluster decode kernel that the device
// takes with `group` query heads per kv head; 0 when the kernel is not available for the group.
MRUN_API int mrun_attn_decode_cluster_max(int group) {
#if MRUN_DECODE_TMA
    if (group < 1 || group > 8) return 0;
    return 16;
#else
    (void)group;
    return 0;
#endif
}

// Decode attention for steps with few (token, kv head) pairs: a thread-block cluster of `cluster`
// blocks (1, 2, 4, 8 or 16) takes one pair, cuts its tiles evenly among its blocks and merges
// through distributed shared memory: no plan, no scratch.  Other arguments as mrun_attn_decode_tma;
// at most 8 query heads per kv head.
MRUN_API int mrun_attn_decode_cluster(const void* q, long q_stride, void* out, void* k_cache, void* v_cache,
                                      const int* block_tables, int max_blocks, const int* token_slot,
                                      const int* positions, int tokens, int cluster, int heads, int kv_heads,
                                      int head_dim, int page_size, float scale, int window, int fused,
                                      const float* q_weight, const float* k_weight, float eps, const float* rot,
                                      int rotary_dim, const int* slots, const int* rows, long pages, int* status,
                                      cudaStream_t stream) {
#if MRUN_DECODE_TMA
    if (int rc = check_common("attn_decode_cluster", heads, kv_heads, head_dim, page_size, max_blocks, window, 8)) return rc;
    MRUN_REQUIRE(tokens >= 0 && (long)tokens * kv_heads <= 65535, "attn_decode_cluster: tokens=%d kv_heads=%d", tokens, kv_heads);
    MRUN_REQUIRE(cluster == 1 || cluster == 2 || cluster == 4 || cluster == 8 || cluster == 16,
                 "attn_decode_cluster: a cluster of %d blocks (1, 2, 4, 8 or 16)", cluster);
    MRUN_REQUIRE(status != nullptr, "attn_decode_cluster: the status word is required");
    MRUN_REQUIRE(page_shift_of(page_size) >= 0, "attn_decode_cluster: page_size=%d is not a power of two", page_size);
    MRUN_REQUIRE(pages > 0 && pages < (1L << 31), "attn_decode_cluster: pages=%ld", pages);
    MRUN_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)q & 15) == 0 &&
                 q_stride % 8 == 0, "attn_decode_cluster: q and the caches must be 16-byte aligned, q_stride a multiple of 8");
    MRUN_REQUIRE(!fused || (rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0),
                 "attn_decode_cluster: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
    MRUN_REQUIRE(!fused || (q_weight == nullptr) == (k_weight == nullptr),
                 "attn_decode_cluster: q and k norm weights come together");
    MRUN_REQUIRE(!fused || q_stride >= (long)(heads + 2 * kv_heads) * head_dim,
                 "attn_decode_cluster: the raw rows must hold q, k and v (stride %ld)", q_stride);
    MRUN_REQUIRE(!(fused && rows), "attn_decode_cluster: a selection of rows does not go with raw q, k, v input");
    if (tokens == 0) return 0;
    const int group = heads / kv_heads;
    CUtensorMap map_k, map_v;
    const int box_rows = page_size < BLOCK_N ? page_size : BLOCK_N;
    if (int rc = paged_cache_map(&map_k, k_cache, pages, kv_heads, page_size, D, box_rows, "attn_decode_cluster")) return rc;
    if (int rc = paged_cache_map(&map_v, v_cache, pages, kv_heads, page_size, D, box_rows, "attn_decode_cluster")) return rc;
    FusedInput in = {};
    if (fused) {
        in.enabled = 1;
        in.q_weight = q_weight;
        in.k_weight = k_weight;
        in.eps = eps;
        in.rot = (const float2*)rot;
        in.rotary_dim = rot ? rotary_dim : 0;
        in.slots = slots;
        in.k_cache = (bf16*)k_cache;
        in.v_cache = (bf16*)v_cache;
    }
    in.rows = rows;
    if (ring_for(group) == 3)
        return launch_cluster<3>(map_k, map_v, q, q_stride, out, block_tables, max_blocks, token_slot, positions, tokens,
                                 cluster, heads, kv_heads, page_size, scale, window, in, status, stream);
    return launch_cluster<2>(map_k, map_v, q, q_stride, out, block_tables, max_blocks, token_slot, positions, tokens, cluster,
                             heads, kv_heads, page_size, scale, window, in, status, stream);
#else
    return mrun_set_error("attn_decode_cluster: not built for head_dim=%d (head sizes 64 and 128 only)", MRUN_HEAD_DIM);
#endif
}

// As mrun_attn_decode, with a page size that is a power of two, `pages` the number of pages of the
// two cache tensors, `rows` null or, for each of the `tokens` tokens (whose positions and state
// slots the arrays of that length give), the row of q and of out it stands for, and `status` one int on the device, zero before the first call; a non-zero
// value afterwards names the role whose wait ran out (1 producer, 2 consumers) and the outputs of
// that launch are void.
MRUN_API int mrun_attn_decode_tma(const void* q, long q_stride, void* out, void* k_cache, void* v_cache,
                                  const int* block_tables, int max_blocks, const int* token_slot,
                                  const int* positions, const int* tile_prefix, const int* assignment, int tokens,
                                  float* part_o, float* part_ml, int* counters, int blocks, int heads, int kv_heads,
                                  int head_dim, int page_size, float scale, int window, int fused,
                                  const float* q_weight, const float* k_weight, float eps, const float* rot,
                                  int rotary_dim, const int* slots, const int* rows, long pages, int* status,
                                  cudaStream_t stream) {
#if MRUN_DECODE_TMA
    if (int rc = check_common("attn_decode_tma", heads, kv_heads, head_dim, page_size, max_blocks, window, 16)) return rc;
    MRUN_REQUIRE(tokens >= 0 && blocks >= 1 && blocks <= 65535, "attn_decode_tma: tokens=%d blocks=%d", tokens, blocks);
    MRUN_REQUIRE(tile_prefix && assignment && part_o && part_ml && counters && status,
                 "attn_decode_tma: the plan, the scratch and the status word are required");
    MRUN_REQUIRE(page_shift_of(page_size) >= 0, "attn_decode_tma: page_size=%d is not a power of two", page_size);
    MRUN_REQUIRE(pages > 0 && pages < (1L << 31), "attn_decode_tma: pages=%ld", pages);
    MRUN_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && ((uintptr_t)q & 15) == 0 &&
                 q_stride % 8 == 0, "attn_decode_tma: q and the caches must be 16-byte aligned, q_stride a multiple of 8");
    MRUN_REQUIRE(!fused || (rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0),
                 "attn_decode_tma: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
    MRUN_REQUIRE(!fused || (q_weight == nullptr) == (k_weight == nullptr),
                 "attn_decode_tma: q and k norm weights come together");
    MRUN_REQUIRE(!fused || q_stride >= (long)(heads + 2 * kv_heads) * head_dim,
                 "attn_decode_tma: the raw rows must hold q, k and v (stride %ld)", q_stride);
    MRUN_REQUIRE(!(fused && rows), "attn_decode_tma: a selection of rows does not go with raw q, k, v input");
    if (tokens == 0) return 0;
    const int group = heads / kv_heads;
    const int ring = ring_for(group);
    if (int rc = ring == 3 ? configure<3>(group, nullptr) : configure<2>(group, nullptr)) return rc;
    CUtensorMap map_k, map_v;
    const int box_rows = page_size < BLOCK_N ? page_size : BLOCK_N;
    if (int rc = paged_cache_map(&map_k, k_cache, pages, kv_heads, page_size, D, box_rows, "attn_decode_tma")) return rc;
    if (int rc = paged_cache_map(&map_v, v_cache, pages, kv_heads, page_size, D, box_rows, "attn_decode_tma")) return rc;
    FusedInput in = {};
    if (fused) {
        in.enabled = 1;
        in.q_weight = q_weight;
        in.k_weight = k_weight;
        in.eps = eps;
        in.rot = (const float2*)rot;
        in.rotary_dim = rot ? rotary_dim : 0;
        in.slots = slots;
        in.k_cache = (bf16*)k_cache;
        in.v_cache = (bf16*)v_cache;
    }
    in.rows = rows;
    const size_t smem = tma_smem_bytes(ring, group);
    if (ring == 3)
        decode_tma_kernel<3><<<dim3(blocks), TMA_THREADS, smem, stream>>>(
            map_k, map_v, (const bf16*)q, q_stride, (bf16*)out, block_tables, max_blocks, token_slot, positions,
            tile_prefix, (const int4*)assignment, tokens, part_o, part_ml, counters, heads, kv_heads, page_size,
            page_shift_of(page_size), scale * LOG2E, window, in, status);
    else
        decode_tma_kernel<2><<<dim3(blocks), TMA_THREADS, smem, stream>>>(
            map_k, map_v, (const bf16*)q, q_stride, (bf16*)out, block_tables, max_blocks, token_slot, positions,
            tile_prefix, (const int4*)assignment, tokens, part_o, part_ml, counters, heads, kv_heads, page_size,
            page_shift_of(page_size), scale * LOG2E, window, in, status);
    MRUN_CHECK_LAUNCH("attn_decode_tma");
    return 0;
#else
    return mrun_set_error("attn_decode_tma: not built for head_dim=%d (head sizes 64 and 128 only)", MRUN_HEAD_DIM);
#endif
}
