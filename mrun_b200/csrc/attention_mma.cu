// Paged grouped-query attention on the tensor cores (bf16 operands, 32-bit accumulation and
// softmax), compiled for one head size: -DMRUN_HEAD_DIM=<multiple of 16, at most 256>.
//
// Two kernels share the tile loader and the fragment code:
//
//  * prefill: one block per (tile of query tokens, kv head).  The tile's rows are (token, query
//    head of the kv head's group) pairs, 64 rows, so a key/value tile read once serves the whole
//    group.  Keys are consumed 64 at a time in position order with an online softmax.
//  * decode: the 64-key tiles of all (token, kv head) pairs are dealt evenly to the blocks.  The
//    rows are the group's query heads of one token (at most 16); the four warps take different
//    16-key slices of each tile and are merged at the end; a pair whose tiles fell to several
//    blocks is merged by the block that finishes last, through scratch memory (32-bit partial
//    outputs with their running max and sum).
//
// Both read keys and values from the pages (cache[page, kv_head, offset, :]) through the block
// table of the token's state slot.  A token at position p sees keys lo..p, lo = 0 or
// p - window + 1.  Keys outside that range, and pages that were given back, are never
// dereferenced: their tile rows are zero-filled.
//
// Math as in the CUDA-core kernel: s = scale * q·k, softmax in 32-bit, o = p·v
// (crates/mrun-engine/src/models/common.rs:129,199-205).  P is rounded to bf16 for the second
// product, as the tensor cores take bf16 operands.
#include <mma.h>

#include "attention_frag.cuh"

namespace {

// Loads keys key0 .. key0+63 of one kv head into a key tile and a value tile, both [64][LD].
// Rows whose key lies outside [lo, hi] or whose page is not held are zero-filled.  A row's place
// in the cache is worked out once and used for both tensors.  `page_shift` is log2(page_size)
// when the page size is a power of two (shift and mask instead of a division), else -1.
__device__ __forceinline__ void load_kv_tiles(bf16* k_tile, bf16* v_tile, const bf16* __restrict__ k_cache,
                                              const bf16* __restrict__ v_cache, const Paging& pg, int key0,
                                              int lo, int hi) {
    if constexpr (THREADS % CHUNKS == 0) {
        // a thread keeps its 16-byte column and walks down the rows
        constexpr int STEP = THREADS / CHUNKS;
        const int chunk = threadIdx.x % CHUNKS, r0 = threadIdx.x / CHUNKS;
#pragma unroll
        for (int row = r0; row < BLOCK_N; row += STEP) {
            const int key = key0 + row;
            bool valid = key >= lo && key <= hi;
            const long at = cache_row<D>(pg, key, valid) + chunk * 8;
            cp_async_16(k_tile + row * LD + chunk * 8, valid ? k_cache + at : k_cache, valid);
            cp_async_16(v_tile + row * LD + chunk * 8, valid ? v_cache + at : v_cache, valid);
        }
    } else {
        for (int c = threadIdx.x; c < BLOCK_N * CHUNKS; c += THREADS) {
            const int row = c / CHUNKS, chunk = c - row * CHUNKS;
            const int key = key0 + row;
            bool valid = key >= lo && key <= hi;
            const long at = cache_row<D>(pg, key, valid) + chunk * 8;
            cp_async_16(k_tile + row * LD + chunk * 8, valid ? k_cache + at : k_cache, valid);
            cp_async_16(v_tile + row * LD + chunk * 8, valid ? v_cache + at : v_cache, valid);
        }
    }
}

// One 16-row warp tile against `n_keys` (a multiple of 16) keys of a K tile and V tile starting
// at tile row `krow0`: scores, mask, online softmax update, and o += p·v.
//   q_tile: the warp's 16 rows [16][LD] in smem.   row_pos/row_lo: visible key range of the
//   thread's two rows (row g and g + 8); row_pos < 0 marks a padding row.
template <int N_KEYS>
__device__ __forceinline__ void attend_tile(const bf16* q_tile, const bf16* k_tile, const bf16* v_tile,
                                            int krow0, int key_base, float scale_log2, bool need_mask,
                                            const int (&row_pos)[2], const int (&row_lo)[2],
                                            float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
    constexpr int NT = N_KEYS / 8;     // score n-tiles
    const int lane = threadIdx.x & 31;
    float s[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;

#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a[4];
        ldmatrix_x4(a, q_tile + ((lane & 7) + ((lane >> 3) & 1) * 8) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            unsigned b[4];
            ldmatrix_x4(b, k_tile + (krow0 + nt * 8 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[nt], a, b[0], b[1]);
            mma_bf16(s[nt + 1], a, b[2], b[3]);
        }
    }

    // scale, mask, row maxima
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            float v = s[nt][e] * scale_log2;
            if (need_mask) {
                const int key = key_base + krow0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                if (key > row_pos[r] || key < row_lo[r]) v = -INFINITY;
            }
            s[nt][e] = v;
            mx[r] = fmaxf(mx[r], v);
        }
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
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const float p = (m[r] == -INFINITY) ? 0.f : exp2f(s[nt][e] - m[r]);
            s[nt][e] = p;
            sum[r] += p;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) l[r] = l[r] * corr[r] + sum[r];   // per-thread partial; reduced at the end
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }

    // o += p · v
#pragma unroll
    for (int kk = 0; kk < N_KEYS / 16; ++kk) {
        unsigned a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < D / 8; dt += 2) {
            unsigned b[4];
            ldmatrix_x4_trans(b, v_tile + (krow0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dt * 8 + (lane >> 4) * 8);
            mma_bf16(o[dt], a, b[0], b[1]);
            mma_bf16(o[dt + 1], a, b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Prefill: 64 rows = tokens_per_tile tokens x group heads.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
prefill_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out,
               const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
               const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ token_slot,
               const int* __restrict__ positions, const int* __restrict__ tile_tok0,
               const int* __restrict__ tile_ntok, int heads, int kv_heads, int page_size, int page_shift,
               float scale_log2, int window) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);           // [64][LD]
    bf16* k_tiles = q_tile + 64 * LD;                           // [2][64][LD]
    bf16* v_tiles = k_tiles + 2 * BLOCK_N * LD;                 // [2][64][LD]

    const int tile = blockIdx.y, kvh = blockIdx.x;      // the list's first tile (the longest, the host sorts) for every kv head first
    const int group = heads / kv_heads;
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* table = block_tables + (size_t)token_slot[tok0] * max_blocks;
    const int n_rows = ntok * group;

    // tokens of a tile are consecutive positions of one request
    const int pos_first = positions[tok0], pos_last = pos_first + ntok - 1;
    const int lo_tile = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
    const int first_block = lo_tile / BLOCK_N, last_block = pos_last / BLOCK_N;

    // q rows: row r = (token r / group, head kvh * group + r % group)
    for (int c = threadIdx.x; c < 64 * CHUNKS; c += THREADS) {
        const int row = c / CHUNKS, chunk = c - row * CHUNKS;
        const bool valid = row < n_rows;
        const bf16* src = q;
        if (valid)
            src = q + (size_t)(tok0 + row / group) * q_stride + (size_t)(kvh * group + row % group) * D + chunk * 8;
        cp_async_16(q_tile + row * LD + chunk * 8, src, valid);
    }
    const Paging pg{table, kv_heads, kvh, page_size, page_shift};
    load_kv_tiles(k_tiles, v_tiles, k_cache, v_cache, pg, first_block * BLOCK_N, lo_tile, pos_last);
    cp_async_commit();

    int row_pos[2], row_lo[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        row_pos[r] = row < n_rows ? pos_first + row / group : -1;
        row_lo[r] = (window > 0 && row_pos[r] - window + 1 > 0) ? row_pos[r] - window + 1 : 0;
    }
    // the warp's rows span tokens [w_first, w_last]: blocks above w_last's position are skipped
    const int w_row0 = warp * 16;
    const bool warp_active = w_row0 < n_rows;
    const int w_pos_last = pos_first + (min(w_row0 + 15, n_rows - 1)) / group;
    const int w_pos_first = pos_first + w_row0 / group;

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

    for (int block = first_block; block <= last_block; ++block) {
        const int stage = (block - first_block) & 1;
        if (block < last_block) {
            load_kv_tiles(k_tiles + (stage ^ 1) * BLOCK_N * LD, v_tiles + (stage ^ 1) * BLOCK_N * LD, k_cache, v_cache,
                          pg, (block + 1) * BLOCK_N, lo_tile, pos_last);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key_base = block * BLOCK_N;
        if (warp_active && key_base <= w_pos_last) {
            const int w_lo = (window > 0 && w_pos_first - window + 1 > 0) ? w_pos_first - window + 1 : 0;
            if (key_base + BLOCK_N - 1 >= w_lo) {
                // full visibility for every row of the warp needs no mask
                const int w_lo_last = (window > 0 && w_pos_last - window + 1 > 0) ? w_pos_last - window + 1 : 0;
                const bool need_mask = key_base + BLOCK_N - 1 > w_pos_first || key_base < w_lo_last;
                attend_tile<BLOCK_N>(q_tile + w_row0 * LD, k_tiles + stage * BLOCK_N * LD,
                                     v_tiles + stage * BLOCK_N * LD, 0, key_base, scale_log2, need_mask, row_pos,
                                     row_lo, m, l, o);
            }
        }
        __syncthreads();
    }

    // finish the row sums over the quad, normalise, stage through q_tile, write coalesced
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    const float inv0 = l[0] > 0.f ? 1.f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.f / l[1] : 0.f;
    bf16* stage_rows = q_tile + w_row0 * LD;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        const int col = dt * 8 + (lane & 3) * 2;
        *reinterpret_cast<unsigned*>(stage_rows + (lane >> 2) * LD + col) = pack_bf16(o[dt][0] * inv0, o[dt][1] * inv0);
        *reinterpret_cast<unsigned*>(stage_rows + ((lane >> 2) + 8) * LD + col) = pack_bf16(o[dt][2] * inv1, o[dt][3] * inv1);
    }
    __syncthreads();
    for (int c = threadIdx.x; c < n_rows * CHUNKS; c += THREADS) {
        const int row = c / CHUNKS, chunk = c - row * CHUNKS;
        bf16* dst = out + ((size_t)(tok0 + row / group) * heads + kvh * group + row % group) * D + chunk * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(q_tile + row * LD + chunk * 8);
    }
}

// ------------------------------------------------------------------------------------------
// Decode: 16 rows = the group's heads of one token.
//
// The work of a step is the list of 64-key tiles of every (token, kv head) pair, numbered kv head
// by kv head and token by token.  Block b takes tiles [b * per, (b + 1) * per): every block streams
// the same number of keys whatever the mix of context lengths, and a step of more pairs than the
// device holds blocks does not run as one full round of blocks and a nearly empty one.  A
// block's range is a sequence of segments, each a run of tiles of one pair; only its first and
// its last segment can be part of a pair.  A partial segment writes its unnormalised 32-bit
// result and its running (max, sum) to scratch (slot 0 if it is the block's first segment, else
// slot 1): part_o [blocks, 2, 16, D], part_ml [blocks, 2, 16, 2].  The block that arrives last at
// the pair's counter merges the pair's pieces in block order and sets the counter back to zero,
// so no second kernel runs and the result does not depend on which block came last.
// ------------------------------------------------------------------------------------------
constexpr int STAGES = 2;      // key/value tiles in flight: three resident blocks with two tiles each beat deeper pipelines

// Sum and maximum over the block's 1024 threads; every thread gets the result.
__device__ __forceinline__ int plan_reduce(int v, bool take_max, int* scratch) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const int other = __shfl_xor_sync(0xffffffffu, v, off);
        v = take_max ? max(v, other) : v + other;
    }
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        v = scratch[threadIdx.x];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const int other = __shfl_xor_sync(0xffffffffu, v, off);
            v = take_max ? max(v, other) : v + other;
        }
        if (threadIdx.x == 0) scratch[32] = v;
    }
    __syncthreads();
    v = scratch[32];
    __syncthreads();
    return v;
}

// prefix[0] = 0, prefix[t + 1] = value(0) + .. + value(t) for t < tokens.  One block of 1024 threads.
template <typename F>
__device__ __forceinline__ void plan_prefix(F value, int tokens, int* __restrict__ prefix, int* scan, int* carry) {
    if (threadIdx.x == 0) {
        *carry = 0;
        prefix[0] = 0;
    }
    __syncthreads();
    for (int base = 0; base < tokens; base += 1024) {
        const int t = base + threadIdx.x;
        scan[threadIdx.x] = t < tokens ? value(t) : 0;
        __syncthreads();
        for (int step = 1; step < 1024; step <<= 1) {            // inclusive scan of the chunk
            const int add = threadIdx.x >= step ? scan[threadIdx.x - step] : 0;
            __syncthreads();
            scan[threadIdx.x] += add;
            __syncthreads();
        }
        if (t < tokens) prefix[t + 1] = *carry + scan[threadIdx.x];
        __syncthreads();
        if (threadIdx.x == 1023) *carry += scan[1023];
        __syncthreads();
    }
}

// The plan of a decode step: tile_prefix[t] = number of 64-key tiles of tokens 0 .. t-1 (a
// padding token has none), so tile_prefix[tokens] is the step's total per kv head.  One block.
//
// blocks_per_head > 0 (steps with few pairs, every block stays with one pair): the step's tiles
// per block `per` is the smallest number, at least min_tiles, with which the pairs of one kv head
// need no more than blocks_per_head blocks and no pair more than max_pieces: a long context gets
// many blocks and a short one a single block, and the longest run of tiles any block streams is as
// short as the launch allows.  Then tile_prefix[tokens + 1 + t] = blocks of tokens 0 .. t-1 and
// tile_prefix[2 * (tokens + 1)] = per.
__global__ void decode_plan_kernel(const int* __restrict__ positions, int tokens, int window,
                                   int* __restrict__ tile_prefix, int blocks_per_head, int min_tiles,
                                   int max_pieces) {
    __shared__ int carry;
    __shared__ int scan[1024];
    __shared__ int scratch[33];
    plan_prefix([&](int t) {
        const int pos = positions[t];
        if (pos < 0) return 0;
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        return pos / BLOCK_N - lo / BLOCK_N + 1;
    }, tokens, tile_prefix, scan, &carry);
    if (blocks_per_head <= 0) return;
    int longest = 0;
    for (int t = threadIdx.x; t < tokens; t += 1024) longest = max(longest, tile_prefix[t + 1] - tile_prefix[t]);
    longest = plan_reduce(longest, true, scratch);
    int lo = max(min_tiles, (longest + max_pieces - 1) / max_pieces);
    int hi = max(lo, longest);                 // with `longest` tiles a block every pair takes one block
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        int need = 0;
        for (int t = threadIdx.x; t < tokens; t += 1024)
            need += (tile_prefix[t + 1] - tile_prefix[t] + mid - 1) / mid;
        need = plan_reduce(need, false, scratch);
        if (need <= blocks_per_head) hi = mid; else lo = mid + 1;
    }
    const int per = lo;
    int* block_prefix = tile_prefix + tokens + 1;
    plan_prefix([&](int t) { return (tile_prefix[t + 1] - tile_prefix[t] + per - 1) / per; }, tokens, block_prefix,
                scan, &carry);
    if (threadIdx.x == 0) block_prefix[tokens + 1] = per;
}

// What block b of the decode kernel starts with, so that it needs one load and no search:
// {first tile, end tile, kv head, token} and {tiles per kv head, tiles per block, blocks per kv head, -}.
//
// Two ways of dealing the tiles.  blocks_per_head == 0, for steps with more (token, kv head)
// pairs than blocks: block b takes tiles [b * per, (b + 1) * per) of the flat list, across pairs.
// blocks_per_head > 0, for steps with few pairs: block i of a kv head belongs to the token whose
// run of blocks (the plan's second prefix) holds i and takes that pair's next `per` tiles, so
// that no block pays the start-up of two pairs for a handful of tiles.
__global__ void decode_assign_kernel(const int* __restrict__ tile_prefix, int tokens, int kv_heads, int blocks,
                                     int min_tiles, int blocks_per_head, int4* __restrict__ assignment) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const int tiles_per_head = tile_prefix[tokens];
    const int total = tiles_per_head * kv_heads;
    int u0 = 0, u1 = 0, kvh = 0, tok = 0, per = 0;
    if (blocks_per_head > 0) {
        const int* block_prefix = tile_prefix + tokens + 1;
        per = block_prefix[tokens + 1];
        kvh = b / blocks_per_head;
        const int i = b - kvh * blocks_per_head;
        if (kvh < kv_heads && i < block_prefix[tokens]) {
            int lo_t = 0, hi_t = tokens - 1;                          // the last token t with block_prefix[t] <= i
            while (lo_t < hi_t) {
                const int mid = (lo_t + hi_t + 1) >> 1;
                if (block_prefix[mid] <= i) lo_t = mid; else hi_t = mid - 1;
            }
            tok = lo_t;
            const int pair_tiles = tile_prefix[tok + 1] - tile_prefix[tok];
            const int j0 = (i - block_prefix[tok]) * per;
            u0 = kvh * tiles_per_head + tile_prefix[tok] + j0;
            u1 = u0 + min(per, pair_tiles - j0);
        }
    } else {
        per = max((total + blocks - 1) / blocks, min_tiles);
        u0 = min(total, b * per);
        u1 = min(total, u0 + per);
        if (u0 < u1) {
            kvh = u0 / tiles_per_head;
            const int r = u0 - kvh * tiles_per_head;
            int lo_t = 0, hi_t = tokens - 1;                      // the last token t with prefix[t] <= r
            while (lo_t < hi_t) {
                const int mid = (lo_t + hi_t + 1) >> 1;
                if (tile_prefix[mid] <= r) lo_t = mid; else hi_t = mid - 1;
            }
            tok = lo_t;
        }
    }
    assignment[2 * b] = make_int4(u0, u1, kvh, tok);
    assignment[2 * b + 1] = make_int4(tiles_per_head, per, blocks_per_head, 0);
}

// grid: `blocks` blocks, the number the plan was made for.
// part_o: [blocks][2][16][D] floats, part_ml: [blocks][2][16][2] floats, counters: [tokens * kv_heads]
// ints, zero before the call and zero again after it.
__global__ void __launch_bounds__(THREADS)
decode_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out,
              const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
              const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ token_slot,
              const int* __restrict__ positions, const int* __restrict__ tile_prefix,
              const int4* __restrict__ assignment, int tokens, float* __restrict__ part_o,
              float* __restrict__ part_ml, int* __restrict__ counters, int heads, int kv_heads, int page_size,
              int page_shift, float scale_log2, int window, const FusedInput fused) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* q_tile = reinterpret_cast<bf16*>(smem_raw);           // [16][LD]
    bf16* k_tiles = q_tile + 16 * LD;                           // [STAGES][64][LD]
    bf16* v_tiles = k_tiles + STAGES * BLOCK_N * LD;            // [STAGES][64][LD]
    float* merge = reinterpret_cast<float*>(k_tiles);           // reused after a segment's loop
    __shared__ int ticket_shared;
    __shared__ __align__(16) bf16 new_k[D], new_v[D];           // this step's own key and value (fused input)
    // Staging of a head vector per warp (fused input).  It lives in the value tile of the last
    // stage, which no copy targets before the first tile of a segment has been consumed; shared
    // memory is what limits the blocks per SM, and a static array here costs one of three.
    float (*head_vec)[D] = reinterpret_cast<float (*)[D]>(v_tiles + (STAGES - 1) * BLOCK_N * LD);
    constexpr int MS = D + 2;

    const int block_id = blockIdx.x, n_blocks_grid = gridDim.x;
    const int group = heads / kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int4 mine = assignment[2 * block_id], shape = assignment[2 * block_id + 1];
    int u = mine.x;
    const int u_end = mine.y;
    const int tiles_per_head = shape.x, per = shape.y, splits = shape.z;
    const int* prefix = tile_prefix;
    int kvh = mine.z, tok = mine.w;                             // the pair of the block's first tile

    // padding rows come out as zeros
    for (int t = block_id; t < tokens; t += n_blocks_grid)
        if (positions[t] < 0)
            for (int i = threadIdx.x; i < heads * D; i += THREADS) out[(size_t)t * heads * D + i] = __float2bfloat16_rn(0.f);

    for (int seg = 0; u < u_end; ++seg) {
        // ---------------------------------------------------------------- which pair, which tiles
        // after the first segment the next pair follows: the next token with tiles, or the first
        // one of the next kv head
        if (seg > 0) {
            ++tok;
            if (u - kvh * tiles_per_head >= tiles_per_head) {
                ++kvh;
                tok = 0;
            }
        }
        const int r = u - kvh * tiles_per_head;
        while (prefix[tok + 1] <= r) ++tok;                      // skip tokens without tiles (padding)
        const int pair_tiles = prefix[tok + 1] - prefix[tok];
        const int j0 = r - prefix[tok];
        const int len = min(u_end - u, pair_tiles - j0);
        const bool complete = j0 == 0 && len == pair_tiles;
        const int pair_start = kvh * tiles_per_head + prefix[tok];

        const int pos = positions[tok];
        const Paging pg{block_tables + (size_t)token_slot[tok] * max_blocks, kv_heads, kvh, page_size, page_shift};
        const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        const int b1 = pos / BLOCK_N;
        const int first_block = lo / BLOCK_N + j0;
        const int last_block = first_block + len - 1;

        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        float o[D / 8][4];
#pragma unroll
        for (int dt = 0; dt < D / 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;

        // prologue: STAGES - 1 tiles in flight (an empty group keeps the counting uniform)
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (first_block + s <= last_block)
                load_kv_tiles(k_tiles + s * BLOCK_N * LD, v_tiles + s * BLOCK_N * LD, k_cache, v_cache, pg,
                              (first_block + s) * BLOCK_N, lo, pos);
            cp_async_commit();
        }
        // q with plain loads, so that the copy groups above stay one per tile; the first barrier of
        // the loop publishes it
        const bool owns_new_token = fused.enabled && last_block == b1;
        if (!fused.enabled) {
            for (int c = threadIdx.x; c < 16 * CHUNKS; c += THREADS) {
                const int row = c / CHUNKS, chunk = c - row * CHUNKS;
                uint4 value = make_uint4(0, 0, 0, 0);
                if (row < group)
                    value = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (size_t)(kvh * group + row) * D + chunk * 8);
                *reinterpret_cast<uint4*>(q_tile + row * LD + chunk * 8) = value;
            }
        } else {
            // q, k and v arrive raw: [q heads | k heads | v heads] of D elements each in the token's row
            const bf16* token_row = q + (size_t)tok * q_stride;
            const float2* cs = fused.rot ? fused.rot + (size_t)tok * (fused.rotary_dim >> 1) : nullptr;
            for (int row = warp; row < 16; row += THREADS / 32) {
                if (row < group)
                    norm_rotate_head(token_row + (size_t)(kvh * group + row) * D, fused.q_weight, fused.eps, cs,
                                     fused.rotary_dim, head_vec[warp], q_tile + row * LD);
                else
                    for (int e = lane; e < D; e += 32) q_tile[row * LD + e] = __float2bfloat16_rn(0.f);
            }
            if (owns_new_token) {
                // the block that holds the pair's last tile makes the token's own key and value: into
                // the page for later steps, and into shared memory for this one
                if (warp == 0)
                    norm_rotate_head(token_row + (size_t)(heads + kvh) * D, fused.k_weight, fused.eps, cs,
                                     fused.rotary_dim, head_vec[0], new_k);
                if (warp == 1)
                    for (int e = lane; e < D; e += 32) new_v[e] = token_row[(size_t)(heads + kv_heads + kvh) * D + e];
                __syncthreads();
                const int slot = fused.slots ? fused.slots[tok] : -1;
                if (slot >= 0) {
                    const int page = slot / page_size, off = slot - page * page_size;
                    const size_t at = (((size_t)page * kv_heads + kvh) * page_size + off) * D;
                    for (int c = threadIdx.x; c < 2 * CHUNKS; c += THREADS) {
                        const bool is_v = c >= CHUNKS;
                        const int chunk = is_v ? c - CHUNKS : c;
                        *reinterpret_cast<uint4*>((is_v ? fused.v_cache : fused.k_cache) + at + chunk * 8) =
                            *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + chunk * 8);
                    }
                }
            }
        }

        int row_pos[2], row_lo[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int row = (lane >> 2) + rr * 8;
            row_pos[rr] = row < group ? pos : -1;
            row_lo[rr] = lo;
        }
        for (int block = first_block; block <= last_block; ++block) {
            const int it = block - first_block;
            cp_async_wait<STAGES - 2>();        // tile `it` has landed
            __syncthreads();                    // ... for every thread, and tile it-1 is no longer read
            const int ahead = block + STAGES - 1;
            if (ahead <= last_block) {
                const int s = (it + STAGES - 1) % STAGES;
                load_kv_tiles(k_tiles + s * BLOCK_N * LD, v_tiles + s * BLOCK_N * LD, k_cache, v_cache, pg,
                              ahead * BLOCK_N, lo, pos);
            }
            cp_async_commit();
            const int stage = it % STAGES;
            const int key_base = block * BLOCK_N;
            if (owns_new_token && block == b1) {
                // the page row of this step's token was not written when the tile was requested
                const int row = pos - key_base;
                for (int c = threadIdx.x; c < 2 * CHUNKS; c += THREADS) {
                    const bool is_v = c >= CHUNKS;
                    const int chunk = is_v ? c - CHUNKS : c;
                    *reinterpret_cast<uint4*>((is_v ? v_tiles : k_tiles) + (stage * BLOCK_N + row) * LD + chunk * 8) =
                        *reinterpret_cast<const uint4*>((is_v ? new_v : new_k) + chunk * 8);
                }
                __syncthreads();
            }
            // warp w takes keys 16w .. 16w+15 of the tile
            if (key_base + warp * 16 <= pos && key_base + warp * 16 + 15 >= lo)
                attend_tile<16>(q_tile, k_tiles + stage * BLOCK_N * LD, v_tiles + stage * BLOCK_N * LD, warp * 16,
                                key_base, scale_log2, true, row_pos, row_lo, m, l, o);
        }
        cp_async_wait<0>();
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
            l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
        }

        // merge the four warps: merge[warp][16 rows][D + 2]
        __syncthreads();
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int row = (lane >> 2) + rr * 8;
            float* dst = merge + (warp * 16 + row) * MS;
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
        __syncthreads();
        const size_t my_slot = (size_t)block_id * 2 + (seg == 0 ? 0 : 1);
        for (int i = threadIdx.x; i < group * D; i += THREADS) {
            const int row = i / D, d = i - row * D;
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mm = fmaxf(mm, merge[(w * 16 + row) * MS + D]);
            float acc = 0.f, ll = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float* src = merge + (w * 16 + row) * MS;
                const float c = (src[D] == -INFINITY) ? 0.f : exp2f(src[D] - mm);
                acc += src[d] * c;
                ll += src[D + 1] * c;
            }
            if (complete) {
                out[((size_t)tok * heads + kvh * group + row) * D + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
            } else {
                part_o[(my_slot * 16 + row) * D + d] = acc;
                if (d == 0) {
                    part_ml[(my_slot * 16 + row) * 2] = mm;
                    part_ml[(my_slot * 16 + row) * 2 + 1] = ll;
                }
            }
        }
        if (!complete) {
            // the blocks that share this pair are p_first .. p_last; the last to arrive merges their
            // pieces in block order
            int p_first, p_last;
            if (splits > 0) {            // the pair's own run of blocks: `splits` blocks a kv head
                p_first = kvh * splits + prefix[tokens + 1 + tok];
                p_last = p_first + (pair_tiles + per - 1) / per - 1;
            } else {
                p_first = pair_start / per;
                p_last = (pair_start + pair_tiles - 1) / per;
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) ticket_shared = atomicAdd(&counters[tok * kv_heads + kvh], 1);
            __syncthreads();
            if (ticket_shared == p_last - p_first) {
                __threadfence();
                // A thread takes four values of a row; the pieces are read four at a time, all loads
                // of a round requested before any is used.
                for (int i = threadIdx.x; i < group * (D / 4); i += THREADS) {
                    const int row = i / (D / 4), d = (i - row * (D / 4)) * 4;
                    // block p's piece of this pair is its first segment iff its range starts inside the pair
                    auto slot_of = [&](int p) -> size_t {
                        return (size_t)p * 2 + ((splits > 0 || p * per >= pair_start) ? 0 : 1);
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
                    *reinterpret_cast<uint2*>(out + ((size_t)tok * heads + kvh * group + row) * D + d) = packed;
                }
                if (threadIdx.x == 0) counters[tok * kv_heads + kvh] = 0;
            }
        }
        __syncthreads();            // the merge area and ticket_shared are reused by the next segment
        u += len;
    }
}

constexpr size_t PREFILL_SMEM = (size_t)(64 + 4 * BLOCK_N) * LD * sizeof(bf16);
constexpr size_t DECODE_SMEM = (size_t)(16 + 2 * STAGES * BLOCK_N) * LD * sizeof(bf16);
static_assert((size_t)4 * 16 * (D + 2) * sizeof(float) <= (size_t)2 * STAGES * BLOCK_N * LD * sizeof(bf16),
              "the warp merge area must fit in the key/value tiles");

}  // namespace

MRUN_API int mrun_attn_head_dim() { return D; }

// Tiles: tile i covers tokens tile_tok0[i] .. +tile_ntok[i]-1 (consecutive positions of one request,
// at most 64 / (heads / kv_heads) of them).
MRUN_API int mrun_attn_prefill(const void* q, long q_stride, void* out, const void* k_cache, const void* v_cache,
                               const int* block_tables, int max_blocks, const int* token_slot,
                               const int* positions, const int* tile_tok0, const int* tile_ntok, int n_tiles,
                               int heads, int kv_heads, int head_dim, int page_size, float scale, int window,
                               cudaStream_t stream) {
    if (int rc = check_common("attn_prefill", heads, kv_heads, head_dim, page_size, max_blocks, window, 64)) return rc;
    MRUN_REQUIRE(n_tiles >= 0, "attn_prefill: n_tiles=%d", n_tiles);
    if (n_tiles == 0) return 0;
    static bool configured = false;
    if (!configured) {
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)PREFILL_SMEM), "attn_prefill");
        configured = true;
    }
    for (int done = 0; done < n_tiles; done += 65535) {          // the grid's second dimension ends at 65535
        const int now = n_tiles - done < 65535 ? n_tiles - done : 65535;
        prefill_kernel<<<dim3(kv_heads, now), THREADS, PREFILL_SMEM, stream>>>(
            (const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks,
            token_slot, positions, tile_tok0 + done, tile_ntok + done, heads, kv_heads, page_size, page_shift_of(page_size),
            scale * LOG2E, window);
        MRUN_CHECK_LAUNCH("attn_prefill");
    }
    return 0;
}

// The plan of a decode step for a window (0 = none) and a launch of `blocks` blocks that take at
// least min_tiles tiles each: assignment gets 8 ints per block.
// splits == 0: the tiles of all pairs are dealt evenly across the blocks; tile_prefix gets
// tokens + 1 ints.  splits > 0: every block stays with one pair; each kv head has blocks / kv_heads
// blocks (a multiple, and at least `tokens`), dealt to its pairs by their length, at most `splits`
// to one pair; tile_prefix gets 2 * (tokens + 1) + 1 ints.  The plan is the same for every layer
// with that window and those sizes, so a step computes it once.
MRUN_API int mrun_attn_decode_plan(const int* positions, int tokens, int window, int kv_heads, int blocks,
                                   int min_tiles, int splits, int* tile_prefix, int* assignment,
                                   cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && window >= 0 && kv_heads >= 1 && blocks >= 1 && min_tiles >= 1 && splits >= 0,
                 "attn_decode_plan: tokens=%d window=%d kv_heads=%d blocks=%d min_tiles=%d splits=%d", tokens, window,
                 kv_heads, blocks, min_tiles, splits);
    MRUN_REQUIRE(splits == 0 || (blocks % kv_heads == 0 && blocks / kv_heads >= tokens),
                 "attn_decode_plan: blocks that stay with one pair need a multiple of kv_heads = %d blocks and at "
                 "least one for each of %d tokens a kv head, not %d", kv_heads, tokens, blocks);
    MRUN_REQUIRE(((uintptr_t)assignment & 15) == 0, "attn_decode_plan: the assignment must be 16-byte aligned");
    const int blocks_per_head = splits > 0 ? blocks / kv_heads : 0;
    decode_plan_kernel<<<1, 1024, 0, stream>>>(positions, tokens, window, tile_prefix, blocks_per_head, min_tiles,
                                               splits);
    MRUN_CHECK_LAUNCH("attn_decode_plan");
    decode_assign_kernel<<<(blocks + 127) / 128, 128, 0, stream>>>(tile_prefix, tokens, kv_heads, blocks, min_tiles,
                                                                  blocks_per_head, (int4*)assignment);
    MRUN_CHECK_LAUNCH("attn_decode_plan: assignment");
    return 0;
}

// Every token is a row of its own (positions[t] < 0 = padding, output zero).  tile_prefix and
// assignment: the plan from mrun_attn_decode_plan for the same positions, window, kv_heads and
// blocks.  blocks: how many blocks share the tiles (as many as the device holds at once is best).
// part_o and part_ml are scratch of blocks * 2 * 16 * (D and 2) floats; counters holds
// tokens * kv_heads ints that are zero before the call and zero again after it.  Calls that share
// scratch must not overlap on the device.
//
// fused != 0: `q` is the projection's raw output, rows of [heads | kv_heads | kv_heads] x D (q, k, v);
// the kernel norms q and k with q_weight / k_weight (null: no norm) and eps, rotates them with
// rot[token] (null: no rotation), writes the token's k and v to cache slot slots[token] (null or
// negative: no write) and attends over the cache plus that token.  fused == 0: q is ready and the
// cache holds the token already; the remaining fused arguments are ignored.
MRUN_API int mrun_attn_decode(const void* q, long q_stride, void* out, void* k_cache, void* v_cache,
                              const int* block_tables, int max_blocks, const int* token_slot,
                              const int* positions, const int* tile_prefix, const int* assignment, int tokens,
                              float* part_o, float* part_ml, int* counters, int blocks, int heads, int kv_heads,
                              int head_dim, int page_size, float scale, int window, int fused,
                              const float* q_weight, const float* k_weight, float eps, const float* rot,
                              int rotary_dim, const int* slots, cudaStream_t stream) {
    if (int rc = check_common("attn_decode", heads, kv_heads, head_dim, page_size, max_blocks, window, 16)) return rc;
    MRUN_REQUIRE(tokens >= 0 && blocks >= 1 && blocks <= 65535, "attn_decode: tokens=%d blocks=%d", tokens, blocks);
    MRUN_REQUIRE(tile_prefix && assignment && part_o && part_ml && counters,
                 "attn_decode: the plan and the scratch are required");
    MRUN_REQUIRE(!fused || (rotary_dim >= 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0),
                 "attn_decode: rotary_dim=%d must be even and at most head_dim=%d", rotary_dim, head_dim);
    MRUN_REQUIRE(!fused || (q_weight == nullptr) == (k_weight == nullptr),
                 "attn_decode: q and k norm weights come together");
    MRUN_REQUIRE(!fused || q_stride >= (long)(heads + 2 * kv_heads) * head_dim,
                 "attn_decode: the raw rows must hold q, k and v (stride %ld)", q_stride);
    if (tokens == 0) return 0;
    static bool configured = false;
    if (!configured) {
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)DECODE_SMEM), "attn_decode");
        configured = true;
    }
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
    MRUN_CHECK_CUDA(mrun::launch_kernel(decode_kernel, dim3(blocks), dim3(THREADS), DECODE_SMEM, stream,
                                     (const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
                                     block_tables, max_blocks, token_slot, positions, tile_prefix,
                                     (const int4*)assignment, tokens, part_o, part_ml, counters, heads, kv_heads,
                                     page_size, page_shift_of(page_size), scale * LOG2E, window, in),
                    "attn_decode");
    return 0;
}

// Blocks of the decode kernel that fit on one multiprocessor (for choosing the number of splits).
MRUN_API int mrun_attn_decode_occupancy() {
    int blocks = 0;
    cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, decode_kernel, THREADS, DECODE_SMEM) != cudaSuccess)
        return -1;
    return blocks;
}

// ------------------------------------------------------------------------------------------
// The same decode kernel for callers that cannot allocate: its scratch is a fixed array in this
// library (see attention_static.h for who needs that, the limits and the rules).
// ------------------------------------------------------------------------------------------
#include "attention_static.h"

#include <mutex>

namespace {

constexpr size_t STATIC_PART_O = (size_t)MRUN_STATIC_MAX_BLOCKS * 2 * 16 * D;      // floats
constexpr size_t STATIC_PART_ML = (size_t)MRUN_STATIC_MAX_BLOCKS * 2 * 16 * 2;     // floats
constexpr size_t STATIC_COUNTERS = MRUN_STATIC_MAX_PAIRS;                          // ints, stored as 4-byte words
constexpr size_t STATIC_ASSIGNMENT = (size_t)MRUN_STATIC_MAX_BLOCKS * 8;            // ints, 16-byte aligned
constexpr size_t STATIC_PREFIX = MRUN_STATIC_MAX_TOKENS + 1;                       // ints

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_static_scratch[STATIC_PART_O + STATIC_PART_ML + STATIC_COUNTERS +
                                                        STATIC_ASSIGNMENT + STATIC_PREFIX];

constexpr int STATIC_MAX_DEVICES = 64;
float* g_static_address[STATIC_MAX_DEVICES] = {};
std::mutex g_static_mutex;

// The array's address on the current device, looked up at the first call on that device.
int static_scratch_address(float** address) {
    int device = -1;
    MRUN_CHECK_CUDA(cudaGetDevice(&device), "attn_decode_static");
    MRUN_REQUIRE(device >= 0 && device < STATIC_MAX_DEVICES, "attn_decode_static: device %d is outside 0..%d", device,
                 STATIC_MAX_DEVICES - 1);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (g_static_address[device] == nullptr) {
        float* found = nullptr;
        MRUN_CHECK_CUDA(cudaGetSymbolAddress((void**)&found, g_static_scratch), "attn_decode_static: scratch address");
        MRUN_REQUIRE(found != nullptr, "attn_decode_static: the scratch array has no address on device %d", device);
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)DECODE_SMEM), "attn_decode_static");
        g_static_address[device] = found;
    }
    *address = g_static_address[device];
    return 0;
}

}  // namespace

MRUN_API int mrun_attn_decode_static(const void* q, long q_stride, void* out, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int max_blocks,
                                     const int* token_slot, const int* positions, int tokens, int blocks,
                                     int min_tiles, int heads, int kv_heads, int head_dim, int page_size, float scale,
                                     int window, cudaStream_t stream) {
    if (int rc = check_common("attn_decode_static", heads, kv_heads, head_dim, page_size, max_blocks, window, 16))
        return rc;
    MRUN_REQUIRE(tokens >= 0 && blocks >= 1 && min_tiles >= 1, "attn_decode_static: tokens=%d blocks=%d min_tiles=%d",
                 tokens, blocks, min_tiles);
    MRUN_REQUIRE(blocks <= MRUN_STATIC_MAX_BLOCKS,
                 "attn_decode_static: blocks = %d exceeds the built-in scratch of %d blocks", blocks,
                 MRUN_STATIC_MAX_BLOCKS);
    MRUN_REQUIRE(tokens <= MRUN_STATIC_MAX_TOKENS,
                 "attn_decode_static: tokens = %d exceeds the built-in scratch of %d tokens", tokens,
                 MRUN_STATIC_MAX_TOKENS);
    MRUN_REQUIRE((long)tokens * kv_heads <= MRUN_STATIC_MAX_PAIRS,
                 "attn_decode_static: tokens * kv_heads = %ld exceeds the built-in scratch of %d counters",
                 (long)tokens * kv_heads, MRUN_STATIC_MAX_PAIRS);
    if (tokens == 0) return 0;
    float* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    float* part_o = scratch;
    float* part_ml = scratch + STATIC_PART_O;
    int* counters = reinterpret_cast<int*>(scratch + STATIC_PART_O + STATIC_PART_ML);
    int* assignment = counters + STATIC_COUNTERS;
    int* tile_prefix = assignment + STATIC_ASSIGNMENT;
    // the counters must start at zero whatever an earlier, possibly interrupted, call left
    MRUN_CHECK_CUDA(cudaMemsetAsync(counters, 0, (size_t)tokens * kv_heads * sizeof(int), stream),
                    "attn_decode_static: clearing the counters");
    decode_plan_kernel<<<1, 1024, 0, stream>>>(positions, tokens, window, tile_prefix, 0, min_tiles, 1);
    MRUN_CHECK_LAUNCH("attn_decode_static: plan");
    decode_assign_kernel<<<(blocks + 127) / 128, 128, 0, stream>>>(tile_prefix, tokens, kv_heads, blocks, min_tiles,
                                                                  0, (int4*)assignment);
    MRUN_CHECK_LAUNCH("attn_decode_static: assignment");
    decode_kernel<<<dim3(blocks), THREADS, DECODE_SMEM, stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks,
        token_slot, positions, tile_prefix, (const int4*)assignment, tokens, part_o, part_ml, counters, heads, kv_heads,
        page_size, page_shift_of(page_size), scale * LOG2E, window, FusedInput{});
    MRUN_CHECK_LAUNCH("attn_decode_static");
    return 0;
}
