// Linear layer on the fifth-generation tensor cores (tcgen05) for medium batches of rows
// (decode with 17 .. 256 requests): y[M, N] = x[M, K] · W[N, K]^T, bf16 operands, 32-bit
// accumulation in tensor memory, bf16 or 32-bit output, optional fused SiLU(gate) * up.
//
// The product is bound by reading W once from HBM, so the operands are swapped: the 128 lanes of
// the MMA take 128 rows of W and the tokens are its N dimension (16 .. 256).  The work is cut
// into units of one [128 weight rows x 64 k] block; every thread block takes an equal, contiguous
// range of units (a stream-K schedule), so that all SMs stream the same number of bytes whatever
// N and K are:
//
//   warp 0, one lane   TMA producer: per unit one box of W [128 x 64] and one of x [TOK x 64] into
//                      a ring of shared-memory stages (128-byte swizzle), each stage guarded by
//                      a full/empty mbarrier pair;
//   warp 1, one lane   MMA issuer: four tcgen05.mma (K = 16) per stage into one of two TMEM
//                      accumulators [128 lanes x TOK columns]; tcgen05.commit frees the stage
//                      and, at the end of a tile's k range, hands the accumulator to the epilogue;
//   warps 2 .. 5       epilogue: tcgen05.ld of the warp's 32 lanes, 16 columns at a time, then
//                      the output, or a 32-bit partial tile when the range covers part of a tile;
//                      it runs while the next tile's products fill the other accumulator.
//
// A tile whose k blocks fell to several thread blocks is finished by the one that arrives last at
// the tile's counter: it adds the partial tiles in block order, so the result does not depend on
// which block came last.
//
// Every wait on an mbarrier is bounded by a cycle budget.  When a wait runs out the block records
// a code in the status word, stops issuing, lets its copies in flight land, frees its tensor
// memory and returns; the host reads the status word after the step and raises.
//
// Reference call sites: crates/mrun-engine/src/load.rs:294-306 (x · Wᵀ),
// crates/mrun-engine/src/models/common.rs:336-339 (the gated feed-forward).
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using bf16 = __nv_bfloat16;

constexpr int BLOCK_ROWS = 128;      // weight rows per tile = MMA M
constexpr int BLOCK_K = 64;          // bf16 per smem row = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr long long WAIT_CYCLES = 3000000000LL;   // about 1.5 s at 2 GHz

enum : int { STATUS_OK = 0, STATUS_PRODUCER_TIMEOUT = 1, STATUS_MMA_TIMEOUT = 2, STATUS_EPILOGUE_TIMEOUT = 3 };

using namespace tc5;

__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    return tc5::mbar_wait(bar, parity, WAIT_CYCLES);
}
// Instruction descriptor: D f32, A and B bf16, both K-major, M = 128, N = tokens.
__host__ __device__ constexpr unsigned instruction_descriptor(int n) {
    return tc5::instruction_descriptor(BLOCK_ROWS, n);
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }

template <int TOK> constexpr int stages_for() {
    // stage = 16 KB of W + TOK * 128 bytes of x; keep the ring under ~200 KB
    return (200 * 1024) / (BLOCK_ROWS * BLOCK_K * 2 + TOK * BLOCK_K * 2) > 12
               ? 12 : (200 * 1024) / (BLOCK_ROWS * BLOCK_K * 2 + TOK * BLOCK_K * 2);
}

// Writes one warp's 32 weight rows x 16 tokens of results.  `row` is the thread's weight row.
template <typename TOut, bool SWIGLU>
__device__ __forceinline__ void write_columns(TOut* __restrict__ y, long ldy, const float (&v)[16], int row, int tok0,
                                              int M, int N, int act) {
    const int lane = threadIdx.x & 31;
    if constexpr (!SWIGLU) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (tok0 + j < M && row < N) store_out<TOut>(y + (size_t)(tok0 + j) * ldy + row, v[j]);
    } else {
        // rows 16q .. 16q+7 are gates, 16q+8 .. 16q+15 the ups of the same outputs
        const bool is_gate = (lane & 8) == 0;
        const int out_col = (row >> 4) * 8 + (row & 7);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float up_raw = __shfl_down_sync(0xffffffffu, v[j], 8);
            if (is_gate && tok0 + j < M && row < N) {
                const float gate = __bfloat162float(__float2bfloat16_rn(v[j]));
                const float up = __bfloat162float(__float2bfloat16_rn(up_raw));
                store_out<TOut>(y + (size_t)(tok0 + j) * ldy + out_col, mrun::gated_mul<false>(act, gate, up));
            }
        }
    }
}

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// The work is cut into units of one 64-wide k block of one 128-row tile, numbered tile by tile.
// Block p takes units [p * per, (p + 1) * per): every block streams the same number of bytes,
// whatever N and K are.  A block's range is a sequence of segments, each a k range of one tile;
// only its first and its last segment can be incomplete tiles.  An incomplete segment is written
// to scratch as a 32-bit partial tile (slot 0 if it is the block's first segment, else slot 1) and
// the block that arrives last at the tile's counter adds the tile's partials in block order.
//
// partial: [blocks][2][128][TOK] floats; counters: [tiles] ints, zero before and after; status: one int.
template <int TOK, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(192)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                TOut* __restrict__ y, long ldy, int M, int N, int k_blocks, int per, int total_units,
                float* __restrict__ partial, int* __restrict__ counters, int* __restrict__ status, int act) {
    constexpr int STAGES = stages_for<TOK>();
    constexpr int W_BYTES = BLOCK_ROWS * BLOCK_K * 2, X_BYTES = TOK * BLOCK_K * 2;
    constexpr unsigned ACC_COLS = TOK < 32 ? 32 : TOK;
    constexpr unsigned TMEM_COLS = 2 * ACC_COLS;                 // two accumulators
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int aborted, ticket_shared;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int u0 = blockIdx.x * per, u1 = min(total_units, u0 + per);
    const int n_units = max(0, u1 - u0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);                         // one arrival per epilogue warp
        }
        aborted = 0;
        mbar_init_fence();
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            for (int i = 0; i < n_units; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) {
                    atomicExch(status, STATUS_PRODUCER_TIMEOUT);
                    atomicExch(&aborted, 1);
                    break;
                }
                if (*(volatile int*)&aborted) break;
                const int u = u0 + i, tile = u / k_blocks, kb = u - tile * k_blocks;
                unsigned char* w_tile = tiles + (size_t)s * (W_BYTES + X_BYTES);
                mbar_expect_tx(&full_bar[s], W_BYTES + X_BYTES);
                tma_load_2d(w_tile, &map_w, kb * BLOCK_K, tile * BLOCK_ROWS, &full_bar[s]);
                tma_load_2d(w_tile + W_BYTES, &map_x, kb * BLOCK_K, 0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc = instruction_descriptor(TOK);
            int seg = -1, acc = 0;
            for (int i = 0; i < n_units; ++i) {
                const int u = u0 + i, tile = u / k_blocks, kb = u - tile * k_blocks;
                const bool first_of_segment = i == 0 || kb == 0;
                if (first_of_segment) {
                    ++seg;
                    acc = seg & 1;
                    // the epilogue must have drained this accumulator (used by segment seg - 2)
                    if (seg >= 2 && !mbar_wait(&acc_empty[acc], ((seg >> 1) - 1) & 1)) {
                        atomicExch(status, STATUS_MMA_TIMEOUT);
                        atomicExch(&aborted, 1);
                        break;
                    }
                    tc_fence_after();
                }
                const int s = i % STAGES;
                if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) {
                    atomicExch(status, STATUS_MMA_TIMEOUT);
                    atomicExch(&aborted, 1);
                    break;
                }
                if (*(volatile int*)&aborted) break;
                tc_fence_after();
                const unsigned char* w_tile = tiles + (size_t)s * (W_BYTES + X_BYTES);
                const unsigned long long a_desc = smem_descriptor(w_tile), b_desc = smem_descriptor(w_tile + W_BYTES);
                const unsigned d_tmem = tmem_base + acc * ACC_COLS;
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k)       // 32 bytes further along k per instruction
                    umma_bf16(d_tmem, a_desc + (unsigned long long)(k * UMMA_K * 2 >> 4),
                              b_desc + (unsigned long long)(k * UMMA_K * 2 >> 4), idesc,
                              (first_of_segment && k == 0) ? 0u : 1u);
                umma_commit(&empty_bar[s]);                      // the stage is free once these have read it
                const bool last_of_segment = i == n_units - 1 || kb == k_blocks - 1;
                if (last_of_segment) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue, warps 2..5
        const int quarter = warp & 3;                                // the TMEM lanes this warp may read
        const int tid = (warp - 2) * 32 + lane;                      // 0..127 among the epilogue threads
        int seg = 0;
        int i = 0;
        while (i < n_units) {
            const int u = u0 + i, tile = u / k_blocks, kb_first = u - tile * k_blocks;
            const int len = min(n_units - i, k_blocks - kb_first);
            const bool complete = kb_first == 0 && len == k_blocks;
            const int acc = seg & 1;
            bool have = mbar_wait(&acc_full[acc], (seg >> 1) & 1);
            if (!have && lane == 0) {
                atomicExch(status, STATUS_EPILOGUE_TIMEOUT);
                atomicExch(&aborted, 1);
            }
            tc_fence_after();
            have = have && !*(volatile int*)&aborted;
            const int row_in_tile = quarter * 32 + lane;
            const int row = tile * BLOCK_ROWS + row_in_tile;
            const unsigned lane_base = tmem_base + acc * ACC_COLS + ((unsigned)(quarter * 32) << 16);
            if (complete) {
                if (have) {
#pragma unroll 1
                    for (int c = 0; c < TOK; c += 16) {
                        if (c >= M) break;
                        float v[16];
                        tmem_load16(lane_base + c, v);
                        write_columns<TOut, SWIGLU>(y, ldy, v, row, c, M, N, act);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc]);
            } else {
                float* mine = partial + (((size_t)blockIdx.x * 2 + (seg == 0 ? 0 : 1)) * BLOCK_ROWS + row_in_tile) * TOK;
#pragma unroll 1
                for (int c = 0; c < TOK; c += 16) {
                    if (c >= M) break;
                    float v[16];
                    if (have) tmem_load16(lane_base + c, v);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<float4*>(mine + c + 4 * q) =
                            have ? make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]) : make_float4(0, 0, 0, 0);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc]);
                // the blocks that share this tile: p_first .. p_last
                const int p_first = (tile * k_blocks) / per, p_last = ((tile + 1) * k_blocks - 1) / per;
                __threadfence();
                epilogue_barrier();
                if (tid == 0) ticket_shared = atomicAdd(&counters[tile], 1);
                epilogue_barrier();
                if (ticket_shared == p_last - p_first) {             // the last to arrive adds them in block order
                    __threadfence();
#pragma unroll 1
                    for (int c = 0; c < TOK; c += 16) {
                        if (c >= M) break;
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                        for (int q = p_first; q <= p_last; ++q) {
                            // block q's piece of this tile is its first segment iff its range starts inside the tile
                            const int slot = (q * per) / k_blocks == tile ? 0 : 1;
                            const float* src = partial + (((size_t)q * 2 + slot) * BLOCK_ROWS + row_in_tile) * TOK + c;
#pragma unroll
                            for (int w4 = 0; w4 < 4; ++w4) {
                                const float4 t = __ldcg(reinterpret_cast<const float4*>(src + 4 * w4));
                                v[4 * w4] += t.x; v[4 * w4 + 1] += t.y; v[4 * w4 + 2] += t.z; v[4 * w4 + 3] += t.w;
                            }
                        }
                        write_columns<TOut, SWIGLU>(y, ldy, v, row, c, M, N, act);
                    }
                    if (tid == 0) counters[tile] = 0;
                }
                epilogue_barrier();                                  // ticket_shared is reused by the next segment
            }
            i += len;
            ++seg;
        }
    }

    // -------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*(volatile int*)&aborted) {
        // copies that were requested may still be landing in this block's shared memory
        const long long start = clock64();
        while (clock64() - start < 4000000LL) __nanosleep(1000);
    }
    if (warp == 0) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------ host

// A [rows x cols] bf16 matrix with `ld` elements between rows, read in boxes of [box_rows x 64].
int make_map(CUtensorMap* map, const void* base, long rows, long cols, long ld, int box_rows) {
    EncodeTiled encode = encode_tiled();
    MRUN_REQUIRE(encode != nullptr, "gemm_tc5: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(bf16)};
    const cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                               elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MRUN_REQUIRE(rc == CUDA_SUCCESS, "gemm_tc5: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    return 0;
}

template <int TOK, typename TOut, bool SWIGLU>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, TOut* y, long ldy, int M, int N, int K, int blocks,
           float* partial, int* counters, int* status, cudaStream_t stream, int act) {
    constexpr int STAGES = stages_for<TOK>();
    constexpr size_t smem = (size_t)STAGES * (BLOCK_ROWS * BLOCK_K * 2 + TOK * BLOCK_K * 2) + 1024;
    static bool configured = false;
    if (!configured) {
        MRUN_CHECK_CUDA(cudaFuncSetAttribute(gemm_tc5_kernel<TOK, TOut, SWIGLU>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "gemm_tc5");
        configured = true;
    }
    const int k_blocks = K / BLOCK_K;
    const int total = ((N + BLOCK_ROWS - 1) / BLOCK_ROWS) * k_blocks;
    const int per = (total + blocks - 1) / blocks;
    const int grid = (total + per - 1) / per;
    gemm_tc5_kernel<TOK, TOut, SWIGLU><<<grid, 192, smem, stream>>>(map_w, map_x, y, ldy, M, N, k_blocks, per, total,
                                                                   partial, counters, status, act);
    MRUN_CHECK_LAUNCH("gemm_tc5");
    return 0;
}

template <typename TOut, bool SWIGLU>
int dispatch(const CUtensorMap& map_w, const void* x, long ldx, TOut* y, long ldy, int M, int N, int K, int blocks,
             float* partial, int* counters, int* status, cudaStream_t stream, int tok, int act) {
    CUtensorMap map_x;
    if (int rc = make_map(&map_x, x, M, K, ldx, tok)) return rc;
    switch (tok) {
        case 32: return launch<32, TOut, SWIGLU>(map_w, map_x, y, ldy, M, N, K, blocks, partial, counters, status, stream, act);
        case 64: return launch<64, TOut, SWIGLU>(map_w, map_x, y, ldy, M, N, K, blocks, partial, counters, status, stream, act);
        case 128: return launch<128, TOut, SWIGLU>(map_w, map_x, y, ldy, M, N, K, blocks, partial, counters, status, stream, act);
        case 256: return launch<256, TOut, SWIGLU>(map_w, map_x, y, ldy, M, N, K, blocks, partial, counters, status, stream, act);
    }
    return mrun_set_error("gemm_tc5: no kernel for a token tile of %d", tok);
}

}  // namespace

// The token tile (MMA N) this kernel uses for M rows, or 0 when it takes no such M.
MRUN_API int mrun_gemm_tc5_token_tile(int M) {
    if (M < 1 || M > 256) return 0;
    return M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
}

// Floats of scratch a call with `blocks` blocks needs (two partial tiles per block).
MRUN_API long mrun_gemm_tc5_scratch_floats(int M, int blocks) {
    const int tok = mrun_gemm_tc5_token_tile(M);
    if (tok == 0) return 0;
    return (long)blocks * 2 * BLOCK_ROWS * tok;
}

// y[M, N] (or, with gate = MRUN_GATE_*, [M, N / 2] of act(gate) * up) = x[M, K] · w[N, K]^T.  x rows ldx elements apart, y rows ldy.
// blocks: how many blocks share the work (the number of SMs); partial: scratch of
// mrun_gemm_tc5_scratch_floats floats; counters: one zero int per 128 rows of w (left zero);
// status: one int the kernel sets non-zero when a wait ran out.
MRUN_API int mrun_gemm_tc5(const void* x, const void* w, void* y, int out_dtype, int gate, int M, int N, int K,
                           long ldx, long ldy, int blocks, float* partial, int* counters, int* status,
                           cudaStream_t stream) {
    MRUN_REQUIRE(M >= 1 && N > 0 && K > 0, "gemm_tc5: bad sizes M=%d N=%d K=%d", M, N, K);
    const int tok = mrun_gemm_tc5_token_tile(M);
    MRUN_REQUIRE(tok != 0, "gemm_tc5: M=%d exceeds the 256 rows this kernel takes", M);
    MRUN_REQUIRE(K % BLOCK_K == 0, "gemm_tc5: K=%d is not a multiple of %d", K, BLOCK_K);
    MRUN_REQUIRE(ldx >= K && ldx % 8 == 0, "gemm_tc5: ldx=%ld must be a multiple of 8 and at least K=%d", ldx, K);
    MRUN_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc5: x and W must be 16-byte aligned");
    if (gate) MRUN_REQUIRE_GATE(gate, "gemm_tc5");
    const int swiglu = gate;
    MRUN_REQUIRE(!swiglu || N % 16 == 0, "gemm_tc5: the gated epilogue needs N=%d to be a multiple of 16", N);
    MRUN_REQUIRE(ldy >= (swiglu ? N / 2 : N), "gemm_tc5: ldy=%ld is below the output width", ldy);
    MRUN_REQUIRE(blocks >= 1 && blocks <= 4096, "gemm_tc5: blocks=%d must be in 1..4096", blocks);
    MRUN_REQUIRE(partial && counters && status, "gemm_tc5: scratch, counters and a status word are required");
    CUtensorMap map_w;
    if (int rc = make_map(&map_w, w, N, K, K, BLOCK_ROWS)) return rc;
    if (out_dtype == MRUN_BF16) {
        if (swiglu)
            return dispatch<bf16, true>(map_w, x, ldx, (bf16*)y, ldy, M, N, K, blocks, partial, counters, status, stream, tok, gate);
        return dispatch<bf16, false>(map_w, x, ldx, (bf16*)y, ldy, M, N, K, blocks, partial, counters, status, stream, tok, gate);
    }
    if (out_dtype == MRUN_F32) {
        MRUN_REQUIRE(!swiglu, "gemm_tc5: the gated epilogue writes bfloat16");
        return dispatch<float, false>(map_w, x, ldx, (float*)y, ldy, M, N, K, blocks, partial, counters, status, stream, tok, gate);
    }
    return mrun_set_error("gemm_tc5: unknown output dtype code %d", out_dtype);
}
