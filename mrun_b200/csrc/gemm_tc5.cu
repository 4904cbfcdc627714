// Linear layer on the fifth-generation tensor cores (tcgen05) for medium batches of rows
// (decode with 17 .. 128 requests): y[M, N] = x[M, K] · W[N, K]^T, bf16 operands, 32-bit
// accumulation in tensor memory, with the same epilogues as the decode GEMM for a handful of
// rows: plain (bf16 or 32-bit), act(gate) * up, or "stream += y, x of the next product, totals of
// squares for its norm"; x may be the unscaled output of such a norm.
//
// The product is bound by reading W once from HBM, so the operands are swapped: the 128 lanes of
// the MMA take 128 rows of W (a tile) and the tokens are its N dimension (32, 64 or 128).  A
// kernel that holds tensor memory has a multiprocessor to itself, so the grid is at most one
// block a multiprocessor, in thread-block clusters:
//
//  * a cluster of `split` blocks takes tiles cluster, cluster + clusters, ... one after the
//    other, and block `rank` of it streams k blocks [rank k / split, (rank + 1) k / split) of
//    every one of them.  The host picks split and clusters per (N, K) so that all blocks stream
//    about the same number of bytes and as many multiprocessors as the device schedules
//    clusters on are busy; the choice does not depend on M, so a row's sums do not either;
//  * warp 0, one lane: TMA producer.  Per k block one box of W [128 x 64] and one of x
//    [TOK x 64] into a ring of shared-memory stages (128-byte swizzle), each stage guarded by a
//    full/empty mbarrier pair.  The first ring of W boxes is asked for before the kernel waits
//    for the kernel before it (programmatic dependent launch): weights are nobody's output;
//  * warp 1, one lane: MMA issuer.  Four tcgen05.mma (K = 16) per stage into one of two
//    accumulators [128 lanes x TOK columns]; tcgen05.commit frees the stage and, after the
//    block's last k block of a tile, hands the accumulator to the epilogue;
//  * warps 2 .. 5: epilogue, a thread a row of the tile.  With split = 1 they write the tile
//    from tensor memory.  Otherwise the tokens are dealt to the cluster's blocks, every block
//    pushes its partial sums of a token into the inbox of the token's owner through distributed
//    shared memory (coalesced remote stores, then one remote mbarrier arrival a warp), and the
//    owner adds the `split` partial sums in rank order and finishes the token.  Inboxes are
//    double-buffered where they fit; an owner lets the others know when a buffer may be
//    overwritten (remote arrivals again).  No scratch in global memory, no counter, no fence.
//
// Every wait on an mbarrier is bounded by a cycle budget.  When a wait runs out the block records
// a code in the status word, stops, lets its copies in flight land, meets its cluster at the
// hardware barrier (which every block reaches, since all its waits are bounded), frees its
// tensor memory and returns; the host reads the status word after the step and raises.
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
constexpr int THREADS = 192;
constexpr int MAX_SPLIT = 8;         // the portable cluster size
constexpr long long WAIT_CYCLES = 3000000000LL;   // about 1.5 s at 2 GHz

enum : int { EPI_PLAIN = 0, EPI_GATED = 1, EPI_RESIDUAL = 2 };
enum : int { STATUS_OK = 0, STATUS_PRODUCER = 1, STATUS_MMA = 2, STATUS_EPILOGUE = 3, STATUS_EXCHANGE = 4 };
// Sums of squares travel as unsigned 64-bit integers in units of 2^-30, as in the decode GEMM.
constexpr float SUMS_SCALE = 1073741824.f, SUMS_UNIT = 1.f / 1073741824.f;

using namespace tc5;

// What a launch does beside the product itself (the decode GEMM's struct, for up to 128 rows).
struct Fusion {
    int act;                              // EPI_GATED: the gate's function (MRUN_GATE_*)
    const unsigned long long* in_sums;    // [M] totals of squares of x's rows, or null: x as it is
    float in_eps, in_inv_width;
    float* resid;                         // EPI_RESIDUAL: resid[M, ldr] += y
    long ldr;
    const float* norm_w;                  // ... xw_out[M, N] = bf16(resid * norm_w)
    bf16* xw_out;
    unsigned long long* out_sums;         // ... out_sums[M] += squares of the new stream
};

template <int TOK> struct Shape {
    static constexpr int W_BYTES = BLOCK_ROWS * BLOCK_K * 2, X_BYTES = TOK * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    // one inbox: split * ceil(M / split) <= M + split - 1 token columns of 128 floats
    static constexpr int INBOX_BYTES = (TOK + MAX_SPLIT) * BLOCK_ROWS * 4;
    static constexpr int INBOXES = TOK <= 64 ? 2 : 1;
    static constexpr int BUDGET = 225 * 1024;
    static constexpr int STAGES = (BUDGET - 1024 - INBOXES * INBOX_BYTES) / STAGE_BYTES;
    static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + INBOXES * INBOX_BYTES;
    static constexpr unsigned TMEM_COLS = 2 * TOK;            // two accumulators; a power of two >= 32
    static_assert(STAGES >= 3, "the ring is too shallow");
};

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// ------------------------------------------------------------------------------------ the cluster
__device__ __forceinline__ unsigned cluster_size() {
    unsigned n;
    asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(n));
    return n;
}
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The address, in the cluster's shared window, of block `rank`'s copy of an own shared address.
__device__ __forceinline__ unsigned cluster_address(unsigned own_shared, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(own_shared), "r"(rank));
    return remote;
}
__device__ __forceinline__ void cluster_store(unsigned address, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(address), "f"(v) : "memory");
}
// One arrival on a barrier of another block of the cluster; what this thread wrote (and, after a
// warp barrier, what its warp wrote) into that block's shared memory is visible to whoever
// passes the barrier's phase with an acquire at cluster scope.
__device__ __forceinline__ void cluster_arrive(unsigned barrier_address) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(barrier_address) : "memory");
}
__device__ __forceinline__ void cluster_fence() { asm volatile("fence.acq_rel.cluster;\n" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait_cluster(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long* bar, unsigned parity, const int* give_up) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (clock64() - start > WAIT_CYCLES) return false;
        if (*(const volatile int*)give_up) return false;
    }
    return true;
}

// One finished sum: row `row` of W (the output column), token `tok`.  Every lane of the warp
// calls it for the same token (the gated and the residual epilogue meet across lanes).
template <typename TOut, int EPI>
__device__ __forceinline__ void finish(TOut* __restrict__ y, long ldy, const Fusion& f, float value, float stream,
                                       float norm_weight, int tok, int row, int N) {
    const int lane = threadIdx.x & 31;
    if constexpr (EPI == EPI_PLAIN) {
        if (row < N) store_out<TOut>(y + (size_t)tok * ldy + row, value);
    } else if constexpr (EPI == EPI_GATED) {
        // rows 16q .. 16q+7 are gates, 16q+8 .. 16q+15 the ups of the same outputs
        const float up_raw = __shfl_down_sync(0xffffffffu, value, 8);
        if ((lane & 8) == 0 && row < N) {
            // the activation sees the gate as the layer would have stored it
            const float gate = __bfloat162float(__float2bfloat16_rn(value));
            const float up = __bfloat162float(__float2bfloat16_rn(up_raw));
            store_out<TOut>(y + (size_t)tok * ldy + (row >> 4) * 8 + (row & 7), mrun::gated_mul<false>(f.act, gate, up));
        }
    } else {
        float v = 0.f;
        if (row < N) {
            v = stream + value;
            f.resid[(size_t)tok * f.ldr + row] = v;
            f.xw_out[(size_t)tok * N + row] = __float2bfloat16_rn(v * norm_weight);
        }
        const float q = mrun::warp_sum(v * v);
        if (lane == 0) atomicAdd(f.out_sums + tok, __float2ull_rn(fminf(q, 1.5e10f) * SUMS_SCALE));
    }
}

template <int TOK, typename TOut, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                TOut* __restrict__ y, long ldy, int M, int N, int k_blocks, int n_tiles, const Fusion f,
                int* __restrict__ status) {
    using S = Shape<TOK>;
    constexpr int STAGES = S::STAGES, INBOXES = S::INBOXES;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* inbox = reinterpret_cast<float*>(ring + STAGES * S::STAGE_BYTES);
    __shared__ unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned long long ready_bar[INBOXES], free_bar[INBOXES];
    __shared__ unsigned tmem_base_slot;
    __shared__ int aborted;
    __shared__ float row_scale[TOK];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = (int)cluster_size(), rank = (int)cluster_rank();
    const int clusters = (int)gridDim.x / split, cluster = (int)blockIdx.x / split;
    const int kb0 = (int)((long)rank * k_blocks / split), kb1 = (int)((long)(rank + 1) * k_blocks / split);
    const int n_k = kb1 - kb0;                                    // >= 1: the host keeps split <= k_blocks
    const int my_tiles = cluster < n_tiles ? (n_tiles - cluster + clusters - 1) / clusters : 0;
    const int total = my_tiles * n_k;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);                         // one arrival per epilogue warp
        }
        for (int b = 0; b < INBOXES; ++b) {
            mbar_init(&ready_bar[b], split * 4);                 // one per epilogue warp of every block
            mbar_init(&free_bar[b], split * 4);
        }
        aborted = 0;
        mbar_init_fence();
    }
    __syncwarp();
    if (warp == 0) tmem_alloc(&tmem_base_slot, S::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    __syncwarp();
    cluster_sync_all();                                          // everybody's barriers exist
    const unsigned tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            const int ahead = total < STAGES ? total : STAGES;
            for (int j = 0; j < ahead; ++j) {                    // weights first: they are nobody's output
                const int tile = cluster + (j / n_k) * clusters, kb = kb0 + j % n_k;
                mbar_expect_tx(&full_bar[j], S::STAGE_BYTES);
                tma_load_2d(ring + (size_t)j * S::STAGE_BYTES, &map_w, kb * BLOCK_K, tile * BLOCK_ROWS, &full_bar[j]);
            }
            mrun::wait_for_kernel_before();
            mrun::dependents_may_start();
            for (int j = 0; j < ahead; ++j)
                tma_load_2d(ring + (size_t)j * S::STAGE_BYTES + S::W_BYTES, &map_x, (kb0 + j % n_k) * BLOCK_K, 0, &full_bar[j]);
            for (int j = ahead; j < total; ++j) {
                const int s = j % STAGES;
                if (!mbar_wait(&empty_bar[s], ((j / STAGES) - 1) & 1, WAIT_CYCLES, &aborted)) {
                    if (!*(volatile int*)&aborted) atomicExch(status, STATUS_PRODUCER);
                    atomicExch(&aborted, 1);
                    break;
                }
                const int tile = cluster + (j / n_k) * clusters, kb = kb0 + j % n_k;
                unsigned char* stage = ring + (size_t)s * S::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
                tma_load_2d(stage, &map_w, kb * BLOCK_K, tile * BLOCK_ROWS, &full_bar[s]);
                tma_load_2d(stage + S::W_BYTES, &map_x, kb * BLOCK_K, 0, &full_bar[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr unsigned idesc = tc5::instruction_descriptor(BLOCK_ROWS, TOK);
            int acc = 0;
            for (int j = 0; j < total; ++j) {
                const int i = j / n_k, kk = j - i * n_k;
                if (kk == 0) {
                    acc = i & 1;
                    // the epilogue must have drained this accumulator (used by tile i - 2)
                    if (i >= 2 && !mbar_wait(&acc_empty[acc], ((i >> 1) - 1) & 1, WAIT_CYCLES, &aborted)) {
                        if (!*(volatile int*)&aborted) atomicExch(status, STATUS_MMA);
                        atomicExch(&aborted, 1);
                        break;
                    }
                    tc_fence_after();
                }
                const int s = j % STAGES;
                if (!mbar_wait(&full_bar[s], (j / STAGES) & 1, WAIT_CYCLES, &aborted)) {
                    if (!*(volatile int*)&aborted) atomicExch(status, STATUS_MMA);
                    atomicExch(&aborted, 1);
                    break;
                }
                tc_fence_after();
                const unsigned char* stage = ring + (size_t)s * S::STAGE_BYTES;
                const unsigned long long a_desc = smem_descriptor(stage), b_desc = smem_descriptor(stage + S::W_BYTES);
                const unsigned d_tmem = tmem_base + acc * TOK;
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k)       // 32 bytes further along k per instruction
                    umma_bf16(d_tmem, a_desc + (unsigned long long)(k * UMMA_K * 2 >> 4),
                              b_desc + (unsigned long long)(k * UMMA_K * 2 >> 4), idesc, (kk == 0 && k == 0) ? 0u : 1u);
                umma_commit(&empty_bar[s]);                      // the stage is free once these have read it
                if (kk == n_k - 1) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue, warps 2..5
        mrun::wait_for_kernel_before();                          // x's totals, the stream; and nothing is written before
        mrun::dependents_may_start();
        const int quarter = warp & 3;                            // the TMEM lanes this warp may read
        const int tid = (warp - 2) * 32 + lane;                  // 0..127 among the epilogue threads
        if (tid < TOK)
            row_scale[tid] = (f.in_sums != nullptr && tid < M)
                ? rsqrtf(__ull2float_rn(f.in_sums[tid]) * SUMS_UNIT * f.in_inv_width + f.in_eps) : 1.f;
        epilogue_barrier();
        const int row_in_tile = quarter * 32 + lane;
        const int cols_per = (M + split - 1) / split;            // tokens a block of the cluster owns
        const int my_col0 = rank * cols_per;
        const int my_cols = max(0, min(M, my_col0 + cols_per) - my_col0);
        const unsigned inbox_address = smem_u32(inbox);
        bool alive = true;
        for (int i = 0; i < my_tiles && alive; ++i) {
            const int tile = cluster + i * clusters, row = tile * BLOCK_ROWS + row_in_tile, acc = i & 1;
            if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[acc], (i >> 1) & 1, WAIT_CYCLES, &aborted))) {
                if (lane == 0) {
                    if (!*(volatile int*)&aborted) atomicExch(status, STATUS_EPILOGUE);
                    atomicExch(&aborted, 1);
                }
                alive = false;
                break;
            }
            tc_fence_after();
            const unsigned lane_base = tmem_base + acc * TOK + ((unsigned)(quarter * 32) << 16);
            float norm_weight = 0.f;
            if constexpr (EPI == EPI_RESIDUAL) norm_weight = row < N ? f.norm_w[row] : 0.f;
            if (split == 1) {
#pragma unroll 1
                for (int c = 0; c < TOK; c += 16) {
                    if (c >= M) break;
                    float v[16], stream[16];
                    if constexpr (EPI == EPI_RESIDUAL) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            stream[j] = (c + j < M && row < N) ? f.resid[(size_t)(c + j) * f.ldr + row] : 0.f;
                    }
                    tmem_load16(lane_base + c, v);
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c + j < M)
                            finish<TOut, EPI>(y, ldy, f, v[j] * row_scale[c + j], EPI == EPI_RESIDUAL ? stream[j] : 0.f,
                                              norm_weight, c + j, row, N);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc]);
                continue;
            }
            const int buf = i % INBOXES;
            if (i >= INBOXES &&
                !__all_sync(0xffffffffu, mbar_wait_cluster(&free_bar[buf], ((i / INBOXES) - 1) & 1, &aborted))) {
                if (lane == 0) {
                    if (!*(volatile int*)&aborted) atomicExch(status, STATUS_EXCHANGE);
                    atomicExch(&aborted, 1);
                }
                alive = false;
                break;
            }
            // push: the partial sums of token t go to slot [buf][rank][t - owner's first] of its owner's inbox
#pragma unroll 1
            for (int c = 0; c < TOK; c += 16) {
                if (c >= M) break;
                float v[16];
                tmem_load16(lane_base + c, v);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = c + j;
                    if (tok < M) {
                        const int owner = tok / cols_per, slot = tok - owner * cols_per;
                        const unsigned at = inbox_address +
                            (unsigned)((((buf * split + rank) * cols_per + slot) * BLOCK_ROWS + row_in_tile) * 4);
                        cluster_store(cluster_address(at, (unsigned)owner), v[j]);
                    }
                }
            }
            tc_fence_before();
            cluster_fence();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&acc_empty[acc]);
                for (int r = 0; r < split; ++r) cluster_arrive(cluster_address(smem_u32(&ready_bar[buf]), (unsigned)r));
            }
            if (!__all_sync(0xffffffffu, mbar_wait_cluster(&ready_bar[buf], (i / INBOXES) & 1, &aborted))) {
                if (lane == 0) {
                    if (!*(volatile int*)&aborted) atomicExch(status, STATUS_EXCHANGE);
                    atomicExch(&aborted, 1);
                }
                alive = false;
                break;
            }
            // add the partial sums of the own tokens in rank order and finish them, four tokens at a time
            const float* mine = inbox + (size_t)buf * split * cols_per * BLOCK_ROWS + row_in_tile;
#pragma unroll 1
            for (int t0 = 0; t0 < my_cols; t0 += 4) {
                float sum[4], stream[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int tok = my_col0 + t0 + u;
                    stream[u] = 0.f;
                    if constexpr (EPI == EPI_RESIDUAL)
                        if (t0 + u < my_cols && row < N) stream[u] = f.resid[(size_t)tok * f.ldr + row];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    sum[u] = 0.f;
                    if (t0 + u < my_cols)
                        for (int p = 0; p < split; ++p) sum[u] += mine[(size_t)(p * cols_per + t0 + u) * BLOCK_ROWS];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int tok = my_col0 + t0 + u;
                    if (t0 + u < my_cols)
                        finish<TOut, EPI>(y, ldy, f, sum[u] * row_scale[tok], stream[u], norm_weight, tok, row, N);
                }
            }
            // the inbox may be overwritten: tell every block of the cluster
            __syncwarp();
            if (lane == 0)
                for (int r = 0; r < split; ++r) cluster_arrive(cluster_address(smem_u32(&free_bar[buf]), (unsigned)r));
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
    __syncwarp();
    cluster_sync_all();              // nobody leaves while another block may still write here or arrive on a barrier here
    if (warp == 0) tmem_dealloc(tmem_base, S::TMEM_COLS);
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

template <int TOK, typename TOut, int EPI>
void launch_config(cudaLaunchConfig_t* config, cudaLaunchAttribute* attributes, int split, int clusters, cudaStream_t stream) {
    *config = cudaLaunchConfig_t{};
    config->gridDim = dim3((unsigned)(split * clusters));
    config->blockDim = dim3(THREADS);
    config->dynamicSmemBytes = Shape<TOK>::SMEM;
    config->stream = stream;
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = (unsigned)split;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config->attrs = attributes;
    config->numAttrs = 2;
}

// How many clusters of `split` blocks of this kernel the device runs at a time (0: none), asked
// once per kernel and cluster size.
template <int TOK, typename TOut, int EPI>
int clusters_at_a_time(int split) {
    static int known[MAX_SPLIT + 1] = {};      // 0 = not asked yet, -1 = none
    static bool configured = false;
    auto kernel = gemm_tc5_kernel<TOK, TOut, EPI>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Shape<TOK>::SMEM) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        configured = true;
    }
    if (known[split] == 0) {
        cudaLaunchConfig_t config;
        cudaLaunchAttribute attributes[2];
        launch_config<TOK, TOut, EPI>(&config, attributes, split, 1, nullptr);
        config.numAttrs = 1;                   // the cluster shape alone
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &config) != cudaSuccess || n < 1) {
            cudaGetLastError();
            n = -1;
        }
        known[split] = n;
    }
    return known[split] > 0 ? known[split] : 0;
}

// The split of k over a cluster and the number of clusters for (N, K): the pair with the fewest
// k blocks on the longest block, a wider split counted as half a k block a tile it exchanges;
// it depends on the sizes and the device only, never on M.
template <int TOK, typename TOut, int EPI>
int plan(int n_tiles, int k_blocks, int forced_split, int* split_out, int* clusters_out) {
    long best = -1;
    for (int split = 1; split <= MAX_SPLIT; ++split) {
        if (forced_split > 0 && split != forced_split) continue;
        if (split > k_blocks) break;
        const int at_a_time = clusters_at_a_time<TOK, TOut, EPI>(split);
        if (at_a_time < 1) continue;
        const int rounds = (n_tiles + at_a_time - 1) / at_a_time;
        const int clusters = (n_tiles + rounds - 1) / rounds;
        const long cost = 2L * rounds * ((k_blocks + split - 1) / split) + (split > 1 ? rounds : 0);
        if (best < 0 || cost < best) {
            best = cost;
            *split_out = split;
            *clusters_out = clusters;
        }
    }
    MRUN_REQUIRE(best >= 0, "gemm_tc5: the device schedules no cluster of this kernel (split %d)", forced_split);
    return 0;
}

template <int TOK, typename TOut, int EPI>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, TOut* y, long ldy, int M, int N, int K, int forced_split,
           const Fusion& f, int* status, cudaStream_t stream) {
    const int k_blocks = K / BLOCK_K, n_tiles = (N + BLOCK_ROWS - 1) / BLOCK_ROWS;
    int split = 1, clusters = 1;
    if (int rc = plan<TOK, TOut, EPI>(n_tiles, k_blocks, forced_split, &split, &clusters)) return rc;
    cudaLaunchConfig_t config;
    cudaLaunchAttribute attributes[2];
    launch_config<TOK, TOut, EPI>(&config, attributes, split, clusters, stream);
    MRUN_CHECK_CUDA(cudaLaunchKernelEx(&config, gemm_tc5_kernel<TOK, TOut, EPI>, map_w, map_x, y, ldy, M, N, k_blocks,
                                       n_tiles, f, status), "gemm_tc5");
    return 0;
}

template <typename TOut, int EPI>
int dispatch(const CUtensorMap& map_w, const void* x, long ldx, TOut* y, long ldy, int M, int N, int K, int forced_split,
             const Fusion& f, int* status, cudaStream_t stream, int tok) {
    CUtensorMap map_x;
    if (int rc = make_map(&map_x, x, M, K, ldx, tok)) return rc;
    switch (tok) {
        case 32: return launch<32, TOut, EPI>(map_w, map_x, y, ldy, M, N, K, forced_split, f, status, stream);
        case 64: return launch<64, TOut, EPI>(map_w, map_x, y, ldy, M, N, K, forced_split, f, status, stream);
        case 128: return launch<128, TOut, EPI>(map_w, map_x, y, ldy, M, N, K, forced_split, f, status, stream);
    }
    return mrun_set_error("gemm_tc5: no kernel for a token tile of %d", tok);
}

}  // namespace

// The token tile (MMA N) this kernel uses for M rows, or 0 when it takes no such M.
MRUN_API int mrun_gemm_tc5_token_tile(int M) {
    if (M < 1 || M > 128) return 0;
    return M <= 32 ? 32 : M <= 64 ? 64 : 128;
}

// How many clusters of `split` blocks the device runs at a time for the token tile of M rows
// (0: none): what the choice of split and clusters rests on.
MRUN_API int mrun_gemm_tc5_clusters(int M, int split) {
    if (split < 1 || split > MAX_SPLIT) return 0;
    switch (mrun_gemm_tc5_token_tile(M)) {
        case 32: return clusters_at_a_time<32, bf16, EPI_PLAIN>(split);
        case 64: return clusters_at_a_time<64, bf16, EPI_PLAIN>(split);
        case 128: return clusters_at_a_time<128, bf16, EPI_PLAIN>(split);
    }
    return 0;
}

// y[M, N] = x[M, K] · w[N, K]^T for 1 .. 128 rows, x rows ldx elements apart, y rows ldy.
//   gate = MRUN_GATE_*: w holds gate and up rows interleaved in runs of eight and y[M, N / 2] =
//     act(gate) * up (bfloat16);
//   in_sums: x is the xw of a product before; row t is scaled by rsqrt(in_sums[t] 2^-30 / K + in_eps);
//   resid (with norm_w, xw_out, out_sums; y unused): resid[M, N] += the product (32-bit, rows N
//     apart), xw_out[M, N] = bf16(resid * norm_w), out_sums[t] += the squares of the new row t
//     in units of 2^-30.
// split: 0 = chosen from the sizes, else the cluster size to use (1 .. 8).  status: one int the
// kernel sets non-zero when a wait ran out.
MRUN_API int mrun_gemm_tc5(const void* x, const void* w, void* y, int out_dtype, int gate, int M, int N, int K,
                           long ldx, long ldy, const void* in_sums, float in_eps, float* resid, const float* norm_w,
                           void* xw_out, void* out_sums, int split, int* status, cudaStream_t stream) {
    MRUN_REQUIRE(M >= 1 && N > 0 && K > 0, "gemm_tc5: bad sizes M=%d N=%d K=%d", M, N, K);
    const int tok = mrun_gemm_tc5_token_tile(M);
    MRUN_REQUIRE(tok != 0, "gemm_tc5: M=%d exceeds the 128 rows this kernel takes", M);
    MRUN_REQUIRE(K % BLOCK_K == 0, "gemm_tc5: K=%d is not a multiple of %d", K, BLOCK_K);
    MRUN_REQUIRE(ldx >= K && ldx % 8 == 0, "gemm_tc5: ldx=%ld must be a multiple of 8 and at least K=%d", ldx, K);
    MRUN_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc5: x and W must be 16-byte aligned");
    MRUN_REQUIRE(split >= 0 && split <= MAX_SPLIT, "gemm_tc5: split=%d must be in 0..%d", split, MAX_SPLIT);
    MRUN_REQUIRE(status != nullptr, "gemm_tc5: a status word is required");
    Fusion f = {};
    f.act = gate;
    f.in_sums = (const unsigned long long*)in_sums;
    f.in_eps = in_eps;
    f.in_inv_width = 1.f / (float)K;
    CUtensorMap map_w;
    if (int rc = make_map(&map_w, w, N, K, K, BLOCK_ROWS)) return rc;
    if (resid != nullptr) {
        MRUN_REQUIRE(!gate && norm_w && xw_out && out_sums, "gemm_tc5: the residual epilogue needs norm_w, xw_out and out_sums and no gate");
        f.resid = resid;
        f.ldr = N;
        f.norm_w = norm_w;
        f.xw_out = (bf16*)xw_out;
        f.out_sums = (unsigned long long*)out_sums;
        return dispatch<bf16, EPI_RESIDUAL>(map_w, x, ldx, (bf16*)nullptr, 0, M, N, K, split, f, status, stream, tok);
    }
    MRUN_REQUIRE(y != nullptr, "gemm_tc5: no output");
    if (gate) {
        MRUN_REQUIRE_GATE(gate, "gemm_tc5");
        MRUN_REQUIRE(out_dtype == MRUN_BF16, "gemm_tc5: the gated epilogue writes bfloat16");
        MRUN_REQUIRE(N % 16 == 0, "gemm_tc5: the gated epilogue needs N=%d to be a multiple of 16", N);
        MRUN_REQUIRE(ldy >= N / 2, "gemm_tc5: ldy=%ld is below the output width", ldy);
        return dispatch<bf16, EPI_GATED>(map_w, x, ldx, (bf16*)y, ldy, M, N, K, split, f, status, stream, tok);
    }
    MRUN_REQUIRE(ldy >= N, "gemm_tc5: ldy=%ld is below the output width", ldy);
    if (out_dtype == MRUN_BF16) return dispatch<bf16, EPI_PLAIN>(map_w, x, ldx, (bf16*)y, ldy, M, N, K, split, f, status, stream, tok);
    if (out_dtype == MRUN_F32) return dispatch<float, EPI_PLAIN>(map_w, x, ldx, (float*)y, ldy, M, N, K, split, f, status, stream, tok);
    return mrun_set_error("gemm_tc5: unknown output dtype code %d", out_dtype);
}
