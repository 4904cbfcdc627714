// Linear layer for a handful of rows (decode): y[M, N] = x[M, K] · W[N, K]^T, M <= 16, bf16
// operands, 32-bit accumulation, bf16 or 32-bit output.  The product is bound by reading W once
// from HBM, so the kernel is built around that stream:
//
//  * a block owns 16 (or 32) rows of W and all of K (8 to 15 rows where whole tiles would fill the
//    device unevenly, see rows_a_block()); its eight warps take the 32-wide k chunks in turn
//    (chunk c goes to warp c mod 8), so at any moment the block reads 512 contiguous bytes of
//    each of its rows;
//  * every thread loads 16 bytes of a W row straight into registers, several chunks ahead, with
//    no shared-memory staging, and the same 16-byte slice of k from x;
//  * tensor-core products m16n8k16 with W as the 16-row operand and the tokens as the 8 columns.
//    Inside a 32-wide chunk thread t of a quad owns k = 8t .. 8t+7 of *both* operands, which is a
//    permutation of the instruction's k order applied to both sides alike, so the sum is the same;
//  * the kernel is launched so that it may start while the kernel before it still runs
//    (programmatic dependent launch): a block asks for its first weights, then waits for that
//    kernel, then reads x;
//  * the eight partial sums are added in shared memory in warp order (fixed, so a row's result
//    does not depend on the batch), and the epilogue writes y, or act(gate) * up when W holds
//    gate and up rows interleaved in runs of eight (rows 16j..16j+7 gate, 16j+8..16j+15 up).
//
// A decode step is a chain of such products with a residual sum and an RMSNorm between them, and
// at a handful of rows a stand-alone norm kernel is all launch latency.  So the norm is split
// over the two products around it.  The product *before* it (epilogue RESIDUAL) adds its result
// to the 32-bit residual stream in place, writes xw = bf16(stream * norm weight) and adds the sum
// of squares of its 16 stream columns, per row, to the row's 64-bit fixed-point total (integer
// atomics: the total does not depend on the order in which the blocks arrive).  The product
// *after* it reads xw as its x and multiplies its sums by rsqrt(total / width + eps):
// RMSNorm(x) · Wᵀ = rsqrt(mean(x²) + eps) · ((x ⊙ w_norm) · Wᵀ).
//
// Reference call sites: crates/mrun-engine/src/load.rs:294-306 (x · Wᵀ),
// crates/mrun-engine/src/models/common.rs:336-339 (the gated feed-forward).
#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int UNROLL_DEEP = 4;      // chunks per batch with one row tile and one token tile per block
constexpr int UNROLL_SHALLOW = 2;   // ... with two row tiles or two token tiles (more registers per chunk)
enum : int { EPI_PLAIN = 0, EPI_GATED = 1, EPI_RESIDUAL = 2 };
// Sums of squares travel as unsigned 64-bit integers in units of 2^-30: room for 1.7e10, steps of
// 1e-9 (a row of unit-scale values sums to its width; eps times the width is 1e-6 times that).
constexpr float SUMS_SCALE = 1073741824.f, SUMS_UNIT = 1.f / 1073741824.f;

// What a launch does beside the product itself.
struct Fusion {
    int act;                     // EPI_GATED: the gate's function (MRUN_GATE_*)
    // x is the xw of a product before: the row's scale is rsqrt(in_sums[row] * 2^-30 / width + eps)
    const unsigned long long* in_sums;   // [16] totals of squares, or null: x is taken as it is
    float in_eps, in_inv_width;
    // EPI_RESIDUAL: resid[M, ldr] += y; xw_out[M, N] = bf16(resid * norm_w); out_sums[16] += squares
    float* resid;
    long ldr;
    const float* norm_w;
    bf16* xw_out;
    unsigned long long* out_sums;
};

__device__ __forceinline__ uint4 load_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }

// NT: token tiles of 8 (M <= 8 NT).  MT: 16-row tiles of W per block.  UNROLL: chunks per batch.
// Blocks a multiprocessor is to hold: three of the kinds with one register set of weights a chunk
// (85 registers a thread), two of the others (128).
constexpr int resident_blocks(int nt, int mt, int unroll) { return nt * mt * unroll <= 2 ? 3 : 2; }

// CUT: a block takes `rows` < MT * 16 rows of W (see rows_a_block()); else its whole tile.
template <int NT, int MT, int UNROLL, typename TOut, int EPI, bool CUT>
__global__ void __launch_bounds__(THREADS, resident_blocks(NT, MT, UNROLL))
skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TOut* __restrict__ y, int M, int N, int K,
              long ldx, long ldy, const Fusion f, int rows_cut) {
    static_assert(EPI != EPI_RESIDUAL || MT == 1, "the residual epilogue sums 16 columns per block");
    __shared__ float red[WARPS][MT * 16][NT * 8 + 1];
    __shared__ float row_scale[NT * 8];
    __shared__ __align__(8) unsigned long long totals[NT * 8];
    __shared__ float stream_tile[EPI == EPI_RESIDUAL ? NT * 8 * 16 : 1], norm_tile[16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rows = CUT ? rows_cut : MT * 16;
    const int n0 = blockIdx.x * rows;
    const int chunks = K >> 5;          // whole 32-wide chunks; K % 32 == 0 is checked by the host

    const bf16* w_rows[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = min(n0 + mt * 16 + g + h * 8, N - 1);   // rows past N are computed and dropped
            w_rows[mt][h] = w + (size_t)row * K + t * 8;
        }
    // a tile cut short (MT = 1, 8 <= rows < 16) ends in its second half: those rows belong to the
    // next block and are not read here
    const bool second_half = !CUT || g + 8 < rows;
    const bf16* x_rows[NT];
    bool x_valid[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        x_valid[nt] = nt * 8 + g < M;
        x_rows[nt] = x + (size_t)(x_valid[nt] ? nt * 8 + g : 0) * ldx + t * 8;
    }

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;

    // two register sets: while one batch of chunks is multiplied the next is in flight
    uint4 wa[2][UNROLL][MT][2], xa[2][UNROLL][NT];
    auto load_w = [&](uint4 (&wb)[UNROLL][MT][2], int c0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = c0 + u * WARPS;
            if (c < chunks) {
                const int k = c << 5;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    wb[u][mt][0] = load_stream(w_rows[mt][0] + k);
                    wb[u][mt][1] = second_half ? load_stream(w_rows[mt][1] + k) : make_uint4(0, 0, 0, 0);
                }
            }
        }
    };
    auto load_x = [&](uint4 (&xb)[UNROLL][NT], int c0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int c = c0 + u * WARPS;
            if (c < chunks) {
                const int k = c << 5;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    xb[u][nt] = x_valid[nt] ? __ldg(reinterpret_cast<const uint4*>(x_rows[nt] + k)) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto compute_batch = [&](const uint4 (&wb)[UNROLL][MT][2], const uint4 (&xb)[UNROLL][NT], int c0) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (c0 + u * WARPS < chunks) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_bf16(acc[mt][nt], wb[u][mt][0].x, wb[u][mt][1].x, wb[u][mt][0].y, wb[u][mt][1].y,
                                 xb[u][nt].x, xb[u][nt].y);
                        mma_bf16(acc[mt][nt], wb[u][mt][0].z, wb[u][mt][1].z, wb[u][mt][0].w, wb[u][mt][1].w,
                                 xb[u][nt].z, xb[u][nt].w);
                    }
            }
        }
    };
    constexpr int STRIDE = UNROLL * WARPS;
    int c0 = warp;
    load_w(wa[0], c0);
    load_w(wa[1], c0 + STRIDE);
    // The weights depend on no kernel: their first two batches were asked for while the kernel
    // before this one may still be running.  Everything else waits for it.
    mrun::wait_for_kernel_before();
    mrun::dependents_may_start();
    load_x(xa[0], c0);
    load_x(xa[1], c0 + STRIDE);
    // the rows' totals of squares are asked for with the first weights (an asynchronous copy:
    // no register waits for it) and used after the last
    if (f.in_sums != nullptr && threadIdx.x < NT * 8) {
        const unsigned dst = (unsigned)__cvta_generic_to_shared(totals + threadIdx.x);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(f.in_sums + threadIdx.x));
    }
    if constexpr (EPI == EPI_RESIDUAL) {
        // so are the block's 16 columns of the stream and of the norm weight (the kernel before
        // this one wrote the stream; no block of this one writes another block's columns)
        for (int i = threadIdx.x; i < 16 * NT * 8 + 16; i += THREADS) {
            const bool is_w = i >= 16 * NT * 8;
            const int row = i & 15, token = (i >> 4) & (NT * 8 - 1);
            if (row < rows && n0 + row < N && (is_w || token < M)) {
                const float* src = is_w ? f.norm_w + n0 + row : f.resid + (size_t)token * f.ldr + n0 + row;
                const unsigned dst = (unsigned)__cvta_generic_to_shared(is_w ? norm_tile + row : stream_tile + i);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src));
            }
        }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    while (c0 < chunks) {
        compute_batch(wa[0], xa[0], c0);
        c0 += STRIDE;
        if (c0 >= chunks) break;
        load_w(wa[0], c0 + STRIDE);
        load_x(xa[0], c0 + STRIDE);
        compute_batch(wa[1], xa[1], c0);
        c0 += STRIDE;
        if (c0 >= chunks) break;
        load_w(wa[1], c0 + STRIDE);
        load_x(xa[1], c0 + STRIDE);
    }

    asm volatile("cp.async.wait_all;\n" ::: "memory");
    if (threadIdx.x < NT * 8)
        row_scale[threadIdx.x] = f.in_sums != nullptr
            ? rsqrtf(__ull2float_rn(totals[threadIdx.x]) * SUMS_UNIT * f.in_inv_width + f.in_eps) : 1.f;
    // partial sums of the eight warps, added in warp order
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[warp][mt * 16 + g][nt * 8 + 2 * t] = acc[mt][nt][0];
            red[warp][mt * 16 + g][nt * 8 + 2 * t + 1] = acc[mt][nt][1];
            red[warp][mt * 16 + g + 8][nt * 8 + 2 * t] = acc[mt][nt][2];
            red[warp][mt * 16 + g + 8][nt * 8 + 2 * t + 1] = acc[mt][nt][3];
        }
    __syncthreads();
    if constexpr (EPI == EPI_PLAIN) {
        for (int i = threadIdx.x; i < MT * 16 * NT * 8; i += THREADS) {
            const int row = i % (MT * 16), token = i / (MT * 16);
            if (token < M && row < rows && n0 + row < N) {
                float s = 0.f;
#pragma unroll
                for (int wi = 0; wi < WARPS; ++wi) s += red[wi][row][token];
                store_out<TOut>(y + (size_t)token * ldy + n0 + row, s * row_scale[token]);
            }
        }
    } else if constexpr (EPI == EPI_GATED) {
        // rows 16j .. 16j+7 are gate rows, 16j+8 .. 16j+15 the up rows of the same outputs
        for (int i = threadIdx.x; i < MT * 8 * NT * 8; i += THREADS) {
            const int col = i % (MT * 8), token = i / (MT * 8);
            const int tile = col >> 3, r = col & 7;
            const int out_col = (n0 >> 1) + col;
            if (token < M && out_col < (N >> 1)) {
                float gate = 0.f, up = 0.f;
#pragma unroll
                for (int wi = 0; wi < WARPS; ++wi) {
                    gate += red[wi][tile * 16 + r][token];
                    up += red[wi][tile * 16 + 8 + r][token];
                }
                // the activation sees the gate as the layer would have stored it
                gate = __bfloat162float(__float2bfloat16_rn(gate * row_scale[token]));
                up = __bfloat162float(__float2bfloat16_rn(up * row_scale[token]));
                store_out<TOut>(y + (size_t)token * ldy + out_col, mrun::gated_mul<false>(f.act, gate, up));
            }
        }
    } else {
        // 16 consecutive threads hold the block's 16 columns of one row: the stream gets the sum,
        // the next product its x, and the 16 squares meet in the group's first lane
        for (int i = threadIdx.x; i < 16 * NT * 8; i += THREADS) {
            const int row = i & 15, token = i >> 4;
            float v = 0.f;
            if (token < M && row < rows && n0 + row < N) {
                float s = 0.f;
#pragma unroll
                for (int wi = 0; wi < WARPS; ++wi) s += red[wi][row][token];
                v = stream_tile[i] + s * row_scale[token];
                f.resid[(size_t)token * f.ldr + n0 + row] = v;
                f.xw_out[(size_t)token * N + n0 + row] = __float2bfloat16_rn(v * norm_tile[row]);
            }
            float q = v * v;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
            if (row == 0 && token < M) atomicAdd(f.out_sums + token, __float2ull_rn(fminf(q, 1.5e10f) * SUMS_SCALE));
        }
    }
}

int sm_count();

// Rows of W a block takes.  A block's tile holds 16 (MT = 1), but the device holds only so many
// blocks at a time, and with 16 rows each some multiprocessors carry a block more than others
// (4,096 rows are 256 blocks for 296 places: 108 multiprocessors stream 32 rows, 40 stream 16).
// Fewer rows a block, 8 at the least, so that the blocks fill the places evenly, shorten what the
// fullest multiprocessor streams: the count that makes (rounds over the places) x (rows a block)
// smallest, the larger count at a tie, and only where that is a quarter less than with 16 (a
// product of 2,560 rows, 160 blocks for 296 places: 9 rows a block; measured on B200, the
// Qwen3-4B shape's output and down projections gain 8 %, the step 2 to 4 %, while the 12 % that
// 14 rows promise a 4,096-row product do not show).  A function of N and the device, never of the batch.
int rows_a_block(int N, int places, int forced) {
    if (forced >= 8 && forced <= 16) return forced;
    const long cost16 = (long)(((N + 15) / 16 + places - 1) / places) * 16;
    int best = 16;
    long best_cost = cost16;
    for (int rows = 15; rows >= 8; --rows) {
        const long cost = (long)(((N + rows - 1) / rows + places - 1) / places) * rows;
        if (cost < best_cost) {
            best_cost = cost;
            best = rows;
        }
    }
    return 4 * best_cost <= 3 * cost16 ? best : 16;
}

template <int NT, int MT, int UNROLL, typename TOut, int EPI>
void launch(const bf16* x, const bf16* w, TOut* y, int M, int N, int K, long ldx, long ldy, const Fusion& f,
            int forced_rows, cudaStream_t stream) {
    if constexpr (MT == 1 && EPI != EPI_GATED) {     // the gated epilogue pairs rows inside whole runs of 16
        const int rows = rows_a_block(N, sm_count() * resident_blocks(NT, MT, UNROLL), forced_rows);
        if (rows < 16) {
            mrun::launch_kernel_overlapped(skinny_kernel<NT, MT, UNROLL, TOut, EPI, true>, dim3((N + rows - 1) / rows),
                                           dim3(THREADS), 0, stream, x, w, y, M, N, K, ldx, ldy, f, rows);
            return;
        }
    }
    mrun::launch_kernel_overlapped(skinny_kernel<NT, MT, UNROLL, TOut, EPI, false>, dim3((N + MT * 16 - 1) / (MT * 16)),
                                   dim3(THREADS), 0, stream, x, w, y, M, N, K, ldx, ldy, f, MT * 16);
}

int sm_count() {
    static int count = 0;          // of the current device at the first call; a tuning input only
    if (count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1)
            count = 148;
    }
    return count;
}

template <typename TOut, int EPI>
void dispatch(const bf16* x, const bf16* w, TOut* y, int M, int N, int K, long ldx, long ldy, const Fusion& f,
              int rows, cudaStream_t stream) {
    const int sms = sm_count();
    const bool two_rounds = (N + 15) / 16 > 2 * sms;      // more 16-row blocks than two a multiprocessor
    if (M <= 8) {
        // With the deep batches two blocks fit on a multiprocessor (registers), with the shallow
        // ones three.  Plenty of blocks: two row tiles a block halve the reads of x.  More than
        // two rounds' worth of 16-row blocks run in one round with the shallow kind; fewer blocks
        // are faster with the deep kind.
        if constexpr (EPI != EPI_RESIDUAL) {
            if (N >= 32 * sms * 4) return launch<1, 2, UNROLL_SHALLOW, TOut, EPI>(x, w, y, M, N, K, ldx, ldy, f, rows, stream);
        }
        if (two_rounds) launch<1, 1, UNROLL_SHALLOW, TOut, EPI>(x, w, y, M, N, K, ldx, ldy, f, rows, stream);
        else launch<1, 1, UNROLL_DEEP, TOut, EPI>(x, w, y, M, N, K, ldx, ldy, f, rows, stream);
    } else {
        // 9 to 16 rows of x: every chunk carries twice the x, so one row tile a block, and with
        // more than two rounds' worth of blocks one chunk per batch
        if (two_rounds) launch<2, 1, 1, TOut, EPI>(x, w, y, M, N, K, ldx, ldy, f, rows, stream);
        else launch<2, 1, UNROLL_SHALLOW, TOut, EPI>(x, w, y, M, N, K, ldx, ldy, f, rows, stream);
    }
}

}  // namespace

// y[M, N] = x[M, K] · w[N, K]^T for M <= 16.  out_dtype: MRUN_BF16 or MRUN_F32.  gate != 0
// (MRUN_GATE_*): W holds gate/up rows interleaved in runs of eight and y gets N / 2 columns of
// act(gate) * up.  x rows are ldx elements apart, y rows ldy.
// in_sums != null: x is the xw that a call with `resid` made, and every row's sums are
// multiplied by rsqrt(in_sums[row] * 2^-30 / K + in_eps).
// resid != null: nothing is written to y; instead resid[M, N] (32-bit, dense) += the product,
// xw_out[M, N] = bf16(resid * norm_w) and out_sums[row] (16 unsigned 64-bit integers, zero before
// the call) gets the row's sum of squares of resid in units of 2^-30.
// rows: the rows of W a block takes, 8..16, or 0 for the count that fills the device most evenly.
MRUN_API int mrun_gemm_skinny(const void* x, const void* w, void* y, int out_dtype, int gate, int M, int N,
                              int K, long ldx, long ldy, const unsigned long long* in_sums, float in_eps,
                              float* resid, const float* norm_w, void* xw_out, unsigned long long* out_sums,
                              int rows, cudaStream_t stream) {
    MRUN_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
    MRUN_REQUIRE(rows == 0 || (rows >= 8 && rows <= 16), "gemm_skinny: rows=%d a block must be 0 (chosen here) or 8..16", rows);
    MRUN_REQUIRE(M <= 16, "gemm_skinny: M=%d exceeds the 16 rows this kernel takes", M);
    MRUN_REQUIRE(K % 32 == 0, "gemm_skinny: K=%d is not a multiple of 32", K);
    MRUN_REQUIRE(ldx >= K && ldx % 8 == 0, "gemm_skinny: ldx=%ld must be a multiple of 8 and at least K=%d", ldx, K);
    MRUN_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_skinny: x and W must be 16-byte aligned");
    Fusion f = {};
    f.act = gate;
    f.in_sums = in_sums;
    f.in_eps = in_eps;
    f.in_inv_width = 1.f / (float)K;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (resid != nullptr) {
        MRUN_REQUIRE(!gate, "gemm_skinny: the residual epilogue has no gate");
        MRUN_REQUIRE(norm_w != nullptr && xw_out != nullptr && out_sums != nullptr,
                     "gemm_skinny: the residual epilogue needs norm_w, xw_out and out_sums");
        if (M == 0) return 0;
        f.resid = resid;
        f.ldr = N;
        f.norm_w = norm_w;
        f.xw_out = (bf16*)xw_out;
        f.out_sums = out_sums;
        dispatch<bf16, EPI_RESIDUAL>(xp, wp, (bf16*)nullptr, M, N, K, ldx, ldy, f, rows, stream);
        MRUN_CHECK_LAUNCH("gemm_skinny");
        return 0;
    }
    if (gate) MRUN_REQUIRE_GATE(gate, "gemm_skinny");
    MRUN_REQUIRE(!gate || N % 16 == 0, "gemm_skinny: the gated epilogue needs N=%d to be a multiple of 16", N);
    MRUN_REQUIRE(ldy >= (gate ? N / 2 : N), "gemm_skinny: ldy=%ld is below the output width", ldy);
    if (M == 0) return 0;
    if (out_dtype == MRUN_BF16) {
        if (gate) dispatch<bf16, EPI_GATED>(xp, wp, (bf16*)y, M, N, K, ldx, ldy, f, rows, stream);
        else dispatch<bf16, EPI_PLAIN>(xp, wp, (bf16*)y, M, N, K, ldx, ldy, f, rows, stream);
    } else if (out_dtype == MRUN_F32) {
        MRUN_REQUIRE(!gate, "gemm_skinny: the gated epilogue writes bfloat16");
        dispatch<float, EPI_PLAIN>(xp, wp, (float*)y, M, N, K, ldx, ldy, f, rows, stream);
    } else {
        return mrun_set_error("gemm_skinny: unknown output dtype code %d", out_dtype);
    }
    MRUN_CHECK_LAUNCH("gemm_skinny");
    return 0;
}

// out[t, k] = bf16(xw[t, k] * rsqrt(sums[t] * 2^-30 / width + eps)): the rows a product with
// `resid` left as xw, finished into plain RMSNorm output for a consumer that is not one of these
// products.
namespace {
__global__ void norm_finish_kernel(const bf16* __restrict__ xw, const unsigned long long* __restrict__ sums, float eps,
                                   float inv_width, bf16* __restrict__ out, int width) {
    const int token = blockIdx.x;
    const float scale = rsqrtf(__ull2float_rn(sums[token]) * SUMS_UNIT * inv_width + eps);
    for (int k = threadIdx.x; k < width; k += blockDim.x)
        out[(size_t)token * width + k] = __float2bfloat16_rn(__bfloat162float(xw[(size_t)token * width + k]) * scale);
}
}  // namespace

MRUN_API int mrun_norm_finish(const void* xw, const unsigned long long* sums, float eps, void* out, int tokens,
                              int width, cudaStream_t stream) {
    MRUN_REQUIRE(tokens >= 0 && tokens <= 65535 && width > 0, "norm_finish: bad sizes tokens=%d width=%d", tokens, width);
    if (tokens == 0) return 0;
    norm_finish_kernel<<<tokens, 256, 0, stream>>>((const bf16*)xw, sums, eps, 1.f / (float)width, (bf16*)out, width);
    MRUN_CHECK_LAUNCH("norm_finish");
    return 0;
}
