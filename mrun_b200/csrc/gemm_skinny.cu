// Linear layer for a handful of rows (decode): y[M, N] = x[M, K] · W[N, K]^T, M <= 16, bf16
// operands, 32-bit accumulation, bf16 or 32-bit output.  The product is bound by reading W once
// from HBM, so the kernel is built around that stream:
//
//  * a block owns 16 (or 32) rows of W and all of K; its eight warps take the 32-wide k chunks in
//    turn (chunk c goes to warp c mod 8), so at any moment the block reads 512 contiguous bytes
//    of each of its rows;
//  * every thread loads 16 bytes of a W row straight into registers, several chunks ahead, with
//    no shared-memory staging, and the same 16-byte slice of k from x;
//  * tensor-core products m16n8k16 with W as the 16-row operand and the tokens as the 8 columns.
//    Inside a 32-wide chunk thread t of a quad owns k = 8t .. 8t+7 of *both* operands, which is a
//    permutation of the instruction's k order applied to both sides alike, so the sum is the same;
//  * the eight partial sums are added in shared memory in warp order (fixed, so a row's result
//    does not depend on the batch), and the epilogue writes y, or SiLU(gate) * up when W holds
//    gate and up rows interleaved in runs of eight (rows 16j..16j+7 gate, 16j+8..16j+15 up).
//
// Reference call sites: crates/mrun-engine/src/load.rs:294-306 (x · Wᵀ),
// crates/mrun-engine/src/models/common.rs:336-339 (the gated feed-forward).
#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
using mrun::pdl_launch_dependents;
using mrun::pdl_wait;
#ifndef MRUN_SKINNY_WARPS
#define MRUN_SKINNY_WARPS 8
#endif
#ifndef MRUN_SKINNY_UNROLL
#define MRUN_SKINNY_UNROLL 4        // chunks per batch with one row tile and one token tile per block
#endif
#ifndef MRUN_SKINNY_UNROLL_WIDE
#define MRUN_SKINNY_UNROLL_WIDE 2   // ... with two row tiles or two token tiles (more registers per chunk)
#endif
#ifndef MRUN_SKINNY_WIDE_N
#define MRUN_SKINNY_WIDE_N (32 * 148 * 4)
#endif
constexpr int WARPS = MRUN_SKINNY_WARPS;
constexpr int THREADS = WARPS * 32;

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
template <int NT, int MT, int UNROLL, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(THREADS)
skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TOut* __restrict__ y, int M, int N, int K,
              long ldx, long ldy) {
    __shared__ float red[WARPS][MT * 16][NT * 8 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * (MT * 16);
    const int chunks = K >> 5;          // whole 32-wide chunks; K % 32 == 0 is checked by the host

    const bf16* w_rows[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = min(n0 + mt * 16 + g + h * 8, N - 1);   // rows past N are computed and dropped
            w_rows[mt][h] = w + (size_t)row * K + t * 8;
        }
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
                    wb[u][mt][1] = load_stream(w_rows[mt][1] + k);
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
    // The weights do not depend on the kernel before this one: their first two batches are
    // requested before waiting for it, the rows of x after.
    constexpr int STRIDE = UNROLL * WARPS;
    int c0 = warp;
    load_w(wa[0], c0);
    load_w(wa[1], c0 + STRIDE);
    pdl_wait();
    pdl_launch_dependents();
    load_x(xa[0], c0);
    load_x(xa[1], c0 + STRIDE);
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
    if constexpr (!SWIGLU) {
        for (int i = threadIdx.x; i < MT * 16 * NT * 8; i += THREADS) {
            const int row = i % (MT * 16), token = i / (MT * 16);
            if (token < M && n0 + row < N) {
                float s = 0.f;
#pragma unroll
                for (int wi = 0; wi < WARPS; ++wi) s += red[wi][row][token];
                store_out<TOut>(y + (size_t)token * ldy + n0 + row, s);
            }
        }
    } else {
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
                gate = __bfloat162float(__float2bfloat16_rn(gate));
                up = __bfloat162float(__float2bfloat16_rn(up));
                store_out<TOut>(y + (size_t)token * ldy + out_col, mrun::silu_mul<false>(gate, up));
            }
        }
    }
}

template <int NT, int MT, int UNROLL, typename TOut, bool SWIGLU>
void launch(const bf16* x, const bf16* w, TOut* y, int M, int N, int K, long ldx, long ldy, cudaStream_t stream) {
    const int blocks = (N + MT * 16 - 1) / (MT * 16);
    mrun::launch_pdl(MRUN_PDL_GEMM, skinny_kernel<NT, MT, UNROLL, TOut, SWIGLU>, dim3(blocks), dim3(THREADS), 0,
                     stream, x, w, y, M, N, K, ldx, ldy);
}

template <typename TOut, bool SWIGLU>
void dispatch(const bf16* x, const bf16* w, TOut* y, int M, int N, int K, long ldx, long ldy, cudaStream_t stream) {
    // two row tiles per block halve the reads of x once there are plenty of blocks
    const bool wide = N >= MRUN_SKINNY_WIDE_N;
    constexpr int DEEP = MRUN_SKINNY_UNROLL, SHALLOW = MRUN_SKINNY_UNROLL_WIDE;
    if (M <= 8) {
        // With the deep batches two blocks fit on an SM (registers), with the shallow ones three.
        // More than two rounds' worth of 16-row blocks (N = 6144: 384 blocks on 148 SMs) run in
        // one round with the shallow kind; fewer blocks are faster with the deep kind.
        if (wide) launch<1, 2, SHALLOW, TOut, SWIGLU>(x, w, y, M, N, K, ldx, ldy, stream);
        else if ((N + 15) / 16 > 2 * 148) launch<1, 1, SHALLOW, TOut, SWIGLU>(x, w, y, M, N, K, ldx, ldy, stream);
        else launch<1, 1, DEEP, TOut, SWIGLU>(x, w, y, M, N, K, ldx, ldy, stream);
    } else {
        // 9 to 16 rows of x: every chunk carries twice the x, so one row tile a block, and with
        // more than two rounds' worth of blocks one chunk per batch (measured at 16 rows, us:
        // QKV 6144x4096 17.6 -> 12.7, gate/up 24576x4096 53.9 -> 37.7 with one chunk; O 4096x4096
        // 10.4 and down 4096x12288 24.3 with two chunks, 11.2 and 28.2 with one)
        if ((N + 15) / 16 > 2 * 148) launch<2, 1, 1, TOut, SWIGLU>(x, w, y, M, N, K, ldx, ldy, stream);
        else launch<2, 1, SHALLOW, TOut, SWIGLU>(x, w, y, M, N, K, ldx, ldy, stream);
    }
}

}  // namespace

// out_dtype: MRUN_BF16 or MRUN_F32.  swiglu != 0: W holds gate/up rows interleaved in runs of
// eight and y gets N / 2 columns of SiLU(gate) * up.  x rows are ldx elements apart, y rows ldy.
MRUN_API int mrun_gemm_skinny(const void* x, const void* w, void* y, int out_dtype, int swiglu, int M, int N,
                              int K, long ldx, long ldy, cudaStream_t stream) {
    MRUN_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_skinny: bad sizes M=%d N=%d K=%d", M, N, K);
    MRUN_REQUIRE(M <= 16, "gemm_skinny: M=%d exceeds the 16 rows this kernel takes", M);
    MRUN_REQUIRE(K % 32 == 0, "gemm_skinny: K=%d is not a multiple of 32", K);
    MRUN_REQUIRE(ldx >= K && ldx % 8 == 0, "gemm_skinny: ldx=%ld must be a multiple of 8 and at least K=%d", ldx, K);
    MRUN_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_skinny: x and W must be 16-byte aligned");
    MRUN_REQUIRE(!swiglu || N % 16 == 0, "gemm_skinny: the gated epilogue needs N=%d to be a multiple of 16", N);
    MRUN_REQUIRE(ldy >= (swiglu ? N / 2 : N), "gemm_skinny: ldy=%ld is below the output width", ldy);
    if (M == 0) return 0;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (out_dtype == MRUN_BF16) {
        if (swiglu) dispatch<bf16, true>(xp, wp, (bf16*)y, M, N, K, ldx, ldy, stream);
        else dispatch<bf16, false>(xp, wp, (bf16*)y, M, N, K, ldx, ldy, stream);
    } else if (out_dtype == MRUN_F32) {
        MRUN_REQUIRE(!swiglu, "gemm_skinny: the gated epilogue writes bfloat16");
        dispatch<float, false>(xp, wp, (float*)y, M, N, K, ldx, ldy, stream);
    } else {
        return mrun_set_error("gemm_skinny: unknown output dtype code %d", out_dtype);
    }
    MRUN_CHECK_LAUNCH("gemm_skinny");
    return 0;
}
