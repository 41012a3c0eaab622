// Weight-streaming matrix product for decode steps: out[M, N] = X[M, K] * W[N, K]^T with few
// rows M (at most 64 tokens), bfloat16 inputs, float32 accumulation.
//
// Reference (davidjoyme/mini-inference engine/core/fused_linear.py:29-34): the library GEMM,
// which its own measurements put at 17-50 % of peak bandwidth for these skinny shapes
// (README.md:29) and which it tunes by timing two weight layouts.  With M <= 64 the product is
// bound by reading W once from HBM, so this kernel is built around that stream:
//   * "swap-AB": the weight rows are the 16-row M side of mma.sync.m16n8k16, the tokens are the
//     8-wide N side, so no tensor-core work is wasted on padding tokens up to 64 or 128;
//   * no shared-memory staging: a thread loads 16 bytes of a weight row straight into the
//     registers of two k-steps (the reduction index is permuted inside each 32-wide window,
//     identically for W and X, which leaves the dot product unchanged);
//   * a block owns 16 or 32 output columns and ALL of K; its 8 warps take the 32-wide k-windows
//     round-robin, so together they read 512 contiguous bytes of each weight row per round;
//     partial sums meet in shared memory in a fixed order.
// The order in which an output element adds its products never depends on M, so a token's
// result does not depend on what else is in the batch.
#include "common.cuh"

using namespace mi;

namespace {

constexpr int GW = 8;        // warps per block

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename OutT> __device__ __forceinline__ OutT cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// NT: 8-token tiles (M <= 8 NT); MT: 16-row weight tiles per block; U: windows in flight per warp
template <int NT, int MT, int U, typename OutT>
__global__ void __launch_bounds__(GW * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ X, int ldx, const __nv_bfloat16* __restrict__ W,
                   OutT* __restrict__ out, int ldo, int M, int N, int K) {
    extern __shared__ float red[];                    // [GW][MT*16][NT*8]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * MT * 16;
    const int nw = K / 32;

    const __nv_bfloat16* wrow[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        wrow[mt][0] = W + (size_t)min(n0 + mt * 16 + g, N - 1) * K + 8 * c;
        wrow[mt][1] = W + (size_t)min(n0 + mt * 16 + g + 8, N - 1) * K + 8 * c;
    }
    const __nv_bfloat16* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        xok[nt] = nt * 8 + g < M;
        xrow[nt] = X + (size_t)(xok[nt] ? nt * 8 + g : 0) * ldx + 8 * c;
    }

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f; }

    for (int w0 = warp; w0 < nw; w0 += GW * U) {
        uint4 a[U][MT][2];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int w = w0 + u * GW;
            if (w < nw) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    a[u][mt][0] = ld_stream16(wrow[mt][0] + (size_t)w * 32);
                    a[u][mt][1] = ld_stream16(wrow[mt][1] + (size_t)w * 32);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int w = w0 + u * GW;
            if (w < nw) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    uint4 b = make_uint4(0, 0, 0, 0);
                    if (xok[nt]) b = __ldg(reinterpret_cast<const uint4*>(xrow[nt] + (size_t)w * 32));
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma16816(acc[mt][nt], a[u][mt][0].x, a[u][mt][1].x, a[u][mt][0].y, a[u][mt][1].y, b.x, b.y);
                        mma16816(acc[mt][nt], a[u][mt][0].z, a[u][mt][1].z, a[u][mt][0].w, a[u][mt][1].w, b.z, b.w);
                    }
                }
            }
        }
    }

    // partial sums -> shared memory [warp][row][token], then a fixed-order sum over the warps
    constexpr int ROWS = MT * 16, TOK = NT * 8;
    float* mine = red + (size_t)warp * ROWS * TOK;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int r = mt * 16 + g, t = nt * 8 + 2 * c;
            mine[r * TOK + t] = acc[mt][nt][0];
            mine[r * TOK + t + 1] = acc[mt][nt][1];
            mine[(r + 8) * TOK + t] = acc[mt][nt][2];
            mine[(r + 8) * TOK + t + 1] = acc[mt][nt][3];
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * TOK; idx += GW * 32) {
        const int t = idx / ROWS, r = idx % ROWS;           // rows fastest: neighbouring threads write neighbours
        if (t < M && n0 + r < N) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < GW; ++w) sum += red[((size_t)w * ROWS + r) * TOK + t];
            out[(size_t)t * ldo + n0 + r] = cvt_out<OutT>(sum);
        }
    }
}

template <int NT, int MT, int U, typename OutT>
int launch(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, cudaStream_t stream) {
    const size_t smem = (size_t)GW * MT * 16 * NT * 8 * sizeof(float);
    auto kern = gemm_skinny_kernel<NT, MT, U, OutT>;
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
    }
    const int blocks = (N + MT * 16 - 1) / (MT * 16);
    kern<<<blocks, GW * 32, smem, stream>>>((const __nv_bfloat16*)X, ldx, (const __nv_bfloat16*)W, (OutT*)out, ldo, M, N, K);
    return (int)cudaGetLastError();
}

template <typename OutT>
int dispatch(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, cudaStream_t stream) {
    const bool wide = (N + 31) / 32 >= 2 * device_sms();          // enough 32-row blocks to fill the GPU twice
    if (M <= 8) return wide ? launch<1, 2, 4, OutT>(X, ldx, W, out, ldo, M, N, K, stream)
                            : launch<1, 1, 4, OutT>(X, ldx, W, out, ldo, M, N, K, stream);
    if (M <= 16) return wide ? launch<2, 2, 4, OutT>(X, ldx, W, out, ldo, M, N, K, stream)
                             : launch<2, 1, 4, OutT>(X, ldx, W, out, ldo, M, N, K, stream);
    if (M <= 32) return wide ? launch<4, 2, 2, OutT>(X, ldx, W, out, ldo, M, N, K, stream)
                             : launch<4, 1, 4, OutT>(X, ldx, W, out, ldo, M, N, K, stream);
    return wide ? launch<8, 2, 2, OutT>(X, ldx, W, out, ldo, M, N, K, stream)
                : launch<8, 1, 2, OutT>(X, ldx, W, out, ldo, M, N, K, stream);
}

}  // namespace

// out_dtype: MI_BF16 or MI_F32.  Returns -2 for shapes this kernel does not take (the caller
// then uses the library GEMM): M > 64, K not a multiple of 32, rows not 16-byte aligned.
MI_EXPORT int mi_gemm_skinny(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K,
                             int out_dtype, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (M > 64 || K % 32 || ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return -2;
    if (out_dtype == MI_F32) return dispatch<float>(X, ldx, W, out, ldo, M, N, K, stream);
    return dispatch<__nv_bfloat16>(X, ldx, W, out, ldo, M, N, K, stream);
}
