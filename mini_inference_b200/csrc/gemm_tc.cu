// Tensor-core GEMM for prompt steps on the 5th-generation tensor cores:
// out[M, N] = X[M, K] * W[N, K]^T, bfloat16 in, float32 accumulation in tensor memory.
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:141-143, 196, 125-126): the
// library GEMM behind F.linear.  Here: one block per 128 x BN output tile; warp 0 streams
// [128 x 64] boxes of X and [BN x 64] boxes of W with TMA (128-byte swizzle) into a ring of
// shared-memory stages; one thread of warp 1 issues tcgen05.mma (M = 128, N = BN, K = 16) on
// shared-memory descriptors, the accumulator lives in BN columns of tensor memory, and each
// stage is handed back to the loader by tcgen05.commit; warps 2-5 read the finished accumulator
// with tcgen05.ld (one row per thread) and store it.  All mbarrier waits are bounded.
#include "sm100.cuh"
#include <map>
#include <mutex>
#include <tuple>

using namespace mi;
using namespace mi::sm100;

namespace {

constexpr int BM = 128, BK = 64;
constexpr int TC_THREADS = 192;

template <typename OutT> __device__ __forceinline__ void store_row32(OutT* dst, const uint32_t (&r)[32], int valid);
template <> __device__ __forceinline__ void store_row32<float>(float* dst, const uint32_t (&r)[32], int valid) {
    if (valid >= 32 && ((uintptr_t)dst % 16 == 0)) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                            __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
    } else {
        for (int i = 0; i < 32 && i < valid; ++i) dst[i] = __uint_as_float(r[i]);
    }
}
template <> __device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&r)[32], int valid) {
    if (valid >= 32 && ((uintptr_t)dst % 16 == 0)) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 v;
            uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2 * j]), __uint_as_float(r[8 * i + 2 * j + 1]));
                w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(dst)[i] = v;
        }
    } else {
        for (int i = 0; i < 32 && i < valid; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
    }
}

template <int BN, int NS, typename OutT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap, OutT* __restrict__ out,
               int ldo, int M, int N, int K, int* __restrict__ error_word) {
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + NS * STAGE);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NS + 1);
    const uint32_t stage0 = smem_u32(base), full0 = smem_u32(bars), empty0 = smem_u32(bars + NS), accum_bar = smem_u32(bars + 2 * NS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nk = K / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accum_bar, 1);
        mbar_init_fence();
        tma_prefetch_desc(&amap);
        tma_prefetch_desc(&bmap);
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            for (int kc = 0; kc < nk; ++kc) {
                const int s = kc % NS;
                if (kc >= NS && !mbar_wait(empty0 + 8 * s, ((kc / NS) - 1) & 1)) { atomicExch(error_word, 11); break; }
                mbar_expect_tx(full0 + 8 * s, STAGE);
                tma_load_2d(stage0 + s * STAGE, &amap, kc * BK, m0, full0 + 8 * s);
                tma_load_2d(stage0 + s * STAGE + A_BYTES, &bmap, kc * BK, n0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(BM, BN, false);
            bool ok = true;
            for (int kc = 0; kc < nk && ok; ++kc) {
                const int s = kc % NS;
                if (!mbar_wait(full0 + 8 * s, (kc / NS) & 1)) { atomicExch(error_word, 12); ok = false; break; }
                tc_fence_after();
                const uint32_t a_addr = stage0 + s * STAGE, b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)
                    umma_ss(tmem, umma_desc_sw128(a_addr + 32 * k, 16, 1024), umma_desc_sw128(b_addr + 32 * k, 16, 1024),
                            idesc, (kc | k) != 0);
                umma_commit(empty0 + 8 * s);             // the stage is free once these MMAs have read it
            }
            umma_commit(accum_bar);                       // the accumulator is complete
        }
    } else {
        // ---------------- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. +31, one row per thread
        const int lg = warp & 3;
        const int row = m0 + lg * 32 + lane;
        if (mbar_wait(accum_bar, 0)) {
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(lg * 32) << 16) + c * 32, r);
                tmem_wait_ld();
                const int col = n0 + c * 32;
                if (row < M && col < N) store_row32<OutT>(out + (size_t)row * ldo + col, r, N - col);
            }
        } else {
            atomicExch(error_word, 13);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, BN);
}

std::mutex tc_mutex;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> tc_weight_maps;

template <int BN, int NS, typename OutT>
int launch_tc(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, int* error_word, cudaStream_t stream) {
    CUtensorMap amap, bmap;
    if (!sm100_host::make_map_bf16(&amap, X, M, K, ldx, BM, BK)) return -5;
    {
        std::lock_guard<std::mutex> lock(tc_mutex);
        auto key = std::make_tuple(W, N, K, BN);
        auto it = tc_weight_maps.find(key);
        if (it == tc_weight_maps.end()) {
            CUtensorMap m;
            if (!sm100_host::make_map_bf16(&m, W, N, K, K, BN, BK)) return -5;
            it = tc_weight_maps.emplace(key, m).first;
        }
        bmap = it->second;
    }
    const size_t smem = (size_t)NS * (BM * BK * 2 + BN * BK * 2) + (2 * NS + 1) * 8 + 16 + 1024;
    auto kern = gemm_tc_kernel<BN, NS, OutT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    return (int)launch_pdl(kern, grid, dim3(TC_THREADS), smem, stream, amap, bmap, (OutT*)out, ldo, M, N, K, error_word);
}

}  // namespace

// Returns -2 for shapes it does not take (K not a multiple of 64, unaligned rows): the caller uses the library GEMM.
MI_EXPORT int mi_gemm_tc(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, int out_dtype,
                         int* error_word, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return -2;
    const long long tiles256 = (long long)((N + 255) / 256) * ((M + BM - 1) / BM);
    const bool wide = N >= 256 && (tiles256 >= 2 * 148 || tiles256 % 148 == 0 || tiles256 % 148 > 74);
    if (out_dtype == MI_F32)
        return wide ? launch_tc<256, 4, float>(X, ldx, W, out, ldo, M, N, K, error_word, stream)
                    : launch_tc<128, 6, float>(X, ldx, W, out, ldo, M, N, K, error_word, stream);
    return wide ? launch_tc<256, 4, __nv_bfloat16>(X, ldx, W, out, ldo, M, N, K, error_word, stream)
                : launch_tc<128, 6, __nv_bfloat16>(X, ldx, W, out, ldo, M, N, K, error_word, stream);
}
