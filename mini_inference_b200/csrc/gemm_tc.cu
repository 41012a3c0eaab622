// Tensor-core GEMM for prompt steps on the 5th-generation tensor cores:
// out[M, N] = X[M, K] * W[N, K]^T, bfloat16 in, float32 accumulation in tensor memory.
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:141-143, 196, 125-126): the
// library GEMM behind F.linear, and for the feed-forward a separate silu(gate) * up pass over its
// result.  Here: a persistent kernel, one block per SM, that walks 128 x BN output tiles.
//   * warp 0 (one thread) streams [128 x 64] boxes of X and [BN x 64] boxes of W with TMA (128-byte
//     swizzle) into a ring of shared-memory stages and runs on into the next tile without a pause;
//   * warp 1 (one thread) issues tcgen05.mma (M = 128, N = BN, K = 16) on shared-memory
//     descriptors; the accumulator lives in tensor memory, which holds TWO of them, so the
//     products of the next tile start while the previous one is still being written out; each
//     stage is handed back to the loader, and each finished accumulator to the epilogue, by
//     tcgen05.commit;
//   * warps 2-5 read a finished accumulator with tcgen05.ld (one row per thread), convert and
//     store it.  In the gated mode the weight boxes of a tile are BN/2 rows of the gate half and
//     the matching BN/2 rows of the up half, so the epilogue has both and writes silu(gate) * up
//     directly: the [M, 2 I] intermediate never reaches memory.
// BN is chosen per shape so that the tiles fill whole waves of blocks (a narrow N with 256-wide
// tiles would leave most SMs idle in the last wave).  All mbarrier waits are bounded; a wait that
// runs out raises the error word and every role leaves its loop.
#include "sm100.cuh"
#include <map>
#include <mutex>
#include <tuple>

using namespace mi;
using namespace mi::sm100;

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int TC_THREADS = 192;
constexpr int ACC_COLS = 256;           // tensor-memory columns per accumulator (two of them: 512 = all of an SM's)

template <typename OutT> __device__ __forceinline__ void store_row32(OutT* dst, const float (&v)[32], int valid);
template <> __device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int valid) {
    if (valid >= 32 && ((uintptr_t)dst % 16 == 0)) {
#pragma unroll
        for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
        for (int i = 0; i < 32 && i < valid; ++i) dst[i] = v[i];
    }
}
template <> __device__ __forceinline__ void store_row32<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[32], int valid) {
    if (valid >= 32 && ((uintptr_t)dst % 16 == 0)) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 p;
            uint32_t* w = reinterpret_cast<uint32_t*>(&p);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * i + 2 * j], v[8 * i + 2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(dst)[i] = p;
        }
    } else {
        for (int i = 0; i < 32 && i < valid; ++i) dst[i] = __float2bfloat16_rn(v[i]);
    }
}

struct TcShape {
    int M, N, K;                        // N: rows of W (in the gated mode 2 I)
    int BN, NS;                         // tile width and ring stages
    int m_tiles, n_tiles;
    int ldo;
    int tma_out;                        // bfloat16 result with 16-byte aligned rows: the epilogue stores boxes with TMA
};

// GATED: W = [gate rows | up rows]; out [M, N / 2] = silu(x gate^T) * (x up^T), both products rounded to bfloat16 first
template <typename OutT, bool GATED>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
               const __grid_constant__ CUtensorMap omap, OutT* __restrict__ out, const TcShape sh, int* __restrict__ error_word) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int BN = sh.BN, NS = sh.NS, STAGE = A_BYTES + BN * BK * 2;
    // bfloat16 results leave through shared memory: per epilogue warp two [32 rows x 64 columns] boxes (128-byte swizzle)
    // that TMA stores write out as whole 128-byte lines (a thread storing its own row would touch 32 lines per instruction)
    unsigned char* stage_out = base + (size_t)NS * STAGE;
    constexpr int OUT_BYTES = sizeof(OutT) == 2 ? 4 * 2 * 4096 : 0;
    uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + OUT_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NS + 4);
    __shared__ volatile int abort_flag;
    const uint32_t stage0 = smem_u32(base), full0 = smem_u32(bars), empty0 = smem_u32(bars + NS);
    const uint32_t acc_full0 = smem_u32(bars + 2 * NS), acc_empty0 = smem_u32(bars + 2 * NS + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = sh.K / BK, tiles = sh.m_tiles * sh.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 4); }
        mbar_init_fence();
        abort_flag = 0;
        tma_prefetch_desc(&amap);
        tma_prefetch_desc(&bmap);
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 2 * ACC_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        // ---------------- loader: tiles in the order n fastest (blocks running together share rows of X and W in L2)
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < tiles && !abort_flag; tile += gridDim.x) {
                const int m0 = (tile / sh.n_tiles) * BM, nt = tile % sh.n_tiles;
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % NS;
                    if (it >= NS && !mbar_wait(empty0 + 8 * s, ((it / NS) - 1) & 1)) { atomicExch(error_word, 11); abort_flag = 1; }
                    if (abort_flag) break;
                    const uint32_t a_dst = stage0 + s * STAGE, b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full0 + 8 * s, STAGE);
                    tma_load_2d(a_dst, &amap, kc * BK, m0, full0 + 8 * s);
                    if (GATED) {                           // BN/2 gate rows and the BN/2 up rows of the same columns
                        const int half = BN / 2, inter = sh.N / 2;
                        tma_load_2d(b_dst, &bmap, kc * BK, nt * half, full0 + 8 * s);
                        tma_load_2d(b_dst + half * BK * 2, &bmap, kc * BK, inter + nt * half, full0 + 8 * s);
                    } else {
                        tma_load_2d(b_dst, &bmap, kc * BK, nt * BN, full0 + 8 * s);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: accumulator t & 1, handed to the epilogue when the tile's last product is done
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(BM, BN, false);
            int it = 0, t = 0;
            for (int tile = blockIdx.x; tile < tiles && !abort_flag; tile += gridDim.x, ++t) {
                const int b = t & 1;
                if (t >= 2 && !mbar_wait(acc_empty0 + 8 * b, ((t >> 1) - 1) & 1)) { atomicExch(error_word, 14); abort_flag = 1; break; }
                tc_fence_after();
                const uint32_t acc = tmem + b * ACC_COLS;
                for (int kc = 0; kc < nk; ++kc, ++it) {
                    const int s = it % NS;
                    if (!mbar_wait(full0 + 8 * s, (it / NS) & 1)) { atomicExch(error_word, 12); abort_flag = 1; }
                    if (abort_flag) break;
                    tc_fence_after();
                    const uint32_t a_addr = stage0 + s * STAGE, b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_ss(acc, umma_desc_sw128(a_addr + 32 * k, 16, 1024), umma_desc_sw128(b_addr + 32 * k, 16, 1024),
                                idesc, (kc | k) != 0);
                    umma_commit(empty0 + 8 * s);           // the stage is free once these MMAs have read it
                }
                if (abort_flag) break;
                umma_commit(acc_full0 + 8 * b);            // the accumulator is complete
            }
        }
    } else {
        // ---------------- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. +31, one row per thread
        const int lg = warp & 3;
        int t = 0, groups = 0;
        for (int tile = blockIdx.x; tile < tiles && !abort_flag; tile += gridDim.x, ++t) {
            const int b = t & 1;
            const int m0 = (tile / sh.n_tiles) * BM, nt = tile % sh.n_tiles;
            const int row = m0 + lg * 32 + lane;
            if (!mbar_wait(acc_full0 + 8 * b, (t >> 1) & 1)) { atomicExch(error_word, 13); abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t acc = tmem + ((uint32_t)(lg * 32) << 16) + b * ACC_COLS;
            const int n_out = GATED ? sh.N / 2 : sh.N;                  // columns of the result
            const int per_tile = GATED ? BN / 2 : BN;
            if (sh.tma_out) {
                // 64 result columns at a time: tensor memory -> registers -> swizzled box -> TMA store
                unsigned char* my_out = stage_out + (warp - 2) * 8192;
                for (int c = 0; c < per_tile / 64; ++c) {
                    float v[64];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int col_in = c * 64 + h * 32;                 // within the tile's result columns
                        if (col_in < per_tile) {
                            uint32_t ra[32];
                            tmem_ld32(acc + col_in, ra);
                            if (GATED) {
                                uint32_t ru[32];
                                tmem_ld32(acc + BN / 2 + col_in, ru);
                                tmem_wait_ld();
#pragma unroll
                                for (int i = 0; i < 32; ++i) {
                                    const float gt = round_to<__nv_bfloat16>(__uint_as_float(ra[i])), up = round_to<__nv_bfloat16>(__uint_as_float(ru[i]));
                                    v[h * 32 + i] = gt / (1.f + expf(-gt)) * up;
                                }
                            } else {
                                tmem_wait_ld();
#pragma unroll
                                for (int i = 0; i < 32; ++i) v[h * 32 + i] = __uint_as_float(ra[i]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[h * 32 + i] = 0.f;
                        }
                    }
                    unsigned char* box = my_out + (groups & 1) * 4096;
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");   // the store two boxes back has read its box
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 p;
                        uint32_t* w = reinterpret_cast<uint32_t*>(&p);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 hh = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
                            w[e] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) = p;
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        const int col = nt * per_tile + c * 64, row0 = m0 + lg * 32;
                        if (col < n_out && row0 < sh.M) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];\n"
                                         :: "l"((uint64_t)&omap), "r"(col), "r"(row0), "r"(smem_u32(box)) : "memory");
                        }
                        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    }
                    ++groups;
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(acc + c * 32, r);
                    tmem_wait_ld();
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                    const int col = nt * BN + c * 32;
                    if (row < sh.M && col < sh.N) store_row32<OutT>(out + (size_t)row * sh.ldo + col, v, sh.N - col);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty0 + 8 * b);  // this warp has read its lanes of the accumulator
        }
        if (sh.tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // the stores have landed
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, 2 * ACC_COLS);
}

std::mutex tc_mutex;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> tc_weight_maps;
int tc_sms = 0;

// tile width: fill whole waves of blocks; per 64 of K a tile costs max(2 BN, 128 + BN) clocks (tensor pipe / shared memory)
int choose_bn(int m_tiles, int n_cols, int sms, bool gated, int col_step) {
    int best = 256;
    long long best_cost = -1;
    for (int bn = 256; bn >= 64; bn -= 32) {
        const int per_tile = gated ? bn / 2 : bn;
        if ((gated && bn % 64) || per_tile % col_step) continue;     // the epilogue writes col_step result columns at a time
        const long long n_tiles = (n_cols + per_tile - 1) / per_tile;
        const long long waves = (m_tiles * n_tiles + sms - 1) / sms;
        const long long cost = waves * (2 * bn > 128 + bn ? 2 * bn : 128 + bn);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

template <typename OutT, bool GATED>
int launch_tc(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, int* error_word, cudaStream_t stream) {
    if (!tc_sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return -4;
        cudaDeviceGetAttribute(&tc_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    TcShape sh;
    sh.M = M; sh.N = N; sh.K = K; sh.ldo = ldo;
    sh.m_tiles = (M + BM - 1) / BM;
    const int n_cols = GATED ? N / 2 : N;
    sh.tma_out = sizeof(OutT) == 2 && ldo % 8 == 0 && ((uintptr_t)out % 16 == 0);
    if (GATED && !sh.tma_out) return -2;
    sh.BN = choose_bn(sh.m_tiles, n_cols, tc_sms, GATED, sh.tma_out ? 64 : 32);
    const int per_tile = GATED ? sh.BN / 2 : sh.BN;
    sh.n_tiles = (n_cols + per_tile - 1) / per_tile;
    const int stage = A_BYTES + sh.BN * BK * 2;
    sh.NS = (226 * 1024 - 2048 - (sizeof(OutT) == 2 ? 4 * 2 * 4096 : 0)) / stage;
    if (sh.NS > 8) sh.NS = 8;
    if (sh.NS < 2) return -2;
    CUtensorMap amap, bmap;
    if (!sm100_host::make_map_bf16(&amap, X, M, K, ldx, BM, BK)) return -5;
    {
        std::lock_guard<std::mutex> lock(tc_mutex);
        auto key = std::make_tuple(W, N, K, per_tile);
        auto it = tc_weight_maps.find(key);
        if (it == tc_weight_maps.end()) {
            CUtensorMap m;
            if (!sm100_host::make_map_bf16(&m, W, N, K, K, per_tile, BK)) return -5;
            it = tc_weight_maps.emplace(key, m).first;
        }
        bmap = it->second;
    }
    const size_t out_bytes = sizeof(OutT) == 2 ? 4 * 2 * 4096 : 0;
    const size_t smem = (size_t)sh.NS * stage + out_bytes + (2 * sh.NS + 4) * 8 + 16 + 1024;
    CUtensorMap omap = amap;
    if (sh.tma_out && !sm100_host::make_map_bf16(&omap, out, M, n_cols, ldo, 32, 64)) return -5;
    auto kern = gemm_tc_kernel<OutT, GATED>;
    static size_t configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);   // + static < 227 KB
        if (e != cudaSuccess) return (int)e;
        configured = 226 * 1024;
    }
    const int tiles = sh.m_tiles * sh.n_tiles;
    const int grid = tiles < tc_sms ? tiles : tc_sms;
    return (int)launch_pdl(kern, dim3(grid), dim3(TC_THREADS), smem, stream, amap, bmap, omap, (OutT*)out, sh, error_word);
}

}  // namespace

// Returns -2 for shapes it does not take (K not a multiple of 64, unaligned rows): the caller uses the library GEMM.
MI_EXPORT int mi_gemm_tc(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, int out_dtype,
                         int* error_word, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return -2;
    if (out_dtype == MI_F32) return launch_tc<float, false>(X, ldx, W, out, ldo, M, N, K, error_word, stream);
    return launch_tc<__nv_bfloat16, false>(X, ldx, W, out, ldo, M, N, K, error_word, stream);
}

// act[M, I] = silu(g) * u with [g | u] = X[M, K] * W[2 I, K]^T (both rounded to bfloat16 first, as the separate kernels
// do); bfloat16 out.  Returns -2 for shapes it does not take (also I not a multiple of 8).
MI_EXPORT int mi_gemm_tc_swiglu(const void* X, int ldx, const void* W, void* act, int M, int inter, int K, int* error_word,
                                cudaStream_t stream) {
    if (M == 0 || inter == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || inter % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16) || ((uintptr_t)act % 16)) return -2;
    return launch_tc<__nv_bfloat16, true>(X, ldx, W, act, inter, M, 2 * inter, K, error_word, stream);
}
