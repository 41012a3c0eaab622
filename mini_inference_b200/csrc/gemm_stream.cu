// Persistent weight-streaming GEMM for decode steps: out[M, N] = X[M, K] * W[N, K]^T, M <= 32,
// bfloat16 in, float32 accumulation.  TMA + mbarrier pipeline, stream-K work split.
//
// Reference (davidjoyme/mini-inference engine/core/fused_linear.py:29-34): the library GEMM; its
// own measurements (README.md:29, results/micro/gemm_qwen3.json) put the skinny decode products
// at 17-83 % of peak bandwidth, worst for the narrow ones (o, down) where few tiles exist and
// whole waves of blocks go idle.  This kernel is organised around the one thing that matters at
// these shapes, keeping every SM's HBM pipe full for the whole call:
//   * one persistent block per SM; a producer thread streams [128 rows x 64 k] weight boxes
//     with TMA (cp.async.bulk.tensor, 128-byte swizzle) into an 8-stage ring (128 KB in flight
//     per SM), signalled by mbarriers; 8 consumer warps turn each box into mma.sync work
//     ("swap-AB": weight rows are the 16-row side, tokens the 8-wide side);
//   * stream-K: the (row tile, k chunk) units of the whole matrix are cut into equal contiguous
//     shares, one per block, whatever N and K are, so no SM waits for a straggler; a row tile
//     cut between blocks is finished by whichever block arrives last, which adds the partial
//     sums in the fixed order of the shares (not of arrival).  The split depends on (N, K, grid)
//     only, never on M, so a token's result does not depend on its company in the batch.
// Every wait on an mbarrier is bounded; a wait that runs out raises an error word and the block
// leaves.  No cluster multicast is used.
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>
#include <map>
#include <mutex>
#include <tuple>

using namespace mi;

namespace {

constexpr int TR = 128;                 // weight rows per tile
constexpr int KC = 64;                  // k per stage (128 bytes: one swizzle row)
constexpr int NS = 8;                   // ring stages
constexpr int STAGE_BYTES = TR * KC * 2;
constexpr int CONSUMERS = 8;            // consumer warps, 16 rows each
constexpr int THREADS = 32 * (1 + CONSUMERS);
constexpr uint32_t SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false when the barrier did not flip within the limit
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i > 64) __nanosleep(40);
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 :: "r"(dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" :: "n"(CONSUMERS * 32) : "memory"); }
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename OutT> __device__ __forceinline__ OutT cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// block that owns unit u when U units are cut into G contiguous shares [floor(U b / G), floor(U (b+1) / G))
__device__ __forceinline__ int owner_of(long long u, long long U, long long G) { return (int)(((u + 1) * G + U - 1) / U - 1); }

template <int NT, typename OutT>
// The register count of the 8-token instance matters beyond this kernel (tests/test_kernel_resources.py guards it): at 112
// registers a decode step at Qwen3-4B sizes takes 3.05 ms, at 115 (an unrelated, never executed branch more in the
// producer) 3.49 ms, while the kernel timed alone is equally fast either way.  Inside a step the blocks of the kernels
// around it share the SMs with this one (programmatic dependent launch); past 112 registers a thread they no longer fit.
// The arithmetic that matches: an SM's registers are four banks of 16,384, one per scheduler; the fullest bank holds 3 of
// this block's 9 warps and must also take 5 of the 20 warps (32 registers each) of the residual-add + norm block that
// follows: 3 * 32 * r + 5 * 32 * 32 <= 16,384 gives r <= 117, and registers are handed out in eights.
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   OutT* __restrict__ out, int ldo, int M, int N, int K, float* __restrict__ workspace, int max_contrib,
                   int* __restrict__ counters, int* __restrict__ error_word) {
    constexpr int TOK = NT * 8;
    constexpr int X_BYTES = TOK * KC * 2;                  // the tokens' slice of the same k chunk
    constexpr int STAGE = STAGE_BYTES + X_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + NS * STAGE);
    __shared__ int last_flag;
    const uint32_t stage0 = smem_u32(base), full0 = smem_u32(bars), empty0 = smem_u32(bars + NS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, CONSUMERS); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();                                         // the next kernel may begin its own preamble

    const int NKC = K / KC, NRT = (N + TR - 1) / TR;
    const long long U = (long long)NRT * NKC, G = gridDim.x;
    const long long u0 = U * blockIdx.x / G, u1 = U * (blockIdx.x + 1) / G;

    if (warp == 0) {
        // ---------------- producer: one thread keeps the ring full.  Weights do not depend on the
        // kernel before this one, so the first ring-full of weight boxes is requested BEFORE waiting
        // for it; the activations of those stages follow once it has finished.
        if (lane == 0) {
            const int ahead = (int)((u1 - u0) < NS ? (u1 - u0) : NS);
            for (int i = 0; i < ahead; ++i) {
                const long long u = u0 + i;
                mbar_expect_tx(full0 + 8 * i, STAGE);
                tma_load_2d(stage0 + i * STAGE, &wmap, (int)(u % NKC) * KC, (int)(u / NKC) * TR, full0 + 8 * i);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d(stage0 + i * STAGE + STAGE_BYTES, &xmap, (int)((u0 + i) % NKC) * KC, 0, full0 + 8 * i);
            for (long long u = u0 + ahead; u < u1; ++u) {
                const int i = (int)(u - u0), s = i % NS;
                if (!mbar_wait(empty0 + 8 * s, ((i / NS) - 1) & 1)) { atomicExch(error_word, 1); break; }
                const int rt = (int)(u / NKC), kc = (int)(u % NKC);
                mbar_expect_tx(full0 + 8 * s, STAGE);
                tma_load_2d(stage0 + s * STAGE, &wmap, kc * KC, rt * TR, full0 + 8 * s);
                tma_load_2d(stage0 + s * STAGE + STAGE_BYTES, &xmap, kc * KC, 0, full0 + 8 * s);
            }
        }
        return;
    }

    // ---------------- consumers: warp cw owns rows cw*16 .. cw*16+15 of every tile
    const int cw = warp - 1, g = lane >> 2, c = lane & 3;
    const int ctid = threadIdx.x - 32;
    pdl_wait();                                            // before the first write to out / workspace
    // four independent accumulation chains per token group (one per 16 k of a stage), added in a fixed order at the
    // end of a share: a chain of dependent mma.sync would leave the warp waiting on each one's latency
    float chain[NT][4][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) { chain[nt][q][0] = chain[nt][q][1] = chain[nt][q][2] = chain[nt][q][3] = 0.f; }
    const int r_lo = cw * 16 + g, r_hi = r_lo + 8;
    int seg_start_kc = (int)(u0 % NKC);

    for (long long u = u0; u < u1; ++u) {
        const int i = (int)(u - u0), s = i % NS;
        const int rt = (int)(u / NKC), kc = (int)(u % NKC);
        if (!mbar_wait(full0 + 8 * s, (i / NS) & 1)) { atomicExch(error_word, 2); return; }
        const unsigned char* st = base + s * STAGE;
        const unsigned char* xs = st + STAGE_BYTES;
        // chunk 2c + win: the eight lanes of a quarter-warp then read eight different 16-byte columns of the
        // swizzled rows (no bank conflicts); which k a lane takes does not matter as long as A and B agree
#pragma unroll
        for (int win = 0; win < 2; ++win) {
            const int ch = 2 * c + win;
            const uint4 a_lo = *reinterpret_cast<const uint4*>(st + r_lo * 128 + ((ch ^ (r_lo & 7)) << 4));
            const uint4 a_hi = *reinterpret_cast<const uint4*>(st + r_hi * 128 + ((ch ^ (r_hi & 7)) << 4));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int t = nt * 8 + g;                  // rows beyond M were filled with zeros by the copy
                const uint4 b = *reinterpret_cast<const uint4*>(xs + t * 128 + ((ch ^ (t & 7)) << 4));
                mma16816(chain[nt][2 * win], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
                mma16816(chain[nt][2 * win + 1], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * s);

        if (kc != NKC - 1 && u != u1 - 1) continue;
        // ---------------- this block's share of row tile rt ends here
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int f = 0; f < 4; ++f) acc[nt][f] = (chain[nt][0][f] + chain[nt][1][f]) + (chain[nt][2][f] + chain[nt][3][f]);
        const bool whole = seg_start_kc == 0 && kc == NKC - 1;
        if (whole && counters != nullptr) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int t = nt * 8 + 2 * c, n_lo = rt * TR + r_lo, n_hi = rt * TR + r_hi;
                if (t < M) {
                    if (n_lo < N) out[(size_t)t * ldo + n_lo] = cvt_out<OutT>(acc[nt][0]);
                    if (n_hi < N) out[(size_t)t * ldo + n_hi] = cvt_out<OutT>(acc[nt][2]);
                }
                if (t + 1 < M) {
                    if (n_lo < N) out[(size_t)(t + 1) * ldo + n_lo] = cvt_out<OutT>(acc[nt][1]);
                    if (n_hi < N) out[(size_t)(t + 1) * ldo + n_hi] = cvt_out<OutT>(acc[nt][3]);
                }
            }
        } else {
            const long long first_unit = (long long)rt * NKC;
            const int first = owner_of(first_unit, U, G), last = owner_of(first_unit + NKC - 1, U, G);
            const int slot = (int)blockIdx.x - first, contrib = last - first + 1;
            float* mine = workspace + ((size_t)rt * max_contrib + slot) * TR * TOK;     // [token][row]
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int t = nt * 8 + 2 * c;
                mine[t * TR + r_lo] = acc[nt][0]; mine[(t + 1) * TR + r_lo] = acc[nt][1];
                mine[t * TR + r_hi] = acc[nt][2]; mine[(t + 1) * TR + r_hi] = acc[nt][3];
            }
            // deferred mode (no counters): the partial sums are the result; whoever reads them adds the shares of a
            // tile in order (mi_deferred_add_rmsnorm / mi_deferred_reduce), and this kernel has no fix-up tail
            if (counters != nullptr) {
            __threadfence();
            consumer_sync();
            if (ctid == 0) last_flag = atomicAdd(&counters[rt], 1) == contrib - 1;
            consumer_sync();
            if (last_flag) {                                   // every other share of this tile is in the workspace
                __threadfence();
                // four rows of one token per thread, every share's piece requested before the first is added (in share
                // order): the block that arrives last is on the kernel's critical path, so this is one round trip to L2
                const float* tile_ws = workspace + (size_t)rt * max_contrib * TR * TOK;
                for (int idx = ctid; idx < TR * TOK / 4; idx += CONSUMERS * 32) {
                    const int t = idx / (TR / 4), r = (idx % (TR / 4)) * 4;
                    if (t >= M || rt * TR + r >= N) continue;
                    const float* src = tile_ws + (size_t)t * TR + r;
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int k0 = 0; k0 < contrib; k0 += 12) {
                        float4 v[12];
#pragma unroll
                        for (int j = 0; j < 12; ++j)
                            v[j] = k0 + j < contrib ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(k0 + j) * TR * TOK))
                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int j = 0; j < 12; ++j) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
                    }
                    OutT* dst = out + (size_t)t * ldo + rt * TR + r;
                    const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (rt * TR + r + e < N) dst[e] = cvt_out<OutT>(vals[e]);
                }
                if (ctid == 0) counters[rt] = 0;               // ready for the next call
            }
            }
            consumer_sync();
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) { chain[nt][q][0] = chain[nt][q][1] = chain[nt][q][2] = chain[nt][q][3] = 0.f; }
        seg_start_kc = 0;
    }
}

// ---------------------------------------------------------------- host side
PFN_cuTensorMapEncodeTiled encode_fn = nullptr;
std::mutex host_mutex;
std::map<std::tuple<const void*, int, int>, CUtensorMap> weight_maps;
int sm_count = 0;

int get_weight_map(const void* W, int N, int K, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(host_mutex);
    if (!encode_fn) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -4;
        encode_fn = (PFN_cuTensorMapEncodeTiled)fn;
    }
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    }
    auto key = std::make_tuple(W, N, K);
    auto it = weight_maps.find(key);
    if (it == weight_maps.end()) {
        CUtensorMap m;
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {KC, TR};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = encode_fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(W), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return -5;
        it = weight_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

template <int NT, typename OutT>
int launch(const CUtensorMap& map, const void* X, int ldx, void* out, int ldo, int M, int N, int K, float* workspace,
           int max_contrib, int* counters, int* error_word, int grid, cudaStream_t stream) {
    // the activations' map is made per call: their address changes from call to call
    CUtensorMap xmap;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
        const cuuint32_t box[2] = {KC, NT * 8};
        const cuuint32_t estr[2] = {1, 1};
        if (encode_fn(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(X), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return -5;
    }
    const size_t smem = (size_t)NS * (STAGE_BYTES + NT * 8 * KC * 2) + 2 * NS * 8 + 1024;
    auto kern = gemm_stream_kernel<NT, OutT>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return (int)launch_pdl(kern, dim3(grid), dim3(THREADS), smem, stream, map, xmap, (OutT*)out, ldo, M, N, K, workspace,
                           max_contrib, counters, error_word);
}

}  // namespace

// Work-split facts the caller needs to size the scratch: grid (blocks), row tiles, and the most
// blocks that can share one row tile.  Returns -2 when the shape is not taken (K % 64, M > 32).
MI_EXPORT int mi_gemm_stream_plan(int M, int N, int K, int* grid, int* row_tiles, int* max_contrib) {
    if (M < 1 || M > 32 || K % KC || K < KC || N < 1) return -2;
    if (!sm_count) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return -4;
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    }
    const long long NKC = K / KC, NRT = (N + TR - 1) / TR, U = NRT * NKC;
    const long long G = U < sm_count ? U : sm_count;
    const long long share = U / G;                       // smallest share
    *grid = (int)G;
    *row_tiles = (int)NRT;
    *max_contrib = (int)((NKC + share - 1) / share + 1);
    return 0;
}

// workspace: float32 [row_tiles * max_contrib * 128 * tokens_padded] with tokens_padded = 8, 16 or 32 for
// M <= 8, 16, 32; counters: int32 [row_tiles], zero before the first call (the kernel leaves them zero);
// error_word: int32, set non-zero if a bounded wait inside the kernel ran out.
MI_EXPORT int mi_gemm_stream(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K,
                             int out_dtype, float* workspace, int* counters, int* error_word, cudaStream_t stream) {
    int grid, row_tiles, max_contrib;
    int rc = mi_gemm_stream_plan(M, N, K, &grid, &row_tiles, &max_contrib);
    if (rc) return rc;
    if (ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16) || (K * 2) % 16) return -2;
    CUtensorMap map;
    rc = get_weight_map(W, N, K, &map);
    if (rc) return rc;
#define GO(NT, OT) launch<NT, OT>(map, X, ldx, out, ldo, M, N, K, workspace, max_contrib, counters, error_word, grid, stream)
    if (out_dtype == MI_F32) return M <= 8 ? GO(1, float) : M <= 16 ? GO(2, float) : GO(4, float);
    return M <= 8 ? GO(1, __nv_bfloat16) : M <= 16 ? GO(2, __nv_bfloat16) : GO(4, __nv_bfloat16);
#undef GO
}

// The same product left as partial sums: workspace [row_tiles][max_contrib][tokens_padded][128] float32 holds, for every
// row tile, the shares of the blocks that worked on it (share s of tile t came from block first_owner(t) + s); nothing is
// added up and nothing is written elsewhere.  mi_deferred_add_rmsnorm (the usual next kernel) or mi_deferred_reduce adds
// the shares in order.  Same shapes and return codes as mi_gemm_stream.
MI_EXPORT int mi_gemm_stream_deferred(const void* X, int ldx, const void* W, int M, int N, int K, float* workspace,
                                      int* error_word, cudaStream_t stream) {
    int grid, row_tiles, max_contrib;
    int rc = mi_gemm_stream_plan(M, N, K, &grid, &row_tiles, &max_contrib);
    if (rc) return rc;
    if (ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16) || (K * 2) % 16) return -2;
    CUtensorMap map;
    rc = get_weight_map(W, N, K, &map);
    if (rc) return rc;
#define GO(NT) launch<NT, __nv_bfloat16>(map, X, ldx, nullptr, 0, M, N, K, workspace, max_contrib, nullptr, error_word, grid, stream)
    return M <= 8 ? GO(1) : M <= 16 ? GO(2) : GO(4);
#undef GO
}
