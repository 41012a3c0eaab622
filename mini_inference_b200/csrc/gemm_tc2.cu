// Two-block tensor-core GEMM for prompt steps (tcgen05 with cta_group::2):
// out[M, N] = X[M, K] * W[N, K]^T, bfloat16 in and out, float32 accumulation in tensor memory.
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:141-143, 196, 125-126): the
// library GEMM behind F.linear, and for the feed-forward a separate silu(gate) * up pass over its
// result.  Two blocks on neighbouring SMs (a cluster of 2) share one 256 x 256 tile: each loads ITS
// 128 rows of X and ITS half of the tile's 256 rows of W (64 KB of operands per 4.2 M multiply-adds;
// a one-block 128 x 256 tile needs 48 KB per 2.1 M), and one thread of the even block issues
// tcgen05.mma.cta_group::2 (M = 256), which reads both blocks' shared memory and writes 128
// accumulator rows into each block's tensor memory.  A persistent grid walks the tiles m fastest, so
// the pairs that run together share a few tiles of W.
//   warp 0 (one thread, both blocks)  TMA loads (cp.async.bulk.tensor with cta_group::2 and NO multicast: every
//            box goes to the issuing block's own shared memory; its bytes are counted on the EVEN block's
//            mbarrier, which that block's loader arms with the bytes of both)
//   warp 1   even block: MMA issue; a stage is handed back to both loaders, a finished accumulator to both
//            epilogues, by tcgen05.commit with a multicast mask.  Both blocks: tensor-memory allocation.
//   warps 2-5 (both blocks)  epilogue: read the block's own 128 accumulator rows with tcgen05.ld, convert,
//            write [32 x 64] swizzled boxes to shared memory and store them with TMA; then tell the even
//            block's accumulator-empty barrier (the odd block's warps arrive there remotely).
// Gated mode: the tile's BN weight rows are BN/2 gate rows (loaded by the even block) and the matching BN/2
// up rows (loaded by the odd block); the epilogue writes silu(gate) * up.
// Two accumulators of 256 columns fill the 512 columns of tensor memory, so a tile's epilogue overlaps
// the next tile's products.  Every mbarrier wait is bounded; a wait that runs out raises the error word and
// every role leaves its loop; both blocks always reach the closing cluster barrier.
//
// Measured (2,048 rows, Qwen3-4B shapes, graph-timed): gate/up 185 us = 1.10 PFLOP/s, qkv 69 us = 0.93 (192 tiles on
// 74 pairs: 2.6 waves), against the library's 138 us = 1.47 and 47 us = 1.37.  With the loads taken out the same
// instruction stream runs in 141 us (1.44 PFLOP/s), with the epilogue taken out as well no faster, and with only the X
// loads or only the W loads still 191 us: the gap to the library is in the load -> MMA hand-over per 64 of K, not in the
// bytes, the ring depth (3 stages: 199 us, 6: 191) or the epilogue.  Tiles narrower than 256 columns lose outright: an MMA of
// 128 columns takes ~150 clocks where 64 are nominal.  So the engine leaves prompt-step products on the library GEMM unless
// MI_TC_GEMM=1.
#include "sm100.cuh"
#include <map>
#include <mutex>
#include <tuple>

using namespace mi;
using namespace mi::sm100;

namespace {

constexpr int BM = 128, BK = 64;                 // rows per block (256 per tile), k per TMA box (128 bytes: one swizzle row)
constexpr int KSUB = 2;                          // boxes along k per ring stage: a stage holds 128 of K
constexpr int A_SUB = BM * BK * 2;               // bytes of one box of X
constexpr int A_BYTES = KSUB * A_SUB;
constexpr int T2_THREADS = 192;
constexpr int ACC_COLS = 256;
constexpr int OUT_BYTES = 4 * 2 * 4096;          // per epilogue warp two [32 x 64] bfloat16 boxes

__device__ __forceinline__ uint32_t cta_rank_in_cluster() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the same shared-memory variable in block `rank` of the cluster, as a shared::cluster address
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" :: "r"(cluster_addr) : "memory");
}
// box -> this block's shared memory; the bytes are counted on the mbarrier at `bar_cluster` (a shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 :: "r"(dst), "l"((uint64_t)map), "r"(x), "r"(y), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" :: "r"(smem_slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" :: "r"(taddr), "r"(cols) : "memory");
}
// D[tensor memory of both blocks] (+)= A[both blocks' rows] * B[both blocks' halves]; issued by ONE thread of the even block
__device__ __forceinline__ void umma_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                 " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate), "r"(0u) : "memory");
}
// one arrival on the mbarrier at this shared-memory offset in every block of `mask` when the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 :: "r"(bar), "h"(mask) : "memory");
}

struct T2Shape {
    int M, N, K;                        // N: rows of W (in the gated mode 2 I)
    int BN, NS;
    int m_tiles, n_tiles;               // tiles of 256 rows x (BN or BN/2 result columns)
};

template <bool GATED>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
                const __grid_constant__ CUtensorMap omap, const T2Shape sh, int* __restrict__ error_word) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int BN = sh.BN, NS = sh.NS, HALF = BN / 2;
    const int B_SUB = HALF * BK * 2, B_BYTES = KSUB * B_SUB, STAGE = A_BYTES + B_BYTES;
    unsigned char* stage_out = base + (size_t)NS * STAGE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(stage_out + OUT_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NS + 4);
    __shared__ volatile int abort_flag;
    const uint32_t stage0 = smem_u32(base), full0 = smem_u32(bars), empty0 = smem_u32(bars + NS);
    const uint32_t acc_full0 = smem_u32(bars + 2 * NS), acc_empty0 = smem_u32(bars + 2 * NS + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cta_rank_in_cluster();         // 0: the block that issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int nk = (sh.K + KSUB * BK - 1) / (KSUB * BK), tiles = sh.m_tiles * sh.n_tiles;   // a box beyond K reads zeros

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full0 + 8 * b, 1); mbar_init(acc_empty0 + 8 * b, 8); }
        mbar_init_fence();
        abort_flag = 0;
        tma_prefetch_desc(&amap);
        tma_prefetch_desc(&bmap);
    }
    __syncthreads();
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 2 * ACC_COLS);
    tc_fence_before();
    cluster_barrier();                                   // both blocks' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        // ---------------- loader (both blocks): this block's rows of X and its half of the tile's rows of W.  Tiles in the
        // order m fastest: the pairs that run together share a few tiles of W, which then comes from memory once
        if (lane == 0) {
            const uint32_t full_even0 = map_to_rank(full0, 0);
            int s = 0, round = 0;                           // ring stage and how often the ring has been filled
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs) {
                const int m0 = (tile % sh.m_tiles) * 2 * BM + (int)rank * BM, nt = tile / sh.m_tiles;
                const int b_row = GATED ? (int)rank * (sh.N / 2) + nt * HALF : nt * BN + (int)rank * HALF;
                for (int kc = 0; kc < nk; ++kc) {
                    if (round > 0 && !mbar_spin(empty0 + 8 * s, (round - 1) & 1)) { atomicExch(error_word, 51); abort_flag = 1; ok = false; break; }
                    const uint32_t a_dst = stage0 + s * STAGE, b_dst = a_dst + A_BYTES, bar = full_even0 + 8 * s;
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE);       // the bytes of both blocks
#pragma unroll
                    for (int u = 0; u < KSUB; ++u) {
                        tma_load_2d_pair(a_dst + u * A_SUB, &amap, (kc * KSUB + u) * BK, m0, bar);
                        tma_load_2d_pair(b_dst + u * B_SUB, &bmap, (kc * KSUB + u) * BK, b_row, bar);
                    }
                    if (++s == NS) { s = 0; ++round; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (even block): accumulator t & 1
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(2 * BM, BN, false);
            // descriptors of a stage's first k-step: only the start-address field (units of 16 bytes) moves from there
            const uint64_t desc_a0 = umma_desc_sw128(stage0, 16, 1024), desc_b0 = umma_desc_sw128(stage0 + A_BYTES, 16, 1024);
            const uint32_t a_sub16 = A_SUB >> 4, b_sub16 = (uint32_t)B_SUB >> 4;
            int s = 0, round = 0, t = 0;
            bool ok = true;
            for (int tile = pair; tile < tiles && ok; tile += pairs, ++t) {
                const int b = t & 1;
                if (t >= 2 && !mbar_wait(acc_empty0 + 8 * b, ((t >> 1) - 1) & 1)) { atomicExch(error_word, 54); abort_flag = 1; break; }
                tc_fence_after();
                const uint32_t acc = tmem + b * ACC_COLS;
                for (int kc = 0; kc < nk; ++kc) {
                    if (!mbar_spin(full0 + 8 * s, round & 1)) { atomicExch(error_word, 52); abort_flag = 1; ok = false; break; }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((uint32_t)(s * STAGE) >> 4);
#pragma unroll
                    for (int k = 0; k < KSUB * BK / 16; ++k)
                        umma_ss_pair(acc, desc_a0 + off + (k >> 2) * a_sub16 + 2 * (k & 3), desc_b0 + off + (k >> 2) * b_sub16 + 2 * (k & 3),
                                     idesc, (kc | k) != 0);
                    umma_commit_pair(empty0 + 8 * s, 3);       // the stage is free in both blocks once these MMAs have read it
                    if (++s == NS) { s = 0; ++round; }
                }
                if (!ok) break;
                umma_commit_pair(acc_full0 + 8 * b, 3);        // the accumulator is complete in both blocks
            }
        }
    } else {
        // ---------------- epilogue (both blocks): warp w reads tensor-memory lanes 32 (w % 4) .. +31, one row per thread
        const int lg = warp & 3;
        const uint32_t acc_empty_even0 = map_to_rank(acc_empty0, 0);
        int t = 0, groups = 0;
        unsigned char* my_out = stage_out + (warp - 2) * 8192;
        const int per_tile = GATED ? HALF : BN;                        // result columns of a tile
        const int n_out = GATED ? sh.N / 2 : sh.N;
        for (int tile = pair; tile < tiles && !abort_flag; tile += pairs, ++t) {
            const int b = t & 1;
            const int m0 = (tile % sh.m_tiles) * 2 * BM + (int)rank * BM, nt = tile / sh.m_tiles;
            if (!mbar_wait(acc_full0 + 8 * b, (t >> 1) & 1)) { atomicExch(error_word, 53); abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t acc = tmem + ((uint32_t)(lg * 32) << 16) + b * ACC_COLS;
            for (int c = 0; c < per_tile / 64; ++c) {
                float v[64];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int col_in = c * 64 + h * 32;
                    uint32_t ra[32];
                    tmem_ld32(acc + col_in, ra);
                    if (GATED) {
                        uint32_t ru[32];
                        tmem_ld32(acc + HALF + col_in, ru);
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_even0 + 8 * b);   // this warp has read its lanes of the accumulator
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // the stores have landed
    }
    tc_fence_before();
    cluster_barrier();            // neither block leaves while the other may still read its shared memory or signal its barriers
    if (warp == 1) tmem_dealloc_pair(tmem, 2 * ACC_COLS);
}

std::mutex t2_mutex;
std::map<std::tuple<const void*, int, int, int>, CUtensorMap> t2_weight_maps;

template <bool GATED>
int launch_tc2(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, int* error_word, cudaStream_t stream) {
    const int n_cols = GATED ? N / 2 : N;
    if (ldo % 8 || ((uintptr_t)out % 16)) return -2;
    T2Shape sh;
    sh.M = M; sh.N = N; sh.K = K;
    sh.m_tiles = (M + 2 * BM - 1) / (2 * BM);
    static int pairs_max = 0;
    auto kern = gemm_tc2_kernel<GATED>;
    const size_t smem_max = 226 * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (!pairs_max) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(2); q.blockDim = dim3(T2_THREADS); q.dynamicSmemBytes = smem_max;
        cudaLaunchAttribute a[1];
        a[0].id = cudaLaunchAttributeClusterDimension;
        a[0].val.clusterDim.x = 2; a[0].val.clusterDim.y = 1; a[0].val.clusterDim.z = 1;
        q.attrs = a; q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess || n < 1) { (void)cudaGetLastError(); return -2; }
        pairs_max = n;
    }
    // tile width: an MMA of 128 or fewer columns takes about as long as one of 256, so the widest tile the result has room for
    int best_bn = 256;
    while (best_bn > 128 && (GATED ? best_bn / 2 : best_bn) > n_cols) best_bn -= 128;
    sh.BN = best_bn;
    const int per_tile = GATED ? sh.BN / 2 : sh.BN;
    sh.n_tiles = (n_cols + per_tile - 1) / per_tile;
    const int stage = A_BYTES + KSUB * (sh.BN / 2) * BK * 2;
    sh.NS = (int)((smem_max - 2048 - OUT_BYTES) / stage);
    if (sh.NS > 8) sh.NS = 8;
    if (sh.NS < 2) return -2;
    CUtensorMap amap, bmap, omap;
    if (!sm100_host::make_map_bf16(&amap, X, M, K, ldx, BM, BK)) return -5;
    {
        std::lock_guard<std::mutex> lock(t2_mutex);
        auto key = std::make_tuple(W, N, K, sh.BN / 2);
        auto it = t2_weight_maps.find(key);
        if (it == t2_weight_maps.end()) {
            CUtensorMap m;
            if (!sm100_host::make_map_bf16(&m, W, N, K, K, sh.BN / 2, BK)) return -5;
            it = t2_weight_maps.emplace(key, m).first;
        }
        bmap = it->second;
    }
    if (!sm100_host::make_map_bf16(&omap, out, M, n_cols, ldo, 32, 64)) return -5;
    const size_t smem = (size_t)sh.NS * stage + OUT_BYTES + (2 * sh.NS + 4) * 8 + 16 + 1024;
    const int tiles = sh.m_tiles * sh.n_tiles;
    const int pairs = tiles < pairs_max ? tiles : pairs_max;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(T2_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kern, amap, bmap, omap, sh, error_word);
}

}  // namespace

// bfloat16 result.  Returns -2 for shapes it does not take (K not a multiple of 64, unaligned rows): the caller uses another GEMM.
MI_EXPORT int mi_gemm_tc2(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, int* error_word,
                          cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return -2;
    return launch_tc2<false>(X, ldx, W, out, ldo, M, N, K, error_word, stream);
}

// act[M, I] = silu(g) * u with [g | u] = X[M, K] * W[2 I, K]^T (both rounded to bfloat16 first, as the separate kernels do).
MI_EXPORT int mi_gemm_tc2_swiglu(const void* X, int ldx, const void* W, void* act, int M, int inter, int K, int* error_word,
                                 cudaStream_t stream) {
    if (M == 0 || inter == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || inter % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16) || ((uintptr_t)act % 16)) return -2;
    return launch_tc2<true>(X, ldx, W, act, inter, M, 2 * inter, K, error_word, stream);
}
