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
// A ring stage holds 128 of K (two boxes per operand): one hand-over between loader and MMA thread per eight MMAs.
// Tiles left over after the whole waves (fewer tiles than pairs, or tiles mod pairs) are cut along K between the pairs
// when K is long enough to pay for it: every share writes its float32 accumulator to a workspace, and once a counter
// says that all shares of a tile are there, the shares' epilogue warps each add up and store a few [32 x 32] units of
// it, shares in order (the same bits on every run).  The shares are a pair's FIRST work, so all of that happens under
// the products of its first whole tile.
//
// Measured (Qwen3-4B shapes, graph-timed, microseconds own / library): 2,048 rows qkv 45.6 / 45.5, gate/up 138 / 138
// (1.48 PFLOP/s), o 32 / 31, down 71 / 72; 4,096 rows gate/up 257 / 292-326, qkv 89 / 88, o 60 / 60, down 139 / 140;
// 256-1,024 rows the library is 5-50 % faster.  With the activation in the epilogue the gate/up kernel replaces the library product and a 27 us
// activation kernel.  What made the difference (gate/up, 2,048 rows): 256-column tiles only (an MMA of 128 columns takes
// ~150 clocks where 64 are nominal; 185 us with them), no index arithmetic between the MMAs of a stage (164), stages of
// 128 of K (137).  The engine times both kernels per shape and row bucket at start-up and keeps the faster.
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
    int pairs;                          // pairs of blocks launched
    int full_waves, rem, split;         // tiles = full_waves * pairs + rem; each of the last rem tiles is cut along K between `split` pairs
};

// what pair `pair` does in its w-th turn: a whole tile (part < 0), or the k-steps [kc0, kc1) of one of the left-over tiles.
// Left-over tiles that are cut come FIRST: their shares are in the workspace, counted and added up while the first whole
// tile's products run (the epilogue warps have nothing else to do then), so the cut costs the share's products and little
// more.  A left-over tile that is not cut is a last, partly filled wave.
struct T2Work { int tile, kc0, kc1, part; };
__device__ __forceinline__ bool t2_work(const T2Shape& sh, int pair, int w, int nk, T2Work& o) {
    o.kc0 = 0; o.kc1 = nk; o.part = -1;
    if (sh.split > 1 && pair < sh.rem * sh.split) {
        if (w == 0) {
            o.tile = sh.full_waves * sh.pairs + pair / sh.split;
            o.part = pair % sh.split;
            o.kc0 = o.part * nk / sh.split;
            o.kc1 = (o.part + 1) * nk / sh.split;
            return true;
        }
        --w;
    }
    if (w < sh.full_waves) { o.tile = w * sh.pairs + pair; return true; }
    if (sh.split > 1 || w > sh.full_waves || pair >= sh.rem) return false;
    o.tile = sh.full_waves * sh.pairs + pair;
    return true;
}

template <bool GATED>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap amap, const __grid_constant__ CUtensorMap bmap,
                const __grid_constant__ CUtensorMap omap, const T2Shape sh, __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ ws,
                int* __restrict__ counters, int* __restrict__ error_word) {
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
    const int pair = blockIdx.x >> 1;
    const int nk = (sh.K + KSUB * BK - 1) / (KSUB * BK);   // a box beyond K reads zeros
    T2Work wk;

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
            for (int w = 0; ok && t2_work(sh, pair, w, nk, wk); ++w) {
                const int m0 = (wk.tile % sh.m_tiles) * 2 * BM + (int)rank * BM, nt = wk.tile / sh.m_tiles;
                const int b_row = GATED ? (int)rank * (sh.N / 2) + nt * HALF : nt * BN + (int)rank * HALF;
                for (int kc = wk.kc0; kc < wk.kc1; ++kc) {
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
            int s = 0, round = 0;
            bool ok = true;
            for (int t = 0; ok && t2_work(sh, pair, t, nk, wk); ++t) {
                const int b = t & 1;
                if (t >= 2 && !mbar_wait(acc_empty0 + 8 * b, ((t >> 1) - 1) & 1)) { atomicExch(error_word, 54); abort_flag = 1; break; }
                tc_fence_after();
                const uint32_t acc = tmem + b * ACC_COLS;
                for (int kc = wk.kc0; kc < wk.kc1; ++kc) {
                    if (!mbar_spin(full0 + 8 * s, round & 1)) { atomicExch(error_word, 52); abort_flag = 1; ok = false; break; }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((uint32_t)(s * STAGE) >> 4);
#pragma unroll
                    for (int k = 0; k < KSUB * BK / 16; ++k)
                        umma_ss_pair(acc, desc_a0 + off + (k >> 2) * a_sub16 + 2 * (k & 3), desc_b0 + off + (k >> 2) * b_sub16 + 2 * (k & 3),
                                     idesc, ((kc - wk.kc0) | k) != 0);
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
        int groups = 0;
        unsigned char* my_out = stage_out + (warp - 2) * 8192;
        const int per_tile = GATED ? HALF : BN;                        // result columns of a tile
        const int n_out = GATED ? sh.N / 2 : sh.N;
        // 64 values per thread (row row0 + lane, columns col .. col + 63) -> a swizzled [32 x 64] bfloat16 box -> TMA store
        auto put_box = [&](const float (&v)[64], int col, int row0) {
            unsigned char* box = my_out + (groups & 1) * 4096;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");   // the store two boxes back has read its box
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint4 p;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&p);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 hh = __floats2bfloat162_rn(v[8 * j + 2 * e], v[8 * j + 2 * e + 1]);
                    pw[e] = *reinterpret_cast<uint32_t*>(&hh);
                }
                *reinterpret_cast<uint4*>(box + lane * 128 + ((j ^ (lane & 7)) << 4)) = p;
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if (col < n_out && row0 < sh.M) {
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];\n"
                                 :: "l"((uint64_t)&omap), "r"(col), "r"(row0), "r"(smem_u32(box)) : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
            }
            ++groups;
        };
        auto activate = [](float gate, float up) {
            const float gt = round_to<__nv_bfloat16>(gate), u = round_to<__nv_bfloat16>(up);
            return gt / (1.f + expf(-gt)) * u;
        };
        for (int t = 0; !abort_flag && t2_work(sh, pair, t, nk, wk); ++t) {
            const int b = t & 1;
            const int m0 = (wk.tile % sh.m_tiles) * 2 * BM + (int)rank * BM, nt = wk.tile / sh.m_tiles;
            if (!mbar_wait(acc_full0 + 8 * b, (t >> 1) & 1)) { atomicExch(error_word, 53); abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t acc = tmem + ((uint32_t)(lg * 32) << 16) + b * ACC_COLS;
            if (wk.part < 0) {
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
                            for (int i = 0; i < 32; ++i) v[h * 32 + i] = activate(__uint_as_float(ra[i]), __uint_as_float(ru[i]));
                        } else {
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[h * 32 + i] = __uint_as_float(ra[i]);
                        }
                    }
                    put_box(v, nt * per_tile + c * 64, m0 + lg * 32);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_empty_even0 + 8 * b);   // this warp has read its lanes of the accumulator
                continue;
            }
            // ---- one of `split` shares of a tile: the share goes to the workspace as float32, [32-column group][column][row]
            // so that a warp's stores and loads are whole lines; when all shares of this block's rows are there (a counter
            // per tile and block rank), each share's block adds up and stores some of the tile's boxes, shares in order
            const int tr = wk.tile - sh.full_waves * sh.pairs, groups32 = BN / 32;
            const size_t share_floats = (size_t)BM * BN;
            float* mine = ws + ((size_t)(tr * sh.split + wk.part) * 2 + rank) * share_floats;
            for (int a = 0; a < groups32; ++a) {
                uint32_t ra[32];
                tmem_ld32(acc + a * 32, ra);
                tmem_wait_ld();
                float* dst = mine + (size_t)(lg * groups32 + a) * 1024 + lane;
#pragma unroll
                for (int i = 0; i < 32; ++i) __stcg(dst + i * 32, __uint_as_float(ra[i]));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_even0 + 8 * b);   // the accumulator is free for the tile after next
            __threadfence();
            __syncwarp();
            int* ctr = counters + tr * 2 + rank;
            const int need = 4 * sh.split;                 // four epilogue warps in each share's block
            if (lane == 0) {
                atomicAdd(ctr, 1);
                bool seen = false;
                for (uint32_t i = 0; i < (1u << 21) && !seen; ++i) {
                    int have;
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(have) : "l"(ctr) : "memory");
                    seen = have >= need;
                    if (!seen) __nanosleep(40);
                }
                if (!seen) { atomicExch(error_word, 55); abort_flag = 1; }
            }
            __syncwarp();
            __threadfence();
            if (!abort_flag) {
                // units of [32 rows x 32 result columns], dealt round to the 4 * split epilogue warps of the shares' blocks;
                // four shares' loads are in flight at a time (one warp's chain of round trips to L2 is what this costs)
                const int gpt = per_tile / 32, units = 4 * gpt, workers = 4 * sh.split;
                auto add_up = [&](float (&sum)[32], const float* src) {      // src: share 0's group; the shares lie share_floats * 2 apart
#pragma unroll
                    for (int i = 0; i < 32; ++i) sum[i] = 0.f;
                    for (int j = 0; j < sh.split; j += 4) {
                        float part[4][32];
#pragma unroll
                        for (int d = 0; d < 4; ++d) {
                            const bool there = j + d < sh.split;
#pragma unroll
                            for (int i = 0; i < 32; ++i) part[d][i] = there ? __ldcg(src + (size_t)(j + d) * 2 * share_floats + i * 32) : 0.f;
                        }
#pragma unroll
                        for (int d = 0; d < 4; ++d)
#pragma unroll
                            for (int i = 0; i < 32; ++i) sum[i] += part[d][i];
                    }
                };
                const float* tile_ws = ws + ((size_t)(tr * sh.split) * 2 + rank) * share_floats + lane;
                for (int unit = wk.part * 4 + (warp - 2); unit < units; unit += workers) {
                    const int lq = unit / gpt, a = unit % gpt;
                    float g[32];
                    add_up(g, tile_ws + (size_t)(lq * groups32 + a) * 1024);
                    if (GATED) {
                        float u[32];
                        add_up(u, tile_ws + (size_t)(lq * groups32 + HALF / 32 + a) * 1024);
#pragma unroll
                        for (int i = 0; i < 32; ++i) g[i] = activate(g[i], u[i]);
                    }
                    const int row = m0 + lq * 32 + lane, col = nt * per_tile + a * 32;
                    if (row < sh.M && col < n_out) {
                        __nv_bfloat16* dst = out + (size_t)row * ldo + col;
                        if (col + 32 <= n_out) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint4 p;
                                uint32_t* pw = reinterpret_cast<uint32_t*>(&p);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    __nv_bfloat162 hh = __floats2bfloat162_rn(g[8 * j + 2 * e], g[8 * j + 2 * e + 1]);
                                    pw[e] = *reinterpret_cast<uint32_t*>(&hh);
                                }
                                *reinterpret_cast<uint4*>(dst + 8 * j) = p;
                            }
                        } else {
                            for (int i = 0; i < n_out - col; ++i) dst[i] = __float2bfloat16_rn(g[i]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && !abort_flag && atomicAdd(ctr, 1) == 2 * need - 1) atomicExch(ctr, 0);   // the last reader leaves the counter as it found it
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
int launch_tc2(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, float* ws, long long ws_bytes,
               int* counters, int num_counters, int* error_word, cudaStream_t stream) {
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
    // whole waves of tiles, one per pair; the tiles left over (or all of them, if there are fewer than pairs) are cut
    // along K between as many pairs as there are for each, so the last wave is as long as its share of K
    const int tiles = sh.m_tiles * sh.n_tiles, nk = (K + KSUB * BK - 1) / (KSUB * BK);
    sh.full_waves = tiles / pairs_max;
    sh.rem = tiles % pairs_max;
    sh.split = 1;
    if (sh.rem > 0 && ws && counters && 2 * sh.rem <= num_counters && ((uintptr_t)ws % 16) == 0) {
        int split = pairs_max / sh.rem;
        if (split > nk / 2) split = nk / 2;
        if (split > 16) split = 16;
        const long long share = 2ll * BM * sh.BN * 4;
        while (split > 1 && (long long)sh.rem * split * share > ws_bytes) --split;
        // a cut saves (1 - 1/split) of a tile's time (~0.7 us per 128 of K).  With whole tiles behind it, it costs the share's
        // own products and the ring's fill (worth it from 4 saved k-steps on: gate/up at 4,096 rows 259 -> 253 us); with none,
        // the ~10 us pass through the workspace is in the open (from 16 on)
        const long long min_saved = sh.full_waves > 0 ? 4 : 16;
        if (split >= 2 && (long long)nk * (split - 1) >= min_saved * split) sh.split = split;
    }
    const int pairs = sh.full_waves > 0 ? pairs_max : sh.rem * sh.split;
    sh.pairs = pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(T2_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kern, amap, bmap, omap, sh, (__nv_bfloat16*)out, ldo, ws, counters, error_word);
}

}  // namespace

// bfloat16 result.  Returns -2 for shapes it does not take (K not a multiple of 64, unaligned rows): the caller uses another GEMM.
// ws (ws_bytes, 16-byte aligned) and counters (num_counters ints, zero) may be null: scratch for cutting the last tiles along K.
// Launches that share them must be ordered on one stream.
MI_EXPORT int mi_gemm_tc2(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N, int K, float* ws,
                          long long ws_bytes, int* counters, int num_counters, int* error_word, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16)) return -2;
    return launch_tc2<false>(X, ldx, W, out, ldo, M, N, K, ws, ws_bytes, counters, num_counters, error_word, stream);
}

// act[M, I] = silu(g) * u with [g | u] = X[M, K] * W[2 I, K]^T (both rounded to bfloat16 first, as the separate kernels do).
MI_EXPORT int mi_gemm_tc2_swiglu(const void* X, int ldx, const void* W, void* act, int M, int inter, int K, float* ws,
                                 long long ws_bytes, int* counters, int num_counters, int* error_word, cudaStream_t stream) {
    if (M == 0 || inter == 0) return 0;
    if (K % BK || K < BK || ldx % 8 || inter % 8 || ((uintptr_t)X % 16) || ((uintptr_t)W % 16) || ((uintptr_t)act % 16)) return -2;
    return launch_tc2<true>(X, ldx, W, act, inter, M, 2 * inter, K, ws, ws_bytes, counters, num_counters, error_word, stream);
}
