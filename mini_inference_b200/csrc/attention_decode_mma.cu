// Split-KV paged decode attention on the tensor cores, bfloat16, head size 64 or 128.
//
// Reference (davidjoyme/mini-inference kernels/paged_attention/decode_triton.py:6-100): one
// program per (request, QUERY head, split) that multiplies k * q element by element on the
// CUDA cores; the 4 query heads that share a kv head each read the same keys again.  Here one
// block serves (request, KV head, split): the G query heads of the group are the rows of a
// 16-row mma tile, so each key and value is read from HBM once per group.
//
// Data path: no shared-memory staging.  Each thread loads 16-byte pieces of K and V straight
// from the pages into the registers that mma.sync.m16n8k16 wants.  That works because the
// reduction index of a dot product may be permuted freely: for the scores the head dimension
// is permuted so that the 8 values a thread feeds to two k-steps are 8 CONSECUTIVE values of
// one key (one 16-byte load; a warp instruction covers 8 keys x 64 B); the query fragments use
// the same permutation.  For P*V the output columns are permuted the same way (column g of
// tile t is d = 8g + t), so a thread's 16-byte load of one value row serves 8 output tiles; a
// byte permute pairs the rows of two keys into one B register.
//
// Each of the 4 warps takes every 4th 16-key block of the split's range with its own running
// (max, sum, output); the warps are merged through shared memory at the end, the splits by
// mi_attn_decode_merge (attention_generic.cu) when there is more than one.
// Needs page_size % 16 == 0 (a 16-key block never straddles a page) and G <= 16.
#include "sm100.cuh"
#include <math.h>
#include <map>
#include <mutex>
#include <tuple>

using namespace mi;

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint4& a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int DEC_WARPS = 4;

// thread-block cluster: the splits of one (request, kv head) can be one cluster and merge through shared memory
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ld_cluster(const float* local, uint32_t rank) {     // the same variable in block `rank`'s shared memory
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

constexpr int DEC_STAGES = 3;      // BULK: 16-key K and V tiles in flight per warp
constexpr int DEC_BAR_BYTES = 256; // room for the rings' mbarriers (warps x DEC_STAGES x 8 bytes)
constexpr int DEC_WARPS_ALONE = 8; // warps of a block that has its SM to itself (the grid is at most one block per SM):
                                   // a warp works through its tiles one after the other, so with few blocks the time
                                   // goes with the number of warps, not with the bytes

// BULK = false: K/V go from the pages straight into registers (one block ahead).
// BULK = true:  each warp keeps a ring of DEC_STAGES (K tile, V tile) pairs in shared memory, filled by TMA tile
//               loads ([16 keys x 64] boxes of the cache seen as a [rows, D] matrix, 128-byte swizzle), signalled
//               by per-warp mbarriers; fragments are then read from shared memory without bank conflicts (the
//               swizzle spreads the 8 keys of a quarter-warp over the banks; the score product takes its 16-byte
//               pieces in the order 2c + (j & 1) so that neighbouring lanes also differ in the column).  More bytes
//               in flight per SM at no register cost.
template <int D, bool BULK, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS > DEC_WARPS ? 1 : BULK ? 2 : 3)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                       const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                       const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                       float* __restrict__ o_part, float* __restrict__ lse_part, const int* __restrict__ decode_segs,
                       const int* __restrict__ seg_q_start, const int* __restrict__ seg_kv_len,
                       const int* __restrict__ block_table, const int* __restrict__ table_rows, int table_stride,
                       int H, int KV, int ps, float scale_log2, int window, int* __restrict__ merge_counters,
                       int* __restrict__ error_word, int cluster_merge) {
    static_assert(WARPS * DEC_STAGES * 8 <= DEC_BAR_BYTES, "the mbarriers must fit in their reserved bytes");
    constexpr int KS = D / 16;          // k-steps of the score product
    constexpr int NT = D / 8;           // output tiles of 8 columns
    constexpr int HALVES = D / 64;      // 64-column halves of a value row
    extern __shared__ float smem_raw[];  // [WARPS][16][D] outputs, then [WARPS][16] max and sum
    float* smem = smem_raw;
    pdl_trigger();
    if (!BULK) pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int G = H / KV;
    const int seg = decode_segs[blockIdx.x], kvh = blockIdx.y;
    const int S = gridDim.z, s = blockIdx.z;
    const int tok = seg_q_start[seg], len = seg_kv_len[seg];
    const int lo = window > 0 ? max(0, len - window) : 0;
    const int blk_lo = lo / 16, blk_hi = (len + 15) / 16;
    const int per = (blk_hi - blk_lo + S - 1) / S;
    const int b0 = blk_lo + s * per, b1 = min(b0 + per, blk_hi);
    // an entry's pages: row `seg` of the table, or row table_rows[seg] of a table that holds a row per live request
    const int* table_row = block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride;

    // query fragments, permuted: the 16 bytes at d = 32 j + 8 c of rows g and g + 8.  They are the
    // same for all warps and live in shared memory ([k-step][lane] x 16 bytes) to keep registers
    // for the loads in flight.
    constexpr int TILE = 16 * D * 2;                                     // bytes of one K or V tile
    constexpr int MERGE_BYTES = WARPS * 16 * (D + 2) * 4;
    constexpr int RING_BYTES = BULK ? WARPS * DEC_STAGES * 2 * TILE : 0;
    constexpr int FRONT = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;   // the merge scratch re-uses the ring
    constexpr int CLUSTER_OFF = (MERGE_BYTES + 1023) / 1024 * 256;               // (floats) this split's result, after the scratch
    unsigned char* smem_bytes = reinterpret_cast<unsigned char*>(smem);
    if (BULK) {                                            // swizzle atoms are 1 KB
        smem_bytes = (unsigned char*)(((uintptr_t)smem_bytes + 1023) & ~(uintptr_t)1023);
        smem = reinterpret_cast<float*>(smem_bytes);
    }
    uint4* q_frag = reinterpret_cast<uint4*>(smem_bytes + FRONT);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_bytes + FRONT + (D / 16) * 32 * 16);
    unsigned char* ring = smem_bytes + warp * (DEC_STAGES * 2 * TILE);
    const uint32_t bar0 = sm100::smem_u32(bars + warp * DEC_STAGES);
    if (BULK && lane == 0) {
        for (int st = 0; st < DEC_STAGES; ++st) sm100::mbar_init(bar0 + 8 * st, 1);
        sm100::mbar_init_fence();
    }
    // BULK: lane 0 asks for the K and V tiles of block `blk` into ring stage st
    auto issue = [&](int blk, int st) {
        if (lane == 0) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // the stage was just read with ordinary loads
            const uint32_t dst = sm100::smem_u32(ring + st * 2 * TILE), bar = bar0 + 8 * st;
            const int page = table_row[(blk * 16) / ps];
            const int row = (page * KV + kvh) * ps + (blk * 16) % ps;            // of the cache seen as [rows, D]
            sm100::mbar_expect_tx(bar, 2 * TILE);
#pragma unroll
            for (int hb = 0; hb < HALVES; ++hb) {
                sm100::tma_load_2d(dst + hb * 2048, &kmap, hb * 64, row, bar);
                sm100::tma_load_2d(dst + TILE + hb * 2048, &vmap, hb * 64, row, bar);
            }
        }
    };

    // BULK: the first stages are requested BEFORE waiting for the kernel ahead: it writes only the newest token's key
    // and value (the last 16-key block of a request), and the block table and lengths were copied in before the step began.
    int primed = 0;
    if (BULK) {
        __syncwarp();
        for (; primed < DEC_STAGES && b0 + warp + primed * WARPS < min(b1, blk_hi - 1); ++primed)
            issue(b0 + warp + primed * WARPS, primed);
        pdl_wait();
    }
    if (warp == 0) {
        const __nv_bfloat16* qrow = q + (size_t)tok * q_stride + (size_t)kvh * G * D;
#pragma unroll
        for (int j = 0; j < KS / 2; ++j) {
            uint4 r0 = make_uint4(0, 0, 0, 0), r1 = make_uint4(0, 0, 0, 0);
            const int d = BULK ? 64 * (j >> 1) + 16 * c + 8 * (j & 1) : 32 * j + 8 * c;   // the keys' pieces use the same order
            if (g < G) r0 = *reinterpret_cast<const uint4*>(qrow + (size_t)g * D + d);
            if (g + 8 < G) r1 = *reinterpret_cast<const uint4*>(qrow + (size_t)(g + 8) * D + d);
            q_frag[(2 * j) * 32 + lane] = make_uint4(r0.x, r1.x, r0.y, r1.y);
            q_frag[(2 * j + 1) * 32 + lane] = make_uint4(r0.z, r1.z, r0.w, r1.w);
        }
    }
    __syncthreads();

    float o[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8; sums are per thread

    uint4 kreg[2][KS / 2];
    uint4 vreg[4][HALVES];
    // fragments of one 16-key block: keys nt*8+g at d = 32 j + 8 c; values of keys 2c, 2c+1, 2c+8, 2c+9 at d = 64 hb + 8 g
    auto frag_k = [&](const __nv_bfloat16* base) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int j = 0; j < KS / 2; ++j)
                kreg[nt][j] = *reinterpret_cast<const uint4*>(base + (size_t)(nt * 8 + g) * D + 32 * j + 8 * c);
    };
    auto frag_v = [&](const __nv_bfloat16* base) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = 2 * c + (i & 1) + 8 * (i >> 1);
#pragma unroll
            for (int hb = 0; hb < HALVES; ++hb)
                vreg[i][hb] = *reinterpret_cast<const uint4*>(base + (size_t)key * D + 64 * hb + 8 * g);
        }
    };
    // BULK: the same fragments from a swizzled tile in shared memory ([64-column half][16 keys][128 bytes])
    auto frag_k_sw = [&](const unsigned char* tile) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int j = 0; j < KS / 2; ++j) {
                const int key = nt * 8 + g, piece = 2 * c + (j & 1);
                kreg[nt][j] = *reinterpret_cast<const uint4*>(tile + (j >> 1) * 2048 + key * 128 + ((piece ^ (key & 7)) << 4));
            }
    };
    auto frag_v_sw = [&](const unsigned char* tile) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = 2 * c + (i & 1) + 8 * (i >> 1);
#pragma unroll
            for (int hb = 0; hb < HALVES; ++hb)
                vreg[i][hb] = *reinterpret_cast<const uint4*>(tile + hb * 2048 + key * 128 + ((g ^ (key & 7)) << 4));
        }
    };
    auto tile_of = [&](const __nv_bfloat16* cache, int blk) {
        const int page = table_row[(blk * 16) / ps];
        return cache + ((size_t)(page * KV + kvh) * ps + (blk * 16) % ps) * D;
    };
    auto load_k = [&](int blk) { frag_k(tile_of(k_cache, blk)); };
    auto load_v = [&](int blk) { frag_v(tile_of(v_cache, blk)); };
    // Software pipeline.  Registers: the keys of block i+1 are requested right after the scores of block i,
    // the values of block i+1 right after block i's P*V.  BULK: DEC_STAGES blocks are in flight in the ring;
    // a block's fragments are copied to registers as soon as it lands and its stage is refilled at once.
    int blk = b0 + warp;
    int nth = 0;
    if (BULK) {
        for (int st = primed; st < DEC_STAGES && blk + st * WARPS < b1; ++st) issue(blk + st * WARPS, st);
    } else if (blk < b1) { load_k(blk); load_v(blk); }
    for (; blk < b1; blk += WARPS, ++nth) {
        if (BULK) {
            const int st = nth % DEC_STAGES;
            if (!sm100::mbar_wait(bar0 + 8 * st, (nth / DEC_STAGES) & 1)) { if (lane == 0) atomicExch(error_word, 31); break; }
            unsigned char* tile = ring + st * 2 * TILE;
            frag_k_sw(tile);
            frag_v_sw(tile + TILE);
            __syncwarp();
            if (blk + DEC_STAGES * WARPS < b1) issue(blk + DEC_STAGES * WARPS, st);
        }
        // scores: 16 (heads) x 16 (keys) as two 8-key tiles
        float sc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
            for (int j = 0; j < KS / 2; ++j) {
                const uint4 qa0 = q_frag[(2 * j) * 32 + lane], qa1 = q_frag[(2 * j + 1) * 32 + lane];
                mma_bf16_16816(sc[nt], qa0, kreg[nt][j].x, kreg[nt][j].y);
                mma_bf16_16816(sc[nt], qa1, kreg[nt][j].z, kreg[nt][j].w);
            }
        }
        if (!BULK && blk + WARPS < b1) load_k(blk + WARPS);   // next block's keys fly during the rest
        // mask, online softmax (base 2)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = blk * 16 + nt * 8 + 2 * c + e;
                const bool ok = key >= lo && key < len;
                sc[nt][e] = ok ? sc[nt][e] * scale_log2 : -INFINITY;
                sc[nt][2 + e] = ok ? sc[nt][2 + e] * scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, sc[nt][e]);
                mx1 = fmaxf(mx1, sc[nt][2 + e]);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);      // finite: every block holds a visible key
        const float al0 = exp2f(m0 - n0), al1 = exp2f(m1 - n1);
        m0 = n0; m1 = n1;
        l0 *= al0; l1 *= al1;
        uint32_t pa[4];
        {
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                p[nt][0] = exp2f(sc[nt][0] - n0); p[nt][1] = exp2f(sc[nt][1] - n0);
                p[nt][2] = exp2f(sc[nt][2] - n1); p[nt][3] = exp2f(sc[nt][3] - n1);
                l0 += p[nt][0] + p[nt][1];
                l1 += p[nt][2] + p[nt][3];
            }
            pa[0] = pack_bf16(p[0][0], p[0][1]); pa[1] = pack_bf16(p[0][2], p[0][3]);
            pa[2] = pack_bf16(p[1][0], p[1][1]); pa[3] = pack_bf16(p[1][2], p[1][3]);
        }
        // O += P V; tile t of half hb: column g is d = 64 hb + 8 g + t
#pragma unroll
        for (int hb = 0; hb < HALVES; ++hb) {
            const uint32_t* r0 = reinterpret_cast<const uint32_t*>(&vreg[0][hb]);   // key 2c
            const uint32_t* r1 = reinterpret_cast<const uint32_t*>(&vreg[1][hb]);   // key 2c + 1
            const uint32_t* r2 = reinterpret_cast<const uint32_t*>(&vreg[2][hb]);   // key 2c + 8
            const uint32_t* r3 = reinterpret_cast<const uint32_t*>(&vreg[3][hb]);   // key 2c + 9
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;
                const uint32_t vb0 = __byte_perm(r0[t >> 1], r1[t >> 1], sel);
                const uint32_t vb1 = __byte_perm(r2[t >> 1], r3[t >> 1], sel);
                float (&acc)[4] = o[hb * 8 + t];
                acc[0] *= al0; acc[1] *= al0; acc[2] *= al1; acc[3] *= al1;
                mma_bf16_16816(acc, pa, vb0, vb1);
            }
        }
        if (!BULK && blk + WARPS < b1) load_v(blk + WARPS);
    }
    if (BULK) __syncthreads();                    // every warp is done with its ring before the merge scratch overwrites it

    // row sums over the quad, then merge the warps
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* so = smem + (size_t)warp * 16 * D;
    float* sm = smem + (size_t)WARPS * 16 * D;
    float* sl = sm + WARPS * 16;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int d0 = 64 * (t >> 3) + 8 * (2 * c) + (t & 7), d1 = d0 + 8;
        so[g * D + d0] = o[t][0]; so[g * D + d1] = o[t][1];
        so[(g + 8) * D + d0] = o[t][2]; so[(g + 8) * D + d1] = o[t][3];
    }
    if (c == 0) {
        sm[warp * 16 + g] = m0; sl[warp * 16 + g] = l0;
        sm[warp * 16 + g + 8] = m1; sl[warp * 16 + g + 8] = l1;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
        const int row = idx / D, d = idx % D;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, sm[w * 16 + row]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = sm[w * 16 + row] == -INFINITY ? 0.f : exp2f(sm[w * 16 + row] - mx);
            num += f * smem[((size_t)w * 16 + row) * D + d];
            den += f * sl[w * 16 + row];
        }
        const float val = den > 0.f ? num / den : 0.f;
        const int h = kvh * G + row;
        if (S == 1) {
            out[((size_t)tok * H + h) * D + d] = __float2bfloat16_rn(val);
        } else if (BULK && cluster_merge) {
            float* cpart = smem + CLUSTER_OFF;             // [16][D] this split's rows, then [16] their log-sum-exp
            cpart[idx] = val;
            if (d == 0) cpart[16 * D + row] = den > 0.f ? (mx + log2f(den)) * 0.6931471805599453f : -INFINITY;
        } else {
            const size_t pi = ((size_t)blockIdx.x * H + h) * S + s;
            o_part[pi * D + d] = val;
            if (d == 0) lse_part[pi] = den > 0.f ? (mx + log2f(den)) * 0.6931471805599453f : -INFINITY;
        }
    }
    if (BULK && cluster_merge && S > 1) {
        // The S splits of this (request, kv head) are one cluster: split 0 reads the others' rows through distributed
        // shared memory and writes the result (no partial sums in global memory, no atomic, no fence);
        // out = sum_s e^(lse_s - max) o_s / sum_s e^(lse_s - max), splits added in index order.
        cluster_sync();
        if (cluster_rank() == 0) {
            const float* cpart = smem + CLUSTER_OFF;
            for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
                const int row = idx / D, d = idx % D, h = kvh * G + row;
                float l[8], v[8], mx = -INFINITY;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    l[r] = r < S ? ld_cluster(cpart + 16 * D + row, r) : -INFINITY;
                    v[r] = r < S ? ld_cluster(cpart + idx, r) : 0.f;
                    mx = fmaxf(mx, l[r]);
                }
                float num = 0.f, den = 0.f;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const float w = expf(l[r] - mx);
                    den += w;
                    num += w * v[r];
                }
                out[((size_t)tok * H + h) * D + d] = __float2bfloat16_rn(num / den);
            }
        }
        cluster_sync();                                    // the others' shared memory stays until split 0 has read it
        return;
    }
    if (S == 1 || merge_counters == nullptr) return;

    // The block that finishes last among the S splits of this (request, kv head) merges them:
    // out = sum_s e^(lse_s - max) o_s / sum_s e^(lse_s - max), splits added in index order.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(&merge_counters[blockIdx.x * KV + kvh], 1) == S - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * D; idx += WARPS * 32) {
        const int row = idx / D, d = idx % D, h = kvh * G + row;
        const size_t base = ((size_t)blockIdx.x * H + h) * S;
        float mx = -INFINITY, num = 0.f, den = 0.f;
        for (int k0 = 0; k0 < S; k0 += 8) {                 // 8 independent loads in flight
            float l[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) l[j] = k0 + j < S ? __ldcg(lse_part + base + k0 + j) : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, l[j]);
        }
        for (int k0 = 0; k0 < S; k0 += 8) {
            float l[8], v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool ok = k0 + j < S;
                l[j] = ok ? __ldcg(lse_part + base + k0 + j) : -INFINITY;
                v[j] = ok ? __ldcg(o_part + (base + k0 + j) * D + d) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float w = expf(l[j] - mx);
                den += w;
                num += w * v[j];
            }
        }
        out[((size_t)tok * H + h) * D + d] = __float2bfloat16_rn(num / den);
    }
    if (threadIdx.x == 0) merge_counters[blockIdx.x * KV + kvh] = 0;       // ready for the next call
}

MI_EXPORT int mi_attn_decode_mma_fused(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                       float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                       const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                       int table_stride, int H, int KV, int D, int ps, int splits, float scale,
                                       int window, int* merge_counters, cudaStream_t stream);
MI_EXPORT int mi_attn_decode_mma_bulk(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                      float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                      const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                      int table_stride, int H, int KV, int D, int ps, int splits, float scale,
                                      int window, int* merge_counters, int* error_word, int cache_pages, cudaStream_t stream);

MI_EXPORT int mi_attn_decode_mma_rows(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                      float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                      const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                      const int* table_rows, int table_stride, int H, int KV, int D, int ps, int splits,
                                      float scale, int window, int* merge_counters, int* error_word, int cache_pages,
                                      int cluster_merge, cudaStream_t stream);

MI_EXPORT int mi_attn_decode_mma(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                 float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                 const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                 int table_stride, int H, int KV, int D, int ps, int splits, float scale, int window,
                                 cudaStream_t stream) {
    return mi_attn_decode_mma_fused(q, q_stride, k_cache, v_cache, out, o_part, lse_part, decode_segs, num_decode,
                                    seg_q_start, seg_kv_len, block_table, table_stride, H, KV, D, ps, splits, scale,
                                    window, nullptr, stream);
}

// merge_counters: int32 [num_decode * KV], zero before the first call (the kernel leaves them zero).
// With it the splits are merged by the last block to finish and no separate merge launch is needed;
// null keeps the partial outputs for mi_attn_decode_merge.
MI_EXPORT int mi_attn_decode_mma_fused(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                       float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                       const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                       int table_stride, int H, int KV, int D, int ps, int splits, float scale,
                                       int window, int* merge_counters, cudaStream_t stream) {
    return mi_attn_decode_mma_bulk(q, q_stride, k_cache, v_cache, out, o_part, lse_part, decode_segs, num_decode,
                                   seg_q_start, seg_kv_len, block_table, table_stride, H, KV, D, ps, splits, scale,
                                   window, merge_counters, nullptr, 0, stream);
}

// error_word != null selects the variant that stages K/V through shared memory with TMA tile loads and per-warp
// mbarriers (bounded waits report through error_word; cache_pages = pages in k_cache / v_cache, for the tensor maps);
// null keeps the register-streaming variant.
namespace {
std::mutex dec_mutex;
std::map<std::tuple<const void*, long long, int>, CUtensorMap> dec_maps;
int cache_map(const void* cache, long long rows, int D, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(dec_mutex);
    auto key = std::make_tuple(cache, rows, D);
    auto it = dec_maps.find(key);
    if (it == dec_maps.end()) {
        CUtensorMap m;
        if (!sm100_host::make_map_bf16(&m, cache, (uint64_t)rows, (uint64_t)D, (uint64_t)D, 16, 64)) return -5;
        it = dec_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}
}  // namespace

MI_EXPORT int mi_attn_decode_mma_bulk(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                      float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                      const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                      int table_stride, int H, int KV, int D, int ps, int splits, float scale,
                                      int window, int* merge_counters, int* error_word, int cache_pages, cudaStream_t stream) {
    return mi_attn_decode_mma_rows(q, q_stride, k_cache, v_cache, out, o_part, lse_part, decode_segs, num_decode, seg_q_start,
                                   seg_kv_len, block_table, nullptr, table_stride, H, KV, D, ps, splits, scale, window,
                                   merge_counters, error_word, cache_pages, 0, stream);
}

// How many clusters of `splits` blocks of the staged kernel the GPU holds at once (0: unknown or none).
MI_EXPORT int mi_attn_decode_cluster_fit(int D, int splits) {
    if ((D != 64 && D != 128) || splits < 2 || splits > 8) return 0;
    const size_t smem = (size_t)DEC_WARPS * DEC_STAGES * 2 * 16 * D * 2 + (size_t)(D / 16) * 32 * 16 + DEC_WARPS * DEC_STAGES * 8 +
                        1024 + DEC_BAR_BYTES;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, splits); cfg.blockDim = dim3(DEC_WARPS * 32); cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e;
    if (D == 128) {
        cudaFuncSetAttribute(attn_decode_mma_kernel<128, true, DEC_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = cudaOccupancyMaxActiveClusters(&n, attn_decode_mma_kernel<128, true, DEC_WARPS>, &cfg);
    } else {
        cudaFuncSetAttribute(attn_decode_mma_kernel<64, true, DEC_WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        e = cudaOccupancyMaxActiveClusters(&n, attn_decode_mma_kernel<64, true, DEC_WARPS>, &cfg);
    }
    return e == cudaSuccess ? n : 0;
}

// The general entry point.  table_rows != null: block_table holds a row per live request ([rows, table_stride], kept on
// the device) and entry i reads row table_rows[i]; null: entry i reads row i.  cluster_merge != 0: with 2..8 splits the
// splits of a (request, kv head) are launched as one thread-block cluster and merged through distributed shared memory
// (o_part, lse_part, merge_counters unused).
MI_EXPORT int mi_attn_decode_mma_rows(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                      float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                      const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                      const int* table_rows, int table_stride, int H, int KV, int D, int ps, int splits,
                                      float scale, int window, int* merge_counters, int* error_word, int cache_pages,
                                      int cluster_merge, cudaStream_t stream) {
    if (num_decode == 0) return 0;
    if ((D != 64 && D != 128) || H % KV || H / KV > 16 || ps % 16 || q_stride % 8) return -2;
    dim3 grid(num_decode, KV, splits);
    const bool bulk = error_word != nullptr;
    CUtensorMap kmap = {}, vmap = {};
    if (bulk) {
        if (cache_pages < 1 || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16)) return -2;
        const long long rows = (long long)cache_pages * KV * ps;
        int rc = cache_map(k_cache, rows, D, &kmap);
        if (rc) return rc;
        if ((rc = cache_map(v_cache, rows, D, &vmap))) return rc;
    }
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 1;
    }
    const bool alone = bulk && (long long)num_decode * KV * splits <= sms;      // at most one block per SM
    const int warps = alone ? DEC_WARPS_ALONE : DEC_WARPS;
    const size_t merge_bytes = (size_t)warps * 16 * (D + 2) * sizeof(float);
    const size_t ring_bytes = bulk ? (size_t)warps * DEC_STAGES * 2 * 16 * D * 2 : 0;
    const size_t smem = (ring_bytes > merge_bytes ? ring_bytes : merge_bytes) + (size_t)(D / 16) * 32 * 16 + warps * DEC_STAGES * 8 +
                        (bulk ? 1024 + DEC_BAR_BYTES : 0);
    const float scale_log2 = scale * 1.4426950408889634f;
    int use_cluster = (error_word != nullptr && cluster_merge && splits >= 2 && splits <= 8) ? 1 : 0;
#define LAUNCH(DD, BB, WW) do { \
        static bool configured = false; \
        if (!configured && smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<DD, BB, WW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        cudaLaunchConfig_t cfg = {}; \
        cfg.gridDim = grid; cfg.blockDim = dim3(WW * 32); cfg.dynamicSmemBytes = smem; cfg.stream = stream; \
        cudaLaunchAttribute attr[2]; \
        attr[0].id = cudaLaunchAttributeClusterDimension; \
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = splits; \
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; \
        attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0; \
        if (use_cluster) { \
            /* clusters are placed whole inside one GPC: if they do not all fit at once, some wait for a second wave, */ \
            /* which costs more than the merge through global memory that the cluster would save */ \
            static int fit[9] = {0}; \
            if (fit[splits] == 0) { \
                cfg.attrs = attr; cfg.numAttrs = 1; \
                int n = 0; \
                if (cudaOccupancyMaxActiveClusters(&n, attn_decode_mma_kernel<DD, BB, WW>, &cfg) != cudaSuccess || n < 1) n = -1; \
                fit[splits] = n; \
            } \
            /* (with a margin: blocks of the kernels before and after share the SMs for a moment) */ \
            if (fit[splits] < 0 || (long long)num_decode * KV * 100 > (long long)fit[splits] * 92) use_cluster = 0; \
        } \
        cfg.attrs = use_cluster ? attr : attr + 1; cfg.numAttrs = use_cluster ? 2 : 1; \
        return (int)cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<DD, BB, WW>, kmap, vmap, \
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
            (__nv_bfloat16*)out, o_part, lse_part, decode_segs, seg_q_start, seg_kv_len, block_table, table_rows, \
            table_stride, H, KV, ps, scale_log2, window, merge_counters, error_word, use_cluster); } while (0)
    if (D == 128) { if (alone) LAUNCH(128, true, DEC_WARPS_ALONE); else if (bulk) LAUNCH(128, true, DEC_WARPS); else LAUNCH(128, false, DEC_WARPS); }
    else { if (alone) LAUNCH(64, true, DEC_WARPS_ALONE); else if (bulk) LAUNCH(64, true, DEC_WARPS); else LAUNCH(64, false, DEC_WARPS); }
#undef LAUNCH
    return (int)cudaGetLastError();
}
