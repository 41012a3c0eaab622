// Paged attention for prompt portions on the 5th-generation tensor cores (tcgen05 + tensor
// memory + TMA), bfloat16, head size 64 or 128, page size a multiple of 8.
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:161-173): gather the context,
// call the library attention once per request.  The mma.sync kernel in attention_prefill_mma.cu
// already reads the pages in place, but the legacy tensor path of this GPU saturates near
// 160 TFLOP/s; this kernel moves both products onto tcgen05:
//   block = 128 query rows of one entry x one query head, 6 warps
//   warp 0   TMA: the query tile once, then 64-key K and V tiles page by page through the block
//            table into a two-stage ring (128-byte swizzle, the layout the MMA descriptors expect)
//   warp 1   one thread issues S = Q K^T (tcgen05.mma, both operands in shared memory, S in 64
//            columns of tensor memory) and O += P V (P read from tensor memory, V from shared
//            memory as an MN-major operand, O in D columns of tensor memory)
//   warps 2-5  one query row per thread (= one tensor-memory lane): read S, mask by position,
//            online softmax in float32 (base 2), write P as packed bfloat16 back to tensor
//            memory; the running output is only rescaled when the row maximum grew by more than
//            2^8 (the exponent offset is kept otherwise), which makes the correction rare;
//            at the end divide by the row sum and store.
// Two blocks fit on an SM (256 tensor-memory columns and 96 KB of shared memory each), so one
// block's softmax overlaps the other's MMAs.  Every mbarrier wait is bounded.
#include "sm100.cuh"
#include <map>
#include <mutex>
#include <tuple>
#include <math.h>

using namespace mi;
using namespace mi::sm100;

__device__ __forceinline__ float max3(float a, float b, float c) {      // one instruction on this architecture
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

#ifdef MI_ATT_TIMING
// phase counters (clock64 ticks summed over blocks): built only with -DMI_ATT_TIMING, read by mi_attn_tc_timing
__device__ unsigned long long att_ticks[16];
#define TICK(var) const long long var = clock64()
#define ADD(slot, a, b) atomicAdd(&att_ticks[slot], (unsigned long long)((b) - (a)))
MI_EXPORT int mi_attn_tc_timing(unsigned long long* out, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out, att_ticks, sizeof(att_ticks));
    if (reset) { unsigned long long z[16] = {}; cudaMemcpyToSymbol(att_ticks, z, sizeof(z)); }
    return (int)e;
}
#else
#define TICK(var)
#define ADD(slot, a, b)
#endif

namespace {

constexpr int BQ = 128, BKV = 64;
constexpr int ATT_THREADS = 224;      // warp 0: Q and K loads, 1: MMA issue, 2-5: softmax, 6: V loads

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ tiles, const int* __restrict__ seg_q_start,
                       const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                       const int* __restrict__ table_rows, int table_stride, int H, int KV, int ps, float scale_log2, int window, int* __restrict__ error_word) {
    constexpr int HALVES = D / 64;                       // 64-element (128-byte) column blocks of a head
    constexpr int Q_BYTES = BQ * D * 2, KV_BYTES = BKV * D * 2;
    constexpr int TMEM_COLS = 256;                       // S0: 64, S1: 64 (P overwrites the first 32 columns of its S), O: D
    constexpr uint32_t S_COL = 0, O_COL = 128;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [Q][K0][K1][V0][V1][barriers]
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + Q_BYTES + 4 * KV_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
    const uint32_t sQ = smem_u32(base), sK = sQ + Q_BYTES, sV = sK + 2 * KV_BYTES;
    const uint32_t q_full = smem_u32(bars), k_full = smem_u32(bars + 1), k_empty = smem_u32(bars + 3),
                   s_full = smem_u32(bars + 5), p_ready = smem_u32(bars + 7), pv_done = smem_u32(bars + 8),
                   v_full = smem_u32(bars + 9), v_empty = smem_u32(bars + 11);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // blocks are handed out x-fastest: all heads of the last (longest) tile first, then the tile before it ...
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int seg = tiles[2 * tile], r0 = tiles[2 * tile + 1];
    const int h = blockIdx.x, kvh = h / (H / KV);
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, pos0 = seg_pos0[seg];
    const int rows = min(BQ, n - r0);
    const int p_first = pos0 + r0, p_last = pos0 + r0 + rows - 1;
    const int kt_lo = window > 0 ? max(0, p_first - window + 1) / BKV : 0;
    const int kt_hi = p_last / BKV;
    const int nt = kt_hi - kt_lo + 1;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(k_full, 1); mbar_init(k_full + 8, 1); mbar_init(k_empty, 1); mbar_init(k_empty + 8, 1);
        mbar_init(v_full, 1); mbar_init(v_full + 8, 1); mbar_init(v_empty, 1); mbar_init(v_empty + 8, 1);
        mbar_init(s_full, 1); mbar_init(s_full + 8, 1); mbar_init(p_ready, 128); mbar_init(pv_done, 1);
        mbar_init_fence();
        tma_prefetch_desc(&qmap); tma_prefetch_desc(&kmap); tma_prefetch_desc(&vmap);
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    pdl_trigger();
    pdl_wait();

    if (warp == 0 || warp == 6) {
        // ---------------- loads.  Warp 0 brings the query tile and the key tiles, warp 6 the value tiles, each
        // through its own two-stage ring: a key stage is free as soon as its QK^T has run, a value stage only
        // after P V, so keys run further ahead.  Lane 0 owns the barriers; the page boxes of a tile are issued
        // by one lane each, so block-table look-ups and TMA issue latencies overlap.
        const bool is_v = warp == 6;
        if (!is_v && lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int hb = 0; hb < HALVES; ++hb)
                tma_load_2d(sQ + hb * (BQ * 128), &qmap, h * D + hb * 64, qs + r0, q_full);
        }
        const int* table_row = block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride;
        const int pages_per_tile = BKV / ps;
        const int ops_per_tile = pages_per_tile * HALVES;
        const uint32_t full = is_v ? v_full : k_full, empty = is_v ? v_empty : k_empty, dst0 = is_v ? sV : sK;
        const CUtensorMap* map = is_v ? &vmap : &kmap;
        bool ok = true;
        for (int i = 0; i < nt; ++i) {
            const int s = i & 1, kt = kt_lo + i;
            if (lane == 0) {
                if (i >= 2 && !mbar_wait(empty + 8 * s, ((i >> 1) - 1) & 1)) { atomicExch(error_word, 21); ok = false; }
                if (ok) mbar_expect_tx(full + 8 * s, KV_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            for (int op = lane; op < ops_per_tile; op += 32) {
                const int pg = op / HALVES, hb = op % HALVES;
                const int j = kt * BKV + pg * ps;
                const int page = j <= p_last ? table_row[j / ps] : 0;              // beyond the last row's keys: null page
                const int y = (page * KV + kvh) * ps;
                tma_load_2d(dst0 + s * KV_BYTES + hb * (BKV * 128) + pg * ps * 128, map, hb * 64, y, full + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc_bf16(BQ, BKV, false);     // S[128 x 64]  = Q (K-major) * K^T (K-major)
            const uint32_t idesc_o = umma_idesc_bf16(BQ, D, true);        // O[128 x D]  += P (tensor memory) * V (MN-major)
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicExch(error_word, 22);
            auto issue_qk = [&](int i) {
                const int s = i & 1;
                if (!mbar_spin(k_full + 8 * s, (i >> 1) & 1)) { atomicExch(error_word, 23); ok = false; return; }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t a = sQ + (ks / 4) * (BQ * 128) + (ks % 4) * 32;
                    const uint32_t b = sK + s * KV_BYTES + (ks / 4) * (BKV * 128) + (ks % 4) * 32;
                    umma_ss(tmem + S_COL + 64 * s, umma_desc_sw128(a, 16, 1024), umma_desc_sw128(b, 16, 1024), idesc_s, ks != 0);
                }
                umma_commit(k_empty + 8 * s);                  // the keys of this stage are free once these finish
                umma_commit(s_full + 8 * s);
            };
            // The scores of tile i+1 are issued BEFORE waiting for the softmax of tile i, into the other
            // S buffer, so the tensor cores work while the softmax warps do.
            if (ok) issue_qk(0);
            for (int i = 0; i < nt && ok; ++i) {
                const int s = i & 1;
                TICK(m0);
                if (i + 1 < nt) issue_qk(i + 1);
                if (!ok) break;
                TICK(m1);
                if (!mbar_spin(p_ready, i & 1)) { atomicExch(error_word, 24); ok = false; break; }
                TICK(m2);
                if (!mbar_spin(v_full + 8 * s, (i >> 1) & 1)) { atomicExch(error_word, 28); ok = false; break; }
                TICK(m3);
                ADD(4, m0, m1); ADD(5, m1, m2); ADD(6, m2, m3);
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                    const uint32_t b = sV + s * KV_BYTES + kk * (16 * 128);
                    umma_ts(tmem + O_COL, tmem + S_COL + 64 * s + kk * 8, umma_desc_sw128(b, BKV * 128, 1024), idesc_o, (i | kk) != 0);
                }
                umma_commit(v_empty + 8 * s);                  // the values of this stage are free once these finish
                umma_commit(pv_done);                          // and O holds tile i
            }
        }
    } else if (warp < 6) {
        // ---------------- softmax: thread <-> query row <-> tensor-memory lane
        const int lg = warp & 3;
        const int row = lg * 32 + lane;                        // row of the tile
        const int p_row = pos0 + r0 + row;
        const uint32_t lane_addr = tmem + ((uint32_t)(lg * 32) << 16);
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < nt && ok; ++i) {
            const int kt = kt_lo + i;
            const uint32_t s_col = S_COL + 64 * (i & 1);
            TICK(t0);
            if (!mbar_spin(s_full + 8 * (i & 1), (i >> 1) & 1)) { atomicExch(error_word, 25); ok = false; break; }
            tc_fence_after();
            TICK(t1);
            uint32_t r[64];                                     // the row's 64 scores, scaled and masked in place
            tmem_ld32(lane_addr + s_col, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tmem_ld32(lane_addr + s_col + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            tmem_wait_ld();
            TICK(ta);
            // Scores stay unscaled in r[]; the scale is folded into the exponent's multiply-add.  Only tiles
            // that touch the diagonal (or the window's edge) for some row of the warp pay for masking.
            const bool inside = kt * BKV + BKV - 1 <= p_row && (window <= 0 || kt * BKV > p_row - window);
            if (!__all_sync(0xffffffffu, inside)) {
#pragma unroll
                for (int c = 0; c < 64; ++c) {
                    const int j = kt * BKV + c;
                    const bool vis = j <= p_row && (window <= 0 || j > p_row - window);
                    if (!vis) r[c] = 0xff800000u;                     // -inf
                }
            }
            // maximum with three-input max (four chains); exponent arguments and row sums with the packed
            // two-float fma/add of this architecture: the softmax warps are bound by instruction issue
            float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 64; c += 8) {
#pragma unroll
                for (int q = 0; q < 4; ++q) mxs[q] = max3(mxs[q], __uint_as_float(r[c + 2 * q]), __uint_as_float(r[c + 2 * q + 1]));
            }
            const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * scale_log2;   // scale > 0
            // keep the exponent offset unless the maximum grew by more than 2^8: rescaling O is then rare
            float alpha = 1.f;
            bool rescale = false;
            if (mx > m_ref + 8.f) {
                alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - mx);
                rescale = i > 0 && m_ref != -INFINITY;
                m_ref = mx;
                l *= alpha;
            }
            const float off = m_ref == -INFINITY ? 0.f : m_ref;
            TICK(tb);
            uint32_t pk[32];
            const float2 scale2 = make_float2(scale_log2, scale_log2), noff2 = make_float2(-off, -off);
            float2 sums[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const float2 arg = __ffma2_rn(make_float2(__uint_as_float(r[2 * c]), __uint_as_float(r[2 * c + 1])), scale2, noff2);
                const float2 p = make_float2(fast_exp2(arg.x), fast_exp2(arg.y));
                sums[c & 3] = __fadd2_rn(sums[c & 3], p);
                __nv_bfloat162 hh = __floats2bfloat162_rn(p.x, p.y);
                pk[c] = *reinterpret_cast<uint32_t*>(&hh);
            }
            const float2 s01 = __fadd2_rn(sums[0], sums[1]), s23 = __fadd2_rn(sums[2], sums[3]);
            const float sum = (s01.x + s01.y) + (s23.x + s23.y);
            l += sum;
            TICK(tc);
            tmem_st32(lane_addr + s_col, pk);                  // P takes the place of the scores it came from
            TICK(t2);
            // Every thread follows pv_done phase by phase (a parity wait can only tell the current phase
            // from the one before it); O holds tile i-1 completely after this.
            if (i > 0 && !mbar_spin(pv_done, (i - 1) & 1)) { atomicExch(error_word, 27); ok = false; }
            if (__any_sync(0xffffffffu, rescale)) {
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(lane_addr + O_COL + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                    tmem_st32(lane_addr + O_COL + c * 32, o);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(p_ready);
            TICK(t3);
#ifdef MI_ATT_TIMING
            if (threadIdx.x == 64) { ADD(0, t0, t1); ADD(1, t1, t2); ADD(2, t2, t3); atomicAdd(&att_ticks[3], 1ull);
                                     ADD(8, t1, ta); ADD(9, ta, tb); ADD(10, tb, tc); ADD(11, tc, t2); }
#endif
        }
        // ---------------- epilogue
        if (ok && !mbar_wait(pv_done, (nt - 1) & 1)) { atomicExch(error_word, 26); ok = false; }
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* orow = out + ((size_t)(qs + r0 + row) * H + h) * D;
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_addr + O_COL + c * 32, o);
                tmem_wait_ld();
                if (row < rows) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint4 w;
                        uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o[8 * v4 + 2 * e]) * inv,
                                                                      __uint_as_float(o[8 * v4 + 2 * e + 1]) * inv);
                            ww[e] = *reinterpret_cast<uint32_t*>(&hh);
                        }
                        reinterpret_cast<uint4*>(orow + c * 32)[v4] = w;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

std::mutex att_mutex;
std::map<std::tuple<const void*, int, int, int, int>, CUtensorMap> cache_maps;

bool cache_map(const void* cache, long long rows, int D, int ps, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(att_mutex);
    auto key = std::make_tuple(cache, (int)(rows & 0x7fffffff), (int)(rows >> 31), D, ps);
    auto it = cache_maps.find(key);
    if (it == cache_maps.end()) {
        CUtensorMap m;
        if (!sm100_host::make_map_bf16(&m, cache, (uint64_t)rows, D, D, ps, 64)) return false;
        it = cache_maps.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

}  // namespace

// tiles: (entry, first row) of 128-row tiles.  cache_rows = pages (with the null page) * KV * page_size.
MI_EXPORT int mi_attn_prefill_tc(const void* q, int q_stride, int num_tokens, const void* k_cache, const void* v_cache,
                                 long long cache_rows, void* out, const int* tiles, int num_tiles, const int* seg_q_start,
                                 const int* seg_pos0, const int* block_table, const int* table_rows, int table_stride, int H,
                                 int KV, int D, int ps, int tile_rows, float scale, int window, int* error_word, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if ((D != 64 && D != 128) || H % KV || tile_rows != BQ || q_stride % 8 || ps % 8 || BKV % ps || ((uintptr_t)q % 16)) return -2;
    CUtensorMap qmap, kmap, vmap;
    if (!sm100_host::make_map_bf16(&qmap, q, num_tokens, (uint64_t)H * D, q_stride, BQ, 64)) return -5;
    if (!cache_map(k_cache, cache_rows, D, ps, &kmap) || !cache_map(v_cache, cache_rows, D, ps, &vmap)) return -5;
    const size_t smem = (size_t)BQ * D * 2 + 4 * (size_t)BKV * D * 2 + 13 * 8 + 16 + 1024;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(H, num_tiles);
#define LAUNCH(DD, IDX) do { \
        static bool configured = false; \
        if (!configured) { \
            cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        return (int)launch_pdl(attn_prefill_tc_kernel<DD>, grid, dim3(ATT_THREADS), smem, stream, qmap, kmap, vmap, \
                               (__nv_bfloat16*)out, tiles, seg_q_start, seg_pos0, block_table, table_rows, table_stride, H, KV, ps, \
                               scale_log2, window, error_word); \
    } while (0)
    if (D == 128) LAUNCH(128, 0);
    LAUNCH(64, 1);
#undef LAUNCH
}
