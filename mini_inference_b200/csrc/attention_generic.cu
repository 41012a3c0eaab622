// Paged attention, generic variant: any head size that is a multiple of 8 (16-byte rows) up to
// 256, any number of heads and groups, float32 or bfloat16 storage, optional window.  All
// arithmetic is float32 on the CUDA cores, in an order that depends only on the request's own
// positions, so the float32 engine gives the same bits however a batch is cut or mixed.
// The bfloat16 fast paths live in attention_mma.cu; this file is the float32 path, the
// fall-back for unusual head sizes, and the reference point of the fast kernels' tests.
//
// Reference (davidjoyme/mini-inference): prompt portions attend over the gathered context with
// a causal (offset) mask, engine/core/model_runner.py:161-173; decoded tokens use the split-KV
// kernel kernels/paged_attention/decode_triton.py:6-100 (online softmax per split, then a
// log-sum-exp merge).  Here both read the pages in place through the block table.
//
// Cache layout: [pages, KV, page_size, D]; key j of a request lives at
//   ((table[j / page_size] * KV + kv_head) * page_size + j % page_size) * D.
#include "common.cuh"
#include <math.h>

using namespace mi;

constexpr int MAX_D = 256;
constexpr int WARPS = 4;

// One warp, one query row, keys lo..hi-1.  q_s: the row's query times scale (shared memory).
// Lane j of a chunk scores key j0 + j; outputs are spread over lanes as d = lane + 32 k.
template <typename T>
__device__ __forceinline__ void attend_range(const float* q_s, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                                             const int* __restrict__ table_row, int kvh, int KV, int D, int ps,
                                             int lo, int hi, float& m, float& l, float (&acc)[MAX_D / 32]) {
    const int lane = threadIdx.x & 31;
    constexpr int VN = Vec16<T>::N;
    for (int j0 = lo; j0 < hi; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j < hi;
        long long off = 0;
        float s = -INFINITY;
        if (valid) {
            off = ((long long)(table_row[j / ps] * KV + kvh) * ps + j % ps) * D;
            const T* kr = k_cache + off;
            float dot = 0.f, tmp[VN];
            for (int c = 0; c < D; c += VN) {
                load16(kr + c, tmp);
#pragma unroll
                for (int e = 0; e < VN; ++e) dot += q_s[c + e] * tmp[e];
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float alpha = expf(m - m_new);              // first chunk: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) acc[k] *= alpha;
        const int n = min(32, hi - j0);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long voff = __shfl_sync(0xffffffffu, off, jj);
            const T* vr = v_cache + voff;
#pragma unroll
            for (int k = 0; k < MAX_D / 32; ++k) {
                const int d = lane + 32 * k;
                if (d < D) acc[k] += pj * to_f32(vr[d]);
            }
        }
    }
}

// ------------------------------------------------------------------ prompt portions
// grid (tiles, H): tile = (entry, first row); each warp takes rows of the tile in turn.
template <typename T>
__global__ void attn_prefill_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                                            const T* __restrict__ v_cache, T* __restrict__ out,
                                            const int* __restrict__ tiles, const int* __restrict__ seg_q_start,
                                            const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                                            const int* __restrict__ table_rows, int table_stride, int H, int KV, int D, int ps, int tile_rows,
                                            float scale, int window) {
    __shared__ float q_s[WARPS][MAX_D];
    const int seg = tiles[2 * blockIdx.x], r0 = tiles[2 * blockIdx.x + 1];
    const int h = blockIdx.y, kvh = h / (H / KV);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, pos0 = seg_pos0[seg];
    const int* table_row = block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride;
    const int r_end = min(r0 + tile_rows, n);
    for (int r = r0 + warp; r < r_end; r += WARPS) {
        const int tok = qs + r, p = pos0 + r;
        const T* qr = q + (size_t)tok * q_stride + (size_t)h * D;
        for (int d = lane; d < D; d += 32) q_s[warp][d] = to_f32(qr[d]) * scale;
        __syncwarp();
        float m = -INFINITY, l = 0.f, acc[MAX_D / 32];
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) acc[k] = 0.f;
        const int lo = window > 0 ? max(0, p - window + 1) : 0;
        attend_range<T>(q_s[warp], k_cache, v_cache, table_row, kvh, KV, D, ps, lo, p + 1, m, l, acc);
        T* orow = out + ((size_t)tok * H + h) * D;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) {
            const int d = lane + 32 * k;
            if (d < D) orow[d] = from_f32<T>(acc[k] / l);
        }
        __syncwarp();
    }
}

// ------------------------------------------------------------------ decoded tokens, split over the keys
// grid (decode entries, ceil(H / 4), splits); one warp per query head.
template <typename T>
__global__ void attn_decode_split_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                                         const T* __restrict__ v_cache, T* __restrict__ out,
                                         float* __restrict__ o_part, float* __restrict__ lse_part,
                                         const int* __restrict__ decode_segs, const int* __restrict__ seg_q_start,
                                         const int* __restrict__ seg_kv_len, const int* __restrict__ block_table,
                                         const int* __restrict__ table_rows, int table_stride, int H, int KV, int D, int ps, float scale, int window) {
    __shared__ float q_s[WARPS][MAX_D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * WARPS + warp;
    if (h >= H) return;
    const int seg = decode_segs[blockIdx.x], kvh = h / (H / KV);
    const int tok = seg_q_start[seg], len = seg_kv_len[seg];
    const int S = gridDim.z, s = blockIdx.z;
    const int lo0 = window > 0 ? max(0, len - window) : 0;     // query position is len - 1
    // every request cuts ITS OWN key range into S pieces of whole 32-key chunks
    // (kernels/paged_attention/decode_triton.py:26-30), so the grid depends on the batch only
    const int piece = (((len - lo0) + S - 1) / S + 31) / 32 * 32;
    const int lo = lo0 + s * piece, hi = min(lo + piece, len);
    const T* qr = q + (size_t)tok * q_stride + (size_t)h * D;
    for (int d = lane; d < D; d += 32) q_s[warp][d] = to_f32(qr[d]) * scale;
    __syncwarp();
    float m = -INFINITY, l = 0.f, acc[MAX_D / 32];
#pragma unroll
    for (int k = 0; k < MAX_D / 32; ++k) acc[k] = 0.f;
    if (lo < hi)
        attend_range<T>(q_s[warp], k_cache, v_cache, block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride, kvh, KV, D, ps,
                        lo, hi, m, l, acc);
    const float inv = l > 0.f ? 1.f / l : 0.f;                  // empty piece: output 0, lse -inf
    if (S == 1) {
        T* orow = out + ((size_t)tok * H + h) * D;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) { const int d = lane + 32 * k; if (d < D) orow[d] = from_f32<T>(acc[k] * inv); }
    } else {
        const size_t idx = ((size_t)blockIdx.x * H + h) * S + s;
        float* orow = o_part + idx * D;
#pragma unroll
        for (int k = 0; k < MAX_D / 32; ++k) { const int d = lane + 32 * k; if (d < D) orow[d] = acc[k] * inv; }
        if (lane == 0) lse_part[idx] = l > 0.f ? m + logf(l) : -INFINITY;
    }
}

// out = sum_s e^(lse_s - max) o_s / sum_s e^(lse_s - max)   (decode_triton.py:78-100)
template <typename T>
__global__ void attn_decode_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ lse_part,
                                         T* __restrict__ out, const int* __restrict__ decode_segs,
                                         const int* __restrict__ seg_q_start, int H, int D, int S) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x, h = blockIdx.y;
    const int tok = seg_q_start[decode_segs[i]];
    const size_t base = ((size_t)i * H + h) * S;
    float mx = -INFINITY;
    for (int s = 0; s < S; ++s) mx = fmaxf(mx, lse_part[base + s]);
    float den = 0.f;
    for (int s = 0; s < S; ++s) den += expf(lse_part[base + s] - mx);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float num = 0.f;
        for (int s = 0; s < S; ++s) num += expf(lse_part[base + s] - mx) * o_part[(base + s) * D + d];
        out[((size_t)tok * H + h) * D + d] = from_f32<T>(num / den);
    }
}

MI_EXPORT int mi_attn_prefill_generic(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                      const int* tiles, int num_tiles, const int* seg_q_start, const int* seg_pos0,
                                      const int* block_table, const int* table_rows, int table_stride, int H, int KV, int D,
                                      int ps, int tile_rows, float scale, int window, int dtype, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if (D > MAX_D || D % 8 || (dtype == MI_F32 && D % 4)) return -2;
    dim3 grid(num_tiles, H);
    if (dtype == MI_BF16)
        attn_prefill_generic_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, stream>>>(
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
            (__nv_bfloat16*)out, tiles, seg_q_start, seg_pos0, block_table, table_rows, table_stride, H, KV, D, ps, tile_rows, scale, window);
    else
        attn_prefill_generic_kernel<float><<<grid, WARPS * 32, 0, stream>>>(
            (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache, (float*)out, tiles, seg_q_start,
            seg_pos0, block_table, table_rows, table_stride, H, KV, D, ps, tile_rows, scale, window);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_attn_decode_generic(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                     float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                     const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                     const int* table_rows, int table_stride, int H, int KV, int D, int ps, int splits, float scale,
                                     int window, int dtype, cudaStream_t stream) {
    if (num_decode == 0) return 0;
    if (D > MAX_D || D % 8) return -2;
    dim3 grid(num_decode, (H + WARPS - 1) / WARPS, splits);
#define ARGS(T) (const T*)q, q_stride, (const T*)k_cache, (const T*)v_cache, (T*)out, o_part, lse_part, decode_segs, \
        seg_q_start, seg_kv_len, block_table, table_rows, table_stride, H, KV, D, ps, scale, window
    if (dtype == MI_BF16) attn_decode_split_kernel<__nv_bfloat16><<<grid, WARPS * 32, 0, stream>>>(ARGS(__nv_bfloat16));
    else attn_decode_split_kernel<float><<<grid, WARPS * 32, 0, stream>>>(ARGS(float));
#undef ARGS
    int err = (int)cudaGetLastError();
    if (err || splits == 1) return err;
    dim3 mgrid(num_decode, H);
    if (dtype == MI_BF16)
        attn_decode_merge_kernel<__nv_bfloat16><<<mgrid, 128, 0, stream>>>(o_part, lse_part, (__nv_bfloat16*)out, decode_segs, seg_q_start, H, D, splits);
    else
        attn_decode_merge_kernel<float><<<mgrid, 128, 0, stream>>>(o_part, lse_part, (float*)out, decode_segs, seg_q_start, H, D, splits);
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_attn_decode_merge(const float* o_part, const float* lse_part, void* out, const int* decode_segs,
                                   int num_decode, const int* seg_q_start, int H, int D, int splits, int dtype,
                                   cudaStream_t stream) {
    if (num_decode == 0) return 0;
    dim3 mgrid(num_decode, H);
    if (dtype == MI_BF16)
        return (int)launch_pdl(attn_decode_merge_kernel<__nv_bfloat16>, mgrid, dim3(128), 0, stream, o_part, lse_part, (__nv_bfloat16*)out, decode_segs, seg_q_start, H, D, splits);
    return (int)launch_pdl(attn_decode_merge_kernel<float>, mgrid, dim3(128), 0, stream, o_part, lse_part, (float*)out, decode_segs, seg_q_start, H, D, splits);
}
