// Paged attention for prompt portions on the tensor cores, bfloat16, head size 64 or 128.
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:161-173): a Python loop over
// requests that GATHERS each request's whole context out of the cache and calls the library's
// attention, with a materialised [n, ctx] mask for portions that start after position 0.
// Here one kernel serves every portion of the step: a block takes 64 query rows of one entry
// and one query head, walks the entry's keys in 64-key tiles read in place through the block
// table (cp.async, double buffered, any page size), and keeps a flash-style online softmax in
// float32.  The causal mask is an index comparison (key <= position, with the portion's start
// offset; optionally key > position - window), so nothing is materialised.
//
// Shared-memory tiles are [64][D] bfloat16 with the 16-byte chunk index XOR-ed with (row & 7),
// so ldmatrix reads are conflict free.  Q*K^T and P*V use mma.sync.m16n8k16 with float32
// accumulators; P is re-used from the score accumulators without leaving registers.
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int BQ = 64, BK = 64, PF_WARPS = 4;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;                     // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of 16-byte chunk `chunk` of row `row` in a swizzled [rows][D] bfloat16 tile
template <int D> __device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32, 3)
attn_prefill_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ tiles, const int* __restrict__ seg_q_start,
                        const int* __restrict__ seg_pos0, const int* __restrict__ block_table,
                        const int* __restrict__ table_rows, int table_stride, int H, int KV, int ps, float scale_log2, int window) {
    constexpr int CH = D / 8;               // 16-byte chunks per row
    constexpr int KS = D / 16;              // k-steps of Q K^T
    constexpr int DT = D / 8;               // 8-column output tiles
    constexpr int TILE_BYTES = BK * D * 2;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sK = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const uint32_t sV = sK + 2 * TILE_BYTES;
    const uint32_t sQ = sK + TILE_BYTES;           // the query tile borrows the second key buffer until it is in registers

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    // blocks are handed out x-fastest: all heads of the last (longest) tile first, then the tile before it ...
    const int tile = gridDim.y - 1 - blockIdx.y;
    const int seg = tiles[2 * tile], r0 = tiles[2 * tile + 1];
    const int h = blockIdx.x, kvh = h / (H / KV);
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, pos0 = seg_pos0[seg];
    const int rows = min(BQ, n - r0);
    const int* table_row = block_table + (size_t)(table_rows ? table_rows[seg] : seg) * table_stride;
    const int p_first = pos0 + r0, p_last = pos0 + r0 + rows - 1;
    const int kt_lo = window > 0 ? max(0, p_first - window + 1) / BK : 0;
    const int kt_hi = p_last / BK;                                          // inclusive

    // ---- loads
    {
        const __nv_bfloat16* qbase = q + (size_t)(qs + r0) * q_stride + (size_t)h * D;
        for (int id = tid; id < BQ * CH; id += PF_WARPS * 32) {
            const int row = id / CH, ch = id % CH;
            const bool ok = row < rows;
            cp_async16(sQ + swz<D>(row, ch), ok ? qbase + (size_t)row * q_stride + ch * 8 : q, ok);
        }
    }
    auto load_kv = [&](int kt, int buf) {
        for (int id = tid; id < BK * CH; id += PF_WARPS * 32) {
            const int row = id / CH, ch = id % CH;
            const int j = kt * BK + row;
            const bool ok = j <= p_last;
            size_t off = 0;
            if (ok) off = ((size_t)(table_row[j / ps] * KV + kvh) * ps + j % ps) * D + ch * 8;
            cp_async16(sK + buf * TILE_BYTES + swz<D>(row, ch), k_cache + off, ok);
            cp_async16(sV + buf * TILE_BYTES + swz<D>(row, ch), v_cache + off, ok);
        }
    };
    load_kv(kt_lo, 0);
    cp_async_commit();

    uint32_t qa[KS][4];
    float o[DT][4];
#pragma unroll
    for (int t = 0; t < DT; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int p_row0 = pos0 + r0 + warp * 16 + g, p_row1 = p_row0 + 8;     // positions of this thread's two rows

    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
        const int mi = lane >> 3;
        ldmatrix_x4(qa[ks], sQ + swz<D>(warp * 16 + (lane & 7) + (mi & 1) * 8, ks * 2 + (mi >> 1)));
    }
    __syncthreads();                               // the borrowed buffer is free again

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int buf = (kt - kt_lo) & 1;
        if (kt < kt_hi) { load_kv(kt + 1, buf ^ 1); cp_async_commit(); }      // lands while this tile is computed
        const uint32_t kbuf = sK + buf * TILE_BYTES, vbuf = sV + buf * TILE_BYTES;
        // ---- S = Q K^T : 16 rows x 64 keys per warp
        float s[BK / 8][4];
#pragma unroll
        for (int nt = 0; nt < BK / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int np = 0; np < BK / 16; ++np) {
                uint32_t b[4];
                const int mi = lane >> 3;
                ldmatrix_x4(b, kbuf + swz<D>((2 * np + (mi >> 1)) * 8 + (lane & 7), ks * 2 + (mi & 1)));
                mma16816(s[2 * np], qa[ks], b[0], b[1]);
                mma16816(s[2 * np + 1], qa[ks], b[2], b[3]);
            }
        // ---- mask + online softmax (base 2); a tile wholly inside every row's visible range needs no mask
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const bool inside = kt * BK + BK - 1 <= p_row0 - g && (window <= 0 || kt * BK > p_row0 - g + 15 - window);
        if (inside) {
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] *= scale_log2;
                mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
                mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < BK / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = kt * BK + nt * 8 + 2 * c + e;
                    const bool ok0 = j <= p_row0 && (window <= 0 || j > p_row0 - window);
                    const bool ok1 = j <= p_row1 && (window <= 0 || j > p_row1 - window);
                    s[nt][e] = ok0 ? s[nt][e] * scale_log2 : -INFINITY;
                    s[nt][2 + e] = ok1 ? s[nt][2 + e] * scale_log2 : -INFINITY;
                    mx0 = fmaxf(mx0, s[nt][e]);
                    mx1 = fmaxf(mx1, s[nt][2 + e]);
                }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float z0 = n0 == -INFINITY ? 0.f : n0, z1 = n1 == -INFINITY ? 0.f : n1;   // a row with no key yet
        const float al0 = exp2f(m0 - z0), al1 = exp2f(m1 - z1);
        m0 = n0; m1 = n1;
        l0 *= al0; l1 *= al1;
#pragma unroll
        for (int nt = 0; nt < BK / 8; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - z0); s[nt][1] = exp2f(s[nt][1] - z0);
            s[nt][2] = exp2f(s[nt][2] - z1); s[nt][3] = exp2f(s[nt][3] - z1);
            l0 += s[nt][0] + s[nt][1];
            l1 += s[nt][2] + s[nt][3];
        }
#pragma unroll
        for (int t = 0; t < DT; ++t) { o[t][0] *= al0; o[t][1] *= al0; o[t][2] *= al1; o[t][3] *= al1; }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack2(s[2 * kk][0], s[2 * kk][1]); pa[1] = pack2(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]); pa[3] = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < DT / 2; ++dp) {
                uint32_t b[4];
                const int mi = lane >> 3;
                ldmatrix_x4_trans(b, vbuf + swz<D>(kk * 16 + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1)));
                mma16816(o[2 * dp], pa, b[0], b[1]);
                mma16816(o[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        cp_async_wait<0>();
        __syncthreads();                       // the next tile has landed and everyone is done with this one
    }

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    const int row0 = r0 + warp * 16 + g, row1 = row0 + 8;
    __nv_bfloat16* obase = out + ((size_t)qs * H + h) * D;
#pragma unroll
    for (int t = 0; t < DT; ++t) {
        const int d = t * 8 + 2 * c;
        if (row0 < n) *reinterpret_cast<uint32_t*>(obase + (size_t)row0 * H * D + d) = pack2(o[t][0] * i0, o[t][1] * i0);
        if (row1 < n) *reinterpret_cast<uint32_t*>(obase + (size_t)row1 * H * D + d) = pack2(o[t][2] * i1, o[t][3] * i1);
    }
}

}  // namespace

MI_EXPORT int mi_attn_prefill_mma(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                  const int* tiles, int num_tiles, const int* seg_q_start, const int* seg_pos0,
                                  const int* block_table, const int* table_rows, int table_stride, int H, int KV, int D, int ps,
                                  int tile_rows, float scale, int window, cudaStream_t stream) {
    if (num_tiles == 0) return 0;
    if ((D != 64 && D != 128) || H % KV || tile_rows != BQ || q_stride % 8) return -2;
    static bool configured[2] = {false, false};
    const size_t smem = (size_t)4 * BK * D * 2;
    dim3 grid(H, num_tiles);
    const float scale_log2 = scale * 1.4426950408889634f;
#define LAUNCH(DD, IDX) do { \
        if (!configured[IDX]) { \
            cudaError_t e = cudaFuncSetAttribute(attn_prefill_mma_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured[IDX] = true; \
        } \
        attn_prefill_mma_kernel<DD><<<grid, PF_WARPS * 32, smem, stream>>>( \
            (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
            (__nv_bfloat16*)out, tiles, seg_q_start, seg_pos0, block_table, table_rows, table_stride, H, KV, ps, scale_log2, window); \
    } while (0)
    if (D == 128) LAUNCH(128, 0); else LAUNCH(64, 1);
#undef LAUNCH
    return (int)cudaGetLastError();
}
