// One persistent kernel for the second half of a pre-norm block when a step has few rows (decode):
//
//     x     += attn * Wo^T                      (phase 0, result added to the residual stream)
//     h      = rmsnorm(x) * w                   (every block, into its own shared memory)
//     gu     = h * Wgu^T                        (phase 1)
//     act    = silu(gu[:, :I]) * gu[:, I:]      (all blocks, a slice each)
//     delta  = act * Wd^T                       (phase 2)
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:120-131, 196): five library
// calls and two elementwise kernels.  At a handful of rows each of them is a short, latency-bound
// launch: the memory pipe empties at every boundary (fill, drain, launch gap), and that idle time,
// not the bytes, is most of a decode step.  Here the three weight matrices are ONE stream:
//   * one block per SM, resident for the whole chain.  Warp 0 (one thread) requests [128 x 64]
//     weight boxes with TMA into an 8-stage ring and simply carries on into the next matrix while
//     the other warps are still finishing, synchronising or normalising: weights depend on nothing,
//     so HBM stays busy across the phase boundaries.
//   * warp 1 (one thread) requests the matching [rows x 64] activation boxes for the phases whose
//     activations live in global memory, once the grid-wide barrier that produces them has passed.
//   * 8 consumer warps run mma.sync on each stage (weights are the 16-row operand, tokens the 8-wide
//     one), with the same stream-K split and fixed-order fix-up as the single GEMM kernel, then meet
//     the other blocks at a grid-wide barrier (a 64-bit ticket counter in global memory).
// Rounding points are the ones of the separate kernels (bfloat16 after every product, after the
// residual sum, after x * rstd and after the norm weight), so a token's result does not depend on
// which path served it beyond the order of float32 additions inside a sum of squares.
// All blocks must be resident at once: the host launches at most one block per SM and checks that
// one fits.  Every wait (mbarrier, flag, grid barrier) is bounded; when one runs out the block
// raises the error word, stops requesting copies, waits for the ones in flight and runs to the end
// without further waiting, so the launch always finishes.  No cluster multicast is used.
#include "sm100.cuh"
#include <map>
#include <mutex>
#include <tuple>

using namespace mi;
using namespace mi::sm100;

namespace {

constexpr int TR = 128;                 // weight rows per tile
constexpr int KC = 64;                  // k per stage (128 bytes: one swizzle row)
#ifndef MI_CHAIN_STAGES
#define MI_CHAIN_STAGES 8
#endif
constexpr int stages_for(int nt) { return nt == 1 ? MI_CHAIN_STAGES : 7; }     // ring stages (what fits beside the rows)
constexpr int W_BYTES = TR * KC * 2;
constexpr int CONSUMERS = 8;            // consumer warps, 16 weight rows each
constexpr int THREADS = 32 * (2 + CONSUMERS);
constexpr int PHASES = 3;
constexpr int MAX_TILES = 2048;         // row tiles of all phases together (their split table lives in shared memory)
constexpr uint32_t FLAG_SPINS = 1u << 22;
constexpr uint32_t DRAIN_TRIES = 1u << 12;

struct Phase {
    int N, K;                           // weight rows (output columns) and reduction length
    int x_in_smem;                      // activations are the block's own normalised rows (else TMA from global)
    int x_after_barriers;               // grid barriers that must have passed before the global activations exist
    int gated_out;                      // the result is [gate | up]: silu(gate) * up goes to act for the next phase
    int add_to_residual;                // epilogue: residual += result (else: store to out)
    int ldo, max_contrib;
    __nv_bfloat16* out;
    float* workspace;                   // [row tiles][max_contrib][tokens][128] partial sums of the tiles cut between blocks
};

struct Chain {
    Phase ph[PHASES];
    __nv_bfloat16* residual;            // [M, hidden], updated in place by phase 0
    const __nv_bfloat16* norm_w;
    __nv_bfloat16* act;                 // [M, inter]
    unsigned long long* grid_counter;   // tickets of the grid-wide barrier; a multiple of gridDim.x between launches
    int* error_word;
    int ld_res, inter, M;
    int prefetch_ahead;                 // weight boxes asked into L2 beyond the ring while the ring is full
    float eps;
};

struct Maps {
    CUtensorMap w[PHASES];
    CUtensorMap x[PHASES];              // x[1] is unused (phase 1 reads shared memory)
};

struct Share { long long u0, u1, U, G; int NKC; };

// A phase with fewer units than blocks is cut among its first U blocks; the others have nothing to do in it.
__device__ __forceinline__ Share share_of(const Phase& p) {
    Share s;
    s.NKC = p.K / KC;
    s.U = (long long)((p.N + TR - 1) / TR) * s.NKC;
    s.G = s.U < (long long)gridDim.x ? s.U : (long long)gridDim.x;
    const long long b = blockIdx.x;
    s.u0 = b < s.G ? s.U * b / s.G : 0;
    s.u1 = b < s.G ? s.U * (b + 1) / s.G : 0;
    return s;
}
// block that owns unit u when U units are cut into G contiguous shares [floor(U b / G), floor(U (b+1) / G))
__device__ __forceinline__ int owner_of(long long u, long long U, long long G) { return (int)(((u + 1) * G + U - 1) / U - 1); }

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" :: "n"(CONSUMERS * 32) : "memory"); }
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned long long ld_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_async_global() { asm volatile("fence.proxy.async.global;\n" ::: "memory"); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float* v) {
    uint4 raw;
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return raw;
}

#ifdef MI_CHAIN_TIMING
// time stamps (globaltimer, ns) of one consumer thread per block: built only with -DMI_CHAIN_TIMING, read by
// mi_decode_chain_timing.  [block][0] start, [1] predecessor finished, then per phase: activations ready, first
// stage landed, units done, grid barrier passed.
__device__ unsigned long long chain_stamps[160][16];
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}
#define STAMP(slot) do { if (ctid == 0 && blockIdx.x < 160) chain_stamps[blockIdx.x][slot] = now_ns(); } while (0)
MI_EXPORT int mi_decode_chain_timing(unsigned long long* out) {
    return (int)cudaMemcpyFromSymbol(out, chain_stamps, sizeof(chain_stamps));
}
#else
#define STAMP(slot)
#endif

template <int NT>
__global__ void __launch_bounds__(THREADS, 1)
decode_chain_kernel(const __grid_constant__ Maps maps, const __grid_constant__ Chain ch) {
    constexpr int TOK = NT * 8;
    constexpr int NS = stages_for(NT);
    constexpr int X_BYTES = TOK * KC * 2;
    constexpr int STAGE = W_BYTES + X_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzle atoms are 1 KB
    const int hidden = ch.ph[1].K;
    unsigned char* hbuf = base + NS * STAGE;               // [hidden / 64][TOK][64] normalised rows, swizzled like a TMA box
    unsigned char* wnorm = hbuf + (size_t)(hidden / KC) * X_BYTES;         // the norm weight, fetched before it is needed
    uint32_t* tile_info = reinterpret_cast<uint32_t*>(wnorm + (size_t)hidden * 2);   // per row tile: first block | blocks << 16
    int tile_base[PHASES + 1];
    tile_base[0] = 0;
#pragma unroll
    for (int p = 0; p < PHASES; ++p) tile_base[p + 1] = tile_base[p] + (ch.ph[p].N + TR - 1) / TR;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tile_info + ((tile_base[PHASES] + 3) & ~3));
    __shared__ volatile int barriers_passed;
    __shared__ volatile int abort_flag;
    const uint32_t stage0 = smem_u32(base), full0 = smem_u32(bars), empty0 = smem_u32(bars + NS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int M = ch.M;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 2); mbar_init(empty0 + 8 * s, CONSUMERS); }
        mbar_init_fence();
        barriers_passed = 0;
        abort_flag = 0;
        for (int p = 0; p < PHASES; ++p) { tma_prefetch_desc(&maps.w[p]); if (!ch.ph[p].x_in_smem) tma_prefetch_desc(&maps.x[p]); }
    }
    __syncthreads();
    pdl_trigger();                                         // the next kernel may begin its own preamble

    if (warp == 0) {
        // ---------------- weight producer: never waits for anything but a free stage.  While the ring is full it
        // asks the L2 for the boxes it will need next, so that HBM keeps working while the consumers are held up at
        // a phase boundary and the ring refills from L2 afterwards.
        if (lane != 0) return;
        struct Cursor { int p; long long u, u1; int NKC; };
        auto settle = [&](Cursor& cu) {                    // move to the next phase that still has units for this block
            while (cu.p < PHASES && cu.u >= cu.u1) {
                if (++cu.p == PHASES) break;
                const Share sh = share_of(ch.ph[cu.p]);
                cu.u = sh.u0; cu.u1 = sh.u1; cu.NKC = sh.NKC;
            }
        };
        Cursor cur;
        { const Share sh = share_of(ch.ph[0]); cur = Cursor{0, sh.u0, sh.u1, sh.NKC}; }
        settle(cur);
        Cursor pf = cur;
        int i = 0, ipf = 0;                                // units requested into the ring / asked into L2 so far
        bool ok = true;
        while (cur.p < PHASES) {
            const int s = i % NS;
            if (i >= NS) {
                const uint32_t parity = ((i / NS) - 1) & 1;
                while (!mbar_test(empty0 + 8 * s, parity)) {
                    while (ipf < i && pf.p < PHASES) { ++pf.u; settle(pf); ++ipf; }       // never behind the ring
                    if (pf.p < PHASES && ipf - i < ch.prefetch_ahead) {
                        tma_prefetch_l2_2d(&maps.w[pf.p], (int)(pf.u % pf.NKC) * KC, (int)(pf.u / pf.NKC) * TR);
                        ++pf.u; settle(pf); ++ipf;
                    } else {
                        if (!mbar_wait(empty0 + 8 * s, parity)) { atomicExch(ch.error_word, 41); abort_flag = 1; }
                        break;
                    }
                }
            }
            if (abort_flag) { ok = false; break; }
            mbar_expect_tx(full0 + 8 * s, W_BYTES);
            tma_load_2d(stage0 + s * STAGE, &maps.w[cur.p], (int)(cur.u % cur.NKC) * KC, (int)(cur.u / cur.NKC) * TR, full0 + 8 * s);
            ++cur.u; settle(cur); ++i;
        }
        if (!ok)                                           // leave only when the copies already requested have landed
            for (int j = i > NS ? i - NS : 0; j < i; ++j)
                for (uint32_t t = 0; t < DRAIN_TRIES && !mbar_try(full0 + 8 * (j % NS), (j / NS) & 1); ++t) {}
        return;
    }

    if (warp == 1) {
        // ---------------- activation producer
        if (lane != 0) return;
        pdl_wait();                                        // phase 0 reads what the kernel before this one wrote
        int i = 0;
        bool ok = true;
        for (int p = 0; p < PHASES && ok; ++p) {
            const Phase& ph = ch.ph[p];
            const Share sh = share_of(ph);
            bool first = true;
            for (long long u = sh.u0; u < sh.u1; ++u, ++i) {
                const int s = i % NS;
                if (i >= NS && !mbar_wait(empty0 + 8 * s, ((i / NS) - 1) & 1)) { atomicExch(ch.error_word, 42); abort_flag = 1; }
                if (abort_flag) { ok = false; break; }
                if (ph.x_in_smem) { mbar_arrive(full0 + 8 * s); continue; }
                if (first && ph.x_after_barriers > 0) {
                    uint32_t spins = 0;
                    while (barriers_passed < ph.x_after_barriers && !abort_flag) {
                        if (++spins > FLAG_SPINS) { atomicExch(ch.error_word, 43); abort_flag = 1; break; }
                        __nanosleep(32);
                    }
                    if (abort_flag) { ok = false; break; }
                    __threadfence();
                    fence_async_global();                  // other blocks wrote these rows with ordinary stores
                }
                first = false;
                mbar_expect_tx(full0 + 8 * s, X_BYTES);
                tma_load_2d(stage0 + s * STAGE + W_BYTES, &maps.x[p], (int)(u % sh.NKC) * KC, 0, full0 + 8 * s);
            }
        }
        if (!ok)
            for (int j = i > NS ? i - NS : 0; j < i; ++j)
                for (uint32_t t = 0; t < DRAIN_TRIES && !mbar_try(full0 + 8 * (j % NS), (j / NS) & 1); ++t) {}
        return;
    }

    // ---------------- consumers: warp cw owns rows cw*16 .. cw*16+15 of every tile
    const int cw = warp - 2, g = lane >> 2, c = lane & 3;
    const int ctid = threadIdx.x - 64;
    const int r_lo = cw * 16 + g, r_hi = r_lo + 8;
    const long long G = gridDim.x;
    int passed = 0;

    // every block arrives once; a block's ticket tells it which round of gridDim.x arrivals it belongs to
    auto grid_barrier = [&]() {
        consumer_sync();
        if (ctid == 0) {
            unsigned long long ticket;                     // release: this block's writes are visible before the count is
            asm volatile("atom.add.release.gpu.global.u64 %0, [%1], 1;\n" : "=l"(ticket) : "l"(ch.grid_counter) : "memory");
            const unsigned long long target = (ticket / (unsigned long long)G + 1ULL) * (unsigned long long)G;
            uint32_t spins = 0;
            while (!abort_flag && ld_acquire(ch.grid_counter) < target) {
                if (++spins > FLAG_SPINS) { atomicExch(ch.error_word, 44); abort_flag = 1; break; }
            }
            barriers_passed = ++passed;
        }
        consumer_sync();
        if (ctid != 0) ++passed;
    };

    // Result of a phase at (token t, column n) once all its blocks have passed a barrier: a tile that one block
    // computed alone is in ph.out (already rounded); a tile cut between blocks is the sum of their partial sums,
    // added in the order of the shares.
    // (four neighbouring columns at once: n is a multiple of 4, so they lie in one tile)
    auto value4_of = [&](const Phase& ph, int p, int t, int n, float (&out)[4]) {
        const int rt = n / TR, r = n % TR;
        const int contrib = (int)(tile_info[tile_base[p] + rt] >> 16);
        if (contrib == 1) {
            const uint2 raw = __ldcg(reinterpret_cast<const uint2*>(ph.out + (size_t)t * ph.ldo + n));
            out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
            out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
            return;
        }
        const float* src = ph.workspace + (size_t)rt * ph.max_contrib * TR * TOK + (size_t)t * TR + r;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k0 = 0; k0 < contrib; k0 += 8) {          // 8 loads in flight, added in share order
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                v[j] = k0 + j < contrib ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(k0 + j) * TR * TOK)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
        }
        out[0] = bf16_round(sum.x); out[1] = bf16_round(sum.y); out[2] = bf16_round(sum.z); out[3] = bf16_round(sum.w);
    };

    // before the kernel ahead has finished: the norm weight and the table of how each row tile is cut between blocks
    for (int idx = ctid; idx < hidden / 8; idx += CONSUMERS * 32)
        reinterpret_cast<uint4*>(wnorm)[idx] = __ldg(reinterpret_cast<const uint4*>(ch.norm_w) + idx);
#pragma unroll
    for (int p = 0; p < PHASES; ++p) {
        const Share sh = share_of(ch.ph[p]);
        for (int rt = ctid; rt < tile_base[p + 1] - tile_base[p]; rt += CONSUMERS * 32) {
            const int first = owner_of((long long)rt * sh.NKC, sh.U, sh.G), last = owner_of((long long)rt * sh.NKC + sh.NKC - 1, sh.U, sh.G);
            tile_info[tile_base[p] + rt] = (uint32_t)first | ((uint32_t)(last - first + 1) << 16);
        }
    }
    consumer_sync();
    STAMP(0);
    pdl_wait();                                            // before the first read or write of global memory
    STAMP(1);
    float acc[NT][4][4];                                   // [token group][chain][fragment]
    int i = 0;
    for (int p = 0; p < PHASES; ++p) {
        const Phase& ph = ch.ph[p];
        const Share sh = share_of(ph);
        const int NKC = sh.NKC;

        if (ph.x_in_smem) {
            // ---------------- h = rmsnorm(residual) * w, every block for itself (one warp per token): the row goes
            // into shared memory as it is read, then is scaled in place
            const int nvec = hidden / 8;
            for (int t = cw; t < TOK; t += CONSUMERS) {
                unsigned char* row = hbuf + t * 128;
                if (t < M) {
                    const uint4* xr = reinterpret_cast<const uint4*>(ch.residual + (size_t)t * ch.ld_res);
                    float ss = 0.f;
                    for (int i0 = lane; i0 < nvec; i0 += 32 * 12) {
                        uint4 raw[12];
#pragma unroll
                        for (int j = 0; j < 12; ++j) { const int idx = i0 + 32 * j; raw[j] = idx < nvec ? __ldcg(xr + idx) : make_uint4(0, 0, 0, 0); }
#pragma unroll
                        for (int j = 0; j < 12; ++j) {
                            const int idx = i0 + 32 * j;
                            if (idx < nvec) {
                                float v[8];
                                unpack8(raw[j], v);
#pragma unroll
                                for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
                                *reinterpret_cast<uint4*>(row + (size_t)(idx >> 3) * X_BYTES + (((idx & 7) ^ (t & 7)) << 4)) = raw[j];
                            }
                        }
                    }
                    const float rstd = rsqrtf(warp_sum(ss) / (float)hidden + ch.eps);
                    for (int idx = lane; idx < nvec; idx += 32) {
                        uint4* slot = reinterpret_cast<uint4*>(row + (size_t)(idx >> 3) * X_BYTES + (((idx & 7) ^ (t & 7)) << 4));
                        float v[8], w[8];
                        unpack8(*slot, v);
                        unpack8(reinterpret_cast<const uint4*>(wnorm)[idx], w);
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = bf16_round(v[e] * rstd) * w[e];
                        *slot = pack8(v);
                    }
                } else {
                    for (int idx = lane; idx < nvec; idx += 32)
                        *reinterpret_cast<uint4*>(row + (size_t)(idx >> 3) * X_BYTES + ((idx & 7) << 4)) = make_uint4(0, 0, 0, 0);
                }
            }
            consumer_sync();
        }

        STAMP(2 + 4 * p);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 4; ++q) { acc[nt][q][0] = acc[nt][q][1] = acc[nt][q][2] = acc[nt][q][3] = 0.f; }
        int seg_start_kc = (int)(sh.u0 % NKC);

        auto store_final = [&](int t, int n, float v) {
            if (ph.add_to_residual) {
                __nv_bfloat16* r = ch.residual + (size_t)t * ch.ld_res + n;
                *r = __float2bfloat16_rn(__bfloat162float(*r) + bf16_round(v));
            } else {
                ph.out[(size_t)t * ph.ldo + n] = __float2bfloat16_rn(v);
            }
        };

        for (long long u = sh.u0; u < sh.u1; ++u, ++i) {
            const int s = i % NS;
            const int rt = (int)(u / NKC), kc = (int)(u % NKC);
            if (!abort_flag && !mbar_wait(full0 + 8 * s, (i / NS) & 1)) { atomicExch(ch.error_word, 45); abort_flag = 1; }
#ifdef MI_CHAIN_TIMING
            if (u == sh.u0) STAMP(3 + 4 * p);
#endif
            const unsigned char* st = base + s * STAGE;
            const unsigned char* xs = ph.x_in_smem ? hbuf + (size_t)kc * X_BYTES : st + W_BYTES;
#ifndef MI_CHAIN_NOMATH
            // four independent accumulation chains per token group (one per 16 k); chunk 2c + win keeps the eight
            // lanes of a quarter-warp on eight different 16-byte columns of the swizzled rows (no bank conflicts)
#pragma unroll
            for (int win = 0; win < 2; ++win) {
                const int chn = 2 * c + win;
                const uint4 a_lo = *reinterpret_cast<const uint4*>(st + r_lo * 128 + ((chn ^ (r_lo & 7)) << 4));
                const uint4 a_hi = *reinterpret_cast<const uint4*>(st + r_hi * 128 + ((chn ^ (r_hi & 7)) << 4));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int t = nt * 8 + g;              // rows beyond M are zeros (TMA fill / zeroed above)
                    const uint4 b = *reinterpret_cast<const uint4*>(xs + t * 128 + ((chn ^ (t & 7)) << 4));
                    mma16816(acc[nt][2 * win], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
                    mma16816(acc[nt][2 * win + 1], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
                }
            }
#endif
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);

            if (kc != NKC - 1 && u != sh.u1 - 1) continue;
            // ---------------- this block's share of row tile rt ends here: add the four chains in a fixed order
            float sum[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int f = 0; f < 4; ++f) sum[nt][f] = (acc[nt][0][f] + acc[nt][1][f]) + (acc[nt][2][f] + acc[nt][3][f]);
            if (seg_start_kc == 0 && kc == NKC - 1) {      // the whole tile was this block's: finish it here
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int t = nt * 8 + 2 * c, n_lo = rt * TR + r_lo, n_hi = rt * TR + r_hi;
                    if (t < M) {
                        if (n_lo < ph.N) store_final(t, n_lo, sum[nt][0]);
                        if (n_hi < ph.N) store_final(t, n_hi, sum[nt][2]);
                    }
                    if (t + 1 < M) {
                        if (n_lo < ph.N) store_final(t + 1, n_lo, sum[nt][1]);
                        if (n_hi < ph.N) store_final(t + 1, n_hi, sum[nt][3]);
                    }
                }
            } else {                                       // a share of a cut tile: leave the partial sums and go on
                const int first = (int)(tile_info[tile_base[p] + rt] & 0xffffu);
                float* mine = ph.workspace + ((size_t)rt * ph.max_contrib + ((int)blockIdx.x - first)) * TR * TOK;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const int t = nt * 8 + 2 * c;
                    mine[t * TR + r_lo] = sum[nt][0]; mine[(t + 1) * TR + r_lo] = sum[nt][1];
                    mine[t * TR + r_hi] = sum[nt][2]; mine[(t + 1) * TR + r_hi] = sum[nt][3];
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int q = 0; q < 4; ++q) { acc[nt][q][0] = acc[nt][q][1] = acc[nt][q][2] = acc[nt][q][3] = 0.f; }
            seg_start_kc = 0;
        }
        STAMP(4 + 4 * p);
        grid_barrier();                                    // every block's results and partial sums of this phase are in memory
#ifdef MI_CHAIN_TIMING
        if (p < 2) STAMP(14 + p);
#endif

        if (ph.gated_out) {
            // ---------------- act = silu(gate) * up over this phase's result, four columns per thread, dealt out over all blocks
            const int vpr = ch.inter / 4, n_items = M * vpr;
            for (int e = blockIdx.x * (CONSUMERS * 32) + ctid; e < n_items; e += (int)G * (CONSUMERS * 32)) {
                const int t = e / vpr, n = (e % vpr) * 4;
                float gt[4], up[4];
                value4_of(ph, p, t, n, gt);
                value4_of(ph, p, t, n + ch.inter, up);
#pragma unroll
                for (int j = 0; j < 4; ++j) gt[j] = gt[j] / (1.f + expf(-gt[j])) * up[j];
                uint2 packed;
                packed.x = pack_pair(gt[0], gt[1]); packed.y = pack_pair(gt[2], gt[3]);
                *reinterpret_cast<uint2*>(ch.act + (size_t)t * ch.inter + n) = packed;
            }
            fence_async_global();                          // the next reader of act is the TMA unit
            grid_barrier();
        } else {
            // ---------------- finish the cut tiles: 16-row slabs of all tiles dealt out over all blocks
            const int n_items = (int)(sh.U / NKC) * (TR / 16);
            for (int item = blockIdx.x; item < n_items; item += (int)G) {
                const int rt = item / (TR / 16), slab = item % (TR / 16);
                if ((tile_info[tile_base[p] + rt] >> 16) == 1) continue;
                for (int e = ctid; e < 4 * M; e += CONSUMERS * 32) {
                    const int t = e / 4, n = rt * TR + slab * 16 + (e % 4) * 4;
                    if (n < ph.N) {
                        float v[4];
                        value4_of(ph, p, t, n, v);
                        if (ph.add_to_residual) {
                            uint2* r = reinterpret_cast<uint2*>(ch.residual + (size_t)t * ch.ld_res + n);
                            const uint2 old = *r;
                            uint2 upd;
                            upd.x = pack_pair(__uint_as_float(old.x << 16) + v[0], __uint_as_float(old.x & 0xffff0000u) + v[1]);
                            upd.y = pack_pair(__uint_as_float(old.y << 16) + v[2], __uint_as_float(old.y & 0xffff0000u) + v[3]);
                            *r = upd;
                        } else {
                            uint2 packed;
                            packed.x = pack_pair(v[0], v[1]); packed.y = pack_pair(v[2], v[3]);
                            *reinterpret_cast<uint2*>(ph.out + (size_t)t * ph.ldo + n) = packed;
                        }
                    }
                }
            }
            if (p + 1 < PHASES) grid_barrier();
        }
        STAMP(5 + 4 * p);
    }
}

// ---------------------------------------------------------------- host side
std::mutex chain_mutex;
std::map<std::tuple<const void*, int, int>, CUtensorMap> chain_weight_maps;

int weight_map(const void* W, int N, int K, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(chain_mutex);
    auto key = std::make_tuple(W, N, K);
    auto it = chain_weight_maps.find(key);
    if (it == chain_weight_maps.end()) {
        CUtensorMap m;
        if (!sm100_host::make_map_bf16(&m, W, N, K, K, TR, KC)) return -5;
        it = chain_weight_maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

int device_sms() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return sms;
}

struct Split { int row_tiles, max_contrib; };
Split split_of(int N, int K, int G) {
    const long long NKC = K / KC, NRT = (N + TR - 1) / TR, U = NRT * NKC;
    const long long share = U / (U < G ? U : G);             // smallest share of a block that has any
    long long mc = (NKC + share - 1) / share + 1;
    if (mc > NKC) mc = NKC;
    if (mc < 1) mc = 1;
    return Split{(int)NRT, (int)mc};
}

size_t smem_bytes(int NT, int hidden, int tiles) {
    const int NS = stages_for(NT);
    return (size_t)NS * (W_BYTES + NT * 8 * KC * 2) + (size_t)(hidden / KC) * (NT * 8 * KC * 2) + (size_t)hidden * 2 +
           (size_t)((tiles + 3) & ~3) * 4 + 2 * NS * 8 + 1024;
}
int tiles_of(int hidden, int inter) { return 2 * ((hidden + TR - 1) / TR) + (2 * inter + TR - 1) / TR; }

template <int NT>
int launch_chain(const Maps& maps, const Chain& ch, int grid, size_t smem, cudaStream_t stream) {
    auto kern = decode_chain_kernel<NT>;
    static size_t configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem);
        if (e != cudaSuccess) return (int)e;
        if (per_sm < 1) return -2;                           // the blocks could not all be resident
        configured = smem;
    }
    return (int)launch_pdl(kern, dim3(grid), dim3(THREADS), smem, stream, maps, ch);
}

}  // namespace

// Scratch the caller must provide for a chain at these sizes (float32 elements).  Returns -2 when the sizes are not
// taken (more than 16 rows, a dimension that is not a multiple of 64, or rows that do not fit in shared memory beside
// the ring): the caller then runs the separate kernels.
MI_EXPORT int mi_decode_chain_plan(int M, int hidden, int q_dim, int inter, long long* workspace_floats) {
    if (M < 1 || M > 16 || hidden % KC || q_dim % KC || inter % KC || hidden < KC || q_dim < KC || inter < KC) return -2;
    const int NT = M <= 8 ? 1 : 2, G = device_sms();
    if (G < 1) return -4;
    if (tiles_of(hidden, inter) > MAX_TILES || smem_bytes(NT, hidden, tiles_of(hidden, inter)) > 227 * 1024) return -2;
    if ((long long)M * inter >= (1ll << 30)) return -2;
    const Split s0 = split_of(hidden, q_dim, G), s1 = split_of(2 * inter, hidden, G), s2 = split_of(hidden, inter, G);
    const long long tile = (long long)TR * NT * 8;
    *workspace_floats = tile * ((long long)s0.row_tiles * s0.max_contrib + (long long)s1.row_tiles * s1.max_contrib +
                                (long long)s2.row_tiles * s2.max_contrib);
    return 0;
}

// residual[M, hidden] += attn[M, q_dim] * Wo^T; out[M, hidden] = (silu(g) * u) * Wd^T with [g | u] = rmsnorm(residual) * Wgu^T.
// gate_up [M, 2 inter] and act [M, inter] are scratch the caller owns, workspace as the plan says; grid_counter is zero
// before the first call (the kernel leaves it ready for the next, for the same device); error_word is set non-zero if a
// bounded wait inside the kernel ran out.  Everything bfloat16; one launch.
MI_EXPORT int mi_decode_chain(const void* attn, int ld_attn, const void* Wo, void* residual, int ld_res, const void* norm_w,
                              float eps, const void* Wgu, void* gate_up, const void* Wd, void* act, void* out, int M, int hidden,
                              int q_dim, int inter, float* workspace, unsigned long long* grid_counter, int* error_word,
                              cudaStream_t stream) {
    if (M == 0) return 0;
    long long ws_floats;
    int rc = mi_decode_chain_plan(M, hidden, q_dim, inter, &ws_floats);
    if (rc) return rc;
    if (ld_attn % 8 || ld_res % 8 || ((uintptr_t)attn % 16) || ((uintptr_t)residual % 16) || ((uintptr_t)act % 16) ||
        ((uintptr_t)gate_up % 16) || ((uintptr_t)norm_w % 16) || ((uintptr_t)Wo % 16) || ((uintptr_t)Wgu % 16) || ((uintptr_t)Wd % 16))
        return -2;
    const int NT = M <= 8 ? 1 : 2, TOK = NT * 8, G = device_sms();
    Maps maps;
    if ((rc = weight_map(Wo, hidden, q_dim, &maps.w[0]))) return rc;
    if ((rc = weight_map(Wgu, 2 * inter, hidden, &maps.w[1]))) return rc;
    if ((rc = weight_map(Wd, hidden, inter, &maps.w[2]))) return rc;
    if (!sm100_host::make_map_bf16(&maps.x[0], attn, M, q_dim, ld_attn, TOK, KC)) return -5;
    if (!sm100_host::make_map_bf16(&maps.x[2], act, M, inter, inter, TOK, KC)) return -5;
    maps.x[1] = maps.x[0];

    const Split s0 = split_of(hidden, q_dim, G), s1 = split_of(2 * inter, hidden, G), s2 = split_of(hidden, inter, G);
    const size_t tile = (size_t)TR * TOK;
    Chain ch = {};
    // N, K, x_in_smem, x_after_barriers, gated_out, add_to_residual, ldo, max_contrib, out, workspace
    ch.ph[0] = Phase{hidden, q_dim, 0, 0, 0, 1, 0, s0.max_contrib, nullptr, workspace};
    ch.ph[1] = Phase{2 * inter, hidden, 1, 0, 1, 0, 2 * inter, s1.max_contrib, (__nv_bfloat16*)gate_up,
                     workspace + tile * s0.row_tiles * s0.max_contrib};
    ch.ph[2] = Phase{hidden, inter, 0, 4, 0, 0, hidden, s2.max_contrib, (__nv_bfloat16*)out,
                     workspace + tile * ((size_t)s0.row_tiles * s0.max_contrib + (size_t)s1.row_tiles * s1.max_contrib)};
    ch.residual = (__nv_bfloat16*)residual;
    ch.norm_w = (const __nv_bfloat16*)norm_w;
    ch.act = (__nv_bfloat16*)act;
    ch.grid_counter = grid_counter;
    ch.error_word = error_word;
    ch.ld_res = ld_res; ch.inter = inter; ch.M = M; ch.eps = eps;
    static const int prefetch_ahead = [] { const char* e = std::getenv("MI_CHAIN_PREFETCH"); return e ? atoi(e) : 16; }();
    ch.prefetch_ahead = prefetch_ahead;
    const size_t smem = smem_bytes(NT, hidden, tiles_of(hidden, inter));
    return NT == 1 ? launch_chain<1>(maps, ch, G, smem, stream) : launch_chain<2>(maps, ch, G, smem, stream);
}
