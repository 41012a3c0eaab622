// Per-head q/k RMSNorm + rotate-half RoPE + write of k and v into the paged cache, one kernel.
//
// Reference (davidjoyme/mini-inference): engine/core/model_runner.py:148-152 (view as heads,
// q_norm/k_norm over head_dim, q*cos + rotate_half(q)*sin) and :156 with
// engine/core/kv_cache.py:378-382 (the write, before attention).  The reference runs this
// as ~15 elementwise kernels and two index copies.
//
// One warp per (token, head) item; warps walk the items with a grid-wide stride, so a long prompt
// costs a few hundred blocks instead of one tiny block per four heads.  Each lane computes
// cos/sin of pos * inv_freq[i] in float32 for the pairs (i, i + D/2) it rotates.  q is rotated in
// place inside the qkv buffer; k (rotated) and v go to cache position `slot` of their kv head:
//   cache[(page * KV + head) * page_size + offset][0..D)   with page = slot / page_size.
#include "common.cuh"

using namespace mi;

constexpr int MAX_HALF = 128;     // head_dim <= 256

template <typename T, typename WT>
__global__ void qk_norm_rope_cache_kernel(T* __restrict__ qkv, const WT* __restrict__ q_w, const WT* __restrict__ k_w,
                                          const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                          const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          int H, int KV, int D, int page_size, float eps, int num_tokens) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int heads = H + 2 * KV;
    const int half = D / 2;
    const long long items = (long long)num_tokens * heads;
    const long long stride = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < items; item += stride) {
    const int t = (int)(item / heads), h = (int)(item % heads);
    // heads 0..H-1 are q, H..H+KV-1 are k, H+KV..H+2KV-1 are v
    T* x = qkv + ((size_t)t * (H + 2 * KV) + h) * D;
    size_t cache_base = 0;
    if (k_cache && h >= H) {
        const int slot = slots[t];
        cache_base = ((size_t)(slot / page_size) * KV * page_size + (slot % page_size)) * D;
    }
    if (h >= H + KV) {                                     // v: copy to the cache as it is
        if (v_cache) {
            T* dst = v_cache + cache_base + (size_t)(h - H - KV) * page_size * D;
            constexpr int V = Vec16<T>::N;
            if (D % V == 0) {
                for (int i = lane; i < D / V; i += 32)
                    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(x)[i];
            } else {
                for (int i = lane; i < D; i += 32) dst[i] = x[i];
            }
        }
        continue;
    }
    const bool is_k = h >= H;
    if (is_k && !k_cache) continue;                          // reads another step's cache: k unused
    const WT* w = is_k ? k_w : q_w;
    // each lane takes PAIRS of neighbouring elements (one 4- or 8-byte access) of both halves
    float ss = 0.f;
    for (int i = 2 * lane; i < half; i += 64) {
        float a0, a1, b0, b1;
        load2(x + i, a0, a1);
        load2(x + i + half, b0, b1);
        ss += a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1;
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const float pos = inv_freq ? (float)positions[t] : 0.f;
    T* dst = is_k ? k_cache + cache_base + (size_t)(h - H) * page_size * D : x;
    for (int i = 2 * lane; i < half; i += 64) {
        float a[2], b[2], o1[2], o2[2];
        load2(x + i, a[0], a[1]);
        load2(x + i + half, b[0], b[1]);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (w) {
                a[e] = round_to<T>(round_to<T>(a[e] * rstd) * to_f32(w[i + e]));
                b[e] = round_to<T>(round_to<T>(b[e] * rstd) * to_f32(w[i + e + half]));
            }
            o1[e] = a[e]; o2[e] = b[e];
            if (inv_freq) {
                float sn, cs;
                sincosf(pos * inv_freq[i + e], &sn, &cs);
                o1[e] = a[e] * cs - b[e] * sn;
                o2[e] = b[e] * cs + a[e] * sn;
            }
        }
        store2(dst + i, o1[0], o1[1]);
        store2(dst + i + half, o2[0], o2[1]);
    }
}
}

// Long prompts: one block per token.  cos/sin of the token's angles are computed once into shared
// memory and shared by all its heads (the warp-per-item kernel above recomputes them per head, which
// is the better trade only when there are few tokens).
template <typename T, typename WT>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_token_kernel(T* __restrict__ qkv, const WT* __restrict__ q_w, const WT* __restrict__ k_w,
                                const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                int H, int KV, int D, int page_size, float eps) {
    __shared__ float cs[MAX_HALF], sn[MAX_HALF];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int half = D / 2, heads = H + 2 * KV;
    if (inv_freq) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &sn[i], &cs[i]);
    }
    __syncthreads();
    size_t cache_base = 0;
    if (k_cache) {
        const int slot = slots[t];
        cache_base = ((size_t)(slot / page_size) * KV * page_size + (slot % page_size)) * D;
    }
    for (int h = warp; h < heads; h += nwarps) {
        T* x = qkv + ((size_t)t * heads + h) * D;
        if (h >= H + KV) {
            if (v_cache) {
                T* dst = v_cache + cache_base + (size_t)(h - H - KV) * page_size * D;
                constexpr int V = Vec16<T>::N;
                if (D % V == 0) {
                    for (int i = lane; i < D / V; i += 32) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(x)[i];
                } else {
                    for (int i = lane; i < D; i += 32) dst[i] = x[i];
                }
            }
            continue;
        }
        const bool is_k = h >= H;
        if (is_k && !k_cache) continue;
        const WT* w = is_k ? k_w : q_w;
        float ss = 0.f;
        for (int i = 2 * lane; i < half; i += 64) {
            float a0, a1, b0, b1;
            load2(x + i, a0, a1);
            load2(x + i + half, b0, b1);
            ss += a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1;
        }
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / (float)D + eps);
        T* dst = is_k ? k_cache + cache_base + (size_t)(h - H) * page_size * D : x;
        for (int i = 2 * lane; i < half; i += 64) {
            float a[2], b[2], o1[2], o2[2];
            load2(x + i, a[0], a[1]);
            load2(x + i + half, b[0], b[1]);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (w) {
                    a[e] = round_to<T>(round_to<T>(a[e] * rstd) * to_f32(w[i + e]));
                    b[e] = round_to<T>(round_to<T>(b[e] * rstd) * to_f32(w[i + e + half]));
                }
                o1[e] = a[e]; o2[e] = b[e];
                if (inv_freq) {
                    const float c = cs[i + e], sv = sn[i + e];
                    o1[e] = a[e] * c - b[e] * sv;
                    o2[e] = b[e] * c + a[e] * sv;
                }
            }
            store2(dst + i, o1[0], o1[1]);
            store2(dst + i + half, o2[0], o2[1]);
        }
    }
}

// Long prompts, head sizes that are a power-of-two number of 16-byte pieces: LPH lanes hold one head in registers (one
// 16-byte load and one 16-byte store per lane and nothing read twice); the lanes of the two halves of a head exchange
// their normalised values with a shuffle for the rotation.  A block is 8 warps = 256 / LPH heads of one token; the
// token's cos/sin are computed once per block while the loads are in flight.  The kernel is bound by instruction issue,
// not by memory (72 % of issue slots at 38 % of copy bandwidth in its first form), so the bfloat16 path keeps two
// elements per register wherever the arithmetic allows.
template <typename T> __device__ __forceinline__ void unpack16_qk(const uint4& raw, float* out) {
    if constexpr (sizeof(T) == 4) {
        out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
        out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
    } else {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
}
template <typename T> __device__ __forceinline__ void store16_qk(T* p, const float* v) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint4 raw;
        uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = raw;
    }
}

template <typename T, typename WT, int LPH>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_vec_kernel(T* __restrict__ qkv, const WT* __restrict__ q_w, const WT* __restrict__ k_w,
                              const float* __restrict__ inv_freq, const int* __restrict__ positions,
                              const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache,
                              int H, int KV, int page_size, float eps) {
    constexpr int V = Vec16<T>::N, D = LPH * V, HALF = D / 2, HPW = 32 / LPH;
    constexpr bool PACKED = sizeof(T) == 2 && sizeof(WT) == 2;     // bfloat16 rows and weights: two elements per register
    __shared__ __align__(16) float cs[HALF < 4 ? 4 : HALF], sn[HALF < 4 ? 4 : HALF];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = H + 2 * KV;
    const int h = (blockIdx.y * 8 + warp) * HPW + lane / LPH, chunk = lane % LPH;
    const bool active = h < heads;
    T* src = qkv + ((size_t)t * heads + (active ? h : 0)) * D + chunk * V;
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    if (inv_freq) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < HALF; i += 256) sincosf(pos * inv_freq[i], &sn[i], &cs[i]);
    }
    const bool is_v = h >= H + KV, is_k = h >= H && !is_v;
    const WT* w = is_k ? k_w : q_w;
    const bool second = chunk >= LPH / 2;
    const int i0 = (second ? chunk - LPH / 2 : chunk) * V;
    float x[V], out[V];
    unpack16_qk<T>(raw, x);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < V; ++e) ss += x[e] * x[e];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)D + eps);
    __syncthreads();                                       // cos/sin are in shared memory
    if constexpr (PACKED) {
        // normalised values stay packed: bf16(x * rstd), then one bfloat16 multiply by the weight (the product of two
        // bfloat16 numbers is exact in float32, so rounding it once is what the separate steps give); the halves
        // exchange four packed registers; the rotation itself is float32
        uint32_t np[4] = {raw.x, raw.y, raw.z, raw.w};
        if (w && !is_v) {
            const uint4 wr = *reinterpret_cast<const uint4*>(w + chunk * V);
            const uint32_t wp[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 yv = __floats2bfloat162_rn(x[2 * i] * rstd, x[2 * i + 1] * rstd);
                __nv_bfloat162 nv = __hmul2(yv, *reinterpret_cast<const __nv_bfloat162*>(&wp[i]));
                np[i] = *reinterpret_cast<uint32_t*>(&nv);
            }
        }
        if (inv_freq && !is_v) {
            float c[V], sv[V];
#pragma unroll
            for (int i = 0; i < V / 4; ++i) {
                const float4 c4 = *reinterpret_cast<const float4*>(cs + i0 + 4 * i), s4 = *reinterpret_cast<const float4*>(sn + i0 + 4 * i);
                c[4 * i] = c4.x; c[4 * i + 1] = c4.y; c[4 * i + 2] = c4.z; c[4 * i + 3] = c4.w;
                sv[4 * i] = s4.x; sv[4 * i + 1] = s4.y; sv[4 * i + 2] = s4.z; sv[4 * i + 3] = s4.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t pp = __shfl_xor_sync(0xffffffffu, np[i], LPH / 2);
                if (!second) pp ^= 0x80008000u;            // first half: n c - partner s
                const float n0 = __uint_as_float(np[i] << 16), n1 = __uint_as_float(np[i] & 0xffff0000u);
                const float p0 = __uint_as_float(pp << 16), p1 = __uint_as_float(pp & 0xffff0000u);
                out[2 * i] = n0 * c[2 * i] + p0 * sv[2 * i];
                out[2 * i + 1] = n1 * c[2 * i + 1] + p1 * sv[2 * i + 1];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __shfl_xor_sync(0xffffffffu, np[i], LPH / 2);      // keeps the warp's lanes together
                out[2 * i] = __uint_as_float(np[i] << 16); out[2 * i + 1] = __uint_as_float(np[i] & 0xffff0000u);
            }
        }
    } else {
        float n[V];
#pragma unroll
        for (int e = 0; e < V; ++e) n[e] = (w && !is_v) ? round_to<T>(round_to<T>(x[e] * rstd) * to_f32(w[chunk * V + e])) : x[e];
#pragma unroll
        for (int e = 0; e < V; ++e) {
            const float partner = __shfl_xor_sync(0xffffffffu, n[e], LPH / 2);
            out[e] = n[e];
            if (inv_freq && !is_v) out[e] = second ? n[e] * cs[i0 + e] + partner * sn[i0 + e] : n[e] * cs[i0 + e] - partner * sn[i0 + e];
        }
    }
    if (!active) return;
    size_t cache_base = 0;
    if (is_v || is_k) {
        const int slot = slots[t];
        cache_base = ((size_t)(slot / page_size) * KV * page_size + (slot % page_size)) * D;
    }
    if (is_v) {
        if (v_cache) store16_qk(v_cache + cache_base + (size_t)(h - H - KV) * page_size * D + chunk * V, out);
    } else if (is_k) {
        if (k_cache) store16_qk(k_cache + cache_base + (size_t)(h - H) * page_size * D + chunk * V, out);
    } else {
        store16_qk(src, out);
    }
}

MI_EXPORT int mi_qk_norm_rope_cache(void* qkv, const void* q_w, const void* k_w, const float* inv_freq,
                                    const int* positions, const int* slots, void* k_cache, void* v_cache,
                                    int T_, int H, int KV, int D, int page_size, float eps, int dtype, int w_dtype,
                                    cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (D % 4 || D / 2 > MAX_HALF) return -2;
    const long long items = (long long)T_ * (H + 2 * KV);
    const int cap = device_sms() * 8;
    const int blocks = (int)((items + 7) / 8 < cap ? (items + 7) / 8 : cap);
#define VEC(T, WT, L) return (int)launch_pdl(qk_norm_rope_cache_vec_kernel<T, WT, L>, dim3(T_, (H + 2 * KV + 256 / L - 1) / (256 / L)), dim3(256), 0, \
            stream, (T*)qkv, (const WT*)q_w, (const WT*)k_w, inv_freq, positions, slots, (T*)k_cache, (T*)v_cache, H, KV, page_size, eps)
#define LAUNCH(T, WT) do { \
        const int lph = D / (16 / (int)sizeof(T)); \
        if (T_ >= 256 && D % (16 / (int)sizeof(T)) == 0 && ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0)) { \
            if (lph == 2) VEC(T, WT, 2); if (lph == 4) VEC(T, WT, 4); if (lph == 8) VEC(T, WT, 8); \
            if (lph == 16) VEC(T, WT, 16); if (lph == 32) VEC(T, WT, 32); } \
        if (T_ >= 256) return (int)launch_pdl(qk_norm_rope_cache_token_kernel<T, WT>, dim3(T_), dim3(256), 0, stream, (T*)qkv, (const WT*)q_w, \
            (const WT*)k_w, inv_freq, positions, slots, (T*)k_cache, (T*)v_cache, H, KV, D, page_size, eps); \
        return (int)launch_pdl(qk_norm_rope_cache_kernel<T, WT>, dim3(blocks), dim3(256), 0, stream, (T*)qkv, (const WT*)q_w, (const WT*)k_w, \
            inv_freq, positions, slots, (T*)k_cache, (T*)v_cache, H, KV, D, page_size, eps, T_); } while (0)
    if (dtype == MI_BF16 && w_dtype == MI_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == MI_BF16) LAUNCH(__nv_bfloat16, float);
    else if (w_dtype == MI_F32) LAUNCH(float, float);
    else return -1;
#undef LAUNCH
#undef VEC
    return (int)cudaGetLastError();
}
