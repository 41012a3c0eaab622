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

MI_EXPORT int mi_qk_norm_rope_cache(void* qkv, const void* q_w, const void* k_w, const float* inv_freq,
                                    const int* positions, const int* slots, void* k_cache, void* v_cache,
                                    int T_, int H, int KV, int D, int page_size, float eps, int dtype, int w_dtype,
                                    cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (D % 4 || D / 2 > MAX_HALF) return -2;
    const long long items = (long long)T_ * (H + 2 * KV);
    const int blocks = (int)((items + 7) / 8 < 148 * 8 ? (items + 7) / 8 : 148 * 8);
#define LAUNCH(T, WT) do { \
        if (T_ >= 256) return (int)launch_pdl(qk_norm_rope_cache_token_kernel<T, WT>, dim3(T_), dim3(256), 0, stream, (T*)qkv, (const WT*)q_w, \
            (const WT*)k_w, inv_freq, positions, slots, (T*)k_cache, (T*)v_cache, H, KV, D, page_size, eps); \
        return (int)launch_pdl(qk_norm_rope_cache_kernel<T, WT>, dim3(blocks), dim3(256), 0, stream, (T*)qkv, (const WT*)q_w, (const WT*)k_w, \
            inv_freq, positions, slots, (T*)k_cache, (T*)v_cache, H, KV, D, page_size, eps, T_); } while (0)
    if (dtype == MI_BF16 && w_dtype == MI_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == MI_BF16) LAUNCH(__nv_bfloat16, float);
    else if (w_dtype == MI_F32) LAUNCH(float, float);
    else return -1;
#undef LAUNCH
    return (int)cudaGetLastError();
}
