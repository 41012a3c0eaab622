// Greedy and temperature sampling over float32 logits, one block per row.
//
// Reference (davidjoyme/mini-inference engine/core/sampler.py:3-11): argmax, or a draw from
// softmax(logits / max(temperature, 1e-5)) with the library's global generator; rows with
// temperature 0 take the argmax.  Here the draw is the Gumbel-max form of the same
// distribution: argmax_i(logit_i / T + g_i), g_i = -log(-log(u_i)), with u_i from a counter
// based hash of (request seed, tokens generated so far, i).  A request's draws therefore do
// not depend on which other requests share its batch, and no probabilities are materialised.
// Ties go to the lowest index, as argmax does on the host.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ uint32_t fmix32(uint32_t h) {
    h ^= h >> 16; h *= 0x85ebca6bu; h ^= h >> 13; h *= 0xc2b2ae35u; h ^= h >> 16;
    return h;
}

__device__ __forceinline__ float gumbel(uint32_t seed, uint32_t counter, uint32_t i) {
    uint32_t h = fmix32(i ^ (seed * 0x9E3779B1u));
    h = fmix32(h ^ (counter * 0x85EBCA77u));
    const float u = ((float)(h >> 8) + 0.5f) * (1.0f / 16777216.0f);     // in (0, 1)
    return -logf(-logf(u));
}

template <int NT>
__global__ void sample_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temps,
                              const uint32_t* __restrict__ seeds, const uint32_t* __restrict__ counters,
                              int* __restrict__ out) {
    __shared__ float best_v[NT / 32];
    __shared__ int best_i[NT / 32];
    mi::pdl_trigger();
    mi::pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temps ? temps[r] : 0.f;
    const bool draw = temp > 0.f;
    const float inv_t = draw ? 1.f / fmaxf(temp, 1e-5f) : 1.f;
    const uint32_t seed = draw ? seeds[r] : 0u, counter = draw ? counters[r] : 0u;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += NT) {
        float v = row[i];
        if (draw) v = v * inv_t + gumbel(seed, counter, (uint32_t)i);
        if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < NT / 32; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        out[r] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Large vocabularies: several blocks per row.  Each block folds its slice into one 64-bit key
// (order-preserving bits of the score, then the inverted index so that the lower index wins a
// tie) and raises the row's slot with atomicMax; the block that arrives last decodes the slot
// into the token id and clears slot and counter for the next call.
__device__ __forceinline__ unsigned long long score_key(float v, int i) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (uint32_t)(0x7fffffff - i);
}

template <int NT, int PER_THREAD>
__global__ void sample_split_kernel(const float* __restrict__ logits, int ld, int vocab, const float* __restrict__ temps,
                                    const uint32_t* __restrict__ seeds, const uint32_t* __restrict__ counters,
                                    int* __restrict__ out, unsigned long long* __restrict__ slots,
                                    int* __restrict__ arrivals) {
    __shared__ unsigned long long best[NT / 32];
    mi::pdl_trigger();
    mi::pdl_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temps ? temps[r] : 0.f;
    const bool draw = temp > 0.f;
    const float inv_t = draw ? 1.f / fmaxf(temp, 1e-5f) : 1.f;
    const uint32_t seed = draw ? seeds[r] : 0u, counter = draw ? counters[r] : 0u;
    unsigned long long key = 0;
    const int base = blockIdx.y * NT * PER_THREAD;
#pragma unroll
    for (int k = 0; k < PER_THREAD; ++k) {
        const int i = base + k * NT + threadIdx.x;
        if (i < vocab) {
            float v = row[i];
            if (draw) v = v * inv_t + gumbel(seed, counter, (uint32_t)i);
            const unsigned long long cand = score_key(v, i);
            key = cand > key ? cand : key;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, o);
        key = other > key ? other : key;
    }
    if ((threadIdx.x & 31) == 0) best[threadIdx.x >> 5] = key;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < NT / 32; ++w) key = best[w] > key ? best[w] : key;
        atomicMax(&slots[r], key);
        __threadfence();
        if (atomicAdd(&arrivals[r], 1) == (int)gridDim.y - 1) {
            __threadfence();
            const unsigned long long top = atomicExch(&slots[r], 0ull);
            out[r] = 0x7fffffff - (int)(uint32_t)(top & 0xffffffffu);
            arrivals[r] = 0;
        }
    }
}

// slots (uint64) and arrivals (int32): one element per row, zero before the first call; the kernel
// leaves them zero.  Pass null to use the one-block-per-row kernel.
MI_EXPORT int mi_sample_split(const float* logits, int ld, int rows, int vocab, const float* temps,
                              const uint32_t* seeds, const uint32_t* counters, int* out,
                              unsigned long long* slots, int* arrivals, cudaStream_t stream) {
    if (rows == 0) return 0;
    constexpr int NT = 256, PER = 16;
    const int chunks = (vocab + NT * PER - 1) / (NT * PER);
    return (int)mi::launch_pdl(sample_split_kernel<NT, PER>, dim3(rows, chunks), dim3(NT), 0, stream, logits, ld, vocab,
                               temps, seeds, counters, out, slots, arrivals);
}

MI_EXPORT int mi_sample(const float* logits, int ld, int rows, int vocab, const float* temps, const uint32_t* seeds,
                        const uint32_t* counters, int* out, cudaStream_t stream) {
    if (rows == 0) return 0;
    return (int)mi::launch_pdl(sample_kernel<1024>, dim3(rows), dim3(1024), 0, stream, logits, ld, vocab, temps, seeds, counters, out);
}
