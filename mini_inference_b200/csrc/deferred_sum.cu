// Consumers of a product that the stream-K GEMM left as partial sums (mi_gemm_stream_deferred).
//
// Reference (davidjoyme/mini-inference engine/core/model_runner.py:125-131): x = x + proj(...), then the next norm.
// The few-row product cuts its row tiles between blocks; adding the shares inside the GEMM costs it a fence, an atomic
// and a round trip to L2 at the very end of the kernel, on the critical path of a decode step.  The residual addition
// and the norm that follow read every element anyway, so they add the shares themselves: in share order, rounded to
// bfloat16 once, exactly what the GEMM's own fix-up would have stored.
#include "common.cuh"

using namespace mi;

namespace {

constexpr int TR = 128, KC = 64;

// shares of row tile rt when U = row_tiles * (K / 64) units are cut into G contiguous pieces (the GEMM's rule)
__device__ __forceinline__ int owner_of(long long u, long long U, long long G) { return (int)(((u + 1) * G + U - 1) / U - 1); }
__device__ __forceinline__ int shares_of(int rt, int NKC, long long U, long long G) {
    return owner_of((long long)rt * NKC + NKC - 1, U, G) - owner_of((long long)rt * NKC, U, G) + 1;
}

// sum of the shares of four neighbouring columns of token t (n a multiple of 4), rounded to bfloat16
__device__ __forceinline__ float4 sum4(const float* __restrict__ ws, int max_contrib, int tok, int shares, int t, int n) {
    const int rt = n / TR, r = n % TR;
    const float* src = ws + ((size_t)rt * max_contrib * tok + t) * TR + r;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k0 = 0; k0 < shares; k0 += 12) {              // every share of a round requested before the first is added
        float4 v[12];
#pragma unroll
        for (int j = 0; j < 12; ++j)
            v[j] = k0 + j < shares ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(k0 + j) * tok * TR)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 12; ++j) { sum.x += v[j].x; sum.y += v[j].y; sum.z += v[j].z; sum.w += v[j].w; }
    }
    return sum;
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// x[t] += bf16(sum of shares); y[t] = rmsnorm(x[t]) * w.  One block per token, one thread per four columns.
// Blocks beyond the M tokens do no arithmetic: they ask for the first `ahead_bytes` of `ahead` (the weight that the next
// kernel streams) to be brought into L2.  A decode step has a handful of tokens, so this kernel leaves most SMs idle.
// They do not wait for the kernel before this one: measured at Qwen3-4B sizes, 8 rows, the requests are worth 2.4 % of a
// decode step when they go out at once (they fill the product's ramp-down and this kernel's time), 1 % when they wait
// for it to finish, and more than ~32 MB of them costs what it gains (they then compete with the next product's own loads).
template <typename WT>
__global__ void __launch_bounds__(1024)
deferred_add_rmsnorm_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ ws, const WT* __restrict__ w,
                            __nv_bfloat16* __restrict__ y, int M, int N, int K, int G, int max_contrib, int tok, float eps,
                            const unsigned char* __restrict__ ahead, long long ahead_bytes) {
    extern __shared__ int shares[];                        // per row tile
    __shared__ float scratch[32];
    pdl_trigger();
    if (l2_ahead_rides(ahead, ahead_bytes, M)) return;
    const int NKC = K / KC, NRT = (N + TR - 1) / TR;
    const long long U = (long long)NRT * NKC;
    for (int rt = threadIdx.x; rt < NRT; rt += blockDim.x) shares[rt] = shares_of(rt, NKC, U, G);
    __syncthreads();
    pdl_wait();
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N / 4; i += blockDim.x) {
        const int n = i * 4;
        const float4 d = sum4(ws, max_contrib, tok, shares[n / TR], t, n);
        uint2* xp = reinterpret_cast<uint2*>(x + (size_t)t * N + n);
        const uint2 old = *xp;
        const float v0 = bf16_round(__uint_as_float(old.x << 16) + bf16_round(d.x));
        const float v1 = bf16_round(__uint_as_float(old.x & 0xffff0000u) + bf16_round(d.y));
        const float v2 = bf16_round(__uint_as_float(old.y << 16) + bf16_round(d.z));
        const float v3 = bf16_round(__uint_as_float(old.y & 0xffff0000u) + bf16_round(d.w));
        *xp = make_uint2(pack2(v0, v1), pack2(v2, v3));
        ss += v0 * v0 + v1 * v1 + v2 * v2 + v3 * v3;
    }
    // block sum in a fixed order
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += scratch[i];
    const float rstd = rsqrtf(total / (float)N + eps);
    for (int i = threadIdx.x; i < N / 4; i += blockDim.x) {
        const int n = i * 4;
        const uint2 cur = *reinterpret_cast<const uint2*>(x + (size_t)t * N + n);      // this thread's own store
        const float v[4] = {__uint_as_float(cur.x << 16), __uint_as_float(cur.x & 0xffff0000u),
                            __uint_as_float(cur.y << 16), __uint_as_float(cur.y & 0xffff0000u)};
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = bf16_round(v[e] * rstd) * to_f32(w[n + e]);
        *reinterpret_cast<uint2*>(y + (size_t)t * N + n) = make_uint2(pack2(o[0], o[1]), pack2(o[2], o[3]));
    }
}

// out[t] = bf16(sum of shares): for a reader that wants the product itself
__global__ void deferred_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int N, int K, int G,
                                       int max_contrib, int tok) {
    pdl_trigger();
    pdl_wait();
    const int NKC = K / KC, NRT = (N + TR - 1) / TR;
    const long long U = (long long)NRT * NKC;
    const int t = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N / 4; i += gridDim.x * blockDim.x) {
        const int n = i * 4;
        const float4 d = sum4(ws, max_contrib, tok, shares_of(n / TR, NKC, U, G), t, n);
        *reinterpret_cast<uint2*>(out + (size_t)t * N + n) = make_uint2(pack2(d.x, d.y), pack2(d.z, d.w));
    }
}

// out[t, j] = silu(g) * u with g = bf16(sum of shares at column j), u = bf16(sum of shares at column inter + j): the
// gate/up product left as partial sums, the activation applied by its only reader (the two roundings are those of the
// product stored in bfloat16 and read back by the separate activation kernel).  Four columns per thread.
__global__ void deferred_swiglu_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int inter, int K, int G,
                                       int max_contrib, int tok) {
    pdl_trigger();
    pdl_wait();
    const int N = 2 * inter;
    const int NKC = K / KC, NRT = (N + TR - 1) / TR;
    const long long U = (long long)NRT * NKC;
    const int t = blockIdx.y;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < inter / 4; i += gridDim.x * blockDim.x) {
        const int n = i * 4;
        const float4 g = sum4(ws, max_contrib, tok, shares_of(n / TR, NKC, U, G), t, n);
        const float4 u = sum4(ws, max_contrib, tok, shares_of((inter + n) / TR, NKC, U, G), t, inter + n);
        const float gv[4] = {bf16_round(g.x), bf16_round(g.y), bf16_round(g.z), bf16_round(g.w)};
        const float uv[4] = {bf16_round(u.x), bf16_round(u.y), bf16_round(u.z), bf16_round(u.w)};
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = gv[e] / (1.f + expf(-gv[e])) * uv[e];
        *reinterpret_cast<uint2*>(out + (size_t)t * inter + n) = make_uint2(pack2(o[0], o[1]), pack2(o[2], o[3]));
    }
}

}  // namespace

// x [M, N] bfloat16 (contiguous) += the product held as partial sums in ws; y = rmsnorm(x) * w.  (N, K, grid, max_contrib,
// tokens_padded) describe the product as mi_gemm_stream_plan did.  N must be a multiple of 4.
// `ahead` (may be null): a 16-byte aligned tensor that the next kernel reads; its first ahead_bytes are requested into L2.
MI_EXPORT int mi_deferred_add_rmsnorm(void* x, const float* ws, const void* w, void* y, int M, int N, int K, int grid,
                                      int max_contrib, int tokens_padded, float eps, int w_dtype, const void* ahead_ptr,
                                      long long ahead_bytes, cudaStream_t stream) {
    if (M == 0) return 0;
    const int extra = l2_ahead_extra(ahead_ptr, ahead_bytes, M);
    const unsigned char* ahead = (const unsigned char*)ahead_ptr;
    if (N % 4 || K % KC || ((uintptr_t)x % 8) || ((uintptr_t)y % 8) || ((uintptr_t)ws % 16)) return -2;
    const int NRT = (N + TR - 1) / TR;
    int threads = ((N / 4 + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    const size_t smem = (size_t)NRT * sizeof(int);
    if (w_dtype == MI_BF16)
        return (int)launch_pdl(deferred_add_rmsnorm_kernel<__nv_bfloat16>, dim3(M + extra), dim3(threads), smem, stream, (__nv_bfloat16*)x, ws,
                               (const __nv_bfloat16*)w, (__nv_bfloat16*)y, M, N, K, grid, max_contrib, tokens_padded, eps, ahead, ahead_bytes);
    return (int)launch_pdl(deferred_add_rmsnorm_kernel<float>, dim3(M + extra), dim3(threads), smem, stream, (__nv_bfloat16*)x, ws,
                           (const float*)w, (__nv_bfloat16*)y, M, N, K, grid, max_contrib, tokens_padded, eps, ahead, ahead_bytes);
}

MI_EXPORT int mi_deferred_reduce(const float* ws, void* out, int M, int N, int K, int grid, int max_contrib, int tokens_padded,
                                 cudaStream_t stream) {
    if (M == 0) return 0;
    if (N % 4 || K % KC || ((uintptr_t)out % 8) || ((uintptr_t)ws % 16)) return -2;
    const int blocks = (N / 4 + 255) / 256;
    return (int)launch_pdl(deferred_reduce_kernel, dim3(blocks, M), dim3(256), 0, stream, ws, (__nv_bfloat16*)out, N, K, grid,
                           max_contrib, tokens_padded);
}

// out [M, inter] bfloat16 = silu(gate) * up where [gate | up] = the product [M, 2 inter] held as partial sums in ws.
// inter must be a multiple of 4.
MI_EXPORT int mi_deferred_swiglu(const float* ws, void* out, int M, int inter, int K, int grid, int max_contrib,
                                 int tokens_padded, cudaStream_t stream) {
    if (M == 0) return 0;
    if (inter % 4 || K % KC || ((uintptr_t)out % 8) || ((uintptr_t)ws % 16)) return -2;
    const int blocks = (inter / 4 + 255) / 256;
    return (int)launch_pdl(deferred_swiglu_kernel, dim3(blocks, M), dim3(256), 0, stream, ws, (__nv_bfloat16*)out, inter, K, grid,
                           max_contrib, tokens_padded);
}
