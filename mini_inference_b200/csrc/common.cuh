// Shared device helpers for the sm_100a kernels of this engine.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdlib>

#define MI_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes used across the C interface
#define MI_F32 0
#define MI_BF16 1

namespace mi {

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream still runs; pdl_wait() blocks until the
// predecessor has completed and its writes are visible, so it must come before the first access to
// anything the predecessor produces (or still reads).  pdl_trigger() lets the NEXT kernel start
// its own preamble early.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// round through the storage type: what a value becomes when it is stored and read again
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of NT threads (NT a multiple of 32, at most 1024); every thread gets the
// same value, added in a fixed order so the result does not depend on what else runs.
template <int NT> __device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < NT / 32; ++w) total += scratch[w];
    return total;
}

// 16 bytes of T: 4 floats or 8 bfloat16
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T> __device__ __forceinline__ void load16(const T* p, float* out) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    if constexpr (sizeof(T) == 4) {
        out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
        out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
    } else {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {            // bf16 -> f32 is a shift into the high half
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
}

// two neighbouring elements in one access (p must be aligned to 2 elements)
template <typename T> __device__ __forceinline__ void load2(const T* p, float& a, float& b) {
    if constexpr (sizeof(T) == 4) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        a = v.x; b = v.y;
    } else {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
        a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xffff0000u);
    }
}
template <typename T> __device__ __forceinline__ void store2(T* p, float a, float b) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float2*>(p) = make_float2(a, b);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<uint32_t*>(&h);
    }
}

// Blocks that only request memory into L2 (a weight that the NEXT kernel streams), riding along with a kernel that leaves
// the memory system idle.  Block `part` of `parts` asks for its share of [base, base + bytes) in pieces of
// L2_AHEAD_PIECE bytes; base is 16-byte aligned.  Nothing is written and nothing waits for the data.
constexpr int L2_AHEAD_PIECE = 2048;
__device__ __forceinline__ void l2_prefetch_share(const unsigned char* base, long long bytes, int part, int parts) {
    const long long step = (long long)parts * blockDim.x * L2_AHEAD_PIECE;
    for (long long off = ((long long)part * blockDim.x + threadIdx.x) * L2_AHEAD_PIECE; off < bytes; off += step) {
        const long long left = bytes - off;
        const uint32_t n = (uint32_t)(left < L2_AHEAD_PIECE ? left & ~15ll : L2_AHEAD_PIECE);
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(base + off), "r"(n) : "memory");
    }
}

// streaming multiprocessors of the current device (asked once)
inline int device_sms() {
    static const int n = [] {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
            sms = 1;
        return sms;
    }();
    return n;
}

// how many request-only blocks to add to a kernel that keeps `busy` blocks for itself: the SMs it leaves idle, less a
// margin of 8 for the blocks of the kernel that follows (at least 8 in any case)
inline int l2_prefetch_blocks(long long bytes, int busy) {
    const long long pieces = (bytes + L2_AHEAD_PIECE - 1) / L2_AHEAD_PIECE;
    long long blocks = (pieces + 127) / 128;
    const int sms = device_sms();
    const long long room = busy < sms - 16 ? sms - 8 - busy : 8;
    if (blocks > room) blocks = room;
    return blocks < 1 ? 1 : (int)blocks;
}
// A kernel that carries such blocks takes (ahead, ahead_bytes, work) as plain parameters and starts with
//     if (l2_ahead_rides(ahead, ahead_bytes, work)) return;
// its launch has `work` blocks of its own plus l2_ahead_extra(...) more.  (Plain parameters, not a struct: with the
// three values in a struct parameter the same requests cost a decode step 3 % instead of saving it 3 %.)
__device__ __forceinline__ bool l2_ahead_rides(const unsigned char* __restrict__ ahead, long long ahead_bytes, int work) {
    if ((int)blockIdx.x < work) return false;
    l2_prefetch_share(ahead, ahead_bytes, (int)blockIdx.x - work, (int)gridDim.x - work);
    return true;
}
inline int l2_ahead_extra(const void*& ahead, long long& ahead_bytes, int work) {
    if (ahead == nullptr || ((uintptr_t)ahead % 16) || ahead_bytes < 16) { ahead = nullptr; ahead_bytes = 0; return 0; }
    return l2_prefetch_blocks(ahead_bytes, work);
}

}  // namespace mi

// Host side: launch with the programmatic-serialization attribute when mi_pdl_enabled() says so.
namespace mi {
inline bool pdl_enabled() {
    static const bool on = [] { const char* e = std::getenv("MI_PDL"); return !(e && e[0] == '0'); }();
    return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace mi
