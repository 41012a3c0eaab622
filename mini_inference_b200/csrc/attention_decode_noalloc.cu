// mi_attn_decode_noalloc: split-KV decode attention whose scratch lives in the library image
// instead of in allocated memory.  See no_alloc.h for who needs this and what it costs.
#include "no_alloc.h"
#include "common.cuh"
#include <mutex>

// the ordinary entry points (attention_decode_mma.cu, attention_generic.cu); they only launch kernels
extern "C" int mi_attn_decode_mma(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                  float* o_part, float* lse_part, const int* decode_segs, int num_decode,
                                  const int* seg_q_start, const int* seg_kv_len, const int* block_table,
                                  int table_stride, int H, int KV, int D, int ps, int splits, float scale, int window,
                                  cudaStream_t stream);
extern "C" int mi_attn_decode_merge(const float* o_part, const float* lse_part, void* out, const int* decode_segs,
                                    int num_decode, const int* seg_q_start, int H, int D, int splits, int dtype,
                                    cudaStream_t stream);

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table,
// NOT a device address: a kernel given `noalloc_scratch` from the host would fault (or, where
// the GPU can reach host memory, quietly use the wrong bytes).  Host code must ask for the
// address with cudaGetSymbolAddress, per device.
static __device__ __align__(256) unsigned char noalloc_scratch[MI_NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
float* scratch_of_device[MAX_DEVICES] = {};
std::mutex setup_mutex;

// Device address of the array on the CURRENT device, looked up once per device.
int scratch_address(float** ptr) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return MI_NOALLOC_SETUP_FAILED;
    std::lock_guard<std::mutex> lock(setup_mutex);
    if (scratch_of_device[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, noalloc_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return MI_NOALLOC_SETUP_FAILED;
        }
        scratch_of_device[dev] = static_cast<float*>(p);
    }
    *ptr = scratch_of_device[dev];
    return MI_NOALLOC_OK;
}

}  // namespace

MI_EXPORT int mi_attn_decode_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache, void* out,
                                     const int* decode_segs, int num_decode, const int* seg_q_start,
                                     const int* seg_kv_len, const int* block_table, int table_stride, int H, int KV,
                                     int D, int page_size, int splits, float scale, int window, cudaStream_t stream) {
    if (num_decode == 0) return MI_NOALLOC_OK;
    if (num_decode < 0 || splits < 1 || H < 1 || KV < 1) return MI_NOALLOC_BAD_SHAPE;
    float* o_part = nullptr;
    float* lse_part = nullptr;
    if (splits > 1) {
        // partial outputs [num_decode, H, splits, D] then their log-sum-exps [num_decode, H, splits]
        const unsigned long long rows = (unsigned long long)num_decode * H * splits;
        const unsigned long long need = rows * (unsigned long long)(D + 1) * sizeof(float);
        if (need > MI_NOALLOC_SCRATCH_BYTES) return MI_NOALLOC_TOO_LARGE;
        float* base = nullptr;
        const int rc = scratch_address(&base);
        if (rc != MI_NOALLOC_OK) return rc;
        o_part = base;
        lse_part = base + rows * D;
    }
    int err = mi_attn_decode_mma(q, q_stride, k_cache, v_cache, out, o_part, lse_part, decode_segs, num_decode,
                                 seg_q_start, seg_kv_len, block_table, table_stride, H, KV, D, page_size, splits,
                                 scale, window, stream);
    if (err != 0 || splits == 1) return err;
    return mi_attn_decode_merge(o_part, lse_part, out, decode_segs, num_decode, seg_q_start, H, D, splits, MI_BF16, stream);
}

MI_EXPORT const char* mi_attn_decode_noalloc_strerror(int code) {
    switch (code) {
        case MI_NOALLOC_OK: return "ok";
        case MI_NOALLOC_BAD_SHAPE:
            return "shape not supported: head size must be 64 or 128, heads per kv head at most 16, page size a multiple of 16";
        case MI_NOALLOC_TOO_LARGE:
            return "num_decode * H * splits * (D + 1) floats exceed the 8 MiB built-in scratch: use fewer splits or the "
                   "ordinary entry points with caller-provided scratch";
        case MI_NOALLOC_SETUP_FAILED:
            return "could not obtain the device address of the built-in scratch on the current device";
        default: return code > 0 ? "CUDA error at kernel launch (the code is a cudaError_t)" : "unknown code";
    }
}
