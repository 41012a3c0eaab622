// Embedding gather, residual-add + RMSNorm, SwiGLU.
//
// Reference call sites (davidjoyme/mini-inference): engine/core/model_runner.py:115 (embed),
// :120-121,133 (norms and residual additions), :124-127 (act(gate) * up).  The reference runs
// each as several library kernels; here the residual addition is fused into the norm that
// follows it, and the norm on the logit rows reads only those rows.
#include "common.cuh"

using namespace mi;

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int hidden, int vocab) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;       // the host refuses such ids; never read out of range
    const T* src = table + (size_t)id * hidden;
    T* dst = out + (size_t)t * hidden;
    constexpr int V = Vec16<T>::N;
    if (hidden % V == 0) {
        const uint4* s = reinterpret_cast<const uint4*>(src);
        uint4* d = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < hidden / V; i += blockDim.x) d[i] = s[i];
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
    }
}

MI_EXPORT int mi_embedding(const int* ids, const void* table, void* out, int T_, int hidden, int vocab,
                           int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    if (dtype == MI_BF16)
        return (int)launch_pdl(embedding_kernel<__nv_bfloat16>, dim3(T_), dim3(128), 0, stream, ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, hidden, vocab);
    return (int)launch_pdl(embedding_kernel<float>, dim3(T_), dim3(128), 0, stream, ids, (const float*)table, (float*)out, hidden, vocab);
}

// ------------------------------------------------------------------ block-table changes
// table[idx[i]] = val[i] for the entries of the device block tables that changed on the host since the last step
// (cache manager).  Launched plainly and without an early launch_dependents: every kernel of the step, also one whose
// preamble reads the table before its own griddepcontrol.wait, starts after this one has ended.  Padding entries
// write 0 at index 0 (the null row).  Indices outside the table are skipped.
__global__ void scatter_i32_kernel(int* __restrict__ table, const int* __restrict__ idx, const int* __restrict__ val,
                                   int n, long long table_size) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int at = idx[i];
    if (at >= 0 && at < table_size) table[at] = val[i];
}

MI_EXPORT int mi_scatter_i32(int* table, const int* idx, const int* val, int n, long long table_size, cudaStream_t stream) {
    if (n <= 0) return 0;
    scatter_i32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(table, idx, val, n, table_size);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ (x += delta); y = rmsnorm(x) * w
// One block per output row.  rows == nullptr: row r of x is updated in place with delta and
// normalised.  rows != nullptr: output row r is the norm of x[rows[r]] (+ delta[rows[r]]),
// x is left as it is.  The sum x + delta is formed in float32 and rounded to the stream's
// type BEFORE its statistics are taken, as if it had been stored and read back.
template <typename T, typename WT, int NT>
__global__ void add_rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta, const WT* __restrict__ w,
                                   T* __restrict__ y, const int* __restrict__ rows, int hidden, float eps,
        const unsigned char* __restrict__ ahead, long long ahead_bytes, int work) {
    __shared__ float scratch[32];
    pdl_trigger();
    if (l2_ahead_rides(ahead, ahead_bytes, work)) return;
    pdl_wait();
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    T* xr = x + src;
    const T* dr = delta ? delta + src : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = to_f32(xr[i]);
        if (dr) {
            v = round_to<T>(v + to_f32(dr[i]));
            if (!rows) xr[i] = from_f32<T>(v);
        }
        ss += v * v;
    }
    const float total = block_sum<NT>(ss, scratch);
    const float rstd = rsqrtf(total / (float)hidden + eps);
    T* yr = y + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += NT) {
        float v = to_f32(xr[i]);                         // in-place mode: this thread's own store above
        if (dr && rows) v = round_to<T>(v + to_f32(dr[i]));
        const float n = round_to<T>(v * rstd);
        yr[i] = from_f32<T>(n * to_f32(w[i]));
    }
}

// Same arithmetic with 16-byte loads and the row held in registers between the two phases
// (hidden a multiple of the vector width, at most NT * VPT vectors).
template <typename T> __device__ __forceinline__ void store16(T* p, const float* v) {
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

// the same on 16 bytes already in registers
template <typename T> __device__ __forceinline__ void unpack16(const uint4& raw, float* out) {
    if constexpr (sizeof(T) == 4) {
        out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
        out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
    } else {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
}
template <typename T> __device__ __forceinline__ uint4 pack16(const float* v) {
    uint4 raw;
    if constexpr (sizeof(T) == 4) {
        raw = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
    } else {
        uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    return raw;
}

template <typename T, typename WT, int NT, int VPT>
__global__ void __launch_bounds__(NT)
add_rmsnorm_vec_kernel(T* __restrict__ x, const T* __restrict__ delta, const WT* __restrict__ w, T* __restrict__ y,
                       const int* __restrict__ rows, int hidden, float eps,
        const unsigned char* __restrict__ ahead, long long ahead_bytes, int work) {
    __shared__ float scratch[32];
    constexpr int V = Vec16<T>::N;
    pdl_trigger();
    if (l2_ahead_rides(ahead, ahead_bytes, work)) return;
    pdl_wait();
    const int r = blockIdx.x;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const int nvec = hidden / V;
    float vals[VPT][V];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * NT;
        if (i < nvec) {
            load16(x + src + (size_t)i * V, vals[k]);
            if (delta) {
                float d[V];
                load16(delta + src + (size_t)i * V, d);
#pragma unroll
                for (int e = 0; e < V; ++e) vals[k][e] = round_to<T>(vals[k][e] + d[e]);
                if (!rows) store16(x + src + (size_t)i * V, vals[k]);
            }
#pragma unroll
            for (int e = 0; e < V; ++e) ss += vals[k][e] * vals[k][e];
        }
    }
    const float rstd = rsqrtf(block_sum<NT>(ss, scratch) / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = threadIdx.x + k * NT;
        if (i < nvec) {
            float o[V];
#pragma unroll
            for (int e = 0; e < V; ++e) o[e] = round_to<T>(vals[k][e] * rstd) * to_f32(w[(size_t)i * V + e]);
            store16(y + (size_t)r * hidden + (size_t)i * V, o);
        }
    }
}

// Very many rows: one WARP per row (shuffles only, no block barrier), 4 rows per block.  Every 16-byte piece of the row and
// of the addition is requested before the first is used: a store to x between two loads of x would make the compiler
// keep them in order, one round trip to memory each.  The summed row stays packed in registers for the second pass.
template <typename T, typename WT, int VPT>
__global__ void __launch_bounds__(128)
add_rmsnorm_warp_kernel(T* __restrict__ x, const T* __restrict__ delta, const WT* __restrict__ w, T* __restrict__ y,
                        const int* __restrict__ rows, int num_rows, int hidden, float eps,
        const unsigned char* __restrict__ ahead, long long ahead_bytes, int work) {
    constexpr int V = Vec16<T>::N;
    pdl_trigger();
    if (l2_ahead_rides(ahead, ahead_bytes, work)) return;
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (r >= num_rows) return;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden;
    const int nvec = hidden / V;
    uint4 xr[VPT], dr[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = lane + k * 32;
        xr[k] = i < nvec ? *reinterpret_cast<const uint4*>(x + src + (size_t)i * V) : make_uint4(0, 0, 0, 0);
    }
    if (delta) {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int i = lane + k * 32;
            dr[k] = i < nvec ? *reinterpret_cast<const uint4*>(delta + src + (size_t)i * V) : make_uint4(0, 0, 0, 0);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = lane + k * 32;
        float v[V];
        unpack16<T>(xr[k], v);
        if (delta) {
            float d[V];
            unpack16<T>(dr[k], d);
#pragma unroll
            for (int e = 0; e < V; ++e) v[e] = round_to<T>(v[e] + d[e]);
            xr[k] = pack16<T>(v);
            if (!rows && i < nvec) *reinterpret_cast<uint4*>(x + src + (size_t)i * V) = xr[k];
        }
#pragma unroll
        for (int e = 0; e < V; ++e) ss += v[e] * v[e];
    }
    const float rstd = rsqrtf(warp_sum(ss) / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int i = lane + k * 32;
        if (i < nvec) {
            float v[V], o[V];
            unpack16<T>(xr[k], v);
#pragma unroll
            for (int e = 0; e < V; ++e) o[e] = round_to<T>(v[e] * rstd) * to_f32(w[(size_t)i * V + e]);
            store16(y + (size_t)r * hidden + (size_t)i * V, o);
        }
    }
}

// ahead (may be null): a 16-byte aligned tensor that the next kernel streams; at few rows extra blocks of this launch ask
// for its first ahead_bytes to be brought into L2 (l2_ahead_rides in common.cuh).
MI_EXPORT int mi_add_rmsnorm_ahead(void* x, const void* delta, const void* w, void* y, const int* rows, int num_rows,
                                   int hidden, float eps, int dtype, int w_dtype, const void* ahead_ptr, long long ahead_bytes,
                                   cudaStream_t stream) {
    if (num_rows == 0) return 0;
    constexpr int NT = 256;
    const int vw = dtype == MI_BF16 ? 8 : 4;
    const bool vec = hidden % vw == 0 && hidden / vw <= NT * (dtype == MI_BF16 ? 4 : 8) &&
                     ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && ((uintptr_t)delta % 16 == 0);
    const int nvec = hidden / vw;
    // one warp per row only for long prompts: measured at width 2560, a 2,048-token step is 1-2 % faster with it, but at
    // 64 rows (16 blocks on 148 SMs) it cost a decode step 7 %, and alone it is behind a block per row up to 1,024 rows
    const bool by_warp = vec && num_rows >= 1024 && nvec <= 32 * 16;
    const int work = by_warp ? (num_rows + 3) / 4 : num_rows;
    const int blocks = work + l2_ahead_extra(ahead_ptr, ahead_bytes, work);
    const unsigned char* ahead = (const unsigned char*)ahead_ptr;
#define LAUNCH(T, WT) do { \
        if (by_warp && nvec <= 32 * 4) return (int)launch_pdl(add_rmsnorm_warp_kernel<T, WT, 4>, dim3(blocks), dim3(128), 0, stream, (T*)x, (const T*)delta, (const WT*)w, (T*)y, rows, num_rows, hidden, eps, ahead, ahead_bytes, work); \
        if (by_warp && nvec <= 32 * 8) return (int)launch_pdl(add_rmsnorm_warp_kernel<T, WT, 8>, dim3(blocks), dim3(128), 0, stream, (T*)x, (const T*)delta, (const WT*)w, (T*)y, rows, num_rows, hidden, eps, ahead, ahead_bytes, work); \
        if (by_warp && nvec <= 32 * 12) return (int)launch_pdl(add_rmsnorm_warp_kernel<T, WT, 12>, dim3(blocks), dim3(128), 0, stream, (T*)x, (const T*)delta, (const WT*)w, (T*)y, rows, num_rows, hidden, eps, ahead, ahead_bytes, work); \
        if (by_warp) return (int)launch_pdl(add_rmsnorm_warp_kernel<T, WT, 16>, dim3(blocks), dim3(128), 0, stream, (T*)x, (const T*)delta, (const WT*)w, (T*)y, rows, num_rows, hidden, eps, ahead, ahead_bytes, work); \
        if (vec) return (int)launch_pdl(add_rmsnorm_vec_kernel<T, WT, NT, (sizeof(T) == 2 ? 4 : 8)>, dim3(blocks), dim3(NT), 0, stream, (T*)x, (const T*)delta, (const WT*)w, (T*)y, rows, hidden, eps, ahead, ahead_bytes, work); \
        return (int)launch_pdl(add_rmsnorm_kernel<T, WT, NT>, dim3(blocks), dim3(NT), 0, stream, (T*)x, (const T*)delta, (const WT*)w, (T*)y, rows, hidden, eps, ahead, ahead_bytes, work); \
    } while (0)
    if (dtype == MI_BF16 && w_dtype == MI_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == MI_BF16) LAUNCH(__nv_bfloat16, float);
    else if (w_dtype == MI_F32) LAUNCH(float, float);
    else return -1;
#undef LAUNCH
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_add_rmsnorm(void* x, const void* delta, const void* w, void* y, const int* rows, int num_rows,
                             int hidden, float eps, int dtype, int w_dtype, cudaStream_t stream) {
    return mi_add_rmsnorm_ahead(x, delta, w, y, rows, num_rows, hidden, eps, dtype, w_dtype, nullptr, 0, stream);
}

// ------------------------------------------------------------------ silu(gate) * up
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inter) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)rows * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / inter, c = i % inter;
        const float g = to_f32(gate_up[r * 2 * inter + c]);
        const float u = to_f32(gate_up[r * 2 * inter + inter + c]);
        out[i] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

// 16 bytes of gate, 16 bytes of up and 16 bytes of output per thread (inter a multiple of the vector width)
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inter) {
    constexpr int V = Vec16<T>::N;
    pdl_trigger();
    pdl_wait();
    const int vec_per_row = inter / V;
    const size_t n = (size_t)rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / vec_per_row, c = (i % vec_per_row) * V;
        float g[V], u[V], o[V];
        load16(gate_up + r * 2 * inter + c, g);
        load16(gate_up + r * 2 * inter + inter + c, u);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = g[e] / (1.f + expf(-g[e])) * u[e];
        store16(out + r * inter + c, o);
    }
}

MI_EXPORT int mi_swiglu(const void* gate_up, void* out, int rows, int inter, int dtype, cudaStream_t stream) {
    const size_t n = (size_t)rows * inter;
    if (n == 0) return 0;
    const int vw = dtype == MI_BF16 ? 8 : 4;
    const bool vec = inter % vw == 0 && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0);
    const size_t work = vec ? n / vw : n;
    const int cap = device_sms() * 16;
    const int blocks = (int)((work + 255) / 256 < cap ? (work + 255) / 256 : cap);
#define LAUNCH(T) do { \
        if (vec) return (int)launch_pdl(swiglu_vec_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)gate_up, (T*)out, rows, inter); \
        return (int)launch_pdl(swiglu_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)gate_up, (T*)out, rows, inter); \
    } while (0)
    if (dtype == MI_BF16) LAUNCH(__nv_bfloat16); else LAUNCH(float);
#undef LAUNCH
    return (int)cudaGetLastError();
}
