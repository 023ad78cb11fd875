// Row softmax over the last dimension for sm_100a: the kernel of the math-path attention
// (scores -> probabilities). Replaces softmax_{f32,f16,bf16} of luma-cuda/kernels/nn.cu:21-76,
// which reads every row three times (max, sum, normalise) with one element per load and does its
// arithmetic in the storage type. Here a row is read once with 16-byte loads, kept in registers,
// reduced in f32 (running max and sum merged across lanes with the online-softmax rule of
// luma-cpu/src/kernels/nn.rs:39-56) and written once, rounded to nearest even: the kernel is bound
// by HBM at 2 * rows * row_size * sizeof(T) bytes.
// 32 elements per thread throughout (4 vectors of 16-bit storage, 8 of f32):
//   rows of up to 1024 elements  : one warp per row (several short rows at a time), no shared memory
//   rows of up to 32768 elements : one CTA of 64 .. 1024 threads per row, one shared-memory exchange
//   longer or unaligned rows     : one CTA per row, two passes over the row (read twice)
#include "common.cuh"
#include "../../include/luma_nn_kernels.h"

namespace fa {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

template <typename T> struct VecOf;
template <> struct VecOf<float> { static constexpr int n = 4; };
template <> struct VecOf<__half> { static constexpr int n = 8; };
template <> struct VecOf<__nv_bfloat16> { static constexpr int n = 8; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&x)[VecOf<T>::n]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VecOf<T>::n; ++i) x[i] = to_f32<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&x)[VecOf<T>::n]) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < VecOf<T>::n; ++i) e[i] = from_f32<T>(x[i]);
    *reinterpret_cast<uint4*>(p) = raw;
}

__device__ __forceinline__ float fast_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// (m, s) = running max and sum of exp(x - m); merging two partial results
__device__ __forceinline__ void merge(float& m, float& s, float m2, float s2) {
    const float mn = fmaxf(m, m2);
    // exp2f(-inf - -inf) would be NaN: an empty partial (s == 0) contributes nothing
    const float a = s == 0.0f ? 0.0f : s * exp2f((m - mn) * kLog2e);
    const float b = s2 == 0.0f ? 0.0f : s2 * exp2f((m2 - mn) * kLog2e);
    m = mn;
    s = a + b;
}
__device__ __forceinline__ void warp_merge(float& m, float& s) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, off);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, off);
        merge(m, s, m2, s2);
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// One warp works on R rows at a time, each row in VPT vectors per lane (R * VPT vectors = 32 elements per lane).
template <typename T, int VPT, int R>
__global__ void __launch_bounds__(256) softmax_warp_kernel(const T* __restrict__ in, T* __restrict__ out, long long rows, int n) {
    constexpr int V = VecOf<T>::n;
    const int lane = threadIdx.x & 31;
    const long long row0 = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * R;
    if (row0 >= rows) return;
    float x[R][VPT][V];
    float m[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        m[r] = -INFINITY;
        const bool live = row0 + r < rows;
        const T* src = in + (row0 + r) * n;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int col = (v * 32 + lane) * V;
            if (live && col < n) {
                load_vec<T>(src + col, x[r][v]);
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) x[r][v][i] = -INFINITY;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int v = 0; v < VPT; ++v)
#pragma unroll
            for (int i = 0; i < V; ++i) m[r] = fmaxf(m[r], x[r][v][i]);
        float s = 0.0f;
        const float ml = m[r] == -INFINITY ? 0.0f : m[r] * kLog2e;   // a lane that saw only -inf: exp2(-inf) = 0
#pragma unroll
        for (int v = 0; v < VPT; ++v)
#pragma unroll
            for (int i = 0; i < V; ++i) {
                x[r][v][i] = fast_ex2(fmaf(x[r][v][i], kLog2e, -ml));   // exp(x - m_lane)
                s += x[r][v][i];
            }
        // exp(x - m_row) / s_row = exp(x - m_lane) * exp(m_lane - m_row) / s_row: the row max first, then
        // every lane's sum rescaled once; a row of -inf only gives NaN (as the reference's arithmetic does)
        const float mr = warp_max(m[r]);
        const float rescale = (m[r] == -INFINITY && mr != -INFINITY) ? 0.0f : fast_ex2((m[r] - mr) * kLog2e);
        const float sr = warp_sum(s * rescale);
        const float f = rescale / sr;
        if (row0 + r < rows) {
            T* dst = out + (row0 + r) * n;
#pragma unroll
            for (int v = 0; v < VPT; ++v) {
                const int col = (v * 32 + lane) * V;
                if (col < n) {
#pragma unroll
                    for (int i = 0; i < V; ++i) x[r][v][i] *= f;
                    store_vec<T>(dst + col, x[r][v]);
                }
            }
        }
    }
}

// One CTA of THREADS threads per row; VPT vectors per thread; one exchange through shared memory.
template <typename T, int VPT, int THREADS>
__global__ void __launch_bounds__(THREADS) softmax_block_kernel(const T* __restrict__ in, T* __restrict__ out, int n) {
    constexpr int V = VecOf<T>::n;
    __shared__ float sh_m[THREADS / 32], sh_s[THREADS / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* src = in + (long long)blockIdx.x * n;
    T* dst = out + (long long)blockIdx.x * n;
    float x[VPT][V];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int col = (v * THREADS + threadIdx.x) * V;
        if (col < n) {
            load_vec<T>(src + col, x[v]);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) x[v][i] = -INFINITY;
        }
    }
    float m = -INFINITY;
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int i = 0; i < V; ++i) m = fmaxf(m, x[v][i]);
    float s = 0.0f;
    const float ml = m == -INFINITY ? 0.0f : m * kLog2e;   // a thread that saw only -inf: exp2(-inf) = 0
#pragma unroll
    for (int v = 0; v < VPT; ++v)
#pragma unroll
        for (int i = 0; i < V; ++i) {
            x[v][i] = fast_ex2(fmaf(x[v][i], kLog2e, -ml));
            s += x[v][i];
        }
    // row max through shared memory, every thread's sum rescaled once, then the row sum
    float mw = warp_max(m);
    if (lane == 0) sh_m[warp] = mw;
    __syncthreads();
    const float mr = warp_max(lane < THREADS / 32 ? sh_m[lane] : -INFINITY);
    const float rescale = (m == -INFINITY && mr != -INFINITY) ? 0.0f : fast_ex2((m - mr) * kLog2e);
    const float sw = warp_sum(s * rescale);
    if (lane == 0) sh_s[warp] = sw;
    __syncthreads();
    const float sr = warp_sum(lane < THREADS / 32 ? sh_s[lane] : 0.0f);
    const float f = rescale / sr;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int col = (v * THREADS + threadIdx.x) * V;
        if (col < n) {
#pragma unroll
            for (int i = 0; i < V; ++i) x[v][i] *= f;
            store_vec<T>(dst + col, x[v]);
        }
    }
}

constexpr int kStreamThreads = 512;

// Any row length: one CTA per row, pass 1 reduces (m, s) online, pass 2 re-reads and writes. VEC = true
// reads 16 bytes per load (rows and base 16-byte aligned), else one element.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kStreamThreads) softmax_stream_kernel(const T* __restrict__ in, T* __restrict__ out, int n) {
    constexpr int V = VEC ? VecOf<T>::n : 1;
    __shared__ float sh_m[kStreamThreads / 32], sh_s[kStreamThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* src = in + (long long)blockIdx.x * n;
    T* dst = out + (long long)blockIdx.x * n;
    float m = -INFINITY, s = 0.0f;
    for (int c = threadIdx.x * V; c < n; c += kStreamThreads * V) {
        float x[VecOf<T>::n];
        if (VEC) load_vec<T>(src + c, x);
        else x[0] = to_f32<T>(src[c]);
        float mv = x[0];
#pragma unroll
        for (int i = 1; i < V; ++i) mv = fmaxf(mv, x[i]);
        if (mv == -INFINITY) continue;
        float sv = 0.0f;
#pragma unroll
        for (int i = 0; i < V; ++i) sv += fast_ex2((x[i] - mv) * kLog2e);
        merge(m, s, mv, sv);
    }
    warp_merge(m, s);
    if (lane == 0) { sh_m[warp] = m; sh_s[warp] = s; }
    __syncthreads();
    m = lane < kStreamThreads / 32 ? sh_m[lane] : -INFINITY;
    s = lane < kStreamThreads / 32 ? sh_s[lane] : 0.0f;
    warp_merge(m, s);
    const float ml = m * kLog2e, inv = 1.0f / s;
    for (int c = threadIdx.x * V; c < n; c += kStreamThreads * V) {
        float x[VecOf<T>::n];
        if (VEC) load_vec<T>(src + c, x);
        else x[0] = to_f32<T>(src[c]);
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = fast_ex2(fmaf(x[i], kLog2e, -ml)) * inv;
        if (VEC) store_vec<T>(dst + c, x);
        else dst[c] = from_f32<T>(x[0]);
    }
}

template <typename T>
int launch_softmax(const T* in, T* out, long long rows, int n, cudaStream_t stream) {
    constexpr int V = VecOf<T>::n;
    // 32 elements per thread (4 vectors of 16-bit, 8 of f32): few enough registers for 4 CTAs of 256
    // threads per SM, whose loads, arithmetic and stores then overlap; with 128 elements per thread
    // (one resident CTA) a bf16 row of 4096 reached 0.54 of the copy bandwidth
    constexpr int P = 32 / V;
    const bool aligned = (n % V) == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int vecs = (n + V - 1) / V;
    const int warps = 8;
    auto warp_grid = [&](int r) { return (unsigned)((rows + (long long)warps * r - 1) / ((long long)warps * r)); };
    const unsigned grid = (unsigned)rows;
    if (aligned && vecs <= 32 * P) {
        const int vpt = (vecs + 31) / 32;
        if (vpt <= 1) softmax_warp_kernel<T, 1, P><<<warp_grid(P), warps * 32, 0, stream>>>(in, out, rows, n);
        else if (vpt <= 2) softmax_warp_kernel<T, 2, P / 2><<<warp_grid(P / 2), warps * 32, 0, stream>>>(in, out, rows, n);
        else if (vpt <= 4) softmax_warp_kernel<T, 4, P / 4><<<warp_grid(P / 4), warps * 32, 0, stream>>>(in, out, rows, n);
        else softmax_warp_kernel<T, P, 1><<<warp_grid(1), warps * 32, 0, stream>>>(in, out, rows, n);
        note_path("softmax_warp", 1);
    } else if (aligned && vecs <= 1024 * P) {
        if (vecs <= 64 * P) softmax_block_kernel<T, P, 64><<<grid, 64, 0, stream>>>(in, out, n);
        else if (vecs <= 128 * P) softmax_block_kernel<T, P, 128><<<grid, 128, 0, stream>>>(in, out, n);
        else if (vecs <= 256 * P) softmax_block_kernel<T, P, 256><<<grid, 256, 0, stream>>>(in, out, n);
        else if (vecs <= 512 * P) softmax_block_kernel<T, P, 512><<<grid, 512, 0, stream>>>(in, out, n);
        else softmax_block_kernel<T, P, 1024><<<grid, 1024, 0, stream>>>(in, out, n);
        note_path("softmax_block", 1);
    } else {
        if (aligned) softmax_stream_kernel<T, true><<<grid, kStreamThreads, 0, stream>>>(in, out, n);
        else softmax_stream_kernel<T, false><<<grid, kStreamThreads, 0, stream>>>(in, out, n);
        note_path("softmax_stream", 1);
    }
    return check_launch("softmax_last_dim");
}

template <typename T>
int softmax_impl(const void* in, void* out, long long rows, int n, void* stream) {
    set_last_error("");
    cudaGetLastError();
    if (in == nullptr || out == nullptr) {
        set_last_error("luma_softmax: input/output must not be null");
        return FLASH_ATTN_ERR_NULL_PTR;
    }
    if (rows <= 0 || n <= 0 || rows > 0x7fffffffLL) {
        set_last_error("luma_softmax: num_rows and row_size must be > 0 (num_rows < 2^31)");
        return FLASH_ATTN_ERR_INVALID_SHAPE;
    }
    cudaPointerAttributes attr;
    int prev = -1;
    if (cudaPointerGetAttributes(&attr, in) == cudaSuccess && attr.type == cudaMemoryTypeDevice) {
        cudaGetDevice(&prev);
        if (prev != attr.device) cudaSetDevice(attr.device);
        else prev = -1;
    } else {
        cudaGetLastError();
    }
    const int rc = launch_softmax<T>(static_cast<const T*>(in), static_cast<T*>(out), rows, n, static_cast<cudaStream_t>(stream));
    if (prev >= 0) cudaSetDevice(prev);
    return rc;
}

}  // namespace
}  // namespace fa

extern "C" {
int luma_softmax_f32(const float* input, float* output, long long num_rows, int row_size, void* stream) {
    return fa::softmax_impl<float>(input, output, num_rows, row_size, stream);
}
int luma_softmax_f16(const flash_attn_f16_t* input, flash_attn_f16_t* output, long long num_rows, int row_size, void* stream) {
    return fa::softmax_impl<__half>(input, output, num_rows, row_size, stream);
}
int luma_softmax_bf16(const flash_attn_bf16_t* input, flash_attn_bf16_t* output, long long num_rows, int row_size, void* stream) {
    return fa::softmax_impl<__nv_bfloat16>(input, output, num_rows, row_size, stream);
}
}
