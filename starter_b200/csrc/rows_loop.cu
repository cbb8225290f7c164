// Row kernels of a model whose layers run in passes, of mixers that stand side by side, and of a squared-relu
// feed-forward:
//
//   add_rows     out = x + e + s      (32-bit rows; e: rows of the same shape or none; s: one vector for all rows or none)
//   add_bias     y += b               (in place, the sum 32-bit, rounded once)
//   scaled_sum   out = sa * a + sb * b
//   relu2        max(z, 0)^2
#include "common.cuh"

__global__ void add_rows_kernel(const float* __restrict__ x, const float* __restrict__ e, const float* __restrict__ s,
                                float* __restrict__ out, long long n, int width) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i];
        if (e != nullptr) v += e[i];
        if (s != nullptr) v += s[i % width];
        out[i] = v;
    }
}

template <class T>
__global__ void add_bias_kernel(T* __restrict__ y, const float* __restrict__ b, long long n, int width) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        y[i] = from_f<T>(to_f<T>(y[i]) + b[i % width]);
}

template <class T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float sa, const T* __restrict__ b, float sb, T* __restrict__ out, long long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f<T>(fmaf(sa, to_f<T>(a[i]), sb * to_f<T>(b[i])));
}

template <class T>
__global__ void relu2_kernel(const T* __restrict__ z, T* __restrict__ out, long long n) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f<T>(z[i]), 0.f);
        out[i] = from_f<T>(v * v);
    }
}

static inline int flat_blocks(long long n) { return (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192); }

extern "C" {

int sb_add_rows(const float* x, const float* e, const float* s, float* out, long long rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    sb_launch(add_rows_kernel, flat_blocks(rows * width), 256, 0, stream, x, e, s, out, rows * width, width);
    SB_LAUNCH_CHECK();
}

int sb_add_bias(int dtype, void* y, const float* b, long long rows, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == SB_F32) sb_launch(add_bias_kernel<float>, flat_blocks(rows * width), 256, 0, stream, (float*)y, b, rows * width, width);
    else sb_launch(add_bias_kernel<__nv_bfloat16>, flat_blocks(rows * width), 256, 0, stream, (__nv_bfloat16*)y, b, rows * width, width);
    SB_LAUNCH_CHECK();
}

int sb_scaled_sum(int dtype, const void* a, float sa, const void* b, float sb, void* out, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == SB_F32)
        sb_launch(scaled_sum_kernel<float>, flat_blocks(n), 256, 0, stream, (const float*)a, sa, (const float*)b, sb, (float*)out, n);
    else
        sb_launch(scaled_sum_kernel<__nv_bfloat16>, flat_blocks(n), 256, 0, stream, (const __nv_bfloat16*)a, sa, (const __nv_bfloat16*)b,
                  sb, (__nv_bfloat16*)out, n);
    SB_LAUNCH_CHECK();
}

int sb_relu2(int dtype, const void* z, void* out, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == SB_F32) sb_launch(relu2_kernel<float>, flat_blocks(n), 256, 0, stream, (const float*)z, (float*)out, n);
    else sb_launch(relu2_kernel<__nv_bfloat16>, flat_blocks(n), 256, 0, stream, (const __nv_bfloat16*)z, (__nv_bfloat16*)out, n);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
