// Row kernels of a layer whose branches read a 32-bit residual itself and are normed on the way back:
//
//   embed_sinusoid   x = table[token] + position vector (column 2i: sin(pos * f_i), column 2i + 1: cos(pos * f_i))
//   causal_conv      out_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j), inputs before the step from a state record
//   branch_norm_add  x += y / sqrt(mean(y^2) + eps) * w * s, and the new x rounded to the run's dtype for the next reader
//   xielu            a+ z^2 + z / 2 for z > 0, a- (exp(z) - 1 - z) + z / 2 otherwise
//
// Angles, sines, the convolution's sum, the norm and the residual sum are 32-bit in every run.
#include "common.cuh"

template <class T>
__global__ void embed_sinusoid_kernel(const int* __restrict__ tokens, const T* __restrict__ table, const float* __restrict__ freqs,
                                      float* __restrict__ out, SbBatch batch, int width, int vocab, int* status) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x;
    int slot, pos;
    row_place(batch, row, slot, pos);
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_BAD_TOKEN);
        tok = 0;
    }
    const T* src = table + (long long)tok * width;
    float* dst = out + (long long)row * width;
    for (int i = threadIdx.x; 2 * i < width; i += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * freqs[i], &sn, &cs);
        dst[2 * i] = to_f<T>(src[2 * i]) + sn;
        if (2 * i + 1 < width) dst[2 * i + 1] = to_f<T>(src[2 * i + 1]) + cs;
    }
}

// One thread per (row, column).  Input t - taps + 1 + j of the row's sequence is a row of this step when it is not
// before the step's first row, else entry taps - 1 + (that index) of the sequence's record [taps - 1][width].
// weight null: the rows are only rounded to O.
template <class O>
__global__ void causal_conv_kernel(const float* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ state,
                                   long long state_slot, SbBatch batch, int width, int taps, O* __restrict__ out) {
    pdl_wait();
    const int row = blockIdx.x;
    int first = 0, t = 0;
    const float* rec = nullptr;
    if (weight != nullptr) {
        const int s = batch.row_seq[row];
        first = batch.cu_q[s];
        t = row - first;
        if (state != nullptr) rec = state + (long long)batch.seq_slot[s] * state_slot;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float a = x[(long long)row * width + c];
        if (weight != nullptr) {
            const float* w = weight + (long long)c * taps;
            float sum = 0.f;
            for (int j = 0; j < taps; ++j) {
                const int src = t - taps + 1 + j;
                const float v = src >= 0 ? x[(long long)(first + src) * width + c] : rec[(long long)(taps - 1 + src) * width + c];
                sum = fmaf(w[j], v, sum);
            }
            a += sum;
        }
        out[(long long)row * width + c] = from_f<O>(a);
    }
}

// One block per sequence, after the kernel above: the record becomes the last taps - 1 inputs of the sequence.  A step
// of fewer rows than that keeps the later entries of the old record: every thread reads its column's entries before it
// writes them, in rising order.
__global__ void causal_conv_state_kernel(const float* __restrict__ x, float* __restrict__ state, long long state_slot, SbBatch batch,
                                         int width, int taps) {
    pdl_wait();
    const int s = blockIdx.x;
    const int first = batch.cu_q[s], n = batch.cu_q[s + 1] - first, keep = taps - 1;
    float* rec = state + (long long)batch.seq_slot[s] * state_slot;
    for (int c = threadIdx.x; c < width; c += blockDim.x)
        for (int e = 0; e < keep; ++e) {
            const int src = n - keep + e;     // index among the step's rows
            rec[(long long)e * width + c] = src >= 0 ? x[(long long)(first + src) * width + c] : rec[(long long)(e + n) * width + c];
        }
}

// One block per row: x += y * rstd(y) * w (* s); rounded (when given) receives the new x in the run's dtype.
template <class T>
__global__ void branch_norm_add_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ w,
                                       const float* __restrict__ s, T* __restrict__ rounded, int width, float eps) {
    __shared__ float red[33];
    pdl_wait();
    const long long base = (long long)blockIdx.x * width;
    float ss = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = to_f<T>(y[base + c]);
        ss = fmaf(v, v, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    pdl_launch_dependents();
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float n = __fmul_rn(__fmul_rn(to_f<T>(y[base + c]), rstd), w[c]);
        if (s != nullptr) n = __fmul_rn(n, s[c]);
        const float v = x[base + c] + n;
        x[base + c] = v;
        if (rounded != nullptr) rounded[base + c] = from_f<T>(v);
    }
}

template <class T>
__global__ void xielu_kernel(const T* __restrict__ z, T* __restrict__ out, long long n, float a_pos, float a_neg) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = to_f<T>(z[i]);
        out[i] = from_f<T>(xielu_value(v, a_pos, a_neg));
    }
}

extern "C" {

int sb_embed_sinusoid(int dtype, const int* tokens, const void* table, const float* freqs, float* out, SbBatch batch, int width,
                      int vocab, int* status, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == SB_F32)
        sb_launch(embed_sinusoid_kernel<float>, batch.n_rows, threads, 0, stream, tokens, (const float*)table, freqs, out, batch, width,
                  vocab, status);
    else
        sb_launch(embed_sinusoid_kernel<__nv_bfloat16>, batch.n_rows, threads, 0, stream, tokens, (const __nv_bfloat16*)table, freqs,
                  out, batch, width, vocab, status);
    SB_LAUNCH_CHECK();
}

int sb_causal_conv(int out_dtype, const float* x, const float* weight, float* state, long long state_slot, SbBatch batch, int width,
                   int taps, void* out, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (weight != nullptr && (taps < 1 || (taps > 1 && state == nullptr))) return (int)cudaErrorInvalidValue;
    const int threads = width >= 1024 ? 256 : 128;
    if (out_dtype == SB_F32)
        sb_launch(causal_conv_kernel<float>, batch.n_rows, threads, 0, stream, x, weight, (const float*)state, state_slot, batch, width,
                  taps, (float*)out);
    else
        sb_launch(causal_conv_kernel<__nv_bfloat16>, batch.n_rows, threads, 0, stream, x, weight, (const float*)state, state_slot, batch,
                  width, taps, (__nv_bfloat16*)out);
    if (weight != nullptr && taps > 1)
        sb_launch(causal_conv_state_kernel, batch.n_seqs, threads, 0, stream, x, state, state_slot, batch, width, taps);
    SB_LAUNCH_CHECK();
}

int sb_branch_norm_add(int dtype, float* x, const void* y, const float* w, const float* s, void* rounded, int rows, int width, float eps,
                       cudaStream_t stream) {
    if (rows <= 0) return 0;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    if (dtype == SB_F32)
        sb_launch(branch_norm_add_kernel<float>, rows, threads, 0, stream, x, (const float*)y, w, s, (float*)rounded, width, eps);
    else
        sb_launch(branch_norm_add_kernel<__nv_bfloat16>, rows, threads, 0, stream, x, (const __nv_bfloat16*)y, w, s,
                  (__nv_bfloat16*)rounded, width, eps);
    SB_LAUNCH_CHECK();
}

int sb_xielu(int dtype, const void* z, void* out, long long n, float a_pos, float a_neg, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (dtype == SB_F32)
        sb_launch(xielu_kernel<float>, blocks, 256, 0, stream, (const float*)z, (float*)out, n, a_pos, a_neg);
    else
        sb_launch(xielu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)z, (__nv_bfloat16*)out, n, a_pos, a_neg);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
