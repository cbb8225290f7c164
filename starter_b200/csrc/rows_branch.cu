// Row kernels of a layer whose branches read a 32-bit residual itself and are normed on the way back:
//
//   embed_sinusoid   x = table[token] + position vector (column 2i: sin(pos * f_i), column 2i + 1: cos(pos * f_i))
//   causal_conv      out_t = x_t + sum_j w[:, j] * x_(t - taps + 1 + j), inputs before the step from a state record
//   branch_norm_add  x += y / sqrt(mean(y^2) + eps) * w * s, and the new x rounded to the run's dtype for the next reader,
//                    or its RMS norm times a second weight when the next reader norms the residual first
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

// A block per row (blockIdx.y shares out the columns when rows are few).  Input t - taps + 1 + j of the row's sequence is a row of this step when it is not
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
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
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
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x)
        for (int e = 0; e < keep; ++e) {
            const int src = n - keep + e;     // index among the step's rows
            rec[(long long)e * width + c] = src >= 0 ? x[(long long)(first + src) * width + c] : rec[(long long)(e + n) * width + c];
        }
}

// Four consecutive values of a branch's output as floats, and four floats out in the run's dtype, in one access each.
__device__ __forceinline__ float4 read_four(const float* src) { return *reinterpret_cast<const float4*>(src); }
__device__ __forceinline__ float4 read_four(const __nv_bfloat16* src) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void write_four(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void write_four(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 h[2] = {__floats2bfloat162_rn(v.x, v.y), __floats2bfloat162_rn(v.z, v.w)};
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(h);
}

// One block per row: x += y * rstd(y) * w (* s); rounded (when given) receives the new x in the run's dtype.  VEC: the
// width is a multiple of 4 and every pointer of 16 bytes: a thread takes four columns at a time.  normed (when given)
// receives the RMS norm of the new x times next_w: what the next branch reads when it norms the residual first; a
// thread then reads back the columns it wrote itself.
template <class T, bool VEC>
__global__ void branch_norm_add_kernel(float* __restrict__ x, const T* __restrict__ y, const float* __restrict__ w,
                                       const float* __restrict__ s, T* __restrict__ rounded, int width, float eps,
                                       const float* __restrict__ next_w, float next_eps, T* __restrict__ normed) {
    __shared__ float red[33];
    float ss2 = 0.f;
    pdl_wait();
    const long long base = (long long)blockIdx.x * width;
    float ss = 0.f;
    if (VEC) {
        for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
            const float4 v = read_four(y + base + c);
            ss = fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, fmaf(v.x, v.x, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            const float v = to_f<T>(y[base + c]);
            ss = fmaf(v, v, ss);
        }
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)width + eps);
    pdl_launch_dependents();
    if (VEC) {
        for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
            const float4 v = read_four(y + base + c), g = read_four(w + c), old = read_four(x + base + c);
            float4 n = make_float4(__fmul_rn(__fmul_rn(v.x, rstd), g.x), __fmul_rn(__fmul_rn(v.y, rstd), g.y),
                                   __fmul_rn(__fmul_rn(v.z, rstd), g.z), __fmul_rn(__fmul_rn(v.w, rstd), g.w));
            if (s != nullptr) {
                const float4 ls = read_four(s + c);
                n = make_float4(__fmul_rn(n.x, ls.x), __fmul_rn(n.y, ls.y), __fmul_rn(n.z, ls.z), __fmul_rn(n.w, ls.w));
            }
            const float4 sum = make_float4(old.x + n.x, old.y + n.y, old.z + n.z, old.w + n.w);
            write_four(x + base + c, sum);
            if (rounded != nullptr) write_four(rounded + base + c, sum);
            ss2 = fmaf(sum.w, sum.w, fmaf(sum.z, sum.z, fmaf(sum.y, sum.y, fmaf(sum.x, sum.x, ss2))));
        }
        if (normed == nullptr) return;
        const float rstd2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)width + next_eps);
        for (int c = 4 * threadIdx.x; c < width; c += 4 * blockDim.x) {
            const float4 v = read_four(x + base + c), g = read_four(next_w + c);
            write_four(normed + base + c, make_float4(v.x * rstd2 * g.x, v.y * rstd2 * g.y, v.z * rstd2 * g.z, v.w * rstd2 * g.w));
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float n = __fmul_rn(__fmul_rn(to_f<T>(y[base + c]), rstd), w[c]);
        if (s != nullptr) n = __fmul_rn(n, s[c]);
        const float v = x[base + c] + n;
        x[base + c] = v;
        if (rounded != nullptr) rounded[base + c] = from_f<T>(v);
        ss2 = fmaf(v, v, ss2);
    }
    if (normed == nullptr) return;
    const float rstd2 = 1.0f / sqrtf(block_sum(ss2, red) / (float)width + next_eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) normed[base + c] = from_f<T>(x[base + c] * rstd2 * next_w[c]);
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
    // few rows (decoding): a row's columns go to several blocks, so that no thread walks a chain of dependent reads
    const int shares = batch.n_rows < 64 ? (width + threads - 1) / threads : 1;
    if (out_dtype == SB_F32)
        sb_launch(causal_conv_kernel<float>, dim3(batch.n_rows, shares), threads, 0, stream, x, weight, (const float*)state, state_slot,
                  batch, width, taps, (float*)out);
    else
        sb_launch(causal_conv_kernel<__nv_bfloat16>, dim3(batch.n_rows, shares), threads, 0, stream, x, weight, (const float*)state,
                  state_slot, batch, width, taps, (__nv_bfloat16*)out);
    if (weight != nullptr && taps > 1)
        sb_launch(causal_conv_state_kernel, dim3(batch.n_seqs, batch.n_seqs < 64 ? (width + threads - 1) / threads : 1), threads, 0,
                  stream, x, state, state_slot, batch, width, taps);
    SB_LAUNCH_CHECK();
}

int sb_branch_norm_add(int dtype, float* x, const void* y, const float* w, const float* s, void* rounded, int rows, int width, float eps,
                       const float* next_w, float next_eps, void* normed, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if ((next_w == nullptr) != (normed == nullptr)) return (int)cudaErrorInvalidValue;
    auto aligned = [](const void* ptr) { return ptr == nullptr || (reinterpret_cast<size_t>(ptr) & 15) == 0; };
    const bool vec = width % 4 == 0 && aligned(x) && aligned(y) && aligned(w) && aligned(s) && aligned(rounded) && aligned(next_w)
                     && aligned(normed);
    const int cols = vec ? width / 4 : width;
    const int threads = cols >= 2048 ? 512 : (cols >= 192 ? 256 : (cols >= 96 ? 128 : 64));
#define SB_BRANCH(T, V) \
    sb_launch(branch_norm_add_kernel<T, V>, rows, threads, 0, stream, x, (const T*)y, w, s, (T*)rounded, width, eps, next_w, next_eps, \
              (T*)normed)
    if (dtype == SB_F32) {
        if (vec) SB_BRANCH(float, true);
        else SB_BRANCH(float, false);
    } else {
        if (vec) SB_BRANCH(__nv_bfloat16, true);
        else SB_BRANCH(__nv_bfloat16, false);
    }
#undef SB_BRANCH
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
