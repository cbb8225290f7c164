// What an attention whose queries and keys pass a short convolution over time needs beside the attention kernels:
//
//   conv_qk_store   u = projection + bias; y_t = sum_j w[:, j] * u_(t - taps + 1 + j) per channel (zeros before the
//                   sequence's start; inputs before the step from the sequence's record); per head the RMS norm of y
//                   with a weight of the head's size (none without weights); queries times
//                   1 + coef * ln(floor((pos + 1) / every) + 1).
//                   The normed keys go to the key rows of the cache, the keys as they leave the convolution (before
//                   the norm) to its value rows: the values of this attention are its keys.
//   head_gate       out = a * sigmoid(z[:, head]) * scale: one gate per head and row.
//
// Bias, convolution, norm, temperature and the gate are 32-bit in every run; the record holds 32-bit numbers.
#include "attention_flex.cuh"

// Input `src` (an index among the step's rows of the sequence; negative: before the step) of channel c of a part.
template <class T>
__device__ __forceinline__ float conv_input(const T* x, long long ld, int first, int src, int c, float bias, const float* rec, int keep,
                                            int rec_width, int rec_c) {
    if (src >= 0) return to_f<T>(x[(long long)(first + src) * ld + c]) + bias;
    return rec[(long long)(keep + src) * rec_width + rec_c];
}

// A block per row; blockIdx.y shares out the row's heads (H query heads, then G key heads).  q [rows, H * D] and
// k [rows, G * D] are views of wider rows.  The record of a sequence is [taps - 1][H * D + G * D] floats.
template <class T>
__global__ void conv_qk_store_kernel(const T* __restrict__ q, long long q_ld, const T* __restrict__ k, long long k_ld,
                                     const float* __restrict__ q_bias, const float* __restrict__ k_bias,
                                     const float* __restrict__ q_conv, const float* __restrict__ k_conv, int taps,
                                     const float* __restrict__ state, long long state_slot, const float* __restrict__ q_norm,
                                     const float* __restrict__ k_norm, float eps, float temp_coef, int temp_every,
                                     T* __restrict__ q_out, SbBatch batch, SbFlex p, int H, int* status) {
    extern __shared__ float ys[];   // [D]
    __shared__ float red[33];
    pdl_wait();
    const int row = blockIdx.x, D = p.k_dim, G = p.n_kv_heads;
    const int s = batch.row_seq[row], slot = batch.seq_slot[s], first = batch.cu_q[s];
    const int t = row - first, pos = batch.lengths[slot] + t;
    const int keep = taps - 1, rec_width = (H + G) * D;
    const float* rec = state != nullptr ? state + (long long)slot * state_slot : nullptr;
    float temp = 1.0f;
    if (temp_every > 0) temp = 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
    for (int u = blockIdx.y; u < H + G; u += gridDim.y) {
        const bool is_q = u < H;
        const int h = is_q ? u : u - H;
        const T* x = is_q ? q : k;
        const long long ld = is_q ? q_ld : k_ld;
        const float* bias = is_q ? q_bias : k_bias;
        const float* conv = is_q ? q_conv : k_conv;
        float ss = 0.f;
        __syncthreads();
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            const int ch = h * D + c;
            const float b = bias != nullptr ? bias[ch] : 0.f;
            float y;
            if (conv == nullptr) {
                y = to_f<T>(x[(long long)row * ld + ch]) + b;
            } else {
                y = 0.f;
                for (int j = 0; j < taps; ++j)
                    y = fmaf(conv[(long long)ch * taps + j],
                             conv_input<T>(x, ld, first, t - keep + j, ch, b, rec, keep, rec_width, (is_q ? 0 : H * D) + ch), y);
            }
            ys[c] = y;
            ss = fmaf(y, y, ss);
        }
        ss = block_sum(ss, red);
        const bool normed = q_norm != nullptr;      // without norm weights queries and keys pass as they are
        const float rstd = normed ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
        if (is_q) {
            T* dst = q_out + ((long long)row * H + h) * D;
            for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = from_f<T>(ys[c] * rstd * (normed ? q_norm[c] : 1.0f) * temp);
        } else {
            const long long tok = flex_token(p, slot, pos, h);
            if (tok < 0) {
                if (threadIdx.x == 0) atomicOr(status, SB_STATUS_NO_PAGE);
                continue;
            }
            T* kd = (T*)p.k + tok * D;
            T* vd = (T*)p.v + flex_value_token(p, tok, h) * p.v_row;
            for (int c = threadIdx.x; c < D; c += blockDim.x) {
                kd[c] = from_f<T>(ys[c] * rstd * (normed ? k_norm[c] : 1.0f));
                vd[c] = from_f<T>(ys[c]);
            }
        }
    }
}

// After the kernel above: a sequence's record becomes its last taps - 1 biased projections.  A step of fewer rows
// than that keeps the later entries of the old record: a thread reads its channel's entries before it writes them.
template <class T>
__global__ void conv_qk_state_kernel(const T* __restrict__ q, long long q_ld, const T* __restrict__ k, long long k_ld,
                                     const float* __restrict__ q_bias, const float* __restrict__ k_bias, int taps,
                                     float* __restrict__ state, long long state_slot, SbBatch batch, int q_width, int k_width) {
    pdl_wait();
    const int s = blockIdx.x;
    const int first = batch.cu_q[s], n = batch.cu_q[s + 1] - first, keep = taps - 1, width = q_width + k_width;
    float* rec = state + (long long)batch.seq_slot[s] * state_slot;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        const bool is_q = c < q_width;
        const int ch = is_q ? c : c - q_width;
        const T* x = is_q ? q : k;
        const long long ld = is_q ? q_ld : k_ld;
        const float* bias = is_q ? q_bias : k_bias;
        const float b = bias != nullptr ? bias[ch] : 0.f;
        for (int e = 0; e < keep; ++e) {
            const int src = n - keep + e;
            rec[(long long)e * width + c] = src >= 0 ? to_f<T>(x[(long long)(first + src) * ld + ch]) + b : rec[(long long)(e + n) * width + c];
        }
    }
}

template <class T>
__global__ void head_gate_kernel(const T* __restrict__ a, const float* __restrict__ z, long long z_ld, int z_col, T* __restrict__ out,
                                 long long out_ld, long long rows, int H, int V, float scale) {
    pdl_wait();
    const long long n = rows * H * V;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / ((long long)H * V);
        const int c = (int)(i - row * H * V), h = c / V;
        const float gate = 1.0f / (1.0f + expf(-z[row * z_ld + z_col + h]));
        out[row * out_ld + c] = from_f<T>(to_f<T>(a[i]) * gate * scale);
    }
}

extern "C" {

int sb_conv_qk_store(int dtype, const void* q, long long q_ld, const void* k, long long k_ld, const float* q_bias, const float* k_bias,
                     const float* q_conv, const float* k_conv, int taps, float* state, long long state_slot, const float* q_norm,
                     const float* k_norm, float eps, float temp_coef, int temp_every, void* q_out, SbBatch batch, SbFlex p, int H,
                     int* status, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    const bool conv = q_conv != nullptr;
    if ((q_conv == nullptr) != (k_conv == nullptr) || (q_norm == nullptr) != (k_norm == nullptr)
        || (conv && (taps < 1 || (taps > 1 && state == nullptr))) || p.v == nullptr
        || p.v_dim != p.k_dim)
        return (int)cudaErrorInvalidValue;
    const int D = p.k_dim, units = H + p.n_kv_heads;
    const int threads = D >= 256 ? 256 : (D >= 96 ? 128 : 64);
    const int per_row = batch.n_rows >= 1024 ? min(units, 4) : (batch.n_rows >= 128 ? min(units, 8) : min(units, 64));
    dim3 grid(batch.n_rows, per_row);
    const size_t smem = (size_t)D * sizeof(float);
    typedef __nv_bfloat16 bf;
    if (dtype == SB_F32)
        sb_launch(conv_qk_store_kernel<float>, grid, threads, smem, stream, (const float*)q, q_ld, (const float*)k, k_ld, q_bias, k_bias,
                  q_conv, k_conv, taps, (const float*)state, state_slot, q_norm, k_norm, eps, temp_coef, temp_every, (float*)q_out, batch,
                  p, H, status);
    else
        sb_launch(conv_qk_store_kernel<bf>, grid, threads, smem, stream, (const bf*)q, q_ld, (const bf*)k, k_ld, q_bias, k_bias, q_conv,
                  k_conv, taps, (const float*)state, state_slot, q_norm, k_norm, eps, temp_coef, temp_every, (bf*)q_out, batch, p, H,
                  status);
    if (conv && taps > 1) {
        const int width = units * D;
        dim3 sgrid(batch.n_seqs, batch.n_seqs < 64 ? (width + 127) / 128 : 1);
        if (dtype == SB_F32)
            sb_launch(conv_qk_state_kernel<float>, sgrid, 128, 0, stream, (const float*)q, q_ld, (const float*)k, k_ld, q_bias, k_bias,
                      taps, state, state_slot, batch, H * D, p.n_kv_heads * D);
        else
            sb_launch(conv_qk_state_kernel<bf>, sgrid, 128, 0, stream, (const bf*)q, q_ld, (const bf*)k, k_ld, q_bias, k_bias, taps, state,
                      state_slot, batch, H * D, p.n_kv_heads * D);
    }
    SB_LAUNCH_CHECK();
}

int sb_head_gate(int dtype, const void* a, const float* z, long long z_ld, int z_col, void* out, long long out_ld, int rows, int H, int V,
                 float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long n = (long long)rows * H * V;
    const int blocks = (int)((n + 255) / 256 < 8192 ? (n + 255) / 256 : 8192);
    if (dtype == SB_F32)
        sb_launch(head_gate_kernel<float>, blocks, 256, 0, stream, (const float*)a, z, z_ld, z_col, (float*)out, out_ld, (long long)rows,
                  H, V, scale);
    else
        sb_launch(head_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)a, z, z_ld, z_col, (__nv_bfloat16*)out,
                  out_ld, (long long)rows, H, V, scale);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
