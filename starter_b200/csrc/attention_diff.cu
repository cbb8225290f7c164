// What the attention with two score maps per head needs beside the attention kernels themselves: the rotation of
// queries and keys with the cache write, and the join of a head's two maps.
//
// Rotation ("rotate half"): of a head's first `rot` columns, column i turns with column i + rot / 2 by the angle
// position * freqs[i]; angle, sine and cosine are 32-bit, and both are multiplied by `mag`.  Later columns pass.
//
// Join: with a1, a2 the two maps' results of one head, o = a1 - lam * a2, then o / sqrt(mean(o^2) + eps) * post, and with
// a gate (pre-activations [rows, H * V], a view of wider rows) times sigmoid(gate), element by element.
#include "attention_flex.cuh"

template <class T>
__device__ __forceinline__ float turned(const T* src, int c, int rot, const float* cs, const float* sn) {
    const int half = rot >> 1;
    if (c < half) return to_f<T>(src[c]) * cs[c] - to_f<T>(src[c + half]) * sn[c];
    if (c < rot) return to_f<T>(src[c]) * cs[c - half] + to_f<T>(src[c - half]) * sn[c - half];
    return to_f<T>(src[c]);
}

// gridDim.y blocks per row share the row's heads out.  q [rows, nq heads, D] and k [rows, n_kv_heads, D] are views of
// wider rows (row strides in elements, heads side by side); v [rows, v_heads * v_dim] likewise.  The turned queries go
// to q_out (contiguous), the turned keys and the values to the row's place in the cache.
template <class T>
__global__ void rotate_half_store_kernel(const T* __restrict__ q, long long q_row, const T* __restrict__ k, long long k_row,
                                         const T* __restrict__ v, long long v_row, T* __restrict__ q_out, SbBatch batch, SbFlex p,
                                         const float* __restrict__ freqs, int rot, float mag, int nq, int* status) {
    extern __shared__ float trig[];
    pdl_wait();
    const int row = blockIdx.x, D = p.k_dim, half = rot >> 1;
    int slot, pos;
    row_place(batch, row, slot, pos);
    float* cs = trig;
    float* sn = trig + half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * freqs[i], &s, &c);
        cs[i] = c * mag;
        sn[i] = s * mag;
    }
    __syncthreads();
    // units of work: a query head, a key head, a value head; the blocks of a row share them out
    const int vh = p.v_heads > 0 ? p.v_heads : p.n_kv_heads, per = p.n_kv_heads / vh;
    const int units = nq + p.n_kv_heads + vh;
    for (int u = blockIdx.y; u < units; u += gridDim.y) {
        if (u < nq) {
            const T* src = q + row * q_row + (long long)u * D;
            T* dst = q_out + ((long long)row * nq + u) * D;
            for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = from_f<T>(turned<T>(src, c, rot, cs, sn));
        } else if (u < nq + p.n_kv_heads) {
            const int h = u - nq;
            const long long tok = flex_token(p, slot, pos, h);
            if (tok < 0) {
                if (threadIdx.x == 0) atomicOr(status, SB_STATUS_NO_PAGE);
                continue;
            }
            const T* src = k + row * k_row + (long long)h * D;
            T* dst = (T*)p.k + tok * D;
            for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = from_f<T>(turned<T>(src, c, rot, cs, sn));
        } else {
            const int h = u - nq - p.n_kv_heads;
            const long long tok = flex_value_token(p, flex_token(p, slot, pos, h * per), h * per);
            if (tok < 0) continue;
            const T* src = v + row * v_row + (long long)h * p.v_dim;
            T* dst = (T*)p.v + tok * p.v_row;
            for (int c = threadIdx.x; c < p.v_dim; c += blockDim.x) dst[c] = src[c];
        }
    }
}

// One warp per (row, head).  a [rows, 2 H, V] holds the maps in the order (key/value head, map, head of the group).
template <class T>
__global__ void diff_combine_kernel(const T* __restrict__ a, T* __restrict__ out, int rows, int H, int G, int V, float lam, float eps,
                                    float post, const T* __restrict__ gate, long long gate_ld) {
    pdl_wait();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)rows * H) return;
    const long long row = wid / H;
    const int h = (int)(wid % H), per = H / G, g = h / per, r = h % per;
    const T* a1 = a + ((row * 2 * H) + (long long)(2 * g) * per + r) * V;
    const T* a2 = a + ((row * 2 * H) + (long long)(2 * g + 1) * per + r) * V;
    float ss = 0.f;
    for (int c = lane; c < V; c += 32) {
        const float o = fmaf(-lam, to_f<T>(a2[c]), to_f<T>(a1[c]));
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float mul = post / sqrtf(ss / (float)V + eps);
    T* o_row = out + (row * H + h) * V;
    if (gate == nullptr) {
        for (int c = lane; c < V; c += 32) o_row[c] = from_f<T>(fmaf(-lam, to_f<T>(a2[c]), to_f<T>(a1[c])) * mul);
        return;
    }
    const T* g_row = gate + row * gate_ld + (long long)h * V;
    for (int c = lane; c < V; c += 32)
        o_row[c] = from_f<T>(fmaf(-lam, to_f<T>(a2[c]), to_f<T>(a1[c])) * mul / (1.0f + expf(-to_f<T>(g_row[c]))));
}

extern "C" {

int sb_rotate_half_store(int dtype, const void* q, long long q_row, const void* k, long long k_row, const void* v, long long v_row,
                         void* q_out, SbBatch batch, SbFlex p, const float* freqs, int rot, float mag, int nq, int* status,
                         cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > p.k_dim || (rot > 0 && freqs == nullptr)) return (int)cudaErrorInvalidValue;
    const int threads = p.k_dim >= 128 || p.v_dim >= 128 ? 128 : 64;
    const int vh = p.v_heads > 0 ? p.v_heads : p.n_kv_heads, units = nq + p.n_kv_heads + vh;
    // few rows: a block per head, so that a decode step's rows are spread over the SMs; many rows: a few blocks per row
    const int per_row = batch.n_rows >= 1024 ? min(units, 4) : (batch.n_rows >= 128 ? min(units, 8) : min(units, 64));
    dim3 grid(batch.n_rows, per_row);
    const size_t smem = (size_t)rot * sizeof(float);
    if (dtype == SB_F32)
        sb_launch(rotate_half_store_kernel<float>, grid, threads, smem, stream, (const float*)q, q_row, (const float*)k, k_row,
                  (const float*)v, v_row, (float*)q_out, batch, p, freqs, rot, mag, nq, status);
    else
        sb_launch(rotate_half_store_kernel<__nv_bfloat16>, grid, threads, smem, stream, (const __nv_bfloat16*)q, q_row,
                  (const __nv_bfloat16*)k, k_row, (const __nv_bfloat16*)v, v_row, (__nv_bfloat16*)q_out, batch, p, freqs, rot, mag, nq,
                  status);
    SB_LAUNCH_CHECK();
}

int sb_diff_combine(int dtype, const void* a, void* out, int rows, int H, int G, int V, float lam, float eps, float post,
                    const void* gate, long long gate_ld, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H < 1 || G < 1 || H % G) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)rows * H;
    const int threads = 128;
    const unsigned int blocks = (unsigned int)((warps * 32 + threads - 1) / threads);
    if (dtype == SB_F32)
        sb_launch(diff_combine_kernel<float>, blocks, threads, 0, stream, (const float*)a, (float*)out, rows, H, G, V, lam, eps, post,
                  (const float*)gate, gate_ld);
    else
        sb_launch(diff_combine_kernel<__nv_bfloat16>, blocks, threads, 0, stream, (const __nv_bfloat16*)a, (__nv_bfloat16*)out, rows, H,
                  G, V, lam, eps, post, (const __nv_bfloat16*)gate, gate_ld);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
