// Attention whose scores meet across heads before the softmax, over a paged cache, and the kernel that fills that cache.
//
//   s_g(i, j) = cap * tanh(q_g(i) . k_c(g)(j) * scale / cap)                  (cap 0: no cap)
//   t_h(i, j) = sum_g T[h, g] s_g(i, j)                                       (T null: t = s)
//   visible:    j <= i and (i - j < window or j < keep_first)                 (window 0: every earlier key)
//   weights:    exp(t_h) / (sum over visible j of exp(t_h) + exp(sink_h))     (sink null: no extra term)
//
// A row's scores of ALL heads against a key are needed before any head's softmax can go on, so a block owns a query
// position with all its heads.  Scores, the cap, the table, the running maximum, the exponentials, the weights and the
// sums over values are 32-bit in every run.  Keys are walked in the order of their positions, the kept first ones
// first and then the window, 32 at a time from the start of either range: a row's result depends on its position and
// its keys only, not on the step that brought it or on its neighbours in the batch.
//
// This file holds the general kernel (any sizes, both dtypes) and the fill kernel; attention_talk_mma.cu holds the
// tensor-core kernel.
#include "attention_flex.cuh"

template <class T> __device__ __forceinline__ float talk_dot(const float* qs, const T* kr, int D);
template <> __device__ __forceinline__ float talk_dot<float>(const float* qs, const float* kr, int D) {
    float dot = 0.f;
    if ((D & 3) == 0) {
        for (int d = 0; d < D; d += 4) {
            const float4 v = *reinterpret_cast<const float4*>(kr + d);
            dot = fmaf(qs[d], v.x, dot);
            dot = fmaf(qs[d + 1], v.y, dot);
            dot = fmaf(qs[d + 2], v.z, dot);
            dot = fmaf(qs[d + 3], v.w, dot);
        }
    } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], kr[d], dot);
    }
    return dot;
}
template <> __device__ __forceinline__ float talk_dot<__nv_bfloat16>(const float* qs, const __nv_bfloat16* kr, int D) {
    float dot = 0.f;
    if ((D & 7) == 0) {
        for (int d = 0; d < D; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                dot = fmaf(qs[d + 2 * e], f.x, dot);
                dot = fmaf(qs[d + 2 * e + 1], f.y, dot);
            }
        }
    } else {
        for (int d = 0; d < D; ++d) dot = fmaf(qs[d], __bfloat162float(kr[d]), dot);
    }
    return dot;
}

// One block per row.  Shared memory: the row's queries as floats [H * D], the table [H * H], raw and mixed scores of a
// turn's 32 keys [H][32] each, the turn's key rows per key/value head [G][32], per head the running maximum and sum,
// and the heads' value sums [H * V].  A warp takes heads warp, warp + warps, ...
//
// With n_splits > 1 (decoding: few rows, many keys) blockIdx.y takes a share of the row's turns and leaves, per head, its
// unnormalised value sums, maximum and sum in ``partial`` [row][head][split][V + 2]; talking_merge_kernel divides.
template <class T>
__global__ void talking_attention_general_kernel(SbFlex p, SbBatch batch, T* __restrict__ out, int n_splits, float* __restrict__ partial) {
    extern __shared__ __align__(16) unsigned char talk_sm[];
    const int H = p.n_heads, G = p.n_kv_heads, D = p.k_dim, V = p.v_dim, per_kv = H / G;
    long long* tok_s = reinterpret_cast<long long*>(talk_sm);            // [G][32]
    float* qs = reinterpret_cast<float*>(tok_s + (size_t)G * 32);          // [H * D]
    float* tb = qs + (size_t)H * D;                                        // [H * H]
    float* raw = tb + (size_t)H * H;                                       // [H][32]
    float* wgt = raw + (size_t)H * 32;                                     // [H][32]
    float* run_m = wgt + (size_t)H * 32;                                   // [H]
    float* run_l = run_m + H;                                              // [H]
    float* acc = run_l + H;                                                // [H * V]
    pdl_wait();
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const T* qr = (const T*)p.q + (long long)row * p.q_row;
    for (int e = threadIdx.x; e < H * D; e += blockDim.x) qs[e] = to_f<T>(qr[(long long)(e / D) * p.q_head + e % D]);
    if (p.talk != nullptr)
        for (int e = threadIdx.x; e < H * H; e += blockDim.x) tb[e] = p.talk[e];
    for (int e = threadIdx.x; e < H * V; e += blockDim.x) acc[e] = 0.f;
    for (int e = threadIdx.x; e < H; e += blockDim.x) {
        run_m[e] = -INFINITY;
        run_l[e] = 0.f;
    }
    __syncthreads();
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int kept_end = min(p.keep_first, lo);       // kept first keys that the window does not hold anyway
    const T* kbase = (const T*)p.k;
    const T* vbase = (const T*)p.v;
    const int kept_turns = (kept_end + 31) / 32, turns = kept_turns + (pos + 1 - lo + 31) / 32;
    const int per_split = (turns + n_splits - 1) / n_splits;
    const int turn_lo = blockIdx.y * per_split, turn_hi = min(turns, turn_lo + per_split);
    {
        for (int turn = turn_lo; turn < turn_hi; ++turn) {
            const int n0 = turn < kept_turns ? turn * 32 : lo + (turn - kept_turns) * 32, end = turn < kept_turns ? kept_end : pos + 1;
            const int n = n0 + lane;
            const bool seen = n < end;
            for (int c = warp; c < G; c += n_warps) tok_s[c * 32 + lane] = seen ? flex_token(p, slot, n, c) : -1;
            __syncthreads();
            for (int g = warp; g < H; g += n_warps) {
                const long long tok = tok_s[(g / per_kv) * 32 + lane];
                float s = 0.f;
                if (tok >= 0) {
                    s = talk_dot<T>(qs + (size_t)g * D, kbase + tok * D, D) * p.scale;
                    if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
                }
                raw[g * 32 + lane] = s;
            }
            __syncthreads();
            for (int h = warp; h < H; h += n_warps) {
                const long long tok = tok_s[(h / per_kv) * 32 + lane];
                float t;
                if (p.talk != nullptr) {
                    t = 0.f;
                    for (int g = 0; g < H; ++g) t = fmaf(tb[h * H + g], raw[g * 32 + lane], t);
                } else {
                    t = raw[h * 32 + lane];
                }
                if (tok < 0) t = -INFINITY;
                const float m_old = run_m[h];
                const float m_new = fmaxf(m_old, warp_max(t));
                if (m_new == -INFINITY) continue;     // nothing visible in this turn (a key without a page)
                const float w = tok >= 0 ? expf(t - m_new) : 0.f;
                const float alpha = expf(m_old - m_new);
                const float sum = warp_sum(w);
                wgt[h * 32 + lane] = w;
                __syncwarp();
                if (lane == 0) {
                    run_m[h] = m_new;
                    run_l[h] = run_l[h] * alpha + sum;
                }
                const long long* toks = tok_s + (h / per_kv) * 32;
                for (int d = lane; d < V; d += 32) {
                    float a = acc[h * V + d] * alpha;
                    for (int t2 = 0; t2 < 32; ++t2) {
                        const long long kt = toks[t2];
                        if (kt >= 0) a = fmaf(wgt[h * 32 + t2], to_f<T>(vbase[flex_value_token(p, kt, h / per_kv) * p.v_row + d]), a);
                    }
                    acc[h * V + d] = a;
                }
                __syncwarp();
            }
            __syncthreads();
        }
    }
    if (n_splits > 1) {
        for (int h = warp; h < H; h += n_warps) {
            float* dst = partial + (((long long)row * H + h) * n_splits + blockIdx.y) * (V + 2);
            for (int d = lane; d < V; d += 32) dst[d] = acc[h * V + d];
            if (lane == 0) {
                dst[V] = run_m[h];
                dst[V + 1] = run_l[h];
            }
        }
        return;
    }
    for (int h = warp; h < H; h += n_warps) {
        float m = run_m[h], l = run_l[h], alpha = 1.f;
        if (p.sink != nullptr) {   // one more term in the denominator, no value behind it
            const float sk = p.sink[h];
            const float m_new = fmaxf(m, sk);
            alpha = expf(m - m_new);
            l = l * alpha + expf(sk - m_new);
        }
        const float inv = alpha / l;
        T* orow = out + ((long long)row * H + h) * V;
        for (int d = lane; d < V; d += 32) orow[d] = from_f<T>(acc[h * V + d] * inv);
    }
}

// One block per (row, head): the splits' sums, scaled to their common maximum (the sink's too), added and divided.
template <class T>
__global__ void talking_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, const float* __restrict__ sink, int n_heads,
                                     int n_splits, int V) {
    pdl_wait();
    const long long rh = (long long)blockIdx.x * n_heads + blockIdx.y;
    const float* base = partial + rh * n_splits * (V + 2);
    float m = sink != nullptr ? sink[blockIdx.y] : -INFINITY;
    for (int sidx = 0; sidx < n_splits; ++sidx) m = fmaxf(m, base[(long long)sidx * (V + 2) + V]);
    float l = sink != nullptr ? expf(sink[blockIdx.y] - m) : 0.f;
    for (int sidx = 0; sidx < n_splits; ++sidx) {
        const float ms = base[(long long)sidx * (V + 2) + V];
        if (ms != -INFINITY) l += base[(long long)sidx * (V + 2) + V + 1] * expf(ms - m);
    }
    for (int c = threadIdx.x; c < V; c += blockDim.x) {
        float o = 0.f;
        for (int sidx = 0; sidx < n_splits; ++sidx) {
            const float ms = base[(long long)sidx * (V + 2) + V];
            if (ms != -INFINITY) o = fmaf(base[(long long)sidx * (V + 2) + c], expf(ms - m), o);
        }
        out[rh * V + c] = from_f<T>(o / l);
    }
}

// One block per row of qkv = [q (H * D) | k (G * D) | v (G * V)]: with norm weights the whole query part is divided by
// its root mean square and multiplied by q_norm, the whole key part likewise with k_norm (32-bit, rounded once); the
// queries go to q_out, keys and values to the row's place in the cache.
template <class T>
__global__ void qk_norm_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, SbBatch batch, SbFlex p, int n_heads,
                                     const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, int* status) {
    __shared__ float red[33];
    pdl_wait();
    const int row = blockIdx.x;
    const int nq = n_heads * p.k_dim, nk = p.n_kv_heads * p.k_dim, nv = p.n_kv_heads * p.v_dim;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const T* r = qkv + (long long)row * (nq + nk + nv);
    float q_rstd = 1.f, k_rstd = 1.f;
    if (q_norm != nullptr) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nq; c += blockDim.x) {
            const float x = to_f<T>(r[c]);
            ss = fmaf(x, x, ss);
        }
        q_rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + eps);
    }
    if (k_norm != nullptr) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < nk; c += blockDim.x) {
            const float x = to_f<T>(r[nq + c]);
            ss = fmaf(x, x, ss);
        }
        k_rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + eps);
    }
    for (int c = threadIdx.x; c < nq; c += blockDim.x) {
        const float x = to_f<T>(r[c]);
        q_out[(long long)row * nq + c] = q_norm != nullptr ? from_f<T>(__fmul_rn(__fmul_rn(x, q_rstd), q_norm[c])) : r[c];
    }
    const long long tok0 = flex_token(p, slot, pos, 0);
    if (tok0 < 0) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_NO_PAGE);
        return;
    }
    for (int c = threadIdx.x; c < nk; c += blockDim.x) {
        const int g = c / p.k_dim, d = c % p.k_dim;
        const float x = to_f<T>(r[nq + c]);
        ((T*)p.k)[(tok0 + (long long)g * SB_PAGE) * p.k_dim + d] =
            k_norm != nullptr ? from_f<T>(__fmul_rn(__fmul_rn(x, k_rstd), k_norm[c])) : r[nq + c];
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        const int g = c / p.v_dim, d = c % p.v_dim;
        ((T*)p.v)[(tok0 + (long long)g * SB_PAGE) * p.v_row + d] = r[nq + nk + c];
    }
}

void sb_talking_merge_bf16(const float* partial, void* out, const float* sink, int n_rows, int n_heads, int n_splits, int v_dim,
                           cudaStream_t stream) {
    sb_launch(talking_merge_kernel<__nv_bfloat16>, dim3(n_rows, n_heads), 64, 0, stream, partial, (__nv_bfloat16*)out, sink, n_heads,
              n_splits, v_dim);
}

extern "C" {

// Bytes of shared memory the general kernel asks for.
long long sb_talking_attention_general_smem(int n_heads, int n_kv_heads, int k_dim, int v_dim) {
    return (long long)n_kv_heads * 32 * sizeof(long long)
           + ((long long)n_heads * k_dim + (long long)n_heads * n_heads + 2ll * n_heads * 32 + 2ll * n_heads + (long long)n_heads * v_dim)
                 * sizeof(float);
}

int sb_talking_attention_general(int dtype, SbFlex p, SbBatch batch, void* out, int n_splits, float* partial, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (n_splits < 1 || n_splits > 65535 || (n_splits > 1 && partial == nullptr)) return (int)cudaErrorInvalidValue;
    if (p.n_heads < 1 || p.n_kv_heads < 1 || p.n_heads % p.n_kv_heads || (p.v_heads > 0 && p.v_heads != p.n_kv_heads))
        return (int)cudaErrorInvalidValue;
    const long long smem = sb_talking_attention_general_smem(p.n_heads, p.n_kv_heads, p.k_dim, p.v_dim);
    if (smem > 227 * 1024) return (int)cudaErrorInvalidValue;
    const int warps = p.n_heads < 8 ? p.n_heads : 8;
#define SB_TALK(T)                                                                                                                 \
    do {                                                                                                                           \
        if (smem > 48 * 1024) {                                                                                                    \
            const cudaError_t err =                                                                                                \
                cudaFuncSetAttribute(talking_attention_general_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (err != cudaSuccess) return (int)err;                                                                               \
        }                                                                                                                          \
        sb_launch(talking_attention_general_kernel<T>, dim3(batch.n_rows, n_splits), 32 * warps, (size_t)smem, stream, p, batch,  \
                  (T*)out, n_splits, partial);                                                                                     \
        if (n_splits > 1)                                                                                                          \
            sb_launch(talking_merge_kernel<T>, dim3(batch.n_rows, p.n_heads), 64, 0, stream, (const float*)partial, (T*)out,       \
                      p.sink, p.n_heads, n_splits, p.v_dim);                                                                       \
    } while (0)
    if (dtype == SB_F32) SB_TALK(float);
    else SB_TALK(__nv_bfloat16);
#undef SB_TALK
    SB_LAUNCH_CHECK();
}

int sb_qk_norm_store(int dtype, const void* qkv, void* q_out, SbBatch batch, SbFlex p, int n_heads, const float* q_norm,
                     const float* k_norm, float eps, int* status, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (p.v_heads > 0 && p.v_heads != p.n_kv_heads) return (int)cudaErrorInvalidValue;
    const int threads = n_heads * p.k_dim >= 2048 ? 256 : 128;
    if (dtype == SB_F32)
        sb_launch(qk_norm_store_kernel<float>, batch.n_rows, threads, 0, stream, (const float*)qkv, (float*)q_out, batch, p, n_heads,
                  q_norm, k_norm, eps, status);
    else
        sb_launch(qk_norm_store_kernel<__nv_bfloat16>, batch.n_rows, threads, 0, stream, (const __nv_bfloat16*)qkv,
                  (__nv_bfloat16*)q_out, batch, p, n_heads, q_norm, k_norm, eps, status);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
