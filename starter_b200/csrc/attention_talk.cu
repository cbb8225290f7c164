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

// The dots of up to four query heads (their rows D apart in qs) with one key row, which is read once; every head's
// sum runs over the columns in rising order.
template <class T> __device__ __forceinline__ void talk_dots(const float* qs, int D, int n_heads, const T* kr, float dot[4]);
template <> __device__ __forceinline__ void talk_dots<float>(const float* qs, int D, int n_heads, const float* kr, float dot[4]) {
    if ((D & 3) == 0) {
#pragma unroll 8
        for (int d = 0; d < D; d += 4) {
            const float4 v = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < n_heads) {
                    const float4 q = *reinterpret_cast<const float4*>(qs + (size_t)j * D + d);
                    dot[j] = fmaf(q.w, v.w, fmaf(q.z, v.z, fmaf(q.y, v.y, fmaf(q.x, v.x, dot[j]))));
                }
        }
    } else {
        for (int d = 0; d < D; ++d) {
            const float v = kr[d];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < n_heads) dot[j] = fmaf(qs[(size_t)j * D + d], v, dot[j]);
        }
    }
}
template <>
__device__ __forceinline__ void talk_dots<__nv_bfloat16>(const float* qs, int D, int n_heads, const __nv_bfloat16* kr, float dot[4]) {
    if ((D & 7) == 0) {
#pragma unroll 8
        for (int d = 0; d < D; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float f[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 two = __bfloat1622float2(h[e]);
                f[2 * e] = two.x, f[2 * e + 1] = two.y;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < n_heads) {
                    const float4 qa = *reinterpret_cast<const float4*>(qs + (size_t)j * D + d);
                    const float4 qb = *reinterpret_cast<const float4*>(qs + (size_t)j * D + d + 4);
                    float a = dot[j];
                    a = fmaf(qa.w, f[3], fmaf(qa.z, f[2], fmaf(qa.y, f[1], fmaf(qa.x, f[0], a))));
                    dot[j] = fmaf(qb.w, f[7], fmaf(qb.z, f[6], fmaf(qb.y, f[5], fmaf(qb.x, f[4], a))));
                }
        }
    } else {
        for (int d = 0; d < D; ++d) {
            const float v = __bfloat162float(kr[d]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (j < n_heads) dot[j] = fmaf(qs[(size_t)j * D + d], v, dot[j]);
        }
    }
}

// N consecutive values of a value row as floats, in one read (the address is a multiple of N values).
template <class T, int N> __device__ __forceinline__ void talk_read(const T* src, float f[N]);
template <> __device__ __forceinline__ void talk_read<float, 2>(const float* src, float f[2]) {
    const float2 v = *reinterpret_cast<const float2*>(src);
    f[0] = v.x, f[1] = v.y;
}
template <> __device__ __forceinline__ void talk_read<float, 4>(const float* src, float f[4]) {
    const float4 v = *reinterpret_cast<const float4*>(src);
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
template <> __device__ __forceinline__ void talk_read<__nv_bfloat16, 2>(const __nv_bfloat16* src, float f[2]) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
    f[0] = v.x, f[1] = v.y;
}
template <> __device__ __forceinline__ void talk_read<__nv_bfloat16, 4>(const __nv_bfloat16* src, float f[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
}

// The value sums of one turn for up to four query heads of one key/value head (bit j of ``live``: head j goes on) when
// a lane holds N consecutive columns (V = 32 * N): a <- a * alpha, then the turn's keys in their order.  A value row is
// read once by the warp for all the heads, eight rows in flight.
template <class T, int N>
__device__ __forceinline__ void talk_values(const SbFlex& p, float* acc0, const float* wgt0, const long long* toks, int kv_head,
                                            const float alpha[4], unsigned live, int V, int lane) {
    const T* vbase = (const T*)p.v;
    float a[4][N];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (live >> j & 1u)
#pragma unroll
            for (int e = 0; e < N; ++e) a[j][e] = acc0[(size_t)j * V + lane * N + e] * alpha[j];
    for (int t0 = 0; t0 < 32; t0 += 8) {
        float f[8][N];
        bool seen[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long long kt = toks[t0 + i];
            seen[i] = kt >= 0;
            if (seen[i]) talk_read<T, N>(vbase + flex_value_token(p, kt, kv_head) * p.v_row + lane * N, f[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (!seen[i]) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (live >> j & 1u) {
                    const float w = wgt0[j * 32 + t0 + i];
#pragma unroll
                    for (int e = 0; e < N; ++e) a[j][e] = fmaf(w, f[i][e], a[j][e]);
                }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (live >> j & 1u)
#pragma unroll
            for (int e = 0; e < N; ++e) acc0[(size_t)j * V + lane * N + e] = a[j][e];
}

// One block per row.  Shared memory: the row's queries as floats [H * D], the table [H * H], raw and mixed scores of a
// turn's 32 keys [H][32] each, the turn's key rows per key/value head [G][32], per head the running maximum and sum,
// and the heads' value sums [H * V].  A warp takes heads warp, warp + warps, ...
//
// With n_splits > 1 (decoding: few rows, many keys) blockIdx.y takes a share of the row's turns and leaves, per head, its
// unnormalised value sums, maximum and sum in ``partial`` [row][head][split][V + 2]; talking_merge_kernel divides.
template <class T>
__global__ void __launch_bounds__(256, 2) talking_attention_general_kernel(SbFlex p, SbBatch batch, T* __restrict__ out, int n_splits, float* __restrict__ partial) {
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
    const int heads_per_unit = max(1, min(min(4, per_kv), H / n_warps));      // query heads that share a key row's read
    const int head_chunks = (per_kv + heads_per_unit - 1) / heads_per_unit;
    // columns of a value row per lane when a warp can read the row in one go (32 lanes x 2 or 4 columns), else 0
    const int per_lane = (V == 64 || V == 128) && p.v_row % (V / 32) == 0 && (reinterpret_cast<size_t>(p.v) & 15) == 0 ? V / 32 : 0;
    {
        for (int turn = turn_lo; turn < turn_hi; ++turn) {
            const int n0 = turn < kept_turns ? turn * 32 : lo + (turn - kept_turns) * 32, end = turn < kept_turns ? kept_end : pos + 1;
            const int n = n0 + lane;
            const bool seen = n < end;
            for (int c = warp; c < G; c += n_warps) tok_s[c * 32 + lane] = seen ? flex_token(p, slot, n, c) : -1;
            __syncthreads();
            // a warp takes a key/value head and up to four of its query heads (fewer when warps would idle), a lane a key
            for (int u = warp; u < G * head_chunks; u += n_warps) {
                const int c = u / head_chunks, g0 = c * per_kv + (u % head_chunks) * heads_per_unit;
                const int ng = min(heads_per_unit, (c + 1) * per_kv - g0);
                const long long tok = tok_s[c * 32 + lane];
                float dot[4] = {0.f, 0.f, 0.f, 0.f};
                if (tok >= 0) talk_dots<T>(qs + (size_t)g0 * D, D, ng, kbase + tok * D, dot);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (j < ng) {
                        float s = dot[j] * p.scale;
                        if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
                        raw[(g0 + j) * 32 + lane] = tok >= 0 ? s : 0.f;
                    }
            }
            __syncthreads();
            // the same units: the heads of a unit share their key/value head's value rows
            for (int u = warp; u < G * head_chunks; u += n_warps) {
                const int c = u / head_chunks, g0 = c * per_kv + (u % head_chunks) * heads_per_unit;
                const int ng = min(heads_per_unit, (c + 1) * per_kv - g0);
                const long long tok = tok_s[c * 32 + lane];
                float alpha[4] = {1.f, 1.f, 1.f, 1.f};
                unsigned live = 0u;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j >= ng) continue;
                    const int h = g0 + j;
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
                    alpha[j] = expf(m_old - m_new);
                    const float sum = warp_sum(w);
                    wgt[h * 32 + lane] = w;
                    if (lane == 0) {
                        run_m[h] = m_new;
                        run_l[h] = run_l[h] * alpha[j] + sum;
                    }
                    live |= 1u << j;
                }
                __syncwarp();
                const long long* toks = tok_s + c * 32;
                if (per_lane == 2) talk_values<T, 2>(p, acc + (size_t)g0 * V, wgt + g0 * 32, toks, c, alpha, live, V, lane);
                else if (per_lane == 4) talk_values<T, 4>(p, acc + (size_t)g0 * V, wgt + g0 * 32, toks, c, alpha, live, V, lane);
                else
                    for (int j = 0; j < ng; ++j) {
                        if (!(live >> j & 1u)) continue;
                        const int h = g0 + j;
                        for (int d = lane; d < V; d += 32) {
                            float a = acc[h * V + d] * alpha[j];
                            for (int t2 = 0; t2 < 32; ++t2) {
                                const long long kt = toks[t2];
                                if (kt >= 0) a = fmaf(wgt[h * 32 + t2], to_f<T>(vbase[flex_value_token(p, kt, c) * p.v_row + d]), a);
                            }
                            acc[h * V + d] = a;
                        }
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
// Up to 64 splits: their scales are worked out once, by a thread each, and read from shared memory.
template <class T>
__global__ void talking_merge_kernel(const float* __restrict__ partial, T* __restrict__ out, const float* __restrict__ sink, int n_heads,
                                     int n_splits, int V) {
    __shared__ float scale_s[64];
    __shared__ float red[2];
    pdl_wait();
    const long long rh = (long long)blockIdx.x * n_heads + blockIdx.y;
    const float* base = partial + rh * n_splits * (V + 2);
    const int tid = threadIdx.x;
    const float ms = tid < n_splits ? base[(long long)tid * (V + 2) + V] : -INFINITY;
    float m = warp_max(ms);
    if ((tid & 31) == 0) red[tid >> 5] = m;
    __syncthreads();
    m = fmaxf(red[0], red[1]);
    if (sink != nullptr) m = fmaxf(m, sink[blockIdx.y]);
    const float sc = ms != -INFINITY ? expf(ms - m) : 0.f;
    scale_s[tid] = sc;
    __syncthreads();
    float l = sink != nullptr ? expf(sink[blockIdx.y] - m) : 0.f;
    for (int sidx = 0; sidx < n_splits; ++sidx)          // in the order of the splits, the same in every thread
        if (scale_s[sidx] != 0.f) l += base[(long long)sidx * (V + 2) + V + 1] * scale_s[sidx];
    for (int c = tid; c < V; c += blockDim.x) {
        float o = 0.f;
        for (int sidx = 0; sidx < n_splits; ++sidx)
            if (scale_s[sidx] != 0.f) o = fmaf(base[(long long)sidx * (V + 2) + c], scale_s[sidx], o);
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
    // gridDim.y == 3 (few rows): block y takes the queries, the keys or the values of the row; else one block takes all
    const bool do_q = gridDim.y == 1 || blockIdx.y == 0, do_k = gridDim.y == 1 || blockIdx.y == 1, do_v = gridDim.y == 1 || blockIdx.y == 2;
    const int nq = n_heads * p.k_dim, nk = p.n_kv_heads * p.k_dim, nv = p.n_kv_heads * p.v_dim;
    int slot, pos;
    row_place(batch, row, slot, pos);
    const T* r = qkv + (long long)row * (nq + nk + nv);
    if (do_q) {
        float q_rstd = 1.f;
        if (q_norm != nullptr) {
            float ss = 0.f;
            for (int c = threadIdx.x; c < nq; c += blockDim.x) {
                const float x = to_f<T>(r[c]);
                ss = fmaf(x, x, ss);
            }
            q_rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)nq + eps);
        }
        for (int c = threadIdx.x; c < nq; c += blockDim.x) {
            const float x = to_f<T>(r[c]);
            q_out[(long long)row * nq + c] = q_norm != nullptr ? from_f<T>(__fmul_rn(__fmul_rn(x, q_rstd), q_norm[c])) : r[c];
        }
    }
    if (!do_k && !do_v) return;
    const long long tok0 = flex_token(p, slot, pos, 0);
    if (tok0 < 0) {
        if (threadIdx.x == 0) atomicOr(status, SB_STATUS_NO_PAGE);
        return;
    }
    if (do_k) {
        float k_rstd = 1.f;
        if (k_norm != nullptr) {
            float ss = 0.f;
            for (int c = threadIdx.x; c < nk; c += blockDim.x) {
                const float x = to_f<T>(r[nq + c]);
                ss = fmaf(x, x, ss);
            }
            k_rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)nk + eps);
        }
        for (int c = threadIdx.x; c < nk; c += blockDim.x) {
            const int g = c / p.k_dim, d = c % p.k_dim;
            const float x = to_f<T>(r[nq + c]);
            ((T*)p.k)[(tok0 + (long long)g * SB_PAGE) * p.k_dim + d] =
                k_norm != nullptr ? from_f<T>(__fmul_rn(__fmul_rn(x, k_rstd), k_norm[c])) : r[nq + c];
        }
    }
    if (do_v)
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
    if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && partial == nullptr)) return (int)cudaErrorInvalidValue;
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
    const int parts = batch.n_rows < 64 ? 3 : 1;     // few rows (decoding): a row's queries, keys and values go to a block each
    if (dtype == SB_F32)
        sb_launch(qk_norm_store_kernel<float>, dim3(batch.n_rows, parts), threads, 0, stream, (const float*)qkv, (float*)q_out, batch, p,
                  n_heads, q_norm, k_norm, eps, status);
    else
        sb_launch(qk_norm_store_kernel<__nv_bfloat16>, dim3(batch.n_rows, parts), threads, 0, stream, (const __nv_bfloat16*)qkv,
                  (__nv_bfloat16*)q_out, batch, p, n_heads, q_norm, k_norm, eps, status);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
