// The matrix memory of an mLSTM layer: the recurrence over a sequence's rows with its running maximum, the division
// by the normaliser, the head's unit norm and the output gate.
//
//   i_t = cap * tanh((zi_t + bi) / cap),   f_t = logsigmoid(cap * tanh((zf_t + bf) / cap))        (one pair per head)
//   m_t = max(f_t + m_(t-1), i_t)                                                                  (m starts at 0)
//   S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t the same with k_t alone
//   h_t = S_t^T (q_t * q_scale) / (max(|n_t . q_t * q_scale|, exp(-m_t)) + 1e-6)
//   y_t = h_t / sqrt(mean(h_t^2) + eps) * norm * sigmoid(g_t) * out_scale                          (mean over the head)
//
// A sequence's record in the state group is [heads][D][V] floats of S, then [heads][D] of n, then [heads] of m, all
// zero when the sequence starts.  The kernel walks a sequence's rows in order from the record and writes it back, so
// a step of many tokens leaves what the same tokens leave one by one.  The normaliser is carried as one more column
// of the state whose "value" is 1: n_t . q_t then falls out of the same sum as the outputs.  Gates, maxima,
// exponentials, state, the division, the unit norm and the output gate are 32-bit; q, k, v, g come in the run's type
// as views of wider rows, the gates' pre-activations in 32-bit.
#include "common.cuh"

#define ML_TB 32   // tokens staged in shared memory at a time
#define ML_IG 8    // threads that share a column group of the state
#define ML_CG 2    // neighbouring columns that a thread holds
#define ML_VB 64   // value channels per block (the block holds one more column: the normaliser)
#define ML_VW (ML_VB + ML_CG)                          // columns of a staged row of values: 16-byte rows with the normaliser's column
#define ML_THREADS (((ML_VB / ML_CG + 1) * ML_IG + 31) / 32 * 32)  // a column group per 8 threads, rounded up to whole warps
#define ML_PF 8    // turns of a tile's loads that a thread keeps in registers ahead of time

__device__ __forceinline__ float log_sigmoid(float z) { return z < 0.f ? z - log1pf(expf(z)) : -log1pf(expf(-z)); }

// What a tile's tokens need of the gates: a[t] = exp(f + m_prev - m), b[t] = exp(i - m), em[t] = exp(-m).  One thread
// per token takes the gates, one thread walks the maxima in order (an addition and a maximum per token: the chain is
// short), then one thread per token takes the exponentials.  m_run holds m between tiles.
__device__ __forceinline__ void mlstm_gates(const float* __restrict__ z, long long z_ld, int i_col, int f_col, float bi, float bf, float cap,
                                            int t0, int nt, float* ig, float* fg, float* as, float* bs, float* em, float* m_run) {
    const int tid = threadIdx.x;
    if (tid < nt) {
        const float zi = z[(long long)(t0 + tid) * z_ld + i_col] + bi, zf = z[(long long)(t0 + tid) * z_ld + f_col] + bf;
        ig[tid] = cap * tanhf(zi / cap);
        fg[tid] = log_sigmoid(cap * tanhf(zf / cap));
    }
    __syncthreads();
    if (tid == 0) {
        float m = *m_run;
        for (int t = 0; t < nt; ++t) {
            as[t] = m;                       // the maximum before this token, until the exponentials below
            m = fmaxf(fg[t] + m, ig[t]);
            em[t] = m;
        }
        *m_run = m;
    }
    __syncthreads();
    if (tid < nt) {
        const float m_prev = as[tid], m_new = em[tid];
        as[tid] = expf(fg[tid] + m_prev - m_new);
        bs[tid] = expf(ig[tid] - m_new);
        em[tid] = expf(-m_new);
    }
    __syncthreads();
}

// One block per (sequence, head, group of ML_VB value channels).  A thread owns, in registers, the entries S[i][j] of
// ML_CG neighbouring columns j for E = ceil(D / 8) key channels i: what it reads of q_t and k_t from shared memory
// serves ML_CG columns.  Column nv of
// the block is the normaliser (its "value" is 1).  The eight threads of a column group are neighbouring lanes and add
// their shares with three shuffles per column.  EXACT: D = 8 * EMAX with EMAX a multiple of 4; a thread's key channels
// are then dealt out four at a time, ((e / 4) * 8 + ig) * 4 + e % 4, so that the eight lanes read 128 consecutive
// bytes, 16 a lane.  With o_raw the head's columns are shared out over several blocks, which leave h_t there for
// mlstm_finish_kernel; without, one block holds the whole head and finishes it itself.
template <class T, int EMAX, bool EXACT>
__global__ void __launch_bounds__(ML_THREADS)
mlstm_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g, long long ld,
                  const float* __restrict__ z, long long z_ld, int i_col, int f_col, const float* __restrict__ i_bias,
                  const float* __restrict__ f_bias, float cap, const float* __restrict__ norm_w, float eps, float q_scale,
                  float out_scale, float* __restrict__ state, long long state_stride, SbBatch batch, int H, int D, int V,
                  T* __restrict__ y, long long y_ld, float* __restrict__ o_raw) {
    extern __shared__ float4 sm4[];
    float* qs = reinterpret_cast<float*>(sm4);   // [ML_TB][D]
    float* ks = qs + ML_TB * D;
    float* vs = ks + ML_TB * D;                  // [ML_TB][ML_VW]: the values, 1 in column nv, 0 beyond
    float* os = vs + ML_TB * ML_VW;              // [ML_TB][ML_VW]
    float* gs = os + ML_TB * ML_VW;              // [ML_TB][ML_VB]: sigmoid(g)
    __shared__ float ig_s[ML_TB], fg_s[ML_TB], as[ML_TB], bs[ML_TB], em[ML_TB], mul_s[ML_TB], m_run;
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, n_threads = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, n_warps = n_threads >> 5;
    const int j0 = blockIdx.z * ML_VB, nv = min(ML_VB, V - j0);
    const int cg = tid / ML_IG, ig = tid % ML_IG, c0 = cg * ML_CG;
    const bool active = c0 <= nv;
    const int E = (D + ML_IG - 1) / ML_IG, i0 = ig * E;
    auto chan = [&](int e) { return EXACT ? ((e >> 2) * ML_IG + ig) * 4 + (e & 3) : i0 + e; };   // key channel of entry e
    const float bi = i_bias[head], bf = f_bias[head];
    pdl_wait();
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    float* rec = state + (long long)slot * state_stride;
    float* Sg = rec + (long long)head * D * V;
    float* ng = rec + (long long)H * D * V + (long long)head * D;
    float* mg = rec + (long long)H * D * V + (long long)H * D + head;
    if (tid == 0) m_run = *mg;
    float S[ML_CG][EMAX];
#pragma unroll
    for (int c = 0; c < ML_CG; ++c)
#pragma unroll
        for (int e = 0; e < EMAX; ++e) {
            S[c][e] = 0.f;
            if (active && e < E && chan(e) < D) {
                if (c0 + c < nv) S[c][e] = Sg[(long long)chan(e) * V + j0 + c0 + c];
                else if (c0 + c == nv) S[c][e] = ng[chan(e)];
            }
        }
    for (int e = tid; e < ML_TB * ML_VW; e += n_threads) vs[e] = (e % ML_VW) == nv ? 1.0f : 0.f;   // columns that no load writes
    // A thread's first ML_PF turns of a tile's loads wait in registers while the tile before is worked on, so that the
    // loads' way to memory and back is hidden behind the recurrence; (token, column) of turn u follow from those of
    // turn 0 by additions.
    T rq[ML_PF], rk[ML_PF], rv[ML_PF], rg[ML_PF];
    const int qk_dt = n_threads / D, qk_di = n_threads % D, v_dt = n_threads / nv, v_dc = n_threads % nv;
    const int qk_t0 = tid / D, qk_i0 = tid % D, v_t0 = tid / nv, v_c0 = tid % nv;
    auto fetch = [&](int t0, int nt) {
        int tt = qk_t0, i = qk_i0;
#pragma unroll
        for (int u = 0; u < ML_PF; ++u) {
            if (tt < nt) {
                const long long at = (long long)(t0 + tt) * ld + head * D + i;
                rq[u] = q[at];
                rk[u] = k[at];
            }
            tt += qk_dt;
            i += qk_di;
            if (i >= D) {
                i -= D;
                ++tt;
            }
        }
        tt = v_t0;
        int c = v_c0;
#pragma unroll
        for (int u = 0; u < ML_PF; ++u) {
            if (tt < nt) {
                const long long at = (long long)(t0 + tt) * ld + head * V + j0 + c;
                rv[u] = v[at];
                if (o_raw == nullptr) rg[u] = g[at];
            }
            tt += v_dt;
            c += v_dc;
            if (c >= nv) {
                c -= nv;
                ++tt;
            }
        }
    };
    if (row0 < row1) fetch(row0, min(ML_TB, row1 - row0));
    __syncthreads();
    for (int t0 = row0; t0 < row1; t0 += ML_TB) {
        const int nt = min(ML_TB, row1 - t0);
        __syncthreads();
        mlstm_gates(z, z_ld, i_col + head, f_col + head, bi, bf, cap, t0, nt, ig_s, fg_s, as, bs, em, &m_run);
        {   // what waited in registers goes to shared memory; turns beyond ML_PF load now
            int e = tid;
#pragma unroll
            for (int u = 0; u < ML_PF; ++u, e += n_threads)
                if (e < nt * D) {
                    qs[e] = to_f<T>(rq[u]) * q_scale;
                    ks[e] = to_f<T>(rk[u]);
                }
#pragma unroll 4
            for (; e < nt * D; e += n_threads) {
                const int tt = e / D, i = e - tt * D;
                const long long at = (long long)(t0 + tt) * ld + head * D + i;
                qs[e] = to_f<T>(q[at]) * q_scale;
                ks[e] = to_f<T>(k[at]);
            }
            int tt = v_t0, c = v_c0;
            e = tid;
#pragma unroll
            for (int u = 0; u < ML_PF; ++u, e += n_threads) {
                if (e < nt * nv) {
                    vs[tt * ML_VW + c] = to_f<T>(rv[u]);
                    if (o_raw == nullptr) gs[tt * ML_VB + c] = 1.0f / (1.0f + expf(-to_f<T>(rg[u])));
                }
                tt += v_dt;
                c += v_dc;
                if (c >= nv) {
                    c -= nv;
                    ++tt;
                }
            }
#pragma unroll 4
            for (; e < nt * nv; e += n_threads) {
                const int t2 = e / nv, c2 = e - t2 * nv;
                const long long at = (long long)(t0 + t2) * ld + head * V + j0 + c2;
                vs[t2 * ML_VW + c2] = to_f<T>(v[at]);
                if (o_raw == nullptr) gs[t2 * ML_VB + c2] = 1.0f / (1.0f + expf(-to_f<T>(g[at])));
            }
        }
        __syncthreads();
        if (t0 + ML_TB < row1) fetch(t0 + ML_TB, min(ML_TB, row1 - t0 - ML_TB));
        {   // every thread walks the tokens (the shuffles want whole warps); a thread without columns reads the first ones
            // and writes nothing
            const int c0r = active ? c0 : 0;
#pragma unroll 2
            for (int tt = 0; tt < nt; ++tt) {
                const float a = as[tt], b = bs[tt];
                float bv[ML_CG], o[ML_CG];
#pragma unroll
                for (int c = 0; c < ML_CG; ++c) {
                    bv[c] = b * vs[tt * ML_VW + c0r + c];
                    o[c] = 0.f;
                }
                if (EXACT) {   // two entries of the state per instruction (fma.rn.f32x2): the time here is the instruction count
                    constexpr int DC = ML_IG * EMAX;
                    const float2 a2 = make_float2(a, a), zero = make_float2(0.f, 0.f);
                    float2 o2[ML_CG];
#pragma unroll
                    for (int c = 0; c < ML_CG; ++c) o2[c] = zero;
#pragma unroll
                    for (int e = 0; e < EMAX; e += 4) {
                        const int at = tt * DC + ((e >> 2) * ML_IG + ig) * 4;
                        const float4 q4 = *reinterpret_cast<const float4*>(qs + at);
                        const float4 k4 = *reinterpret_cast<const float4*>(ks + at);
#pragma unroll
                        for (int c = 0; c < ML_CG; ++c) {
                            const float2 bv2 = make_float2(bv[c], bv[c]);
                            float2 s01 = make_float2(S[c][e], S[c][e + 1]), s23 = make_float2(S[c][e + 2], S[c][e + 3]);
                            s01 = fma_pair(a2, s01, fma_pair(make_float2(k4.x, k4.y), bv2, zero));
                            s23 = fma_pair(a2, s23, fma_pair(make_float2(k4.z, k4.w), bv2, zero));
                            o2[c] = fma_pair(make_float2(q4.x, q4.y), s01, o2[c]);
                            o2[c] = fma_pair(make_float2(q4.z, q4.w), s23, o2[c]);
                            S[c][e] = s01.x;
                            S[c][e + 1] = s01.y;
                            S[c][e + 2] = s23.x;
                            S[c][e + 3] = s23.y;
                        }
                    }
#pragma unroll
                    for (int c = 0; c < ML_CG; ++c) o[c] = o2[c].x + o2[c].y;
                } else {
                    const float* qt = qs + tt * D + i0;
                    const float* kt = ks + tt * D + i0;
#pragma unroll
                    for (int e = 0; e < EMAX; ++e) {
                        if (e < E && i0 + e < D) {
                            const float qe = qt[e], ke = kt[e];
#pragma unroll
                            for (int c = 0; c < ML_CG; ++c) {
                                S[c][e] = fmaf(a, S[c][e], ke * bv[c]);
                                o[c] = fmaf(qe, S[c][e], o[c]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int c = 0; c < ML_CG; ++c) {
                    o[c] += __shfl_xor_sync(0xffffffffu, o[c], 1);
                    o[c] += __shfl_xor_sync(0xffffffffu, o[c], 2);
                    o[c] += __shfl_xor_sync(0xffffffffu, o[c], 4);
                }
                if (ig == 0 && active) {
#pragma unroll
                    for (int c = 0; c < ML_CG; ++c) os[tt * ML_VW + c0 + c] = o[c];
                }
            }
        }
        __syncthreads();
        if (o_raw != nullptr) {
            for (int e = tid; e < nt * nv; e += n_threads) {
                const int tt = e / nv, c = e - tt * nv;
                const float den = fmaxf(fabsf(os[tt * ML_VW + nv]), em[tt]) + 1e-6f;
                o_raw[((long long)(t0 + tt) * H + head) * V + j0 + c] = os[tt * ML_VW + c] / den;
            }
            continue;
        }
        for (int tt = warp; tt < nt; tt += n_warps) {   // the division and the head's root mean square, a warp per token
            const float den = fmaxf(fabsf(os[tt * ML_VW + nv]), em[tt]) + 1e-6f;
            float ss = 0.f;
            for (int c = lane; c < nv; c += 32) {
                const float h = os[tt * ML_VW + c] / den;
                os[tt * ML_VW + c] = h;
                ss = fmaf(h, h, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) mul_s[tt] = out_scale / sqrtf(ss / (float)V + eps);
        }
        __syncthreads();
        for (int e = tid; e < nt * nv; e += n_threads) {
            const int tt = e / nv, c = e - tt * nv;
            y[(long long)(t0 + tt) * y_ld + head * V + c] =
                from_f<T>(os[tt * ML_VW + c] * mul_s[tt] * norm_w[head * V + c] * gs[tt * ML_VB + c]);
        }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < ML_CG; ++c)
#pragma unroll
        for (int e = 0; e < EMAX; ++e) {
            if (active && e < E && chan(e) < D) {
                if (c0 + c < nv) Sg[(long long)chan(e) * V + j0 + c0 + c] = S[c][e];
                else if (c0 + c == nv && blockIdx.z == 0) ng[chan(e)] = S[c][e];
            }
        }
    if (tid == 0 && blockIdx.z == 0) *mg = m_run;
}

// One warp per (row, head): the head's unit norm over its V values of h, the norm weight, the gate and the scale.
template <class T>
__global__ void mlstm_finish_kernel(const float* __restrict__ o_raw, const T* __restrict__ g, long long ld, const float* __restrict__ norm_w,
                                    float eps, float out_scale, int rows, int H, int V, T* __restrict__ y, long long y_ld) {
    pdl_wait();
    const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)rows * H) return;
    const long long row = wid / H;
    const int head = (int)(wid % H);
    const float* o = o_raw + (row * H + head) * V;
    float ss = 0.f;
    for (int c = lane; c < V; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float mul = out_scale / sqrtf(ss / (float)V + eps);
    for (int c = lane; c < V; c += 32) {
        const float gv = to_f<T>(g[row * ld + head * V + c]);
        y[row * y_ld + head * V + c] = from_f<T>(o[c] * mul * norm_w[head * V + c] * (1.0f / (1.0f + expf(-gv))));
    }
}

// Heads beyond what the kernel above holds in registers: the state stays in global memory (it is the sequence's
// record anyway); thread j owns column j (column V: the normaliser) and walks its key channels token by token.
template <class T>
__global__ void mlstm_scan_wide_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ g,
                                       long long ld, const float* __restrict__ z, long long z_ld, int i_col, int f_col,
                                       const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                                       const float* __restrict__ norm_w, float eps, float q_scale, float out_scale,
                                       float* __restrict__ state, long long state_stride, SbBatch batch, int H, int D, int V,
                                       T* __restrict__ y, long long y_ld) {
    extern __shared__ float sm[];
    float* qs = sm;          // the token's q and k * b, [D] each
    float* ks = qs + D;
    float* os = ks + D;      // the token's sums [V + 1]
    __shared__ float red[33];
    __shared__ float ig_s[1], fg_s[1], as[1], bs[1], em[1], m_run;
    pdl_wait();
    const int s = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
    const int slot = batch.seq_slot[s], row0 = batch.cu_q[s], row1 = batch.cu_q[s + 1];
    float* rec = state + (long long)slot * state_stride;
    float* Sg = rec + (long long)head * D * V;
    float* ng = rec + (long long)H * D * V + (long long)head * D;
    float* mg = rec + (long long)H * D * V + (long long)H * D + head;
    if (tid == 0) m_run = *mg;
    __syncthreads();
    for (int t = row0; t < row1; ++t) {
        __syncthreads();
        mlstm_gates(z, z_ld, i_col + head, f_col + head, i_bias[head], f_bias[head], cap, t, 1, ig_s, fg_s, as, bs, em, &m_run);
        for (int i = tid; i < D; i += blockDim.x) {
            const long long at = (long long)t * ld + head * D + i;
            qs[i] = to_f<T>(q[at]) * q_scale;
            ks[i] = to_f<T>(k[at]) * bs[0];
        }
        __syncthreads();
        const float a = as[0];
        for (int j = tid; j <= V; j += blockDim.x) {   // the same thread owns column j at every token
            const float vj = j < V ? to_f<T>(v[(long long)t * ld + head * V + j]) : 1.0f;
            float o = 0.f;
            for (int i = 0; i < D; ++i) {
                float* cell = j < V ? Sg + (long long)i * V + j : ng + i;
                const float nv = fmaf(a, *cell, ks[i] * vj);
                *cell = nv;
                o = fmaf(qs[i], nv, o);
            }
            os[j] = o;
        }
        __syncthreads();
        const float den = fmaxf(fabsf(os[V]), em[0]) + 1e-6f;
        float ss = 0.f;
        for (int j = tid; j < V; j += blockDim.x) {
            const float h = os[j] / den;
            ss = fmaf(h, h, ss);
        }
        ss = block_sum(ss, red);
        const float mul = out_scale / sqrtf(ss / (float)V + eps);
        for (int j = tid; j < V; j += blockDim.x) {
            const float gv = to_f<T>(g[(long long)t * ld + head * V + j]);
            y[(long long)t * y_ld + head * V + j] = from_f<T>(os[j] / den * mul * norm_w[head * V + j] * (1.0f / (1.0f + expf(-gv))));
        }
    }
    __syncthreads();
    if (tid == 0) *mg = m_run;
}

extern "C" {

// q, k [rows, H * D], v, g [rows, H * V]: views whose rows are `ld` elements apart; z [rows, z_ld] 32-bit with head h's
// input gate at column i_col + h and forget gate at f_col + h; state [slots] records of H * D * V + H * D + H floats,
// `state_stride` floats apart; y [rows, H * V] with rows y_ld apart; o_raw: [rows, H * V] floats of scratch for heads
// of more than ML_VB value channels.
int sb_mlstm_scan(int dtype, const void* q, const void* k, const void* v, const void* g, long long ld, const float* z, long long z_ld,
                  int i_col, int f_col, const float* i_bias, const float* f_bias, float cap, const float* norm_w, float eps,
                  float q_scale, float out_scale, float* state, long long state_stride, SbBatch batch, int H, int D, int V, void* y,
                  long long y_ld, float* o_raw, cudaStream_t stream) {
    if (batch.n_seqs <= 0 || batch.n_rows <= 0) return 0;
    if (D < 1 || V < 1 || D > 4096 || V > 4096 || H > 65535 || !(cap > 0.f)) return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf;
    const int chunks = (V + ML_VB - 1) / ML_VB;
    if (D > 128 || chunks > 64 || (chunks > 1 && o_raw == nullptr)) {
        dim3 grid(batch.n_seqs, H);
        const int wt = V + 1 < 1024 ? (V + 1 + 31) / 32 * 32 : 1024;
        const size_t wsmem = (size_t)(2 * D + V + 1) * sizeof(float);
        if (dtype == SB_F32)
            sb_launch(mlstm_scan_wide_kernel<float>, grid, wt, wsmem, stream, (const float*)q, (const float*)k, (const float*)v,
                      (const float*)g, ld, z, z_ld, i_col, f_col, i_bias, f_bias, cap, norm_w, eps, q_scale, out_scale, state,
                      state_stride, batch, H, D, V, (float*)y, y_ld);
        else
            sb_launch(mlstm_scan_wide_kernel<bf>, grid, wt, wsmem, stream, (const bf*)q, (const bf*)k, (const bf*)v, (const bf*)g, ld, z,
                      z_ld, i_col, f_col, i_bias, f_bias, cap, norm_w, eps, q_scale, out_scale, state, state_stride, batch, H, D, V,
                      (bf*)y, y_ld);
        SB_LAUNCH_CHECK();
    }
    const size_t smem = (size_t)(ML_TB * (2 * D + 2 * ML_VW + ML_VB)) * sizeof(float);
    dim3 grid(batch.n_seqs, H, chunks);
    const int threads = (((min(V, ML_VB) + 1 + ML_CG - 1) / ML_CG) * ML_IG + 31) / 32 * 32;
    float* raw = chunks > 1 ? o_raw : nullptr;
#define SB_ML(T, EMAX, EXACT)                                                                                                        \
    do {                                                                                                                             \
        if (smem > 48 * 1024) {                                                                                                      \
            const cudaError_t err = cudaFuncSetAttribute(mlstm_scan_kernel<T, EMAX, EXACT>,                                          \
                                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
            if (err != cudaSuccess) return (int)err;                                                                                 \
        }                                                                                                                            \
        sb_launch(mlstm_scan_kernel<T, EMAX, EXACT>, grid, threads, smem, stream, (const T*)q, (const T*)k, (const T*)v, (const T*)g, \
                  ld, z, z_ld, i_col, f_col, i_bias, f_bias, cap, norm_w, eps, q_scale, out_scale, state, state_stride, batch, H, D, \
                  V, (T*)y, y_ld, raw);                                                                                              \
    } while (0)
#define SB_ML_SIZES(T)                            \
    do {                                          \
        if (D == 32) SB_ML(T, 4, true);           \
        else if (D == 64) SB_ML(T, 8, true);      \
        else if (D == 128) SB_ML(T, 16, true);    \
        else if (D <= 32) SB_ML(T, 4, false);     \
        else if (D <= 64) SB_ML(T, 8, false);     \
        else SB_ML(T, 16, false);                 \
    } while (0)
    if (dtype == SB_F32) SB_ML_SIZES(float);
    else SB_ML_SIZES(bf);
#undef SB_ML_SIZES
#undef SB_ML
    if (raw != nullptr) {
        const long long warps = (long long)batch.n_rows * H;
        const unsigned int blocks = (unsigned int)((warps * 32 + 255) / 256);
        if (dtype == SB_F32)
            sb_launch(mlstm_finish_kernel<float>, blocks, 256, 0, stream, (const float*)raw, (const float*)g, ld, norm_w, eps, out_scale,
                      batch.n_rows, H, V, (float*)y, y_ld);
        else
            sb_launch(mlstm_finish_kernel<bf>, blocks, 256, 0, stream, (const float*)raw, (const bf*)g, ld, norm_w, eps, out_scale,
                      batch.n_rows, H, V, (bf*)y, y_ld);
    }
    SB_LAUNCH_CHECK();
}

}  // extern "C"
