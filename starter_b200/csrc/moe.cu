// Mixture of experts: the router, the order of the chosen (token, expert) pairs by expert, the experts' products for a
// handful of pairs, and the weighted sum that brings a token's experts together.
//
//   s = softmax(W_r h) over experts + identity outputs                      (32-bit)
//   chosen = the `top` largest of s + correction;  weight = s / (sum of the chosen s + 1e-20) * scale
//   y = base + sum over chosen e of weight_e * (e is an identity output ? h : down_e(act(gate_e h, up_e h)))
//
// A pair is (row, k): the k-th choice of a row.  Pairs of identity outputs read no matrix.  For many rows the pairs are
// put in the order of their experts (a slot per pair), so that one grouped product per matrix serves the step; for a
// few pairs each pair streams its expert's matrices through the kernels below (a warp per output column).
#include "common.cuh"

#define MOE_MAX_OUTPUTS 1024   // experts + identity outputs that the router kernel takes
#define MOE_MAX_TOP 32

#define MOE_ROUTE_ROWS 8   // rows that share one read of a router row

__device__ __forceinline__ float4 load4f(const float* p) { return *reinterpret_cast<const float4*>(p); }

// n values of the run's type into shared memory as floats; bfloat16 rows whose width is a multiple of 8 go 16 bytes a read.
template <class T> __device__ __forceinline__ void stage_rows(float* dst, const T* src, int n, bool vec) {
#pragma unroll 8
    for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = to_f<T>(src[e]);
}
template <> __device__ __forceinline__ void stage_rows<__nv_bfloat16>(float* dst, const __nv_bfloat16* src, int n, bool vec) {
    if (!vec || (reinterpret_cast<uintptr_t>(src) & 15)) {
#pragma unroll 8
        for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = __bfloat162float(src[e]);
        return;
    }
#pragma unroll 4
    for (int e = threadIdx.x * 8; e < n; e += blockDim.x * 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + e);
        const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(hh[0]), b = __bfloat1622float2(hh[1]), c = __bfloat1622float2(hh[2]), d = __bfloat1622float2(hh[3]);
        *reinterpret_cast<float4*>(dst + e) = make_float4(a.x, a.y, b.x, b.y);
        *reinterpret_cast<float4*>(dst + e + 4) = make_float4(c.x, c.y, d.x, d.y);
    }
}

// Router logits, 32-bit.  A block of 8 warps takes R rows (R <= 8) and 8 router rows: the rows of h are staged in shared
// memory as floats, warp w reads router row blockIdx.y * 8 + w once (16 bytes per lane where the width allows, four
// turns in flight) and forms its dot product with all R rows.  With few rows R is 1 and the router's rows are spread
// over rows * outputs / 8 blocks, so that a decode step does not wait on a handful of SMs.  A row's logit is summed in
// the same order whatever R.
template <class T>
__global__ void __launch_bounds__(256)
moe_logits_kernel(const T* __restrict__ h, const float* __restrict__ router, float* __restrict__ logits, int rows, int width,
                  int n_out, int R) {
    extern __shared__ __align__(16) float route_sm[];
    float* hs = route_sm;                         // [R][width]
    pdl_wait();
    const int row0 = blockIdx.x * R, nr = min(R, rows - row0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    stage_rows<T>(hs, h + (long long)row0 * width, nr * width, (width & 7) == 0);
    __syncthreads();
    for (int e = blockIdx.y * 8 + warp; e < n_out; e += gridDim.y * 8) {
    const float* wr = router + (long long)e * width;
    float acc[MOE_ROUTE_ROWS];
#pragma unroll
    for (int r = 0; r < MOE_ROUTE_ROWS; ++r) acc[r] = 0.f;
    if ((width & 3) == 0) {
#pragma unroll 4
        for (int c = lane * 4; c < width; c += 128) {
            const float4 w4 = load4f(wr + c);
#pragma unroll
            for (int r = 0; r < MOE_ROUTE_ROWS; ++r)
                if (r < nr) {
                    const float4 x = load4f(hs + (size_t)r * width + c);
                    acc[r] = fmaf(x.x, w4.x, fmaf(x.y, w4.y, fmaf(x.z, w4.z, fmaf(x.w, w4.w, acc[r]))));
                }
        }
    } else {
        for (int c = lane; c < width; c += 32) {
            const float wv = wr[c];
#pragma unroll
            for (int r = 0; r < MOE_ROUTE_ROWS; ++r)
                if (r < nr) acc[r] = fmaf(hs[(size_t)r * width + c], wv, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < MOE_ROUTE_ROWS; ++r)
        if (r < nr) {
            const float d = warp_sum(acc[r]);
            if (lane == 0) logits[(long long)(row0 + r) * n_out + e] = d;
        }
    }
}

// One warp per row: softmax over all outputs, the `top` largest of score + correction (of equals the lowest index), and
// their weights.  bias (or null) is added to the logits first; correction may be null.  over_chosen: the `top` largest
// LOGITS (+ correction) are chosen and weighted by the softmax over the chosen logits alone.
__global__ void __launch_bounds__(256)
moe_choose_kernel(const float* __restrict__ logits, const float* __restrict__ correction, const float* __restrict__ bias,
                  int over_chosen, int* __restrict__ chosen, float* __restrict__ weight, int rows, int n_out, int top, float scale) {
    extern __shared__ __align__(16) float route_sm[];
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * 8 + warp;
    if (row >= rows) return;
    float* s_s = route_sm + (size_t)warp * 2 * n_out;   // scores
    float* c_s = s_s + n_out;                           // choice scores; -inf once taken
    const float* lr = logits + row * n_out;
    float mx = -INFINITY;
    for (int e = lane; e < n_out; e += 32) {
        s_s[e] = bias != nullptr ? lr[e] + bias[e] : lr[e];
        mx = fmaxf(mx, s_s[e]);
    }
    mx = warp_max(mx);
    if (!over_chosen) {
        float sum = 0.f;
        for (int e = lane; e < n_out; e += 32) {
            const float w = expf(s_s[e] - mx);
            s_s[e] = w;
            sum += w;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < n_out; e += 32) s_s[e] *= inv;
    }
    for (int e = lane; e < n_out; e += 32) c_s[e] = correction != nullptr ? s_s[e] + correction[e] : s_s[e];
    __syncwarp();
    float total = 0.f;
    int mine = 0;   // lane k keeps the k-th choice
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_out; e += 32)
            if (c_s[e] > best) {
                best = c_s[e];
                at = e;
            }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) {
                best = ob;
                at = oa;
            }
        }
        if (at == 0x7fffffff) at = 0;
        if (lane == k) mine = at;
        total += s_s[at];
        __syncwarp();
        if (lane == 0) c_s[at] = -INFINITY;
        __syncwarp();
    }
    if (over_chosen) {   // softmax over the chosen logits: lane k holds the k-th
        const float z = lane < top ? s_s[mine] : -INFINITY;
        const float zm = warp_max(z);
        const float w = lane < top ? expf(z - zm) : 0.f;
        const float all = warp_sum(w);
        if (lane < top) {
            chosen[row * top + lane] = mine;
            weight[row * top + lane] = w / all * scale;
        }
        return;
    }
    if (lane < top) {
        chosen[row * top + lane] = mine;
        weight[row * top + lane] = s_s[mine] / (total + 1e-20f) * scale;
    }
}

// One block: counts per expert, their running sums (ends[e] = pairs of experts 0..e), and a slot for every pair of a
// real expert, expert by expert (-1 for pairs of identity outputs).  Within an expert the pairs keep their order.
__global__ void moe_sort_kernel(const int* __restrict__ chosen, int n_pairs, int n_experts, int* __restrict__ ends,
                                int* __restrict__ slot_of_pair, int* __restrict__ pair_of_slot) {
    extern __shared__ int cnt[];   // [n_experts] counts, then starts
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e >= 0 && e < n_experts) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int c = cnt[e];
            cnt[e] = run;
            run += c;
            ends[e] = run;
        }
    }
    __syncthreads();
    // in order: a warp takes an expert and walks the pairs with ballots, so that a pair's slot does not depend on timing
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    for (int e = warp; e < n_experts; e += n_warps) {
        int at = cnt[e];
        for (int p0 = 0; p0 < n_pairs; p0 += 32) {
            const int p = p0 + lane;
            const bool hit = p < n_pairs && chosen[p] == e;
            const unsigned int mask = __ballot_sync(0xffffffffu, hit);
            if (hit) {
                const int slot = at + __popc(mask & ((1u << lane) - 1u));
                slot_of_pair[p] = slot;
                pair_of_slot[slot] = p;
            }
            at += __popc(mask);
        }
    }
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = chosen[p];
        if (e < 0 || e >= n_experts) slot_of_pair[p] = -1;
    }
}

// xs[slot] = h[row of the slot's pair], 16 bytes per thread where the rows allow.
template <class T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ pair_of_slot, const int* __restrict__ ends,
                                  int n_experts, int top, int width, T* __restrict__ xs) {
    pdl_wait();
    const int slot = blockIdx.x;
    if (slot >= ends[n_experts - 1]) return;
    const T* src = h + (long long)(pair_of_slot[slot] / top) * width;
    T* dst = xs + (long long)slot * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
}

// Dot products of one row with up to two matrix rows: 16 bytes per lane and turn for bfloat16 rows whose width is a
// multiple of 8 (x is staged in shared memory as floats), a column per lane otherwise.
template <class T>
__device__ __forceinline__ void dot2(const float* xs, const T* r0, const T* r1, int n, int lane, float& d0, float& d1) {
    d0 = d1 = 0.f;
    for (int i = lane; i < n; i += 32) {
        const float x = xs[i];
        d0 = fmaf(x, to_f<T>(r0[i]), d0);
        if (r1 != nullptr) d1 = fmaf(x, to_f<T>(r1[i]), d1);
    }
}
template <>
__device__ __forceinline__ void dot2<__nv_bfloat16>(const float* xs, const __nv_bfloat16* r0, const __nv_bfloat16* r1, int n, int lane,
                                                    float& d0, float& d1) {
    d0 = d1 = 0.f;
    if ((n & 7) != 0) {
        for (int i = lane; i < n; i += 32) {
            const float x = xs[i];
            d0 = fmaf(x, __bfloat162float(r0[i]), d0);
            if (r1 != nullptr) d1 = fmaf(x, __bfloat162float(r1[i]), d1);
        }
        return;
    }
#pragma unroll 4
    for (int i = lane * 8; i < n; i += 256) {   // unrolled: eight 16-byte reads of the matrix in flight per lane
        const uint4 a = *reinterpret_cast<const uint4*>(r0 + i);
        uint4 b = make_uint4(0u, 0u, 0u, 0u);
        if (r1 != nullptr) b = *reinterpret_cast<const uint4*>(r1 + i);
        const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
        const float4 x0 = *reinterpret_cast<const float4*>(xs + i), x1 = *reinterpret_cast<const float4*>(xs + i + 4);
        const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 fa = __bfloat1622float2(ah[e]), fb = __bfloat1622float2(bh[e]);
            d0 = fmaf(xv[2 * e], fa.x, d0);
            d0 = fmaf(xv[2 * e + 1], fa.y, d0);
            d1 = fmaf(xv[2 * e], fb.x, d1);
            d1 = fmaf(xv[2 * e + 1], fb.y, d1);
        }
    }
}

// A pair's gate and up products with the activation: act[pair][c] for the block's columns, a warp per column.
template <class T>
__global__ void __launch_bounds__(256)
moe_pair_gate_up_kernel(const T* __restrict__ h, const int* __restrict__ chosen, const T* __restrict__ w_gate_up, T* __restrict__ act,
                        int top, int n_experts, int width, int ff, float alpha, float limit, int silu) {
    extern __shared__ __align__(16) float pair_x[];
    pdl_wait();
    const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int e = chosen[pair];
    if (e < 0 || e >= n_experts) return;
    const T* hr = h + (long long)(pair / top) * width;
    stage_rows<T>(pair_x, hr, width, (width & 7) == 0);
    __syncthreads();
    const T* wg = w_gate_up + (long long)e * 2 * ff * width;
    for (int c = blockIdx.y * n_warps + warp; c < ff; c += gridDim.y * n_warps) {
        float g, u;
        dot2<T>(pair_x, wg + (long long)c * width, wg + (long long)(ff + c) * width, width, lane, g, u);
        g = warp_sum(g);
        u = warp_sum(u);
        if (lane == 0) {
            if (silu) {   // silu(gate) * up, nothing clamped
                g = rnd<T>(g);
                act[(long long)pair * ff + c] = from_f<T>(g / (1.0f + expf(-g)) * rnd<T>(u));
            } else {
                g = fminf(rnd<T>(g), limit);
                u = fminf(fmaxf(rnd<T>(u), -limit), limit);
                act[(long long)pair * ff + c] = from_f<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
            }
        }
    }
}

// A pair's down product: down[pair][c], a warp per two columns.
template <class T>
__global__ void __launch_bounds__(256)
moe_pair_down_kernel(const T* __restrict__ act, const int* __restrict__ chosen, const T* __restrict__ w_down, T* __restrict__ down,
                     int n_experts, int width, int ff) {
    extern __shared__ __align__(16) float pair_x[];
    pdl_wait();
    const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int e = chosen[pair];
    if (e < 0 || e >= n_experts) return;
    const T* ar = act + (long long)pair * ff;
    stage_rows<T>(pair_x, ar, ff, (ff & 7) == 0);
    __syncthreads();
    const T* wd = w_down + (long long)e * width * ff;
    for (int c = 2 * (blockIdx.y * n_warps + warp); c < width; c += 2 * gridDim.y * n_warps) {
        float d0, d1;
        dot2<T>(pair_x, wd + (long long)c * ff, c + 1 < width ? wd + (long long)(c + 1) * ff : nullptr, ff, lane, d0, d1);
        d0 = warp_sum(d0);
        d1 = warp_sum(d1);
        if (lane == 0) {
            down[(long long)pair * width + c] = from_f<T>(d0);
            if (c + 1 < width) down[(long long)pair * width + c + 1] = from_f<T>(d1);
        }
    }
}

// y[row] = base[row] + sum_k weight[row][k] * (identity ? h[row] : down[place of pair (row, k)]), summed in 32-bit in
// the order of k.  slot_of_pair null: a pair's result lies at the pair's own index.  VEC (bfloat16 rows whose width is
// a multiple of 8): eight columns per thread, 16-byte accesses.
template <class T, bool VEC>
__global__ void moe_combine_kernel(const T* __restrict__ h, const T* __restrict__ down, const T* __restrict__ base,
                                   const int* __restrict__ chosen, const float* __restrict__ weight, const int* __restrict__ slot_of_pair,
                                   T* __restrict__ y, int top, int n_experts, int width) {
    __shared__ int place_s[MOE_MAX_TOP];
    __shared__ float w_s[MOE_MAX_TOP];
    pdl_wait();
    const long long row = blockIdx.x;
    if (threadIdx.x < top) {
        const long long pair = row * top + threadIdx.x;
        const int e = chosen[pair];
        w_s[threadIdx.x] = weight[pair];
        place_s[threadIdx.x] = (e < 0 || e >= n_experts) ? -1 : (slot_of_pair != nullptr ? slot_of_pair[pair] : (int)pair);
    }
    __syncthreads();
    if (VEC) {
        typedef __nv_bfloat16 bf;
        for (int c = threadIdx.x * 8; c < width; c += blockDim.x * 8) {
            float acc[8], hv[8];
            const uint4 hraw = *reinterpret_cast<const uint4*>((const bf*)h + row * width + c);
            uint4 braw = make_uint4(0u, 0u, 0u, 0u);
            if (base != nullptr) braw = *reinterpret_cast<const uint4*>((const bf*)base + row * width + c);
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&hraw);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&braw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(hh[e]), b = __bfloat1622float2(bh[e]);
                hv[2 * e] = f.x;
                hv[2 * e + 1] = f.y;
                acc[2 * e] = b.x;
                acc[2 * e + 1] = b.y;
            }
            for (int k = 0; k < top; ++k) {
                const int at = place_s[k];
                const float w = w_s[k];
                if (at < 0) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(w, hv[e], acc[e]);
                } else {
                    const uint4 draw = *reinterpret_cast<const uint4*>((const bf*)down + (long long)at * width + c);
                    const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&draw);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __bfloat1622float2(dh[e]);
                        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
                        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
                    }
                }
            }
            uint4 res;
            __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
            for (int e = 0; e < 4; ++e) rh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
            *reinterpret_cast<uint4*>((bf*)y + row * width + c) = res;
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float acc = base != nullptr ? to_f<T>(base[row * width + c]) : 0.f;
            const float hv = to_f<T>(h[row * width + c]);
            for (int k = 0; k < top; ++k) {
                const int at = place_s[k];
                acc = fmaf(w_s[k], at < 0 ? hv : to_f<T>(down[(long long)at * width + c]), acc);
            }
            y[row * width + c] = from_f<T>(acc);
        }
    }
}

extern "C" {

int sb_moe_route(int dtype, const void* h, const float* router, const float* correction, const float* bias, int over_chosen,
                 float* logits, int* chosen, float* weight, int rows, int width, int n_out, int top, float scale,
                 cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (n_out < 1 || n_out > MOE_MAX_OUTPUTS || top < 1 || top > MOE_MAX_TOP || top > n_out) return (int)cudaErrorInvalidValue;
    int R = rows >= 1024 ? 8 : (rows >= 256 ? 4 : (rows >= 64 ? 2 : 1));
    while (R > 1 && (size_t)R * width * sizeof(float) > 96 * 1024) R >>= 1;
    const size_t smem = (size_t)R * width * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    // one row per block: the router's rows are spread over blocks of eight; several rows: a block stages them once and
    // its warps walk all the router's rows
    dim3 grid((unsigned int)((rows + R - 1) / R), R == 1 ? (unsigned int)((n_out + 7) / 8) : 1u);
#define SB_ROUTE(T)                                                                                                              \
    do {                                                                                                                         \
        if (smem > 48 * 1024) {                                                                                                  \
            const cudaError_t err = cudaFuncSetAttribute(moe_logits_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (err != cudaSuccess) return (int)err;                                                                             \
        }                                                                                                                        \
        sb_launch(moe_logits_kernel<T>, grid, 256, smem, stream, (const T*)h, router, logits, rows, width, n_out, R);            \
    } while (0)
    if (dtype == SB_F32) SB_ROUTE(float);
    else SB_ROUTE(__nv_bfloat16);
#undef SB_ROUTE
    sb_launch(moe_choose_kernel, (unsigned int)((rows + 7) / 8), 256, (size_t)16 * n_out * sizeof(float), stream, (const float*)logits,
              correction, bias, over_chosen, chosen, weight, rows, n_out, top, scale);
    SB_LAUNCH_CHECK();
}

int sb_moe_sort(const int* chosen, int n_pairs, int n_experts, int* ends, int* slot_of_pair, int* pair_of_slot, cudaStream_t stream) {
    if (n_pairs <= 0 || n_experts <= 0) return 0;
    if (n_experts > 8192) return (int)cudaErrorInvalidValue;
    sb_launch(moe_sort_kernel, 1, 1024, (size_t)n_experts * sizeof(int), stream, chosen, n_pairs, n_experts, ends, slot_of_pair,
              pair_of_slot);
    SB_LAUNCH_CHECK();
}

int sb_moe_gather(int dtype, const void* h, const int* pair_of_slot, const int* ends, int n_experts, int n_pairs, int top, int width,
                  void* xs, cudaStream_t stream) {
    if (n_pairs <= 0 || n_experts <= 0) return 0;
    const int threads = width >= 1024 ? 256 : 128;
    if (dtype == SB_F32)
        sb_launch(moe_gather_kernel<float>, n_pairs, threads, 0, stream, (const float*)h, pair_of_slot, ends, n_experts, top, width,
                  (float*)xs);
    else
        sb_launch(moe_gather_kernel<__nv_bfloat16>, n_pairs, threads, 0, stream, (const __nv_bfloat16*)h, pair_of_slot, ends, n_experts,
                  top, width, (__nv_bfloat16*)xs);
    SB_LAUNCH_CHECK();
}

int sb_moe_pairs(int dtype, const void* h, const int* chosen, const void* w_gate_up, const void* w_down, void* act, void* down,
                 int n_pairs, int top, int n_experts, int width, int ff, float alpha, float limit, int silu, cudaStream_t stream) {
    if (n_pairs <= 0 || n_experts <= 0) return 0;
    const int threads = 256, warps = threads / 32;
    // enough blocks along the columns for a few per SM when the pairs are few
    const int want = n_pairs >= 1184 ? 1 : (1184 + n_pairs - 1) / n_pairs;   // eight blocks of eight warps per SM
    dim3 g1(n_pairs, (unsigned int)max(1, min(want, (ff + warps - 1) / warps)));
    dim3 g2(n_pairs, (unsigned int)max(1, min(want, (width + 2 * warps - 1) / (2 * warps))));
    const size_t s1 = (size_t)width * sizeof(float), s2 = (size_t)ff * sizeof(float);
    if (s1 > 200 * 1024 || s2 > 200 * 1024) return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf;
#define SB_PAIRS(T)                                                                                                              \
    do {                                                                                                                         \
        if (s1 > 48 * 1024) cudaFuncSetAttribute(moe_pair_gate_up_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1); \
        if (s2 > 48 * 1024) cudaFuncSetAttribute(moe_pair_down_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s2);   \
        sb_launch(moe_pair_gate_up_kernel<T>, g1, threads, s1, stream, (const T*)h, chosen, (const T*)w_gate_up, (T*)act, top,     \
                  n_experts, width, ff, alpha, limit, silu);                                                                         \
        sb_launch(moe_pair_down_kernel<T>, g2, threads, s2, stream, (const T*)act, chosen, (const T*)w_down, (T*)down, n_experts,  \
                  width, ff);                                                                                                    \
    } while (0)
    if (dtype == SB_F32) SB_PAIRS(float);
    else SB_PAIRS(bf);
#undef SB_PAIRS
    SB_LAUNCH_CHECK();
}

int sb_moe_combine(int dtype, const void* h, const void* down, const void* base, const int* chosen, const float* weight,
                   const int* slot_of_pair, void* y, int rows, int top, int n_experts, int width, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP) return (int)cudaErrorInvalidValue;
    typedef __nv_bfloat16 bf;
    if (dtype == SB_F32)
        sb_launch(moe_combine_kernel<float, false>, rows, width >= 1024 ? 256 : 128, 0, stream, (const float*)h, (const float*)down,
                  (const float*)base, chosen, weight, slot_of_pair, (float*)y, top, n_experts, width);
    else if (width % 8 == 0)
        sb_launch(moe_combine_kernel<bf, true>, rows, width >= 2048 ? 256 : (width >= 1024 ? 128 : 64), 0, stream, (const bf*)h,
                  (const bf*)down, (const bf*)base, chosen, weight, slot_of_pair, (bf*)y, top, n_experts, width);
    else
        sb_launch(moe_combine_kernel<bf, false>, rows, width >= 1024 ? 256 : 128, 0, stream, (const bf*)h, (const bf*)down,
                  (const bf*)base, chosen, weight, slot_of_pair, (bf*)y, top, n_experts, width);
    SB_LAUNCH_CHECK();
}

}  // extern "C"
