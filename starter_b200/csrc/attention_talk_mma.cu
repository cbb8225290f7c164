// The attention of attention_talk.cu on the tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit sums), for the
// rows of prompts.
//
// A row's scores of ALL heads against a key meet in the table before any head's softmax can go on, so a block owns
// 16 consecutive positions of one sequence with all their heads; a warp owns HPW heads.  Keys and values come TK at
// a time (a part of one page), for all key/value heads, through cp.async; rows of a tile that no row of the block
// sees are filled with zeros instead of being read.  Per tile:
//
//   1. every warp multiplies its heads' 16 query rows with the tile's keys of their key/value head, scales and caps
//      the scores (32-bit; tanh through exp) and leaves them in shared memory, [head][row][key];
//   2. every thread takes (row, key) pairs of the tile and forms ALL heads' mixed scores t_h = sum_g T[h, g] s_g of its
//      pairs in place (32-bit fused multiply-adds in the order g = 0, 1, ..., two heads per instruction: this is the
//      part the tensor cores cannot take without rounding the scores), so that a score is read once, not once per head;
//   3. every warp masks its heads' mixed scores and goes on with their running maximum, exponentials and sums; a
//      weight meets its value as two bfloat16 numbers hi + lo, so that it keeps 16 bits.
//
// The next tile's keys are fetched while steps 2 and 3 run, the next values (two buffers) as well.  A tile that every row of
// the block sees whole skips the mask.  With n_splits > 1 neighbouring blocks take a share each of the 16 positions'
// tiles (the positions with the most tiles first, all their shares together) and leave, per row and head, their
// unnormalised value sums, maximum and sum in ``partial`` [row][head][split][V + 2]; the merge kernel
// of attention_talk.cu adds the sink and divides.
#include "attention_flex.cuh"
#include "mma_utils.cuh"

#define TM_ROWS 16

// attention_talk.cu: the splits' sums of every (row, head) scaled to their common maximum (the sink's too), added and divided.
void sb_talking_merge_bf16(const float* partial, void* out, const float* sink, int n_rows, int n_heads, int n_splits, int v_dim,
                           cudaStream_t stream);

__device__ __forceinline__ void talk_cp_or_zero(void* smem_dst, const void* gmem_src, bool real) {
    const unsigned int s = (unsigned int)__cvta_generic_to_shared(smem_dst);
    const int n = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem_src), "r"(n));
}

// cap * tanh(x / cap) with tanh(y) = 1 - 2 / (exp(2 y) + 1): exp overflows to infinity and underflows to zero at the
// right ends, and the absolute error stays near 1e-7 * cap.
__device__ __forceinline__ float talk_cap(float x, float cap, float two_over_cap) {
    const float e = __expf(x * two_over_cap);
    return cap * (1.f - __fdividef(2.f, e + 1.f));
}

template <int VD, int HPW, int TK, int THREADS, int HMAX>
__global__ void __launch_bounds__(THREADS)
talking_attention_mma_kernel(SbFlex p, SbBatch batch, __nv_bfloat16* __restrict__ out, int tiles_per_seq, int n_splits,
                             float* __restrict__ partial) {
    typedef __nv_bfloat16 bf;
    constexpr int NT = VD / 8, JT = TK / 8, SLD = TK + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = p.n_heads, G = p.n_kv_heads, KD = p.k_dim, per_kv = H / G;
    const int kld = KD + 8, vld = VD + 8;
    bf* Qs = reinterpret_cast<bf*>(smem_raw);                         // [H][16][kld]
    bf* Ks = Qs + (size_t)H * TM_ROWS * kld;                          // [G][TK][kld]
    bf* Vs = Ks + (size_t)G * TK * kld;                               // [2][G][TK][vld]
    float* Ss = reinterpret_cast<float*>(Vs + (size_t)2 * G * TK * vld);   // [H][16][SLD]
    float* Tt = Ss + (size_t)H * TM_ROWS * SLD;                       // [H][HMAX]: Tt[g][h] = T[h][g], zeros beyond H

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g8 = lane >> 2, t4 = lane & 3;
    const int split = blockIdx.x % n_splits, bx = blockIdx.x / n_splits;
    const int s = bx / tiles_per_seq, tile = tiles_per_seq - 1 - bx % tiles_per_seq;
    if (p.talk != nullptr)
        for (int e = tid; e < H * HMAX; e += blockDim.x) {
            const int g = e / HMAX, h = e % HMAX;
            Tt[e] = h < H ? p.talk[h * H + g] : 0.f;
        }
    pdl_wait();
    const int slot = batch.seq_slot[s], q0 = batch.cu_q[s], nq = batch.cu_q[s + 1] - q0;
    const int first = tile * TM_ROWS;
    if (first >= nq) return;
    const int n_here = min(TM_ROWS, nq - first);
    const int pos_first = batch.lengths[slot] + first, pos_last = pos_first + n_here - 1;
    const int lo_blk = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int kept_blk = min(p.keep_first, lo_blk);       // kept first keys that the block's window does not hold anyway
    const int ta_end = (kept_blk + TK - 1) / TK;
    const int tb_start = max(lo_blk / TK, ta_end), tb_end = pos_last / TK;
    const int n_tiles = ta_end + (tb_end - tb_start + 1);
    const int per_split = (n_tiles + n_splits - 1) / n_splits;
    const int it_lo = split * per_split, it_hi = min(n_tiles, it_lo + per_split);

    {   // the queries of all heads
        const int cpr = KD / 8;
        for (int c = tid; c < H * TM_ROWS * cpr; c += blockDim.x) {
            const int hr = c / cpr, cc = c % cpr, h = hr / TM_ROWS, r = hr % TM_ROWS;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (r < n_here)
                val = *reinterpret_cast<const uint4*>((const bf*)p.q + (long long)(q0 + first + r) * p.q_row + (long long)h * p.q_head + cc * 8);
            *reinterpret_cast<uint4*>(Qs + (size_t)hr * kld + cc * 8) = val;
        }
    }
    auto tile_start = [&](int it) { return (it < ta_end ? it : tb_start + it - ta_end) * TK; };
    auto tile_page = [&](int n0) {
        const int lp = flex_table_column(p, n0 / SB_PAGE);
        return lp < p.table_width ? p.table[(long long)slot * p.table_width + lp] : -1;
    };
    auto block_sees = [&](int key) { return key < kept_blk || (key >= lo_blk && key <= pos_last); };
    // A thread fetches the same 16 bytes of a row in every pass: column cc of a power-of-two count per row, rows
    // cr0, cr0 + rows_per_pass, ... of the tile's [G][TK] rows.
    const int kshift = 32 - __clz(max(KD / 8, 1) - 1), k_cc = tid & ((1 << kshift) - 1), k_cr0 = tid >> kshift;
    const int k_pass = max(1, (int)blockDim.x >> kshift);
    constexpr int vshift = VD == 64 ? 3 : 4;
    const int v_cc = tid & ((1 << vshift) - 1), v_cr0 = tid >> vshift, v_pass = max(1, (int)blockDim.x >> vshift);
    auto load_keys = [&](int it) {
        const int n0 = tile_start(it), page = tile_page(n0);
        if (k_cc * 8 >= KD || k_cr0 >= G * TK) return;
        const long long base = (long long)(page < 0 ? 0 : page) * G * SB_PAGE + (n0 % SB_PAGE);
        for (int cr = k_cr0; cr < G * TK; cr += k_pass) {
            const int kv = cr / TK, r = cr % TK;
            talk_cp_or_zero(Ks + (size_t)cr * kld + k_cc * 8, (const bf*)p.k + (base + kv * SB_PAGE + r) * KD + k_cc * 8,
                            page >= 0 && block_sees(n0 + r));
        }
    };
    auto load_values = [&](int it) {
        const int n0 = tile_start(it), page = tile_page(n0);
        if (v_cr0 >= G * TK) return;
        bf* dst = Vs + (size_t)(it & 1) * G * TK * vld;
        const long long base = (long long)(page < 0 ? 0 : page) * G * SB_PAGE + (n0 % SB_PAGE);
        for (int cr = v_cr0; cr < G * TK; cr += v_pass) {
            const int kv = cr / TK, r = cr % TK;
            talk_cp_or_zero(dst + (size_t)cr * vld + v_cc * 8, (const bf*)p.v + (base + kv * SB_PAGE + r) * p.v_row + v_cc * 8,
                            page >= 0 && block_sees(n0 + r));
        }
    };

    // this thread's two rows (g8 and g8 + 8) and its warp's heads
    const int r_pos[2] = {pos_first + g8, pos_first + g8 + 8};
    const bool r_valid[2] = {g8 < n_here, g8 + 8 < n_here};
    int r_lo[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) r_lo[half] = p.window > 0 ? max(0, r_pos[half] - p.window + 1) : 0;
    const int h0 = w * HPW;
    float m_run[HPW][2], l_run[HPW][2], acc[HPW][NT][4];
#pragma unroll
    for (int hi = 0; hi < HPW; ++hi) {
        m_run[hi][0] = m_run[hi][1] = -INFINITY;
        l_run[hi][0] = l_run[hi][1] = 0.f;
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[hi][i][e] = 0.f;
    }
    const float cap = p.softcap, two_over_cap = cap > 0.f ? 2.f / cap : 0.f;
    const int lo_last = p.window > 0 ? max(0, pos_last - p.window + 1) : 0;     // the last row's window starts here

    if (it_lo < it_hi) {
        load_keys(it_lo);
        load_values(it_lo);
    }
    cp_async_commit();
    for (int it = it_lo; it < it_hi; ++it) {
        const int n0 = tile_start(it);
        // every row of the block sees every key of this tile: nothing to mask
        const bool whole = n_here == TM_ROWS && n0 + TK - 1 <= pos_first && (n0 >= lo_last || n0 + TK <= p.keep_first);
        cp_async_wait<0>();
        __syncthreads();             // this tile's keys and values are here; everyone has left the last tile's scores
        // 1. scores of this warp's heads
#pragma unroll
        for (int hi = 0; hi < HPW; ++hi) {
            const int h = h0 + hi;
            if (h >= H) break;
            float sacc[JT][4];
#pragma unroll
            for (int i = 0; i < JT; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[i][e] = 0.f;
            const bf* qa = Qs + ((size_t)h * TM_ROWS + (lane & 15)) * kld + (lane >> 4) * 8;
            const bf* kb = Ks + ((size_t)(h / per_kv) * TK + (lane & 7) + (lane >> 4) * 8) * kld + ((lane >> 3) & 1) * 8;
            for (int k0 = 0; k0 < KD; k0 += 16) {
                unsigned int a[4];
                ldmatrix_x4(a, qa + k0);
#pragma unroll
                for (int i = 0; i < JT; i += 2) {
                    unsigned int b[4];
                    ldmatrix_x4(b, kb + (size_t)i * 8 * kld + k0);
                    mma_bf16(sacc[i], a, b[0], b[1]);
                    mma_bf16(sacc[i + 1], a, b[2], b[3]);
                }
            }
            float* srow = Ss + ((size_t)h * TM_ROWS + g8) * SLD + 2 * t4;
#pragma unroll
            for (int i = 0; i < JT; ++i) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    v[e] = sacc[i][e] * p.scale;
                    if (cap > 0.f) v[e] = talk_cap(v[e], cap, two_over_cap);
                }
                *reinterpret_cast<float2*>(srow + i * 8) = make_float2(v[0], v[1]);
                *reinterpret_cast<float2*>(srow + 8 * SLD + i * 8) = make_float2(v[2], v[3]);
            }
        }
        __syncthreads();             // all heads' scores are in place; nobody reads the keys any more
        if (it + 1 < it_hi) {
            load_keys(it + 1);
            load_values(it + 1);
            cp_async_commit();
        }
        // 2. the table: a pair's scores of all heads, read once, become its mixed scores of all heads, in place
        if (p.talk != nullptr) {
            // an item: a pair and 16 of the heads' mixed scores; with more than 16 heads a pair's two items read all its
            // scores before either writes
            constexpr int PARTS = HMAX / 16, ITEMS = TM_ROWS * TK * PARTS;
            for (int base = 0; base < ITEMS; base += blockDim.x) {
                const int item = base + tid, pr = item / PARTS, h_first = (item % PARTS) * 16;
                const bool on = item < ITEMS;
                float* col = Ss + (pr / TK) * SLD + (pr % TK);
                float2 mixed[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) mixed[c] = make_float2(0.f, 0.f);
                if (on) {
#pragma unroll 4
                    for (int g = 0; g < H; ++g) {
                        const float sg = col[(size_t)g * TM_ROWS * SLD];
                        const float2 s2 = make_float2(sg, sg);
                        const float4* tw = reinterpret_cast<const float4*>(Tt + g * HMAX + h_first);
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (h_first + 4 * c < H) {
                                const float4 w4 = tw[c];
                                mixed[2 * c] = fma_pair(make_float2(w4.x, w4.y), s2, mixed[2 * c]);
                                mixed[2 * c + 1] = fma_pair(make_float2(w4.z, w4.w), s2, mixed[2 * c + 1]);
                            }
                    }
                }
                if (PARTS > 1) __syncthreads();
                if (on) {
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        if (h_first + 2 * c < H) col[(size_t)(h_first + 2 * c) * TM_ROWS * SLD] = mixed[c].x;
                        if (h_first + 2 * c + 1 < H) col[(size_t)(h_first + 2 * c + 1) * TM_ROWS * SLD] = mixed[c].y;
                    }
                }
            }
            __syncthreads();         // every head's mixed scores are in place
        }
        if (h0 >= H) continue;
        // 3. the mask, the softmax's bookkeeping
        float t[HPW][JT][4];
#pragma unroll
        for (int hi = 0; hi < HPW; ++hi) {
            const float* srow = Ss + ((size_t)min(h0 + hi, H - 1) * TM_ROWS + g8) * SLD + 2 * t4;
#pragma unroll
            for (int i = 0; i < JT; ++i) {
                const float2 top = *reinterpret_cast<const float2*>(srow + i * 8);
                const float2 bot = *reinterpret_cast<const float2*>(srow + 8 * SLD + i * 8);
                t[hi][i][0] = top.x, t[hi][i][1] = top.y, t[hi][i][2] = bot.x, t[hi][i][3] = bot.y;
            }
        }
        const bf* Vb = Vs + (size_t)(it & 1) * G * TK * vld;
#pragma unroll
        for (int hi = 0; hi < HPW; ++hi) {
            const int h = h0 + hi;
            if (h >= H) break;
            float mx[2] = {-INFINITY, -INFINITY};
            if (whole) {
#pragma unroll
                for (int i = 0; i < JT; ++i)
#pragma unroll
                    for (int half = 0; half < 2; ++half)
                        mx[half] = max_of_three(mx[half], t[hi][i][2 * half], t[hi][i][2 * half + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < JT; ++i)
#pragma unroll
                    for (int half = 0; half < 2; ++half)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int n = n0 + 8 * i + 2 * t4 + e;
                            const bool seen = r_valid[half] && n <= r_pos[half] && (n >= r_lo[half] || n < p.keep_first);
                            const float sc = seen ? t[hi][i][2 * half + e] : -INFINITY;
                            t[hi][i][2 * half + e] = sc;
                            mx[half] = fmaxf(mx[half], sc);
                        }
            }
            float alpha[2], m_new[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
                mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
                m_new[half] = fmaxf(m_run[hi][half], mx[half]);
                alpha[half] = m_new[half] == -INFINITY ? 1.f : __expf(m_run[hi][half] - m_new[half]);
            }
#pragma unroll
            for (int i = 0; i < JT; ++i)
#pragma unroll
                for (int half = 0; half < 2; ++half)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float wv = m_new[half] == -INFINITY ? 0.f : __expf(t[hi][i][2 * half + e] - m_new[half]);
                        t[hi][i][2 * half + e] = wv;
                        sum[half] += wv;
                    }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                sum[half] += __shfl_xor_sync(0xffffffffu, sum[half], 1);
                sum[half] += __shfl_xor_sync(0xffffffffu, sum[half], 2);
                l_run[hi][half] = l_run[hi][half] * alpha[half] + sum[half];
                m_run[hi][half] = m_new[half];
            }
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[hi][i][0] *= alpha[0];
                acc[hi][i][1] *= alpha[0];
                acc[hi][i][2] *= alpha[1];
                acc[hi][i][3] *= alpha[1];
            }
            const bf* vb = Vb + ((size_t)(h / per_kv) * TK + (lane & 7) + ((lane >> 3) & 1) * 8) * vld + (lane >> 4) * 8;
#pragma unroll
            for (int kk = 0; kk < TK / 16; ++kk) {
                unsigned int ah[4], al[4];
#pragma unroll
                for (int part = 0; part < 4; ++part) {
                    const float w0 = t[hi][2 * kk + (part >> 1)][2 * (part & 1)], w1 = t[hi][2 * kk + (part >> 1)][2 * (part & 1) + 1];
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(w0, w1);
                    const float2 back = __bfloat1622float2(h2);
                    ah[part] = *reinterpret_cast<const unsigned int*>(&h2);
                    al[part] = pack_bf16(w0 - back.x, w1 - back.y);
                }
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    unsigned int b[4];
                    ldmatrix_x4_trans(b, vb + (size_t)kk * 16 * vld + i * 8);
                    mma_bf16(acc[hi][i], ah, b[0], b[1]);
                    mma_bf16(acc[hi][i], al, b[0], b[1]);
                    mma_bf16(acc[hi][i + 1], ah, b[2], b[3]);
                    mma_bf16(acc[hi][i + 1], al, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int hi = 0; hi < HPW; ++hi) {
        const int h = h0 + hi;
        if (h >= H) break;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (!r_valid[half]) continue;
            const long long row = q0 + first + g8 + 8 * half;
            if (n_splits > 1) {
                float* dst = partial + ((row * H + h) * n_splits + split) * (VD + 2);
#pragma unroll
                for (int i = 0; i < NT; ++i)
                    *reinterpret_cast<float2*>(dst + i * 8 + 2 * t4) = make_float2(acc[hi][i][2 * half], acc[hi][i][2 * half + 1]);
                if (t4 == 0) {
                    dst[VD] = m_run[hi][half];
                    dst[VD + 1] = l_run[hi][half];
                }
                continue;
            }
            float a = 1.f, l = l_run[hi][half];
            if (p.sink != nullptr) {   // one more term in the denominator, no value behind it
                const float sk = p.sink[h], mf = fmaxf(m_run[hi][half], sk);
                a = expf(m_run[hi][half] - mf);
                l = l * a + expf(sk - mf);
            }
            const float mul = a / l;
            bf* o = out + (row * H + h) * VD;
#pragma unroll
            for (int i = 0; i < NT; ++i)
                *reinterpret_cast<__nv_bfloat162*>(o + i * 8 + 2 * t4) =
                    __floats2bfloat162_rn(acc[hi][i][2 * half] * mul, acc[hi][i][2 * half + 1] * mul);
        }
    }
}

static long long talk_mma_smem(int H, int G, int KD, int VD, int HPW, int TK) {
    return ((long long)H * TM_ROWS * (KD + 8) + (long long)G * TK * (KD + 8) + 2ll * G * TK * (VD + 8)) * 2
           + ((long long)H * TM_ROWS * (TK + 8) + (long long)H * (H <= 16 ? 16 : 32)) * 4;
}

// Heads per warp and keys per tile for these sizes (0, 0 when the kernel does not take them): one head per warp up to
// 16 heads, two up to 32 (a warp's value sums fill HPW * VD / 2 registers per thread, and 16 warps leave a thread 128
// registers), and 32 keys at a time where the registers and the shared memory hold them, else 16.
static void talk_mma_shape(int H, int G, int KD, int VD, int& HPW, int& TK) {
    HPW = TK = 0;
    if (H < 1 || G < 1 || H % G || KD < 16 || KD % 16 || KD > 256 || (VD != 64 && VD != 128)) return;
    const int hpw = H <= 16 ? 1 : H <= 32 && VD == 64 ? 2 : 0;
    if (!hpw) return;
    for (int tk = hpw == 2 ? 16 : 32; tk >= 16; tk /= 2)
        if (talk_mma_smem(H, G, KD, VD, hpw, tk) <= 227 * 1024) {
            HPW = hpw;
            TK = tk;
            return;
        }
}

template <int VD, int HPW, int TK, int THREADS, int HMAX>
static int launch_talk_mma(SbFlex p, SbBatch batch, void* out, int max_q_len, int n_splits, float* partial, cudaStream_t stream) {
    const long long smem = talk_mma_smem(p.n_heads, p.n_kv_heads, p.k_dim, VD, HPW, TK);
    static long long allowed = 48 * 1024;
    if (smem > allowed) {
        const cudaError_t e = cudaFuncSetAttribute(talking_attention_mma_kernel<VD, HPW, TK, THREADS, HMAX>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    const int tiles = (max_q_len + TM_ROWS - 1) / TM_ROWS, n_warps = (p.n_heads + HPW - 1) / HPW;
    sb_launch(talking_attention_mma_kernel<VD, HPW, TK, THREADS, HMAX>, dim3((unsigned int)(batch.n_seqs * tiles * n_splits)), 32 * n_warps,
              (size_t)smem, stream, p, batch, (__nv_bfloat16*)out, tiles, n_splits, partial);
    if (n_splits > 1) sb_talking_merge_bf16(partial, out, p.sink, batch.n_rows, p.n_heads, n_splits, VD, stream);
    SB_LAUNCH_CHECK();
}

extern "C" {

// Bytes of shared memory the tensor-core kernel asks for, or -1 when it does not take these sizes.
long long sb_talking_attention_mma_smem(int n_heads, int n_kv_heads, int k_dim, int v_dim) {
    int HPW, TK;
    talk_mma_shape(n_heads, n_kv_heads, k_dim, v_dim, HPW, TK);
    return HPW ? talk_mma_smem(n_heads, n_kv_heads, k_dim, v_dim, HPW, TK) : -1;
}

int sb_talking_attention_mma(SbFlex p, SbBatch batch, void* out, int max_q_len, int n_splits, float* partial, cudaStream_t stream) {
    if (batch.n_rows <= 0) return 0;
    if (p.v_heads > 0 && p.v_heads != p.n_kv_heads) return (int)cudaErrorInvalidValue;
    if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && partial == nullptr)) return (int)cudaErrorInvalidValue;
    int HPW, TK;
    talk_mma_shape(p.n_heads, p.n_kv_heads, p.k_dim, p.v_dim, HPW, TK);
    const int threads = p.n_heads > 8 * HPW ? 512 : 256;
#define SB_TALK_MMA(V, W, K, T) \
    if (p.v_dim == V && HPW == W && TK == K && threads == T) \
        return launch_talk_mma<V, W, K, T, 16 * W>(p, batch, out, max_q_len, n_splits, partial, stream)
    SB_TALK_MMA(64, 1, 32, 256);
    SB_TALK_MMA(64, 1, 16, 256);
    SB_TALK_MMA(64, 1, 32, 512);
    SB_TALK_MMA(64, 1, 16, 512);
    SB_TALK_MMA(64, 2, 16, 512);
    SB_TALK_MMA(128, 1, 32, 256);
    SB_TALK_MMA(128, 1, 16, 256);
    SB_TALK_MMA(128, 1, 32, 512);
    SB_TALK_MMA(128, 1, 16, 512);
#undef SB_TALK_MMA
    return (int)cudaErrorInvalidValue;
}

}  // extern "C"
