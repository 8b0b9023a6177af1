// Paged causal softmax attention whose weights are mixed across heads before they meet the
// values, with keys and values of different widths:
//
//   p_g(i, j) = softmax_j(q_g(i) . k_kv(g)(j) * scale)        per query head g, float32
//   w_h(i, j) = sum_g M[h][g] p_g(i, j)                       M is [H, H], float32
//   out_h(i)  = sum_j w_h(i, j) v_kv(h)(j)
//
// (M null: w = p, plain grouped-query attention.) Because the mix needs every head's
// finished softmax, a query is done in two passes over its keys: the first finds each head's
// maximum and sum, the second makes the normalised weights 32 keys at a time, mixes them and
// adds the values in. Keys are taken 32 at a time from the window's start, so the order of
// every sum depends on the position alone and a position's result is bit-identical however
// the tokens were cut into steps or batched.
//
// Cache planes of one layer: keys [page][kv head][offset][dk], values [page][kv head][offset][dv].
#include "mma_sync.cuh"

#define AM_WARPS 8
#define AM_MAX_H 64

// One block per token: the generic form, any storage type and any sizes (H <= 64).
// Shared memory: q [H][dk], M [H][H], p [H][32], acc [H][dv], all float32.
template <typename T>
__global__ void __launch_bounds__(AM_WARPS * 32)
attention_mixed_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                       long long out_stride, int H, int Hkv, int dk, int dv,
                       const T* __restrict__ k_cache, const T* __restrict__ v_cache, int page_size,
                       const int* __restrict__ block_tables, int max_blocks,
                       const int* __restrict__ seq_ids, const int* __restrict__ positions,
                       const float* __restrict__ mix, float scale, int window) {
    extern __shared__ float smem[];
    float* qs = smem;                       // [H][dk]
    float* ms = qs + (size_t)H * dk;        // [H][H]
    float* ps = ms + (size_t)H * H;         // [H][32]
    float* acc = ps + (size_t)H * 32;       // [H][dv]
    __shared__ float stat_m[AM_MAX_H], stat_r[AM_MAX_H];
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int p = positions[t];
    T* o = out + (size_t)t * out_stride;
    if (p < 0) {                            // a padded row: no keys, zeros out
        for (int i = threadIdx.x; i < H * dv; i += blockDim.x) o[i] = from_f32<T>(0.f);
        return;
    }
    const int b = seq_ids[t];
    const int group = H / Hkv;
    const int* bt = block_tables + (size_t)b * max_blocks;
    const T* qv = q + (size_t)t * q_stride;
    for (int i = threadIdx.x; i < H * dk; i += blockDim.x) qs[i] = to_f32(qv[i]);
    for (int i = threadIdx.x; i < H * H; i += blockDim.x)
        ms[i] = mix ? mix[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    for (int i = threadIdx.x; i < H * dv; i += blockDim.x) acc[i] = 0.f;
    __syncthreads();
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;

    // pass 1: each head's maximum and sum of exponentials (a warp owns heads warp, warp+8, ..)
    for (int h = warp; h < H; h += AM_WARPS) {
        const int kvh = h / group;
        const float* qh = qs + (size_t)h * dk;
        float m = -INFINITY, l = 0.f;
        for (int base = lo; base <= p; base += 32) {
            const int j = base + lane;
            float s = -INFINITY;
            if (j <= p) {
                const int page = bt[j / page_size];
                const T* kr = k_cache + (((size_t)page * Hkv + kvh) * page_size + (j % page_size)) * dk;
                float a = 0.f;
                for (int d = 0; d < dk; ++d) a += qh[d] * to_f32(kr[d]);
                s = a * scale;
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float w = j <= p ? expf(s - m_new) : 0.f;
            l = l * expf(m - m_new) + warp_sum(w);
            m = m_new;
        }
        if (lane == 0) {
            stat_m[h] = m;
            stat_r[h] = 1.f / l;
        }
    }
    __syncthreads();

    // pass 2: normalised weights of 32 keys, mixed across heads, times the values
    for (int base = lo; base <= p; base += 32) {
        const int j = base + lane;
        const int nvalid = (p - base + 1) < 32 ? (p - base + 1) : 32;
        for (int h = warp; h < H; h += AM_WARPS) {
            const int kvh = h / group;
            const float* qh = qs + (size_t)h * dk;
            float w = 0.f;
            if (j <= p) {
                const int page = bt[j / page_size];
                const T* kr = k_cache + (((size_t)page * Hkv + kvh) * page_size + (j % page_size)) * dk;
                float a = 0.f;
                for (int d = 0; d < dk; ++d) a += qh[d] * to_f32(kr[d]);
                w = expf(a * scale - stat_m[h]) * stat_r[h];
            }
            ps[h * 32 + lane] = w;
        }
        __syncthreads();
        for (int h = warp; h < H; h += AM_WARPS) {
            const int kvh = h / group;
            float w = 0.f;
            for (int g = 0; g < H; ++g) w += ms[h * H + g] * ps[g * 32 + lane];
            for (int c0 = 0; c0 < dv; c0 += 32) {
                const int c = c0 + lane;
                float a = 0.f;
                for (int jj = 0; jj < nvalid; ++jj) {
                    const float wj = __shfl_sync(0xffffffffu, w, jj);
                    const int kj = base + jj;
                    const int page = bt[kj / page_size];
                    const T* vr = v_cache + (((size_t)page * Hkv + kvh) * page_size + (kj % page_size)) * dv;
                    if (c < dv) a += wj * to_f32(vr[c]);
                }
                if (c < dv) acc[(size_t)h * dv + c] += a;
            }
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < H * dv; i += blockDim.x) o[i] = from_f32<T>(acc[i]);
}

TGO_API int tgo_attention_mixed(const void* q, long long q_stride, void* out, long long out_stride,
                                int dtype, int T, int H, int Hkv, int dk, int dv,
                                const void* k_cache, const void* v_cache, int page_size,
                                const int* block_tables, int max_blocks, const int* seq_ids,
                                const int* positions, const float* mix, float scale, int window,
                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dk <= 0 || dv <= 0 || H <= 0 || H > AM_MAX_H || Hkv <= 0 || H % Hkv || page_size <= 0 ||
        max_blocks <= 0 || window < 0)
        return TGO_E_BAD_ARG;
    const size_t smem = ((size_t)H * dk + (size_t)H * H + (size_t)H * 32 + (size_t)H * dv) * sizeof(float);
    if (smem > 200 * 1024) return TGO_E_BAD_ARG;
    const dim3 grid(T), block(AM_WARPS * 32);
    if (dtype == TGO_BF16) {
        auto kern = attention_mixed_kernel<bf16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, grid, block, smem, stream, (const bf16*)q, q_stride, (bf16*)out,
                              out_stride, H, Hkv, dk, dv, (const bf16*)k_cache, (const bf16*)v_cache,
                              page_size, block_tables, max_blocks, seq_ids, positions, mix, scale, window);
    }
    if (dtype == TGO_F32) {
        auto kern = attention_mixed_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, grid, block, smem, stream, (const float*)q, q_stride, (float*)out,
                              out_stride, H, Hkv, dk, dv, (const float*)k_cache, (const float*)v_cache,
                              page_size, block_tables, max_blocks, seq_ids, positions, mix, scale, window);
    }
    return TGO_E_BAD_ARG;
}

// ------------------------------------------------------------------ prompt portions, bfloat16
// One block per tile of up to 16 consecutive tokens of one request, all heads: Q K^T and
// W V on the tensor cores (mma.sync m16n8k16, float32 accumulators), softmax and the mix of
// the heads in float32 registers. A warp owns a head (eight warps up to eight heads, sixteen
// up to sixteen).
//
//   pass 1   keys in blocks of 32: each warp makes its heads' scores and keeps, per query
//            row, the running maximum and sum (in registers, to the end of the kernel);
//   pass 2   the same scores again, now normalised: p = exp(s - m) / l goes to shared memory
//            [head][row][key] as float32; after a barrier each warp mixes, for its OUTPUT
//            heads, the 16 x 16 weights it needs straight into the A operand of the second
//            product (w_h = sum_g M[h][g] p_g, rounded to bfloat16 there) and multiplies by
//            the 32 values of its kv head (their operand comes out of shared memory
//            transposed, by ldmatrix). Keys and values reach shared memory by 16-byte
//            asynchronous copies.
//
// Blocks of keys start at multiples of 32 from key 0, so the sums' order depends on the
// position alone. Needs dk % 16 == 0, dv % 8 == 0, dv <= 128, H <= 16, no window.
#define AT_KB 32
#define AT_PS 40                  // floats per row of the weights in shared memory

// 2^x by the special-function unit (float32 in and out, about two units in the last place);
// 2^(-inf) = 0
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct MixedTileSmem {
    int qs, ks, vs, ps;           // offsets in bytes
    size_t total;
};
static inline MixedTileSmem mixed_tile_smem(int H, int G, int dk, int dv) {
    MixedTileSmem m;
    size_t o = 0;
    m.qs = (int)o; o += (size_t)16 * (H * dk + 8) * 2;
    m.ks = (int)o; o += (size_t)G * AT_KB * (dk + 8) * 2;
    m.vs = (int)o; o += (size_t)G * AT_KB * (dv + 8) * 2;
    o = (o + 15) / 16 * 16;
    m.ps = (int)o; o += (size_t)H * 16 * AT_PS * 4;
    m.total = o;
    return m;
}

template <int NW, int HPW, int NT>
__global__ void __launch_bounds__(NW * 32)
attention_mixed_tile_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                            long long out_stride, int H, int G, int dk, int dv,
                            const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                            int page_size, const int* __restrict__ block_tables, int max_blocks,
                            const int* __restrict__ seq_ids, const int* __restrict__ positions,
                            const float* __restrict__ mix, float scale,
                            const int* __restrict__ tile_tok0, const int* __restrict__ tile_ntok,
                            int off_k, int off_v, int off_p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = (bf16*)smem_raw;
    bf16* Ks = (bf16*)(smem_raw + off_k);
    bf16* Vt = (bf16*)(smem_raw + off_v);
    float* Ps = (float*)(smem_raw + off_p);
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    // the list's last tiles first: within a request they are the ones with the most keys
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int tok0 = tile_tok0[tile], ntok = tile_ntok[tile];
    const int b = seq_ids[tok0], p0 = positions[tok0];
    const int* bt = block_tables + (size_t)b * max_blocks;
    const int group = H / G;
    const int QS = H * dk + 8, KS = dk + 8, VS = dv + 8;
    const int last_key = p0 + ntok - 1;
    const int nblocks = last_key / AT_KB + 1;
    // positions of this thread's two rows (rows past the tile stand in for its last token)
    const int pos_lo = p0 + (r < ntok ? r : ntok - 1);
    const int pos_hi = p0 + (r + 8 < ntok ? r + 8 : ntok - 1);

    for (int i = threadIdx.x; i < 16 * H * dk; i += blockDim.x) {
        const int row = i / (H * dk), col = i % (H * dk);
        Qs[row * QS + col] = row < ntok ? q[(size_t)(tok0 + row) * q_stride + col] : from_f32<bf16>(0.f);
    }

    // 16-byte asynchronous copies, all of a block's in flight at once (rows past the last key
    // are filled with zeros); the caller waits for them before its barrier
    auto load_keys = [&](int kb) {
        const int chunks = dk / 8;
        for (int i = threadIdx.x; i < G * AT_KB * chunks; i += blockDim.x) {
            const int ch = i % chunks, key = (i / chunks) % AT_KB, g = i / (chunks * AT_KB);
            const int j = kb * AT_KB + key;
            const bool live = j <= last_key;
            const int page = live ? bt[j / page_size] : 0;
            cp_async16(Ks + ((size_t)g * AT_KB + key) * KS + ch * 8,
                       k_cache + (((size_t)page * G + g) * page_size + (live ? j % page_size : 0)) * dk + ch * 8,
                       live);
        }
    };
    auto load_values = [&](int kb) {
        const int chunks = dv / 8;
        for (int i = threadIdx.x; i < G * AT_KB * chunks; i += blockDim.x) {
            const int ch = i % chunks, key = (i / chunks) % AT_KB, g = i / (chunks * AT_KB);
            const int j = kb * AT_KB + key;
            const bool live = j <= last_key;
            const int page = live ? bt[j / page_size] : 0;
            cp_async16(Vt + ((size_t)g * AT_KB + key) * VS + ch * 8,
                       v_cache + (((size_t)page * G + g) * page_size + (live ? j % page_size : 0)) * dv + ch * 8,
                       live);
        }
    };
    // scores of head g against the 32 keys in shared memory: sc[nt][0..3], the accumulator
    // layout (rows r and r + 8, keys nt * 8 + 2c and + 1), times scale * log2(e) (the
    // exponentials below are powers of two, one special-function instruction each), masked
    const float scale2 = scale * 1.4426950408889634f;
    auto scores = [&](int g, int kb, float (&sc)[4][4]) {
        const int kvh = g / group;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) sc[nt][x] = 0.f;
        const bf16* qb = Qs + g * dk;
        const bf16* kbase = Ks + (size_t)kvh * AT_KB * KS;
        for (int ks = 0; ks < dk; ks += 16) {
            uint32_t a[4];
            ldmatrix_x4(a, qb + ((lane & 7) + ((lane >> 3) & 1) * 8) * QS + ks + (lane >> 4) * 8);
#pragma unroll
            for (int np = 0; np < 2; ++np) {                 // two tiles of 8 keys at a time
                uint32_t kf[4];
                ldmatrix_x4(kf, kbase + (np * 16 + (lane & 7) + (lane >> 4) * 8) * KS + ks + ((lane >> 3) & 1) * 8);
                mma_bf16(sc[2 * np], a, kf[0], kf[1]);
                mma_bf16(sc[2 * np + 1], a, kf[2], kf[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int j = kb * AT_KB + nt * 8 + 2 * c;
            sc[nt][0] = j <= pos_lo ? sc[nt][0] * scale2 : -INFINITY;
            sc[nt][1] = j + 1 <= pos_lo ? sc[nt][1] * scale2 : -INFINITY;
            sc[nt][2] = j <= pos_hi ? sc[nt][2] * scale2 : -INFINITY;
            sc[nt][3] = j + 1 <= pos_hi ? sc[nt][3] * scale2 : -INFINITY;
        }
    };

    float m_lo[HPW], m_hi[HPW], l_lo[HPW], l_hi[HPW];
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
        m_lo[s] = m_hi[s] = -INFINITY;
        l_lo[s] = l_hi[s] = 0.f;
    }
    // ---- pass 1
    for (int kb = 0; kb < nblocks; ++kb) {
        __syncthreads();
        load_keys(kb);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int s = 0; s < HPW; ++s) {
            const int g = warp + s * NW;
            if (g >= H) continue;
            float sc[4][4];
            scores(g, kb, sc);
            float blo = -INFINITY, bhi = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                blo = fmaxf(blo, fmaxf(sc[nt][0], sc[nt][1]));
                bhi = fmaxf(bhi, fmaxf(sc[nt][2], sc[nt][3]));
            }
            blo = fmaxf(blo, __shfl_xor_sync(0xffffffffu, blo, 1));
            blo = fmaxf(blo, __shfl_xor_sync(0xffffffffu, blo, 2));
            bhi = fmaxf(bhi, __shfl_xor_sync(0xffffffffu, bhi, 1));
            bhi = fmaxf(bhi, __shfl_xor_sync(0xffffffffu, bhi, 2));
            const float nlo = fmaxf(m_lo[s], blo), nhi = fmaxf(m_hi[s], bhi);
            float slo = 0.f, shi = 0.f;
            if (nlo > -INFINITY) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) slo += fast_exp2(sc[nt][0] - nlo) + fast_exp2(sc[nt][1] - nlo);
            }
            if (nhi > -INFINITY) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) shi += fast_exp2(sc[nt][2] - nhi) + fast_exp2(sc[nt][3] - nhi);
            }
            slo += __shfl_xor_sync(0xffffffffu, slo, 1);
            slo += __shfl_xor_sync(0xffffffffu, slo, 2);
            shi += __shfl_xor_sync(0xffffffffu, shi, 1);
            shi += __shfl_xor_sync(0xffffffffu, shi, 2);
            l_lo[s] = (m_lo[s] > -INFINITY ? l_lo[s] * fast_exp2(m_lo[s] - nlo) : 0.f) + slo;
            l_hi[s] = (m_hi[s] > -INFINITY ? l_hi[s] * fast_exp2(m_hi[s] - nhi) : 0.f) + shi;
            m_lo[s] = nlo;
            m_hi[s] = nhi;
        }
    }
    // ---- pass 2
    float mrow[HPW][16];
    float O[HPW][NT][4];
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
        const int h = warp + s * NW;
#pragma unroll
        for (int g = 0; g < 16; ++g)
            mrow[s][g] = (h < H && g < H) ? (mix ? mix[h * H + g] : (g == h ? 1.f : 0.f)) : 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) O[s][nt][x] = 0.f;
    }
    const int nt_used = dv / 8;
    for (int kb = 0; kb < nblocks; ++kb) {
        __syncthreads();
        load_keys(kb);
        load_values(kb);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int s = 0; s < HPW; ++s) {
            const int g = warp + s * NW;
            if (g >= H) continue;
            float sc[4][4];
            scores(g, kb, sc);
            const float rlo = 1.f / l_lo[s], rhi = 1.f / l_hi[s];
            float* pg = Ps + (size_t)g * 16 * AT_PS;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                *(float2*)(pg + r * AT_PS + nt * 8 + 2 * c) =
                    make_float2(fast_exp2(sc[nt][0] - m_lo[s]) * rlo, fast_exp2(sc[nt][1] - m_lo[s]) * rlo);
                *(float2*)(pg + (r + 8) * AT_PS + nt * 8 + 2 * c) =
                    make_float2(fast_exp2(sc[nt][2] - m_hi[s]) * rhi, fast_exp2(sc[nt][3] - m_hi[s]) * rhi);
            }
        }
        __syncthreads();
#pragma unroll
        for (int s = 0; s < HPW; ++s) {
            const int h = warp + s * NW;
            if (h >= H) continue;
            const bf16* vb = Vt + (size_t)(h / group) * AT_KB * VS;
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                float w[8];
#pragma unroll
                for (int x = 0; x < 8; ++x) w[x] = 0.f;
#pragma unroll
                for (int g = 0; g < 16; ++g) {
                    if (g < H) {
                        const float* pg = Ps + (size_t)g * 16 * AT_PS + kk * 16 + 2 * c;
                        const float2 x0 = *(const float2*)(pg + r * AT_PS);
                        const float2 x1 = *(const float2*)(pg + (r + 8) * AT_PS);
                        const float2 x2 = *(const float2*)(pg + r * AT_PS + 8);
                        const float2 x3 = *(const float2*)(pg + (r + 8) * AT_PS + 8);
                        const float mg = mrow[s][g];
                        w[0] += mg * x0.x; w[1] += mg * x0.y; w[2] += mg * x1.x; w[3] += mg * x1.y;
                        w[4] += mg * x2.x; w[5] += mg * x2.y; w[6] += mg * x3.x; w[7] += mg * x3.y;
                    }
                }
                uint32_t a[4];
                a[0] = pack_bf16(w[0], w[1]);
                a[1] = pack_bf16(w[2], w[3]);
                a[2] = pack_bf16(w[4], w[5]);
                a[3] = pack_bf16(w[6], w[7]);
#pragma unroll
                for (int dp = 0; dp < NT / 2; ++dp) {            // two tiles of 8 columns at a time
                    if (2 * dp < nt_used) {
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, vb + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS +
                                                  dp * 16 + (lane >> 4) * 8);
                        mma_bf16(O[s][2 * dp], a, vf[0], vf[1]);
                        if (2 * dp + 1 < nt_used) mma_bf16(O[s][2 * dp + 1], a, vf[2], vf[3]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int s = 0; s < HPW; ++s) {
        const int h = warp + s * NW;
        if (h >= H) continue;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            if (nt >= nt_used) continue;
            const int col = h * dv + nt * 8 + 2 * c;
            if (r < ntok)
                *(uint32_t*)(out + (size_t)(tok0 + r) * out_stride + col) = pack_bf16(O[s][nt][0], O[s][nt][1]);
            if (r + 8 < ntok)
                *(uint32_t*)(out + (size_t)(tok0 + r + 8) * out_stride + col) = pack_bf16(O[s][nt][2], O[s][nt][3]);
        }
    }
}

// 1 if the tile kernel takes these sizes (bfloat16 only), else 0.
TGO_API int tgo_attention_mixed_tile_supports(int H, int Hkv, int dk, int dv, int window) {
    if (H <= 0 || Hkv <= 0 || H % Hkv || H > 16 || dk % 16 || dk <= 0 || dv % 8 || dv <= 0 || dv > 128 ||
        window != 0)
        return 0;
    return mixed_tile_smem(H, Hkv, dk, dv).total <= 200 * 1024 ? 1 : 0;
}

template <int NW, int HPW, int NT>
static int launch_mixed_tile(int tiles, size_t smem, cudaStream_t stream, const bf16* q, long long q_stride,
                             bf16* out, long long out_stride, int H, int G, int dk, int dv, const bf16* kc,
                             const bf16* vc, int page_size, const int* bt, int max_blocks, const int* seq_ids,
                             const int* positions, const float* mix, float scale, const int* tok0,
                             const int* ntok, MixedTileSmem m) {
    auto kern = attention_mixed_tile_kernel<NW, HPW, NT>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return tgo_launch_pdl(kern, dim3(tiles), dim3(NW * 32), smem, stream, q, q_stride, out, out_stride, H,
                          G, dk, dv, kc, vc, page_size, bt, max_blocks, seq_ids, positions, mix, scale, tok0,
                          ntok, m.ks, m.vs, m.ps);
}

// Tiles: tile_tok0[i] is the first token row of tile i, tile_ntok[i] (1..16) its tokens, all
// of one request at consecutive positions. out rows must allow 4-byte stores (even strides).
TGO_API int tgo_attention_mixed_tile(const void* q, long long q_stride, void* out, long long out_stride,
                                     int tiles, int H, int Hkv, int dk, int dv, const void* k_cache,
                                     const void* v_cache, int page_size, const int* block_tables,
                                     int max_blocks, const int* seq_ids, const int* positions,
                                     const float* mix, float scale, const int* tile_tok0,
                                     const int* tile_ntok, cudaStream_t stream) {
    if (tiles <= 0) return 0;
    if (!tgo_attention_mixed_tile_supports(H, Hkv, dk, dv, 0) || page_size <= 0 || max_blocks <= 0 ||
        (out_stride & 1) || ((uintptr_t)out & 3) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return TGO_E_BAD_ARG;
    const MixedTileSmem m = mixed_tile_smem(H, Hkv, dk, dv);
#define MT_ARGS tiles, m.total, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride, H, Hkv, dk, dv, \
        (const bf16*)k_cache, (const bf16*)v_cache, page_size, block_tables, max_blocks, seq_ids, positions, \
        mix, scale, tile_tok0, tile_ntok, m
    // a warp a head: eight warps up to eight heads, sixteen above (more warps to hide each other's
    // waits: the block is alone on its multiprocessor at the larger sizes)
    if (H <= 8) return dv <= 64 ? launch_mixed_tile<8, 1, 8>(MT_ARGS) : launch_mixed_tile<8, 1, 16>(MT_ARGS);
    return dv <= 64 ? launch_mixed_tile<16, 1, 8>(MT_ARGS) : launch_mixed_tile<16, 1, 16>(MT_ARGS);
#undef MT_ARGS
}

// ---------------------------------------------------------------------- decode steps, bfloat16
// One token a request: the keys of a token are cut into `splits` ranges (multiples of 32
// keys), a block per (token, range), all heads in the block, so that a few requests still
// fill the GPU. Three launches, no atomics, sums in a fixed order:
//
//   scores   s_g(j) = q_g . k(j) * scale for the range's keys (a lane a key, 16-byte loads of
//            its row, q in shared memory) -> scratch [token][head][key]; then per head the
//            range's maximum and sum of exponentials -> [token][range][head];
//   values   every block joins the ranges' maxima and sums into each head's final ones, turns
//            its range's scores into weights 32 keys at a time, mixes them across heads, and
//            adds w_h v into float32 partial outputs [token][range][H * dv], the 32 values of
//            every kv head staged in shared memory by 16-byte loads;
//   join     out = sum over the ranges, in range order.
#define AD_THREADS 256
#define AD_MAX_GROUP 16

__device__ __forceinline__ void split_range(int p, int splits, int s, int& lo, int& hi) {
    int chunk = (p + splits) / splits;              // ceil((p + 1) / splits)
    chunk = (chunk + 31) & ~31;
    lo = s * chunk;
    hi = lo + chunk < p + 1 ? lo + chunk : p + 1;
    if (lo > hi) lo = hi;
}

__global__ void __launch_bounds__(AD_THREADS)
mixed_decode_scores_kernel(const bf16* __restrict__ q, long long q_stride, int H, int G, int dk,
                           const bf16* __restrict__ k_cache, int page_size,
                           const int* __restrict__ block_tables, int max_blocks,
                           const int* __restrict__ seq_ids, const int* __restrict__ positions,
                           float scale, int splits, float* __restrict__ scores, int score_stride,
                           float2* __restrict__ stats) {
    extern __shared__ float qs[];                   // [H][dk]
    pdl_wait();
    const int t = blockIdx.x, s = blockIdx.y;
    const int p = positions[t];
    if (p < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_tables + (size_t)seq_ids[t] * max_blocks;
    const int group = H / G;
    for (int i = threadIdx.x; i < H * dk; i += AD_THREADS) qs[i] = to_f32(q[(size_t)t * q_stride + i]);
    __syncthreads();
    int lo, hi;
    split_range(p, splits, s, lo, hi);
    float* srow = scores + (size_t)t * H * score_stride;
    // a thread a (key, kv head) pair, keys fastest: it reads the key's row 16 bytes at a time
    // (two loads ahead of their use) and multiplies it by the q of every head of the kv head,
    // read from shared memory
    const int nkeys = hi - lo;
    for (int item = threadIdx.x; item < nkeys * G; item += AD_THREADS) {
        const int j = lo + item % nkeys, kvh = item / nkeys;
        const int page = bt[j / page_size];
        {
            const bf16* kr = k_cache + (((size_t)page * G + kvh) * page_size + (j % page_size)) * dk;
            float acc[AD_MAX_GROUP];
#pragma unroll
            for (int x = 0; x < AD_MAX_GROUP; ++x) acc[x] = 0.f;
            for (int ch = 0; ch < dk; ch += 16) {
                uint4 raw[2];
                raw[0] = *(const uint4*)(kr + ch);
                raw[1] = ch + 8 < dk ? *(const uint4*)(kr + ch + 8) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (ch + half * 8 >= dk) break;
                    const __nv_bfloat162* e = (const __nv_bfloat162*)&raw[half];
                    float kf[8];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const float2 f = __bfloat1622float2(e[x]);
                        kf[2 * x] = f.x;
                        kf[2 * x + 1] = f.y;
                    }
#pragma unroll
                    for (int gl = 0; gl < AD_MAX_GROUP; ++gl) {
                        if (gl < group) {
                            const float4* qh = (const float4*)(qs + (size_t)(kvh * group + gl) * dk + ch + half * 8);
                            const float4 q0 = qh[0], q1 = qh[1];
                            acc[gl] += q0.x * kf[0] + q0.y * kf[1] + q0.z * kf[2] + q0.w * kf[3] +
                                       q1.x * kf[4] + q1.y * kf[5] + q1.z * kf[6] + q1.w * kf[7];
                        }
                    }
                }
            }
#pragma unroll
            for (int gl = 0; gl < AD_MAX_GROUP; ++gl)
                if (gl < group) srow[(size_t)(kvh * group + gl) * score_stride + j] = acc[gl] * scale;
        }
    }
    __syncthreads();
    for (int g = warp; g < H; g += AD_THREADS / 32) {
        const float* sg = srow + (size_t)g * score_stride;
        float m = -INFINITY;
        for (int j = lo + lane; j < hi; j += 32) m = fmaxf(m, sg[j]);
        m = warp_max(m);
        float l = 0.f;
        for (int j = lo + lane; j < hi; j += 32) l += expf(sg[j] - m);
        l = warp_sum(l);
        if (lane == 0) stats[((size_t)t * splits + s) * H + g] = make_float2(m, hi > lo ? l : 0.f);
    }
}

template <bool TC>
__global__ void __launch_bounds__(AD_THREADS)
mixed_decode_values_kernel(int H, int G, int dv, const bf16* __restrict__ v_cache, int page_size,
                           const int* __restrict__ block_tables, int max_blocks,
                           const int* __restrict__ seq_ids, const int* __restrict__ positions,
                           const float* __restrict__ mix, int splits,
                           const float* __restrict__ scores, int score_stride,
                           const float2* __restrict__ stats, float* __restrict__ partial) {
    extern __shared__ __align__(16) unsigned char raw_smem[];
    float* fm = (float*)raw_smem;                   // [H] final maximum
    float* fr = fm + H;                             // [H] 1 / final sum
    float* ms = fr + H;                             // [H][H]
    // the two weight tables start at a multiple of four floats: rows of them are read 8 bytes
    // at a time, and the values behind them 16
    float* ps = fm + ((2 * H + H * H + 3) & ~3);    // [H][32] weights
    float* ws = ps + H * 32;                        // [H][32] weights mixed across heads
    // [G][32][dv + 8], 16-byte aligned.
    // TC (H <= 16, dv % 16 == 0): the product w V runs on the tensor cores with the heads as the
    // 16 rows of the tile: per kv head a [16 x 32] x [32 x dv] product of which the rows of that
    // kv head's heads are kept; warp w owns the (kv head, 16 columns) items w, w + 8, ...
    bf16* vs = (bf16*)(ws + H * 32);
    const int VSD = dv + 8;
    constexpr int TC_ITEMS = 8;                    // items a warp may own: G * dv / 16 <= 64
    float otc[TC ? TC_ITEMS : 1][2][4];
#pragma unroll
    for (int x = 0; x < (TC ? TC_ITEMS : 1); ++x)
#pragma unroll
        for (int y = 0; y < 2; ++y)
#pragma unroll
            for (int z = 0; z < 4; ++z) otc[x][y][z] = 0.f;
    pdl_wait();
    const int t = blockIdx.x, s = blockIdx.y;
    const int p = positions[t];
    if (p < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int* bt = block_tables + (size_t)seq_ids[t] * max_blocks;
    const int group = H / G;
    for (int g = threadIdx.x; g < H; g += AD_THREADS) {
        float m = -INFINITY;
        for (int x = 0; x < splits; ++x) m = fmaxf(m, stats[((size_t)t * splits + x) * H + g].x);
        float l = 0.f;
        for (int x = 0; x < splits; ++x) {
            const float2 st = stats[((size_t)t * splits + x) * H + g];
            if (st.y > 0.f) l += st.y * expf(st.x - m);
        }
        fm[g] = m;
        fr[g] = 1.f / l;
    }
    for (int i = threadIdx.x; i < H * H; i += AD_THREADS)
        ms[i] = mix ? mix[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    int lo, hi;
    split_range(p, splits, s, lo, hi);
    const float* srow = scores + (size_t)t * H * score_stride;
    const int pairs = H * dv / 2;                   // output column pairs
    // this thread's pairs: threadIdx.x, + 256, ...; up to 4 (H * dv <= 2048)
    float2 acc[4];
#pragma unroll
    for (int x = 0; x < 4; ++x) acc[x] = make_float2(0.f, 0.f);
    for (int base = lo; base < hi; base += 32) {
        const int n = hi - base < 32 ? hi - base : 32;
        __syncthreads();
        for (int g = warp; g < H; g += AD_THREADS / 32)
            ps[g * 32 + lane] = lane < n ? __expf(srow[(size_t)g * score_stride + base + lane] - fm[g]) * fr[g] : 0.f;
        // the 32 values of every kv head: 16-byte asynchronous copies, all in flight at once
        const int chunks = dv / 8;
        for (int i = threadIdx.x; i < G * 32 * chunks; i += AD_THREADS) {
            const int ch = i % chunks, key = (i / chunks) % 32, g = i / (chunks * 32);
            const bool live = key < n;
            const int j = live ? base + key : base;
            cp_async16(vs + ((size_t)g * 32 + key) * VSD + ch * 8,
                       v_cache + (((size_t)bt[j / page_size] * G + g) * page_size + (j % page_size)) * dv + ch * 8,
                       live);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        for (int h = warp; h < H; h += AD_THREADS / 32) {
            float w = 0.f;
            for (int g = 0; g < H; ++g) w += ms[h * H + g] * ps[g * 32 + lane];
            ws[h * 32 + lane] = w;
        }
        __syncthreads();
        if (TC) {
            const int r = lane >> 2, c = lane & 3;
            uint32_t a[2][4];
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                const float* w0 = ws + r * 32 + kk * 16 + 2 * c;          // rows past H: zeros below
                const float* w1 = ws + (r + 8) * 32 + kk * 16 + 2 * c;
                const float2 z = make_float2(0.f, 0.f);
                const float2 x0 = r < H ? *(const float2*)w0 : z, x1 = r + 8 < H ? *(const float2*)w1 : z;
                const float2 x2 = r < H ? *(const float2*)(w0 + 8) : z, x3 = r + 8 < H ? *(const float2*)(w1 + 8) : z;
                a[kk][0] = pack_bf16(x0.x, x0.y);
                a[kk][1] = pack_bf16(x1.x, x1.y);
                a[kk][2] = pack_bf16(x2.x, x2.y);
                a[kk][3] = pack_bf16(x3.x, x3.y);
            }
            const int per_head = dv / 16;
#pragma unroll
            for (int x = 0; x < TC_ITEMS; ++x) {
                const int item = warp + x * (AD_THREADS / 32);
                if (item < G * per_head) {
                    const bf16* vb = vs + (size_t)(item / per_head) * 32 * VSD + (item % per_head) * 16;
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        uint32_t vf[4];
                        ldmatrix_x4_trans(vf, vb + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VSD +
                                                  (lane >> 4) * 8);
                        mma_bf16(otc[x][0], a[kk], vf[0], vf[1]);
                        mma_bf16(otc[x][1], a[kk], vf[2], vf[3]);
                    }
                }
            }
        } else {
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                const int pr = threadIdx.x + x * AD_THREADS;
                if (pr < pairs) {
                    const int h = (2 * pr) / dv, c = (2 * pr) % dv;
                    const bf16* vb = vs + (size_t)(h / group) * 32 * VSD + c;
                    const float* wh = ws + h * 32;
                    float2 a = acc[x];
                    for (int jj = 0; jj < n; ++jj) {
                        const float2 v2 = __bfloat1622float2(*(const __nv_bfloat162*)(vb + (size_t)jj * VSD));
                        a.x += wh[jj] * v2.x;
                        a.y += wh[jj] * v2.y;
                    }
                    acc[x] = a;
                }
            }
        }
    }
    float* po = partial + ((size_t)t * splits + s) * H * dv;
    if (TC) {
        const int r = lane >> 2, c = lane & 3;
        const int per_head = dv / 16;
#pragma unroll
        for (int x = 0; x < TC_ITEMS; ++x) {
            const int item = warp + x * (AD_THREADS / 32);
            if (item < G * per_head) {
                const int kvh = item / per_head, col = (item % per_head) * 16 + 2 * c;
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    if (r < H && r / group == kvh)
                        *(float2*)(po + (size_t)r * dv + col + 8 * y) = make_float2(otc[x][y][0], otc[x][y][1]);
                    if (r + 8 < H && (r + 8) / group == kvh)
                        *(float2*)(po + (size_t)(r + 8) * dv + col + 8 * y) = make_float2(otc[x][y][2], otc[x][y][3]);
                }
            }
        }
    } else {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int pr = threadIdx.x + x * AD_THREADS;
            if (pr < pairs) *(float2*)(po + 2 * pr) = acc[x];
        }
    }
}

__global__ void mixed_decode_join_kernel(const float* __restrict__ partial, int splits, int width,
                                         const int* __restrict__ positions, bf16* __restrict__ out,
                                         long long out_stride) {
    pdl_wait();
    const int t = blockIdx.x;
    const bool live = positions[t] >= 0;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float a = 0.f;
        if (live)
            for (int s = 0; s < splits; ++s) a += partial[((size_t)t * splits + s) * width + i];
        out[(size_t)t * out_stride + i] = from_f32<bf16>(a);
    }
}

static inline size_t mixed_decode_values_smem(int H, int G, int dv) {
    return (size_t)(((2 * H + H * H + 3) & ~3) + 2 * H * 32) * 4 + (size_t)G * 32 * (dv + 8) * 2;
}

TGO_API int tgo_attention_mixed_decode_supports(int H, int Hkv, int dk, int dv, int window) {
    if (H <= 0 || Hkv <= 0 || H % Hkv || H > AM_MAX_H || H / Hkv > AD_MAX_GROUP || dk % 8 || dk <= 0 ||
        dv % 8 || dv <= 0 || H * dv > 8 * AD_THREADS || window != 0)
        return 0;
    const size_t smem2 = mixed_decode_values_smem(H, Hkv, dv);
    return ((size_t)H * dk * 4 <= 160 * 1024 && smem2 <= 160 * 1024) ? 1 : 0;
}

// scores: float32 [T, H, score_stride] scratch (score_stride >= the longest context, a
// multiple of 32 is not needed); stats: [T, splits, H] pairs of float32; partial: float32
// [T, splits, H * dv]. All three are scratch of the call.
TGO_API int tgo_attention_mixed_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                       int T, int H, int Hkv, int dk, int dv, const void* k_cache,
                                       const void* v_cache, int page_size, const int* block_tables,
                                       int max_blocks, const int* seq_ids, const int* positions,
                                       const float* mix, float scale, int splits, float* scores,
                                       int score_stride, float* stats, float* partial,
                                       cudaStream_t stream) {
    if (T <= 0) return 0;
    if (!tgo_attention_mixed_decode_supports(H, Hkv, dk, dv, 0) || splits <= 0 || splits > 65535 ||
        page_size <= 0 || max_blocks <= 0 || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
        return TGO_E_BAD_ARG;
    const size_t smem1 = (size_t)H * dk * 4;
    const size_t smem2 = mixed_decode_values_smem(H, Hkv, dv);
    if (smem1 > 48 * 1024)
        cudaFuncSetAttribute(mixed_decode_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    // the product w V on the tensor cores where a tile of 16 rows holds all heads
    const bool tc = H <= 16 && dv % 16 == 0 && Hkv * (dv / 16) <= 64;
    auto values = tc ? mixed_decode_values_kernel<true> : mixed_decode_values_kernel<false>;
    if (smem2 > 48 * 1024)
        cudaFuncSetAttribute(values, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    int rc = tgo_launch_pdl(mixed_decode_scores_kernel, dim3(T, splits), dim3(AD_THREADS), smem1, stream,
                            (const bf16*)q, q_stride, H, Hkv, dk, (const bf16*)k_cache, page_size, block_tables,
                            max_blocks, seq_ids, positions, scale, splits, scores, score_stride, (float2*)stats);
    if (rc) return rc;
    rc = tgo_launch_pdl(values, dim3(T, splits), dim3(AD_THREADS), smem2, stream, H, Hkv,
                        dv, (const bf16*)v_cache, page_size, block_tables, max_blocks, seq_ids, positions, mix,
                        splits, (const float*)scores, score_stride, (const float2*)stats, partial);
    if (rc) return rc;
    return tgo_launch_pdl(mixed_decode_join_kernel, dim3(T), dim3(256), 0, stream, (const float*)partial,
                          splits, H * dv, positions, (bf16*)out, out_stride);
}
