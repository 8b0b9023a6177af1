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
#include "common.cuh"

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
