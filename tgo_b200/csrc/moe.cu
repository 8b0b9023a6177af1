// A routed feed-forward (mixture of experts): every token goes to the `top` experts with the
// largest router logits, weighted by the softmax over those logits alone.
//
//   route      logits = Wr x + br in float32 (Wr, br float32; x in the storage type), the top
//              experts (ties: the lower index), their weights, and a count per expert
//   plan       expert e's (token, choice) pairs get places offsets[e] .. offsets[e+1]-1; the
//              places are cut into row tiles of one expert each
//   scatter    pair -> place (within an expert the order is whatever the atomics give; a
//              pair's result does not depend on its place)
//   up         hidden[place] = act(x Wg_e^T) * (x Wu_e^T) for the token of the pair at `place`
//   down       y[pair] = hidden[place] Wd_e^T, float32
//   combine    out[t] = sum_j weight[t][j] y[t top + j] (+ extra[t]), j in order, all float32
//
// The products here are tiled plain-FMA products with float32 sums over k in order: a row's
// result does not depend on which tile or batch it falls in.
#include "common.cuh"

#define MOE_TM 64
#define MOE_TN 64
#define MOE_TK 16

// ------------------------------------------------------------------------------- route
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ wr,
                 const float* __restrict__ br, int Tn, int d, int E, int top, int* __restrict__ ids,
                 float* __restrict__ wts, int* __restrict__ counts) {
    extern __shared__ float smem[];
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= Tn) return;
    float* lg = smem + (size_t)warp * E;
    const T* row = x + (size_t)t * x_stride;
    for (int e = 0; e < E; ++e) {
        const float* w = wr + (size_t)e * d;
        float a = 0.f;
        for (int i = lane; i < d; i += 32) a = fmaf(w[i], to_f32(row[i]), a);
        a = warp_sum(a);
        if (lane == 0) lg[e] = a + (br ? br[e] : 0.f);
    }
    __syncwarp();
    float first = 0.f, sum = 0.f, mine = 0.f;
    int mine_e = 0;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int be = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = lg[e];
            if (v > best || (v == best && e < be)) { best = v; be = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > best || (ov == best && oe < be)) { best = ov; be = oe; }
        }
        if (j == 0) first = best;
        const float w = expf(best - first);
        sum += w;
        if (lane == j) { mine = w; mine_e = be; }
        if (lane == 0) lg[be] = -INFINITY;
        __syncwarp();
    }
    if (lane < top) {
        ids[(size_t)t * top + lane] = mine_e;
        wts[(size_t)t * top + lane] = mine / sum;
        atomicAdd(&counts[mine_e], 1);
    }
}

// -------------------------------------------------------------------------------- plan
// One thread: offsets [E + 1], tiles (expert, first place, rows) and their count in
// tile_info[0]; the fill counters go back to zero.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                int* __restrict__ fill, int* __restrict__ tile_info,
                                int* __restrict__ tiles, int max_tiles) {
    pdl_wait();
    if (threadIdx.x || blockIdx.x) return;
    int at = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
        offsets[e] = at;
        fill[e] = 0;
        const int c = counts[e];
        for (int r = 0; r < c && nt < max_tiles; r += MOE_TM) {
            tiles[3 * nt] = e;
            tiles[3 * nt + 1] = at + r;
            tiles[3 * nt + 2] = c - r < MOE_TM ? c - r : MOE_TM;
            ++nt;
        }
        at += c;
    }
    offsets[E] = at;
    tile_info[0] = nt;
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, int pairs,
                                   const int* __restrict__ offsets, int* __restrict__ fill,
                                   int* __restrict__ perm, int* __restrict__ place) {
    pdl_wait();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pairs) return;
    const int e = ids[p];
    const int at = offsets[e] + atomicAdd(&fill[e], 1);
    perm[at] = p;
    place[p] = at;
}

// ----------------------------------------------------------------------------- products
__device__ __forceinline__ float moe_act(float z, int act) {
    if (act == 1) return z > 0.f ? z : 0.f;
    if (act == 2) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return z / (1.f + expf(-z));
}

// hidden[place][f] = act(x_tok . Wg[e][f]) * (x_tok . Wu[e][f]); Wg, Wu [E, ff, d].
template <typename T>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ wg,
              const T* __restrict__ wu, T* __restrict__ hidden, int d, int ff, int top, int act,
              const int* __restrict__ perm, const int* __restrict__ tile_info,
              const int* __restrict__ tiles) {
    __shared__ float xs[MOE_TK][MOE_TM + 4];
    __shared__ float gs[MOE_TK][MOE_TN + 4];
    __shared__ float us[MOE_TK][MOE_TN + 4];
    __shared__ int toks[MOE_TM];
    pdl_wait();
    if ((int)blockIdx.y >= tile_info[0]) return;
    const int e = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * MOE_TN;
    if (threadIdx.x < MOE_TM) toks[threadIdx.x] = threadIdx.x < rows ? perm[r0 + threadIdx.x] / top : -1;
    __syncthreads();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* wge = wg + (size_t)e * ff * d;
    const T* wue = wu + (size_t)e * ff * d;
    float ag[4][4], au[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) ag[i][j] = au[i][j] = 0.f;
    for (int k0 = 0; k0 < d; k0 += MOE_TK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int row = idx / MOE_TK, kk = idx % MOE_TK;
            const int gk = k0 + kk, gn = n0 + row;
            const int tok = toks[row];
            xs[kk][row] = (tok >= 0 && gk < d) ? to_f32(x[(size_t)tok * x_stride + gk]) : 0.f;
            const bool in = gn < ff && gk < d;
            gs[kk][row] = in ? to_f32(wge[(size_t)gn * d + gk]) : 0.f;
            us[kk][row] = in ? to_f32(wue[(size_t)gn * d + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float a[4], g[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { g[j] = gs[kk][tx * 4 + j]; u[j] = us[kk][tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ag[i][j] = fmaf(a[i], g[j], ag[i][j]);
                    au[i][j] = fmaf(a[i], u[j], au[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = ty * 4 + i;
        if (row >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < ff)
                hidden[(size_t)(r0 + row) * ff + gn] = from_f32<T>(moe_act(ag[i][j], act) * au[i][j]);
        }
    }
}

// y[pair][n] = hidden[place] . Wd[e][n]; Wd [E, d, ff]; y float32 [pairs, d].
template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ hidden, const T* __restrict__ wd, float* __restrict__ y, int d,
                int ff, const int* __restrict__ perm, const int* __restrict__ tile_info,
                const int* __restrict__ tiles) {
    __shared__ float hs[MOE_TK][MOE_TM + 4];
    __shared__ float ws[MOE_TK][MOE_TN + 4];
    pdl_wait();
    if ((int)blockIdx.y >= tile_info[0]) return;
    const int e = tiles[3 * blockIdx.y], r0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * MOE_TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const T* wde = wd + (size_t)e * d * ff;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < ff; k0 += MOE_TK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int idx = threadIdx.x + r * 256;
            const int row = idx / MOE_TK, kk = idx % MOE_TK;
            const int gk = k0 + kk, gn = n0 + row;
            hs[kk][row] = (row < rows && gk < ff) ? to_f32(hidden[(size_t)(r0 + row) * ff + gk]) : 0.f;
            ws[kk][row] = (gn < d && gk < ff) ? to_f32(wde[(size_t)gn * ff + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = hs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = ty * 4 + i;
        if (row >= rows) continue;
        const int pair = perm[r0 + row];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < d) y[(size_t)pair * d + gn] = acc[i][j];
        }
    }
}

// out[t][c] = sum_j wts[t][j] y[t top + j][c] + extra[t][c]
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts,
                                   const float* __restrict__ extra, float* __restrict__ out, int d,
                                   int top) {
    pdl_wait();
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float a = 0.f;
        for (int j = 0; j < top; ++j) a = fmaf(wts[(size_t)t * top + j], y[((size_t)t * top + j) * d + c], a);
        if (extra) a += extra[(size_t)t * d + c];
        out[(size_t)t * d + c] = a;
    }
}

TGO_API int tgo_moe_tile_rows() { return MOE_TM; }

// ids, place int32 [T top]; wts float32 [T top]; counts, fill int32 [E]; offsets int32 [E + 1];
// perm int32 [T top]; tile_info int32 [1]; tiles int32 [3 max_tiles].
TGO_API int tgo_moe_route(const void* x, long long x_stride, int dtype, const float* wr,
                          const float* br, int T, int d, int E, int top, int* ids, float* wts,
                          int* counts, int* fill, int* offsets, int* perm, int* place,
                          int* tile_info, int* tiles, int max_tiles, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || E <= 0 || E > 2048 || top <= 0 || top > 32 || top > E || max_tiles <= 0)
        return TGO_E_BAD_ARG;
    int rc = (int)cudaMemsetAsync(counts, 0, sizeof(int) * E, stream);
    if (rc) return rc;
    const size_t smem = (size_t)4 * E * sizeof(float);
    if (dtype == TGO_BF16)
        moe_route_kernel<bf16><<<(T + 3) / 4, 128, smem, stream>>>((const bf16*)x, x_stride, wr, br, T, d, E,
                                                                  top, ids, wts, counts);
    else if (dtype == TGO_F32)
        moe_route_kernel<float><<<(T + 3) / 4, 128, smem, stream>>>((const float*)x, x_stride, wr, br, T, d,
                                                                   E, top, ids, wts, counts);
    else
        return TGO_E_BAD_ARG;
    if ((rc = launch_status())) return rc;
    rc = tgo_launch_pdl(moe_plan_kernel, dim3(1), dim3(32), 0, stream, (const int*)counts, E, offsets, fill,
                        tile_info, tiles, max_tiles);
    if (rc) return rc;
    const int pairs = T * top;
    return tgo_launch_pdl(moe_scatter_kernel, dim3((pairs + 255) / 256), dim3(256), 0, stream,
                          (const int*)ids, pairs, (const int*)offsets, fill, perm, place);
}

// x [T, d] rows (stride x_stride); wg, wu [E, ff, d]; wd [E, d, ff]; hidden [T top, ff] in the
// storage type; y float32 [T top, d]; extra float32 [T, d] or null; out float32 [T, d].
TGO_API int tgo_moe_experts(const void* x, long long x_stride, int dtype, const void* wg,
                            const void* wu, const void* wd, void* hidden, float* y,
                            const float* wts, const float* extra, float* out, int T, int d, int ff,
                            int top, int act, const int* perm, const int* tile_info,
                            const int* tiles, int max_tiles, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || ff <= 0 || top <= 0 || max_tiles <= 0 || max_tiles > 65535 || act < 0 || act > 2)
        return TGO_E_BAD_ARG;
    const dim3 g1((ff + MOE_TN - 1) / MOE_TN, max_tiles), g2((d + MOE_TN - 1) / MOE_TN, max_tiles);
    int rc;
    if (dtype == TGO_BF16) {
        rc = tgo_launch_pdl(moe_up_kernel<bf16>, g1, dim3(256), 0, stream, (const bf16*)x, x_stride,
                            (const bf16*)wg, (const bf16*)wu, (bf16*)hidden, d, ff, top, act, perm, tile_info,
                            tiles);
        if (rc) return rc;
        rc = tgo_launch_pdl(moe_down_kernel<bf16>, g2, dim3(256), 0, stream, (const bf16*)hidden,
                            (const bf16*)wd, y, d, ff, perm, tile_info, tiles);
        if (rc) return rc;
        return tgo_launch_pdl(moe_combine_kernel, dim3(T), dim3(256), 0, stream, (const float*)y, wts,
                              extra, out, d, top);
    }
    if (dtype != TGO_F32) return TGO_E_BAD_ARG;
    rc = tgo_launch_pdl(moe_up_kernel<float>, g1, dim3(256), 0, stream, (const float*)x, x_stride,
                        (const float*)wg, (const float*)wu, (float*)hidden, d, ff, top, act, perm, tile_info,
                        tiles);
    if (rc) return rc;
    rc = tgo_launch_pdl(moe_down_kernel<float>, g2, dim3(256), 0, stream, (const float*)hidden,
                        (const float*)wd, y, d, ff, perm, tile_info, tiles);
    if (rc) return rc;
    return tgo_launch_pdl(moe_combine_kernel, dim3(T), dim3(256), 0, stream, (const float*)y, wts,
                          extra, out, d, top);
}
