// Retention: linear attention with one fixed decay per head, no softmax and no denominator.
// Per request and head a float32 state S [dk][dv] is carried from token to token:
//
//   S_t = decay * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
//
// q and k are rotated (half-split pairs, from the step's cos/sin table) as they are loaded,
// and k is then multiplied by k_scale; all of it in float32, whatever the storage type of the
// projections. A step's tokens of one request are taken in chunks of up to RT_CHUNK tokens:
// inside a chunk (local index i, j; n tokens)
//
//   o_i = sum_{j<=i} decay^(i-j) (q_i . k_j) v_j  +  decay^(i+1) S^T q_i
//   S  <- decay^n S + sum_j decay^(n-1-j) k_j v_j^T
//
// which is the recurrence written out; a single token (a decode step) is a chunk of one.
// The columns of S are independent, so a block owns a slice of dv columns of one
// (request, head): grid (requests, heads, slices). The powers of the decay come from a table
// made by repeated multiplication.
#include "common.cuh"

#define RT_CHUNK 32
#define RT_THREADS 256

// What q, k and v go through as they are read (a parameter of every kernel here):
// 0 nothing, 1 SiLU, in float32.
template <typename T>
__device__ __forceinline__ float taken(T x, int act) {
    const float f = to_f32(x);
    return act == 1 ? f / (1.f + expf(-f)) : f;
}

template <typename T>
__device__ __forceinline__ float rotated(const T* __restrict__ x, const float* __restrict__ cs,
                                         int i, int rot, int act) {
    const int half = rot >> 1;
    if (i < half) return taken(x[i], act) * cs[i] - taken(x[i + half], act) * cs[half + i];
    if (i < rot) return taken(x[i], act) * cs[i - half] + taken(x[i - half], act) * cs[i];
    return taken(x[i], act);
}

template <typename T>
__global__ void __launch_bounds__(RT_THREADS)
retention_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                 long long k_stride, const T* __restrict__ v, long long v_stride,
                 float* __restrict__ out, int H, int dk, int dv, int vs,
                 const float* __restrict__ decay, float k_scale, int act, const float* __restrict__ rope,
                 int rot, const int* __restrict__ q_start, const int* __restrict__ state_slots,
                 float* __restrict__ state) {
    extern __shared__ float smem[];
    const int dkp = dk + 1;
    float* Qs = smem;                               // [RT_CHUNK][dk + 1]
    float* Ks = Qs + RT_CHUNK * dkp;                // [RT_CHUNK][dk + 1]
    float* Vs = Ks + RT_CHUNK * dkp;                // [RT_CHUNK][vs]
    float* As = Vs + RT_CHUNK * vs;                 // [RT_CHUNK][RT_CHUNK + 1]
    float* Ss = As + RT_CHUNK * (RT_CHUNK + 1);     // [dk][vs]
    float* pw = Ss + (size_t)dk * vs;               // [RT_CHUNK + 1]
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int c0 = blockIdx.z * vs;
    const int nc = (dv - c0) < vs ? (dv - c0) : vs;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    if (t1 <= t0) return;
    const float g = decay[h];
    float* Sg = state + (((size_t)state_slots[b] * H + h) * dk) * dv + c0;
    for (int i = threadIdx.x; i < dk * vs; i += RT_THREADS) {
        const int d = i / vs, c = i % vs;
        Ss[i] = c < nc ? Sg[(size_t)d * dv + c] : 0.f;
    }
    if (threadIdx.x == 0) {
        float x = 1.f;
        for (int i = 0; i <= RT_CHUNK; ++i) {
            pw[i] = x;
            x *= g;
        }
    }
    for (int ts = t0; ts < t1; ts += RT_CHUNK) {
        const int n = (t1 - ts) < RT_CHUNK ? (t1 - ts) : RT_CHUNK;
        __syncthreads();
        for (int i = threadIdx.x; i < n * dk; i += RT_THREADS) {
            const int r = i / dk, d = i % dk;
            const size_t t = (size_t)(ts + r);
            const float* cs = rope ? rope + t * rot : nullptr;
            const T* qr = q + t * q_stride + (size_t)h * dk;
            const T* kr = k + t * k_stride + (size_t)h * dk;
            Qs[r * dkp + d] = cs ? rotated(qr, cs, d, rot, act) : taken(qr[d], act);
            Ks[r * dkp + d] = (cs ? rotated(kr, cs, d, rot, act) : taken(kr[d], act)) * k_scale;
        }
        for (int i = threadIdx.x; i < n * vs; i += RT_THREADS) {
            const int r = i / vs, c = i % vs;
            Vs[i] = c < nc ? taken(v[(size_t)(ts + r) * v_stride + (size_t)h * dv + c0 + c], act) : 0.f;
        }
        __syncthreads();
        // A[i][j] = decay^(i-j) q_i . k_j for j <= i
        for (int idx = threadIdx.x; idx < n * n; idx += RT_THREADS) {
            const int i = idx / n, j = idx % n;
            float a = 0.f;
            if (j <= i) {
                const float* qi = Qs + i * dkp;
                const float* kj = Ks + j * dkp;
                for (int d = 0; d < dk; ++d) a += qi[d] * kj[d];
                a *= pw[i - j];
            }
            As[i * (RT_CHUNK + 1) + j] = a;
        }
        __syncthreads();
        // o_i[c] = sum_j A[i][j] v_j[c] + decay^(i+1) sum_d q_i[d] S[d][c]
        for (int idx = threadIdx.x; idx < n * vs; idx += RT_THREADS) {
            const int i = idx / vs, c = idx % vs;
            if (c >= nc) continue;
            const float* qi = Qs + i * dkp;
            float far = 0.f;
            for (int d = 0; d < dk; ++d) far += qi[d] * Ss[d * vs + c];
            float near = 0.f;
            const float* ai = As + i * (RT_CHUNK + 1);
            for (int j = 0; j <= i; ++j) near += ai[j] * Vs[j * vs + c];
            out[((size_t)(ts + i) * H + h) * dv + c0 + c] = near + pw[i + 1] * far;
        }
        __syncthreads();
        // S[d][c] = decay^n S[d][c] + sum_j decay^(n-1-j) k_j[d] v_j[c]
        for (int idx = threadIdx.x; idx < dk * vs; idx += RT_THREADS) {
            const int d = idx / vs, c = idx % vs;
            float a = 0.f;
            for (int j = 0; j < n; ++j) a += pw[n - 1 - j] * Ks[j * dkp + d] * Vs[j * vs + c];
            Ss[idx] = pw[n] * Ss[idx] + a;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < dk * vs; i += RT_THREADS) {
        const int d = i / vs, c = i % vs;
        if (c < nc) Sg[(size_t)d * dv + c] = Ss[i];
    }
}

static inline size_t retention_smem(int dk, int vs) {
    return ((size_t)2 * RT_CHUNK * (dk + 1) + (size_t)RT_CHUNK * vs + (size_t)RT_CHUNK * (RT_CHUNK + 1) +
            (size_t)dk * vs + RT_CHUNK + 1) * sizeof(float);
}

// q, k: [T, >= H*dk] rows (strided), v: [T, >= H*dv]; out float32 [T, H*dv]; state float32
// [slots, H, dk, dv]; decay float32 [H] on the device; rope [T, rot] (cos then sin) or null.
TGO_API int tgo_retention(const void* q, long long q_stride, const void* k, long long k_stride,
                          const void* v, long long v_stride, int dtype, float* out, int B, int H,
                          int dk, int dv, const float* decay, float k_scale, int act, const float* rope,
                          int rot, const int* q_start, const int* state_slots, float* state,
                          cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || dk <= 0 || dv <= 0 || rot < 0 || rot > dk || (rot & 1) || H > 65535)
        return TGO_E_BAD_ARG;
    int vs = 32;                                    // columns of the state a block owns
    while (vs > 8 && retention_smem(dk, vs) > 200 * 1024) vs >>= 1;
    const size_t smem = retention_smem(dk, vs);
    if (smem > 200 * 1024) return TGO_E_BAD_ARG;
    const dim3 grid(B, H, (dv + vs - 1) / vs), block(RT_THREADS);
    if (grid.z > 65535) return TGO_E_BAD_ARG;
    if (dtype == TGO_BF16) {
        auto kern = retention_kernel<bf16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, grid, block, smem, stream, (const bf16*)q, q_stride,
                              (const bf16*)k, k_stride, (const bf16*)v, v_stride, out, H, dk, dv, vs,
                              decay, k_scale, act, rope, rot, q_start, state_slots, state);
    }
    if (dtype == TGO_F32) {
        auto kern = retention_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, grid, block, smem, stream, (const float*)q, q_stride,
                              (const float*)k, k_stride, (const float*)v, v_stride, out, H, dk, dv,
                              vs, decay, k_scale, act, rope, rot, q_start, state_slots, state);
    }
    return TGO_E_BAD_ARG;
}

// ------------------------------------------------------------------ a step of single tokens
// One token a request: o = decay S^T q + (q . k) v and S <- decay S + k v^T straight from and
// to global memory, a block per (request, head, 32 columns of S), every element of S read
// once and written once.
#define RD_THREADS 128
template <typename T>
__global__ void __launch_bounds__(RD_THREADS)
retention_decode_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                        long long k_stride, const T* __restrict__ v, long long v_stride,
                        float* __restrict__ out, int H, int dk, int dv,
                        const float* __restrict__ decay, float k_scale, int act,
                        const float* __restrict__ rope, int rot,
                        const int* __restrict__ state_slots, float* __restrict__ state) {
    extern __shared__ float smem[];
    float* qs = smem;                 // [dk]
    float* ks = qs + dk;              // [dk]
    float* red = ks + dk;             // [RD_THREADS / 32][32]
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
    const int c = blockIdx.z * 32 + lane;
    const size_t t = (size_t)b;
    const float* cs = rope ? rope + t * rot : nullptr;
    const T* qr = q + t * q_stride + (size_t)h * dk;
    const T* kr = k + t * k_stride + (size_t)h * dk;
    for (int d = threadIdx.x; d < dk; d += RD_THREADS) {
        qs[d] = cs ? rotated(qr, cs, d, rot, act) : taken(qr[d], act);
        ks[d] = (cs ? rotated(kr, cs, d, rot, act) : taken(kr[d], act)) * k_scale;
    }
    __syncthreads();
    const float g = decay[h];
    const float vc = c < dv ? taken(v[t * v_stride + (size_t)h * dv + c], act) : 0.f;
    float* Sg = state + (((size_t)state_slots[b] * H + h) * dk) * dv;
    float far = 0.f, qk = 0.f;
    constexpr int RG = RD_THREADS / 32;
    // eight rows of the state a thread and turn: all their loads first (the stores into the
    // same array would otherwise hold every next load back), then the arithmetic and the stores
    for (int d0 = rg; d0 < dk; d0 += RG * 8) {
        float sv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int d = d0 + u * RG;
            sv[u] = (d < dk && c < dv) ? Sg[(size_t)d * dv + c] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int d = d0 + u * RG;
            if (d < dk) {
                qk += qs[d] * ks[d];
                if (c < dv) {
                    far += qs[d] * sv[u];
                    Sg[(size_t)d * dv + c] = g * sv[u] + ks[d] * vc;
                }
            }
        }
    }
    __shared__ float qk_part[RG];
    red[rg * 32 + lane] = far;
    if (lane == 0) qk_part[rg] = qk;        // every lane of a row group holds the same part
    __syncthreads();
    if (rg == 0 && c < dv) {
        float f = 0.f, a = 0.f;
#pragma unroll
        for (int x = 0; x < RG; ++x) {
            f += red[x * 32 + lane];
            a += qk_part[x];
        }
        out[(t * H + h) * dv + c] = g * f + a * vc;
    }
}

// --------------------------------------------------------------- prompt portions, by chunks
// The tokens of a step are cut into chunks of up to RC_CHUNK tokens of one request (a list
// the host makes: first token row and count of each chunk). Three launches, every chunk of
// every head in parallel in the first and the third:
//
//   summaries   U_c = sum_j decay^(n-1-j) k_j v_j^T                [dk, dv] per (chunk, head)
//   scan        per request and head, chunk after chunk: P_c = S; S <- decay^n S + U_c (the
//               state before each chunk replaces its summary; the last S is the new state)
//   outputs     o_i = sum_{j<=i} decay^(i-j) (q_i . k_j) v_j + decay^(i+1) P_c^T q_i
#define RC_CHUNK 64
#define RC_THREADS 256
#define RC_VS 64                      // columns of V and of the state taken at a time

template <typename T>
__device__ __forceinline__ void load_rotated(float* dst, int ld, const T* __restrict__ x, long long stride,
                                             int h, int dk, const float* __restrict__ rope, int rot,
                                             int tok0, int n, float mul, int act) {
    // four elements a turn, their loads first: a row of the chunk is short, and a loop that
    // waits for every element's loads in turn is bound by their latency
    for (int i0 = threadIdx.x; i0 < n * dk; i0 += 4 * RC_THREADS) {
        float val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * RC_THREADS;
            if (i < n * dk) {
                const int r = i / dk, d = i % dk;
                const size_t t = (size_t)(tok0 + r);
                const T* row = x + t * stride + (size_t)h * dk;
                val[u] = (rope ? rotated(row, rope + t * rot, d, rot, act) : taken(row[d], act)) * mul;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * RC_THREADS;
            if (i < n * dk) dst[(i / dk) * ld + i % dk] = val[u];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(RC_THREADS)
retention_summaries_kernel(const T* __restrict__ k, long long k_stride, const T* __restrict__ v,
                           long long v_stride, int H, int dk, int dv,
                           const float* __restrict__ decay, float k_scale, int act,
                           const float* __restrict__ rope, int rot,
                           const int* __restrict__ chunk_tok0, const int* __restrict__ chunk_ntok,
                           float* __restrict__ U) {
    extern __shared__ float smem[];
    const int ldk = dk + 1;
    float* Ks = smem;                         // [RC_CHUNK][dk + 1], rows times decay^(n-1-j)
    float* Vs = Ks + RC_CHUNK * ldk;          // [RC_CHUNK][RC_VS]
    float* pw = Vs + RC_CHUNK * RC_VS;        // [RC_CHUNK + 1]
    pdl_wait();
    const int ci = blockIdx.x, h = blockIdx.y;
    const int tok0 = chunk_tok0[ci], n = chunk_ntok[ci];
    if (threadIdx.x == 0) {
        float x = 1.f;
        const float g = decay[h];
        for (int i = 0; i <= RC_CHUNK; ++i) { pw[i] = x; x *= g; }
    }
    load_rotated(Ks, ldk, k, k_stride, h, dk, rope, rot, tok0, n, k_scale, act);
    __syncthreads();
    for (int i = threadIdx.x; i < n * dk; i += RC_THREADS) Ks[(i / dk) * ldk + i % dk] *= pw[n - 1 - i / dk];
    float* Uo = U + ((size_t)ci * H + h) * dk * dv;
    for (int c0 = 0; c0 < dv; c0 += RC_VS) {
        const int nc = dv - c0 < RC_VS ? dv - c0 : RC_VS;
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < n * RC_VS; i += RC_THREADS) {
            const int r = i / RC_VS, c = i % RC_VS;
            Vs[i] = c < nc ? taken(v[(size_t)(tok0 + r) * v_stride + (size_t)h * dv + c0 + c], act) : 0.f;
        }
        __syncthreads();
        // U[d][c] over 4 x 4 register tiles: tiles of rows d0.., columns cc..
        const int tiles_c = RC_VS / 4, tiles_d = (dk + 3) / 4;
        for (int tile = threadIdx.x; tile < tiles_d * tiles_c; tile += RC_THREADS) {
            const int d0 = (tile / tiles_c) * 4, cc = (tile % tiles_c) * 4;
            float acc[4][4] = {};
            for (int j = 0; j < n; ++j) {
                const float4 vv = *(const float4*)(Vs + j * RC_VS + cc);
                float kk[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) kk[x] = d0 + x < dk ? Ks[j * ldk + d0 + x] : 0.f;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    acc[x][0] += kk[x] * vv.x; acc[x][1] += kk[x] * vv.y;
                    acc[x][2] += kk[x] * vv.z; acc[x][3] += kk[x] * vv.w;
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y)
                    if (d0 + x < dk && cc + y < nc) Uo[(size_t)(d0 + x) * dv + c0 + cc + y] = acc[x][y];
        }
    }
}

// grid (requests, heads, ceil(dk * dv / 256)): a thread an element of the state
__global__ void retention_scan_kernel(int H, int dk, int dv, const float* __restrict__ decay,
                                      const int* __restrict__ q_start,
                                      const int* __restrict__ state_slots,
                                      const int* __restrict__ chunk_first, float* __restrict__ U,
                                      float* __restrict__ state) {
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    if (e >= dk * dv) return;
    const int n_tok = q_start[b + 1] - q_start[b];
    if (n_tok <= 0) return;
    const int chunks = (n_tok + RC_CHUNK - 1) / RC_CHUNK;
    const float g = decay[h];
    float gfull = 1.f;
    for (int i = 0; i < RC_CHUNK; ++i) gfull *= g;
    float* sp = state + ((size_t)state_slots[b] * H + h) * dk * dv + e;
    float s = *sp;
    const int c0 = chunk_first[b];
    const size_t step = (size_t)H * dk * dv;
    float* ub = U + ((size_t)c0 * H + h) * dk * dv + e;
    for (int cb = 0; cb < chunks; cb += 16) {        // sixteen summaries loaded ahead of their use
        float u[16];
#pragma unroll
        for (int x = 0; x < 16; ++x) u[x] = cb + x < chunks ? ub[(size_t)(cb + x) * step] : 0.f;
#pragma unroll
        for (int x = 0; x < 16; ++x) {
            const int c = cb + x;
            if (c < chunks) {
                ub[(size_t)c * step] = s;
                float gn = gfull;
                if (c == chunks - 1) {
                    gn = 1.f;
                    for (int i = 0; i < n_tok - c * RC_CHUNK; ++i) gn *= g;
                }
                s = gn * s + u[x];
            }
        }
    }
    *sp = s;
}

template <typename T>
__global__ void __launch_bounds__(RC_THREADS)
retention_outputs_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                         long long k_stride, const T* __restrict__ v, long long v_stride,
                         float* __restrict__ out, int H, int dk, int dv,
                         const float* __restrict__ decay, float k_scale, int act,
                         const float* __restrict__ rope, int rot,
                         const int* __restrict__ chunk_tok0, const int* __restrict__ chunk_ntok,
                         const float* __restrict__ P) {
    extern __shared__ float smem[];
    const int ldk = dk + 1, lda = RC_CHUNK + 1;
    float* Qs = smem;                          // [RC_CHUNK][dk + 1]
    float* Ks = Qs + RC_CHUNK * ldk;           // [RC_CHUNK][dk + 1]
    float* As = Ks + RC_CHUNK * ldk;           // [RC_CHUNK][RC_CHUNK + 1]
    float* Vs = As + RC_CHUNK * lda;           // [RC_CHUNK][RC_VS]
    float* Ss = Vs + RC_CHUNK * RC_VS;         // [dk][RC_VS]
    float* pw = Ss + (size_t)dk * RC_VS;       // [RC_CHUNK + 1]
    pdl_wait();
    const int ci = blockIdx.x, h = blockIdx.y;
    const int tok0 = chunk_tok0[ci], n = chunk_ntok[ci];
    if (threadIdx.x == 0) {
        float x = 1.f;
        const float g = decay[h];
        for (int i = 0; i <= RC_CHUNK; ++i) { pw[i] = x; x *= g; }
    }
    load_rotated(Qs, ldk, q, q_stride, h, dk, rope, rot, tok0, n, 1.f, act);
    load_rotated(Ks, ldk, k, k_stride, h, dk, rope, rot, tok0, n, k_scale, act);
    __syncthreads();
    // A[i][j] = decay^(i-j) q_i . k_j (j <= i), 4 x 4 tiles
    {
        const int tiles = RC_CHUNK / 4;
        for (int tile = threadIdx.x; tile < tiles * tiles; tile += RC_THREADS) {
            const int i0 = (tile / tiles) * 4, j0 = (tile % tiles) * 4;
            if (i0 >= n || j0 >= n) continue;
            float acc[4][4] = {};
            if (j0 <= i0 + 3) {
                for (int d = 0; d < dk; ++d) {
                    float qq[4], kk[4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        qq[x] = Qs[(i0 + x) * ldk + d];
                        kk[x] = Ks[(j0 + x) * ldk + d];
                    }
#pragma unroll
                    for (int x = 0; x < 4; ++x)
#pragma unroll
                        for (int y = 0; y < 4; ++y) acc[x][y] += qq[x] * kk[y];
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y) {
                    const int i = i0 + x, j = j0 + y;
                    As[i * lda + j] = (j <= i && i < n) ? acc[x][y] * pw[i - j] : 0.f;
                }
        }
    }
    const float* Pc = P + ((size_t)ci * H + h) * dk * dv;
    for (int c0 = 0; c0 < dv; c0 += RC_VS) {
        const int nc = dv - c0 < RC_VS ? dv - c0 : RC_VS;
        __syncthreads();
#pragma unroll 4
        for (int i = threadIdx.x; i < n * RC_VS; i += RC_THREADS) {
            const int r = i / RC_VS, c = i % RC_VS;
            Vs[i] = c < nc ? taken(v[(size_t)(tok0 + r) * v_stride + (size_t)h * dv + c0 + c], act) : 0.f;
        }
#pragma unroll 8
        for (int i = threadIdx.x; i < dk * RC_VS; i += RC_THREADS) {
            const int d = i / RC_VS, c = i % RC_VS;
            Ss[i] = c < nc ? Pc[(size_t)d * dv + c0 + c] : 0.f;
        }
        __syncthreads();
        const int tiles_c = RC_VS / 4, tiles_i = (n + 3) / 4;
        for (int tile = threadIdx.x; tile < tiles_i * tiles_c; tile += RC_THREADS) {
            const int i0 = (tile / tiles_c) * 4, cc = (tile % tiles_c) * 4;
            float near[4][4] = {}, far[4][4] = {};
            const int jmax = i0 + 3 < n - 1 ? i0 + 3 : n - 1;
            for (int j = 0; j <= jmax; ++j) {
                const float4 vv = *(const float4*)(Vs + j * RC_VS + cc);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float a = As[(i0 + x) * lda + j];        // rows >= n were zeroed or unused
                    near[x][0] += a * vv.x; near[x][1] += a * vv.y; near[x][2] += a * vv.z; near[x][3] += a * vv.w;
                }
            }
            for (int d = 0; d < dk; ++d) {
                const float4 ss = *(const float4*)(Ss + d * RC_VS + cc);
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float qq = Qs[(i0 + x) * ldk + d];
                    far[x][0] += qq * ss.x; far[x][1] += qq * ss.y; far[x][2] += qq * ss.z; far[x][3] += qq * ss.w;
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x)
#pragma unroll
                for (int y = 0; y < 4; ++y)
                    if (i0 + x < n && cc + y < nc)
                        out[((size_t)(tok0 + i0 + x) * H + h) * dv + c0 + cc + y] =
                            near[x][y] + pw[i0 + x + 1] * far[x][y];
        }
    }
}

static inline size_t summaries_smem(int dk) {
    return ((size_t)RC_CHUNK * (dk + 1) + (size_t)RC_CHUNK * RC_VS + RC_CHUNK + 1) * sizeof(float);
}
static inline size_t outputs_smem(int dk) {
    return ((size_t)2 * RC_CHUNK * (dk + 1) + (size_t)RC_CHUNK * (RC_CHUNK + 1) + (size_t)RC_CHUNK * RC_VS +
            (size_t)dk * RC_VS + RC_CHUNK + 1) * sizeof(float);
}

TGO_API int tgo_retention_chunk_tokens() { return RC_CHUNK; }

// 1 if the chunked kernels (and the single-token kernel) take these sizes.
TGO_API int tgo_retention_chunked_supports(int H, int dk, int dv) {
    return (H > 0 && H <= 65535 && dk > 0 && dv > 0 && outputs_smem(dk) <= 200 * 1024) ? 1 : 0;
}

template <typename T>
static int retention_chunked(const T* q, long long q_stride, const T* k, long long k_stride, const T* v,
                             long long v_stride, float* out, int B, int H, int dk, int dv, const float* decay,
                             float k_scale, int act, const float* rope, int rot, const int* q_start,
                             const int* state_slots, float* state, int chunks, const int* chunk_tok0,
                             const int* chunk_ntok, const int* chunk_first, float* scratch, int single,
                             cudaStream_t stream) {
    if (single) {
        const size_t smem = ((size_t)2 * dk + RD_THREADS) * sizeof(float);
        return tgo_launch_pdl(retention_decode_kernel<T>, dim3(B, H, (dv + 31) / 32), dim3(RD_THREADS), smem,
                              stream, q, q_stride, k, k_stride, v, v_stride, out, H, dk, dv, decay, k_scale, act,
                              rope, rot, state_slots, state);
    }
    const size_t s1 = summaries_smem(dk), s3 = outputs_smem(dk);
    auto k1 = retention_summaries_kernel<T>;
    auto k3 = retention_outputs_kernel<T>;
    if (s1 > 48 * 1024) cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s1);
    if (s3 > 48 * 1024) cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s3);
    int rc = tgo_launch_pdl(k1, dim3(chunks, H), dim3(RC_THREADS), s1, stream, k, k_stride, v, v_stride, H, dk,
                            dv, decay, k_scale, act, rope, rot, chunk_tok0, chunk_ntok, scratch);
    if (rc) return rc;
    rc = tgo_launch_pdl(retention_scan_kernel, dim3(B, H, (dk * dv + 255) / 256), dim3(256), 0, stream, H, dk,
                        dv, decay, q_start, state_slots, chunk_first, scratch, state);
    if (rc) return rc;
    return tgo_launch_pdl(k3, dim3(chunks, H), dim3(RC_THREADS), s3, stream, q, q_stride, k, k_stride, v,
                          v_stride, out, H, dk, dv, decay, k_scale, act, rope, rot, chunk_tok0, chunk_ntok,
                          (const float*)scratch);
}

// As tgo_retention, by chunks. chunk_tok0 / chunk_ntok: the chunks (at most
// tgo_retention_chunk_tokens() tokens of one request each, a request's chunks in order and
// next to each other); chunk_first [B]: index of each request's first chunk; scratch: float32
// [chunks, H, dk, dv]. single != 0: every request brings one token (no chunk lists needed).
TGO_API int tgo_retention_chunked(const void* q, long long q_stride, const void* k, long long k_stride,
                                  const void* v, long long v_stride, int dtype, float* out, int B, int H,
                                  int dk, int dv, const float* decay, float k_scale, int act, const float* rope,
                                  int rot, const int* q_start, const int* state_slots, float* state,
                                  int chunks, const int* chunk_tok0, const int* chunk_ntok,
                                  const int* chunk_first, float* scratch, int single, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (!tgo_retention_chunked_supports(H, dk, dv) || rot < 0 || rot > dk || (rot & 1) ||
        (!single && (chunks <= 0 || !chunk_tok0 || !chunk_ntok || !chunk_first || !scratch)))
        return TGO_E_BAD_ARG;
    if (dtype == TGO_BF16)
        return retention_chunked<bf16>((const bf16*)q, q_stride, (const bf16*)k, k_stride, (const bf16*)v,
                                       v_stride, out, B, H, dk, dv, decay, k_scale, act, rope, rot, q_start,
                                       state_slots, state, chunks, chunk_tok0, chunk_ntok, chunk_first, scratch,
                                       single, stream);
    if (dtype == TGO_F32)
        return retention_chunked<float>((const float*)q, q_stride, (const float*)k, k_stride, (const float*)v,
                                        v_stride, out, B, H, dk, dv, decay, k_scale, act, rope, rot, q_start,
                                        state_slots, state, chunks, chunk_tok0, chunk_ntok, chunk_first,
                                        scratch, single, stream);
    return TGO_E_BAD_ARG;
}
