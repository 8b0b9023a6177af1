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

template <typename T>
__device__ __forceinline__ float rotated(const T* __restrict__ x, const float* __restrict__ cs,
                                         int i, int rot) {
    const int half = rot >> 1;
    if (i < half) return to_f32(x[i]) * cs[i] - to_f32(x[i + half]) * cs[half + i];
    if (i < rot) return to_f32(x[i]) * cs[i - half] + to_f32(x[i - half]) * cs[i];
    return to_f32(x[i]);
}

template <typename T>
__global__ void __launch_bounds__(RT_THREADS)
retention_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                 long long k_stride, const T* __restrict__ v, long long v_stride,
                 float* __restrict__ out, int H, int dk, int dv, int vs,
                 const float* __restrict__ decay, float k_scale, const float* __restrict__ rope,
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
            Qs[r * dkp + d] = cs ? rotated(qr, cs, d, rot) : to_f32(qr[d]);
            Ks[r * dkp + d] = (cs ? rotated(kr, cs, d, rot) : to_f32(kr[d])) * k_scale;
        }
        for (int i = threadIdx.x; i < n * vs; i += RT_THREADS) {
            const int r = i / vs, c = i % vs;
            Vs[i] = c < nc ? to_f32(v[(size_t)(ts + r) * v_stride + (size_t)h * dv + c0 + c]) : 0.f;
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
                          int dk, int dv, const float* decay, float k_scale, const float* rope,
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
                              decay, k_scale, rope, rot, q_start, state_slots, state);
    }
    if (dtype == TGO_F32) {
        auto kern = retention_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return tgo_launch_pdl(kern, grid, block, smem, stream, (const float*)q, q_stride,
                              (const float*)k, k_stride, (const float*)v, v_stride, out, H, dk, dv,
                              vs, decay, k_scale, rope, rot, q_start, state_slots, state);
    }
    return TGO_E_BAD_ARG;
}
