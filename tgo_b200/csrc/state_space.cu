// A selective state-space mixer's recurrent part (the form known as Mamba-2): a short causal
// convolution per channel with its last inputs kept per request, and the scan
//
//   dt_t = softplus(raw_t + dt_bias_h)                      per head h, float32
//   S_t  = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T      S is [N, P], float32
//   y_t  = S_t^T C_t + D_h x_t
//
// over each request's tokens of the step, from and into the request's float32 state. Head h
// reads B and C of group floor(h / (H / G)). Everything after the convolution's input is
// float32 whatever the storage type of the projections.
//
// A request's state row (float32, `state_stride` floats apart) holds the scan's state
// [H][N][P] at `ssm_offset` and the convolution's last taps - 1 inputs [taps - 1][C] (oldest
// first) at `conv_offset`.
#include "common.cuh"

// ------------------------------------------------------------------------- convolution
// y[t][c] = silu(bias[c] + sum_j w[c][j] x[t - (taps - 1 - j)][c]); inputs before the step's
// first token come from the request's kept inputs, zeros before the request's start (a fresh
// state row is zero). x is a column view [T, C] in the storage type; y float32 [T, C].
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_act_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w,
                       const float* __restrict__ bias, float* __restrict__ y, int C, int taps,
                       const int* __restrict__ seq_ids, const int* __restrict__ q_start,
                       const int* __restrict__ state_slots, const float* __restrict__ state,
                       long long state_stride, long long conv_offset) {
    pdl_wait();
    const int t = blockIdx.x;
    const int b = seq_ids[t];
    const int r = t - q_start[b];                       // place among the request's tokens
    const float* kept = state + (size_t)state_slots[b] * state_stride + conv_offset;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float a = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;               // how many tokens before this one
            float v;
            if (back <= r) v = to_f32(x[(size_t)(t - back) * x_stride + c]);
            else v = kept[(size_t)(taps - 1 - (back - r)) * C + c];
            a = fmaf(w[(size_t)c * taps + j], v, a);
        }
        y[(size_t)t * C + c] = a / (1.f + expf(-a));
    }
}

// After the convolution has run: the kept inputs of every request become the last taps - 1
// of (kept inputs, then the step's inputs). A thread per (request, channel).
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_keep_kernel(const T* __restrict__ x, long long x_stride, int C, int taps,
                        const int* __restrict__ q_start, const int* __restrict__ state_slots,
                        float* __restrict__ state, long long state_stride, long long conv_offset) {
    pdl_wait();
    const int b = blockIdx.x;
    const int t0 = q_start[b], n = q_start[b + 1] - t0;
    float* kept = state + (size_t)state_slots[b] * state_stride + conv_offset;
    const int keep = taps - 1;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        // ascending i reads kept[n + i] before any later write could reach it (n + i >= i)
        for (int i = 0; i < keep; ++i) {
            const int at = n + i;                        // place in (kept, then new)
            const float v = at < keep ? kept[(size_t)at * C + c]
                                      : to_f32(x[(size_t)(t0 + at - keep) * x_stride + c]);
            kept[(size_t)i * C + c] = v;
        }
    }
}

TGO_API int tgo_causal_conv_act(const void* x, long long x_stride, int dtype, const float* w,
                                const float* bias, float* y, int T, int B, int C, int taps,
                                const int* seq_ids, const int* q_start, const int* state_slots,
                                float* state, long long state_stride, long long conv_offset,
                                cudaStream_t stream) {
    if (T <= 0 || B <= 0) return 0;
    if (C <= 0 || taps <= 0 || taps > 64 || state_stride < conv_offset + (long long)(taps - 1) * C)
        return TGO_E_BAD_ARG;
    const int cy = (C + 255) / 256 > 64 ? 64 : (C + 255) / 256;
    int rc;
    if (dtype == TGO_BF16)
        rc = tgo_launch_pdl(causal_conv_act_kernel<bf16>, dim3(T, cy), dim3(256), 0, stream, (const bf16*)x,
                            x_stride, w, bias, y, C, taps, seq_ids, q_start, state_slots,
                            (const float*)state, state_stride, conv_offset);
    else if (dtype == TGO_F32)
        rc = tgo_launch_pdl(causal_conv_act_kernel<float>, dim3(T, cy), dim3(256), 0, stream, (const float*)x,
                            x_stride, w, bias, y, C, taps, seq_ids, q_start, state_slots,
                            (const float*)state, state_stride, conv_offset);
    else
        return TGO_E_BAD_ARG;
    if (rc || taps == 1) return rc;
    if (dtype == TGO_BF16)
        return tgo_launch_pdl(causal_conv_keep_kernel<bf16>, dim3(B, cy), dim3(256), 0, stream, (const bf16*)x,
                              x_stride, C, taps, q_start, state_slots, state, state_stride, conv_offset);
    return tgo_launch_pdl(causal_conv_keep_kernel<float>, dim3(B, cy), dim3(256), 0, stream, (const float*)x,
                          x_stride, C, taps, q_start, state_slots, state, state_stride, conv_offset);
}

// -------------------------------------------------------------------------------- scan
// A block per (request, head, 32 columns of P). 256 threads: thread (column c = tid / 8,
// slice s = tid % 8) keeps rows n = 32 i + 4 s + j (j = 0..3) of its column of S in registers
// for the whole walk over the request's tokens; a token's y[c] is the sum of the eight
// slices' partial sums (three shuffles, the same order for every token). The tokens' B, C, x
// and dt come through shared memory SS_TOK at a time, two buffers: the next tokens load while
// these are walked; B and C are read four rows at a time. The order of every sum depends on
// the sizes alone, so a token's result does not depend on how the tokens were cut or batched
// beyond the state's own history, which is the same sequence of updates whatever the cut.
#define SS_TOK 16
#define SS_COLS 32

// a 4-byte asynchronous copy into shared memory (zeros when !valid)
__device__ __forceinline__ void ss_copy4(float* dst, const float* src, bool valid) {
    const int n = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n));
}

template <typename T, int NI>
__global__ void __launch_bounds__(256)
selective_scan_kernel(const float* __restrict__ xbc, int C, const T* __restrict__ dt_raw,
                      long long dt_stride, const float* __restrict__ dt_bias,
                      const float* __restrict__ A_log, const float* __restrict__ D,
                      float* __restrict__ y, int H, int G, int N, int P,
                      const int* __restrict__ q_start, const int* __restrict__ state_slots,
                      float* __restrict__ state, long long state_stride, long long ssm_offset) {
    constexpr int NP = NI * 8;                           // N rounded up to whole rounds of 32
    extern __shared__ __align__(16) float smem[];
    // per buffer: B [SS_TOK][NP], C [SS_TOK][NP], x [SS_TOK][SS_COLS], dt [SS_TOK], decay [SS_TOK]
    constexpr int BUF = 2 * SS_TOK * NP + SS_TOK * SS_COLS + 2 * SS_TOK;
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * SS_COLS;
    const int g = h / (H / G);
    const int inner = H * P;
    const int col = threadIdx.x >> 3, s = threadIdx.x & 7;
    const int c = c0 + col;
    const bool live = c < P;
    const int t0 = q_start[b], n_tok = q_start[b + 1] - t0;
    float* Sg = state + (size_t)state_slots[b] * state_stride + ssm_offset + (size_t)h * N * P;
    // the state comes and goes through shared memory, so that global memory sees whole rows
    // of 32 columns (the staging buffers are idle then; [N][33] floats fit in them)
    float S[NI];
    for (int i = threadIdx.x; i < N * SS_COLS; i += 256) {
        const int n = i / SS_COLS, cc = i % SS_COLS;
        smem[n * (SS_COLS + 1) + cc] = c0 + cc < P ? Sg[(size_t)n * P + c0 + cc] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int n = 32 * (i >> 2) + 4 * s + (i & 3);
        S[i] = n < N ? smem[n * (SS_COLS + 1) + col] : 0.f;
    }
    __syncthreads();
    const float A = expf(A_log[h]);
    const float Dh = D ? D[h] : 0.f;
    const float bias = dt_bias ? dt_bias[h] : 0.f;
    auto stage = [&](int base, int buf) {
        float* Bs = smem + buf * BUF;
        float* Cs = Bs + SS_TOK * NP;
        float* xs = Cs + SS_TOK * NP;
        float* dts = xs + SS_TOK * SS_COLS;
        float* das = dts + SS_TOK;
        const int nt = n_tok - base < SS_TOK ? n_tok - base : SS_TOK;
        for (int i = threadIdx.x; i < nt * NP; i += 256) {
            const int r = i / NP, n = i % NP;
            const float* row = xbc + (size_t)(t0 + base + r) * C + inner + (size_t)g * N;
            ss_copy4(Bs + i, n < N ? row + n : xbc, n < N);
            ss_copy4(Cs + i, n < N ? row + (size_t)G * N + n : xbc, n < N);
        }
        for (int i = threadIdx.x; i < nt * SS_COLS; i += 256) {
            const int r = i / SS_COLS, cc = i % SS_COLS;
            const bool ok = c0 + cc < P;
            ss_copy4(xs + i, ok ? xbc + (size_t)(t0 + base + r) * C + (size_t)h * P + c0 + cc : xbc, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::);
        if (threadIdx.x < nt) {
            const float z = to_f32(dt_raw[(size_t)(t0 + base + threadIdx.x) * dt_stride + h]) + bias;
            const float dt = z > 20.f ? z : log1pf(expf(z));
            dts[threadIdx.x] = dt;
            das[threadIdx.x] = expf(-A * dt);
        }
    };
    stage(0, 0);
    for (int base = 0, buf = 0; base < n_tok; base += SS_TOK, buf ^= 1) {
        const int nt = n_tok - base < SS_TOK ? n_tok - base : SS_TOK;
        if (base + SS_TOK < n_tok) {
            stage(base + SS_TOK, buf ^ 1);                // the buffer the last pass left
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const float* Bs = smem + buf * BUF;
        const float* Cs = Bs + SS_TOK * NP;
        const float* xs = Cs + SS_TOK * NP;
        const float* dts = xs + SS_TOK * SS_COLS;
        const float* das = dts + SS_TOK;
        for (int r = 0; r < nt; ++r) {
            const float x = xs[r * SS_COLS + col];
            const float dx = dts[r] * x, da = das[r];
            float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < NI / 4; ++i4) {
                const float4 bq = *(const float4*)(Bs + r * NP + 32 * i4 + 4 * s);
                const float4 cq = *(const float4*)(Cs + r * NP + 32 * i4 + 4 * s);
                S[4 * i4 + 0] = fmaf(da, S[4 * i4 + 0], dx * bq.x);
                S[4 * i4 + 1] = fmaf(da, S[4 * i4 + 1], dx * bq.y);
                S[4 * i4 + 2] = fmaf(da, S[4 * i4 + 2], dx * bq.z);
                S[4 * i4 + 3] = fmaf(da, S[4 * i4 + 3], dx * bq.w);
                part[0] = fmaf(S[4 * i4 + 0], cq.x, part[0]);
                part[1] = fmaf(S[4 * i4 + 1], cq.y, part[1]);
                part[2] = fmaf(S[4 * i4 + 2], cq.z, part[2]);
                part[3] = fmaf(S[4 * i4 + 3], cq.w, part[3]);
            }
            float sum = (part[0] + part[1]) + (part[2] + part[3]);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            if (s == 0 && live) y[(size_t)(t0 + base + r) * inner + (size_t)h * P + c] = sum + Dh * x;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int n = 32 * (i >> 2) + 4 * s + (i & 3);
        if (n < N) smem[n * (SS_COLS + 1) + col] = S[i];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < N * SS_COLS; i += 256) {
        const int n = i / SS_COLS, cc = i % SS_COLS;
        if (c0 + cc < P) Sg[(size_t)n * P + c0 + cc] = smem[n * (SS_COLS + 1) + cc];
    }
}

template <typename T, int NI>
static int launch_scan(const float* xbc, int C, const T* dt_raw, long long dt_stride,
                       const float* dt_bias, const float* A_log, const float* D, float* y, int B,
                       int H, int G, int N, int P, const int* q_start, const int* state_slots,
                       float* state, long long state_stride, long long ssm_offset,
                       cudaStream_t stream) {
    const size_t smem = 2 * ((size_t)2 * SS_TOK * NI * 8 + SS_TOK * SS_COLS + 2 * SS_TOK) * sizeof(float);
    auto kernel = selective_scan_kernel<T, NI>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return tgo_launch_pdl(kernel, dim3(B, H, (P + SS_COLS - 1) / SS_COLS), dim3(256),
                          smem, stream, xbc, C, dt_raw, dt_stride, dt_bias, A_log, D, y, H, G, N, P,
                          q_start, state_slots, state, state_stride, ssm_offset);
}

template <typename T>
static int scan_by_size(const float* xbc, int C, const T* dt_raw, long long dt_stride,
                        const float* dt_bias, const float* A_log, const float* D, float* y, int B,
                        int H, int G, int N, int P, const int* q_start, const int* state_slots,
                        float* state, long long state_stride, long long ssm_offset,
                        cudaStream_t stream) {
#define SS_GO(NI) launch_scan<T, NI>(xbc, C, dt_raw, dt_stride, dt_bias, A_log, D, y, B, H, G, N, P, \
                                     q_start, state_slots, state, state_stride, ssm_offset, stream)
    const int ni = (N + 7) / 8;
    if (ni <= 4) return SS_GO(4);
    if (ni <= 8) return SS_GO(8);
    if (ni <= 16) return SS_GO(16);
    return SS_GO(32);
#undef SS_GO
}

// xbc float32 [T, C], C = H P + 2 G N: the convolution's output (x, then B, then C of every
// group); dt_raw a column view [T, H] in the storage type; y float32 [T, H P].
TGO_API int tgo_selective_scan(const float* xbc, int C, const void* dt_raw, long long dt_stride,
                               int dtype, const float* dt_bias, const float* A_log, const float* D,
                               float* y, int B, int H, int G, int N, int P, const int* q_start,
                               const int* state_slots, float* state, long long state_stride,
                               long long ssm_offset, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || N > 256 || P <= 0 || H > 65535 ||
        C != H * P + 2 * G * N || state_stride < ssm_offset + (long long)H * N * P)
        return TGO_E_BAD_ARG;
    if (dtype == TGO_BF16)
        return scan_by_size<bf16>(xbc, C, (const bf16*)dt_raw, dt_stride, dt_bias, A_log, D, y, B, H, G, N,
                                  P, q_start, state_slots, state, state_stride, ssm_offset, stream);
    if (dtype == TGO_F32)
        return scan_by_size<float>(xbc, C, (const float*)dt_raw, dt_stride, dt_bias, A_log, D, y, B, H, G, N,
                                   P, q_start, state_slots, state, state_stride, ssm_offset, stream);
    return TGO_E_BAD_ARG;
}
