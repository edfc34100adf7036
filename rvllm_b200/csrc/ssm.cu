// Kernels of a selective state-space mixer (state-space duality form): a short causal convolution per
// channel with SiLU, and the recurrence
//     S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T ,   y_t = S_t^T C_t + D_h x_t
// per head h (S is N x P; B and C are shared by the heads of a group), with dt = softplus(raw + bias).
//
// Both carry state from step to step per request: the convolution its last taps - 1 inputs, the
// recurrence S.  A request's state lives in one row of a float32 state tensor (`state`, rows of
// `state_stride` floats): S as [heads][N][P] at offset 0, the convolution's inputs as
// [taps - 1][channels] (oldest first) at `conv_off`.  The tokens that a sequence brings to a step are
// contiguous rows [cu_seqlens[s], cu_seqlens[s + 1]); state_slots[s] < 0 marks a padding row, which
// reads and writes no state.  Decays, step sizes, the state and the sums are float32 whatever the
// storage type of the activations.
#include "common.cuh"

__device__ __forceinline__ float rv_load_any(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void rv_store_any(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

#define RV_MAX_TAPS 16

// ------------------------------------------------------------------ causal convolution + SiLU
// out[t, c] = silu(bias[c] + sum_j w[c, j] * in(t - (taps - 1) + j, c)); inputs before the step's first token of the
// sequence come from the request's state (zeros at the start of a sequence: a fresh slot is zeroed).
// `in` is a slice of a wider row: column col0 .. col0 + channels of rows of `in_stride` elements.
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const void* __restrict__ in, int in_dtype, int in_stride, int col0,
                        const void* __restrict__ w, const void* __restrict__ bias, int w_dtype,
                        const int* __restrict__ token_seq, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ state_slots, const float* __restrict__ state, size_t state_stride,
                        size_t conv_off, void* __restrict__ out, int out_dtype, int n_tokens, int channels, int taps, int t0) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = t0 + blockIdx.y;
    if (c >= channels || t >= n_tokens) return;
    const int seq = token_seq[t];
    const int start = cu_seqlens[seq];
    const int i = t - start;
    const int slot = state_slots[seq];
    const float* hist = slot >= 0 ? state + (size_t)slot * state_stride + conv_off : nullptr;
    float acc = bias ? rv_load_param(bias, w_dtype, c) : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int idx = i - (taps - 1) + j;
        float v;
        if (idx >= 0) v = rv_load_any(in, in_dtype, (size_t)(start + idx) * in_stride + col0 + c);
        else v = hist ? hist[(size_t)(taps - 1 + idx) * channels + c] : 0.f;
        acc = fmaf(rv_load_param(w, w_dtype, c * taps + j), v, acc);
    }
    rv_store_any(out, out_dtype, (size_t)t * channels + c, acc / (1.0f + expf(-acc)));
}

// After the convolution of a step: the state becomes the last taps - 1 inputs of each sequence.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const void* __restrict__ in, int in_dtype, int in_stride, int col0,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                         float* __restrict__ state, size_t state_stride, size_t conv_off, int channels, int taps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    if (c >= channels) return;
    const int slot = state_slots[seq];
    if (slot < 0) return;
    const int start = cu_seqlens[seq], n = cu_seqlens[seq + 1] - start;
    float* hist = state + (size_t)slot * state_stride + conv_off;
    float keep[RV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < RV_MAX_TAPS; ++k) {
        if (k < taps - 1) {
            const int idx = n - (taps - 1) + k;            // index among the step's tokens of this sequence
            keep[k] = idx >= 0 ? rv_load_any(in, in_dtype, (size_t)(start + idx) * in_stride + col0 + c)
                               : hist[(size_t)(k + n) * channels + c];
        }
    }
#pragma unroll
    for (int k = 0; k < RV_MAX_TAPS; ++k)
        if (k < taps - 1) hist[(size_t)k * channels + c] = keep[k];
}

RV_EXPORT int rv_causal_conv_silu(const void* in, int in_dtype, int in_stride, int col0, const void* w, const void* bias,
                                  int w_dtype, const int* token_seq, const int* cu_seqlens, const int* state_slots,
                                  float* state, long long state_stride, long long conv_off, void* out, int out_dtype,
                                  int n_tokens, int n_seqs, int channels, int taps, cudaStream_t stream) {
    if (n_tokens < 0 || n_seqs < 0 || channels <= 0 || taps < 1 || taps > RV_MAX_TAPS || col0 < 0 || in_stride < col0 + channels)
        return RV_ERR_BAD_SIZE;
    if ((in_dtype | w_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0 || n_seqs == 0) return RV_OK;
    if (n_tokens > 65535 * 8 || n_seqs > 65535) return RV_ERR_BAD_SIZE;
    const int threads = channels >= 256 ? 256 : 128;
    const int bx = (channels + threads - 1) / threads;
    for (int t0 = 0; t0 < n_tokens; t0 += 65535) {          // (gridDim.y is limited)
        const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
        RV_LAUNCH_ST = rv_launch(causal_conv_silu_kernel, dim3(bx, nt), dim3(threads), 0, stream,
                                 in, in_dtype, in_stride, col0, w, bias, w_dtype, token_seq, cu_seqlens, state_slots,
                                 (const float*)state, (size_t)state_stride, (size_t)conv_off, out, out_dtype,
                                 n_tokens, channels, taps, t0);
        if (RV_LAUNCH_ST != RV_OK) return rv_launch_status();
    }
    if (taps > 1)
        RV_LAUNCH_ST = rv_launch(conv_state_update_kernel, dim3(bx, n_seqs), dim3(threads), 0, stream, in, in_dtype, in_stride, col0,
                                 cu_seqlens, state_slots, state, (size_t)state_stride, (size_t)conv_off, channels, taps);
    return rv_launch_status();
}

// ------------------------------------------------------------------ the recurrence
// Grid (P / 32 column blocks, heads, sequences); 128 threads = 32 columns p x 4 slices of the state dimension: thread
// (p, s) keeps S[n][p] for n = 4 i + s in registers and the four slices of a column add their parts of y with shuffles.
// The tokens of a sequence are walked in chunks of RV_SCAN_CHUNK: B, C, the decay and dt x of a chunk are staged in
// shared memory, then the chunk runs without a barrier per token.
#define RV_SCAN_CHUNK 16
#define RV_SCAN_COLS 32

template <int NPT>
__global__ void __launch_bounds__(128)
ssm_scan_kernel(const void* __restrict__ xbc, int x_dtype, int channels,           // [T, channels]: x | B | C after the convolution
                const void* __restrict__ dt_in, int dt_dtype, int dt_stride, int dt_col0,   // raw dt: column dt_col0 + h of rows of dt_stride
                const void* __restrict__ dt_bias, const void* __restrict__ a_log, const void* __restrict__ d_skip, int p_dtype,
                const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
                float* __restrict__ state, size_t state_stride, float* __restrict__ y,
                int heads, int P, int N, int groups) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ float sm[];
    float* sB = sm;                                   // [chunk][N]
    float* sC = sB + RV_SCAN_CHUNK * N;               // [chunk][N]
    float* sX = sC + RV_SCAN_CHUNK * N;               // [chunk][32]   dt * x
    float* sY = sX + RV_SCAN_CHUNK * RV_SCAN_COLS;    // [chunk][32]
    float* sDec = sY + RV_SCAN_CHUNK * RV_SCAN_COLS;  // [chunk]       exp(-exp(A_log) dt)
    float* sDt = sDec + RV_SCAN_CHUNK;                // [chunk]
    const int seq = blockIdx.z, h = blockIdx.y, p0 = blockIdx.x * RV_SCAN_COLS;
    const int start = cu_seqlens[seq], n_tok = cu_seqlens[seq + 1] - start;
    const int slot = state_slots[seq];
    const int inner = heads * P;
    const int lane_p = threadIdx.x >> 2, slice = threadIdx.x & 3;
    const int p = p0 + lane_p;
    const bool p_ok = p < P;
    if (slot < 0) {                                    // a padding row: no state; its output is zero
        for (int i = threadIdx.x; i < n_tok * RV_SCAN_COLS; i += blockDim.x) {
            const int tk = i / RV_SCAN_COLS, pp = p0 + (i - tk * RV_SCAN_COLS);
            if (pp < P) y[(size_t)(start + tk) * inner + h * P + pp] = 0.f;
        }
        return;
    }
    const int g = h / (heads / groups);
    const float A = -expf(rv_load_param(a_log, p_dtype, h));
    const float bias = rv_load_param(dt_bias, p_dtype, h);
    const float Dh = rv_load_param(d_skip, p_dtype, h);
    float* S = state + (size_t)slot * state_stride + (size_t)h * N * P;
    float s[NPT];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = 4 * i + slice;
        s[i] = (p_ok && n < N) ? S[(size_t)n * P + p] : 0.f;
    }
    const size_t b_col = (size_t)inner + (size_t)g * N, c_col = (size_t)inner + (size_t)groups * N + (size_t)g * N;
    for (int t0 = 0; t0 < n_tok; t0 += RV_SCAN_CHUNK) {
        const int nt = n_tok - t0 < RV_SCAN_CHUNK ? n_tok - t0 : RV_SCAN_CHUNK;
        __syncthreads();                               // the chunk before has been read (and its sY written out)
        if (threadIdx.x < nt) {
            const int tk = threadIdx.x;
            const float raw = rv_load_any(dt_in, dt_dtype, (size_t)(start + t0 + tk) * dt_stride + dt_col0 + h) + bias;
            const float dt = raw > 20.f ? raw : log1pf(expf(raw));
            sDt[tk] = dt;
            sDec[tk] = expf(A * dt);
        }
        for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
            const int tk = i / N, n = i - tk * N;
            const size_t rowb = (size_t)(start + t0 + tk) * channels;
            sB[tk * N + n] = rv_load_any(xbc, x_dtype, rowb + b_col + n);
            sC[tk * N + n] = rv_load_any(xbc, x_dtype, rowb + c_col + n);
        }
        for (int i = threadIdx.x; i < nt * RV_SCAN_COLS; i += blockDim.x) {
            const int tk = i / RV_SCAN_COLS, pp = p0 + (i - tk * RV_SCAN_COLS);
            sX[i] = pp < P ? rv_load_any(xbc, x_dtype, (size_t)(start + t0 + tk) * channels + h * P + pp) : 0.f;
        }
        __syncthreads();
        for (int tk = 0; tk < nt; ++tk) {
            const float dec = sDec[tk];
            const float xv = sX[tk * RV_SCAN_COLS + lane_p];
            const float dx = sDt[tk] * xv;
            const float* Bt = sB + tk * N;
            const float* Ct = sC + tk * N;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
                const int n = 4 * i + slice;
                if (n < N) {
                    s[i] = fmaf(dec, s[i], dx * Bt[n]);
                    acc = fmaf(s[i], Ct[n], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (slice == 0) sY[tk * RV_SCAN_COLS + lane_p] = fmaf(Dh, xv, acc);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nt * RV_SCAN_COLS; i += blockDim.x) {
            const int tk = i / RV_SCAN_COLS, pp = p0 + (i - tk * RV_SCAN_COLS);
            if (pp < P) y[(size_t)(start + t0 + tk) * inner + h * P + pp] = sY[i];
        }
    }
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = 4 * i + slice;
        if (p_ok && n < N) S[(size_t)n * P + p] = s[i];
    }
}

RV_EXPORT int rv_ssm_scan(const void* xbc, int x_dtype, int channels, const void* dt_in, int dt_dtype, int dt_stride, int dt_col0,
                          const void* dt_bias, const void* a_log, const void* d_skip, int p_dtype, const int* cu_seqlens,
                          const int* state_slots, float* state, long long state_stride, float* y, int n_seqs, int heads, int P,
                          int N, int groups, cudaStream_t stream) {
    if (n_seqs < 0 || heads <= 0 || P <= 0 || N <= 0 || groups <= 0 || heads % groups) return RV_ERR_BAD_SIZE;
    if (channels < heads * P + 2 * groups * N || dt_stride < dt_col0 + heads || dt_col0 < 0) return RV_ERR_BAD_SIZE;
    if ((x_dtype | dt_dtype | p_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (N > 256 || heads > 65535 || n_seqs > 65535) return RV_ERR_UNSUPPORTED;
    if (n_seqs == 0) return RV_OK;
    const dim3 grid((P + RV_SCAN_COLS - 1) / RV_SCAN_COLS, heads, n_seqs);
    const size_t smem = sizeof(float) * ((size_t)2 * RV_SCAN_CHUNK * N + 2 * RV_SCAN_CHUNK * RV_SCAN_COLS + 2 * RV_SCAN_CHUNK);
#define RV_SCAN_LAUNCH(NPT)                                                                                                  \
    RV_LAUNCH_ST = rv_launch(ssm_scan_kernel<NPT>, dim3(grid), dim3(128), smem, stream, xbc, x_dtype, channels, dt_in, dt_dtype, \
                             dt_stride, dt_col0, dt_bias, a_log, d_skip, p_dtype, cu_seqlens, state_slots, state,           \
                             (size_t)state_stride, y, heads, P, N, groups)
    if (N <= 16) RV_SCAN_LAUNCH(4);
    else if (N <= 32) RV_SCAN_LAUNCH(8);
    else if (N <= 64) RV_SCAN_LAUNCH(16);
    else if (N <= 128) RV_SCAN_LAUNCH(32);
    else RV_SCAN_LAUNCH(64);
#undef RV_SCAN_LAUNCH
    return rv_launch_status();
}
