// Row-wise kernels for layers that normalise the OUTPUT of a sublayer into a float32 residual
// stream, and for attention whose queries and keys are normalised over the whole projection:
//
//   residual_rmsnorm      r <- r + y / sqrt(mean(y^2) + eps) * gamma   (r float32; also a copy of the new r
//                         in the activations' type, which the next sublayer's products read)
//                         with a second norm (weight, eps) the copy is the new r under THAT norm: the input of the next sublayer
//                         of a layer that normalises in front of and behind every sublayer
//   stream_add            x += (e) + v: what a model adds to the stream between two runs of a span of layers
//   polynorm              a n(z) + b n(z^2) + c n(z^3) + e, n = division by the row's root mean square
//   softcap               x <- c tanh(x / c) on float logits
//   act_mul               rows [gate | up] -> act(gate) * up, act = SiLU or the tanh form of GELU
//   qk_norm_rope_write    rows [q | k | gate logits]: q and k each divided by the root mean square of their
//                         WHOLE row part and multiplied by a weight of that width, the leading `rot` elements
//                         of every head rotated (pairs i, i + rot/2), q written out, k written into the
//                         token's cache slot as the key and - unnormalised, unrotated - as the value;
//                         sigmoid of the gate logits written as float
//   gated_group_rmsnorm   (y * silu(z)) normalised in equal parts of a row, times a weight
//
// All arithmetic is float; storage is float or bfloat16 per argument.  Any width.
#include "common.cuh"

__device__ __forceinline__ float rv_load_any(const void* p, int dtype, size_t i) {
    return dtype == RV_DTYPE_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void rv_store_any(void* p, int dtype, size_t i, float v) {
    if (dtype == RV_DTYPE_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// ------------------------------------------------------------------ residual + RMSNorm of a sublayer's output
__global__ void __launch_bounds__(256)
residual_rmsnorm_kernel(const void* __restrict__ y, int y_dtype, const void* __restrict__ gamma, int gamma_dtype,
                        const float* res_in, float* res_out, void* __restrict__ rounded, int rounded_dtype,
                        int cols, float eps, const void* __restrict__ next_gamma, int next_dtype, float next_eps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * cols;
    float ss = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = rv_load_any(y, y_dtype, base + i);
        ss = fmaf(v, v, ss);
    }
    ss = rv_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)cols + eps);
    if (!next_gamma) {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            float v = rv_load_any(y, y_dtype, base + i) * r * rv_load_param(gamma, gamma_dtype, i);
            if (res_in) v += res_in[base + i];
            if (res_out) res_out[base + i] = v;
            if (rounded) rv_store_any(rounded, rounded_dtype, base + i, v);
        }
        return;
    }
    // the new stream is written, its own mean square gathered on the way, and the copy for the next sublayer is the
    // new stream under that sublayer's norm (every thread reads back what it wrote itself)
    float s2 = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float v = rv_load_any(y, y_dtype, base + i) * r * rv_load_param(gamma, gamma_dtype, i);
        if (res_in) v += res_in[base + i];
        res_out[base + i] = v;
        s2 = fmaf(v, v, s2);
    }
    s2 = rv_block_sum(s2, scratch);
    const float r2 = 1.0f / sqrtf(s2 / (float)cols + next_eps);
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
        rv_store_any(rounded, rounded_dtype, base + i, res_out[base + i] * r2 * rv_load_param(next_gamma, next_dtype, i));
}

RV_EXPORT int rv_residual_rmsnorm_next(const void* y, int y_dtype, const void* gamma, int gamma_dtype, const float* res_in,
                                       float* res_out, void* rounded, int rounded_dtype, int rows, int cols, float eps,
                                       const void* next_gamma, int next_dtype, float next_eps, cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if ((y_dtype | gamma_dtype | rounded_dtype | next_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (next_gamma && (!res_out || !rounded)) return RV_ERR_UNSUPPORTED;
    if (rows == 0) return RV_OK;
    RV_LAUNCH_ST = rv_launch(residual_rmsnorm_kernel, dim3(rows), dim3(cols >= 1024 ? 256 : 128), 0, stream, y, y_dtype, gamma,
                             gamma_dtype, res_in, res_out, rounded, rounded_dtype, cols, eps, next_gamma, next_dtype, next_eps);
    return rv_launch_status();
}

RV_EXPORT int rv_residual_rmsnorm(const void* y, int y_dtype, const void* gamma, int gamma_dtype, const float* res_in,
                                  float* res_out, void* rounded, int rounded_dtype, int rows, int cols, float eps,
                                  cudaStream_t stream) {
    return rv_residual_rmsnorm_next(y, y_dtype, gamma, gamma_dtype, res_in, res_out, rounded, rounded_dtype, rows, cols, eps,
                                    nullptr, 0, 0.f, stream);
}

// ------------------------------------------------------------------ additions to the stream, PolyNorm, capped logits
// x[t, :] += (e[t, :]) + v[:], float32 stream; e optional; v a row of a parameter table in either type.
__global__ void stream_add_kernel(float* __restrict__ x, const float* __restrict__ e, const void* __restrict__ v, int v_dtype,
                                  int cols, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float a = x[i] + rv_load_param(v, v_dtype, (int)(i % cols));
        if (e) a += e[i];
        x[i] = a;
    }
}

RV_EXPORT int rv_stream_add(float* x, const float* e, const void* v, int v_dtype, int rows, int cols, cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if (v_dtype & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * cols;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(stream_add_kernel, dim3(blocks), dim3(256), 0, stream, x, e, v, v_dtype, cols, total);
    return rv_launch_status();
}

// out = a n(z) + b n(z^2) + c n(z^3) + e, n(v) = v / sqrt(mean(v^2) + eps) over the row; coef = (a, b, c, e) float.
// The row is read once: it waits in shared memory (as float) between the pass that gathers the three mean squares and
// the pass that writes; rows too long for that are read twice.
__global__ void __launch_bounds__(512)
polynorm_kernel(const void* __restrict__ z, int z_dtype, const float* __restrict__ coef, void* __restrict__ out, int out_dtype,
                int cols, float eps, int keep) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    extern __shared__ float row[];
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * cols;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    const bool vec = keep && z_dtype == RV_DTYPE_F32 && (cols & 3) == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 15) == 0;      // float rows in 16-byte words
    if (vec) {
        const float4* src = reinterpret_cast<const float4*>((const float*)z + base);
        for (int i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 q = src[i];
            reinterpret_cast<float4*>(row)[i] = q;
            const float v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float v2 = v[j] * v[j], v3 = v2 * v[j];
                s1 = fmaf(v[j], v[j], s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
            }
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = rv_load_any(z, z_dtype, base + i), v2 = v * v, v3 = v2 * v;
            if (keep) row[i] = v;
            s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
        }
    }
    s1 = rv_block_sum(s1, scratch);
    s2 = rv_block_sum(s2, scratch);
    s3 = rv_block_sum(s3, scratch);
    const float n = (float)cols;
    const float a = coef[0] / sqrtf(s1 / n + eps), b = coef[1] / sqrtf(s2 / n + eps), c = coef[2] / sqrtf(s3 / n + eps), e = coef[3];
    if (vec) {
        for (int i = threadIdx.x; i < cols / 4; i += blockDim.x) {
            const float4 q = reinterpret_cast<const float4*>(row)[i];
            const float v[4] = {q.x, q.y, q.z, q.w};
            float r[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float v2 = v[j] * v[j]; r[j] = a * v[j] + b * v2 + c * (v2 * v[j]) + e; }
            if (out_dtype == RV_DTYPE_F32) {
                reinterpret_cast<float4*>((float*)out + base)[i] = make_float4(r[0], r[1], r[2], r[3]);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
                uint2 w;
                w.x = *reinterpret_cast<uint32_t*>(&lo); w.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>((__nv_bfloat16*)out + base)[i] = w;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = keep ? row[i] : rv_load_any(z, z_dtype, base + i), v2 = v * v;
        rv_store_any(out, out_dtype, base + i, a * v + b * v2 + c * (v2 * v) + e);
    }
}

RV_EXPORT int rv_polynorm(const void* z, int z_dtype, const float* coef, void* out, int out_dtype, int rows, int cols, float eps,
                          cudaStream_t stream) {
    if (rows < 0 || cols <= 0) return RV_ERR_BAD_SIZE;
    if ((z_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const int keep = cols <= 24 * 1024 ? 1 : 0;            // 96 KB of floats: two CTAs still fit an SM
    static RvPerDevice configured;
    if (int st = rv_configure_smem(configured, polynorm_kernel, 96 * 1024)) return st;
    RV_LAUNCH_ST = rv_launch(polynorm_kernel, dim3(rows), dim3(cols >= 4096 ? 512 : (cols >= 1024 ? 256 : 128)), keep ? (size_t)cols * 4 : 0,
                             stream, z, z_dtype, coef, out, out_dtype, cols, eps, keep);
    return rv_launch_status();
}

// x <- cap * tanh(x / cap), float, in place.
__global__ void softcap_kernel(float* __restrict__ x, float cap, size_t total) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    const float inv = 1.0f / cap;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

RV_EXPORT int rv_softcap(float* x, float cap, long long total, cudaStream_t stream) {
    if (total < 0 || !(cap > 0.f)) return RV_ERR_BAD_SIZE;
    if (total == 0) return RV_OK;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, x, cap, (size_t)total);
    return rv_launch_status();
}

// ------------------------------------------------------------------ activation-gated product
__device__ __forceinline__ float rv_gelu_tanh(float z) {
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(u));
}
__device__ __forceinline__ float rv_silu(float z) { return z / (1.0f + expf(-z)); }

__global__ void act_mul_kernel(const void* __restrict__ gate_up, int in_dtype, void* __restrict__ out, int out_dtype,
                               int inter, size_t total, int act) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / inter, c = i - row * inter;
        const float g = rv_load_any(gate_up, in_dtype, row * 2 * inter + c);
        const float u = rv_load_any(gate_up, in_dtype, row * 2 * inter + inter + c);
        rv_store_any(out, out_dtype, i, (act == 1 ? rv_gelu_tanh(g) : rv_silu(g)) * u);
    }
}

RV_EXPORT int rv_act_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, int rows, int inter, int act,
                         cudaStream_t stream) {
    if (rows < 0 || inter <= 0) return RV_ERR_BAD_SIZE;
    if ((in_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (act != 0 && act != 1) return RV_ERR_UNSUPPORTED;
    if (rows == 0) return RV_OK;
    const size_t total = (size_t)rows * inter;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    RV_LAUNCH_ST = rv_launch(act_mul_kernel, dim3(blocks), dim3(256), 0, stream, gate_up, in_dtype, out, out_dtype, inter, total, act);
    return rv_launch_status();
}

// ------------------------------------------------------------------ whole-row q/k norm, rotation, cache write, gate
// One block per token.  Row layout: [q: nh*hd | k: nkv*hd | gate logits: nh] (gate part only if gate_out).
__global__ void __launch_bounds__(256)
qk_norm_rope_write_kernel(const void* __restrict__ proj, int in_dtype, int row_stride,
                          const void* __restrict__ q_gamma, const void* __restrict__ k_gamma, int gamma_dtype,
                          const int* __restrict__ positions, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                          int rot, int table_rows, const int* __restrict__ slot_mapping, void* __restrict__ cache,
                          void* __restrict__ q_out, int out_dtype, float* __restrict__ gate_out,
                          int nh, int nkv, int hd, int page_size, float eps, int write_kv) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const size_t row = (size_t)t * row_stride;
    const int qw = nh * hd, kw = nkv * hd;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < qw; i += blockDim.x) { const float v = rv_load_any(proj, in_dtype, row + i); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < kw; i += blockDim.x) { const float v = rv_load_any(proj, in_dtype, row + qw + i); sk = fmaf(v, v, sk); }
    sq = rv_block_sum(sq, scratch);
    sk = rv_block_sum(sk, scratch);
    const float rq = 1.0f / sqrtf(sq / (float)qw + eps), rk = 1.0f / sqrtf(sk / (float)kw + eps);
    int pos = positions[t];
    if (pos < 0) pos = 0;
    if (pos >= table_rows) pos = table_rows - 1;      // the host refuses such positions; never read outside
    const int half = rot >> 1;
    const int slot = write_kv ? slot_mapping[t] : -1;
    const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
    // one item = one element of q or k that is not the second of a rotation pair: i < half (pair with i + half) or i >= rot
    const int per_head = hd - half;
    const int n_items = (nh + (write_kv ? nkv : 0)) * per_head;
    for (int item = threadIdx.x; item < n_items; item += blockDim.x) {
        const int head = item / per_head;
        int i = item - head * per_head;
        const bool paired = i < half;
        if (!paired) i += half;                        // elements rot .. hd-1 pass unrotated
        const bool is_q = head < nh;
        const int col = is_q ? head * hd : (head - nh) * hd;      // within q or within k
        const size_t src = row + (is_q ? 0 : qw) + col;
        const void* gamma = is_q ? q_gamma : k_gamma;
        const float r = is_q ? rq : rk;
        void* dst;
        size_t d0;
        if (is_q) { dst = q_out; d0 = (size_t)t * qw + col; }
        else {
            if (slot < 0) continue;
            dst = cache;
            d0 = ((((size_t)page * 2) * nkv + (head - nh)) * page_size + off) * hd;
        }
        const float raw_a = rv_load_any(proj, in_dtype, src + i);
        const float a = raw_a * r * rv_load_param(gamma, gamma_dtype, col + i);
        if (paired) {
            const float raw_b = rv_load_any(proj, in_dtype, src + i + half);
            const float b = raw_b * r * rv_load_param(gamma, gamma_dtype, col + i + half);
            float c = 1.f, s = 0.f;
            if (cos_t) { c = cos_t[(size_t)pos * half + i]; s = sin_t[(size_t)pos * half + i]; }
            rv_store_any(dst, out_dtype, d0 + i, a * c - b * s);
            rv_store_any(dst, out_dtype, d0 + i + half, b * c + a * s);
            if (!is_q) {                                // the value is the key as projected
                const size_t v0 = d0 + (size_t)nkv * page_size * hd;
                rv_store_any(cache, out_dtype, v0 + i, raw_a);
                rv_store_any(cache, out_dtype, v0 + i + half, raw_b);
            }
        } else {
            rv_store_any(dst, out_dtype, d0 + i, a);
            if (!is_q) rv_store_any(cache, out_dtype, d0 + (size_t)nkv * page_size * hd + i, raw_a);
        }
    }
    if (gate_out)
        for (int h = threadIdx.x; h < nh; h += blockDim.x) {
            const float g = rv_load_any(proj, in_dtype, row + qw + kw + h);
            gate_out[(size_t)t * nh + h] = 1.0f / (1.0f + expf(-g));
        }
}

RV_EXPORT int rv_qk_norm_rope_write(const void* proj, int in_dtype, int row_stride, const void* q_gamma, const void* k_gamma,
                                    int gamma_dtype, const int* positions, const float* cos_t, const float* sin_t, int rot,
                                    int table_rows, const int* slot_mapping, void* cache, void* q_out, int out_dtype,
                                    float* gate_out, int n_tokens, int nh, int nkv, int hd, int page_size, float eps,
                                    int write_kv, cudaStream_t stream) {
    if (n_tokens < 0 || nh <= 0 || nkv <= 0 || hd <= 0 || page_size <= 0 || table_rows <= 0) return RV_ERR_BAD_SIZE;
    if (rot < 0 || rot > hd || (rot & 1)) return RV_ERR_BAD_SIZE;
    if (row_stride < (nh + nkv) * hd + (gate_out ? nh : 0)) return RV_ERR_BAD_SIZE;
    if ((in_dtype | gamma_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (n_tokens == 0) return RV_OK;
    if (!cos_t) rot = 0;
    RV_LAUNCH_ST = rv_launch(qk_norm_rope_write_kernel, dim3(n_tokens), dim3(256), 0, stream, proj, in_dtype, row_stride, q_gamma,
                             k_gamma, gamma_dtype, positions, cos_t, sin_t, rot, table_rows, slot_mapping, cache, q_out,
                             out_dtype, gate_out, nh, nkv, hd, page_size, eps, write_kv);
    return rv_launch_status();
}

// ------------------------------------------------------------------ gate, then RMSNorm in equal parts of a row
// out[t, c] = n(y[t, c] * silu(z[t, c])) * gamma[c], n = RMSNorm over the part of the row that c lies in.
// Grid (tokens, parts).  z is read from rows of `z_stride` elements (a slice of a wider projection).
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ y, const void* __restrict__ z, int z_dtype, int z_stride,
                           const void* __restrict__ gamma, int gamma_dtype, void* __restrict__ out, int out_dtype,
                           int width, int part, float eps) {
    rv_pdl_launch_dependents();
    rv_pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x, c0 = blockIdx.y * part;
    const size_t yb = (size_t)t * width + c0, zb = (size_t)t * z_stride + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = y[yb + i] * rv_silu(rv_load_any(z, z_dtype, zb + i));
        ss = fmaf(v, v, ss);
    }
    ss = rv_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(ss / (float)part + eps);
    for (int i = threadIdx.x; i < part; i += blockDim.x) {
        const float v = y[yb + i] * rv_silu(rv_load_any(z, z_dtype, zb + i));
        rv_store_any(out, out_dtype, yb + i, v * r * rv_load_param(gamma, gamma_dtype, c0 + i));
    }
}

RV_EXPORT int rv_gated_group_rmsnorm(const float* y, const void* z, int z_dtype, int z_stride, const void* gamma, int gamma_dtype,
                                     void* out, int out_dtype, int rows, int width, int parts, float eps, cudaStream_t stream) {
    if (rows < 0 || width <= 0 || parts <= 0 || width % parts || z_stride < width || parts > 65535) return RV_ERR_BAD_SIZE;
    if ((z_dtype | gamma_dtype | out_dtype) & ~1) return RV_ERR_BAD_DTYPE;
    if (rows == 0) return RV_OK;
    const int part = width / parts;
    RV_LAUNCH_ST = rv_launch(gated_group_rmsnorm_kernel, dim3(rows, parts), dim3(part >= 1024 ? 256 : 128), 0, stream, y, z, z_dtype,
                             z_stride, gamma, gamma_dtype, out, out_dtype, width, part, eps);
    return rv_launch_status();
}
