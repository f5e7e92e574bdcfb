// Kernels around a residual that is kept as several streams (hyper-connections), a norm taken in
// groups, and the token shift.
//
// The residual is float32 [T, S, W]: S streams of width W for every token (S = 1 is the ordinary
// residual).  A sublayer reads u = sum_s c_in[s] x_s, normalises it, and its output y goes back as
// x_t <- sum_s mix[s, t] x_s + c_out[t] y for all streams t at once.  All arithmetic is float32; one
// rounding at the store of what the next product reads.
#include "common.cuh"

#define ST_MAX_STREAMS 16

// ---------------------------------------------------------------------------------------------
// out[r, :] = groupnorm_rms(sum_s coef[s] x[row(r), s, :]) * w
// The width is cut into ``groups`` equal consecutive parts, each divided by its own
// sqrt(mean(part^2) + eps).  coef null: the plain sum of the streams.  One block per row; the sums
// are taken per group in an order that depends on the width and the group count only.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void streams_norm_kernel(const float* __restrict__ x, const float* __restrict__ coef,
                                    const float* __restrict__ w, T* __restrict__ out, const int* __restrict__ rows,
                                    int S, int W, int groups, float eps) {
    ce_pdl_begin();
    extern __shared__ __align__(16) float st_smem[];
    float* u = st_smem;                 // W
    float* scratch = st_smem + W;       // 32
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * S * W;
    float c[ST_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < ST_MAX_STREAMS; ++s) c[s] = s < S ? (coef ? coef[s] : 1.0f) : 0.f;
    for (int j = threadIdx.x; j < W; j += blockDim.x) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < ST_MAX_STREAMS; ++s)
            if (s < S) a = fmaf(c[s], xr[(size_t)s * W + j], a);
        u[j] = a;
    }
    __syncthreads();
    int gw = W / groups;
    T* o = out + (size_t)r * W;
    for (int g = 0; g < groups; ++g) {
        const float* ug = u + g * gw;
        float ss = 0.f;
        for (int j = threadIdx.x; j < gw; j += blockDim.x) ss = fmaf(ug[j], ug[j], ss);
        ss = ce_block_sum(ss, scratch);
        float inv = 1.0f / sqrtf(ss / (float)gw + eps);
        for (int j = threadIdx.x; j < gw; j += blockDim.x) CeType<T>::store(o + g * gw + j, ug[j] * inv * w[g * gw + j]);
    }
}

extern "C" int ce_streams_norm(const float* x, const float* coef, const float* w, void* out, int out_dtype,
                               const int* rows, int R, int S, int W, int groups, float eps, cudaStream_t stream) {
    if (R == 0) return CE_OK;
    if (!x || !w || !out) return ce_fail(CE_ERR_ARG, "ce_streams_norm: null pointer");
    if (S <= 0 || S > ST_MAX_STREAMS) return ce_fail(CE_ERR_SIZE, "ce_streams_norm: %d streams (1..%d)", S, ST_MAX_STREAMS);
    if (W <= 0 || groups <= 0 || W % groups) return ce_fail(CE_ERR_SIZE, "ce_streams_norm: width %d in %d groups", W, groups);
    size_t smem = (size_t)(W + 32) * sizeof(float);
    if (smem > 200 * 1024) return ce_fail(CE_ERR_SIZE, "ce_streams_norm: width %d is too large", W);
    int threads = W / groups >= 1024 ? 512 : 256;
    if (out_dtype == CE_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ce_note("streams_norm_kernel");
        ce_launch(streams_norm_kernel<float>, R, threads, smem, stream, x, coef, w, (float*)out, rows, S, W, groups, eps);
    } else if (out_dtype == CE_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ce_note("streams_norm_kernel");
        ce_launch(streams_norm_kernel<__nv_bfloat16>, R, threads, smem, stream, x, coef, w, (__nv_bfloat16*)out, rows, S, W, groups, eps);
    } else
        return ce_fail(CE_ERR_ARG, "ce_streams_norm: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_streams_norm");
}

// ---------------------------------------------------------------------------------------------
// Token shift: out[t] = h[t] + (prev(t) - h[t]) * mu, where prev(t) is the row of the token before t
// in its sequence as it was before the shift: h[t - 1] inside the step, the row kept in
// state[slot] for the first token of a portion, zeros at position 0.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mu,
                                   const float* __restrict__ state, T* __restrict__ out,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ seq_slot, const int* __restrict__ q_start, int W) {
    ce_pdl_begin();
    int t = blockIdx.x;
    int b = seq_of_token[t];
    const float* prev = nullptr;
    if (t > q_start[b]) prev = h + (size_t)(t - 1) * W;
    else if (positions[t] > 0) prev = state + (size_t)seq_slot[b] * W;
    const float* hr = h + (size_t)t * W;
    T* o = out + (size_t)t * W;
    for (int j = threadIdx.x; j < W; j += blockDim.x) {
        float v = hr[j], p = prev ? prev[j] : 0.f;
        CeType<T>::store(o + j, fmaf(p - v, mu[j], v));
    }
}

extern "C" int ce_token_shift(const float* h, const float* mu, const float* state, void* out, int out_dtype,
                              const int* positions, const int* seq_of_token, const int* seq_slot, const int* q_start,
                              int T, int W, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!h || !mu || !state || !out || !positions || !seq_of_token || !seq_slot || !q_start)
        return ce_fail(CE_ERR_ARG, "ce_token_shift: null pointer");
    int threads = W >= 1024 ? 256 : 128;
    if (out_dtype == CE_F32) {
        ce_note("token_shift_kernel");
        ce_launch(token_shift_kernel<float>, T, threads, 0, stream, h, mu, state, (float*)out, positions, seq_of_token, seq_slot, q_start, W);
    } else if (out_dtype == CE_BF16) {
        ce_note("token_shift_kernel");
        ce_launch(token_shift_kernel<__nv_bfloat16>, T, threads, 0, stream, h, mu, state, (__nv_bfloat16*)out, positions, seq_of_token, seq_slot, q_start, W);
    } else
        return ce_fail(CE_ERR_ARG, "ce_token_shift: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_token_shift");
}

// state[slot(b), :] = h[last token of sequence b, :]
__global__ void save_last_rows_kernel(const float* __restrict__ h, float* __restrict__ state,
                                      const int* __restrict__ seq_slot, const int* __restrict__ q_start, int W) {
    ce_pdl_begin();
    int b = blockIdx.x;
    int last = q_start[b + 1] - 1;
    if (last < q_start[b]) return;
    const float* hr = h + (size_t)last * W;
    float* s = state + (size_t)seq_slot[b] * W;
    for (int j = threadIdx.x; j < W; j += blockDim.x) s[j] = hr[j];
}

extern "C" int ce_save_last_rows(const float* h, float* state, const int* seq_slot, const int* q_start, int B, int W,
                                 cudaStream_t stream) {
    if (B == 0) return CE_OK;
    if (!h || !state || !seq_slot || !q_start) return ce_fail(CE_ERR_ARG, "ce_save_last_rows: null pointer");
    ce_note("save_last_rows_kernel");
    ce_launch(save_last_rows_kernel, B, 256, 0, stream, h, state, seq_slot, q_start, W);
    return ce_check_launch("ce_save_last_rows");
}

// ---------------------------------------------------------------------------------------------
// x[t, :, :] <- mix^T applied to the old streams + c_out * (y + bias): for every (token, column) the S
// old values are read, the S new ones written.  mix is [from, to]; bias may be null.
// ---------------------------------------------------------------------------------------------
template <int SMAX>
__global__ void streams_write_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                                     const float* __restrict__ c_out, const float* __restrict__ bias, int S, int W,
                                     size_t total) {
    ce_pdl_begin();
    __shared__ float m[SMAX * SMAX], co[SMAX];
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) m[i] = mix[i];
    for (int i = threadIdx.x; i < S; i += blockDim.x) co[i] = c_out[i];
    __syncthreads();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t t = e / W;
        int j = (int)(e % W);
        float* xr = x + t * S * W + j;
        float old[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) old[s] = s < S ? xr[(size_t)s * W] : 0.f;
        float yv = y[e] + (bias ? bias[j] : 0.f);
#pragma unroll
        for (int to = 0; to < SMAX; ++to) {
            if (to < S) {
                float a = 0.f;
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) a = fmaf(m[s * S + to], old[s], a);
                xr[(size_t)to * W] = fmaf(co[to], yv, a);
            }
        }
    }
}

extern "C" int ce_streams_write(float* x, const float* y, const float* mix, const float* c_out, const float* bias,
                                int T, int S, int W, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!x || !y || !mix || !c_out) return ce_fail(CE_ERR_ARG, "ce_streams_write: null pointer");
    if (S <= 0 || S > ST_MAX_STREAMS) return ce_fail(CE_ERR_SIZE, "ce_streams_write: %d streams (1..%d)", S, ST_MAX_STREAMS);
    size_t total = (size_t)T * W;
    int blocks = (int)((total + 255) / 256 < (size_t)148 * 16 ? (total + 255) / 256 : (size_t)148 * 16);
    ce_note("streams_write_kernel");
    if (S <= 4) ce_launch(streams_write_kernel<4>, blocks, 256, 0, stream, x, y, mix, c_out, bias, S, W, total);
    else if (S <= 8) ce_launch(streams_write_kernel<8>, blocks, 256, 0, stream, x, y, mix, c_out, bias, S, W, total);
    else ce_launch(streams_write_kernel<ST_MAX_STREAMS>, blocks, 128, 0, stream, x, y, mix, c_out, bias, S, W, total);
    return ce_check_launch("ce_streams_write");
}

// x[t, s, :] = x0[t, :] for every stream s
__global__ void streams_broadcast_kernel(const float* __restrict__ x0, float* __restrict__ x, int S, int W, size_t total) {
    ce_pdl_begin();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t t = e / W;
        int j = (int)(e % W);
        float v = x0[e];
        for (int s = 0; s < S; ++s) x[(t * S + s) * W + j] = v;
    }
}

extern "C" int ce_streams_broadcast(const float* x0, float* x, int T, int S, int W, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!x0 || !x) return ce_fail(CE_ERR_ARG, "ce_streams_broadcast: null pointer");
    size_t total = (size_t)T * W;
    int blocks = (int)((total + 255) / 256 < (size_t)148 * 16 ? (total + 255) / 256 : (size_t)148 * 16);
    ce_note("streams_broadcast_kernel");
    ce_launch(streams_broadcast_kernel, blocks, 256, 0, stream, x0, x, S, W, total);
    return ce_check_launch("ce_streams_broadcast");
}

// out[m, :] += bias (out float32 or the activation dtype, bias float32)
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, const float* __restrict__ bias, int N, int ld, size_t total) {
    ce_pdl_begin();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t m = e / N;
        int j = (int)(e % N);
        T* p = out + m * ld + j;
        CeType<T>::store(p, CeType<T>::load(p) + bias[j]);
    }
}

extern "C" int ce_add_bias(void* out, int dtype, const float* bias, int M, int N, int ld, cudaStream_t stream) {
    if (M == 0 || N == 0) return CE_OK;
    if (!out || !bias) return ce_fail(CE_ERR_ARG, "ce_add_bias: null pointer");
    size_t total = (size_t)M * N;
    int blocks = (int)((total + 255) / 256 < (size_t)148 * 16 ? (total + 255) / 256 : (size_t)148 * 16);
    if (dtype == CE_F32) {
        ce_note("add_bias_kernel");
        ce_launch(add_bias_kernel<float>, blocks, 256, 0, stream, (float*)out, bias, N, ld, total);
    } else if (dtype == CE_BF16) {
        ce_note("add_bias_kernel");
        ce_launch(add_bias_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)out, bias, N, ld, total);
    } else
        return ce_fail(CE_ERR_ARG, "ce_add_bias: unknown dtype %d", dtype);
    return ce_check_launch("ce_add_bias");
}
