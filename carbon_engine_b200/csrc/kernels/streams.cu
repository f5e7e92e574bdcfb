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

// The same for widths and groups that are multiples of four: float4 loads of every stream, float4 through shared
// memory, four outputs a store.
__device__ __forceinline__ void st_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void st_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 r;
    r.x = *reinterpret_cast<unsigned*>(&lo); r.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = r;
}

template <typename T, int SMAX>
__global__ void streams_norm_vec_kernel(const float* __restrict__ x, const float* __restrict__ coef,
                                        const float* __restrict__ w, T* __restrict__ out, const int* __restrict__ rows,
                                        int S, int W, int groups, float eps) {
    ce_pdl_begin();
    extern __shared__ __align__(16) float st_smem[];
    float4* u4 = reinterpret_cast<float4*>(st_smem);        // W / 4
    float* scratch = st_smem + W;                           // 32
    int r = blockIdx.x, n4 = W >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * S * W);
    float c[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) c[s] = s < S ? (coef ? coef[s] : 1.0f) : 0.f;
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
        float4 v[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
            if (s < S) v[s] = xr[(size_t)s * n4 + j];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
            if (s < S) { acc.x = fmaf(c[s], v[s].x, acc.x); acc.y = fmaf(c[s], v[s].y, acc.y); acc.z = fmaf(c[s], v[s].z, acc.z); acc.w = fmaf(c[s], v[s].w, acc.w); }
        u4[j] = acc;
    }
    __syncthreads();
    int g4 = n4 / groups;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    T* o = out + (size_t)r * W;
    for (int g = 0; g < groups; ++g) {
        const float4* ug = u4 + g * g4;
        float ss = 0.f;
        for (int j = threadIdx.x; j < g4; j += blockDim.x) {
            float4 v = ug[j];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = ce_block_sum(ss, scratch);
        float inv = 1.0f / sqrtf(ss / (float)(4 * g4) + eps);
        for (int j = threadIdx.x; j < g4; j += blockDim.x) {
            float4 v = ug[j], wv = w4[g * g4 + j];
            st_store4(o + 4 * (g * g4 + j), v.x * inv * wv.x, v.y * inv * wv.y, v.z * inv * wv.z, v.w * inv * wv.w);
        }
    }
}

template <typename T>
static void launch_streams_norm(const float* x, const float* coef, const float* w, T* out, const int* rows, int R, int S, int W,
                                int groups, float eps, size_t smem, cudaStream_t stream) {
    bool vec = W % 4 == 0 && (W / groups) % 4 == 0 && ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out)) & 15) == 0 && S <= 8;
    if (vec) {
        int threads = W >= 4096 ? 512 : W >= 1024 ? 256 : 128;
        ce_note("streams_norm_vec_kernel");
        if (S <= 4) {
            if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_vec_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            ce_launch(streams_norm_vec_kernel<T, 4>, R, threads, smem, stream, x, coef, w, out, rows, S, W, groups, eps);
        } else {
            if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_vec_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            ce_launch(streams_norm_vec_kernel<T, 8>, R, threads, smem, stream, x, coef, w, out, rows, S, W, groups, eps);
        }
        return;
    }
    int threads = W / groups >= 1024 ? 512 : 256;
    if (smem > 48 * 1024) cudaFuncSetAttribute(streams_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce_note("streams_norm_kernel");
    ce_launch(streams_norm_kernel<T>, R, threads, smem, stream, x, coef, w, out, rows, S, W, groups, eps);
}

extern "C" int ce_streams_norm(const float* x, const float* coef, const float* w, void* out, int out_dtype,
                               const int* rows, int R, int S, int W, int groups, float eps, cudaStream_t stream) {
    if (R == 0) return CE_OK;
    if (!x || !w || !out) return ce_fail(CE_ERR_ARG, "ce_streams_norm: null pointer");
    if (S <= 0 || S > ST_MAX_STREAMS) return ce_fail(CE_ERR_SIZE, "ce_streams_norm: %d streams (1..%d)", S, ST_MAX_STREAMS);
    if (W <= 0 || groups <= 0 || W % groups) return ce_fail(CE_ERR_SIZE, "ce_streams_norm: width %d in %d groups", W, groups);
    size_t smem = (size_t)(W + 32) * sizeof(float);
    if (smem > 200 * 1024) return ce_fail(CE_ERR_SIZE, "ce_streams_norm: width %d is too large", W);
    if (out_dtype == CE_F32) launch_streams_norm<float>(x, coef, w, (float*)out, rows, R, S, W, groups, eps, smem, stream);
    else if (out_dtype == CE_BF16) launch_streams_norm<__nv_bfloat16>(x, coef, w, (__nv_bfloat16*)out, rows, R, S, W, groups, eps, smem, stream);
    else return ce_fail(CE_ERR_ARG, "ce_streams_norm: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_streams_norm");
}

// ---------------------------------------------------------------------------------------------
// Token shift: out[t] = h[t] + (prev(t) - h[t]) * mu, where prev(t) is the row of the token before t
// in its sequence as it was before the shift: h[t - 1] inside the step, the row kept in
// state[slot] for the first token of a portion, zeros at position 0.  With ``save`` the kept row becomes the
// portion's last row (written by the block that read the old one, so the two never race).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_kernel(const float* __restrict__ h, const float* __restrict__ mu,
                                   float* __restrict__ state, T* __restrict__ out,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ seq_slot, const int* __restrict__ q_start, int W, int save) {
    ce_pdl_begin();
    int t = blockIdx.x;
    int b = seq_of_token[t];
    const float* hr = h + (size_t)t * W;
    T* o = out + (size_t)t * W;
    if (t > q_start[b]) {
        const float* prev = h + (size_t)(t - 1) * W;
        for (int j = threadIdx.x; j < W; j += blockDim.x) {
            float v = hr[j];
            CeType<T>::store(o + j, fmaf(prev[j] - v, mu[j], v));
        }
        return;
    }
    // The first token of the sequence's portion: the only block that touches the sequence's kept row.  Each
    // thread reads its elements of the row and then (save) puts the portion's last row in their place.
    float* kept = state + (size_t)seq_slot[b] * W;
    const float* last = h + (size_t)(q_start[b + 1] - 1) * W;
    bool first = positions[t] == 0;
    for (int j = threadIdx.x; j < W; j += blockDim.x) {
        float v = hr[j], p = first ? 0.f : kept[j];
        CeType<T>::store(o + j, fmaf(p - v, mu[j], v));
        if (save) kept[j] = last[j];
    }
}

extern "C" int ce_token_shift(const float* h, const float* mu, float* state, void* out, int out_dtype,
                              const int* positions, const int* seq_of_token, const int* seq_slot, const int* q_start,
                              int T, int W, int save, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!h || !mu || !state || !out || !positions || !seq_of_token || !seq_slot || !q_start)
        return ce_fail(CE_ERR_ARG, "ce_token_shift: null pointer");
    int threads = W >= 1024 ? 256 : 128;
    if (out_dtype == CE_F32) {
        ce_note("token_shift_kernel");
        ce_launch(token_shift_kernel<float>, T, threads, 0, stream, h, mu, state, (float*)out, positions, seq_of_token, seq_slot, q_start, W, save);
    } else if (out_dtype == CE_BF16) {
        ce_note("token_shift_kernel");
        ce_launch(token_shift_kernel<__nv_bfloat16>, T, threads, 0, stream, h, mu, state, (__nv_bfloat16*)out, positions, seq_of_token, seq_slot, q_start, W, save);
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

// The same, four columns a thread (width a multiple of four, 16-byte aligned rows).
template <int SMAX>
__global__ void streams_write_vec_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ mix,
                                         const float* __restrict__ c_out, const float* __restrict__ bias, int S, int W4,
                                         size_t total4) {
    ce_pdl_begin();
    __shared__ float m[SMAX * SMAX], co[SMAX];
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) m[i] = mix[i];
    for (int i = threadIdx.x; i < S; i += blockDim.x) co[i] = c_out[i];
    __syncthreads();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += stride) {
        size_t t = e / W4;
        int j = (int)(e % W4);
        float4* xr = reinterpret_cast<float4*>(x) + t * S * W4 + j;
        float4 old[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
            if (s < S) old[s] = xr[(size_t)s * W4];
        float4 yv = reinterpret_cast<const float4*>(y)[e];
        if (bias) {
            float4 b = reinterpret_cast<const float4*>(bias)[j];
            yv.x += b.x; yv.y += b.y; yv.z += b.z; yv.w += b.w;
        }
#pragma unroll
        for (int to = 0; to < SMAX; ++to) {
            if (to < S) {
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) {
                        float c = m[s * S + to];
                        a.x = fmaf(c, old[s].x, a.x); a.y = fmaf(c, old[s].y, a.y); a.z = fmaf(c, old[s].z, a.z); a.w = fmaf(c, old[s].w, a.w);
                    }
                float c = co[to];
                xr[(size_t)to * W4] = make_float4(fmaf(c, yv.x, a.x), fmaf(c, yv.y, a.y), fmaf(c, yv.z, a.z), fmaf(c, yv.w, a.w));
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
    if (W % 4 == 0 && S <= 4 && ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)bias)) & 15) == 0) {
        size_t total4 = total / 4;
        int vblocks = (int)((total4 + 255) / 256 < (size_t)148 * 16 ? (total4 + 255) / 256 : (size_t)148 * 16);
        ce_note("streams_write_vec_kernel");
        ce_launch(streams_write_vec_kernel<4>, vblocks, 256, 0, stream, x, y, mix, c_out, bias, S, W / 4, total4);
        return ce_check_launch("ce_streams_write");
    }
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
