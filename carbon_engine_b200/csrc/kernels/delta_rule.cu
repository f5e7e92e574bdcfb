// The generalized delta rule: a recurrent mixer whose per-head state S [d, d] (key channel x value
// channel, float32) is carried from token to token:
//
//     S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T        o_t = S_t^T r_t
//
// with the decay w_t = exp(-exp(-1/2) sigmoid(W2 tanh(z_t) + w0)) per key channel (z_t: a narrow
// projection of the token), the removal rate a_t = sigmoid(a_raw + bias), and the unit key
// u_t = k_t / sqrt(sum k_t^2 + 1e-6).  Both the decay and the removal read the OLD state.  Afterwards
// every head's o_t is divided by its root mean square, multiplied by a weight and by sigmoid(gate).
//
// One block per (head, sequence) walks the sequence's tokens of this step in order, from the state its
// slot holds, and stores the state back.  The columns of S are independent of one another, so a column
// lives in the registers of DR_R neighbouring lanes (each holds every DR_R-th row); the two sums over
// rows a token needs (u^T S and S^T r) are a per-thread run plus a butterfly over those lanes: the
// order of every sum depends on d only.  The per-token vectors of a tile of tokens (decays, rates, unit
// keys) are prepared by all threads together before the walk.  Everything is float32.
#include "common.cuh"

#define DR_R 4                   // lanes that share a column of the state

struct DeltaArgs {
    const float* proj;           // [T, ld]: one product's output row, columns at the offsets below
    const float* w2;             // [H*d, L]
    const float* w0;             // [H*d]
    const float* a_bias;         // [H*d]
    const float* norm_w;         // [H*d]
    float* state;                // [slots, H, d, d]
    void* out;                   // [T, H*d]
    const int* seq_slot;
    const int* q_start;
    int ld, off_r, off_k, off_v, off_a, off_g, off_z, H, d, L, tile;
    float eps;
};

__device__ __forceinline__ float dr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename T, int RPT>
__global__ void __launch_bounds__(DR_R * DR_R * RPT) general_delta_kernel(DeltaArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) float dr_smem[];
    int d = a.d, L = a.L, TT = a.tile;
    float* kk = dr_smem;                 // [TT][d] keys
    float* uu = kk + TT * d;             // unit keys
    float* au = uu + TT * d;             // removal rate x unit key (the rate alone until the norm is known)
    float* ww = au + TT * d;             // decays
    float* rr = ww + TT * d;             // receptance
    float* vv = rr + TT * d;             // values
    float* gg = vv + TT * d;             // gate logits
    float* oo = gg + TT * d;             // outputs before the norm
    float* th = oo + TT * d;             // [TT][L] tanh of the narrow projection
    float* red = th + TT * L;            // [TT] a per-token scalar

    int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
    int t_begin = a.q_start[b], t_end = a.q_start[b + 1];
    if (t_end <= t_begin) return;
    int j = tid / DR_R, g = tid % DR_R;          // column of the state, and which rows of it
    bool owner = j < d;
    float* sp = a.state + ((size_t)a.seq_slot[b] * a.H + h) * d * d;
    float S[RPT];
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
        int i = g + DR_R * m;
        S[m] = (owner && i < d) ? sp[(size_t)i * d + j] : 0.f;
    }
    int lane = tid & 31, warp = tid >> 5, nwarp = nthr >> 5;
    const float decay_rate = 0.60653065971263342f;       // exp(-1/2)

    for (int t0 = t_begin; t0 < t_end; t0 += TT) {
        int n = min(TT, t_end - t0);
        for (int e = tid; e < n * L; e += nthr) {
            int tok = e / L, l = e % L;
            th[e] = tanhf(a.proj[(size_t)(t0 + tok) * a.ld + a.off_z + l]);
        }
        __syncthreads();
        for (int e = tid; e < n * d; e += nthr) {
            int tok = e / d, c = e % d, col = h * d + c;
            const float* row = a.proj + (size_t)(t0 + tok) * a.ld;
            float z = a.w0[col];
            const float* w2r = a.w2 + (size_t)col * L;
            const float* tr = th + tok * L;
            for (int l = 0; l < L; ++l) z = fmaf(w2r[l], tr[l], z);
            ww[e] = expf(-decay_rate * dr_sigmoid(z));
            au[e] = dr_sigmoid(row[a.off_a + col] + a.a_bias[col]);
            kk[e] = row[a.off_k + col];
            rr[e] = row[a.off_r + col];
            vv[e] = row[a.off_v + col];
            gg[e] = row[a.off_g + col];
        }
        __syncthreads();
        for (int tok = warp; tok < n; tok += nwarp) {        // sum of squares of each key: a warp per token
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) ss = fmaf(kk[tok * d + c], kk[tok * d + c], ss);
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[tok] = 1.0f / sqrtf(ss + 1e-6f);
        }
        __syncthreads();
        for (int e = tid; e < n * d; e += nthr) {
            float u = kk[e] * red[e / d];
            uu[e] = u;
            au[e] *= u;
        }
        __syncthreads();
        // the walk: no barrier inside, every thread reads the prepared vectors and its own registers
        for (int tok = 0; tok < n; ++tok) {
            const float* u_ = uu + tok * d;
            const float* au_ = au + tok * d;
            const float* w_ = ww + tok * d;
            const float* k_ = kk + tok * d;
            const float* r_ = rr + tok * d;
            float dot = 0.f;
#pragma unroll
            for (int m = 0; m < RPT; ++m) {
                int i = g + DR_R * m;
                if (i < d) dot = fmaf(u_[i], S[m], dot);
            }
#pragma unroll
            for (int o = 1; o < DR_R; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            float vj = owner ? vv[tok * d + j] : 0.f;
            float out = 0.f;
#pragma unroll
            for (int m = 0; m < RPT; ++m) {
                int i = g + DR_R * m;
                if (i < d) {
                    float s = fmaf(k_[i], vj, fmaf(w_[i], S[m], -au_[i] * dot));
                    S[m] = s;
                    out = fmaf(s, r_[i], out);
                }
            }
#pragma unroll
            for (int o = 1; o < DR_R; o <<= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
            if (owner && g == 0) oo[tok * d + j] = out;
        }
        __syncthreads();
        for (int tok = warp; tok < n; tok += nwarp) {        // root mean square of each token's head output
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) ss = fmaf(oo[tok * d + c], oo[tok * d + c], ss);
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) red[tok] = 1.0f / sqrtf(ss / (float)d + a.eps);
        }
        __syncthreads();
        for (int e = tid; e < n * d; e += nthr) {
            int tok = e / d, c = e % d, col = h * d + c;
            float y = oo[e] * red[tok] * a.norm_w[col] * dr_sigmoid(gg[e]);
            CeType<T>::store((T*)a.out + (size_t)(t0 + tok) * a.H * d + col, y);
        }
        __syncthreads();
    }
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
        int i = g + DR_R * m;
        if (owner && i < d) sp[(size_t)i * d + j] = S[m];
    }
}

template <typename T, int RPT>
static void launch_delta(const DeltaArgs& a, int B, size_t smem, cudaStream_t stream) {
    int threads = (a.d * DR_R + 31) / 32 * 32;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(general_delta_kernel<T, RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce_note("general_delta_kernel");
    ce_launch(general_delta_kernel<T, RPT>, dim3(a.H, B), threads, smem, stream, a);
}

template <typename T>
static int dispatch_delta(const DeltaArgs& a, int B, size_t smem, cudaStream_t stream) {
    int rpt = (a.d + DR_R - 1) / DR_R;
    if (rpt <= 8) launch_delta<T, 8>(a, B, smem, stream);
    else if (rpt <= 16) launch_delta<T, 16>(a, B, smem, stream);
    else launch_delta<T, 32>(a, B, smem, stream);
    return ce_check_launch("ce_general_delta");
}

extern "C" int ce_general_delta(const float* proj, const float* w2, const float* w0, const float* a_bias,
                                const float* norm_w, float* state, void* out, int out_dtype, const int* seq_slot,
                                const int* q_start, int B, int ld, int off_r, int off_k, int off_v, int off_a, int off_g,
                                int off_z, int H, int d, int L, float eps, cudaStream_t stream) {
    if (B == 0) return CE_OK;
    if (!proj || !w2 || !w0 || !a_bias || !norm_w || !state || !out || !seq_slot || !q_start)
        return ce_fail(CE_ERR_ARG, "ce_general_delta: null pointer");
    if (d <= 0 || d > 128) return ce_fail(CE_ERR_SIZE, "ce_general_delta: head size %d not in 1..128", d);
    if (H <= 0 || L <= 0 || B > 65535) return ce_fail(CE_ERR_SIZE, "ce_general_delta: %d heads, rank %d, %d sequences", H, L, B);
    int tile = d <= 64 ? 16 : d <= 128 ? 8 : 4;
    DeltaArgs a{proj, w2, w0, a_bias, norm_w, state, out, seq_slot, q_start, ld, off_r, off_k, off_v, off_a, off_g, off_z,
                H, d, L, tile, eps};
    size_t smem = (size_t)(8 * tile * d + tile * L + tile) * sizeof(float);
    if (smem > 200 * 1024) return ce_fail(CE_ERR_SIZE, "ce_general_delta: rank %d is too large", L);
    if (out_dtype == CE_F32) return dispatch_delta<float>(a, B, smem, stream);
    if (out_dtype == CE_BF16) return dispatch_delta<__nv_bfloat16>(a, B, smem, stream);
    return ce_fail(CE_ERR_ARG, "ce_general_delta: unknown dtype %d", out_dtype);
}
