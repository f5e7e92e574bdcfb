// The generalized delta rule: a recurrent mixer whose per-head state S [d, d] (key channel x value
// channel, float32) is carried from token to token:
//
//     S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T        o_t = S_t^T r_t
//
// with the decay w_t = exp(-exp(-1/2) sigmoid(z_t + w0)) per key channel (z_t: the token's decay logits, a
// product of their own), the removal rate a_t = sigmoid(a_raw + bias), and the unit key
// u_t = k_t / sqrt(sum k_t^2 + 1e-6).  Both the decay and the removal read the OLD state.  Afterwards
// every head's o_t is divided by its root mean square, multiplied by a weight and by sigmoid(gate).
//
// Three kernels, all float32:
//   prepare  every token on its own: w_t, u_t and a_t * u_t of every head               (parallel over tokens)
//   walk     one block per (head, sequence, slice of value channels) walks the sequence's tokens of this
//            step in order, from the state its slot holds, and stores the state back        (the recurrence)
//   finish   every (token, head): root mean square, weight, gate, one rounding at the store   (parallel)
//
// The columns of S (value channels) are independent of one another, so a slice of DR_COLS columns is a block
// of its own and a column lives in the registers of DR_R neighbouring lanes (each holds a run of RPT
// consecutive rows, read from shared memory four at a time); the two sums over rows a token needs (u^T S and S^T r) are a per-thread run plus a butterfly over
// those lanes: the order of every sum depends on d only, never on how the tokens were cut into steps.  The
// per-token vectors arrive in shared memory a tile of tokens ahead of the walk (cp.async, two buffers).
// A warp issues in order, and a token's step is a chain of dependent instructions, so what counts is how few
// instructions a warp spends per token: sixteen lanes a column leave each thread four to sixteen rows.
#include "common.cuh"

// Measured at 2,048 tokens of one sequence with 32 and with 64 heads of 64: 16 lanes a column in blocks of 8 columns
// took 0.50 and 0.69 ms, 32 lanes 0.51 and 0.94, 8 lanes (64 heads) 0.97, 4 lanes (32 heads) 1.24.  Fewer lanes leave a
// thread more rows, that is more instructions per token in a warp that issues them in order; more lanes add
// exchanges and warps.  The numbers are fixed, never chosen from the batch, so a request's sums do not depend on
// its neighbours.
#define DR_R 16                  // lanes that share a column of the state (the walk's exchanges are written for 16)
#define DR_COLS 8                // value channels a block walks
#define DR_TILE 16               // tokens a buffer holds (at most DR_R: lane g of a column stores token g's output)

__device__ __forceinline__ float dr_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// out[t, l] = tanh(proj[t, off + l]) in the activation dtype: the input of the decay's second product
template <typename T>
__global__ void tanh_cols_kernel(const float* __restrict__ proj, T* __restrict__ out, int ld, int off, int L, size_t total) {
    ce_pdl_begin();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t t = e / L;
        int l = (int)(e % L);
        CeType<T>::store(out + e, tanhf(proj[t * ld + off + l]));
    }
}

extern "C" int ce_tanh_cols(const float* proj, void* out, int out_dtype, int T, int ld, int off, int L, cudaStream_t stream) {
    if (T == 0 || L == 0) return CE_OK;
    if (!proj || !out) return ce_fail(CE_ERR_ARG, "ce_tanh_cols: null pointer");
    size_t total = (size_t)T * L;
    int blocks = (int)((total + 255) / 256 < (size_t)148 * 8 ? (total + 255) / 256 : (size_t)148 * 8);
    if (out_dtype == CE_F32) { ce_note("tanh_cols_kernel"); ce_launch(tanh_cols_kernel<float>, blocks, 256, 0, stream, proj, (float*)out, ld, off, L, total); }
    else if (out_dtype == CE_BF16) { ce_note("tanh_cols_kernel"); ce_launch(tanh_cols_kernel<__nv_bfloat16>, blocks, 256, 0, stream, proj, (__nv_bfloat16*)out, ld, off, L, total); }
    else return ce_fail(CE_ERR_ARG, "ce_tanh_cols: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_tanh_cols");
}

struct DeltaArgs {
    const float* proj;           // [T, ld]: r, k, v, a, g at the column offsets below
    const float* zz;             // [T, H*d] decay logits before w0
    const float* w0;             // [H*d]
    const float* a_bias;         // [H*d]
    const float* norm_w;         // [H*d]
    float* prep;                 // [T, 3, H*d]: decay, unit key, rate x unit key
    float* raw;                  // [T, H*d] o_t before the norm
    float* state;                // [slots, H, d, d]
    void* out;                   // [T, H*d]
    const int* seq_slot;
    const int* q_start;
    int ld, off_r, off_k, off_v, off_a, off_g, H, d;
    float eps;
};

// One block per token, a warp per head in turn.
__global__ void delta_prepare_kernel(DeltaArgs a) {
    ce_pdl_begin();
    int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int d = a.d, n = a.H * d;
    const float* row = a.proj + (size_t)t * a.ld;
    const float* zr = a.zz + (size_t)t * n;
    float* pw = a.prep + (size_t)t * 3 * n;
    const float decay_rate = 0.60653065971263342f;       // exp(-1/2)
    for (int h = warp; h < a.H; h += nwarp) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) {
            float k = row[a.off_k + h * d + c];
            ss = fmaf(k, k, ss);
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float inv = 1.0f / sqrtf(ss + 1e-6f);
        for (int c = lane; c < d; c += 32) {
            int col = h * d + c;
            float u = row[a.off_k + col] * inv;
            pw[col] = expf(-decay_rate * dr_sigmoid(zr[col] + a.w0[col]));
            pw[n + col] = u;
            pw[2 * n + col] = dr_sigmoid(row[a.off_a + col] + a.a_bias[col]) * u;
        }
    }
}

__device__ __forceinline__ void dr_cp4(float* dst, const float* src) {
    unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(src));
}
__device__ __forceinline__ void dr_cp16(float* dst, const float* src) {
    unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(src));
}

// Copies of one tile of tokens into a buffer: five vectors of d per token (rows padded to DP floats) and DR_COLS values.
template <int DP, bool VEC>
__device__ __forceinline__ void dr_stage(const DeltaArgs& a, float* buf, int t0, int n_tok, int h, int col0, int ncols) {
    int d = a.d, n = a.H * d, tid = threadIdx.x, nthr = blockDim.x;
    float* vbuf = buf + 5 * DR_TILE * DP;
    if (VEC) {
        constexpr int DP4 = DP / 4;
        for (int e = tid; e < 5 * DR_TILE * DP4; e += nthr) {
            int which = e / (DR_TILE * DP4), tok = (e / DP4) % DR_TILE, c = (e % DP4) * 4;
            if (tok < n_tok && c < d) {
                size_t t = (size_t)(t0 + tok);
                const float* src = which < 3 ? a.prep + (t * 3 + which) * n + h * d + c
                                             : a.proj + t * a.ld + (which == 3 ? a.off_k : a.off_r) + h * d + c;
                dr_cp16(buf + (which * DR_TILE + tok) * DP + c, src);
            }
        }
    } else {
        for (int e = tid; e < 5 * DR_TILE * DP; e += nthr) {
            int which = e / (DR_TILE * DP), tok = (e / DP) % DR_TILE, c = e % DP;
            if (tok < n_tok && c < d) {
                size_t t = (size_t)(t0 + tok);
                const float* src = which < 3 ? a.prep + (t * 3 + which) * n + h * d + c
                                             : a.proj + t * a.ld + (which == 3 ? a.off_k : a.off_r) + h * d + c;
                dr_cp4(buf + (which * DR_TILE + tok) * DP + c, src);
            }
        }
    }
    for (int e = tid; e < DR_TILE * DR_COLS; e += nthr) {
        int tok = e / DR_COLS, c = e % DR_COLS;
        if (tok < n_tok && c < ncols)
            dr_cp4(vbuf + tok * DR_COLS + c, a.proj + (size_t)(t0 + tok) * a.ld + a.off_v + h * d + col0 + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int RPT, bool VEC>
__global__ void __launch_bounds__(DR_R * DR_COLS) delta_walk_kernel(DeltaArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) float dr_smem[];
    int d = a.d, n = a.H * d;
    int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * DR_COLS, tid = threadIdx.x;
    int t_begin = a.q_start[b], t_end = a.q_start[b + 1];
    if (t_end <= t_begin) return;
    int ncols = min(DR_COLS, d - col0);
    int jj = tid / DR_R, g = tid % DR_R, j = col0 + jj;
    int i0 = g * RPT;                         // this thread's rows: i0 .. i0 + RPT - 1 (RPT is a multiple of 4)
    bool owner = jj < ncols;
    float* sp = a.state + ((size_t)a.seq_slot[b] * a.H + h) * d * d;
    float S[RPT];
#pragma unroll
    for (int m = 0; m < RPT; ++m) S[m] = (owner && i0 + m < d) ? sp[(size_t)(i0 + m) * d + j] : 0.f;
    // a row of the staged vectors is padded to DR_R * RPT floats, so that every thread reads whole float4
    constexpr int dp = DR_R * RPT;
    int buf_floats = 5 * DR_TILE * dp + DR_TILE * DR_COLS;
    for (int e = tid; e < 2 * buf_floats; e += blockDim.x) dr_smem[e] = 0.f;       // the padding stays zero
    __syncthreads();
    int n_tiles = (t_end - t_begin + DR_TILE - 1) / DR_TILE;
    dr_stage<dp, VEC>(a, dr_smem, t_begin, min(DR_TILE, t_end - t_begin), h, col0, ncols);
    for (int tile = 0; tile < n_tiles; ++tile) {
        int t0 = t_begin + tile * DR_TILE, n_tok = min(DR_TILE, t_end - t0);
        float* buf = dr_smem + (tile & 1) * buf_floats;
        if (tile + 1 < n_tiles) {
            dr_stage<dp, VEC>(a, dr_smem + ((tile + 1) & 1) * buf_floats, t0 + DR_TILE, min(DR_TILE, t_end - t0 - DR_TILE), h, col0, ncols);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* vbuf = buf + 5 * DR_TILE * dp;
        // The sum over rows of S^T r is not needed by the next token: every thread keeps its part for each token of
        // the tile, and the butterflies of all tokens run together after the walk (their latencies overlap).
        float part[DR_TILE];
#pragma unroll
        for (int tok = 0; tok < DR_TILE; ++tok) {
            part[tok] = 0.f;
            if (tok < n_tok) {
                const float4* w_ = reinterpret_cast<const float4*>(buf + (0 * DR_TILE + tok) * dp + i0);
                const float4* u_ = reinterpret_cast<const float4*>(buf + (1 * DR_TILE + tok) * dp + i0);
                const float4* au_ = reinterpret_cast<const float4*>(buf + (2 * DR_TILE + tok) * dp + i0);
                const float4* k_ = reinterpret_cast<const float4*>(buf + (3 * DR_TILE + tok) * dp + i0);
                const float4* r_ = reinterpret_cast<const float4*>(buf + (4 * DR_TILE + tok) * dp + i0);
                // u^T S over this thread's rows in four runs (a fixed order), then over the column's lanes
                float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
                for (int m = 0; m < RPT / 4; ++m) {
                    float4 u = u_[m];
                    p0 = fmaf(u.x, S[4 * m], p0); p1 = fmaf(u.y, S[4 * m + 1], p1);
                    p2 = fmaf(u.z, S[4 * m + 2], p2); p3 = fmaf(u.w, S[4 * m + 3], p3);
                }
                float dot = (p0 + p1) + (p2 + p3);
                // over the column's sixteen lanes in two rounds of four: the three exchanges of a round are in flight
                // together, and every lane adds the same pairs, so all sixteen hold the same sum
                {
                    float e1 = __shfl_xor_sync(0xffffffffu, dot, 1), e2 = __shfl_xor_sync(0xffffffffu, dot, 2),
                          e3 = __shfl_xor_sync(0xffffffffu, dot, 3);
                    dot = (dot + e1) + (e2 + e3);
                    float f1 = __shfl_xor_sync(0xffffffffu, dot, 4), f2 = __shfl_xor_sync(0xffffffffu, dot, 8),
                          f3 = __shfl_xor_sync(0xffffffffu, dot, 12);
                    dot = (dot + f1) + (f2 + f3);
                }
                float vj = owner ? vbuf[tok * DR_COLS + jj] : 0.f;
                float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
#pragma unroll
                for (int m = 0; m < RPT / 4; ++m) {
                    float4 w = w_[m], au = au_[m], k = k_[m], r = r_[m];
                    float s0 = fmaf(k.x, vj, fmaf(w.x, S[4 * m], -au.x * dot));
                    float s1 = fmaf(k.y, vj, fmaf(w.y, S[4 * m + 1], -au.y * dot));
                    float s2 = fmaf(k.z, vj, fmaf(w.z, S[4 * m + 2], -au.z * dot));
                    float s3 = fmaf(k.w, vj, fmaf(w.w, S[4 * m + 3], -au.w * dot));
                    S[4 * m] = s0; S[4 * m + 1] = s1; S[4 * m + 2] = s2; S[4 * m + 3] = s3;
                    q0 = fmaf(s0, r.x, q0); q1 = fmaf(s1, r.y, q1); q2 = fmaf(s2, r.z, q2); q3 = fmaf(s3, r.w, q3);
                }
                part[tok] = (q0 + q1) + (q2 + q3);
            }
        }
#pragma unroll
        for (int o = 1; o < DR_R; o <<= 1)
#pragma unroll
            for (int tok = 0; tok < DR_TILE; ++tok) part[tok] += __shfl_xor_sync(0xffffffffu, part[tok], o);
        // lane g of a column stores token g of the tile (DR_TILE <= DR_R)
        float mine = part[0];
#pragma unroll
        for (int tok = 1; tok < DR_TILE; ++tok) mine = g == tok ? part[tok] : mine;
        if (owner && g < n_tok) a.raw[(size_t)(t0 + g) * n + h * d + j] = mine;
        __syncthreads();             // the buffer is free for the tile after the next
    }
#pragma unroll
    for (int m = 0; m < RPT; ++m)
        if (owner && i0 + m < d) sp[(size_t)(i0 + m) * d + j] = S[m];
}

// One block per token, a warp per head in turn: root mean square over the head, weight, gate.
template <typename T>
__global__ void delta_finish_kernel(DeltaArgs a) {
    ce_pdl_begin();
    int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    int d = a.d, n = a.H * d;
    const float* o = a.raw + (size_t)t * n;
    const float* row = a.proj + (size_t)t * a.ld;
    for (int h = warp; h < a.H; h += nwarp) {
        float ss = 0.f;
        for (int c = lane; c < d; c += 32) ss = fmaf(o[h * d + c], o[h * d + c], ss);
        for (int k = 16; k > 0; k >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, k);
        float inv = 1.0f / sqrtf(ss / (float)d + a.eps);
        for (int c = lane; c < d; c += 32) {
            int col = h * d + c;
            CeType<T>::store((T*)a.out + (size_t)t * n + col, o[col] * inv * a.norm_w[col] * dr_sigmoid(row[a.off_g + col]));
        }
    }
}

template <int RPT>
static void launch_walk(const DeltaArgs& a, int B, bool vec, cudaStream_t stream) {
    size_t smem = (size_t)2 * (5 * DR_TILE * DR_R * RPT + DR_TILE * DR_COLS) * sizeof(float);
    dim3 grid(a.H, B, (a.d + DR_COLS - 1) / DR_COLS);
    ce_note("delta_walk_kernel");
    if (vec) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_walk_kernel<RPT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ce_launch(delta_walk_kernel<RPT, true>, grid, DR_R * DR_COLS, smem, stream, a);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_walk_kernel<RPT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ce_launch(delta_walk_kernel<RPT, false>, grid, DR_R * DR_COLS, smem, stream, a);
    }
}

// proj [T, ld] float32 with r, k, v, a, g at their offsets; zz [T, H*d] the decay logits; prep [T, 3*H*d] and raw
// [T, H*d] float32 work space; state [slots, H, d, d]; out [T, H*d] in out_dtype.
extern "C" int ce_general_delta(const float* proj, const float* zz, const float* w0, const float* a_bias, const float* norm_w,
                                float* prep, float* raw, float* state, void* out, int out_dtype, const int* seq_slot,
                                const int* q_start, int T, int B, int ld, int off_r, int off_k, int off_v, int off_a, int off_g,
                                int H, int d, float eps, int stage, cudaStream_t stream) {
    // stage: 1 prepare, 2 walk, 3 finish (each one launch, so that each is counted and timed by itself)
    if (B == 0 || T == 0) return CE_OK;
    if (stage < 1 || stage > 3) return ce_fail(CE_ERR_ARG, "ce_general_delta: stage %d", stage);
    if (!proj || !zz || !w0 || !a_bias || !norm_w || !prep || !raw || !state || !out || !seq_slot || !q_start)
        return ce_fail(CE_ERR_ARG, "ce_general_delta: null pointer");
    if (d <= 0 || d > 256) return ce_fail(CE_ERR_SIZE, "ce_general_delta: head size %d not in 1..256", d);
    if (H <= 0 || B > 65535) return ce_fail(CE_ERR_SIZE, "ce_general_delta: %d heads, %d sequences", H, B);
    if (out_dtype != CE_F32 && out_dtype != CE_BF16) return ce_fail(CE_ERR_ARG, "ce_general_delta: unknown dtype %d", out_dtype);
    DeltaArgs a{proj, zz, w0, a_bias, norm_w, prep, raw, state, out, seq_slot, q_start, ld, off_r, off_k, off_v, off_a, off_g, H, d, eps};
    int threads = H >= 8 ? 256 : 32 * H;
    if (stage == 1) {
        ce_note("delta_prepare_kernel");
        ce_launch(delta_prepare_kernel, T, threads, 0, stream, a);
        return ce_check_launch("ce_general_delta");
    }
    if (stage == 3) {
        ce_note("delta_finish_kernel");
        if (out_dtype == CE_F32) ce_launch(delta_finish_kernel<float>, T, threads, 0, stream, a);
        else ce_launch(delta_finish_kernel<__nv_bfloat16>, T, threads, 0, stream, a);
        return ce_check_launch("ce_general_delta");
    }
    // 16-byte copies where every source address is a multiple of 16: all of the row stride, the offsets and d
    bool vec = d % 4 == 0 && ld % 4 == 0 && off_k % 4 == 0 && off_r % 4 == 0 &&
               (((uintptr_t)proj | (uintptr_t)prep) & 15) == 0;
    int rpt = (d + DR_R - 1) / DR_R;
    if (rpt <= 4) launch_walk<4>(a, B, vec, stream);
    else if (rpt <= 8) launch_walk<8>(a, B, vec, stream);
    else launch_walk<16>(a, B, vec, stream);
    return ce_check_launch("ce_general_delta");
}
