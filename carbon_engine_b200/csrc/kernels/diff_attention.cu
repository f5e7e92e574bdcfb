// Differential attention over the paged cache, in float32 arithmetic, for any number of new tokens
// per sequence, and the kernel that prepares its operands.
//
// Every query head carries two maps (two query vectors of size d); every key/value head carries two
// key vectors of size d and ONE value vector of size dv.  Each map is a softmax attention of its own
// over the same values: a1 and a2.  The head's output is
//     o = a1 - lambda * a2,   o <- o / sqrt(mean(o^2) + eps) * out_scale,   o <- o * sigmoid(gate)
// with one lambda for the layer and one gate logit per (token, head).
//
// In the cache the two maps of a key head are two "heads" of the K pool: K pool [pages, 2 G, page, d],
// V pool [pages, G, page, dv].  Which keys a query sees: causal, optionally the last ``window`` keys,
// optionally only the keys of its own block of ``chunk`` positions (blocks counted from position 0).
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// Operands: one product's output row [q heads | k heads | v heads | ...] gets its bias added, q and k
// rotated over their first ``rd`` elements (pairs (i, i + rd/2)), q written back in place, k and v
// stored at the token's place in the pools.  q and k heads have size d, v heads size dv.
// ---------------------------------------------------------------------------------------------
struct PrepArgs {
    void* qkv;
    void* k_pool;            // [num_pages, nk, page_size, d]
    void* v_pool;            // [num_pages, nv, page_size, dv]
    const float* bias;       // [(nq + nk) * d + nv * dv] or null
    const float* cos_table;  // [max_pos, rd/2] or null: no rotation
    const float* sin_table;
    const int* positions;
    const int* seq_of_token;
    const int* seq_slot;
    const int* block_table;
    int* status;
    int T, stride, nq, nk, nv, d, dv, rd, page_size, max_pages, num_pages, max_pos, write_kv;
};

template <typename T>
__global__ void bias_rope_kvwrite_kernel(PrepArgs a) {
    ce_pdl_begin();
    int t = blockIdx.x;
    int p = a.positions[t];
    T* row = (T*)a.qkv + (size_t)t * a.stride;
    int d = a.d, half = a.rd / 2;
    bool rotate = a.cos_table != nullptr && half > 0;
    if (rotate && (p < 0 || p >= a.max_pos)) {
        if (threadIdx.x == 0) atomicExch(a.status, 3);
        rotate = false;
    }
    long long kbase = -1;       // element offset of (page, head 0, offset, 0) in a pool with head size 1
    int page = -1, off = 0;
    if (a.write_kv) {
        int slot = a.seq_slot[a.seq_of_token[t]];
        page = a.block_table[(size_t)slot * a.max_pages + p / a.page_size];
        off = p % a.page_size;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.status, 2);
            page = -1;
        }
    }
    (void)kbase;
    const float* cs = rotate ? a.cos_table + (size_t)p * half : nullptr;
    const float* sn = rotate ? a.sin_table + (size_t)p * half : nullptr;
    // q and k heads: one thread per (head, element below d - half): it owns element i and, inside the rotated
    // part, its partner i + half
    int nqk = a.nq + a.nk;
    int per_head = d - (rotate ? half : 0);
    for (int e = threadIdx.x; e < nqk * per_head; e += blockDim.x) {
        int h = e / per_head, i = e % per_head;
        int col = h * d;
        T* hp = row + col;
        const float* bp = a.bias ? a.bias + col : nullptr;
        T* kdst = nullptr;
        if (h >= a.nq && a.write_kv && page >= 0)
            kdst = (T*)a.k_pool + (((size_t)page * a.nk + (h - a.nq)) * a.page_size + off) * d;
        if (rotate && i < half) {
            float u = CeType<T>::load(hp + i) + (bp ? bp[i] : 0.f);
            float v = CeType<T>::load(hp + i + half) + (bp ? bp[i + half] : 0.f);
            float c = cs[i], s = sn[i];
            float ru = u * c - v * s, rv = v * c + u * s;
            if (h < a.nq) { CeType<T>::store(hp + i, ru); CeType<T>::store(hp + i + half, rv); }
            else if (kdst) { CeType<T>::store(kdst + i, ru); CeType<T>::store(kdst + i + half, rv); }
        } else {
            int j = rotate ? i + half : i;          // elements past the rotated part
            float u = CeType<T>::load(hp + j) + (bp ? bp[j] : 0.f);
            if (h < a.nq) CeType<T>::store(hp + j, u);
            else if (kdst) CeType<T>::store(kdst + j, u);
        }
    }
    if (a.write_kv && page >= 0) {
        int vcol = nqk * d;
        for (int e = threadIdx.x; e < a.nv * a.dv; e += blockDim.x) {
            int h = e / a.dv, j = e % a.dv;
            float u = CeType<T>::load(row + vcol + e) + (a.bias ? a.bias[vcol + e] : 0.f);
            CeType<T>::store((T*)a.v_pool + (((size_t)page * a.nv + h) * a.page_size + off) * a.dv + j, u);
        }
    }
}

extern "C" int ce_bias_rope_kvwrite(void* qkv, void* k_pool, void* v_pool, int dtype, const float* bias,
                                    const float* cos_table, const float* sin_table, const int* positions,
                                    const int* seq_of_token, const int* seq_slot, const int* block_table, int* status,
                                    int T, int stride, int nq, int nk, int nv, int d, int dv, int rd, int page_size,
                                    int max_pages, int num_pages, int max_pos, int write_kv, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!qkv || !positions || !seq_of_token || !seq_slot || !status) return ce_fail(CE_ERR_ARG, "ce_bias_rope_kvwrite: null pointer");
    if (write_kv && (!k_pool || !v_pool || !block_table)) return ce_fail(CE_ERR_ARG, "ce_bias_rope_kvwrite: no cache to write to");
    if (rd < 0 || rd > d || rd % 2) return ce_fail(CE_ERR_SIZE, "ce_bias_rope_kvwrite: %d rotated elements of %d", rd, d);
    if (stride < (nq + nk) * d + nv * dv) return ce_fail(CE_ERR_SIZE, "ce_bias_rope_kvwrite: row stride %d is too small", stride);
    PrepArgs a{qkv, k_pool, v_pool, bias, rd > 0 ? cos_table : nullptr, sin_table, positions, seq_of_token, seq_slot,
               block_table, status, T, stride, nq, nk, nv, d, dv, rd, page_size, max_pages, num_pages, max_pos, write_kv};
    int work = (nq + nk) * d;
    int threads = work >= 2048 ? 512 : work >= 512 ? 256 : 128;
    if (dtype == CE_F32) { ce_note("bias_rope_kvwrite_kernel"); ce_launch(bias_rope_kvwrite_kernel<float>, T, threads, 0, stream, a); }
    else if (dtype == CE_BF16) { ce_note("bias_rope_kvwrite_kernel"); ce_launch(bias_rope_kvwrite_kernel<__nv_bfloat16>, T, threads, 0, stream, a); }
    else return ce_fail(CE_ERR_ARG, "ce_bias_rope_kvwrite: unknown dtype %d", dtype);
    return ce_check_launch("ce_bias_rope_kvwrite");
}

// ---------------------------------------------------------------------------------------------
// The attention itself.  One block per (token, query head).  Keys are taken in runs of 128 positions
// that start at multiples of 128, with an online softmax per map across the runs, so the order of every
// sum depends on the query's position only: not on how the tokens were cut into steps, not on the batch,
// not on the pages.
// ---------------------------------------------------------------------------------------------
#define DA_THREADS 128
#define DA_MAX_ACC 8             // dv <= DA_THREADS * DA_MAX_ACC

struct DiffArgs {
    const void* q;               // [T, q_stride]; head h: map 1 at column h*2*d, map 2 at h*2*d + d
    const void* k_pool;
    const void* v_pool;
    const void* gate;            // [T, gate_stride] gate logits, head h at column h; null: no gate
    void* out;                   // [T, nh*dv]
    const int* positions;
    const int* seq_of_token;
    const int* seq_slot;
    const int* block_table;
    int* status;
    int T, nh, nkv, d, dv, q_stride, gate_stride, page_size, max_pages, num_pages, window, chunk;
    float scale, lambda, eps, out_scale;
};

template <typename T>
__global__ void diff_attention_kernel(DiffArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char da_smem[];
    long long* vrow = (long long*)da_smem;             // DA_THREADS
    float* p1 = (float*)(vrow + DA_THREADS);           // DA_THREADS
    float* p2 = p1 + DA_THREADS;                       // DA_THREADS
    float* scratch = p2 + DA_THREADS;                  // 32
    float* qs = scratch + 32;                          // 2 d

    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, d = a.d, dv = a.dv;
    int kvh = h / (a.nh / a.nkv);
    int p = a.positions[t];
    int slot = a.seq_slot[a.seq_of_token[t]];
    const int* table = a.block_table + (size_t)slot * a.max_pages;
    const T* qrow = (const T*)a.q + (size_t)t * a.q_stride + (size_t)h * 2 * d;
    for (int j = tid; j < 2 * d; j += DA_THREADS) qs[j] = CeType<T>::load(qrow + j);
    __syncthreads();

    int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    if (a.chunk > 0) lo = max(lo, p / a.chunk * a.chunk);
    float m1 = -INFINITY, l1 = 0.f, m2 = -INFINITY, l2 = 0.f;
    float acc1[DA_MAX_ACC], acc2[DA_MAX_ACC];
#pragma unroll
    for (int i = 0; i < DA_MAX_ACC; ++i) acc1[i] = acc2[i] = 0.f;

    for (int k0 = lo / DA_THREADS * DA_THREADS; k0 <= p; k0 += DA_THREADS) {
        int key = k0 + tid;
        bool valid = key >= lo && key <= p;
        float s1 = -INFINITY, s2 = -INFINITY;
        long long vr = -1;
        if (valid) {
            int page = table[key / a.page_size];
            if (page < 0 || page >= a.num_pages) {
                atomicExch(a.status, 4);
                valid = false;
            } else {
                int off = key % a.page_size;
                const T* k1 = (const T*)a.k_pool + (((size_t)page * 2 * a.nkv + 2 * kvh) * a.page_size + off) * d;
                const T* k2 = k1 + (size_t)a.page_size * d;
                float d1 = 0.f, d2 = 0.f;
                for (int j = 0; j < d; ++j) {
                    d1 = fmaf(qs[j], CeType<T>::load(k1 + j), d1);
                    d2 = fmaf(qs[d + j], CeType<T>::load(k2 + j), d2);
                }
                s1 = d1 * a.scale;
                s2 = d2 * a.scale;
                vr = (((long long)page * a.nkv + kvh) * a.page_size + off) * dv;
            }
        }
        float n1 = fmaxf(m1, ce_block_max(s1, scratch));
        __syncthreads();
        float n2 = fmaxf(m2, ce_block_max(s2, scratch));
        float e1 = valid ? expf(s1 - n1) : 0.f, e2 = valid ? expf(s2 - n2) : 0.f;
        __syncthreads();                 // everyone has read scratch before it is reused
        p1[tid] = e1;
        p2[tid] = e2;
        vrow[tid] = vr;
        float c1 = ce_block_sum(e1, scratch);
        __syncthreads();
        float c2 = ce_block_sum(e2, scratch);   // syncs: p1, p2 and vrow are visible afterwards
        float f1 = m1 == -INFINITY ? 0.f : expf(m1 - n1), f2 = m2 == -INFINITY ? 0.f : expf(m2 - n2);
        l1 = l1 * f1 + c1;
        l2 = l2 * f2 + c2;
        m1 = n1;
        m2 = n2;
        int n = min(DA_THREADS, p - k0 + 1);
#pragma unroll
        for (int i = 0; i < DA_MAX_ACC; ++i) {
            int j = tid + i * DA_THREADS;
            if (j < dv) {
                float o1 = acc1[i] * f1, o2 = acc2[i] * f2;
                for (int kk = 0; kk < n; ++kk) {
                    long long r = vrow[kk];
                    if (r >= 0) {
                        float v = CeType<T>::load((const T*)a.v_pool + r + j);
                        o1 = fmaf(p1[kk], v, o1);
                        o2 = fmaf(p2[kk], v, o2);
                    }
                }
                acc1[i] = o1;
                acc2[i] = o2;
            }
        }
        __syncthreads();
    }
    float i1 = l1 > 0.f ? 1.0f / l1 : 0.f, i2 = l2 > 0.f ? 1.0f / l2 : 0.f;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < DA_MAX_ACC; ++i) {
        int j = tid + i * DA_THREADS;
        float o = j < dv ? acc1[i] * i1 - a.lambda * (acc2[i] * i2) : 0.f;
        acc1[i] = o;
        ss = fmaf(o, o, ss);
    }
    __syncthreads();
    ss = ce_block_sum(ss, scratch);
    float g = 1.0f;
    if (a.gate) {
        float z = CeType<T>::load((const T*)a.gate + (size_t)t * a.gate_stride + h);
        g = 1.0f / (1.0f + expf(-z));
    }
    float mul = a.out_scale * g / sqrtf(ss / (float)dv + a.eps);
    T* orow = (T*)a.out + ((size_t)t * a.nh + h) * dv;
#pragma unroll
    for (int i = 0; i < DA_MAX_ACC; ++i) {
        int j = tid + i * DA_THREADS;
        if (j < dv) CeType<T>::store(orow + j, acc1[i] * mul);
    }
}

extern "C" int ce_diff_attention(const void* q, const void* k_pool, const void* v_pool, const void* gate, void* out,
                                 int dtype, const int* positions, const int* seq_of_token, const int* seq_slot,
                                 const int* block_table, int* status, int T, int nh, int nkv, int d, int dv,
                                 int q_stride, int gate_stride, int page_size, int max_pages, int num_pages, int window,
                                 int chunk, float scale, float lambda, float eps, float out_scale, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !seq_of_token || !seq_slot || !block_table || !status)
        return ce_fail(CE_ERR_ARG, "ce_diff_attention: null pointer");
    if (d <= 0 || dv <= 0 || dv > DA_THREADS * DA_MAX_ACC || d > 4096)
        return ce_fail(CE_ERR_SIZE, "ce_diff_attention: head sizes %d / %d", d, dv);
    if (nkv <= 0 || nh % nkv != 0)
        return ce_fail(CE_ERR_SIZE, "ce_diff_attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    DiffArgs a{q, k_pool, v_pool, gate, out, positions, seq_of_token, seq_slot, block_table, status, T, nh, nkv, d, dv,
               q_stride, gate_stride, page_size, max_pages, num_pages, window, chunk, scale, lambda, eps, out_scale};
    size_t smem = (size_t)(2 * d + 2 * DA_THREADS + 32) * sizeof(float) + DA_THREADS * sizeof(long long);
    dim3 grid(T, nh);
    if (dtype == CE_F32) { ce_note("diff_attention_kernel"); ce_launch(diff_attention_kernel<float>, grid, DA_THREADS, smem, stream, a); }
    else if (dtype == CE_BF16) { ce_note("diff_attention_kernel"); ce_launch(diff_attention_kernel<__nv_bfloat16>, grid, DA_THREADS, smem, stream, a); }
    else return ce_fail(CE_ERR_ARG, "ce_diff_attention: unknown dtype %d", dtype);
    return ce_check_launch("ce_diff_attention");
}
