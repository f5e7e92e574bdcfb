// Differential attention for portions of prompts in bfloat16 on the tensor cores (mma.sync m16n8k16),
// over the paged cache.  The float32 kernel of diff_attention.cu is its plain twin.
//
// One block per (tile of 64 query tokens of one sequence, query head), eight warps: warps 0..3 compute
// map 1 for 16 query rows each, warps 4..7 map 2 for the same rows.  Each warp is a flash attention of its
// own (S = Q K^T in float32, online softmax, P rounded to bfloat16, O += P V in float32) over tiles of 64
// keys; both maps read the same V tile and their own K tile.  At the end the warps of map 2 hand their
// normalised rows over through shared memory and the warps of map 1 finish the head:
// o = a1 - lambda a2, unit root mean square over the head times out_scale, times sigmoid(gate), one store.
//
// K and V tiles come from the pages by cp.async into two buffers, a tile ahead of the arithmetic; the page of
// every key row of a tile is looked up two tiles ahead, so that no copy waits for a table entry.
//
// One-token sequences of a decode step are tiles of one row: a query sees at most a mask block of keys, so there is
// nothing to split among blocks.  Such a tile is work for one warp a map, and that warp's instructions, one after
// another, are what the block's time is made of (about 1,700 a tile of 64 keys, 4.5 us).  So where the launch has no
// more blocks than the GPU has SMs, the kernel gets four K/V buffers and the four warps of a map take four tiles of
// keys side by side, each with a running maximum and sum of its own; their partial rows are merged through shared
// memory in the order of the warps (batch 8, 16 heads, mask blocks of 1,024 nearly full: 0.56 -> 0.50 ms a step).
// Measured and dropped: four buffers in flight with one warp still walking all tiles (no effect), and the warps taking
// every fourth tile with the block still meeting at a barrier after each tile (no effect: the tiles stayed in a row).
//
// Visible keys per row: causal, optionally the last ``window``, optionally only the row's own block of
// ``chunk`` positions; a tile of queries may straddle blocks, so the mask is applied per element.
#include "common.cuh"

#define FA_BM 64
#define FA_BN 64
#define FA_SUB 32                // keys of a tile whose scores a warp holds at a time
#define FA_THREADS 256
#define FA_PAD 8                 // bf16 elements of padding per shared-memory row (16 bytes: conflict-free ldmatrix)

struct FlashDiffArgs {
    const __nv_bfloat16* q;      // [T, q_stride]; head h: map 1 at column h*2*d, map 2 at h*2*d + d
    const __nv_bfloat16* k_pool; // [pages, 2 nkv, page, d]
    const __nv_bfloat16* v_pool; // [pages, nkv, page, dv]
    const __nv_bfloat16* gate;   // [T, gate_stride] or null
    __nv_bfloat16* out;          // [T, nh*dv]
    const int* positions;
    const int* seq_slot;
    const int* q_start;
    const int* block_table;
    const int* tiles;            // (sequence, first token of the tile within the sequence's tokens of the step)
    int* status;
    int nh, nkv, d, dv, q_stride, gate_stride, page_size, max_pages, num_pages, window, chunk;
    int share;                   // 1: four K/V buffers are there, and tiles of at most 16 rows spread their key tiles over a map's warps
    float scale, lambda, eps, out_scale;
};

__device__ __forceinline__ void fa_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void fa_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void fa_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned fa_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// DK: 16-element steps of a map the registers hold (d <= 16 DK); DVT: 8-column tiles of a value head (dv <= 8 DVT)
template <int DK, int DVT>
__global__ void __launch_bounds__(FA_THREADS, (DVT <= 16 ? 2 : 1)) diff_attention_mma_kernel(FlashDiffArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char fa_smem[];
    const int d = a.d, dv = a.dv, ldk = d + FA_PAD, ldv = dv + FA_PAD;
    __nv_bfloat16* Qs = (__nv_bfloat16*)fa_smem;             // [2][64][ldk]
    __nv_bfloat16* stage0 = Qs + 2 * FA_BM * ldk;            // two buffers of K [2][64][ldk] and V [64][ldv]
    const int stage_elems = 2 * FA_BN * ldk + FA_BN * ldv;
    float* comb = (float*)stage0;                            // [64][dv] map 2's rows, once the key tiles are done
    __shared__ int s_pos[FA_BM];
    __shared__ int s_page[4][FA_BN];                         // page of every key row of the tile a buffer will hold

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int map = warp >> 2, part_of_map = warp & 3;
    // the tile list is in the order of the tokens; the later tiles of a sequence see the most keys, and go first
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int b = a.tiles[2 * tile], q0 = a.tiles[2 * tile + 1], h = blockIdx.y;
    const int kvh = h / (a.nh / a.nkv);
    const int t0 = a.q_start[b] + q0, n_rows = min(FA_BM, a.q_start[b + 1] - t0);
    // few rows: the warps of a map all take rows 0..15 and share the key tiles; else warp w of a map takes rows 16 w ..
    bool share_keys = a.share != 0 && n_rows <= 16;
    if (share_keys) {                // ... and only where there are at least two tiles of keys to share
        int pf = a.positions[t0], pl = a.positions[t0 + n_rows - 1];
        int lo = a.window > 0 ? max(0, pf - a.window + 1) : 0;
        if (a.chunk > 0) lo = max(lo, pf / a.chunk * a.chunk);
        share_keys = pl - lo / FA_BN * FA_BN >= FA_BN;
    }
    const int row0 = share_keys ? 0 : part_of_map * 16;
    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_pages;

    if (tid < FA_BM) s_pos[tid] = tid < n_rows ? a.positions[t0 + tid] : -1;
    // the queries of both maps
    const int c8 = d >> 3;
    for (int e = tid; e < 2 * FA_BM * c8; e += FA_THREADS) {
        int m = e / (FA_BM * c8), r = (e / c8) % FA_BM, c = (e % c8) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + r) * a.q_stride + (size_t)h * 2 * d + m * d + c);
        *reinterpret_cast<uint4*>(Qs + (m * FA_BM + r) * ldk + c) = v;
    }
    __syncthreads();
    const int pos_first = s_pos[0], pos_last = s_pos[n_rows - 1];
    int lo_blk = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    if (a.chunk > 0) lo_blk = max(lo_blk, pos_first / a.chunk * a.chunk);
    // this thread's two rows
    const int ra = row0 + (lane >> 2), rb = ra + 8;
    const int pos_a = s_pos[ra], pos_b = s_pos[rb];
    int lo_a = a.window > 0 ? max(0, pos_a - a.window + 1) : 0, lo_b = a.window > 0 ? max(0, pos_b - a.window + 1) : 0;
    if (a.chunk > 0 && pos_a >= 0) lo_a = max(lo_a, pos_a / a.chunk * a.chunk);
    if (a.chunk > 0 && pos_b >= 0) lo_b = max(lo_b, pos_b / a.chunk * a.chunk);

    unsigned qf[DK][4];
#pragma unroll
    for (int ks = 0; ks < DK; ++ks)
        if (ks * 16 < d)
            fa_ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                           Qs + (map * FA_BM + row0 + (lane & 15)) * ldk + ks * 16 + (lane >> 4) * 8);
    float o[DVT][4];
#pragma unroll
    for (int i = 0; i < DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    // scores are kept in the base-2 domain: one multiplication by scale * log2(e), then 2^(s - m) is one subtraction and one MUFU
    const float scale2 = a.scale * 1.4426950408889634f;

    // the page of key row r of the tile at k0, or -1 (no such key, or a page the request does not hold)
    auto page_of = [&](int k0, int r) -> int {
        int key = k0 + r;
        if (key > pos_last) return -1;
        int page = table[key / a.page_size];
        if (page < 0 || page >= a.num_pages) { atomicExch(a.status, 4); return -1; }
        return page;
    };
    // copies of the tile at k0 into buffer ``which``, whose rows' pages are in s_page[which]
    auto stage = [&](int k0, int which) {
        __nv_bfloat16* Kd = stage0 + which * stage_elems;
        __nv_bfloat16* Vd = Kd + 2 * FA_BN * ldk;
        const int* pages = s_page[which];
        {   // K: two threads a row of the 2 x 64 rows (map, key), each every second 16-byte piece
            int row = tid >> 1, m = row >> 6, r = row & (FA_BN - 1);
            __nv_bfloat16* dst = Kd + row * ldk;
            int page = pages[r];
            if (page >= 0) {
                const __nv_bfloat16* src = a.k_pool + (((size_t)page * 2 * a.nkv + 2 * kvh + m) * a.page_size + (k0 + r) % a.page_size) * d;
                for (int c = (tid & 1) * 8; c < d; c += 16) {
                    unsigned sa = (unsigned)__cvta_generic_to_shared(dst + c);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + c));
                }
            } else {
                for (int c = (tid & 1) * 8; c < d; c += 16) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        {   // V: four threads a row, each every fourth piece
            int r = tid >> 2;
            __nv_bfloat16* dst = Vd + r * ldv;
            int page = pages[r];
            if (page >= 0) {
                const __nv_bfloat16* src = a.v_pool + (((size_t)page * a.nkv + kvh) * a.page_size + (k0 + r) % a.page_size) * dv;
                for (int c = (tid & 3) * 8; c < dv; c += 32) {
                    unsigned sa = (unsigned)__cvta_generic_to_shared(dst + c);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + c));
                }
            } else {
                for (int c = (tid & 3) * 8; c < dv; c += 32) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // a tile of keys that every row of this warp sees whole needs no mask: all 16 rows are tokens, the tile ends at or
    // before the first row's position and begins at or after the last row's first visible key
    const bool rows_full = row0 + 15 < n_rows;
    const int warp_pos_first = s_pos[row0];
    int warp_lo_last = 0;
    if (rows_full) {
        int pl = s_pos[row0 + 15];
        warp_lo_last = a.window > 0 ? max(0, pl - a.window + 1) : 0;
        if (a.chunk > 0) warp_lo_last = max(warp_lo_last, pl / a.chunk * a.chunk);
    }
    // scores, softmax and P V of the tile of keys at k0, which lies in buffer ``cur``
    auto tile_math = [&](int k0, int cur) {
        const __nv_bfloat16* Ks = stage0 + cur * stage_elems;
        const __nv_bfloat16* Vs = Ks + 2 * FA_BN * ldk;

        const __nv_bfloat16* Km = Ks + map * FA_BN * ldk;
        // a warp none of whose 16 rows is a token (a decode step's tile has one row) only helps with the copies
        if (row0 < n_rows) {
        // the tile's keys in two runs of FA_SUB: scores, softmax and P V of a run before the next (half the registers)
#pragma unroll 1
        for (int sub = 0; sub < FA_BN; sub += FA_SUB) {
            const int ks0 = k0 + sub;
            if (ks0 > pos_last) break;
            float s[FA_SUB / 8][4];
#pragma unroll
            for (int i = 0; i < FA_SUB / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DK; ++ks) {
                if (ks * 16 < d) {
#pragma unroll
                    for (int nt = 0; nt < FA_SUB / 8; nt += 2) {
                        unsigned b0, b1, b2, b3;
                        fa_ldmatrix_x4(b0, b1, b2, b3, Km + (sub + nt * 8 + (lane >> 4) * 8 + (lane & 7)) * ldk + ks * 16 + ((lane >> 3) & 1) * 8);
                        fa_mma(s[nt], qf[ks], b0, b1);
                        fa_mma(s[nt + 1], qf[ks], b2, b3);
                    }
                }
            }
            // scale, mask, running maximum
            float mx_a = -INFINITY, mx_b = -INFINITY;
            if (rows_full && ks0 + FA_SUB - 1 <= warp_pos_first && ks0 >= warp_lo_last) {
#pragma unroll
                for (int nt = 0; nt < FA_SUB / 8; ++nt) {
                    s[nt][0] *= scale2; s[nt][1] *= scale2; s[nt][2] *= scale2; s[nt][3] *= scale2;
                    mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
                    mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < FA_SUB / 8; ++nt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        int key = ks0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        bool upper = e < 2;
                        bool see = upper ? (key <= pos_a && key >= lo_a) : (key <= pos_b && key >= lo_b);
                        float v = see ? s[nt][e] * scale2 : -INFINITY;
                        s[nt][e] = v;
                        if (upper) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                    }
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            float n_a = fmaxf(m_a, mx_a), n_b = fmaxf(m_b, mx_b);
            float use_a = n_a == -INFINITY ? 0.f : n_a, use_b = n_b == -INFINITY ? 0.f : n_b;
            float f_a = m_a == -INFINITY ? 0.f : ce_exp2_fast(m_a - use_a);
            float f_b = m_b == -INFINITY ? 0.f : ce_exp2_fast(m_b - use_b);
            const bool moved = n_a != m_a || n_b != m_b;
            m_a = n_a; m_b = n_b;
            float sum_a = 0.f, sum_b = 0.f;
            unsigned pf[FA_SUB / 16][4];
#pragma unroll
            for (int nt = 0; nt < FA_SUB / 8; ++nt) {
                float p0 = ce_exp2_fast(s[nt][0] - use_a), p1 = ce_exp2_fast(s[nt][1] - use_a);
                float p2 = ce_exp2_fast(s[nt][2] - use_b), p3 = ce_exp2_fast(s[nt][3] - use_b);
                sum_a += p0 + p1;
                sum_b += p2 + p3;
                pf[nt >> 1][(nt & 1) * 2] = fa_pack(p0, p1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = fa_pack(p2, p3);
            }
            sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1); sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
            sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1); sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
            l_a = l_a * f_a + sum_a;
            l_b = l_b * f_b + sum_b;
            if (__any_sync(0xffffffffu, moved)) {            // a maximum rose somewhere in the warp: what is summed so far shrinks
#pragma unroll
                for (int i = 0; i < DVT; ++i) { o[i][0] *= f_a; o[i][1] *= f_a; o[i][2] *= f_b; o[i][3] *= f_b; }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < FA_SUB / 16; ++kk) {
#pragma unroll
                for (int nt = 0; nt < DVT; nt += 2) {
                    if (nt * 8 < dv) {
                        unsigned b0, b1, b2, b3;
                        fa_ldmatrix_x4_trans(b0, b1, b2, b3, Vs + (sub + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ldv + nt * 8 + (lane >> 4) * 8);
                        fa_mma(o[nt], pf[kk], b0, b1);
                        fa_mma(o[nt + 1], pf[kk], b2, b3);
                    }
                }
            }
        }
        }
    };
    const int k_first = lo_blk / FA_BN * FA_BN;
    if (!share_keys) {
        if (tid < FA_BN) {
            s_page[0][tid] = page_of(k_first, tid);
            s_page[1][tid] = page_of(k_first + FA_BN, tid);
        }
        __syncthreads();
        stage(k_first, 0);
        int it = 0;
        for (int k0 = k_first; k0 <= pos_last; k0 += FA_BN, ++it) {
            const int cur = it & 1;
            const bool more = k0 + FA_BN <= pos_last;
            int page_ahead = -1;                    // for the tile after the next: asked for now, stored after the arithmetic
            if (tid < FA_BN && more) page_ahead = page_of(k0 + 2 * FA_BN, tid);
            if (more) {
                stage(k0 + FA_BN, cur ^ 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncthreads();
            tile_math(k0, cur);
            if (tid < FA_BN) s_page[cur][tid] = page_ahead;      // buffer ``cur`` will hold the tile after the next
            __syncthreads();
        }
    } else {
        // Four tiles of keys at a time, one for each warp of a map: a tile of one query row is work for one warp, whose
        // instructions one after another are what the block's time is made of, so the warps take the tiles side by side
        // and their partial rows are merged afterwards.
        for (int g0 = k_first; g0 <= pos_last; g0 += 4 * FA_BN) {
            if (tid < FA_BN)
                for (int w = 0; w < 4; ++w) s_page[w][tid] = page_of(g0 + w * FA_BN, tid);
            __syncthreads();
            for (int w = 0; w < 4; ++w)
                if (g0 + w * FA_BN <= pos_last) stage(g0 + w * FA_BN, w);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            if (g0 + part_of_map * FA_BN <= pos_last) tile_math(g0 + part_of_map * FA_BN, part_of_map);
            __syncthreads();
        }
    }
    const int cq = (lane & 3) * 2;
    if (share_keys) {
        // partial rows of the four warps of each map, after the place of map 2's finished rows: the sums so far [2][4][16][dv]
        // and (maximum, sum) [2][4][16][2]; warp 0 of each map then adds them up in the order of the warps
        float* part = comb + FA_BM * dv;
        float* ml = part + 2 * 4 * 16 * dv;
        const int r_lo = lane >> 2, r_hi = r_lo + 8;
        if (part_of_map != 0) {
            float* mine = part + ((map * 4 + part_of_map) * 16) * dv;
#pragma unroll
            for (int nt = 0; nt < DVT; ++nt) {
                if (nt * 8 < dv) {
                    *reinterpret_cast<float2*>(mine + r_lo * dv + nt * 8 + cq) = make_float2(o[nt][0], o[nt][1]);
                    *reinterpret_cast<float2*>(mine + r_hi * dv + nt * 8 + cq) = make_float2(o[nt][2], o[nt][3]);
                }
            }
            if ((lane & 3) == 0) {
                float* m2 = ml + ((map * 4 + part_of_map) * 16) * 2;
                m2[r_lo * 2] = m_a; m2[r_lo * 2 + 1] = l_a;
                m2[r_hi * 2] = m_b; m2[r_hi * 2 + 1] = l_b;
            }
        }
        __syncthreads();
        if (part_of_map == 0) {
            float big_a = m_a, big_b = m_b;
#pragma unroll
            for (int w = 1; w < 4; ++w) {
                const float* m2 = ml + ((map * 4 + w) * 16) * 2;
                big_a = fmaxf(big_a, m2[r_lo * 2]);
                big_b = fmaxf(big_b, m2[r_hi * 2]);
            }
            float f_a = m_a == -INFINITY ? 0.f : ce_exp2_fast(m_a - big_a), f_b = m_b == -INFINITY ? 0.f : ce_exp2_fast(m_b - big_b);
            l_a *= f_a; l_b *= f_b;
#pragma unroll
            for (int i = 0; i < DVT; ++i) { o[i][0] *= f_a; o[i][1] *= f_a; o[i][2] *= f_b; o[i][3] *= f_b; }
#pragma unroll
            for (int w = 1; w < 4; ++w) {
                const float* m2 = ml + ((map * 4 + w) * 16) * 2;
                const float* theirs = part + ((map * 4 + w) * 16) * dv;
                float ma = m2[r_lo * 2], mb = m2[r_hi * 2];
                float g_a = ma == -INFINITY ? 0.f : ce_exp2_fast(ma - big_a), g_b = mb == -INFINITY ? 0.f : ce_exp2_fast(mb - big_b);
                l_a = fmaf(m2[r_lo * 2 + 1], g_a, l_a);
                l_b = fmaf(m2[r_hi * 2 + 1], g_b, l_b);
#pragma unroll
                for (int nt = 0; nt < DVT; ++nt) {
                    if (nt * 8 < dv) {
                        float2 xa = *reinterpret_cast<const float2*>(theirs + r_lo * dv + nt * 8 + cq);
                        float2 xb = *reinterpret_cast<const float2*>(theirs + r_hi * dv + nt * 8 + cq);
                        o[nt][0] = fmaf(xa.x, g_a, o[nt][0]); o[nt][1] = fmaf(xa.y, g_a, o[nt][1]);
                        o[nt][2] = fmaf(xb.x, g_b, o[nt][2]); o[nt][3] = fmaf(xb.y, g_b, o[nt][3]);
                    }
                }
            }
        }
        __syncthreads();             // the partial rows are read before map 2's finished rows go to the same memory's start
    }
    const bool finishes = !share_keys || part_of_map == 0;       // the warps that hold finished rows
    float i_a = l_a > 0.f ? 1.0f / l_a : 0.f, i_b = l_b > 0.f ? 1.0f / l_b : 0.f;
    if (map == 1 && finishes) {
#pragma unroll
        for (int nt = 0; nt < DVT; ++nt) {
            if (nt * 8 < dv) {
                *reinterpret_cast<float2*>(comb + ra * dv + nt * 8 + cq) = make_float2(o[nt][0] * i_a, o[nt][1] * i_a);
                *reinterpret_cast<float2*>(comb + rb * dv + nt * 8 + cq) = make_float2(o[nt][2] * i_b, o[nt][3] * i_b);
            }
        }
    }
    __syncthreads();
    if (map == 0 && finishes) {
        float ss_a = 0.f, ss_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < DVT; ++nt) {
            if (nt * 8 < dv) {
                float2 xa = *reinterpret_cast<const float2*>(comb + ra * dv + nt * 8 + cq);
                float2 xb = *reinterpret_cast<const float2*>(comb + rb * dv + nt * 8 + cq);
                o[nt][0] = o[nt][0] * i_a - a.lambda * xa.x; o[nt][1] = o[nt][1] * i_a - a.lambda * xa.y;
                o[nt][2] = o[nt][2] * i_b - a.lambda * xb.x; o[nt][3] = o[nt][3] * i_b - a.lambda * xb.y;
                ss_a += o[nt][0] * o[nt][0] + o[nt][1] * o[nt][1];
                ss_b += o[nt][2] * o[nt][2] + o[nt][3] * o[nt][3];
            }
        }
        ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 1); ss_a += __shfl_xor_sync(0xffffffffu, ss_a, 2);
        ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 1); ss_b += __shfl_xor_sync(0xffffffffu, ss_b, 2);
        float g_a = 1.f, g_b = 1.f;
        if (a.gate) {
            if (ra < n_rows) g_a = 1.0f / (1.0f + expf(-__bfloat162float(a.gate[(size_t)(t0 + ra) * a.gate_stride + h])));
            if (rb < n_rows) g_b = 1.0f / (1.0f + expf(-__bfloat162float(a.gate[(size_t)(t0 + rb) * a.gate_stride + h])));
        }
        float mul_a = a.out_scale * g_a / sqrtf(ss_a / (float)dv + a.eps), mul_b = a.out_scale * g_b / sqrtf(ss_b / (float)dv + a.eps);
#pragma unroll
        for (int nt = 0; nt < DVT; ++nt) {
            if (nt * 8 < dv) {
                if (ra < n_rows)
                    *reinterpret_cast<unsigned*>(a.out + ((size_t)(t0 + ra) * a.nh + h) * dv + nt * 8 + cq) = fa_pack(o[nt][0] * mul_a, o[nt][1] * mul_a);
                if (rb < n_rows)
                    *reinterpret_cast<unsigned*>(a.out + ((size_t)(t0 + rb) * a.nh + h) * dv + nt * 8 + cq) = fa_pack(o[nt][2] * mul_b, o[nt][3] * mul_b);
            }
        }
    }
}

extern "C" int ce_diff_attention_mma_supported(int d, int dv, int q_stride) {
    return d >= 16 && d <= 128 && d % 16 == 0 && dv >= 16 && dv <= 256 && dv % 16 == 0 && q_stride % 8 == 0;
}

template <int DK, int DVT>
static void launch_flash_diff(const FlashDiffArgs& a, int n_tiles, cudaStream_t stream) {
    size_t smem = (size_t)(2 * FA_BM * (a.d + FA_PAD) + (a.share ? 4 : 2) * (2 * FA_BN * (a.d + FA_PAD) + FA_BN * (a.dv + FA_PAD))) * sizeof(__nv_bfloat16);
    if (smem > 40 * 1024)            // the kernel's static arrays count toward the 48 KB a launch gets without asking
        cudaFuncSetAttribute(diff_attention_mma_kernel<DK, DVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce_note("diff_attention_mma_kernel");
    ce_launch(diff_attention_mma_kernel<DK, DVT>, dim3(n_tiles, a.nh), FA_THREADS, smem, stream, a);
}

extern "C" int ce_diff_attention_mma(const void* q, const void* k_pool, const void* v_pool, const void* gate, void* out,
                                     const int* positions, const int* seq_slot, const int* q_start, const int* block_table,
                                     const int* tiles, int* status, int n_tiles, int nh, int nkv, int d, int dv, int q_stride,
                                     int gate_stride, int page_size, int max_pages, int num_pages, int window, int chunk,
                                     float scale, float lambda, float eps, float out_scale, cudaStream_t stream) {
    if (n_tiles == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !seq_slot || !q_start || !block_table || !tiles || !status)
        return ce_fail(CE_ERR_ARG, "ce_diff_attention_mma: null pointer");
    if (!ce_diff_attention_mma_supported(d, dv, q_stride))
        return ce_fail(CE_ERR_SIZE, "ce_diff_attention_mma: head sizes %d / %d or row stride %d not supported", d, dv, q_stride);
    if (nkv <= 0 || nh % nkv != 0)
        return ce_fail(CE_ERR_SIZE, "ce_diff_attention_mma: %d heads are not a multiple of %d kv heads", nh, nkv);
    if ((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) || (((uintptr_t)out) & 3))
        return ce_fail(CE_ERR_SIZE, "ce_diff_attention_mma: operands must be 16-byte aligned");
    FlashDiffArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (const __nv_bfloat16*)gate,
                    (__nv_bfloat16*)out, positions, seq_slot, q_start, block_table, tiles, status, nh, nkv, d, dv, q_stride,
                    gate_stride, page_size, max_pages, num_pages, window, chunk, 0, scale, lambda, eps, out_scale};
    // Few blocks (a decode step: a block per sequence and head): four buffers, so that the warps of a map can take four tiles
    // of keys side by side, if they and the partial rows to merge fit; many blocks (prompts): two buffers, two blocks an SM.
    if ((long long)n_tiles * nh <= (long long)ce_sm_count()) {       // one block an SM then: more blocks than SMs would wait their turn
        size_t q_bytes = (size_t)2 * FA_BM * (d + FA_PAD) * sizeof(__nv_bfloat16);
        size_t stage_bytes = (size_t)(2 * FA_BN * (d + FA_PAD) + FA_BN * (dv + FA_PAD)) * sizeof(__nv_bfloat16);
        size_t merge_bytes = (size_t)(FA_BM * dv + 2 * 4 * 16 * dv + 2 * 4 * 16 * 2) * sizeof(float);
        if (q_bytes + 4 * stage_bytes <= 200 * 1024 && merge_bytes <= 4 * stage_bytes) a.share = 1;
    }
    if (d <= 64) {
        if (dv <= 64) launch_flash_diff<4, 8>(a, n_tiles, stream);
        else if (dv <= 128) launch_flash_diff<4, 16>(a, n_tiles, stream);
        else launch_flash_diff<4, 32>(a, n_tiles, stream);
    } else {
        if (dv <= 64) launch_flash_diff<8, 8>(a, n_tiles, stream);
        else if (dv <= 128) launch_flash_diff<8, 16>(a, n_tiles, stream);
        else launch_flash_diff<8, 32>(a, n_tiles, stream);
    }
    return ce_check_launch("ce_diff_attention_mma");
}
