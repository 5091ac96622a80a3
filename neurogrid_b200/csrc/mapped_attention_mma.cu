// The attention of mapped_attention.cu for long bfloat16 steps, on the tensor cores (mma.sync m16n8k16).
//
// Same mathematics: float32 scores, float32 online softmax (as powers of two, on the special-function unit), float32 weights.  The products run on the tensor cores
// without giving that up: q and k are bfloat16 as the cache holds them, so q.k is a float32 sum of exact products;
// a float32 weight p enters the weighted sum as three bfloat16 terms hi + mid + lo (what is left is below 2^-24 p),
// each term's products with the bfloat16 values exact in the float32 accumulators.  A distance bias per head
// (slope * (position - key position), taken off the score) and a sink per head (exp(sink) in the softmax's sum, no
// value) are optional.
//
// A block takes consecutive rows of one entry and one query head: 64 rows (one map) or 32 rows (two maps; a warp
// per map and 16 rows, the maps combined in the epilogue), and walks the keys the block's rows can see, kept first
// tokens then the window, in tiles of 64: keys (of each map) and values are staged once in shared memory for the four
// warps (16-byte asynchronous copies through the block table, a tile ahead of the one being worked on), S = Q K^T in registers, mask and cap per element,
// P V with P straight from the accumulators' layout, values through ldmatrix.trans.  Specialised on the key and
// value sizes (-DNG_MA_D, -DNG_MA_DV: multiples of 16, up to 128).
#include "ng_common.cuh"

#if !defined(NG_MA_D) || !defined(NG_MA_DV)
#error "compile with -DNG_MA_D=<key size> -DNG_MA_DV=<value size>"
#endif
static_assert(NG_MA_D % 16 == 0 && NG_MA_D >= 16 && NG_MA_D <= 128, "key size: a multiple of 16 up to 128");
static_assert(NG_MA_DV % 16 == 0 && NG_MA_DV >= 16 && NG_MA_DV <= 128, "value size: a multiple of 16 up to 128");

typedef __nv_bfloat16 bf16;
constexpr int D = NG_MA_D, DV = NG_MA_DV;
constexpr int KT = 64, WARPS = 4, THREADS = 128;
constexpr int QP = D + 8, KP = D + 8, VP = DV + 8;      // row pitches in elements: 16 bytes of padding against bank conflicts

struct MmaParams {
    const bf16* q; const bf16* k_pages; const bf16* v_pages; const int* table; int table_stride;
    const int* cu_q; const int* ctx_before; bf16* out; int out_ld;
    int nH, nG, page_size, num_pages, window, keep_first;
    int chunk;                         // > 0: a row sees only the keys of its own chunk of that many positions (counted from 0)
    float scale, softcap, lambda, post_scale, eps; int head_norm;
    float* partial; int n_splits;      // GROUP: runs of keys, their states [row, head, run, map, DV + 2]
    const float* slopes; const float* sinks;    // per head or null: slope * (pos - key position) off every score; exp(sink) in the sum
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory without passing registers; `real` false: zeros instead (nothing is read)
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool real) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = real ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(n) : "memory");
}
// 2^x on the special-function unit (relative error about 2^-22; 2^-inf = 0)
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// tanh(x) = 1 - 2 / (1 + e^(2x)): exact limits at both ends, absolute error of a few 1e-7
__device__ __forceinline__ float tanh_ex2(float x) {
    return 1.f - __fdividef(2.f, 1.f + ex2f(x * 2.8853900817779268f));
}
__device__ __forceinline__ uint32_t pack2(float x, float y) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// p = hi + mid + lo in bfloat16 terms, two weights at a time
__device__ __forceinline__ void split3(float x, float y, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
    const float xh = __bfloat162float(__float2bfloat16_rn(x)), yh = __bfloat162float(__float2bfloat16_rn(y));
    const float xr = x - xh, yr = y - yh;
    const float xm = __bfloat162float(__float2bfloat16_rn(xr)), ym = __bfloat162float(__float2bfloat16_rn(yr));
    hi = pack2(xh, yh);
    mid = pack2(xm, ym);
    lo = pack2(xr - xm, yr - ym);
}

// GROUP: for entries that bring one token.  The rows of the tile are then the query heads of one KV group (up to 16; they
// share keys and values and here also the position), a block takes (run of keys, entry, KV group), and instead of the
// finished heads it leaves each run's state (maximum, sum, weighted values) for the kernel that merges runs.
template <int M, bool GROUP>
__global__ void __launch_bounds__(THREADS, 3)
mapped_attention_mma_kernel(const MmaParams p) {
    constexpr int ROWS = (WARPS / M) * 16;               // rows of a block
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                        // [M][ROWS][QP]
    bf16* Ks = Qs + M * ROWS * QP;                                       // [2][M][KT][KP]
    bf16* Vs = Ks + 2 * M * KT * KP;                                     // [2][KT][VP]
    float* Os = reinterpret_cast<float*>(Ks);                            // epilogue: [M][ROWS][DV], over the tiles
    __shared__ int kpos_s[3][KT];                                        // per tile in flight or in use (three: see the loop)
    __shared__ long long koff_s[3][KT];
    __shared__ int tile_bad_s[3][2];                                     // a key of the tile has no page                                  // element offset of the key's page slot, -1: none
    ng_pdl_trigger();
    const int entry = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = p.cu_q[entry], q_len = p.cu_q[entry + 1] - q0;
    const int r0 = GROUP ? 0 : blockIdx.x * ROWS;        // first row of the block within the entry
    ng_pdl_wait();
    if (GROUP ? q_len != 1 : r0 >= q_len) return;
    const int before = p.ctx_before[entry];
    const int group_heads = p.nH / p.nG;
    const int n_rows = GROUP ? group_heads : min(ROWS, q_len - r0);
    const int g = GROUP ? blockIdx.z : blockIdx.z / group_heads;
    const int head = GROUP ? g * group_heads : blockIdx.z;               // GROUP: the first head of the tile's rows
    const int map = M == 2 ? (warp & 1) : 0;
    const int wt = M == 2 ? (warp >> 1) : warp;          // the warp's tile of 16 rows
    const bf16* qg = ng_after_wait(p.q);
    // ---- Q: rows r0.., both maps, into shared memory (rows beyond the entry: zeros)
    for (int i = tid; i < M * ROWS * (D / 8); i += THREADS) {
        const int ch = i % (D / 8), row = (i / (D / 8)) % ROWS, m = i / ((D / 8) * ROWS);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < n_rows)
            v = *reinterpret_cast<const uint4*>(qg + ((size_t)(q0 + (GROUP ? 0 : r0 + row)) * p.nH + head + (GROUP ? row : 0)) * M * D +
                                                (size_t)m * D + ch * 8);
        *reinterpret_cast<uint4*>(Qs + ((size_t)m * ROWS + row) * QP + ch * 8) = v;
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldsm_x4(qf[ks], Qs + ((size_t)map * ROWS + wt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QP + ks * 16 + (lane >> 4) * 8);
    // ---- the keys the block's rows see: kept first tokens [0, n_sink), then [lo, last position]
    const int pos_first = before + r0, pos_last = GROUP ? pos_first : before + r0 + n_rows - 1;
    int lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    if (p.chunk > 0) lo = max(lo, (pos_first / p.chunk) * p.chunk);       // the first row's chunk starts earliest
    const int n_sink = min(p.keep_first, lo);
    const int all_keys = n_sink + (pos_last - lo + 1);
    int t_begin = 0, n_keys = all_keys;                  // the block's run of the key list: [t_begin, n_keys)
    if (GROUP && p.n_splits > 1) {
        const int tiles = (all_keys + KT - 1) / KT, per = (tiles + p.n_splits - 1) / p.n_splits;
        t_begin = min(all_keys, (int)blockIdx.x * per * KT);
        n_keys = min(all_keys, t_begin + per * KT);
    }
    const int gq = lane >> 2, tq = lane & 3;
    const int row_a = wt * 16 + gq, row_b = row_a + 8;   // this thread's two rows within the block
    const int pos_a = GROUP ? pos_first : pos_first + row_a, pos_b = GROUP ? pos_first : pos_first + row_b;
    const int w_first = GROUP ? pos_first : pos_first + wt * 16;                     // the warp's positions
    const int w_last = GROUP ? pos_first : min(pos_last, w_first + 15);
    const int w_span = GROUP ? 0 : 15;
    // chunk starts: of this thread's two rows, and of the warp's first and last row
    const int cs_a = p.chunk > 0 ? (pos_a / p.chunk) * p.chunk : 0, cs_b = p.chunk > 0 ? (pos_b / p.chunk) * p.chunk : 0;
    const int cs_first = p.chunk > 0 ? (w_first / p.chunk) * p.chunk : 0;
    const int cs_last = p.chunk > 0 ? ((w_first + w_span) / p.chunk) * p.chunk : 0;
    const bool warp_live = wt * 16 < n_rows;
    // the distance bias of this thread's two rows, in the softmax's powers of two (GROUP: a row is a head)
    float slope_a = 0.f, slope_b = 0.f;
    if (p.slopes) {
        slope_a = p.slopes[GROUP ? head + min(row_a, n_rows - 1) : head] * 1.4426950408889634f;
        slope_b = p.slopes[GROUP ? head + min(row_b, n_rows - 1) : head] * 1.4426950408889634f;
    }
    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const int* trow = p.table + (size_t)entry * p.table_stride;

    // Two buffers: while the warps work on a tile, the next one is on its way (cp.async, 16 bytes a copy; a key that
    // is not there is filled with zeros).  A tile's page slots are looked up one iteration ahead of its copies.
    auto lookup = [&](int t0, int b) {
        if (tid < KT) {
            const int t = t0 + tid;
            int kpos = -1;
            long long off = -1;
            if (t < n_keys) {
                kpos = t < n_sink ? t : lo + (t - n_sink);
                const int page = trow[kpos / p.page_size];
                if (page >= 0 && page < p.num_pages) off = (long long)page * p.page_size + (kpos % p.page_size);
                else kpos = -1;
            }
            kpos_s[b][tid] = kpos;
            koff_s[b][tid] = off;
            const unsigned bad = __ballot_sync(0xffffffffu, t < n_keys && off < 0);      // KT = 64: warps 0 and 1, whole
            if (lane == 0) tile_bad_s[b][warp] = bad != 0u;
        }
    };
    auto copy_tile = [&](int b, int mb) {
        bf16* kb = Ks + (size_t)b * M * KT * KP;
        bf16* vb = Vs + (size_t)b * KT * VP;
        for (int i = tid; i < M * KT * (D / 8); i += THREADS) {
            const int ch = i % (D / 8), key = (i / (D / 8)) % KT, m = i / ((D / 8) * KT);
            const long long off = koff_s[mb][key];
            const long long page = off >= 0 ? off / p.page_size : 0, slot = off >= 0 ? off % p.page_size : 0;
            cp_async16(kb + ((size_t)m * KT + key) * KP + ch * 8,
                       p.k_pages + (((size_t)page * p.nG * M + (size_t)g * M + m) * p.page_size + slot) * D + ch * 8, off >= 0);
        }
        for (int i = tid; i < KT * (DV / 8); i += THREADS) {
            const int ch = i % (DV / 8), key = i / (DV / 8);
            const long long off = koff_s[mb][key];
            const long long page = off >= 0 ? off / p.page_size : 0, slot = off >= 0 ? off % p.page_size : 0;
            cp_async16(vb + (size_t)key * VP + ch * 8,
                       p.v_pages + (((size_t)page * p.nG + g) * p.page_size + slot) * DV + ch * 8, off >= 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    lookup(t_begin, 0);
    __syncthreads();
    copy_tile(0, 0);
    int buf = 0, it = 0;
    for (int t0 = t_begin; t0 < n_keys; t0 += KT, buf ^= 1, ++it) {
        const bool more = t0 + KT < n_keys;
        // the lookup of tile it+1 goes to slot (it+1) % 3: slower warps may still read tile it-1's positions (slot
        // (it-1) % 3) and tile it's copies were made from slot it % 3; the slot's last readers (tile it-2) passed the
        // barrier of the iteration before
        if (more) lookup(t0 + KT, (it + 1) % 3);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                 // this tile has landed; the other data buffer is free
        if (more) copy_tile(buf ^ 1, (it + 1) % 3);
        const int* kpos_t = kpos_s[it % 3];
        // does any row of the warp see any key of the tile?  (positions ascend within both parts of the list)
        bool any = warp_live;
        if (any) {
            const int t_last = min(n_keys, t0 + KT) - 1;
            const int k_first = t0 < n_sink ? t0 : lo + (t0 - n_sink);
            const int k_last = t_last < n_sink ? t_last : lo + (t_last - n_sink);
            const bool sink_part = t0 < n_sink;
            const int w_lo = max(p.window > 0 ? max(0, w_first - p.window + 1) : 0, cs_first);   // lowest key the warp's rows see
            any = k_first <= w_last && (sink_part || k_last >= w_lo || k_first < p.keep_first);
        }
        if (!any) continue;
        // ---- S = Q K^T
        float s[KT / 8][4];
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        const bf16* kt = Ks + ((size_t)buf * M + map) * KT * KP;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int jp = 0; jp < KT / 16; ++jp) {
                uint32_t b[4];
                ldsm_x4(b, kt + ((size_t)jp * 16 + (lane & 7) + (lane >> 4) * 8) * KP + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[2 * jp], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * jp + 1], qf[ks], b[2], b[3]);
            }
        }
        // ---- scale, cap, mask; online softmax in float32, in powers of two (scores times log2 e)
        // a tile that every row of the warp sees whole (the bulk of a long window) needs no mask
        bool interior;
        const int tile_first = t0 < n_sink ? t0 : lo + (t0 - n_sink);      // an interior tile's keys are tile_first + column
        {
            const int k_first = tile_first, k_last = k_first + KT - 1;
            interior = t0 + KT <= n_keys && (t0 >= n_sink || t0 + KT <= n_sink) && (GROUP || wt * 16 + 15 < n_rows) &&
                       k_last <= w_first && (p.window <= 0 || w_first + w_span - k_first < p.window || k_last < p.keep_first) &&
                       k_first >= cs_last &&
                       !tile_bad_s[it % 3][0] && !tile_bad_s[it % 3][1];
        }
        constexpr float LOG2E = 1.4426950408889634f;
        const float sc2 = p.scale * LOG2E, inv_cap = p.softcap > 0.f ? p.scale / p.softcap : 0.f, cap2 = p.softcap * LOG2E;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = p.softcap > 0.f ? cap2 * tanh_ex2(s[j][e] * inv_cap) : s[j][e] * sc2;
                const int pos = (e < 2) ? pos_a : pos_b;
                if (p.slopes) {
                    const int kp = interior ? tile_first + j * 8 + 2 * tq + (e & 1) : kpos_t[j * 8 + 2 * tq + (e & 1)];
                    v -= ((e < 2) ? slope_a : slope_b) * (float)(pos - kp);
                }
                if (!interior) {
                    const int kpos = kpos_t[j * 8 + 2 * tq + (e & 1)];
                    const bool row_ok = ((e < 2) ? row_a : row_b) < n_rows;
                    const bool vis = row_ok && kpos >= ((e < 2) ? cs_a : cs_b) && kpos <= pos &&
                                     (p.window <= 0 || pos - kpos < p.window || kpos < p.keep_first);
                    v = vis ? v : -INFINITY;
                }
                s[j][e] = v;
                if (e < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
            }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        const float ca = m_a == -INFINITY ? 0.f : ex2f(m_a - mn_a), cb = m_b == -INFINITY ? 0.f : ex2f(m_b - mn_b);
        const float ua = mn_a == -INFINITY ? 0.f : mn_a, ub = mn_b == -INFINITY ? 0.f : mn_b;
        m_a = mn_a; m_b = mn_b;
        l_a *= ca; l_b *= cb;
#pragma unroll
        for (int j = 0; j < DV / 8; ++j) { o[j][0] *= ca; o[j][1] *= ca; o[j][2] *= cb; o[j][3] *= cb; }
#pragma unroll
        for (int j = 0; j < KT / 8; ++j) {
            s[j][0] = ex2f(s[j][0] - ua); s[j][1] = ex2f(s[j][1] - ua);        // 2^-inf = 0 for what the mask hides
            s[j][2] = ex2f(s[j][2] - ub); s[j][3] = ex2f(s[j][3] - ub);
            l_a += s[j][0] + s[j][1];
            l_b += s[j][2] + s[j][3];
        }
        // ---- O += P V, P as three bfloat16 terms
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t ah[4], am[4], al[4];
            split3(s[2 * kk][0], s[2 * kk][1], ah[0], am[0], al[0]);
            split3(s[2 * kk][2], s[2 * kk][3], ah[1], am[1], al[1]);
            split3(s[2 * kk + 1][0], s[2 * kk + 1][1], ah[2], am[2], al[2]);
            split3(s[2 * kk + 1][2], s[2 * kk + 1][3], ah[3], am[3], al[3]);
#pragma unroll
            for (int np = 0; np < DV / 16; ++np) {
                uint32_t b[4];
                ldsm_x4_t(b, Vs + (size_t)buf * KT * VP + ((size_t)kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VP + np * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * np], al, b[0], b[1]);        // smallest terms first
                mma_bf16(o[2 * np + 1], al, b[2], b[3]);
                mma_bf16(o[2 * np], am, b[0], b[1]);
                mma_bf16(o[2 * np + 1], am, b[2], b[3]);
                mma_bf16(o[2 * np], ah, b[0], b[1]);
                mma_bf16(o[2 * np + 1], ah, b[2], b[3]);
            }
        }
    }
    // ---- epilogue: each map's a = O / l into shared memory, then the maps combined row by row
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // (an empty run has copies in flight that nobody waited for)
    __syncthreads();                                     // every warp has left the tiles
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (GROUP) {
        // the run's state per head and map, as the kernel that merges runs reads it: maximum (natural logarithm), sum,
        // weighted values relative to that maximum
        if (warp_live) {
            constexpr float LN2 = 0.6931471805599453f;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int r = half ? row_b : row_a;
                if (r < n_rows) {
                    float* ps = p.partial + ((((size_t)q0 * p.nH + head + r) * p.n_splits + blockIdx.x) * M + map) * (DV + 2);
                    if (tq == 0) { ps[0] = (half ? m_b : m_a) * LN2; ps[1] = half ? l_b : l_a; }
#pragma unroll
                    for (int j = 0; j < DV / 8; ++j) {
                        ps[2 + j * 8 + 2 * tq] = o[j][2 * half];
                        ps[2 + j * 8 + 2 * tq + 1] = o[j][2 * half + 1];
                    }
                }
            }
        }
        return;
    }
    if (p.sinks) {                                       // the term without key or value, once per row
        const float sk = p.sinks[head] * 1.4426950408889634f;
        if (m_a != -INFINITY) l_a += ex2f(sk - m_a);
        if (m_b != -INFINITY) l_b += ex2f(sk - m_b);
    }
    const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
        float* oa = Os + ((size_t)map * ROWS + row_a) * DV + j * 8 + 2 * tq;
        float* ob = Os + ((size_t)map * ROWS + row_b) * DV + j * 8 + 2 * tq;
        oa[0] = o[j][0] * ia; oa[1] = o[j][1] * ia;
        ob[0] = o[j][2] * ib; ob[1] = o[j][3] * ib;
    }
    __syncthreads();
    for (int row = warp; row < n_rows; row += WARPS) {
        float v[DV / 32 + 1];
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < DV / 32 + 1; ++u) {
            const int c = lane + 32 * u;
            v[u] = 0.f;
            if (c < DV) {
                v[u] = Os[(size_t)row * DV + c];
                if (M == 2) v[u] -= p.lambda * Os[((size_t)ROWS + row) * DV + c];
                ss += v[u] * v[u];
            }
        }
        float r = 1.f;
        if (p.head_norm) r = rsqrtf(ng_warp_sum(ss) / (float)DV + p.eps) * p.post_scale;
        bf16* dst = p.out + (size_t)(q0 + r0 + row) * p.out_ld + (size_t)head * DV;
#pragma unroll
        for (int u = 0; u < DV / 32 + 1; ++u) {
            const int c = lane + 32 * u;
            if (c < DV) dst[c] = __float2bfloat16_rn(v[u] * r);
        }
    }
}

template <int M, bool GROUP>
static int mma_launch(const MmaParams& p, int n_entries, int max_q, cudaStream_t stream) {
    constexpr int ROWS = (WARPS / M) * 16;
    const size_t tiles = ((size_t)M * ROWS * QP + 2 * ((size_t)M * KT * KP + (size_t)KT * VP)) * sizeof(bf16);
    const size_t epi = (size_t)M * ROWS * QP * sizeof(bf16) + (size_t)M * ROWS * DV * sizeof(float);
    const size_t smem = tiles > epi ? tiles : epi;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(mapped_attention_mma_kernel<M, GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        attr = true;
    }
    dim3 grid(GROUP ? p.n_splits : (max_q + ROWS - 1) / ROWS, n_entries, GROUP ? p.nG : p.nH);
    if (grid.y > 65535 || grid.z > 65535) return NG_BAD_SIZE;
    NG_LAUNCH((mapped_attention_mma_kernel<M, GROUP>), grid, THREADS, smem, stream, p);
    return ng_launch_status();
}

// q [N, nH * n_maps * D] bfloat16; keys [P, nG * n_maps, page, D]; values [P, nG, page, DV]; out rows out_ld apart.
// Rows are named by cu_q (first row of each entry) and ctx_before (tokens of the request before the step).
NG_EXPORT int ng_mapped_attention_mma(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                      int table_stride, const int* cu_q, const int* ctx_before, void* out, int out_ld,
                                      int n_entries, int max_q, int nH, int nG, int n_maps, int d, int dv, int page_size,
                                      int num_pages, int window, int keep_first, float scale, float softcap, float lambda,
                                      float post_scale, float eps, int head_norm, const float* slopes, const float* sinks,
                                      int chunk, cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0) return NG_OK;
    if (d != D || dv != DV || nH <= 0 || nG <= 0 || nH % nG || page_size <= 0 || n_maps < 1 || n_maps > 2 || out_ld < nH * dv ||
        window < 0 || keep_first < 0 || chunk < 0 || (chunk > 0 && keep_first > 0) || ((uintptr_t)q & 15) ||
        ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
        return NG_BAD_SIZE;
    MmaParams p{(const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, table, table_stride, cu_q, ctx_before, (bf16*)out,
                out_ld, nH, nG, page_size, num_pages, window, keep_first, chunk, scale, softcap, lambda, post_scale, eps, head_norm,
                nullptr, 1, slopes, sinks};
    return n_maps == 2 ? mma_launch<2, false>(p, n_entries, max_q, stream) : mma_launch<1, false>(p, n_entries, max_q, stream);
}

// The same for entries of one token: the heads of a KV group are the rows of a tile (nH / nG <= 16), every row's keys are
// cut into n_splits runs, and each run's state goes to partial (float32 [N, nH, n_splits, n_maps, DV + 2]: maximum, sum,
// weighted values), from where the kernel that merges runs (mapped_attention.cu) finishes the heads.  Entries of another
// length are left alone.
NG_EXPORT int ng_mapped_attention_group(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                        int table_stride, const int* cu_q, const int* ctx_before, float* partial,
                                        int n_entries, int n_splits, int nH, int nG, int n_maps, int d, int dv, int page_size,
                                        int num_pages, int window, int keep_first, float scale, float softcap,
                                        const float* slopes, int chunk, cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (d != D || dv != DV || nH <= 0 || nG <= 0 || nH % nG || nH / nG > 16 || page_size <= 0 || n_maps < 1 || n_maps > 2 ||
        window < 0 || keep_first < 0 || chunk < 0 || (chunk > 0 && keep_first > 0) || n_splits < 1 || n_splits > 65535 || !partial ||
        ((uintptr_t)q & 15) ||
        ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
        return NG_BAD_SIZE;
    MmaParams p{(const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, table, table_stride, cu_q, ctx_before, nullptr, 0,
                nH, nG, page_size, num_pages, window, keep_first, chunk, scale, softcap, 0.f, 1.f, 0.f, 0, partial, n_splits, slopes,
                nullptr};
    return n_maps == 2 ? mma_launch<2, true>(p, n_entries, 1, stream) : mma_launch<1, true>(p, n_entries, 1, stream);
}
