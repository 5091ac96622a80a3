// Latent attention, the row kernels around its attention core.
//
// latent_prep: a row of the stacked down projection is [c_q raw (rq) | c raw (rkv) | key part raw (rot) | gate logits (nH)].
//   c_q = c_q raw / sqrt(mean(c_q raw^2) + eps) * wq        -> cq_out [n_rows, rq]      (activation type)
//   c   = c raw   / sqrt(mean(c raw^2) + eps) * wkv         -> the row's place in the layer's pages
//                                                             [pages, 1, page_size, rp], columns rkv+rot..rp zero
//   key part (rot columns, not normed), rotated by the row's position: pair i is (2i, 2i+1) or, with half
//   pairing, (i, i + rot/2), its angle position * inv_freq[i]  -> columns rkv..rkv+rot of the same place
//   gate = sigmoid(gate logits)                             -> gate_out [n_rows, nH]    (float32; nH: gate columns)
// rkv = 0 (no pages): a layer that reads another layer's latents.
// Both norms, the angles and the gate are float32; only what a matrix product or the cache reads is rounded.
//
// latent_rope_q: columns off..off+rot of every head of q [n_rows, nH * rp] are rotated in place the same way.
//
// head_up_gate: out[row, h, :] = (W[h] o[row, h, :rank]) * gate[row, h, :] for W [nH, dv, rank]: what a head's
//   weighted latents become when the expansion to values cannot be folded into the output projection (a gate per
//   element sits between them).
//
// head_gate: y[row, h, :] *= gate[row, h] for rows of [n_rows, nH * width] (for a core that does not gate itself).
#include "ng_common.cuh"

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ x, const float* __restrict__ wq, const float* __restrict__ wkv,
                   T* __restrict__ cq_out, T* __restrict__ pages, float* __restrict__ gate_out,
                   const int* __restrict__ table, int table_stride, const int* __restrict__ positions,
                   const int* __restrict__ row_entry, int rq, int rkv, int rp, int nH, int page_size, int num_pages,
                   float eps, int* __restrict__ status, int rot, const float* __restrict__ inv_freq, int half_pairing) {
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int entry = row_entry[row];
    if (entry < 0) return;
    const T* xr = x + (size_t)row * (rq + rkv + rot + nH);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rq; i += blockDim.x) {
        const float v = ng_ld(xr + i);
        ss += v * v;
    }
    ss = ng_block_sum(ss, red);
    const float r1 = rsqrtf(ss / (float)rq + eps);
    for (int i = threadIdx.x; i < rq; i += blockDim.x) ng_st(cq_out + (size_t)row * rq + i, ng_ld(xr + i) * r1 * wq[i]);
    if (rkv > 0) {
        ss = 0.f;
        for (int i = threadIdx.x; i < rkv; i += blockDim.x) {
            const float v = ng_ld(xr + rq + i);
            ss += v * v;
        }
        ss = ng_block_sum(ss, red);
        const float r2 = rsqrtf(ss / (float)rkv + eps);
        const int pos = positions[row];
        const int page = pos >= 0 ? table[(size_t)entry * table_stride + pos / page_size] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(status, NG_STATUS_BAD_PAGE);
        } else {
            T* dst = pages + ((size_t)page * page_size + (pos % page_size)) * rp;
            for (int i = threadIdx.x; i < rp; i += blockDim.x)
                if (i < rkv || i >= rkv + rot) ng_st(dst + i, i < rkv ? ng_ld(xr + rq + i) * r2 * wkv[i] : 0.f);
            const T* kr = xr + rq + rkv;
            for (int i = threadIdx.x; i < rot / 2; i += blockDim.x) {
                const int c1 = half_pairing ? i : 2 * i, c2 = half_pairing ? i + rot / 2 : 2 * i + 1;
                float sn, cs;
                sincosf((float)pos * inv_freq[i], &sn, &cs);
                const float a = ng_ld(kr + c1), b = ng_ld(kr + c2);
                ng_st(dst + rkv + c1, a * cs - b * sn);
                ng_st(dst + rkv + c2, b * cs + a * sn);
            }
        }
    }
    for (int h = threadIdx.x; h < nH; h += blockDim.x)
        gate_out[(size_t)row * nH + h] = 1.f / (1.f + expf(-ng_ld(xr + rq + rkv + rot + h)));
}

template <typename T>
__global__ void latent_rope_q_kernel(T* __restrict__ q, const int* __restrict__ positions, const int* __restrict__ row_entry,
                                     const float* __restrict__ inv_freq, int nH, int rp, int off, int rot, int half_pairing) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    if (row_entry[row] < 0) return;
    const float pos = (float)positions[row];
    T* qr = q + (size_t)row * nH * rp;
    const int half = rot / 2;
    for (int idx = threadIdx.x; idx < nH * half; idx += blockDim.x) {
        const int h = idx / half, i = idx - h * half;
        const int c1 = half_pairing ? i : 2 * i, c2 = half_pairing ? i + half : 2 * i + 1;
        T* p = qr + (size_t)h * rp + off;
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        const float a = ng_ld(p + c1), b = ng_ld(p + c2);
        ng_st(p + c1, a * cs - b * sn);
        ng_st(p + c2, b * cs + a * sn);
    }
}

// A block takes HU_ROWS rows of one head: their weighted latents lie in shared memory (float32), a warp takes output
// columns in turn with its lanes dealt over the latent's coordinates, so W[h] is read once per HU_ROWS rows, in order.
// A (row, column) sum is formed the same way whatever else the step holds.  A step of few rows deals a head's output
// columns to gridDim.z blocks, so that the weights are streamed by many blocks.
#define HU_ROWS 16
template <typename T>
__global__ void __launch_bounds__(256)
head_up_gate_kernel(const T* __restrict__ o, const T* __restrict__ w, const float* __restrict__ gate, T* __restrict__ out,
                    int n_rows, int nH, int rp, int rank, int dv, int ldo) {
    extern __shared__ float os[];                     // [HU_ROWS][rank]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int r0 = blockIdx.x * HU_ROWS, head = blockIdx.y;
    const int rows = min(HU_ROWS, n_rows - r0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int idx = threadIdx.x; idx < HU_ROWS * rank; idx += blockDim.x) {
        const int r = idx / rank, c = idx - r * rank;
        os[idx] = r < rows ? ng_ld(o + ((size_t)(r0 + r) * nH + head) * rp + c) : 0.f;
    }
    __syncthreads();
    const T* wh = w + (size_t)head * dv * rank;
    for (int v = blockIdx.z * nwarp + warp; v < dv; v += nwarp * gridDim.z) {
        float acc[HU_ROWS];
#pragma unroll
        for (int r = 0; r < HU_ROWS; ++r) acc[r] = 0.f;
        for (int c = lane; c < rank; c += 32) {
            const float wv = ng_ld(wh + (size_t)v * rank + c);
#pragma unroll
            for (int r = 0; r < HU_ROWS; ++r) acc[r] = fmaf(wv, os[r * rank + c], acc[r]);
        }
#pragma unroll
        for (int r = 0; r < HU_ROWS; ++r) acc[r] = ng_warp_sum(acc[r]);
        if (lane < rows) {
            float y = 0.f;
#pragma unroll
            for (int r = 0; r < HU_ROWS; ++r)
                if (r == lane) y = acc[r];
            const size_t col = (size_t)head * dv + v;
            if (gate) y *= gate[(size_t)(r0 + lane) * nH * dv + col];
            ng_st(out + (size_t)(r0 + lane) * ldo + col, y);
        }
    }
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ y, const float* __restrict__ gate, size_t total, int nH, int width) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t rh = i / width;              // row * nH + head
    ng_st(y + i, ng_ld(y + i) * gate[rh]);
}

// latent_core: the attention core over the latent pages.  Every head of a row reads the same latent both as
// key and as value (the expansions to per-head keys and values are folded into the matrices around the core),
// so a block takes one row, stages the row's visible latents tile by tile (32 keys, float32) in shared memory
// once for all heads, and each warp runs the online softmax of its heads over the tile: a lane per key for the
// scores, a lane per column for the weighted sum.  Scores, weights and sums are float32; keys are walked in
// ascending order from the window's first key, so a row's result does not depend on the cut or the batch.
// The head's gate multiplies the result before it is stored.
#define LC_TILE 32
#define LC_MAX_J 8       // columns per lane: rank <= 256
#define LC_VPT 8         // 16-byte vectors a thread fetches per tile: 32 keys x 256 float32 columns / 256 threads

template <typename T, int HPW, int NJ>
__global__ void __launch_bounds__(512)
latent_core_kernel(const T* __restrict__ q, const T* __restrict__ pages, const int* __restrict__ table, int table_stride,
                   const int* __restrict__ positions, const int* __restrict__ row_entry, const float* __restrict__ gate,
                   T* __restrict__ out, int nH, int rp, int page_size, int num_pages, int window, float scale,
                   int n_splits, float* __restrict__ partial) {
    extern __shared__ float sm[];
    const int ldt = rp + 1;
    float* Ts = sm;                        // [LC_TILE][rp+1]
    float* qs = sm + LC_TILE * ldt;        // [nH][rp], scaled
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int entry = row_entry[row];
    T* orow = out + (size_t)row * nH * rp;
    if (entry < 0) {
        for (int i = tid; i < nH * rp; i += blockDim.x) ng_st(orow + i, 0.f);
        return;
    }
    const int pos_row = positions[row];
    const int lo_row = window > 0 ? max(0, pos_row - window + 1) : 0;
    // with n_splits > 1 the row's tiles are dealt to n_splits blocks in runs; each leaves its running maximum, sum
    // and weighted sum in `partial` and a second kernel merges the runs in ascending order
    const int tiles = (pos_row - lo_row + LC_TILE) / LC_TILE;
    const int per = (tiles + n_splits - 1) / n_splits;
    const int lo = lo_row + (int)blockIdx.y * per * LC_TILE;
    const int pos = min(pos_row, lo + per * LC_TILE - 1);          // lo > pos: this block has no keys
    const int* trow = table + (size_t)entry * table_stride;
    for (int i = tid; i < nH * rp; i += blockDim.x) qs[i] = ng_ld(q + (size_t)row * nH * rp + i) * scale;
    float m[HPW], l[HPW], acc[HPW][NJ];
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        m[u] = -INFINITY;
        l[u] = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j) acc[u][j] = 0.f;
    }
    // Tiles are fetched 16 bytes a thread and load, a tile ahead: the loads of tile t+1 are in flight while the
    // warps work on tile t.  LC_VPT vectors a thread cover 32 keys of up to 256 columns at 256 threads and more.
    constexpr int VEC = 16 / (int)sizeof(T);
    const int vec_per_key = rp / VEC;                       // rp is a multiple of 16
    uint4 pre[LC_VPT];
    auto fetch = [&](int k0) {
        const int n = min(LC_TILE, pos + 1 - k0);
#pragma unroll
        for (int v = 0; v < LC_VPT; ++v) {
            const int idx = tid + v * blockDim.x;
            pre[v] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < n * vec_per_key) {
                const int kp = k0 + idx / vec_per_key;
                const int page = trow[kp / page_size];
                if (page >= 0 && page < num_pages)
                    pre[v] = *reinterpret_cast<const uint4*>(pages + ((size_t)page * page_size + (kp % page_size)) * rp
                                                             + (size_t)(idx % vec_per_key) * VEC);
            }
        }
    };
    if (lo <= pos) fetch(lo);
    for (int k0 = lo; k0 <= pos; k0 += LC_TILE) {
        const int n = min(LC_TILE, pos + 1 - k0);
        __syncthreads();
#pragma unroll
        for (int v = 0; v < LC_VPT; ++v) {
            const int idx = tid + v * blockDim.x;
            if (idx < n * vec_per_key) {
                const T* e = reinterpret_cast<const T*>(&pre[v]);
                float* dst = Ts + (idx / vec_per_key) * ldt + (idx % vec_per_key) * VEC;
#pragma unroll
                for (int c = 0; c < VEC; ++c) dst[c] = ng_ld(e + c);
            }
        }
        if (k0 + LC_TILE <= pos) fetch(k0 + LC_TILE);
        __syncthreads();
#pragma unroll
        for (int u = 0; u < HPW; ++u) {
            const int head = warp + u * nwarp;
            if (head >= nH) break;
            const float* qh = qs + (size_t)head * rp;
            float s = -INFINITY;
            if (lane < n) {                     // four partial sums: the chain of one would wait on every load
                const float* tk = Ts + lane * ldt;
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll 4
                for (int d = 0; d < rp; d += 4) {
                    const float4 qv = *reinterpret_cast<const float4*>(qh + d);
                    s0 = fmaf(qv.x, tk[d], s0);
                    s1 = fmaf(qv.y, tk[d + 1], s1);
                    s2 = fmaf(qv.z, tk[d + 2], s2);
                    s3 = fmaf(qv.w, tk[d + 3], s3);
                }
                s = (s0 + s1) + (s2 + s3);
            }
            const float m_new = fmaxf(m[u], ng_warp_max(s));
            const float corr = expf(m[u] - m_new);
            const float p = lane < n ? expf(s - m_new) : 0.f;
            l[u] = l[u] * corr + ng_warp_sum(p);
            m[u] = m_new;
#pragma unroll
            for (int j = 0; j < NJ; ++j) acc[u][j] *= corr;
#pragma unroll 4
            for (int k = 0; k < n; ++k) {
                const float pk = __shfl_sync(0xffffffffu, p, k);
                const float* tk = Ts + k * ldt;
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    const int d = lane + 32 * j;
                    if (d < rp) acc[u][j] = fmaf(pk, tk[d], acc[u][j]);
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int head = warp + u * nwarp;
        if (head >= nH) break;
        if (n_splits > 1) {
            float* dst = partial + (((size_t)row * nH + head) * n_splits + blockIdx.y) * (rp + 2);
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int d = lane + 32 * j;
                if (d < rp) dst[d] = acc[u][j];
            }
            if (lane == 0) {
                dst[rp] = m[u];
                dst[rp + 1] = l[u];
            }
            continue;
        }
        const float f = (l[u] > 0.f ? 1.f / l[u] : 0.f) * (gate ? gate[(size_t)row * nH + head] : 1.f);
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int d = lane + 32 * j;
            if (d < rp) ng_st(orow + (size_t)head * rp + d, acc[u][j] * f);
        }
    }
}

// merges the runs of a (row, head) in ascending order: a warp each
template <typename T>
__global__ void latent_merge_kernel(const float* __restrict__ partial, const float* __restrict__ gate,
                                    const int* __restrict__ row_entry, T* __restrict__ out, int n_rows, int nH, int rp,
                                    int n_splits) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= n_rows * nH) return;
    const int row = w / nH;
    if (row_entry[row] < 0) return;                 // the core wrote zeros there
    const float* src = partial + (size_t)w * n_splits * (rp + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, src[(size_t)s * (rp + 2) + rp]);
    float L = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = src[(size_t)s * (rp + 2) + rp];
        if (ms > -INFINITY) L += src[(size_t)s * (rp + 2) + rp + 1] * expf(ms - M);
    }
    const float f = (L > 0.f ? 1.f / L : 0.f) * (gate ? gate[w] : 1.f);
    for (int d = lane; d < rp; d += 32) {
        float a = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = src[(size_t)s * (rp + 2) + rp];
            if (ms > -INFINITY) a += src[(size_t)s * (rp + 2) + d] * expf(ms - M);
        }
        ng_st(out + (size_t)w * rp + d, a * f);
    }
}

// q, out: [n_rows, nH*rp]; pages: [num_pages, 1, page_size, rp]; gate: float32 [n_rows, nH] or null.
// `n_splits` > 1: every row's keys are cut into that many runs, each a block of its own (steps of few rows);
// `partial` then holds n_rows * nH * n_splits * (rp + 2) float32 values.
NG_EXPORT int ng_latent_core(const void* q, const void* pages, const int* table, int table_stride, const int* positions,
                             const int* row_entry, const float* gate, void* out, int n_rows, int nH, int rp, int page_size,
                             int num_pages, int window, float scale, int n_splits, float* partial, int act_bf16,
                             cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (nH <= 0 || rp <= 0 || rp > 32 * LC_MAX_J || page_size <= 0 || nH > 64 || n_splits < 1 || n_splits > 64 ||
        (n_splits > 1 && !partial))
        return NG_BAD_SIZE;
    const int nwarp = nH <= 8 ? 8 : nH <= 16 ? nH : 16;           // at least 256 threads: all of them fetch the tiles
    const int hpw = (nH + nwarp - 1) / nwarp;
    const size_t smem = ((size_t)LC_TILE * (rp + 1) + (size_t)nH * rp) * sizeof(float);
    if (smem > 200 * 1024) return NG_BAD_SIZE;
#define LC_LAUNCH(TT, HH, JJ)                                                                                          \
    {                                                                                                                  \
        static bool configured = false;                                                                                \
        if (!configured) {                                                                                             \
            if (cudaFuncSetAttribute(latent_core_kernel<TT, HH, JJ>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                     200 * 1024) != cudaSuccess)                                                       \
                return NG_LAUNCH_FAILED;                                                                               \
            configured = true;                                                                                         \
        }                                                                                                              \
        NG_LAUNCH((latent_core_kernel<TT, HH, JJ>), dim3(n_rows, n_splits), nwarp * 32, smem, stream, (const TT*)q,   \
                  (const TT*)pages, table, table_stride, positions, row_entry, gate, (TT*)out, nH, rp, page_size,      \
                  num_pages, window, scale, n_splits, partial);                                                        \
    }
    // columns a lane keeps of a head's sum: the smallest of 1, 2, 4, 8 that covers the latent
#define LC_BY_J(TT, HH)                                                                                                \
    {                                                                                                                  \
        if (rp <= 32) LC_LAUNCH(TT, HH, 1) else if (rp <= 64) LC_LAUNCH(TT, HH, 2) else if (rp <= 128) LC_LAUNCH(TT, HH, 4) \
        else LC_LAUNCH(TT, HH, 8)                                                                                      \
    }
    if (act_bf16) {
        if (hpw == 1) LC_BY_J(__nv_bfloat16, 1) else if (hpw == 2) LC_BY_J(__nv_bfloat16, 2) else LC_BY_J(__nv_bfloat16, 4)
    } else {
        if (hpw == 1) LC_BY_J(float, 1) else if (hpw == 2) LC_BY_J(float, 2) else LC_BY_J(float, 4)
    }
    if (n_splits > 1) {
        const unsigned blocks = (unsigned)(((size_t)n_rows * nH + 7) / 8);
        if (act_bf16)
            NG_LAUNCH((latent_merge_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (const float*)partial, gate, row_entry,
                      (__nv_bfloat16*)out, n_rows, nH, rp, n_splits);
        else
            NG_LAUNCH((latent_merge_kernel<float>), blocks, 256, 0, stream, (const float*)partial, gate, row_entry,
                      (float*)out, n_rows, nH, rp, n_splits);
    }
    return ng_launch_status();
}

NG_EXPORT int ng_latent_prep(const void* x, const float* wq, const float* wkv, void* cq_out, void* pages,
                             float* gate_out, const int* table, int table_stride, const int* positions,
                             const int* row_entry, int n_rows, int rq, int rkv, int rp, int nH, int page_size,
                             int num_pages, float eps, int* status, int rot, const float* inv_freq, int half_pairing,
                             int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (rq <= 0 || rkv < 0 || rot < 0 || (rot & 1) || (rot && !inv_freq) || (rkv == 0 && rot) || rp < rkv + rot || nH <= 0 ||
        page_size <= 0 || (rkv > 0 && !pages))
        return NG_BAD_SIZE;
    if (act_bf16)
        NG_LAUNCH((latent_prep_kernel<__nv_bfloat16>), n_rows, 128, 0, stream, (const __nv_bfloat16*)x, wq, wkv,
                  (__nv_bfloat16*)cq_out, (__nv_bfloat16*)pages, gate_out, table, table_stride, positions, row_entry,
                  rq, rkv, rp, nH, page_size, num_pages, eps, status, rot, inv_freq, half_pairing);
    else
        NG_LAUNCH((latent_prep_kernel<float>), n_rows, 128, 0, stream, (const float*)x, wq, wkv, (float*)cq_out,
                  (float*)pages, gate_out, table, table_stride, positions, row_entry, rq, rkv, rp, nH, page_size,
                  num_pages, eps, status, rot, inv_freq, half_pairing);
    return ng_launch_status();
}

NG_EXPORT int ng_latent_rope_q(void* q, const int* positions, const int* row_entry, const float* inv_freq, int n_rows,
                               int nH, int rp, int off, int rot, int half_pairing, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0 || rot == 0) return NG_OK;
    if (nH <= 0 || rp <= 0 || off < 0 || rot < 0 || (rot & 1) || off + rot > rp || !inv_freq) return NG_BAD_SIZE;
    if (act_bf16)
        NG_LAUNCH((latent_rope_q_kernel<__nv_bfloat16>), n_rows, 128, 0, stream, (__nv_bfloat16*)q, positions, row_entry,
                  inv_freq, nH, rp, off, rot, half_pairing);
    else
        NG_LAUNCH((latent_rope_q_kernel<float>), n_rows, 128, 0, stream, (float*)q, positions, row_entry, inv_freq, nH, rp,
                  off, rot, half_pairing);
    return ng_launch_status();
}

// o [n_rows, nH * rp] (the first `rank` columns of a head are read), w [nH, dv, rank], gate float32 [n_rows, nH * dv] or
// null, out rows `ldo` elements apart (a block of columns of a wider buffer).
NG_EXPORT int ng_head_up_gate(const void* o, const void* w, const float* gate, void* out, int n_rows, int nH, int rp,
                              int rank, int dv, int ldo, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (nH <= 0 || nH > 65535 || rank <= 0 || rank > rp || dv <= 0 || ldo < nH * dv) return NG_BAD_SIZE;
    const size_t smem = (size_t)HU_ROWS * rank * sizeof(float);
    if (smem > 160 * 1024) return NG_BAD_SIZE;
    const int tiles = (n_rows + HU_ROWS - 1) / HU_ROWS;
    const int slices = tiles * nH >= 256 ? 1 : max(1, min((dv + 7) / 8, 256 / (tiles * nH)));
    dim3 grid(tiles, nH, slices);
#define HU_LAUNCH(TT)                                                                                                  \
    {                                                                                                                  \
        static bool configured = false;                                                                                \
        if (!configured) {                                                                                             \
            if (cudaFuncSetAttribute(head_up_gate_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) \
                != cudaSuccess)                                                                                        \
                return NG_LAUNCH_FAILED;                                                                               \
            configured = true;                                                                                         \
        }                                                                                                              \
        NG_LAUNCH((head_up_gate_kernel<TT>), grid, 256, smem, stream, (const TT*)o, (const TT*)w, gate, (TT*)out,      \
                  n_rows, nH, rp, rank, dv, ldo);                                                                      \
    }
    if (act_bf16) HU_LAUNCH(__nv_bfloat16) else HU_LAUNCH(float)
    return ng_launch_status();
}

NG_EXPORT int ng_head_gate(void* y, const float* gate, int n_rows, int nH, int width, int act_bf16,
                           cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (nH <= 0 || width <= 0) return NG_BAD_SIZE;
    const size_t total = (size_t)n_rows * nH * width;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_bf16)
        NG_LAUNCH((head_gate_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (__nv_bfloat16*)y, gate, total, nH, width);
    else
        NG_LAUNCH((head_gate_kernel<float>), blocks, 256, 0, stream, (float*)y, gate, total, nH, width);
    return ng_launch_status();
}
