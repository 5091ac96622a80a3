// Attention whose softmax weights stay float32, over paged keys and values of different sizes, with one or two
// score maps per head, a sliding window that keeps the first tokens, and a soft cap on the scores.
//
//   q     [N, nH * M * d]          M maps per head laid out head by head as [map 0, map 1]
//   keys  [pages, nG * M, page, d] values [pages, nG, page, dv]        query head h reads group h / (nH / nG)
//   s_m(j) = cap(scale * q_m . k_m,j)        cap(s) = softcap * tanh(s / softcap), or s when softcap == 0
//   a_m    = softmax_j(s_m) v_j  over the visible j: j <= pos and (pos - j < window or j < keep_first);
//            window 0 = every j <= pos; with `chunk` > 0 also floor(j / chunk) = floor(pos / chunk)
//   M == 1: o = a_0                          M == 2: o = a_0 - lambda * a_1
//   slopes (per head, optional): slope_h * (pos - j) is taken off s(j) after the cap
//   sinks (per head, optional): the softmax's denominator also holds exp(sink_h), a term without key or value
//   head_norm: o <- o * rsqrt(mean(o^2) + eps) * post_scale  over the head's dv values
//
// Two kernels.  ``qkv_prep``: per-head RMS norm of q and k (one weight vector shared by heads and maps; or, `whole`,
// one norm over all of a row's q and one over all of its k, with weights of that length), q times a temperature
// 1 + coef * ln(floor((pos + 1) / every) + 1), rotation of the first rot_dims coordinates of every map in pairs (2i, 2i+1), q to its buffer, k and v into
// their pages.  ``mapped_attention``: a block per (row, query head, run of keys); a warp takes 32 keys of a
// 128-key tile with a lane per key for the scores of both maps (the key's row read in 16-byte pieces, q from
// shared memory), keeps an online softmax per map in float32 and adds the weighted values with a lane per pair
// of value columns; the warps' states are merged in warp order, the runs (few-row steps cut a row's keys into
// several) by a second kernel.  Everything after the loads is float32; the two maps share every value load.
#include "ng_common.cuh"

#define MA_THREADS 128
#define MA_WARPS 4
#define MA_TILE (32 * MA_WARPS)
#define MA_DVU 4          // value columns per lane: 2 * MA_DVU, so dv <= 256
#define MA_MAX_PAIRS 8    // pairs of a head per lane in the prep kernel: d <= 512

// ------------------------------------------------------------------------------------------ prep
template <typename T>
__global__ void __launch_bounds__(MA_THREADS)
qkv_prep_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ qw,
                const float* __restrict__ kw, const float* __restrict__ inv_freq, int rot_dims,
                T* __restrict__ k_pages, T* __restrict__ v_pages, const int* __restrict__ table, int table_stride,
                const int* __restrict__ positions, const int* __restrict__ row_entry, int nQ, int nK, int nV, int d,
                int dv, int page_size, int num_pages, float eps, int* __restrict__ status, int whole, float temp_coef,
                int temp_every, int ld, int half_pairing, int unit_norm) {
    extern __shared__ float rot[];                      // cos[rot_dims/2], sin[rot_dims/2]
    __shared__ float red[32];
    ng_pdl_trigger();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int entry = row_entry[row];
    const int pos = positions[row];
    const int half_rot = rot_dims / 2;
    for (int i = threadIdx.x; i < half_rot; i += MA_THREADS) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        rot[i] = c;
        rot[half_rot + i] = s;
    }
    __syncthreads();
    ng_pdl_wait();
    qkv = ng_after_wait(qkv);
    const T* in = qkv + (size_t)row * ld;             // ld: a row's pitch (columns behind v belong to the caller)
    T* qo = q_out + (size_t)row * nQ * d;
    if (entry < 0) {                                   // padding row: defined output, no cache write
        for (int j = blockIdx.y * MA_THREADS + threadIdx.x; j < nQ * d; j += MA_THREADS * gridDim.y) ng_st(qo + j, 0.f);
        return;
    }
    size_t k_base = 0, v_base = 0;
    bool page_ok = true;
    if (nK + nV > 0) {
        const int page = table[(size_t)entry * table_stride + pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        if (!page_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, NG_STATUS_BAD_PAGE);
        const size_t p = page_ok ? page : 0, slot = pos % page_size;
        k_base = (p * nK * page_size + slot) * d;
        v_base = (p * nV * page_size + slot) * dv;
    }
    const int half = d / 2;
    // one norm over all of the row's q and one over all of its k: every block of the row forms both sums itself
    float r_q = 1.f, r_k = 1.f;
    if (whole) {
        float sq = 0.f, sk = 0.f;
        for (int j = threadIdx.x; j < nQ * d; j += MA_THREADS) { const float t = ng_ld(in + j); sq = fmaf(t, t, sq); }
        for (int j = threadIdx.x; j < nK * d; j += MA_THREADS) { const float t = ng_ld(in + (size_t)nQ * d + j); sk = fmaf(t, t, sk); }
        sq = ng_block_sum(sq, red);
        sk = ng_block_sum(sk, red);
        r_q = rsqrtf(sq / (float)(nQ * d) + eps);
        if (nK > 0) r_k = rsqrtf(sk / (float)(nK * d) + eps);
    }
    const float temp = temp_coef != 0.f ? 1.f + temp_coef * logf((float)((pos + 1) / temp_every + 1)) : 1.f;
    // few rows: the heads are dealt over gridDim.y blocks of a row; many rows: one block walks all heads of its row
    for (int hh = blockIdx.y * MA_WARPS + warp; hh < nQ + nK; hh += MA_WARPS * gridDim.y) {
        const bool is_q = hh < nQ;
        if (!is_q && !page_ok) continue;
        const T* src = in + (size_t)hh * d;
        const float* w = is_q ? qw : kw;
        if (w && whole) w += (size_t)(is_q ? hh : hh - nQ) * d;        // a weight per coordinate of the projection
        const float post = is_q ? temp : 1.f;
        float x1[MA_MAX_PAIRS], x2[MA_MAX_PAIRS];
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < MA_MAX_PAIRS; ++u) {
            const int i = lane + 32 * u;
            x1[u] = x2[u] = 0.f;
            if (i < half) {
                // pair i: (2i, 2i+1), or with half pairing (i, i + rot_dims/2) inside the rotated coordinates
                const bool hp = half_pairing && i < half_rot;
                x1[u] = ng_ld(src + (hp ? i : 2 * i));
                x2[u] = ng_ld(src + (hp ? i + half_rot : 2 * i + 1));
            }
            ss += x1[u] * x1[u] + x2[u] * x2[u];
        }
        if ((d & 1) && lane == 0) {                     // an odd last coordinate has no partner
            const float t = ng_ld(src + d - 1);
            ss += t * t;
        }
        float r = 1.f;
        if (w) r = whole ? (is_q ? r_q : r_k) : rsqrtf(ng_warp_sum(ss) / (float)d + eps);
        // a norm without weights: a rotation does not change a head's sum of squares, so the factor of the
        // unrotated head is the factor of the rotated one
        else if (unit_norm) r = rsqrtf(ng_warp_sum(ss) / (float)d + eps);
        T* dst = is_q ? qo + (size_t)hh * d : k_pages + k_base + (size_t)(hh - nQ) * page_size * d;
#pragma unroll
        for (int u = 0; u < MA_MAX_PAIRS; ++u) {
            const int i = lane + 32 * u;
            if (i < half) {
                const bool hp = half_pairing && i < half_rot;
                const int c1 = hp ? i : 2 * i, c2 = hp ? i + half_rot : 2 * i + 1;
                float y1 = x1[u], y2 = x2[u];
                if (w) { y1 = y1 * r * w[c1]; y2 = y2 * r * w[c2]; }
                else if (unit_norm) { y1 *= r; y2 *= r; }
                y1 *= post; y2 *= post;
                if (i < half_rot) {
                    const float c = rot[i], s = rot[half_rot + i];
                    const float z1 = y1 * c - y2 * s, z2 = y2 * c + y1 * s;
                    y1 = z1; y2 = z2;
                }
                ng_st(dst + c1, y1);
                ng_st(dst + c2, y2);
            }
        }
        if ((d & 1) && lane == 0) {
            float t = ng_ld(src + d - 1);
            if (w) t = t * r * w[d - 1];
            else if (unit_norm) t *= r;
            ng_st(dst + d - 1, t * post);
        }
    }
    if (page_ok) {
        const T* vs = in + (size_t)(nQ + nK) * d;
        for (int j = blockIdx.y * MA_THREADS + threadIdx.x; j < nV * dv; j += MA_THREADS * gridDim.y) {
            const int hv = j / dv, c = j - hv * dv;
            v_pages[v_base + (size_t)hv * page_size * dv + c] = vs[j];
        }
    }
}

NG_EXPORT int ng_qkv_prep(const void* qkv, void* q_out, const float* qw, const float* kw, const float* inv_freq,
                          int rot_dims, void* k_pages, void* v_pages, const int* table, int table_stride,
                          const int* positions, const int* row_entry, int n_rows, int nQ, int nK, int nV, int d, int dv,
                          int page_size, int num_pages, float eps, int* status, int whole, float temp_coef, int temp_every,
                          int ld, int half_pairing, int unit_norm, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (temp_every < 1 || (whole && (!qw || (nK > 0 && !kw)))) return NG_BAD_SIZE;
    if (ld < (nQ + nK) * d + nV * dv || (unit_norm && (whole || qw || kw))) return NG_BAD_SIZE;
    if (d <= 0 || d > 64 * MA_MAX_PAIRS || dv <= 0 || nQ <= 0 || nK < 0 || nV < 0 || page_size <= 0 || rot_dims < 0 ||
        rot_dims > d || (rot_dims & 1) || (rot_dims > 0 && !inv_freq))
        return NG_BAD_SIZE;
    const size_t smem = (size_t)rot_dims * sizeof(float);
    const int head_blocks = n_rows >= 256 ? 1 : min(64, (nQ + nK + MA_WARPS - 1) / MA_WARPS);
    const dim3 grid(n_rows, head_blocks);
    if (act_bf16)
        NG_LAUNCH((qkv_prep_kernel<__nv_bfloat16>), grid, MA_THREADS, smem, stream, (const __nv_bfloat16*)qkv,
                  (__nv_bfloat16*)q_out, qw, kw, inv_freq, rot_dims, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, table,
                  table_stride, positions, row_entry, nQ, nK, nV, d, dv, page_size, num_pages, eps, status, whole, temp_coef,
                  temp_every, ld, half_pairing, unit_norm);
    else
        NG_LAUNCH((qkv_prep_kernel<float>), grid, MA_THREADS, smem, stream, (const float*)qkv, (float*)q_out, qw, kw,
                  inv_freq, rot_dims, (float*)k_pages, (float*)v_pages, table, table_stride, positions, row_entry, nQ, nK, nV,
                  d, dv, page_size, num_pages, eps, status, whole, temp_coef, temp_every, ld, half_pairing, unit_norm);
    return ng_launch_status();
}

// ------------------------------------------------------------------------------------------ core
struct MaParams {
    const void* q; const void* k_pages; const void* v_pages; const int* table; int table_stride;
    const int* positions; const int* row_entry; void* out; int out_ld; float* partial;
    int nH, nG, d, dv, page_size, num_pages, window, keep_first, n_splits, chunk;
    float scale, softcap, lambda, post_scale, eps; int head_norm;
    const float* slopes; const float* sinks;            // per head, or null
};

// the two bfloat16 values of a 32-bit word as float32: a bfloat16 is the upper half of a float32, so a shift and a
// mask do it on the integer units (no conversion instruction)
__device__ __forceinline__ float ma_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float ma_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// dot of a key's row with q (shared memory, float32): 16-byte pieces when the row allows it
__device__ __forceinline__ float ma_dot(const __nv_bfloat16* k, const float* q, int d, bool vec) {
    float s = 0.f;
    if (vec) {
#pragma unroll 4
        for (int c = 0; c < d; c += 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(k + c);
            const float4 qa = *reinterpret_cast<const float4*>(q + c), qb = *reinterpret_cast<const float4*>(q + c + 4);
            s = fmaf(qa.x, ma_lo(u.x), s); s = fmaf(qa.y, ma_hi(u.x), s);
            s = fmaf(qa.z, ma_lo(u.y), s); s = fmaf(qa.w, ma_hi(u.y), s);
            s = fmaf(qb.x, ma_lo(u.z), s); s = fmaf(qb.y, ma_hi(u.z), s);
            s = fmaf(qb.z, ma_lo(u.w), s); s = fmaf(qb.w, ma_hi(u.w), s);
        }
    } else {
        for (int c = 0; c < d; ++c) s = fmaf(q[c], __bfloat162float(k[c]), s);
    }
    return s;
}
__device__ __forceinline__ float ma_dot(const float* k, const float* q, int d, bool vec) {
    float s = 0.f;
    if (vec) {
#pragma unroll 4
        for (int c = 0; c < d; c += 4) {
            const float4 u = *reinterpret_cast<const float4*>(k + c), qa = *reinterpret_cast<const float4*>(q + c);
            s = fmaf(qa.x, u.x, s); s = fmaf(qa.y, u.y, s); s = fmaf(qa.z, u.z, s); s = fmaf(qa.w, u.w, s);
        }
    } else {
        for (int c = 0; c < d; ++c) s = fmaf(q[c], k[c], s);
    }
    return s;
}
__device__ __forceinline__ float2 ma_ld_pair(const __nv_bfloat16* v, int c, int dv, bool vec) {
    if (vec) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(v + c);
        return make_float2(ma_lo(w), ma_hi(w));
    }
    return make_float2(c < dv ? __bfloat162float(v[c]) : 0.f, c + 1 < dv ? __bfloat162float(v[c + 1]) : 0.f);
}
__device__ __forceinline__ float2 ma_ld_pair(const float* v, int c, int dv, bool vec) {
    if (vec) return *reinterpret_cast<const float2*>(v + c);
    return make_float2(c < dv ? v[c] : 0.f, c + 1 < dv ? v[c + 1] : 0.f);
}

// the last step for one (row, head): maps combined, the head over its root mean square; `a` holds per map the sums
// sum_j p_j v_j,c (not yet divided by `l`), for the columns c = threadIdx.x, + MA_THREADS, ...
template <typename T, int M>
__device__ __forceinline__ void ma_finish(const MaParams& p, T* o, const float* acc /*[M][dv]*/, const float* l,
                                          float* red) {
    float inv[M];
#pragma unroll
    for (int m = 0; m < M; ++m) inv[m] = l[m] > 0.f ? 1.f / l[m] : 0.f;
    float ss = 0.f;
    float keep[(2 * MA_DVU * 32 + MA_THREADS - 1) / MA_THREADS];
    int n = 0;
    for (int c = threadIdx.x; c < p.dv; c += MA_THREADS, ++n) {
        float v = acc[c] * inv[0];
        if (M == 2) v -= p.lambda * (acc[p.dv + c] * inv[1]);
        keep[n] = v;
        ss += v * v;
    }
    float r = 1.f;
    if (p.head_norm) r = rsqrtf(ng_block_sum(ss, red) / (float)p.dv + p.eps) * p.post_scale;
    n = 0;
    for (int c = threadIdx.x; c < p.dv; c += MA_THREADS, ++n) ng_st(o + c, keep[n] * r);
}

// DVU: pairs of value columns a lane holds (dv <= 64 * DVU): registers and work follow the head's real size
template <typename T, int M, int DVU>
__global__ void __launch_bounds__(MA_THREADS)
mapped_attention_kernel(const MaParams p) {
    extern __shared__ float sm[];
    __shared__ float red[32];
    __shared__ float st_m[MA_WARPS][M], st_l[MA_WARPS][M], fin_l[M];
    float* q_s = sm;                                    // [M][d4], d4 = d rounded up to 4: every map 16-byte aligned
    const int d4 = (p.d + 3) & ~3;
    float* acc_s = sm + M * d4;                        // [MA_WARPS][M][dv], later [M][dv] merged in place of warp 0
    ng_pdl_trigger();
    const int row = blockIdx.x, head = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int d = p.d, dv = p.dv;
    const int entry = p.row_entry[row];
    const int pos = p.positions[row];
    T* o = reinterpret_cast<T*>(p.out) + (size_t)row * p.out_ld + (size_t)head * dv;
    float* part = p.partial ? p.partial + (((size_t)row * p.nH + head) * p.n_splits + split) * M * (dv + 2) : nullptr;
    ng_pdl_wait();
    if (entry < 0) {
        if (!part) { for (int c = threadIdx.x; c < dv; c += MA_THREADS) ng_st(o + c, 0.f); }
        else { for (int c = threadIdx.x; c < M * (dv + 2); c += MA_THREADS) part[c] = (c % (dv + 2)) == 0 ? -INFINITY : 0.f; }
        return;
    }
    const T* q = reinterpret_cast<const T*>(ng_after_wait(p.q)) + ((size_t)row * p.nH + head) * M * d;
    for (int c = threadIdx.x; c < M * d; c += MA_THREADS) q_s[(c / d) * d4 + (c % d)] = ng_ld(q + c);
    __syncthreads();
    const int g = head / (p.nH / p.nG);
    const float slope = p.slopes ? p.slopes[head] : 0.f;
    int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    if (p.chunk > 0) lo = max(lo, (pos / p.chunk) * p.chunk);      // chunks count from the sequence's position 0
    const int n_sink = min(p.keep_first, lo);
    const int n_keys = n_sink + (pos - lo + 1);          // logical key t: position t (t < n_sink) or lo + t - n_sink
    int t0 = 0, t1 = n_keys;
    if (p.n_splits > 1) {
        const int tiles = (n_keys + MA_TILE - 1) / MA_TILE, per = (tiles + p.n_splits - 1) / p.n_splits;
        t0 = min(n_keys, split * per * MA_TILE);
        t1 = min(n_keys, t0 + per * MA_TILE);
    }
    const T* kp = reinterpret_cast<const T*>(p.k_pages);
    const T* vp = reinterpret_cast<const T*>(p.v_pages);
    const int* trow = p.table + (size_t)entry * p.table_stride;
    const bool kvec = sizeof(T) == 2 ? (d % 8 == 0 && ((uintptr_t)kp & 15) == 0) : (d % 4 == 0 && ((uintptr_t)kp & 15) == 0);
    const bool vvec = (dv % 2 == 0) && ((uintptr_t)vp & (2 * sizeof(T) - 1)) == 0;
    float m_run[M], l_run[M], acc[M][DVU][2];
#pragma unroll
    for (int m = 0; m < M; ++m) {
        m_run[m] = -INFINITY; l_run[m] = 0.f;
#pragma unroll
        for (int u = 0; u < DVU; ++u) acc[m][u][0] = acc[m][u][1] = 0.f;
    }
    for (int tb = t0 + warp * 32; tb < t1; tb += MA_TILE) {
        const int t = tb + lane;
        const bool valid = t < t1;
        const int kpos = valid ? (t < n_sink ? t : lo + (t - n_sink)) : pos;
        const int page = trow[kpos / p.page_size];
        const bool ok = valid && page >= 0 && page < p.num_pages;
        const size_t slot = kpos % p.page_size, pg = ok ? page : 0;
        const size_t vbase = ((pg * p.nG + g) * p.page_size + slot) * dv;
        float pr[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
            const size_t kbase = ((pg * p.nG * M + g * M + m) * p.page_size + slot) * d;
            float s = -INFINITY;
            if (ok) {
                s = ma_dot(kp + kbase, q_s + m * d4, d, kvec) * p.scale;
                if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
                s -= slope * (float)(pos - kpos);
            }
            const float m_new = fmaxf(m_run[m], ng_warp_max(s));
            const float corr = m_run[m] == -INFINITY ? 0.f : expf(m_run[m] - m_new);
            pr[m] = ok ? expf(s - m_new) : 0.f;
            l_run[m] = l_run[m] * corr + ng_warp_sum(pr[m]);
            m_run[m] = m_new;
#pragma unroll
            for (int u = 0; u < DVU; ++u) { acc[m][u][0] *= corr; acc[m][u][1] *= corr; }
        }
        // eight keys at a time, their values requested before the first is used; a lane beyond the run's end has the
        // weight 0 and the address of a key that is there (the row's own), so nothing is skipped inside a group
        const int cnt = min(32, t1 - tb);
        for (int j0 = 0; j0 < cnt; j0 += 8) {
            float2 vv[8][DVU];
            float pj[8][M];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const size_t vb = __shfl_sync(0xffffffffu, vbase, j0 + jj);
#pragma unroll
                for (int m = 0; m < M; ++m) pj[jj][m] = __shfl_sync(0xffffffffu, pr[m], j0 + jj);
#pragma unroll
                for (int u = 0; u < DVU; ++u) {
                    const int c = 2 * lane + 64 * u;
                    vv[jj][u] = c < dv ? ma_ld_pair(vp + vb, c, dv, vvec) : make_float2(0.f, 0.f);
                }
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
#pragma unroll
                for (int u = 0; u < DVU; ++u)
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        acc[m][u][0] = fmaf(pj[jj][m], vv[jj][u].x, acc[m][u][0]);
                        acc[m][u][1] = fmaf(pj[jj][m], vv[jj][u].y, acc[m][u][1]);
                    }
        }
    }
    // the warps' states, merged in warp order
#pragma unroll
    for (int m = 0; m < M; ++m) {
        if (lane == 0) { st_m[warp][m] = m_run[m]; st_l[warp][m] = l_run[m]; }
#pragma unroll
        for (int u = 0; u < DVU; ++u) {
            const int c = 2 * lane + 64 * u;
            if (c < dv) acc_s[((size_t)warp * M + m) * dv + c] = acc[m][u][0];
            if (c + 1 < dv) acc_s[((size_t)warp * M + m) * dv + c + 1] = acc[m][u][1];
        }
    }
    __syncthreads();
    float mt[M], f[M][MA_WARPS];
#pragma unroll
    for (int m = 0; m < M; ++m) {
        mt[m] = -INFINITY;
#pragma unroll
        for (int w = 0; w < MA_WARPS; ++w) mt[m] = fmaxf(mt[m], st_m[w][m]);
        float lt = 0.f;
#pragma unroll
        for (int w = 0; w < MA_WARPS; ++w) {
            f[m][w] = st_m[w][m] == -INFINITY ? 0.f : expf(st_m[w][m] - mt[m]);
            lt += st_l[w][m] * f[m][w];
        }
        if (threadIdx.x == 0) fin_l[m] = lt;
    }
    float merged[M][(2 * DVU * 32 + MA_THREADS - 1) / MA_THREADS];
    {
        int n = 0;
        for (int c = threadIdx.x; c < dv; c += MA_THREADS, ++n)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float a = 0.f;
#pragma unroll
                for (int w = 0; w < MA_WARPS; ++w) a += acc_s[((size_t)w * M + m) * dv + c] * f[m][w];
                merged[m][n] = a;
            }
    }
    __syncthreads();
    if (part) {                                         // one run of several: (max, sum, weighted values) per map
        int n = 0;
        for (int c = threadIdx.x; c < dv; c += MA_THREADS, ++n)
#pragma unroll
            for (int m = 0; m < M; ++m) part[(size_t)m * (dv + 2) + 2 + c] = merged[m][n];
        if (threadIdx.x == 0) {
#pragma unroll
            for (int m = 0; m < M; ++m) { part[(size_t)m * (dv + 2)] = mt[m]; part[(size_t)m * (dv + 2) + 1] = fin_l[m]; }
        }
        return;
    }
    {
        int n = 0;
        for (int c = threadIdx.x; c < dv; c += MA_THREADS, ++n)
#pragma unroll
            for (int m = 0; m < M; ++m) acc_s[(size_t)m * dv + c] = merged[m][n];
    }
    __syncthreads();
    float lf[M];
#pragma unroll
    for (int m = 0; m < M; ++m) lf[m] = fin_l[m] + (p.sinks ? expf(p.sinks[head] - mt[m]) : 0.f);
    ma_finish<T, M>(p, o, acc_s, lf, red);
}

// the runs of a (row, head) merged in run order, then the same last step
template <typename T, int M>
__global__ void __launch_bounds__(MA_THREADS)
mapped_attention_merge_kernel(const MaParams p) {
    extern __shared__ float sm[];                       // [M][dv]
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y;
    const int dv = p.dv;
    T* o = reinterpret_cast<T*>(p.out) + (size_t)row * p.out_ld + (size_t)head * dv;
    if (p.row_entry[row] < 0) {
        for (int c = threadIdx.x; c < dv; c += MA_THREADS) ng_st(o + c, 0.f);
        return;
    }
    const float* part = ng_after_wait(p.partial) + ((size_t)row * p.nH + head) * p.n_splits * M * (dv + 2);
    float lf[M];
#pragma unroll
    for (int m = 0; m < M; ++m) {
        float mt = -INFINITY;
        for (int s = 0; s < p.n_splits; ++s) mt = fmaxf(mt, part[((size_t)s * M + m) * (dv + 2)]);
        float lt = 0.f;
        for (int s = 0; s < p.n_splits; ++s) {
            const float* ps = part + ((size_t)s * M + m) * (dv + 2);
            const float f = ps[0] == -INFINITY ? 0.f : expf(ps[0] - mt);
            lt += ps[1] * f;
        }
        lf[m] = lt + (p.sinks ? expf(p.sinks[head] - mt) : 0.f);
        for (int c = threadIdx.x; c < dv; c += MA_THREADS) {
            float a = 0.f;
            for (int s = 0; s < p.n_splits; ++s) {
                const float* ps = part + ((size_t)s * M + m) * (dv + 2);
                const float f = ps[0] == -INFINITY ? 0.f : expf(ps[0] - mt);
                a += ps[2 + c] * f;
            }
            sm[(size_t)m * dv + c] = a;
        }
    }
    __syncthreads();
    ma_finish<T, M>(p, o, sm, lf, red);
}

template <typename T, int M>
static int ma_launch(const MaParams& p, int n_rows, cudaStream_t stream) {
    const size_t smem = ((size_t)M * ((p.d + 3) & ~3) + (size_t)MA_WARPS * M * p.dv) * sizeof(float);
    if (smem > 48 * 1024) return NG_BAD_SIZE;
    dim3 grid(n_rows, p.nH, p.n_splits);
    if (p.dv <= 64) NG_LAUNCH((mapped_attention_kernel<T, M, 1>), grid, MA_THREADS, smem, stream, p);
    else if (p.dv <= 128) NG_LAUNCH((mapped_attention_kernel<T, M, 2>), grid, MA_THREADS, smem, stream, p);
    else NG_LAUNCH((mapped_attention_kernel<T, M, 4>), grid, MA_THREADS, smem, stream, p);
    if (p.n_splits > 1) {
        dim3 g2(n_rows, p.nH);
        NG_LAUNCH((mapped_attention_merge_kernel<T, M>), g2, MA_THREADS, (size_t)M * p.dv * sizeof(float), stream, p);
    }
    return ng_launch_status();
}

// partial: float32 [n_rows, nH, n_splits, n_maps, dv + 2] when n_splits > 1
NG_EXPORT int ng_mapped_attention(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                  int table_stride, const int* positions, const int* row_entry, void* out, int out_ld,
                                  float* partial, int n_rows, int nH, int nG, int n_maps, int d, int dv, int page_size,
                                  int num_pages, int window, int keep_first, int n_splits, float scale, float softcap,
                                  float lambda, float post_scale, float eps, int head_norm, const float* slopes,
                                  const float* sinks, int chunk, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (d <= 0 || dv <= 0 || dv > 64 * MA_DVU || nH <= 0 || nG <= 0 || nH % nG || page_size <= 0 || n_maps < 1 ||
        n_maps > 2 || n_splits < 1 || n_splits > 65535 || nH > 65535 || (n_splits > 1 && !partial) || out_ld < nH * dv ||
        window < 0 || keep_first < 0 || chunk < 0 || (chunk > 0 && keep_first > 0))
        return NG_BAD_SIZE;
    MaParams p{q, k_pages, v_pages, table, table_stride, positions, row_entry, out, out_ld, n_splits > 1 ? partial : nullptr,
               nH, nG, d, dv, page_size, num_pages, window, keep_first, n_splits, chunk, scale, softcap, lambda, post_scale, eps,
               head_norm, slopes, sinks};
    if (act_bf16) return n_maps == 2 ? ma_launch<__nv_bfloat16, 2>(p, n_rows, stream) : ma_launch<__nv_bfloat16, 1>(p, n_rows, stream);
    return n_maps == 2 ? ma_launch<float, 2>(p, n_rows, stream) : ma_launch<float, 1>(p, n_rows, stream);
}

// The runs' states of every (row, head) merged and the heads finished (maps combined, head norm), for states that another
// kernel left in `partial` (float32 [n_rows, nH, n_splits, n_maps, dv + 2]: maximum, sum, weighted values).  Rows of no
// entry get zeros.  `sinks` (per head, or null) adds exp(sink) to every head's sum.
NG_EXPORT int ng_mapped_attention_merge(float* partial, const int* row_entry, void* out, int out_ld, int n_rows, int nH,
                                        int n_maps, int dv, int n_splits, float lambda, float post_scale, float eps,
                                        int head_norm, const float* sinks, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (!partial || dv <= 0 || dv > 64 * MA_DVU || nH <= 0 || nH > 65535 || n_maps < 1 || n_maps > 2 || n_splits < 1 || out_ld < nH * dv)
        return NG_BAD_SIZE;
    MaParams p{nullptr, nullptr, nullptr, nullptr, 0, nullptr, row_entry, out, out_ld, partial, nH, 1, 0, dv, 1, 0, 0, 0, n_splits, 0,
               0.f, 0.f, lambda, post_scale, eps, head_norm, nullptr, sinks};
    dim3 grid(n_rows, nH);
    const size_t smem = (size_t)n_maps * dv * sizeof(float);
    if (act_bf16) {
        if (n_maps == 2) NG_LAUNCH((mapped_attention_merge_kernel<__nv_bfloat16, 2>), grid, MA_THREADS, smem, stream, p);
        else NG_LAUNCH((mapped_attention_merge_kernel<__nv_bfloat16, 1>), grid, MA_THREADS, smem, stream, p);
    } else {
        if (n_maps == 2) NG_LAUNCH((mapped_attention_merge_kernel<float, 2>), grid, MA_THREADS, smem, stream, p);
        else NG_LAUNCH((mapped_attention_merge_kernel<float, 1>), grid, MA_THREADS, smem, stream, p);
    }
    return ng_launch_status();
}
