// Gated linear attention: a linear-attention recurrence whose state decays per key channel and token.
//
//   per head:  S_t = diag(alpha_t) S_(t-1) + k_t v_t^T      (S: [dk, dv], float32, one per request and head;
//                                                            alpha_t scales the rows, which belong to key channels)
//              o_t = S_t^T (q_t * dk^(-1/2))
//              out_t = o_t / sqrt(mean(o_t^2) + eps) * w * silu(g_t) * out_scale       (w: [dv], shared by heads)
//   alpha_t = sigmoid(z_t)^(1/tau) = exp(-softplus(-z_t) / tau), z_t one logit per head and key channel.
//
// Input rows are [q (nH*dk) | k (nH*dk) | v (nH*dv) | g (nH*dv)] and z [nH*dk], both of the activation type (rows of
// `out` lie ldo elements apart: it may be a block of columns of a wider buffer);
// the decay with its logarithm and exponential, the state, the read-out, the head's norm and the gate are float32.
//
// Token by token: one block per (entry, head) walks the entry's tokens in order, so a token's result does not
// depend on how its request was cut or on what else is in the step.  Thread (g, j) keeps rows g*R .. g*R+R-1 of
// column j of S in registers; the groups' partial dot products are added in ascending g.  The slot is read at the
// start (zero when the request has no tokens yet) and written at the end.
//
// Chunk by chunk (long portions): chunks of GC tokens run side by side.  With b_t the running sum of log alpha
// inside a chunk (b_t <= 0, per key channel), n the chunk's tokens and S the state before it:
//     U       = sum_s (exp(b_n - b_s) * k_s) v_s^T                       (what the chunk adds to the state)
//     S'      = diag(exp(b_n)) S + U
//     A[t][s] = sum_i q_t[i] k_s[i] exp(b_t[i] - b_s[i])   for s <= t    (scores inside the chunk)
//     o_t     = sum_s A[t][s] v_s + S^T (q_t * exp(b_t))
// Every exponent is a difference that is not positive, so nothing overflows however fast a channel forgets.
// `local` forms U of every chunk and leaves exp(b_n) beside it; `scan` walks a request's chunks in order, one thread
// per state element, leaves each chunk's S where its U was and the last S' in the request's slot; `out` forms o of
// every chunk; `finish` norms each head and applies the gate.  float32 FFMA throughout; results differ from the
// token-by-token kernel's by rounding only.  Chunk c of entry e keeps its U / S in slot cu_q[e] / GC + e + c of the
// scratch: slots of different entries do not meet, and rows / GC + entries + 1 slots are enough.
#include "ng_common.cuh"

__device__ __forceinline__ float gl_log_alpha(float z, float inv_tau) {
    // log sigmoid(z) = -softplus(-z) = min(z, 0) - log1p(exp(-|z|))
    return (fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau;
}

template <typename T, int R, int MAXT>
__global__ void __launch_bounds__(MAXT)
gated_linear_kernel(const T* __restrict__ x, const T* __restrict__ z, const float* __restrict__ norm_w,
                    float* __restrict__ state, T* __restrict__ out, const int* __restrict__ cu_q,
                    const int* __restrict__ ctx_before, const int* __restrict__ slots, int nH, int dk, int dv, int G,
                    float inv_tau, float eps, float out_scale, int ldo) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dk]
    float* ks = qs + dk;            // [dk]
    float* as = ks + dk;            // [dk]
    float* part = as + dk;          // [G * dv]
    float* red = part + G * dv;     // [32]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.x, head = blockIdx.y;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    if (qlen <= 0) return;
    const int ctx = ctx_before[e];
    const int tid = threadIdx.x;
    const int j = tid % dv, g = tid / dv;          // blockDim.x is a multiple of 32 >= G * dv
    const bool live = g < G;
    const int i0 = g * R;
    const size_t ld = 2 * (size_t)nH * (dk + dv), ldz = (size_t)nH * dk;
    const size_t off_q = (size_t)head * dk, off_k = (size_t)nH * dk + off_q;
    const size_t off_v = 2 * (size_t)nH * dk + (size_t)head * dv, off_g = off_v + (size_t)nH * dv;
    float* S = state + ((size_t)slots[e] * nH + head) * dk * dv;
    const float qscale = rsqrtf((float)dk);
    const float wj = tid < dv ? norm_w[tid] : 0.f;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = i0 + r;
        s[r] = (live && ctx > 0 && i < dk) ? S[(size_t)i * dv + j] : 0.f;
    }
    for (int t = 0; t < qlen; ++t) {
        const T* row = x + (size_t)(q0 + t) * ld;
        const T* zr = z + (size_t)(q0 + t) * ldz + off_q;
        for (int i = tid; i < dk; i += blockDim.x) {
            qs[i] = ng_ld(row + off_q + i) * qscale;
            ks[i] = ng_ld(row + off_k + i);
            as[i] = expf(gl_log_alpha(ng_ld(zr + i), inv_tau));
        }
        __syncthreads();
        if (live) {
            const float vj = ng_ld(row + off_v + j);
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = i0 + r;
                if (i < dk) {
                    s[r] = fmaf(as[i], s[r], ks[i] * vj);
                    acc = fmaf(s[r], qs[i], acc);
                }
            }
            part[g * dv + j] = acc;
        }
        __syncthreads();
        float o = 0.f;
        if (tid < dv)
            for (int gg = 0; gg < G; ++gg) o += part[gg * dv + tid];
        const float ss = ng_block_sum(tid < dv ? o * o : 0.f, red);
        if (tid < dv) {
            const float gate = ng_ld(row + off_g + tid);
            const float y = o * rsqrtf(ss / (float)dv + eps) * wj * (gate / (1.f + expf(-gate))) * out_scale;
            ng_st(out + (size_t)(q0 + t) * ldo + (size_t)head * dv + tid, y);
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = i0 + r;
            if (i < dk) S[(size_t)i * dv + j] = s[r];
        }
    }
}

NG_EXPORT int ng_gated_linear(const void* x, const void* z, const float* norm_w, float* state, void* out,
                              const int* cu_q, const int* ctx_before, const int* slots, int n_entries, int nH, int dk,
                              int dv, float tau, float eps, float out_scale, int ldo, int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (nH <= 0 || dk <= 0 || dv <= 0 || !(tau > 0.f) || ldo < nH * dv) return NG_BAD_SIZE;
    // rows of S per thread and the block size that goes with them: 16 rows up to 512 threads, else 64 rows
    int R = 16, maxt = 512;
    int G = (dk + R - 1) / R;
    if ((size_t)G * dv > 512) {
        R = 64;
        G = (dk + R - 1) / R;
        maxt = (size_t)G * dv > 256 ? 1024 : 256;
    }
    if ((size_t)G * dv > 1024) return NG_BAD_SIZE;
    const int threads = ((G * dv + 31) / 32) * 32;
    const size_t smem = (3 * (size_t)dk + (size_t)G * dv + 32) * sizeof(float);
    if (smem > 48 * 1024) return NG_BAD_SIZE;
    dim3 grid(n_entries, nH);
    if (grid.y > 65535) return NG_BAD_SIZE;
    const float inv_tau = 1.f / tau;
#define GL_LAUNCH(TT, RR, MT)                                                                                        \
    NG_LAUNCH((gated_linear_kernel<TT, RR, MT>), grid, threads, smem, stream, (const TT*)x, (const TT*)z, norm_w,   \
              state, (TT*)out, cu_q, ctx_before, slots, nH, dk, dv, G, inv_tau, eps, out_scale, ldo)
    if (act_bf16) {
        if (R == 16) GL_LAUNCH(__nv_bfloat16, 16, 512);
        else if (maxt == 256) GL_LAUNCH(__nv_bfloat16, 64, 256);
        else GL_LAUNCH(__nv_bfloat16, 64, 1024);
    } else {
        if (R == 16) GL_LAUNCH(float, 16, 512);
        else if (maxt == 256) GL_LAUNCH(float, 64, 256);
        else GL_LAUNCH(float, 64, 1024);
    }
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------------------- portions, chunk by chunk
#define GC 32
#define GC_THREADS 256

// Bs[t][i] = sum of log alpha over the chunk's tokens 0..t (rows past n repeat b_n): every thread forms its share of
// the logarithms, then a thread per key channel adds them up along the chunk.  Rows of Bs lie ldb apart.  Ends with a barrier.
template <typename T>
__device__ __forceinline__ void gl_cumsum(const T* __restrict__ z, size_t ldz, size_t off, int row0, int n, int dk,
                                          float inv_tau, float* Bs, int ldb) {
    for (int idx = threadIdx.x; idx < GC * dk; idx += GC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        Bs[t * ldb + i] = t < n ? gl_log_alpha(ng_ld(z + (size_t)(row0 + t) * ldz + off + i), inv_tau) : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < dk; i += GC_THREADS) {
        float b = 0.f;
#pragma unroll 8
        for (int t = 0; t < GC; ++t) {
            b += Bs[t * ldb + i];
            Bs[t * ldb + i] = b;
        }
    }
    __syncthreads();
}

struct GlGeom {
    int nH, dk, dv, per_slot;        // per_slot = dk * dv + dk: a chunk's U (later the state before it) and its whole decay
    float inv_tau;
};

// what a chunk adds to the state, U = sum_s (exp(b_n - b_s) k_s) v_s^T, and exp(b_n) behind it
template <typename T>
__global__ void __launch_bounds__(GC_THREADS)
gl_chunk_local_kernel(const T* __restrict__ x, const T* __restrict__ z, float* __restrict__ scratch,
                      const int* __restrict__ cu_q, GlGeom g) {
    extern __shared__ float sm[];
    const int dk = g.dk, dv = g.dv;
    float* Bs = sm;                   // [GC][dk]
    float* Ks = Bs + GC * dk;         // [GC][dk]
    float* Vs = Ks + GC * dk;         // [GC][dv]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int c = blockIdx.x, e = blockIdx.y, head = blockIdx.z;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    if (c * GC >= qlen) return;
    const int n = min(GC, qlen - c * GC), row0 = q0 + c * GC;
    float* U = scratch + ((size_t)(q0 / GC + e + c) * g.nH + head) * g.per_slot;
    const size_t ld = 2 * (size_t)g.nH * (dk + dv), ldz = (size_t)g.nH * dk;
    const size_t off_q = (size_t)head * dk, off_k = (size_t)g.nH * dk + off_q;
    const size_t off_v = 2 * (size_t)g.nH * dk + (size_t)head * dv;
    gl_cumsum(z, ldz, off_q, row0, n, dk, g.inv_tau, Bs, dk);
    for (int idx = threadIdx.x; idx < GC * dk; idx += GC_THREADS) {
        const int s = idx / dk, i = idx - s * dk;
        Ks[idx] = s < n ? expf(Bs[(n - 1) * dk + i] - Bs[idx]) * ng_ld(x + (size_t)(row0 + s) * ld + off_k + i) : 0.f;
    }
    for (int idx = threadIdx.x; idx < GC * dv; idx += GC_THREADS) {
        const int s = idx / dv, j = idx - s * dv;
        Vs[idx] = s < n ? ng_ld(x + (size_t)(row0 + s) * ld + off_v + j) : 0.f;
    }
    __syncthreads();
    const int tj_n = dv / 4;
    for (int tile = threadIdx.x; tile < (dk / 4) * tj_n; tile += GC_THREADS) {
        const int ti = tile / tj_n, tj = tile - ti * tj_n;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll 4
        for (int s = 0; s < GC; ++s) {
            const float4 kv = *reinterpret_cast<const float4*>(Ks + s * dk + 4 * ti);
            const float4 vv = *reinterpret_cast<const float4*>(Vs + s * dv + 4 * tj);
            const float ka[4] = {kv.x, kv.y, kv.z, kv.w}, va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(ka[a], va[b], acc[a][b]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
            *reinterpret_cast<float4*>(U + (size_t)(4 * ti + a) * dv + 4 * tj) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
    for (int i = threadIdx.x; i < dk; i += GC_THREADS) U[(size_t)dk * dv + i] = expf(Bs[(n - 1) * dk + i]);
}

// a request's chunks in order, a thread per state element: each chunk's place receives the state before it
__global__ void __launch_bounds__(GC_THREADS)
gl_chunk_scan_kernel(float* __restrict__ scratch, float* __restrict__ state, const int* __restrict__ cu_q,
                     const int* __restrict__ ctx_before, const int* __restrict__ slots, GlGeom g) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.y, head = blockIdx.z;
    const int idx = blockIdx.x * GC_THREADS + threadIdx.x;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    if (qlen <= 0 || idx >= g.dk * g.dv) return;
    const int chunks = (qlen + GC - 1) / GC, i = idx / g.dv;
    float* S = state + ((size_t)slots[e] * g.nH + head) * g.dk * g.dv;
    float* U = ng_after_wait(scratch) + ((size_t)(q0 / GC + e) * g.nH + head) * g.per_slot;
    float s = ctx_before[e] > 0 ? S[idx] : 0.f;
    // eight chunks' terms are requested together, then the recurrence walks them: a load per step would wait for
    // the store before it (the compiler cannot tell the places apart)
    const size_t step = (size_t)g.nH * g.per_slot;
    for (int c0 = 0; c0 < chunks; c0 += 8, U += 8 * step) {
        float u[8], d[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool in = c0 + k < chunks;
            u[k] = in ? U[k * step + idx] : 0.f;
            d[k] = in ? U[k * step + (size_t)g.dk * g.dv + i] : 1.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < chunks) {
                U[k * step + idx] = s;
                s = fmaf(d[k], s, u[k]);
            }
        }
    }
    S[idx] = s;
}

// o_t = sum_(s<=t) A[t][s] v_s + S^T (q_t exp(b_t)) of every chunk, S the state before it; float32 into `raw`
template <typename T>
__global__ void __launch_bounds__(GC_THREADS)
gl_chunk_out_kernel(const T* __restrict__ x, const T* __restrict__ z, const float* __restrict__ scratch,
                    float* __restrict__ raw, const int* __restrict__ cu_q, GlGeom g) {
    extern __shared__ float sm[];
    const int dk = g.dk, dv = g.dv;
    const int ldk = dk + 1;           // a row's pitch: the scores walk rows with a lane per row, a pitch of dk would put them in one bank
    float* Bs = sm;                   // [GC][ldk]
    float* Qs = Bs + GC * ldk;        // [GC][ldk]
    float* Ks = Qs + GC * ldk;        // [GC][ldk]
    float* Vs = Ks + GC * ldk + (4 - (3 * GC * ldk) % 4) % 4;      // [GC][dv], 16-byte aligned
    float* As = Vs + GC * dv;         // [GC][GC + 1]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int c = blockIdx.x, e = blockIdx.y, head = blockIdx.z;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    if (c * GC >= qlen) return;
    const int n = min(GC, qlen - c * GC), row0 = q0 + c * GC;
    const float* S = ng_after_wait(scratch) + ((size_t)(q0 / GC + e + c) * g.nH + head) * g.per_slot;
    const size_t ld = 2 * (size_t)g.nH * (dk + dv), ldz = (size_t)g.nH * dk;
    const size_t off_q = (size_t)head * dk, off_k = (size_t)g.nH * dk + off_q;
    const size_t off_v = 2 * (size_t)g.nH * dk + (size_t)head * dv;
    const float qscale = rsqrtf((float)dk);
    gl_cumsum(z, ldz, off_q, row0, n, dk, g.inv_tau, Bs, ldk);
    for (int idx = threadIdx.x; idx < GC * dk; idx += GC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        Qs[t * ldk + i] = t < n ? ng_ld(x + (size_t)(row0 + t) * ld + off_q + i) * qscale : 0.f;
        Ks[t * ldk + i] = t < n ? ng_ld(x + (size_t)(row0 + t) * ld + off_k + i) : 0.f;
    }
    for (int idx = threadIdx.x; idx < GC * dv; idx += GC_THREADS) {
        const int s = idx / dv, j = idx - s * dv;
        Vs[idx] = s < n ? ng_ld(x + (size_t)(row0 + s) * ld + off_v + j) : 0.f;
    }
    __syncthreads();
    // scores inside the chunk; every exponent is a difference that is not positive
    for (int idx = threadIdx.x; idx < GC * GC; idx += GC_THREADS) {
        const int t = idx / GC, s = idx - t * GC;
        float a = 0.f;
        if (s <= t && t < n) {
            const float *qt = Qs + t * ldk, *ks = Ks + s * ldk, *bt = Bs + t * ldk, *bs = Bs + s * ldk;
            float a0 = 0.f, a1 = 0.f;
            for (int i = 0; i < dk; i += 2) {
                a0 = fmaf(qt[i] * ks[i], __expf(bt[i] - bs[i]), a0);
                a1 = fmaf(qt[i + 1] * ks[i + 1], __expf(bt[i + 1] - bs[i + 1]), a1);
            }
            a = a0 + a1;
        }
        As[t * (GC + 1) + s] = a;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GC * dk; idx += GC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        Qs[t * ldk + i] *= expf(Bs[t * ldk + i]);
    }
    __syncthreads();
    const int tj_n = dv / 4;
    for (int tile = threadIdx.x; tile < (GC / 4) * tj_n; tile += GC_THREADS) {
        const int tt = tile / tj_n, tj = tile - tt * tj_n;
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll 4
        for (int s = 0; s < GC; ++s) {
            const float4 vv = *reinterpret_cast<const float4*>(Vs + s * dv + 4 * tj);
            const float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float w = As[(4 * tt + a) * (GC + 1) + s];
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(w, va[b], acc[a][b]);
            }
        }
#pragma unroll 8
        for (int i = 0; i < dk; ++i) {
            const float4 sv = *reinterpret_cast<const float4*>(S + (size_t)i * dv + 4 * tj);
            const float sa[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const float w = Qs[(4 * tt + a) * (dk + 1) + i];
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(w, sa[b], acc[a][b]);
            }
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
            if (4 * tt + a < n)
                *reinterpret_cast<float4*>(raw + (size_t)(row0 + 4 * tt + a) * g.nH * dv + (size_t)head * dv + 4 * tj) =
                    make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
    }
}

// each head's o over its root mean square, times the weight, silu(gate) and out_scale: a warp per (row, head)
template <typename T>
__global__ void gl_finish_kernel(const float* __restrict__ raw, const T* __restrict__ x, const float* __restrict__ norm_w,
                                 T* __restrict__ out, const int* __restrict__ row_entry_or_null, int n_rows, GlGeom g, float eps,
                                 float out_scale, int ldo) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= n_rows * g.nH) return;
    const int row = w / g.nH, head = w - row * g.nH;
    const float* o = ng_after_wait(raw) + (size_t)row * g.nH * g.dv + (size_t)head * g.dv;
    const T* gate = x + (size_t)row * 2 * g.nH * (g.dk + g.dv) + 2 * (size_t)g.nH * g.dk + (size_t)g.nH * g.dv + (size_t)head * g.dv;
    float ss = 0.f;
    for (int j = lane; j < g.dv; j += 32) ss = fmaf(o[j], o[j], ss);
    const float r = rsqrtf(ng_warp_sum(ss) / (float)g.dv + eps);
    for (int j = lane; j < g.dv; j += 32) {
        const float gt = ng_ld(gate + j);
        ng_st(out + (size_t)row * ldo + (size_t)head * g.dv + j, o[j] * r * norm_w[j] * (gt / (1.f + expf(-gt))) * out_scale);
    }
}

static size_t gl_out_smem(int dk, int dv) { return ((size_t)3 * GC * (dk + 1) + 4 + (size_t)GC * dv + GC * (GC + 1)) * sizeof(float); }

// whether the chunk-by-chunk kernels take the head sizes: rows and columns in fours, the tiles within shared memory
NG_EXPORT int ng_gated_linear_chunked_takes(int dk, int dv) {
    return dk > 0 && dv > 0 && dk % 4 == 0 && dv % 4 == 0 && gl_out_smem(dk, dv) <= 160 * 1024;
}

// raw: float32 [n_rows, nH * dv]; scratch: (n_rows / GC + n_entries + 1) * nH * (dk * dv + dk) float32 values
NG_EXPORT int ng_gated_linear_chunked(const void* x, const void* z, const float* norm_w, float* state, void* out,
                                      float* raw, float* scratch, const int* cu_q, const int* ctx_before, const int* slots,
                                      int n_entries, int n_rows, int max_q, int nH, int dk, int dv, float tau, float eps,
                                      float out_scale, int ldo, int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0 || n_rows <= 0) return NG_OK;
    if (nH <= 0 || nH > 65535 || n_entries > 65535 || max_q <= 0 || !(tau > 0.f) || ldo < nH * dv ||
        !ng_gated_linear_chunked_takes(dk, dv) || !raw || !scratch)
        return NG_BAD_SIZE;
    const GlGeom g{nH, dk, dv, dk * dv + dk, 1.f / tau};
    const int chunks = (max_q + GC - 1) / GC;
    const dim3 grid(chunks, n_entries, nH), sgrid((dk * dv + GC_THREADS - 1) / GC_THREADS, n_entries, nH);
    const size_t smem_local = ((size_t)2 * GC * dk + (size_t)GC * dv) * sizeof(float), smem_out = gl_out_smem(dk, dv);
    const unsigned fblocks = (unsigned)(((size_t)n_rows * nH + 7) / 8);
#define GL_CHUNKED(TT)                                                                                                 \
    {                                                                                                                  \
        static bool configured = false;                                                                                \
        if (!configured) {                                                                                             \
            if (cudaFuncSetAttribute(gl_chunk_local_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess || \
                cudaFuncSetAttribute(gl_chunk_out_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)     \
                return NG_LAUNCH_FAILED;                                                                               \
            configured = true;                                                                                         \
        }                                                                                                              \
        NG_LAUNCH((gl_chunk_local_kernel<TT>), grid, GC_THREADS, smem_local, stream, (const TT*)x, (const TT*)z, scratch, cu_q, g); \
        NG_LAUNCH((gl_chunk_scan_kernel), sgrid, GC_THREADS, 0, stream, scratch, state, cu_q, ctx_before, slots, g);   \
        NG_LAUNCH((gl_chunk_out_kernel<TT>), grid, GC_THREADS, smem_out, stream, (const TT*)x, (const TT*)z,           \
                  (const float*)scratch, raw, cu_q, g);                                                                \
        NG_LAUNCH((gl_finish_kernel<TT>), fblocks, 256, 0, stream, (const float*)raw, (const TT*)x, norm_w, (TT*)out,  \
                  (const int*)nullptr, n_rows, g, eps, out_scale, ldo);                                                \
    }
    if (act_bf16) GL_CHUNKED(__nv_bfloat16) else GL_CHUNKED(float)
    return ng_launch_status();
}
