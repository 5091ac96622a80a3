// The gated delta rule: a linear recurrence whose state is corrected towards each token's value, over a ragged
// batch of prompt portions and single tokens.
//
//   per value head h (query/key head h / (nH / nG)), S [dk, dv] float32, one per request and head:
//       S <- g_t S ;  u = beta_t (v_t - S^T k_t) ;  S <- S + k_t u^T ;  o_t = S^T q_t
//   q, k, v: projections passed through a short causal convolution per channel and silu; q and k then unit
//   vectors per head (x / sqrt(sum x^2 + 1e-6)), q times dk^(-1/2);
//   beta_t = sigmoid(b_t),  g_t = exp(-exp(A_log_h) softplus(a_t + dt_bias_h));
//   out_t = o_t / sqrt(mean(o_t^2) + eps) * w * silu(gate_t)  per head.
//
// Input rows p [N, ldp] of the activation type hold the stacked projections [q | k | v | gate | a | b].  Three
// kernels.  `conv_silu`: the convolution of the q, k, v channels with silu, float32 out; the request's slot
// keeps its last L-1 inputs.  `gated_delta`: a block per (slice of value columns, head, entry) walks the
// entry's tokens in order (a token's result does not depend on the cut or on the batch); the columns of S are
// independent of one another, so a column is dealt to KS neighbouring lanes, each with R of its rows in
// registers, and the two dot products of a token are finished with shuffles.  Tokens are staged GD_TB at a time
// in shared memory (unit norms, beta and the decay are formed there, float32).  `finish`: the head's norm, its
// weight and the gate.  Everything after the projections is float32.
#include "ng_common.cuh"

#define GD_MAX_L 8
#define GD_CONV_TILE 32
#define GD_CONV_THREADS 128
#define GD_TB 16
#define GD_KS 8
#define GD_CB 16
#define GD_THREADS (GD_KS * GD_CB)

__device__ __forceinline__ float gd_silu(float z) { return z / (1.f + expf(-z)); }

// ------------------------------------------------------------------------------------------ convolution + silu
// Grid (channel blocks, token tiles, entries); a thread owns one channel of one tile and walks its tokens in order.
// Only tile 0 of an entry reads the slot, and only it writes the slot, after its reads.
template <typename T, int L>
__global__ void __launch_bounds__(GD_CONV_THREADS)
gd_conv_silu_kernel(const T* __restrict__ p, int ldp, const float* __restrict__ w, float* __restrict__ state,
                    float* __restrict__ out, const int* __restrict__ cu_q, const int* __restrict__ ctx_before,
                    const int* __restrict__ slots, int C) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.z;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    const int t0 = blockIdx.y * GD_CONV_TILE;
    const int d = blockIdx.x * GD_CONV_THREADS + threadIdx.x;
    if (t0 >= qlen || d >= C) return;
    const int ctx = ctx_before[e];
    float* st = state + (size_t)slots[e] * (L - 1) * C + d;        // st[j*C]: the input at position ctx-(L-1)+j
    const T* ur = p + (size_t)q0 * ldp + d;
    float* orow = out + (size_t)q0 * C + d;
    float wk[L], hist[L - 1], old[L - 1];
#pragma unroll
    for (int k = 0; k < L; ++k) wk[k] = w[(size_t)d * L + k];
    const bool first = t0 == 0;
#pragma unroll
    for (int j = 0; j < L - 1; ++j) old[j] = (first && ctx - (L - 1) + j >= 0) ? st[(size_t)j * C] : 0.f;
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
        const int ti = t0 - (L - 1) + j;
        hist[j] = ti >= 0 ? ng_ld(ur + (size_t)ti * ldp) : old[j];
    }
    const int t1 = min(t0 + GD_CONV_TILE, qlen);
    for (int t = t0; t < t1; ++t) {
        const float x = ng_ld(ur + (size_t)t * ldp);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < L - 1; ++k) acc = fmaf(wk[k], hist[k], acc);
        acc = fmaf(wk[L - 1], x, acc);
        orow[(size_t)t * C] = gd_silu(acc);
#pragma unroll
        for (int k = 0; k < L - 2; ++k) hist[k] = hist[k + 1];
        hist[L - 2] = x;
    }
    if (first) {
#pragma unroll
        for (int j = 0; j < L - 1; ++j) {
            const int ti = qlen - (L - 1) + j;
            float v = 0.f;
            if (ti >= 0) v = ng_ld(ur + (size_t)ti * ldp);
            else {
#pragma unroll
                for (int k = 0; k < L - 1; ++k)
                    if (k == ti + (L - 1)) v = old[k];
            }
            st[(size_t)j * C] = v;
        }
    }
}

// p: [n_rows, ldp] of the activation type, the convolved channels are its first C columns; w: [C, L] float32 (tap L-1
// on the current token); state: [slots, L-1, C] float32; out: [n_rows, C] float32 = silu(conv).
NG_EXPORT int ng_gd_conv_silu(const void* p, int ldp, const float* w, float* state, float* out, const int* cu_q,
                              const int* ctx_before, const int* slots, int n_entries, int max_q, int C, int L,
                              int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0) return NG_OK;
    if (C <= 0 || ldp < C || L < 2 || L > GD_MAX_L) return NG_BAD_SIZE;
    dim3 grid((C + GD_CONV_THREADS - 1) / GD_CONV_THREADS, (max_q + GD_CONV_TILE - 1) / GD_CONV_TILE, n_entries);
    if (grid.y > 65535 || grid.z > 65535) return NG_BAD_SIZE;
#define GD_CONV_CASE(LL)                                                                                              \
    case LL:                                                                                                          \
        if (act_bf16)                                                                                                 \
            NG_LAUNCH((gd_conv_silu_kernel<__nv_bfloat16, LL>), grid, GD_CONV_THREADS, 0, stream,                     \
                      (const __nv_bfloat16*)p, ldp, w, state, out, cu_q, ctx_before, slots, C);                       \
        else                                                                                                          \
            NG_LAUNCH((gd_conv_silu_kernel<float, LL>), grid, GD_CONV_THREADS, 0, stream, (const float*)p, ldp, w,    \
                      state, out, cu_q, ctx_before, slots, C);                                                        \
        break;
    switch (L) {
        GD_CONV_CASE(2) GD_CONV_CASE(3) GD_CONV_CASE(4) GD_CONV_CASE(5) GD_CONV_CASE(6) GD_CONV_CASE(7) GD_CONV_CASE(8)
    }
    return ng_launch_status();
}

// ------------------------------------------------------------------------------------------ recurrence
struct GdParams {
    const float* conv;      // [N, C] float32: q (nG*dk) | k (nG*dk) | v (nH*dv), after convolution and silu
    const void* p;          // [N, ldp] activation type: a at off_a + head, b at off_b + head
    int ldp, off_a, off_b;
    const float* a_log; const float* dt_bias;
    float* state;           // [slots, nH, dk, dv]
    float* o_raw;           // [N, nH*dv]
    const int* cu_q; const int* ctx_before; const int* slots;
    int nH, nG, dk, dv;
};

template <typename T, int R>
__global__ void __launch_bounds__(GD_THREADS)
gated_delta_kernel(const GdParams P) {
    extern __shared__ float sm[];
    const int dk = P.dk, dv = P.dv;
    float* qs = sm;                         // [GD_TB][dk]
    float* ks = qs + GD_TB * dk;            // [GD_TB][dk]
    float* vs = ks + GD_TB * dk;            // [GD_TB][GD_CB]
    float* bs = vs + GD_TB * GD_CB;         // [GD_TB] beta
    float* gs = bs + GD_TB;                 // [GD_TB] decay
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.z, head = blockIdx.y, c0 = blockIdx.x * GD_CB;
    const int q0 = P.cu_q[e];
    const int qlen = P.cu_q[e + 1] - q0;
    if (qlen <= 0) return;
    const int ctx = P.ctx_before[e];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = tid % GD_KS, col = c0 + tid / GD_KS;
    const bool col_ok = col < dv;
    const int qk_head = head / (P.nH / P.nG);
    const int C = 2 * P.nG * dk + P.nH * dv;
    const size_t off_q = (size_t)qk_head * dk, off_k = (size_t)P.nG * dk + off_q;
    const size_t off_v = 2 * (size_t)P.nG * dk + (size_t)head * dv;
    float* S = P.state + ((size_t)P.slots[e] * P.nH + head) * dk * dv;
    const float* conv = ng_after_wait(P.conv);
    const T* pr = reinterpret_cast<const T*>(ng_after_wait(P.p));
    const float neg_rate = -expf(P.a_log[head]);
    const float dtb = P.dt_bias[head];
    const float q_scale = rsqrtf((float)dk);
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = part + GD_KS * r;
        s[r] = (col_ok && ctx > 0 && i < dk) ? S[(size_t)i * dv + col] : 0.f;
    }
    for (int t0 = 0; t0 < qlen; t0 += GD_TB) {
        const int nt = min(GD_TB, qlen - t0);
        for (int idx = tid; idx < nt * dk; idx += GD_THREADS) {
            const int t = idx / dk, i = idx - t * dk;
            const float* row = conv + (size_t)(q0 + t0 + t) * C;
            qs[t * dk + i] = row[off_q + i];
            ks[t * dk + i] = row[off_k + i];
        }
        for (int idx = tid; idx < nt * GD_CB; idx += GD_THREADS) {
            const int t = idx / GD_CB, c = idx - t * GD_CB;
            vs[idx] = (c0 + c < dv) ? conv[(size_t)(q0 + t0 + t) * C + off_v + c0 + c] : 0.f;
        }
        if (tid < nt) {
            const T* row = pr + (size_t)(q0 + t0 + tid) * P.ldp;
            const float a = ng_ld(row + P.off_a + head) + dtb, b = ng_ld(row + P.off_b + head);
            const float sp = a > 20.f ? a : log1pf(expf(a));
            bs[tid] = 1.f / (1.f + expf(-b));
            gs[tid] = expf(neg_rate * sp);
        }
        __syncthreads();
        // unit vectors: a warp per (token, q or k)
        for (int task = warp; task < 2 * nt; task += GD_THREADS / 32) {
            float* x = (task & 1 ? ks : qs) + (task >> 1) * dk;
            float ss = 0.f;
            for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
            const float r = rsqrtf(ng_warp_sum(ss) + 1e-6f) * (task & 1 ? 1.f : q_scale);
            for (int i = lane; i < dk; i += 32) x[i] *= r;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float* kt = ks + t * dk;
            const float* qt = qs + t * dk;
            const float g = gs[t], beta = bs[t], v = vs[t * GD_CB + tid / GD_KS];
            float kr[R];
            float dot = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = part + GD_KS * r;
                kr[r] = i < dk ? kt[i] : 0.f;
                s[r] *= g;
                dot = fmaf(s[r], kr[r], dot);
            }
#pragma unroll
            for (int o = GD_KS / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            const float u = beta * (v - dot);
            float out = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = part + GD_KS * r;
                s[r] = fmaf(kr[r], u, s[r]);
                out = fmaf(s[r], i < dk ? qt[i] : 0.f, out);
            }
#pragma unroll
            for (int o = GD_KS / 2; o > 0; o >>= 1) out += __shfl_xor_sync(0xffffffffu, out, o);
            if (part == 0 && col_ok) P.o_raw[(size_t)(q0 + t0 + t) * P.nH * dv + (size_t)head * dv + col] = out;
        }
        __syncthreads();
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = part + GD_KS * r;
            if (i < dk) S[(size_t)i * dv + col] = s[r];
        }
    }
}

NG_EXPORT int ng_gated_delta(const float* conv, const void* p, int ldp, int off_a, int off_b, const float* a_log,
                             const float* dt_bias, float* state, float* o_raw, const int* cu_q, const int* ctx_before,
                             const int* slots, int n_entries, int nH, int nG, int dk, int dv, int act_bf16,
                             cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (nH <= 0 || nG <= 0 || nH % nG || dk <= 0 || dk > 32 * GD_KS || dv <= 0 || n_entries > 65535 || nH > 65535)
        return NG_BAD_SIZE;
    GdParams P{conv, p, ldp, off_a, off_b, a_log, dt_bias, state, o_raw, cu_q, ctx_before, slots, nH, nG, dk, dv};
    dim3 grid((dv + GD_CB - 1) / GD_CB, nH, n_entries);
    const size_t smem = ((size_t)2 * GD_TB * dk + GD_TB * GD_CB + 2 * GD_TB) * sizeof(float);
    const int rows = (dk + GD_KS - 1) / GD_KS;
#define GD_CASE(RR)                                                                                                   \
    do {                                                                                                              \
        if (act_bf16) NG_LAUNCH((gated_delta_kernel<__nv_bfloat16, RR>), grid, GD_THREADS, smem, stream, P);          \
        else NG_LAUNCH((gated_delta_kernel<float, RR>), grid, GD_THREADS, smem, stream, P);                           \
    } while (0)
    if (rows <= 4) GD_CASE(4);
    else if (rows <= 8) GD_CASE(8);
    else if (rows <= 16) GD_CASE(16);
    else GD_CASE(32);
    return ng_launch_status();
}

// ------------------------------------------------------------------------------------------ head norm and gate
// out[row, h*dv + c] = o / sqrt(mean_c(o^2) + eps) * w[c] * silu(gate); a warp per (row, head); rows of no entry: zeros
template <typename T>
__global__ void __launch_bounds__(128)
gd_finish_kernel(const float* __restrict__ o_raw, const T* __restrict__ p, int ldp, int off_gate, const float* __restrict__ w,
                 const int* __restrict__ row_entry, T* __restrict__ out, int n_rows, int nH, int dv, float eps) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (task >= (long long)n_rows * nH) return;
    const int row = (int)(task / nH), head = (int)(task % nH);
    T* dst = out + (size_t)row * nH * dv + (size_t)head * dv;
    if (row_entry[row] < 0) {
        for (int c = lane; c < dv; c += 32) ng_st(dst + c, 0.f);
        return;
    }
    const float* o = ng_after_wait(o_raw) + (size_t)row * nH * dv + (size_t)head * dv;
    const T* gate = ng_after_wait(p) + (size_t)row * ldp + off_gate + (size_t)head * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[c], o[c], ss);
    const float r = rsqrtf(ng_warp_sum(ss) / (float)dv + eps);
    for (int c = lane; c < dv; c += 32) ng_st(dst + c, o[c] * r * w[c] * gd_silu(ng_ld(gate + c)));
}

NG_EXPORT int ng_gd_finish(const float* o_raw, const void* p, int ldp, int off_gate, const float* w, const int* row_entry,
                           void* out, int n_rows, int nH, int dv, float eps, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (nH <= 0 || dv <= 0) return NG_BAD_SIZE;
    const long long blocks = ((long long)n_rows * nH + 3) / 4;
    if (blocks > 0x7fffffffLL) return NG_BAD_SIZE;
    if (act_bf16)
        NG_LAUNCH((gd_finish_kernel<__nv_bfloat16>), (unsigned)blocks, 128, 0, stream, o_raw, (const __nv_bfloat16*)p, ldp,
                  off_gate, w, row_entry, (__nv_bfloat16*)out, n_rows, nH, dv, eps);
    else
        NG_LAUNCH((gd_finish_kernel<float>), (unsigned)blocks, 128, 0, stream, o_raw, (const float*)p, ldp, off_gate, w,
                  row_entry, (float*)out, n_rows, nH, dv, eps);
    return ng_launch_status();
}
