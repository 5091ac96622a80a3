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

// ------------------------------------------------------------------------------------------ portions, chunk by chunk
// The same recurrence for long portions, regrouped so that most of the work of a portion's chunks runs side by side.
// With chunks of GC tokens, S the state before a chunk, cl_t = sum_(s<=t) log g_s inside the chunk (so that the decay
// from token s to token t is exp(cl_t - cl_s), never above one), and k, q the unit vectors:
//     A[t][s] = beta_t exp(cl_t - cl_s) (k_t . k_s)   for s < t
//     (I + A) U  = beta V - diag(beta exp(cl)) K S    hence  U = U' - W S,  (I + A) U' = beta V,  (I + A) W = beta exp(cl) K
//     S'         = exp(cl_last) S + K~^T U,           K~_t = exp(cl_last - cl_t) k_t
//     o_t        = exp(cl_t) S^T q_t + sum_(s<=t) exp(cl_t - cl_s) (q_t . k_s) u_s
// `prep` (a block per chunk and head, all chunks side by side) solves the two triangular systems by substitution, a
// thread per column, and leaves W (transposed), K~ and cl in the scratch and U' where the outputs will be.  `scan` (a
// block per request, head and 16 value columns) walks the chunks in order: U = U' - W S in place, S' from K~ and U; the
// state before each chunk goes to the scratch; the next chunk's tiles are copied asynchronously meanwhile.  `out` (a
// block per chunk and head) forms o from q, k, cl, U and the chunk's S, in U's place.
// Float32 FFMA throughout; the results differ from the token-by-token kernel's by rounding only.  Chunk c of entry e
// uses slot cu_q[e] / GC + e + c of the scratch, as the chunks of different entries then never meet.
#define GC 32
#define GC_THREADS 128
#define GC_DVS 16          // value columns of a scan block
#define GS_THREADS 256     // threads of a scan block: two warps a scheduler, one hides the other's shared-memory latency
#define GC_RED 20          // floats between two threads' partial tiles (no bank conflicts for 16-byte accesses)
#define GC_LDT 36          // floats between the rows of a transposed tile [dim][GC]: 16-byte rows, and a quarter warp's
                           // 16-byte accesses to one column of four tokens meet every bank once

struct GcParams {
    const float* conv; const void* p;
    int ldp, off_a, off_b;
    const float* a_log; const float* dt_bias;
    float* state; float* o_raw;
    float* wt;              // [slots][nH][dk][GC]
    float* kt;              // [slots][nH][GC][dk]
    float* cl;              // [slots][nH][GC]
    float* sb;              // [slots][nH][dk][dv]: the state before each chunk
    const int* cu_q; const int* ctx_before; const int* slots;
    int nH, nG, dk, dv;
};

// rows of unit vectors into shared memory [GC][dk+1]: all loads first (many in flight), then a warp per row for the
// norm; rows past n are zero.  Ends with the block in step.
__device__ __forceinline__ void gc_load_unit(const float* __restrict__ src, size_t ld, int n, int dk, float mul, float* dst) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ldk = dk + 1;
    const int dk4 = dk >> 2;
#pragma unroll 4
    for (int idx = threadIdx.x; idx < GC * dk4; idx += GC_THREADS) {      // 16-byte reads: dk, ld and the start in fours
        const int t = idx / dk4, i = (idx - t * dk4) * 4;
        const float4 x = t < n ? *reinterpret_cast<const float4*>(src + (size_t)t * ld + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        float* d = dst + t * ldk + i;
        d[0] = x.x, d[1] = x.y, d[2] = x.z, d[3] = x.w;
    }
    __syncthreads();
    for (int t = warp; t < n; t += GC_THREADS / 32) {
        float* x = dst + t * ldk;
        float ss = 0.f;
        for (int i = lane; i < dk; i += 32) ss = fmaf(x[i], x[i], ss);
        const float r = rsqrtf(ng_warp_sum(ss) + 1e-6f) * mul;
        for (int i = lane; i < dk; i += 32) x[i] *= r;
    }
    __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(GC_THREADS)
gd_chunk_prep_kernel(const GcParams P) {
    extern __shared__ float sm[];
    const int dk = P.dk, dv = P.dv, nH = P.nH, ldk = dk + 1;
    float* Ks = sm;                        // [GC][dk+1]
    float* As = Ks + GC * ldk;             // [GC][GC]
    float* cl = As + GC * GC;              // [GC]
    float* bt = cl + GC;                   // [GC]
    float* Vs = bt + GC;                   // [GC][dv]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int c = blockIdx.x, head = blockIdx.y, e = blockIdx.z;
    const int q0 = P.cu_q[e], qlen = P.cu_q[e + 1] - q0;
    if (c * GC >= qlen) return;
    const int n = min(GC, qlen - c * GC), row0 = q0 + c * GC;
    const size_t slot = (size_t)(q0 / GC + e + c) * nH + head;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = 2 * P.nG * dk + nH * dv;
    const size_t off_k = (size_t)P.nG * dk + (size_t)(head / (nH / P.nG)) * dk;
    const size_t off_v = 2 * (size_t)P.nG * dk + (size_t)head * dv;
    const float* conv = ng_after_wait(P.conv) + (size_t)row0 * C;
    const int dv4 = dv >> 2;
#pragma unroll 4
    for (int idx = tid; idx < GC * dv4; idx += GC_THREADS) {
        const int t = idx / dv4, v = (idx - t * dv4) * 4;
        *reinterpret_cast<float4*>(Vs + t * dv + v) =
            t < n ? *reinterpret_cast<const float4*>(conv + (size_t)t * C + off_v + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    gc_load_unit(conv + off_k, C, n, dk, 1.f, Ks);
    if (warp == 0) {
        float lg = 0.f, b = 0.f;
        if (lane < n) {
            const T* row = reinterpret_cast<const T*>(ng_after_wait(P.p)) + (size_t)(row0 + lane) * P.ldp;
            const float a = ng_ld(row + P.off_a + head) + P.dt_bias[head], bb = ng_ld(row + P.off_b + head);
            const float sp = a > 20.f ? a : log1pf(expf(a));
            b = 1.f / (1.f + expf(-bb));
            lg = -expf(P.a_log[head]) * sp;
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, lg, o);
            if (lane >= o) lg += v;
        }
        cl[lane] = lg;
        bt[lane] = b;
        P.cl[slot * GC + lane] = lg;
    }
    __syncthreads();
    {   // A: a 2 x 4 tile per thread
        const int i0 = (tid / 8) * 2, j0 = (tid % 8) * 4;
        float a[2][4] = {};
        if (j0 <= i0) {
            for (int d = 0; d < dk; ++d) {
                const float ka = Ks[i0 * ldk + d], kb = Ks[(i0 + 1) * ldk + d];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const float kv = Ks[(j0 + cc) * ldk + d];
                    a[0][cc] = fmaf(ka, kv, a[0][cc]);
                    a[1][cc] = fmaf(kb, kv, a[1][cc]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int i = i0 + r, j = j0 + cc;
                As[i * GC + j] = j < i ? a[r][cc] * bt[i] * expf(cl[i] - cl[j]) : 0.f;
            }
    }
    __syncthreads();
    // K~ for the state's update
    const float last = cl[GC - 1];
    float* kt = P.kt + slot * GC * dk;
    for (int idx = tid; idx < GC * dk; idx += GC_THREADS) {
        const int t = idx / dk, i = idx - t * dk;
        kt[idx] = Ks[t * ldk + i] * expf(last - cl[t]);
    }
    // the two systems, a column per thread: x_t = rhs_t - sum_(s<t) A[t][s] x_s
    float* wt = P.wt + slot * dk * GC;
    for (int col = tid; col < dk + dv; col += GC_THREADS) {
        const bool isk = col < dk;
        float x[GC];
#pragma unroll
        for (int t = 0; t < GC; ++t) {
            float acc;
            if (isk) acc = bt[t] * expf(cl[t]) * Ks[t * ldk + col];
            else acc = bt[t] * Vs[t * dv + (col - dk)];
#pragma unroll
            for (int s4 = 0; s4 < (t & ~3); s4 += 4) {
                const float4 av = *reinterpret_cast<const float4*>(As + t * GC + s4);
                acc = fmaf(-av.x, x[s4], acc);
                acc = fmaf(-av.y, x[s4 + 1], acc);
                acc = fmaf(-av.z, x[s4 + 2], acc);
                acc = fmaf(-av.w, x[s4 + 3], acc);
            }
#pragma unroll
            for (int s = (t & ~3); s < t; ++s) acc = fmaf(-As[t * GC + s], x[s], acc);
            x[t] = acc;
        }
        if (isk) {
#pragma unroll
            for (int t = 0; t < GC; t += 4)
                *reinterpret_cast<float4*>(wt + (size_t)col * GC + t) = make_float4(x[t], x[t + 1], x[t + 2], x[t + 3]);
        } else {
            float* dst = P.o_raw + (size_t)row0 * nH * dv + (size_t)head * dv + (col - dk);
#pragma unroll
            for (int t = 0; t < GC; ++t)
                if (t < n) dst[(size_t)t * nH * dv] = x[t];
        }
    }
}

__device__ __forceinline__ void gc_copy16(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void gc_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void gc_copy_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// NT: 4 x 2 tiles of the state's slice [dk][GC_DVS] a thread keeps in registers (ceil(dk / 4 * (GC_DVS / 2) / GS_THREADS))
template <int NT>
__global__ void __launch_bounds__(GS_THREADS)
gd_chunk_scan_kernel(const GcParams P) {
    extern __shared__ float4 sm_aligned[];
    float* sm = reinterpret_cast<float*>(sm_aligned);
    const int dk = P.dk, dv = P.dv, nH = P.nH;
    const int per = 2 * GC * dk + GC * GC_DVS;       // a chunk's tiles: W^T [dk][GC], K~ [GC][dk], U' [GC][GC_DVS]
    float* tiles = sm;                               // two of them
    float* Ss = tiles + 2 * per;                     // [dk][GC_DVS]
    float* Us = Ss + dk * GC_DVS;                    // [GC][GC_DVS]
    float* red = Us + GC * GC_DVS;                   // [warps][32 lanes][GC_RED]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int v0 = blockIdx.x * GC_DVS, head = blockIdx.y, e = blockIdx.z;
    const int q0 = P.cu_q[e], qlen = P.cu_q[e + 1] - q0;
    if (qlen <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nc = (qlen + GC - 1) / GC;
    const size_t slot0 = (size_t)(q0 / GC + e) * nH + head;
    float* u_all = ng_after_wait(P.o_raw) + (size_t)q0 * nH * dv + (size_t)head * dv + v0;
    const float* wt_all = ng_after_wait(P.wt);
    const float* kt_all = ng_after_wait(P.kt);
    const float* cl_all = ng_after_wait(P.cl);
    float* St = P.state + ((size_t)P.slots[e] * nH + head) * dk * dv + v0;
    const bool carried = P.ctx_before[e] > 0;
    const int cg2 = (tid & 7) * 2;                   // the thread's two value columns of the state and of U
    const int cg4 = (lane & 3) * 4;                  // its four columns in W S
    float s[NT][4][2];
#pragma unroll
    for (int m = 0; m < NT; ++m) {
        const int i0 = ((tid + m * GS_THREADS) >> 3) * 4;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float2 v = make_float2(0.f, 0.f);
            if (carried && i0 + r < dk) v = *reinterpret_cast<const float2*>(St + (size_t)(i0 + r) * dv + cg2);
            s[m][r][0] = v.x, s[m][r][1] = v.y;
            if (i0 + r < dk) *reinterpret_cast<float2*>(Ss + (i0 + r) * GC_DVS + cg2) = v;
        }
    }
    auto fetch = [&](int c) {
        float* dst = tiles + (c & 1) * per;
        const size_t slot = slot0 + (size_t)c * nH;
        const float* w = wt_all + slot * dk * GC;
        const float* k = kt_all + slot * GC * dk;
        for (int idx = tid * 4; idx < GC * dk; idx += GS_THREADS * 4) {
            gc_copy16(dst + idx, w + idx);
            gc_copy16(dst + GC * dk + idx, k + idx);
        }
        const int n = min(GC, qlen - c * GC);
        float* up = dst + 2 * GC * dk;
        for (int idx = tid; idx < GC * (GC_DVS / 4); idx += GS_THREADS) {
            const int t = idx / (GC_DVS / 4), c4 = (idx % (GC_DVS / 4)) * 4;
            if (t < n) gc_copy16(up + t * GC_DVS + c4, u_all + (size_t)(c * GC + t) * nH * dv + c4);
            else *reinterpret_cast<float4*>(up + t * GC_DVS + c4) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        gc_copy_commit();
    };
    fetch(0);
    const int dkq = (dk + GS_THREADS / 32 - 1) / (GS_THREADS / 32);     // a warp's share of the rows of S in U = U' - W S
    for (int c = 0; c < nc; ++c) {
        gc_copy_wait();
        __syncthreads();                             // chunk c's tiles and the state's slice are in shared memory
        if (c + 1 < nc) fetch(c + 1);
        const float* Wt = tiles + (c & 1) * per;
        const float* Kt = Wt + GC * dk;
        const float* Up = Kt + GC * dk;
        const size_t slot = slot0 + (size_t)c * nH;
        const float last = cl_all[slot * GC + GC - 1];      // asked for here, used after the first product
        float* sb = P.sb + slot * dk * dv + v0;
#pragma unroll
        for (int m = 0; m < NT; ++m) {
            const int i0 = ((tid + m * GS_THREADS) >> 3) * 4;
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (i0 + r < dk) *reinterpret_cast<float2*>(sb + (size_t)(i0 + r) * dv + cg2) = make_float2(s[m][r][0], s[m][r][1]);
        }
        {   // W S: warp w takes rows w*dkq .. of S, lane (t group, column group) a 4 x 4 tile of the product
            const int t0 = (lane >> 2) * 4;
            float acc[4][4] = {};
            const int i1 = min(dk, (warp + 1) * dkq);
#pragma unroll 4
            for (int i = warp * dkq; i < i1; ++i) {
                const float4 w4 = *reinterpret_cast<const float4*>(Wt + i * GC + t0);
                const float4 s4 = *reinterpret_cast<const float4*>(Ss + i * GC_DVS + cg4);
                const float wv[4] = {w4.x, w4.y, w4.z, w4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) acc[r][cc] = fmaf(wv[r], sv[cc], acc[r][cc]);
            }
            float* dst = red + (warp * 32 + lane) * GC_RED;
#pragma unroll
            for (int r = 0; r < 4; ++r) *reinterpret_cast<float4*>(dst + r * 4) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        }
        __syncthreads();
        {   // U = U' - (the warps' parts, in ascending order): thread -> token tid / 8, its two columns
            const int t = tid >> 3;
            float2 u = *reinterpret_cast<const float2*>(Up + t * GC_DVS + cg2);
            float2 a = make_float2(0.f, 0.f);
#pragma unroll
            for (int w = 0; w < GS_THREADS / 32; ++w) {
                const float2 x = *reinterpret_cast<const float2*>(red + (w * 32 + (t >> 2) * 4 + (cg2 >> 2)) * GC_RED + (t & 3) * 4 + (cg2 & 3));
                a.x += x.x, a.y += x.y;
            }
            u.x -= a.x, u.y -= a.y;
            *reinterpret_cast<float2*>(Us + t * GC_DVS + cg2) = u;
            if (c * GC + t < qlen) *reinterpret_cast<float2*>(u_all + (size_t)(c * GC + t) * nH * dv + cg2) = u;
        }
        __syncthreads();
        const float gam = expf(last);
#pragma unroll
        for (int m = 0; m < NT; ++m) {
            const int i0 = ((tid + m * GS_THREADS) >> 3) * 4;
            if (i0 < dk) {
#pragma unroll
                for (int r = 0; r < 4; ++r) s[m][r][0] *= gam, s[m][r][1] *= gam;
#pragma unroll 4
                for (int t = 0; t < GC; ++t) {
                    const float4 k4 = *reinterpret_cast<const float4*>(Kt + t * dk + i0);
                    const float2 u2 = *reinterpret_cast<const float2*>(Us + t * GC_DVS + cg2);
                    const float kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        s[m][r][0] = fmaf(kv[r], u2.x, s[m][r][0]);
                        s[m][r][1] = fmaf(kv[r], u2.y, s[m][r][1]);
                    }
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) *reinterpret_cast<float2*>(Ss + (i0 + r) * GC_DVS + cg2) = make_float2(s[m][r][0], s[m][r][1]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < NT; ++m) {
        const int i0 = ((tid + m * GS_THREADS) >> 3) * 4;
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (i0 + r < dk) *reinterpret_cast<float2*>(St + (size_t)(i0 + r) * dv + cg2) = make_float2(s[m][r][0], s[m][r][1]);
    }
}

// rows of unit vectors, transposed, into shared memory [dk][GC_LDT] (dst[i][t] = x_t[i]): a warp takes four rows at
// a time, a lane every 32nd coordinate of each; the rows' sums of squares first, then the rows again (from L1), scaled,
// four tokens of a coordinate in one 16-byte store; rows past n are zero.  Ends with the block in step.
__device__ __forceinline__ void gc_load_unit_t(const float* __restrict__ src, size_t ld, int n, int dk, float mul, float* dst) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int t0 = warp * 4; t0 < GC; t0 += (GC_THREADS / 32) * 4) {
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = lane; i < dk; i += 32) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float x = t0 + r < n ? src[(size_t)(t0 + r) * ld + i] : 0.f;
                ss[r] = fmaf(x, x, ss[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) ss[r] = rsqrtf(ng_warp_sum(ss[r]) + 1e-6f) * mul;
        for (int i = lane; i < dk; i += 32) {
            float x[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) x[r] = t0 + r < n ? src[(size_t)(t0 + r) * ld + i] * ss[r] : 0.f;
            *reinterpret_cast<float4*>(dst + i * GC_LDT + t0) = make_float4(x[0], x[1], x[2], x[3]);
        }
    }
    __syncthreads();
}

// A block per chunk and head.  q and k lie transposed in shared memory, so that a thread's eight tokens of a coordinate
// are two 16-byte reads; the state before the chunk and U are read from global memory as they are needed (a warp
// reads whole rows' segments), four value columns a thread.  U's place is overwritten with o, so a pass of tiles
// (all eight-token groups of its columns) is read whole before any of it is written.
__global__ void __launch_bounds__(GC_THREADS)
gd_chunk_out_kernel(const GcParams P) {
    extern __shared__ float4 sm_aligned[];
    float* sm = reinterpret_cast<float*>(sm_aligned);
    const int dk = P.dk, dv = P.dv, nH = P.nH;
    float* Qt = sm;                        // [dk][GC_LDT]
    float* Kt = Qt + dk * GC_LDT;          // [dk][GC_LDT]
    float* Pt = Kt + dk * GC_LDT;          // [GC][GC_LDT]: Pt[j][i] = exp(cl_i - cl_j) (q_i . k_j), j <= i
    float* cl = Pt + GC * GC_LDT;          // [GC]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int c = blockIdx.x, head = blockIdx.y, e = blockIdx.z;
    const int q0 = P.cu_q[e], qlen = P.cu_q[e + 1] - q0;
    if (c * GC >= qlen) return;
    const int n = min(GC, qlen - c * GC), row0 = q0 + c * GC;
    const size_t slot = (size_t)(q0 / GC + e + c) * nH + head;
    const int tid = threadIdx.x;
    const int C = 2 * P.nG * dk + nH * dv;
    const size_t off_q = (size_t)(head / (nH / P.nG)) * dk, off_k = (size_t)P.nG * dk + off_q;
    const float* conv = ng_after_wait(P.conv) + (size_t)row0 * C;
    if (tid < GC) cl[tid] = ng_after_wait(P.cl)[slot * GC + tid];
    gc_load_unit_t(conv + off_q, C, n, dk, rsqrtf((float)dk), Qt);
    gc_load_unit_t(conv + off_k, C, n, dk, 1.f, Kt);
    {   // scores inside the chunk: four queries x two keys a thread
        const int i4 = (tid & 7) * 4, j2 = (tid >> 3) * 2;
        float a[2][4] = {};
        if (j2 <= i4 + 3) {
#pragma unroll 4
            for (int d = 0; d < dk; ++d) {
                const float4 q4 = *reinterpret_cast<const float4*>(Qt + d * GC_LDT + i4);
                const float2 k2 = *reinterpret_cast<const float2*>(Kt + d * GC_LDT + j2);
                const float qv[4] = {q4.x, q4.y, q4.z, q4.w}, kv[2] = {k2.x, k2.y};
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) a[r][cc] = fmaf(kv[r], qv[cc], a[r][cc]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int j = j2 + r;
            float w[4];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) w[cc] = j <= i4 + cc ? a[r][cc] * expf(cl[i4 + cc] - cl[j]) : 0.f;
            *reinterpret_cast<float4*>(Pt + j * GC_LDT + i4) = make_float4(w[0], w[1], w[2], w[3]);
        }
    }
    __syncthreads();
    const float* sb = ng_after_wait(P.sb) + slot * dk * dv;
    float* o = ng_after_wait(P.o_raw) + (size_t)row0 * nH * dv + (size_t)head * dv;
    const size_t ldo = (size_t)nH * dv;
    for (int base = 0; base < dv; base += GC_THREADS) {      // dv tiles: (dv / 4 column groups) x (four groups of eight tokens)
        const int tile = base + tid, t8 = (tile & 3) * 8, c0 = (tile >> 2) * 4;
        const bool active = c0 < dv;
        float acc[8][4] = {};
        if (active) {
#pragma unroll 4
            for (int d = 0; d < dk; ++d) {       // from the state: Q S
                const float4 s4 = *reinterpret_cast<const float4*>(sb + (size_t)d * dv + c0);
                const float4 qa = *reinterpret_cast<const float4*>(Qt + d * GC_LDT + t8);
                const float4 qb = *reinterpret_cast<const float4*>(Qt + d * GC_LDT + t8 + 4);
                const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                for (int r = 0; r < 8; ++r)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) acc[r][cc] = fmaf(qv[r], sv[cc], acc[r][cc]);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float g = expf(cl[t8 + r]);
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) acc[r][cc] *= g;
            }
            const int j1 = min(n, t8 + 8);       // inside the chunk: P U, the keys up to the group's last token
#pragma unroll 4
            for (int j = 0; j < j1; ++j) {
                const float4 u4 = *reinterpret_cast<const float4*>(o + (size_t)j * ldo + c0);
                const float4 pa = *reinterpret_cast<const float4*>(Pt + j * GC_LDT + t8);
                const float4 pb = *reinterpret_cast<const float4*>(Pt + j * GC_LDT + t8 + 4);
                const float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w}, uv[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                for (int r = 0; r < 8; ++r)
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) acc[r][cc] = fmaf(pv[r], uv[cc], acc[r][cc]);
            }
        }
        __syncthreads();                         // every read of this pass's columns of U is done
        if (active) {
#pragma unroll
            for (int r = 0; r < 8; ++r)
                if (t8 + r < n)
                    *reinterpret_cast<float4*>(o + (size_t)(t8 + r) * ldo + c0) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        }
    }
}

static inline size_t gc_prep_smem(int dk, int dv) { return ((size_t)GC * (dk + 1) + GC * GC + 2 * GC + GC * dv) * sizeof(float); }
static inline size_t gc_scan_smem(int dk) {
    return ((size_t)2 * (2 * GC * dk + GC * GC_DVS) + dk * GC_DVS + GC * GC_DVS + GS_THREADS * GC_RED) * sizeof(float);
}
static inline size_t gc_out_smem(int dk) { return ((size_t)2 * dk * GC_LDT + GC * GC_LDT + GC) * sizeof(float); }

// Whether the chunked kernels take these head sizes: key rows in fours, at most 256; value columns in sixteens.
NG_EXPORT int ng_gd_chunked_takes(int dk, int dv) {
    return dk > 0 && dk % 4 == 0 && dk <= 256 && dv > 0 && dv % GC_DVS == 0;
}

// float32 values of the chunked kernels' scratch for a step of n_rows rows in n_entries entries
NG_EXPORT long long ng_gd_chunked_scratch(int n_rows, int n_entries, int nH, int dk, int dv) {
    return ((long long)n_rows / GC + n_entries + 1) * nH * ((long long)2 * GC * dk + GC + (long long)dk * dv);
}

// As ng_gated_delta for steps with long portions; `scratch`: ng_gd_chunked_scratch float32 values, 16-byte aligned.
NG_EXPORT int ng_gated_delta_chunked(const float* conv, const void* p, int ldp, int off_a, int off_b, const float* a_log,
                                     const float* dt_bias, float* state, float* o_raw, float* scratch, const int* cu_q,
                                     const int* ctx_before, const int* slots, int n_entries, int n_rows, int max_q, int nH,
                                     int nG, int dk, int dv, int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0 || n_rows <= 0 || max_q <= 0) return NG_OK;
    if (nH <= 0 || nG <= 0 || nH % nG || !ng_gd_chunked_takes(dk, dv) || !scratch || ((uintptr_t)scratch & 15) ||
        ((uintptr_t)o_raw & 15) || ((uintptr_t)state & 15) || ((uintptr_t)conv & 15))
        return NG_BAD_SIZE;
    const size_t n_slots = (size_t)n_rows / GC + n_entries + 1;
    GcParams P;
    P.conv = conv, P.p = p, P.ldp = ldp, P.off_a = off_a, P.off_b = off_b, P.a_log = a_log, P.dt_bias = dt_bias;
    P.state = state, P.o_raw = o_raw;
    P.wt = scratch;
    P.kt = P.wt + n_slots * nH * GC * dk;
    P.cl = P.kt + n_slots * nH * GC * dk;
    P.sb = P.cl + n_slots * nH * GC;
    P.cu_q = cu_q, P.ctx_before = ctx_before, P.slots = slots;
    P.nH = nH, P.nG = nG, P.dk = dk, P.dv = dv;
    const size_t sp = gc_prep_smem(dk, dv), ss = gc_scan_smem(dk), so = gc_out_smem(dk);
    static bool configured = false;
    if (!configured) {
        const int cap = 200 * 1024;
        if (cudaFuncSetAttribute(gd_chunk_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
            cudaFuncSetAttribute(gd_chunk_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
            cudaFuncSetAttribute(gd_chunk_scan_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
            cudaFuncSetAttribute(gd_chunk_scan_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess ||
            cudaFuncSetAttribute(gd_chunk_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, cap) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        configured = true;
    }
    if (sp > 200 * 1024 || ss > 200 * 1024 || so > 200 * 1024) return NG_BAD_SIZE;
    const unsigned chunks = (unsigned)((max_q + GC - 1) / GC);
    dim3 pgrid(chunks, nH, n_entries), sgrid(dv / GC_DVS, nH, n_entries), ogrid(chunks, nH, n_entries);
    if (nH > 65535 || n_entries > 65535) return NG_BAD_SIZE;
    if (act_bf16) NG_LAUNCH((gd_chunk_prep_kernel<__nv_bfloat16>), pgrid, GC_THREADS, sp, stream, P);
    else NG_LAUNCH((gd_chunk_prep_kernel<float>), pgrid, GC_THREADS, sp, stream, P);
    if (dk <= 128) NG_LAUNCH((gd_chunk_scan_kernel<1>), sgrid, GS_THREADS, ss, stream, P);
    else NG_LAUNCH((gd_chunk_scan_kernel<2>), sgrid, GS_THREADS, ss, stream, P);
    NG_LAUNCH(gd_chunk_out_kernel, ogrid, GC_THREADS, so, stream, P);
    return ng_launch_status();
}
