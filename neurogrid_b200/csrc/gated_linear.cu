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
