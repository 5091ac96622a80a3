// Hyper-connections: the residual stream kept as S copies ("streams") that every sublayer reads through a weighted
// sum and writes through a mixing matrix.
//
// One kernel does what lies between two sublayers, a block per row, all float32:
//   1. the streams x_1..x_S of the row are read (X [n, S, H]); with `x0` given they are all x0 (a sequence's start:
//      every stream holds the embedding output) and are written out as such;
//   2. with `delta` (the output y of the sublayer before: [n, H] of the activation type, or float32 partial sums that
//      are added in ascending order) all streams are replaced at once from the old ones,
//          x_t <- sum_s mix[s, t] x_s + out_w[t] * y            (mix is indexed [from, to]);
//   3. with `in_w`: u = sum_t in_w[t] x_t is what the next sublayer reads, and `out` receives
//      u / sqrt(mean(u^2) + eps) * norm_w in the activation type (one rounding);
//   4. with `sum_out`: the sum of the streams (float32 [n, H]), which is what the model's last norm reads.
#include "ng_common.cuh"

#define HC_MAX_STREAMS 16

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
hc_step_kernel(float* __restrict__ X, const float* __restrict__ x0, const TD* __restrict__ delta, int n_partials,
               size_t partial_stride, const float* __restrict__ mix, const float* __restrict__ out_w,
               const float* __restrict__ in_w, const float* __restrict__ norm_w, TO* __restrict__ out,
               float* __restrict__ sum_out, int S, int H, float eps) {
    extern __shared__ float u_s[];                     // [H]: what the next sublayer reads, before its norm
    __shared__ float red[32];
    __shared__ float mix_s[HC_MAX_STREAMS * HC_MAX_STREAMS], ow_s[HC_MAX_STREAMS], iw_s[HC_MAX_STREAMS];
    ng_pdl_trigger();
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = delta ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        ow_s[i] = delta ? out_w[i] : 0.f;
        iw_s[i] = in_w ? in_w[i] : 0.f;
    }
    __syncthreads();
    ng_pdl_wait();
    delta = ng_after_wait(delta);
    x0 = ng_after_wait(x0);
    const size_t row = blockIdx.x;
    float* xr = X + row * (size_t)S * H;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float xs[HC_MAX_STREAMS];
        if (x0) {
            const float v = x0[row * H + j];
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s) xs[s] = v;
        } else {
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s) xs[s] = s < S ? xr[(size_t)s * H + j] : 0.f;
        }
        if (delta) {
            float y = 0.f;
            for (int p = 0; p < n_partials; ++p) y += ng_ld(delta + p * partial_stride + row * H + j);   // ascending p
            float nx[HC_MAX_STREAMS];
#pragma unroll
            for (int t = 0; t < HC_MAX_STREAMS; ++t) {
                float a = 0.f;
                if (t < S) {
#pragma unroll
                    for (int s = 0; s < HC_MAX_STREAMS; ++s)
                        if (s < S) a = fmaf(mix_s[s * S + t], xs[s], a);
                    a = fmaf(ow_s[t], y, a);
                }
                nx[t] = a;
            }
#pragma unroll
            for (int t = 0; t < HC_MAX_STREAMS; ++t) xs[t] = nx[t];
        }
        if (delta || x0) {
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) xr[(size_t)s * H + j] = xs[s];
        }
        if (in_w) {
            float u = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) u = fmaf(iw_s[s], xs[s], u);
            u_s[j] = u;
            ss = fmaf(u, u, ss);
        }
        if (sum_out) {
            float t = 0.f;
#pragma unroll
            for (int s = 0; s < HC_MAX_STREAMS; ++s)
                if (s < S) t += xs[s];
            sum_out[row * H + j] = t;
        }
    }
    if (!in_w) return;
    ss = ng_block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    // each thread re-reads exactly the elements it wrote itself
    for (int j = threadIdx.x; j < H; j += blockDim.x) ng_st(out + row * H + j, u_s[j] * r * norm_w[j]);
}

// delta: null, one [n, H] tensor of the activation type, or (delta_f32) n_partials float32 tensors [n, H] that lie
// partial_stride elements apart.  x0, in_w (with norm_w and out) and sum_out are optional; mix and out_w go with delta.
NG_EXPORT int ng_hc_step(float* X, const float* x0, const void* delta, int delta_f32, int n_partials,
                         long long partial_stride, const float* mix, const float* out_w, const float* in_w,
                         const float* norm_w, void* out, float* sum_out, int n_rows, int S, int H, float eps, int act_bf16,
                         cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (S < 1 || S > HC_MAX_STREAMS || H <= 0 || n_partials < 1 || (delta && (!mix || !out_w)) || (in_w && (!norm_w || !out)) ||
        (size_t)H * sizeof(float) > 160 * 1024)
        return NG_BAD_SIZE;
    const size_t smem = in_w ? (size_t)H * sizeof(float) : 0;
    const int threads = H >= 1024 ? 256 : 128;
    const size_t ps = (size_t)partial_stride;
#define HC_LAUNCH(TD, TO, NP, PS)                                                                                      \
    {                                                                                                                  \
        static bool configured = false;                                                                                \
        if (!configured) {                                                                                             \
            if (cudaFuncSetAttribute(hc_step_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024)  \
                != cudaSuccess)                                                                                        \
                return NG_LAUNCH_FAILED;                                                                               \
            configured = true;                                                                                         \
        }                                                                                                              \
        NG_LAUNCH((hc_step_kernel<TD, TO>), n_rows, threads, smem, stream, X, x0, (const TD*)delta, NP, PS, mix, out_w, \
                  in_w, norm_w, (TO*)out, sum_out, S, H, eps);                                                         \
    }
    if (act_bf16 && delta_f32) HC_LAUNCH(float, __nv_bfloat16, n_partials, ps)
    else if (act_bf16) HC_LAUNCH(__nv_bfloat16, __nv_bfloat16, 1, 0)
    else HC_LAUNCH(float, float, (delta_f32 ? n_partials : 1), ps)
    return ng_launch_status();
}
