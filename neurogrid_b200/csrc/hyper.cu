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

// S > 0: the number of copies is a compile-time constant and every loop over them is unrolled (the copies of a column
// live in registers); S == 0: any number up to HC_MAX_STREAMS, read from `S_rt`.  A thread takes VEC (1 or 4) neighbouring
// columns at a time.
template <typename TD, typename TO, int S_CT, int VEC>
__global__ void __launch_bounds__(512)
hc_step_kernel(float* __restrict__ X, const float* __restrict__ x0, const TD* __restrict__ delta, int n_partials,
               size_t partial_stride, const float* __restrict__ mix, const float* __restrict__ out_w,
               const float* __restrict__ in_w, const float* __restrict__ norm_w, TO* __restrict__ out,
               float* __restrict__ sum_out, int S_rt, int H, float eps) {
    extern __shared__ float u_s[];                     // [H]: what the next sublayer reads, before its norm
    __shared__ float red[32];
    __shared__ float mix_s[HC_MAX_STREAMS * HC_MAX_STREAMS], ow_s[HC_MAX_STREAMS], iw_s[HC_MAX_STREAMS];
    constexpr int SM = S_CT > 0 ? S_CT : HC_MAX_STREAMS;
    const int S = S_CT > 0 ? S_CT : S_rt;
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
    for (int j = threadIdx.x * VEC; j < H; j += blockDim.x * VEC) {
        float xs[SM][VEC];
        if (x0) {
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                const float t = x0[row * H + j + v];
#pragma unroll
                for (int s = 0; s < SM; ++s) xs[s][v] = t;
            }
        } else {
#pragma unroll
            for (int s = 0; s < SM; ++s) {
                if (s < S) {
                    if (VEC == 4) {
                        const float4 t = *reinterpret_cast<const float4*>(xr + (size_t)s * H + j);
                        xs[s][0] = t.x; xs[s][1 % VEC] = t.y; xs[s][2 % VEC] = t.z; xs[s][3 % VEC] = t.w;
                    } else {
                        xs[s][0] = xr[(size_t)s * H + j];
                    }
                } else {
#pragma unroll
                    for (int v = 0; v < VEC; ++v) xs[s][v] = 0.f;
                }
            }
        }
        if (delta) {
            float y[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) {
                y[v] = 0.f;
                for (int p = 0; p < n_partials; ++p) y[v] += ng_ld(delta + p * partial_stride + row * H + j + v);   // ascending p
            }
            float nx[SM][VEC];
#pragma unroll
            for (int t = 0; t < SM; ++t) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < SM; ++s)
                        if (s < S && t < S) a = fmaf(mix_s[s * S + t], xs[s][v], a);
                    nx[t][v] = t < S ? fmaf(ow_s[t], y[v], a) : 0.f;
                }
            }
#pragma unroll
            for (int t = 0; t < SM; ++t)
#pragma unroll
                for (int v = 0; v < VEC; ++v) xs[t][v] = nx[t][v];
        }
        if (delta || x0) {
#pragma unroll
            for (int s = 0; s < SM; ++s) {
                if (s < S) {
                    if (VEC == 4)
                        *reinterpret_cast<float4*>(xr + (size_t)s * H + j) = make_float4(xs[s][0], xs[s][1 % VEC], xs[s][2 % VEC], xs[s][3 % VEC]);
                    else
                        xr[(size_t)s * H + j] = xs[s][0];
                }
            }
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
            if (in_w) {
                float u = 0.f;
#pragma unroll
                for (int s = 0; s < SM; ++s)
                    if (s < S) u = fmaf(iw_s[s], xs[s][v], u);
                u_s[j + v] = u;
                ss = fmaf(u, u, ss);
            }
            if (sum_out) {
                float t = 0.f;
#pragma unroll
                for (int s = 0; s < SM; ++s)
                    if (s < S) t += xs[s][v];
                sum_out[row * H + j + v] = t;
            }
        }
    }
    if (!in_w) return;
    ss = ng_block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    // each thread re-reads exactly the elements it wrote itself
    for (int j = threadIdx.x * VEC; j < H; j += blockDim.x * VEC)
#pragma unroll
        for (int v = 0; v < VEC; ++v) ng_st(out + row * H + j + v, u_s[j + v] * r * norm_w[j + v]);
}

template <typename TD, typename TO, int S_CT, int VEC>
static int hc_launch(float* X, const float* x0, const void* delta, int n_partials, size_t ps, const float* mix,
                     const float* out_w, const float* in_w, const float* norm_w, void* out, float* sum_out, int n_rows, int S,
                     int H, float eps, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(hc_step_kernel<TD, TO, S_CT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) !=
            cudaSuccess)
            return NG_LAUNCH_FAILED;
        configured = true;
    }
    const size_t smem = in_w ? (size_t)H * sizeof(float) : 0;
    // few rows: a row's columns are dealt to many threads (the launch is a chain of loads otherwise)
    const int per = (H + VEC - 1) / VEC;
    int threads = n_rows <= 64 ? 512 : 256;
    while (threads > 64 && threads / 2 >= per) threads /= 2;
    NG_LAUNCH((hc_step_kernel<TD, TO, S_CT, VEC>), n_rows, threads, smem, stream, X, x0, (const TD*)delta, n_partials, ps, mix,
              out_w, in_w, norm_w, (TO*)out, sum_out, S, H, eps);
    return ng_launch_status();
}

template <typename TD, typename TO>
static int hc_by_streams(float* X, const float* x0, const void* delta, int n_partials, size_t ps, const float* mix,
                         const float* out_w, const float* in_w, const float* norm_w, void* out, float* sum_out, int n_rows, int S,
                         int H, float eps, cudaStream_t stream) {
    const bool vec = H % 4 == 0 && ((uintptr_t)X & 15) == 0;
#define HC_CASE(SS)                                                                                                    \
    case SS:                                                                                                           \
        return vec ? hc_launch<TD, TO, SS, 4>(X, x0, delta, n_partials, ps, mix, out_w, in_w, norm_w, out, sum_out, n_rows, S, H, eps, stream) \
                   : hc_launch<TD, TO, SS, 1>(X, x0, delta, n_partials, ps, mix, out_w, in_w, norm_w, out, sum_out, n_rows, S, H, eps, stream);
    switch (S) {
        HC_CASE(1) HC_CASE(2) HC_CASE(3) HC_CASE(4) HC_CASE(5) HC_CASE(6) HC_CASE(7) HC_CASE(8)
        default:
            return hc_launch<TD, TO, 0, 1>(X, x0, delta, n_partials, ps, mix, out_w, in_w, norm_w, out, sum_out, n_rows, S, H, eps, stream);
    }
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
    const size_t ps = (size_t)partial_stride;
    if (act_bf16 && delta_f32)
        return hc_by_streams<float, __nv_bfloat16>(X, x0, delta, n_partials, ps, mix, out_w, in_w, norm_w, out, sum_out, n_rows, S, H, eps, stream);
    if (act_bf16)
        return hc_by_streams<__nv_bfloat16, __nv_bfloat16>(X, x0, delta, 1, 0, mix, out_w, in_w, norm_w, out, sum_out, n_rows, S, H, eps, stream);
    return hc_by_streams<float, float>(X, x0, delta, delta_f32 ? n_partials : 1, ps, mix, out_w, in_w, norm_w, out, sum_out, n_rows, S, H, eps, stream);
}
