// Routed experts: the router and the weighting of the experts' activations.
//
// moe_router: logits z = W_r x + b in float32 (x is the activation row, W_r and b float32); the top_k
//   experts with the largest logits are chosen (of equal logits the lower index) and weighted by the
//   softmax over the chosen logits.  Output: dense weights [n_rows, n_experts] float32, zero for the
//   experts a row does not use.
// moe_scale: act[row, e*ff + j] *= weights[row, e] for the first n_experts*ff columns of an activation
//   row of width ld (what lies behind them, a shared expert's columns, stays as it is).  With the
//   weights applied, one product with all experts' down projections side by side is the weighted sum.
#include "ng_common.cuh"

#define MOE_MAX_TOP 32

__device__ __forceinline__ float4 moe_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 moe_ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

template <typename T>
__global__ void __launch_bounds__(512)
moe_router_kernel(const T* __restrict__ x, const float* __restrict__ wr, const float* __restrict__ br,
                  float* __restrict__ weights, int H, int E, int top_k) {
    extern __shared__ float z[];               // [E]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const T* xr = x + (size_t)row * H;
    for (int e = warp; e < E; e += nwarp) {
        const float* w = wr + (size_t)e * H;
        float acc = 0.f;
        if (H % 4 == 0) {                           // four columns a lane and load; the order depends on H alone
#pragma unroll 4
            for (int i = lane * 4; i < H; i += 128) {
                const float4 xv = moe_ld4(xr + i), wv = moe_ld4(w + i);
                acc = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc))));
            }
        } else {
            for (int i = lane; i < H; i += 32) acc = fmaf(ng_ld(xr + i), w[i], acc);
        }
        acc = ng_warp_sum(acc);
        if (lane == 0) z[e] = acc + (br ? br[e] : 0.f);
    }
    __syncthreads();
    float* out = weights + (size_t)row * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) out[e] = 0.f;
    __syncthreads();
    if (threadIdx.x == 0) {
        int idx[MOE_MAX_TOP];
        float val[MOE_MAX_TOP];
        for (int k = 0; k < top_k; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                const float v = z[e];
                if (best < 0 || v > bv) {
                    bool taken = false;
                    for (int m = 0; m < k; ++m) taken |= idx[m] == e;
                    if (!taken) { best = e; bv = v; }
                }
            }
            idx[k] = best;
            val[k] = bv;
        }
        float sum = 0.f;
        const float top = val[0];               // the largest
        for (int k = 0; k < top_k; ++k) {
            val[k] = expf(val[k] - top);
            sum += val[k];
        }
        for (int k = 0; k < top_k; ++k) out[idx[k]] = val[k] / sum;
    }
}

template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, const float* __restrict__ weights, int n_rows, int E, int ff, int ld,
                                 int ldw, int cols) {
    // columns behind E*ff (a shared expert's) are reached only when its gate, weights[row, E], multiplies them
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    T* p = act + (size_t)row * ld + c;
    ng_st(p, ng_ld(p) * weights[(size_t)row * ldw + (c < E * ff ? c / ff : E)]);
}

// out[row, c] = silu(gate_up[row, c]) * gate_up[row, I + c] * (c < E*ff ? weights[row, c / ff] : 1): the SwiGLU of all
// experts side by side with the routing weight applied at once (steps whose gate/up product has no fused epilogue).
// `shared_gated`: the columns behind E*ff (a shared expert's) are multiplied by weights[row, E].  Rows of `weights`
// lie ldw apart.
template <typename T>
__global__ void moe_swiglu_scaled_kernel(const T* __restrict__ gate_up, const float* __restrict__ weights,
                                         T* __restrict__ out, int I, int E, int ff, int ldw, int shared_gated) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= I) return;
    const float g = ng_ld(gate_up + (size_t)row * 2 * I + c), u = ng_ld(gate_up + (size_t)row * 2 * I + I + c);
    T act;
    ng_st(&act, g / (1.f + expf(-g)) * u);           // rounded as the unweighted activation is, then weighted
    const float w = c < E * ff ? weights[(size_t)row * ldw + c / ff] : (shared_gated ? weights[(size_t)row * ldw + E] : 1.f);
    ng_st(out + (size_t)row * I + c, ng_ld(&act) * w);
}

// the same, eight columns a thread with 16-byte accesses (bfloat16; I and ff multiples of 8, so that the eight share an expert)
__global__ void moe_swiglu_scaled_vec_kernel(const __nv_bfloat16* __restrict__ gate_up, const float* __restrict__ weights,
                                             __nv_bfloat16* __restrict__ out, int I, int E, int ff, int ldw, int shared_gated) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= I) return;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + (size_t)row * 2 * I + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + (size_t)row * 2 * I + I + c);
    const float w = c < E * ff ? weights[(size_t)row * ldw + c / ff] : (shared_gated ? weights[(size_t)row * ldw + E] : 1.f);
    const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(&gv);
    const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&uv);
    uint4 ov;
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(&ov);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float gk = __bfloat162float(g[k]);
        const __nv_bfloat16 act = __float2bfloat16_rn(gk / (1.f + expf(-gk)) * __bfloat162float(u[k]));
        o[k] = __float2bfloat16_rn(__bfloat162float(act) * w);
    }
    *reinterpret_cast<uint4*>(out + (size_t)row * I + c) = ov;
}

NG_EXPORT int ng_moe_swiglu_scaled(const void* gate_up, const float* weights, void* out, int n_rows, int I, int E, int ff,
                                   int ldw, int shared_gated, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (E <= 0 || ff <= 0 || I < E * ff || n_rows > 65535 || ldw < E + (shared_gated ? 1 : 0)) return NG_BAD_SIZE;
    if (act_bf16 && I % 8 == 0 && ff % 8 == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        dim3 vgrid((I / 8 + 127) / 128, n_rows);
        NG_LAUNCH((moe_swiglu_scaled_vec_kernel), vgrid, 128, 0, stream, (const __nv_bfloat16*)gate_up, weights,
                  (__nv_bfloat16*)out, I, E, ff, ldw, shared_gated);
        return ng_launch_status();
    }
    dim3 grid((I + 255) / 256, n_rows);
    if (act_bf16)
        NG_LAUNCH((moe_swiglu_scaled_kernel<__nv_bfloat16>), grid, 256, 0, stream, (const __nv_bfloat16*)gate_up, weights,
                  (__nv_bfloat16*)out, I, E, ff, ldw, shared_gated);
    else
        NG_LAUNCH((moe_swiglu_scaled_kernel<float>), grid, 256, 0, stream, (const float*)gate_up, weights, (float*)out, I, E, ff,
                  ldw, shared_gated);
    return ng_launch_status();
}

NG_EXPORT int ng_moe_router(const void* x, const float* wr, const float* br, float* weights, int n_rows, int H,
                            int E, int top_k, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (H <= 0 || E <= 0 || top_k < 1 || top_k > E || top_k > MOE_MAX_TOP || E > 8192) return NG_BAD_SIZE;
    const size_t smem = (size_t)E * sizeof(float);
    // a warp per expert where rows are few (each dot product is a chain of loads), four warps a row otherwise
    const int threads = n_rows <= 64 ? 32 * (E < 4 ? 4 : E > 16 ? 16 : E) : 128;
    if (act_bf16)
        NG_LAUNCH((moe_router_kernel<__nv_bfloat16>), n_rows, threads, smem, stream, (const __nv_bfloat16*)x, wr, br, weights,
                  H, E, top_k);
    else
        NG_LAUNCH((moe_router_kernel<float>), n_rows, threads, smem, stream, (const float*)x, wr, br, weights, H, E, top_k);
    return ng_launch_status();
}

NG_EXPORT int ng_moe_scale(void* act, const float* weights, int n_rows, int E, int ff, int ld, int ldw, int shared_gated,
                           int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (E <= 0 || ff <= 0 || ld < E * ff || n_rows > 65535 || ldw < E + (shared_gated ? 1 : 0)) return NG_BAD_SIZE;
    const int cols = shared_gated ? ld : E * ff;
    dim3 grid((cols + 255) / 256, n_rows);
    if (act_bf16)
        NG_LAUNCH((moe_scale_kernel<__nv_bfloat16>), grid, 256, 0, stream, (__nv_bfloat16*)act, weights, n_rows, E, ff, ld, ldw, cols);
    else
        NG_LAUNCH((moe_scale_kernel<float>), grid, 256, 0, stream, (float*)act, weights, n_rows, E, ff, ld, ldw, cols);
    return ng_launch_status();
}

// ------------------------------------------------------------------------------------------ sigmoid scores, groups
// moe_router_sigmoid: scores s = sigmoid(W_r x) in float32.  Choice scores are s + correction (no correction: s); the
//   experts form n_groups equal groups of neighbours, a group's score is the sum of its two largest choice scores (of
//   its one score where a group is one expert), and only experts of the keep_groups best groups can be chosen (of equal
//   scores the lower index wins, for groups and for experts).  The top_k chosen experts are weighted by their scores s
//   (without the correction) over their sum + 1e-20.  Output: dense weights [n_rows, ldw], zero for experts a row does
//   not use; with `wsg` (float32 [H]) column E receives sigmoid(wsg . x), the gate of a shared expert.
//   `softmax_scores`: s = softmax(W_r x) over all experts instead of the sigmoid.  `group_max`: a group's score is its
//   largest choice score.  `route_scale` multiplies the weights.
template <typename T>
__global__ void __launch_bounds__(512)
moe_router_sigmoid_kernel(const T* __restrict__ x, const float* __restrict__ wr, const float* __restrict__ corr,
                          const float* __restrict__ wsg, float* __restrict__ weights, int H, int E, int ldw, int top_k,
                          int n_groups, int keep_groups, int softmax_scores, int group_max, float route_scale) {
    extern __shared__ float z[];               // [E] scores s, [E] choice scores, [n_groups] group scores
    float* choice = z + E;
    float* gscore = choice + E;
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const T* xr = x + (size_t)row * H;
    float* out = weights + (size_t)row * ldw;
    for (int e = warp; e < E + (wsg ? 1 : 0); e += nwarp) {
        const float* w = e < E ? wr + (size_t)e * H : wsg;
        float acc = 0.f;
        if (H % 4 == 0) {
#pragma unroll 4
            for (int i = lane * 4; i < H; i += 128) {
                const float4 xv = moe_ld4(xr + i), wv = moe_ld4(w + i);
                acc = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc))));
            }
        } else {
            for (int i = lane; i < H; i += 32) acc = fmaf(ng_ld(xr + i), w[i], acc);
        }
        acc = ng_warp_sum(acc);
        if (lane == 0) {
            const float s = 1.f / (1.f + expf(-acc));
            if (e < E) { z[e] = softmax_scores ? acc : s; choice[e] = s + (corr ? corr[e] : 0.f); out[e] = 0.f; }
            else out[E] = s;
        }
    }
    __syncthreads();
    if (softmax_scores) {                  // the first warp: largest logit, the exponentials' sum in index order per lane
        if (warp == 0) {
            float mx = -INFINITY;
            for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
            mx = ng_warp_max(mx);
            float sum = 0.f;
            for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
            sum = ng_warp_sum(sum);
            for (int e = lane; e < E; e += 32) {
                const float s = expf(z[e] - mx) / sum;
                z[e] = s;
                choice[e] = s + (corr ? corr[e] : 0.f);
            }
        }
        __syncthreads();
    }
    const int per = E / n_groups;
    for (int g = threadIdx.x; g < n_groups; g += blockDim.x) {
        float a = -INFINITY, b = -INFINITY;             // the two largest of the group
        for (int e = g * per; e < (g + 1) * per; ++e) {
            const float v = choice[e];
            if (v > a) { b = a; a = v; } else if (v > b) b = v;
        }
        gscore[g] = per > 1 && !group_max ? a + b : a;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (keep_groups < n_groups) {
            // a group stays when fewer than keep_groups groups come before it (a larger score, or an equal one at a lower index)
            for (int g = 0; g < n_groups; ++g) {
                int ahead = 0;
                for (int o = 0; o < n_groups; ++o) ahead += (gscore[o] > gscore[g]) || (gscore[o] == gscore[g] && o < g);
                if (ahead >= keep_groups)
                    for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
            }
        }
        int idx[MOE_MAX_TOP];
        float sum = 0.f;
        for (int k = 0; k < top_k; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e) {
                const float v = choice[e];
                if (best < 0 || v > bv) {
                    bool taken = false;
                    for (int m = 0; m < k; ++m) taken |= idx[m] == e;
                    if (!taken) { best = e; bv = v; }
                }
            }
            idx[k] = best;
            sum += z[best];
        }
        for (int k = 0; k < top_k; ++k) out[idx[k]] = z[idx[k]] / (sum + 1e-20f) * route_scale;
    }
}

NG_EXPORT int ng_moe_router_sigmoid(const void* x, const float* wr, const float* corr, const float* wsg, float* weights,
                                    int n_rows, int H, int E, int ldw, int top_k, int n_groups, int keep_groups,
                                    int softmax_scores, int group_max, float route_scale, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (H <= 0 || E <= 0 || top_k < 1 || top_k > E || top_k > MOE_MAX_TOP || E > 4096 || n_groups < 1 || E % n_groups ||
        keep_groups < 1 || keep_groups > n_groups || top_k > keep_groups * (E / n_groups) || ldw < E + (wsg ? 1 : 0))
        return NG_BAD_SIZE;
    const size_t smem = (size_t)(2 * E + n_groups) * sizeof(float);
    const int threads = n_rows <= 64 ? 32 * (E < 4 ? 4 : E > 16 ? 16 : E) : 128;
    if (act_bf16)
        NG_LAUNCH((moe_router_sigmoid_kernel<__nv_bfloat16>), n_rows, threads, smem, stream, (const __nv_bfloat16*)x, wr, corr,
                  wsg, weights, H, E, ldw, top_k, n_groups, keep_groups, softmax_scores, group_max, route_scale);
    else
        NG_LAUNCH((moe_router_sigmoid_kernel<float>), n_rows, threads, smem, stream, (const float*)x, wr, corr, wsg, weights, H,
                  E, ldw, top_k, n_groups, keep_groups, softmax_scores, group_max, route_scale);
    return ng_launch_status();
}

// moe_clamped_glu_scaled: out[row, c] = g' sigmoid(alpha g') (u' + 1) * weight, g' = min(g, limit), u' = clamp(u, -limit, limit),
//   g = gate_up[row, c], u = gate_up[row, I + c].  Columns below E*ff belong to expert c / ff: limit_e, weight
//   weights[row, c / ff]; the columns behind them to a shared expert: limit_s, weight weights[row, E] when `shared_gated`,
//   else 1.  Float32 until the one rounding of the result.
template <typename T>
__global__ void moe_clamped_glu_scaled_kernel(const T* __restrict__ gate_up, const float* __restrict__ weights, int ldw,
                                              T* __restrict__ out, int I, int E, int ff, float limit_e, float limit_s,
                                              float alpha, int shared_gated) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= I) return;
    const bool routed = c < E * ff;
    const float limit = routed ? limit_e : limit_s;
    const float g = fminf(ng_ld(gate_up + (size_t)row * 2 * I + c), limit);
    const float u = fminf(fmaxf(ng_ld(gate_up + (size_t)row * 2 * I + I + c), -limit), limit);
    const float w = routed ? weights[(size_t)row * ldw + c / ff] : (shared_gated ? weights[(size_t)row * ldw + E] : 1.f);
    ng_st(out + (size_t)row * I + c, g / (1.f + expf(-alpha * g)) * (u + 1.f) * w);
}

NG_EXPORT int ng_moe_clamped_glu_scaled(const void* gate_up, const float* weights, int ldw, void* out, int n_rows, int I,
                                        int E, int ff, float limit_e, float limit_s, float alpha, int shared_gated,
                                        int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (E <= 0 || ff <= 0 || I < E * ff || n_rows > 65535 || ldw < E + (shared_gated ? 1 : 0)) return NG_BAD_SIZE;
    dim3 grid((I + 255) / 256, n_rows);
    if (act_bf16)
        NG_LAUNCH((moe_clamped_glu_scaled_kernel<__nv_bfloat16>), grid, 256, 0, stream, (const __nv_bfloat16*)gate_up, weights,
                  ldw, (__nv_bfloat16*)out, I, E, ff, limit_e, limit_s, alpha, shared_gated);
    else
        NG_LAUNCH((moe_clamped_glu_scaled_kernel<float>), grid, 256, 0, stream, (const float*)gate_up, weights, ldw,
                  (float*)out, I, E, ff, limit_e, limit_s, alpha, shared_gated);
    return ng_launch_status();
}
