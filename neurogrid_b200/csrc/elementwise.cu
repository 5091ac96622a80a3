// Embedding gather, residual-add + RMSNorm, SwiGLU gate: the memory-bound row kernels.
//
// Reference counterparts (plain one-thread-per-element kernels): gather
// gpu/cuda/kernels.cu:669-708, RMSNorm gpu/cuda/bf16_utils.cu:57-116, fused add+norm (fp16
// only) gpu/cuda/kernels.cu:196-262, SiLU and multiply gpu/cuda/bf16_utils.cu:122-213.
// Here the residual stream is float32 in both compute dtypes; the residual add, the sum of
// squares and the scaling are done in float32 and only the GEMM operand is rounded.
#include "ng_common.cuh"

// ---------------------------------------------------------------------------------- embed
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int H, int V, int* __restrict__ status, int accumulate,
                             int bad_bit, float scale) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    int tok = tokens[row];
    const bool bad = tok < 0 || tok >= V;
    if (bad) {
        if (threadIdx.x == 0) atomicOr(status, bad_bit);
        tok = 0;
    }
    const T* src = table + (size_t)tok * H;
    float* dst = out + (size_t)row * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = bad ? 0.f : ng_ld(src + j) * scale;
        dst[j] = accumulate ? dst[j] + v : v;
    }
}

// out[row] = table[index[row]], or out[row] += ... when `accumulate` (a table of learned positions
// added to the token embeddings: the index is then the row's position).  An index outside the
// table gives zeros and sets `bad_bit` in the status word.
// Every looked-up row is multiplied by `scale` (1 for most models) in float32.
NG_EXPORT int ng_embed(const void* table, int table_bf16, const int* tokens, float* out, int n_rows,
                       int H, int V, int* status, int accumulate, int bad_bit, float scale, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (H <= 0 || V <= 0) return NG_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_bf16)
        NG_LAUNCH((embed_kernel<__nv_bfloat16>), n_rows, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, H, V,
                  status, accumulate, bad_bit, scale);
    else
        NG_LAUNCH((embed_kernel<float>), n_rows, threads, 0, stream, (const float*)table, tokens, out, H, V, status,
                  accumulate, bad_bit, scale);
    return ng_launch_status();
}

// dst[i] = src[idx[i]] where idx[i] >= 0 (else dst[i] stays): tokens sampled on the device feed the
// next step without passing through the host
__global__ void gather_i32_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ idx, int n) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && idx[i] >= 0) dst[i] = src[idx[i]];
}

NG_EXPORT int ng_gather_i32(int* dst, const int* src, const int* idx, int n, cudaStream_t stream) {
    if (n <= 0) return NG_OK;
    NG_LAUNCH((gather_i32_kernel), (n + 127) / 128, 128, 0, stream, dst, src, idx, n);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- add + rmsnorm
// One block per output row i.  src row = rows ? rows[i] : i.
//   if delta: h[src] += delta[src] (float32 sum, written back)      -- the residual sum
//   out[i] = h[src] * rsqrt(mean(h[src]^2) + eps) * w                -- rounded to TO once
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps, int n_partials,
                                   size_t partial_stride) {
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    float* hr = h + (size_t)src * H;
    float ss = 0.f;
    if (delta) {
        const TD* dr = delta + (size_t)src * H;
        for (int j = threadIdx.x; j < H; j += blockDim.x) {
            float v = hr[j];
            for (int s = 0; s < n_partials; ++s) v += ng_ld(dr + s * partial_stride + j);   // ascending s
            hr[j] = v;
            ss += v * v;
        }
    } else {
        for (int j = threadIdx.x; j < H; j += blockDim.x) {
            const float v = hr[j];
            ss += v * v;
        }
    }
    ss = ng_block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)i * H;
    // each thread re-reads exactly the elements it wrote itself
    for (int j = threadIdx.x; j < H; j += blockDim.x) ng_st(orow + j, hr[j] * r * w[j]);
}

// Same result for H % 4 == 0 and H <= 4 * NV * blockDim: each thread keeps its NV float4 of the
// row in registers, so the row is read once and the launch is one pass.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename TD, typename TO, int NV>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                       const float* __restrict__ w, TO* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps, int n_partials,
                                       size_t partial_stride) {
    __shared__ float red[32];
    ng_pdl_trigger();
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;                  // the batch description: older than the step's kernels
    float* hr = h + (size_t)src * H;
    float4 v[NV], ww[NV];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < NV; ++u) {                       // the norm's weights: before the wait for the kernel in front
        const int j = 4 * (threadIdx.x + u * blockDim.x);
        ww[u] = j < H ? ld4(w + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    ng_pdl_wait();
    delta = ng_after_wait(delta);
#pragma unroll
    for (int u = 0; u < NV; ++u) {
        const int j = 4 * (threadIdx.x + u * blockDim.x);
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (j < H) {
            v[u] = ld4(hr + j);
            if (delta) {
                for (int s = 0; s < n_partials; ++s) {                        // ascending s: a fixed order
                    const float4 d = ld4(delta + s * partial_stride + (size_t)src * H + j);
                    v[u].x += d.x; v[u].y += d.y; v[u].z += d.z; v[u].w += d.w;
                }
                st4(hr + j, v[u]);
            }
            ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
        }
    }
    ss = ng_block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)i * H;
#pragma unroll
    for (int u = 0; u < NV; ++u) {
        const int j = 4 * (threadIdx.x + u * blockDim.x);
        if (j < H)
            st4(orow + j, make_float4(v[u].x * r * ww[u].x, v[u].y * r * ww[u].y, v[u].z * r * ww[u].z, v[u].w * r * ww[u].w));
    }
}

template <typename TD, typename TO>
static void launch_add_rmsnorm(float* h, const void* delta, const float* w, void* out, const int* rows, int n_out,
                               int H, float eps, int n_partials, size_t pstride, cudaStream_t stream) {
    const bool aligned = H % 4 == 0 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                         ((uintptr_t)w % 16 == 0) && ((uintptr_t)delta % 16 == 0);
    if (aligned && H <= 4 * 4 * 256) {
        const int threads = H <= 4 * 128 ? 128 : 256;
        const int nv = (H / 4 + threads - 1) / threads;
        if (nv <= 1) NG_LAUNCH((add_rmsnorm_vec_kernel<TD, TO, 1>), n_out, threads, 0, stream, h, (const TD*)delta, w, (TO*)out, rows, H, eps, n_partials, pstride);
        else if (nv == 2) NG_LAUNCH((add_rmsnorm_vec_kernel<TD, TO, 2>), n_out, threads, 0, stream, h, (const TD*)delta, w, (TO*)out, rows, H, eps, n_partials, pstride);
        else NG_LAUNCH((add_rmsnorm_vec_kernel<TD, TO, 4>), n_out, threads, 0, stream, h, (const TD*)delta, w, (TO*)out, rows, H, eps, n_partials, pstride);
        return;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    NG_LAUNCH((add_rmsnorm_kernel<TD, TO>), n_out, threads, 0, stream, h, (const TD*)delta, w, (TO*)out, rows, H, eps, n_partials, pstride);
}

// delta: one [n, H] tensor of the activation dtype, or (delta_f32) n_partials float32 tensors
// [n, H] that lie partial_stride elements apart and are added in ascending order.
NG_EXPORT int ng_add_rmsnorm(float* h, const void* delta, const float* w, void* out, const int* rows,
                             int n_out, int H, float eps, int act_bf16, int delta_f32, int n_partials,
                             long long partial_stride, cudaStream_t stream) {
    if (n_out <= 0) return NG_OK;
    if (H <= 0 || n_partials < 1) return NG_BAD_SIZE;
    const size_t ps = (size_t)partial_stride;
    if (act_bf16 && delta_f32) launch_add_rmsnorm<float, __nv_bfloat16>(h, delta, w, out, rows, n_out, H, eps, n_partials, ps, stream);
    else if (act_bf16) launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(h, delta, w, out, rows, n_out, H, eps, 1, 0, stream);
    else launch_add_rmsnorm<float, float>(h, delta, w, out, rows, n_out, H, eps, delta_f32 ? n_partials : 1, ps, stream);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- add + layernorm
// One block per output row i, src row = rows ? rows[i] : i:
//   h[src] += delta[src] (float32 sum, written back; delta as for add_rmsnorm)
//   out[i] = (h[src] - mean) * rsqrt(var + eps) * w,   var = mean of the squared deviations; no bias
//   h[src] += post[.] afterwards if `post` is given: a vector that belongs to the sum the layer adds to the
//   stream later (the bias of a product whose epilogue adds straight into the stream)
// Each thread keeps its NV elements of the row in registers: the row is read once.
template <typename TD, typename TO, int NV>
__global__ void add_layernorm_kernel(float* __restrict__ h, const TD* __restrict__ delta, const float* __restrict__ w,
                                     TO* __restrict__ out, const int* __restrict__ rows, const float* __restrict__ post,
                                     int H, float eps, int n_partials, size_t partial_stride) {
    __shared__ float red[32];
    ng_pdl_trigger();
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    float* hr = h + (size_t)src * H;
    float v[NV];
    ng_pdl_wait();
    delta = ng_after_wait(delta);
    float sum = 0.f;
#pragma unroll
    for (int u = 0; u < NV; ++u) {
        const int j = threadIdx.x + u * blockDim.x;
        v[u] = 0.f;
        if (j < H) {
            v[u] = hr[j];
            if (delta)
                for (int s = 0; s < n_partials; ++s) v[u] += ng_ld(delta + s * partial_stride + (size_t)src * H + j);
            sum += v[u];
        }
    }
    const float mean = ng_block_sum(sum, red) / (float)H;
    float sq = 0.f;
#pragma unroll
    for (int u = 0; u < NV; ++u) {
        const int j = threadIdx.x + u * blockDim.x;
        if (j < H) sq += (v[u] - mean) * (v[u] - mean);
    }
    const float r = rsqrtf(ng_block_sum(sq, red) / (float)H + eps);
    TO* orow = out + (size_t)i * H;
#pragma unroll
    for (int u = 0; u < NV; ++u) {
        const int j = threadIdx.x + u * blockDim.x;
        if (j < H) {
            ng_st(orow + j, (v[u] - mean) * r * w[j]);
            if (delta || post) hr[j] = v[u] + (post ? post[j] : 0.f);
        }
    }
}

template <typename TD, typename TO>
static int launch_add_layernorm(float* h, const void* delta, const float* w, void* out, const int* rows, const float* post,
                                int n_out, int H, float eps, int n_partials, size_t ps, cudaStream_t stream) {
    const int threads = H <= 1024 ? 128 : H <= 4096 ? 256 : 1024;
    const int nv = (H + threads - 1) / threads;
#define LN_GO(NV) NG_LAUNCH((add_layernorm_kernel<TD, TO, NV>), n_out, threads, 0, stream, h, (const TD*)delta, w, (TO*)out, \
                            rows, post, H, eps, n_partials, ps)
    if (nv <= 2) LN_GO(2);
    else if (nv <= 4) LN_GO(4);
    else if (nv <= 8) LN_GO(8);
    else if (nv <= 16) LN_GO(16);
    else return NG_BAD_SIZE;
#undef LN_GO
    return ng_launch_status();
}

// `rows` and `post` do not go together with a delta on gathered rows: a gathered row may be named twice.
NG_EXPORT int ng_add_layernorm(float* h, const void* delta, const float* w, void* out, const int* rows, const float* post,
                               int n_out, int H, float eps, int act_bf16, int delta_f32, int n_partials,
                               long long partial_stride, cudaStream_t stream) {
    if (n_out <= 0) return NG_OK;
    if (H <= 0 || n_partials < 1 || (rows && post)) return NG_BAD_SIZE;
    const size_t ps = (size_t)partial_stride;
    if (act_bf16 && delta_f32) return launch_add_layernorm<float, __nv_bfloat16>(h, delta, w, out, rows, post, n_out, H, eps, n_partials, ps, stream);
    if (act_bf16) return launch_add_layernorm<__nv_bfloat16, __nv_bfloat16>(h, delta, w, out, rows, post, n_out, H, eps, 1, 0, stream);
    return launch_add_layernorm<float, float>(h, delta, w, out, rows, post, n_out, H, eps, delta_f32 ? n_partials : 1, ps, stream);
}

// h[row] += delta[row] only (the last residual sum of a model whose output is not normed here)
template <typename TD>
__global__ void add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n, int n_partials) {
    ng_pdl_trigger();
    ng_pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = h[i];
    for (int s = 0; s < n_partials; ++s) v += ng_ld(delta + s * n + i);
    h[i] = v;
}

NG_EXPORT int ng_residual_add(float* h, const void* delta, long long n, int delta_bf16, int n_partials,
                              cudaStream_t stream) {
    if (n <= 0) return NG_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (delta_bf16) NG_LAUNCH((add_kernel<__nv_bfloat16>), blocks, 256, 0, stream, h, (const __nv_bfloat16*)delta, (size_t)n, 1);
    else NG_LAUNCH((add_kernel<float>), blocks, 256, 0, stream, h, (const float*)delta, (size_t)n, n_partials);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- swiglu
// gu is [n_rows, 2*I]: gate = gu[:, :I], up = gu[:, I:];  out = act(gate) * up, float32 math;
// act: silu, or (`gelu`) the tanh form of gelu, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  `out` rows lie
// `ldo` elements apart (a column block of a wider buffer).
__device__ __forceinline__ float ng_gate_act(float g, int gelu) {
    if (gelu) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.f + expf(-g));
}
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int ldo, int gelu) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t row = blockIdx.x;
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= I) return;
    const float g = ng_ld(gu + row * 2 * (size_t)I + j);
    const float u = ng_ld(gu + row * 2 * (size_t)I + I + j);
    ng_st(out + row * (size_t)ldo + j, ng_gate_act(g, gelu) * u);
}

// bfloat16, I % 8 == 0: eight elements (16 bytes of gate, 16 of up) per thread
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I, int ldo,
                                     int gelu) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t row = blockIdx.x;
    const int j = 8 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (j >= I) return;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + row * 2 * (size_t)I + j);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + row * 2 * (size_t)I + I + j);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float ga = __low2float(g2[k]), gb = __high2float(g2[k]);
        const float ua = __low2float(u2[k]), ub = __high2float(u2[k]);
        o2[k] = __floats2bfloat162_rn(ng_gate_act(ga, gelu) * ua, ng_gate_act(gb, gelu) * ub);
    }
    *reinterpret_cast<uint4*>(out + row * (size_t)ldo + j) = o4;
}

NG_EXPORT int ng_swiglu(const void* gu, void* out, int n_rows, int I, int ldo, int gelu, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (I <= 0 || (I + 255) / 256 > 65535 || ldo < I) return NG_BAD_SIZE;
    if (act_bf16 && I % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        dim3 grid8(n_rows, (I / 8 + 127) / 128);
        NG_LAUNCH((swiglu_bf16x8_kernel), grid8, 128, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, ldo, gelu);
        return ng_launch_status();
    }
    dim3 grid(n_rows, (I + 255) / 256);
    if (act_bf16) NG_LAUNCH((swiglu_kernel<__nv_bfloat16>), grid, 256, 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, ldo, gelu);
    else NG_LAUNCH((swiglu_kernel<float>), grid, 256, 0, stream, (const float*)gu, (float*)out, I, ldo, gelu);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- token-pair embedding
// h[row] += table[idx], idx = (previous token * mul_prev + token * mul_cur) mod buckets, and idx = buckets (the
// table's last row) for a request's first token.  The previous token of an entry's first row is the request's last
// token of the step before, kept in its state slot (int32 [slots]); `pair_state_kernel` leaves there each entry's
// last token of this step, after every row has read.
template <typename T>
__global__ void pair_embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens, const int* __restrict__ state,
                                  const int* __restrict__ cu_q, const int* __restrict__ ctx_before,
                                  const int* __restrict__ slots, const int* __restrict__ row_entry, float* __restrict__ h,
                                  int H, int V, int buckets, long long mul_prev, long long mul_cur, int* __restrict__ status) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int e = row_entry[row];
    if (e < 0) return;
    const int tok = tokens[row];
    if (tok < 0 || tok >= V) return;                       // the embedding kernel has set the status bit
    int prev = -1;
    if (row > cu_q[e]) prev = tokens[row - 1];
    else if (ctx_before[e] > 0) prev = state[slots[e]];
    if (prev >= V) {
        if (threadIdx.x == 0) atomicOr(status, NG_STATUS_BAD_TOKEN);
        prev = -1;
    }
    const long long idx = prev < 0 ? (long long)buckets : ((long long)prev * mul_prev + (long long)tok * mul_cur) % buckets;
    const T* src = table + (size_t)idx * H;
    float* dst = h + (size_t)row * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) dst[j] += ng_ld(src + j);
}

__global__ void pair_state_kernel(const int* __restrict__ tokens, int* __restrict__ state, const int* __restrict__ cu_q,
                                  const int* __restrict__ slots, int n_entries) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_entries) return;
    const int q0 = cu_q[e], q1 = cu_q[e + 1];
    if (q1 > q0) state[slots[e]] = tokens[q1 - 1];
}

NG_EXPORT int ng_pair_embed(const void* table, int table_bf16, const int* tokens, int* state, const int* cu_q,
                            const int* ctx_before, const int* slots, const int* row_entry, float* h, int n_rows,
                            int n_entries, int H, int V, int buckets, long long mul_prev, long long mul_cur, int* status,
                            cudaStream_t stream) {
    if (n_rows <= 0 || n_entries <= 0) return NG_OK;
    if (H <= 0 || V <= 0 || buckets <= 0 || mul_prev < 0 || mul_cur < 0) return NG_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_bf16)
        NG_LAUNCH((pair_embed_kernel<__nv_bfloat16>), n_rows, threads, 0, stream, (const __nv_bfloat16*)table, tokens, state,
                  cu_q, ctx_before, slots, row_entry, h, H, V, buckets, mul_prev, mul_cur, status);
    else
        NG_LAUNCH((pair_embed_kernel<float>), n_rows, threads, 0, stream, (const float*)table, tokens, state, cu_q,
                  ctx_before, slots, row_entry, h, H, V, buckets, mul_prev, mul_cur, status);
    NG_LAUNCH((pair_state_kernel), (n_entries + 127) / 128, 128, 0, stream, tokens, state, cu_q, slots, n_entries);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- two normed inputs, averaged
// y[row] = 0.5 * (a / rms(a) * wa + b / rms(b) * wb), rms over the row with eps inside the root, float32.  a and b are
// [N, H] of type TI or stacks of float32 partial sums; `accumulate`: out[row] += y, else out[row] = y (out float32).
template <typename TO, typename TA, typename TB>
__global__ void __launch_bounds__(256)
pair_norm_mean_kernel(const TA* __restrict__ a, int a_parts, size_t a_stride, const TB* __restrict__ b, int b_parts,
                      size_t b_stride, const float* __restrict__ wa, const float* __restrict__ wb, float* __restrict__ out,
                      int H, float eps, int accumulate) {
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t base = (size_t)blockIdx.x * H;
    float sa = 0.f, sb = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float x = ng_ld_sum<TO>(a, base + j, a_parts, a_stride), y = ng_ld_sum<TO>(b, base + j, b_parts, b_stride);
        sa += x * x;
        sb += y * y;
    }
    sa = ng_block_sum(sa, red);
    sb = ng_block_sum(sb, red);
    const float ra = rsqrtf(sa / (float)H + eps), rb = rsqrtf(sb / (float)H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float x = ng_ld_sum<TO>(a, base + j, a_parts, a_stride), y = ng_ld_sum<TO>(b, base + j, b_parts, b_stride);
        const float v = 0.5f * (x * ra * wa[j] + y * rb * wb[j]);
        out[base + j] = accumulate ? out[base + j] + v : v;
    }
}

// a_f32 / b_f32: the input is float32 (a_parts partial sums `a_stride` elements apart), else of the activation type
NG_EXPORT int ng_pair_norm_mean(const void* a, int a_f32, int a_parts, long long a_stride, const void* b, int b_f32,
                                int b_parts, long long b_stride, const float* wa, const float* wb, float* out, int n_rows,
                                int H, float eps, int accumulate, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (H <= 0 || a_parts < 1 || b_parts < 1) return NG_BAD_SIZE;
    typedef __nv_bfloat16 bf;
#define PNM(TO, TA, TB)                                                                                               \
    NG_LAUNCH((pair_norm_mean_kernel<TO, TA, TB>), n_rows, 256, 0, stream, (const TA*)a, a_parts, (size_t)a_stride,    \
              (const TB*)b, b_parts, (size_t)b_stride, wa, wb, out, H, eps, accumulate)
    if (act_bf16) {
        if (a_f32 && b_f32) PNM(bf, float, float);
        else if (a_f32) PNM(bf, float, bf);
        else if (b_f32) PNM(bf, bf, float);
        else PNM(bf, bf, bf);
    } else {
        PNM(float, float, float);
    }
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- small in-place maps
// kind 0: x <- relu(x)^2 (over [n] elements of the activation type);  kind 1: x <- cap * tanh(x / cap) (float32);
// kind 2: x <- x * param
template <typename T>
__global__ void unary_kernel(T* __restrict__ x, size_t n, int kind, float param) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = ng_ld(x + i);
    float y;
    if (kind == 0) { const float r = fmaxf(v, 0.f); y = r * r; }
    else if (kind == 2) y = v * param;
    else y = param * tanhf(v / param);
    ng_st(x + i, y);
}

NG_EXPORT int ng_unary(void* x, long long n, int kind, float param, int x_bf16, cudaStream_t stream) {
    if (n <= 0) return NG_OK;
    if (kind < 0 || kind > 2 || (kind == 1 && !(param > 0.f))) return NG_BAD_SIZE;
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return NG_BAD_SIZE;
    if (x_bf16) NG_LAUNCH((unary_kernel<__nv_bfloat16>), (unsigned)blocks, 256, 0, stream, (__nv_bfloat16*)x, (size_t)n, kind, param);
    else NG_LAUNCH((unary_kernel<float>), (unsigned)blocks, 256, 0, stream, (float*)x, (size_t)n, kind, param);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- an output gate, element by element
// y[row, j] = y[row, j] * act(g[row, j]) * scale over [n_rows, I]; act 0: none (g unused), 1: sigmoid, 2: silu; float32
// math, one rounding.  Rows of y lie `ldy` elements apart and rows of g `ldg` (blocks of columns of wider buffers).
template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ y, const T* __restrict__ g, int I, int ldy, int ldg, int act, float scale) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t row = blockIdx.x;
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= I) return;
    float f = scale;
    if (act) {
        const float z = ng_ld(g + row * (size_t)ldg + j);
        const float s = 1.f / (1.f + expf(-z));
        f *= act == 1 ? s : z * s;
    }
    ng_st(y + row * (size_t)ldy + j, ng_ld(y + row * (size_t)ldy + j) * f);
}

NG_EXPORT int ng_gate_mul(void* y, const void* g, int n_rows, int I, int ldy, int ldg, int act, float scale, int act_bf16,
                          cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (I <= 0 || (I + 255) / 256 > 65535 || ldy < I || act < 0 || act > 2 || (act && (!g || ldg < I))) return NG_BAD_SIZE;
    dim3 grid(n_rows, (I + 255) / 256);
    if (act_bf16) NG_LAUNCH((gate_mul_kernel<__nv_bfloat16>), grid, 256, 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)g, I, ldy, ldg, act, scale);
    else NG_LAUNCH((gate_mul_kernel<float>), grid, 256, 0, stream, (float*)y, (const float*)g, I, ldy, ldg, act, scale);
    return ng_launch_status();
}
