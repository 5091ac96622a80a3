// Latent attention core for long steps (bfloat16) on the tensor cores, with float32 scores, weights and sums.
//
// Every head of a row reads the same latent pages as keys and as values, so the heads of ONE row are the 16
// rows of an m16n8k16 tile: a warp takes a row, copies 32 latents at a time into shared memory (cp.async, a tile ahead),
// and forms
//     S[16 heads x 32 keys] = Q C^T      bfloat16 x bfloat16 products are exact, the sum is float32: float32 scores
//     online softmax in float32 (a quad of lanes holds a head's 32 scores)
//     O[16 heads x rank]   += P C        with the float32 weights P cut into three bfloat16 terms hi + mid + lo
//                                        (p - hi - mid - lo is below 2^-24 p): each term's products are exact
//                                        in the float32 accumulators, so the weighted sum is a float32 sum
// The head's gate multiplies the result in the store.  Up to 16 heads (rows of the tile past the heads are zero; with
// eight heads or fewer the tile's lower half takes the next query row),
// rank a multiple of 32 fixed at compile time (-DNG_LAT_RANK).  Keys are walked in ascending order from the
// window's first key: a row's result does not depend on the cut or the batch.
#include "ng_common.cuh"

#ifndef NG_LAT_RANK
#error "compile with -DNG_LAT_RANK=<padded latent width, a multiple of 32 up to 256>"
#endif
static_assert(NG_LAT_RANK % 32 == 0 && NG_LAT_RANK >= 32 && NG_LAT_RANK <= 256, "latent width: a multiple of 32 up to 256");

#define LM_R NG_LAT_RANK
#define LM_TILE 32
#if NG_LAT_RANK > 160
#define LM_WARPS 2                // two tiles a warp (one being copied, one being used): about 70 KB a block either way
#else
#define LM_WARPS 4
#endif
#define LM_LD (LM_R + 8)          // shared-memory row in elements: 16 bytes of padding keep ldmatrix off one bank

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void lm_ldsm4(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_ldsm4_t(uint32_t (&r)[4], const bf16* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes global -> shared, asynchronously; `bytes` 0 writes zeros instead
__device__ __forceinline__ void lm_cp16(bf16* dst, const bf16* src, int bytes) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void lm_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void lm_cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void lm_cp_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

__device__ __forceinline__ uint32_t lm_pack(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// (x, y) as three bfloat16 pairs whose sum is (x, y) to float32 accuracy
__device__ __forceinline__ void lm_split3(float x, float y, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
    const bf16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    const float xr = x - __bfloat162float(xh), yr = y - __bfloat162float(yh);
    const bf16 xm = __float2bfloat16_rn(xr), ym = __float2bfloat16_rn(yr);
    hi = lm_pack(__bfloat162float(xh), __bfloat162float(yh));
    mid = lm_pack(__bfloat162float(xm), __bfloat162float(ym));
    lo = lm_pack(xr - __bfloat162float(xm), yr - __bfloat162float(ym));
}

// PAIR (models of up to eight heads): the tile's lower eight rows are the heads of the NEXT query row, so no half of
// a tile is empty.  Two rows share their key tiles when they are neighbours of one request (same entry, positions p and
// p + 1); otherwise the warp takes them one after the other, each in the upper half.
template <bool PAIR>
__global__ void __launch_bounds__(LM_WARPS * 32)
latent_core_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages, const int* __restrict__ table,
                       int table_stride, const int* __restrict__ positions, const int* __restrict__ row_entry,
                       const float* __restrict__ gate, bf16* __restrict__ out, int n_rows, int nH, int page_size,
                       int num_pages, int window, float scale) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * LM_WARPS + warp;
    const int first = PAIR ? 2 * unit : unit;
    if (first >= n_rows) return;
    const int quad = lane >> 2, tq = lane & 3;             // heads quad and quad + 8; columns 2 tq, 2 tq + 1 of an 8-wide tile
    bf16* bufs = reinterpret_cast<bf16*>(lm_smem) + (size_t)warp * 2 * LM_TILE * LM_LD;      // this warp's two tiles
    bool together = false;
    int n_pass = 1;
    if (PAIR && first + 1 < n_rows) {
        const int e0 = row_entry[first], e1 = row_entry[first + 1];
        together = e0 >= 0 && e0 == e1 && positions[first + 1] == positions[first] + 1;
        n_pass = together ? 1 : 2;
    }
    for (int pass = 0; pass < (PAIR ? n_pass : 1); ++pass) {
    const int row = first + pass;                          // the row of the tile's upper half
    const int row1 = together ? first + 1 : -1;            // PAIR: the row of its lower half, if it has one
    bf16* orow = out + (size_t)row * nH * LM_R;
    const int entry = row_entry[row];
    if (entry < 0) {
        for (int i = lane; i < nH * LM_R; i += 32) orow[i] = __float2bfloat16_rn(0.f);
        continue;
    }
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int pos1 = row1 >= 0 ? pos + 1 : pos;            // the lower half's last and first visible key
    const int lo1 = PAIR ? (window > 0 ? max(0, pos1 - window + 1) : 0) : lo;
    const int pos_hi = pos1;                               // the last key any row of the tile sees
    const int* trow = table + (size_t)entry * table_stride;

    // the queries as A fragments: rows quad (upper half) and quad + 8 (lower half), all of the latent's columns
    uint32_t qa[LM_R / 16][4];
    {
        const bf16* q0 = q + ((size_t)row * nH + quad) * LM_R;
        const bf16* q1 = PAIR ? q + ((size_t)max(row1, 0) * nH + quad) * LM_R : q0 + (size_t)8 * LM_R;
        const bool h0 = quad < nH, h1 = PAIR ? (row1 >= 0 && quad < nH) : quad + 8 < nH;
#pragma unroll
        for (int ks = 0; ks < LM_R / 16; ++ks) {
            const int d = ks * 16 + tq * 2;
            qa[ks][0] = h0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
            qa[ks][1] = h1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
            qa[ks][2] = h0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
            qa[ks][3] = h1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        }
    }
    float o[LM_R / 8][4];
#pragma unroll
    for (int t = 0; t < LM_R / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    constexpr int CPK = LM_R / 8;                              // 16-byte pieces of a key
    // a tile is copied asynchronously while the one before it is used; keys past the tile's last visible one are zero
    auto stage = [&](int k0, bf16* dst) {
        const int n = min(LM_TILE, pos_hi + 1 - k0);
#pragma unroll
        for (int i = 0; i < CPK; ++i) {
            const int c = lane + 32 * i;
            const int k = c / CPK, part = c % CPK;
            const bf16* src = pages;
            int bytes = 0;
            if (k < n) {
                const int kp = k0 + k;
                const int page = trow[kp / page_size];
                if (page >= 0 && page < num_pages) {
                    src = pages + ((size_t)page * page_size + (kp % page_size)) * LM_R + part * 8;
                    bytes = 16;
                }
            }
            lm_cp16(dst + k * LM_LD + part * 8, src, bytes);
        }
        lm_cp_commit();
    };
    __syncwarp();                                              // (a second pass: the tiles of the first are done with)
    stage(lo, bufs);
    int it = 0;
    for (int k0 = lo; k0 <= pos_hi; k0 += LM_TILE, ++it) {
        const int n = min(LM_TILE, pos_hi + 1 - k0);
        const bf16* tile = bufs + (size_t)(it & 1) * LM_TILE * LM_LD;
        if (k0 + LM_TILE <= pos_hi) {
            stage(k0 + LM_TILE, bufs + (size_t)((it + 1) & 1) * LM_TILE * LM_LD);
            lm_cp_wait_but_one();
        } else {
            lm_cp_wait_all();
        }
        __syncwarp();
        // scores: four tiles of 8 keys
        float s[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < LM_R / 16; ks += 2) {
                uint32_t b[4];                                  // (ks: columns 0-7, 8-15), (ks + 1: columns 0-7, 8-15) of these 8 keys
                lm_ldsm4(b, tile + (nt * 8 + (lane & 7)) * LM_LD + ks * 16 + (lane >> 3) * 8);
                lm_mma(s[nt], qa[ks], b[0], b[1]);
                lm_mma(s[nt], qa[ks + 1], b[2], b[3]);
            }
        }
        // online softmax of the upper half's rows (values 0, 1 of a tile) and the lower half's (values 2, 3)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int kidx = k0 + nt * 8 + tq * 2 + e;
                const bool ok0 = PAIR ? kidx <= pos : nt * 8 + tq * 2 + e < n;
                const bool ok1 = PAIR ? (row1 >= 0 && kidx >= lo1 && kidx <= pos1) : ok0;
                s[nt][e] = ok0 ? s[nt][e] * scale : -INFINITY;
                s[nt][2 + e] = ok1 ? s[nt][2 + e] * scale : -INFINITY;
                mx0 = fmaxf(mx0, s[nt][e]);
                mx1 = fmaxf(mx1, s[nt][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        // a half that has seen no key yet (a lower half without a row) keeps a running maximum of -inf: subtract 0 there
        const float b0 = mn0, b1 = PAIR && mn1 == -INFINITY ? 0.f : mn1;     // (the upper half always sees the tile's first key)
        const float c0 = expf(m0 - b0), c1 = expf(m1 - b1);
        m0 = mn0;
        m1 = mn1;
        float r0 = 0.f, r1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                s[nt][e] = expf(s[nt][e] - b0);
                s[nt][2 + e] = expf(s[nt][2 + e] - b1);
                r0 += s[nt][e];
                r1 += s[nt][2 + e];
            }
        }
        l0 = l0 * c0 + r0;                                       // a lane's share; the quad's shares are added at the end
        l1 = l1 * c1 + r1;
#pragma unroll
        for (int t = 0; t < LM_R / 8; ++t) {
            o[t][0] *= c0;
            o[t][1] *= c0;
            o[t][2] *= c1;
            o[t][3] *= c1;
        }
        // weighted sum: two steps of 16 keys, the weights as three bfloat16 terms
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            uint32_t ph[4], pm[4], pl[4];
            lm_split3(s[2 * kk][0], s[2 * kk][1], ph[0], pm[0], pl[0]);
            lm_split3(s[2 * kk][2], s[2 * kk][3], ph[1], pm[1], pl[1]);
            lm_split3(s[2 * kk + 1][0], s[2 * kk + 1][1], ph[2], pm[2], pl[2]);
            lm_split3(s[2 * kk + 1][2], s[2 * kk + 1][3], ph[3], pm[3], pl[3]);
            // four column tiles at a time: the three terms of one accumulator lie four instructions apart, so the
            // tensor pipe is not held up by the chain of an accumulator's own additions
#pragma unroll
            for (int dt = 0; dt < LM_R / 8; dt += 4) {
                uint32_t b[4], c[4];                            // (dt: keys 0-7, 8-15), (dt + 1: ...) and (dt + 2), (dt + 3) of this step
                lm_ldsm4_t(b, tile + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LM_LD + (dt + (lane >> 4)) * 8);
                lm_ldsm4_t(c, tile + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LM_LD + (dt + 2 + (lane >> 4)) * 8);
                lm_mma(o[dt], pl, b[0], b[1]);                  // smallest terms first
                lm_mma(o[dt + 1], pl, b[2], b[3]);
                lm_mma(o[dt + 2], pl, c[0], c[1]);
                lm_mma(o[dt + 3], pl, c[2], c[3]);
                lm_mma(o[dt], pm, b[0], b[1]);
                lm_mma(o[dt + 1], pm, b[2], b[3]);
                lm_mma(o[dt + 2], pm, c[0], c[1]);
                lm_mma(o[dt + 3], pm, c[2], c[3]);
                lm_mma(o[dt], ph, b[0], b[1]);
                lm_mma(o[dt + 1], ph, b[2], b[3]);
                lm_mma(o[dt + 2], ph, c[0], c[1]);
                lm_mma(o[dt + 3], ph, c[2], c[3]);
            }
        }
        __syncwarp();                                            // the tile is free for the copy after next
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // where the two halves' results go: (row, head quad) and, lower half, (row, head quad + 8) or (the next row, head quad)
    const int h0 = quad, h1 = PAIR ? quad : quad + 8;
    const int out_row1 = PAIR ? row1 : row;
    const bool st0 = h0 < nH, st1 = out_row1 >= 0 && h1 < nH;
    const float f0 = st0 ? (l0 > 0.f ? 1.f / l0 : 0.f) * (gate ? gate[(size_t)row * nH + h0] : 1.f) : 0.f;
    const float f1 = st1 ? (l1 > 0.f ? 1.f / l1 : 0.f) * (gate ? gate[(size_t)out_row1 * nH + h1] : 1.f) : 0.f;
    bf16* orow1 = out + (size_t)max(out_row1, 0) * nH * LM_R;
#pragma unroll
    for (int t = 0; t < LM_R / 8; ++t) {
        const int d = t * 8 + tq * 2;
        if (st0) *reinterpret_cast<uint32_t*>(orow + (size_t)h0 * LM_R + d) = lm_pack(o[t][0] * f0, o[t][1] * f0);
        if (st1) *reinterpret_cast<uint32_t*>(orow1 + (size_t)h1 * LM_R + d) = lm_pack(o[t][2] * f1, o[t][3] * f1);
    }
    }
}

// q, out: bfloat16 [n_rows, nH * NG_LAT_RANK]; pages: bfloat16 [num_pages, 1, page_size, NG_LAT_RANK]; gate float32 or null
NG_EXPORT int ng_latent_core_mma(const void* q, const void* pages, const int* table, int table_stride, const int* positions,
                                 const int* row_entry, const float* gate, void* out, int n_rows, int nH, int rp,
                                 int page_size, int num_pages, int window, float scale, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (rp != LM_R || nH <= 0 || nH > 16 || page_size <= 0) return NG_BAD_SIZE;
    const size_t smem = (size_t)LM_WARPS * 2 * LM_TILE * LM_LD * sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(latent_core_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(latent_core_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        configured = true;
    }
    if (nH <= 8) {                  // two query rows a tile
        const int units = (n_rows + 1) / 2;
        NG_LAUNCH((latent_core_mma_kernel<true>), (units + LM_WARPS - 1) / LM_WARPS, LM_WARPS * 32, smem, stream, (const bf16*)q,
                  (const bf16*)pages, table, table_stride, positions, row_entry, gate, (bf16*)out, n_rows, nH, page_size,
                  num_pages, window, scale);
    } else {
        NG_LAUNCH((latent_core_mma_kernel<false>), (n_rows + LM_WARPS - 1) / LM_WARPS, LM_WARPS * 32, smem, stream, (const bf16*)q,
                  (const bf16*)pages, table, table_stride, positions, row_entry, gate, (bf16*)out, n_rows, nH, page_size,
                  num_pages, window, scale);
    }
    return ng_launch_status();
}
