// Layer norm with weight and bias over the 32-bit residual stream, and the "normed branch" sum of
// sandwich blocks:
//
//     LN(v; w, b) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w + b
//
// One kernel does, per row, up to two things in one pass:
//   (1) branch sum:  x[row] += mult * LN(y[row]; pw, pb)     (y: a sublayer's 32-bit output, or the
//       partial sums [S][T][D] of a product that was split over K, added here in ascending order)
//   (2) norm:        out[r] = LN(x[row]; w, b)                (in the compute type)
// so that the norm behind a sublayer and the norm ahead of the next one cost one trip over the row.
// Means and variances are 32-bit; the variance is the mean of the squared deviations (two passes
// over the row, which sits in shared memory).  `rms` = 1 selects the root-mean-square form (no
// mean, no bias) with the same interface.  Without a weight for (2) the output is the row itself in
// the compute type: a sublayer that reads the stream as it is.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

__device__ __forceinline__ float ld_w(const void* p, int dt, int i) {
    return dt == GFB_BF16 ? __bfloat162float(((const __nv_bfloat16*)p)[i]) : ((const float*)p)[i];
}

// statistics of the row held in `row` (shared memory): returns (mean, 1/sqrt(var + eps)); rms: (0, 1/sqrt(mean sq + eps))
__device__ __forceinline__ float2 row_stats(const float* row, int D, float eps, int rms, float* scratch) {
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) s += row[i];
        mean = gfb_block_sum(s, scratch) / (float)D;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { float dv = row[i] - mean; ss += dv * dv; }
    ss = gfb_block_sum(ss, scratch);
    return make_float2(mean, 1.0f / sqrtf(ss / (float)D + eps));
}

template <typename TO>
__global__ void layernorm_kernel(float* __restrict__ x, const float* __restrict__ y, int S, size_t slice,
                                 const void* pw, const void* pb, int p_dt, float peps, float mult,
                                 const void* w, const void* b, int w_dt, float eps, TO* __restrict__ out,
                                 const int* __restrict__ rows, int D, int rms) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int r = blockIdx.x;
    const size_t base = (size_t)(rows ? rows[r] : r) * D;
    if (y != nullptr) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = y[base + i];
            for (int k = 1; k < S; k++) v += y[(size_t)k * slice + base + i];
            row[i] = v;
        }
        __syncthreads();
        const float2 st = row_stats(row, D, peps, rms, scratch);
        __syncthreads();
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float n = (row[i] - st.x) * st.y * ld_w(pw, p_dt, i);
            if (!rms && pb != nullptr) n += ld_w(pb, p_dt, i);
            const float v = x[base + i] + mult * n;
            x[base + i] = v;
            row[i] = v;
        }
    } else if (out != nullptr) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) row[i] = x[base + i];
    }
    if (out == nullptr) return;
    __syncthreads();
    TO* o = out + (size_t)r * D;
    if (w == nullptr) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_from_f32<TO>(row[i]);
        return;
    }
    const float2 st = row_stats(row, D, eps, rms, scratch);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float n = (row[i] - st.x) * st.y * ld_w(w, w_dt, i);
        if (!rms && b != nullptr) n += ld_w(b, w_dt, i);
        o[i] = gfb_from_f32<TO>(n);
    }
}

// The same with the row in registers: float4 loads and stores, every load of a row (the branch, its partial sums, x)
// in flight at once, and the statistics from the registers.  For D % 4 == 0 and D <= 4 * LN_VEC * blockDim.
constexpr int LN_VEC = 8;

__device__ __forceinline__ float4 ld_w4(const void* p, int dt, int i4) {
    if (dt == GFB_BF16) {
        const uint2 raw = reinterpret_cast<const uint2*>(p)[i4];
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return reinterpret_cast<const float4*>(p)[i4];
}

// (mean, 1 / sqrt(mean of squared deviations + eps)) of the row spread over the block's registers
template <int NV>
__device__ __forceinline__ float2 reg_stats(const float4 (&v)[NV], int nvec, int D, float eps, int rms, float* scratch) {
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < NV; k++)
            if ((int)threadIdx.x + k * (int)blockDim.x < nvec) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        mean = gfb_block_sum(s, scratch) / (float)D;
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; k++)
        if ((int)threadIdx.x + k * (int)blockDim.x < nvec) {
            const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
            ss += (a * a + b * b) + (c * c + d * d);
        }
    ss = gfb_block_sum(ss, scratch);
    return make_float2(mean, 1.0f / sqrtf(ss / (float)D + eps));
}

// NV: float4 per thread; W: partial sums of the branch whose loads are in flight together (a decode step's few rows
// wait for one trip to L2 instead of one per partial sum; the sums are added in ascending order all the same).
template <typename TO, int NV, int W>
__global__ void __launch_bounds__(256)
layernorm_vec_kernel(float* __restrict__ x, const float* __restrict__ y, int S, size_t slice,
                                     const void* pw, const void* pb, int p_dt, float peps, float mult,
                                     const void* w, const void* b, int w_dt, float eps, TO* __restrict__ out,
                                     const int* __restrict__ rows, int D, int rms) {
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int r = blockIdx.x;
    const int nvec = D >> 2;
    const size_t base = (size_t)(rows ? rows[r] : r) * D;
    float4 v[NV];
    float4* xr = reinterpret_cast<float4*>(x + base);
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        v[k] = i < nvec ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (y != nullptr) {
        float4 u[NV];
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            u[k] = i < nvec ? reinterpret_cast<const float4*>(y + base)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int p = 1; p < S; p += W) {                    // further partial sums, ascending, W of them loaded together
            float4 a[W][NV];
#pragma unroll
            for (int q = 0; q < W; q++) {
                const float4* pr = reinterpret_cast<const float4*>(y + (size_t)min(p + q, S - 1) * slice + base);
#pragma unroll
                for (int k = 0; k < NV; k++) {
                    const int i = threadIdx.x + k * blockDim.x;
                    a[q][k] = i < nvec ? pr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int q = 0; q < W; q++)
                if (p + q < S) {
#pragma unroll
                    for (int k = 0; k < NV; k++) { u[k].x += a[q][k].x; u[k].y += a[q][k].y; u[k].z += a[q][k].z; u[k].w += a[q][k].w; }
                }
        }
        const float2 st = reg_stats(u, nvec, D, peps, rms, scratch);
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < nvec) {
                const float4 g = ld_w4(pw, p_dt, i);
                float4 n = make_float4((u[k].x - st.x) * st.y * g.x, (u[k].y - st.x) * st.y * g.y,
                                       (u[k].z - st.x) * st.y * g.z, (u[k].w - st.x) * st.y * g.w);
                if (!rms && pb != nullptr) { const float4 c = ld_w4(pb, p_dt, i); n.x += c.x; n.y += c.y; n.z += c.z; n.w += c.w; }
                v[k].x += mult * n.x; v[k].y += mult * n.y; v[k].z += mult * n.z; v[k].w += mult * n.w;
                xr[i] = v[k];
            }
        }
    }
    if (out == nullptr) return;
    const float2 st = w == nullptr ? make_float2(0.f, 1.f) : reg_stats(v, nvec, D, eps, rms, scratch);
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nvec) {
            const float4 g = w == nullptr ? make_float4(1.f, 1.f, 1.f, 1.f) : ld_w4(w, w_dt, i);
            float4 n = make_float4((v[k].x - st.x) * st.y * g.x, (v[k].y - st.x) * st.y * g.y,
                                   (v[k].z - st.x) * st.y * g.z, (v[k].w - st.x) * st.y * g.w);
            if (!rms && b != nullptr && w != nullptr) { const float4 c = ld_w4(b, w_dt, i); n.x += c.x; n.y += c.y; n.z += c.z; n.w += c.w; }
            TO* o = out + (size_t)r * D + 4 * i;
            if (sizeof(TO) == 4) {
                *reinterpret_cast<float4*>(o) = n;
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(n.x, n.y), hi = __floats2bfloat162_rn(n.z, n.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(o) = pk;
            }
        }
    }
}

// x float32 [T, D].  y (or null): float32 [max(S,1)][T][D] (S = 0 or 1: one tensor; S > 1: partial sums), with its norm
// (pw, pb, p_dt, peps) and the factor mult.  out (or null): [R, D] of type out_dt with its norm (w, b, w_dt, eps);
// rows (or null) gathers input rows for `out` and cannot be combined with y.
GFB_API int gfb_layernorm(float* x, const float* y, int S, long slice, const void* pw, const void* pb, int p_dt, float peps,
                          float mult, const void* w, const void* b, int w_dt, float eps, void* out, int out_dt,
                          const int* rows, int R, int D, int rms, cudaStream_t stream) {
    if (R <= 0 || D <= 0) return 0;
    if (y != nullptr && rows != nullptr) return gfb_fail("gfb_layernorm: a branch sum cannot be combined with a row gather");
    if (y == nullptr && out == nullptr) return 0;
    if ((size_t)D * sizeof(float) > 200 * 1024) return gfb_fail("gfb_layernorm: a row of %d elements does not fit shared memory", D);
    cudaError_t e;
    const bool aligned = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)out | (uintptr_t)w | (uintptr_t)b | (uintptr_t)pw | (uintptr_t)pb) & 15) == 0;
    if (D % 4 == 0 && slice % 4 == 0 && aligned && D <= 4 * LN_VEC * 256) {
        // few rows: many threads (up to 256) with few vectors each (the row's latency is what counts); many rows:
        // fewer threads with up to eight, so that more rows are resident per SM
        int per = R <= 256 ? 2 : LN_VEC;
        if ((D / 4 + per - 1) / per > 256) per = (D / 4 + 255) / 256;
        per = per <= 2 ? 2 : per <= 4 ? 4 : LN_VEC;
        int vthreads = ((D / 4 + per - 1) / per + 31) / 32 * 32;
        if (vthreads < 64) vthreads = 64;
        if (vthreads > 256) vthreads = 256;
        if (D / 4 <= per * vthreads) {
#define VGO(TO, NV, W) e = gfb_launch(layernorm_vec_kernel<TO, NV, W>, dim3(R), dim3(vthreads), 0, stream, x, y, S, (size_t)slice, pw, pb, \
                                      p_dt, peps, mult, w, b, w_dt, eps, (TO*)out, rows, D, rms)
#define VPICK(TO) do { if (per == 2) VGO(TO, 2, 6); else if (per == 4) VGO(TO, 4, 3); else VGO(TO, 8, 1); } while (0)
            if (out == nullptr || out_dt == GFB_F32) VPICK(float);
            else if (out_dt == GFB_BF16) VPICK(__nv_bfloat16);
            else return gfb_fail("gfb_layernorm: unknown output type %d", out_dt);
#undef VPICK
#undef VGO
            return gfb_check(e, "gfb_layernorm (vector)");
        }
    }
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    const size_t smem = (size_t)D * sizeof(float);
#define GO(TO)                                                                                                         \
    do {                                                                                                               \
        static size_t allowed = 48 * 1024;                                                                             \
        if (smem > allowed) {                                                                                          \
            cudaFuncSetAttribute(layernorm_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);       \
            allowed = 200 * 1024;                                                                                      \
        }                                                                                                              \
        e = gfb_launch(layernorm_kernel<TO>, dim3(R), dim3(threads), smem, stream, x, y, S, (size_t)slice, pw, pb, p_dt, peps, \
                       mult, w, b, w_dt, eps, (TO*)out, rows, D, rms);                                                 \
    } while (0)
    if (out == nullptr || out_dt == GFB_F32) GO(float);
    else if (out_dt == GFB_BF16) GO(__nv_bfloat16);
    else return gfb_fail("gfb_layernorm: unknown output type %d", out_dt);
#undef GO
    return gfb_check(e, "gfb_layernorm");
}

// ---------------------------------------------------------------- one row, several norms ---------
// For blocks whose sublayers all read the SAME normed row (parallel blocks): per row
//   (1) x[row] += sum_b s_b * y_b[row]      up to two branches, each a 32-bit tensor or the partial sums of a
//                                           product split over K (added in ascending order), each with a
//                                           per-column factor s_b (or none); written back
//   (2) out_k[r] = (x - mean) / sqrt(var + eps_k) * w_k      up to two outputs from ONE mean and variance
// The row sits in shared memory; statistics are 32-bit, the variance is the mean of squared deviations.
struct LnBranch {
    const float* y;      // [max(S, 1)][T][D], or null
    int S;
    const void* scale;   // [D] of type scale_dt, or null
};
struct LnOut {
    const void* w;       // [D] of type w_dt
    float eps;
    void* out;           // [R][D], or null
};

template <typename TO>
__global__ void layernorm_multi_kernel(float* __restrict__ x, LnBranch b0, LnBranch b1, int scale_dt, size_t slice,
                                       LnOut o0, LnOut o1, int w_dt, const int* __restrict__ rows, int D, int rms) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int r = blockIdx.x;
    const size_t base = (size_t)(rows ? rows[r] : r) * D;
    const bool sums = b0.y != nullptr || b1.y != nullptr;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        float v = x[base + i];
        if (b0.y != nullptr) {
            float u = b0.y[base + i];
            for (int k = 1; k < b0.S; k++) u += b0.y[(size_t)k * slice + base + i];
            v += b0.scale != nullptr ? ld_w(b0.scale, scale_dt, i) * u : u;
        }
        if (b1.y != nullptr) {
            float u = b1.y[base + i];
            for (int k = 1; k < b1.S; k++) u += b1.y[(size_t)k * slice + base + i];
            v += b1.scale != nullptr ? ld_w(b1.scale, scale_dt, i) * u : u;
        }
        if (sums) x[base + i] = v;
        row[i] = v;
    }
    if (o0.out == nullptr && o1.out == nullptr) return;
    __syncthreads();
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) s += row[i];
        mean = gfb_block_sum(s, scratch) / (float)D;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float dv = row[i] - mean; ss += dv * dv; }
    const float var = gfb_block_sum(ss, scratch) / (float)D;
    if (o0.out != nullptr) {
        const float rstd = 1.0f / sqrtf(var + o0.eps);
        TO* o = (TO*)o0.out + (size_t)r * D;
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_from_f32<TO>((row[i] - mean) * rstd * ld_w(o0.w, w_dt, i));
    }
    if (o1.out != nullptr) {
        const float rstd = 1.0f / sqrtf(var + o1.eps);
        TO* o = (TO*)o1.out + (size_t)r * D;
        for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = gfb_from_f32<TO>((row[i] - mean) * rstd * ld_w(o1.w, w_dt, i));
    }
}

// x float32 [T, D].  Branch b (y_b null: none): float32 [max(S_b,1)][T][D] with the per-column factor scale_b ([D] of
// scale_dt, or null).  Output k (out_k null: none): [R, D] of out_dt = norm of the new x with weight w_k and eps_k.
// rows (or null) gathers input rows and cannot be combined with a branch.
GFB_API int gfb_layernorm_multi(float* x, const float* y0, int S0, const void* scale0, const float* y1, int S1,
                                const void* scale1, int scale_dt, long slice, const void* w0, float eps0, void* out0,
                                const void* w1, float eps1, void* out1, int w_dt, int out_dt, const int* rows, int R, int D,
                                int rms, cudaStream_t stream) {
    if (R <= 0 || D <= 0) return 0;
    if ((y0 != nullptr || y1 != nullptr) && rows != nullptr) return gfb_fail("gfb_layernorm_multi: a branch sum cannot be combined with a row gather");
    if (y0 == nullptr && y1 == nullptr && out0 == nullptr && out1 == nullptr) return 0;
    if ((size_t)D * sizeof(float) > 200 * 1024) return gfb_fail("gfb_layernorm_multi: a row of %d elements does not fit shared memory", D);
    LnBranch b0{y0, S0, scale0}, b1{y1, S1, scale1};
    LnOut o0{w0, eps0, out0}, o1{w1, eps1, out1};
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    const size_t smem = (size_t)D * sizeof(float);
    cudaError_t e;
#define GO(TO)                                                                                                         \
    do {                                                                                                               \
        static size_t allowed = 48 * 1024;                                                                             \
        if (smem > allowed) {                                                                                          \
            cudaFuncSetAttribute(layernorm_multi_kernel<TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); \
            allowed = 200 * 1024;                                                                                      \
        }                                                                                                              \
        e = gfb_launch(layernorm_multi_kernel<TO>, dim3(R), dim3(threads), smem, stream, x, b0, b1, scale_dt,          \
                       (size_t)slice, o0, o1, w_dt, rows, D, rms);                                                     \
    } while (0)
    if ((out0 == nullptr && out1 == nullptr) || out_dt == GFB_F32) GO(float);
    else if (out_dt == GFB_BF16) GO(__nv_bfloat16);
    else return gfb_fail("gfb_layernorm_multi: unknown output type %d", out_dt);
#undef GO
    return gfb_check(e, "gfb_layernorm_multi");
}
