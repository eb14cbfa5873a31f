// Unary activations over a tensor, in place or to another tensor of the same type: the exact
// (erf) GELU, the tanh form of GELU, SiLU, and the square of ReLU.  Arithmetic is 32-bit.  Products apply the same
// functions in their epilogue where they can; this kernel serves the shapes that cannot.
// Also a sigmoid gate on the columns of a tensor, one gate per group of columns (a head, or a single column), and the
// last step of differential attention: the difference of a head's two maps, normed over the head.
#include "common.cuh"

GFB_DEFINE_LAST_ERROR()

enum { ACT_GELU = 4, ACT_GELU_TANH = 5, ACT_SILU = 6, ACT_RELU2 = 7 };     // numbered as the product kernels' epilogues

template <typename T>
__global__ void activation_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n, int kind) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float z = gfb_to_f32(x[i]);
    float r;
    if (kind == ACT_GELU) r = 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    else if (kind == ACT_GELU_TANH) r = 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    else if (kind == ACT_RELU2) { const float p = fmaxf(z, 0.f); r = p * p; }
    else r = z / (1.0f + expf(-z));
    out[i] = gfb_from_f32<T>(r);
}

GFB_API int gfb_activation(const void* x, void* out, int dt, long n, int kind, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind != ACT_GELU && kind != ACT_GELU_TANH && kind != ACT_SILU && kind != ACT_RELU2) return gfb_fail("gfb_activation: unknown activation %d", kind);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaError_t e;
    if (dt == GFB_BF16) e = gfb_launch(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, (size_t)n, kind);
    else if (dt == GFB_F32) e = gfb_launch(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, (float*)out, (size_t)n, kind);
    else return gfb_fail("gfb_activation: unknown type %d", dt);
    return gfb_check(e, "gfb_activation");
}

// y[t, c] *= sigmoid(gate[t, gate_off + c / group])
template <typename T, typename TG>
__global__ void sigmoid_gate_kernel(T* __restrict__ y, const TG* __restrict__ gate, int C, int ld_gate, int gate_off, int group, size_t n) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t t = i / C;
    const int c = (int)(i - t * C);
    const float z = gfb_to_f32(gate[t * ld_gate + gate_off + c / group]);
    y[i] = gfb_from_f32<T>(gfb_to_f32(y[i]) / (1.0f + expf(-z)));
}

// y [T, C] of type dt and gate [T, ld_gate] of type gate_dt (dt, or 32-bit); the gates of a row start at column gate_off, one per
// `group` columns of y.
GFB_API int gfb_sigmoid_gate(void* y, const void* gate, int dt, int gate_dt, int T, int C, int ld_gate, int gate_off, int group, cudaStream_t stream) {
    const size_t n = (size_t)T * C;
    if (n == 0) return 0;
    if (group < 1 || C % group) return gfb_fail("gfb_sigmoid_gate: groups of %d columns in rows of %d", group, C);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    cudaError_t e;
    if (dt == GFB_BF16 && gate_dt == GFB_BF16) e = gfb_launch(sigmoid_gate_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)y, (const __nv_bfloat16*)gate, C, ld_gate, gate_off, group, n);
    else if (dt == GFB_BF16 && gate_dt == GFB_F32) e = gfb_launch(sigmoid_gate_kernel<__nv_bfloat16, float>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)y, (const float*)gate, C, ld_gate, gate_off, group, n);
    else if (dt == GFB_F32 && gate_dt == GFB_F32) e = gfb_launch(sigmoid_gate_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (float*)y, (const float*)gate, C, ld_gate, gate_off, group, n);
    else return gfb_fail("gfb_sigmoid_gate: unsupported types %d and %d", dt, gate_dt);
    return gfb_check(e, "gfb_sigmoid_gate");
}

// a [T, H, 2, dv]: the outputs of a head's two score maps; out[t, h, :] = o / sqrt(mean(o^2) + eps) * out_scale with
// o = a[t, h, 0, :] - lambda a[t, h, 1, :].  A warp per (token, head); 32-bit.
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* __restrict__ a, T* __restrict__ out, long items, int dv, float lambda, float eps, float out_scale) {
    gfb_pdl_launch();
    gfb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= items) return;
    const T* a1 = a + (size_t)item * 2 * dv;
    const T* a2 = a1 + dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) {
        const float o = gfb_to_f32(a1[i]) - lambda * gfb_to_f32(a2[i]);
        ss = fmaf(o, o, ss);
    }
    ss = gfb_warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)dv + eps);
    T* dst = out + (size_t)item * dv;
    for (int i = lane; i < dv; i += 32) dst[i] = gfb_from_f32<T>((gfb_to_f32(a1[i]) - lambda * gfb_to_f32(a2[i])) * f);
}

GFB_API int gfb_diff_combine(const void* a, void* out, int dt, int T, int H, int dv, float lambda, float eps, float out_scale, cudaStream_t stream) {
    const long items = (long)T * H;
    if (items <= 0 || dv <= 0) return 0;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    cudaError_t e;
    if (dt == GFB_BF16) e = gfb_launch(diff_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, (const __nv_bfloat16*)a, (__nv_bfloat16*)out, items, dv, lambda, eps, out_scale);
    else if (dt == GFB_F32) e = gfb_launch(diff_combine_kernel<float>, dim3(blocks), dim3(128), 0, stream, (const float*)a, (float*)out, items, dv, lambda, eps, out_scale);
    else return gfb_fail("gfb_diff_combine: unknown type %d", dt);
    return gfb_check(e, "gfb_diff_combine");
}
