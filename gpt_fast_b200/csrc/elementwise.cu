// Unary activations over a tensor, in place or to another tensor of the same type: the exact
// (erf) GELU, the tanh form of GELU, SiLU, and the square of ReLU.  Arithmetic is 32-bit.  Products apply the same
// functions in their epilogue where they can; this kernel serves the shapes that cannot.
// Also a sigmoid gate on the columns of a tensor, one gate per group of columns (a head, or a single column).
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
