// Activations and small sums that have no better home.
//
//   xielu:       out = f(z + bias), f(v) = ap v^2 + v / 2 for v > 0, an (exp(v) - 1 - v) + v / 2 for v <= 0;
//                z float32 [rows, F], bias optional, out in the compute type.
//   scaled_sum:  out = sa a + sb b, float32 (the results of two mixers that ran side by side).
#include "common.cuh"

namespace {

template <typename T>
__global__ void xielu_kernel(const float* __restrict__ z, const void* __restrict__ bias, int bias_bf16, float ap, float an,
                             T* __restrict__ out, size_t total, int F) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = z[i];
    if (bias) v += load_as_float(bias, bias_bf16, i % F);
    const float r = v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
    out[i] = from_float<T>(r);
}

__global__ void scaled_sum_kernel(const float* __restrict__ a, float sa, const float* __restrict__ b, float sb,
                                  float* __restrict__ out, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = fmaf(sb, b[i], sa * a[i]);
}

}  // namespace

LLMP_API int llmp_xielu(const float* z, const void* bias, int bias_dtype, float ap, float an, void* out, int out_dtype,
                        long rows, int F, cudaStream_t stream) {
    if (rows <= 0 || F <= 0) return 0;
    const size_t total = (size_t)rows * F;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LLMP_BF16)
        xielu_kernel<bf16><<<blocks, 256, 0, stream>>>(z, bias, (int)(bias_dtype == LLMP_BF16), ap, an, (bf16*)out, total, F);
    else
        xielu_kernel<float><<<blocks, 256, 0, stream>>>(z, bias, (int)(bias_dtype == LLMP_BF16), ap, an, (float*)out, total, F);
    return llmp_check_launch("xielu");
}

LLMP_API int llmp_scaled_sum(const float* a, float sa, const float* b, float sb, float* out, long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    scaled_sum_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a, sa, b, sb, out, (size_t)total);
    return llmp_check_launch("scaled_sum");
}
