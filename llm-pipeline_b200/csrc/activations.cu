// Activations and small sums that have no better home.
//
//   xielu:       out = f(z + bias), f(v) = ap v^2 + v / 2 for v > 0, an (exp(v) - 1 - v) + v / 2 for v <= 0;
//                z float32 [rows, F], bias optional, out in the compute type.
//   scaled_sum:  out = sa a + sb b, float32 (the results of two mixers that ran side by side).
//   gated_act:   out = act(gate) * up for rows [gate | up] of 2 F entries (float32 or the compute type), act = the tanh form
//                of GELU, 0.5 v (1 + tanh(sqrt(2 / pi) (v + 0.044715 v^3))), or SiLU; float32 arithmetic, out in the compute type.
//   sigmoid_gate: out = x * sigmoid(g), g float32 rows (a view), x and out in the compute type (out may be x).
//   convert_rows: out = in for float32 rows (a view) into dense rows of the compute type.
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

template <typename TI, typename T>
__global__ void gated_act_kernel(const TI* __restrict__ gu, long gu_t, T* __restrict__ out, size_t total, int F, int act) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / F;
    const int c = (int)(i % F);
    const float g = to_float(gu[row * gu_t + c]), u = to_float(gu[row * gu_t + F + c]);
    float v;
    if (act == 1) v = 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else v = g / (1.f + expf(-g));
    out[i] = from_float<T>(v * u);
}

// four entries a thread: float32 rows in 16-byte pieces, bfloat16 out in 8-byte pieces
__global__ void gated_act_vec_kernel(const float* __restrict__ gu, long gu_t, bf16* __restrict__ out, size_t total4, int F4, int act) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const size_t row = i / F4;
    const int c = (int)(i % F4);
    const float4 g = reinterpret_cast<const float4*>(gu + row * gu_t)[c], u = reinterpret_cast<const float4*>(gu + row * gu_t)[F4 + c];
    const float gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
    float r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float v = gs[k];
        const float a = act == 1 ? 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))) : v / (1.f + expf(-v));
        r[k] = a * us[k];
    }
    const __nv_bfloat162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
    reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
}

template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ x, const float* __restrict__ g, long g_t, T* __restrict__ out, size_t total, int C) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float gv = g[(i / C) * g_t + i % C];
    out[i] = from_float<T>(to_float(x[i]) / (1.f + expf(-gv)));
}

// four entries a thread: bfloat16 rows in 8-byte pieces, the float32 gate in 16-byte pieces
__global__ void sigmoid_gate_vec_kernel(const bf16* __restrict__ x, const float* __restrict__ g, long g_t, bf16* __restrict__ out, size_t total4, int C4) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const float4 gv = reinterpret_cast<const float4*>(g + (i / C4) * g_t)[i % C4];
    const uint2 raw = reinterpret_cast<const uint2*>(x)[i];
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const __nv_bfloat162 a = __floats2bfloat162_rn(__low2float(lo) / (1.f + expf(-gv.x)), __high2float(lo) / (1.f + expf(-gv.y)));
    const __nv_bfloat162 b = __floats2bfloat162_rn(__low2float(hi) / (1.f + expf(-gv.z)), __high2float(hi) / (1.f + expf(-gv.w)));
    reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b));
}

template <typename T>
__global__ void convert_rows_kernel(const float* __restrict__ in, long in_t, T* __restrict__ out, size_t total, int C) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) out[i] = from_float<T>(in[(i / C) * in_t + i % C]);
}

}  // namespace

LLMP_API int llmp_gated_act(const void* gu, int in_dtype, long gu_t, void* out, int out_dtype, long rows, int F, int act,
                            cudaStream_t stream) {
    if (rows <= 0 || F <= 0) return 0;
    LLMP_REQUIRE(act == 0 || act == 1, "gated_act: unknown activation %d", act);
    LLMP_REQUIRE(in_dtype == LLMP_F32 || in_dtype == out_dtype, "gated_act: rows of the compute type give the compute type");
    const size_t total = (size_t)rows * F;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LLMP_F32) llmp_launch_dependent(gated_act_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, gu_t, (float*)out, total, F, act);
    else if (in_dtype == LLMP_F32 && F % 4 == 0 && gu_t % 4 == 0 && (size_t)gu % 16 == 0 && (size_t)out % 8 == 0)
        llmp_launch_dependent(gated_act_vec_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (const float*)gu, gu_t, (bf16*)out, total / 4, F / 4, act);
    else if (in_dtype == LLMP_F32) llmp_launch_dependent(gated_act_kernel<float, bf16>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, gu_t, (bf16*)out, total, F, act);
    else llmp_launch_dependent(gated_act_kernel<bf16, bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gu, gu_t, (bf16*)out, total, F, act);
    return llmp_check_launch("gated_act");
}

LLMP_API int llmp_sigmoid_gate(const void* x, const float* g, long g_t, void* out, int dtype, long rows, int C, cudaStream_t stream) {
    if (rows <= 0 || C <= 0) return 0;
    const size_t total = (size_t)rows * C;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == LLMP_BF16 && C % 4 == 0 && g_t % 4 == 0 && (size_t)g % 16 == 0 && (size_t)x % 8 == 0 && (size_t)out % 8 == 0)
        llmp_launch_dependent(sigmoid_gate_vec_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, stream, (const bf16*)x, g, g_t, (bf16*)out, total / 4, C / 4);
    else if (dtype == LLMP_BF16) llmp_launch_dependent(sigmoid_gate_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)x, g, g_t, (bf16*)out, total, C);
    else llmp_launch_dependent(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, g, g_t, (float*)out, total, C);
    return llmp_check_launch("sigmoid_gate");
}

LLMP_API int llmp_convert_rows(const float* in, long in_t, void* out, int out_dtype, long rows, int C, cudaStream_t stream) {
    if (rows <= 0 || C <= 0) return 0;
    const size_t total = (size_t)rows * C;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == LLMP_BF16) llmp_launch_dependent(convert_rows_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, in, in_t, (bf16*)out, total, C);
    else llmp_launch_dependent(convert_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, in, in_t, (float*)out, total, C);
    return llmp_check_launch("convert_rows");
}

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
