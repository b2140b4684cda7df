// Residual add and RMS norm with several weights: a block of layers whose sublayers read differently weighted norms of
// the same residual takes all of them from one pass over the row.
//
//   x = residual + ((a + bias) + b)        a, b: the pending outputs of two sublayers (each optional, float32 or compute type)
//   residual <- x                           (unless `rows` selects rows: then the residual stays as it is)
//   out[j] = x / sqrt(mean(x^2) + eps) * w[j]      j = 0 .. k - 1; entry i of row m at out + j * out_block + m * out_row + i
//                                                  (matrices of their own, or side by side in one row)
// All arithmetic is float32; the outputs are float32 or the compute type. One block per row; the row stays in registers
// up to 4,096 entries and is recomputed from its sources beyond.
#include "common.cuh"

namespace {

constexpr int NM_THREADS = 256;
constexpr int NM_REGS = 16;

struct NormMultiArgs {
    float* residual;
    const void* a; int a_bf16;
    const void* b; int b_bf16;
    const void* bias; int bias_bf16;
    const void* w; int w_bf16; int k;
    float eps;
    void* out; int out_bf16; long out_block; long out_row;
    const int* rows;
    int D;
};

__device__ __forceinline__ float nm_value(const NormMultiArgs& p, size_t row, int i) {
    float add = 0.f;
    bool any = false;
    if (p.a) { add = load_as_float(p.a, p.a_bf16, row * p.D + i); any = true; }
    if (p.bias) { add += load_as_float(p.bias, p.bias_bf16, i); any = true; }
    if (p.b) { add += load_as_float(p.b, p.b_bf16, row * p.D + i); any = true; }
    const float r = p.residual[row * p.D + i];
    return any ? r + add : r;
}

__global__ void __launch_bounds__(NM_THREADS) add_rmsnorm_multi_kernel(const NormMultiArgs p) {
    __shared__ float scratch[32];
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const int m = blockIdx.x;
    const size_t row = p.rows ? (size_t)p.rows[m] : (size_t)m;
    const int D = p.D;
    const bool in_regs = D <= NM_THREADS * NM_REGS;
    float xr[NM_REGS];
    float ss = 0.f;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NM_REGS; ++j) {
            const int i = threadIdx.x + j * NM_THREADS;
            xr[j] = i < D ? nm_value(p, row, i) : 0.f;
            ss = fmaf(xr[j], xr[j], ss);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += NM_THREADS) {
            const float v = nm_value(p, row, i);
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(ss / (float)D + p.eps);
    const bool keep = p.rows == nullptr && (p.a || p.b || p.bias);
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NM_REGS; ++j) {
            const int i = threadIdx.x + j * NM_THREADS;
            if (i < D) {
                const float v = xr[j];
                for (int q = 0; q < p.k; ++q) {
                    const float o = v * rstd * load_as_float(p.w, p.w_bf16, (size_t)q * D + i);
                    const size_t at = (size_t)q * p.out_block + (size_t)m * p.out_row + i;
                    if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(o);
                    else reinterpret_cast<float*>(p.out)[at] = o;
                }
                if (keep) p.residual[row * D + i] = v;
            }
        }
    } else {
        for (int i = threadIdx.x; i < D; i += NM_THREADS) {
            const float v = nm_value(p, row, i);
            for (int q = 0; q < p.k; ++q) {
                const float o = v * rstd * load_as_float(p.w, p.w_bf16, (size_t)q * D + i);
                const size_t at = (size_t)q * p.out_block + (size_t)m * p.out_row + i;
                if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(o);
                else reinterpret_cast<float*>(p.out)[at] = o;
            }
            if (keep) p.residual[row * D + i] = v;
        }
    }
}

// The same with 16-byte accesses, for widths that are multiples of 4 up to 4,096 and aligned operands: a thread keeps up
// to four pieces of four entries in registers.
constexpr int NM_PIECES = 4;

__device__ __forceinline__ float4 nm_load4(const void* p, int is_bf16, size_t i4) {
    if (!is_bf16) return reinterpret_cast<const float4*>(p)[i4];
    const uint2 raw = reinterpret_cast<const uint2*>(p)[i4];
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

__global__ void __launch_bounds__(NM_THREADS) add_rmsnorm_multi_vec_kernel(const NormMultiArgs p) {
    __shared__ float scratch[32];
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const int m = blockIdx.x;
    const size_t row = p.rows ? (size_t)p.rows[m] : (size_t)m;
    const int D4 = p.D >> 2;
    const bool any = p.a || p.b || p.bias;
    float4 x[NM_PIECES];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NM_PIECES; ++j) {
        const int i = threadIdx.x + j * NM_THREADS;
        x[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < D4) {
            float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.a) add = nm_load4(p.a, p.a_bf16, row * D4 + i);
            if (p.bias) { const float4 v = nm_load4(p.bias, p.bias_bf16, i); add.x += v.x; add.y += v.y; add.z += v.z; add.w += v.w; }
            if (p.b) { const float4 v = nm_load4(p.b, p.b_bf16, row * D4 + i); add.x += v.x; add.y += v.y; add.z += v.z; add.w += v.w; }
            const float4 r = reinterpret_cast<const float4*>(p.residual)[row * D4 + i];
            x[j] = any ? make_float4(r.x + add.x, r.y + add.y, r.z + add.z, r.w + add.w) : r;
            ss = fmaf(x[j].x, x[j].x, ss); ss = fmaf(x[j].y, x[j].y, ss); ss = fmaf(x[j].z, x[j].z, ss); ss = fmaf(x[j].w, x[j].w, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.f / sqrtf(ss / (float)p.D + p.eps);
    const bool keep = p.rows == nullptr && any;
#pragma unroll
    for (int j = 0; j < NM_PIECES; ++j) {
        const int i = threadIdx.x + j * NM_THREADS;
        if (i < D4) {
            for (int q = 0; q < p.k; ++q) {
                const float4 w = nm_load4(p.w, p.w_bf16, (size_t)q * D4 + i);
                const float4 o = make_float4(x[j].x * rstd * w.x, x[j].y * rstd * w.y, x[j].z * rstd * w.z, x[j].w * rstd * w.w);
                const size_t at = ((size_t)q * p.out_block + (size_t)m * p.out_row) / 4 + i;
                if (p.out_bf16) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                    reinterpret_cast<uint2*>(p.out)[at] = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
                } else {
                    reinterpret_cast<float4*>(p.out)[at] = o;
                }
            }
            if (keep) reinterpret_cast<float4*>(p.residual)[row * D4 + i] = x[j];
        }
    }
}

}  // namespace

LLMP_API int llmp_add_rmsnorm_multi(float* residual, const void* a, int a_dtype, const void* b, int b_dtype, const void* bias,
                                    int bias_dtype, const void* w, int w_dtype, int k, float eps, void* out, int out_dtype,
                                    long out_block, long out_row, const int* rows, int M, int D, cudaStream_t stream) {
    if (M <= 0) return 0;
    LLMP_REQUIRE(D > 0 && k >= 1 && k <= 8 && out_row >= D && out_block >= D, "add_rmsnorm_multi: bad sizes rows=%d width=%d weights=%d", M, D, k);
    NormMultiArgs p;
    p.residual = residual; p.a = a; p.a_bf16 = a_dtype == LLMP_BF16; p.b = b; p.b_bf16 = b_dtype == LLMP_BF16;
    p.bias = bias; p.bias_bf16 = bias_dtype == LLMP_BF16; p.w = w; p.w_bf16 = w_dtype == LLMP_BF16; p.k = k; p.eps = eps;
    p.out = out; p.out_bf16 = out_dtype == LLMP_BF16; p.out_block = out_block; p.out_row = out_row; p.rows = rows; p.D = D;
    auto aligned = [](const void* q, int bf) { return q == nullptr || ((size_t)q % (bf ? 8 : 16)) == 0; };
    const bool vec = D % 4 == 0 && D <= 4 * NM_THREADS * NM_PIECES && out_block % 4 == 0 && out_row % 4 == 0 && aligned(residual, 0) &&
                     aligned(a, p.a_bf16) && aligned(b, p.b_bf16) && aligned(bias, p.bias_bf16) && aligned(w, p.w_bf16) && aligned(out, p.out_bf16);
    if (vec) llmp_launch_dependent(add_rmsnorm_multi_vec_kernel, dim3(M), dim3(NM_THREADS), 0, stream, p);
    else llmp_launch_dependent(add_rmsnorm_multi_kernel, dim3(M), dim3(NM_THREADS), 0, stream, p);
    return llmp_check_launch("add_rmsnorm_multi");
}
