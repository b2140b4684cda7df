// The state-space recurrence with one scalar decay per head and token, and the gated group norm behind it.
//
// Per head h (group g = h / (H / G)), with x_t [P], B_t and C_t [N] of the token and S [N, P] the head's state:
//   dt = softplus(dt_raw[t, h] + dt_bias[h]),  a = exp(-exp(A_log[h]) * dt)
//   S <- a S + dt B_t x_t^T,   y_t = S^T C_t + D[h] x_t
// Everything is float32. A block owns (request, head) and walks the request's tokens in order; thread (p, r) holds the
// rows r, r + R, r + 2R .. of column p in registers, the partial sums over rows meet in shared memory. The state lives
// in the request's slot as two copies that take turns by the parity of the last position written.
//
// gated_group_norm: rows [tokens, W] cut into groups of `gs` entries.
//   mode 0: v = y * silu(gate);  out = v / sqrt(mean_group(v^2) + eps) * weight[column]
//   mode 1: out = y / sqrt(mean_group(y^2) + eps) * weight[column % gs] * sigmoid(gate)
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

struct ScanArgs {
    const float* xbc; long xbc_t;            // [tokens, H P + 2 G N]: x | B | C
    const float* dt; long dt_t;              // [tokens, >= H]
    const float* dt_bias; const float* a_log; const float* d_skip;    // [H]
    float* state; long state_slot; long state_half;                   // copy: [H][N][P]
    const int* q_start; const int* slots; const int* positions;
    float* y; long y_t;                      // [tokens, H P]
    int H, G, N, P;
};

template <int NT>
__global__ void ssd_scan_kernel(const ScanArgs a) {
    extern __shared__ float smem[];
    const int r = blockIdx.x, h = blockIdx.y;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    if (end <= begin) return;
    const int N = a.N, P = a.P;
    const int R = blockDim.x / P;                       // row groups; threads past R * P only help with the copies
    const int p = threadIdx.x % P, rr = threadIdx.x / P;
    const bool owner = rr < R;
    float* buf = smem;                                  // [2][2 N + P]: B, C, x of a token, two tokens in turn
    float* part = smem + 2 * (2 * N + P);               // [R][P]
    const int g = h / (a.H / a.G);
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot + (size_t)h * N * P;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + end - begin - 1) & 1) * a.state_half;
    float S[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int n = rr + i * R;
        S[i] = (owner && n < N) ? rd[(size_t)n * P + p] : 0.f;
    }
    const float neg_a = -expf(a.a_log[h]), bias = a.dt_bias[h], skip = a.d_skip[h];
    const size_t x_at = (size_t)h * P, b_at = (size_t)a.H * P + (size_t)g * N, c_at = b_at + (size_t)a.G * N;
    auto fetch = [&](int t, float* dst) {
        const float* row = a.xbc + (size_t)t * a.xbc_t;
        for (int i = threadIdx.x; i < 2 * N + P; i += blockDim.x)
            dst[i] = i < N ? row[b_at + i] : (i < 2 * N ? row[c_at + i - N] : row[x_at + i - 2 * N]);
    };
    fetch(begin, buf);
    for (int t = begin; t < end; ++t) {
        float* cur = buf + ((t - begin) & 1) * (2 * N + P);
        __syncthreads();
        const float dt = softplus_f(a.dt[(size_t)t * a.dt_t + h] + bias);
        const float decay = expf(neg_a * dt);
        const float xv = cur[2 * N + p];
        if (owner) {
            const float dx = dt * xv;
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int n = rr + i * R;
                if (n < N) {
                    S[i] = fmaf(decay, S[i], cur[n] * dx);
                    sum = fmaf(S[i], cur[N + n], sum);
                }
            }
            part[rr * P + p] = sum;
        }
        if (t + 1 < end) fetch(t + 1, buf + ((t + 1 - begin) & 1) * (2 * N + P));
        __syncthreads();
        if (rr == 0) {
            float y = 0.f;
            for (int i = 0; i < R; ++i) y += part[i * P + p];
            a.y[(size_t)t * a.y_t + x_at + p] = fmaf(skip, xv, y);
        }
    }
    if (owner) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int n = rr + i * R;
            if (n < N) wr[(size_t)n * P + p] = S[i];
        }
    }
}

struct NormArgs {
    const float* y; long y_t; const float* gate; long gate_t; const float* weight;
    void* out; long out_t; int tokens, W, gs, mode; float eps;
};

template <typename T>
__global__ void gated_group_norm_kernel(const NormArgs a) {
    const int groups = a.W / a.gs;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)a.tokens * groups) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(item / groups), c0 = (int)(item % groups) * a.gs;
    const float* y = a.y + (size_t)t * a.y_t + c0;
    const float* gate = a.gate + (size_t)t * a.gate_t + c0;
    float ss = 0.f;
    for (int i = lane; i < a.gs; i += 32) {
        float v = y[i];
        if (a.mode == 0) { const float z = gate[i]; v *= z / (1.f + expf(-z)); }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)a.gs + a.eps);
    T* out = reinterpret_cast<T*>(a.out) + (size_t)t * a.out_t + c0;
    for (int i = lane; i < a.gs; i += 32) {
        float v = y[i];
        const float z = gate[i];
        if (a.mode == 0) v = v * (z / (1.f + expf(-z))) * inv * a.weight[c0 + i];
        else v = v * inv * a.weight[i] * (1.f / (1.f + expf(-z)));
        out[i] = from_float<T>(v);
    }
}

}  // namespace

LLMP_API int llmp_ssd_scan(const float* xbc, long xbc_t, const float* dt, long dt_t, const float* dt_bias, const float* a_log,
                           const float* d_skip, float* state, long state_slot, long state_half, const int* q_start,
                           const int* slots, const int* positions, float* y, long y_t, int R, int H, int G, int N, int P,
                           cudaStream_t stream) {
    if (R <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && N > 0 && P > 0 && P <= 1024, "ssd_scan: bad sizes heads=%d groups=%d state=%d vdim=%d",
                 H, G, N, P);
    LLMP_REQUIRE(H <= 65535, "ssd_scan: too many heads %d", H);
    ScanArgs a;
    a.xbc = xbc; a.xbc_t = xbc_t; a.dt = dt; a.dt_t = dt_t; a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip;
    a.state = state; a.state_slot = state_slot; a.state_half = state_half; a.q_start = q_start; a.slots = slots;
    a.positions = positions; a.y = y; a.y_t = y_t; a.H = H; a.G = G; a.N = N; a.P = P;
    // threads in whole columns; the rows a thread holds are bounded by the registers a block of that size may use
    int threads = 0;
    const int choices[4][2] = {{256, 32}, {512, 32}, {256, 64}, {1024, 8}};
    for (int i = 0; i < 4 && !threads; ++i) {
        const int groups = choices[i][0] / P;
        if (groups > 0 && (N + groups - 1) / groups <= choices[i][1]) threads = choices[i][0];
    }
    LLMP_REQUIRE(threads > 0, "ssd_scan: a state of %d x %d does not fit the registers of a block", N, P);
    const int rows = threads / P;
    const int per = (N + rows - 1) / rows;
    const size_t smem = ((size_t)2 * (2 * N + P) + (size_t)rows * P) * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "ssd_scan: state size %d does not fit shared memory", N);
    dim3 grid(R, H);
#define LLMP_SCAN(NT)                                                  \
    do {                                                               \
        LLMP_ALLOW_SMEM(ssd_scan_kernel<NT>, smem);                    \
        ssd_scan_kernel<NT><<<grid, threads, smem, stream>>>(a);       \
    } while (0)
    if (per <= 8) LLMP_SCAN(8);
    else if (per <= 16) LLMP_SCAN(16);
    else if (per <= 32) LLMP_SCAN(32);
    else LLMP_SCAN(64);
#undef LLMP_SCAN
    return llmp_check_launch("ssd_scan");
}

LLMP_API int llmp_gated_group_norm(const float* y, long y_t, const float* gate, long gate_t, const float* weight, void* out,
                                   int out_dtype, long out_t, int tokens, int W, int gs, int mode, float eps,
                                   cudaStream_t stream) {
    if (tokens <= 0) return 0;
    LLMP_REQUIRE(W > 0 && gs > 0 && W % gs == 0 && (mode == 0 || mode == 1), "gated_group_norm: %d entries in groups of %d, mode %d",
                 W, gs, mode);
    NormArgs a;
    a.y = y; a.y_t = y_t; a.gate = gate; a.gate_t = gate_t; a.weight = weight; a.out = out; a.out_t = out_t;
    a.tokens = tokens; a.W = W; a.gs = gs; a.mode = mode; a.eps = eps;
    const long items = (long)tokens * (W / gs);
    const int warps = 4;
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    if (out_dtype == LLMP_BF16) gated_group_norm_kernel<bf16><<<blocks, warps * 32, 0, stream>>>(a);
    else gated_group_norm_kernel<float><<<blocks, warps * 32, 0, stream>>>(a);
    return llmp_check_launch("gated_group_norm");
}
