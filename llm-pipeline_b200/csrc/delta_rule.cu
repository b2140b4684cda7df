// The gated delta rule: a matrix state per head that decays channel by channel and is corrected along the current key.
//
// Per head h (query/key head g = h / (H / G)), with q_t, k_t [d] unit vectors (q also times d^(-1/2)), v_t [dv],
// beta_t in (0, 1) and decay_t [d] in (0, 1), S [d, dv] the head's state:
//   S <- diag(decay_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
// The read-out sees the token's own write: o_t = (diag(decay_t) S)^T q_t + u (k_t . q_t), so one pass over the state
// gives both products and the correction is added afterwards.
//
// delta_prep (a block per token, in place): q and k become unit vectors per head, x / sqrt(sum(x^2) + 1e-6), q also
// times d^(-1/2); the decay's pre-activation becomes exp(-exp(A_log[h]) * softplus(pre + dt_bias)); beta's becomes its
// sigmoid. delta_scan: a block owns (request, head) and walks the request's tokens in order; thread (j, r) holds rows
// r, r + R, .. of column j in registers. The state lives in the request's slot as two copies that take turns by the
// parity of the last position written. Everything is float32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_d(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

struct PrepArgs {
    float* q; long q_t; float* k; long k_t;       // [tokens, G d]
    float* decay; long decay_t;                   // [tokens, H d]
    float* beta; long beta_t;                     // [tokens, H]
    const float* a_log; const float* dt_bias;     // [H], [H d]
    int H, G, d;
};

__global__ void delta_prep_kernel(const PrepArgs a) {
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const float q_scale = 1.f / sqrtf((float)a.d);
    for (int item = warp; item < 2 * a.G; item += nw) {
        const bool is_q = item < a.G;
        float* row = is_q ? a.q + (size_t)t * a.q_t + (size_t)item * a.d : a.k + (size_t)t * a.k_t + (size_t)(item - a.G) * a.d;
        float ss = 0.f;
        for (int i = lane; i < a.d; i += 32) ss = fmaf(row[i], row[i], ss);
        ss = warp_sum(ss);
        const float f = (is_q ? q_scale : 1.f) / sqrtf(ss + 1e-6f);
        for (int i = lane; i < a.d; i += 32) row[i] *= f;
    }
    float* decay = a.decay + (size_t)t * a.decay_t;
    for (int i = threadIdx.x; i < a.H * a.d; i += blockDim.x)
        decay[i] = expf(-expf(a.a_log[i / a.d]) * softplus_d(decay[i] + a.dt_bias[i]));
    float* beta = a.beta + (size_t)t * a.beta_t;
    for (int i = threadIdx.x; i < a.H; i += blockDim.x) beta[i] = 1.f / (1.f + expf(-beta[i]));
}

struct DeltaArgs {
    const float* q; long q_t; const float* k; long k_t; const float* v; long v_t;
    const float* decay; long decay_t; const float* beta; long beta_t;
    float* state; long state_slot; long state_half;      // copy: [H][d][dv]
    const int* q_start; const int* slots; const int* positions;
    float* o; long o_t;                                  // [tokens, H dv]
    int H, G, d, dv;
};

template <int NT>
__global__ void delta_scan_kernel(const DeltaArgs a) {
    extern __shared__ float smem[];
    const int r = blockIdx.x, h = blockIdx.y;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    if (end <= begin) return;
    const int d = a.d, dv = a.dv;
    const int R = blockDim.x / dv;
    const int j = threadIdx.x % dv, rr = threadIdx.x / dv;
    const bool owner = rr < R;
    const int row = 3 * d + dv;                          // k, q, decay, v of a token
    float* buf = smem;                                   // [2][row]
    float* part = smem + 2 * row;                        // [R][2 dv + 1]: S^T k, S^T q, k . q
    const int ps = 2 * dv + 1;
    const int g = h / (a.H / a.G);
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot + (size_t)h * d * dv;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + end - begin - 1) & 1) * a.state_half;
    float S[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int c = rr + i * R;
        S[i] = (owner && c < d) ? rd[(size_t)c * dv + j] : 0.f;
    }
    auto fetch = [&](int t, float* dst) {
        const float* kr = a.k + (size_t)t * a.k_t + (size_t)g * d;
        const float* qr = a.q + (size_t)t * a.q_t + (size_t)g * d;
        const float* gr = a.decay + (size_t)t * a.decay_t + (size_t)h * d;
        const float* vr = a.v + (size_t)t * a.v_t + (size_t)h * dv;
        for (int i = threadIdx.x; i < row; i += blockDim.x)
            dst[i] = i < d ? kr[i] : (i < 2 * d ? qr[i - d] : (i < 3 * d ? gr[i - 2 * d] : vr[i - 3 * d]));
    };
    fetch(begin, buf);
    for (int t = begin; t < end; ++t) {
        const float* cur = buf + ((t - begin) & 1) * row;
        __syncthreads();
        const float beta = a.beta[(size_t)t * a.beta_t + h];
        if (owner) {
            float sk = 0.f, sq = 0.f, kq = 0.f;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int c = rr + i * R;
                if (c < d) {
                    S[i] *= cur[2 * d + c];
                    sk = fmaf(S[i], cur[c], sk);
                    sq = fmaf(S[i], cur[d + c], sq);
                    kq = fmaf(cur[c], cur[d + c], kq);
                }
            }
            part[rr * ps + j] = sk;
            part[rr * ps + dv + j] = sq;
            if (j == 0) part[rr * ps + 2 * dv] = kq;
        }
        if (t + 1 < end) fetch(t + 1, buf + ((t + 1 - begin) & 1) * row);
        __syncthreads();
        if (owner) {
            float sk = 0.f, sq = 0.f, kq = 0.f;
            for (int i = 0; i < R; ++i) {
                sk += part[i * ps + j];
                sq += part[i * ps + dv + j];
                kq += part[i * ps + 2 * dv];
            }
            const float u = beta * (cur[3 * d + j] - sk);
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int c = rr + i * R;
                if (c < d) S[i] = fmaf(cur[c], u, S[i]);
            }
            if (rr == 0) a.o[(size_t)t * a.o_t + (size_t)h * dv + j] = fmaf(u, kq, sq);
        }
    }
    if (owner) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int c = rr + i * R;
            if (c < d) wr[(size_t)c * dv + j] = S[i];
        }
    }
}

}  // namespace

LLMP_API int llmp_delta_prep(float* q, long q_t, float* k, long k_t, float* decay, long decay_t, float* beta, long beta_t,
                             const float* a_log, const float* dt_bias, int tokens, int H, int G, int d, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0, "delta_prep: bad sizes heads=%d qk_heads=%d dim=%d", H, G, d);
    PrepArgs a;
    a.q = q; a.q_t = q_t; a.k = k; a.k_t = k_t; a.decay = decay; a.decay_t = decay_t; a.beta = beta; a.beta_t = beta_t;
    a.a_log = a_log; a.dt_bias = dt_bias; a.H = H; a.G = G; a.d = d;
    delta_prep_kernel<<<tokens, 256, 0, stream>>>(a);
    return llmp_check_launch("delta_prep");
}

LLMP_API int llmp_delta_scan(const float* q, long q_t, const float* k, long k_t, const float* v, long v_t, const float* decay,
                             long decay_t, const float* beta, long beta_t, float* state, long state_slot, long state_half,
                             const int* q_start, const int* slots, const int* positions, float* o, long o_t, int R, int H,
                             int G, int d, int dv, cudaStream_t stream) {
    if (R <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && dv <= 1024 && H <= 65535,
                 "delta_scan: bad sizes heads=%d qk_heads=%d dim=%d vdim=%d", H, G, d, dv);
    DeltaArgs a;
    a.q = q; a.q_t = q_t; a.k = k; a.k_t = k_t; a.v = v; a.v_t = v_t; a.decay = decay; a.decay_t = decay_t;
    a.beta = beta; a.beta_t = beta_t; a.state = state; a.state_slot = state_slot; a.state_half = state_half;
    a.q_start = q_start; a.slots = slots; a.positions = positions; a.o = o; a.o_t = o_t; a.H = H; a.G = G; a.d = d; a.dv = dv;
    // threads in whole columns; the rows a thread holds are bounded by the registers a block of that size may use
    int threads = 0;
    const int choices[4][2] = {{256, 32}, {512, 32}, {256, 64}, {1024, 8}};
    for (int i = 0; i < 4 && !threads; ++i) {
        const int groups = choices[i][0] / dv;
        if (groups > 0 && (d + groups - 1) / groups <= choices[i][1]) threads = choices[i][0];
    }
    LLMP_REQUIRE(threads > 0, "delta_scan: a state of %d x %d does not fit the registers of a block", d, dv);
    const int rows = threads / dv;
    const int per = (d + rows - 1) / rows;
    const size_t smem = ((size_t)2 * (3 * d + dv) + (size_t)rows * (2 * dv + 1)) * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "delta_scan: heads of %d x %d do not fit shared memory", d, dv);
    dim3 grid(R, H);
#define LLMP_DELTA(NT)                                                   \
    do {                                                                 \
        LLMP_ALLOW_SMEM(delta_scan_kernel<NT>, smem);                    \
        delta_scan_kernel<NT><<<grid, threads, smem, stream>>>(a);       \
    } while (0)
    if (per <= 8) LLMP_DELTA(8);
    else if (per <= 16) LLMP_DELTA(16);
    else if (per <= 32) LLMP_DELTA(32);
    else LLMP_DELTA(64);
#undef LLMP_DELTA
    return llmp_check_launch("delta_scan");
}
