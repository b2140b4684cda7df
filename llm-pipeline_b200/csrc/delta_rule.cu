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
// sigmoid. delta_scan: a block owns (request, head, a range of value columns) and walks the request's tokens in order;
// lane (j, r) holds rows r, r + R, .. of column j in registers. The state lives in the request's slot as two copies that
// take turns by the parity of the last position written. Everything is float32.
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

constexpr int DS_THREADS = 128;   // threads of a block that hold the state; one more warp copies the inputs
constexpr int DS_COPY_WARPS = 4;   // warps that copy the inputs, one per scheduler: a single warp's chain of addresses and copies was the bound
constexpr int DS_STAGES = 3;      // stages of the input ring

__device__ __forceinline__ void ds_cp_async_4(float* smem_dst, const float* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void ds_cp_async_16(float* smem_dst, const float* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
// `n` floats from global to shared memory by the lanes of one warp, in 16-byte pieces where `vec` says both are aligned
__device__ __forceinline__ void ds_copy_row(float* dst, const float* src, int n, bool vec, int lane) {
    if (vec) for (int e = lane * 4; e < n; e += 128) ds_cp_async_16(dst + e, src + e);
    else for (int e = lane; e < n; e += 32) ds_cp_async_4(dst + e, src + e);
}

template <int V> struct DsVec { float v[V]; };
template <int V> __device__ __forceinline__ DsVec<V> ds_load(const float* p) {
    DsVec<V> r;
    if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
    else if constexpr (V == 2) { const float2 t = *reinterpret_cast<const float2*>(p); r.v[0] = t.x; r.v[1] = t.y; }
    else r.v[0] = *p;
    return r;
}

// A block owns (request, head, a range of value columns); the columns of the state never meet, so nothing passes
// between blocks. Within a warp, R consecutive lanes share a column: lane (column, r) holds NT state rows of its column
// in registers, in runs of V = min(NT, 4) rows (run i of lane r: rows (i R + r) V ..), so that a lane reads its keys,
// queries and decays as 16-byte words and the lanes of a column read consecutive words; rows past d are zeros that
// stay zeros. The sums over rows are rounds of shuffles. Four more warps copy the tokens' inputs through a ring of
// DS_STAGES stages of `stage_tokens` tokens (cp.async, 16 bytes where the rows allow it), so a block synchronises once
// per stage, not per token, and the warps that hold the state do no address arithmetic for the copies.
template <int NT, int R>
__global__ void __launch_bounds__(DS_THREADS + 32 * DS_COPY_WARPS) delta_scan_kernel(const DeltaArgs a, const int stage_tokens, const int vec) {
    extern __shared__ __align__(16) float smem[];
    constexpr int V = NT < 4 ? NT : 4;
    constexpr int DP = NT * R;                           // rows with padding
    constexpr int COLS = DS_THREADS / R;                 // columns of a block
    constexpr int ROW = 3 * DP + COLS + 4;               // k, q, decay (padded), the block's columns of v, beta
    const int r = blockIdx.x, h = blockIdx.y;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    if (end <= begin) return;
    const int d = a.d, dv = a.dv;
    const bool loader = threadIdx.x >= DS_THREADS;
    const int copy_warp = ((int)threadIdx.x - DS_THREADS) >> 5;      // which of the copying warps (negative for the others)
    const int lane = threadIdx.x & 31;
    const int rr = threadIdx.x % R, col = (threadIdx.x / R) % COLS;
    const int j0 = blockIdx.z * COLS, j = j0 + col;
    const bool valid = !loader && j < dv;
    const int g = h / (a.H / a.G);
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot + (size_t)h * d * dv;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + end - begin - 1) & 1) * a.state_half;
    float S[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int c = ((i / V) * R + rr) * V + i % V;
        S[i] = (valid && c < d) ? rd[(size_t)c * dv + j] : 0.f;
    }
    // the padding of every row of the ring, once: keys and queries 0, decay 1, values 0
    for (int i = threadIdx.x; i < DS_STAGES * stage_tokens * ROW; i += blockDim.x) {
        const int e = i % ROW;
        smem[i] = (e >= 2 * DP && e < 3 * DP) ? 1.f : 0.f;
    }
    __syncthreads();
    const int ncols = min(COLS, dv - j0);
    const int stages = (end - begin + stage_tokens - 1) / stage_tokens;
    auto issue = [&](int s) {                            // the copying warp only
        if (s < stages) {
            float* dst0 = smem + (size_t)(s % DS_STAGES) * stage_tokens * ROW;
            const int t0 = begin + s * stage_tokens;
            const int cnt = min(stage_tokens, end - t0);
            for (int tt = copy_warp; tt < cnt; tt += DS_COPY_WARPS) {
                const int t = t0 + tt;
                float* dst = dst0 + (size_t)tt * ROW;
                ds_copy_row(dst, a.k + (size_t)t * a.k_t + (size_t)g * d, d, vec & 1, lane);
                ds_copy_row(dst + DP, a.q + (size_t)t * a.q_t + (size_t)g * d, d, vec & 1, lane);
                ds_copy_row(dst + 2 * DP, a.decay + (size_t)t * a.decay_t + (size_t)h * d, d, vec & 2, lane);
                ds_copy_row(dst + 3 * DP, a.v + (size_t)t * a.v_t + (size_t)h * dv + j0, ncols, vec & 4, lane);
                if (lane == 0) ds_cp_async_4(dst + 3 * DP + COLS, a.beta + (size_t)t * a.beta_t + h);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    if (loader) { issue(0); issue(1); }
    for (int s = 0; s < stages; ++s) {
        if (loader) asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        __syncthreads();                                 // stage s is here; everyone has left stage s - 1
        if (loader) {
            issue(s + 2);                                // into the buffer of stage s - 1
            continue;
        }
        const float* base = smem + (size_t)(s % DS_STAGES) * stage_tokens * ROW;
        const int t0 = begin + s * stage_tokens;
        const int cnt = min(stage_tokens, end - t0);
        for (int tt = 0; tt < cnt; ++tt) {
            const float* cur = base + (size_t)tt * ROW;
            float kc[NT];
            float sk[2] = {0.f, 0.f}, sq[2] = {0.f, 0.f}, kq = 0.f;
#pragma unroll
            for (int i4 = 0; i4 < NT / V; ++i4) {
                const int at = (i4 * R + rr) * V;
                const DsVec<V> kk = ds_load<V>(cur + at), qq = ds_load<V>(cur + DP + at), gg = ds_load<V>(cur + 2 * DP + at);
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const int i = i4 * V + e;
                    kc[i] = kk.v[e];
                    S[i] *= gg.v[e];
                    sk[e & 1] = fmaf(S[i], kk.v[e], sk[e & 1]);
                    sq[e & 1] = fmaf(S[i], qq.v[e], sq[e & 1]);
                    kq = fmaf(kk.v[e], qq.v[e], kq);
                }
            }
            float sks = sk[0] + sk[1], sqs = sq[0] + sq[1];
#pragma unroll
            for (int m = R >> 1; m > 0; m >>= 1) {
                sks += __shfl_xor_sync(0xffffffffu, sks, m);
                sqs += __shfl_xor_sync(0xffffffffu, sqs, m);
                kq += __shfl_xor_sync(0xffffffffu, kq, m);
            }
            const float u = cur[3 * DP + COLS] * (cur[3 * DP + col] - sks);
#pragma unroll
            for (int i = 0; i < NT; ++i) S[i] = fmaf(kc[i], u, S[i]);
            if (rr == 0 && valid) a.o[(size_t)(t0 + tt) * a.o_t + (size_t)h * dv + j] = fmaf(u, kq, sqs);
        }
    }
    if (loader) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (valid) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int c = ((i / V) * R + rr) * V + i % V;
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
    LLMP_REQUIRE((dv + 3) / 4 <= 65535, "delta_scan: too many value columns %d", dv);
    DeltaArgs a;
    a.q = q; a.q_t = q_t; a.k = k; a.k_t = k_t; a.v = v; a.v_t = v_t; a.decay = decay; a.decay_t = decay_t;
    a.beta = beta; a.beta_t = beta_t; a.state = state; a.state_slot = state_slot; a.state_half = state_half;
    a.q_start = q_start; a.slots = slots; a.positions = positions; a.o = o; a.o_t = o_t; a.H = H; a.G = G; a.d = d; a.dv = dv;
    // lanes that share a column: the fewest (a power of two up to 32) that leave a lane at most 16 rows (32 past 512 rows)
    int rows = 1;
    while (rows < 32 && (d + rows - 1) / rows > 16) rows *= 2;
    const int per = (d + rows - 1) / rows;
    LLMP_REQUIRE(per <= 32, "delta_scan: a state of %d rows does not fit the registers of a warp", d);
    int nt = 1;
    while (nt < per) nt *= 2;
    if (rows > 1) nt = nt < 16 ? 16 : nt;
    const int cols = DS_THREADS / rows;
    const size_t row_bytes = (size_t)(3 * nt * rows + cols + 4) * sizeof(float);
    int stage_tokens = 8;
    while (stage_tokens > 1 && DS_STAGES * stage_tokens * row_bytes > 96 * 1024) stage_tokens /= 2;
    const size_t smem = DS_STAGES * stage_tokens * row_bytes;
    LLMP_REQUIRE(smem <= 200 * 1024, "delta_scan: heads of %d x %d do not fit shared memory", d, dv);
    auto aligned = [](const void* p, long stride) { return ((uintptr_t)p & 15) == 0 && stride % 4 == 0; };
    int vec = 0;
    if (d % 4 == 0 && aligned(q, q_t) && aligned(k, k_t)) vec |= 1;
    if (d % 4 == 0 && aligned(decay, decay_t)) vec |= 2;
    if (dv % 4 == 0 && (nt * rows) % 4 == 0 && aligned(v, v_t)) vec |= 4;     // the columns' place in a ring row is aligned too
    dim3 grid(R, H, (dv + cols - 1) / cols);
#define LLMP_DELTA(NT, RW)                                                                          \
    if (nt == NT && rows == RW) {                                                                   \
        LLMP_ALLOW_SMEM((delta_scan_kernel<NT, RW>), smem);                                         \
        delta_scan_kernel<NT, RW><<<grid, DS_THREADS + 32 * DS_COPY_WARPS, smem, stream>>>(a, stage_tokens, vec);   \
    } else
    LLMP_DELTA(1, 1) LLMP_DELTA(2, 1) LLMP_DELTA(4, 1) LLMP_DELTA(8, 1) LLMP_DELTA(16, 1) LLMP_DELTA(16, 2) LLMP_DELTA(16, 4)
    LLMP_DELTA(16, 8) LLMP_DELTA(16, 16) LLMP_DELTA(16, 32) LLMP_DELTA(32, 32)
    {
        llmp_set_error("delta_scan: no instance for %d rows a lane on %d lanes", nt, rows);
        return 1;
    }
#undef LLMP_DELTA
    return llmp_check_launch("delta_scan");
}
