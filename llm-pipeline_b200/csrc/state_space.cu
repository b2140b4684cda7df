// The state-space recurrence with one scalar decay per head and token, and the gated group norm behind it.
//
// Per head h (group g = h / (H / G)), with x_t [P], B_t and C_t [N] of the token and S [N, P] the head's state:
//   dt = softplus(dt_raw[t, h] + dt_bias[h]),  a = exp(-exp(A_log[h]) * dt)
//   S <- a S + dt B_t x_t^T,   y_t = S^T C_t + D[h] x_t
// Everything is float32. A block owns (request, head, a range of columns) and walks the request's tokens in order; lane
// (p, r) holds the rows r, r + R, r + 2R .. of column p in registers, the sums over rows are shuffles. The state lives
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

constexpr int SS_THREADS = 128;   // threads of a block that hold the state; one more warp copies the inputs
constexpr int SS_COPY_WARPS = 4;   // warps that copy the inputs, one per scheduler: a single warp's chain of addresses and copies was the bound
constexpr int SS_STAGES = 3;      // stages of the input ring

__device__ __forceinline__ void ss_cp_async_4(float* smem_dst, const float* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void ss_cp_async_16(float* smem_dst, const float* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void ss_copy_row(float* dst, const float* src, int n, bool vec, int lane) {
    if (vec) for (int e = lane * 4; e < n; e += 128) ss_cp_async_16(dst + e, src + e);
    else for (int e = lane; e < n; e += 32) ss_cp_async_4(dst + e, src + e);
}

template <int V> struct SsVec { float v[V]; };
template <int V> __device__ __forceinline__ SsVec<V> ss_load(const float* p) {
    SsVec<V> r;
    if constexpr (V == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w; }
    else if constexpr (V == 2) { const float2 t = *reinterpret_cast<const float2*>(p); r.v[0] = t.x; r.v[1] = t.y; }
    else r.v[0] = *p;
    return r;
}

// A block owns (request, head, a range of the head's columns); the columns of the state never meet. Within a warp, R
// consecutive lanes share a column: lane (column, r) holds NT state rows of its column in registers, in runs of
// V = min(NT, 4) rows (run i of lane r: rows (i R + r) V ..), so that B and C are read as 16-byte words; rows past N
// see B = C = 0 and stay zero. The sum over rows is a round of shuffles. Four more warps copy the tokens' inputs
// through a ring of SS_STAGES stages of `stage_tokens` tokens (cp.async, 16 bytes where the rows allow it), a token
// each in turn, and the first of them turns each token's raw step size into (dt, decay) before the stage's barrier:
// one barrier per stage, not per token.
template <int NT, int R>
__global__ void __launch_bounds__(SS_THREADS + 32 * SS_COPY_WARPS) ssd_scan_kernel(const ScanArgs a, const int stage_tokens, const int vec) {
    extern __shared__ __align__(16) float smem[];
    constexpr int V = NT < 4 ? NT : 4;
    constexpr int NP = NT * R;                          // rows with padding
    constexpr int COLS = SS_THREADS / R;
    constexpr int ROW = 2 * NP + COLS + 4;              // B, C (padded), the block's columns of x, dt, decay
    const int r = blockIdx.x, h = blockIdx.y;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    if (end <= begin) return;
    const int N = a.N, P = a.P;
    const bool loader = threadIdx.x >= SS_THREADS;
    const int copy_warp = ((int)threadIdx.x - SS_THREADS) >> 5;      // which of the copying warps (negative for the others)
    const int lane = threadIdx.x & 31;
    const int rr = threadIdx.x % R, col = (threadIdx.x / R) % COLS;
    const int j0 = blockIdx.z * COLS, p = j0 + col;
    const bool valid = !loader && p < P;
    const int g = h / (a.H / a.G);
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot + (size_t)h * N * P;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + end - begin - 1) & 1) * a.state_half;
    float S[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int n = ((i / V) * R + rr) * V + i % V;
        S[i] = (valid && n < N) ? rd[(size_t)n * P + p] : 0.f;
    }
    for (int i = threadIdx.x; i < SS_STAGES * stage_tokens * ROW; i += blockDim.x) smem[i] = 0.f;
    __syncthreads();
    const float neg_a = -expf(a.a_log[h]), bias = a.dt_bias[h], skip = a.d_skip[h];
    const size_t x_at = (size_t)h * P, b_at = (size_t)a.H * P + (size_t)g * N, c_at = b_at + (size_t)a.G * N;
    const int ncols = min(COLS, P - j0);
    const int stages = (end - begin + stage_tokens - 1) / stage_tokens;
    auto issue = [&](int s) {                           // the copying warp only
        if (s < stages) {
            float* dst0 = smem + (size_t)(s % SS_STAGES) * stage_tokens * ROW;
            const int t0 = begin + s * stage_tokens;
            const int cnt = min(stage_tokens, end - t0);
            for (int tt = copy_warp; tt < cnt; tt += SS_COPY_WARPS) {
                const float* src = a.xbc + (size_t)(t0 + tt) * a.xbc_t;
                float* dst = dst0 + (size_t)tt * ROW;
                ss_copy_row(dst, src + b_at, N, vec & 1, lane);
                ss_copy_row(dst + NP, src + c_at, N, vec & 1, lane);
                ss_copy_row(dst + 2 * NP, src + x_at + j0, ncols, vec & 2, lane);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    if (loader) { issue(0); issue(1); }
    for (int s = 0; s < stages; ++s) {
        float* base = smem + (size_t)(s % SS_STAGES) * stage_tokens * ROW;
        const int t0 = begin + s * stage_tokens;
        const int cnt = min(stage_tokens, end - t0);
        if (loader) {
            for (int tt = lane; tt < cnt && copy_warp == 0; tt += 32) {   // step sizes and decays of the stage's tokens
                const float dt = softplus_f(a.dt[(size_t)(t0 + tt) * a.dt_t + h] + bias);
                base[(size_t)tt * ROW + 2 * NP + COLS] = dt;
                base[(size_t)tt * ROW + 2 * NP + COLS + 1] = expf(neg_a * dt);
            }
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        }
        __syncthreads();                                // stage s is here; everyone has left stage s - 1
        if (loader) {
            issue(s + 2);                               // into the buffer of stage s - 1
            continue;
        }
        for (int tt = 0; tt < cnt; ++tt) {
            const float* cur = base + (size_t)tt * ROW;
            const float dt = cur[2 * NP + COLS], decay = cur[2 * NP + COLS + 1];
            const float xv = cur[2 * NP + col];
            const float dx = dt * xv;
            float y[2] = {0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < NT / V; ++i4) {
                const int at = (i4 * R + rr) * V;
                const SsVec<V> bb = ss_load<V>(cur + at), cc = ss_load<V>(cur + NP + at);
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const int i = i4 * V + e;
                    S[i] = fmaf(decay, S[i], bb.v[e] * dx);
                    y[e & 1] = fmaf(S[i], cc.v[e], y[e & 1]);
                }
            }
            float ys = y[0] + y[1];
#pragma unroll
            for (int m = R >> 1; m > 0; m >>= 1) ys += __shfl_xor_sync(0xffffffffu, ys, m);
            if (rr == 0 && valid) a.y[(size_t)(t0 + tt) * a.y_t + x_at + p] = fmaf(skip, xv, ys);
        }
    }
    if (loader) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    if (valid) {
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int n = ((i / V) * R + rr) * V + i % V;
            if (n < N) wr[(size_t)n * P + p] = S[i];
        }
    }
}

struct NormArgs {
    const float* y; long y_t; const float* gate; long gate_t; const float* weight;
    void* out; long out_t; int tokens, W, gs, mode; float eps;
};

// TEAM: a warp takes a group (several groups a block), or the whole block takes one.
template <typename T, bool TEAM>
__global__ void gated_group_norm_kernel(const NormArgs a) {
    __shared__ float scratch[32];
    const int groups = a.W / a.gs;
    const long item = TEAM ? (long)blockIdx.x : (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long)a.tokens * groups) return;
    const int lane = TEAM ? threadIdx.x : threadIdx.x & 31;
    const int step = TEAM ? blockDim.x : 32;
    const int t = (int)(item / groups), c0 = (int)(item % groups) * a.gs;
    const float* y = a.y + (size_t)t * a.y_t + c0;
    const float* gate = a.gate + (size_t)t * a.gate_t + c0;
    float ss = 0.f;
    for (int i = lane; i < a.gs; i += step) {
        float v = y[i];
        if (a.mode == 0) { const float z = gate[i]; v *= z / (1.f + expf(-z)); }
        ss = fmaf(v, v, ss);
    }
    ss = TEAM ? block_sum(ss, scratch) : warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)a.gs + a.eps);
    T* out = reinterpret_cast<T*>(a.out) + (size_t)t * a.out_t + c0;
    for (int i = lane; i < a.gs; i += step) {
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
    LLMP_REQUIRE(H <= 65535 && (P + 3) / 4 <= 65535, "ssd_scan: too many heads %d or columns %d", H, P);
    ScanArgs a;
    a.xbc = xbc; a.xbc_t = xbc_t; a.dt = dt; a.dt_t = dt_t; a.dt_bias = dt_bias; a.a_log = a_log; a.d_skip = d_skip;
    a.state = state; a.state_slot = state_slot; a.state_half = state_half; a.q_start = q_start; a.slots = slots;
    a.positions = positions; a.y = y; a.y_t = y_t; a.H = H; a.G = G; a.N = N; a.P = P;
    // lanes that share a column: the fewest (a power of two up to 32) that leave a lane at most 16 rows (32 past 512 rows)
    int rows = 1;
    while (rows < 32 && (N + rows - 1) / rows > 16) rows *= 2;
    const int per = (N + rows - 1) / rows;
    LLMP_REQUIRE(per <= 32, "ssd_scan: a state of %d rows does not fit the registers of a warp", N);
    int nt = 1;
    while (nt < per) nt *= 2;
    if (rows > 1) nt = nt < 16 ? 16 : nt;
    const int cols = SS_THREADS / rows;
    const size_t row_bytes = (size_t)(2 * nt * rows + cols + 4) * sizeof(float);
    int stage_tokens = 8;
    while (stage_tokens > 1 && SS_STAGES * stage_tokens * row_bytes > 96 * 1024) stage_tokens /= 2;
    const size_t smem = SS_STAGES * stage_tokens * row_bytes;
    LLMP_REQUIRE(smem <= 200 * 1024, "ssd_scan: state size %d does not fit shared memory", N);
    int vec = 0;
    if (((uintptr_t)xbc & 15) == 0 && xbc_t % 4 == 0 && P % 4 == 0) {
        if (N % 4 == 0 && ((long)H * P) % 4 == 0) vec |= 1;
        if ((nt * rows) % 4 == 0) vec |= 2;     // the columns' place in a row of the ring is 16-byte aligned
    }
    dim3 grid(R, H, (P + cols - 1) / cols);
#define LLMP_SCAN(NT, RW)                                                                         \
    if (nt == NT && rows == RW) {                                                                 \
        LLMP_ALLOW_SMEM((ssd_scan_kernel<NT, RW>), smem);                                         \
        ssd_scan_kernel<NT, RW><<<grid, SS_THREADS + 32 * SS_COPY_WARPS, smem, stream>>>(a, stage_tokens, vec);   \
    } else
    LLMP_SCAN(1, 1) LLMP_SCAN(2, 1) LLMP_SCAN(4, 1) LLMP_SCAN(8, 1) LLMP_SCAN(16, 1) LLMP_SCAN(16, 2) LLMP_SCAN(16, 4)
    LLMP_SCAN(16, 8) LLMP_SCAN(16, 16) LLMP_SCAN(16, 32) LLMP_SCAN(32, 32)
    {
        llmp_set_error("ssd_scan: no instance for %d rows a lane on %d lanes", nt, rows);
        return 1;
    }
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
    if (gs >= 512) {                     // a block per group; the choice depends on the group's size alone
        const int threads = gs >= 2048 ? 512 : 256;
        if (out_dtype == LLMP_BF16) gated_group_norm_kernel<bf16, true><<<(unsigned)items, threads, 0, stream>>>(a);
        else gated_group_norm_kernel<float, true><<<(unsigned)items, threads, 0, stream>>>(a);
        return llmp_check_launch("gated_group_norm");
    }
    const int warps = 4;
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    if (out_dtype == LLMP_BF16) gated_group_norm_kernel<bf16, false><<<blocks, warps * 32, 0, stream>>>(a);
    else gated_group_norm_kernel<float, false><<<blocks, warps * 32, 0, stream>>>(a);
    return llmp_check_launch("gated_group_norm");
}
