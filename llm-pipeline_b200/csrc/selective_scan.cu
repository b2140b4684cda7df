// The selective state-space recurrence with a decay per channel and state entry.
//
// For every channel c of `inner` and state entry n of `states`, token by token:
//   dt_c = softplus(dt_raw_c + dt_bias_c)
//   S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n          (A < 0 comes from the caller; S is zero before the first token)
//   y_c = sum_n S[c, n] C_n + D_c x_c;      out_c = y_c * silu(z_c)   (without z: y_c)
// x (after its convolution and activation), dt_raw, B, C and z are float32 rows of the step; everything here is float32
// where the output is bfloat16. Where the output is float32 (the engine's true 32-bit path) the decays, the state and the
// read-out of a step are float64 between the float32 state a step reads and the one it leaves: a float32 recurrence over a
// thousand tokens with decays near one drifts by tens of units in the last place, which this keeps out of the sharper path.
// out has the compute type. Between steps a request keeps S in its state slot, as two copies [inner][states] that take
// turns by the parity of the last position written, so a step of one token never overwrites what it read.
//
// A block of 64 threads takes 64 / L channels of one request: L lanes of a warp share a channel and hold NS state entries
// each (entry n = k L + lane, so the lanes read neighbouring words), the sum over n ends with log2(L) shuffles. The
// request's tokens are walked in chunks of 8: the block first brings the chunk's B and C rows into shared memory and every
// thread its channel's x and step sizes into registers (all loads of a chunk in flight together, softplus and the decays
// off the chain), then the chain itself is one multiply-add per token and entry. L and NS follow from `states` alone, so
// a row's operations do not depend on the step.
#include "common.cuh"

namespace {

constexpr int SS_THREADS = 64;
constexpr int SS_CHUNK = 8;

struct ScanArgs {
    const float* x; long x_t;
    const float* dt; long dt_t;
    const float* dt_bias;                 // [inner]
    const float* B; const float* C; long bc_t;
    const float* A;                       // [inner, states]
    const float* D;                       // [inner]
    const float* z; long z_t;             // or null
    float* state; long state_slot; long state_half;
    const int* q_start; const int* slots; const int* positions;
    void* out; long out_t;
    int inner, states, L;
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float ss_exp(float v) { return expf(v); }
__device__ __forceinline__ double ss_exp(double v) { return exp(v); }

template <typename T, typename ACC, int NS>
__global__ void __launch_bounds__(SS_THREADS) selective_scan_kernel(const ScanArgs a) {
    extern __shared__ float bc_s[];                            // [SS_CHUNK][2 states]
    const int r = blockIdx.x;
    const int L = a.L, Nst = a.states;
    const int per_block = SS_THREADS / L;
    const int c = blockIdx.y * per_block + threadIdx.x / L;
    const int l = threadIdx.x % L;
    const bool ok = c < a.inner;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    if (end <= begin) return;
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + end - begin - 1) & 1) * a.state_half;
    ACC S[NS];
    float A[NS];
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        const int n = k * L + l;
        const bool have = ok && n < Nst;
        S[k] = have ? (ACC)rd[(size_t)c * Nst + n] : (ACC)0;
        A[k] = have ? a.A[(size_t)c * Nst + n] : 0.f;
    }
    const float dt_b = ok ? a.dt_bias[c] : 0.f;
    const float Dc = ok ? a.D[c] : 0.f;
    T* out = reinterpret_cast<T*>(a.out);
    for (int t0 = begin; t0 < end; t0 += SS_CHUNK) {
        const int nt = min(SS_CHUNK, end - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 2 * Nst; i += SS_THREADS) {
            const int tt = i / (2 * Nst), j = i % (2 * Nst);
            bc_s[i] = j < Nst ? a.B[(size_t)(t0 + tt) * a.bc_t + j] : a.C[(size_t)(t0 + tt) * a.bc_t + j - Nst];
        }
        float xr[SS_CHUNK], dr[SS_CHUNK], zr[SS_CHUNK];
#pragma unroll
        for (int tt = 0; tt < SS_CHUNK; ++tt) {
            const bool have = ok && tt < nt;
            xr[tt] = have ? a.x[(size_t)(t0 + tt) * a.x_t + c] : 0.f;
            dr[tt] = have ? a.dt[(size_t)(t0 + tt) * a.dt_t + c] : 0.f;
            zr[tt] = have && a.z && l == 0 ? a.z[(size_t)(t0 + tt) * a.z_t + c] : 0.f;
        }
#pragma unroll
        for (int tt = 0; tt < SS_CHUNK; ++tt) dr[tt] = softplus_f(dr[tt] + dt_b);
        __syncthreads();
#pragma unroll
        for (int tt = 0; tt < SS_CHUNK; ++tt) {
            if (tt < nt) {
                const ACC dtv = dr[tt], dx = dtv * (ACC)xr[tt];
                const float* Bs = bc_s + tt * 2 * Nst;
                const float* Cs = Bs + Nst;
                ACC y = 0;
#pragma unroll
                for (int k = 0; k < NS; ++k) {
                    const int n = k * L + l;
                    if (n < Nst) {
                        S[k] = fma(ss_exp(dtv * (ACC)A[k]), S[k], dx * (ACC)Bs[n]);
                        y = fma(S[k], (ACC)Cs[n], y);
                    }
                }
                for (int o = L >> 1; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
                if (ok && l == 0) {
                    y = fma((ACC)Dc, (ACC)xr[tt], y);
                    float yf = (float)y;
                    if (a.z) yf *= zr[tt] / (1.f + expf(-zr[tt]));
                    out[(size_t)(t0 + tt) * a.out_t + c] = from_float<T>(yf);
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        const int n = k * L + l;
        if (ok && n < Nst) wr[(size_t)c * Nst + n] = (float)S[k];
    }
}

}  // namespace

LLMP_API int llmp_selective_scan(const float* x, long x_t, const float* dt, long dt_t, const float* dt_bias, const float* B,
                                 const float* C, long bc_t, const float* A, const float* D, const float* z, long z_t, float* state,
                                 long state_slot, long state_half, const int* q_start, const int* slots, const int* positions,
                                 void* out, int out_dtype, long out_t, int R, int inner, int states, cudaStream_t stream) {
    if (R <= 0) return 0;
    LLMP_REQUIRE(inner > 0 && states > 0 && states <= 256, "selective_scan: %d channels with %d state entries (up to 256 are served)",
                 inner, states);
    LLMP_REQUIRE(state_half >= (long)inner * states, "selective_scan: the state piece is shorter than the state");
    const int NS = states <= 128 ? 4 : 8;
    int L = 1;
    while (L * NS < states) L *= 2;
    ScanArgs a;
    a.x = x; a.x_t = x_t; a.dt = dt; a.dt_t = dt_t; a.dt_bias = dt_bias; a.B = B; a.C = C; a.bc_t = bc_t; a.A = A; a.D = D;
    a.z = z; a.z_t = z_t; a.state = state; a.state_slot = state_slot; a.state_half = state_half; a.q_start = q_start;
    a.slots = slots; a.positions = positions; a.out = out; a.out_t = out_t; a.inner = inner; a.states = states; a.L = L;
    const int per_block = SS_THREADS / L;
    const long blocks_y = ((long)inner + per_block - 1) / per_block;
    LLMP_REQUIRE(blocks_y <= 65535, "selective_scan: too many channels %d", inner);
    dim3 grid(R, (unsigned)blocks_y);
    const size_t smem = (size_t)SS_CHUNK * 2 * states * sizeof(float);
    if (out_dtype == LLMP_BF16) {
        if (NS == 4) selective_scan_kernel<bf16, float, 4><<<grid, SS_THREADS, smem, stream>>>(a);
        else selective_scan_kernel<bf16, float, 8><<<grid, SS_THREADS, smem, stream>>>(a);
    } else {
        if (NS == 4) selective_scan_kernel<float, double, 4><<<grid, SS_THREADS, smem, stream>>>(a);
        else selective_scan_kernel<float, double, 8><<<grid, SS_THREADS, smem, stream>>>(a);
    }
    return llmp_check_launch("selective_scan");
}
