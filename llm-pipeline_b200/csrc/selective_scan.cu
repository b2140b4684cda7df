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
// A block of 128 threads takes 128 / L channels of one request: L lanes of a warp share a channel and hold NS state entries
// each (entry n = k L + lane, so the lanes read neighbouring words), the sum over n ends with log2(L) shuffles. The
// request's tokens are walked in chunks of 8 with the next chunk on its way while this one is worked on: its B and C rows
// by asynchronous copies into the other half of a shared buffer, its x, step sizes and gates as loads into registers that
// nothing reads before the chunk's turn; one barrier a chunk. What a token needs once (its loads, the softplus, the gate,
// the store) is done by one lane of the channel for it, the lanes taking a chunk's tokens in turn, so it costs a chunk one
// pass and not eight; the walk gets a token's step size from its lane by a shuffle. The chain itself is one multiply-add
// per token and entry. Where the output is bfloat16 they use the special-function unit's exponential and
// logarithm. L and NS follow from `states` alone, so a row's operations do not depend on the step.
#include "common.cuh"

namespace {

constexpr int SS_THREADS = 128;
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

// the recurrence's arithmetic in the accumulator's type: exact library functions for float64 (the true 32-bit path), the
// special-function unit for float32 (the bfloat16 path, whose products carry 8 bits)
__device__ __forceinline__ double ss_exp(double v) { return exp(v); }
__device__ __forceinline__ float ss_exp(float v) { return __expf(v); }
__device__ __forceinline__ double ss_softplus(double v) { return v > 20.0 ? v : log1p(exp(v)); }
__device__ __forceinline__ float ss_softplus(float v) { return v > 15.f ? v : __logf(1.f + __expf(v)); }

__device__ __forceinline__ void ss_cp_async_4(float* smem_dst, const float* gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}

template <typename T, typename ACC, int L, int NS>
__global__ void __launch_bounds__(SS_THREADS) selective_scan_kernel(const ScanArgs a) {
    extern __shared__ float bc_s[];                            // [2][SS_CHUNK][2 states]
    constexpr int OWN = (SS_CHUNK + L - 1) / L;                // tokens of a chunk that a lane looks after
    const int r = blockIdx.x;
    const int Nst = a.states;
    constexpr int per_block = SS_THREADS / L;
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
    const bool gated = a.z != nullptr;
    T* out = reinterpret_cast<T*>(a.out);
    const int chunk_floats = SS_CHUNK * 2 * Nst;

    auto copy_bc = [&](int t0, int nt, float* dst) {           // rows [B | C] of nt tokens
        for (int tt = 0; tt < nt; ++tt) {
            for (int j = threadIdx.x; j < 2 * Nst; j += SS_THREADS)
                ss_cp_async_4(dst + tt * 2 * Nst + j, j < Nst ? a.B + (size_t)(t0 + tt) * a.bc_t + j : a.C + (size_t)(t0 + tt) * a.bc_t + j - Nst);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    // a lane looks after the tokens l, l + L, .. of a chunk: it loads their x, step size and gate, takes the softplus, and
    // at the chunk's end gates and stores their outputs; the walk gets a token's step size from its lane by a shuffle
    float xr[OWN], dr[OWN], zr[OWN];
    auto load_rows = [&](int t0, int nt, float (&xv)[OWN], float (&dv)[OWN], float (&zv)[OWN]) {
#pragma unroll
        for (int o = 0; o < OWN; ++o) {
            const int tt = o * L + l;
            const bool have = ok && tt < nt;
            xv[o] = have ? a.x[(size_t)(t0 + tt) * a.x_t + c] : 0.f;
            dv[o] = have ? a.dt[(size_t)(t0 + tt) * a.dt_t + c] : 0.f;
            zv[o] = have && gated ? a.z[(size_t)(t0 + tt) * a.z_t + c] : 0.f;
        }
    };
    copy_bc(begin, min(SS_CHUNK, end - begin), bc_s);
    load_rows(begin, min(SS_CHUNK, end - begin), xr, dr, zr);
    int buf = 0;
    for (int t0 = begin; t0 < end; t0 += SS_CHUNK, buf ^= 1) {
        const int nt = min(SS_CHUNK, end - t0);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();                                       // this chunk's rows are in; the other half was read a round ago
        float xn[OWN], dn[OWN], zn[OWN];
        const int t1 = t0 + SS_CHUNK;
        const bool more = t1 < end;
        if (more) {
            copy_bc(t1, min(SS_CHUNK, end - t1), bc_s + (buf ^ 1) * chunk_floats);
            load_rows(t1, min(SS_CHUNK, end - t1), xn, dn, zn);
        }
        ACC dts[OWN], dxs[OWN], ys[OWN];
#pragma unroll
        for (int o = 0; o < OWN; ++o) {
            dts[o] = ss_softplus((ACC)(dr[o] + dt_b));
            dxs[o] = dts[o] * (ACC)xr[o];
            ys[o] = 0;
        }
        const float* rows = bc_s + buf * chunk_floats;
#pragma unroll
        for (int tt = 0; tt < SS_CHUNK; ++tt) {
            if (tt < nt) {                                     // the same for every thread of the block
                const int o = tt / L, owner = tt % L;
                const ACC dtv = L > 1 ? __shfl_sync(0xffffffffu, dts[o], owner, L) : dts[o];
                const ACC dx = L > 1 ? __shfl_sync(0xffffffffu, dxs[o], owner, L) : dxs[o];
                const float* Bs = rows + tt * 2 * Nst;
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
#pragma unroll
                for (int w = L >> 1; w > 0; w >>= 1) y += __shfl_xor_sync(0xffffffffu, y, w);
                if (owner == l) ys[o] = y;
            }
        }
#pragma unroll
        for (int o = 0; o < OWN; ++o) {
            const int tt = o * L + l;
            if (ok && tt < nt) {
                float yf = (float)fma((ACC)Dc, (ACC)xr[o], ys[o]);
                if (gated) yf *= sizeof(ACC) == 8 ? zr[o] / (1.f + expf(-zr[o])) : __fdividef(zr[o], 1.f + __expf(-zr[o]));
                out[(size_t)(t0 + tt) * a.out_t + c] = from_float<T>(yf);
            }
        }
        if (more) {
#pragma unroll
            for (int o = 0; o < OWN; ++o) { xr[o] = xn[o]; dr[o] = dn[o]; zr[o] = zn[o]; }
        }
    }
#pragma unroll
    for (int k = 0; k < NS; ++k) {
        const int n = k * L + l;
        if (ok && n < Nst) wr[(size_t)c * Nst + n] = (float)S[k];
    }
}

template <int L, int NS>
void launch_scan(const ScanArgs& a, int out_dtype, int R, cudaStream_t stream) {
    constexpr int per_block = SS_THREADS / L;
    dim3 grid(R, (unsigned)((a.inner + per_block - 1) / per_block));
    const size_t smem = (size_t)2 * SS_CHUNK * 2 * a.states * sizeof(float);
    if (out_dtype == LLMP_BF16) selective_scan_kernel<bf16, float, L, NS><<<grid, SS_THREADS, smem, stream>>>(a);
    else selective_scan_kernel<float, double, L, NS><<<grid, SS_THREADS, smem, stream>>>(a);
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
    // two state entries a lane up to 64 entries, then 32 lanes with more each
    int L = 1;
    while (L < 32 && L * 2 < states) L *= 2;
    const int NS = (states + L - 1) / L;
    ScanArgs a;
    a.x = x; a.x_t = x_t; a.dt = dt; a.dt_t = dt_t; a.dt_bias = dt_bias; a.B = B; a.C = C; a.bc_t = bc_t; a.A = A; a.D = D;
    a.z = z; a.z_t = z_t; a.state = state; a.state_slot = state_slot; a.state_half = state_half; a.q_start = q_start;
    a.slots = slots; a.positions = positions; a.out = out; a.out_t = out_t; a.inner = inner; a.states = states; a.L = L;
    LLMP_REQUIRE(((long)inner * L + SS_THREADS - 1) / SS_THREADS <= 65535, "selective_scan: too many channels %d", inner);
    switch (L) {
        case 1: if (NS <= 1) launch_scan<1, 1>(a, out_dtype, R, stream); else launch_scan<1, 2>(a, out_dtype, R, stream); break;
        case 2: launch_scan<2, 2>(a, out_dtype, R, stream); break;
        case 4: launch_scan<4, 2>(a, out_dtype, R, stream); break;
        case 8: launch_scan<8, 2>(a, out_dtype, R, stream); break;
        case 16: launch_scan<16, 2>(a, out_dtype, R, stream); break;
        default:
            if (NS <= 2) launch_scan<32, 2>(a, out_dtype, R, stream);
            else if (NS <= 4) launch_scan<32, 4>(a, out_dtype, R, stream);
            else launch_scan<32, 8>(a, out_dtype, R, stream);
    }
    return llmp_check_launch("selective_scan");
}
