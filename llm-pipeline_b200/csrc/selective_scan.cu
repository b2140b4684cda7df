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
// A block is one warp and takes 32 / L channels of one request (no warp waits for another; a long prompt is a chain of
// dependent steps, and what hides their latency is the number of warps): L lanes share a channel and hold NS state entries
// each (entry n = k L + lane, so the lanes read neighbouring words), the sum over n ends with log2(L) shuffles. The
// request's tokens are walked in chunks of 8 with the next chunks on their way while this one is worked on: the B and C
// rows of three chunks by asynchronous copies into a ring of stages in shared memory, x, step sizes and gates of the next
// chunk as loads into registers that nothing reads before the chunk's turn. What a token needs once (its loads, the softplus, the gate,
// the store) is done by one lane of the channel for it, the lanes taking a chunk's tokens in turn, so it costs a chunk one
// pass and not eight; the walk gets a token's step size from its lane by a shuffle. The chain itself is one multiply-add
// per token and entry. Where the output is bfloat16 they use the special-function unit's exponential and
// logarithm. L and NS follow from `states` alone, so a row's operations do not depend on the step.
#include "common.cuh"

namespace {

constexpr int SS_THREADS = 32;
constexpr int SS_CHUNK = 8;
constexpr int SS_AHEAD = 3;                // chunks whose inputs are under way beside the one at work
constexpr int SS_STAGES = SS_AHEAD + 1;

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
    extern __shared__ float bc_s[];                            // the ring: SS_STAGES stages of a chunk's inputs
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
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
    constexpr int CPW = SS_THREADS / L;                        // channels of the block
    const int stage_floats = SS_CHUNK * 2 * Nst;               // a chunk's rows [B | C]

    // a chunk's B and C rows go to a stage of the ring by 4-byte asynchronous copies, SS_AHEAD chunks before their turn
    auto copy_stage = [&](int t0, int nt, float* dst) {
        for (int tt = 0; tt < nt; ++tt) {
            for (int j = threadIdx.x; j < 2 * Nst; j += SS_THREADS)
                ss_cp_async_4(dst + tt * 2 * Nst + j, j < Nst ? a.B + (size_t)(t0 + tt) * a.bc_t + j : a.C + (size_t)(t0 + tt) * a.bc_t + j - Nst);
        }
        // rows past the portion's end take part in the chunk's arithmetic with step size 0: they must hold numbers
        for (int j = nt * 2 * Nst + threadIdx.x; j < SS_CHUNK * 2 * Nst; j += SS_THREADS) dst[j] = 0.f;
    };
    // a lane looks after the tokens l, l + L, .. of a chunk: it loads their x, step size and gate (a chunk ahead, into
    // registers that nothing reads before the chunk's turn), takes the softplus, and at the chunk's end gates and stores
    // their outputs; the walk gets a token's step size from its lane by a shuffle
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
    load_rows(begin, min(SS_CHUNK, end - begin), xr, dr, zr);
    const int chunks = (end - begin + SS_CHUNK - 1) / SS_CHUNK;
#pragma unroll
    for (int i = 0; i < SS_AHEAD; ++i) {
        if (i < chunks) copy_stage(begin + i * SS_CHUNK, min(SS_CHUNK, end - begin - i * SS_CHUNK), bc_s + i * stage_floats);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    for (int i = 0; i < chunks; ++i) {
        const int t0 = begin + i * SS_CHUNK;
        const int nt = min(SS_CHUNK, end - t0);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(SS_AHEAD - 1) : "memory");
        __syncthreads();                                       // this chunk's stage is in; the stage read a round ago is free
        if (i + SS_AHEAD < chunks) {
            const int t1 = t0 + SS_AHEAD * SS_CHUNK;
            copy_stage(t1, min(SS_CHUNK, end - t1), bc_s + ((i + SS_AHEAD) % SS_STAGES) * stage_floats);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const float* rows = bc_s + (i % SS_STAGES) * stage_floats;
        float xn[OWN], dn[OWN], zn[OWN];
        const bool more = i + 1 < chunks;
        if (more) load_rows(t0 + SS_CHUNK, min(SS_CHUNK, end - t0 - SS_CHUNK), xn, dn, zn);
        // straight-line code for the chunk, so that the tokens' independent parts (shuffles, decays, the sums over the
        // lanes) overlap and only the multiply-adds on S form a chain. A token past the portion's end has step size 0:
        // decay 1 and nothing added.
        ACC dts[OWN], dxs[OWN], ys[OWN];
#pragma unroll
        for (int o = 0; o < OWN; ++o) {
            dts[o] = o * L + l < nt ? ss_softplus((ACC)(dr[o] + dt_b)) : (ACC)0;
            dxs[o] = dts[o] * (ACC)xr[o];
            ys[o] = 0;
        }
        ACC dtv[SS_CHUNK], dxv[SS_CHUNK], yv[SS_CHUNK];
#pragma unroll
        for (int tt = 0; tt < SS_CHUNK; ++tt) {
            dtv[tt] = L > 1 ? __shfl_sync(0xffffffffu, dts[tt / L], tt % L, L) : dts[tt / L];
            dxv[tt] = L > 1 ? __shfl_sync(0xffffffffu, dxs[tt / L], tt % L, L) : dxs[tt / L];
            yv[tt] = 0;
        }
#pragma unroll
        for (int k = 0; k < NS; ++k) {
            const int n = k * L + l;
            const bool have = n < Nst;
            float Bv[SS_CHUNK], Cv[SS_CHUNK];
            ACC dA[SS_CHUNK];
#pragma unroll
            for (int tt = 0; tt < SS_CHUNK; ++tt) {
                Bv[tt] = have ? rows[tt * 2 * Nst + n] : 0.f;
                Cv[tt] = have ? rows[tt * 2 * Nst + Nst + n] : 0.f;
                dA[tt] = ss_exp(dtv[tt] * (ACC)A[k]);
            }
#pragma unroll
            for (int tt = 0; tt < SS_CHUNK; ++tt) {
                S[k] = fma(dA[tt], S[k], dxv[tt] * (ACC)Bv[tt]);
                yv[tt] = fma(S[k], (ACC)Cv[tt], yv[tt]);
            }
        }
#pragma unroll
        for (int w = L >> 1; w > 0; w >>= 1) {
#pragma unroll
            for (int tt = 0; tt < SS_CHUNK; ++tt) yv[tt] += __shfl_xor_sync(0xffffffffu, yv[tt], w);
        }
#pragma unroll
        for (int tt = 0; tt < SS_CHUNK; ++tt)
            if (tt % L == l) ys[tt / L] = yv[tt];
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
    const size_t smem = (size_t)SS_STAGES * SS_CHUNK * 2 * a.states * sizeof(float);
    if (out_dtype == LLMP_BF16) {
        LLMP_ALLOW_SMEM((selective_scan_kernel<bf16, float, L, NS>), smem);
        llmp_launch_dependent(selective_scan_kernel<bf16, float, L, NS>, grid, dim3(SS_THREADS), smem, stream, a);
    } else {
        LLMP_ALLOW_SMEM((selective_scan_kernel<float, double, L, NS>), smem);
        llmp_launch_dependent(selective_scan_kernel<float, double, L, NS>, grid, dim3(SS_THREADS), smem, stream, a);
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
    // a lane per state entry up to 32 entries, then 32 lanes with more each: a long prompt is a chain of dependent steps
    // per warp, and what hides their latency is the number of warps (measured: 0.59 ms for 2,048 tokens of 4,096 channels
    // with 16 entries so; 1.08 ms with 8 entries a lane, a sixth of the instructions but an eighth of the warps)
    int L = 1;
    while (L < 32 && L < states) L *= 2;
    const int NS = (states + L - 1) / L;
    ScanArgs a;
    a.x = x; a.x_t = x_t; a.dt = dt; a.dt_t = dt_t; a.dt_bias = dt_bias; a.B = B; a.C = C; a.bc_t = bc_t; a.A = A; a.D = D;
    a.z = z; a.z_t = z_t; a.state = state; a.state_slot = state_slot; a.state_half = state_half; a.q_start = q_start;
    a.slots = slots; a.positions = positions; a.out = out; a.out_t = out_t; a.inner = inner; a.states = states; a.L = L;
    LLMP_REQUIRE(((long)inner * L + SS_THREADS - 1) / SS_THREADS <= 65535, "selective_scan: too many channels %d", inner);
    switch (L) {
        case 1: launch_scan<1, 1>(a, out_dtype, R, stream); break;
        case 2: launch_scan<2, 1>(a, out_dtype, R, stream); break;
        case 4: launch_scan<4, 1>(a, out_dtype, R, stream); break;
        case 8: launch_scan<8, 1>(a, out_dtype, R, stream); break;
        case 16: launch_scan<16, 1>(a, out_dtype, R, stream); break;
        default:
            if (NS <= 1) launch_scan<32, 1>(a, out_dtype, R, stream);
            else if (NS <= 2) launch_scan<32, 2>(a, out_dtype, R, stream);
            else if (NS <= 4) launch_scan<32, 4>(a, out_dtype, R, stream);
            else launch_scan<32, 8>(a, out_dtype, R, stream);
    }
    return llmp_check_launch("selective_scan");
}
