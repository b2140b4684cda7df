// Short causal convolution over time, channel by channel, with its activation and the state it carries.
//
//   out[t, c] = act(sum_{j = 0 .. K-1} taps[c, j] * in[t - (K-1) + j, c] + bias[c])
//
// act: nothing, SiLU, or "add the current input" (out = in + conv(in): a convolution beside the identity, which layers
// put in front of a sublayer). Besides the float32 output (or instead of it) the result can be written in the compute
// type, the channels cut into equal runs that go to separate matrices (two sublayers' inputs filtered in one launch).
//
// taps[c, K-1] multiplies the current token; inputs before a request's first token are zero. Between steps a request keeps
// its last K - 1 inputs in its state slot, oldest first. The slot holds two copies that take turns by the parity of the
// last position written (a step reads the copy of the position before its first token and writes the copy of its last
// token), so a step of one token never overwrites what it read.
//
// Two forms with the same arithmetic (the products are summed from the oldest input to the current one, then the bias):
//   serial:   a thread per (request, channel) walks the request's tokens with the last inputs in registers and writes the
//             state at the end; for steps whose requests bring few tokens (decode steps above all).
//   parallel: a thread per (tile of 16 tokens of the step, channel) walks the tile the same way, taking the inputs before
//             the tile from the step's rows or, before the portion's first token, from the state; a second kernel then
//             moves the state on.
// Inputs and outputs are float32 (what follows is a recurrence in 32-bit); taps and bias have the type they were stored in.
#include "common.cuh"

namespace {

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_SERIAL_TOKENS = 32;

struct ConvArgs {
    const float* x; long x_t;                 // [tokens, >= C], stride of a token
    const void* taps; int taps_bf16;          // [C, K]
    const void* bias; int bias_bf16;          // [C] or null
    float* state; long state_slot; long state_half;   // slot s, copy h: state + s * state_slot + h * state_half, [K - 1][C]
    const int* q_start; const int* slots; const int* positions; const int* token_request;
    float* out; long out_t;                   // [tokens, C] float32, or null
    void* out2; int out2_bf16; long out2_t; long out2_block; int out2_split;   // a second output, or null: channel c of token
                                              // t at out2 + (c / split) * block + t * out2_t + c % split
    int C, K, act;
};

// act 0: the sum itself; 1: SiLU of it; 2: the sum plus the current input (a convolution beside the identity)
__device__ __forceinline__ float conv_act(float v, float xin, int act) {
    return act == 1 ? v / (1.f + expf(-v)) : (act == 2 ? v + xin : v);
}

// where channel c lies in the second output's first row: a thread's channel is fixed, so it divides once
__device__ __forceinline__ size_t conv_out2_base(const ConvArgs& a, int c) {
    return a.out2 ? (size_t)(c / a.out2_split) * a.out2_block + c % a.out2_split : 0;
}

__device__ __forceinline__ void conv_store(const ConvArgs& a, int t, int c, float v, size_t base2) {
    if (a.out) a.out[(size_t)t * a.out_t + c] = v;
    if (a.out2) {
        const size_t at = base2 + (size_t)t * a.out2_t;
        if (a.out2_bf16) reinterpret_cast<bf16*>(a.out2)[at] = __float2bfloat16_rn(v);
        else reinterpret_cast<float*>(a.out2)[at] = v;
    }
}

__global__ void short_conv_serial_kernel(const ConvArgs a) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    if (end <= begin) return;
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + end - begin - 1) & 1) * a.state_half;
    const int K = a.K;
    float w[CONV_MAX_TAPS], tap[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        tap[j] = j < K ? load_as_float(a.taps, a.taps_bf16, (size_t)c * K + j) : 0.f;
        w[j] = j < K - 1 ? rd[(size_t)j * a.C + c] : 0.f;
    }
    const float b = a.bias ? load_as_float(a.bias, a.bias_bf16, c) : 0.f;
    const size_t base2 = conv_out2_base(a, c);
    for (int t = begin; t < end; ++t) {
        const float xin = a.x[(size_t)t * a.x_t + c];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < K - 1) acc = fmaf(w[j], tap[j], acc);
        float last = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j == K - 1) last = tap[j];
        acc = fmaf(xin, last, acc);
        conv_store(a, t, c, conv_act(acc + b, xin, a.act), base2);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < K - 1) w[j] = (j + 1 < K - 1) ? w[j + 1] : xin;
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
        if (j < K - 1) wr[(size_t)j * a.C + c] = w[j];
}

constexpr int CONV_TILE_TOKENS = 16;

// A block takes CONV_TILE_TOKENS consecutive tokens of the step and 128 channels; a thread walks its channel through
// the tile with the last K - 1 inputs in registers, and fills them anew where the tile begins or a new request does
// (from the step's rows, or from the slot's copy for places before the portion).
__global__ void short_conv_parallel_kernel(const ConvArgs a, const int N) {
    const int t0 = blockIdx.x * CONV_TILE_TOKENS;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int K = a.K;
    float w[CONV_MAX_TAPS], tap[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        tap[j] = j < K ? load_as_float(a.taps, a.taps_bf16, (size_t)c * K + j) : 0.f;
        w[j] = 0.f;
    }
    float last = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j)
        if (j == K - 1) last = tap[j];
    const float b = a.bias ? load_as_float(a.bias, a.bias_bf16, c) : 0.f;
    const size_t base2 = conv_out2_base(a, c);
    const int t1 = min(t0 + CONV_TILE_TOKENS, N);
    int r_prev = -1;
    for (int t = t0; t < t1; ++t) {
        const int r = a.token_request[t];
        if (r != r_prev) {
            r_prev = r;
            const int begin = a.q_start[r];
            const int p0 = a.positions[begin];
            const float* rd = a.state + (size_t)a.slots[r] * a.state_slot + ((p0 + 1) & 1) * a.state_half;
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
                if (j < K - 1) {
                    const int at = t - (K - 1) + j;
                    w[j] = at >= begin ? a.x[(size_t)at * a.x_t + c] : rd[(size_t)(K - 1 + at - begin) * a.C + c];
                }
            }
        }
        const float xin = a.x[(size_t)t * a.x_t + c];
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < K - 1) acc = fmaf(w[j], tap[j], acc);
        acc = fmaf(xin, last, acc);
        conv_store(a, t, c, conv_act(acc + b, xin, a.act), base2);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < K - 1) w[j] = (j + 1 < K - 1) ? w[j + 1] : xin;
    }
}

__global__ void short_conv_state_kernel(const ConvArgs a) {
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int begin = a.q_start[r], end = a.q_start[r + 1];
    const int n = end - begin;
    if (n <= 0) return;
    const int p0 = a.positions[begin];
    float* slot = a.state + (size_t)a.slots[r] * a.state_slot;
    const float* rd = slot + ((p0 + 1) & 1) * a.state_half;
    float* wr = slot + ((p0 + n - 1) & 1) * a.state_half;
    const int K = a.K;
    float w[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        w[j] = 0.f;
        if (j < K - 1) {
            const int rel = n - (K - 1) + j;          // place in the portion; negative: still in the old state
            w[j] = rel >= 0 ? a.x[(size_t)(begin + rel) * a.x_t + c] : rd[(size_t)(K - 1 + rel) * a.C + c];
        }
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
        if (j < K - 1) wr[(size_t)j * a.C + c] = w[j];
}

}  // namespace

LLMP_API int llmp_short_conv_serial_tokens() { return CONV_SERIAL_TOKENS; }

LLMP_API int llmp_short_conv(const float* x, long x_t, const void* taps, int taps_dtype, const void* bias, int bias_dtype,
                             float* state, long state_slot, long state_half, const int* q_start, const int* slots,
                             const int* positions, const int* token_request, float* out, long out_t, void* out2, int out2_dtype,
                             long out2_t, long out2_block, int out2_split, int N, int R, int C, int K, int act, int max_q_len,
                             cudaStream_t stream) {
    if (N <= 0 || R <= 0) return 0;
    LLMP_REQUIRE(C > 0 && K >= 1 && K <= CONV_MAX_TAPS, "short_conv: %d taps (1 to %d are served) over %d channels", K,
                 CONV_MAX_TAPS, C);
    LLMP_REQUIRE(x_t >= C && (out == nullptr || out_t >= C) && state_half >= (long)(K - 1) * C, "short_conv: strides shorter than the rows");
    LLMP_REQUIRE(out != nullptr || out2 != nullptr, "short_conv: no output");
    LLMP_REQUIRE(out2 == nullptr || (out2_split > 0 && out2_t >= (out2_split < C ? out2_split : C)), "short_conv: bad second output");
    ConvArgs a;
    a.x = x; a.x_t = x_t; a.taps = taps; a.taps_bf16 = taps_dtype == LLMP_BF16; a.bias = bias; a.bias_bf16 = bias_dtype == LLMP_BF16;
    a.state = state; a.state_slot = state_slot; a.state_half = state_half; a.q_start = q_start; a.slots = slots;
    a.positions = positions; a.token_request = token_request; a.out = out; a.out_t = out_t; a.C = C; a.K = K; a.act = act;
    a.out2 = out2; a.out2_bf16 = out2_dtype == LLMP_BF16; a.out2_t = out2_t; a.out2_block = out2_block; a.out2_split = out2_split > 0 ? out2_split : C;
    const int threads = 128;
    const int col_blocks = (C + threads - 1) / threads;
    LLMP_REQUIRE(col_blocks <= 65535, "short_conv: too many channels %d", C);
    if (max_q_len <= CONV_SERIAL_TOKENS) {
        llmp_launch_dependent(short_conv_serial_kernel, dim3(R, col_blocks), dim3(threads), 0, stream, a);
        return llmp_check_launch("short_conv");
    }
    short_conv_parallel_kernel<<<dim3((N + CONV_TILE_TOKENS - 1) / CONV_TILE_TOKENS, col_blocks), threads, 0, stream>>>(a, N);
    if (K > 1) short_conv_state_kernel<<<dim3(R, col_blocks), threads, 0, stream>>>(a);
    return llmp_check_launch("short_conv (parallel)");
}
