// Softmax attention with grouped key/value heads whose scores are capped and lose a distance bias, over a sliding
// window that keeps the first tokens, with a sink in the denominator and a gate on the output.
//
// With H query heads, G key/value heads (head h uses key/value head h / (H / G)), keys of d and values of dv entries,
// for the token at position i and a key at position j <= i:
//   seen(i, j) = i - j < window  or  j < keep_first                     (window 0: every j <= i)
//   s = (q . k) * scale;  s <- cap * tanh(s / cap) if cap > 0;  s <- s - slope[h] * (i - j)  if slopes are given
//   p_j = exp(s_j) / (exp(sink[h]) + sum_seen exp(s_j))                 (without a sink: the plain softmax)
//   o_h = sum_j p_j v_j;   o_h <- o_h * sigmoid(gate)  if a gate is given
// Scores, the cap, the bias, the softmax and the weighted sums are float32.
//
// capped_qkv_post: adds the projections' biases to the float32 product [q | k | v], divides every value head by its
// root mean square (if asked), writes the queries in the compute type and the token's cache rows [k | v] per key/value
// head into its page slot.
//
// capped_attention (any sizes, float32 or bfloat16): a block per (token, key/value head, up to 8 heads of the group), a
// warp per query head. Keys are walked in tiles of 32 aligned to key 0; tiles that hold no key the token sees are
// skipped, and rows of keys it does not see are never read (their pages may be gone). A row's operations depend on its
// position alone, not on the step.
#include "common.cuh"

namespace {

constexpr int CA_KEYS = 32;
constexpr int CA_WARPS = 8;

template <typename T>
__global__ void capped_qkv_post_kernel(const float* __restrict__ qkv, long qkv_t, const void* __restrict__ bias, int bias_bf16,
                                       float v_eps, int v_norm, T* __restrict__ q_out, long q_out_t, const int* __restrict__ slots,
                                       T* __restrict__ pages, int page_size, int H, int G, int d, int dv) {
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const int n = blockIdx.x;
    const float* row = qkv + (size_t)n * qkv_t;
    const int slot = slots ? slots[n] : -1;
    const int rs = d + dv;
    T* page_row = nullptr;
    if (pages && slot >= 0) page_row = pages + (((size_t)(slot / page_size) * G) * page_size + slot % page_size) * rs;
    const size_t head_stride = (size_t)page_size * rs;
    for (int i = threadIdx.x; i < (H + G) * d; i += blockDim.x) {
        const int head = i / d, c = i % d;
        const float v = row[i] + (bias ? load_as_float(bias, bias_bf16, i) : 0.f);
        if (head < H) q_out[(size_t)n * q_out_t + i] = from_float<T>(v);
        else if (page_row) page_row[(size_t)(head - H) * head_stride + c] = from_float<T>(v);
    }
    if (!page_row) return;
    // values: a warp per key/value head in turn
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int v_at = (H + G) * d;
    for (int g = warp; g < G; g += nw) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) {
            const float v = row[v_at + g * dv + c] + (bias ? load_as_float(bias, bias_bf16, v_at + g * dv + c) : 0.f);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float f = v_norm ? 1.f / sqrtf(ss / (float)dv + v_eps) : 1.f;
        for (int c = lane; c < dv; c += 32) {
            const float v = row[v_at + g * dv + c] + (bias ? load_as_float(bias, bias_bf16, v_at + g * dv + c) : 0.f);
            page_row[(size_t)g * head_stride + d + c] = from_float<T>(v * f);
        }
    }
}

struct CappedArgs {
    const void* q; long q_t;                  // [tokens, H d]
    const void* pages;                        // [page, kv head, token in page, d + dv]
    const int* tables; int width;
    const int* token_request; const int* positions;
    const float* slopes;                      // [H] or null
    const float* sink;                        // [H] or null
    const float* gate; long gate_t;           // float32 [tokens, H dv] (a view) or null
    void* out; long out_t;                    // [tokens, H dv]
    int H, G, d, dv, page_size, window, keep;
    float scale, cap;
};

template <typename T, int NO>
__global__ void __launch_bounds__(CA_WARPS * 32) capped_attention_kernel(const CappedArgs a) {
    extern __shared__ float smem[];
    const int d = a.d, dv = a.dv, rs = a.d + a.dv;
    const int ks = d | 1;                                    // odd row stride: the lanes of a warp hit different banks
    float* Ks = smem;                                        // [CA_KEYS][ks]
    float* Vs = Ks + CA_KEYS * ks;                           // [CA_KEYS][dv]
    float* qs = Vs + CA_KEYS * dv;                           // [CA_WARPS][d]
    float* ps = qs + CA_WARPS * d;                           // [CA_WARPS][CA_KEYS]
    const int n = blockIdx.x;
    const int hpg = a.H / a.G;
    const int chunks = (hpg + CA_WARPS - 1) / CA_WARPS;
    const int g = blockIdx.y / chunks;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hl = (blockIdx.y % chunks) * CA_WARPS + warp;
    const bool active = hl < hpg;
    const int h = g * hpg + hl;
    const int pos = a.positions[n];
    const int* table = a.tables + (size_t)a.token_request[n] * a.width;
    const T* pages = reinterpret_cast<const T*>(a.pages);
    const int lo_w = a.window > 0 ? max(0, pos - a.window + 1) : 0;       // first key of the window
    const int keep_end = min(a.keep, lo_w);                               // kept keys before the window: [0, keep_end)
    float slope = 0.f, m_run = -INFINITY, l_run = 0.f;
    if (active) {
        const T* q = reinterpret_cast<const T*>(a.q) + (size_t)n * a.q_t + (size_t)h * d;
        for (int i = lane; i < d; i += 32) qs[warp * d + i] = to_float(q[i]);
        if (a.slopes) slope = a.slopes[h];
        if (a.sink) { m_run = a.sink[h]; l_run = 1.f; }
    }
    float o[NO];
#pragma unroll
    for (int i = 0; i < NO; ++i) o[i] = 0.f;
    for (int k0 = 0; k0 <= pos; k0 += CA_KEYS) {
        if (k0 >= keep_end && k0 + CA_KEYS <= lo_w) {        // the tile lies between the kept keys and the window
            k0 = (lo_w / CA_KEYS) * CA_KEYS - CA_KEYS;
            continue;
        }
        __syncthreads();
        for (int j = warp; j < CA_KEYS; j += CA_WARPS) {     // a warp copies a key's row
            const int key = k0 + j;
            const bool seen = key <= pos && (key >= lo_w || key < keep_end);
            if (seen) {
                const int page = table[key / a.page_size];
                const T* row = pages + (((size_t)page * a.G + g) * a.page_size + key % a.page_size) * rs;
                for (int i = lane; i < d; i += 32) Ks[j * ks + i] = to_float(row[i]);
                for (int i = lane; i < dv; i += 32) Vs[j * dv + i] = to_float(row[d + i]);
            } else {
                for (int i = lane; i < d; i += 32) Ks[j * ks + i] = 0.f;
                for (int i = lane; i < dv; i += 32) Vs[j * dv + i] = 0.f;
            }
        }
        __syncthreads();
        if (!active) continue;
        const int key = k0 + lane;
        const bool valid = key <= pos && (key >= lo_w || key < keep_end);
        float s = 0.f;
        const float* kr = Ks + lane * ks;
        const float* qw = qs + warp * d;
        for (int i = 0; i < d; ++i) s = fmaf(qw[i], kr[i], s);
        s *= a.scale;
        if (a.cap > 0.f) s = a.cap * tanhf(s / a.cap);
        s -= slope * (float)(pos - key);
        s = valid ? s : -INFINITY;
        const float m_new = fmaxf(m_run, warp_max(s));       // finite: a tile that is walked holds a key the token sees
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m_run - m_new);             // 0 at the first tile without a sink (m_run = -inf)
        l_run = l_run * alpha + warp_sum(p);
        m_run = m_new;
        ps[warp * CA_KEYS + lane] = p;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NO; ++i) {
            const int c = lane + 32 * i;
            if (c < dv) {
                float acc = o[i] * alpha;
                for (int j = 0; j < CA_KEYS; ++j) acc = fmaf(ps[warp * CA_KEYS + j], Vs[j * dv + c], acc);
                o[i] = acc;
            }
        }
        __syncwarp();
    }
    if (!active) return;
    const float inv = 1.f / l_run;
    T* dst = reinterpret_cast<T*>(a.out) + (size_t)n * a.out_t + (size_t)h * dv;
    const float* gate = a.gate ? a.gate + (size_t)n * a.gate_t + (size_t)h * dv : nullptr;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) {
            float v = o[i] * inv;
            if (gate) v = v / (1.f + expf(-gate[c]));
            dst[c] = from_float<T>(v);
        }
    }
}

template <typename T>
int launch_capped(const CappedArgs& a, int N, cudaStream_t stream) {
    const size_t smem = ((size_t)CA_KEYS * ((a.d | 1) + a.dv) + (size_t)CA_WARPS * a.d + CA_WARPS * CA_KEYS) * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "capped_attention: heads of %d + %d entries do not fit shared memory", a.d, a.dv);
    const int hpg = a.H / a.G;
    const long blocks_y = (long)a.G * ((hpg + CA_WARPS - 1) / CA_WARPS);
    LLMP_REQUIRE(blocks_y <= 65535, "capped_attention: too many heads %d", a.H);
    dim3 grid(N, (unsigned)blocks_y);
#define LLMP_CA_LAUNCH(NO)                                                         \
    do {                                                                           \
        LLMP_ALLOW_SMEM((capped_attention_kernel<T, NO>), smem);                   \
        capped_attention_kernel<T, NO><<<grid, CA_WARPS * 32, smem, stream>>>(a);  \
    } while (0)
    if (a.dv <= 64) LLMP_CA_LAUNCH(2);
    else if (a.dv <= 128) LLMP_CA_LAUNCH(4);
    else if (a.dv <= 256) LLMP_CA_LAUNCH(8);
    else LLMP_CA_LAUNCH(16);
#undef LLMP_CA_LAUNCH
    return llmp_check_launch("capped_attention");
}

}  // namespace

LLMP_API int llmp_capped_qkv_post(const float* qkv, long qkv_t, const void* bias, int bias_dtype, float v_eps, int v_norm, void* q_out,
                                  int dtype, long q_out_t, const int* slots, void* pages, int page_size, int N, int H, int G, int d,
                                  int dv, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0, "capped_qkv_post: bad sizes heads=%d kv=%d dim=%d vdim=%d", H, G, d, dv);
    LLMP_REQUIRE(pages == nullptr || page_size > 0, "capped_qkv_post: pages without a page size");
    if (dtype == LLMP_F32)
        llmp_launch_dependent(capped_qkv_post_kernel<float>, dim3(N), dim3(256), 0, stream, qkv, qkv_t, bias, (int)(bias_dtype == LLMP_BF16), v_eps, v_norm, (float*)q_out,
                                                             q_out_t, slots, (float*)pages, page_size, H, G, d, dv);
    else
        llmp_launch_dependent(capped_qkv_post_kernel<bf16>, dim3(N), dim3(256), 0, stream, qkv, qkv_t, bias, (int)(bias_dtype == LLMP_BF16), v_eps, v_norm, (bf16*)q_out,
                                                            q_out_t, slots, (bf16*)pages, page_size, H, G, d, dv);
    return llmp_check_launch("capped_qkv_post");
}

LLMP_API int llmp_capped_attention(const void* q, long q_t, const void* pages, int dtype, const int* tables, int width,
                                   const int* token_request, const int* positions, const float* slopes, const float* sink,
                                   const float* gate, long gate_t, void* out, long out_t, int N, int H, int G, int d, int dv,
                                   int page_size, int window, int keep, float scale, float cap, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && dv <= 512 && page_size > 0 && width > 0 && window >= 0 && keep >= 0,
                 "capped_attention: bad sizes heads=%d kv=%d dim=%d vdim=%d page=%d width=%d", H, G, d, dv, page_size, width);
    CappedArgs a;
    a.q = q; a.q_t = q_t; a.pages = pages; a.tables = tables; a.width = width; a.token_request = token_request; a.positions = positions;
    a.slopes = slopes; a.sink = sink; a.gate = gate; a.gate_t = gate_t; a.out = out; a.out_t = out_t;
    a.H = H; a.G = G; a.d = d; a.dv = dv; a.page_size = page_size; a.window = window; a.keep = keep; a.scale = scale; a.cap = cap;
    return dtype == LLMP_F32 ? launch_capped<float>(a, N, stream) : launch_capped<bf16>(a, N, stream);
}
