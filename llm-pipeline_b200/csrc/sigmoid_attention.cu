// Attention without softmax: the weight of a visible key is a sigmoid of its capped score, and the heads' weights are
// mixed before they meet the values.
//
// With H query heads, G key/value heads (head h uses key/value head h / (H / G)), keys of d and values of dv entries:
//   s_g(i, j) = (q_g(i) . k(j)) * scale;  s <- cap * tanh(s / cap) if cap > 0
//   w_g(i, j) = sigmoid(s_g(i, j) + pb[g])  for j <= i, else 0          (not normalised over keys)
//   m_h(i, j) = sum_g T[h, g] w_g(i, j)
//   o_h(i)    = sum_j m_h(i, j) v_kv(h)(j)
// Scores, weights, their mix and the weighted sums are float32.
//
// sig_qkv_post: adds the projections' biases to the float32 product [q | k | v], rotates the first `rot` entries of
// every query and key head (entry i with entry i + rot / 2, float32 tables), writes the queries in the compute type and
// the token's cache rows [k | v] per key/value head into its page slot.
//
// sigmoid_attention (any sizes, float32 or bfloat16): a block per (token, key segment) with a warp per query head.
// Keys are walked in tiles of 32 aligned to key 0: a lane scores one key for its warp's head, the weights of all heads
// meet in shared memory, are mixed there, and each warp adds its head's values. Since nothing is normalised over keys,
// key segments (fixed ranges of key indices) simply add up: with more than one segment the blocks leave float32
// partial sums that a second kernel adds in the order of the segments.
#include "common.cuh"

namespace {

constexpr int SA_KEYS = 32;
constexpr int SA_MAX_WARPS = 16;

template <typename T>
__global__ void sig_qkv_post_kernel(const float* __restrict__ qkv, long qkv_t, const void* __restrict__ bias, int bias_bf16,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                    T* __restrict__ q_out, long q_out_t, const int* __restrict__ slots, T* __restrict__ pages,
                                    int page_size, int H, int G, int d, int dv) {
    const int n = blockIdx.x;
    const float* row = qkv + (size_t)n * qkv_t;
    const int half = rot / 2;
    const int slot = slots ? slots[n] : -1;
    const int rs = d + dv;
    T* page_row = nullptr;
    if (pages && slot >= 0) page_row = pages + (((size_t)(slot / page_size) * G) * page_size + slot % page_size) * rs;
    const size_t head_stride = (size_t)page_size * rs;
    // queries and keys: (H + G) heads of d entries
    for (int i = threadIdx.x; i < (H + G) * d; i += blockDim.x) {
        const int head = i / d, c = i % d;
        const int at = head * d + c;                               // q heads then k heads lie side by side in the product
        float v = row[at] + (bias ? load_as_float(bias, bias_bf16, at) : 0.f);
        if (c < rot) {
            const int pair = c < half ? c + half : c - half;
            const float o = row[head * d + pair] + (bias ? load_as_float(bias, bias_bf16, head * d + pair) : 0.f);
            const int f = c < half ? c : c - half;
            const float cs = cos_t[(size_t)n * half + f], sn = sin_t[(size_t)n * half + f];
            v = c < half ? v * cs - o * sn : v * cs + o * sn;
        }
        if (head < H) q_out[(size_t)n * q_out_t + at] = from_float<T>(v);
        else if (page_row) page_row[(size_t)(head - H) * head_stride + c] = from_float<T>(v);
    }
    if (page_row) {
        const int v_at = (H + G) * d;
        for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
            const float v = row[v_at + i] + (bias ? load_as_float(bias, bias_bf16, v_at + i) : 0.f);
            page_row[(size_t)(i / dv) * head_stride + d + i % dv] = from_float<T>(v);
        }
    }
}

struct SigArgs {
    const void* q; long q_t;                  // [tokens, H d]
    const void* pages;                        // [page, kv head, token in page, d + dv]
    const int* tables; int width;
    const int* token_request; const int* positions;
    const float* talk; const float* pb;       // [H, H], [H]
    void* out; long out_t;                    // [tokens, H dv] (one segment) ...
    float* partial;                           // ... or float32 [tokens, segments, H dv]
    int H, G, d, dv, page_size, segments, segment_keys;
    float scale, cap;
};

template <typename T, int NO>
__global__ void __launch_bounds__(SA_MAX_WARPS * 32) sigmoid_attention_kernel(const SigArgs a) {
    extern __shared__ float smem[];
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.H, d = a.d, dv = a.dv, rs = a.d + a.dv;
    float* qs = smem;                          // [H][d]
    float* ws = qs + H * d;                    // [H][32] weights of the tile
    float* ms = ws + H * SA_KEYS;              // [H][32] mixed
    float* tk = ms + H * SA_KEYS;              // [H][H]
    const int n = blockIdx.x, seg = blockIdx.y;
    const int pos = a.positions[n];
    const int lo = seg * a.segment_keys;
    const int hi = a.segments > 1 ? min(pos, lo + a.segment_keys - 1) : pos;     // last key of this block
    const int hpg = H / a.G;
    const int* table = a.tables + (size_t)a.token_request[n] * a.width;
    const T* pages = reinterpret_cast<const T*>(a.pages);
    const T* q = reinterpret_cast<const T*>(a.q) + (size_t)n * a.q_t;
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) qs[i] = to_float(q[i]);
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = a.talk[i];
    const int heads_per_warp = (H + nw - 1) / nw;
    // accumulators: head `warp + k nw`, value columns lane + 32 i
    float acc[2][NO];
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int i = 0; i < NO; ++i) acc[k][i] = 0.f;
    __syncthreads();
    for (int k0 = lo; k0 <= hi; k0 += SA_KEYS) {
        const int key = k0 + lane;
        const bool valid = key <= hi;
        const int page = valid ? table[key / a.page_size] : -1;
        for (int k = 0; k < heads_per_warp; ++k) {
            const int g = warp + k * nw;
            if (g >= H) break;
            float w = 0.f;
            if (page >= 0) {
                const T* kr = pages + (((size_t)page * a.G + g / hpg) * a.page_size + key % a.page_size) * rs;
                const float* qg = qs + g * d;
                float s = 0.f;
                for (int i = 0; i < d; ++i) s = fmaf(qg[i], to_float(kr[i]), s);
                s *= a.scale;
                if (a.cap > 0.f) s = a.cap * tanhf(s / a.cap);
                w = 1.f / (1.f + expf(-(s + a.pb[g])));
            }
            ws[g * SA_KEYS + lane] = w;
        }
        __syncthreads();
        for (int k = 0; k < heads_per_warp; ++k) {
            const int h = warp + k * nw;
            if (h >= H) break;
            float m = 0.f;
            for (int g = 0; g < H; ++g) m = fmaf(tk[h * H + g], ws[g * SA_KEYS + lane], m);
            ms[h * SA_KEYS + lane] = m;
        }
        __syncwarp();
        const int j_hi = min(SA_KEYS - 1, hi - k0);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int h = warp + k * nw;
            if (k < heads_per_warp && h < H) {
                const float* mh = ms + h * SA_KEYS;
                for (int j = 0; j <= j_hi; ++j) {
                    const int kj = k0 + j;
                    const int pg = table[kj / a.page_size];
                    if (pg < 0) continue;
                    const T* vr = pages + (((size_t)pg * a.G + h / hpg) * a.page_size + kj % a.page_size) * rs + d;
                    const float m = mh[j];
#pragma unroll
                    for (int i = 0; i < NO; ++i) {
                        const int c = lane + 32 * i;
                        if (c < dv) acc[k][i] = fmaf(m, to_float(vr[c]), acc[k][i]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int h = warp + k * nw;
        if (k < heads_per_warp && h < H) {
#pragma unroll
            for (int i = 0; i < NO; ++i) {
                const int c = lane + 32 * i;
                if (c >= dv) continue;
                if (a.segments > 1) a.partial[((size_t)n * a.segments + seg) * H * dv + (size_t)h * dv + c] = acc[k][i];
                else reinterpret_cast<T*>(a.out)[(size_t)n * a.out_t + (size_t)h * dv + c] = from_float<T>(acc[k][i]);
            }
        }
    }
}

// out[n, c] = sum over the segments that hold a visible key of partial[n, segment, c], in their order.
template <typename T>
__global__ void sigmoid_segments_kernel(const float* __restrict__ partial, const int* __restrict__ positions, T* __restrict__ out,
                                        long out_t, int W, int segments, int segment_keys) {
    const int n = blockIdx.x;
    const int used = min(segments, positions[n] / segment_keys + 1);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < used; ++k) s += partial[((size_t)n * segments + k) * W + c];
        out[(size_t)n * out_t + c] = from_float<T>(s);
    }
}

}  // namespace

LLMP_API int llmp_sig_qkv_post(const float* qkv, long qkv_t, const void* bias, int bias_dtype, const float* cos_t,
                               const float* sin_t, int rot, void* q_out, int dtype, long q_out_t, const int* slots, void* pages,
                               int page_size, int N, int H, int G, int d, int dv, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && d > 0 && dv > 0 && rot >= 0 && rot <= d && rot % 2 == 0, "sig_qkv_post: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d rotated=%d",
                 H, G, d, dv, rot);
    LLMP_REQUIRE(!rot || (cos_t && sin_t), "sig_qkv_post: a rotation needs its tables");
    LLMP_REQUIRE(!pages || (slots && page_size > 0), "sig_qkv_post: pages need slots and a page size");
    if (dtype == LLMP_BF16)
        sig_qkv_post_kernel<bf16><<<N, 256, 0, stream>>>(qkv, qkv_t, bias, (int)(bias_dtype == LLMP_BF16), cos_t, sin_t, rot, (bf16*)q_out,
                                                         q_out_t, slots, (bf16*)pages, page_size, H, G, d, dv);
    else
        sig_qkv_post_kernel<float><<<N, 256, 0, stream>>>(qkv, qkv_t, bias, (int)(bias_dtype == LLMP_BF16), cos_t, sin_t, rot, (float*)q_out,
                                                          q_out_t, slots, (float*)pages, page_size, H, G, d, dv);
    return llmp_check_launch("sig_qkv_post");
}

LLMP_API int llmp_sigmoid_attention(const void* q, long q_t, const void* pages, int dtype, const int* tables, int width,
                                    const int* token_request, const int* positions, const float* talk, const float* pb,
                                    void* out, long out_t, float* partial, int segments, int segment_keys, int N, int H, int G,
                                    int d, int dv, int page_size, float scale, float cap, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && dv > 0 && dv <= 512 && page_size > 0 && width > 0,
                 "sigmoid_attention: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d page=%d width=%d", H, G, d, dv, page_size, width);
    LLMP_REQUIRE(H <= 2 * SA_MAX_WARPS, "sigmoid_attention: the general kernel takes up to %d heads, got %d", 2 * SA_MAX_WARPS, H);
    LLMP_REQUIRE(segments >= 1 && segments <= 65535 && (segments == 1 || (partial && segment_keys > 0 && segment_keys % SA_KEYS == 0)),
                 "sigmoid_attention: %d segments of %d keys", segments, segment_keys);
    SigArgs a;
    a.q = q; a.q_t = q_t; a.pages = pages; a.tables = tables; a.width = width; a.token_request = token_request;
    a.positions = positions; a.talk = talk; a.pb = pb; a.out = out; a.out_t = out_t; a.partial = partial;
    a.H = H; a.G = G; a.d = d; a.dv = dv; a.page_size = page_size; a.segments = segments; a.segment_keys = segments > 1 ? segment_keys : 0;
    a.scale = scale; a.cap = cap;
    const int nw = H < SA_MAX_WARPS ? H : SA_MAX_WARPS;
    const size_t smem = ((size_t)H * d + 2 * (size_t)H * SA_KEYS + (size_t)H * H) * sizeof(float);
    LLMP_REQUIRE(smem <= 200 * 1024, "sigmoid_attention: %d heads of %d entries do not fit shared memory", H, d);
    dim3 grid(N, segments);
#define LLMP_SA(T, NO)                                                               \
    do {                                                                             \
        LLMP_ALLOW_SMEM((sigmoid_attention_kernel<T, NO>), smem);                    \
        sigmoid_attention_kernel<T, NO><<<grid, nw * 32, smem, stream>>>(a);         \
    } while (0)
#define LLMP_SA_DV(T)                          \
    do {                                       \
        if (dv <= 32) LLMP_SA(T, 1);           \
        else if (dv <= 64) LLMP_SA(T, 2);      \
        else if (dv <= 128) LLMP_SA(T, 4);     \
        else if (dv <= 256) LLMP_SA(T, 8);     \
        else LLMP_SA(T, 16);                   \
    } while (0)
    if (dtype == LLMP_F32) LLMP_SA_DV(float); else LLMP_SA_DV(bf16);
#undef LLMP_SA_DV
#undef LLMP_SA
    if (segments > 1) {
        if (dtype == LLMP_F32)
            sigmoid_segments_kernel<float><<<N, 256, 0, stream>>>(partial, positions, (float*)out, out_t, H * dv, segments, segment_keys);
        else
            sigmoid_segments_kernel<bf16><<<N, 256, 0, stream>>>(partial, positions, (bf16*)out, out_t, H * dv, segments, segment_keys);
    }
    return llmp_check_launch("sigmoid_attention");
}
