// Sigmoid attention with mixed heads on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulate),
// with the contract of llmp_sigmoid_attention for bfloat16 pages and up to SM_MAX_HEADS query heads.
//
// A block takes a tile of up to 16 consecutive new tokens of one request and one range of keys, with a warp per
// query head. Keys are walked in tiles of 32 aligned to key 0. For a key tile
//   1. warp g multiplies its head's 16 queries with the 32 keys of its key/value head, caps the scores, takes the
//      sigmoid (float32) and leaves the 16 x 32 weights in shared memory, in the layout of the accumulator registers;
//   2. warp h adds the weights of all heads with the coefficients of row h of the mixing matrix (float32; every lane
//      reads the entries that it holds itself in the accumulator layout, so the reads are dense);
//   3. warp h rounds its mixed weights to bfloat16 and multiplies them with the 32 values of its key/value head.
// Nothing is normalised over keys, so the output registers simply add up over key tiles and key ranges: with more
// than one range the blocks leave float32 partial sums that a second kernel adds in the order of the ranges.
// The keys of the next tile are copied (cp.async) while the weights are mixed and multiplied with the values, the
// values of the next tile while the next scores are made.
#include "common.cuh"

namespace {

constexpr int SM_MAX_HEADS = 16;
constexpr int SM_ROWS = 16;
constexpr int SM_KEYS = 32;

struct SigMmaArgs {
    const bf16* q; long q_t;
    const bf16* pages;
    const int* tables; int width;
    const int* q_start; const int* ctx_len;
    const int* tile_req; const int* tile_tok0; int num_tiles;
    const float* talk; const float* pb;
    bf16* out; long out_t;
    float* partial;
    int H, G, page_size, segments, segment_keys;
    float scale, cap;
};

__device__ __forceinline__ void sm_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void sm_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void sm_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void sm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned sm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// sigmoid(cap tanh(s / cap) + b) with tanh(x) = 1 - 2 / (1 + e^(2x)); the exponentials' relative error is about 2^-21,
// which leaves the weight's absolute error near 1e-7.
__device__ __forceinline__ float sm_weight(float s, float cap, float inv_cap, float b) {
    if (cap > 0.f) s = cap * (1.f - __fdividef(2.f, 1.f + __expf(2.f * s * inv_cap)));
    return __fdividef(1.f, 1.f + __expf(-(s + b)));
}

// D16: dim / 16, DV16: vdim / 16. One warp per query head.
template <int D16, int DV16>
__global__ void __launch_bounds__(SM_MAX_HEADS * 32, 1) sigmoid_attention_mma_kernel(const SigMmaArgs a) {
    extern __shared__ __align__(16) unsigned char sm_smem[];
    constexpr int D = D16 * 16, DV = DV16 * 16;
    constexpr int KS = D + 8, VS = DV + 8;                          // padded rows: conflict-free ldmatrix
    const int H = a.H, G = a.G, hpg = H / G, rs = D + DV;
    bf16* Qs = reinterpret_cast<bf16*>(sm_smem);                    // [H][16][KS]
    bf16* Ks = Qs + (size_t)H * SM_ROWS * KS;                       // [G][32][KS]
    bf16* Vs = Ks + (size_t)G * SM_KEYS * KS;                       // [G][32][VS]
    float4* Ws = reinterpret_cast<float4*>(Vs + (size_t)G * SM_KEYS * VS);   // [H][4][32 lanes] of 4 floats
    float* tk = reinterpret_cast<float*>(Ws + (size_t)H * 4 * 32);  // [H][H]
    __shared__ long long key_off[SM_KEYS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
    const int gr = lane >> 2, t = lane & 3;
    const int tile = a.num_tiles - 1 - (int)blockIdx.x;             // the tiles that see most keys start first
    const int seg = blockIdx.y;
    const int r = a.tile_req[tile], tok0 = a.tile_tok0[tile];
    const int q_begin = a.q_start[r];
    const int q_len = a.q_start[r + 1] - q_begin;
    const int pos0 = a.ctx_len[r] - q_len;
    int ntok = q_len - tok0;
    if (ntok > SM_ROWS) ntok = SM_ROWS;
    const int first = q_begin + tok0;                               // the tile's first row among the step's tokens
    int lo = 0, hi = pos0 + tok0 + ntok - 1;                        // keys of this block (inclusive)
    if (a.segments > 1) {
        lo = seg * a.segment_keys;
        hi = min(hi, lo + a.segment_keys - 1);
        if (lo > hi) return;                                        // nothing of this range is visible: its sums are never read
    }
    const int* table = a.tables + (size_t)r * a.width;

    constexpr int QV = D / 8, VV = DV / 8;
    for (int e = tid; e < H * SM_ROWS * QV; e += nthreads) {
        const int c = (e % QV) * 8, row = (e / QV) % SM_ROWS, h = e / (QV * SM_ROWS);
        const bool ok = row < ntok;
        sm_cp_async_16(Qs + ((size_t)h * SM_ROWS + row) * KS + c, ok ? a.q + (size_t)(first + row) * a.q_t + (size_t)h * D + c : a.q, ok);
    }
    for (int i = tid; i < H * H; i += nthreads) tk[i] = a.talk[i];
    auto issue_keys = [&](int j0) {
        if (j0 <= hi) {
            if (tid < SM_KEYS) {
                const int j = j0 + tid;
                long long off = -1;
                if (j <= hi) {
                    const int page = table[j / a.page_size];
                    if (page >= 0) off = (long long)(((size_t)page * G) * a.page_size + (j % a.page_size)) * rs;
                }
                key_off[tid] = off;
            }
            __syncthreads();
            for (int e = tid; e < G * SM_KEYS * QV; e += nthreads) {
                const int c = (e % QV) * 8, key = (e / QV) % SM_KEYS, kv = e / (QV * SM_KEYS);
                const long long off = key_off[key];
                const bool ok = off >= 0;
                sm_cp_async_16(Ks + ((size_t)kv * SM_KEYS + key) * KS + c, ok ? a.pages + off + (size_t)kv * a.page_size * rs + c : a.pages, ok);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    auto issue_values = [&](int j0) {        // after issue_keys of the same tile: its offsets are still in place
        if (j0 <= hi) {
            for (int e = tid; e < G * SM_KEYS * VV; e += nthreads) {
                const int c = (e % VV) * 8, key = (e / VV) % SM_KEYS, kv = e / (VV * SM_KEYS);
                const long long off = key_off[key];
                const bool ok = off >= 0;
                sm_cp_async_16(Vs + ((size_t)kv * SM_KEYS + key) * VS + c, ok ? a.pages + off + (size_t)kv * a.page_size * rs + D + c : a.pages, ok);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    const int h = warp;                                             // this warp's head, in all three steps
    const int kvh = h / hpg;
    int row_pos[2];
    row_pos[0] = gr < ntok ? pos0 + tok0 + gr : -1;
    row_pos[1] = gr + 8 < ntok ? pos0 + tok0 + gr + 8 : -1;
    const float bias = a.pb[h], inv_cap = a.cap > 0.f ? 1.f / a.cap : 0.f;
    float o[2 * DV16][4];
#pragma unroll
    for (int i = 0; i < 2 * DV16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const int tile_lo = (lo / SM_KEYS) * SM_KEYS;                   // lo is a multiple of the key tile anyway
    issue_keys(tile_lo);                                            // group: the queries and the first keys
    issue_values(tile_lo);
    const bf16* Qw = Qs + ((size_t)h * SM_ROWS + (lane & 15)) * KS + (lane >> 4) * 8;
    const bf16* Kw = Ks + (size_t)kvh * SM_KEYS * KS;
    const bf16* Vw = Vs + (size_t)kvh * SM_KEYS * VS;
    for (int j0 = tile_lo; j0 <= hi; j0 += SM_KEYS) {
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");     // this tile's keys are here
        __syncthreads();
        float s[4][4];
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D16; ++ks) {
            unsigned qa[4];
            sm_ldmatrix_x4(qa, Qw + ks * 16);
#pragma unroll
            for (int nb = 0; nb < 4; nb += 2) {
                unsigned kf[4];
                sm_ldmatrix_x4(kf, Kw + (size_t)((nb + (lane >> 4)) * 8 + (lane & 7)) * KS + ks * 16 + ((lane >> 3) & 1) * 8);
                sm_mma(s[nb], qa, kf[0], kf[1]);
                sm_mma(s[nb + 1], qa, kf[2], kf[3]);
            }
        }
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) {
            float w[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int j = j0 + nb * 8 + 2 * t + (c & 1);
                w[c] = j <= row_pos[c >> 1] ? sm_weight(s[nb][c] * a.scale, a.cap, inv_cap, bias) : 0.f;
            }
            Ws[((size_t)h * 4 + nb) * 32 + lane] = make_float4(w[0], w[1], w[2], w[3]);
        }
        __syncthreads();                                            // all weights are in place, the keys are free
        issue_keys(j0 + SM_KEYS);
#pragma unroll
        for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
        for (int g = 0; g < H; ++g) {
            const float c = tk[h * H + g];
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
                const float4 w = Ws[((size_t)g * 4 + nb) * 32 + lane];
                s[nb][0] = fmaf(c, w.x, s[nb][0]); s[nb][1] = fmaf(c, w.y, s[nb][1]);
                s[nb][2] = fmaf(c, w.z, s[nb][2]); s[nb][3] = fmaf(c, w.w, s[nb][3]);
            }
        }
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");     // this tile's values are here
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            unsigned pa[4];
            pa[0] = sm_pack(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = sm_pack(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = sm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = sm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int nb2 = 0; nb2 < DV16; ++nb2) {
                unsigned v[4];
                sm_ldmatrix_x4_trans(v, Vw + (size_t)(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + nb2 * 16 + (lane >> 4) * 8);
                sm_mma(o[nb2 * 2], pa, v[0], v[1]);
                sm_mma(o[nb2 * 2 + 1], pa, v[2], v[3]);
            }
        }
        __syncthreads();                                            // the values and the weights are free
        issue_values(j0 + SM_KEYS);
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");

#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (row_pos[h2] < 0) continue;
        const size_t n = (size_t)first + gr + 8 * h2;
        if (a.segments > 1) {
            float* dst = a.partial + (n * a.segments + seg) * H * DV + (size_t)h * DV + 2 * t;
#pragma unroll
            for (int nb = 0; nb < 2 * DV16; ++nb) *reinterpret_cast<float2*>(dst + nb * 8) = make_float2(o[nb][2 * h2], o[nb][2 * h2 + 1]);
        } else {
            bf16* dst = a.out + n * a.out_t + (size_t)h * DV + 2 * t;
#pragma unroll
            for (int nb = 0; nb < 2 * DV16; ++nb) *reinterpret_cast<unsigned*>(dst + nb * 8) = sm_pack(o[nb][2 * h2], o[nb][2 * h2 + 1]);
        }
    }
}

size_t sm_smem_bytes(int H, int G, int d, int dv) {
    return sizeof(bf16) * ((size_t)H * SM_ROWS * (d + 8) + (size_t)G * SM_KEYS * (d + 8) + (size_t)G * SM_KEYS * (dv + 8)) +
           sizeof(float) * ((size_t)H * 16 * 32 + (size_t)H * H);
}

}  // namespace

namespace {

// out[n, c] = sum over the key ranges that hold a visible key of partial[n, range, c], in their order.
__global__ void sigmoid_mma_ranges_kernel(const float* __restrict__ partial, const int* __restrict__ positions, bf16* __restrict__ out,
                                          long out_t, int W, int segments, int segment_keys) {
    const int n = blockIdx.x;
    const int used = min(segments, positions[n] / segment_keys + 1);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < used; ++k) s += partial[((size_t)n * segments + k) * W + c];
        out[(size_t)n * out_t + c] = from_float<bf16>(s);
    }
}

}  // namespace

// Whether the tensor-core kernel takes these sizes (bfloat16 only).
LLMP_API int llmp_sigmoid_attention_mma_supports(int H, int G, int d, int dv) {
    if (H <= 0 || G <= 0 || H % G || H > SM_MAX_HEADS) return 0;
    auto instance = [](int x) { return x == 16 || x == 32 || x == 64 || x == 96 || x == 128; };
    if (!instance(d) || !instance(dv)) return 0;
    return sm_smem_bytes(H, G, d, dv) <= 220 * 1024 ? 1 : 0;
}

LLMP_API int llmp_sigmoid_attention_mma(const void* q, long q_t, const void* pages, const int* tables, int width, const int* q_start,
                                        const int* ctx_len, const int* positions, const int* tile_req, const int* tile_tok0,
                                        int num_tiles, const float* talk, const float* pb, void* out, long out_t, float* partial,
                                        int segments, int segment_keys, int N, int H, int G, int d, int dv, int page_size,
                                        float scale, float cap, cudaStream_t stream) {
    if (N <= 0 || num_tiles <= 0) return 0;
    LLMP_REQUIRE(llmp_sigmoid_attention_mma_supports(H, G, d, dv), "sigmoid_attention_mma: no kernel for heads=%d kv_heads=%d dim=%d vdim=%d",
                 H, G, d, dv);
    LLMP_REQUIRE(page_size > 0 && width > 0 && q_t % 8 == 0 && out_t % 2 == 0, "sigmoid_attention_mma: page=%d width=%d, rows must be 16-byte aligned",
                 page_size, width);
    LLMP_REQUIRE(segments >= 1 && segments <= 65535 && (segments == 1 || (partial && segment_keys > 0 && segment_keys % SM_KEYS == 0)),
                 "sigmoid_attention_mma: %d key ranges of %d keys", segments, segment_keys);
    SigMmaArgs a;
    a.q = (const bf16*)q; a.q_t = q_t; a.pages = (const bf16*)pages; a.tables = tables; a.width = width; a.q_start = q_start;
    a.ctx_len = ctx_len; a.tile_req = tile_req; a.tile_tok0 = tile_tok0; a.num_tiles = num_tiles; a.talk = talk; a.pb = pb;
    a.out = (bf16*)out; a.out_t = out_t; a.partial = partial; a.H = H; a.G = G; a.page_size = page_size; a.segments = segments;
    a.segment_keys = segments > 1 ? segment_keys : 0; a.scale = scale; a.cap = cap;
    const size_t smem = sm_smem_bytes(H, G, d, dv);
    dim3 grid(num_tiles, segments);
#define LLMP_SM_CASE(A, B)                                                                   \
    if (d == 16 * A && dv == 16 * B) {                                                       \
        LLMP_ALLOW_SMEM((sigmoid_attention_mma_kernel<A, B>), smem);                         \
        sigmoid_attention_mma_kernel<A, B><<<grid, H * 32, smem, stream>>>(a);               \
    } else
#define LLMP_SM_ROW(A) LLMP_SM_CASE(A, 1) LLMP_SM_CASE(A, 2) LLMP_SM_CASE(A, 4) LLMP_SM_CASE(A, 6) LLMP_SM_CASE(A, 8)
    LLMP_SM_ROW(1) LLMP_SM_ROW(2) LLMP_SM_ROW(4) LLMP_SM_ROW(6) LLMP_SM_ROW(8)
    {
        llmp_set_error("sigmoid_attention_mma: dim=%d vdim=%d has no instance", d, dv);
        return 1;
    }
#undef LLMP_SM_ROW
#undef LLMP_SM_CASE
    if (segments > 1)
        sigmoid_mma_ranges_kernel<<<N, 256, 0, stream>>>(partial, positions, (bf16*)out, out_t, H * dv, segments, segment_keys);
    return llmp_check_launch("sigmoid_attention_mma");
}
