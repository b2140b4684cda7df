// Attention over a cache of latent vectors: every token leaves one row [rank + rot] in the pages (a normed latent
// vector c and a rotated key part that all heads share); a head's unrotated key and its value are linear maps of c.
// Both maps are moved to the query's side: with q_lat = W_uk^T q_plain a score is (q_lat . c + q_rot . k_rot) * scale,
// and a head's value output is W_uv (sum_j p_j c_j). So all heads read the same rows, as keys [rank + rot] and, their
// first `rank` entries, as values. Scores, softmax and the weighted sums are float32.
//
//   latent_kv_post: per token, the norm of the latent part, the rotation of the shared key part and of every head's
//                   rotated query part, and the write of the row to the token's place in the pages.
//   latent_attention_kernel: the general kernel (float32 or bfloat16, any sizes, any mix of portions): one warp per
//                   (token, head), key tiles of 32 aligned to key 0, so a row's operations do not depend on the step.
#include "common.cuh"

#define LA_KEYS 32
#define LA_WARPS 8

template <typename T>
__global__ void latent_kv_post_kernel(T* __restrict__ qd, long ld, int H, int d, int r, int rank, const void* __restrict__ nw,
                                      int nw_bf16, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                      int rot_dims, const int* __restrict__ slots, T* __restrict__ pages) {
    __shared__ float scratch[32];
    const int n = blockIdx.x;
    T* q = qd + (size_t)n * ld;
    const T* dkv = q + (size_t)H * (d + r);
    const int half = rot_dims / 2;
    const float* cs = cos_t + (size_t)n * half;
    const float* sn = sin_t + (size_t)n * half;
    const int slot = slots ? slots[n] : -1;
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = to_float(dkv[c]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)rank + eps);
    if (slot >= 0) {
        T* row = pages + (size_t)slot * (rank + r);
        for (int c = threadIdx.x; c < rank; c += blockDim.x)
            row[c] = from_float<T>(to_float(dkv[c]) * rstd * load_as_float(nw, nw_bf16, c));
        for (int i = threadIdx.x; i < r; i += blockDim.x) {
            float v;
            if (i < half) v = to_float(dkv[rank + i]) * cs[i] - to_float(dkv[rank + i + half]) * sn[i];
            else if (i < rot_dims) v = to_float(dkv[rank + i]) * cs[i - half] + to_float(dkv[rank + i - half]) * sn[i - half];
            else v = to_float(dkv[rank + i]);
            row[rank + i] = from_float<T>(v);
        }
    }
    // every head's rotated query part, in place (a pair is read and written by one thread)
    for (int e = threadIdx.x; e < H * half; e += blockDim.x) {
        const int h = e / half, i = e % half;
        T* qr = q + (size_t)h * (d + r) + d;
        const float a = to_float(qr[i]), b = to_float(qr[i + half]);
        qr[i] = from_float<T>(a * cs[i] - b * sn[i]);
        qr[i + half] = from_float<T>(b * cs[i] + a * sn[i]);
    }
}

LLMP_API int llmp_latent_kv_post(void* qd, int dtype, long ld, int H, int d, int r, int rank, const void* norm_w, int norm_w_dtype,
                                 float eps, const float* cos_t, const float* sin_t, int rot_dims, const int* slots, void* pages,
                                 int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && d >= 0 && r >= 0 && rank > 0 && rot_dims >= 0 && rot_dims <= r && rot_dims % 2 == 0,
                 "latent_kv_post: bad sizes heads=%d dim=%d rot=%d rank=%d rotated=%d", H, d, r, rank, rot_dims);
    LLMP_REQUIRE(rot_dims == 0 || (cos_t && sin_t), "latent_kv_post: a rotation needs its tables");
    if (dtype == LLMP_F32)
        latent_kv_post_kernel<float><<<N, 128, 0, stream>>>((float*)qd, ld, H, d, r, rank, norm_w, norm_w_dtype == LLMP_BF16, eps, cos_t,
                                                            sin_t, rot_dims, slots, (float*)pages);
    else
        latent_kv_post_kernel<bf16><<<N, 128, 0, stream>>>((bf16*)qd, ld, H, d, r, rank, norm_w, norm_w_dtype == LLMP_BF16, eps, cos_t,
                                                           sin_t, rot_dims, slots, (bf16*)pages);
    return llmp_check_launch("latent_kv_post");
}

// The same step for float32 products that arrive apart: `q` [N, H (d + r)] (every head's plain and rotated query part),
// `dkv` [N, rank + r] or null (a layer that reads another layer's rows writes none). The queries leave in the compute type
// with their rotated parts rotated, the row goes to the pages. `interleaved`: entry 2i is paired with entry 2i + 1 instead
// of entry i with entry i + rot_dims / 2.
template <typename T>
__global__ void latent_rows_post_kernel(const float* __restrict__ q, long q_t, const float* __restrict__ dkv, long dkv_t, int H, int d,
                                        int r, int rank, const void* __restrict__ nw, int nw_bf16, float eps,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims, int interleaved,
                                        T* __restrict__ q_out, long q_out_t, const int* __restrict__ slots, T* __restrict__ pages) {
    __shared__ float scratch[32];
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    const int n = blockIdx.x;
    const int half = rot_dims / 2;
    const float* cs = cos_t + (size_t)n * half;
    const float* sn = sin_t + (size_t)n * half;
    const int slot = (slots && dkv) ? slots[n] : -1;
    if (slot >= 0) {
        const float* row_in = dkv + (size_t)n * dkv_t;
        float ss = 0.f;
        for (int c = threadIdx.x; c < rank; c += blockDim.x) ss = fmaf(row_in[c], row_in[c], ss);
        ss = block_sum(ss, scratch);
        const float rstd = 1.f / sqrtf(ss / (float)rank + eps);
        T* row = pages + (size_t)slot * (rank + r);
        for (int c = threadIdx.x; c < rank; c += blockDim.x)
            row[c] = from_float<T>(row_in[c] * rstd * load_as_float(nw, nw_bf16, c));
        for (int i = threadIdx.x; i < r; i += blockDim.x) {
            float v = row_in[rank + i];
            if (i < rot_dims) {
                const int f = interleaved ? i >> 1 : (i < half ? i : i - half);
                const bool first = interleaved ? !(i & 1) : i < half;
                const int partner = interleaved ? i ^ 1 : (i < half ? i + half : i - half);
                const float o = row_in[rank + partner];
                v = first ? v * cs[f] - o * sn[f] : v * cs[f] + o * sn[f];
            }
            row[rank + i] = from_float<T>(v);
        }
    }
    const float* q_in = q + (size_t)n * q_t;
    T* qo = q_out + (size_t)n * q_out_t;
    const int per = d + r;
    for (int e = threadIdx.x; e < H * per; e += blockDim.x) {
        const int i = e % per - d;                     // place in the head's rotated part, negative in the plain part
        float v = q_in[e];
        if (i >= 0 && i < rot_dims) {
            const int f = interleaved ? i >> 1 : (i < half ? i : i - half);
            const bool first = interleaved ? !(i & 1) : i < half;
            const int partner = interleaved ? i ^ 1 : (i < half ? i + half : i - half);
            const float o = q_in[e - i + partner];
            v = first ? v * cs[f] - o * sn[f] : v * cs[f] + o * sn[f];
        }
        qo[e] = from_float<T>(v);
    }
}

LLMP_API int llmp_latent_rows_post(const float* q, long q_t, const float* dkv, long dkv_t, int H, int d, int r, int rank,
                                   const void* norm_w, int norm_w_dtype, float eps, const float* cos_t, const float* sin_t,
                                   int rot_dims, int interleaved, void* q_out, int dtype, long q_out_t, const int* slots, void* pages,
                                   int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && d >= 0 && r >= 0 && rank > 0 && rot_dims >= 0 && rot_dims <= r && rot_dims % 2 == 0,
                 "latent_rows_post: bad sizes heads=%d dim=%d rot=%d rank=%d rotated=%d", H, d, r, rank, rot_dims);
    LLMP_REQUIRE(rot_dims == 0 || (cos_t && sin_t), "latent_rows_post: a rotation needs its tables");
    LLMP_REQUIRE(dkv == nullptr || pages == nullptr || norm_w != nullptr, "latent_rows_post: the latent's norm weight is missing");
    if (dtype == LLMP_F32)
        llmp_launch_dependent(latent_rows_post_kernel<float>, dim3(N), dim3(128), 0, stream, q, q_t, dkv, dkv_t, H, d, r, rank, norm_w, (int)(norm_w_dtype == LLMP_BF16), eps,
                                                              cos_t, sin_t, rot_dims, interleaved, (float*)q_out, q_out_t, slots, (float*)pages);
    else
        llmp_launch_dependent(latent_rows_post_kernel<bf16>, dim3(N), dim3(128), 0, stream, q, q_t, dkv, dkv_t, H, d, r, rank, norm_w, (int)(norm_w_dtype == LLMP_BF16), eps,
                                                             cos_t, sin_t, rot_dims, interleaved, (bf16*)q_out, q_out_t, slots, (bf16*)pages);
    return llmp_check_launch("latent_rows_post");
}

struct LatentArgs {
    const void* q_lat; long ql_t, ql_h;      // [token, head, rank] with strides in elements
    const void* q_rot; long qr_t, qr_h;      // [token, head, rot]
    const void* pages;                       // [pages * page_size, rank + rot]
    const int* tables; int width;            // [requests, width]
    const int* token_request; const int* positions;
    void* out; long o_t, o_h;                // [token, head, rank]
    int H, rank, rot, page_size;
    float scale;
    const float* sink;                       // [H] or null: exp(sink[h]) is added to head h's denominator
};

template <typename T, int NO>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(const LatentArgs a) {
    extern __shared__ float smem[];
    const int dk = a.rank + a.rot;
    const int ks = dk | 1;                                   // odd row stride: the lanes of a warp hit different banks
    float* Ks = smem;                                        // [LA_KEYS][ks]
    float* qs = Ks + LA_KEYS * ks;                           // [LA_WARPS][dk]
    float* ps = qs + LA_WARPS * dk;                          // [LA_WARPS][LA_KEYS]
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * LA_WARPS + warp;
    const bool active = h < a.H;
    const int pos = a.positions[n];
    const int* table = a.tables + (size_t)a.token_request[n] * a.width;
    const T* pages = reinterpret_cast<const T*>(a.pages);
    if (active) {
        const T* ql = reinterpret_cast<const T*>(a.q_lat) + (size_t)n * a.ql_t + (size_t)h * a.ql_h;
        const T* qr = reinterpret_cast<const T*>(a.q_rot) + (size_t)n * a.qr_t + (size_t)h * a.qr_h;
        for (int i = lane; i < a.rank; i += 32) qs[warp * dk + i] = to_float(ql[i]) * a.scale;
        for (int i = lane; i < a.rot; i += 32) qs[warp * dk + a.rank + i] = to_float(qr[i]) * a.scale;
    }
    float o[NO];
#pragma unroll
    for (int i = 0; i < NO; ++i) o[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    if (active && a.sink) { m_run = a.sink[h]; l_run = 1.f; }      // the sink: a key of that score without a value
    for (int k0 = 0; k0 <= pos; k0 += LA_KEYS) {
        __syncthreads();
        for (int j = warp; j < LA_KEYS; j += LA_WARPS) {     // a warp copies a key's row
            const int key = k0 + j;
            if (key <= pos) {
                const int page = table[key / a.page_size];
                const T* row = pages + ((size_t)page * a.page_size + key % a.page_size) * dk;
                for (int i = lane; i < dk; i += 32) Ks[j * ks + i] = to_float(row[i]);
            } else {
                for (int i = lane; i < dk; i += 32) Ks[j * ks + i] = 0.f;
            }
        }
        __syncthreads();
        if (!active) continue;
        const bool valid = k0 + lane <= pos;
        float s = 0.f;
        const float* kr = Ks + lane * ks;
        const float* qw = qs + warp * dk;
        for (int i = 0; i < dk; ++i) s = fmaf(qw[i], kr[i], s);
        s = valid ? s : -INFINITY;
        const float m_new = fmaxf(m_run, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m_run - m_new);             // 0 at the first tile (m_run = -inf, m_new finite: key k0 is visible)
        l_run = l_run * alpha + warp_sum(p);
        m_run = m_new;
        ps[warp * LA_KEYS + lane] = p;
        __syncwarp();
        const int keys = min(LA_KEYS, pos - k0 + 1);
#pragma unroll
        for (int i = 0; i < NO; ++i) {
            const int c = lane + 32 * i;
            if (c < a.rank) {
                float acc = o[i] * alpha;
                for (int j = 0; j < keys; ++j) acc = fmaf(ps[warp * LA_KEYS + j], Ks[j * ks + c], acc);
                o[i] = acc;
            }
        }
        __syncwarp();
    }
    if (!active) return;
    const float inv = 1.f / l_run;
    T* dst = reinterpret_cast<T*>(a.out) + (size_t)n * a.o_t + (size_t)h * a.o_h;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        const int c = lane + 32 * i;
        if (c < a.rank) dst[c] = from_float<T>(o[i] * inv);
    }
}

template <typename T>
static int launch_latent(const LatentArgs& a, int N, cudaStream_t stream) {
    const int dk = a.rank + a.rot;
    const size_t smem = ((size_t)LA_KEYS * (dk | 1) + (size_t)LA_WARPS * dk + LA_WARPS * LA_KEYS) * sizeof(float);
    LLMP_REQUIRE(smem <= 220 * 1024, "latent_attention: rows of %d entries do not fit shared memory", dk);
    dim3 grid(N, (a.H + LA_WARPS - 1) / LA_WARPS);
#define LLMP_LA_LAUNCH(NO)                                                         \
    do {                                                                           \
        LLMP_ALLOW_SMEM((latent_attention_kernel<T, NO>), smem);                   \
        latent_attention_kernel<T, NO><<<grid, LA_WARPS * 32, smem, stream>>>(a);  \
    } while (0)
    if (a.rank <= 128) LLMP_LA_LAUNCH(4);
    else if (a.rank <= 256) LLMP_LA_LAUNCH(8);
    else if (a.rank <= 512) LLMP_LA_LAUNCH(16);
    else LLMP_LA_LAUNCH(32);
#undef LLMP_LA_LAUNCH
    return llmp_check_launch("latent_attention");
}

LLMP_API int llmp_latent_attention(const void* q_lat, long ql_t, long ql_h, const void* q_rot, long qr_t, long qr_h, const void* pages,
                                   int dtype, const int* tables, int width, const int* token_request, const int* positions, void* out,
                                   long o_t, long o_h, int N, int H, int rank, int rot, int page_size, float scale,
                                   const float* sink, cudaStream_t stream) {
    if (N <= 0) return 0;
    LLMP_REQUIRE(H > 0 && rank > 0 && rank <= 1024 && rot >= 0 && page_size > 0 && width > 0,
                 "latent_attention: bad sizes heads=%d rank=%d rot=%d page=%d width=%d", H, rank, rot, page_size, width);
    LLMP_REQUIRE((H + LA_WARPS - 1) / LA_WARPS <= 65535, "latent_attention: too many heads %d", H);
    LatentArgs a;
    a.q_lat = q_lat; a.ql_t = ql_t; a.ql_h = ql_h;
    a.q_rot = q_rot; a.qr_t = qr_t; a.qr_h = qr_h;
    a.pages = pages; a.tables = tables; a.width = width; a.token_request = token_request; a.positions = positions;
    a.out = out; a.o_t = o_t; a.o_h = o_h;
    a.H = H; a.rank = rank; a.rot = rot; a.page_size = page_size; a.scale = scale; a.sink = sink;
    return dtype == LLMP_F32 ? launch_latent<float>(a, N, stream) : launch_latent<bf16>(a, N, stream);
}
