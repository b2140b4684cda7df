// Latent attention on the tensor cores (bfloat16, mma.sync m16n8k16, float32 sums), with the interface of
// llmp_latent_attention: rows (token, head) attend over cached rows [rank + rot] that all heads share; a cached row is
// the key, its first `rank` entries are the value.
//
// A block takes a tile of 64 rows (consecutive tokens of one request, the head running fastest, so the key tile it
// streams serves every head), one chunk of value columns (128, or 256 for latents above 128), and, in a step whose
// requests bring few tokens over long contexts, one segment of the keys. Eight warps: warp w owns the 16 rows of row
// group w & 3 and, of every 64-key tile, the 32 keys of half w >> 2, with a running softmax and output chunk of its
// own in registers; at the end the two warps of a row group add their sums in shared memory, first half first. A warp
// whose rows do not exist (a decode step fills 16 of the 64 rows or fewer) only helps with the copies. Keys are walked in tiles of 64 aligned to key 0 (the same
// operations for a row however the prompt was cut), copied from the pages with 16-byte cp.async; the key tile in shared memory is also the value tile. With
// segments, a block leaves its unnormalised sums, maximum and row sum in scratch and a second kernel adds the segments
// of a row in ascending order (segments are fixed ranges of key indices, so this too is the same for every step).
#include "common.cuh"

#define LM_ROWS 64
#define LM_KEYS 64
#define LM_THREADS 256

struct LatentMmaParams {
    const bf16* q_lat; long ql_t, ql_h;
    const bf16* q_rot; long qr_t, qr_h;
    bf16* out; long o_t, o_h;
    const bf16* pages;
    const int* tables; int table_stride;
    const int* q_start; const int* ctx_len; const int* tile_req; const int* tile_tok0;
    float* part_o; float* part_ml;
    int N, H, rank, rot, page_size, hpc, tokens_per_cta, head_chunks, num_tiles, v_chunks, seg_keys;
    float scale;
    const float* sink;          // [H] or null: exp(sink[h]) joins head h's denominator (in the kernel with the row's last keys, or in the merge)
};

__device__ __forceinline__ void lm_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void lm_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void lm_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void lm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float lm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ unsigned lm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// The barrier of a key half's four warps: ids 1 and 2 (0 is the block's own).
__device__ __forceinline__ void lm_half_barrier(int half) {
    if (half == 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
    else asm volatile("bar.sync 2, 128;\n" ::: "memory");
}

template <int LM_VCHUNK>
__global__ void __launch_bounds__(LM_THREADS, 1) latent_attention_mma_kernel(const LatentMmaParams p) {
    extern __shared__ __align__(16) unsigned char lm_smem[];
    __shared__ long long key_off[LM_KEYS];
    const int dk = p.rank + p.rot;
    const int STRIDE = dk + 8;                                   // padded rows: conflict-free ldmatrix
    const int vec_per_row = dk / 8;
    const int dk16 = dk / 16;
    bf16* Qs = reinterpret_cast<bf16*>(lm_smem);                 // [LM_ROWS][STRIDE]
    bf16* Ks = Qs + (size_t)LM_ROWS * STRIDE;                    // [LM_KEYS][STRIDE]: keys, and in their first columns values

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rg = warp & 3, half = warp >> 2;                  // row group and key half of this warp
    // later tiles of a prompt see more keys: the blocks of the last tile start first
    const int tile = p.num_tiles - 1 - (int)(blockIdx.x / (unsigned)p.head_chunks);
    const int hc = (int)(blockIdx.x % (unsigned)p.head_chunks);
    const int vchunk = blockIdx.y, seg = blockIdx.z;
    const int r = p.tile_req[tile];
    const int tok0 = p.tile_tok0[tile];
    const int hpc = p.hpc;
    const int head0 = hc * hpc;
    int heads = p.H - head0;
    if (heads > hpc) heads = hpc;
    const int q_begin = p.q_start[r];
    const int q_len = p.q_start[r + 1] - q_begin;
    const int pos0 = p.ctx_len[r] - q_len;
    int ntok = q_len - tok0;
    if (ntok > p.tokens_per_cta) ntok = p.tokens_per_cta;
    const int* table = p.tables + (size_t)r * p.table_stride;
    int hi = pos0 + tok0 + ntok - 1;                             // last key (inclusive)
    int lo = 0;
    if (p.seg_keys > 0) {
        lo = seg * p.seg_keys;
        if (lo > hi) return;                                     // no row of this tile sees the segment; the merge knows
        if (hi > lo + p.seg_keys - 1) hi = lo + p.seg_keys - 1;
    }
    const int v0 = vchunk * LM_VCHUNK;
    int v16 = (p.rank - v0) / 16;
    if (v16 > LM_VCHUNK / 16) v16 = LM_VCHUNK / 16;

    // query rows: row = token * hpc + head; columns [latent | rotated]
    for (int e = tid; e < LM_ROWS * vec_per_row; e += LM_THREADS) {
        const int row = e / vec_per_row, c = (e % vec_per_row) * 8;
        const int tl = row / hpc, h = row % hpc;
        const bool ok = tl < ntok && h < heads;
        const bf16* src = p.q_lat;
        if (ok) {
            const size_t n = (size_t)(q_begin + tok0 + tl);
            src = c < p.rank ? p.q_lat + n * p.ql_t + (size_t)(head0 + h) * p.ql_h + c
                             : p.q_rot + n * p.qr_t + (size_t)(head0 + h) * p.qr_h + (c - p.rank);
        }
        lm_cp_async_16(Qs + (size_t)row * STRIDE + c, src, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");

    int row_pos[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = rg * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        row_pos[h2] = (tl < ntok && h < heads) ? pos0 + tok0 + tl : -1;
    }
    float o[LM_VCHUNK / 8][4];
#pragma unroll
    for (int i = 0; i < LM_VCHUNK / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};

    const float scale_log2 = p.scale * 1.4426950408889634f;
    const int warp_last_tok = (rg * 16 + 15) / hpc;
    const int warp_hi_pos = pos0 + tok0 + (warp_last_tok < ntok ? warp_last_tok : ntok - 1);
    const int warp_first_tok = (rg * 16) / hpc;
    const bool warp_has_rows = warp_first_tok < ntok;
    const int warp_lo_pos = pos0 + tok0 + (warp_first_tok < ntok ? warp_first_tok : ntok - 1);
    const bf16* Qw = Qs + (size_t)(rg * 16 + (lane & 15)) * STRIDE + (lane >> 4) * 8;
    // The four warps of a key half are a pipeline of their own: they copy and read only their 32 rows of the key tile and
    // meet at a barrier of their own, so one half's copies run under the other half's products.
    const int gtid = tid & 127;                                   // thread within the half's four warps
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                                              // the query tile is in place for everybody
    for (int j0 = (lo / LM_KEYS) * LM_KEYS; j0 <= hi; j0 += LM_KEYS) {
        if (gtid < 32) {
            const int j = j0 + half * 32 + gtid;
            long long off = -1;
            if (j <= hi) {
                const int page = table[j / p.page_size];
                if (page >= 0) off = (long long)((size_t)page * p.page_size + (j % p.page_size)) * dk;
            }
            key_off[half * 32 + gtid] = off;
        }
        lm_half_barrier(half);
        for (int e = gtid; e < 32 * vec_per_row; e += 128) {
            const int key = half * 32 + e / vec_per_row, c = (e % vec_per_row) * 8;
            const long long off = key_off[key];
            lm_cp_async_16(Ks + (size_t)key * STRIDE + c, off >= 0 ? p.pages + off + c : p.pages, off >= 0);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        lm_half_barrier(half);
        do {
            const int jh = j0 + half * 32;
            if (!warp_has_rows || jh > warp_hi_pos || jh > hi) break;      // no row of this warp sees these keys
            float s[4][4];
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll 4
            for (int ks = 0; ks < dk16; ++ks) {
                unsigned qa[4];
                lm_ldmatrix_x4(qa, Qw + ks * 16);
#pragma unroll
                for (int nb = 0; nb < 4; nb += 2) {
                    unsigned kf[4];
                    lm_ldmatrix_x4(kf, Ks + (size_t)(half * 32 + (nb + (lane >> 4)) * 8 + (lane & 7)) * STRIDE + ks * 16 + ((lane >> 3) & 1) * 8);
                    lm_mma(s[nb], qa, kf[0], kf[1]);
                    lm_mma(s[nb + 1], qa, kf[2], kf[3]);
                }
            }
            // mask where the causal diagonal or the segment's end crosses these keys
            const bool need_mask = (jh + 31 > warp_lo_pos) || (jh + 31 > hi);
            float mx[2] = {-INFINITY, -INFINITY};
            if (need_mask) {
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int j = jh + nb * 8 + 2 * t + (c & 1);
                        if (j > row_pos[c >> 1] || j > hi) s[nb][c] = -INFINITY;
                    }
                }
            }
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mx[c >> 1] = fmaxf(mx[c >> 1], s[nb][c]);
            }
            float alpha[2], m_scaled[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
                const float m_new = fmaxf(m_run[h2], mx[h2] * scale_log2);
                alpha[h2] = (m_new > -INFINITY) ? lm_ex2(m_run[h2] - m_new) : 1.f;
                m_run[h2] = m_new;
                m_scaled[h2] = (m_new > -INFINITY) ? m_new : 0.f;
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float pr = lm_ex2(fmaf(s[nb][c], scale_log2, -m_scaled[c >> 1]));
                    s[nb][c] = pr;
                    sum[c >> 1] += pr;
                }
            }
            l_run[0] = l_run[0] * alpha[0] + sum[0];
            l_run[1] = l_run[1] * alpha[1] + sum[1];
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int i = 0; i < LM_VCHUNK / 8; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                unsigned pa[4];
                pa[0] = lm_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = lm_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = lm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = lm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int nb2 = 0; nb2 < LM_VCHUNK / 16; ++nb2) {
                    if (nb2 < v16) {
                        unsigned v[4];
                        lm_ldmatrix_x4_trans(v, Ks + (size_t)(half * 32 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + v0 + nb2 * 16 + (lane >> 4) * 8);
                        lm_mma(o[nb2 * 2], pa, v[0], v[1]);
                        lm_mma(o[nb2 * 2 + 1], pa, v[2], v[3]);
                    }
                }
            }
        } while (false);
        lm_half_barrier(half);      // the half's rows may be overwritten now
    }

#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    }
    // The two halves of a row group meet: the second half's warp leaves its maximum, row sum and sums in shared memory
    // (the query and key tiles are no longer read), the first half's warp adds them to its own and stores.
    {
        float* xo = reinterpret_cast<float*>(lm_smem);            // [4 row groups][32 lanes][LM_VCHUNK / 2 + 4]
        constexpr int PER_LANE = LM_VCHUNK / 2 + 4;
        float* mine = xo + ((size_t)rg * 32 + lane) * PER_LANE;
        __syncthreads();                                          // both halves are done with the query and key tiles
        if (half == 1) {
#pragma unroll
            for (int i = 0; i < LM_VCHUNK / 8; ++i)
                *reinterpret_cast<float4*>(mine + 4 * i) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
            *reinterpret_cast<float4*>(mine + LM_VCHUNK / 2) = make_float4(m_run[0], m_run[1], l_run[0], l_run[1]);
        }
        __syncthreads();
        if (half == 1) return;
        const float4 other = *reinterpret_cast<const float4*>(mine + LM_VCHUNK / 2);
        const float om[2] = {other.x, other.y}, ol[2] = {other.z, other.w};
        float wa[2], wb[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const float m = fmaxf(m_run[h2], om[h2]);
            wa[h2] = (m_run[h2] > -INFINITY) ? lm_ex2(m_run[h2] - m) : 0.f;
            wb[h2] = (om[h2] > -INFINITY) ? lm_ex2(om[h2] - m) : 0.f;
            l_run[h2] = l_run[h2] * wa[h2] + ol[h2] * wb[h2];
            m_run[h2] = m;
        }
#pragma unroll
        for (int i = 0; i < LM_VCHUNK / 8; ++i) {
            const float4 x = *reinterpret_cast<const float4*>(mine + 4 * i);
            o[i][0] = o[i][0] * wa[0] + x.x * wb[0];
            o[i][1] = o[i][1] * wa[0] + x.y * wb[0];
            o[i][2] = o[i][2] * wa[1] + x.z * wb[1];
            o[i][3] = o[i][3] * wa[1] + x.w * wb[1];
        }
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (row_pos[h2] < 0) continue;
        const int row = rg * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        const size_t n = (size_t)(q_begin + tok0 + tl);
        if (p.seg_keys > 0) {
            const size_t at = ((size_t)seg * p.N + n) * p.H + head0 + h;
            float* dst = p.part_o + at * p.rank + v0 + 2 * t;
#pragma unroll
            for (int nb = 0; nb < LM_VCHUNK / 8; ++nb)
                if (nb < 2 * v16) *reinterpret_cast<float2*>(dst + nb * 8) = make_float2(o[nb][2 * h2], o[nb][2 * h2 + 1]);
            if (vchunk == 0 && t == 0) {
                p.part_ml[at * 2] = m_run[h2];
                p.part_ml[at * 2 + 1] = l_run[h2];
            }
        } else {
            float inv = l_run[h2] > 0.f ? 1.f / l_run[h2] : 0.f;
            if (p.sink) {                                         // a key of score sink[h] without a value
                const float sk = p.sink[head0 + h] * 1.4426950408889634f;
                const float m = fmaxf(m_run[h2], sk);
                const float w = m_run[h2] > -INFINITY ? lm_ex2(m_run[h2] - m) : 0.f;
                inv = w / (l_run[h2] * w + lm_ex2(sk - m));
            }
            bf16* dst = p.out + n * p.o_t + (size_t)(head0 + h) * p.o_h + v0 + 2 * t;
#pragma unroll
            for (int nb = 0; nb < LM_VCHUNK / 8; ++nb)
                if (nb < 2 * v16) *reinterpret_cast<unsigned*>(dst + nb * 8) = lm_pack(o[nb][2 * h2] * inv, o[nb][2 * h2 + 1] * inv);
        }
    }
}

// Adds the segments of a row: out = sum_s 2^(m_s - m) o_s / sum_s 2^(m_s - m) l_s over the segments that hold keys the
// row sees, in ascending order. grid (tokens, heads).
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ positions,
                                    bf16* __restrict__ out, long o_t, long o_h, int N, int H, int rank, int seg_keys,
                                    const float* __restrict__ sink) {
    const int n = blockIdx.x, h = blockIdx.y;
    const int segs = positions[n] / seg_keys + 1;
    const float sk = sink ? sink[h] * 1.4426950408889634f : -INFINITY;
    float m = sk;
    for (int s = 0; s < segs; ++s) m = fmaxf(m, part_ml[(((size_t)s * N + n) * H + h) * 2]);
    float l = sink ? lm_ex2(sk - m) : 0.f;
    for (int s = 0; s < segs; ++s) {
        const size_t at = ((size_t)s * N + n) * H + h;
        l += lm_ex2(part_ml[at * 2] - m) * part_ml[at * 2 + 1];
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < segs; ++s) {
            const size_t at = ((size_t)s * N + n) * H + h;
            acc = fmaf(lm_ex2(part_ml[at * 2] - m), part_o[at * rank + c], acc);
        }
        out[(size_t)n * o_t + (size_t)h * o_h + c] = __float2bfloat16_rn(acc * inv);
    }
}

LLMP_API int llmp_latent_mma_tokens_per_tile(int H) { return LM_ROWS / (H < 16 ? H : 16); }

LLMP_API int llmp_latent_mma_supports(int rank, int rot, int page_size) {
    const size_t smem = sizeof(bf16) * (size_t)(LM_ROWS + LM_KEYS) * (rank + rot + 8);
    return rank > 0 && rank % 16 == 0 && rot >= 0 && rot % 16 == 0 && page_size > 0 && smem <= 200 * 1024;
}

// scratch: float32, segments * N * H * (rank + 2) entries when seg_keys > 0 (segments = ceil(longest context / seg_keys)).
LLMP_API int llmp_latent_attention_mma(const void* q_lat, long ql_t, long ql_h, const void* q_rot, long qr_t, long qr_h,
                                       const void* pages, const int* tables, int table_stride, const int* q_start, const int* ctx_len,
                                       const int* positions, const int* tile_req, const int* tile_tok0, int num_tiles, void* out,
                                       long o_t, long o_h, int N, int H, int rank, int rot, int page_size, float scale, int seg_keys,
                                       int segments, float* scratch, const float* sink, cudaStream_t stream) {
    if (N <= 0 || num_tiles <= 0) return 0;
    LLMP_REQUIRE(llmp_latent_mma_supports(rank, rot, page_size), "latent_attention_mma: sizes rank=%d rot=%d are not served", rank, rot);
    LLMP_REQUIRE(ql_t % 8 == 0 && ql_h % 8 == 0 && qr_t % 8 == 0 && qr_h % 8 == 0 && o_t % 2 == 0 && o_h % 2 == 0 &&
                 (size_t)q_lat % 16 == 0 && (size_t)q_rot % 16 == 0 && (size_t)out % 4 == 0 && (size_t)pages % 16 == 0,
                 "latent_attention_mma: query rows must be 16-byte aligned");
    LLMP_REQUIRE(seg_keys == 0 || (seg_keys % LM_KEYS == 0 && segments > 0 && segments <= 65535 && scratch != nullptr),
                 "latent_attention_mma: segments of %d keys", seg_keys);
    LatentMmaParams p;
    p.q_lat = (const bf16*)q_lat; p.ql_t = ql_t; p.ql_h = ql_h;
    p.q_rot = (const bf16*)q_rot; p.qr_t = qr_t; p.qr_h = qr_h;
    p.out = (bf16*)out; p.o_t = o_t; p.o_h = o_h;
    p.pages = (const bf16*)pages; p.tables = tables; p.table_stride = table_stride;
    p.q_start = q_start; p.ctx_len = ctx_len; p.tile_req = tile_req; p.tile_tok0 = tile_tok0;
    p.N = N; p.H = H; p.rank = rank; p.rot = rot; p.page_size = page_size;
    p.hpc = H < 16 ? H : 16;
    p.tokens_per_cta = LM_ROWS / p.hpc;
    p.head_chunks = (H + p.hpc - 1) / p.hpc;
    p.num_tiles = num_tiles;
    const int vchunk = rank > 128 ? 256 : 128;
    p.v_chunks = (rank + vchunk - 1) / vchunk;
    p.seg_keys = seg_keys;
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)segments * N * H * rank : nullptr;
    p.scale = scale;
    p.sink = sink;
    LLMP_REQUIRE((long)num_tiles * p.head_chunks < (1L << 31) && p.v_chunks <= 65535, "latent_attention_mma: too many tiles");
    size_t smem = sizeof(bf16) * (size_t)(LM_ROWS + LM_KEYS) * (rank + rot + 8);
    const size_t meet = sizeof(float) * 4 * 32 * (size_t)(vchunk / 2 + 4);       // where the halves of a row group meet
    if (smem < meet) smem = meet;
    dim3 grid((unsigned)(num_tiles * p.head_chunks), p.v_chunks, seg_keys > 0 ? segments : 1);
    if (vchunk == 128) {
        LLMP_ALLOW_SMEM(latent_attention_mma_kernel<128>, smem);
        latent_attention_mma_kernel<128><<<grid, LM_THREADS, smem, stream>>>(p);
    } else {
        LLMP_ALLOW_SMEM(latent_attention_mma_kernel<256>, smem);
        latent_attention_mma_kernel<256><<<grid, LM_THREADS, smem, stream>>>(p);
    }
    if (seg_keys > 0)
        latent_merge_kernel<<<dim3(N, H), 128, 0, stream>>>(p.part_o, p.part_ml, positions, (bf16*)out, o_t, o_h, N, H, rank, seg_keys, sink);
    return llmp_check_launch("latent_attention_mma");
}
