// The capped window attention of capped_attention.cu over bfloat16 pages on the tensor cores (mma.sync m16n8k16, float32
// accumulate), with the same arguments and result, for key sizes d and value sizes dv of 16, 32, 64 or 128.
//
// A block takes one tile of query rows of one request and one key/value head: CM_ROWS = 64 rows, a row being (token,
// query head of the group) with the head running fastest, so the key/value tile it streams serves all query heads of
// the group. A cached row is [key | value]. Each of the four warps owns 16 rows and keeps their running softmax and output
// in registers. Keys are walked in tiles of 64 aligned to key 0 (the same operations for a row however the prompt was
// cut): first the tiles of the kept first tokens that lie before the window of the tile's first token, then from that
// window's first key to the last token's own; half tiles that no row of a warp sees are skipped, rows of pages that
// are gone are never read. Per score: scale, cap (tanh by the special-function unit), the head's slope times the
// distance, the mask; the softmax runs in units of log2 and starts from the sink (a key of that score without a value).
// The gate, sigmoid of a float32 row, is applied as the output is stored.
//
// The key/value tiles go through a ring of buffers: two for prompts (the copy of the next tile runs under the products of
// this one, and two blocks share an SM), four for steps of single tokens.
//
// Steps of one token a request (`split`): the tile's rows fit one warp's 16, and the four warps share every tile instead:
// warp w takes keys 16 w to 16 w + 15 of it and keeps sums of its own; at the end the four meet in shared memory and warp 0
// adds them in their order and stores. (With whole half tiles dealt out in turn, two warps worked while two waited at the
// tile's barrier: 2.0 against 1.5 microseconds a tile at keys and values of 128.)
#include "common.cuh"

#include <type_traits>

#define CM_ROWS 64
#define CM_KEYS 64
#define CM_THREADS 128

namespace {

struct CappedMmaParams {
    const bf16* q;
    bf16* out;
    const bf16* pages;
    const int* block_tables;
    const int* q_start;
    const int* ctx_len;
    const int* tile_req;
    const int* tile_tok0;
    const float* slopes;             // [heads] or null
    const float* sink;               // [heads] or null
    const float* gate;               // float32 [tokens, heads dv] or null
    long q_stride, out_stride, gate_stride;
    int table_stride;
    int nq, nkv, page_size, window, keep;
    int heads_per_cta, tokens_per_cta, head_chunks, num_tiles, split, stages;
    float scale, cap;
};

__device__ __forceinline__ void cm_cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void cm_ldmatrix_x4(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void cm_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem_ptr) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void cm_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x and tanh by the special-function unit (the probabilities are rounded to bfloat16 anyway)
__device__ __forceinline__ float cm_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float cm_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ unsigned cm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

constexpr float CM_LOG2E = 1.4426950408889634f;

template <int D16, int V16>
__global__ void __launch_bounds__(CM_THREADS, 2) capped_attention_mma_kernel(const CappedMmaParams p) {
    extern __shared__ __align__(16) unsigned char cm_smem[];
    pdl_wait();                                    // what the kernels before wrote is complete
    pdl_trigger();
    constexpr int D = D16 * 16, DV = V16 * 16;
    constexpr int RS = D + DV;                                   // a cached row
    constexpr int QSTRIDE = D + 8, KSTRIDE = RS + 8;             // padded rows: conflict-free ldmatrix
    bf16* Qs = reinterpret_cast<bf16*>(cm_smem);                 // [CM_ROWS][QSTRIDE]
    bf16* ring = Qs + CM_ROWS * QSTRIDE;                         // [stages][CM_KEYS][KSTRIDE]
    constexpr int STAGE_ELEMS = CM_KEYS * KSTRIDE;
    __shared__ long long key_off[4][CM_KEYS];
    const bool split = p.split != 0;                             // four warps on the 16 rows of a one-token tile

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rw = split ? 0 : warp;                             // which 16 rows of the tile this warp works on
    const int per_tile = p.nkv * p.head_chunks;
    const int tile = p.num_tiles - 1 - (int)(blockIdx.x / (unsigned)per_tile);      // long tiles first
    const int in_tile = (int)(blockIdx.x % (unsigned)per_tile);
    const int r = p.tile_req[tile];
    const int tok0 = p.tile_tok0[tile];
    const int kvh = in_tile / p.head_chunks, chunk = in_tile % p.head_chunks;
    const int G = p.nq / p.nkv;
    const int hpc = p.heads_per_cta;
    const int head0 = chunk * hpc;
    int heads = G - head0;
    if (heads > hpc) heads = hpc;
    const int q_begin = p.q_start[r];
    const int q_len = p.q_start[r + 1] - q_begin;
    const int ctx = p.ctx_len[r];
    const int pos0 = ctx - q_len;
    int ntok = q_len - tok0;
    if (ntok > p.tokens_per_cta) ntok = p.tokens_per_cta;
    const int* table = p.block_tables + (size_t)r * p.table_stride;

    // keys this block needs: the kept first tokens before its first token's window, then from that window's start to
    // the position of its last token
    const int hi = pos0 + tok0 + ntok - 1;                       // last key (inclusive)
    int lo = 0;
    if (p.window > 0) {
        lo = pos0 + tok0 - p.window + 1;
        if (lo < 0) lo = 0;
    }
    const int keep_end = p.keep < lo ? p.keep : lo;              // kept keys that lie before the window: [0, keep_end)
    const int tile_lo = (lo / CM_KEYS) * CM_KEYS;
    // the walk: tiles 0, 64, .. below keep_end, then tile_lo, tile_lo + 64, .. up to hi
    auto next_tile = [&](int j0) {
        const int n = j0 + CM_KEYS;
        return (n >= keep_end && n < tile_lo) ? tile_lo : n;
    };
    const int first_tile = keep_end > 0 ? 0 : tile_lo;

    // query rows: row = token * hpc + head
    constexpr int QVEC = D / 8;
    for (int e = tid; e < CM_ROWS * QVEC; e += CM_THREADS) {
        const int row = e / QVEC, c = (e % QVEC) * 8;
        const int tl = row / hpc, h = row % hpc;
        const bool ok = tl < ntok && h < heads;
        const bf16* src = ok ? p.q + (size_t)(q_begin + tok0 + tl) * p.q_stride + (size_t)(kvh * G + head0 + h) * D + c : p.q;
        cm_cp_async_16(Qs + row * QSTRIDE + c, src, ok);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");

    constexpr int KVEC = RS / 8;
    // A tile's copy has two parts: where its 64 rows lie (a look into the block table by the first 64 threads, whose
    // answer travels while the tile before is worked on and is written to shared memory before that round's last
    // barrier), and the copy itself, which reads those places a round later.
    auto plan_tile = [&](int j0) -> long long {
        long long off = -1;
        if (tid < CM_KEYS) {
            const int j = j0 + tid;
            if (j <= hi && (j >= lo || j < keep_end)) {
                const int page = table[j / p.page_size];
                if (page >= 0) off = (long long)(((size_t)page * p.nkv + kvh) * p.page_size + (j % p.page_size)) * RS;
            }
        }
        return off;
    };
    auto copy_tile = [&](int buf) {
        bf16* dst = ring + (size_t)buf * STAGE_ELEMS;
        for (int e = tid; e < CM_KEYS * KVEC; e += CM_THREADS) {
            const int key = e / KVEC, c = (e % KVEC) * 8;
            const long long off = key_off[buf][key];
            const bool ok = off >= 0;
            cm_cp_async_16(dst + key * KSTRIDE + c, ok ? p.pages + off + c : p.pages, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    // positions, slopes and sinks of this lane's two rows (row g and row g + 8 of the warp's 16); position -1: no such row
    int row_pos[2];
    float slope2[2], m_run[2], l_run[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        const int row = rw * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        const bool exists = tl < ntok && h < heads;
        row_pos[h2] = exists ? pos0 + tok0 + tl : -1;
        const int head = kvh * G + head0 + (exists ? h : 0);
        slope2[h2] = p.slopes ? p.slopes[head] * CM_LOG2E : 0.f;
        m_run[h2] = -INFINITY;
        l_run[h2] = 0.f;
        if (p.sink && exists && (!split || warp == 0)) {
            m_run[h2] = p.sink[head] * CM_LOG2E;
            l_run[h2] = t == 0 ? 1.f : 0.f;                     // the lanes of a quad add their sums at the end
        }
    }

    float o[2 * V16][4];
#pragma unroll
    for (int i = 0; i < 2 * V16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const float scale_log2 = p.scale * CM_LOG2E;
    const float cap_log2 = p.cap * CM_LOG2E, inv_cap = p.cap > 0.f ? p.scale / p.cap : 0.f;
    const int warp_first_tok = (rw * 16) / hpc;
    const int warp_last_tok = (rw * 16 + 15) / hpc;
    const bool warp_has_rows = warp_first_tok < ntok;            // a warp without rows only helps with the copies
    const int warp_hi_pos = pos0 + tok0 + (warp_last_tok < ntok ? warp_last_tok : ntok - 1);
    const int warp_lo_pos = pos0 + tok0 + (warp_first_tok < ntok ? warp_first_tok : ntok - 1);
    const bf16* Qw = Qs + (size_t)(rw * 16 + (lane & 15)) * QSTRIDE + (lane >> 4) * 8;     // this lane's ldmatrix row of Q
    // the ring: stages - 1 tiles are under way beside the one at work (every round commits one group of copies, an empty
    // one once the walk's tiles are all asked for, so that the count of groups to wait for stays the same)
    const int stages = p.stages;
    int j_plan = first_tile;                                     // the next tile to look up
    for (int s0 = 0; s0 < stages; ++s0) {                        // the first tiles' places: all lookups in flight together
        if (tid < CM_KEYS) key_off[s0][tid] = j_plan <= hi ? plan_tile(j_plan) : -1;
        if (j_plan <= hi) j_plan = next_tile(j_plan);
    }
    __syncthreads();
    int j_issue = first_tile, buf_issue = 0;
    for (int s0 = 0; s0 < stages - 1; ++s0) {
        if (j_issue <= hi) {
            copy_tile(buf_issue);
            j_issue = next_tile(j_issue);
        } else {
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        buf_issue = buf_issue + 1 == stages ? 0 : buf_issue + 1;
    }
    int buf = 0;
    for (int j0 = first_tile; j0 <= hi; j0 = next_tile(j0)) {
        if (j_issue <= hi) {
            copy_tile(buf_issue);                                // its buffer was read last in the round before: see the barrier below
            j_issue = next_tile(j_issue);
        } else {
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        }
        // the places of the tile that this round's buffer takes next: asked for now, written down at the round's end
        const bool planning = j_plan <= hi;
        const long long off_next = planning ? plan_tile(j_plan) : -1;
        if (planning) j_plan = next_tile(j_plan);
        buf_issue = buf_issue + 1 == stages ? 0 : buf_issue + 1;
        if (stages == 4) asm volatile("cp.async.wait_group 3;\n" ::: "memory");
        else asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        __syncthreads();
        const bf16* KVs = ring + (size_t)buf * STAGE_ELEMS;
        // the part of a tile that starts at its key `kbase` and has NB blocks of 8 keys: scores, softmax step, values
        auto part = [&](auto nbc, const int kbase) {
            constexpr int NB = decltype(nbc)::value;
            const int jh = j0 + kbase;
            if (jh > warp_hi_pos) return;                        // every row of this warp lies before these keys
            const bool kept = jh < p.keep;                       // kept first tokens stay in sight of every row
            if (!kept && p.window > 0 && jh + NB * 8 - 1 < warp_lo_pos - p.window + 1) return;    // or sees none of them any more
            float s[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < D16; ++ks) {
                unsigned qa[4];
                cm_ldmatrix_x4(qa, Qw + ks * 16);
#pragma unroll
                for (int nb = 0; nb < NB; nb += 2) {
                    unsigned kf[4];
                    cm_ldmatrix_x4(kf, KVs + (size_t)(kbase + (nb + (lane >> 4)) * 8 + (lane & 7)) * KSTRIDE + ks * 16 +
                                           ((lane >> 3) & 1) * 8);
                    cm_mma(s[nb], qa, kf[0], kf[1]);
                    cm_mma(s[nb + 1], qa, kf[2], kf[3]);
                }
            }
            // scores in units of log2: scale (and cap), the distance bias, the mask
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int j = jh + nb * 8 + 2 * t + (c & 1);
                    const int pos = row_pos[c >> 1];
                    float v = p.cap > 0.f ? cap_log2 * cm_tanh(s[nb][c] * inv_cap) : s[nb][c] * scale_log2;
                    v = fmaf(-slope2[c >> 1], (float)(pos - j), v);
                    const bool ok = j <= pos && (p.window <= 0 || j >= pos - p.window + 1 || j < p.keep);
                    v = ok ? v : -INFINITY;
                    s[nb][c] = v;
                    mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
            }
            float alpha[2], m_use[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 1));
                mx[h2] = fmaxf(mx[h2], __shfl_xor_sync(0xffffffffu, mx[h2], 2));
                const float m_new = fmaxf(m_run[h2], mx[h2]);
                alpha[h2] = (m_new > -INFINITY) ? cm_ex2(m_run[h2] - m_new) : 1.f;
                m_run[h2] = m_new;
                m_use[h2] = (m_new > -INFINITY) ? m_new : 0.f;          // a row without any key keeps p = 2^(-inf) = 0
            }
            float sum[2] = {0.f, 0.f};
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float pr = cm_ex2(s[nb][c] - m_use[c >> 1]);
                    s[nb][c] = pr;
                    sum[c >> 1] += pr;
                }
            }
            l_run[0] = l_run[0] * alpha[0] + sum[0];
            l_run[1] = l_run[1] * alpha[1] + sum[1];
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int i = 0; i < 2 * V16; ++i) {
                    o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
                }
            }
            // O += P V, 16 keys per step
#pragma unroll
            for (int kk = 0; kk < NB / 2; ++kk) {
                unsigned pa[4];
                pa[0] = cm_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = cm_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = cm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = cm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int nb2 = 0; nb2 < V16; ++nb2) {
                    unsigned v[4];
                    cm_ldmatrix_x4_trans(v, KVs + (size_t)(kbase + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * KSTRIDE + D +
                                                nb2 * 16 + (lane >> 4) * 8);
                    cm_mma(o[nb2 * 2], pa, v[0], v[1]);
                    cm_mma(o[nb2 * 2 + 1], pa, v[2], v[3]);
                }
            }
        };
        if (split) {
            part(std::integral_constant<int, 2>{}, warp * 16);  // a quarter of the tile's keys for each of the four warps
        } else if (warp_has_rows) {
            part(std::integral_constant<int, 4>{}, 0);
            part(std::integral_constant<int, 4>{}, 32);
        }
        if (tid < CM_KEYS) key_off[buf][tid] = off_next;         // this round's tile was copied long ago: its places make room
        __syncthreads();                                         // the tile's buffer may be overwritten now
        buf = buf + 1 == stages ? 0 : buf + 1;
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");       // the query copy, where no key tile followed it

#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 1);
        l_run[h2] += __shfl_xor_sync(0xffffffffu, l_run[h2], 2);
    }
    if (split) {
        // the four warps' sums of the same 16 rows meet: warps 1 to 3 leave theirs in shared memory (the query and key tiles
        // are no longer read), warp 0 adds them to its own in their order
        float* xo = reinterpret_cast<float*>(cm_smem);           // [3 warps][32 lanes][8 V16 + 4]
        constexpr int PER_LANE = 8 * V16 + 4;
        __syncthreads();
        if (warp > 0) {
            float* mine = xo + ((size_t)(warp - 1) * 32 + lane) * PER_LANE;
#pragma unroll
            for (int i = 0; i < 2 * V16; ++i) *reinterpret_cast<float4*>(mine + 4 * i) = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
            *reinterpret_cast<float4*>(mine + 8 * V16) = make_float4(m_run[0], m_run[1], l_run[0], l_run[1]);
        }
        __syncthreads();
        if (warp > 0) return;
        for (int w = 0; w < 3; ++w) {
            const float* theirs = xo + ((size_t)w * 32 + lane) * PER_LANE;
            const float4 ml = *reinterpret_cast<const float4*>(theirs + 8 * V16);
            const float om[2] = {ml.x, ml.y}, ol[2] = {ml.z, ml.w};
            float wa[2], wb[2];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const float m = fmaxf(m_run[h2], om[h2]);
                wa[h2] = (m_run[h2] > -INFINITY) ? cm_ex2(m_run[h2] - m) : 0.f;
                wb[h2] = (om[h2] > -INFINITY) ? cm_ex2(om[h2] - m) : 0.f;
                l_run[h2] = l_run[h2] * wa[h2] + ol[h2] * wb[h2];
                m_run[h2] = m;
            }
#pragma unroll
            for (int i = 0; i < 2 * V16; ++i) {
                const float4 x = *reinterpret_cast<const float4*>(theirs + 4 * i);
                o[i][0] = o[i][0] * wa[0] + x.x * wb[0];
                o[i][1] = o[i][1] * wa[0] + x.y * wb[0];
                o[i][2] = o[i][2] * wa[1] + x.z * wb[1];
                o[i][3] = o[i][3] * wa[1] + x.w * wb[1];
            }
        }
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
        if (row_pos[h2] < 0) continue;
        const int row = rw * 16 + g + 8 * h2;
        const int tl = row / hpc, h = row % hpc;
        const float inv = l_run[h2] > 0.f ? 1.f / l_run[h2] : 0.f;
        const size_t n = (size_t)(q_begin + tok0 + tl);
        const int col0 = (kvh * G + head0 + h) * DV + 2 * t;
        bf16* dst = p.out + n * p.out_stride + col0;
        const float* gate = p.gate ? p.gate + n * p.gate_stride + col0 : nullptr;
#pragma unroll
        for (int nb = 0; nb < 2 * V16; ++nb) {
            float a = o[nb][2 * h2] * inv, b = o[nb][2 * h2 + 1] * inv;
            if (gate) {
                const float2 gv = *reinterpret_cast<const float2*>(gate + nb * 8);
                a = a / (1.f + __expf(-gv.x));
                b = b / (1.f + __expf(-gv.y));
            }
            *reinterpret_cast<unsigned*>(dst + nb * 8) = cm_pack(a, b);
        }
    }
}

bool cm_size_served(int n) { return n == 16 || n == 32 || n == 64 || n == 128; }

template <int D16, int V16>
int launch_capped_mma(const CappedMmaParams& p, unsigned grid, cudaStream_t stream) {
    const size_t q_bytes = sizeof(bf16) * (size_t)CM_ROWS * (D16 * 16 + 8);
    const size_t stage = sizeof(bf16) * (size_t)CM_KEYS * (D16 * 16 + V16 * 16 + 8);
    // two buffers for prompts, so that two blocks share an SM; four for steps of single tokens, whose few blocks are each a
    // chain of copies that should be under way early
    CappedMmaParams q = p;
    q.stages = (p.split && q_bytes + 4 * stage <= 200 * 1024) ? 4 : 2;
    size_t smem = q_bytes + q.stages * stage;
    const size_t meet = sizeof(float) * 3 * 32 * (size_t)(8 * V16 + 4);          // where the warps of a one-token tile meet
    if (smem < meet) smem = meet;
    // the kernel also has 2 KB of static shared memory: ask for the larger limit as soon as the two together pass 48 KB
    LLMP_ALLOW_SMEM((capped_attention_mma_kernel<D16, V16>), smem + 4096);
    llmp_launch_dependent(capped_attention_mma_kernel<D16, V16>, dim3(grid), dim3(CM_THREADS), smem, stream, q);
    return 0;
}

}  // namespace

LLMP_API int llmp_capped_mma_supports(int d, int dv) { return cm_size_served(d) && cm_size_served(dv); }

// Query tokens per block for a group size: 64 rows of (token, head).
LLMP_API int llmp_capped_mma_tokens_per_tile(int nq, int nkv) {
    const int G = nq / nkv;
    const int hpc = G < 16 ? G : 16;
    return CM_ROWS / hpc;
}

LLMP_API int llmp_capped_attention_mma(const void* q, long q_stride, void* out, long out_stride, const void* pages,
                                       const int* block_tables, int table_stride, const int* q_start, const int* ctx_len,
                                       const int* tile_req, const int* tile_tok0, int num_tiles, const float* slopes, const float* sink,
                                       const float* gate, long gate_stride, int nq, int nkv, int d, int dv, int page_size, int window,
                                       int keep, float scale, float cap, int split, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    LLMP_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && llmp_capped_mma_supports(d, dv) && page_size > 0 && window >= 0 && keep >= 0,
                 "capped_attention_mma: sizes heads=%d kv_heads=%d dim=%d vdim=%d are not served", nq, nkv, d, dv);
    CappedMmaParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.pages = (const bf16*)pages; p.block_tables = block_tables;
    p.q_start = q_start; p.ctx_len = ctx_len; p.tile_req = tile_req; p.tile_tok0 = tile_tok0;
    p.slopes = slopes; p.sink = sink; p.gate = gate; p.gate_stride = gate_stride;
    p.q_stride = q_stride; p.out_stride = out_stride; p.table_stride = table_stride; p.nq = nq; p.nkv = nkv;
    p.page_size = page_size; p.window = window; p.keep = window > 0 ? keep : 0; p.scale = scale; p.cap = cap;
    const int G = nq / nkv;
    p.heads_per_cta = G < 16 ? G : 16;
    p.tokens_per_cta = CM_ROWS / p.heads_per_cta;
    p.head_chunks = (G + p.heads_per_cta - 1) / p.heads_per_cta;
    p.num_tiles = num_tiles;
    p.split = split ? 1 : 0;
    p.stages = 2;
    LLMP_REQUIRE((long)num_tiles * nkv * p.head_chunks < (1L << 31), "capped_attention_mma: too many tiles");
    LLMP_REQUIRE((q_stride % 8) == 0 && (out_stride % 2) == 0 && ((size_t)q % 16) == 0 && ((size_t)pages % 16) == 0 &&
                 ((size_t)out % 4) == 0 && (gate == nullptr || ((gate_stride % 2) == 0 && ((size_t)gate % 8) == 0)),
                 "capped_attention_mma: rows must be 16-byte aligned");
    const unsigned grid = (unsigned)(num_tiles * nkv * p.head_chunks);
    int rc = 1;
#define CM_V(DD, VV) case VV: rc = launch_capped_mma<DD, VV>(p, grid, stream); break;
#define CM_D(DD)                                                         \
    case DD:                                                             \
        switch (dv / 16) { CM_V(DD, 1) CM_V(DD, 2) CM_V(DD, 4) CM_V(DD, 8) } \
        break;
    switch (d / 16) { CM_D(1) CM_D(2) CM_D(4) CM_D(8) }
#undef CM_D
#undef CM_V
    if (rc) return rc;
    return llmp_check_launch("capped_attention_mma");
}
