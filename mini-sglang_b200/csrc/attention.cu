// Causal grouped-query attention over the paged cache, for prompt portions and single decoded
// tokens in one batch.
//
// Every request r of the step brings q_len[r] = q_start[r+1] - q_start[r] new tokens whose keys
// and values are already in the cache; kv_len[r] counts them too.  The query at offset j of
// request r sits at position kv_len[r] - q_len[r] + j and sees keys 0..position (or the last
// `window` of them).  Query head h reads kv head h / (n_q / n_kv).
//
// Cache layout (one K and one V array per layer): [page][kv head][slot in page][d]; the key at
// position i of request r lives in page block_table[r][i / P], slot i % P.
//
// Work is cut into (query tile, kv head [, head chunk], kv split).  A query tile packs
// (token, head-in-group) pairs as rows so that the heads of a group share the K/V they read.
// Key tiles are anchored at absolute positions (tile k = keys [k*KT, (k+1)*KT)); a request with
// nsplit[r] > 1 spreads its key tiles over that many blocks, which write unnormalised partial
// sums to scratch memory; msgl_attention_combine merges them in split order.
//
// Kernels:
//   attn_tc2_kernel / attn_tc_kernel   bfloat16, head size 128, query runs longer than a decode tile: tcgen05
//                               tensor cores with accumulators in tensor memory (attention_tc2.cuh, attention_tc.cuh)
//   attn_mma_kernel<D>          bfloat16, the same runs at other head sizes (16..256 in steps of 16): mma.sync
//                               m16n8k16, 64 rows per block, each warp owns 16 rows and walks all keys of a tile
//   attn_decode_t_kernel<D,...> bfloat16, short query runs (decode), head sizes in steps of 32: keys on the M
//                               dimension of the mma, K straight from global memory into registers, kv splits
//   attn_decode_even_kernel<D,...> the same arithmetic for a decode step whose keys the host has dealt out evenly over
//                               a fixed number of blocks per kv head (requests of very different lengths)
//   attn_decode_kernel<D,...>   the same for head sizes 16 mod 32: heads on the M dimension
//   attn_simt_kernel<T>         any head size up to 512, float32 arithmetic throughout; this is
//                               the true 32-bit path and the fallback for odd head sizes
//   attn_combine_kernel<T>      merge of the kv splits
// Scores, softmax and the accumulation are float32 in all of them.  In a step of single tokens the blocks take the
// requests in the order the step gives (`order`: longest first), the kv heads of one request in adjacent blocks.
#include "common.cuh"
#include <math.h>

#ifndef MSGL_HEAD_DIM
#define MSGL_HEAD_DIM 128
#endif
#ifndef MSGL_DEC_WARPS
#define MSGL_DEC_WARPS 4          // warps of the decode kernel
#endif
#ifndef MSGL_DEC_STAGES
#define MSGL_DEC_STAGES 2         // cp.async stages per warp of the decode kernel (measured best with the L2 prefetch)
#endif
#ifndef MSGL_DEC_PFV
#define MSGL_DEC_PFV 0            // 1: V is prefetched into L2 together with K
#endif
#ifndef MSGL_DEC_PFK
#define MSGL_DEC_PFK 2            // how many units ahead of its use K is prefetched into L2 (beyond the register load)
#endif

struct AttnParams {
    const void* q;            // [T, n_q, d]
    void* out;                // [T, n_q, d]
    const void* k_cache;
    const void* v_cache;
    const int* q_start;       // [B + 1]
    const int* kv_len;        // [B]
    const int* block_table;   // [B, bt_stride]
    const int* nsplit;        // [B] or null (1 everywhere)
    const int* order;         // [B] or null: with uniform_decode, the request that the i-th block along x takes
    const int* even;          // null, or the even cut of a uniform decode launch (attn_decode_even_kernel): [0] blocks in use,
                              // then start unit of every block [even_nb + 1], first request of every block [even_nb], first
                              // unit of every request [B + 1], first block of every request [B]
    int even_nb;              // blocks per (kv head, chunk of q heads) that the launch has
    float* part_o;            // [(split * T + token) * n_q + head][d]
    float* part_ml;           // [(split * T + token) * n_q + head][2]  (max in log2 units, sum)
    int B, T, n_q, n_kv, d, page_size, bt_stride, window, max_split;
    int page_shift;           // log2(page_size) when it is a power of two, else -1
    float scale;
    int qlen_min, qlen_max;   // this launch takes the requests with qlen_min <= q_len <= qlen_max
    int uniform_decode;       // every request has exactly one token: tile index == request index
};

// position -> (page index within the request, slot within the page)
__device__ __forceinline__ int page_index(const AttnParams& p, int key) {
    return p.page_shift >= 0 ? (key >> p.page_shift) : (key / p.page_size);
}
__device__ __forceinline__ int page_slot(const AttnParams& p, int key) {
    return p.page_shift >= 0 ? (key & (p.page_size - 1)) : (key % p.page_size);
}

struct TileInfo {
    int req, t0, n_tok;       // request, first token of the tile within the request, tokens in the tile
    int q_len, kv_len, q_base;
};

// Map blockIdx.x to (request, tile) by walking the per-request tile counts with one warp.
// tile_idx / n_tile_idx: this block's index among the launch's query tiles (default: blockIdx.x of gridDim.x)
__device__ __forceinline__ bool find_tile(const AttnParams& p, int tile_tokens, TileInfo& ti, int* sh /* >= 4 ints */,
                                          int tile_idx = -1, int n_tile_idx = 0) {
    if (tile_idx < 0) { tile_idx = (int)blockIdx.x; n_tile_idx = (int)gridDim.x; }
    if (p.uniform_decode) {
        // blocks are handed to the SMs in index order: the host (or the kernel that made the step's fields) lists
        // the requests by falling number of keys, so that the longest start first and the shortest fill the end
        if (tile_idx >= p.B) return false;
        const int r = p.order ? p.order[tile_idx] : tile_idx;
        if (r < 0 || r >= p.B) return false;
        ti.req = r; ti.t0 = 0; ti.n_tok = 1; ti.q_len = 1; ti.kv_len = p.kv_len[r]; ti.q_base = p.q_start[r];
        return true;
    }
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int base = 0, found_req = -1, found_t0 = 0;
        for (int r0 = 0; r0 < p.B && found_req < 0; r0 += 32) {
            const int r = r0 + lane;
            int nt = 0;
            if (r < p.B) {
                const int ql = p.q_start[r + 1] - p.q_start[r];
                if (ql >= p.qlen_min && ql <= p.qlen_max) nt = (ql + tile_tokens - 1) / tile_tokens;
            }
            int inc = nt;  // inclusive scan
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            // heaviest tiles first: with a causal mask the last tiles of a request walk the most keys, and
            // blocks are handed out in index order
            const int target = (n_tile_idx - 1 - tile_idx) - base;
            const unsigned hit = __ballot_sync(0xffffffffu, target < inc);
            if (hit) {
                const int src = __ffs(hit) - 1;
                const int inc_src = __shfl_sync(0xffffffffu, inc, src);
                const int nt_src = __shfl_sync(0xffffffffu, nt, src);
                found_req = r0 + src;
                found_t0 = (target - (inc_src - nt_src)) * tile_tokens;
            }
            base += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) { sh[0] = found_req; sh[1] = found_t0; }
    }
    __syncthreads();
    ti.req = sh[0];
    ti.t0 = sh[1];
    if (ti.req < 0) return false;
    ti.q_base = p.q_start[ti.req];
    ti.q_len = p.q_start[ti.req + 1] - ti.q_base;
    ti.kv_len = p.kv_len[ti.req];
    ti.n_tok = min(tile_tokens, ti.q_len - ti.t0);
    return true;
}

// This block's place in the launch: (index among the query tiles, index along y = kv head and chunk of q heads).  With an
// order given (uniform decode) consecutive blocks take the kv heads of one request, so that across the whole launch the
// requests are walked in that order: the longest first.
__device__ __forceinline__ void block_place(const AttnParams& p, int& tile_idx, int& y) {
    if (p.uniform_decode && p.order) {
        const int lin = (int)(blockIdx.y * gridDim.x + blockIdx.x);
        tile_idx = lin / (int)gridDim.y;
        y = lin - tile_idx * (int)gridDim.y;
    } else {
        tile_idx = (int)blockIdx.x;
        y = (int)blockIdx.y;
    }
}

// Which key tiles a block walks: the tiles that hold keys [k_lo, p_max], cut into ns splits.
__device__ __forceinline__ void key_tile_range(const AttnParams& p, const TileInfo& ti, int KT, int split, int ns,
                                               int& p_min, int& p_max, int& kt_begin, int& kt_end) {
    p_min = ti.kv_len - ti.q_len + ti.t0;
    p_max = p_min + ti.n_tok - 1;
    int k_lo = 0;
    if (p.window > 0) k_lo = max(0, p_min - p.window + 1);
    const int first = k_lo / KT, last = p_max / KT;
    const int n_t = last - first + 1;
    const int per = (n_t + ns - 1) / ns;
    kt_begin = first + split * per;
    kt_end = min(first + (split + 1) * per, last + 1);
    if (kt_begin > kt_end) kt_begin = kt_end;
}

// ---------------------------------------------------------------------------------------
// bfloat16 tensor-core kernel
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
// the same with 32-bit shared-memory addresses, so that the hot loops add compile-time offsets to one
// base register instead of converting a generic pointer for every access
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_u32(unsigned s, const void* gmem, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(n));
}
__device__ __forceinline__ void ldmatrix_x4_u32(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans_u32(unsigned (&r)[4], unsigned s) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// 2^x by the special-function unit (relative error about 2^-22; -inf gives 0), for the bfloat16 kernels
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

constexpr int MMA_KT = 64;        // keys per tile
constexpr int MMA_WARPS = 4;
constexpr int MMA_THREADS = MMA_WARPS * 32;

template <int D>
__global__ void __launch_bounds__(MMA_THREADS) attn_mma_kernel(const AttnParams p) {
    constexpr int R = 64;                           // rows per block
    constexpr int LDS = D + 8;                      // padded row of a shared-memory tile (elements)
    constexpr int WK = 64;                          // keys of a tile that one warp handles
    constexpr int NKB = WK / 8;                     // 8-key blocks per warp
    constexpr int NDB = D / 8;                      // 8-wide output column blocks
    constexpr int CH = D / 8;                       // 16-byte chunks per row

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* KVs = Qs + R * LDS;              // [stage][K|V][MMA_KT][LDS]
    __shared__ int sh_tile[4];

    const int G = p.n_q / p.n_kv;
    const int Gc = G <= R ? G : R;
    const int n_chunks = G <= R ? 1 : (G + R - 1) / R;
    const int QT = G <= R ? R / G : 1;
    int tile_idx, by;
    block_place(p, tile_idx, by);
    const int kvh = by / n_chunks;
    const int chunk = by - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, QT, ti, sh_tile, tile_idx, (int)gridDim.x)) return;
    const int ns = p.nsplit ? min(max(p.nsplit[ti.req], 1), p.max_split) : 1;
    const int split = blockIdx.z;
    if (split >= ns) return;

    int p_min, p_max, kt_begin, kt_end;
    key_tile_range(p, ti, MMA_KT, split, ns, p_min, p_max, kt_begin, kt_end);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
    const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;

    // ---- Q rows into shared memory (zero rows where the tile has no token/head)
    for (int idx = tid; idx < R * CH; idx += MMA_THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const int tl = r / Gc, hl = r - tl * Gc;
        const int hg = chunk * R + hl;
        const bool valid = tl < ti.n_tok && hg < G && tl < QT;
        const size_t tok = (size_t)(ti.q_base + ti.t0 + (valid ? tl : 0));
        const __nv_bfloat16* src = qg + (tok * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * D + c * 8;
        cp_async16(Qs + r * LDS + c * 8, valid ? (const void*)src : (const void*)qg, valid);
    }

    // a thread copies half a row of K and of V per tile: row tid / 2, 16-byte chunks 2j + (tid & 1);
    // the row's page is looked up once per tile, one tile ahead of the copy that needs it
    const int ld_row = tid >> 1, ld_half = tid & 1;
    auto tile_page = [&](int kt) -> int {
        const int key = kt * MMA_KT + ld_row;
        return (kt < kt_end && key <= p_max) ? bt[page_index(p, key)] : -1;
    };
    constexpr unsigned STAGE_BYTES = 2u * MMA_KT * LDS * 2u, TILE_BYTES = MMA_KT * LDS * 2u;
    const unsigned q_s = smem_u32(Qs), kv_s = smem_u32(KVs);
    const unsigned ld_dst = kv_s + (unsigned)(ld_row * LDS + ld_half * 8) * 2u;
    auto load_kv = [&](int stage, int kt, int pg) {
        const unsigned ks = ld_dst + (unsigned)stage * STAGE_BYTES, vs = ks + TILE_BYTES;
        const int key = kt * MMA_KT + ld_row;
        const bool valid = pg >= 0;
        size_t off = 0;
        if (valid) off = (((size_t)pg * p.n_kv + kvh) * p.page_size + page_slot(p, key)) * D;
        const __nv_bfloat16* ksrc = kc + off + ld_half * 8;
        const __nv_bfloat16* vsrc = vc + off + ld_half * 8;
#pragma unroll
        for (int j = 0; j < CH / 2; ++j) {
            cp_async16_u32(ks + j * 32, ksrc + j * 16, valid);
            cp_async16_u32(vs + j * 32, vsrc + j * 16, valid);
        }
    };

    // per-thread rows: g = lane / 4 (and g + 8) of this warp's 16 rows
    const int row_base = warp * 16;
    const int key_base = 0;
    const int r_lo = row_base + (lane >> 2), r_hi = r_lo + 8;
    const int pos_lo = p_min + r_lo / Gc, pos_hi = p_min + r_hi / Gc;   // position of each row's query
    const float sc = p.scale * 1.4426950408889634f;                     // scores in log2 units
    // per-lane parts of the ldmatrix addresses (bytes)
    const unsigned q_a = q_s + (unsigned)((row_base + (lane & 15)) * LDS + (lane >> 4) * 8) * 2u;
    const unsigned k_lane = (unsigned)((key_base + (lane & 7) + ((lane >> 4) & 1) * 8) * LDS + ((lane >> 3) & 1) * 8) * 2u;
    const unsigned v_lane = (unsigned)((key_base + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + ((lane >> 4) & 1) * 8) * 2u;

    float o[NDB][4];
#pragma unroll
    for (int i = 0; i < NDB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    const int n_tiles = kt_end - kt_begin;
    if (n_tiles > 0) load_kv(0, kt_begin, tile_page(kt_begin));
    cp_async_commit();
    int pg_next = tile_page(kt_begin + 1);

    for (int it = 0; it < n_tiles; ++it) {
        const int kt = kt_begin + it;
        if (it + 1 < n_tiles) {
            load_kv((it + 1) & 1, kt + 1, pg_next);
            cp_async_commit();
            pg_next = tile_page(kt + 2);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const unsigned ks_a = kv_s + (unsigned)(it & 1) * STAGE_BYTES + k_lane, vs_a = ks_a - k_lane + TILE_BYTES + v_lane;

        // ---- S = Q K^T
        float s[NKB][4];
#pragma unroll
        for (int i = 0; i < NKB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            unsigned a[4];
            ldmatrix_x4_u32(a, q_a + kk * 32);
#pragma unroll
            for (int nb2 = 0; nb2 < NKB / 2; ++nb2) {
                unsigned b[4];
                ldmatrix_x4_u32(b, ks_a + (unsigned)(nb2 * 16 * LDS + kk * 16) * 2u);
                mma_bf16_16816(s[2 * nb2], a, b[0], b[1]);
                mma_bf16_16816(s[2 * nb2 + 1], a, b[2], b[3]);
            }
        }

        // ---- scale, mask, online softmax
        const int key0 = kt * MMA_KT + key_base;
        const bool need_mask = (kt * MMA_KT + MMA_KT - 1 > p_min) ||
                               (p.window > 0 && kt * MMA_KT <= p_max - p.window);
        // raw scores stay unscaled: the scale is folded into the exponent, 2^(s * sc - m)
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < NKB; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nb][e];
                if (need_mask) {
                    const int key = key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = (e < 2) ? pos_lo : pos_hi;
                    bool ok = key <= pos;
                    if (p.window > 0) ok = ok && (key > pos - p.window);
                    if (!ok) v = -INFINITY;
                    s[nb][e] = v;
                }
                if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo * sc), mn_hi = fmaxf(m_hi, mx_hi * sc);       // -inf * sc = -inf (sc > 0)
        const float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
        const float al_lo = fast_exp2(m_lo - mu_lo), al_hi = fast_exp2(m_hi - mu_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        l_lo *= al_lo; l_hi *= al_hi;
#pragma unroll
        for (int nb = 0; nb < NKB; ++nb) {
            s[nb][0] = fast_exp2(fmaf(s[nb][0], sc, -mu_lo)); s[nb][1] = fast_exp2(fmaf(s[nb][1], sc, -mu_lo));
            s[nb][2] = fast_exp2(fmaf(s[nb][2], sc, -mu_hi)); s[nb][3] = fast_exp2(fmaf(s[nb][3], sc, -mu_hi));
            l_lo += s[nb][0] + s[nb][1];
            l_hi += s[nb][2] + s[nb][3];
        }
        if (__any_sync(0xffffffffu, al_lo != 1.f || al_hi != 1.f)) {      // the running maxima rarely move after the first tiles
#pragma unroll
            for (int i = 0; i < NDB; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
        }

        // ---- O += P V
#pragma unroll
        for (int j = 0; j < NKB / 2; ++j) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
            a[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
            a[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
            a[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
            for (int nd2 = 0; nd2 < D / 16; ++nd2) {
                unsigned b[4];
                ldmatrix_x4_trans_u32(b, vs_a + (unsigned)(j * 16 * LDS + nd2 * 16) * 2u);
                mma_bf16_16816(o[2 * nd2], a, b[0], b[1]);
                mma_bf16_16816(o[2 * nd2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    // row sums over the four threads that share a row
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(p.out);
    const bool direct = ns == 1;

    {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = half ? r_hi : r_lo;
            const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * R + hl;
            if (!(tl < ti.n_tok && hg < G && tl < QT)) continue;
            const size_t tok = (size_t)(ti.q_base + ti.t0 + tl);
            const int head = kvh * G + hg;
            const float l = half ? l_hi : l_lo, m = half ? m_hi : m_lo;
            if (direct) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16* dst = og + (tok * p.n_q + head) * D;
#pragma unroll
                for (int nd = 0; nd < NDB; ++nd) {
                    const int col = nd * 8 + (lane & 3) * 2;
                    *reinterpret_cast<__nv_bfloat162*>(dst + col) =
                        __floats2bfloat162_rn(o[nd][half * 2] * inv, o[nd][half * 2 + 1] * inv);
                }
            } else {
                const size_t prow = ((size_t)split * p.T + tok) * p.n_q + head;
                float* dst = p.part_o + prow * D;
#pragma unroll
                for (int nd = 0; nd < NDB; ++nd) {
                    const int col = nd * 8 + (lane & 3) * 2;
                    *reinterpret_cast<float2*>(dst + col) = make_float2(o[nd][half * 2], o[nd][half * 2 + 1]);
                }
                if ((lane & 3) == 0) { p.part_ml[prow * 2] = m; p.part_ml[prow * 2 + 1] = l; }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// bfloat16 decode kernel: 16 rows per block (the heads of one group, one or a few tokens), the
// block's keys dealt out to NW warps in units of 16.  Every warp streams its own units through a
// private ring of ST shared-memory stages with cp.async and never waits for another warp until
// the merge at the end, so loads stay in flight while other warps compute.
// ---------------------------------------------------------------------------------------
constexpr int DEC_WT = 16;        // keys per warp unit
#ifndef MSGL_DEC_LAZY
#define MSGL_DEC_LAZY 8
#endif
constexpr float DEC_LAZY = (float)MSGL_DEC_LAZY;   // log2 of how far a score may lie above its column's reference before the reference moves (decode_t_run)

template <int D, int NW, int ST>
__global__ void __launch_bounds__(NW * 32) attn_decode_kernel(const AttnParams p) {
    constexpr int R = 16;
    constexpr int LDS = D + 8;
    constexpr int NDB = D / 8;
    constexpr int CH = D / 8;                       // 16-byte chunks per row
    constexpr int THREADS = NW * 32;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);              // [16][LDS]
    __nv_bfloat16* ring = Qs + R * LDS;                                          // [NW][ST][K|V][16][LDS]
    __shared__ int sh_tile[4];

    const int G = p.n_q / p.n_kv;
    const int Gc = G <= R ? G : R;
    const int n_chunks = G <= R ? 1 : (G + R - 1) / R;
    const int QT = G <= R ? R / G : 1;
    int tile_idx, by;
    block_place(p, tile_idx, by);
    const int kvh = by / n_chunks;
    const int chunk = by - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, QT, ti, sh_tile, tile_idx, (int)gridDim.x)) return;
    const int ns = p.nsplit ? min(max(p.nsplit[ti.req], 1), p.max_split) : 1;
    const int split = blockIdx.z;
    if (split >= ns) return;

    int p_min, p_max, kt_begin, kt_end;
    key_tile_range(p, ti, MMA_KT, split, ns, p_min, p_max, kt_begin, kt_end);
    const int u_begin = kt_begin * (MMA_KT / DEC_WT);
    const int u_end = min(kt_end * (MMA_KT / DEC_WT), p_max / DEC_WT + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
    const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;

    for (int idx = tid; idx < R * CH; idx += THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const int tl = r / Gc, hl = r - tl * Gc;
        const int hg = chunk * R + hl;
        const bool valid = tl < ti.n_tok && hg < G && tl < QT;
        const size_t tok = (size_t)(ti.q_base + ti.t0 + (valid ? tl : 0));
        const __nv_bfloat16* src = qg + (tok * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * D + c * 8;
        cp_async16(Qs + r * LDS + c * 8, valid ? (const void*)src : (const void*)qg, valid);
    }
    cp_async_commit();

    // this warp's units: u_begin + warp, + NW, ...
    const int n_my = (u_end - u_begin > warp) ? (u_end - u_begin - warp + NW - 1) / NW : 0;
    __nv_bfloat16* my_ring = ring + (size_t)warp * ST * 2 * DEC_WT * LDS;
    const int l_key = lane >> 1, l_half = lane & 1;

    // Page of this lane's key in unit i of this warp, or -1 past the last key.  The lookup is a
    // dependent global load, so it is issued one iteration before the copy that needs it.
    auto unit_page = [&](int i) -> int {
        const int key = (u_begin + warp + i * NW) * DEC_WT + l_key;
        return (i < n_my && key <= p_max) ? bt[page_index(p, key)] : -1;
    };
    auto load_unit = [&](int i, int pg) {      // unit i of this warp into stage i % ST
        __nv_bfloat16* Ks = my_ring + (size_t)(i % ST) * 2 * DEC_WT * LDS;
        __nv_bfloat16* Vs = Ks + DEC_WT * LDS;
        const int key = (u_begin + warp + i * NW) * DEC_WT + l_key;
        const bool valid = pg >= 0;
        size_t off = 0;
        if (valid) off = (((size_t)pg * p.n_kv + kvh) * p.page_size + page_slot(p, key)) * D;
#pragma unroll
        for (int j = 0; j < CH / 2; ++j) {
            const int c = l_half * (CH / 2) + j;
            cp_async16(Ks + l_key * LDS + c * 8, kc + off + c * 8, valid);
            cp_async16(Vs + l_key * LDS + c * 8, vc + off + c * 8, valid);
        }
    };

    int pg_first[ST - 1];
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) pg_first[i] = unit_page(i);
    int pg_next = unit_page(ST - 1);
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        if (i < n_my) load_unit(i, pg_first[i]);
        cp_async_commit();
    }
    // Q has landed once all but the newest ST-1 groups are complete
    cp_async_wait<ST - 1>();
    __syncthreads();

    unsigned qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], Qs + (lane & 15) * LDS + kk * 16 + (lane >> 4) * 8);

    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const int pos_lo = p_min + r_lo / Gc, pos_hi = p_min + r_hi / Gc;
    const float sc = p.scale * 1.4426950408889634f;

    float o[NDB][4];
#pragma unroll
    for (int i = 0; i < NDB; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    for (int i = 0; i < n_my; ++i) {
        if (i + ST - 1 < n_my) load_unit(i + ST - 1, pg_next);
        cp_async_commit();
        pg_next = unit_page(i + ST);
        cp_async_wait<ST - 1>();
        __syncwarp();
        const __nv_bfloat16* Ks = my_ring + (size_t)(i % ST) * 2 * DEC_WT * LDS;
        const __nv_bfloat16* Vs = Ks + DEC_WT * LDS;
        const int key0 = (u_begin + warp + i * NW) * DEC_WT;

        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            unsigned b[4];
            ldmatrix_x4(b, Ks + ((lane & 7) + ((lane >> 4) & 1) * 8) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16_16816(s[0], qf[kk], b[0], b[1]);
            mma_bf16_16816(s[1], qf[kk], b[2], b[3]);
        }
        const bool need_mask = (key0 + DEC_WT - 1 > p_min) || (p.window > 0 && key0 <= p_max - p.window);
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nb][e] * sc;
                if (need_mask) {
                    const int key = key0 + nb * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = (e < 2) ? pos_lo : pos_hi;
                    bool ok = key <= pos;
                    if (p.window > 0) ok = ok && (key > pos - p.window);
                    if (!ok) v = -INFINITY;
                }
                s[nb][e] = v;
                if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
        const float al_lo = fast_exp2(m_lo - mu_lo), al_hi = fast_exp2(m_hi - mu_hi);
        m_lo = mn_lo; m_hi = mn_hi;
        l_lo *= al_lo; l_hi *= al_hi;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            s[nb][0] = fast_exp2(s[nb][0] - mu_lo); s[nb][1] = fast_exp2(s[nb][1] - mu_lo);
            s[nb][2] = fast_exp2(s[nb][2] - mu_hi); s[nb][3] = fast_exp2(s[nb][3] - mu_hi);
            l_lo += s[nb][0] + s[nb][1];
            l_hi += s[nb][2] + s[nb][3];
        }
        if (al_lo != 1.f || al_hi != 1.f) {
#pragma unroll
            for (int j = 0; j < NDB; ++j) { o[j][0] *= al_lo; o[j][1] *= al_lo; o[j][2] *= al_hi; o[j][3] *= al_hi; }
        }
        unsigned a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int nd2 = 0; nd2 < D / 16; ++nd2) {
            unsigned b[4];
            ldmatrix_x4_trans(b, Vs + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + nd2 * 16 + ((lane >> 4) & 1) * 8);
            mma_bf16_16816(o[2 * nd2], a, b[0], b[1]);
            mma_bf16_16816(o[2 * nd2 + 1], a, b[2], b[3]);
        }
        __syncwarp();
    }
    cp_async_wait<0>();

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // merge the warps (same rows, disjoint keys) through shared memory, in warp order
    float* Om = reinterpret_cast<float*>(ring);             // [NW][16][D]
    float* Mm = Om + NW * 16 * D;                           // [NW][16]
    float* Lm = Mm + NW * 16;                               // [NW][16]
    __syncthreads();
#pragma unroll
    for (int nd = 0; nd < NDB; ++nd) {
        const int col = nd * 8 + (lane & 3) * 2;
        float* d0 = Om + ((size_t)warp * 16 + (lane >> 2)) * D + col;
        float* d1 = d0 + 8 * D;
        *reinterpret_cast<float2*>(d0) = make_float2(o[nd][0], o[nd][1]);
        *reinterpret_cast<float2*>(d1) = make_float2(o[nd][2], o[nd][3]);
    }
    if ((lane & 3) == 0) {
        Mm[warp * 16 + (lane >> 2)] = m_lo; Mm[warp * 16 + (lane >> 2) + 8] = m_hi;
        Lm[warp * 16 + (lane >> 2)] = l_lo; Lm[warp * 16 + (lane >> 2) + 8] = l_hi;
    }
    __syncthreads();
    __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(p.out);
    const int n_rows = min(ti.n_tok, QT) * Gc;              // valid rows come first
    for (int idx = tid; idx < n_rows * D; idx += THREADS) {
        const int r = idx / D, col = idx - r * D;
        const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * R + hl;
        if (hg >= G) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, Mm[w * 16 + r]);
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = fast_exp2(Mm[w * 16 + r] - Mu);
            acc += f * Om[((size_t)w * 16 + r) * D + col];
            L += f * Lm[w * 16 + r];
        }
        const size_t tok = (size_t)(ti.q_base + ti.t0 + tl);
        const int head = kvh * G + hg;
        if (ns == 1) {
            og[(tok * p.n_q + head) * D + col] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t prow = ((size_t)split * p.T + tok) * p.n_q + head;
            p.part_o[prow * D + col] = acc;
            if (col == 0) { p.part_ml[prow * 2] = M; p.part_ml[prow * 2 + 1] = L; }
        }
    }
}

// ---------------------------------------------------------------------------------------
// bfloat16 decode kernel, transposed: the 16 keys of a unit ride the M dimension of the mma and
// the (token, head) pairs of the block ride N (8 per n-block), so
//     S^T[key][col] = K[key][:] . Q[col][:]          O^T[dim][col] += V^T[dim][key] P^T[key][col]
//  * K goes from global memory straight into the A-operand registers (16-byte loads; the k index
//    inside each 32-element group is permuted the same way for K and Q, which leaves the dot
//    products unchanged), Q sits in B-operand registers for the whole block: neither touches
//    shared memory;
//  * V streams through a per-warp cp.async ring and is read with ldmatrix.trans as A operand;
//  * P^T gets from accumulator to B-operand layout with movmatrix;
//  * every warp walks its own units (block's units dealt round-robin) without block barriers;
//    warps are merged in warp order at the end.
// Compared with putting the heads on M this halves the tensor work and the accumulator
// registers (few heads per kv head waste N = 8, not M = 16), so 16 warps fit an SM.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ void mma_bf16_regs(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                              unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg16_stream(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}

// One run of keys of one request through the transposed decode arithmetic: units [u_begin, u_end) of DEC_WT keys, the block's
// warps taking them in turn; the result goes to the output (ns == 1) or to piece `split` of the request's partial results.
// wait_here: this is the block's first run, the wait for the kernel before this one falls behind its first prefetches;
// release_here: it is the last one, the next kernel may start beside its reduction.
template <int D, int NW, int ST, int NBH>
__device__ __forceinline__ void decode_t_run(const AttnParams& p, const TileInfo& ti, int ns, int split, int u_begin, int u_end,
                                             int p_min, int p_max, int kvh, int chunk, bool wait_here, bool release_here,
                                             __nv_bfloat16* ring) {
    constexpr int LDS = D + 8;
    constexpr int C = 8 * NBH;                      // (token, head) columns per block
    constexpr int KP = D / 32;                      // 32-element groups of the head size
    constexpr int MT = D / 16;                      // 16-row tiles of O^T
    constexpr int CH = D / 8;
    constexpr int THREADS = NW * 32;
    const int G = p.n_q / p.n_kv;
    const int Gc = G <= C ? G : C;
    const int QT = G <= C ? C / G : 1;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
    const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;

    // the columns this lane sees in the accumulators: nb*8 + 2t and + 1
    int pos_c[NBH][2];
#pragma unroll
    for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) pos_c[nb][e] = p_min + (nb * 8 + 2 * t + e) / Gc;

    const int n_my = (u_end - u_begin > warp) ? (u_end - u_begin - warp + NW - 1) / NW : 0;
    __nv_bfloat16* my_ring = ring + (size_t)warp * ST * DEC_WT * LDS;
    const int v_key = lane >> 1, v_half = lane & 1;

    // page of key (unit i, row lane & 15), or -1 past the last key; one lookup per lane and unit
    auto unit_page = [&](int i) -> int {
        const int key = (u_begin + warp + i * NW) * DEC_WT + (lane & 15);
        return (i < n_my && key <= p_max) ? bt[page_index(p, key)] : -1;
    };
    auto load_v = [&](int i, int pg_row) {         // V of unit i -> stage i % ST; pg_row: page of row v_key
        __nv_bfloat16* Vs = my_ring + (size_t)(i % ST) * DEC_WT * LDS;
        const int key = (u_begin + warp + i * NW) * DEC_WT + v_key;
        const bool valid = pg_row >= 0;
        size_t off = 0;
        if (valid) off = (((size_t)pg_row * p.n_kv + kvh) * p.page_size + page_slot(p, key)) * D;
#pragma unroll
        for (int j = 0; j < CH / 2; ++j) {
            const int c = 2 * j + v_half;
            cp_async16(Vs + v_key * LDS + c * 8, vc + off + c * 8, valid);
        }
    };
    // K of unit i into L2 ahead of the register load (no registers, no shared memory spent on it);
    // pg_row: page of row lane >> 1, each lane touches 128-byte lines of that row
    auto prefetch_k = [&](int i, int pg_row) {
        if (pg_row < 0) return;
        const int key = (u_begin + warp + i * NW) * DEC_WT + v_key;
        const size_t off = (((size_t)pg_row * p.n_kv + kvh) * p.page_size + page_slot(p, key)) * D;
#pragma unroll
        for (int ln = 0; ln < (D + 127) / 128; ++ln) {
            const int e = (2 * ln + v_half) * 64;
            if (e < D) {
                asm volatile("prefetch.global.L2 [%0];\n" ::"l"(kc + off + e));
#if MSGL_DEC_PFV
                asm volatile("prefetch.global.L2 [%0];\n" ::"l"(vc + off + e));
#endif
            }
        }
    };
    uint4 k_lo[KP], k_hi[KP];
    auto load_k = [&](int i, int pg_lo, int pg_hi) {      // K of unit i -> registers (rows g and g + 8)
        const int key0 = (u_begin + warp + i * NW) * DEC_WT;
        const __nv_bfloat16* lo = kc + (((size_t)max(pg_lo, 0) * p.n_kv + kvh) * p.page_size + page_slot(p, key0 + g)) * D + 8 * t;
        const __nv_bfloat16* hi = kc + (((size_t)max(pg_hi, 0) * p.n_kv + kvh) * p.page_size + page_slot(p, key0 + 8 + g)) * D + 8 * t;
#pragma unroll
        for (int j = 0; j < KP; ++j) {
            k_lo[j] = pg_lo >= 0 ? ldg16_stream(lo + 32 * j) : make_uint4(0u, 0u, 0u, 0u);
            k_hi[j] = pg_hi >= 0 ? ldg16_stream(hi + 32 * j) : make_uint4(0u, 0u, 0u, 0u);
        }
    };

    // first keys towards L2, then wait for the kernel before this one
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int pg = unit_page(i);
        prefetch_k(i, __shfl_sync(0xffffffffu, pg, v_key));
    }
    if (wait_here) {
        pdl_wait();
        pdl_after_wait();
    }

    // Q as B operand: lane (g, t) holds Q[column nb*8 + g][32 j + 8 t .. + 7]
    uint4 qf[NBH][KP];
#pragma unroll
    for (int nb = 0; nb < NBH; ++nb) {
        const int c = nb * 8 + g;
        const int tl = c / Gc, hl = c - tl * Gc, hg = chunk * C + hl;
        const bool valid = tl < ti.n_tok && tl < QT && hg < G;
        const __nv_bfloat16* src = qg + ((size_t)(ti.q_base + ti.t0 + (valid ? tl : 0)) * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * D + 8 * t;
#pragma unroll
        for (int j = 0; j < KP; ++j)
            qf[nb][j] = valid ? *reinterpret_cast<const uint4*>(src + 32 * j) : make_uint4(0u, 0u, 0u, 0u);
    }
    // prologue: V of the first ST-1 units, K of unit 0, page of the next unit to fetch
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        const int pg = unit_page(i);
        const int pg_row = __shfl_sync(0xffffffffu, pg, v_key);
        if (i < n_my) load_v(i, pg_row);
        cp_async_commit();
        if (i == 0 && n_my > 0) load_k(0, __shfl_sync(0xffffffffu, pg, g), __shfl_sync(0xffffffffu, pg, g + 8));
        if (i > 0 && i < n_my) prefetch_k(i, pg_row);
    }
    int pg_pf_next = unit_page(MSGL_DEC_PFK);      // for the L2 prefetch issued in iteration 0 (when it has a distance of its own)
    int pg_v_next = unit_page(ST - 1);             // for the V copy issued in iteration 0
    int pg_k_next = unit_page(1);                  // for the K load issued in iteration 0

    float o[NBH][MT][4];
#pragma unroll
    for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) { o[nb][mt][0] = o[nb][mt][1] = o[nb][mt][2] = o[nb][mt][3] = 0.f; }
    float m_c[NBH][2], l_c[NBH][2];
#pragma unroll
    for (int nb = 0; nb < NBH; ++nb) { m_c[nb][0] = m_c[nb][1] = -INFINITY; l_c[nb][0] = l_c[nb][1] = 0.f; }
    const float sc = p.scale * 1.4426950408889634f;

    for (int i = 0; i < n_my; ++i) {
        // ---- S^T = K Q^T from registers
        float s[NBH][4], s2[NBH][4];
#pragma unroll
        for (int nb = 0; nb < NBH; ++nb) {
            s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
            s2[nb][0] = s2[nb][1] = s2[nb][2] = s2[nb][3] = 0.f;
#pragma unroll
            for (int j = 0; j < KP; ++j) {
                mma_bf16_regs(s[nb], k_lo[j].x, k_hi[j].x, k_lo[j].y, k_hi[j].y, qf[nb][j].x, qf[nb][j].y);
                mma_bf16_regs(s2[nb], k_lo[j].z, k_hi[j].z, k_lo[j].w, k_hi[j].w, qf[nb][j].z, qf[nb][j].w);
            }
        }
        // ---- next K into the same registers, next V into the ring
        {
            const int pk = pg_k_next;
            if (i + 1 < n_my) load_k(i + 1, __shfl_sync(0xffffffffu, pk, g), __shfl_sync(0xffffffffu, pk, g + 8));
            const int pv = __shfl_sync(0xffffffffu, pg_v_next, v_key);
            if (i + ST - 1 < n_my) load_v(i + ST - 1, pv);
            cp_async_commit();
            if (MSGL_DEC_PFK == ST - 1) {
                if (i + ST - 1 < n_my) prefetch_k(i + ST - 1, pv);
            } else if (MSGL_DEC_PFK > 0) {
                const int pf = __shfl_sync(0xffffffffu, pg_pf_next, v_key);
                if (i + MSGL_DEC_PFK < n_my) prefetch_k(i + MSGL_DEC_PFK, pf);
                pg_pf_next = unit_page(i + MSGL_DEC_PFK + 1);
            }
            pg_k_next = unit_page(i + 2);
            pg_v_next = unit_page(i + ST);
        }
        // ---- scale, mask, online softmax per column
        const int key0 = (u_begin + warp + i * NW) * DEC_WT;
        const bool need_mask = (key0 + DEC_WT - 1 > p_min) || (p.window > 0 && key0 <= p_max - p.window);
        unsigned pb0[NBH], pb1[NBH];
        float v[NBH][4];
        bool behind = false;              // a score lies further above its column's reference than DEC_LAZY allows
#pragma unroll
        for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v[nb][e] = (s[nb][e] + s2[nb][e]) * sc;
                if (need_mask) {
                    const int key = key0 + g + ((e & 2) ? 8 : 0);
                    const int pos = pos_c[nb][e & 1];
                    bool ok = key <= pos;
                    if (p.window > 0) ok = ok && (key > pos - p.window);
                    if (!ok) v[nb][e] = -INFINITY;
                }
                behind = behind || v[nb][e] > m_c[nb][e & 1] + DEC_LAZY;
            }
        // The reference m of a column's exponentials need not be the maximum so far: any m that keeps 2^(s - m) within
        // the range of bfloat16 and float32 gives the same softmax.  So the maximum over the unit's keys (three shuffles
        // a column) is only looked for when some score of the warp lies more than DEC_LAZY above its reference (always
        // for a column's first finite score); then the references move and the sums and accumulators are scaled.
        if (__any_sync(0xffffffffu, behind)) {
            float alpha[NBH][2];
#pragma unroll
            for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float mx = fmaxf(v[nb][e], v[nb][e + 2]);
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float mn = fmaxf(m_c[nb][e], mx);
                    const float mu = (mn == -INFINITY) ? 0.f : mn;
                    alpha[nb][e] = fast_exp2(m_c[nb][e] - mu);
                    m_c[nb][e] = mn;
                    l_c[nb][e] *= alpha[nb][e];
                }
#pragma unroll
            for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    o[nb][mt][0] *= alpha[nb][0]; o[nb][mt][1] *= alpha[nb][1];
                    o[nb][mt][2] *= alpha[nb][0]; o[nb][mt][3] *= alpha[nb][1];
                }
        }
#pragma unroll
        for (int nb = 0; nb < NBH; ++nb) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float mu = (m_c[nb][e] == -INFINITY) ? 0.f : m_c[nb][e];
                v[nb][e] = fast_exp2(v[nb][e] - mu);
                v[nb][e + 2] = fast_exp2(v[nb][e + 2] - mu);
                l_c[nb][e] += v[nb][e] + v[nb][e + 2];
            }
            // accumulator layout (key g | g+8 ; columns 2t, 2t+1) -> B operand layout (keys 2t, 2t+1 ; column g)
            pb0[nb] = movmatrix_trans(pack_bf16(v[nb][0], v[nb][1]));
            pb1[nb] = movmatrix_trans(pack_bf16(v[nb][2], v[nb][3]));
        }
        // ---- O^T += V^T P^T
        cp_async_wait<ST - 1>();
        __syncwarp();
        const __nv_bfloat16* Vs = my_ring + (size_t)(i % ST) * DEC_WT * LDS;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            unsigned a[4];
            ldmatrix_x4_trans(a, Vs + ((lane & 7) + ((lane >> 4) & 1) * 8) * LDS + mt * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int nb = 0; nb < NBH; ++nb) mma_bf16_16816(o[nb][mt], a, pb0[nb], pb1[nb]);
        }
        __syncwarp();
    }
    if (release_here) pdl_late();
    cp_async_wait<0>();

    // column sums over the 8 lanes that share a column pair
#pragma unroll
    for (int nb = 0; nb < NBH; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float l = l_c[nb][e];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            l_c[nb][e] = l;
        }

    // merge the warps through shared memory, in warp order
    float* Om = reinterpret_cast<float*>(ring);             // [NW][C][D]
    float* Mm = Om + NW * C * D;                            // [NW][C]
    float* Lm = Mm + NW * C;                                // [NW][C]
    __syncthreads();
#pragma unroll
    for (int nb = 0; nb < NBH; ++nb) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int c = nb * 8 + 2 * t + (e & 1);
                const int dim = mt * 16 + g + ((e & 2) ? 8 : 0);
                Om[((size_t)warp * C + c) * D + dim] = o[nb][mt][e];
            }
        if (g == 0) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                Mm[warp * C + nb * 8 + 2 * t + e] = m_c[nb][e];
                Lm[warp * C + nb * 8 + 2 * t + e] = l_c[nb][e];
            }
        }
    }
    __syncthreads();
    __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(p.out);
    const int n_cols = min(min(ti.n_tok, QT) * Gc, C);      // valid columns come first
    for (int idx = tid; idx < n_cols * D; idx += THREADS) {
        const int c = idx / D, col = idx - c * D;
        const int tl = c / Gc, hl = c - tl * Gc, hg = chunk * C + hl;
        if (hg >= G) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, Mm[w * C + c]);
        const float Mu = (M == -INFINITY) ? 0.f : M;
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = fast_exp2(Mm[w * C + c] - Mu);
            acc += f * Om[((size_t)w * C + c) * D + col];
            L += f * Lm[w * C + c];
        }
        const size_t tok = (size_t)(ti.q_base + ti.t0 + tl);
        const int head = kvh * G + hg;
        if (ns == 1) {
            og[(tok * p.n_q + head) * D + col] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t prow = ((size_t)split * p.T + tok) * p.n_q + head;
            p.part_o[prow * D + col] = acc;
            if (col == 0) { p.part_ml[prow * 2] = M; p.part_ml[prow * 2 + 1] = L; }
        }
    }
}

template <int D, int NW, int ST, int NBH>
__global__ void __launch_bounds__(NW * 32, (NBH == 1 && D <= 128) ? 4 : 2) attn_decode_t_kernel(const AttnParams p) {
    constexpr int C = 8 * NBH;
    static_assert(D % 32 == 0, "the transposed decode kernel needs head sizes in steps of 32");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [NW][ST][16][LDS]  (V only)
    __shared__ int sh_tile[4];

    // What the kernel before this one writes are q and the new tokens' cache rows.  Lengths, splits and block
    // tables come from the step's staging copy, so the block finds its work and asks for its first keys to be
    // brought into L2 while that kernel still runs, and waits for it only then.
    pdl_launch_dependents();
    const int G = p.n_q / p.n_kv;
    const int n_chunks = G <= C ? 1 : (G + C - 1) / C;
    const int QT = G <= C ? C / G : 1;
    int tile_idx, by;
    block_place(p, tile_idx, by);
    const int kvh = by / n_chunks;
    const int chunk = by - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, QT, ti, sh_tile, tile_idx, (int)gridDim.x)) return;
    const int ns = p.nsplit ? min(max(p.nsplit[ti.req], 1), p.max_split) : 1;
    const int split = blockIdx.z;
    if (split >= ns) return;

    int p_min, p_max, kt_begin, kt_end;
    key_tile_range(p, ti, MMA_KT, split, ns, p_min, p_max, kt_begin, kt_end);
    const int u_begin = kt_begin * (MMA_KT / DEC_WT);
    const int u_end = min(kt_end * (MMA_KT / DEC_WT), p_max / DEC_WT + 1);
    decode_t_run<D, NW, ST, NBH>(p, ti, ns, split, u_begin, u_end, p_min, p_max, kvh, chunk, true, true, ring);
}

// The same arithmetic for a decode step (one token a request) with the keys of all requests dealt out evenly: the launch
// has a fixed number of blocks per kv head, block j takes units [start[j], start[j + 1]) of the requests' units laid end
// to end, whatever requests they belong to.  A request that several blocks share is merged by attn_combine_kernel from
// its pieces (piece = block index - first block of the request); one that lies within a block is written out at once.
// The host deals the units out (engine/step.py: plan_even_cut); this kernel only reads the result.
template <int D, int NW, int ST, int NBH>
__global__ void __launch_bounds__(NW * 32, (NBH == 1 && D <= 128) ? 4 : 2) attn_decode_even_kernel(const AttnParams p) {
    constexpr int C = 8 * NBH;
    static_assert(D % 32 == 0, "the transposed decode kernel needs head sizes in steps of 32");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);

    pdl_launch_dependents();
    const int G = p.n_q / p.n_kv;
    const int n_chunks = G <= C ? 1 : (G + C - 1) / C;
    const int kvh = blockIdx.y / n_chunks;
    const int chunk = blockIdx.y - kvh * n_chunks;
    const int j = blockIdx.x;
    const int NB = p.even_nb;
    if (j >= NB || j >= p.even[0]) return;
    const int* blk_start = p.even + 1;
    const int* blk_req = blk_start + NB + 1;
    const int* req_start = blk_req + NB;
    const int* req_first_blk = req_start + p.B + 1;
    int lo = blk_start[j];
    const int hi = blk_start[j + 1];
    int r = blk_req[j];
    bool first = true;
    while (lo < hi && r >= 0 && r < p.B) {
        const int c0 = req_start[r], c1 = req_start[r + 1];
        if (c1 <= lo || c0 > lo) { ++r; continue; }          // never with a well-formed cut; keeps the walk inside the arrays
        const int seg_hi = min(hi, c1);
        TileInfo ti;
        ti.req = r; ti.t0 = 0; ti.n_tok = 1; ti.q_len = 1; ti.kv_len = p.kv_len[r]; ti.q_base = p.q_start[r];
        const int pos = ti.kv_len - 1;
        const int k_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const int first_unit = k_lo / DEC_WT;
        const int ns = p.nsplit ? min(max(p.nsplit[r], 1), p.max_split) : 1;
        const int piece = j - req_first_blk[r];
        const bool last = seg_hi >= hi;
        if (piece >= 0 && piece < ns) {
            if (!first) __syncthreads();       // the reduction of the run before this one has left the ring
            decode_t_run<D, NW, ST, NBH>(p, ti, ns, piece, first_unit + (lo - c0), min(first_unit + (seg_hi - c0), pos / DEC_WT + 1),
                                         pos, pos, kvh, chunk, first, last, ring);
            first = false;
        }
        lo = seg_hi;
        ++r;
    }
}

// ---------------------------------------------------------------------------------------
// float32-arithmetic kernel for any head size (the true 32-bit path; also takes bfloat16 data)
// ---------------------------------------------------------------------------------------
constexpr int SIMT_R = 16;        // rows per block
constexpr int SIMT_KT = 32;       // keys per tile
constexpr int SIMT_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(SIMT_THREADS) attn_simt_kernel(const AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int D = p.d;
    float* Qs = reinterpret_cast<float*>(smem_raw);          // [R][D]
    float* Os = Qs + SIMT_R * D;                             // [R][D]
    float* Ks = Os + SIMT_R * D;                             // [KT][D + 1]
    float* Vs = Ks + SIMT_KT * (D + 1);                      // [KT][D]
    float* Ss = Vs + SIMT_KT * D;                            // [R][KT]
    float* Ms = Ss + SIMT_R * SIMT_KT;                       // [R]
    float* Ls = Ms + SIMT_R;                                 // [R]
    float* As = Ls + SIMT_R;                                 // [R]
    __shared__ int sh_tile[4];

    constexpr int R = SIMT_R;
    const int G = p.n_q / p.n_kv;
    const int Gc = G <= R ? G : R;
    const int n_chunks = G <= R ? 1 : (G + R - 1) / R;
    const int QT = G <= R ? R / G : 1;
    int tile_idx, by;
    block_place(p, tile_idx, by);
    const int kvh = by / n_chunks;
    const int chunk = by - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, QT, ti, sh_tile, tile_idx, (int)gridDim.x)) return;
    const int ns = p.nsplit ? min(max(p.nsplit[ti.req], 1), p.max_split) : 1;
    const int split = blockIdx.z;
    if (split >= ns) return;
    int p_min, p_max, kt_begin, kt_end;
    key_tile_range(p, ti, SIMT_KT, split, ns, p_min, p_max, kt_begin, kt_end);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* qg = reinterpret_cast<const T*>(p.q);
    const T* kc = reinterpret_cast<const T*>(p.k_cache);
    const T* vc = reinterpret_cast<const T*>(p.v_cache);
    const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;
    const float sc = p.scale * 1.4426950408889634f;

    for (int idx = tid; idx < R * D; idx += SIMT_THREADS) {
        const int r = idx / D, c = idx - r * D;
        const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * R + hl;
        const bool valid = tl < ti.n_tok && hg < G && tl < QT;
        float v = 0.f;
        if (valid) v = to_f32<T>(qg[((size_t)(ti.q_base + ti.t0 + tl) * p.n_q + (size_t)kvh * G + hg) * D + c]);
        Qs[idx] = v;
        Os[idx] = 0.f;
    }
    if (tid < R) { Ms[tid] = -INFINITY; Ls[tid] = 0.f; As[tid] = 0.f; }
    __syncthreads();

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int key0 = kt * SIMT_KT;
        for (int idx = tid; idx < SIMT_KT * D; idx += SIMT_THREADS) {
            const int kl = idx / D, c = idx - kl * D;
            const int key = key0 + kl;
            float kv = 0.f, vv = 0.f;
            if (key <= p_max) {
                const int pg = bt[page_index(p, key)];
                const int sl = page_slot(p, key);
                const size_t off = (((size_t)pg * p.n_kv + kvh) * p.page_size + sl) * D + c;
                kv = to_f32<T>(kc[off]);
                vv = to_f32<T>(vc[off]);
            }
            Ks[kl * (D + 1) + c] = kv;
            Vs[kl * D + c] = vv;
        }
        __syncthreads();
        // scores: one (row, key) pair per thread and pass; a warp shares the row
        for (int idx = tid; idx < R * SIMT_KT; idx += SIMT_THREADS) {
            const int r = idx / SIMT_KT, kl = idx - r * SIMT_KT;
            const float* qr = Qs + r * D;
            const float* kr = Ks + kl * (D + 1);
            float acc = 0.f;
            for (int c = 0; c < D; ++c) acc = fmaf(qr[c], kr[c], acc);
            const int key = key0 + kl;
            const int pos = p_min + r / Gc;
            bool ok = key <= pos && (r / Gc) < ti.n_tok;
            if (p.window > 0) ok = ok && (key > pos - p.window);
            Ss[idx] = ok ? acc * sc : -INFINITY;
        }
        __syncthreads();
        // online softmax, one warp per row, one lane per key
        for (int r = warp; r < R; r += SIMT_THREADS / 32) {
            const float v = Ss[r * SIMT_KT + lane];
            const float mx = warp_max(v);
            const float m_old = Ms[r];
            const float m_new = fmaxf(m_old, mx);
            const float mu = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = exp2f(m_old - mu);
            const float pv = exp2f(v - mu);
            const float sum = warp_sum(pv);
            Ss[r * SIMT_KT + lane] = pv;
            if (lane == 0) { Ms[r] = m_new; Ls[r] = Ls[r] * alpha + sum; As[r] = alpha; }
        }
        __syncthreads();
        for (int idx = tid; idx < R * D; idx += SIMT_THREADS) {
            const int r = idx / D, c = idx - r * D;
            float acc = Os[idx] * As[r];
            const float* pr = Ss + r * SIMT_KT;
#pragma unroll 8
            for (int kl = 0; kl < SIMT_KT; ++kl) acc = fmaf(pr[kl], Vs[kl * D + c], acc);
            Os[idx] = acc;
        }
        __syncthreads();
    }

    T* og = reinterpret_cast<T*>(p.out);
    for (int idx = tid; idx < R * D; idx += SIMT_THREADS) {
        const int r = idx / D, c = idx - r * D;
        const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * R + hl;
        if (!(tl < ti.n_tok && hg < G && tl < QT)) continue;
        const size_t tok = (size_t)(ti.q_base + ti.t0 + tl);
        const int head = kvh * G + hg;
        if (ns == 1) {
            const float l = Ls[r];
            og[(tok * p.n_q + head) * D + c] = from_f32<T>(l > 0.f ? Os[idx] / l : 0.f);
        } else {
            const size_t prow = ((size_t)split * p.T + tok) * p.n_q + head;
            p.part_o[prow * D + c] = Os[idx];
            if (c == 0) { p.part_ml[prow * 2] = Ms[r]; p.part_ml[prow * 2 + 1] = Ls[r]; }
        }
    }
}

// ---------------------------------------------------------------------------------------
// merge of the kv splits, in split order: out = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    const int* __restrict__ token_req, const int* __restrict__ nsplit,
                                    T* __restrict__ out, int T_, int n_q, int d, int max_split) {
    // one block per (token, head); threads over the head's elements
    pdl_launch_dependents();
    pdl_wait();
    pdl_after_wait();
    pdl_small();
    const int tok = blockIdx.x, h = blockIdx.y;
    const int req = token_req ? token_req[tok] : tok;
    const int ns = min(max(nsplit[req], 1), max_split);
    if (ns <= 1) return;
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(((size_t)s * T_ + tok) * n_q + h) * 2]);
    const float Mu = (M == -INFINITY) ? 0.f : M;
    float L = 0.f;
    for (int s = 0; s < ns; ++s) {
        const size_t prow = ((size_t)s * T_ + tok) * n_q + h;
        L += exp2f(part_ml[prow * 2] - Mu) * part_ml[prow * 2 + 1];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < ns; ++s) {
            const size_t prow = ((size_t)s * T_ + tok) * n_q + h;
            acc += exp2f(part_ml[prow * 2] - Mu) * part_o[prow * d + c];
        }
        out[((size_t)tok * n_q + h) * d + c] = from_f32<T>(acc * inv);
    }
}

#if MSGL_HEAD_DIM == 128
#include "attention_tc.cuh"
#include "attention_tc2.cuh"
#endif

// ---------------------------------------------------------------------------------------
// C entry points
// ---------------------------------------------------------------------------------------
MSGL_API int msgl_attention_head_dim() { return MSGL_HEAD_DIM; }

// rows per block and tokens per query tile of a variant, for the host's grid arithmetic
// variant: 0 = simt, 1 = mma 64-row, 2 = mma key-split (16-row)
MSGL_API int msgl_attention_tile_rows(int variant) { return variant == 1 ? 64 : 16; }

// tokens per query tile of the decode variant for a group size (q heads per kv head)
MSGL_API int msgl_attention_decode_tile_tokens(int G) {
    if (MSGL_HEAD_DIM % 32 == 0 && G <= 16) return (G <= 8 ? 8 : 16) / G;
    return G <= 16 ? 16 / G : 1;
}

// how many blocks of the decode kernel fit one SM, for the host's choice of kv splits
// 1 if the decode launch of this library can take an even cut (msgl_attention's `even`) for G q heads per kv head
MSGL_API int msgl_attention_decode_even_ok(int G) { return (MSGL_HEAD_DIM % 32 == 0 && G <= 16) ? 1 : 0; }

MSGL_API int msgl_attention_decode_blocks_per_sm(int G) {
    size_t smem;
    int reg_limit;
    if (MSGL_HEAD_DIM % 32 == 0 && G <= 16) {
        smem = sizeof(__nv_bfloat16) * (size_t)MSGL_DEC_WARPS * MSGL_DEC_STAGES * 16 * (MSGL_HEAD_DIM + 8) + 1024;
        reg_limit = (G <= 8 && MSGL_HEAD_DIM <= 128) ? 4 : 2;
    } else {
        constexpr int ST = (MSGL_HEAD_DIM <= 128) ? MSGL_DEC_STAGES : 2;
        smem = sizeof(__nv_bfloat16) * ((size_t)16 * (MSGL_HEAD_DIM + 8) + (size_t)MSGL_DEC_WARPS * ST * 2 * 16 * (MSGL_HEAD_DIM + 8)) + 1024;
        reg_limit = 3;
    }
    int n = (int)((227 * 1024) / smem);
    n = n < reg_limit ? n : reg_limit;
    return n < 1 ? 1 : n;
}

static size_t simt_smem_bytes(int d) {
    return sizeof(float) * ((size_t)2 * SIMT_R * d + (size_t)SIMT_KT * (2 * d + 1) + SIMT_R * SIMT_KT + 3 * SIMT_R);
}

template <int D> static size_t mma_smem_bytes() {
    constexpr int R = 64;
    return sizeof(__nv_bfloat16) * ((size_t)R * (D + 8) + (size_t)4 * MMA_KT * (D + 8));
}

// grid_x: number of query tiles the launch has to cover (the host knows every q_len).
MSGL_API int msgl_attention(const void* q, void* out, const void* k_cache, const void* v_cache, const int* q_start,
                            const int* kv_len, const int* block_table, const int* nsplit, float* part_o,
                            float* part_ml, int B, int T_, int n_q, int n_kv, int d, int page_size, int bt_stride,
                            int window, int max_split, float scale, int qlen_min, int qlen_max, int uniform_decode,
                            int variant, int grid_x, int dtype, const int* order, const int* even, int even_nb,
                            cudaStream_t stream) {
    if (grid_x <= 0 || B <= 0) return MSGL_OK;
    if (n_kv <= 0 || n_q % n_kv != 0 || d <= 0 || page_size <= 0 || max_split < 1) return MSGL_ERR_SIZE;
    if (max_split > 1 && (part_o == nullptr || part_ml == nullptr || nsplit == nullptr)) return MSGL_ERR_SIZE;
    AttnParams p;
    p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len;
    p.block_table = block_table; p.nsplit = nsplit; p.order = order; p.even = nullptr; p.even_nb = 0;
    p.part_o = part_o; p.part_ml = part_ml;
    p.B = B; p.T = T_; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.page_size = page_size; p.bt_stride = bt_stride;
    p.window = window; p.max_split = max_split;
    p.page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) { int sh = 0; while ((1 << sh) < page_size) ++sh; p.page_shift = sh; } p.scale = scale; p.qlen_min = qlen_min; p.qlen_max = qlen_max;
    p.uniform_decode = uniform_decode;
    const int G = n_q / n_kv;
    const int R = variant == 1 ? 64 : 16;
    const int n_chunks = G <= R ? 1 : (G + R - 1) / R;
    dim3 grid(grid_x, n_kv * n_chunks, max_split);
    // an even cut is read by the transposed decode kernel only (nsplit then counts a request's pieces, not equal splits)
    if (even != nullptr && !(variant == 2 && MSGL_HEAD_DIM % 32 == 0 && G <= 16 && dtype == MSGL_BF16)) return MSGL_ERR_SIZE;
    if (variant == 0) {
        if (d > 512) return MSGL_ERR_SIZE;
        const size_t smem = simt_smem_bytes(d);
        if (smem > 227 * 1024) return MSGL_ERR_SIZE;
        static size_t simt_attr[MSGL_MAX_DEVICES][2] = {};   // largest size already granted per device and element type
        size_t* granted = simt_attr[msgl_device()];
        if (dtype == MSGL_F32) {
            if (smem > 48 * 1024 && smem > granted[0]) {
                cudaFuncSetAttribute(attn_simt_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                granted[0] = smem;
            }
            attn_simt_kernel<float><<<grid, SIMT_THREADS, smem, stream>>>(p);
        } else if (dtype == MSGL_BF16) {
            if (smem > 48 * 1024 && smem > granted[1]) {
                cudaFuncSetAttribute(attn_simt_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                granted[1] = smem;
            }
            attn_simt_kernel<__nv_bfloat16><<<grid, SIMT_THREADS, smem, stream>>>(p);
        } else {
            return MSGL_ERR_DTYPE;
        }
        return msgl_check_launch();
    }
    if (dtype != MSGL_BF16) return MSGL_ERR_DTYPE;
    if (d != MSGL_HEAD_DIM) return MSGL_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return MSGL_ERR_ALIGN;
    if (variant == 1) {
        const size_t smem = mma_smem_bytes<MSGL_HEAD_DIM>();
        static MsglOncePerDevice attr_set;   // set once per device, outside any stream capture (the first launch is never captured)
        if (attr_set.due()) {
            cudaFuncSetAttribute(attn_mma_kernel<MSGL_HEAD_DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            attr_set.mark();
        }
        attn_mma_kernel<MSGL_HEAD_DIM><<<grid, MMA_THREADS, smem, stream>>>(p);
    } else if (variant == 2) {
        constexpr int NW = MSGL_DEC_WARPS;
        if (MSGL_HEAD_DIM % 32 == 0 && G <= 16) {
            // transposed kernel: columns = (token, head) pairs, 8 or 16 per block
            constexpr int DT = (MSGL_HEAD_DIM % 32 == 0) ? MSGL_HEAD_DIM : 32;      // keeps the template legal for other head sizes
            constexpr int ST = MSGL_DEC_STAGES;
            const size_t smem = sizeof(__nv_bfloat16) * (size_t)NW * ST * DEC_WT * (DT + 8);
            const int C = G <= 8 ? 8 : 16;
            grid.y = n_kv;      // G <= C: one chunk
            static MsglOncePerDevice attr_set;
            if (attr_set.due()) {
                cudaFuncSetAttribute(attn_decode_t_kernel<DT, NW, ST, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                cudaFuncSetAttribute(attn_decode_t_kernel<DT, NW, ST, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                cudaFuncSetAttribute(attn_decode_even_kernel<DT, NW, ST, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                cudaFuncSetAttribute(attn_decode_even_kernel<DT, NW, ST, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                attr_set.mark();
            }
            if (even != nullptr) {
                // the keys of a decode step dealt out evenly over even_nb blocks per kv head
                if (!uniform_decode || even_nb < 1 || T_ != B) return MSGL_ERR_SIZE;
                p.even = even; p.even_nb = even_nb;
                grid = dim3(even_nb, n_kv, 1);
                if (C == 8) msgl_launch_pdl(attn_decode_even_kernel<DT, NW, ST, 1>, grid, dim3(NW * 32), smem, stream, p);
                else msgl_launch_pdl(attn_decode_even_kernel<DT, NW, ST, 2>, grid, dim3(NW * 32), smem, stream, p);
                return msgl_check_launch();
            }
            if (C == 8) msgl_launch_pdl(attn_decode_t_kernel<DT, NW, ST, 1>, grid, dim3(NW * 32), smem, stream, p);
            else msgl_launch_pdl(attn_decode_t_kernel<DT, NW, ST, 2>, grid, dim3(NW * 32), smem, stream, p);
        } else {
            constexpr int ST = (MSGL_HEAD_DIM <= 128) ? MSGL_DEC_STAGES : 2;   // the ring must fit 227 KB
            const size_t smem = sizeof(__nv_bfloat16) * ((size_t)16 * (MSGL_HEAD_DIM + 8) +
                                                         (size_t)NW * ST * 2 * DEC_WT * (MSGL_HEAD_DIM + 8));
            static MsglOncePerDevice attr_set;
            if (attr_set.due()) {
                cudaFuncSetAttribute(attn_decode_kernel<MSGL_HEAD_DIM, NW, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                attr_set.mark();
            }
            attn_decode_kernel<MSGL_HEAD_DIM, NW, ST><<<grid, NW * 32, smem, stream>>>(p);
        }
    } else {
        return MSGL_ERR_SIZE;
    }
    return msgl_check_launch();
}

// tcgen05 prefill attention (head size 128, bfloat16): the requests with qlen_min <= q_len <= qlen_max, no kv
// splits.  `status` is a device int the kernel sets to 1 if a block gave up waiting (never expected).
// cache_pages: pages in the cache arrays (their first dimension), for the tensor maps of the TMA path.
// version 1: 128 query rows per block, two blocks per SM, any page size; version 2: 256 rows per block in
// ping-pong, TMA page sizes only (MSGL_ERR_SIZE otherwise: the caller then uses version 1).  grid_x counts
// tiles of 128 / group (version 1) or 256 / group (version 2) tokens.
MSGL_API int msgl_attention_tc(const void* q, void* out, const void* k_cache, const void* v_cache, const int* q_start,
                               const int* kv_len, const int* block_table, int B, int T_, int n_q, int n_kv, int d,
                               int page_size, int bt_stride, int window, float scale, int qlen_min, int qlen_max,
                               int grid_x, int cache_pages, int version, int* status, cudaStream_t stream) {
#if MSGL_HEAD_DIM == 128
    if (grid_x <= 0 || B <= 0) return MSGL_OK;
    if (d != 128 || n_kv <= 0 || n_q % n_kv != 0 || page_size <= 0 || grid_x > 65535) return MSGL_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) return MSGL_ERR_ALIGN;
    AttnParams p;
    p.q = q; p.out = out; p.k_cache = k_cache; p.v_cache = v_cache; p.q_start = q_start; p.kv_len = kv_len;
    p.block_table = block_table; p.nsplit = nullptr; p.order = nullptr; p.even = nullptr; p.even_nb = 0;
    p.part_o = nullptr; p.part_ml = nullptr;
    p.B = B; p.T = T_; p.n_q = n_q; p.n_kv = n_kv; p.d = d; p.page_size = page_size; p.bt_stride = bt_stride;
    p.window = window; p.max_split = 1;
    p.page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) { int sh = 0; while ((1 << sh) < page_size) ++sh; p.page_shift = sh; }
    p.scale = scale; p.qlen_min = qlen_min; p.qlen_max = qlen_max; p.uniform_decode = 0;
    const int G = n_q / n_kv;
    const int n_chunks = G <= TC_ROWS ? 1 : (G + TC_ROWS - 1) / TC_ROWS;
    const size_t smem = (size_t)TC_SMEM_BYTES + 1024;
    static MsglOncePerDevice attr_set;
    if (attr_set.due()) {      // first call on this device, never inside a stream capture
        if (cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaFuncSetAttribute(attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC2_SMEM_ALLOC) != cudaSuccess)
            return msgl_check_launch();
        attr_set.mark();
    }
    // TMA boxes are whole pages (or 128-row pieces of larger ones): page sizes 8, 16, 32, 64, 128, 256, ...; the cache
    // base must be 128-byte aligned.  Anything else gathers rows with cp.async.
    int tma_box = 0;
    CUtensorMap kmap = {}, vmap = {};
    const bool pow2 = (page_size & (page_size - 1)) == 0;
    if (pow2 && page_size >= 8 && cache_pages > 0 && ((((uintptr_t)k_cache | (uintptr_t)v_cache) & 127) == 0)) {
        const int box = page_size < TC_KT ? page_size : TC_KT;
        const long long rows = (long long)cache_pages * n_kv * page_size;
        if (tc_matrix_map(k_cache, rows, 128, 256, box, &kmap) && tc_matrix_map(v_cache, rows, 128, 256, box, &vmap)) tma_box = box;
    }
    if (version == 2) {
        if (tma_box == 0) return MSGL_ERR_SIZE;
        attn_tc2_kernel<<<dim3(n_kv * n_chunks, grid_x, 1), TC2_THREADS, TC2_SMEM_ALLOC, stream>>>(p, status, kmap, vmap, tma_box);
        return msgl_check_launch();
    }
    attn_tc_kernel<<<dim3(n_kv * n_chunks, grid_x, 1), TC_THREADS, smem, stream>>>(p, status, kmap, vmap, tma_box);
    return msgl_check_launch();
#else
    return MSGL_ERR_SIZE;
#endif
}

MSGL_API int msgl_attention_combine(const float* part_o, const float* part_ml, const int* token_req,
                                    const int* nsplit, void* out, int T_, int n_q, int d, int max_split, int dtype,
                                    cudaStream_t stream) {
    if (T_ <= 0 || max_split <= 1) return MSGL_OK;
    const int threads = d >= 128 ? 128 : (d >= 64 ? 64 : 32);
    const dim3 grid(T_, n_q);
    if (dtype == MSGL_F32)
        msgl_launch_pdl(attn_combine_kernel<float>, grid, dim3(threads), 0, stream, part_o, part_ml, token_req, nsplit, (float*)out, T_, n_q, d, max_split);
    else if (dtype == MSGL_BF16)
        msgl_launch_pdl(attn_combine_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, part_o, part_ml, token_req, nsplit,
                        (__nv_bfloat16*)out, T_, n_q, d, max_split);
    else
        return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}
