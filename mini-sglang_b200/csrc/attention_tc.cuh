// Prefill attention on the 5th-generation tensor cores (tcgen05), head size 128, bfloat16.
//
// A block owns 128 query rows -- (token, head-in-group) pairs of one kv head, so a GQA group shares
// the keys it reads -- and walks the request's keys in tiles of 128:
//
//     S = Q K^T        tcgen05.mma 128x128x16 (x8 over the head size), Q and K from shared memory,
//                      accumulator in tensor memory (fp32, 128 columns)
//     softmax          thread t owns row t = TMEM lane t.  Two passes over S with tcgen05.ld: the row
//                      maximum, then P = 2^(s*scale - m) rounded to bfloat16 and written back with
//                      tcgen05.st over the columns of S it has consumed (two keys per 32-bit column)
//     O += P V         tcgen05.mma 128x128x16 (x8 over the keys): the A operand P comes from tensor
//                      memory, V from shared memory as it lies in the cache ([key][d]: MN-major B
//                      operand, no transpose); accumulator in tensor memory (128 columns)
//
// Reading an operand from shared memory is what bounds the tensor core here (a 128x128x16 step reads
// 8 KB and takes as long as that read); with P in tensor memory the second product reads half as much,
// the threads store P without swizzle arithmetic or proxy fence, and S and P share their columns.
//
// Roles: warps 0-3 do the softmax, warp 4 gathers Q and the K tiles from the paged cache, warp 5 the
// V tiles, one lane of warp 6 issues the tensor-core work.  They meet only at mbarriers.  A block
// computes S(i), softmax(i), P V(i) one after the other; two blocks share an SM (256 of its 512
// TMEM columns and 97 KB of its shared memory each), so one block's softmax runs beside the
// other's products, and K(i+1), V(i+1) arrive meanwhile.
//
// K, V and Q sit in shared memory in the 128-byte-swizzled layout the tensor core reads through
// matrix descriptors: a [rows x 128] tile is two halves of 64 columns; in a half, row r is 128
// contiguous bytes at r*128 and its 16-byte chunk c is stored at chunk position c ^ (r & 7).
// K and V tiles come by TMA (cp.async.bulk.tensor, 2-d tiled, 128-byte swizzle): the cache is one
// [rows x 128] tensor, a page of a kv head is a run of page_size rows, so a tile is 128 / page_size
// boxes per half, each issued by one lane and all completing on the stage's mbarrier.  V rows past the
// last key a block may see are zeroed afterwards (free cache slots may hold anything, and 0 x NaN
// would spoil O); K rows there only reach masked scores.  Page sizes that are no multiple of 8 (or
// above 128) fall back to cp.async gathers of single rows.  Q is gathered once by all threads.
// When a row's reference maximum moves, O is rescaled in TMEM (load, multiply, store) by the thread
// that owns the row; a warp skips that when none of its rows moved.
//
// Every wait on an mbarrier is bounded; a block that gives up writes a code to p.status, frees its
// TMEM and returns (its output rows are then wrong, which the host reports as an error).
#pragma once
#include "tc_common.cuh"

constexpr int TC_ROWS = 128;      // query rows per block
constexpr int TC_KT = 128;        // keys per tile
constexpr int TC_D = 128;         // head size
constexpr int TC_SOFTMAX_THREADS = 128;    // warps 0-3: one thread per query row
constexpr int TC_THREADS = 224;            // + warp 4: Q/K loader, warp 5: V loader, warp 6: tensor-core issuer
constexpr unsigned TC_QHALF_BYTES = 128u * 128u;           // one 64-column half of the [128 x 128] Q tile
constexpr unsigned TC_Q_BYTES = 2u * TC_QHALF_BYTES;       // 32 KB
constexpr unsigned TC_KHALF_BYTES = (unsigned)TC_KT * 128u;  // one 64-column half of a [128 keys x 128] K or V tile
constexpr unsigned TC_KV_BYTES = 2u * TC_KHALF_BYTES;      // 32 KB
constexpr unsigned TC_SMEM_BYTES = TC_Q_BYTES + 2u * TC_KV_BYTES;    // 96 KB: two blocks per SM
constexpr float TC_LAZY = 16.f;      // the exponent's reference follows the running maximum only past this many powers of two

// byte offset of (row, 16-byte chunk c) inside a swizzled tile whose 64-column halves are `half_bytes` apart
__device__ __forceinline__ unsigned tc_tile_off(int row, int c, unsigned half_bytes) {
    return (unsigned)(c >> 3) * half_bytes + (unsigned)row * 128u + (unsigned)(((c & 7) ^ (row & 7)) << 4);
}

// tma_box: rows of one TMA box (min(page_size, 128)) or 0 for the cp.async gathers
__global__ void __launch_bounds__(TC_THREADS, 2) attn_tc_kernel(const AttnParams p, int* status,
                                                                const __grid_constant__ CUtensorMap kmap,
                                                                const __grid_constant__ CUtensorMap vmap, int tma_box) {
    // No static shared memory: two blocks have to fit an SM.  The first 256 bytes of the dynamic allocation
    // hold the barriers and scalars, the operand tiles start at the next 1024-byte boundary: Q | K | V.
    extern __shared__ __align__(16) unsigned char tc_smem[];
    unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(tc_smem + 128);
    int* sh_tile = reinterpret_cast<int*>(tc_smem + 144);
    const unsigned smem_base = smem_u32(tc_smem);
    const unsigned smem0 = (smem_base + 256u + 1023u) & ~1023u;
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;      // an earlier block gave up: do not pile up
    if (smem0 + TC_SMEM_BYTES > smem_base + TC_SMEM_BYTES + 1024u) {      // allocation not aligned as assumed
        if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 2);
        return;
    }
    const unsigned q_s = smem0, k_s = q_s + TC_Q_BYTES, v_s = k_s + TC_KV_BYTES;
    // mbarriers (8 bytes each); tile i completes phase i of each, so its parity is i & 1
    const unsigned bar_s = smem_base;              // S(i) is in TMEM (tensor core commits)
    const unsigned bar_o = smem_base + 8;          // P V(i) is done: O holds tiles 0..i, P may be overwritten (tensor core commits)
    const unsigned bar_p = smem_base + 16;         // P(i) is in TMEM and O is rescaled (one arrival per softmax warp)
    const unsigned bar_kf = smem_base + 24;        // the K stage holds tile i (TMA: one arrival + bytes; cp.async: 32 lanes)
    const unsigned bar_vf = smem_base + 32;        // the V stage holds tile i
    const unsigned bar_kr = smem_base + 40;        // S(i) has read the K stage (tensor core commits)
    const unsigned bar_vr = smem_base + 48;        // P V(i) has read the V stage (tensor core commits)
    const unsigned bar_q = smem_base + 56;         // Q is in shared memory (all threads)
    const unsigned bar_vt = smem_base + 64;        // TMA copies of a V tile whose tail rows are zeroed afterwards
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int G = p.n_q / p.n_kv;
    const int Gc = G <= TC_ROWS ? G : TC_ROWS;
    const int n_chunks = G <= TC_ROWS ? 1 : (G + TC_ROWS - 1) / TC_ROWS;
    const int QT = G <= TC_ROWS ? TC_ROWS / G : 1;
    // The grid is (kv heads, query tiles): blocks are handed out head-first, so all heads of the heaviest tile
    // start before any lighter tile (with one tile index per blockIdx.x the first heads would take every SM).
    const int kvh = blockIdx.x / n_chunks;
    const int chunk = blockIdx.x - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, QT, ti, sh_tile, (int)blockIdx.y, (int)gridDim.y)) return;
    // key tiles of TC_KT anchored at absolute positions
    const int p_min = ti.kv_len - ti.q_len + ti.t0;
    const int p_max = p_min + ti.n_tok - 1;
    const int k_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt_begin = k_lo / TC_KT, kt_end = p_max / TC_KT + 1;
    const int n_tiles = kt_end - kt_begin;

    if (tid == 0) {
        tc_mbar_init(bar_s, 1); tc_mbar_init(bar_o, 1); tc_mbar_init(bar_p, TC_SOFTMAX_THREADS / 32);
        tc_mbar_init(bar_kf, tma_box > 0 ? 1 : 32); tc_mbar_init(bar_vf, tma_box > 0 ? 1 : 32);
        tc_mbar_init(bar_kr, 1); tc_mbar_init(bar_vr, 1);
        tc_mbar_init(bar_q, TC_THREADS); tc_mbar_init(bar_vt, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // 256 columns of tensor memory: S / P (128) | O (128); two blocks share an SM's 512
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;\n" ::"r"(smem_u32(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_s;
    const unsigned t_s = tmem, t_o = tmem + 128;
    int fail = 0;

    {   // Q: 128 rows x 16 chunks of 16 bytes, spread over all threads; rows without a query are zero-filled
        const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
        for (int idx = tid; idx < TC_ROWS * 16; idx += TC_THREADS) {
            const int r = idx >> 4, c = idx & 15;
            const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * TC_ROWS + hl;
            const bool valid = tl < ti.n_tok && tl < QT && hg < G;
            const __nv_bfloat16* src = qg + ((size_t)(ti.q_base + ti.t0 + (valid ? tl : 0)) * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * TC_D;
            cp_async16_u32(q_s + tc_tile_off(r, c, TC_QHALF_BYTES), src + c * 8, valid);
        }
        tc_cp_async_arrive(bar_q);
    }

    if (warp == 4 || warp == 5) {
        // =========================== loaders: warp 4 brings Q once and the K tiles, warp 5 the V tiles
        const bool is_k = warp == 4;
        const __nv_bfloat16* cache = reinterpret_cast<const __nv_bfloat16*>(is_k ? p.k_cache : p.v_cache);
        const unsigned dst_tile = is_k ? k_s : v_s;
        const unsigned bar_full = is_k ? bar_kf : bar_vf, bar_free = is_k ? bar_kr : bar_vr;
        const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;
#ifdef MSGL_TC_PROFILE
        long long lp[2] = {0, 0};
        long long l0 = clock64(), l1;
#define TC_LMARK(i) { l1 = clock64(); lp[i] += l1 - l0; l0 = l1; }
#else
#define TC_LMARK(i)
#endif
        if (tma_box > 0) {
            // ---- TMA: lane b brings box b (tma_box rows, both 64-column halves) of the tile
            const CUtensorMap* map = is_k ? &kmap : &vmap;
            const int n_box = TC_KT / tma_box;
            unsigned vt_phase = 0;
            for (int j = 0; j < n_tiles; ++j) {
                const int key0 = (kt_begin + j) * TC_KT;
                const int key_b = key0 + lane * tma_box;
                const bool active = lane < n_box && key_b <= p_max;      // boxes past the last visible key are not fetched
                int y = 0;
                if (active) y = (bt[page_index(p, key_b)] * p.n_kv + kvh) * p.page_size + page_slot(p, key_b);
                const unsigned n_act = __popc(__ballot_sync(0xffffffffu, active));
                const bool ragged = !is_k && p_max < key0 + TC_KT - 1;   // V rows past p_max have to be zero
                if (j >= 1 && !tc_mbar_wait(bar_free, (j - 1) & 1)) { fail = 1; break; }    // the tensor core has read tile j-1
                TC_LMARK(0)
                const unsigned bar = ragged ? bar_vt : bar_full;
                if (lane == 0) tc_mbar_expect_tx(bar, n_act * 2u * (unsigned)tma_box * 128u);
                if (active) {
                    const unsigned dst = dst_tile + (unsigned)(lane * tma_box) * 128u;
                    tc_tma_load(dst, map, 0, y, bar);
                    tc_tma_load(dst + TC_KHALF_BYTES, map, 64, y, bar);
                }
                if (ragged) {
                    if (!tc_mbar_wait(bar_vt, vt_phase)) { fail = 1; break; }
                    vt_phase ^= 1u;
                    const int r0 = p_max + 1 - key0;                     // first row without a visible key
                    for (int idx = r0 * 16 + lane; idx < TC_KT * 16; idx += 32) {
                        const unsigned a = dst_tile + (unsigned)((idx >> 3) & 1) * TC_KHALF_BYTES + (unsigned)(idx >> 4) * 128u + (unsigned)(idx & 7) * 16u;
                        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(a), "r"(0u) : "memory");
                    }
                    tc_fence_async_smem();
                    __syncwarp();
                    if (lane == 0) tc_mbar_arrive(bar_full);
                }
                TC_LMARK(1)
            }
        } else {
            // ---- cp.async: lane l gathers rows l, l + 32, l + 64, l + 96 of the tile, sixteen 16-byte chunks each
            auto row_page = [&](int kt, int row) -> int {
                const int key = kt * TC_KT + row;
                return (kt < kt_end && key <= p_max) ? bt[page_index(p, key)] : -1;
            };
            int pg[4], npg[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) pg[h] = row_page(kt_begin, h * 32 + lane);
            for (int j = 0; j < n_tiles; ++j) {
                const int kt = kt_begin + j;
#pragma unroll
                for (int h = 0; h < 4; ++h) npg[h] = row_page(kt + 1, h * 32 + lane);   // next tile's pages, ahead of need
                if (j >= 1 && !tc_mbar_wait(bar_free, (j - 1) & 1)) { fail = 1; break; }
                TC_LMARK(0)
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const int row = h * 32 + lane;
                    const bool valid = pg[h] >= 0;                       // rows past the end are zero-filled
                    size_t off = 0;
                    if (valid) off = (((size_t)pg[h] * p.n_kv + kvh) * p.page_size + page_slot(p, kt * TC_KT + row)) * TC_D;
#pragma unroll
                    for (int c = 0; c < 16; ++c) cp_async16_u32(dst_tile + tc_tile_off(row, c, TC_KHALF_BYTES), cache + off + c * 8, valid);
                }
                tc_cp_async_arrive(bar_full);
#pragma unroll
                for (int h = 0; h < 4; ++h) pg[h] = npg[h];
                TC_LMARK(1)
            }
        }
#ifdef MSGL_TC_PROFILE
        if (status != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && is_k) {
            long long* out_p = reinterpret_cast<long long*>(status) + 30;
            out_p[0] = lp[0]; out_p[1] = lp[1];
        }
#endif
        cp_async_commit();
        cp_async_wait<0>();
    } else if (warp == 6) {
        // =========================== issuer: one lane feeds the tensor core
        if (lane == 0 && n_tiles > 0) {
            const unsigned idesc_s = tc_idesc(false, TC_KT), idesc_o = tc_idesc(true, TC_D);
            // Every operand has one place for the whole block, so the descriptors are built once: a single thread
            // building them between the products would take longer than the products themselves.
            unsigned long long dq[8], dk[8], dv[8];
            unsigned tp_[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                dq[kk] = tc_desc(q_s + (unsigned)(kk >> 2) * TC_QHALF_BYTES + (unsigned)(kk & 3) * 32u, 16, 1024);
                dk[kk] = tc_desc(k_s + (unsigned)(kk >> 2) * TC_KHALF_BYTES + (unsigned)(kk & 3) * 32u, 16, 1024);
                dv[kk] = tc_desc(v_s + (unsigned)kk * 2048u, TC_KHALF_BYTES, 1024);
                tp_[kk] = t_s + (unsigned)kk * 8u;
            }
            bool ok = true;
#ifdef MSGL_TC_PROFILE
            long long ip[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long i0 = clock64(), i1;
#define TC_IMARK(i) { i1 = clock64(); ip[i] += i1 - i0; i0 = i1; }
#else
#define TC_IMARK(i)
#endif
            ok = tc_mbar_wait(bar_q, 0);
            for (int it = 0; it < n_tiles && ok; ++it) {
                ok = tc_mbar_wait(bar_kf, it & 1);
                if (!ok) break;
                TC_IMARK(0)
                tc_fence_async_smem(); tc_fence_after();
                // S(it) = Q K(it)^T: 8 steps of 16 along the head size.  The tensor core works in order, so these run
                // after P V(it-1), which reads P from the columns that S(it) overwrites.
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) tc_mma(t_s, dq[kk], dk[kk], idesc_s, kk > 0 ? 1u : 0u);
                tc_commit(bar_s);
                tc_commit(bar_kr);
                TC_IMARK(1)
                ok = tc_mbar_wait(bar_p, it & 1);
                TC_IMARK(2)
                ok = ok && tc_mbar_wait(bar_vf, it & 1);
                if (!ok) break;
                TC_IMARK(3)
                tc_fence_async_smem(); tc_fence_after();
                // O += P V(it): 8 steps of 16 keys; P from tensor memory (8 columns a step), V as stored (MN-major)
#pragma unroll
                for (int kk = 0; kk < TC_KT / 16; ++kk) tc_mma_ta(t_o, tp_[kk], dv[kk], idesc_o, (it == 0 && kk == 0) ? 0u : 1u);
                tc_commit(bar_o);
                tc_commit(bar_vr);
                TC_IMARK(4)
            }
            if (!ok) fail = 1;
#ifdef MSGL_TC_PROFILE
            if (status != nullptr && blockIdx.x == 0 && blockIdx.y == 0) {
                long long* out_p = reinterpret_cast<long long*>(status) + 22;
                for (int i = 0; i < 8; ++i) out_p[i] = ip[i];
            }
#endif
        }
    } else {
        // =========================== softmax: thread t owns query row t (TMEM lane t)
        const unsigned lane_sel = (unsigned)(warp * 32) << 16;
        const int my_tl = tid / Gc;
        const int my_pos = p_min + my_tl;
        const bool my_valid = my_tl < ti.n_tok && my_tl < QT && (chunk * TC_ROWS + (tid - my_tl * Gc)) < G;
        const float sc = p.scale * 1.4426950408889634f;
        float m_run = -INFINITY, l_run = 0.f;
#ifdef MSGL_TC_PROFILE
        long long tp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long t0 = clock64(), t1;
#define TC_MARK(i) { t1 = clock64(); tp[i] += t1 - t0; t0 = t1; }
#else
#define TC_MARK(i)
#endif
        for (int it = 0; it < n_tiles; ++it) {
            if (!tc_mbar_wait(bar_s, it & 1)) { fail = 1; break; }
            tc_fence_after();
            TC_MARK(0)
            const unsigned ts = t_s + lane_sel;
            const int key0 = (kt_begin + it) * TC_KT;
            const bool need_mask = (key0 + TC_KT - 1 > p_min) || (p.window > 0 && key0 <= p_max - p.window);
            // ---- one pass over S in chunks of 32 columns (the next chunk is on its way while this one is worked on):
            // P = 2^(s*scale - m) against the reference m of the row, which follows the running maximum only when a
            // chunk exceeds it by more than 2^TC_LAZY.  P and the sums then stay far inside the range of bfloat16 and
            // float32, the result is the same softmax, and neither a pass for the maximum nor, after the first
            // chunks, a rescaling is needed.  When the reference does move, the row's sum, its part of O (at the end of
            // the tile) and the chunks of P already written for this tile are scaled by 2^(m_old - m_new).
            float o_scale = 1.f;
            float sa[32], sb[32];
            auto chunk = [&](float (&sv)[32], int cb) {
                if (need_mask) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int key = key0 + cb * 32 + j;
                        bool okk = key <= my_pos;
                        if (p.window > 0) okk = okk && (key > my_pos - p.window);
                        if (!okk) sv[j] = -INFINITY;
                    }
                }
                float c4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
                for (int j = 4; j < 32; ++j) c4[j & 3] = fmaxf(c4[j & 3], sv[j]);
                const float cm = fmaxf(fmaxf(c4[0], c4[1]), fmaxf(c4[2], c4[3])) * sc;
                const bool bump = cm > m_run + TC_LAZY;                  // also the first finite chunk of a row (m_run = -inf)
                if (__any_sync(0xffffffffu, bump)) {                     // TMEM accesses are warp-wide: all lanes go along
                    const float a = bump ? fast_exp2(m_run - cm) : 1.f;  // 0 for the first chunk
                    if (bump) m_run = cm;
                    l_run *= a;
                    o_scale *= a;
                    if (cb > 0) {
                        tc_wait_st();
#pragma unroll 1
                        for (int pc = 0; pc < cb; ++pc) {
                            unsigned pk[16];
                            tc_ld16(ts + pc * 16, pk);
                            tc_wait_ld16(pk);
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                pk[j] = pack_bf16(__uint_as_float(pk[j] << 16) * a, __uint_as_float(pk[j] & 0xffff0000u) * a);
                            tc_st16(ts + pc * 16, pk);
                        }
                    }
                }
                const float mu = (m_run == -INFINITY) ? 0.f : m_run;
                float sum4[4] = {0.f, 0.f, 0.f, 0.f};
                unsigned pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float e0 = fast_exp2(fmaf(sv[j], sc, -mu)), e1 = fast_exp2(fmaf(sv[j + 1], sc, -mu));
                    sum4[(j >> 1) & 3] += e0 + e1;
                    pk[j >> 1] = pack_bf16(e0, e1);
                }
                l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                tc_st16(ts + cb * 16, pk);             // columns [16 cb, 16 cb + 16): S columns below 32 (cb + 1) are consumed
            };
            tc_ld32(ts, sa);
            tc_wait_ld(sa);
            tc_ld32(ts + 32, sb);
            chunk(sa, 0);
            tc_wait_ld(sb);
            tc_ld32(ts + 64, sa);
            chunk(sb, 1);                              // writes columns 16..31: chunk 1 is in registers, chunk 2 (64..95) on its way
            tc_wait_ld(sa);
            tc_ld32(ts + 96, sb);
            chunk(sa, 2);
            tc_wait_ld(sb);
            chunk(sb, 3);
            TC_MARK(1)
            // ---- O of the tiles before: rescale where a reference moved.  A warp owns its 32 rows (TMEM lanes), so
            // it decides alone.  (P V(it-1) is done: S(it) came after it.)
            if (it >= 1 && __any_sync(0xffffffffu, o_scale != 1.f)) {
#pragma unroll 1
                for (int cb = 0; cb < 4; ++cb) {
                    float v0[32];
                    tc_ld32(t_o + lane_sel + cb * 32, v0);
                    tc_wait_ld(v0);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v0[j] *= o_scale;
                    tc_st32(t_o + lane_sel + cb * 32, v0);
                }
            }
            TC_MARK(2)
            TC_MARK(3)
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(bar_p);
            TC_MARK(4)
        }
#ifdef MSGL_TC_PROFILE
        if (status != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (tid == 0 || tid == 37)) {
            long long* out_p = reinterpret_cast<long long*>(status) + 2 + (tid ? 10 : 0);
            for (int i = 0; i < 8; ++i) out_p[i] = tp[i];
            out_p[8] = n_tiles;
        }
#endif
        // epilogue: the last P V product, normalise, write
        if (!fail && n_tiles > 0) {
            if (!tc_mbar_wait(bar_o, (n_tiles - 1) & 1)) fail = 1;
            tc_fence_after();
        }
        if (!__any_sync(0xffffffffu, fail) && n_tiles > 0) {
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            const int hl = tid - my_tl * Gc;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) +
                                 ((size_t)(ti.q_base + ti.t0 + (my_valid ? my_tl : 0)) * p.n_q + (size_t)kvh * G + (my_valid ? chunk * TC_ROWS + hl : 0)) * TC_D;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                float v[32];
                tc_ld32(t_o + lane_sel + cb * 32, v);                    // every thread of the warp takes part
                tc_wait_ld(v);
                if (my_valid) {
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        uint4 pk;
                        pk.x = pack_bf16(v[j] * inv, v[j + 1] * inv);
                        pk.y = pack_bf16(v[j + 2] * inv, v[j + 3] * inv);
                        pk.z = pack_bf16(v[j + 4] * inv, v[j + 5] * inv);
                        pk.w = pack_bf16(v[j + 6] * inv, v[j + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + cb * 32 + j) = pk;
                    }
                }
            }
        }
    }
    tc_fence_before();
    const bool failed = __syncthreads_or(fail) != 0;
    if (failed && status != nullptr && tid == 0) atomicExch(status, 1);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;\n" ::"r"(tmem) : "memory");
}
