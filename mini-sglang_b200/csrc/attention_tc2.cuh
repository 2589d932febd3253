// Prefill attention on tcgen05 with two query tiles per block in ping-pong (head size 128, bfloat16,
// page sizes that TMA can fetch).  Uses the helpers of attention_tc.cuh.
//
// A block owns 256 query rows of one kv head: tile A (rows 0..127) and tile B (rows 128..255), each
// (token, head-in-group) pairs of consecutive tokens, and walks the keys in tiles of 128.  It is
// alone on its SM: all 512 columns of tensor memory (S_A | S_B | O_A | O_B, 128 each) and 193 KB
// of shared memory (Q_A, Q_B and two stages each of K and V, which both tiles share).
//
// The exponentials of a 128 x 128 tile keep the special-function unit busy for about as long as its
// two products keep the tensor core busy, so the two have to run side by side all the time.  One
// thread issues the products in the order
//
//     S_A(j)   P V_B(j-1)   S_B(j)   P V_A(j)   S_A(j+1)   ...
//
// (S_X = Q_X K^T into tensor memory; P V_X accumulates O_X with P_X read from tensor memory), and two
// groups of four warps do the softmax of tile A and of tile B, one thread a row with the row's 128
// scores in registers: while group A works on S_A(j) the tensor core has P V_B(j-1) and S_B(j)
// to do, while group B works on S_B(j) it has P V_A(j) and S_A(j+1).  P_X overwrites S_X, so
// S_X(j+1) is issued after P V_X(j); the tensor core executes in order.
//
// Warps: 0-3 softmax A, 4-7 softmax B, 8 K loader, 9 V loader (TMA, see attention_tc.cuh), 10 issuer,
// 11 idle after the Q gather.  All waits are bounded as in attention_tc.cuh.
#pragma once

// two float32 values in one 64-bit register, for the packed float32 instructions of sm_100
__device__ __forceinline__ unsigned long long f2_pack(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

constexpr int TC2_ROWS = 256;               // query rows per block (two tiles of 128)
constexpr int TC2_THREADS = 384;
constexpr unsigned TC2_SMEM_BYTES = 2u * TC_Q_BYTES + 4u * TC_KV_BYTES;      // 192 KB
constexpr unsigned TC2_SMEM_ALLOC = TC2_SMEM_BYTES + 256u + 1024u;

__global__ void __launch_bounds__(TC2_THREADS, 1) attn_tc2_kernel(const AttnParams p, int* status,
                                                                  const __grid_constant__ CUtensorMap kmap,
                                                                  const __grid_constant__ CUtensorMap vmap, int tma_box) {
    extern __shared__ __align__(16) unsigned char tc_smem[];
    unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(tc_smem + 192);
    int* sh_tile = reinterpret_cast<int*>(tc_smem + 208);
    const unsigned smem_base = smem_u32(tc_smem);
    const unsigned smem0 = (smem_base + 256u + 1023u) & ~1023u;
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;      // an earlier block gave up: do not pile up
    if (smem0 + TC2_SMEM_BYTES > smem_base + TC2_SMEM_ALLOC) {            // allocation not aligned as assumed
        if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 2);
        return;
    }
    const unsigned q_s = smem0, k_s = q_s + 2u * TC_Q_BYTES, v_s = k_s + 2u * TC_KV_BYTES;
    // mbarriers (8 bytes each).  Per tile X in {A, B}: tile j completes phase j of bar_s, bar_p, bar_o.
    auto bar_s = [&](int x) { return smem_base + 8u * (unsigned)x; };              // S_X(j) is in TMEM (tensor core commits)
    auto bar_p = [&](int x) { return smem_base + 16u + 8u * (unsigned)x; };        // P_X(j) is in TMEM, O_X rescaled (4 softmax warps)
    auto bar_o = [&](int x) { return smem_base + 32u + 8u * (unsigned)x; };        // P V_X(j) is done (tensor core commits)
    auto bar_kf = [&](int st) { return smem_base + 48u + 8u * (unsigned)st; };     // K stage holds a tile (TMA bytes)
    auto bar_kr = [&](int st) { return smem_base + 64u + 8u * (unsigned)st; };     // both S products have read the K stage
    auto bar_vf = [&](int st) { return smem_base + 80u + 8u * (unsigned)st; };     // V stage holds a tile
    auto bar_vr = [&](int st) { return smem_base + 96u + 8u * (unsigned)st; };     // both P V products have read the V stage
    const unsigned bar_q = smem_base + 112u;                                        // Q is in shared memory (all threads)
    const unsigned bar_vt = smem_base + 120u;                                       // TMA copies of a V tile whose tail rows are zeroed afterwards
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int G = p.n_q / p.n_kv;
    const int Gc = G <= TC_ROWS ? G : TC_ROWS;
    const int n_chunks = G <= TC_ROWS ? 1 : (G + TC_ROWS - 1) / TC_ROWS;
    const int QH = G <= TC_ROWS ? TC_ROWS / G : 1;             // tokens of one 128-row tile
    // The grid is (kv heads, query tiles): blocks are handed out head-first, so all heads of the heaviest tile
    // start before any lighter tile (with one tile index per blockIdx.x the first heads would take every SM).
    const int kvh = blockIdx.x / n_chunks;
    const int chunk = blockIdx.x - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, 2 * QH, ti, sh_tile, (int)blockIdx.y, (int)gridDim.y)) return;
    // positions of the block's tokens and its key tiles (anchored at absolute positions)
    const int p_min = ti.kv_len - ti.q_len + ti.t0;
    const int p_max = p_min + ti.n_tok - 1;
    const int ntok_a = min(ti.n_tok, QH), ntok_b = ti.n_tok - ntok_a;
    const int pmax_a = p_min + ntok_a - 1;
    const int k_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt_begin = k_lo / TC_KT;
    const int n_a = pmax_a / TC_KT + 1 - kt_begin;                        // key tiles of tile A
    const int n_b = ntok_b > 0 ? p_max / TC_KT + 1 - kt_begin : 0;         // key tiles of tile B (0: no token there)
    const int n_tiles = max(n_a, n_b);

    if (tid == 0) {
        for (int x = 0; x < 2; ++x) {
            tc_mbar_init(bar_s(x), 1); tc_mbar_init(bar_p(x), 4); tc_mbar_init(bar_o(x), 1);
            tc_mbar_init(bar_kf(x), 1); tc_mbar_init(bar_kr(x), 1); tc_mbar_init(bar_vf(x), 1); tc_mbar_init(bar_vr(x), 1);
        }
        tc_mbar_init(bar_q, TC2_THREADS); tc_mbar_init(bar_vt, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // all 512 columns of tensor memory: S_A | S_B | O_A | O_B
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(smem_u32(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_s;
    int fail = 0;

    {   // Q: 256 rows x 16 chunks of 16 bytes, spread over all threads; rows without a query are zero-filled
        const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
        for (int idx = tid; idx < TC2_ROWS * 16; idx += TC2_THREADS) {
            const int r = idx >> 4, c = idx & 15;
            const int x = r >> 7, rr = r & 127;
            const int tl = x * QH + rr / Gc, hl = rr % Gc, hg = chunk * TC_ROWS + hl;
            const bool valid = rr / Gc < QH && tl < ti.n_tok && hg < G;
            const __nv_bfloat16* src = qg + ((size_t)(ti.q_base + ti.t0 + (valid ? tl : 0)) * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * TC_D;
            cp_async16_u32(q_s + (unsigned)x * TC_Q_BYTES + tc_tile_off(rr, c, TC_QHALF_BYTES), src + c * 8, valid);
        }
        tc_cp_async_arrive(bar_q);
    }

    if (warp == 8 || warp == 9) {
        // =========================== loaders: warp 8 brings the K tiles, warp 9 the V tiles; lane b brings box b
        const bool is_k = warp == 8;
        const CUtensorMap* map = is_k ? &kmap : &vmap;
        const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;
        const int n_box = TC_KT / tma_box;
        unsigned vt_phase = 0;
        auto box_row = [&](int j) -> int {            // first cache row of this lane's box of tile j, or -1
            const int key_b = (kt_begin + j) * TC_KT + lane * tma_box;
            if (j >= n_tiles || lane >= n_box || key_b > p_max) return -1;          // boxes past the last visible key are not fetched
            return (bt[page_index(p, key_b)] * p.n_kv + kvh) * p.page_size + page_slot(p, key_b);
        };
        int y = box_row(0);
        for (int j = 0; j < n_tiles; ++j) {
            const int st = j & 1;
            const int y_next = box_row(j + 1);                                    // looked up a tile ahead
            const int key0 = (kt_begin + j) * TC_KT;
            const unsigned dst_tile = (is_k ? k_s : v_s) + (unsigned)st * TC_KV_BYTES;
            const unsigned n_act = __popc(__ballot_sync(0xffffffffu, y >= 0));
            const bool ragged = !is_k && p_max < key0 + TC_KT - 1;               // V rows past p_max have to be zero
            if (j >= 2 && !tc_mbar_wait(is_k ? bar_kr(st) : bar_vr(st), ((j >> 1) - 1) & 1)) { fail = 1; break; }   // tile j-2 has been read
            const unsigned bar = ragged ? bar_vt : (is_k ? bar_kf(st) : bar_vf(st));
            if (lane == 0) tc_mbar_expect_tx(bar, n_act * 2u * (unsigned)tma_box * 128u);
            if (y >= 0) {
                const unsigned dst = dst_tile + (unsigned)(lane * tma_box) * 128u;
                tc_tma_load(dst, map, 0, y, bar);
                tc_tma_load(dst + TC_KHALF_BYTES, map, 64, y, bar);
            }
            if (ragged) {
                if (!tc_mbar_wait(bar_vt, vt_phase)) { fail = 1; break; }
                vt_phase ^= 1u;
                const int r0 = p_max + 1 - key0;                                 // first row without a visible key
                for (int idx = r0 * 16 + lane; idx < TC_KT * 16; idx += 32) {
                    const unsigned a = dst_tile + (unsigned)((idx >> 3) & 1) * TC_KHALF_BYTES + (unsigned)(idx >> 4) * 128u + (unsigned)(idx & 7) * 16u;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(a), "r"(0u) : "memory");
                }
                tc_fence_async_smem();
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(bar_vf(st));
            }
            y = y_next;
        }
    } else if (warp == 10) {
        // =========================== issuer: one lane feeds the tensor core
        if (lane == 0 && n_tiles > 0) {
            const unsigned idesc_s = tc_idesc(false, TC_KT), idesc_o = tc_idesc(true, TC_D);
            // Q's descriptors and P's addresses are fixed; K's and V's differ between the two stages by a constant
            // in the address field.  A single thread building descriptors between the products would take longer
            // than the products themselves.
            unsigned long long dq[2][8], dk[8], dv[8];
            unsigned tp_[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const unsigned qo = (unsigned)(kk >> 2) * TC_QHALF_BYTES + (unsigned)(kk & 3) * 32u;
                dq[0][kk] = tc_desc(q_s + qo, 16, 1024);
                dq[1][kk] = tc_desc(q_s + TC_Q_BYTES + qo, 16, 1024);
                dk[kk] = tc_desc(k_s + (unsigned)(kk >> 2) * TC_KHALF_BYTES + (unsigned)(kk & 3) * 32u, 16, 1024);
                dv[kk] = tc_desc(v_s + (unsigned)kk * 2048u, TC_KHALF_BYTES, 1024);
                tp_[kk] = (unsigned)kk * 8u;
            }
            const unsigned long long stage_step = (unsigned long long)(TC_KV_BYTES >> 4);     // address field counts 16-byte units
            auto issue_s = [&](int x, int j) {                            // S_X(j) = Q_X K(j)^T: 8 steps of 16 along the head size
                const unsigned long long ks = (j & 1) ? stage_step : 0ull;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) tc_mma(tmem + (unsigned)x * 128u, dq[x][kk], dk[kk] + ks, idesc_s, kk > 0 ? 1u : 0u);
                tc_commit(bar_s(x));
            };
            auto issue_o = [&](int x, int j) {                            // O_X += P_X V(j): 8 steps of 16 keys, P from tensor memory
                const unsigned long long vs = (j & 1) ? stage_step : 0ull;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    tc_mma_ta(tmem + 256u + (unsigned)x * 128u, tmem + (unsigned)x * 128u + tp_[kk], dv[kk] + vs, idesc_o, (j == 0 && kk == 0) ? 0u : 1u);
                tc_commit(bar_o(x));
            };
            bool ok = tc_mbar_wait(bar_q, 0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = tc_mbar_wait(bar_kf(j & 1), (j >> 1) & 1);
                if (!ok) break;
                tc_fence_async_smem(); tc_fence_after();
                if (j < n_a) issue_s(0, j);
                if (j >= 1) {
                    if (j - 1 < n_b) {
                        ok = tc_mbar_wait(bar_p(1), (j - 1) & 1) && tc_mbar_wait(bar_vf((j - 1) & 1), ((j - 1) >> 1) & 1);
                        if (!ok) break;
                        tc_fence_async_smem(); tc_fence_after();
                        issue_o(1, j - 1);
                    }
                    tc_commit(bar_vr((j - 1) & 1));                       // P V_A(j-1) and P V_B(j-1) have been issued
                }
                if (j < n_b) issue_s(1, j);
                tc_commit(bar_kr(j & 1));
                if (j < n_a) {
                    ok = tc_mbar_wait(bar_p(0), j & 1) && tc_mbar_wait(bar_vf(j & 1), (j >> 1) & 1);
                    if (!ok) break;
                    tc_fence_async_smem(); tc_fence_after();
                    issue_o(0, j);
                }
            }
            if (ok && n_tiles - 1 < n_b) {
                const int j = n_tiles - 1;
                ok = tc_mbar_wait(bar_p(1), j & 1) && tc_mbar_wait(bar_vf(j & 1), (j >> 1) & 1);
                if (ok) { tc_fence_async_smem(); tc_fence_after(); issue_o(1, j); }
            }
            if (!ok) fail = 1;
        }
    } else if (warp < 8) {
        // =========================== softmax: group x = warp / 4 owns tile x; thread r of the group owns its row r
        const int x = warp >> 2, row = tid & 127;
        const int n_mine = x ? n_b : n_a;
        const unsigned lane_sel = (unsigned)((warp & 3) * 32) << 16;
        const unsigned ts = tmem + (unsigned)x * 128u + lane_sel, to = tmem + 256u + (unsigned)x * 128u + lane_sel;
        const int my_tl = x * QH + row / Gc;
        const int my_pos = p_min + my_tl;
        const bool my_valid = row / Gc < QH && my_tl < ti.n_tok && (chunk * TC_ROWS + row % Gc) < G;
        const int pmin_x = p_min + x * QH, pmax_x = x ? p_max : pmax_a;
        const float sc = p.scale * 1.4426950408889634f;
        float m_run = -INFINITY, l_run = 0.f, o_scale = 1.f;
#ifdef MSGL_TC_PROFILE
        long long tp[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long t0 = clock64(), t1;
#define TC2_MARK(i) { t1 = clock64(); tp[i] += t1 - t0; t0 = t1; }
#else
#define TC2_MARK(i)
#endif
        for (int it = 0; it < n_mine; ++it) {
            if (!tc_mbar_wait(bar_s(x), it & 1)) { fail = 1; break; }
            tc_fence_after();
            TC2_MARK(0)
            const int key0 = (kt_begin + it) * TC_KT;
            const bool need_mask = (key0 + TC_KT - 1 > pmin_x) || (p.window > 0 && key0 <= pmax_x - p.window);
            float s0[32], s1[32], s2[32], s3[32];
            tc_ld32(ts, s0); tc_ld32(ts + 32, s1); tc_ld32(ts + 64, s2); tc_ld32(ts + 96, s3);
            tc_wait_ld(s0); tc_wait_ld(s1); tc_wait_ld(s2); tc_wait_ld(s3);
            TC2_MARK(1)
            if (need_mask) {
                auto mask = [&](float (&sv)[32], int cb) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int key = key0 + cb * 32 + j;
                        bool okk = key <= my_pos;
                        if (p.window > 0) okk = okk && (key > my_pos - p.window);
                        if (!okk) sv[j] = -INFINITY;
                    }
                };
                mask(s0, 0); mask(s1, 1); mask(s2, 2); mask(s3, 3);
            }
            // The reference m of a row's exponentials need not be its maximum: any m that keeps 2^(s*scale - m) inside
            // the range of bfloat16 and float32 gives the same softmax.  So the maximum is only looked for where a row
            // has no reference yet (its first tile) or where the sum of a tile shows that the reference had fallen behind
            // by so much that the exponentials overflowed (then the tile is done again); a sum above 2^TC_LAZY moves
            // the reference by that sum's logarithm for the tiles to come.  Whenever the reference moves, the row's
            // sum is scaled at once and its part of O before the next product is added.
            auto row_max = [&]() -> float {
                float c8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) c8[j] = fmaxf(fmaxf(s0[j], s1[j]), fmaxf(s2[j], s3[j]));
#pragma unroll
                for (int j = 8; j < 32; ++j) c8[j & 7] = fmaxf(c8[j & 7], fmaxf(fmaxf(s0[j], s1[j]), fmaxf(s2[j], s3[j])));
                return fmaxf(fmaxf(fmaxf(c8[0], c8[1]), fmaxf(c8[2], c8[3])), fmaxf(fmaxf(c8[4], c8[5]), fmaxf(c8[6], c8[7]))) * sc;
            };
            auto move_reference = [&](float m_new) {                      // m_new > m_run (or the first finite one)
                const float a = fast_exp2(m_run - m_new);                // 0 for the first
                m_run = m_new;
                l_run *= a;
                o_scale *= a;
            };
            if (__any_sync(0xffffffffu, m_run == -INFINITY)) {
                const float cm = row_max();
                if (m_run == -INFINITY && cm > -INFINITY) move_reference(cm);
            }
            // O of the tiles before: a warp owns its 32 rows (TMEM lanes), so it decides alone.  (P V(it-1) is
            // done: S(it) was issued after it.)
            auto rescale_o = [&]() {
                if (it >= 1 && __any_sync(0xffffffffu, o_scale != 1.f)) {
#pragma unroll 1
                    for (int cb = 0; cb < 4; ++cb) {
                        float v0[32];
                        tc_ld32(to + cb * 32, v0);
                        tc_wait_ld(v0);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v0[j] *= o_scale;
                        tc_st32(to + cb * 32, v0);
                    }
                }
                o_scale = 1.f;
            };
            rescale_o();
            TC2_MARK(2)
            float tile_sum;
            auto exponentials = [&]() {
                // two neighbouring scores at a time through the packed float32 instructions (fma.rn.f32x2, add.rn.f32x2): the
                // softmax warps are bound by the number of instructions they issue, and these halve the multiply-adds and adds
                const float mu = (m_run == -INFINITY) ? 0.f : m_run;
                const unsigned long long sc2 = f2_pack(sc, sc), nmu2 = f2_pack(-mu, -mu);
                unsigned long long sum2[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) sum2[j] = 0ull;                  // (0.f, 0.f)
                auto expo = [&](const float (&sv)[32], int cb) {
                    unsigned pk[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float x0, x1;
                        f2_unpack(f2_fma(f2_pack(sv[j], sv[j + 1]), sc2, nmu2), x0, x1);
                        const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
                        sum2[(j >> 1) & 7] = f2_add(sum2[(j >> 1) & 7], f2_pack(e0, e1));
                        pk[j >> 1] = pack_bf16(e0, e1);
                    }
                    tc_st16(ts + cb * 16, pk);         // P columns [16 cb, 16 cb + 16); the row's scores are all in registers
                };
                expo(s0, 0); expo(s1, 1); expo(s2, 2); expo(s3, 3);
                const unsigned long long t4 = f2_add(f2_add(f2_add(sum2[0], sum2[1]), f2_add(sum2[2], sum2[3])),
                                                     f2_add(f2_add(sum2[4], sum2[5]), f2_add(sum2[6], sum2[7])));
                float lo, hi;
                f2_unpack(t4, lo, hi);
                tile_sum = lo + hi;
            };
            exponentials();
            if (__any_sync(0xffffffffu, !(tile_sum < 1.0e30f))) {        // overflow (inf, or nan from inf - inf): again, from the maximum
                const float cm = row_max();
                if (cm > m_run) move_reference(cm);
                rescale_o();
                tc_wait_st();
                exponentials();
            }
            l_run += tile_sum;
            if (tile_sum > 65536.f) move_reference(m_run + log2f(tile_sum));     // 2^TC_LAZY; takes effect with the next tile (O: before its product)
            TC2_MARK(3)
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(bar_p(x));
            TC2_MARK(4)
        }
#ifdef MSGL_TC_PROFILE
        if (status != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (tid == 0 || tid == 128)) {
            long long* out_p = reinterpret_cast<long long*>(status) + 2 + (tid ? 10 : 0);
            for (int i = 0; i < 8; ++i) out_p[i] = tp[i];
            out_p[8] = n_mine;
        }
#endif
        // epilogue: the last P V product, normalise, write
        if (!fail && n_mine > 0) {
            if (!tc_mbar_wait(bar_o(x), (n_mine - 1) & 1)) fail = 1;
            tc_fence_after();
        }
        if (!__any_sync(0xffffffffu, fail) && n_mine > 0) {
            const float inv = l_run > 0.f ? o_scale / l_run : 0.f;        // o_scale: a move of the reference after the last tile
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) +
                                 ((size_t)(ti.q_base + ti.t0 + (my_valid ? my_tl : 0)) * p.n_q + (size_t)kvh * G + (my_valid ? chunk * TC_ROWS + row % Gc : 0)) * TC_D;
#pragma unroll 1
            for (int cb = 0; cb < 4; ++cb) {
                float v[32];
                tc_ld32(to + cb * 32, v);                                // every thread of the warp takes part
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
    cp_async_commit();
    cp_async_wait<0>();
    tc_fence_before();
    const bool failed = __syncthreads_or(fail) != 0;
    if (failed && status != nullptr && tid == 0) atomicExch(status, 1);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}
