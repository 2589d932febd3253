// Prefill attention on the 5th-generation tensor cores (tcgen05), head size 128, bfloat16.
//
// A block owns 128 query rows -- (token, head-in-group) pairs of one kv head, so a GQA group shares
// the keys it reads -- and walks the request's keys in tiles of 128:
//
//     S = Q K^T        tcgen05.mma 128x128x16 (x8 over the head size), accumulator in TMEM (fp32)
//     softmax          thread t owns row t = TMEM lane t: tcgen05.ld, running maximum and sum in
//                      registers (no shuffles), P = 2^(s*scale - m) rounded to bfloat16 into shared memory
//     O += P V         tcgen05.mma 128x128x16 (x8 over the keys), accumulator in TMEM; V is used as it
//                      lies in the cache ([key][d]: MN-major B operand), no transpose
//
// Operands sit in shared memory in the 128-byte-swizzled layout the tensor core reads through
// matrix descriptors: a [rows x 128] tile is two halves of 64 columns; in a half, row r is 128
// contiguous bytes at r*128 and its 16-byte chunk c is stored at chunk position c ^ (r & 7).  K and
// V rows are gathered from the paged cache with cp.async straight into that layout (any page size).
// S is double-buffered in TMEM, so the tensor core computes the next tile's scores while the
// threads are busy with this tile's softmax.  When a row's reference maximum moves, O is rescaled in TMEM
// (load, multiply, store) by the thread that owns the row; the block skips that when no row moved.
//
// Every wait on an mbarrier is bounded; a block that gives up writes a code to p.status, frees its
// TMEM and returns (its output rows are then wrong, which the host reports as an error).
#pragma once

constexpr int TC_ROWS = 128;      // query rows per block
constexpr int TC_KT = 64;         // keys per tile
constexpr int TC_D = 128;         // head size
constexpr int TC_THREADS = 128;
constexpr unsigned TC_QHALF_BYTES = 128u * 128u;           // one 64-column half of the [128 x 128] Q tile
constexpr unsigned TC_Q_BYTES = 2u * TC_QHALF_BYTES;       // 32 KB
constexpr unsigned TC_KHALF_BYTES = (unsigned)TC_KT * 128u;  // one 64-column half of a [64 keys x 128] K or V tile
constexpr unsigned TC_KV_BYTES = 2u * TC_KHALF_BYTES;      // 16 KB
constexpr unsigned TC_P_BYTES = 128u * 128u;               // P: [128 rows x 64 keys] = one half, 16 KB
constexpr unsigned TC_SMEM_BYTES = TC_Q_BYTES + 4u * TC_KV_BYTES + TC_P_BYTES;    // 112 KB: two blocks per SM
constexpr long long TC_SPIN_LIMIT = 20000000LL;            // polls of an mbarrier before a block gives up

__device__ __forceinline__ void tc_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ bool tc_mbar_wait(unsigned bar, unsigned parity) {
    for (long long it = 0; it < TC_SPIN_LIMIT; ++it) {
        unsigned done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tc_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4), version 1, 128-byte swizzle
__device__ __forceinline__ unsigned long long tc_desc(unsigned saddr, unsigned lbo_bytes, unsigned sbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((saddr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;                     // descriptor version of sm_100
    d |= 2ull << 61;                     // SWIZZLE_128B
    return d;
}

// instruction descriptor, kind::f16: D fp32, A and B bfloat16, M = 128, N = n; b_mn: B is MN-major
__device__ __forceinline__ unsigned tc_idesc(bool b_mn, unsigned n) {
    unsigned d = 0;
    d |= 1u << 4;                        // D format: F32
    d |= 1u << 7;                        // A format: BF16
    d |= 1u << 10;                       // B format: BF16
    d |= (b_mn ? 1u : 0u) << 16;         // B major: 0 = K, 1 = MN
    d |= (n >> 3) << 17;                 // N
    d |= (128u >> 4) << 24;              // M
    return d;
}

__device__ __forceinline__ void tc_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                       unsigned idesc, unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st32(unsigned taddr, const float (&v)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};\n"
                 ::"r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])),
                   "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// byte offset of (row, 16-byte chunk c) inside a swizzled tile whose 64-column halves are `half_bytes` apart
__device__ __forceinline__ unsigned tc_tile_off(int row, int c, unsigned half_bytes) {
    return (unsigned)(c >> 3) * half_bytes + (unsigned)row * 128u + (unsigned)(((c & 7) ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(TC_THREADS, 2) attn_tc_kernel(const AttnParams p, int* status) {
    // No static shared memory: two blocks have to fit an SM, and every byte of its 228 KB counts.  The first 64
    // bytes of the dynamic allocation hold the barriers and scalars, the operand tiles start at the next
    // 1024-byte boundary: Q | K0 | K1 | V0 | V1 | P.
    extern __shared__ __align__(16) unsigned char tc_smem[];
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(tc_smem);            // S0 done, S1 done, O done, (spare)
    unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(tc_smem + 32);
    int* sh_tile = reinterpret_cast<int*>(tc_smem + 48);
    const unsigned smem0 = (smem_u32(tc_smem) + 64u + 1023u) & ~1023u;
    if (smem0 + TC_SMEM_BYTES > smem_u32(tc_smem) + TC_SMEM_BYTES + 1024u) {      // allocation not aligned as assumed
        if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 2);
        return;
    }
    const unsigned q_s = smem0, k_s = q_s + TC_Q_BYTES, v_s = k_s + 2 * TC_KV_BYTES, p_s = v_s + 2 * TC_KV_BYTES;
    const int tid = threadIdx.x, warp = tid >> 5;

    const int G = p.n_q / p.n_kv;
    const int Gc = G <= TC_ROWS ? G : TC_ROWS;
    const int n_chunks = G <= TC_ROWS ? 1 : (G + TC_ROWS - 1) / TC_ROWS;
    const int QT = G <= TC_ROWS ? TC_ROWS / G : 1;
    const int kvh = blockIdx.y / n_chunks;
    const int chunk = blockIdx.y - kvh * n_chunks;

    TileInfo ti;
    if (!find_tile(p, QT, ti, sh_tile)) return;
    // key tiles of TC_KT anchored at absolute positions
    const int p_min = ti.kv_len - ti.q_len + ti.t0;
    const int p_max = p_min + ti.n_tok - 1;
    const int k_lo = p.window > 0 ? max(0, p_min - p.window + 1) : 0;
    const int kt_begin = k_lo / TC_KT, kt_end = p_max / TC_KT + 1;
    const int n_tiles = kt_end - kt_begin;

    const unsigned bar_s0 = smem_u32(&bars[0]), bar_s1 = smem_u32(&bars[1]), bar_o = smem_u32(&bars[2]);
    if (tid == 0) {
        tc_mbar_init(bar_s0, 1);
        tc_mbar_init(bar_s1, 1);
        tc_mbar_init(bar_o, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // 256 columns of tensor memory: S0 (64) | S1 (64) | O (128); two blocks share an SM's 512
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;\n" ::"r"(smem_u32(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_s;
    const unsigned lane_sel = (unsigned)(warp * 32) << 16;          // this warp's quarter of the 128 lanes
    const unsigned t_s0 = tmem, t_s1 = tmem + 64, t_o = tmem + 128;

    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
    const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
    const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
    const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;

    // ---- Q rows -> swizzled tile (thread t copies row t: 16 chunks)
    {
        const int r = tid;
        const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * TC_ROWS + hl;
        const bool valid = tl < ti.n_tok && tl < QT && hg < G;
        const __nv_bfloat16* src = qg + ((size_t)(ti.q_base + ti.t0 + (valid ? tl : 0)) * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * TC_D;
#pragma unroll
        for (int c = 0; c < 16; ++c) cp_async16_u32(q_s + tc_tile_off(r, c, TC_QHALF_BYTES), src + c * 8, valid);
    }
    // two threads copy a key row of a tile (thread t: row t / 2, chunks 8 (t & 1) ..); K and V are separate
    // copies because their buffers come free at different times (K after S of the tile, V after its P V product)
    const int ld_row = tid >> 1, ld_c0 = (tid & 1) * 8;
    auto tile_page = [&](int kt) -> int {
        const int key = kt * TC_KT + ld_row;
        return (kt >= kt_begin && kt < kt_end && key <= p_max) ? bt[page_index(p, key)] : -1;
    };
    auto load_rows = [&](unsigned dst_tile, const __nv_bfloat16* cache, int kt, int pg) {
        const int key = kt * TC_KT + ld_row;
        const bool valid = pg >= 0;
        size_t off = 0;
        if (valid) off = (((size_t)pg * p.n_kv + kvh) * p.page_size + page_slot(p, key)) * TC_D;
#pragma unroll
        for (int c = 0; c < 8; ++c)
            cp_async16_u32(dst_tile + tc_tile_off(ld_row, ld_c0 + c, TC_KHALF_BYTES), cache + off + (ld_c0 + c) * 8, valid);
    };

    const unsigned idesc_s = tc_idesc(false, TC_KT), idesc_o = tc_idesc(true, TC_D);
    // S = Q K^T for the K tile in `stage` into S buffer `buf`: 8 steps of 16 along the head size
    auto issue_s = [&](int stage, int buf) {
        const unsigned kb = k_s + (unsigned)stage * TC_KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            const unsigned qo = (unsigned)(kk >> 2) * TC_QHALF_BYTES + (unsigned)(kk & 3) * 32u;
            const unsigned ko = (unsigned)(kk >> 2) * TC_KHALF_BYTES + (unsigned)(kk & 3) * 32u;
            tc_mma(buf ? t_s1 : t_s0, tc_desc(q_s + qo, 16, 1024), tc_desc(kb + ko, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(buf ? bar_s1 : bar_s0);
    };
    // O += P V: 4 steps of 16 keys; V is the B operand as stored (MN-major): its halves are 64 columns of d
    auto issue_o = [&](int stage, bool first) {
        const unsigned vb = v_s + (unsigned)stage * TC_KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < TC_KT / 16; ++kk) {
            const unsigned pa = p_s + (unsigned)kk * 32u;                       // P: K-major over the 64 keys
            const unsigned vbk = vb + (unsigned)kk * 16u * 128u;                // 16 keys further down
            tc_mma(t_o, tc_desc(pa, 16, 1024), tc_desc(vbk, TC_KHALF_BYTES, 1024), idesc_o, (first && kk == 0) ? 0u : 1u);
        }
        tc_commit(bar_o);
    };

    const int my_tl = tid / Gc;
    const int my_pos = p_min + my_tl;                                  // position of this row's query
    const bool my_valid = my_tl < ti.n_tok && my_tl < QT && (chunk * TC_ROWS + (tid - my_tl * Gc)) < G;
    const float sc = p.scale * 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    int fail = 0;
    unsigned par_s[2] = {0u, 0u}, par_o = 0u;

    // prologue: {Q, K(0)}, {K(1)}, {V(0)} as three copy groups; S(0) as soon as the first has landed
    load_rows(k_s, kc, kt_begin, tile_page(kt_begin));
    cp_async_commit();
    load_rows(k_s + TC_KV_BYTES, kc, kt_begin + 1, tile_page(kt_begin + 1));
    cp_async_commit();
    load_rows(v_s, vc, kt_begin, tile_page(kt_begin));
    cp_async_commit();
    int pg_k = tile_page(kt_begin + 2);            // page of this thread's row in the next K tile to fetch
    int pg_v = tile_page(kt_begin + 1);            // ... and in the next V tile
    cp_async_wait<2>();
    tc_fence_async_smem();
    __syncthreads();
    if (n_tiles > 0 && tid == 0) { tc_fence_after(); issue_s(0, 0); }

    for (int it = 0; it < n_tiles; ++it) {
        const int kt = kt_begin + it;
        const int buf = it & 1;
        // a. this tile's scores are in tensor memory; its K buffer is free again
        if (!tc_mbar_wait(buf ? bar_s1 : bar_s0, par_s[buf])) fail = 1;
        par_s[buf] ^= 1u;
        tc_fence_after();
        // b. the next tile's scores start now (K(it+1) was fetched an iteration ago) and run under this softmax
        cp_async_wait<1>();
        tc_fence_async_smem();
        if (__syncthreads_or(fail)) break;
        if (it + 1 < n_tiles && tid == 0) { tc_fence_after(); issue_s((it + 1) & 1, (it + 1) & 1); }
        // c. K(it+2) into the buffer S(it) has just released
        load_rows(k_s + (unsigned)(it & 1) * TC_KV_BYTES, kc, kt + 2, pg_k);
        cp_async_commit();
        pg_k = tile_page(kt + 3);
        // d. the row's 64 scores: two loads of 32 columns, kept in registers for both passes
        const unsigned ts = (buf ? t_s1 : t_s0) + lane_sel;
        const int key0 = kt * TC_KT;
        const bool need_mask = (key0 + TC_KT - 1 > p_min) || (p.window > 0 && key0 <= p_max - p.window);
        float sv[2][32];
        tc_ld32(ts, sv[0]);
        tc_ld32(ts + 32, sv[1]);
        if (need_mask) {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int key = key0 + h * 32 + j;
                    bool ok = key <= my_pos;
                    if (p.window > 0) ok = ok && (key > my_pos - p.window);
                    if (!ok) sv[h][j] = -INFINITY;
                }
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four chains: the maximum is not one long dependency
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 32; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], sv[h][j]);
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // The exponent's reference only follows the running maximum when that has grown by more than 2^8: P then
        // stays below 256 (no trouble for bfloat16 or the float32 sums), the result is the same softmax, and O is
        // rescaled a handful of times per row instead of once per tile.
        const float m_new = fmaxf(m_run, mx * sc);
        const float m_use = (m_new > m_run + 8.f) ? m_new : m_run;
        const float mu = (m_use == -INFINITY) ? 0.f : m_use;
        const float alpha = fast_exp2(m_run - mu);
        m_run = m_use;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                sv[h][j] = fast_exp2(fmaf(sv[h][j], sc, -mu));
                sum4[j & 3] += sv[h][j];
            }
        l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        // e. the previous tile's P V product is done: P, its V buffer and O may be touched
        if (it >= 1) {
            if (!tc_mbar_wait(bar_o, par_o)) fail = 1;
            par_o ^= 1u;
            tc_fence_after();
        }
        // f. V(it+1) into the buffer that product has released
        load_rows(v_s + (unsigned)((it + 1) & 1) * TC_KV_BYTES, vc, kt + 1, pg_v);
        cp_async_commit();
        pg_v = tile_page(kt + 2);
        // g. P -> shared memory (bfloat16, swizzled, K-major over the keys): 8 chunks of 8 keys
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const unsigned dst = p_s + tc_tile_off(tid, h * 4 + c4, TC_P_BYTES);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst),
                             "r"(pack_bf16(sv[h][c4 * 8 + 0], sv[h][c4 * 8 + 1])), "r"(pack_bf16(sv[h][c4 * 8 + 2], sv[h][c4 * 8 + 3])),
                             "r"(pack_bf16(sv[h][c4 * 8 + 4], sv[h][c4 * 8 + 5])), "r"(pack_bf16(sv[h][c4 * 8 + 6], sv[h][c4 * 8 + 7])) : "memory");
            }
        // rescale O where a maximum moved; the whole block skips it when none did
        if (it >= 1 && __syncthreads_or(alpha != 1.f)) {
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                float v[32];
                tc_ld32(t_o + lane_sel + cb * 32, v);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] *= alpha;
                tc_st32(t_o + lane_sel + cb * 32, v);
            }
            tc_wait_st();
        }
        // h./i. V(it) has landed (fetched an iteration ago); O += P V
        cp_async_wait<2>();
        tc_fence_before();
        tc_fence_async_smem();
        if (__syncthreads_or(fail)) break;
        if (tid == 0) { tc_fence_after(); issue_o(it & 1, it == 0); }
    }
    cp_async_wait<0>();
    // ---- epilogue: wait for the last P V product, normalise, write
    if (n_tiles > 0 && !fail) {
        if (!tc_mbar_wait(bar_o, par_o)) fail = 1;
        tc_fence_after();
    }
    const bool failed = __syncthreads_or(fail) != 0;
    if (!failed && n_tiles > 0) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const int hl = tid - my_tl * Gc;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) +
                             ((size_t)(ti.q_base + ti.t0 + (my_valid ? my_tl : 0)) * p.n_q + (size_t)kvh * G + (my_valid ? chunk * TC_ROWS + hl : 0)) * TC_D;
#pragma unroll
        for (int cb = 0; cb < 4; ++cb) {
            float v[32];
            tc_ld32(t_o + lane_sel + cb * 32, v);              // every thread of the warp takes part
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
    if (failed && status != nullptr && tid == 0) atomicExch(status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;\n" ::"r"(tmem) : "memory");
}
