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
// Roles: warps 0-3 do the softmax (thread t owns row t), warp 4 gathers K and V rows from the paged
// cache, one lane of warp 5 issues the tensor-core work.  They meet only at mbarriers, so the
// tensor core computes the next tile's scores and the loader fetches two tiles ahead while the
// softmax threads work on the current tile.
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
constexpr int TC_SOFTMAX_THREADS = 128;    // warps 0-3: one thread per query row
constexpr int TC_THREADS = 192;            // + warp 4: K/V loader, warp 5: tensor-core issuer
constexpr unsigned TC_QHALF_BYTES = 128u * 128u;           // one 64-column half of the [128 x 128] Q tile
constexpr unsigned TC_Q_BYTES = 2u * TC_QHALF_BYTES;       // 32 KB
constexpr unsigned TC_KHALF_BYTES = (unsigned)TC_KT * 128u;  // one 64-column half of a [64 keys x 128] K or V tile
constexpr unsigned TC_KV_BYTES = 2u * TC_KHALF_BYTES;      // 16 KB
constexpr unsigned TC_P_BYTES = 128u * 128u;               // P: [128 rows x 64 keys] = one half, 16 KB
constexpr unsigned TC_SMEM_BYTES = TC_Q_BYTES + 4u * TC_KV_BYTES + TC_P_BYTES;    // 112 KB: two blocks per SM
constexpr long long TC_SPIN_LIMIT = 4000000LL;             // polls of an mbarrier before a block gives up (a fraction of a second)

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
__device__ __forceinline__ void tc_mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// arrives on `bar` when all cp.async copies this thread has issued so far have landed
__device__ __forceinline__ void tc_cp_async_arrive(unsigned bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
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
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// the registers of tc_ld32 hold their values only after this
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
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
    // No static shared memory: two blocks have to fit an SM, and every byte of its 228 KB counts.  The first 256
    // bytes of the dynamic allocation hold the barriers and scalars, the operand tiles start at the next
    // 1024-byte boundary: Q | K0 | K1 | V0 | V1 | P.
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
    const unsigned q_s = smem0, k_s = q_s + TC_Q_BYTES, v_s = k_s + 2 * TC_KV_BYTES, p_s = v_s + 2 * TC_KV_BYTES;
    // mbarriers (8 bytes each)
    const unsigned bar_s0 = smem_base, bar_s1 = smem_base + 8;            // scores of a tile are in TMEM (tensor core commits)
    const unsigned bar_o = smem_base + 16;                                  // a P V product is done (tensor core commits)
    const unsigned bar_kf0 = smem_base + 24, bar_kf1 = smem_base + 32;      // K stage holds a tile (32 loader lanes)
    const unsigned bar_vf0 = smem_base + 40, bar_vf1 = smem_base + 48;      // V stage holds a tile
    const unsigned bar_sf0 = smem_base + 56, bar_sf1 = smem_base + 64;      // S buffer has been read (128 softmax threads)
    const unsigned bar_pf = smem_base + 72;                                 // P is in shared memory, O rescaled (128 threads)
    // A stage's "free" barrier is separate from bar_s / bar_o although the same tensor-core work completes it: a
    // waiter must never fall two phases behind a barrier, and the loader could, behind bar_o.
    const unsigned bar_kr0 = smem_base + 80, bar_kr1 = smem_base + 88;      // K stage may be overwritten
    const unsigned bar_vr0 = smem_base + 96, bar_vr1 = smem_base + 104;     // V stage may be overwritten
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

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

    if (tid == 0) {
        tc_mbar_init(bar_s0, 1); tc_mbar_init(bar_s1, 1); tc_mbar_init(bar_o, 1);
        tc_mbar_init(bar_kf0, 32); tc_mbar_init(bar_kf1, 32); tc_mbar_init(bar_vf0, 32); tc_mbar_init(bar_vf1, 32);
        tc_mbar_init(bar_sf0, TC_SOFTMAX_THREADS); tc_mbar_init(bar_sf1, TC_SOFTMAX_THREADS);
        tc_mbar_init(bar_pf, TC_SOFTMAX_THREADS);
        tc_mbar_init(bar_kr0, 1); tc_mbar_init(bar_kr1, 1); tc_mbar_init(bar_vr0, 1); tc_mbar_init(bar_vr1, 1);
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
    const unsigned t_s0 = tmem, t_s1 = tmem + 64, t_o = tmem + 128;
    int fail = 0;

    if (warp == 4) {
        // =========================== loader: Q once, then K(j), V(j) two tiles ahead of their use
        const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(p.q);
        const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(p.k_cache);
        const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(p.v_cache);
        const int* bt = p.block_table + (size_t)ti.req * p.bt_stride;
#pragma unroll 1
        for (int rr = 0; rr < 4; ++rr) {                                 // Q: 128 rows, 4 per lane
            const int r = rr * 32 + lane;
            const int tl = r / Gc, hl = r - tl * Gc, hg = chunk * TC_ROWS + hl;
            const bool valid = tl < ti.n_tok && tl < QT && hg < G;
            const __nv_bfloat16* src = qg + ((size_t)(ti.q_base + ti.t0 + (valid ? tl : 0)) * p.n_q + (size_t)kvh * G + (valid ? hg : 0)) * TC_D;
#pragma unroll
            for (int c = 0; c < 16; ++c) cp_async16_u32(q_s + tc_tile_off(r, c, TC_QHALF_BYTES), src + c * 8, valid);
        }
        auto row_page = [&](int kt, int row) -> int {
            const int key = kt * TC_KT + row;
            return (kt < kt_end && key <= p_max) ? bt[page_index(p, key)] : -1;
        };
        auto load_tile = [&](unsigned dst_tile, const __nv_bfloat16* cache, int kt, int pg0, int pg1) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {                                // 64 rows, 2 per lane
                const int row = h * 32 + lane;
                const int pg = h ? pg1 : pg0;
                const int key = kt * TC_KT + row;
                const bool valid = pg >= 0;
                size_t off = 0;
                if (valid) off = (((size_t)pg * p.n_kv + kvh) * p.page_size + page_slot(p, key)) * TC_D;
#pragma unroll
                for (int c = 0; c < 16; ++c) cp_async16_u32(dst_tile + tc_tile_off(row, c, TC_KHALF_BYTES), cache + off + c * 8, valid);
            }
        };
        int pg0 = row_page(kt_begin, lane), pg1 = row_page(kt_begin, 32 + lane);
        for (int j = 0; j < n_tiles; ++j) {
            const int kt = kt_begin + j, st = j & 1;
            const int npg0 = row_page(kt + 1, lane), npg1 = row_page(kt + 1, 32 + lane);     // next tile's pages, ahead of need
            if (j >= 2 && !tc_mbar_wait(st ? bar_kr1 : bar_kr0, ((j - 2) >> 1) & 1)) { fail = 1; break; }   // S(j-2) has read this K stage
            load_tile(k_s + (unsigned)st * TC_KV_BYTES, kc, kt, pg0, pg1);
            tc_cp_async_arrive(st ? bar_kf1 : bar_kf0);                   // (for j == 0 this also covers Q)
            if (j >= 2 && !tc_mbar_wait(st ? bar_vr1 : bar_vr0, ((j - 2) >> 1) & 1)) { fail = 1; break; }   // P V(j-2) has read this V stage
            load_tile(v_s + (unsigned)st * TC_KV_BYTES, vc, kt, pg0, pg1);
            tc_cp_async_arrive(st ? bar_vf1 : bar_vf0);
            pg0 = npg0; pg1 = npg1;
        }
        cp_async_commit();
        cp_async_wait<0>();
    } else if (warp == 5) {
        // =========================== issuer: one lane feeds the tensor core
        if (lane == 0 && n_tiles > 0) {
            const unsigned idesc_s = tc_idesc(false, TC_KT), idesc_o = tc_idesc(true, TC_D);
            auto issue_s = [&](int j) {                                   // S(j) = Q K(j)^T: 8 steps of 16 along the head size
                const unsigned kb = k_s + (unsigned)(j & 1) * TC_KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const unsigned qo = (unsigned)(kk >> 2) * TC_QHALF_BYTES + (unsigned)(kk & 3) * 32u;
                    const unsigned ko = (unsigned)(kk >> 2) * TC_KHALF_BYTES + (unsigned)(kk & 3) * 32u;
                    tc_mma((j & 1) ? t_s1 : t_s0, tc_desc(q_s + qo, 16, 1024), tc_desc(kb + ko, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit((j & 1) ? bar_s1 : bar_s0);
                tc_commit((j & 1) ? bar_kr1 : bar_kr0);
            };
            auto issue_o = [&](int j) {                                   // O += P V(j): 4 steps of 16 keys; V as stored (MN-major)
                const unsigned vb = v_s + (unsigned)(j & 1) * TC_KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < TC_KT / 16; ++kk)
                    tc_mma(t_o, tc_desc(p_s + (unsigned)kk * 32u, 16, 1024), tc_desc(vb + (unsigned)kk * 2048u, TC_KHALF_BYTES, 1024),
                           idesc_o, (j == 0 && kk == 0) ? 0u : 1u);
                tc_commit(bar_o);
                tc_commit((j & 1) ? bar_vr1 : bar_vr0);
            };
#ifdef MSGL_TC_PROFILE
            long long ip[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            long long i0 = clock64(), i1;
#define TC_IMARK(i) { i1 = clock64(); ip[i] += i1 - i0; i0 = i1; }
#else
#define TC_IMARK(i)
#endif
            bool ok = tc_mbar_wait(bar_kf0, 0);
            if (ok) { tc_fence_async_smem(); tc_fence_after(); issue_s(0); }
            TC_IMARK(7)
            for (int it = 0; it < n_tiles && ok; ++it) {
                if (it + 1 < n_tiles) {                                   // the next tile's scores run under this tile's softmax
                    const int j = it + 1;
                    ok = tc_mbar_wait((j & 1) ? bar_kf1 : bar_kf0, (j >> 1) & 1);
                    TC_IMARK(0)
                    if (ok && j >= 2) ok = tc_mbar_wait((j & 1) ? bar_sf1 : bar_sf0, ((j - 2) >> 1) & 1);   // S buffer read by softmax(j-2)
                    if (!ok) break;
                    TC_IMARK(1)
                    tc_fence_async_smem(); tc_fence_after();
                    issue_s(j);
                    TC_IMARK(2)
                }
                ok = tc_mbar_wait(bar_pf, it & 1);
                TC_IMARK(3)
                ok = ok && tc_mbar_wait((it & 1) ? bar_vf1 : bar_vf0, (it >> 1) & 1);
                if (!ok) break;
                TC_IMARK(4)
                tc_fence_async_smem(); tc_fence_after();
                issue_o(it);
                TC_IMARK(5)
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
            const int buf = it & 1;
            if (!tc_mbar_wait(buf ? bar_s1 : bar_s0, (it >> 1) & 1)) { fail = 1; break; }
            tc_fence_after();
            TC_MARK(0)
            const unsigned ts = (buf ? t_s1 : t_s0) + lane_sel;
            float sv[2][32];
            tc_ld32(ts, sv[0]);
            tc_ld32(ts + 32, sv[1]);
            tc_wait_ld();
            tc_fence_before();
            tc_mbar_arrive(buf ? bar_sf1 : bar_sf0);                      // the buffer may take the scores of tile it+2
            TC_MARK(1)
            const int key0 = (kt_begin + it) * TC_KT;
            const bool need_mask = (key0 + TC_KT - 1 > p_min) || (p.window > 0 && key0 <= p_max - p.window);
            if (need_mask) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int key = key0 + h * 32 + j;
                        bool okk = key <= my_pos;
                        if (p.window > 0) okk = okk && (key > my_pos - p.window);
                        if (!okk) sv[h][j] = -INFINITY;
                    }
            }
            float mx8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) mx8[j] = -INFINITY;               // eight chains: the maximum is not one long dependency
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 32; ++j) mx8[j & 7] = fmaxf(mx8[j & 7], sv[h][j]);
            const float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])), fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
            // The exponent's reference only follows the running maximum when that has grown by more than 2^8: P then
            // stays below 256 (no trouble for bfloat16 or the float32 sums), the result is the same softmax, and O is
            // rescaled a handful of times per row instead of once per tile.
            const float m_new = fmaxf(m_run, mx * sc);
            const float m_use = (m_new > m_run + 8.f) ? m_new : m_run;
            const float mu = (m_use == -INFINITY) ? 0.f : m_use;
            const float alpha = fast_exp2(m_run - mu);
            m_run = m_use;
            float sum8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum8[j] = 0.f;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    sv[h][j] = fast_exp2(fmaf(sv[h][j], sc, -mu));
                    sum8[j & 7] += sv[h][j];
                }
            l_run = l_run * alpha + (((sum8[0] + sum8[1]) + (sum8[2] + sum8[3])) + ((sum8[4] + sum8[5]) + (sum8[6] + sum8[7])));
            TC_MARK(2)
            // the previous tile's P V product is done: P and O may be touched
            if (it >= 1) {
                if (!tc_mbar_wait(bar_o, (it - 1) & 1)) { fail = 1; break; }
                tc_fence_after();
            }
            TC_MARK(3)
            // P -> shared memory (bfloat16, swizzled, K-major over the keys): 8 chunks of 8 keys
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const unsigned dst = p_s + tc_tile_off(tid, h * 4 + c4, TC_P_BYTES);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst),
                                 "r"(pack_bf16(sv[h][c4 * 8 + 0], sv[h][c4 * 8 + 1])), "r"(pack_bf16(sv[h][c4 * 8 + 2], sv[h][c4 * 8 + 3])),
                                 "r"(pack_bf16(sv[h][c4 * 8 + 4], sv[h][c4 * 8 + 5])), "r"(pack_bf16(sv[h][c4 * 8 + 6], sv[h][c4 * 8 + 7])) : "memory");
                }
            // rescale O where a reference maximum moved.  A warp owns its 32 rows (TMEM lanes), so it decides alone.
            if (it >= 1 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
                for (int cb = 0; cb < 4; cb += 2) {
                    float v0[32], v1[32];
                    tc_ld32(t_o + lane_sel + cb * 32, v0);
                    tc_ld32(t_o + lane_sel + cb * 32 + 32, v1);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) { v0[j] *= alpha; v1[j] *= alpha; }
                    tc_st32(t_o + lane_sel + cb * 32, v0);
                    tc_st32(t_o + lane_sel + cb * 32 + 32, v1);
                }
                tc_wait_st();
            }
            TC_MARK(4)
            tc_fence_async_smem();                                        // P: generic-proxy writes -> visible to the tensor core
            tc_fence_before();
            tc_mbar_arrive(bar_pf);
            TC_MARK(5)
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
#pragma unroll
            for (int cb = 0; cb < 4; ++cb) {
                float v[32];
                tc_ld32(t_o + lane_sel + cb * 32, v);                    // every thread of the warp takes part
                tc_wait_ld();
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
