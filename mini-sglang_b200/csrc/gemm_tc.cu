// Matrix product for many tokens on the 5th-generation tensor cores: out[M, N] = x[M, K] . W[N, K]^T in
// bfloat16 with float32 accumulation, optionally with SwiGLU in the epilogue
// (out[M, I] = silu(x . Wgate^T) * (x . Wup^T) for W = [Wgate; Wup]), so that the [M, 2I] intermediate of the
// feed-forward never exists.
//
// A block is persistent and walks output tiles of 128 tokens x 256 weight rows (SwiGLU: 128 gate rows and the
// 128 up rows that belong to them, i.e. 128 output columns).  Per tile it runs over K in slabs of 64:
//
//     warp 0    TMA: x tile [128 x 64] and W tile [256 x 64] of a slab into one of four 48 KB stages
//               (cp.async.bulk.tensor, 128-byte swizzle; rows and columns past the matrices arrive as zeros)
//     warp 1    one lane issues four tcgen05.mma 128x256x16 per slab into one of two 256-column accumulators
//               in tensor memory and commits the stage back to the loader
//     warps 2-5 epilogue: thread = token row = TMEM lane; tcgen05.ld in chunks of 32 columns, SwiGLU or bias,
//               one rounding to bfloat16, 64-byte stores; the other accumulator is being filled meanwhile
//
// Tiles are numbered token-tile fastest, so the blocks that run together share the W tiles they stream
// (W is read from memory about once, x stays in L2).  Every wait is bounded; a block that gives up sets
// status[2] and frees its tensor memory (results are then invalid and the host raises).
//
// gemm_tc2_kernel further down is the same product on pairs of SMs (tiles of 256 x 256, tcgen05 cta_group::2);
// it is the one the engine takes, this one stays selectable.
#include "common.cuh"
#include "tc_common.cuh"

constexpr int GT_BM = 128, GT_BN = 256, GT_BK = 64, GT_STAGES = 4;
constexpr unsigned GT_A_BYTES = GT_BM * 128u, GT_B_BYTES = GT_BN * 128u, GT_STAGE_BYTES = GT_A_BYTES + GT_B_BYTES;     // 16 + 32 KB
constexpr unsigned GT_SMEM_ALLOC = GT_STAGES * GT_STAGE_BYTES + 256u + 1024u;
constexpr int GT_THREADS = 192;

// One thread's row of a finished accumulator (256 float32 columns at `acc`, this thread's lane already selected)
// -> bfloat16 output: SwiGLU of columns c and 128 + c, or the plain values (+ bias).
// c_lo, c_hi: the 32-column chunks to drain (of 4 for SwiGLU, of 8 else), so that two warps can share a row.
template <bool SWIGLU>
__device__ __forceinline__ void gt_drain(unsigned acc, int row, int col0, int M, int n_valid, const __nv_bfloat16* __restrict__ bias,
                                         __nv_bfloat16* __restrict__ out, long long ldo, int c_lo, int c_hi) {
    __nv_bfloat16* orow = out + (size_t)(row < M ? row : 0) * ldo + col0;
    if (SWIGLU) {
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
            float gate[32], up[32];
            tc_ld32(acc + c * 32, gate);
            tc_ld32(acc + 128 + c * 32, up);
            tc_wait_ld(gate);
            tc_wait_ld(up);
            if (row < M) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    if (col0 + c * 32 + j + 8 <= n_valid) {
                        unsigned pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float g0 = gate[j + 2 * e], g1 = gate[j + 2 * e + 1];
                            const __nv_bfloat162 v = __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * up[j + 2 * e],
                                                                           g1 / (1.f + expf(-g1)) * up[j + 2 * e + 1]);
                            pk[e] = *reinterpret_cast<const unsigned*>(&v);
                        }
                        *reinterpret_cast<uint4*>(orow + c * 32 + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    } else {
                        for (int e = 0; e < 8; ++e)
                            if (col0 + c * 32 + j + e < n_valid) {
                                const float g0 = gate[j + e];
                                orow[c * 32 + j + e] = __float2bfloat16_rn(g0 / (1.f + expf(-g0)) * up[j + e]);
                            }
                    }
                }
            }
        }
    } else {
#pragma unroll 1
        for (int c = c_lo; c < c_hi; ++c) {
            float v[32];
            tc_ld32(acc + c * 32, v);
            tc_wait_ld(v);
            if (row < M) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    const int col = col0 + c * 32 + j;
                    if (bias != nullptr) {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (col + e < n_valid) v[j + e] += __bfloat162float(bias[col + e]);
                    }
                    if (col + 8 <= n_valid) {
                        unsigned pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(v[j + 2 * e], v[j + 2 * e + 1]);
                            pk[e] = *reinterpret_cast<const unsigned*>(&h);
                        }
                        *reinterpret_cast<uint4*>(orow + c * 32 + j) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    } else {
                        for (int e = 0; e < 8; ++e)
                            if (col + e < n_valid) orow[c * 32 + j + e] = __float2bfloat16_rn(v[j + e]);
                    }
                }
            }
        }
    }
}

// Split-K: the same accumulator row as float32 partial sums.  part: [M, ldp] of this split; accumulator column c of the
// tile goes to column colmap(c): plain c -> n * 256 + c; SwiGLU: gate c < 128 -> n * 128 + c, up c >= 128 -> I + n * 128 + (c - 128),
// i.e. the partials have the layout of the un-fused [M, 2 I] product.
__device__ __forceinline__ void gt_drain_partial(unsigned acc, int row, int M, float* __restrict__ part, long long ldp, int col_lo, int col_hi_base,
                                                 int n_valid_lo, int n_valid_hi, int c_lo, int c_hi) {
    float* prow = part + (size_t)(row < M ? row : 0) * ldp;
#pragma unroll 1
    for (int c = c_lo; c < c_hi; ++c) {
        float v[32];
        tc_ld32(acc + c * 32, v);
        tc_wait_ld(v);
        if (row < M) {
            // chunks 0-3 are the tile's first 128 columns, 4-7 its second 128
            const int col = (c < 4) ? col_lo + c * 32 : col_hi_base + (c - 4) * 32;
            const int lim = (c < 4) ? n_valid_lo : n_valid_hi;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                if (col + j + 4 <= lim) *reinterpret_cast<float4*>(prow + col + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                else
                    for (int e = 0; e < 4; ++e)
                        if (col + j + e < lim) prow[col + j + e] = v[j + e];
            }
        }
    }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(GT_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                const __grid_constant__ CUtensorMap wmap,
                                                                const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                                                int M, int N, int K, long long ldo, int I, int* status) {
    extern __shared__ __align__(16) unsigned char gt_smem[];
    const unsigned smem_base = tc_smem_u32(gt_smem);
    const unsigned tiles0 = (smem_base + 256u + 1023u) & ~1023u;
    unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(gt_smem + 192);
    if (status != nullptr && *reinterpret_cast<volatile int*>(status + 2) != 0) return;
    if (tiles0 + GT_STAGES * GT_STAGE_BYTES > smem_base + GT_SMEM_ALLOC) {
        if (threadIdx.x == 0 && status != nullptr) atomicExch(status + 2, 2);
        return;
    }
    auto bar_full = [&](int s) { return smem_base + 8u * (unsigned)s; };                  // stage holds a slab (TMA bytes)
    auto bar_empty = [&](int s) { return smem_base + 32u + 8u * (unsigned)s; };           // the slab's products are done (tensor core commits)
    auto bar_acc_full = [&](int b) { return smem_base + 64u + 8u * (unsigned)b; };        // accumulator b holds a tile
    auto bar_acc_empty = [&](int b) { return smem_base + 80u + 8u * (unsigned)b; };       // the epilogue has read accumulator b (4 warps)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int n_valid = SWIGLU ? I : N;                            // output columns
    const int bn_out = SWIGLU ? GT_BN / 2 : GT_BN;                 // output columns of a tile
    const int MT = (M + GT_BM - 1) / GT_BM, NT = (n_valid + bn_out - 1) / bn_out;
    const int n_tiles = MT * NT, n_slabs = (K + GT_BK - 1) / GT_BK;

    if (tid == 0) {
        for (int s = 0; s < GT_STAGES; ++s) { tc_mbar_init(bar_full(s), 1); tc_mbar_init(bar_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { tc_mbar_init(bar_acc_full(b), 1); tc_mbar_init(bar_acc_empty(b), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // all 512 columns of tensor memory: two accumulators of 256
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(tc_smem_u32(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_base_s;
    int fail = 0;

    if (warp == 0) {
        // =========================== loader
        if (lane == 0) {
            int g = 0;                                                 // slabs fetched so far, over all tiles
            for (int t = blockIdx.x; t < n_tiles && !fail; t += gridDim.x) {
                const int m = t % MT, n = t / MT;
                for (int k = 0; k < n_slabs; ++k, ++g) {
                    const int st = g % GT_STAGES;
                    if (!tc_mbar_wait(bar_empty(st), ((g / GT_STAGES) & 1) ^ 1)) { fail = 1; break; }    // (passes at once the first time round)
                    const unsigned a_s = tiles0 + (unsigned)st * GT_STAGE_BYTES, b_s = a_s + GT_A_BYTES;
                    tc_mbar_expect_tx(bar_full(st), GT_STAGE_BYTES);
                    tc_tma_load(a_s, &xmap, k * GT_BK, m * GT_BM, bar_full(st));
                    if (SWIGLU) {
                        tc_tma_load(b_s, &wmap, k * GT_BK, n * 128, bar_full(st));                       // gate rows
                        tc_tma_load(b_s + 128u * 128u, &wmap, k * GT_BK, I + n * 128, bar_full(st));     // their up rows
                    } else {
                        tc_tma_load(b_s, &wmap, k * GT_BK, n * GT_BN, bar_full(st));
                        tc_tma_load(b_s + 128u * 128u, &wmap, k * GT_BK, n * GT_BN + 128, bar_full(st));
                    }
                }
            }
        }
    } else if (warp == 1) {
        // =========================== issuer
        if (lane == 0) {
            const unsigned idesc = tc_idesc(false, GT_BN);
            // descriptors of stage 0; a stage further is a constant more in the address field (16-byte units)
            const unsigned long long da0 = tc_desc(tiles0, 16, 1024), db0 = tc_desc(tiles0 + GT_A_BYTES, 16, 1024);
            const unsigned long long stage_step = GT_STAGE_BYTES >> 4;
            int g = 0, it = 0;
            for (int t = blockIdx.x; t < n_tiles && !fail; t += gridDim.x, ++it) {
                const int b = it & 1;
                if (!tc_mbar_wait(bar_acc_empty(b), ((it >> 1) & 1) ^ 1)) { fail = 1; break; }           // the epilogue has drained this accumulator
                tc_fence_after();
                const unsigned d_t = tmem + (unsigned)b * 256u;
                for (int k = 0; k < n_slabs; ++k, ++g) {
                    const int st = g % GT_STAGES;
                    if (!tc_mbar_wait(bar_full(st), (g / GT_STAGES) & 1)) { fail = 1; break; }
                    tc_fence_after();
                    const unsigned long long da = da0 + (unsigned long long)st * stage_step, db = db0 + (unsigned long long)st * stage_step;
#pragma unroll
                    for (int kk = 0; kk < GT_BK / 16; ++kk)                                             // 32 bytes further along K per step
                        tc_mma(d_t, da + (unsigned long long)(2 * kk), db + (unsigned long long)(2 * kk), idesc, (k > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(bar_empty(st));
                }
                if (fail) break;
                tc_commit(bar_acc_full(b));
            }
        }
    } else {
        // =========================== epilogue: thread = token row of the tile = TMEM lane
        const int q = warp & 3;                                        // the lanes 32 q .. 32 q + 31 are this warp's
        const unsigned lane_sel = (unsigned)(q * 32) << 16;
        int it = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++it) {
            const int m = t % MT, n = t / MT, b = it & 1;
            if (!tc_mbar_wait(bar_acc_full(b), (it >> 1) & 1)) { fail = 1; break; }
            tc_fence_after();
            gt_drain<SWIGLU>(tmem + (unsigned)b * 256u + lane_sel, m * GT_BM + q * 32 + lane, n * bn_out, M, n_valid, bias, out, ldo, 0, SWIGLU ? 4 : 8);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(bar_acc_empty(b));
        }
    }
    tc_fence_before();
    const bool failed = __syncthreads_or(fail) != 0;
    if (failed && status != nullptr && tid == 0) atomicExch(status + 2, 1);
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// The same product on pairs of SMs (a cluster of two blocks, tcgen05 with cta_group::2): a pair owns tiles of
// 256 tokens x 256 weight rows.  Each block of the pair brings its own 128 token rows and its own 128 weight rows
// of a slab into its own shared memory (32 KB a stage, so seven stages fit), the first block of the pair issues
// tcgen05.mma 256x256x16, which reads both blocks' shared memory and fills both blocks' tensor memory, and each
// block drains the accumulator rows of its own 128 tokens.  Per SM and flop that is two thirds of the shared-memory
// traffic of the one-block kernel and half of its weight fetches from L2.
//
// Barriers live at the same offsets in both blocks.  full[s] of the first block counts the bytes of both blocks'
// copies (the second block's copies signal it across the pair); empty[s] and acc_full[b] of both blocks are signalled
// together by tcgen05.commit with a mask over the pair; acc_empty[b] of the first block collects the eight epilogue
// warps of both blocks.
// ---------------------------------------------------------------------------------------------------------------
#ifndef MSGL_GT2_STAGES
#define MSGL_GT2_STAGES 7
#endif
constexpr int GT2_STAGES = MSGL_GT2_STAGES;
constexpr int GT2_THREADS = 320;            // loader, issuer, 8 epilogue warps (two per quarter of the lanes, half of the columns each)
constexpr unsigned GT2_HALF_BYTES = 128u * 128u, GT2_STAGE_BYTES = 2u * GT2_HALF_BYTES;            // x rows + weight rows: 16 + 16 KB
constexpr unsigned GT2_SMEM_ALLOC = GT2_STAGES * GT2_STAGE_BYTES + 256u + 1024u;

__device__ __forceinline__ unsigned gt2_cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned gt2_map_to(unsigned saddr, unsigned rank) {       // the same offset in block `rank` of the cluster
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void gt2_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ bool gt2_mbar_wait_cluster(unsigned bar, unsigned parity) {     // arrivals may come from the other block
    for (long long it = 0; it < TC_SPIN_LIMIT; ++it) {
        unsigned done;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void gt2_mbar_arrive_remote(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// TMA copy into this block's shared memory whose bytes are counted by a barrier of either block of the pair
__device__ __forceinline__ void gt2_tma_load(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar_cluster_addr) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(reinterpret_cast<unsigned long long>(map)), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void gt2_mma(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc,
                                        unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void gt2_commit_pair(unsigned bar) {       // the barrier at this offset in both blocks
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}

template <bool SWIGLU>
__global__ void __launch_bounds__(GT2_THREADS, 1) gemm_tc2_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                 const __grid_constant__ CUtensorMap wmap,
                                                                 const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                                                 int M, int N, int K, long long ldo, int I, int* status,
                                                                 int splits, float* __restrict__ part) {
    // splits > 1 (few tokens: too few tiles to fill the GPU): K is cut into `splits` ranges of slabs, a work item is
    // (tile, range), and the accumulators go out as float32 partial sums part[range][M][N] for gemm_splitk_reduce_kernel.
    extern __shared__ __align__(16) unsigned char gt_smem[];
    const unsigned smem_base = tc_smem_u32(gt_smem);
    const unsigned tiles0 = (smem_base + 256u + 1023u) & ~1023u;
    unsigned& tmem_base_s = *reinterpret_cast<unsigned*>(gt_smem + 192);
    const unsigned rank = gt2_cluster_rank();                       // 0: issues the products of the pair
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const bool fits = tiles0 + GT2_STAGES * GT2_STAGE_BYTES <= smem_base + GT2_SMEM_ALLOC;      // the same in both blocks
    auto bar_full = [&](int s) { return smem_base + 8u * (unsigned)s; };
    auto bar_empty = [&](int s) { return smem_base + 64u + 8u * (unsigned)s; };
    auto bar_acc_full = [&](int b) { return smem_base + 128u + 8u * (unsigned)b; };
    auto bar_acc_empty = [&](int b) { return smem_base + 144u + 8u * (unsigned)b; };
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    const int n_valid = SWIGLU ? I : N;
    const int bn_out = SWIGLU ? 128 : 256;
    const int MT = (M + 255) / 256, NT = (n_valid + bn_out - 1) / bn_out;
    const int n_slabs = (K + GT_BK - 1) / GT_BK;
    const int n_tiles = MT * NT * splits;                   // work items: the ranges of a tile are neighbours, so they run at the same time
    auto item = [&](int t, int& m, int& n, int& k_begin, int& k_end) {
        const int ks = t % splits, tile = t / splits;
        m = tile % MT; n = tile / MT;
        k_begin = (int)((long long)ks * n_slabs / splits);
        k_end = (int)((long long)(ks + 1) * n_slabs / splits);
    };

    if (tid == 0) {
        for (int s = 0; s < GT2_STAGES; ++s) { tc_mbar_init(bar_full(s), 1); tc_mbar_init(bar_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { tc_mbar_init(bar_acc_full(b), 1); tc_mbar_init(bar_acc_empty(b), 16); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {   // one warp of each block of the pair: all 512 columns in both
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(tc_smem_u32(&tmem_base_s)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    gt2_cluster_sync();                                             // both blocks' barriers and tensor memory exist
    tc_fence_after();
    const unsigned tmem = tmem_base_s;
    int fail = fits ? 0 : 2;

    if (warp == 0) {
        // =========================== loader (both blocks): own token rows, own weight rows
        if (lane == 0 && !fail) {
            const unsigned full0 = gt2_map_to(bar_full(0), 0);                                          // the first block's full[0]
            int g = 0;
            pdl_wait();                   // x is the output of the kernel before: everything up to here ran beside its end
            for (int t = pair; t < n_tiles && !fail; t += n_pairs) {
                int m, n, k_begin, k_end;
                item(t, m, n, k_begin, k_end);
                const int w_row = SWIGLU ? (rank == 0 ? n * 128 : I + n * 128) : n * 256 + (int)rank * 128;
                for (int k = k_begin; k < k_end; ++k, ++g) {
                    const int st = g % GT2_STAGES;
                    if (!tc_mbar_wait(bar_empty(st), ((g / GT2_STAGES) & 1) ^ 1)) { fail = 1; break; }
                    const unsigned a_s = tiles0 + (unsigned)st * GT2_STAGE_BYTES, b_s = a_s + GT2_HALF_BYTES;
                    if (rank == 0) tc_mbar_expect_tx(bar_full(st), 2u * GT2_STAGE_BYTES);                  // both blocks' bytes
                    gt2_tma_load(a_s, &xmap, k * GT_BK, m * 256 + (int)rank * 128, full0 + 8u * (unsigned)st);
                    gt2_tma_load(b_s, &wmap, k * GT_BK, w_row, full0 + 8u * (unsigned)st);
                }
            }
            pdl_late();                   // the last slabs are on their way: the next kernel may set itself up
        }
    } else if (warp == 1) {
        // =========================== issuer (first block only)
        if (lane == 0 && rank == 0 && !fail) {
            const unsigned idesc = (tc_idesc(false, 256) & ~(0x1Fu << 24)) | ((256u >> 4) << 24);        // M = 256 over the pair
            const unsigned long long da0 = tc_desc(tiles0, 16, 1024), db0 = tc_desc(tiles0 + GT2_HALF_BYTES, 16, 1024);
            const unsigned long long stage_step = GT2_STAGE_BYTES >> 4;
            int g = 0, it = 0;
            for (int t = pair; t < n_tiles && !fail; t += n_pairs, ++it) {
                const int b = it & 1;
                if (!gt2_mbar_wait_cluster(bar_acc_empty(b), ((it >> 1) & 1) ^ 1)) { fail = 1; break; }
                tc_fence_after();
                const unsigned d_t = tmem + (unsigned)b * 256u;
                int m_, n_, k_begin, k_end;
                item(t, m_, n_, k_begin, k_end);
                for (int k = k_begin; k < k_end; ++k, ++g) {
                    const int st = g % GT2_STAGES;
                    if (!gt2_mbar_wait_cluster(bar_full(st), (g / GT2_STAGES) & 1)) { fail = 1; break; }
                    tc_fence_after();
                    const unsigned long long da = da0 + (unsigned long long)st * stage_step, db = db0 + (unsigned long long)st * stage_step;
#pragma unroll
                    for (int kk = 0; kk < GT_BK / 16; ++kk)
                        gt2_mma(d_t, da + (unsigned long long)(2 * kk), db + (unsigned long long)(2 * kk), idesc, (k > k_begin || kk > 0) ? 1u : 0u);
                    gt2_commit_pair(bar_empty(st));
                }
                if (fail) break;
                gt2_commit_pair(bar_acc_full(b));
            }
        }
    } else if (!fail) {
        // =========================== epilogue (both blocks): the accumulator rows of the block's own 128 tokens
        const int q = warp & 3, second = warp >= 6 ? 1 : 0;              // warps 2-5: first half of the columns, 6-9: second half
        constexpr int n_chunks = SWIGLU ? 4 : 8;
        const unsigned lane_sel = (unsigned)(q * 32) << 16;
        const unsigned acc_empty0 = gt2_map_to(bar_acc_empty(0), 0);
        int it = 0;
        for (int t = pair; t < n_tiles; t += n_pairs, ++it) {
            int m, n, k_begin, k_end;
            item(t, m, n, k_begin, k_end);
            const int b = it & 1;
            if (!tc_mbar_wait(bar_acc_full(b), (it >> 1) & 1)) { fail = 1; break; }
            tc_fence_after();
            const int row = m * 256 + (int)rank * 128 + q * 32 + lane;
            if (part != nullptr) {
                float* mine = part + (size_t)(t % splits) * (size_t)M * (size_t)N;
                if (SWIGLU) gt_drain_partial(tmem + (unsigned)b * 256u + lane_sel, row, M, mine, N, n * 128, I + n * 128, I, N, second * 4, second * 4 + 4);
                else gt_drain_partial(tmem + (unsigned)b * 256u + lane_sel, row, M, mine, N, n * 256, n * 256 + 128, N, N, second * 4, second * 4 + 4);
            } else {
                gt_drain<SWIGLU>(tmem + (unsigned)b * 256u + lane_sel, row, n * bn_out, M, n_valid, bias, out, ldo,
                                 second * (n_chunks / 2), (second + 1) * (n_chunks / 2));
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) gt2_mbar_arrive_remote(acc_empty0 + 8u * (unsigned)b);
        }
    }
    tc_fence_before();
    const bool failed = __syncthreads_or(fail) != 0;
    if (failed && status != nullptr && tid == 0) atomicExch(status + 2, fail == 2 ? 2 : 1);
    gt2_cluster_sync();                                             // nobody of the pair reads tensor or shared memory of the other any more
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

// mode 0: out[M, N] = x . W^T (+ bias); mode 1: W = [gate; up] ([2I, K], N = 2I), out[M, I] = silu(gate) * up.
// bfloat16 everywhere; x rows ldx elements apart, out rows ldo; K, ldx multiples of 8 and ldo, (mode 1: I) multiples
// of 8 for the 16-byte stores; bases 16-byte aligned.  status: device int[>= 3]; word 2 is set if a block gave up.
// Returns MSGL_ERR_SIZE where the tensor maps cannot be made (the caller then uses the library GEMM).
MSGL_API int msgl_gemm_tc(const void* W, const void* X, const void* bias, void* out, int M, int N, int K, long long ldx,
                          long long ldo, int mode, void* status, cudaStream_t stream) {
    if (M <= 0) return MSGL_OK;
    if (N <= 0 || K <= 0 || (K & 7) || (ldx & 7) || (ldo & 7) || status == nullptr) return MSGL_ERR_SIZE;
    if (((uintptr_t)W | (uintptr_t)X | (uintptr_t)out) & 15) return MSGL_ERR_ALIGN;
    const int I = N / 2;
    if (mode == 1 && ((N & 1) || (I & 7) || bias != nullptr)) return MSGL_ERR_SIZE;
    CUtensorMap xm, wm;
    if (!tc_matrix_map(X, M, K, ldx * 2, 128, &xm) || !tc_matrix_map(W, N, K, (long long)K * 2, 128, &wm)) return MSGL_ERR_SIZE;
    static MsglOncePerDevice attr_set;
    if (attr_set.due()) {      // first call on this device, never inside a stream capture
        if (cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_ALLOC) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_ALLOC) != cudaSuccess)
            return msgl_check_launch();
        attr_set.mark();
    }
    const int n_valid = mode == 1 ? I : N, bn_out = mode == 1 ? GT_BN / 2 : GT_BN;
    const long long tiles = (long long)((M + GT_BM - 1) / GT_BM) * ((n_valid + bn_out - 1) / bn_out);
    const int sms = msgl_sm_count();
    const int grid = (int)(tiles < sms ? tiles : sms);
    if (mode == 1)
        gemm_tc_kernel<true><<<grid, GT_THREADS, GT_SMEM_ALLOC, stream>>>(xm, wm, nullptr, (__nv_bfloat16*)out, M, N, K, ldo, I, (int*)status);
    else
        gemm_tc_kernel<false><<<grid, GT_THREADS, GT_SMEM_ALLOC, stream>>>(xm, wm, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, M, N, K, ldo, 0,
                                                                           (int*)status);
    return msgl_check_launch();
}

// out = sum over the ranges of part[range][M][N], added in range order (the result does not depend on timing), then bias or
// SwiGLU and one rounding; a thread takes 4 neighbouring output columns of one token.
template <bool SWIGLU>
__global__ void gemm_splitk_reduce_kernel(const float* __restrict__ part, int splits, int M, int N, int I,
                                          const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, long long ldo) {
    pdl_launch_dependents();
    pdl_wait();
    pdl_after_wait();
    const int n_out = SWIGLU ? I : N;
    const int per_row = (n_out + 3) / 4;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * per_row) return;
    const int m = (int)(idx / per_row), c = (int)(idx - (long long)m * per_row) * 4;
    const size_t plane = (size_t)M * N;
    float a[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
    const bool whole = c + 4 <= n_out && (!SWIGLU || (I & 3) == 0);
    for (int sp = 0; sp < splits; ++sp) {
        const float* row = part + sp * plane + (size_t)m * N;
        if (whole) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(row + c));
            a[0] += v.x; a[1] += v.y; a[2] += v.z; a[3] += v.w;
            if (SWIGLU) {
                const float4 w = __ldcg(reinterpret_cast<const float4*>(row + I + c));
                u[0] += w.x; u[1] += w.y; u[2] += w.z; u[3] += w.w;
            }
        } else {
            for (int e = 0; e < 4; ++e)
                if (c + e < n_out) { a[e] += __ldcg(row + c + e); if (SWIGLU) u[e] += __ldcg(row + I + c + e); }
        }
    }
    __nv_bfloat16* orow = out + (size_t)m * ldo + c;
    for (int e = 0; e < 4; ++e) {
        if (c + e >= n_out) break;
        float y = a[e];
        if (SWIGLU) y = y / (1.f + expf(-y)) * u[e];
        else if (bias != nullptr) y += __bfloat162float(bias[c + e]);
        orow[e] = __float2bfloat16_rn(y);
    }
}

// The same on pairs of SMs (gemm_tc2_kernel); same arguments and return values.
// splits > 1: split-K with `partials` = splits * M * N float32 of scratch (see gemm_tc2_kernel); needs N % 4 == 0.
MSGL_API int msgl_gemm_tc2_splitk(const void* W, const void* X, const void* bias, void* out, int M, int N, int K, long long ldx,
                                  long long ldo, int mode, int splits, void* partials, void* status, cudaStream_t stream) {
    if (M <= 0) return MSGL_OK;
    if (splits < 1 || (splits > 1 && (partials == nullptr || (N & 3) || splits > (K + GT_BK - 1) / GT_BK))) return MSGL_ERR_SIZE;
    if (N <= 0 || K <= 0 || (K & 7) || (ldx & 7) || (ldo & 7) || status == nullptr) return MSGL_ERR_SIZE;
    if (((uintptr_t)W | (uintptr_t)X | (uintptr_t)out) & 15) return MSGL_ERR_ALIGN;
    const int I = N / 2;
    if (mode == 1 && ((N & 1) || (I & 7) || bias != nullptr)) return MSGL_ERR_SIZE;
    CUtensorMap xm, wm;
    if (!tc_matrix_map(X, M, K, ldx * 2, 128, &xm) || !tc_matrix_map(W, N, K, (long long)K * 2, 128, &wm)) return MSGL_ERR_SIZE;
    const int n_valid = mode == 1 ? I : N, bn_out = mode == 1 ? 128 : 256;
    const long long tiles = (long long)((M + 255) / 256) * ((n_valid + bn_out - 1) / bn_out) * splits;      // work items
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.blockDim = dim3(GT2_THREADS); cfg.dynamicSmemBytes = GT2_SMEM_ALLOC; cfg.stream = stream; cfg.attrs = attr;
    cfg.numAttrs = msgl_pdl_enabled() ? 2 : 1;
    static int pairs_of[MSGL_MAX_DEVICES][2] = {};      // per device and mode: how many pairs the device holds at once (asked once, outside any capture)
    int* max_pairs = pairs_of[msgl_device()];
    if (max_pairs[mode] == 0) {
        cudaError_t e = mode == 1
            ? cudaFuncSetAttribute(gemm_tc2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT2_SMEM_ALLOC)
            : cudaFuncSetAttribute(gemm_tc2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT2_SMEM_ALLOC);
        if (e != cudaSuccess) return msgl_check_launch();
        const int sms = msgl_sm_count();
        int n = 0;
        cfg.gridDim = dim3(2 * (sms / 2));
        e = mode == 1 ? cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<true>, &cfg)
                      : cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<false>, &cfg);
        if (e != cudaSuccess || n <= 0) { cudaGetLastError(); return MSGL_ERR_SIZE; }
        max_pairs[mode] = n < sms / 2 ? n : sms / 2;
    }
    const int pairs = (int)(tiles < max_pairs[mode] ? tiles : max_pairs[mode]);
    cfg.gridDim = dim3(2 * pairs);
    const __nv_bfloat16* b = mode == 1 ? nullptr : (const __nv_bfloat16*)bias;
    __nv_bfloat16* o = (__nv_bfloat16*)out;
    int* st = (int*)status;
    const int Iarg = mode == 1 ? I : 0;
    float* part = (float*)partials;
    if (splits <= 1) part = nullptr;
    cudaError_t e = mode == 1 ? cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<true>, xm, wm, b, o, M, N, K, ldo, Iarg, st, splits, part)
                              : cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<false>, xm, wm, b, o, M, N, K, ldo, Iarg, st, splits, part);
    (void)e;
    if (part == nullptr) return msgl_check_launch();
    // the ranges' partial sums -> output (bias / SwiGLU, one rounding), in range order
    const int n_out = mode == 1 ? I : N;
    const long long groups = (long long)M * ((n_out + 3) / 4);
    const int threads = 256;
    const unsigned blocks = (unsigned)((groups + threads - 1) / threads);
    if (mode == 1) msgl_launch_pdl(gemm_splitk_reduce_kernel<true>, dim3(blocks), dim3(threads), 0, stream, (const float*)part, splits, M, N, I, b, o, ldo);
    else msgl_launch_pdl(gemm_splitk_reduce_kernel<false>, dim3(blocks), dim3(threads), 0, stream, (const float*)part, splits, M, N, I, b, o, ldo);
    return msgl_check_launch();
}

MSGL_API int msgl_gemm_tc2(const void* W, const void* X, const void* bias, void* out, int M, int N, int K, long long ldx,
                           long long ldo, int mode, void* status, cudaStream_t stream) {
    return msgl_gemm_tc2_splitk(W, X, bias, out, M, N, K, ldx, ldo, mode, 1, nullptr, status, stream);
}

// How many ranges of K the split-K product should use for these sizes on the current device: the count (at most 8, at
// least 8 slabs of 64 each) for which the work items fill the pairs of SMs in the fewest rounds of the shortest items.
MSGL_API int msgl_gemm_tc2_splits(int M, int N, int K, int mode) {
    const int n_out = mode == 1 ? N / 2 : N, bn_out = mode == 1 ? 128 : 256;
    const long long tiles = (long long)((M + 255) / 256) * ((n_out + bn_out - 1) / bn_out);
    const int n_slabs = (K + GT_BK - 1) / GT_BK;
    const int pairs = msgl_sm_count() / 2;
    int best = 1;
    double best_cost = 1e30;
    for (int sp = 1; sp <= 8 && sp * 8 <= n_slabs; ++sp) {
        const long long items = tiles * sp;
        const long long rounds = (items + pairs - 1) / pairs;
        const double cost = (double)rounds * ((n_slabs + sp - 1) / sp + 3) + (sp > 1 ? 0.5 * sp : 0.0);      // + 3: filling the pipeline
        if (cost < best_cost - 1e-9) { best_cost = cost; best = sp; }
    }
    return best;
}
