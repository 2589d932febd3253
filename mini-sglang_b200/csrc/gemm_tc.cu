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
#include "common.cuh"
#include "tc_common.cuh"

constexpr int GT_BM = 128, GT_BN = 256, GT_BK = 64, GT_STAGES = 4;
constexpr unsigned GT_A_BYTES = GT_BM * 128u, GT_B_BYTES = GT_BN * 128u, GT_STAGE_BYTES = GT_A_BYTES + GT_B_BYTES;     // 16 + 32 KB
constexpr unsigned GT_SMEM_ALLOC = GT_STAGES * GT_STAGE_BYTES + 256u + 1024u;
constexpr int GT_THREADS = 192;

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
            const unsigned acc = tmem + (unsigned)b * 256u + lane_sel;
            const int row = m * GT_BM + q * 32 + lane;
            const int col0 = n * bn_out;
            __nv_bfloat16* orow = out + (size_t)(row < M ? row : 0) * ldo + col0;
            if (SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
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
                for (int c = 0; c < 8; ++c) {
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
    const CUtensorMap* xm = tc_matrix_map(X, M, K, ldx * 2, 128);
    const CUtensorMap* wm = tc_matrix_map(W, N, K, (long long)K * 2, 128);
    if (xm == nullptr || wm == nullptr) return MSGL_ERR_SIZE;
    static bool attr_set = false;
    if (!attr_set) {      // first call, never inside a stream capture
        if (cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_ALLOC) != cudaSuccess ||
            cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GT_SMEM_ALLOC) != cudaSuccess)
            return msgl_check_launch();
        attr_set = true;
    }
    const int n_valid = mode == 1 ? I : N, bn_out = mode == 1 ? GT_BN / 2 : GT_BN;
    const long long tiles = (long long)((M + GT_BM - 1) / GT_BM) * ((n_valid + bn_out - 1) / bn_out);
    int sms = 148, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(tiles < sms ? tiles : sms);
    if (mode == 1)
        gemm_tc_kernel<true><<<grid, GT_THREADS, GT_SMEM_ALLOC, stream>>>(*xm, *wm, nullptr, (__nv_bfloat16*)out, M, N, K, ldo, I, (int*)status);
    else
        gemm_tc_kernel<false><<<grid, GT_THREADS, GT_SMEM_ALLOC, stream>>>(*xm, *wm, (const __nv_bfloat16*)bias, (__nv_bfloat16*)out, M, N, K, ldo, 0,
                                                                           (int*)status);
    return msgl_check_launch();
}
