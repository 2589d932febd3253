// Weight-streaming matrix product for decode: out[M, N] = x[M, K] . W[N, K]^T with M <= 16 tokens.
//
// With so few tokens the product is bound by reading W once from HBM, so the kernel is built
// around that stream:
//   * a block owns 16 output rows (rows of W) and all of K; its warps take the 32-element chunks
//     of K round-robin, so together they read each row contiguously;
//   * every lane fetches 16 bytes of two weight rows (and of its token rows) per chunk, exactly the
//     registers that mma.sync m16n8k16 takes as its A (and B) operand.  The k index inside a
//     32-chunk is permuted (lane t owns k = 8t .. 8t+7) for W and x alike, so the dot products are
//     unchanged and no lane ever needs another lane's data: no ldmatrix, no barrier in the loop;
//   * the fetches are cp.async copies into a lane-private slot of a shared-memory ring, GS_PF
//     chunks ahead of the math.  The ring is only a deep prefetch queue (each lane reads back what
//     it copied), which keeps ~100 KB per SM in flight without spending registers on it;
//   * the tokens ride the n dimension of the mma (8 per n-block, 1 or 2 n-blocks), fp32 accumulate;
//   * the warps' partial sums are added in warp order through shared memory (a fixed order, so
//     the result does not depend on timing), then bias / SwiGLU and one rounding to the output type.
//
// SwiGLU mode: W is [2I, K] with the gate rows first; a block takes 8 gate rows and the 8 up rows
// that belong to them, which land in the two row halves of the accumulator fragment, so
// out[M, I] = silu(gate) * up is formed in registers and the [M, 2I] intermediate never exists.
//
// Requirements (checked by the entry point, which returns MSGL_ERR_SIZE otherwise and the caller
// uses the library GEMM): bfloat16 inputs, K % 32 == 0, N % 16 == 0 (I % 8 == 0 in SwiGLU mode),
// 16-byte aligned rows.
#include "common.cuh"

#ifndef MSGL_GS_WARPS
#define MSGL_GS_WARPS 8
#endif
#ifndef MSGL_GS_PF
#define MSGL_GS_PF 5
#endif
constexpr int GS_WARPS = MSGL_GS_WARPS;
constexpr int GS_PF = MSGL_GS_PF;      // chunks in flight per warp (ring depth)

__device__ __forceinline__ void mma_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                          unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {      // read once: do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ldg_keep(const void* p) {        // x: read by every block, keep cached
    return __ldg(reinterpret_cast<const uint4*>(p));
}

template <typename OutT> __device__ __forceinline__ void store_out(OutT* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void cp_async16_g(void* smem, const void* gmem) {
    const unsigned s_ = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s_), "l"(gmem));
}
__device__ __forceinline__ void cp_async16_a(void* smem, const void* gmem) {      // .ca: x stays in L1
    const unsigned s_ = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(s_), "l"(gmem));
}

template <int NB, bool SWIGLU, typename OutT>
__global__ void __launch_bounds__(GS_WARPS * 32) gemm_small_m_kernel(
    const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X, const __nv_bfloat16* __restrict__ bias,
    OutT* __restrict__ out, int M, int N, int K, long long ldx, long long ldo, int I) {
    // ring[warp][stage][2 + NB][lane] of 16-byte slots; reused for the reduction at the end
    extern __shared__ __align__(16) unsigned char gs_smem[];
    constexpr int SLOTS = 2 + NB;
    uint4* ring = reinterpret_cast<uint4*>(gs_smem);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    uint4* my = ring + ((size_t)warp * GS_PF * SLOTS) * 32 + lane;

    // the two weight rows this lane feeds into the A fragment
    size_t row_lo, row_hi;
    if (SWIGLU) {
        row_lo = (size_t)blockIdx.x * 8 + g;          // gate row
        row_hi = (size_t)I + row_lo;                  // its up row
    } else {
        row_lo = (size_t)blockIdx.x * 16 + g;
        row_hi = row_lo + 8;
    }
    const __nv_bfloat16* w_lo = W + row_lo * K + 8 * t;
    const __nv_bfloat16* w_hi = W + row_hi * K + 8 * t;
    // x rows (tokens) this lane feeds into the B fragments; rows past M read row 0 and are dropped later
    const __nv_bfloat16* xr[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int tok = nb * 8 + g;
        xr[nb] = X + (size_t)(tok < M ? tok : 0) * ldx + 8 * t;
    }

    float c[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) { c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f; }

    const int n_chunks = K >> 5;
    const int n_my = (n_chunks > warp) ? (n_chunks - warp + GS_WARPS - 1) / GS_WARPS : 0;

    auto fetch_w = [&](int i) {        // weights of chunk i of this warp -> stage i % GS_PF
        uint4* st = my + (size_t)(i % GS_PF) * SLOTS * 32;
        const size_t k0 = (size_t)(warp + i * GS_WARPS) << 5;
        cp_async16_g(st, w_lo + k0);
        cp_async16_g(st + 32, w_hi + k0);
    };
    auto fetch_x = [&](int i) {        // the tokens' part of the same chunk
        uint4* st = my + (size_t)(i % GS_PF) * SLOTS * 32;
        const size_t k0 = (size_t)(warp + i * GS_WARPS) << 5;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) cp_async16_a(st + (2 + nb) * 32, xr[nb] + k0);
    };
    auto fetch = [&](int i) { fetch_w(i); fetch_x(i); };
    // The weights do not depend on the kernel before this one: their first chunks are already on the
    // way while that kernel finishes.  x (its output) is only touched after the wait.
    pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < GS_PF - 1; ++i)
        if (i < n_my) fetch_w(i);
    pdl_wait();
    pdl_after_wait();
#pragma unroll
    for (int i = 0; i < GS_PF - 1; ++i) {
        if (i < n_my) fetch_x(i);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    for (int i = 0; i < n_my; ++i) {
        if (i + GS_PF - 1 < n_my) fetch(i + GS_PF - 1);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(GS_PF - 1));
        // a lane reads only the slots it filled itself: no barrier needed
        const uint4* st = my + (size_t)(i % GS_PF) * SLOTS * 32;
        const uint4 wl = st[0], wh = st[32];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const uint4 xv = st[(2 + nb) * 32];
            mma_16816(c[nb], wl.x, wh.x, wl.y, wh.y, xv.x, xv.y);
            mma_16816(c[nb], wl.z, wh.z, wl.w, wh.w, xv.z, xv.w);
        }
    }
    pdl_late();         // the stream is read: the next kernel may set itself up beside the reduction
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();                      // every warp is done with the ring: reuse it for the sums
    float (*red)[16][8 * NB + 1] = reinterpret_cast<float (*)[16][8 * NB + 1]>(gs_smem);

    // partial sums of the warps -> shared memory; accumulator layout: c0,c1 = (row g, tokens 2t, 2t+1),
    // c2,c3 = (row g + 8, same tokens)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        red[warp][g][nb * 8 + 2 * t] = c[nb][0];
        red[warp][g][nb * 8 + 2 * t + 1] = c[nb][1];
        red[warp][g + 8][nb * 8 + 2 * t] = c[nb][2];
        red[warp][g + 8][nb * 8 + 2 * t + 1] = c[nb][3];
    }
    __syncthreads();
    if (SWIGLU) {
        // 8 output columns x (8 NB) tokens
        for (int idx = threadIdx.x; idx < 8 * 8 * NB; idx += GS_WARPS * 32) {
            const int r = idx / (8 * NB), tok = idx - r * (8 * NB);
            if (tok >= M) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < GS_WARPS; ++w) { gate += red[w][r][tok]; up += red[w][r + 8][tok]; }
            const float y = gate / (1.f + expf(-gate)) * up;
            store_out<OutT>(out + (size_t)tok * ldo + (size_t)blockIdx.x * 8 + r, y);
        }
    } else {
        for (int idx = threadIdx.x; idx < 16 * 8 * NB; idx += GS_WARPS * 32) {
            const int r = idx / (8 * NB), tok = idx - r * (8 * NB);
            if (tok >= M) continue;
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < GS_WARPS; ++w) acc += red[w][r][tok];
            const size_t col = (size_t)blockIdx.x * 16 + r;
            if (bias) acc += __bfloat162float(bias[col]);
            store_out<OutT>(out + (size_t)tok * ldo + col, acc);
        }
    }
}

// mode: 0 = plain (out [M, N]), 1 = SwiGLU (W [2I, K], out [M, I], N = 2I).  out_f32: output type.
MSGL_API int msgl_gemm_small_m(const void* W, const void* X, const void* bias, void* out, int M, int N, int K,
                               long long ldx, long long ldo, int mode, int out_f32, cudaStream_t stream) {
    if (M <= 0) return MSGL_OK;
    if (M > 16 || K <= 0 || (K & 31) || N <= 0) return MSGL_ERR_SIZE;
    if (((uintptr_t)W | (uintptr_t)X) & 15) return MSGL_ERR_ALIGN;
    if ((ldx & 7) != 0) return MSGL_ERR_ALIGN;
    const __nv_bfloat16* w = (const __nv_bfloat16*)W;
    const __nv_bfloat16* x = (const __nv_bfloat16*)X;
    const __nv_bfloat16* b = (const __nv_bfloat16*)bias;
    const int threads = GS_WARPS * 32;
    const size_t smem1 = (size_t)GS_WARPS * GS_PF * 3 * 32 * 16, smem2 = (size_t)GS_WARPS * GS_PF * 4 * 32 * 16;
    static MsglOncePerDevice attr_set;
    if (attr_set.due()) {      // first call on this device, never inside a stream capture
        cudaFuncSetAttribute(gemm_small_m_kernel<1, true, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        cudaFuncSetAttribute(gemm_small_m_kernel<2, true, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        cudaFuncSetAttribute(gemm_small_m_kernel<1, false, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        cudaFuncSetAttribute(gemm_small_m_kernel<2, false, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        cudaFuncSetAttribute(gemm_small_m_kernel<1, false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        cudaFuncSetAttribute(gemm_small_m_kernel<2, false, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
        attr_set.mark();
    }
    if (mode == 1) {
        if ((N & 15) || bias != nullptr) return MSGL_ERR_SIZE;
        const int I = N / 2;
        if (I & 7) return MSGL_ERR_SIZE;
        const int grid = I / 8;
        if (out_f32) return MSGL_ERR_DTYPE;
        if (M <= 8)
            msgl_launch_pdl(gemm_small_m_kernel<1, true, __nv_bfloat16>, dim3(grid), dim3(threads), smem1, stream, w, x, nullptr, (__nv_bfloat16*)out, M, N, K, ldx, ldo, I);
        else
            msgl_launch_pdl(gemm_small_m_kernel<2, true, __nv_bfloat16>, dim3(grid), dim3(threads), smem2, stream, w, x, nullptr, (__nv_bfloat16*)out, M, N, K, ldx, ldo, I);
        return msgl_check_launch();
    }
    if (N & 15) return MSGL_ERR_SIZE;
    const int grid = N / 16;
    if (out_f32) {
        if (M <= 8) msgl_launch_pdl(gemm_small_m_kernel<1, false, float>, dim3(grid), dim3(threads), smem1, stream, w, x, b, (float*)out, M, N, K, ldx, ldo, 0);
        else msgl_launch_pdl(gemm_small_m_kernel<2, false, float>, dim3(grid), dim3(threads), smem2, stream, w, x, b, (float*)out, M, N, K, ldx, ldo, 0);
    } else {
        if (M <= 8) msgl_launch_pdl(gemm_small_m_kernel<1, false, __nv_bfloat16>, dim3(grid), dim3(threads), smem1, stream, w, x, b, (__nv_bfloat16*)out, M, N, K, ldx, ldo, 0);
        else msgl_launch_pdl(gemm_small_m_kernel<2, false, __nv_bfloat16>, dim3(grid), dim3(threads), smem2, stream, w, x, b, (__nv_bfloat16*)out, M, N, K, ldx, ldo, 0);
    }
    return msgl_check_launch();
}
