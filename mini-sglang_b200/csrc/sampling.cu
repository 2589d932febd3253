// Sampling over float32 logits, one block per row.
//
//   temperature == 0 : argmax (lowest index wins a tie)
//   temperature  > 0 : p = softmax(logits / T);  token = argmax_j p_j / (e_j + 1e-10), e_j ~ Exp(1)
//                      (an exponential race, which draws from p)
// The noise comes from Philox4x32-10 with key = seed and counter = (j / 4, row_key, step, 0),
// word j % 4; u = ((word >> 9) + 0.5) * 2^-23; e = -log(u).  It depends on the request's key
// and step only, never on which other rows are in the batch.
#include "common.cuh"

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct ArgBest { float v; int i; };

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgBest block_argmax(ArgBest a, ArgBest* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    ArgBest r = (lane < nwarps) ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest b;
        b.v = __shfl_xor_sync(0xffffffffu, r.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, r.i, o);
        r = better(r, b);
    }
    return r;
}

__global__ void sample_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                              const float* __restrict__ temperatures, const int* __restrict__ row_keys,
                              const int* __restrict__ steps, unsigned long long seed, int* __restrict__ out) {
    __shared__ ArgBest sbest[32];
    __shared__ float sred[32];
    pdl_launch_dependents();
    pdl_wait();
    pdl_after_wait();
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperatures ? temperatures[r] : 0.f;

    ArgBest best{-INFINITY, 0x7fffffff};
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) best = better(best, ArgBest{row[j], j});
    best = block_argmax(best, sbest);
    if (!(temp > 0.f)) {
        if (threadIdx.x == 0) out[r] = best.i;
        return;
    }
    const float mx = best.v;
    const float inv_t = 1.f / temp;
    float s = 0.f;
    for (int j = threadIdx.x; j < vocab; j += blockDim.x) s += expf((row[j] - mx) * inv_t);
    const float total = block_sum(s, sred);
    const float inv_total = 1.f / total;

    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    const uint32_t key = (uint32_t)row_keys[r], step = (uint32_t)steps[r];
    ArgBest pick{-INFINITY, 0x7fffffff};
    const int nblk = (vocab + 3) >> 2;
    for (int b = threadIdx.x; b < nblk; b += blockDim.x) {
        uint32_t w[4];
        philox4x32_10((uint32_t)b, key, step, 0u, k0, k1, w);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int j = b * 4 + q;
            if (j < vocab) {
                const float u = ((float)(w[q] >> 9) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
                const float e = -logf(u);
                const float p = expf((row[j] - mx) * inv_t) * inv_total;
                pick = better(pick, ArgBest{p / (e + 1e-10f), j});
            }
        }
    }
    pick = block_argmax(pick, sbest);
    if (threadIdx.x == 0) out[r] = pick.i;
}

MSGL_API int msgl_sample(const float* logits, int rows, int vocab, long long row_stride, const float* temperatures,
                         const int* row_keys, const int* steps, unsigned long long seed, int* out,
                         cudaStream_t stream) {
    if (rows <= 0) return MSGL_OK;
    if (vocab <= 0) return MSGL_ERR_SIZE;
    const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 256 : 128);
    msgl_launch_pdl(sample_kernel, dim3(rows), dim3(threads), 0, stream, logits, vocab, row_stride, temperatures, row_keys, steps, seed, out);
    return msgl_check_launch();
}
