// Sampling over float32 logits.
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

// A row is cut into gridDim.y slices, one block each, so that a handful of rows still fills the GPU (one block per
// row read 600 KB of logits through one SM, load by load: 70 us for 8 rows of 151,936).  Every block leaves its
// slice's best (value, index) in `part`; the block that finishes a row last (a ticket per row) merges the slices.
// `better` is associative and commutative with ties going to the lowest index, so the result does not depend on
// which block comes last.  Two passes:
//   pass 0  argmax of the logits: the token of a greedy row, and the row's maximum for pass 1
//   pass 1  (rows with temperature > 0) the exponential race: argmax_j exp((l_j - max) / T) / (e_j + 1e-10).
//           The softmax's denominator is the same for the whole row and cannot change which j wins, so it is
//           not computed.
// part: [rows][slices] (value, index); row_max: [rows]; tickets: [rows] ints, zero before the launch and zero
// again after it.
__device__ __forceinline__ bool last_block_of_row(int* ticket, int n_blocks) {
    __shared__ int sh_last;
    __threadfence();                       // this block's partial is visible before its ticket is
    __syncthreads();
    if (threadIdx.x == 0) sh_last = (atomicAdd(ticket, 1) == n_blocks - 1);
    __syncthreads();
    if (sh_last) __threadfence();          // the other blocks' partials are visible to this one
    return sh_last != 0;
}

template <int PASS>
__global__ void sample_slices_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                                     const float* __restrict__ temperatures, const int* __restrict__ row_keys,
                                     const int* __restrict__ steps, unsigned long long seed, ArgBest* __restrict__ part,
                                     float* __restrict__ row_max, int* __restrict__ tickets, int* __restrict__ out) {
    __shared__ ArgBest sbest[32];
    pdl_launch_dependents();
    pdl_wait();
    pdl_after_wait();
    const int r = blockIdx.x, S = gridDim.y, sl = blockIdx.y;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperatures ? temperatures[r] : 0.f;
    if (PASS == 1 && !(temp > 0.f)) return;            // a greedy row was finished by pass 0
    // slices in steps of 4 vocabulary entries (one Philox call yields 4 words)
    const int per = (((vocab + S - 1) / S) + 3) & ~3;
    const int j0 = sl * per, j1 = min(vocab, j0 + per);
    ArgBest best{-INFINITY, 0x7fffffff};
    if (PASS == 0) {
        int j = j0 + threadIdx.x;
        const int bd = (int)blockDim.x;
        for (; j + 7 * bd < j1; j += 8 * bd) {      // eight loads in flight
            float v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) v[q] = __ldg(row + j + q * bd);
#pragma unroll
            for (int q = 0; q < 8; ++q) best = better(best, ArgBest{v[q], j + q * bd});
        }
        for (; j < j1; j += blockDim.x) best = better(best, ArgBest{row[j], j});
    } else {
        const float mx = row_max[r], inv_t = 1.f / temp;
        const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
        const uint32_t key = (uint32_t)row_keys[r], step = (uint32_t)steps[r];
        for (int b = (j0 >> 2) + threadIdx.x; b * 4 < j1; b += blockDim.x) {
            uint32_t w[4];
            philox4x32_10((uint32_t)b, key, step, 0u, k0, k1, w);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int j = b * 4 + q;
                if (j < j1) {
                    const float u = ((float)(w[q] >> 9) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
                    const float e = -logf(u);
                    const float pj = expf((row[j] - mx) * inv_t);
                    best = better(best, ArgBest{pj / (e + 1e-10f), j});
                }
            }
        }
    }
    best = block_argmax(best, sbest);
    if (threadIdx.x == 0) part[(size_t)r * S + sl] = best;
    if (!last_block_of_row(tickets + r, S)) return;
    ArgBest all{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < S; i += blockDim.x) all = better(all, part[(size_t)r * S + i]);
    all = block_argmax(all, sbest);
    if (threadIdx.x == 0) {
        tickets[r] = 0;
        if (PASS == 0) {
            row_max[r] = all.v;
            if (!(temp > 0.f)) out[r] = all.i;
        } else {
            out[r] = all.i;
        }
    }
}

// part: rows * slices (value, index) pairs of 8 bytes; row_max: rows floats; tickets: rows ints that are zero before
// the call and zero again when the kernels have run.  slices: blocks per row (the caller sizes it to the device).
MSGL_API int msgl_sample(const float* logits, int rows, int vocab, long long row_stride, const float* temperatures,
                         const int* row_keys, const int* steps, unsigned long long seed, int* out, void* part,
                         float* row_max, int* tickets, int slices, cudaStream_t stream) {
    if (rows <= 0) return MSGL_OK;
    if (vocab <= 0 || slices < 1 || part == nullptr || row_max == nullptr || tickets == nullptr) return MSGL_ERR_SIZE;
    if (temperatures != nullptr && (row_keys == nullptr || steps == nullptr)) return MSGL_ERR_SIZE;
    const int threads = 256;
    msgl_launch_pdl(sample_slices_kernel<0>, dim3(rows, slices), dim3(threads), 0, stream, logits, vocab, row_stride, temperatures,
                    row_keys, steps, seed, (ArgBest*)part, row_max, tickets, out);
    if (temperatures != nullptr)
        msgl_launch_pdl(sample_slices_kernel<1>, dim3(rows, slices), dim3(threads), 0, stream, logits, vocab, row_stride, temperatures,
                        row_keys, steps, seed, (ArgBest*)part, row_max, tickets, out);
    return msgl_check_launch();
}
