// Memory-bound kernels of the decoder: embedding, RMSNorm with the residual sum fused in,
// per-head q/k norm + rotary position encoding + cache write in one pass, SwiGLU.
//
// Conventions
//  * activations are `T` (float or bfloat16); the residual stream is always float32, so the
//    residual sum is computed and kept in 32-bit;
//  * all arithmetic inside a kernel is float32; one rounding at the store;
//  * every size is a run-time parameter (rows, widths, head counts, head size, page size);
//    sizes a kernel cannot take are refused with MSGL_ERR_SIZE by the C entry point;
//  * reductions are done in an order fixed by the launch shape only.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// embedding: res[t, :] = float(E[ids[t], :])
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V) {
    pdl_launch_dependents();
    pdl_wait();
    pdl_after_wait();
    pdl_small();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {  // host code validates ids; an id out of range yields zeros, never a wild read
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const T* row = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32<T>(row[i]);
}

// ids[t] < 0 stands for prev[-1 - ids[t]] (a token that an earlier kernel sampled and the host has not read)
__global__ void resolve_ids_kernel(int* __restrict__ ids, const int* __restrict__ prev, int T_, int n_prev) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T_) return;
    const int v = ids[t];
    if (v < 0) {
        const int r = -1 - v;
        ids[t] = r < n_prev ? prev[r] : 0;
    }
}

MSGL_API int msgl_resolve_ids(void* ids, const void* prev, int T_, int n_prev, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    resolve_ids_kernel<<<(T_ + 255) / 256, 256, 0, stream>>>((int*)ids, (const int*)prev, T_, n_prev);
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// Step metadata of a decode step, made on the device (the reference fills cu_seqlens and the page table on the device
// inside its CUDA-graph hooks, mini_sglang/layers/attn/fa3_attn_backend.py:50-81,221-233).  The block tables of a cache
// group are mirrored in device memory; the host sends, per step, what changed in them (whole rows of the requests that
// got a page) and three numbers per request; the fields that the captured graph reads are written here.
// ---------------------------------------------------------------------------------------
// deltas: [n, (slot, count, offset) x n, page ids ...]: row `slot` of the mirror gets `count` page ids from deltas[offset..]
__global__ void table_delta_kernel(const int* __restrict__ deltas, int* __restrict__ table, int row_stride) {
    const int rec = blockIdx.x;
    const int slot = deltas[1 + 3 * rec], count = min(deltas[2 + 3 * rec], row_stride), off = deltas[3 + 3 * rec];
    for (int i = threadIdx.x; i < count; i += blockDim.x) table[(size_t)slot * row_stride + i] = deltas[off + i];
}

// One block per row r of a captured batch of b rows, the first B of them live: request slot[r] feeds token id[r] at position
// pos[r].  Rows past B are padding: a request of one token on the dump page.  common != 0: the fields that all cache groups
// share are written too.
__global__ void decode_meta_kernel(const int* __restrict__ id, const int* __restrict__ slot, const int* __restrict__ pos,
                                   const int* __restrict__ nsplit_in, int B, int b, const int* __restrict__ table, int row_stride,
                                   int page_size, int mp, int common, int* __restrict__ input_ids, int* __restrict__ positions,
                                   int* __restrict__ token_req, int* __restrict__ q_start, int* __restrict__ kv_len,
                                   int* __restrict__ slots, int* __restrict__ out_loc, int* __restrict__ nsplit,
                                   int* __restrict__ block_table, int window, int* __restrict__ order,
                                   const int* __restrict__ even_in, int* __restrict__ even_out, int n_even) {
    const int r = blockIdx.x;
    // the even cut of the step's keys comes ready-made from the host: the blocks copy it between them
    for (int i = r * blockDim.x + threadIdx.x; i < n_even; i += b * blockDim.x) even_out[i] = even_in[i];
    const bool live = r < B;
    const int sl = live ? slot[r] : 0, ps = live ? pos[r] : 0;
    const int* row = table + (size_t)sl * row_stride;
    // order[i] = the row with the i-th most keys per kv split (ties: the lower row first; padding rows last): this
    // row's place is the number of rows that come before it
    __shared__ int before;
    if (threadIdx.x == 0) before = 0;
    __syncthreads();
    {
        auto load_of = [&](int j) -> int {
            if (j >= B) return 0;
            int keys = pos[j] + 1;
            if (window > 0) keys = min(keys, window + 1);
            return (keys + max(nsplit_in[j], 1) - 1) / max(nsplit_in[j], 1);
        };
        const int mine = load_of(r);
        int n = 0;
        for (int j = threadIdx.x; j < b; j += blockDim.x) {
            const int other = load_of(j);
            n += (other > mine || (other == mine && j < r)) ? 1 : 0;
        }
        if (n) atomicAdd(&before, n);
    }
    __syncthreads();
    if (threadIdx.x == 0) order[before] = r;
    if (threadIdx.x == 0) {
        if (common) {
            input_ids[r] = live ? id[r] : 0;
            positions[r] = ps;
            token_req[r] = r;
            q_start[r] = r;
            if (r == b - 1) q_start[b] = b;
            kv_len[r] = ps + 1;
            slots[r] = sl;
        }
        const int pi = ps / page_size;
        out_loc[r] = (live && pi < row_stride) ? row[pi] * page_size + (ps - pi * page_size) : 0;
        nsplit[r] = live ? nsplit_in[r] : 1;
    }
    for (int i = threadIdx.x; i < mp; i += blockDim.x) block_table[(size_t)r * mp + i] = (live && i < row_stride) ? row[i] : 0;
}

MSGL_API int msgl_table_delta(const int* deltas, int n_records, int* table, int row_stride, cudaStream_t stream) {
    if (n_records <= 0) return MSGL_OK;
    table_delta_kernel<<<n_records, 128, 0, stream>>>(deltas, table, row_stride);
    return msgl_check_launch();
}

MSGL_API int msgl_decode_meta(const int* id, const int* slot, const int* pos, const int* nsplit_in, int B, int b, const int* table,
                              int row_stride, int page_size, int mp, int common, int* input_ids, int* positions, int* token_req,
                              int* q_start, int* kv_len, int* slots, int* out_loc, int* nsplit, int* block_table,
                              int window, int* order, const int* even_in, int* even_out, int n_even, cudaStream_t stream) {
    if (b <= 0) return MSGL_OK;
    if (B < 0 || B > b || page_size < 1 || mp < 1 || row_stride < 1 || order == nullptr) return MSGL_ERR_SIZE;
    if (n_even < 0 || (n_even > 0 && (even_in == nullptr || even_out == nullptr))) return MSGL_ERR_SIZE;
    decode_meta_kernel<<<b, 128, 0, stream>>>(id, slot, pos, nsplit_in, B, b, table, row_stride, page_size, mp, common, input_ids,
                                             positions, token_req, q_start, kv_len, slots, out_loc, nsplit, block_table,
                                             window, order, even_in, even_out, n_even);
    return msgl_check_launch();
}

MSGL_API int msgl_embedding(const int* ids, const void* table, float* out, int T_, int H, int V,
                            int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
    if (dtype == MSGL_F32)
        msgl_launch_pdl(embedding_kernel<float>, dim3(T_), dim3(threads), 0, stream, ids, (const float*)table, out, H, V);
    else if (dtype == MSGL_BF16)
        msgl_launch_pdl(embedding_kernel<__nv_bfloat16>, dim3(T_), dim3(threads), 0, stream, ids, (const __nv_bfloat16*)table, out, H, V);
    else
        return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// RMSNorm, optionally with the residual sum in front and a row gather:
//   v      = (res_in ? res_in[src] : 0) + (x ? float(x[src]) : 0)        src = row_idx ? row_idx[r] : r
//   res_out[r] = v                                                        (if res_out)
//   y[r]   = T(v * rsqrt(mean(v^2) + eps) * w)
// One block per row; the row is kept in shared memory between the two passes when it fits.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const float* res_in, float* res_out,
                               const int* __restrict__ row_idx, const void* __restrict__ w, int w_is_f32,
                               float eps, T* __restrict__ y, int H, int cache_row) {
    extern __shared__ float srow[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t src = (size_t)(row_idx ? row_idx[r] : r) * H;
    const size_t dst = (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = 0.f;
        if (res_in) v = res_in[src + i];
        if (x) v += to_f32<T>(x[src + i]);
        if (res_out) res_out[dst + i] = v;
        if (cache_row) srow[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v;
        if (cache_row) {
            v = srow[i];
        } else {  // row too long for shared memory: recompute from the inputs
            v = 0.f;
            if (res_out) v = res_out[dst + i];
            else {
                if (res_in) v = res_in[src + i];
                if (x) v += to_f32<T>(x[src + i]);
            }
        }
        y[dst + i] = from_f32<T>(v * inv * load_weight(w, i, w_is_f32));
    }
}

// Vectorised variant: 8 elements per thread and pass, the whole row held in registers between the
// two passes (VPT vectors per thread).  Used when the row length is a multiple of 8 and every
// pointer is 16-byte aligned; same arithmetic and the same reduction tree per launch shape.
template <typename T> struct Vec8 {};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
        *reinterpret_cast<uint4*>(p) = u;
    }
};

template <typename T, int VPT>
__global__ void rmsnorm_vec_kernel(const T* __restrict__ x, const float* res_in, float* res_out,
                                   const int* __restrict__ row_idx, const void* __restrict__ w, int w_is_f32,
                                   float eps, T* __restrict__ y, int H) {
    __shared__ float red[32];
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const size_t src = (size_t)(row_idx ? row_idx[r] : r) * H;
    const size_t dst = (size_t)r * H;
    const int nvec = H >> 3;
    // the norm's weights (and the row index) are nobody's output: fetched while the kernel before this one finishes
    float wv[VPT][8];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) << 3;
        if ((i >> 3) < nvec) {
            if (w_is_f32) Vec8<float>::load(reinterpret_cast<const float*>(w) + i, wv[j]);
            else Vec8<__nv_bfloat16>::load(reinterpret_cast<const __nv_bfloat16*>(w) + i, wv[j]);
        }
    }
    pdl_wait();
    pdl_after_wait();
    pdl_small();
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) << 3;
        if ((i >> 3) < nvec) {
            if (res_in) Vec8<float>::load(res_in + src + i, v[j]);
            else {
#pragma unroll
                for (int k = 0; k < 8; ++k) v[j][k] = 0.f;
            }
            if (x) {
                float xv[8];
                Vec8<T>::load(x + src + i, xv);
#pragma unroll
                for (int k = 0; k < 8; ++k) v[j][k] += xv[k];
            }
            if (res_out) Vec8<float>::store(res_out + dst + i, v[j]);
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += v[j][k] * v[j][k];
        }
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) << 3;
        if ((i >> 3) < nvec) {
            float o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = v[j][k] * inv * wv[j][k];
            Vec8<T>::store(y + dst + i, o);
        }
    }
}

template <typename T>
static bool launch_rmsnorm_vec(const void* x, const float* res_in, float* res_out, const int* row_idx, const void* w,
                               int w_is_f32, float eps, void* y, int rows, int H, cudaStream_t stream) {
    const uintptr_t all = (uintptr_t)x | (uintptr_t)res_in | (uintptr_t)res_out | (uintptr_t)w | (uintptr_t)y;
    if ((H & 7) || (all & 15)) return false;
    const int nvec = H >> 3;
    int threads = ((nvec + 31) / 32) * 32;
    int vpt = 1;
    while (threads > 512) { vpt *= 2; threads = (((nvec + vpt - 1) / vpt + 31) / 32) * 32; }
    if (vpt > 4) return false;
    const T* xp = (const T*)x;
    T* yp = (T*)y;
    if (vpt == 1) msgl_launch_pdl(rmsnorm_vec_kernel<T, 1>, dim3(rows), dim3(threads), 0, stream, xp, res_in, res_out, row_idx, w, w_is_f32, eps, yp, H);
    else if (vpt == 2) msgl_launch_pdl(rmsnorm_vec_kernel<T, 2>, dim3(rows), dim3(threads), 0, stream, xp, res_in, res_out, row_idx, w, w_is_f32, eps, yp, H);
    else msgl_launch_pdl(rmsnorm_vec_kernel<T, 4>, dim3(rows), dim3(threads), 0, stream, xp, res_in, res_out, row_idx, w, w_is_f32, eps, yp, H);
    return true;
}

MSGL_API int msgl_rmsnorm(const void* x, const float* res_in, float* res_out, const int* row_idx,
                          const void* w, int w_is_f32, float eps, void* y, int rows, int H,
                          int dtype, cudaStream_t stream) {
    if (rows <= 0) return MSGL_OK;
    if (H <= 0) return MSGL_ERR_SIZE;
    if (dtype == MSGL_F32 && launch_rmsnorm_vec<float>(x, res_in, res_out, row_idx, w, w_is_f32, eps, y, rows, H, stream))
        return msgl_check_launch();
    if (dtype == MSGL_BF16 && launch_rmsnorm_vec<__nv_bfloat16>(x, res_in, res_out, row_idx, w, w_is_f32, eps, y, rows, H, stream))
        return msgl_check_launch();
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const int cache_row = (size_t)H * 4 <= 40 * 1024;
    const size_t smem = cache_row ? (size_t)H * 4 : 0;
    if (dtype == MSGL_F32)
        rmsnorm_kernel<float><<<rows, threads, smem, stream>>>((const float*)x, res_in, res_out, row_idx, w, w_is_f32,
                                                               eps, (float*)y, H, cache_row);
    else if (dtype == MSGL_BF16)
        rmsnorm_kernel<__nv_bfloat16><<<rows, threads, smem, stream>>>((const __nv_bfloat16*)x, res_in, res_out, row_idx,
                                                                       w, w_is_f32, eps, (__nv_bfloat16*)y, H, cache_row);
    else
        return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// q/k per-head RMSNorm (optional) + rotary position encoding from a float32 table (optional)
// + write of k and v into the paged cache + q to a dense buffer.  One warp per (token, head).
//
//   qkv row layout: [ q: n_q*d | k: n_kv*d | v: n_kv*d ],  row stride `qkv_stride` elements
//   table: [max_pos, rot] float32 = cos(angles) | sin(angles), rot/2 each; halves of the
//          first `rot` elements of a head are rotated against each other: halves (element i with i + rot/2, NeoX style)
//          or, with `interleaved`, neighbours (2 p with 2 p + 1)
//   cache layout per layer: [page][kv head][slot in page][d]; token slot s = page*P + offset
// ---------------------------------------------------------------------------------------
#define QKR_MAX_PER_LANE 16   // head sizes up to 512

template <typename T>
__global__ void qknorm_rope_kvwrite_kernel(const T* __restrict__ qkv, int qkv_stride,
                                           const int* __restrict__ positions, const int* __restrict__ out_loc,
                                           const void* __restrict__ qw, const void* __restrict__ kw, int w_is_f32,
                                           float eps, const float* __restrict__ table, int rot, int max_pos,
                                           T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                           int page_size, int n_q, int n_kv, int d, int interleaved) {
    const int t = blockIdx.x;
    const int warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * warps + (threadIdx.x >> 5);
    const int n_heads = n_q + 2 * n_kv;
    if (head >= n_heads) return;
    const bool is_q = head < n_q;
    const bool is_k = !is_q && head < n_q + n_kv;
    const bool writes_cache = (k_cache != nullptr) && (out_loc != nullptr);
    if (!is_q && !writes_cache) return;

    const T* src = qkv + (size_t)t * qkv_stride + (size_t)head * d;
    float v[QKR_MAX_PER_LANE];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < QKR_MAX_PER_LANE; ++j) {
        const int i = lane + 32 * j;
        v[j] = (i < d) ? to_f32<T>(src[i]) : 0.f;
        ss += v[j] * v[j];
    }
    const void* nw = is_q ? qw : (is_k ? kw : nullptr);
    if (nw != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
        for (int j = 0; j < QKR_MAX_PER_LANE; ++j) {
            const int i = lane + 32 * j;
            if (i < d) v[j] = v[j] * inv * load_weight(nw, i, w_is_f32);
        }
    }
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * n_q + head) * d;
    } else {
        const int slot = out_loc[t];
        const int page = slot / page_size, off = slot - page * page_size;
        const int kvh = is_k ? head - n_q : head - n_q - n_kv;
        T* base = is_k ? k_cache : v_cache;
        dst = base + (((size_t)page * n_kv + kvh) * page_size + off) * d;
    }
    if (table != nullptr && (is_q || is_k)) {
        // rotate: element i < rot/2 pairs with i + rot/2.  The partner lives in another lane or
        // register, so the head goes through shared memory once.
        extern __shared__ float sh[];
        float* hv = sh + (size_t)(threadIdx.x >> 5) * d;
#pragma unroll
        for (int j = 0; j < QKR_MAX_PER_LANE; ++j) {
            const int i = lane + 32 * j;
            if (i < d) hv[i] = v[j];
        }
        __syncwarp();
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
        const float* cs = table + (size_t)pos * rot;
        const int half = rot >> 1;
        for (int i = lane; i < d; i += 32) {
            float o;
            if (i >= rot) {
                o = hv[i];
            } else if (interleaved) {           // pairs (2 p, 2 p + 1) share angle p
                const int p = i >> 1;
                o = (i & 1) ? hv[i - 1] * cs[half + p] + hv[i] * cs[p] : hv[i] * cs[p] - hv[i + 1] * cs[half + p];
            } else if (i < half) {              // halves: element i pairs with i + rot / 2
                o = hv[i] * cs[i] - hv[i + half] * cs[half + i];
            } else {
                const int p = i - half;
                o = hv[p] * cs[half + p] + hv[i] * cs[p];
            }
            dst[i] = from_f32<T>(o);
        }
    } else {
#pragma unroll
        for (int j = 0; j < QKR_MAX_PER_LANE; ++j) {
            const int i = lane + 32 * j;
            if (i < d) dst[i] = from_f32<T>(v[j]);
        }
    }
}

// Fast path for head sizes 32, 64, 128, 256 with full rotation: a lane owns E = d / 32 consecutive
// elements, so loads and stores are contiguous, and its rotation partner (element + d/2) sits in
// lane ^ 16 -- no shared memory.  Same arithmetic as the general kernel above.
// E consecutive elements of T as one access of E * sizeof(T) bytes (2 ... 32 bytes, aligned to that size)
template <typename T, int E> struct Pack {
    static constexpr int BYTES = E * (int)sizeof(T);
    static __device__ __forceinline__ void load(const T* p, float (&v)[E]) {
        __align__(16) T tmp[E];
        if constexpr (BYTES == 32) {
            reinterpret_cast<uint4*>(tmp)[0] = reinterpret_cast<const uint4*>(p)[0];
            reinterpret_cast<uint4*>(tmp)[1] = reinterpret_cast<const uint4*>(p)[1];
        } else if constexpr (BYTES == 16) {
            *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(p);
        } else if constexpr (BYTES == 8) {
            *reinterpret_cast<uint2*>(tmp) = *reinterpret_cast<const uint2*>(p);
        } else if constexpr (BYTES == 4) {
            *reinterpret_cast<unsigned*>(tmp) = *reinterpret_cast<const unsigned*>(p);
        } else {
#pragma unroll
            for (int j = 0; j < E; ++j) tmp[j] = p[j];
        }
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = to_f32<T>(tmp[j]);
    }
    static __device__ __forceinline__ void store(T* p, const float (&v)[E]) {
        __align__(16) T tmp[E];
#pragma unroll
        for (int j = 0; j < E; ++j) tmp[j] = from_f32<T>(v[j]);
        if constexpr (BYTES == 32) {
            reinterpret_cast<uint4*>(p)[0] = reinterpret_cast<const uint4*>(tmp)[0];
            reinterpret_cast<uint4*>(p)[1] = reinterpret_cast<const uint4*>(tmp)[1];
        } else if constexpr (BYTES == 16) {
            *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(tmp);
        } else if constexpr (BYTES == 8) {
            *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(tmp);
        } else if constexpr (BYTES == 4) {
            *reinterpret_cast<unsigned*>(p) = *reinterpret_cast<const unsigned*>(tmp);
        } else {
#pragma unroll
            for (int j = 0; j < E; ++j) p[j] = tmp[j];
        }
    }
};

// A warp owns one head of QKR_TOK consecutive tokens: their rows are fetched first, then worked on one after the
// other, so that several loads are in flight per lane (one token a warp leaves the kernel bound by block turnover).
constexpr int QKR_TOK = 4;
template <typename T, int E>
__global__ void qknorm_rope_kvwrite_vec_kernel(const T* __restrict__ qkv, int qkv_stride,
                                               const int* __restrict__ positions, const int* __restrict__ out_loc,
                                               const void* __restrict__ qw, const void* __restrict__ kw, int w_is_f32,
                                               float eps, const float* __restrict__ table, int max_pos,
                                               T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                               int page_size, int n_q, int n_kv, int T_) {
    constexpr int d = 32 * E;
    pdl_launch_dependents();
    const int t0 = blockIdx.x * QKR_TOK;
    const int warps = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * warps + (threadIdx.x >> 5);
    const int n_heads = n_q + 2 * n_kv;
    if (head >= n_heads) return;
    const bool is_q = head < n_q;
    const bool is_k = !is_q && head < n_q + n_kv;
    const bool writes_cache = (k_cache != nullptr) && (out_loc != nullptr);
    if (!is_q && !writes_cache) return;

    // positions, cache slots and norm weights are nobody's output: fetched while the kernel before this one finishes
    float v[QKR_TOK][E];
    int pos[QKR_TOK], slot[QKR_TOK];
#pragma unroll
    for (int i = 0; i < QKR_TOK; ++i) {
        const int t = t0 + i < T_ ? t0 + i : T_ - 1;                     // past the end: the last token again, not stored
        pos[i] = (table != nullptr && (is_q || is_k)) ? positions[t] : 0;
        slot[i] = is_q ? 0 : out_loc[t];
    }
    const void* nw = is_q ? qw : (is_k ? kw : nullptr);
    float w[E];
    if (nw != nullptr) {
#pragma unroll
        for (int j = 0; j < E; ++j) w[j] = load_weight(nw, lane * E + j, w_is_f32);
    }
    pdl_wait();
    pdl_after_wait();
    pdl_small();
#pragma unroll
    for (int i = 0; i < QKR_TOK; ++i) {
        const int t = t0 + i < T_ ? t0 + i : T_ - 1;
        Pack<T, E>::load(qkv + (size_t)t * qkv_stride + (size_t)head * d + lane * E, v[i]);
    }
#pragma unroll
    for (int i = 0; i < QKR_TOK; ++i) {
        if (t0 + i >= T_) break;
        if (nw != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < E; ++j) ss += v[i][j] * v[i][j];
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)d + eps);
#pragma unroll
            for (int j = 0; j < E; ++j) v[i][j] = v[i][j] * inv * w[j];
        }
        if (table != nullptr && (is_q || is_k)) {
            const int ps = pos[i] < 0 ? 0 : (pos[i] >= max_pos ? max_pos - 1 : pos[i]);
            const float* cs = table + (size_t)ps * d;
            const int pi = (lane & 15) * E;           // index of the pair within the half
            const bool upper = lane >= 16;
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, v[i][j], 16);
                const float c = cs[pi + j], sn = cs[d / 2 + pi + j];
                v[i][j] = upper ? (other * sn + v[i][j] * c) : (v[i][j] * c - other * sn);
            }
        }
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)(t0 + i) * n_q + head) * d;
        } else {
            const int page = slot[i] / page_size, off = slot[i] - page * page_size;
            const int kvh = is_k ? head - n_q : head - n_q - n_kv;
            T* base = is_k ? k_cache : v_cache;
            dst = base + (((size_t)page * n_kv + kvh) * page_size + off) * d;
        }
        Pack<T, E>::store(dst + lane * E, v[i]);
    }
}

MSGL_API int msgl_qknorm_rope_kvwrite(const void* qkv, int qkv_stride, const int* positions, const int* out_loc,
                                      const void* qw, const void* kw, int w_is_f32, float eps,
                                      const float* table, int rot, int max_pos, void* q_out, void* k_cache,
                                      void* v_cache, int page_size, int n_q, int n_kv, int d, int T_, int dtype,
                                      int interleaved, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (d <= 0 || d > 32 * QKR_MAX_PER_LANE || rot < 0 || rot > d || (rot & 1) || page_size <= 0) return MSGL_ERR_SIZE;
    const int n_heads = n_q + 2 * n_kv;
    const int warps = n_heads < 8 ? n_heads : 8;
    dim3 grid(T_, (n_heads + warps - 1) / warps);
    const size_t smem = table ? (size_t)warps * d * sizeof(float) : 0;
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 31) == 0 &&
                         (qkv_stride % (d / 32 > 0 ? d / 32 : 1)) == 0;
    if (aligned && (d == 32 || d == 64 || d == 128 || d == 256) && (table == nullptr || (rot == d && !interleaved)) &&
        (dtype == MSGL_F32 || dtype == MSGL_BF16)) {
#define QKR_VEC(TT, EE)                                                                                              \
    msgl_launch_pdl(qknorm_rope_kvwrite_vec_kernel<TT, EE>, dim3((T_ + QKR_TOK - 1) / QKR_TOK, grid.y), dim3(warps * 32), 0, stream, \
        (const TT*)qkv, qkv_stride, positions, out_loc, qw, kw, w_is_f32, eps, table, max_pos, (TT*)q_out,           \
        (TT*)k_cache, (TT*)v_cache, page_size, n_q, n_kv, T_)
        const int E = d / 32;
        if (dtype == MSGL_F32) {
            if (E == 1) QKR_VEC(float, 1); else if (E == 2) QKR_VEC(float, 2); else if (E == 4) QKR_VEC(float, 4); else QKR_VEC(float, 8);
        } else {
            if (E == 1) QKR_VEC(__nv_bfloat16, 1); else if (E == 2) QKR_VEC(__nv_bfloat16, 2);
            else if (E == 4) QKR_VEC(__nv_bfloat16, 4); else QKR_VEC(__nv_bfloat16, 8);
        }
#undef QKR_VEC
        return msgl_check_launch();
    }
    if (dtype == MSGL_F32)
        qknorm_rope_kvwrite_kernel<float><<<grid, warps * 32, smem, stream>>>(
            (const float*)qkv, qkv_stride, positions, out_loc, qw, kw, w_is_f32, eps, table, rot, max_pos,
            (float*)q_out, (float*)k_cache, (float*)v_cache, page_size, n_q, n_kv, d, interleaved);
    else if (dtype == MSGL_BF16)
        qknorm_rope_kvwrite_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
            (const __nv_bfloat16*)qkv, qkv_stride, positions, out_loc, qw, kw, w_is_f32, eps, table, rot, max_pos,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, page_size, n_q, n_kv, d, interleaved);
    else
        return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(a) = a / (1 + exp(-a)) in float32
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float a = to_f32<T>(gu[t * 2 * I + i]);
        const float b = to_f32<T>(gu[t * 2 * I + I + i]);
        out[idx] = from_f32<T>(a / (1.f + expf(-a)) * b);
    }
}

// 8 bfloat16 per thread and step when the row width allows it; a block walks one token row, two steps' loads ahead
__global__ void swiglu_bf16x8_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out, int I8) {
    const uint4* row = gu + (size_t)blockIdx.x * 2 * I8;
    uint4* orow = out + (size_t)blockIdx.x * I8;
    auto act = [](const uint4& a, const uint4& b) -> uint4 {
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 af = __bfloat1622float2(ap[k]);
            const float2 bf = __bfloat1622float2(bp[k]);
            op[k] = __floats2bfloat162_rn(af.x / (1.f + expf(-af.x)) * bf.x, af.y / (1.f + expf(-af.y)) * bf.y);
        }
        return o;
    };
    int i = threadIdx.x;
    for (; i + (int)blockDim.x < I8; i += 2 * blockDim.x) {
        const int i2 = i + blockDim.x;
        const uint4 a0 = row[i], b0 = row[I8 + i], a1 = row[i2], b1 = row[I8 + i2];
        orow[i] = act(a0, b0);
        orow[i2] = act(a1, b1);
    }
    if (i < I8) orow[i] = act(row[i], row[I8 + i]);
}

MSGL_API int msgl_swiglu(const void* gu, void* out, int T_, int I, int dtype, cudaStream_t stream) {
    if (T_ <= 0) return MSGL_OK;
    if (I <= 0) return MSGL_ERR_SIZE;
    const size_t total = (size_t)T_ * I;
    const int threads = 256;
    if (dtype == MSGL_BF16 && (I % 8) == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        swiglu_bf16x8_kernel<<<(unsigned)T_, threads, 0, stream>>>((const uint4*)gu, (uint4*)out, I / 8);
        return msgl_check_launch();
    }
    size_t blocks = (total + threads - 1) / threads;
    const size_t most = (size_t)msgl_sm_count() * 32;      // grid-stride beyond 32 blocks an SM
    if (blocks > most) blocks = most;
    if (dtype == MSGL_F32)
        swiglu_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
    else if (dtype == MSGL_BF16)
        swiglu_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu,
                                                                               (__nv_bfloat16*)out, I, total);
    else
        return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}

// ---------------------------------------------------------------------------------------
// float32 -> T conversion of rows (used where a float32 stream feeds a T consumer)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ in, T* __restrict__ out, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(in[i]);
}

MSGL_API int msgl_cast_from_f32(const float* in, void* out, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return MSGL_OK;
    size_t blocks = ((size_t)n + 255) / 256;
    const size_t most = (size_t)msgl_sm_count() * 32;      // grid-stride beyond 32 blocks an SM
    if (blocks > most) blocks = most;
    if (dtype == MSGL_F32)
        cast_from_f32_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>(in, (float*)out, (size_t)n);
    else if (dtype == MSGL_BF16)
        cast_from_f32_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(in, (__nv_bfloat16*)out, (size_t)n);
    else
        return MSGL_ERR_DTYPE;
    return msgl_check_launch();
}
