// One persistent kernel for a whole decode step of a few requests (one new token each).
//
// A decode step of a dense decoder is a chain of about nine short kernels per layer (norm, qkv product, q/k
// norm + rotation + cache write, attention over the cache, merge of the kv splits, output product, norm,
// gate/up product, down product).  With up to 8 tokens every product only streams its weights once, so the
// step is bound by memory, and what it loses against that bound is mostly the hand-over between kernels: each
// boundary drains the memory pipe and fills it again (measured on B200 at Qwen3-8B's sizes: about 3.6 us per
// boundary, 325 boundaries, 1.2 of 4.1 ms).  Here the whole step is ONE launch of as many blocks as the GPU
// holds at once (cooperative launch); the blocks walk the phases of every layer together and meet at a grid
// barrier between phases.  Before a block waits at a barrier it has already asked for the first weights of
// its next piece of work (they do not depend on anything computed in the step), so the weight stream goes on
// across the barrier.
//
// Phases of a layer (5 barriers); in every product a block owns an equal share of the weight rows:
//   A  qkv = norm_in(res) . Wqkv^T (+ b)        x = bf16(res * w_norm) was written by the phase that produced res,
//                                               with partial sums of res^2; the outputs are scaled by
//                                               rsqrt(mean + eps) at the end, which is the normed product
//   B  attention of every (request, kv head, kv split): q heads normed and rotated on the fly; the piece that
//      holds a request's last keys norms and rotates the new key, writes key and value into the paged cache and
//      takes them into its own sums from shared memory; the piece that finishes a (request, kv head) last (a
//      ticket) merges the splits, in split order
//   C  res += attn . Wo^T                       the residual sum is the product's epilogue (float32, in place), and
//                                               with it bf16(res * w_post) and the partial sums of res^2 for D
//   D  act = silu(g) * u, [g; u] = norm_post(res) . Wgu^T     scaled as in A
//   E  res += act . Wdown^T                     with bf16(res * w) for the norm that comes next (next layer's, or the final one)
// then the head: logits = norm_final(res) . Wlm^T in float32.
//
// What a block reads that another block wrote during the step is read past the L1 cache (ld.global.cg /
// cp.async.cg) or after a grid barrier, whose acquire makes the SM drop what its L1 held: L1 is not coherent between
// SMs and the kernel does not end between a write and its reads.  Weights, tables and the cache contents of earlier steps never change while the
// kernel runs.
//
// Every wait has a limit (polls and time); a block that gives up sets a status word, which ends the waits of all
// others, and every block returns.  Nothing is left to free.
//
// Sizes: bfloat16; up to 8 requests; head size MSGL_HEAD_DIM (a multiple of 32); up to 16 query heads per kv head;
// hidden and intermediate sizes multiples of 32; all keys kept (no window).  The entry point refuses anything
// else (MSGL_ERR_SIZE) and the caller takes the kernel-by-kernel path.
#include "common.cuh"
#include <math.h>

#ifndef MSGL_HEAD_DIM
#define MSGL_HEAD_DIM 128
#endif

namespace ds {

constexpr int WARPS = 16;          // one block of 16 warps per SM (ring depth 6 measured faster than 8 and 5)
constexpr int THREADS = WARPS * 32;
#ifndef MSGL_DS_PF
#define MSGL_DS_PF 6
#endif
constexpr int PF = MSGL_DS_PF;     // weight chunks in flight per warp
constexpr int WT = 16;             // keys per warp unit of the attention phase
constexpr int ST = 2;              // V stages per warp
constexpr int KT = 64;             // key tiles by which a request's keys are cut into splits (anchored at position 0)
constexpr int D = MSGL_HEAD_DIM;
constexpr int LDS = D + 8;         // row pitch of key/value/query tiles in shared memory (elements)
constexpr int MAX_M = 8;

typedef __nv_bfloat16 bf16;

}  // namespace ds

// One run of a layer.  Plain C layout: the host fills an array of these and copies it to the device once.
struct DsLayer {
    const void* w_qkv;        // [(n_q + 2 n_kv) d, H]
    const void* b_qkv;        // [(n_q + 2 n_kv) d] or null
    const void* w_o;          // [H, n_q d]
    const void* w_gu;         // [2 I, H], gate rows first
    const void* w_down;       // [H, I]
    const void* norm_in;      // [H]
    const void* norm_post;    // [H]
    const void* q_norm;       // [d] or null
    const void* k_norm;       // [d] or null
    void* k_cache;            // [pages + 1, n_kv, page, d]
    void* v_cache;
    float eps_in, eps_post, eps_qk;
    int norm_f32;             // norm_in / norm_post weights are float32 (else bfloat16)
    int qk_norm_f32;
    int pad_;
};

struct DsStep {
    const DsLayer* layers;
    int n_layers;
    int M;                                   // requests = tokens of the step
    int H, n_q, n_kv, I, V;
    int page_size, page_shift, bt_stride, max_split;
    float scale;
    const float* rope;                       // [max_pos, rot] cos | sin, or null
    int rot, max_pos;
    const int* ids;                          // [M]
    const int* positions;                    // [M]
    const int* kv_len;                       // [M] keys of the request including the new one
    const int* block_table;                  // [M, bt_stride]
    const int* out_loc;                      // [M] cache slot of the new token (page * page_size + offset)
    const int* nsplit;                       // [M] or null
    const void* embed;                       // [V, H] bfloat16
    const void* final_norm;                  // [H]
    int final_f32;
    float eps_final;
    const void* lm_head;                     // [V, H]
    float* res;                              // [M, H]       scratch from here on
    void* xn;                                // [M, H] bf16(res * weight of the next norm)
    float* ssq;                              // [blocks, 8] partial sums of res^2 per token
    void* qkv;                               // [M, (n_q + 2 n_kv) d]
    void* attn;                              // [M, n_q d]
    void* act;                               // [M, I]
    float* part_o;                           // [max_split, M, n_q, d]
    float* part_ml;                          // [max_split, M, n_q, 2]
    int* tickets;                            // [M * n_kv], zero between launches
    float* logits;                           // [M, V] out
    unsigned* bar;                           // grid barrier counter, zeroed by the entry point before the launch
    int* status;                             // word 0 set to 1 if a wait ran out
};

namespace ds {

// ---------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s_ = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s_), "l"(gmem));
}
__device__ __forceinline__ void cp_async16_if(void* smem, const void* gmem, bool valid) {
    const unsigned s_ = (unsigned)__cvta_generic_to_shared(smem);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s_), "l"(gmem), "r"(n));
}
#ifndef MSGL_DS_X_CA
#define MSGL_DS_X_CA 1
#endif
// x rows are read by every block of an SM: with .ca the second block finds them in L1.  Safe after a grid barrier: its
// acquire makes the SM drop what L1 held before.
__device__ __forceinline__ void cp_async16_x(void* smem, const void* gmem) {
    const unsigned s_ = (unsigned)__cvta_generic_to_shared(smem);
#if MSGL_DS_X_CA
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(s_), "l"(gmem));
#else
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s_), "l"(gmem));
#endif
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ unsigned movmatrix_trans(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {       // weights / old keys: read once, never written here
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float ld_w(const void* w, int i, int f32) {
    return f32 ? reinterpret_cast<const float*>(w)[i] : __bfloat162float(reinterpret_cast<const bf16*>(w)[i]);
}

// ---------------------------------------------------------------------------------------
// grid barrier: a counter that only grows; the n-th barrier is passed when it reaches n * blocks
// ---------------------------------------------------------------------------------------
#ifndef MSGL_DS_PROFILE
#define MSGL_DS_PROFILE 0
#endif

struct GridBar {
    unsigned* counter;
    int* status;
    unsigned target;       // value the counter has when every block has arrived at the current barrier
    unsigned blocks;
    unsigned long long t_pass;     // MSGL_DS_PROFILE: when thread 0 passed the last barrier
};

__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

// true: every block has arrived and what they wrote before is visible.  false: the wait ran out (or another block's
// did): the caller returns at once.
__device__ __forceinline__ bool grid_sync(GridBar& b) {
    __shared__ int sh_ok;
    b.target += b.blocks;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(b.counter, 1u);
        int ok = 1;
        unsigned polls = 0;
        unsigned long long t0 = 0;
        while (ld_acquire(b.counter) < b.target) {
            ++polls;
            if ((polls & 1023u) == 0) {
                if (t0 == 0) t0 = global_ns();
                // two seconds, or 2^28 polls whatever the timer says, or another block has given up
                if (global_ns() - t0 > 2000000000ull || polls > (1u << 28) || *reinterpret_cast<volatile int*>(b.status) != 0) {
                    atomicExch(b.status, 1);
                    ok = 0;
                    break;
                }
            }
        }
        __threadfence();
        sh_ok = ok;
#if MSGL_DS_PROFILE
        b.t_pass = global_ns();
#endif
    }
    __syncthreads();
    return sh_ok != 0;
}

}  // namespace ds

namespace ds {

// ---------------------------------------------------------------------------------------
// matrix products of the step: out[M, N] = x[M, K] . W[N, K]^T for M <= 8, bound by reading W once
// ---------------------------------------------------------------------------------------
// Every block owns an equal share of W's rows (N / blocks of them, give or take one), so the blocks of a phase finish
// together and the barrier behind it is short.  A block walks its rows in tiles of 16 (8 gate rows and their 8 up rows
// with SwiGLU; the last tile may be short: rows past the block's share are not fetched).  The warps take the 32-element
// chunks of K round-robin and every lane copies 16 bytes of two weight rows per chunk with cp.async into a slot of its
// own in a shared-memory ring, PF chunks ahead, straight into the register layout of mma.sync's A operand (the k index
// inside a chunk is permuted the same way for W and x).  The ring runs on across the tiles, and it is started BEFORE the
// grid barrier that guards the phase's input.
//
// x is bfloat16 [M, K] in global memory, either copied whole into shared memory once per block (XSRC 1; K * 16 bytes
// whatever M) or streamed chunk by chunk through the ring (XSRC 0, for the long K of the down product).
//
// A norm in front of a product is folded in like this: the phase that produces the residual stream (EPI 2) also writes
// xn = bf16(res * w_next), the un-scaled input of the next product, for the columns it owns, and the sum of res^2 over
// those columns per token (one partial per block, added in block order by the reader).  The product that follows
// multiplies its sums by rsqrt(mean(res^2) + eps): the scale is one number per row, so this is the normed product.
struct GemmJob {
    const bf16* W;
    int n_rows;                  // output columns (SwiGLU: gate/up pairs = I)
    int K, I, M;
    const bf16* X;               // [M, ldx] bfloat16
    long long ldx;
    const float* ssq;            // not null: [producer blocks][8] partial sums of squares of x's float32 source
    int n_ssq;
    float eps;
    const bf16* bias;
    void* out;
    long long ldo;
    // EPI 2: what the next product wants of the stream
    const void* next_w;          // its norm's weight [H]
    int next_w_f32;
    bf16* xn;                    // [M, ldo] bf16(res * next_w)
    float* ssq_out;              // [blocks][8]
};

constexpr int RING2_BYTES = WARPS * PF * 2 * 512;
constexpr int RING3_BYTES = WARPS * PF * 3 * 512;
constexpr int RED_FLOATS = WARPS * 16 * 9;
constexpr int RED_BYTES = (RED_FLOATS + 128 + 8) * 4;

// MODE 0: plain, 1: SwiGLU.  XSRC 1: x staged whole in shared memory, 0: streamed.  EPI 0: bfloat16 out, 1: float32
// out, 2: added into the float32 residual stream, with xn and the partial sums of squares for the next product.
template <int MODE, int XSRC, int EPI>
__device__ __forceinline__ bool gemm_phase(const GemmJob& j, unsigned char* sm, int arena, GridBar& bar) {
    constexpr int SLOTS = XSRC ? 2 : 3;
    uint4* ring = reinterpret_cast<uint4*>(sm);
    uint4* xs = reinterpret_cast<uint4*>(sm + RING2_BYTES);
    float* red = reinterpret_cast<float*>(sm + arena - RED_BYTES);
    float* ssq_red = red + RED_FLOATS;         // [128]
    float* rs = ssq_red + 128;                 // [8]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    uint4* my = ring + (size_t)warp * PF * SLOTS * 32 + lane;
    const int K = j.K;
    const int n_chunks = K >> 5;
    const int n_my = (n_chunks > warp) ? (n_chunks - warp + WARPS - 1) / WARPS : 0;
    const int bid = blockIdx.x, nblk = gridDim.x;
    const int r0 = (int)((long long)bid * j.n_rows / nblk), r1 = (int)((long long)(bid + 1) * j.n_rows / nblk);
    constexpr int TR = MODE == 1 ? 8 : 16;     // output columns per tile
    const int n_tiles = (r1 - r0 + TR - 1) / TR;
    const int total = n_tiles * n_my;

    // prefetch cursor: flat item ordinal, tile ordinal, chunk ordinal, weight rows of that tile
    int f_pf = 0, pf_u = 0, pf_i = 0;
    const bf16 *pw_lo = j.W, *pw_hi = j.W;
    bool v_lo = false, v_hi = false;
    auto set_tile = [&](int uo) {
        const int base = r0 + uo * TR;
        size_t row_lo, row_hi;
        if (MODE == 1) { row_lo = (size_t)base + g; row_hi = (size_t)j.I + row_lo; v_lo = v_hi = base + g < r1; }
        else { row_lo = (size_t)base + g; row_hi = row_lo + 8; v_lo = base + g < r1; v_hi = base + g + 8 < r1; }
        pw_lo = j.W + (v_lo ? row_lo : 0) * K + 8 * t;
        pw_hi = j.W + (v_hi ? row_hi : 0) * K + 8 * t;
    };
    if (n_tiles > 0) set_tile(0);
    const bf16* xr = j.X + (size_t)(g < j.M ? g : 0) * j.ldx + 8 * t;
    auto fetch_w = [&]() {
        uint4* st = my + (size_t)(f_pf % PF) * SLOTS * 32;
        const size_t k0 = (size_t)(warp + pf_i * WARPS) << 5;
        cp_async16_if(st, pw_lo + k0, v_lo);
        cp_async16_if(st + 32, pw_hi + k0, v_hi);
    };
    auto fetch_x = [&](int f, int i) {
        uint4* st = my + (size_t)(f % PF) * SLOTS * 32;
        const size_t k0 = (size_t)(warp + i * WARPS) << 5;
        cp_async16_x(st + 64, xr + k0);
    };
    auto advance = [&]() {
        ++f_pf;
        if (++pf_i == n_my) {
            pf_i = 0;
            ++pf_u;
            if (pf_u < n_tiles) set_tile(pf_u);
        }
    };
    // the first weights: nothing computed in this step reaches them, so they are asked for before the barrier
    int pre = 0;
#pragma unroll
    for (int n = 0; n < PF - 1; ++n)
        if (f_pf < total) { fetch_w(); advance(); ++pre; }
    if (!grid_sync(bar)) return false;

    if (XSRC == 1) {
        // x whole into shared memory, every warp the chunks it will read itself; all copies in flight at once
        for (int i = 0; i < n_my; ++i) {
            const int c = warp + i * WARPS;
            cp_async16_if(xs + (size_t)c * 32 + lane, xr + ((size_t)c << 5), g < j.M);
        }
    }
    if (j.ssq != nullptr) {
        // the rows' scales from the producers' partial sums, added in block order: warp m takes token m
        if (warp < 8) {
            float s = 0.f;
            for (int b0 = 0; b0 < j.n_ssq; b0 += 32) {
                const int b = b0 + lane;
                float v = (b < j.n_ssq && warp < j.M) ? __ldcg(j.ssq + (size_t)b * 8 + warp) : 0.f;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {            // inclusive order-preserving sum: lanes add their left neighbours
                    const float u = __shfl_up_sync(0xffffffffu, v, o);
                    if (lane >= o) v += u;
                }
                s += __shfl_sync(0xffffffffu, v, 31);
            }
            if (lane == 0) rs[warp] = rsqrtf(s / (float)K + j.eps);
        }
    }
    // x of the chunks whose weights are already on their way; one group per item, as in the loop (the first group also
    // holds the early weight copies and the staged x)
#pragma unroll
    for (int n = 0; n < PF - 1; ++n) {
        if (XSRC == 0 && n < pre) fetch_x(n, n % (n_my > 0 ? n_my : 1));
        cp_commit();
    }

    float ss_acc = 0.f;                        // EPI 2: this thread's share of the sums of squares of the new stream
    int f = 0;
    for (int uo = 0; uo < n_tiles; ++uo) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i = 0; i < n_my; ++i, ++f) {
            if (f_pf < total) {
                fetch_w();
                if (XSRC == 0) fetch_x(f_pf, pf_i);
                advance();
            }
            cp_commit();
            cp_wait<PF - 1>();
            const uint4* st = my + (size_t)(f % PF) * SLOTS * 32;
            const uint4 wl = st[0], wh = st[32];
            const uint4 xv = XSRC ? xs[(size_t)(warp + i * WARPS) * 32 + lane] : st[64];
            mma16816(c, wl.x, wh.x, wl.y, wh.y, xv.x, xv.y);
            mma16816(c, wl.z, wh.z, wl.w, wh.w, xv.z, xv.w);
        }
        // the warps' partial sums, added in warp order
        red[(warp * 16 + g) * 9 + 2 * t] = c[0];
        red[(warp * 16 + g) * 9 + 2 * t + 1] = c[1];
        red[(warp * 16 + g + 8) * 9 + 2 * t] = c[2];
        red[(warp * 16 + g + 8) * 9 + 2 * t + 1] = c[3];
        __syncthreads();
        const int base = r0 + uo * TR;
        if (MODE == 1) {
            if (tid < 64) {
                const int r = tid >> 3, tok = tid & 7;
                if (tok < j.M && base + r < r1) {
                    float gate = 0.f, up = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) { gate += red[(w * 16 + r) * 9 + tok]; up += red[(w * 16 + r + 8) * 9 + tok]; }
                    if (j.ssq != nullptr) { gate *= rs[tok]; up *= rs[tok]; }
                    const float y = gate / (1.f + expf(-gate)) * up;
                    reinterpret_cast<bf16*>(j.out)[(size_t)tok * j.ldo + base + r] = __float2bfloat16_rn(y);
                }
            }
        } else {
            if (tid < 128) {
                const int r = tid >> 3, tok = tid & 7;
                if (tok < j.M && base + r < r1) {
                    float acc = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; ++w) acc += red[(w * 16 + r) * 9 + tok];
                    if (j.ssq != nullptr) acc *= rs[tok];
                    const size_t col = (size_t)base + r;
                    if (j.bias) acc += __bfloat162float(j.bias[col]);
                    const size_t o = (size_t)tok * j.ldo + col;
                    if (EPI == 0) reinterpret_cast<bf16*>(j.out)[o] = __float2bfloat16_rn(acc);
                    else if (EPI == 1) reinterpret_cast<float*>(j.out)[o] = acc;
                    else {
                        float* rp = reinterpret_cast<float*>(j.out) + o;
                        const float v = __ldcg(rp) + acc;
                        *rp = v;
                        j.xn[o] = __float2bfloat16_rn(v * ld_w(j.next_w, (int)col, j.next_w_f32));
                        ss_acc += v * v;
                    }
                }
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
    if (EPI == 2) {
        // per token: the 16 threads that hold its columns (tid = 8 r + tok), added in order of r
        if (tid < 128) ssq_red[tid] = ss_acc;
        __syncthreads();
        if (tid < 8) {
            float s = 0.f;
#pragma unroll
            for (int r = 0; r < 16; ++r) s += ssq_red[8 * r + tid];
            j.ssq_out[(size_t)bid * 8 + tid] = s;
        }
    }
    return true;
}

// res[m, :] = float(E[ids[m], :]): the float32 residual stream starts here, with what the first product wants of it
// (xn and the partial sums of squares, as after an EPI 2 product); every block takes an equal share of the columns.
__device__ __forceinline__ void embed_phase(const DsStep& p, const void* next_w, int next_w_f32, unsigned char* sm) {
    float* ssq_red = reinterpret_cast<float*>(sm);          // [THREADS]
    const int bid = blockIdx.x, nblk = gridDim.x, tid = threadIdx.x;
    const int c0 = (int)((long long)bid * p.H / nblk), c1 = (int)((long long)(bid + 1) * p.H / nblk);
    const bf16* E = reinterpret_cast<const bf16*>(p.embed);
    bf16* xn = reinterpret_cast<bf16*>(p.xn);
    const int tok = tid & 7, lanes = THREADS >> 3;          // thread = (column lane, token)
    float ss = 0.f;
    if (tok < p.M) {
        int id = p.ids[tok];
        id = id < 0 ? 0 : (id >= p.V ? p.V - 1 : id);
        for (int c = c0 + (tid >> 3); c < c1; c += lanes) {
            const float v = __bfloat162float(E[(size_t)id * p.H + c]);
            p.res[(size_t)tok * p.H + c] = v;
            xn[(size_t)tok * p.H + c] = __float2bfloat16_rn(v * ld_w(next_w, c, next_w_f32));
            ss += v * v;
        }
    }
    ssq_red[tid] = ss;
    __syncthreads();
    if (tid < 8) {
        float s = 0.f;
        for (int l = 0; l < lanes; ++l) s += ssq_red[8 * l + tid];
        p.ssq[(size_t)bid * 8 + tid] = s;
    }
    __syncthreads();
}

}  // namespace ds

namespace ds {

// ---------------------------------------------------------------------------------------
// attention of the step: one new token per request over its paged cache
// ---------------------------------------------------------------------------------------
// A unit is (request, kv head, kv split); all query heads of the kv head share every key and value read.  Keys ride
// the M dimension of mma.sync (16 per warp unit, straight from global memory into A-operand registers with the k
// index permuted as for the products above), the heads ride N (8 columns); values go through a per-warp cp.async ring
// and ldmatrix.trans.  The request's old keys (positions below the new token's) are cut into `ns` splits by tiles of
// KT keys anchored at position 0; the last split also takes the new key and value, which it has just normed, rotated
// and written to the cache, from a tile in shared memory.
constexpr int VRING_BYTES = WARPS * ST * WT * LDS * 2;
constexpr int QS_BYTES = 8 * LDS * 2;
constexpr int NEW_BYTES = WT * LDS * 2;
constexpr int HV_BYTES = WARPS * D * 4;
constexpr int ATT_BYTES = VRING_BYTES + QS_BYTES + 2 * NEW_BYTES + HV_BYTES;
static_assert(D % 32 == 0, "head sizes in steps of 32");
static_assert(WARPS * 8 * D * 4 + 2 * WARPS * 8 * 4 <= VRING_BYTES, "the merge buffers alias the V ring");

// One warp: a head vector of the qkv row -> (RMSNorm with weight) -> (rotation) -> bfloat16 into shared memory and,
// if dst_g is given, into global memory (the cache).  hv: D floats of scratch for this warp.
__device__ __forceinline__ void prep_head(const bf16* src, const void* nw, int nw_f32, float eps, const float* cs, int rot,
                                          float* hv, bf16* dst_s, bf16* dst_g) {
    constexpr int E = D / 32;
    const int lane = threadIdx.x & 31;
    float v[E];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(src) + lane + 32 * e);
        v[e] = __bfloat162float(__ushort_as_bfloat16(raw));
        ss += v[e] * v[e];
    }
    if (nw != nullptr) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) v[e] = v[e] * inv * ld_w(nw, lane + 32 * e, nw_f32);
    }
    if (cs != nullptr) {
#pragma unroll
        for (int e = 0; e < E; ++e) hv[lane + 32 * e] = v[e];
        __syncwarp();
        const int half = rot >> 1;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const int i = lane + 32 * e;
            float o;
            if (i < half) o = hv[i] * cs[i] - hv[i + half] * cs[half + i];
            else if (i < rot) o = hv[i - half] * cs[i] + hv[i] * cs[i - half];
            else o = hv[i];
            v[e] = o;
        }
        __syncwarp();
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const bf16 b = __float2bfloat16_rn(v[e]);
        dst_s[lane + 32 * e] = b;
        if (dst_g != nullptr) dst_g[lane + 32 * e] = b;
    }
}

__device__ __forceinline__ void attn_unit(const DsStep& p, const DsLayer& L, unsigned char* sm, int m, int kvh, int split, int ns) {
    constexpr int KP = D / 32, MT = D / 16, CH = D / 8, C = 8;
    __shared__ int sh_last;
    bf16* vring = reinterpret_cast<bf16*>(sm);
    bf16* qs = reinterpret_cast<bf16*>(sm + VRING_BYTES);
    bf16* kn = qs + 8 * LDS;
    bf16* vn = kn + WT * LDS;
    float* hv = reinterpret_cast<float*>(sm + VRING_BYTES + QS_BYTES + 2 * NEW_BYTES);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int G = p.n_q / p.n_kv;
    const int qkv_ld = (p.n_q + 2 * p.n_kv) * D;
    const bf16* qkv = reinterpret_cast<const bf16*>(p.qkv) + (size_t)m * qkv_ld;
    const bf16* kc = reinterpret_cast<const bf16*>(L.k_cache);
    const bf16* vc = reinterpret_cast<const bf16*>(L.v_cache);
    const int* bt = p.block_table + (size_t)m * p.bt_stride;
    const int p_max = p.kv_len[m] - 1;             // the new token's position; older keys are 0 .. p_max - 1
    const int n_old = p_max > 0 ? p_max : 0;
    const bool last = split == ns - 1;
    const float* cs = nullptr;
    if (p.rope != nullptr) {
        int pos = p.positions[m];
        pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
        cs = p.rope + (size_t)pos * p.rot;
    }
    auto page_index = [&](int key) { return p.page_shift >= 0 ? (key >> p.page_shift) : (key / p.page_size); };
    auto page_slot = [&](int key) { return p.page_shift >= 0 ? (key & (p.page_size - 1)) : (key % p.page_size); };

    __syncthreads();                               // the unit before this one is done with the shared memory
    if (last) {
        for (int i = tid; i < 2 * WT * LDS / 8; i += THREADS) reinterpret_cast<uint4*>(kn)[i] = make_uint4(0u, 0u, 0u, 0u);
        __syncthreads();
    }
    for (int hl = warp; hl < G; hl += WARPS)
        prep_head(qkv + ((size_t)kvh * G + hl) * D, L.q_norm, L.qk_norm_f32, L.eps_qk, cs, p.rot, hv + warp * D, qs + hl * LDS, nullptr);
    if (last && warp < 2) {
        const int slot = p.out_loc[m];
        const int page = slot / p.page_size, off = slot - page * p.page_size;
        const size_t at = (((size_t)page * p.n_kv + kvh) * p.page_size + off) * D;
        if (warp == 0) {
            prep_head(qkv + ((size_t)p.n_q + kvh) * D, L.k_norm, L.qk_norm_f32, L.eps_qk, cs, p.rot, hv, kn,
                      reinterpret_cast<bf16*>(L.k_cache) + at);
        } else {
            prep_head(qkv + ((size_t)p.n_q + p.n_kv + kvh) * D, nullptr, 0, 0.f, nullptr, 0, hv + D, vn,
                      reinterpret_cast<bf16*>(L.v_cache) + at);
        }
    }
    __syncthreads();

    // the old keys of this split, in warp units of WT keys
    const int n_t = (n_old + KT - 1) / KT;
    const int per = (n_t + ns - 1) / ns;
    const int kt_begin = min(split * per, n_t), kt_end = min((split + 1) * per, n_t);
    const int u_begin = kt_begin * (KT / WT);
    const int u_end = min(kt_end * (KT / WT), (n_old + WT - 1) / WT);
    const int n_my = (u_end - u_begin > warp) ? (u_end - u_begin - warp + WARPS - 1) / WARPS : 0;
    bf16* my_ring = vring + (size_t)warp * ST * WT * LDS;
    const int v_key = lane >> 1, v_half = lane & 1;

    auto unit_page = [&](int i) -> int {           // page of key (unit i, row lane & 15), or -1 past the last old key
        const int key = (u_begin + warp + i * WARPS) * WT + (lane & 15);
        return (i < n_my && key < n_old) ? bt[page_index(key)] : -1;
    };
    auto load_v = [&](int i, int pg_row) {
        bf16* Vs = my_ring + (size_t)(i % ST) * WT * LDS;
        const int key = (u_begin + warp + i * WARPS) * WT + v_key;
        const bool valid = pg_row >= 0;
        size_t off = 0;
        if (valid) off = (((size_t)pg_row * p.n_kv + kvh) * p.page_size + page_slot(key)) * D;
#pragma unroll
        for (int jj = 0; jj < CH / 2; ++jj) {
            const int c = 2 * jj + v_half;
            cp_async16_if(Vs + v_key * LDS + c * 8, vc + off + c * 8, valid);
        }
    };
    auto prefetch_k = [&](int i, int pg_row) {
        if (pg_row < 0) return;
        const int key = (u_begin + warp + i * WARPS) * WT + v_key;
        const size_t off = (((size_t)pg_row * p.n_kv + kvh) * p.page_size + page_slot(key)) * D;
#pragma unroll
        for (int ln = 0; ln < (D + 127) / 128; ++ln) {
            const int e = (2 * ln + v_half) * 64;
            if (e < D) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(kc + off + e));
        }
    };
    uint4 k_lo[KP], k_hi[KP];
    auto load_k = [&](int i, int pg_lo, int pg_hi) {
        const int key0 = (u_begin + warp + i * WARPS) * WT;
        const bf16* lo = kc + (((size_t)max(pg_lo, 0) * p.n_kv + kvh) * p.page_size + page_slot(key0 + g)) * D + 8 * t;
        const bf16* hi = kc + (((size_t)max(pg_hi, 0) * p.n_kv + kvh) * p.page_size + page_slot(key0 + 8 + g)) * D + 8 * t;
#pragma unroll
        for (int jj = 0; jj < KP; ++jj) {
            k_lo[jj] = pg_lo >= 0 ? ldg_stream(lo + 32 * jj) : make_uint4(0u, 0u, 0u, 0u);
            k_hi[jj] = pg_hi >= 0 ? ldg_stream(hi + 32 * jj) : make_uint4(0u, 0u, 0u, 0u);
        }
    };

    // Q as B operand: lane (g, t) holds Q[head g][32 j + 8 t .. + 7]
    uint4 qf[KP];
#pragma unroll
    for (int jj = 0; jj < KP; ++jj)
        qf[jj] = g < G ? *reinterpret_cast<const uint4*>(qs + g * LDS + 32 * jj + 8 * t) : make_uint4(0u, 0u, 0u, 0u);

    float o[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) { o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f; }
    float m_c[2] = {-INFINITY, -INFINITY}, l_c[2] = {0.f, 0.f};
    const float sc = p.scale * 1.4426950408889634f;
    float s[4], s2[4];

    auto scores = [&]() {                          // S^T = K Q^T from registers
        s[0] = s[1] = s[2] = s[3] = 0.f;
        s2[0] = s2[1] = s2[2] = s2[3] = 0.f;
#pragma unroll
        for (int jj = 0; jj < KP; ++jj) {
            mma16816(s, k_lo[jj].x, k_hi[jj].x, k_lo[jj].y, k_hi[jj].y, qf[jj].x, qf[jj].y);
            mma16816(s2, k_lo[jj].z, k_hi[jj].z, k_lo[jj].w, k_hi[jj].w, qf[jj].z, qf[jj].w);
        }
    };
    // online softmax of 16 keys starting at key0 (keys above `bound` do not count) and O^T += V^T P^T
    auto softmax_pv = [&](int key0, int bound, const bf16* Vs) {
        const bool need_mask = key0 + WT - 1 > bound;
        float v[4], alpha[2];
        bool rescale = false;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            v[e] = (s[e] + s2[e]) * sc;
            if (need_mask && key0 + g + ((e & 2) ? 8 : 0) > bound) v[e] = -INFINITY;
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float mx = fmaxf(v[e], v[e + 2]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float mn = fmaxf(m_c[e], mx);
            const float mu = (mn == -INFINITY) ? 0.f : mn;
            alpha[e] = fast_exp2(m_c[e] - mu);
            m_c[e] = mn;
            v[e] = fast_exp2(v[e] - mu);
            v[e + 2] = fast_exp2(v[e + 2] - mu);
            l_c[e] = l_c[e] * alpha[e] + v[e] + v[e + 2];
            rescale = rescale || alpha[e] != 1.f;
        }
        const unsigned pb0 = movmatrix_trans(pack_bf16(v[0], v[1]));
        const unsigned pb1 = movmatrix_trans(pack_bf16(v[2], v[3]));
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1];
                o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1];
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            unsigned a[4];
            ldmatrix_x4_trans(a, Vs + ((lane & 7) + ((lane >> 4) & 1) * 8) * LDS + mt * 16 + ((lane >> 3) & 1) * 8);
            mma16816(o[mt], a[0], a[1], a[2], a[3], pb0, pb1);
        }
    };

    // prologue: first keys towards L2, V of the first ST-1 units, K of unit 0
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        const int pg = unit_page(i);
        const int pg_row = __shfl_sync(0xffffffffu, pg, v_key);
        if (i < n_my) load_v(i, pg_row);
        cp_commit();
        if (i == 0 && n_my > 0) load_k(0, __shfl_sync(0xffffffffu, pg, g), __shfl_sync(0xffffffffu, pg, g + 8));
    }
    {
        const int pg = unit_page(1);
        prefetch_k(1, __shfl_sync(0xffffffffu, pg, v_key));
    }
    int pg_pf_next = unit_page(2);
    int pg_v_next = unit_page(ST - 1);
    int pg_k_next = unit_page(1);
    for (int i = 0; i < n_my; ++i) {
        scores();
        {
            const int pk = pg_k_next;
            if (i + 1 < n_my) load_k(i + 1, __shfl_sync(0xffffffffu, pk, g), __shfl_sync(0xffffffffu, pk, g + 8));
            const int pv = __shfl_sync(0xffffffffu, pg_v_next, v_key);
            if (i + ST - 1 < n_my) load_v(i + ST - 1, pv);
            cp_commit();
            const int pf = __shfl_sync(0xffffffffu, pg_pf_next, v_key);
            if (i + 2 < n_my) prefetch_k(i + 2, pf);
            pg_pf_next = unit_page(i + 3);
            pg_k_next = unit_page(i + 2);
            pg_v_next = unit_page(i + ST);
        }
        cp_wait<ST - 1>();
        __syncwarp();
        softmax_pv((u_begin + warp + i * WARPS) * WT, n_old - 1, my_ring + (size_t)(i % ST) * WT * LDS);
        __syncwarp();
    }
    cp_wait<0>();
    if (last && warp == 0) {                        // the new key and value, from shared memory
#pragma unroll
        for (int jj = 0; jj < KP; ++jj) {
            k_lo[jj] = *reinterpret_cast<const uint4*>(kn + g * LDS + 32 * jj + 8 * t);
            k_hi[jj] = *reinterpret_cast<const uint4*>(kn + (g + 8) * LDS + 32 * jj + 8 * t);
        }
        scores();
        softmax_pv(p_max, p_max, vn);
    }

    // column sums over the 8 lanes that share a column pair
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        float l = l_c[e];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        l_c[e] = l;
    }
    // merge the warps through shared memory, in warp order
    float* Om = reinterpret_cast<float*>(vring);          // [WARPS][C][D]
    float* Mm = Om + WARPS * C * D;                       // [WARPS][C]
    float* Lm = Mm + WARPS * C;
    __syncthreads();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = 2 * t + (e & 1);
            const int dim = mt * 16 + g + ((e & 2) ? 8 : 0);
            Om[((size_t)warp * C + c) * D + dim] = o[mt][e];
        }
    if (g == 0) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            Mm[warp * C + 2 * t + e] = m_c[e];
            Lm[warp * C + 2 * t + e] = l_c[e];
        }
    }
    __syncthreads();
    bf16* og = reinterpret_cast<bf16*>(p.attn);
    for (int idx = tid; idx < G * D; idx += THREADS) {
        const int c = idx / D, col = idx - c * D;
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) Mx = fmaxf(Mx, Mm[w * C + c]);
        const float Mu = (Mx == -INFINITY) ? 0.f : Mx;
        float acc = 0.f, Ls = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float f = fast_exp2(Mm[w * C + c] - Mu);
            acc += f * Om[((size_t)w * C + c) * D + col];
            Ls += f * Lm[w * C + c];
        }
        const int head = kvh * G + c;
        if (ns == 1) {
            og[((size_t)m * p.n_q + head) * D + col] = __float2bfloat16_rn(Ls > 0.f ? acc / Ls : 0.f);
        } else {
            const size_t prow = ((size_t)split * p.M + m) * p.n_q + head;
            p.part_o[prow * D + col] = acc;
            if (col == 0) { p.part_ml[prow * 2] = Mx; p.part_ml[prow * 2 + 1] = Ls; }
        }
    }
    if (ns == 1) return;
    // the unit that finishes this (request, kv head) last merges the splits, in split order
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* tk = p.tickets + m * p.n_kv + kvh;
        const int mine = atomicAdd(tk, 1);
        sh_last = (mine == ns - 1);
        if (sh_last) *tk = 0;
    }
    __syncthreads();
    if (!sh_last) return;
    __threadfence();
    for (int idx = tid; idx < G * D; idx += THREADS) {
        const int c = idx / D, col = idx - c * D;
        const int head = kvh * G + c;
        float Mx = -INFINITY;
        for (int sp = 0; sp < ns; ++sp) Mx = fmaxf(Mx, __ldcg(p.part_ml + (((size_t)sp * p.M + m) * p.n_q + head) * 2));
        const float Mu = (Mx == -INFINITY) ? 0.f : Mx;
        float acc = 0.f, Ls = 0.f;
        for (int sp = 0; sp < ns; ++sp) {
            const size_t prow = ((size_t)sp * p.M + m) * p.n_q + head;
            const float f = exp2f(__ldcg(p.part_ml + prow * 2) - Mu);
            Ls += f * __ldcg(p.part_ml + prow * 2 + 1);
            acc += f * __ldcg(p.part_o + prow * D + col);
        }
        og[((size_t)m * p.n_q + head) * D + col] = __float2bfloat16_rn(Ls > 0.f ? acc / Ls : 0.f);
    }
}

__device__ __forceinline__ bool attn_phase(const DsStep& p, const DsLayer& L, unsigned char* sm, GridBar& bar) {
    if (!grid_sync(bar)) return false;
    // units in the order (request, split, kv head); a request has n_kv * ns of them
    int first[MAX_M + 1];
    first[0] = 0;
#pragma unroll
    for (int m = 0; m < MAX_M; ++m) {
        int ns = 0;
        if (m < p.M) ns = p.nsplit ? min(max(p.nsplit[m], 1), p.max_split) : 1;
        first[m + 1] = first[m] + ns * p.n_kv;
    }
    for (int u = blockIdx.x; u < first[MAX_M]; u += gridDim.x) {
        int m = 0;
#pragma unroll
        for (int q = 1; q < MAX_M; ++q) m += (u >= first[q]) ? 1 : 0;
        const int r = u - first[m];
        const int ns = (first[m + 1] - first[m]) / p.n_kv;
        attn_unit(p, L, sm, m, r % p.n_kv, r / p.n_kv, ns);
    }
    return true;
}

}  // namespace ds

// ---------------------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------------------
#ifndef MSGL_DS_PROFILE
#define MSGL_DS_PROFILE 0
#endif
// With MSGL_DS_PROFILE=1 blocks 0 and gridDim.x - 1 add up, per kind of phase, the time from entering the phase to
// passing its barrier and from there to leaving it (ns, in words 8.. of the status buffer: [block 0 | last][6 kinds][2]).
#if MSGL_DS_PROFILE
#define DS_PROF_BEGIN(kind) const int prof_kind_ = (kind); const unsigned long long prof_t0_ = ds::global_ns()
#define DS_PROF_END() do { if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) { \
        const unsigned long long t2 = ds::global_ns(); const unsigned long long mid = bar.t_pass; \
        int* w = p.status + 5 + ((blockIdx.x == 0 ? 0 : 6) + prof_kind_) * 2; \
        w[0] += (int)(mid - prof_t0_); w[1] += (int)(t2 - mid); } } while (0)
#else
#define DS_PROF_BEGIN(kind)
#define DS_PROF_END()
#endif

__global__ void __launch_bounds__(ds::THREADS, 1) decode_step_kernel(const __grid_constant__ DsStep p, int arena) {
    using namespace ds;
    extern __shared__ __align__(16) unsigned char ds_smem[];
    GridBar bar{p.bar, p.status, 0u, gridDim.x, 0ull};
    const int nblk = gridDim.x;
    const int qkv_n = (p.n_q + 2 * p.n_kv) * D;
    {
        const bool none = p.n_layers == 0;
        embed_phase(p, none ? p.final_norm : p.layers[0].norm_in, none ? p.final_f32 : p.layers[0].norm_f32, ds_smem);
    }
    GemmJob j;
    j.M = p.M;
    j.n_ssq = nblk;
    j.xn = reinterpret_cast<bf16*>(p.xn);
    j.ssq_out = p.ssq;
    for (int l = 0; l < p.n_layers; ++l) {
        const DsLayer& L = p.layers[l];
        // A: qkv = norm_in(res) . Wqkv^T (+ b)
        j.W = reinterpret_cast<const bf16*>(L.w_qkv); j.n_rows = qkv_n; j.K = p.H; j.I = 0;
        j.X = reinterpret_cast<const bf16*>(p.xn); j.ldx = p.H; j.ssq = p.ssq; j.eps = L.eps_in;
        j.bias = reinterpret_cast<const bf16*>(L.b_qkv); j.out = p.qkv; j.ldo = qkv_n;
        { DS_PROF_BEGIN(0); if (!gemm_phase<0, 1, 0>(j, ds_smem, arena, bar)) return; DS_PROF_END(); }
        // B: attention
        { DS_PROF_BEGIN(1); if (!attn_phase(p, L, ds_smem, bar)) return; DS_PROF_END(); }
        // C: res += attn . Wo^T; xn = bf16(res * w_post)
        j.W = reinterpret_cast<const bf16*>(L.w_o); j.n_rows = p.H; j.K = p.n_q * D;
        j.X = reinterpret_cast<const bf16*>(p.attn); j.ldx = (long long)p.n_q * D; j.ssq = nullptr;
        j.bias = nullptr; j.out = p.res; j.ldo = p.H; j.next_w = L.norm_post; j.next_w_f32 = L.norm_f32;
        { DS_PROF_BEGIN(2); if (!gemm_phase<0, 1, 2>(j, ds_smem, arena, bar)) return; DS_PROF_END(); }
        // D: act = silu(g) * u, [g; u] = norm_post(res) . Wgu^T
        j.W = reinterpret_cast<const bf16*>(L.w_gu); j.n_rows = p.I; j.K = p.H; j.I = p.I;
        j.X = reinterpret_cast<const bf16*>(p.xn); j.ldx = p.H; j.ssq = p.ssq; j.eps = L.eps_post;
        j.bias = nullptr; j.out = p.act; j.ldo = p.I;
        { DS_PROF_BEGIN(3); if (!gemm_phase<1, 1, 0>(j, ds_smem, arena, bar)) return; DS_PROF_END(); }
        // E: res += act . Wdown^T; xn = bf16(res * weight of the norm that comes next)
        const bool last = l + 1 == p.n_layers;
        j.W = reinterpret_cast<const bf16*>(L.w_down); j.n_rows = p.H; j.K = p.I; j.I = 0;
        j.X = reinterpret_cast<const bf16*>(p.act); j.ldx = p.I; j.ssq = nullptr;
        j.bias = nullptr; j.out = p.res; j.ldo = p.H;
        j.next_w = last ? p.final_norm : p.layers[l + 1].norm_in;
        j.next_w_f32 = last ? p.final_f32 : p.layers[l + 1].norm_f32;
        { DS_PROF_BEGIN(4); if (!gemm_phase<0, 0, 2>(j, ds_smem, arena, bar)) return; DS_PROF_END(); }
    }
    // head: logits = norm_final(res) . Wlm^T, float32
    j.W = reinterpret_cast<const bf16*>(p.lm_head); j.n_rows = p.V; j.K = p.H; j.I = 0;
    j.X = reinterpret_cast<const bf16*>(p.xn); j.ldx = p.H; j.ssq = p.ssq; j.eps = p.eps_final;
    j.bias = nullptr; j.out = p.logits; j.ldo = p.V;
    { DS_PROF_BEGIN(5); gemm_phase<0, 1, 1>(j, ds_smem, arena, bar); DS_PROF_END(); }
}

// ---------------------------------------------------------------------------------------
// C entry points
// ---------------------------------------------------------------------------------------
MSGL_API int msgl_decode_step_head_dim() { return MSGL_HEAD_DIM; }
MSGL_API int msgl_decode_step_layer_bytes() { return (int)sizeof(DsLayer); }
MSGL_API int msgl_decode_step_struct_bytes() { return (int)sizeof(DsStep); }

// shared memory a block needs for these sizes, or -1 if the kernel does not take them
static int ds_arena_bytes(int M, int H, int n_q, int n_kv, int I, int V) {
    using namespace ds;
    if (M < 1 || M > MAX_M || n_kv < 1 || n_q < n_kv || n_q % n_kv || n_q / n_kv > 8) return -1;
    if (H <= 0 || (H & 31) || I <= 0 || (I & 31) || V <= 0) return -1;
    const int k_staged = H > n_q * MSGL_HEAD_DIM ? H : n_q * MSGL_HEAD_DIM;
    int need = RING2_BYTES + k_staged * 16 + RED_BYTES;           // products whose x is copied whole into shared memory
    if (RING3_BYTES + RED_BYTES > need) need = RING3_BYTES + RED_BYTES;
    if (ATT_BYTES > need) need = ATT_BYTES;
    need = (need + 127) & ~127;
    return need <= 227 * 1024 ? need : -1;
}

// How many blocks the kernel runs with on the current device for these sizes (what the kv splits are planned for);
// 0 if it does not take the sizes.  First call on a device: outside any stream capture.
MSGL_API int msgl_decode_step_blocks(int M, int H, int n_q, int n_kv, int I, int V) {
    const int arena = ds_arena_bytes(M, H, n_q, n_kv, I, V);
    if (arena < 0) return 0;
    static int granted[MSGL_MAX_DEVICES] = {};
    const int dev = msgl_device();
    if (arena > granted[dev]) {
        if (cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, arena) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        granted[dev] = arena;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, ds::THREADS, arena) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        return 0;
    }
    if (per_sm > 1) per_sm = 1;
    return per_sm * msgl_sm_count();
}

// One decode step.  `step` is a host copy of DsStep whose pointers are device pointers.  Returns MSGL_ERR_SIZE for
// sizes the kernel does not take (nothing is launched then).
MSGL_API int msgl_decode_step(const DsStep* step, cudaStream_t stream) {
    const DsStep& p = *step;
    if (p.M <= 0) return MSGL_OK;
    const int arena = ds_arena_bytes(p.M, p.H, p.n_q, p.n_kv, p.I, p.V);
    if (arena < 0 || p.n_layers < 0 || p.page_size < 1 || p.max_split < 1 || p.bt_stride < 1) return MSGL_ERR_SIZE;
    if (p.rope != nullptr && (p.rot < 2 || (p.rot & 1) || p.rot > MSGL_HEAD_DIM || p.max_pos < 1)) return MSGL_ERR_SIZE;
    if (p.bar == nullptr || p.status == nullptr || p.tickets == nullptr || p.xn == nullptr || p.ssq == nullptr) return MSGL_ERR_SIZE;
    const int blocks = msgl_decode_step_blocks(p.M, p.H, p.n_q, p.n_kv, p.I, p.V);
    if (blocks <= 0) return MSGL_ERR_SIZE;
    if (cudaMemsetAsync(p.bar, 0, sizeof(unsigned), stream) != cudaSuccess) return msgl_check_launch();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(ds::THREADS);
    cfg.dynamicSmemBytes = arena;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;       // every block resident at once: the barriers cannot starve
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, decode_step_kernel, p, arena);
    return msgl_check_launch();
}
