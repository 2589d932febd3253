// See attention_noalloc.h.  The kernels are the ones of attention.cu, compiled into this library
// as well; only the place the partial results go to differs.
#include "attention.cu"
#include "attention_noalloc.h"

// Scratch for the kv-split partials: [split][request][head][d] sums, then [split][request][head][2]
// (maximum, row sum).  Device memory owned by the library image on each GPU.
static __device__ __align__(256) float g_noalloc_scratch[MSGL_NOALLOC_SCRATCH_FLOATS];

#define MSGL_NOALLOC_MAX_DEVICES 64
static float* g_scratch_addr[MSGL_NOALLOC_MAX_DEVICES];   // device address of the array, per device; null = not looked up yet

MSGL_API unsigned long long msgl_attention_noalloc_capacity_floats(void) { return MSGL_NOALLOC_SCRATCH_FLOATS; }

MSGL_API int msgl_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                           const int* q_start, const int* kv_len, const int* block_table,
                                           const int* nsplit, int B, int n_q, int n_kv, int d, int page_size,
                                           int bt_stride, int window, int max_split, float scale, int dtype,
                                           cudaStream_t stream) {
    if (B <= 0) return MSGL_OK;
    if (n_q <= 0 || d <= 0 || max_split < 1 || nsplit == nullptr) return MSGL_ERR_SIZE;
    const unsigned long long rows = (unsigned long long)max_split * (unsigned long long)B * (unsigned long long)n_q;
    if (rows * (unsigned long long)(d + 2) > MSGL_NOALLOC_SCRATCH_FLOATS) return MSGL_ERR_SCRATCH;

    // In host code `g_noalloc_scratch` names a host-side stand-in of the device array, not memory a
    // kernel can use; the device address has to be asked for, once per device, with it current.
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MSGL_NOALLOC_MAX_DEVICES) return MSGL_ERR_LAUNCH;
    float* scratch = g_scratch_addr[dev];
    if (scratch == nullptr) {
        if (cudaGetSymbolAddress((void**)&scratch, g_noalloc_scratch) != cudaSuccess || scratch == nullptr)
            return MSGL_ERR_LAUNCH;
        g_scratch_addr[dev] = scratch;
    }
    float* part_o = scratch;
    float* part_ml = scratch + rows * (unsigned long long)d;

    // tensor-core decode kernel where this library was built for the head size, else the float32 one
    const int variant = (dtype == MSGL_BF16 && d == MSGL_HEAD_DIM) ? 2 : 0;
    int rc = msgl_attention(q, out, k_cache, v_cache, q_start, kv_len, block_table, nsplit, part_o, part_ml, B, B, n_q,
                            n_kv, d, page_size, bt_stride, window, max_split, scale, 1, 1, /*uniform_decode=*/1, variant,
                            /*grid_x=*/B, dtype, /*order=*/nullptr, /*even=*/nullptr, 0, stream);
    if (rc != MSGL_OK) return rc;
    return msgl_attention_combine(part_o, part_ml, /*token_req=*/nullptr, nsplit, out, B, n_q, d, max_split, dtype, stream);
}
