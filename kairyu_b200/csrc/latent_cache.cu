// The cache write of latent attention: a token's compressed key/value row
//
//     c[t] = z[t] * rsqrt(mean(z[t]^2) + eps) * w        z = columns [offset, offset + R) of a packed product
//
// is normed in 32-bit and stored once, in the cache's dtype, at the token's place in its request's
// pages (one "head" of R columns).  Keys and values of every head are products of this row, so it
// is all such a layer keeps.  Positions below write_from[row] lie in pages the request only
// reads and are skipped.  One block per token.
#include "common.cuh"

template <typename TZ, typename TW, typename TC>
__global__ void __launch_bounds__(128)
latent_norm_write_kernel(const TZ* __restrict__ z, int z_stride, int offset, int R, const TW* __restrict__ w, float eps,
                         const int* __restrict__ positions, const int* __restrict__ row_ids,
                         const int* __restrict__ block_table, int max_pages, const int* __restrict__ write_from,
                         TC* __restrict__ cache, int page_size, int num_pages, int num_rows, int* flag) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int row = row_ids[t];
    pdl_wait();
    const TZ* zr = z + (size_t)t * z_stride + offset;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_float(zr[i]);
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    if (row < 0 || row >= num_rows) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_ROW);
        return;
    }
    if (write_from && pos < write_from[row]) return;
    const int page_index = pos / page_size;
    const int page = page_index < max_pages ? block_table[(size_t)row * max_pages + page_index] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && flag) atomicOr(flag, KB_FLAG_BAD_PAGE);
        return;
    }
    const float inv = rsqrtf(total / (float)R + eps);
    TC* dst = cache + ((size_t)page * page_size + (pos % page_size)) * R;
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_float<TC>(to_float(zr[i]) * inv * to_float(w[i]));
}

KB_EXPORT int kb_latent_norm_write(const void* z, int z_stride, int offset, int R, int is_bf16, const void* w, int w_is_bf16,
                                   float eps, const int* positions, const int* row_ids, const int* block_table, int max_pages,
                                   const int* write_from, void* cache, int page_size, int num_pages, int num_rows, int T,
                                   int* flag, cudaStream_t stream) {
    if (T == 0) return 0;
    if (!z || !w || !positions || !row_ids || !block_table || !cache) return KB_ERR_NULL;
    if (R < 1 || page_size < 1) return KB_ERR_BAD_ARG;
#define LAUNCH(TZ, TW)                                                                                                   \
    kb_launch(latent_norm_write_kernel<TZ, TW, TZ>, dim3(T), dim3(128), 0, stream, (const TZ*)z, z_stride, offset, R,     \
              (const TW*)w, eps, positions, row_ids, block_table, max_pages, write_from, (TZ*)cache, page_size, num_pages, \
              num_rows, flag)
    if (is_bf16) {
        if (w_is_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16); else LAUNCH(__nv_bfloat16, float);
    } else {
        if (w_is_bf16) LAUNCH(float, __nv_bfloat16); else LAUNCH(float, float);
    }
#undef LAUNCH
    return kb_launch_result();
}
