// bfloat16 differential attention on tensor cores (mma.sync m16n8k16, 32-bit scores, softmax,
// accumulation, combination and head norm): one flash-attention kernel that keeps TWO online
// softmaxes a query row, one per score map, over the same value tile.
//
//   q      [tokens, Hq * 2 * D]             a head's two maps side by side
//   keys   [pages, page_size, Hkv, 2 * D]   the same per key/value head;  values [pages, page_size, Hkv, DV]
//   s_m = cap * tanh(q_m . k_m * scale / cap) (cap <= 0: none), softmax over the keys a query sees
//   (itself and the window - 1 before it), a_m = P_m V, o = a_1 - lambda a_2,
//   head_norm: o <- o * rsqrt(mean(o^2) + eps) * out_scale.
//
// A block works on a tile of up to 64 rows and streams the keys 64 at a time through two
// cp.async buffers (a key row brings both maps' keys; the value tile is read once for both maps).
// What a row is depends on the launch:
//   portions (grid Hq x tiles): row r is query q0 + r of one request's portion, for query head h;
//   single tokens (grid Hkv x rows): row r is query head kvh * (Hq / Hkv) + r of the request's one
//       token, so the heads that share a key/value head share one pass over its keys.  Up to 16 heads a
//       key/value head take the kernel further down, whose warps share a tile by keys instead of by rows.
// Warp w owns rows 16 w .. 16 w + 15.  D and DV are multiples of 16 up to 128; the kernel is
// instantiated for padded sizes in {32, 64, 128} and zero-fills the columns above.
// Key tiles start at absolute multiples of 64, so a single token's result depends on its own
// position only; a portion's depends on where its tiles start, within rounding.
#include "attention_mma.cuh"

#define DAM_ROWS 64
#define DAM_KEYS 64
#define DAM_THREADS 128

template <int DKP, int DVP>
struct DiffTile {
    static constexpr int KSTRIDE = 2 * DKP + 8;  // the 16 extra bytes keep ldmatrix free of bank conflicts
    static constexpr int VSTRIDE = DVP + 8;
    static constexpr size_t BYTES = (size_t)(DAM_ROWS * KSTRIDE + 2 * DAM_KEYS * KSTRIDE + 2 * DAM_KEYS * VSTRIDE) * sizeof(__nv_bfloat16);
};

// tanh to about 1e-7 absolute from the fast exponential: 1 - 2 / (e^{2x} + 1)
__device__ __forceinline__ float tanh_from_exp(float x) { return 1.0f - 2.0f / (__expf(2.0f * x) + 1.0f); }

// A 64-key tile of keys and values into shared memory.  Two threads a key row: the page is looked up once a
// row, and the row's 16-byte chunks (both maps' keys, then the values) go alternately to the two threads.
// Zero-filled: keys outside [key_lo, key_end), keys on an absent page, padding columns.
template <int DKP, int DVP>
__device__ __forceinline__ void load_diff_tiles(__nv_bfloat16* tile_k, __nv_bfloat16* tile_v, const __nv_bfloat16* __restrict__ k_cache,
                                                const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ table, int max_pages,
                                                int num_pages, int page_size, int page_shift, int Hkv, int kvh, int D, int DV, int key0,
                                                int key_lo, int key_end) {
    constexpr int KCH = 2 * DKP / 8, VCH = DVP / 8, MCH = DKP / 8;
    constexpr int KS = DiffTile<DKP, DVP>::KSTRIDE, VS = DiffTile<DKP, DVP>::VSTRIDE;
    static_assert(DAM_THREADS == 2 * DAM_KEYS && KCH % 2 == 0 && VCH % 2 == 0, "two threads a key row");
    const int r = threadIdx.x >> 1, half = threadIdx.x & 1;
    const int key = key0 + r;
    bool valid = key >= key_lo && key < key_end;
    size_t place = 0;
    if (valid) {
        const int page_index = page_shift >= 0 ? (key >> page_shift) : (key / page_size);
        const int page = page_index < max_pages ? table[page_index] : -1;
        if (page < 0 || page >= num_pages)
            valid = false;
        else
            place = ((size_t)page * page_size + (key - page_index * page_size)) * Hkv + kvh;
    }
    const __nv_bfloat16* k_row = k_cache + place * 2 * D;
    const __nv_bfloat16* v_row = v_cache + place * DV;
    __nv_bfloat16* k_dst = tile_k + r * KS;
    __nv_bfloat16* v_dst = tile_v + r * VS;
#pragma unroll
    for (int i = 0; i < KCH / 2; ++i) {
        const int cc = 2 * i + half;
        const int map = cc / MCH, col = (cc % MCH) * 8;
        const bool ok = valid && col < D;
        cp_async16(k_dst + map * DKP + col, ok ? k_row + map * D + col : k_cache, ok);
    }
#pragma unroll
    for (int i = 0; i < VCH / 2; ++i) {
        const int col = (2 * i + half) * 8;
        const bool ok = valid && col < DV;
        cp_async16(v_dst + col, ok ? v_row + col : v_cache, ok);
    }
}

template <int DKP, int DVP>
__global__ void __launch_bounds__(DAM_THREADS)
diff_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
                          const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                          const int* __restrict__ qo_indptr, const int* __restrict__ seq_lens, const int* __restrict__ block_table,
                          int max_pages, const int* __restrict__ list_rows, const int* __restrict__ list_second, int single, int Hq,
                          int Hkv, int D, int DV, int page_size, int num_pages, float scale, float cap, int window, float lambda,
                          int head_norm, float eps, float out_scale, int* flag) {
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int KS = DiffTile<DKP, DVP>::KSTRIDE, VS = DiffTile<DKP, DVP>::VSTRIDE;
    constexpr int KSTEPS = DKP / 16, DTILES = DVP / 8, MCH = DKP / 8;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sK = sQ + DAM_ROWS * KS;          // two buffers
    __nv_bfloat16* sV = sK + 2 * DAM_KEYS * KS;      // two buffers

    const int group = Hq / Hkv;
    int row, kvh, first_pos, rows_here, last_pos;
    const __nv_bfloat16* q_row0;   // the tile's row 0
    __nv_bfloat16* out_row0;
    size_t q_step, out_step;       // from one tile row to the next
    if (single) {
        kvh = blockIdx.x;
        row = list_rows[blockIdx.y];
        const int token = list_second[blockIdx.y];
        first_pos = last_pos = seq_lens[row] - 1;
        rows_here = group;
        q_row0 = q + (size_t)token * q_stride + (size_t)kvh * group * 2 * D;
        out_row0 = out + (size_t)token * out_stride + (size_t)kvh * group * DV;
        q_step = 2 * D;
        out_step = DV;
    } else {
        // later tiles of a portion see more keys: hand them out first
        const int tile = gridDim.y - 1 - blockIdx.y;
        const int h = blockIdx.x;
        kvh = h / group;
        row = list_rows[tile];
        const int q0 = list_second[tile];
        const int tok0 = qo_indptr[row];
        const int portion = qo_indptr[row + 1] - tok0;
        rows_here = min(DAM_ROWS, portion - q0);
        first_pos = seq_lens[row] - portion + q0;
        last_pos = first_pos + rows_here - 1;
        q_row0 = q + (size_t)(tok0 + q0) * q_stride + (size_t)h * 2 * D;
        out_row0 = out + (size_t)(tok0 + q0) * out_stride + (size_t)h * DV;
        q_step = q_stride;
        out_step = out_stride;
    }
    const int pos_step = single ? 0 : 1;  // rows of a single token share its position
    const int* table = block_table + (size_t)row * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int key_end = last_pos + 1;
    const int key_lo = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
    const int first_kt = key_lo / DAM_KEYS, last_kt = (key_end - 1) / DAM_KEYS;
    const int page_shift = shift_of(page_size);

    // the queries: both maps of a row, zero beyond the tile's rows and in the padding columns
    for (int c = threadIdx.x; c < DAM_ROWS * 2 * MCH; c += DAM_THREADS) {
        const int r = c / (2 * MCH), cc = c % (2 * MCH);
        const int map = cc / MCH, col = (cc % MCH) * 8;
        const bool valid = r < rows_here && col < D;
        cp_async16(sQ + r * KS + map * DKP + col, valid ? q_row0 + (size_t)r * q_step + map * D + col : q, valid);
    }
    load_diff_tiles<DKP, DVP>(sK, sV, k_cache, v_cache, table, max_pages, num_pages, page_size, page_shift, Hkv, kvh, D, DV,
                              first_kt * DAM_KEYS, key_lo, key_end);
    cp_async_commit();

    float o[2][DTILES][4];
    float m_run[2][2], l_run[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int i = 0; i < DTILES; ++i) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.0f;
        m_run[m][0] = m_run[m][1] = -INFINITY;
        l_run[m][0] = l_run[m][1] = 0.0f;
    }
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;
    const int qpos0 = first_pos + (warp * 16 + g) * pos_step;
    const int qpos1 = first_pos + (warp * 16 + g + 8) * pos_step;
    const int mm = lane >> 3;

    int stage = 0;
    for (int kt = first_kt; kt <= last_kt; ++kt) {
        if (kt + 1 <= last_kt) {
            load_diff_tiles<DKP, DVP>(sK + (stage ^ 1) * DAM_KEYS * KS, sV + (stage ^ 1) * DAM_KEYS * VS, k_cache, v_cache, table, max_pages,
                                      num_pages, page_size, page_shift, Hkv, kvh, D, DV, (kt + 1) * DAM_KEYS, key_lo, key_end);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* tK = sK + stage * DAM_KEYS * KS;
        const __nv_bfloat16* tV = sV + stage * DAM_KEYS * VS;
        const int key_base = kt * DAM_KEYS + tq * 2;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float s[DAM_KEYS / 8][4];
#pragma unroll
            for (int nt = 0; nt < DAM_KEYS / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                uint32_t a[4];
                ldmatrix_x4(a, sQ + (warp * 16 + (mm & 1) * 8 + (lane & 7)) * KS + m * DKP + ks * 16 + (mm >> 1) * 8);
#pragma unroll
                for (int np = 0; np < DAM_KEYS / 16; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, tK + (np * 16 + (mm >> 1) * 8 + (lane & 7)) * KS + m * DKP + ks * 16 + (mm & 1) * 8);
                    mma_16816(s[2 * np], a, b[0], b[1]);
                    mma_16816(s[2 * np + 1], a, b[2], b[3]);
                }
            }
            // scale, cap, mask; scores end up in units of log2 for exp2
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < DAM_KEYS / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key_base + nt * 8 + e;
                    const bool ok0 = key <= qpos0 && (window <= 0 || key > qpos0 - window);
                    const bool ok1 = key <= qpos1 && (window <= 0 || key > qpos1 - window);
                    float v0 = s[nt][e], v1 = s[nt][2 + e];
                    if (cap > 0.0f) {
                        v0 = cap2 * tanh_from_exp(v0 * scale * inv_cap);
                        v1 = cap2 * tanh_from_exp(v1 * scale * inv_cap);
                    } else {
                        v0 *= scale2;
                        v1 *= scale2;
                    }
                    s[nt][e] = ok0 ? v0 : -INFINITY;
                    s[nt][2 + e] = ok1 ? v1 : -INFINITY;
                    mx0 = fmaxf(mx0, s[nt][e]);
                    mx1 = fmaxf(mx1, s[nt][2 + e]);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m_run[m][0], mx0), mn1 = fmaxf(m_run[m][1], mx1);
            const float base0 = mn0 == -INFINITY ? 0.0f : mn0;  // a row that has seen no key yet stays at zero
            const float base1 = mn1 == -INFINITY ? 0.0f : mn1;
            const float alpha0 = exp2f(m_run[m][0] - base0), alpha1 = exp2f(m_run[m][1] - base1);
            m_run[m][0] = mn0;
            m_run[m][1] = mn1;
            float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
            for (int nt = 0; nt < DAM_KEYS / 8; ++nt) {
                s[nt][0] = exp2f(s[nt][0] - base0);
                s[nt][1] = exp2f(s[nt][1] - base0);
                s[nt][2] = exp2f(s[nt][2] - base1);
                s[nt][3] = exp2f(s[nt][3] - base1);
                sum0 += s[nt][0] + s[nt][1];
                sum1 += s[nt][2] + s[nt][3];
            }
            l_run[m][0] = l_run[m][0] * alpha0 + sum0;
            l_run[m][1] = l_run[m][1] * alpha1 + sum1;
#pragma unroll
            for (int dt = 0; dt < DTILES; ++dt) {
                o[m][dt][0] *= alpha0;
                o[m][dt][1] *= alpha0;
                o[m][dt][2] *= alpha1;
                o[m][dt][3] *= alpha1;
            }
            // O_m += P_m V
#pragma unroll
            for (int kk = 0; kk < DAM_KEYS / 16; ++kk) {
                uint32_t a[4];
                a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, tV + (kk * 16 + (mm & 1) * 8 + (lane & 7)) * VS + dp * 16 + (mm >> 1) * 8);
                    mma_16816(o[m][2 * dp], a, b[0], b[1]);
                    mma_16816(o[m][2 * dp + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();  // the buffer is refilled by the next turn's request
        stage ^= 1;
    }

    // finish: the maps' sums across the quad, o = a_1 - lambda a_2, the head norm, the store
    float inv[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float l = l_run[m][half];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            inv[m][half] = l > 0.0f ? 1.0f / l : 0.0f;
        }
    float squares0 = 0.0f, squares1 = 0.0f;
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            o[0][dt][e] = o[0][dt][e] * inv[0][0] - lambda * (o[1][dt][e] * inv[1][0]);
            o[0][dt][2 + e] = o[0][dt][2 + e] * inv[0][1] - lambda * (o[1][dt][2 + e] * inv[1][1]);
            squares0 += o[0][dt][e] * o[0][dt][e];
            squares1 += o[0][dt][2 + e] * o[0][dt][2 + e];
        }
    }
    float factor0 = 1.0f, factor1 = 1.0f;
    if (head_norm) {
        squares0 += __shfl_xor_sync(0xffffffffu, squares0, 1);
        squares0 += __shfl_xor_sync(0xffffffffu, squares0, 2);
        squares1 += __shfl_xor_sync(0xffffffffu, squares1, 1);
        squares1 += __shfl_xor_sync(0xffffffffu, squares1, 2);
        factor0 = rsqrtf(squares0 / (float)DV + eps) * out_scale;  // the padding columns hold zeros
        factor1 = rsqrtf(squares1 / (float)DV + eps) * out_scale;
    }
    const int r0 = warp * 16 + g, r1 = r0 + 8;
#pragma unroll
    for (int dt = 0; dt < DTILES; ++dt) {
        const int col = dt * 8 + tq * 2;
        if (col >= DV) continue;
        if (r0 < rows_here)
            *reinterpret_cast<__nv_bfloat162*>(out_row0 + (size_t)r0 * out_step + col) = __floats2bfloat162_rn(o[0][dt][0] * factor0, o[0][dt][1] * factor0);
        if (r1 < rows_here)
            *reinterpret_cast<__nv_bfloat162*>(out_row0 + (size_t)r1 * out_step + col) = __floats2bfloat162_rn(o[0][dt][2] * factor1, o[0][dt][3] * factor1);
    }
    (void)flag;
}


// ------------------------------------------------------------------ single tokens, up to 16 query heads a key/value head
// The heads of one key/value head are the 16 rows of ONE m16 tile, and the four warps share a 64-key tile
// by keys: warp w takes keys 16 w .. 16 w + 15 of every tile with online softmaxes of its own, so no tensor-core
// work is spent on rows that are not there.  The warps' partial results (running maximum, sum and accumulator
// per map and row) meet in shared memory at the end, in warp order; a result depends on the token's position alone.
template <int DKP, int DVP>
struct SingleTile {
    static constexpr int KS = DiffTile<DKP, DVP>::KSTRIDE, VS = DiffTile<DKP, DVP>::VSTRIDE;
    static constexpr int STAGES = 3;  // two tiles on their way while one is worked on: a block is a chain of loads, and few blocks an SM run
    static constexpr size_t STREAM = (size_t)(16 * KS + STAGES * DAM_KEYS * KS + STAGES * DAM_KEYS * VS) * sizeof(__nv_bfloat16);
    static constexpr size_t MERGE = (size_t)(4 * 2 * 16 * DVP + 2 * 4 * 2 * 16 + 16 * DVP) * sizeof(float);
    static constexpr size_t BYTES = STREAM > MERGE ? STREAM : MERGE;
};

template <int DKP, int DVP>
__global__ void __launch_bounds__(DAM_THREADS)
diff_attention_single_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out, int out_stride,
                             const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                             const int* __restrict__ seq_lens, const int* __restrict__ block_table, int max_pages,
                             const int* __restrict__ list_rows, const int* __restrict__ list_tokens, int Hq, int Hkv, int D, int DV,
                             int page_size, int num_pages, float scale, float cap, int window, float lambda, int head_norm, float eps,
                             float out_scale) {
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int KS = SingleTile<DKP, DVP>::KS, VS = SingleTile<DKP, DVP>::VS;
    constexpr int KSTEPS = DKP / 16, DTILES = DVP / 8, MCH = DKP / 8;
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // 16 rows
    __nv_bfloat16* sK = sQ + 16 * KS;
    constexpr int STAGES = SingleTile<DKP, DVP>::STAGES;
    __nv_bfloat16* sV = sK + STAGES * DAM_KEYS * KS;

    const int group = Hq / Hkv;
    const int kvh = blockIdx.x;
    const int row = list_rows[blockIdx.y];
    const int token = list_tokens[blockIdx.y];
    const int pos = seq_lens[row] - 1;
    const __nv_bfloat16* q_row0 = q + (size_t)token * q_stride + (size_t)kvh * group * 2 * D;
    const int* table = block_table + (size_t)row * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3, mm = lane >> 3;
    const int key_end = pos + 1;
    const int key_lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int first_kt = key_lo / DAM_KEYS, last_kt = (key_end - 1) / DAM_KEYS;
    const int page_shift = shift_of(page_size);

    for (int c = threadIdx.x; c < 16 * 2 * MCH; c += DAM_THREADS) {
        const int r = c / (2 * MCH), cc = c % (2 * MCH);
        const int map = cc / MCH, col = (cc % MCH) * 8;
        const bool valid = r < group && col < D;
        cp_async16(sQ + r * KS + map * DKP + col, valid ? q_row0 + (size_t)r * 2 * D + map * D + col : q, valid);
    }
    // one copy group a tile, also where there is no tile left, so that "all but the last two groups" always names the tile at hand
#pragma unroll
    for (int ahead = 0; ahead < STAGES - 1; ++ahead) {
        if (first_kt + ahead <= last_kt)
            load_diff_tiles<DKP, DVP>(sK + ahead * DAM_KEYS * KS, sV + ahead * DAM_KEYS * VS, k_cache, v_cache, table, max_pages, num_pages, page_size,
                                      page_shift, Hkv, kvh, D, DV, (first_kt + ahead) * DAM_KEYS, key_lo, key_end);
        cp_async_commit();
    }

    float o[2][DTILES][4];
    float m_run[2][2], l_run[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
#pragma unroll
        for (int i = 0; i < DTILES; ++i) o[m][i][0] = o[m][i][1] = o[m][i][2] = o[m][i][3] = 0.0f;
        m_run[m][0] = m_run[m][1] = -INFINITY;
        l_run[m][0] = l_run[m][1] = 0.0f;
    }
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;
    const float cap2 = cap * LOG2E, scale2 = scale * LOG2E;

    int stage = 0;
    for (int kt = first_kt; kt <= last_kt; ++kt) {
        if (kt + STAGES - 1 <= last_kt) {
            const int into = (stage + STAGES - 1) % STAGES;  // the buffer the turn before this one worked on
            load_diff_tiles<DKP, DVP>(sK + into * DAM_KEYS * KS, sV + into * DAM_KEYS * VS, k_cache, v_cache, table, max_pages, num_pages, page_size,
                                      page_shift, Hkv, kvh, D, DV, (kt + STAGES - 1) * DAM_KEYS, key_lo, key_end);
        }
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        const __nv_bfloat16* tK = sK + stage * DAM_KEYS * KS + warp * 16 * KS;  // this warp's 16 keys
        const __nv_bfloat16* tV = sV + stage * DAM_KEYS * VS + warp * 16 * VS;
        const int key_base = kt * DAM_KEYS + warp * 16 + tq * 2;
        if (kt * DAM_KEYS + warp * 16 <= pos && kt * DAM_KEYS + warp * 16 + 15 >= key_lo) {  // some key of the 16 is seen
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                float s[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    uint32_t a[4], b[4];
                    ldmatrix_x4(a, sQ + ((mm & 1) * 8 + (lane & 7)) * KS + m * DKP + ks * 16 + (mm >> 1) * 8);
                    ldmatrix_x4(b, tK + ((mm >> 1) * 8 + (lane & 7)) * KS + m * DKP + ks * 16 + (mm & 1) * 8);
                    mma_16816(s[0], a, b[0], b[1]);
                    mma_16816(s[1], a, b[2], b[3]);
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = key_base + nt * 8 + e;
                        const bool ok = key <= pos && key >= key_lo;  // every row is the same token
                        float v0 = s[nt][e], v1 = s[nt][2 + e];
                        if (cap > 0.0f) {
                            v0 = cap2 * tanh_from_exp(v0 * scale * inv_cap);
                            v1 = cap2 * tanh_from_exp(v1 * scale * inv_cap);
                        } else {
                            v0 *= scale2;
                            v1 *= scale2;
                        }
                        s[nt][e] = ok ? v0 : -INFINITY;
                        s[nt][2 + e] = ok ? v1 : -INFINITY;
                        mx0 = fmaxf(mx0, s[nt][e]);
                        mx1 = fmaxf(mx1, s[nt][2 + e]);
                    }
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float mn0 = fmaxf(m_run[m][0], mx0), mn1 = fmaxf(m_run[m][1], mx1);
                const float base0 = mn0 == -INFINITY ? 0.0f : mn0, base1 = mn1 == -INFINITY ? 0.0f : mn1;
                const float alpha0 = exp2f(m_run[m][0] - base0), alpha1 = exp2f(m_run[m][1] - base1);
                m_run[m][0] = mn0;
                m_run[m][1] = mn1;
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    s[nt][0] = exp2f(s[nt][0] - base0);
                    s[nt][1] = exp2f(s[nt][1] - base0);
                    s[nt][2] = exp2f(s[nt][2] - base1);
                    s[nt][3] = exp2f(s[nt][3] - base1);
                    sum0 += s[nt][0] + s[nt][1];
                    sum1 += s[nt][2] + s[nt][3];
                }
                l_run[m][0] = l_run[m][0] * alpha0 + sum0;
                l_run[m][1] = l_run[m][1] * alpha1 + sum1;
                uint32_t a[4];
                a[0] = pack_bf16(s[0][0], s[0][1]);
                a[1] = pack_bf16(s[0][2], s[0][3]);
                a[2] = pack_bf16(s[1][0], s[1][1]);
                a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    o[m][2 * dp][0] *= alpha0; o[m][2 * dp][1] *= alpha0; o[m][2 * dp][2] *= alpha1; o[m][2 * dp][3] *= alpha1;
                    o[m][2 * dp + 1][0] *= alpha0; o[m][2 * dp + 1][1] *= alpha0; o[m][2 * dp + 1][2] *= alpha1; o[m][2 * dp + 1][3] *= alpha1;
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, tV + ((mm & 1) * 8 + (lane & 7)) * VS + dp * 16 + (mm >> 1) * 8);
                    mma_16816(o[m][2 * dp], a, b[0], b[1]);
                    mma_16816(o[m][2 * dp + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();
        stage = (stage + 1) % STAGES;
    }
    cp_async_wait<0>();

    // the warps' partial results meet (the key and value buffers are free now)
    float* part_o = reinterpret_cast<float*>(smem_raw);   // [warp][map][16][DVP]
    float* part_m = part_o + 4 * 2 * 16 * DVP;            // [warp][map][16]
    float* part_l = part_m + 4 * 2 * 16;
    float* final_o = part_l + 4 * 2 * 16;                 // [16][DVP]
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float l0 = l_run[m][0], l1 = l_run[m][1];
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
        const int slot = (warp * 2 + m) * 16;
        if (tq == 0) {
            part_m[slot + g] = m_run[m][0];
            part_m[slot + g + 8] = m_run[m][1];
            part_l[slot + g] = l0;
            part_l[slot + g + 8] = l1;
        }
#pragma unroll
        for (int dt = 0; dt < DTILES; ++dt) {
            const int col = dt * 8 + tq * 2;
            *reinterpret_cast<float2*>(part_o + (size_t)(slot + g) * DVP + col) = make_float2(o[m][dt][0], o[m][dt][1]);
            *reinterpret_cast<float2*>(part_o + (size_t)(slot + g + 8) * DVP + col) = make_float2(o[m][dt][2], o[m][dt][3]);
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * DVP; idx += DAM_THREADS) {
        const int r = idx / DVP, c = idx % DVP;
        float both[2];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            float top = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) top = fmaxf(top, part_m[(w * 2 + m) * 16 + r]);
            float denom = 0.0f, value = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = part_m[(w * 2 + m) * 16 + r];
                const float weight = mw == -INFINITY ? 0.0f : exp2f(mw - top);
                denom += part_l[(w * 2 + m) * 16 + r] * weight;
                value += part_o[(size_t)((w * 2 + m) * 16 + r) * DVP + c] * weight;
            }
            both[m] = denom > 0.0f ? value / denom : 0.0f;
        }
        final_o[idx] = both[0] - lambda * both[1];
    }
    __syncthreads();
    for (int r = warp; r < group; r += 4) {
        float squares = 0.0f;
        for (int c = lane; c < DV; c += 32) squares += final_o[r * DVP + c] * final_o[r * DVP + c];
        const float factor = head_norm ? rsqrtf(warp_sum(squares) / (float)DV + eps) * out_scale : 1.0f;
        __nv_bfloat16* dst = out + (size_t)token * out_stride + (size_t)(kvh * group + r) * DV;
        for (int c = lane; c < DV; c += 32) dst[c] = __float2bfloat16_rn(final_o[r * DVP + c] * factor);
    }
}

template <int DKP, int DVP>
static int launch_diff(const void* q, int q_stride, void* out, int out_stride, const void* k_cache, const void* v_cache, const int* qo_indptr,
                       const int* seq_lens, const int* block_table, int max_pages, const int* list_rows, const int* list_second, int count,
                       int single, int Hq, int Hkv, int D, int DV, int page_size, int num_pages, float scale, float cap, int window,
                       float lambda, int head_norm, float eps, float out_scale, int* flag, cudaStream_t stream) {
    constexpr size_t smem = DiffTile<DKP, DVP>::BYTES;
    static bool configured = false;
    if (!configured) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(diff_attention_mma_kernel<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = true;
    }
    dim3 grid(single ? Hkv : Hq, count);
    if (single && Hq / Hkv <= 16) {
        constexpr size_t bytes = SingleTile<DKP, DVP>::BYTES;
        static bool single_configured = false;
        if (!single_configured) {
            if (bytes > 48 * 1024) cudaFuncSetAttribute(diff_attention_single_kernel<DKP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            single_configured = true;
        }
        kb_launch(diff_attention_single_kernel<DKP, DVP>, grid, dim3(DAM_THREADS), bytes, stream, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,
                  out_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, seq_lens, block_table, max_pages, list_rows, list_second,
                  Hq, Hkv, D, DV, page_size, num_pages, scale, cap, window, lambda, head_norm, eps, out_scale);
        return kb_launch_result();
    }
    kb_launch(diff_attention_mma_kernel<DKP, DVP>, grid, dim3(DAM_THREADS), smem, stream, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out,
              out_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, qo_indptr, seq_lens, block_table, max_pages, list_rows,
              list_second, single, Hq, Hkv, D, DV, page_size, num_pages, scale, cap, window, lambda, head_norm, eps, out_scale, flag);
    return kb_launch_result();
}

static int padded(int d) { return d <= 32 ? 32 : d <= 64 ? 64 : 128; }

KB_EXPORT int kb_diff_attention_mma_supported(int D, int DV, int Hq, int Hkv) {
    return D >= 16 && D <= 128 && D % 16 == 0 && DV >= 16 && DV <= 128 && DV % 16 == 0 && Hkv >= 1 && Hq % Hkv == 0 && Hq / Hkv <= DAM_ROWS;
}

// `single` = 0: list_rows / list_second are the request row and the first query of each 64-query tile of the
// step's portions (count tiles; qo_indptr gives the portions).  `single` = 1: they are the request row and the
// flat token index of each single-token row (count rows).
KB_EXPORT int kb_diff_attention_mma(const void* q, int q_stride, void* out, int out_stride, const void* k_cache, const void* v_cache,
                                    const int* qo_indptr, const int* seq_lens, const int* block_table, int max_pages, const int* list_rows,
                                    const int* list_second, int count, int single, int Hq, int Hkv, int D, int DV, int page_size,
                                    int num_pages, float scale, float cap, int window, float lambda, int head_norm, float eps,
                                    float out_scale, int* flag, cudaStream_t stream) {
    if (count == 0) return 0;
    if (!q || !out || !k_cache || !v_cache || !seq_lens || !block_table || !list_rows || !list_second || (!single && !qo_indptr)) return KB_ERR_NULL;
    if (!kb_diff_attention_mma_supported(D, DV, Hq, Hkv)) return KB_ERR_UNSUPPORTED_SIZE;
    if (count > 65535 || q_stride % 8 || out_stride % 2 || ((uintptr_t)q % 16) || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16)) return KB_ERR_BAD_ARG;
#define ARGS q, q_stride, out, out_stride, k_cache, v_cache, qo_indptr, seq_lens, block_table, max_pages, list_rows, list_second, count, single, \
             Hq, Hkv, D, DV, page_size, num_pages, scale, cap, window, lambda, head_norm, eps, out_scale, flag, stream
    const int dk = padded(D), dv = padded(DV);
    if (dk == 32) return dv == 32 ? launch_diff<32, 32>(ARGS) : dv == 64 ? launch_diff<32, 64>(ARGS) : launch_diff<32, 128>(ARGS);
    if (dk == 64) return dv == 32 ? launch_diff<64, 32>(ARGS) : dv == 64 ? launch_diff<64, 64>(ARGS) : launch_diff<64, 128>(ARGS);
    return dv == 32 ? launch_diff<128, 32>(ARGS) : dv == 64 ? launch_diff<128, 64>(ARGS) : launch_diff<128, 128>(ARGS);
#undef ARGS
}
