// Attention over a cache of latents: every token keeps one vector [c ; r] -- a normed latent c of C values from
// which every head's unrotated key and value are linear maps (k_h = Wuk_h c, v_h = Wuv_h c), and one rotated
// key part r of R values that all heads share.  A query head brings D unrotated and R rotated values.  The score
//     s = (q_plain . Wuk_h c + q_rot . r) * scale
// is computed without ever making the keys: q_plain is carried through the key map once per query,
//     qc = Wuk_h^T q_plain   (C values),   s = (qc . c + q_rot . r) * scale,
// and the values are made after the weighted sum: o_h = Wuv_h (sum_t p_t c_t).  Both maps cost D x C and V x C
// multiply-adds per (row, head), whatever the number of keys, and the cache row is read as it lies.
//
// `llmx_latent_write`: per row, RMS norm of the first C values of the down projection's output (weight, eps),
// rotation of the last R by the row's position, both stored to the row's cache slot.
// `llmx_latent_attention`: one block per (row, head): rotation of the query's rotated part, the key map, an online
// softmax over the row's keys lo..p (lo = max(0, p - window + 1), window <= 0: all), warps taking every fourth key
// in increasing order and merged in warp order, then the value map.  Scores, weights and sums are 32-bit.
//
// Rotation: pairs (2i, 2i + 1), i < dims / 2, of the rotated part turn by angle p * f_i, f_i = base^(-2i / dims), given
// as a float table; the angle is the float product, its cosine and sine the precise functions.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;

template <typename KVT>
__global__ void __launch_bounds__(128)
latent_write_kernel(const float* __restrict__ dkv, int stride, const float* __restrict__ w, float eps,
                    const float* __restrict__ freq, int rot_pairs, const int* __restrict__ positions,
                    const int* __restrict__ slots, KVT* __restrict__ cache, int C, int R) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[32];
    const int row = blockIdx.x;
    const int slot = slots[row];
    if (slot < 0) return;
    const float* src = dkv + (size_t)row * stride;
    KVT* dst = cache + (size_t)slot * (C + R);
    float s = 0.0f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) s = fmaf(src[i], src[i], s);
    const float rr = 1.0f / sqrtf(block_sum(s, scratch) / (float)C + eps);
    for (int i = threadIdx.x; i < C; i += blockDim.x) dst[i] = from_float<KVT>(src[i] * rr * w[i]);
    const float p = (float)positions[row];
    for (int i = threadIdx.x; i < R / 2; i += blockDim.x) {
        const float a = src[C + 2 * i], b = src[C + 2 * i + 1];
        if (i < rot_pairs) {
            float sn, cs;
            sincosf(p * freq[i], &sn, &cs);
            dst[C + 2 * i] = from_float<KVT>(a * cs - b * sn);
            dst[C + 2 * i + 1] = from_float<KVT>(b * cs + a * sn);
        } else {
            dst[C + 2 * i] = from_float<KVT>(a);
            dst[C + 2 * i + 1] = from_float<KVT>(b);
        }
    }
    if ((R & 1) && threadIdx.x == 0) dst[C + R - 1] = from_float<KVT>(src[C + R - 1]);
}

// PL: values of a cache row a lane holds (C + R <= 32 * PL).
template <typename WT, typename KVT, int PL>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_kernel(const float* __restrict__ q, int q_stride, const KVT* __restrict__ cache,
                        const WT* __restrict__ w_uk, const WT* __restrict__ w_uv, WT* __restrict__ out,
                        const float* __restrict__ freq, int rot_pairs, const int* __restrict__ row_request,
                        const int* __restrict__ positions, const int* __restrict__ block_tables, int table_stride,
                        int heads, int D, int R, int V, int C, int page_size, int window, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int W = C + R;
    float* qraw = smem;                       // D + R: the query head, its rotated part turned
    float* qk = qraw + D + R;                 // W: [Wuk^T q_plain ; q_rot] * scale
    float* part = qk + W;                     // WARPS * (C + 2)
    const int row = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_tables + (size_t)row_request[row] * table_stride;

    const float* qrow = q + (size_t)row * q_stride + (size_t)h * (D + R);
    for (int i = threadIdx.x; i < D + R; i += blockDim.x) qraw[i] = qrow[i];
    __syncthreads();
    for (int i = threadIdx.x; i < R / 2; i += blockDim.x) {
        const float a = qraw[D + 2 * i], b = qraw[D + 2 * i + 1];
        float ra = a, rb = b;
        if (i < rot_pairs) {
            float sn, cs;
            sincosf((float)pos * freq[i], &sn, &cs);
            ra = a * cs - b * sn;
            rb = b * cs + a * sn;
        }
        qk[C + 2 * i] = ra * scale;
        qk[C + 2 * i + 1] = rb * scale;
    }
    if ((R & 1) && threadIdx.x == 0) qk[C + R - 1] = qraw[D + R - 1] * scale;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const WT* col = w_uk + (size_t)h * D * C + c;
        float s = 0.0f;
        for (int d = 0; d < D; ++d) s = fmaf(qraw[d], to_float(col[(size_t)d * C]), s);
        qk[c] = s * scale;
    }
    __syncthreads();

    float qv[PL], acc[PL];
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        qv[i] = e < W ? qk[e] : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int t = lo + warp; t <= pos; t += WARPS) {
        const KVT* kp = cache + ((size_t)table[t / page_size] * page_size + t % page_size) * W;
        float kv[PL];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < PL; ++i) {
            const int e = lane + 32 * i;
            kv[i] = e < W ? to_float(kp[e]) : 0.0f;
            s = fmaf(qv[i], kv[i], s);
        }
        s = warp_sum(s);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < PL; ++i) acc[i] = fmaf(e, kv[i], acc[i] * corr);
        m = m_new;
    }
    float* mine = part + warp * (C + 2);
#pragma unroll
    for (int i = 0; i < PL; ++i) {
        const int e = lane + 32 * i;
        if (e < C) mine[e] = acc[i];
    }
    if (lane == 0) {
        mine[C] = m;
        mine[C + 1] = l;
    }
    __syncthreads();
    // The four partial states merged in warp order; the weighted sum of latents ends in part[0 .. C).
    float mm = -INFINITY;
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, part[w * (C + 2) + C]);
    float f[WARPS], ll = 0.0f;
    for (int w = 0; w < WARPS; ++w) {
        const float mw = part[w * (C + 2) + C];
        f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
        ll += part[w * (C + 2) + C + 1] * f[w];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float o = 0.0f;
        for (int w = 0; w < WARPS; ++w) o += part[w * (C + 2) + c] * f[w];
        qk[c] = o / ll;                        // qk is free now: the merged latent
    }
    __syncthreads();
    WT* orow = out + ((size_t)row * heads + h) * V;
    for (int v = warp; v < V; v += WARPS) {
        const WT* wr = w_uv + ((size_t)h * V + v) * C;
        float s = 0.0f;
        for (int c = lane; c < C; c += 32) s = fmaf(to_float(wr[c]), qk[c], s);
        s = warp_sum(s);
        if (lane == 0) orow[v] = from_float<WT>(s);
    }
}

template <typename WT, typename KVT>
int launch_attention(int pl, dim3 grid, size_t smem, cudaStream_t stream, const float* q, int q_stride, const void* cache,
                     const void* w_uk, const void* w_uv, void* out, const float* freq, int rot_pairs, const int* row_request,
                     const int* positions, const int* block_tables, int table_stride, int heads, int D, int R, int V, int C,
                     int page_size, int window, float scale) {
#define LLMX_LAT(P)                                                                                                       \
    do {                                                                                                                  \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(latent_attention_kernel<WT, KVT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(latent_attention_kernel<WT, KVT, P>, grid, dim3(WARPS * 32), smem, stream, q, q_stride,             \
                      (const KVT*)cache, (const WT*)w_uk, (const WT*)w_uv, (WT*)out, freq, rot_pairs, row_request,        \
                      positions, block_tables, table_stride, heads, D, R, V, C, page_size, window, scale);               \
    } while (0)
    if (pl <= 2) LLMX_LAT(2);
    else if (pl <= 4) LLMX_LAT(4);
    else if (pl <= 8) LLMX_LAT(8);
    else if (pl <= 12) LLMX_LAT(12);
    else if (pl <= 20) LLMX_LAT(20);
    else if (pl <= 32) LLMX_LAT(32);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_LAT
    return launch_status();
}
}  // namespace

// dkv float [rows, stride]: C latent values then R rotated-part values; w float [C]; freq float [rot_pairs];
// slots[row] = page * page_size + offset (negative: skip the row); cache [pages * page_size, C + R] of `cache_dtype`.
LLMX_EXPORT int llmx_latent_write(const float* dkv, int stride, const float* w, float eps, const float* freq, int rot_pairs,
                                  const int* positions, const int* slots, void* cache, int cache_dtype, int rows, int C,
                                  int R, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || R < 0 || 2 * rot_pairs > R) return LLMX_ERR_BAD_ARGUMENT;
    if (cache_dtype == LLMX_BF16)
        launch_kernel(latent_write_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, dkv, stride, w, eps, freq, rot_pairs, positions, slots, (__nv_bfloat16*)cache, C, R);
    else if (cache_dtype == LLMX_F32)
        launch_kernel(latent_write_kernel<float>, dim3(rows), dim3(128), 0, stream, dkv, stride, w, eps, freq, rot_pairs, positions, slots, (float*)cache, C, R);
    else return LLMX_ERR_UNSUPPORTED;
    return launch_status();
}

// q float [rows, q_stride]: per head D unrotated then R rotated-part values; w_uk [heads * D, C] and w_uv [heads * V, C]
// of `w_dtype`, which is also the type of out [rows, heads * V].
LLMX_EXPORT int llmx_latent_attention(const float* q, int q_stride, const void* cache, int cache_dtype, const void* w_uk,
                                      const void* w_uv, int w_dtype, void* out, const float* freq, int rot_pairs,
                                      const int* row_request, const int* positions, const int* block_tables,
                                      int table_stride, int rows, int heads, int D, int R, int V, int C, int page_size,
                                      int window, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (heads <= 0 || heads > 65535 || D <= 0 || R < 0 || V <= 0 || C <= 0 || 2 * rot_pairs > R || page_size <= 0)
        return LLMX_ERR_BAD_ARGUMENT;
    const int W = C + R;
    const int pl = (W + 31) / 32;
    const size_t smem = (size_t)(D + R + W + WARPS * (C + 2)) * sizeof(float);
    if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;
    const dim3 grid(rows, heads);
#define LLMX_GO(WT, KVT)                                                                                                  \
    return launch_attention<WT, KVT>(pl, grid, smem, stream, q, q_stride, cache, w_uk, w_uv, out, freq, rot_pairs,       \
                                     row_request, positions, block_tables, table_stride, heads, D, R, V, C, page_size,   \
                                     window, scale)
    if (w_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_GO(__nv_bfloat16, __nv_bfloat16);
    if (w_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_GO(__nv_bfloat16, float);
    if (w_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_GO(float, __nv_bfloat16);
    if (w_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_GO(float, float);
#undef LLMX_GO
    return LLMX_ERR_UNSUPPORTED;
}
