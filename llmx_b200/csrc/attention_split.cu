// Softmax attention whose keys and values have widths of their own, over pages that hold one [key ; value] row per
// token and key/value head: cache [pages, 1, kv_heads, page_size, D + V].
//
// Two kernels.  `llmx_qk_norm_rope_write` finishes the rows of the stacked q/k/v product: an RMS norm per head with a
// weight of D values shared by the heads (optional), a rotation of the first 2 * rot_half values of every query and
// key head (value i pairs with value i + rot_half; the angle is position * freq[i], made in 32-bit here, so there is
// no table whose length bounds the context), queries to `q_out`, keys and values to the row's cache slot.
// `llmx_attention_split` is the plain form of the attention: one block per (row, head); a row at position p reads the
// keys lo..p of its own request, where lo is the larger of p - window + 1 (window > 0) and the start of p's chunk,
// floor(p / chunk) * chunk (chunk > 0: positions are counted from the start of the request, so chunks do not move
// with the way a prompt was cut); query head h reads key/value head h / (heads / kv_heads).
//   s_t = dot(q, k_t) * scale;  m = max s;  e_t = exp(s_t - m);  l = sum e_t;  o = sum_t (e_t / l) v_t
// in the online form, 32-bit.  Each warp walks every fourth key in increasing order and the four partial states are
// merged in warp order, so the order of a row's sums depends on its own keys only.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;  // head widths up to 256

template <typename QT, typename KVT>
__global__ void __launch_bounds__(128)
qk_write_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ q_weight,
                const float* __restrict__ k_weight, float eps, const float* __restrict__ freq, int rot_half,
                const int* __restrict__ positions, const int* __restrict__ slots, QT* __restrict__ q_out,
                KVT* __restrict__ cache, int heads, int kv_heads, int D, int V, int page_size) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float pos = (float)positions[row];
    const int slot = slots[row];
    const float* src = proj + (size_t)row * stride;
    const int v_off = (heads + kv_heads) * D;
    for (int item = warp; item < heads + kv_heads; item += warps) {
        const bool is_q = item < heads;
        const float* x = src + (size_t)item * D;                     // q heads, then k heads, lie one after the other
        const float* w = is_q ? q_weight : k_weight;
        float val[MAX_PER_LANE];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            val[i] = d < D ? x[d] : 0.0f;
            ss = fmaf(val[i], val[i], ss);
        }
        QT* qdst = is_q ? q_out + ((size_t)row * heads + item) * D : nullptr;
        KVT* kdst = nullptr;
        if (!is_q) {
            if (slot < 0) continue;                                  // a row whose cache write is skipped
            const int g = item - heads;
            kdst = cache + (((size_t)(slot / page_size) * kv_heads + g) * page_size + slot % page_size) * (size_t)(D + V);
        }
        // A rotated value needs its partner, which another lane holds: each lane reads the partner from the input again
        // and norms it with the head's factor (through shared memory would cost a barrier a head).
        float rr = 1.0f;
        if (w != nullptr) rr = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d >= D) continue;
            float out = w != nullptr ? val[i] * rr * w[d] : val[i];
            if (d < 2 * rot_half) {
                const bool low = d < rot_half;
                const int fi = low ? d : d - rot_half;
                const int pd = low ? d + rot_half : d - rot_half;
                float partner = x[pd];
                if (w != nullptr) partner = partner * rr * w[pd];
                float s, c;
                sincosf(pos * freq[fi], &s, &c);
                out = low ? out * c - partner * s : out * c + partner * s;
            }
            if (is_q) qdst[d] = from_float<QT>(out);
            else kdst[d] = from_float<KVT>(out);
        }
        if (!is_q) {
            const float* vsrc = src + v_off + (size_t)(item - heads) * V;
            for (int d = lane; d < V; d += 32) kdst[D + d] = from_float<KVT>(vsrc[d]);
        }
    }
}

template <typename QT, typename KVT>
__global__ void __launch_bounds__(WARPS * 32)
attention_split_kernel(const QT* __restrict__ q, const KVT* __restrict__ cache, QT* __restrict__ out,
                       const int* __restrict__ row_request, const int* __restrict__ positions,
                       const int* __restrict__ block_tables, int table_stride, int heads, int kv_heads, int D, int V,
                       int page_size, int window, int chunk, float scale) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];  // WARPS * (V + 2)
    const int row = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = h / (heads / kv_heads);
    const int pos = positions[row];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const int* table = block_tables + (size_t)row_request[row] * table_stride;
    const int W = D + V;

    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const QT* qrow = q + ((size_t)row * heads + h) * D;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        qv[i] = d < D ? to_float(qrow[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int t = lo + warp; t <= pos; t += WARPS) {
        const int page = table[t / page_size], off = t % page_size;
        const KVT* kp = cache + (((size_t)page * kv_heads + g) * page_size + off) * (size_t)W;
        const KVT* vp = kp + D;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < D) s = fmaf(qv[i], to_float(kp[d]), s);
        }
        s = warp_sum(s) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
        const float e = expf(s - m_new);
        l = l * corr + e;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            if (d < V) acc[i] = fmaf(e, to_float(vp[d]), acc[i] * corr);
        }
        m = m_new;
    }
    float* mine = smem + warp * (V + 2);
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int d = lane + 32 * i;
        if (d < V) mine[d] = acc[i];
    }
    if (lane == 0) {
        mine[V] = m;
        mine[V + 1] = l;
    }
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, smem[w * (V + 2) + V]);
        float ll = 0.0f;
        float f[WARPS];
        for (int w = 0; w < WARPS; ++w) {
            const float mw = smem[w * (V + 2) + V];
            f[w] = mw == -INFINITY ? 0.0f : expf(mw - mm);
            ll += smem[w * (V + 2) + V + 1] * f[w];
        }
        QT* orow = out + ((size_t)row * heads + h) * V;
        for (int d = lane; d < V; d += 32) {
            float o = 0.0f;
            for (int w = 0; w < WARPS; ++w) o += smem[w * (V + 2) + d] * f[w];
            orow[d] = from_float<QT>(o / ll);
        }
    }
}
}  // namespace

// proj float32 [rows, stride]: queries (heads * D), keys (kv_heads * D), values (kv_heads * V) in this order.
// q_weight, k_weight float32 [D] or null (no norm); freq float32 [rot_half]; q_out [rows, heads * D] of `q_dtype`;
// cache [pages, 1, kv_heads, page_size, D + V] of `cache_dtype`; slots int32 [rows] (page * page_size + offset; negative
// skips the row's cache write).
LLMX_EXPORT int llmx_qk_norm_rope_write(const float* proj, int stride, const float* q_weight, const float* k_weight,
                                        float eps, const float* freq, int rot_half, const int* positions,
                                        const int* slots, void* q_out, int q_dtype, void* cache, int cache_dtype, int rows,
                                        int heads, int kv_heads, int D, int V, int page_size, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (D <= 0 || V <= 0 || D > 32 * MAX_PER_LANE || 2 * rot_half > D || rot_half < 0 || (rot_half > 0 && freq == nullptr) ||
        (q_weight == nullptr) != (k_weight == nullptr))
        return LLMX_ERR_UNSUPPORTED;
#define LLMX_QKW(QT, KVT)                                                                                              \
    launch_kernel(qk_write_kernel<QT, KVT>, dim3(rows), dim3(128), 0, stream, proj, stride, q_weight, k_weight, eps,   \
                  freq, rot_half, positions, slots, (QT*)q_out, (KVT*)cache, heads, kv_heads, D, V, page_size)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_QKW(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_QKW(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_QKW(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_QKW(float, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_QKW
    return launch_status();
}

// q [rows, heads, D] and out [rows, heads, V] of `q_dtype`; the cache as above, of `cache_dtype`.
LLMX_EXPORT int llmx_attention_split(const void* q, int q_dtype, const void* cache, int cache_dtype, void* out,
                                     const int* row_request, const int* positions, const int* block_tables,
                                     int table_stride, int rows, int heads, int kv_heads, int D, int V, int page_size,
                                     int window, int chunk, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (D <= 0 || V <= 0 || D > 32 * MAX_PER_LANE || V > 32 * MAX_PER_LANE || heads % kv_heads || heads > 65535)
        return LLMX_ERR_UNSUPPORTED;
    dim3 grid(rows, heads);
    const size_t shmem = (size_t)WARPS * (V + 2) * sizeof(float);
#define LLMX_SPLIT(QT, KVT)                                                                                            \
    launch_kernel(attention_split_kernel<QT, KVT>, dim3(grid), dim3(WARPS * 32), shmem, stream, (const QT*)q,         \
                  (const KVT*)cache, (QT*)out, row_request, positions, block_tables, table_stride, heads, kv_heads, D, \
                  V, page_size, window, chunk, scale)
    if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) LLMX_SPLIT(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) LLMX_SPLIT(__nv_bfloat16, float);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) LLMX_SPLIT(float, __nv_bfloat16);
    else if (q_dtype == LLMX_F32 && cache_dtype == LLMX_F32) LLMX_SPLIT(float, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_SPLIT
    return launch_status();
}
