// A mixture of experts whose routing is a table: token id -> the `top` experts that token uses (no router product).
//
// A step's rows are sorted by expert on the device, so that nothing about the routing is read on the host and a step
// can be recorded and replayed.  A *pair* is (row, k): row r with the k-th expert of its token, numbered r * top + k.
//   llmx_moe_route       one block an expert walks the pairs in order and lists those that name it (so a list is in
//                        row order, whatever else the launch holds); then one block cuts the lists into tiles of
//                        TILE_ROWS pairs: (expert, first place in the list), compactly, with their number.
//   llmx_moe_gate_up     act[pair, f] = silu(h[row] . Wg_e[f]) * (h[row] . Wu_e[f])         (gate and up rows stacked per expert)
//   llmx_moe_down        y[pair, c]   = act[pair] . Wd_e[c]                                 (32-bit)
//   llmx_moe_combine     x[row]      += weight * sum_k y[row * top + k]                      (k in order: one order of sums)
// The products run one block a (tile of an expert's pairs, tile of output columns): rows are gathered through the
// list, the expert's weights are read once a tile.  Two forms: on the CUDA cores with explicit fmaf and k in
// increasing order (32-bit weights and rows: the true 32-bit path; also bfloat16 shapes the tensor-core form does not
// take), and on the tensor cores (mma.sync m16n8k16, bfloat16 in, 32-bit sums) for bfloat16 with K a multiple of 32.
#include "common.cuh"
#include <math.h>
#include <mma.h>

namespace {
constexpr int TILE_ROWS = 32;     // pairs a tile holds

__global__ void __launch_bounds__(256)
route_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int top, int rows, int experts, int vocab,
             int* __restrict__ lists, int* __restrict__ counts) {
    pdl_trigger();
    pdl_wait();
    __shared__ int warp_count[8];
    __shared__ int base;
    const int e = blockIdx.x;
    const int pairs = rows * top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int p0 = 0; p0 < pairs; p0 += 256) {
        const int p = p0 + threadIdx.x;
        bool mine = false;
        if (p < pairs) {
            const int tok = token_ids[p / top];
            mine = tok >= 0 && tok < vocab && table[(size_t)tok * top + p % top] == e;
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(ballot);
        __syncthreads();
        int before = base;
        for (int w = 0; w < warp; ++w) before += warp_count[w];
        if (mine) lists[(size_t)e * pairs + before + __popc(ballot & ((1u << lane) - 1u))] = p;
        __syncthreads();
        if (threadIdx.x == 0) {
            int total = 0;
            for (int w = 0; w < 8; ++w) total += warp_count[w];
            base += total;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) counts[e] = base;
}

// tiles: [0] their number, then (expert, first place) pairs from tiles[2] on.
__global__ void tiles_kernel(const int* __restrict__ counts, int experts, int* __restrict__ tiles) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0) return;
    int n = 0;
    for (int e = 0; e < experts; ++e)
        for (int at = 0; at < counts[e]; at += TILE_ROWS) {
            tiles[2 + 2 * n] = e;
            tiles[3 + 2 * n] = at;
            ++n;
        }
    tiles[0] = n;
}

// ---- the product on the CUDA cores ---------------------------------------------------------------------------------
// A block: TILE_ROWS pairs x 64 output columns, K in steps of 16; a thread owns 2 pairs x 4 columns (and, GATED, the
// same of the up rows).  A's rows are gathered: pair p reads row p / a_div of `a`.
constexpr int CC_COLS = 64, CC_K = 16;

template <typename T, bool GATED, typename OutT>
__global__ void __launch_bounds__(256)
moe_cores_kernel(const T* __restrict__ a, int a_div, const T* __restrict__ w, const int* __restrict__ lists,
                 const int* __restrict__ counts, const int* __restrict__ tiles, int pairs, OutT* __restrict__ out, int N,
                 int K) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[2 + 2 * blockIdx.x], at = tiles[3 + 2 * blockIdx.x];
    const int n_here = min(TILE_ROWS, counts[e] - at);
    const int* list = lists + (size_t)e * pairs + at;
    const int col0 = blockIdx.y * CC_COLS;
    __shared__ float As[CC_K][TILE_ROWS + 1];
    __shared__ float Ws[GATED ? 2 : 1][CC_K][CC_COLS + 1];
    __shared__ int src_pair[TILE_ROWS];
    if (threadIdx.x < TILE_ROWS) src_pair[threadIdx.x] = threadIdx.x < n_here ? list[threadIdx.x] : -1;
    __syncthreads();
    const int tr = threadIdx.x / 16, tc = threadIdx.x % 16;        // pairs 2 tr, 2 tr + 1; columns tc + 16 j
    float acc[2][4] = {}, acc2[2][4] = {};
    const T* wbase = w + (size_t)e * (GATED ? 2 : 1) * N * K;
    for (int k0 = 0; k0 < K; k0 += CC_K) {
        for (int i = threadIdx.x; i < TILE_ROWS * CC_K; i += 256) {
            const int r = i / CC_K, kk = i % CC_K;
            const int p = src_pair[r];
            As[kk][r] = (p >= 0 && k0 + kk < K) ? to_float(a[(size_t)(p / a_div) * K + k0 + kk]) : 0.0f;
        }
        for (int i = threadIdx.x; i < CC_COLS * CC_K; i += 256) {
            const int c = i / CC_K, kk = i % CC_K;
            const bool ok = col0 + c < N && k0 + kk < K;
            Ws[0][kk][c] = ok ? to_float(wbase[(size_t)(col0 + c) * K + k0 + kk]) : 0.0f;
            if (GATED) Ws[1][kk][c] = ok ? to_float(wbase[(size_t)(N + col0 + c) * K + k0 + kk]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < CC_K; ++kk) {
            const float a0 = As[kk][2 * tr], a1 = As[kk][2 * tr + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = Ws[0][kk][tc + 16 * j];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
                if (GATED) {
                    const float b2 = Ws[1][kk][tc + 16 * j];
                    acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
                    acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = src_pair[2 * tr + i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tc + 16 * j;
            if (c >= N) continue;
            float v = acc[i][j];
            if (GATED) v = v / (1.0f + expf(-v)) * acc2[i][j];
            out[(size_t)p * N + c] = from_float<OutT>(v);
        }
    }
}

// ---- the product on the tensor cores -------------------------------------------------------------------------------
// A block of four warps: TILE_ROWS (32) pairs x 64 output columns, K in steps of 32.  The weights are the A operand of
// mma.sync m16n8k16 (16 output columns a tile), the gathered rows the B operand (8 pairs a tile): warp w owns output
// columns 16 w .. 16 w + 15 for all 32 pairs (four tiles, and GATED four more for the up rows).  Operands go through
// shared memory as bfloat16 with rows padded by 8 values, so that the fragment reads of a warp fall into different
// banks; the next k step's values are fetched into registers while this one is multiplied.
constexpr int TC_COLS = 64, TC_K = 32, TC_PAD = 8;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool GATED, typename OutT>
__global__ void __launch_bounds__(128)
moe_tc_kernel(const __nv_bfloat16* __restrict__ a, int a_div, const __nv_bfloat16* __restrict__ w,
              const int* __restrict__ lists, const int* __restrict__ counts, const int* __restrict__ tiles, int pairs,
              OutT* __restrict__ out, int N, int K) {
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[2 + 2 * blockIdx.x], at = tiles[3 + 2 * blockIdx.x];
    const int n_here = min(TILE_ROWS, counts[e] - at);
    const int* list = lists + (size_t)e * pairs + at;
    const int col0 = blockIdx.y * TC_COLS;
    constexpr int NW = GATED ? 2 : 1;
    __shared__ __align__(16) __nv_bfloat16 Ws[NW][TC_COLS][TC_K + TC_PAD];
    __shared__ __align__(16) __nv_bfloat16 Bs[TILE_ROWS][TC_K + TC_PAD];
    __shared__ int src_pair[TILE_ROWS];
    if (threadIdx.x < TILE_ROWS) src_pair[threadIdx.x] = threadIdx.x < n_here ? list[threadIdx.x] : -1;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tig = lane & 3;
    const __nv_bfloat16* wbase = w + (size_t)e * NW * N * K;
    // What this thread copies a k step: 16-byte pieces (8 values).  Weights: NW * 64 rows x 4 pieces; rows: 32 x 4.
    constexpr int W_PIECES = NW * TC_COLS * (TC_K / 8) / 128, B_PIECES = TILE_ROWS * (TC_K / 8) / 128;
    uint4 wreg[W_PIECES], breg[B_PIECES];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < W_PIECES; ++i) {
            const int piece = threadIdx.x + 128 * i;
            const int which = piece / (TC_COLS * (TC_K / 8)), rest = piece % (TC_COLS * (TC_K / 8));
            const int c = rest / (TC_K / 8), kp = rest % (TC_K / 8);
            wreg[i] = col0 + c < N ? *reinterpret_cast<const uint4*>(wbase + (size_t)(which * N + col0 + c) * K + k0 + 8 * kp)
                                   : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < B_PIECES; ++i) {
            const int piece = threadIdx.x + 128 * i;
            const int r = piece / (TC_K / 8), kp = piece % (TC_K / 8);
            const int p = src_pair[r];
            breg[i] = p >= 0 ? *reinterpret_cast<const uint4*>(a + (size_t)(p / a_div) * K + k0 + 8 * kp) : make_uint4(0, 0, 0, 0);
        }
    };
    auto store = [&]() {
#pragma unroll
        for (int i = 0; i < W_PIECES; ++i) {
            const int piece = threadIdx.x + 128 * i;
            const int which = piece / (TC_COLS * (TC_K / 8)), rest = piece % (TC_COLS * (TC_K / 8));
            *reinterpret_cast<uint4*>(&Ws[which][rest / (TC_K / 8)][8 * (rest % (TC_K / 8))]) = wreg[i];
        }
#pragma unroll
        for (int i = 0; i < B_PIECES; ++i) {
            const int piece = threadIdx.x + 128 * i;
            *reinterpret_cast<uint4*>(&Bs[piece / (TC_K / 8)][8 * (piece % (TC_K / 8))]) = breg[i];
        }
    };
    float acc[NW][4][4] = {};
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += TC_K) {
        store();
        __syncthreads();
        if (k0 + TC_K < K) fetch(k0 + TC_K);
#pragma unroll
        for (int ks = 0; ks < TC_K; ks += 16) {
            uint32_t bf[4][2];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                bf[t][0] = *reinterpret_cast<const uint32_t*>(&Bs[8 * t + gid][ks + 2 * tig]);
                bf[t][1] = *reinterpret_cast<const uint32_t*>(&Bs[8 * t + gid][ks + 8 + 2 * tig]);
            }
#pragma unroll
            for (int which = 0; which < NW; ++which) {
                uint32_t af[4];
                af[0] = *reinterpret_cast<const uint32_t*>(&Ws[which][16 * warp + gid][ks + 2 * tig]);
                af[1] = *reinterpret_cast<const uint32_t*>(&Ws[which][16 * warp + gid + 8][ks + 2 * tig]);
                af[2] = *reinterpret_cast<const uint32_t*>(&Ws[which][16 * warp + gid][ks + 8 + 2 * tig]);
                af[3] = *reinterpret_cast<const uint32_t*>(&Ws[which][16 * warp + gid + 8][ks + 8 + 2 * tig]);
#pragma unroll
                for (int t = 0; t < 4; ++t) mma_bf16(acc[which][t], af, bf[t]);
            }
        }
        __syncthreads();
    }
    // d[0], d[1]: output column 16 w + gid, pairs 8 t + 2 tig, + 1;  d[2], d[3]: output column 16 w + gid + 8.
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int p = src_pair[8 * t + 2 * tig + (i & 1)];
            const int c = col0 + 16 * warp + gid + (i >> 1) * 8;
            if (p < 0 || c >= N) continue;
            float v = acc[0][t][i];
            if (GATED) v = v / (1.0f + expf(-v)) * acc[NW - 1][t][i];
            out[(size_t)p * N + c] = from_float<OutT>(v);
        }
}

__global__ void combine_kernel(const float* __restrict__ y, float* __restrict__ x, int top, int width, float weight,
                               long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long row = i / width;
    const int c = (int)(i % width);
    float s = 0.0f;
    for (int k = 0; k < top; ++k) s += y[((size_t)row * top + k) * width + c];
    x[i] = fmaf(weight, s, x[i]);
}

inline int max_tiles(int pairs, int experts) { return (pairs + TILE_ROWS - 1) / TILE_ROWS + experts; }
}  // namespace

// token_ids int32 [rows]; table int32 [vocab, top]; lists int32 [experts, rows * top]; counts int32 [experts]; tiles int32
// [2 + 2 * (ceil(rows * top / 32) + experts)].
LLMX_EXPORT int llmx_moe_route(const int* token_ids, const int* table, int top, int rows, int experts, int vocab, int* lists,
                               int* counts, int* tiles, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (top <= 0 || experts <= 0 || experts > 65535) return LLMX_ERR_BAD_ARGUMENT;
    launch_kernel(route_kernel, dim3(experts), dim3(256), 0, stream, token_ids, table, top, rows, experts, vocab, lists, counts);
    int status = launch_status();
    if (status) return status;
    launch_kernel(tiles_kernel, dim3(1), dim3(32), 0, stream, (const int*)counts, experts, tiles);
    return launch_status();
}

// a [rows of `a_div` pairs each, K] and w [experts, (gated ? 2 : 1) * N, K] of `dtype`; out [pairs, N] of `out_dtype`
// (gated: silu(gate) * up; else the plain product, float32).  `tensor_cores`: allowed where the shapes fit.
LLMX_EXPORT int llmx_moe_product(const void* a, int a_div, const void* w, int dtype, const int* lists, const int* counts,
                                 const int* tiles, int pairs, int experts, void* out, int out_dtype, int N, int K,
                                 int gated, int tensor_cores, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (N <= 0 || K <= 0 || a_div <= 0) return LLMX_ERR_BAD_ARGUMENT;
    if (!gated && out_dtype != LLMX_F32) return LLMX_ERR_UNSUPPORTED;
    const int tiles_x = max_tiles(pairs, experts);
    if (tensor_cores && dtype == LLMX_BF16 && K % TC_K == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0) {
        dim3 grid(tiles_x, (N + TC_COLS - 1) / TC_COLS);
        if (grid.y > 65535) return LLMX_ERR_UNSUPPORTED;
        const __nv_bfloat16* ab = (const __nv_bfloat16*)a;
        const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
        if (gated && out_dtype == LLMX_BF16)
            launch_kernel(moe_tc_kernel<true, __nv_bfloat16>, dim3(grid), dim3(128), 0, stream, ab, a_div, wb, lists, counts, tiles, pairs, (__nv_bfloat16*)out, N, K);
        else if (gated)
            launch_kernel(moe_tc_kernel<true, float>, dim3(grid), dim3(128), 0, stream, ab, a_div, wb, lists, counts, tiles, pairs, (float*)out, N, K);
        else
            launch_kernel(moe_tc_kernel<false, float>, dim3(grid), dim3(128), 0, stream, ab, a_div, wb, lists, counts, tiles, pairs, (float*)out, N, K);
        return launch_status();
    }
    dim3 grid(tiles_x, (N + CC_COLS - 1) / CC_COLS);
    if (grid.y > 65535) return LLMX_ERR_UNSUPPORTED;
#define LLMX_MOE(T, G, O) \
    launch_kernel(moe_cores_kernel<T, G, O>, dim3(grid), dim3(256), 0, stream, (const T*)a, a_div, (const T*)w, lists, counts, tiles, pairs, (O*)out, N, K)
    if (dtype == LLMX_BF16 && gated && out_dtype == LLMX_BF16) LLMX_MOE(__nv_bfloat16, true, __nv_bfloat16);
    else if (dtype == LLMX_BF16 && gated && out_dtype == LLMX_F32) LLMX_MOE(__nv_bfloat16, true, float);
    else if (dtype == LLMX_BF16 && !gated) LLMX_MOE(__nv_bfloat16, false, float);
    else if (dtype == LLMX_F32 && gated && out_dtype == LLMX_F32) LLMX_MOE(float, true, float);
    else if (dtype == LLMX_F32 && !gated) LLMX_MOE(float, false, float);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_MOE
    return launch_status();
}

// x [rows, width] += weight * sum over k of y [rows * top, width], k in increasing order.
LLMX_EXPORT int llmx_moe_combine(const float* y, float* x, int rows, int top, int width, float weight, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const long long n = (long long)rows * width;
    launch_kernel(combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, y, x, top, width, weight, n);
    return launch_status();
}
