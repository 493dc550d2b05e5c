// Linear recurrences over a matrix state per (request, head): decayed linear attention and the gated delta rule.
//
// Per head the state S is [D, V] (key width x value width), 32-bit, one per request in a state slot, and for the
// step's rows t of a request, in order:
//     a_t = decay_h (a constant per head)                  or  g_t (a gate per row and head)
//     u_t = v_t                                            or  beta_t * (v_t - a_t * S^T k_t)      (delta rule)
//     S  <- a_t * S + k_t u_t^T
//     o_t = S^T q_t                                        (the read-out sees the row's own write)
// Column j of S (the D values that meet v's entry j) never meets another column, so the work is cut by columns:
// LANES threads own one column, each holding D / LANES of its values in registers for all of the request's rows;
// the two dot products are sums over a lane's values and then over the LANES lanes by shuffles, in an order that the
// sizes alone fix.  A block holds columns of one head (and of one request); the rows' q and k are read by every
// worker from the cache.  The state is read from `slot_in` (zeros at a request's first token, whatever the slot
// holds) and written to `slot_out` once, after the request's last row of the step: a step of one row and a step of
// a thousand run the same code.  State layout in a slot: [H][V][D] floats, so a worker's column is contiguous.
//
// The short convolution in front of the delta rule lives here too (`llmx_conv_prepare`): a causal filter of
// `taps` taps per channel over the request's rows, continued from the last taps-1 inputs kept in the state slot,
// then silu; q and k heads made unit vectors (x / sqrt(sum x^2 + 1e-6), q also times D^-1/2); beta = sigmoid(b);
// g = exp(-exp(A_log) * softplus(a + dt_bias)).  All of it 32-bit.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int LANES = 8;            // threads that share one column of the state
constexpr int COLS = 16;            // columns a block owns (128 threads)

template <int PER, bool DELTA>
__global__ void __launch_bounds__(LANES * COLS)
recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int q_stride,
                  int k_stride, int v_stride, const float* __restrict__ decay, const float* __restrict__ gate,
                  const float* __restrict__ beta, int gate_stride, float* __restrict__ state, long long slot_floats,
                  const int* __restrict__ row_start, const int* __restrict__ row_count, const int* __restrict__ history,
                  const int* __restrict__ slot_in, const int* __restrict__ slot_out, float* __restrict__ out, int heads,
                  int qk_heads, int D, int V) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int blocks_per_head = (V + COLS - 1) / COLS;
    const int h = blockIdx.y / blocks_per_head;
    const int col = (blockIdx.y % blocks_per_head) * COLS + threadIdx.x / LANES;
    const int lane = threadIdx.x % LANES;
    const int n = row_count[r];
    if (n <= 0) return;
    const bool live = col < V;
    const int j = live ? col : V - 1;                 // idle workers shadow a real column and store nothing
    const int a0 = row_start[r];
    const int hq = h / (heads / qk_heads);
    float S[PER];
    const float* sin_ = state + (size_t)slot_in[r] * slot_floats + ((size_t)h * V + j) * D;
    const bool fresh = history[r] == 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane + i * LANES;
        S[i] = (!fresh && d < D) ? sin_[d] : 0.0f;
    }
    const float dec = DELTA ? 0.0f : decay[h];
    for (int t = 0; t < n; ++t) {
        const size_t row = (size_t)(a0 + t);
        const float* qp = q + row * q_stride + (size_t)hq * D;
        const float* kp = k + row * k_stride + (size_t)hq * D;
        float kk[PER], qq[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + i * LANES;
            kk[i] = d < D ? kp[d] : 0.0f;
            qq[i] = d < D ? qp[d] : 0.0f;
        }
        float u = v[row * v_stride + (size_t)h * V + j];
        float a = dec;
        if (DELTA) {
            a = gate[row * gate_stride + h];
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < PER; ++i) dot = fmaf(S[i], kk[i], dot);
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            u = beta[row * gate_stride + h] * (u - a * dot);
        }
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            S[i] = fmaf(a, S[i], kk[i] * u);
            acc = fmaf(S[i], qq[i], acc);
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (live && lane == 0) out[row * ((size_t)heads * V) + (size_t)h * V + j] = acc;
    }
    if (live) {
        float* sout = state + (size_t)slot_out[r] * slot_floats + ((size_t)h * V + j) * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + i * LANES;
            if (d < D) sout[d] = S[i];
        }
    }
}

// One block per row (conv, activation, unit vectors, gates) and, after those, one block per request (the inputs the
// next step's convolution will need).
__global__ void __launch_bounds__(256)
conv_prepare_kernel(const float* __restrict__ proj, int stride, int channels, int q_channels, int k_channels,
                    const float* __restrict__ taps_w, int taps, float* __restrict__ ready,
                    const float* __restrict__ a_log, const float* __restrict__ dt_bias, int b_off, int a_off,
                    float* __restrict__ gates, int heads, int D, float q_factor, float* __restrict__ state,
                    long long slot_floats, long long conv_off, const int* __restrict__ row_request,
                    const int* __restrict__ row_start, const int* __restrict__ row_count,
                    const int* __restrict__ history, const int* __restrict__ slot_in,
                    const int* __restrict__ slot_out, int rows) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float vals[];                  // the row's channels after the filter and silu
    const int keep = taps - 1;
    if ((int)blockIdx.x >= rows) {
        const int r = blockIdx.x - rows;
        const int n = row_count[r], a0 = row_start[r], hist = history[r];
        if (n <= 0) return;
        const float* old = state + (size_t)slot_in[r] * slot_floats + conv_off;
        float* fresh = state + (size_t)slot_out[r] * slot_floats + conv_off;
        for (int c = threadIdx.x; c < channels; c += blockDim.x)
            for (int s = 0; s < keep; ++s) {         // ascending: in place (slot_in == slot_out) reads run ahead of writes
                const int ii = n - keep + s;         // the input's place relative to the step's first row
                float x = 0.0f;
                if (ii >= 0) x = proj[(size_t)(a0 + ii) * stride + c];
                else if (hist + ii >= 0) x = old[(size_t)(keep + ii) * channels + c];
                fresh[(size_t)s * channels + c] = x;
            }
        return;
    }
    const int row = blockIdx.x;
    const int r = row_request[row];
    const int i0 = row - row_start[r], hist = history[r];
    const float* old = state + (size_t)slot_in[r] * slot_floats + conv_off;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float y = 0.0f;
        for (int jt = 0; jt < taps; ++jt) {
            const int ii = i0 - keep + jt;
            float x = 0.0f;
            if (ii >= 0) x = proj[(size_t)(row_start[r] + ii) * stride + c];
            else if (hist + ii >= 0) x = old[(size_t)(keep + ii) * channels + c];
            y = fmaf(taps_w[(size_t)c * taps + jt], x, y);
        }
        vals[c] = y / (1.0f + expf(-y));
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int unit_heads = (q_channels + k_channels) / D;          // q heads, then k heads
    for (int g = warp; g < unit_heads; g += warps) {
        float s = 0.0f;
        for (int d = lane; d < D; d += 32) s = fmaf(vals[g * D + d], vals[g * D + d], s);
        s = warp_sum(s);
        const float f = (g * D < q_channels ? q_factor : 1.0f) / sqrtf(s + 1e-6f);
        for (int d = lane; d < D; d += 32) ready[(size_t)row * channels + g * D + d] = vals[g * D + d] * f;
    }
    for (int c = q_channels + k_channels + threadIdx.x; c < channels; c += blockDim.x) ready[(size_t)row * channels + c] = vals[c];
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float b = proj[(size_t)row * stride + b_off + h];
        const float z = proj[(size_t)row * stride + a_off + h] + dt_bias[h];
        const float sp = z > 20.0f ? z : log1pf(expf(z));
        gates[(size_t)row * 2 * heads + h] = expf(-expf(a_log[h]) * sp);
        gates[(size_t)row * 2 * heads + heads + h] = 1.0f / (1.0f + expf(-b));
    }
}

template <bool DELTA>
int launch_recurrence(int per, dim3 grid, cudaStream_t stream, const float* q, const float* k, const float* v, int q_stride,
                      int k_stride, int v_stride, const float* decay, const float* gate, const float* beta, int gate_stride,
                      float* state, long long slot_floats, const int* row_start, const int* row_count, const int* history,
                      const int* slot_in, const int* slot_out, float* out, int heads, int qk_heads, int D, int V) {
#define LLMX_REC(P)                                                                                                       \
    launch_kernel(recurrence_kernel<P, DELTA>, grid, dim3(LANES * COLS), 0, stream, q, k, v, q_stride, k_stride, v_stride,  \
                  decay, gate, beta, gate_stride, state, slot_floats, row_start, row_count, history, slot_in, slot_out,  \
                  out, heads, qk_heads, D, V)
    if (per <= 2) LLMX_REC(2);
    else if (per <= 4) LLMX_REC(4);
    else if (per <= 8) LLMX_REC(8);
    else if (per <= 16) LLMX_REC(16);
    else if (per <= 32) LLMX_REC(32);
    else return LLMX_ERR_UNSUPPORTED;
#undef LLMX_REC
    return launch_status();
}
}  // namespace

// q, k [rows, qk_heads * D] and v [rows, heads * V] floats with row strides of their own (they may lie inside one wider
// matrix); `decay` [heads] for the constant-decay form, or `gate`/`beta` [rows, .] (row stride `gate_stride`, entry h)
// for the delta rule; `state` the slots' storage, `slot_floats` apart, the recurrence's [H][V][D] at its start;
// out [rows, heads * V] floats.  The metadata arrays are the step's, on the device.
LLMX_EXPORT int llmx_linear_recurrence(const float* q, const float* k, const float* v, int q_stride, int k_stride,
                                       int v_stride, const float* decay, const float* gate, const float* beta,
                                       int gate_stride, float* state, long long slot_floats, const int* row_start,
                                       const int* row_count, const int* history, const int* slot_in, const int* slot_out,
                                       float* out, int requests, int heads, int qk_heads, int D, int V,
                                       cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || qk_heads <= 0 || heads % qk_heads || D <= 0 || V <= 0 || D > 32 * LANES) return LLMX_ERR_UNSUPPORTED;
    if ((decay == nullptr) == (gate == nullptr) || (gate != nullptr && beta == nullptr)) return LLMX_ERR_BAD_ARGUMENT;
    const long long by = (long long)heads * ((V + COLS - 1) / COLS);
    if (by > 65535) return LLMX_ERR_UNSUPPORTED;
    const dim3 grid(requests, (unsigned)by);
    const int per = (D + LANES - 1) / LANES;
    if (gate)
        return launch_recurrence<true>(per, grid, stream, q, k, v, q_stride, k_stride, v_stride, decay, gate, beta, gate_stride,
                                       state, slot_floats, row_start, row_count, history, slot_in, slot_out, out, heads,
                                       qk_heads, D, V);
    return launch_recurrence<false>(per, grid, stream, q, k, v, q_stride, k_stride, v_stride, decay, gate, beta, gate_stride,
                                    state, slot_floats, row_start, row_count, history, slot_in, slot_out, out, heads, qk_heads,
                                    D, V);
}

// proj [rows, stride]: channels 0 .. channels-1 are q (q_channels), k (k_channels) and v, each of whole heads of
// D (q, k) values; columns b_off + h and a_off + h hold the rows' beta and decay projections.  ready [rows, channels]
// receives q, k, v after filter, silu and unit scaling; gates [rows, 2 * heads]: g then beta.  taps_w [channels, taps].
// The last taps-1 inputs of a request lie at `conv_off` floats into its state slot, [taps - 1][channels].
LLMX_EXPORT int llmx_conv_prepare(const float* proj, int stride, int channels, int q_channels, int k_channels,
                                  const float* taps_w, int taps, float* ready, const float* a_log, const float* dt_bias,
                                  int b_off, int a_off, float* gates, int heads, int D, float q_factor, float* state,
                                  long long slot_floats, long long conv_off, const int* row_request, const int* row_start,
                                  const int* row_count, const int* history, const int* slot_in, const int* slot_out,
                                  int rows, int requests, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (taps < 1 || channels <= 0 || D <= 0 || q_channels % D || k_channels % D || q_channels + k_channels > channels)
        return LLMX_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)channels * sizeof(float);
    if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) cudaFuncSetAttribute(conv_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(conv_prepare_kernel, dim3(rows + requests), dim3(256), smem, stream, proj, stride, channels, q_channels,
                  k_channels, taps_w, taps, ready, a_log, dt_bias, b_off, a_off, gates, heads, D, q_factor, state,
                  slot_floats, conv_off, row_request, row_start, row_count, history, slot_in, slot_out, rows);
    return launch_status();
}
