// Linear recurrences over a matrix state per (request, head): decayed linear attention and the gated delta rule.
//
// Per head the state S is [D, V] (key width x value width), 32-bit, one per request in a state slot, and for the
// step's rows t of a request, in order:
//     a_t = decay_h (a constant per head)                  or  g_t (a gate per row and head)
//     u_t = v_t                                            or  beta_t * (v_t - a_t * S^T k_t)      (delta rule)
//     S  <- a_t * S + k_t u_t^T
//     o_t = S^T q_t                                        (the read-out sees the row's own write)
// Two more forms share the code.  The scaled form (a selective state space): a_t a gate per row and head,
// u_t = beta_t * v_t (beta the row's step size), and o_t += skip_h * v_t.  The delta rule with a decay per key
// channel: S <- diag(g_t) S with g_t [D] per row and head, then u_t = beta_t * (v_t - S^T k_t), S <- S + k_t u_t^T.
// Column j of S (the D values that meet v's entry j) never meets another column, so the work is cut by columns:
// a few threads own one column, each holding a share of its values in registers for all of the request's rows;
// the two dot products are sums over a lane's values and then over the column's lanes by shuffles.  A block holds
// columns of one head (and of one request); the rows' q and k are read by every worker from the cache.  The state is
// read from `slot_in` (zeros at a request's first token, whatever the slot holds) and written to `slot_out` once,
// after the request's last row of the step.  State layout in a slot: [H][V][D] floats, so a worker's column is
// contiguous.
//
// The short convolution in front of the delta rule lives here too (`llmx_conv_prepare`): a causal filter of
// `taps` taps per channel over the request's rows, continued from the last taps-1 inputs kept in the state slot,
// then silu; q and k heads made unit vectors (x / sqrt(sum x^2 + 1e-6), q also times D^-1/2); beta = sigmoid(b);
// g = exp(-exp(A_log) * softplus(a + dt_bias)).  All of it 32-bit.  The filter may carry a bias per channel, the unit
// scaling may be left out (no q or k channels named), and the gates come in three kinds (`gate_kind`): 0, the delta
// rule's (g per head, then beta = sigmoid); 1, a selective state space's (dt = softplus(a + dt_bias) with no clamp,
// then g = exp(-exp(A_log) dt) and dt itself per head); 2, the delta rule's with a decay per key channel
// (beta = sigmoid per head, and g [heads * D] from a second matrix `decay_in` [rows, heads * D] with dt_bias
// [heads * D]).
#include "common.cuh"
#include <math.h>

namespace {
constexpr int REC_THREADS = 128;
// What a row does to the state: a constant decay per head; the delta rule with one gate per row and head; a gate per
// row and head with the input scaled by beta and a skip term; the delta rule with a gate per row, head and key channel.
constexpr int M_CONST = 0, M_DELTA = 1, M_SCALED = 2, M_DELTA_VEC = 3;

// The form for steps of a row or a few: LANES (8) threads share one column of the state, each holding PER of its D
// values (D <= LANES * PER), so a sum over the lanes is three shuffle steps; a block of 128 threads owns 16 columns of
// one head.  A row's q, k, v and gates are fetched one row ahead.
template <int PER, int LANES, int MODE>
__global__ void __launch_bounds__(REC_THREADS)
recurrence_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int q_stride,
                  int k_stride, int v_stride, const float* __restrict__ decay, const float* __restrict__ gate,
                  const float* __restrict__ beta, int gate_stride, int beta_stride, const float* __restrict__ skip,
                  float* __restrict__ state, long long slot_floats,
                  const int* __restrict__ row_start, const int* __restrict__ row_count, const int* __restrict__ history,
                  const int* __restrict__ slot_in, const int* __restrict__ slot_out, float* __restrict__ out, int heads,
                  int qk_heads, int D, int V) {
    pdl_trigger();
    pdl_wait();
    constexpr int COLS = REC_THREADS / LANES;
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
    constexpr bool VEC = MODE == M_DELTA_VEC;
    constexpr int GP = VEC ? PER : 1;
    const float dec = MODE == M_CONST ? decay[h] : VEC ? 1.0f : 0.0f;
    const float sk = MODE == M_SCALED && skip != nullptr ? skip[h] : 0.0f;
    float kk[PER], qq[PER], nk[PER], nq[PER], gg[GP], ng[GP];
    float u = 0.0f, a = dec, bt = 0.0f, nu = 0.0f, na = dec, nb = 0.0f;
    auto fetch = [&](int t, float* fk, float* fq, float* fg, float& fu, float& fa, float& fb) {
        const size_t row = (size_t)(a0 + t);
        const float* qp = q + row * q_stride + (size_t)hq * D;
        const float* kp = k + row * k_stride + (size_t)hq * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + i * LANES;
            fk[i] = d < D ? kp[d] : 0.0f;
            fq[i] = d < D ? qp[d] : 0.0f;
        }
        fu = v[row * v_stride + (size_t)h * V + j];
        if (MODE == M_DELTA || MODE == M_SCALED) fa = gate[row * gate_stride + h];
        if (MODE != M_CONST) fb = beta[row * beta_stride + h];
        if (VEC) {
            const float* gp = gate + row * gate_stride + (size_t)h * D;
#pragma unroll
            for (int i = 0; i < GP; ++i) {
                const int d = lane + i * LANES;
                fg[i] = d < D ? gp[d] : 1.0f;
            }
        }
    };
    fetch(0, kk, qq, gg, u, a, bt);
    for (int t = 0; t < n; ++t) {
        if (t + 1 < n) fetch(t + 1, nk, nq, ng, nu, na, nb);
        const float raw = u;
        if (VEC) {
#pragma unroll
            for (int i = 0; i < PER; ++i) S[i] *= gg[i < GP ? i : 0];
        }
        if (MODE == M_DELTA || VEC) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < PER; ++i) dot = fmaf(S[i], kk[i], dot);
#pragma unroll
            for (int o = LANES / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            u = bt * (u - a * dot);
        }
        if (MODE == M_SCALED) u = bt * u;
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            S[i] = fmaf(a, S[i], kk[i] * u);
            acc = fmaf(S[i], qq[i], acc);
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (MODE == M_SCALED) acc = fmaf(sk, raw, acc);
        if (live && lane == 0) out[(size_t)(a0 + t) * ((size_t)heads * V) + (size_t)h * V + j] = acc;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            kk[i] = nk[i];
            qq[i] = nq[i];
        }
#pragma unroll
        for (int i = 0; i < GP; ++i) gg[i] = ng[i];
        u = nu;
        a = (MODE == M_DELTA || MODE == M_SCALED) ? na : dec;
        bt = nb;
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

// The wide form for long runs of rows: a warp a column, eight columns of one head a block, and the rows' q, k, v and
// gates brought to shared memory sixteen rows at a time by cp.async (the next sixteen in flight meanwhile), so that
// a row waits for shared memory and for the row before it, not for the L2 cache.
constexpr int WIDE_THREADS = 256, WIDE_COLS = 8, WIDE_CH = 16;

__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

__device__ __forceinline__ void cp_async_16f(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// A lane holds the PER neighbouring values d = PER * lane .. of its column, so that a row's q and k are one
// 16-byte read each from shared memory when PER is 4.
template <int PER>
__device__ __forceinline__ void read_run(const float* p, int lane, int D, float (&out)[PER]) {
    if (PER == 4 && D % 4 == 0) {
        const float4 x = lane * 4 < D ? *reinterpret_cast<const float4*>(p + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        out[0] = x.x;
        out[1] = x.y;
        out[2] = x.z;
        out[3] = x.w;
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) out[i] = lane * PER + i < D ? p[lane * PER + i] : 0.0f;
    }
}

template <int PER, int MODE>
__global__ void __launch_bounds__(WIDE_THREADS)
recurrence_wide_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int q_stride,
                       int k_stride, int v_stride, const float* __restrict__ decay, const float* __restrict__ gate,
                       const float* __restrict__ beta, int gate_stride, int beta_stride, const float* __restrict__ skip,
                       float* __restrict__ state, long long slot_floats,
                       const int* __restrict__ row_start, const int* __restrict__ row_count,
                       const int* __restrict__ history, const int* __restrict__ slot_in,
                       const int* __restrict__ slot_out, float* __restrict__ out, int heads, int qk_heads, int D, int V) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float stage[];   // [2][WIDE_CH][row_floats]: q (Dp), k (Dp), [gates per channel (Dp)], v (8 columns), gate, beta, pad
    constexpr bool VEC = MODE == M_DELTA_VEC;
    constexpr int NV = VEC ? 3 : 2;                  // vectors of D values a row brings
    const int Dp = PER * 32;                         // a row's q and k padded to the lanes' runs (the pad is never written: zeros are read by the guard)
    const int row_floats = NV * Dp + WIDE_COLS + 4;  // a multiple of 4: every row starts on 16 bytes
    const int r = blockIdx.x;
    const int blocks_per_head = (V + WIDE_COLS - 1) / WIDE_COLS;
    const int h = blockIdx.y / blocks_per_head;
    const int first_col = (blockIdx.y % blocks_per_head) * WIDE_COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = first_col + warp;
    const int n = row_count[r];
    if (n <= 0) return;
    const bool live = col < V;
    const int j = live ? col : V - 1;
    const int a0 = row_start[r];
    const int hq = h / (heads / qk_heads);
    float S[PER];
    const float* sin_ = state + (size_t)slot_in[r] * slot_floats + ((size_t)h * V + j) * D;
    const bool fresh = history[r] == 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int d = lane * PER + i;
        S[i] = (!fresh && d < D) ? sin_[d] : 0.0f;
    }
    const float dec = MODE == M_CONST ? decay[h] : VEC ? 1.0f : 0.0f;
    const float sk = MODE == M_SCALED && skip != nullptr ? skip[h] : 0.0f;
    // What this thread copies of every chunk is the same from chunk to chunk, so its places are worked out once:
    // pieces of 16 bytes of q and k when rows allow it (else single values), and one of the chunk's small values.
    const bool vec = D % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k & 15) == 0 &&
                     (!VEC || (gate_stride % 4 == 0 && ((uintptr_t)gate & 15) == 0));
    const int unit = vec ? 4 : 1;
    const int per_vec = D / unit;
    const int per_row = NV * per_vec;                // copies a row's q and k (and channel gates) take
    constexpr int MAX_COPIES = NV * PER * 32 * WIDE_CH / WIDE_THREADS;     // at most, with single values
    const int small_t = threadIdx.x / (WIDE_COLS + 2), small_e = threadIdx.x % (WIDE_COLS + 2);
    auto issue = [&](int chunk, int which) {
        float* buf = stage + (size_t)which * WIDE_CH * row_floats;
        const int t0 = chunk * WIDE_CH, rows = min(WIDE_CH, n - t0);
        const int copies = rows * per_row;
        int p = threadIdx.x, t = p / per_row, e = p % per_row;
        const int dt = WIDE_THREADS / per_row, de = WIDE_THREADS % per_row;
#pragma unroll 4
        for (int i = 0; i < MAX_COPIES; ++i) {
            if (p >= copies) break;
            const size_t row = (size_t)(a0 + t0 + t);
            const int which_vec = e / per_vec;       // 0: q, 1: k, 2: the gates per channel
            const int off = (e - which_vec * per_vec) * unit;
            const float* src = which_vec == 0 ? q + row * q_stride + (size_t)hq * D + off
                             : which_vec == 1 ? k + row * k_stride + (size_t)hq * D + off
                                              : gate + row * gate_stride + (size_t)h * D + off;
            float* dst = buf + (size_t)t * row_floats + which_vec * Dp + off;
            if (vec) cp_async_16f(dst, src);
            else cp_async_4(dst, src);
            p += WIDE_THREADS;
            t += dt;
            e += de;
            if (e >= per_row) {
                e -= per_row;
                ++t;
            }
        }
        if (small_t < rows && (small_e < WIDE_COLS || (small_e == WIDE_COLS ? (MODE == M_DELTA || MODE == M_SCALED) : MODE != M_CONST))) {
            const size_t row = (size_t)(a0 + t0 + small_t);
            const float* src = small_e < WIDE_COLS ? v + row * v_stride + (size_t)h * V + min(first_col + small_e, V - 1)
                             : small_e == WIDE_COLS ? gate + row * gate_stride + h : beta + row * beta_stride + h;
            cp_async_4(buf + (size_t)small_t * row_floats + NV * Dp + small_e, src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int chunks = (n + WIDE_CH - 1) / WIDE_CH;
    issue(0, 0);
    for (int c = 0; c < chunks; ++c) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                             // chunk c has landed; everyone has left the other buffer
        if (c + 1 < chunks) issue(c + 1, (c + 1) & 1);
        const float* buf = stage + (size_t)(c & 1) * WIDE_CH * row_floats;
        const int rows = min(WIDE_CH, n - c * WIDE_CH);
        for (int t = 0; t < rows; ++t) {
            const float* rowp = buf + (size_t)t * row_floats;
            float kk[PER], qq[PER];
            read_run<PER>(rowp, lane, D, qq);
            read_run<PER>(rowp + Dp, lane, D, kk);
            float u = rowp[NV * Dp + warp];
            const float raw = u;
            float a = dec;
            if (VEC) {
                float gg[PER];
                read_run<PER>(rowp + 2 * Dp, lane, D, gg);
#pragma unroll
                for (int i = 0; i < PER; ++i) S[i] *= gg[i];     // past D: S stays zero whatever the pad holds... the guard reads zeros there
            }
            if (MODE == M_DELTA || MODE == M_SCALED) a = rowp[NV * Dp + WIDE_COLS];
            if (MODE == M_DELTA || VEC) {
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < PER; ++i) dot = fmaf(S[i], kk[i], dot);
                dot = warp_sum(dot);
                u = rowp[NV * Dp + WIDE_COLS + 1] * (u - a * dot);
            }
            if (MODE == M_SCALED) u = rowp[NV * Dp + WIDE_COLS + 1] * u;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                S[i] = fmaf(a, S[i], kk[i] * u);
                acc = fmaf(S[i], qq[i], acc);
            }
            acc = warp_sum(acc);
            if (MODE == M_SCALED) acc = fmaf(sk, raw, acc);
            if (live && lane == 0) out[(size_t)(a0 + c * WIDE_CH + t) * ((size_t)heads * V) + (size_t)h * V + j] = acc;
        }
    }
    if (live) {
        float* sout = state + (size_t)slot_out[r] * slot_floats + ((size_t)h * V + j) * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane * PER + i;
            if (d < D) sout[d] = S[i];
        }
    }
}

// One block per row (conv, activation, unit vectors, gates) and, after those, one block per request (the inputs the
// next step's convolution will need).
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

__global__ void __launch_bounds__(256)
conv_prepare_kernel(const float* __restrict__ proj, int stride, int first, int channels, int q_channels, int k_channels,
                    const float* __restrict__ taps_w, const float* __restrict__ taps_b, int taps,
                    float* __restrict__ ready, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                    int b_off, int a_off, int gate_kind, const float* __restrict__ decay_in, int decay_stride,
                    float* __restrict__ gates, int gates_stride, int heads, int D, float q_factor,
                    float* __restrict__ state, long long slot_floats, long long conv_off,
                    const int* __restrict__ row_request, const int* __restrict__ row_start,
                    const int* __restrict__ row_count, const int* __restrict__ history, const int* __restrict__ slot_in,
                    const int* __restrict__ slot_out, int rows) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float vals[];                  // the row's channels after the filter and silu
    const int keep = taps - 1;
    proj += first;                                   // the filtered channels start at column `first` of the projections
    if ((int)blockIdx.x >= rows) {
        const int r = blockIdx.x - rows;
        const int n = row_count[r], a0 = row_start[r], hist = history[r];
        if (n <= 0) return;
        const float* old = state + (size_t)slot_in[r] * slot_floats + conv_off;
        float* fresh = state + (size_t)slot_out[r] * slot_floats + conv_off;
        for (int c = threadIdx.x; c < channels; c += blockDim.x)
            for (int s = 0; s < keep; ++s) {         // slot_in and slot_out differ: the rows' blocks read the old inputs meanwhile
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
        float y = taps_b ? taps_b[c] : 0.0f;
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
    proj -= first;
    float* grow = gates + (size_t)row * gates_stride;
    if (gate_kind == 2) {
        for (int h = threadIdx.x; h < heads; h += blockDim.x)
            grow[h] = 1.0f / (1.0f + expf(-proj[(size_t)row * stride + b_off + h]));
        for (int c = threadIdx.x; c < heads * D; c += blockDim.x) {
            const float z = decay_in[(size_t)row * decay_stride + c] + dt_bias[c];
            grow[heads + c] = expf(-expf(a_log[c / D]) * softplus_f(z));
        }
        return;
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float z = proj[(size_t)row * stride + a_off + h] + dt_bias[h];
        if (gate_kind == 1) {
            const float dt = z > 20.0f ? z : log1pf(expf(z));      // the same function beyond 20 up to rounding: no clamp of dt itself
            grow[h] = expf(-expf(a_log[h]) * dt);
            grow[heads + h] = dt;
        } else {
            const float b = proj[(size_t)row * stride + b_off + h];
            grow[h] = expf(-expf(a_log[h]) * softplus_f(z));
            grow[heads + h] = 1.0f / (1.0f + expf(-b));
        }
    }
}

template <int MODE>
int launch_recurrence(int D, bool wide, int requests, cudaStream_t stream, const float* q, const float* k, const float* v,
                      int q_stride, int k_stride, int v_stride, const float* decay, const float* gate, const float* beta,
                      int gate_stride, int beta_stride, const float* skip, float* state, long long slot_floats, const int* row_start, const int* row_count,
                      const int* history, const int* slot_in, const int* slot_out, float* out, int heads, int qk_heads,
                      int V) {
#define LLMX_REC(P, L)                                                                                                    \
    do {                                                                                                                  \
        const long long by = (long long)heads * ((V + REC_THREADS / L - 1) / (REC_THREADS / L));                          \
        if (by > 65535) return LLMX_ERR_UNSUPPORTED;                                                                      \
        launch_kernel(recurrence_kernel<P, L, MODE>, dim3(requests, (unsigned)by), dim3(REC_THREADS), 0, stream, q, k, v,  \
                      q_stride, k_stride, v_stride, decay, gate, beta, gate_stride, beta_stride, skip, state,          \
                      slot_floats, row_start, row_count, history, slot_in, slot_out, out, heads, qk_heads, D, V);       \
        return launch_status();                                                                                           \
    } while (0)
    if (wide) {
#define LLMX_WIDE(P)                                                                                                      \
    do {                                                                                                                  \
        const long long by = (long long)heads * ((V + WIDE_COLS - 1) / WIDE_COLS);                                        \
        if (by > 65535) return LLMX_ERR_UNSUPPORTED;                                                                      \
        const size_t smem = (size_t)2 * WIDE_CH * ((MODE == M_DELTA_VEC ? 3 : 2) * P * 32 + WIDE_COLS + 4) * sizeof(float);   \
        if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;                                                               \
        if (smem > 48 * 1024)                                                                                             \
            cudaFuncSetAttribute(recurrence_wide_kernel<P, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(recurrence_wide_kernel<P, MODE>, dim3(requests, (unsigned)by), dim3(WIDE_THREADS), smem, stream, q, \
                      k, v, q_stride, k_stride, v_stride, decay, gate, beta, gate_stride, beta_stride, skip, state,      \
                      slot_floats, row_start, row_count, history, slot_in, slot_out, out, heads, qk_heads, D, V);       \
        return launch_status();                                                                                           \
    } while (0)
        if (D <= 32) LLMX_WIDE(1);
        if (D <= 64) LLMX_WIDE(2);
        if (D <= 128) LLMX_WIDE(4);
        if (D <= 256) LLMX_WIDE(8);
        if (D <= 512) LLMX_WIDE(16);
#undef LLMX_WIDE
    } else {
        if (D <= 16) LLMX_REC(2, 8);
        if (D <= 32) LLMX_REC(4, 8);
        if (D <= 64) LLMX_REC(8, 8);
        if (D <= 128) LLMX_REC(16, 8);
        if (D <= 256) LLMX_REC(32, 8);
        if (D <= 512) LLMX_REC(16, 32);          // a warp a column: 64 values a lane would not stay in registers
    }
#undef LLMX_REC
    return LLMX_ERR_UNSUPPORTED;
}
}  // namespace

// q, k [rows, qk_heads * D] and v [rows, heads * V] floats with row strides of their own (they may lie inside one wider
// matrix).  `mode` 0: a constant `decay` [heads].  1: the delta rule, `gate` and `beta` [rows, .] (row strides
// `gate_stride`, `beta_stride`, entry h).  2: the scaled form, a = gate, u = beta * v, out += skip_h * v (`skip` [heads]
// or null).  3: the delta rule with `gate` [rows, heads * D] (entry h * D + d), a decay per key channel.  `state`: the
// slots' storage, `slot_floats` apart, the recurrence's [H][V][D] at its start; out [rows, heads * V] floats.  The
// metadata arrays are the step's, on the device.
LLMX_EXPORT int llmx_linear_recurrence(const float* q, const float* k, const float* v, int q_stride, int k_stride,
                                       int v_stride, int mode, const float* decay, const float* gate, const float* beta,
                                       int gate_stride, int beta_stride, const float* skip, float* state,
                                       long long slot_floats, const int* row_start, const int* row_count,
                                       const int* history, const int* slot_in, const int* slot_out, float* out,
                                       int requests, int heads, int qk_heads, int D, int V, int max_rows,
                                       cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (heads <= 0 || qk_heads <= 0 || heads % qk_heads || D <= 0 || V <= 0 || D > 512) return LLMX_ERR_UNSUPPORTED;
    if (mode < 0 || mode > 3 || (mode == M_CONST ? decay == nullptr : (gate == nullptr || beta == nullptr))) return LLMX_ERR_BAD_ARGUMENT;
    const bool wide = max_rows > 8;            // `max_rows`: the most rows one request brings (a matter of speed only)
#define LLMX_MODE(M)                                                                                                      \
    return launch_recurrence<M>(D, wide, requests, stream, q, k, v, q_stride, k_stride, v_stride, decay, gate, beta,      \
                                gate_stride, beta_stride, skip, state, slot_floats, row_start, row_count, history, slot_in, \
                                slot_out, out, heads, qk_heads, V)
    if (mode == M_CONST) LLMX_MODE(M_CONST);
    if (mode == M_DELTA) LLMX_MODE(M_DELTA);
    if (mode == M_SCALED) LLMX_MODE(M_SCALED);
    LLMX_MODE(M_DELTA_VEC);
#undef LLMX_MODE
}

// proj [rows, stride]: columns first .. first + channels - 1 are filtered: q (q_channels), k (k_channels), each of whole
// heads of D values that are made unit vectors, and the rest; columns b_off + h and a_off + h hold the rows' beta and
// decay (or step size) projections.  ready [rows, channels] receives the channels after filter (+ `taps_b` if given),
// silu and unit scaling.  gates [rows, gates_stride]: kind 0: g [heads], beta [heads]; kind 1: g [heads], dt [heads];
// kind 2: beta [heads], g [heads * D] made from `decay_in` [rows, heads * D] (row stride `decay_stride`).
// taps_w [channels, taps].  The last taps-1 inputs of a request lie at `conv_off` floats into its state slot,
// [taps - 1][channels].
LLMX_EXPORT int llmx_conv_prepare(const float* proj, int stride, int first, int channels, int q_channels, int k_channels,
                                  const float* taps_w, const float* taps_b, int taps, float* ready, const float* a_log,
                                  const float* dt_bias, int b_off, int a_off, int gate_kind, const float* decay_in,
                                  int decay_stride, float* gates, int gates_stride, int heads, int D, float q_factor,
                                  float* state, long long slot_floats, long long conv_off, const int* row_request,
                                  const int* row_start, const int* row_count, const int* history, const int* slot_in,
                                  const int* slot_out, int rows, int requests, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (taps < 1 || channels <= 0 || D <= 0 || q_channels % D || k_channels % D || q_channels + k_channels > channels ||
        gate_kind < 0 || gate_kind > 2 || (gate_kind == 2 && decay_in == nullptr))
        return LLMX_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)channels * sizeof(float);
    if (smem > 200 * 1024) return LLMX_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) cudaFuncSetAttribute(conv_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(conv_prepare_kernel, dim3(rows + requests), dim3(256), smem, stream, proj, stride, first, channels,
                  q_channels, k_channels, taps_w, taps_b, taps, ready, a_log, dt_bias, b_off, a_off, gate_kind, decay_in,
                  decay_stride, gates, gates_stride, heads, D, q_factor, state, slot_floats, conv_off, row_request,
                  row_start, row_count, history, slot_in, slot_out, rows);
    return launch_status();
}
