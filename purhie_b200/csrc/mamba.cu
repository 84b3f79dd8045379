// The two kernels of a selective state-space mixer (Mamba's first form) that are not matrix products: the short
// causal convolution with its activation, and the scan.
//
// Convolution: per channel c and token i of a request, y = silu(bias_c + sum_j taps[c][j] * u[i - (K - 1) + j]) where u
// is the first half of the in-projection's rows [u | z]; inputs before the step's first token come from the request's
// state (the last K - 1 inputs of earlier steps, zero for a new request), so a prompt cut anywhere gives the same sums.
//
// Scan: per channel c and state index n, with dt = softplus(dt_raw + dt_bias_c):
//     S[c][n] <- exp(dt * A[c][n]) * S[c][n] + (dt * x_c) * B_n;      y_c = sum_n S[c][n] * C_n + D_c * x_c
// then y_c * silu(z_c).  S lives in float32 in the request's state slot and is carried from token to token; dt, the
// exponentials, the decays and the sums are float32.  A channel is shared by L lanes that hold N / L states each and
// add their parts with a butterfly, so the order of every sum depends on N alone.  Tokens of a request are walked in
// order by the same lanes; requests and channels are spread over the grid.  When the scan is done it also moves the
// request's convolution inputs on (the last K - 1 of them), which nothing reads any more in this step.
//
// State of one request: [C x N floats of S][(K - 1) x C floats of convolution inputs, oldest first].
#include "common.cuh"

namespace {

using namespace ph;

constexpr int MAX_TAPS = 16;
constexpr int SCAN_THREADS = 128;
constexpr int MAX_PER_LANE = 8;

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
// exp of a decay's exponent (<= 0): the library's function in a float32 model; in a bfloat16 model the hardware's
// base-2 exponential, still float32 arithmetic, relative error about 2^-21
template <typename TD> __device__ __forceinline__ float decay_exp(float v) { return expf(v); }
template <> __device__ __forceinline__ float decay_exp<__nv_bfloat16>(float v) { return __expf(v); }
__device__ __forceinline__ float softplus_f(float v) { return log1pf(expf(-fabsf(v))) + fmaxf(v, 0.0f); }

template <typename TI, typename TO>
__global__ void causal_conv_silu_kernel(const TI* __restrict__ u, long long row_stride, int C, const float* __restrict__ taps,
                                        const float* __restrict__ bias, int K, const float* __restrict__ state,
                                        long long state_stride, long long conv_offset, const int32_t* __restrict__ row_seg,
                                        const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_slot,
                                        TO* __restrict__ out, int T) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)T * C) return;
    const int t = (int)(idx / C), c = (int)(idx % C);
    const int s = row_seg[t], first = seg_start[s];
    const int i = t - first;                                   // index within the step's portion of the request
    const float* past = state + (size_t)seg_slot[s] * state_stride + conv_offset;
    float acc = bias ? bias[c] : 0.0f;
    for (int j = 0; j < K; ++j) {
        const int src = i - (K - 1) + j;
        const float v = src >= 0 ? to_float<TI>(u[(size_t)(first + src) * row_stride + c]) : past[(size_t)(src + K - 1) * C + c];
        acc = fmaf(taps[(size_t)c * K + j], v, acc);
    }
    out[(size_t)t * C + c] = from_float<TO>(silu_f(acc));
}

// The same for eight consecutive channels per thread (C a multiple of 8, 16-byte aligned rows) and KT taps known at
// compile time: one 16-byte load per tap of the model's dtype, the thread's 8 x KT taps fetched as one contiguous run.
template <typename TI, typename TO, int KT>
__global__ void causal_conv_silu_vec_kernel(const TI* __restrict__ u, long long row_stride, int C, const float* __restrict__ taps,
                                            const float* __restrict__ bias, const float* __restrict__ state,
                                            long long state_stride, long long conv_offset, const int32_t* __restrict__ row_seg,
                                            const int32_t* __restrict__ seg_start, const int32_t* __restrict__ seg_slot,
                                            TO* __restrict__ out, int T) {
    pdl_launch_dependents();
    const int per_row = C / 8;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool on = idx < (long long)T * per_row;
    const int t = on ? (int)(idx / per_row) : 0, c0 = on ? (int)(idx % per_row) * 8 : 0;
    float tp[8 * KT], acc[8];
#pragma unroll
    for (int q = 0; q < 2 * KT; ++q) {                      // weights: not written by any kernel of the step
        const float4 w4 = *reinterpret_cast<const float4*>(taps + (size_t)c0 * KT + 4 * q);
        tp[4 * q] = w4.x; tp[4 * q + 1] = w4.y; tp[4 * q + 2] = w4.z; tp[4 * q + 3] = w4.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias ? bias[c0 + e] : 0.0f;
    pdl_wait();
    if (!on) return;
    const int s = row_seg[t], first = seg_start[s];
    const int i = t - first;
    const float* past = state + (size_t)seg_slot[s] * state_stride + conv_offset;
#pragma unroll
    for (int j = 0; j < KT; ++j) {
        const int src = i - (KT - 1) + j;
        float v[8];
        if (src >= 0) load8(u + (size_t)(first + src) * row_stride + c0, v);
        else load8(past + (size_t)(src + KT - 1) * C + c0, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(tp[e * KT + j], v[e], acc[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = silu_f(acc[e]);
    store8(out + (size_t)t * C + c0, acc);
}

// MODE 0: a request's rows in one go: S from the state slot, y out, S back into the slot.
// MODE 1: one chunk of a request's rows from S = 0: the chunk's own contribution P and its sum of dt (the decay over the
//         whole chunk is exp(A * sum)), no y.
// MODE 2: one chunk from the S it starts with (carry[chunk], which scan_carry made from the state slot, P and the
//         sums), y out; nothing goes back into the slot but, after a request's last chunk, the convolution's inputs.
// A long prompt is cut into chunks so that its tokens are spread over the grid: the recurrence is run twice per
// chunk (modes 1 and 2) with one short pass over the chunks between (scan_carry).  items: (first row, rows, request's
// segment, 1 if the request's last chunk) per block row.
template <typename TX, typename TL, typename TZ, typename TO, int MODE>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                      const TL* __restrict__ low, long long low_stride, int b_col, int c_col, int N, const float* __restrict__ A,
                      const float* __restrict__ D, const TZ* __restrict__ uz, long long uz_stride, int C, int K,
                      float* __restrict__ state, long long state_stride, const int32_t* __restrict__ seg_start,
                      const int32_t* __restrict__ seg_slot, const int32_t* __restrict__ items, float* __restrict__ carry,
                      float* __restrict__ dt_sum, TO* __restrict__ out, int L, int P) {
    pdl_launch_dependents();
    pdl_wait();
    const int item = blockIdx.y;
    const int seg = items ? items[4 * item + 2] : item;
    const int first = items ? items[4 * item] : seg_start[seg];
    const int rows = items ? items[4 * item + 1] : seg_start[seg + 1] - first;
    const bool last = items ? items[4 * item + 3] != 0 : true;
    const int group = threadIdx.x / L, lane = threadIdx.x % L;
    const int c = blockIdx.x * (SCAN_THREADS / L) + group;
    const bool live = c < C;                                   // dead lanes still take part in the shuffles
    const int cc = live ? c : C - 1;
    float* st = state + (size_t)seg_slot[seg] * state_stride;
    const float* init = MODE == 0 ? st : MODE == 2 ? carry + (size_t)item * C * N : nullptr;
    float S[MAX_PER_LANE], a[MAX_PER_LANE];
#pragma unroll
    for (int p = 0; p < MAX_PER_LANE; ++p) {
        const int n = lane + L * p;
        const bool on = p < P && n < N;
        S[p] = (on && init) ? init[(size_t)cc * N + n] : 0.0f;
        a[p] = on ? A[(size_t)cc * N + n] : 0.0f;
    }
    const float bias = dt_bias ? dt_bias[cc] : 0.0f, d_skip = D ? D[cc] : 0.0f;
    float sum = 0.0f;
    for (int i = 0; i < rows; ++i) {
        const int t = first + i;
        const float dt = softplus_f(dt_raw[(size_t)t * C + cc] + bias);
        const float xv = to_float<TX>(x[(size_t)t * C + cc]);
        const float dx = dt * xv;
        const TL* lr = low + (size_t)t * low_stride;
        float acc = 0.0f;
        sum += dt;
#pragma unroll
        for (int p = 0; p < MAX_PER_LANE; ++p) {
            const int n = lane + L * p;
            if (p < P && n < N) {
                S[p] = expf(dt * a[p]) * S[p] + dx * to_float<TL>(lr[b_col + n]);
                if (MODE != 1) acc += S[p] * to_float<TL>(lr[c_col + n]);
            }
        }
        if (MODE != 1) {
            for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && lane == 0) {
                const float z = to_float<TZ>(uz[(size_t)t * uz_stride + C + c]);
                out[(size_t)t * C + c] = from_float<TO>((acc + d_skip * xv) * silu_f(z));
            }
        }
    }
    if (!live) return;
    if (MODE != 2) {
        float* dst = MODE == 0 ? st : carry + (size_t)item * C * N;
#pragma unroll
        for (int p = 0; p < MAX_PER_LANE; ++p) {
            const int n = lane + L * p;
            if (p < P && n < N) dst[(size_t)c * N + n] = S[p];
        }
        if (MODE == 1 && lane == 0) dt_sum[(size_t)item * C + c] = sum;
    }
    if (MODE != 1 && last && lane == 0 && K > 1) {
        // the last K - 1 convolution inputs, oldest first: from this step's rows, or moved up from what was kept
        const int seg_first = seg_start[seg], seg_rows = first + rows - seg_first;
        float* past = st + (size_t)C * N;
        for (int k = 0; k < K - 1; ++k) {
            const int src = seg_rows - (K - 1) + k;
            past[(size_t)k * C + c] = src >= 0 ? to_float<TZ>(uz[(size_t)(seg_first + src) * uz_stride + c]) : past[(size_t)(k + seg_rows) * C + c];
        }
    }
}

// Modes 1 and 2 again for the usual state sizes (NS = 8 or 16 states per channel, B and C 16-byte aligned in the low
// rows): a thread per channel holds all of the channel's states, so the step size, its softplus and the gate are
// computed once per token and channel, B and C arrive as 16-byte loads that the whole warp shares, and the next token's
// inputs are asked for before the current one's arithmetic.  y's sum over the states runs n = 0, 1, ... in the thread.
template <typename TD, int MODE, int NS>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_chunk_kernel(const TD* __restrict__ x, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                  const TD* __restrict__ low, long long low_stride, int b_col, int c_col, const float* __restrict__ A,
                  const float* __restrict__ D, const TD* __restrict__ uz, long long uz_stride, int C, int K,
                  float* __restrict__ state, long long state_stride, const int32_t* __restrict__ seg_start,
                  const int32_t* __restrict__ seg_slot, const int32_t* __restrict__ items, float* __restrict__ carry,
                  float* __restrict__ dt_sum, TD* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
    if (c >= C) return;
    const int item = blockIdx.y;
    const int first = items[4 * item], rows = items[4 * item + 1], seg = items[4 * item + 2];
    const bool last = items[4 * item + 3] != 0;
    float S[NS], a[NS];
    float* mine = carry + ((size_t)item * C + c) * NS;
#pragma unroll
    for (int q = 0; q < NS / 4; ++q) {
        const float4 av = *reinterpret_cast<const float4*>(A + (size_t)c * NS + 4 * q);
        a[4 * q] = av.x; a[4 * q + 1] = av.y; a[4 * q + 2] = av.z; a[4 * q + 3] = av.w;
        float4 sv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (MODE == 2) sv = *reinterpret_cast<const float4*>(mine + 4 * q);
        S[4 * q] = sv.x; S[4 * q + 1] = sv.y; S[4 * q + 2] = sv.z; S[4 * q + 3] = sv.w;
    }
    const float bias = dt_bias ? dt_bias[c] : 0.0f, d_skip = D ? D[c] : 0.0f;
    float sum = 0.0f;
    float dtr = dt_raw[(size_t)first * C + c];
    TD xr = x[(size_t)first * C + c], zr = MODE == 2 ? uz[(size_t)first * uz_stride + C + c] : TD();
    for (int i = 0; i < rows; ++i) {
        const int t = first + i;
        const float dt = softplus_f(dtr + bias);
        const float xv = to_float<TD>(xr), zv = to_float<TD>(zr);
        if (i + 1 < rows) {
            dtr = dt_raw[(size_t)(t + 1) * C + c];
            xr = x[(size_t)(t + 1) * C + c];
            if (MODE == 2) zr = uz[(size_t)(t + 1) * uz_stride + C + c];
        }
        const TD* lr = low + (size_t)t * low_stride;
        float Bv[NS], Cv[NS];
#pragma unroll
        for (int q = 0; q < NS / 8; ++q) {
            load8(lr + b_col + 8 * q, Bv + 8 * q);
            if (MODE == 2) load8(lr + c_col + 8 * q, Cv + 8 * q);
        }
        const float dx = dt * xv;
        float acc = 0.0f;
        sum += dt;
#pragma unroll
        for (int n = 0; n < NS; ++n) {
            S[n] = decay_exp<TD>(dt * a[n]) * S[n] + dx * Bv[n];
            if (MODE == 2) acc += S[n] * Cv[n];
        }
        if (MODE == 2) out[(size_t)t * C + c] = from_float<TD>((acc + d_skip * xv) * silu_f(zv));
    }
    if (MODE == 1) {
#pragma unroll
        for (int q = 0; q < NS / 4; ++q)
            *reinterpret_cast<float4*>(mine + 4 * q) = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
        dt_sum[(size_t)item * C + c] = sum;
    }
    if (MODE == 2 && last && K > 1) {
        const int seg_first = seg_start[seg], seg_rows = first + rows - seg_first;
        float* past = state + (size_t)seg_slot[seg] * state_stride + (size_t)C * NS;
        for (int k = 0; k < K - 1; ++k) {
            const int src = seg_rows - (K - 1) + k;
            past[(size_t)k * C + c] = src >= 0 ? to_float<TD>(uz[(size_t)(seg_first + src) * uz_stride + c]) : past[(size_t)(k + seg_rows) * C + c];
        }
    }
}

// Between the two passes over the chunks: for every request, chunk by chunk in order, carry[chunk] <- the S the chunk
// starts with, S <- exp(A * dt_sum[chunk]) * S + P[chunk] (P is what mode 1 left in carry[chunk]); the last S goes into
// the request's state slot.  One thread per (channel, state index); seg_items[s] .. seg_items[s + 1] are the chunks of
// segment s.
__global__ void scan_carry_kernel(float* __restrict__ carry, const float* __restrict__ dt_sum, const float* __restrict__ A,
                                  float* __restrict__ state, long long state_stride, const int32_t* __restrict__ seg_slot,
                                  const int32_t* __restrict__ seg_items, int C, int N) {
    pdl_launch_dependents();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)C * N) return;
    const int seg = blockIdx.y, c = (int)(idx / N);
    float* st = state + (size_t)seg_slot[seg] * state_stride;
    const float a = A[idx];
    float S = st[idx];
    for (int item = seg_items[seg]; item < seg_items[seg + 1]; ++item) {
        float* slot = carry + (size_t)item * C * N + idx;
        const float p = *slot;
        *slot = S;
        S = expf(a * dt_sum[(size_t)item * C + c]) * S + p;
    }
    st[idx] = S;
}

}  // namespace

PH_EXPORT int ph_causal_conv_silu(const void* u, int u_dtype, long long row_stride, int C, const float* taps, const float* bias,
                                  int K, const float* state, long long state_stride, long long conv_offset,
                                  const int32_t* row_seg, const int32_t* seg_start, const int32_t* seg_slot, void* out,
                                  int out_dtype, int T, cudaStream_t stream) {
    if (!u || !taps || !state || !row_seg || !seg_start || !seg_slot || !out || T < 0 || C < 1 || K < 1 || row_stride < C ||
        !valid_dtype(u_dtype) || !valid_dtype(out_dtype))
        return fail(PH_ERR_ARG, "causal_conv_silu: bad arguments (T %d, C %d, K %d)", T, C, K);
    if (K > MAX_TAPS) return fail(PH_ERR_UNSUPPORTED, "causal_conv_silu: %d taps exceed the supported %d", K, MAX_TAPS);
    if (T == 0) return PH_OK;
    if (K >= 2 && K <= 4 && C % 8 == 0 && row_stride % 8 == 0 && conv_offset % 4 == 0 && state_stride % 4 == 0 &&
        (((uintptr_t)u | (uintptr_t)out | (uintptr_t)state | (uintptr_t)taps) & 15) == 0) {
        const unsigned vblocks = (unsigned)(((long long)T * (C / 8) + 255) / 256);
#define LAUNCH_CONV(TI, TO, KT)                                                                                                  \
    launch_overlapped(causal_conv_silu_vec_kernel<TI, TO, KT>, dim3(vblocks), dim3(256), 0, stream, (const TI*)u, row_stride, C, taps, \
                      bias, state, state_stride, conv_offset, row_seg, seg_start, seg_slot, (TO*)out, T)
        PH_DISPATCH(u_dtype, TI, PH_DISPATCH(out_dtype, TO, {
            if (K == 2) LAUNCH_CONV(TI, TO, 2); else if (K == 3) LAUNCH_CONV(TI, TO, 3); else LAUNCH_CONV(TI, TO, 4); }));
#undef LAUNCH_CONV
        return check_launch("causal_conv_silu");
    }
    const unsigned blocks = (unsigned)(((long long)T * C + 255) / 256);
    PH_DISPATCH(u_dtype, TI, PH_DISPATCH(out_dtype, TO,
        launch_overlapped(causal_conv_silu_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)u, row_stride, C, taps,
                          bias, K, state, state_stride, conv_offset, row_seg, seg_start, seg_slot, (TO*)out, T)));
    return check_launch("causal_conv_silu");
}

// x [T, C] (after the convolution), dt_raw [T, C] float32 (the step projection before its bias and softplus), low
// [T, low_stride] with B at b_col and C at c_col (N each), uz [T, uz_stride] = [u | z] of the in-projection, state
// [slots, state_stride] as laid out above, out [T, C].  data_dtype is the type of x, low, uz and out.
// items null: one pass, a block row per request.  Else n_items chunks (first row, rows, segment, last) with the chunks of
// segment s at seg_items[s] .. seg_items[s + 1], and scratch carry [n_items, C, N] and dt_sum [n_items, C]: three launches.
PH_EXPORT int ph_selective_scan(const void* x, const float* dt_raw, const float* dt_bias, const void* low, long long low_stride,
                                int b_col, int c_col, int N, const float* A, const float* D, const void* uz, long long uz_stride,
                                int C, int K, float* state, long long state_stride, const int32_t* seg_start,
                                const int32_t* seg_slot, int S, const int32_t* items, int n_items, const int32_t* seg_items,
                                float* carry, float* dt_sum, void* out, int data_dtype, cudaStream_t stream) {
    if (!x || !dt_raw || !low || !A || !uz || !state || !seg_start || !seg_slot || !out || S < 0 || C < 1 || N < 1 || K < 1 ||
        b_col < 0 || c_col < 0 || low_stride < N || uz_stride < 2LL * C || !valid_dtype(data_dtype))
        return fail(PH_ERR_ARG, "selective_scan: bad arguments (S %d, C %d, N %d)", S, C, N);
    if (items && (n_items < 1 || !seg_items || !carry || !dt_sum)) return fail(PH_ERR_ARG, "selective_scan: chunks need their lists and scratch");
    if (state_stride < (long long)C * N + (long long)(K - 1) * C)
        return fail(PH_ERR_ARG, "selective_scan: a state of %lld floats does not hold %d x %d states and %d x %d inputs", state_stride, C, N, K - 1, C);
    if (N > 32 * MAX_PER_LANE) return fail(PH_ERR_UNSUPPORTED, "selective_scan: %d states per channel exceed the supported %d", N, 32 * MAX_PER_LANE);
    if (K > MAX_TAPS) return fail(PH_ERR_UNSUPPORTED, "selective_scan: %d taps exceed the supported %d", K, MAX_TAPS);
    if (S == 0) return PH_OK;
    const int block_rows = items ? n_items : S;
    if (block_rows > 65535 || S > 65535) return fail(PH_ERR_UNSUPPORTED, "selective_scan: %d block rows exceed the supported 65535", block_rows);
    // lanes per channel: the fewest (a power of two) that leave a lane at most four states, at most a warp
    int L = 1;
    while (L < 32 && (N + L - 1) / L > 4) L *= 2;
    const int P = (N + L - 1) / L;
    const int per_block = SCAN_THREADS / L;
    dim3 grid((C + per_block - 1) / per_block, block_rows);
#define LAUNCH_SCAN(TD, MODE)                                                                                                   \
    launch_overlapped(selective_scan_kernel<TD, TD, TD, TD, MODE>, grid, dim3(SCAN_THREADS), 0, stream, (const TD*)x, dt_raw, dt_bias, \
                      (const TD*)low, low_stride, b_col, c_col, N, A, D, (const TD*)uz, uz_stride, C, K, state, state_stride,    \
                      seg_start, seg_slot, items, carry, dt_sum, (TD*)out, L, P)
    if (!items) {
        PH_DISPATCH(data_dtype, TD, LAUNCH_SCAN(TD, 0));
        return check_launch("selective_scan");
    }
    const int vec = data_dtype == PH_F32 ? 4 : 8;      // elements of 16 bytes
    const bool per_channel = (N == 8 || N == 16) && b_col % vec == 0 && c_col % vec == 0 && low_stride % vec == 0 &&
                             (((uintptr_t)low | (uintptr_t)A | (uintptr_t)carry) & 15) == 0;
    const dim3 cgrid((C + SCAN_THREADS - 1) / SCAN_THREADS, n_items);
#define LAUNCH_CHUNK(TD, MODE, NS)                                                                                                \
    launch_overlapped(scan_chunk_kernel<TD, MODE, NS>, cgrid, dim3(SCAN_THREADS), 0, stream, (const TD*)x, dt_raw, dt_bias,        \
                      (const TD*)low, low_stride, b_col, c_col, A, D, (const TD*)uz, uz_stride, C, K, state, state_stride, seg_start, \
                      seg_slot, items, carry, dt_sum, (TD*)out)
    if (per_channel) PH_DISPATCH(data_dtype, TD, { if (N == 8) LAUNCH_CHUNK(TD, 1, 8); else LAUNCH_CHUNK(TD, 1, 16); });
    else PH_DISPATCH(data_dtype, TD, LAUNCH_SCAN(TD, 1));
    launch_overlapped(scan_carry_kernel, dim3((unsigned)(((long long)C * N + 255) / 256), S), dim3(256), 0, stream, carry,
                      (const float*)dt_sum, A, state, state_stride, seg_slot, seg_items, C, N);
    if (per_channel) PH_DISPATCH(data_dtype, TD, { if (N == 8) LAUNCH_CHUNK(TD, 2, 8); else LAUNCH_CHUNK(TD, 2, 16); });
    else PH_DISPATCH(data_dtype, TD, LAUNCH_SCAN(TD, 2));
#undef LAUNCH_CHUNK
#undef LAUNCH_SCAN
    return check_launch("selective_scan");
}
