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

template <typename TX, typename TL, typename TZ, typename TO>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dt_raw, const float* __restrict__ dt_bias,
                      const TL* __restrict__ low, long long low_stride, int b_col, int c_col, int N, const float* __restrict__ A,
                      const float* __restrict__ D, const TZ* __restrict__ uz, long long uz_stride, int C, int K,
                      float* __restrict__ state, long long state_stride, const int32_t* __restrict__ seg_start,
                      const int32_t* __restrict__ seg_slot, TO* __restrict__ out, int L, int P) {
    pdl_launch_dependents();
    pdl_wait();
    const int seg = blockIdx.y;
    const int group = threadIdx.x / L, lane = threadIdx.x % L;
    const int c = blockIdx.x * (SCAN_THREADS / L) + group;
    const bool live = c < C;                                   // dead lanes still take part in the shuffles
    const int cc = live ? c : C - 1;
    const int first = seg_start[seg], rows = seg_start[seg + 1] - first;
    float* st = state + (size_t)seg_slot[seg] * state_stride;
    float S[MAX_PER_LANE], a[MAX_PER_LANE];
#pragma unroll
    for (int p = 0; p < MAX_PER_LANE; ++p) {
        const int n = lane + L * p;
        const bool on = p < P && n < N;
        S[p] = on ? st[(size_t)cc * N + n] : 0.0f;
        a[p] = on ? A[(size_t)cc * N + n] : 0.0f;
    }
    const float bias = dt_bias ? dt_bias[cc] : 0.0f, d_skip = D ? D[cc] : 0.0f;
    for (int i = 0; i < rows; ++i) {
        const int t = first + i;
        const float dt = softplus_f(dt_raw[(size_t)t * C + cc] + bias);
        const float xv = to_float<TX>(x[(size_t)t * C + cc]);
        const float dx = dt * xv;
        const TL* lr = low + (size_t)t * low_stride;
        float acc = 0.0f;
#pragma unroll
        for (int p = 0; p < MAX_PER_LANE; ++p) {
            const int n = lane + L * p;
            if (p < P && n < N) {
                S[p] = expf(dt * a[p]) * S[p] + dx * to_float<TL>(lr[b_col + n]);
                acc += S[p] * to_float<TL>(lr[c_col + n]);
            }
        }
        for (int o = L >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (live && lane == 0) {
            const float z = to_float<TZ>(uz[(size_t)t * uz_stride + C + c]);
            out[(size_t)t * C + c] = from_float<TO>((acc + d_skip * xv) * silu_f(z));
        }
    }
    if (!live) return;
#pragma unroll
    for (int p = 0; p < MAX_PER_LANE; ++p) {
        const int n = lane + L * p;
        if (p < P && n < N) st[(size_t)c * N + n] = S[p];
    }
    if (lane == 0 && K > 1) {
        // the last K - 1 convolution inputs, oldest first: from this step's rows, or moved up from what was kept
        float* past = st + (size_t)C * N;
        for (int k = 0; k < K - 1; ++k) {
            const int src = rows - (K - 1) + k;
            past[(size_t)k * C + c] = src >= 0 ? to_float<TZ>(uz[(size_t)(first + src) * uz_stride + c]) : past[(size_t)(k + rows) * C + c];
        }
    }
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
    const unsigned blocks = (unsigned)(((long long)T * C + 255) / 256);
    PH_DISPATCH(u_dtype, TI, PH_DISPATCH(out_dtype, TO,
        launch_overlapped(causal_conv_silu_kernel<TI, TO>, dim3(blocks), dim3(256), 0, stream, (const TI*)u, row_stride, C, taps,
                          bias, K, state, state_stride, conv_offset, row_seg, seg_start, seg_slot, (TO*)out, T)));
    return check_launch("causal_conv_silu");
}

// x [T, C] (after the convolution), dt_raw [T, C] float32 (the step projection before its bias and softplus), low
// [T, low_stride] with B at b_col and C at c_col (N each), uz [T, uz_stride] = [u | z] of the in-projection, state
// [slots, state_stride] as laid out above, out [T, C].  data_dtype is the type of x, low, uz and out.
PH_EXPORT int ph_selective_scan(const void* x, const float* dt_raw, const float* dt_bias, const void* low, long long low_stride,
                                int b_col, int c_col, int N, const float* A, const float* D, const void* uz, long long uz_stride,
                                int C, int K, float* state, long long state_stride, const int32_t* seg_start,
                                const int32_t* seg_slot, int S, void* out, int data_dtype, cudaStream_t stream) {
    if (!x || !dt_raw || !low || !A || !uz || !state || !seg_start || !seg_slot || !out || S < 0 || C < 1 || N < 1 || K < 1 ||
        b_col < 0 || c_col < 0 || low_stride < N || uz_stride < 2LL * C || !valid_dtype(data_dtype))
        return fail(PH_ERR_ARG, "selective_scan: bad arguments (S %d, C %d, N %d)", S, C, N);
    if (state_stride < (long long)C * N + (long long)(K - 1) * C)
        return fail(PH_ERR_ARG, "selective_scan: a state of %lld floats does not hold %d x %d states and %d x %d inputs", state_stride, C, N, K - 1, C);
    if (N > 32 * MAX_PER_LANE) return fail(PH_ERR_UNSUPPORTED, "selective_scan: %d states per channel exceed the supported %d", N, 32 * MAX_PER_LANE);
    if (K > MAX_TAPS) return fail(PH_ERR_UNSUPPORTED, "selective_scan: %d taps exceed the supported %d", K, MAX_TAPS);
    if (S == 0) return PH_OK;
    if (S > 65535) return fail(PH_ERR_UNSUPPORTED, "selective_scan: %d requests in one step exceed the supported 65535", S);
    // lanes per channel: the fewest (a power of two) that leave a lane at most four states, at most a warp
    int L = 1;
    while (L < 32 && (N + L - 1) / L > 4) L *= 2;
    const int P = (N + L - 1) / L;
    const int per_block = SCAN_THREADS / L;
    dim3 grid((C + per_block - 1) / per_block, S);
    PH_DISPATCH(data_dtype, TD,
        launch_overlapped(selective_scan_kernel<TD, TD, TD, TD>, grid, dim3(SCAN_THREADS), 0, stream, (const TD*)x, dt_raw, dt_bias,
                          (const TD*)low, low_stride, b_col, c_col, N, A, D, (const TD*)uz, uz_stride, C, K, state, state_stride,
                          seg_start, seg_slot, (TD*)out, L, P));
    return check_launch("selective_scan");
}
