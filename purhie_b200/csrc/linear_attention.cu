// Gated linear attention: a matrix-valued state per head that decays channel by channel, and what surrounds it.
//
//   decayed_scan   per request and head, token by token in the order of the rows:
//                      a_t = sigmoid(z_t + b)^(1/tau)            per key channel, as exp(-softplus(-(z_t + b)) / tau)
//                      S   <- diag(a_t) S + k_t v_t^T            S is [D, DV] float32 and lives in the request's state slot
//                      o_t  = S^T (q_t * q_scale)
//                  followed, for the rows the block has just written, by the per-head RMS norm over DV with a weight
//                  shared by the heads and the gate silu(g_t): y_t = o_t * rsqrt(mean(o_t^2) + eps) * w * silu(g_t)
//                  (head_norm_gate as a launch of its own where a head's columns are spread over several blocks).
//                  A block owns one (request, head): thread (part, column) keeps D / parts state values of its column in
//                  registers, the token's q, k and decay are staged in shared memory one token ahead, and the parts'
//                  partial sums meet in shared memory in a fixed order.  A prompt cut anywhere walks the same
//                  recurrence in the same order, so the result does not depend on the cut, the batch or the slot.
//   rms_pair_mean  out = (a * rsqrt(mean(a^2) + eps) * wa + b * rsqrt(mean(b^2) + eps) * wb) * factor per row: the
//                  outputs of two mixers that read the same input, each RMS-normed over the model width, combined.
// Everything here is float32 arithmetic; q, k, v and g may be stored in bfloat16.
#include "common.cuh"

#include <math.h>

namespace {

using namespace ph;

// log(sigmoid(x)) without overflow: -(max(-x, 0) + log1p(exp(-|x|)))
__device__ __forceinline__ float log_sigmoid(float x) { return -(fmaxf(-x, 0.0f) + log1pf(expf(-fabsf(x)))); }

struct ScanParams {
    const void* q; const void* k; const void* v; const void* g;     // rows of the compute dtype, `stride` elements apart
    long long stride;
    const float* z; long long z_stride;                              // [T, H * D] float32: the decay's logits without their bias
    const float* z_bias;                                             // [H * D] or null
    float inv_tau, q_scale, eps;
    const float* norm_w;                                             // [DV]
    float* state; long long slot_stride;                             // [slots][H][D][DV]
    const int32_t* seg_start; const int32_t* seg_slot;
    float* raw;                                                      // [T, H * DV] float32 scratch: o before the norm
    void* out;                                                       // [T, H * DV] in the compute dtype
    int H, D, DV;
    int tile;                                                        // columns of a head per block (a multiple of 32)
    int fused_norm;                                                  // the block holds all of a head's columns and norms its rows
};

// y = o * rsqrt(mean over the head's DV values of o^2 + eps) * w * silu(g) for the rows [row0, row0 + n) of head h, a warp per row
template <typename TX>
__device__ __forceinline__ void norm_gate_rows(const ScanParams& p, int h, int row0, int n, int warp, int warps, int lane) {
    const int H = p.H, DV = p.DV;
    const TX* gb = static_cast<const TX*>(p.g) + (size_t)h * DV;
    TX* out = static_cast<TX*>(p.out);
    for (int t = warp; t < n; t += warps) {
        const size_t at = (size_t)(row0 + t) * H * DV + (size_t)h * DV;
        float ss = 0.0f;
        for (int c = lane; c < DV; c += 32) { const float o = p.raw[at + c]; ss += o * o; }
        const float inv = rsqrtf(warp_sum(ss) / (float)DV + p.eps);
        for (int c = lane; c < DV; c += 32) {
            const float gate = to_float<TX>(gb[(size_t)(row0 + t) * p.stride + c]);
            out[at + c] = from_float<TX>(p.raw[at + c] * inv * p.norm_w[c] * (gate / (1.0f + expf(-gate))));
        }
    }
}

// DPT state values per thread; blockDim.x = parts * DVP with DVP the block's columns (p.tile).
template <typename TX, int DPT>
__global__ void __launch_bounds__(16384 / DPT) decayed_scan_kernel(ScanParams p) {
    extern __shared__ float smem[];
    const int D = p.D, DV = p.DV, H = p.H;
    const int DVP = p.tile;
    const int parts = blockDim.x / DVP;
    const int Dpad = parts * DPT;
    float* stage = smem;                              // [2][3][Dpad]: q, k, decay of a token
    float* partial = smem + 2 * 3 * Dpad;             // [2][parts][DVP]
    const int seg = blockIdx.x, h = blockIdx.y;
    const int part = threadIdx.x / DVP, col = blockIdx.z * DVP + threadIdx.x % DVP, lcol = threadIdx.x % DVP;
    const int d0 = part * DPT;
    const bool live = col < DV;
    pdl_launch_dependents();
    pdl_wait();
    const int row0 = p.seg_start[seg], n = p.seg_start[seg + 1] - row0;
    if (n <= 0) return;
    float* S = p.state + (size_t)p.seg_slot[seg] * p.slot_stride + (size_t)h * D * DV;
    float s[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) s[i] = (live && d0 + i < D) ? S[(size_t)(d0 + i) * DV + col] : 0.0f;

    const TX* qb = static_cast<const TX*>(p.q) + (size_t)h * D;
    const TX* kb = static_cast<const TX*>(p.k) + (size_t)h * D;
    const TX* vb = static_cast<const TX*>(p.v) + (size_t)h * DV;
    auto stage_token = [&](int t, int buf) {
        float* dst = stage + (size_t)buf * 3 * Dpad;
        const size_t row = (size_t)(row0 + t);
        for (int i = threadIdx.x; i < 3 * Dpad; i += blockDim.x) {
            const int which = i / Dpad, d = i % Dpad;
            float val = 0.0f;
            if (d < D) {
                if (which == 0) val = to_float<TX>(qb[row * p.stride + d]) * p.q_scale;
                else if (which == 1) val = to_float<TX>(kb[row * p.stride + d]);
                else {
                    const float zz = p.z[row * p.z_stride + (size_t)h * D + d] + (p.z_bias ? p.z_bias[(size_t)h * D + d] : 0.0f);
                    val = expf(log_sigmoid(zz) * p.inv_tau);
                }
            }
            dst[i] = val;
        }
    };
    stage_token(0, 0);
    float v_next = live ? to_float<TX>(vb[(size_t)row0 * p.stride + col]) : 0.0f;
    __syncthreads();
    for (int t = 0; t < n; ++t) {
        const int buf = t & 1;
        const float vt = v_next;
        if (t + 1 < n) {
            stage_token(t + 1, buf ^ 1);
            v_next = live ? to_float<TX>(vb[(size_t)(row0 + t + 1) * p.stride + col]) : 0.0f;
        }
        const float* qs = stage + (size_t)buf * 3 * Dpad + d0;
        const float* ks = qs + Dpad;
        const float* as = ks + Dpad;
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qs + i), k4 = *reinterpret_cast<const float4*>(ks + i),
                         a4 = *reinterpret_cast<const float4*>(as + i);
            s[i] = fmaf(a4.x, s[i], k4.x * vt);         acc = fmaf(s[i], q4.x, acc);
            s[i + 1] = fmaf(a4.y, s[i + 1], k4.y * vt); acc = fmaf(s[i + 1], q4.y, acc);
            s[i + 2] = fmaf(a4.z, s[i + 2], k4.z * vt); acc = fmaf(s[i + 2], q4.z, acc);
            s[i + 3] = fmaf(a4.w, s[i + 3], k4.w * vt); acc = fmaf(s[i + 3], q4.w, acc);
        }
        partial[((size_t)buf * parts + part) * DVP + lcol] = acc;
        __syncthreads();
        if (part == 0 && live) {
            float o = 0.0f;
            for (int j = 0; j < parts; ++j) o += partial[((size_t)buf * parts + j) * DVP + lcol];
            p.raw[(size_t)(row0 + t) * H * DV + (size_t)h * DV + col] = o;
        }
    }
    if (live)
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (d0 + i < D) S[(size_t)(d0 + i) * DV + col] = s[i];
    if (!p.fused_norm) return;
    // the rows this block wrote: norm over the head's DV values, the weight, the gate
    __syncthreads();
    norm_gate_rows<TX>(p, h, row0, n, threadIdx.x >> 5, blockDim.x >> 5, threadIdx.x & 31);
}

template <typename TX>
__global__ void head_norm_gate_kernel(ScanParams p, int T) {
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5;
    const long long item = (long long)blockIdx.x * warps + (threadIdx.x >> 5);
    if (item >= (long long)T * p.H) return;
    norm_gate_rows<TX>(p, (int)(item % p.H), (int)(item / p.H), 1, 0, 1, threadIdx.x & 31);
}

template <typename TA, typename TB>
__global__ void rms_pair_mean_kernel(const TA* __restrict__ a, int a_splits, long long a_stride, const float* __restrict__ wa,
                                     const TB* __restrict__ b, int b_splits, long long b_stride, const float* __restrict__ wb,
                                     float eps, float factor, float* __restrict__ out, int E) {
    extern __shared__ float buf[];            // [2][E]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * E;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        float x = 0.0f, y = 0.0f;
        for (int s = 0; s < a_splits; ++s) x += to_float<TA>(a[(size_t)s * a_stride + row + i]);
        for (int s = 0; s < b_splits; ++s) y += to_float<TB>(b[(size_t)s * b_stride + row + i]);
        buf[i] = x; buf[E + i] = y;
        sa += x * x; sb += y * y;
    }
    const float ia = rsqrtf(block_sum_any(sa, scratch) / (float)E + eps);
    const float ib = rsqrtf(block_sum_any(sb, scratch) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[row + i] = (buf[i] * ia * wa[i] + buf[E + i] * ib * wb[i]) * factor;
}

}  // namespace

PH_EXPORT int ph_decayed_scan(const void* q, const void* k, const void* v, const void* g, int dtype, long long stride, const float* z,
                              long long z_stride, const float* z_bias, float tau, float q_scale, const float* norm_w, float eps,
                              float* state, long long slot_stride, const int32_t* seg_start, const int32_t* seg_slot, int S, int T, int H,
                              int D, int DV, float* raw, void* out, cudaStream_t stream) {
    if (!q || !k || !v || !g || !z || !norm_w || !state || !seg_start || !seg_slot || !raw || !out || S < 0 || H < 1 || D < 1 || DV < 1 ||
        !(tau > 0.0f) || !valid_dtype(dtype))
        return fail(PH_ERR_ARG, "decayed_scan: bad arguments (S %d, H %d, D %d, DV %d)", S, H, D, DV);
    if (S == 0) return PH_OK;
    // the fewest state values per thread with which one block holds all columns of a head; else blocks of fewer columns
    const int DVP = (DV + 31) & ~31;
    int dpt = 0, tile = 0;
    for (int c = 16; c <= 64 && !dpt; c *= 2)
        if ((long long)DVP * ((D + c - 1) / c) <= 16384 / c) { dpt = c; tile = DVP; }
    if (!dpt) {
        dpt = 16;
        tile = 1024 / ((D + 15) / 16) / 32 * 32;
        if (tile < 32) return fail(PH_ERR_UNSUPPORTED, "decayed_scan: %d key channels per head do not fit one block", D);
    }
    const int parts = (D + dpt - 1) / dpt;
    ScanParams p;
    p.q = q; p.k = k; p.v = v; p.g = g; p.stride = stride; p.z = z; p.z_stride = z_stride; p.z_bias = z_bias;
    p.inv_tau = 1.0f / tau; p.q_scale = q_scale; p.eps = eps; p.norm_w = norm_w; p.state = state; p.slot_stride = slot_stride;
    p.seg_start = seg_start; p.seg_slot = seg_slot; p.raw = raw; p.out = out; p.H = H; p.D = D; p.DV = DV;
    p.tile = tile; p.fused_norm = tile == DVP;
    const size_t smem = (size_t)(2 * 3 * parts * dpt + 2 * parts * tile) * sizeof(float);
    const dim3 grid(S, H, (DVP + tile - 1) / tile), block(tile * parts);
#define LAUNCH_SCAN(TX, DPT) launch_overlapped(decayed_scan_kernel<TX, DPT>, grid, block, smem, stream, p)
    PH_DISPATCH(dtype, TX, {
        if (dpt == 16) LAUNCH_SCAN(TX, 16);
        else if (dpt == 32) LAUNCH_SCAN(TX, 32);
        else LAUNCH_SCAN(TX, 64);
    });
#undef LAUNCH_SCAN
    if (!p.fused_norm) {
        if (T < 1) return fail(PH_ERR_ARG, "decayed_scan: the number of rows is needed when a head is spread over blocks");
        const long long items = (long long)T * H;
        PH_DISPATCH(dtype, TX, launch_overlapped(head_norm_gate_kernel<TX>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, p, T));
    }
    return check_launch("decayed_scan");
}

PH_EXPORT int ph_rms_pair_mean(const void* a, int a_dtype, int a_splits, long long a_stride, const float* wa, const void* b, int b_dtype,
                               int b_splits, long long b_stride, const float* wb, float eps, float factor, float* out, int T, int E,
                               cudaStream_t stream) {
    if (!a || !b || !wa || !wb || !out || T < 0 || E < 1 || a_splits < 1 || b_splits < 1 || !valid_dtype(a_dtype) || !valid_dtype(b_dtype))
        return fail(PH_ERR_ARG, "rms_pair_mean: bad arguments (T %d, E %d)", T, E);
    if (T == 0) return PH_OK;
    const size_t smem = (size_t)2 * E * sizeof(float);
    if (smem > 200 * 1024) return fail(PH_ERR_UNSUPPORTED, "rms_pair_mean: two rows of %d do not fit shared memory", E);
    const int threads = E >= 2048 ? 512 : E >= 512 ? 256 : 128;
#define LAUNCH_PAIR(TA, TB)                                                                                                      \
    do {                                                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(rms_pair_mean_kernel<TA, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_overlapped(rms_pair_mean_kernel<TA, TB>, dim3(T), dim3(threads), smem, stream, (const TA*)a, a_splits, a_stride, wa, \
                          (const TB*)b, b_splits, b_stride, wb, eps, factor, out, E);                                           \
    } while (0)
    PH_DISPATCH(a_dtype, TA, PH_DISPATCH(b_dtype, TB, LAUNCH_PAIR(TA, TB)));
#undef LAUNCH_PAIR
    return check_launch("rms_pair_mean");
}
