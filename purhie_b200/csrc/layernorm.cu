// Layer norm with weight and bias, with the residual add folded in front of it, and with a transform of the addend
// folded in front of that: one pass per row does
//     a = sum over the splits of add[s][t]                       (the output of a mixer or feed-forward)
//     a = (a - mean(a)) / sqrt(var(a) + post_eps) * post_w + post_b      (when post_w is given: a norm on the addend)
//     v = x[t] + add_scale * a                                   (stored back to x[t] when write_x)
//     y = (v - mean(v)) / sqrt(var(v) + eps) * w + b             (when w is given; y = v when only y is: a part that
//                                                                 reads the residual itself, in its own dtype)
// which is what a layer of the form x <- x + m * norm_b(f(norm_a(x))) needs between f and the next f.  The variance
// is the mean of the squared deviations from the mean (two passes over the row, which sits in registers or shared memory);
// all sums are float32 in an order that depends on the row width only.  Embedding rows may be scaled on the way
// into the residual (embed_gather_scaled).
#include "common.cuh"

namespace {

using namespace ph;

// mean and 1 / sqrt(variance + eps) of the E floats in buf (every thread gets both)
__device__ __forceinline__ void row_stats(const float* buf, int E, float eps, float* scratch, float& mean, float& inv) {
    float s = 0.0f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) s += buf[i];
    mean = block_sum_any(s, scratch) / (float)E;
    float q = 0.0f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
        const float d = buf[i] - mean;
        q += d * d;
    }
    const float var = block_sum_any(q, scratch) / (float)E;
    inv = 1.0f / sqrtf(var + eps);
}

template <typename TA, typename TY>
__global__ void add_layernorm_kernel(float* __restrict__ x, const TA* __restrict__ add, int add_splits, long long add_split_stride,
                                     const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps,
                                     float add_scale, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                     const int32_t* __restrict__ rows, int E, TY* __restrict__ y, int write_x) {
    extern __shared__ float buf[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float* xr = x + (size_t)t * E;
    if (add) {
        const TA* a = add + (size_t)t * E;
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float v = 0.0f;
            for (int s = 0; s < add_splits; ++s) v += to_float<TA>(a[(size_t)s * add_split_stride + i]);
            buf[i] = v;
        }
        __syncthreads();
        float mean = 0.0f, inv = 1.0f;
        if (post_w) row_stats(buf, E, post_eps, scratch, mean, inv);
        for (int i = threadIdx.x; i < E; i += blockDim.x) {
            float v = buf[i];
            if (post_w) v = (v - mean) * inv * post_w[i] + (post_b ? post_b[i] : 0.0f);
            v = xr[i] + add_scale * v;
            if (write_x) xr[i] = v;
            buf[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < E; i += blockDim.x) buf[i] = xr[i];
    }
    if (!w) {
        if (y) {
            __syncthreads();
            for (int i = threadIdx.x; i < E; i += blockDim.x) y[(size_t)r * E + i] = from_float<TY>(buf[i]);
        }
        return;
    }
    __syncthreads();
    float mean, inv;
    row_stats(buf, E, eps, scratch, mean, inv);
    TY* yr = y + (size_t)r * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) yr[i] = from_float<TY>((buf[i] - mean) * inv * w[i] + (b ? b[i] : 0.0f));
}

// The same with a row held in registers, four consecutive elements per thread and round (E a multiple of 4, rows
// 16-byte aligned, at most ROUNDS * 4 * blockDim elements): every load of a pass is in flight at once, which is what a
// decode step's handful of rows needs.  Sums are taken per thread over its own elements, then over the block: their
// order depends on E alone.
template <typename TA, typename TY, int ROUNDS>
__global__ void add_layernorm_vec_kernel(float* __restrict__ x, const TA* __restrict__ add, int add_splits, long long add_split_stride,
                                         const float* __restrict__ post_w, const float* __restrict__ post_b, float post_eps,
                                         float add_scale, const float* __restrict__ w, const float* __restrict__ b, float eps,
                                         const int32_t* __restrict__ rows, int E, TY* __restrict__ y, int write_x) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int t = rows ? rows[r] : r;
    float* xr = x + (size_t)t * E;
    float4 v[ROUNDS];
    const float inv_e = 1.0f / (float)E;
    auto stats = [&](float e, float& mean, float& inv) {
        float s = 0.0f;
#pragma unroll
        for (int k = 0; k < ROUNDS; ++k)
            if ((threadIdx.x + k * blockDim.x) * 4 < E) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        mean = block_sum_any(s, scratch) * inv_e;
        float q = 0.0f;
#pragma unroll
        for (int k = 0; k < ROUNDS; ++k)
            if ((threadIdx.x + k * blockDim.x) * 4 < E) {
                const float dx = v[k].x - mean, dy = v[k].y - mean, dz = v[k].z - mean, dw = v[k].w - mean;
                q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        inv = 1.0f / sqrtf(block_sum_any(q, scratch) * inv_e + e);
    };
    float4 xv[ROUNDS];
#pragma unroll
    for (int k = 0; k < ROUNDS; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        xv[k] = i < E ? load4(xr + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (add) {
        const TA* a = add + (size_t)t * E;
#pragma unroll
        for (int k = 0; k < ROUNDS; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 4;
            v[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (i < E)
                for (int s = 0; s < add_splits; ++s) {
                    const float4 u = load4(a + (size_t)s * add_split_stride + i);
                    v[k].x += u.x; v[k].y += u.y; v[k].z += u.z; v[k].w += u.w;
                }
        }
        float mean = 0.0f, inv = 1.0f;
        if (post_w) stats(post_eps, mean, inv);
#pragma unroll
        for (int k = 0; k < ROUNDS; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 4;
            if (i >= E) continue;
            float4 u = v[k];
            if (post_w) {
                const float4 pw = load4(post_w + i), pb = post_b ? load4(post_b + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                u.x = (u.x - mean) * inv * pw.x + pb.x; u.y = (u.y - mean) * inv * pw.y + pb.y;
                u.z = (u.z - mean) * inv * pw.z + pb.z; u.w = (u.w - mean) * inv * pw.w + pb.w;
            }
            u.x = xv[k].x + add_scale * u.x; u.y = xv[k].y + add_scale * u.y;
            u.z = xv[k].z + add_scale * u.z; u.w = xv[k].w + add_scale * u.w;
            if (write_x) *reinterpret_cast<float4*>(xr + i) = u;
            v[k] = u;
        }
    } else {
#pragma unroll
        for (int k = 0; k < ROUNDS; ++k) v[k] = xv[k];
    }
    if (!w) {
        if (y) {
#pragma unroll
            for (int k = 0; k < ROUNDS; ++k) {
                const int i = (threadIdx.x + k * blockDim.x) * 4;
                if (i >= E) continue;
                const float o[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
                store4(y + (size_t)r * E + i, o);
            }
        }
        return;
    }
    float mean, inv;
    stats(eps, mean, inv);
    TY* yr = y + (size_t)r * E;
#pragma unroll
    for (int k = 0; k < ROUNDS; ++k) {
        const int i = (threadIdx.x + k * blockDim.x) * 4;
        if (i >= E) continue;
        const float4 ww = load4(w + i), bb = b ? load4(b + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float o[4] = {(v[k].x - mean) * inv * ww.x + bb.x, (v[k].y - mean) * inv * ww.y + bb.y,
                            (v[k].z - mean) * inv * ww.z + bb.z, (v[k].w - mean) * inv * ww.w + bb.w};
        store4(yr + i, o);
    }
}

template <typename TT>
__global__ void embed_gather_scaled_kernel(const TT* __restrict__ table, const int32_t* __restrict__ ids, float* __restrict__ out,
                                           int E, int V, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);       // ids are validated on the host; never read outside
    const TT* row = table + (size_t)id * E;
    float* o = out + (size_t)t * E;
    for (int i = threadIdx.x; i < E; i += blockDim.x) o[i] = to_float<TT>(row[i]) * scale;
}

}  // namespace

PH_EXPORT int ph_add_layernorm(float* x, const void* add, int add_dtype, int add_splits, long long add_split_stride,
                               const float* post_w, const float* post_b, float post_eps, float add_scale, const float* w,
                               const float* b, float eps, const int32_t* rows, int n_rows, int E, void* y, int y_dtype,
                               int write_x, cudaStream_t stream) {
    if (!x || n_rows < 0 || E < 1 || (w && !y) || (add && (add_splits < 1 || !valid_dtype(add_dtype))) || !valid_dtype(y_dtype))
        return fail(PH_ERR_ARG, "add_layernorm: bad arguments (rows %d, E %d)", n_rows, E);
    if (rows && write_x) return fail(PH_ERR_ARG, "add_layernorm: gathered rows do not write the residual back");
    if (n_rows == 0) return PH_OK;
    const size_t smem = (size_t)E * sizeof(float);
    if (smem > 200 * 1024) return fail(PH_ERR_UNSUPPORTED, "add_layernorm: a row of %d does not fit shared memory", E);
    // a row in registers where it fits: blocks of up to 1,024 threads, up to four rounds of four elements each
    const uintptr_t all = (uintptr_t)x | (uintptr_t)add | (uintptr_t)post_w | (uintptr_t)post_b | (uintptr_t)w | (uintptr_t)b | (uintptr_t)y;
    if (E % 4 == 0 && E <= 16384 && (all & 15) == 0 && add_split_stride % 4 == 0) {
        const int quads = E / 4;
        // few rows: as many threads as the row has quads (latency); many rows: a quarter of that (the rows fill the device)
        const int rounds = n_rows >= 256 ? (quads <= 128 ? 1 : quads <= 256 ? 2 : 4) : (quads <= 1024 ? 1 : quads <= 2048 ? 2 : 4);
        const int threads = ((quads + rounds - 1) / rounds + 31) / 32 * 32;
#define LAUNCH_LN_VEC(TA, TY)                                                                                                       \
    do {                                                                                                                            \
        if (rounds == 1)                                                                                                            \
            launch_overlapped(add_layernorm_vec_kernel<TA, TY, 1>, dim3(n_rows), dim3(threads), 0, stream, x, (const TA*)add, add_splits, \
                              add_split_stride, post_w, post_b, post_eps, add_scale, w, b, eps, rows, E, (TY*)y, write_x);           \
        else if (rounds == 2)                                                                                                       \
            launch_overlapped(add_layernorm_vec_kernel<TA, TY, 2>, dim3(n_rows), dim3(threads), 0, stream, x, (const TA*)add, add_splits, \
                              add_split_stride, post_w, post_b, post_eps, add_scale, w, b, eps, rows, E, (TY*)y, write_x);           \
        else                                                                                                                        \
            launch_overlapped(add_layernorm_vec_kernel<TA, TY, 4>, dim3(n_rows), dim3(threads), 0, stream, x, (const TA*)add, add_splits, \
                              add_split_stride, post_w, post_b, post_eps, add_scale, w, b, eps, rows, E, (TY*)y, write_x);           \
    } while (0)
        PH_DISPATCH(add ? add_dtype : PH_F32, TA, PH_DISPATCH(y_dtype, TY, LAUNCH_LN_VEC(TA, TY)));
#undef LAUNCH_LN_VEC
        return check_launch("add_layernorm");
    }
#define LAUNCH_LN(TA, TY)                                                                                              \
    do {                                                                                                               \
        if (smem > 48 * 1024)                                                                                          \
            cudaFuncSetAttribute(add_layernorm_kernel<TA, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_overlapped(add_layernorm_kernel<TA, TY>, dim3(n_rows), dim3(256), smem, stream, x, (const TA*)add, add_splits, \
                          add_split_stride, post_w, post_b, post_eps, add_scale, w, b, eps, rows, E, (TY*)y, write_x);  \
    } while (0)
    PH_DISPATCH(add ? add_dtype : PH_F32, TA, PH_DISPATCH(y_dtype, TY, LAUNCH_LN(TA, TY)));
#undef LAUNCH_LN
    return check_launch("add_layernorm");
}

PH_EXPORT int ph_embed_gather_scaled(const void* table, int table_dtype, const int32_t* ids, float* out, int T, int E, int V,
                                     float scale, cudaStream_t stream) {
    if (!table || !ids || !out || T < 0 || E < 1 || V < 1 || !valid_dtype(table_dtype))
        return fail(PH_ERR_ARG, "embed_gather_scaled: bad arguments (T %d, E %d, V %d, dtype %d)", T, E, V, table_dtype);
    if (T == 0) return PH_OK;
    PH_DISPATCH(table_dtype, TT, launch_overlapped(embed_gather_scaled_kernel<TT>, dim3(T), dim3(256), 0, stream,
                                                   (const TT*)table, ids, out, E, V, scale));
    return check_launch("embed_gather_scaled");
}
