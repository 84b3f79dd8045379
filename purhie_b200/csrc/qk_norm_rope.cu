// Per-head RMSNorm of q and k, rotary position encoding, and the write of k and v into cache pages,
// in one launch over the fused [q | k | v] rows that the projection produced.
//
// One warp per (token, head).  For a q or k head: optional bias, v = v * rsqrt(mean_D(v^2) + eps) * w,
// then rotate-half pairs (i, i + n_rot/2): (a, b) -> (a cos - b sin, a sin + b cos) with the angle of the
// token's absolute position (interleaved = 1 pairs (2i, 2i + 1) instead); dimensions >= n_rot pass
// through.  A v head (DV wide, which need not be the width of a key) is biased and copied, or, with value mixing,
// blended with the values that the first mixing layer of the step left for the same token:
// v <- (1 - lambda) v + lambda v_first (mode 2), that first layer storing its own v as v_first (mode 1); the blended
// v is what goes to the cache.  The table row of a position holds n_rot / 2 cosines, then
// n_rot / 2 sines, one per pair.
// Sums and angles are float32; the cos/sin table is made on the host in double precision.
// Reference: src/attention.hip:273-313 (attn_prep: bias, norm, rotation, cache write), :219-240
// (the norm and the rotation), src/qwen_ops.cpp:15-24 (rotate-half pairing).
//
// Cache addressing: token slot s = page * page_size + offset; element (s, head h, d) of K lives at
// k_base + page * page_stride + (h * page_size + offset) * D + d, and the same for V from v_base.
#include "common.cuh"

namespace {

using namespace ph;

constexpr int WARPS = 4;

// A factor per token that the norm in front of the qkv product left out: rsqrt(sum over the chunks of sumsq[t][chunk] /
// width + eps).  The product is linear, so the factor is applied to its result here (before the bias).  sumsq null: 1.
struct RowFactor {
    const float* sumsq;
    int chunks, width;
    float eps;
};
__device__ __forceinline__ float row_factor(const RowFactor& rf, int t) {
    if (!rf.sumsq) return 1.0f;
    float s = 0.0f;
    for (int k = 0; k < rf.chunks; ++k) s += rf.sumsq[(size_t)t * rf.chunks + k];
    return rsqrtf(s / (float)rf.width + rf.eps);
}
constexpr int MAX_D = 512;

// A pair (a, b) turned by an angle with cosine c and sine s: (a c - b s, b c + a s), each as one product rounded and
// one fused multiply-add, written out so that every kernel of this file gives the same bits for the same pair.
// The sum of squares of four values, the same roundings wherever it is taken.
__device__ __forceinline__ float squares4(float a, float b, float c, float d) {
    return __fmaf_rn(d, d, __fmaf_rn(c, c, __fmaf_rn(b, b, __fmul_rn(a, a))));
}
__device__ __forceinline__ float turn_first(float a, float b, float c, float s) { return __fmaf_rn(a, c, -__fmul_rn(b, s)); }
__device__ __forceinline__ float turn_second(float a, float b, float c, float s) { return __fmaf_rn(a, s, __fmul_rn(b, c)); }

template <typename TI, typename TQ, typename TKV>
__global__ void qk_norm_rope_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                    const float* __restrict__ bias, const float* __restrict__ q_w,
                                    const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                    int n_rot, int max_pos, const int32_t* __restrict__ positions,
                                    const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                    TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                    int page_size, int HQ, int HKV, int D, int interleaved, RowFactor rf, int DV,
                                    float* __restrict__ v_first, const float* __restrict__ v_lambda, int v_mode) {
    __shared__ float buf[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * WARPS + warp;
    const int t = blockIdx.x;
    const int n_heads = HQ + 2 * HKV;
    if (head >= n_heads) return;
    const int width = (HQ + HKV) * D + HKV * DV;
    const bool is_q = head < HQ, is_k = !is_q && head < HQ + HKV;
    const size_t head_at = (is_q || is_k) ? (size_t)head * D : (size_t)(HQ + HKV) * D + (size_t)(head - HQ - HKV) * DV;
    const int hd = (is_q || is_k) ? D : DV;                    // this head's width
    const TI* src = qkv + (size_t)t * width + head_at;
    const float* b = bias ? bias + head_at : nullptr;
    float* row = buf[warp];
    const float rs = row_factor(rf, t);

    float ss = 0.0f;
    for (int d = lane; d < hd; d += 32) {
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += to_float<TI>(src[(size_t)s * split_stride + d]);
        v *= rs;
        if (b) v += b[d];
        row[d] = v;
        ss += v * v;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    if (!is_q && !is_k) {
        // v head: copy, or blend with the step's first values
        if (!slot_mapping) return;
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int h = head - HQ - HKV;
        TKV* dst = v_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * DV;
        float* first = v_first ? v_first + ((size_t)t * HKV + h) * DV : nullptr;
        const float lam = v_mode == 2 ? *v_lambda : 0.0f;
        __syncwarp();
        for (int d = lane; d < DV; d += 32) {
            float v = row[d];
            if (v_mode == 1) first[d] = v;
            else if (v_mode == 2) v = (1.0f - lam) * v + lam * first[d];
            dst[d] = from_float<TKV>(v);
        }
        return;
    }
    if (w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        for (int d = lane; d < D; d += 32) row[d] = row[d] * inv * w[d];
    }
    __syncwarp();
    float outv[MAX_D / 32];
    const int half = n_rot / 2;
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);     // positions are validated on the host
    const float* cs = cos_sin ? cos_sin + (size_t)pos * n_rot : nullptr;
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d >= D) break;
        float v = row[d];
        if (cs && d < n_rot) {
            if (interleaved) {
                const int j = d >> 1;
                const float c = cs[j], s = cs[half + j];
                v = (d & 1) ? turn_second(row[d - 1], row[d], c, s) : turn_first(row[d], row[d + 1], c, s);
            } else {
                const int j = d < half ? d : d - half;
                const float c = cs[j], s = cs[half + j];
                v = d < half ? turn_first(row[d], row[d + half], c, s) : turn_second(row[d - half], row[d], c, s);
            }
        }
        outv[i] = v;
    }
    if (is_q) {
        TQ* dst = q_out + ((size_t)t * HQ + head) * D;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d >= D) break;
            dst[d] = from_float<TQ>(outv[i]);
        }
    } else if (slot_mapping) {
        const int slot = slot_mapping[t];
        if (slot < 0) return;
        const int h = head - HQ;
        TKV* dst = k_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D;
#pragma unroll
        for (int i = 0; i < MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d >= D) break;
            dst[d] = from_float<TKV>(outv[i]);
        }
    }
}

// Fast path for head_dim 128 rotated over its whole width in half pairs, for a few tokens (where the launch is
// short of warps): one warp per token and HPW consecutive heads (1 as launched),
// four consecutive dimensions per lane, every load in flight at once, the rotation partner (64 dimensions away)
// fetched from lane ^ 16 by shuffle.  The order of the additions is the same for every launch shape.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a); u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename TI, typename TQ, typename TKV, int HPW>
__global__ void qk_norm_rope_d128_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                         const float* __restrict__ bias, const float* __restrict__ q_w,
                                         const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                         int max_pos, const int32_t* __restrict__ positions,
                                         const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                         TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                         int page_size, int HQ, int HKV, RowFactor rf, int interleaved,
                                         float* __restrict__ v_first, const float* __restrict__ v_lambda, int v_mode) {
    constexpr int D = 128;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head0 = (blockIdx.y * WARPS + warp) * HPW;      // this warp's HPW consecutive heads of token t
    const int t = blockIdx.x;
    const int n_heads = HQ + 2 * HKV;
    if (head0 >= n_heads) return;
    const int d0 = lane * 4;
    // what no kernel of this step writes (positions, slots, the table, the norms' weights) is fetched while the
    // kernel in front still runs
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float4 c = make_float4(1.0f, 1.0f, 1.0f, 1.0f), sn = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (cos_sin) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
        if (interleaved) {                                   // pairs (2i, 2i + 1): this lane's two pairs are 2 lane, 2 lane + 1
            const float2 cc = *reinterpret_cast<const float2*>(cos_sin + (size_t)pos * D + 2 * lane);
            const float2 ss = *reinterpret_cast<const float2*>(cos_sin + (size_t)pos * D + 64 + 2 * lane);
            c = make_float4(cc.x, cc.y, 0.0f, 0.0f);
            sn = make_float4(ss.x, ss.y, 0.0f, 0.0f);
        } else {
            const int j = (lane & 15) * 4;                   // pair index of this lane's first dimension
            c = ld4(cos_sin + (size_t)pos * D + j);
            sn = ld4(cos_sin + (size_t)pos * D + 64 + j);
        }
    }
    const float lam = v_mode == 2 ? *v_lambda : 0.0f;
    const float4 gq = q_w ? ld4(q_w + d0) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    const float4 gk = k_w ? ld4(k_w + d0) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    pdl_wait();
    const float rs = row_factor(rf, t);
    // every head's loads are issued before any of them is used
    float4 v[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (head0 + i >= n_heads) continue;
        const TI* src = qkv + (size_t)t * n_heads * D + (size_t)(head0 + i) * D + d0;
        for (int s0 = 0; s0 < splits; s0 += 8) {             // eight partial sums in flight, added in order
            float4 u[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                u[j] = s0 + j < splits ? ld4(src + (size_t)(s0 + j) * split_stride) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < splits) { v[i].x += u[j].x; v[i].y += u[j].y; v[i].z += u[j].z; v[i].w += u[j].w; }
        }
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int head = head0 + i;
        if (head >= n_heads) break;
        float4 x = make_float4(v[i].x * rs, v[i].y * rs, v[i].z * rs, v[i].w * rs);
        if (bias) {
            const float4 b = ld4(bias + (size_t)head * D + d0);
            x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
        }
        const bool is_q = head < HQ, is_k = !is_q && head < HQ + HKV;
        if (!is_q && !is_k) {
            if (slot < 0) continue;
            const int h = head - HQ - HKV;
            if (v_mode) {                                    // the step's first values: kept, or blended in
                float* first = v_first + ((size_t)t * HKV + h) * D + d0;
                if (v_mode == 1) st4(first, x);
                else {
                    const float4 f = ld4(first);
                    x = make_float4((1.0f - lam) * x.x + lam * f.x, (1.0f - lam) * x.y + lam * f.y, (1.0f - lam) * x.z + lam * f.z,
                                    (1.0f - lam) * x.w + lam * f.w);
                }
            }
            st4(v_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, x);
            continue;
        }
        const float* w = is_q ? q_w : k_w;
        if (w) {
            const float ss = warp_sum(squares4(x.x, x.y, x.z, x.w));
            const float inv = rsqrtf(ss / (float)D + eps);
            const float4 g = is_q ? gq : gk;
            x.x = x.x * inv * g.x; x.y = x.y * inv * g.y; x.z = x.z * inv * g.z; x.w = x.w * inv * g.w;
        }
        if (cos_sin && interleaved) {
            x = make_float4(turn_first(x.x, x.y, c.x, sn.x), turn_second(x.x, x.y, c.x, sn.x), turn_first(x.z, x.w, c.y, sn.y),
                            turn_second(x.z, x.w, c.y, sn.y));
        } else if (cos_sin) {
            float4 o;
            o.x = __shfl_xor_sync(0xffffffffu, x.x, 16); o.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
            o.z = __shfl_xor_sync(0xffffffffu, x.z, 16); o.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
            if (lane < 16) {       // first half: a cos - b sin
                x = make_float4(turn_first(x.x, o.x, c.x, sn.x), turn_first(x.y, o.y, c.y, sn.y), turn_first(x.z, o.z, c.z, sn.z),
                                turn_first(x.w, o.w, c.w, sn.w));
            } else {               // second half: a sin + b cos (a is the partner)
                x = make_float4(turn_second(o.x, x.x, c.x, sn.x), turn_second(o.y, x.y, c.y, sn.y), turn_second(o.z, x.z, c.z, sn.z),
                                turn_second(o.w, x.w, c.w, sn.w));
            }
        }
        if (is_q) {
            st4(q_out + ((size_t)t * HQ + head) * D + d0, x);
        } else if (slot >= 0) {
            const int h = head - HQ;
            st4(k_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, x);
        }
    }
}

// The same for many tokens: eight consecutive dimensions per lane (one 16-byte load of bfloat16), a half-warp per
// head, a warp walks ITERS pairs of heads of one token with every load issued first.  The sum of squares is added
// in the order of the kernel above (four-element groups, then a butterfly over the 32 groups: here over 16 lanes
// for the even and the odd group apart, then the two), so both give the same bits.  The rotation partner (64
// dimensions away) sits eight lanes away in the same half-warp.
struct F8 { float4 a, b; };
__device__ __forceinline__ F8 ld8(const float* p) { return {ld4(p), ld4(p + 4)}; }
__device__ __forceinline__ F8 ld8(const __nv_bfloat16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    return {make_float4(__low2float(h[0]), __high2float(h[0]), __low2float(h[1]), __high2float(h[1])),
            make_float4(__low2float(h[2]), __high2float(h[2]), __low2float(h[3]), __high2float(h[3]))};
}
__device__ __forceinline__ void st8(float* p, const F8& v) { st4(p, v.a); st4(p + 4, v.b); }
__device__ __forceinline__ void st8(__nv_bfloat16* p, const F8& v) {
    __nv_bfloat162 h0 = __floats2bfloat162_rn(v.a.x, v.a.y), h1 = __floats2bfloat162_rn(v.a.z, v.a.w);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(v.b.x, v.b.y), h3 = __floats2bfloat162_rn(v.b.z, v.b.w);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ void add4(float4& x, const float4& y) { x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w; }
__device__ __forceinline__ float4 shfl4(const float4& v, int m) {
    return make_float4(__shfl_xor_sync(0xffffffffu, v.x, m), __shfl_xor_sync(0xffffffffu, v.y, m),
                       __shfl_xor_sync(0xffffffffu, v.z, m), __shfl_xor_sync(0xffffffffu, v.w, m));
}
// first half of the head: a cos - b sin; second half: a sin + b cos with a the partner
__device__ __forceinline__ float4 rotate4(const float4& x, const float4& o, const float4& c, const float4& sn, bool first) {
    if (first) return make_float4(turn_first(x.x, o.x, c.x, sn.x), turn_first(x.y, o.y, c.y, sn.y), turn_first(x.z, o.z, c.z, sn.z),
                                  turn_first(x.w, o.w, c.w, sn.w));
    return make_float4(turn_second(o.x, x.x, c.x, sn.x), turn_second(o.y, x.y, c.y, sn.y), turn_second(o.z, x.z, c.z, sn.z),
                       turn_second(o.w, x.w, c.w, sn.w));
}

template <typename TI, typename TQ, typename TKV, int ITERS>
__global__ void qk_norm_rope_d128_wide_kernel(const TI* __restrict__ qkv, int splits, long long split_stride,
                                              const float* __restrict__ bias, const float* __restrict__ q_w,
                                              const float* __restrict__ k_w, float eps, const float* __restrict__ cos_sin,
                                              int max_pos, const int32_t* __restrict__ positions,
                                              const int32_t* __restrict__ slot_mapping, TQ* __restrict__ q_out,
                                              TKV* __restrict__ k_base, TKV* __restrict__ v_base, long long page_stride,
                                              int page_size, int HQ, int HKV, RowFactor rf, int interleaved,
                                              float* __restrict__ v_first, const float* __restrict__ v_lambda, int v_mode) {
    constexpr int D = 128;
    pdl_launch_dependents();
    pdl_wait();
    const float lam = v_mode == 2 ? *v_lambda : 0.0f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    const int head0 = (blockIdx.y * WARPS + warp) * 2 * ITERS + half;      // this half-warp's heads: head0, head0 + 2, ...
    const int t = blockIdx.x;
    const int n_heads = HQ + 2 * HKV;
    const int d0 = l16 * 8;
    const float rs = row_factor(rf, t);
    F8 v[ITERS];
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
        v[i] = {make_float4(0.0f, 0.0f, 0.0f, 0.0f), make_float4(0.0f, 0.0f, 0.0f, 0.0f)};
        const int head = head0 + 2 * i;
        if (head >= n_heads) continue;
        const TI* src = qkv + (size_t)t * n_heads * D + (size_t)head * D + d0;
        for (int s0 = 0; s0 < splits; ++s0) {
            const F8 u = ld8(src + (size_t)s0 * split_stride);
            add4(v[i].a, u.a);
            add4(v[i].b, u.b);
        }
    }
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float4 c0 = make_float4(1.0f, 1.0f, 1.0f, 1.0f), c1 = c0, s0 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), s1 = s0;
    if (cos_sin) {
        int pos = positions[t];
        pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
        const float* row = cos_sin + (size_t)pos * D;
        if (interleaved) {                                   // pairs (2i, 2i + 1): this lane's four pairs start at 4 l16
            c0 = ld4(row + 4 * l16);
            s0 = ld4(row + 64 + 4 * l16);
        } else {
            const int j = (l16 & 7) * 8;                     // pair index of this lane's first dimension
            c0 = ld4(row + j); c1 = ld4(row + j + 4);
            s0 = ld4(row + 64 + j); s1 = ld4(row + 64 + j + 4);
        }
    }
    const bool first = l16 < 8;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
        const int head = head0 + 2 * i;
        const bool live = head < n_heads;                     // the shuffles below are run by every lane
        F8 x = v[i];
        x.a = make_float4(x.a.x * rs, x.a.y * rs, x.a.z * rs, x.a.w * rs);
        x.b = make_float4(x.b.x * rs, x.b.y * rs, x.b.z * rs, x.b.w * rs);
        if (bias && live) {
            const F8 b = ld8(bias + (size_t)head * D + d0);
            add4(x.a, b.a);
            add4(x.b, b.b);
        }
        const bool is_q = head < HQ, is_k = !is_q && head < HQ + HKV;
        const float* w = is_q ? q_w : k_w;
        // sum of squares: the two four-element groups of the lane apart over the half-warp, then together
        float p0 = squares4(x.a.x, x.a.y, x.a.z, x.a.w);
        float p1 = squares4(x.b.x, x.b.y, x.b.z, x.b.w);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            p0 += __shfl_xor_sync(0xffffffffu, p0, o);
            p1 += __shfl_xor_sync(0xffffffffu, p1, o);
        }
        F8 y = x;
        if (w && (is_q || is_k) && live) {
            const float inv = rsqrtf((p0 + p1) / (float)D + eps);
            const F8 g = ld8(w + d0);
            y.a = make_float4(x.a.x * inv * g.a.x, x.a.y * inv * g.a.y, x.a.z * inv * g.a.z, x.a.w * inv * g.a.w);
            y.b = make_float4(x.b.x * inv * g.b.x, x.b.y * inv * g.b.y, x.b.z * inv * g.b.z, x.b.w * inv * g.b.w);
        }
        const float4 oa = shfl4(y.a, 8), ob = shfl4(y.b, 8);
        if (!live) continue;
        if (!is_q && !is_k) {
            if (slot >= 0) {
                const int h = head - HQ - HKV;
                if (v_mode) {                                // the step's first values: kept, or blended in
                    float* fp = v_first + ((size_t)t * HKV + h) * D + d0;
                    if (v_mode == 1) st8(fp, x);
                    else {
                        const F8 f = ld8(fp);
                        const float k = 1.0f - lam;
                        x.a = make_float4(k * x.a.x + lam * f.a.x, k * x.a.y + lam * f.a.y, k * x.a.z + lam * f.a.z, k * x.a.w + lam * f.a.w);
                        x.b = make_float4(k * x.b.x + lam * f.b.x, k * x.b.y + lam * f.b.y, k * x.b.z + lam * f.b.z, k * x.b.w + lam * f.b.w);
                    }
                }
                st8(v_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, x);
            }
            continue;
        }
        if (cos_sin && interleaved) {
            const float4 a = y.a, b = y.b;
            y.a = make_float4(turn_first(a.x, a.y, c0.x, s0.x), turn_second(a.x, a.y, c0.x, s0.x), turn_first(a.z, a.w, c0.y, s0.y),
                              turn_second(a.z, a.w, c0.y, s0.y));
            y.b = make_float4(turn_first(b.x, b.y, c0.z, s0.z), turn_second(b.x, b.y, c0.z, s0.z), turn_first(b.z, b.w, c0.w, s0.w),
                              turn_second(b.z, b.w, c0.w, s0.w));
        } else if (cos_sin) {
            y.a = rotate4(y.a, oa, c0, s0, first);
            y.b = rotate4(y.b, ob, c1, s1, first);
        }
        if (is_q) {
            st8(q_out + ((size_t)t * HQ + head) * D + d0, y);
        } else if (slot >= 0) {
            const int h = head - HQ;
            st8(k_base + (size_t)(slot / page_size) * page_stride + ((size_t)h * page_size + slot % page_size) * D + d0, y);
        }
    }
}

}  // namespace

PH_EXPORT int ph_qk_norm_rope_kv_write(const void* qkv, int qkv_dtype, int splits, long long split_stride,
                                       const float* bias, const float* q_norm_w, const float* k_norm_w, float eps,
                                       const float* cos_sin, int n_rot, int max_pos, const int32_t* positions,
                                       const int32_t* slot_mapping, void* q_out, int q_dtype, void* k_base,
                                       void* v_base, int kv_dtype, long long page_stride, int page_size, int T,
                                       int HQ, int HKV, int D, int interleaved, const float* row_sumsq, int row_chunks,
                                       int row_width, float row_eps, int DV, float* v_first, const float* v_lambda, int v_mode,
                                       cudaStream_t stream) {
    if (!qkv || !positions || !q_out || T < 0 || HQ < 1 || HKV < 0 || D < 2 || splits < 1 || !valid_dtype(qkv_dtype) ||
        !valid_dtype(q_dtype) || !valid_dtype(kv_dtype))
        return fail(PH_ERR_ARG, "qk_norm_rope: bad arguments (T %d, HQ %d, HKV %d, D %d)", T, HQ, HKV, D);
    if (DV <= 0) DV = D;
    if (D > MAX_D || DV > MAX_D) return fail(PH_ERR_UNSUPPORTED, "qk_norm_rope: head_dim %d / %d exceeds the supported %d", D, DV, MAX_D);
    if (v_mode < 0 || v_mode > 2 || (v_mode && !v_first) || (v_mode == 2 && !v_lambda))
        return fail(PH_ERR_ARG, "qk_norm_rope: value mixing needs the step's first values (and its factor when it blends)");
    if (cos_sin && (n_rot < 2 || n_rot > D || (n_rot & 1) || max_pos < 1))
        return fail(PH_ERR_ARG, "qk_norm_rope: rotary width %d must be even and at most head_dim %d", n_rot, D);
    if (slot_mapping && (!k_base || !v_base || page_size < 1))
        return fail(PH_ERR_ARG, "qk_norm_rope: a cache write needs the pool and its page size");
    if (row_sumsq && (row_chunks < 1 || row_width < 1)) return fail(PH_ERR_ARG, "qk_norm_rope: a row factor needs its chunks and the row width");
    if (T == 0) return PH_OK;
    const RowFactor rf = {row_sumsq, row_chunks, row_width, row_eps};
    dim3 grid(T, (HQ + 2 * HKV + WARPS - 1) / WARPS);
    const bool fast = D == 128 && DV == D && (!cos_sin || n_rot == 128) && split_stride % 4 == 0 && (((uintptr_t)v_first) & 15) == 0 &&
                      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_base | (uintptr_t)v_base | (uintptr_t)bias |
                        (uintptr_t)q_norm_w | (uintptr_t)k_norm_w | (uintptr_t)cos_sin) & 15) == 0 && page_stride % 8 == 0;
    if (fast) {
        const int n_heads = HQ + 2 * HKV;
        // enough tokens to fill the device with warps that walk three pairs of heads each: the wide kernel
        const bool many = (long long)T * n_heads >= 16384 && page_stride % 8 == 0 && split_stride % 8 == 0;
        const dim3 fgrid(T, many ? (n_heads + WARPS * 6 - 1) / (WARPS * 6) : (n_heads + WARPS - 1) / WARPS);
#define LAUNCH_FAST(TI, TQ, TKV)                                                                                    \
    do {                                                                                                            \
        if (many)                                                                                                   \
            launch_overlapped(qk_norm_rope_d128_wide_kernel<TI, TQ, TKV, 3>, fgrid, dim3(WARPS * 32), 0, stream, (const TI*)qkv, \
                              splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, max_pos, positions,     \
                              slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, rf, \
                              interleaved, v_first, v_lambda, v_mode);                                               \
        else                                                                                                        \
            launch_overlapped(qk_norm_rope_d128_kernel<TI, TQ, TKV, 1>, fgrid, dim3(WARPS * 32), 0, stream, (const TI*)qkv, \
                              splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, max_pos, positions,     \
                              slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, rf, \
                              interleaved, v_first, v_lambda, v_mode);                                               \
    } while (0)
        PH_DISPATCH(qkv_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH_FAST(TI, TQ, TKV))));
#undef LAUNCH_FAST
        return check_launch("qk_norm_rope");
    }
#define LAUNCH(TI, TQ, TKV)                                                                                       \
    qk_norm_rope_kernel<TI, TQ, TKV><<<grid, WARPS * 32, 0, stream>>>(                                            \
        (const TI*)qkv, splits, split_stride, bias, q_norm_w, k_norm_w, eps, cos_sin, n_rot, max_pos, positions,  \
        slot_mapping, (TQ*)q_out, (TKV*)k_base, (TKV*)v_base, page_stride, page_size, HQ, HKV, D, interleaved, rf, DV,     \
        v_first, v_lambda, v_mode)
    PH_DISPATCH(qkv_dtype, TI, PH_DISPATCH(q_dtype, TQ, PH_DISPATCH(kv_dtype, TKV, LAUNCH(TI, TQ, TKV))));
#undef LAUNCH
    return check_launch("qk_norm_rope");
}
