// Layer norm (mean and variance, weight and bias) as a join of the residual stream, with
// the same fusion the RMS norm family has: the norm of a branch's output, the residual
// sum (times a constant multiplier) and the norm that feeds the next branch in one launch.
//
//   y == null:  x = N(h[rows]; w_next, b_next)       (x = h[rows] without w_next)
//   else:       b = sum_s y[s];  b = N(b; w_post, b_post) if w_post;  b *= mult;
//               h += b if add_residual;  v = h (or b);
//               x = N(v; w_next, b_next) if w_next, else x = v if x is given.
//   N(v; w, b) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w + b
//   (rms != 0:   v / sqrt(mean(v^2) + eps) * w + b, b optional).
//
// Statistics, the residual stream and the sums are 32-bit whatever the branch's and the
// output's dtype.  One CTA per row with the row in registers (EPT values per thread); the
// variance is taken from the deviations (two passes over registers), not from E[v^2].
#include "common.cuh"
#include <type_traits>

namespace {

struct NormSide {
    const float* w;            // [H] or null: this side is absent
    const float* b;            // [H] or null: no bias
    float eps;
};

template <int EPT>
__device__ __forceinline__ void normalise(float (&v)[EPT], const float (&w)[EPT],
                                          const float (&bv)[EPT], int H, float eps, int rms,
                                          float* red) {
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < EPT; ++k) s += v[k];               // lanes beyond H hold 0
        mean = block_sum(s, red) / (float)H;
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        const float d = i < H ? v[k] - mean : 0.f;
        v[k] = d;
        ss += d * d;
    }
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
    for (int k = 0; k < EPT; ++k) v[k] = v[k] * r * w[k] + bv[k];
}

template <typename TY, typename TX, int EPT>
__global__ void __launch_bounds__(1024)
layer_norm_join_kernel(float* __restrict__ h, const TY* __restrict__ y, int n_splits,
                       size_t split_stride, NormSide post, NormSide next, TX* __restrict__ x,
                       const int* __restrict__ rows, int H, float mult, int add_residual,
                       int rms) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    // weights and the row gather do not depend on the kernel before
    float wp[EPT], bp[EPT], wn[EPT], bn[EPT];
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        const bool in = i < H;
        wp[k] = (in && post.w) ? post.w[i] : 1.f;
        bp[k] = (in && post.b) ? post.b[i] : 0.f;
        wn[k] = (in && next.w) ? next.w[i] : 1.f;
        bn[k] = (in && next.b) ? next.b[i] : 0.f;
    }
    const size_t src = (size_t)(rows ? rows[r] : r) * H;
    const size_t dst = (size_t)r * H;
    pdl_wait();
    pdl_launch_next();
    float v[EPT];
    if (y) {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            float s = 0.f;
            if (i < H)
                for (int sp = 0; sp < n_splits; ++sp) s += to_f32(y[(size_t)sp * split_stride + src + i]);
            v[k] = s;
        }
        if (post.w) normalise<EPT>(v, wp, bp, H, post.eps, rms, red);
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            v[k] *= mult;
            if (add_residual && i < H) {
                v[k] += h[src + i];
                h[src + i] = v[k];
            }
            if (i >= H) v[k] = 0.f;
        }
    } else {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            v[k] = i < H ? h[src + i] : 0.f;
        }
    }
    if (next.w) normalise<EPT>(v, wn, bn, H, next.eps, rms, red);
    if (x) {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < H) x[dst + i] = from_f32<TX>(v[k]);
        }
    }
}

// Many rows (prompts), 32-bit branch input, width a multiple of 4: GT threads share a row
// (32: a warp per row and no block-wide barrier, for rows up to 2,048 values; 256: a CTA
// per row, for wider ones), 16-byte loads issued up front, the row in registers.
template <typename TX> struct LnPack4;
template <> struct LnPack4<float> {
    __device__ static void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct LnPack4<__nv_bfloat16> {
    __device__ static void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&a);
        u.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = u;
    }
};

template <int GT>
__device__ __forceinline__ float group_sum(float v, float* red) {
    if (GT == 32) return warp_sum(v);
    return block_sum(v, red);
}

template <int NV, int GT>
__device__ __forceinline__ void normalise4(float4 (&v)[NV], const NormSide& side, int H4, int H,
                                           int lane, int rms, float* red) {
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        mean = group_sum<GT>(s, red) / (float)H;
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (lane + GT * i < H4) {
            v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
    }
    const float r = 1.0f / sqrtf(group_sum<GT>(ss, red) / (float)H + side.eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int idx = lane + GT * i;
        if (idx < H4) {
            const float4 w = reinterpret_cast<const float4*>(side.w)[idx];
            float4 b = make_float4(0, 0, 0, 0);
            if (side.b) b = reinterpret_cast<const float4*>(side.b)[idx];
            v[i].x = v[i].x * r * w.x + b.x; v[i].y = v[i].y * r * w.y + b.y;
            v[i].z = v[i].z * r * w.z + b.z; v[i].w = v[i].w * r * w.w + b.w;
        }
    }
}

template <typename TX, int NV, int GT>
__global__ void __launch_bounds__(GT == 32 ? 128 : 256)
layer_norm_rows_kernel(float* __restrict__ h, const float* __restrict__ y, int n_splits,
                       size_t split_stride, NormSide post, NormSide next, TX* __restrict__ x,
                       int R, int H, float mult, int add_residual, int rms) {
    pdl_wait();
    pdl_launch_next();
    __shared__ float red[33];
    const int lane = GT == 32 ? (threadIdx.x & 31) : threadIdx.x;
    const int row = GT == 32 ? blockIdx.x * 4 + (threadIdx.x >> 5) : blockIdx.x;
    if (row >= R) return;                          // (whole warps, or nobody, leave)
    const int H4 = H >> 2;
    const size_t base = (size_t)row * H;
    float4 v[NV];
    if (y) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + GT * i;
            v[i] = idx < H4 ? reinterpret_cast<const float4*>(y + base)[idx]
                            : make_float4(0, 0, 0, 0);
        }
        for (int s = 1; s < n_splits; ++s) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int idx = lane + GT * i;
                if (idx < H4) {
                    const float4 t = reinterpret_cast<const float4*>(y + s * split_stride + base)[idx];
                    v[i].x += t.x; v[i].y += t.y; v[i].z += t.z; v[i].w += t.w;
                }
            }
        }
        if (post.w) normalise4<NV, GT>(v, post, H4, H, lane, rms, red);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + GT * i;
            // (the stream's row is asked for here, not up front: with both in registers the
            // widest rows spill, and a prompt has rows enough to hide the trip)
            float4 hv = make_float4(0, 0, 0, 0);
            if (add_residual && idx < H4) hv = reinterpret_cast<const float4*>(h + base)[idx];
            v[i].x = v[i].x * mult + hv.x; v[i].y = v[i].y * mult + hv.y;
            v[i].z = v[i].z * mult + hv.z; v[i].w = v[i].w * mult + hv.w;
            if (idx >= H4) v[i] = make_float4(0, 0, 0, 0);
            else if (add_residual) reinterpret_cast<float4*>(h + base)[idx] = v[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + GT * i;
            v[i] = idx < H4 ? reinterpret_cast<const float4*>(h + base)[idx]
                            : make_float4(0, 0, 0, 0);
        }
    }
    if (next.w) normalise4<NV, GT>(v, next, H4, H, lane, rms, red);
    if (x) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int idx = lane + GT * i;
            if (idx < H4) LnPack4<TX>::store(x + base + 4 * idx, v[i]);
        }
    }
}

template <typename TX>
bool launch_layer_norm_rows(float* h, const float* y, int n_splits, size_t split_stride,
                            NormSide post, NormSide next, TX* x, int R, int H, float mult,
                            int add_residual, int rms, cudaStream_t stream) {
#define AGV_LNR(NV, GT)                                                                         \
    agv_launch(layer_norm_rows_kernel<TX, NV, GT>, (unsigned)(GT == 32 ? (R + 3) / 4 : R),      \
               GT == 32 ? 128 : 256, 0, stream, h, y, n_splits, split_stride, post, next, x, R, \
               H, mult, add_residual, rms)
    if (H <= 2048) {
        const int nv = (H / 4 + 31) / 32;
        if (nv <= 2) AGV_LNR(2, 32);
        else if (nv <= 4) AGV_LNR(4, 32);
        else if (nv <= 8) AGV_LNR(8, 32);
        else if (nv <= 12) AGV_LNR(12, 32);
        else AGV_LNR(16, 32);
    } else {
        const int nv = (H / 4 + 255) / 256;
        if (nv <= 4) AGV_LNR(4, 256);
        else if (nv <= 8) AGV_LNR(8, 256);
        else if (nv <= 16) AGV_LNR(16, 256);
        else return false;
    }
#undef AGV_LNR
    return true;
}

template <typename TY, typename TX>
int launch_layer_norm(float* h, const void* y, int n_splits, size_t split_stride, NormSide post,
                      NormSide next, void* x, const int* rows, int R, int H, float mult,
                      int add_residual, int rms, cudaStream_t stream) {
    if constexpr (std::is_same<TY, float>::value) {
        // many rows of 32-bit input that move in 16-byte pieces
        auto al = [](const void* p) { return !p || agv_aligned(p, 16); };
        if (R > 64 && !rows && H % 4 == 0 && split_stride % 4 == 0 && al(h) && al(y) && al(x) &&
            al(post.w) && al(post.b) && al(next.w) && al(next.b)) {
            if (launch_layer_norm_rows<TX>(h, (const float*)y, n_splits, split_stride, post, next,
                                           (TX*)x, R, H, mult, add_residual, rms, stream)) {
                AGV_LAUNCH_OK("layer_norm_rows_kernel");
                return 0;
            }
        }
    }
    // about four values a thread, at most 1,024 threads
    int threads = ((H + 3) / 4 + 31) / 32 * 32;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    const int ept = (H + threads - 1) / threads;
#define AGV_LN(E)                                                                              \
    agv_launch(layer_norm_join_kernel<TY, TX, E>, (unsigned)R, threads, 0, stream, h,          \
               (const TY*)y, n_splits, split_stride, post, next, (TX*)x, rows, H, mult,        \
               add_residual, rms)
    if (ept <= 1) AGV_LN(1);
    else if (ept <= 2) AGV_LN(2);
    else if (ept <= 4) AGV_LN(4);
    else if (ept <= 8) AGV_LN(8);
    else AGV_LN(16);
#undef AGV_LN
    AGV_LAUNCH_OK("layer_norm_join_kernel");
    return 0;
}

}  // namespace

// h: [*, H] 32-bit residual stream.  y: [n_splits, R, H] branch output (y_dtype) or null.
// x: [R, H] output (x_dtype) or null.  rows: optional gather of h rows (only with y == null).
// w_post / b_post, w_next / b_next: 32-bit [H]; a bias may be null.  mult multiplies the
// (normed) branch before it joins the stream.  rms != 0: no mean is taken off.
AGV_API int agv_layer_norm_join(float* h, const void* y, int y_dtype, int n_splits,
                                long long split_stride, const float* w_post, const float* b_post,
                                const float* w_next, const float* b_next, void* x, int x_dtype,
                                const int* rows, int R, int H, float eps_post, float eps_next,
                                float mult, int add_residual, int rms, cudaStream_t stream) {
    AGV_REQUIRE(R >= 0 && H > 0, "layer_norm: bad sizes R=%d H=%d", R, H);
    AGV_REQUIRE(H <= 16 * 1024, "layer_norm: rows of %d values exceed the %d this kernel keeps in "
                "registers", H, 16 * 1024);
    AGV_REQUIRE(y || (x && h), "layer_norm: without a branch input, h and x are needed");
    AGV_REQUIRE(!y || n_splits >= 1, "layer_norm: n_splits must be >= 1");
    AGV_REQUIRE(!(y && rows), "layer_norm: row gather is only for the plain norm");
    AGV_REQUIRE(!add_residual || h, "layer_norm: the residual sum needs h");
    AGV_REQUIRE(!w_next || x, "layer_norm: w_next given without an output");
    AGV_REQUIRE((w_post || !b_post) && (w_next || !b_next), "layer_norm: a bias without a weight");
    if (R == 0) return 0;
    NormSide post{w_post, b_post, eps_post}, next{w_next, b_next, eps_next};
#define AGV_LN_CASE(TY, TX)                                                                     \
    return launch_layer_norm<TY, TX>(h, y, n_splits, (size_t)split_stride, post, next, x, rows, \
                                     R, H, mult, add_residual, rms, stream)
    const int yd = y ? y_dtype : AGV_F32;
    const int xd = x ? x_dtype : AGV_F32;
    if (yd == AGV_F32 && xd == AGV_F32) AGV_LN_CASE(float, float);
    if (yd == AGV_F32 && xd == AGV_BF16) AGV_LN_CASE(float, __nv_bfloat16);
    if (yd == AGV_BF16 && xd == AGV_BF16) AGV_LN_CASE(__nv_bfloat16, __nv_bfloat16);
    if (yd == AGV_BF16 && xd == AGV_F32) AGV_LN_CASE(__nv_bfloat16, float);
#undef AGV_LN_CASE
    return agv_fail(-1, "layer_norm: unknown dtypes y=%d x=%d", y_dtype, x_dtype);
}

// logits <- cap * tanh(logits / cap), in place, 32-bit.
namespace {
__global__ void soft_cap_kernel(float* __restrict__ z, long long n, float cap, float inv_cap) {
    pdl_wait();
    pdl_launch_next();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        z[i] = cap * tanhf(z[i] * inv_cap);
}
}  // namespace

AGV_API int agv_soft_cap(float* z, long long n, float cap, cudaStream_t stream) {
    AGV_REQUIRE(n >= 0 && cap > 0.f, "soft_cap: needs a positive cap");
    if (n == 0) return 0;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    agv_launch(soft_cap_kernel, (unsigned)blocks, 256, 0, stream, z, n, cap, 1.0f / cap);
    AGV_LAUNCH_OK("soft_cap_kernel");
    return 0;
}
