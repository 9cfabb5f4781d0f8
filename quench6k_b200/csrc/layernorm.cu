// Layer norm with weight and bias over rows of the FP32 residual stream, in the three places a
// block with norms on both sides of a sublayer needs it, as one kernel:
//
//   1. "after":  h[row] += LN(y[row]; wa, ba)      y: a sublayer's FP32 result, or [splits, R, D] partial sums added in order
//   2. "plus":   h[row] += extra[row]              (the embedding output re-entering a repeated span of layers)
//   3. "before": out[r]  = T(LN(h[row]; w, b))     the next sublayer's input in the operand dtype
//
// Any subset may be asked for in one launch; 1 and 3 together close one sublayer and open the next
// with a single pass over the row.  LN(x) = (x - mean) / sqrt(var + eps) * w + b with the mean first
// and the variance as the mean of squared deviations from it, all in FP32, summed in a fixed order.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256) layernorm_kernel(float* h, const float* y, int splits, size_t split_stride, const float* wa,
                                                        const float* ba, const float* extra, const float* w, const float* b,
                                                        const int* rows, T* out, int D, float eps) {
    pdl_enter();
    extern __shared__ float row[];            // D floats
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t at = (size_t)(rows ? rows[r] : r) * D;
    float* hr = h + at;
    if (y) {
        float s = 0.0f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = y[at + i];
            for (int k = 1; k < splits; ++k) v += y[k * split_stride + at + i];
            row[i] = v;
            s += v;
        }
        const float mean = block_sum(s, red) / (float)D;
        float q = 0.0f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            const float d = row[i] - mean;
            q = fmaf(d, d, q);
        }
        const float inv = rsqrtf(block_sum(q, red) / (float)D + eps);
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = hr[i] + ((row[i] - mean) * inv * wa[i] + ba[i]);
            if (extra) v += extra[at + i];
            hr[i] = v;
            row[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            float v = hr[i];
            if (extra) {
                v += extra[at + i];
                hr[i] = v;
            }
            row[i] = v;
        }
    }
    if (!w) return;
    float s = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) s += row[i];
    const float mean = block_sum(s, red) / (float)D;
    float q = 0.0f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float d = row[i] - mean;
        q = fmaf(d, d, q);
    }
    const float inv = rsqrtf(block_sum(q, red) / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) out[(size_t)r * D + i] = from_f32<T>((row[i] - mean) * inv * w[i] + b[i]);
}

// The same with the row in registers (D a multiple of 4, at most 1024 * V4): one read of every input, 16-byte accesses.
template <typename T, int V4>
__global__ void __launch_bounds__(256) layernorm_reg_kernel(float* h, const float* y, int splits, size_t split_stride, const float* wa,
                                                            const float* ba, const float* extra, const float* w, const float* b,
                                                            const int* rows, T* out, int D, float eps) {
    pdl_enter();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t at = (size_t)(rows ? rows[r] : r) * D;
    float4 v[V4];
    bool has[V4];
#pragma unroll
    for (int j = 0; j < V4; ++j) has[j] = (threadIdx.x + 256 * j) * 4 < D;
    auto stats = [&](float& mean, float& inv) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < V4; ++j)
            if (has[j]) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
        mean = block_sum(s, red) / (float)D;
        float q = 0.0f;
#pragma unroll
        for (int j = 0; j < V4; ++j)
            if (has[j]) {
                const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
                q += fmaf(a0, a0, a1 * a1) + fmaf(a2, a2, a3 * a3);
            }
        inv = rsqrtf(block_sum(q, red) / (float)D + eps);
    };
    if (y) {
#pragma unroll
        for (int j = 0; j < V4; ++j)
            if (has[j]) {
                const size_t i = at + (threadIdx.x + 256 * j) * 4;
                v[j] = *reinterpret_cast<const float4*>(y + i);
                for (int k = 1; k < splits; ++k) {
                    const float4 o = *reinterpret_cast<const float4*>(y + k * split_stride + i);
                    v[j].x += o.x, v[j].y += o.y, v[j].z += o.z, v[j].w += o.w;
                }
            }
        float mean, inv;
        stats(mean, inv);
#pragma unroll
        for (int j = 0; j < V4; ++j)
            if (has[j]) {
                const int c = (threadIdx.x + 256 * j) * 4;
                const float4 hv = *reinterpret_cast<const float4*>(h + at + c);
                const float4 ww = *reinterpret_cast<const float4*>(wa + c), bb = *reinterpret_cast<const float4*>(ba + c);
                float4 n;
                n.x = hv.x + ((v[j].x - mean) * inv * ww.x + bb.x), n.y = hv.y + ((v[j].y - mean) * inv * ww.y + bb.y);
                n.z = hv.z + ((v[j].z - mean) * inv * ww.z + bb.z), n.w = hv.w + ((v[j].w - mean) * inv * ww.w + bb.w);
                if (extra) {
                    const float4 e = *reinterpret_cast<const float4*>(extra + at + c);
                    n.x += e.x, n.y += e.y, n.z += e.z, n.w += e.w;
                }
                *reinterpret_cast<float4*>(h + at + c) = n;
                v[j] = n;
            }
    } else {
#pragma unroll
        for (int j = 0; j < V4; ++j)
            if (has[j]) {
                const int c = (threadIdx.x + 256 * j) * 4;
                v[j] = *reinterpret_cast<const float4*>(h + at + c);
                if (extra) {
                    const float4 e = *reinterpret_cast<const float4*>(extra + at + c);
                    v[j].x += e.x, v[j].y += e.y, v[j].z += e.z, v[j].w += e.w;
                    *reinterpret_cast<float4*>(h + at + c) = v[j];
                }
            }
    }
    if (!w) return;
    float mean, inv;
    stats(mean, inv);
#pragma unroll
    for (int j = 0; j < V4; ++j)
        if (has[j]) {
            const int c = (threadIdx.x + 256 * j) * 4;
            const float4 ww = *reinterpret_cast<const float4*>(w + c), bb = *reinterpret_cast<const float4*>(b + c);
            T* o = out + (size_t)r * D + c;
            o[0] = from_f32<T>((v[j].x - mean) * inv * ww.x + bb.x);
            o[1] = from_f32<T>((v[j].y - mean) * inv * ww.y + bb.y);
            o[2] = from_f32<T>((v[j].z - mean) * inv * ww.z + bb.z);
            o[3] = from_f32<T>((v[j].w - mean) * inv * ww.w + bb.w);
        }
}

}  // namespace

// h: FP32 [*, D], updated in place when y or extra is given.  y: FP32 [R, D] or [splits, R, D] (slices split_stride floats
// apart) or null; wa, ba: the weight and bias of the norm applied to y.  extra: FP32 like h, or null.  w, b, out: the norm
// whose result leaves in `dtype`, or null.  rows: int32 [R] picks the rows (only with y == null and extra == null).
Q6K_API int q6k_layernorm(float* h, const float* y, int splits, long long split_stride, const float* wa, const float* ba,
                          const float* extra, const float* w, const float* b, const int* rows, void* out, int R, int D, float eps,
                          int dtype, cudaStream_t st) {
    if (R == 0) return 0;
    Q6K_REQUIRE(R > 0 && D > 0 && D <= 48 * 1024 / 4, "layernorm: bad sizes R=%d D=%d (rows of at most 12288)", R, D);
    Q6K_REQUIRE(!y || (wa && ba && splits >= 1), "layernorm: a sublayer result needs the weight and bias of its norm");
    Q6K_REQUIRE(!rows || (!y && !extra), "layernorm: picked rows are only normalised, not updated");
    Q6K_REQUIRE(!w || (b && out), "layernorm: an output needs weight, bias and a buffer");
    const bool aligned = D % 4 == 0 && D <= 4096 && (!y || split_stride % 4 == 0);
#define LN_REG(V4)                                                                                                          \
    Q6K_DISPATCH(dtype, q6k_launch(layernorm_reg_kernel<T, V4>, dim3(R), 256, 0, st, h, y, splits, (size_t)split_stride, wa, ba, extra, w, \
                                   b, rows, (T*)out, D, eps););
    if (aligned && D <= 1024) { LN_REG(1) }
    else if (aligned && D <= 2048) { LN_REG(2) }
    else if (aligned) { LN_REG(4) }
    else
        Q6K_DISPATCH(dtype, q6k_launch(layernorm_kernel<T>, dim3(R), 256, (size_t)D * sizeof(float), st, h, y, splits, (size_t)split_stride,
                                       wa, ba, extra, w, b, rows, (T*)out, D, eps););
#undef LN_REG
    return q6k_check_launch("layernorm");
}
