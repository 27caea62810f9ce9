// Layer norm with weight and bias, the gated residual with a norm behind the sublayer, the weighted average of the
// residual streams of all layers so far, and element-wise activations. Statistics, gates and sums are 32-bit in
// every engine dtype; a row's result depends only on the row (one warp per row, a lane adds in index order, the
// warp's sum is a fixed butterfly), never on how many rows the call has.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int ROWS_PER_BLOCK = 4;

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// y[r, :] = (x[src, :] - mean) / sqrt(var + eps) * w + b, var = mean of the squared deviations.
template <typename TY>
__global__ void __launch_bounds__(32 * ROWS_PER_BLOCK)
layernorm_kernel(const float* x, const int* __restrict__ row_idx, const void* __restrict__ w, int w_dtype,
                 const void* __restrict__ b, int b_dtype, TY* __restrict__ y, int rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* src = x + (size_t)(row_idx ? row_idx[r] : r) * d;
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s += src[i];
    const float mean = bl_warp_sum(s) / (float)d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { const float c = src[i] - mean; ss += c * c; }
    const float inv = 1.0f / sqrtf(bl_warp_sum(ss) / (float)d + eps);
    TY* dst = y + (size_t)r * d;
    for (int i = lane; i < d; i += 32)
        bl_store(dst + i, (src[i] - mean) * inv * bl_load_any(w, w_dtype, i) + (b ? bl_load_any(b, b_dtype, i) : 0.f));
}

// x[r, :] += LN(sub[r, :] * sigmoid(gate[r, :])) * w + b: the gate on a sublayer's result, the norm behind the
// sublayer and the residual sum in one pass. gate may be null (no gate) and has its own row stride.
__global__ void __launch_bounds__(32 * ROWS_PER_BLOCK)
gated_norm_residual_kernel(float* x, const float* sub, const float* gate, int ld_gate, const void* __restrict__ w,
                           int w_dtype, const void* __restrict__ b, int b_dtype, int rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* s_row = sub + (size_t)r * d;
    const float* g_row = gate ? gate + (size_t)r * ld_gate : nullptr;
    auto gated = [&](int i) { return g_row ? s_row[i] * sigmoidf_(g_row[i]) : s_row[i]; };
    float s = 0.f;
    for (int i = lane; i < d; i += 32) s += gated(i);
    const float mean = bl_warp_sum(s) / (float)d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { const float c = gated(i) - mean; ss += c * c; }
    const float inv = 1.0f / sqrtf(bl_warp_sum(ss) / (float)d + eps);
    float* dst = x + (size_t)r * d;
    for (int i = lane; i < d; i += 32)
        dst[i] += (gated(i) - mean) * inv * bl_load_any(w, w_dtype, i) + (b ? bl_load_any(b, b_dtype, i) : 0.f);
}

// out[e] = sum_j c[j] * streams[j * stride + e], j ascending.
__global__ void depth_mix_kernel(const float* streams, size_t stride, const void* __restrict__ c, int c_dtype, int n,
                                 float* out, size_t count) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) acc = fmaf(bl_load_any(c, c_dtype, j), streams[(size_t)j * stride + e], acc);
        out[e] = acc;
    }
}

template <typename TI, typename TO, int ACT>
__global__ void activation_kernel(const TI* x, TO* y, size_t count) {
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < count; e += (size_t)gridDim.x * blockDim.x) {
        const float v = bl_load(x + e);
        float o;
        if (ACT == BL_ACT_GELU_ERF) o = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
        else if (ACT == BL_ACT_GELU_TANH) o = 0.5f * v * (1.0f + tanhf(0.79788456080286535588f * (v + 0.044715f * v * v * v)));
        else o = bl_silu(v);
        bl_store(y + e, o);
    }
}

int grid_for(size_t count, int threads) {
    size_t b = (count + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

extern "C" int bl_layernorm(const float* x, const int* row_idx, const void* w, int w_dtype, const void* b, int b_dtype,
                            void* y, int y_dtype, int rows, int d, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0) BL_FAIL("bl_layernorm: bad width %d", d);
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
    if (y_dtype == BL_F32)
        layernorm_kernel<float><<<blocks, 32 * ROWS_PER_BLOCK, 0, s>>>(x, row_idx, w, w_dtype, b, b_dtype, (float*)y, rows, d, eps);
    else if (y_dtype == BL_BF16)
        layernorm_kernel<__nv_bfloat16><<<blocks, 32 * ROWS_PER_BLOCK, 0, s>>>(x, row_idx, w, w_dtype, b, b_dtype,
                                                                                 (__nv_bfloat16*)y, rows, d, eps);
    else
        BL_FAIL("bl_layernorm: unknown output dtype %d", y_dtype);
    BL_CHECK_LAUNCH("bl_layernorm");
    return 0;
}

extern "C" int bl_gated_norm_residual(float* x, const float* sub, const float* gate, int ld_gate, const void* w, int w_dtype,
                                      const void* b, int b_dtype, int rows, int d, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (d <= 0 || (gate && ld_gate < d)) BL_FAIL("bl_gated_norm_residual: bad width %d or gate stride %d", d, ld_gate);
    const int blocks = (rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
    gated_norm_residual_kernel<<<blocks, 32 * ROWS_PER_BLOCK, 0, (cudaStream_t)stream>>>(x, sub, gate, ld_gate, w, w_dtype, b,
                                                                                         b_dtype, rows, d, eps);
    BL_CHECK_LAUNCH("bl_gated_norm_residual");
    return 0;
}

extern "C" int bl_depth_mix(const float* streams, long long stride, const void* coeffs, int c_dtype, int n, float* out,
                            long long count, void* stream) {
    if (count <= 0) return 0;
    if (n <= 0 || stride < count) BL_FAIL("bl_depth_mix: %d streams with stride %lld for %lld values", n, stride, count);
    depth_mix_kernel<<<grid_for((size_t)count, 256), 256, 0, (cudaStream_t)stream>>>(streams, (size_t)stride, coeffs, c_dtype, n,
                                                                                     out, (size_t)count);
    BL_CHECK_LAUNCH("bl_depth_mix");
    return 0;
}

extern "C" int bl_activation(const void* x, int x_dtype, void* y, int y_dtype, long long count, int act, void* stream) {
    if (count <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int g = grid_for((size_t)count, 256);
    if (act != BL_ACT_SILU && act != BL_ACT_GELU_ERF && act != BL_ACT_GELU_TANH) BL_FAIL("bl_activation: unknown activation %d", act);
#define BL_GO3(TI, TO) do { \
        if (act == BL_ACT_GELU_ERF) activation_kernel<TI, TO, BL_ACT_GELU_ERF><<<g, 256, 0, s>>>((const TI*)x, (TO*)y, (size_t)count); \
        else if (act == BL_ACT_GELU_TANH) activation_kernel<TI, TO, BL_ACT_GELU_TANH><<<g, 256, 0, s>>>((const TI*)x, (TO*)y, (size_t)count); \
        else activation_kernel<TI, TO, BL_ACT_SILU><<<g, 256, 0, s>>>((const TI*)x, (TO*)y, (size_t)count); } while (0)
    if (x_dtype == BL_F32 && y_dtype == BL_F32) BL_GO3(float, float);
    else if (x_dtype == BL_F32 && y_dtype == BL_BF16) BL_GO3(float, __nv_bfloat16);
    else if (x_dtype == BL_BF16 && y_dtype == BL_BF16) BL_GO3(__nv_bfloat16, __nv_bfloat16);
    else BL_FAIL("bl_activation: unsupported dtypes %d -> %d", x_dtype, y_dtype);
#undef BL_GO3
    BL_CHECK_LAUNCH("bl_activation");
    return 0;
}
