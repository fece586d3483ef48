// Row kernels of layers that normalise what a sublayer gives back, and the polynomial activation.
//
//   norm_into   residual[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w   (float, in place), and, when
//               asked, the new residual row in the activation type: what the next sublayer reads.
//   polynorm    out[t] = a * N(z[t]) + b * N(z[t]^2) + c * N(z[t]^3) + e, powers taken element by
//               element, N(u) = u * rsqrt(mean(u^2) + eps) over the row.
//
// One block per row; statistics and the residual sum in float whatever the activation type.  A
// row's sums are formed in an order that depends on the block size only.
#include "common.cuh"

namespace {

template <typename AT>
__global__ void norm_into_kernel(float* __restrict__ residual, const AT* __restrict__ y, const float* __restrict__ w, AT* __restrict__ out,
                                 int hidden, float eps) {
    __shared__ float scratch[33];
    pdl_begin();
    const AT* src = y + (size_t)blockIdx.x * hidden;
    float* r = residual + (size_t)blockIdx.x * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_f32(src[i]);
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = r[i] + to_f32(src[i]) * inv * w[i];
        r[i] = v;
        if (out) out[(size_t)blockIdx.x * hidden + i] = from_f32<AT>(v);
    }
}

template <typename AT>
__global__ void polynorm_kernel(const AT* __restrict__ z, long long z_ld, const float* __restrict__ coefficients, AT* __restrict__ out,
                                int width, float eps) {
    __shared__ float scratch[33];
    pdl_begin();
    const AT* src = z + (size_t)blockIdx.x * z_ld;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32(src[i]);
        const float v2 = v * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v2 * v2 * v2;
    }
    s2 = block_sum(s2, scratch);
    s4 = block_sum(s4, scratch);
    s6 = block_sum(s6, scratch);
    const float a = coefficients[0] * rsqrtf(s2 / (float)width + eps);
    const float b = coefficients[1] * rsqrtf(s4 / (float)width + eps);
    const float c = coefficients[2] * rsqrtf(s6 / (float)width + eps);
    const float e = coefficients[3];
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32(src[i]);
        out[(size_t)blockIdx.x * width + i] = from_f32<AT>(a * v + b * (v * v) + c * (v * v * v) + e);
    }
}

int block_for(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }

}  // namespace

SHISO_API int shiso_norm_into(float* residual, const void* y, int act_dtype, const float* w, void* out, int tokens, int hidden, float eps,
                              cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (hidden <= 0) return SHISO_ERR_SHAPE;
    if (act_dtype == SHISO_F32)
        launch_kernel(norm_into_kernel<float>, tokens, block_for(hidden), 0, stream, residual, (const float*)y, w, (float*)out, hidden, eps);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(norm_into_kernel<__nv_bfloat16>, tokens, block_for(hidden), 0, stream, residual, (const __nv_bfloat16*)y, w,
                      (__nv_bfloat16*)out, hidden, eps);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

SHISO_API int shiso_polynorm(const void* z, long long z_ld, int act_dtype, const float* coefficients, void* out, int tokens, int width,
                             float eps, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (width <= 0) return SHISO_ERR_SHAPE;
    if (act_dtype == SHISO_F32)
        launch_kernel(polynorm_kernel<float>, tokens, block_for(width), 0, stream, (const float*)z, z_ld, coefficients, (float*)out, width, eps);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(polynorm_kernel<__nv_bfloat16>, tokens, block_for(width), 0, stream, (const __nv_bfloat16*)z, z_ld, coefficients,
                      (__nv_bfloat16*)out, width, eps);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
