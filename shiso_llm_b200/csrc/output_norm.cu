// Row kernels of layers that normalise what a sublayer gives back, and the polynomial activation.
//
//   norm_into   residual[t] += y[t] * rsqrt(mean(y[t]^2) + eps) * w   (float, in place), and, when
//               asked, the new residual row in the activation type: what the next sublayer reads.
//   polynorm    out[t] = a * N(z[t]) + b * N(z[t]^2) + c * N(z[t]^3) + e, powers taken element by
//               element, N(u) = u * rsqrt(mean(u^2) + eps) over the row.
//
// One block per row; statistics and the residual sum in float whatever the activation type.  A
// row's sums are formed in an order that depends on the row's width only.
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

// bfloat16 rows of a multiple of 8 entries: 16 bytes a thread and access.  The second pass
// reads the row again (from the cache it is still in) instead of holding it in registers, so any
// width runs.

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(words[i] << 16);
        v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return *reinterpret_cast<uint4*>(h);
}

__global__ void norm_into_vec_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ y, const float* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[33];
    pdl_begin();
    const int pieces = hidden >> 3;
    const uint4* src = reinterpret_cast<const uint4*>(y + (size_t)blockIdx.x * hidden);
    float4* r = reinterpret_cast<float4*>(residual + (size_t)blockIdx.x * hidden);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
        float v[8];
        unpack8(src[i], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
        float v[8];
        unpack8(src[i], v);
        const float4 r0 = r[2 * i], r1 = r[2 * i + 1], w0 = w4[2 * i], w1 = w4[2 * i + 1];
        const float old[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = old[e] + v[e] * inv * ws[e];
        r[2 * i] = make_float4(v[0], v[1], v[2], v[3]);
        r[2 * i + 1] = make_float4(v[4], v[5], v[6], v[7]);
        if (out) reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * hidden)[i] = pack8(v);
    }
}

__global__ void polynorm_vec_kernel(const __nv_bfloat16* __restrict__ z, long long z_ld, const float* __restrict__ coefficients,
                                    __nv_bfloat16* __restrict__ out, int width, float eps) {
    __shared__ float scratch[33];
    pdl_begin();
    const int pieces = width >> 3;
    const uint4* src = reinterpret_cast<const uint4*>(z + (size_t)blockIdx.x * z_ld);
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
        float v[8];
        unpack8(src[i], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v2 = v[e] * v[e];
            s2 += v2;
            s4 += v2 * v2;
            s6 += v2 * v2 * v2;
        }
    }
    s2 = block_sum(s2, scratch);
    s4 = block_sum(s4, scratch);
    s6 = block_sum(s6, scratch);
    const float a = coefficients[0] * rsqrtf(s2 / (float)width + eps);
    const float b = coefficients[1] * rsqrtf(s4 / (float)width + eps);
    const float c = coefficients[2] * rsqrtf(s6 / (float)width + eps);
    const float e0 = coefficients[3];
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * width);
    for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
        float v[8];
        unpack8(src[i], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = a * v[e] + b * (v[e] * v[e]) + c * (v[e] * v[e] * v[e]) + e0;
        dst[i] = pack8(v);
    }
}

int block_for(int width) { return width >= 2048 ? 512 : (width >= 512 ? 256 : 128); }
int vec_block_for(int width) { return width >= 8192 ? 512 : (width >= 2048 ? 256 : 128); }
bool aligned16(const void* a, const void* b, const void* c, const void* d) {
    return !(((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) & 15);
}

}  // namespace

SHISO_API int shiso_norm_into(float* residual, const void* y, int act_dtype, const float* w, void* out, int tokens, int hidden, float eps,
                              cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (hidden <= 0) return SHISO_ERR_SHAPE;
    if (act_dtype == SHISO_F32)
        launch_kernel(norm_into_kernel<float>, tokens, block_for(hidden), 0, stream, residual, (const float*)y, w, (float*)out, hidden, eps);
    else if (act_dtype == SHISO_BF16 && hidden % 8 == 0 && aligned16(residual, y, w, out))
        launch_kernel(norm_into_vec_kernel, tokens, vec_block_for(hidden), 0, stream, residual, (const __nv_bfloat16*)y, w, (__nv_bfloat16*)out,
                      hidden, eps);
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
    else if (act_dtype == SHISO_BF16 && width % 8 == 0 && z_ld % 8 == 0 && aligned16(z, out, nullptr, nullptr))
        launch_kernel(polynorm_vec_kernel, tokens, vec_block_for(width), 0, stream, (const __nv_bfloat16*)z, z_ld, coefficients,
                      (__nv_bfloat16*)out, width, eps);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(polynorm_kernel<__nv_bfloat16>, tokens, block_for(width), 0, stream, (const __nv_bfloat16*)z, z_ld, coefficients,
                      (__nv_bfloat16*)out, width, eps);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
