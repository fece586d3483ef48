// Row kernels of a residual stream whose norm has no statistics, and of attention heads that are
// normalised together.
//
// add_dyt_kernel:      x = residual (+ up to two block outputs), stored back; out = tanh(alpha x) * w + b.
// stream_add_kernel:   out = residual + up to three blocks of rows (each float or bfloat16) + one vector
//                      that is the same for every row; out may be the residual itself.
// gate_rows_kernel:    x *= sigmoid(gate), entry by entry, in place.
// glu_act_kernel:      the gated pair of a feed-forward over rows [gate | up]: silu(g) u, the tanh form
//                      of gelu(g) u, or min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1).
// joined_norm_store:   rows [q | k | (v) | ..]: one RMS norm over all query columns together and one
//                      over all key columns, each with a weight per column; the queries times a
//                      temperature 1 + coef * ln(floor((p + 1) / every) + 1) of the row's position p,
//                      written back in place; normed keys to the paged key cache; to the value cache
//                      the value columns, or (values_from_keys) the key columns as they came.
//
// Everything is evaluated in float with the library's tanhf, expf and logf, whatever the row type.
#include "common.cuh"

enum { GLU_SILU = 0, GLU_GELU_TANH = 1, GLU_SWISH_CLAMPED = 2 };

__device__ __forceinline__ float glu_pair(float g, float u, int act, float limit) {
    if (act == GLU_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    if (act == GLU_SWISH_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return g / (1.0f + expf(-g)) * u;
}

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
    return dtype == SHISO_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// --------------------------------------------------------------------------- tanh norm

// Loads and stores of N neighbouring entries at once (N = 1, 4 or 8 as the alignment allows).
template <int N> __device__ __forceinline__ void load_n(const float* p, float* v) {
    if constexpr (N == 1) {
        v[0] = p[0];
    } else {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            const float4 q = *reinterpret_cast<const float4*>(p + i);
            v[i] = q.x, v[i + 1] = q.y, v[i + 2] = q.z, v[i + 3] = q.w;
        }
    }
}
template <int N> __device__ __forceinline__ void load_n(const __nv_bfloat16* p, float* v) {
    if constexpr (N == 1) {
        v[0] = __bfloat162float(p[0]);
    } else if constexpr (N == 4) {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&q.x), b = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
        v[0] = __low2float(a), v[1] = __high2float(a), v[2] = __low2float(b), v[3] = __high2float(b);
    } else {
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            v[2 * i] = __low2float(a), v[2 * i + 1] = __high2float(a);
        }
    }
}
template <int N> __device__ __forceinline__ void store_n(float* p, const float* v) {
    if constexpr (N == 1) {
        p[0] = v[0];
    } else {
#pragma unroll
        for (int i = 0; i < N; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
}
template <int N> __device__ __forceinline__ void store_n(__nv_bfloat16* p, const float* v) {
    if constexpr (N == 1) {
        p[0] = __float2bfloat16_rn(v[0]);
    } else {
        uint32_t w[N / 2];
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            const __nv_bfloat162 a = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&a);
        }
        if constexpr (N == 4) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
        else *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// One thread per N neighbouring columns of a row.
template <typename AT, int N>
__global__ void __launch_bounds__(256)
add_dyt_kernel(float* __restrict__ residual, const AT* __restrict__ d0, const AT* __restrict__ d1, const int* __restrict__ rows,
               const float* __restrict__ w, const float* __restrict__ b, float alpha, AT* __restrict__ out, int out_rows, int hidden) {
    pdl_begin();
    const int per_row = hidden / N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)out_rows * per_row) return;
    const int r = (int)(i / per_row), c = (int)(i % per_row) * N;
    const size_t src = (size_t)(rows ? rows[r] : r) * hidden + c;
    float x[N], d[N], wv[N], bv[N];
    load_n<N>(residual + src, x);
    if (d0) {
        load_n<N>(d0 + src, d);
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] += d[e];
    }
    if (d1) {
        load_n<N>(d1 + src, d);
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] += d[e];
    }
    if (!rows && (d0 || d1)) store_n<N>(residual + src, x);
    load_n<N>(w + c, wv);
    load_n<N>(b + c, bv);
#pragma unroll
    for (int e = 0; e < N; ++e) x[e] = tanhf(alpha * x[e]) * wv[e] + bv[e];
    store_n<N>(out + (size_t)r * hidden + c, x);
}

// residual float [T, hidden]; d0, d1: block outputs in the output type, or null; rows: the rows
// wanted (the residual is then left alone), or null for all of them (the sum is stored back).
SHISO_API int shiso_add_dyt(float* residual, const void* d0, const void* d1, const int* rows, const float* w, const float* b,
                            float alpha, void* out, int out_dtype, int out_rows, int hidden, cudaStream_t stream) {
    if (out_rows <= 0 || hidden <= 0) return SHISO_OK;
    const bool aligned = ((((uintptr_t)residual) | ((uintptr_t)d0) | ((uintptr_t)d1) | ((uintptr_t)w) | ((uintptr_t)b) | ((uintptr_t)out)) & 15) == 0;
    const int n = !aligned ? 1 : (out_dtype == SHISO_BF16 && hidden % 8 == 0) ? 8 : hidden % 4 == 0 ? 4 : 1;
    const unsigned blocks = ceil_div_u((long long)out_rows * (hidden / n), 256);
#define DYT_GO(AT, N)                                                                                                  \
    launch_kernel(add_dyt_kernel<AT, N>, blocks, 256, 0, stream, residual, (const AT*)d0, (const AT*)d1, rows, w, b, alpha, \
                  (AT*)out, out_rows, hidden)
    if (out_dtype == SHISO_F32) {
        if (n == 4) DYT_GO(float, 4);
        else DYT_GO(float, 1);
    } else if (out_dtype == SHISO_BF16) {
        if (n == 8) DYT_GO(__nv_bfloat16, 8);
        else if (n == 4) DYT_GO(__nv_bfloat16, 4);
        else DYT_GO(__nv_bfloat16, 1);
    } else {
        return SHISO_ERR_DTYPE;
    }
#undef DYT_GO
    return launch_status();
}

// --------------------------------------------------------------------------- rows added to the stream

struct StreamAddArgs {
    const float* residual;
    float* out;
    const void* d[3];
    int dtype[3];
    const float* vector;  // [hidden] or null
    long long total;
    int hidden;
};

__global__ void __launch_bounds__(256) stream_add_kernel(const StreamAddArgs a) {
    pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    float x = a.residual[i];
#pragma unroll
    for (int j = 0; j < 3; ++j)
        if (a.d[j]) x += load_as_f32(a.d[j], a.dtype[j], (size_t)i);
    if (a.vector) x += a.vector[i % a.hidden];
    a.out[i] = x;
}

SHISO_API int shiso_stream_add(const float* residual, float* out, const void* d0, int d0_dtype, const void* d1, int d1_dtype,
                               const void* d2, int d2_dtype, const float* vector, int tokens, int hidden, cudaStream_t stream) {
    if (tokens <= 0 || hidden <= 0) return SHISO_OK;
    StreamAddArgs a = {residual, out, {d0, d1, d2}, {d0_dtype, d1_dtype, d2_dtype}, vector, (long long)tokens * hidden, hidden};
    for (int j = 0; j < 3; ++j)
        if (a.d[j] && a.dtype[j] != SHISO_F32 && a.dtype[j] != SHISO_BF16) return SHISO_ERR_DTYPE;
    launch_kernel(stream_add_kernel, ceil_div_u(a.total, 256), 256, 0, stream, a);
    return launch_status();
}

// --------------------------------------------------------------------------- gated pairs

template <typename AT>
__global__ void __launch_bounds__(256)
glu_act_kernel(const AT* __restrict__ gate_up, AT* __restrict__ out, int inter, long long total, int act, float limit) {
    pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / inter;
    const int c = (int)(i % inter);
    const AT* row = gate_up + (size_t)t * 2 * inter;
    out[i] = from_f32<AT>(glu_pair(to_f32(row[c]), to_f32(row[inter + c]), act, limit));
}

SHISO_API int shiso_glu_act(const void* gate_up, void* out, int act_dtype, int tokens, int inter, int act, float limit,
                            cudaStream_t stream) {
    if (tokens <= 0 || inter <= 0) return SHISO_OK;
    if (act < GLU_SILU || act > GLU_SWISH_CLAMPED) return SHISO_ERR_SHAPE;
    const long long total = (long long)tokens * inter;
    const unsigned blocks = ceil_div_u(total, 256);
    if (act_dtype == SHISO_F32)
        launch_kernel(glu_act_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, total, act, limit);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(glu_act_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter,
                      total, act, limit);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

// --------------------------------------------------------------------------- a gate per entry

// x[t, c] *= sigmoid(gate[t, c]) in place; rows of x and of the gate have their own strides.
template <typename AT, int N>
__global__ void __launch_bounds__(256)
gate_rows_kernel(AT* __restrict__ x, long long x_ld, const AT* __restrict__ gate, long long gate_ld, int tokens, int cols) {
    pdl_begin();
    const int per_row = cols / N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * per_row) return;
    const int t = (int)(i / per_row), c = (int)(i % per_row) * N;
    float v[N], g[N];
    load_n<N>(x + (size_t)t * x_ld + c, v);
    load_n<N>(gate + (size_t)t * gate_ld + c, g);
#pragma unroll
    for (int e = 0; e < N; ++e) v[e] *= 1.0f / (1.0f + expf(-g[e]));
    store_n<N>(x + (size_t)t * x_ld + c, v);
}

SHISO_API int shiso_gate_rows(void* x, long long x_ld, const void* gate, long long gate_ld, int act_dtype, int tokens, int cols,
                              cudaStream_t stream) {
    if (tokens <= 0 || cols <= 0) return SHISO_OK;
    if (act_dtype == SHISO_F32) {
        const bool vec = cols % 4 == 0 && x_ld % 4 == 0 && gate_ld % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)gate)) & 15) == 0;
        const unsigned blocks = ceil_div_u((long long)tokens * (cols / (vec ? 4 : 1)), 256);
        if (vec) launch_kernel(gate_rows_kernel<float, 4>, blocks, 256, 0, stream, (float*)x, x_ld, (const float*)gate, gate_ld, tokens, cols);
        else launch_kernel(gate_rows_kernel<float, 1>, blocks, 256, 0, stream, (float*)x, x_ld, (const float*)gate, gate_ld, tokens, cols);
    } else if (act_dtype == SHISO_BF16) {
        const bool vec = cols % 8 == 0 && x_ld % 8 == 0 && gate_ld % 8 == 0 && ((((uintptr_t)x) | ((uintptr_t)gate)) & 15) == 0;
        const unsigned blocks = ceil_div_u((long long)tokens * (cols / (vec ? 8 : 1)), 256);
        if (vec)
            launch_kernel(gate_rows_kernel<__nv_bfloat16, 8>, blocks, 256, 0, stream, (__nv_bfloat16*)x, x_ld, (const __nv_bfloat16*)gate,
                          gate_ld, tokens, cols);
        else
            launch_kernel(gate_rows_kernel<__nv_bfloat16, 1>, blocks, 256, 0, stream, (__nv_bfloat16*)x, x_ld, (const __nv_bfloat16*)gate,
                          gate_ld, tokens, cols);
    } else {
        return SHISO_ERR_DTYPE;
    }
    return launch_status();
}

// --------------------------------------------------------------------------- heads normalised together

// One block per row.  Columns [0, q_cols) are the queries, [q_cols, q_cols + k_cols) the keys,
// v_cols columns from v_col on the values (v_col = q_cols when the values are the keys as they came).
// A thread takes N neighbouring columns at a time (N > 1: every extent and stride is a multiple of N
// and every pointer 16-byte aligned); the order of a row's sums depends on the block's size only.
template <typename AT, int N>
__global__ void __launch_bounds__(256)
joined_norm_store_kernel(AT* __restrict__ proj, long long ld, int q_cols, int k_cols, int v_col, int v_cols, const float* __restrict__ q_w,
                         const float* __restrict__ k_w, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                         const int* __restrict__ table, int table_width, AT* __restrict__ k_cache, AT* __restrict__ v_cache,
                         int page_size, float eps, float temp_coef, int temp_every) {
    pdl_begin();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    AT* row = proj + (size_t)t * ld;
    const int pos = positions[t];
    const int first = threadIdx.x * N, stride = blockDim.x * N;
    float v[N], w[N];
    float sq = 0.0f, sk = 0.0f;
    for (int i = first; i < q_cols; i += stride) {
        load_n<N>(row + i, v);
#pragma unroll
        for (int e = 0; e < N; ++e) sq += v[e] * v[e];
    }
    for (int i = first; i < k_cols; i += stride) {
        load_n<N>(row + q_cols + i, v);
#pragma unroll
        for (int e = 0; e < N; ++e) sk += v[e] * v[e];
    }
    float q_inv = rsqrtf(block_sum(sq, scratch) / (float)q_cols + eps);
    const float k_inv = rsqrtf(block_sum(sk, scratch) / (float)k_cols + eps);
    if (temp_every > 0) q_inv *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    const int page = table[(size_t)seq_of_token[t] * table_width + pos / page_size];
    if (page >= 0) {
        const size_t at = (size_t)page * page_size + pos % page_size;
        AT* k_dst = k_cache + at * k_cols;
        AT* v_dst = v_cache + at * v_cols;
        for (int i = first; i < k_cols; i += stride) {
            load_n<N>(row + q_cols + i, v);
            load_n<N>(k_w + i, w);
#pragma unroll
            for (int e = 0; e < N; ++e) v[e] = v[e] * k_inv * w[e];
            store_n<N>(k_dst + i, v);
        }
        for (int i = first; i < v_cols; i += stride) {  // the values as they stand: a copy
            load_n<N>(row + v_col + i, v);
            store_n<N>(v_dst + i, v);
        }
    }
    for (int i = first; i < q_cols; i += stride) {
        load_n<N>(row + i, v);
        load_n<N>(q_w + i, w);
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = v[e] * q_inv * w[e];
        store_n<N>(row + i, v);
    }
}

SHISO_API int shiso_joined_norm_store(void* proj, long long ld, int act_dtype, int q_cols, int k_cols, int v_col, int v_cols,
                                      const float* q_w, const float* k_w, const int* positions, const int* seq_of_token,
                                      const int* table, int table_width, void* k_cache, void* v_cache, int tokens, int page_size,
                                      float eps, float temp_coef, int temp_every, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (q_cols <= 0 || k_cols <= 0 || v_cols <= 0 || v_col < q_cols || page_size <= 0 || temp_every < 0) return SHISO_ERR_SHAPE;
    const int n = act_dtype == SHISO_BF16 ? 8 : 4;
    const bool wide = q_cols % n == 0 && k_cols % n == 0 && v_col % n == 0 && v_cols % n == 0 && ld % n == 0 &&
                      ((((uintptr_t)proj) | ((uintptr_t)q_w) | ((uintptr_t)k_w) | ((uintptr_t)k_cache) | ((uintptr_t)v_cache)) & 15) == 0;
    const int threads = q_cols >= (wide ? 1024 * n / 2 : 1024) ? 256 : 128;
#define JOINED_GO(AT, N)                                                                                                       \
    launch_kernel(joined_norm_store_kernel<AT, N>, tokens, threads, 0, stream, (AT*)proj, ld, q_cols, k_cols, v_col, v_cols, q_w, k_w, \
                  positions, seq_of_token, table, table_width, (AT*)k_cache, (AT*)v_cache, page_size, eps, temp_coef, temp_every)
    if (act_dtype == SHISO_F32) {
        if (wide) JOINED_GO(float, 4);
        else JOINED_GO(float, 1);
    } else if (act_dtype == SHISO_BF16) {
        if (wide) JOINED_GO(__nv_bfloat16, 8);
        else JOINED_GO(__nv_bfloat16, 1);
    } else {
        return SHISO_ERR_DTYPE;
    }
#undef JOINED_GO
    return launch_status();
}
