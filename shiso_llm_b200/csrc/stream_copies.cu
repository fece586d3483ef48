// Row kernels of models that keep several copies of the residual stream and mix tokens with
// their predecessor: the hashed-pair embedding, the read/write of stream copies
// (hyper-connections) fused with the RMS norm, the token-shift blends, and a unary map.
//
// Everything here is float arithmetic on float streams; only the rows handed to a product are
// rounded to the activation type.
#include <type_traits>

#include "common.cuh"

// --------------------------------------------------------------------------- hashed-pair embedding

__device__ __forceinline__ int step_token(const int* ids, const int* feed_index, const int* fed_tokens, int t) {
    int id = ids[t];
    if (feed_index) {
        const int from = feed_index[t];
        if (from >= 0) id = fed_tokens[from];
    }
    return id;
}

// x_t = scale * E[id_t] + B[(id_{t-1} * mul_prev + id_t * mul_cur) mod buckets]; B[buckets] for a
// sequence's first token.  The previous token of a portion's first row is what the request's
// slot holds (token + 1).  The slots are written by the kernel below, after this one.
template <typename WT>
__global__ void embed_hashed_pair_kernel(const int* __restrict__ ids, const int* __restrict__ feed_index, const int* fed_tokens,
                                         const WT* __restrict__ table, const WT* __restrict__ pair_table,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                         const int* __restrict__ start_pos, const int* __restrict__ slots,
                                         const int* state, long long state_stride, float* __restrict__ out,
                                         int hidden, int vocab, float scale, int buckets, int mul_prev, int mul_cur) {
    pdl_begin();
    const int t = blockIdx.x;
    const int id = step_token(ids, feed_index, fed_tokens, t);
    const int s = seq_of_token[t];
    int prev = -1;
    if (t > q_start[s]) prev = step_token(ids, feed_index, fed_tokens, t - 1);
    else if (start_pos[s] > 0) prev = state[(long long)slots[s] * state_stride] - 1;
    const bool valid = id >= 0 && id < vocab;
    long long row = buckets;
    if (prev >= 0 && valid) row = ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    const WT* e = table + (size_t)(valid ? id : 0) * hidden;
    const WT* b = pair_table + (size_t)row * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = valid ? to_f32(e[i]) * scale + to_f32(b[i]) : 0.0f;
}

__global__ void store_last_token_kernel(const int* __restrict__ ids, const int* __restrict__ feed_index, const int* fed_tokens,
                                        const int* __restrict__ q_start, const int* __restrict__ slots, int* state,
                                        long long state_stride, int num_seqs) {
    pdl_begin();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= num_seqs) return;
    const int a = q_start[s], e = q_start[s + 1];
    if (e > a) state[(long long)slots[s] * state_stride] = step_token(ids, feed_index, fed_tokens, e - 1) + 1;
}

SHISO_API int shiso_embed_hashed_pair(const int* ids, const int* feed_index, const int* fed_tokens, const void* table,
                                      const void* pair_table, int table_dtype, const int* seq_of_token, const int* q_start,
                                      const int* start_pos, const int* slots, int* state, long long state_stride, float* out,
                                      int tokens, int num_seqs, int hidden, int vocab, float scale, int buckets, int mul_prev,
                                      int mul_cur, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if ((feed_index == nullptr) != (fed_tokens == nullptr) || buckets <= 0) return SHISO_ERR_SHAPE;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == SHISO_F32)
        launch_kernel(embed_hashed_pair_kernel<float>, tokens, threads, 0, stream, ids, feed_index, fed_tokens, (const float*)table,
                      (const float*)pair_table, seq_of_token, q_start, start_pos, slots, (const int*)state, state_stride, out,
                      hidden, vocab, scale, buckets, mul_prev, mul_cur);
    else if (table_dtype == SHISO_BF16)
        launch_kernel(embed_hashed_pair_kernel<__nv_bfloat16>, tokens, threads, 0, stream, ids, feed_index, fed_tokens,
                      (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table, seq_of_token, q_start, start_pos, slots,
                      (const int*)state, state_stride, out, hidden, vocab, scale, buckets, mul_prev, mul_cur);
    else
        return SHISO_ERR_DTYPE;
    launch_kernel(store_last_token_kernel, ceil_div_u(num_seqs, 128), 128, 0, stream, ids, feed_index, fed_tokens, q_start, slots,
                  state, state_stride, num_seqs);
    return launch_status();
}

// --------------------------------------------------------------------------- copies of the stream

constexpr int MAX_COPIES = 8;

// One block per token row.  With `y`: the copies become x_r' = sum_s mix[s, r] x_s + write[r] * y
// (stored to `dst` when given).  With `read`: u = sum_r read[r] x_r' is normalised,
// u * rsqrt(mean(u^2) + eps) * norm_w, into `normed`.  With `sum_out`: sum_r x_r'.  `src` has
// `copies` lanes `src_stride` floats apart (0: one stream stands for every copy).
template <typename AT>
__global__ void hyper_mix_kernel(const float* src, long long src_stride, const AT* __restrict__ y,
                                 const float* __restrict__ mix, const float* __restrict__ write, float* dst, long long dst_stride,
                                 const float* __restrict__ read, const float* __restrict__ norm_w, float eps,
                                 AT* __restrict__ normed, float* __restrict__ sum_out, int hidden, int copies) {
    extern __shared__ float row_u[];  // [hidden] when `read`
    __shared__ float scratch[33];
    __shared__ float s_mix[MAX_COPIES * MAX_COPIES], s_write[MAX_COPIES], s_read[MAX_COPIES];
    if (threadIdx.x < copies * copies && y) s_mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < copies) {
        if (y) s_write[threadIdx.x] = write[threadIdx.x];
        if (read) s_read[threadIdx.x] = read[threadIdx.x];
    }
    __syncthreads();
    pdl_begin();
    const size_t at = (size_t)blockIdx.x * hidden;
    float squares = 0.0f;
    // W neighbouring elements a thread: 4 (16-byte loads and stores of the float copies) where rows allow it
    auto walk = [&](auto width) {
        constexpr int W = decltype(width)::value;
        for (int i = threadIdx.x * W; i < hidden; i += blockDim.x * W) {
            float x[MAX_COPIES][W], nx[MAX_COPIES][W];
#pragma unroll
            for (int s = 0; s < MAX_COPIES; ++s) {
                if (s < copies) {
                    const float* p = src + (size_t)s * src_stride + at + i;
                    if (W == 4) {
                        const float4 v = *reinterpret_cast<const float4*>(p);
                        x[s][0] = v.x; x[s][W > 1 ? 1 : 0] = v.y; x[s][W > 2 ? 2 : 0] = v.z; x[s][W > 3 ? 3 : 0] = v.w;
                    } else {
                        x[s][0] = p[0];
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < W; ++e) x[s][e] = 0.0f;
                }
            }
            if (y) {
                float yy[W];
#pragma unroll
                for (int e = 0; e < W; ++e) yy[e] = to_f32(y[at + i + e]);
#pragma unroll
                for (int r = 0; r < MAX_COPIES; ++r) {
#pragma unroll
                    for (int e = 0; e < W; ++e) nx[r][e] = 0.0f;
                    if (r < copies) {
#pragma unroll
                        for (int e = 0; e < W; ++e) {
                            float v = 0.0f;
#pragma unroll
                            for (int s = 0; s < MAX_COPIES; ++s)
                                if (s < copies) v += s_mix[s * copies + r] * x[s][e];
                            nx[r][e] = v + s_write[r] * yy[e];
                        }
                        if (dst) {
                            float* p = dst + (size_t)r * dst_stride + at + i;
                            if (W == 4) *reinterpret_cast<float4*>(p) = make_float4(nx[r][0], nx[r][W > 1 ? 1 : 0], nx[r][W > 2 ? 2 : 0], nx[r][W > 3 ? 3 : 0]);
                            else p[0] = nx[r][0];
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < MAX_COPIES; ++r)
#pragma unroll
                    for (int e = 0; e < W; ++e) nx[r][e] = x[r][e];
            }
#pragma unroll
            for (int e = 0; e < W; ++e) {
                if (read) {
                    float u = 0.0f;
#pragma unroll
                    for (int r = 0; r < MAX_COPIES; ++r)
                        if (r < copies) u += s_read[r] * nx[r][e];
                    row_u[i + e] = u;
                    squares += u * u;
                }
                if (sum_out) {
                    float total = 0.0f;
#pragma unroll
                    for (int r = 0; r < MAX_COPIES; ++r)
                        if (r < copies) total += nx[r][e];
                    sum_out[at + i + e] = total;
                }
            }
        }
    };
    if (hidden % 4 == 0) walk(std::integral_constant<int, 4>{});
    else walk(std::integral_constant<int, 1>{});
    if (!read) return;
    const float scale = rsqrtf(block_sum(squares, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) normed[at + i] = from_f32<AT>(row_u[i] * scale * norm_w[i]);
}

SHISO_API int shiso_hyper_mix(const float* src, long long src_stride, const void* y, const float* mix, const float* write,
                              float* dst, long long dst_stride, const float* read, const float* norm_w, float eps, void* normed,
                              float* sum_out, int act_dtype, int tokens, int hidden, int copies, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (copies < 1 || copies > MAX_COPIES || hidden > 12000) return SHISO_ERR_SHAPE;
    if ((y != nullptr) != (mix != nullptr) || (y != nullptr) != (write != nullptr) || (read != nullptr) != (normed != nullptr))
        return SHISO_ERR_UNSUPPORTED;
    const int threads = hidden >= 2048 ? 256 : 128;
    const size_t smem = read ? (size_t)hidden * sizeof(float) : 0;
    if (act_dtype == SHISO_F32)
        launch_kernel(hyper_mix_kernel<float>, tokens, threads, smem, stream, src, src_stride, (const float*)y, mix, write, dst,
                      dst_stride, read, norm_w, eps, (float*)normed, sum_out, hidden, copies);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(hyper_mix_kernel<__nv_bfloat16>, tokens, threads, smem, stream, src, src_stride, (const __nv_bfloat16*)y, mix,
                      write, dst, dst_stride, read, norm_w, eps, (__nv_bfloat16*)normed, sum_out, hidden, copies);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

// --------------------------------------------------------------------------- token shift

// out[c, t, :] = h_t + (h_{t-1} - h_t) * mu[c, :] for c < blends, with h_{t-1} the row before in
// the same sequence, the request's stored row for a portion's first token, zeros at position 0.
template <typename AT>
__global__ void token_shift_blend_kernel(const AT* __restrict__ h, const float* __restrict__ mu, const float* state,
                                         long long state_stride, const int* __restrict__ seq_of_token,
                                         const int* __restrict__ q_start, const int* __restrict__ start_pos,
                                         const int* __restrict__ slots, AT* __restrict__ out, int tokens, int hidden, int blends) {
    pdl_begin();
    const int t = blockIdx.x;
    const int s = seq_of_token[t];
    const bool first = t == q_start[s];
    const bool none = first && start_pos[s] == 0;
    const float* kept = state + (long long)slots[s] * state_stride;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float cur = to_f32(h[(size_t)t * hidden + i]);
        const float prev = none ? 0.0f : (first ? kept[i] : to_f32(h[(size_t)(t - 1) * hidden + i]));
        const float diff = prev - cur;
        for (int c = 0; c < blends; ++c)
            out[((size_t)c * tokens + t) * hidden + i] = from_f32<AT>(cur + diff * mu[(size_t)c * hidden + i]);
    }
}

template <typename AT>
__global__ void store_last_row_kernel(const AT* __restrict__ h, float* state, long long state_stride,
                                      const int* __restrict__ q_start, const int* __restrict__ slots, int hidden) {
    pdl_begin();
    const int s = blockIdx.x;
    const int a = q_start[s], e = q_start[s + 1];
    if (e <= a) return;
    float* kept = state + (long long)slots[s] * state_stride;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) kept[i] = to_f32(h[(size_t)(e - 1) * hidden + i]);
}

SHISO_API int shiso_token_shift_blend(const void* h, int act_dtype, const float* mu, float* state, long long state_stride,
                                      const int* seq_of_token, const int* q_start, const int* start_pos, const int* slots,
                                      void* out, int tokens, int num_seqs, int hidden, int blends, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (act_dtype == SHISO_F32) {
        launch_kernel(token_shift_blend_kernel<float>, tokens, threads, 0, stream, (const float*)h, mu, (const float*)state,
                      state_stride, seq_of_token, q_start, start_pos, slots, (float*)out, tokens, hidden, blends);
        launch_kernel(store_last_row_kernel<float>, num_seqs, threads, 0, stream, (const float*)h, state, state_stride, q_start,
                      slots, hidden);
    } else if (act_dtype == SHISO_BF16) {
        launch_kernel(token_shift_blend_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (const __nv_bfloat16*)h, mu,
                      (const float*)state, state_stride, seq_of_token, q_start, start_pos, slots, (__nv_bfloat16*)out, tokens,
                      hidden, blends);
        launch_kernel(store_last_row_kernel<__nv_bfloat16>, num_seqs, threads, 0, stream, (const __nv_bfloat16*)h, state,
                      state_stride, q_start, slots, hidden);
    } else {
        return SHISO_ERR_DTYPE;
    }
    return launch_status();
}

// --------------------------------------------------------------------------- unary maps

enum { SHISO_UNARY_TANH = 0, SHISO_UNARY_SILU = 1, SHISO_UNARY_RELU2 = 2, SHISO_UNARY_COPY = 3 };  // relu2: the square of max(x, 0); copy: the value in the output's type

template <typename IT, typename OT>
__global__ void unary_kernel(const IT* __restrict__ x, OT* __restrict__ out, long long count, int kind) {
    pdl_begin();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
        const float v = to_f32(x[i]);
        float r;
        if (kind == SHISO_UNARY_TANH) r = tanhf(v);
        else if (kind == SHISO_UNARY_SILU) r = v / (1.0f + expf(-v));
        else if (kind == SHISO_UNARY_RELU2) r = v > 0.0f ? v * v : 0.0f;
        else r = v;
        out[i] = from_f32<OT>(r);
    }
}

SHISO_API int shiso_unary(const void* x, int in_dtype, void* out, int out_dtype, long long count, int kind, cudaStream_t stream) {
    if (count <= 0) return SHISO_OK;
    if (kind < SHISO_UNARY_TANH || kind > SHISO_UNARY_COPY) return SHISO_ERR_UNSUPPORTED;
    const unsigned blocks = (unsigned)((count + 255) / 256 < 4096 ? (count + 255) / 256 : 4096);
    if (in_dtype == SHISO_F32 && out_dtype == SHISO_F32)
        launch_kernel(unary_kernel<float, float>, blocks, 256, 0, stream, (const float*)x, (float*)out, count, kind);
    else if (in_dtype == SHISO_F32 && out_dtype == SHISO_BF16)
        launch_kernel(unary_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream, (const float*)x, (__nv_bfloat16*)out, count, kind);
    else if (in_dtype == SHISO_BF16 && out_dtype == SHISO_BF16)
        launch_kernel(unary_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x,
                      (__nv_bfloat16*)out, count, kind);
    else if (in_dtype == SHISO_BF16 && out_dtype == SHISO_F32)
        launch_kernel(unary_kernel<__nv_bfloat16, float>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, (float*)out, count, kind);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
