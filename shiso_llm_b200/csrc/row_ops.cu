// Row kernels of parallel layers and their mixers: layer norm fused with the residual sum of
// several block outputs, RMS norm in groups with a gate, the causal convolution of a
// state-space mixer, rotation of head columns, and the store of a latent cache row.
//
// Statistics, sums, angles and gates are float arithmetic whatever the activation type; rows
// handed to a product are rounded to the activation type once, on store.  Inputs may be column
// ranges of wider rows (a row stride in elements comes with every such pointer), so loads are
// scalar and coalesced across a warp.
#include "common.cuh"

// --------------------------------------------------------------------------- layer norm

// residual[row] (+ d1[row] + d2[row], stored back when rows == nullptr), then
// (x - mean) / sqrt(mean((x - mean)^2) + eps) * w.  One block per output row; the row is kept
// in shared memory so that the variance is taken from the deviations themselves.
template <typename AT>
__global__ void add_layernorm_kernel(float* __restrict__ residual, const AT* __restrict__ d1, const AT* __restrict__ d2,
                                     const int* __restrict__ rows, const float* __restrict__ w, AT* __restrict__ out,
                                     int hidden, float eps) {
    pdl_begin();
    __shared__ float scratch[33];
    extern __shared__ float row_cache[];
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = residual + (size_t)src * hidden;
    const AT* a = d1 ? d1 + (size_t)src * hidden : nullptr;
    const AT* b = d2 ? d2 + (size_t)src * hidden : nullptr;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = r[i];
        if (a) {
            float d = to_f32(a[i]);
            if (b) d += to_f32(b[i]);
            v += d;
            if (!rows) r[i] = v;
        }
        row_cache[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_cache[i] - mean;
        ss += d * d;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    AT* o = out + (size_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<AT>((row_cache[i] - mean) * inv * w[i]);
}

SHISO_API int shiso_add_layernorm(float* residual, const void* d1, const void* d2, const int* rows, const float* w, void* out,
                                  int act_dtype, int out_rows, int hidden, float eps, cudaStream_t stream) {
    if (out_rows <= 0) return SHISO_OK;
    if (hidden <= 0) return SHISO_ERR_SHAPE;
    if (d2 && !d1) return SHISO_ERR_UNSUPPORTED;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (smem > 200 * 1024) return SHISO_ERR_SHAPE;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    if (act_dtype == SHISO_F32) {
        auto k = add_layernorm_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(k, out_rows, threads, smem, stream, residual, (const float*)d1, (const float*)d2, rows, w, (float*)out, hidden, eps);
    } else if (act_dtype == SHISO_BF16) {
        auto k = add_layernorm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_kernel(k, out_rows, threads, smem, stream, residual, (const __nv_bfloat16*)d1, (const __nv_bfloat16*)d2, rows, w,
                      (__nv_bfloat16*)out, hidden, eps);
    } else {
        return SHISO_ERR_DTYPE;
    }
    return launch_status();
}

// --------------------------------------------------------------------------- RMS norm in groups, with a gate

enum { SHISO_GATE_NONE = 0, SHISO_GATE_SILU_BEFORE = 1, SHISO_GATE_SIGMOID_AFTER = 2 };

// One block per (row, group): the group's columns times silu(gate) (mode 1), divided by their
// root mean square, times w, times sigmoid(gate) (mode 2).
template <typename XT, typename AT>
__global__ void group_rmsnorm_kernel(const XT* __restrict__ x, long long x_ld, const AT* __restrict__ gate, long long gate_ld,
                                     const float* __restrict__ w, AT* __restrict__ out, int width, int groups, int mode, float eps) {
    pdl_begin();
    __shared__ float scratch[33];
    extern __shared__ float row_cache[];
    const int t = blockIdx.x / groups, g = blockIdx.x % groups;
    const int per = width / groups;
    const XT* xr = x + (size_t)t * x_ld + (size_t)g * per;
    const AT* gr = gate ? gate + (size_t)t * gate_ld + (size_t)g * per : nullptr;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        float v = to_f32(xr[i]);
        if (mode == SHISO_GATE_SILU_BEFORE) {
            const float z = to_f32(gr[i]);
            v *= z / (1.0f + expf(-z));
        }
        row_cache[i] = v;
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)per + eps);
    AT* o = out + (size_t)t * width + (size_t)g * per;
    const float* wg = w + (size_t)g * per;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        float v = row_cache[i] * inv * wg[i];
        if (mode == SHISO_GATE_SIGMOID_AFTER) v *= 1.0f / (1.0f + expf(-to_f32(gr[i])));
        o[i] = from_f32<AT>(v);
    }
}

SHISO_API int shiso_group_rmsnorm(const void* x, int x_dtype, long long x_ld, const void* gate, long long gate_ld, const float* w,
                                  void* out, int act_dtype, int tokens, int width, int groups, int mode, float eps,
                                  cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (width <= 0 || groups <= 0 || width % groups) return SHISO_ERR_SHAPE;
    if ((mode != SHISO_GATE_NONE) != (gate != nullptr)) return SHISO_ERR_UNSUPPORTED;
    const int per = width / groups;
    const size_t smem = (size_t)per * sizeof(float);
    if (smem > 200 * 1024) return SHISO_ERR_SHAPE;
    const int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    const unsigned blocks = (unsigned)tokens * groups;
#define SHISO_GRN(XT, AT)                                                                                                        \
    {                                                                                                                            \
        auto k = group_rmsnorm_kernel<XT, AT>;                                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                  \
        launch_kernel(k, blocks, threads, smem, stream, (const XT*)x, x_ld, (const AT*)gate, gate_ld, w, (AT*)out, width, groups, \
                      mode, eps);                                                                                                \
    }
    if (x_dtype == SHISO_F32 && act_dtype == SHISO_F32) SHISO_GRN(float, float)
    else if (x_dtype == SHISO_F32 && act_dtype == SHISO_BF16) SHISO_GRN(float, __nv_bfloat16)
    else if (x_dtype == SHISO_BF16 && act_dtype == SHISO_BF16) SHISO_GRN(__nv_bfloat16, __nv_bfloat16)
    else return SHISO_ERR_DTYPE;
#undef SHISO_GRN
    return launch_status();
}

// --------------------------------------------------------------------------- causal convolution per channel

#define SHISO_CONV_MAX_TAPS 8

#define SHISO_CONV_ROWS 8  // rows a thread walks with the window in registers

// y_t[c] = act(bias[c] + sum_j taps[c, j] * x_{t-(L-1)+j}[c]); inputs before a portion's first row
// come from the request's slot (its last L-1 inputs, oldest first, float; zeros for a new
// request).  A thread per (run of eight rows, channel): where the run lies in one sequence the
// window moves through registers (a row's inputs are read once, not once per tap; taps and window
// are kept at the END of arrays of the largest size, zeros before, so that every index is a
// constant); a run that crosses into another sequence takes its rows one by one.  The slot is
// read here and written by the kernel below.
template <typename AT>
__global__ void causal_conv_kernel(const AT* __restrict__ x, long long x_ld, const float* __restrict__ taps,
                                   const float* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                   const int* __restrict__ state_slots, AT* __restrict__ y, int tokens, int channels, int n_taps,
                                   int silu) {
    pdl_begin();
    constexpr int M = SHISO_CONV_MAX_TAPS;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int runs = (tokens + SHISO_CONV_ROWS - 1) / SHISO_CONV_ROWS;
    if (i >= (long long)runs * channels) return;
    const int run = (int)(i / channels), c = (int)(i % channels);
    const int t0 = run * SHISO_CONV_ROWS, t_end = min(t0 + SHISO_CONV_ROWS, tokens);
    const float b = bias ? bias[c] : 0.0f;
    const int off = M - n_taps;  // tap j sits at tp[off + j]: the current row's tap is always tp[M - 1]
    float tp[M];
#pragma unroll
    for (int k = 0; k < M; ++k) tp[k] = k >= off ? taps[(size_t)c * n_taps + (k - off)] : 0.0f;
    const int s0 = seq_of_token[t0];
    if (seq_of_token[t_end - 1] == s0) {
        const int first = q_start[s0];
        const float* slot = state + (size_t)state_slots[s0] * slot_stride;
        float w[M - 1];  // w[k], k >= off: the input n_taps - 1 - (k - off) rows before the current one
#pragma unroll
        for (int k = 0; k < M - 1; ++k) {
            w[k] = 0.0f;
            if (k >= off) {
                const int src = t0 - (n_taps - 1) + (k - off);
                w[k] = src >= first ? to_f32(x[(size_t)src * x_ld + c]) : slot[(size_t)(n_taps - 1 - (first - src)) * channels + c];
            }
        }
        for (int t = t0; t < t_end; ++t) {
            const float xin = to_f32(x[(size_t)t * x_ld + c]);
            float acc = fmaf(tp[M - 1], xin, b);
#pragma unroll
            for (int k = 0; k < M - 1; ++k) acc = fmaf(tp[k], w[k], acc);
#pragma unroll
            for (int k = 0; k < M - 2; ++k) w[k] = w[k + 1];
            w[M - 2] = xin;
            if (silu) acc = acc / (1.0f + expf(-acc));
            y[(size_t)t * channels + c] = from_f32<AT>(acc);
        }
        return;
    }
    for (int t = t0; t < t_end; ++t) {
        const int s = seq_of_token[t];
        const int first = q_start[s];
        const float* slot = state + (size_t)state_slots[s] * slot_stride;
        float acc = b;
        for (int j = 0; j < n_taps; ++j) {
            const int src = t - (n_taps - 1) + j;  // a row of this step, or behind its first row
            float v;
            if (src >= first) v = to_f32(x[(size_t)src * x_ld + c]);
            else v = slot[(size_t)(n_taps - 1 - (first - src)) * channels + c];
            acc = fmaf(taps[(size_t)c * n_taps + j], v, acc);
        }
        if (silu) acc = acc / (1.0f + expf(-acc));
        y[(size_t)t * channels + c] = from_f32<AT>(acc);
    }
}

// The slot's new content: the last L-1 inputs of the sequence (rows of this step, and what the
// slot held where the portion is shorter).  A thread per (sequence, channel) walks the L-1 rows
// in an order that never reads a value it has overwritten.
template <typename AT>
__global__ void causal_conv_state_kernel(const AT* __restrict__ x, long long x_ld, float* __restrict__ state, long long slot_stride,
                                         const int* __restrict__ q_start, const int* __restrict__ state_slots, int num_seqs,
                                         int channels, int n_taps) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)num_seqs * channels) return;
    const int s = (int)(i / channels), c = (int)(i % channels);
    const int first = q_start[s], n = q_start[s + 1] - first;
    if (n <= 0) return;
    float* slot = state + (size_t)state_slots[s] * slot_stride;
    const int keep = n_taps - 1;
    float next[SHISO_CONV_MAX_TAPS];
    for (int r = 0; r < keep; ++r) {
        const int back = keep - r;  // this row holds the input `back` positions before the next token
        next[r] = back <= n ? to_f32(x[(size_t)(first + n - back) * x_ld + c]) : slot[(size_t)(r + n) * channels + c];
    }
    for (int r = 0; r < keep; ++r) slot[(size_t)r * channels + c] = next[r];
}

SHISO_API int shiso_causal_conv(const void* x, long long x_ld, int act_dtype, const float* taps, const float* bias, float* state,
                                long long slot_stride, const int* seq_of_token, const int* q_start, const int* state_slots, void* y,
                                int tokens, int num_seqs, int channels, int n_taps, int silu, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (n_taps < 2 || n_taps > SHISO_CONV_MAX_TAPS || channels <= 0) return SHISO_ERR_SHAPE;
    const unsigned blocks = ceil_div_u((long long)((tokens + SHISO_CONV_ROWS - 1) / SHISO_CONV_ROWS) * channels, 256);
    const unsigned sblocks = ceil_div_u((long long)num_seqs * channels, 256);
    if (act_dtype == SHISO_F32) {
        launch_kernel(causal_conv_kernel<float>, blocks, 256, 0, stream, (const float*)x, x_ld, taps, bias, (const float*)state,
                      slot_stride, seq_of_token, q_start, state_slots, (float*)y, tokens, channels, n_taps, silu);
        launch_kernel(causal_conv_state_kernel<float>, sblocks, 256, 0, stream, (const float*)x, x_ld, state, slot_stride, q_start,
                      state_slots, num_seqs, channels, n_taps);
    } else if (act_dtype == SHISO_BF16) {
        launch_kernel(causal_conv_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, x_ld, taps, bias,
                      (const float*)state, slot_stride, seq_of_token, q_start, state_slots, (__nv_bfloat16*)y, tokens, channels,
                      n_taps, silu);
        launch_kernel(causal_conv_state_kernel<__nv_bfloat16>, sblocks, 256, 0, stream, (const __nv_bfloat16*)x, x_ld, state,
                      slot_stride, q_start, state_slots, num_seqs, channels, n_taps);
    } else {
        return SHISO_ERR_DTYPE;
    }
    return launch_status();
}

// --------------------------------------------------------------------------- rotation of head columns

// out[t, h, :] = x[t, h, :] with pair (i, i + rotary_dim/2) - or, with `interleaved`, the neighbours
// (2i, 2i + 1) - turned by positions[t] * inv_freq[i], cosine and sine times `magnitude`; columns
// from rotary_dim on are copied.  x and out are [T, H, width] with their own row and head strides.
template <typename AT>
__global__ void rotate_heads_kernel(const AT* __restrict__ x, long long x_ld, long long x_hs, AT* __restrict__ out, long long out_ld,
                                    long long out_hs, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                    int tokens, int heads, int width, int rotary_dim, float magnitude, int interleaved) {
    pdl_begin();
    const int half = rotary_dim / 2;
    const int per_head = width - half;  // a thread per pair, or per column behind the rotated ones
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * heads * per_head) return;
    const int c = (int)(i % per_head);
    const int h = (int)((i / per_head) % heads);
    const int t = (int)(i / ((long long)per_head * heads));
    const AT* src = x + (size_t)t * x_ld + (size_t)h * x_hs;
    AT* dst = out + (size_t)t * out_ld + (size_t)h * out_hs;
    if (c < half) {
        const float angle = (float)positions[t] * inv_freq[c];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        sn *= magnitude, cs *= magnitude;
        const int a = interleaved ? 2 * c : c, b = interleaved ? 2 * c + 1 : c + half;
        const float u = to_f32(src[a]), v = to_f32(src[b]);
        dst[a] = from_f32<AT>(u * cs - v * sn);
        dst[b] = from_f32<AT>(v * cs + u * sn);
    } else {
        dst[c + half] = src[c + half];
    }
}

SHISO_API int shiso_rotate_heads(const void* x, long long x_ld, long long x_hs, void* out, long long out_ld, long long out_hs,
                                 int act_dtype, const float* inv_freq, const int* positions, int tokens, int heads, int width,
                                 int rotary_dim, float magnitude, int interleaved, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0 || width <= 0) return SHISO_OK;
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > width) return SHISO_ERR_SHAPE;
    const unsigned blocks = ceil_div_u((long long)tokens * heads * (width - rotary_dim / 2), 256);
    if (act_dtype == SHISO_F32)
        launch_kernel(rotate_heads_kernel<float>, blocks, 256, 0, stream, (const float*)x, x_ld, x_hs, (float*)out, out_ld, out_hs,
                      inv_freq, positions, tokens, heads, width, rotary_dim, magnitude, interleaved);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(rotate_heads_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)x, x_ld, x_hs,
                      (__nv_bfloat16*)out, out_ld, out_hs, inv_freq, positions, tokens, heads, width, rotary_dim, magnitude, interleaved);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}

// --------------------------------------------------------------------------- the latent cache row

// rows[t] = [latent (rank) | shared key part (width - rank)]: the latent divided by its root mean
// square, times w; the rest rotated by the position (pairs and magnitude as in rotate_heads_kernel);
// both stored as the position's cache row.  One block per row.
template <typename AT>
__global__ void latent_store_kernel(const AT* __restrict__ rows, long long ld, const float* __restrict__ w,
                                    const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                    const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int table_width,
                                    AT* __restrict__ cache, int rank, int width, int rotary_dim, int page_size, float eps,
                                    float magnitude, int interleaved) {
    pdl_begin();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_of_token[t] * table_width + pos / page_size];
    if (page < 0) return;
    const AT* src = rows + (size_t)t * ld;
    AT* dst = cache + ((size_t)page * page_size + pos % page_size) * width;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_f32(src[i]);
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<AT>(to_f32(src[i]) * inv * w[i]);
    const int half = rotary_dim / 2, rest = width - rank;
    for (int c = threadIdx.x; c < rest - half; c += blockDim.x) {
        if (c < half) {
            float sn, cs;
            sincosf((float)pos * inv_freq[c], &sn, &cs);
            sn *= magnitude, cs *= magnitude;
            const int a = rank + (interleaved ? 2 * c : c), b = rank + (interleaved ? 2 * c + 1 : c + half);
            const float u = to_f32(src[a]), v = to_f32(src[b]);
            dst[a] = from_f32<AT>(u * cs - v * sn);
            dst[b] = from_f32<AT>(v * cs + u * sn);
        } else {
            dst[rank + c + half] = src[rank + c + half];
        }
    }
}

SHISO_API int shiso_latent_store(const void* rows, long long ld, int act_dtype, const float* w, const float* inv_freq,
                                 const int* positions, const int* seq_of_token, const int* block_table, int table_width, void* cache,
                                 int tokens, int rank, int width, int rotary_dim, int page_size, float eps, float magnitude,
                                 int interleaved, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (rank <= 0 || width < rank || rotary_dim % 2 || rotary_dim > width - rank) return SHISO_ERR_SHAPE;
    const int threads = rank >= 512 ? 256 : 128;
    if (act_dtype == SHISO_F32)
        launch_kernel(latent_store_kernel<float>, tokens, threads, 0, stream, (const float*)rows, ld, w, inv_freq, positions,
                      seq_of_token, block_table, table_width, (float*)cache, rank, width, rotary_dim, page_size, eps, magnitude, interleaved);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(latent_store_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (const __nv_bfloat16*)rows, ld, w, inv_freq,
                      positions, seq_of_token, block_table, table_width, (__nv_bfloat16*)cache, rank, width, rotary_dim, page_size, eps, magnitude,
                      interleaved);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
