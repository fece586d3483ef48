// Grouped-query attention whose mask, weighting and head preparation are parameters.
//
//   prepare   per (row, head): an RMS norm over the head (none, before the rotation, or after it;
//             with a [dim] weight or without), the rotation of the first rotary_dim entries in
//             half-split pairs (i, i + rotary_dim/2) by position * inv_freq[i], cosine and sine
//             times `magnitude`; queries are written back in place, keys go to the paged cache,
//             values are copied to theirs (they may be narrower or wider than the keys).
//   attention the general kernel, one CTA per (row, query head).  What a row at position i sees:
//               window  j <= i with i - j < size, and besides those the first keep_first
//                       positions of the sequence, at their true positions;
//               chunk   j <= i with j / size == i / size, chunks counted from position 0.
//             A score is (q . k) * scale, then softcap * tanh(score / softcap) when a cap is
//             given.  Weights are a softmax over the visible keys, or sigmoid(score + bias[head])
//             per key with no normalisation.  The head's output may be multiplied by
//             sigmoid(gate[row, head]) - or, with a wide gate, every output entry by the sigmoid of its own column.
//
// The visible keys form two lists in position order - the kept first positions that lie before
// the window, then the window or chunk - and each list is cut into runs of 32 keys from its
// start; run c belongs to warp c % 8 of CTA (c / 8) % splits, the warps' partial results are
// merged in warp order and, with more than one CTA a (row, head), the CTAs' by a second launch in
// CTA order (sigmoid weights simply add up; softmax shares are brought to one maximum).  The
// caller picks `splits` from the mask's size: a row near the end of a window or chunk of 1,024
// keys is 32 runs, which one CTA walks four deep while most SMs of a decode step idle.
// What a row adds up, and in which order, depends on its position and on `splits` only: not on
// how the sequence was cut into steps, not on the pages.  Scores, weights, statistics and
// output sums are float.
//
// Cache rows: row(p) = table[p / page_size] * page_size + p % page_size, as everywhere.
#include "common.cuh"

namespace {

constexpr int MA_WARPS = 8;
constexpr int MA_MAX_DIM = 256;
constexpr int MA_SLOTS = MA_MAX_DIM / 32;  // prepare: a lane holds entries lane + 32 * e
constexpr int MA_PAIRS = MA_MAX_DIM / 64;  // attention: a lane holds value channels 2 * lane + 64 * e and the next

enum { MA_NORM_NONE = 0, MA_NORM_BEFORE = 1, MA_NORM_AFTER = 2 };
enum { MA_MASK_WINDOW = 0, MA_MASK_CHUNK = 1 };

template <typename AT>
__global__ void __launch_bounds__(MA_WARPS * 32)
head_prepare_store_kernel(AT* __restrict__ proj, long long ld, int q_col, int k_col, int v_col, const float* __restrict__ q_w,
                          const float* __restrict__ k_w, const float* __restrict__ inv_freq, const int* __restrict__ positions,
                          const int* __restrict__ seq_of_token, const int* __restrict__ table, int table_width,
                          AT* __restrict__ k_cache, AT* __restrict__ v_cache, int heads, int kv_heads, int dim, int vdim,
                          int rotary_dim, int page_size, float eps, float magnitude, int norm_mode, int store) {
    __shared__ float buf[MA_WARPS][MA_MAX_DIM];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int item = blockIdx.y * MA_WARPS + warp;
    if (item >= heads + kv_heads) return;
    const bool is_q = item < heads;
    const int head = is_q ? item : item - heads;
    if (!is_q && !store) return;
    AT* src = proj + (size_t)t * ld + (is_q ? q_col : k_col) + (size_t)head * dim;
    const float* w = is_q ? q_w : k_w;
    const int pos = positions[t];
    float x[MA_SLOTS];
#pragma unroll
    for (int e = 0; e < MA_SLOTS; ++e) {
        const int c = lane + 32 * e;
        x[e] = c < dim ? to_f32(src[c]) : 0.0f;
    }
    if (norm_mode == MA_NORM_BEFORE) {
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) ss += x[e] * x[e];
        const float inv = rsqrtf(warp_sum(ss) / (float)dim + eps);
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) {
            const int c = lane + 32 * e;
            if (c < dim) x[e] = x[e] * inv * (w ? w[c] : 1.0f);
        }
    }
    if (rotary_dim > 0) {
        const int half = rotary_dim >> 1;
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) buf[warp][lane + 32 * e] = x[e];
        __syncwarp();
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) {
            const int c = lane + 32 * e;
            if (c < rotary_dim) {
                const int pair = c < half ? c : c - half;
                float s, co;
                sincosf((float)pos * inv_freq[pair], &s, &co);
                s *= magnitude;
                co *= magnitude;
                const float u = buf[warp][pair], v = buf[warp][pair + half];
                x[e] = c < half ? u * co - v * s : v * co + u * s;
            }
        }
    }
    if (norm_mode == MA_NORM_AFTER) {
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) ss += x[e] * x[e];
        const float inv = rsqrtf(warp_sum(ss) / (float)dim + eps);
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) {
            const int c = lane + 32 * e;
            if (c < dim) x[e] = x[e] * inv * (w ? w[c] : 1.0f);
        }
    }
    if (is_q) {
#pragma unroll
        for (int e = 0; e < MA_SLOTS; ++e) {
            const int c = lane + 32 * e;
            if (c < dim) src[c] = from_f32<AT>(x[e]);
        }
        return;
    }
    const int page = table[(size_t)seq_of_token[t] * table_width + pos / page_size];
    if (page < 0) return;
    const size_t row = (size_t)page * page_size + pos % page_size;
    AT* kd = k_cache + (row * kv_heads + head) * dim;
#pragma unroll
    for (int e = 0; e < MA_SLOTS; ++e) {
        const int c = lane + 32 * e;
        if (c < dim) kd[c] = from_f32<AT>(x[e]);
    }
    const AT* vs = proj + (size_t)t * ld + v_col + (size_t)head * vdim;
    AT* vd = v_cache + (row * kv_heads + head) * vdim;
    for (int c = lane; c < vdim; c += 32) vd[c] = vs[c];
}

// The same for bfloat16 rows whose sizes allow 16-byte accesses (head sizes, the rotation's half
// and every column offset in multiples of 8): a thread holds 8 neighbouring entries of a head,
// `group` lanes (a power of two, at least dim / 8) a head, a CTA one row of the step.  The
// rotation's cosines and sines are formed once per row, in shared memory, not once per head; the
// partner entries (half a rotation away) come from the lane that holds them.  Which of the two
// kernels runs depends on the sizes only, so a sequence's cache rows all come from one of them.
constexpr int MA_VEC_THREADS = 256;

__global__ void __launch_bounds__(MA_VEC_THREADS)
head_prepare_store_vec_kernel(__nv_bfloat16* __restrict__ proj, long long ld, int q_col, int k_col, int v_col,
                              const float* __restrict__ q_w, const float* __restrict__ k_w, const float* __restrict__ inv_freq,
                              const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ table,
                              int table_width, __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int heads,
                              int kv_heads, int dim, int vdim, int rotary_dim, int page_size, float eps, float magnitude,
                              int norm_mode, int store, int group) {
    __shared__ float cs[MA_MAX_DIM / 2], sn[MA_MAX_DIM / 2];
    pdl_begin();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    for (int i = threadIdx.x; i < half; i += MA_VEC_THREADS) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        sn[i] = s * magnitude;
        cs[i] = c * magnitude;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int sub = threadIdx.x % group, c0 = sub * 8;
    const int units = heads + (store ? kv_heads : 0);
    const int per_pass = MA_VEC_THREADS / group * gridDim.y;
    size_t cache_row = 0;
    bool have_row = false;
    if (store) {
        const int page = table[(size_t)seq_of_token[t] * table_width + pos / page_size];
        have_row = page >= 0;
        cache_row = (size_t)max(page, 0) * page_size + pos % page_size;
    }
    for (int base = blockIdx.y * (MA_VEC_THREADS / group); base < units; base += per_pass) {  // uniform: every lane takes part in the shuffles
        const int unit = base + threadIdx.x / group;
        const bool live = unit < units && c0 < dim;
        const bool is_q = unit < heads;
        const int head = is_q ? unit : unit - heads;
        __nv_bfloat16* src = proj + (size_t)t * ld + (is_q ? q_col : k_col) + (size_t)head * dim + c0;
        const float* w = is_q ? q_w : k_w;
        float x[8];
        if (live) {
            const uint4 raw = *reinterpret_cast<const uint4*>(src);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x[2 * i] = __uint_as_float(words[i] << 16);
                x[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = 0.0f;
        }
        auto unit_norm = [&]() {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
            for (int off = group >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            const float inv = rsqrtf(ss / (float)dim + eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = x[i] * inv * (w && live ? w[c0 + i] : 1.0f);
        };
        if (norm_mode == MA_NORM_BEFORE) unit_norm();
        if (rotary_dim > 0) {
            const bool low = c0 < half, turns = c0 < rotary_dim;
            const int partner = (lane - sub) + (low ? sub + half / 8 : sub - half / 8);
            const int pair = low ? c0 : c0 - half;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float other = __shfl_sync(0xffffffffu, x[i], turns ? partner : lane);
                if (turns) x[i] = low ? x[i] * cs[pair + i] - other * sn[pair + i] : x[i] * cs[pair + i] + other * sn[pair + i];
            }
        }
        if (norm_mode == MA_NORM_AFTER) unit_norm();
        if (!live) continue;
        uint4 packed;
        {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            packed = *reinterpret_cast<uint4*>(h);
        }
        if (is_q) {
            *reinterpret_cast<uint4*>(src) = packed;
            continue;
        }
        if (!have_row) continue;
        *reinterpret_cast<uint4*>(k_cache + (cache_row * kv_heads + head) * dim + c0) = packed;
    }
    if (store && have_row) {  // the values: 16-byte pieces, copied as they are
        const int pieces = kv_heads * vdim / 8;
        const uint4* vs = reinterpret_cast<const uint4*>(proj + (size_t)t * ld + v_col);
        uint4* vd = reinterpret_cast<uint4*>(v_cache + cache_row * kv_heads * vdim);
        for (int i = blockIdx.y * MA_VEC_THREADS + threadIdx.x; i < pieces; i += MA_VEC_THREADS * gridDim.y) vd[i] = vs[i];
    }
}

__device__ __forceinline__ float2 ma_load_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ma_load_pair(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// q . key over `dim` channels; 16-byte loads of the key where its rows allow them.
__device__ __forceinline__ float ma_dot(const float* __restrict__ q, const float* __restrict__ key, int dim, bool wide) {
    float dot = 0.0f;
    if (wide) {
#pragma unroll 4
        for (int c = 0; c < dim; c += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(key + c);
            dot += q[c] * k4.x + q[c + 1] * k4.y + q[c + 2] * k4.z + q[c + 3] * k4.w;
        }
    } else {
        for (int c = 0; c < dim; ++c) dot += q[c] * key[c];
    }
    return dot;
}
__device__ __forceinline__ float ma_dot(const float* __restrict__ q, const __nv_bfloat16* __restrict__ key, int dim, bool wide) {
    float dot = 0.0f;
    if (wide) {
#pragma unroll 8
        for (int c = 0; c < dim; c += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(key + c);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                dot += q[c + 2 * i] * __uint_as_float(w[i] << 16);
                dot += q[c + 2 * i + 1] * __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    } else {
        for (int c = 0; c < dim; ++c) dot += q[c] * __bfloat162float(key[c]);
    }
    return dot;
}

struct MaskedArgs {
    const int* table;
    const int* positions;
    const int* seq_of_token;
    const float* key_bias;  // [heads], sigmoid weighting only; may be null
    long long q_ld, out_ld, gate_ld;
    int table_width, heads, kv_heads, dim, vdim, page_size, mask_kind, size, keep_first;
    int gate_wide;   // the gate has a column per output entry (heads * vdim) instead of one per head
    int splits;      // CTAs that share a (row, head)'s runs of keys; more than one: partial results go to `scratch`
    float* scratch;  // [rows * heads * splits][vdim + 2]: sums, running maximum, sum of weights
    float scale, softcap;
};

// The two lists of a row at `pos`: [0, kept) and [first, pos].
__device__ __forceinline__ void ma_lists(const MaskedArgs& a, int pos, int& kept, int& first) {
    if (a.mask_kind == MA_MASK_CHUNK) {
        first = pos / a.size * a.size;
        kept = 0;
    } else {
        first = max(0, pos - a.size + 1);
        kept = min(a.keep_first, first);
    }
}

// A warp folds 32 keys (positions first + base ..) into its running result: a lane takes a key and
// forms the whole dot product; the lanes then share the value channels.
template <typename AT, bool SIGMOID>
__device__ __forceinline__ void ma_fold(const MaskedArgs& a, const AT* __restrict__ k_cache, const AT* __restrict__ v_cache,
                                        const int* pages, int first, int count, int base, int kv_head, const float* q, float bias,
                                        float& running_max, float& running_sum, float (&acc)[MA_PAIRS][2], int lane,
                                        float* run_weight, long long* run_row) {
    const int n = min(32, count - base);
    long long row = -1;
    float score = -INFINITY;
    if (lane < n) {
        const int p = first + base + lane;
        const int page = pages[p / a.page_size];
        if (page >= 0) {
            row = (long long)page * a.page_size + p % a.page_size;
            const bool wide = (a.dim * (int)sizeof(AT)) % 16 == 0;
            score = ma_dot(q, k_cache + ((size_t)row * a.kv_heads + kv_head) * a.dim, a.dim, wide) * a.scale;
            if (a.softcap > 0.0f) score = a.softcap * tanhf(score / a.softcap);
        }
    }
    float weight;
    if (SIGMOID) {
        weight = row >= 0 ? 1.0f / (1.0f + expf(-(score + bias))) : 0.0f;
    } else {
        const float new_max = fmaxf(running_max, warp_max(score));
        if (new_max == -INFINITY) return;
        const float keep = expf(running_max - new_max);  // 0 while nothing was seen
        weight = row >= 0 ? expf(score - new_max) : 0.0f;
        running_sum = running_sum * keep + warp_sum(weight);
        running_max = new_max;
#pragma unroll
        for (int e = 0; e < MA_PAIRS; ++e) {
            acc[e][0] *= keep;
            acc[e][1] *= keep;
        }
    }
    const bool paired = a.vdim % 2 == 0;
    // the run's weights and rows go through the warp's shared memory: every lane reads them all
    __syncwarp();
    run_weight[lane] = weight;
    run_row[lane] = row >= 0 ? ((long long)row * a.kv_heads + kv_head) * a.vdim : -1;
    __syncwarp();
    // (no branch between two loads - a key the run does not have reads row 0 with weight zero -
    // so that the value rows of eight keys are asked for together)
#pragma unroll 8
    for (int kk = 0; kk < 32; ++kk) {
        const long long r = run_row[kk];
        const bool live = r >= 0;
        const float w = live ? run_weight[kk] : 0.0f;
        const AT* value = v_cache + (live ? r : 0);
#pragma unroll
        for (int e = 0; e < MA_PAIRS; ++e) {
            const int c = e * 64 + 2 * lane;
            if (paired) {
                if (c < a.vdim) {
                    const float2 v2 = ma_load_pair(value + c);
                    acc[e][0] += live ? w * v2.x : 0.0f;
                    acc[e][1] += live ? w * v2.y : 0.0f;
                }
            } else {
                if (c < a.vdim) acc[e][0] += live ? w * to_f32(value[c]) : 0.0f;
                if (c + 1 < a.vdim) acc[e][1] += live ? w * to_f32(value[c + 1]) : 0.0f;
            }
        }
    }
}

template <typename AT, bool SIGMOID>
__global__ void __launch_bounds__(MA_WARPS * 32)
masked_attention_kernel(const AT* __restrict__ q, const AT* __restrict__ k_cache, const AT* __restrict__ v_cache, AT* out,
                        const AT* __restrict__ gate, MaskedArgs a) {
    __shared__ float sq[MA_MAX_DIM];
    __shared__ float run_weight[MA_WARPS][32];
    __shared__ long long run_row[MA_WARPS][32];
    __shared__ float part_max[MA_WARPS], part_sum[MA_WARPS];
    __shared__ float part_acc[MA_WARPS][MA_MAX_DIM];
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x / a.splits, split = blockIdx.x % a.splits;
    const int t = item / a.heads, head = item % a.heads;
    const int kv_head = head / (a.heads / a.kv_heads);
    for (int c = threadIdx.x; c < a.dim; c += blockDim.x) sq[c] = to_f32(q[(size_t)t * a.q_ld + (size_t)head * a.dim + c]);
    __syncthreads();
    const int pos = a.positions[t], seq = a.seq_of_token[t];
    int kept, first;
    ma_lists(a, pos, kept, first);
    const int seen = pos - first + 1;
    const int kept_runs = (kept + 31) / 32, runs = kept_runs + (seen + 31) / 32;
    const float bias = SIGMOID && a.key_bias ? a.key_bias[head] : 0.0f;
    const int* pages = a.table + (size_t)seq * a.table_width;
    float running_max = -INFINITY, running_sum = 0.0f;
    float acc[MA_PAIRS][2];
#pragma unroll
    for (int e = 0; e < MA_PAIRS; ++e) acc[e][0] = acc[e][1] = 0.0f;
    for (int run = split * MA_WARPS + warp; run < runs; run += MA_WARPS * a.splits) {
        if (run < kept_runs)
            ma_fold<AT, SIGMOID>(a, k_cache, v_cache, pages, 0, kept, run * 32, kv_head, sq, bias, running_max, running_sum, acc, lane,
                                 run_weight[warp], run_row[warp]);
        else
            ma_fold<AT, SIGMOID>(a, k_cache, v_cache, pages, first, seen, (run - kept_runs) * 32, kv_head, sq, bias, running_max,
                                 running_sum, acc, lane, run_weight[warp], run_row[warp]);
    }
    if (lane == 0) {
        part_max[warp] = running_max;
        part_sum[warp] = running_sum;
    }
#pragma unroll
    for (int e = 0; e < MA_PAIRS; ++e) {
        const int c = e * 64 + 2 * lane;
        part_acc[warp][c] = acc[e][0];
        part_acc[warp][c + 1] = acc[e][1];
    }
    __syncthreads();
    if (a.splits > 1) {
        // this CTA's share, merged in warp order; the merge kernel adds the shares up in split order
        float* part = a.scratch + (size_t)blockIdx.x * (a.vdim + 2);
        float top = -INFINITY, total = 0.0f;
        float factor[MA_WARPS];
#pragma unroll
        for (int w = 0; w < MA_WARPS; ++w) top = fmaxf(top, part_max[w]);
#pragma unroll
        for (int w = 0; w < MA_WARPS; ++w) {
            factor[w] = SIGMOID ? 1.0f : (part_max[w] == -INFINITY ? 0.0f : expf(part_max[w] - top));
            total += part_sum[w] * factor[w];
        }
        for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < MA_WARPS; ++w) sum += part_acc[w][c] * factor[w];
            part[c] = sum;
        }
        if (threadIdx.x == 0) {
            part[a.vdim] = top;
            part[a.vdim + 1] = total;
        }
        return;
    }
    AT* dst = out + (size_t)t * a.out_ld + (size_t)head * a.vdim;
    float gated = 1.0f;
    if (gate && !a.gate_wide) gated = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * a.gate_ld + head])));
    const AT* wide = gate && a.gate_wide ? gate + (size_t)t * a.gate_ld + (size_t)head * a.vdim : nullptr;
    if (SIGMOID) {
        for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < MA_WARPS; ++w) sum += part_acc[w][c];
            dst[c] = from_f32<AT>(sum * (wide ? 1.0f / (1.0f + expf(-to_f32(wide[c]))) : gated));
        }
        return;
    }
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < MA_WARPS; ++w) top = fmaxf(top, part_max[w]);
    if (top == -INFINITY) {
        for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) dst[c] = from_f32<AT>(0.0f);
        return;
    }
    float factor[MA_WARPS];
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < MA_WARPS; ++w) {
        factor[w] = part_max[w] == -INFINITY ? 0.0f : expf(part_max[w] - top);
        total += part_sum[w] * factor[w];
    }
    for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < MA_WARPS; ++w) sum += part_acc[w][c] * factor[w];
        dst[c] = from_f32<AT>(sum / total * (wide ? 1.0f / (1.0f + expf(-to_f32(wide[c]))) : gated));
    }
}

// Adds up the shares of a (row, head) in split order; softmax shares are brought to one maximum first.
template <typename AT, bool SIGMOID>
__global__ void __launch_bounds__(128)
masked_attention_merge_kernel(AT* out, const AT* __restrict__ gate, MaskedArgs a) {
    pdl_begin();
    const int t = blockIdx.x / a.heads, head = blockIdx.x % a.heads;
    const float* parts = a.scratch + (size_t)blockIdx.x * a.splits * (a.vdim + 2);
    AT* dst = out + (size_t)t * a.out_ld + (size_t)head * a.vdim;
    float gated = 1.0f;
    if (gate && !a.gate_wide) gated = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * a.gate_ld + head])));
    const AT* wide = gate && a.gate_wide ? gate + (size_t)t * a.gate_ld + (size_t)head * a.vdim : nullptr;
    float top = -INFINITY, total = 0.0f;
    if (!SIGMOID) {
        for (int s = 0; s < a.splits; ++s) top = fmaxf(top, parts[(size_t)s * (a.vdim + 2) + a.vdim]);
        if (top == -INFINITY) {
            for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) dst[c] = from_f32<AT>(0.0f);
            return;
        }
        for (int s = 0; s < a.splits; ++s) {
            const float m = parts[(size_t)s * (a.vdim + 2) + a.vdim];
            total += parts[(size_t)s * (a.vdim + 2) + a.vdim + 1] * (m == -INFINITY ? 0.0f : expf(m - top));
        }
    }
    for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
        float sum = 0.0f;
        for (int s = 0; s < a.splits; ++s) {
            const float* part = parts + (size_t)s * (a.vdim + 2);
            const float f = SIGMOID ? 1.0f : (part[a.vdim] == -INFINITY ? 0.0f : expf(part[a.vdim] - top));
            sum += part[c] * f;
        }
        dst[c] = from_f32<AT>((SIGMOID ? sum : sum / total) * (wide ? 1.0f / (1.0f + expf(-to_f32(wide[c]))) : gated));
    }
}

template <typename AT>
int launch_prepare(void* proj, long long ld, int q_col, int k_col, int v_col, const float* q_w, const float* k_w, const float* inv_freq,
                   const int* positions, const int* seq_of_token, const int* table, int table_width, void* k_cache, void* v_cache,
                   int tokens, int heads, int kv_heads, int dim, int vdim, int rotary_dim, int page_size, float eps, float magnitude,
                   int norm_mode, int store, cudaStream_t stream) {
    if constexpr (sizeof(AT) == 2) {
        const bool wide = dim % 8 == 0 && vdim % 8 == 0 && rotary_dim % 16 == 0 && ld % 8 == 0 && q_col % 8 == 0 && k_col % 8 == 0 &&
                          v_col % 8 == 0 && !(((uintptr_t)proj | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15);
        if (wide) {
            int group = 1;
            while (group * 8 < dim) group *= 2;
            const int units = heads + (store ? kv_heads : 0);
            // a row's heads are shared out over CTAs of 256 / group heads
            const int passes = ceil_div_u(units * group, MA_VEC_THREADS);
            const dim3 vgrid(tokens, passes);
            launch_kernel(head_prepare_store_vec_kernel, vgrid, MA_VEC_THREADS, 0, stream, (__nv_bfloat16*)proj, ld, q_col, k_col, v_col, q_w,
                          k_w, inv_freq, positions, seq_of_token, table, table_width, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads,
                          kv_heads, dim, vdim, rotary_dim, page_size, eps, magnitude, norm_mode, store, group);
            return launch_status();
        }
    }
    const dim3 grid(tokens, ceil_div_u(heads + (store ? kv_heads : 0), MA_WARPS));
    launch_kernel(head_prepare_store_kernel<AT>, grid, MA_WARPS * 32, 0, stream, (AT*)proj, ld, q_col, k_col, v_col, q_w, k_w, inv_freq,
                  positions, seq_of_token, table, table_width, (AT*)k_cache, (AT*)v_cache, heads, kv_heads, dim, vdim, rotary_dim,
                  page_size, eps, magnitude, norm_mode, store);
    return launch_status();
}

template <typename AT>
int launch_attention(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate, const MaskedArgs& a,
                     int tokens, int sigmoid, cudaStream_t stream) {
    const unsigned items = (unsigned)tokens * a.heads, blocks = items * a.splits;
    if (sigmoid)
        launch_kernel(masked_attention_kernel<AT, true>, blocks, MA_WARPS * 32, 0, stream, (const AT*)q, (const AT*)k_cache,
                      (const AT*)v_cache, (AT*)out, (const AT*)gate, a);
    else
        launch_kernel(masked_attention_kernel<AT, false>, blocks, MA_WARPS * 32, 0, stream, (const AT*)q, (const AT*)k_cache,
                      (const AT*)v_cache, (AT*)out, (const AT*)gate, a);
    if (a.splits > 1) {
        const int first = launch_status();
        if (first != SHISO_OK) return first;
        if (sigmoid)
            launch_kernel(masked_attention_merge_kernel<AT, true>, items, 128, 0, stream, (AT*)out, (const AT*)gate, a);
        else
            launch_kernel(masked_attention_merge_kernel<AT, false>, items, 128, 0, stream, (AT*)out, (const AT*)gate, a);
    }
    return launch_status();
}

}  // namespace

SHISO_API int shiso_head_prepare_store(void* proj, long long ld, int act_dtype, int q_col, int k_col, int v_col, const float* q_w,
                                       const float* k_w, const float* inv_freq, const int* positions, const int* seq_of_token,
                                       const int* table, int table_width, void* k_cache, void* v_cache, int tokens, int heads,
                                       int kv_heads, int dim, int vdim, int rotary_dim, int page_size, float eps, float magnitude,
                                       int norm_mode, int store, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (dim <= 0 || dim > MA_MAX_DIM || vdim <= 0 || heads <= 0 || kv_heads < 0 || rotary_dim < 0 || rotary_dim > dim || rotary_dim % 2 ||
        norm_mode < MA_NORM_NONE || norm_mode > MA_NORM_AFTER)
        return SHISO_ERR_SHAPE;
    if (rotary_dim > 0 && !inv_freq) return SHISO_ERR_SHAPE;
    if (act_dtype == SHISO_F32)
        return launch_prepare<float>(proj, ld, q_col, k_col, v_col, q_w, k_w, inv_freq, positions, seq_of_token, table, table_width, k_cache,
                                     v_cache, tokens, heads, kv_heads, dim, vdim, rotary_dim, page_size, eps, magnitude, norm_mode, store,
                                     stream);
    if (act_dtype == SHISO_BF16)
        return launch_prepare<__nv_bfloat16>(proj, ld, q_col, k_col, v_col, q_w, k_w, inv_freq, positions, seq_of_token, table, table_width,
                                             k_cache, v_cache, tokens, heads, kv_heads, dim, vdim, rotary_dim, page_size, eps, magnitude,
                                             norm_mode, store, stream);
    return SHISO_ERR_DTYPE;
}

SHISO_API int shiso_masked_attention(const void* q, long long q_ld, int act_dtype, const void* k_cache, const void* v_cache,
                                     const int* table, int table_width, const int* positions, const int* seq_of_token, void* out,
                                     long long out_ld, const void* gate, long long gate_ld, const float* key_bias, int tokens,
                                     int heads, int kv_heads, int dim, int vdim, int page_size, float scale, float softcap,
                                     int mask_kind, int size, int keep_first, int sigmoid, int splits, float* scratch,
                                     int gate_wide, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (splits < 1 || (splits > 1 && !scratch)) return SHISO_ERR_SHAPE;
    if (dim <= 0 || dim > MA_MAX_DIM || vdim <= 0 || vdim > MA_MAX_DIM || kv_heads <= 0 || heads % kv_heads || size < 1 || keep_first < 0 ||
        (mask_kind != MA_MASK_WINDOW && mask_kind != MA_MASK_CHUNK))
        return SHISO_ERR_SHAPE;
    if ((long long)tokens * heads * splits > 0x7fffffffLL) return SHISO_ERR_SHAPE;
    MaskedArgs a;
    a.table = table;
    a.positions = positions;
    a.seq_of_token = seq_of_token;
    a.key_bias = key_bias;
    a.q_ld = q_ld;
    a.out_ld = out_ld;
    a.gate_ld = gate_ld;
    a.gate_wide = gate_wide;
    a.table_width = table_width;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.dim = dim;
    a.vdim = vdim;
    a.page_size = page_size;
    a.mask_kind = mask_kind;
    a.size = size;
    a.keep_first = keep_first;
    a.splits = splits;
    a.scratch = scratch;
    a.scale = scale;
    a.softcap = softcap;
    if (act_dtype == SHISO_F32) return launch_attention<float>(q, k_cache, v_cache, out, gate, a, tokens, sigmoid, stream);
    if (act_dtype == SHISO_BF16) return launch_attention<__nv_bfloat16>(q, k_cache, v_cache, out, gate, a, tokens, sigmoid, stream);
    return SHISO_ERR_DTYPE;
}
