// Masked attention for steps that hold prompt portions (bfloat16): the tiled kernel.
//
// The same function as the general kernel of masked_attention.cu - a window with kept first
// positions or chunks counted from position 0, scores optionally capped through a tanh, weights a
// softmax or one sigmoid per key, a gate per head on the output - computed 64 query rows at a
// time on the tensor cores.  One CTA owns 64 consecutive rows of one sequence and one query
// head; four warps, 16 rows each.  It walks the key tiles (64 positions, aligned to multiples of
// 64 of the sequence) that its rows can see: first the tiles that hold kept first positions and
// lie before the span of the rows' windows, then that span up to the last row.  Key and value
// tiles are gathered from the paged cache through the block table with cp.async, two stages;
// S = Q K^T and O += P V are m16n8k16 products (bfloat16 in, float out); scores, the cap, the
// weights and the softmax statistics are float, P is rounded to bfloat16 for the second product.
//
// The key size is a run-time number (a multiple of 16): query fragments are read from shared
// memory for every 16 channels instead of being kept in registers.  The value size is a template
// parameter (multiples of 16 up to 128), because the output accumulators live in registers.
// Keys outside every row's range are zero-filled, never read: a window group's table has holes
// there.  A masked key scores minus infinity under the softmax and weighs zero under the sigmoid.
#include "mma_tiles.cuh"

namespace {

using namespace mma_tiles;

constexpr int BM = 64;  // query rows per CTA
constexpr int BN = 64;  // keys per tile
constexpr int MT_THREADS = 128;
constexpr int MT_MAX_DIM = 256;
constexpr int MT_MAX_VDIM = 128;

enum { MT_MASK_WINDOW = 0, MT_MASK_CHUNK = 1 };

struct TileArgs {
    const __nv_bfloat16* q;        // [T, ...] rows q_ld apart, head h at column h * dim
    const __nv_bfloat16* k_cache;  // [pages, page, kv_heads, dim]
    const __nv_bfloat16* v_cache;  // [pages, page, kv_heads, vdim]
    const __nv_bfloat16* gate;     // [T, ...] rows gate_ld apart, head h at column h; or null
    const float* key_bias;         // [heads] or null
    const int* block_table;        // [S, width]
    const int* q_start;            // [S + 1]
    const int* start_pos;          // [S]
    __nv_bfloat16* out;            // [T, ...] rows out_ld apart, head h at column h * vdim
    long long q_ld, out_ld, gate_ld;
    int gate_wide;                 // the gate has a column per output entry (head h's at h * DV) instead of one per head
    int width, num_seqs, heads, kv_heads, dim, page_size, mask_kind, size, keep_first;
    float scale, softcap;
};

// The first position a row at `pos` sees besides the kept ones (it may be negative for a window).
__device__ __forceinline__ int low_edge(const TileArgs& a, int pos) {
    return a.mask_kind == MT_MASK_CHUNK ? pos / a.size * a.size : pos - a.size + 1;
}

// tanh through one exponential: 1 - 2 / (1 + e^(2y)); the absolute error is a few 1e-7.
__device__ __forceinline__ float tanh_exp(float y) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * y)); }

template <int DV, bool SIGMOID>
__global__ void __launch_bounds__(MT_THREADS)
masked_tiles_kernel(TileArgs a) {
    pdl_wait();
    constexpr int V_ROW = DV * 2 + 16;  // 16 bytes of padding: ldmatrix rows fall on distinct banks
    constexpr int V_CHUNKS = DV / 8;    // 16-byte pieces per row
    constexpr int DTILES = DV / 8;
    const int dim = a.dim;
    const int k_row = dim * 2 + 16, k_chunks = dim / 8, ksteps = dim / 16;
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* q_s = smem;                      // [BM][k_row]
    uint8_t* k_s = q_s + BM * k_row;          // [2][BN][k_row]
    uint8_t* v_s = k_s + 2 * BN * k_row;      // [2][BN][V_ROW]
    __shared__ int tile_seq, tile_row0;

    if (threadIdx.x == 0) {
        // the last tiles of a portion have the most keys: they take the first CTAs of every head
        int left = gridDim.y - 1 - blockIdx.y, found = -1, row0 = 0;
        for (int s = 0; s < a.num_seqs; ++s) {
            const int tiles = (a.q_start[s + 1] - a.q_start[s] + BM - 1) / BM;
            if (left < tiles) {
                found = s;
                row0 = left * BM;
                break;
            }
            left -= tiles;
        }
        tile_seq = found;
        tile_row0 = row0;
    }
    __syncthreads();
    const int seq = tile_seq;
    if (seq < 0) return;
    const int row0 = tile_row0;
    const int first_token = a.q_start[seq] + row0;
    const int rows = min(BM, a.q_start[seq + 1] - first_token);
    const int first_pos = a.start_pos[seq] + row0;
    const int last_pos = first_pos + rows - 1;
    const int head = blockIdx.x;
    const int kv_head = head / (a.heads / a.kv_heads);
    const int* table = a.block_table + (size_t)seq * a.width;
    const int keep = a.mask_kind == MT_MASK_WINDOW ? a.keep_first : 0;
    const int key_lo = max(0, low_edge(a, first_pos));  // low edges do not fall as positions rise
    const int tile_first = key_lo / BN, tile_last = last_pos / BN;
    const int kept_tiles = min((keep + BN - 1) / BN, tile_first);
    const int num_tiles = kept_tiles + tile_last - tile_first + 1;
    auto tile_of = [&](int it) { return it < kept_tiles ? it : tile_first + (it - kept_tiles); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int row_block = warp * 16;

    // ---- Q tile -> shared (rows past the portion are zero)
    if ((a.q_ld % 8) == 0 && ((uintptr_t)a.q & 15) == 0) {
        for (int c = tid; c < BM * k_chunks; c += MT_THREADS) {
            const int r = c / k_chunks, ch = c % k_chunks;
            const __nv_bfloat16* src = a.q + (size_t)(first_token + min(r, rows - 1)) * a.q_ld + (size_t)head * dim + ch * 8;
            cp_async16(q_s + r * k_row + ch * 16, src, r < rows);
        }
    } else {
        for (int c = tid; c < BM * dim; c += MT_THREADS) {
            const int r = c / dim, ch = c % dim;
            __nv_bfloat16 v = __float2bfloat16_rn(0.0f);
            if (r < rows) v = a.q[(size_t)(first_token + r) * a.q_ld + (size_t)head * dim + ch];
            *reinterpret_cast<__nv_bfloat16*>(q_s + r * k_row + ch * 2) = v;
        }
    }
    auto load_kv = [&](int tile, int stage) {
        uint8_t* kd = k_s + stage * BN * k_row;
        uint8_t* vd = v_s + stage * BN * V_ROW;
        for (int c = tid; c < BN * k_chunks; c += MT_THREADS) {
            const int r = c / k_chunks, ch = c % k_chunks;
            const int key = tile * BN + r;
            bool valid = key <= last_pos && (key >= key_lo || key < keep);
            int page = -1;
            if (valid) page = table[key / a.page_size];
            valid = page >= 0;
            const size_t row = valid ? (size_t)page * a.page_size + key % a.page_size : 0;
            cp_async16(kd + r * k_row + ch * 16, a.k_cache + (row * a.kv_heads + kv_head) * dim + ch * 8, valid);
        }
        for (int c = tid; c < BN * V_CHUNKS; c += MT_THREADS) {
            const int r = c / V_CHUNKS, ch = c % V_CHUNKS;
            const int key = tile * BN + r;
            bool valid = key <= last_pos && (key >= key_lo || key < keep);
            int page = -1;
            if (valid) page = table[key / a.page_size];
            valid = page >= 0;
            const size_t row = valid ? (size_t)page * a.page_size + key % a.page_size : 0;
            cp_async16(vd + r * V_ROW + ch * 16, a.v_cache + (row * a.kv_heads + kv_head) * DV + ch * 8, valid);
        }
    };
    load_kv(tile_of(0), 0);
    asm volatile("cp.async.commit_group;" ::: "memory");

    float o_acc[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    const int my_pos[2] = {first_pos + row_block + g, first_pos + row_block + g + 8};
    const int my_lo[2] = {low_edge(a, my_pos[0]), low_edge(a, my_pos[1])};
    const int warp_first = first_pos + row_block, warp_last = warp_first + 15;
    const int warp_lo_first = low_edge(a, warp_first), warp_lo_last = low_edge(a, warp_last);
    const float bias = SIGMOID && a.key_bias ? a.key_bias[head] : 0.0f;
    const bool capped = a.softcap > 0.0f;
    const float into_cap = capped ? a.scale / a.softcap : 0.0f;
    constexpr float LOG2E = 1.4426950408889634f;
    // softmax scores are kept in log2 units; the sigmoid takes them as they are
    const float unit = SIGMOID ? 1.0f : LOG2E;
    const float plain_factor = a.scale * unit, cap_factor = a.softcap * unit;
    const uint32_t q_base = smem_addr(q_s + (row_block + (lane & 7) + ((lane >> 3) & 1) * 8) * k_row + (lane >> 4) * 16);

    for (int it = 0; it < num_tiles; ++it) {
        const int stage = it & 1;
        const int tile = tile_of(it);
        if (it + 1 < num_tiles) load_kv(tile_of(it + 1), stage ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();
        const uint8_t* kt = k_s + stage * BN * k_row;
        const uint8_t* vt = v_s + stage * BN * V_ROW;
        const int key0 = tile * BN;
        // a warp none of whose rows sees a key of this tile adds nothing
        const bool warp_has_keys = row_block < rows && key0 <= warp_last && (key0 + BN - 1 >= warp_lo_first || key0 < keep);
        if (warp_has_keys) {
            // ---- S = Q K^T for this warp's 16 rows x 64 keys
            float s_acc[BN / 8][4];
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) s_acc[j][0] = s_acc[j][1] = s_acc[j][2] = s_acc[j][3] = 0.0f;
            const uint32_t k_base = smem_addr(kt + ((lane & 7) + (lane >> 4) * 8) * k_row + ((lane >> 3) & 1) * 16);
#pragma unroll 2
            for (int kk = 0; kk < ksteps; ++kk) {
                uint32_t qf[4];
                ldmatrix_x4(q_base + kk * 32, qf[0], qf[1], qf[2], qf[3]);
#pragma unroll
                for (int j = 0; j < BN / 8; j += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(k_base + j * 8 * k_row + kk * 32, b0, b1, b2, b3);
                    mma_bf16(s_acc[j], qf, b0, b1);
                    mma_bf16(s_acc[j + 1], qf, b2, b3);
                }
            }
            // ---- scale, cap, mask
            if (capped) {
#pragma unroll
                for (int j = 0; j < BN / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s_acc[j][e] = cap_factor * tanh_exp(s_acc[j][e] * into_cap);
            } else {
#pragma unroll
                for (int j = 0; j < BN / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s_acc[j][e] *= plain_factor;
            }
            // every key of the tile is seen by every row of this warp: no mask to evaluate
            const bool all_seen = key0 + BN - 1 <= warp_first && (key0 >= warp_lo_last || key0 + BN - 1 < keep);
            uint32_t p_frag[BN / 16][4];
            if (SIGMOID) {
#pragma unroll
                for (int j = 0; j < BN / 8; ++j) {
                    float p[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                        const bool seen = all_seen || (key <= my_pos[e >> 1] && (key >= my_lo[e >> 1] || key < keep));
                        p[e] = seen ? __fdividef(1.0f, 1.0f + __expf(-(s_acc[j][e] + bias))) : 0.0f;
                    }
                    p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
                    p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
                }
            } else {
                float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = key0 + j * 8 + t4 * 2 + (e & 1);
                        const bool seen = all_seen || (key <= my_pos[e >> 1] && (key >= my_lo[e >> 1] || key < keep));
                        const float v = seen ? s_acc[j][e] : -INFINITY;
                        s_acc[j][e] = v;
                        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
                    }
                }
                float correction[2], use_max[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float m = tile_max[r];
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                    const float new_max = fmaxf(row_max[r], m);
                    use_max[r] = new_max == -INFINITY ? 0.0f : new_max;  // a row that has seen no key yet
                    correction[r] = exp2f(row_max[r] - use_max[r]);
                    row_max[r] = new_max;
                }
                float tile_sum[2] = {0.0f, 0.0f};
#pragma unroll
                for (int j = 0; j < BN / 8; ++j) {
                    float p[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        p[e] = exp2f(s_acc[j][e] - use_max[e >> 1]);
                        tile_sum[e >> 1] += p[e];
                    }
                    p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p[0], p[1]);
                    p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * correction[r] + tile_sum[r];
#pragma unroll
                for (int i = 0; i < DTILES; ++i) {
                    o_acc[i][0] *= correction[0];
                    o_acc[i][1] *= correction[0];
                    o_acc[i][2] *= correction[1];
                    o_acc[i][3] *= correction[1];
                }
            }
            // ---- O += P V
            const uint32_t v_base = smem_addr(vt + ((lane & 7) + ((lane >> 3) & 1) * 8) * V_ROW + (lane >> 4) * 16);
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
                for (int dn = 0; dn < DTILES; dn += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(v_base + ks * 16 * V_ROW + dn * 16, b0, b1, b2, b3);
                    mma_bf16(o_acc[dn], p_frag[ks], b0, b1);
                    mma_bf16(o_acc[dn + 1], p_frag[ks], b2, b3);
                }
            }
        }
        __syncthreads();  // the stage is refilled by the next iteration's prefetch
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    pdl_trigger();

    // ---- normalise (softmax), gate, store
    float factor[2] = {1.0f, 1.0f};
    if (!SIGMOID) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float s = row_sum[r];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            factor[r] = s > 0.0f ? 1.0f / s : 0.0f;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row_block + g + r * 8;
        if (row < rows) {
            float f = factor[r];
            if (a.gate && !a.gate_wide) f *= 1.0f / (1.0f + expf(-__bfloat162float(a.gate[(size_t)(first_token + row) * a.gate_ld + head])));
            const __nv_bfloat16* wide = a.gate && a.gate_wide ? a.gate + (size_t)(first_token + row) * a.gate_ld + (size_t)head * DV : nullptr;
            __nv_bfloat16* dst = a.out + (size_t)(first_token + row) * a.out_ld + (size_t)head * DV;
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
                float f0 = f, f1 = f;
                if (wide) {
                    f0 *= 1.0f / (1.0f + expf(-__bfloat162float(wide[i * 8 + t4 * 2])));
                    f1 *= 1.0f / (1.0f + expf(-__bfloat162float(wide[i * 8 + t4 * 2 + 1])));
                }
                *reinterpret_cast<uint32_t*>(dst + i * 8 + t4 * 2) = pack_bf16(o_acc[i][r * 2] * f0, o_acc[i][r * 2 + 1] * f1);
            }
        }
    }
}

template <int DV, bool SIGMOID>
int launch_tiles(const TileArgs& a, int tiles, cudaStream_t stream) {
    const int smem = (BM + 2 * BN) * (a.dim * 2 + 16) + 2 * BN * (DV * 2 + 16);
    auto kernel = masked_tiles_kernel<DV, SIGMOID>;
    static bool configured = false;
    if (!configured) {
        const int most = (BM + 2 * BN) * (MT_MAX_DIM * 2 + 16) + 2 * BN * (DV * 2 + 16);
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    launch_kernel(kernel, dim3(a.heads, tiles), MT_THREADS, smem, stream, a);
    return launch_status();
}

template <int DV>
int launch_weights(const TileArgs& a, int tiles, int sigmoid, cudaStream_t stream) {
    return sigmoid ? launch_tiles<DV, true>(a, tiles, stream) : launch_tiles<DV, false>(a, tiles, stream);
}

}  // namespace

// Whether the tiled kernel takes these head sizes (the caller falls back to the general kernel).
SHISO_API int shiso_masked_attention_tiles_supported(int dim, int vdim) {
    return dim >= 16 && dim <= MT_MAX_DIM && dim % 16 == 0 && vdim >= 16 && vdim <= MT_MAX_VDIM && vdim % 16 == 0;
}

// `max_tiles` >= sum over sequences of ceil(q_len / 64); surplus CTAs exit at once.
SHISO_API int shiso_masked_attention_tiles(const void* q, long long q_ld, const void* k_cache, const void* v_cache, const int* table,
                                           int table_width, const int* q_start, const int* start_pos, void* out, long long out_ld,
                                           const void* gate, long long gate_ld, const float* key_bias, int num_seqs, int max_tiles,
                                           int heads, int kv_heads, int dim, int vdim, int page_size, float scale, float softcap,
                                           int mask_kind, int size, int keep_first, int sigmoid, int gate_wide, cudaStream_t stream) {
    if (num_seqs <= 0 || max_tiles <= 0) return SHISO_OK;
    if (kv_heads <= 0 || heads % kv_heads || size < 1 || keep_first < 0 || (mask_kind != MT_MASK_WINDOW && mask_kind != MT_MASK_CHUNK))
        return SHISO_ERR_SHAPE;
    if (!shiso_masked_attention_tiles_supported(dim, vdim) || max_tiles > 65535) return SHISO_ERR_UNSUPPORTED;
    if ((out_ld % 2) || (((uintptr_t)out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)) return SHISO_ERR_ALIGN;
    TileArgs a;
    a.q = (const __nv_bfloat16*)q;
    a.k_cache = (const __nv_bfloat16*)k_cache;
    a.v_cache = (const __nv_bfloat16*)v_cache;
    a.gate = (const __nv_bfloat16*)gate;
    a.key_bias = key_bias;
    a.block_table = table;
    a.q_start = q_start;
    a.start_pos = start_pos;
    a.out = (__nv_bfloat16*)out;
    a.q_ld = q_ld;
    a.out_ld = out_ld;
    a.gate_ld = gate_ld;
    a.gate_wide = gate_wide;
    a.width = table_width;
    a.num_seqs = num_seqs;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.dim = dim;
    a.page_size = page_size;
    a.mask_kind = mask_kind;
    a.size = size;
    a.keep_first = keep_first;
    a.scale = scale;
    a.softcap = softcap > 0.0f ? softcap : 0.0f;
    switch (vdim) {
        case 16: return launch_weights<16>(a, max_tiles, sigmoid, stream);
        case 32: return launch_weights<32>(a, max_tiles, sigmoid, stream);
        case 48: return launch_weights<48>(a, max_tiles, sigmoid, stream);
        case 64: return launch_weights<64>(a, max_tiles, sigmoid, stream);
        case 80: return launch_weights<80>(a, max_tiles, sigmoid, stream);
        case 96: return launch_weights<96>(a, max_tiles, sigmoid, stream);
        case 112: return launch_weights<112>(a, max_tiles, sigmoid, stream);
        case 128: return launch_weights<128>(a, max_tiles, sigmoid, stream);
        default: return SHISO_ERR_UNSUPPORTED;
    }
}
