// Products in batches of small matrices, and the routing of a mixture of experts.
//
// tile_gemm_kernel: out[m, b, :] = W[b] x[m, b, :] for batches b that are either the heads of one
// row (x, out: [M, batches, .] with row and batch strides) or experts that own a range of rows
// (rows grouped by expert, the ranges given by per-expert counts; the input row of grouped row m is
// gather[m] / gather_div).  CUDA cores, float accumulation, a tile of 32 rows x 64 outputs per CTA
// and 32 columns of K per pass; an output's sum runs over K in order, whatever else is in its tile, so
// a row's result does not depend on the batch.  Epilogues: none; times sigmoid(gate[m, b]); or, for
// a matrix that stacks gate over up rows, the gated pair glu_pair(gate, up): silu(gate) * up, the
// tanh form of gelu(gate) * up, or the clamped pair min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1).
// bfloat16 inputs whose strides allow 16-byte copies take tile_gemm_mma_kernel instead: the same
// tiles on the tensor cores.
//
// Routing: moe_route_kernel (a warp per row: scores, group-limited choice of the top experts by
// score + correction, weights), moe_count / moe_place (rows grouped by expert with two passes of
// integer atomics: which place a row gets inside its expert's range is arbitrary, its arithmetic is
// not touched by it), moe_combine_kernel (a token's weighted sum over its choices, in the order of
// the choices; a choice beyond the experts with matrices is an identity expert and adds the
// token's input itself).
#include "common.cuh"

#define TG_BM 32
#define TG_BN 64
#define TG_BK 32
#define MOE_MAX_EXPERTS 256
#define MOE_MAX_TOP 16

enum { GLU_SILU = 0, GLU_GELU_TANH = 1, GLU_SWISH_CLAMPED = 2 };

// The gated pair of a feed-forward, in float with the library's expf and tanhf.
__device__ __forceinline__ float glu_pair(float g, float u, int act, float limit) {
    if (act == GLU_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    if (act == GLU_SWISH_CLAMPED) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
    }
    return g / (1.0f + expf(-g)) * u;
}

struct TileGemmArgs {
    const void* x;
    long long x_ld, x_bs;
    const int* gather;
    int gather_div;
    const void* w;
    long long w_bs;
    void* out;
    long long out_ld, out_bs;
    const int* counts;  // per-batch row counts (rows grouped by batch), or nullptr: every batch has rows 0..M-1
    const void* gate;
    long long gate_ld;
    int M, N, K, batches;
    int act;      // the gated pair of a stacked gate/up matrix (GLU_*)
    float limit;  // its clamp
};

template <typename XT, typename WT, typename OT, bool GLU>
__global__ void __launch_bounds__(256) tile_gemm_kernel(const TileGemmArgs a) {
    __shared__ float xs[TG_BK][TG_BM + 1];
    __shared__ float ws[GLU ? 2 : 1][TG_BK][TG_BN + 1];
    __shared__ int s_batch, s_row0, s_rows;
    const int tid = threadIdx.x;
    pdl_wait();
    int batch, row0, row_end;
    if (a.counts) {
        // blockIdx.y counts row tiles over all batches: find the batch this tile falls into
        if (tid == 0) {
            int tile = blockIdx.y, start = 0, b = 0, found = -1;
            for (; b < a.batches; ++b) {
                const int c = a.counts[b], tiles = (c + TG_BM - 1) / TG_BM;
                if (tile < tiles) { found = b; break; }
                tile -= tiles;
                start += c;
            }
            s_batch = found;
            s_row0 = start + tile * TG_BM;
            s_rows = found >= 0 ? start + a.counts[found] : 0;
        }
        __syncthreads();
        batch = s_batch, row0 = s_row0, row_end = s_rows;
        if (batch < 0) return;
    } else {
        batch = blockIdx.z, row0 = blockIdx.y * TG_BM, row_end = a.M;
        if (row0 >= row_end) return;
    }
    const int n0 = blockIdx.x * TG_BN;
    const XT* x = (const XT*)a.x + (size_t)batch * a.x_bs;
    const WT* w = (const WT*)a.w + (size_t)batch * a.w_bs;
    const int ty = tid >> 4, tx = tid & 15;  // rows ty*2, ty*2+1; outputs tx + 16 j
    float acc[2][4] = {}, acc2[2][4] = {};
    // which input row each of this thread's loads comes from (fixed over the K loop)
    const int lrow = tid >> 3, lk = (tid & 7) * 4;  // x tile: 32 rows x 32 k: 8 threads a row, 4 k each
    long long xrow = -1;
    if (row0 + lrow < row_end) {
        const int m = row0 + lrow;
        xrow = a.gather ? a.gather[m] / a.gather_div : m;
    }
    for (int k0 = 0; k0 < a.K; k0 += TG_BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            xs[lk + e][lrow] = (xrow >= 0 && k < a.K) ? to_f32(x[(size_t)xrow * a.x_ld + k]) : 0.0f;
        }
        // w tile: 64 outputs x 32 k: 4 threads an output row, 8 k each
        {
            const int wn = tid >> 2, wk = (tid & 3) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const int k = k0 + wk + e, n = n0 + wn;
                const bool ok = n < a.N && k < a.K;
                ws[0][wk + e][wn] = ok ? to_f32(w[(size_t)n * a.K + k]) : 0.0f;
                if (GLU) ws[1][wk + e][wn] = ok ? to_f32(w[(size_t)(a.N + n) * a.K + k]) : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TG_BK; ++k) {
            const float x0 = xs[k][ty * 2], x1 = xs[k][ty * 2 + 1];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float wv = ws[0][k][tx + 16 * j];
                acc[0][j] = fmaf(x0, wv, acc[0][j]);
                acc[1][j] = fmaf(x1, wv, acc[1][j]);
                if (GLU) {
                    const float uv = ws[1][k][tx + 16 * j];
                    acc2[0][j] = fmaf(x0, uv, acc2[0][j]);
                    acc2[1][j] = fmaf(x1, uv, acc2[1][j]);
                }
            }
        }
        __syncthreads();
    }
    pdl_trigger();
    OT* out = (OT*)a.out + (size_t)batch * a.out_bs;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = row0 + ty * 2 + i;
        if (m >= row_end) continue;
        float scale = 1.0f;
        if (a.gate) scale = 1.0f / (1.0f + expf(-to_f32(((const XT*)a.gate)[(size_t)m * a.gate_ld + batch])));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (GLU) v = glu_pair(v, acc2[i][j], a.act, a.limit);
            out[(size_t)m * a.out_ld + n] = from_f32<OT>(v * scale);
        }
    }
}

// ---- the same products on the tensor cores (bfloat16 inputs) -------------------------------
// 64 rows x 128 outputs per CTA and 32 columns of K per stage, eight warps of 32 x 32 outputs,
// mma.sync m16n8k16 with float accumulators; rows (gathered through the same index) and matrix rows
// come by 16-byte cp.async into four stages of padded shared-memory rows that ldmatrix reads without
// bank conflicts.  With a stacked gate/up matrix both halves are accumulated and the epilogue
// writes silu(gate) * up.  Needs K, the row strides and the batch strides to be multiples of 8.
#define TM_BM 64
#define TM_BN 128
#define TM_BK 32
#define TM_ROW (TM_BK * 2 + 16)  // bytes of a padded shared-memory row: TM_BK bfloat16 + 16 bytes
#define TM_STAGES 4
#define TM_PIECES (TM_BK / 8)  // 16-byte pieces of a row

__device__ __forceinline__ uint32_t tm_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tm_cp16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tm_smem(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tm_ldmatrix(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void tm_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename OT, bool GLU>
__global__ void __launch_bounds__(256) tile_gemm_mma_kernel(const TileGemmArgs a) {
    extern __shared__ __align__(16) uint8_t tm_sm[];
    uint8_t* xs = tm_sm;                                  // [TM_STAGES][TM_BM][TM_ROW]
    uint8_t* ws = xs + TM_STAGES * TM_BM * TM_ROW;        // [TM_STAGES][(GLU ? 2 : 1) * TM_BN][TM_ROW]
    constexpr int WROWS = (GLU ? 2 : 1) * TM_BN;
    __shared__ int s_batch, s_row0, s_rows;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    int batch, row0, row_end;
    if (a.counts) {
        if (tid == 0) {
            int tile = blockIdx.y, start = 0, b = 0, found = -1;
            for (; b < a.batches; ++b) {
                const int c = a.counts[b], tiles = (c + TM_BM - 1) / TM_BM;
                if (tile < tiles) { found = b; break; }
                tile -= tiles;
                start += c;
            }
            s_batch = found;
            s_row0 = start + tile * TM_BM;
            s_rows = found >= 0 ? start + a.counts[found] : 0;
        }
        __syncthreads();
        batch = s_batch, row0 = s_row0, row_end = s_rows;
        if (batch < 0) return;
    } else {
        batch = blockIdx.z, row0 = blockIdx.y * TM_BM, row_end = a.M;
        if (row0 >= row_end) return;
    }
    const int n0 = blockIdx.x * TM_BN;
    const __nv_bfloat16* x = (const __nv_bfloat16*)a.x + (size_t)batch * a.x_bs;
    const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)batch * a.w_bs;
    // this thread's copies per stage: TM_BM * TM_PIECES / 256 pieces of input rows, WROWS * TM_PIECES / 256 of matrix rows
    constexpr int XCOPIES = TM_BM * TM_PIECES / 256, WCOPIES = WROWS * TM_PIECES / 256;
    const __nv_bfloat16* xsrc[XCOPIES];
#pragma unroll
    for (int i = 0; i < XCOPIES; ++i) {
        const int r = (tid + i * 256) / TM_PIECES;
        xsrc[i] = nullptr;
        if (row0 + r < row_end) {
            const int m = row0 + r;
            xsrc[i] = x + (size_t)(a.gather ? a.gather[m] / a.gather_div : m) * a.x_ld;
        }
    }
    auto load = [&](int k0, int stage) {
#pragma unroll
        for (int i = 0; i < XCOPIES; ++i) {
            const int idx = tid + i * 256, r = idx / TM_PIECES, piece = idx % TM_PIECES, k = k0 + piece * 8;
            const bool ok = xsrc[i] != nullptr && k < a.K;
            tm_cp16(xs + (stage * TM_BM + r) * TM_ROW + piece * 16, ok ? xsrc[i] + k : x, ok);
        }
#pragma unroll
        for (int i = 0; i < WCOPIES; ++i) {
            const int idx = tid + i * 256, r = idx / TM_PIECES, piece = idx % TM_PIECES, k = k0 + piece * 8;
            const int half = r / TM_BN, n = n0 + r % TM_BN;  // rows of the stage: gate rows, then up rows
            const bool ok = n < a.N && k < a.K;
            tm_cp16(ws + (stage * WROWS + r) * TM_ROW + piece * 16, ok ? w + ((size_t)half * a.N + n) * a.K + k : w, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int wm = warp >> 2, wn = warp & 3;
    float acc[2][4][4] = {}, acc2[GLU ? 2 : 1][4][4] = {};
    const int steps = (a.K + TM_BK - 1) / TM_BK;
    // the next stages are on their way while stage s is worked on; one barrier a step: when a
    // thread passes it, stage s has landed for everybody and nobody still reads stage s - 1,
    // which is the one the next copies fill
#pragma unroll
    for (int p = 0; p < TM_STAGES - 1; ++p) {
        if (p < steps) load(p * TM_BK, p);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int s = 0; s < steps; ++s) {
        const int stage = s % TM_STAGES;
        asm volatile("cp.async.wait_group %0;" ::"n"(TM_STAGES - 2) : "memory");
        __syncthreads();
        if (s + TM_STAGES - 1 < steps) load((s + TM_STAGES - 1) * TM_BK, (s + TM_STAGES - 1) % TM_STAGES);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const uint8_t* xt = xs + stage * TM_BM * TM_ROW;
        const uint8_t* wt = ws + stage * WROWS * TM_ROW;
#pragma unroll
        for (int kk = 0; kk < TM_BK / 16; ++kk) {
            uint32_t af[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) {
                const int r = wm * 32 + mi * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int col = kk * 16 + (lane >> 4) * 8;
                tm_ldmatrix(tm_smem(xt + r * TM_ROW + col * 2), af[mi][0], af[mi][1], af[mi][2], af[mi][3]);
            }
#pragma unroll
            for (int nj = 0; nj < 4; nj += 2) {
                const int r = wn * 32 + nj * 8 + (lane & 7) + (lane >> 4) * 8;
                const int col = kk * 16 + ((lane >> 3) & 1) * 8;
                uint32_t b0, b1, b2, b3;
                tm_ldmatrix(tm_smem(wt + r * TM_ROW + col * 2), b0, b1, b2, b3);
#pragma unroll
                for (int mi = 0; mi < 2; ++mi) {
                    tm_mma(acc[mi][nj], af[mi], b0, b1);
                    tm_mma(acc[mi][nj + 1], af[mi], b2, b3);
                }
                if (GLU) {
                    tm_ldmatrix(tm_smem(wt + (TM_BN + r) * TM_ROW + col * 2), b0, b1, b2, b3);
#pragma unroll
                    for (int mi = 0; mi < 2; ++mi) {
                        tm_mma(acc2[mi][nj], af[mi], b0, b1);
                        tm_mma(acc2[mi][nj + 1], af[mi], b2, b3);
                    }
                }
            }
        }
    }
    pdl_trigger();
    OT* out = (OT*)a.out + (size_t)batch * a.out_bs;
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int m = row0 + wm * 32 + mi * 16 + g + hrow * 8;
            if (m >= row_end) continue;
            float scale = 1.0f;
            if (a.gate) scale = 1.0f / (1.0f + expf(-to_f32(((const __nv_bfloat16*)a.gate)[(size_t)m * a.gate_ld + batch])));
#pragma unroll
            for (int nj = 0; nj < 4; ++nj) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn * 32 + nj * 8 + t4 * 2 + e;
                    if (n >= a.N) continue;
                    float v = acc[mi][nj][hrow * 2 + e];
                    if (GLU) v = glu_pair(v, acc2[mi][nj][hrow * 2 + e], a.act, a.limit);
                    out[(size_t)m * a.out_ld + n] = from_f32<OT>(v * scale);
                }
            }
        }
    }
}

template <typename OT, bool GLU>
static int launch_tile_gemm_mma(const TileGemmArgs& a, int rows_upper, int extra_tiles, int z, cudaStream_t stream) {
    const dim3 grid((a.N + TM_BN - 1) / TM_BN, (rows_upper + TM_BM - 1) / TM_BM + extra_tiles, z);
    const size_t smem = (size_t)TM_STAGES * (TM_BM + (GLU ? 2 : 1) * TM_BN) * TM_ROW;
    auto kern = tile_gemm_mma_kernel<OT, GLU>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kern, grid, dim3(256), smem, stream, a);
    return launch_status();
}

static bool tile_gemm_mma_fits(const TileGemmArgs& a, int x_dtype, int w_dtype) {
    return x_dtype == SHISO_BF16 && w_dtype == SHISO_BF16 && a.K % 8 == 0 && a.x_ld % 8 == 0 && a.x_bs % 8 == 0 && a.w_bs % 8 == 0 &&
           (((uintptr_t)a.x | (uintptr_t)a.w) & 15) == 0;
}

template <bool GLU>
static int launch_tile_gemm(const TileGemmArgs& a, int x_dtype, int w_dtype, int out_dtype, int rows_upper, int extra_tiles, int z,
                            cudaStream_t stream) {
    // rows_upper rows in all; with rows grouped by batch, every batch may end in a tile that is not full (extra_tiles)
    if (tile_gemm_mma_fits(a, x_dtype, w_dtype)) {
        if (out_dtype == SHISO_BF16) return launch_tile_gemm_mma<__nv_bfloat16, GLU>(a, rows_upper, extra_tiles, z, stream);
        if (out_dtype == SHISO_F32) return launch_tile_gemm_mma<float, GLU>(a, rows_upper, extra_tiles, z, stream);
    }
    const dim3 grid((a.N + TG_BN - 1) / TG_BN, (rows_upper + TG_BM - 1) / TG_BM + extra_tiles, z);
    typedef __nv_bfloat16 bf;
#define TG_GO(XT, WT, OT)                                                                 \
    {                                                                                     \
        launch_kernel(tile_gemm_kernel<XT, WT, OT, GLU>, grid, dim3(256), 0, stream, a);  \
        return launch_status();                                                           \
    }
    if (x_dtype == SHISO_F32 && w_dtype == SHISO_F32 && out_dtype == SHISO_F32) TG_GO(float, float, float)
    if (x_dtype == SHISO_BF16 && w_dtype == SHISO_BF16 && out_dtype == SHISO_BF16) TG_GO(bf, bf, bf)
    if (x_dtype == SHISO_BF16 && w_dtype == SHISO_BF16 && out_dtype == SHISO_F32) TG_GO(bf, bf, float)
    if (x_dtype == SHISO_BF16 && w_dtype == SHISO_F32 && out_dtype == SHISO_BF16) TG_GO(bf, float, bf)
    if (x_dtype == SHISO_BF16 && w_dtype == SHISO_F32 && out_dtype == SHISO_F32) TG_GO(bf, float, float)
#undef TG_GO
    return SHISO_ERR_DTYPE;
}

// out[t, h, :] = W[h] x[t, h, :] (times sigmoid(gate[t, h])): x [T, H, K] and out [T, H, N] with row and head strides.
SHISO_API int shiso_head_linear(const void* x, long long x_ld, long long x_hs, int x_dtype, const void* w, int w_dtype, void* out,
                                long long out_ld, long long out_hs, int out_dtype, const void* gate, long long gate_ld, int tokens,
                                int heads, int n, int k, cudaStream_t stream) {
    if (tokens <= 0 || heads <= 0 || n <= 0) return SHISO_OK;
    if (k <= 0 || heads > 65535) return SHISO_ERR_SHAPE;
    TileGemmArgs a = {x, x_ld, x_hs, nullptr, 1, w, (long long)n * k, out, out_ld, out_hs, nullptr, gate, gate_ld, tokens, n, k, heads};
    return launch_tile_gemm<false>(a, x_dtype, w_dtype, out_dtype, tokens, 0, heads, stream);
}

// --------------------------------------------------------------------------- routing

// A warp per row.  scores = softmax(logits) (or sigmoids); experts and groups are ranked by the
// choice score = score + correction[e] (which may be negative); experts in `group_count` groups of
// neighbours, a group's value its largest choice score; the `group_keep` best groups stay; among
// their experts the `top` largest choice scores win (the lower index on a tie); weight = score
// (/ (the chosen scores' sum + renorm_eps)) * scale.  Rows of logits are `ld` apart.
__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction,
                                 int* __restrict__ ids, float* __restrict__ weights, int tokens, int experts, int top,
                                 int group_count, int group_keep, float scale, int sigmoid, int renormalize, float renorm_eps) {
    pdl_begin();
    __shared__ float s_scores[8][MOE_MAX_EXPERTS];
    __shared__ float s_choice[8][MOE_MAX_EXPERTS];  // NaN once taken: no comparison picks it again
    __shared__ float s_group[8][MOE_MAX_EXPERTS];   // a group's best choice score; NaN once kept
    __shared__ unsigned char s_kept[8][MOE_MAX_EXPERTS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 8 + warp;
    if (t >= tokens) return;
    float* sc = s_scores[warp];
    float* ch = s_choice[warp];
    float* gs = s_group[warp];
    unsigned char* kept = s_kept[warp];
    const float* z = logits + (size_t)t * ld;
    float mx = -INFINITY;
    for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < experts; e += 32) {
        const float v = sigmoid ? 1.0f / (1.0f + expf(-z[e])) : expf(z[e] - mx);
        sc[e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    const float inv = sigmoid ? 1.0f : 1.0f / sum;
    for (int e = lane; e < experts; e += 32) {
        const float v = sc[e] * inv;
        sc[e] = v;
        ch[e] = correction ? v + correction[e] : v;
    }
    __syncwarp();
    const int per = experts / group_count;
    for (int g = lane; g < group_count; g += 32) {
        float best = -INFINITY;
        for (int e = 0; e < per; ++e) best = fmaxf(best, ch[g * per + e]);
        gs[g] = best;
        kept[g] = 0;
    }
    __syncwarp();
    for (int r = 0; r < group_keep; ++r) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int g = lane; g < group_count; g += 32) {
            const float v = gs[g];
            if (v > best || (v == best && g < at)) best = v, at = g;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
        }
        if (lane == 0 && at < group_count) gs[at] = NAN, kept[at] = 1;
        __syncwarp();
    }
    float chosen_sum = 0.0f;
    float my_w = 0.0f;
    int my_id = 0;
    for (int r = 0; r < top; ++r) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = ch[e];
            if (kept[e / per] && (v > best || (v == best && e < at))) best = v, at = e;
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ov > best || (ov == best && oa < at)) best = ov, at = oa;
        }
        if (at >= experts) at = 0;  // cannot happen while the kept groups hold `top` experts
        const float score = sc[at];
        chosen_sum += score;
        if (lane == r) my_w = score, my_id = at;
        __syncwarp();
        if (lane == 0) ch[at] = NAN;  // taken
        __syncwarp();
    }
    if (lane < top) {
        ids[(size_t)t * top + lane] = my_id;
        weights[(size_t)t * top + lane] = (renormalize ? my_w / (chosen_sum + renorm_eps) : my_w) * scale;
    }
}

SHISO_API int shiso_moe_route(const float* logits, long long ld, const float* correction, int* ids, float* weights, int tokens,
                              int experts, int top, int group_count, int group_keep, float scale, int sigmoid, int renormalize,
                              float renorm_eps, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    if (experts <= 0 || experts > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP || top > experts || group_count <= 0 ||
        experts % group_count || group_keep <= 0 || group_keep > group_count || group_keep * (experts / group_count) < top ||
        ld < experts)
        return SHISO_ERR_SHAPE;
    launch_kernel(moe_route_kernel, ceil_div_u(tokens, 8), 256, 0, stream, logits, ld, correction, ids, weights, tokens, experts, top,
                  group_count, group_keep, scale, sigmoid, renormalize, renorm_eps);
    return launch_status();
}

__global__ void moe_zero_kernel(int* __restrict__ counts, int experts) {
    pdl_begin();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
}

__global__ void moe_count_kernel(const int* __restrict__ ids, int* __restrict__ counts, int* __restrict__ rank, int total) {
    pdl_begin();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) rank[i] = atomicAdd(&counts[ids[i]], 1);
}

// place[i] = first row of the choice's expert + its rank there; source[place] = i
__global__ void moe_place_kernel(const int* __restrict__ ids, const int* __restrict__ counts, const int* __restrict__ rank,
                                 int* __restrict__ place, int* __restrict__ source, int total, int experts) {
    pdl_begin();
    __shared__ int first[MOE_MAX_EXPERTS];
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < experts; ++e) {
            first[e] = at;
            at += counts[e];
        }
    }
    __syncthreads();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int p = first[ids[i]] + rank[i];
    place[i] = p;
    source[p] = i;
}

// out[t] = extra[t] (* sigmoid(extra_gate[t])) + sum_j weights[t, j] * y[place[t * top + j]], the choices in
// their order; a choice whose id is `experts` or more is an identity expert: it adds weights[t, j] * x[t].
template <typename AT>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ place, const float* __restrict__ weights,
                                   const int* __restrict__ ids, const AT* __restrict__ x, const AT* __restrict__ extra,
                                   const float* __restrict__ extra_gate, long long extra_gate_ld, AT* __restrict__ out, int tokens,
                                   int hidden, int top, int experts) {
    pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)tokens * hidden) return;
    const int t = (int)(i / hidden), c = (int)(i % hidden);
    float acc = 0.0f;
    for (int j = 0; j < top; ++j) {
        const size_t at = (size_t)t * top + j;
        const float v = ids[at] >= experts ? to_f32(x[i]) : y[(size_t)place[at] * hidden + c];
        acc = fmaf(weights[at], v, acc);
    }
    if (extra) {
        float e = to_f32(extra[i]);
        if (extra_gate) e *= 1.0f / (1.0f + expf(-extra_gate[(size_t)t * extra_gate_ld]));
        acc += e;
    }
    out[i] = from_f32<AT>(acc);
}

// The experts of one step.  ids / weights [T, top]; gate_up [E, 2 ff, hidden]; down [E, hidden, ff];
// ids from E up to E + identity - 1 are identity experts (no matrices: their rows are grouped
// behind the others' and never multiplied); `act` / `limit`: the experts' gated pair; extra: rows
// added to every token (a shared expert's), times sigmoid(extra_gate[t * extra_gate_ld]) if given.
// scratch: ints [E + identity + 3 * T * top], mid [T * top, ff] (activation type), y [T * top, hidden] (float).
SHISO_API int shiso_routed_experts(const void* x, int act_dtype, const int* ids, const float* weights, const void* gate_up,
                                   const void* down, int w_dtype, const void* extra, const float* extra_gate,
                                   long long extra_gate_ld, void* out, int* ints, void* mid, float* y, int tokens, int hidden, int ff,
                                   int experts, int identity, int top, int act, float limit, cudaStream_t stream) {
    if (tokens <= 0) return SHISO_OK;
    const int outputs = experts + identity;
    if (experts <= 0 || identity < 0 || outputs > MOE_MAX_EXPERTS || top <= 0 || hidden <= 0 || ff <= 0 || act < GLU_SILU ||
        act > GLU_SWISH_CLAMPED)
        return SHISO_ERR_SHAPE;
    const int total = tokens * top;
    int* counts = ints;
    int* rank = ints + outputs;
    int* place = rank + total;
    int* source = place + total;
    launch_kernel(moe_zero_kernel, 1, 256, 0, stream, counts, outputs);
    launch_kernel(moe_count_kernel, ceil_div_u(total, 256), 256, 0, stream, ids, counts, rank, total);
    launch_kernel(moe_place_kernel, ceil_div_u(total, 256), 256, 0, stream, ids, (const int*)counts, (const int*)rank, place, source,
                  total, outputs);
    int status = launch_status();
    if (status) return status;
    TileGemmArgs up = {x, hidden, 0, source, top, gate_up, (long long)2 * ff * hidden, mid, ff, 0, counts, nullptr, 0, total, ff, hidden, experts, act, limit};
    status = launch_tile_gemm<true>(up, act_dtype, w_dtype, act_dtype, total, experts, 1, stream);
    if (status) return status;
    TileGemmArgs dn = {mid, ff, 0, nullptr, 1, down, (long long)hidden * ff, y, hidden, 0, counts, nullptr, 0, total, hidden, ff, experts, 0, 0.0f};
    status = launch_tile_gemm<false>(dn, act_dtype, w_dtype, SHISO_F32, total, experts, 1, stream);
    if (status) return status;
    const unsigned blocks = ceil_div_u((long long)tokens * hidden, 256);
    if (act_dtype == SHISO_F32)
        launch_kernel(moe_combine_kernel<float>, blocks, 256, 0, stream, (const float*)y, (const int*)place, weights, ids,
                      (const float*)x, (const float*)extra, extra_gate, extra_gate_ld, (float*)out, tokens, hidden, top, experts);
    else if (act_dtype == SHISO_BF16)
        launch_kernel(moe_combine_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const float*)y, (const int*)place, weights, ids,
                      (const __nv_bfloat16*)x, (const __nv_bfloat16*)extra, extra_gate, extra_gate_ld, (__nv_bfloat16*)out, tokens,
                      hidden, top, experts);
    else
        return SHISO_ERR_DTYPE;
    return launch_status();
}
