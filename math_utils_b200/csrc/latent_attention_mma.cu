// Attention over a cache of latent rows on tensor cores (mma.sync m16n8k16, bfloat16, float32 accumulation).
//
// All heads of a token read the SAME rows, so the (token, head) pairs of a few consecutive tokens of one sequence are
// the rows of one matrix tile: 32 query rows a block.  A page of 64 cached rows [64][width] serves both products:
//   S = Q K^T   with K the page as it lies (row-major, dimension along k),
//   O += P V    with V the first kv_rank columns of the same page (ldmatrix.trans turns them into the k-major operand).
// Eight warps: two groups of 16 query rows times four parts.  For S a warp takes 16 of the page's 64 keys; the row
// maxima and sums of the four parts meet in shared memory; P goes to shared memory as bfloat16; for O a warp takes a
// quarter of the kv_rank output columns over all 64 keys.  Pages arrive by cp.async, the next one while this one is
// worked on.  Softmax state and O stay in float32 registers.  With n_splits > 1 (single-token steps) a block takes a
// share of the pages and leaves an unnormalised partial result for the merge kernel.
//
// TWO (an option for designs that want the softmax's weights at 32 bits): P enters the second product as two bfloat16
// terms, the rounded weight and what the rounding left (some 16 bits of mantissa instead of 8), and the row sums are
// those of the unrounded weights.
//
// Sizes taken: width a multiple of 16, kv_rank = 32 * NT with NT in {2, 4, 8, 12, 16}, pages of 64 positions.
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int LM_ROWS = 32, LM_KEYS = 64, LM_THREADS = 256;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// tiles: int32 [n][2] = (first flat token, count <= 64) of runs of tokens of one sequence, or null: token t alone.
// grid: (tiles * sub-tiles, n_splits, head chunks).
template <int NT, bool TWO>
__global__ void __launch_bounds__(LM_THREADS)
latent_attention_mma_kernel(const float* __restrict__ q, const __nv_bfloat16* __restrict__ rows,
                            const int* __restrict__ block_table, int max_pages, const int* __restrict__ tok_pos,
                            const int* __restrict__ tok_seq, const int* __restrict__ tiles, int n_heads, int width,
                            float scale, int n_splits, __nv_bfloat16* __restrict__ out, long long ldo,
                            float* __restrict__ part_o, float* __restrict__ part_ml, const float* __restrict__ sink) {
    constexpr int KV_RANK = 32 * NT;
    extern __shared__ __align__(16) unsigned char lm_raw[];
    const int w8 = width + 8;                                    // padded row: conflict-free fragment loads
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(lm_raw);            // [2][64][w8]
    __nv_bfloat16* Qs = Ks + 2 * LM_KEYS * w8;                               // [32][w8]
    __nv_bfloat16* Ps = Qs + LM_ROWS * w8;                                   // [32][72]
    __nv_bfloat16* Pl = Ps + LM_ROWS * 72;                                   // [32][72]: what rounding P left (TWO)
    float* red_max = reinterpret_cast<float*>(Pl + LM_ROWS * 72);            // [4][32]
    float* red_sum = red_max + 4 * LM_ROWS;                                  // [4][32]
    int* row_pos = reinterpret_cast<int*>(red_sum + 4 * LM_ROWS);            // [32]
    int* row_src = row_pos + LM_ROWS;                                        // [32] token * n_heads + head, or -1
    pdl_trigger();
    pdl_wait();
    const int heads_here = min(n_heads, LM_ROWS);                // heads per chunk
    const int head0 = blockIdx.z * LM_ROWS;
    const int n_h = min(heads_here, n_heads - head0);
    const int tq = max(1, LM_ROWS / heads_here);                 // tokens per block
    int first, count;
    if (tiles) {
        const int subs = (64 + tq - 1) / tq;
        const int tile = blockIdx.x / subs, sub = blockIdx.x % subs;
        first = tiles[2 * tile] + sub * tq;
        count = min(tq, tiles[2 * tile + 1] - sub * tq);
        if (count <= 0) return;
    } else {
        first = blockIdx.x;
        count = 1;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rg = warp >> 2, g = warp & 3, gq = lane >> 2, t4 = lane & 3;
    const int pos0 = tok_pos[first];
    if (tid < LM_ROWS) {
        const int i = tid / heads_here, h = tid % heads_here;
        const bool valid = i < count && h < n_h;
        row_pos[tid] = valid ? pos0 + i : pos0;
        row_src[tid] = valid ? (first + i) * n_heads + head0 + h : -1;
    }
    __syncthreads();
    // the queries, rounded to bfloat16: a warp a row, lanes along it in pairs (no division; width is even)
    for (int r = warp; r < LM_ROWS; r += LM_THREADS / 32) {
        const int src = row_src[r];
        const float2* from = reinterpret_cast<const float2*>(q + (long long)(src >= 0 ? src : 0) * width);
        __nv_bfloat162* to = reinterpret_cast<__nv_bfloat162*>(Qs + r * w8);
        for (int d = lane; d < width / 2; d += 32) {
            const float2 v = src >= 0 ? from[d] : make_float2(0.0f, 0.0f);
            to[d] = __floats2bfloat162_rn(v.x, v.y);
        }
    }
    const int n_keys = pos0 + count;
    const int n_pages = (n_keys + LM_KEYS - 1) / LM_KEYS;
    const int per = (n_pages + n_splits - 1) / n_splits;
    const int p_lo = blockIdx.y * per, p_hi = min(n_pages, p_lo + per);
    const int* pages = block_table + (long long)tok_seq[first] * max_pages;

    auto load_page = [&](int p, int buf) {
        const __nv_bfloat16* src = rows + (long long)pages[p] * LM_KEYS * width;
        __nv_bfloat16* dst = Ks + buf * LM_KEYS * w8;
        for (int r = warp; r < LM_KEYS; r += LM_THREADS / 32)       // a warp a row, lanes along it: no division
            for (int o = lane * 8; o < width; o += 256) cp_async16(dst + r * w8 + o, src + r * width + o);
        cp_async_commit();
    };

    float o_acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    const int ra = rg * 16 + gq, rb = ra + 8;                    // this thread's two query rows

    if (p_lo < p_hi) load_page(p_lo, 0);
    for (int p = p_lo; p < p_hi; ++p) {
        const int buf = (p - p_lo) & 1;
        if (p + 1 < p_hi) {
            load_page(p + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __nv_bfloat16* K = Ks + buf * LM_KEYS * w8;
        // ---- S = Q K^T for rows rg * 16 .. + 16 and keys g * 16 .. + 16
        float s[2][4] = {};
        // fragments by ldmatrix: Q rows rg * 16 .. (row-major, k along the row), K rows = keys g * 16 .. (the same)
        const __nv_bfloat16* qf = Qs + (rg * 16 + (lane & 15)) * w8 + (lane >> 4) * 8;
        const __nv_bfloat16* kf = K + (g * 16 + (lane & 7) + (lane >> 4) * 8) * w8 + ((lane >> 3) & 1) * 8;
#pragma unroll 4
        for (int k0 = 0; k0 < width; k0 += 16) {
            uint32_t a[4], b[4];
            ldmatrix_x4(a, qf + k0);
            ldmatrix_x4(b, kf + k0);
            mma_bf16(s[0], a[0], a[1], a[2], a[3], b[0], b[1]);
            mma_bf16(s[1], a[0], a[1], a[2], a[3], b[2], b[3]);
        }
        const int pos_a = row_pos[ra], pos_b = row_pos[rb];
        float top_a = -INFINITY, top_b = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int key = p * LM_KEYS + g * 16 + j * 8 + 2 * t4;
            s[j][0] = key <= pos_a ? s[j][0] * scale : -INFINITY;
            s[j][1] = key + 1 <= pos_a ? s[j][1] * scale : -INFINITY;
            s[j][2] = key <= pos_b ? s[j][2] * scale : -INFINITY;
            s[j][3] = key + 1 <= pos_b ? s[j][3] * scale : -INFINITY;
            top_a = fmaxf(top_a, fmaxf(s[j][0], s[j][1]));
            top_b = fmaxf(top_b, fmaxf(s[j][2], s[j][3]));
        }
        top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 1));
        top_a = fmaxf(top_a, __shfl_xor_sync(0xffffffffu, top_a, 2));
        top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 1));
        top_b = fmaxf(top_b, __shfl_xor_sync(0xffffffffu, top_b, 2));
        if (t4 == 0) { red_max[g * LM_ROWS + ra] = top_a; red_max[g * LM_ROWS + rb] = top_b; }
        __syncthreads();
        float new_a = m_a, new_b = m_b;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            new_a = fmaxf(new_a, red_max[i * LM_ROWS + ra]);
            new_b = fmaxf(new_b, red_max[i * LM_ROWS + rb]);
        }
        const float corr_a = new_a == -INFINITY ? 1.0f : expf(m_a - new_a);
        const float corr_b = new_b == -INFINITY ? 1.0f : expf(m_b - new_b);
        float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float p0 = new_a == -INFINITY ? 0.0f : expf(s[j][0] - new_a), p1 = new_a == -INFINITY ? 0.0f : expf(s[j][1] - new_a);
            const float p2 = new_b == -INFINITY ? 0.0f : expf(s[j][2] - new_b), p3 = new_b == -INFINITY ? 0.0f : expf(s[j][3] - new_b);
            const __nv_bfloat162 pa = __floats2bfloat162_rn(p0, p1), pb = __floats2bfloat162_rn(p2, p3);
            const int col = g * 16 + j * 8 + 2 * t4;
            if (TWO) {
                sum_a += p0 + p1;
                sum_b += p2 + p3;
                *reinterpret_cast<__nv_bfloat162*>(Pl + ra * 72 + col) =
                    __floats2bfloat162_rn(p0 - __low2float(pa), p1 - __high2float(pa));
                *reinterpret_cast<__nv_bfloat162*>(Pl + rb * 72 + col) =
                    __floats2bfloat162_rn(p2 - __low2float(pb), p3 - __high2float(pb));
            } else {
                // the sums use what the second product will see: the rounded weights
                sum_a += __low2float(pa) + __high2float(pa);
                sum_b += __low2float(pb) + __high2float(pb);
            }
            *reinterpret_cast<__nv_bfloat162*>(Ps + ra * 72 + col) = pa;
            *reinterpret_cast<__nv_bfloat162*>(Ps + rb * 72 + col) = pb;
        }
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
        if (t4 == 0) { red_sum[g * LM_ROWS + ra] = sum_a; red_sum[g * LM_ROWS + rb] = sum_b; }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            o_acc[i][0] *= corr_a; o_acc[i][1] *= corr_a;
            o_acc[i][2] *= corr_b; o_acc[i][3] *= corr_b;
        }
        m_a = new_a; m_b = new_b;
        __syncthreads();
        l_a = l_a * corr_a + red_sum[ra] + red_sum[LM_ROWS + ra] + red_sum[2 * LM_ROWS + ra] + red_sum[3 * LM_ROWS + ra];
        l_b = l_b * corr_b + red_sum[rb] + red_sum[LM_ROWS + rb] + red_sum[2 * LM_ROWS + rb] + red_sum[3 * LM_ROWS + rb];
        // ---- O += P V for the output columns g * 8 NT .. + 8 NT
        const __nv_bfloat16* pa_ptr = Ps + ra * 72 + 2 * t4;
        const __nv_bfloat16* pb_ptr = Ps + rb * 72 + 2 * t4;
        const __nv_bfloat16* vbase = K + ((lane & 7) + ((lane >> 3) & 1) * 8) * w8 + g * 8 * NT + (lane >> 4) * 8;
#pragma unroll
        for (int k0 = 0; k0 < LM_KEYS; k0 += 16) {
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(pa_ptr + k0), a1 = *reinterpret_cast<const uint32_t*>(pb_ptr + k0);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(pa_ptr + k0 + 8), a3 = *reinterpret_cast<const uint32_t*>(pb_ptr + k0 + 8);
            uint32_t l0 = 0u, l1 = 0u, l2 = 0u, l3 = 0u;
            if (TWO) {
                const __nv_bfloat16* la = Pl + ra * 72 + 2 * t4 + k0;
                const __nv_bfloat16* lb = Pl + rb * 72 + 2 * t4 + k0;
                l0 = *reinterpret_cast<const uint32_t*>(la), l1 = *reinterpret_cast<const uint32_t*>(lb);
                l2 = *reinterpret_cast<const uint32_t*>(la + 8), l3 = *reinterpret_cast<const uint32_t*>(lb + 8);
            }
#pragma unroll
            for (int i = 0; i < NT; i += 2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vbase + k0 * w8 + i * 8);
                mma_bf16(o_acc[i], a0, a1, a2, a3, b[0], b[1]);
                mma_bf16(o_acc[i + 1], a0, a1, a2, a3, b[2], b[3]);
                if (TWO) {
                    mma_bf16(o_acc[i], l0, l1, l2, l3, b[0], b[1]);
                    mma_bf16(o_acc[i + 1], l0, l1, l2, l3, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    const int src_a = row_src[ra], src_b = row_src[rb];
    if (n_splits == 1) {
        float inv_a = 1.0f / l_a, inv_b = 1.0f / l_b;
        if (sink) {
            // exp(sink[head]) joins the denominator (no value behind it); with splits the merge kernel adds it
            if (src_a >= 0) {
                const float sk = sink[src_a % n_heads], top = fmaxf(m_a, sk), f = expf(m_a - top);
                inv_a = f / (l_a * f + expf(sk - top));
            }
            if (src_b >= 0) {
                const float sk = sink[src_b % n_heads], top = fmaxf(m_b, sk), f = expf(m_b - top);
                inv_b = f / (l_b * f + expf(sk - top));
            }
        }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int d = g * 8 * NT + i * 8 + 2 * t4;
            if (src_a >= 0)
                *reinterpret_cast<__nv_bfloat162*>(out + (long long)(src_a / n_heads) * ldo + (src_a % n_heads) * KV_RANK + d) =
                    __floats2bfloat162_rn(o_acc[i][0] * inv_a, o_acc[i][1] * inv_a);
            if (src_b >= 0)
                *reinterpret_cast<__nv_bfloat162*>(out + (long long)(src_b / n_heads) * ldo + (src_b % n_heads) * KV_RANK + d) =
                    __floats2bfloat162_rn(o_acc[i][2] * inv_b, o_acc[i][3] * inv_b);
        }
        return;
    }
    const int split = blockIdx.y;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int d = g * 8 * NT + i * 8 + 2 * t4;
        if (src_a >= 0)
            *reinterpret_cast<float2*>(part_o + ((long long)src_a * n_splits + split) * KV_RANK + d) = make_float2(o_acc[i][0], o_acc[i][1]);
        if (src_b >= 0)
            *reinterpret_cast<float2*>(part_o + ((long long)src_b * n_splits + split) * KV_RANK + d) = make_float2(o_acc[i][2], o_acc[i][3]);
    }
    if (g == 0 && t4 == 0) {
        if (src_a >= 0) { part_ml[((long long)src_a * n_splits + split) * 2] = m_a; part_ml[((long long)src_a * n_splits + split) * 2 + 1] = l_a; }
        if (src_b >= 0) { part_ml[((long long)src_b * n_splits + split) * 2] = m_b; part_ml[((long long)src_b * n_splits + split) * 2 + 1] = l_b; }
    }
}

inline size_t lm_smem(int width) {
    return (size_t)(2 * LM_KEYS + LM_ROWS) * (width + 8) * 2 + 2 * LM_ROWS * 72 * 2 + 2 * 4 * LM_ROWS * 4 + 2 * LM_ROWS * 4;
}

template <int NT, bool TWO>
int launch_lm(dim3 grid, size_t smem, cudaStream_t s, const float* q, const __nv_bfloat16* rows, const int* block_table,
              int max_pages, const int* tok_pos, const int* tok_seq, const int* tiles, int n_heads, int width, float scale,
              int n_splits, __nv_bfloat16* out, long long ldo, float* part_o, float* part_ml, const float* sink) {
    static bool set = false;
    if (!set) {
        if (cudaFuncSetAttribute(latent_attention_mma_kernel<NT, TWO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
            cudaSuccess)
            return MU_ERR_LAUNCH;
        set = true;
    }
    return launch_pdl(latent_attention_mma_kernel<NT, TWO>, grid, dim3(LM_THREADS), smem, s, 1, q, rows, block_table, max_pages,
                      tok_pos, tok_seq, tiles, n_heads, width, scale, n_splits, out, ldo, part_o, part_ml,
                      n_splits == 1 ? sink : nullptr);
}

}  // namespace mu

// Whether mu_latent_attention_mma takes these sizes.
MU_EXPORT int mu_latent_attention_mma_fits(int kv_rank, int width, int page_tokens) {
    const int nt = kv_rank / 32;
    return page_tokens == 64 && kv_rank % 32 == 0 && (nt == 2 || nt == 4 || nt == 8 || nt == 12 || nt == 16) &&
           width % 16 == 0 && width >= kv_rank && mu::lm_smem(width) <= 200 * 1024;
}

// q float32 [n_tokens][n_heads][width]; out bfloat16 [n_tokens][ldo], head h at columns h * kv_rank.
// tiles (n_tiles of them) for steps with several tokens a sequence; null: every token is a sequence's one token.
// With n_splits > 1 the partial results go to part_o / part_ml, for mu_latent_merge.  sink (one float per head, or
// null): exp(sink[h]) joins head h's softmax denominator; with splits it is the merge that adds it.  two_term: the
// softmax's weights enter the second product as two bfloat16 terms.
MU_EXPORT int mu_latent_attention_mma(const float* q, const void* rows, const int* block_table, int max_pages,
                                      const int* tok_pos, const int* tok_seq, const int* tiles, int n_tiles, int n_tokens,
                                      int n_heads, int kv_rank, int width, float scale, int n_splits, void* out,
                                      long long ldo, float* part_o, float* part_ml, void* stream, const float* sink,
                                      int two_term) {
    if (n_tokens <= 0) return MU_OK;
    if (!q || !rows || !block_table || !tok_pos || !tok_seq || !out || n_heads <= 0 || n_splits < 1 || n_splits > 65535 ||
        (n_splits > 1 && (!part_o || !part_ml || tiles)) || (tiles && n_tiles <= 0) || (ldo & 1))
        return MU_ERR_BAD_ARGUMENT;
    if (!mu_latent_attention_mma_fits(kv_rank, width, 64)) return MU_ERR_UNSUPPORTED_SIZE;
    const int heads_here = n_heads < mu::LM_ROWS ? n_heads : mu::LM_ROWS;
    const int tq = mu::LM_ROWS / heads_here > 1 ? mu::LM_ROWS / heads_here : 1;
    const int subs = (64 + tq - 1) / tq;
    const dim3 grid(tiles ? n_tiles * subs : n_tokens, n_splits, (n_heads + mu::LM_ROWS - 1) / mu::LM_ROWS);
    const size_t smem = mu::lm_smem(width);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define MU_LM(N)                                                                                                       \
    case N:                                                                                                            \
        if (two_term)                                                                                                  \
            return mu::launch_lm<N, true>(grid, smem, s, q, (const bf*)rows, block_table, max_pages, tok_pos, tok_seq, \
                                          tiles, n_heads, width, scale, n_splits, (bf*)out, ldo, part_o, part_ml, sink); \
        return mu::launch_lm<N, false>(grid, smem, s, q, (const bf*)rows, block_table, max_pages, tok_pos, tok_seq,    \
                                       tiles, n_heads, width, scale, n_splits, (bf*)out, ldo, part_o, part_ml, sink);
    switch (kv_rank / 32) { MU_LM(2) MU_LM(4) MU_LM(8) MU_LM(12) MU_LM(16) }
#undef MU_LM
    return MU_ERR_UNSUPPORTED_SIZE;
}
