// What an attention layer does to its projections before the cache, for designs that norm a WHOLE projection:
//
// mu_qkv_norm_rows   per token: the queries [q_width] are brought to unit rms over all their entries at once (eps
//                    inside the root), multiplied by a weight of q_width entries and written back in place; the
//                    keys [k_width] likewise with their own weight, into the token's cache row; each kv head's
//                    values are brought to unit rms over their vdim entries (no weight; optional) and go behind the
//                    keys.  The cache row is mapped_attention.cu's with one score map:
//                        row = [ keys: kv head 0, kv head 1, ... | values: kv head 0, kv head 1, ... ].
//                    Values shared between layers (`first`, float32 [T][kv heads * vdim], rows of this step's tokens):
//                    mode 1 writes the layer's values there; mode 2 replaces the layer's values by
//                    (1 - lambda) v + lambda first before they reach the cache.  Statistics, norms and the blend are
//                    float32; the cache row is rounded once.  Queries, keys and values go to blocks of their own,
//                    and a block reads its part of the row once.
// mu_residual_add_norm   x += m * y on the float32 residual stream (y a sublayer's float32 output; y null: nothing is
//                    added), then h = x / sqrt(mean(x^2) + eps) * w in the compute dtype: the join of one sublayer and
//                    the input norm of the next in one pass over the row.  With w null only the addition is made.
#include "common.cuh"

#include <math.h>

namespace mu {

constexpr int QN_KEEP = 8;        // entries of a projection a thread keeps between the sum and the output

// One projection of one token to unit rms over all its entries, times a weight: read once (entries and weights are
// on their way before the sum is known), kept in registers, written to dst.
template <typename TE>
__device__ __forceinline__ void whole_norm_row(const TE* src, const float* __restrict__ weight, int width, float eps,
                                               TE* dst, float* scratch) {
    const int tid = threadIdx.x, step = blockDim.x;
    float kept[QN_KEEP], w[QN_KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < QN_KEEP; ++i) {
        const int d = tid + i * step;
        kept[i] = d < width ? to_float(src[d]) : 0.0f;
        w[i] = d < width ? weight[d] : 0.0f;
        ss = fmaf(kept[i], kept[i], ss);
    }
    for (int d = tid + QN_KEEP * step; d < width; d += step) {
        const float x = to_float(src[d]);
        ss = fmaf(x, x, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    // (src and dst may be the same row: an entry is read and written by the same thread)
    for (int d = tid + QN_KEEP * step; d < width; d += step) dst[d] = from_float<TE>(to_float(src[d]) * inv * weight[d]);
#pragma unroll
    for (int i = 0; i < QN_KEEP; ++i) {
        const int d = tid + i * step;
        if (d < width) dst[d] = from_float<TE>(kept[i] * inv * w[i]);
    }
}

// blockIdx.y: 0 the queries, 1 the keys, 2 the values; the three do not wait for one another.
template <typename TE>
__global__ void __launch_bounds__(128)
qkv_norm_rows_kernel(TE* q, long long ldq, const TE* __restrict__ k, long long ldk,
                     const TE* __restrict__ v, long long ldv, const float* __restrict__ q_weight,
                     const float* __restrict__ k_weight, float eps, int q_width, int k_width, int n_kv_heads, int vdim,
                     int value_norm, float* __restrict__ first, int first_mode, float lambda,
                     const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                     const int* __restrict__ block_table, int max_pages, int page_tokens, TE* __restrict__ rows) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, what = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
    if (what == 0) {
        TE* row = q + (long long)t * ldq;
        whole_norm_row<TE>(row, q_weight, q_width, eps, row, scratch);
        return;
    }
    const int pos = tok_pos[t];
    const long long page = block_table[(long long)tok_seq[t] * max_pages + pos / page_tokens];
    TE* dst = rows + (page * page_tokens + pos % page_tokens) * ((long long)k_width + (long long)n_kv_heads * vdim);
    if (what == 1) {
        whole_norm_row<TE>(k + (long long)t * ldk, k_weight, k_width, eps, dst, scratch);
        return;
    }
    TE* vdst = dst + k_width;
    for (int g = warp; g < n_kv_heads; g += warps) {
        const TE* src = v + (long long)t * ldv + (long long)g * vdim;
        const long long at0 = ((long long)t * n_kv_heads + g) * vdim;
        float kept[QN_KEEP], other[QN_KEEP];                 // a head's values, and the shared ones they blend with
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < QN_KEEP; ++i) {
            const int d = lane + 32 * i;
            kept[i] = d < vdim ? to_float(src[d]) : 0.0f;
            other[i] = first_mode == 2 && d < vdim ? first[at0 + d] : 0.0f;
            ss = fmaf(kept[i], kept[i], ss);
        }
        for (int d = lane + 32 * QN_KEEP; d < vdim; d += 32) {
            const float x = to_float(src[d]);
            ss = fmaf(x, x, ss);
        }
        const float inv = value_norm ? 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps) : 1.0f;
#pragma unroll
        for (int i = 0; i < QN_KEEP; ++i) {
            const int d = lane + 32 * i;
            if (d >= vdim) continue;
            float y = kept[i] * inv;
            if (first_mode == 1) first[at0 + d] = y;
            else if (first_mode == 2) y = (1.0f - lambda) * y + lambda * other[i];
            vdst[(long long)g * vdim + d] = from_float<TE>(y);
        }
        for (int d = lane + 32 * QN_KEEP; d < vdim; d += 32) {
            float y = to_float(src[d]) * inv;
            if (first_mode == 1) first[at0 + d] = y;
            else if (first_mode == 2) y = (1.0f - lambda) * y + lambda * first[at0 + d];
            vdst[(long long)g * vdim + d] = from_float<TE>(y);
        }
    }
}

constexpr int RA_KEEP = 8;        // entries of the row a thread keeps between the sum and the output

template <typename TE>
__global__ void __launch_bounds__(256)
residual_add_norm_kernel(float* __restrict__ x, long long ldx, const float* __restrict__ y, long long ldy, float mult,
                         const float* __restrict__ weight, float eps, int width, TE* __restrict__ h, long long ldh) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    float* xs = x + (long long)t * ldx;
    const float* ys = y ? y + (long long)t * ldy : nullptr;
    float kept[RA_KEEP];
    float sq = 0.0f;
#pragma unroll
    for (int i = 0; i < RA_KEEP; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        kept[i] = 0.0f;
        if (d < width) {
            kept[i] = ys ? fmaf(mult, ys[d], xs[d]) : xs[d];
            if (ys) xs[d] = kept[i];
        }
        sq += kept[i] * kept[i];
    }
    for (int d = threadIdx.x + RA_KEEP * blockDim.x; d < width; d += blockDim.x) {
        const float v = ys ? fmaf(mult, ys[d], xs[d]) : xs[d];
        if (ys) xs[d] = v;
        sq += v * v;
    }
    if (!weight) return;
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    TE* hs = h + (long long)t * ldh;
#pragma unroll
    for (int i = 0; i < RA_KEEP; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d < width) hs[d] = from_float<TE>(kept[i] * inv * weight[d]);
    }
    for (int d = threadIdx.x + RA_KEEP * blockDim.x; d < width; d += blockDim.x)
        hs[d] = from_float<TE>(xs[d] * inv * weight[d]);      // written by this very thread above
}

}  // namespace mu

// k and v null: queries only (a layer that reads another layer's rows).  first_mode 0: no shared values.
MU_EXPORT int mu_qkv_norm_rows(void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                               const float* q_weight, const float* k_weight, float eps, int n_tokens, int q_width,
                               int k_width, int n_kv_heads, int vdim, int value_norm, float* first, int first_mode,
                               float lambda, const int* tok_pos, const int* tok_seq, const int* block_table,
                               int max_pages, int page_tokens, void* rows, int is_bf16, void* stream) {
    if (n_tokens <= 0) return MU_OK;
    if (!q || !q_weight || q_width <= 0 || (k != nullptr) != (v != nullptr) || first_mode < 0 || first_mode > 2 ||
        (first_mode && !first))
        return MU_ERR_BAD_ARGUMENT;
    if (k && (!k_weight || !tok_pos || !tok_seq || !block_table || !rows || page_tokens <= 0 || k_width <= 0 ||
              n_kv_heads <= 0 || vdim <= 0))
        return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_tokens, k ? 3 : 1), block(128);
    typedef __nv_bfloat16 bf;
    if (is_bf16)
        return mu::launch_pdl(mu::qkv_norm_rows_kernel<bf>, grid, block, 0, s, 1, (bf*)q, ldq, (const bf*)k, ldk,
                              (const bf*)v, ldv, q_weight, k_weight, eps, q_width, k_width, n_kv_heads, vdim, value_norm,
                              first, first_mode, lambda, tok_pos, tok_seq, block_table, max_pages, page_tokens, (bf*)rows);
    return mu::launch_pdl(mu::qkv_norm_rows_kernel<float>, grid, block, 0, s, 1, (float*)q, ldq, (const float*)k, ldk,
                          (const float*)v, ldv, q_weight, k_weight, eps, q_width, k_width, n_kv_heads, vdim, value_norm,
                          first, first_mode, lambda, tok_pos, tok_seq, block_table, max_pages, page_tokens, (float*)rows);
}

MU_EXPORT int mu_residual_add_norm(float* x, long long ldx, const float* y, long long ldy, float mult, const float* weight,
                                   float eps, int n_rows, int width, void* h, long long ldh, int is_bf16, void* stream) {
    if (n_rows <= 0 || width <= 0) return MU_OK;
    if (!x || (weight && !h) || (!weight && !y)) return MU_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_rows), block(width > 1024 ? 256 : 128);
    typedef __nv_bfloat16 bf;
    if (is_bf16)
        return mu::launch_pdl(mu::residual_add_norm_kernel<bf>, grid, block, 0, s, 1, x, ldx, y, ldy, mult, weight, eps,
                              width, (bf*)h, ldh);
    return mu::launch_pdl(mu::residual_add_norm_kernel<float>, grid, block, 0, s, 1, x, ldx, y, ldy, mult, weight, eps,
                          width, (float*)h, ldh);
}
